"""Media preprocessing for the server: Qwen3-VL image / video preprocessing into ViT patches, content hashes,
a URL fetcher that only reaches public addresses, and placeholder expansion in the token stream
(reference behaviour: server/qwserve/vision.py:54-112,115-202,281-327,346-376).

Geometry: 16x16 pixel patches, 2 frames per temporal patch, 2x2 patches merged into one language-model token;
a patch row is 3*2*16*16 = 1536 floats, rows ordered so the four patches of a merge window are adjacent."""
from __future__ import annotations

import base64
import hashlib
import io
import ipaddress
import json
import math
import os
import shutil
import socket
import subprocess
import urllib.request
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple
from urllib.parse import urlsplit

import numpy as np

PATCH, MERGE, FRAMES_PER_PATCH = 16, 2, 2
UNIT = PATCH * MERGE
FETCH_LIMIT = 64 << 20


def fetch_policy():
    """(remote allowed, private addresses allowed), read from the environment at call time."""
    return os.environ.get("QW_MEDIA_FETCH", "1") != "0", os.environ.get("QW_MEDIA_ALLOW_PRIVATE", "0") == "1"


@dataclass
class MediaItem:
    kind: str                               # "image" | "video"
    patches: np.ndarray                     # float32 [t*h*w, 1536]
    grid: Tuple[int, int, int]              # (t, h, w) in patches
    key: bytes                              # 8 bytes of sha256 over grid and patches
    timestamps: List[float] = field(default_factory=list)
    spans: List[Tuple[int, int]] = field(default_factory=list)     # (first token, count) in the expanded prompt

    @property
    def n_tokens(self) -> int:
        t, h, w = self.grid
        return t * h * w // (MERGE * MERGE)


# ---- sizes
def smart_resize(height: int, width: int, min_pixels: int, max_pixels: int, unit: int = UNIT) -> Tuple[int, int]:
    """Nearest size with both sides multiples of ``unit`` whose area lies in [min_pixels, max_pixels], keeping
    the aspect ratio as far as the rounding allows."""
    if max(height, width) > 200 * min(height, width):
        raise ValueError("image aspect ratio must be under 200")
    h = max(unit, round(height / unit) * unit)
    w = max(unit, round(width / unit) * unit)
    if h * w > max_pixels:
        s = math.sqrt(height * width / max_pixels)
        h = max(unit, math.floor(height / s / unit) * unit)
        w = max(unit, math.floor(width / s / unit) * unit)
    elif h * w < min_pixels:
        s = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * s / unit) * unit
        w = math.ceil(width * s / unit) * unit
    return h, w


def video_smart_resize(n_frames: int, height: int, width: int, min_pixels: int, max_pixels: int,
                       unit: int = UNIT) -> Tuple[int, int]:
    """As smart_resize with the budget counted over the whole clip (frames rounded up to temporal patches)."""
    if max(height, width) > 200 * min(height, width):
        raise ValueError("video aspect ratio must be under 200")
    t = math.ceil(n_frames / FRAMES_PER_PATCH) * FRAMES_PER_PATCH
    h = max(unit, round(height / unit) * unit)
    w = max(unit, round(width / unit) * unit)
    if t * h * w > max_pixels:
        s = math.sqrt(t * height * width / max_pixels)
        h = max(unit, math.floor(height / s / unit) * unit)
        w = max(unit, math.floor(width / s / unit) * unit)
    elif t * h * w < min_pixels:
        s = math.sqrt(min_pixels / (t * height * width))
        h = math.ceil(height * s / unit) * unit
        w = math.ceil(width * s / unit) * unit
    return h, w


# ---- pixels -> patches
def normalize(rgb: np.ndarray, mean: Sequence[float], std: Sequence[float]) -> np.ndarray:
    """uint8 [..., 3] -> float32 in the model's input scale."""
    return (rgb.astype(np.float32) / 255.0 - np.asarray(mean, np.float32)) / np.asarray(std, np.float32)


def patchify(frames: np.ndarray) -> Tuple[np.ndarray, Tuple[int, int, int]]:
    """frames float32 [T, H, W, 3] (T a multiple of 2; H, W multiples of 32) -> rows [t*h*w, 3*2*16*16] in
    merge-window order: (t, h/2, w/2, 2, 2) over rows, (channel, frame, y, x) within a row."""
    T, H, W, _ = frames.shape
    t, h, w = T // FRAMES_PER_PATCH, H // PATCH, W // PATCH
    x = frames.reshape(t, FRAMES_PER_PATCH, h // MERGE, MERGE, PATCH, w // MERGE, MERGE, PATCH, 3)
    #            0  1                 2           3      4      5           6      7      8
    x = x.transpose(0, 2, 5, 3, 6, 8, 1, 4, 7)
    return np.ascontiguousarray(x.reshape(t * h * w, 3 * FRAMES_PER_PATCH * PATCH * PATCH)), (t, h, w)


def content_key(patches: np.ndarray, grid) -> bytes:
    d = hashlib.sha256(np.asarray(grid, np.int32).tobytes())
    d.update(patches.tobytes())
    return d.digest()[:8]


class Preprocessor:
    def __init__(self, model_dir: Optional[str] = None):
        def cfg(name):
            p = os.path.join(model_dir, name) if model_dir else ""
            return json.load(open(p)) if p and os.path.exists(p) else {}
        img, vid = cfg("preprocessor_config.json"), cfg("video_preprocessor_config.json")
        s = img.get("size", {})
        self.img_min = int(s.get("shortest_edge", 56 * 56))
        # images above ~2 MP are scaled down by default: tower time grows with the square of the token count
        self.img_max = min(int(s.get("longest_edge", 28 * 28 * 1280)), int(os.environ.get("QW_VISION_MAX_PIXELS", 1920 * 1088)))
        self.img_mean, self.img_std = img.get("image_mean", [0.5] * 3), img.get("image_std", [0.5] * 3)
        v = vid.get("size", {})
        self.vid_min = int(v.get("shortest_edge", 128 * 32 * 32))
        self.vid_max = int(v.get("longest_edge", 32 * 32 * 768))
        if os.environ.get("QW_VIDEO_MAX_PIXELS"):
            self.vid_max = min(self.vid_max, int(os.environ["QW_VIDEO_MAX_PIXELS"]))
        self.vid_mean, self.vid_std = vid.get("image_mean", [0.5] * 3), vid.get("image_std", [0.5] * 3)
        self.fps = float(vid.get("fps", 2.0))
        self.min_frames, self.max_frames = int(vid.get("min_frames", 4)), int(vid.get("max_frames", 768))

    def image(self, pil) -> MediaItem:
        from PIL import Image
        pil = pil.convert("RGB")
        h, w = smart_resize(pil.height, pil.width, self.img_min, self.img_max)
        if (w, h) != pil.size:
            pil = pil.resize((w, h), Image.BICUBIC)
        x = normalize(np.asarray(pil), self.img_mean, self.img_std)
        rows, grid = patchify(np.ascontiguousarray(np.broadcast_to(x[None], (FRAMES_PER_PATCH,) + x.shape)))
        return MediaItem("image", rows, grid, content_key(rows, grid))

    def sample_indices(self, total: int, src_fps: float) -> np.ndarray:
        n = int(total / max(src_fps, 1e-6) * self.fps)
        n = min(max(n, self.min_frames), self.max_frames, total)
        return np.linspace(0, total - 1, n).round().astype(int)

    def video(self, frames: np.ndarray, src_fps: float) -> MediaItem:
        """frames uint8 [N, H, W, 3] decoded at ``src_fps`` (all of them in memory: tests and short clips)."""
        idx = self.sample_indices(len(frames), src_fps)
        return self.video_sampled((frames[i] for i in idx), idx, src_fps, frames.shape[1], frames.shape[2])

    def video_sampled(self, picked, idx: np.ndarray, src_fps: float, h0: int, w0: int) -> MediaItem:
        """``picked`` yields the frames at the source indices ``idx`` (uint8 [h0, w0, 3]), one at a time; each is resized
        and normalised as it arrives, so only the sampled frames at model resolution are ever held."""
        from PIL import Image
        h, w = video_smart_resize(len(idx), h0, w0, self.vid_min, self.vid_max)
        out = []
        for f in picked:
            if (h, w) != (h0, w0):
                f = np.asarray(Image.fromarray(f).resize((w, h), Image.BICUBIC))
            out.append(normalize(f, self.vid_mean, self.vid_std))
        if len(out) != len(idx):
            raise ValueError("the video ended before its last sampled frame")
        if len(out) % FRAMES_PER_PATCH:
            out.append(out[-1])
            idx = np.append(idx, idx[-1])
        rows, grid = patchify(np.stack(out))
        stamps = [float((idx[2 * j] + idx[2 * j + 1]) / 2 / src_fps) for j in range(grid[0])]
        return MediaItem("video", rows, grid, content_key(rows, grid), stamps)

    def video_bytes(self, data: bytes) -> MediaItem:
        """Decode with the ffmpeg executable, streaming: raw rgb24 frames come over a pipe one at a time and are never
        all in memory (a minute of 1080p is 11 GB raw).  Two passes over the file: the first counts the frames ffmpeg
        really decodes (container metadata is not reliable), the second keeps the sampled ones and stops ffmpeg after the
        last of them.  (Reference behaviour: server/qwserve/vision.py:205-275.)"""
        if not shutil.which("ffmpeg") or not shutil.which("ffprobe"):
            raise ValueError("video input needs ffmpeg and ffprobe on PATH")
        import tempfile
        with tempfile.NamedTemporaryFile(suffix=".bin") as f:
            f.write(data)
            f.flush()
            try:
                probe = subprocess.run(["ffprobe", "-v", "error", "-select_streams", "v:0", "-show_entries",
                                        "stream=width,height,r_frame_rate", "-of", "json", f.name],
                                       capture_output=True, timeout=60, check=True)
                st = json.loads(probe.stdout)["streams"][0]
                w, h = int(st["width"]), int(st["height"])
                num, _, den = str(st["r_frame_rate"]).partition("/")
                fps = float(num) / max(1.0, float(den or 1))
            except (subprocess.SubprocessError, ValueError, KeyError, IndexError) as ex:
                raise ValueError(f"not a video ffprobe can read ({type(ex).__name__})") from ex
            if w <= 0 or h <= 0 or fps <= 0:
                raise ValueError("the video reports no size or frame rate")
            with VideoPipe(f.name, w, h) as pipe:                    # pass 1: how many frames are really there
                total = sum(1 for _ in pipe.frames())
            if total == 0:
                raise ValueError("no frames decoded")
            idx = self.sample_indices(total, fps)
            with VideoPipe(f.name, w, h) as pipe:                    # pass 2: keep the sampled ones, stop after the last
                return self.video_sampled(pipe.pick(idx), idx, fps, h, w)


FFMPEG_SECONDS = 300.0


class VideoPipe:
    """One ffmpeg process turning a file into raw rgb24 frames on its standard output, read one frame at a time.

        with VideoPipe(path, w, h) as pipe:
            for frame in pipe.frames(): ...          # uint8 [h, w, 3] views of one reused buffer

    Leaving the block after the stream was read to its end checks ffmpeg's exit code (a decode error is a bad video);
    leaving it earlier just ends the process.  A watchdog ends an ffmpeg that runs longer than ``FFMPEG_SECONDS``.
    Diagnostics go to a scratch file, since an unread pipe would block the child once it fills."""

    def __init__(self, path: str, w: int, h: int):
        self.cmd = ["ffmpeg", "-v", "error", "-i", path, "-f", "rawvideo", "-pix_fmt", "rgb24", "-"]
        self.shape = (h, w, 3)
        self.nbytes = h * w * 3
        self.exhausted = False

    def __enter__(self):
        import tempfile
        import threading
        self.log = tempfile.TemporaryFile()
        self.child = subprocess.Popen(self.cmd, stdout=subprocess.PIPE, stderr=self.log, bufsize=0)
        self.watchdog = threading.Timer(FFMPEG_SECONDS, self.child.kill)
        self.watchdog.daemon = True
        self.watchdog.start()
        return self

    def frames(self):
        buf = np.empty(self.nbytes, np.uint8)
        view = memoryview(buf)
        while True:
            have = 0
            while have < self.nbytes:
                got = self.child.stdout.readinto(view[have:])
                if not got:
                    break
                have += got
            if have == 0:
                self.exhausted = True
                return
            if have < self.nbytes:
                raise ValueError("the decoded video does not match the size it reports")
            yield buf.reshape(self.shape)

    def pick(self, idx: Sequence[int]):
        """Copies of the frames at the ascending source indices ``idx`` (an index may repeat); decoding stops after the last."""
        want = [int(i) for i in idx]
        at = 0
        for n, frame in enumerate(self.frames()):
            if at < len(want) and want[at] == n:
                keep = frame.copy()
                while at < len(want) and want[at] == n:
                    yield keep
                    at += 1
            if at == len(want):
                return
        if at < len(want):
            raise ValueError("the video has fewer frames than on the first pass")

    def __exit__(self, exc_type, exc, tb):
        self.watchdog.cancel()
        self.child.stdout.close()
        if not self.exhausted:
            self.child.kill()
        code = self.child.wait()
        try:
            if exc_type is None and self.exhausted and code != 0:
                self.log.seek(0)
                tail = self.log.read()[-300:].decode(errors="replace").strip()
                raise ValueError(f"ffmpeg failed ({code}): {tail}")
        finally:
            self.log.close()
        return False


# ---- fetching
_GROUP_V4, _GROUP_V6 = ipaddress.ip_network("224.0.0.0/4"), ipaddress.ip_network("ff00::/8")


def _public(host: str) -> bool:
    try:
        infos = socket.getaddrinfo(host, None)
    except socket.gaierror:
        return False
    for info in infos:
        ip = ipaddress.ip_address(info[4][0])
        group = ip in (_GROUP_V4 if ip.version == 4 else _GROUP_V6)          # one-to-many group addresses
        if ip.is_private or ip.is_loopback or ip.is_link_local or group or ip.is_reserved or ip.is_unspecified:
            return False
    return bool(infos)


def check_url(url: str) -> None:
    remote, private = fetch_policy()
    u = urlsplit(url)
    if u.scheme not in ("http", "https"):
        raise ValueError(f"unsupported URL scheme {u.scheme!r}")
    if not remote:
        raise ValueError("fetching remote media is disabled")
    if not u.hostname:
        raise ValueError("URL has no host")
    if not private and not _public(u.hostname):
        raise ValueError("URL does not resolve to a public address")


class _Recheck(urllib.request.HTTPRedirectHandler):
    def redirect_request(self, req, fp, code, msg, headers, newurl):
        check_url(newurl)                     # a redirect must not lead where the first URL could not
        return super().redirect_request(req, fp, code, msg, headers, newurl)


def fetch(url: str) -> bytes:
    """Bytes of a ``data:`` URL or of an http(s) URL on a public address, at most 64 MiB."""
    if url.startswith("data:"):
        head, _, payload = url.partition(",")
        return base64.b64decode(payload) if head.endswith(";base64") else urllib.request.unquote_to_bytes(payload)
    check_url(url)
    opener = urllib.request.build_opener(_Recheck)
    with opener.open(url, timeout=30) as r:
        data = r.read(FETCH_LIMIT + 1)
    if len(data) > FETCH_LIMIT:
        raise ValueError("media larger than 64 MiB")
    return data


def media_of_part(pre: Preprocessor, part: dict) -> Optional[MediaItem]:
    """The media item of one OpenAI content part; None for text."""
    def url_of(v):
        return v.get("url") if isinstance(v, dict) else v
    kind = part.get("type", "")
    if "video" in part or "video_url" in part or kind in ("video", "video_url"):
        return pre.video_bytes(fetch(url_of(part.get("video") or part.get("video_url") or {})))
    if "image_url" in part or "image" in part or kind in ("image", "image_url"):
        from PIL import Image
        try:
            return pre.image(Image.open(io.BytesIO(fetch(url_of(part.get("image_url") or part.get("image") or {})))))
        except Image.DecompressionBombError as ex:
            raise ValueError(f"image too large: {ex}") from ex
    return None


def expand_placeholders(ids: List[int], media: List[MediaItem], tok) -> List[int]:
    """Replace every placeholder token by its item's vision tokens and record each item's spans.  An image pad
    becomes n_tokens pads; a video pad becomes, per temporal patch, the text "<T seconds>" then
    vision_start, the patch's pads, vision_end."""
    ipad, vpad = tok.token_to_id("<|image_pad|>"), tok.token_to_id("<|video_pad|>")
    vs, ve = tok.token_to_id("<|vision_start|>"), tok.token_to_id("<|vision_end|>")
    out: List[int] = []
    queue = list(media)
    for t in ids:
        if t != ipad and t != vpad or t is None:
            out.append(t)
            continue
        if not queue:
            raise ValueError("media do not match the prompt's placeholders")
        m = queue.pop(0)
        if (m.kind == "image") != (t == ipad):
            raise ValueError("media do not match the prompt's placeholders")
        m.spans = []
        if m.kind == "image":
            m.spans.append((len(out), m.n_tokens))
            out += [ipad] * m.n_tokens
        else:
            per = m.grid[1] * m.grid[2] // (MERGE * MERGE)
            for ts in m.timestamps:
                out += tok.encode(f"<{ts:.1f} seconds>", add_special_tokens=False).ids
                out.append(vs)
                m.spans.append((len(out), per))
                out += [vpad] * per
                out.append(ve)
    if queue:
        raise ValueError("more media than placeholders in the prompt")
    return out
