"""Unit tier of the server: vision preprocessing, URL fetch policy, placeholder expansion, tool-call parsing,
output routing, detokeniser, and ctypes struct layouts against the C header
(the reference's counterparts: server/tests/test_vision_preprocess.py, test_fetch.py, test_tool_calls.py,
test_marshal.py)."""
import base64
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

from server_fixtures import make_tokenizer

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_smart_resize_properties():
    from qwserve.vision import smart_resize, video_smart_resize
    for h, w in [(480, 640), (1080, 1920), (33, 3000), (4000, 3000), (17, 19)]:
        H, W = smart_resize(h, w, 56 * 56, 1920 * 1088)
        assert H % 32 == 0 and W % 32 == 0 and 56 * 56 <= H * W <= 1920 * 1088
        if 56 * 56 <= h * w <= 1920 * 1088 and min(h, w) >= 32:
            assert abs(H - h) <= 16 and abs(W - w) <= 16
    with pytest.raises(ValueError):
        smart_resize(10, 4000, 3136, 10**6)
    H, W = video_smart_resize(7, 720, 1280, 128 * 32 * 32, 32 * 32 * 768)
    assert H % 32 == 0 and W % 32 == 0 and 8 * H * W <= 32 * 32 * 768


def test_patchify_matches_loops():
    from qwserve.vision import patchify
    rng = np.random.default_rng(0)
    fr = rng.standard_normal((4, 64, 96, 3)).astype(np.float32)
    rows, (t, h, w) = patchify(fr)
    assert (t, h, w) == (2, 4, 6) and rows.shape == (48, 1536)
    r = 0
    for ti in range(t):
        for hb in range(h // 2):
            for wb in range(w // 2):
                for dy in range(2):
                    for dx in range(2):
                        py, px = (hb * 2 + dy) * 16, (wb * 2 + dx) * 16
                        ref = fr[ti * 2:ti * 2 + 2, py:py + 16, px:px + 16, :].transpose(3, 0, 1, 2).reshape(-1)
                        assert np.array_equal(rows[r], ref)
                        r += 1


def test_image_preprocess_and_key():
    from PIL import Image
    from qwserve.vision import Preprocessor
    pre = Preprocessor(None)
    img = Image.fromarray((np.arange(100 * 130 * 3) % 255).astype(np.uint8).reshape(100, 130, 3))
    a, b = pre.image(img), pre.image(img.copy())
    assert a.grid == (1, 6, 8) and a.n_tokens == 12 and a.patches.shape == (48, 1536)
    assert a.key == b.key and len(a.key) == 8
    assert pre.image(img.transpose(Image.FLIP_LEFT_RIGHT)).key != a.key
    assert np.abs(a.patches).max() <= 1.0 + 1e-6
    # the two frames of an image's temporal patch are the same picture
    r = a.patches[0].reshape(3, 2, 16, 16)
    assert np.array_equal(r[:, 0], r[:, 1])


def test_video_sampling_and_timestamps():
    from qwserve.vision import Preprocessor
    pre = Preprocessor(None)
    frames = np.zeros((90, 64, 64, 3), np.uint8)        # 3 s at 30 fps -> 6 frames at 2 fps
    idx = pre.sample_indices(90, 30.0)
    assert len(idx) == 6 and idx[0] == 0 and idx[-1] == 89
    m = pre.video(frames, 30.0)
    assert m.kind == "video" and m.grid[0] == 3 and len(m.timestamps) == 3 and m.timestamps[0] < m.timestamps[-1]


def test_fetch_policy(monkeypatch):
    from qwserve import vision
    data = b"\x89PNG fake"
    assert vision.fetch("data:image/png;base64," + base64.b64encode(data).decode()) == data
    for bad in ("http://127.0.0.1/x.png", "http://localhost/x", "http://10.1.2.3/x", "http://169.254.169.254/latest", "file:///etc/passwd",
                "ftp://example.com/x"):
        with pytest.raises(ValueError):
            vision.check_url(bad)
    monkeypatch.setenv("QW_MEDIA_FETCH", "0")
    with pytest.raises(ValueError):
        vision.check_url("https://example.com/a.png")
    monkeypatch.setenv("QW_MEDIA_FETCH", "1")
    monkeypatch.setenv("QW_MEDIA_ALLOW_PRIVATE", "1")
    vision.check_url("http://127.0.0.1/x.png")


def test_expand_placeholders():
    from qwserve.vision import MediaItem, expand_placeholders
    tok = make_tokenizer()
    ipad, vpad = tok.token_to_id("<|image_pad|>"), tok.token_to_id("<|video_pad|>")
    img = MediaItem("image", np.zeros((16, 1536), np.float32), (1, 4, 4), b"12345678")
    vid = MediaItem("video", np.zeros((32, 1536), np.float32), (2, 4, 4), b"abcdefgh", timestamps=[0.5, 1.5])
    ids = [1, ipad, 2, vpad, 3]
    out = expand_placeholders(ids, [img, vid], tok)
    assert out.count(ipad) == 4 and out.count(vpad) == 8
    assert img.spans == [(1, 4)] and len(vid.spans) == 2 and all(out[s:s + n] == [vpad] * n for s, n in vid.spans)
    assert "<0.5 seconds>" in tok.decode(out, skip_special_tokens=True)
    with pytest.raises(ValueError):
        expand_placeholders([ipad], [], tok)
    with pytest.raises(ValueError):
        expand_placeholders([1], [img], tok)
    with pytest.raises(ValueError):
        expand_placeholders([vpad], [img], tok)


def test_tool_call_parser():
    import json
    from qwserve.tool_calls import parse_tool_call
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"type": "object", "properties": {
        "n": {"type": "integer"}, "x": {"type": "number"}, "ok": {"type": "boolean"}, "obj": {"type": "object"}, "s": {"type": "string"}}}}}]
    txt = ("<function=f>\n<parameter=n>\n7\n</parameter>\n<parameter=x>\n1.5\n</parameter>\n<parameter=ok>\ntrue\n</parameter>\n"
           "<parameter=obj>\n{\"a\": [1, 2]}\n</parameter>\n<parameter=s>\nif a < b and c > d:\n  pass\n</parameter>\n</function>")
    c = parse_tool_call(txt, tools)
    a = json.loads(c["function"]["arguments"])
    assert a == {"n": 7, "x": 1.5, "ok": True, "obj": {"a": [1, 2]}, "s": "if a < b and c > d:\n  pass"}
    assert c["type"] == "function" and c["id"].startswith("call_")
    # truncated output: the open value runs to the end
    c = parse_tool_call("<function=f>\n<parameter=s>\nhalf a val", tools)
    assert json.loads(c["function"]["arguments"]) == {"s": "half a val"}
    # no schema: JSON where it parses, text otherwise
    c = parse_tool_call("<function=g>\n<parameter=k>\n[1,2]\n</parameter>\n<parameter=t>\nplain\n</parameter>\n</function>")
    assert json.loads(c["function"]["arguments"]) == {"k": [1, 2], "t": "plain"}
    assert parse_tool_call("no call here") is None


def test_output_parser_and_detok():
    from qwserve.detok import IncrementalDetok
    from qwserve.output_parser import OutputParser, TagIds
    p = OutputParser(TagIds(1, 2, 3, 4), start_in_think=True)
    chans = [(r.channel if r else None) for r in map(p.push, [10, 11, 2, 12, 3, 13, 14, 4, 15, 1, 16, 2])]
    assert chans == ["reasoning", "reasoning", None, "content", None, "tool", "tool", None, "content", None, "reasoning", None]
    assert p.tool_tokens == [[13, 14]] and p.reasoning_tokens == 3
    tok = make_tokenizer()
    ids = tok.encode("añ日🙂z", add_special_tokens=False).ids
    d = IncrementalDetok(lambda x: tok.decode(x, skip_special_tokens=False))
    pieces = [d.push(i) for i in ids]
    assert "".join(pieces) + d.flush() == "añ日🙂z" and all("�" not in s for s in pieces)
    assert sum(1 for s in pieces if s == "") >= 5      # held back inside multi-byte characters


def test_ctypes_structs_match_header(tmp_path):
    """sizeof / offsetof as the C compiler sees the header == the ctypes mirrors."""
    from qwserve import engine as E
    src = tmp_path / "sz.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "qw/capi.h"\nint main(){'
                   'printf("%zu %zu %zu %zu %zu %zu %zu %zu\\n", sizeof(qw_sampling), offsetof(qw_sampling, seed), sizeof(qw_cache_stats),'
                   'sizeof(qw_slot_timing), sizeof(qw_media), offsetof(qw_media, patches), sizeof(qw_step_req), offsetof(qw_step_req, sampling));return 0;}')
    exe = tmp_path / "sz"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    want = [C.sizeof(E.Sampling), E.Sampling.seed.offset, C.sizeof(E.CacheStats), C.sizeof(E.SlotTiming), C.sizeof(E.Media),
            E.Media.patches.offset, C.sizeof(E.StepReq), E.StepReq.sampling.offset]
    assert got == want


def test_spill_plan_from_serving_options():
    """--kv-spill on --slot-max-tokens N: N tokens per slot, the first max(slots) resident, the rest in host pages."""
    from qwb200.capi_impl import spill_plan
    assert spill_plan([131072, 32768, 32768, 32768], 0, False) == (131072, None, 0)
    assert spill_plan([8192, 8192], 65536, False) == (65536, None, 0)                       # a larger capacity, all resident
    cap, dev, host = spill_plan([32768] * 6, 131072, True)
    assert (cap, dev, host) == (131072, 6 * 128, 6 * 384)
    cap, dev, host = spill_plan([8192, 4096], 10000, True)                                  # rounded up to whole pages
    assert cap == 10240 and dev == 2 * 32 and host == 2 * 8
    assert spill_plan([32768] * 2, 16384, True) == (16384, None, 0)                         # nothing to spill
    assert spill_plan([1024], 4096, False, dev_pages=2, host_pages=6) == (4096, 2, 6)       # explicit pages win
    # the reference's per-slot list: tokens beyond each slot's device part; slots it does not name get slot_max_tokens - slots[i]
    assert spill_plan([32768, 32768], 0, False, slot_spill=[0, 98304]) == (131072, 2 * 128, 2 * 384)
    assert spill_plan([131072, 32768, 32768], 262144, False, slot_spill=[0]) == (262144, 3 * 512, 3 * 512)
    assert spill_plan([8192, 8192], 0, False, slot_spill=[0, 0]) == (8192, None, 0)          # all zero: no spill
    with pytest.raises(ValueError):
        spill_plan([8192], 0, False, slot_spill=[256, 256])


def test_capi_prefill_batch_reads_and_writes_the_callers_arrays():
    """qw_prefill_batch's Python side: slots and limits come from the caller's arrays, every slot's piece runs in one call of
    the session ops, and the flags go back into the caller's array."""
    import ctypes as C
    import types
    from qwb200.capi_impl import CApi, SessionOps
    seen = []

    class Ses:
        def prefill_some(self, slot, max_tokens):
            seen.append((slot, max_tokens))
            return slot != 2                      # slot 2's prompt is not in yet
    ops = SessionOps(Ses(), None)
    api = CApi(ops)
    slots, mt, done = (C.c_int32 * 3)(1, 2, 0), (C.c_int64 * 3)(2048, 2048, 512), (C.c_int32 * 3)(9, 9, 9)
    assert api.prefill_batch(3, C.addressof(slots), C.addressof(mt), C.addressof(done)) == 0
    assert seen == [(1, 2048), (2, 2048), (0, 512)] and list(done) == [1, 0, 1]


def test_sampling_defaults_from_the_checkpoint(tmp_path):
    """Built-in defaults by mode < the checkpoint's generation_config.json < the request's own fields."""
    import json as _json
    from qwserve.api import DEFAULTS_PLAIN, DEFAULTS_THINKING, model_sampling_defaults, sampling_of
    assert model_sampling_defaults(None) == {} and model_sampling_defaults(str(tmp_path)) == {}
    (tmp_path / "generation_config.json").write_text("{ not json")
    assert model_sampling_defaults(str(tmp_path)) == {}
    (tmp_path / "generation_config.json").write_text(_json.dumps(
        {"temperature": 0.6, "top_k": 40, "top_p": "0.9", "do_sample": True, "min_p": False, "eos_token_id": [1, 2], "repetition_penalty": 1.05}))
    d = model_sampling_defaults(str(tmp_path))
    assert d == {"temperature": 0.6, "top_k": 40, "repetition_penalty": 1.05}          # numbers only: no strings, no booleans, no other keys
    s = sampling_of({}, thinking=True)
    near = lambda x, y: abs(x - y) < 1e-6                                                 # the struct holds 32-bit floats
    assert near(s.temperature, DEFAULTS_THINKING["temperature"]) and near(s.top_p, DEFAULTS_THINKING["top_p"]) and s.top_k == DEFAULTS_THINKING["top_k"]
    s = sampling_of({}, thinking=False, model_defaults=d)
    assert near(s.temperature, 0.6) and s.top_k == 40 and near(s.repetition_penalty, 1.05) and near(s.top_p, DEFAULTS_PLAIN["top_p"])
    s = sampling_of({"temperature": 0.0, "top_k": 1, "seed": 7}, thinking=False, model_defaults=d)
    assert s.temperature == 0.0 and s.top_k == 1 and s.seed == 7 and near(s.repetition_penalty, 1.05)
    a, b = sampling_of({}, True), sampling_of({}, True)
    assert a.seed != b.seed                                                               # no seed given: a fresh one per request


def test_tool_call_parser_round_trip_and_truncation_fuzz():
    """Generated calls: any set of typed arguments rendered in the model's format parses back to the same values, and
    no prefix of a rendered call (a generation cut off anywhere) makes the parser raise."""
    import json
    from hypothesis import given, settings, strategies as st
    from qwserve.tool_calls import parse_tool_call
    ident = st.text(alphabet="abcdefghijklmnopqrstuvwxyz_", min_size=1, max_size=8)
    plain = st.text(alphabet=st.characters(blacklist_categories=("Cs",), blacklist_characters="\r"), max_size=40).filter(
        lambda s: "<parameter=" not in s and "</parameter>" not in s and "</function>" not in s and "<function=" not in s
        and not s.startswith("\n") and not s.endswith("\n"))
    value = st.one_of(st.tuples(st.just("integer"), st.integers(-10**9, 10**9)),
                      st.tuples(st.just("number"), st.floats(allow_nan=False, allow_infinity=False, width=32)),
                      st.tuples(st.just("boolean"), st.booleans()),
                      st.tuples(st.just("string"), plain),
                      st.tuples(st.just("array"), st.lists(st.integers(0, 9), max_size=4)),
                      st.tuples(st.just("object"), st.dictionaries(ident, st.integers(0, 9), max_size=3)))

    def render(name, args):
        out = [f"<function={name}>"]
        for k, (ty, v) in args.items():
            txt = v if ty == "string" else json.dumps(v)
            out.append(f"<parameter={k}>\n{txt}\n</parameter>")
        return "\n".join(out) + "\n</function>"

    @settings(max_examples=150, deadline=None)
    @given(ident, st.dictionaries(ident, value, max_size=5), st.integers(0, 10**6))
    def check(name, args, cut):
        tools = [{"type": "function", "function": {"name": name, "parameters": {"type": "object", "properties": {
            k: {"type": ty} for k, (ty, _) in args.items()}}}}]
        text = render(name, args)
        call = parse_tool_call("some words before " + text, tools)
        assert call["function"]["name"] == name
        assert json.loads(call["function"]["arguments"]) == {k: v for k, (_, v) in args.items()}
        part = parse_tool_call(text[:cut % (len(text) + 1)], tools)            # cut anywhere: a call or nothing, never an exception
        assert part is None or json.loads(part["function"]["arguments"]) is not None
    check()


def _fake_ffmpeg(tmp_path, monkeypatch, frames=90, w=64, h=48, fps="30/1", fail=False, short_second_pass=False):
    """Stand-ins for ffprobe / ffmpeg on PATH: the "video" decodes to `frames` raw frames, frame i filled with byte i."""
    import stat
    import sys
    d = tmp_path / "bin"
    d.mkdir(exist_ok=True)
    (d / "ffprobe").write_text(f"#!{sys.executable}\nimport json\nprint(json.dumps({{'streams': [{{'width': {w}, 'height': {h}, 'r_frame_rate': '{fps}'}}]}}))\n")
    count = tmp_path / "passes"
    (d / "ffmpeg").write_text(
        f"#!{sys.executable}\nimport os, sys\n"
        f"p = {str(count)!r}\nn = int(open(p).read()) + 1 if os.path.exists(p) else 1\nopen(p, 'w').write(str(n))\n"
        f"frames = {frames} - (5 if {short_second_pass} and n == 2 else 0)\n"
        f"try:\n"
        f"    for i in range(frames):\n        sys.stdout.buffer.write(bytes([i % 256]) * ({w} * {h} * 3))\n"
        f"    sys.stdout.buffer.flush()\nexcept BrokenPipeError:\n    os._exit(0)\n"
        f"if {fail}:\n    sys.stderr.write('moov atom not found')\n    sys.exit(1)\n")
    for n in ("ffprobe", "ffmpeg"):
        os.chmod(d / n, os.stat(d / n).st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(d) + os.pathsep + os.environ["PATH"])


def test_video_is_decoded_as_a_stream(tmp_path, monkeypatch):
    """Two passes over the file (count, then pick): the sampled frames are the ones the sampling rule names, equal to
    decoding everything first, and a failing or shrinking ffmpeg is reported as a bad video, not a crash."""
    from qwserve import vision
    from qwserve.vision import Preprocessor, VideoPipe
    pre = Preprocessor(None)
    _fake_ffmpeg(tmp_path, monkeypatch)
    with VideoPipe("x.mp4", 64, 48) as pipe:
        assert sum(1 for _ in pipe.frames()) == 90
    with VideoPipe("x.mp4", 64, 48) as pipe:
        picked = list(pipe.pick([0, 3, 3, 89]))
    assert [int(f[0, 0, 0]) for f in picked] == [0, 3, 3, 89] and picked[0].shape == (48, 64, 3)
    with VideoPipe("x.mp4", 64, 48) as pipe:                                  # stopping early just ends ffmpeg
        assert [int(f[0, 0, 0]) for f in pipe.pick([2])] == [2]
    (tmp_path / "passes").unlink()
    m = pre.video_bytes(b"not really a video")
    assert int((tmp_path / "passes").read_text()) == 2                       # one counting pass, one picking pass
    all_frames = np.stack([np.full((48, 64, 3), i, np.uint8) for i in range(90)])
    want = pre.video(all_frames, 30.0)
    assert m.kind == "video" and m.grid == want.grid and m.timestamps == want.timestamps and m.key == want.key
    assert np.array_equal(m.patches, want.patches)
    _fake_ffmpeg(tmp_path, monkeypatch, fail=True)
    with pytest.raises(ValueError, match="ffmpeg failed .*moov atom"):
        pre.video_bytes(b"broken")
    _fake_ffmpeg(tmp_path, monkeypatch, short_second_pass=True)
    (tmp_path / "passes").unlink()
    with pytest.raises(ValueError, match="fewer frames"):
        pre.video_bytes(b"shrinks")
    _fake_ffmpeg(tmp_path, monkeypatch, w=0)
    with pytest.raises(ValueError, match="no size"):
        pre.video_bytes(b"no size")
