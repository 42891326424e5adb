"""Converted-weights cache: the per-rank, engine-layout tensors that loading produces (sliced, re-ordered q4 nibbles,
folded norm weights, ...) written once to ``<dir>/rank<r>.qww`` and read back on later starts instead of converting
the checkpoint again (reference: src/engine/weights.hip:33-176).

The file is valid only for the key it was recorded under: a hash of a format version, rank, rank count, the model
shapes and every checkpoint file's path, size and modification time.  It is written to ``.tmp`` and renamed when
complete; a replay must consume exactly the recorded records in order, anything else is an error (a half-matching
cache would silently serve wrong weights).

Layout: ``QWWEIGH1`` | u32 version | u64 key | records...; a record is u32 header length, a JSON header
``{"name", "entries": [[path, dtype, shape, offset, nbytes], ...], "scalars": {path: value}}`` and the tensors' bytes,
each starting on a 64-byte boundary (offsets are relative to the first byte after the header)."""
from __future__ import annotations

import glob
import json
import os
import struct
from typing import Dict, List, Optional

import numpy as np
import torch

MAGIC = b"QWWEIGH1"
VERSION = 1
_DT = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16, "int32": torch.int32, "int64": torch.int64,
       "uint8": torch.uint8, "int8": torch.int8, "int16": torch.int16}


def _fnv(data: bytes, h: int = 0xcbf29ce484222325) -> int:
    for b in data:
        h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


def cache_key(model_dir: str, rank: int, ranks: int, shapes: str) -> int:
    """Hash of everything a converted file depends on."""
    h = _fnv(f"v{VERSION}|rank{rank}/{ranks}|{shapes}".encode())
    for p in sorted(glob.glob(os.path.join(model_dir, "*.safetensors")) + glob.glob(os.path.join(model_dir, "config.json"))):
        st = os.stat(p)
        h = _fnv(f"{os.path.basename(p)}|{st.st_size}|{st.st_mtime_ns}".encode(), h)
    return h


def _flatten(obj, prefix, tensors, scalars):
    for k, v in obj.items():
        path = f"{prefix}/{k}" if prefix else str(k)
        if isinstance(v, dict):
            _flatten(v, path, tensors, scalars)
        elif isinstance(v, torch.Tensor):
            tensors.append((path, v))
        else:
            scalars[path] = v


def _unflatten(paths) -> Dict[str, object]:
    root: Dict[str, object] = {}
    for path, v in paths:
        parts = path.split("/")
        d = root
        for p in parts[:-1]:
            d = d.setdefault(p, {})
        d[parts[-1]] = v
    return root


class WeightCache:
    def __init__(self, directory: str, rank: int, key: int):
        os.makedirs(directory, exist_ok=True)
        self.path = os.path.join(directory, f"rank{rank}.qww")
        self.key = key
        self.replaying = False
        self._f = None
        self._buf: Optional[np.memmap] = None
        self._pos = 0
        self.records = 0
        if os.path.exists(self.path):
            with open(self.path, "rb") as f:
                head = f.read(20)
            if len(head) == 20 and head[:8] == MAGIC and struct.unpack("<IQ", head[8:]) == (VERSION, key):
                self.replaying = True
                self._buf = np.memmap(self.path, dtype=np.uint8, mode="r")
                self._pos = 20
        if not self.replaying:
            self._f = open(self.path + ".tmp", "wb")
            self._f.write(MAGIC + struct.pack("<IQ", VERSION, key))

    # ---- record
    def put(self, name: str, obj: Dict[str, object]) -> None:
        assert not self.replaying and self._f is not None
        tensors: List = []
        scalars: Dict[str, object] = {}
        _flatten(obj, "", tensors, scalars)
        entries, off, blobs = [], 0, []
        for path, t in tensors:
            c = t.detach().contiguous().cpu()
            raw = c.view(torch.uint8).numpy().tobytes() if c.numel() else b""
            off = (off + 63) & ~63
            entries.append([path, str(c.dtype).replace("torch.", ""), list(c.shape), off, len(raw)])
            blobs.append((off, raw))
            off += len(raw)
        header = json.dumps({"name": name, "entries": entries, "scalars": scalars, "size": off}).encode()
        pad = (-(self._f.tell() + 4 + len(header))) % 64           # data starts 64-byte aligned in the file too
        header += b" " * pad
        self._f.write(struct.pack("<I", len(header)) + header)
        start = self._f.tell()
        for o, raw in blobs:
            self._f.seek(start + o)
            self._f.write(raw)
        self._f.truncate(start + off)          # also when the last tensor is empty or padding follows it
        self._f.seek(start + off)
        self.records += 1

    # ---- replay
    def get(self, name: str, device) -> Dict[str, object]:
        assert self.replaying and self._buf is not None
        if self._pos + 4 > len(self._buf):
            raise RuntimeError(f"weight cache {self.path}: no record left for '{name}'")
        (hl,) = struct.unpack("<I", bytes(self._buf[self._pos:self._pos + 4]))
        hdr = json.loads(bytes(self._buf[self._pos + 4:self._pos + 4 + hl]).decode())
        if hdr["name"] != name:
            raise RuntimeError(f"weight cache {self.path}: expected record '{name}', found '{hdr['name']}'")
        start = self._pos + 4 + hl
        out = [(p, v) for p, v in hdr["scalars"].items()]
        for path, dt, shape, off, nbytes in hdr["entries"]:
            if nbytes == 0:
                out.append((path, torch.empty(shape, dtype=_DT[dt], device=device)))
                continue
            raw = torch.from_numpy(np.array(self._buf[start + off:start + off + nbytes], copy=True))
            out.append((path, raw.view(_DT[dt]).view(shape).to(device)))
        self._pos = start + hdr["size"]
        self.records += 1
        return _unflatten(out)

    def close(self) -> None:
        """Record: publish the file.  Replay: everything recorded must have been consumed."""
        if self.replaying:
            if self._buf is not None and self._pos != len(self._buf):
                raise RuntimeError(f"weight cache {self.path}: {len(self._buf) - self._pos} bytes were not consumed")
            self._buf = None
        elif self._f is not None:
            self._f.flush()
            os.fsync(self._f.fileno())
            self._f.close()
            self._f = None
            os.replace(self.path + ".tmp", self.path)
