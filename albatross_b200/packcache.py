"""On-disk cache of the quantised, packed big matrices of a checkpoint.

The reference prepares its weights from the `.pth` file on every start (reference/rwkv7.py:79-96: load, transposed
view, fp16 cast, ln0 fold). Quantising 6.7 G parameters on top of that takes seconds every time, although the result
only depends on the checkpoint and the format. This module writes the packed matrices once, next to the checkpoint
(`<MODEL_NAME>.<format>.abpack`), and later constructions map that file and copy the arrays straight to the device:
no fp32 copy of a matrix is made, neither on the host nor on the device, and the source tensors are touched only for
their fingerprints (a few pages each when the checkpoint is memory-mapped).

File layout (little endian):
    bytes 0..7      magic  b"ABPACK01"
    bytes 8..15     length n of the JSON header
    bytes 16..16+n  JSON: {"layout": LAYOUT_VERSION, "format": "int8" | "nvfp4" | "fp16",
                           "entries": {name: {"fingerprint": hex, "fmt", "n_out", "k", "tscale",
                                              "arrays": {"w" | "scale" | "col_scale": [offset, nbytes, dtype, shape]}}}}
    then the arrays, each starting on a 4096-byte boundary (offsets are relative to the start of the file).

An entry is used only if its fingerprint equals that of the source tensor presented at load time, the file's format
equals the requested one and the layout version is the current one; anything else is re-quantised (and the file is
rewritten with the fresh entries). The fingerprint covers shape, dtype, and — `mode="sample"` — 4096 evenly spaced
elements plus the first and last 64 (cheap on a memory-mapped checkpoint: a changed or re-trained tensor differs
there, a single flipped element elsewhere would not be seen) or — `mode="full"` — every byte of the tensor.
"""
from __future__ import annotations

import hashlib
import json
import os
import struct
from typing import Dict, Optional

import numpy as np
import torch

from . import _lib
from .quant import PackedMatrix

MAGIC = b"ABPACK01"
LAYOUT_VERSION = 1        # bump when the kernels' weight layout changes (nibble order, scale layout, ...)
ALIGN = 4096
_FMT_NAMES = {"int8": _lib.FMT_I8, "nvfp4": _lib.FMT_FP4, "fp16": _lib.FMT_F16, None: _lib.FMT_F16, "none": _lib.FMT_F16}
_NP = {"int8": np.int8, "uint8": np.uint8, "float16": np.float16, "float32": np.float32}


def fingerprint(t: torch.Tensor, mode: str = "sample") -> str:
    """Hex digest identifying the contents of a source tensor (see the module docstring for what `mode` covers)."""
    h = hashlib.blake2b(digest_size=16)
    h.update(repr((tuple(t.shape), str(t.dtype), mode)).encode())
    flat = t.detach().reshape(-1)
    n = flat.numel()
    if mode == "full" or n <= 8192:
        sample = flat
    else:
        idx = torch.linspace(0, n - 1, 4096, dtype=torch.float64).to(torch.int64)
        sample = torch.cat([flat[:64], flat[idx.to(flat.device)], flat[-64:]])
    h.update(sample.to("cpu").contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


class PackCache:
    """Reader and writer of one cache file. `get` returns a PackedMatrix on `device` or None; `put` records a freshly
    quantised matrix; `close` rewrites the file if anything was added or found stale."""

    def __init__(self, path: str, fmt: Optional[str], mode: str = "sample"):
        self.path, self.fmt, self.mode = path, ("fp16" if fmt in (None, "none") else fmt), mode
        self._entries: Dict[str, dict] = {}
        self._map: Optional[np.memmap] = None
        self._new: Dict[str, tuple] = {}        # name -> (fingerprint, PackedMatrix)
        self._dirty = False
        self.hits = self.misses = 0
        if os.path.exists(path):
            try:
                self._open()
            except (OSError, ValueError, KeyError, json.JSONDecodeError):
                self._entries, self._map, self._dirty = {}, None, True      # unreadable: start over

    def _open(self) -> None:
        with open(self.path, "rb") as f:
            head = f.read(16)
            if len(head) != 16 or head[:8] != MAGIC:
                raise ValueError("not a pack cache")
            (n,) = struct.unpack("<Q", head[8:])
            meta = json.loads(f.read(n).decode())
        if meta.get("layout") != LAYOUT_VERSION or meta.get("format") != self.fmt:
            self._dirty = True              # another layout or format: nothing is reusable
            return
        self._entries = meta["entries"]
        self._map = np.memmap(self.path, dtype=np.uint8, mode="c")   # private copy-on-write mapping: never written, but torch wants a writable buffer

    # ------------------------------------------------------------------------------------------
    def get(self, name: str, source: torch.Tensor, device) -> Optional[PackedMatrix]:
        e = self._entries.get(name)
        fp = fingerprint(source, self.mode)
        if e is None or e["fingerprint"] != fp or self._map is None:
            self.misses += 1
            self._dirty = True
            self._pending_fp = (name, fp)
            return None
        self.hits += 1
        arrs = {}
        for key, (off, nbytes, dtype, shape) in e["arrays"].items():
            view = self._map[off:off + nbytes].view(_NP[dtype]).reshape(shape)
            arrs[key] = torch.from_numpy(view).to(device, non_blocking=True)     # mapped file -> device, no host copy
        return PackedMatrix(int(e["fmt"]), int(e["n_out"]), int(e["k"]), arrs["w"], arrs.get("scale"),
                            arrs.get("col_scale"), float(e["tscale"]))

    def put(self, name: str, source: torch.Tensor, pm: PackedMatrix) -> None:
        pend = getattr(self, "_pending_fp", None)
        fp = pend[1] if pend and pend[0] == name else fingerprint(source, self.mode)
        self._new[name] = (fp, pm)
        self._dirty = True

    # ------------------------------------------------------------------------------------------
    def close(self) -> None:
        """Write the file if it is missing, stale or incomplete: kept entries are copied from the old mapping, new ones
        from the device. The new file replaces the old one atomically."""
        if not self._dirty and not self._new:
            return
        items = []   # (name, meta, {key: numpy array or (offset, nbytes) into the old map})
        for name, e in self._entries.items():
            if name not in self._new and self._map is not None:
                items.append((name, dict(e), {k: ("old",) + tuple(v) for k, v in e["arrays"].items()}))
        for name, (fp, pm) in self._new.items():
            arrays = {"w": pm.w}
            if pm.scale is not None:
                arrays["scale"] = pm.scale
            if pm.col_scale is not None:
                arrays["col_scale"] = pm.col_scale
            meta = {"fingerprint": fp, "fmt": int(pm.fmt), "n_out": int(pm.n_out), "k": int(pm.k), "tscale": float(pm.tscale)}
            items.append((name, meta, {k: ("new", v) for k, v in arrays.items()}))
        # header size is needed for the offsets: lay the arrays out after a generously sized header
        approx = 4096 + 512 * sum(len(a) for _, _, a in items) + 256 * len(items)
        data0 = (16 + approx + ALIGN - 1) // ALIGN * ALIGN
        off = data0
        for _, meta, arrays in items:
            meta["arrays"] = {}
            for key, src in arrays.items():
                if src[0] == "old":
                    _, _, nbytes, dtype, shape = src
                else:
                    t = src[1]
                    nbytes, dtype, shape = t.numel() * t.element_size(), str(t.dtype).replace("torch.", ""), list(t.shape)
                meta["arrays"][key] = [off, int(nbytes), dtype, list(shape)]
                off = (off + int(nbytes) + ALIGN - 1) // ALIGN * ALIGN
        header = json.dumps({"layout": LAYOUT_VERSION, "format": self.fmt,
                             "entries": {name: meta for name, meta, _ in items}}).encode()
        assert 16 + len(header) <= data0, "pack cache header larger than reserved"
        tmp = self.path + ".tmp%d" % os.getpid()
        with open(tmp, "wb") as f:
            f.write(MAGIC + struct.pack("<Q", len(header)) + header)
            for _, meta, arrays in items:
                for key, src in arrays.items():
                    f.seek(meta["arrays"][key][0])
                    if src[0] == "old":
                        f.write(self._map[src[1]:src[1] + src[2]].tobytes())
                    else:
                        f.write(src[1].detach().to("cpu").contiguous().view(torch.uint8).numpy().tobytes())
            f.truncate(max(off, f.tell()))
        self._map = None
        os.replace(tmp, self.path)
        self._new.clear()
        self._dirty = False
