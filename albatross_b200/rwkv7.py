"""Drop-in `RWKV_x070` for the reference model class (reference/rwkv7.py:71-221).

Same constructor argument (`args.MODEL_NAME` without ".pth", `n_layer`, `n_embd`, `head_size`,
`vocab_size`), same `forward(idx, state, full_output=False)` / `forward_batch(idxs, state,
full_output=False)` signatures, same state-list layout (3 tensors per layer, reference/rwkv7.py:102-105
and :122-125) and the same checkpoint key schema. Differences a caller can observe:

  * the big matrices (`att.{receptance,key,value,output}.weight`, `ffn.{key,value}.weight`,
    `head.weight`) are quantised at load (`quant="int8" | "nvfp4"`, or kept fp16 with `quant=None`);
    `model.z[...]` holds `PackedMatrix` objects for them (their `numel()` still counts parameters,
    which is what reference benchmark.py:49-51 reads);
  * every state tensor is updated IN PLACE (the reference replaces the two x_prev entries and, on
    the single-token path, the kv entry); the returned list is a new list of the same tensors;
  * kernels run on the current torch stream (the reference kernel uses the legacy default stream).

All arithmetic runs in the CUDA library bound by `_lib`; there is no PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib
from .quant import PackedMatrix, pack_fp16, quantize

HEAD_SIZE = 64
DTYPE = torch.half
_BIG = ("att.receptance.weight", "att.key.weight", "att.value.weight", "att.output.weight",
        "ffn.key.weight", "ffn.value.weight", "head.weight")


def _is_big(name: str) -> bool:
    return any(name.endswith(s) for s in _BIG)


# --------------------------------------------------------------------------------------------
# Operator-level wrappers (reference/rwkv7.py:37-67)
# --------------------------------------------------------------------------------------------
def _wkv(B, T, C_, state, r, w, k, v, a, b):
    H = C_ // HEAD_SIZE
    assert HEAD_SIZE == C_ // H
    assert all(x.dtype == DTYPE for x in [r, w, k, v, a, b])
    assert all(x.is_contiguous() for x in [r, w, k, v, a, b])
    assert state.dtype == torch.float32 and state.is_contiguous() and state.is_cuda
    y = torch.empty_like(r)
    _lib.check(_lib.lib.ab_wkv7_fwd(B, T, C_, H, state.data_ptr(), r.data_ptr(), w.data_ptr(), k.data_ptr(),
                                    v.data_ptr(), a.data_ptr(), b.data_ptr(), y.data_ptr(),
                                    torch.cuda.current_stream().cuda_stream), "ab_wkv7_fwd")
    return y


def RWKV7_OP(state, r, w, k, v, a, b):
    """WKV-7 over a [T, C] sequence; `state` [H,64,64] fp32 is updated in place (reference/rwkv7.py:37-50)."""
    T, C_ = r.size()
    return _wkv(1, T, C_, state, r, w, k, v, a, b)


def RWKV7_BATCH_OP(state, r, w, k, v, a, b):
    """WKV-7 over [B, T, C]; `state` [B,H,64,64] fp32 is updated in place (reference/rwkv7.py:52-67)."""
    B, T, C_ = r.size()
    return _wkv(B, T, C_, state, r, w, k, v, a, b)


def sampler_simple_batch(logits: torch.Tensor, noise: float = 1.0, seed: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Next-token ids [B, 1] (int64) from fp16 logits [B, V] on the device: argmax of logits + U(0, noise), as
    reference/utils.py:43-45 computes with an argsort. `seed` selects the noise (vary it per step). `out`: an int64
    tensor of B elements to write the ids into, on the device or in pinned host memory (the kernel then stores them
    straight to the host: read them after synchronising the stream)."""
    assert logits.dim() == 2 and logits.dtype == DTYPE and logits.is_cuda and logits.is_contiguous()
    if out is None:
        out = torch.empty((logits.shape[0], 1), dtype=torch.int64, device=logits.device)
    assert out.dtype == torch.int64 and out.numel() == logits.shape[0] and out.is_contiguous() and (out.is_cuda or out.is_pinned())
    _lib.check(_lib.lib.ab_sample_rows_i64(logits.data_ptr(), logits.shape[0], logits.shape[1], float(noise), int(seed) & 0xFFFFFFFF,
                                           out.data_ptr(), torch.cuda.current_stream().cuda_stream), "ab_sample_rows_i64")
    return out.view(logits.shape[0], 1)


class _State(list):
    """The state list forward() hands back. It remembers which model has validated it and which decode program
    belongs to its tensors, so that the next forward() with it skips both look-ups (96 tensors at 32 blocks: 40 us of
    Python per token otherwise); any in-place change of the list forgets that."""
    __slots__ = ("_ab",)

    def __init__(self, items=(), ab=None):
        super().__init__(items)
        self._ab = ab

    def _changed(name):
        def f(self, *a, **k):
            self._ab = None
            return getattr(list, name)(self, *a, **k)
        f.__name__ = name
        return f

    for _n in ("__setitem__", "__delitem__", "__iadd__", "__imul__", "append", "extend", "insert", "pop", "remove", "clear",
               "sort", "reverse"):
        locals()[_n] = _changed(_n)
    del _n, _changed


# --------------------------------------------------------------------------------------------
# Model
# --------------------------------------------------------------------------------------------
class RWKV_x070:
    def __init__(self, args, quant: Optional[str] = "int8", state_dict: Optional[Iterable[Tuple[str, torch.Tensor]]] = None,
                 device: str = "cuda", use_graph: bool = True, decode_mode: Optional[str] = None,
                 layer_range: Optional[Tuple[int, int]] = None, pack_cache=None):
        if not torch.cuda.is_available():
            raise RuntimeError("albatross_b200 needs a CUDA device (sm_100a); there is no CPU path")
        self.args = args
        self.n_embd = args.n_embd
        # layer_range = (first, last+1): hold only these blocks (one stage of a layer pipeline); the embedding
        # table is kept by the stage with block 0, the final norm and head by the stage with the last block
        self.layer_range = tuple(layer_range) if layer_range is not None else (0, args.n_layer)
        self.total_layers = args.n_layer
        self.n_layer = self.layer_range[1] - self.layer_range[0]
        self.is_first = self.layer_range[0] == 0
        self.is_last = self.layer_range[1] == args.n_layer
        self.quant = quant
        self.device = torch.device(device)
        self.use_graph = use_graph and os.environ.get("ALBATROSS_NO_GRAPH", "0") != "1"
        # batch-1 decode: "persistent" = one resident kernel per token; "graph" = one launch per phase,
        # replayed from a CUDA graph; "eager" = one launch per phase from the host
        self.decode_mode = decode_mode or os.environ.get("ALBATROSS_DECODE_MODE") or ("persistent" if self.use_graph else "eager")
        assert self.decode_mode in ("persistent", "graph", "eager")

        items = state_dict
        # pack_cache: path of the file that keeps the quantised matrices between runs (packcache.py). Loading from
        # a `.pth` file uses `<MODEL_NAME>.<format>.abpack` next to it unless pack_cache=False (or the environment
        # says ALBATROSS_PACK_CACHE=0); with an in-memory state dict a path must be given explicitly.
        if pack_cache is None:
            pack_cache = items is None and quant is not None and os.environ.get("ALBATROSS_PACK_CACHE", "1") != "0"
        if pack_cache is True:
            pack_cache = "%s.%s.abpack" % (args.MODEL_NAME, quant or "fp16") if items is None else None
        self._cache = None
        if pack_cache:
            from .packcache import PackCache
            self._cache = PackCache(str(pack_cache), quant, mode=os.environ.get("ALBATROSS_PACK_CACHE_MODE", "sample"))
        if items is None:
            # memory-mapped: a tensor's pages are read when it is used, so the checkpoint streams through block by
            # block and matrices served by the pack cache are never read beyond their fingerprint samples
            items = torch.load(args.MODEL_NAME + ".pth", map_location="cpu", mmap=True).items()
        elif isinstance(items, dict):
            items = items.items()
        self.z: Dict[str, object] = {}
        self._extra: Dict[str, object] = {}
        lo, hi = self.layer_range
        for name, t in items:
            if name.startswith("blocks."):
                li = int(name.split(".")[1])
                if "ln0" in name:
                    if not self.is_first:
                        continue
                elif not (lo <= li < hi):
                    continue
                else:
                    name = "blocks.%d.%s" % (li - lo, name.split(".", 2)[2])   # local block index
            elif name.startswith("emb."):
                if not self.is_first:
                    continue
            elif not self.is_last:      # ln_out.*, head.weight
                continue
            self._ingest(name, t)
        if self._cache is not None:
            self.pack_cache_stats = (self._cache.hits, self._cache.misses)
            try:
                self._cache.close()
            except OSError:      # read-only model directory: run without writing the cache
                pass
            self._cache = None
        z = self.z
        self.n_head, self.head_size = self._r_k_shape
        assert HEAD_SIZE == self.head_size
        assert self.head_size == args.head_size
        # ln0 is folded into the embedding table once (reference/rwkv7.py:93)
        if self.is_first:
            z["emb.weight"] = F.layer_norm(z["emb.weight"], (args.n_embd,), weight=z["blocks.0.ln0.weight"],
                                           bias=z["blocks.0.ln0.bias"]).contiguous()
            for s in ("0", "1", "2"):  # layer 0 never uses its v adapter (reference/rwkv7.py:94-96, :239)
                z["blocks.0.att.v" + s] = z["blocks.0.att.a" + s]
        self.vocab = z["emb.weight"].shape[0] if self.is_first else (z["head.weight"].n_out if self.is_last else args.vocab_size)
        self._build_native()
        self._ws: Dict[Tuple[int, int], torch.Tensor] = {}
        self._graphs: Dict[tuple, tuple] = {}
        self._programs: Dict[tuple, tuple] = {}
        self._options: Dict[str, int] = {}
        # token ids travel host -> device from a ring of pinned slots; a slot is reused only after the
        # asynchronous copy that read it has completed, so callers need not synchronise between steps
        self._tok_ring = torch.empty(64, dtype=torch.int32).pin_memory()
        self._tok_events = [None] * 64
        self._tok_n = 0

    # ---- load-time preparation (reference/rwkv7.py:86-96) -----------------------------------
    def _ingest(self, name: str, t: torch.Tensor) -> None:
        dev = self.device
        if _is_big(name):
            # storage is [out, in] row-major; the reference views it as [in, out]. Quantise per output row.
            if self._cache is not None:
                pm = self._cache.get(name, t, dev)
                if pm is None:
                    pm = quantize(t.to(dev, non_blocking=True), self.quant)
                    self._cache.put(name, t, pm)
                self.z[name] = pm
                return
            w = t.to(dev, non_blocking=True)
            self.z[name] = quantize(w, self.quant)
            return
        t = t.to(dev).squeeze().to(DTYPE)
        if name.endswith("att.r_k"):
            self._r_k_shape = tuple(t.shape)
            t = t.flatten()
        self.z[name] = t.contiguous()
        # adapter matrices in kernel layout
        leaf = name.rsplit(".", 1)[-1]
        if leaf in ("w1", "a1", "v1", "g1"):   # [D, rank] -> rows of [rank, D]
            self._extra[name + "t"] = pack_fp16(self.z[name].t().contiguous())
        elif leaf in ("w2", "a2", "v2", "g2"):  # [rank, D] -> rows of [D, rank] for the batched path
            self._extra[name + "t"] = pack_fp16(self.z[name].t().contiguous())

    def _build_native(self) -> None:
        z, ex = self.z, self._extra
        L = self.n_layer
        self._layers = (_lib.Layer * L)()
        empty = _lib.Mat()
        for i in range(L):
            b, a, f = f"blocks.{i}.", f"blocks.{i}.att.", f"blocks.{i}.ffn."
            ly = self._layers[i]
            ptr = lambda key: z[key].data_ptr()
            ly.ln1_w, ly.ln1_b, ly.ln2_w, ly.ln2_b = ptr(b + "ln1.weight"), ptr(b + "ln1.bias"), ptr(b + "ln2.weight"), ptr(b + "ln2.bias")
            for c in "rwkvag":
                setattr(ly, "x_" + c, ptr(a + "x_" + c))
            for n in ("w0", "a0", "v0", "k_k", "k_a", "r_k"):
                setattr(ly, n, ptr(a + n))
            ly.lnx_w, ly.lnx_b, ly.ffn_x_k = ptr(a + "ln_x.weight"), ptr(a + "ln_x.bias"), ptr(f + "x_k")
            ly.receptance, ly.key = z[a + "receptance.weight"].as_mat(), z[a + "key.weight"].as_mat()
            ly.value, ly.output = z[a + "value.weight"].as_mat(), z[a + "output.weight"].as_mat()
            ly.ffn_key, ly.ffn_value = z[f + "key.weight"].as_mat(), z[f + "value.weight"].as_mat()
            for n in ("w", "a", "v", "g"):
                if n == "v" and i == 0 and self.is_first:
                    setattr(ly, "v1t", empty)
                    setattr(ly, "v2t", empty)
                    ly.v2 = None
                    continue
                setattr(ly, n + "1t", ex[a + n + "1t"].as_mat())
                setattr(ly, n + "2t", ex[a + n + "2t"].as_mat())
                setattr(ly, n + "2", ptr(a + n + "2"))
        d = _lib.ModelDesc()
        d.n_layer, d.n_embd, d.vocab = L, self.n_embd, self.vocab
        if self.is_first:
            d.emb = z["emb.weight"].data_ptr()
        if self.is_last:
            d.lnout_w, d.lnout_b = z["ln_out.weight"].data_ptr(), z["ln_out.bias"].data_ptr()
            d.head = z["head.weight"].as_mat()
        d.layers = C.cast(self._layers, C.POINTER(_lib.Layer))
        self._desc = d
        h = C.c_void_p()
        _lib.check(_lib.lib.ab_model_create(C.byref(d), C.byref(h)), "ab_model_create")
        self._handle = h
        if self.layer_range[0] > 0:
            _lib.check(_lib.lib.ab_model_set_option(h, b"layer_offset", self.layer_range[0]), "ab_model_set_option")

    def __del__(self):
        h = getattr(self, "_handle", None)
        if h and _lib is not None and getattr(_lib, "lib", None) is not None:
            _lib.lib.ab_model_destroy(h)
            self._handle = None

    def set_option(self, name: str, value: int) -> None:
        _lib.check(_lib.lib.ab_model_set_option(self._handle, name.encode(), int(value)), "ab_model_set_option")
        self._options[name] = int(value)
        self._graphs.clear()
        self._programs.clear()

    # ---- state ------------------------------------------------------------------------------
    def new_state(self, batch: Optional[int] = None) -> List[torch.Tensor]:
        """Zero state in the reference's layout (reference/rwkv7.py:100-105, :120-125); a pipeline stage holds
        the entries of its own blocks only."""
        args, lead = self.args, (() if batch is None else (batch,))
        st: List[torch.Tensor] = []
        for _ in range(self.n_layer):  # state: 0=att_x_prev 1=att_kv 2=ffn_x_prev
            st.append(torch.zeros(lead + (args.n_embd,), dtype=DTYPE, device=self.device))
            st.append(torch.zeros(lead + (args.n_embd // args.head_size, args.head_size, args.head_size),
                                  dtype=torch.float, device=self.device))
            st.append(torch.zeros(lead + (args.n_embd,), dtype=DTYPE, device=self.device))
        return st

    def _check_state(self, state: List[torch.Tensor], batch: Optional[int]) -> None:
        ab = getattr(state, "_ab", None)
        if ab is not None and ab[0] is self and ab[1] == batch:
            return                                  # validated when this model handed the list out, unchanged since
        D, H = self.n_embd, self.n_embd // HEAD_SIZE
        lead = () if batch is None else (batch,)
        assert len(state) == 3 * self.n_layer, "state must hold 3 tensors per layer"
        for i, t in enumerate(state):
            want = lead + ((H, HEAD_SIZE, HEAD_SIZE) if i % 3 == 1 else (D,))
            dt = torch.float32 if i % 3 == 1 else DTYPE
            assert tuple(t.shape) == want and t.dtype == dt and t.is_cuda and t.is_contiguous(), \
                f"state[{i}]: expected {want} {dt} contiguous on CUDA, got {tuple(t.shape)} {t.dtype}"

    def _workspace(self, B: int, T: int) -> torch.Tensor:
        key = (B, T)
        ws = self._ws.get(key)
        if ws is None:
            n = _lib.lib.ab_workspace_bytes(self._handle, B, T)
            ws = torch.zeros(n + 256, dtype=torch.uint8, device=self.device)   # split-K counters start at zero
            self._ws = {k: v for k, v in self._ws.items() if k == (1, 1)}  # keep the decode workspace only
            self._ws[key] = ws
        return ws

    def _run(self, B: int, T: int, tokens_dev: torch.Tensor, state: List[torch.Tensor], logits: torch.Tensor,
             full_output: bool) -> None:
        ws = self._workspace(B, T)
        base = (ws.data_ptr() + 255) & ~255
        ptrs = (C.c_void_p * len(state))(*[t.data_ptr() for t in state])
        _lib.check(_lib.lib.ab_forward(self._handle, B, T, tokens_dev.data_ptr(), ptrs, base, logits.data_ptr(),
                                       int(full_output), torch.cuda.current_stream().cuda_stream), "ab_forward")

    def _check_ids(self, ids) -> None:
        """Token ids are validated on the host, where they still are Python numbers: an id outside the embedding
        table raises IndexError as `z['emb.weight'][idx]` does in the reference (reference/rwkv7.py:132, :163,
        :195). (The kernels clamp such an id and set a status bit all the same; they never read past the table.)"""
        flat = ids if isinstance(ids, (list, tuple)) else [ids]
        if flat and isinstance(flat[0], (list, tuple)):
            lo = min(min(r) for r in flat)
            hi = max(max(r) for r in flat)
        else:
            lo, hi = min(flat), max(flat)
        if lo < -self.vocab or hi >= self.vocab:
            raise IndexError(f"token id {lo if lo < -self.vocab else hi} is out of range for a vocabulary of {self.vocab}")

    def _wrap_id(self, idx: int) -> int:
        return int(idx) + self.vocab if idx < 0 else int(idx)     # torch indexing counts negative ids from the end

    # ---- the reference's public entry points ------------------------------------------------
    def forward(self, idx, state, full_output=False):
        if state is None:
            state = self.new_state()
        if type(idx) is list:
            if len(idx) > 1:
                return self.forward_seq(idx, state, full_output)
            return self.forward_one(idx[0], state)
        return self.forward_one(idx, state)

    def forward_batch(self, idxs, state, full_output=False):
        assert type(idxs) is list
        assert len(set([len(x) for x in idxs])) == 1, 'currently all token inputs in a batch must have the same length'
        if state is None:
            state = self.new_state(len(idxs))
        return self.forward_seq_batch(idxs, state, full_output)

    @torch.no_grad()
    def forward_one(self, idx: int, state: List[torch.Tensor]):
        self._check_state(state, None)
        self._check_ids(idx)
        idx = self._wrap_id(idx)
        if self.decode_mode == "persistent":
            return self._forward_one_persistent(idx, state)
        if self.decode_mode == "eager":
            tok = torch.tensor([int(idx)], dtype=torch.int32, device=self.device)
            logits = torch.empty(self.vocab, dtype=DTYPE, device=self.device)
            self._run(1, 1, tok, state, logits, False)
            return logits, self._hand_back(state, None)
        key = self._state_key(state)
        entry = self._graphs.get(key)
        if entry is None:
            entry = self._capture(state)
            if len(self._graphs) >= 4:
                self._graphs.pop(next(iter(self._graphs)))
            self._graphs[key] = entry
        graph, tok_dev, logits_buf = entry
        self._send_token(idx, tok_dev)
        graph.replay()
        return logits_buf.clone(), _State(state, (self, None, key))

    def _send_token(self, idx: int, tok_dev: torch.Tensor) -> None:
        slot = self._tok_n % 64
        self._tok_n += 1
        ev = self._tok_events[slot]
        if ev is not None:
            ev.synchronize()
        self._tok_ring[slot] = int(idx)
        tok_dev.copy_(self._tok_ring[slot:slot + 1], non_blocking=True)
        if ev is None:
            ev = self._tok_events[slot] = torch.cuda.Event()
        ev.record()

    def _hand_back(self, state: List[torch.Tensor], batch: Optional[int]):
        """The caller's next state: the same tensors (updated in place) in a list that remembers this model's checks."""
        return _State(state, (self, batch, self._state_key(state)))

    def _state_key(self, state: List[torch.Tensor]):
        ab = getattr(state, "_ab", None)
        if ab is not None and ab[0] is self:
            return ab[2]
        return tuple(t.data_ptr() for t in state)

    def _program_for(self, state: List[torch.Tensor]):
        key = self._state_key(state)
        entry = self._programs.get(key)
        if entry is None:
            tok_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
            logits_buf = torch.empty(self.vocab, dtype=DTYPE, device=self.device)
            prog = torch.zeros(_lib.lib.ab_decode_program_bytes(self._handle) + 256, dtype=torch.uint8, device=self.device)
            prog_ptr = (prog.data_ptr() + 255) & ~255
            ws = self._workspace(1, 1)
            ptrs = (C.c_void_p * len(state))(*[t.data_ptr() for t in state])
            _lib.check(_lib.lib.ab_decode_program_build(self._handle, tok_dev.data_ptr(), ptrs, (ws.data_ptr() + 255) & ~255,
                                                        logits_buf.data_ptr(), prog_ptr,
                                                        torch.cuda.current_stream().cuda_stream), "ab_decode_program_build")
            if len(self._programs) >= 4:
                self._programs.pop(next(iter(self._programs)))
            entry = self._programs[key] = (prog, prog_ptr, tok_dev, logits_buf)
        return entry

    def decode_timeline(self, state: List[torch.Tensor]):
        """Per-phase (start, end) timestamps in ns of the last persistent decode step on `state`, as seen by
        block 0; needs set_option("timeline", 1) before the program for `state` was built."""
        prog, prog_ptr, _, _ = self._program_for(state)
        merged = self._options.get("merge_ups", 0) and self.n_head <= 148
        fused = self._options.get("fuse_heads", 1) and not self._options.get("merge_ups", 0) and 2 * self.n_head + 4 <= 148
        per_block = 5 if (merged or fused) else 6
        n = per_block * self.n_layer + 1
        hdr = _lib.lib.ab_decode_timeline_offset(self._handle)
        off = (prog_ptr - prog.data_ptr()) + hdr
        torch.cuda.synchronize()
        raw = prog[off:off + 48 * n].view(torch.int64).cpu().numpy()
        self.last_timeline_detail = raw[2 * n:].reshape(n, 4)   # per phase: input ready, prepared, streamed, reduced
        return raw[:2 * n].reshape(n, 2)

    def decode_timeline_all(self, state: List[torch.Tensor]):
        """Timestamps of every block for the last persistent decode step on `state`: array [blocks, phases, 6] of ns
        (phase start, phase end, inputs arrived, inputs prepared, weights streamed, partial sums reduced); needs
        set_option("timeline", 1) and set_option("timeline_block", -1) before the program was built."""
        prog, prog_ptr, _, _ = self._program_for(state)
        fused = self._options.get("fuse_heads", 1) and not self._options.get("merge_ups", 0) and 2 * self.n_head + 4 <= 148
        n = (5 if (fused or self._options.get("merge_ups", 0)) else 6) * self.n_layer + 1
        stride = 6 * (6 * self.n_layer + 1)
        off = (prog_ptr - prog.data_ptr()) + _lib.lib.ab_decode_timeline_offset(self._handle)
        torch.cuda.synchronize()
        n_blocks = torch.cuda.get_device_properties(self.device).multi_processor_count   # one block per SM
        raw = prog[off:off + 8 * stride * n_blocks].view(torch.int64).cpu().numpy().reshape(n_blocks, stride)
        import numpy as np
        return np.concatenate([raw[:, :2 * n].reshape(n_blocks, n, 2), raw[:, 2 * n:6 * n].reshape(n_blocks, n, 4)], axis=2)

    def _forward_one_persistent(self, idx: int, state: List[torch.Tensor]):
        key = self._state_key(state)
        _, prog_ptr, tok_dev, logits_buf = self._program_for(state)
        self._send_token(idx, tok_dev)
        _lib.check(_lib.lib.ab_decode_run(self._handle, prog_ptr, torch.cuda.current_stream().cuda_stream), "ab_decode_run")
        return logits_buf.clone(), _State(state, (self, None, key))

    def _capture(self, state: List[torch.Tensor]):
        """Record one decode step (all launches of ab_forward at B=T=1) into a CUDA graph.

        Capture replays nothing: the state is not touched until the first replay. A warm-up step on
        a scratch copy of the state runs first so that lazy one-time set-up inside the library
        (function attributes) happens outside the capture."""
        tok_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
        logits_buf = torch.empty(self.vocab, dtype=DTYPE, device=self.device)
        scratch = [t.clone() for t in state]
        self._run(1, 1, tok_dev, scratch, logits_buf, False)
        torch.cuda.synchronize()
        del scratch
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._run(1, 1, tok_dev, state, logits_buf, False)
        return graph, tok_dev, logits_buf

    @torch.no_grad()
    def forward_seq(self, idx: List[int], state: List[torch.Tensor], full_output: bool = False):
        self._check_state(state, None)
        T = len(idx)
        self._check_ids(idx)
        tok = torch.tensor([self._wrap_id(t) for t in idx], dtype=torch.int32, device=self.device)
        logits = torch.empty((T, self.vocab) if full_output else (self.vocab,), dtype=DTYPE, device=self.device)
        self._run(1, T, tok, state, logits, full_output)
        return logits, self._hand_back(state, None)

    @torch.no_grad()
    def forward_seq_batch(self, idxs: List[List[int]], state: List[torch.Tensor], full_output: bool = False):
        B, T = len(idxs), len(idxs[0])
        self._check_state(state, B)
        tok = torch.tensor(idxs, dtype=torch.int64)
        lo, hi = torch.aminmax(tok)                  # the range check of _check_ids, on the tensor (B * T ids)
        if int(lo) < -self.vocab or int(hi) >= self.vocab:
            self._check_ids(idxs)                    # raises the IndexError with the offending id
        tok = torch.where(tok < 0, tok + self.vocab, tok).to(torch.int32)
        if T == 1 and B > 1 and self.use_graph:
            return self._forward_batch_graph(B, tok, state)
        tok = tok.to(self.device)
        shape = (B, T, self.vocab) if full_output else (B, self.vocab)
        logits = torch.empty(shape, dtype=DTYPE, device=self.device)
        self._run(B, T, tok, state, logits, full_output)
        return logits, self._hand_back(state, B)

    def _forward_batch_graph(self, B: int, tok_host: torch.Tensor, state: List[torch.Tensor]):
        """One batched decode step (T = 1) replayed from a CUDA graph: the ~260 launches of the step, and the tensor
        maps the products encode on the host for every launch, are recorded once per (batch, state tensors)."""
        skey = self._state_key(state)
        key = (B,) + skey
        entry = self._graphs.get(key)
        if entry is None:
            tok_dev = torch.zeros(B, dtype=torch.int32, device=self.device)
            logits_buf = torch.empty(B, self.vocab, dtype=DTYPE, device=self.device)
            pinned = torch.empty(B, dtype=torch.int32).pin_memory()
            scratch = [t.clone() for t in state]         # warm-up outside the capture (lazy one-time set-up in the library)
            self._run(B, 1, tok_dev, scratch, logits_buf, False)
            torch.cuda.synchronize()
            del scratch
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self._run(B, 1, tok_dev, state, logits_buf, False)
            if len(self._graphs) >= 4:
                self._graphs.pop(next(iter(self._graphs)))
            # the entry keeps the workspace the launches were recorded with alive (the model may replace its own
            # reference when another shape comes along)
            entry = self._graphs[key] = (graph, tok_dev, logits_buf, pinned, torch.cuda.Event(), self._ws[(B, 1)])
        graph, tok_dev, logits_buf, pinned, ev, _ws = entry
        ev.synchronize()                                  # the copy that read the pinned ids last step has completed
        pinned.copy_(tok_host.view(-1))
        tok_dev.copy_(pinned, non_blocking=True)
        ev.record()
        graph.replay()
        return logits_buf.clone(), _State(state, (self, B, skey))

    # ---- sequences of unequal length: prefill one by one, decode together -----------------------------------
    # The reference cannot batch prompts of different lengths (reference/rwkv7.py:116-117 asserts equal lengths) nor
    # move a sequence in or out of a running batch. Every sequence owns an independent recurrent state, so both are
    # state bookkeeping: prefill each prompt on its own (`forward`, T = its length), copy its 3 * n_layer state tensors
    # into a slot of the batched state, and step the batch with `forward_batch`.
    @staticmethod
    def insert_state(batch_state: List[torch.Tensor], slot: int, seq_state: List[torch.Tensor]) -> None:
        """Copy a single-sequence state (tensors without batch dimension) into slot `slot` of a batched state, in place."""
        assert len(batch_state) == len(seq_state)
        for dst, src in zip(batch_state, seq_state):
            assert dst.shape[1:] == src.shape and dst.dtype == src.dtype, "state layouts differ"
            dst[slot].copy_(src)

    @staticmethod
    def extract_state(batch_state: List[torch.Tensor], slot: int) -> List[torch.Tensor]:
        """The state of the sequence in slot `slot` as a single-sequence state (a copy)."""
        return [t[slot].clone() for t in batch_state]

    @torch.no_grad()
    def prefill_batch(self, prompts: List[List[int]], state: Optional[List[torch.Tensor]] = None,
                      slots: Optional[List[int]] = None):
        """Prefill prompts of any lengths and return (logits [len(prompts), V], batched state).

        With `state` / `slots` given, the sequences are written into those slots of an existing batched state (a
        finished sequence's slot is reused by a new prompt while the others keep decoding); otherwise a new batched
        state with one slot per prompt is made. Prompts of equal length are prefilled together."""
        assert type(prompts) is list and all(type(p) is list and len(p) > 0 for p in prompts)
        if state is None:
            state = self.new_state(len(prompts))
            slots = list(range(len(prompts)))
        assert slots is not None and len(slots) == len(prompts)
        logits = torch.empty(len(prompts), self.vocab, dtype=DTYPE, device=self.device)
        by_len: Dict[int, List[int]] = {}
        for i, p in enumerate(prompts):
            by_len.setdefault(len(p), []).append(i)
        for T, idxs in by_len.items():
            if len(idxs) == 1 or T == 1:
                for i in idxs:
                    lg, st = self.forward(prompts[i] if T > 1 else prompts[i][0], None)
                    logits[i] = lg
                    self.insert_state(state, slots[i], st)
            else:
                lg, st = self.forward_batch([prompts[i] for i in idxs], None)
                logits[idxs] = lg
                for j, i in enumerate(idxs):
                    self.insert_state(state, slots[i], [t[j] for t in st])
        return logits, state

    @torch.no_grad()
    def forward_stage(self, state: List[torch.Tensor], v_first: torch.Tensor, tokens: Optional[torch.Tensor] = None,
                      x_in: Optional[torch.Tensor] = None, x_out: Optional[torch.Tensor] = None):
        """One pipeline stage of a batched decode step (T = 1). The first stage takes `tokens` (int32 [B] on
        the device), later stages `x_in` (fp16 [B, D]); `v_first` (fp16 [B, D]) is written by the first stage
        and read by the others; every stage but the last fills `x_out`, the last returns logits [B, V]."""
        B = v_first.shape[0]
        self._check_state(state, B)
        ws = self._workspace(B, 1)
        ptrs = (C.c_void_p * len(state))(*[t.data_ptr() for t in state])
        logits = None
        if self.is_last:
            logits = torch.empty(B, self.vocab, dtype=DTYPE, device=self.device)
        _lib.check(_lib.lib.ab_forward_stage(
            self._handle, B, 1, None if tokens is None else tokens.data_ptr(), None if x_in is None else x_in.data_ptr(),
            v_first.data_ptr(), ptrs, (ws.data_ptr() + 255) & ~255, None if x_out is None else x_out.data_ptr(),
            None if logits is None else logits.data_ptr(), torch.cuda.current_stream().cuda_stream), "ab_forward_stage")
        return logits

    # ---- bookkeeping for benchmarks ---------------------------------------------------------
    def packed_matrices(self, suffix: str) -> List[PackedMatrix]:
        """The packed matrices whose checkpoint key ends in `suffix`, in block order (e.g. "ffn.key.weight")."""
        keys = sorted((k for k, v in self.z.items() if k.endswith(suffix) and isinstance(v, PackedMatrix)),
                      key=lambda k: int(k.split(".")[1]) if k.startswith("blocks.") else -1)
        return [self.z[k] for k in keys]

    def matrix_params(self) -> int:
        """Multiply-accumulates per sequence and step: elements of every matrix a decode step multiplies by."""
        n = 0
        for k, v in self.z.items():
            if isinstance(v, PackedMatrix):
                n += v.n_out * v.k
            elif k.split(".")[-1] in ("w1", "w2", "a1", "a2", "v1", "v2", "g1", "g2") and not k.startswith("blocks.0.att.v"):
                n += v.numel()
        return n

    def weight_bytes(self, include_emb: bool = False) -> int:
        """Bytes a decode step streams: every tensor except the embedding table (cf. benchmark.py:47-52)."""
        n = 0
        for k, v in self.z.items():
            if "emb" in k and not include_emb:
                continue
            if k.startswith("blocks.0.att.v") and k[-2:] in ("v0", "v1", "v2"):
                continue
            if "ln0" in k:
                continue
            n += v.nbytes() if isinstance(v, PackedMatrix) else v.numel() * v.element_size()
        return n
