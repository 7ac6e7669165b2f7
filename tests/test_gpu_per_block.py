"""Block-by-block parity at the 7.2B shapes (baseline configs 3 and 4): every one of the 32 blocks, int8 and NVFP4.

A randomly initialised 32-block network amplifies rounding differences with depth, so comparing only the final
logits of two correct implementations says little. Here every block is checked on its own, teacher-forced: block i
of the library (a one-block pipeline stage, `layer_range=(i, i + 1)`) gets the ORACLE's input of block i (hidden
state, `v_first`) and its output, its new kv state and its two token-shift states are compared with the oracle's.
The same loop also feeds the library's own outputs forward (free-running), which gives the error as a function of
depth, and the last block's logits are compared as well.

  * batched kernels (tensor-core products, batched WKV): 320 sequences, two decode steps (the second step starts
    from a non-zero state);
  * batch-1 kernels (matrix-vector products, fused per-head WKV): sequence 0 alone, through the same stage entry
    point with option "stage_gemv".

The oracle here is oracle/rwkv7_oracle.py evaluated in fp32 on the GPU's own copy of the weights: the big
matrices are what the library's kernels de-quantise (`ab_dequant`, proved bit-identical to the numpy definition of
the formats in test_gpu_kernels.py), the small parameters are rounded to fp16 as reference/rwkv7.py:90 does.
Reference lines: reference/rwkv7.py:135-153 (single token), :198-216 (batch).
"""
import json
import os

import pytest
import torch

from albatross_b200 import RWKV_x070, synth
from albatross_b200.quant import PackedMatrix
from oracle.rwkv7_oracle import Oracle, is_big

pytestmark = pytest.mark.gpu

# Tolerances, all as max |ours - oracle| / max |oracle| over the tensor:
BLOCK_REL_TOL = 2e-2     # a block's output and its token-shift states, worst of the 320 sequences (the stated tolerance)
BLOCK_MEDIAN_TOL = 3e-3  # ... and the median sequence
STATE_REL_TOL = 5e-3     # the new kv state
LOGIT_REL_TOL = 2e-2     # the stated tolerance on fp16 logits
# Why the worst sequence is ten times the median: where a head's read-out y = S r nearly cancels (first steps from a zero
# state: y = v (k . r) with k . r close to 0), the group norm (eps 64e-5, reference/rwkv7.py:248, :298) turns the fp16
# rounding of r and k into a large relative change of that head's 64 outputs. The fp16 reference has the same
# sensitivity against an fp32 evaluation; it is a property of the input, identical in the batch-1 and batched kernels.
B, STEPS = 320, 2
CFG = "7.2b"


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-30))


def _block_keys(i, L):
    specs = list(synth.tensor_specs(*synth.CONFIGS[CFG][:3], synth.CONFIGS[CFG][3]))
    pre = f"blocks.{i}."
    for key, shape, dist in specs:
        if key.startswith(pre) and "ln0" not in key:
            yield key, shape, dist
        elif i == 0 and (key.startswith("emb.") or "ln0" in key):
            yield key, shape, dist
        elif i == L - 1 and (key.startswith("ln_out.") or key.startswith("head.")):
            yield key, shape, dist


def _oracle_z(model: RWKV_x070, raw: dict, i: int) -> dict:
    """The oracle's prepared weights of global block i, on the GPU, from the model's own packed matrices."""
    z = {}
    for key, t in raw.items():
        if is_big(key):
            local = key if not key.startswith("blocks.") else "blocks.0." + key.split(".", 2)[2]
            pm = model.z[local]
            assert isinstance(pm, PackedMatrix)
            z[key] = pm.dequantize().t()                       # [in, out] view of the [out, in] storage
        else:
            v = t.squeeze().to(torch.float16).float()          # reference/rwkv7.py:90 casts everything to fp16
            z[key] = v.flatten() if key.endswith("att.r_k") else v
    return z


@pytest.mark.parametrize("fmt", ["int8", "nvfp4"])
def test_every_block_of_the_7_2b_shapes_matches_the_oracle(fmt):
    L, D, V, _ = synth.CONFIGS[CFG]
    H = D // 64
    args = synth.make_args(CFG)
    dev = "cuda"
    g = torch.Generator().manual_seed(11)
    toks = torch.randint(0, V, (STEPS, B), generator=g)

    # oracle hidden state / v_first entering the current block, per step; the library's own (free-running) copies
    x_or = [None] * STEPS
    x_free = [None] * STEPS
    vf_or = [torch.zeros(B, 1, D, device=dev) for _ in range(STEPS)]
    vf_free = [torch.zeros(B, D, dtype=torch.float16, device=dev) for _ in range(STEPS)]
    report = {"fmt": fmt, "blocks": []}
    worst = {"x": 0.0, "x_median_row": 0.0, "kv": 0.0, "shift": 0.0, "x_gemv": 0.0, "kv_gemv": 0.0}
    logits_err = {}

    for i in range(L):
        raw = {k: synth.make_tensor(0, k, shape, dist, dev) for k, shape, dist in _block_keys(i, L)}
        model = RWKV_x070(args, quant=fmt, state_dict=raw, layer_range=(i, i + 1))
        z = _oracle_z(model, raw, i)
        if i == 0:     # both sides start from the embedding rows with ln0 folded in (reference/rwkv7.py:93, :132)
            emb = model.z["emb.weight"]                        # fp16, ln0 folded by the library at load
            for t in range(STEPS):
                x_or[t] = emb[toks[t].to(dev)].float().unsqueeze(1)       # [B,1,D]
                x_free[t] = emb[toks[t].to(dev)].clone()
            z.pop("emb.weight", None)
        o = Oracle(z, L, D)
        st_or = [torch.zeros(B, D, device=dev), torch.zeros(B, H, 64, 64, device=dev), torch.zeros(B, D, device=dev)]
        st_one = [torch.zeros(D, device=dev), torch.zeros(H, 64, 64, device=dev), torch.zeros(D, device=dev)]
        st_tf, st_fr = model.new_state(B), model.new_state(B)
        model.set_option("stage_gemv", 1)
        st_gv = model.new_state(1)
        blk = {"block": i}
        for t in range(STEPS):
            x_in = x_or[t][:, 0].to(torch.float16).contiguous()
            vf_in = vf_or[t][:, 0].to(torch.float16).contiguous()
            # ---- oracle, batch path and (sequence 0) single-token path, from the same inputs
            want, vfo = o.block_tokens(i, x_or[t], vf_or[t], st_or, 0)
            want1, _ = o.block_one(i, x_or[t][0, 0], vf_or[t][0, 0], st_one, 0)
            # ---- library, teacher-forced: batched kernels on all sequences, batch-1 kernels on sequence 0
            out = torch.empty(B, D, dtype=torch.float16, device=dev)
            logits = model.forward_stage(st_tf, vf_in, x_in=x_in, x_out=None if model.is_last else out)
            vf1 = vf_in[:1].clone()
            out1 = torch.empty(1, D, dtype=torch.float16, device=dev)
            logits1 = model.forward_stage(st_gv, vf1, x_in=x_in[:1].contiguous(), x_out=None if model.is_last else out1)
            # ---- library, free-running: its own previous outputs
            outf = torch.empty(B, D, dtype=torch.float16, device=dev)
            logits_f = model.forward_stage(st_fr, vf_free[t], x_in=x_free[t], x_out=None if model.is_last else outf)
            if model.is_last:
                ref = o.head_logits(want[:, 0])
                logits_err = {"teacher_forced": _rel(logits, ref), "free_running": _rel(logits_f, ref),
                              "batch1_kernels": _rel(logits1[0], o.head_logits(want1)),
                              "argmax_agree_teacher_forced": float((logits.argmax(-1) == ref.argmax(-1)).float().mean()),
                              "argmax_agree_free_running": float((logits_f.argmax(-1) == ref.argmax(-1)).float().mean())}
            else:
                row_err = (out.float() - want[:, 0]).abs().amax(1) / want.abs().max()
                e = {"x": _rel(out, want[:, 0]), "x_median_row": float(row_err.median()), "kv": _rel(st_tf[1], st_or[1]),
                     "shift": max(_rel(st_tf[0], st_or[0]), _rel(st_tf[2], st_or[2])),
                     "x_gemv": _rel(out1[0], want1), "kv_gemv": _rel(st_gv[1][0], st_one[1]),
                     "x_free": _rel(outf, want[:, 0])}
                blk[f"step{t}"] = e
                for k_ in worst:
                    worst[k_] = max(worst[k_], e[k_])
                x_free[t] = outf
            x_or[t], vf_or[t] = want, vfo
        report["blocks"].append(blk)
        del model, z, raw, o
        torch.cuda.empty_cache()

    report["worst_teacher_forced"] = worst
    report["logits"] = logits_err
    report["free_running_x_error_by_depth"] = {str(d): report["blocks"][d - 1][f"step{STEPS - 1}"]["x_free"]
                                               for d in (1, 2, 4, 8, 16, 31)}
    out_dir = os.environ.get("AB_TEST_REPORT_DIR", "")    # where to leave the figures as a file, if anywhere
    if out_dir and os.path.isdir(out_dir):
        with open(os.path.join(out_dir, f"per_block_parity_{fmt}.json"), "w") as f:
            json.dump(report, f, indent=1)
    print(fmt, "worst teacher-forced:", worst, "logits:", logits_err, "free-running by depth:",
          report["free_running_x_error_by_depth"])
    assert worst["x"] <= BLOCK_REL_TOL and worst["x_gemv"] <= BLOCK_REL_TOL, worst
    assert worst["x_median_row"] <= BLOCK_MEDIAN_TOL, worst
    assert worst["kv"] <= STATE_REL_TOL and worst["kv_gemv"] <= STATE_REL_TOL, worst
    assert worst["shift"] <= BLOCK_REL_TOL, worst
    assert logits_err["teacher_forced"] <= LOGIT_REL_TOL and logits_err["batch1_kernels"] <= LOGIT_REL_TOL, logits_err
