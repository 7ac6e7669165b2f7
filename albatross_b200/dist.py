"""Multi-GPU decode for RWKV-7: batch sharding and a layer pipeline (one process per GPU).

The reference is single-process and single-GPU (reference/rwkv7.py hard-codes device "cuda"); both modes here
are additions that follow from the model's structure:

* batch sharding — every sequence owns its RNN state (state tensors carry a leading batch dimension,
  reference/rwkv7.py:123-125) and the weights are read-only, so each rank keeps a full copy of the weights and a
  slice of the batch. No collective runs inside a decode step.
* layer pipeline — rank s holds blocks [s*L/S, (s+1)*L/S). Two [B, D] fp16 tensors cross each stage boundary
  per step: the hidden state x and v_first (the value projection of block 0, read by every later block,
  reference/rwkv7.py:239-240, :292-293). The last stage sends the sampled token ids [B] back to the first.
  Micro-batches keep the stages busy: sequences are independent, so splitting the batch is exact.

The transport is torch.distributed point-to-point (NCCL over NVLink on GPUs; gloo in the CPU tests). The
scheduling logic takes the per-stage computation as a callable, so it is tested without a GPU.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced split of n items: the first n % world ranks get one more."""
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def stage_layers(n_layer: int, n_stages: int, stage: int) -> Tuple[int, int]:
    """Blocks [first, last+1) of a pipeline stage."""
    return shard_bounds(n_layer, n_stages, stage)


class BatchShard:
    """Rank-local view of a globally batched decode: which sequences this rank owns, and optional
    gathering of the per-step results (token ids) for logging. The decode step itself needs no communication."""

    def __init__(self, global_batch: int, group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.global_batch = global_batch
        self.lo, self.hi = shard_bounds(global_batch, self.world, self.rank)

    @property
    def local_batch(self) -> int:
        return self.hi - self.lo

    def local(self, items: Sequence):
        return items[self.lo:self.hi]

    def gather_tokens(self, local_tokens: torch.Tensor) -> torch.Tensor:
        """All ranks' next-token ids in global sequence order (ranks may own different counts)."""
        if self.world == 1:
            return local_tokens
        counts = [shard_bounds(self.global_batch, self.world, r) for r in range(self.world)]
        width = max(h - l for l, h in counts)
        pad = torch.zeros(width, dtype=local_tokens.dtype, device=local_tokens.device)
        pad[:local_tokens.numel()] = local_tokens
        out = [torch.empty_like(pad) for _ in range(self.world)]
        dist.all_gather(out, pad, group=self.group)
        return torch.cat([o[:h - l] for o, (l, h) in zip(out, counts)])


class PipelineDecoder:
    """Decode steps through S pipeline stages with M micro-batches in flight.

    stage_fn(mb, x_in, v_first) -> (x_out, v_first) for stages other than the last, where x_in is None on the
    first stage (it embeds the micro-batch's current tokens itself, via `tokens_of(mb)`), and
    stage_fn(mb, x_in, v_first) -> next token ids [b] on the last stage.
    Buffers are [b, D] tensors created by `make_buffer(mb)`; token ids travel as int64.
    """

    def __init__(self, stage_fn: Callable, n_micro: int, make_buffer: Callable[[int], torch.Tensor],
                 make_tokens: Callable[[int], torch.Tensor], group: Optional[dist.ProcessGroup] = None):
        self.stage_fn, self.n_micro = stage_fn, n_micro
        self.make_buffer, self.make_tokens = make_buffer, make_tokens
        self.group = group
        self.S = dist.get_world_size(group)
        self.s = dist.get_rank(group)
        self.first, self.last = self.s == 0, self.s == self.S - 1

    def step(self, tokens: Optional[List[torch.Tensor]]) -> Optional[List[torch.Tensor]]:
        """One decode step for every micro-batch. `tokens[mb]` (first stage only) are the current token ids.
        Returns the next token ids per micro-batch on the first stage (received from the last), else None.

        Order: every stage walks the micro-batches in order; a stage's receive for micro-batch mb matches the
        previous stage's send for mb, so the stages overlap on different micro-batches."""
        nxt = [None] * self.n_micro
        pending = []   # token ids on their way back to the first stage (non-blocking: the first stage is still
                       # busy sending later micro-batches forward and receives them after its own loop)
        for mb in range(self.n_micro):
            x_in = v_first = None
            if not self.first:
                x_in, v_first = self.make_buffer(mb), self.make_buffer(mb)
                dist.recv(x_in, src=self.s - 1, group=self.group)
                dist.recv(v_first, src=self.s - 1, group=self.group)
            if self.last:
                out = self.stage_fn(mb, x_in, v_first) if not self.first else self.stage_fn(mb, tokens[mb], None)
                if self.S > 1:
                    pending.append((dist.isend(out, dst=0, group=self.group), out))
                else:
                    nxt[mb] = out
            else:
                x_out, v_first = self.stage_fn(mb, tokens[mb] if self.first else x_in, v_first)
                dist.send(x_out, dst=self.s + 1, group=self.group)
                dist.send(v_first, dst=self.s + 1, group=self.group)
        for req, _keep in pending:
            req.wait()
        if self.first and self.S > 1:
            for mb in range(self.n_micro):
                t = self.make_tokens(mb)
                dist.recv(t, src=self.S - 1, group=self.group)
                nxt[mb] = t
        return nxt if self.first else None
