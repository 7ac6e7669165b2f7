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
    first stage (it embeds the micro-batch's current tokens itself), and
    stage_fn(mb, x_in, v_first) -> next token ids [b] on the last stage.
    Buffers are [b, D] tensors created by `make_buffer(mb)`; token ids travel as int64 (`make_tokens(mb)`).

    Transport: point-to-point over torch.distributed. The two tensors of a stage boundary go out as ONE batched
    operation (`batch_isend_irecv`), and the token ids travel back from the last to the first stage on a process
    group of their own, so that the return path never queues behind (or in front of) the forward traffic of the same
    pair of ranks. Nothing waits for a send at the point where it is issued.
    """

    def __init__(self, stage_fn: Callable, n_micro: int, make_buffer: Callable[[int], torch.Tensor],
                 make_tokens: Callable[[int], torch.Tensor], group: Optional[dist.ProcessGroup] = None):
        self.stage_fn, self.n_micro = stage_fn, n_micro
        self.make_buffer, self.make_tokens = make_buffer, make_tokens
        self.group = group
        self.S = dist.get_world_size(group)
        self.s = dist.get_rank(group)
        self.first, self.last = self.s == 0, self.s == self.S - 1
        # every rank of the group calls this (new_group is collective); ranks are the global ranks of `group`
        self.back_group = None
        if self.S > 1:
            ranks = dist.get_process_group_ranks(group) if group is not None else list(range(self.S))
            self.back_group = dist.new_group(ranks=ranks)
        self._ranks = dist.get_process_group_ranks(group) if group is not None else list(range(self.S))

    def _peer(self, stage: int) -> int:
        return self._ranks[stage]

    def step(self, tokens: Optional[List[torch.Tensor]]) -> Optional[List[torch.Tensor]]:
        """One decode step for every micro-batch (see `run`)."""
        return self.run(tokens, 1)

    def run(self, tokens: Optional[List[torch.Tensor]], n_steps: int) -> Optional[List[torch.Tensor]]:
        """`n_steps` decode steps for every micro-batch, greedy / sampled inside `stage_fn` of the last stage.
        `tokens[mb]` (first stage only) are the current token ids. Returns the token ids that follow the last step per
        micro-batch on the first stage (received from the last stage), else None.

        Every stage walks the items (step, micro-batch) in the same order; a stage's receive for an item matches the
        previous stage's send for it. The first stage starts step t + 1 of a micro-batch as soon as that micro-batch's
        token ids of step t have come back, so with at least as many micro-batches as stages no stage idles between
        steps: there is no barrier per step."""
        sends = []      # (work handles, tensors kept alive) of everything sent in this call
        nxt: List[Optional[torch.Tensor]] = [None] * self.n_micro
        for t in range(n_steps):
            for mb in range(self.n_micro):
                x_in = v_first = None
                if self.first:
                    if t == 0:
                        cur = tokens[mb]
                    elif self.S > 1:
                        cur = self.make_tokens(mb)
                        dist.recv(cur, src=self._peer(self.S - 1), group=self.back_group)
                    else:
                        cur = nxt[mb]
                else:
                    x_in, v_first = self.make_buffer(mb), self.make_buffer(mb)
                    ops = [dist.P2POp(dist.irecv, x_in, self._peer(self.s - 1), self.group),
                           dist.P2POp(dist.irecv, v_first, self._peer(self.s - 1), self.group)]
                    for w in dist.batch_isend_irecv(ops):
                        w.wait()
                if self.last:
                    out = self.stage_fn(mb, x_in, v_first) if not self.first else self.stage_fn(mb, cur, None)
                    if self.S > 1:
                        sends.append((dist.isend(out, dst=self._peer(0), group=self.back_group), out))
                    else:
                        nxt[mb] = out
                else:
                    x_out, v_first = self.stage_fn(mb, cur if self.first else x_in, v_first)
                    ops = [dist.P2POp(dist.isend, x_out, self._peer(self.s + 1), self.group),
                           dist.P2POp(dist.isend, v_first, self._peer(self.s + 1), self.group)]
                    sends.append((dist.batch_isend_irecv(ops), (x_out, v_first)))
        if self.first and self.S > 1:
            for mb in range(self.n_micro):
                tk = self.make_tokens(mb)
                dist.recv(tk, src=self._peer(self.S - 1), group=self.back_group)
                nxt[mb] = tk
        for work, _keep in sends:
            for w in (work if isinstance(work, list) else [work]):
                w.wait()
        return nxt if self.first else None
