"""CPU, world_size 2 and 4 over gloo: batch sharding bookkeeping and the pipeline schedule (with a fake stage)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from albatross_b200.dist import BatchShard, PipelineDecoder, shard_bounds, stage_layers


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _init(rank, world, port):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)


def test_shard_bounds_partition():
    for n in (1, 7, 320, 2560):
        for w in (1, 2, 3, 8):
            spans = [shard_bounds(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [h - l for l, h in spans]
            assert max(sizes) - min(sizes) <= 1
    assert [stage_layers(32, 4, s) for s in range(4)] == [(0, 8), (8, 16), (16, 24), (24, 32)]


def _shard_worker(rank, world, port, q):
    _init(rank, world, port)
    sh = BatchShard(7)
    mine = torch.arange(sh.lo, sh.hi) * 10
    allt = sh.gather_tokens(mine)
    q.put((rank, allt.tolist(), sh.local(list(range(7)))))
    dist.destroy_process_group()


def test_batch_shard_gather_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_shard_worker, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in ps]
    res = sorted(q.get(timeout=120) for _ in ps)
    [p.join(timeout=60) for p in ps]
    assert res[0][1] == res[1][1] == [i * 10 for i in range(7)]
    assert res[0][2] == [0, 1, 2, 3] and res[1][2] == [4, 5, 6]


def _pipe_worker(rank, world, port, q, n_micro, steps):
    """Fake model: stage s adds (s + 1) to x; v_first is set by stage 0 to 100 * token and must arrive
    unchanged at the last stage, which returns token' = x.sum() + v_first.sum() (mod 1000)."""
    _init(rank, world, port)
    b, D = 3, 4

    def stage_fn(mb, inp, v_first):
        if rank == 0:
            x = inp.float().unsqueeze(1).repeat(1, D)       # "embedding" of the token ids
            v_first = 100.0 * x
        else:
            x = inp
        x = x + (rank + 1)
        if rank == world - 1:
            return ((x.sum(1) + v_first.sum(1)).long() % 1000)
        return x, v_first

    pd = PipelineDecoder(stage_fn, n_micro, lambda mb: torch.empty(b, D), lambda mb: torch.empty(b, dtype=torch.long))
    toks = [torch.arange(b) + 10 * mb for mb in range(n_micro)] if rank == 0 else None
    hist = []
    for _ in range(steps):
        nxt = pd.step(toks)
        if rank == 0:
            hist.append([t.tolist() for t in nxt])
            toks = nxt
    q.put((rank, hist))
    dist.destroy_process_group()


@pytest.mark.parametrize("world,n_micro", [(2, 1), (2, 3), (4, 4)])
def test_pipeline_schedule_matches_sequential(world, n_micro):
    steps = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_pipe_worker, args=(r, world, port, q, n_micro, steps)) for r in range(world)]
    [p.start() for p in ps]
    res = dict(q.get(timeout=180) for _ in ps)
    [p.join(timeout=60) for p in ps]
    # sequential model of the same fake network
    b, D = 3, 4
    toks = [torch.arange(b) + 10 * mb for mb in range(n_micro)]
    want = []
    for _ in range(steps):
        nxt = []
        for t in toks:
            x = t.float().unsqueeze(1).repeat(1, D)
            vf = 100.0 * x
            for s in range(world):
                x = x + (s + 1)
            nxt.append((x.sum(1) + vf.sum(1)).long() % 1000)
        want.append([t.tolist() for t in nxt])
        toks = nxt
    assert res[0] == want
