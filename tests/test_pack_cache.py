"""CPU: the on-disk cache of packed matrices round-trips bit for bit and notices a changed tensor."""
import os

import torch

from albatross_b200 import packcache, quant


def _mats(seed):
    g = torch.Generator().manual_seed(seed)
    return {"blocks.0.att.key.weight": torch.randn(64, 128, generator=g) * 0.02,
            "blocks.0.ffn.value.weight": torch.randn(128, 256, generator=g) * 0.02,
            "head.weight": torch.randn(512, 128, generator=g) * 0.02}


def _same(a: quant.PackedMatrix, b: quant.PackedMatrix) -> bool:
    ok = (a.fmt, a.n_out, a.k, a.tscale) == (b.fmt, b.n_out, b.k, b.tscale) and torch.equal(a.w.cpu(), b.w.cpu())
    for x, y in ((a.scale, b.scale), (a.col_scale, b.col_scale)):
        ok = ok and ((x is None and y is None) or torch.equal(x.cpu(), y.cpu()))
    return ok


def test_round_trip_and_invalidation(tmp_path):
    for fmt in ("int8", "nvfp4"):
        path = str(tmp_path / f"m.{fmt}.abpack")
        src = _mats(0)
        c = packcache.PackCache(path, fmt)
        fresh = {}
        for name, t in src.items():
            assert c.get(name, t, "cpu") is None                   # nothing cached yet
            fresh[name] = quant.quantize(t, fmt)
            c.put(name, t, fresh[name])
        c.close()
        assert os.path.exists(path)
        # second load: every matrix comes from the file, bit for bit what the quantiser produced
        c = packcache.PackCache(path, fmt)
        for name, t in src.items():
            got = c.get(name, t, "cpu")
            assert got is not None and _same(got, fresh[name])
        assert (c.hits, c.misses) == (3, 0)
        c.close()
        # one tensor changed (a different checkpoint under the same name): that entry alone is stale
        src2 = dict(src)
        src2["head.weight"] = src["head.weight"] * 1.5
        c = packcache.PackCache(path, fmt)
        assert c.get("blocks.0.att.key.weight", src2["blocks.0.att.key.weight"], "cpu") is not None
        assert c.get("head.weight", src2["head.weight"], "cpu") is None
        new = quant.quantize(src2["head.weight"], fmt)
        c.put("head.weight", src2["head.weight"], new)
        c.close()
        c = packcache.PackCache(path, fmt)
        assert _same(c.get("head.weight", src2["head.weight"], "cpu"), new)
        assert _same(c.get("blocks.0.ffn.value.weight", src["blocks.0.ffn.value.weight"], "cpu"), fresh["blocks.0.ffn.value.weight"])
        c.close()
        # a file written for another format is not reused
        other = "nvfp4" if fmt == "int8" else "int8"
        c = packcache.PackCache(path, other)
        assert c.get("head.weight", src2["head.weight"], "cpu") is None


def test_full_fingerprint_sees_a_single_changed_element():
    t = torch.zeros(100000)
    u = t.clone()
    u[12345] = 1.0
    assert packcache.fingerprint(t, "full") != packcache.fingerprint(u, "full")
    assert packcache.fingerprint(t, "sample") == packcache.fingerprint(t.clone(), "sample")
    assert packcache.fingerprint(t, "sample") != packcache.fingerprint(t.to(torch.float16), "sample")


def test_corrupt_file_is_ignored(tmp_path):
    path = str(tmp_path / "bad.abpack")
    with open(path, "wb") as f:
        f.write(b"not a cache")
    c = packcache.PackCache(path, "int8")
    t = torch.randn(16, 32)
    assert c.get("head.weight", t, "cpu") is None
    c.put("head.weight", t, quant.quantize(t, "int8"))
    c.close()
    c = packcache.PackCache(path, "int8")
    assert c.get("head.weight", t, "cpu") is not None
