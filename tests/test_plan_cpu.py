"""CPU: the block partition of the matrix-vector kernels (host-side planner of the library, no GPU needed)."""
import ctypes as C

import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from albatross_b200 import _lib, synth

F16, I8, FP4 = 0, 1, 2


def _check(fmt, rows, k, n_blocks):
    n = len(fmt)
    arr = lambda v: (C.c_int32 * n)(*v)
    items, spread = C.c_int32(0), C.c_int32(0)
    rc = _lib.lib.ab_gemv_plan_selftest(arr(fmt), arr(rows), arr(k), n, n_blocks, C.byref(items), C.byref(spread))
    assert rc == 0, _lib.lib.ab_last_error().decode()
    return items.value, spread.value


@pytest.mark.parametrize("cfg", ["tiny", "0.1b", "7.2b"])
@pytest.mark.parametrize("big", [I8, FP4])
def test_every_phase_of_the_decode_program_is_covered(cfg, big):
    L, D, V, (rw, ra, rv, rg) = synth.CONFIGS[cfg]
    phases = {
        "rkv+downs": ([big] * 3 + [F16] * 4, [D] * 3 + [rw, ra, rv, rg], [D] * 7),
        "ups": ([F16] * 4, [D] * 4, [rw, ra, rv, rg]),
        "output": ([big], [D], [D]),
        "ffn key": ([big], [4 * D], [D]),
        "ffn value": ([big], [D], [4 * D]),
        "head": ([big], [V], [D]),
    }
    for name, (fmt, rows, k) in phases.items():
        items, spread = _check(fmt, rows, k, 148)
        assert items >= 1, name
        if cfg == "7.2b":
            assert spread <= 12, (name, spread)      # the most loaded block is at most 12 % above the mean cost


@settings(max_examples=60, deadline=None)
@given(st.lists(st.tuples(st.sampled_from([F16, I8, FP4]), st.integers(1, 3000), st.integers(1, 64)), min_size=1, max_size=7),
       st.integers(1, 200))
def test_random_segment_lists_are_covered_exactly_once(segs, n_blocks):
    fmt = [s[0] for s in segs]
    rows = [s[1] for s in segs]
    k = [s[2] * 32 for s in segs]          # NVFP4 rows need k % 32 == 0
    _check(fmt, rows, k, n_blocks)


def test_state_list_forgets_its_checks_when_changed():
    """The list forward() hands back carries the model's validation and program key; any in-place change of the list
    drops them, so a changed list is checked from scratch (it is still a plain list to its user)."""
    from albatross_b200.rwkv7 import _State
    owner = object()
    mark = (owner, None, (1, 2, 3))
    for change in (lambda s: s.__setitem__(0, "x"), lambda s: s.append("x"), lambda s: s.pop(), lambda s: s.extend(["y"]),
                   lambda s: s.insert(0, "z"), lambda s: s.clear(), lambda s: s.reverse(), lambda s: s.__delitem__(0),
                   lambda s: s.__iadd__(["w"])):
        st = _State(["a", "b", "c"], mark)
        assert st._ab is mark and isinstance(st, list) and list(st) == ["a", "b", "c"]
        change(st)
        assert st._ab is None
    st = _State(["a", "b"], mark)
    assert st[1] == "b" and len(st) == 2 and st._ab is mark          # reading keeps them
    assert not hasattr(list(st), "_ab") and _State(st)._ab is None   # a copy starts unchecked
