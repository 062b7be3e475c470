"""Native host runtime: control-block validation and the graph-exec cache (host-only parts)."""
import ctypes as C

import pytest

from hipengine_b200.core import native


pytestmark = pytest.mark.skipif(not native.lib_available(), reason="native library not built")


def test_control_block_validation():
    from hipengine_b200.core import runtime as RT
    ok = RT.make_control(RT.STAGES_FULL_CYCLE, n_requests=2, depth=3)
    assert RT.validate(ok) == 0
    assert RT.validate(RT.make_control(RT.STAGE_DECODE_STEP, 8, 0)) == 0
    bad = RT.make_control(RT.STAGES_FULL_CYCLE, 2, 3)
    bad.magic = 1
    assert RT.validate(bad) == -2
    bad = RT.make_control(RT.STAGES_FULL_CYCLE, 2, 3)
    bad.struct_bytes -= 8
    assert RT.validate(bad) == -4
    assert RT.validate(RT.make_control(RT.STAGES_FULL_CYCLE, 0, 3)) == -6
    assert RT.validate(RT.make_control(RT.STAGES_FULL_CYCLE, 2, 17)) == -7
    assert RT.validate(RT.make_control(1 << 9, 2, 3)) == -8
    assert RT.validate(RT.make_control(RT.STAGE_DECODE_STEP | RT.STAGE_VERIFY, 2, 0)) == -9
    assert RT.validate(RT.make_control(RT.STAGE_PROPOSE, 2, 3)) == -10
    assert RT.validate(RT.make_control(RT.STAGE_VERIFY | RT.STAGE_COMMIT, 2, 3)) == -11
    assert RT.validate(RT.make_control(RT.STAGE_VERIFY | RT.STAGE_ACCEPT, 2, 0)) == -12
    # a refused block never reaches the device: launch returns the validation code and counts nothing
    res = RT.cycle_launch(bad, 0, 0)
    assert res.rc != 0 and res.launches == 0


def test_graph_exec_cache_bookkeeping():
    from hipengine_b200.core import runtime as RT
    cache = RT.GraphExecCache()
    cache.clear()
    e0, h0, m0 = cache.stats()
    assert e0 == 0
    assert cache.get(42) is None
    cache.put(42, 0xDEAD0000)
    assert cache.get(42) == 0xDEAD0000
    e, h, m = cache.stats()
    assert (e, h - h0, m - m0) == (1, 1, 1)
    assert cache.launch(7, 0) == -2                      # unknown bucket: refused, nothing launched
    assert cache.erase(42) and not cache.erase(42)
    cache.clear()
