"""The allocation-free entry point `candle_moe_forward_static`.

Some hosts cannot give the block a workspace: their device memory belongs to a pool of their own,
or they sit in a decode loop that must not risk an allocation.  For them the library carries a
fixed 16 MiB scratch array; this test drives that entry point through the C ABI and checks it
against the ordinary `candle_moe_forward` (caller-provided workspace) on the same inputs, twice in
a row, because the second call finds the first call's leftovers in the shared array.

The file name sorts last so that a run stopping at the first failure has already run every other
test.
"""
import ctypes as C

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def test_forward_static_matches_forward_twice(orc):
    import torch
    assert torch.cuda.is_available()
    from candle_b200 import _lib
    L = _lib.load()
    mw = orc.make_moe_weights(31, 512, 1024, 8, 2, orc.Q4K, orc.Q6K)
    blk = H.device_block(orc, mw)
    st = torch.cuda.current_stream().cuda_stream
    for call, T in enumerate((24, 7)):
        x = torch.from_numpy(orc.make_activations(40 + call, T, 512)).cuda()
        want = blk.forward(x).cpu().numpy()
        y = torch.full((T, 512), float("nan"), dtype=torch.float32, device="cuda")
        rc = L.candle_moe_forward_static(st, C.byref(blk._cw), x.data_ptr(), T, y.data_ptr())
        assert rc == 0, rc
        torch.cuda.synchronize()
        got = y.cpu().numpy()
        assert np.isfinite(got).all()
        assert H.max_rel(got, want) <= H.MAX_REL_TOL and H.rel_l2(got, want) <= H.REL_L2_TOL
        ref = orc.moe_forward(mw, x.cpu().numpy())  # and against the CPU oracle directly
        assert H.max_rel(got, ref.y) <= H.MAX_REL_TOL and H.rel_l2(got, ref.y) <= H.REL_L2_TOL


def test_forward_static_refuses_oversized_calls(orc):
    """More rows than the built-in scratch can serve: a clear error code, nothing enqueued."""
    import torch
    from candle_b200 import _lib
    L = _lib.load()
    mw = orc.make_moe_weights(32, 512, 1024, 8, 2, orc.Q4K, orc.Q6K)
    blk = H.device_block(orc, mw)
    T = 4096  # [T*k, ff] f32 alone is 32 MiB
    need = C.c_size_t(0)
    assert L.candle_moe_workspace_bytes(C.byref(blk._cw), T, C.byref(need)) == 0 and need.value > (16 << 20)
    x = torch.zeros((T, 512), dtype=torch.float32, device="cuda")
    y = torch.zeros_like(x)
    rc = L.candle_moe_forward_static(torch.cuda.current_stream().cuda_stream, C.byref(blk._cw), x.data_ptr(), T,
                                     y.data_ptr())
    assert rc == -7
    with pytest.raises(_lib.CandleMoeError, match="STATIC_SCRATCH"):
        _lib.check("candle_moe_forward_static", rc)
