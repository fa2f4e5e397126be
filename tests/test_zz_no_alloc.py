"""GPU: lmb_linear_static_scratch, the lut_linear entry point for callers that cannot allocate
device memory (a plugin inside a process whose framework owns the whole GPU memory pool, a
latency-bound thread that may not enter the driver's allocator).  It must give what lmb_linear
gives, call after call, although every call shares one built-in scratch array that still holds
the previous call's partial sums.  Collected last on purpose."""
import ctypes

import numpy as np
import pytest

from lutmac_b200 import _lib, synth
from lutmac_b200.blocks import INT4, TERNARY
from tests.conftest import rel_l2

pytestmark = pytest.mark.gpu


def device_synchronize():
    """Wait for every stream of the current CUDA context (the context's own stream is
    non-blocking, so it does not order itself against the default stream used below)."""
    assert ctypes.CDLL("libcuda.so.1").cuCtxSynchronize() == 0


def planned_k_slices(w, M, K):
    """K slices the planner cuts a batch-1 GEMV of this weight into (1 = the scratch is unused)."""
    out = (ctypes.c_int * 5)()
    _lib.check(_lib.lib().lmb_debug_plan_weight(w.h, 148, out))
    return out[3]


# (kind, M, K, must the planner split K?): the first and the last use the built-in array -- the last
# is the down projection of the 70B-shaped decoder, the largest split of the decoder shapes --
# the middle ones run in one slice and only exercise the entry point's plain path
@pytest.mark.parametrize("kind,M,K,split", [(INT4, 64, 8192, True), (TERNARY, 100, 4096, False), (INT4, 512, 2048, False),
                                            (TERNARY, 8192, 28672, True)])
def test_static_scratch_matches_lmb_linear_twice(ctx, oracle, kind, M, K, split):
    rng = np.random.default_rng(kind * 7 + M)
    t = synth.tensor(rng, kind, M, K)
    w = ctx.upload(t)
    if split:
        assert planned_k_slices(w, M, K) > 1, "this case is meant to go through the built-in scratch array"
    results = []
    for call in range(2):  # two calls in a row: the second one finds the first one's leftovers
        x = synth.activations(rng, K)
        dx = ctx.to_device(x)
        dy_ref, dy = ctx.malloc(M * 4), ctx.malloc(M * 4)
        dy.zero()
        ctx.linear(w, dx, dy_ref, flags=_lib.AUTO_ROTATE)
        want = dy_ref.download(np.float32)  # synchronises the context's stream
        # the new entry point takes no context: it runs on the stream it is given (here the
        # default stream)
        device_synchronize()
        _lib.check(_lib.lib().lmb_linear_static_scratch(w.h, None, dx.ptr, K, dy.ptr, _lib.AUTO_ROTATE, None))
        device_synchronize()
        got = dy.download(np.float32)
        assert rel_l2(got, want) < 1e-5, (call, rel_l2(got, want))
        assert rel_l2(got, oracle.lut_linear(kind, t.quant_bits, t.blocks, M, K, None, x)[0]) < 1e-5
        results.append(got)
    assert not np.array_equal(results[0], results[1])  # different inputs gave different outputs
    w.free()


def test_static_scratch_refuses_a_split_beyond_its_array(ctx_lut):
    ctx = ctx_lut  # table-lookup layout: at most 12 blocks of tables per CTA
    rng = np.random.default_rng(0)
    # 13 blocks per row exceed one CTA's table budget, so K is split at least in two:
    # >= 2 slices x 66016 padded rows > 131072 floats
    t = synth.ternary_tensor(rng, 66000, 3328)
    w = ctx.upload(t)
    dx, dy = ctx.malloc(t.K * 4), ctx.malloc(t.M * 4)
    st = _lib.lib().lmb_linear_static_scratch(w.h, None, dx.ptr, t.K, dy.ptr, 0, None)
    assert st == _lib.ERR_LIMIT
    assert b"512 KiB" in _lib.lib().lmb_last_error()
    w.free()
