"""GPU parity of the GEMV / lut_linear / FWHT path against the CPU oracle and the reference
fixtures, through the C ABI.  Tolerance: 1e-5 relative L2 for float outputs (fp32
accumulation); integer artefacts (bit-planes, LUT indices, re-tiled codes) bit-exact.
"""
import os

import numpy as np
import pytest

from lutmac_b200 import _lib, api, synth
from lutmac_b200.blocks import (BINARY, BLOCK_DTYPES, INT2, INT3, INT4, INT5, INT6, INT8, KIND_NAMES, TERNARY, PackedTensor,
                                blocks_per_row)
from tests.conftest import rel_l2

pytestmark = pytest.mark.gpu

TOL = 1e-5
KINDS = (TERNARY, BINARY, INT2, INT3, INT4, INT5, INT6, INT8)
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
GEMV_SHAPES = ((1, 4), (3, 256), (16, 256), (33, 300), (40, 768), (64, 2048))


def gold(name):
    return np.load(os.path.join(GOLD, name + ".npz"))


def run_linear(ctx, t, x, batch=1, bias=None, flags=0, x_len=None):
    w = ctx.upload(t)
    dx = ctx.to_device(np.ascontiguousarray(x, np.float32))
    dy = ctx.malloc(batch * t.M * 4)
    db = ctx.to_device(bias) if bias is not None else None
    xl = t.K if x_len is None else x_len
    ctx.linear(w, dx, dy, batch=batch, bias=db, flags=flags, x_len=xl, x_stride=xl)
    y = dy.download(np.float32).reshape(batch, t.M)
    w.free()
    return y


# ---- reference fixtures through the kernel API -----------------------------------------------------

@pytest.mark.parametrize("kind", KINDS)
def test_gemv_host_matches_reference_fixtures(kind):
    g = gold("gemv")
    for (M, K) in GEMV_SHAPES:
        key = f"{KIND_NAMES[kind]}_{M}x{K}"
        blocks = g[key + "_blocks"].view(BLOCK_DTYPES[kind])
        y = api.GEMV_BY_KIND[kind](blocks, blocks.size, g[key + "_x"], None, M, K)
        want = g[key + "_y"]
        # tiny outputs (M <= 3) can hold a near-cancelled element; bound those absolutely too
        assert rel_l2(y, want) < TOL or np.max(np.abs(y - want)) < 1e-6, (key, rel_l2(y, want))


def test_lut_linear_matches_reference_fixtures(ctx):
    g = gold("linear")
    for i in range(int(g["n_cases"][0])):
        kind, qb, M, K, batch, has_bias = (int(v) for v in g[f"lin{i}_meta"])
        if kind not in KINDS:
            continue
        t = PackedTensor(kind, g[f"lin{i}_blocks"].view(BLOCK_DTYPES[kind]), M, K, quant_bits=qb)
        bias = g[f"lin{i}_bias"] if has_bias else None
        y = api.lut_linear(t, bias, g[f"lin{i}_x"], None, batch, ctx=ctx)
        assert rel_l2(y, g[f"lin{i}_y"]) < TOL, (i, KIND_NAMES[kind])


def test_reference_known_answers(ctx, oracle):
    # tests/test_lut_gemm.cpp:135-165 (=10), :218-260 (=-6.5), :262-307 (=0)
    x = np.zeros(256, np.float32)
    x[:4] = [1, 2, 3, 4]
    b = oracle.quantize(TERNARY, np.ones((1, 4), np.float32))
    assert api.lut_gemv(b, 1, x, None, 1, 4)[0] == pytest.approx(10.0, abs=1e-6)
    w = np.array([((i % 15) - 7) * 0.5 for i in range(32)], np.float32).reshape(1, 32)
    x = np.zeros(256, np.float32)
    x[:32] = 1.0
    assert api.int4_gemv(oracle.quantize(INT4, w), 1, x, None, 1, 32)[0] == pytest.approx(-6.5, abs=0.01)
    w = np.array([1.0 if i % 2 == 0 else -1.0 for i in range(256)], np.float32).reshape(1, 256)
    assert abs(api.lut_gemv_binary(oracle.quantize(BINARY, w), 1, np.ones(256, np.float32), None, 1, 256)[0]) <= 1.0


# ---- CUDA vs oracle on seeded inputs -----------------------------------------------------------------

EDGE_SHAPES = [(1, 256), (3, 4), (16, 512), (31, 768), (32, 256), (33, 1000), (100, 2048), (257, 300), (520, 1536)]


@pytest.mark.parametrize("kind", KINDS)
def test_gemv_vs_oracle_edge_shapes(ctx, oracle, kind):
    rng = np.random.default_rng(100 + kind)
    for (M, K) in EDGE_SHAPES:
        t = synth.tensor(rng, kind, M, K)
        kp = blocks_per_row(K) * 256
        x = synth.activations(rng, kp)
        y = run_linear(ctx, t, x, x_len=kp)[0]
        want = oracle.gemv(kind, t.blocks, x, M, K)
        err = rel_l2(y, want)
        assert err < TOL or np.max(np.abs(y - want)) < 1e-6, (KIND_NAMES[kind], M, K, err)


@pytest.mark.parametrize("kind,M,K", [(TERNARY, 2048, 2048), (INT4, 2048, 2048), (INT4, 512, 2048),
                                      (INT4, 8192, 2048), (INT4, 2048, 8192), (INT2, 1536, 1536),
                                      (INT2, 8960, 1536), (INT2, 1536, 8960), (INT8, 4096, 2048),
                                      (TERNARY, 1024, 8192), (TERNARY, 512, 28672), (BINARY, 2048, 2048),
                                      (INT3, 2048, 2048)])
def test_gemv_vs_oracle_config_shapes(ctx, oracle, kind, M, K):
    rng = np.random.default_rng(7)
    t = synth.tensor(rng, kind, M, K)
    x = synth.activations(rng, blocks_per_row(K) * 256)
    y = run_linear(ctx, t, x, x_len=x.size)[0]
    want = oracle.gemv_rows_parallel(kind, t.blocks, x, M, K, 8)
    truth = oracle.gemv_f64(kind, t.blocks, x, M, K)
    assert rel_l2(y, want) < TOL
    assert rel_l2(y, truth) < TOL


# (R row tiles per CTA, K slices, row groups per cluster): clusters of 2 / 4 / 8 CTAs that share the
# conversion of the activations and / or add up their K slices through distributed shared memory;
# (8, 2, 0) and (2, 4, 0) are the same splits through the global scratch buffer
FORCED_PLANS = ((8, 1, 2), (8, 1, 8), (4, 1, 4), (8, 2, 1), (8, 2, 2), (8, 4, 2), (4, 2, 4), (2, 8, 1), (1, 4, 1), (1, 1, 8), (8, 2, 0), (2, 4, 0))


@pytest.mark.parametrize("kind", (TERNARY, INT2, INT4, INT8, BINARY, INT3, INT5, INT6))
def test_every_work_split_gives_the_same_result(ctx, oracle, kind):
    """Thread-block clusters change where partial sums and converted activations travel, not the
    arithmetic: K slices are added in slice order either way, so a cluster split is bit-identical
    to the same split through global scratch, and all of them match the oracle."""
    rng = np.random.default_rng(300 + kind)
    L = _lib.lib()
    try:
        for (M, K) in ((1000, 2048), (70, 2300), (4096, 8192)):
            t = synth.tensor(rng, kind, M, K)
            x = synth.activations(rng, blocks_per_row(K) * 256)
            want = oracle.gemv_rows_parallel(kind, t.blocks, x, M, K, 8)
            got = {}
            for plan in FORCED_PLANS:
                _lib.check(L.lmb_debug_force_plan(*plan))
                y = run_linear(ctx, t, x, x_len=x.size)[0]
                got[plan] = y
                assert rel_l2(y, want) < TOL, (KIND_NAMES[kind], M, K, plan, rel_l2(y, want))
                if K % 256 == 0 and kind in (TERNARY, INT2, BINARY):  # lut_linear rotates these (lut_gemm_scalar.cpp:92-93)
                    yr = run_linear(ctx, t, x, x_len=x.size, flags=_lib.AUTO_ROTATE)[0]
                    wr = oracle.lut_linear(kind, t.quant_bits, t.blocks, M, K, None, x)[0]
                    assert rel_l2(yr, wr) < TOL, (KIND_NAMES[kind], M, K, plan, "rotated", rel_l2(yr, wr))
            if K == 8192:  # both splits are feasible for 32 blocks per row
                assert np.array_equal(got[(8, 2, 1)], got[(8, 2, 0)]), (KIND_NAMES[kind], "cluster split-K differs from scratch split-K")
                assert np.array_equal(got[(8, 2, 2)], got[(8, 2, 0)]), KIND_NAMES[kind]
    finally:
        _lib.check(L.lmb_debug_force_plan(0, 0, 0))


def test_config1_ternary_gemv_and_linear(ctx, oracle):
    t, x = synth.config1(seed=0)
    y = run_linear(ctx, t, x)[0]
    assert rel_l2(y, oracle.gemv(TERNARY, t.blocks, x, t.M, t.K)) < TOL
    yl = run_linear(ctx, t, x, flags=_lib.AUTO_ROTATE)[0]
    assert rel_l2(yl, oracle.lut_linear(TERNARY, t.quant_bits, t.blocks, t.M, t.K, None, x)[0]) < TOL
    assert rel_l2(yl, y) > 1e-2  # the rotation really changes the result


@pytest.mark.parametrize("kind", KINDS)
def test_lut_linear_pad_rotate_bias_batch(ctx, oracle, kind):
    rng = np.random.default_rng(200 + kind)
    for (M, K, batch) in ((40, 300, 3), (64, 1024, 2), (7, 4, 1)):
        t = synth.tensor(rng, kind, M, K)
        x = np.concatenate([synth.activations(rng, K) for _ in range(batch)])
        bias = rng.standard_normal(M).astype(np.float32)
        y = api.lut_linear(t, bias, x, None, batch, ctx=ctx).reshape(batch, M)
        want = oracle.lut_linear(kind, t.quant_bits, t.blocks, M, K, bias, x, batch)
        assert rel_l2(y, want) < TOL, (KIND_NAMES[kind], M, K, batch)


# ---- integer artefacts: bit-exact -----------------------------------------------------------------------

@pytest.mark.parametrize("kind", KINDS)
def test_device_weight_roundtrip_bit_exact(ctx, kind):
    rng = np.random.default_rng(300 + kind)
    for (M, K) in ((33, 300), (64, 512)):
        t = synth.tensor(rng, kind, M, K)
        w = ctx.upload(t)
        back = w.download()
        for f in BLOCK_DTYPES[kind].names:
            assert np.array_equal(back[f], t.blocks[f]), (KIND_NAMES[kind], f)
        w.free()


def test_ternary_lut_indices_bit_exact(ctx_lut, oracle):
    ctx = ctx_lut
    rng = np.random.default_rng(5)
    t = synth.ternary_tensor(rng, 40, 512)
    w = ctx.upload(t)
    idx = w.ternary_indices()
    for r in (0, 7, 39):
        for b in range(2):
            blk = t.blocks[r * 2 + b]
            for g in range(64):
                assert tuple(idx[r, b, g]) == oracle.extract_indices(blk["sign_plane"], blk["zero_plane"], g)
    w.free()


def test_lut_tables_and_fwht_bit_exact(ctx, oracle):
    rng = np.random.default_rng(6)
    x = synth.activations(rng, 1024)
    assert np.array_equal(api.debug_luts(ctx, x, False), oracle.precompute_luts(x))
    xr = oracle.apply_hadamard_rotation(x)
    assert np.array_equal(api.debug_luts(ctx, x, True), oracle.precompute_luts(xr))
    y = x.copy()
    api.apply_hadamard_rotation(y)
    assert np.array_equal(y, xr)
    g = gold("transform")
    z = g["fwht_in"].copy()
    api.apply_hadamard_rotation(z)
    assert np.array_equal(z, g["fwht_out"])  # includes the untouched trailing partial block


def test_errors_are_reported(ctx):
    rng = np.random.default_rng(1)
    t = synth.int4_tensor(rng, 8, 256)
    with pytest.raises(ValueError):
        api.int4_gemv(t.blocks, t.blocks.size, np.zeros(100, np.float32), None, 8, 256)
    with pytest.raises(_lib.LutmacError):
        _lib.check(_lib.lib().lmb_weight_upload(ctx.h, 77, t.blocks.ctypes.data, 8, 256, None))


@pytest.mark.parametrize("kind", (INT4, TERNARY, INT2))
def test_prepared_group_equals_single_launches(ctx, oracle, kind):
    """q/k/v/o/gate/up/down-like shapes of one layer issued as ONE launch."""
    rng = np.random.default_rng(400 + kind)
    shapes = [(256, 512), (64, 512), (64, 512), (256, 512), (1024, 512), (1024, 512), (512, 1024), (33, 300)]
    ts = [synth.tensor(rng, kind, M, K) for M, K in shapes]
    xs = [synth.activations(rng, K) for _, K in shapes]
    ws = [ctx.upload(t) for t in ts]
    dxs = [ctx.to_device(x) for x in xs]
    dys = [ctx.malloc(t.M * 4) for t in ts]
    grp = api.Group(ctx, ws, dxs, dys)
    for _ in range(2):  # twice: split-K counters must be back at zero after a launch
        for dy in dys:
            dy.zero()
        grp.launch()
        for t, x, dy in zip(ts, xs, dys):
            want = oracle.lut_linear(kind, t.quant_bits, t.blocks, t.M, t.K, None, x)[0]
            assert rel_l2(dy.download(np.float32), want) < TOL, (KIND_NAMES[kind], t.M, t.K)


def test_split_k_is_deterministic(ctx):
    rng = np.random.default_rng(11)
    t = synth.int4_tensor(rng, 64, 8192)  # few rows, many blocks: K is split over CTAs
    x = synth.activations(rng, 8192)
    ys = [run_linear(ctx, t, x)[0] for _ in range(3)]
    assert np.array_equal(ys[0], ys[1]) and np.array_equal(ys[0], ys[2])


def test_host_group_matches_oracle(ctx, oracle):
    rng = np.random.default_rng(77)
    shapes = [(256, 512), (64, 512), (1024, 512), (512, 1024), (33, 300)]
    ts = [synth.int4_tensor(rng, M, K) for M, K in shapes]
    ws = [ctx.upload(t) for t in ts]
    hg = api.HostGroup(ctx, ws)
    for _ in range(2):
        xs = [synth.activations(rng, K) for _, K in shapes]
        outs = hg.run(xs)
        for t, x, y in zip(ts, xs, outs):
            assert rel_l2(y, oracle.lut_linear(INT4, 4, t.blocks, t.M, t.K, None, x)[0]) < TOL


@pytest.mark.parametrize("kind,qbits", [(TERNARY, 2), (INT2, 2), (BINARY, 1), (INT3, 3)])
@pytest.mark.parametrize("which", ["mma", "lut"])
def test_both_device_layouts(ctx, ctx_lut, oracle, which, kind, qbits):
    """Ternary, INT2 and binary weights run on the integer tensor-core kernel by default and on
    the table-lookup kernel on request; both must match the oracle, with and without rotation,
    and download bit-exactly."""
    c = ctx if which == "mma" else ctx_lut
    rng = np.random.default_rng(21)
    for (M, K) in EDGE_SHAPES + [(2048, 2048), (1024, 8192)]:
        t = synth.tensor(rng, kind, M, K)
        x = synth.activations(rng, K)
        for flags in (0, _lib.AUTO_ROTATE):
            y = run_linear(c, t, x, flags=flags)[0]
            want = (oracle.lut_linear(kind, qbits, t.blocks, M, K, None, x)[0] if flags
                    else oracle.gemv(kind, t.blocks, np.pad(x, (0, blocks_per_row(K) * 256 - K)), M, K))
            err = rel_l2(y, want)
            assert err < TOL or np.max(np.abs(y - want)) < 1e-6, (which, M, K, flags, err)
    t = synth.tensor(rng, kind, 70, 768)
    w = c.upload(t)
    back = w.download()
    for f in BLOCK_DTYPES[kind].names:
        assert np.array_equal(back[f], t.blocks[f]), f
    w.free()


@pytest.mark.parametrize("kind,qbits", [(INT4, 4), (TERNARY, 2), (INT2, 2), (BINARY, 1), (INT8, 8), (INT5, 5), (INT6, 6), (INT3, 3)])
def test_batched_sequences_share_the_weight_pass(ctx, oracle, kind, qbits):
    """Batches of 2, 4 and 8 sequences are evaluated in one pass over the weights on the
    integer tensor-core kernels (two sequences per MMA); every batch size, odd ones included,
    must give each sequence the result it gets alone.  Split K and bias included."""
    rng = np.random.default_rng(5)
    for (M, K) in [(96, 768), (40, 300), (256, 6144), (2048, 2048)]:
        t = synth.tensor(rng, kind, M, K)
        bias = rng.standard_normal(M).astype(np.float32)
        for batch in (2, 3, 4, 5, 8, 9, 17):
            x = np.concatenate([synth.activations(rng, K) * (10.0 ** (i % 3 - 1)) for i in range(batch)])
            y = run_linear(ctx, t, x, bias=bias, batch=batch, flags=_lib.AUTO_ROTATE)
            want = oracle.lut_linear(kind, qbits, t.blocks, M, K, bias, x, batch)
            for b in range(batch):
                assert rel_l2(y[b], want[b]) < TOL, (KIND_NAMES[kind], M, K, batch, b)


def test_extreme_activation_ranges(ctx, oracle):
    """The integer tensor-core kernels quantise x per 256-block with a shared exponent: blocks
    of very different magnitude, tiny values, and an all-zero block must still match."""
    rng = np.random.default_rng(31)
    for kind in (INT4, TERNARY, INT2, BINARY, INT3, INT5, INT6, INT8):
        t = synth.tensor(rng, kind, 96, 1024)
        x = synth.activations(rng, 1024)
        x[:256] *= 1e-20
        x[256:512] *= 1e12
        x[512:768] = 0.0
        x[768] = 1e4
        y = run_linear(ctx, t, x)[0]
        want = oracle.gemv_f64(kind, t.blocks, x, 96, 1024)
        assert rel_l2(y, want) < TOL, KIND_NAMES[kind]


@pytest.mark.parametrize("kind,M,K", [(TERNARY, 8192, 8192), (INT2, 8960, 1536), (INT2, 1536, 8960), (INT4, 2048, 8192),
                                      (INT8, 4096, 2048)])
def test_error_against_fp64_truth_is_not_above_the_reference_kernel(ctx, oracle, reference, kind, M, K):
    """Both the CUDA path and the reference kernel are fp32 approximations of the same exact sum.
    Against the fp64 evaluation of that sum the CUDA result must not be further off than the
    reference's own scalar kernel (twice its error, or 3e-7, whichever is larger)."""
    rng = np.random.default_rng(kind * 31 + M)
    t = synth.tensor(rng, kind, M, K)
    x = synth.activations(rng, K)
    xr = reference.apply_hadamard_rotation(x) if t.needs_rotation() else x  # what lut_linear feeds its kernel
    truth = oracle.gemv_f64(kind, t.blocks, xr, M, K)
    got = api.lut_linear(t, None, x, None, 1, ctx=ctx)
    ref = reference.lut_linear(kind, t.quant_bits, t.blocks, M, K, None, x)[0]
    e_gpu, e_ref = rel_l2(got, truth), rel_l2(ref, truth)
    print(f"kind {kind} {M}x{K}: rel L2 vs fp64 truth: CUDA {e_gpu:.3e}, reference kernel {e_ref:.3e}")
    assert e_gpu <= max(2.0 * e_ref, 3e-7), (e_gpu, e_ref)
