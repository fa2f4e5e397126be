"""CPU: the C-ABI library loads and exports every symbol include/lutmac_b200.h declares, the
host-side re-tiling is a bit-exact bijection, and the host logic (block structs, synthetic
generators, byte accounting, tensor-parallel sharding) behaves.  No compute call needs a GPU."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from lutmac_b200 import _lib, api, synth, tp
from lutmac_b200.blocks import (BINARY, BLOCK_BYTES, BLOCK_DTYPES, INT2, INT3, INT4, INT5, INT6, INT8, KIND_NAMES,
                                TERNARY, PackedTensor, algorithmic_bytes, blocks_per_row)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ALL_KINDS = (TERNARY, BINARY, INT2, INT3, INT4, INT5, INT6, INT8)


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "lutmac_b200.h")).read()
    declared = set(re.findall(r"\b(lmb_[a-z0-9_]+)\s*\(", header))
    declared -= {"lmb_allreduce_fn", "lmb_allgather_fn"}
    assert len(declared) > 40
    L = _lib.lib()
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} declared in the header but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)


def test_drop_in_defines_the_reference_entry_points():
    """shim/lutmac_b200_dropin.cpp, compiled against the reference's headers (shim/Makefile), defines
    the functions include/lutmac/lut_gemm.hpp and transform.hpp declare for the path."""
    import subprocess
    obj = os.path.join(ROOT, "shim", "_build", "dropin.o")
    if not os.path.exists(obj):
        pytest.skip("shim/_build/dropin.o not built (make -C shim REF=<reference checkout>)")
    syms = subprocess.run(["nm", "-C", "--defined-only", obj], capture_output=True, text=True, check=True).stdout
    for name in ("lut_gemv_scalar", "lut_gemv_avx2", "lut_gemv_binary_scalar", "lut_gemv_binary_avx2", "int2_gemv_scalar",
                 "int2_gemv_avx2", "int3_gemv_scalar", "int3_gemv_avx2", "int4_gemv_scalar", "int4_gemv_avx2", "int5_gemv_scalar",
                 "int6_gemv_scalar", "int8_gemv_scalar", "int8_gemv_avx2", "lut_linear", "fwht_256", "apply_hadamard_rotation"):
        assert re.search(r" T lutmac::" + name + r"\(", syms), name


def test_range_checking_library_exports_the_same_abi():
    """liblutmac_b200_dbg.so (python -m lutmac_b200.build --debug-bounds) is the same library compiled with
    -DLMB_DEBUG_BOUNDS: every declared entry point, loadable without a GPU."""
    import ctypes
    from lutmac_b200 import _lib
    path = os.path.join(ROOT, "lutmac_b200", "liblutmac_b200_dbg.so")
    if not os.path.exists(path):
        pytest.skip("liblutmac_b200_dbg.so not built")
    L = ctypes.CDLL(path)
    missing = [name for name in _lib.SIGNATURES if not hasattr(L, name)]
    assert not missing, missing


def test_block_sizes_match_the_reference_structs():
    L = _lib.lib()
    for kind in ALL_KINDS:
        assert L.lmb_block_bytes(kind) == BLOCK_BYTES[kind] == BLOCK_DTYPES[kind].itemsize
    assert L.lmb_block_bytes(7) == 0


def test_status_strings_and_argument_errors():
    L = _lib.lib()
    assert L.lmb_strerror(0) == b"ok"
    assert L.lmb_retile_host(77, None, 1, 1, None) == _lib.ERR_ARG
    assert b"unknown block kind" in L.lmb_last_error()
    with pytest.raises(_lib.LutmacError):
        _lib.check(L.lmb_retile_host(TERNARY, None, 4, 256, None))


@pytest.mark.parametrize("kind", ALL_KINDS)
def test_retile_roundtrip_is_bit_exact(kind):
    rng = np.random.default_rng(kind)
    for (M, K) in ((1, 4), (33, 300), (64, 512), (100, 1024)):
        t = synth.tensor(rng, kind, M, K)
        tiled = api.retile_host(t)
        assert tiled.size == (M + 31) // 32 * blocks_per_row(K) * 32 * BLOCK_BYTES[kind]
        back = api.untile_host(kind, tiled, M, K)
        for f in BLOCK_DTYPES[kind].names:
            assert np.array_equal(back[f], t.blocks[f]), (KIND_NAMES[kind], M, K, f)


def test_ternary_mma_layout_roundtrip_is_bit_exact():
    """Device-only layout 16: ternary as 2-bit codes in integer-MMA operand order."""
    rng = np.random.default_rng(16)
    L = _lib.lib()
    for (M, K) in ((33, 300), (64, 512), (100, 1024)):
        t = synth.ternary_tensor(rng, M, K)
        tiled = np.zeros(L.lmb_tiled_bytes(16, M, K), np.uint8)
        _lib.check(L.lmb_retile_host(16, t.blocks.ctypes.data, M, K, tiled.ctypes.data))
        back = np.zeros(M * blocks_per_row(K), BLOCK_DTYPES[TERNARY])
        _lib.check(L.lmb_untile_host(16, tiled.ctypes.data, M, K, back.ctypes.data))
        for f in BLOCK_DTYPES[TERNARY].names:
            assert np.array_equal(back[f], t.blocks[f]), (M, K, f)


def test_ternary_tiles_hold_the_reference_lut_indices(oracle):
    """The device layout stores P = ~zero & ~sign and N = ~zero & sign: their nibbles are
    exactly extract_indices' (pos, neg)."""
    rng = np.random.default_rng(0)
    t = synth.ternary_tensor(rng, 40, 512)
    tiled = api.retile_host(t)
    bpr = 2
    for r in (0, 17, 39):
        for b in range(bpr):
            tile = tiled[((r // 32) * bpr + b) * 32 * 68:][:32 * 68]
            blk = t.blocks[r * bpr + b]
            for g in range(64):
                byte, c, j, lane = g // 2, (g // 2) // 8, (g // 2) % 8, r % 32
                p, n = tile[(c * 32 + lane) * 16 + j], tile[(c * 32 + lane) * 16 + 8 + j]
                got = ((p >> 4, n >> 4) if g % 2 == 0 else (p & 15, n & 15))
                assert got == oracle.extract_indices(blk["sign_plane"], blk["zero_plane"], g)


def test_algorithmic_bytes_worked_numbers():
    assert algorithmic_bytes(TERNARY, 2048, 2048) == 1130496            # config 1
    assert algorithmic_bytes(INT4, 2048, 2048) == 2162688 + 8192 + 8192
    assert algorithmic_bytes(INT4, 8192, 2048) == 8650752 + 8192 + 32768
    assert algorithmic_bytes(INT8, 128256, 2048) == 128256 * 8 * 260 + 8192 + 4 * 128256


def test_synthetic_generators_are_seeded_and_well_formed():
    a = synth.config1(0)
    b = synth.config1(0)
    assert np.array_equal(a[0].blocks, b[0].blocks) and np.array_equal(a[1], b[1])
    t, x = a
    assert t.kind == TERNARY and (t.M, t.K) == (2048, 2048) and t.needs_rotation()
    assert not (t.blocks["sign_plane"] & t.blocks["zero_plane"]).any()  # canonical: no sign under zero
    frac = np.unpackbits(t.blocks["zero_plane"]).mean()
    assert 0.32 < frac < 0.35
    assert 0.005 < (np.abs(x) > 6).mean() < 0.02  # ~1 % outliers x10
    assert np.all(t.blocks["scale"].reshape(2048, 8) == t.blocks["scale"].reshape(2048, 8)[:, :1])  # per-row scale
    layer = synth.config2_layer(np.random.default_rng(0))
    assert [(v.M, v.K) for v in layer.values()] == [(M, K) for _, M, K in synth.LLAMA32_1B_SHAPES]
    assert not synth.int4_tensor(np.random.default_rng(0), 4, 256).needs_rotation()


def test_padding_columns_carry_zero_weights(oracle):
    rng = np.random.default_rng(3)
    for kind in (TERNARY, INT4, INT8):
        t = synth.tensor(rng, kind, 5, 300)
        for r in range(5):
            for c in range(300, 512):
                assert oracle.block_get(kind, t.blocks, r * 2 + c // 256, c % 256) == 0.0


def test_tp_sharding_reassembles(oracle):
    rng = np.random.default_rng(9)
    t = synth.ternary_tensor(rng, 64, 1024)
    x = oracle.apply_hadamard_rotation(synth.activations(rng, 1024))
    full = oracle.gemv(TERNARY, t.blocks, x, 64, 1024)
    rows = np.concatenate([oracle.gemv(TERNARY, tp.shard_rows(t, r, 4).blocks, x, 16, 1024) for r in range(4)])
    assert np.array_equal(rows, full)
    parts = [oracle.gemv(TERNARY, tp.shard_blocks(t, r, 2).blocks, x[r * 512:(r + 1) * 512], 64, 512) for r in range(2)]
    assert np.allclose(parts[0] + parts[1], full, rtol=1e-5, atol=1e-6)


def _plan(kind, M, K, batch=1, other_rows=0, sms=148):
    out = (C.c_int * 5)()
    assert _lib.lib().lmb_debug_plan(kind, M, K, batch, other_rows, sms, out) == 0
    return dict(zip(("R", "S", "n_rg", "n_ks", "nseq"), out))


def test_planner_cuts_launches_sensibly():
    """Host logic of the CTA planner (no GPU): slices fit the shared-memory budget, a launch of a
    few big jobs is planned for latency as a whole (not one row-tile per CTA), prepared groups
    that oversubscribe the GPU get the coarsest cut, batches share the weight pass."""
    TERNARY_MMA, INT2_MMA = 16, 17
    for kind, cap in ((INT4, 48), (TERNARY_MMA, 48), (INT3, 12)):
        for M, K in ((2048, 2048), (8192, 28672), (128, 70000), (33, 300)):
            p = _plan(kind, M, K)
            assert 1 <= p["S"] <= cap and p["R"] in (1, 2, 4, 8)
            assert (p["S"] * p["n_ks"]) >= (K + 255) // 256 > p["S"] * (p["n_ks"] - 1)
            assert p["n_rg"] == -(-((M + 31) // 32) // p["R"])
    # gate/up pair of a 70B-shaped layer: two jobs of 896 row-tiles must not be cut into 1792 CTAs
    pair = _plan(TERNARY_MMA, 28672, 8192, other_rows=28672)
    assert pair["n_rg"] * pair["n_ks"] <= 2 * 148
    # one job of the bench suite among 111 others: coarsest cut, no K split
    q = _plan(INT4, 2048, 2048, other_rows=23552 * 16 - 2048)
    assert (q["R"], q["n_ks"]) == (8, 1)
    # alone, the same job is spread over the GPU
    alone = _plan(INT4, 2048, 8192)
    assert alone["n_rg"] * alone["n_ks"] >= 148
    # batches: 2, 4, 8 sequences per pass on the tensor-core kinds, 1 on the table-lookup kinds
    assert [_plan(INT2_MMA, 8960, 1536, b)["nseq"] for b in (1, 2, 3, 5, 32)] == [1, 2, 4, 8, 8]
    assert _plan(3, 8960, 1536, 8)["nseq"] == 1
