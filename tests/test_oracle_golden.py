"""CPU: pins the oracle (oracle/lutmac_oracle.c) against
 (a) the known-answer vectors of the reference's own tests, and
 (b) the fixtures under tests/golden/, which hold outputs of the unmodified reference.
"""
import os

import numpy as np
import pytest

from lutmac_b200 import synth
from lutmac_b200.blocks import (BINARY, BLOCK_DTYPES, INT2, INT3, INT4, INT5, INT6, INT8, KIND_NAMES, TERNARY,
                                blocks_per_row)
from tests.conftest import rel_l2

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
ALL_KINDS = (TERNARY, BINARY, INT2, INT3, INT4, INT5, INT6, INT8)
GEMV_SHAPES = ((1, 4), (3, 256), (16, 256), (33, 300), (40, 768), (64, 2048))


def gold(name):
    return np.load(os.path.join(GOLD, name + ".npz"))


def mt19937_uniform(seed, n, lo=-1.0, hi=1.0):
    """std::mt19937(seed) + std::uniform_real_distribution<float>(lo, hi) as libstdc++ draws
    it: one 32-bit output per value, converted to float and divided by 2^32."""
    bg = np.random.MT19937()
    bg._legacy_seeding(seed)
    raw = bg.random_raw(n).astype(np.uint32)
    u = raw.astype(np.float32) / np.float32(4294967296.0)
    u = np.minimum(u, np.nextafter(np.float32(1.0), np.float32(0.0)))
    return (u * np.float32(hi - lo) + np.float32(lo)).astype(np.float32)


# ---- (a) known-answer vectors of the reference's tests -------------------------------------------

def test_lut_precomputation_kat(oracle):
    # tests/test_lut_gemm.cpp:17-55
    lut = oracle.precompute_lut([1.0, 2.0, 3.0, 4.0])
    expected = [0, 4, 3, 7, 2, 6, 5, 9, 1, 5, 4, 8, 3, 7, 6, 10]
    assert np.allclose(lut, expected, atol=1e-3)


def test_index_extraction_kat(oracle):
    # tests/test_lut_gemm.cpp:57-88: weights [+1,-1,0,+1] -> pos 0b1001, neg 0b0100
    sign = np.array([0b01000000, 0, 0, 0], np.uint8)
    zero = np.array([0b00100000, 0, 0, 0], np.uint8)
    assert oracle.extract_indices(sign, zero, 0) == (0b1001, 0b0100)


def test_gemv_correctness_kat(oracle):
    # tests/test_lut_gemm.cpp:135-165: 1x4 all-ones weights, x = [1,2,3,4] -> 10 (scale 1)
    w = np.ones((1, 4), np.float32)
    blocks = oracle.quantize(TERNARY, w)
    x = np.zeros(256, np.float32)
    x[:4] = [1, 2, 3, 4]
    y = oracle.gemv(TERNARY, blocks, x, 1, 4)
    assert y[0] == pytest.approx(10.0, abs=1e-6)


def test_scalar_gemv_smoke(oracle):
    # tests/test_lut_gemm.cpp:90-133
    M, K = 4, 16
    w = np.array([(0.5 if i % 3 == 0 else -0.5 if i % 3 == 1 else 0.0) for i in range(M * K)], np.float32).reshape(M, K)
    blocks = oracle.quantize(TERNARY, w)
    x = np.zeros(256, np.float32)
    x[:K] = 1.0
    assert np.abs(oracle.gemv(TERNARY, blocks, x, M, K)).sum() > 1e-3


def test_int4_ramp_kat(oracle):
    # tests/test_lut_gemm.cpp:218-260: ramp (i%15-7)*0.5, x = 1 -> sum of weights = -6.5
    K = 32
    w = np.array([((i % 15) - 7) * 0.5 for i in range(K)], np.float32).reshape(1, K)
    blocks = oracle.quantize(INT4, w)
    x = np.zeros(256, np.float32)
    x[:K] = 1.0
    y = oracle.gemv(INT4, blocks, x, 1, K)
    assert w.sum() == pytest.approx(-6.5)
    assert y[0] == pytest.approx(-6.5, abs=0.01)


def test_binary_alternating_kat(oracle):
    # tests/test_lut_gemm.cpp:262-307
    K = 256
    w = np.array([1.0 if i % 2 == 0 else -1.0 for i in range(K)], np.float32).reshape(1, K)
    blocks = oracle.quantize(BINARY, w)
    y = oracle.gemv(BINARY, blocks, np.ones(K, np.float32), 1, K)
    assert abs(y[0]) <= 1.0


@pytest.mark.parametrize("kind,seed,M,K,tol", [(INT8, 42, 256, 512, 1e-3), (TERNARY, 42, 16, 256, 1e-4),
                                               (INT2, 43, 16, 256, 1e-3), (INT3, 44, 16, 256, 1e-3)])
def test_vs_dequantised_reference(oracle, kind, seed, M, K, tol):
    # tests/test_lut_gemm.cpp:309-369 and tests/test_tmac_correctness.cpp:13-136: quantize
    # mt19937(seed) U(-1,1) weights, compare the kernel with sum(get(i) * x[i]).
    v = mt19937_uniform(seed, M * K + K)
    w, x = v[:M * K].reshape(M, K), v[M * K:]
    blocks = oracle.quantize(kind, w)
    y = oracle.gemv(kind, blocks, x, M, K)
    bpr = blocks_per_row(K)
    ref = np.zeros(M, np.float32)
    for r in range(M):
        acc = np.float32(0)
        for c in range(K):
            acc += np.float32(oracle.block_get(kind, blocks, r * bpr + c // 256, c % 256)) * x[c]
        ref[r] = acc
    assert np.max(np.abs(y - ref)) < tol


def test_bitplane_roundtrip(oracle):
    # tests/test_quantization.cpp:43-86
    t = np.array([1, -1, 0, 1, 0, 0, -1, 1, 1, 1, -1, -1, 0, 1, 0, -1], np.int8)
    s, z = oracle.pack_to_bitplanes(t)
    assert np.array_equal(oracle.unpack_from_bitplanes(s, z, 16), t)


def test_ternary_threshold_rule(oracle):
    # tests/test_quantization.cpp:13-41 / quantize.hpp:83-88 through the tensor quantizer
    w = np.array([[0.5, -0.5, 0.05, 0.3, -0.01] + [0.0] * 11], np.float32)
    blocks = oracle.quantize(TERNARY, w).view(BLOCK_DTYPES[TERNARY])
    thr = 0.5 * np.abs(w).mean()
    t = oracle.unpack_from_bitplanes(blocks["sign_plane"][0], blocks["zero_plane"][0], 16)
    expect = [0 if abs(v) < thr else (1 if v > 0 else -1) for v in w[0]]
    assert list(t) == expect


# ---- (b) fixtures produced by the unmodified reference ----------------------------------------------------

@pytest.mark.parametrize("kind", ALL_KINDS)
def test_gemv_matches_reference_fixtures(oracle, kind):
    g = gold("gemv")
    for (M, K) in GEMV_SHAPES:
        key = f"{KIND_NAMES[kind]}_{M}x{K}"
        blocks = g[key + "_blocks"].view(BLOCK_DTYPES[kind])
        y = oracle.gemv(kind, blocks, g[key + "_x"], M, K)
        # the reference is built with -ffast-math: compare to tolerance, not bits
        assert rel_l2(y, g[key + "_y"]) < 2e-6, key
        if kind in (TERNARY, BINARY, INT2, INT3, INT4):
            assert rel_l2(oracle.gemv_lutform(kind, blocks, g[key + "_x"], M, K), g[key + "_y"]) < 1e-5, key


def test_lut_linear_matches_reference_fixtures(oracle):
    g = gold("linear")
    for i in range(int(g["n_cases"][0])):
        kind, qb, M, K, batch, has_bias = (int(v) for v in g[f"lin{i}_meta"])
        blocks = g[f"lin{i}_blocks"].view(BLOCK_DTYPES[kind])
        bias = g[f"lin{i}_bias"] if has_bias else None
        y = oracle.lut_linear(kind, qb, blocks, M, K, bias, g[f"lin{i}_x"], batch)
        assert rel_l2(y, g[f"lin{i}_y"]) < 2e-6, i


def test_transforms_match_reference_fixtures(oracle):
    g = gold("transform")
    assert np.array_equal(oracle.apply_hadamard_rotation(g["fwht_in"]), g["fwht_out"])  # bit-exact
    assert np.array_equal(oracle.fwht_256(g["fwht_in"][:256]), g["fwht256_out"])
    assert np.array_equal(g["fwht_out"][1024:], g["fwht_in"][1024:])  # partial block untouched
    assert np.array_equal(oracle.precompute_lut(g["lut_in"]), g["lut_out"])
    assert np.array_equal(oracle.precompute_luts(g["luts_in"]).reshape(-1), g["luts_out"])


def test_fwht_is_textbook_hadamard(oracle):
    x = np.random.default_rng(0).standard_normal(256).astype(np.float32)
    H = np.array([[1.0]])
    for _ in range(8):
        H = np.block([[H, H], [H, -H]])
    assert rel_l2(oracle.fwht_256(x), H @ x.astype(np.float64) / 16.0) < 1e-6


@pytest.mark.parametrize("kind", (TERNARY, BINARY, INT2, INT3, INT4, INT8))
def test_quantizers_match_reference_fixtures(oracle, kind):
    g = gold("quantize")
    for (M, K) in ((4, 16), (3, 300), (16, 512)):
        key = f"{KIND_NAMES[kind]}_{M}x{K}"
        mine = oracle.quantize(kind, g[key + "_w"]).view(BLOCK_DTYPES[kind])
        want = g[key + "_blocks"].view(BLOCK_DTYPES[kind])
        for f in BLOCK_DTYPES[kind].names:
            if f.startswith("scale"):
                # float artefact of a -ffast-math build (reassociated sums, reciprocal division)
                assert np.allclose(mine[f], want[f], rtol=1e-6, atol=0), (key, f)
            else:
                assert np.array_equal(mine[f], want[f]), (key, f)  # codes and bit-planes bit-exact
    s, z = oracle.pack_to_bitplanes(g["pack_t"])
    assert np.array_equal(s, g["pack_s"]) and np.array_equal(z, g["pack_z"])
    assert np.array_equal(oracle.unpack_from_bitplanes(s, z, 64), g["unpack_t"])


def test_glue_ops_match_reference_fixtures(oracle):
    g = gold("glue")
    assert rel_l2(oracle.rms_norm(g["rms_x"], g["rms_w"], 1e-5), g["rms_y"]) < 1e-6
    q, k = oracle.apply_rope(g["rope_q"], g["rope_k"], 37, 4, 2, 64, 500000.0, 32.0)
    assert rel_l2(q, g["rope_q_out"]) < 1e-6 and rel_l2(k, g["rope_k_out"]) < 1e-6
    assert rel_l2(oracle.softmax(g["softmax_x"]), g["softmax_y"]) < 1e-6


@pytest.mark.parametrize("name,kind,over", [("int4", INT4, {}), ("ternary", TERNARY, {}),
                                            ("int2_bias", INT2, {"qkv_bias": True}), ("int8", INT8, {"n_kv_heads": 1})])
def test_model_forward_matches_reference_fixtures(oracle, name, kind, over):
    from oracle.oracle import OracleModel
    g = gold("model")
    spec = synth.model_spec(synth.tiny_model_shape(**over), kind, seed=11, max_seq=2048)
    m = OracleModel(oracle, spec)
    for p, t in enumerate(g["tokens"]):
        logits = m.forward(int(t), p)
        assert rel_l2(logits, g[name + "_logits"][p]) < 1e-5, (name, p)
