"""GPU parity of one decode step (Model::forward) against the reference fixtures and the oracle:
logits within 1e-5 relative L2 (fp32 accumulation), single sequence and batched."""
import os

import numpy as np
import pytest

from lutmac_b200 import synth
from lutmac_b200.blocks import INT2, INT4, INT8, TERNARY
from lutmac_b200.model import Model
from tests.conftest import rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-5
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

CASES = [("int4", INT4, {}), ("ternary", TERNARY, {}), ("int2_bias", INT2, {"qkv_bias": True}),
         ("int8", INT8, {"n_kv_heads": 1})]


@pytest.mark.parametrize("persistent", ["0", "1"])
@pytest.mark.parametrize("name,kind,over", CASES)
def test_forward_matches_reference_fixtures(ctx, name, kind, over, persistent, monkeypatch):
    """Both forms of the batch-1 step: one launch per projection (0) and embedding + all layers as
    one persistent kernel (1)."""
    monkeypatch.setenv("LMB_MODEL_PERSISTENT", persistent)
    g = np.load(os.path.join(GOLD, "model.npz"))
    spec = synth.model_spec(synth.tiny_model_shape(**over), kind, seed=11, max_seq=2048)
    m = Model(spec, ctx)
    for p, t in enumerate(g["tokens"]):
        logits = m.forward(int(t), p)
        assert rel_l2(logits, g[name + "_logits"][p]) < TOL, (name, p)
    m.close()


@pytest.mark.parametrize("plan", [(8, 1, 2), (2, 2, 2), (1, 4, 2), (4, 2, 1), (1, 1, 8), (8, 2, 0)])
@pytest.mark.parametrize("kind,over", [(TERNARY, {}), (INT2, {"qkv_bias": True})])
def test_decode_step_with_clustered_projections(ctx, oracle, kind, over, plan, monkeypatch):
    """Forced work splits for every projection that can take them (R row tiles per CTA, K slices, row
    groups per thread-block cluster): the CTAs of a cluster convert the activations together, RMSNorm
    comes from the per-block sums of squares they publish to each other, and K slices are added
    through distributed shared memory.  (8, 2, 0) is a split through global scratch."""
    from lutmac_b200 import _lib
    from oracle.oracle import OracleModel
    monkeypatch.setenv("LMB_MODEL_PERSISTENT", "0")
    spec = synth.model_spec(synth.tiny_model_shape(hidden=1024, inter=2048, n_heads=16, n_kv_heads=4, **over), kind, seed=21, max_seq=32)
    L = _lib.lib()
    _lib.check(L.lmb_debug_force_plan(*plan))
    try:
        m = Model(spec, ctx)
        o = OracleModel(oracle, spec)
        for p, t in enumerate((3, 77, 200, 5)):
            assert rel_l2(m.forward(t, p), o.forward(t, p)) < TOL, (plan, p)
        m.close()
    finally:
        _lib.check(L.lmb_debug_force_plan(0, 0, 0))


def test_forward_vs_oracle_longer_context_and_kv(ctx, oracle):
    from oracle.oracle import OracleModel
    spec = synth.model_spec(synth.tiny_model_shape(n_layers=3, hidden=512, inter=768, n_heads=8, n_kv_heads=2), INT4,
                            seed=3, max_seq=64)
    m = Model(spec, ctx)
    o = OracleModel(oracle, spec)
    rng = np.random.default_rng(0)
    toks = rng.integers(0, spec.cfg["vocab"], size=40)
    for p, t in enumerate(toks):
        want = o.forward(int(t), p)
        got = m.forward(int(t), p)
        if p % 13 == 0 or p == len(toks) - 1:
            assert rel_l2(got, want) < TOL, p
    assert rel_l2(m.kv_export(), o.kv) < TOL
    # KV hand-off: a fresh model that imports the oracle's cache continues identically
    m2 = Model(spec, ctx)
    m2.kv_import(o.kv)
    want = o.forward(5, len(toks))
    assert rel_l2(m2.forward(5, len(toks)), want) < TOL
    m.close()
    m2.close()


def test_batched_decode_equals_independent_sequences(ctx, oracle):
    from oracle.oracle import OracleModel
    spec = synth.model_spec(synth.tiny_model_shape(qkv_bias=True), INT2, seed=5, max_seq=32)
    B = 3
    m = Model(spec, ctx, max_batch=B)
    oracles = [OracleModel(oracle, spec) for _ in range(B)]
    rng = np.random.default_rng(1)
    for p in range(6):
        toks = rng.integers(0, spec.cfg["vocab"], size=B)
        got = m.forward(toks, [p] * B)
        for b in range(B):
            assert rel_l2(got[b], oracles[b].forward(int(toks[b]), p)) < TOL, (p, b)
    m.close()


@pytest.mark.parametrize("env", [{"LMB_MODEL_PERSISTENT": "0"}, {"LMB_MODEL_PERSISTENT": "0", "LMB_MODEL_FUSED": "0"},
                                 {"LMB_MODEL_PERSISTENT": "0", "LMB_MODEL_GRAPH": "0"},
                                 {"LMB_MODEL_PERSISTENT": "0", "LMB_MODEL_FUSED": "0", "LMB_MODEL_GRAPH": "0"},
                                 {"LMB_MODEL_PERSISTENT": "1", "LMB_ATTN_GROUP": "0"}, {"LMB_MODEL_PERSISTENT": "0", "LMB_ATTN_GROUP": "0"},
                                 {"LMB_MODEL_PERSISTENT": "0", "LMB_MODEL_HANDOFF": "0"}, {"LMB_MODEL_PERSISTENT": "0", "LMB_MODEL_HANDOFF": "1"}])
def test_unfused_and_ungraphed_steps_match_the_fixtures(ctx, env, monkeypatch):
    """With LMB_MODEL_PERSISTENT=0 the step is one launch per projection, which can in turn run
    without norm/activation fusion (the sequence batched tensor-parallel runs use) and without
    graph capture; with 1, batch 1 runs as one persistent kernel.  In models at least 4096 wide
    (and with LMB_MODEL_HANDOFF=1 in any model, as here) o_proj and down_proj prepare the hidden
    state for the next projections, whose CTAs then copy those records; LMB_MODEL_HANDOFF=0 makes
    every consumer CTA convert its own activations instead.  LMB_ATTN_GROUP=0 selects the
    attention form with one CTA per query head instead of one per KV head, in either kind of step.
    The switches are read when the model is created."""
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    g = np.load(os.path.join(GOLD, "model.npz"))
    for name, kind, over in CASES[:2]:
        spec = synth.model_spec(synth.tiny_model_shape(**over), kind, seed=11, max_seq=2048)
        m = Model(spec, ctx)
        for p, t in enumerate(g["tokens"]):
            assert rel_l2(m.forward(int(t), p), g[name + "_logits"][p]) < TOL, (env, name, p)
        m.close()


def test_batch_of_eight_shares_the_weight_pass(ctx, oracle):
    from oracle.oracle import OracleModel
    spec = synth.model_spec(synth.tiny_model_shape(), TERNARY, seed=9, max_seq=32)
    B = 8
    m = Model(spec, ctx, max_batch=B)
    oracles = [OracleModel(oracle, spec) for _ in range(B)]
    rng = np.random.default_rng(2)
    for p in range(4):
        toks = rng.integers(0, spec.cfg["vocab"], size=B)
        got = m.forward(toks, [p] * B)
        for b in range(B):
            assert rel_l2(got[b], oracles[b].forward(int(toks[b]), p)) < TOL, (p, b)
    m.close()


def test_batch_size_changes_on_a_graphed_model(oracle):
    """Batch 1 -> 8 -> 1 on one live model whose steps are captured graphs, on a context of its own
    whose split-K scratch starts small: the larger batch needs more scratch, the buffers are
    reallocated, and the graph captured for batch 1 must not be replayed with its stale pointers."""
    from lutmac_b200.api import Context
    from oracle.oracle import OracleModel
    from lutmac_b200 import _lib
    own = Context(0)
    own.set_option(_lib.OPT_SCRATCH_FLOATS, 1024)  # every growth below frees and reallocates the buffer
    # hidden 2048 / inter 6144: the down projection is split along K at batch 1 (few row-tiles)
    spec = synth.model_spec(synth.tiny_model_shape(hidden=2048, inter=6144, n_heads=8, n_kv_heads=2, head_dim=64,
                                                   n_layers=2, vocab=384), TERNARY, seed=13, max_seq=16)
    B = 8
    m = Model(spec, own, max_batch=B)
    oracles = [OracleModel(oracle, spec) for _ in range(B)]
    rng = np.random.default_rng(4)
    pos = [0] * B
    for step, nb in enumerate((1, 1, B, B, 1, 3, 1, B)):
        toks = rng.integers(0, spec.cfg["vocab"], size=nb)
        got = m.forward(toks, pos[:nb])
        for b in range(nb):
            assert rel_l2(got[b], oracles[b].forward(int(toks[b]), pos[b])) < TOL, (step, nb, b)
            pos[b] += 1
    m.close()
    own.close()


def test_persistent_step_wait_expires_and_reports(ctx, monkeypatch):
    """The CTAs of the persistent decode step wait for each other through arrival counters.  Here
    every wait expects one arrival more than there are CTAs and polls only 200 times: the first
    wait runs out, the kernel records the phase and returns by itself, the step reports
    LMB_ERR_TIMEOUT, and the same model decodes correctly again afterwards."""
    from lutmac_b200 import _lib
    from lutmac_b200._lib import LutmacError
    monkeypatch.setenv("LMB_MODEL_PERSISTENT", "1")
    g = np.load(os.path.join(GOLD, "model.npz"))
    spec = synth.model_spec(synth.tiny_model_shape(), INT4, seed=11, max_seq=2048)
    m = Model(spec, ctx)
    assert rel_l2(m.forward(int(g["tokens"][0]), 0), g["int4_logits"][0]) < TOL
    _lib.check(_lib.lib().lmb_debug_model_waits(m.h, 1, 200))
    with pytest.raises(LutmacError) as e:
        m.forward(int(g["tokens"][1]), 1)
    assert e.value.status == _lib.ERR_TIMEOUT
    _lib.check(_lib.lib().lmb_debug_model_waits(m.h, 0, 0))
    for p, t in enumerate(g["tokens"]):  # the cache slots are rewritten with the same values
        assert rel_l2(m.forward(int(t), p), g["int4_logits"][p]) < TOL, p
    m.close()


def test_model_errors(ctx):
    from lutmac_b200._lib import LutmacError
    spec = synth.model_spec(synth.tiny_model_shape(), INT4, seed=1, max_seq=8)
    m = Model(spec, ctx)
    with pytest.raises(LutmacError):
        m.forward(1, 8)  # beyond the KV cache
    m.close()


def test_launch_timeline_records_every_launch_of_a_step():
    """lmb_debug_launch_timeline: one slot of device time stamps per GEMV / attention launch of a
    step (5 per layer + the head), in order: started <= past the wait <= activations ready <= main
    loop done <= finished, and a launch does not finish before the one it depends on."""
    import ctypes as C
    from lutmac_b200 import _lib
    from lutmac_b200.api import Context
    ctx = Context(0)  # a context of its own: recording is switched on before anything is captured into a graph
    L = _lib.lib()
    n = C.c_size_t()
    _lib.check(L.lmb_debug_launch_timeline(ctx.h, 256, None, C.byref(n)))
    spec = synth.model_spec(synth.tiny_model_shape(n_layers=3), INT4, seed=2, max_seq=16)
    m = Model(spec, ctx)
    for p in range(3):
        m.forward(7 + p, p)
    _lib.check(L.lmb_debug_launch_timeline(ctx.h, 0, None, C.byref(n)))  # clears what the steps so far recorded
    m.forward(11, 3)
    out = (C.c_uint64 * (8 * 256))()
    _lib.check(L.lmb_debug_launch_timeline(ctx.h, 0, out, C.byref(n)))
    assert n.value == 5 * 3 + 1
    t = np.array(list(out)[:8 * n.value], np.uint64).reshape(n.value, 8)
    for i in range(n.value):
        start, first_wait, last_wait, ready, main, done, first_done = (int(t[i][k]) for k in range(7))
        assert 0 < start <= first_wait <= last_wait <= ready <= main <= done, (i, t[i])
        assert first_wait <= first_done <= done + 1000, (i, t[i])  # each stamp reads the timer itself: a launch of one CTA stamps "first done" a few ns after "done"
        if i:
            assert done >= int(t[i - 1][5]), (i, "finished before its predecessor")
    m.close()
