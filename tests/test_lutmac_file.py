"""The .lutmac loader against files written by the reference's own save_lutmac (fixtures under
tests/golden/): header and tensor table (CPU), then load_model + forward logits (GPU) against
the logits the reference's load_model + Model::forward produced from the same files."""
import ctypes as C
import os

import numpy as np
import pytest

from lutmac_b200 import _lib, synth
from lutmac_b200.blocks import BLOCK_BYTES, INT4, INT8, TERNARY
from tests.conftest import rel_l2

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
SHAPE = dict(vocab=256, hidden=256, inter=256, n_layers=1, n_heads=4, n_kv_heads=1, head_dim=64)
CASES = [("tiny_int4", INT4, {}), ("tiny_ternary_bias", TERNARY, {"qkv_bias": True})]


def _open(name):
    f = C.c_void_p()
    _lib.check(_lib.lib().lmb_file_open(os.path.join(GOLD, name + ".lutmac").encode(), C.byref(f)))
    return f


@pytest.mark.parametrize("name,kind,over", CASES)
def test_header_and_tensor_table(name, kind, over):
    L = _lib.lib()
    f = _open(name)
    cfg = _lib.ModelConfig()
    _lib.check(L.lmb_file_config(f, C.byref(cfg)))
    assert (cfg.vocab_size, cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers) == (256, 256, 256, 1)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (4, 1, 64)
    assert cfg.max_seq_len == 2048  # max_position_embeddings is never read back by the reference
    assert cfg.rope_theta == pytest.approx(10000.0) and cfg.rms_norm_eps == pytest.approx(1e-5)
    n = C.c_size_t()
    _lib.check(L.lmb_file_tensor_count(f, C.byref(n)))
    spec = synth.model_spec(synth.tiny_model_shape(**dict(SHAPE, **over)), kind, seed=21, max_seq=2048)
    seen = {}
    for i in range(n.value):
        nm, k, qb = C.c_char_p(), C.c_int(), C.c_int()
        d0, d1, nb = C.c_size_t(), C.c_size_t(), C.c_size_t()
        _lib.check(L.lmb_file_tensor_info(f, i, C.byref(nm), C.byref(k), C.byref(qb), C.byref(d0), C.byref(d1), C.byref(nb)))
        seen[nm.value.decode()] = (k.value, qb.value, d0.value, d1.value, nb.value, i)
    emb = seen["model.embed_tokens.weight"]
    assert emb[:5] == (INT8, 8, 256, 256, 256)
    q = seen["model.layers.0.self_attn.q_proj.weight"]
    # ternary tensors carry "quant_bits": 1.58 in the file, which the reference reads back as 1
    assert q[:5] == (kind, 1 if kind == TERNARY else 4, 256, 256, 256)
    assert seen["model.norm.weight"][0] == -1 and seen["model.norm.weight"][2] == 256
    assert ("model.layers.0.self_attn.q_proj.bias" in seen) == bool(over.get("qkv_bias"))
    # the bytes of a tensor are the reference's block array, untouched
    want = spec.layers[0]["q"].blocks
    buf = np.zeros(want.nbytes, np.uint8)
    _lib.check(L.lmb_file_read_tensor(f, q[5], buf.ctypes.data, buf.nbytes))
    assert np.array_equal(buf, want.view(np.uint8).reshape(-1))
    assert want.nbytes == 256 * BLOCK_BYTES[kind]
    L.lmb_file_close(f)


def test_malformed_files_are_rejected(tmp_path):
    L = _lib.lib()
    good = open(os.path.join(GOLD, "tiny_int4.lutmac"), "rb").read()
    cases = {"magic": b"LUTMAC02" + good[8:], "version": good[:8] + (2).to_bytes(4, "little") + good[12:],
             "truncated": good[:40], "empty": b""}
    for name, data in cases.items():
        p = tmp_path / (name + ".lutmac")
        p.write_bytes(data)
        f = C.c_void_p()
        assert L.lmb_file_open(str(p).encode(), C.byref(f)) == _lib.ERR_FORMAT, name
    f = C.c_void_p()
    assert L.lmb_file_open(str(tmp_path / "missing.lutmac").encode(), C.byref(f)) == _lib.ERR_FORMAT
    # a tensor that runs past the end of the file
    p = tmp_path / "short.lutmac"
    p.write_bytes(good[:len(good) - 5000])
    _lib.check(L.lmb_file_open(str(p).encode(), C.byref(f)))
    n = C.c_size_t()
    L.lmb_file_tensor_count(f, C.byref(n))
    buf = np.zeros(1 << 20, np.uint8)
    assert L.lmb_file_read_tensor(f, n.value - 1, buf.ctypes.data, buf.nbytes) == _lib.ERR_FORMAT
    L.lmb_file_close(f)


@pytest.mark.gpu
@pytest.mark.parametrize("name,kind,over", CASES)
def test_load_model_logits_match_reference(ctx, name, kind, over):
    from lutmac_b200.model import Model
    g = np.load(os.path.join(GOLD, "files.npz"))
    m = Model.load(os.path.join(GOLD, name + ".lutmac"), ctx)
    for p, t in enumerate(g["tokens"]):
        assert rel_l2(m.forward(int(t), p), g[name + "_logits"][p]) < 1e-5, (name, p)
    m.close()
