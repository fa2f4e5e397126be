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
UNTIED = "tiny_untied_head"  # lm_head.weight is a tensor of its own, different from embed_tokens


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
    # the header is not trusted: every entry is checked against the file before anything is read
    hsize = int.from_bytes(good[12:16], "little")
    header = good[16:16 + hsize]

    def with_header(new):
        assert len(new) == len(header)  # same length: the data offsets stay valid
        return good[:16] + new + good[16 + hsize:]

    at = header.index(b'"num_blocks": 256')
    more = {
        # a tensor that runs past the end of the file
        "short": good[:len(good) - 5000],
        # more blocks claimed than shape[0] * ceil(shape[1] / 256): the upload would read past the buffer
        "num_blocks": with_header(header[:at] + b'"num_blocks": 257' + header[at + 17:]),
        # shape list without its closing bracket
        "shape": with_header(header.replace(b'"shape": [256, 256]', b'"shape": [256, 256 ', 1)),
    }
    for name, data in more.items():
        p = tmp_path / (name + ".lutmac")
        p.write_bytes(data)
        assert L.lmb_file_open(str(p).encode(), C.byref(f)) == _lib.ERR_FORMAT, name
        assert L.lmb_last_error()


def test_untied_head_is_listed_as_its_own_tensor():
    L = _lib.lib()
    f = _open(UNTIED)
    n = C.c_size_t()
    _lib.check(L.lmb_file_tensor_count(f, C.byref(n)))
    names = []
    for i in range(n.value):
        nm = C.c_char_p()
        _lib.check(L.lmb_file_tensor_info(f, i, C.byref(nm), None, None, None, None, None))
        names.append(nm.value.decode())
    assert "lm_head.weight" in names and "model.embed_tokens.weight" in names
    L.lmb_file_close(f)


@pytest.mark.gpu
def test_untied_head_is_not_replaced_by_the_embedding(ctx, oracle):
    """A file whose lm_head.weight differs from embed_tokens (every tensor is read into one
    buffer, so the two arrive at the same host address): logits against the reference's
    load_model + forward and against the oracle of the same spec."""
    from lutmac_b200.model import Model
    from oracle.oracle import OracleModel
    g = np.load(os.path.join(GOLD, "files.npz"))
    spec = synth.model_spec(synth.tiny_model_shape(**SHAPE), INT4, seed=21, max_seq=2048, untied_head=True)
    assert not np.array_equal(spec.lm_head.blocks["data"], spec.embed.blocks["data"])
    m = Model.load(os.path.join(GOLD, UNTIED + ".lutmac"), ctx)
    m2 = Model(spec, ctx)  # the same model assembled tensor by tensor
    o = OracleModel(oracle, spec)
    for p, t in enumerate(g["tokens"]):
        got = m.forward(int(t), p).copy()
        assert rel_l2(got, g[UNTIED + "_logits"][p]) < 1e-5, p
        assert rel_l2(got, o.forward(int(t), p)) < 1e-5, p
        assert rel_l2(m2.forward(int(t), p), g[UNTIED + "_logits"][p]) < 1e-5, p
    m.close()
    m2.close()


@pytest.mark.gpu
def test_zero_head_count_is_rejected(ctx, tmp_path):
    good = open(os.path.join(GOLD, "tiny_int4.lutmac"), "rb").read()
    bad = good.replace(b'"num_key_value_heads": 1', b'"num_key_value_heads": 0', 1)
    assert bad != good
    p = tmp_path / "nokv.lutmac"
    p.write_bytes(bad)
    h = C.c_void_p()
    assert _lib.lib().lmb_model_load(ctx.h, str(p).encode(), 1, 0, 0, 1, C.byref(h)) == _lib.ERR_ARG


@pytest.mark.gpu
@pytest.mark.parametrize("name,kind,over", CASES)
def test_load_model_logits_match_reference(ctx, name, kind, over):
    from lutmac_b200.model import Model
    g = np.load(os.path.join(GOLD, "files.npz"))
    m = Model.load(os.path.join(GOLD, name + ".lutmac"), ctx)
    for p, t in enumerate(g["tokens"]):
        assert rel_l2(m.forward(int(t), p), g[name + "_logits"][p]) < 1e-5, (name, p)
    m.close()
