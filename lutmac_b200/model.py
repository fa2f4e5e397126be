"""Host-side mirror of the reference's Model (include/lutmac/model.hpp:53-142) over the C ABI:
forward(token_id, position), get_logits(), reset_cache().  Weights, KV cache and activations
live on the device; batched decode and tensor parallelism are additions the reference lacks.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _lib
from ._lib import check, lib
from .api import Context, _vp, default_context

SLOTS = {"embed": 0, "lm_head": 1, "q": 2, "k": 3, "v": 4, "o": 5, "gate": 6, "up": 7, "down": 8}
VECS = {"input_norm": 0, "post_norm": 1, "q_bias": 2, "k_bias": 3, "v_bias": 4, "final_norm": 5}


class Model:
    """Built from a model spec (lutmac_b200.synth.ModelSpec or anything with the same fields:
    cfg, embed, lm_head, final_norm, layers)."""

    def __init__(self, spec, ctx: Optional[Context] = None, max_batch: int = 1, tp_rank: int = 0, tp_size: int = 1):
        self.ctx = ctx or default_context()
        self.spec = spec
        c = spec.cfg
        self.vocab = c["vocab"]
        self.max_batch = max_batch
        cfg = _lib.ModelConfig(c["vocab"], c["hidden"], c["inter"], c["n_layers"], c["n_heads"], c["n_kv_heads"],
                               c["head_dim"], c["max_seq"], c["rope_theta"], c["rope_factor"], c["eps"], max_batch,
                               tp_rank, tp_size, int(bool(c.get("gemma"))), 1 if c.get("gelu") else 0)
        h = C.c_void_p()
        check(lib().lmb_model_create(self.ctx.h, C.byref(cfg), C.byref(h)))
        self.h = h
        self._set_weight(0, "embed", spec.embed)
        # a head that is the embedding's own block array is tied (one device copy), as load_model
        # does for files without an lm_head tensor; anything else is uploaded as its own tensor
        tied = (tp_size == 1 and spec.lm_head.kind == spec.embed.kind and spec.lm_head.blocks is spec.embed.blocks)
        if tied:
            check(lib().lmb_model_tie_head(self.h))
        else:
            self._set_weight(0, "lm_head", spec.lm_head)
        self._set_vector(0, "final_norm", spec.final_norm)
        uploaded = {}
        for i, L in enumerate(spec.layers):
            for name in ("q", "k", "v", "o", "gate", "up", "down"):
                self._set_weight(i, name, L[name])
            for name in ("input_norm", "post_norm", "q_bias", "k_bias", "v_bias"):
                if L.get(name) is not None:
                    self._set_vector(i, name, L[name])
        self._logits = np.empty((max_batch, self.vocab), np.float32)

    @classmethod
    def load(cls, path: str, ctx: Optional[Context] = None, max_batch: int = 1, max_seq: int = 0, tp_rank: int = 0,
             tp_size: int = 1) -> "Model":
        """load_model(path) of the reference (include/lutmac/model.hpp:147): parse a .lutmac file
        and build the device-resident model from it (max_seq = 0 keeps the reference's 2048)."""
        self = cls.__new__(cls)
        self.ctx = ctx or default_context()
        f = C.c_void_p()
        check(lib().lmb_file_open(path.encode(), C.byref(f)))
        cfg = _lib.ModelConfig()
        check(lib().lmb_file_config(f, C.byref(cfg)))
        lib().lmb_file_close(f)
        h = C.c_void_p()
        check(lib().lmb_model_load(self.ctx.h, path.encode(), max_batch, max_seq, tp_rank, tp_size, C.byref(h)))
        self.h = h
        self.spec = None
        self.vocab = cfg.vocab_size
        self.max_batch = max_batch
        self._logits = np.empty((max_batch, self.vocab), np.float32)
        return self

    def _set_weight(self, layer, name, t):
        check(lib().lmb_model_set_weight(self.h, layer, SLOTS[name], t.kind, t.quant_bits, _vp(t.blocks), t.M, t.K))

    def _set_vector(self, layer, name, v):
        v = np.ascontiguousarray(v, np.float32)
        check(lib().lmb_model_set_vector(self.h, layer, VECS[name], _vp(v), v.size))

    def forward(self, token_id, position, fetch: bool = True):
        """One decode step.  Scalars decode one sequence (the reference's signature); sequences
        decode a batch.  Returns the logits ([vocab] or [batch, vocab]) unless fetch is False."""
        scalar = np.isscalar(token_id)
        toks = np.atleast_1d(np.asarray(token_id, np.int32))
        pos = np.atleast_1d(np.asarray(position, np.uint64))
        assert toks.size == pos.size <= self.max_batch
        out = self._logits[:toks.size]
        check(lib().lmb_model_forward(self.h, toks.ctypes.data_as(C.POINTER(C.c_int)),
                                      pos.ctypes.data_as(C.POINTER(C.c_size_t)), toks.size,
                                      _vp(out) if fetch else None))
        if not fetch:
            return None
        return out[0] if scalar else out

    def get_logits(self) -> np.ndarray:
        return self._logits

    def reset_cache(self):
        check(lib().lmb_model_reset(self.h))

    def kv_export(self, seq: int = 0) -> np.ndarray:
        c = self.spec.cfg
        out = np.empty(c["n_layers"] * 2 * c["max_seq"] * c["n_kv_heads"] * c["head_dim"], np.float32)
        check(lib().lmb_model_kv_export(self.h, seq, _vp(out)))
        return out

    def kv_import(self, kv: np.ndarray, seq: int = 0):
        kv = np.ascontiguousarray(kv, np.float32)
        check(lib().lmb_model_kv_import(self.h, seq, _vp(kv)))

    def step_bytes(self, position: int) -> int:
        n = C.c_uint64()
        check(lib().lmb_model_step_bytes(self.h, position, C.byref(n)))
        return n.value

    def close(self):
        if getattr(self, "h", None):
            lib().lmb_model_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
