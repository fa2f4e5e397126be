"""TEST INFRASTRUCTURE ONLY: ctypes access to the CPU oracle (oracle/lutmac_oracle.c) and,
when it has been built, to the unmodified reference compiled as oracle/_ref/libref_lutmac.so.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "liblutmac_oracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libref_lutmac.so")

TERNARY, BINARY, INT2, INT3, INT4, INT5, INT6, INT8 = 0, 1, 2, 3, 4, 5, 6, 8
BLOCK_BYTES = {TERNARY: 68, BINARY: 36, INT2: 72, INT3: 100, INT4: 132, INT5: 164, INT6: 196, INT8: 260}

_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)
_u8p = C.POINTER(C.c_uint8)
_i8p = C.POINTER(C.c_int8)


def reference_dir() -> str:
    """The reference checkout: $LUTMAC_REFERENCE_DIR, else `reference_path` of the BASELINE.json beside
    this package; "" when neither names a directory that holds the reference's headers."""
    cands = [os.environ.get("LUTMAC_REFERENCE_DIR", "")]
    try:
        import json
        with open(os.path.join(os.path.dirname(_HERE), "BASELINE.json")) as f:
            cands.append(json.load(f).get("reference_path", ""))
    except (OSError, ValueError):
        pass
    for c in cands:
        if c and os.path.exists(os.path.join(c, "include", "lutmac", "types.hpp")):
            return c
    return ""


def build(force: bool = False) -> None:
    """Compile the oracle (and the reference library when its sources are present)."""
    ref_dir = reference_dir()
    ref_present = bool(ref_dir)
    need = force or not os.path.exists(ORACLE_SO) or (ref_present and not os.path.exists(REF_SO))
    if not need:
        src_m = max(os.path.getmtime(os.path.join(_HERE, f)) for f in ("lutmac_oracle.c", "lutmac_oracle.h"))
        need = os.path.getmtime(ORACLE_SO) < src_m
        if ref_present and os.path.exists(REF_SO):
            need = need or os.path.getmtime(REF_SO) < os.path.getmtime(os.path.join(_HERE, "ref_shim.cpp"))
    if need:
        subprocess.run(["make", "-C", _HERE, "REF=" + ref_dir], check=True, capture_output=True)


def _ptr(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def _blocks_ptr(blocks: np.ndarray):
    assert blocks.flags["C_CONTIGUOUS"]
    return C.c_void_p(blocks.ctypes.data)


class OrcTensor(C.Structure):
    _fields_ = [("kind", C.c_int), ("quant_bits", C.c_int), ("blocks", C.c_void_p), ("M", C.c_size_t), ("K", C.c_size_t)]


class OrcLayer(C.Structure):
    _fields_ = [("input_norm", _f32p), ("post_norm", _f32p),
                ("q", OrcTensor), ("k", OrcTensor), ("v", OrcTensor), ("o", OrcTensor),
                ("gate", OrcTensor), ("up", OrcTensor), ("down", OrcTensor),
                ("q_bias", _f32p), ("k_bias", _f32p), ("v_bias", _f32p)]


class OrcModel(C.Structure):
    _fields_ = [("vocab", C.c_size_t), ("hidden", C.c_size_t), ("inter", C.c_size_t), ("n_layers", C.c_size_t),
                ("n_heads", C.c_size_t), ("n_kv_heads", C.c_size_t), ("head_dim", C.c_size_t), ("max_seq", C.c_size_t),
                ("rope_theta", C.c_float), ("rope_factor", C.c_float), ("eps", C.c_float),
                ("embed", OrcTensor), ("lm_head", OrcTensor), ("final_norm", _f32p),
                ("layers", C.POINTER(OrcLayer)), ("kv_cache", _f32p), ("n_threads", C.c_int), ("gemma", C.c_int),
                ("gelu", C.c_int)]


class Oracle:
    """The plain-C restatement."""

    def __init__(self):
        build()
        L = self.lib = C.CDLL(ORACLE_SO)
        L.orc_gemv.argtypes = [C.c_int, C.c_void_p, _f32p, _f32p, C.c_size_t, C.c_size_t]
        L.orc_gemv_f64.argtypes = [C.c_int, C.c_void_p, _f32p, _f64p, C.c_size_t, C.c_size_t]
        L.orc_gemv_lutform.argtypes = [C.c_int, C.c_void_p, _f32p, _f32p, C.c_size_t, C.c_size_t]
        L.orc_block_get.argtypes = [C.c_int, C.c_void_p, C.c_size_t]
        L.orc_block_get.restype = C.c_float
        L.orc_block_bytes.argtypes = [C.c_int]
        L.orc_block_bytes.restype = C.c_size_t
        L.orc_lut_linear.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, _f32p, _f32p, _f32p, C.c_size_t]
        L.orc_quantize.argtypes = [C.c_int, _f32p, C.c_size_t, C.c_size_t, C.c_void_p]
        L.orc_quantize.restype = C.c_size_t
        L.orc_fwht_256.argtypes = [_f32p]
        L.orc_apply_hadamard_rotation.argtypes = [_f32p, C.c_size_t]
        L.orc_precompute_lut.argtypes = [_f32p, _f32p]
        L.orc_precompute_luts.argtypes = [_f32p, C.c_size_t, _f32p]
        L.orc_extract_indices.argtypes = [_u8p, _u8p, C.c_size_t, _u8p, _u8p]
        L.orc_pack_to_bitplanes.argtypes = [_i8p, C.c_size_t, _u8p, _u8p]
        L.orc_unpack_from_bitplanes.argtypes = [_u8p, _u8p, C.c_size_t, _i8p]
        L.orc_rms_norm.argtypes = [_f32p, _f32p, _f32p, C.c_size_t, C.c_float]
        L.orc_apply_rope.argtypes = [_f32p, _f32p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_float, C.c_float]
        L.orc_softmax.argtypes = [_f32p, C.c_size_t]
        L.orc_model_forward.argtypes = [C.POINTER(OrcModel), C.c_int, C.c_size_t, _f32p]
        L.orc_model_forward_f64.argtypes = [C.POINTER(OrcModel), C.c_int, C.c_size_t, _f64p]
        self.prefix = "orc"

    # -- kernel API ---------------------------------------------------------------------
    def gemv(self, kind, blocks, act, M, K):
        act = np.ascontiguousarray(act, np.float32)
        assert act.size >= (K + 255) // 256 * 256, "activations must cover whole 256-blocks"
        out = np.empty(M, np.float32)
        self.lib.orc_gemv(kind, _blocks_ptr(blocks), _ptr(act, _f32p), _ptr(out, _f32p), M, K)
        return out

    def gemv_f64(self, kind, blocks, act, M, K):
        act = np.ascontiguousarray(act, np.float32)
        out = np.empty(M, np.float64)
        self.lib.orc_gemv_f64(kind, _blocks_ptr(blocks), _ptr(act, _f32p), _ptr(out, _f64p), M, K)
        return out

    def gemv_lutform(self, kind, blocks, act, M, K):
        act = np.ascontiguousarray(act, np.float32)
        out = np.empty(M, np.float32)
        self.lib.orc_gemv_lutform(kind, _blocks_ptr(blocks), _ptr(act, _f32p), _ptr(out, _f32p), M, K)
        return out

    def gemv_rows_parallel(self, kind, blocks, act, M, K, threads):
        """The same kernel on row slices of the block array, one slice per thread."""
        act = np.ascontiguousarray(act, np.float32)
        out = np.empty(M, np.float32)
        bpr = (K + 255) // 256
        bb = BLOCK_BYTES[kind]
        base = blocks.ctypes.data

        def run(t):
            r0, r1 = M * t // threads, M * (t + 1) // threads
            if r1 > r0:
                self.lib.orc_gemv(kind, C.c_void_p(base + r0 * bpr * bb), _ptr(act, _f32p),
                                  C.cast(out.ctypes.data + 4 * r0, _f32p), r1 - r0, K)

        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(run, range(threads)))
        return out

    def block_get(self, kind, blocks, block_idx, i):
        bb = BLOCK_BYTES[kind]
        return self.lib.orc_block_get(kind, C.c_void_p(blocks.ctypes.data + block_idx * bb), i)

    def lut_linear(self, kind, quant_bits, blocks, M, K, bias, x, batch=1):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(batch * M, np.float32)
        b = None if bias is None else _ptr(np.ascontiguousarray(bias, np.float32), _f32p)
        self.lib.orc_lut_linear(kind, quant_bits, _blocks_ptr(blocks), M, K, b, _ptr(x, _f32p), _ptr(out, _f32p), batch)
        return out.reshape(batch, M)

    # -- quantizers -------------------------------------------------------------------------
    def quantize(self, kind, w):
        w = np.ascontiguousarray(w, np.float32)
        M, K = w.shape
        n = M * ((K + 255) // 256)
        out = np.zeros(n * BLOCK_BYTES[kind], np.uint8)
        got = self.lib.orc_quantize(kind, _ptr(w, _f32p), M, K, C.c_void_p(out.ctypes.data))
        assert got == n
        return out

    def pack_to_bitplanes(self, t):
        t = np.ascontiguousarray(t, np.int8)
        s = np.zeros((t.size + 7) // 8, np.uint8)
        z = np.zeros_like(s)
        self.lib.orc_pack_to_bitplanes(_ptr(t, _i8p), t.size, _ptr(s, _u8p), _ptr(z, _u8p))
        return s, z

    def unpack_from_bitplanes(self, s, z, n):
        t = np.zeros(n, np.int8)
        self.lib.orc_unpack_from_bitplanes(_ptr(s, _u8p), _ptr(z, _u8p), n, _ptr(t, _i8p))
        return t

    # -- helpers --------------------------------------------------------------------------------
    def fwht_256(self, x):
        x = np.array(x, np.float32, copy=True)
        self.lib.orc_fwht_256(_ptr(x, _f32p))
        return x

    def apply_hadamard_rotation(self, x):
        x = np.array(x, np.float32, copy=True)
        self.lib.orc_apply_hadamard_rotation(_ptr(x, _f32p), x.size)
        return x

    def precompute_lut(self, a4):
        a4 = np.ascontiguousarray(a4, np.float32)
        lut = np.empty(16, np.float32)
        self.lib.orc_precompute_lut(_ptr(a4, _f32p), _ptr(lut, _f32p))
        return lut

    def precompute_luts(self, a):
        a = np.ascontiguousarray(a, np.float32)
        luts = np.empty(a.size // 4 * 16, np.float32)
        self.lib.orc_precompute_luts(_ptr(a, _f32p), a.size, _ptr(luts, _f32p))
        return luts.reshape(-1, 16)

    def extract_indices(self, sign_plane, zero_plane, g):
        s = np.ascontiguousarray(sign_plane, np.uint8)
        z = np.ascontiguousarray(zero_plane, np.uint8)
        p, n = C.c_uint8(), C.c_uint8()
        self.lib.orc_extract_indices(_ptr(s, _u8p), _ptr(z, _u8p), g, C.byref(p), C.byref(n))
        return p.value, n.value

    def rms_norm(self, x, w, eps):
        x = np.ascontiguousarray(x, np.float32)
        w = np.ascontiguousarray(w, np.float32)
        out = np.empty_like(x)
        self.lib.orc_rms_norm(_ptr(x, _f32p), _ptr(w, _f32p), _ptr(out, _f32p), x.size, eps)
        return out

    def apply_rope(self, q, k, position, nh, nkv, hd, theta, factor):
        q = np.array(q, np.float32, copy=True)
        k = np.array(k, np.float32, copy=True)
        self.lib.orc_apply_rope(_ptr(q, _f32p), _ptr(k, _f32p), position, nh, nkv, hd, theta, factor)
        return q, k

    def softmax(self, x):
        x = np.array(x, np.float32, copy=True)
        self.lib.orc_softmax(_ptr(x, _f32p), x.size)
        return x


class OracleModel:
    """One decode step through orc_model_forward.  `spec` is a lutmac_b200.synth.ModelSpec-like
    object: .cfg (dict) and .tensors / .vectors as produced by the synthetic generators."""

    def __init__(self, oracle: Oracle, spec, n_threads: int = 1):
        self.o = oracle
        self.spec = spec
        cfg = spec.cfg
        self._keep = []

        def tens(t):
            self._keep.append(t.blocks)
            return OrcTensor(t.kind, t.quant_bits, t.blocks.ctypes.data, t.M, t.K)

        def vec(v):
            if v is None:
                return None
            v = np.ascontiguousarray(v, np.float32)
            self._keep.append(v)
            return _ptr(v, _f32p)

        n_layers = cfg["n_layers"]
        self.layers = (OrcLayer * n_layers)()
        for i, L in enumerate(spec.layers):
            self.layers[i] = OrcLayer(vec(L["input_norm"]), vec(L["post_norm"]), tens(L["q"]), tens(L["k"]), tens(L["v"]),
                                      tens(L["o"]), tens(L["gate"]), tens(L["up"]), tens(L["down"]),
                                      vec(L.get("q_bias")), vec(L.get("k_bias")), vec(L.get("v_bias")))
        kv_dim = cfg["n_kv_heads"] * cfg["head_dim"]
        self.kv = np.zeros(n_layers * 2 * cfg["max_seq"] * kv_dim, np.float32)
        self.m = OrcModel(cfg["vocab"], cfg["hidden"], cfg["inter"], n_layers, cfg["n_heads"], cfg["n_kv_heads"],
                          cfg["head_dim"], cfg["max_seq"], cfg["rope_theta"], cfg["rope_factor"], cfg["eps"],
                          tens(spec.embed), tens(spec.lm_head), vec(spec.final_norm), self.layers,
                          _ptr(self.kv, _f32p), n_threads, int(bool(cfg.get("gemma"))), int(bool(cfg.get("gelu"))))

    def forward(self, token, position):
        logits = np.empty(self.spec.cfg["vocab"], np.float32)
        self.o.lib.orc_model_forward(C.byref(self.m), int(token), int(position), _ptr(logits, _f32p))
        return logits

    def forward_f64(self, token, position):
        """The step evaluated in fp64 throughout over the current cache (which it does not update)."""
        logits = np.empty(self.spec.cfg["vocab"], np.float64)
        self.o.lib.orc_model_forward_f64(C.byref(self.m), int(token), int(position), _ptr(logits, _f64p))
        return logits


class Reference:
    """The unmodified reference, compiled from its own sources (present only where the
    reference checkout was available at build time)."""

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_SO)

    def __init__(self):
        if not os.path.exists(REF_SO):
            build()
        L = self.lib = C.CDLL(REF_SO)
        L.ref_gemv.argtypes = [C.c_int, C.c_void_p, C.c_size_t, _f32p, _f32p, C.c_size_t, C.c_size_t]
        L.ref_block_get.argtypes = [C.c_int, C.c_void_p, C.c_size_t]
        L.ref_block_get.restype = C.c_float
        L.ref_block_bytes.argtypes = [C.c_int]
        L.ref_block_bytes.restype = C.c_size_t
        L.ref_lut_linear.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, _f32p, _f32p, _f32p, C.c_size_t]
        L.ref_tensor_create.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_size_t]
        L.ref_tensor_create.restype = C.c_void_p
        L.ref_tensor_free.argtypes = [C.c_void_p]
        L.ref_lut_linear_t.argtypes = [C.c_void_p, _f32p, _f32p, _f32p, C.c_size_t]
        L.ref_quantize.argtypes = [C.c_int, _f32p, C.c_size_t, C.c_size_t, C.c_void_p, C.POINTER(C.c_int)]
        L.ref_quantize.restype = C.c_size_t
        L.ref_fwht_256.argtypes = [_f32p]
        L.ref_apply_hadamard_rotation.argtypes = [_f32p, C.c_size_t]
        L.ref_precompute_lut.argtypes = [_f32p, _f32p]
        L.ref_precompute_luts.argtypes = [_f32p, C.c_size_t, _f32p]
        L.ref_extract_indices.argtypes = [_u8p, _u8p, C.c_size_t, _u8p, _u8p]
        L.ref_pack_to_bitplanes.argtypes = [_i8p, C.c_size_t, _u8p, _u8p]
        L.ref_unpack_from_bitplanes.argtypes = [_u8p, _u8p, C.c_size_t, _i8p]
        L.ref_rms_norm.argtypes = [_f32p, _f32p, _f32p, C.c_size_t, C.c_float]
        L.ref_apply_rope.argtypes = [_f32p, _f32p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_float, C.c_float]
        L.ref_softmax.argtypes = [_f32p, C.c_size_t]
        L.ref_model_create.argtypes = [C.c_size_t] * 8 + [C.c_float] * 3
        L.ref_model_create.restype = C.c_void_p
        L.ref_model_free.argtypes = [C.c_void_p]
        L.ref_model_set_variant.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.ref_model_set_tensor.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_size_t]
        L.ref_model_set_vector.argtypes = [C.c_void_p, C.c_int, C.c_int, _f32p, C.c_size_t]
        L.ref_model_forward.argtypes = [C.c_void_p, C.c_int, C.c_size_t]
        L.ref_model_logits.argtypes = [C.c_void_p]
        L.ref_model_logits.restype = _f32p
        L.ref_model_kv.argtypes = [C.c_void_p, C.POINTER(C.c_size_t)]
        L.ref_model_kv.restype = _f32p
        L.ref_model_reset.argtypes = [C.c_void_p]
        L.ref_load_model.argtypes = [C.c_char_p]
        L.ref_load_model.restype = C.c_void_p

    def save_lutmac(self, path, spec):
        """Write a model spec through the reference's own save_lutmac (src/format.cpp:146-290)."""
        c = spec.cfg
        ents = spec_file_tensors(spec)
        arr = (RefFileTensor * len(ents))()
        keep = []
        for i, (name, kind, qb, data, M, K) in enumerate(ents):
            nb = name.encode()
            keep.append((nb, data))
            arr[i] = RefFileTensor(nb, kind, qb, data.ctypes.data, M, K)
        self.lib.ref_save_lutmac.argtypes = [C.c_char_p] + [C.c_size_t] * 7 + [C.c_float] * 3 + [C.POINTER(RefFileTensor), C.c_size_t, C.c_int, C.c_int]
        rc = self.lib.ref_save_lutmac(path.encode(), c["vocab"], c["hidden"], c["inter"], c["n_layers"], c["n_heads"],
                                      c["n_kv_heads"], c["head_dim"], c["rope_theta"], c["rope_factor"], c["eps"], arr, len(ents),
                                      int(bool(c.get("gemma"))), int(bool(c.get("gelu"))))
        assert rc == 0, "save_lutmac failed"

    def load_model_logits(self, path, tokens, vocab):
        """load_model + forward per token through the reference; returns [len(tokens), vocab]."""
        h = self.lib.ref_load_model(path.encode())
        assert h, "reference load_model returned null"
        out = []
        for p, t in enumerate(tokens):
            self.lib.ref_model_forward(h, int(t), p)
            out.append(np.ctypeslib.as_array(self.lib.ref_model_logits(h), shape=(vocab,)).copy())
        self.lib.ref_model_free(h)
        return np.stack(out)

    def gemv(self, kind, blocks, act, M, K):
        act = np.ascontiguousarray(act, np.float32)
        assert act.size >= (K + 255) // 256 * 256
        out = np.empty(M, np.float32)
        bpr = (K + 255) // 256
        if kind == BINARY:
            # lut_gemv_binary_scalar runs on the reference's ThreadPool, whose parallel_for
            # (include/lutmac/thread_pool.hpp:20-49) waits for min(n, workers) completions but
            # enqueues only ceil(n / ceil(n / workers)) tasks: for many (n, workers) pairs (e.g.
            # n = 33 on 8 cores, n = 2048 on 224) it spins forever.  One row per call is always
            # safe (one task, one completion) and does not change any row's arithmetic.
            bb = BLOCK_BYTES[kind]
            for r in range(M):
                self.lib.ref_gemv(kind, C.c_void_p(blocks.ctypes.data + r * bpr * bb), bpr, _ptr(act, _f32p),
                                  C.cast(out.ctypes.data + 4 * r, _f32p), 1, K)
            return out
        self.lib.ref_gemv(kind, _blocks_ptr(blocks), M * bpr, _ptr(act, _f32p), _ptr(out, _f32p), M, K)
        return out

    def gemv_rows_parallel(self, kind, blocks, act, M, K, threads):
        act = np.ascontiguousarray(act, np.float32)
        out = np.empty(M, np.float32)
        bpr = (K + 255) // 256
        bb = BLOCK_BYTES[kind]
        base = blocks.ctypes.data

        def run(t):
            r0, r1 = M * t // threads, M * (t + 1) // threads
            if r1 > r0:
                self.lib.ref_gemv(kind, C.c_void_p(base + r0 * bpr * bb), (r1 - r0) * bpr, _ptr(act, _f32p),
                                  C.cast(out.ctypes.data + 4 * r0, _f32p), r1 - r0, K)

        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(run, range(threads)))
        return out

    def block_get(self, kind, blocks, block_idx, i):
        bb = BLOCK_BYTES[kind]
        return self.lib.ref_block_get(kind, C.c_void_p(blocks.ctypes.data + block_idx * bb), i)

    def lut_linear(self, kind, quant_bits, blocks, M, K, bias, x, batch=1):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(batch * M, np.float32)
        b = None if bias is None else _ptr(np.ascontiguousarray(bias, np.float32), _f32p)
        self.lib.ref_lut_linear(kind, quant_bits, _blocks_ptr(blocks), M, K, b, _ptr(x, _f32p), _ptr(out, _f32p), batch)
        return out.reshape(batch, M)

    def quantize(self, kind, w):
        w = np.ascontiguousarray(w, np.float32)
        M, K = w.shape
        qb = C.c_int()
        n = self.lib.ref_quantize(kind, _ptr(w, _f32p), M, K, None, C.byref(qb))
        out = np.zeros(n * BLOCK_BYTES[kind], np.uint8)
        self.lib.ref_quantize(kind, _ptr(w, _f32p), M, K, C.c_void_p(out.ctypes.data), C.byref(qb))
        return out, qb.value

    def pack_to_bitplanes(self, t):
        t = np.ascontiguousarray(t, np.int8)
        s = np.zeros((t.size + 7) // 8, np.uint8)
        z = np.zeros_like(s)
        self.lib.ref_pack_to_bitplanes(_ptr(t, _i8p), t.size, _ptr(s, _u8p), _ptr(z, _u8p))
        return s, z

    def unpack_from_bitplanes(self, s, z, n):
        t = np.zeros(n, np.int8)
        self.lib.ref_unpack_from_bitplanes(_ptr(s, _u8p), _ptr(z, _u8p), n, _ptr(t, _i8p))
        return t

    def fwht_256(self, x):
        x = np.array(x, np.float32, copy=True)
        self.lib.ref_fwht_256(_ptr(x, _f32p))
        return x

    def apply_hadamard_rotation(self, x):
        x = np.array(x, np.float32, copy=True)
        self.lib.ref_apply_hadamard_rotation(_ptr(x, _f32p), x.size)
        return x

    def precompute_lut(self, a4):
        a4 = np.ascontiguousarray(a4, np.float32)
        lut = np.empty(16, np.float32)
        self.lib.ref_precompute_lut(_ptr(a4, _f32p), _ptr(lut, _f32p))
        return lut

    def precompute_luts(self, a):
        a = np.ascontiguousarray(a, np.float32)
        luts = np.empty(a.size // 4 * 16, np.float32)
        self.lib.ref_precompute_luts(_ptr(a, _f32p), a.size, _ptr(luts, _f32p))
        return luts.reshape(-1, 16)

    def extract_indices(self, sign_plane, zero_plane, g):
        s = np.ascontiguousarray(sign_plane, np.uint8)
        z = np.ascontiguousarray(zero_plane, np.uint8)
        p, n = C.c_uint8(), C.c_uint8()
        self.lib.ref_extract_indices(_ptr(s, _u8p), _ptr(z, _u8p), g, C.byref(p), C.byref(n))
        return p.value, n.value

    def rms_norm(self, x, w, eps):
        x = np.ascontiguousarray(x, np.float32)
        w = np.ascontiguousarray(w, np.float32)
        out = np.empty_like(x)
        self.lib.ref_rms_norm(_ptr(x, _f32p), _ptr(w, _f32p), _ptr(out, _f32p), x.size, eps)
        return out

    def apply_rope(self, q, k, position, nh, nkv, hd, theta, factor):
        q = np.array(q, np.float32, copy=True)
        k = np.array(k, np.float32, copy=True)
        self.lib.ref_apply_rope(_ptr(q, _f32p), _ptr(k, _f32p), position, nh, nkv, hd, theta, factor)
        return q, k

    def softmax(self, x):
        x = np.array(x, np.float32, copy=True)
        self.lib.ref_softmax(_ptr(x, _f32p), x.size)
        return x


class RefFileTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("kind", C.c_int), ("quant_bits", C.c_int), ("data", C.c_void_p),
                ("M", C.c_size_t), ("K", C.c_size_t)]


def spec_file_tensors(spec):
    """(name, kind or -1, quant_bits, array, M, K) for every tensor of a model spec, with the names
    load_model maps to slots (src/model.cpp:589-664); an lm_head entry only when the head has a
    block array of its own (otherwise load_model ties it to the embedding)."""
    out = [(spec.embed.name or "model.embed_tokens.weight", spec.embed.kind, spec.embed.quant_bits, spec.embed.blocks,
            spec.embed.M, spec.embed.K),
           ("model.norm.weight", -1, 32, np.ascontiguousarray(spec.final_norm, np.float32), spec.final_norm.size, 0)]
    for i, L in enumerate(spec.layers):
        pre = f"model.layers.{i}."
        for key, nm in (("input_norm", "input_layernorm.weight"), ("post_norm", "post_attention_layernorm.weight"),
                        ("q_bias", "self_attn.q_proj.bias"), ("k_bias", "self_attn.k_proj.bias"),
                        ("v_bias", "self_attn.v_proj.bias")):
            if L.get(key) is not None:
                v = np.ascontiguousarray(L[key], np.float32)
                out.append((pre + nm, -1, 32, v, v.size, 0))
        for key, nm in (("q", "self_attn.q_proj.weight"), ("k", "self_attn.k_proj.weight"), ("v", "self_attn.v_proj.weight"),
                        ("o", "self_attn.o_proj.weight"), ("gate", "mlp.gate_proj.weight"), ("up", "mlp.up_proj.weight"),
                        ("down", "mlp.down_proj.weight")):
            t = L[key]
            out.append((pre + nm, t.kind, t.quant_bits, t.blocks, t.M, t.K))
    if spec.lm_head.blocks is not spec.embed.blocks:
        t = spec.lm_head
        out.append(("lm_head.weight", t.kind, t.quant_bits, t.blocks, t.M, t.K))
    return out


class ReferenceModel:
    """lutmac::Model assembled in memory from a synthetic model spec."""

    SLOT = {"embed": 0, "lm_head": 1, "q": 2, "k": 3, "v": 4, "o": 5, "gate": 6, "up": 7, "down": 8}
    VEC = {"input_norm": 0, "post_norm": 1, "q_bias": 2, "k_bias": 3, "v_bias": 4}

    def __init__(self, ref: Reference, spec):
        self.r = ref
        self.spec = spec
        c = spec.cfg
        L = ref.lib
        self.h = L.ref_model_create(c["vocab"], c["hidden"], c["inter"], c["n_layers"], c["n_heads"], c["n_kv_heads"],
                                    c["head_dim"], c["max_seq"], c["rope_theta"], c["rope_factor"], c["eps"])
        L.ref_model_set_variant(self.h, int(bool(c.get("gemma"))), int(bool(c.get("gelu"))))

        def st(layer, slot, t):
            L.ref_model_set_tensor(self.h, layer, slot, t.kind, t.quant_bits, _blocks_ptr(t.blocks), t.M, t.K)

        st(0, 0, spec.embed)
        st(0, 1, spec.lm_head)
        fn = np.ascontiguousarray(spec.final_norm, np.float32)
        L.ref_model_set_vector(self.h, 0, 5, _ptr(fn, _f32p), fn.size)
        for i, lay in enumerate(spec.layers):
            for name, slot in self.SLOT.items():
                if slot >= 2:
                    st(i, slot, lay[name])
            for name, which in self.VEC.items():
                v = lay.get(name)
                if v is not None:
                    v = np.ascontiguousarray(v, np.float32)
                    L.ref_model_set_vector(self.h, i, which, _ptr(v, _f32p), v.size)

    def forward(self, token, position):
        self.r.lib.ref_model_forward(self.h, int(token), int(position))
        p = self.r.lib.ref_model_logits(self.h)
        return np.ctypeslib.as_array(p, shape=(self.spec.cfg["vocab"],)).copy()

    def kv(self):
        n = C.c_size_t()
        p = self.r.lib.ref_model_kv(self.h, C.byref(n))
        return np.ctypeslib.as_array(p, shape=(n.value,))

    def close(self):
        if self.h:
            self.r.lib.ref_model_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
