"""Host-side mirror of the reference's kernel and layer API over the C ABI.

Same names, argument meaning and error behaviour as include/lutmac/lut_gemm.hpp
(lut_gemv, lut_gemv_binary, int2_gemv ... int8_gemv, lut_linear) and
include/lutmac/transform.hpp (fwht_256, apply_hadamard_rotation), operating on numpy arrays.
Every function runs the CUDA kernels; none computes on the host.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _lib
from ._lib import check, lib
from .blocks import (BINARY, BLOCK_BYTES, BLOCK_DTYPES, INT2, INT3, INT4, INT5, INT6, INT8, TERNARY, PackedTensor,
                     blocks_per_row)


def _vp(a: np.ndarray) -> C.c_void_p:
    return C.c_void_p(a.ctypes.data)


class Context:
    """One device + one stream (lmb_ctx)."""

    def __init__(self, device: int = 0):
        h = C.c_void_p()
        check(lib().lmb_ctx_create(device, C.byref(h)))
        self.h = h
        self.device = device

    def close(self):
        if getattr(self, "h", None):
            lib().lmb_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sync(self):
        check(lib().lmb_ctx_sync(self.h))

    def set_option(self, option: int, value: int):
        check(lib().lmb_ctx_set_option(self.h, option, value))

    def set_stream(self, cuda_stream: Optional[int]):
        check(lib().lmb_ctx_set_stream(self.h, C.c_void_p(cuda_stream or 0)))

    def launch_count(self) -> int:
        n = C.c_uint64()
        check(lib().lmb_ctx_launch_count(self.h, C.byref(n)))
        return n.value

    # device memory ---------------------------------------------------------------------------
    def malloc(self, nbytes: int) -> "DeviceBuffer":
        return DeviceBuffer(self, nbytes)

    def to_device(self, a: np.ndarray) -> "DeviceBuffer":
        a = np.ascontiguousarray(a)
        buf = DeviceBuffer(self, a.nbytes)
        buf.upload(a)
        return buf

    def timer_start(self):
        check(lib().lmb_timer_start(self.h))

    def timer_stop(self) -> float:
        ms = C.c_float()
        check(lib().lmb_timer_stop(self.h, C.byref(ms)))
        return ms.value

    # CUDA graphs -----------------------------------------------------------------------------
    def graph_begin(self):
        check(lib().lmb_graph_begin(self.h))

    def graph_end(self) -> "Graph":
        g = C.c_void_p()
        check(lib().lmb_graph_end(self.h, C.byref(g)))
        return Graph(self, g)

    # weights -----------------------------------------------------------------------------------
    def upload(self, t: PackedTensor, rows=None, blks=None) -> "DeviceWeight":
        return DeviceWeight(self, t, rows, blks)

    # layer API on device buffers --------------------------------------------------------------------
    def linear(self, w: "DeviceWeight", x: "DeviceBuffer", y: "DeviceBuffer", batch: int = 1, bias=None,
               flags: int = _lib.AUTO_ROTATE, x_len: Optional[int] = None, x_stride: Optional[int] = None):
        x_len = w.K if x_len is None else x_len
        x_stride = x_len if x_stride is None else x_stride
        check(lib().lmb_linear(self.h, w.h, bias.ptr if bias is not None else None, x.ptr, x_len, x_stride, y.ptr,
                               batch, flags))


_default_ctx = {}


def default_context(device: int = 0) -> Context:
    if device not in _default_ctx:
        _default_ctx[device] = Context(device)
    return _default_ctx[device]


class Graph:
    """An instantiated CUDA graph of kernel launches captured on a context."""

    def __init__(self, ctx: Context, h):
        self.ctx, self.h = ctx, h

    def launch(self):
        check(lib().lmb_graph_launch(self.ctx.h, self.h))

    def __del__(self):
        try:
            if self.h:
                lib().lmb_graph_destroy(self.h)
                self.h = None
        except Exception:
            pass


class Group:
    """n independent batch-1 lut_linear calls of one block kind, planned once, one launch."""

    def __init__(self, ctx: Context, weights, xs, ys, flags: int = _lib.AUTO_ROTATE):
        n = len(weights)
        self.ctx = ctx
        self._keep = (list(weights), list(xs), list(ys))
        W = (C.c_void_p * n)(*[w.h for w in weights])
        X = (C.c_void_p * n)(*[x.ptr for x in xs])
        Y = (C.c_void_p * n)(*[y.ptr for y in ys])
        h = C.c_void_p()
        check(lib().lmb_group_create(ctx.h, n, W, X, Y, flags, C.byref(h)))
        self.h = h

    def launch(self):
        check(lib().lmb_group_launch(self.ctx.h, self.h))

    def __del__(self):
        try:
            if self.h:
                lib().lmb_group_destroy(self.h)
                self.h = None
        except Exception:
            pass


class HostGroup:
    """The host-buffer form of Group: numpy inputs in, numpy outputs out, one launch."""

    def __init__(self, ctx: Context, weights, flags: int = _lib.AUTO_ROTATE):
        n = len(weights)
        self.ctx, self.weights = ctx, list(weights)
        W = (C.c_void_p * n)(*[w.h for w in weights])
        h = C.c_void_p()
        check(lib().lmb_group_create_host(ctx.h, n, W, flags, C.byref(h)))
        self.h = h
        # inputs and outputs as views of the group's pinned staging buffers: data written to
        # `ins` and read from `outs` is transferred without an intermediate host copy
        self.ins, self.outs = [], []
        for i, w in enumerate(weights):
            pi, po = C.c_void_p(), C.c_void_p()
            check(lib().lmb_group_host_io(h, i, C.byref(pi), C.byref(po)))
            self.ins.append(np.ctypeslib.as_array((C.c_float * w.K).from_address(pi.value)))
            self.outs.append(np.ctypeslib.as_array((C.c_float * w.M).from_address(po.value)))
        self._Y = (C.c_void_p * n)(*[y.ctypes.data for y in self.outs])
        self._Xown = (C.c_void_p * n)(*[x.ctypes.data for x in self.ins])
        self._key, self._xs, self._X = None, None, None

    def run(self, inputs=None):
        """One step: host to device, one launch, device to host.  inputs=None takes the step's
        inputs from `self.ins` (pinned memory); the results are in `self.outs`."""
        if inputs is None:
            check(lib().lmb_group_run_host(self.ctx.h, self.h, self._Xown, self._Y))
            return self.outs
        # the pointer table is rebuilt only when the caller passes other array objects than last
        # time (building it costs more than the launch it feeds)
        key = tuple(map(id, inputs))
        if key != self._key:
            self._xs = [np.ascontiguousarray(x, np.float32) for x in inputs]
            self._X = (C.c_void_p * len(self._xs))(*[x.ctypes.data for x in self._xs])
            # inputs that had to be converted are copies: their contents would go stale
            self._key = key if all(a is b for a, b in zip(self._xs, inputs)) else None
        check(lib().lmb_group_run_host(self.ctx.h, self.h, self._X, self._Y))
        return self.outs

    def __del__(self):
        try:
            if self.h:
                lib().lmb_group_destroy(self.h)
                self.h = None
        except Exception:
            pass


class DeviceBuffer:
    def __init__(self, ctx: Context, nbytes: int):
        self.ctx = ctx
        self.nbytes = nbytes
        p = C.c_void_p()
        check(lib().lmb_malloc(ctx.h, nbytes, C.byref(p)))
        self.ptr = p

    def upload(self, a: np.ndarray, offset: int = 0):
        a = np.ascontiguousarray(a)
        assert offset + a.nbytes <= self.nbytes
        check(lib().lmb_memcpy_h2d(self.ctx.h, C.c_void_p(self.ptr.value + offset), _vp(a), a.nbytes))

    def download(self, dtype=np.float32, count: Optional[int] = None, offset: int = 0) -> np.ndarray:
        dt = np.dtype(dtype)
        n = (self.nbytes - offset) // dt.itemsize if count is None else count
        out = np.empty(n, dt)
        check(lib().lmb_memcpy_d2h(self.ctx.h, _vp(out), C.c_void_p(self.ptr.value + offset), out.nbytes))
        return out

    def zero(self):
        check(lib().lmb_memset(self.ctx.h, self.ptr, 0, self.nbytes))

    def free(self):
        if self.ptr and self.ctx.h:
            lib().lmb_free(self.ctx.h, self.ptr)
        self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class DeviceWeight:
    """A weight matrix resident on the device in the tiled layout (lmb_weight)."""

    def __init__(self, ctx: Context, t: PackedTensor, rows=None, blks=None):
        self.ctx = ctx
        h = C.c_void_p()
        if rows is None and blks is None:
            check(lib().lmb_weight_upload(ctx.h, t.kind, _vp(t.blocks), t.M, t.K, C.byref(h)))
        else:
            r0, r1 = rows if rows is not None else (0, t.M)
            b0, b1 = blks if blks is not None else (0, blocks_per_row(t.K))
            check(lib().lmb_weight_upload_shard(ctx.h, t.kind, _vp(t.blocks), t.M, t.K, r0, r1, b0, b1, C.byref(h)))
        self.h = h
        kind, M, K, nb = C.c_int(), C.c_size_t(), C.c_size_t(), C.c_size_t()
        check(lib().lmb_weight_info(h, C.byref(kind), C.byref(M), C.byref(K), C.byref(nb)))
        self.kind, self.M, self.K, self.device_bytes = kind.value, M.value, K.value, nb.value
        self.quant_bits = t.quant_bits

    def download(self) -> np.ndarray:
        out = np.zeros(self.M * blocks_per_row(self.K), BLOCK_DTYPES[self.kind])
        check(lib().lmb_weight_download(self.ctx.h, self.h, _vp(out)))
        return out

    def ternary_indices(self) -> np.ndarray:
        """[M, bpr, 64, 2] (pos, neg) LUT indices as the kernel consumes them."""
        out = np.zeros(self.M * blocks_per_row(self.K) * 128, np.uint8)
        check(lib().lmb_debug_ternary_indices(self.ctx.h, self.h, _vp(out)))
        return out.reshape(self.M, blocks_per_row(self.K), 64, 2)

    def free(self):
        if getattr(self, "h", None):
            lib().lmb_weight_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


# ---- the reference's kernel API (host pointers) ------------------------------------------------------

def _gemv(kind, blocks, num_blocks, activations, output, M, K):
    """X_gemv(blocks, num_blocks, activations, output, M, K) of lut_gemm.hpp:172-408: activations
    must hold ceil(K/256)*256 floats, num_blocks is ignored, output receives M floats."""
    blocks = np.ascontiguousarray(blocks)
    act = np.ascontiguousarray(activations, np.float32)
    if act.size < blocks_per_row(K) * 256:
        raise ValueError("activations must be readable for ceil(K/256)*256 floats (the reference kernels read whole blocks)")
    if blocks.nbytes < M * blocks_per_row(K) * BLOCK_BYTES[kind]:
        raise ValueError("block array is smaller than M*ceil(K/256) blocks")
    out = output if output is not None else np.empty(M, np.float32)
    assert out.dtype == np.float32 and out.flags["C_CONTIGUOUS"] and out.size >= M
    check(lib().lmb_gemv_host(kind, _vp(blocks), num_blocks, _vp(act), _vp(out), M, K))
    return out


def lut_gemv(blocks, num_blocks, activations, output, M, K):
    """Ternary LUT GEMV (lut_gemm.hpp:189-204)."""
    return _gemv(TERNARY, blocks, num_blocks, activations, output, M, K)


def lut_gemv_binary(blocks, num_blocks, activations, output, M, K):
    """lut_gemm.hpp:172-184"""
    return _gemv(BINARY, blocks, num_blocks, activations, output, M, K)


def int2_gemv(blocks, num_blocks, activations, output, M, K):
    """lut_gemm.hpp:280-292"""
    return _gemv(INT2, blocks, num_blocks, activations, output, M, K)


def int3_gemv(blocks, num_blocks, activations, output, M, K):
    """lut_gemm.hpp:322-334"""
    return _gemv(INT3, blocks, num_blocks, activations, output, M, K)


def int4_gemv(blocks, num_blocks, activations, output, M, K):
    """lut_gemm.hpp:238-250"""
    return _gemv(INT4, blocks, num_blocks, activations, output, M, K)


def int5_gemv(blocks, num_blocks, activations, output, M, K):
    """lut_gemm.hpp:346-355"""
    return _gemv(INT5, blocks, num_blocks, activations, output, M, K)


def int6_gemv(blocks, num_blocks, activations, output, M, K):
    """lut_gemm.hpp:357-366"""
    return _gemv(INT6, blocks, num_blocks, activations, output, M, K)


def int8_gemv(blocks, num_blocks, activations, output, M, K):
    """lut_gemm.hpp:396-408"""
    return _gemv(INT8, blocks, num_blocks, activations, output, M, K)


GEMV_BY_KIND = {TERNARY: lut_gemv, BINARY: lut_gemv_binary, INT2: int2_gemv, INT3: int3_gemv, INT4: int4_gemv,
                INT5: int5_gemv, INT6: int6_gemv, INT8: int8_gemv}


# ---- the reference's layer API ---------------------------------------------------------------------------

def lut_linear(weight: PackedTensor, bias, input, output=None, batch_size: int = 1, ctx: Optional[Context] = None):
    """lut_linear(weight, bias, input, output, batch_size) of lut_gemm.hpp:419 /
    lut_gemm_scalar.cpp:68-180: pads K to 256, rotates the input when the weight is ternary or
    has quant_bits <= 2, runs the GEMV, adds the bias.  The device copy of `weight` is made on
    first use and cached on the tensor.  Returns silently (output untouched) when the weight is
    not 2-D, like the reference."""
    if len(weight.shape) != 2:
        return output
    ctx = ctx or default_context()
    if weight._device is None or weight._device.ctx is not ctx:
        weight._device = DeviceWeight(ctx, weight)
    w = weight._device
    x = np.ascontiguousarray(input, np.float32).reshape(-1)
    assert x.size >= batch_size * weight.K
    out = output if output is not None else np.empty(batch_size * weight.M, np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    flags = _lib.ROTATE if weight.needs_rotation() else 0
    check(lib().lmb_linear_host(ctx.h, w.h, None if b is None else _vp(b), _vp(x), _vp(out), batch_size, flags))
    return out


def lut_linear_multi(weights: Sequence[PackedTensor], inputs: Sequence[np.ndarray], ctx: Optional[Context] = None):
    """Several independent batch-1 lut_linear calls issued together (one staged copy each way)."""
    ctx = ctx or default_context()
    n = len(weights)
    for t in weights:
        if t._device is None or t._device.ctx is not ctx:
            t._device = DeviceWeight(ctx, t)
    rot = {t.needs_rotation() for t in weights}
    assert len(rot) == 1, "lut_linear_multi: mixed rotation requirements"
    xs = [np.ascontiguousarray(x, np.float32) for x in inputs]
    outs = [np.empty(t.M, np.float32) for t in weights]
    W = (C.c_void_p * n)(*[t._device.h for t in weights])
    X = (C.c_void_p * n)(*[x.ctypes.data for x in xs])
    Y = (C.c_void_p * n)(*[y.ctypes.data for y in outs])
    check(lib().lmb_linear_host_multi(ctx.h, n, W, X, Y, _lib.ROTATE if rot.pop() else 0))
    return outs


# ---- the reference's quantizers ---------------------------------------------------------------------------------

def quantize_tensor(kind: int, weights: np.ndarray, rotate_first: bool = False, ctx: Optional[Context] = None,
                    name: str = "") -> PackedTensor:
    """quantize_tensor / quantize_tensor_binary / _int2 / _int3 / _int4 / _int8 of
    include/lutmac/quantize.hpp on the device: a 2-D fp32 array to a PackedTensor of `kind`.
    rotate_first applies the block-wise Hadamard rotation to the flat weight array before
    quantizing, as the reference's quantize tool does for its ternary, binary and 2-bit formats
    (tools/lutmac-quantize.cpp:423-453)."""
    w = np.ascontiguousarray(weights, np.float32)
    assert w.ndim == 2
    M, K = w.shape
    ctx = ctx or default_context()
    blocks = np.zeros(M * blocks_per_row(K), BLOCK_DTYPES[kind])
    check(lib().lmb_quantize_host(ctx.h, kind, _vp(w), M, K, 1 if rotate_first else 0, _vp(blocks)))
    return PackedTensor(kind, blocks, M, K, name=name)


# ---- the reference's transform API -------------------------------------------------------------------------

def apply_hadamard_rotation(data: np.ndarray, n: Optional[int] = None) -> np.ndarray:
    """In place on a float32 array: FWHT/16 of every full 256-block (transform.hpp:19)."""
    assert data.dtype == np.float32 and data.flags["C_CONTIGUOUS"]
    check(lib().lmb_apply_hadamard_rotation_host(_vp(data), data.size if n is None else n))
    return data


def fwht_256(data: np.ndarray) -> np.ndarray:
    """In place on 256 floats (transform.hpp:14)."""
    assert data.size >= 256
    return apply_hadamard_rotation(data, 256)


def retile_host(t: PackedTensor) -> np.ndarray:
    """The device tile layout of a tensor, computed on the host (no GPU needed)."""
    out = np.zeros(lib().lmb_tiled_bytes(t.kind, t.M, t.K), np.uint8)
    check(lib().lmb_retile_host(t.kind, _vp(t.blocks), t.M, t.K, _vp(out)))
    return out


def untile_host(kind: int, tiled: np.ndarray, M: int, K: int) -> np.ndarray:
    out = np.zeros(M * blocks_per_row(K), BLOCK_DTYPES[kind])
    check(lib().lmb_untile_host(kind, _vp(tiled), M, K, _vp(out)))
    return out


def debug_luts(ctx: Context, x: np.ndarray, rotate: bool) -> np.ndarray:
    """[groups, 16] LUT tables as the GEMV prologue builds them."""
    x = np.ascontiguousarray(x, np.float32)
    nb = (x.size + 255) // 256
    dx = ctx.to_device(x)
    dl = ctx.malloc(nb * 1024 * 4)
    check(lib().lmb_debug_luts(ctx.h, dx.ptr, x.size, _lib.ROTATE if rotate else 0, dl.ptr))
    return dl.download(np.float32).reshape(nb * 64, 16)
