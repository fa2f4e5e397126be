"""The range-checking build (liblutmac_b200_dbg.so, -DLMB_DEBUG_BOUNDS): kernels check their weight-tile
loads, output and scratch stores and cache slices against the buffers' extents, skip an access that
would leave its buffer and record it; nothing traps.  The library is chosen when lutmac_b200._lib is
imported, so the checks run in a child process."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import ctypes as C, sys
import numpy as np
sys.path.insert(0, %r)
from lutmac_b200 import _lib, synth
from lutmac_b200.api import Context
from lutmac_b200.blocks import INT4, TERNARY, blocks_per_row
from lutmac_b200.model import Model
from oracle.oracle import Oracle, OracleModel
assert _lib.LIB_PATH.endswith("_dbg.so")
L = _lib.lib()
ctx = Context(0)
orc = Oracle()
rel = lambda a, b: float(np.linalg.norm(np.asarray(a, np.float64) - b) / np.linalg.norm(b))

def report():
    out = (C.c_ulonglong * 4)()
    _lib.check(L.lmb_debug_bounds(ctx.h, out))
    return list(out)

def gemv(t, x):
    w = ctx.upload(t); dx = ctx.to_device(x); dy = ctx.malloc(t.M * 4)
    ctx.linear(w, dx, dy, flags=0, x_len=x.size, x_stride=x.size)
    y = dy.download(np.float32); w.free()
    return y

rng = np.random.default_rng(0)
report()
# 1. ordinary work is clean: split-K through scratch, clusters, odd shapes, a decode step with a KV cache
for kind, M, K in ((TERNARY, 1000, 2048), (INT4, 70, 2300), (TERNARY, 8192, 8192), (INT4, 4096, 8192)):
    t = synth.tensor(rng, kind, M, K)
    x = synth.activations(rng, blocks_per_row(K) * 256)
    for plan in ((0, 0, 0), (8, 2, 0), (8, 2, 2)):
        _lib.check(L.lmb_debug_force_plan(*plan))
        assert rel(gemv(t, x), orc.gemv(kind, t.blocks, x, M, K)) < 1e-5
_lib.check(L.lmb_debug_force_plan(0, 0, 0))
spec = synth.model_spec(synth.tiny_model_shape(), INT4, seed=1, max_seq=16)
m, o = Model(spec, ctx), OracleModel(orc, spec)
for pos, tok in enumerate((3, 77, 200)):
    assert rel(m.forward(tok, pos), o.forward(tok, pos)) < 1e-5
m.close()
r = report()
assert r[0] == 0 and r[3] == 0, ("violations in ordinary work", r)
# 2. a launch told that its weight buffer ends 4 KiB early: the last tiles are refused, recorded, not read
t = synth.tensor(rng, TERNARY, 1024, 2048)
x = synth.activations(rng, 2048)
_lib.check(L.lmb_debug_bounds_shrink(4096))
gemv(t, x)
r = report()
assert r[0] == 1 and r[3] > 0, ("expected refused weight-tile loads", r)
# 3. and the record is cleared, the context still works
_lib.check(L.lmb_debug_bounds_shrink(0))
assert rel(gemv(t, x), orc.gemv(TERNARY, t.blocks, x, 1024, 2048)) < 1e-5
assert report()[0] == 0
print("debug-bounds ok")
'''


def test_range_checking_build_is_clean_and_catches_a_short_buffer():
    lib = os.path.join(ROOT, "lutmac_b200", "liblutmac_b200_dbg.so")
    assert os.path.exists(lib), "build it with: python -m lutmac_b200.build --debug-bounds"
    env = dict(os.environ, LMB_DEBUG_BOUNDS="1")
    p = subprocess.run([sys.executable, "-c", CHILD % ROOT], env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and "debug-bounds ok" in p.stdout, p.stdout[-2000:] + p.stderr[-4000:]
