"""GPU: tensor-parallel decode (row shards for q/k/v/gate/up/lm_head, 256-column block shards for
o/down, partial vectors through peer memory or NCCL) against the oracle of the unsharded model
(needs as many devices as ranks), and the failure path of the bounded peer wait (one device)."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _device_count():
    import ctypes as C
    from lutmac_b200 import _lib
    n = C.c_int()
    return n.value if _lib.lib().lmb_device_count(C.byref(n)) == 0 else 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_decode_matches_oracle(world):
    if _device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + world), os.path.join(ROOT, "tests", "_tp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("TP_RESULT ")][-1]
    res = json.loads(line[len("TP_RESULT "):])
    print(f"tensor parallel over {world} GPUs, logits rel L2 vs the oracle of the unsharded model: {res}")
    assert set(res) == {"int4", "ternary", "int4_nccl", "int4_batch_1", "int4_batch_1_persistent", "int2_batch_1_persistent",
                        "ternary_hidden_8192", "ternary_hidden_8192_persistent", "ternary_batch_16"}
    for name, err in res.items():
        assert err < 1e-5, (name, err)


def test_bounded_peer_wait_expires_and_reports(ctx):
    """A partial vector that never arrives: the consumer kernel polls a short, fixed number of
    times, sets the time-out flag, finishes with what it has and returns -- the device stays
    usable and the host sees the flag.  The ranks are emulated on one GPU (every "peer" block is
    the local one); nothing is killed, hung or faulted."""
    import ctypes as C
    from lutmac_b200 import _lib
    out = (C.c_int * 4)()
    # all four ranks posted: no time-out, the sum is 1+2+3+4 in every element, the epoch advances
    _lib.check(_lib.lib().lmb_debug_tp_wait(ctx.h, 4, 4, 1000, 64, out))
    assert list(out) == [0, 1, 0, 1]
    # rank 3 never posts: the wait runs out (64 polls of about 40 ns per word), the flag is set, the
    # kernel still leaves its counters consistent (epoch advanced, CTA counter back at zero)
    _lib.check(_lib.lib().lmb_debug_tp_wait(ctx.h, 4, 3, 1000, 64, out))
    assert list(out) == [1, 1, 0, 1]
    # nobody posts at all (two ranks)
    _lib.check(_lib.lib().lmb_debug_tp_wait(ctx.h, 2, 0, 8192, 16, out))
    assert list(out) == [1, 1, 0, 1]
    # the same three cases for the consumer that also prepares the next projections' activations
    # (batch-1 steps with integer tensor-core layouts): one CTA per 256-block of the hidden state
    L = _lib.lib()
    _lib.check(L.lmb_debug_tp_wait_prepare(ctx.h, 4, 4, 1024, 64, out))
    assert list(out) == [0, 1, 0, 1]
    _lib.check(L.lmb_debug_tp_wait_prepare(ctx.h, 4, 3, 1024, 64, out))
    assert list(out) == [1, 1, 0, 1]
    _lib.check(L.lmb_debug_tp_wait_prepare(ctx.h, 8, 0, 8192, 16, out))
    assert list(out) == [1, 1, 0, 1]
    # the context is still usable afterwards
    import numpy as np
    x = ctx.to_device(np.arange(256, dtype=np.float32))
    assert x.download(np.float32)[255] == 255.0
