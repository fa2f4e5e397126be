"""GPU, needs >= 2 devices: tensor-parallel decode (row shards for q/k/v/gate/up/lm_head, 256-column
block shards for o/down, NCCL all-reduce / all-gather) against the oracle of the unsharded model."""
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


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_decode_matches_oracle(world):
    if _device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + world), os.path.join(ROOT, "tests", "_tp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("TP_RESULT ")][-1]
    res = json.loads(line[len("TP_RESULT "):])
    for name, err in res.items():
        assert err < 1e-5, (name, err)
