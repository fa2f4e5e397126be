"""Worker of tests/test_gpu_tp.py: one process per GPU (launched by torch.distributed.run).
Every rank builds the same random decoder, keeps its tensor-parallel shard, decodes a few
tokens; rank 0 checks the logits against the CPU oracle of the unsharded model."""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

# Shapes that shard over 2, 4 and 8 ranks: whole heads per rank and o/down shards of whole 256-column blocks.
SMALL = dict(hidden=512, inter=2048, n_heads=16, n_kv_heads=8, head_dim=128, n_layers=3)
# One layer with the hidden size and head layout of the 70B-shaped stack (the exchanged vector is 32 KiB).
WIDE = dict(hidden=8192, inter=8192, n_heads=64, n_kv_heads=8, head_dim=128, n_layers=1, vocab=1024)
STEPS2 = ((3, 9), (100, 4), (7, 7), (500, 1))

STEPS1 = ((3,), (100,), (7,), (500,))
# name, kind name, LMB_TP_PEERS, LMB_MODEL_PERSISTENT, shape overrides, batch, token ids per step, sequences rank 0 checks
CASES = (
    ("int4", "INT4", "1", "0", SMALL, 2, STEPS2, (0, 1)),
    ("ternary", "TERNARY", "1", "0", SMALL, 2, STEPS2, (0, 1)),
    ("int4_nccl", "INT4", "0", "0", SMALL, 2, STEPS2, (0, 1)),
    # batch 1, one launch per projection, partial vectors through peer memory
    ("int4_batch_1", "INT4", "1", "0", SMALL, 1, STEPS1, (0,)),
    # batch 1: embedding, all layers and the exchanges between the ranks inside one persistent kernel
    ("int4_batch_1_persistent", "INT4", "1", "1", SMALL, 1, STEPS1, (0,)),
    ("int2_batch_1_persistent", "INT2", "1", "1", SMALL, 1, STEPS1, (0,)),
    ("ternary_hidden_8192", "TERNARY", "1", "0", WIDE, 1, ((3,), (900,), (77,)), (0,)),
    ("ternary_hidden_8192_persistent", "TERNARY", "1", "1", WIDE, 1, ((3,), (900,), (77,)), (0,)),
    ("ternary_batch_16", "TERNARY", "1", "0", SMALL, 16, None, (0, 7, 15)),
)


def main():
    import torch.distributed as dist
    from lutmac_b200 import blocks, synth, tp
    from lutmac_b200.api import Context
    from lutmac_b200.model import Model
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dist.init_process_group("gloo")  # rendezvous only; the data path is NCCL / peer memory inside the library
    ctx = Context(local)
    tp.init_tp(ctx, dist, peer_floats=16 * 8192)
    out = {}
    for name, kind_name, peers, persistent, over, batch, steps, check in CASES:
        kind = getattr(blocks, kind_name)
        os.environ["LMB_TP_PEERS"] = peers  # both are read when the model is created
        os.environ["LMB_MODEL_PERSISTENT"] = persistent
        spec = synth.model_spec(synth.tiny_model_shape(**over), kind, seed=7, max_seq=32)
        if steps is None:
            rng = np.random.default_rng(5)
            steps = [tuple(int(t) for t in rng.integers(0, spec.cfg["vocab"], size=batch)) for _ in range(3)]
        m = Model(spec, ctx, max_batch=batch, tp_rank=rank, tp_size=world)
        logits = []
        for p, t in enumerate(steps):
            logits.append(m.forward(np.array(t), [p] * batch).copy())
        m.close()
        assert not tp.peer_timed_out(ctx), "a rank gave up waiting for a partial vector"
        if rank == 0:
            from oracle.oracle import Oracle, OracleModel
            orc = Oracle()
            worst = 0.0
            for b in check:
                om = OracleModel(orc, spec, n_threads=8)
                for p, t in enumerate(steps):
                    want = om.forward(t[b], p)
                    got = logits[p][b]
                    worst = max(worst, float(np.linalg.norm(got - want) / np.linalg.norm(want)))
            out[name] = worst
        dist.barrier()
    if rank == 0:
        print("TP_RESULT " + json.dumps(out), flush=True)
    from lutmac_b200._lib import lib
    lib().lmb_tp_destroy(ctx.h)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
