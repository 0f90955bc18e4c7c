"""world_size-2 test of the replica host logic on CPU (gloo): batch sharding,
the one-time weight broadcast and output gathering. Each rank runs the CPU
oracle on its shard (no GPU here); the concatenation must equal the
single-process result bit for bit."""
import os
import socket

import numpy as np
import torch.multiprocessing as mp

from altius_b200 import replicas


def test_shard_bounds_cover_the_batch_once():
    for n, w in ((256, 8), (7, 2), (5, 8), (32, 1)):
        b = replicas.shard_bounds(n, w)
        assert b[0][0] == 0 and b[-1][1] == n
        assert all(b[i][1] == b[i + 1][0] for i in range(w - 1))
        assert max(hi - lo for lo, hi in b) - min(hi - lo for lo, hi in b) <= 1


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    from altius_b200 import configs
    from oracle import InterpreterSessionBuilder
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # Every rank builds the same per-rank graph (batch 2). Rank 0 holds the real
    # weights; the other starts from a different seed and must end up with
    # rank 0's bytes after the broadcast.
    model_local, _ = configs.vit_base_16(batch=2, depth=1, seed=0 if rank == 0 else 99)
    blob, _ = replicas.broadcast_weights(model_local, "cpu", src=0)
    replicas.unpack_into(model_local, blob.numpy())
    _, feeds = configs.vit_base_16(batch=4, depth=1, seed=0)
    x = replicas.shard_batch(feeds["input"], rank, world)
    out = InterpreterSessionBuilder(model_local).build().run([x])
    full = replicas.gather_outputs(out, world)
    np.save(os.path.join(out_dir, f"rank{rank}.npy"), full[0])
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_replicas_match_single_process(tmp_path):
    from altius_b200 import configs
    from oracle import InterpreterSessionBuilder
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    model, feeds = configs.vit_base_16(batch=4, depth=1, seed=0)
    want = InterpreterSessionBuilder(model).build().run([feeds["input"]])[0]
    for r in range(2):
        got = np.load(os.path.join(tmp_path, f"rank{r}.npy"))
        assert got.shape == want.shape
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
