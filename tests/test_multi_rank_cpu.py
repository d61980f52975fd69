"""World-size-2 test of the multi-rank host logic on CPU (gloo): the path shards by independent samples
with no data-path collective, so what has to hold between ranks is (1) the contiguous block partition
covers every sample exactly once and concatenating the ranks' results restores the input order of
predict_multi, and (2) the benchmark's aggregation (max of the ranks' times, sum of their samples).
The per-rank "engine" here is the CPU oracle; the GPU engine itself is covered by the gpu tests."""
import json
import os
import socket
import sys

import numpy as np
import torch.distributed as dist
import torch.multiprocessing as mp
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n_samples, out_dir):
    for p in (os.path.join(ROOT, "frugally-deep_b200"), os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
        sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import fdeep_b200
    from fdeep_b200 import model_writer as mw
    from oracle import OracleModel
    text = json.dumps(mw.build_small_cnn())
    x = mw.inputs_small_cnn(n_samples)
    lo, hi = fdeep_b200.capi.shard_block(n_samples, world, rank)
    m = OracleModel(json_text=text)
    outs = m.predict_multi([[x[i]] for i in range(lo, hi)], threads=2) if hi > lo else []
    local = np.stack([o[0] for o in outs]) if outs else np.zeros((0, 10), np.float32)
    # gather the blocks on rank 0 in rank order
    sizes = [None] * world
    dist.all_gather_object(sizes, (lo, hi))
    gathered = [None] * world
    dist.all_gather_object(gathered, local)
    # benchmark aggregation: the slowest rank defines the step time, samples add up
    t = torch.tensor([0.010 * (rank + 1)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total = torch.tensor([hi - lo], dtype=torch.int64)
    dist.all_reduce(total, op=dist.ReduceOp.SUM)
    if rank == 0:
        np.save(os.path.join(out_dir, "gathered.npy"), np.concatenate(gathered, axis=0))
        with open(os.path.join(out_dir, "meta.json"), "w") as f:
            json.dump({"sizes": sizes, "max_time": float(t.item()), "total": int(total.item())}, f)
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_partition_and_aggregate(tmp_path, built_library):
    sys.path.insert(0, os.path.join(ROOT, "frugally-deep_b200"))
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import fdeep_b200
    from fdeep_b200 import model_writer as mw
    from oracle import OracleModel
    n = 11  # odd on purpose: ragged last block
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), n, str(tmp_path)), nprocs=world, join=True)
    meta = json.load(open(tmp_path / "meta.json"))
    assert meta["sizes"] == [[0, 6], [6, 11]]
    assert meta["total"] == n
    assert abs(meta["max_time"] - 0.020) < 1e-12
    got = np.load(tmp_path / "gathered.npy")
    want = OracleModel(json_text=json.dumps(mw.build_small_cnn())).predict_multi([[x] for x in mw.inputs_small_cnn(n)], threads=2)
    np.testing.assert_array_equal(got, np.stack([w[0] for w in want]))


def test_shard_block_covers_everything(built_library):
    sys.path.insert(0, os.path.join(ROOT, "frugally-deep_b200"))
    import fdeep_b200
    for n in (0, 1, 7, 8, 255, 256, 1000):
        for parts in (1, 2, 3, 4, 8):
            cover = []
            for p in range(parts):
                lo, hi = fdeep_b200.capi.shard_block(n, parts, p)
                assert 0 <= lo <= hi <= n
                cover += list(range(lo, hi))
            assert cover == list(range(n))
