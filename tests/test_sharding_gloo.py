"""CPU, two gloo ranks: sequences sharded over ranks reproduce the single-process id table,
whatever the rank count, and timings are reduced with a maximum."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "tests"))

torch = pytest.importorskip("torch")
import torch.multiprocessing as mp  # noqa: E402


def fake_decode(prompt, draws):
    """Stand-in for the device loop: any deterministic function of the sequence's own inputs."""
    acc = (np.cumsum(prompt.astype(np.int64)) % 997).astype(np.int32)
    return np.concatenate([prompt, acc[: len(draws)] + (draws * 100).astype(np.int32)])


def table(n_total, world, rank):
    from conftest import load_package
    load_package()
    from grad_cpp_b200 import sharding
    lo, hi = sharding.shard_range(n_total, world, rank)
    seqs = [fake_decode(sharding.seq_prompt(11, g, 500, 6), sharding.seq_draws(11, g, 4)) for g in range(lo, hi)]
    return sharding.pad_ids(seqs, 12)


def worker(rank, world, port, n_total, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from conftest import load_package
    load_package()
    from grad_cpp_b200 import sharding
    full = sharding.gather_ids(table(n_total, world, rank), world)
    tmax = sharding.max_over_ranks([1.0 + rank, 5.0 - rank], world)
    if rank == 0:
        np.save(Path(out_dir) / "gathered.npy", full)
        np.save(Path(out_dir) / "tmax.npy", np.array(tmax))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_single_process_table(tmp_path):
    n_total, world = 10, 2
    port = 29500 + os.getpid() % 2000
    mp.spawn(worker, args=(world, port, n_total, str(tmp_path)), nprocs=world, join=True)
    got = np.load(tmp_path / "gathered.npy")
    want = table(n_total, 1, 0)
    assert np.array_equal(got, want)
    assert list(np.load(tmp_path / "tmax.npy")) == [2.0, 5.0]


def test_shard_ranges_partition_the_sequences():
    from conftest import load_package
    load_package()
    from grad_cpp_b200 import sharding
    for n, w in ((10, 3), (256, 8), (5, 8), (0, 2)):
        spans = [sharding.shard_range(n, w, r) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert max(b - a for a, b in spans) - min(b - a for a, b in spans) <= 1
