"""The N > 1 path on CPUs: world_size-2 (and 3) gloo process groups exercise the partition of
worlds over ranks, the seeding that makes results independent of the partition, and the
MAX-over-ranks timing reduction that bench.py uses.  No GPU involved."""
import importlib.util
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _load(name, path):
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def _load_sharding():
    return _load("w8a8_sharding", ROOT / "worldmodel.cu_b200" / "sharding.py")


def _load_oracle():
    return _load("w8a8_ref", ROOT / "oracle" / "w8a8_ref.py")


def test_partition_is_disjoint_balanced_and_complete():
    sh = _load_sharding()
    for n_worlds in (0, 1, 7, 64):
        for ws in (1, 2, 3, 4, 8):
            seen = []
            sizes = []
            for r in range(ws):
                w = sh.worlds_of_rank(n_worlds, ws, r)
                seen += list(w)
                sizes.append(len(w))
                first, count = sh.rows_of_rank(n_worlds, 2048, ws, r)
                assert first == w.start * 2048 and count == len(w) * 2048
            assert seen == list(range(n_worlds))
            assert max(sizes) - min(sizes) <= 1
    assert [len(sh.worlds_of_rank(64, 8, r)) for r in range(8)] == [8] * 8
    with pytest.raises(ValueError):
        sh.worlds_of_rank(4, 2, 2)
    assert sh.job_throughput([10, 10], [1.0, 2.0]) == 10.0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world_size, port, n_worlds, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world_size)
    try:
        sh, ref = _load_sharding(), _load_oracle()
        torch.set_num_threads(1)
        d, nq, hid, rows_per_world = 128, 384, 512, 8
        layer = ref.make_layer(0, d, nq, hid)  # weights replicated: every rank builds the same
        mine = sh.world_seeds(n_worlds, world_size, rank)
        outs = {w: ref.layer_forward(ref.make_tokens(rows_per_world, w, torch.float16, d), layer) for w in mine}
        torch.save(outs, os.path.join(out_dir, f"rank{rank}.pt"))
        # timing reduction: the job's time is the slowest rank's
        slowest = sh.max_over_ranks(10.0 + rank)
        total = sh.sum_over_ranks(float(len(mine)))
        dist.barrier()
        assert slowest == 10.0 + world_size - 1
        assert total == float(n_worlds)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world_size", [2, 3])
def test_gloo_ranks_cover_all_worlds_and_match_single_process(tmp_path, world_size):
    n_worlds = 5
    mp.spawn(_worker, args=(world_size, _free_port(), n_worlds, str(tmp_path)), nprocs=world_size, join=True)
    ref = _load_oracle()
    layer = ref.make_layer(0, 128, 384, 512)
    merged = {}
    for r in range(world_size):
        part = torch.load(tmp_path / f"rank{r}.pt")
        assert not (set(part) & set(merged))  # no world computed twice
        merged.update(part)
    assert sorted(merged) == list(range(n_worlds))
    for w in range(n_worlds):  # identical to what one process computes: no cross-rank interaction
        want = ref.layer_forward(ref.make_tokens(8, w, torch.float16, 128), layer)
        assert torch.equal(merged[w], want)
