"""Host-side logic of the only multi-GPU mode of the path: independent worlds (blocks of token
rows) are dealt out to ranks, every rank runs the same operator sequence on its own rows with
replicated weights, and nothing is exchanged on the data path.  The only communication is a
barrier around the timed region and a MAX reduction of the per-rank device time.

Kept free of CUDA so that it can be exercised with the gloo backend on CPUs."""
from __future__ import annotations

from typing import List, Sequence, Tuple


def worlds_of_rank(n_worlds: int, world_size: int, rank: int) -> range:
    """Contiguous, balanced partition: rank r owns worlds [start, stop); sizes differ by at most one."""
    if n_worlds < 0 or world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad partition request n_worlds={n_worlds} world_size={world_size} rank={rank}")
    base, extra = divmod(n_worlds, world_size)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def rows_of_rank(n_worlds: int, rows_per_world: int, world_size: int, rank: int) -> Tuple[int, int]:
    """(first row, row count) of a rank in the concatenated [n_worlds * rows_per_world, d] token matrix."""
    w = worlds_of_rank(n_worlds, world_size, rank)
    return w.start * rows_per_world, len(w) * rows_per_world


def world_seeds(n_worlds: int, world_size: int, rank: int) -> List[int]:
    """Each world is seeded by its global id, so results do not depend on how worlds are dealt out."""
    return list(worlds_of_rank(n_worlds, world_size, rank))


def max_over_ranks(value: float, group=None, device="cpu") -> float:
    """MAX all-reduce of a per-rank scalar (the slowest rank's time is the job's time)."""
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def sum_over_ranks(value: float, group=None, device="cpu") -> float:
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return float(t.item())


def job_throughput(units_per_rank: Sequence[float], seconds_per_rank: Sequence[float]) -> float:
    """Whole-job throughput: all units of all ranks divided by the slowest rank's time."""
    if len(units_per_rank) != len(seconds_per_rank) or not units_per_rank:
        raise ValueError("need one unit count and one time per rank")
    return float(sum(units_per_rank)) / max(seconds_per_rank)
