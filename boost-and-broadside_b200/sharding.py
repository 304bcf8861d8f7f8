"""Environment-batch sharding across ranks: contiguous env ranges, no data-path collective.

Environments are independent in every operation of the trunk (attention is within an
environment, the recurrence is per ship), so rank r of W simply takes environments
[lo, hi) and the matching contiguous token rows and hidden rows (hidden rows are env-major,
models/yemong/policy.py:284 of the reference).
"""

from __future__ import annotations

import dataclasses

import torch

from .workloads import Workload


def env_shard(n_envs: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous environment range of `rank`; sizes differ by at most one."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n_envs, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_workload(w: Workload, rank: int, world: int) -> Workload:
    """The part of a workload that `rank` owns (views where possible)."""
    if w.kind == "ragged":
        n = w.n_tokens.numel()
        lo, hi = env_shard(n, rank, world)
        tok = torch.zeros(n + 1, dtype=torch.long)
        ship = torch.zeros(n + 1, dtype=torch.long)
        tok[1:] = w.n_tokens.cumsum(0)
        ship[1:] = w.n_ships.cumsum(0)
        return dataclasses.replace(
            w, x=w.x[tok[lo] : tok[hi]], alive=w.alive[tok[lo] : tok[hi]],
            hidden=w.hidden[:, ship[lo] : ship[hi]], n_tokens=w.n_tokens[lo:hi], n_ships=w.n_ships[lo:hi],
            bullets=None if w.bullets is None else w.bullets[lo:hi],
            bullet_mask=None if w.bullet_mask is None else w.bullet_mask[lo:hi],
            meta=dict(w.meta, n_envs=hi - lo),
        )
    env_dim = 1 if w.kind == "sequence" else 0
    n = w.x.shape[env_dim]
    lo, hi = env_shard(n, rank, world)
    ships = w.meta.get("ships", 0)
    sl = (slice(None),) * env_dim + (slice(lo, hi),)
    return dataclasses.replace(
        w, x=w.x[sl], alive=None if w.alive is None else w.alive[sl],
        hidden=None if w.hidden is None else w.hidden[:, lo * ships : hi * ships],
        done=None if w.done is None else w.done[:, lo:hi],
        # bullets of a step are env-major like x (a sequence's are (T * n_envs, ...): not sharded here)
        bullets=None if w.bullets is None or env_dim else w.bullets[lo:hi],
        bullet_mask=None if w.bullet_mask is None or env_dim else w.bullet_mask[lo:hi],
        meta=dict(w.meta, n_envs=hi - lo),
    )


def max_over_ranks(value: float, device: torch.device | str = "cpu") -> float:
    """Max of a per-rank scalar (device time) over the default process group."""
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])
