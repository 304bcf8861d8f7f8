"""Seeded synthetic inputs for the five benchmark / parity configurations.

Everything is drawn on the CPU from ``torch.Generator`` seeds so that a CPU checker and
the GPU kernels see identical bits; callers move the tensors where they need them.

    C1  one spatial block, 256 envs x 8 ships, float32
    C2  trunk step, 8192 envs x (8 ships + 4 fields), bf16 autocast, hidden N(0, 0.5)
    C3  trunk step, 1024 envs x 152 ships (64 v 88), casualty fraction U(0, 0.7) per env
    C4  trunk sequence, T=32 x 4096 envs x 8 ships, done ~ Bernoulli(0.02)
    C5  trunk step, 16384 ragged envs, tokens U{2..128}, 0-4 fields, sharded by rank
    C2B C2 with the 80 bullet slots per environment (8 ships x 10) that the first spatial
        sublayer of each block cross-attends to; slots active ~ Bernoulli(0.3), a quarter of
        the environments with nothing in flight
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .config import ModelConfig

RL_FIELDS = dict(d_model=128, n_heads=4, n_yemong_blocks=2, n_spatial_per_block=2, n_temporal_per_block=1,
                 n_bullet_cross_per_block=1)


def rl_config() -> ModelConfig:
    """Trunk dims of the reference's ``rl`` / ``rl-fields`` profiles (config/defaults.py:21-31)."""
    return ModelConfig(**RL_FIELDS)


def team_alive(gen: torch.Generator, n_envs: int, n_ships: int, n_fields: int, p_alive: float = 0.9) -> torch.Tensor:
    """Ships alive ~ Bernoulli(p), first half team 0 and second half team 1 with at least one
    alive per team; field tokens always alive (env/observation.py:281 of the reference)."""
    alive = torch.rand(n_envs, n_ships, generator=gen) < p_alive
    half = n_ships // 2
    for lo, hi in ((0, half), (half, n_ships)):
        if hi <= lo:
            continue
        none = ~alive[:, lo:hi].any(dim=1)
        if none.any():
            pick = torch.randint(lo, hi, (int(none.sum()),), generator=gen)
            alive[none.nonzero().squeeze(1), pick] = True
    if n_fields:
        alive = torch.cat([alive, torch.ones(n_envs, n_fields, dtype=torch.bool)], dim=1)
    return alive


def casualty_alive(gen: torch.Generator, n_envs: int, team_sizes: tuple[int, int]) -> torch.Tensor:
    """Per-env casualty fraction f ~ U(0, 0.7); every ship dead with probability f; at least
    one alive per team."""
    n = sum(team_sizes)
    frac = torch.rand(n_envs, 1, generator=gen) * 0.7
    alive = torch.rand(n_envs, n, generator=gen) >= frac
    lo = 0
    for size in team_sizes:
        none = ~alive[:, lo : lo + size].any(dim=1)
        if none.any():
            pick = torch.randint(lo, lo + size, (int(none.sum()),), generator=gen)
            alive[none.nonzero().squeeze(1), pick] = True
        lo += size
    return alive


@dataclass
class Workload:
    name: str
    kind: str  # "spatial" | "step" | "sequence" | "ragged"
    mode: str  # "fp32" | "bf16"
    x: torch.Tensor
    alive: torch.Tensor | None
    hidden: torch.Tensor | None = None
    done: torch.Tensor | None = None
    n_tokens: torch.Tensor | None = None  # ragged only
    n_ships: torch.Tensor | None = None
    bullets: torch.Tensor | None = None      # (envs, NB, D) encoded bullet tokens
    bullet_mask: torch.Tensor | None = None  # (envs, NB) bool active slots
    meta: dict = field(default_factory=dict)

    @property
    def entity_tokens(self) -> int:
        """Real tokens processed by one pass (ships + fields, times T)."""
        if self.kind == "ragged":
            return int(self.n_tokens.sum())
        return self.x.numel() // self.x.shape[-1]


def c1(n_envs: int = 256, seed: int = 1) -> Workload:
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(n_envs, 8, 128, generator=gen)
    alive = team_alive(gen, n_envs, 8, 0)
    return Workload("C1", "spatial", "fp32", x, alive, meta=dict(n_envs=n_envs, ships=8, fields=0))


def c2(n_envs: int = 8192, seed: int = 2, ships: int = 8, fields: int = 4) -> Workload:
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(n_envs, ships + fields, 128, generator=gen)
    alive = team_alive(gen, n_envs, ships, fields)
    hidden = torch.randn(2, n_envs * ships, 512, generator=gen) * 0.5
    return Workload("C2", "step", "bf16", x, alive, hidden, meta=dict(n_envs=n_envs, ships=ships, fields=fields))


def c2b(n_envs: int = 8192, seed: int = 6, bullets_per_env: int = 80) -> Workload:
    """C2 plus encoded bullet tokens (the bullet encoder ends in an RMSNorm, so N(0, 1) values)."""
    w = c2(n_envs=n_envs, seed=seed)
    gen = torch.Generator().manual_seed(seed + 1000)
    w.name = "C2B"
    w.bullets = torch.randn(n_envs, bullets_per_env, 128, generator=gen)
    w.bullet_mask = torch.rand(n_envs, bullets_per_env, generator=gen) < 0.3
    w.bullet_mask[torch.rand(n_envs, generator=gen) < 0.25] = False
    w.meta["bullets"] = bullets_per_env
    return w


def c3(n_envs: int = 1024, seed: int = 3, teams: tuple[int, int] = (64, 88)) -> Workload:
    gen = torch.Generator().manual_seed(seed)
    n = sum(teams)
    x = torch.randn(n_envs, n, 128, generator=gen)
    alive = casualty_alive(gen, n_envs, teams)
    hidden = torch.randn(2, n_envs * n, 512, generator=gen) * 0.5
    return Workload("C3", "step", "bf16", x, alive, hidden, meta=dict(n_envs=n_envs, ships=n, fields=0))


def c4(n_envs: int = 4096, timesteps: int = 32, seed: int = 4) -> Workload:
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(timesteps, n_envs, 8, 128, generator=gen)
    alive = torch.ones(timesteps, n_envs, 8, dtype=torch.bool)
    hidden = torch.randn(2, n_envs * 8, 512, generator=gen) * 0.5
    done = torch.rand(timesteps, n_envs, generator=gen) < 0.02
    return Workload("C4", "sequence", "bf16", x, alive, hidden, done,
                    meta=dict(n_envs=n_envs, ships=8, fields=0, timesteps=timesteps))


def c5(n_envs: int = 16384, seed: int = 5, max_tokens: int = 128) -> Workload:
    """Ragged fleets: tokens n ~ U{2..max}, fields m ~ U{0..4} capped so that ships n - m >= 2
    and even (two equal teams); ships Bernoulli(0.9) alive with one alive per team."""
    gen = torch.Generator().manual_seed(seed)
    n = torch.randint(2, max_tokens + 1, (n_envs,), generator=gen)
    m = torch.randint(0, 5, (n_envs,), generator=gen)
    m = torch.minimum(m, n - 2)
    ships = n - m
    odd = ships % 2 == 1
    ships = ships - odd.long()  # an odd ship count gives one token to the fields ...
    m = m + odd.long()
    too_many = m > 4            # ... unless that breaks the field cap: drop the token instead
    n = n - too_many.long()
    m = m - too_many.long()
    total = int(n.sum())
    x = torch.randn(total, 128, generator=gen)
    alive = torch.ones(total, dtype=torch.bool)
    draw = torch.rand(total, generator=gen) < 0.9
    off = 0
    for e in range(n_envs):
        s = int(ships[e])
        a = draw[off : off + s].clone()
        half = s // 2
        if not a[:half].any():
            a[0] = True
        if not a[half:].any():
            a[half] = True
        alive[off : off + s] = a
        off += int(n[e])
    hidden = torch.randn(2, int(ships.sum()), 512, generator=gen) * 0.5
    return Workload("C5", "ragged", "bf16", x, alive, hidden, n_tokens=n, n_ships=ships,
                    meta=dict(n_envs=n_envs, max_tokens=max_tokens))


def algorithmic_bytes(w: Workload, n_params: int, n_hidden_layers: int = 2, d_model: int = 128) -> int:
    """Compulsory HBM bytes of one pass: x in + x out in float32, hidden in + out once per
    call, one byte per token of mask (+ one per (t, env) done flag), weights once at
    2 B/param (bf16) or 4 B/param (fp32); bullet tokens and their mask once."""
    tokens = w.entity_tokens
    b = 2 * 4 * d_model * tokens + tokens
    if w.bullets is not None:
        b += w.bullets.numel() * 4 + w.bullet_mask.numel()
    if w.hidden is not None:
        b += 2 * w.hidden.numel() * 4
    if w.done is not None:
        b += w.done.numel()
    b += n_params * (2 if w.mode == "bf16" else 4)
    return b


def algorithmic_flops(w: Workload, cfg: ModelConfig) -> int:
    """2 x MACs: spatial sublayer 16 D^2 per token + 4 D n_keys attention flops, temporal
    sublayer 17 D^2 per ship token, 16 D^2 per field token."""
    D = cfg.d_model
    ns = cfg.n_yemong_blocks * cfg.n_spatial_per_block
    nt = cfg.n_yemong_blocks * cfg.n_temporal_per_block
    if w.kind == "spatial":
        tokens, keys = w.entity_tokens, w.x.shape[1]
        return tokens * (2 * 16 * D * D + 4 * D * keys)
    if w.kind == "ragged":
        n = w.n_tokens.double()
        s = w.n_ships.double()
        att = float((n * n).sum()) * 4 * D
        return int(ns * (float(n.sum()) * 2 * 16 * D * D + att) + nt * 2 * D * D * (17 * float(s.sum()) + 16 * float((n - s).sum())))
    T = w.x.shape[0] if w.kind == "sequence" else 1
    envs, ships, fields = w.meta["n_envs"], w.meta["ships"], w.meta["fields"]
    keys = ships + fields
    tok = T * envs * keys
    total = ns * tok * (2 * 16 * D * D + 4 * D * keys) + nt * T * envs * 2 * D * D * (17 * ships + 16 * fields)
    if w.bullets is not None:
        # per reading sublayer: kv_bullet (2 D^2 MACs per bullet) and one more softmax over NB keys
        nb = w.bullets.shape[1]
        n_read = cfg.n_yemong_blocks * cfg.n_bullet_cross_per_block
        total += n_read * (T * envs * nb * 2 * 2 * D * D + tok * 4 * D * nb)
    return int(total)
