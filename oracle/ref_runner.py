"""The reference's own trunk, run from the copy under ``oracle/_ref`` (see make_ref.py).

TEST INFRASTRUCTURE, not product code: only tests and bench.py's reference legs import this.
It builds the reference's ``YemongBlock`` modules (models/yemong/griffin.py:335) from the
reference's ``ModelConfig`` with ``torch.manual_seed(0)`` and their own default init, and chains
them exactly as the reference's policy does: models/yemong/policy.py:315-354 for a rollout step,
policy.py:422-478 for the recurrent-PPO sequence forward.  Nothing here is a restatement: every
arithmetic operation runs inside the reference's modules.
"""

from __future__ import annotations

import sys

import torch

from . import make_ref

RL_FIELDS = dict(d_model=128, n_heads=4, n_yemong_blocks=2, n_spatial_per_block=2, n_temporal_per_block=1,
                 n_bullet_cross_per_block=1)
CONV_KERNEL = 4


def available() -> bool:
    return make_ref.ref_path() is not None


def _import_ref():
    path = make_ref.ref_path()
    if path is None:
        raise RuntimeError("oracle/_ref is absent: run `python oracle/make_ref.py` where the reference tree exists")
    if path not in sys.path:
        sys.path.insert(0, path)
    from boost_and_broadside.config import ModelConfig
    from boost_and_broadside.models.yemong.griffin import YemongBlock

    return ModelConfig, YemongBlock


class ReferenceTrunk(torch.nn.Module):
    """``yemong_layers`` of the reference's YemongPolicy and the two loops that drive them."""

    def __init__(self, fields: dict | None = None, seed: int = 0):
        super().__init__()
        ModelConfig, YemongBlock = _import_ref()
        self.cfg = ModelConfig(**(fields or RL_FIELDS))
        torch.manual_seed(seed)
        self.yemong_layers = torch.nn.ModuleList([YemongBlock(self.cfg) for _ in range(self.cfg.n_yemong_blocks)])
        self.n_temporal = self.cfg.n_temporal_per_block

    def step(self, x, alive, hidden, bullets=None, bullet_mask=None):
        """models/yemong/policy.py:315-354: x (B, N+M, D), hidden (L, B*N, 4D) -> (x, new hidden)."""
        B, _, D = x.shape
        n_layers, B_rec = hidden.shape[0], hidden.shape[1]
        n_rec = B_rec // B
        rglru = hidden[:, :, :D]
        conv = hidden[:, :, D:].reshape(n_layers, B_rec, CONV_KERNEL - 1, D)
        new_h, new_cb = [], []
        for i, layer in enumerate(self.yemong_layers):
            sl = slice(i * self.n_temporal, (i + 1) * self.n_temporal)
            x, h, cb = layer.step(x, alive, rglru[sl], conv[sl], n_rec, bullets, bullet_mask)
            new_h.append(h)
            new_cb.append(cb)
        width = (CONV_KERNEL - 1) * D
        h_t = torch.cat(new_h, dim=0) if new_h else rglru
        cb_t = torch.cat(new_cb, dim=0).reshape(n_layers, B_rec, width) if new_cb else conv.reshape(n_layers, B_rec, width)
        return x, torch.cat([h_t, cb_t], dim=-1)

    def sequence(self, x, alive, hidden, done, bullets=None, bullet_mask=None):
        """models/yemong/policy.py:422-478: x (T, B, N+M, D) -> x (the final states are discarded there)."""
        T, B, _, D = x.shape
        n_layers, B_rec = hidden.shape[0], hidden.shape[1]
        n_rec = B_rec // B
        rglru = hidden[:, :, :D]
        conv = hidden[:, :, D:].reshape(n_layers, B_rec, CONV_KERNEL - 1, D)
        for i, layer in enumerate(self.yemong_layers):
            sl = slice(i * self.n_temporal, (i + 1) * self.n_temporal)
            x, _, _ = layer.sequence(x, alive, rglru[sl], conv[sl], done, n_rec, bullets, bullet_mask)
        return x

    def step_ragged(self, x, alive, hidden, n_tokens, n_ships):
        """A ragged batch, which one call of the reference cannot express (griffin.py:398-399 takes
        one ship count per call): environments are grouped by (tokens, ships) and each group is one
        reference step.  x (total_tokens, D), hidden (L, total_ships, 4D)."""
        D = x.shape[-1]
        tok_off = [0]
        ship_off = [0]
        for n, s in zip(n_tokens, n_ships):
            tok_off.append(tok_off[-1] + n)
            ship_off.append(ship_off[-1] + s)
        groups: dict[tuple[int, int], list[int]] = {}
        for e, key in enumerate(zip(n_tokens, n_ships)):
            groups.setdefault(key, []).append(e)
        y = torch.empty_like(x)
        new_hidden = torch.empty_like(hidden)
        for (n, s), envs in groups.items():
            tok_idx = torch.cat([torch.arange(tok_off[e], tok_off[e] + n) for e in envs]).to(x.device)
            xg = x[tok_idx].reshape(len(envs), n, D)
            ag = alive[tok_idx].reshape(len(envs), n)
            if s > 0:
                ship_idx = torch.cat([torch.arange(ship_off[e], ship_off[e] + s) for e in envs]).to(x.device)
                hg = hidden[:, ship_idx]
            else:
                ship_idx = None
                hg = hidden[:, :0]
            if s > 0:
                yg, hn = self.step(xg, ag, hg)
                new_hidden[:, ship_idx] = hn
            else:
                # no recurrent token: the policy's split (n_rec = 0) sends every token down the field path
                yg, _ = self.step(xg, ag, hg)
            y[tok_idx] = yg.reshape(-1, D)
        return y, new_hidden


def workload_runner(trunk: ReferenceTrunk, w, device: str = "cpu", token_dtype: torch.dtype | None = None):
    """A zero-argument callable that runs workload ``w`` (boost-and-broadside_b200/workloads.py)
    through the reference trunk on ``device`` under the workload's precision; ``token_dtype``
    converts the tokens first (bfloat16: what the reference's encoder produces under CUDA autocast)."""
    dev = torch.device(device)

    def to(t):
        return None if t is None else t.to(dev)

    x, alive, hidden = to(w.x), to(w.alive), to(w.hidden)
    if token_dtype is not None:
        x = x.to(token_dtype)
    ctx = (lambda: torch.autocast(dev.type, dtype=torch.bfloat16)) if w.mode == "bf16" else (lambda: torch.autocast(dev.type, enabled=False))
    if w.kind == "step":
        B = w.meta["n_envs"]
        xb = x.reshape(B, -1, x.shape[-1])
        ab = alive.reshape(B, -1)
        bul, mask = to(w.bullets), to(w.bullet_mask)

        def run():
            with torch.no_grad(), ctx():
                return trunk.step(xb, ab, hidden, bul, mask)
    elif w.kind == "sequence":
        T = x.shape[0]
        B = w.meta["n_envs"]
        xb = x.reshape(T, B, -1, x.shape[-1])
        ab = alive.reshape(T, B, -1)
        done = to(w.done)

        def run():
            with torch.no_grad(), ctx():
                return trunk.sequence(xb, ab, hidden, done)
    else:
        nt, ns = w.n_tokens.tolist(), w.n_ships.tolist()

        def run():
            with torch.no_grad(), ctx():
                return trunk.step_ragged(x, alive, hidden, nt, ns)
    return run


def reference_policy(num_ships: int, fields: dict | None = None, seed: int = 0):
    """The reference's whole ``YemongPolicy`` (models/yemong/policy.py:136) with its standard ship and
    bullet FeatureCoordinators (train/rl/features.py), default init under ``torch.manual_seed(seed)``,
    eleven value components and the win components pooled per team, as the reference's trainer builds it."""
    _import_ref()
    from boost_and_broadside.config import ModelConfig, ShipConfig
    from boost_and_broadside.models.yemong.policy import YemongPolicy
    from boost_and_broadside.train.rl.features import build_bullet_coordinator, build_standard_coordinator

    ships = ShipConfig()
    torch.manual_seed(seed)
    return YemongPolicy(ModelConfig(**(fields or RL_FIELDS)), build_standard_coordinator(ships), num_value_components=11,
                        num_ships=num_ships, team_pma_k=(0, 1), bullet_coordinator=build_bullet_coordinator(ships)).eval()


def random_observation(n_envs: int, n_ships: int, n_fields: int, n_bullets: int, seed: int, device: str = "cpu"):
    """A seeded random observation in the reference's own container (env/observation.py): every key the
    standard coordinators read, ``n_ships`` ships (two teams) then ``n_fields`` fields per environment,
    ``n_bullets`` bullet slots of which about 40 % are active."""
    _import_ref()
    from boost_and_broadside.env.observation import BulletObsKey, ObsKey, YemongObservation

    g = torch.Generator().manual_seed(seed)
    B, T, NB = n_envs, n_ships + n_fields, n_bullets
    r = lambda *s: torch.rand(*s, generator=g)   # noqa: E731
    n = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    team = torch.cat([torch.zeros(n_ships // 2), torch.ones(n_ships - n_ships // 2),
                      torch.full((n_fields,), 2.0)]).long().expand(B, -1).contiguous()
    data = {
        ObsKey.POS: r(B, T, 2), ObsKey.VEL: n(B, T, 2) * 100, ObsKey.ATT: n(B, T, 2), ObsKey.ANG_VEL: n(B, T, 1),
        ObsKey.HEALTH: r(B, T, 1), ObsKey.POWER: r(B, T, 1), ObsKey.COOLDOWN: r(B, T, 1), ObsKey.TEAM_ID: team,
        ObsKey.ALIVE: torch.ones(B, T, dtype=torch.bool), ObsKey.PREVIOUS_ACTION: torch.randint(0, 2, (B, T, 3), generator=g),
        ObsKey.RADIUS: r(B, T, 1), ObsKey.LOCAL_LOG_INDEX: n(B, T, 1) * 0.1, ObsKey.LOCAL_INDEX_GRADIENT: n(B, T, 2) * 0.1,
        ObsKey.FIELD_TRANSITION_WIDTH: r(B, T, 1), ObsKey.FIELD_INSIDE_LOG_INDEX: n(B, T, 1) * 0.1,
        ObsKey.FIELD_OUTSIDE_LOG_INDEX: n(B, T, 1) * 0.1, ObsKey.FIELD_LOG_INDEX_RATIO: n(B, T, 1) * 0.1,
        ObsKey.FIELD_DAMAGE: r(B, T, 1),
    }
    bullets = {
        BulletObsKey.POS: r(B, NB, 2) * 1024.0, BulletObsKey.VEL: n(B, NB, 2) * 400.0, BulletObsKey.DAMAGE: r(B, NB, 1),
        BulletObsKey.LIFETIME: r(B, NB, 1), BulletObsKey.LOCAL_LOG_INDEX: n(B, NB, 1) * 0.1,
        BulletObsKey.LOCAL_INDEX_GRADIENT: n(B, NB, 2) * 0.1, BulletObsKey.TEAM_ID: torch.randint(0, 2, (B, NB), generator=g),
        BulletObsKey.ACTIVE: r(B, NB) < 0.4,
    }
    to = lambda d: {k: v.to(device) for k, v in d.items()}  # noqa: E731
    return YemongObservation(data=to(data), bullets=to(bullets))
