"""Seeded random geometries through the public modules against the CPU oracle: fleet sizes,
field counts, masks (dead ships, environments without a live key), done flags, folded resets,
bullet rings and ragged mixes that the hand-picked cases do not enumerate."""

import pytest
import torch

from oracle import trunk_oracle as O
from tests.helpers import assert_close, autocast_for, build_trunk, trunk_params

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(seed: int):
    g = torch.Generator().manual_seed(1000 + seed)
    r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))  # noqa: E731
    ships = r(1, 40) if seed % 4 else r(60, 150)
    fields = r(0, 4)
    n_envs = r(1, 30) if ships < 60 else r(1, 4)
    nb = r(1, 90) if seed % 3 else 0
    return g, n_envs, ships, fields, nb


def _inputs(g, n_envs, ships, fields, nb, T=None):
    lead = (n_envs,) if T is None else (T, n_envs)
    x = torch.randn(*lead, ships + fields, 128, generator=g)
    alive = torch.rand(*lead, ships + fields, generator=g) < 0.7
    alive.reshape(-1, ships + fields)[0] = False                      # one environment without a live key
    hidden = torch.randn(2, n_envs * ships, 512, generator=g) * 0.5
    E = n_envs if T is None else T * n_envs
    bul = torch.randn(E, nb, 128, generator=g) if nb else None
    bm = (torch.rand(E, nb, generator=g) < 0.4) if nb else None
    if nb:
        bm[E - 1] = False
    return x, alive, hidden, bul, bm


def _d(t):
    return None if t is None else t.to(DEV)


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
@pytest.mark.parametrize("seed", range(12))
def test_random_step(seed, mode):
    g, n_envs, ships, fields, nb = _case(seed)
    x, alive, hidden, bul, bm = _inputs(g, n_envs, ships, fields, nb)
    reset = torch.rand(n_envs, generator=g) < 0.3
    trunk = build_trunk([128, 4, 2, 2, 1, 1])
    P = trunk_params(trunk)
    h_in = O.reset_hidden_for_envs(hidden, reset, ships)
    ref_y, ref_h = O.trunk_step(x, alive, h_in, P, 4, mode, bul, bm)
    trunk = trunk.to(DEV)
    with torch.no_grad(), autocast_for(mode, DEV):
        y, h = trunk.step(_d(x), _d(alive), _d(hidden), reset_env=_d(reset), bullets=_d(bul), bullet_mask=_d(bm))
    what = f"seed {seed}: {n_envs} envs x ({ships}+{fields}), {nb} bullets"
    assert_close(y, ref_y, mode, what + " y")
    assert_close(h, ref_h, mode, what + " hidden")


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
@pytest.mark.parametrize("seed", range(6))
def test_random_sequence(seed, mode):
    g, n_envs, ships, fields, nb = _case(seed + 100)
    ships, n_envs = min(ships, 24), min(n_envs, 6)
    T = 2 + seed
    x, alive, hidden, bul, bm = _inputs(g, n_envs, ships, fields, nb, T)
    done = torch.rand(T, n_envs, generator=g) < 0.3
    trunk = build_trunk([128, 4, 2, 2, 1, 1])
    ref_y, ref_h = O.trunk_sequence(x, alive, hidden, done, trunk_params(trunk), 4, mode, bul, bm)
    trunk = trunk.to(DEV)
    with torch.no_grad(), autocast_for(mode, DEV):
        y, h = trunk.sequence(_d(x), _d(alive), _d(hidden), _d(done), bullets=_d(bul), bullet_mask=_d(bm))
    what = f"seed {seed}: T={T}, {n_envs} envs x ({ships}+{fields}), {nb} bullets"
    assert_close(y, ref_y, mode, what + " y")
    assert_close(h, ref_h, mode, what + " hidden")


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
@pytest.mark.parametrize("seed", range(4))
def test_random_ragged(seed, mode):
    from boost_and_broadside_b200 import RaggedBatch

    g = torch.Generator().manual_seed(2000 + seed)
    n_envs = int(torch.randint(1, 40, (1,), generator=g))
    n_tok = torch.randint(1, 129, (n_envs,), generator=g)
    n_ship = (torch.rand(n_envs, generator=g) * (n_tok + 1)).long().clamp(max=n_tok)  # 0 .. n_tok ships
    total, total_s = int(n_tok.sum()), int(n_ship.sum())
    x = torch.randn(total, 128, generator=g)
    alive = torch.rand(total, generator=g) < 0.8
    hidden = torch.randn(2, total_s, 512, generator=g) * 0.5
    nb = (0, 17, 64, 5)[seed]
    bul = torch.randn(n_envs, nb, 128, generator=g) if nb else None
    bm = (torch.rand(n_envs, nb, generator=g) < 0.5) if nb else None
    trunk = build_trunk([128, 4, 2, 2, 1, 1])
    ref_y, ref_h = O.trunk_step_ragged(x, alive, hidden, n_tok.tolist(), n_ship.tolist(), trunk_params(trunk), 4, mode,
                                       bul, bm)
    trunk = trunk.to(DEV)
    with torch.no_grad(), autocast_for(mode, DEV):
        y, h = trunk.step_ragged(_d(x), _d(alive), _d(hidden), RaggedBatch(n_tok, n_ship), bullets=_d(bul),
                                 bullet_mask=_d(bm))
    assert_close(y, ref_y, mode, f"ragged seed {seed} y")
    assert_close(h, ref_h, mode, f"ragged seed {seed} hidden")
