"""The token encoders in front of the trunk (rows f-2 / f-4): ``ShipEncoder`` (shared and split
layouts) and ``BulletEncoder`` against the golden fixtures the reference's modules produced
(tests/golden/encoder_*.npz, CPU autocast) and, on the GPU, against the reference's own encoders
on whole observations (oracle/_ref), and chained into the trunk with bfloat16 tokens.

Tolerances: float32 max-abs <= 1e-4; bf16 normalised max error <= 2e-2 (measured about 4e-3: the
chain ends in two bf16 roundings of O(1) values).
"""

from __future__ import annotations

import sys

import pytest
import torch

from oracle import make_ref, ref_runner
from tests.helpers import assert_close, golden, stored_weights

pytestmark = pytest.mark.gpu
DEV = "cuda"


class _Coordinator:
    """Stand-in with the two numbers a ShipEncoder / BulletEncoder constructor reads."""

    def __init__(self, total, ship=None, field=None):
        self.total_input_dimension = total
        self._scoped = {"SHIP": ship, "FIELD": field}

    def scoped_input_dimension(self, scope):
        return self._scoped[scope.name if hasattr(scope, "name") else str(scope)]


class FeatureScope:   # the enum the split layout looks up next to the coordinator's class
    class _S:
        def __init__(self, name):
            self.name = name

    SHIP = _S("SHIP")
    FIELD = _S("FIELD")


def _cfg(split=False):
    from boost_and_broadside_b200 import ModelConfig

    return ModelConfig(d_model=128, n_heads=4, n_yemong_blocks=2, encoder_split=split, n_bullet_cross_per_block=1)


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
def test_encoder_chains_match_the_reference_fixtures(mode):
    from boost_and_broadside_b200 import BulletEncoder, ShipEncoder

    ctx = torch.autocast(DEV, dtype=torch.bfloat16) if mode == "bf16" else torch.autocast(DEV, enabled=False)
    want_dtype = torch.bfloat16 if mode == "bf16" else torch.float32

    g = golden("encoder_ship_shared")
    enc = ShipEncoder(_cfg(), _Coordinator(66)).eval()
    enc.load_state_dict(stored_weights(g), strict=True)
    enc = enc.to(DEV)
    with torch.no_grad(), ctx:
        y = enc.encode_raw(g["raw"].to(DEV))
    assert y.dtype == want_dtype
    assert_close(y, g["y_" + mode], mode, "ship encoder (shared)")

    g = golden("encoder_ship_split")
    enc = ShipEncoder(_cfg(split=True), _Coordinator(89, ship=61, field=28), num_ships=8).eval()
    enc.load_state_dict(stored_weights(g), strict=True)
    enc = enc.to(DEV)
    with torch.no_grad(), ctx:
        y = enc.encode_raw(g["ship_raw"].to(DEV), g["field_raw"].to(DEV))
    assert_close(y, g["y_" + mode], mode, "ship encoder (split)")

    g = golden("encoder_bullet")
    benc = BulletEncoder(_cfg(), _Coordinator(26)).eval()
    benc.load_state_dict(stored_weights(g), strict=True)
    benc = benc.to(DEV)
    with torch.no_grad(), ctx:
        y = benc.encode_raw(g["raw"].to(DEV))
    assert y.dtype == want_dtype
    assert_close(y, g["y_" + mode], mode, "bullet encoder")


def _observation(B, N, M, NB, seed):
    """A random observation in the reference's own container (env/observation.py)."""
    sys.path.insert(0, make_ref.ref_path())
    from boost_and_broadside.env.observation import BulletObsKey, ObsKey, YemongObservation

    g = torch.Generator().manual_seed(seed)
    T = N + M
    r = lambda *s: torch.rand(*s, generator=g)
    n = lambda *s: torch.randn(*s, generator=g)
    team = torch.cat([torch.zeros(N // 2), torch.ones(N - N // 2), torch.full((M,), 2.0)]).long().expand(B, -1).contiguous()
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
    to = lambda d: {k: v.to(DEV) for k, v in d.items()}
    return YemongObservation(data=to(data), bullets=to(bullets))


@pytest.mark.skipif(not ref_runner.available(), reason="oracle/_ref has not been built")
@pytest.mark.parametrize("mode", ["fp32", "bf16"])
@pytest.mark.parametrize("split", [False, True])
def test_encoders_on_observations_against_the_reference_and_into_the_trunk(split, mode):
    """The reference's own ShipEncoder / BulletEncoder and this package's, same seed, same
    observation, through the reference's FeatureCoordinator; then the encoded tokens (bfloat16 under
    autocast) straight into the trunk with the encoded bullets."""
    sys.path.insert(0, make_ref.ref_path())
    from boost_and_broadside.config import ModelConfig as RefConfig
    from boost_and_broadside.config import ShipConfig
    from boost_and_broadside.models.yemong import encoder as ref_encoder
    from boost_and_broadside.train.rl.features import build_bullet_coordinator, build_standard_coordinator

    import boost_and_broadside_b200 as bnb

    cfg = RefConfig(d_model=128, n_heads=4, n_yemong_blocks=2, n_spatial_per_block=2, n_temporal_per_block=1,
                    n_bullet_cross_per_block=1, encoder_split=split)
    ships = ShipConfig()
    sc, bc = build_standard_coordinator(ships), build_bullet_coordinator(ships)
    B, N, M, NB = 24, 8, 4, 80
    torch.manual_seed(0)
    ref_ship, ref_bul = ref_encoder.ShipEncoder(cfg, sc, num_ships=N).eval().to(DEV), ref_encoder.BulletEncoder(cfg, bc).eval().to(DEV)
    torch.manual_seed(0)
    our_ship, our_bul = bnb.ShipEncoder(cfg, sc, num_ships=N).eval().to(DEV), bnb.BulletEncoder(cfg, bc).eval().to(DEV)
    assert list(ref_ship.state_dict()) == list(our_ship.state_dict()) and list(ref_bul.state_dict()) == list(our_bul.state_dict())
    assert all(torch.equal(a, b) for a, b in zip(ref_ship.state_dict().values(), our_ship.state_dict().values()))
    obs = _observation(B, N, M, NB, seed=7)
    ctx = torch.autocast(DEV, dtype=torch.bfloat16) if mode == "bf16" else torch.autocast(DEV, enabled=False)
    with torch.no_grad(), ctx:
        want_x, want_b = ref_ship(obs), ref_bul(obs)
        got_x, got_b = our_ship(obs), our_bul(obs)
    assert got_x.dtype == want_x.dtype and got_b.dtype == want_b.dtype
    assert got_x.shape == (B, N + M, 128) and got_b.shape == (B, NB, 128)
    assert_close(got_x, want_x, mode, "ship tokens")
    assert_close(got_b, want_b, mode, "bullet tokens")

    # encoded tokens and bullets into the trunk, dtype as produced
    torch.manual_seed(0)
    trunk = bnb.YemongTrunk(cfg).eval().to(DEV)
    ref_trunk = ref_runner.ReferenceTrunk().eval().to(DEV)
    hidden = torch.randn(2, B * N, 512, device=DEV) * 0.5
    from boost_and_broadside.env.observation import BulletObsKey

    alive, mask = obs["alive"], obs.bullets[BulletObsKey.ACTIVE]
    with torch.no_grad(), ctx:
        y, nh = trunk.step(got_x, alive, hidden, bullets=got_b, bullet_mask=mask)
        ry, rnh = ref_trunk.step(want_x, alive, hidden, want_b, mask)
    assert y.dtype == ry.dtype
    assert_close(y, ry.float(), mode, "trunk output from encoded tokens", scale=1.0 if mode == "fp32" else 1.0)
    assert_close(nh, rnh, mode, "hidden from encoded tokens")
