"""Host-side mirror of the reference interface: parameter names, shapes, init, errors."""

import os
import sys

import numpy as np
import pytest
import torch

from tests.helpers import build_trunk, checksum, golden


def test_state_dict_keys_match_reference_layout():
    trunk = build_trunk([128, 4, 2, 2, 1, 1])
    keys = set(trunk.state_dict())
    for i in range(2):
        for j in range(2):
            base = f"yemong_layers.{i}.spatial.{j}."
            for n in ("norm1.weight", "qkv.weight", "out_proj.weight", "norm2.weight", "ffn.gate_proj.weight",
                      "ffn.up_proj.weight", "ffn.down_proj.weight"):
                assert base + n in keys
        assert f"yemong_layers.{i}.spatial.0.kv_bullet.weight" in keys
        assert f"yemong_layers.{i}.spatial.1.kv_bullet.weight" not in keys
        base = f"yemong_layers.{i}.temporal.0."
        for n in ("norm1.weight", "linear1.weight", "conv.weight", "conv.bias", "rg_lru.log_lambda",
                  "rg_lru.linear_a.weight", "rg_lru.linear_a.bias", "rg_lru.linear_x.weight", "rg_lru.linear_x.bias",
                  "linear2.weight", "linear_out.weight", "norm2.weight", "gated_mlp.gate_proj.weight",
                  "gated_mlp.up_proj.weight", "gated_mlp.down_proj.weight"):
            assert base + n in keys
        assert f"yemong_layers.{i}.field_sub.0.weight" in keys
    sd = trunk.state_dict()
    assert sd["yemong_layers.0.spatial.0.qkv.weight"].shape == (384, 128)
    assert sd["yemong_layers.0.spatial.0.kv_bullet.weight"].shape == (256, 128)
    assert sd["yemong_layers.0.temporal.0.conv.weight"].shape == (128, 1, 4)
    assert all(v.dtype == torch.float32 for v in sd.values())
    assert sum(v.numel() for v in trunk.parameters()) == 1_707_776
    assert torch.equal(sd["yemong_layers.1.field_sub.0.weight"], torch.eye(128))
    assert torch.equal(sd["yemong_layers.0.temporal.0.rg_lru.log_lambda"], torch.linspace(0.0, 4.0, 128))


@pytest.mark.parametrize("name", ["trunk_step_d128_8s4f", "trunk_step_d64_3s2f", "trunk_seq_d128_t6_8s0f"])
def test_seeded_init_reproduces_reference_weights(name):
    """The mirror modules draw parameters in the reference's order, so seed 0 gives the
    reference's weights (checksums stored when the golden vectors were made)."""
    g = golden(name)
    trunk = build_trunk(g["dims"])
    got = checksum(trunk.state_dict())
    assert np.allclose(got, g["wsum"].numpy(), rtol=0, atol=1e-9), (got, g["wsum"])


def test_hidden_layout_helpers():
    trunk = build_trunk([64, 4, 3, 1, 2, 0])
    h = trunk.initial_hidden(5, 3, torch.device("cpu"))
    assert h.shape == (6, 15, 256) and h.dtype == torch.float32 and not h.any()
    assert trunk.n_hidden_layers == 6
    assert trunk.yemong_layers[0].n_temporal == 2


def test_no_cpu_path():
    from boost_and_broadside_b200 import ModelConfig, TransformerBlock

    block = TransformerBlock(ModelConfig(128, 4, 1))
    with pytest.raises(RuntimeError, match="no CPU path"):
        block(torch.zeros(1, 2, 128))
    trunk = build_trunk([128, 4, 1, 1, 1, 0])
    with pytest.raises(RuntimeError, match="no CPU path"):
        trunk.step(torch.zeros(1, 2, 128), None, torch.zeros(1, 2, 512))


def test_config_validation_mirrors_reference():
    from boost_and_broadside_b200 import ModelConfig

    with pytest.raises(ValueError):
        ModelConfig(130, 4, 1)
    with pytest.raises(ValueError):
        ModelConfig(128, 4, 1, n_spatial_per_block=1, n_bullet_cross_per_block=2)
    assert ModelConfig(128, 4, 2, 2, 1).n_hidden_layers == 2


def test_ragged_batch_offsets():
    from boost_and_broadside_b200 import RaggedBatch

    rb = RaggedBatch(torch.tensor([4, 2, 7]), torch.tensor([2, 2, 6]))
    geom, offsets = rb.build(torch.device("cpu"))
    n_envs, _, _, max_tokens, total_tokens, total_ships, n_tiles = geom
    assert n_envs == 3 and total_tokens == 13 and total_ships == 10 and max_tokens == 7
    assert offsets[0].tolist() == [0, 4, 6, 13] and offsets[1].tolist() == [0, 2, 4, 10]
    assert n_tiles == 1 and offsets[2].tolist() == [0, 3] and sorted(offsets[3].tolist()) == [0, 1, 2]
    with pytest.raises(RuntimeError):
        RaggedBatch(torch.tensor([2]), torch.tensor([3])).build(torch.device("cpu"))


def test_workload_generators_follow_the_configurations():
    from boost_and_broadside_b200 import workloads as W

    w = W.c1()
    assert w.x.shape == (256, 8, 128) and w.alive[:, :4].any(1).all() and w.alive[:, 4:].any(1).all()
    w = W.c2(n_envs=64)
    assert w.x.shape == (64, 12, 128) and w.hidden.shape == (2, 512, 512) and w.alive[:, 8:].all()
    assert abs(float(w.hidden.std()) - 0.5) < 0.01
    w = W.c3(n_envs=16)
    assert w.x.shape == (16, 152, 128) and w.alive[:, :64].any(1).all() and w.alive[:, 64:].any(1).all()
    w = W.c4(n_envs=8, timesteps=32)
    assert w.x.shape == (32, 8, 8, 128) and w.done.shape == (32, 8)
    w = W.c5(n_envs=500)
    n, s = w.n_tokens, w.n_ships
    assert int(n.min()) >= 2 and int(n.max()) <= 128 and bool((s >= 2).all()) and bool((s % 2 == 0).all())
    assert bool(((n - s) >= 0).all()) and bool(((n - s) <= 4).all())
    assert w.x.shape[0] == int(n.sum()) and w.hidden.shape[1] == int(s.sum())


def test_operators_are_registered_with_shape_only_fakes():
    """The opaque operators trace without touching a device: torch.compile records one node per
    trunk call and infers the output shapes from the fake implementations."""
    import boost_and_broadside_b200  # noqa: F401  (registers the operators)
    from torch._subclasses.fake_tensor import FakeTensorMode

    assert hasattr(torch.ops.bnb_b200, "trunk_forward") and hasattr(torch.ops.bnb_b200, "spatial_forward")
    with FakeTensorMode():
        x = torch.empty(5, 12, 128, device="cuda")
        hidden = torch.empty(2, 40, 512, device="cuda")
        w = [torch.empty(4, device="cuda")]
        y, h = torch.ops.bnb_b200.trunk_forward(x.reshape(60, 128), None, hidden, None, None, None, None, w, [],
                                                [0] * 16)
        assert y.shape == (60, 128) and h.shape == (2, 40, 512) and y.dtype == torch.float32
        y = torch.ops.bnb_b200.spatial_forward(x, None, None, None, w, 4, 1, 0)
        assert y.shape == (5, 12, 128)


@pytest.mark.skipif(not os.environ.get("BNB_REFERENCE_SRC"), reason="set BNB_REFERENCE_SRC to the reference's src/ folder")
def test_class_swap_inside_the_reference_policy():
    """The drop-in itself: the reference's YemongPolicy built with this package's YemongBlock in
    place of its own has the same state_dict keys and, from the same seed, the same values, and
    loads the reference's state_dict strictly.  Construction only; nothing is computed."""
    sys.path.insert(0, os.environ["BNB_REFERENCE_SRC"])
    import boost_and_broadside.models.yemong.policy as ref_policy
    from boost_and_broadside.config import ModelConfig as RefConfig
    from boost_and_broadside.config import ShipConfig
    from boost_and_broadside.train.rl.features import build_bullet_coordinator, build_standard_coordinator

    import boost_and_broadside_b200 as bnb

    cfg = RefConfig(d_model=128, n_heads=4, n_yemong_blocks=2, n_spatial_per_block=2, n_temporal_per_block=1,
                    n_bullet_cross_per_block=1)
    ships = ShipConfig()

    def make():
        torch.manual_seed(0)
        return ref_policy.YemongPolicy(cfg, build_standard_coordinator(ships), num_value_components=12, num_ships=8,
                                       team_pma_k=(), bullet_coordinator=build_bullet_coordinator(ships))

    reference = make()
    original = ref_policy.YemongBlock
    ref_policy.YemongBlock = bnb.YemongBlock
    try:
        swapped = make()
    finally:
        ref_policy.YemongBlock = original
    assert isinstance(swapped.yemong_layers[0], bnb.YemongBlock)
    a, b = reference.state_dict(), swapped.state_dict()
    assert list(a.keys()) == list(b.keys())
    assert all(torch.equal(a[k], b[k]) for k in a)
    swapped.load_state_dict(a, strict=True)
