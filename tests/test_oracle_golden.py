"""The CPU oracle against outputs of the reference itself (tests/golden/*.npz)."""

import pytest
import torch

from oracle import trunk_oracle as O
from tests.helpers import assert_close, build_trunk, golden, stored_weights, trunk_params

MODES = ("fp32", "bf16")


def _spatial_params(g, D, H):
    w = stored_weights(g)
    if w:
        return w
    from boost_and_broadside_b200 import ModelConfig, TransformerBlock

    torch.manual_seed(0)
    return dict(TransformerBlock(ModelConfig(D, H, 2)).state_dict())


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", ["spatial_d128_n8", "spatial_d128_n152", "spatial_d64_n5", "spatial_d32_n3", "spatial_d32h2_n40"])
def test_spatial_block(name, mode):
    g = golden(name)
    D, H = (int(v) for v in g["dims"])
    p = _spatial_params(g, D, H)
    y = O.spatial_block(g["x"], g["alive"], p, H, mode)
    assert_close(y, g["y_" + mode], mode, name)
    y = O.spatial_block(g["x"], None, p, H, mode)
    assert_close(y, g["y_nomask_" + mode], mode, name + " (no mask)")


def test_all_dead_environment_is_uniform_mean():
    """An environment without a live key averages v over all its keys (attention.py:101-112)."""
    g = golden("spatial_d128_n8")
    assert not g["alive"][-1].any()
    q = torch.randn(1, 2, 5, 8)
    v = torch.randn(1, 2, 5, 8)
    out = O.masked_attention(q, torch.randn(1, 2, 5, 8), v, torch.zeros(1, 5, dtype=torch.bool), "fp32")
    assert torch.allclose(out, v.mean(dim=2, keepdim=True).expand_as(out), atol=1e-6)


def _temporal_params(g, D):
    w = stored_weights(g)
    if w:
        sub = w.pop("__sub.weight")
        return w, sub
    from boost_and_broadside_b200 import GriffinTemporalBlock

    torch.manual_seed(0)
    tb = GriffinTemporalBlock(D)
    sub = torch.nn.Linear(D, D, bias=False)
    p = dict(tb.state_dict())
    p["conv.bias"] = g["conv_bias"]
    return p, sub.weight.detach()


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", ["temporal_d128_t1", "temporal_d128_t9", "temporal_d64_t6"])
def test_temporal_block(name, mode):
    g = golden(name)
    D = int(g["dims"][0])
    p, sub = _temporal_params(g, D)
    y, h, c = O.temporal_sequence(g["x"], g["h0"], g["conv"], None, p, mode)
    assert_close(y, g["y_" + mode], mode, name + " y")
    assert_close(h, g["h_" + mode], mode, name + " h")
    assert_close(c, g["c_" + mode], mode, name + " conv")
    if "yd_" + mode in g:
        y, h, c = O.temporal_sequence(g["x"], g["h0"], g["conv"], g["done"], p, mode)
        assert_close(y, g["yd_" + mode], mode, name + " y (done)")
        assert_close(h, g["hd_" + mode], mode, name + " h (done)")
        assert_close(c, g["cd_" + mode], mode, name + " conv (done)")
    yf = O.temporal_nonrecurrent(g["x"], p, sub, mode)
    assert_close(yf, g["yf_" + mode], mode, name + " field path")


STEP_CASES = ["trunk_step_d128_8s4f", "trunk_step_d128_8s0f", "trunk_step_d128_30s2f", "trunk_step_d64_3s2f",
              "trunk_step_d32_2s1f_b132"]
SEQ_CASES = ["trunk_seq_d128_t6_8s0f", "trunk_seq_d128_t5_4s2f", "trunk_seq_d64_t7_3s2f"]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", STEP_CASES)
def test_trunk_step(name, mode):
    g = golden(name)
    trunk = build_trunk(g["dims"], g)
    H = int(g["dims"][1])
    y, nh = O.trunk_step(g["x"], g["alive"], g["hidden"], trunk_params(trunk), H, mode)
    assert_close(y, g["y_" + mode], mode, name + " y")
    assert_close(nh, g["hidden_" + mode], mode, name + " hidden")


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", SEQ_CASES)
def test_trunk_sequence(name, mode):
    g = golden(name)
    trunk = build_trunk(g["dims"], g)
    H = int(g["dims"][1])
    P = trunk_params(trunk)
    y, nh = O.trunk_sequence(g["x"], g["alive"], g["hidden"], g["done"], P, H, mode)
    assert_close(y, g["y_" + mode], mode, name + " y")
    assert_close(nh, g["hidden_" + mode], mode, name + " hidden")
    y, nh = O.trunk_sequence(g["x"], g["alive"], g["hidden"], None, P, H, mode)
    assert_close(y, g["y_nodone_" + mode], mode, name + " y (no done)")
    assert_close(nh, g["hidden_nodone_" + mode], mode, name + " hidden (no done)")


@pytest.mark.parametrize("name", SEQ_CASES)
def test_sequence_equals_steps_with_resets(name):
    """The load-bearing property of the trunk (tests/models/test_encoder.py:516-569 of the
    reference): one sequence forward equals stepping with reset_hidden_for_envs."""
    g = golden(name)
    trunk = build_trunk(g["dims"], g)
    H = int(g["dims"][1])
    P = trunk_params(trunk)
    y_seq, _ = O.trunk_sequence(g["x"], g["alive"], g["hidden"], g["done"], P, H, "fp32")
    y_steps, _ = O.trunk_sequence_by_steps(g["x"], g["alive"], g["hidden"], g["done"], P, H, "fp32")
    assert float((y_seq - y_steps).abs().max()) < 1e-4
    assert_close(y_steps, g["y_steps_fp32"], "fp32", name + " reference step loop")


def test_ragged_grouping_matches_uniform():
    g = golden("trunk_step_d128_8s4f")
    trunk = build_trunk(g["dims"], g)
    P = trunk_params(trunk)
    B, NM, D = g["x"].shape
    y0, h0 = O.trunk_step(g["x"], g["alive"], g["hidden"], P, 4, "fp32")
    y1, h1 = O.trunk_step_ragged(g["x"].reshape(-1, D), g["alive"].reshape(-1), g["hidden"], [NM] * B, [8] * B, P, 4, "fp32")
    assert torch.equal(y0.reshape(-1, D), y1) and torch.equal(h0, h1)


# ----------------------------------------------------------------------------- bullet cross-attention


def _bullet_spatial_params(g, D, H):
    w = stored_weights(g)
    if w:
        return w
    from boost_and_broadside_b200 import ModelConfig, TransformerBlock

    torch.manual_seed(0)
    p = dict(TransformerBlock(ModelConfig(D, H, 2), reads_bullets=True).state_dict())
    p["norm_bullet.weight"] = g["norm_bullet"]
    return p


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", ["bullets_spatial_d128_n12_nb80", "bullets_spatial_d32_n3_nb7"])
def test_spatial_block_with_bullets(name, mode):
    """attention.py:149-166: second softmax over bullet keys, gated per environment."""
    g = golden(name)
    D, H = (int(v) for v in g["dims"])
    p = _bullet_spatial_params(g, D, H)
    assert not g["bullet_mask"][1].any() and g["bullet_mask"][2].all()
    y = O.spatial_block(g["x"], g["alive"], p, H, mode, g["bullets"], g["bullet_mask"])
    assert_close(y, g["y_" + mode], mode, name)
    y = O.spatial_block(g["x"], g["alive"], p, H, mode, g["bullets"], None)
    assert_close(y, g["y_nobmask_" + mode], mode, name + " (no bullet mask)")
    y0 = O.spatial_block(g["x"], g["alive"], p, H, mode)
    assert_close(y0, g["y_nobullets_" + mode], mode, name + " (no bullets)")
    # an environment with nothing in flight gets exactly the bullet-free result
    y = O.spatial_block(g["x"], g["alive"], p, H, mode, g["bullets"], g["bullet_mask"])
    assert torch.equal(y[1], y0[1])


@pytest.mark.parametrize("mode", MODES)
def test_trunk_step_with_bullets(mode):
    g = golden("bullets_trunk_step_d128_8s4f")
    trunk = build_trunk(g["dims"], g)
    y, nh = O.trunk_step(g["x"], g["alive"], g["hidden"], trunk_params(trunk), 4, mode, g["bullets"], g["bullet_mask"])
    assert_close(y, g["y_" + mode], mode, "bullets step y")
    assert_close(nh, g["hidden_" + mode], mode, "bullets step hidden")


@pytest.mark.parametrize("mode", MODES)
def test_trunk_sequence_with_bullets(mode):
    g = golden("bullets_trunk_seq_d128_t4_4s2f")
    trunk = build_trunk(g["dims"], g)
    y, nh = O.trunk_sequence(g["x"], g["alive"], g["hidden"], g["done"], trunk_params(trunk), 4, mode,
                             g["bullets"], g["bullet_mask"])
    assert_close(y, g["y_" + mode], mode, "bullets sequence y")
    assert_close(nh, g["hidden_" + mode], mode, "bullets sequence hidden")


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
def test_encoder_chains_match_the_reference(mode):
    """ShipEncoder (shared and split layouts) and BulletEncoder MLP chains against the fixtures the
    reference's modules produced (models/yemong/encoder.py)."""
    from oracle.trunk_oracle import encoder_mlp

    g = golden("encoder_ship_shared")
    w = stored_weights(g)
    y = encoder_mlp(g["raw"], w["feature_extractor.0.weight"], w["feature_extractor.0.bias"], w["feature_extractor.1.weight"],
                    w["feature_extractor.3.weight"], w["feature_extractor.3.bias"], w["feature_extractor.4.weight"], mode)
    assert_close(y, g["y_" + mode], mode, "ship encoder (shared)")
    g = golden("encoder_ship_split")
    w = stored_weights(g)
    shared = (w["shared_proj.0.weight"], w["shared_proj.0.bias"], w["shared_proj.1.weight"])
    ys = encoder_mlp(g["ship_raw"], w["ship_proj.0.weight"], w["ship_proj.0.bias"], w["ship_proj.1.weight"], *shared, mode)
    yf = encoder_mlp(g["field_raw"], w["field_proj.0.weight"], w["field_proj.0.bias"], w["field_proj.1.weight"], *shared, mode)
    assert_close(torch.cat([ys, yf], dim=-2), g["y_" + mode], mode, "ship encoder (split)")
    g = golden("encoder_bullet")
    w = stored_weights(g)
    y = encoder_mlp(g["raw"], w["net.0.weight"], w["net.0.bias"], w["net.1.weight"], w["net.3.weight"], w["net.3.bias"],
                    w["net.4.weight"], mode)
    assert_close(y, g["y_" + mode], mode, "bullet encoder")


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
def test_policy_heads_match_the_reference(mode):
    """action_head, value_head_local, value_head_win and next_state_head.net against the fixture a
    stock reference YemongPolicy produced (models/yemong/policy.py:185-214)."""
    from oracle.trunk_oracle import head_mlp

    g = golden("policy_heads")
    w = stored_weights(g)
    for name in ("action_head", "value_head_local", "value_head_win", "next_state_head"):
        y = head_mlp(g["x"], w[name + ".0.weight"], w[name + ".0.bias"], w[name + ".1.weight"], w[name + ".3.weight"],
                     w[name + ".3.bias"], mode)
        assert y.shape == g[f"{name}_{mode}"].shape
        assert_close(y, g[f"{name}_{mode}"], mode, name)
