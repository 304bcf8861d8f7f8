"""The assertions of the reference's own unit tests for this path, restated on this package's
modules at the reference's test dims (d_model 64 / 32, 4 heads):

    TestTransformerBlock          tests/models/test_encoder.py:106-176 of the reference
    TestRGLRU                     :179-268
    TestYemongBlockStructure      :408-589
    TestNonRecurrentFieldPath     :1041-1203

The reference drives the trunk through its encoder and heads; the encoder is outside this
package, so the trunk-level properties are checked from random encoded tokens instead of raw
observations (the properties -- shapes, step == sequence, episode boundaries, the field path
ignoring recurrent state -- are properties of the trunk, not of the encoder).  The tolerances are
the reference's own (1e-4 / 1e-5 / 1e-6 max-abs in float32).
"""

from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


def cfg(n_blocks=2, n_spatial=1, n_temporal=1, d_model=64, n_heads=4):
    from boost_and_broadside_b200 import ModelConfig

    return ModelConfig(d_model=d_model, n_heads=n_heads, n_yemong_blocks=n_blocks, n_spatial_per_block=n_spatial,
                       n_temporal_per_block=n_temporal)


def trunk_of(c):
    from boost_and_broadside_b200 import YemongTrunk

    torch.manual_seed(0)
    return YemongTrunk(c).eval().to(DEV)


# ------------------------------------------------------------------ TestTransformerBlock


def block64():
    from boost_and_broadside_b200 import TransformerBlock

    torch.manual_seed(0)
    return TransformerBlock(cfg()).eval().to(DEV)


def test_transformer_block_output_shape_unchanged():
    x = torch.randn(3, 8, 64, device=DEV)
    with torch.no_grad():
        out = block64()(x)
    assert out.shape == (3, 8, 64)


def test_transformer_block_with_a_partial_alive_mask():
    x = torch.randn(2, 4, 64, device=DEV)
    alive = torch.ones(2, 4, dtype=torch.bool, device=DEV)
    alive[0, 2] = False
    with torch.no_grad():
        out = block64()(x, alive_mask=alive)
    assert out.shape == (2, 4, 64) and torch.isfinite(out).all()


def test_transformer_block_all_dead_mask_gives_no_nan():
    x = torch.randn(1, 4, 64, device=DEV)
    alive = torch.zeros(1, 4, dtype=torch.bool, device=DEV)
    with torch.no_grad():
        out = block64()(x, alive_mask=alive)
    assert not torch.isnan(out).any()


def test_transformer_block_under_autocast_returns_float32_close_to_the_float32_result():
    """The reference's autocast regression test guards the dtype of its SDPA mask; there is no
    SDPA call here, so the observable contract is checked instead: a float32 result under
    torch.autocast, within the bf16 tolerance of the float32 run."""
    blk = block64()
    x = torch.randn(2, 4, 64, device=DEV)
    alive = torch.ones(2, 4, dtype=torch.bool, device=DEV)
    alive[0, 2] = False
    with torch.no_grad():
        ref = blk(x, alive_mask=alive)
        with torch.autocast(DEV, dtype=torch.bfloat16):
            out = blk(x, alive_mask=alive)
    assert out.dtype == torch.float32
    assert float((out - ref).abs().max() / ref.abs().max()) <= 2e-2


# ------------------------------------------------------------------ GatedMLP on its own


@pytest.mark.parametrize("d_model", [32, 64, 128])
def test_gated_mlp_forward_matches_its_torch_composition(d_model):
    from boost_and_broadside_b200 import GatedMLP

    torch.manual_seed(0)
    mlp = GatedMLP(d_model).eval().to(DEV)
    x = torch.randn(5, 7, d_model, device=DEV)
    with torch.no_grad():
        got = mlp(x)
        want = mlp.down_proj(F.gelu(mlp.gate_proj(x)) * mlp.up_proj(x))
        assert got.dtype == torch.float32 and got.shape == x.shape
        assert float((got - want).abs().max()) <= 1e-5
        with torch.autocast(DEV, dtype=torch.bfloat16):
            got16 = mlp(x)
            want16 = mlp.down_proj(F.gelu(mlp.gate_proj(x)) * mlp.up_proj(x))
    assert got16.dtype == torch.bfloat16 == want16.dtype
    assert float((got16.float() - want16.float()).abs().max() / want16.float().abs().max()) <= 2e-2


# ------------------------------------------------------------------ TestRGLRU


def rglru(d_model=32):
    from boost_and_broadside_b200 import RGLRU

    torch.manual_seed(0)
    return RGLRU(d_model).eval().to(DEV)


def sequential(unit, x_seq, h0):
    h = h0.clone()
    outs = []
    with torch.no_grad():
        for t in range(x_seq.shape[1]):
            h = unit._step(x_seq[:, t], h)
            outs.append(h)
    return torch.stack(outs, dim=1), h


def torch_step(unit, x, h):
    """griffin.py:169-186 with torch operators on the unit's own parameters."""
    r = torch.sigmoid(unit.linear_a(x))
    i = torch.sigmoid(unit.linear_x(x))
    a = torch.sigmoid(unit.log_lambda) ** (unit.c * r)
    gate = torch.sqrt(torch.clamp((1.0 - a) * (1.0 + a), min=1e-6))
    return a * h + gate * (i * x)


@pytest.mark.parametrize("B,T,atol", [(4, 128, 1e-4), (8, 1, 1e-5)])
def test_rglru_sequence_matches_the_sequential_step_loop(B, T, atol):
    unit = rglru()
    torch.manual_seed(1)
    x_seq, h0 = torch.randn(B, T, 32, device=DEV), torch.randn(B, 32, device=DEV)
    ref_out, ref_h = sequential(unit, x_seq, h0)
    with torch.no_grad():
        out, h = unit.forward_sequence(x_seq, h0)
        # and the step itself is the reference's formula
        want = torch_step(unit, x_seq[:, 0], h0)
    assert out.shape == (B, T, 32)
    assert torch.allclose(out, ref_out, atol=atol) and torch.allclose(h, ref_h, atol=atol)
    assert torch.allclose(out[:, 0], want, atol=1e-5)


def test_rglru_done_mask_cuts_the_state():
    unit = rglru()
    torch.manual_seed(4)
    x_seq, h0 = torch.randn(2, 8, 32, device=DEV), torch.randn(2, 32, device=DEV)
    done = torch.zeros(2, 8, dtype=torch.bool, device=DEV)
    done[0, 3] = True
    with torch.no_grad():
        with_done, _ = unit.forward_sequence(x_seq, h0, done)
        no_done, _ = unit.forward_sequence(x_seq, h0)
        fresh, _ = unit.forward_sequence(x_seq[:, 4:], torch.zeros(2, 32, device=DEV))
    assert torch.allclose(with_done[0, :4], no_done[0, :4], atol=1e-6)
    assert not torch.allclose(with_done[0, 4:], no_done[0, 4:], atol=1e-6)
    assert torch.allclose(with_done[1], no_done[1], atol=1e-6)
    assert torch.allclose(with_done[0, 4:], fresh[0], atol=1e-5)


def test_rglru_outputs_are_finite_in_the_training_precision():
    """The reference casts the module to bfloat16; here the parameters stay float32 (the reference's
    trainer keeps them so too) and the training precision is torch.autocast."""
    unit = rglru()
    torch.manual_seed(3)
    x_seq, h0 = torch.randn(4, 128, 32, device=DEV), torch.randn(4, 32, device=DEV)
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        out, h = unit.forward_sequence(x_seq, h0)
    assert torch.isfinite(out).all() and torch.isfinite(h).all()


# ------------------------------------------------------------------ TestYemongBlockStructure


@pytest.mark.parametrize("n_blocks,n_spatial,n_temporal", [(2, 1, 1), (2, 2, 1), (1, 4, 2), (3, 2, 1), (2, 2, 0)])
def test_sublayer_counts_match_config(n_blocks, n_spatial, n_temporal):
    trunk = trunk_of(cfg(n_blocks, n_spatial, n_temporal))
    assert len(trunk.yemong_layers) == n_blocks
    for block in trunk.yemong_layers:
        assert len(block.spatial) == n_spatial and len(block.temporal) == n_temporal


@pytest.mark.parametrize("n_blocks,n_temporal", [(2, 1), (2, 2), (1, 3), (3, 1), (2, 0)])
def test_hidden_state_has_one_slot_per_temporal_sublayer(n_blocks, n_temporal):
    from boost_and_broadside_b200 import CONV_KERNEL

    B, N, M = 2, 3, 2
    c = cfg(n_blocks, 2, n_temporal)
    trunk = trunk_of(c)
    hidden = trunk.initial_hidden(B, N + M, torch.device(DEV))
    assert hidden.shape == (n_blocks * n_temporal, B * (N + M), CONV_KERNEL * 64)
    assert c.n_hidden_layers == n_blocks * n_temporal
    x = torch.randn(B, N + M, 64, device=DEV)
    alive = torch.ones(B, N + M, dtype=torch.bool, device=DEV)
    with torch.no_grad():
        y, new_hidden = trunk.step(x, alive, hidden)
    assert new_hidden.shape == hidden.shape and y.shape == x.shape


def _step_loop(trunk, xs, alive, hidden, done=None, n_rec=None):
    ys = []
    with torch.no_grad():
        for t in range(xs.shape[0]):
            y, hidden = trunk.step(xs[t], alive[t], hidden)
            ys.append(y)
            if done is not None:
                hidden = trunk.reset_hidden_for_envs(hidden, done[t], n_rec)
    return torch.stack(ys, dim=0)


@pytest.mark.parametrize("n_blocks,n_spatial,n_temporal", [(2, 1, 1), (2, 2, 1), (1, 3, 2)])
def test_step_matches_sequence(n_blocks, n_spatial, n_temporal):
    """Rollout stepping and the full-sequence re-evaluation agree to 1e-5: the property PPO's ratio
    depends on."""
    B, N, M, T = 2, 3, 2, 6
    trunk = trunk_of(cfg(n_blocks, n_spatial, n_temporal))
    torch.manual_seed(7)
    xs = torch.randn(T, B, N + M, 64, device=DEV)
    alive = torch.ones(T, B, N + M, dtype=torch.bool, device=DEV)
    hidden0 = trunk.initial_hidden(B, N + M, torch.device(DEV))   # every token recurrent, as the reference's test sizes it
    step_y = _step_loop(trunk, xs, alive, hidden0)
    with torch.no_grad():
        seq_y, _ = trunk.sequence(xs, alive, hidden0)
    assert torch.allclose(step_y, seq_y, atol=1e-5), float((step_y - seq_y).abs().max())


def test_step_matches_sequence_across_an_episode_boundary():
    """With reset_hidden_for_envs after the done step on the rollout side and done_mask on the
    sequence side: state and conv buffer both restart."""
    B, N, M, T = 2, 3, 2, 8
    trunk = trunk_of(cfg(2, 2, 1))
    torch.manual_seed(11)
    xs = torch.randn(T, B, N + M, 64, device=DEV)
    alive = torch.ones(T, B, N + M, dtype=torch.bool, device=DEV)
    done = torch.zeros(T, B, dtype=torch.bool, device=DEV)
    done[3] = True
    hidden0 = trunk.initial_hidden(B, N + M, torch.device(DEV))
    step_y = _step_loop(trunk, xs, alive, hidden0, done, N + M)
    with torch.no_grad():
        seq_y, _ = trunk.sequence(xs, alive, hidden0, done)
    assert torch.allclose(step_y, seq_y, atol=1e-5), float((step_y - seq_y).abs().max())


# ------------------------------------------------------------------ TestNonRecurrentFieldPath


def test_field_sub_is_identity_initialised():
    trunk = trunk_of(cfg(2, 2, 2))
    for block in trunk.yemong_layers:
        assert len(block.field_sub) == len(block.temporal)
        for sub in block.field_sub:
            assert torch.equal(sub.weight, torch.eye(64, device=DEV))


def test_forward_nonrecurrent_matches_manual_composition():
    """The field path is the Griffin block with only the scan swapped out; the composition is built
    from the block's own sub-modules (GatedMLP.forward included)."""
    from boost_and_broadside_b200 import GriffinTemporalBlock

    D = 32
    torch.manual_seed(0)
    block = GriffinTemporalBlock(D).eval().to(DEV)
    sub = torch.nn.Linear(D, D, bias=False).to(DEV)
    torch.nn.init.eye_(sub.weight)
    x = torch.randn(2, 5, D, device=DEV)
    with torch.no_grad():
        got = block.forward_nonrecurrent(x, sub)
        normed = block.norm1(x)
        b1 = sub(block.linear1(normed))
        b2 = F.gelu(block.linear2(normed))
        x1 = x + block.linear_out(b1 * b2)
        want = x1 + block.gated_mlp(block.norm2(x1))
    assert torch.allclose(got, want, atol=1e-5), float((got - want).abs().max())


def _field_case(n_blocks):
    B, N, M = 2, 3, 2
    trunk = trunk_of(cfg(n_blocks, 2, 1))
    torch.manual_seed(5)
    x = torch.randn(B, N + M, 64, device=DEV)
    alive = torch.ones(B, N + M, dtype=torch.bool, device=DEV)
    zero = trunk.initial_hidden(B, N, torch.device(DEV))    # ships only carry state
    torch.manual_seed(3)
    big = torch.randn_like(zero) * 5.0
    with torch.no_grad():
        out_zero, _ = trunk.step(x, alive, zero)
        out_big, _ = trunk.step(x, alive, big)
    return N, out_zero, out_big


def test_single_block_field_tokens_ignore_recurrent_state():
    N, out_zero, out_big = _field_case(1)
    assert torch.allclose(out_zero[:, N:], out_big[:, N:], atol=1e-6), "field tokens moved with the recurrent state"
    assert not torch.allclose(out_zero[:, :N], out_big[:, :N], atol=1e-4), "ship tokens should depend on the state"


def test_later_blocks_relay_recurrent_state_into_fields():
    N, out_zero, out_big = _field_case(2)
    assert not torch.allclose(out_zero[:, N:], out_big[:, N:], atol=1e-4)


@pytest.mark.parametrize("n_temporal", [1, 2])
def test_step_matches_sequence_with_fields(n_temporal):
    B, N, M, T = 2, 3, 2, 5
    trunk = trunk_of(cfg(2, 2, n_temporal))
    torch.manual_seed(11)
    xs = torch.randn(T, B, N + M, 64, device=DEV)
    alive = torch.ones(T, B, N + M, dtype=torch.bool, device=DEV)
    hidden0 = trunk.initial_hidden(B, N, torch.device(DEV))
    step_y = _step_loop(trunk, xs, alive, hidden0)
    with torch.no_grad():
        seq_y, _ = trunk.sequence(xs, alive, hidden0)
    assert torch.allclose(step_y, seq_y, atol=1e-5), float((step_y - seq_y).abs().max())


def test_zero_field_profile_is_unaffected():
    B, N = 2, 4
    trunk = trunk_of(cfg(2, 2, 1))
    x = torch.randn(B, N, 64, device=DEV)
    hidden = trunk.initial_hidden(B, N, torch.device(DEV))
    with torch.no_grad():
        y, new_hidden = trunk.step(x, torch.ones(B, N, dtype=torch.bool, device=DEV), hidden)
    assert y.shape == (B, N, 64) and new_hidden.shape == hidden.shape
