"""Parity of the CUDA trunk, called through the C ABI, against the reference's golden
vectors and against the CPU oracle on seeded inputs.  Needs a B200; every test is
marked gpu."""

import pytest
import torch

from oracle import trunk_oracle as O
from tests.helpers import assert_close, autocast_for, build_trunk, golden, stored_weights, trunk_params

pytestmark = pytest.mark.gpu
MODES = ("fp32", "bf16")
DEV = "cuda"


def _to(t, dev=DEV):
    return None if t is None else t.to(dev)


# ------------------------------------------------------------------ golden vectors


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", ["spatial_d128_n8", "spatial_d128_n152", "spatial_d64_n5", "spatial_d32_n3", "spatial_d32h2_n40"])
def test_spatial_block_golden(name, mode):
    from boost_and_broadside_b200 import ModelConfig, TransformerBlock

    g = golden(name)
    D, H = (int(v) for v in g["dims"])
    torch.manual_seed(0)
    block = TransformerBlock(ModelConfig(D, H, 2)).eval()
    w = stored_weights(g)
    if w:
        block.load_state_dict(w)
    block = block.to(DEV)
    with torch.no_grad(), autocast_for(mode, DEV):
        y = block(_to(g["x"]), _to(g["alive"]))
        y_nomask = block(_to(g["x"]), None)
    assert_close(y, g["y_" + mode], mode, name)
    assert_close(y_nomask, g["y_nomask_" + mode], mode, name + " (no mask)")


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", ["temporal_d128_t1", "temporal_d128_t9", "temporal_d64_t6"])
def test_temporal_block_golden(name, mode):
    from boost_and_broadside_b200 import GriffinTemporalBlock

    g = golden(name)
    D = int(g["dims"][0])
    torch.manual_seed(0)
    tb = GriffinTemporalBlock(D).eval()
    sub = torch.nn.Linear(D, D, bias=False)
    w = stored_weights(g)
    if w:
        sub.weight.data.copy_(w.pop("__sub.weight"))
        tb.load_state_dict(w)
    else:
        tb.conv.bias.data.copy_(g["conv_bias"])
    tb, sub = tb.to(DEV), sub.to(DEV)
    with torch.no_grad(), autocast_for(mode, DEV):
        y, h, c = tb.forward_sequence(_to(g["x"]), _to(g["h0"]), _to(g["conv"]), None)
        yf = tb.forward_nonrecurrent(_to(g["x"]), sub)
    assert_close(y, g["y_" + mode], mode, name + " y")
    assert_close(h, g["h_" + mode], mode, name + " h")
    assert_close(c, g["c_" + mode], mode, name + " conv")
    assert_close(yf, g["yf_" + mode], mode, name + " field path")
    if "yd_" + mode in g:
        with torch.no_grad(), autocast_for(mode, DEV):
            y, h, c = tb.forward_sequence(_to(g["x"]), _to(g["h0"]), _to(g["conv"]), _to(g["done"]))
        assert_close(y, g["yd_" + mode], mode, name + " y (done)")
        assert_close(h, g["hd_" + mode], mode, name + " h (done)")
        assert_close(c, g["cd_" + mode], mode, name + " conv (done)")


STEP_CASES = ["trunk_step_d128_8s4f", "trunk_step_d128_8s0f", "trunk_step_d128_30s2f", "trunk_step_d64_3s2f",
              "trunk_step_d32_2s1f_b132"]
SEQ_CASES = ["trunk_seq_d128_t6_8s0f", "trunk_seq_d128_t5_4s2f", "trunk_seq_d64_t7_3s2f"]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", STEP_CASES)
def test_trunk_step_golden(name, mode):
    g = golden(name)
    trunk = build_trunk(g["dims"], g).to(DEV)
    with torch.no_grad(), autocast_for(mode, DEV):
        y, nh = trunk.step(_to(g["x"]), _to(g["alive"]), _to(g["hidden"]))
    assert_close(y, g["y_" + mode], mode, name + " y")
    assert_close(nh, g["hidden_" + mode], mode, name + " hidden")


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", SEQ_CASES)
def test_trunk_sequence_golden(name, mode):
    g = golden(name)
    trunk = build_trunk(g["dims"], g).to(DEV)
    with torch.no_grad(), autocast_for(mode, DEV):
        y, nh = trunk.sequence(_to(g["x"]), _to(g["alive"]), _to(g["hidden"]), _to(g["done"]))
        y2, nh2 = trunk.sequence(_to(g["x"]), _to(g["alive"]), _to(g["hidden"]), None)
    assert_close(y, g["y_" + mode], mode, name + " y")
    assert_close(nh, g["hidden_" + mode], mode, name + " hidden")
    assert_close(y2, g["y_nodone_" + mode], mode, name + " y (no done)")
    assert_close(nh2, g["hidden_nodone_" + mode], mode, name + " hidden (no done)")
    # the reference's own step loop with reset_hidden_for_envs gives the same outputs
    assert_close(y, g["y_steps_" + mode], mode, name + " vs reference step loop", scale=1.0)


@pytest.mark.parametrize("mode", MODES)
def test_block_api_matches_policy_loop(mode):
    """YemongBlock.step chained as models/yemong/policy.py:327-340 equals YemongTrunk.step."""
    from boost_and_broadside_b200 import CONV_KERNEL

    g = golden("trunk_step_d128_8s4f")
    trunk = build_trunk(g["dims"], g).to(DEV)
    x, alive, hidden = _to(g["x"]), _to(g["alive"]), _to(g["hidden"])
    B, NM, D = x.shape
    L, R, _ = hidden.shape
    n_rec = R // B
    with torch.no_grad(), autocast_for(mode, DEV):
        hs = hidden[:, :, :D]
        cs = hidden[:, :, D:].reshape(L, R, CONV_KERNEL - 1, D)
        new_h, new_c = [], []
        cur = x
        for i, layer in enumerate(trunk.yemong_layers):
            cur, h, cb = layer.step(cur, alive, hs[i : i + 1], cs[i : i + 1], n_rec, None, None)
            new_h.append(h)
            new_c.append(cb)
        nh = torch.cat([torch.cat(new_h), torch.cat(new_c).reshape(L, R, (CONV_KERNEL - 1) * D)], dim=-1)
    assert_close(cur, g["y_" + mode], mode, "block loop y")
    assert_close(nh, g["hidden_" + mode], mode, "block loop hidden")


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", SEQ_CASES)
def test_block_sequence_api_matches_policy_loop(name, mode):
    """YemongBlock.sequence (griffin.py:419-472) called directly and chained as
    models/yemong/policy.py:455-478 does -- slices of the packed hidden state, done mask, the
    recurrent-token count -- reproduces the reference's sequence output; its returned final states
    equal the trunk's."""
    from boost_and_broadside_b200 import CONV_KERNEL

    g = golden(name)
    trunk = build_trunk(g["dims"], g).to(DEV)
    x, alive, hidden, done = _to(g["x"]), _to(g["alive"]), _to(g["hidden"]), _to(g["done"])
    T, B, NM, D = x.shape
    L, R, _ = hidden.shape
    n_rec = R // B
    n_t = trunk.yemong_layers[0].n_temporal
    with torch.no_grad(), autocast_for(mode, DEV):
        hs = hidden[:, :, :D]
        cs = hidden[:, :, D:].reshape(L, R, CONV_KERNEL - 1, D)
        cur = x
        hs_out, cs_out = [], []
        for i, layer in enumerate(trunk.yemong_layers):
            sl = slice(i * n_t, (i + 1) * n_t)
            cur, h, cb = layer.sequence(cur, alive, hs[sl], cs[sl], done, n_rec, None, None)
            assert h.shape == (n_t, R, D) and cb.shape == (n_t, R, CONV_KERNEL - 1, D)
            hs_out.append(h)
            cs_out.append(cb)
        nh = torch.cat([torch.cat(hs_out), torch.cat(cs_out).reshape(L, R, (CONV_KERNEL - 1) * D)], dim=-1)
        y_trunk, nh_trunk = trunk.sequence(x, alive, hidden, done)
    assert_close(cur, g["y_" + mode], mode, name + " block loop y")
    assert_close(nh, g["hidden_" + mode], mode, name + " block loop hidden")
    assert torch.equal(cur, y_trunk) and torch.equal(nh, nh_trunk)


# ------------------------------------------------------------------ configurations vs the oracle


def _oracle_step(trunk, w, mode):
    return O.trunk_step(w.x, w.alive, w.hidden, trunk_params(trunk), trunk.n_heads, mode)


def _head_argmax(y_ref, y_new, tol):
    """Argmax over the power / turn / shoot logit slices (constants.py:46-48 of the reference)
    of one fixed random action head applied to both trunk outputs.  Returns (flips outside
    near-ties, near-tie rows)."""
    gen = torch.Generator().manual_seed(99)
    head = torch.randn(12, y_ref.shape[-1], generator=gen) / y_ref.shape[-1] ** 0.5
    lr = y_ref.reshape(-1, y_ref.shape[-1]) @ head.t()
    ln = y_new.reshape(-1, y_new.shape[-1]) @ head.t()
    flips = ties = 0
    for lo, hi in ((0, 3), (3, 10), (10, 12)):
        a, b = lr[:, lo:hi], ln[:, lo:hi]
        top2 = a.topk(2, dim=1).values
        near = (top2[:, 0] - top2[:, 1]) < tol
        diff = a.argmax(1) != b.argmax(1)
        flips += int((diff & ~near).sum())
        ties += int(near.sum())
    return flips, ties


def test_c1_spatial_block_fp32():
    """256 envs x 8 ships, float32, one spatial block at the rl profile's dims."""
    from boost_and_broadside_b200 import ModelConfig, TransformerBlock
    from boost_and_broadside_b200 import workloads as W

    w = W.c1()
    torch.manual_seed(0)
    block = TransformerBlock(ModelConfig(128, 4, 2)).eval()
    ref = O.spatial_block(w.x, w.alive, dict(block.state_dict()), 4, "fp32")
    with torch.no_grad():
        y = block.to(DEV)(w.x.to(DEV), w.alive.to(DEV))
    assert_close(y, ref, "fp32", "C1")
    flips, _ = _head_argmax(ref, y.cpu(), 1e-3)
    assert flips == 0


@pytest.mark.parametrize("mode", MODES)
def test_c2_rollout_step(mode):
    """Trunk step at 4v4 + 4 fields (reduced to 512 envs so the oracle finishes in seconds)."""
    from boost_and_broadside_b200 import workloads as W

    w = W.c2(n_envs=512)
    trunk = build_trunk([128, 4, 2, 2, 1, 1])
    ref_y, ref_h = _oracle_step(trunk, w, mode)
    trunk = trunk.to(DEV)
    with torch.no_grad(), autocast_for(mode, DEV):
        y, nh = trunk.step(w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV))
    assert_close(y, ref_y, mode, "C2 y")
    assert_close(nh, ref_h, mode, "C2 hidden")
    tol = 1e-3 if mode == "fp32" else 2e-2 * float(ref_y.abs().max())
    flips, ties = _head_argmax(ref_y, y.cpu(), tol)
    assert flips == 0, f"{flips} argmax flips outside {ties} near-tie rows"


@pytest.mark.parametrize("mode", MODES)
def test_c3_large_fleet(mode):
    """64 v 88 = 152 tokens per env with heavy key padding (32 envs)."""
    from boost_and_broadside_b200 import workloads as W

    w = W.c3(n_envs=32)
    trunk = build_trunk([128, 4, 2, 2, 1, 1])
    ref_y, ref_h = _oracle_step(trunk, w, mode)
    trunk = trunk.to(DEV)
    with torch.no_grad(), autocast_for(mode, DEV):
        y, nh = trunk.step(w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV))
    assert_close(y, ref_y, mode, "C3 y")
    assert_close(nh, ref_h, mode, "C3 hidden")


@pytest.mark.parametrize("mode", MODES)
def test_c4_sequence_forward(mode):
    """T = 32 with done flags, checked against the sequence oracle and the step loop."""
    from boost_and_broadside_b200 import workloads as W

    w = W.c4(n_envs=48, timesteps=32)
    trunk = build_trunk([128, 4, 2, 2, 1, 1])
    P = trunk_params(trunk)
    ref_y, ref_h = O.trunk_sequence(w.x, w.alive, w.hidden, w.done, P, 4, mode)
    loop_y, _ = O.trunk_sequence_by_steps(w.x, w.alive, w.hidden, w.done, P, 4, mode)
    trunk = trunk.to(DEV)
    with torch.no_grad(), autocast_for(mode, DEV):
        y, nh = trunk.sequence(w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV), w.done.to(DEV))
    assert_close(y, ref_y, mode, "C4 y")
    assert_close(nh, ref_h, mode, "C4 hidden")
    assert_close(y, loop_y, mode, "C4 y vs sequential step loop")


@pytest.mark.parametrize("mode", MODES)
def test_c5_ragged_fleets(mode):
    """Mixed fleet sizes 2..128 with 0-4 fields per env (192 envs)."""
    from boost_and_broadside_b200 import RaggedBatch
    from boost_and_broadside_b200 import workloads as W

    w = W.c5(n_envs=192)
    trunk = build_trunk([128, 4, 2, 2, 1, 1])
    ref_y, ref_h = O.trunk_step_ragged(w.x, w.alive, w.hidden, w.n_tokens.tolist(), w.n_ships.tolist(),
                                       trunk_params(trunk), 4, mode)
    trunk = trunk.to(DEV)
    with torch.no_grad(), autocast_for(mode, DEV):
        y, nh = trunk.step_ragged(w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV), RaggedBatch(w.n_tokens, w.n_ships))
    assert_close(y, ref_y, mode, "C5 y")
    assert_close(nh, ref_h, mode, "C5 hidden")


# ------------------------------------------------------------------ size-independent properties


def test_full_size_step_properties():
    """At the full 8192-env step: bit-identical repeat runs, independence of environments
    (a slice of the batch gives the same rows), finite outputs, and dead keys that carry no
    influence (changing a dead ship's token leaves every other token unchanged)."""
    from boost_and_broadside_b200 import workloads as W

    w = W.c2()
    trunk = build_trunk([128, 4, 2, 2, 1, 1]).to(DEV)
    x, alive, hidden = w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV)
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        y1, h1 = trunk.step(x, alive, hidden)
        y2, h2 = trunk.step(x, alive, hidden)
        assert torch.equal(y1, y2) and torch.equal(h1, h2)
        assert torch.isfinite(y1).all() and torch.isfinite(h1).all()
        lo, hi = 1000, 1640
        ys, hs = trunk.step(x[lo:hi], alive[lo:hi], hidden[:, lo * 8 : hi * 8])
        # 640 environments are 64 tiles: the one-CTA-per-SM variant of the kernel (four threads per
        # row) runs them, the full batch runs on the two-CTA variant, and the bits still agree
        assert torch.equal(ys, y1[lo:hi]) and torch.equal(hs, h1[:, lo * 8 : hi * 8])
        # perturb dead ships only
        dead = ~alive
        x2 = x.clone()
        x2[dead] += 3.0
        y3, _ = trunk.step(x2, alive, hidden)
        live_rows = alive
        assert torch.equal(y3[live_rows], y1[live_rows])


def test_step_equals_sequence_of_one():
    g = golden("trunk_step_d128_8s4f")
    trunk = build_trunk(g["dims"], g).to(DEV)
    x, alive, hidden = _to(g["x"]), _to(g["alive"]), _to(g["hidden"])
    with torch.no_grad():
        y1, h1 = trunk.step(x, alive, hidden)
        y2, h2 = trunk.sequence(x[None], alive[None], hidden, None)
    assert_close(y2[0], y1, "fp32", "T=1 sequence y", scale=0.1)
    assert_close(h2, h1, "fp32", "T=1 sequence hidden", scale=0.1)


def test_reset_folded_into_step_equals_reset_then_step():
    from boost_and_broadside_b200 import workloads as W

    w = W.c2(n_envs=64)
    trunk = build_trunk([128, 4, 2, 2, 1, 1]).to(DEV)
    x, alive, hidden = w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV)
    done = torch.rand(64, generator=torch.Generator().manual_seed(5)) < 0.3
    done = done.to(DEV)
    with torch.no_grad():
        cleared = trunk.reset_hidden_for_envs(hidden, done, 8)
        ref = hidden * (~done.repeat_interleave(8)).float()[None, :, None]
        assert torch.equal(cleared, ref)
        y1, h1 = trunk.step(x, alive, cleared)
        y2, h2 = trunk.step(x, alive, hidden, reset_env=done)
    assert torch.equal(y1, y2) and torch.equal(h1, h2)


# ------------------------------------------------------------------ edge cases


def test_edge_cases():
    from boost_and_broadside_b200 import ModelConfig, TransformerBlock

    torch.manual_seed(0)
    block = TransformerBlock(ModelConfig(128, 4, 2)).eval()
    P = dict(block.state_dict())
    block = block.to(DEV)
    gen = torch.Generator().manual_seed(11)
    with torch.no_grad():
        # empty batch
        y = block(torch.zeros(0, 8, 128, device=DEV), torch.zeros(0, 8, dtype=torch.bool, device=DEV))
        assert y.shape == (0, 8, 128)
        # a single token per environment, alive and dead
        x = torch.randn(5, 1, 128, generator=gen)
        alive = torch.tensor([[True], [False], [True], [False], [True]])
        assert_close(block(x.to(DEV), alive.to(DEV)), O.spatial_block(x, alive, P, 4, "fp32"), "fp32", "N=1")
        # every environment fully dead: finite, equals the uniform-mean rule
        x = torch.randn(3, 6, 128, generator=gen)
        alive = torch.zeros(3, 6, dtype=torch.bool)
        y = block(x.to(DEV), alive.to(DEV))
        assert torch.isfinite(y).all()
        assert_close(y, O.spatial_block(x, alive, P, 4, "fp32"), "fp32", "all dead")
        # non-contiguous input view
        xb = torch.randn(4, 8, 256, generator=gen).to(DEV)[:, :, :128]
        assert_close(block(xb, None), O.spatial_block(xb.cpu(), None, P, 4, "fp32"), "fp32", "strided x")


def test_errors_are_python_exceptions():
    from boost_and_broadside_b200 import ModelConfig, TransformerBlock, YemongTrunk

    block = TransformerBlock(ModelConfig(128, 4, 2), reads_bullets=True).to(DEV)
    x = torch.zeros(2, 3, 128, device=DEV)
    with pytest.raises(RuntimeError):
        block(x, None, torch.zeros(3, 5, 128, device=DEV), None)  # bullets of another batch size
    with pytest.raises(RuntimeError):
        block(x, None, torch.zeros(2, 5, 128, device=DEV), torch.ones(2, 4, dtype=torch.bool, device=DEV))
    with pytest.raises(RuntimeError):
        block(torch.zeros(2, 3, 64, device=DEV))
    with pytest.raises(RuntimeError):
        block(torch.zeros(2, 3, 128))  # CPU tensor: no CPU path
    with pytest.raises(ValueError):
        bad = TransformerBlock(ModelConfig(160, 5, 1)).to(DEV)  # d_model above the built maximum
        bad(torch.zeros(1, 2, 160, device=DEV))
    trunk = YemongTrunk(ModelConfig(128, 4, 2, 2, 1)).to(DEV)
    with pytest.raises(RuntimeError):
        trunk.step(x, None, torch.zeros(3, 6, 512, device=DEV))


# ------------------------------------------------------------------ bullet cross-attention


def _bullet_block(g, D, H):
    from boost_and_broadside_b200 import ModelConfig, TransformerBlock

    torch.manual_seed(0)
    block = TransformerBlock(ModelConfig(D, H, 2), reads_bullets=True).eval()
    w = stored_weights(g)
    if w:
        block.load_state_dict(w)
    else:
        block.norm_bullet.weight.data.copy_(g["norm_bullet"])
    return block.to(DEV)


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", ["bullets_spatial_d128_n12_nb80", "bullets_spatial_d32_n3_nb7"])
def test_spatial_block_with_bullets_golden(name, mode):
    """attention.py:149-166 against the reference's own outputs: with the active mask (one
    environment with nothing in flight, one with a full ring), without a mask, without bullets."""
    g = golden(name)
    D, H = (int(v) for v in g["dims"])
    block = _bullet_block(g, D, H)
    x, alive, bul, bm = _to(g["x"]), _to(g["alive"]), _to(g["bullets"]), _to(g["bullet_mask"])
    with torch.no_grad(), autocast_for(mode, DEV):
        y = block(x, alive, bul, bm)
        y_nomask = block(x, alive, bul, None)
        y_none = block(x, alive)
    assert_close(y, g["y_" + mode], mode, name)
    assert_close(y_nomask, g["y_nobmask_" + mode], mode, name + " (no bullet mask)")
    assert_close(y_none, g["y_nobullets_" + mode], mode, name + " (no bullets)")
    if mode == "fp32":  # one engine for both calls: the gated-off branch changes nothing, exactly
        assert torch.equal(y[1], y_none[1])
    else:               # bf16 may take different kernels with and without bullets
        assert_close(y[1], y_none[1], mode, name + " (nothing in flight)")


def test_inactive_bullets_do_not_influence_output():
    """tests/models/test_encoder.py:700-751 of the reference, at the sublayer: garbling the
    inactive slots changes nothing, garbling an active one does."""
    g = golden("bullets_spatial_d128_n12_nb80")
    block = _bullet_block(g, 128, 4)
    x, alive, bul, bm = _to(g["x"]), _to(g["alive"]), _to(g["bullets"]), _to(g["bullet_mask"])
    garbled = torch.where(bm[..., None], bul, torch.full_like(bul, 1.0e3))
    for mode in MODES:
        with torch.no_grad(), autocast_for(mode, DEV):
            assert torch.equal(block(x, alive, bul, bm), block(x, alive, garbled, bm))
            moved = bul.clone()
            moved[bm] += 1.0
            assert not torch.equal(block(x, alive, bul, bm), block(x, alive, moved, bm))


@pytest.mark.parametrize("mode", MODES)
def test_trunk_with_bullets_golden(mode):
    g = golden("bullets_trunk_step_d128_8s4f")
    trunk = build_trunk(g["dims"], g).to(DEV)
    with torch.no_grad(), autocast_for(mode, DEV):
        y, nh = trunk.step(_to(g["x"]), _to(g["alive"]), _to(g["hidden"]), bullets=_to(g["bullets"]),
                           bullet_mask=_to(g["bullet_mask"]))
    assert_close(y, g["y_" + mode], mode, "bullets step y")
    assert_close(nh, g["hidden_" + mode], mode, "bullets step hidden")
    g = golden("bullets_trunk_seq_d128_t4_4s2f")
    with torch.no_grad(), autocast_for(mode, DEV):
        y, nh = trunk.sequence(_to(g["x"]), _to(g["alive"]), _to(g["hidden"]), _to(g["done"]),
                               bullets=_to(g["bullets"]), bullet_mask=_to(g["bullet_mask"]))
    assert_close(y, g["y_" + mode], mode, "bullets sequence y")
    assert_close(nh, g["hidden_" + mode], mode, "bullets sequence hidden")


@pytest.mark.parametrize("mode", MODES)
def test_block_step_with_bullets_vs_oracle(mode):
    """YemongBlock.step with the reference's argument list (griffin.py:376-385), seeded inputs."""
    from boost_and_broadside_b200 import ModelConfig, YemongBlock

    torch.manual_seed(3)
    cfg = ModelConfig(128, 4, 1, 2, 1, n_bullet_cross_per_block=2)
    blk = YemongBlock(cfg).eval()
    P = {k: v.detach().float() for k, v in blk.state_dict().items()}
    B, N, M, NB = 37, 6, 3, 60
    gen = torch.Generator().manual_seed(11)
    x = torch.randn(B, N + M, 128, generator=gen)
    alive = torch.rand(B, N + M, generator=gen) < 0.8
    h = torch.randn(1, B * N, 128, generator=gen) * 0.5
    cb = torch.randn(1, B * N, 3, 128, generator=gen) * 0.5
    bul = torch.randn(B, NB, 128, generator=gen)
    bm = torch.rand(B, NB, generator=gen) < 0.3
    bm[0] = False
    ry, rh, rc = O.yemong_block_step(x, alive, h, cb, N, P, 4, mode, bul, bm)
    blk = blk.to(DEV)
    with torch.no_grad(), autocast_for(mode, DEV):
        y, nh, nc = blk.step(_to(x), _to(alive), _to(h), _to(cb), N, _to(bul), _to(bm))
    assert_close(y, ry, mode, "block step y")
    assert_close(nh, rh, mode, "block step h")
    assert_close(nc, rc, mode, "block step conv")


@pytest.mark.parametrize("mode", MODES)
def test_step_matches_sequence_with_bullets(mode):
    """tests/models/test_encoder.py:782-814 of the reference, at the trunk: one sequence forward
    with per-step bullets equals stepping with reset_hidden_for_envs after finished steps; the
    bullets add no recurrent state (770-780)."""
    g = golden("bullets_trunk_seq_d128_t4_4s2f")
    trunk = build_trunk(g["dims"], g).to(DEV)
    x, alive, hidden, done = _to(g["x"]), _to(g["alive"]), _to(g["hidden"]), _to(g["done"])
    T, B = x.shape[0], x.shape[1]
    NB = g["bullets"].shape[1]
    bul = _to(g["bullets"]).reshape(T, B, NB, -1)
    bm = _to(g["bullet_mask"]).reshape(T, B, NB)
    with torch.no_grad(), autocast_for(mode, DEV):
        y_seq, h_seq = trunk.sequence(x, alive, hidden, done, bullets=bul.reshape(T * B, NB, -1),
                                      bullet_mask=bm.reshape(T * B, NB))
        h = hidden
        ys = []
        for t in range(T):
            y, h = trunk.step(x[t], alive[t], h, bullets=bul[t], bullet_mask=bm[t])
            assert h.shape == hidden.shape
            ys.append(y)
            h = trunk.reset_hidden_for_envs(h, done[t], x.shape[2] - 2)
    assert_close(torch.stack(ys), y_seq, mode, "steps vs sequence with bullets", scale=1.0 if mode == "fp32" else 1.0)
    assert_close(y_seq, g["y_" + mode], mode, "sequence vs reference")


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("ships,fields,nb", [(2, 0, 4), (16, 3, 160), (8, 4, 1)])
def test_bullets_at_unseen_fleet_sizes(mode, ships, fields, nb):
    """tests/models/test_encoder.py:886-906: the same weights at other fleet and ring sizes."""
    from boost_and_broadside_b200 import workloads as W

    trunk = build_trunk([128, 4, 2, 2, 1, 1])
    P = trunk_params(trunk)
    w = W.c2(n_envs=9, seed=41, ships=ships, fields=fields)
    gen = torch.Generator().manual_seed(43)
    bul = torch.randn(9, nb, 128, generator=gen)
    bm = torch.rand(9, nb, generator=gen) < 0.5
    ref_y, ref_h = O.trunk_step(w.x, w.alive, w.hidden, P, 4, mode, bul, bm)
    trunk = trunk.to(DEV)
    with torch.no_grad(), autocast_for(mode, DEV):
        y, nh = trunk.step(_to(w.x), _to(w.alive), _to(w.hidden), bullets=_to(bul), bullet_mask=_to(bm))
    assert_close(y, ref_y, mode, "y")
    assert_close(nh, ref_h, mode, "hidden")


def test_single_sublayer_methods_refuse_inputs_that_require_grad():
    """Gradients flow through YemongBlock / YemongTrunk step and sequence (tests/test_gpu_gradients.py);
    the single-sublayer methods are forward-only and say so instead of dropping the gradient."""
    from boost_and_broadside_b200 import ModelConfig, TransformerBlock

    block = TransformerBlock(ModelConfig(128, 4, 1, 1, 1)).to(DEV)
    with pytest.raises(NotImplementedError):
        block(torch.randn(2, 3, 128, device=DEV, requires_grad=True))


@pytest.mark.parametrize("mode", MODES)
def test_long_sequence_does_not_drift(mode):
    """T = 100 timesteps with resets (three times the length of the recurrent-PPO minibatch): the
    in-kernel time walk stays within the parity tolerance against the oracle's sequential loop."""
    from boost_and_broadside_b200 import workloads as W

    trunk = build_trunk([128, 4, 2, 2, 1, 1])
    w = W.c4(n_envs=5, timesteps=100, seed=91)
    ref_y, ref_h = O.trunk_sequence(w.x, w.alive, w.hidden, w.done, trunk_params(trunk), 4, mode)
    trunk = trunk.to(DEV)
    with torch.no_grad(), autocast_for(mode, DEV):
        y, h = trunk.sequence(_to(w.x), _to(w.alive), _to(w.hidden), _to(w.done))
    assert_close(y, ref_y, mode, "T=100 y")
    assert_close(h, ref_h, mode, "T=100 hidden")
