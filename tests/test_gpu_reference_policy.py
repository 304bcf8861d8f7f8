"""The drop-in itself, on the GPU: the reference's own ``YemongPolicy`` (from the copy under
oracle/_ref, see oracle/make_ref.py) built twice from one seed -- stock, and with this package's
``YemongBlock`` in place of the reference's -- run from the encoded tokens to the heads exactly as
``get_action_and_value`` / ``evaluate_actions`` do (models/yemong/policy.py:315-371, 422-490), and
compared on logits, value, next-state prediction, new hidden state and the argmax of every logit
slice (power 0:3, turn 3:10, shoot 10:12; constants.py:46-48).

Tolerances: float32 max-abs <= 1e-4; bf16 autocast normalised max error <= 2e-2; argmax identical
outside rows whose reference top-2 gap is below the float tolerance (those are counted and
printed, not hidden).
"""

from __future__ import annotations

import sys

import pytest
import torch

from oracle import make_ref, ref_runner

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_runner.available(), reason="oracle/_ref has not been built")]

DEV = "cuda"
SLICES = ((0, 3), (3, 10), (10, 12))
CONV_KERNEL = 4


def build_policies(num_ships: int):
    sys.path.insert(0, make_ref.ref_path())
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
        return ref_policy.YemongPolicy(cfg, build_standard_coordinator(ships), num_value_components=11,
                                       num_ships=num_ships, team_pma_k=(0, 1),
                                       bullet_coordinator=build_bullet_coordinator(ships)).eval()

    stock = make()
    original = ref_policy.YemongBlock
    ref_policy.YemongBlock = bnb.YemongBlock
    try:
        swapped = make()
    finally:
        ref_policy.YemongBlock = original
    assert isinstance(swapped.yemong_layers[0], bnb.YemongBlock)
    assert not isinstance(stock.yemong_layers[0], bnb.YemongBlock)
    swapped.load_state_dict(stock.state_dict(), strict=True)
    return stock.to(DEV), swapped.to(DEV)


def step_from_tokens(policy, x, alive, hidden, team_id, bullets, bullet_mask):
    """policy.py:315-371 from the encoder's output on: trunk loop, hidden repack, heads."""
    B, NM, D = x.shape
    n_layers, n_temporal = hidden.shape[0], policy._n_temporal
    B_rec = hidden.shape[1]
    n_rec = B_rec // B
    rglru = hidden[:, :, :D]
    conv = hidden[:, :, D:].reshape(n_layers, B_rec, CONV_KERNEL - 1, D)
    new_h, new_cb = [], []
    for i, layer in enumerate(policy.yemong_layers):
        sl = slice(i * n_temporal, (i + 1) * n_temporal)
        x, h, cb = layer.step(x, alive, rglru[sl], conv[sl], n_rec, bullets, bullet_mask)
        new_h.append(h)
        new_cb.append(cb)
    new_hidden = torch.cat([torch.cat(new_h, 0), torch.cat(new_cb, 0).reshape(n_layers, B_rec, (CONV_KERNEL - 1) * D)], -1)
    N = policy._num_ships
    xs, al, tid = x[:, :N], alive[:, :N], team_id[:, :N]
    logits = policy.action_head(xs)
    pred = policy.next_state_head(xs)
    value = policy.value_head_local(xs)
    win = policy.value_head_win(policy.team_pma(xs, tid, al))
    value = value.clone()
    for i, k in enumerate(policy._team_pma_k):
        value[:, :, k] = win[:, :, i]
    return logits.float(), value.float(), pred.float(), new_hidden.float(), x.float()


def sequence_from_tokens(policy, x, alive, hidden, done, bullets, bullet_mask):
    """policy.py:422-490 from the encoder's output on: the sequence loop, then the action head."""
    T, B, NM, D = x.shape
    n_layers, n_temporal = hidden.shape[0], policy._n_temporal
    B_rec = hidden.shape[1]
    n_rec = B_rec // B
    rglru = hidden[:, :, :D]
    conv = hidden[:, :, D:].reshape(n_layers, B_rec, CONV_KERNEL - 1, D)
    for i, layer in enumerate(policy.yemong_layers):
        sl = slice(i * n_temporal, (i + 1) * n_temporal)
        x, _, _ = layer.sequence(x, alive, rglru[sl], conv[sl], done, n_rec, bullets, bullet_mask)
    N = policy._num_ships
    return policy.action_head(x[:, :, :N]).float(), x.float()


def inputs(B: int, n_ships: int, n_fields: int, nb: int, seed: int, T: int = 0):
    g = torch.Generator().manual_seed(seed)
    lead = (T, B) if T else (B,)
    x = torch.randn(*lead, n_ships + n_fields, 128, generator=g)
    alive = torch.rand(*lead, n_ships, generator=g) < 0.85
    alive[..., 0] = True
    alive[..., n_ships // 2] = True
    if n_fields:
        alive = torch.cat([alive, torch.ones(*lead, n_fields, dtype=torch.bool)], -1)
    hidden = torch.randn(2, B * n_ships, 512, generator=g) * 0.5
    team = torch.cat([torch.zeros(n_ships // 2), torch.ones(n_ships - n_ships // 2), torch.zeros(n_fields)]).long().expand(B, -1)
    E = T * B if T else B
    bullets = torch.randn(E, nb, 128, generator=g) if nb else None
    mask = (torch.rand(E, nb, generator=g) < 0.4) if nb else None
    if nb:
        mask[0] = False   # one environment with nothing in flight
    done = (torch.rand(T, B, generator=g) < 0.1) if T else None
    to = lambda t: None if t is None else t.to(DEV)
    return to(x), to(alive), to(hidden), to(team), to(bullets), to(mask), to(done)


def compare(name, got, ref, mode):
    if mode == "fp32":
        err = float((got - ref).abs().max())
        assert err <= 1e-4, f"{name}: max-abs {err:.3e} > 1e-4"
    else:
        err = float((got - ref).abs().max() / ref.abs().max())
        assert err <= 2e-2, f"{name}: normalised error {err:.3e} > 2e-2"
    return err


def argmax_report(got, ref, tol):
    """Flips of the per-slice argmax; a flip only counts where the reference's top-2 gap exceeds tol."""
    flips = near = 0
    for lo, hi in SLICES:
        g, r = got[..., lo:hi], ref[..., lo:hi]
        top2 = r.topk(2, dim=-1).values
        tie = (top2[..., 0] - top2[..., 1]) <= tol
        differ = g.argmax(-1) != r.argmax(-1)
        flips += int((differ & ~tie).sum())
        near += int(tie.sum())
    return flips, near


CASES = [(64, 2, 0, 0), (96, 8, 4, 0), (48, 8, 4, 80), (6, 152, 0, 0)]


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
@pytest.mark.parametrize("B,n_ships,n_fields,nb", CASES)
def test_reference_policy_step_through_swapped_blocks(B, n_ships, n_fields, nb, mode):
    stock, swapped = build_policies(n_ships)
    x, alive, hidden, team, bullets, mask, _ = inputs(B, n_ships, n_fields, nb, seed=B + n_ships)
    ctx = torch.autocast(DEV, dtype=torch.bfloat16) if mode == "bf16" else torch.autocast(DEV, enabled=False)
    with torch.no_grad(), ctx:
        ref = step_from_tokens(stock, x, alive, hidden, team, bullets, mask)
        got = step_from_tokens(swapped, x, alive, hidden, team, bullets, mask)
    errs = {n: compare(n, g, r, mode) for n, g, r in zip(("logits", "value", "pred_next", "hidden", "x"), got, ref)}
    logit_tol = 1e-4 if mode == "fp32" else 2e-2 * float(ref[0].abs().max())
    flips, near = argmax_report(got[0], ref[0], logit_tol)
    print(f"policy step B={B} N={n_ships}+{n_fields} nb={nb} {mode}: " +
          " ".join(f"{k} {v:.2e}" for k, v in errs.items()) + f"; argmax flips {flips}, near-tie rows {near} of {3 * B * n_ships}")
    assert flips == 0


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
def test_reference_policy_sequence_through_swapped_blocks(mode):
    stock, swapped = build_policies(8)
    x, alive, hidden, _, bullets, mask, done = inputs(12, 8, 4, 20, seed=5, T=7)
    ctx = torch.autocast(DEV, dtype=torch.bfloat16) if mode == "bf16" else torch.autocast(DEV, enabled=False)
    with torch.no_grad(), ctx:
        ref = sequence_from_tokens(stock, x, alive, hidden, done, bullets, mask)
        got = sequence_from_tokens(swapped, x, alive, hidden, done, bullets, mask)
    e_logits = compare("logits", got[0], ref[0], mode)
    e_x = compare("x", got[1], ref[1], mode)
    flips, near = argmax_report(got[0], ref[0], 1e-4 if mode == "fp32" else 2e-2 * float(ref[0].abs().max()))
    print(f"policy sequence T=7 {mode}: logits {e_logits:.2e} x {e_x:.2e}; argmax flips {flips}, near-tie rows {near}")
    assert flips == 0


@pytest.mark.parametrize("B,n_ships,n_fields", [(96, 8, 4), (40, 2, 0)])
def test_bfloat16_tokens_in_and_out_as_the_reference_under_cuda_autocast(B, n_ships, n_fields):
    """With the bfloat16 tokens its own encoder produces under torch.autocast("cuda", bfloat16), the
    reference's trunk returns bfloat16 (its residual adds stay in bf16).  This package takes the
    same tensor without a float32 copy, carries the residual in float32 inside the kernel and rounds
    once on the way out: bfloat16 out, the bits of the float32-token call rounded, and within the
    bf16 tolerance of the reference."""
    stock, swapped = build_policies(n_ships)
    x, alive, hidden, team, _, _, _ = inputs(B, n_ships, n_fields, 0, seed=3 * B)
    x16 = x.to(torch.bfloat16)
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        ref = step_from_tokens(stock, x16, alive, hidden, team, None, None)
        got = step_from_tokens(swapped, x16, alive, hidden, team, None, None)
        # the dtype contract itself, on the blocks
        rx, _, _ = stock.yemong_layers[0].step(x16, alive, hidden[:1, :, :128], hidden[:1, :, 128:].reshape(1, -1, 3, 128), n_ships)
        gx, gh, _ = swapped.yemong_layers[0].step(x16, alive, hidden[:1, :, :128], hidden[:1, :, 128:].reshape(1, -1, 3, 128), n_ships)
        fx, fh, _ = swapped.yemong_layers[0].step(x16.float(), alive, hidden[:1, :, :128], hidden[:1, :, 128:].reshape(1, -1, 3, 128), n_ships)
    assert rx.dtype == torch.bfloat16 and gx.dtype == torch.bfloat16 and fx.dtype == torch.float32
    assert torch.equal(gx, fx.to(torch.bfloat16)) and torch.equal(gh, fh)
    errs = {n: compare(n, g, r, "bf16") for n, g, r in zip(("logits", "value", "pred_next", "hidden", "x"), got, ref)}
    flips, near = argmax_report(got[0], ref[0], 2e-2 * float(ref[0].abs().max()))
    print(f"bf16 tokens B={B} N={n_ships}+{n_fields}: " + " ".join(f"{k} {v:.2e}" for k, v in errs.items()) +
          f"; argmax flips {flips}, near-tie rows {near}")
    assert flips == 0
