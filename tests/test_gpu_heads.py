"""The policy's heads on the GPU against the reference's own modules (the copy under oracle/_ref):
``action_head``, ``value_head_local``, ``value_head_win`` and ``next_state_head`` of a stock
``YemongPolicy`` (models/yemong/policy.py:185-214), their ``state_dict`` loaded into this package's
``HeadMLP`` / ``NextStateHead``, on trunk-like inputs.

Tolerances: float32 max-abs <= 1e-4; bf16 autocast normalised max error <= 2e-2 and the output
dtype is bfloat16 as the reference's.
"""

from __future__ import annotations

import pytest
import torch

from oracle import ref_runner
from tests.helpers import assert_close, golden, stored_weights
from tests.test_gpu_reference_policy import build_policies

pytestmark = pytest.mark.gpu
needs_ref = pytest.mark.skipif(not ref_runner.available(), reason="oracle/_ref has not been built")
DEV = "cuda"


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
def test_heads_match_the_reference_fixture(mode):
    """tests/golden/policy_heads.npz: the four heads of a stock reference policy on CPU."""
    import boost_and_broadside_b200 as bnb

    g = golden("policy_heads")
    w = stored_weights(g)
    ctx = torch.autocast(DEV, dtype=torch.bfloat16) if mode == "bf16" else torch.autocast(DEV, enabled=False)
    for name in ("action_head", "value_head_local", "value_head_win", "next_state_head"):
        sd = {k[len(name) + 1:]: v for k, v in w.items() if k.startswith(name + ".")}
        head = bnb.HeadMLP(128, sd["3.weight"].shape[0])
        head.load_state_dict(sd, strict=True)
        with torch.no_grad(), ctx:
            y = head.to(DEV)(g["x"].to(DEV))
        assert y.dtype == (torch.bfloat16 if mode == "bf16" else torch.float32)
        assert_close(y, g[f"{name}_{mode}"], mode, name)


def heads_of(policy):
    import boost_and_broadside_b200 as bnb

    D = 128
    pairs = []
    for name in ("action_head", "value_head_local", "value_head_win"):
        ref = getattr(policy, name)
        mine = bnb.HeadMLP(D, ref[3].out_features).to(DEV)
        mine.load_state_dict(ref.state_dict(), strict=True)
        pairs.append((name, ref, mine))
    ref = policy.next_state_head
    mine = bnb.NextStateHead(D, ref.pred_dim).to(DEV)
    mine.load_state_dict(ref.state_dict(), strict=True)
    pairs.append(("next_state_head", ref, mine))
    return pairs


@needs_ref
@pytest.mark.parametrize("mode", ["fp32", "bf16"])
@pytest.mark.parametrize("shape", [(64, 8), (3, 5, 8), (1, 1), (4097,)])
def test_heads_match_the_reference_policy_heads(shape, mode):
    stock, _ = build_policies(8)
    g = torch.Generator().manual_seed(len(shape) * 7 + shape[0])
    x = (torch.randn(*shape, 128, generator=g) * 1.5).to(DEV)
    ctx = torch.autocast(DEV, dtype=torch.bfloat16) if mode == "bf16" else torch.autocast(DEV, enabled=False)
    report = []
    for name, ref, mine in heads_of(stock):
        with torch.no_grad(), ctx:
            r, m = ref(x), mine(x)
            if mode == "bf16":
                r16, m16 = ref(x.to(torch.bfloat16)), mine(x.to(torch.bfloat16))   # the trunk's bf16 output as input
        assert m.shape == r.shape and m.dtype == r.dtype, (name, m.shape, r.shape, m.dtype, r.dtype)
        if mode == "fp32":
            err = float((m - r).abs().max())
            assert err <= 1e-4, f"{name}: max-abs {err:.3e}"
        else:
            err = float((m.float() - r.float()).abs().max() / r.float().abs().max())
            assert err <= 2e-2, f"{name}: normalised {err:.3e}"
            e16 = float((m16.float() - r16.float()).abs().max() / r16.float().abs().max())
            assert m16.dtype == r16.dtype and e16 <= 2e-2, f"{name}: bf16 input, normalised {e16:.3e}"
        report.append(f"{name} {err:.2e}")
    print(f"heads {shape} {mode}: " + " ".join(report))


def test_head_reads_bfloat16_tokens_as_they_are():
    """Under autocast a head handed bfloat16 tokens (the trunk's output dtype there) stages them
    without a float32 copy (``BNB_BF16_IO``): bit-equal to the same values widened first; a width
    whose hidden layer the tiled kernel is not built for (192) falls back to the float32-reading call."""
    import boost_and_broadside_b200 as bnb

    torch.manual_seed(3)
    for d_model, out in ((128, 12), (64, 11), (96, 3)):
        head = bnb.HeadMLP(d_model, out).to(DEV)
        x16 = (torch.randn(1000, 7, d_model, device=DEV) * 0.7).to(torch.bfloat16)
        with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
            a, b = head(x16), head(x16.float())
        assert a.dtype == torch.bfloat16 and tuple(a.shape) == (1000, 7, out)
        assert torch.equal(a, b), d_model


def test_head_on_an_empty_batch_and_a_wrong_width():
    import boost_and_broadside_b200 as bnb

    head = bnb.HeadMLP(128, 12).to(DEV)
    with torch.no_grad():
        assert head(torch.empty(0, 8, 128, device=DEV)).shape == (0, 8, 12)
        with pytest.raises(RuntimeError, match="width 128"):
            head(torch.zeros(4, 64, device=DEV))
        with pytest.raises(RuntimeError):
            head(torch.zeros(4, 128))   # a CPU tensor: there is no CPU path


@needs_ref
@pytest.mark.parametrize("mode", ["fp32", "bf16"])
@pytest.mark.parametrize("B,N", [(64, 8), (5, 2), (3, 40), (2, 152)])
def test_team_pma_matches_the_reference(B, N, mode):
    """TeamPMA (policy.py:78-121) of a stock reference policy against this package's, same
    parameters: random teams (ids outside 0..1 included: they are clamped for the gather), dead
    ships, an environment with a whole team dead and one with everybody dead."""
    import boost_and_broadside_b200 as bnb

    stock, _ = build_policies(8)
    ref = stock.team_pma
    with torch.no_grad():   # away from the near-zero seeds of the default init
        ref.seeds.normal_(0.0, 0.5)
        ref.norm.weight.uniform_(0.5, 1.5)
    mine = bnb.TeamPMA(128, 4).to(DEV)
    mine.load_state_dict(ref.state_dict(), strict=True)
    g = torch.Generator().manual_seed(B * 31 + N)
    x = (torch.randn(B, N, 128, generator=g) * 1.5).to(DEV)
    team = torch.randint(0, 2, (B, N), generator=g)
    alive = torch.rand(B, N, generator=g) < 0.7
    alive[0] = team[0] == 0            # team 1 entirely dead in environment 0
    if B > 1:
        alive[1] = False               # nobody alive in environment 1
    team, alive = team.to(DEV), alive.to(DEV)
    ctx = torch.autocast(DEV, dtype=torch.bfloat16) if mode == "bf16" else torch.autocast(DEV, enabled=False)
    with torch.no_grad(), ctx:
        r, m = ref(x, team, alive), mine(x, team, alive)
        if mode == "bf16":
            r16, m16 = ref(x.to(torch.bfloat16), team, alive), mine(x.to(torch.bfloat16), team, alive)
    assert m.shape == r.shape and m.dtype == r.dtype
    assert torch.isfinite(m).all()
    if mode == "fp32":
        err = float((m - r).abs().max())
        assert err <= 1e-4, f"max-abs {err:.3e}"
    else:
        err = float((m.float() - r.float()).abs().max() / r.float().abs().max())
        assert err <= 2e-2, f"normalised {err:.3e}"
        assert m16.dtype == r16.dtype == torch.bfloat16
        e16 = float((m16.float() - r16.float()).abs().max() / r16.float().abs().max())
        assert e16 <= 2e-2, f"bf16 input, normalised {e16:.3e}"
    # rows of a team without a living ship are exactly zero, as in the reference
    rows = m[0][team[0] == 1]          # team 1 of environment 0 has no ship alive
    if rows.numel():
        assert float(rows.abs().max()) == 0.0
    print(f"team_pma B={B} N={N} {mode}: {err:.2e}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_action_distribution_matches_torch_categorical(dtype):
    """sample_action / evaluate_action against torch.distributions.Categorical over the three
    logit slices, which is what the reference's _sample_action / _evaluate_action build
    (policy.py:551-602): log-probability and entropy of given actions, and the empirical
    distribution of 200 000 draws per slice (total variation below 1e-2)."""
    import boost_and_broadside_b200 as bnb
    from torch.distributions import Categorical

    g = torch.Generator().manual_seed(3)
    logits = (torch.randn(4, 7, 12, generator=g) * 2.0).to(DEV).to(dtype)
    slices = ((0, 3), (3, 10), (10, 12))
    actions = torch.stack([torch.randint(0, hi - lo, (4, 7), generator=g) for lo, hi in slices], -1).to(DEV)
    dists = [Categorical(logits=logits[..., lo:hi]) for lo, hi in slices]
    ref_lp = sum(d.log_prob(actions[..., i]) for i, d in enumerate(dists))
    ref_ent = sum(d.entropy() for d in dists)
    with torch.no_grad():
        lp, ent = bnb.evaluate_action(logits, actions)
    assert lp.dtype == ref_lp.dtype and lp.shape == ref_lp.shape
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    scale = 1.0 if dtype == torch.float32 else float(ref_lp.float().abs().max())
    assert float((lp.float() - ref_lp.float()).abs().max()) <= tol * scale
    assert float((ent.float() - ref_ent.float()).abs().max()) <= tol * max(1.0, float(ref_ent.float().abs().max()))

    one = logits[0, 0].float().expand(200_000, 12).contiguous().to(dtype)
    with torch.no_grad():
        a, lp_s = bnb.sample_action(one, generator=torch.Generator(device=DEV).manual_seed(1))
    assert a.dtype == torch.int64 and tuple(a.shape) == (200_000, 3)
    for i, (lo, hi) in enumerate(slices):
        want = torch.softmax(one[0, lo:hi].float(), -1)
        got = torch.bincount(a[:, i], minlength=hi - lo).float() / a.shape[0]
        assert float((got - want).abs().sum()) / 2 <= 1e-2, (i, got.tolist(), want.tolist())
    # the log-probability returned with the draws is that of the drawn actions
    lp_again, _ = bnb.evaluate_action(one, a)
    assert torch.equal(lp_s, lp_again)
