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


def test_head_on_an_empty_batch_and_a_wrong_width():
    import boost_and_broadside_b200 as bnb

    head = bnb.HeadMLP(128, 12).to(DEV)
    with torch.no_grad():
        assert head(torch.empty(0, 8, 128, device=DEV)).shape == (0, 8, 12)
        with pytest.raises(RuntimeError, match="width 128"):
            head(torch.zeros(4, 64, device=DEV))
        with pytest.raises(RuntimeError):
            head(torch.zeros(4, 128))   # a CPU tensor: there is no CPU path
