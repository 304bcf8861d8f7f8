"""The whole rollout step on this package's kernels: ``YemongPolicy.get_action_and_value``
(models/yemong/policy.py:291-373) with the reference's state_dict loaded, on the reference's own
observation container and FeatureCoordinators, against the stock reference policy (oracle/_ref) run
module by module on the same observation: value, next-state prediction, new hidden state, and the
log-probability of the actions this package drew, scored under the reference's logits.

Tolerances: float32 max-abs <= 1e-4; bf16 autocast normalised max error <= 2e-2.
"""

from __future__ import annotations

import pytest
import torch

from oracle import ref_runner
from tests.test_gpu_encoders import _observation
from tests.test_gpu_reference_policy import build_policies, step_from_tokens

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_runner.available(), reason="oracle/_ref has not been built")]
DEV = "cuda"


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
@pytest.mark.parametrize("B,N,M,NB", [(24, 8, 4, 80), (7, 2, 0, 6)])
def test_rollout_step_matches_the_reference_policy(B, N, M, NB, mode):
    import boost_and_broadside_b200 as bnb
    from torch.distributions import Categorical

    stock, _ = build_policies(N)
    with torch.no_grad():   # the default init leaves the win head and the seeds near zero
        stock.team_pma.seeds.normal_(0.0, 0.5)
        for p in stock.value_head_win.parameters():
            p.add_(0.05 * torch.randn_like(p))
    cfg = stock.yemong_layers[0]
    ref_cfg = bnb.ModelConfig(d_model=128, n_heads=4, n_yemong_blocks=2, n_spatial_per_block=2, n_temporal_per_block=1,
                              n_bullet_cross_per_block=1)
    mine = bnb.YemongPolicy(ref_cfg, stock.coordinator, num_value_components=11, num_ships=N, team_pma_k=(0, 1),
                            bullet_coordinator=stock.bullet_encoder.coordinator).to(DEV).eval()
    assert list(mine.state_dict()) == list(stock.state_dict())
    mine.load_state_dict(stock.state_dict(), strict=True)
    del cfg

    obs = _observation(B, N, M, NB, seed=B)
    obs["alive"][:, 1] = False
    hidden = torch.randn(mine.n_hidden_layers, B * N, 512, device=DEV) * 0.5
    ctx = torch.autocast(DEV, dtype=torch.bfloat16) if mode == "bf16" else torch.autocast(DEV, enabled=False)
    with torch.no_grad(), ctx:
        x = stock.encoder(obs)
        bullets, mask = stock._encode_bullets(obs)
        logits, value, pred, new_hidden, _ = step_from_tokens(stock, x, obs["alive"], hidden, obs["team_id"], bullets, mask)
        action, logprob, v, pn, nh = mine.get_action_and_value(obs, hidden, generator=torch.Generator(device=DEV).manual_seed(0))
    assert tuple(action.shape) == (B, N, 3) and action.dtype == torch.int64
    assert tuple(logprob.shape) == (B, N) and tuple(v.shape) == (B, N, 11)

    def err(got, ref):
        got, ref = got.float(), ref.float()
        return float((got - ref).abs().max()) if mode == "fp32" else float((got - ref).abs().max() / ref.abs().max())

    tol = 1e-4 if mode == "fp32" else 2e-2
    errs = {"value": err(v, value), "pred_next": err(pn, pred), "hidden": err(nh, new_hidden)}
    ref_lp = sum(Categorical(logits=logits[..., lo:hi]).log_prob(action[..., i]) for i, (lo, hi) in enumerate(((0, 3), (3, 10), (10, 12))))
    errs["logprob"] = err(logprob, ref_lp)
    print(f"rollout step B={B} N={N}+{M} NB={NB} {mode}: " + " ".join(f"{k} {e:.2e}" for k, e in errs.items()))
    for k, e in errs.items():
        assert e <= (tol if k != "logprob" or mode == "fp32" else 4e-2), f"{k}: {e:.3e}"
    assert 0 <= int(action[..., 0].max()) < 3 and 0 <= int(action[..., 1].max()) < 7 and 0 <= int(action[..., 2].max()) < 2


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
def test_evaluate_actions_forward_matches_the_reference_policy(mode):
    """``YemongPolicy.evaluate_actions`` (policy.py:379-516) without gradients, on a (T, B, N+M)
    observation with bullets and done flags, against the stock reference policy's own call."""
    import boost_and_broadside_b200 as bnb

    T, B, N, M, NB = 4, 6, 8, 4, 24
    stock, _ = build_policies(N)
    with torch.no_grad():
        stock.team_pma.seeds.normal_(0.0, 0.5)
        for p in stock.value_head_win.parameters():
            p.add_(0.05 * torch.randn_like(p))
    cfg = bnb.ModelConfig(d_model=128, n_heads=4, n_yemong_blocks=2, n_spatial_per_block=2, n_temporal_per_block=1,
                          n_bullet_cross_per_block=1)
    mine = bnb.YemongPolicy(cfg, stock.coordinator, num_value_components=11, num_ships=N, team_pma_k=(0, 1),
                            bullet_coordinator=stock.bullet_encoder.coordinator).to(DEV).eval()
    mine.load_state_dict(stock.state_dict(), strict=True)
    flat = _observation(T * B, N, M, NB, seed=77)
    obs = type(flat)(data={k: v.reshape(T, B, *v.shape[1:]) for k, v in flat.data.items()},
                     bullets={k: v.reshape(T, B, *v.shape[1:]) for k, v in flat.bullets.items()})
    gen = torch.Generator().manual_seed(5)
    alive = obs["alive"].clone()
    alive[:, :, 3] = False
    actions = torch.stack([torch.randint(0, n, (T, B, N), generator=gen) for n in (3, 7, 2)], -1).to(DEV)
    done = (torch.rand(T, B, generator=gen) < 0.25).to(DEV)
    hidden = (torch.randn(2, B * N, 512, generator=gen) * 0.5).to(DEV)
    ctx = torch.autocast(DEV, dtype=torch.bfloat16) if mode == "bf16" else torch.autocast(DEV, enabled=False)
    with torch.no_grad(), ctx:
        ref = stock.evaluate_actions(obs, actions, hidden, alive, done, return_encoder_output=True)
        got = mine.evaluate_actions(obs, actions, hidden, alive, done, return_encoder_output=True)
    names = ("logprob", "entropy", "value", "logits", "encoder output", "pred_next")
    tol = 1e-4 if mode == "fp32" else 3e-2
    report = []
    for name, g, r in zip(names, got, ref):
        assert g.shape == r.shape, (name, g.shape, r.shape)
        g, r = g.float(), r.float()
        e = float((g - r).abs().max()) if mode == "fp32" else float((g - r).abs().max() / r.abs().max())
        assert e <= tol, f"{name}: {e:.3e}"
        report.append(f"{name} {e:.1e}")
    print(f"evaluate_actions forward {mode}: " + " ".join(report))


def test_rollout_step_under_torch_compile_is_one_graph_and_matches_eager():
    """``torch.compile(policy.get_action_and_value, mode="reduce-overhead", fullgraph=True)`` -- the
    reference's own way of running its policy (train/rl/ppo.py:396-400): every call into the C ABI is
    an opaque operator, so there is no graph break, and value / prediction / hidden state equal the
    eager call bit for bit (the action draw uses the device generator and is only checked for range)."""
    import boost_and_broadside_b200 as bnb

    B, N, M, NB = 16, 8, 4, 24
    stock, _ = build_policies(N)
    cfg = bnb.ModelConfig(d_model=128, n_heads=4, n_yemong_blocks=2, n_spatial_per_block=2, n_temporal_per_block=1,
                          n_bullet_cross_per_block=1)
    mine = bnb.YemongPolicy(cfg, stock.coordinator, num_value_components=11, num_ships=N, team_pma_k=(0, 1),
                            bullet_coordinator=stock.bullet_encoder.coordinator).to(DEV).eval()
    mine.load_state_dict(stock.state_dict(), strict=True)
    obs = _observation(B, N, M, NB, seed=11)
    hidden = torch.randn(mine.n_hidden_layers, B * N, 512, device=DEV) * 0.5
    compiled = torch.compile(mine.get_action_and_value, mode="reduce-overhead", fullgraph=True)
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        _, _, v0, p0, h0 = mine.get_action_and_value(obs, hidden)
        for _ in range(3):   # warm-up, capture, replay
            a, lp, v, p, h = compiled(obs, hidden)
            v, p, h, a, lp = v.clone(), p.clone(), h.clone(), a.clone(), lp.clone()
    assert torch.equal(v, v0) and torch.equal(p, p0) and torch.equal(h, h0)
    assert tuple(a.shape) == (B, N, 3) and 0 <= int(a[..., 1].min()) and int(a[..., 1].max()) < 7
    assert bool(torch.isfinite(lp.float()).all())
