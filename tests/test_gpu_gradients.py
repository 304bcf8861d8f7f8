"""Backward through the trunk on the GPU (``bnb_trunk_sequence_bwd`` behind ``loss.backward()``):

* against the gradients the reference's own autograd produced (tests/golden/grad_trunk_seq_*.npz):
  d x, d hidden0, d bullets and every parameter gradient of <y, dy> + <final hidden, dhidden>
  through the sequence forward of models/yemong/policy.py:422-478;
* against the gradient oracle (torch autograd over oracle/trunk_oracle.py) on seeded cases the
  fixtures do not hold (larger batches, one-block trunks, a step);
* through the reference's own ``YemongPolicy`` with swapped blocks (oracle/_ref), heads and all;
* the reference's grad-checkpoint pin (tests/models/test_encoder.py:1316-1362) restated: this
  backward always recomputes, and it must give the gradients of the stored-activation autograd.

Tolerance: float32 forward and backward, normalised max error <= 1e-4 per tensor.  Under bf16
autocast the forward runs on the tensor-core kernels and the backward is still float32 of the
float32 function; against the reference's bf16 autograd the gate is 3e-2 normalised per tensor (measured about 1e-2).
"""

from __future__ import annotations

import pytest
import torch

from oracle import ref_runner
from oracle import trunk_oracle as O
from tests.helpers import build_trunk, golden, grad_fixture_compare, norm_err, trunk_params

pytestmark = pytest.mark.gpu
DEV = "cuda"
CASES = ["d128_t5_4s2f", "d128_t4_4s2f_nb12", "d64_t7_3s2f", "d128_t1_8s0f"]


def run_backward(trunk, g, mode):
    T, B, NM, D = g["x"].shape
    x = g["x"].to(DEV).requires_grad_(True)
    hidden = g["hidden"].to(DEV).requires_grad_(True)
    bullets = g["bullets"].to(DEV).requires_grad_(True) if "bullets" in g else None
    mask = g["bullet_mask"].to(DEV) if "bullet_mask" in g else None
    done = g["done"].to(DEV) if "done" in g else None
    ctx = torch.autocast(DEV, dtype=torch.bfloat16) if mode == "bf16" else torch.autocast(DEV, enabled=False)
    with ctx:
        y, nh = trunk.sequence(x, g["alive"].to(DEV), hidden, done, bullets=bullets, bullet_mask=mask)
    loss = (y.float() * g["dy"].to(DEV)).sum() + (nh.float() * g["dhidden"].to(DEV)).sum()
    loss.backward()
    named = {k: p.grad for k, p in trunk.named_parameters() if p.grad is not None}
    return x.grad, hidden.grad, None if bullets is None else bullets.grad, named


@pytest.fixture(params=["keep", "recompute"])
def grad_mode(request, monkeypatch):
    """Both ways a differentiated call can run: the training forward that keeps its activations
    (bnb_trunk_sequence_fwd_train), and the plain forward whose backward recomputes them."""
    monkeypatch.setenv("BNB_GRAD_MODE", request.param)
    return request.param


@pytest.mark.parametrize("tag", CASES)
def test_gradients_match_the_reference_autograd_fp32(tag, grad_mode):
    g = golden("grad_trunk_seq_" + tag)
    trunk = build_trunk(g["dims"]).to(DEV).train()
    dx, dh0, db, named = run_backward(trunk, g, "fp32")
    has_fields = int(g["dims"][7]) > 0
    if not has_fields:   # field_sub never runs without field tokens: no gradient, as in the reference
        for k in [k for k in g if k.startswith("g_fp32::") and "field_sub" in k or k.startswith("gsub_fp32::") and "field_sub" in k]:
            named.setdefault(k.split("::", 1)[1], torch.zeros(tuple(g[k].shape) if k.startswith("g_") else (int(g["dims"][0]),) * 2))
    if "bullets" not in g:   # the bullet branch's parameters likewise
        for k in list(g):
            if k.split("::")[0] in ("g_fp32", "gsub_fp32") and ("kv_bullet" in k or "norm_bullet" in k):
                name = k.split("::", 1)[1]
                D = int(g["dims"][0])
                named.setdefault(name, torch.zeros((2 * D, D) if "kv_bullet" in name else (D,)))
    worst = grad_fixture_compare(g, "fp32", dx, dh0, db, named, tol=1e-4)
    print(f"gradients {tag} fp32 ({grad_mode}): worst normalised error {worst[1]:.2e} ({worst[0]})")


@pytest.mark.parametrize("tag", CASES[:3])
def test_gradients_under_bf16_autocast_stay_near_the_reference_bf16_autograd(tag, grad_mode):
    g = golden("grad_trunk_seq_" + tag)
    trunk = build_trunk(g["dims"]).to(DEV).train()
    dx, dh0, db, named = run_backward(trunk, g, "bf16")
    D = int(g["dims"][0])
    for k in list(g):
        if k.split("::")[0] in ("g_bf16", "gsub_bf16"):
            name = k.split("::", 1)[1]
            if name not in named:
                named[name] = torch.zeros((2 * D, D) if "kv_bullet" in name else (D, D) if "field_sub" in name else (D,))
    assert dx.dtype == torch.float32
    worst = grad_fixture_compare(g, "bf16", dx, dh0, db, named, tol=3e-2)
    print(f"gradients {tag} bf16 forward ({grad_mode}): worst normalised error vs the reference's bf16 autograd {worst[1]:.2e} ({worst[0]})")


ORACLE_CASES = [
    # dims (D, H, blocks, spatial, temporal, cross, N, M), T, B, NB
    ([128, 4, 2, 2, 1, 1, 8, 4], 6, 40, 0),
    ([128, 4, 1, 1, 1, 1, 4, 2], 3, 9, 20),
    ([128, 4, 1, 2, 2, 0, 5, 0], 4, 7, 0),
    ([64, 4, 2, 1, 1, 0, 3, 3], 9, 5, 0),
    ([32, 4, 1, 1, 1, 0, 2, 1], 2, 3, 0),
    ([128, 4, 1, 1, 0, 0, 40, 0], 1, 6, 0),    # spatial sublayers only, a wide environment
    ([128, 4, 2, 2, 1, 1, 152, 0], 1, 2, 0),   # 152 keys per environment
]


@pytest.mark.parametrize("dims,T,B,NB", ORACLE_CASES)
def test_gradients_match_the_oracle_on_seeded_cases(dims, T, B, NB, grad_mode):
    D, H, _, _, nt, _, N, M = dims
    gen = torch.Generator().manual_seed(T * 100 + B)
    trunk = build_trunk(dims).to(DEV).train()
    with torch.no_grad():
        for p in trunk.parameters():   # away from the identity-like defaults (norm gains 1, field_sub eye)
            p.add_(0.05 * torch.randn(p.shape, generator=gen).to(DEV))
    L = trunk.n_hidden_layers
    x = torch.randn(T, B, N + M, D, generator=gen)
    alive = torch.rand(T, B, N + M, generator=gen) < 0.8
    alive[..., 0] = True
    alive[0, 0] = False
    hidden = torch.randn(L, B * N, 4 * D, generator=gen) * 0.5
    done = torch.rand(T, B, generator=gen) < 0.25
    bullets = torch.randn(T * B, NB, D, generator=gen) if NB else None
    mask = (torch.rand(T * B, NB, generator=gen) < 0.5) if NB else None
    if NB:
        mask[1] = False
    dy = torch.randn(T, B, N + M, D, generator=gen)
    dh = torch.randn(L, B * N, 4 * D, generator=gen)

    P = trunk_params(trunk.cpu())
    trunk.to(DEV)
    odx, odh, odb, ograds = O.trunk_sequence_grad(x, alive, hidden, done, P, H, dy, dh if L else None, bullets, mask)

    xg = x.to(DEV).requires_grad_(True)
    hg = hidden.to(DEV).requires_grad_(True)
    bg = bullets.to(DEV).requires_grad_(True) if NB else None
    y, nh = trunk.sequence(xg, alive.to(DEV), hg, done.to(DEV), bullets=bg, bullet_mask=None if mask is None else mask.to(DEV))
    loss = (y * dy.to(DEV)).sum()
    if L:
        loss = loss + (nh * dh.to(DEV)).sum()
    loss.backward()
    worst = ("", 0.0)

    def check(name, got, ref):
        nonlocal worst
        if ref.abs().max() == 0:
            assert got is None or float(got.abs().max()) == 0.0, name
            return
        e = norm_err(got.cpu(), ref)
        assert e <= 1e-4, f"{name}: normalised gradient error {e:.3e}"
        if e > worst[1]:
            worst = (name, e)

    check("dx", xg.grad, odx)
    if L:
        check("dhidden0", hg.grad, odh)
    if NB:
        check("dbullets", bg.grad, odb)
    n = 0
    for i, blk in enumerate(ograds):
        for k, ref in blk.items():
            p = dict(trunk.named_parameters())[f"yemong_layers.{i}.{k}"]
            check(f"yemong_layers.{i}.{k}", p.grad if p.grad is not None else torch.zeros_like(p), ref)
            n += 1
    assert n == len(list(trunk.parameters()))
    print(f"gradients vs oracle dims={dims} T={T} B={B} NB={NB}: worst {worst[1]:.2e} ({worst[0]})")


def test_step_backward_equals_the_one_step_sequence():
    dims = [128, 4, 2, 2, 1, 0, 6, 2]
    trunk = build_trunk(dims).to(DEV).train()
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(5, 8, 128, generator=gen).to(DEV)
    alive = (torch.rand(5, 8, generator=gen) < 0.8).to(DEV)
    hidden = (torch.randn(2, 30, 512, generator=gen) * 0.5).to(DEV)
    dy = torch.randn(5, 8, 128, generator=gen).to(DEV)
    outs = []
    for seq in (False, True):
        trunk.zero_grad()
        xg, hg = x.clone().requires_grad_(True), hidden.clone().requires_grad_(True)
        if seq:
            y, nh = trunk.sequence(xg[None], alive[None], hg)
            y = y[0]
        else:
            y, nh = trunk.step(xg, alive, hg)
        ((y * dy).sum() + nh.sum()).backward()
        outs.append((xg.grad.clone(), hg.grad.clone(), {k: p.grad.clone() for k, p in trunk.named_parameters() if p.grad is not None}))
    assert norm_err(outs[0][0], outs[1][0]) <= 1e-5 and norm_err(outs[0][1], outs[1][1]) <= 1e-5
    for k in outs[1][2]:
        assert norm_err(outs[0][2][k], outs[1][2][k]) <= 1e-5, k


def test_backward_of_unsupported_calls_raises_instead_of_dropping_gradients():
    from boost_and_broadside_b200 import RaggedBatch

    trunk = build_trunk([128, 4, 1, 1, 1, 0, 2, 0]).to(DEV).train()
    x = torch.randn(3, 2, 128, device=DEV, requires_grad=True)
    hidden = torch.zeros(1, 6, 512, device=DEV)
    y, _ = trunk.step(x, None, hidden, reset_env=torch.zeros(3, dtype=torch.bool, device=DEV))
    with pytest.raises(NotImplementedError, match="reset_env"):
        y.sum().backward()
    rb = RaggedBatch(torch.tensor([2, 2, 2]), torch.tensor([2, 2, 2]))
    y, _ = trunk.step_ragged(x.reshape(-1, 128), None, hidden, rb)
    with pytest.raises(NotImplementedError, match="ragged"):
        y.sum().backward()


@pytest.mark.skipif(not ref_runner.available(), reason="oracle/_ref has not been built")
@pytest.mark.parametrize("mode", ["fp32", "bf16"])
def test_reference_policy_backward_through_swapped_blocks(mode, grad_mode):
    """evaluate_actions' trunk loop and heads (policy.py:422-490) on the reference's own policy,
    stock and with this package's blocks, same loss, gradients of every parameter compared."""
    from tests.test_gpu_reference_policy import build_policies, inputs, sequence_from_tokens

    stock, swapped = build_policies(8)
    stock.train()
    swapped.train()
    x, alive, hidden, _, bullets, mask, done = inputs(6, 8, 4, 20, seed=9, T=5)
    gen = torch.Generator().manual_seed(1)
    grads = []
    for policy in (stock, swapped):
        policy.zero_grad()
        xg = x.clone().requires_grad_(True)
        ctx = torch.autocast(DEV, dtype=torch.bfloat16) if mode == "bf16" else torch.autocast(DEV, enabled=False)
        with ctx:
            logits, xo = sequence_from_tokens(policy, xg, alive, hidden, done, bullets, mask)
        if not grads:
            w_logits = torch.randn(logits.shape, generator=gen).to(DEV)
            w_x = torch.randn(xo.shape, generator=gen).to(DEV)
        ((logits * w_logits).sum() + (xo * w_x).sum()).backward()
        grads.append((xg.grad.float().clone(), {k: p.grad.float().clone() for k, p in policy.named_parameters() if p.grad is not None}))
    tol = 1e-4 if mode == "fp32" else 3e-2
    worst = ("dx", norm_err(grads[1][0], grads[0][0]))
    assert worst[1] <= tol, f"dx: {worst[1]:.3e}"
    checked = 0
    for k, ref in grads[0][1].items():
        if not k.startswith(("yemong_layers", "action_head")):
            continue
        got = grads[1][1].get(k)
        if got is None:
            assert float(ref.abs().max()) == 0.0, k
            continue
        e = norm_err(got, ref)
        assert e <= tol, f"{k}: normalised gradient error {e:.3e} > {tol:.0e}"
        checked += 1
        if e > worst[1]:
            worst = (k, e)
    assert checked > 40
    print(f"policy backward {mode}: {checked} parameter gradients, worst {worst[1]:.2e} ({worst[0]})")


def test_recompute_backward_matches_stored_activation_autograd():
    """The reference pins grad_checkpoint as a memory-only change (tests/models/test_encoder.py:
    1316-1362): identical gradients with and without recomputation.  This backward always
    recomputes; the stored-activation gradient here is torch autograd over the float32 restatement, compared on the parameter the reference's test checks and on d x."""
    dims = [128, 4, 2, 2, 1, 0, 8, 0]
    T, B = 4, 2
    trunk = build_trunk(dims).to(DEV).train()
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(T, B, 8, 128, generator=gen)
    hidden = torch.zeros(2, B * 8, 512)
    alive = torch.ones(T, B, 8, dtype=torch.bool)
    xg = x.to(DEV).requires_grad_(True)
    y, _ = trunk.sequence(xg, alive.to(DEV), hidden.to(DEV))
    y.sum().backward()
    g0 = trunk.yemong_layers[0].temporal[0].linear1.weight.grad.cpu()
    dx = xg.grad.cpu()
    P = trunk_params(trunk.cpu())
    odx, _, _, og = O.trunk_sequence_grad(x, alive, hidden, None, P, 4, torch.ones(T, B, 8, 128), None)
    assert norm_err(g0, og[0]["temporal.0.linear1.weight"]) <= 1e-4
    assert norm_err(dx, odx) <= 1e-4


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
@pytest.mark.parametrize("name", ["trunk_seq_d128_t6_8s0f", "trunk_seq_d128_t5_4s2f", "trunk_seq_d64_t7_3s2f",
                                  "bullets_trunk_seq_d128_t4_4s2f"])
def test_training_forward_matches_the_forward_fixtures(name, mode, monkeypatch):
    """The forward a differentiated call runs (bnb_trunk_sequence_fwd_train) against the same
    reference outputs the inference forward is held to: y and the final state."""
    from tests.helpers import assert_close

    monkeypatch.setenv("BNB_GRAD_MODE", "keep")
    g = golden(name)
    trunk = build_trunk(g["dims"], g).to(DEV).train()
    ctx = torch.autocast(DEV, dtype=torch.bfloat16) if mode == "bf16" else torch.autocast(DEV, enabled=False)
    bullets = g["bullets"].to(DEV) if "bullets" in g else None
    mask = g["bullet_mask"].to(DEV) if "bullet_mask" in g else None
    with ctx:
        y, nh = trunk.sequence(g["x"].to(DEV), g["alive"].to(DEV), g["hidden"].to(DEV), g["done"].to(DEV),
                               bullets=bullets, bullet_mask=mask)
    assert y.requires_grad
    assert_close(y, g["y_" + mode], mode, name + " y")
    assert_close(nh, g["hidden_" + mode], mode, name + " hidden")


def test_a_second_backward_through_kept_activations_is_refused(monkeypatch):
    monkeypatch.setenv("BNB_GRAD_MODE", "keep")
    trunk = build_trunk([128, 4, 1, 1, 1, 0, 2, 0]).to(DEV).train()
    x = torch.randn(2, 3, 2, 128, device=DEV, requires_grad=True)
    y, _ = trunk.sequence(x, None, torch.zeros(1, 6, 512, device=DEV))
    y.sum().backward(retain_graph=True)
    with pytest.raises(RuntimeError, match="consumed"):
        y.sum().backward()


def test_training_step_under_torch_compile(grad_mode):
    """The reference trains through torch.compile(policy) (train/rl/ppo.py:396-400): the sequence
    forward and its backward must trace as opaque operators (fullgraph) and give the eager gradients."""
    import torch._dynamo

    torch._dynamo.reset()
    dims = [128, 4, 2, 2, 1, 0, 6, 2]
    trunk = build_trunk(dims).to(DEV).train()
    gen = torch.Generator().manual_seed(8)
    x = torch.randn(4, 5, 8, 128, generator=gen).to(DEV)
    alive = (torch.rand(4, 5, 8, generator=gen) < 0.8).to(DEV)
    hidden = (torch.randn(2, 30, 512, generator=gen) * 0.5).to(DEV)
    done = (torch.rand(4, 5, generator=gen) < 0.2).to(DEV)
    dy = torch.randn(4, 5, 8, 128, generator=gen).to(DEV)

    def loss_fn(x, alive, hidden, done, dy):
        with torch.autocast(DEV, dtype=torch.bfloat16):
            y, _ = trunk.sequence(x, alive, hidden, done)
        return (y.float() * dy).sum()

    def grads(fn):
        trunk.zero_grad(set_to_none=True)
        xg = x.clone().requires_grad_(True)
        fn(xg, alive, hidden, done, dy).backward()
        return xg.grad.clone(), {k: p.grad.clone() for k, p in trunk.named_parameters() if p.grad is not None}

    gx0, gp0 = grads(loss_fn)
    compiled = torch.compile(loss_fn, fullgraph=True)
    for _ in range(2):
        gx1, gp1 = grads(compiled)
    assert norm_err(gx1, gx0) <= 1e-5
    assert gp0.keys() == gp1.keys()
    for k in gp0:
        assert norm_err(gp1[k], gp0[k]) <= 1e-4, k   # atomics: the last bits vary from run to run
    torch._dynamo.reset()


@pytest.mark.skipif(not ref_runner.available(), reason="oracle/_ref has not been built")
@pytest.mark.parametrize("checkpoint", [False, True])
@pytest.mark.parametrize("mode", ["fp32", "bf16"])
def test_reference_evaluate_actions_with_swapped_blocks(mode, grad_mode, checkpoint):
    """``YemongPolicy.evaluate_actions`` itself (policy.py:379-516), the call ppo.py:1974 differentiates:
    the reference's own policy, stock and with this package's blocks, on a (T, B, N+M) observation in
    the reference's container with bullets and done flags; the reference's own loss of its
    grad-checkpoint test (log-probability + value + next-state prediction, summed); outputs and the
    gradient of every parameter of the policy -- encoders and heads included, which stay the
    reference's modules and receive their gradient through this package's trunk backward."""
    from tests.test_gpu_encoders import _observation
    from tests.test_gpu_reference_policy import build_policies

    T, B, N, M, NB = 4, 5, 8, 4, 12
    stock, swapped = build_policies(N)
    stock.train()
    swapped.train()
    # the reference's grad_checkpoint switch (policy.py:451-467): torch.utils.checkpoint around each block
    stock._grad_checkpoint = swapped._grad_checkpoint = checkpoint
    flat = _observation(T * B, N, M, NB, seed=21)
    obs = type(flat)(data={k: v.reshape(T, B, *v.shape[1:]) for k, v in flat.data.items()},
                     bullets={k: v.reshape(T, B, *v.shape[1:]) for k, v in flat.bullets.items()})
    gen = torch.Generator().manual_seed(2)
    alive = obs["alive"].clone()
    alive[:, :, 2] = False
    actions = torch.stack([torch.randint(0, n, (T, B, N), generator=gen) for n in (3, 7, 2)], -1).to(DEV)
    done = (torch.rand(T, B, generator=gen) < 0.25).to(DEV)
    hidden = (torch.randn(2, B * N, 512, generator=gen) * 0.5).to(DEV)
    results = []
    for policy in (stock, swapped):
        policy.zero_grad()
        ctx = torch.autocast(DEV, dtype=torch.bfloat16) if mode == "bf16" else torch.autocast(DEV, enabled=False)
        with ctx:
            lp, ent, val, logits, _, pn = policy.evaluate_actions(obs, actions, hidden, alive, done)
        (lp.float().sum() + val.float().sum() + pn.float().sum() + 0.1 * ent.float().sum()).backward()
        results.append(((lp.float(), ent.float(), val.float(), logits.float(), pn.float()),
                        {k: p.grad.float().clone() for k, p in policy.named_parameters() if p.grad is not None}))
    tol = 1e-4 if mode == "fp32" else 3e-2
    for name, got, ref in zip(("logprob", "entropy", "value", "logits", "pred_next"), results[1][0], results[0][0]):
        assert norm_err(got, ref) <= tol, f"{name}: {norm_err(got, ref):.3e}"
    worst, checked = ("", 0.0), 0
    for k, ref in results[0][1].items():
        got = results[1][1].get(k)
        if got is None:
            assert float(ref.abs().max()) == 0.0, k
            continue
        if float(ref.abs().max()) == 0.0:
            assert float(got.abs().max()) == 0.0, k
            continue
        e = norm_err(got, ref)
        assert e <= tol, f"{k}: normalised gradient error {e:.3e} > {tol:.0e}"
        checked += 1
        if e > worst[1]:
            worst = (k, e)
    assert checked > 80
    print(f"evaluate_actions {mode} ({grad_mode}, checkpoint {checkpoint}): {checked} parameter gradients, worst {worst[1]:.2e} ({worst[0]})")


def test_aligned_shapes_take_the_unguarded_products_and_agree_with_the_guarded_ones():
    """With every matrix a whole number of 128 x 128 tiles and 32-wide slices (here 32 environments x
    8 ships x T = 4 = 1024 token rows, d_model 128) the bf16-mode products run without bounds tests.
    Environments are independent, so the token and state gradients of those 32 environments must be
    bit-identical when a 33rd environment is appended (1056 rows: the guarded kernels); and every
    parameter gradient stays within the bf16 gate of the float32-mode gradient."""
    dims = [128, 4, 2, 2, 1, 0, 8, 0]
    D, N, T = 128, 8, 4
    gen = torch.Generator().manual_seed(123)
    trunk = build_trunk(dims).to(DEV).train()
    with torch.no_grad():
        for p in trunk.parameters():
            p.add_(0.05 * torch.randn(p.shape, generator=gen).to(DEV))
    L = trunk.n_hidden_layers

    def make(B):
        g = torch.Generator().manual_seed(7)
        x = torch.randn(T, 33, N, D, generator=g)[:, :B].contiguous()
        alive = (torch.rand(T, 33, N, generator=g) < 0.8)[:, :B].contiguous()
        hidden = (torch.randn(L, 33, N, 4 * D, generator=g) * 0.5)[:, :B].reshape(L, B * N, 4 * D).contiguous()
        done = (torch.rand(T, 33, generator=g) < 0.25)[:, :B].contiguous()
        dy = torch.randn(T, 33, N, D, generator=g)[:, :B].contiguous()
        return [t.to(DEV) for t in (x, alive, hidden, done, dy)]

    def backward(B, bf16):
        x, alive, hidden, done, dy = make(B)
        trunk.zero_grad(set_to_none=True)
        xg, hg = x.requires_grad_(True), hidden.requires_grad_(True)
        ctx = torch.autocast(DEV, dtype=torch.bfloat16) if bf16 else torch.autocast(DEV, enabled=False)
        with ctx:
            y, nh = trunk.sequence(xg, alive, hg, done)
        ((y.float() * dy).sum() + nh.sum()).backward()
        return xg.grad, hg.grad.reshape(L, B, N, 4 * D), {k: p.grad.clone() for k, p in trunk.named_parameters() if p.grad is not None}

    dx32, dh32, g32 = backward(32, True)
    dx33, dh33, _ = backward(33, True)
    assert torch.equal(dx32, dx33[:, :32]) and torch.equal(dh32, dh33[:, :32])
    _, _, gref = backward(32, False)
    worst = max((norm_err(g32[k].cpu(), gref[k].cpu()), k) for k in gref if float(gref[k].abs().max()) > 0)
    print(f"aligned bf16 products vs float32-mode gradients: worst normalised error {worst[0]:.2e} ({worst[1]})")
    assert worst[0] <= 3e-2
