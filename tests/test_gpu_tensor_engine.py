"""The tensor-core (tcgen05) engine against the CPU oracle and against the SIMT engine on
the same inputs, called through the C ABI with the engine chosen explicitly."""

import warnings

import pytest
import torch

from oracle import trunk_oracle as O
from tests.helpers import assert_close, build_trunk, golden, norm_err, trunk_params

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _engines():
    from boost_and_broadside_b200 import _capi

    return _capi, _capi.ENGINE_SIMT, _capi.ENGINE_TENSOR


def _status_ok():
    from boost_and_broadside_b200 import _capi

    st = _capi.tensor_engine_status(torch.device("cuda", torch.cuda.current_device()))
    assert st == 0, f"tensor engine status word {st}: a bounded wait ran out"


@pytest.mark.parametrize("n_envs,ships,fields", [(10, 8, 4), (23, 8, 4), (16, 8, 0), (7, 30, 2), (3, 1, 0), (5, 2, 3), (2, 64, 0), (1, 128, 0)])
def test_step_tensor_vs_oracle_and_simt(n_envs, ships, fields):
    from boost_and_broadside_b200 import workloads as W

    _capi, SIMT, TENSOR = _engines()
    w = W.c2(n_envs=n_envs, seed=21, ships=ships, fields=fields)
    trunk = build_trunk([128, 4, 2, 2, 1, 1])
    ref_y, ref_h = O.trunk_step(w.x, w.alive, w.hidden, trunk_params(trunk), 4, "bf16")
    trunk = trunk.to(DEV)
    x, alive, hidden = w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV)
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        ys, hs = trunk.step(x, alive, hidden, engine=SIMT)
        yt, ht = trunk.step(x, alive, hidden, engine=TENSOR)
    _status_ok()
    assert_close(yt, ref_y, "bf16", "tensor y vs oracle")
    assert_close(ht, ref_h, "bf16", "tensor hidden vs oracle")
    assert norm_err(yt.cpu(), ys.cpu()) < 1e-2
    assert norm_err(ht.cpu(), hs.cpu()) < 1e-2


def test_single_spatial_and_temporal_sublayers():
    """One sublayer at a time through bnb_spatial_block_fwd / bnb_temporal_block_fwd."""
    from boost_and_broadside_b200 import GriffinTemporalBlock, ModelConfig, TransformerBlock

    gen = torch.Generator().manual_seed(3)
    torch.manual_seed(0)
    block = TransformerBlock(ModelConfig(128, 4, 2)).eval()
    P = dict(block.state_dict())
    x = torch.randn(21, 12, 128, generator=gen)
    alive = torch.rand(21, 12, generator=gen) < 0.8
    alive[3] = False
    ref = O.spatial_block(x, alive, P, 4, "bf16")
    block = block.to(DEV)
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        y = block(x.to(DEV), alive.to(DEV))
    _status_ok()
    assert_close(y, ref, "bf16", "spatial sublayer")

    torch.manual_seed(0)
    tb = GriffinTemporalBlock(128).eval()
    sub = torch.nn.Linear(128, 128, bias=False)
    P = dict(tb.state_dict())
    xs = torch.randn(150, 5, 128, generator=gen)
    h0 = torch.randn(150, 128, generator=gen) * 0.5
    cb = torch.randn(150, 3, 128, generator=gen) * 0.5
    done = torch.rand(150, 5, generator=gen) < 0.3
    ref_y, ref_h, ref_c = O.temporal_sequence(xs, h0, cb, done, P, "bf16")
    ref_f = O.temporal_nonrecurrent(xs, P, sub.weight.detach(), "bf16")
    tb, sub = tb.to(DEV), sub.to(DEV)
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        y, h, c = tb.forward_sequence(xs.to(DEV), h0.to(DEV), cb.to(DEV), done.to(DEV))
        _status_ok()
        yf = tb.forward_nonrecurrent(xs.to(DEV), sub)
        _status_ok()
    assert_close(y, ref_y, "bf16", "temporal y")
    assert_close(h, ref_h, "bf16", "temporal h")
    assert_close(c, ref_c, "bf16", "temporal conv")
    assert_close(yf, ref_f, "bf16", "field path")


def test_sequence_tensor_vs_oracle():
    from boost_and_broadside_b200 import workloads as W

    _capi, SIMT, TENSOR = _engines()
    w = W.c4(n_envs=37, timesteps=9, seed=31)
    trunk = build_trunk([128, 4, 2, 2, 1, 1])
    ref_y, ref_h = O.trunk_sequence(w.x, w.alive, w.hidden, w.done, trunk_params(trunk), 4, "bf16")
    trunk = trunk.to(DEV)
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        y, nh = trunk.sequence(w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV), w.done.to(DEV), engine=TENSOR)
    _status_ok()
    assert_close(y, ref_y, "bf16", "sequence y")
    assert_close(nh, ref_h, "bf16", "sequence hidden")


def test_weights_are_repacked_after_an_update():
    """The packed image is derived data: an in-place parameter update must be picked up."""
    from boost_and_broadside_b200 import workloads as W

    _capi, SIMT, TENSOR = _engines()
    w = W.c2(n_envs=20, seed=41)
    trunk = build_trunk([128, 4, 2, 2, 1, 1]).to(DEV)
    x, alive, hidden = w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV)
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        y0, _ = trunk.step(x, alive, hidden, engine=TENSOR)
        for p in trunk.parameters():
            p.mul_(1.05)
        y1, _ = trunk.step(x, alive, hidden, engine=TENSOR)
        ys, _ = trunk.step(x, alive, hidden, engine=SIMT)
    assert norm_err(y1.cpu(), y0.cpu()) > 1e-3
    assert norm_err(y1.cpu(), ys.cpu()) < 1e-2


@pytest.mark.parametrize("n_envs,teams", [(3, (64, 88)), (2, (100, 100)), (1, (65, 64)), (2, (250, 262))])
def test_large_environments_split_attention_path(n_envs, teams):
    """Environments larger than one 128-row tile: q|k|v through scratch and a separate
    attention kernel with a running-maximum softmax over key blocks."""
    from boost_and_broadside_b200 import workloads as W

    _capi, SIMT, TENSOR = _engines()
    w = W.c3(n_envs=n_envs, seed=51, teams=teams)
    trunk = build_trunk([128, 4, 2, 2, 1, 1])
    ref_y, ref_h = O.trunk_step(w.x, w.alive, w.hidden, trunk_params(trunk), 4, "bf16")
    trunk = trunk.to(DEV)
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        y, nh = trunk.step(w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV), engine=TENSOR)
    _status_ok()
    assert_close(y, ref_y, "bf16", "large env y")
    assert_close(nh, ref_h, "bf16", "large env hidden")


def test_large_environment_sequence_and_all_dead():
    from boost_and_broadside_b200 import workloads as W

    _capi, SIMT, TENSOR = _engines()
    gen = torch.Generator().manual_seed(61)
    T, B, N = 3, 2, 152
    x = torch.randn(T, B, N, 128, generator=gen)
    alive = torch.rand(T, B, N, generator=gen) < 0.6
    alive[1, 0] = False  # an environment without a live key at one timestep
    hidden = torch.randn(2, B * N, 512, generator=gen) * 0.5
    done = torch.rand(T, B, generator=gen) < 0.4
    trunk = build_trunk([128, 4, 2, 2, 1, 1])
    ref_y, ref_h = O.trunk_sequence(x, alive, hidden, done, trunk_params(trunk), 4, "bf16")
    trunk = trunk.to(DEV)
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        y, nh = trunk.sequence(x.to(DEV), alive.to(DEV), hidden.to(DEV), done.to(DEV), engine=TENSOR)
    _status_ok()
    assert_close(y, ref_y, "bf16", "large env sequence y")
    assert_close(nh, ref_h, "bf16", "large env sequence hidden")


def test_tensor_engine_refuses_what_it_is_not_built_for():
    _capi, SIMT, TENSOR = _engines()
    gen = torch.Generator().manual_seed(71)
    x = torch.randn(1, 600, 128, generator=gen).to(DEV)   # more tokens per environment than the split path stages
    hidden = torch.zeros(2, 600, 512, device=DEV)
    trunk = build_trunk([128, 4, 2, 2, 1, 1]).to(DEV)
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        with pytest.raises(ValueError):
            trunk.step(x, None, hidden, engine=TENSOR)
        y, _ = trunk.step(x, None, hidden)  # AUTO falls back to SIMT
    assert torch.isfinite(y).all()


def test_step_can_be_replayed_from_a_cuda_graph():
    """The reference's default launch mode wraps the policy in CUDA graphs
    (torch.compile(mode="reduce-overhead"), cli.py:204-211): a trunk step must be capturable
    after one warm-up call (no synchronisation, no allocation outside torch's allocator)."""
    from boost_and_broadside_b200 import workloads as W

    w = W.c2(n_envs=64, seed=81)
    trunk = build_trunk([128, 4, 2, 2, 1, 1]).to(DEV)
    x, alive, hidden = w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV)
    side = torch.cuda.Stream()
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        y_ref, h_ref = trunk.step(x, alive, hidden)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            trunk.step(x, alive, hidden)  # warm-up on the capture stream: scratch, kernel attributes
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            y_g, h_g = trunk.step(x, alive, hidden)
        x.add_(0.25)                      # new input in the captured buffer
        y_new, h_new = trunk.step(x, alive, hidden)
        g.replay()
        torch.cuda.synchronize()
    assert not torch.equal(y_new, y_ref)
    assert torch.equal(y_g, y_new) and torch.equal(h_g, h_new)


@pytest.mark.parametrize("name", ["C3", "C4", "C5"])
def test_full_size_configurations_tensor_vs_simt(name):
    """At the full sizes of the large-fleet, sequence and ragged configurations the CPU oracle
    is too slow, so the tensor-core engine is checked against the CUDA-core engine (itself
    checked against the oracle at reduced sizes) on every output element, plus finiteness."""
    from boost_and_broadside_b200 import RaggedBatch
    from boost_and_broadside_b200 import workloads as W

    _capi, SIMT, TENSOR = _engines()
    trunk = build_trunk([128, 4, 2, 2, 1, 1]).to(DEV)
    if name == "C3":
        w = W.c3()
        run = lambda eng: trunk.step(w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV), engine=eng)
    elif name == "C4":
        w = W.c4(n_envs=2048)  # half the environments: 2 x 268 MB of activations per engine
        run = lambda eng: trunk.sequence(w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV), w.done.to(DEV), engine=eng)
    else:
        w = W.c5()
        rb = RaggedBatch(w.n_tokens, w.n_ships)
        run = lambda eng: trunk.step_ragged(w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV), rb, engine=eng)
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        yt, ht = run(TENSOR)
        _status_ok()
        ys, hs = run(SIMT)
    assert torch.isfinite(yt).all() and torch.isfinite(ht).all()
    ey = float((yt - ys).abs().max()) / float(ys.abs().max())
    eh = float((ht - hs).abs().max()) / float(hs.abs().max())
    assert ey < 2e-2 and eh < 2e-2, (ey, eh)


# ------------------------------------------------------------------ bullet cross-attention


def _bullets(n_envs, nb, seed, p_active=0.4):
    gen = torch.Generator().manual_seed(seed)
    bul = torch.randn(n_envs, nb, 128, generator=gen)
    mask = torch.rand(n_envs, nb, generator=gen) < p_active
    mask[0] = False                    # nothing in flight
    if n_envs > 1:
        mask[1] = True                 # full ring buffer
    return bul, mask


@pytest.mark.parametrize("n_envs,ships,fields,nb", [(10, 8, 4, 80), (37, 8, 0, 33), (5, 30, 2, 300), (3, 1, 0, 1), (2, 100, 52, 80)])
def test_step_with_bullets_tensor_vs_oracle_and_simt(n_envs, ships, fields, nb):
    """Bullet-reading sublayers on the tensor engine: the bullet key/value projection as a tile
    program over bullet rows, then one attention kernel for both softmaxes; environments of up
    to one tile and larger ones (152 tokens)."""
    from boost_and_broadside_b200 import workloads as W

    _capi, SIMT, TENSOR = _engines()
    w = W.c2(n_envs=n_envs, seed=23, ships=ships, fields=fields)
    bul, mask = _bullets(n_envs, nb, 5)
    trunk = build_trunk([128, 4, 2, 2, 1, 1])
    ref_y, ref_h = O.trunk_step(w.x, w.alive, w.hidden, trunk_params(trunk), 4, "bf16", bul, mask)
    ref_y0, _ = O.trunk_step(w.x, w.alive, w.hidden, trunk_params(trunk), 4, "bf16")
    assert norm_err(ref_y, ref_y0) > 1e-2          # the bullets matter in this case
    trunk = trunk.to(DEV)
    x, alive, hidden, bul_d, mask_d = (t.to(DEV) for t in (w.x, w.alive, w.hidden, bul, mask))
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        ys, hs = trunk.step(x, alive, hidden, engine=SIMT, bullets=bul_d, bullet_mask=mask_d)
        yt, ht = trunk.step(x, alive, hidden, engine=TENSOR, bullets=bul_d, bullet_mask=mask_d)
        yn, _ = trunk.step(x, alive, hidden, engine=TENSOR, bullets=bul_d, bullet_mask=None)
    _status_ok()
    assert_close(yt, ref_y, "bf16", "tensor y vs oracle")
    assert_close(ht, ref_h, "bf16", "tensor hidden vs oracle")
    assert norm_err(yt.cpu(), ys.cpu()) < 1e-2
    assert norm_err(ht.cpu(), hs.cpu()) < 1e-2
    ref_n, _ = O.trunk_step(w.x, w.alive, w.hidden, trunk_params(trunk.cpu()), 4, "bf16", bul, None)
    assert_close(yn, ref_n, "bf16", "tensor y vs oracle, no bullet mask")


@pytest.mark.parametrize("n_envs,ships,fields,nb,masked", [(40, 8, 4, 80, True), (6, 100, 52, 33, True), (9, 8, 4, 17, False)])
def test_bfloat16_bullet_tokens_equal_their_float32_copy(n_envs, ships, fields, nb, masked):
    """Bullet tokens handed over as bfloat16 (what the reference's BulletEncoder returns under CUDA
    autocast; ``BnbBullets.tokens_bf16``) are read by the key/value tile program as they are: the
    result is bit-identical to the call with the same values widened to float32 first, for
    environments of one tile and larger ones, with and without a mask, step and sequence."""
    from boost_and_broadside_b200 import workloads as W

    _capi, SIMT, TENSOR = _engines()
    w = W.c2(n_envs=n_envs, seed=31, ships=ships, fields=fields)
    bul, mask = _bullets(n_envs, nb, 9)
    trunk = build_trunk([128, 4, 2, 2, 1, 1]).to(DEV)
    x, alive, hidden = (t.to(DEV) for t in (w.x, w.alive, w.hidden))
    bul16 = bul.to(DEV).to(torch.bfloat16)
    mask_d = mask.to(DEV) if masked else None
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        # the exact engine reads float32 only: the module converts for it (first: its scratch overlays the status word)
        ys, _ = trunk.step(x, alive, hidden, engine=SIMT, bullets=bul16, bullet_mask=mask_d)
        y16, h16 = trunk.step(x, alive, hidden, engine=TENSOR, bullets=bul16, bullet_mask=mask_d)
        y32, h32 = trunk.step(x, alive, hidden, engine=TENSOR, bullets=bul16.float(), bullet_mask=mask_d)
    _status_ok()
    assert torch.equal(y16, y32) and torch.equal(h16, h32)
    assert norm_err(y16.cpu(), ys.cpu()) < 1e-2


@pytest.mark.parametrize("n_envs,ships,fields,nb", [(40, 8, 4, 80), (6, 100, 52, 33), (5, 100, 52, 0)])
def test_bfloat16_tokens_on_the_multi_launch_paths(n_envs, ships, fields, nb):
    """bfloat16 tokens in and out (``BNB_BF16_IO``) where the step takes several launches --
    sublayers that read bullets, environments larger than a tile: y comes back bfloat16 without a
    float32 copy on either side, the residual stream is rounded where one launch hands over to the
    next, so it agrees with the float32-token call to bfloat16 rounding (<= 1e-2 normalised) and
    the new state, which never passes through the token dtype's last rounding, to the same bound."""
    from boost_and_broadside_b200 import workloads as W

    _capi, SIMT, TENSOR = _engines()
    w = W.c2(n_envs=n_envs, seed=41, ships=ships, fields=fields)
    trunk = build_trunk([128, 4, 2, 2, 1, 1]).to(DEV)
    x, alive, hidden = (t.to(DEV) for t in (w.x, w.alive, w.hidden))
    x16 = x.to(torch.bfloat16)
    bul16 = mask_d = None
    if nb:
        bul, mask = _bullets(n_envs, nb, 13)
        bul16, mask_d = bul.to(DEV).to(torch.bfloat16), mask.to(DEV)
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        y16, h16 = trunk.step(x16, alive, hidden, engine=TENSOR, bullets=bul16, bullet_mask=mask_d)
        y32, h32 = trunk.step(x16.float(), alive, hidden, engine=TENSOR, bullets=bul16, bullet_mask=mask_d)
    _status_ok()
    assert y16.dtype == torch.bfloat16 and y32.dtype == torch.float32
    assert norm_err(y16.float().cpu(), y32.cpu()) < 1e-2
    assert norm_err(h16.cpu(), h32.cpu()) < 1e-2


def test_bfloat16_bullet_tokens_on_a_shape_the_tensor_kernels_do_not_serve():
    """3000 bullet slots per environment are more than the attention kernel stages: the call is
    served by the float32-reading kernels, which refuse bfloat16 tokens (BNB_ERR_UNSUPPORTED_DIMS);
    the module then hands them a float32 copy, and the result equals the float32 call."""
    from boost_and_broadside_b200 import workloads as W

    w = W.c2(n_envs=2, seed=37, ships=8, fields=4)
    bul, mask = _bullets(2, 3000, 11, p_active=0.1)
    trunk = build_trunk([128, 4, 2, 2, 1, 1]).to(DEV)
    x, alive, hidden = (t.to(DEV) for t in (w.x, w.alive, w.hidden))
    bul16 = bul.to(DEV).to(torch.bfloat16)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")   # the once-per-process note that the exact kernels served a bf16 call
        with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
            y16, h16 = trunk.step(x, alive, hidden, bullets=bul16, bullet_mask=mask.to(DEV))
            y32, h32 = trunk.step(x, alive, hidden, bullets=bul16.float(), bullet_mask=mask.to(DEV))
            # bfloat16 tokens as well: the same retry, and the module rounds the float32 result
            yb, hb = trunk.step(x.to(torch.bfloat16), alive, hidden, bullets=bul16, bullet_mask=mask.to(DEV))
            yf, hf = trunk.step(x.to(torch.bfloat16).float(), alive, hidden, bullets=bul16.float(), bullet_mask=mask.to(DEV))
    assert torch.equal(y16, y32) and torch.equal(h16, h32)
    assert bool(torch.isfinite(y16.float()).all())
    assert yb.dtype == torch.bfloat16 and torch.equal(yb, yf.to(torch.bfloat16)) and torch.equal(hb, hf)


def test_sequence_with_bullets_tensor_vs_oracle():
    from boost_and_broadside_b200 import workloads as W

    _capi, SIMT, TENSOR = _engines()
    w = W.c4(n_envs=9, timesteps=5, seed=29)
    T, B = w.x.shape[0], w.x.shape[1]
    bul, mask = _bullets(T * B, 40, 6)
    trunk = build_trunk([128, 4, 2, 2, 1, 1])
    ref_y, ref_h = O.trunk_sequence(w.x, w.alive, w.hidden, w.done, trunk_params(trunk), 4, "bf16", bul, mask)
    trunk = trunk.to(DEV)
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        yt, ht = trunk.sequence(w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV), w.done.to(DEV), engine=TENSOR,
                                bullets=bul.to(DEV), bullet_mask=mask.to(DEV))
    _status_ok()
    assert_close(yt, ref_y, "bf16", "sequence y vs oracle")
    assert_close(ht, ref_h, "bf16", "sequence hidden vs oracle")


def test_bullets_full_size_step_is_sliced_and_engines_agree():
    """The rollout-step configuration with 160 bullet slots per environment: 8192 x 160 bullet
    rows exceed one slice of the key/value scratch on both engines, so the projection and the
    attention run slice by slice; tensor and SIMT engines must agree and every environment
    without an active bullet must equal the bullet-free result."""
    from boost_and_broadside_b200 import workloads as W

    _capi, SIMT, TENSOR = _engines()
    w = W.c2(seed=31)
    n_envs = w.x.shape[0]
    batch = _capi.uniform_batch(n_envs, w.x.shape[1], 8)
    nb = 160
    share = _capi.lib.bnb_scratch_bytes(128, batch, 1, nb) - _capi.lib.bnb_scratch_bytes(128, batch, 1, 0)
    assert share < n_envs * nb * 256 * 2  # less than all keys and values, even in bf16: more than one slice
    gen = torch.Generator().manual_seed(7)
    bul = torch.randn(n_envs, nb, 128, generator=gen)
    mask = torch.rand(n_envs, nb, generator=gen) < 0.3
    idle = torch.rand(n_envs, generator=gen) < 0.25
    mask[idle] = False
    trunk = build_trunk([128, 4, 2, 2, 1, 1]).to(DEV)
    x, alive, hidden, bul_d, mask_d = (t.to(DEV) for t in (w.x, w.alive, w.hidden, bul, mask))
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        ys, hs = trunk.step(x, alive, hidden, engine=SIMT, bullets=bul_d, bullet_mask=mask_d)
        yt, ht = trunk.step(x, alive, hidden, engine=TENSOR, bullets=bul_d, bullet_mask=mask_d)
        y0, _ = trunk.step(x, alive, hidden, engine=TENSOR)
    _status_ok()
    assert torch.isfinite(yt).all() and torch.isfinite(ht).all()
    assert norm_err(yt.cpu(), ys.cpu()) < 2e-2
    assert norm_err(ht.cpu(), hs.cpu()) < 2e-2
    idle_d = idle.to(DEV)
    assert norm_err(yt[idle_d].cpu(), y0[idle_d].cpu()) < 1e-2      # gated off; kernels differ, values agree
    assert norm_err(yt[~idle_d].cpu(), y0[~idle_d].cpu()) > 1e-2    # and the bullets matter elsewhere


# ------------------------------------------------------------------ torch.compile


@pytest.mark.parametrize("mode", ["default", "reduce-overhead"])
def test_trunk_step_under_torch_compile(mode):
    """The reference wraps its policy in torch.compile (train/rl/ppo.py:396-400, CUDA graphs with
    reduce-overhead).  The trunk is one opaque operator there: no graph break (fullgraph), the
    same bits as the eager call, and replayable from the compiled CUDA graph."""
    import torch._dynamo

    from boost_and_broadside_b200 import workloads as W

    torch._dynamo.reset()
    trunk = build_trunk([128, 4, 2, 2, 1, 1]).to(DEV)
    w = W.c2b(n_envs=64, seed=51)
    x, alive, hidden, bul, bm = (t.to(DEV) for t in (w.x, w.alive, w.hidden, w.bullets, w.bullet_mask))

    def step(x, alive, hidden, bul, bm):
        with torch.autocast(DEV, dtype=torch.bfloat16):
            y, h = trunk.step(x, alive, hidden, bullets=bul, bullet_mask=bm)
        return y * 1.0, h          # something for the compiler to fuse around the operator

    compiled = torch.compile(step, fullgraph=True, mode=mode)
    with torch.no_grad():
        y0, h0 = step(x, alive, hidden, bul, bm)
        for _ in range(3):         # warm-up, capture, replay
            y1, h1 = compiled(x, alive, hidden, bul, bm)
            y1, h1 = y1.clone(), h1.clone()
    _status_ok()
    assert torch.equal(y0, y1) and torch.equal(h0, h1)
    # a changed input flows through the replay
    with torch.no_grad():
        y2, _ = compiled(x + 1.0, alive, hidden, bul, bm)
        y3, _ = step(x + 1.0, alive, hidden, bul, bm)
    assert torch.equal(y2.clone(), y3)
    torch._dynamo.reset()


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
def test_ragged_step_with_bullets(mode):
    """Mixed fleet sizes in one call, every environment with its ring of bullet slots; bf16 runs
    the tensor engine (tile plan + PRE | attention | POST for the reading sublayers), fp32 the
    SIMT engine."""
    from boost_and_broadside_b200 import RaggedBatch
    from boost_and_broadside_b200 import workloads as W

    w = W.c5(n_envs=57, seed=61)
    bul, mask = _bullets(57, 24, 8)
    trunk = build_trunk([128, 4, 2, 2, 1, 1])
    ref_y, ref_h = O.trunk_step_ragged(w.x, w.alive, w.hidden, w.n_tokens.tolist(), w.n_ships.tolist(),
                                       trunk_params(trunk), 4, mode, bul, mask)
    trunk = trunk.to(DEV)
    ctx = torch.autocast(DEV, dtype=torch.bfloat16) if mode == "bf16" else torch.autocast(DEV, enabled=False)
    with torch.no_grad(), ctx:
        y, h = trunk.step_ragged(w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV), RaggedBatch(w.n_tokens, w.n_ships),
                                 bullets=bul.to(DEV), bullet_mask=mask.to(DEV))
    if mode == "bf16":
        _status_ok()   # the status word only exists in the tensor engine's scratch layout
    assert_close(y, ref_y, mode, "ragged y")
    assert_close(h, ref_h, mode, "ragged hidden")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_second_device_while_the_first_is_current():
    """Replicas: the trunk follows its tensors' device, whatever the current device is (weight
    images, scratch and kernel attributes are kept per device)."""
    from boost_and_broadside_b200 import workloads as W

    w = W.c2b(n_envs=40, seed=71)
    trunk0 = build_trunk([128, 4, 2, 2, 1, 1]).to("cuda:0")
    trunk1 = build_trunk([128, 4, 2, 2, 1, 1]).to("cuda:1")
    outs = []
    with torch.cuda.device(0), torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        for dev, trunk in (("cuda:0", trunk0), ("cuda:1", trunk1)):
            y, h = trunk.step(w.x.to(dev), w.alive.to(dev), w.hidden.to(dev), bullets=w.bullets.to(dev),
                              bullet_mask=w.bullet_mask.to(dev))
            assert y.device == torch.device(dev)
            outs.append((y.cpu(), h.cpu()))
    torch.cuda.synchronize(0)
    torch.cuda.synchronize(1)
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


def test_norm_gains_folded_into_the_weight_image():
    """The tensor engine multiplies the RMSNorm gains into the packed weights of the Linear layers
    that consume the normed activations.  Fresh modules have unit gains, so give every norm a
    random gain (and the conv / gate biases random values) and compare with the oracle and with
    the exact engine; then change one gain in place and check that the image follows."""
    from boost_and_broadside_b200 import workloads as W

    _capi, SIMT, TENSOR = _engines()
    trunk = build_trunk([128, 4, 2, 2, 1, 1])
    gen = torch.Generator().manual_seed(81)
    with torch.no_grad():
        for name, p in trunk.named_parameters():
            if "norm" in name:
                p.copy_(1.0 + 0.3 * torch.randn(p.shape, generator=gen))
            elif name.endswith("bias"):
                p.copy_(0.2 * torch.randn(p.shape, generator=gen))
    w = W.c2b(n_envs=33, seed=83)
    ref_y, ref_h = O.trunk_step(w.x, w.alive, w.hidden, trunk_params(trunk), 4, "bf16", w.bullets, w.bullet_mask)
    trunk = trunk.to(DEV)
    args = [t.to(DEV) for t in (w.x, w.alive, w.hidden)]
    kw = dict(bullets=w.bullets.to(DEV), bullet_mask=w.bullet_mask.to(DEV))
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        ys, hs = trunk.step(*args, engine=SIMT, **kw)   # first: it uses the head of the scratch as data
        yt, ht = trunk.step(*args, engine=TENSOR, **kw)
    _status_ok()
    assert_close(yt, ref_y, "bf16", "y vs oracle")
    assert_close(ht, ref_h, "bf16", "hidden vs oracle")
    assert norm_err(yt.cpu(), ys.cpu()) < 1e-2 and norm_err(ht.cpu(), hs.cpu()) < 1e-2
    with torch.no_grad():
        trunk.yemong_layers[1].temporal[0].norm2.weight.mul_(1.5)
        trunk.yemong_layers[0].spatial[0].norm_bullet.weight.mul_(0.5)
    ref_y2, ref_h2 = O.trunk_step(w.x, w.alive, w.hidden, trunk_params(trunk.cpu()), 4, "bf16", w.bullets, w.bullet_mask)
    trunk = trunk.to(DEV)
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        yt2, ht2 = trunk.step(*args, engine=TENSOR, **kw)
    assert norm_err(ref_y2, ref_y) > 1e-2          # the change matters
    assert_close(yt2, ref_y2, "bf16", "y after a gain update")
    assert_close(ht2, ref_h2, "bf16", "hidden after a gain update")
