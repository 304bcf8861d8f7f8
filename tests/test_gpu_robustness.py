"""What happens around the kernels when things go sideways: a bounded wait that runs out, parameters
updated behind the version counter, a scratch buffer outgrown while a CUDA graph still points at it.

No test here faults, traps or hangs the GPU.  The wait test uses the library's own hook
(bnb_debug_wait_test): one weight copy is left out, the wait for it gives up after a short poll
limit, the kernel drains and returns, and the status word says which wait it was.
"""

from __future__ import annotations

import pytest
import torch

from tests.helpers import build_trunk

pytestmark = pytest.mark.gpu
DEV = "cuda"
DIMS = [128, 4, 2, 2, 1, 1]


def _inputs(n_envs, seed=11):
    from boost_and_broadside_b200 import workloads as W

    w = W.c2(n_envs=n_envs, seed=seed)
    return w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV)


def test_a_bounded_wait_that_runs_out_is_reported_and_the_context_stays_usable():
    from boost_and_broadside_b200 import _capi

    lib = _capi.lib
    trunk = build_trunk(DIMS).to(DEV)
    x, alive, hidden = _inputs(10)   # one tile, one CTA
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        y_ok, h_ok = trunk.step(x, alive, hidden)
        torch.cuda.synchronize()
        lib.bnb_clear_status()
        assert lib.bnb_last_status() == 0
        # CTA 0 never receives the weights of its sixth ring operation (the first gate|up pair of the
        # first sublayer); waits poll 4096 times instead of 2^20
        lib.bnb_debug_wait_test(5, 1 << 12)
        try:
            trunk.step(x, alive, hidden)
            torch.cuda.synchronize()   # the kernel returned: nothing spun forever, nothing faulted
        finally:
            lib.bnb_debug_wait_test(-1, 0)
        assert lib.bnb_last_status() == 101   # BNB_STATUS_WAIT_WEIGHTS
        assert b"weight copy" in lib.bnb_status_string(101)
        # the next call refuses to go on silently ...
        with pytest.raises(RuntimeError, match="bounded wait"):
            trunk.step(x, alive, hidden)
        # ... once; after that the same context computes the same bits as before
        y2, h2 = trunk.step(x, alive, hidden)
        torch.cuda.synchronize()
        assert lib.bnb_last_status() == 0
    assert torch.equal(y2, y_ok) and torch.equal(h2, h_ok)


def _scale_some_parameters_behind_the_version_counter(trunk):
    """``p.data.copy_`` as the reference's running-average update does (train/rl/opponents.py:112):
    the values change, ``_version`` does not."""
    changed = 0
    for name, p in trunk.named_parameters():
        if name.endswith(("qkv.weight", "gate_proj.weight", "norm2.weight", "linear1.weight", "log_lambda")):
            v = p._version
            p.data.copy_(p.data * 1.25 + 0.01)
            assert p._version == v
            changed += 1
    assert changed > 0


def test_weight_images_follow_updates_that_bump_no_version_counter():
    from boost_and_broadside_b200 import _capi

    trunk = build_trunk(DIMS).to(DEV)
    x, alive, hidden = _inputs(64)
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        y0, _ = trunk.step(x, alive, hidden)
        _scale_some_parameters_behind_the_version_counter(trunk)
        y1, h1 = trunk.step(x, alive, hidden)
        y_simt, h_simt = trunk.step(x, alive, hidden, engine=_capi.ENGINE_SIMT)   # reads the float32 parameters directly
    assert not torch.equal(y0, y1)
    assert float((y1 - y_simt).abs().max() / y_simt.abs().max()) <= 2e-2
    assert float((h1 - h_simt).abs().max() / h_simt.abs().max()) <= 2e-2


def test_a_replayed_cuda_graph_repacks_from_the_live_parameters():
    trunk = build_trunk(DIMS).to(DEV)
    x, alive, hidden = _inputs(64)
    side = torch.cuda.Stream()
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            trunk.step(x, alive, hidden)   # warm-up on the capture stream
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            y_g, h_g = trunk.step(x, alive, hidden)
        g.replay()
        torch.cuda.synchronize()
        y_before = y_g.clone()
        for p in trunk.parameters():
            if p.dim() == 2:
                p.mul_(1.1)                                  # an optimizer-style in-place update
        _scale_some_parameters_behind_the_version_counter(trunk)   # and the averaging-style one
        g.replay()
        torch.cuda.synchronize()
        y_eager, h_eager = trunk.step(x, alive, hidden)
        torch.cuda.synchronize()
    assert not torch.equal(y_before, y_g)
    assert torch.equal(y_g, y_eager) and torch.equal(h_g, h_eager)


def test_an_outgrown_scratch_buffer_stays_valid_for_the_graphs_that_hold_it():
    """A graph captured at a small batch keeps the address of the scratch buffer of that time.  A
    larger call later makes the binding allocate a bigger buffer; the old one must neither be freed
    nor handed to anybody else, or the small graph's replay would scribble over foreign memory."""
    from boost_and_broadside_b200 import _capi, workloads as W

    trunk = build_trunk(DIMS).to(DEV)
    side = torch.cuda.Stream()
    # bullets make the call use scratch beyond the status word (q|k|v, keys and values of a slice)
    ws = W.c2b(n_envs=16, seed=3)
    small = [t.to(DEV) for t in (ws.x, ws.alive, ws.hidden, ws.bullets, ws.bullet_mask)]
    with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            y_small, _ = trunk.step(small[0], small[1], small[2], bullets=small[3], bullet_mask=small[4])
            key = (torch.cuda.current_device(), _capi.stream_handle(torch.device(DEV, torch.cuda.current_device())))
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            y_g, _ = trunk.step(small[0], small[1], small[2], bullets=small[3], bullet_mask=small[4])
        old = _capi._scratch[key]
        wl = W.c2b(n_envs=max(4096, 4 * old.numel() // (80 * 512) + 1), seed=4)
        large = [t.to(DEV) for t in (wl.x, wl.alive, wl.hidden, wl.bullets, wl.bullet_mask)]
        with torch.cuda.stream(side):
            trunk.step(large[0], large[1], large[2], bullets=large[3], bullet_mask=large[4])
        side.synchronize()
        new = _capi._scratch[key]
        assert new.data_ptr() != old.data_ptr() and new.numel() > old.numel()
        assert any(b.data_ptr() == old.data_ptr() for b in _capi._scratch_outgrown)
        del large
        # whatever torch allocates now must not land on the old buffer
        canaries = [torch.full((old.numel() // 4,), 7.0, device=DEV) for _ in range(4)]
        g.replay()
        torch.cuda.synchronize()
    assert all(bool((c == 7.0).all()) for c in canaries)
    assert torch.equal(y_g, y_small)


def test_mismatched_state_and_mask_shapes_are_refused_on_the_host():
    """A hidden tensor whose rows do not divide by the environments, or a mask shorter than the
    tokens, would make the kernels read the wrong rows or past the end: the methods raise instead."""
    from boost_and_broadside_b200 import RaggedBatch

    trunk = build_trunk(DIMS).to(DEV)
    x, alive, hidden = _inputs(6)
    with torch.no_grad():
        with pytest.raises(RuntimeError, match="hidden has"):
            trunk.step(x, alive, hidden[:, :-1])
        with pytest.raises(RuntimeError, match="alive must have shape"):
            trunk.step(x, alive[:, :-1], hidden)
        with pytest.raises(RuntimeError, match="reset_env must have shape"):
            trunk.step(x, alive, hidden, reset_env=torch.zeros(5, dtype=torch.bool, device=DEV))
        xs, als = x[None].expand(3, -1, -1, -1), alive[None].expand(3, -1, -1)
        with pytest.raises(RuntimeError, match="initial_hidden has"):
            trunk.sequence(xs, als, hidden[:, :-1])
        with pytest.raises(RuntimeError, match="done_mask must have shape"):
            trunk.sequence(xs, als, hidden, torch.zeros(2, 6, dtype=torch.bool, device=DEV))
        with pytest.raises(RuntimeError, match="alive_mask must have shape"):
            trunk.sequence(xs, als[:2], hidden)
        rb = RaggedBatch(torch.full((6,), 12), torch.full((6,), 8))
        with pytest.raises(RuntimeError, match="alive must have shape"):
            trunk.step_ragged(x.reshape(-1, 128), alive.reshape(-1)[:-1], hidden, rb)


def test_a_bf16_call_that_falls_to_the_exact_engine_is_counted_and_warned_about():
    """BNB_ENGINE_AUTO picks the exact kernels for shapes the tensor-core kernels are not built for
    (here d_model 64); the call is counted by the library and the binding warns once."""
    import warnings

    from boost_and_broadside_b200 import _capi

    trunk = build_trunk([64, 4, 1, 1, 1, 0]).to(DEV)
    x = torch.randn(4, 6, 64, device=DEV)
    alive = torch.ones(4, 6, dtype=torch.bool, device=DEV)
    hidden = trunk.initial_hidden(4, 6, torch.device(DEV))
    before = _capi.lib.bnb_auto_fallback_count()
    _capi._fallback_warned = False
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        with torch.no_grad(), torch.autocast(DEV, dtype=torch.bfloat16):
            trunk.step(x, alive, hidden)
            trunk.step(x, alive, hidden)
    assert _capi.lib.bnb_auto_fallback_count() >= before + 2
    assert sum("exact (SIMT) kernels" in str(w.message) for w in seen) == 1
