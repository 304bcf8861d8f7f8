"""bnb_spatial_block_fwd_static: the spatial sublayer for callers that cannot allocate.

A caller that owns no device allocator (a bare FFI stub) or that must not allocate next to
another framework's memory pool cannot supply the scratch that bnb_spatial_block_fwd asks
for.  The static variant keeps that scratch inside the library.  This test drives it
through the C ABI exactly as such a caller would (inputs and outputs only, no scratch, no
torch allocation between the calls) and checks it against the ordinary entry point, twice
in a row because every call reuses the same array and whatever the previous call left in it.

The file name sorts last on purpose, so a run that stops at the first failure has already
run every other test.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(mode_bf16: bool, n_envs: int, seed: int):
    from boost_and_broadside_b200 import ModelConfig, TransformerBlock, _capi
    from boost_and_broadside_b200 import workloads as W
    from boost_and_broadside_b200.yemong._weights import spatial_struct

    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(0)
    block = TransformerBlock(ModelConfig(128, 4, 2)).eval().to(dev)
    w = W.c1(n_envs=n_envs, seed=seed)
    x = w.x.to(dev).reshape(-1, 128).contiguous()
    alive = w.alive.to(dev).reshape(-1).contiguous().view(torch.uint8)
    batch = _capi.uniform_batch(n_envs, 8, 8)
    weights = spatial_struct(block, dev)
    precision = _capi.BNB_BF16 if mode_bf16 else _capi.BNB_FP32
    return _capi, dev, block, x, alive, batch, weights, precision


@pytest.mark.parametrize("mode_bf16", [False, True])
def test_static_entry_point_matches_the_ordinary_one_twice(mode_bf16):
    _capi, dev, block, x, alive, batch, weights, precision = _setup(mode_bf16, 256, 1)
    lib = _capi.lib
    stream = _capi.stream_handle(dev)

    # ordinary entry point, caller-provided scratch
    y_ref = torch.empty_like(x)
    scratch = torch.empty(lib.bnb_scratch_bytes(128, batch, 1, 0), dtype=torch.uint8, device=dev)
    st = lib.bnb_spatial_block_fwd(weights, 128, 4, x.data_ptr(), alive.data_ptr(), None, y_ref.data_ptr(), batch, 1,
                                   precision, _capi.ENGINE_SIMT, scratch.data_ptr(), scratch.numel(), stream)
    assert st == 0, lib.bnb_status_string(st)

    # a second, different input so that the second static call cannot pass on stale scratch
    _, _, _, x2, alive2, _, _, _ = _setup(mode_bf16, 256, 7)
    y_ref2 = torch.empty_like(x2)
    st = lib.bnb_spatial_block_fwd(weights, 128, 4, x2.data_ptr(), alive2.data_ptr(), None, y_ref2.data_ptr(), batch, 1,
                                   precision, _capi.ENGINE_SIMT, scratch.data_ptr(), scratch.numel(), stream)
    assert st == 0, lib.bnb_status_string(st)

    y1 = torch.empty_like(x)
    y2 = torch.empty_like(x2)
    st = lib.bnb_spatial_block_fwd_static(weights, 128, 4, x.data_ptr(), alive.data_ptr(), y1.data_ptr(), batch, 1,
                                          precision, stream)
    assert st == 0, lib.bnb_status_string(st)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(dev)[0]
    st = lib.bnb_spatial_block_fwd_static(weights, 128, 4, x2.data_ptr(), alive2.data_ptr(), y2.data_ptr(), batch, 1,
                                          precision, stream)
    assert st == 0, lib.bnb_status_string(st)
    torch.cuda.synchronize()
    free_after = torch.cuda.mem_get_info(dev)[0]

    tol = 1e-4 if not mode_bf16 else 2e-2 * float(y_ref.abs().max())
    assert float((y1 - y_ref).abs().max()) <= tol
    assert float((y2 - y_ref2).abs().max()) <= tol
    assert torch.isfinite(y1).all() and torch.isfinite(y2).all()
    assert free_after == free_before, "the static entry point changed the amount of free device memory"


def test_static_entry_point_rejects_batches_beyond_its_limit():
    _capi, dev, block, x, alive, batch, weights, precision = _setup(False, 257, 1)  # 2056 rows > 2048
    lib = _capi.lib
    y = torch.full_like(x, 7.0)
    st = lib.bnb_spatial_block_fwd_static(weights, 128, 4, x.data_ptr(), alive.data_ptr(), y.data_ptr(), batch, 1,
                                          precision, _capi.stream_handle(dev))
    assert st == 9  # BNB_ERR_EXCEEDS_STATIC_LIMIT
    assert b"fixed scratch" in lib.bnb_status_string(st)
    torch.cuda.synchronize()
    assert bool((y == 7.0).all()), "a rejected call must not launch anything"
