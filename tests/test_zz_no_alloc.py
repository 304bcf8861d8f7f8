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


def _case(mode_bf16: bool, n_envs: int, seed: int, d_model: int = 128, n_heads: int = 4, tokens: int = 8,
          with_alive: bool = True, n_groups: int = 1, ragged: bool = False):
    """Module, inputs and C structs of one spatial-sublayer call."""
    from boost_and_broadside_b200 import ModelConfig, TransformerBlock, _capi
    from boost_and_broadside_b200.yemong._weights import spatial_struct

    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(0)
    block = TransformerBlock(ModelConfig(d_model, n_heads, 2)).eval()
    g = torch.Generator().manual_seed(seed)
    keep = []
    if ragged:
        sizes = torch.randint(1, tokens + 1, (n_envs,), generator=g)
        tok_off = torch.zeros(n_envs + 1, dtype=torch.int32)
        tok_off[1:] = sizes.cumsum(0)
        total = int(tok_off[-1])
        off_d = tok_off.to(dev)
        keep.append(off_d)
        batch = _capi.Batch(n_envs, 0, 0, int(sizes.max()), total, total, off_d.data_ptr(), off_d.data_ptr(), None, None, 0)
        env_sizes = sizes.tolist()
    else:
        total = n_envs * tokens
        batch = _capi.uniform_batch(n_envs, tokens, tokens)
        env_sizes = [tokens] * n_envs
    x = torch.randn(n_groups, total, d_model, generator=g)
    alive = (torch.rand(n_groups, total, generator=g) < 0.8) if with_alive else None
    precision = _capi.BNB_BF16 if mode_bf16 else _capi.BNB_FP32
    block_d = block.to(dev)
    return dict(capi=_capi, dev=dev, block=block_d, x_cpu=x, alive_cpu=alive, x=x.to(dev).contiguous(),
                alive=None if alive is None else alive.to(dev).contiguous().view(torch.uint8), batch=batch,
                weights=spatial_struct(block_d, dev), precision=precision, D=d_model, H=n_heads, groups=n_groups,
                env_sizes=env_sizes, keep=keep)


def _ordinary(c):
    lib = c["capi"].lib
    y = torch.empty_like(c["x"])
    scratch = torch.empty(lib.bnb_scratch_bytes(c["D"], c["batch"], c["groups"], 0), dtype=torch.uint8, device=c["dev"])
    st = lib.bnb_spatial_block_fwd(c["weights"], c["D"], c["H"], c["x"].data_ptr(), c["capi"].ptr(c["alive"]), None,
                                   y.data_ptr(), c["batch"], c["groups"], c["precision"], c["capi"].ENGINE_SIMT,
                                   scratch.data_ptr(), scratch.numel(), c["capi"].stream_handle(c["dev"]))
    assert st == 0, lib.bnb_status_string(st)
    return y


def _static(c, y=None):
    lib = c["capi"].lib
    y = torch.empty_like(c["x"]) if y is None else y
    st = lib.bnb_spatial_block_fwd_static(c["weights"], c["D"], c["H"], c["x"].data_ptr(), c["capi"].ptr(c["alive"]),
                                          y.data_ptr(), c["batch"], c["groups"], c["precision"],
                                          c["capi"].stream_handle(c["dev"]))
    return st, y


def _oracle(c, mode):
    """The CPU oracle on the same inputs, environment by environment size."""
    from oracle import trunk_oracle as O

    sd = {k: v.detach().cpu() for k, v in c["block"].state_dict().items()}
    out = torch.empty_like(c["x_cpu"])
    for gi in range(c["groups"]):
        off = 0
        for n in c["env_sizes"]:
            a = None if c["alive_cpu"] is None else c["alive_cpu"][gi, off : off + n][None]
            out[gi, off : off + n] = O.spatial_block(c["x_cpu"][gi, off : off + n][None], a, sd, c["H"], mode)[0]
            off += n
    return out


@pytest.mark.parametrize("mode_bf16", [False, True])
def test_static_entry_point_matches_the_ordinary_one_twice(mode_bf16):
    """Two calls in a row through the array the library holds, each bit-identical to the ordinary
    entry point (the same deterministic kernels, only the scratch differs) and within tolerance of
    the CPU oracle; the amount of free device memory does not move."""
    c1 = _case(mode_bf16, 256, 1)
    c2 = _case(mode_bf16, 256, 7)   # a different input: the second call cannot pass on stale scratch
    y_ref1, y_ref2 = _ordinary(c1), _ordinary(c2)
    y1, y2 = torch.empty_like(c1["x"]), torch.empty_like(c2["x"])
    st, _ = _static(c1, y1)
    assert st == 0, c1["capi"].lib.bnb_status_string(st)
    torch.cuda.synchronize()
    for attempt in range(2):   # another process on the same GPU can move the figure: look twice
        free_before = torch.cuda.mem_get_info(c1["dev"])[0]
        st, _ = _static(c2, y2)
        assert st == 0, c1["capi"].lib.bnb_status_string(st)
        torch.cuda.synchronize()
        if torch.cuda.mem_get_info(c1["dev"])[0] == free_before:
            break
    else:
        raise AssertionError("the static entry point changed the amount of free device memory")
    assert torch.equal(y1, y_ref1) and torch.equal(y2, y_ref2)
    mode = "bf16" if mode_bf16 else "fp32"
    ref = _oracle(c1, mode)
    err = float((y1.cpu() - ref).abs().max())
    assert err <= (1e-4 if not mode_bf16 else 2e-2 * float(ref.abs().max())), err


@pytest.mark.parametrize("kwargs", [
    dict(d_model=64, n_heads=2, tokens=5, n_envs=40),
    dict(with_alive=False, n_envs=30, tokens=12),
    dict(n_groups=2, n_envs=24, tokens=8),
    dict(ragged=True, n_envs=50, tokens=20),
])
def test_static_entry_point_on_other_geometries(kwargs):
    """Narrower model, no alive mask, a replicated batch and a ragged one: always the ordinary
    entry point's bits."""
    n_envs = kwargs.pop("n_envs")
    c = _case(False, n_envs, 3, **kwargs)
    y_ref = _ordinary(c)
    st, y = _static(c)
    assert st == 0, c["capi"].lib.bnb_status_string(st)
    torch.cuda.synchronize()
    assert torch.equal(y, y_ref)
    ref = _oracle(c, "fp32")
    assert float((y.cpu() - ref).abs().max()) <= 1e-4


def test_static_entry_point_rejects_batches_beyond_its_limit():
    c = _case(False, 257, 1)  # 2056 rows > 2048
    lib = c["capi"].lib
    y = torch.full_like(c["x"], 7.0)
    st, _ = _static(c, y)
    assert st == 9  # BNB_ERR_EXCEEDS_STATIC_LIMIT
    assert b"fixed scratch" in lib.bnb_status_string(st)
    torch.cuda.synchronize()
    assert bool((y == 7.0).all()), "a rejected call must not launch anything"


def test_static_entry_point_validates_like_the_ordinary_one():
    """The argument checks of bnb_spatial_block_fwd apply unchanged (one shared routine)."""
    c = _case(False, 4, 1)
    lib, capi = c["capi"].lib, c["capi"]
    bad = capi.Batch(4, 8, 9, 8, 32, 36, None, None, None, None, 0)   # more ships than tokens
    y = torch.empty_like(c["x"])
    st = lib.bnb_spatial_block_fwd_static(c["weights"], 128, 4, c["x"].data_ptr(), None, y.data_ptr(), bad, 1, 0,
                                          capi.stream_handle(c["dev"]))
    assert st == 5  # BNB_ERR_BAD_ARGUMENT
    st = lib.bnb_spatial_block_fwd_static(c["weights"], 128, 4, c["x"].data_ptr() + 4, None, y.data_ptr(), c["batch"], 1, 0,
                                          capi.stream_handle(c["dev"]))
    assert st == 2  # BNB_ERR_MISALIGNED
