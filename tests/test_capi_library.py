"""The C-ABI library loads and exports every symbol include/bnb_trunk.h declares; host-side
argument validation returns status codes without touching a device."""

import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "bnb_trunk.h")


def declared_functions() -> list[str]:
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bnb_[a-z_0-9]+)\s*\(", text)))


def test_header_and_binding_agree():
    from boost_and_broadside_b200 import _capi

    assert declared_functions() == sorted(_capi.EXPORTS)


def test_library_exports_every_declared_symbol():
    from boost_and_broadside_b200 import _capi

    lib = C.CDLL(_capi.LIB_PATH)
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in bnb_trunk.h but not exported"
    assert _capi.lib.bnb_abi_version() == 3
    assert _capi.lib.bnb_status_string(0) == b"ok"
    assert b"null" in _capi.lib.bnb_status_string(1)


def test_supported_query_is_host_only():
    from boost_and_broadside_b200 import _capi

    q = _capi.lib.bnb_supported
    assert q(128, 4, 12, _capi.BNB_FP32, _capi.ENGINE_AUTO) == 1
    assert q(128, 4, 152, _capi.BNB_BF16, _capi.ENGINE_AUTO) == 1
    assert q(64, 4, 8, _capi.BNB_BF16, _capi.ENGINE_SIMT) == 1
    assert q(32, 4, 8, _capi.BNB_FP32, _capi.ENGINE_SIMT) == 1
    assert q(100, 4, 8, _capi.BNB_FP32, _capi.ENGINE_AUTO) == 0      # not a multiple of 32
    assert q(256, 4, 8, _capi.BNB_FP32, _capi.ENGINE_AUTO) == 0      # above the built width
    assert q(128, 3, 8, _capi.BNB_FP32, _capi.ENGINE_AUTO) == 0      # heads do not divide
    assert q(128, 4, 0, _capi.BNB_FP32, _capi.ENGINE_AUTO) == 0
    assert q(128, 4, 8, 7, _capi.ENGINE_AUTO) == 0


def test_argument_validation_returns_status_codes():
    """Bad arguments are rejected on the host before any launch."""
    from boost_and_broadside_b200 import _capi

    lib = _capi.lib
    batch = _capi.uniform_batch(4, 8, 8)
    w = _capi.SpatialWeights()  # all null
    st = lib.bnb_spatial_block_fwd(w, 128, 4, None, None, None, None, batch, 1, 0, 0, None, 0, None)
    assert st == 1  # BNB_ERR_NULL_POINTER
    st = lib.bnb_spatial_block_fwd(w, 100, 4, None, None, None, None, batch, 1, 0, 0, None, 0, None)
    assert st == 3  # BNB_ERR_UNSUPPORTED_DIMS
    bad = _capi.Batch(4, 8, 9, 8, 32, 36, None, None)  # more ships than tokens
    st = lib.bnb_spatial_block_fwd(w, 128, 4, None, None, None, None, bad, 1, 0, 0, None, 0, None)
    assert st == 5  # BNB_ERR_BAD_ARGUMENT
    fake = 0x1000
    w = _capi.SpatialWeights(*([fake] * 7), None, None, None)
    st = lib.bnb_spatial_block_fwd(w, 128, 4, fake + 4, None, None, fake, batch, 1, 0, 0, fake, 1 << 30, None)
    assert st == 2  # BNB_ERR_MISALIGNED
    st = lib.bnb_spatial_block_fwd(w, 128, 4, fake, None, None, fake, batch, 1, 0, 1, fake, 16, None)
    assert st == 6  # BNB_ERR_SCRATCH_TOO_SMALL
    st = lib.bnb_spatial_block_fwd(w, 128, 4, fake, None, None, fake, batch, 1, 9, 0, fake, 1 << 30, None)
    assert st == 5
    # bullet arguments: a half-given parameter pair, and a bullet set without tokens
    half = _capi.SpatialWeights(*([fake] * 8), None, None)
    assert lib.bnb_spatial_block_fwd(half, 128, 4, fake, None, None, fake, batch, 1, 0, 0, fake, 1 << 30, None) == 1
    reads = _capi.SpatialWeights(*([fake] * 9), None)
    no_tokens = _capi.Bullets(None, None, 10)
    assert lib.bnb_spatial_block_fwd(reads, 128, 4, fake, None, no_tokens, fake, batch, 1, 0, 0, fake, 1 << 30, None) == 1
    no_slots = _capi.Bullets(fake, None, 0)
    assert lib.bnb_spatial_block_fwd(reads, 128, 4, fake, None, no_slots, fake, batch, 1, 0, 0, fake, 1 << 30, None) == 5
    # the bullet share of the scratch is bounded whatever the batch
    big = _capi.uniform_batch(1 << 20, 12, 8)
    assert lib.bnb_scratch_bytes(128, big, 1, 80) - lib.bnb_scratch_bytes(128, big, 1, 0) <= (512 << 20) + (8 << 20)
    assert lib.bnb_scratch_bytes(128, batch, 1, 80) > lib.bnb_scratch_bytes(128, batch, 1, 0)
    # an empty batch is a successful no-op
    empty = _capi.uniform_batch(0, 8, 8)
    assert lib.bnb_spatial_block_fwd(w, 128, 4, None, None, None, None, empty, 1, 0, 0, None, 0, None) == 0
    assert lib.bnb_scratch_bytes(128, batch, 1, 0) >= 4 * 8 * 4 * 128 * 4


def test_missing_library_fails_loudly(tmp_path):
    from boost_and_broadside_b200 import _capi

    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _capi.load_library(str(tmp_path / "libbnb_trunk.so"))


def test_plan_tiles_is_a_host_function():
    """Best-fit-decreasing packing of whole environments into 128-row tiles, on the host."""
    import torch

    from boost_and_broadside_b200 import _capi

    sizes = torch.tensor([100, 28, 1, 128, 64, 64, 2, 127], dtype=torch.int32)
    off = torch.zeros(len(sizes) + 1, dtype=torch.int32)
    off[1:] = sizes.cumsum(0)
    plan = torch.zeros(len(sizes) + 1, dtype=torch.int32)
    ids = torch.zeros(len(sizes), dtype=torch.int32)
    n = C.c_int(0)
    st = _capi.lib.bnb_plan_tiles(off.data_ptr(), len(sizes), plan.data_ptr(), ids.data_ptr(), len(sizes) + 1, C.byref(n))
    assert st == 0
    # best-fit decreasing: 128 | 127+1 | 100+28 | 64+64 | 2  -> five tiles, every environment once
    assert n.value == 5
    begins = plan[: n.value + 1].tolist()
    assert begins[0] == 0 and begins[-1] == len(sizes)
    assert sorted(ids.tolist()) == list(range(len(sizes)))
    for t in range(n.value):
        assert sum(int(sizes[e]) for e in ids[begins[t] : begins[t + 1]].tolist()) <= 128
    # an environment larger than a tile is refused
    off2 = torch.tensor([0, 129], dtype=torch.int32)
    st = _capi.lib.bnb_plan_tiles(off2.data_ptr(), 1, plan.data_ptr(), ids.data_ptr(), 2, C.byref(n))
    assert st == 4  # BNB_ERR_TOO_MANY_TOKENS
    assert _capi.lib.bnb_plan_tiles(None, 1, plan.data_ptr(), ids.data_ptr(), 2, C.byref(n)) == 1
