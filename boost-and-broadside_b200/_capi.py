"""ctypes binding of ``libbnb_trunk.so`` (declared in include/bnb_trunk.h).

The library is the only compute path: if it is missing or does not export the declared
symbols, importing this module raises.  Nothing here falls back to PyTorch arithmetic.
"""

from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libbnb_trunk.so")

BNB_FP32, BNB_BF16, BNB_BF16_IO = 0, 1, 2
ERR_UNSUPPORTED_DIMS = 3   # BNB_ERR_UNSUPPORTED_DIMS: the kernels asked for do not serve these shapes / dtypes
ENGINE_AUTO, ENGINE_SIMT, ENGINE_TENSOR = 0, 1, 2
ABI_VERSION = 3

_fp = C.c_void_p


class SpatialWeights(C.Structure):
    _fields_ = [(n, _fp) for n in ("norm1_w", "qkv_w", "out_w", "norm2_w", "gate_w", "up_w", "down_w",
                                   "norm_bullet_w", "kv_bullet_w", "packed")]


class SpatialGrads(C.Structure):
    _fields_ = [(n, _fp) for n in ("norm1_w", "qkv_w", "out_w", "norm2_w", "gate_w", "up_w", "down_w",
                                   "norm_bullet_w", "kv_bullet_w")]


class TemporalGrads(C.Structure):
    _fields_ = [
        (n, _fp)
        for n in (
            "norm1_w", "linear1_w", "conv_w", "conv_b", "log_lambda", "a_w", "a_b", "x_w", "x_b",
            "linear2_w", "out_w", "norm2_w", "gate_w", "up_w", "down_w", "field_sub_w",
        )
    ]


class Bullets(C.Structure):
    _fields_ = [("tokens", _fp), ("active", _fp), ("per_env", C.c_int32), ("tokens_bf16", C.c_int32)]


class TemporalWeights(C.Structure):
    _fields_ = [
        (n, _fp)
        for n in (
            "norm1_w", "linear1_w", "conv_w", "conv_b", "log_lambda", "a_w", "a_b", "x_w", "x_b",
            "linear2_w", "out_w", "norm2_w", "gate_w", "up_w", "down_w", "field_sub_w", "packed",
        )
    ]


class Batch(C.Structure):
    _fields_ = [
        ("n_envs", C.c_int32),
        ("tokens_per_env", C.c_int32),
        ("ships_per_env", C.c_int32),
        ("max_tokens_per_env", C.c_int32),
        ("total_tokens", C.c_int32),
        ("total_ships", C.c_int32),
        ("tok_off", _fp),
        ("ship_off", _fp),
        ("tile_env_begin", _fp),
        ("tile_env_ids", _fp),
        ("n_tiles", C.c_int32),
    ]


EXPORTS = {
    "bnb_abi_version": (C.c_int, []),
    "bnb_status_string": (C.c_char_p, [C.c_int]),
    "bnb_launch_count": (C.c_ulonglong, []),
    "bnb_auto_fallback_count": (C.c_ulonglong, []),
    "bnb_supported": (C.c_int, [C.c_int] * 5),
    "bnb_plan_tiles": (C.c_int, [_fp, C.c_int, _fp, _fp, C.c_int, C.POINTER(C.c_int)]),
    "bnb_scratch_bytes": (C.c_size_t, [C.c_int, C.POINTER(Batch), C.c_int, C.c_int]),
    "bnb_spatial_block_fwd": (
        C.c_int,
        [C.POINTER(SpatialWeights), C.c_int, C.c_int, _fp, _fp, C.POINTER(Bullets), _fp, C.POINTER(Batch), C.c_int,
         C.c_int, C.c_int, _fp, C.c_size_t, _fp],
    ),
    "bnb_spatial_block_fwd_static": (
        C.c_int,
        [C.POINTER(SpatialWeights), C.c_int, C.c_int, _fp, _fp, _fp, C.POINTER(Batch), C.c_int, C.c_int, _fp],
    ),
    "bnb_temporal_block_fwd": (
        C.c_int,
        [C.POINTER(TemporalWeights), C.c_int, _fp, _fp, _fp, _fp, _fp, C.POINTER(Batch), C.c_int, C.c_int, C.c_int,
         _fp, C.c_size_t, _fp],
    ),
    "bnb_trunk_step": (
        C.c_int,
        [C.POINTER(SpatialWeights), C.POINTER(TemporalWeights), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
         _fp, _fp, C.POINTER(Bullets), _fp, _fp, _fp, _fp, C.POINTER(Batch), C.c_int, C.c_int, _fp, C.c_size_t, _fp],
    ),
    "bnb_trunk_sequence": (
        C.c_int,
        [C.POINTER(SpatialWeights), C.POINTER(TemporalWeights), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
         _fp, _fp, C.POINTER(Bullets), _fp, _fp, _fp, _fp, C.POINTER(Batch), C.c_int, C.c_int, C.c_int, _fp, C.c_size_t,
         _fp],
    ),
    "bnb_trunk_bwd_scratch_bytes": (C.c_size_t, [C.c_int] * 4 + [C.POINTER(Batch), C.c_int, C.c_int, C.c_int]),
    "bnb_trunk_sequence_bwd": (C.c_int, [C.POINTER(SpatialWeights), C.POINTER(TemporalWeights), C.POINTER(SpatialGrads),
                                         C.POINTER(TemporalGrads)] + [C.c_int] * 5 + [_fp, _fp, C.POINTER(Bullets), _fp, _fp,
                                         C.POINTER(Batch), C.c_int, C.c_int, _fp, _fp, _fp, _fp, _fp, _fp, C.c_size_t, _fp, C.c_size_t, _fp]),
    "bnb_trunk_kept_bytes": (C.c_size_t, [C.c_int] * 5 + [C.POINTER(Batch), C.c_int, C.c_int, C.c_int]),
    "bnb_trunk_sequence_fwd_train": (
        C.c_int,
        [C.POINTER(SpatialWeights), C.POINTER(TemporalWeights), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
         _fp, _fp, C.POINTER(Bullets), _fp, _fp, _fp, _fp, C.POINTER(Batch), C.c_int, C.c_int, _fp, C.c_size_t, _fp, C.c_size_t,
         _fp]),
    "bnb_reset_hidden": (C.c_int, [_fp, _fp, _fp, C.c_int, C.c_int, C.POINTER(Batch), _fp]),
    "bnb_packed_spatial_bytes": (C.c_size_t, [C.c_int]),
    "bnb_packed_temporal_bytes": (C.c_size_t, [C.c_int]),
    "bnb_pack_spatial": (C.c_int, [C.POINTER(SpatialWeights), C.c_int, C.c_int, _fp, _fp]),
    "bnb_pack_temporal": (C.c_int, [C.POINTER(TemporalWeights), C.c_int, _fp, _fp]),
    "bnb_gated_mlp_fwd": (C.c_int, [_fp, _fp, _fp, C.c_int, _fp, _fp, C.c_int, C.c_int, _fp]),
    "bnb_rglru_fwd": (C.c_int, [_fp] * 5 + [C.c_int, _fp, _fp, _fp, _fp, _fp, C.c_int, C.c_int, C.c_int, _fp]),
    "bnb_encoder_mlp_fwd": (C.c_int, [_fp] * 6 + [C.c_int] * 4 + [_fp, _fp, C.c_int, C.c_int, _fp]),
    "bnb_head_mlp_fwd": (C.c_int, [_fp] * 5 + [C.c_int] * 4 + [_fp, _fp, C.c_int, C.c_int, _fp]),
    "bnb_action_dist_fwd": (C.c_int, [_fp] * 6 + [C.c_int, C.c_int, _fp]),
    "bnb_team_pma_scratch_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "bnb_team_pma_fwd": (C.c_int, [_fp] * 4 + [C.c_int, C.c_int, _fp, _fp, _fp, _fp] + [C.c_int] * 4 + [_fp, C.c_size_t, _fp]),
    "bnb_pack_trunk": (C.c_int, [C.POINTER(SpatialWeights), C.c_int, C.POINTER(TemporalWeights), C.c_int, C.c_int, C.c_int, _fp]),
    "bnb_last_status": (C.c_int, []),
    "bnb_clear_status": (None, []),
    "bnb_debug_wait_test": (None, [C.c_int, C.c_int]),
}


def load_library(path: str = LIB_PATH) -> C.CDLL:
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python boost-and-broadside_b200/build.py` "
            "(nvcc, sm_100a). The trunk has no CPU or PyTorch fallback."
        )
    lib = C.CDLL(path)
    for name, (res, args) in EXPORTS.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    if lib.bnb_abi_version() != ABI_VERSION:
        raise RuntimeError(f"libbnb_trunk.so has ABI {lib.bnb_abi_version()}, binding expects {ABI_VERSION}")
    return lib


lib = load_library()


class BnbError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, fn: str, status: int):
        self.status = status
        super().__init__(f"{fn}: {lib.bnb_status_string(status).decode()} (status {status})")


def check(fn: str, status: int) -> None:
    if status != 0:
        if status == ERR_UNSUPPORTED_DIMS:
            raise ValueError(f"{fn}: {lib.bnb_status_string(status).decode()}")
        raise BnbError(fn, status)


_fallbacks_seen = 0
_fallback_warned = False


def note_engine_choice(what: str) -> None:
    """Warn, once per process, when a bfloat16 call left to BNB_ENGINE_AUTO was served by the exact
    kernels: the result is right, the speed is several times lower, and nothing else says so."""
    global _fallbacks_seen, _fallback_warned
    n = lib.bnb_auto_fallback_count()
    if n != _fallbacks_seen:
        _fallbacks_seen = n
        if not _fallback_warned:
            _fallback_warned = True
            import warnings

            warnings.warn(
                f"{what}: this bfloat16 call runs on the exact (SIMT) kernels, not the fused tensor-core kernels, "
                "because they are not built for its shape (d_model 128 with 4 heads, at most 512 tokens per "
                "environment); bnb_auto_fallback_count() counts such calls", RuntimeWarning, stacklevel=3)


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(
            f"{what} is on {t.device}; the trunk kernels run on CUDA only (sm_100a) and have no CPU path"
        )


def f32c(t: torch.Tensor) -> torch.Tensor:
    """float32, contiguous view or copy of t."""
    if t.dtype != torch.float32:
        t = t.float()
    return t if t.is_contiguous() else t.contiguous()


def u8(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """One byte per element view of a bool tensor (or a converted copy)."""
    if t is None:
        return None
    if t.dtype == torch.bool:
        t = t if t.is_contiguous() else t.contiguous()
        return t.view(torch.uint8)
    return (t != 0).contiguous().view(torch.uint8)


def current_precision(device: torch.device) -> int:
    """BNB_BF16 inside torch.autocast(device, bfloat16), else BNB_FP32."""
    if torch.is_autocast_enabled(device.type):
        dt = torch.get_autocast_dtype(device.type)
        if dt != torch.bfloat16:
            raise RuntimeError(f"autocast dtype {dt} is not supported by the trunk kernels (bfloat16 only)")
        return BNB_BF16
    return BNB_FP32


def stream_handle(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_scratch: dict[tuple[int, int], torch.Tensor] = {}
# Scratch buffers that were outgrown.  They are never freed: launches still in flight on their
# stream, and CUDA graphs captured while they were current, hold their address.
_scratch_outgrown: list[torch.Tensor] = []
_alloc_worker = None


def persistent_bytes(device: torch.device, nbytes: int) -> torch.Tensor:
    """A byte buffer that outlives the call that creates it (scratch, weight images).

    It is allocated on a helper thread: torch.compile's CUDA-graph trees route every allocation
    made by the *calling* thread, during warm-up as well as capture, into the graph's private
    pool and insist that nothing in that pool survives the call; allocations of other threads
    stay in the ordinary pool.  The buffers are only ever used by work enqueued after their
    creation, and they are created before the first capture (the warm-up call needs them).
    """
    global _alloc_worker
    if _alloc_worker is None:
        import concurrent.futures

        _alloc_worker = concurrent.futures.ThreadPoolExecutor(max_workers=1, thread_name_prefix="bnb-alloc")

    def make() -> torch.Tensor:
        with torch.cuda.device(device):
            return torch.empty(nbytes, dtype=torch.uint8, device=device)

    return _alloc_worker.submit(make).result()


def scratch_for(device: torch.device, nbytes: int) -> torch.Tensor:
    """A scratch buffer owned by torch's allocator, grown on demand, one per device and stream."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream_handle(device))
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            _scratch_outgrown.append(buf)
        # grow geometrically, so that a run settles on a few buffers however its batch sizes vary
        want = max(nbytes, 1 << 20, 0 if buf is None else 2 * buf.numel() if 2 * buf.numel() < (8 << 30) else 0)
        buf = persistent_bytes(device, want)
        _scratch[key] = buf
    return buf


class BulletArgs:
    """The bullet tokens of a call in the form the C ABI takes, or ``None`` for a call without.

    ``bullets`` (E, NB, D) float and ``bullet_mask`` (E, NB) bool | None, E = the number of
    environments of the call (T*B for a sequence); models/yemong/attention.py:85-87.
    Holds the converted tensors so they outlive the asynchronous launch.
    """

    def __init__(self, bullets: Optional[torch.Tensor], bullet_mask: Optional[torch.Tensor], n_envs: int, d_model: int,
                 keep_bf16: bool = False):
        self.struct = None
        self.is_bf16 = False
        self.per_env = 0
        if bullets is None:
            return
        if bullets.dim() != 3 or bullets.shape[0] != n_envs or bullets.shape[2] != d_model or bullets.shape[1] < 1:
            raise RuntimeError(f"bullets must have shape ({n_envs}, NB >= 1, {d_model}), got {tuple(bullets.shape)}")
        require_cuda(bullets, "bullets")
        if bullet_mask is not None and tuple(bullet_mask.shape) != tuple(bullets.shape[:2]):
            raise RuntimeError(f"bullet_mask must have shape {tuple(bullets.shape[:2])}, got {tuple(bullet_mask.shape)}")
        # bfloat16 tokens (the BulletEncoder's output under CUDA autocast) go in as they are when the
        # caller knows the tensor-core kernels serve the call; anything else as float32
        self.is_bf16 = keep_bf16 and bullets.dtype == torch.bfloat16
        self.tokens = (bullets if bullets.is_contiguous() else bullets.contiguous()) if self.is_bf16 else f32c(bullets)
        self.active = u8(bullet_mask)
        self.per_env = int(bullets.shape[1])
        self.struct = Bullets(self.tokens.data_ptr(), ptr(self.active), self.per_env, 1 if self.is_bf16 else 0)

    @property
    def arg(self):
        return None if self.struct is None else C.byref(self.struct)


def uniform_batch(n_envs: int, tokens: int, ships: int) -> Batch:
    return Batch(n_envs, tokens, ships, tokens, n_envs * tokens, n_envs * ships, None, None, None, None, 0)


def tensor_engine_status(device: torch.device) -> int:
    """Status word the tensor-core kernels left in the scratch buffer of the current stream
    (0 = every bounded wait completed).  Synchronises; meant for tests and debugging."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream_handle(device))
    buf = _scratch.get(key)
    if buf is None:
        return 0
    torch.cuda.synchronize(device)
    return int(buf[:4].view(torch.int32).item())
