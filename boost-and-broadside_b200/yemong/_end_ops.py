"""Opaque ``torch.library`` operators for the ends of the policy step: the encoder / head MLP
chain, TeamPMA and the action distribution.

Same reason as ``_ops.py``: ``torch.compile(policy.get_action_and_value, mode="reduce-overhead")``
(how the reference runs its policy, train/rl/ppo.py:396-400) must see one opaque node per call
into the C ABI, with a shape-only fake implementation, so that the FeatureCoordinator's torch
operators around them are fused by the compiler and the whole step replays as one CUDA graph.
All of them are forward-only.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

from .. import _capi


def _out_dtype(precision: int) -> torch.dtype:
    return torch.bfloat16 if precision == _capi.BNB_BF16 else torch.float32


def _check_params(dev: torch.device, what: str, *ps: Optional[Tensor]) -> None:
    for p in ps:
        if p is not None and (p.device != dev or p.dtype != torch.float32 or not p.is_contiguous()):
            raise RuntimeError(f"{what} parameters must be contiguous float32 on the input's device")


@torch.library.custom_op("bnb_b200::mlp_chain", mutates_args=(), device_types="cuda")
def mlp_chain(x: Tensor, w1: Tensor, b1: Tensor, g1: Tensor, w2: Tensor, b2: Tensor, g2: Optional[Tensor],
              precision: int) -> Tensor:
    """Linear(w1, b1) -> RMSNorm(g1) -> GELU -> Linear(w2, b2) [-> RMSNorm(g2)] over the rows of
    x (rows, in): ``bnb_encoder_mlp_fwd`` with g2 (the encoders), ``bnb_head_mlp_fwd`` without (the
    heads).  Returns (rows, out), bfloat16 under the bfloat16 contract, else float32.  The weights
    are zero-padded to the kernels' multiples of 32 here, from the live parameters, on every call."""
    dev = x.device
    in_dim, hidden, out_dim = w1.shape[1], w1.shape[0], w2.shape[0]
    with torch.cuda.device(dev):
        # a head fed bfloat16 tokens under the bfloat16 contract reads them as they are
        x16 = g2 is None and precision == _capi.BNB_BF16 and x.dtype == torch.bfloat16 and in_dim % 32 == 0
        flat = (x if x.is_contiguous() else x.contiguous()) if x16 else _capi.f32c(x)
        rows = flat.shape[0]
        y = torch.empty(rows, out_dim, device=dev, dtype=_out_dtype(precision))
        if g2 is not None:
            in_pad = (in_dim + 31) // 32 * 32
            w1p = w1.detach()
            if in_pad != in_dim:
                w1p = torch.nn.functional.pad(w1p, (0, in_pad - in_dim))
            w1p = w1p.contiguous()
            _check_params(dev, "encoder", w1p, b1, g1, w2, b2, g2)
            st = _capi.lib.bnb_encoder_mlp_fwd(w1p.data_ptr(), b1.data_ptr(), g1.data_ptr(), w2.data_ptr(), b2.data_ptr(),
                                               g2.data_ptr(), in_dim, in_pad, hidden, out_dim, flat.data_ptr(), y.data_ptr(),
                                               rows, precision, _capi.stream_handle(dev))
            _capi.check("bnb_encoder_mlp_fwd", st)
        else:
            out_pad = (out_dim + 31) // 32 * 32
            w2p = torch.nn.functional.pad(w2.detach(), (0, 0, 0, out_pad - out_dim)).contiguous()
            b2p = torch.nn.functional.pad(b2.detach(), (0, out_pad - out_dim)).contiguous()
            _check_params(dev, "head", w1, b1, g1, w2p, b2p)
            args = (w1.data_ptr(), b1.data_ptr(), g1.data_ptr(), w2p.data_ptr(), b2p.data_ptr(), in_dim, hidden, out_dim, out_pad)
            st = _capi.lib.bnb_head_mlp_fwd(*args, flat.data_ptr(), y.data_ptr(), rows, _capi.BNB_BF16_IO if x16 else precision,
                                            _capi.stream_handle(dev))
            if st == _capi.ERR_UNSUPPORTED_DIMS and x16:   # widths the tiled kernel does not serve: the float32-reading kernel
                flat = _capi.f32c(x)
                st = _capi.lib.bnb_head_mlp_fwd(*args, flat.data_ptr(), y.data_ptr(), rows, precision, _capi.stream_handle(dev))
            _capi.check("bnb_head_mlp_fwd", st)
    return y


@mlp_chain.register_fake
def _(x, w1, b1, g1, w2, b2, g2, precision):
    return x.new_empty((x.shape[0], w2.shape[0]), dtype=_out_dtype(precision))


@torch.library.custom_op("bnb_b200::team_pma", mutates_args=(), device_types="cuda")
def team_pma(x: Tensor, team_id: Tensor, alive: Tensor, seeds: Tensor, in_proj: Tensor, out_proj: Tensor, norm_w: Tensor,
             n_heads: int, precision: int) -> Tensor:
    """``bnb_team_pma_fwd``: x (B, N, D), team_id (B, N) int, alive (B, N) bool -> (B, N, D) in x's
    dtype when that is bfloat16, else float32."""
    dev = x.device
    B, N, D = x.shape
    _check_params(dev, "TeamPMA", seeds, in_proj, out_proj, norm_w)
    with torch.cuda.device(dev):
        xin = _capi.f32c(x)
        tid = team_id.to(torch.int32).contiguous()
        al = _capi.u8(alive)
        y = torch.empty(B, N, D, device=dev, dtype=torch.bfloat16 if x.dtype == torch.bfloat16 else torch.float32)
        nbytes = _capi.lib.bnb_team_pma_scratch_bytes(D, B, N)
        scratch = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=dev)
        st = _capi.lib.bnb_team_pma_fwd(seeds.data_ptr(), in_proj.data_ptr(), out_proj.data_ptr(), norm_w.data_ptr(), D, n_heads,
                                        xin.data_ptr(), tid.data_ptr(), al.data_ptr(), y.data_ptr(),
                                        1 if y.dtype == torch.bfloat16 else 0, B, N, precision, scratch.data_ptr(),
                                        scratch.numel(), _capi.stream_handle(dev))
    _capi.check("bnb_team_pma_fwd", st)
    return y


@team_pma.register_fake
def _(x, team_id, alive, seeds, in_proj, out_proj, norm_w, n_heads, precision):
    return x.new_empty(x.shape, dtype=torch.bfloat16 if x.dtype == torch.bfloat16 else torch.float32)


@torch.library.custom_op("bnb_b200::action_dist", mutates_args=(), device_types="cuda")
def action_dist(logits: Tensor, uniforms: Optional[Tensor], given: Optional[Tensor], want_entropy: bool) -> Tuple[Tensor, Tensor, Tensor]:
    """``bnb_action_dist_fwd`` over logits (R, 12): with ``uniforms`` (R, 3) draws an action per row
    by inverse CDF, with ``given`` (R, 3) int64 scores those actions.  Returns (action (R, 3) int64,
    logprob (R,), entropy (R,)), all float32 but the action; the action is empty when ``given`` was
    passed, the entropy is empty unless asked for."""
    dev = logits.device
    precision = _capi.BNB_BF16 if logits.dtype == torch.bfloat16 else _capi.BNB_FP32
    with torch.cuda.device(dev):
        flat = _capi.f32c(logits)
        R = flat.shape[0]
        logprob = torch.empty(R, device=dev, dtype=torch.float32)
        entropy = torch.empty(R if want_entropy else 0, device=dev, dtype=torch.float32)
        action = torch.empty(R if given is None else 0, 3, device=dev, dtype=torch.int64)
        g = None if given is None else given.to(torch.int64).contiguous()
        u = None if uniforms is None else _capi.f32c(uniforms)
        st = _capi.lib.bnb_action_dist_fwd(flat.data_ptr(), _capi.ptr(u), _capi.ptr(g), action.data_ptr() if given is None else None,
                                           logprob.data_ptr(), entropy.data_ptr() if want_entropy else None, R, precision,
                                           _capi.stream_handle(dev))
    _capi.check("bnb_action_dist_fwd", st)
    return action, logprob, entropy


@action_dist.register_fake
def _(logits, uniforms, given, want_entropy):
    R = logits.shape[0]
    return (logits.new_empty((R if given is None else 0, 3), dtype=torch.int64), logits.new_empty((R,), dtype=torch.float32),
            logits.new_empty((R if want_entropy else 0,), dtype=torch.float32))
