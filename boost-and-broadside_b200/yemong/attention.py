"""Spatial transformer sublayer, mirroring the reference's ``models/yemong/attention.py``.

``GatedMLP`` and ``TransformerBlock`` keep the reference's constructor arguments,
parameter names, shapes and float32 dtype (attention.py:21-74), so a reference
``state_dict`` loads unchanged.  ``TransformerBlock.forward`` has the reference signature
(attention.py:76-82) and runs ``bnb_spatial_block_fwd`` of the CUDA library through the opaque
``bnb_b200::spatial_forward`` operator.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .. import _capi
from . import _ops
from ._weights import spatial_tensors


class GatedMLP(nn.Module):
    """down_proj(gelu(gate_proj(x)) * up_proj(x)), no biases (attention.py:21-37).

    Inside a sublayer the product runs fused in the sublayer kernels; ``forward`` serves callers
    that use the module on its own (the reference's tests do) through ``bnb_gated_mlp_fwd``.
    """

    def __init__(self, d_model: int, expand: int = 4) -> None:
        super().__init__()
        if expand != 4:
            raise ValueError("the CUDA GatedMLP is built for expand = 4 (the reference's only value)")
        hidden = expand * d_model
        self.d_model = d_model
        self.gate_proj = nn.Linear(d_model, hidden, bias=False)
        self.up_proj = nn.Linear(d_model, hidden, bias=False)
        self.down_proj = nn.Linear(hidden, d_model, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """(..., D) -> (..., D); bfloat16 inside ``torch.autocast`` (as the reference's last Linear
        returns it), else float32."""
        D = self.d_model
        if x.shape[-1] != D:
            raise RuntimeError(f"expected x of shape (..., {D}), got {tuple(x.shape)}")
        _capi.require_cuda(x, "x")
        if torch.is_grad_enabled() and x.requires_grad:
            raise NotImplementedError("the CUDA trunk is forward-only; call it under torch.no_grad()")
        dev = x.device
        precision = _capi.current_precision(dev)
        with torch.cuda.device(dev):
            flat = _capi.f32c(x).reshape(-1, D)
            y = torch.empty_like(flat)
            ws = [self.gate_proj.weight, self.up_proj.weight, self.down_proj.weight]
            for w in ws:
                if w.device != dev or w.dtype != torch.float32 or not w.is_contiguous():
                    raise RuntimeError("GatedMLP parameters must be contiguous float32 on the input's device")
            st = _capi.lib.bnb_gated_mlp_fwd(ws[0].data_ptr(), ws[1].data_ptr(), ws[2].data_ptr(), D, flat.data_ptr(),
                                             y.data_ptr(), flat.shape[0], precision, _capi.stream_handle(dev))
        _capi.check("bnb_gated_mlp_fwd", st)
        y = y.reshape(x.shape)
        return y.to(torch.bfloat16) if precision == _capi.BNB_BF16 else y


class TransformerBlock(nn.Module):
    """Pre-norm block: RMSNorm -> masked MHSA -> residual -> RMSNorm -> GatedMLP -> residual.

    Args:
        model_config: supplies ``d_model`` and ``n_heads``.
        reads_bullets: allocate the bullet key/value parameters (attention.py:64-71);
            such a block cross-attends to ``bullets`` when they are passed.
    """

    def __init__(self, model_config, reads_bullets: bool = False) -> None:
        super().__init__()
        D = model_config.d_model
        self.n_heads = model_config.n_heads
        self.head_dim = D // model_config.n_heads
        self.d_model = D
        self.reads_bullets = reads_bullets

        self.norm1 = nn.RMSNorm(D)
        self.qkv = nn.Linear(D, 3 * D, bias=False)
        self.out_proj = nn.Linear(D, D, bias=False)
        if reads_bullets:
            self.norm_bullet = nn.RMSNorm(D)
            self.kv_bullet = nn.Linear(D, 2 * D, bias=False)
        self.norm2 = nn.RMSNorm(D)
        self.ffn = GatedMLP(D)

    def forward(
        self,
        x: torch.Tensor,
        alive_mask: torch.Tensor | None = None,
        bullets: torch.Tensor | None = None,
        bullet_mask: torch.Tensor | None = None,
    ) -> torch.Tensor:
        """(B, N, D) -> (B, N, D); ``alive_mask`` (B, N) bool masks dead entities as keys.

        ``bullets`` (B, NB, D) are extra keys/values of a block built with ``reads_bullets``,
        ``bullet_mask`` (B, NB) bool marks the active ring-buffer slots (attention.py:149-166).
        """
        if x.dim() != 3 or x.shape[-1] != self.d_model:
            raise RuntimeError(f"expected x of shape (B, N, {self.d_model}), got {tuple(x.shape)}")
        _capi.require_cuda(x, "x")
        if torch.is_grad_enabled() and x.requires_grad:
            raise NotImplementedError("the CUDA trunk is forward-only; call it under torch.no_grad()")
        B, N, D = x.shape
        if alive_mask is not None and tuple(alive_mask.shape) != (B, N):
            raise RuntimeError(f"alive_mask must have shape {(B, N)}, got {tuple(alive_mask.shape)}")
        return _ops.spatial_forward(
            x, alive_mask, bullets if self.reads_bullets else None, bullet_mask if self.reads_bullets else None,
            spatial_tensors(self), self.n_heads, _capi.current_precision(x.device), _capi.ENGINE_AUTO,
        )
