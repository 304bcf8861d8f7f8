"""Output heads behind the trunk, mirroring the reference's ``models/yemong/policy.py``.

The policy's four heads -- ``action_head``, ``value_head_local``, ``value_head_win``
(policy.py:185-206) and ``NextStateHead.net`` (policy.py:56-72) -- are one shape:
``Sequential(Linear(D, 2D), RMSNorm(2D), GELU(), Linear(2D, out))``.  ``HeadMLP`` is that
``nn.Sequential`` with the same child indices (0, 1, 3 carry parameters), so the reference's
``state_dict`` entries load unchanged, and a forward that runs the whole chain in one kernel,
``bnb_head_mlp_fwd``.  Under ``torch.autocast(bfloat16)`` a head returns bfloat16, as the
reference's last Linear does.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .. import _capi


class HeadMLP(nn.Sequential):
    """Linear(d_model, 2*d_model) -> RMSNorm -> GELU -> Linear(2*d_model, out_dim)."""

    def __init__(self, d_model: int, out_dim: int) -> None:
        super().__init__(
            nn.Linear(d_model, 2 * d_model),
            nn.RMSNorm(2 * d_model),
            nn.GELU(),
            nn.Linear(2 * d_model, out_dim),
        )

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x (..., d_model) -> (..., out_dim)."""
        if torch.is_grad_enabled() and x.requires_grad:
            raise NotImplementedError("the CUDA heads are forward-only; call them under torch.no_grad()")
        _capi.require_cuda(x, "the head's input")
        lin1, norm, lin2 = self[0], self[1], self[3]
        dev = x.device
        in_dim, hidden, out_dim = lin1.in_features, lin1.out_features, lin2.out_features
        if x.shape[-1] != in_dim:
            raise RuntimeError(f"expected tokens of width {in_dim}, got {tuple(x.shape)}")
        precision = _capi.current_precision(dev)
        out_pad = (out_dim + 31) // 32 * 32
        with torch.cuda.device(dev):
            flat = _capi.f32c(x).reshape(-1, in_dim)
            # the second Linear with zero rows up to a multiple of 32 (a few KB, rebuilt per call
            # from the live parameters, so it cannot go stale)
            w2 = torch.nn.functional.pad(lin2.weight.detach(), (0, 0, 0, out_pad - out_dim)).contiguous()
            b2 = torch.nn.functional.pad(lin2.bias.detach(), (0, out_pad - out_dim)).contiguous()
            ps = [lin1.weight, lin1.bias, norm.weight, w2, b2]
            for p in ps:
                if p.device != dev or p.dtype != torch.float32 or not p.is_contiguous():
                    raise RuntimeError("head parameters must be contiguous float32 on the input's device")
            y = torch.empty(flat.shape[0], out_dim, device=dev,
                            dtype=torch.bfloat16 if precision == _capi.BNB_BF16 else torch.float32)
            st = _capi.lib.bnb_head_mlp_fwd(*(p.data_ptr() for p in ps), in_dim, hidden, out_dim, out_pad,
                                            flat.data_ptr(), y.data_ptr(), flat.shape[0], precision,
                                            _capi.stream_handle(dev))
        _capi.check("bnb_head_mlp_fwd", st)
        return y.reshape(*x.shape[:-1], out_dim)


class NextStateHead(nn.Module):
    """Next-state deltas and absolutes per ship (policy.py:56-75): ``net`` is a ``HeadMLP``."""

    def __init__(self, d_model: int, pred_dim: int) -> None:
        super().__init__()
        self.pred_dim = pred_dim
        self.net = HeadMLP(d_model, pred_dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.net(x)
