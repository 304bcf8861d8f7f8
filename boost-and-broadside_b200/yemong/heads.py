"""Output heads behind the trunk, mirroring the reference's ``models/yemong/policy.py``.

``TeamPMA`` (policy.py:78-121) pools each team's alive ships with a learned seed
(``bnb_team_pma_fwd``).  The policy's four heads -- ``action_head``, ``value_head_local``, ``value_head_win``
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
from . import _end_ops


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
        in_dim, out_dim = lin1.in_features, lin2.out_features
        if x.shape[-1] != in_dim:
            raise RuntimeError(f"expected tokens of width {in_dim}, got {tuple(x.shape)}")
        y = _end_ops.mlp_chain(x.reshape(-1, in_dim), lin1.weight, lin1.bias, norm.weight, lin2.weight, lin2.bias, None,
                               _capi.current_precision(x.device))
        return y.reshape(*x.shape[:-1], out_dim)


class NextStateHead(nn.Module):
    """Next-state deltas and absolutes per ship (policy.py:56-75): ``net`` is a ``HeadMLP``."""

    def __init__(self, d_model: int, pred_dim: int) -> None:
        super().__init__()
        self.pred_dim = pred_dim
        self.net = HeadMLP(d_model, pred_dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.net(x)


class TeamPMA(nn.Module):
    """Pooling by multi-head attention over per-team ship embeddings (policy.py:78-121): for each
    team a learned seed attends over that team's alive ships; every ship receives its team's pooled,
    normed embedding.  Same sub-modules and parameter names as the reference (``seeds``,
    ``attn.in_proj_weight``, ``attn.out_proj.weight``, ``norm.weight``); ``attn`` only holds the
    parameters here, the arithmetic runs in ``bnb_team_pma_fwd``."""

    def __init__(self, d_model: int, n_heads: int) -> None:
        super().__init__()
        self.d_model = d_model
        self.n_heads = n_heads
        self.seeds = nn.Parameter(torch.zeros(2, d_model))
        self.attn = nn.MultiheadAttention(d_model, n_heads, batch_first=True, bias=False)
        self.norm = nn.RMSNorm(d_model)

    def forward(self, x: torch.Tensor, team_id: torch.Tensor, alive: torch.Tensor) -> torch.Tensor:
        """x (B, N, D), team_id (B, N) int, alive (B, N) bool -> (B, N, D) in x's dtype."""
        if torch.is_grad_enabled() and x.requires_grad:
            raise NotImplementedError("the CUDA TeamPMA is forward-only; call it under torch.no_grad()")
        _capi.require_cuda(x, "x")
        if x.dim() != 3 or x.shape[-1] != self.d_model:
            raise RuntimeError(f"expected x of shape (B, N, {self.d_model}), got {tuple(x.shape)}")
        B, N, D = x.shape
        if tuple(team_id.shape) != (B, N) or tuple(alive.shape) != (B, N):
            raise RuntimeError(f"team_id and alive must have shape {(B, N)}")
        return _end_ops.team_pma(x, team_id, alive, self.seeds, self.attn.in_proj_weight, self.attn.out_proj.weight,
                                 self.norm.weight, self.n_heads, _capi.current_precision(x.device))


def _action_dist(logits: torch.Tensor, given: torch.Tensor | None, want_entropy: bool, generator=None):
    if torch.is_grad_enabled() and logits.requires_grad:
        raise NotImplementedError("the CUDA action distribution is forward-only; call it under torch.no_grad()")
    _capi.require_cuda(logits, "logits")
    if logits.shape[-1] != 12:
        raise RuntimeError(f"expected 12 action logits in the last dim, got {tuple(logits.shape)}")
    dev = logits.device
    lead = logits.shape[:-1]
    flat = logits.reshape(-1, 12)
    if given is None:
        uniforms = torch.rand(flat.shape[0], 3, device=dev, generator=generator)
        g = None
    else:
        if tuple(given.shape) != (*lead, 3):
            raise RuntimeError(f"actions must have shape {(*lead, 3)}, got {tuple(given.shape)}")
        uniforms = None
        g = given.reshape(-1, 3)
    action, logprob, entropy = _end_ops.action_dist(flat, uniforms, g, want_entropy)
    out_dtype = logits.dtype if logits.dtype == torch.bfloat16 else torch.float32
    logprob = logprob.reshape(lead).to(out_dtype)
    entropy = entropy.reshape(lead).to(out_dtype) if want_entropy else None
    return (action.reshape(*lead, 3) if given is None else None), logprob, entropy


def sample_action(logits: torch.Tensor, generator: torch.Generator | None = None):
    """``_sample_action`` (policy.py:551-575): logits (..., 12) -> (action (..., 3) int64, logprob (...)).
    The draws are inverse-CDF samples of uniforms from ``torch.rand`` on the device (the caller's
    generator): the same distribution as the reference's, not the same random stream."""
    action, logprob, _ = _action_dist(logits, None, False, generator)
    return action, logprob


def evaluate_action(logits: torch.Tensor, actions: torch.Tensor):
    """``_evaluate_action`` (policy.py:578-602), forward only: (logprob (...), entropy (...))."""
    _, logprob, entropy = _action_dist(logits, actions, True)
    return logprob, entropy
