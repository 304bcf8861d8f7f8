"""Griffin temporal sublayer and Yemong block, mirroring ``models/yemong/griffin.py``.

Constructor arguments, sub-module names, parameter names/shapes/dtype and method
signatures follow the reference (griffin.py:160-167, 236-247, 335-368, 376-385, 419-429).
The arithmetic runs in the CUDA library: ``bnb_temporal_block_fwd`` for a temporal
sublayer, ``bnb_trunk_step`` / ``bnb_trunk_sequence`` (with one block) for a Yemong block.
"""

from __future__ import annotations

import os

import torch
import torch.nn as nn

from .. import _capi
from . import _ops
from ._weights import packed_image, spatial_tensors, temporal_struct, temporal_tensors
from .attention import GatedMLP, TransformerBlock

CONV_KERNEL: int = 4  # causal depthwise conv kernel size (griffin.py:22)


def _no_grad_inputs(*tensors) -> None:
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors):
        raise NotImplementedError("this method is forward-only (gradients flow through YemongBlock / YemongTrunk "
                                  "step and sequence); call it under torch.no_grad()")


class RGLRU(nn.Module):
    """Real-Gated Linear Recurrent Unit (griffin.py:143-219).

    r = sigmoid(W_a x + b_a), i = sigmoid(W_x x + b_x), a = sigmoid(Lambda)^(c r),
    h = a h + sqrt(1 - a^2) (i x).  Inside a temporal sublayer the update runs fused in the
    temporal kernels; ``_step`` and ``forward_sequence`` serve callers that use the unit on its own
    (the reference's tests do) through ``bnb_rglru_fwd``.
    """

    def __init__(self, d_model: int, c: float = 8.0) -> None:
        super().__init__()
        if c != 8.0:
            raise ValueError("the CUDA RG-LRU is built for c = 8 (the reference's only value)")
        self.c = c
        self.d_model = d_model
        self.log_lambda = nn.Parameter(torch.linspace(0.0, 4.0, d_model))
        self.linear_a = nn.Linear(d_model, d_model, bias=True)
        self.linear_x = nn.Linear(d_model, d_model, bias=True)

    def _run(self, x_t: torch.Tensor, h0: torch.Tensor, done_t: torch.Tensor | None):
        """x_t (T, R, D) time-major float32 contiguous -> (states (T, R, D), final state (R, D))."""
        T, R, D = x_t.shape
        dev = x_t.device
        precision = _capi.current_precision(dev)
        ps = [self.linear_a.weight, self.linear_a.bias, self.linear_x.weight, self.linear_x.bias, self.log_lambda]
        for p in ps:
            if p.device != dev or p.dtype != torch.float32 or not p.is_contiguous():
                raise RuntimeError("RGLRU parameters must be contiguous float32 on the input's device")
        with torch.cuda.device(dev):
            h = _capi.f32c(h0)
            y = torch.empty_like(x_t)
            h_out = torch.empty_like(h)
            st = _capi.lib.bnb_rglru_fwd(*(p.data_ptr() for p in ps), D, x_t.data_ptr(), y.data_ptr(), h.data_ptr(),
                                         h_out.data_ptr(), _capi.ptr(done_t), R, T, precision, _capi.stream_handle(dev))
        _capi.check("bnb_rglru_fwd", st)
        return y, h_out

    def _check(self, x: torch.Tensor, h: torch.Tensor, dims: int) -> None:
        if x.dim() != dims or x.shape[-1] != self.d_model:
            raise RuntimeError(f"expected an input of {dims} dims ending in {self.d_model}, got {tuple(x.shape)}")
        if tuple(h.shape) != (x.shape[0], self.d_model):
            raise RuntimeError(f"expected a state of shape {(x.shape[0], self.d_model)}, got {tuple(h.shape)}")
        _capi.require_cuda(x, "x")
        _no_grad_inputs(x, h)

    def _step(self, x: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        """One step (griffin.py:169-186): x, h (B_seq, D) -> new h, which is also the output."""
        self._check(x, h, 2)
        _, h_out = self._run(_capi.f32c(x).unsqueeze(0), h, None)
        return h_out

    def forward_sequence(self, x_seq: torch.Tensor, h0: torch.Tensor, done_mask: torch.Tensor | None = None):
        """A full sequence (griffin.py:188-219): x_seq (B_seq, T, D), h0 (B_seq, D), done_mask
        (B_seq, T) bool (True at t cuts the state before step t + 1) -> (states (B_seq, T, D),
        final state (B_seq, D))."""
        self._check(x_seq, h0, 3)
        if done_mask is not None and tuple(done_mask.shape) != tuple(x_seq.shape[:2]):
            raise RuntimeError(f"done_mask must have shape {tuple(x_seq.shape[:2])}, got {tuple(done_mask.shape)}")
        x_t = _capi.f32c(x_seq.transpose(0, 1))
        done_t = None if done_mask is None else _capi.u8(done_mask.transpose(0, 1))
        y, h_out = self._run(x_t, h0, done_t)
        return y.transpose(0, 1).contiguous(), h_out


class GriffinTemporalBlock(nn.Module):
    """norm -> (linear1 -> causal conv -> RG-LRU) * GeLU(linear2) -> linear_out -> residual
    -> GatedMLP(norm) -> residual, applied per ship across time (griffin.py:222-286)."""

    def __init__(self, d_model: int) -> None:
        super().__init__()
        self.d_model = d_model
        self.norm1 = nn.RMSNorm(d_model)
        self.linear1 = nn.Linear(d_model, d_model, bias=False)
        self.conv = nn.Conv1d(d_model, d_model, kernel_size=CONV_KERNEL, groups=d_model, bias=True)
        self.rg_lru = RGLRU(d_model)
        self.linear2 = nn.Linear(d_model, d_model, bias=False)
        self.linear_out = nn.Linear(d_model, d_model, bias=False)
        self.norm2 = nn.RMSNorm(d_model)
        self.gated_mlp = GatedMLP(d_model)

    def _packed_ptr(self, sub, dev: torch.device, precision: int):
        return packed_image("temporal", temporal_tensors(self, sub), 4, dev, precision, _capi.ENGINE_AUTO)

    def forward_sequence(
        self,
        x_seq: torch.Tensor,  # (B_seq, T, D)
        h0: torch.Tensor,  # (B_seq, D)
        conv_buf: torch.Tensor,  # (B_seq, CONV_KERNEL-1, D)
        done_mask: torch.Tensor | None = None,  # (B_seq, T) bool
    ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Returns (out (B_seq, T, D), new_h (B_seq, D), new_conv_buf (B_seq, 3, D))."""
        D = self.d_model
        if x_seq.dim() != 3 or x_seq.shape[-1] != D:
            raise RuntimeError(f"expected x_seq of shape (B_seq, T, {D}), got {tuple(x_seq.shape)}")
        _capi.require_cuda(x_seq, "x_seq")
        _no_grad_inputs(x_seq, h0, conv_buf)
        R, T, _ = x_seq.shape
        if tuple(h0.shape) != (R, D) or tuple(conv_buf.shape) != (R, CONV_KERNEL - 1, D):
            raise RuntimeError("h0 / conv_buf shapes do not match x_seq")
        dev = x_seq.device
        precision = _capi.current_precision(dev)
        with torch.cuda.device(dev):
            x_t = _capi.f32c(x_seq.transpose(0, 1))  # (T, R, D), time-major for the kernel
            hidden = torch.cat([h0.float(), conv_buf.float().reshape(R, (CONV_KERNEL - 1) * D)], dim=-1).contiguous()
            done = None if done_mask is None else _capi.u8(done_mask.transpose(0, 1))
            y = torch.empty_like(x_t)
            new_hidden = torch.empty_like(hidden)
            batch = _capi.uniform_batch(R, 1, 1)  # every row is its own one-ship environment
            w = temporal_struct(self, None, dev, self._packed_ptr(None, dev, precision))
            scratch = _capi.scratch_for(dev, _capi.lib.bnb_scratch_bytes(D, batch, T, 0))
            st = _capi.lib.bnb_temporal_block_fwd(
                w, D, x_t.data_ptr(), y.data_ptr(), hidden.data_ptr(), new_hidden.data_ptr(), _capi.ptr(done),
                batch, T, precision, _capi.ENGINE_AUTO, scratch.data_ptr(), scratch.numel(), _capi.stream_handle(dev),
            )
        _capi.check("bnb_temporal_block_fwd", st)
        return (
            y.transpose(0, 1).contiguous(),
            new_hidden[:, :D].contiguous(),
            new_hidden[:, D:].reshape(R, CONV_KERNEL - 1, D),
        )

    def forward_nonrecurrent(self, x: torch.Tensor, sub: nn.Linear) -> torch.Tensor:
        """The block with conv + RG-LRU replaced by the Linear ``sub`` (griffin.py:288-317)."""
        D = self.d_model
        if x.shape[-1] != D:
            raise RuntimeError(f"expected x of shape (..., {D}), got {tuple(x.shape)}")
        _capi.require_cuda(x, "x")
        _no_grad_inputs(x)
        dev = x.device
        precision = _capi.current_precision(dev)
        with torch.cuda.device(dev):
            flat = _capi.f32c(x).reshape(-1, D)
            R = flat.shape[0]
            y = torch.empty_like(flat)
            batch = _capi.uniform_batch(R, 1, 0)  # every row is a field token
            w = temporal_struct(self, sub, dev, self._packed_ptr(sub, dev, precision))
            scratch = _capi.scratch_for(dev, _capi.lib.bnb_scratch_bytes(D, batch, 1, 0))
            st = _capi.lib.bnb_temporal_block_fwd(
                w, D, flat.data_ptr(), y.data_ptr(), None, None, None, batch, 1, precision, _capi.ENGINE_AUTO,
                scratch.data_ptr(), scratch.numel(), _capi.stream_handle(dev),
            )
        _capi.check("bnb_temporal_block_fwd", st)
        return y.reshape(x.shape)


def _keep(x: torch.Tensor, geom: list[int], n_bullets: int) -> bool:
    """Keep activations for the backward, or recompute them?  While a compiler traces the call the
    answer comes from BNB_GRAD_MODE alone (the memory query is a library call a tracer cannot see
    through); otherwise ``_ops.keep_activations`` also looks at the free memory."""
    if torch.compiler.is_compiling():
        return os.environ.get("BNB_GRAD_MODE", "") != "recompute" and 0 < geom[_ops.G_MAX_TOKENS]
    return _ops.keep_activations(x.device, geom, x.shape[-1], n_bullets)


def run_trunk(
    blocks,
    n_heads: int,
    x: torch.Tensor,
    alive: torch.Tensor | None,
    hidden: torch.Tensor,
    done: torch.Tensor | None,
    reset_env: torch.Tensor | None,
    batch_geom: list[int],
    timesteps: int | None,
    engine: int = _capi.ENGINE_AUTO,
    offsets: list[torch.Tensor] | None = None,
    bullets: torch.Tensor | None = None,
    bullet_mask: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Run ``blocks`` (YemongBlock modules of one structure) over x.

    x is (total_tokens, D) for a step (timesteps None) or (T, total_tokens, D) for a
    sequence; hidden is (L, total_ships, 4D) packed; ``batch_geom`` is the batch part of the
    operator's integer list (``_ops.uniform_geom`` for environments of one size), ``offsets``
    the device prefix sums of a ragged batch; bullets (T * n_envs, NB, D) and bullet_mask
    (T * n_envs, NB) feed the spatial sublayers that read them.  Returns (y, new_hidden).

    Everything below the parameter gathering happens inside the opaque operator
    ``bnb_b200::trunk_forward``, so ``torch.compile`` records one node for the whole trunk.
    """
    n_blocks = len(blocks)
    n_spatial = len(blocks[0].spatial) if n_blocks else 0
    n_temporal = len(blocks[0].temporal) if n_blocks else 0
    n_cross = sum(1 for sp in blocks[0].spatial if sp.reads_bullets) if n_blocks else 0
    has_fields = batch_geom[4] > batch_geom[5]          # total_tokens > total_ships
    weights: list[torch.Tensor] = []
    for blk in blocks:
        for sp in blk.spatial:
            weights += spatial_tensors(sp)
        for j, tp in enumerate(blk.temporal):
            weights += temporal_tensors(tp, blk.field_sub[j] if has_fields else None)
    geom = [n_blocks, n_spatial, n_temporal, n_heads, n_cross, 1 if has_fields else 0, *batch_geom,
            0 if timesteps is None else timesteps, engine, _capi.current_precision(x.device)]
    if (torch.is_grad_enabled() and not offsets and reset_env is None
            and (x.requires_grad or hidden.requires_grad or (bullets is not None and bullets.requires_grad)
                 or any(w.requires_grad for w in weights))
            and _keep(x, geom, bullets.shape[1] if n_cross and bullets is not None else 0)):
        # a call that will be differentiated: the forward that keeps its activations for the backward
        y, nh, _ = _ops.trunk_forward_train(x, alive, hidden, done, bullets if n_cross else None,
                                            bullet_mask if n_cross else None, weights, geom)
        return y, nh
    return _ops.trunk_forward(x, alive, hidden, done, reset_env, bullets if n_cross else None,
                              bullet_mask if n_cross else None, weights, offsets or [], geom)


class YemongBlock(nn.Module):
    """Spatial sublayers followed by temporal sublayers (griffin.py:320-368)."""

    def __init__(self, model_config) -> None:
        super().__init__()
        self.d_model = model_config.d_model
        self.n_heads = model_config.n_heads
        self.spatial = nn.ModuleList(
            [
                TransformerBlock(model_config, reads_bullets=i < model_config.n_bullet_cross_per_block)
                for i in range(model_config.n_spatial_per_block)
            ]
        )
        self.temporal = nn.ModuleList(
            [GriffinTemporalBlock(model_config.d_model) for _ in range(model_config.n_temporal_per_block)]
        )
        self.field_sub = nn.ModuleList(
            [
                nn.Linear(model_config.d_model, model_config.d_model, bias=False)
                for _ in range(model_config.n_temporal_per_block)
            ]
        )
        for sub in self.field_sub:
            nn.init.eye_(sub.weight)

    @property
    def n_temporal(self) -> int:
        """Hidden-state slots this block consumes."""
        return len(self.temporal)

    @staticmethod
    def _pack_state(h: torch.Tensor, conv_buf: torch.Tensor) -> torch.Tensor:
        L, R, D = h.shape
        return torch.cat([h.float(), conv_buf.float().reshape(L, R, (CONV_KERNEL - 1) * D)], dim=-1).contiguous()

    def step(
        self,
        x: torch.Tensor,  # (B, N+M, D)
        alive: torch.Tensor,  # (B, N+M) bool
        h: torch.Tensor,  # (n_temporal, B*N, D)
        conv_buf: torch.Tensor,  # (n_temporal, B*N, CONV_KERNEL-1, D)
        num_recurrent: int | None = None,
        bullets: torch.Tensor | None = None,
        bullet_mask: torch.Tensor | None = None,
    ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Single-step forward (griffin.py:376-417): returns (x, new_h, new_conv_buf)."""
        _capi.require_cuda(x, "x")
        B, NM, D = x.shape
        n_rec = NM if num_recurrent is None else num_recurrent
        batch = _ops.uniform_geom(B, NM, n_rec)
        hidden = self._pack_state(h, conv_buf)
        y, nh = run_trunk([self], self.n_heads, x.reshape(B * NM, D), None if alive is None else alive.reshape(-1),
                          hidden, None, None, batch, None, bullets=bullets, bullet_mask=bullet_mask)
        L, R = nh.shape[0], nh.shape[1]
        if L == 0:
            return y.reshape(B, NM, D), h[:0], conv_buf[:0]
        return y.reshape(B, NM, D), nh[:, :, :D].contiguous(), nh[:, :, D:].reshape(L, R, CONV_KERNEL - 1, D)

    def sequence(
        self,
        x: torch.Tensor,  # (T, B, N+M, D)
        alive_mask: torch.Tensor,  # (T, B, N+M) bool
        h0: torch.Tensor,  # (n_temporal, B*N, D)
        conv_buf0: torch.Tensor,  # (n_temporal, B*N, CONV_KERNEL-1, D)
        done_mask: torch.Tensor | None = None,  # (T, B) bool
        num_recurrent: int | None = None,
        bullets: torch.Tensor | None = None,
        bullet_mask: torch.Tensor | None = None,
    ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Full-sequence forward (griffin.py:419-472): returns (x, final h, final conv_buf)."""
        _capi.require_cuda(x, "x")
        T, B, NM, D = x.shape
        n_rec = NM if num_recurrent is None else num_recurrent
        batch = _ops.uniform_geom(B, NM, n_rec)
        hidden = self._pack_state(h0, conv_buf0)
        y, nh = run_trunk(
            [self], self.n_heads, x.reshape(T, B * NM, D), None if alive_mask is None else alive_mask.reshape(T, -1),
            hidden, done_mask, None, batch, T, bullets=bullets, bullet_mask=bullet_mask,
        )
        L, R = nh.shape[0], nh.shape[1]
        if L == 0:
            return y.reshape(T, B, NM, D), h0[:0], conv_buf0[:0]
        return (
            y.reshape(T, B, NM, D),
            nh[:, :, :D].contiguous(),
            nh[:, :, D:].reshape(L, R, CONV_KERNEL - 1, D),
        )
