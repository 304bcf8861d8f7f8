"""The trunk loop of ``YemongPolicy`` as one module.

``YemongTrunk`` owns ``yemong_layers`` (same attribute name and parameter names as the
policy, models/yemong/policy.py:183-187) and replaces, with one C-ABI call each,

* the trunk loop + hidden unpack/repack of ``get_action_and_value`` (policy.py:315-354),
* the trunk loop of ``evaluate_actions`` (policy.py:422-478),
* ``reset_hidden_for_envs`` (policy.py:268-285) and ``initial_hidden`` (234-254).

The hidden layout is the policy's: (n_layers, B*N, CONV_KERNEL*D) float32, row
``env*N + ship``, ``[..., :D]`` the RG-LRU state and ``[..., D:]`` the three stored
linear1 outputs oldest first (policy.py:27-34).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from .. import _capi
from . import _ops
from .griffin import CONV_KERNEL, YemongBlock, run_trunk


@dataclass
class RaggedBatch:
    """Environments of different sizes packed env-major.

    ``n_tokens[e]`` tokens per environment, the first ``n_ships[e]`` of them ships.  Token
    rows of x and hidden rows follow each other environment by environment.
    """

    n_tokens: torch.Tensor  # (B,) int, host or device
    n_ships: torch.Tensor  # (B,) int

    def build(self, device: torch.device) -> tuple[list[int], list[torch.Tensor]]:
        """Batch integers (the ``_ops`` geometry entries) and the device prefix sums / tile plan."""
        nt = self.n_tokens.to("cpu", torch.int64)
        ns = self.n_ships.to("cpu", torch.int64)
        if nt.shape != ns.shape or nt.dim() != 1:
            raise RuntimeError("n_tokens and n_ships must be 1-D tensors of equal length")
        if bool((ns > nt).any()) or bool((ns < 0).any()):
            raise RuntimeError("each environment needs 0 <= n_ships <= n_tokens")
        B = nt.numel()
        tok_off = torch.zeros(B + 1, dtype=torch.int32)
        ship_off = torch.zeros(B + 1, dtype=torch.int32)
        tok_off[1:] = nt.cumsum(0)
        ship_off[1:] = ns.cumsum(0)
        tok_d = tok_off.to(device)
        ship_d = ship_off.to(device)
        # tile plan for the tensor-core engine (environments of at most 128 tokens only)
        tiles_d, ids_d, n_tiles = None, None, 0
        if B and int(nt.max()) <= 128 and int(nt.min()) >= 1:
            plan = torch.zeros(B + 1, dtype=torch.int32)
            ids = torch.zeros(B, dtype=torch.int32)
            n = _capi.C.c_int(0)
            st = _capi.lib.bnb_plan_tiles(tok_off.data_ptr(), B, plan.data_ptr(), ids.data_ptr(), B + 1, _capi.C.byref(n))
            _capi.check("bnb_plan_tiles", st)
            n_tiles = n.value
            tiles_d = plan[: n_tiles + 1].to(device)
            ids_d = ids.to(device)
        geom = [B, 0, 0, int(nt.max()) if B else 0, int(tok_off[-1]), int(ship_off[-1]), n_tiles]
        self.tile_fill = float(tok_off[-1]) / (128.0 * n_tiles) if n_tiles else 0.0
        offsets = [tok_d, ship_d] + ([tiles_d, ids_d] if tiles_d is not None else [])
        return geom, offsets


class YemongTrunk(nn.Module):
    """``n_yemong_blocks`` Yemong blocks applied in order, with the policy's packed state."""

    def __init__(self, model_config) -> None:
        super().__init__()
        self.d_model = model_config.d_model
        self.n_heads = model_config.n_heads
        self.n_temporal = model_config.n_temporal_per_block
        self.yemong_layers = nn.ModuleList([YemongBlock(model_config) for _ in range(model_config.n_yemong_blocks)])

    @property
    def n_hidden_layers(self) -> int:
        return len(self.yemong_layers) * self.n_temporal

    def initial_hidden(self, num_envs: int, num_recurrent_tokens: int, device: torch.device) -> torch.Tensor:
        return torch.zeros(self.n_hidden_layers, num_envs * num_recurrent_tokens, CONV_KERNEL * self.d_model, device=device)

    def reset_hidden_for_envs(self, hidden: torch.Tensor, done_mask: torch.Tensor, num_recurrent_tokens: int) -> torch.Tensor:
        """Zero the state of every recurrent token of finished environments (policy.py:268-285)."""
        _capi.require_cuda(hidden, "hidden")
        L, R, W = hidden.shape
        B = done_mask.shape[0]
        if R != B * num_recurrent_tokens or W != CONV_KERNEL * self.d_model:
            raise RuntimeError("hidden shape does not match done_mask / num_recurrent_tokens")
        dev = hidden.device
        with torch.cuda.device(dev):
            hin = _capi.f32c(hidden)
            out = torch.empty_like(hin)
            batch = _capi.uniform_batch(B, num_recurrent_tokens, num_recurrent_tokens)
            done = _capi.u8(done_mask)
            st = _capi.lib.bnb_reset_hidden(hin.data_ptr(), out.data_ptr(), done.data_ptr(), L, self.d_model, batch,
                                            _capi.stream_handle(dev))
        _capi.check("bnb_reset_hidden", st)
        return out

    def _check(self, x: torch.Tensor, hidden: torch.Tensor) -> None:
        _capi.require_cuda(x, "x")
        if x.shape[-1] != self.d_model:
            raise RuntimeError(f"expected last dim {self.d_model}, got {tuple(x.shape)}")
        if hidden.dim() != 3 or hidden.shape[0] != self.n_hidden_layers or hidden.shape[2] != CONV_KERNEL * self.d_model:
            raise RuntimeError(
                f"hidden must be ({self.n_hidden_layers}, B*N, {CONV_KERNEL * self.d_model}), got {tuple(hidden.shape)}"
            )

    @staticmethod
    def _check_mask(mask: torch.Tensor | None, shape: tuple, what: str) -> None:
        """Masks are read on the device one byte per element: a short one would be read out of bounds."""
        if mask is not None and tuple(mask.shape) != tuple(shape):
            raise RuntimeError(f"{what} must have shape {tuple(shape)}, got {tuple(mask.shape)}")

    def step(
        self,
        x: torch.Tensor,  # (B, N+M, D)
        alive: torch.Tensor | None,  # (B, N+M) bool
        hidden: torch.Tensor,  # (n_layers, B*N, 4D)
        reset_env: torch.Tensor | None = None,  # (B,) bool: treat incoming state as zero
        engine: int = _capi.ENGINE_AUTO,
        bullets: torch.Tensor | None = None,  # (B, NB, D) encoded bullet tokens
        bullet_mask: torch.Tensor | None = None,  # (B, NB) bool active slots
    ) -> tuple[torch.Tensor, torch.Tensor]:
        """One rollout step of the trunk: returns (x_out (B, N+M, D), new_hidden)."""
        self._check(x, hidden)
        B, NM, D = x.shape
        n_rec = hidden.shape[1] // B if self.n_hidden_layers else NM
        if self.n_hidden_layers and (hidden.shape[1] != B * n_rec or n_rec > NM):
            raise RuntimeError(f"hidden has {hidden.shape[1]} rows: not a multiple of the {B} environments, or more than their tokens")
        self._check_mask(alive, (B, NM), "alive")
        self._check_mask(reset_env, (B,), "reset_env")
        batch = _ops.uniform_geom(B, NM, n_rec)
        y, nh = run_trunk(list(self.yemong_layers), self.n_heads, x.reshape(B * NM, D),
                          None if alive is None else alive.reshape(-1), hidden, None, reset_env, batch, None, engine,
                          bullets=bullets, bullet_mask=bullet_mask)
        return y.reshape(B, NM, D), nh

    def sequence(
        self,
        x: torch.Tensor,  # (T, B, N+M, D)
        alive_mask: torch.Tensor | None,  # (T, B, N+M) bool
        initial_hidden: torch.Tensor,  # (n_layers, B*N, 4D)
        done_mask: torch.Tensor | None = None,  # (T, B) bool
        engine: int = _capi.ENGINE_AUTO,
        bullets: torch.Tensor | None = None,  # (T*B, NB, D) encoded bullet tokens
        bullet_mask: torch.Tensor | None = None,  # (T*B, NB) bool active slots
    ) -> tuple[torch.Tensor, torch.Tensor]:
        """The trunk over T timesteps from one initial state: returns (x_out, final_hidden)."""
        self._check(x, initial_hidden)
        T, B, NM, D = x.shape
        n_rec = initial_hidden.shape[1] // B if self.n_hidden_layers else NM
        if self.n_hidden_layers and (initial_hidden.shape[1] != B * n_rec or n_rec > NM):
            raise RuntimeError(f"initial_hidden has {initial_hidden.shape[1]} rows: not a multiple of the {B} environments, or more than their tokens")
        self._check_mask(alive_mask, (T, B, NM), "alive_mask")
        self._check_mask(done_mask, (T, B), "done_mask")
        batch = _ops.uniform_geom(B, NM, n_rec)
        y, nh = run_trunk(list(self.yemong_layers), self.n_heads, x.reshape(T, B * NM, D),
                          None if alive_mask is None else alive_mask.reshape(T, -1), initial_hidden, done_mask, None,
                          batch, T, engine, bullets=bullets, bullet_mask=bullet_mask)
        return y.reshape(T, B, NM, D), nh

    def step_ragged(
        self,
        x: torch.Tensor,  # (sum tokens, D)
        alive: torch.Tensor | None,  # (sum tokens,) bool
        hidden: torch.Tensor,  # (n_layers, sum ships, 4D)
        ragged: RaggedBatch,
        engine: int = _capi.ENGINE_AUTO,
        bullets: torch.Tensor | None = None,  # (B, NB, D): the same ring size in every environment
        bullet_mask: torch.Tensor | None = None,  # (B, NB) bool
    ) -> tuple[torch.Tensor, torch.Tensor]:
        """One step over environments of different sizes (ships first, then fields, per env)."""
        self._check(x, hidden)
        batch, offsets = ragged.build(x.device)
        if x.dim() != 2 or x.shape[0] != batch[4] or hidden.shape[1] != batch[5]:
            raise RuntimeError("x / hidden rows do not match the ragged batch")
        self._check_mask(alive, (batch[4],), "alive")
        y, nh = run_trunk(list(self.yemong_layers), self.n_heads, x, alive, hidden, None, None, batch, None, engine,
                          offsets=offsets, bullets=bullets, bullet_mask=bullet_mask)
        return y, nh
