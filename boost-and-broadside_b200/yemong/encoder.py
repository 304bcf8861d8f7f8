"""Token encoders in front of the trunk, mirroring the reference's ``models/yemong/encoder.py``.

``ShipEncoder`` and ``BulletEncoder`` keep the reference's constructor arguments, sub-module names
and parameter shapes (encoder.py:41-51, 73-102), so a reference ``state_dict`` loads unchanged.  The
``FeatureCoordinator`` that turns an observation into raw per-entity vectors is the caller's object
and runs as it is (torch operators on the observation's device); the MLP chain behind it --
Linear, RMSNorm, GELU, Linear, RMSNorm -- runs in one kernel, ``bnb_encoder_mlp_fwd``.

Under ``torch.autocast(bfloat16)`` the encoders return bfloat16 tokens, as the reference's do (its
chain ends in an RMSNorm of a bf16 Linear output); ``YemongBlock`` / ``YemongTrunk`` take those
without a float32 copy.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .. import _capi
from . import _end_ops


def _encoder_chain(raw: torch.Tensor, lin1: nn.Linear, norm1: nn.RMSNorm, lin2: nn.Linear, norm2: nn.RMSNorm) -> torch.Tensor:
    """norm2(lin2(gelu(norm1(lin1(raw))))) over the last dim of ``raw`` through the C ABI
    (one opaque operator, ``bnb_b200::mlp_chain``)."""
    _capi.require_cuda(raw, "the raw feature vector")
    in_dim, out_dim = lin1.in_features, lin2.out_features
    if raw.shape[-1] != in_dim:
        raise RuntimeError(f"expected raw features of width {in_dim}, got {tuple(raw.shape)}")
    precision = _capi.current_precision(raw.device)
    y = _end_ops.mlp_chain(raw.reshape(-1, in_dim), lin1.weight, lin1.bias, norm1.weight, lin2.weight, lin2.bias, norm2.weight,
                           precision)
    return y.reshape(*raw.shape[:-1], out_dim)


def _no_grad(*tensors) -> None:
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors):
        raise NotImplementedError("the CUDA encoders are forward-only; call them under torch.no_grad()")


class BulletEncoder(nn.Module):
    """Raw bullet channels -> d_model tokens (encoder.py:25-55)."""

    def __init__(self, model_config, coordinator) -> None:
        super().__init__()
        self.coordinator = coordinator
        hidden = model_config.bullet_encoder_hidden
        self.net = nn.Sequential(
            nn.Linear(coordinator.total_input_dimension, hidden),
            nn.RMSNorm(hidden),
            nn.GELU(),
            nn.Linear(hidden, model_config.d_model),
            nn.RMSNorm(model_config.d_model),
        )

    def encode_raw(self, raw: torch.Tensor) -> torch.Tensor:
        """``net`` on raw feature vectors (..., total_input_dimension) -> (..., d_model)."""
        _no_grad(raw)
        return _encoder_chain(raw, self.net[0], self.net[1], self.net[3], self.net[4])

    def forward(self, obs) -> torch.Tensor:
        """obs carrying bullet channels -> (..., N*K, d_model)."""
        return self.encode_raw(self.coordinator.get_input_vector(obs))


class ShipEncoder(nn.Module):
    """Each entity's raw observation channels -> a d_model token (encoder.py:58-130), in the
    shared layout (one chain for every token) or the split one (a first projection per entity
    type, a shared second one)."""

    def __init__(self, model_config, coordinator, num_ships: int | None = None) -> None:
        super().__init__()
        self.coordinator = coordinator
        self.split = model_config.encoder_split
        self.num_ships = num_ships
        D = model_config.d_model
        if not self.split:
            self.feature_extractor = nn.Sequential(
                nn.Linear(coordinator.total_input_dimension, 2 * D),
                nn.RMSNorm(2 * D),
                nn.GELU(),
                nn.Linear(2 * D, D),
                nn.RMSNorm(D),
            )
            return
        if num_ships is None:
            raise ValueError("encoder_split requires num_ships to locate the ship/field boundary")
        scope = _feature_scope(coordinator)
        ship_dim = coordinator.scoped_input_dimension(scope.SHIP)
        field_dim = coordinator.scoped_input_dimension(scope.FIELD)
        self.ship_proj = nn.Sequential(nn.Linear(ship_dim, 2 * D), nn.RMSNorm(2 * D), nn.GELU())
        self.field_proj = nn.Sequential(nn.Linear(field_dim, 2 * D), nn.RMSNorm(2 * D), nn.GELU())
        self.shared_proj = nn.Sequential(nn.Linear(2 * D, D), nn.RMSNorm(D))

    def encode_raw(self, raw: torch.Tensor, field_raw: torch.Tensor | None = None) -> torch.Tensor:
        """The MLP chain on raw feature vectors.  Shared layout: ``raw`` (..., N+M, width).  Split
        layout: ``raw`` holds the ship vectors (..., N, ship width) and ``field_raw`` the field
        vectors (..., M, field width) or None; the result is their tokens, ships first."""
        _no_grad(raw, field_raw)
        if not self.split:
            fx = self.feature_extractor
            return _encoder_chain(raw, fx[0], fx[1], fx[3], fx[4])
        out = _encoder_chain(raw, self.ship_proj[0], self.ship_proj[1], self.shared_proj[0], self.shared_proj[1])
        if field_raw is not None and field_raw.shape[-2] > 0:
            f = _encoder_chain(field_raw, self.field_proj[0], self.field_proj[1], self.shared_proj[0], self.shared_proj[1])
            out = torch.cat([out, f], dim=-2)
        return out

    def forward(self, obs) -> torch.Tensor:
        """YemongObservation -> (..., N+M, d_model) tokens."""
        if not self.split:
            return self.encode_raw(self.coordinator.get_input_vector(obs))
        scope = _feature_scope(self.coordinator)
        n, total = self.num_ships, obs.pos.shape[-2]
        ship_raw = self.coordinator.get_scoped_input_vector(obs.slice_tokens(0, n), scope.SHIP)
        field_raw = None
        if total > n:
            field_raw = self.coordinator.get_scoped_input_vector(obs.slice_tokens(n, total), scope.FIELD)
        return self.encode_raw(ship_raw, field_raw)


def _feature_scope(coordinator):
    """The ``FeatureScope`` enum of the coordinator's own module (train/rl/features.py): the
    coordinator is the caller's object, so its enum is looked up next to its class."""
    import sys

    return getattr(sys.modules[type(coordinator).__module__], "FeatureScope")
