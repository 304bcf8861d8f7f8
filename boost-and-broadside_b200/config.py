"""The architecture fields the trunk reads, mirroring the reference's ``ModelConfig``
(config/core.py:213-275).  Any object with these attributes is accepted by the modules,
so the reference's own frozen dataclass can be passed unchanged."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class ModelConfig:
    d_model: int
    n_heads: int
    n_yemong_blocks: int
    n_spatial_per_block: int = 1
    n_temporal_per_block: int = 1
    encoder_split: bool = False
    n_bullet_cross_per_block: int = 0
    bullet_encoder_hidden: int = 64
    grad_checkpoint: bool = False

    @property
    def n_hidden_layers(self) -> int:
        return self.n_yemong_blocks * self.n_temporal_per_block

    @property
    def reads_bullets(self) -> bool:
        return self.n_bullet_cross_per_block > 0 and self.n_yemong_blocks > 0

    def __post_init__(self) -> None:
        if self.d_model % self.n_heads != 0:
            raise ValueError(f"d_model={self.d_model} must be divisible by n_heads={self.n_heads}")
        for name in ("n_yemong_blocks", "n_spatial_per_block", "n_temporal_per_block"):
            if getattr(self, name) < 0:
                raise ValueError(f"{name} must be >= 0, got {getattr(self, name)}")
        if not 0 <= self.n_bullet_cross_per_block <= self.n_spatial_per_block:
            raise ValueError(
                "n_bullet_cross_per_block must be between 0 and n_spatial_per_block "
                f"({self.n_spatial_per_block}), got {self.n_bullet_cross_per_block}"
            )
