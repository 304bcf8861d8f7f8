"""Parameter pointer tables handed to the C ABI (BnbSpatialWeights / BnbTemporalWeights)."""

from __future__ import annotations

import torch

from .. import _capi


def _p(t: torch.Tensor, dev: torch.device, name: str) -> int:
    if t.device != dev:
        raise RuntimeError(f"parameter {name} is on {t.device}, input on {dev}")
    if t.dtype != torch.float32 or not t.is_contiguous():
        raise RuntimeError(f"parameter {name} must be contiguous float32 (got {t.dtype})")
    return t.data_ptr()


def spatial_struct(block, dev: torch.device, packed: int | None = None) -> _capi.SpatialWeights:
    return _capi.SpatialWeights(
        _p(block.norm1.weight, dev, "norm1.weight"),
        _p(block.qkv.weight, dev, "qkv.weight"),
        _p(block.out_proj.weight, dev, "out_proj.weight"),
        _p(block.norm2.weight, dev, "norm2.weight"),
        _p(block.ffn.gate_proj.weight, dev, "ffn.gate_proj.weight"),
        _p(block.ffn.up_proj.weight, dev, "ffn.up_proj.weight"),
        _p(block.ffn.down_proj.weight, dev, "ffn.down_proj.weight"),
        packed,
    )


def temporal_struct(tb, sub, dev: torch.device, packed: int | None = None) -> _capi.TemporalWeights:
    return _capi.TemporalWeights(
        _p(tb.norm1.weight, dev, "norm1.weight"),
        _p(tb.linear1.weight, dev, "linear1.weight"),
        _p(tb.conv.weight, dev, "conv.weight"),
        _p(tb.conv.bias, dev, "conv.bias"),
        _p(tb.rg_lru.log_lambda, dev, "rg_lru.log_lambda"),
        _p(tb.rg_lru.linear_a.weight, dev, "rg_lru.linear_a.weight"),
        _p(tb.rg_lru.linear_a.bias, dev, "rg_lru.linear_a.bias"),
        _p(tb.rg_lru.linear_x.weight, dev, "rg_lru.linear_x.weight"),
        _p(tb.rg_lru.linear_x.bias, dev, "rg_lru.linear_x.bias"),
        _p(tb.linear2.weight, dev, "linear2.weight"),
        _p(tb.linear_out.weight, dev, "linear_out.weight"),
        _p(tb.norm2.weight, dev, "norm2.weight"),
        _p(tb.gated_mlp.gate_proj.weight, dev, "gated_mlp.gate_proj.weight"),
        _p(tb.gated_mlp.up_proj.weight, dev, "gated_mlp.up_proj.weight"),
        _p(tb.gated_mlp.down_proj.weight, dev, "gated_mlp.down_proj.weight"),
        None if sub is None else _p(sub.weight, dev, "field_sub.weight"),
        packed,
    )
