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
        _p(block.norm_bullet.weight, dev, "norm_bullet.weight") if block.reads_bullets else None,
        _p(block.kv_bullet.weight, dev, "kv_bullet.weight") if block.reads_bullets else None,
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


def packed_image(owner, kind: str, key, params, make_struct, n_heads: int, dev: torch.device, precision: int, engine: int):
    """Device address of the tensor-core weight image of one sublayer, or None.

    The image is derived data: it is rebuilt whenever a parameter's storage or version
    changes, lives in a cache on `owner` and is never part of a state_dict.
    """
    if precision != _capi.BNB_BF16 or engine == _capi.ENGINE_SIMT:
        return None
    D = params[0].shape[-1]
    if not _capi.lib.bnb_supported(D, n_heads, 1, _capi.BNB_BF16, _capi.ENGINE_TENSOR):
        return None
    nbytes = _capi.lib.bnb_packed_spatial_bytes(D) if kind == "spatial" else _capi.lib.bnb_packed_temporal_bytes(D)
    if nbytes == 0:
        return None
    cache = owner.__dict__.setdefault("_bnb_packed", {})
    stamp = tuple((p.data_ptr(), p._version) for p in params)
    ckey = (kind, key, dev.index)
    hit = cache.get(ckey)
    if hit is not None and hit[0] == stamp:
        return hit[1].data_ptr()
    buf = hit[1] if hit is not None else torch.empty(nbytes, dtype=torch.uint8, device=dev)
    stream = _capi.stream_handle(dev)
    if kind == "spatial":
        st = _capi.lib.bnb_pack_spatial(make_struct(), D, n_heads, buf.data_ptr(), stream)
        _capi.check("bnb_pack_spatial", st)
    else:
        st = _capi.lib.bnb_pack_temporal(make_struct(), D, buf.data_ptr(), stream)
        _capi.check("bnb_pack_temporal", st)
    cache[ckey] = (stamp, buf)
    return buf.data_ptr()
