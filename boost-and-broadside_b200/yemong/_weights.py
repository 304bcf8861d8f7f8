"""Parameter pointer tables handed to the C ABI (BnbSpatialWeights / BnbTemporalWeights) and
the cache of derived tensor-core weight images.

A sublayer's parameters travel as a flat list of tensors in a fixed order, so the same code
serves the module methods and the opaque ``torch.library`` operators (which see tensors, not
modules):

    spatial   norm1, qkv, out_proj, norm2, ffn.gate, ffn.up, ffn.down [, norm_bullet, kv_bullet]
    temporal  norm1, linear1, conv.weight, conv.bias, log_lambda, a.weight, a.bias, x.weight,
              x.bias, linear2, linear_out, norm2, mlp.gate, mlp.up, mlp.down [, field_sub]
"""

from __future__ import annotations

import weakref

import torch

from .. import _capi

N_SPATIAL = 7          # + 2 when the sublayer reads bullets
N_TEMPORAL = 15        # + 1 with the field substitute


def spatial_tensors(block) -> list[torch.Tensor]:
    ts = [block.norm1.weight, block.qkv.weight, block.out_proj.weight, block.norm2.weight,
          block.ffn.gate_proj.weight, block.ffn.up_proj.weight, block.ffn.down_proj.weight]
    if block.reads_bullets:
        ts += [block.norm_bullet.weight, block.kv_bullet.weight]
    return ts


def temporal_tensors(tb, sub=None) -> list[torch.Tensor]:
    ts = [tb.norm1.weight, tb.linear1.weight, tb.conv.weight, tb.conv.bias, tb.rg_lru.log_lambda,
          tb.rg_lru.linear_a.weight, tb.rg_lru.linear_a.bias, tb.rg_lru.linear_x.weight, tb.rg_lru.linear_x.bias,
          tb.linear2.weight, tb.linear_out.weight, tb.norm2.weight, tb.gated_mlp.gate_proj.weight,
          tb.gated_mlp.up_proj.weight, tb.gated_mlp.down_proj.weight]
    if sub is not None:
        ts.append(sub.weight)
    return ts


def _p(t: torch.Tensor, dev: torch.device, what: str) -> int:
    if t.device != dev:
        raise RuntimeError(f"{what} parameter is on {t.device}, input on {dev}")
    if t.dtype != torch.float32 or not t.is_contiguous():
        raise RuntimeError(f"{what} parameter must be contiguous float32 (got {t.dtype})")
    return t.data_ptr()


def spatial_struct_from(ts: list[torch.Tensor], dev: torch.device, packed: int | None = None) -> _capi.SpatialWeights:
    if len(ts) not in (N_SPATIAL, N_SPATIAL + 2):
        raise RuntimeError(f"a spatial sublayer has {N_SPATIAL} or {N_SPATIAL + 2} parameters, got {len(ts)}")
    ptrs = [_p(t, dev, "spatial") for t in ts] + [None] * (N_SPATIAL + 2 - len(ts))
    return _capi.SpatialWeights(*ptrs, packed)


def temporal_struct_from(ts: list[torch.Tensor], dev: torch.device, packed: int | None = None) -> _capi.TemporalWeights:
    if len(ts) not in (N_TEMPORAL, N_TEMPORAL + 1):
        raise RuntimeError(f"a temporal sublayer has {N_TEMPORAL} or {N_TEMPORAL + 1} parameters, got {len(ts)}")
    ptrs = [_p(t, dev, "temporal") for t in ts] + [None] * (N_TEMPORAL + 1 - len(ts))
    return _capi.TemporalWeights(*ptrs, packed)


def spatial_struct(block, dev: torch.device, packed: int | None = None) -> _capi.SpatialWeights:
    return spatial_struct_from(spatial_tensors(block), dev, packed)


def temporal_struct(tb, sub, dev: torch.device, packed: int | None = None) -> _capi.TemporalWeights:
    return temporal_struct_from(temporal_tensors(tb, sub), dev, packed)


# (kind, device, ids of the parameter tensors) -> (stamp, image buffer, weak references)
_images: dict[tuple, tuple] = {}


def packed_image(kind: str, ts: list[torch.Tensor], n_heads: int, dev: torch.device, precision: int, engine: int):
    """Device address of the tensor-core weight image of one sublayer, or None.

    The image is derived data: it is rebuilt whenever a parameter's storage or version
    changes, lives in a process-wide cache that drops an entry when one of its parameters is
    garbage-collected, and is never part of a state_dict.
    """
    if precision != _capi.BNB_BF16 or engine == _capi.ENGINE_SIMT:
        return None
    D = ts[0].shape[-1]
    if not _capi.lib.bnb_supported(D, n_heads, 1, _capi.BNB_BF16, _capi.ENGINE_TENSOR):
        return None
    nbytes = _capi.lib.bnb_packed_spatial_bytes(D) if kind == "spatial" else _capi.lib.bnb_packed_temporal_bytes(D)
    if nbytes == 0:
        return None
    key = (kind, dev.index, tuple(id(t) for t in ts))
    stamp = tuple((t.data_ptr(), t._version) for t in ts)
    hit = _images.get(key)
    if hit is not None and not all(r() is t for r, t in zip(hit[2], ts)):
        hit = None  # an id was reused by another tensor
    if hit is not None and hit[0] == stamp:
        return hit[1].data_ptr()
    buf = hit[1] if hit is not None else _capi.persistent_bytes(dev, nbytes)
    stream = _capi.stream_handle(dev)
    if kind == "spatial":
        st = _capi.lib.bnb_pack_spatial(spatial_struct_from(ts, dev), D, n_heads, buf.data_ptr(), stream)
        _capi.check("bnb_pack_spatial", st)
    else:
        st = _capi.lib.bnb_pack_temporal(temporal_struct_from(ts, dev), D, buf.data_ptr(), stream)
        _capi.check("bnb_pack_temporal", st)
    refs = tuple(weakref.ref(t, lambda _r, k=key: _images.pop(k, None)) for t in ts)
    _images[key] = (stamp, buf, refs)
    return buf.data_ptr()
