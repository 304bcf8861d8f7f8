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


# (kind, device, ids of the parameter tensors) -> (image buffer, weak references)
_images: dict[tuple, tuple] = {}
# Buffers whose parameters were garbage-collected.  They are kept (a bounded number of them): a
# launch still in flight, or a captured CUDA graph, may hold their address.
_retired: list[torch.Tensor] = []
_RETIRED_MAX = 512


def _retire(key: tuple) -> None:
    hit = _images.pop(key, None)
    if hit is not None:
        _retired.append(hit[0])
        if len(_retired) > _RETIRED_MAX:
            del _retired[0]


def image_buffer(kind: str, ts: list[torch.Tensor], n_heads: int, dev: torch.device, precision: int, engine: int):
    """Device address of the buffer that holds the tensor-core weight image of one sublayer, or
    None when the call does not use the tensor engine.  Nothing is packed here: the image is
    written by ``bnb_pack_trunk`` / ``bnb_pack_*`` **on every call**, on the call's stream, so it
    cannot go stale -- not after an optimizer step, not after ``p.data.copy_()`` (which bumps no
    version counter; the reference's running-average policy is updated that way,
    train/rl/opponents.py:112), and not in a replayed CUDA graph (the pack launch is part of the
    captured work and re-reads the live float32 parameters).  The buffer itself is persistent and
    keyed on the identity of the parameter tensors; it is derived data and never part of a
    state_dict."""
    if precision != _capi.BNB_BF16 or engine == _capi.ENGINE_SIMT:
        return None
    D = ts[0].shape[-1]
    if not _capi.lib.bnb_supported(D, n_heads, 1, _capi.BNB_BF16, _capi.ENGINE_TENSOR):
        return None
    nbytes = _capi.lib.bnb_packed_spatial_bytes(D) if kind == "spatial" else _capi.lib.bnb_packed_temporal_bytes(D)
    if nbytes == 0:
        return None
    key = (kind, dev.index, tuple(id(t) for t in ts))
    hit = _images.get(key)
    if hit is not None and not all(r() is t for r, t in zip(hit[1], ts)):
        _retire(key)  # an id was reused by another tensor
        hit = None
    if hit is None:
        buf = _capi.persistent_bytes(dev, nbytes)
        refs = tuple(weakref.ref(t, lambda _r, k=key: _retire(k)) for t in ts)
        hit = (buf, refs)
        _images[key] = hit
    return hit[0].data_ptr()


def packed_image(kind: str, ts: list[torch.Tensor], n_heads: int, dev: torch.device, precision: int, engine: int):
    """``image_buffer`` plus the pack launch of this one sublayer (callers that run a single
    sublayer; a trunk call packs all of its sublayers with one ``bnb_pack_trunk`` instead)."""
    ptr = image_buffer(kind, ts, n_heads, dev, precision, engine)
    if ptr is None:
        return None
    D = ts[0].shape[-1]
    stream = _capi.stream_handle(dev)
    if kind == "spatial":
        st = _capi.lib.bnb_pack_spatial(spatial_struct_from(ts, dev), D, n_heads, ptr, stream)
        _capi.check("bnb_pack_spatial", st)
    else:
        st = _capi.lib.bnb_pack_temporal(temporal_struct_from(ts, dev), D, ptr, stream)
        _capi.check("bnb_pack_temporal", st)
    return ptr
