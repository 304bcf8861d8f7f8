"""Opaque ``torch.library`` operators around the C ABI.

``torch.compile(policy)`` (the reference trains and evaluates through it,
train/rl/ppo.py:396-400) must neither trace into ctypes nor break CUDA-graph capture, so the
calls into the library are registered as custom operators: Dynamo sees one opaque node with a
shape-only fake implementation; the real implementation below builds the ctypes argument
structs, looks up (or rebuilds) the tensor-core weight images, takes scratch from torch's
allocator and launches on the current stream.  Nothing here synchronises.

``trunk_forward`` carries an autograd formula (``trunk_backward`` -> ``bnb_trunk_sequence_bwd``,
environments of one size, recomputing activations); a call known to need gradients goes through
``trunk_forward_train`` instead, which keeps its activations for the backward.  Either way a step or
sequence through ``YemongBlock`` / ``YemongTrunk`` can be differentiated with respect to tokens,
recurrent state, bullet tokens and parameters.  The
single-sublayer operators are forward-only and their module methods refuse inputs that require grad.
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch
from torch import Tensor

import os

from .. import _capi
from ._weights import N_SPATIAL, N_TEMPORAL, image_buffer, packed_image, spatial_struct_from, temporal_struct_from

# geom: the integers of a call, in this order
(G_BLOCKS, G_SPATIAL, G_TEMPORAL, G_HEADS, G_BULLET_CROSS, G_FIELD_SUB, G_ENVS, G_TOKENS_PER_ENV, G_SHIPS_PER_ENV,
 G_MAX_TOKENS, G_TOTAL_TOKENS, G_TOTAL_SHIPS, G_TILES, G_TIMESTEPS, G_ENGINE, G_PRECISION) = range(16)


def _debug_check(fn: str, dev: torch.device, precision: int) -> None:
    """With BNB_DEBUG_SYNC=1 in the environment every call waits for its kernels and raises if
    one of the tensor-core kernels' bounded waits ran out (status word at the head of the scratch
    buffer).  Off by default: the check synchronises, so it cannot run under graph capture."""
    if precision == _capi.BNB_BF16 and os.environ.get("BNB_DEBUG_SYNC") == "1" and not torch.cuda.is_current_stream_capturing():
        st = _capi.tensor_engine_status(dev)
        if 100 < st < 200:   # the ST_TIMEOUT_* codes; other values are scratch data of the exact engine
            raise RuntimeError(f"{fn}: a bounded wait of the tensor-core kernels ran out (code {st})")


def _raise_pending_status(dev: torch.device) -> None:
    """A bounded wait of an earlier call on this device ran out (its kernels drained and its
    outputs were garbage): say so once, at the next call, without synchronising."""
    with torch.cuda.device(dev):
        st = _capi.lib.bnb_last_status()
        if st:
            _capi.lib.bnb_clear_status()
            raise RuntimeError(
                f"an earlier tensor-core call on {dev} gave up a bounded wait: {_capi.lib.bnb_status_string(st).decode()} "
                f"(status {st}); its outputs, and any state carried from them, are invalid")


def uniform_geom(n_envs: int, tokens: int, ships: int) -> List[int]:
    """Batch part of ``geom`` for environments of one size (entries G_ENVS .. G_TILES)."""
    return [n_envs, tokens, ships, tokens, n_envs * tokens, n_envs * ships, 0]


def _batch(geom: List[int], offsets: List[Tensor]) -> "_capi.Batch":
    if offsets:
        tok, ship = offsets[0], offsets[1]
        tiles = offsets[2] if len(offsets) > 2 else None
        ids = offsets[3] if len(offsets) > 3 else None
        return _capi.Batch(geom[G_ENVS], 0, 0, geom[G_MAX_TOKENS], geom[G_TOTAL_TOKENS], geom[G_TOTAL_SHIPS],
                           tok.data_ptr(), ship.data_ptr(), _capi.ptr(tiles), _capi.ptr(ids), geom[G_TILES])
    return _capi.Batch(geom[G_ENVS], geom[G_TOKENS_PER_ENV], geom[G_SHIPS_PER_ENV], geom[G_MAX_TOKENS],
                       geom[G_TOTAL_TOKENS], geom[G_TOTAL_SHIPS], None, None, None, None, 0)


@torch.library.custom_op("bnb_b200::trunk_forward", mutates_args=(), device_types="cuda")
def trunk_forward(
    x: Tensor,
    alive: Optional[Tensor],
    hidden: Tensor,
    done: Optional[Tensor],
    reset_env: Optional[Tensor],
    bullets: Optional[Tensor],
    bullet_mask: Optional[Tensor],
    weights: List[Tensor],
    offsets: List[Tensor],
    geom: List[int],
) -> Tuple[Tensor, Tensor]:
    """Blocks of (spatial sublayers, temporal sublayers) over x: ``bnb_trunk_step`` when
    geom[G_TIMESTEPS] is 0, else ``bnb_trunk_sequence`` over that many timesteps.

    x (total_tokens, D) or (T, total_tokens, D), float32 or bfloat16; hidden (L, total_ships, 4D) packed;
    ``weights`` the parameters of every sublayer, block-major, spatial before temporal inside a
    block, each sublayer in the order of ``_weights.spatial_tensors`` / ``temporal_tensors``;
    ``offsets`` empty for environments of one size, else [tok_off, ship_off(, tile_env_begin,
    tile_env_ids)].  Returns (y like x: bfloat16 for bfloat16 tokens, else float32; new hidden like
    hidden, float32).
    """
    dev = x.device
    D = x.shape[-1]
    n_blocks, n_spatial, n_temporal = geom[G_BLOCKS], geom[G_SPATIAL], geom[G_TEMPORAL]
    n_heads, n_cross, field_sub = geom[G_HEADS], geom[G_BULLET_CROSS], geom[G_FIELD_SUB]
    engine, precision = geom[G_ENGINE], geom[G_PRECISION]
    T = max(1, geom[G_TIMESTEPS])
    with torch.cuda.device(dev):
        batch = _batch(geom, offsets)
        # bfloat16 tokens (what the reference's encoder hands its trunk under CUDA autocast) stay
        # bfloat16 on the way in and out where the fused kernel serves the call; the residual stream
        # inside the call is float32 either way.  Anything else is converted to float32 here.
        io16 = (x.dtype == torch.bfloat16 and precision == _capi.BNB_BF16 and engine != _capi.ENGINE_SIMT
                and geom[G_MAX_TOKENS] > 0
                and bool(_capi.lib.bnb_supported(D, n_heads, geom[G_MAX_TOKENS], _capi.BNB_BF16, _capi.ENGINE_TENSOR))
                and (not offsets or len(offsets) > 2))
        hin = _capi.f32c(hidden)
        alive_u8 = _capi.u8(alive)
        done_u8 = _capi.u8(done)
        reset_u8 = _capi.u8(reset_env)
        hout = torch.empty_like(hin)
        sw = (_capi.SpatialWeights * max(1, n_blocks * n_spatial))()
        tw = (_capi.TemporalWeights * max(1, n_blocks * n_temporal))()
        pos = 0
        for i in range(n_blocks):
            for j in range(n_spatial):
                n = N_SPATIAL + (2 if j < n_cross else 0)
                ts = list(weights[pos : pos + n])
                pos += n
                sw[i * n_spatial + j] = spatial_struct_from(
                    ts, dev, image_buffer("spatial", ts, n_heads, dev, precision, engine))
            for j in range(n_temporal):
                n = N_TEMPORAL + (1 if field_sub else 0)
                ts = list(weights[pos : pos + n])
                pos += n
                tw[i * n_temporal + j] = temporal_struct_from(
                    ts, dev, image_buffer("temporal", ts, 4, dev, precision, engine))
        if pos != len(weights):
            raise RuntimeError(f"expected {pos} parameter tensors for this trunk structure, got {len(weights)}")
        bul16 = (precision == _capi.BNB_BF16 and engine != _capi.ENGINE_SIMT and geom[G_MAX_TOKENS] > 0
                 and bool(_capi.lib.bnb_supported(D, n_heads, geom[G_MAX_TOKENS], _capi.BNB_BF16, _capi.ENGINE_TENSOR)))
        stream = _capi.stream_handle(dev)
        _raise_pending_status(dev)
        ns_total, nt_total = n_blocks * n_spatial, n_blocks * n_temporal
        if all(sw[i].packed for i in range(ns_total)) and all(tw[i].packed for i in range(nt_total)) and ns_total + nt_total > 0:
            # the weight images of the whole trunk, rewritten from the live parameters on every call
            _capi.check("bnb_pack_trunk", _capi.lib.bnb_pack_trunk(sw, ns_total, tw, nt_total, D, n_heads, stream))
        fn = "bnb_trunk_step" if geom[G_TIMESTEPS] == 0 else "bnb_trunk_sequence"

        def run(tokens16: bool, bullets16: bool):
            xin = (x if x.is_contiguous() else x.contiguous()) if tokens16 else _capi.f32c(x)
            y = torch.empty_like(xin)
            bul = _capi.BulletArgs(bullets if n_cross > 0 else None, bullet_mask, T * batch.n_envs, D, keep_bf16=bullets16)
            scratch = _capi.scratch_for(dev, _capi.lib.bnb_scratch_bytes(D, batch, T, bul.per_env))
            head = (sw, tw, n_blocks, n_spatial, n_temporal, D, n_heads, xin.data_ptr(), _capi.ptr(alive_u8), bul.arg,
                    y.data_ptr(), _capi.ptr(hin), _capi.ptr(hout))
            tail = (_capi.BNB_BF16_IO if tokens16 else precision, engine, scratch.data_ptr(), scratch.numel(), stream)
            if geom[G_TIMESTEPS] == 0:
                st = _capi.lib.bnb_trunk_step(*head, _capi.ptr(reset_u8), batch, *tail)
            else:
                st = _capi.lib.bnb_trunk_sequence(*head, _capi.ptr(done_u8), batch, T, *tail)
            return st, y, bul.is_bf16

        st, y, used_bul16 = run(io16, bul16)
        if st == _capi.ERR_UNSUPPORTED_DIMS and (io16 or used_bul16):
            # the call fell to the float32-reading kernels (a shape the tensor-core kernels do not serve,
            # e.g. more bullet slots than their attention stages; nothing was launched): once more with
            # float32 copies of the tokens and the bullet tokens
            st, y, _ = run(False, False)
    _capi.check(fn, st)
    _capi.note_engine_choice(fn)
    _debug_check(fn, dev, precision)
    if x.dtype == torch.bfloat16 and y.dtype != torch.bfloat16:
        y = y.to(torch.bfloat16)   # the same contract on the paths that compute from a float32 copy
    return y, hout


@trunk_forward.register_fake
def _trunk_forward_fake(x, alive, hidden, done, reset_env, bullets, bullet_mask, weights, offsets, geom):
    out_dtype = torch.bfloat16 if x.dtype == torch.bfloat16 else torch.float32
    return (x.new_empty(x.shape, dtype=out_dtype), hidden.new_empty(hidden.shape, dtype=torch.float32))


def _grad_precision(geom: List[int]) -> int:
    """Precision of the training forward and the backward: bf16 operands after an autocast forward."""
    return _capi.BNB_BF16 if geom[G_PRECISION] == _capi.BNB_BF16 else _capi.BNB_FP32


def _kept_size(geom: List[int], d_model: int, bullets_per_env: int) -> int:
    """Bytes of the kept-activation buffer of a training forward (host arithmetic only)."""
    need = _capi.lib.bnb_trunk_kept_bytes(geom[G_BLOCKS], geom[G_SPATIAL], geom[G_TEMPORAL], d_model, geom[G_HEADS],
                                          _batch(geom, []), max(1, geom[G_TIMESTEPS]), bullets_per_env, _grad_precision(geom))
    return max(256, int(need))


def _sublayer_lists(weights: List[Tensor], n_blocks: int, n_spatial: int, n_temporal: int, n_cross: int, field_sub: int):
    """``weights`` cut into the per-sublayer lists, block-major, spatial before temporal."""
    spatial, temporal, pos = [], [], 0
    for _ in range(n_blocks):
        for j in range(n_spatial):
            n = N_SPATIAL + (2 if j < n_cross else 0)
            spatial.append(list(weights[pos : pos + n]))
            pos += n
        for _j in range(n_temporal):
            n = N_TEMPORAL + (1 if field_sub else 0)
            temporal.append(list(weights[pos : pos + n]))
            pos += n
    if pos != len(weights):
        raise RuntimeError(f"expected {pos} parameter tensors for this trunk structure, got {len(weights)}")
    return spatial, temporal


@torch.library.custom_op("bnb_b200::trunk_backward", mutates_args=(), device_types="cuda")
def trunk_backward(
    dy: Tensor,
    dhidden_out: Optional[Tensor],
    kept: Optional[Tensor],
    x: Tensor,
    alive: Optional[Tensor],
    hidden: Tensor,
    done: Optional[Tensor],
    bullets: Optional[Tensor],
    bullet_mask: Optional[Tensor],
    weights: List[Tensor],
    geom: List[int],
) -> List[Tensor]:
    """Gradients of ``trunk_forward`` (environments of one size, no ``reset_env``) through
    ``bnb_trunk_sequence_bwd``: float32 tensors throughout; after a forward under bf16 autocast the
    Linear products round their operands to bfloat16, as the reference's backward does there.  Returns
    [d x, d hidden, d bullets (empty without bullets), every parameter gradient in one flat buffer
    (``_split_grads`` cuts it into one view per tensor of ``weights``)].
    ``kept``: the activations ``trunk_forward_train`` kept for this call (the backward consumes
    them), or None: every sublayer's intermediates are recomputed."""
    dev = x.device
    D = x.shape[-1]
    n_blocks, n_spatial, n_temporal = geom[G_BLOCKS], geom[G_SPATIAL], geom[G_TEMPORAL]
    n_heads, n_cross, field_sub = geom[G_HEADS], geom[G_BULLET_CROSS], geom[G_FIELD_SUB]
    T = max(1, geom[G_TIMESTEPS])
    with torch.cuda.device(dev):
        batch = _batch(geom, [])
        xin, hin, dyin = _capi.f32c(x), _capi.f32c(hidden), _capi.f32c(dy)
        dho = None if dhidden_out is None else _capi.f32c(dhidden_out)
        alive_u8, done_u8 = _capi.u8(alive), _capi.u8(done)
        spatial, temporal = _sublayer_lists(weights, n_blocks, n_spatial, n_temporal, n_cross, field_sub)
        # one zeroed buffer for every parameter gradient (the kernels accumulate into it), cut into
        # views at 16-byte boundaries
        flat_grads = torch.zeros(sum(_grad_sizes(weights)), dtype=torch.float32, device=dev)
        grads = _split_grads(flat_grads, weights)
        g_spatial, g_temporal = _sublayer_lists(grads, n_blocks, n_spatial, n_temporal, n_cross, field_sub)
        sw = (_capi.SpatialWeights * max(1, len(spatial)))()
        tw = (_capi.TemporalWeights * max(1, len(temporal)))()
        sg = (_capi.SpatialGrads * max(1, len(spatial)))()
        tg = (_capi.TemporalGrads * max(1, len(temporal)))()
        for i, (ts, gs) in enumerate(zip(spatial, g_spatial)):
            sw[i] = spatial_struct_from(ts, dev)
            sg[i] = _capi.SpatialGrads(*[g.data_ptr() for g in gs], *([None] * (N_SPATIAL + 2 - len(gs))))
        for i, (ts, gs) in enumerate(zip(temporal, g_temporal)):
            tw[i] = temporal_struct_from(ts, dev)
            tg[i] = _capi.TemporalGrads(*[g.data_ptr() for g in gs], *([None] * (N_TEMPORAL + 1 - len(gs))))
        bul = _capi.BulletArgs(bullets if n_cross > 0 else None, bullet_mask, T * batch.n_envs, D)
        dx = torch.empty_like(xin)
        dh = torch.zeros_like(hin)
        dbul = torch.zeros_like(bul.tokens) if bul.struct is not None else xin.new_empty(0)
        nbytes = _capi.lib.bnb_trunk_bwd_scratch_bytes(n_blocks, n_spatial, n_temporal, D, batch, T, bul.per_env,
                                                       _grad_precision(geom))
        scratch = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=dev)   # released after the call's stream work
        st = _capi.lib.bnb_trunk_sequence_bwd(
            sw, tw, sg, tg, n_blocks, n_spatial, n_temporal, D, n_heads, xin.data_ptr(), _capi.ptr(alive_u8), bul.arg,
            _capi.ptr(hin), _capi.ptr(done_u8), batch, T, _grad_precision(geom),
            dyin.data_ptr(), _capi.ptr(dho), dx.data_ptr(),
            _capi.ptr(dh), _capi.ptr(dbul) if bul.struct is not None else None, _capi.ptr(kept),
            0 if kept is None else kept.numel(), scratch.data_ptr(), scratch.numel(), _capi.stream_handle(dev),
        )
    _capi.check("bnb_trunk_sequence_bwd", st)
    return [dx, dh, dbul, flat_grads]


@trunk_backward.register_fake
def _trunk_backward_fake(dy, dhidden_out, kept, x, alive, hidden, done, bullets, bullet_mask, weights, geom):
    dbul = x.new_empty(bullets.shape, dtype=torch.float32) if bullets is not None and geom[G_BULLET_CROSS] > 0 else x.new_empty(0, dtype=torch.float32)
    return [x.new_empty(x.shape, dtype=torch.float32), hidden.new_empty(hidden.shape, dtype=torch.float32), dbul,
            x.new_empty(sum(_grad_sizes(weights)), dtype=torch.float32)]


def _grad_sizes(weights: List[Tensor]) -> List[int]:
    """Elements each parameter gradient takes in the flat buffer (16-byte granules)."""
    return [(w.numel() + 3) // 4 * 4 for w in weights]


def _split_grads(flat: Tensor, weights: List[Tensor]) -> List[Tensor]:
    views, off = [], 0
    for w, n in zip(weights, _grad_sizes(weights)):
        views.append(flat[off : off + w.numel()].view(w.shape))
        off += n
    return views


def _shape_grads(out, x, hidden, bullets, weights):
    dx, dh, dbul, dws = out[0], out[1], out[2], _split_grads(out[3], weights)
    dx = dx.reshape(x.shape).to(x.dtype)
    dh = dh.reshape(hidden.shape).to(hidden.dtype)
    dbul = dbul.reshape(bullets.shape).to(bullets.dtype) if bullets is not None and dbul.numel() else None
    return dx, dh, dbul, [g.to(w.dtype) for g, w in zip(dws, weights)]


def _trunk_setup_context(ctx, inputs, output):
    x, alive, hidden, done, reset_env, bullets, bullet_mask, weights, offsets, geom = inputs
    ctx.geom = list(geom)
    ctx.unsupported = ("a ragged batch" if offsets else "reset_env" if reset_env is not None else "")
    ctx.n_offsets = len(offsets)
    ctx.save_for_backward(x, alive, hidden, done, bullets, bullet_mask, *weights)


def _trunk_backward_formula(ctx, dy, dhidden_out):
    if ctx.unsupported:
        raise NotImplementedError(f"the CUDA trunk's backward does not cover {ctx.unsupported}; run that call under torch.no_grad()")
    x, alive, hidden, done, bullets, bullet_mask, *weights = ctx.saved_tensors
    out = trunk_backward(dy, dhidden_out, None, x, alive, hidden, done, bullets, bullet_mask, list(weights), ctx.geom)
    dx, dh, dbul, dws = _shape_grads(out, x, hidden, bullets, weights)
    # one entry per input; a list input takes a list of the same length
    return dx, None, dh, None, None, dbul, None, dws, [None] * ctx.n_offsets, None


trunk_forward.register_autograd(_trunk_backward_formula, setup_context=_trunk_setup_context)


@torch.library.custom_op("bnb_b200::trunk_forward_train", mutates_args=(), device_types="cuda")
def trunk_forward_train(
    x: Tensor,
    alive: Optional[Tensor],
    hidden: Tensor,
    done: Optional[Tensor],
    bullets: Optional[Tensor],
    bullet_mask: Optional[Tensor],
    weights: List[Tensor],
    geom: List[int],
) -> Tuple[Tensor, Tensor, Tensor]:
    """``trunk_forward`` for a call that will be differentiated (environments of one size, no
    ``reset_env``): ``bnb_trunk_sequence_fwd_train`` runs the trunk sublayer by sublayer and keeps
    every sublayer's intermediates, as autograd does for the reference without grad_checkpoint;
    the backward then skips its recomputation.  Returns (y, new hidden, kept activations); y is
    float32, or bfloat16 for bfloat16 tokens."""
    dev = x.device
    D = x.shape[-1]
    n_blocks, n_spatial, n_temporal = geom[G_BLOCKS], geom[G_SPATIAL], geom[G_TEMPORAL]
    n_heads, n_cross, field_sub = geom[G_HEADS], geom[G_BULLET_CROSS], geom[G_FIELD_SUB]
    T = max(1, geom[G_TIMESTEPS])
    with torch.cuda.device(dev):
        batch = _batch(geom, [])
        xin, hin = _capi.f32c(x), _capi.f32c(hidden)
        alive_u8, done_u8 = _capi.u8(alive), _capi.u8(done)
        spatial, temporal = _sublayer_lists(weights, n_blocks, n_spatial, n_temporal, n_cross, field_sub)
        sw = (_capi.SpatialWeights * max(1, len(spatial)))()
        tw = (_capi.TemporalWeights * max(1, len(temporal)))()
        for i, ts in enumerate(spatial):
            sw[i] = spatial_struct_from(ts, dev)
        for i, ts in enumerate(temporal):
            tw[i] = temporal_struct_from(ts, dev)
        bul = _capi.BulletArgs(bullets if n_cross > 0 else None, bullet_mask, T * batch.n_envs, D)
        y = torch.empty_like(xin)
        hout = torch.empty_like(hin)
        kept = torch.empty(_kept_size(geom, D, bul.per_env), dtype=torch.uint8, device=dev)
        nbytes = _capi.lib.bnb_trunk_bwd_scratch_bytes(n_blocks, n_spatial, n_temporal, D, batch, T, bul.per_env,
                                                       _grad_precision(geom))
        scratch = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=dev)
        st = _capi.lib.bnb_trunk_sequence_fwd_train(
            sw, tw, n_blocks, n_spatial, n_temporal, D, n_heads, xin.data_ptr(), _capi.ptr(alive_u8), bul.arg, y.data_ptr(),
            _capi.ptr(hin), _capi.ptr(hout), _capi.ptr(done_u8), batch, T,
            _grad_precision(geom), kept.data_ptr(), kept.numel(),
            scratch.data_ptr(), scratch.numel(), _capi.stream_handle(dev),
        )
    _capi.check("bnb_trunk_sequence_fwd_train", st)
    if x.dtype == torch.bfloat16:
        y = y.to(torch.bfloat16)
    return y, hout, kept


@trunk_forward_train.register_fake
def _trunk_forward_train_fake(x, alive, hidden, done, bullets, bullet_mask, weights, geom):
    out_dtype = torch.bfloat16 if x.dtype == torch.bfloat16 else torch.float32
    per_env = bullets.shape[1] if bullets is not None and geom[G_BULLET_CROSS] > 0 else 0
    return (x.new_empty(x.shape, dtype=out_dtype), hidden.new_empty(hidden.shape, dtype=torch.float32),
            x.new_empty(_kept_size(geom, x.shape[-1], per_env), dtype=torch.uint8))


def _train_setup_context(ctx, inputs, output):
    x, alive, hidden, done, bullets, bullet_mask, weights, geom = inputs
    ctx.geom = list(geom)
    ctx.consumed = False
    ctx.mark_non_differentiable(output[2])
    # autograd would otherwise materialise a zero "gradient" the size of the kept activations
    ctx.set_materialize_grads(False)
    ctx.save_for_backward(x, alive, hidden, done, bullets, bullet_mask, output[2], *weights)


def _train_backward_formula(ctx, dy, dhidden_out, _dkept):
    if ctx.consumed:
        raise RuntimeError("the kept activations of this trunk call were consumed by an earlier backward; for a second "
                           "backward through the same graph set BNB_GRAD_MODE=recompute")
    ctx.consumed = True
    x, alive, hidden, done, bullets, bullet_mask, kept, *weights = ctx.saved_tensors
    if dy is None:
        dy = torch.zeros_like(x, dtype=torch.float32)
    out = trunk_backward(dy, dhidden_out, kept, x, alive, hidden, done, bullets, bullet_mask, list(weights), ctx.geom)
    dx, dh, dbul, dws = _shape_grads(out, x, hidden, bullets, weights)
    return dx, None, dh, None, dbul, None, dws, None


trunk_forward_train.register_autograd(_train_backward_formula, setup_context=_train_setup_context)


def keep_activations(dev: torch.device, geom: List[int], d_model: int, n_bullets: int) -> bool:
    """Whether a differentiated call keeps its activations (faster) or lets the backward recompute
    them (about a sixth of the memory): BNB_GRAD_MODE=keep | recompute decides; otherwise keep when
    the kept buffer plus the backward's scratch fit in 70 % of the memory that is free or cached."""
    mode = os.environ.get("BNB_GRAD_MODE", "")
    if mode == "recompute":
        return False
    with torch.cuda.device(dev):
        batch = _batch(geom, [])
        T = max(1, geom[G_TIMESTEPS])
        need = _capi.lib.bnb_trunk_kept_bytes(geom[G_BLOCKS], geom[G_SPATIAL], geom[G_TEMPORAL], d_model, geom[G_HEADS], batch, T,
                                              n_bullets, _grad_precision(geom))
        if need == 0:
            return False
        if mode == "keep":
            return True
        need += _capi.lib.bnb_trunk_bwd_scratch_bytes(geom[G_BLOCKS], geom[G_SPATIAL], geom[G_TEMPORAL], d_model, batch, T, n_bullets,
                                                      _grad_precision(geom))
        free, _ = torch.cuda.mem_get_info(dev)
        cached = torch.cuda.memory_reserved(dev) - torch.cuda.memory_allocated(dev)
    return need <= 0.7 * (free + cached)


@torch.library.custom_op("bnb_b200::spatial_forward", mutates_args=(), device_types="cuda")
def spatial_forward(
    x: Tensor,
    alive: Optional[Tensor],
    bullets: Optional[Tensor],
    bullet_mask: Optional[Tensor],
    weights: List[Tensor],
    n_heads: int,
    precision: int,
    engine: int,
) -> Tensor:
    """One spatial sublayer, ``bnb_spatial_block_fwd``: x (B, N, D), alive (B, N) or None,
    bullets (B, NB, D) / bullet_mask (B, NB) or None; returns float32 (B, N, D)."""
    dev = x.device
    B, N, D = x.shape
    ts = list(weights)
    with torch.cuda.device(dev):
        xin = _capi.f32c(x)
        alive_u8 = _capi.u8(alive)
        y = torch.empty_like(xin)
        batch = _capi.uniform_batch(B, N, N)
        bul = _capi.BulletArgs(bullets if len(ts) > N_SPATIAL else None, bullet_mask, B, D)
        nbytes = _capi.lib.bnb_scratch_bytes(D, batch, 1, bul.per_env)
        scratch = _capi.scratch_for(dev, nbytes)
        _raise_pending_status(dev)
        w = spatial_struct_from(ts, dev, packed_image("spatial", ts, n_heads, dev, precision, engine))
        st = _capi.lib.bnb_spatial_block_fwd(
            w, D, n_heads, xin.data_ptr(), _capi.ptr(alive_u8), bul.arg, y.data_ptr(), batch, 1, precision, engine,
            scratch.data_ptr(), scratch.numel(), _capi.stream_handle(dev),
        )
    _capi.check("bnb_spatial_block_fwd", st)
    _capi.note_engine_choice("bnb_spatial_block_fwd")
    _debug_check("bnb_spatial_block_fwd", dev, precision)
    return y


@spatial_forward.register_fake
def _spatial_forward_fake(x, alive, bullets, bullet_mask, weights, n_heads, precision, engine):
    return x.new_empty(x.shape, dtype=torch.float32)
