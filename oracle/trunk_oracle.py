"""CPU restatement of the YemongPolicy trunk: TEST INFRASTRUCTURE ONLY.

This file is the checker for the CUDA kernels.  Only the test-suite, the smoke
check and the benchmark's CPU-baseline leg may import it; the product path never
does (the product raises when its CUDA library is missing).

It restates, with plain tensor arithmetic on the CPU (matmul, exp, erf, sigmoid,
pow; no ``nn.Module``), what the reference computes on its trunk hot path:

* spatial sublayer         models/yemong/attention.py:76-169 (TransformerBlock)
* gated MLP                models/yemong/attention.py:21-37  (GatedMLP, erf GeLU)
* RMS norm                 nn.RMSNorm with eps=None -> finfo(float32).eps
* temporal sublayer        models/yemong/griffin.py:249-286  (forward_sequence)
* causal depthwise conv    models/yemong/griffin.py:67-140   (tap validity + taps)
* RG-LRU gates and update  models/yemong/griffin.py:169-219
* recurrence               models/yemong/griffin.py:25-64 (Hillis-Steele scan; stated
                           here as the sequential loop it is pinned against in the
                           reference's own tests, tests/models/test_encoder.py:198-225)
* field (non-recurrent)    models/yemong/griffin.py:288-317
* block step / sequence    models/yemong/griffin.py:376-472
* trunk loop, hidden pack  models/yemong/policy.py:315-354 (step), 422-478 (sequence)
* done reset               models/yemong/policy.py:268-285

Precision modes
---------------
``fp32``  every operation in float32 (the reference without autocast).
``bf16``  the reference under ``torch.autocast(bfloat16)``: every Linear casts its
          input, weight and bias to bf16, accumulates in fp32 and rounds its output
          to bf16; attention q/k/v/out are bf16; GeLU and the gate*up product are
          bf16; RMSNorm, residual stream, conv taps, pow, gate, recurrence and the
          hidden state stay fp32.  Values are carried in float32 containers and
          rounded to bf16 at exactly those points.

Parity pinned: against outputs of the reference itself (imported on CPU), stored in
tests/golden/*.npz by tests/golden/make_golden.py.  The reference's trained-weight
fixture (tests/fixtures/migration/landmark_682_reference.npz) cannot be used because
the weights it belongs to are not distributed with the source.
"""

from __future__ import annotations

import math
from typing import Mapping, Sequence

import torch

CONV_KERNEL = 4  # models/yemong/griffin.py:22
RMS_EPS = float(torch.finfo(torch.float32).eps)
RGLRU_C = 8.0  # models/yemong/griffin.py:160

Params = Mapping[str, torch.Tensor]


# --------------------------------------------------------------------------- helpers


def _r(x: torch.Tensor, mode: str) -> torch.Tensor:
    """Round to bf16 (kept in a float32 container) in bf16 mode; identity in fp32."""
    if mode == "bf16":
        return x.to(torch.bfloat16).to(torch.float32)
    return x


def rms_norm(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * weight, always float32."""
    x = x.to(torch.float32)
    inv = torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + RMS_EPS)
    return x * inv * weight


def linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None, mode: str) -> torch.Tensor:
    """y = x W^T (+ b).  bf16 mode: what autocast does to nn.Linear: input, weight and bias
    cast to bf16, product accumulated in fp32, result rounded to bf16 (returned in float32)."""
    if mode == "bf16":
        y = torch.nn.functional.linear(
            x.to(torch.bfloat16), w.to(torch.bfloat16), None if b is None else b.to(torch.bfloat16)
        )
        return y.to(torch.float32)
    y = x @ w.t()
    if b is not None:
        y = y + b
    return y


def gelu_erf(x: torch.Tensor) -> torch.Tensor:
    return 0.5 * x * (1.0 + torch.erf(x * (1.0 / math.sqrt(2.0))))


def gated_mlp(x: torch.Tensor, p: Params, prefix: str, mode: str) -> torch.Tensor:
    """down(gelu(gate(x)) * up(x)); attention.py:36-37."""
    g = linear(x, p[prefix + "gate_proj.weight"], None, mode)
    u = linear(x, p[prefix + "up_proj.weight"], None, mode)
    h = _r(_r(gelu_erf(g), mode) * u, mode)
    return linear(h, p[prefix + "down_proj.weight"], None, mode)


# --------------------------------------------------------------------------- spatial


class _AttentionLse(torch.autograd.Function):
    """softmax(s) v with the backward of a fused attention kernel, which is what the reference's
    F.scaled_dot_product_attention runs (attention.py:131, 157): the probabilities are recomputed
    as exp(s - lse) from the saved log-sum-exp, and the row term is <d out, out>.  For any row with
    a live key this is the plain softmax gradient.  Where every key is dead, lse = max + log(n)
    rounds to max in float32 (max is the huge negative bias), the recomputed probabilities are 1
    instead of 1/n, and the gradient is n times the textbook one -- the reference's own gradients
    (tests/golden/grad_trunk_seq_d128_t1_8s0f.npz) show exactly that."""

    @staticmethod
    def forward(ctx, q, k, v, bias, scale):
        s = (q @ k.transpose(-1, -2)) * scale
        if bias is not None:
            s = s + bias
        m = s.amax(dim=-1, keepdim=True)
        e = torch.exp(s - m)
        l = e.sum(dim=-1, keepdim=True)
        out = (e / l) @ v
        ctx.save_for_backward(q, k, v, bias if bias is not None else torch.zeros(()), m + torch.log(l), out)
        ctx.scale, ctx.has_bias = scale, bias is not None
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, bias, lse, out = ctx.saved_tensors
        s = (q @ k.transpose(-1, -2)) * ctx.scale
        if ctx.has_bias:
            s = s + bias
        p = torch.exp(s - lse)
        dv = p.transpose(-1, -2) @ dout
        dp = dout @ v.transpose(-1, -2)
        delta = (dout * out).sum(dim=-1, keepdim=True)
        ds = p * (dp - delta) * ctx.scale
        return ds @ k, ds.transpose(-1, -2) @ q, dv, None, None


def masked_attention(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, alive: torch.Tensor | None, mode: str
) -> torch.Tensor:
    """softmax(q k^T / sqrt(dh) + key_bias) v per environment and head.

    q, k, v: (B, H, N, dh).  ``alive`` (B, N) bool or None.  The reference adds
    ``(1 - alive) * finfo(dtype).min / 2`` to the scores (attention.py:101-112):
    a dead key then has weight exactly 0 while any key of its environment is alive,
    and when none is alive all scores saturate to the same value, which makes the
    result the plain mean of v over every key of the environment.  The float32 sum absorbs
    the score of a dead key (|s| is far below the spacing of floats near the bias), so any
    huge negative bias gives the same bits; -1e30 is used here.
    """
    dh = q.shape[-1]
    bias = None if alive is None else (~alive[:, None, None, :]).to(q.dtype) * -1.0e30
    return _r(_AttentionLse.apply(q, k, v, bias, 1.0 / math.sqrt(dh)), mode)


def spatial_block(
    x: torch.Tensor,
    alive: torch.Tensor | None,
    p: Params,
    n_heads: int,
    mode: str,
    bullets: torch.Tensor | None = None,
    bullet_mask: torch.Tensor | None = None,
) -> torch.Tensor:
    """TransformerBlock.forward; attention.py:76-99,114-169.

    A sublayer reads bullets when its parameters hold ``kv_bullet.weight`` (the
    reference's ``reads_bullets``) and ``bullets`` (B, NB, D) is given: a second
    softmax over the environment's bullet keys, gated to zero for an environment with
    no active bullet when a mask is given, summed with the self-attention output
    before the shared output projection (attention.py:149-166).
    """
    B, N, D = x.shape
    dh = D // n_heads
    n = rms_norm(x, p["norm1.weight"])
    qkv = linear(n, p["qkv.weight"], None, mode)
    q, k, v = qkv.split(D, dim=-1)
    q = q.view(B, N, n_heads, dh).permute(0, 2, 1, 3)
    k = k.view(B, N, n_heads, dh).permute(0, 2, 1, 3)
    v = v.view(B, N, n_heads, dh).permute(0, 2, 1, 3)
    o = masked_attention(q, k, v, alive, mode)
    if bullets is not None and "kv_bullet.weight" in p:
        NB = bullets.shape[1]
        kvb = linear(rms_norm(bullets, p["norm_bullet.weight"]), p["kv_bullet.weight"], None, mode)
        kb, vb = kvb.split(D, dim=-1)
        kb = kb.view(B, NB, n_heads, dh).permute(0, 2, 1, 3)
        vb = vb.view(B, NB, n_heads, dh).permute(0, 2, 1, 3)
        ob = masked_attention(q, kb, vb, bullet_mask, mode)
        if bullet_mask is not None:
            ob = ob * bullet_mask.any(dim=-1)[:, None, None, None].to(ob.dtype)
        o = _r(o + ob, mode)
    o = o.permute(0, 2, 1, 3).reshape(B, N, D)
    x1 = x + linear(o, p["out_proj.weight"], None, mode)
    m = rms_norm(x1, p["norm2.weight"])
    return x1 + gated_mlp(m, p, "ffn.", mode)


# --------------------------------------------------------------------------- temporal


def conv_lag_validity(done: torch.Tensor) -> torch.Tensor:
    """(R, T) bool done flags -> (R, T) int count of valid past lags (0..3).

    griffin.py:67-93: output step t may read lag j only if no episode boundary lies
    in (t-j, t]; a boundary sits at t when done[t-1] (t >= 1); t = 0 continues the
    stored buffer, so all three stored lags are valid there.
    """
    R, T = done.shape
    valid = torch.empty(R, T, dtype=torch.int64)
    cur = torch.full((R,), CONV_KERNEL - 1, dtype=torch.int64)
    for t in range(T):
        if t >= 1:
            cur = torch.where(done[:, t - 1], torch.zeros_like(cur), (cur + 1).clamp(max=CONV_KERNEL - 1))
        valid[:, t] = cur
    return valid


def temporal_sequence(
    x_seq: torch.Tensor,
    h0: torch.Tensor,
    conv_buf: torch.Tensor,
    done: torch.Tensor | None,
    p: Params,
    mode: str,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """GriffinTemporalBlock.forward_sequence; griffin.py:249-286 with 169-219, 96-140.

    x_seq (R, T, D), h0 (R, D), conv_buf (R, 3, D) oldest first, done (R, T) bool | None.
    Returns out (R, T, D), final h (R, D), last three *unmasked* linear1 outputs (R, 3, D).
    """
    R, T, D = x_seq.shape
    n = rms_norm(x_seq, p["norm1.weight"])
    b1 = linear(n, p["linear1.weight"], None, mode)  # (R, T, D)
    padded = torch.cat([conv_buf.to(torch.float32), b1], dim=1)  # (R, T+3, D)
    w = p["conv.weight"].reshape(D, CONV_KERNEL)  # (D, 4); tap k reads lag 3-k
    cb = p["conv.bias"]
    lag_ok = conv_lag_validity(done) if done is not None else None

    u = torch.zeros(R, T, D)
    for k in range(CONV_KERNEL):
        tap = padded[:, k : k + T, :] * w[:, k]
        if lag_ok is not None:
            lag = CONV_KERNEL - 1 - k
            tap = tap * (lag_ok >= lag).to(tap.dtype).unsqueeze(-1)
        u = u + tap
    u = u + cb
    new_conv = padded[:, -(CONV_KERNEL - 1) :, :].clone()

    # RG-LRU gates (griffin.py:203-212).  Under autocast r and i are bf16, a is fp32.
    r = _r(torch.sigmoid(linear(u, p["rg_lru.linear_a.weight"], p["rg_lru.linear_a.bias"], mode)), mode)
    i = _r(torch.sigmoid(linear(u, p["rg_lru.linear_x.weight"], p["rg_lru.linear_x.bias"], mode)), mode)
    a = torch.sigmoid(p["rg_lru.log_lambda"]) ** (RGLRU_C * r)
    gate = torch.sqrt(torch.clamp((1.0 - a) * (1.0 + a), min=1e-6))
    b = gate * (i * u)
    if done is not None:
        reset = torch.zeros_like(done)
        reset[:, 1:] = done[:, :-1]
        a = a.masked_fill(reset.unsqueeze(-1), 0.0)

    h = h0.to(torch.float32)
    hs = []
    for t in range(T):
        h = a[:, t] * h + b[:, t]
        hs.append(h)
    b1_out = torch.stack(hs, dim=1)  # (R, T, D)

    b2 = _r(gelu_erf(linear(n, p["linear2.weight"], None, mode)), mode)
    x1 = x_seq + linear(b1_out * b2, p["linear_out.weight"], None, mode)
    x2 = x1 + gated_mlp(rms_norm(x1, p["norm2.weight"]), p, "gated_mlp.", mode)
    return x2, h, new_conv


def temporal_nonrecurrent(x: torch.Tensor, p: Params, sub_w: torch.Tensor, mode: str) -> torch.Tensor:
    """GriffinTemporalBlock.forward_nonrecurrent; griffin.py:288-317."""
    n = rms_norm(x, p["norm1.weight"])
    b1 = linear(linear(n, p["linear1.weight"], None, mode), sub_w, None, mode)
    b2 = _r(gelu_erf(linear(n, p["linear2.weight"], None, mode)), mode)
    x1 = x + linear(_r(b1 * b2, mode), p["linear_out.weight"], None, mode)
    return x1 + gated_mlp(rms_norm(x1, p["norm2.weight"]), p, "gated_mlp.", mode)


# --------------------------------------------------------------------------- blocks


def _sub(p: Params, prefix: str) -> dict[str, torch.Tensor]:
    return {k[len(prefix) :]: v for k, v in p.items() if k.startswith(prefix)}


def block_counts(p: Params) -> tuple[int, int]:
    """(n_spatial, n_temporal) read off the parameter names of one Yemong block."""
    ns = len({k.split(".")[1] for k in p if k.startswith("spatial.")})
    nt = len({k.split(".")[1] for k in p if k.startswith("temporal.")})
    return ns, nt


def yemong_block_sequence(
    x: torch.Tensor,
    alive: torch.Tensor | None,
    h0: torch.Tensor,
    conv0: torch.Tensor,
    done: torch.Tensor | None,
    n_rec: int | None,
    p: Params,
    n_heads: int,
    mode: str,
    bullets: torch.Tensor | None = None,
    bullet_mask: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """YemongBlock.sequence; griffin.py:419-472.

    x (T, B, NM, D), alive (T, B, NM) | None, h0 (nt, B*n_rec, D), conv0 (nt, B*n_rec, 3, D),
    done (T, B) | None, bullets (T*B, NB, D) | None, bullet_mask (T*B, NB) | None.
    """
    T, B, NM, D = x.shape
    n_rec = NM if n_rec is None else n_rec
    ns, nt = block_counts(p)
    for j in range(ns):
        a = None if alive is None else alive.reshape(T * B, NM)
        x = spatial_block(
            x.reshape(T * B, NM, D), a, _sub(p, f"spatial.{j}."), n_heads, mode, bullets, bullet_mask
        ).reshape(T, B, NM, D)
    done_rt = None if done is None else done.permute(1, 0).repeat_interleave(n_rec, dim=0)
    new_h, new_c = [], []
    for j in range(nt):
        tp = _sub(p, f"temporal.{j}.")
        ships, fields = x[:, :, :n_rec, :], x[:, :, n_rec:, :]
        seq = ships.permute(1, 2, 0, 3).reshape(B * n_rec, T, D)
        out, hT, cT = temporal_sequence(seq, h0[j], conv0[j], done_rt, tp, mode)
        ships = out.reshape(B, n_rec, T, D).permute(2, 0, 1, 3)
        if fields.shape[2]:
            fields = temporal_nonrecurrent(fields, tp, p[f"field_sub.{j}.weight"], mode)
        x = torch.cat([ships, fields], dim=2)
        new_h.append(hT)
        new_c.append(cT)
    if not new_h:
        return x, h0[:0], conv0[:0]
    return x, torch.stack(new_h), torch.stack(new_c)


def yemong_block_step(x, alive, h, conv, n_rec, p, n_heads, mode, bullets=None, bullet_mask=None):
    """YemongBlock.step; griffin.py:376-417 (the T = 1 case of the sequence, no done)."""
    y, nh, nc = yemong_block_sequence(
        x.unsqueeze(0), None if alive is None else alive.unsqueeze(0), h, conv, None, n_rec, p, n_heads, mode,
        bullets, bullet_mask,
    )
    return y.squeeze(0), nh, nc


# --------------------------------------------------------------------------- trunk


def unpack_hidden(hidden: torch.Tensor, D: int) -> tuple[torch.Tensor, torch.Tensor]:
    """(L, R, 4D) -> h (L, R, D), conv (L, R, 3, D) oldest first; policy.py:323-324."""
    L, R, _ = hidden.shape
    return hidden[:, :, :D], hidden[:, :, D:].reshape(L, R, CONV_KERNEL - 1, D)


def pack_hidden(h: torch.Tensor, conv: torch.Tensor) -> torch.Tensor:
    L, R, D = h.shape
    return torch.cat([h, conv.reshape(L, R, (CONV_KERNEL - 1) * D)], dim=-1)


def trunk_step(
    x: torch.Tensor,
    alive: torch.Tensor | None,
    hidden: torch.Tensor,
    blocks: Sequence[Params],
    n_heads: int,
    mode: str,
    bullets: torch.Tensor | None = None,
    bullet_mask: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Trunk loop of get_action_and_value; policy.py:315-354.

    x (B, NM, D) fp32, alive (B, NM) bool, hidden (L, B*n_rec, 4D) fp32,
    bullets (B, NB, D) | None and bullet_mask (B, NB) | None.
    Returns the trunk output (B, NM, D) and the repacked new hidden.
    """
    B, NM, D = x.shape
    n_rec = hidden.shape[1] // B if hidden.shape[0] else NM
    hs, cs = unpack_hidden(hidden, D)
    slot = 0
    new_h, new_c = [], []
    for p in blocks:
        _, nt = block_counts(p)
        x, nh, nc = yemong_block_step(
            x, alive, hs[slot : slot + nt], cs[slot : slot + nt], n_rec, p, n_heads, mode, bullets, bullet_mask
        )
        slot += nt
        new_h.append(nh)
        new_c.append(nc)
    if not new_h or sum(t.shape[0] for t in new_h) == 0:
        return x, hidden
    return x, pack_hidden(torch.cat(new_h), torch.cat(new_c))


def trunk_sequence(
    x: torch.Tensor,
    alive: torch.Tensor | None,
    hidden0: torch.Tensor,
    done: torch.Tensor | None,
    blocks: Sequence[Params],
    n_heads: int,
    mode: str,
    bullets: torch.Tensor | None = None,
    bullet_mask: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Trunk loop of evaluate_actions; policy.py:422-478.

    x (T, B, NM, D), alive (T, B, NM), hidden0 (L, B*n_rec, 4D), done (T, B) | None,
    bullets (T*B, NB, D) | None, bullet_mask (T*B, NB) | None.
    Returns the trunk output and the final hidden (the reference drops the latter).
    """
    T, B, NM, D = x.shape
    n_rec = hidden0.shape[1] // B if hidden0.shape[0] else NM
    hs, cs = unpack_hidden(hidden0, D)
    slot = 0
    new_h, new_c = [], []
    for p in blocks:
        _, nt = block_counts(p)
        x, nh, nc = yemong_block_sequence(
            x, alive, hs[slot : slot + nt], cs[slot : slot + nt], done, n_rec, p, n_heads, mode, bullets, bullet_mask
        )
        slot += nt
        new_h.append(nh)
        new_c.append(nc)
    if not new_h or sum(t.shape[0] for t in new_h) == 0:
        return x, hidden0
    return x, pack_hidden(torch.cat(new_h), torch.cat(new_c))


def reset_hidden_for_envs(hidden: torch.Tensor, done: torch.Tensor, n_rec: int) -> torch.Tensor:
    """Zero the packed state of every recurrent token of finished envs; policy.py:268-285."""
    keep = (~done.repeat_interleave(n_rec)).to(hidden.dtype)
    return hidden * keep[None, :, None]


def trunk_sequence_by_steps(x, alive, hidden0, done, blocks, n_heads, mode):
    """The sequence result built the slow way: one trunk_step per timestep with
    reset_hidden_for_envs after finished steps (tests/models/test_encoder.py:516-569).
    Only the per-step outputs are comparable with trunk_sequence; the final state of
    this loop has the last step's reset applied, the sequence's has not."""
    T = x.shape[0]
    B = x.shape[1]
    n_rec = hidden0.shape[1] // B
    hidden = hidden0
    outs = []
    for t in range(T):
        y, hidden = trunk_step(x[t], None if alive is None else alive[t], hidden, blocks, n_heads, mode)
        outs.append(y)
        if done is not None:
            hidden = reset_hidden_for_envs(hidden, done[t], n_rec)
    return torch.stack(outs), hidden


def trunk_step_ragged(
    x_flat: torch.Tensor,
    alive_flat: torch.Tensor,
    hidden: torch.Tensor,
    n_tokens: Sequence[int],
    n_ships: Sequence[int],
    blocks: Sequence[Params],
    n_heads: int,
    mode: str,
    bullets: torch.Tensor | None = None,
    bullet_mask: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Trunk step over environments of different sizes.

    The reference expresses one (ships, fields) split per call (griffin.py:398-399),
    so a mixed batch is evaluated by grouping environments of equal shape and calling
    the uniform path once per group.  x_flat (sum tokens, D) env-major, hidden
    (L, sum ships, 4D) env-major, bullets (n_envs, NB, D) / bullet_mask (n_envs, NB) optional.
    """
    D = x_flat.shape[-1]
    tok_off = [0]
    ship_off = [0]
    for nt, ns in zip(n_tokens, n_ships):
        tok_off.append(tok_off[-1] + nt)
        ship_off.append(ship_off[-1] + ns)
    y = torch.empty_like(x_flat)
    new_hidden = torch.empty_like(hidden)
    groups: dict[tuple[int, int], list[int]] = {}
    for e, key in enumerate(zip(n_tokens, n_ships)):
        groups.setdefault(key, []).append(e)
    for (nt, ns), envs in groups.items():
        tok_idx = torch.cat([torch.arange(tok_off[e], tok_off[e + 1]) for e in envs])
        ship_idx = torch.cat([torch.arange(ship_off[e], ship_off[e + 1]) for e in envs])
        xg = x_flat[tok_idx].reshape(len(envs), nt, D)
        ag = alive_flat[tok_idx].reshape(len(envs), nt)
        hg = hidden[:, ship_idx, :]
        bg = None if bullets is None else bullets[envs]
        mg = None if bullet_mask is None else bullet_mask[envs]
        yg, nhg = trunk_step(xg, ag, hg, blocks, n_heads, mode, bg, mg)
        y[tok_idx] = yg.reshape(-1, D)
        new_hidden[:, ship_idx, :] = nhg
    return y, new_hidden


# --------------------------------------------------------------------------- params


def split_trunk_state_dict(sd: Mapping[str, torch.Tensor], prefix: str = "yemong_layers.") -> list[dict[str, torch.Tensor]]:
    """Split a state dict with keys '<prefix>{i}.spatial.{j}...' into per-block dicts."""
    out: dict[int, dict[str, torch.Tensor]] = {}
    for k, v in sd.items():
        if not k.startswith(prefix):
            continue
        rest = k[len(prefix) :]
        i, name = rest.split(".", 1)
        out.setdefault(int(i), {})[name] = v.detach().to(torch.float32)
    return [out[i] for i in sorted(out)]


def synthetic_trunk_state_dict(d_model: int = 128, n_blocks: int = 2, n_spatial: int = 2, n_temporal: int = 1,
                               n_bullet_cross: int = 1, seed: int = 0) -> dict[str, torch.Tensor]:
    """A state dict with the trunk's keys and shapes (models/yemong/griffin.py:335-368,
    attention.py:51-74) and weights of the layers' fan-in scale, for timing the restatement where
    neither the reference's modules nor their init are at hand.  NOT the reference's init: its
    values match the reference in distribution only, which is all a timing needs."""
    g = torch.Generator().manual_seed(seed)
    D = d_model

    def lin(out_f: int, in_f: int) -> torch.Tensor:
        bound = in_f ** -0.5
        return (torch.rand(out_f, in_f, generator=g) * 2 - 1) * bound

    sd: dict[str, torch.Tensor] = {}
    for i in range(n_blocks):
        for j in range(n_spatial):
            p = f"yemong_layers.{i}.spatial.{j}."
            sd[p + "norm1.weight"] = torch.ones(D)
            sd[p + "qkv.weight"] = lin(3 * D, D)
            sd[p + "out_proj.weight"] = lin(D, D)
            if j < n_bullet_cross:
                sd[p + "norm_bullet.weight"] = torch.ones(D)
                sd[p + "kv_bullet.weight"] = lin(2 * D, D)
            sd[p + "norm2.weight"] = torch.ones(D)
            sd[p + "ffn.gate_proj.weight"] = lin(4 * D, D)
            sd[p + "ffn.up_proj.weight"] = lin(4 * D, D)
            sd[p + "ffn.down_proj.weight"] = lin(D, 4 * D)
        for j in range(n_temporal):
            p = f"yemong_layers.{i}.temporal.{j}."
            sd[p + "norm1.weight"] = torch.ones(D)
            sd[p + "linear1.weight"] = lin(D, D)
            sd[p + "conv.weight"] = (torch.rand(D, 1, 4, generator=g) * 2 - 1) * 0.5
            sd[p + "conv.bias"] = (torch.rand(D, generator=g) * 2 - 1) * 0.5
            sd[p + "rg_lru.log_lambda"] = torch.linspace(0, 4, D)
            for n in ("linear_a", "linear_x"):
                sd[p + f"rg_lru.{n}.weight"] = lin(D, D)
                sd[p + f"rg_lru.{n}.bias"] = (torch.rand(D, generator=g) * 2 - 1) * D ** -0.5
            sd[p + "linear2.weight"] = lin(D, D)
            sd[p + "linear_out.weight"] = lin(D, D)
            sd[p + "norm2.weight"] = torch.ones(D)
            sd[p + "gated_mlp.gate_proj.weight"] = lin(4 * D, D)
            sd[p + "gated_mlp.up_proj.weight"] = lin(4 * D, D)
            sd[p + "gated_mlp.down_proj.weight"] = lin(D, 4 * D)
            sd[f"yemong_layers.{i}.field_sub.{j}.weight"] = torch.eye(D)
    return sd


# --------------------------------------------------------------------------- encoders


def encoder_mlp(raw: torch.Tensor, w1, b1, g1, w2, b2, g2, mode: str) -> torch.Tensor:
    """Linear -> RMSNorm -> GELU -> Linear -> RMSNorm with biases, the chain of ShipEncoder's
    ``feature_extractor`` / ``ship_proj + shared_proj`` and BulletEncoder's ``net``
    (models/yemong/encoder.py:45-51, 84-90, 98-102).  Under autocast every stage hands on
    bfloat16: the Linear outputs, the RMSNorm of a bf16 input (computed in float32 with the
    float32 eps, rounded once) and the GELU."""
    h = linear(raw, w1, b1, mode)
    n = _r(rms_norm(h, g1), mode)
    a = _r(gelu_erf(n), mode)
    o = linear(a, w2, b2, mode)
    return _r(rms_norm(o, g2), mode)


def head_mlp(x: torch.Tensor, w1, b1, g1, w2, b2, mode: str) -> torch.Tensor:
    """Linear -> RMSNorm -> GELU -> Linear with biases: ``action_head``, ``value_head_local``,
    ``value_head_win`` and ``NextStateHead.net`` (models/yemong/policy.py:56-72, 185-206).  The
    encoder chain without its last norm."""
    h = linear(x, w1, b1, mode)
    n = _r(rms_norm(h, g1), mode)
    a = _r(gelu_erf(n), mode)
    return linear(a, w2, b2, mode)


# --------------------------------------------------------------------------- gradients


def trunk_sequence_grad(x, alive, hidden0, done, blocks, n_heads, dy, dhidden, bullets=None, bullet_mask=None,
                        mode: str = "fp32"):
    """Gradients of <trunk_sequence output, dy> + <final hidden, dhidden> by torch autograd over the
    restatement above: what ``loss.backward()`` computes through ``evaluate_actions``'s trunk loop
    (policy.py:422-478, train/rl/ppo.py:1974).  Returns (dx, dhidden0, dbullets | None, [per-block
    dict of parameter gradients])."""
    xg = x.detach().clone().requires_grad_(True)
    hg = hidden0.detach().clone().requires_grad_(True)
    bg = None if bullets is None else bullets.detach().clone().requires_grad_(True)
    leaves = [{k: v.detach().clone().requires_grad_(True) for k, v in p.items()} for p in blocks]
    y, nh = trunk_sequence(xg, alive, hg, done, leaves, n_heads, mode, bg, bullet_mask)
    loss = (y * dy).sum()
    if dhidden is not None:
        loss = loss + (nh * dhidden).sum()
    loss.backward()
    grads = [{k: (v.grad if v.grad is not None else torch.zeros_like(v)) for k, v in p.items()} for p in leaves]
    return xg.grad, hg.grad, None if bg is None else bg.grad, grads
