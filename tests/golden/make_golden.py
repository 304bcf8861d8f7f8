"""Generate the golden input/output vectors under tests/golden/ from the reference itself.

Run once, on a machine that holds the reference source tree, as

    python tests/golden/make_golden.py --reference <path to the reference's src/>

It imports the reference's own ``TransformerBlock``, ``GriffinTemporalBlock`` and
``YemongBlock`` (models/yemong/attention.py, griffin.py), builds them with
``torch.manual_seed(0)`` and the module's default init, feeds seeded inputs, chains
blocks exactly as the policy does (models/yemong/policy.py:315-354 for a step,
422-478 for a sequence) and stores inputs, outputs and either the weights (small
widths) or a checksum of them (d_model = 128, where the mirror modules of this
repository must reproduce the same init from the same seed).

"bf16" cases run the reference under ``torch.autocast("cpu", dtype=torch.bfloat16)``,
the same context the trainer uses on the GPU (train/rl/ppo.py:1417).

The committed *.npz files are what the tests read; nothing at test time needs the
reference tree.
"""

from __future__ import annotations

import argparse
import contextlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def autocast(mode: str):
    if mode == "bf16":
        return torch.autocast("cpu", dtype=torch.bfloat16)
    return contextlib.nullcontext()


def checksum(sd) -> np.ndarray:
    tot = 0.0
    tot_abs = 0.0
    n = 0
    for k in sorted(sd):
        v = sd[k].detach().double()
        tot += float(v.sum())
        tot_abs += float(v.abs().sum())
        n += v.numel()
    return np.array([tot, tot_abs, float(n)], dtype=np.float64)


def team_alive(gen, B, n_ships, n_fields, p=0.9):
    """Ship alive ~ Bernoulli(p), first half team 0, second half team 1, at least one
    alive per team; field tokens always alive."""
    alive = torch.rand(B, n_ships, generator=gen) < p
    half = n_ships // 2
    for b in range(B):
        for lo, hi in ((0, half), (half, n_ships)):
            if hi > lo and not alive[b, lo:hi].any():
                alive[b, lo + int(torch.randint(0, hi - lo, (1,), generator=gen))] = True
    if n_fields:
        alive = torch.cat([alive, torch.ones(B, n_fields, dtype=torch.bool)], dim=1)
    return alive


ONLY = ""


def save(name, **arrays):
    if not name.startswith(ONLY):
        return
    out = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            v = v.detach().cpu().numpy()
        out[k] = v
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **out)
    print(f"{name}: {os.path.getsize(path) / 1024:.1f} KB")


def weights_as_arrays(sd, prefix="w::"):
    return {prefix + k: v.detach().clone() for k, v in sd.items()}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path to the src/ folder of the reference tree")
    ap.add_argument("--only", default="", help="write only the files whose name starts with this prefix")
    args = ap.parse_args()
    global ONLY
    ONLY = args.only
    sys.path.insert(0, args.reference)

    from boost_and_broadside.config import ModelConfig
    from boost_and_broadside.models.yemong.attention import TransformerBlock
    from boost_and_broadside.models.yemong.griffin import CONV_KERNEL, GriffinTemporalBlock, YemongBlock

    torch.set_num_threads(max(1, min(8, os.cpu_count() or 1)))

    def cfg(D, H, nb=2, ns=2, nt=1, nbul=0):
        return ModelConfig(
            d_model=D, n_heads=H, n_yemong_blocks=nb, n_spatial_per_block=ns,
            n_temporal_per_block=nt, n_bullet_cross_per_block=nbul,
        )

    # ------------------------------------------------------------------ spatial block
    for D, H, B, N, tag in (
        (128, 4, 12, 8, "d128_n8"),       # 4v4, no fields: the fp32 parity configuration
        (128, 4, 2, 152, "d128_n152"),    # 64 v 88 large fleet
        (64, 4, 3, 5, "d64_n5"),          # the reference's own unit-test width
        (32, 4, 4, 3, "d32_n3"),          # the trainer-test width (head dim 8)
        (32, 2, 3, 40, "d32h2_n40"),      # head dim 16, more keys than one warp
    ):
        torch.manual_seed(0)
        block = TransformerBlock(cfg(D, H)).eval()
        gen = torch.Generator().manual_seed(1)
        x = torch.randn(B, N, D, generator=gen)
        if N == 152:
            frac = torch.rand(B, 1, generator=gen) * 0.7
            alive = torch.rand(B, N, generator=gen) >= frac
            alive[:, 0] = True
            alive[:, 64] = True
        else:
            alive = team_alive(gen, B, N, 0)
            alive[B - 1] = False          # one environment with no live key at all
            if B > 2:
                alive[B - 2] = True
        out = {}
        for mode in ("fp32", "bf16"):
            with torch.no_grad(), autocast(mode):
                out["y_" + mode] = block(x, alive).float()
                out["y_nomask_" + mode] = block(x, None).float()
        extra = weights_as_arrays(block.state_dict()) if D < 64 else {}
        save(
            f"spatial_{tag}", x=x, alive=alive, dims=np.array([D, H]),
            wsum=checksum(block.state_dict()), **out, **extra,
        )

    # ------------------------------------------------------------------ temporal block
    for D, R, T, tag in ((128, 16, 1, "d128_t1"), (128, 6, 9, "d128_t9"), (64, 5, 6, "d64_t6")):
        torch.manual_seed(0)
        tb = GriffinTemporalBlock(D).eval()
        sub = torch.nn.Linear(D, D, bias=False)
        gen = torch.Generator().manual_seed(2)
        with torch.no_grad():
            # move the conv and gate parameters off their trivial values
            tb.conv.bias.copy_(torch.randn(D, generator=gen) * 0.1)
        x = torch.randn(R, T, D, generator=gen)
        h0 = torch.randn(R, D, generator=gen) * 0.5
        cb = torch.randn(R, CONV_KERNEL - 1, D, generator=gen) * 0.5
        done = torch.rand(R, T, generator=gen) < 0.25
        out = {}
        for mode in ("fp32", "bf16"):
            with torch.no_grad(), autocast(mode):
                y, h, c = tb.forward_sequence(x, h0, cb, None)
                out["y_" + mode], out["h_" + mode], out["c_" + mode] = y.float(), h.float(), c.float()
                if T >= 2:  # the reference's tap-validity builder needs T >= 2 (griffin.py:81-92)
                    y, h, c = tb.forward_sequence(x, h0, cb, done)
                    out["yd_" + mode], out["hd_" + mode], out["cd_" + mode] = y.float(), h.float(), c.float()
                out["yf_" + mode] = tb.forward_nonrecurrent(x, sub).float()
        sd = dict(tb.state_dict())
        sd["__sub.weight"] = sub.weight
        save(
            f"temporal_{tag}", x=x, h0=h0, conv=cb, done=done, dims=np.array([D]),
            conv_bias=tb.conv.bias, wsum=checksum(sd), **out,
            **(weights_as_arrays(sd) if D < 128 else {}),
        )

    # ------------------------------------------------------------------ trunk step / sequence
    def build_trunk(c):
        torch.manual_seed(0)
        return torch.nn.ModuleList([YemongBlock(c) for _ in range(c.n_yemong_blocks)]).eval()

    def ref_step(layers, c, x, alive, hidden, bullets=None, bullet_mask=None):
        """policy.py:315-354 restated with the reference's own blocks."""
        B, NM, D = x.shape
        L = hidden.shape[0]
        nt = c.n_temporal_per_block
        B_rec = hidden.shape[1]
        n_rec = B_rec // B
        hs = hidden[:, :, :D]
        cs = hidden[:, :, D:].reshape(L, B_rec, CONV_KERNEL - 1, D)
        nh, nc = [], []
        for i, layer in enumerate(layers):
            sl = slice(i * nt, (i + 1) * nt)
            x, h, cb = layer.step(x, alive, hs[sl], cs[sl], n_rec, bullets, bullet_mask)
            nh.append(h)
            nc.append(cb)
        new_h = torch.cat(nh, dim=0)
        new_c = torch.cat(nc, dim=0).reshape(L, B_rec, (CONV_KERNEL - 1) * D)
        return x, torch.cat([new_h, new_c], dim=-1)

    def ref_seq(layers, c, x, alive, hidden, done, bullets=None, bullet_mask=None):
        """policy.py:422-478 restated with the reference's own blocks."""
        T, B, NM, D = x.shape
        L = hidden.shape[0]
        nt = c.n_temporal_per_block
        B_rec = hidden.shape[1]
        n_rec = B_rec // B
        hs = hidden[:, :, :D]
        cs = hidden[:, :, D:].reshape(L, B_rec, CONV_KERNEL - 1, D)
        nh, nc = [], []
        for i, layer in enumerate(layers):
            sl = slice(i * nt, (i + 1) * nt)
            x, h, cb = layer.sequence(x, alive, hs[sl], cs[sl], done, n_rec, bullets, bullet_mask)
            nh.append(h)
            nc.append(cb)
        new_h = torch.cat(nh, dim=0)
        new_c = torch.cat(nc, dim=0).reshape(L, B_rec, (CONV_KERNEL - 1) * D)
        return x, torch.cat([new_h, new_c], dim=-1)

    step_cases = (
        # tag, cfg, B, ships, fields, store weights
        ("d128_8s4f", cfg(128, 4, 2, 2, 1, 1), 6, 8, 4, False),   # rollout step, 4v4 + 4 fields
        ("d128_8s0f", cfg(128, 4, 2, 2, 1, 1), 5, 8, 0, False),
        ("d128_30s2f", cfg(128, 4, 2, 2, 1, 1), 3, 30, 2, False),
        ("d64_3s2f", cfg(64, 4, 2, 2, 1, 0), 4, 3, 2, False),
        ("d32_2s1f_b132", cfg(32, 4, 1, 3, 2, 0), 3, 2, 1, True),
    )
    for tag, c, B, N, M, store in step_cases:
        layers = build_trunk(c)
        D = c.d_model
        gen = torch.Generator().manual_seed(3)
        x = torch.randn(B, N + M, D, generator=gen)
        alive = team_alive(gen, B, N, M)
        hidden = torch.randn(c.n_hidden_layers, B * N, CONV_KERNEL * D, generator=gen) * 0.5
        out = {}
        for mode in ("fp32", "bf16"):
            with torch.no_grad(), autocast(mode):
                y, nh = ref_step(layers, c, x, alive, hidden)
                out["y_" + mode], out["hidden_" + mode] = y.float(), nh.float()
        sd = {f"yemong_layers.{k}": v for k, v in layers.state_dict().items()}
        save(
            f"trunk_step_{tag}", x=x, alive=alive, hidden=hidden,
            dims=np.array([D, c.n_heads, c.n_yemong_blocks, c.n_spatial_per_block,
                           c.n_temporal_per_block, c.n_bullet_cross_per_block, N, M]),
            wsum=checksum(sd), **out, **(weights_as_arrays(sd) if store else {}),
        )

    seq_cases = (
        ("d128_t6_8s0f", cfg(128, 4, 2, 2, 1, 1), 6, 4, 8, 0, False),   # PPO minibatch forward shape
        ("d128_t5_4s2f", cfg(128, 4, 2, 2, 1, 1), 5, 3, 4, 2, False),
        ("d64_t7_3s2f", cfg(64, 4, 2, 2, 1, 0), 7, 2, 3, 2, False),
    )
    for tag, c, T, B, N, M, store in seq_cases:
        layers = build_trunk(c)
        D = c.d_model
        gen = torch.Generator().manual_seed(4)
        x = torch.randn(T, B, N + M, D, generator=gen)
        alive = team_alive(gen, T * B, N, M).reshape(T, B, N + M)
        hidden = torch.randn(c.n_hidden_layers, B * N, CONV_KERNEL * D, generator=gen) * 0.5
        done = torch.rand(T, B, generator=gen) < 0.3
        out = {}
        for mode in ("fp32", "bf16"):
            with torch.no_grad(), autocast(mode):
                y, nh = ref_seq(layers, c, x, alive, hidden, done)
                out["y_" + mode], out["hidden_" + mode] = y.float(), nh.float()
                y, nh = ref_seq(layers, c, x, alive, hidden, None)
                out["y_nodone_" + mode], out["hidden_nodone_" + mode] = y.float(), nh.float()
                # the reference's sequential construction: step + reset_hidden_for_envs
                hcur = hidden
                ys = []
                for t in range(T):
                    yt, hcur = ref_step(layers, c, x[t], alive[t], hcur)
                    ys.append(yt.float())
                    keep = (~done[t].repeat_interleave(N)).to(hcur.dtype)
                    hcur = hcur * keep[None, :, None]
                out["y_steps_" + mode] = torch.stack(ys)
        sd = {f"yemong_layers.{k}": v for k, v in layers.state_dict().items()}
        save(
            f"trunk_seq_{tag}", x=x, alive=alive, hidden=hidden, done=done,
            dims=np.array([D, c.n_heads, c.n_yemong_blocks, c.n_spatial_per_block,
                           c.n_temporal_per_block, c.n_bullet_cross_per_block, N, M]),
            wsum=checksum(sd), **out, **(weights_as_arrays(sd) if store else {}),
        )

    # ------------------------------------------------------------------ bullet cross-attention
    def bullet_inputs(gen, B, NB, D):
        """Encoded bullet tokens (the bullet encoder ends in an RMSNorm, so O(1) values) and
        the active mask: env 1 has nothing in flight, env 2 a full ring buffer."""
        bullets = torch.randn(B, NB, D, generator=gen)
        mask = torch.rand(B, NB, generator=gen) < 0.5
        if B > 1:
            mask[1] = False
        if B > 2:
            mask[2] = True
        return bullets, mask

    for D, H, B, N, NB, tag in ((128, 4, 6, 12, 80, "d128_n12_nb80"), (32, 4, 4, 3, 7, "d32_n3_nb7")):
        torch.manual_seed(0)
        block = TransformerBlock(cfg(D, H), reads_bullets=True).eval()
        gen = torch.Generator().manual_seed(5)
        with torch.no_grad():
            block.norm_bullet.weight.copy_(1.0 + 0.1 * torch.randn(D, generator=gen))
        x = torch.randn(B, N, D, generator=gen)
        alive = team_alive(gen, B, N, 0)
        bullets, mask = bullet_inputs(gen, B, NB, D)
        out = {}
        for mode in ("fp32", "bf16"):
            with torch.no_grad(), autocast(mode):
                out["y_" + mode] = block(x, alive, bullets, mask).float()
                out["y_nobmask_" + mode] = block(x, alive, bullets, None).float()
                out["y_nobullets_" + mode] = block(x, alive).float()
        save(
            f"bullets_spatial_{tag}", x=x, alive=alive, bullets=bullets, bullet_mask=mask, dims=np.array([D, H]),
            wsum=checksum(block.state_dict()), norm_bullet=block.norm_bullet.weight,
            **out, **(weights_as_arrays(block.state_dict()) if D < 64 else {}),
        )

    c = cfg(128, 4, 2, 2, 1, 1)
    layers = build_trunk(c)
    sd = {f"yemong_layers.{k}": v for k, v in layers.state_dict().items()}
    D = c.d_model
    dims = np.array([D, c.n_heads, c.n_yemong_blocks, c.n_spatial_per_block, c.n_temporal_per_block,
                     c.n_bullet_cross_per_block, 0, 0])

    B, N, M, NB = 5, 8, 4, 80
    gen = torch.Generator().manual_seed(6)
    x = torch.randn(B, N + M, D, generator=gen)
    alive = team_alive(gen, B, N, M)
    hidden = torch.randn(c.n_hidden_layers, B * N, CONV_KERNEL * D, generator=gen) * 0.5
    bullets, mask = bullet_inputs(gen, B, NB, D)
    out = {}
    for mode in ("fp32", "bf16"):
        with torch.no_grad(), autocast(mode):
            y, nh = ref_step(layers, c, x, alive, hidden, bullets, mask)
            out["y_" + mode], out["hidden_" + mode] = y.float(), nh.float()
    dims[6:] = (N, M)
    save("bullets_trunk_step_d128_8s4f", x=x, alive=alive, hidden=hidden, bullets=bullets, bullet_mask=mask,
         dims=dims.copy(), wsum=checksum(sd), **out)

    T, B, N, M, NB = 4, 3, 4, 2, 12
    gen = torch.Generator().manual_seed(7)
    x = torch.randn(T, B, N + M, D, generator=gen)
    alive = team_alive(gen, T * B, N, M).reshape(T, B, N + M)
    hidden = torch.randn(c.n_hidden_layers, B * N, CONV_KERNEL * D, generator=gen) * 0.5
    done = torch.rand(T, B, generator=gen) < 0.3
    bullets, mask = bullet_inputs(gen, T * B, NB, D)
    out = {}
    for mode in ("fp32", "bf16"):
        with torch.no_grad(), autocast(mode):
            y, nh = ref_seq(layers, c, x, alive, hidden, done, bullets, mask)
            out["y_" + mode], out["hidden_" + mode] = y.float(), nh.float()
    dims[6:] = (N, M)
    save("bullets_trunk_seq_d128_t4_4s2f", x=x, alive=alive, hidden=hidden, done=done, bullets=bullets,
         bullet_mask=mask, dims=dims.copy(), wsum=checksum(sd), **out)

    # ------------------------------------------------------------------ gradients (row f-3)
    # The sequence forward of policy.py:422-478 differentiated by the reference's own autograd:
    # loss = <y, dy> + <new hidden, dhidden> with seeded random cotangents.  Stored: inputs,
    # cotangents, d x, d hidden0, d bullets in full; each parameter gradient in full when it has at
    # most 4096 elements, else every 13th element of the flattened gradient plus its sum and
    # absolute sum (the full matrices would be megabytes per case).
    GRAD_STRIDE = 13

    def grad_case(tag, c, T, B, N, M, NB, seed, with_done=True):
        layers = build_trunk(c)
        D = c.d_model
        gen = torch.Generator().manual_seed(seed)
        x = torch.randn(T, B, N + M, D, generator=gen)
        alive = team_alive(gen, T * B, N, M).reshape(T, B, N + M)
        alive[0, 0, :N] = False          # one environment-step with every ship dead
        hidden = torch.randn(c.n_hidden_layers, B * N, CONV_KERNEL * D, generator=gen) * 0.5
        done = (torch.rand(T, B, generator=gen) < 0.3) if with_done else None
        bullets = mask = None
        if NB:
            bullets, mask = bullet_inputs(gen, T * B, NB, D)
        dy = torch.randn(T, B, N + M, D, generator=gen)
        dhid = torch.randn(c.n_hidden_layers, B * N, CONV_KERNEL * D, generator=gen)
        arrays = dict(x=x, alive=alive, hidden=hidden, dy=dy, dhidden=dhid)
        if done is not None:
            arrays["done"] = done
        if NB:
            arrays.update(bullets=bullets, bullet_mask=mask)
        for mode in ("fp32", "bf16"):
            xg = x.clone().requires_grad_(True)
            hg = hidden.clone().requires_grad_(True)
            bg = bullets.clone().requires_grad_(True) if NB else None
            for p_ in layers.parameters():
                p_.grad = None
            with autocast(mode):
                y, nh = ref_seq(layers, c, xg, alive, hg, done, bg, mask)
            ((y.float() * dy).sum() + (nh.float() * dhid).sum()).backward()
            arrays["dx_" + mode] = xg.grad
            arrays["dhidden0_" + mode] = hg.grad
            if NB:
                arrays["dbullets_" + mode] = bg.grad
            for name, p_ in layers.named_parameters():
                key = f"yemong_layers.{name}"
                g = p_.grad if p_.grad is not None else torch.zeros_like(p_)
                if g.numel() <= 4096:
                    arrays[f"g_{mode}::{key}"] = g.clone()
                else:
                    arrays[f"gsub_{mode}::{key}"] = g.flatten()[::GRAD_STRIDE].clone()
                    arrays[f"gsum_{mode}::{key}"] = torch.stack([g.double().sum(), g.double().abs().sum()])
        sd = {f"yemong_layers.{k}": v for k, v in layers.state_dict().items()}
        save(f"grad_trunk_seq_{tag}", dims=np.array([D, c.n_heads, c.n_yemong_blocks, c.n_spatial_per_block,
                                                     c.n_temporal_per_block, c.n_bullet_cross_per_block, N, M]),
             stride=np.array([GRAD_STRIDE]), wsum=checksum(sd), **arrays)

    grad_case("d128_t5_4s2f", cfg(128, 4, 2, 2, 1, 1), 5, 3, 4, 2, 0, seed=31)
    grad_case("d128_t4_4s2f_nb12", cfg(128, 4, 2, 2, 1, 1), 4, 3, 4, 2, 12, seed=32)
    grad_case("d64_t7_3s2f", cfg(64, 4, 2, 2, 1, 0), 7, 2, 3, 2, 0, seed=33)
    grad_case("d128_t1_8s0f", cfg(128, 4, 1, 1, 1, 0), 1, 4, 8, 0, 0, seed=34, with_done=False)

    # ------------------------------------------------------------------ encoders (rows f-2, f-4)
    # The MLP chains of ShipEncoder (shared and split layouts) and BulletEncoder
    # (models/yemong/encoder.py:25-130) on raw feature vectors of the coordinators' widths.
    from boost_and_broadside.config import ShipConfig
    from boost_and_broadside.models.yemong.encoder import BulletEncoder, ShipEncoder
    from boost_and_broadside.train.rl.features import FeatureScope, build_bullet_coordinator, build_standard_coordinator

    ships = ShipConfig()
    sc, bc = build_standard_coordinator(ships), build_bullet_coordinator(ships)
    gen = torch.Generator().manual_seed(21)
    torch.manual_seed(0)
    enc = ShipEncoder(cfg(128, 4), sc, num_ships=8).eval()
    raw = torch.randn(7, 12, sc.total_input_dimension, generator=gen) * 1.5
    out = {}
    for mode in ("fp32", "bf16"):
        with torch.no_grad(), autocast(mode):
            out["y_" + mode] = enc.feature_extractor(raw).float()
    save("encoder_ship_shared", raw=raw, **out, **weights_as_arrays(enc.state_dict()))

    torch.manual_seed(0)
    enc = ShipEncoder(ModelConfig(d_model=128, n_heads=4, n_yemong_blocks=2, encoder_split=True), sc, num_ships=8).eval()
    ship_raw = torch.randn(7, 8, sc.scoped_input_dimension(FeatureScope.SHIP), generator=gen) * 1.5
    field_raw = torch.randn(7, 4, sc.scoped_input_dimension(FeatureScope.FIELD), generator=gen) * 1.5
    out = {}
    for mode in ("fp32", "bf16"):
        with torch.no_grad(), autocast(mode):
            hidden = torch.cat([enc.ship_proj(ship_raw), enc.field_proj(field_raw)], dim=-2)
            out["y_" + mode] = enc.shared_proj(hidden).float()
    save("encoder_ship_split", ship_raw=ship_raw, field_raw=field_raw, **out, **weights_as_arrays(enc.state_dict()))

    torch.manual_seed(0)
    benc = BulletEncoder(cfg(128, 4, nbul=1), bc).eval()
    raw = torch.randn(5, 80, bc.total_input_dimension, generator=gen) * 1.5
    out = {}
    for mode in ("fp32", "bf16"):
        with torch.no_grad(), autocast(mode):
            out["y_" + mode] = benc.net(raw).float()
    save("encoder_bullet", raw=raw, **out, **weights_as_arrays(benc.state_dict()))

    # ------------------------------------------------------------------ heads (row f-4)
    # action_head, value_head_local, value_head_win and next_state_head.net of a stock YemongPolicy
    # (models/yemong/policy.py:56-72, 185-214) on trunk-like tokens.
    from boost_and_broadside.models.yemong.policy import YemongPolicy

    torch.manual_seed(0)
    policy = YemongPolicy(cfg(128, 4, nbul=1), sc, num_value_components=11, num_ships=8, team_pma_k=(0, 1),
                          bullet_coordinator=bc).eval()
    x = torch.randn(9, 8, 128, generator=gen) * 1.5
    arrays = {"x": x}
    heads = {"action_head": policy.action_head, "value_head_local": policy.value_head_local,
             "value_head_win": policy.value_head_win, "next_state_head": policy.next_state_head.net}
    for name, head in heads.items():
        for mode in ("fp32", "bf16"):
            with torch.no_grad(), autocast(mode):
                arrays[f"{name}_{mode}"] = head(x).float()
        arrays.update(weights_as_arrays(head.state_dict(), prefix=f"w::{name}."))
    save("policy_heads", **arrays)


if __name__ == "__main__":
    main()
