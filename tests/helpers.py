"""Shared pieces of the parity tests: golden loader, error metrics, module builders."""

from __future__ import annotations

import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Tolerances of the parity contract.
FP32_MAX_ABS = 1e-4        # float32 path: max |a - b|
BF16_NORM_MAX = 2e-2       # bf16 path: max |a - b| / max |ref|


def golden(name: str) -> dict:
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    return {k: torch.from_numpy(z[k]) for k in z.files}


def stored_weights(g: dict) -> dict:
    return {k[3:]: v for k, v in g.items() if k.startswith("w::")}


def checksum(sd) -> np.ndarray:
    tot = tot_abs = 0.0
    n = 0
    for k in sorted(sd):
        v = sd[k].detach().double()
        tot += float(v.sum())
        tot_abs += float(v.abs().sum())
        n += v.numel()
    return np.array([tot, tot_abs, float(n)])


def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double() - b.double()).abs().max())


def norm_err(a: torch.Tensor, ref: torch.Tensor) -> float:
    """max |a - ref| / max |ref|: the normalised error of the bf16 parity gate."""
    return max_abs(a, ref) / max(float(ref.abs().max()), 1e-30)


def assert_close(a, ref, mode: str, what: str = "", scale: float = 1.0) -> None:
    a = a.detach().cpu().float()
    ref = ref.detach().cpu().float()
    assert a.shape == ref.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(a).all(), f"{what}: non-finite values"
    if mode == "fp32":
        e = max_abs(a, ref)
        assert e <= FP32_MAX_ABS * scale, f"{what}: max abs error {e:.3e} > {FP32_MAX_ABS * scale:.1e}"
    else:
        e = norm_err(a, ref)
        assert e <= BF16_NORM_MAX * scale, f"{what}: normalised error {e:.3e} > {BF16_NORM_MAX * scale:.1e}"


def model_config(dims):
    from boost_and_broadside_b200 import ModelConfig

    D, H, nb, ns, nt, nbul = (int(v) for v in dims[:6])
    return ModelConfig(d_model=D, n_heads=H, n_yemong_blocks=nb, n_spatial_per_block=ns,
                       n_temporal_per_block=nt, n_bullet_cross_per_block=nbul)


def build_trunk(dims, g: dict | None = None):
    """The mirror trunk with the fixture's weights: seed-0 init, or the stored tensors."""
    from boost_and_broadside_b200 import YemongTrunk

    torch.manual_seed(0)
    trunk = YemongTrunk(model_config(dims)).eval()
    if g is not None:
        w = stored_weights(g)
        if w:
            trunk.load_state_dict(w, strict=True)
    return trunk


def trunk_params(trunk) -> list[dict]:
    from oracle.trunk_oracle import split_trunk_state_dict

    return split_trunk_state_dict(trunk.state_dict())


def autocast_for(mode: str, device: str):
    import contextlib

    if mode == "bf16":
        return torch.autocast(device, dtype=torch.bfloat16)
    return contextlib.nullcontext()


def grad_fixture_compare(g: dict, mode: str, dx, dhidden0, dbullets, named_grads: dict, tol: float):
    """Compare gradients with a grad_trunk_seq_* fixture (see make_golden.py: parameter gradients
    are stored in full up to 4096 elements, else as every ``stride``-th element plus sum and
    absolute sum).  Every tensor must be within ``tol`` normalised; returns the worst (name, error)."""
    stride = int(g["stride"][0])
    worst = ("", 0.0)

    def check(name, got, ref):
        nonlocal worst
        got = got.detach().cpu().float()
        assert got.shape == ref.shape, f"{name}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
        assert torch.isfinite(got).all(), f"{name}: non-finite gradient"
        e = norm_err(got, ref)
        assert e <= tol, f"{name}: normalised gradient error {e:.3e} > {tol:.1e}"
        if e > worst[1]:
            worst = (name, e)

    check("dx", dx, g["dx_" + mode])
    check("dhidden0", dhidden0, g["dhidden0_" + mode])
    if "dbullets_" + mode in g:
        check("dbullets", dbullets, g["dbullets_" + mode])
    seen = 0
    for key, ref in g.items():
        if key.startswith(f"g_{mode}::"):
            check(key[len(mode) + 4:], named_grads[key[len(mode) + 4:]], ref)
            seen += 1
        elif key.startswith(f"gsub_{mode}::"):
            name = key[len(mode) + 7:]
            got = named_grads[name].detach().cpu().float()
            check(name, got.flatten()[::stride], ref)
            sums = g[f"gsum_{mode}::{name}"]
            # the sums see every element; float32 summation order differs, so a loose gate
            assert abs(float(got.double().abs().sum()) - float(sums[1])) <= 1e-3 * float(sums[1]) + 1e-6, name
            seen += 1
    assert seen == len(named_grads), f"fixture holds {seen} parameter gradients, got {len(named_grads)}"
    return worst
