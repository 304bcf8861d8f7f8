"""The benchmark configurations at (or near) their full sizes, CUDA path against the CPU oracle.

At these sizes the launches are the ones bench.py times: many tiles per CTA, several waves, the
persistent loop of the tile kernel -- a reduced batch of a few dozen tiles never reaches them.
The oracle runs the full C2 and C3 batches in a few seconds on the host cores; C4 and C5 are
compared at a quarter of their environments (still thousands of tiles).

Every case also reports the argmax of the three action-logit slices (constants.py:46-48 of the
reference) of a fixed head applied to both outputs: flips outside near-ties must be zero, and the
number of near-tie rows is printed.
"""

from __future__ import annotations

import pytest
import torch

from oracle import trunk_oracle as O
from tests.helpers import assert_close, autocast_for, build_trunk, norm_err, trunk_params
from tests.test_gpu_parity import _head_argmax

pytestmark = pytest.mark.gpu
DEV = "cuda"
DIMS = [128, 4, 2, 2, 1, 1]


def _report(name, mode, y, ref_y, nh, ref_h):
    tol = 1e-3 if mode == "fp32" else 2e-2 * float(ref_y.abs().max())
    flips, ties = _head_argmax(ref_y, y.cpu(), tol)
    rows = ref_y.numel() // ref_y.shape[-1]
    print(f"{name} {mode}: y err {norm_err(y.cpu(), ref_y):.2e}" + (f" hidden err {norm_err(nh.cpu(), ref_h):.2e}" if nh is not None else "") +
          f"; argmax flips {flips}, near-tie rows {ties} of {3 * rows}")
    assert flips == 0, f"{name}: {flips} argmax flips outside {ties} near-tie rows"


@pytest.mark.parametrize("mode", ["bf16", "fp32"])
def test_c2_full_batch_against_the_oracle(mode):
    """8192 envs x 12 tokens: 820 tiles on 148 CTAs, the launch bench.py times."""
    from boost_and_broadside_b200 import workloads as W

    w = W.c2()
    trunk = build_trunk(DIMS)
    ref_y, ref_h = O.trunk_step(w.x, w.alive, w.hidden, trunk_params(trunk), 4, mode)
    trunk = trunk.to(DEV)
    with torch.no_grad(), autocast_for(mode, DEV):
        y, nh = trunk.step(w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV))
    assert_close(y, ref_y, mode, "C2 full y")
    assert_close(nh, ref_h, mode, "C2 full hidden")
    _report("C2 full", mode, y, ref_y, nh, ref_h)


def test_c3_full_batch_against_the_oracle():
    """1024 envs x 152 tokens, heavy key padding: the split-attention path at full size."""
    from boost_and_broadside_b200 import workloads as W

    w = W.c3()
    trunk = build_trunk(DIMS)
    ref_y, ref_h = O.trunk_step(w.x, w.alive, w.hidden, trunk_params(trunk), 4, "bf16")
    trunk = trunk.to(DEV)
    with torch.no_grad(), autocast_for("bf16", DEV):
        y, nh = trunk.step(w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV))
    assert_close(y, ref_y, "bf16", "C3 full y")
    assert_close(nh, ref_h, "bf16", "C3 full hidden")
    _report("C3 full", "bf16", y, ref_y, nh, ref_h)


def test_c4_quarter_batch_against_the_oracle():
    """T = 32 x 1024 envs x 8 ships with done flags: 2048 spatial tiles per sublayer, 64 tiles
    walking 32 timesteps each."""
    from boost_and_broadside_b200 import workloads as W

    w = W.c4(n_envs=1024, timesteps=32)
    trunk = build_trunk(DIMS)
    ref_y, ref_h = O.trunk_sequence(w.x, w.alive, w.hidden, w.done, trunk_params(trunk), 4, "bf16")
    trunk = trunk.to(DEV)
    with torch.no_grad(), autocast_for("bf16", DEV):
        y, nh = trunk.sequence(w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV), w.done.to(DEV))
    assert_close(y, ref_y, "bf16", "C4 y")
    assert_close(nh, ref_h, "bf16", "C4 hidden")
    _report("C4 1024 envs", "bf16", y, ref_y, nh, ref_h)


def test_c5_quarter_batch_against_the_oracle():
    """4096 ragged environments (2..128 tokens): about 2100 best-fit tiles."""
    from boost_and_broadside_b200 import RaggedBatch
    from boost_and_broadside_b200 import workloads as W

    w = W.c5(n_envs=4096)
    trunk = build_trunk(DIMS)
    ref_y, ref_h = O.trunk_step_ragged(w.x, w.alive, w.hidden, w.n_tokens.tolist(), w.n_ships.tolist(),
                                       trunk_params(trunk), 4, "bf16")
    trunk = trunk.to(DEV)
    with torch.no_grad(), autocast_for("bf16", DEV):
        y, nh = trunk.step_ragged(w.x.to(DEV), w.alive.to(DEV), w.hidden.to(DEV), RaggedBatch(w.n_tokens, w.n_ships))
    assert_close(y, ref_y, "bf16", "C5 y")
    assert_close(nh, ref_h, "bf16", "C5 hidden")
    _report("C5 4096 envs", "bf16", y, ref_y, nh, ref_h)
