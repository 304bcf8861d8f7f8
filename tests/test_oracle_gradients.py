"""The gradient oracle (torch autograd over the CPU restatement, oracle/trunk_oracle.py
``trunk_sequence_grad``) against gradients the reference's own autograd produced
(tests/golden/grad_trunk_seq_*.npz, written by tests/golden/make_golden.py): d x, d hidden0,
d bullets and every parameter gradient of <y, dy> + <new hidden, dhidden> through the sequence
forward of models/yemong/policy.py:422-478.

Tolerance: float32, normalised max error <= 1e-4 per tensor (max |a - b| / max |ref|; gradients
span orders of magnitude between tensors, so the absolute gate of the forward tests does not fit).
"""

from __future__ import annotations

import pytest
import torch

from oracle import trunk_oracle as O
from tests.helpers import build_trunk, checksum, golden, grad_fixture_compare, trunk_params

CASES = ["d128_t5_4s2f", "d128_t4_4s2f_nb12", "d64_t7_3s2f", "d128_t1_8s0f"]


@pytest.mark.parametrize("tag", CASES)
def test_oracle_gradients_match_the_reference_autograd(tag):
    g = golden("grad_trunk_seq_" + tag)
    trunk = build_trunk(g["dims"])
    assert abs(checksum(trunk.state_dict())[1] - float(g["wsum"][1])) < 1e-3 * float(g["wsum"][1])
    P = trunk_params(trunk)
    H = int(g["dims"][1])
    dx, dh0, db, grads = O.trunk_sequence_grad(g["x"], g["alive"], g["hidden"], g.get("done"), P, H, g["dy"], g["dhidden"],
                                               g.get("bullets"), g.get("bullet_mask"))
    named = {}
    for i, blk in enumerate(grads):
        for k, v in blk.items():
            named[f"yemong_layers.{i}.{k}"] = v
    worst = grad_fixture_compare(g, "fp32", dx, dh0, db, named, tol=1e-4)
    print(f"{tag}: worst normalised gradient error {worst[1]:.2e} ({worst[0]})")
