"""Replay of recorded real-serving routes (a sample of the reference's decode corpus,
tests/golden/tk_info.npz): the per-expert pair counts of four live launches — up to 25x the
mean on the hottest expert — are turned into routes exactly as the reference's replay does
(test/mega_common.cuh:460-482) on a world of 8 ranks x 32 experts, and the whole layer is
checked against the oracle: tables bit-exact, reduce bit-exact, end-to-end y within 1e-2."""
import os

import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tk_info.npz")


@pytest.mark.parametrize("which", [0, 1, 2, 3])
def test_recorded_routes_replay(which):
    from test_gpu_parity import _run_case
    g = np.load(GOLD)
    counts = g["counts"][which]
    R, EPR, topk = 8, 32, 8
    tokens = int(counts.sum()) // (R * topk)
    case = orc.gen_case(R, EPR, topk, 512, 256, tokens, seed=100 + which, routing="uniform", scaled=True)
    case = orc.with_routes(case, orc.routes_from_counts(counts, R, tokens, topk))
    # windows of 128 rows: the hottest expert of the skewed launches needs several
    assert counts.max() > 128 or which == 2
    _run_case(case, full_stage_checks=(which == 0))
