"""The selection rule of the sparse-attention indexer, on the CPU oracle: the four cases of the
reference's tests/TinyTitan/Kernels/Attention/QSAIndexerTests.swift (budget 64, compress ratio 4,
selection width 67) with the same scores and the same expectations."""
import numpy as np

import oracle

RATIO, BUDGET = 4, 64
WIDTH = BUDGET + RATIO - 1


def test_inside_the_window_nothing_is_dropped():
    # QSAIndexerTests.swift:41-50: 67 visible keys are all kept, 68 are not
    assert WIDTH == 67
    keep, idx = oracle.qsa_select_keys(np.zeros(17, np.float32), 67, RATIO, WIDTH)
    assert keep.all() and len(idx) == 67
    keep, _ = oracle.qsa_select_keys(np.zeros(18, np.float32), 68, RATIO, WIDTH)
    assert keep.sum() == 67


def test_ragged_tail_is_kept_regardless_of_score():
    # :52-69: 103 visible = 25 complete blocks + 3 tail cells, every block scores 1000
    keep, idx = oracle.qsa_select_keys(np.full(26, 1000, np.float32), 103, RATIO, WIDTH)
    assert keep[100] and keep[101] and keep[102]
    assert keep.sum() == WIDTH and len(idx) == WIDTH


def test_budget_cuts_the_last_admitted_block():
    # :71-94: 68 visible, block 0 best ... block 16 worst: 16 whole blocks and 3 cells of the 17th
    scores = np.zeros(18, np.float32)
    scores[:17] = 17 - np.arange(17)
    keep, _ = oracle.qsa_select_keys(scores, 68, RATIO, WIDTH)
    assert keep.sum() == 67 and keep[64] and keep[66] and not keep[67]


def test_equal_scores_break_toward_the_lower_block():
    # :96-113: 72 visible, all scores equal: the lowest block indices win
    keep, idx = oracle.qsa_select_keys(np.full(19, 5, np.float32), 72, RATIO, WIDTH)
    assert keep.sum() == 67 and idx[0] == 0 and idx[-1] == 66


def test_pool_is_the_mean_of_the_members_present():
    # qsa.metal:14-35: a ragged last block divides by its own member count
    r = np.random.default_rng(0)
    raw = r.normal(size=(10, 128)).astype(np.float16).astype(np.float32)
    pooled = oracle.qsa_pool_blocks(raw, 4, 10, 0, 3)
    assert np.allclose(pooled[2], raw[8:10].mean(0), atol=2e-3)
    assert np.allclose(pooled[0], raw[0:4].mean(0), atol=2e-3)
    assert 3 not in oracle.qsa_pool_blocks(raw, 4, 10, 3, 1)


def test_scores_rectify_per_head_before_the_sum():
    # qsa.metal:67-96: a head that dislikes a block contributes nothing rather than cancelling another
    q = np.zeros((1, 2, 8), np.float32); q[0, 0, 0] = 1; q[0, 1, 0] = -1
    pooled = np.zeros((1, 8), np.float32); pooled[0, 0] = 3
    assert oracle.qsa_block_scores(q, pooled)[0, 0] == 3.0
