"""CPU tests of how the persistent matvec launch deals its CTAs out to the independent matrices of a step
(``matvec_chain_deal``, host arithmetic of the library: no device needed).  The deal decides how long the
benchmark's step takes - every group of CTAs should finish at the same time - so its properties are pinned here."""
import itertools

import pytest

from ullm_b200 import backend

Q4, Q6 = backend.Q4_K, backend.Q6_K
BLOCK = [(Q4, 8192, 8192), (Q4, 1024, 8192), (Q4, 1024, 8192), (Q4, 8192, 8192), (Q4, 28672, 8192), (Q4, 28672, 8192), (Q6, 8192, 28672)]


def model_time(mat, m, q6_cost=1.05):
    """The library's model of an op's time on m CTAs (matvec_chain.cu: fixed + work / m, in us)."""
    dt, out, cols = mat
    row_bytes = cols // 256 * (144 if dt == Q4 else 210)
    return 0.5 + cols * 7.0e-5 + out * row_bytes * (1.0 if dt == Q4 else q6_cost) / 33000.0 / m


def test_the_70b_block_on_148_ctas():
    deal = backend.chain_deal(BLOCK, 148)
    assert sum(deal) == 148 and min(deal) >= 1
    # the two 1024-row matrices get two CTAs each: with one, that CTA alone would outlast every other group
    assert deal[1] == 2 and deal[2] == 2
    assert deal[0] == deal[3] and deal[4] == deal[5]  # equal matrices, equal shares
    times = [model_time(m, n) for m, n in zip(BLOCK, deal)]
    big = [t for t, n in zip(times, deal) if n > 2]
    assert max(big) / min(big) < 1.12, times  # the large groups finish within a CTA's worth of each other


@pytest.mark.parametrize("world", [2, 4, 8])
def test_rank_shares_keep_every_matrix_served(world):
    mats = [(dt, out // world, cols) for dt, out, cols in BLOCK]
    deal = backend.chain_deal(mats, 148)
    assert sum(deal) == 148 and min(deal) >= 1
    assert deal[1] >= 2 and deal[2] >= 2


def test_the_deal_minimises_the_slowest_group():
    """Against brute force on small cases: no other split of the CTAs has a smaller largest group time."""
    mats = [(Q4, 512, 2048), (Q6, 256, 4096), (Q4, 4096, 1024)]
    for grid in (3, 7, 12):
        deal = backend.chain_deal(mats, grid)
        assert sum(deal) == grid
        mine = max(model_time(m, n) for m, n in zip(mats, deal))
        best = min(max(model_time(m, n) for m, n in zip(mats, split))
                   for split in itertools.product(range(1, grid), repeat=3) if sum(split) == grid)
        assert mine <= best * (1 + 1e-9)


def test_no_more_ctas_than_pairs_of_rows_and_argument_errors():
    deal = backend.chain_deal([(Q4, 4, 2048), (Q4, 4096, 2048)], 148)
    assert deal[0] <= 2 and sum(deal) == 148
    with pytest.raises(backend.UllmError):
        backend.chain_deal([(Q4, 64, 256)] * 3, 2)  # fewer CTAs than matrices
    with pytest.raises(backend.UllmError):
        backend.chain_deal([(backend.MLX_U32, 64, 1024)], 8)  # not a format of the persistent launch
