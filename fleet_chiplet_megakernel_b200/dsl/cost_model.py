"""Which way a linear layer is split over the GPU (python/mirage/mpk/dsl/cost_model.py of the reference).

The reference chooses between its standard tasks and the XCD-gang kernels of MI300.  On B200 the choice
is a function of the batch: the native runtime makes the same decision from ``max_num_batched_tokens``
when it lowers the graph, so these functions describe it (for tools and for the DSL's ``strategy="auto"``)
rather than steer it."""

B200_STRATEGIES = ("row_owner", "stream_k", "tcgen05")


def select_strategy(output_size, reduction_size, batch_size, target_cc=100, num_xcds=8, l2_per_xcd=4 * 1024 * 1024):
    """-> "row_owner" (1-2 tokens: every SM owns whole output rows over the full K, no cross-SM finish),
    "stream_k" (3-16 tokens: 128x128 weight tiles dealt as contiguous (row block, k) ranges, mma.sync),
    "tcgen05" (17+ tokens: the same tiles on the 5th-generation tensor cores with TMEM accumulators).
    For other architectures the answer is the reference's "standard"."""
    if target_cc != 100:
        return "standard"
    if batch_size <= 2:
        return "row_owner"
    if batch_size <= 16:
        return "stream_k"
    return "tcgen05"


def select_k_splits(reduction_size, m_tiles, workers_per_xcd=148, k_per_block=128):
    """How many CTAs share one 128-row block of a stream-K linear with ``m_tiles`` row blocks on
    ``workers_per_xcd`` SMs: the k-range of a block is cut where the contiguous tile ranges of the CTAs
    end, so about workers / row-blocks pieces (1: no block is split).  ``k_per_block`` is the k extent of a
    weight tile."""
    if m_tiles <= 0:
        return 1
    k_tiles = max(1, -(-reduction_size // k_per_block))
    return max(1, min(k_tiles, -(-workers_per_xcd // m_tiles)))
