"""Which kernel runs for which geometry: the host-side choices, without a GPU."""
import pytest

from llama_rs_metal_b200.kernels import attention_dispatch, gemm_dispatch


def _room(head_dim, size, rows):
    """Clusters a B200 holds at once: the region partials are sent into costs head size 64 its
    fourth CTA per SM."""
    per_sm = (4 if size == 1 else 3) if head_dim <= 64 else 2
    return per_sm * 148 // size


@pytest.fixture(autouse=True)
def every_cluster_size_launchable(monkeypatch):
    monkeypatch.setattr(attention_dispatch, "_resident_clusters", _room)


def test_cluster_size_fills_the_device_and_never_exceeds_the_pages():
    size = attention_dispatch.decode_cluster_size
    assert size(1, 8, 4, 64, 4096) == 14           # few sequences: the largest cluster
    assert size(8, 8, 4, 64, 4096) == 6            # 64 clusters x 6 = 384 CTAs, under 3 per SM
    assert size(64, 8, 4, 64, 4096) == 1           # 512 (sequence, head) pairs already fill it
    assert size(1, 8, 4, 64, 100) == 2             # two pages: no more CTAs than pages
    assert size(1, 8, 4, 64, 1) == 1
    assert size(8, 8, 4, 128, 4096) == 4           # head size 128: two CTAs per SM fit
    for seqs in (1, 3, 8, 20, 33, 64, 200):
        for keys in (1, 64, 65, 1000, 40000):
            s = size(seqs, 8, 4, 64, keys)
            assert 1 <= s <= attention_dispatch.MAX_CLUSTER and s <= max(1, -(-keys // 64))
            assert s == 1 or seqs * 8 * s <= 4 * 148      # what runs at once


def test_cluster_size_respects_what_the_device_can_launch(monkeypatch):
    monkeypatch.setattr(attention_dispatch, "_resident_clusters",
                        lambda head_dim, size, rows: _room(head_dim, size, rows) if size <= 5 else 0)
    assert attention_dispatch.decode_cluster_size(1, 8, 4, 64, 4096) == 5


def test_split_count_of_the_separate_kernels():
    splits = attention_dispatch.decode_splits
    assert splits(1, 8, 4, 4096, 0) == 64          # one page each
    assert splits(1, 8, 4, 131072, 0) == 74        # 592 CTAs over 8 pairs
    assert splits(64, 8, 4, 4096, 0) == 2
    assert splits(8, 8, 4, 4096, 64) == 2          # a window of 64 keys spans at most two pages
    assert splits(8, 8, 40, 4096, 0) == 4          # 40 query heads per kv head: three row groups per pair


def test_one_launch_or_three():
    fused = attention_dispatch.decode_prefers_fused
    assert fused(1, 8, 4, 64, 4096) and fused(8, 8, 4, 64, 4096) and fused(64, 8, 4, 64, 4096)
    assert fused(64, 8, 4, 64, 32768)              # bound by bandwidth either way: fewer launches win
    assert not fused(1, 8, 4, 64, 32768)           # 14 CTAs per pair would walk 37 pages each
    assert not fused(1, 8, 4, 64, 131072)
    assert not fused(2, 8, 4, 64, 65536) and not fused(4, 8, 4, 64, 65536)   # too few CTAs for the bandwidth
    assert fused(8, 8, 4, 64, 8192) and fused(1, 8, 4, 64, 16384)
    assert fused(32, 8, 4, 64, 16384) and fused(64, 8, 4, 64, 16384)         # many pairs: the splits get too few each
    attention_dispatch.force_cluster_size = 2      # tests pin the cluster size: always the one launch
    try:
        assert fused(1, 8, 4, 64, 131072)
    finally:
        attention_dispatch.force_cluster_size = None


def test_tile_shape_of_prompt_products():
    choice = gemm_dispatch.tile_choice              # 0: 128 x 128, 1: 128 x 256, 2: 256 x 256, 3: 128 x 192
    assert choice(2048, 16384, 2048, 3) == 1
    assert choice(2048, 3072, 2048, 0) == 3         # 192 tiles of 128 x 256 would fill 148 SMs 1.3 times: 256 of 128 x 192 do better
    assert choice(4096, 3072, 2048, 0) == 1
    assert choice(2048, 2048, 8192, 2) == 1         # 64 large tiles would leave most SMs idle
    assert choice(8192, 2048, 8192, 2) == 2         # long K: the 256 x 256 tile pays
    # with 74 pairs of SMs to be had, 256 x 256 tiles over pairs where they fill the pairs well
    assert choice(2048, 16384, 2048, 3, 74) == 4    # 512 tiles: 7 rounds of 74
    assert choice(2048, 2048, 8192, 2, 74) == 4     # 64 tiles in one round, long K
    assert choice(2048, 3072, 2048, 0, 74) == 3     # 96 tiles would take two rounds for 1.3 rounds' work
    assert choice(512, 3072, 2048, 0, 74) == 0      # 24 tiles would leave two thirds of the pairs idle
    assert choice(8192, 6144, 4096, 0, 74) == 4
    assert choice(2048, 2048, 2048, 2, 74) == 1     # one short tile per pair: the pair's start-up is not paid back
    assert choice(8192, 2048, 8192, 2, 74) == 4     # where pairs are to be had they replace the 256 x 256 tile
    assert choice(8192, 16384, 2048, 3) == 1        # short K and a costly epilogue: it does not
    assert choice(256, 2048) == 0                   # 32 small tiles keep more SMs busy than 16 or 8 larger ones
    assert choice(128, 128) == 0
    gemm_dispatch.umma_width = 128
    try:
        assert choice(2048, 16384, 2048, 3) == 0
    finally:
        gemm_dispatch.umma_width = None


def test_few_rows_plan():
    plan = gemm_dispatch._few_rows_plan
    assert plan(64, 16384, 2048, 3) == (True, 1)   # many column tiles: the tensor-core kernel as it is
    assert plan(64, 3072, 2048, 0) == (False, 1)   # few tiles and nothing to split: the streaming kernel
    use, slices = plan(64, 2048, 8192, 4)          # K slices as planes for the next norm to add
    assert use and 2 <= slices <= 64
    assert plan(64, 2048, 8192, 2) == (False, 1)   # added in place: never cut (nothing meets by atomics)
    assert plan(24, 2048, 2048, 4) == (False, 1)   # a small one streams


def test_sliced_plan_of_products_with_a_few_hundred_rows():
    plan = gemm_dispatch._sliced_plan                 # (tile: 0 = 128 x 128, 1 = 128 x 256; K slices)
    assert plan(128, 2048, 8192) == (0, 8)            # 16 tiles: eight slices fill 128 SMs, and the norm adds eight at a time
    assert plan(512, 2048, 8192) == (1, 4)            # 32 wide tiles in four slices
    assert plan(1024, 2048, 8192) == (1, 2)
    assert plan(2048, 2048, 8192) == (0, 1)           # enough tiles: added in place, no planes
    assert plan(768, 2048, 2048) == (0, 1)            # short K: the planes would cost more than the idle SMs
    for M in (65, 100, 300, 900):
        for N, K in ((2048, 2048), (2048, 8192), (4096, 14336), (520, 1000)):
            tile, splits = plan(M, N, K)
            assert tile in (0, 1) and 1 <= splits <= max(1, -(-K // 64) // 4)


def test_unequal_sequences_get_a_cluster_size_more():
    from llama_rs_metal_b200.engine.step import fill_class
    assert fill_class([100, 100, 99]) == 4 and fill_class([4000, 2000, 2100]) == 3
    assert fill_class([4000, 100, 100, 100]) == 2 and fill_class([8000] + [10] * 31) == 1
    assert fill_class([]) == 4 and fill_class([7]) == 4
    size = attention_dispatch.decode_cluster_size
    assert size(16, 8, 4, 64, 4096) == 3 and size(16, 8, 4, 64, 4096, fill=3) == 4   # 512 CTAs: some wait their turn
    assert size(8, 8, 4, 64, 4096, fill=3) == 7
    assert size(1, 8, 4, 64, 4096, fill=1) == 14                                        # one sequence is never unequal
    assert size(64, 8, 4, 64, 4096, fill=2) == 1                                        # 1,024 CTAs would be two full rounds
