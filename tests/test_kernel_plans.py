"""The host-side choices of grids for the decode kernels (no GPU needed): every choice must be one
that the kernels accept, whatever sizes a configuration brings."""

import itertools

from tokamak_b200.csrc import ops


def test_decode_splits_stay_in_one_wave_and_keep_the_warps_level():
    for n_items, hkv, kv_len in itertools.product((1, 2, 3, 4, 7, 8, 16, 37, 64, 300), (1, 2, 5, 8, 16),
                                                  (1, 15, 16, 17, 100, 1024, 4096, 40000, 131072)):
        s = ops.decode_splits(n_items, hkv, kv_len)
        assert 1 <= s <= 128
        tiles = -(-kv_len // 16)
        if s > 1:
            assert n_items * hkv * s <= 444                      # one wave: three blocks of two stages per SM
            per_split = -(-tiles // s)
            assert per_split >= 8                                # a block has enough to stream
            assert s * per_split >= tiles
    # the measured cases
    assert ops.decode_splits(8, 8, 4096) == 6            # 384 blocks: two stages, three to an SM
    assert ops.decode_splits(16, 8, 4096) == 3
    assert ops.decode_splits(1, 8, 4096) == 32           # 256 blocks: three stages, two to an SM
    assert ops.decode_splits(32, 8, 4096) == 1
    assert ops.decode_splits(64, 8, 4096) == 1


def test_swapped_gemm_plan_is_one_cluster_of_at_most_eight():
    for n_out, k, tokens in itertools.product((128, 1000, 4096, 6144, 24576, 34816, 151936), (64, 320, 1024, 4096, 17408),
                                              (1, 8, 16, 17, 64)):
        splits, stages, cluster = ops.swapped_gemm_plan(n_out, k, tokens)
        assert 1 <= splits <= 8 and cluster == splits
        assert stages in (3, 4)
        assert splits <= max(1, -(-k // 64))                      # no split without a k block
    # the shapes of the Qwen3-8B decode step at batch 8: q|k|v, output, gate/up, down, head
    assert ops.swapped_gemm_plan(6144, 4096, 8) == (8, 4, 8)
    assert ops.swapped_gemm_plan(4096, 4096, 8) == (8, 4, 8)
    assert ops.swapped_gemm_plan(24576, 4096, 8) == (2, 4, 2)
    assert ops.swapped_gemm_plan(4096, 12288, 8) == (8, 4, 8)
    assert ops.swapped_gemm_plan(151936, 4096, 8) == (1, 4, 1)
    # larger token tiles have larger stages: four of them only where two blocks per SM are enough
    assert ops.swapped_gemm_plan(151936, 4096, 64)[1] == 3
    assert ops.swapped_gemm_plan(4096, 4096, 64)[1] == 4


def test_pair_gemm_is_for_grids_that_fill_the_gpu():
    assert ops.pair_gemm_takes(2048, 4096, 4096)
    assert not ops.pair_gemm_takes(256, 4096, 4096)               # 16 tiles: the library is faster
    assert not ops.pair_gemm_takes(2048, 4096, 4100)              # inner size no multiple of 8


def test_sampling_refuses_sizes_its_histograms_cannot_hold():
    import pytest
    ops._sampling_takes(64, 151936)
    ops._sampling_takes(ops.SAMPLING_MAX_ROWS, ops.SAMPLING_MAX_VOCAB)
    with pytest.raises(ops.KernelError, match="sampling kernel takes"):
        ops._sampling_takes(1, ops.SAMPLING_MAX_VOCAB + 1)
    with pytest.raises(ops.KernelError, match="sampling kernel takes"):
        ops._sampling_takes(ops.SAMPLING_MAX_ROWS + 1, 1000)
