"""The choices that depend on sizes only (no GPU needed): which form a matrix product takes, how
far K is split, and when rotation and page store ride in the product's epilogue."""
import pytest
import torch

from geneinfer_b200.ops import kernels


@pytest.mark.parametrize("N,K", [(3072, 2048), (2048, 2048), (16384, 2048), (2048, 8192), (128256, 2048), (5120, 3072),
                                 (4096, 14336), (200, 136), (64, 64)])
def test_product_plans_are_valid_for_every_token_count(N, K):
    for M in list(range(1, 140)) + [200, 256, 511, 512, 2048, 8192]:
        swap, block_q, splits = kernels.gemm_tc_plan(M, N, K)
        assert splits >= 1 and block_q in (16, 32, 64, 128, 256)
        k_blocks = (K + 63) // 64
        assert splits <= max(1, k_blocks), "a range of K without a block"
        if swap:
            assert M <= 128 and block_q >= min(M, 128) and block_q <= 128, (M, block_q)
            tiles = (N + 127) // 128
            assert splits == 1 or tiles * splits <= 148, "more CTAs than SMs stream the weights"
        else:
            assert M > 32, "few tokens keep the weights on the 128-row side"
            assert splits <= 8
        assert (swap, block_q, splits) == kernels.gemm_tc_plan(M, N, K), "the plan depends on the sizes only"


def test_many_tokens_split_k_only_while_tiles_are_few():
    assert kernels.gemm_tc_plan(2048, 2048, 8192) == (False, 256, 1)          # 128 tiles: no split
    swap, block_q, splits = kernels.gemm_tc_plan(512, 2048, 8192)             # 32 tiles: K in ranges
    assert not swap and block_q == 256 and 2 <= splits <= 8
    assert kernels.gemm_tc_plan(256, 128256, 2048)[2] == 1                    # the head: many tiles


def test_rotation_in_the_product_epilogue_is_taken_only_where_built():
    cos64, cos32, cos_partial = torch.zeros(8, 32), torch.zeros(8, 16), torch.zeros(8, 8)
    ok = kernels.gemm_rope_store_supported
    # few tokens: any rotation, the head size must divide 128
    assert ok(1, 2048, 32, 8, 64, cos64, False) and ok(32, 2048, 32, 8, 64, cos64, True)
    assert ok(8, 256, 4, 4, 16, cos_partial, False) and ok(8, 2048, 24, 8, 128, None, False)
    assert not ok(8, 240, 5, 5, 48, None, False) and not ok(8, 2048, 2, 1, 256, None, False)
    # between the two forms: product and rope+store kernel
    assert not ok(33, 2048, 32, 8, 64, cos64, False) and not ok(128, 2048, 32, 8, 64, cos64, False)
    # many tokens: whole heads, half-split pairing, enough tiles that K is not split
    assert ok(2048, 2048, 32, 8, 64, cos64, False) and ok(300, 192, 5, 1, 64, cos64, False)
    assert not ok(2048, 2048, 32, 8, 64, cos64, True), "interleaved pairs"
    assert not ok(2048, 2048, 32, 8, 64, cos32, False), "partial rotation"
    assert not ok(2048, 256, 4, 4, 16, cos_partial, False), "head size 16"
    assert not ok(256, 2048, 32, 8, 64, cos64, False), "K is split for so few tiles"
    assert not ok(2048, 2044, 32, 8, 64, cos64, False), "rows TMA cannot address"
