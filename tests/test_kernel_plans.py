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
            assert M <= 128 and block_q <= 128, (M, block_q)
            assert block_q >= min(M, 128) or (M > 32 and block_q in (32, 64)), "narrower token tiles only above 32 tokens"
            tiles = (N + 127) // 128
            token_tiles = (M + block_q - 1) // block_q
            assert splits == 1 or tiles * token_tiles * splits <= 148, "more CTAs than SMs stream the weights"
            for accumulate in (False, True):
                sw, bq, sp = kernels.gemm_tc_plan(M, N, K, accumulate)
                assert not sw or sp == 1 or tiles * ((M + bq - 1) // bq) * sp <= 148
        else:
            assert M > 32, "few tokens keep the weights on the 128-row side"
            assert splits <= 8
        assert (swap, block_q, splits) == kernels.gemm_tc_plan(M, N, K), "the plan depends on the sizes only"


def test_plans_between_33_and_128_tokens():
    """Token tiles of 32 for matrices of few row tiles (the forms with cluster reduce, early loads and rotation in the
    epilogue apply), the many-token form with ranges of K for a long K above 64 tokens."""
    assert kernels.gemm_tc_plan(64, 2048, 2048, True) == (True, 32, 4) and kernels.gemm_tc_plan(64, 3072, 2048) == (True, 32, 3)
    assert kernels.gemm_tc_plan(64, 16384, 2048) == (True, 64, 1)
    assert kernels.gemm_tc_plan(128, 2048, 2048, True) == (True, 32, 2) and kernels.gemm_tc_plan(128, 3072, 2048) == (True, 64, 1)
    assert kernels.gemm_tc_plan(128, 6144, 4096) == (True, 64, 1) and not kernels.gemm_tc_plan(128, 4096, 4096, True)[0]
    assert not kernels.gemm_tc_plan(128, 2048, 8192, True)[0]


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
    # up to 64 tokens in token tiles of 32 where the matrix has few row tiles; else product and rope+store kernel
    assert ok(33, 2048, 32, 8, 64, cos64, False) and ok(64, 2048, 32, 8, 64, cos64, False)
    assert not ok(48, 4096, 32, 8, 128, cos64, False), "48 row tiles: token tiles of 64"
    assert not ok(65, 2048, 32, 8, 64, cos64, False) and not ok(128, 2048, 32, 8, 64, cos64, False)
    # many tokens: whole heads, half-split pairing, enough tiles that K is not split
    assert ok(2048, 2048, 32, 8, 64, cos64, False) and ok(300, 192, 5, 1, 64, cos64, False)
    assert not ok(2048, 2048, 32, 8, 64, cos64, True), "interleaved pairs"
    assert not ok(2048, 2048, 32, 8, 64, cos32, False), "partial rotation"
    assert not ok(2048, 256, 4, 4, 16, cos_partial, False), "head size 16"
    assert not ok(256, 2048, 32, 8, 64, cos64, False), "K is split for so few tiles"
    assert not ok(2048, 2044, 32, 8, 64, cos64, False), "rows TMA cannot address"
