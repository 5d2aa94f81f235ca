"""The host-side choices of the kernel library that need no GPU: how the weight-streaming
product spreads K over its warps and how many warps its blocks have, and into how many shares of K the few-token tcgen05
product cuts the tiles that do not fill a round of the GPU.  The library loads without a
GPU (it is compiled at the first call, a few seconds, if this checkout has not built it
yet); without nvcc the tests are skipped."""
import ctypes

import pytest


@pytest.fixture(scope="module")
def lib():
    from zlm_b200.csrc.build import find_nvcc, library_path
    try:
        find_nvcc()
    except Exception as e:                          # no compiler here: nothing to test against
        pytest.skip(f"nvcc is not available: {e}")
    return ctypes.CDLL(library_path(build_if_needed=True, verbose=False))


@pytest.mark.parametrize("K,seg", [(4096, 512), (8192, 512), (12288, 512),          # multiples of 4096: 512, the order
                                   (1024, 128), (2048, 256), (3072, 384),            # the persistent kernel adds in
                                   (5120, 640), (25600, 640), (6144, 384), (7168, 128),
                                   (1000, 512), (520, 512), (4104, 512), (64, 512)])  # ragged: 512 and a tail
def test_gemv_segment_spreads_k_evenly(lib, K, seg):
    assert lib.zlm_gemv_segment(K) == seg
    if K % 1024 == 0:
        assert K % (8 * seg) == 0                   # whole chunks of 8 warps x seg columns: no warp idles


@pytest.mark.parametrize("N,K,narrow,warps", [
    (4096, 4096, 5, 8), (4096, 12288, 5, 8), (3072, 1024, 5, 8),   # one round of wide blocks: wide
    (6144, 4096, 5, 4),          # 384 blocks: the 88 after the first round of 296 would run alone
    (10240, 5120, 5, 4), (5120, 8192, 5, 4), (6144, 1024, 5, 4),
    (12800, 4096, 5, 8),         # 800 blocks: 740 narrow ones at once would leave 60 with half the loads in flight
    (24576, 4096, 5, 8),         # 1,536: five rounds of wide blocks and a short one, or two of narrow and a short one
    (24576, 4096, 4, 4),         # with two token tiles four narrow blocks fit: 592 + 592 + 352
    (10240, 5120, 4, 8),
])
def test_gemv_block_width_by_the_estimate_of_both_forms(lib, N, K, narrow, warps):
    """Each case was timed on a B200 in both forms; the estimate names the faster one (or either,
    where they were within a twentieth)."""
    assert lib.zlm_gemv_plan_warps(N, K, 148, 2, narrow) == warps
    assert lib.zlm_gemv_plan_warps(N, K, 0, 2, narrow) == 8        # nothing known about the device: wide


@pytest.mark.parametrize("T,N,K,shares", [
    (64, 6144, 4096, 3),        # 48 tiles: three shares fill 144 of 148 SMs
    (64, 4096, 4096, 4),        # 32 tiles x 4
    (64, 4096, 12288, 4),
    (64, 24576, 4096, 3),       # 192 tiles: 148 in one piece, 44 x 3 shares
    (64, 151936, 4096, 8),      # 1,187 tiles: 8 rounds in one piece, the last 3 tiles x 8
    (64, 18944, 4096, 1),       # 148 tiles: exactly one round, nothing to cut
    (300, 8000, 1024, 2),       # three token tiles per output tile; shares of at least 8 k blocks
    (40, 4096, 264, 1),         # K too short to cut
    (2048, 4096, 4096, 1),      # many tokens: the persistent forms, no shares
])
def test_few_token_shares_of_k(lib, T, N, K, shares):
    assert lib.zlm_gemm_tc_ksplit(T, N, K) == shares


def test_tcgen05_product_takes_what_tma_can_address(lib):
    assert lib.zlm_gemm_tc_supported(64, 4096, 4096, 4096) == 1
    assert lib.zlm_gemm_tc_supported(64, 4096, 4100, 4100) == 0      # rows of K elements must be 16-byte multiples
    assert lib.zlm_gemm_tc_supported(64, 4096, 4096, 4100) == 0


@pytest.mark.parametrize("T,N,K,width", [
    (2048, 4096, 4096, 240),     # 144 tiles of 240 on 74 pairs: two full rounds (128 of 256: the second 73 % full)
    (2048, 6144, 4096, 240),
    (2048, 24576, 4096, 256),    # 768 tiles: 11 rounds either way, the wide tile reuses the activations more
    (2048, 5120, 8192, 224),     # three rounds at every width: the narrowest of them
    (2048, 1024, 2048, 128),     # 32 tiles of 256 would leave more than half of the pairs idle
    (65143, 4096, 4096, 256),    # many rounds: the width hardly matters, so the widest
    (300, 4096, 4096, 0),        # few tokens: the other forms
])
def test_many_token_tile_width(lib, T, N, K, width):
    assert lib.zlm_gemm_tc_tile_width(T, N, K) == width


@pytest.mark.parametrize("R,max_new,nq,nkv,heads", [
    (1, 2048, 32, 8, 2),     # 256 blocks of two heads: enough for 148 SMs
    (1, 2048, 16, 8, 1),     # two heads per block would be 128 blocks, the longest twice as long
    (1, 8192, 16, 8, 2),     # long prompt: the spread work outweighs the longest block
    (1, 2048, 64, 8, 2),
    (1, 2048, 8, 8, 1),      # groups of one head
    (1, 2048, 24, 8, 1),     # odd groups
    (5, 300, 32, 8, 2),
    (64, 2048, 16, 8, 2),    # many prompts: plenty of blocks
])
def test_prefill_attention_heads_per_block(lib, R, max_new, nq, nkv, heads):
    assert lib.zlm_attention_prefill_tc_heads(R, max_new, nq, nkv) == heads


@pytest.mark.parametrize("rows,pages,want", [
    (8, 40, (7, 6)), (8, 48, (7, 7)), (8, 64, (7, 10)),        # 64 pairs: a part for every block the device holds
    (16, 64, (3, 22)), (24, 40, (2, 20)), (32, 64, (1, 64)), (48, 40, (1, 40)),   # but no second wave
    (1, 40, (10, 4)), (1, 64, (16, 4)), (1, 16, (8, 2)), (4, 64, (7, 10)),        # few pairs: fewer, longer parts
    (64, 40, (2, 24)), (64, 8, (1, 8)),                        # more pairs than the device holds: two waves
])
def test_decode_attention_cut(rows, pages, want):
    """The cut of the decode attention at 8 kv heads on a device that holds 444 blocks, as timed."""
    from zlm_b200.kernels import decode_splits
    splits, per = decode_splits(rows, 8, pages, 444)
    assert (splits, per) == want
    assert splits * per >= pages and (splits - 1) * per < pages      # the parts cover the pages, none is empty by design
    assert rows * 8 > 444 or splits * rows * 8 <= 444 * 1.1          # one wave of blocks wherever the pairs allow it


def test_decode_attention_cut_always_covers_the_pages():
    """Whatever the batch, the heads and the length: the parts cover every page, none of them is
    empty by design, and there are no more of them than the combine takes."""
    from zlm_b200.kernels import decode_splits
    for blocks in (444, 132 * 3, 8):
        for rows in (1, 2, 3, 4, 7, 8, 16, 17, 27, 28, 31, 32, 55, 56, 64, 200, 1024):
            for nkv in (1, 2, 5, 8, 16, 64):
                for pages in list(range(1, 70)) + [128, 500, 2048, 16384]:
                    splits, per = decode_splits(rows, nkv, pages, blocks)
                    assert per >= 1 and 1 <= splits <= 1024, (rows, nkv, pages, blocks, splits, per)
                    assert splits * per >= pages, (rows, nkv, pages, blocks, splits, per)
                    assert (splits - 1) * per < pages, (rows, nkv, pages, blocks, splits, per)
