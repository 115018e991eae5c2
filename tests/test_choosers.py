"""The host-side rules that pick tile widths and slice counts: pure arithmetic,
checked without a GPU against the properties the kernels rely on."""
from types import SimpleNamespace

import numpy as np

from infernum_b200.cache import CacheManager
from infernum_b200.ops import attention_fast, gemm_tc
from infernum_b200.parts.base import PagedCacheSpec


def test_pair_tiling_is_one_the_kernel_accepts_and_never_worse_than_full_width():
    def cost(T, N, tiling, pairs=74):
        bn_a, cols_a, bn_b = tiling
        t_tiles = -(-T // 256)
        cols_a = min(cols_a, -(-N // bn_a))
        rest = max(0, N - cols_a * bn_a)
        tiles = [bn_a] * (cols_a * t_tiles) + [bn_b] * (-(-rest // bn_b) * t_tiles if rest else 0)
        load = [0] * pairs
        for i, w in enumerate(tiles):
            load[i % pairs] += w + gemm_tc.PAIR_TILE_OVERHEAD
        return max(load)

    for T in (200, 256, 512, 1000, 2048, 5000):
        for N, sw in ((4096, False), (6144, False), (28672, True), (1000, False), (128256, False), (384, True)):
            t = gemm_tc.choose_pair_tiling(T, N, 148, sw)
            step = 128 if sw else 16
            assert t[0] % step == 0 and t[2] % step == 0 and 32 <= t[0] <= 256 and 32 <= t[2] <= 256
            assert 0 <= t[1] <= -(-N // t[0])
            assert cost(T, N, t) <= cost(T, N, (256, 1 << 20, 256))


def test_which_products_go_to_the_pair_kernel():
    assert not gemm_tc.pair_suits(64) and not gemm_tc.pair_suits(520) and not gemm_tc.pair_suits(512)
    assert gemm_tc.pair_suits(768) and gemm_tc.pair_suits(2048) and gemm_tc.pair_suits(2056)
    # the gate/up product with its activation pays from one full tile of tokens on
    assert gemm_tc.pair_suits(256, fused_activation=True) and gemm_tc.pair_suits(512, fused_activation=True)
    assert not gemm_tc.pair_suits(320, fused_activation=True) and not gemm_tc.pair_suits(100, fused_activation=True)


def test_decode_slices_fill_idle_sms_and_never_oversubscribe_a_cluster():
    for n in (1, 2, 3, 4, 8, 16, 32, 64, 200):
        for kv in (64, 300, 1100, 4096, 32768):
            s = attention_fast.choose_splits(n, 8, kv, 148)
            tiles = -(-kv // 64)
            assert 1 <= s <= max(1, tiles) or s in (16, 24)
            if 2 * n * 8 > 296:
                assert s == 1           # the grid fills the SMs without slices
            if s > 8:
                assert tiles >= 128    # a second kernel merges: only for very long requests
    assert attention_fast.choose_splits(8, 8, 1100, 148) == 4
    assert attention_fast.choose_splits(64, 8, 4096, 148) == 1


def test_prompt_slices_only_when_row_tiles_leave_sms_idle():
    rt = SimpleNamespace(options={"sm_count": 148})
    f = attention_fast.choose_prompt_splits
    assert f([2048], 32, 8, 2048, rt) == 1            # 512 CTAs: plenty
    assert f([512], 32, 8, 4096, rt) == 2             # 128 CTAs, 64 key tiles each
    assert f([256], 32, 8, 4096, rt) == 4
    assert f([512], 32, 8, 512, rt) == 1              # too few key tiles to share out
    assert f([1] * 16 + [512], 32, 8, 4096, rt, small_limit=2) == 2   # decoded tokens do not count
    assert f(None, 32, 8, 4096, rt) == 1


def test_block_table_mirrors_follow_every_change():
    need = SimpleNamespace(position=0, paged=PagedCacheSpec(1, 8, 5), state=None, cache_of=None)
    cache = CacheManager([need], page_size=4, num_pages=16, max_requests=2)
    rc = cache.admit("a")
    assert rc.serial == 1 and [list(t) for t in rc.table_arrays()] == [[]]
    cache.extend(rc, 9)
    first = rc.table_arrays()
    assert first[0].dtype == np.int32 and list(first[0]) == rc.tables[0] and len(first[0]) == 3
    assert rc.table_arrays() is first                  # unchanged tables: the same arrays
    cache.commit(rc, 9)                                # window 5: the first page is given back
    assert rc.tables[0][0] == -1 and list(rc.table_arrays()[0]) == rc.tables[0]
    cache.extend(rc, 1)
    cache.commit(rc, 1)
    assert list(rc.table_arrays()[0]) == rc.tables[0]
    cache.release(rc)
    again = cache.admit("a")
    assert again.serial == 2 and again is not rc
    cache.check_invariants()


def test_token_groups_are_even_and_bounded():
    """Groups of token tiles keep the tokens of a round inside the byte bound,
    never fewer than two tiles, and are evened out over the prompt."""
    from infernum_b200.ops import gemm_tc
    bound, most = gemm_tc.POLICY["pair_group_bytes"], gemm_tc.POLICY["pair_group_max_tiles"]
    for T in (256, 600, 2048, 2049, 4096, 5000, 8192, 16384, 40000):
        for K in (64, 4096, 14336, 28672, 200000):
            tg = gemm_tc.choose_token_group(T, K)
            t_tiles = -(-T // 256)
            assert 1 <= tg <= max(2, most)
            assert tg <= 2 or tg * 256 * K * 2 <= bound
            groups = -(-t_tiles // tg)
            assert groups * tg - t_tiles < groups  # no group more than one tile short
    assert gemm_tc.choose_token_group(2048, 4096) == 8      # one group: as before there were groups
    assert gemm_tc.choose_token_group(2048, 14336) == 8
    assert gemm_tc.choose_token_group(8192, 14336) == 8     # four groups of 2,048 tokens
