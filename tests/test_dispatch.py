"""Which kernel and how many CTAs a call gets: the host-side rules of ``kernels.fast`` that
follow sizes only (no GPU needed)."""

from axon_b200.kernels import fast


def test_decode_attention_never_starts_more_ctas_than_fit():
    for batch in (1, 2, 3, 8, 16, 31, 32, 64, 128, 300):
        for kv_heads in (1, 2, 4, 8):
            for kv_len in (1, 63, 64, 65, 500, 2048, 40000):
                s = fast.decode_split_count(batch, kv_heads, kv_len)
                tiles = -(-kv_len // 64)
                assert 1 <= s <= min(tiles, fast.FA_MAX_SPLITS)
                assert s == 1 or batch * kv_heads * s <= fast.FA_TARGET_CTAS
    # the sizes of the measurement: 8 requests x 4 kv heads share 256 CTAs
    assert fast.decode_split_count(8, 4, 2048) == 8
    assert fast.decode_split_count(64, 4, 2048) == 1
    assert fast.decode_split_count(1, 4, 2048) == 16        # 32 shares of one tile would only make the fold longer
    assert fast.decode_split_count(8, 4, 100) == 1          # two tiles: a second kernel to fold them costs more
    assert fast.decode_split_count(8, 4, 2080) == 7         # 33 tiles: 7 shares are as short as 8 (5 tiles)
    # between 32 and 37 requests two shares still fit at once, and halve the longest CTA
    assert fast.decode_split_count(36, 4, 2048) == 2 and fast.decode_split_count(24, 4, 2048) == 3
    assert fast.decode_split_count(38, 4, 2048) == 1


def test_which_products_take_the_swapped_kernel():
    # always for decode batches up to 64 rows
    assert fast._takes_swapped_kernel(1, 152064) and fast._takes_swapped_kernel(64, 37888)
    # beyond that only where 256 x 256 tiles would leave most SMs idle
    assert fast._takes_swapped_kernel(128, 3584) and fast._takes_swapped_kernel(256, 4608)
    assert not fast._takes_swapped_kernel(128, 37888)        # 148 tiles fill the machine
    assert fast._takes_swapped_kernel(1024, 3584)
    assert not fast._takes_swapped_kernel(1025, 3584) and not fast._takes_swapped_kernel(2048, 3584)
