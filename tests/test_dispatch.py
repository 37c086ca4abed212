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
    # one request at a long context: up to 64 shares (128 CTAs of 16 tiles left half the machine idle)
    assert fast.decode_split_count(1, 4, 32768) == 57 and fast.decode_split_count(2, 4, 32768) == 37


def test_which_products_take_the_swapped_kernel():
    takes = fast._takes_swapped_kernel
    # decode batches up to 32 rows always, and nothing beyond what the kernel takes
    assert takes(1, 152064, 3584) and takes(32, 37888, 3584) and takes(8, 3584, 18944)
    assert not takes(1025, 3584, 18944) and not takes(2048, 3584, 3584)
    # wide products that fold themselves (gate/up, the head) fill the machine with tiles from 64 rows on
    assert not takes(64, 37888, 3584) and not takes(128, 17920, 1536) and not takes(128, 152064, 3584)
    # products that leave their partial sums to the reader (q/k/v, o, down) stay swapped through
    # decode steps of 256 requests at every width: measured in steps, 2 to 4 times faster there
    for N, K in ((2048, 1536), (1536, 1536), (1536, 8960), (4608, 3584), (3584, 3584), (3584, 18944),
                 (7168, 5120), (5120, 5120), (5120, 27648)):
        for M in (64, 128) + ((256,) if K < 5120 else ()):      # (the 32B widths were measured up to 128)
            assert takes(M, N, K, deferred=True), (M, N, K)
    # ... and as long as the MMAs do not bind (measured in prefill steps of 384 to 1,024 tokens:
    # 7B down 79 against 102 us at 512 rows, 123 against 113 us at 1,024)
    assert takes(512, 3584, 18944, deferred=True) and takes(384, 4608, 3584, deferred=True)
    assert not takes(1024, 3584, 18944, deferred=True) and not takes(1024, 4608, 3584, deferred=True)
    # folding itself, the swapped kernel keeps only long K onto few columns
    assert takes(128, 3584, 18944) and takes(128, 1536, 8960) and not takes(128, 2048, 1536) and not takes(192, 4608, 3584)


#: Times of products inside captured chains on a B200, microseconds (swapped, tiled) at 64, 128,
#: 256 and 512 rows: q/k/v, o, gate/up and down of the 1.5B, 7B and 32B widths, and the 7B head.
MEASURED_CHAINS = {
    (2048, 1536): [(13.7, 9.7), (20.5, 10.3), (36.7, 10.5), (41.4, 10.9)],
    (1536, 1536): [(14.0, 9.8), (20.7, 10.6), (37.6, 10.7), (38.3, 11.0)],
    (17920, 1536): [(22.3, 15.0), (29.7, 15.2), (45.7, 18.1), (87.0, 24.9)],
    (1536, 8960): [(22.4, 45.7), (32.9, 46.6), (57.3, 46.9), (46.8, 47.6)],
    (4608, 3584): [(16.6, 20.7), (21.7, 21.5), (34.6, 22.2), (35.6, 23.3)],
    (3584, 3584): [(18.3, 20.3), (24.9, 21.2), (42.2, 22.0), (42.2, 22.8)],
    (37888, 3584): [(52.6, 47.1), (82.3, 48.1), (125.6, 56.7), (248.8, 98.5)],
    (3584, 18944): [(40.5, 99.2), (47.4, 100.5), (70.2, 100.9), (104.3, 102.1)],
    (7168, 5120): [(24.2, 30.0), (38.9, 30.7), (53.1, 31.8), (43.3, 35.8)],
    (5120, 5120): [(20.8, 28.7), (32.2, 29.6), (45.2, 30.6), (58.2, 32.8)],
    (55296, 5120): [(108.2, 93.4), (146.8, 94.9), (219.5, 118.3), (437.3, 205.7)],
    (5120, 27648): [(62.1, 154.6), (98.3, 147.3), (117.9, 147.0), (187.4, 147.8)],
    (152064, 3584): [(190.3, 186.4), (260.4, 201.7), (390.6, 263.5), (771.1, 499.2)],
}


def test_the_rule_picks_the_faster_kernel_of_the_measured_chains():
    """No pick costs more than 25 % over the faster kernel, all picks together less than 2 %, and
    up to 256 rows (where the two kernels compete) each model is within 40 % of what was measured."""
    from axon_b200.kernels import lib
    model = lib.cuda().axon_gemm_modelled_us
    picked = best = 0.0
    for (N, K), cells in MEASURED_CHAINS.items():
        for M, (swapped, tiled) in zip((64, 128, 256, 512), cells):
            took = swapped if fast._takes_swapped_kernel(M, N, K) else tiled
            assert took <= 1.25 * min(swapped, tiled), (M, N, K, took)
            picked += took
            best += min(swapped, tiled)
            for kind, seen in ((0, swapped), (1, tiled)) if M <= 256 else ():
                got = model(kind, M, N, K, fast.SPLIT_TARGET_CTAS)
                assert abs(got - seen) <= 0.4 * seen, (M, N, K, "swapped tiled".split()[kind], got, seen)
    assert picked <= 1.02 * best
