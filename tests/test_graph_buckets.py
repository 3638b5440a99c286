"""The length buckets that key captured decode steps: every length fits its bucket, buckets grow with the
length but never leave more than an eighth of a long bucket unused."""
from spissa_b200.engine.graph import length_bucket, wide_bucket


def test_buckets_hold_their_lengths_and_stay_tight():
    page = 64
    seen = set()
    for n in list(range(1, 3000)) + list(range(3000, 200000, 97)):
        b = length_bucket(n, page)
        w = wide_bucket(n, page)
        assert b >= n and b % page == 0
        assert w >= n and w & (w - 1) == 0 and w >= 4 * page
        if n > 8 * page:
            assert b - n < max(8 * page, n // 8 + page), (n, b)
        seen.add(b)
    assert len(seen) < 400                      # a capture every few hundred steps at most
    assert length_bucket(2048, page) == 2048 and length_bucket(2049, page) == 2560
    assert wide_bucket(2049, page) == 4096
