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


def test_tile_width_of_the_tensor_core_product():
    """256 columns when the tiles fill most SMs, 128 when they do not, 192 where that saves a round of tiles."""
    from spissa_b200.parts.linear import tile_width
    assert tile_width(2048, 16384, 148) == 256          # 1,024 tiles: seven rounds either way
    assert tile_width(2048, 2048, 148) == 256           # 128 tiles: one round
    assert tile_width(2048, 3072, 148) == 192           # 192 tiles of 256 columns are two rounds, the second a third full
    assert tile_width(2048, 5120, 148) == 192
    assert tile_width(2048, 6144, 148) == 256           # three rounds of 256 against four of 192
    assert tile_width(300, 3072, 148) == 128            # 36 tiles of 256 columns leave most SMs idle
    assert tile_width(64, 3072, 148) == 128             # one row of tiles: never 192 (the kernel that splits K has no such tile)


def test_graph_table_evicts_the_graph_used_longest_ago():
    from spissa_b200.engine.graph import GraphTable

    class G:
        pass

    t = GraphTable(3)
    assert not t.wants_capture("a") and t.wants_capture("a")          # captured the second time a key is seen
    gone = []
    for k in "abc":
        t.put(k, G())
    assert t.get("a") is not None                                      # a is the most recently used now
    t.put("d", G(), before_evict=lambda g: gone.append(g))
    assert len(t) == 3 and t.get("b") is None and t.get("a") is not None and len(gone) == 1 and t.evictions == 1
    t.put("e", G())
    assert t.get("c") is None and {k for k in "ade" if t.get(k) is not None} == {"a", "d", "e"}
    for i in range(1000):                                              # sightings of keys that never come back
        t.wants_capture(("once", i))
    assert len(t.seen) <= 8 * 3 + 1
