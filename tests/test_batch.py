"""The step's descriptors on the host: packing, field alignment, the decode
context bucket, and the decode split choice (pure arithmetic, no GPU)."""

from reflex_b200.engine.batch import decode_context_bucket, layout, pack_host


def test_pack_host_lays_out_rows_and_wanted_places():
    tokens = [[5, 6, 7], [9], [1, 2]]
    words, offs, new_counts, row0, want_rows = pack_host(tokens, [4, 0, 2], [10, 0, 63], [[0, 2], [], [1]])
    assert new_counts == [3, 1, 2] and row0 == [0, 3, 4, 6] and want_rows == [0, 2, 5]

    def field(name):
        p, n = offs[name]
        return words[p:p + n].tolist()

    assert field("tokens") == [5, 6, 7, 9, 1, 2]
    assert field("row_pos") == [10, 11, 12, 0, 63, 64]
    assert field("row_slot") == [4, 4, 4, 0, 2, 2]
    assert field("seq_slot") == [4, 0, 2] and field("seq_start") == [10, 0, 63]
    assert field("seq_new") == [3, 1, 2] and field("seq_row0") == [0, 3, 4, 6]
    assert field("want_rows") == [0, 2, 5]
    # every field starts on 16 bytes (kernels read them with wide loads; TMA needs it)
    assert all(p % 4 == 0 for p, _ in offs.values())
    assert len(words) == layout(6, 3, 3)[1]


def test_decode_context_bucket_rounds_up_and_never_down():
    last = 0
    for ctx in range(1, 70000, 37):
        b = decode_context_bucket(ctx)
        assert b >= ctx and b % 64 == 0 and b >= last
        last = b
    assert decode_context_bucket(1) == 256 and decode_context_bucket(256) == 256
    assert decode_context_bucket(257) == 512 and decode_context_bucket(2048) == 2048
    assert decode_context_bucket(2049) == 4096 and decode_context_bucket(4097) == 8192


def test_decode_splits_grow_with_context_and_shrink_with_batch():
    from reflex_b200.ops import decode_splits

    for rows in (1, 8, 64):
        picks = [decode_splits(rows, 32, 8, pages) for pages in (1, 4, 16, 64, 256)]
        assert picks == sorted(picks) and picks[0] == 1
    for pages in (12, 64, 256):
        picks = [decode_splits(rows, 32, 8, pages) for rows in (1, 8, 64, 256)]
        assert picks == sorted(picks, reverse=True)
        assert all(1 <= s <= 64 and s <= pages for s in picks)
