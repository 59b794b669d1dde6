"""Host-side planning of the hierarchical window (no GPU compute): length groups and backbone spans follow the
reference's rules (src/gpu/hierarchical.rs:117-200, 245-261)."""
import importlib

H = importlib.import_module("neural-networks_b200.hier")


def test_groups_are_power_of_two_buckets_in_ascending_order():
    lens = [2, 3, 1, 4, 7, 2, 5, 1, 3, 9, 2, 4, 6, 16, 0]
    g = H.group_by_len(lens, cap=0)
    assert g == [[2, 7, 14], [0, 5, 10], [1, 3, 8, 11], [4, 6, 12], [9, 13]]  # buckets 1, 2, 4, 8, 16; 0 counts as 1
    assert sorted(w for grp in g for w in grp) == list(range(len(lens)))
    assert H.group_by_len(lens, no_group=True) == [list(range(len(lens)))]


def test_row_cap_cuts_a_bucket_into_same_shape_pieces_appended_behind_all_buckets():
    lens = [3] * 7 + [1] * 2
    # bucket 4 holds seven words of tmax 3: a cap of 8 rows allows 8 // (3 + 1) = 2 words a piece
    g = H.group_by_len(lens, cap=8)
    assert g == [[7, 8], [0, 1], [2, 3], [4, 5], [6]]
    assert H.group_by_len(lens, cap=0) == [[7, 8], [0, 1, 2, 3, 4, 5, 6]]
    assert H.group_by_len([5, 5, 5], cap=1) == [[0], [1], [2]]  # never less than one word a piece


def test_backbone_spans_are_balanced_and_tile_the_words():
    assert H.chunk_spans(12, 4) == [(0, 4), (4, 4), (8, 4)]
    assert H.chunk_spans(13, 5) == [(0, 5), (5, 4), (9, 4)]  # three near-equal pieces, not 5 + 5 + 3
    assert H.chunk_spans(5, 9) == [(0, 5)] and H.chunk_spans(5, 5) == [(0, 5)]
    for n in range(1, 40):
        for c in range(1, 12):
            spans = H.chunk_spans(n, c)
            assert spans[0][0] == 0 and sum(l for _, l in spans) == n and max(l for _, l in spans) <= max(c, 1)
            assert all(a + l == b for (a, l), (b, _) in zip(spans, spans[1:]))


def test_up_size_and_block_patterns_follow_the_reference():
    assert H.up_of(128) == 341 and H.up_of(384) == 1024
    cfg = H.HierCfg(vocab=256, hc=128, wh=384, enc_blocks=3, bb_blocks=10, dec_blocks=2, heads=8, dqk=48, w_token=255)
    assert (cfg.enc_kinds, cfg.bb_kinds, cfg.dec_kinds) == ("sms", "smmmmmmmsm", "sm")
    assert cfg.stage("enc")[1:] == (128, 16, 8, 8) and cfg.stage("bb")[1:] == (384, 8, 48, 48)
