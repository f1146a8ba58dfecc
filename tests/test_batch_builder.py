"""The packed arrays of a step (C++ BatchBuilder).  No GPU."""
import numpy as np
import pytest
import torch

from kvcm.cache import core


def seq_with_pages(sid, tokens, table, slot=0):
    s = core.Sequence()
    s.id = sid
    s.tokens = list(tokens)
    s.tables = [list(table)]
    s.state_slot = slot
    return s


def build(entries, B=4, max_blocks=8, tile=4, **pad):
    b = core.BatchBuilder(B, max_blocks, 1, tile)
    cap = b.capacity_for(64, 16, 64)
    buf = torch.zeros(cap, dtype=torch.int32)
    lay = b.build(entries, buf.data_ptr(), cap, **pad)
    return lay, buf.numpy()


def arr(buf, off, n):
    return buf[off:off + n].tolist()


def test_single_rows_first_then_portions_and_logit_rows_in_caller_order():
    a = seq_with_pages(1, range(100, 110), [5, 2, 7], slot=3)        # portion of 6 at 4..9
    d = seq_with_pages(2, range(200, 209), [1, 0, 4], slot=1)        # decode at position 8
    lay, buf = build([(a, 4, 6, [0, 5]), (d, 8, 1, [0])])
    assert (lay.rows, lay.seqs, lay.decode_seqs, lay.logit_rows) == (7, 2, 1, 3)
    assert lay.entry_order == [1, 0]
    assert arr(buf, lay.off_tokens, 7) == [208, 104, 105, 106, 107, 108, 109]
    assert arr(buf, lay.off_positions, 7) == [8, 4, 5, 6, 7, 8, 9]
    assert arr(buf, lay.off_row_seq, 7) == [0, 1, 1, 1, 1, 1, 1]
    # slot = page * B + offset
    assert arr(buf, lay.off_slot_mapping, 7) == [4 * 4 + 0, 2 * 4 + 0, 2 * 4 + 1, 2 * 4 + 2, 2 * 4 + 3, 7 * 4 + 0, 7 * 4 + 1]
    assert arr(buf, lay.off_seq_q_start, 2) == [0, 1]
    assert arr(buf, lay.off_seq_q_len, 2) == [1, 6]
    assert arr(buf, lay.off_seq_ctx_len, 2) == [9, 10]
    assert arr(buf, lay.off_seq_state_slot, 2) == [1, 3]
    assert arr(buf, lay.off_logit_rows, 3) == [1, 6, 0]              # a's places first: caller's order
    assert arr(buf, lay.off_block_tables, 16) == [1, 0, 4, -1, -1, -1, -1, -1, 5, 2, 7, -1, -1, -1, -1, -1]
    assert lay.prefill_tiles == 2 and arr(buf, lay.off_tile_seq, 2) == [1, 1] and arr(buf, lay.off_tile_q0, 2) == [0, 4]
    assert (lay.max_ctx, lay.max_decode_ctx, lay.max_q_len) == (10, 9, 6)


def test_padding_rows_read_and_write_nothing():
    d = seq_with_pages(2, range(9), [1, 0, 4])
    lay, buf = build([(d, 8, 1, [0])], pad_rows=4, pad_seqs=4, pad_logit_rows=4)
    assert (lay.rows, lay.seqs, lay.real_rows, lay.real_seqs, lay.logit_rows) == (4, 4, 1, 1, 4)
    assert arr(buf, lay.off_slot_mapping, 4) == [16, -1, -1, -1]
    assert arr(buf, lay.off_positions, 4) == [8, -1, -1, -1]         # context = position + 1 = 0
    assert arr(buf, lay.off_seq_ctx_len, 4) == [9, 0, 0, 0]
    assert arr(buf, lay.off_logit_rows, 4) == [0, 0, 0, 0]
    a = seq_with_pages(1, range(10), [5, 2, 7])
    with pytest.raises(Exception):
        build([(a, 0, 6, [])], pad_rows=8, pad_seqs=3)               # padding is for decode steps


def test_layout_of_a_padded_shape_is_fixed():
    d1 = seq_with_pages(1, range(9), [1, 0, 4])
    d2 = seq_with_pages(2, range(3), [6])
    l1, _ = build([(d1, 8, 1, [0])], pad_rows=4, pad_seqs=4, pad_logit_rows=4)
    l2, _ = build([(d1, 8, 1, [0]), (d2, 2, 1, [0])], pad_rows=4, pad_seqs=4, pad_logit_rows=4)
    for f in ("off_tokens", "off_slot_mapping", "off_logit_rows", "off_block_tables", "total_ints"):
        assert getattr(l1, f) == getattr(l2, f)


@pytest.mark.parametrize("entry, word", [
    ((0, 11, []), "outside"), ((9, 2, []), "outside"), ((0, 4, [4]), "wanted place"),
    ((0, 0, []), "outside"),
])
def test_inconsistent_entries_are_refused(entry, word):
    a = seq_with_pages(1, range(10), [5, 2, 7])
    with pytest.raises(Exception) as e:
        build([(a, *entry)])
    assert word in str(e.value)


def test_missing_page_is_refused():
    a = seq_with_pages(1, range(10), [5, -1, 7])
    with pytest.raises(Exception, match="no page"):
        build([(a, 4, 2, [])])
    build([(a, 8, 2, [])])                                           # page 1 is not touched: fine
