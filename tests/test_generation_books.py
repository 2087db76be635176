"""The generation loop's books in the native host runtime (no GPU): what a request has generated, whether
it goes on, which requests fit the cache together (model.rs:373-442 per request of a batch)."""
import pytest

from rust_inference_b200.cache.pager import SlotPager
from rust_inference_b200.engine.books import LENGTH, LIVE, STOP, GenerationBooks


def test_tokens_stops_and_lengths():
    b = GenerationBooks(max_tokens=3, max_seq_len=100, stop_ids=[9, 7])
    assert [b.add([1, 2]), b.add([3]), b.add([4, 5, 6])] == [0, 1, 2]
    assert b.book([0, 1, 2], [11, 9, 12]) == [LIVE, STOP, LIVE]          # a stop id ends its request and is not kept
    assert b.tokens(1) == [] and b.finish_reason(1) == "stop" and b.finish_reason(0) is None
    assert b.book([0, 2], [13, 7]) == [LIVE, STOP]
    assert b.book([0], [14]) == [LENGTH]                                  # the third token is the last
    assert b.tokens(0) == [11, 13, 14] and b.finish_reason(0) == "length" and b.token_count(2) == 1
    with pytest.raises(ValueError, match="ended already"):
        b.book([0], [1])
    with pytest.raises(ValueError, match="does not exist"):
        b.book([5], [1])


def test_no_position_left_is_a_length_end():
    b = GenerationBooks(max_tokens=50, max_seq_len=70)
    b.add([1] * 68)
    # positions 68 and 69 can still be fed: the tokens drawn first and second go on, the third has nowhere to go
    assert b.goes_on([0, 0, 0], [1, 2, 3]) == [True, True, False]
    assert b.book([0], [5]) == [LIVE] and b.book([0], [5]) == [LIVE] and b.book([0], [5]) == [LENGTH]
    with pytest.raises(ValueError, match="exceeds max_seq_len"):
        b.add([1] * 71)
    with pytest.raises(ValueError, match="empty prompt"):
        b.add([])


def test_goes_on_knows_lengths_not_stops():
    b = GenerationBooks(max_tokens=4, max_seq_len=100, stop_ids=[9])
    b.add([1])
    assert b.goes_on([0] * 5, [0, 1, 3, 4, 5]) == [True, True, True, False, False]


def test_admission_counts_pages_for_the_whole_generation():
    pager = SlotPager(n_slots=4, n_pages=4, page_size=64, max_seq_len=256)
    b = GenerationBooks(max_tokens=10, max_seq_len=256)
    for _ in range(3):
        b.add([1] * 60)                                       # 60 + 10 positions: two pages each
    assert b.admit(pager, 0, None) == 2 and b.admit(pager, 2, None) == 1 and b.admit(pager, 0, 1) == 1
    assert b.admit(pager, 3, None) == 0                       # nothing left to admit
    big = GenerationBooks(max_tokens=4, max_seq_len=1000)
    big.add([1] * 300)
    with pytest.raises(RuntimeError, match="does not fit the cache even alone"):
        big.admit(pager, 0, None)
    slot = pager.alloc_slot()
    pager.reserve_many([(slot, 130)])                          # three pages taken: one left
    with pytest.raises(RuntimeError, match="does not fit"):
        b.admit(pager, 0, None)


def test_history_is_prompt_and_generated_tokens():
    b = GenerationBooks(max_tokens=10, max_seq_len=100, stop_ids=[9], keep_history=True)
    b.add([1, 2, 3])
    b.add([4])
    b.book([0, 1], [50, 60])
    b.book([0, 1], [51, 9])
    assert b.recent([0, 1], 64) == [[1, 2, 3, 50, 51], [4, 60]]           # the stop id is not part of the history
    assert b.recent([0, 1], 2) == [[50, 51], [4, 60]] and b.recent([0], 0) == [[]]
    plain = GenerationBooks(max_tokens=10, max_seq_len=100)
    plain.add([1])
    with pytest.raises(ValueError, match="keep no history"):
        plain.recent([0], 4)
