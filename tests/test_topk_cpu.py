"""The oracle's top-k block selection against the reference's own unit tests of cpu::topk_blocks
(crates/breccia-kernels/src/qsa/cpu.rs:518-534)."""
from oracle.topk_ref import dense_blocks, topk_blocks


def test_ties_resolve_towards_the_lower_block():
    scores = [1.0, 3.0, 3.0, 2.0]
    assert topk_blocks(scores, 2) == [1, 2]
    assert topk_blocks(scores, 4, own_block=9) == [1, 2, 3, 0, 9]
    assert topk_blocks(scores, 3, own_block=3) == [1, 2, 3]      # an own block already selected is not appended twice


def test_dead_blocks_are_never_selected():
    assert topk_blocks([float("-inf"), float("-inf"), 1.0], 3) == [2]
    assert topk_blocks([-1.0e30, float("nan"), -5.0], 3) == [2]


def test_dense_selection_is_every_block_up_to_the_rows_own():
    assert dense_blocks(10, 3, 16) == [0, 1, 2, 3]
    assert dense_blocks(4, 7, 16) == [0, 1, 2, 3, 7]              # own block beyond the scored range is appended
    assert dense_blocks(4, 7, 4) == [0, 1, 2, 3]
