"""The index arithmetic of `store_rows_coalesced` and `aux_to_rows` (lumen_b200/csrc/sm100.cuh, gemm.cu), restated on
the CPU: the XOR swizzle is a permutation of the warp's staging slots, the read-back returns each row's segments in
order, every store instruction covers whole rows, and neither the row-per-lane accesses nor the segment-per-lane
accesses put two lanes of a quarter warp (one shared-memory transaction of 16-byte accesses) on the same banks."""

import pytest


def swz(segs, row):
    return row & 7 if segs == 8 else (row >> 1) & 3


def banks(slot):  # the four 4-byte banks a 16-byte slot occupies
    return {(slot * 4 + k) % 32 for k in range(4)}


def conflict_free(slots_by_lane):
    for first in range(0, 32, 8):  # 16-byte accesses are served a quarter warp at a time
        seen = set()
        for lane in range(first, first + 8):
            b = banks(slots_by_lane[lane])
            assert not (b & seen), (first, lane)
            seen |= b


@pytest.mark.parametrize("segs", [8, 4])
def test_store_rows_coalesced_indexing(segs):
    stage = {}
    for q in range(segs):  # lane = row writes its q-th segment
        slots = [lane * segs + (q ^ swz(segs, lane)) for lane in range(32)]
        conflict_free(slots)
        for lane, slot in enumerate(slots):
            assert slot not in stage and 0 <= slot < 32 * segs
            stage[slot] = (lane, q)
    assert len(stage) == 32 * segs  # a permutation of the staging area
    rows_per_instruction = 32 // segs
    covered = set()
    for t in range(segs):  # one store instruction per t
        slots, pieces = [], []
        for lane in range(32):
            q, sub = lane % segs, lane // segs
            r = t * rows_per_instruction + sub
            slot = r * segs + (q ^ swz(segs, r))
            slots.append(slot)
            assert stage[slot] == (r, q)  # the lane stores segment q of row r at out + r * ld + q * 16
            pieces.append((r, q))
        conflict_free(slots)
        for r in {p[0] for p in pieces}:  # whole rows: every segment of each row the instruction touches
            assert {q for rr, q in pieces if rr == r} == set(range(segs))
        covered |= set(pieces)
    assert covered == {(r, q) for r in range(32) for q in range(segs)}


def test_aux_to_rows_indexing():
    """aux_load fetches segment l % 4 of rows l / 4 + 8 t; aux_to_rows hands every lane its own row's four segments."""
    stage = {}
    for t in range(4):
        slots = []
        for lane in range(32):
            r, q = t * 8 + (lane >> 2), lane & 3
            slot = r * 4 + (q ^ ((r >> 1) & 3))
            slots.append(slot)
            assert slot not in stage
            stage[slot] = (r, q)
        conflict_free(slots)
    assert len(stage) == 128
    for q in range(4):
        slots = [lane * 4 + (q ^ ((lane >> 1) & 3)) for lane in range(32)]
        conflict_free(slots)
        assert [stage[s] for s in slots] == [(lane, q) for lane in range(32)]
