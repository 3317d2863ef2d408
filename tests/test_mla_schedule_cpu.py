"""The MLA launch schedule is host arithmetic shared with the kernel (the same function maps a
cluster to its pieces of work on both sides): every (sequence, chunk) must belong to exactly one
piece, partial slots must be distinct per sequence, and the merge step's piece count must match.
No GPU is needed: 148 SMs are assumed when no device is current."""
import ctypes

import pytest

from trinity_lowering import kernels


@pytest.fixture(scope="module")
def lib():
    handle = ctypes.CDLL(str(kernels.library_path()))
    handle.trinity_sm100_mla_schedule.argtypes = [ctypes.c_int32] * 3 + [ctypes.POINTER(ctypes.c_int32)]
    handle.trinity_sm100_mla_schedule_segment.argtypes = [ctypes.c_int32] * 6 + [ctypes.POINTER(ctypes.c_int64)]
    handle.trinity_sm100_mla_default_splits.argtypes = [ctypes.c_int32] * 2
    handle.trinity_sm100_mla_balanced_slots.argtypes = [ctypes.c_int32] * 2
    return handle


def pieces_of(lib, batch, seq, mode):
    info = (ctypes.c_int32 * 4)()
    assert lib.trinity_sm100_mla_schedule(batch, seq, mode, info) == 0
    balanced, grid_y, slots, chunks = list(info)
    found = []
    for z in range(1 if balanced else batch):
        for y in range(grid_y):
            index = 0
            while True:
                segment = (ctypes.c_int64 * 5)()
                rc = lib.trinity_sm100_mla_schedule_segment(batch, seq, mode, y, z, index, segment)
                assert rc in (0, 1)
                if rc == 0:
                    break
                found.append(((y, z), tuple(segment)))
                index += 1
            # past the grid there is nothing
    assert lib.trinity_sm100_mla_schedule_segment(batch, seq, mode, grid_y, 0, 0, (ctypes.c_int64 * 5)()) == 0
    return balanced, grid_y, slots, chunks, found


@pytest.mark.parametrize("batch,seq", [(64, 4096), (100, 4096), (8, 16384), (5, 1000), (1, 65536), (256, 512),
                                        (150, 64), (3, 129), (1, 1), (37, 4100), (74, 2048)])
@pytest.mark.parametrize("mode", [-1, 0, 1, 3])
def test_every_chunk_belongs_to_exactly_one_piece(lib, batch, seq, mode):
    balanced, grid_y, slots, chunks, found = pieces_of(lib, batch, seq, mode)
    assert chunks == (seq + 63) // 64
    covered = {}
    per_sequence = {}
    for cluster, (sequence, first, count, slot, whole) in found:
        assert 0 <= sequence < batch and count >= 1 and 0 <= first and first + count <= chunks
        assert whole == (1 if count == chunks and (balanced or slots == 1) else 0)
        for chunk in range(first, first + count):
            assert (sequence, chunk) not in covered, "a chunk is processed twice"
            covered[(sequence, chunk)] = cluster
        per_sequence.setdefault(sequence, []).append((first, slot))
    assert len(covered) == batch * chunks, "a chunk is never processed"
    for sequence, parts in per_sequence.items():
        parts.sort()
        # slots of a sequence are b * slots + 0, 1, 2, ... in chunk order: what the merge step reads
        assert [slot for _, slot in parts] == [sequence * slots + i for i in range(len(parts))]
        assert len(parts) <= slots
    if mode > 0:
        assert not balanced and slots == min(mode, chunks) and grid_y == slots
    if mode < 0 and batch * chunks >= 8:
        assert balanced
    if balanced:
        # runs differ by at most one chunk, and a cluster's pieces are consecutive sequences
        sizes = {}
        for cluster, (sequence, first, count, slot, whole) in found:
            sizes[cluster] = sizes.get(cluster, 0) + count
        assert max(sizes.values()) - min(sizes.values()) <= 1 and len(sizes) == grid_y <= 74
        assert slots == lib.trinity_sm100_mla_balanced_slots(batch, seq) or mode == 0
    if mode == 0:
        assert slots == lib.trinity_sm100_mla_default_splits(batch, seq)


def test_bad_arguments_are_refused(lib):
    info = (ctypes.c_int32 * 4)()
    assert lib.trinity_sm100_mla_schedule(0, 64, 0, info) < 0
    assert lib.trinity_sm100_mla_schedule(1, 64, 0, None) < 0
    assert lib.trinity_sm100_mla_schedule_segment(1, 64, 0, -1, 0, 0, (ctypes.c_int64 * 5)()) < 0
