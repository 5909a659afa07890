"""The thread-to-element map of the bf16-wire gradient all-reduce (csrc/coll_index.h).

The kernel's cross-GPU barrier is per block index: block b of a replica waits
only for block b of every peer.  So after the first barrier, what block b of
replica r reads from a peer's staging buffer must have been written, before
that barrier, by block b of that peer; and after the second barrier, what
block b of any replica reads back must have been written by block b of the
slice's owner.  The host library evaluates the same header the kernel uses, so
this runs without a GPU.
"""
import numpy as np
import pytest

from diloco_swarm_b200.parallel.collectives import shard_size, touch_map

CASES = [
    # (R, count, grid, block)
    (2, 40000, 148, 512), (4, 40000, 148, 512), (8, 40000, 148, 512),
    (4, 7087872, 148, 512),          # one GPT-2 small block: shard 1 771 968 is no multiple of 8 * 148 * 512
    (3, 4096, 7, 64), (8, 8 * 8 * 5 + 8, 4, 32), (2, 8, 2, 32), (5, 1000 * 8, 3, 96),
]


@pytest.mark.parametrize("R,count,grid,block", CASES)
def test_every_phase_of_a_block_stays_within_what_the_same_block_wrote(R, count, grid, block):
    offset = 1024
    shard = shard_size(count, R, 8)
    cast = [touch_map(offset, count, shard, R, r, 0, grid, block) for r in range(R)]
    widen = [touch_map(offset, count, shard, R, r, 2, grid, block) for r in range(R)]
    # cast-in and widen-out cover every vector exactly as each other, identically on all replicas
    for r in range(R):
        assert (cast[r] >= 0).all()
        assert np.array_equal(cast[r], cast[0]) and np.array_equal(widen[r], cast[0])
    covered = np.zeros(count // 8, dtype=bool)
    for r in range(R):
        red = touch_map(offset, count, shard, R, r, 1, grid, block)
        mine = red >= 0
        lo, hi = r * shard // 8, min(count, (r + 1) * shard) // 8
        assert mine[lo:hi].all() and not mine[:lo].any() and not mine[hi:].any(), "reduce covers exactly the own slice"
        # the block that reduces a vector is the block that cast it in on every peer (first barrier) and the
        # block that reads it back on every peer (second barrier)
        assert np.array_equal(red[mine], cast[0][mine])
        covered |= mine
    assert covered.all()


def test_a_plain_grid_stride_would_not_have_the_property():
    """The map this replaces (one grid-stride loop over the whole bucket in the cast phase, one over the own
    slice in the reduce phase) pairs different blocks whenever the slice start is not a multiple of the
    grid's stride; this is the case the slice-wise walk exists for."""
    R, count, grid, block = 4, 7087872, 148, 512
    shard = shard_size(count, R, 8)
    nth = grid * block
    v = np.arange(count // 8)
    cast_block = (v % nth) // block
    r = 1
    lo = r * shard // 8
    reduce_block = ((v - lo) % nth) // block
    own = (v >= lo) & (v < lo + shard // 8)
    assert (cast_block[own] != reduce_block[own]).any()
    assert np.array_equal(touch_map(0, count, shard, R, r, 1, grid, block)[own], touch_map(0, count, shard, R, 0, 0, grid, block)[own])


def test_bad_arguments_are_refused():
    with pytest.raises(ValueError):
        touch_map(0, 64, 16, 4, 4, 1, 4, 32)          # rank out of range
    with pytest.raises(ValueError):
        touch_map(4, 64, 16, 4, 0, 0, 4, 32)          # offset not a multiple of the vector width
