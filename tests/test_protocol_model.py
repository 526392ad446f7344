"""Interleaving checks of the peer-memory flag protocol on its host model (no device needed)."""

import pytest

from plexus_b200.parallel.protocol_model import (ProtocolViolation, check_exhaustive, check_random,
                                                 expand_program)


def test_event_expansion_matches_the_kernel_sequence():
    ev = expand_program(["two"], p=2, me=0)
    kinds = [e[0] for e in ev]
    # scatter push, publish + wait + read of op 1, broadcast push of op 2, publish + wait + read of op 2
    assert kinds == ["wbeg", "wend", "flag", "wait", "rbeg", "rend", "wbeg", "wend", "flag", "wait", "rbeg", "rend"]
    assert ev[0] == ("wbeg", 1, 1, 0, 1) and ev[6] == ("wbeg", 1, 0, 0, 2)  # buffers alternate with the op number


@pytest.mark.parametrize("program", [
    ["one"] * 4,
    ["two"] * 3,
    ["one", "two", "one", "two", "one"],
    ["two", "one", "one", "two"],
])
def test_every_interleaving_of_two_ranks_is_race_free(program):
    assert check_exhaustive(program, p=2) > 100


def test_every_interleaving_of_three_ranks_is_race_free():
    assert check_exhaustive(["one", "two", "one"], p=3, max_states=3_000_000) > 1000


@pytest.mark.parametrize("p", [4, 8])
def test_random_interleavings_of_larger_groups(p):
    check_random(["one", "two", "one", "one", "two", "two", "one"], p=p, schedules=300 if p == 4 else 80, seed=p)


def test_single_buffering_is_caught_as_a_race():
    """Negative control: without double buffering a fast rank overwrites a slot that is still unread."""
    with pytest.raises(ProtocolViolation):
        check_exhaustive(["one", "one"], p=2, buffers=1)
    with pytest.raises(ProtocolViolation):
        check_exhaustive(["two"], p=2, buffers=1)


# ---- tile-granular protocol (reduction finished inside the compute kernel, one tile behind)
@pytest.mark.parametrize("kw", [
    dict(num_ops=3, p=2, ctas=2, tiles=3),
    dict(num_ops=2, p=2, ctas=2, tiles=4),
    dict(num_ops=4, p=2, ctas=1, tiles=2),
    dict(num_ops=3, p=3, ctas=1, tiles=2),
], ids=lambda k: "-".join(f"{a}{b}" for a, b in k.items()))
def test_tile_granular_protocol_is_race_and_deadlock_free(kw):
    from plexus_b200.parallel.protocol_model import check_tile_protocol

    assert check_tile_protocol(**kw) > 300


def test_tile_granular_protocol_random_schedules_on_larger_groups():
    from plexus_b200.parallel.protocol_model import check_tile_protocol

    check_tile_protocol(num_ops=4, p=4, ctas=3, tiles=7, schedules=60, seed=1)
    check_tile_protocol(num_ops=3, p=8, ctas=2, tiles=5, schedules=15, seed=2, lag=2)


def test_tile_granular_protocol_needs_double_buffering():
    from plexus_b200.parallel.protocol_model import ProtocolViolation, check_tile_protocol

    with pytest.raises(ProtocolViolation):
        check_tile_protocol(num_ops=3, p=2, ctas=1, tiles=2, buffers=1)


@pytest.mark.parametrize("kw", [dict(num_ops=2, p=2, chunks=2), dict(num_ops=3, p=2, chunks=2),
                                dict(num_ops=3, p=2, chunks=1), dict(num_ops=2, p=3, chunks=1)])
def test_segment_reduce_protocol_is_race_and_deadlock_free(kw):
    """One symmetric buffer per rank, no double buffering: partials written locally, every rank's
    segment read from all buffers and the reduced segment written into all of them between two flag
    barriers, copy out after the second; main and side stream per rank.  All interleavings."""
    from plexus_b200.parallel.protocol_model import check_segment_protocol

    assert check_segment_protocol(**kw) > 500


def test_segment_reduce_protocol_random_schedules_on_larger_groups():
    from plexus_b200.parallel.protocol_model import check_segment_protocol

    assert check_segment_protocol(num_ops=3, p=4, chunks=2, schedules=200, seed=1) == 200
    assert check_segment_protocol(num_ops=2, p=8, chunks=2, schedules=40, seed=2) == 40


def test_segment_reduce_protocol_needs_the_second_barrier_and_the_join():
    """Negative controls: copying out right after the own segment is written reads a peer's segment
    too early; computing the next op's partials without joining the side stream overwrites a chunk
    that is still being reduced."""
    from plexus_b200.parallel.protocol_model import ProtocolViolation, check_segment_protocol

    with pytest.raises(ProtocolViolation):
        check_segment_protocol(num_ops=2, p=2, chunks=2, second_barrier=False)
    with pytest.raises(ProtocolViolation):
        check_segment_protocol(num_ops=2, p=2, chunks=2, join=False)
