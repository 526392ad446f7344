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
    check_random(["one", "two", "one", "one", "two", "two", "one"], p=p, schedules=300, seed=p)


def test_single_buffering_is_caught_as_a_race():
    """Negative control: without double buffering a fast rank overwrites a slot that is still unread."""
    with pytest.raises(ProtocolViolation):
        check_exhaustive(["one", "one"], p=2, buffers=1)
    with pytest.raises(ProtocolViolation):
        check_exhaustive(["two"], p=2, buffers=1)
