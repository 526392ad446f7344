"""Executable model of the peer-memory flag protocol, for exhaustive interleaving checks on the host.

The kernels in ``csrc/kernels/comm_fused.cu`` synchronise ranks with nothing but per-buffer epoch
flags: op number ``e`` of an axis uses receive buffer ``e % 2``; a producer stores into its slot of
every peer's buffer without waiting; the consumer launch publishes ``flag[e % 2][me] = e`` on every
peer, waits until all peers' flags in its own array reach ``e``, then reads the slots.  The claim is
that double buffering alone prevents a slot from being rewritten before its reader is done.  No race
detector can be run on the device here, so the claim is checked on a model instead:

* every rank runs the same program of ops (``"one"`` = one-shot all-reduce / all-gather,
  ``"two"`` = two-shot all-reduce, which is a reduce-scatter op followed by a gather op whose pushes
  are issued by the first op's consumer kernel);
* each op is expanded into the events a stream executes in order: slot writes (begin / end, so a
  reader can observe a write in progress), flag publications, the wait, slot reads (begin / end);
* a scheduler interleaves the ranks' events in every possible order (depth-first with memoisation)
  or at random; a read that overlaps a write of the same slot, or that sees another op's data, is
  reported.

``buffers=1`` models the protocol without double buffering and must fail (negative control).
"""

from __future__ import annotations

import random
from typing import Dict, List, Optional, Sequence, Tuple

Event = Tuple  # (kind, ...)


def expand_program(program: Sequence[str], p: int, me: int, buffers: int = 2) -> List[Event]:
    """Stream-ordered events of rank ``me``; ops are numbered from 1 as on the device."""
    peers = [q for q in range(p) if q != me]
    ev: List[Event] = []
    e = 0

    def push(epoch):
        b = epoch % buffers
        for q in peers:
            ev.append(("wbeg", q, b, me, epoch))
            ev.append(("wend", q, b, me, epoch))

    def consume(epoch, then_push: Optional[int] = None):
        b = epoch % buffers
        for q in peers:
            ev.append(("flag", q, b, me, epoch))
        ev.append(("wait", b, epoch))
        for q in peers:
            ev.append(("rbeg", b, q, epoch))
            ev.append(("rend", b, q, epoch))
        if then_push is not None:
            push(then_push)  # same kernel: stores of the next op's data follow the reads

    for kind in program:
        if kind == "one":
            e += 1
            push(e)
            consume(e)
        elif kind == "two":
            e += 1
            push(e)
            consume(e, then_push=e + 1)
            e += 1
            consume(e)
        else:
            raise ValueError(kind)
    return ev


class ProtocolViolation(AssertionError):
    pass


class _State:
    __slots__ = ("pc", "slot", "writing", "reading", "flag")

    def __init__(self, p: int, buffers: int):
        self.pc = [0] * p
        # slot[owner][buffer][src] = epoch of the data it holds; writing/reading = activity counters
        self.slot = [[[0] * p for _ in range(buffers)] for _ in range(p)]
        self.writing = [[[0] * p for _ in range(buffers)] for _ in range(p)]
        self.reading = [[[0] * p for _ in range(buffers)] for _ in range(p)]
        self.flag = [[[0] * p for _ in range(buffers)] for _ in range(p)]

    def key(self):
        return (tuple(self.pc), repr(self.slot), repr(self.writing), repr(self.reading), repr(self.flag))

    def copy(self, p, buffers):
        s = _State.__new__(_State)
        s.pc = list(self.pc)
        for name in ("slot", "writing", "reading", "flag"):
            setattr(s, name, [[list(x) for x in o] for o in getattr(self, name)])
        return s


def _enabled(st: _State, progs, r: int, p: int) -> bool:
    if st.pc[r] >= len(progs[r]):
        return False
    ev = progs[r][st.pc[r]]
    if ev[0] == "wait":
        _, b, epoch = ev
        return all(st.flag[r][b][q] >= epoch for q in range(p) if q != r)
    return True


def _apply(st: _State, progs, r: int) -> None:
    ev = progs[r][st.pc[r]]
    kind = ev[0]
    if kind == "wbeg":
        _, owner, b, src, epoch = ev
        if st.reading[owner][b][src]:
            raise ProtocolViolation(f"rank {src} starts writing op {epoch} into a slot rank {owner} is reading")
        st.writing[owner][b][src] += 1
    elif kind == "wend":
        _, owner, b, src, epoch = ev
        st.writing[owner][b][src] -= 1
        st.slot[owner][b][src] = epoch
    elif kind == "flag":
        _, owner, b, src, epoch = ev
        if st.flag[owner][b][src] >= epoch:
            raise ProtocolViolation("flags must increase")
        st.flag[owner][b][src] = epoch
    elif kind == "rbeg":
        _, b, src, epoch = ev
        if st.writing[r][b][src]:
            raise ProtocolViolation(f"rank {r} reads slot of rank {src} for op {epoch} while it is being written")
        if st.slot[r][b][src] != epoch:
            raise ProtocolViolation(
                f"rank {r} expected data of op {epoch} from rank {src}, slot holds op {st.slot[r][b][src]}")
        st.reading[r][b][src] += 1
    elif kind == "rend":
        _, b, src, epoch = ev
        if st.writing[r][b][src] or st.slot[r][b][src] != epoch:
            raise ProtocolViolation(f"slot of rank {src} on rank {r} changed during the read of op {epoch}")
        st.reading[r][b][src] -= 1
    st.pc[r] += 1


def check_exhaustive(program: Sequence[str], p: int = 2, buffers: int = 2, max_states: int = 2_000_000) -> int:
    """Explore every interleaving (memoised); returns the number of distinct states visited.

    Raises :class:`ProtocolViolation` on a race or stale read, ``RuntimeError`` on deadlock."""
    progs = [expand_program(program, p, r, buffers) for r in range(p)]
    start = _State(p, buffers)
    seen = {start.key()}
    stack = [start]
    while stack:
        st = stack.pop()
        moves = [r for r in range(p) if _enabled(st, progs, r, p)]
        if not moves:
            if any(st.pc[r] < len(progs[r]) for r in range(p)):
                raise RuntimeError(f"deadlock at {st.pc}")
            continue
        for r in moves:
            nxt = st.copy(p, buffers)
            _apply(nxt, progs, r)
            k = nxt.key()
            if k not in seen:
                seen.add(k)
                if len(seen) > max_states:
                    raise RuntimeError("state space larger than max_states")
                stack.append(nxt)
    return len(seen)


def check_random(program: Sequence[str], p: int, buffers: int = 2, schedules: int = 2000, seed: int = 0) -> None:
    """Random interleavings, biased so that some ranks race ahead of others."""
    rng = random.Random(seed)
    progs = [expand_program(program, p, r, buffers) for r in range(p)]
    for _ in range(schedules):
        st = _State(p, buffers)
        weight = [rng.choice((1, 1, 4, 16)) for _ in range(p)]
        while True:
            moves = [r for r in range(p) if _enabled(st, progs, r, p)]
            if not moves:
                if any(st.pc[r] < len(progs[r]) for r in range(p)):
                    raise RuntimeError(f"deadlock at {st.pc}")
                break
            r = rng.choices(moves, [weight[m] for m in moves])[0]
            _apply(st, progs, r)


# ------------------------------------------------------------------------------------------------
# Tile-granular variant: the reduction is finished inside the compute kernel.
#
# Every rank runs C persistent CTAs per op; CTA c owns tiles c, c + C, ...  For tile t it stores its
# partial into slot tile t of every peer and raises the per-tile flag there, then - one tile behind -
# waits for the peers' flags of its previous tile and reads their partials.  Ops alternate between
# two buffers; a rank's CTAs all finish op e before any starts op e + 1 (kernel boundary).  The
# questions the model answers: can the waits deadlock (they are on other GPUs' kernels), and can a
# fast rank's op e + 2 overwrite a slot tile that a slow peer still reads for op e?
def expand_tile_program(num_ops: int, p: int, me: int, cta: int, ctas: int, tiles: int, buffers: int = 2,
                        lag: int = 1) -> List[Event]:
    peers = [q for q in range(p) if q != me]
    mine = list(range(cta, tiles, ctas))
    ev: List[Event] = []

    def consume(e, b, t):
        ev.append(("twait", b, t, e))
        for q in peers:
            ev.append(("trbeg", b, q, t, e))
            ev.append(("trend", b, q, t, e))

    for e in range(1, num_ops + 1):
        b = e % buffers
        for k, t in enumerate(mine):
            for q in peers:
                ev.append(("twbeg", q, b, me, t, e))
                ev.append(("twend", q, b, me, t, e))
            for q in peers:
                ev.append(("tflag", q, b, me, t, e))
            if k >= lag:
                consume(e, b, mine[k - lag])
        for t in mine[max(0, len(mine) - lag):]:
            consume(e, b, t)
        ev.append(("kbar", e))  # end of this CTA's part of the kernel
    return ev


def check_tile_protocol(num_ops: int = 3, p: int = 2, ctas: int = 2, tiles: int = 4, buffers: int = 2,
                        lag: int = 1, max_states: int = 3_000_000, schedules: int = 0, seed: int = 0) -> int:
    """Exhaustive (``schedules == 0``) or random exploration of the tile-granular protocol.

    Returns the number of distinct states (exhaustive) or of schedules run.  Raises
    :class:`ProtocolViolation` on a race / stale read and ``RuntimeError`` on deadlock."""
    threads = [(r, c) for r in range(p) for c in range(ctas)]
    progs = [expand_tile_program(num_ops, p, r, c, ctas, tiles, buffers, lag) for r, c in threads]
    nthreads = len(threads)

    def enabled(pc, slot, flag, arrived, i):
        if pc[i] >= len(progs[i]):
            return False
        ev = progs[i][pc[i]]
        r = threads[i][0]
        if ev[0] == "twait":
            _, b, t, e = ev
            return all(flag.get((r, b, q, t), 0) >= e for q in range(p) if q != r)
        return True

    def apply(pc, slot, busy, flag, arrived, i):
        ev = progs[i][pc[i]]
        r = threads[i][0]
        kind = ev[0]
        if kind == "twbeg":
            _, owner, b, src, t, e = ev
            cell = (owner, b, src, t)
            if busy.get(("r",) + cell, 0):
                raise ProtocolViolation(f"rank {src} op {e} overwrites tile {t} that rank {owner} is still reading")
            busy[("w",) + cell] = busy.get(("w",) + cell, 0) + 1
        elif kind == "twend":
            _, owner, b, src, t, e = ev
            cell = (owner, b, src, t)
            busy[("w",) + cell] -= 1
            slot[cell] = e
        elif kind == "tflag":
            _, owner, b, src, t, e = ev
            if flag.get((owner, b, src, t), 0) >= e:
                raise ProtocolViolation("flags must increase")
            flag[(owner, b, src, t)] = e
        elif kind == "trbeg":
            _, b, src, t, e = ev
            cell = (r, b, src, t)
            if busy.get(("w",) + cell, 0) or slot.get(cell, 0) != e:
                raise ProtocolViolation(f"rank {r} op {e} tile {t}: slot of rank {src} holds op {slot.get(cell, 0)}"
                                        " or is being written")
            busy[("r",) + cell] = busy.get(("r",) + cell, 0) + 1
        elif kind == "trend":
            _, b, src, t, e = ev
            cell = (r, b, src, t)
            if busy.get(("w",) + cell, 0) or slot.get(cell, 0) != e:
                raise ProtocolViolation(f"rank {r} op {e} tile {t}: slot changed during the read")
            busy[("r",) + cell] -= 1
        elif kind == "kbar":
            arrived[(r, ev[1])] = arrived.get((r, ev[1]), 0) + 1
        pc[i] += 1

    def blocked_at_barrier(pc, arrived, i):
        # a CTA that finished op e may only start op e + 1 when all CTAs of its rank finished op e
        if pc[i] == 0 or pc[i] >= len(progs[i]):
            return False
        prev = progs[i][pc[i] - 1]
        return prev[0] == "kbar" and arrived.get((threads[i][0], prev[1]), 0) < ctas

    def freeze(d):
        return tuple(sorted((k, v) for k, v in d.items() if v))

    def moves(pc, slot, flag, arrived):
        return [i for i in range(nthreads)
                if not blocked_at_barrier(pc, arrived, i) and enabled(pc, slot, flag, arrived, i)]

    def done(pc):
        return all(pc[i] >= len(progs[i]) for i in range(nthreads))

    if schedules:
        rng = random.Random(seed)
        for _ in range(schedules):
            pc, slot, busy, flag, arrived = [0] * nthreads, {}, {}, {}, {}
            weight = [rng.choice((1, 1, 4, 16)) for _ in range(nthreads)]
            while True:
                mv = moves(pc, slot, flag, arrived)
                if not mv:
                    if not done(pc):
                        raise RuntimeError(f"deadlock at {pc}")
                    break
                apply(pc, slot, busy, flag, arrived, rng.choices(mv, [weight[m] for m in mv])[0])
        return schedules

    start = ([0] * nthreads, {}, {}, {}, {})
    seen = {(tuple(start[0]), (), (), (), ())}
    stack = [start]
    while stack:
        pc, slot, busy, flag, arrived = stack.pop()
        mv = moves(pc, slot, flag, arrived)
        if not mv:
            if not done(pc):
                raise RuntimeError(f"deadlock at {pc}")
            continue
        for i in mv:
            n = (list(pc), dict(slot), dict(busy), dict(flag), dict(arrived))
            apply(*n, i)
            key = (tuple(n[0]), freeze(n[1]), freeze(n[2]), freeze(n[3]), freeze(n[4]))
            if key not in seen:
                seen.add(key)
                if len(seen) > max_states:
                    raise RuntimeError("state space larger than max_states")
                stack.append(n)
    return len(seen)


# ------------------------------------------------------------------------------------------------
# Segment reduce on a symmetric buffer (csrc/kernels/nvls_reduce.cu, parallel/fused.py).
#
# Every rank owns ONE buffer S (no double buffering), cut in row chunks, each chunk in one segment per
# rank.  Per op and chunk c a rank's main stream writes its partial into its own S[c]; its side stream
# then runs: barrier (flags) - read segment `me` of chunk c from EVERY rank's S (the switch does that
# for a multimem load) - write the reduced segment into EVERY rank's S - barrier - copy the whole local
# chunk out.  The main stream meanwhile computes the next chunk and joins the side stream before the
# next op.  Questions: can the single buffer be overwritten (by the next op's partials, or by a
# reduced segment) while somebody still reads it, does every read see the right data, can the waits
# deadlock?  `second_barrier=False` and `join=False` are negative controls.
def _segment_streams(num_ops: int, p: int, me: int, chunks: int, second_barrier: bool = True,
                     join: bool = True) -> Tuple[List[Event], List[Event]]:
    peers = [q for q in range(p) if q != me]
    main: List[Event] = []
    side: List[Event] = []
    epoch = 0
    for k in range(1, num_ops + 1):
        if k > 1 and join:
            main.append(("join", k - 1))
        for c in range(chunks):
            main.append(("cwbeg", c, k))
            main.append(("cwend", c, k))
            main.append(("ready", c, k))
            side.append(("sync", c, k))
            epoch += 1
            for q in peers:
                side.append(("flag", q, epoch))
            side.append(("wait", epoch))
            for q in range(p):
                side.append(("prbeg", q, c, k))
                side.append(("prend", q, c, k))
            for q in range(p):
                side.append(("rwbeg", q, c, k))
                side.append(("rwend", q, c, k))
            epoch += 1
            if second_barrier:
                for q in peers:
                    side.append(("flag", q, epoch))
                side.append(("wait", epoch))
            for s in range(p):
                side.append(("crbeg", c, s, k))
                side.append(("crend", c, s, k))
        side.append(("sdone", k))
    return main, side


def check_segment_protocol(num_ops: int = 2, p: int = 2, chunks: int = 2, second_barrier: bool = True,
                           join: bool = True, max_states: int = 3_000_000, schedules: int = 0,
                           seed: int = 0) -> int:
    """Exhaustive (``schedules == 0``) or random exploration of the segment-reduce protocol.

    Returns the number of distinct states (exhaustive) or of schedules run.  Raises
    :class:`ProtocolViolation` on a race / wrong data and ``RuntimeError`` on deadlock."""
    threads = [(r, s) for r in range(p) for s in (0, 1)]  # stream 0 = main, 1 = side
    progs = []
    for r in range(p):
        progs.extend(_segment_streams(num_ops, p, r, chunks, second_barrier, join))
    n = len(threads)

    # state: pc, cell value {(owner, chunk, seg): ("P" | "R", op)}, busy counters, flags, ready marks, side progress
    def enabled(pc, flag, ready, sdone, i):
        if pc[i] >= len(progs[i]):
            return False
        ev = progs[i][pc[i]]
        r = threads[i][0]
        if ev[0] == "wait":
            return all(flag.get((r, q), 0) >= ev[1] for q in range(p) if q != r)
        if ev[0] == "sync":
            return ready.get((r, ev[1], ev[2]), 0) == 1
        if ev[0] == "join":
            return sdone.get(r, 0) >= ev[1]
        return True

    def apply(pc, val, busy, flag, ready, sdone, i):
        ev = progs[i][pc[i]]
        r = threads[i][0]
        kind = ev[0]
        if kind == "cwbeg":  # the compute kernel overwrites the whole local chunk with partials of op k
            _, c, k = ev
            for s in range(p):
                cell = (r, c, s)
                if busy.get(("r",) + cell, 0) or busy.get(("w",) + cell, 0):
                    raise ProtocolViolation(
                        f"rank {r} op {k} writes its partial of chunk {c} while segment {s} is in use")
                busy[("w",) + cell] = 1
        elif kind == "cwend":
            _, c, k = ev
            for s in range(p):
                busy[("w",) + (r, c, s)] = 0
                val[(r, c, s)] = ("P", k)
        elif kind == "ready":
            ready[(r, ev[1], ev[2])] = 1
        elif kind == "flag":
            _, owner, e = ev
            if flag.get((owner, r), 0) >= e:
                raise ProtocolViolation("flags must increase")
            flag[(owner, r)] = e
        elif kind == "prbeg":  # read the partial of segment r of chunk c from rank q's buffer
            _, q, c, k = ev
            cell = (q, c, r)
            if busy.get(("w",) + cell, 0) or val.get(cell) != ("P", k):
                raise ProtocolViolation(
                    f"rank {r} op {k}: partial of rank {q}, chunk {c} is {val.get(cell)} or being written")
            busy[("r",) + cell] = busy.get(("r",) + cell, 0) + 1
        elif kind == "prend":
            _, q, c, k = ev
            cell = (q, c, r)
            if busy.get(("w",) + cell, 0) or val.get(cell) != ("P", k):
                raise ProtocolViolation(f"rank {r} op {k}: partial of rank {q} changed during the read")
            busy[("r",) + cell] -= 1
        elif kind == "rwbeg":  # write the reduced segment r of chunk c into rank q's buffer
            _, q, c, k = ev
            cell = (q, c, r)
            if busy.get(("r",) + cell, 0) or busy.get(("w",) + cell, 0):
                raise ProtocolViolation(
                    f"rank {r} op {k}: reduced segment written into rank {q}'s chunk {c} while in use")
            busy[("w",) + cell] = 1
        elif kind == "rwend":
            _, q, c, k = ev
            busy[("w",) + (q, c, r)] = 0
            val[(q, c, r)] = ("R", k)
        elif kind == "crbeg":  # copy out: the local chunk must hold the reduced data of op k
            _, c, s, k = ev
            cell = (r, c, s)
            if busy.get(("w",) + cell, 0) or val.get(cell) != ("R", k):
                raise ProtocolViolation(f"rank {r} op {k}: copies segment {s} of chunk {c} holding {val.get(cell)}")
            busy[("r",) + cell] = busy.get(("r",) + cell, 0) + 1
        elif kind == "crend":
            _, c, s, k = ev
            cell = (r, c, s)
            if busy.get(("w",) + cell, 0) or val.get(cell) != ("R", k):
                raise ProtocolViolation(f"rank {r} op {k}: segment {s} of chunk {c} changed during the copy")
            busy[("r",) + cell] -= 1
        elif kind == "sdone":
            sdone[r] = ev[1]
        pc[i] += 1

    def freeze(d):
        return tuple(sorted((k, v) for k, v in d.items() if v))

    def moves(pc, flag, ready, sdone):
        return [i for i in range(n) if enabled(pc, flag, ready, sdone, i)]

    def done(pc):
        return all(pc[i] >= len(progs[i]) for i in range(n))

    if schedules:
        rng = random.Random(seed)
        for _ in range(schedules):
            pc, val, busy, flag, ready, sdone = [0] * n, {}, {}, {}, {}, {}
            weight = [rng.choice((1, 1, 4, 16)) for _ in range(n)]
            while True:
                mv = moves(pc, flag, ready, sdone)
                if not mv:
                    if not done(pc):
                        raise RuntimeError(f"deadlock at {pc}")
                    break
                apply(pc, val, busy, flag, ready, sdone, rng.choices(mv, [weight[m] for m in mv])[0])
        return schedules

    start = ([0] * n, {}, {}, {}, {}, {})
    seen = {(tuple(start[0]), ())}
    stack = [start]
    while stack:
        pc, val, busy, flag, ready, sdone = stack.pop()
        mv = moves(pc, flag, ready, sdone)
        if not mv:
            if not done(pc):
                raise RuntimeError(f"deadlock at {pc}")
            continue
        for i in mv:
            nxt = (list(pc), dict(val), dict(busy), dict(flag), dict(ready), dict(sdone))
            apply(*nxt, i)
            # flags, marks and accesses in progress follow from the program counters; what a cell holds
            # also depends on the order of the writes to it
            key = (tuple(nxt[0]), freeze(nxt[1]))
            if key not in seen:
                seen.add(key)
                if len(seen) > max_states:
                    raise RuntimeError("state space larger than max_states")
                stack.append(nxt)
    return len(seen)
