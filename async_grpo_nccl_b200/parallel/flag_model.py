"""Host-side model of the peer-memory epoch-flag barrier (``csrc/kernels/symm.cu::flag_barrier_kernel``,
``parallel/symm.py::PeerGroup.barrier``), small enough to explore every interleaving.

Protocol per rank and epoch ``e`` (epochs count up from 1, flags start at 0):
  arrive: for every peer r, ``flags[r][me] = e``   (release stores, one atomic step each)
  wait:   until ``flags[me][r] >= e`` for every r  (acquire loads; bounded on the device: a wait that cannot complete
                                                     ends with a status code instead of spinning forever)

``explore(world, epochs, skip)`` walks all interleavings of these steps (depth first over the scheduler's choices) and
returns what can happen: whether any rank ever left barrier ``e`` before every rank had entered it (a safety
violation), and in which final states the run can end (all done, or a set of ranks blocked at an epoch, which on the
device is the timeout the host raises on). ``skip = (rank, epoch)`` makes that rank leave out its arrival in that epoch,
the failure the GPU test injects with a flag nobody sets.
"""
from __future__ import annotations

from typing import Dict, FrozenSet, Optional, Set, Tuple

State = Tuple[Tuple[Tuple[int, ...], ...], Tuple[Tuple[int, int, int], ...]]  # flags, per rank (epoch, phase, next peer)


def explore(world: int, epochs: int, skip: Optional[Tuple[int, int]] = None) -> Dict[str, object]:
    flags0 = tuple(tuple(0 for _ in range(world)) for _ in range(world))
    pcs0 = tuple((1, 0, 0) for _ in range(world))  # phase 0 = arriving (next peer index), 1 = waiting, epoch > epochs = done
    seen: Set[State] = set()
    finals: Set[FrozenSet[Tuple[int, int]]] = set()
    violations = []

    def moves(flags, pcs):
        for me, (e, phase, nxt) in enumerate(pcs):
            if e > epochs:
                continue
            if phase == 0:
                yield me
            elif all(flags[me][r] >= e for r in range(world)):
                yield me

    def step(flags, pcs, me):
        e, phase, nxt = pcs[me]
        if phase == 0:
            if skip == (me, e):  # the faulty rank goes straight to waiting without publishing its arrival
                return flags, pcs[:me] + ((e, 1, 0),) + pcs[me + 1:]
            row = list(flags[nxt])
            row[me] = e
            flags = flags[:nxt] + (tuple(row),) + flags[nxt + 1:]
            npc = (e, 0, nxt + 1) if nxt + 1 < world else (e, 1, 0)
            return flags, pcs[:me] + (npc,) + pcs[me + 1:]
        # leaving the barrier of epoch e: legal only if every rank has entered that barrier (it may still be publishing
        # its arrival to the others, but everything it did before the barrier is done)
        if not all(pc[0] >= e for pc in pcs):
            violations.append((me, e, pcs))
        if skip is not None and skip[1] == e and skip[0] != me:
            violations.append(("passed a barrier that a rank skipped", me, e))
        return flags, pcs[:me] + ((e + 1, 0, 0),) + pcs[me + 1:]

    stack = [(flags0, pcs0)]
    while stack:
        flags, pcs = stack.pop()
        if (flags, pcs) in seen:
            continue
        seen.add((flags, pcs))
        ms = list(moves(flags, pcs))
        if not ms:
            finals.add(frozenset((r, e) for r, (e, _, _) in enumerate(pcs) if e <= epochs))
            continue
        for me in ms:
            stack.append(step(flags, pcs, me))
    return {"states": len(seen), "violations": violations, "finals": finals}
