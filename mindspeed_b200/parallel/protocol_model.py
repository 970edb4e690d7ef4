"""Host model of the flag protocols of the fused compute+collective kernels, checked over every interleaving.

The kernels in ``csrc/kernels/gemm2_comm_sm100.cu`` coordinate GPUs through words in each rank's symmetric heap: entry
flags carrying the call's epoch, per-tile arrival counters, per-owner completion flags.  Whether that protocol is free of
races (a rank reading a buffer before its writer has finished, a writer of the next call overwriting what a slower rank
still reads, a counter reset racing with an increment) cannot be established by running it - a run shows one schedule.
This module states the protocol as small per-rank programs over a shared memory and explores ALL interleavings of their
steps (memoised depth-first search over global states), reporting

  * ``deadlock``   - a state where some thread waits on a condition no remaining step can make true (on the device: a
                     bounded wait that runs out and sets the status word);
  * ``stale read`` - a read that does not see the value written for this call by the expected writer.

Each rank runs ``epochs`` consecutive calls; a call is a list of phases, a phase a set of threads that run concurrently
(the copy warp and the consumers of one kernel), the next phase starts when all of them are done (stream order / kernel
end).  Data buffers hold a tag (writer, epoch) per slot instead of values.

``all_gather_gemm_program`` / ``gemm_reduce_scatter_program`` transcribe the two kernel modes (with the optional
all-reduce tail); their ``entry_handshake`` / ``wait_done`` / ``wait_ready`` switches remove one protocol element each so
that tests can show the checker finds the race the element exists to prevent.
reference: the vendor collectives this replaces synchronise inside the library (mindspeed/ops/csrc/atb/lcal_coc.cpp:39-266);
there is no counterpart to check there.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Tuple

# --- operations ----------------------------------------------------------------------------------------------------
# ("store", rank, key, value)              flag word := value                      (st.release.sys to a peer / local store)
# ("add", rank, key, delta)                flag word += delta                      (red.add / atomicAdd without using the result)
# ("fetch_add", key, delta)                local word += delta, old value -> the thread's register
# ("if_reg_ne", value, skip)               skip the next ``skip`` ops unless register == value
# ("wait_ge", key, value)                  block until local word >= value         (ld.acquire spin, bounded on the device)
# ("write", rank, buf, slot, tag)          data slot := tag
# ("read", buf, slot, tag)                 local data slot must hold tag
# ("rread", rank, buf, slot, tag)          a peer's data slot must hold tag        (plain peer load)
Op = tuple


@dataclasses.dataclass
class Violation:
    kind: str
    detail: str
    trace: List[str]


def _freeze(mem: Dict) -> Tuple:
    return tuple(sorted(mem.items()))


class Explorer:
    """programs[rank] = list of phases; phase = list of threads; thread = list of ops."""

    def __init__(self, programs: List[List[List[List[Op]]]], max_states: int = 2_000_000):
        self.programs, self.max_states = programs, max_states
        self.states = 0

    def _initial(self):
        return tuple((0, tuple((0, 0) for _ in self.programs[r][0]) if self.programs[r] else ()) for r in range(len(self.programs)))

    def _normalise(self, ranks):
        """Advance ranks whose current phase is complete."""
        out = []
        for r, (ph, threads) in enumerate(ranks):
            prog = self.programs[r]
            while ph < len(prog) and all(pc >= len(prog[ph][t]) for t, (pc, _) in enumerate(threads)):
                ph += 1
                threads = tuple((0, 0) for _ in prog[ph]) if ph < len(prog) else ()
            out.append((ph, threads))
        return tuple(out)

    def run(self) -> Optional[Violation]:
        start = (self._normalise(self._initial()), _freeze({}))
        seen = {start}
        stack = [(start, [])]
        while stack:
            (ranks, fmem), trace = stack.pop()
            self.states += 1
            if self.states > self.max_states:
                raise RuntimeError("state budget exceeded; shrink the configuration")
            mem = dict(fmem)
            done = all(ph >= len(self.programs[r]) for r, (ph, _) in enumerate(ranks))
            if done:
                continue
            moved = False
            for r, (ph, threads) in enumerate(ranks):
                if ph >= len(self.programs[r]):
                    continue
                for t, (pc, reg) in enumerate(threads):
                    ops = self.programs[r][ph][t]
                    if pc >= len(ops):
                        continue
                    res = self._step(r, ops, pc, reg, mem)
                    if res is None:
                        continue                                   # blocked wait
                    if isinstance(res, Violation):
                        res.trace = trace + [f"rank {r} phase {ph} thread {t}: {ops[pc]}"]
                        return res
                    npc, nreg, nmem = res
                    moved = True
                    nthreads = threads[:t] + ((npc, nreg),) + threads[t + 1:]
                    nranks = self._normalise(ranks[:r] + ((ph, nthreads),) + ranks[r + 1:])
                    nxt = (nranks, _freeze(nmem))
                    if nxt not in seen:
                        seen.add(nxt)
                        stack.append((nxt, trace + [f"rank {r} phase {ph} thread {t}: {ops[pc]}"]))
            if not moved:
                waiting = [f"rank {r}: {self.programs[r][ph][t][pc]}" for r, (ph, th) in enumerate(ranks)
                           if ph < len(self.programs[r]) for t, (pc, _) in enumerate(th) if pc < len(self.programs[r][ph][t])]
                return Violation("deadlock", "; ".join(waiting), trace)
        return None

    @staticmethod
    def _step(r, ops, pc, reg, mem):
        op = ops[pc]
        k = op[0]
        if k == "store":
            m = dict(mem)
            m[("f", op[1], op[2])] = op[3]
            return pc + 1, reg, m
        if k == "add":
            m = dict(mem)
            m[("f", op[1], op[2])] = m.get(("f", op[1], op[2]), 0) + op[3]
            return pc + 1, reg, m
        if k == "fetch_add":
            m = dict(mem)
            old = m.get(("f", r, op[1]), 0)
            m[("f", r, op[1])] = old + op[2]
            return pc + 1, old, m
        if k == "if_reg_ne":
            return (pc + 1 if reg == op[1] else pc + 1 + op[2]), reg, mem
        if k == "wait_ge":
            return (pc + 1, reg, mem) if mem.get(("f", r, op[1]), 0) >= op[2] else None
        if k == "write":
            m = dict(mem)
            m[("d", op[1], op[2], op[3])] = op[4]
            return pc + 1, reg, m
        if k == "rread":
            got = mem.get(("d", op[1], op[2], op[3]))
            if got != op[4]:
                return Violation("stale read", f"rank {r} read {op[2]}[{op[3]}] of rank {op[1]} = {got}, expected {op[4]}", [])
            return pc + 1, reg, mem
        if k == "read":
            got = mem.get(("d", r, op[1], op[2]))
            if got != op[3]:
                return Violation("stale read", f"rank {r} read {op[1]}[{op[2]}] = {got}, expected {op[3]}", [])
            return pc + 1, reg, mem
        raise ValueError(f"unknown op {op}")


def check(programs, max_states: int = 2_000_000) -> Tuple[Optional[Violation], int]:
    ex = Explorer(programs, max_states)
    v = ex.run()
    return v, ex.states


# --- the kernels' protocols ----------------------------------------------------------------------------------------------
def _entry(r, W, e):
    """All-to-all epoch handshake: tell every peer this rank has entered call ``e``, wait until every peer has."""
    return [[("store", p, ("entry", r), e) for p in range(W) if p != r] + [("wait_ge", ("entry", p), e) for p in range(W) if p != r]]


def all_gather_gemm_program(W: int, epochs: int = 2, chunks: int = 2, entry_handshake: bool = True, wait_ready: bool = True):
    """All-gather -> GEMM.  Before the launch the host zeroes the arrival counters and the rank's own rows are in slab ``r`` of
    its gathered buffer.  Copy warp: W-1 phases, in phase s everything goes to rank r-s, ``chunks`` bulk stores per tile each
    followed by an add on the peer's arrival counter.  Consumer: own slab, then slabs r+1, r+2, ..., each after its counter
    has reached the chunk count."""
    progs = []
    for r in range(W):
        prog = []
        for e in range(1, epochs + 1):
            host = [("store", r, ("ready", s), 0) for s in range(W) if s != r] + \
                   [("write", r, "gathered", (r, c), (r, e)) for c in range(chunks)]
            prog.append([host])
            if entry_handshake:
                prog.append(_entry(r, W, e))
            copy, use = [], [("read", "gathered", (r, c), (r, e)) for c in range(chunks)]
            for s in range(1, W):
                dst = (r - s) % W
                for c in range(chunks):
                    copy += [("write", dst, "gathered", (r, c), (r, e)), ("add", dst, ("ready", r), 1)]
                src = (r + s) % W
                if wait_ready:
                    use.append(("wait_ge", ("ready", src), chunks))
                use += [("read", "gathered", (src, c), (src, e)) for c in range(chunks)]
            prog.append([copy, use])
        progs.append(prog)
    return progs


def gemm_reduce_scatter_program(W: int, epochs: int = 2, warps: int = 2, all_reduce: bool = False, entry_handshake: bool = True,
                                wait_done: bool = True):
    """GEMM -> reduce-scatter (-> all-gather of the reduced rows).  ``warps`` epilogue warps per rank each store their piece
    of every owner's tile into slab ``r`` of the owner's staging area, owners visited r, r+1, ...; a local per-owner counter
    counts finished warps, the last one resets it and raises this rank's flag at the owner.  Then every rank waits for the
    W flags of its own staging area and sums the slabs; with ``all_reduce`` the reduced rows go to every peer's output
    followed by a second flag round, and the output is read after the kernel."""
    progs = []
    for r in range(W):
        prog = []
        for e in range(1, epochs + 1):
            if entry_handshake:
                prog.append(_entry(r, W, e))
            threads = []
            for w in range(warps):
                ops = []
                for s in range(W):
                    o = (r + s) % W
                    ops += [("write", o, "staging", (r, w), (r, e)),
                            ("fetch_add", ("phase", o), 1),
                            ("if_reg_ne", warps - 1, 2),
                            ("store", r, ("phase", o), 0),
                            ("store", o, ("done", r), e)]
                threads.append(ops)
            prog.append(threads)
            red = []
            for p in range(W):
                if wait_done:
                    red.append(("wait_ge", ("done", p), e))
                red += [("read", "staging", (p, w), (p, e)) for w in range(warps)]
            if all_reduce:
                red += [("write", q, "out", r, (r, e)) for q in range(W)]
                red += [("store", q, ("ar", r), e) for q in range(W) if q != r]
                red += [("wait_ge", ("ar", p), e) for p in range(W) if p != r]
            prog.append([red])
            if all_reduce:
                prog.append([[("read", "out", p, (p, e)) for p in range(W)]])       # the next kernel on the stream reads the output
        progs.append(prog)
    return progs


def moe_pull_program(W: int, epochs: int = 3, slots: int = 2, readers: int = 2, entry_handshake: bool = True):
    """MoE dispatch / combine (``csrc/kernels/moe_comm.cu``): every rank stages its rows in slot ``call % slots`` of its own
    symmetric buffer (stream-ordered before the kernel), the kernel starts with the epoch handshake and then ``readers``
    thread blocks pull the rows they need from every peer's slot with plain loads.  There are no exit flags: with two slots
    a slot is rewritten only two calls later, and reaching that call's staging copy means this rank has passed the
    handshake of the call in between, which every peer joins only after leaving the call that read the slot."""
    progs = []
    for r in range(W):
        prog = []
        for e in range(1, epochs + 1):
            slot = e % slots
            prog.append([[("write", r, "staged", slot, (r, e))]])
            if entry_handshake:
                prog.append(_entry(r, W, e))
            prog.append([[("rread", p, "staged", slot, (p, e)) for p in range(W)] for _ in range(readers)])
        progs.append(prog)
    return progs

