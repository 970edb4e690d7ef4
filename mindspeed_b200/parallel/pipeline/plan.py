"""Pipeline schedules as data: per-rank operation orders -> a global time-slot table.

A schedule is described by
  * a placement: which model stage each (rank, chunk) holds, and
  * for every rank the ORDER in which it runs its operations  F(chunk, mb), B(chunk, mb), W(chunk, mb)
    (W = deferred weight-gradient work of a micro-batch, when B computes input gradients only).
``assign_slots`` simulates all ranks together: an operation runs in the first slot after both the previous
operation of its rank and the producer of its input (on a neighbouring stage) have finished.  The result is a
lockstep table in which every tensor is sent in the slot after it was produced and received in that same slot,
so matching sends and receives always sit in the same communication group: deadlock-free by construction, and
the simulation itself rejects inconsistent orders.  The same table gives the bubble fraction analytically.

Schedules
  1F1B                         Megatron non-interleaved
  interleaved 1F1B             v chunks per rank, stage = chunk*pp + rank
  DualPipeV                    2 chunks per rank in a V (stage r and 2pp-1-r), B/W split, F&B pairing
                               (phase structure: mindspeed/core/pipeline_parallel/dualpipev/dualpipev_schedules.py:310-346,
                               docs/zh/features/dualpipev.md:22-45)
  DualPipe                     bidirectional: two model replicas fed from both ends (DeepSeek-V3 report, section 3.2.1)
  Chimera                      bidirectional 1F1B pipelines (Li & Hoefler, SC'21); not present in the reference
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class Op:
    kind: str   # "F", "B", "W", "R" (scheduler-placed recompute of a forward whose activations were dropped)
    chunk: int
    mb: int

    def __repr__(self):
        return f"{self.kind}{self.chunk}.{self.mb}"


@dataclass
class Placement:
    pp: int
    chunks: int
    # stage_of[(rank, chunk)] -> (pipeline id, stage index inside that pipeline)
    stage_of: Dict[Tuple[int, int], Tuple[int, int]]
    num_stages: int                    # stages per pipeline
    replicas: int = 1                  # model replicas (bidirectional schedules hold 2)

    def holder(self, pipe: int, stage: int) -> Tuple[int, int]:
        for k, v in self.stage_of.items():
            if v == (pipe, stage):
                return k
        raise KeyError((pipe, stage))


def placement_1f1b(pp):
    return Placement(pp, 1, {(r, 0): (0, r) for r in range(pp)}, pp)


def placement_interleaved(pp, v):
    return Placement(pp, v, {(r, c): (0, c * pp + r) for r in range(pp) for c in range(v)}, pp * v)


def placement_v(pp):
    d = {}
    for r in range(pp):
        d[(r, 0)] = (0, r)
        d[(r, 1)] = (0, 2 * pp - 1 - r)
    return Placement(pp, 2, d, 2 * pp)


def placement_bidirectional(pp):
    """chunk 0: pipeline 0 running rank 0 -> pp-1; chunk 1: pipeline 1 running pp-1 -> 0 (a second model replica)."""
    d = {}
    for r in range(pp):
        d[(r, 0)] = (0, r)
        d[(r, 1)] = (1, pp - 1 - r)
    return Placement(pp, 2, d, pp, replicas=2)


# ------------------------------------------------------------------------------------------------
# per-rank orders
# ------------------------------------------------------------------------------------------------
def order_1f1b(pp, n_mb) -> List[List[Op]]:
    out = []
    for r in range(pp):
        warm = min(pp - r - 1, n_mb)
        ops = [Op("F", 0, i) for i in range(warm)]
        f, b = warm, 0
        for _ in range(n_mb - warm):
            ops.append(Op("F", 0, f)); f += 1
            ops.append(Op("B", 0, b)); b += 1
        while b < n_mb:
            ops.append(Op("B", 0, b)); b += 1
        out.append(ops)
    return out


def order_interleaved(pp, v, n_mb, nano: bool = False) -> List[List[Op]]:
    """Megatron interleaved 1F1B: micro-batches advance in groups of pp through the v chunks.

    ``nano`` (``--use-nanopipe``): backward is split into the input-gradient part B and the weight-gradient part W.  On rank
    r the first 2 r backward steps run B only - the ranks before it in the pipeline get their output gradients one
    weight-gradient GEMM earlier per step, which is what shortens the start of the backward wave - and their W parts run
    after the rank's last backward, in what would be its tail bubble; every other backward is followed by a W at once
    (reference: mindspeed/core/pipeline_parallel/ripipe_schedules.py:166-170, 542-552, 738-744)."""
    if n_mb % pp != 0:
        raise ValueError("interleaved schedule needs the number of micro-batches to be a multiple of the pipeline size")
    total = n_mb * v

    def fwd_id(k):   # k-th forward on a rank -> (chunk, mb)
        g, i = divmod(k, pp * v)
        return (i // pp), g * pp + i % pp

    def bwd_id(k):
        g, i = divmod(k, pp * v)
        return v - 1 - (i // pp), g * pp + i % pp

    out = []
    for r in range(pp):
        warm = min((pp - r - 1) * 2 + (v - 1) * pp, total)
        ops = []
        f = b = 0
        for _ in range(warm):
            c, m = fwd_id(f); ops.append(Op("F", c, m)); f += 1
        num_dx = min(2 * r, total) if nano else 0
        late: List[Op] = []

        def back():
            nonlocal b
            c, m = bwd_id(b)
            ops.append(Op("B", c, m))
            if nano:
                (late if b < num_dx else ops).append(Op("W", c, m))
            b += 1
        for _ in range(total - warm):
            c, m = fwd_id(f); ops.append(Op("F", c, m)); f += 1
            back()
        while b < total:
            back()
        out.append(ops + late)
    return out


def order_dualpipev(pp, n_mb, split_w=True) -> List[List[Op]]:
    """DualPipeV (cut-in-half) order.  Every rank holds chunk 0 (down the V) and chunk 1 (back up).
    Phases per rank i with P = 2*pp: warm-up forwards of chunk 0, interleaved F0/F1, 1B1W1F, steady F&B pairs,
    1B-1pair, interleaved backwards, cool-down with the deferred W work (reference phase counts:
    dualpipev_schedules.py:320-334)."""
    if n_mb < 2 * pp:
        raise ValueError("DualPipeV needs at least 2 * pp micro-batches")
    P = 2 * pp
    out = []
    for i in range(pp):
        ops: List[Op] = []
        f = [0, 0]; b = [0, 0]; w = [0, 0]

        def F(c):
            ops.append(Op("F", c, f[c])); f[c] += 1

        def B(c, full=False):
            ops.append(Op("B", c, b[c])); b[c] += 1
            if full or not split_w:
                ops.append(Op("W", c, w[c])); w[c] += 1

        def W(c):
            if split_w and w[c] < b[c]:
                ops.append(Op("W", c, w[c])); w[c] += 1

        # 1. warm-up: forwards of chunk 0
        for _ in range(P - 2 - 2 * i):
            F(0)
        # 2. interleaved forward: F0 then F1
        for _ in range(i + 1):
            F(0); F(1)
        # 3. 1B1W1F: backward of chunk 1 (input grad), its weight grad, forward of chunk 1
        for _ in range(P // 2 - i - 1):
            B(1); W(1); F(1)
        # 4. steady state: pairs (F0 & B1) then (F1 & B0), full backward (no W split) as comm hides under the pair
        steady = n_mb - P + i + 1
        for _ in range(max(steady, 0)):
            if f[0] < n_mb:
                F(0)
            B(1, full=True)
            if f[1] < n_mb:
                F(1)
            B(0, full=True)
        # 5. 1B1overlap: remaining forwards of chunk 1 paired with backwards
        while f[1] < n_mb:
            B(1, full=True); F(1); B(0, full=True)
        # 6. interleaved backward / 7. cool-down: drain backwards, W deferred behind them
        while b[0] < n_mb or b[1] < n_mb:
            if b[1] < n_mb and (b[1] <= b[0] or b[0] >= n_mb):
                B(1)
            elif b[0] < n_mb:
                B(0)
            W(1); W(0)
        while w[0] < n_mb or w[1] < n_mb:
            if w[1] < n_mb:
                ops.append(Op("W", 1, w[1])); w[1] += 1
            if w[0] < n_mb:
                ops.append(Op("W", 0, w[0])); w[0] += 1
        out.append(ops)
    return out


def order_bidirectional(pp, n_mb, split_w=False) -> List[List[Op]]:
    """Chimera / DualPipe order: micro-batches 0..n/2-1 enter pipeline 0 at rank 0, n/2..n-1 enter pipeline 1 at rank
    pp-1 (local ids 0..n/2-1 per chunk).  Each pipeline follows 1F1B on its own stages; the two are interleaved
    forward-first so that one direction's bubbles are filled by the other."""
    if n_mb % 2 != 0:
        raise ValueError("bidirectional schedules need an even number of micro-batches")
    half = n_mb // 2
    a = order_1f1b(pp, half)                     # pipeline 0: stage == rank
    out = []
    for r in range(pp):
        down = a[r]
        up = [Op(o.kind, 1, o.mb) for o in a[pp - 1 - r]]   # pipeline 1: this rank is stage pp-1-r
        ops, i, j = [], 0, 0
        # merge: alternate, giving priority to the pipeline in which this rank is the earlier stage
        first, second = (down, up) if r < pp - 1 - r or (r == pp - 1 - r) else (up, down)
        while i < len(first) or j < len(second):
            if i < len(first):
                ops.append(first[i]); i += 1
            if j < len(second):
                ops.append(second[j]); j += 1
        if split_w:
            ops2 = []
            for o in ops:
                ops2.append(o)
            ops = ops2
        out.append(ops)
    return out


def greedy_orders(placement: Placement, n_mb: int, split_w: bool = False, cost=None) -> List[List[Op]]:
    """Event-driven list scheduling: every rank, whenever it is free, runs the ready operation of highest priority
    (backward first, then a forward if the 1F1B-style in-flight cap of that chunk allows it, weight-gradient work
    last, so W fills bubbles).  Produces per-rank orders that are consistent by construction; used for the
    bidirectional schedules and as the zero-bubble style variant of the V schedule."""
    cost = cost or ({"F": 1, "B": 1, "W": 1} if split_w else {"F": 1, "B": 2, "W": 0})
    pp, S = placement.pp, placement.num_stages
    pipes = sorted({v[0] for v in placement.stage_of.values()})
    per_pipe = n_mb // len(pipes)
    done: Dict[Tuple[int, int, str, int], int] = {}
    nextF = {k: 0 for k in placement.stage_of}
    nextB = {k: 0 for k in placement.stage_of}
    nextW = {k: 0 for k in placement.stage_of}
    free_at = [0] * pp
    orders: List[List[Op]] = [[] for _ in range(pp)]
    total = len(placement.stage_of) * per_pipe * (3 if split_w else 2)
    count, t = 0, 0
    while count < total:
        for r in range(pp):
            if free_at[r] > t:
                continue
            chunks = [c for (rr, c) in placement.stage_of if rr == r]
            # deepest stage first: it is closest to the loss, so its backward unblocks everybody else
            chunks.sort(key=lambda c: -placement.stage_of[(r, c)][1])
            pick = None
            for c in chunks:                      # 1. backward
                pipe, st = placement.stage_of[(r, c)]
                m = nextB[(r, c)]
                if m < per_pipe and done.get((pipe, st, "F", m), 1 << 30) <= t and \
                        (st == S - 1 or done.get((pipe, st + 1, "B", m), 1 << 30) <= t):
                    pick = Op("B", c, m)
                    break
            if pick is None:
                for c in chunks:                  # 2. forward under the in-flight cap
                    pipe, st = placement.stage_of[(r, c)]
                    m = nextF[(r, c)]
                    if m < per_pipe and (st == 0 or done.get((pipe, st - 1, "F", m), 1 << 30) <= t) and \
                            nextF[(r, c)] - nextB[(r, c)] < S - st:
                        pick = Op("F", c, m)
                        break
            if pick is None and split_w:
                for c in chunks:                  # 3. weight gradients fill the gap
                    if nextW[(r, c)] < nextB[(r, c)]:
                        pick = Op("W", c, nextW[(r, c)])
                        break
            if pick is None:
                continue
            pipe, st = placement.stage_of[(r, pick.chunk)]
            fin = t + max(cost[pick.kind], 1)
            done[(pipe, st, pick.kind, pick.mb)] = fin
            free_at[r] = fin
            orders[r].append(pick)
            {"F": nextF, "B": nextB, "W": nextW}[pick.kind][(r, pick.chunk)] += 1
            count += 1
        t += 1
        if t > 100000:
            raise RuntimeError("greedy pipeline scheduling did not terminate")
    return orders


# ------------------------------------------------------------------------------------------------
# slot assignment
# ------------------------------------------------------------------------------------------------
@dataclass
class Message:
    kind: str        # "act" (forward activation) or "grad" (activation gradient)
    src: int
    dst: int
    src_chunk: int
    dst_chunk: int
    mb: int
    slot: int        # slot in which it is sent AND received


@dataclass
class Plan:
    placement: Placement
    table: List[List[List[Op]]]            # [rank][slot] -> ops
    messages: List[Message]
    n_mb: int
    num_slots: int = 0
    sends: Dict[Tuple[int, int], List[Message]] = field(default_factory=dict)   # (rank, slot)
    recvs: Dict[Tuple[int, int], List[Message]] = field(default_factory=dict)

    def bubble_fraction(self, cost: Dict[str, float] = None) -> float:
        cost = dict({"F": 1.0, "B": 2.0, "W": 0.0, "R": 1.0}, **(cost or {}))
        busy = [sum(cost[o.kind] for ops in rank for o in ops) for rank in self.table]
        slot_cost = [max((sum(cost[o.kind] for o in self.table[r][t]) for r in range(len(self.table))), default=0)
                     for t in range(self.num_slots)]
        total = sum(slot_cost)
        return 1.0 - (sum(busy) / len(busy)) / total if total > 0 else 0.0


def assign_slots(placement: Placement, orders: List[List[Op]], n_mb: int, pair_fb: bool = False) -> Plan:
    pp = placement.pp
    done: Dict[Tuple[int, int, str, int], int] = {}   # (pipe, stage, kind, mb) -> slot finished
    ptr = [0] * pp
    table: List[List[List[Op]]] = [[] for _ in range(pp)]
    S = placement.num_stages
    t = 0
    remaining = sum(len(o) for o in orders)
    guard = 0
    while remaining > 0:
        progressed = False
        finished_now = []
        for r in range(pp):
            ops_here: List[Op] = []
            if ptr[r] < len(orders[r]):
                op = orders[r][ptr[r]]
                pipe, stage = placement.stage_of[(r, op.chunk)]
                ok = True
                if op.kind == "F" and stage > 0:
                    ok = done.get((pipe, stage - 1, "F", op.mb), 1 << 30) < t
                elif op.kind == "B":
                    ok = done.get((pipe, stage, "F", op.mb), 1 << 30) < t
                    if ok and stage < S - 1:
                        ok = done.get((pipe, stage + 1, "B", op.mb), 1 << 30) < t
                elif op.kind == "W":
                    ok = (pipe, stage, "B", op.mb) in done
                elif op.kind == "R":
                    ok = done.get((pipe, stage, "F", op.mb), 1 << 30) < t
                if ok:
                    ops_here.append(op)
                    finished_now.append((pipe, stage, op.kind, op.mb, r))
                    ptr[r] += 1
                    remaining -= 1
                    progressed = True
                    # forward/backward overlap: an F directly followed by a B of another micro-batch (or the other way round)
                    # shares the slot when that op's inputs are ready too - the executor interleaves the two
                    if pair_fb and op.kind in ("F", "B") and ptr[r] < len(orders[r]):
                        nx = orders[r][ptr[r]]
                        if {nx.kind, op.kind} == {"F", "B"} and (nx.chunk, nx.mb) != (op.chunk, op.mb):
                            npipe, nstage = placement.stage_of[(r, nx.chunk)]
                            if nx.kind == "F":
                                nok = nstage == 0 or done.get((npipe, nstage - 1, "F", nx.mb), 1 << 30) < t
                            else:
                                nok = done.get((npipe, nstage, "F", nx.mb), 1 << 30) < t and \
                                    (nstage == S - 1 or done.get((npipe, nstage + 1, "B", nx.mb), 1 << 30) < t)
                            if nok:
                                ops_here.append(nx)
                                finished_now.append((npipe, nstage, nx.kind, nx.mb, r))
                                ptr[r] += 1
                                remaining -= 1
                    # a W directly after its B may share the slot (same rank, no communication in between)
                    while ptr[r] < len(orders[r]) and orders[r][ptr[r]].kind == "W":
                        w = orders[r][ptr[r]]
                        wp, ws = placement.stage_of[(r, w.chunk)]
                        if (wp, ws, "B", w.mb) in done or any(x[:4] == (wp, ws, "B", w.mb) for x in finished_now):
                            ops_here.append(w)
                            finished_now.append((wp, ws, "W", w.mb, r))
                            ptr[r] += 1
                            remaining -= 1
                        else:
                            break
            table[r].append(ops_here)
        for (pipe, stage, kind, mb, r) in finished_now:
            done[(pipe, stage, kind, mb)] = t
        t += 1
        guard = 0 if progressed else guard + 1
        if guard > 2:
            stuck = {r: orders[r][ptr[r]] for r in range(pp) if ptr[r] < len(orders[r])}
            raise RuntimeError(f"pipeline order deadlocks at slot {t}: waiting ops {stuck}")
    plan = Plan(placement, table, [], n_mb, num_slots=t)
    # messages: output of F at stage s -> holder of stage s+1; input-grad of B at stage s -> holder of stage s-1
    for r in range(pp):
        for slot, ops in enumerate(table[r]):
            for op in ops:
                pipe, stage = placement.stage_of[(r, op.chunk)]
                if op.kind == "F" and stage < S - 1:
                    dr, dc = placement.holder(pipe, stage + 1)
                    plan.messages.append(Message("act", r, dr, op.chunk, dc, op.mb, slot + 1))
                elif op.kind == "B" and stage > 0:
                    dr, dc = placement.holder(pipe, stage - 1)
                    plan.messages.append(Message("grad", r, dr, op.chunk, dc, op.mb, slot + 1))
    for m in plan.messages:
        if m.src == m.dst:
            continue   # V turn-around or same-rank hand-over: no communication
        plan.sends.setdefault((m.src, m.slot), []).append(m)
        plan.recvs.setdefault((m.dst, m.slot), []).append(m)
    plan.num_slots = max(plan.num_slots, max((m.slot for m in plan.messages), default=0) + 1)
    for r in range(pp):
        while len(table[r]) < plan.num_slots:
            table[r].append([])
    return plan


def simulate_orders(placement: Placement, orders: List[List[Op]], cost: Dict[str, float]):
    """Event-driven execution of fixed per-rank orders with operation costs; returns (makespan, bubble fraction)."""
    S = placement.num_stages
    fin: Dict[Tuple[int, int, str, int], float] = {}
    ptr = [0] * placement.pp
    clock = [0.0] * placement.pp
    left = sum(len(o) for o in orders)
    while left > 0:
        moved = False
        for r in range(placement.pp):
            while ptr[r] < len(orders[r]):
                op = orders[r][ptr[r]]
                pipe, st = placement.stage_of[(r, op.chunk)]
                deps = []
                if op.kind == "F" and st > 0:
                    deps.append((pipe, st - 1, "F", op.mb))
                if op.kind == "B":
                    deps.append((pipe, st, "F", op.mb))
                    if st < S - 1:
                        deps.append((pipe, st + 1, "B", op.mb))
                if op.kind == "W":
                    deps.append((pipe, st, "B", op.mb))
                if op.kind == "R":
                    deps.append((pipe, st, "F", op.mb))
                if any(d not in fin for d in deps):
                    break
                start = max([clock[r]] + [fin[d] for d in deps])
                clock[r] = start + cost[op.kind]
                fin[(pipe, st, op.kind, op.mb)] = clock[r]
                ptr[r] += 1
                left -= 1
                moved = True
        if not moved:
            raise RuntimeError("orders deadlock")
    makespan = max(clock)
    busy = sum(sum(cost[o.kind] for o in ops) for ops in orders) / placement.pp
    return makespan, 1.0 - busy / makespan


def validate(plan: Plan) -> None:
    """Every (stage, mb) has exactly one F and one B, F before B, dependencies respected across ranks."""
    seen = {}
    for r, rank in enumerate(plan.table):
        for slot, ops in enumerate(rank):
            for op in ops:
                key = (plan.placement.stage_of[(r, op.chunk)], op.kind, op.mb)
                if key in seen:
                    raise AssertionError(f"duplicate {op} on rank {r}")
                seen[key] = slot
    S = plan.placement.num_stages
    pipes = {v[0] for v in plan.placement.stage_of.values()}
    per_pipe = plan.n_mb // len(pipes)
    for pipe in pipes:
        for s in range(S):
            for mb in range(per_pipe):
                f, b = seen[((pipe, s), "F", mb)], seen[((pipe, s), "B", mb)]
                assert f < b, (pipe, s, mb)
                if s > 0:
                    assert seen[((pipe, s - 1), "F", mb)] < f
                    assert b < seen[((pipe, s - 1), "B", mb)]


def plan_from_stage_lists(pp: int, n_mb: int, stages: Dict[str, List[str]]) -> Plan:
    """A stored schedule of the non-interleaved pipeline: ``{"stage0": ["F1", "F2", "B1", ...], "stage1": [...]}`` - per
    pipeline rank the order of its forward (F) and backward (B) steps with 1-based micro-batch numbers, the form
    ``--pp-schedule-list`` carries (reference: mindspeed/core/pipeline_parallel/flexible_schedules.py:265-305, 431-446).
    The lists are checked (every micro-batch once per kind, backward after forward) and turned into a slot table; an order
    in which two ranks wait for each other is reported instead of being run."""
    orders: List[List[Op]] = []
    for r in range(pp):
        key = f"stage{r}"
        if key not in stages:
            raise ValueError(f"--pp-schedule-list has no entry {key!r} (pipeline size {pp})")
        ops, seen = [], set()
        for tag in stages[key]:
            kind, num = tag[:1].upper(), tag[1:]
            if kind not in ("F", "B") or not num.isdigit() or not (1 <= int(num) <= n_mb):
                raise ValueError(f"{key}: {tag!r} is not F<k> or B<k> with 1 <= k <= {n_mb}")
            mb = int(num) - 1
            if (kind, mb) in seen or (kind == "B" and ("F", mb) not in seen):
                raise ValueError(f"{key}: {tag!r} is repeated or comes before its forward")
            seen.add((kind, mb))
            ops.append(Op(kind, 0, mb))
        if len(seen) != 2 * n_mb:
            raise ValueError(f"{key}: {len(seen)} steps listed, {2 * n_mb} expected (one F and one B per micro-batch)")
        orders.append(ops)
    plan = assign_slots(placement_1f1b(pp), orders, n_mb)
    validate(plan)
    return plan


def insert_recompute(orders: List[List[Op]], mode: str = "bubble") -> List[List[Op]]:
    """Scheduler-placed recompute (RiPipe): the forward of (chunk, mb) drops its activations and an ``R`` op rebuilds
    them before the backward.

      * a forward whose backward follows it directly keeps its activations: no R (this removes the recompute of
        the last stage's steady state and of every stage's final micro-batches);
      * mode "bubble":  R sits directly in front of its B.  R needs nothing from other ranks, so in the slot table it
        runs while the rank would otherwise wait for the gradient from downstream - inside the bubble when there is
        one;
      * mode "advance": R is moved one operation earlier than that, so the rebuilt activations are already there when
        the gradient arrives and the recompute never sits between the arrival of a gradient and its backward.
    reference: mindspeed/core/pipeline_parallel/ripipe_schedules.py:41-799 (--recompute-in-bubble / --recompute-in-advance).
    """
    if mode not in ("bubble", "advance"):
        raise ValueError("recompute mode must be 'bubble' or 'advance'")
    out = []
    for ops in orders:
        new: List[Op] = []
        for i, op in enumerate(ops):
            if op.kind == "B":
                prev = ops[i - 1] if i > 0 else None
                keep = prev is not None and prev.kind == "F" and (prev.chunk, prev.mb) == (op.chunk, op.mb)
                if not keep:
                    r = Op("R", op.chunk, op.mb)
                    if mode == "advance" and new and not (new[-1].kind == "F" and (new[-1].chunk, new[-1].mb) == (op.chunk, op.mb)):
                        new.insert(len(new) - 1, r)
                    else:
                        new.append(r)
            new.append(op)
        out.append(new)
    return out


def recomputed_forwards(orders: List[List[Op]]) -> List[set]:
    """Per rank: the (chunk, mb) pairs whose forward must not keep activations (they have an R op)."""
    return [{(o.chunk, o.mb) for o in ops if o.kind == "R"} for ops in orders]


def build_plan(name: str, pp: int, n_mb: int, vpp: Optional[int] = None, split_w: bool = True,
               recompute: Optional[str] = None, pair_fb: bool = False) -> Plan:
    if name == "1f1b":
        pl, orders = placement_1f1b(pp), order_1f1b(pp, n_mb)
    elif name in ("interleaved", "nanopipe"):
        pl, orders = placement_interleaved(pp, vpp), order_interleaved(pp, vpp, n_mb, nano=(name == "nanopipe"))
    elif name == "dualpipev":
        pl = placement_v(pp)
        orders = order_dualpipev(pp, n_mb, split_w)
    elif name == "dualpipev_greedy":
        pl = placement_v(pp)
        orders = greedy_orders(pl, n_mb, split_w)
    elif name in ("dualpipe", "chimera"):
        pl = placement_bidirectional(pp)
        if n_mb % 2 != 0:
            raise ValueError("bidirectional schedules need an even number of micro-batches")
        orders = greedy_orders(pl, n_mb, split_w and name == "dualpipe")
    else:
        raise ValueError(name)
    if recompute:
        orders = insert_recompute(orders, recompute)
    return assign_slots(pl, orders, n_mb, pair_fb=pair_fb)
