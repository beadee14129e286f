"""Randomised interleaving simulation of the device-side synchronisation protocols.

compute-sanitizer's racecheck is not available where this library is developed, so the protocols that carry the
cross-CTA and cross-GPU ordering are restated here as small state machines (one Python generator per CTA or thread
role; every ``yield`` is a point where any other role may run) and executed under thousands of random schedules:

* ``rank_barrier``            epoch inboxes in every rank's signal pad (csrc/device/sync.cuh)
* ticket + arrival counters   fused GEMM -> all-reduce: producers bump the owner's per-tile counter, reducer CTAs draw
                              tickets, wait for ``world`` arrivals, re-arm the counter; the ticket counter is re-armed
                              by whoever draws the last ticket (csrc/gemm/gemm_kernel.cuh: draw_ticket, ar_reducer_role)
* two-SM in-place reduction   warps draw sub-unit items (next ticket drawn ahead), the unit's last finished item re-arms
                              its arrival and done counters, GEMM CTAs join the reducers, ranks run ahead into the next
                              launch; only the closing rank barrier keeps a new arrival from meeting an un-re-armed unit
                              (csrc/gemm/gemm_pair.cu: signal warp, draw_ticket_warp, pair_ar_reducer)
* push all-reduce             one barrier per call; two sets of pieces selected by a call counter that the last block
                              of a call bumps; ranks run ahead into later calls (csrc/collectives/allreduce_push.cu)
* flag-in-data all-reduce     no barrier: 8-byte cells of data + call number, two sets, message lengths that differ
                              from call to call, and the restart of the call numbers by recover()
                              (csrc/collectives/allreduce_ll.cu)
* last-arriver split-K sum    per-quadrant arrival counter re-armed by the CTA that completes it
                              (csrc/gemm/gemm_kernel.cuh, csrc/gemm/gemm_skinny.cu)

What is checked: no role waits forever, every unit of work is done exactly once and only after its inputs were
complete, and every counter is back at its initial value when a launch ends, so the next launch (run here back to
back on the same memory) starts from the state it expects.  The memory model is sequential consistency: these
tests find protocol errors (lost updates, double consumption, stale re-arms), not missing fences.
"""
import random

import pytest


def run_schedule(roles, rng, max_steps=200000):
    """Runs generator roles to completion under a random schedule; a role that yields "blocked" made no progress."""
    live = list(roles)
    idle_rounds = 0
    steps = 0
    while live:
        steps += 1
        assert steps < max_steps, "schedule did not terminate"
        g = rng.choice(live)
        try:
            state = next(g)
        except StopIteration:
            live.remove(g)
            idle_rounds = 0
            continue
        if state == "blocked":
            idle_rounds += 1
            # every live role blocked many times in a row: nobody can make progress any more
            assert idle_rounds < 50 * len(live) + 1000, "deadlock: every remaining role is waiting"
        else:
            idle_rounds = 0


# ---------------------------------------------------------------------------------------------------------------------
# rank_barrier
# ---------------------------------------------------------------------------------------------------------------------
class Pads:
    def __init__(self, world, slots):
        self.epoch = [[0] * slots for _ in range(world)]                      # per rank, per slot (own memory)
        self.inbox = [[[0] * world for _ in range(slots)] for _ in range(world)]  # [rank][slot][peer]


def barrier_block(pads, world, rank, slot, rounds, log):
    """Block `slot` of `rank`: `rounds` barriers with a little "work" in between (an entry in the log)."""
    for r in range(rounds):
        log.append(("enter", rank, slot, r))
        yield
        pads.epoch[rank][slot] += 1          # thread 0: s_epoch = *ep + 1; *ep = s_epoch
        e = pads.epoch[rank][slot]
        yield
        for peer in range(world):            # threads 0..world-1 run concurrently on the device; any order is one of them
            pads.inbox[peer][slot][rank] = e  # st.release.sys to the peer's inbox
            yield
        for peer in range(world):
            while pads.inbox[rank][slot][peer] - e < 0:  # wait_word_ge: (int)(v - want) >= 0
                yield "blocked"
            yield
        log.append(("leave", rank, slot, r))
        yield


@pytest.mark.parametrize("world,slots,rounds", [(2, 1, 4), (3, 2, 3), (4, 2, 3), (8, 1, 2)])
def test_rank_barrier_orders_every_round(world, slots, rounds):
    for seed in range(300):
        rng = random.Random(seed * 7919 + world)
        pads, log = Pads(world, slots), []
        roles = [barrier_block(pads, world, r, s, rounds, log) for r in range(world) for s in range(slots)]
        run_schedule(roles, rng)
        # nobody leaves round r of a slot before everybody has entered it
        for s in range(slots):
            for r in range(rounds):
                first_leave = min(i for i, ev in enumerate(log) if ev == ("leave", ev[1], s, r) and ev[0] == "leave")
                last_enter = max(i for i, ev in enumerate(log) if ev[0] == "enter" and ev[2] == s and ev[3] == r)
                assert last_enter < first_leave, (seed, s, r)
        assert all(pads.epoch[r][s] == rounds for r in range(world) for s in range(slots))


# ---------------------------------------------------------------------------------------------------------------------
# fused GEMM -> all-reduce: arrival counters, tickets, re-arming, two launches back to back
# ---------------------------------------------------------------------------------------------------------------------
class ArState:
    def __init__(self, world, tiles):
        self.world, self.tiles = world, tiles
        self.owned_max = (tiles + world - 1) // world
        self.counter = [[0] * self.owned_max for _ in range(world)]  # arrivals per owned tile, in the owner's pad
        self.ticket = [0] * world
        self.pushed = [[set() for _ in range(self.owned_max)] for _ in range(world)]  # which source ranks have pushed
        self.reduced = [[0] * self.owned_max for _ in range(world)]


def gemm_cta(st, rank, my_tiles, launch, pads, slot, reducer_ctas_total):
    """A GEMM CTA of `rank`: computes its tiles, pushes each to the owner, signals; then joins the reducers."""
    for seq in my_tiles:
        owner, k = seq % st.world, seq // st.world
        yield
        st.pushed[owner][k].add((launch, rank))   # bulk tensor stores into the owner's staging buffer
        yield
        st.counter[owner][k] += 1                 # signal warp: red.release.sys on the owner's counter
        yield
    yield from reducer_cta(st, rank, launch, pads, slot, reducer_ctas_total)


def reducer_cta(st, rank, launch, pads, slot, drawers):
    owned = (st.tiles - rank + st.world - 1) // st.world
    while True:
        t = st.ticket[rank]                       # atomicAdd(ticket, 1)
        st.ticket[rank] += 1
        if t == owned + drawers - 1:
            st.ticket[rank] = 0                   # the last ticket that can ever be drawn re-arms the counter
        yield
        if t >= owned:
            break
        k = t
        while st.counter[rank][k] < st.world:     # wait_word_ge(cnt, world)
            yield "blocked"
        st.counter[rank][k] = 0                   # single consumer: re-arm now
        yield
        # every rank's slice of THIS launch must be in place when the tile is summed
        assert st.pushed[rank][k] == {(launch, r) for r in range(st.world)}, (rank, k, st.pushed[rank][k])
        st.pushed[rank][k] = set()
        st.reduced[rank][k] += 1
        yield
    # final barrier between block `slot` of every rank (rank_barrier)
    yield from barrier_block(pads, st.world, rank, slot, 1, [])


@pytest.mark.parametrize("world,tiles,gemm_ctas,comm_ctas", [(2, 5, 2, 1), (2, 8, 3, 2), (4, 9, 2, 1), (3, 4, 1, 2)])
def test_fused_all_reduce_counters_and_tickets(world, tiles, gemm_ctas, comm_ctas):
    ctas = gemm_ctas + comm_ctas
    for seed in range(150):
        rng = random.Random(seed * 104729 + tiles)
        st, pads = ArState(world, tiles), Pads(world, ctas)
        for launch in range(2):  # the second launch runs on the memory the first one left behind
            roles = []
            for rank in range(world):
                for c in range(gemm_ctas):
                    roles.append(gemm_cta(st, rank, list(range(c, tiles, gemm_ctas)), launch, pads, c, ctas))
                for c in range(comm_ctas):
                    roles.append(reducer_cta(st, rank, launch, pads, gemm_ctas + c, ctas))
            run_schedule(roles, rng)
            for rank in range(world):
                owned = (tiles - rank + world - 1) // world
                assert st.reduced[rank][:owned] == [launch + 1] * owned, (seed, launch, rank, st.reduced[rank])
                assert st.ticket[rank] == 0 and all(c == 0 for c in st.counter[rank]), (seed, launch, rank)


# ---------------------------------------------------------------------------------------------------------------------
# two-SM fused GEMM -> all-reduce: in-place reduction by WARPS that draw sub-unit items, a per-unit "done" counter whose
# last increment re-arms the unit, GEMM CTAs that join the reducers, and ranks that run ahead into the next launch
# (csrc/gemm/gemm_pair.cu: signal warp, draw_ticket_warp, pair_ar_reducer)
# ---------------------------------------------------------------------------------------------------------------------
class PairArState:
    def __init__(self, world, units, subs, launches):
        self.world, self.units, self.subs = world, units, subs
        self.owned_max = (units + world - 1) // world
        self.cnt = [[0] * self.owned_max for _ in range(world)]     # arrivals per owned unit (owner's pad)
        self.done = [[0] * self.owned_max for _ in range(world)]    # finished items per owned unit
        self.ticket = [0] * world
        self.arrived = [[set() for _ in range(self.owned_max)] for _ in range(world)]  # (launch, source rank)
        self.reduced = {}                                           # (launch, rank, k, sub) -> times
        self.gemm_done = {}                                         # (launch, rank, cta) -> True once its tiles are out
        self.warps_done = {}                                        # (launch, rank, cta) -> warps that left the item loop
        self.ctas_done = [[0] * launches for _ in range(world)]     # CTAs of (rank, launch) that have ended

    def owned(self, rank):
        return (self.units - rank + self.world - 1) // self.world


def pair_signal_part(st, rank, cta, my_units, launch, ctas_per_rank):
    """The GEMM part of a CTA: starts when the rank's previous launch has ended (stream order), stores each of its
    half-tiles into the rank's own copy of C and adds one arrival on the owner's counter."""
    while launch > 0 and st.ctas_done[rank][launch - 1] < ctas_per_rank:
        yield "blocked"
    for u in my_units:
        owner, k = u % st.world, u // st.world
        yield
        # an arrival of this launch must find the unit re-armed: nothing of an earlier launch may be left in it
        assert all(l == launch for l, _ in st.arrived[owner][k]), (launch, rank, u, st.arrived[owner][k])
        assert st.cnt[owner][k] < st.world
        st.arrived[owner][k].add((launch, rank))
        st.cnt[owner][k] += 1                     # fence.acq_rel.sys + red.release.sys.add
        yield
    st.gemm_done[(launch, rank, cta)] = True
    yield


def pair_reducer_warp(st, rank, cta, launch, drawers, ctas_per_rank, is_comm_cta):
    """One warp of a CTA in the reducer role (communication CTAs from the start, GEMM CTAs after their tiles)."""
    while launch > 0 and st.ctas_done[rank][launch - 1] < ctas_per_rank:
        yield "blocked"
    while not is_comm_cta and not st.gemm_done.get((launch, rank, cta)):
        yield "blocked"
    items = st.owned(rank) * st.subs

    def draw():
        t = st.ticket[rank]                       # lane 0: atomicAdd(ticket, 1)
        st.ticket[rank] += 1
        if t == items + drawers - 1:
            st.ticket[rank] = 0                   # the last ticket that can ever be drawn re-arms the ticket counter
        return t

    nxt = draw()
    yield
    while True:
        i = nxt
        if i >= items:
            break
        nxt = draw()                              # drawn before the item is processed
        yield
        k, sub = divmod(i, st.subs)
        while st.cnt[rank][k] < st.world:         # lane 0: wait_word_ge(cnt, world)
            yield "blocked"
        yield
        assert st.arrived[rank][k] == {(launch, r) for r in range(st.world)}, (launch, rank, k, st.arrived[rank][k])
        key = (launch, rank, k, sub)
        st.reduced[key] = st.reduced.get(key, 0) + 1   # multimem.ld_reduce + multimem.st of the item's rows
        yield
        d = st.done[rank][k]                      # lane 0: atomicAdd(done, 1)
        st.done[rank][k] += 1
        if d == st.subs - 1:                      # the unit's last item: re-arm both counters
            st.arrived[rank][k] = set()
            st.cnt[rank][k] = 0
            st.done[rank][k] = 0
        yield
    st.warps_done[(launch, rank, cta)] = st.warps_done.get((launch, rank, cta), 0) + 1
    yield


def pair_cta_tail(st, rank, cta, launch, warps, pads):
    """__syncthreads_and over the CTA's warps, then the rank barrier between CTA `cta` of every rank, then the end."""
    while st.warps_done.get((launch, rank, cta), 0) < warps:
        yield "blocked"
    yield from barrier_block(pads, st.world, rank, cta, 1, [])
    st.ctas_done[rank][launch] += 1
    yield


@pytest.mark.parametrize("world,units,gemm_ctas,comm_ctas,subs,warps",
                         [(2, 6, 2, 1, 2, 2), (2, 9, 3, 1, 3, 2), (4, 10, 2, 1, 2, 2), (3, 7, 2, 2, 2, 3)])
def test_two_sm_in_place_reduction_with_joining_warps_and_ranks_running_ahead(world, units, gemm_ctas, comm_ctas, subs, warps):
    ctas, launches = gemm_ctas + comm_ctas, 3
    for seed in range(120):
        rng = random.Random(seed * 611953 + units)
        st, pads = PairArState(world, units, subs, launches), Pads(world, ctas)
        roles = []
        for launch in range(launches):  # all launches are live at once: only stream order per rank holds them apart
            for rank in range(world):
                for c in range(ctas):
                    is_comm = c >= gemm_ctas
                    if not is_comm:
                        roles.append(pair_signal_part(st, rank, c, list(range(c, units, gemm_ctas)), launch, ctas))
                    for _ in range(warps):
                        roles.append(pair_reducer_warp(st, rank, c, launch, ctas * warps, ctas, is_comm))
                    roles.append(pair_cta_tail(st, rank, c, launch, warps, pads))
        run_schedule(roles, rng, max_steps=2000000)
        for launch in range(launches):
            for rank in range(world):
                for k in range(st.owned(rank)):
                    for sub in range(subs):
                        assert st.reduced.get((launch, rank, k, sub)) == 1, (seed, launch, rank, k, sub)
        assert len(st.reduced) == launches * units * subs
        for rank in range(world):
            assert st.ticket[rank] == 0 and not any(st.cnt[rank]) and not any(st.done[rank]), (seed, rank)


# ---------------------------------------------------------------------------------------------------------------------
# split-K: last arriver sums and re-arms
# ---------------------------------------------------------------------------------------------------------------------
def splitk_cta(state, tile, split, splits, launch):
    yield
    state["partial"][tile][split] = launch          # fp32 partial tile written to the workspace
    yield                                           # __threadfence
    prev = state["count"][tile]                     # atomicAdd(qcnt, 1)
    state["count"][tile] += 1
    yield
    if prev == splits - 1:
        state["count"][tile] = 0                    # re-arm for the next call
        yield
        assert state["partial"][tile] == [launch] * splits, (tile, state["partial"][tile])
        state["summed"][tile] += 1


@pytest.mark.parametrize("tiles,splits", [(1, 2), (3, 5), (4, 8)])
def test_split_k_last_arriver(tiles, splits):
    for seed in range(200):
        rng = random.Random(seed * 31 + splits)
        state = {"partial": [[None] * splits for _ in range(tiles)], "count": [0] * tiles, "summed": [0] * tiles}
        for launch in range(3):
            roles = [splitk_cta(state, t, s, splits, launch) for t in range(tiles) for s in range(splits)]
            run_schedule(roles, rng)
            assert state["summed"] == [launch + 1] * tiles and state["count"] == [0] * tiles


def test_the_simulator_finds_a_planted_bug():
    """Sanity of the method: a reducer that re-arms the counter AFTER summing (instead of before any later arrival can
    happen) is harmless, but one that draws tickets without the re-arm rule leaves the ticket counter dirty."""
    world, tiles = 2, 4
    st, pads = ArState(world, tiles), Pads(world, 2)

    def broken_reducer(rank):
        owned = (tiles - rank + world - 1) // world
        while True:
            t = st.ticket[rank]
            st.ticket[rank] += 1  # never re-armed
            yield
            if t >= owned:
                break
            while st.counter[rank][t] < world:
                yield "blocked"
            st.counter[rank][t] = 0
            yield

    roles = [gemm_cta(st, r, list(range(tiles)), 0, pads, 0, 2) for r in range(world)]
    roles += [broken_reducer(r) for r in range(world)]
    with pytest.raises(AssertionError):
        run_schedule(roles, random.Random(0))
        assert all(t == 0 for t in st.ticket)


def test_the_simulator_catches_a_counter_that_is_not_re_armed():
    """Without the re-arm (``*cnt = 0``) the second launch finds the first launch's arrivals still counted and sums a
    tile before this launch's slices are in place: some schedule must trip the reducer's input check."""
    world, tiles, ctas = 2, 2, 2

    def reducer_without_rearm(st, rank, launch, pads, slot):
        owned = (st.tiles - rank + st.world - 1) // st.world
        while True:
            t = st.ticket[rank]
            st.ticket[rank] += 1
            if t == owned + 1 - 1:  # one drawer per rank in this set-up
                st.ticket[rank] = 0
            yield
            if t >= owned:
                break
            while st.counter[rank][t] < st.world * 1:  # stale arrivals of the previous launch satisfy this at once
                yield "blocked"
            yield
            assert st.pushed[rank][t] == {(launch, r) for r in range(st.world)}, "summed before the inputs were complete"
            st.pushed[rank][t] = set()
            yield
        yield from barrier_block(pads, st.world, rank, slot, 1, [])

    def producer(st, rank, launch, pads, slot):
        for seq in range(st.tiles):
            owner, k = seq % st.world, seq // st.world
            yield
            st.pushed[owner][k].add((launch, rank))
            yield
            st.counter[owner][k] += 1
            yield
        yield from barrier_block(pads, st.world, rank, slot, 1, [])

    tripped = 0
    for seed in range(60):
        st, pads = ArState(world, tiles), Pads(world, ctas)
        try:
            for launch in range(2):
                roles = [producer(st, r, launch, pads, 0) for r in range(world)]
                roles += [reducer_without_rearm(st, r, launch, pads, 1) for r in range(world)]
                run_schedule(roles, random.Random(seed))
        except AssertionError:
            tripped += 1
    assert tripped > 0


def test_the_simulator_needs_the_closing_barrier_of_the_two_sm_reduction(monkeypatch):
    """Without the rank barrier at the end of the launch a rank that runs ahead delivers an arrival of the next launch
    into a unit its peer has not re-armed yet: the simulation must find that."""
    import sys
    me = sys.modules[__name__]

    def tail_without_barrier(st, rank, cta, launch, warps, pads):
        while st.warps_done.get((launch, rank, cta), 0) < warps:
            yield "blocked"
        st.ctas_done[rank][launch] += 1
        yield

    monkeypatch.setattr(me, "pair_cta_tail", tail_without_barrier)
    with pytest.raises(AssertionError):
        test_two_sm_in_place_reduction_with_joining_warps_and_ranks_running_ahead(2, 6, 2, 1, 2, 2)


# ---------------------------------------------------------------------------------------------------------------------
# push all-reduce: ONE barrier per call, two sets of pieces selected by a call counter kept on the device
# (csrc/collectives/allreduce_push.cu, push_norm_kernel in csrc/collectives/fused_norm.cu)
# ---------------------------------------------------------------------------------------------------------------------
class PushState:
    def __init__(self, world, blocks, sets):
        self.world, self.blocks, self.sets = world, blocks, sets
        self.calls = [0] * world                  # call-epoch word: push calls this rank has completed
        self.ticket = [0] * world                 # blocks of the running call that have finished
        # staging[rank][set][block][source] = id of the call whose piece lies there
        self.staging = [[[[None] * world for _ in range(blocks)] for _ in range(sets)] for _ in range(world)]
        self.kernels_done = [[0] * 64 for _ in range(world)]  # blocks of (rank, call) that have ended


def push_block(st, pads, rank, block, call):
    """Block `block` of call `call` on `rank`; a rank's calls run in stream order, its blocks concurrently."""
    while call > 0 and st.kernels_done[rank][call - 1] < st.blocks:
        yield "blocked"
    s = st.calls[rank] % st.sets                  # every block reads the counter before any block of this call bumps it
    yield
    for peer in range(st.world):                  # push this block's stripe into piece `rank` on every rank
        if peer != rank:
            st.staging[peer][s][block][rank] = call
            yield
    yield from barrier_block(pads, st.world, rank, block, 1, [])
    for src in range(st.world):                   # sum the pieces from local memory (the own one comes from the input)
        if src != rank:
            assert st.staging[rank][s][block][src] == call, (rank, block, call, src, st.staging[rank][s][block][src])
            yield
    t = st.ticket[rank]                           # the block that finishes last moves on to the other set
    st.ticket[rank] += 1
    if t == st.blocks - 1:
        st.ticket[rank] = 0
        st.calls[rank] += 1
    st.kernels_done[rank][call] += 1
    yield


def _run_push(world, blocks, sets, calls, seeds):
    for seed in range(seeds):
        rng = random.Random(seed * 15485863 + world)
        st, pads = PushState(world, blocks, sets), Pads(world, blocks)
        roles = [push_block(st, pads, r, b, c) for c in range(calls) for r in range(world) for b in range(blocks)]
        run_schedule(roles, rng, max_steps=2000000)
        assert st.calls == [calls] * world and st.ticket == [0] * world


@pytest.mark.parametrize("world,blocks", [(2, 1), (2, 3), (4, 2), (8, 1)])
def test_push_all_reduce_needs_no_closing_barrier_with_two_sets(world, blocks):
    _run_push(world, blocks, sets=2, calls=5, seeds=150)


def test_push_all_reduce_with_one_set_is_caught():
    """With a single set of pieces a rank that runs ahead overwrites a piece its peer has not summed yet."""
    with pytest.raises(AssertionError):
        _run_push(2, 1, sets=1, calls=4, seeds=200)


# ---------------------------------------------------------------------------------------------------------------------
# flag-in-data all-reduce: NO barrier; 8-byte cells {data, call number}; two sets of cells selected by the call counter;
# message lengths differ from call to call; recover() restarts the call numbers
# (csrc/collectives/allreduce_ll.cu, ll_norm_kernel in csrc/collectives/fused_norm.cu, Communicator.recover)
# ---------------------------------------------------------------------------------------------------------------------
class CellState:
    def __init__(self, world, words, sets):
        self.world, self.words, self.sets = world, words, sets
        self.calls = [0] * world
        # cells[rank][set][source][word] = (data, flag); data is the (era, call) that stored it
        self.cells = [[[[(None, 0)] * words for _ in range(world)] for _ in range(sets)] for _ in range(world)]
        self.done = [dict() for _ in range(world)]   # (era, call) -> True once the rank's kernel of that call has ended

    def restart(self, zero_cells):
        """What recover() does between two host barriers (no kernel of any rank is running)."""
        self.calls = [0] * self.world
        if zero_cells:
            for per_rank in self.cells:
                for per_set in per_rank:
                    for src in range(self.world):
                        per_set[src] = [(None, 0)] * self.words


def cell_kernel(st, rank, era, call, length, prev):
    """One single-block kernel of call `call` (of `length` words) on `rank`; `prev` is the rank's previous kernel."""
    while prev is not None and not st.done[rank].get(prev):
        yield "blocked"
    seq = st.calls[rank]
    flag, s = seq + 1, seq % st.sets
    yield
    for w in range(length):                       # store the words, flag attached, into piece `rank` of every peer
        for peer in range(st.world):
            if peer != rank:
                st.cells[peer][s][rank][w] = ((era, call), flag)
                yield
    for w in range(length):                       # poll the peers' cells of the same words
        for src in range(st.world):
            if src == rank:
                continue
            while st.cells[rank][s][src][w][1] != flag:
                yield "blocked"
            data = st.cells[rank][s][src][w][0]
            assert data == (era, call), (rank, src, w, "wanted", (era, call), "summed", data)
            yield
    st.calls[rank] = seq + 1
    st.done[rank][(era, call)] = True
    yield


def _run_cells(world, sets, lengths_by_era, zero_on_restart, seeds):
    words = max(max(ls) for ls in lengths_by_era)
    for seed in range(seeds):
        rng = random.Random(seed * 32452843 + world)
        st = CellState(world, words, sets)
        for era, lengths in enumerate(lengths_by_era):
            if era > 0:
                st.restart(zero_on_restart)
            roles = []
            for r in range(world):
                prev = None
                for c, n in enumerate(lengths):
                    roles.append(cell_kernel(st, r, era, c, n, prev))
                    prev = (era, c)
            run_schedule(roles, rng, max_steps=2000000)
            assert st.calls == [len(lengths)] * world


@pytest.mark.parametrize("world", [2, 4, 8])
def test_flag_in_data_cells_need_no_barrier_with_two_sets(world):
    _run_cells(world, sets=2, lengths_by_era=[[3, 1, 4, 2, 4, 1, 3]], zero_on_restart=True, seeds=120)


def test_flag_in_data_cells_with_one_set_are_caught():
    """With one set a rank that runs ahead overwrites cells of the call its peer is still summing."""
    with pytest.raises(AssertionError):
        _run_cells(2, sets=1, lengths_by_era=[[2, 2, 2, 2]], zero_on_restart=True, seeds=300)


def test_restarting_the_call_numbers_needs_zeroed_cells():
    """After the call numbers restart, a long message whose number matches one from before finds stale cells unless
    the cells were zeroed; with the zeroing the same sequence is clean."""
    eras = [[1, 1, 4], [1, 1, 4]]
    _run_cells(2, sets=2, lengths_by_era=eras, zero_on_restart=True, seeds=100)
    with pytest.raises(AssertionError):
        _run_cells(2, sets=2, lengths_by_era=eras, zero_on_restart=False, seeds=100)
