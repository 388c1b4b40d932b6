"""Protocol models of the cross-rank handshakes, run under random schedules on the CPU.

The fused kernels never reset a flag: buffers and counters that peers write are double-buffered by the parity of a
device-resident epoch, counters only grow, and the value a waiter expects is `base + rows` with `base` advanced at the
end of every call. Whether that is enough (no waiter passes early, no buffer is overwritten while it is still read)
is a property of the protocol, not of the CUDA code, so it is checked here by executing a small model of every rank's
producer and consumer threads under thousands of random interleavings. The same model with the parity removed must
fail, which shows that the checker can see the hazard it is guarding against.

What is modelled: the push gather of AG-GEMM (`csrc/kernels/gemm_sm100.cu`, communication warps and TMA producer), the
slot / counter scheme of GEMM-RS (epilogue stores, signalling warp, reduce phase), and the barrier-free packet
all-reduce (`csrc/kernels/allreduce_ll.cu`).
"""
from __future__ import annotations

import random

import pytest


class Violation(Exception):
    pass


def _run(threads, rng, max_steps=200000):
    """threads: list of generators; each `yield` is a point where another thread may run. A generator yields False while
    it is blocked on a condition (so that a schedule in which everybody is blocked is reported as a deadlock)."""
    live = list(threads)
    blocked_streak = 0
    for _ in range(max_steps):
        if not live:
            return
        t = rng.choice(live)
        try:
            progressed = next(t)
        except StopIteration:
            live.remove(t)
            blocked_streak = 0
            continue
        blocked_streak = 0 if progressed is not False else blocked_streak + 1
        if blocked_streak > 50 * len(live) + 50:
            raise Violation("deadlock: every live thread is blocked")
    raise Violation("schedule did not finish")


# ---------------------------------------------------------------------------------------------- AG push gather
def _ag_push_model(world, rows_per_rank, block, calls, rng, use_parity=True):
    M = world * rows_per_rank
    nblk = (M + block - 1) // block
    npar = 2 if use_parity else 1
    data = [[[None] * M for _ in range(npar)] for _ in range(world)]       # data[rank][parity][row] = (epoch, source)
    cnt = [[[0] * nblk for _ in range(npar)] for _ in range(world)]        # symmetric counters, only ever grow
    base = [[[0] * nblk for _ in range(npar)] for _ in range(world)]       # local
    done_epoch = [0] * world                                              # device-resident epoch of each rank
    finished = [[0, 0] for _ in range(world)]                             # [pusher, consumer] progress per rank

    def rows_in_block(b):
        return min(block, M - b * block)

    def pusher(r):
        for e in range(1, calls + 1):
            while not (finished[r][0] == e - 1 and finished[r][1] == e - 1 and done_epoch[r] == e - 1):
                yield False                                              # kernel e starts when kernel e - 1 has retired
            par = e % npar
            for step in range(world):                                    # step s goes to rank r - s
                dst = (r - step) % world
                for row in range(r * rows_per_rank, (r + 1) * rows_per_rank):
                    data[dst][par][row] = (e, r)
                    yield True
                    cnt[dst][par][row // block] += 1                     # fence + red.release after the stores
                    yield True
            finished[r][0] = e
            yield True

    def consumer(r):
        for e in range(1, calls + 1):
            while not (finished[r][1] == e - 1 and done_epoch[r] == e - 1):
                yield False
            par = e % npar
            first = (r * rows_per_rank) // block
            for k in range(nblk):                                        # own rows first, then the ring order
                b = (first + k) % nblk
                want = base[r][par][b] + rows_in_block(b)
                while cnt[r][par][b] < want:
                    yield False
                for row in range(b * block, b * block + rows_in_block(b)):
                    got = data[r][par][row]
                    if got != (e, row // rows_per_rank):
                        raise Violation(f"rank {r} call {e} block {b} row {row}: read {got}")
                    yield True
            finished[r][1] = e
            while finished[r][0] != e:                                   # last CTA out: both roles are done
                yield False
            for b in range(nblk):
                base[r][par][b] += rows_in_block(b)
            done_epoch[r] = e
            yield True

    _run([pusher(r) for r in range(world)] + [consumer(r) for r in range(world)], rng)


@pytest.mark.parametrize("world,rows,block", [(2, 2, 2), (3, 3, 2), (4, 2, 3), (2, 5, 4)])
def test_ag_push_gather_protocol_is_safe_under_random_schedules(world, rows, block):
    for seed in range(150):
        _ag_push_model(world, rows, block, calls=5, rng=random.Random(seed))


def test_ag_push_gather_without_parity_is_caught():
    """One buffer and one counter set: a fast rank's next call overwrites rows (or inflates counters of blocks that
    straddle two sources) while a slow rank is still in the previous call. The checker must find it."""
    failures = 0
    for seed in range(150):
        try:
            _ag_push_model(3, 3, 2, calls=5, rng=random.Random(seed), use_parity=False)
        except Violation:
            failures += 1
    assert failures > 0


# ---------------------------------------------------------------------------------------------- GEMM-RS slots + counters
def _gemm_rs_model(world, rows_per_rank, tiles_n, calls, rng, use_parity=True):
    """Every rank computes a partial of every row and column tile, stores it into the owner's slot [source][row][tile],
    and adds the delivered rows to the owner's counter for that source; the owner sums the slots of a row block once
    every source has delivered `rows * tiles_n`."""
    npar = 2 if use_parity else 1
    slots = [[[[[None] * tiles_n for _ in range(rows_per_rank)] for _ in range(world)] for _ in range(npar)] for _ in range(world)]
    cnt = [[0] * world for _ in range(world)]        # cnt[owner][source], only ever grows (not parity-split: see below)
    base = [[0] * world for _ in range(world)]
    done_epoch = [0] * world
    finished = [[0, 0] for _ in range(world)]

    def producer(r):
        for e in range(1, calls + 1):
            while not (finished[r][0] == e - 1 and finished[r][1] == e - 1 and done_epoch[r] == e - 1):
                yield False
            par = e % npar
            for step in range(1, world + 1):          # the segment after this rank's first, its own last
                owner = (r + step) % world
                for t in range(tiles_n):
                    for row in range(rows_per_rank):
                        slots[owner][par][r][row][t] = (e, r)
                        yield True
                    cnt[owner][r] += rows_per_rank    # signalling warp: fence, then red.release
                    yield True
            finished[r][0] = e
            yield True

    def reducer(r):
        for e in range(1, calls + 1):
            while not (finished[r][0] == e and done_epoch[r] == e - 1):   # the reduce phase follows the GEMM tiles
                yield False
            par = e % npar
            for s in range(world):
                while cnt[r][s] < base[r][s] + rows_per_rank * tiles_n:
                    yield False
            for s in range(world):
                for row in range(rows_per_rank):
                    for t in range(tiles_n):
                        got = slots[r][par][s][row][t]
                        if got != (e, s):
                            raise Violation(f"rank {r} call {e}: slot of source {s} row {row} tile {t} holds {got}")
                        yield True
            for s in range(world):
                base[r][s] += rows_per_rank * tiles_n
            finished[r][1] = e
            done_epoch[r] = e
            yield True

    _run([producer(r) for r in range(world)] + [reducer(r) for r in range(world)], rng)


@pytest.mark.parametrize("world,rows,tiles", [(2, 2, 2), (3, 2, 2), (4, 1, 3)])
def test_gemm_rs_slot_protocol_is_safe_under_random_schedules(world, rows, tiles):
    """A source can run at most one call ahead of an owner (its call e + 1 cannot end before the owner has delivered
    its rows of call e + 1, i.e. has finished call e), so parity slots plus growing counters are enough: the counter
    of (owner, source) reaches `base + rows * tiles` exactly when the source's stores of THIS call have landed."""
    for seed in range(150):
        _gemm_rs_model(world, rows, tiles, calls=5, rng=random.Random(seed))


def test_gemm_rs_single_slot_buffer_is_caught():
    failures = 0
    for seed in range(150):
        try:
            _gemm_rs_model(3, 2, 2, calls=5, rng=random.Random(seed), use_parity=False)
        except Violation:
            failures += 1
    assert failures > 0


# ---------------------------------------------------------------------------------------------- packet all-reduce
def _ll_allreduce_model(world, words, calls, rng, use_parity=True):
    """Low-latency all-reduce: every word travels as a {data, epoch} packet into slot [source] of every peer's
    workspace; the receiver polls the packets of call e for flag == e. There is no barrier at all, so the only thing
    that keeps a fast rank from overwriting packets a slow rank has not read yet is the parity double-buffering."""
    npar = 2 if use_parity else 1
    ws = [[[[(0, 0)] * words for _ in range(world)] for _ in range(npar)] for _ in range(world)]  # ws[rank][par][src][w]
    done = [0] * world

    def rank_thread(r):
        for e in range(1, calls + 1):
            par = e % npar
            mine = [(r + 1) * 1000 + e * 10 + w for w in range(words)]
            for k in range(1, world):
                peer = (r + k) % world
                for w in range(words):
                    ws[peer][par][r][w] = (mine[w], e)       # one aligned 8-byte store: data and flag land together
                    yield True
            for w in range(words):
                total = 0
                for s in range(world):
                    if s == r:
                        total += mine[w]
                        continue
                    while ws[r][par][s][w][1] != e:
                        yield False
                    total += ws[r][par][s][w][0]
                    yield True
                want = sum((s + 1) * 1000 + e * 10 + w for s in range(world))
                if total != want:
                    raise Violation(f"rank {r} call {e} word {w}: {total} != {want}")
            done[r] = e
            yield True

    _run([rank_thread(r) for r in range(world)], rng)


@pytest.mark.parametrize("world,words", [(2, 3), (4, 2), (8, 1)])
def test_packet_allreduce_needs_no_barrier_with_parity_buffers(world, words):
    for seed in range(200):
        _ll_allreduce_model(world, words, calls=6, rng=random.Random(seed))


def test_packet_allreduce_single_buffer_is_caught():
    """With one buffer a rank that runs ahead replaces packets of call e by packets of call e + 1 before a slow peer has
    read them; the slow peer then waits for a flag that never comes back (reported as a deadlock)."""
    failures = 0
    for seed in range(200):
        try:
            _ll_allreduce_model(3, 2, calls=6, rng=random.Random(seed), use_parity=False)
        except Violation:
            failures += 1
    assert failures > 0


# ---------------------------------------------------------------------------------------------- AG pull gather
def _ag_pull_model(world, calls, rng, compare="ge", use_parity=True):
    """Pull gather of AG-GEMM / AG grouped GEMM: every rank copies its shard into its own symmetric buffer (by epoch
    parity), publishes ready[rank] = epoch on every peer, and pulls a peer's shard once that peer's flag compares true.
    A rank leaves a call as soon as it has pulled everything it needs: it does not wait for anybody to pull from it."""
    npar = 2 if use_parity else 1
    buf = [[None] * npar for _ in range(world)]            # buf[rank][parity] = (epoch, rank) of the shard held there
    ready = [[0] * world for _ in range(world)]            # ready[on rank][source] = last epoch published by source

    def rank_thread(r):
        for e in range(1, calls + 1):
            par = e % npar
            buf[r][par] = (e, r)
            yield True
            for peer in range(world):                       # fence, then a release store of the epoch to every peer
                ready[peer][r] = e
                yield True
            for k in range(1, world):
                src = (r + k) % world
                while not (ready[r][src] == e if compare == "eq" else ready[r][src] >= e):
                    yield False
                got = buf[src][par]
                if got != (e, src):
                    raise Violation(f"rank {r} call {e}: pulled {got} from rank {src}")
                yield True

    _run([rank_thread(r) for r in range(world)], rng)


@pytest.mark.parametrize("world", [2, 3, 4])
def test_ag_pull_gather_is_safe_with_at_least_compare_and_parity(world):
    for seed in range(300):
        _ag_pull_model(world, calls=6, rng=random.Random(seed))


def test_ag_pull_gather_with_equality_compare_deadlocks():
    """A peer that has pulled everything it needs may publish the next epoch before a slow rank has looked at the flag;
    waiting for equality then never ends (on the GPU: until the wait's time budget runs out). Seen at eight ranks."""
    with pytest.raises(Violation, match="deadlock"):
        for seed in range(300):
            _ag_pull_model(3, calls=6, rng=random.Random(seed), compare="eq")


def test_ag_pull_gather_without_parity_is_caught():
    with pytest.raises(Violation):
        for seed in range(300):
            _ag_pull_model(3, calls=6, rng=random.Random(seed), use_parity=False)


# ---------------------------------------------------------------------------------------------- decode GEMM stage ring
def _two_producer_ring_model(stages, kblocks, rng, publish_after_arming=True):
    """The stage ring of the decode GEMM (`csrc/kernels/gemm_skinny_sm100.cu`): a weight producer arms the barrier of a
    stage for the whole stage and requests the weight tile, then publishes how many k-blocks are armed; an activation
    producer (which first waits for the previous kernel) requests the activation tile of k-block i once `armed > i`; the
    MMA thread consumes a stage when both tiles have landed and then frees it. Checked: an activation tile never lands in
    a stage whose barrier is not armed for that k-block (it would complete the transaction count of the wrong phase or
    overwrite a tile that is still being multiplied), and every k-block is multiplied with its own two tiles."""
    armed_for = [None] * stages      # k-block the stage's barrier is armed for (None = free)
    w_in = [None] * stages           # k-block whose weight tile sits in the stage
    x_in = [None] * stages           # k-block whose activation tile sits in the stage
    state = {"armed": 0, "dependency": False, "consumed": 0}

    def weights():
        for i in range(kblocks):
            s = i % stages
            while armed_for[s] is not None:      # wait on the stage's empty barrier
                yield False
            if publish_after_arming:
                armed_for[s] = i                 # expect_tx: the barrier now counts the bytes of both tiles
                yield True
                state["armed"] = i + 1           # published right after the weight tile was requested
                yield True
                w_in[s] = i                      # the weight tile lands (any time after the request)
            else:                                # broken variant: the count is published before the barrier is armed
                state["armed"] = i + 1
                yield True
                armed_for[s] = i
                yield True
                w_in[s] = i
            yield True

    def activations():
        while not state["dependency"]:           # griddepcontrol.wait
            yield False
        for i in range(kblocks):
            s = i % stages
            while state["armed"] <= i:
                yield False
            if armed_for[s] != i:
                raise Violation(f"activation tile of k-block {i} requested into a stage armed for {armed_for[s]}")
            x_in[s] = i
            yield True

    def mma():
        for i in range(kblocks):
            s = i % stages
            while not (armed_for[s] == i and w_in[s] == i and x_in[s] == i):   # full barrier: both tiles of this phase
                yield False
            yield True                                                          # the MMAs read the stage
            if w_in[s] != i or x_in[s] != i:
                raise Violation(f"stage {s} changed under the MMA of k-block {i}")
            armed_for[s] = None                                                 # tcgen05.commit on the empty barrier
            state["consumed"] += 1
            yield True

    def previous_kernel():
        for _ in range(rng.randrange(0, 3 * stages)):
            yield True
        state["dependency"] = True
        yield True

    _run([weights(), activations(), mma(), previous_kernel()], rng)
    assert state["consumed"] == kblocks


@pytest.mark.parametrize("stages,kblocks", [(1, 5), (3, 7), (6, 6), (13, 40)])
def test_decode_gemm_two_producer_ring_is_safe_under_random_schedules(stages, kblocks):
    for seed in range(300):
        _two_producer_ring_model(stages, kblocks, random.Random(seed))


def test_decode_gemm_ring_publishing_before_arming_is_caught():
    with pytest.raises(Violation):
        for seed in range(300):
            _two_producer_ring_model(2, 12, random.Random(seed), publish_after_arming=False)


# ---------------------------------------------------------------------------------------------- per-CTA call counters
def test_per_cta_call_counters_stay_equal_for_any_sequence_of_grid_sizes():
    """The packet all-reduce (`csrc/kernels/allreduce_ll.cu`) keeps one copy of its call counter per CTA: CTA b reads
    copy b on entry, uses `copy + 1` as the packet flag and stores it back when it leaves; CTA 0 also advances the copies
    of the CTAs that the launch does not have. Every rank must derive the same flag for the same call whatever the grid
    sizes of the calls so far, i.e. all copies must be equal after every launch."""
    rng = random.Random(7)
    max_ctas = 256
    copies = [0] * max_ctas
    for call in range(1, 400):
        grid = rng.choice([1, 2, 8, 8, 8, 37, 148, 256])
        order = list(range(grid))
        rng.shuffle(order)                      # CTAs enter and leave in any order
        flags = {b: copies[b] + 1 for b in order}
        assert set(flags.values()) == {call}    # every CTA of the launch uses the same flag, and it is the call's number
        for b in order:
            copies[b] = flags[b]
            if b == 0:
                for j in range(grid, max_ctas):
                    copies[j] = flags[0]
        assert copies == [call] * max_ctas
