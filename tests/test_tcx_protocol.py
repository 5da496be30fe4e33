"""CPU model of the barrier protocol of the prefill kernel with the dequantized weights in tensor memory
(qgemm_tcx_kernel, minit_b200/csrc/qgemm_tc.cu): every role is a generator, every mbarrier a pending count with a phase,
asynchronous completions (TMA bytes, tcgen05.commit) arrive after random delays, the scheduler is random.

Roles as in the kernel: two producer threads (x tiles | packed words), two MMA-issuing threads (one per 128-column half;
commits complete in issue order), two groups of eight converter warps on alternate k-blocks (each group writes slot
``it % NSLOT`` of the A operand), eight epilogue warps.  Barriers: ``full[s]`` = x arrive + x bytes + 8 converter warps,
``qfull[s]`` = words arrive + bytes, ``empty[s]`` = 2 commits, ``tfull`` = 2 commits, ``tempty`` = 8 epilogue warps.  Waits
are by phase parity computed from the k-block counter, and three of them are EARLY looks (a test issued one turn ahead
whose answer replaces the wait), exactly as in the kernel.

The model fails on: no progress; over-arrival; an arrival that lands in another k-block's phase; a parity test that says
yes for a phase that has not completed; a stage buffer, an A slot or the accumulators overwritten before their readers
are done; MMAs issued on a slot or a stage that holds another k-block.  Configurations: the kernel's (STAGES, NSLOT)
pairs -- (6, 2) for 192-row tiles, (6, 3) for 160, (12, 4) for 64 -- over items of random length (whole tiles and the
parts of tiles cut along K).  The last case must FAIL: converters that skip the wait for their A slot, and MMAs that
skip the wait for the epilogue, are reported as the overwrites they cause."""
import random

import pytest


class Hazard(RuntimeError):
    pass


class Bar:
    def __init__(self, name, count, ring=None):
        self.name, self.count, self.pending, self.phase, self.ring = name, count, count, 0, ring

    def arrive(self, who, unit=None, index=None):
        if unit is not None and self.ring is not None:
            expect = index + self.phase * self.ring
            if expect != unit:
                raise Hazard(f"{self.name}: {who} arrives for k-block {unit}, the barrier is in the phase of k-block {expect}")
        self.pending -= 1
        if self.pending < 0:
            raise Hazard(f"{self.name}: over-arrival by {who}")
        if self.pending == 0:
            self.phase += 1
            self.pending = self.count

    def test(self, parity):                     # mbarrier.test_wait.parity
        return (self.phase & 1) != parity


def run(STAGES, NSLOT, items, seed, conv_warps=8, epi_warps=8, slot_wait=True, acc_wait=True):
    rnd = random.Random(seed)
    full = [Bar(f"full{s}", 2 + conv_warps, STAGES) for s in range(STAGES)]
    qfull = [Bar(f"qfull{s}", 2, STAGES) for s in range(STAGES)]
    empty = [Bar(f"empty{s}", 2, STAGES) for s in range(STAGES)]
    tfull, tempty = Bar("tfull", 2), Bar("tempty", epi_warps)
    total = sum(items)
    first = [sum(items[:i]) for i in range(len(items))]           # global index of each item's first k-block

    # what the buffers hold and who is done with them
    b_stage = [None] * STAGES                                     # k-block whose x tile is in stage s
    q_stage = [None] * STAGES                                     # ... whose packed words
    slot = [None] * NSLOT                                         # k-block whose weights are in A slot
    slot_writers = [0] * NSLOT
    q_readers = [0] * total                                       # converter warps that have read the words of a k-block
    mma_done = [0] * total                                        # issuing threads whose MMAs of a k-block have completed
    epi_done = [0] * len(items)                                   # epilogue warps done with an item's accumulators
    acc_item = [None, None]                                       # item whose sums each 128-column half holds
    pending = []                                                  # asynchronous completions in flight (generators)

    def phase_done(bar_list, unit):
        s = unit % STAGES
        return bar_list[s].phase > unit // STAGES

    def wait(bar, parity):
        while not bar.test(parity):
            yield

    def delayed(fn):
        def g():
            for _ in range(rnd.randint(0, 6)):
                yield
            fn()
        pending.append(g())

    def producer(words):
        for it in range(total):
            s, ph = it % STAGES, (it // STAGES) & 1
            yield from wait(empty[s], ph ^ 1)
            if it >= STAGES:                                      # the previous content must be dead
                old = it - STAGES
                if mma_done[old] < 2:
                    raise Hazard(f"{'words' if words else 'x'} of k-block {it} loaded into stage {s} before the MMAs of k-block {old} completed")
                if words and q_readers[old] < conv_warps:
                    raise Hazard(f"words of k-block {it} loaded over words of k-block {old} that {conv_warps - q_readers[old]} converter warps still read")
            bars = qfull if words else full
            bars[s].arrive("producer", it, s)

            def landed(it=it, s=s, bars=bars):
                (q_stage if words else b_stage)[s] = it
                bars[s].arrive("tma bytes", it, s)
            delayed(landed)
            yield

    def issuer(nt):
        queue = []                                                # commits of this thread, completing in order

        def complete():
            while queue:
                for _ in range(rnd.randint(0, 5)):
                    yield
                queue.pop(0)()
        runner = [None]

        def commit(fn):
            queue.append(fn)
            if runner[0] is None or runner[0] not in pending:
                runner[0] = complete()
                pending.append(runner[0])

        it, early = 0, False
        for lt, length in enumerate(items):
            if acc_wait:
                yield from wait(tempty, (lt & 1) ^ 1)
            if lt > 0 and epi_done[lt - 1] < epi_warps:
                raise Hazard(f"MMAs of item {lt} start while {epi_warps - epi_done[lt - 1]} epilogue warps still read item {lt - 1}")
            for k in range(length):
                s, ph, a = it % STAGES, (it // STAGES) & 1, it % NSLOT
                if early:
                    if not phase_done(full, it):
                        raise Hazard(f"early look at full[{s}] said yes for k-block {it} before its phase completed")
                else:
                    yield from wait(full[s], ph)
                nit = it + 1
                early = full[nit % STAGES].test((nit // STAGES) & 1)
                if slot[a] != it or slot_writers[a] < conv_warps:
                    raise Hazard(f"MMAs of k-block {it} read A slot {a}, which holds k-block {slot[a]} from {slot_writers[a]} warps")
                if b_stage[s] != it:
                    raise Hazard(f"MMAs of k-block {it} read stage {s}, which holds the x tile of k-block {b_stage[s]}")
                acc_item[nt] = lt

                def done(it=it, s=s):
                    mma_done[it] += 1
                    empty[s].arrive(f"commit {nt}", it, s)
                commit(done)
                it += 1
                yield
            commit(lambda: tfull.arrive(f"commit {nt}"))
            yield

    def converter(grp, w):
        it, q_early = 0, False
        for length in items:
            for k in range(length):
                if (it & 1) != grp:
                    it += 1
                    continue
                s, ph, a = it % STAGES, (it // STAGES) & 1, it % NSLOT
                if q_early:
                    if not phase_done(qfull, it):
                        raise Hazard(f"early look at qfull[{s}] said yes for k-block {it} before its phase completed")
                else:
                    yield from wait(qfull[s], ph)
                prev = it - NSLOT
                a_free = True
                if it >= NSLOT:
                    a_free = empty[prev % STAGES].test((prev // STAGES) & 1)
                    if a_free and mma_done[prev] < 2:
                        raise Hazard(f"early look at empty[{prev % STAGES}] said yes for k-block {prev} before both commits")
                nxt = it + 2
                q_early = qfull[nxt % STAGES].test((nxt // STAGES) & 1)
                if q_stage[s] != it:
                    raise Hazard(f"converter reads stage {s} for k-block {it}, it holds the words of k-block {q_stage[s]}")
                yield                                              # the conversion arithmetic
                q_readers[it] += 1
                if not a_free and slot_wait:
                    yield from wait(empty[prev % STAGES], (prev // STAGES) & 1)
                if it >= NSLOT and mma_done[prev] < 2:
                    raise Hazard(f"A slot {a} rewritten for k-block {it} before the MMAs of k-block {prev} completed")
                if slot[a] != it:
                    slot[a], slot_writers[a] = it, 0
                slot_writers[a] += 1
                yield
                full[s].arrive(f"converter {grp}.{w}", it, s)
                it += 1
                yield

    def epilogue(w):
        for lt in range(len(items)):
            yield from wait(tfull, lt & 1)
            if acc_item != [lt, lt]:
                raise Hazard(f"epilogue of item {lt} reads accumulators of items {acc_item}")
            last = first[lt] + items[lt] - 1
            if mma_done[last] < 2:
                raise Hazard(f"epilogue of item {lt} starts before its last MMAs completed")
            yield
            epi_done[lt] += 1
            tempty.arrive(f"epilogue {w}")
            yield

    procs = [producer(False), producer(True), issuer(0), issuer(1)]
    procs += [converter(g, w) for g in range(2) for w in range(conv_warps)]
    procs += [epilogue(w) for w in range(epi_warps)]
    idle = 0
    while procs:
        pool = procs + pending
        p = rnd.choice(pool)

        def snapshot():
            return (tuple(b.phase for b in full + qfull + empty + [tfull, tempty]), tuple(b.pending for b in full + qfull + empty + [tfull, tempty]),
                    sum(q_readers), sum(slot_writers), len(pending))
        before = snapshot()
        try:
            next(p)
        except StopIteration:
            (procs if p in procs else pending).remove(p)
            idle = 0
            continue
        idle = idle + 1 if snapshot() == before else 0
        if idle > 50000:
            raise Hazard(f"no progress: phases {[b.phase for b in full]} {[b.phase for b in empty]} tfull {tfull.phase} tempty {tempty.phase}")
    assert all(v == 2 for v in mma_done) and all(v == epi_warps for v in epi_done)


CONFIGS = {"192 rows": (6, 2), "160 rows": (6, 3), "64 rows": (12, 4)}


@pytest.mark.parametrize("name", list(CONFIGS))
def test_tcx_protocol(name):
    stages, nslot = CONFIGS[name]
    shapes = [[1], [2], [3, 1], [5, 7, 2], [13, 1, 1, 6], [24, 24], [7] * 5, [1] * 9, [64, 3]]
    for items in shapes:
        for seed in range(8):
            run(stages, nslot, items, seed)


def test_fewer_converter_warps_is_not_special():
    for seed in range(8):
        run(6, 2, [9, 4, 11], seed, conv_warps=3, epi_warps=2)


def test_missing_waits_are_caught():
    """the model sees the hazards the two slowest hand-overs guard against"""
    with pytest.raises(Hazard, match="A slot"):
        for seed in range(40):
            run(6, 2, [17, 9], seed, slot_wait=False)        # converters that do not wait for the MMAs that read their slot
    with pytest.raises(Hazard, match="epilogue warps still read"):
        for seed in range(40):
            run(6, 2, [3, 3, 3], seed, acc_wait=False)       # MMAs that do not wait for the epilogue of the previous item
