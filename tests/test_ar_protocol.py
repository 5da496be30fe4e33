"""CPU model of the mailbox all-reduce of minit_b200/csrc/ar_mailbox.cuh, one-shot and two-shot, under a random scheduler.

Every rank has a buffer of mailboxes [call parity][sender rank][cell]; a cell is (value, epoch) written by ONE store, so a
reader that sees the call's epoch sees the value.  A rank's calls run one after the other (kernel boundaries); inside a
call every thread owns one column: it pushes, then collects, as the integer mid-batch kernel's epilogue does
(ar_push1 / ar_pull_rows, and ar_push_to / ar_read_from for the two-shot form).  Checked:

* every rank ends every call with the sum over ranks added in rank order -- the same bits on all ranks;
* no store lands on a cell whose previous content its owner has not consumed yet (the header's claim that two
  parities suffice because a peer can be at most one call ahead), also when one-shot and two-shot calls alternate and
  when some ranks own no column;
* nobody waits forever.

The last case is a configuration that must FAIL: with a single parity a peer that is one call ahead overwrites cells
that have not been read."""
import random

import pytest


class Overwrite(RuntimeError):
    pass


class Rank:
    def __init__(self, rank, world, parities, cells):
        self.rank, self.world = rank, world
        self.box = [[[(0.0, 0)] * cells for _ in range(world)] for _ in range(parities)]   # [parity][sender][cell] = (value, epoch)
        self.read_upto = [[[0] * cells for _ in range(world)] for _ in range(parities)]    # epoch of the last value consumed from the cell
        self.finished = 0                                                                  # control word 0: epoch of the last finished call
        self.out = {}                                                                      # (epoch, row, col) -> result


def store(ranks, dst, parities, sender, cell, value, epoch):
    p = epoch % parities
    old_value, old_epoch = ranks[dst].box[p][sender][cell]
    if old_epoch and ranks[dst].read_upto[p][sender][cell] < old_epoch:
        raise Overwrite(f"rank {sender} overwrites cell {cell} of call {old_epoch} in rank {dst}'s buffer at call {epoch} before it was read")
    ranks[dst].box[p][sender][cell] = (value, epoch)


def poll(rank, parities, sender, cell, epoch):
    p = epoch % parities
    value, got = rank.box[p][sender][cell]
    if got != epoch:
        return None
    rank.read_upto[p][sender][cell] = epoch
    return value


def owner_of(col, n, world):
    per = max(1, (n + world - 1) // world)
    return min(col // per, world - 1)


def column_thread(ranks, me, parities, epoch, col, m, n, partial, two_shot):
    """one thread of the epilogue: all rows of a column"""
    world = me.world
    cells = [row * n + col for row in range(m)]
    mine = [partial(me.rank, epoch, row, col) for row in range(m)]
    own = owner_of(col, n, world) if two_shot else None
    if two_shot and own != me.rank:
        for cell, v in zip(cells, mine):
            store(ranks, own, parities, me.rank, cell, v, epoch)
            yield
        for row, cell in enumerate(cells):                      # the owner's sum
            while (v := poll(me, parities, own, cell, epoch)) is None:
                yield
            me.out[(epoch, row, col)] = v
        return
    if not two_shot:
        for cell, v in zip(cells, mine):
            for r in range(world):
                if r != me.rank:
                    store(ranks, r, parities, me.rank, cell, v, epoch)
                    yield
    sums = []
    for row, cell in enumerate(cells):                          # collect: rank order, own value in its place
        total = 0.0
        for r in range(world):
            if r == me.rank:
                total += mine[row]
                continue
            while (v := poll(me, parities, r, cell, epoch)) is None:
                yield
            total += v
        sums.append(total)
    if two_shot:
        for cell, v in zip(cells, sums):
            for r in range(world):
                if r != me.rank:
                    store(ranks, r, parities, me.rank, cell, v, epoch)
                    yield
    for row, v in enumerate(sums):
        me.out[(epoch, row, col)] = v


def rank_program(ranks, me, parities, calls, m, n, partial, mode, rnd):
    for _ in range(calls):
        epoch = me.finished + 1
        two_shot = mode == "two" or (mode == "alternate" and epoch % 2 == 0)
        threads = [column_thread(ranks, me, parities, epoch, col, m, n, partial, two_shot) for col in range(n)]
        while threads:
            t = rnd.choice(threads)
            try:
                next(t)
            except StopIteration:
                threads.remove(t)
            yield
        me.finished = epoch                                     # the last CTA to leave publishes the epoch


def run(world, calls, m, n, mode, seed, parities=2):
    rnd = random.Random(seed)
    values = {}

    def partial(rank, epoch, row, col):
        return values.setdefault((rank, epoch, row, col), rnd.uniform(-1, 1))

    ranks = [Rank(r, world, parities, m * n) for r in range(world)]
    programs = {r: rank_program(ranks, ranks[r], parities, calls, m, n, partial, mode, rnd) for r in range(world)}
    weights = [rnd.choice((1, 1, 5)) for _ in range(world)]      # some ranks run faster than others
    idle = 0
    while programs:
        r = rnd.choices(list(programs), [weights[k] for k in programs])[0]
        before = sum(rk.finished for rk in ranks) + sum(len(rk.out) for rk in ranks)
        try:
            next(programs[r])
        except StopIteration:
            del programs[r]
        after = sum(rk.finished for rk in ranks) + sum(len(rk.out) for rk in ranks)
        idle = idle + 1 if before == after else 0
        if idle > 200000:
            raise RuntimeError(f"no progress: ranks at calls {[rk.finished for rk in ranks]}")
    for epoch in range(1, calls + 1):
        for row in range(m):
            for col in range(n):
                expect = 0.0
                for r in range(world):
                    expect += values[(r, epoch, row, col)]
                for rk in ranks:
                    assert rk.out[(epoch, row, col)] == expect, f"rank {rk.rank} call {epoch} ({row},{col})"


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("mode", ["one", "two", "alternate"])
def test_mailbox_all_reduce(world, mode):
    for seed in range(6):
        run(world, calls=5, m=3, n=8, mode=mode, seed=seed)


def test_fewer_columns_than_ranks():
    """two-shot with ranks that own no column: they still depend on every owner in every call"""
    for seed in range(6):
        run(world=8, calls=5, m=2, n=3, mode="two", seed=seed)
        run(world=4, calls=6, m=1, n=2, mode="alternate", seed=seed)


def test_single_parity_is_caught():
    with pytest.raises(Overwrite):
        for seed in range(40):
            run(world=3, calls=4, m=2, n=4, mode="one", seed=seed, parities=1)
