"""CPU model of the barrier protocol of the integer tensor-core kernel (minit_b200/csrc/qgemm_mid.cu): every role is a
generator, every mbarrier a pending count with a phase, the scheduler is random.  It fails on a deadlock, on an arrival
that lands in another k-block's phase, and on over-arrival.  The ring lengths below are the kernel's (MdCfg); the last
case is a configuration that must FAIL: eight producer lanes over six activation stages make a lane skip phases of a
barrier, its parity wait then passes one phase early (this is the fault the model was written to find; the kernel now
has one issuing thread per ring, which cannot skip a phase)."""
import random

import pytest

class Bar:
    def __init__(self, name, count):
        self.name, self.count, self.pending, self.phase = name, count, count, 0
        self.arrivals_this_phase = []

    def arrive(self, who, n=1):
        self.pending -= n
        self.arrivals_this_phase.append(who)
        if self.pending < 0:
            raise RuntimeError(f"{self.name}: over-arrival by {who}; arrivals {self.arrivals_this_phase}")
        if self.pending == 0:
            self.phase += 1
            self.pending = self.count
            self.arrivals_this_phase = []

    def done(self, parity):            # test_wait.parity(P): true when the phase with parity P has completed
        return (self.phase & 1) != parity


def run(nrun, AST, BST, PST, NT, FOLD, seed, planes=1, blanes=1, cgroups=2, DBUF=2, SZST=3):
    """planes / blanes: threads that issue the packed-weight copies / the activation-stage copies, each taking every
    planes-th (blanes-th) k-block.  The kernel uses one of each, walking its ring in order; the thread of the activation
    stages also loads the blocks of scales and zero words (ring of SZST, a new block every few k-blocks and at every
    column tile, so a block can be a single k-block long)."""
    rnd = random.Random(seed)
    block = []                                   # scale / zero block of every k-block: random lengths 1 .. 10
    while len(block) < nrun:
        block += [(block[-1] + 1) if block else 0] * rnd.randint(1, 10)
    block = block[:nrun]
    szfull = [Bar(f"szfull{s}", 1) for s in range(SZST)]
    szempty = [Bar(f"szempty{s}", FOLD) for s in range(SZST)]
    pfull = [Bar(f"pfull{s}", 1) for s in range(PST)]
    pempty = [Bar(f"pempty{s}", 4) for s in range(PST)]
    full = [Bar(f"full{s}", 4 + 1 + FOLD) for s in range(BST)]
    done = [Bar(f"done{s}", NT) for s in range(BST)]
    bempty = [Bar(f"bempty{s}", FOLD) for s in range(BST)]
    for s in range(DBUF):
        full[s].arrive("init", FOLD)
    log = []
    # expected unit of every arrival, to check aliasing: full[s] phase p must only get arrivals of unit s + p*BST
    def check(barlist, idx, ring, unit, who):
        b = barlist[idx]
        exp = idx + b.phase * ring
        if exp != unit:
            raise RuntimeError(f"{b.name}: {who} arrives for unit {unit} but the barrier is in the phase of unit {exp}")

    def p_lane(l):
        for i in range(l, nrun, planes):
            ps = i % PST
            if i >= PST:
                while not pempty[ps].done(((i // PST) & 1) ^ 1):
                    yield
            check(pfull, ps, PST, i, f"P{l}")
            pfull[ps].arrive(f"P{l}:{i}")
            yield

    def b_lane(l):
        for i in range(l, nrun, blanes):
            bs = i % BST
            if blanes == 1 and (i == 0 or block[i] != block[i - 1]):
                n = block[i]
                if n >= SZST:
                    while not szempty[n % SZST].done(((n // SZST) & 1) ^ 1):
                        yield
                szfull[n % SZST].arrive(f"B{l}:block{n}")
                yield
            if i >= BST:
                while not bempty[bs].done(((i // BST) & 1) ^ 1):
                    yield
            check(full, bs, BST, i, f"B{l}")
            full[bs].arrive(f"B{l}:{i}")
            yield

    def conv(g, w):
        for i in range(g, nrun, cgroups):
            ps, bs = i % PST, i % BST
            while not pfull[ps].done((i // PST) & 1):
                yield
            yield
            check(pempty, ps, PST, i, f"C{g}{w}")
            pempty[ps].arrive(f"C{g}{w}:{i}")
            if i >= AST:
                u = i - AST
                while not done[u % BST].done((u // BST) & 1):
                    yield
            yield
            check(full, bs, BST, i, f"C{g}{w}")
            full[bs].arrive(f"C{g}{w}:{i}")
            yield

    def mma(nt):
        for i in range(nrun):
            bs = i % BST
            while not full[bs].done((i // BST) & 1):
                yield
            yield
            check(done, bs, BST, i, f"M{nt}")
            done[bs].arrive(f"M{nt}:{i}")
            yield

    def fold(w):
        cur = -1
        for j in range(nrun):
            bs = j % BST
            while not done[bs].done((j // BST) & 1):
                yield
            yield
            if blanes == 1 and block[j] != cur:
                if cur >= 0:
                    szempty[cur % SZST].arrive(f"F{w}:block{cur}")
                cur = block[j]
                while not szfull[cur % SZST].done((cur // SZST) & 1):
                    yield
                yield
            t = (j + DBUF) % BST
            check(full, t, BST, j + DBUF, f"F{w}")
            full[t].arrive(f"F{w}:{j}")
            yield
            check(bempty, bs, BST, j, f"F{w}")
            bempty[bs].arrive(f"F{w}:{j}")
            yield

    procs = [p_lane(l) for l in range(planes)] + [b_lane(l) for l in range(blanes)] + \
            [conv(g, w) for g in range(cgroups) for w in range(4)] + [mma(nt) for nt in range(NT)] + [fold(w) for w in range(FOLD)]
    alive = list(range(len(procs)))
    idle = 0
    while alive:
        k = rnd.choice(alive)
        before = (tuple(b.phase for b in pfull + pempty + full + done + bempty + szfull + szempty), tuple(b.pending for b in pfull + pempty + full + done + bempty + szfull + szempty))
        try:
            next(procs[k])
        except StopIteration:
            alive.remove(k)
            idle = 0
            continue
        after = (tuple(b.phase for b in pfull + pempty + full + done + bempty + szfull + szempty), tuple(b.pending for b in pfull + pempty + full + done + bempty + szfull + szempty))
        idle = idle + 1 if before == after else 0
        if idle > 20000:
            raise RuntimeError(f"deadlock: alive {alive}")
    return True



CONFIGS = {
    "int4 rows<=16": dict(AST=4, BST=8, PST=8, NT=2, DBUF=4), "int4 rows<=32": dict(AST=4, BST=8, PST=8, NT=2),
    "int4 rows<=64": dict(AST=4, BST=6, PST=12, NT=1), "int8 rows<=16": dict(AST=4, BST=8, PST=4, NT=2, DBUF=4), "int8 rows<=32": dict(AST=4, BST=8, PST=4, NT=2),
    "int8 rows<=64": dict(AST=4, BST=6, PST=4, NT=1),
}


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_protocol_has_no_deadlock_and_no_phase_aliasing(name):
    for nrun in (1, 2, 3, 5, 7, 13, 24, 40):
        for seed in range(8):
            assert run(nrun, FOLD=8, seed=seed, **CONFIGS[name])


def test_model_catches_a_lane_that_skips_phases():
    with pytest.raises(RuntimeError, match="arrives for unit"):
        for seed in range(8):
            run(24, AST=4, BST=6, PST=12, NT=1, FOLD=8, seed=seed, planes=4, blanes=8)
