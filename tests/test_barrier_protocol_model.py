"""Randomised interleaving model of the weight-gradient kernel's barrier protocol (CPU only).

The single-CTA ragged reduction of ``csrc/gemm_sm100.cuh`` runs five kinds of warps against one
ring of shared-memory slots: the TMA producer, two MMA-issuing warps that alternate tiles, the
tail warp that clears rows past a group's end, and the epilogue.  This model restates their
loops (ring counters, which warp arrives on which barrier, when a resident B operand is
released) with mbarriers of the hardware's parity semantics -- ``try_wait(P)`` is true iff the
barrier's current phase parity differs from P, so a waiter that falls two phases behind cannot
tell -- and a tensor pipe in which a commit only covers the MMAs of the warp that issued it.
Random schedules then check that nothing deadlocks, that no barrier gets more arrivals than it
expects, that every MMA reads exactly the blocks it was meant to read (slots are invalidated
when a load is issued and tagged when it lands), and that accumulators reach the epilogue in
tile order.  It covers both tile walks and both ring geometries (4 + 4 slots; 6 A + 3 B slots).
"""
import random

GEOM = {True: (6, 3), False: (4, 4)}   # unit walk: (A slots, B slots)


class Bar:
    def __init__(self, count):
        self.count = count
        self.pending = count
        self.phase = 0

    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0, "too many arrivals"
        if self.pending == 0:
            self.phase += 1
            self.pending = self.count

    def ready(self, parity):
        return (self.phase & 1) != parity


def tiles_of(units, m_tiles, unit_mode):
    """Walk of one CTA: list of (unit, m, num_kb, tail)"""
    out = []
    for u, (nkb, tail) in enumerate(units):
        for m in range(m_tiles):
            out.append((u, m, nkb, tail))
    return out


def run(seed, unit_mode, dual=True, bempty_count=None):
    rnd = random.Random(seed)
    m_tiles = rnd.choice([1, 2, 3, 4, 5])
    units = [(rnd.choice([0, 1, 2, 3, 4, 5, 7]), rnd.random() < 0.7) for _ in range(rnd.randint(1, 6))]
    walk = tiles_of(units, m_tiles, unit_mode)
    NA, NB = GEOM[unit_mode]
    full = [Bar(1) for _ in range(NA)]
    empty = [Bar(3 if dual else 2) for _ in range(NA)]
    bempty = [Bar(bempty_count or (2 if dual else 1)) for _ in range(NB)]
    fixed = [Bar(1) for _ in range(NA)]
    tfull = [Bar(1), Bar(1)]
    tempty = [Bar(4), Bar(4)]
    slotA = [None] * NA       # tag of the block in the A half
    slotB = [None] * NB
    inflight = []             # loads: [remaining, fn]
    pipe = []                 # tensor pipe FIFO: entries ("mma", issuer, check_fn) / ("commit", issuer, bar)
    log = {"acc_done": []}

    def resident(nkb):
        return unit_mode and nkb <= NB

    # ---------------- producer
    def producer():
        stage = phase = bstage = bphase = 0
        for (u, m, nkb, tail) in walk:
            res = resident(nkb)
            load_b = (not res) or m == 0
            for kb in range(nkb):
                while not empty[stage].ready(phase ^ 1):
                    yield
                if load_b:
                    while not bempty[bstage].ready(bphase ^ 1):
                        yield
                slotA[stage] = ("loading",)
                a_tag = ("A", u, m, kb)
                b_tag = ("B", u, kb)
                bs = bstage
                if load_b:
                    slotB[bs] = ("loading",)

                def land(stage=stage, a_tag=a_tag, bs=bs, b_tag=b_tag, load_b=load_b):
                    slotA[stage] = a_tag
                    if load_b:
                        slotB[bs] = b_tag
                    full[stage].arrive()
                inflight.append([rnd.randint(1, 12), land])
                if load_b:
                    bstage += 1
                    if bstage == NB:
                        bstage = 0
                        bphase ^= 1
                stage += 1
                if stage == NA:
                    stage = 0
                    phase ^= 1
                yield

    # ---------------- issuers
    def issuer_fn(issuer):
        seq = 0
        stage = phase = 0
        acc = issuer if dual else 0
        acc_phase = 0
        fixed_phase = 0
        bstage = unit_b0 = 0
        for (u, m, nkb, tail) in walk:
            res = resident(nkb)
            mine = (not dual) or (seq & 1) == issuer
            release_b = (not res) or m == m_tiles - 1
            pass_b = False
            if dual:
                if mine:
                    release_b = (not res) or m + 2 > m_tiles - 1
                else:
                    release_b = False
                    pass_b = (not res) or m_tiles == 1
            if res and m == 0:
                unit_b0 = bstage
            if mine:
                while not tempty[acc].ready(acc_phase ^ 1):
                    yield
            for kb in range(nkb):
                is_tail = tail and kb == nkb - 1
                bslot = (unit_b0 + kb) % NB if res else bstage
                while not full[stage].ready(phase):
                    yield
                if is_tail:
                    while not fixed[stage].ready((fixed_phase >> stage) & 1):
                        yield
                    fixed_phase ^= 1 << stage
                if not mine:
                    empty[stage].arrive()
                    if pass_b:
                        bempty[bslot].arrive()
                else:
                    expectA, expectB = ("A", u, m, kb), ("B", u, kb)

                    def check(stage=stage, bslot=bslot, expectA=expectA, expectB=expectB, tailz=is_tail):
                        assert slotA[stage] == expectA, (slotA[stage], expectA)
                        assert slotB[bslot] == expectB, (slotB[bslot], expectB)
                    pipe.append(("mma", issuer, check))
                    pipe.append(("commit", issuer, empty[stage]))
                    if release_b:
                        pipe.append(("commit", issuer, bempty[bslot]))
                if not res:
                    bstage = (bstage + 1) % NB
                stage += 1
                if stage == NA:
                    stage = 0
                    phase ^= 1
                yield
            if res and m == m_tiles - 1:
                bstage = (unit_b0 + nkb) % NB
            if mine:
                pipe.append(("commit", issuer, tfull[acc]))
            seq += 1
            if dual:
                if mine:
                    acc_phase ^= 1
            else:
                acc ^= 1
                if acc == 0:
                    acc_phase ^= 1
            yield

    # ---------------- tail warp
    def tail_fn():
        stage = phase = 0
        for (u, m, nkb, tail) in walk:
            for kb in range(nkb):
                while not full[stage].ready(phase):
                    yield
                if tail and kb == nkb - 1:
                    fixed[stage].arrive()
                empty[stage].arrive()
                stage += 1
                if stage == NA:
                    stage = 0
                    phase ^= 1
                yield

    # ---------------- epilogue (4 warps modelled as one agent arriving 4 times)
    def epi_fn():
        acc = acc_phase = 0
        for i, _ in enumerate(walk):
            while not tfull[acc].ready(acc_phase):
                yield
            log["acc_done"].append(i)
            for _ in range(rnd.randint(0, 3)):
                yield
            for _ in range(4):
                tempty[acc].arrive()
            acc ^= 1
            if acc == 0:
                acc_phase ^= 1
            yield

    agents = {"prod": producer(), "i0": issuer_fn(0), "tail": tail_fn(), "epi": epi_fn()}
    if dual:
        agents["i1"] = issuer_fn(1)
    idle = 0
    while agents:
        progressed = False
        # hardware progress: loads and the tensor pipe
        for ld in list(inflight):
            ld[0] -= 1
            if ld[0] <= 0:
                ld[1]()
                inflight.remove(ld)
                progressed = True
        # a commit tracks only the MMAs of the thread that issued it: fire every commit that
        # has no earlier MMA of the same issuer in front of it, even past the other issuer's
        fired = True
        while fired:
            fired = False
            seen_mma = set()
            for idx, (kind, who, x) in enumerate(pipe):
                if kind == "mma":
                    seen_mma.add(who)
                elif who not in seen_mma:
                    x.arrive()
                    del pipe[idx]
                    fired = progressed = True
                    break
        if pipe and rnd.random() < 0.6:
            # MMAs execute in issue order
            for idx, (kind, who, x) in enumerate(pipe):
                if kind == "mma":
                    x()
                    del pipe[idx]
                    progressed = True
                    break
        name = rnd.choice(list(agents))
        before = (tuple(b.phase for b in full + empty + bempty + fixed + tfull + tempty), len(pipe),
                  len(inflight))
        try:
            next(agents[name])
        except StopIteration:
            del agents[name]
            progressed = True
        after = (tuple(b.phase for b in full + empty + bempty + fixed + tfull + tempty), len(pipe),
                 len(inflight))
        if before != after:
            progressed = True
        idle = 0 if progressed or pipe or inflight else idle + 1
        assert idle < 5000, f"deadlock: remaining {list(agents)} seed {seed} unit_mode {unit_mode} " \
                             f"m_tiles {m_tiles} units {units}"
    while pipe:
        kind, who, x = pipe.pop(0)
        x() if kind == "mma" else x.arrive()   # drain (order no longer matters)
    assert log["acc_done"] == list(range(len(walk)))


def test_protocol_has_no_deadlock_or_stale_read():
    for seed in range(40):
        for unit_mode in (True, False):
            run(seed, unit_mode, dual=True)


def test_model_detects_a_missing_arrival():
    """The model must be able to fail: with the B-consumed barrier expecting one arrival although
    two issuing warps report on it, the phases drift and the run ends in an assertion."""
    import pytest
    with pytest.raises(AssertionError):
        for seed in range(20):
            run(seed, True, dual=True, bempty_count=1)
