"""Model check of the persistent attention kernel's synchronisation (csrc/flash_prefill_sm100.cu).

The kernel's roles (TMA producer, MMA issuer, eight softmax warps) talk through mbarriers whose
waits name a phase PARITY, through an in-order tensor pipe whose commits arrive asynchronously, and
through buffers that are reused across key tiles and work items (Q buffers, the K / V ring, the
score / probability columns and the output accumulators in tensor memory).  Here the same protocol
runs as Python coroutines under random schedules, with every buffer tracked, and the test fails on

  * a parity wait that the hardware would answer differently from the phase the code means
    (a wait that is two phases late never succeeds; one that is a phase early succeeds at once),
  * a buffer overwritten before its readers are done, or read before it holds what the reader expects,
  * a deadlock (every role blocked, nothing in flight).

It is the substitute for a race detector on this path: the interleavings are those the hardware may
produce (asynchronous copies and MMAs complete at arbitrary later times, roles advance in any order).
"""
import random

import pytest

from tests.test_attention_schedule_cpu import fa_item


class Bar:
    def __init__(self, name, count=1):
        self.name, self.count, self.arrived, self.done = name, count, 0, 0

    def arrive(self):
        self.arrived += 1
        if self.arrived == self.count:
            self.arrived, self.done = 0, self.done + 1

    def ready(self, k):
        """What mbarrier.try_wait.parity answers for the parity of absolute phase k (k = -1: the
        'previous' phase of a fresh barrier, which counts as complete), checked against intent."""
        hw = (self.done & 1) != (k & 1)
        assert self.done <= k + 1, f"{self.name}: waiting for phase {k} but the barrier is at {self.done}: the wait can never succeed"
        if hw:
            assert self.done == k + 1, f"{self.name}: parity says phase {k} is complete, barrier is at {self.done}"
        return hw


class Sim:
    def __init__(self, hd, items, seed, fault=None):
        self.fault = fault                       # a deliberately broken protocol, to test the checker
        self.sep = hd == 64
        self.NQ, self.NR = (2, 8) if hd == 64 else (1, 5)
        self.items = items                       # [(b, head, m0, n0, n1)] of this CTA
        self.rng = random.Random(seed)
        B = Bar
        self.QF = [[B(f"QF{q}{x}") for x in range(2)] for q in range(self.NQ)]
        self.QE = [[B(f"QE{q}{x}") for x in range(2)] for q in range(self.NQ)]
        self.RF = [B(f"RF{s}") for s in range(self.NR)]
        self.RE = [B(f"RE{s}") for s in range(self.NR)]
        self.SF = [B(f"SF{x}") for x in range(2)]
        self.PF = [B(f"PF{x}", 4) for x in range(2)]
        self.OF = [B(f"OF{x}") for x in range(2)]
        self.CF = [B(f"CF{x}", 4) for x in range(2)]
        # buffers
        self.qbuf = [[None] * 2 for _ in range(self.NQ)]          # (item index) or None
        self.ring = [None] * self.NR                               # ring entry number or None
        self.ring_loading = [False] * self.NR
        self.q_loading = [[False] * 2 for _ in range(self.NQ)]
        self.S = [[("free", None)] * 4 for _ in range(2)]          # per stream, per warp slice
        self.P = [[("free", None)] * 4 for _ in range(2)]          # only used when sep
        self.O = [dict(item=None, tiles=0, readers=4) for _ in range(2)]
        self.pipe = []                                             # in-order tensor pipe
        self.copies = []                                           # TMA copies in flight
        self.outputs = set()

    # ---- flat tile sequence of this CTA -------------------------------------------------
    def tiles(self):
        e = 0
        for i, it in enumerate(self.items):
            for j in range(max(it[3], it[4])):
                yield i, j, e
                e += 2

    # ---- roles -------------------------------------------------------------------------
    def producer(self):
        qn, e = [0, 0], 0
        for i, it in enumerate(self.items):
            for x in range(2):
                if it[3 + x] == 0:
                    continue
                qb = qn[x] % self.NQ
                while not self.QE[qb][x].ready(qn[x] // self.NQ - 1):
                    yield
                assert self.qbuf[qb][x] is None and not self.q_loading[qb][x], "Q buffer reloaded while in use"
                self.q_loading[qb][x] = True
                self.copies.append(("q", qb, x, i))
                qn[x] += 1
                yield
            for j in range(max(it[3], it[4])):
                for kv in range(2):
                    slot = e % self.NR
                    while not self.RE[slot].ready(e // self.NR - 1):
                        yield
                    assert self.ring[slot] is None and not self.ring_loading[slot], "ring slot reloaded while in use"
                    self.ring_loading[slot] = True
                    self.copies.append(("r", slot, e))
                    e += 1
                    yield

    def mma(self):
        NQ, NR, sep = self.NQ, self.NR, self.sep
        seq = list(self.tiles())
        if not seq:
            return
        sq, pg = [0, 0], [0, 0]
        k_seen = -1
        ps = 0                                                      # index into seq of the S cursor

        def n(idx, x):
            return self.items[seq[idx][0]][3 + x]

        def issue_s(x, blocking):
            nonlocal k_seen
            i, j, e = seq[ps]
            qb, slot = sq[x] % NQ, e % NR
            need_q = j == 0
            while True:
                q_ok = (not need_q) or self.QF[qb][x].ready(sq[x] // NQ)
                k_ok = k_seen == e or (q_ok and self.RF[slot].ready(e // NR))
                if q_ok and k_ok:
                    break
                if not blocking:
                    return False
                yield
            k_seen = e
            self.pipe.append(("S", x, i, j, qb, slot, e))
            self.pipe.append(("commit", self.SF[x]))
            if j == (max(0, n(ps, x) - 2) if self.fault == "q_released_a_tile_early" else n(ps, x) - 1):
                self.pipe.append(("qfree", qb, x))
                self.pipe.append(("commit", self.QE[qb][x]))
                sq[x] += 1
            return True

        def issue_pv(x, idx):
            i, j, e = seq[idx]
            slot = (e + 1) % NR
            while not self.PF[x].ready(pg[x]):
                yield
            while not self.RF[slot].ready((e + 1) // NR):
                yield
            self.pipe.append(("PV", x, i, j, slot, e + 1))
            self.pipe.append(("commit", self.OF[x]))
            pg[x] += 1

        def run(gen):                                               # drive a sub-generator, keep its result
            result = yield from gen
            return result

        # scores of the very first tile
        yield from run(issue_s(0, True))
        if n(0, 1) > 0:
            yield from run(issue_s(1, True))
        self.pipe.append(("rfree", seq[0][2] % NR))
        self.pipe.append(("commit", self.RE[seq[0][2] % NR]))
        ps = 1
        for pv in range(len(seq)):
            i, j, e = seq[pv]
            act = [j < n(pv, 0), j < n(pv, 1)]
            valid = ps < len(seq)
            todo = [valid and seq[ps][1] < n(ps, 0), valid and seq[ps][1] < n(ps, 1)]
            any_s = todo[0] or todo[1]
            if sep:
                for x in range(2):
                    if todo[x] and act[x]:
                        while self.fault != "no_wait_for_loaded_scores" and not self.CF[x].ready(pg[x]):
                            yield
                        yield from run(issue_s(x, True))
                        todo[x] = False
                    if act[x]:
                        yield from issue_pv(x, pv)
            else:
                if act[0]:
                    yield from issue_pv(0, pv)
                if todo[0]:
                    if (yield from run(issue_s(0, not act[1]))):
                        todo[0] = False
                if act[1]:
                    yield from issue_pv(1, pv)
            self.pipe.append(("rfree", (e + 1) % NR))
            self.pipe.append(("commit", self.RE[(e + 1) % NR]))
            for x in range(2):
                if todo[x]:
                    yield from run(issue_s(x, True))
            if any_s:
                self.pipe.append(("rfree", seq[ps][2] % NR))
                self.pipe.append(("commit", self.RE[seq[ps][2] % NR]))
            if valid:
                ps += 1
            yield

    def softmax(self, x, w):
        g = 0
        for i, it in enumerate(self.items):
            nt = it[3 + x]
            if nt == 0:
                continue
            for j in range(nt):
                while not self.SF[x].ready(g):
                    yield
                assert self.S[x][w] == ("scores", (i, j)), f"stream {x} warp {w}: scores of {(i, j)} expected, found {self.S[x][w]}"
                self.S[x][w] = ("loaded", (i, j)) if not self.sep else ("free", None)
                if self.sep:
                    self.CF[x].arrive()
                yield
                rescale = j > 0 and self.rng.random() < 0.3
                if rescale or (self.sep and j > 0 and self.fault != "p_stored_without_waiting_for_o_mma"):
                    while not self.OF[x].ready(g - 1):
                        yield
                    if rescale:
                        o = self.O[x]
                        assert o["item"] == i and o["tiles"] == j, "rescale of an accumulator that is not at the previous tile"
                buf = self.P if self.sep else self.S
                if self.sep:
                    assert buf[x][w] == ("free", None), f"P of stream {x} overwritten before its O MMA read it"
                buf[x][w] = ("probs", (i, j))
                self.PF[x].arrive()
                g += 1
                yield
            while self.fault != "epilogue_without_waiting_for_o_mma" and not self.OF[x].ready(g - 1):
                yield
            o = self.O[x]
            assert o["item"] == i and o["tiles"] == nt, f"epilogue of item {i} stream {x} found {o}"
            self.outputs.add((i, x, w))
            o["readers"] += 1                                         # this warp's rows have left the accumulator
            yield

    # ---- asynchronous machinery ----------------------------------------------------------
    def step_pipe(self):
        op = self.pipe.pop(0)
        kind = op[0]
        if kind == "commit":
            op[1].arrive()
        elif kind == "S":
            _, x, i, j, qb, slot, e = op
            assert self.qbuf[qb][x] == i, f"S MMA of item {i} read Q buffer holding {self.qbuf[qb][x]}"
            assert self.ring[slot] == e, f"S MMA read ring slot {slot} holding {self.ring[slot]}, wanted {e}"
            for w in range(4):
                if self.sep:
                    assert self.S[x][w] == ("free", None), f"scores of stream {x} overwritten before they were loaded"
                else:
                    assert self.S[x][w][0] == "free", f"scores of stream {x} overwritten while {self.S[x][w]}"
                self.S[x][w] = ("scores", (i, j))
        elif kind == "PV":
            _, x, i, j, slot, e = op
            assert self.ring[slot] == e, f"O MMA read ring slot {slot} holding {self.ring[slot]}, wanted {e}"
            buf = self.P if self.sep else self.S
            for w in range(4):
                assert buf[x][w] == ("probs", (i, j)), f"O MMA of {(i, j)} read {buf[x][w]}"
                buf[x][w] = ("free", None)
            o = self.O[x]
            if j == 0:
                assert o["readers"] == 4, "accumulator overwritten before the previous item's epilogue read it"
                o.update(item=i, tiles=1, readers=0)
            else:
                assert o["item"] == i and o["tiles"] == j
                o["tiles"] += 1
        elif kind == "qfree":
            self.qbuf[op[1]][op[2]] = None
        elif kind == "rfree":
            self.ring[op[1]] = None

    def step_copy(self):
        c = self.copies.pop(self.rng.randrange(len(self.copies)))
        if c[0] == "q":
            _, qb, x, i = c
            self.qbuf[qb][x], self.q_loading[qb][x] = i, False
            self.QF[qb][x].arrive()
        else:
            _, slot, e = c
            self.ring[slot], self.ring_loading[slot] = e, False
            self.RF[slot].arrive()

    def run(self, max_steps=2_000_000):
        roles = [self.producer(), self.mma()] + [self.softmax(x, w) for x in range(2) for w in range(4)]
        alive = list(range(len(roles)))
        idle = 0
        for _ in range(max_steps):
            if not alive and not self.pipe and not self.copies:
                return
            choices = list(alive) + (["pipe"] if self.pipe else []) + (["copy"] if self.copies else [])
            before = self.snapshot()
            c = self.rng.choice(choices)
            if c == "pipe":
                self.step_pipe()
            elif c == "copy":
                self.step_copy()
            else:
                try:
                    next(roles[c])
                except StopIteration:
                    alive.remove(c)
            idle = idle + 1 if self.snapshot() == before and c not in ("pipe", "copy") else 0
            assert idle < 20000 or self.pipe or self.copies, "deadlock: every role is waiting and nothing is in flight"
        raise AssertionError("did not finish")

    def snapshot(self):
        bars = [b.done * 8 + b.arrived for grp in (self.RF, self.RE, self.SF, self.PF, self.OF, self.CF) for b in grp]
        bars += [b.done for row in self.QF + self.QE for b in row]
        return (tuple(bars), len(self.pipe), len(self.copies), len(self.outputs))


def cta_items(c, G, S, kv_len, n_q, batch, causal):
    n_items = ((S + 255) // 256) * n_q * batch
    out = []
    for r in range((n_items + G - 1) // G):
        it = fa_item(r, c, G, S, kv_len, 0, n_q, batch, causal)
        if it is not None:
            out.append(it)
    return out


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("S,n_q,batch,causal,G", [
    (512, 3, 2, False, 2),      # two full query blocks per head, several items per CTA
    (300, 4, 1, False, 3),      # second block has no rows for its second stream
    (700, 2, 1, True, 2),       # causal: stream B has one key tile more than stream A
    (1100, 3, 1, True, 4),      # causal, odd number of query tiles, snake deal
    (100, 5, 1, True, 2),       # single-stream items only
])
def test_protocol_under_random_schedules(hd, S, n_q, batch, causal, G):
    n_items = ((S + 255) // 256) * n_q * batch
    G = min(G, n_items)
    for c in range(G):
        items = cta_items(c, G, S, S, n_q, batch, causal)
        for seed in range(6):
            sim = Sim(hd, items, seed * 131 + c)
            sim.run()
            want = {(i, x, w) for i, it in enumerate(items) for x in range(2) if it[3 + x] > 0 for w in range(4)}
            assert sim.outputs == want


def test_protocol_on_random_problems():
    """Random shapes (ragged sequence lengths, longer key ranges than queries, one to five CTAs),
    one random CTA and one random schedule each."""
    rng = random.Random(7)
    for _ in range(60):
        hd = rng.choice([64, 128])
        S = rng.choice([1, 64, 128, 129, 200, 256, 257, 300, 511, 512, 700, 900, 1100, 1300])
        n_q, batch, causal = rng.randint(1, 5), rng.randint(1, 3), rng.random() < 0.5
        kv_len = S if causal else rng.choice([S, S + 77, 3 * S + 5])
        n_items = ((S + 255) // 256) * n_q * batch
        G = min(rng.randint(1, 5), n_items)
        items = cta_items(rng.randrange(G), G, S, kv_len, n_q, batch, causal)
        Sim(hd, items, rng.randrange(1 << 30)).run()


@pytest.mark.parametrize("hd,fault", [(64, "no_wait_for_loaded_scores"), (64, "p_stored_without_waiting_for_o_mma"),
                                      (128, "q_released_a_tile_early"), (128, "epilogue_without_waiting_for_o_mma"),
                                      (64, "epilogue_without_waiting_for_o_mma")])
def test_the_model_catches_broken_protocols(hd, fault):
    """The checker is only worth something if it fails on a protocol that is wrong: each of these
    drops one wait (or releases one buffer early) and must be reported under some schedule."""
    items = cta_items(0, 2, 700, 700, 2, 1, True)
    caught = 0
    for seed in range(12):
        try:
            Sim(hd, items, seed, fault=fault).run()
        except AssertionError:
            caught += 1
    assert caught > 0


def test_the_model_catches_a_late_wait():
    """The checker itself: a wait that is two phases behind is reported, not silently passed."""
    b = Bar("x")
    b.arrive(); b.arrive()
    with pytest.raises(AssertionError):
        b.ready(0)
