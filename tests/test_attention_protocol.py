"""Barrier protocols of the attention kernels, replayed on the CPU.

The kernels of csrc/attention.cu (two query tiles per CTA) and csrc/attention_bwd.cu (P and dS in TMEM) are
warp-specialised: a TMA producer, one thread issuing the matrix products, and softmax / recompute warps hand
buffers to one another through mbarriers that are waited on by phase parity.  This file restates each role's sequence
of waits, arrivals and commits and runs the roles under many random interleavings: no interleaving may dead-lock, a
wait may only pass for the completion it was written for (a barrier running a phase ahead of a waiter would alias on
parity), a ring stage may only be refilled after its release, and a score buffer in TMEM may only be overwritten after
the products that read P / dS from it have been issued.  A product's completion is modelled at its commit (ordering,
not timing); a TMA load completes when it is issued.
"""
import random

import pytest


class Barrier:
    def __init__(self, count):
        self.count, self.pending, self.completions = count, count, 0

    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0, "more arrivals than the barrier was initialised for"
        if self.pending == 0:
            self.pending = self.count
            self.completions += 1

    def passes(self, parity):
        # mbarrier.try_wait.parity P succeeds once the phase of parity P is over
        return (self.completions & 1) != parity


def run(roles, seed):
    """Round-robin in random order; a role is a generator yielding ("wait", barrier, parity, generation) or None."""
    rng = random.Random(seed)
    live = {i: iter(r) for i, r in enumerate(roles)}
    blocked = {}
    while live:
        progressed = False
        order = list(live)
        rng.shuffle(order)
        for i in order:
            if i in blocked:
                bar, parity, gen = blocked[i]
                if not bar.passes(parity):
                    continue
                assert bar.completions == gen + 1, f"wait for completion {gen} passed at {bar.completions}"
                del blocked[i]
            try:
                req = next(live[i])
                progressed = True
            except StopIteration:
                del live[i]
                progressed = True
                continue
            if req is not None:
                blocked[i] = req[1:]
        assert progressed, f"dead-lock with roles {sorted(live)} blocked"


def wait(bar, generation):
    return ("wait", bar, generation & 1, generation)


# --------------------------------------------------------------------------------------------- forward, two tiles
def forward_roles(n_a, n_b, NS, always_rescale):
    full = [Barrier(1) for _ in range(NS)]
    empty = [Barrier(1) for _ in range(NS)]
    q = Barrier(1)
    s_full, p_full, o_done = [Barrier(1), Barrier(1)], [Barrier(4), Barrier(4)], [Barrier(1), Barrier(1)]
    stage_item = [None] * NS       # which ring item a stage holds
    released = set()

    def producer():
        q.arrive()
        yield None
        for t in range(2 * n_b):
            s = t % NS
            if t >= NS:
                yield wait(empty[s], t // NS - 1)
                assert stage_item[s] in released, "ring stage refilled before its release"
            stage_item[s] = t
            full[s].arrive()
            yield None

    def issuer():
        yield wait(q, 0)
        item = lambda t: wait(full[t % NS], t // NS)
        yield item(0)
        s_full[0].arrive(); s_full[1].arrive()
        released.add(0); empty[0].arrive()
        yield None
        for j in range(n_b):
            yield item(2 * j + 1)
            assert stage_item[(2 * j + 1) % NS] == 2 * j + 1
            if j + 1 < n_b:
                yield item(2 * j + 2)
                assert stage_item[(2 * j + 2) % NS] == 2 * j + 2
            if j < n_a:
                yield wait(p_full[0], j)
                o_done[0].arrive()
                if j + 1 < n_a:
                    s_full[0].arrive()
                yield None
            yield wait(p_full[1], j)
            o_done[1].arrive()
            released.add(2 * j + 1); empty[(2 * j + 1) % NS].arrive()
            if j + 1 < n_b:
                s_full[1].arrive()
                released.add(2 * j + 2); empty[(2 * j + 2) % NS].arrive()
            yield None

    def softmax(g, n_kv):
        for j in range(n_kv):
            yield wait(s_full[g], j)
            if j > 0 and always_rescale:
                yield wait(o_done[g], j - 1)
            p_full[g].arrive()
            yield None
        yield wait(o_done[g], n_kv - 1)

    return [producer(), issuer()] + [softmax(0, n_a) for _ in range(4)] + [softmax(1, n_b) for _ in range(4)]


@pytest.mark.parametrize("n_a,n_b", [(1, 2), (3, 4), (7, 8), (31, 32), (2, 4), (6, 8), (30, 32)])
@pytest.mark.parametrize("NS", [4, 5, 6])
def test_forward_two_tile_protocol(n_a, n_b, NS):
    for seed in range(12):
        run(forward_roles(n_a, n_b, NS, always_rescale=bool(seed & 1)), seed)


# --------------------------------------------------------------------------------------------- backward
def backward_roles(n_iter, NB, TS, NG):
    r = Barrier(1)
    t_full = [Barrier(1) for _ in range(TS)]
    t_empty = [Barrier(1) for _ in range(TS)]
    xy_full, ds_full = [Barrier(1) for _ in range(2)], [Barrier(4 * NG) for _ in range(2)]
    acc = Barrier(1)
    stage_tile = [None] * TS
    released = set()
    holds = [None] * NB            # tile whose P / dS a score buffer holds, until the products reading it are issued

    def producer():
        r.arrive()
        yield None
        for it in range(n_iter):
            st = it % TS
            if it >= TS:
                yield wait(t_empty[st], it // TS - 1)
                assert stage_tile[st] in released, "streamed tile overwritten before its release"
            stage_tile[st] = it
            t_full[st].arrive()
            yield None

    def issue_acc(u):
        yield wait(ds_full[u % NB], u // NB)
        assert holds[u % NB] == u and stage_tile[u % TS] == u
        holds[u % NB] = None
        released.add(u)
        t_empty[u % TS].arrive()
        yield None

    def issuer():
        yield wait(r, 0)
        for it in range(n_iter):
            s, st = it % NB, it % TS
            if NB == 1 and it >= 1:
                yield from issue_acc(it - 1)
            yield wait(t_full[st], it // TS)
            assert holds[s] is None, "scores written over P / dS that the gradient products have not read"
            holds[s] = it
            xy_full[s].arrive()
            yield None
            if NB == 2 and it >= 1:
                yield from issue_acc(it - 1)
        yield from issue_acc(n_iter - 1)
        acc.arrive()

    def recompute():
        for it in range(n_iter):
            s = it % NB
            yield wait(xy_full[s], it // NB)
            assert holds[s] == it
            ds_full[s].arrive()
            yield None
        yield wait(acc, 0)

    return [producer(), issuer()] + [recompute() for _ in range(4 * NG)]


@pytest.mark.parametrize("n_iter", [1, 2, 3, 7, 64])
@pytest.mark.parametrize("NB,TS,NG", [(2, 5, 4), (2, 6, 2), (1, 3, 2), (2, 3, 2), (2, 2, 4)])
def test_backward_protocol(n_iter, NB, TS, NG):
    for seed in range(8):
        run(backward_roles(n_iter, NB, TS, NG), seed)
