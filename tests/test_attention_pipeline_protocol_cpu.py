"""Host model of the barrier protocol of the pipelined attention backward kernel (``csrc/ops/attention_bwd.cu``), no GPU.

Five kinds of actors share one CTA: the TMA producer, the MMA thread (whose products retire in issue order), the
arithmetic threads (P from S, dS from dP), the drain threads (dQ from tensor memory to the staging boxes) and the
asynchronous engines themselves (TMA loads, tensor cores). They meet at mbarriers that complete once per (head, query
tile) step and are waited for by phase parity. The model runs the same sequence of waits, arrivals and commits under
random interleavings and checks

* that every schedule finishes (no cyclic wait), for any number of steps,
* that a waiter never falls a whole phase behind a barrier (the parity it waits for would otherwise be ambiguous),
* that every buffer holds what its reader expects: S / P / next S share tensor-memory columns, dP / dQ share the next
  ones, Q has two buffers, dO one, dS one, the per-query statistics two.
"""

import random

import pytest


class _Barrier:
    def __init__(self, name: str, count: int) -> None:
        self.name, self.count, self.pending, self.completed = name, count, count, 0

    def arrive(self) -> None:
        self.pending -= 1
        if self.pending == 0:
            self.pending = self.count
            self.completed += 1


class _Model:
    def __init__(self, steps: int, arithmetic: int, drain: int, seed: int) -> None:
        self.n, self.rng = steps, random.Random(seed)
        self.bar = {name: _Barrier(name, count) for name, count in [
            ("KV", 1), ("Q_FULL0", 1), ("Q_FULL1", 1), ("Q_EMPTY0", 1), ("Q_EMPTY1", 1), ("DO_FULL", 1), ("DO_EMPTY", 1),
            ("S_FULL", 1), ("DP_FULL", 1), ("P_READY", arithmetic), ("DS_READY", arithmetic), ("DQ_FULL", 1),
            ("DQ_DRAINED", drain), ("ROWS", arithmetic)]}
        self.tmem = {"S": None, "dP": None}
        self.smem = {"Q0": None, "Q1": None, "dO": None, "dS": None, "rows0": None, "rows1": None}
        self.tensor_core: list = []  # issued products, retired in order
        self.tma: list = []          # loads in flight, completed in any order
        self.arithmetic, self.drain = arithmetic, drain

    # a wait for completion number `index` of a barrier, by parity: legal only while the waiter is less than one full
    # phase behind, i.e. while at most `index + 1` completions have happened
    def wait(self, name: str, index: int):
        return ("wait", name, index)

    def check(self, cond: bool, *what) -> None:
        assert cond, what

    # ------------------------------------------------------------------ actors
    def producer(self):
        self.tma.append(lambda: self.bar["KV"].arrive())
        for it in range(self.n):
            b = it & 1
            if it >= 2:
                yield self.wait(f"Q_EMPTY{b}", (it >> 1) - 1)

            def load_q(it=it, b=b):
                self.smem[f"Q{b}"] = it
                self.bar[f"Q_FULL{b}"].arrive()
            self.tma.append(load_q)
            if it >= 1:
                yield self.wait("DO_EMPTY", it - 1)

            def load_do(it=it):
                self.smem["dO"] = it
                self.bar["DO_FULL"].arrive()
            self.tma.append(load_do)

    def mma(self):
        def s(it):
            def run():
                self.check(self.smem[f"Q{it & 1}"] == it, "S reads the wrong Q", it, self.smem)
                self.check(self.tmem["S"] in (None, ("P consumed", it - 1)), "S overwrites live columns", it, self.tmem)
                self.tmem["S"] = ("S", it)
                self.bar["S_FULL"].arrive()
            return run

        def dp(it):
            def run():
                self.check(self.smem["dO"] == it, "dP reads the wrong dO", it, self.smem)
                self.check(self.tmem["dP"] in (None, ("dQ drained", it - 1)), "dP overwrites live columns", it, self.tmem)
                self.tmem["dP"] = ("dP", it)
                self.bar["DP_FULL"].arrive()
            return run

        yield self.wait("KV", 0)
        yield self.wait("Q_FULL0", 0)
        self.tensor_core.append(s(0))
        yield self.wait("DO_FULL", 0)
        self.tensor_core.append(dp(0))
        for it in range(self.n):
            yield self.wait("P_READY", it)

            def dv(it=it):
                self.check(self.tmem["S"] == ("P", it) and self.smem["dO"] == it, "dV operands", it, self.tmem, self.smem)
                self.tmem["S"] = ("P consumed", it)
                self.bar["DO_EMPTY"].arrive()
            self.tensor_core.append(dv)
            if it + 1 < self.n:
                yield self.wait(f"Q_FULL{(it + 1) & 1}", (it + 1) >> 1)
                self.tensor_core.append(s(it + 1))
            yield self.wait("DS_READY", it)

            def dq(it=it):
                self.check(self.smem["dS"] == ("dS", it) and self.tmem["dP"] == ("dP consumed", it), "dQ operands", it, self.smem, self.tmem)
                self.tmem["dP"] = ("dQ", it)
                self.bar["DQ_FULL"].arrive()
            self.tensor_core.append(dq)

            def dk(it=it):
                self.check(self.smem["dS"] == ("dS", it) and self.smem[f"Q{it & 1}"] == it, "dK operands", it, self.smem)
                self.smem["dS"] = ("free", it)
                self.bar[f"Q_EMPTY{it & 1}"].arrive()
            self.tensor_core.append(dk)
            if it + 1 < self.n:
                yield self.wait("DQ_DRAINED", it)
                yield self.wait("DO_FULL", it + 1)
                self.tensor_core.append(dp(it + 1))

    def arithmetic_thread(self):
        def last_arrival(name: str, effect):
            if self.bar[name].pending == 1:
                effect()
            self.bar[name].arrive()

        self.smem["rows0"] = 0 if self.smem["rows0"] in (None, 0) else self.smem["rows0"]
        self.bar["ROWS"].arrive()
        for it in range(self.n):
            yield self.wait("S_FULL", it)
            yield self.wait("ROWS", it)
            self.check(self.tmem["S"] in (("S", it), ("P", it)), "P reads", it, self.tmem)
            self.check(self.smem[f"rows{it & 1}"] == it, "lse of the wrong step", it, self.smem)
            yield ("yield",)
            last_arrival("P_READY", lambda it=it: self.tmem.__setitem__("S", ("P", it)))
            yield self.wait("DP_FULL", it)
            if it + 1 < self.n:
                # every thread has finished dS(it - 1), the last reader of this buffer: dP(it) was issued after dQ(it - 1)
                self.check(self.smem[f"rows{(it + 1) & 1}"] in (None, it - 1, it + 1), "statistics overwritten early", it, self.smem)
                self.smem[f"rows{(it + 1) & 1}"] = it + 1
                self.bar["ROWS"].arrive()
            self.check(self.tmem["dP"] in (("dP", it), ("dP consumed", it)), "dS reads", it, self.tmem)
            self.check(self.smem[f"rows{it & 1}"] == it, "delta of the wrong step", it, self.smem)
            self.check(self.smem["dS"] in (None, ("free", it - 1), ("dS being written", it)), "dS tile still in use", it, self.smem)
            self.smem["dS"] = ("dS being written", it)
            yield ("yield",)

            def done(it=it):
                self.tmem["dP"] = ("dP consumed", it)
                self.smem["dS"] = ("dS", it)
            last_arrival("DS_READY", done)
        # the epilogue reads dK / dV: the last dK has been committed
        yield self.wait(f"Q_EMPTY{(self.n - 1) & 1}", (self.n - 1) >> 1)

    def drain_thread(self):
        for it in range(self.n):
            yield self.wait("DQ_FULL", it)
            self.check(self.tmem["dP"] == ("dQ", it), "drain reads", it, self.tmem)
            yield ("yield",)
            if self.bar["DQ_DRAINED"].pending == 1:
                self.tmem["dP"] = ("dQ drained", it)
            self.bar["DQ_DRAINED"].arrive()

    # ------------------------------------------------------------------ scheduler
    def run(self) -> None:
        actors = {"producer": self.producer(), "mma": self.mma()}
        actors.update({f"arithmetic{i}": self.arithmetic_thread() for i in range(self.arithmetic)})
        actors.update({f"drain{i}": self.drain_thread() for i in range(self.drain)})
        waiting = dict.fromkeys(actors)
        live = set(actors)
        while live:
            progressed = False
            names = list(live)
            self.rng.shuffle(names)
            for name in names:
                if self.tensor_core and self.rng.random() < 0.4:
                    self.tensor_core.pop(0)()
                    progressed = True
                if self.tma and self.rng.random() < 0.4:
                    self.tma.pop(self.rng.randrange(len(self.tma)))()
                    progressed = True
                w = waiting[name]
                if w is not None:
                    _, bar, index = w
                    done = self.bar[bar].completed
                    assert done <= index + 1, f"{name} fell a whole phase behind {bar}: waits for completion {index}, {done} happened"
                    if done <= index:
                        continue
                    waiting[name] = None
                try:
                    event = next(actors[name])
                except StopIteration:
                    live.discard(name)
                    progressed = True
                    continue
                progressed = True
                if event[0] == "wait":
                    waiting[name] = event
            if not progressed:
                if self.tensor_core:
                    self.tensor_core.pop(0)()
                elif self.tma:
                    self.tma.pop(0)()
                else:
                    raise AssertionError(f"deadlock: {{k: waiting[k] for k in live}} = { {k: waiting[k] for k in live} }")
        while self.tensor_core:
            self.tensor_core.pop(0)()


@pytest.mark.parametrize("steps", [1, 2, 3, 4, 7, 16])
def test_every_schedule_finishes_without_a_hazard(steps):
    for seed in range(120):
        _Model(steps, arithmetic=4, drain=2, seed=seed).run()


def test_the_model_notices_a_missing_dependency():
    """Sanity of the model itself: without the wait for the drained dQ the next dP lands in live columns."""

    class Broken(_Model):
        def wait(self, name, index):
            return ("yield",) if name == "DQ_DRAINED" else super().wait(name, index)

    with pytest.raises(AssertionError):
        for seed in range(200):
            Broken(6, arithmetic=4, drain=2, seed=seed).run()
