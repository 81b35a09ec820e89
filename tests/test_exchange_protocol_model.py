"""A model of the low-latency exchange protocol (skn_allreduce_ll_kernel in csrc/skn_comm.cu), run on the CPU.

What is modelled: `world` ranks execute exchanges q = 0, 1, 2, ... one after another.  In exchange q a rank
stores the word {its value, tag q + 1} into slot [q % 2][its rank] of every peer's inbox and then polls its own
inbox until the slots of all peers carry tag q + 1; only then does it start exchange q + 1.  Stores travel
with arbitrary delays but stay in order per (source, destination) pair, which is what a GPU guarantees for
stores of one thread to one address.  What is checked, under many random schedules and for 2 to 8 ranks:
every rank finishes every exchange (no rank ever waits for a slot that has already been overwritten by a
later exchange: two buffers suffice for any number of ranks) and every value it reads is the one its peer
sent in that exchange.  The CUDA kernel itself is tested on the GPU (tests/test_gpu_multi.py, two ranks).
"""
import random

import pytest

NBUF = 2


def run_model(world: int, exchanges: int, seed: int, max_events: int = 2_000_000):
    rnd = random.Random(seed)
    inbox = [[[(None, 0) for _ in range(world)] for _ in range(NBUF)] for _ in range(world)]   # [owner][buf][src] = (value, tag)
    in_flight = {(s, d): [] for s in range(world) for d in range(world) if s != d}             # FIFO of stores per pair
    q = [0] * world                      # exchange each rank is in
    pushed = [False] * world             # has it issued this exchange's stores
    got = [[None] * world for _ in range(world)]      # values read so far in the current exchange
    results = [[] for _ in range(world)]
    events = 0
    while any(x < exchanges for x in q):
        events += 1
        assert events < max_events, f"no progress: ranks at {q} (a rank waits for a slot that will never match)"
        actions = []
        for r in range(world):
            if q[r] >= exchanges:
                continue
            if not pushed[r]:
                actions.append(("push", r))
            else:
                actions.append(("poll", r))
        for key, fifo in in_flight.items():
            if fifo:
                actions.append(("deliver", key))
        kind, arg = rnd.choice(actions)
        if kind == "push":
            r = arg
            for p in range(world):
                if p != r:
                    in_flight[(r, p)].append((q[r] % NBUF, (f"v{r}.{q[r]}", q[r] + 1)))
            pushed[r] = True
        elif kind == "deliver":
            s, d = arg
            buf, word = in_flight[arg].pop(0)
            inbox[d][buf][s] = word
        else:
            r = arg
            tag = q[r] + 1
            for s in range(world):
                if s != r and got[r][s] is None:
                    value, t = inbox[r][q[r] % NBUF][s]
                    if t == tag:
                        got[r][s] = value
            if all(got[r][s] is not None for s in range(world) if s != r):
                results[r].append([got[r][s] if s != r else f"v{r}.{q[r]}" for s in range(world)])
                got[r] = [None] * world
                pushed[r] = False
                q[r] += 1
    return results


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_two_buffers_suffice_and_every_read_is_this_exchanges_value(world):
    for seed in range(12):
        res = run_model(world, exchanges=9, seed=1000 * world + seed)
        for r in range(world):
            assert len(res[r]) == 9
            for qn, row in enumerate(res[r]):
                assert row == [f"v{s}.{qn}" for s in range(world)], (world, seed, r, qn)


def test_the_model_catches_a_protocol_with_one_buffer():
    """The same model with a single buffer deadlocks or reads a later exchange's value for some schedule, which is
    why the kernel keeps two: the check above is not vacuous."""
    global NBUF
    saved = NBUF
    NBUF = 1
    try:
        failed = False
        for seed in range(40):
            try:
                res = run_model(3, exchanges=6, seed=seed, max_events=20000)
                for r in range(3):
                    for qn, row in enumerate(res[r]):
                        if row != [f"v{s}.{qn}" for s in range(3)]:
                            failed = True
            except AssertionError:
                failed = True
            if failed:
                break
        assert failed
    finally:
        NBUF = saved
