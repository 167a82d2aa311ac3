"""Host model of the device-side synchronisation protocols (no GPU): random interleavings of the steps that the kernels
perform, checked against the property each protocol has to guarantee.

* epoch barrier (``csrc/comm/peer.cu``): every rank publishes the epoch number into its word of every peer's control
  block and waits until all words of its own block have reached the epoch. Property: no rank leaves barrier ``e``
  before every rank has entered it. The model also shows why barriers issued from two streams need two control blocks:
  with one block, a younger barrier that overtakes an older one makes the older one's store move a flag backwards and a
  waiter can miss its epoch (the model finds that schedule; with separate blocks it cannot happen).
* ready flags of the all-gather inside the GEMM (``csrc/comm/tp_gemm.cu``): a gather CTA copies a row block and then
  publishes ``ready[block] = epoch`` with release semantics; a GEMM CTA reads a block only after it saw the flag.
  Property: no block is consumed before it was copied, for every order in which producers and consumers are scheduled.
"""

import random


def _run_barriers(world: int, schedule_seed: int, domains: int, barriers_per_stream: int = 3):
    """Each rank runs ``domains`` streams; stream ``s`` issues barriers with epochs 1..n on control block ``s % blocks``.
    A barrier kernel is two atomic steps per peer word: store own epoch (any order over peers), then poll until all
    words >= epoch. Kernels of one stream run in order; kernels of different streams of a rank interleave freely.
    Returns (violations, stuck): a violation is a rank that left barrier (stream, e) before some rank entered it."""
    rng = random.Random(schedule_seed)
    blocks = domains  # one control block per stream: the engine's layout
    flags = [[[0] * world for _ in range(world)] for _ in range(blocks)]  # flags[block][reader][writer]
    entered = set()
    # kernel state per (rank, stream): index of current barrier, phase 0 = not started, 1 = stored, 2 = done
    state = {(r, s): [1, 0] for r in range(world) for s in range(domains)}
    violations = 0
    for _ in range(200000):
        live = [k for k, (e, _) in state.items() if e <= barriers_per_stream]
        if not live:
            return violations, False
        rank, stream = rng.choice(live)
        epoch, phase = state[(rank, stream)]
        block = stream % blocks
        if phase == 0:
            entered.add((rank, stream, epoch))
            for peer in range(world):
                flags[block][peer][rank] = epoch
            state[(rank, stream)][1] = 1
        else:
            if all(flags[block][rank][w] >= epoch for w in range(world)):
                if any((w, stream, epoch) not in entered for w in range(world)):
                    violations += 1
                state[(rank, stream)] = [epoch + 1, 0]
    return violations, True


def test_epoch_barrier_never_releases_early_and_always_finishes():
    for seed in range(200):
        for world in (2, 4, 8):
            violations, stuck = _run_barriers(world, seed, domains=1)
            assert violations == 0 and not stuck
    for seed in range(100):
        violations, stuck = _run_barriers(4, seed, domains=2)  # main stream + side stream, one control block each
        assert violations == 0 and not stuck


def test_one_control_block_shared_by_two_streams_can_lose_an_epoch():
    """The hazard that the second control block removes: two streams of every rank count epochs on the same words."""
    rng = random.Random(0)
    world = 2
    lost = False
    for _ in range(2000):
        flags = [[0] * world for _ in range(world)]
        # rank 0: the younger barrier (epoch 2, side stream) stores first, then the older one (epoch 1) stores
        order = [(0, 2), (0, 1), (1, 1), (1, 2)]
        rng.shuffle(order)
        for rank, epoch in order:
            for peer in range(world):
                flags[peer][rank] = epoch  # plain store: a later store of a smaller epoch moves the flag backwards
        # a waiter of epoch 2 that polls now may see 1 although epoch 2 had been published
        if any(flags[r][w] < 2 for r in range(world) for w in range(world)):
            lost = True
            break
    assert lost


def test_ready_flags_order_copy_before_consumption():
    for seed in range(300):
        rng = random.Random(seed)
        blocks, epoch = 12, 5
        copied = [False] * blocks
        ready = [epoch - 1] * blocks  # left over from the previous call
        consumed = []
        producers = list(range(blocks))
        rng.shuffle(producers)
        pending_copy, pending_flag = producers[:], []
        waiting = list(range(blocks))
        rng.shuffle(waiting)
        for _ in range(10000):
            if not waiting:
                break
            move = rng.random()
            if move < 0.3 and pending_copy:
                b = pending_copy.pop(0)
                copied[b] = True  # bulk copy has landed ...
                pending_flag.append(b)
            elif move < 0.6 and pending_flag:
                b = pending_flag.pop(0)
                ready[b] = epoch  # ... and only then the release store of the flag
            else:
                b = waiting[0]
                if ready[b] >= epoch:  # acquire load
                    assert copied[b], "a row block was read before its copy had landed"
                    consumed.append(waiting.pop(0))
        assert sorted(consumed) == list(range(blocks))
