"""The tensor-parallel protocols, modelled on the host at world 2 / 4 / 8 (threads over shared memory): the sequence-flag
barrier of the one-shot collectives, the push / pull pairing of the one-token projections with its two alternating call
sites, and the tile ownership of the sequence-parallel prefill. The device kernels implement exactly these rules; the
models check that the rules themselves are sound for every world size (no early pass, no lost update, a partition)."""
import threading

import numpy as np
import pytest

from owl_engine_b200.parallel.symm import PrefillPipe


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sequence_flag_barrier_never_passes_early(world):
    rounds = 60
    flags = np.zeros((world, world), dtype=np.int64)        # flags[dst][src]
    arrived = np.zeros(rounds + 1, dtype=np.int64)
    lock = threading.Lock()
    bad = []

    def rank(r):
        seq = 0
        for k in range(1, rounds + 1):
            with lock:
                arrived[k] += 1
            seq += 1
            for peer in range(world):
                flags[peer][r] = seq                         # release store into every peer's table
            while not all(flags[r][p] - seq >= 0 for p in range(world)):
                pass
            if arrived[k] != world:                          # passed before everybody arrived
                bad.append((r, k, int(arrived[k])))
    ts = [threading.Thread(target=rank, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join(60) for t in ts]
    assert not bad and not any(t.is_alive() for t in ts)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_push_pull_pairing_with_two_alternating_sites(world):
    """Each rank: producer writes its partial into slot [rank] of every rank's buffer of site w and publishes seq[w]; the
    consumer waits for every flag >= its local producer's seq[w], sums the slots in rank order. Sites alternate 0, 1, 0, ..
    and a fast rank may run ahead by at most one site, which two buffers cover: every rank must compute the same sums."""
    steps = 40
    slots = np.zeros((world, 2, world), dtype=np.int64)     # [dst rank][site][src rank]
    flags = np.zeros((world, 2, world), dtype=np.int64)
    sums = np.zeros((world, steps), dtype=np.int64)

    def rank(r):
        seq = [0, 0]
        rng = np.random.default_rng(r)
        for s in range(steps):
            w = s & 1
            val = (s + 1) * 1000 + r                         # this rank's partial of step s
            if rng.random() < 0.2:
                for _ in range(200):                         # jitter: some ranks lag
                    pass
            for peer in range(world):
                slots[peer][w][r] = val
            seq[w] += 1
            for peer in range(world):
                flags[peer][w][r] = seq[w]
            while not all(flags[r][w][p] - seq[w] >= 0 for p in range(world)):
                pass
            sums[r][s] = sum(int(slots[r][w][p]) for p in range(world))
    ts = [threading.Thread(target=rank, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join(120) for t in ts]
    assert not any(t.is_alive() for t in ts)
    want = np.array([sum((s + 1) * 1000 + r for r in range(world)) for s in range(steps)])
    for r in range(world):
        assert (sums[r] == want).all(), (r, np.nonzero(sums[r] != want)[0][:5])


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("t", [128, 300, 2048, 2049])
def test_prefill_tile_ownership_is_a_partition(world, t):
    tiles = (t + 127) // 128
    seen = {}
    for rank in range(world):
        ml = PrefillPipe.max_local_for(t, world)
        mine = list(range(rank, tiles, world))
        assert len(mine) <= ml
        for j in mine:
            for row in range(j * 128, min(t, j * 128 + 128)):
                assert row not in seen
                seen[row] = (rank, (j // world) * 128 + row % 128)
    assert sorted(seen) == list(range(t))
    # local_row is the inverse map every rank uses to find a row's owner
    for row in (0, t // 2, t - 1):
        j = row // 128
        assert seen[row] == (j % world, (j // world) * 128 + row % 128)
