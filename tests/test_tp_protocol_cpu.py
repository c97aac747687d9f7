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
def test_word_exchange_of_the_one_token_projections(world):
    """The exchange inside the one-token projections: a producer stores, per pair of sums, ONE word (data, number of this
    exchange) into slot [rank] of every rank's buffer of the call site -- words of one exchange land in any order and at any time
    -- and reads the call site's sequence word without writing it; a consumer accepts a word only when its number matches,
    adds the slots in rank order and advances the sequence word when its last "CTA" leaves. Two call sites alternate. Every
    rank must compute the same sums from exactly this exchange's data, with stale words of the site's previous use in place."""
    steps, n_words, n_ctas = 30, 6, 3
    words = np.zeros((world, 2, world, n_words, 2), dtype=np.int64)      # [dst][site][src][word] = (data, number)
    seq_word = np.zeros((world, 2), dtype=np.int64)                      # per rank, per call site
    left = np.zeros((world, 2), dtype=np.int64)
    sums = np.zeros((world, steps, n_words), dtype=np.int64)
    lock = threading.Lock()

    def rank(r):
        rng = np.random.default_rng(100 + r)
        for s in range(steps):
            w = s & 1
            number = seq_word[r][w] + 1                      # the producer only reads the word
            order = rng.permutation(n_words * world)
            for o in order:                                   # words reach the peers in any order
                peer, i = divmod(int(o), n_words)
                words[peer][w][r][i] = (1000 * (s + 1) + 10 * r + i, number)   # one atomic 8-byte store in the kernel
            # the consumer kernel: several CTAs, each reads the word, polls, the last one to leave advances the word
            want = seq_word[r][w] + 1
            acc = np.zeros(n_words, dtype=np.int64)
            for cta in range(n_ctas):
                assert seq_word[r][w] + 1 == want             # nobody advanced it while CTAs of this grid still start
                got = np.zeros(n_words, dtype=np.int64)
                for src in range(world):
                    for i in range(n_words):
                        while True:
                            d, n = words[r][w][src][i]
                            if n == want:
                                break
                        got[i] += d
                acc = got
                with lock:
                    left[r][w] += 1
                    if left[r][w] == n_ctas:
                        left[r][w] = 0
                        seq_word[r][w] = want
            sums[r][s] = acc
    ts = [threading.Thread(target=rank, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join(120) for t in ts]
    assert not any(t.is_alive() for t in ts)
    for s in range(steps):
        want = np.array([sum(1000 * (s + 1) + 10 * r + i for r in range(world)) for i in range(n_words)])
        for r in range(world):
            assert np.array_equal(sums[r][s], want), (r, s)
    assert (seq_word == steps // 2).all()


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
