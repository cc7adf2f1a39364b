"""Host-side model of the mbarrier protocol of the GEMM kernels (single CTA and CTA pair).

The kernels' roles (TMA producer, MMA issuer, epilogue) are written here as Python generators that perform the same
waits, arrivals and phase flips as the device loops in ``ksa_b200/csrc/gemm.cu`` and ``gemm2.cu``; a scheduler
interleaves them at random.  The model checks what the phase bits are supposed to guarantee: nobody overwrites a
stage that has not been consumed, nothing is consumed before it was fully produced, accumulator buffers are not
rewritten before the epilogue has drained them, and every role terminates (no deadlock) for any interleaving.
"""
import random

import pytest


class MBar:
    """``mbarrier`` with an arrival count and a transaction-byte count; a phase completes when both reach zero."""

    def __init__(self, count):
        self.count, self.pending, self.tx, self.phase = count, count, 0, 0

    def _maybe_flip(self):
        if self.pending == 0 and self.tx == 0:
            self.phase ^= 1
            self.pending = self.count

    def arrive(self, expect_tx=0):
        assert self.pending > 0, "more arrivals than the barrier was initialised for"
        self.tx += expect_tx
        self.pending -= 1
        self._maybe_flip()

    def complete_tx(self, nbytes):
        self.tx -= nbytes
        self._maybe_flip()

    def done(self, parity):          # try_wait.parity: has the phase with this parity completed?
        return self.phase != parity


def run(roles, rng, limit=200000):
    live = list(roles)
    for _ in range(limit):
        if not live:
            return
        r = rng.choice(live)
        try:
            next(r)
        except StopIteration:
            live.remove(r)
    raise AssertionError("roles did not finish: deadlock or livelock in the protocol")


def wait(bar, parity):
    while not bar.done(parity):
        yield


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("stages,tiles,kblocks", [(4, 5, 3), (6, 3, 13), (2, 7, 1), (6, 1, 6)])
def test_gemm_pipeline_protocol(pair, stages, tiles, kblocks):
    n_cta = 2 if pair else 1
    stage_bytes = 100
    for seed in range(20):
        rng = random.Random(seed)
        full = [MBar(1) for _ in range(stages)]                        # lives in the leader
        empty = [[MBar(1) for _ in range(stages)] for _ in range(n_cta)]
        acc_full = [[MBar(1) for _ in range(2)] for _ in range(n_cta)]
        acc_empty = [MBar(4 * n_cta) for _ in range(2)]                # leader: one arrival per epilogue warp
        smem = [[None] * stages for _ in range(n_cta)]                 # what each stage currently holds
        inflight = []                                                  # TMA copies issued but not yet landed
        tmem = [[None, None] for _ in range(n_cta)]                    # accumulator buffers: list of consumed k-blocks
        results = [[] for _ in range(n_cta)]

        def producer(cta):
            stage, phase = 0, 0
            for tile in range(tiles):
                for kb in range(kblocks):
                    yield from wait(empty[cta][stage], phase ^ 1)
                    assert smem[cta][stage] is None, "stage overwritten before the MMA consumed it"
                    if cta == 0:
                        full[stage].arrive(expect_tx=stage_bytes * n_cta)
                    inflight.append((cta, stage, (tile, kb)))
                    stage += 1
                    if stage == stages:
                        stage, phase = 0, phase ^ 1
                    yield

        def tma_engine():
            while True:
                if inflight:
                    cta, stage, what = inflight.pop(rng.randrange(len(inflight)))
                    smem[cta][stage] = what
                    full[stage].complete_tx(stage_bytes)               # the peer's bytes land on the leader's barrier
                elif all(p is None for p in prods):
                    return
                yield

        def mma():
            stage, phase = 0, 0
            for local, tile in enumerate(range(tiles)):
                buf, acc_phase = local & 1, (local >> 1) & 1
                yield from wait(acc_empty[buf], acc_phase ^ 1)
                for c in range(n_cta):
                    assert tmem[c][buf] is None, "accumulator rewritten before the epilogue drained it"
                    tmem[c][buf] = []
                for kb in range(kblocks):
                    yield from wait(full[stage], phase)
                    for c in range(n_cta):
                        assert smem[c][stage] == (tile, kb), "MMA read a stage that was not (fully) produced"
                        tmem[c][buf].append((tile, kb))
                        smem[c][stage] = None
                    for c in range(n_cta):                              # one multicast commit frees the stage in both
                        empty[c][stage].arrive()
                    stage += 1
                    if stage == stages:
                        stage, phase = 0, phase ^ 1
                    yield
                for c in range(n_cta):
                    acc_full[c][buf].arrive()

        def epilogue(cta, warp):
            for local, tile in enumerate(range(tiles)):
                buf, acc_phase = local & 1, (local >> 1) & 1
                yield from wait(acc_full[cta][buf], acc_phase)
                assert tmem[cta][buf] == [(tile, kb) for kb in range(kblocks)]
                if warp == 0:
                    results[cta].append(tile)
                yield
                drained[cta][buf] += 1
                if drained[cta][buf] == 4:                              # last warp of this CTA: buffer is free here
                    drained[cta][buf] = 0
                    tmem[cta][buf] = None
                acc_empty[buf].arrive()

        drained = [[0, 0] for _ in range(n_cta)]
        prods = [producer(c) for c in range(n_cta)]

        def tracked(i):
            yield from prods[i]
            prods[i] = None
        roles = [tracked(c) for c in range(n_cta)] + [tma_engine(), mma()]
        roles += [epilogue(c, w) for c in range(n_cta) for w in range(4)]
        run(roles, rng)
        assert all(r == list(range(tiles)) for r in results)


def test_model_detects_a_missing_phase_flip():
    """The model is not vacuous: a producer that forgets to flip its phase bit is caught."""
    rng = random.Random(0)
    empty, full = [MBar(1) for _ in range(2)], [MBar(1) for _ in range(2)]
    smem = [None, None]

    def producer():
        stage = 0
        for i in range(6):
            yield from wait(empty[stage], 1)      # bug: always waits for parity 1
            assert smem[stage] is None, "stage overwritten before it was consumed"
            smem[stage] = i
            full[stage].arrive()
            stage ^= 1
            yield

    def consumer():
        stage, phase = 0, 0
        for i in range(6):
            yield from wait(full[stage], phase)
            smem[stage] = None
            empty[stage].arrive()
            stage ^= 1
            if stage == 0:
                phase ^= 1
            yield

    with pytest.raises(AssertionError):
        for seed in range(50):
            rng = random.Random(seed)
            empty, full = [MBar(1) for _ in range(2)], [MBar(1) for _ in range(2)]
            smem = [None, None]
            run([producer(), consumer()], rng, limit=5000)


# ---------------------------------------------------------------------------------------------------------------------
# The shared-memory ring of the communication warp (run_gather_job_bulk in ksa_b200/csrc/comm.cuh): ONE thread issues
# bulk loads into stage n % S while fewer than S chunks are between "load issued" and "store has read its stage",
# waits for the oldest load, issues its bulk store, and then waits until every store but the newest has read its
# stage (wait_group.read 1); at the end of a shard it waits for all stores (wait_group 0).
def _ring_thread(S, shards, rng, state, forget_store_wait=False):
    full = [MBar(1) for _ in range(S)]
    ring = [None] * S                 # chunk a stage holds (None: free)
    loads, stores = [], []            # copies in flight
    out = state["out"]

    def thread():
        issued = stored = freed = 0
        for shard, chunks in enumerate(shards):
            next_load = next_store = 0
            while next_store < chunks:
                while next_load < chunks and issued - freed < S:
                    s = issued % S
                    assert ring[s] is None and all(st != s for st, _ in stores), \
                        "a stage was refilled while a store still reads it"
                    full[s].arrive(expect_tx=1)
                    loads.append((s, (shard, next_load)))
                    issued += 1
                    next_load += 1
                    yield
                s = stored % S
                yield from wait(full[s], (stored // S) & 1)
                assert ring[s] == (shard, next_store), "a store read a stage before its load had landed"
                stores.append((s, (shard, next_store)))
                stored += 1
                next_store += 1
                if not forget_store_wait:
                    while len(stores) > 1:                 # wait_group.read 1
                        yield
                freed = stored - 1
                yield
            while stores:                                  # wait_group 0 at the end of a shard
                yield
            freed = stored
            state["done"].append(shard)
        state["stop"] = True

    def engine():
        while not state["stop"]:
            if loads and (not stores or rng.random() < 0.5):
                s, what = loads.pop(rng.randrange(len(loads)))
                ring[s] = what
                full[s].complete_tx(1)
            elif stores:
                s, what = stores.pop(0)                    # stores of one thread complete in order
                out.append(what)
                ring[s] = None
            yield

    return thread(), engine()


@pytest.mark.parametrize("S", [4, 2, 3, 8])
def test_bulk_ring_protocol(S):
    shards = [7, 1, 0, 13]
    for seed in range(25):
        rng = random.Random(seed)
        state = {"out": [], "done": [], "stop": False}
        run(list(_ring_thread(S, shards, rng, state)), rng)
        assert state["out"] == [(sh, c) for sh, n in enumerate(shards) for c in range(n)]
        assert state["done"] == list(range(len(shards)))


def test_bulk_ring_model_catches_a_missing_store_wait():
    """Not vacuous: without the wait for the older stores a stage is refilled while the copy engine still reads it."""
    with pytest.raises(AssertionError, match="refilled|before its load"):
        for seed in range(40):
            rng = random.Random(seed)
            state = {"out": [], "done": [], "stop": False}
            run(list(_ring_thread(2, [9, 9], rng, state, forget_store_wait=True)), rng)


# ---------------------------------------------------------------------------------------------------------------------
# Staging buffers of the scattering epilogue (ksa_b200/csrc/gemm2.cu): every epilogue warp owns two 4 KB buffers; piece
# p of the accumulator is packed into buffer p % 2 and sent with a TMA store that reads the buffer asynchronously.
# Before the first write of a piece the warp waits until at most the newest store is still reading
# (cp.async.bulk.wait_group.read 1), which is the store of piece p - 1, in the other buffer.
def _staging_warp(pieces, rng, state, wait_allowance=1):
    stores = []                      # (buffer, piece) stores that still read their buffer, oldest first
    buf = [None, None]

    def warp():
        for p in range(pieces):
            b = p % 2
            while len(stores) > wait_allowance:          # wait_group.read <allowance>
                yield
            assert all(sb != b for sb, _ in stores), "a staging buffer was rewritten while a store still reads it"
            buf[b] = ("half0", p)
            yield
            buf[b] = ("full", p)
            stores.append((b, p))
            yield
        while stores:                                    # wait_group 0 before the kernel ends
            yield
        state["stop"] = True

    def engine():
        while not state["stop"]:
            if stores and rng.random() < 0.4:
                b, p = stores.pop(0)
                assert buf[b] == ("full", p), "a store read a buffer that holds another piece"
                state["out"].append(p)
            yield
    return warp(), engine()


def test_epilogue_staging_buffers():
    for seed in range(30):
        rng = random.Random(seed)
        state = {"out": [], "stop": False}
        run(list(_staging_warp(13, rng, state)), rng)
        assert state["out"] == list(range(13))
    # not vacuous: allowing two stores in flight lets piece p overwrite the buffer that the store of piece p - 2 reads
    with pytest.raises(AssertionError, match="rewritten|another piece"):
        for seed in range(40):
            rng = random.Random(seed)
            state = {"out": [], "stop": False}
            run(list(_staging_warp(13, rng, state, wait_allowance=2)), rng)
