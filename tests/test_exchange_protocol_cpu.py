"""Host-side models of the cross-GPU flag protocols (context-parallel exchange slots, tensor-parallel partial slots).

Each rank is a generator that performs the waits, writes and flag stores of ``ksa_b200/parallel/cp.py`` /
``ksa_b200/parallel/tp.py`` (and of the kernels they launch) in program order; a scheduler interleaves the ranks at
random.  The models check that no rank ever reads a slot that holds another exchange's data, that every run ends, and
that a withheld flag ends in an error status after the bounded wait instead of a stale read or an endless spin.
"""
import random

import pytest

WAIT_LIMIT = 400      # scheduler turns a model "kernel" spins before it gives up, like the cycle limit on the device


class Timeout(Exception):
    pass


def wait_ge(read, target, status, rank):
    spins = 0
    while read() < target:
        spins += 1
        if spins > WAIT_LIMIT:
            status[rank] = 5          # the status code of a peer-flag timeout
            raise Timeout()
        yield


def run(ranks, rng, limit=400000):
    live = list(ranks)
    for _ in range(limit):
        if not live:
            return
        r = rng.choice(live)
        try:
            next(r)
        except (StopIteration, Timeout):
            live.remove(r)
    raise AssertionError("ranks did not finish")


def cp_rank(rank, P, E, slots, ready, consumed, status, withhold=None):
    """Exchange e: publish into slot e % 2, pull from every earlier rank, tell everybody the slot was read."""
    last_use = [None, None]
    for e in range(E):
        s = e % 2
        if last_use[s] is not None:
            for p in range(P):
                yield from wait_ge(lambda p=p: consumed[rank][s][p], last_use[s] + 1, status, rank)
        last_use[s] = e
        slots[rank][s] = ("data", rank, e)
        yield
        if withhold != (rank, e):
            for p in range(P):
                ready[p][s][rank] = e + 1
                yield
        for owner in range(rank):                      # halo and summaries come from earlier ranks
            yield from wait_ge(lambda o=owner: ready[rank][s][o], e + 1, status, rank)
            assert slots[owner][s] == ("data", owner, e), f"rank {rank} read a stale or future block of rank {owner}"
            yield
        for p in range(P):
            consumed[p][s][rank] = e + 1
            yield


@pytest.mark.parametrize("P,E", [(2, 7), (4, 6), (8, 4)])
def test_context_parallel_exchange_slots(P, E):
    for seed in range(15):
        rng = random.Random(seed)
        slots = [[None, None] for _ in range(P)]
        ready = [[[0] * P for _ in range(2)] for _ in range(P)]        # ready[on rank][slot][producer]
        consumed = [[[0] * P for _ in range(2)] for _ in range(P)]     # consumed[on rank][slot][consumer]
        status = [0] * P
        run([cp_rank(r, P, E, slots, ready, consumed, status) for r in range(P)], rng)
        assert status == [0] * P


def test_context_parallel_withheld_flag_times_out_without_a_stale_read():
    P, E = 4, 6
    rng = random.Random(1)
    slots = [[None, None] for _ in range(P)]
    ready = [[[0] * P for _ in range(2)] for _ in range(P)]
    consumed = [[[0] * P for _ in range(2)] for _ in range(P)]
    status = [0] * P
    run([cp_rank(r, P, E, slots, ready, consumed, status, withhold=(1, 3)) for r in range(P)], rng)
    assert status[2] == 5 and status[3] == 5        # the ranks behind the silent one report a peer-flag timeout
    assert status[0] in (0, 5)                       # rank 0 reads nobody; it may time out later on a full slot


def tp_rank(rank, T, E, partial, flags, status, withhold=None):
    """All-reduce e (1-based flag value): the GEMM writes the partial block into slot (e-1) % 2, the fused kernel
    announces it, waits for every peer's announcement and reads all blocks."""
    for e in range(1, E + 1):
        s = (e - 1) % 2
        partial[rank][s] = ("partial", rank, e)
        yield
        if withhold != (rank, e):
            for p in range(T):
                flags[p][rank] = max(flags[p][rank], e)
                yield
        for p in range(T):
            yield from wait_ge(lambda p=p: flags[rank][p], e, status, rank)
        for p in range(T):
            assert partial[p][s] == ("partial", p, e), f"rank {rank} summed a block of another all-reduce from rank {p}"
            yield


@pytest.mark.parametrize("T", [2, 4, 8])
def test_tensor_parallel_partial_slots(T):
    for seed in range(15):
        rng = random.Random(seed)
        partial = [[None, None] for _ in range(T)]
        flags = [[0] * T for _ in range(T)]            # flags[on rank][announcing rank]
        status = [0] * T
        run([tp_rank(r, T, 9, partial, flags, status) for r in range(T)], rng)
        assert status == [0] * T
    # a rank that never announces all-reduce 4: everybody else gives up with the timeout status, nobody sums garbage
    rng = random.Random(3)
    partial = [[None, None] for _ in range(T)]
    flags = [[0] * T for _ in range(T)]
    status = [0] * T
    run([tp_rank(r, T, 9, partial, flags, status, withhold=(0, 4)) for r in range(T)], rng)
    assert all(status[r] == 5 for r in range(1, T))


def tp_rank_scatter(rank, T, E, recv, flags, status, slots=2):
    """All-reduce e in the scattered form: the row-parallel GEMM of rank r stores its partial of p's rows into block r
    of slot (e-1) % slots ON RANK p (P2P stores from the epilogue), the reduction kernel then announces, waits for every
    peer's announcement and reads only its own slot."""
    for e in range(1, E + 1):
        s = (e - 1) % slots
        for p in range(T):                                   # the epilogue's stores land one owner after the other
            recv[p][s][rank] = ("partial", rank, e)
            yield
        for p in range(T):
            flags[p][rank] = max(flags[p][rank], e)
            yield
        for p in range(T):
            yield from wait_ge(lambda p=p: flags[rank][p], e, status, rank)
        for q in range(T):
            assert recv[rank][s][q] == ("partial", q, e), f"rank {rank} summed a block of another all-reduce from rank {q}"
            yield


@pytest.mark.parametrize("T", [2, 4, 8])
def test_tensor_parallel_scattered_partials_two_slots(T):
    """The peers write into a rank's slot while it may still be reducing the previous all-reduce: two slots are enough,
    because a peer can only start the GEMM of all-reduce e+2 after this rank has announced e+1, i.e. after its
    reduction of e has ended."""
    for seed in range(20):
        rng = random.Random(seed)
        recv = [[[None] * T for _ in range(2)] for _ in range(T)]      # recv[on rank][slot][from rank]
        flags = [[0] * T for _ in range(T)]
        status = [0] * T
        run([tp_rank_scatter(r, T, 9, recv, flags, status) for r in range(T)], rng)
        assert status == [0] * T
    with pytest.raises(AssertionError, match="another all-reduce"):
        for seed in range(40):
            rng = random.Random(seed)
            recv = [[[None] * 3 for _ in range(1)] for _ in range(3)]
            flags = [[0] * 3 for _ in range(3)]
            run([tp_rank_scatter(r, 3, 6, recv, flags, [0] * 3, slots=1) for r in range(3)], rng)


def test_one_slot_would_not_be_enough():
    """The models are not vacuous: with a single slot a fast rank overwrites a block that a slow peer still reads."""
    def tp_one_slot(rank, T, E, partial, flags, status):
        for e in range(1, E + 1):
            partial[rank][0] = ("partial", rank, e)
            yield
            for p in range(T):
                flags[p][rank] = max(flags[p][rank], e)
                yield
            for p in range(T):
                yield from wait_ge(lambda p=p: flags[rank][p], e, status, rank)
            for p in range(T):
                assert partial[p][0] == ("partial", p, e)
                yield
    with pytest.raises(AssertionError):
        for seed in range(40):
            rng = random.Random(seed)
            partial = [[None] for _ in range(3)]
            flags = [[0] * 3 for _ in range(3)]
            run([tp_one_slot(r, 3, 6, partial, flags, [0] * 3) for r in range(3)], rng)


# ---------------------------------------------------------------------------------------------------------------------
# All-gather -> GEMM in one launch (ksa_b200/csrc/gemm2.cu + run_gather_job_bulk in comm.cuh): the communication warps
# copy the remote shards chunk by chunk; whenever a warp leaves one of the SEGS segments of a shard it waits for its
# stores and adds the number of chunks of that segment it wrote to done[shard][segment].  The TMA producers walk the
# tile rows starting at the first row block that lies entirely in the rank's own shard and wait, for every segment a
# row block touches, until its counter has reached the segment's chunk count.
SEGS = 4


def seg_begin(n_chunks, g):
    return (n_chunks * g + SEGS - 1) // SEGS


def seg_of(n_chunks, c):
    return max(g for g in range(SEGS) if seg_begin(n_chunks, g) <= c)


def _ag_gemm_roles(world, rank, rows, shard_rows, tile_rows, n_cta, ring, landed, done, status, reads, ready=True):
    chunk = 3                                             # rows per bulk copy
    n_chunks = (shard_rows + chunk - 1) // chunk
    tiles_m = (rows + tile_rows - 1) // tile_rows
    first_row = rank * shard_rows
    rotate = ((first_row + tile_rows - 1) // tile_rows) % tiles_m if 0 < first_row < rows else 0

    def comm_warp(cta):
        for step in range(1, world):
            r = (rank + step) % world
            yield from wait_ge(lambda: 1 if ready else 0, 1, status, 0)       # the shard's ready flag
            inflight, moved, seg = [], 0, None
            for c in range(cta, n_chunks, n_cta):
                if seg is None:
                    seg = seg_of(n_chunks, c)
                while len(inflight) >= ring:                                   # a stage frees when its store was read
                    landed[r].update(inflight.pop(0))
                    yield
                inflight.append(range(r * shard_rows + c * chunk, min(r * shard_rows + (c + 1) * chunk, (r + 1) * shard_rows)))
                moved += 1
                yield
                nxt = c + n_cta
                if nxt >= n_chunks or nxt >= seg_begin(n_chunks, seg + 1):     # leaves the segment: wait_group 0, report
                    for rows_ in inflight:
                        landed[r].update(rows_)
                        yield
                    inflight = []
                    done[r][seg] += moved
                    moved, seg = 0, (seg_of(n_chunks, nxt) if nxt < n_chunks else None)
                    yield

    def producer(pair, n_pairs):
        seen = set()
        for t in range(pair, tiles_m, n_pairs):
            mb = (t + rotate) % tiles_m
            lo, hi = mb * tile_rows, min((mb + 1) * tile_rows, rows)
            for s in range(lo // shard_rows, (hi - 1) // shard_rows + 1):
                if s == rank:
                    continue
                in_lo, in_hi = max(lo - s * shard_rows, 0), min(hi - 1 - s * shard_rows, shard_rows - 1)
                for g in range(seg_of(n_chunks, in_lo // chunk), seg_of(n_chunks, in_hi // chunk) + 1):
                    if (s, g) in seen:
                        continue
                    need = seg_begin(n_chunks, g + 1) - seg_begin(n_chunks, g)
                    yield from wait_ge(lambda s=s, g=g: done[s][g], need, status, 1)
                    seen.add((s, g))
            for row in range(lo, hi):                                          # the TMA loads of this tile
                s = row // shard_rows
                assert s == rank or row in landed[s], f"tile row {mb} read row {row} before that part of shard {s} had landed"
            reads.append(mb)
            yield
    n_pairs = max(n_cta // 2, 1)
    return [comm_warp(c) for c in range(n_cta)] + [producer(p, n_pairs) for p in range(n_pairs)]


@pytest.mark.parametrize("world,rank,rows,tile_rows", [(4, 1, 130, 8), (2, 0, 64, 8), (8, 7, 129, 4), (4, 3, 50, 16),
                                                       (2, 1, 300, 16)])
def test_all_gather_gemm_dependencies(world, rank, rows, tile_rows):
    shard_rows = (rows + world - 1) // world
    n_chunks = (shard_rows + 2) // 3
    for seed in range(20):
        rng = random.Random(seed)
        landed = [set() for _ in range(world)]
        done = [[0] * SEGS for _ in range(world)]
        status = [0, 0]
        reads = []
        run(_ag_gemm_roles(world, rank, rows, shard_rows, tile_rows, 6, 2, landed, done, status, reads), rng)
        assert status == [0, 0]
        assert sorted(reads) == list(range((rows + tile_rows - 1) // tile_rows))      # every tile row exactly once
        for r in range(world):                                                         # every chunk counted once
            assert sum(done[r]) == (0 if r == rank else n_chunks)


def test_all_gather_gemm_gives_up_when_shards_never_become_ready():
    world, rank, rows, tile_rows = 4, 0, 64, 8
    rng = random.Random(0)
    landed, done, status, reads = [set() for _ in range(world)], [[0] * SEGS for _ in range(world)], [0, 0], []
    run(_ag_gemm_roles(world, rank, rows, 16, tile_rows, 4, 2, landed, done, status, reads, ready=False), rng)
    assert status == [5, 5]                                   # the gather and then the math report the flag timeout
    assert all(mb * tile_rows < 16 for mb in reads)           # only tiles of the own shard were computed


def test_segment_arithmetic_covers_every_chunk_once():
    for n in list(range(1, 40)) + [5160, 5161]:
        begins = [seg_begin(n, g) for g in range(SEGS + 1)]
        assert begins[0] == 0 and begins[-1] == n and begins == sorted(begins)
        for c in range(min(n, 64)):
            g = seg_of(n, c)
            assert begins[g] <= c < begins[g + 1]


def test_device_segment_helpers_agree_with_the_model(tmp_path):
    """``bulk_segs`` / ``bulk_seg_begin`` / ``bulk_seg_of`` of ``ksa_b200/csrc/comm.cuh`` (``__host__ __device__``),
    compiled for the host, against the definitions above: every chunk lies in exactly the segment the helpers name,
    for every segment count up to the maximum."""
    import os
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc on this machine")
    csrc = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ksa_b200", "csrc")
    src = tmp_path / "segcheck.cu"
    src.write_text(r"""
#include "comm.cuh"
#include <cstdio>
using namespace ksa;
int main() {
  long long bad = 0;
  for (long long n = 1; n < 1500; ++n)
    for (int S = 1; S <= kBulkSegs; ++S) {
      if (bulk_seg_begin(n, S, 0) != 0 || bulk_seg_begin(n, S, S) != n) ++bad;
      for (long long c = 0; c < n; ++c) {
        const int g = bulk_seg_of(n, S, c);
        if (g < 0 || g >= S || bulk_seg_begin(n, S, g) > c || bulk_seg_begin(n, S, g + 1) <= c) ++bad;
      }
    }
  printf("%lld %d %d %d %d %d\n", bad, kBulkSegs, bulk_segs(10320, 148, 4), bulk_segs(5160, 148, 4), bulk_segs(2580, 148, 4),
         bulk_segs(10320, 148, 1));
  return 0;
}
""")
    exe = tmp_path / "segcheck"
    subprocess.run([nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I", csrc, "-o", str(exe), str(src)],
                   check=True, capture_output=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert out[0] == "0", f"{out[0]} chunks fall outside the segment the helpers name"
    assert int(out[1]) == SEGS
    # 84.5 MB, 42 MB and 21 MB shards moved by 148 CTAs: 4, 2 and 1 segments; a cap of 1 gives per-shard counters
    assert [int(v) for v in out[2:]] == [4, 2, 1, 1]
