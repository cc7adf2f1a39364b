"""Parquet pipeline: sharding covers every row exactly once, shuffling is reproducible, packing and resume work."""
import pyarrow as pa
import pyarrow.parquet as pq
import pytest

from ksa_b200.data import DistributedParquetDataset, ParquetReader, ShuffledParquetReader


def _files(tmp_path, n_files=4, rows=25):
    k = 0
    for f in range(n_files):
        ids = [[k + i, k + i, k + i] for i in range(rows)]
        pq.write_table(pa.table({"uid": list(range(k, k + rows)), "input_ids": ids}), tmp_path / f"part{f}.parquet")
        k += rows
    return str(tmp_path), n_files * rows


def test_readers(tmp_path):
    d, n = _files(tmp_path)
    rows = list(ParquetReader(d))
    assert [r["uid"] for r in rows] == list(range(n)) and rows[30]["__index__"] == 5 and rows[0]["__total__"] == 25
    a = [r["uid"] for r in ShuffledParquetReader(d, buffer_size=16, seed=3)]
    b = [r["uid"] for r in ShuffledParquetReader(d, buffer_size=16, seed=3)]
    assert a == b and sorted(a) == list(range(n)) and a != list(range(n))


@pytest.mark.parametrize("shard_by", ["file", "sample"])
def test_shards_partition_the_data_and_resume(tmp_path, shard_by):
    d, n = _files(tmp_path)
    seen = []
    for r in range(2):
        ds = DistributedParquetDataset(d, rank=r, world_size=2, shard_by=shard_by, seed=1, shuffle_buffer_size=8)
        seen.append([s["uid"] for s in ds])
    assert sorted(seen[0] + seen[1]) == list(range(n)) and not set(seen[0]) & set(seen[1])
    ds = DistributedParquetDataset(d, rank=0, world_size=2, shard_by=shard_by, seed=1, shuffle_buffer_size=8)
    it = iter(ds)
    first = [next(it)["uid"] for _ in range(7)]
    state = ds.state_dict()
    rest = [s["uid"] for s in it]
    ds2 = DistributedParquetDataset(d, rank=0, world_size=2, shard_by=shard_by, seed=1, shuffle_buffer_size=8)
    ds2.load_state_dict(state)
    assert [s["uid"] for s in ds2] == rest and first + rest == seen[0]


def test_process_hook_and_packing(tmp_path):
    d, n = _files(tmp_path, n_files=2, rows=10)
    ds = DistributedParquetDataset(d, shuffle=False, pack_to=8,
                                   process=lambda r: None if r["uid"] % 2 else {"input_ids": r["input_ids"]})
    out = list(ds)
    assert all(s["input_ids"].shape == (1, 8) for s in out) and len(out) == (10 * 3) // 8
    assert out[0]["input_ids"][0].tolist() == [0, 0, 0, 2, 2, 2, 4, 4] and out[0]["cu_seqlens"].tolist() == [0, 3, 6, 8]
    with pytest.raises(ValueError):
        list(DistributedParquetDataset(d, rank=0, world_size=4, shard_by="file"))


def test_image_buckets_and_resolution_budgets():
    """Aspect-ratio / resolution helpers of the image branch of the parquet pipeline (``muse/data/utils.py:90-252``)."""
    from ksa_b200.data.image_buckets import (BucketBatcher, aspect_ratio_buckets, closest_ratio, closest_size,
                                             parse_resolution_budgets, resolution_level)
    for size in (256, 512, 1024, 2048):
        b = aspect_ratio_buckets(size)
        assert b["1.0"] == (size, size)
        assert min(float(k) for k in b) == 0.25 and max(float(k) for k in b) == 4.0
        for k, (h, w) in b.items():
            assert h % (size // 16) == 0 and w % (size // 16) == 0
            assert 0.75 * size * size < h * w <= size * size
            assert abs(float(k) - h / w) < 0.006
            assert (w, h) in b.values()                               # portrait and landscape mirror each other
    assert aspect_ratio_buckets(256)["0.25"] == (128, 512) and aspect_ratio_buckets(256)["4.0"] == (512, 128)
    assert aspect_ratio_buckets(300) == aspect_ratio_buckets(512)     # between two levels: the next one up
    big = aspect_ratio_buckets(4096)
    assert big["1.0"] == (4096, 4096) and big["0.25"] == (2048, 8192)
    # the reference's examples for the level of an image
    assert resolution_level(512, 512) == 512 and resolution_level(1024, 1024) == 1024
    assert resolution_level(768, 1280) == 768 and resolution_level(256, 1024) == 512 and resolution_level(200, 200) == 256
    assert resolution_level(900, 900, [512, 1024]) == 512
    b512 = aspect_ratio_buckets(512)
    assert closest_ratio(480, 640, b512) == "0.76" or abs(float(closest_ratio(480, 640, b512)) - 0.75) < 0.04
    h, w = closest_size(1080, 1920, b512)
    assert abs(h / w - 1080 / 1920) < 0.04 and h * w <= 512 * 512
    cfg = parse_resolution_budgets("512:3, 1024:2")
    assert cfg.levels == [512, 1024] and cfg.batch_size(1024) == 2
    with pytest.raises(ValueError):
        parse_resolution_budgets("512")
    batcher = BucketBatcher(cfg)
    out = [batcher.add(i, 600, 600) for i in range(3)]                # level 512, square bucket, batch of 3
    assert out[:2] == [None, None] and out[2] == (512, (512, 512), [0, 1, 2])
    assert batcher.add("wide", 800, 1600) is None and batcher.add("tall", 1600, 800) is None
    assert batcher.add("wide2", 810, 1590)[2] == ["wide", "wide2"]    # level 1024, batch of 2, same bucket
    assert [g for _, _, g in batcher.flush()] == [["tall"]] and batcher.flush() == []
