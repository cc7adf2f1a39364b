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
