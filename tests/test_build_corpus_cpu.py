"""The corpus builder writes what the mmap reader reads: plain text, question / answer data with a loss mask,
synthetic ids, and rows of a mixture file."""
import json

import numpy as np
import pytest

from ksa_b200.data import KaiMMapDataset, MMapDataset
from ksa_b200.data.mmap_dataset import loss_mask_file_path, parse_data_prefix
from ksa_b200.tools.build_corpus import (ByteTokenizer, CorpusWriter, append_to_mix_file, build_from_documents,
                                         build_synthetic, iter_documents, main)


def test_text_lines_round_trip_through_the_reader(tmp_path):
    src = tmp_path / "web.txt"
    lines = ["hello world", "", "zweite Zeile: äöü", "third"]
    src.write_text("\n".join(lines) + "\n", encoding="utf-8")
    info = main(["--input", str(src), "--output-prefix", str(tmp_path / "data" / "web"), "--tokenizer", "bytes"])
    tok = ByteTokenizer()
    want = []
    for l in lines:
        if l:
            want += tok.encode(l) + [tok.eos_token_id]
    assert info == {"prefix": str(tmp_path / "data" / "web"), "dtype": "uint16", "tokens": len(want), "documents": 3,
                    "loss_mask": False}
    ds = MMapDataset(info["prefix"], 8)
    assert not ds.is_qa_dataset and ds.size == len(want)
    got = np.concatenate([ds[i]["text"][:8] for i in range(len(ds))])
    assert got.tolist() == want[:len(got)]
    assert tok.decode(want[:11]) == "hello world"


def test_question_answer_lines_carry_a_loss_mask(tmp_path):
    src = tmp_path / "qa.jsonl"
    rows = [{"q": "2+2=", "a": "4"}, {"q": "capital of France? ", "a": "Paris"}]
    src.write_text("".join(json.dumps(r) + "\n" for r in rows))
    prefix = str(tmp_path / "qa")
    info = main(["--input", str(src), "--output-prefix", prefix, "--prompt-key", "q", "--answer-key", "a"])
    assert info["loss_mask"] and info["documents"] == 2
    tokens = np.fromfile(prefix + ".bin", dtype=np.uint16)
    mask = np.fromfile(loss_mask_file_path(prefix), dtype=np.uint16)
    assert tokens.shape == mask.shape
    want_mask = []
    for r in rows:
        want_mask += [0] * len(r["q"].encode()) + [1] * (len(r["a"].encode()) + 1)     # answer + end of document
    assert mask.tolist() == want_mask
    ds = MMapDataset(prefix, 4)
    assert ds.is_qa_dataset and ds[0]["text"].shape == (8,)          # tokens || mask
    # rewriting the same prefix without answers removes the stale mask file
    build_from_documents([("plain", None)], ByteTokenizer(), prefix)
    assert not MMapDataset(prefix, 2).is_qa_dataset
    with pytest.raises(ValueError):
        build_from_documents([("a", "b"), ("c", None)], ByteTokenizer(), str(tmp_path / "mixed"))
    (tmp_path / "plain.txt").write_text("x\n")
    with pytest.raises(ValueError):                                  # question / answer mode needs JSON lines
        list(iter_documents([str(tmp_path / "plain.txt")], prompt_key="q", answer_key="a"))


def test_synthetic_corpus_dtype_follows_the_vocabulary_and_ids_are_checked(tmp_path):
    small = build_synthetic(str(tmp_path / "s"), 1000, 5000, seed=1)
    big = build_synthetic(str(tmp_path / "b"), 1000, 151936, seed=1)
    assert small["dtype"] == "uint16" and big["dtype"] == "uint32"
    ids = np.fromfile(str(tmp_path / "b.bin"), dtype=np.uint32)
    assert ids.size == 1000 and ids.max() < 151936 and ids.max() > 65535
    again = build_synthetic(str(tmp_path / "b2"), 1000, 151936, seed=1)
    assert again["tokens"] == 1000 and np.array_equal(ids, np.fromfile(str(tmp_path / "b2.bin"), dtype=np.uint32))
    with CorpusWriter(str(tmp_path / "w"), "uint16") as w:
        with pytest.raises(ValueError):
            w.add([70000])
        w.add(range(10))
        w.add([], None)
    assert np.fromfile(str(tmp_path / "w.bin"), dtype=np.uint16).tolist() == list(range(10))
    # many small documents cross the write buffer
    with CorpusWriter(str(tmp_path / "m"), "uint32", buffer_tokens=7) as w:
        for i in range(50):
            w.add([i, i + 1, i + 2])
    assert np.fromfile(str(tmp_path / "m.bin"), dtype=np.uint32).size == 150


def test_mixture_file_rows_feed_the_blended_dataset(tmp_path):
    mix = str(tmp_path / "mix.txt")
    for name, weight, n in (("web", 0.7, 64 * 30 + 1), ("code", 0.3, 64 * 20 + 1)):
        main(["--synthetic", str(n), "--vocab-size", "300", "--output-prefix", str(tmp_path / name),
              "--mix-file", mix, "--weight", str(weight), "--domain", name])
    append_to_mix_file(mix, str(tmp_path / "web"), 0.6, "web")               # replaces the row, keeps one per prefix
    flat, domains = parse_data_prefix(mix)
    assert [float(flat[0]), flat[1], float(flat[2]), flat[3]] == [0.3, str(tmp_path / "code"), 0.6, str(tmp_path / "web")]
    assert domains == {str(tmp_path / "code"): "code", str(tmp_path / "web"): "web"}
    with pytest.raises(ValueError):
        append_to_mix_file(mix, str(tmp_path / "x"), 1.0)                     # two columns into a three-column file
    ds = KaiMMapDataset(data_prefix=mix, seq_length=64, seed=7, global_batch_size=2)
    batch = next(iter(ds))
    assert batch["input_ids"].shape[-1] == 64 and int(batch["input_ids"].max()) < 300
