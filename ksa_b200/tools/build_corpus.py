"""Build a pre-tokenised corpus in the on-disk format that ``MMapDataset`` reads.

The reference ships the reader (``muse/data/datasets/kai_mmap.py:44-147``), the ``.bin.meta`` files of its corpora and
a mixture file (``data/train_data_list_8k.txt``) but no writer; this tool is the missing half.

    <prefix>.bin             token ids, back to back, in ``<dtype>``
    <prefix>.bin.meta        the numpy dtype name (``uint16`` / ``uint32``)
    <prefix>_loss_mask.bin   optional, same length and dtype: 1 where a token is trained on (question / answer data)

Examples::

    # plain text, one document per line, tokenised with a local Hugging Face tokenizer directory
    python -m ksa_b200.tools.build_corpus --input web.txt --tokenizer /models/qwen3 --output-prefix data/web \
        --mix-file data/train_data_list_8k.txt --domain common_knowledge --weight 0.45

    # JSON lines with question / answer fields: the question is context only (loss mask 0)
    python -m ksa_b200.tools.build_corpus --input qa.jsonl --prompt-key question --answer-key answer \
        --tokenizer /models/qwen3 --output-prefix data/qa

    # uniform-random ids (benchmarks, smoke runs)
    python -m ksa_b200.tools.build_corpus --synthetic 10000000 --vocab-size 151936 --output-prefix data/random

Documents are streamed: nothing larger than one write buffer is held in memory.
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Callable, Iterable, Iterator, List, Optional, Sequence, Tuple

import numpy as np

from ..data.mmap_dataset import data_file_path, loss_mask_file_path, meta_file_path

__all__ = ["ByteTokenizer", "CorpusWriter", "build_from_documents", "build_synthetic", "append_to_mix_file", "main"]


class ByteTokenizer:
    """UTF-8 bytes as token ids 0..255 and 256 as end of document: a tokenizer for tests and for machines without
    one (``--tokenizer bytes``)."""

    eos_token_id = 256
    vocab_size = 257

    def encode(self, text: str) -> List[int]:
        return list(text.encode("utf-8"))

    def decode(self, ids: Sequence[int]) -> str:
        return bytes(i for i in ids if i < 256).decode("utf-8", errors="replace")


def load_tokenizer(spec: str):
    """``bytes`` or a local directory with Hugging Face tokenizer files."""
    if spec == "bytes":
        return ByteTokenizer()
    from transformers import AutoTokenizer
    return AutoTokenizer.from_pretrained(spec, local_files_only=True, trust_remote_code=False)


def _encode(tokenizer, text: str) -> List[int]:
    if isinstance(tokenizer, ByteTokenizer):
        return tokenizer.encode(text)
    return tokenizer.encode(text, add_special_tokens=False)


class CorpusWriter:
    """Appends token ids (and, once a mask has been given, loss-mask values) to ``<prefix>.bin``; ``close`` writes
    the meta file.  ``dtype`` None picks ``uint16`` when ``vocab_size`` fits, else ``uint32``."""

    def __init__(self, prefix: str, dtype: Optional[str] = None, vocab_size: Optional[int] = None,
                 with_loss_mask: bool = False, buffer_tokens: int = 1 << 22):
        if dtype is None:
            dtype = "uint16" if vocab_size is not None and vocab_size <= 1 << 16 else "uint32"
        if dtype not in ("uint16", "uint32", "int32", "int64"):
            raise ValueError(f"unsupported corpus dtype {dtype!r}")
        self.prefix, self.dtype = prefix, dtype
        self._np = np.dtype(getattr(np, dtype))
        self._limit = int(np.iinfo(self._np).max)
        os.makedirs(os.path.dirname(os.path.abspath(prefix)) or ".", exist_ok=True)
        self._tok = open(data_file_path(prefix), "wb")
        self._mask = open(loss_mask_file_path(prefix), "wb") if with_loss_mask else None
        if not with_loss_mask and os.path.exists(loss_mask_file_path(prefix)):
            os.remove(loss_mask_file_path(prefix))       # a stale mask would turn the corpus into a QA corpus
        self._buf: List[np.ndarray] = []
        self._mbuf: List[np.ndarray] = []
        self._buffered = 0
        self._buffer_tokens = buffer_tokens
        self.tokens = 0
        self.documents = 0

    def add(self, ids: Sequence[int], loss_mask: Optional[Sequence[int]] = None) -> None:
        a = np.asarray(ids, dtype=np.int64)
        if a.size == 0:
            return
        if a.min() < 0 or a.max() > self._limit:
            raise ValueError(f"token id outside the range of {self.dtype}: [{a.min()}, {a.max()}]")
        if (loss_mask is not None) != (self._mask is not None):
            raise ValueError("a corpus either has a loss mask for every document or for none")
        self._buf.append(a.astype(self._np))
        if loss_mask is not None:
            m = np.asarray(loss_mask, dtype=np.int64)
            if m.shape != a.shape:
                raise ValueError("loss mask and tokens differ in length")
            self._mbuf.append(m.astype(self._np))
        self._buffered += a.size
        self.tokens += a.size
        self.documents += 1
        if self._buffered >= self._buffer_tokens:
            self._flush()

    def _flush(self) -> None:
        if self._buf:
            np.concatenate(self._buf).tofile(self._tok)
        if self._mbuf:
            np.concatenate(self._mbuf).tofile(self._mask)
        self._buf, self._mbuf, self._buffered = [], [], 0

    def close(self) -> dict:
        self._flush()
        self._tok.close()
        if self._mask is not None:
            self._mask.close()
        with open(meta_file_path(self.prefix), "w") as f:
            f.write(self.dtype)
        return {"prefix": self.prefix, "dtype": self.dtype, "tokens": self.tokens, "documents": self.documents,
                "loss_mask": self._mask is not None}

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        if not self._tok.closed:
            self.close()


def iter_documents(paths: Iterable[str], text_key: Optional[str] = "text", prompt_key: Optional[str] = None,
                   answer_key: Optional[str] = None) -> Iterator[Tuple[str, Optional[str]]]:
    """``(text, None)`` per document, or ``(prompt, answer)`` in question / answer mode.  ``.jsonl`` / ``.json``
    files hold one JSON object per line; any other file is plain text with one document per non-empty line."""
    for path in paths:
        is_json = path.endswith((".jsonl", ".json"))
        with open(path, encoding="utf-8") as f:
            for n, line in enumerate(f, 1):
                line = line.rstrip("\n")
                if not line.strip():
                    continue
                if not is_json:
                    if prompt_key or answer_key:
                        raise ValueError("question / answer mode needs JSON lines input")
                    yield line, None
                    continue
                try:
                    obj = json.loads(line)
                except json.JSONDecodeError as e:
                    raise ValueError(f"{path}:{n}: not a JSON object: {e}") from None
                if prompt_key and answer_key:
                    yield str(obj[prompt_key]), str(obj[answer_key])
                else:
                    yield str(obj[text_key]), None


def build_from_documents(docs: Iterable[Tuple[str, Optional[str]]], tokenizer, prefix: str, dtype: Optional[str] = None,
                         append_eos: bool = True, progress: Optional[Callable[[int, int], None]] = None) -> dict:
    """Tokenise ``docs`` into ``prefix``.  A document with an answer part gets loss mask 0 on its prompt tokens and 1
    on its answer tokens (end-of-document included); the corpus then carries ``<prefix>_loss_mask.bin``."""
    eos = getattr(tokenizer, "eos_token_id", None)
    if append_eos and eos is None:
        raise ValueError("the tokenizer has no end-of-document token; pass append_eos=False")
    vocab = getattr(tokenizer, "vocab_size", None)
    try:
        vocab = max(int(vocab or 0), len(tokenizer))     # added special tokens sit above vocab_size
    except TypeError:
        pass
    it = iter(docs)
    first = next(it, None)
    if first is None:
        raise ValueError("no documents")
    qa = first[1] is not None
    with CorpusWriter(prefix, dtype, vocab, with_loss_mask=qa) as w:
        def one(doc):
            text, answer = doc
            if qa != (answer is not None):
                raise ValueError("documents with and without an answer part cannot share a corpus")
            ids = _encode(tokenizer, text)
            if not qa:
                w.add(ids + ([eos] if append_eos else []))
                return
            ans = _encode(tokenizer, answer) + ([eos] if append_eos else [])
            w.add(ids + ans, [0] * len(ids) + [1] * len(ans))
        one(first)
        for doc in it:
            one(doc)
            if progress is not None and w.documents % 10000 == 0:
                progress(w.documents, w.tokens)
        return w.close()


def build_synthetic(prefix: str, n_tokens: int, vocab_size: int, seed: int = 0, dtype: Optional[str] = None) -> dict:
    """Uniform-random token ids, written in blocks."""
    rng = np.random.default_rng(seed)
    with CorpusWriter(prefix, dtype, vocab_size) as w:
        left = int(n_tokens)
        while left > 0:
            n = min(left, 1 << 24)
            w.add(rng.integers(0, vocab_size, n))
            left -= n
        return w.close()


def append_to_mix_file(mix_file: str, prefix: str, weight: float, domain: Optional[str] = None) -> None:
    """Add (or replace) the row of ``prefix`` in a mixture file: ``domain<TAB>weight<TAB>prefix`` (three columns, as
    ``data/train_data_list_8k.txt`` of the reference) or ``weight<TAB>prefix``."""
    rows: List[List[str]] = []
    if os.path.exists(mix_file):
        with open(mix_file) as f:
            rows = [r.split() for r in f.read().splitlines() if r.strip()]
    cols = 3 if domain is not None else 2
    if any(len(r) != cols for r in rows):
        raise ValueError(f"{mix_file} has rows of a different shape than the new one ({cols} columns)")
    rows = [r for r in rows if r[-1] != prefix]
    rows.append(([domain] if domain is not None else []) + [repr(float(weight)), prefix])
    os.makedirs(os.path.dirname(os.path.abspath(mix_file)) or ".", exist_ok=True)
    with open(mix_file, "w") as f:
        f.write("".join("\t".join(r) + "\n" for r in rows))


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", nargs="*", default=[], help="text files (a document per line) or .jsonl files")
    ap.add_argument("--output-prefix", required=True)
    ap.add_argument("--tokenizer", default="bytes", help="'bytes' or a local directory with tokenizer files")
    ap.add_argument("--json-key", default="text")
    ap.add_argument("--prompt-key", default=None)
    ap.add_argument("--answer-key", default=None)
    ap.add_argument("--no-eos", action="store_true", help="do not append the end-of-document token")
    ap.add_argument("--dtype", default=None, choices=["uint16", "uint32"])
    ap.add_argument("--synthetic", type=int, default=0, help="write this many uniform-random ids instead of reading input")
    ap.add_argument("--vocab-size", type=int, default=151936)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--mix-file", default=None, help="mixture file to add the corpus to")
    ap.add_argument("--weight", type=float, default=1.0)
    ap.add_argument("--domain", default=None)
    a = ap.parse_args(argv)
    if bool(a.prompt_key) != bool(a.answer_key):
        ap.error("--prompt-key and --answer-key go together")
    if a.synthetic:
        info = build_synthetic(a.output_prefix, a.synthetic, a.vocab_size, a.seed, a.dtype)
    else:
        if not a.input:
            ap.error("--input or --synthetic is required")
        tok = load_tokenizer(a.tokenizer)
        docs = iter_documents(a.input, a.json_key, a.prompt_key, a.answer_key)
        info = build_from_documents(docs, tok, a.output_prefix, a.dtype, append_eos=not a.no_eos,
                                    progress=lambda d, t: print(f"[build_corpus] {d} documents, {t} tokens", flush=True))
    if a.mix_file:
        append_to_mix_file(a.mix_file, a.output_prefix, a.weight, a.domain)
    print(json.dumps(info))
    return info


if __name__ == "__main__":
    main()
