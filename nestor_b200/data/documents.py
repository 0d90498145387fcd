"""Documents inside an end-of-text-separated flat token stream, and the tokenizer side that writes one.

Reading: ``document_spans`` recovers ``[start, end)`` spans (end = the end-of-text position) by
scanning the stream in chunks; ``select_documents`` filters by length; ``load_document`` copies one
out. Writing: worker-initialised tiktoken encoding with per-document min/max token filters,
``.meta.json`` sidecars, and text iteration over parquet / jsonl(.gz|.zst) / txt inputs.
Behavioural parity with ``nestor/data/token_documents.py`` of the reference. No torch import —
the preprocessing scripts run on CPU-only nodes.
"""

from __future__ import annotations

import gzip
import io
import json
from collections.abc import Iterator
from pathlib import Path
from typing import Any

import numpy as np

DEFAULT_EOT = 100257  # cl100k_base end-of-text id


def read_bin_meta(bin_path: Path) -> dict[str, Any]:
    side = Path(f"{bin_path}.meta.json")
    return json.loads(side.read_text()) if side.is_file() else {}


def open_token_bin(bin_path: Path) -> tuple[np.memmap, int]:
    """Memory-map a token file; dtype and end-of-text id come from the sidecar (uint32 / cl100k otherwise)."""

    meta = read_bin_meta(bin_path)
    dtype = np.uint16 if meta.get("token_dtype") == "uint16" else np.uint32
    return np.memmap(bin_path, dtype=dtype, mode="r"), int(meta.get("eot_token", DEFAULT_EOT))


def document_spans(tokens: np.ndarray, eot_token: int, chunk_tokens: int = 1 << 28) -> np.ndarray:
    """``[num_docs, 2]`` int64 spans; a trailing run without a terminator is not a document."""

    begins, ends = [], []
    next_start = 0
    for base in range(0, len(tokens), chunk_tokens):
        hits = np.flatnonzero(np.asarray(tokens[base : base + chunk_tokens]) == eot_token).astype(np.int64) + base
        if hits.size == 0:
            continue
        begins.append(np.concatenate(([next_start], hits[:-1] + 1)))
        ends.append(hits)
        next_start = int(hits[-1]) + 1
    if not begins:
        return np.zeros((0, 2), dtype=np.int64)
    return np.stack((np.concatenate(begins), np.concatenate(ends)), axis=1)


def select_documents(spans: np.ndarray, *, min_tokens: int = 1, max_docs: int | None = None) -> np.ndarray:
    keep = spans[(spans[:, 1] - spans[:, 0]) >= max(min_tokens, 1)]
    return keep if max_docs is None else keep[:max_docs]


def load_document(tokens: np.ndarray, span: np.ndarray, *, max_tokens: int | None = None) -> np.ndarray:
    a, b = int(span[0]), int(span[1])
    if max_tokens is not None:
        b = min(b, a + max_tokens)
    return np.array(tokens[a:b], dtype=np.int64, copy=True)


# ------------------------------------------------------------------------ tokenizer side
_ENCODING: Any = None
_MIN_TOKENS = 0
_MAX_TOKENS: int | None = None


class _ByteEncoding:
    """``--tokenizer bytes``: UTF-8 bytes as ids 0..255 and 256 as end-of-text. Needs no vocabulary file, so the
    preprocessing tools also run on machines without network access (tests, smoke corpora)."""

    eot_token = 256

    def encode_ordinary_batch(self, texts: list[str]) -> list[list[int]]:
        return [list(t.encode("utf-8")) for t in texts]


def load_encoding(tokenizer_name: str) -> Any:
    """The tiktoken encoding of that name, or the byte-level stand-in for ``"bytes"``."""

    if tokenizer_name == "bytes":
        return _ByteEncoding()
    import tiktoken
    return tiktoken.get_encoding(tokenizer_name)


def init_tokenizer_worker(tokenizer_name: str, min_doc_tokens: int = 0, max_doc_tokens: int | None = None) -> None:
    """Pool initialiser: load the encoding once per worker process and set the length filter."""

    global _ENCODING, _MIN_TOKENS, _MAX_TOKENS
    _ENCODING = load_encoding(tokenizer_name)
    _MIN_TOKENS, _MAX_TOKENS = int(min_doc_tokens), max_doc_tokens


def encode_documents(texts: list[str]) -> tuple[np.ndarray, int]:
    """Encode a batch of documents to one uint32 stream, each kept document followed by end-of-text."""

    assert _ENCODING is not None, "call init_tokenizer_worker first"
    eot = _ENCODING.eot_token
    stream: list[int] = []
    kept = 0
    for ids in _ENCODING.encode_ordinary_batch(texts):
        if _MAX_TOKENS is not None:
            ids = ids[:_MAX_TOKENS]
        if len(ids) < max(_MIN_TOKENS, 1):
            continue
        stream.extend(ids)
        stream.append(eot)
        kept += 1
    return np.asarray(stream, dtype=np.uint32), kept


def write_bin_meta(bin_path: Path, *, num_tokens: int, num_docs: int, tokenizer_name: str,
                   extra: dict[str, Any] | None = None, eot_token: int | None = None) -> None:
    if eot_token is None:
        eot_token = load_encoding(tokenizer_name).eot_token
    meta: dict[str, Any] = {"token_dtype": "uint32", "num_tokens": int(num_tokens), "num_docs": int(num_docs),
                            "tokenizer": tokenizer_name, "eot_token": int(eot_token)}
    meta.update(extra or {})
    Path(f"{bin_path}.meta.json").write_text(json.dumps(meta, indent=2))


def iter_document_texts(path: Path, text_key: str = "text") -> Iterator[str]:
    """Yield document texts from ``.parquet``, ``.jsonl`` (optionally ``.gz`` / ``.zst``), ``.json.gz`` or ``.txt``."""

    name = path.name
    if name.endswith(".parquet"):
        import pyarrow.parquet as pq
        for batch in pq.ParquetFile(path).iter_batches(batch_size=256, columns=[text_key]):
            yield from (t for t in batch.column(0).to_pylist() if t)
        return
    if name.endswith(".txt"):
        text = path.read_text(encoding="utf-8", errors="replace")
        if text:
            yield text
        return
    if not name.endswith((".jsonl", ".jsonl.gz", ".json.gz", ".jsonl.zst")):
        raise ValueError(f"unsupported input type: {path}")
    if name.endswith(".gz"):
        handle: Any = gzip.open(path, "rt", encoding="utf-8")
    elif name.endswith(".zst"):
        try:
            import zstandard as zstd
            raw: Any = zstd.ZstdDecompressor().stream_reader(open(path, "rb"))
        except ImportError:
            # no zstandard package: Arrow ships the same codec and reads the stream as well
            import pyarrow as pa
            raw = pa.CompressedInputStream(pa.OSFile(str(path), "rb"), "zstd")
        handle = io.TextIOWrapper(raw, encoding="utf-8")
    else:
        handle = open(path, encoding="utf-8")
    with handle:
        for line in handle:
            line = line.strip()
            if not line:
                continue
            try:
                text = json.loads(line).get(text_key)
            except json.JSONDecodeError:
                continue
            if text:
                yield text
