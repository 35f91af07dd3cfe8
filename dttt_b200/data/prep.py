"""Building and indexing token streams: ``python -m dttt_b200.data {prepare,prepare_grouped,filter,unigram,stats,windows,synth}``.

A stream is a directory ``{name}_{hash16}`` holding ``tokens.u32`` (little-endian uint32, every document followed by
one EOS) and ``meta.json``; the names, the hash inputs and the meta keys are those of the reference's data CLI
(``src/ttt/data.py:5-24,195-515``), so streams written by either implementation are interchangeable.

The code is organised around three small objects instead of one function per sub-command:

``DocumentFeed``   where documents come from, as an iterator of *units* (a unit is a list of documents that is admitted or
                   dropped as a whole: a single document, or all files of a repository).  ``ParquetRows`` yields one-document
                   units row group by row group with the next row group read ahead on a thread; ``ParquetGroups`` sorts the
                   rows by a key and yields one unit per key.  Anything iterable over lists of strings can stand in.
``EncoderPool``    tokenises batches of units on worker processes and returns them in submission order, so the bytes on
                   disk do not depend on the worker count.
``StreamSink``     the output: a local file written under a temporary name and renamed when complete, or, under a gcsfuse
                   mount, a resumable upload straight to the bucket (``src/ttt/data.py:98-143``: the mount would stage the
                   whole file on the local disk first).

``StreamIndex`` answers questions about a finished stream (document lengths, training windows, unigram counts, length
tables, filtered copies).
"""
from __future__ import annotations

import contextlib
import hashlib
import html
import json
import os
import re
import time
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import numpy as np

Unit = List[str]


# ------------------------------------------------------------------------------------------------ identity of a stream
def tokenizer_fingerprint(tok) -> Dict[str, object]:
    opt = lambda v: None if v is None else int(v)
    return {"class": type(tok).__name__, "len": int(len(tok)), "vocab_size": int(getattr(tok, "vocab_size", -1)),
            "eos_token_id": opt(tok.eos_token_id), "bos_token_id": opt(tok.bos_token_id)}


def source_hash(files: Sequence[str], fp: Dict[str, object], min_doc_tokens: int, bos: bool, clean: str = "") -> str:
    """16 hex digits over (absolute path and size of every input file, tokenizer fingerprint, admission rule)."""
    h = hashlib.sha256()
    for path in sorted(map(os.path.abspath, files)):
        h.update(path.encode() + str(os.path.getsize(path)).encode())
    h.update(json.dumps(fp, sort_keys=True).encode())
    h.update(f"min_doc_tokens={min_doc_tokens};bos={bos};sep=eos".encode() + (f";clean={clean}".encode() if clean else b""))
    return h.hexdigest()[:16]


_CLEANERS: Dict[str, Callable[[str], str]] = {
    "": lambda s: s,
    "html": lambda s: re.sub(r"\n{3,}", "\n\n", re.sub(r"<[^>]{1,200}>", "", html.unescape(s))),
}


def clean_text(text: str, mode: str) -> str:
    try:
        return _CLEANERS[mode](text)
    except KeyError:
        raise ValueError(f"unknown clean mode {mode!r}") from None


# ------------------------------------------------------------------------------------------------ output
def bucket_object(path: str, mounts_file: str = "/proc/mounts") -> Optional[Tuple[str, str]]:
    """``(bucket, object name)`` when ``path`` lies under a gcsfuse mount (a ``fuse`` file system whose source is a bare
    bucket name), else ``None``.  The deepest matching mount wins."""
    target = os.path.abspath(path)
    try:
        with open(mounts_file) as fh:
            rows = [ln.split() for ln in fh]
    except OSError:
        return None
    hits = [(mnt, src) for src, mnt, kind, *_ in (r for r in rows if len(r) >= 3)
            if kind == "fuse" and not set(src) & {"/", ":"} and (target == mnt or target.startswith(mnt.rstrip("/") + "/"))]
    if not hits:
        return None
    mnt, src = max(hits, key=lambda h: len(h[0]))
    return src, target[len(mnt.rstrip("/")) + 1:]


def _bucket_client():
    from google.cloud import storage
    return storage.Client()


class StreamSink:
    """A binary output that appears under its final name only when complete.  ``client`` (anything with the
    ``google.cloud.storage.Client`` interface) is looked up lazily and only for paths under a gcsfuse mount."""

    def __init__(self, path: str, client=None, mounts_file: str = "/proc/mounts", upload_chunk: int = 64 << 20):
        self.path, self.where = path, bucket_object(path, mounts_file)
        self._client, self._chunk = client, upload_chunk
        self._fh = self._tmp_blob = None
        self.bytes = 0

    def _blob(self, name: str):
        self._client = self._client or _bucket_client()
        return self._client.bucket(self.where[0]).blob(name)

    def exists(self) -> bool:
        """Existence that does not go through the mount's (negative) stat cache."""
        return self._blob(self.where[1]).exists() if self.where else os.path.exists(self.path)

    def __enter__(self) -> "StreamSink":
        if self.where:
            self._tmp_blob = self._blob(self.where[1] + ".tmp")
            self._fh = self._tmp_blob.open("wb", chunk_size=self._chunk, ignore_flush=True)
        else:
            os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)
            self._fh = open(self.path + ".tmp", "wb")
        return self

    def write(self, data) -> None:
        b = data if isinstance(data, (bytes, bytearray, memoryview)) else np.ascontiguousarray(data, dtype="<u4").tobytes()
        self._fh.write(b)
        self.bytes += len(b)

    def __exit__(self, exc_type, exc, tb) -> None:
        self._fh.close()
        if self.where:
            if exc_type is None:
                final = self._blob(self.where[1])
                token = None
                while True:                                       # server-side copy of any size, then drop the temporary object
                    token, _, _ = final.rewrite(self._tmp_blob, token=token) if token else final.rewrite(self._tmp_blob)
                    if token is None:
                        break
            with contextlib.suppress(Exception):
                self._tmp_blob.delete()
        elif exc_type is None:
            os.replace(self.path + ".tmp", self.path)
        else:
            with contextlib.suppress(OSError):
                os.remove(self.path + ".tmp")


@contextlib.contextmanager
def atomic_output(path: str):
    """A ``StreamSink`` as a plain context manager yielding something with ``write``."""
    with StreamSink(path) as sink:
        yield sink


def _write_json(path: str, obj: dict) -> None:
    with StreamSink(path) as sink:
        sink.write(json.dumps(obj, indent=2).encode())


# ------------------------------------------------------------------------------------------------ where documents come from
class ParquetRows:
    """Every row of ``files`` is a document and its own unit.  Row groups are read in file order; while one is being
    tokenised the next is read on a thread (``pre_buffer`` and a 64 MiB buffer make that a few large reads)."""

    def __init__(self, files: Sequence[str], text_key: str, clean: str = ""):
        import pyarrow.parquet as pq
        self.handles = [pq.ParquetFile(p, pre_buffer=True, buffer_size=64 << 20) for p in files]
        self.slots = [(h, g) for h in self.handles for g in range(h.num_row_groups)]
        self.text_key, self.clean = text_key, clean

    def __len__(self) -> int:
        return len(self.slots)

    def _load(self, slot) -> List[Unit]:
        handle, group = slot
        column = handle.read_row_group(group, columns=[self.text_key])[self.text_key].to_pylist()
        return [[clean_text(t, self.clean)] for t in column]

    def __iter__(self) -> Iterator[List[Unit]]:
        from concurrent.futures import ThreadPoolExecutor
        if not self.slots:
            return
        with ThreadPoolExecutor(1) as reader:
            ahead = reader.submit(self._load, self.slots[0])
            for nxt in self.slots[1:] + [None]:
                units = ahead.result()
                ahead = reader.submit(self._load, nxt) if nxt is not None else None
                yield units


class ParquetGroups:
    """Rows sharing ``group_key`` form one unit (e.g. the files of one repository), ordered by ``order_key`` inside it;
    groups come in key order.  Everything is read and sorted in memory first."""

    def __init__(self, files: Sequence[str], text_key: str, group_key: str, order_key: str):
        import pyarrow as pa
        import pyarrow.compute as pc
        import pyarrow.parquet as pq
        # large_string: the offsets of an ordinary string column overflow at 2 GB once the files are concatenated
        layout = pa.schema([(group_key, pa.string()), (order_key, pa.string()), (text_key, pa.large_string())])
        rows = pa.concat_tables([pq.read_table(p, columns=layout.names, pre_buffer=True).cast(layout) for p in files])
        rows = rows.sort_by([(group_key, "ascending"), (order_key, "ascending")])
        keys = rows.column(group_key).combine_chunks()
        if len(keys):
            changed = pc.not_equal(keys.slice(1), keys.slice(0, len(keys) - 1)).to_numpy(zero_copy_only=False)
            self.edges = np.concatenate([[0], np.flatnonzero(changed) + 1, [len(keys)]])
        else:
            self.edges = np.zeros(1, np.int64)
        self.texts = rows.column(text_key)

    def __len__(self) -> int:
        return 1

    def __iter__(self) -> Iterator[List[Unit]]:
        yield (self.texts.slice(int(a), int(b - a)).to_pylist() for a, b in zip(self.edges[:-1], self.edges[1:]))


# ------------------------------------------------------------------------------------------------ tokenising
@dataclass(frozen=True)
class Admission:
    """Which units are written.  ``per_unit = False``: a unit is one document and is kept when it has at least
    ``min_tokens`` tokens of its own (separator not counted).  ``per_unit = True``: the unit's documents are counted
    together, each with its EOS (and BOS), and the unit is kept or dropped as a whole."""
    min_tokens: int = 0
    per_unit: bool = False


_ENCODER = None


def _load_encoder(tokenizer_path: str) -> None:
    # one single-threaded tokenizer per worker: the Rust side would otherwise start a thread pool per process,
    # and a pool that exists across fork() can deadlock the child
    global _ENCODER
    os.environ["TOKENIZERS_PARALLELISM"] = "false"
    from transformers import PreTrainedTokenizerFast
    _ENCODER = PreTrainedTokenizerFast.from_pretrained(tokenizer_path)


def _encode_units(job) -> Tuple[np.ndarray, int, int, int]:
    """``(units, eos, bos, admission)`` -> ``(uint32 tokens, units kept, units dropped, documents written)``.  The output
    array is sized once from the admitted documents' lengths and filled in place."""
    units, eos, bos, rule = job
    lead = 0 if bos is None else 1
    admitted: List[List[int]] = []
    kept = dropped = 0
    for unit in units:
        docs = _ENCODER(unit, add_special_tokens=False, return_attention_mask=False)["input_ids"]
        weight = sum(len(d) + 1 + lead for d in docs) if rule.per_unit else len(docs[0])
        if weight < rule.min_tokens:
            dropped += 1
        else:
            kept += 1
            admitted.extend(docs)
    sizes = np.fromiter((len(d) for d in admitted), np.int64, len(admitted)) + (1 + lead)
    out = np.empty(int(sizes.sum()), np.uint32)
    ends = np.cumsum(sizes)
    for doc, end, size in zip(admitted, ends, sizes):
        start = end - size
        if lead:
            out[start] = bos
        out[start + lead:end - 1] = doc
    out[ends - 1] = eos
    return out, kept, dropped, len(admitted)


def _portions(units: Iterable[Unit], chars: int) -> Iterator[List[Unit]]:
    """Consecutive units cut into jobs of roughly ``chars`` characters of text."""
    job, size = [], 0
    for unit in units:
        job.append(unit)
        size += sum(map(len, unit))
        if size >= chars:
            yield job
            job, size = [], 0
    if job:
        yield job


class EncoderPool:
    def __init__(self, tokenizer_path: str, workers: int):
        from multiprocessing import Pool
        self.pool = Pool(max(1, workers), initializer=_load_encoder, initargs=(tokenizer_path,))

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.pool.terminate() if exc[0] else self.pool.close()
        self.pool.join()

    def encode(self, units: Iterable[Unit], eos: int, bos: Optional[int], rule: Admission, chars: int):
        """Results of the portions of ``units`` in order (``imap`` keeps submission order)."""
        return self.pool.imap(_encode_units, ((job, eos, bos, rule) for job in _portions(units, chars)), chunksize=1)


def build_stream(name: str, feed, files: Sequence[str], tokenizer_path: str, out_dir: str, rule: Admission, bos: bool,
                 hash_tag: str, workers: int, portion_chars: int, describe: Callable[[dict], dict]) -> str:
    """Tokenise ``feed`` into ``{out_dir}/{name}_{hash}``; returns the directory (at once if it is already complete).
    ``describe(counters)`` turns ``{units_kept, units_dropped, docs, tokens}`` into the sub-command's meta fields."""
    from transformers import PreTrainedTokenizerFast
    tok = PreTrainedTokenizerFast.from_pretrained(tokenizer_path)
    if tok.eos_token_id is None:
        raise ValueError("tokenizer has no eos_token_id; documents are separated by EOS")
    ident = tokenizer_fingerprint(tok)
    eos, bos_id = int(tok.eos_token_id), (int(tok.bos_token_id) if bos else None)
    home = os.path.join(out_dir, f"{name}_{source_hash(files, ident, rule.min_tokens, bos, hash_tag)}")
    if StreamSink(os.path.join(home, "meta.json")).exists():
        print(f"[data] {home} already prepared")
        return home
    os.makedirs(home, exist_ok=True)
    feed = feed() if callable(feed) else feed
    tally = dict(units_kept=0, units_dropped=0, docs=0, tokens=0)
    began = time.time()
    with EncoderPool(tokenizer_path, workers) as pool, StreamSink(os.path.join(home, "tokens.u32")) as sink:
        for i, units in enumerate(feed):
            for tokens, kept, dropped, docs in pool.encode(units, eos, bos_id, rule, portion_chars):
                sink.write(tokens)
                tally["units_kept"] += kept; tally["units_dropped"] += dropped; tally["docs"] += docs; tally["tokens"] += len(tokens)
            mins = (time.time() - began) / 60
            print(f"[data] {name}: part {i + 1}/{len(feed)}  {tally['tokens'] / 1e9:.2f}B tokens  {mins:.1f} min", flush=True)
    _write_json(os.path.join(home, "meta.json"),
                {"name": name, "files": [{"path": os.path.abspath(p), "size": os.path.getsize(p)} for p in files], "tokenizer": ident,
                 "min_doc_tokens": rule.min_tokens, "bos": bos, "sep": "eos", **describe(tally)})
    return home


def prepare(name: str, files: Sequence[str], text_key: str, tokenizer_path: str, out_dir: str, min_doc_tokens: int = 0,
            bos: bool = False, workers: int = 32, clean: str = "") -> str:
    """Parquet text -> stream, one document per row; documents shorter than ``min_doc_tokens`` are dropped."""
    return build_stream(name, lambda: ParquetRows(files, text_key, clean), files, tokenizer_path, out_dir, Admission(min_doc_tokens),
                        bos, clean, workers, 4 << 20,
                        lambda t: {"clean": clean, "num_docs": t["docs"], "dropped_docs": t["units_dropped"], "num_tokens": t["tokens"]})


def prepare_grouped(name: str, files: Sequence[str], text_key: str, group_key: str, order_key: str, tokenizer_path: str,
                    out_dir: str, min_group_tokens: int, workers: int = 32, bos: bool = False) -> str:
    """Like ``prepare`` with the rows grouped by ``group_key``: a group's documents are written consecutively (each with
    its EOS) and the group is kept or dropped by its total token count."""
    return build_stream(name, lambda: ParquetGroups(files, text_key, group_key, order_key), files, tokenizer_path, out_dir,
                        Admission(min_group_tokens, per_unit=True), bos, f"group={group_key}", workers, 8 << 20,
                        lambda t: {"group_key": group_key, "num_groups": t["units_kept"], "dropped_groups": t["units_dropped"],
                                   "num_docs": t["docs"], "num_tokens": t["tokens"]})


# ------------------------------------------------------------------------------------------------ questions about a stream
class StreamIndex:
    """A finished stream directory: its meta data, a read-only view of the tokens and what can be derived from the
    positions of the separators."""

    def __init__(self, home: str, block_tokens: int = 1 << 24):
        self.home, self.block = home, block_tokens
        with open(os.path.join(home, "meta.json")) as fh:
            self.meta = json.load(fh)
        ident = self.meta.get("tokenizer")
        eos = ident.get("eos_token_id") if isinstance(ident, dict) else None
        self.eos = int(eos if eos is not None else self.meta.get("eos_token_id", 128001))
        self.path = os.path.join(home, "tokens.u32")
        self.tokens = np.memmap(self.path, dtype="<u4", mode="r")

    def blocks(self, lo: int = 0, hi: Optional[int] = None) -> Iterator[Tuple[int, np.ndarray]]:
        hi = len(self.tokens) if hi is None else hi
        for at in range(lo, hi, self.block):
            yield at, np.asarray(self.tokens[at:min(hi, at + self.block)])

    def boundaries(self) -> np.ndarray:
        """One past the last token of every document: the position after each EOS, plus the end of the stream when the
        last document has none."""
        found = [at + np.flatnonzero(blk == self.eos) + 1 for at, blk in self.blocks()]
        cuts = np.concatenate(found).astype(np.int64) if found else np.zeros(0, np.int64)
        n = len(self.tokens)
        return cuts if n == 0 or (len(cuts) and cuts[-1] == n) else np.append(cuts, n)

    def lengths(self) -> np.ndarray:
        return np.diff(self.boundaries(), prepend=0)

    def windows(self, seq_len: int, holdout_tokens: int) -> np.ndarray:
        """Starts of the non-overlapping ``seq_len`` windows that lie inside ONE document (aligned at its first token, its
        EOS excluded) and end before the held-out tail."""
        cuts = self.boundaries()
        first = np.concatenate([[0], cuts[:-1]]) if len(cuts) else cuts
        per_doc = np.maximum((cuts - first - 1) // seq_len, 0)
        owner = np.repeat(np.arange(len(cuts)), per_doc)
        rank = np.arange(len(owner)) - np.repeat(np.cumsum(per_doc) - per_doc, per_doc)
        starts = first[owner] + rank * seq_len
        return starts[starts + seq_len <= len(self.tokens) - holdout_tokens].astype(np.int64)

    def histogram(self, vocab: int, budget_tokens: int) -> np.ndarray:
        """Token counts over evenly spaced blocks covering about ``budget_tokens`` tokens."""
        n = len(self.tokens)
        picks = max(1, min(n, budget_tokens) // self.block)
        total = np.zeros(vocab, np.int64)
        for at in np.linspace(0, max(0, n - self.block), picks).astype(np.int64):
            total += np.bincount(np.asarray(self.tokens[at:at + self.block]).astype(np.int64), minlength=vocab)[:vocab]
        return total

    def length_table(self, thresholds: Sequence[int]) -> dict:
        ln = self.lengths()
        mass = int(ln.sum())
        table = {"docs": int(len(ln)), "tokens": mass, "mean_len": float(ln.mean()) if len(ln) else 0.0,
                 "median_len": float(np.median(ln)) if len(ln) else 0.0}
        for t in thresholds:
            big = ln[ln >= t]
            table[f">={t}"] = {"docs": int(len(big)), "tokens": int(big.sum()), "token_share": float(big.sum() / max(mass, 1))}
        return table

    def copy_documents(self, keep: np.ndarray, sink: StreamSink) -> int:
        """Write the documents flagged in ``keep`` to ``sink``; neighbours that are both kept are copied as one range."""
        cuts = self.boundaries()
        first = np.concatenate([[0], cuts[:-1]])
        flags = np.concatenate([[False], keep, [False]]).astype(np.int8)
        edges = np.diff(flags)
        written = 0
        for a, b in zip(np.flatnonzero(edges == 1), np.flatnonzero(edges == -1)):      # documents [a, b) are kept
            for _, blk in self.blocks(int(first[a]), int(cuts[b - 1])):
                sink.write(blk)
                written += len(blk)
        return written


def doc_lengths(src_dir: str, block_tokens: int = 1 << 24) -> np.ndarray:
    """Lengths (EOS included) of every document of a stream; a last document without EOS counts too."""
    return StreamIndex(src_dir, block_tokens).lengths()


def doc_windows(src_dir: str, seq_len: int, holdout_tokens: int) -> np.ndarray:
    return StreamIndex(src_dir).windows(seq_len, holdout_tokens)


def windows_path(src_dir: str, seq_len: int, holdout_tokens: int) -> str:
    return os.path.join(src_dir, f"windows_{seq_len}_{holdout_tokens}.npy")


def unigram_counts(src_dirs: Sequence[str], vocab: int, sample_tokens: int = 2_000_000_000, block_tokens: int = 1 << 24) -> np.ndarray:
    return sum((StreamIndex(d, block_tokens).histogram(vocab, sample_tokens) for d in src_dirs), np.zeros(vocab, np.int64))


def length_stats(src_dir: str, thresholds=(4096, 8192, 16384, 32768, 131072)) -> dict:
    return StreamIndex(src_dir).length_table(thresholds)


def filter_stream(src_dir: str, name: str, out_dir: str, min_doc_tokens: int = 0, max_doc_tokens: int = 0,
                  exclude: Iterable[int] = (), block_tokens: int = 1 << 24) -> str:
    """A copy of a stream with only the documents of ``min <= length < max`` tokens (EOS included; 0 = no bound) that are
    not listed in ``exclude`` (document numbers of the source)."""
    src = StreamIndex(src_dir, block_tokens)
    banned = np.unique(np.asarray(list(exclude), np.int64))
    rule = f"filter:{min_doc_tokens}:{max_doc_tokens}:{hashlib.sha256(banned.tobytes()).hexdigest()[:8] if len(banned) else ''}"
    ident = hashlib.sha256((os.path.abspath(src.path) + str(os.path.getsize(src.path)) + rule).encode()).hexdigest()[:16]
    home = os.path.join(out_dir, f"{name}_{ident}")
    if os.path.exists(os.path.join(home, "meta.json")):
        return home
    os.makedirs(home, exist_ok=True)
    ln = src.lengths()
    fits = (ln >= min_doc_tokens if min_doc_tokens > 0 else np.ones(len(ln), bool)) & (ln < max_doc_tokens if max_doc_tokens > 0 else True)
    listed = np.zeros(len(ln), bool)
    listed[banned[(banned >= 0) & (banned < len(ln))]] = True
    keep = fits & ~listed
    with StreamSink(os.path.join(home, "tokens.u32")) as sink:
        written = src.copy_documents(keep, sink)
    meta = {"name": name, "files": [{"path": os.path.abspath(src.path), "size": os.path.getsize(src.path)}],
            "derived_from": os.path.abspath(src_dir), "tokenizer": src.meta.get("tokenizer"), "min_doc_tokens": min_doc_tokens,
            "max_doc_tokens": max_doc_tokens, "bos": src.meta.get("bos", False), "sep": "eos", "clean": src.meta.get("clean", ""),
            "num_docs": int(keep.sum()), "dropped_docs": int((~keep).sum()), "num_tokens": written}
    if len(banned):
        meta.update(exclude=banned.tolist(), excluded_docs=int((fits & listed).sum()))
    _write_json(os.path.join(home, "meta.json"), meta)
    return home


# ------------------------------------------------------------------------------------------------ command line
def _parser():
    import argparse
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.data")
    sub = ap.add_subparsers(dest="cmd", required=True)

    def command(name, *options, **kw):
        p = sub.add_parser(name, **kw)
        for flag, settings in options:
            p.add_argument(flag, **settings)

    out_dir = ("--out", dict(default="bucket/data/tokens"))
    tokenizer = ("--tokenizer", dict(required=True))
    workers = ("--workers", dict(type=int, default=32))
    many = lambda flag: (flag, dict(nargs="+", required=True))
    command("prepare", ("--name", dict(required=True)), many("--files"), ("--text_key", dict(default="text")), tokenizer, out_dir,
            ("--min_doc_tokens", dict(type=int, default=0)), ("--bos", dict(action="store_true")), workers,
            ("--clean", dict(default="", choices=sorted(_CLEANERS))))
    command("prepare_grouped", ("--name", dict(required=True)), many("--files"), ("--text_key", dict(default="content")),
            ("--group_key", dict(default="max_stars_repo_name")), ("--order_key", dict(default="max_stars_repo_path")), tokenizer,
            out_dir, ("--min_group_tokens", dict(type=int, default=4096)), workers)
    command("unigram", many("--src"), ("--vocab", dict(type=int, default=128256)),
            ("--sample_tokens", dict(type=int, default=2_000_000_000)), ("--out", dict(required=True)))
    command("stats", many("--src"), ("--out", dict(default="")))
    command("filter", ("--src", dict(required=True)), ("--name", dict(required=True)), out_dir,
            ("--min_doc_tokens", dict(type=int, default=0)), ("--max_doc_tokens", dict(type=int, default=0)), ("--exclude", dict(default="")))
    command("windows", many("--src"), ("--seq_len", dict(type=int, default=8192)), ("--holdout", dict(type=int, default=4_194_304)))
    command("synth", ("--out", dict(required=True)), ("--name", dict(default="synthetic")), ("--tokens", dict(type=int, default=10_000_000)),
            ("--vocab", dict(type=int, default=128256)), ("--eos", dict(type=int, default=128001)), ("--mean_doc", dict(type=int, default=2048)),
            ("--seed", dict(type=int, default=0)), ("--zipf", dict(type=float, default=1.1)), help="write a synthetic Zipf stream")
    return ap


def main(argv: Optional[List[str]] = None) -> None:
    a = _parser().parse_args(argv)
    if a.cmd == "prepare":
        prepare(a.name, a.files, a.text_key, a.tokenizer, a.out, a.min_doc_tokens, a.bos, a.workers, a.clean)
    elif a.cmd == "prepare_grouped":
        prepare_grouped(a.name, a.files, a.text_key, a.group_key, a.order_key, a.tokenizer, a.out, a.min_group_tokens, a.workers)
    elif a.cmd == "filter":
        listed = ()
        if a.exclude:
            with open(a.exclude) as fh:
                listed = json.load(fh)
        print(filter_stream(a.src, a.name, a.out, a.min_doc_tokens, a.max_doc_tokens, listed))
    elif a.cmd == "unigram":
        counts = unigram_counts(a.src, a.vocab, a.sample_tokens)
        with StreamSink(a.out) as sink:
            sink.write(counts.tobytes())
        print(f"[data] unigram: {counts.sum() / 1e9:.2f}B tokens counted, {int((counts > 0).sum())} distinct ids -> {a.out}")
    elif a.cmd == "stats":
        report = json.dumps({os.path.basename(os.path.normpath(d)): length_stats(d) for d in a.src}, indent=2)
        if a.out:
            with open(a.out, "w") as fh:
                fh.write(report)
        print(report)
    elif a.cmd == "windows":
        for d in a.src:
            starts = doc_windows(d, a.seq_len, a.holdout)
            np.save(windows_path(d, a.seq_len, a.holdout), starts)
            print(f"[data] {d}: {len(starts)} windows -> {windows_path(d, a.seq_len, a.holdout)}", flush=True)
    elif a.cmd == "synth":
        from .synth import write_stream, zipf_tokens
        toks = zipf_tokens(a.tokens, a.vocab, a.seed, a.zipf, a.eos, a.mean_doc, exclude=(a.eos + 1,))
        print(write_stream(os.path.join(a.out, a.name), toks, a.eos, a.name, a.vocab))
