"""Building and indexing token streams: ``python -m dttt_b200.data {prepare,prepare_grouped,filter,unigram,stats,windows,synth}``.

Capabilities of the reference's data CLI (``src/ttt/data.py:195-515,915-985``) on the same on-disk format
(``streams.py``): tokenise parquet text into an EOS-separated uint32 stream (row groups read ahead of a worker
pool, output order = file / row-group / document order regardless of the worker count), tokenise with
documents grouped by a key (e.g. a repository) and kept or dropped as a group, filter a stream by document
length or an exclusion list, count unigrams over evenly spaced blocks, report length statistics, and index the
single-document training windows.  ``synth`` writes a Zipf stream for machines without data.  Outputs go to a
``.tmp`` name first and are renamed when complete.
"""
from __future__ import annotations

import contextlib
import hashlib
import html
import json
import os
import re
import time
from typing import Dict, Iterable, List, Optional, Sequence

import numpy as np

_TAG = re.compile(r"<[^>]{1,200}>")
_BLANKS = re.compile(r"\n{3,}")


def tokenizer_fingerprint(tok) -> Dict[str, object]:
    return {"class": tok.__class__.__name__, "len": int(len(tok)), "vocab_size": int(getattr(tok, "vocab_size", -1)),
            "eos_token_id": int(tok.eos_token_id) if tok.eos_token_id is not None else None,
            "bos_token_id": int(tok.bos_token_id) if tok.bos_token_id is not None else None}


def source_hash(files: Sequence[str], fp: Dict[str, object], min_doc_tokens: int, bos: bool, clean: str = "") -> str:
    h = hashlib.sha256()
    for f in sorted(os.path.abspath(p) for p in files):
        h.update(f.encode())
        h.update(str(os.path.getsize(f)).encode())
    h.update(json.dumps(fp, sort_keys=True).encode())
    h.update(f"min_doc_tokens={min_doc_tokens};bos={bos};sep=eos".encode())
    if clean:
        h.update(f";clean={clean}".encode())
    return h.hexdigest()[:16]


def clean_text(text: str, mode: str) -> str:
    if not mode:
        return text
    if mode == "html":
        return _BLANKS.sub("\n\n", _TAG.sub("", html.unescape(text)))
    raise ValueError(f"unknown clean mode {mode!r}")


@contextlib.contextmanager
def atomic_output(path: str):
    """Write to ``path + '.tmp'`` and rename on success."""
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    tmp = path + ".tmp"
    fh = open(tmp, "wb")
    try:
        yield fh
        fh.close()
        os.replace(tmp, path)
    except BaseException:
        fh.close()
        with contextlib.suppress(OSError):
            os.remove(tmp)
        raise


def _write_meta(d: str, meta: dict) -> None:
    with atomic_output(os.path.join(d, "meta.json")) as fh:
        fh.write(json.dumps(meta, indent=2).encode())


_TOK = None


def _worker_init(tokenizer_path: str) -> None:
    global _TOK
    from transformers import PreTrainedTokenizerFast
    _TOK = PreTrainedTokenizerFast.from_pretrained(tokenizer_path)


def _encode_docs(args):
    texts, eos, bos, min_tokens = args
    enc = _TOK(texts, add_special_tokens=False, return_attention_mask=False)["input_ids"]
    parts, kept, dropped = [], 0, 0
    for ids in enc:
        if len(ids) + 1 < min_tokens:
            dropped += 1
            continue
        if bos is not None:
            parts.append(np.array([bos], np.uint32))
        parts.append(np.asarray(ids, np.uint32))
        parts.append(np.array([eos], np.uint32))
        kept += 1
    return (np.concatenate(parts) if parts else np.zeros(0, np.uint32)), kept, dropped


def _batches(items: List, target_chars: int = 8 << 20):
    cur, size = [], 0
    for t in items:
        cur.append(t)
        size += len(t) if isinstance(t, str) else sum(len(x) for x in t)
        if size >= target_chars:
            yield cur
            cur, size = [], 0
    if cur:
        yield cur


def prepare(name: str, files: Sequence[str], text_key: str, tokenizer_path: str, out_dir: str, min_doc_tokens: int = 0,
            bos: bool = False, workers: int = 32, clean: str = "") -> str:
    import pyarrow.parquet as pq
    from concurrent.futures import ThreadPoolExecutor
    from multiprocessing import Pool
    from transformers import PreTrainedTokenizerFast
    tok = PreTrainedTokenizerFast.from_pretrained(tokenizer_path)
    fp = tokenizer_fingerprint(tok)
    if tok.eos_token_id is None:
        raise ValueError("tokenizer has no eos_token_id; documents are separated by EOS")
    eos, bos_id = int(tok.eos_token_id), (int(tok.bos_token_id) if bos else None)
    d = os.path.join(out_dir, f"{name}_{source_hash(files, fp, min_doc_tokens, bos, clean)}")
    if os.path.exists(os.path.join(d, "meta.json")):
        print(f"[data] {d} already prepared")
        return d
    os.makedirs(d, exist_ok=True)
    units = [(pf, rg) for pf in (pq.ParquetFile(p, pre_buffer=True, buffer_size=64 << 20) for p in files)
             for rg in range(pf.num_row_groups)]
    read = lambda u: [clean_text(t, clean) for t in u[0].read_row_group(u[1], columns=[text_key])[text_key].to_pylist()]
    kept = dropped = total = 0
    t0 = time.time()
    with Pool(workers, initializer=_worker_init, initargs=(tokenizer_path,)) as pool, ThreadPoolExecutor(1) as reader, \
            atomic_output(os.path.join(d, "tokens.u32")) as out:
        nxt = reader.submit(read, units[0])
        for i in range(len(units)):
            texts = nxt.result()
            if i + 1 < len(units):
                nxt = reader.submit(read, units[i + 1])
            for arr, k, dr in pool.imap(_encode_docs, ((b, eos, bos_id, min_doc_tokens) for b in _batches(texts)), chunksize=1):
                out.write(arr.astype("<u4").tobytes())
                kept, dropped, total = kept + k, dropped + dr, total + len(arr)
            print(f"[data] {name}: row group {i + 1}/{len(units)}  {total / 1e9:.2f}B tokens  {(time.time() - t0) / 60:.1f} min", flush=True)
    _write_meta(d, {"name": name, "files": [{"path": os.path.abspath(p), "size": os.path.getsize(p)} for p in files],
                    "tokenizer": fp, "min_doc_tokens": min_doc_tokens, "bos": bos, "sep": "eos", "clean": clean,
                    "num_docs": kept, "dropped_docs": dropped, "num_tokens": total})
    return d


def _encode_groups(args):
    groups, eos, bos, min_group = args
    parts, kept, dropped, docs = [], 0, 0, 0
    for texts in groups:
        enc = _TOK(texts, add_special_tokens=False, return_attention_mask=False)["input_ids"]
        if sum(len(ids) + 1 + (bos is not None) for ids in enc) < min_group:
            dropped += 1
            continue
        for ids in enc:
            if bos is not None:
                parts.append(np.array([bos], np.uint32))
            parts.append(np.asarray(ids, np.uint32))
            parts.append(np.array([eos], np.uint32))
        kept, docs = kept + 1, docs + len(enc)
    return (np.concatenate(parts) if parts else np.zeros(0, np.uint32)), kept, dropped, docs


def prepare_grouped(name: str, files: Sequence[str], text_key: str, group_key: str, order_key: str, tokenizer_path: str,
                    out_dir: str, min_group_tokens: int, workers: int = 32, bos: bool = False) -> str:
    import pyarrow as pa
    import pyarrow.parquet as pq
    from multiprocessing import Pool
    from transformers import PreTrainedTokenizerFast
    tok = PreTrainedTokenizerFast.from_pretrained(tokenizer_path)
    fp = tokenizer_fingerprint(tok)
    eos, bos_id = int(tok.eos_token_id), (int(tok.bos_token_id) if bos else None)
    d = os.path.join(out_dir, f"{name}_{source_hash(files, fp, min_group_tokens, bos, f'group={group_key}')}")
    if os.path.exists(os.path.join(d, "meta.json")):
        print(f"[data] {d} already prepared")
        return d
    os.makedirs(d, exist_ok=True)
    schema = pa.schema([(group_key, pa.string()), (order_key, pa.string()), (text_key, pa.large_string())])
    table = pa.concat_tables([pq.read_table(p, columns=[group_key, order_key, text_key], pre_buffer=True).cast(schema) for p in files])
    table = table.sort_by([(group_key, "ascending"), (order_key, "ascending")])
    keys = table.column(group_key).to_pylist()
    bounds = [0] + [i for i in range(1, len(keys)) if keys[i] != keys[i - 1]] + [len(keys)]
    texts = table.column(text_key)
    groups = (texts.slice(bounds[g], bounds[g + 1] - bounds[g]).to_pylist() for g in range(len(bounds) - 1))
    kept = dropped = total = docs = 0
    with Pool(workers, initializer=_worker_init, initargs=(tokenizer_path,)) as pool, atomic_output(os.path.join(d, "tokens.u32")) as out:
        for arr, k, dr, nd in pool.imap(_encode_groups, ((b, eos, bos_id, min_group_tokens) for b in _batches(list(groups))), chunksize=1):
            out.write(arr.astype("<u4").tobytes())
            kept, dropped, total, docs = kept + k, dropped + dr, total + len(arr), docs + nd
    _write_meta(d, {"name": name, "files": [{"path": os.path.abspath(p), "size": os.path.getsize(p)} for p in files],
                    "tokenizer": fp, "min_doc_tokens": min_group_tokens, "bos": bos, "sep": "eos", "group_key": group_key,
                    "num_groups": kept, "dropped_groups": dropped, "num_docs": docs, "num_tokens": total})
    return d


def _read_meta(src_dir: str) -> dict:
    with open(os.path.join(src_dir, "meta.json")) as fh:
        return json.load(fh)


def _eos_of(meta: dict) -> int:
    tok = meta.get("tokenizer", {})
    return int(tok["eos_token_id"]) if isinstance(tok, dict) and tok.get("eos_token_id") is not None else int(meta.get("eos_token_id", 128001))


def doc_lengths(src_dir: str, block_tokens: int = 1 << 24) -> np.ndarray:
    """Lengths (EOS included) of every document of a stream, one pass; a last document without EOS counts too."""
    eos = _eos_of(_read_meta(src_dir))
    stream = np.memmap(os.path.join(src_dir, "tokens.u32"), dtype="<u4", mode="r")
    pieces, carry = [], 0
    for start in range(0, len(stream), block_tokens):
        blk = np.asarray(stream[start:start + block_tokens])
        ends = np.flatnonzero(blk == eos)
        if not len(ends):
            carry += len(blk)
            continue
        ln = np.diff(np.concatenate([[-1], ends]))
        ln[0] += carry
        pieces.append(ln)
        carry = len(blk) - ends[-1] - 1
    if carry:
        pieces.append(np.array([carry]))
    return np.concatenate(pieces).astype(np.int64) if pieces else np.zeros(0, np.int64)


def filter_stream(src_dir: str, name: str, out_dir: str, min_doc_tokens: int = 0, max_doc_tokens: int = 0,
                  exclude: Iterable[int] = (), block_tokens: int = 1 << 24) -> str:
    """Keep the documents with ``min <= length < max`` (EOS included; 0 = no bound) that are not in ``exclude``
    (document indices of the source)."""
    meta = _read_meta(src_dir)
    eos = _eos_of(meta)
    src = os.path.join(src_dir, "tokens.u32")
    excl = np.unique(np.asarray(list(exclude), np.int64))
    tag = f"filter:{min_doc_tokens}:{max_doc_tokens}:{hashlib.sha256(excl.tobytes()).hexdigest()[:8] if len(excl) else ''}"
    d = os.path.join(out_dir, f"{name}_{hashlib.sha256((os.path.abspath(src) + str(os.path.getsize(src)) + tag).encode()).hexdigest()[:16]}")
    if os.path.exists(os.path.join(d, "meta.json")):
        return d
    os.makedirs(d, exist_ok=True)
    lengths = doc_lengths(src_dir, block_tokens)
    keep = np.ones(len(lengths), bool)
    if min_doc_tokens > 0:
        keep &= lengths >= min_doc_tokens
    if max_doc_tokens > 0:
        keep &= lengths < max_doc_tokens
    hit = np.isin(np.arange(len(lengths)), excl)
    excluded = int((keep & hit).sum())
    keep &= ~hit
    starts = np.concatenate([[0], np.cumsum(lengths)[:-1]])
    stream = np.memmap(src, dtype="<u4", mode="r")
    total = 0
    with atomic_output(os.path.join(d, "tokens.u32")) as out:
        # runs of consecutive kept documents are copied as one slice
        idx = np.flatnonzero(keep)
        if len(idx):
            breaks = np.flatnonzero(np.diff(idx) != 1)
            run_a = np.concatenate([[0], breaks + 1])
            run_b = np.concatenate([breaks, [len(idx) - 1]])
            for a, b in zip(run_a, run_b):
                lo, hi = int(starts[idx[a]]), int(starts[idx[b]] + lengths[idx[b]])
                for p in range(lo, hi, block_tokens):
                    seg = np.asarray(stream[p:min(hi, p + block_tokens)])
                    out.write(seg.astype("<u4").tobytes())
                    total += len(seg)
    out_meta = {"name": name, "files": [{"path": os.path.abspath(src), "size": os.path.getsize(src)}],
                "derived_from": os.path.abspath(src_dir), "tokenizer": meta.get("tokenizer"), "min_doc_tokens": min_doc_tokens,
                "max_doc_tokens": max_doc_tokens, "bos": meta.get("bos", False), "sep": "eos", "clean": meta.get("clean", ""),
                "num_docs": int(keep.sum()), "dropped_docs": int((~keep).sum()), "num_tokens": total}
    if len(excl):
        out_meta.update(exclude=excl.tolist(), excluded_docs=excluded)
    _write_meta(d, out_meta)
    return d


def windows_path(src_dir: str, seq_len: int, holdout_tokens: int) -> str:
    return os.path.join(src_dir, f"windows_{seq_len}_{holdout_tokens}.npy")


def doc_windows(src_dir: str, seq_len: int, holdout_tokens: int) -> np.ndarray:
    """Start offsets of every non-overlapping ``seq_len`` window inside ONE document (aligned at the document's
    first token, EOS excluded) that ends before the held-out tail."""
    lengths = doc_lengths(src_dir)
    starts = np.concatenate([[0], np.cumsum(lengths)[:-1]]) if len(lengths) else np.zeros(0, np.int64)
    n_win = (lengths - 1) // seq_len
    keep = n_win > 0
    starts, n_win = starts[keep], n_win[keep]
    within = np.arange(n_win.sum()) - np.repeat(np.cumsum(n_win) - n_win, n_win)
    out = np.repeat(starts, n_win) + seq_len * within
    return out[out + seq_len <= int(lengths.sum()) - holdout_tokens].astype(np.int64)


def unigram_counts(src_dirs: Sequence[str], vocab: int, sample_tokens: int = 2_000_000_000, block_tokens: int = 1 << 24) -> np.ndarray:
    counts = np.zeros(vocab, np.int64)
    for d in src_dirs:
        mm = np.memmap(os.path.join(d, "tokens.u32"), dtype="<u4", mode="r")
        n = len(mm)
        n_blocks = max(1, min(n, sample_tokens) // block_tokens)
        for st in np.linspace(0, max(0, n - block_tokens), n_blocks).astype(np.int64):
            counts += np.bincount(np.asarray(mm[st:st + block_tokens]).astype(np.int64), minlength=vocab)[:vocab]
    return counts


def length_stats(src_dir: str, thresholds=(4096, 8192, 16384, 32768, 131072)) -> dict:
    ln = doc_lengths(src_dir)
    total = int(ln.sum())
    out = {"docs": int(len(ln)), "tokens": total, "mean_len": float(ln.mean()) if len(ln) else 0.0,
           "median_len": float(np.median(ln)) if len(ln) else 0.0}
    for t in thresholds:
        m = ln >= t
        out[f">={t}"] = {"docs": int(m.sum()), "tokens": int(ln[m].sum()), "token_share": float(ln[m].sum() / max(total, 1))}
    return out


def main(argv: Optional[List[str]] = None) -> None:
    import argparse
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.data")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("prepare")
    p.add_argument("--name", required=True); p.add_argument("--files", nargs="+", required=True)
    p.add_argument("--text_key", default="text"); p.add_argument("--tokenizer", required=True)
    p.add_argument("--out", default="bucket/data/tokens"); p.add_argument("--min_doc_tokens", type=int, default=0)
    p.add_argument("--bos", action="store_true"); p.add_argument("--workers", type=int, default=32)
    p.add_argument("--clean", default="", choices=["", "html"])
    g = sub.add_parser("prepare_grouped")
    g.add_argument("--name", required=True); g.add_argument("--files", nargs="+", required=True)
    g.add_argument("--text_key", default="content"); g.add_argument("--group_key", default="max_stars_repo_name")
    g.add_argument("--order_key", default="max_stars_repo_path"); g.add_argument("--tokenizer", required=True)
    g.add_argument("--out", default="bucket/data/tokens"); g.add_argument("--min_group_tokens", type=int, default=4096)
    g.add_argument("--workers", type=int, default=32)
    u = sub.add_parser("unigram")
    u.add_argument("--src", nargs="+", required=True); u.add_argument("--vocab", type=int, default=128256)
    u.add_argument("--sample_tokens", type=int, default=2_000_000_000); u.add_argument("--out", required=True)
    st = sub.add_parser("stats")
    st.add_argument("--src", nargs="+", required=True); st.add_argument("--out", default="")
    q = sub.add_parser("filter")
    q.add_argument("--src", required=True); q.add_argument("--name", required=True); q.add_argument("--out", default="bucket/data/tokens")
    q.add_argument("--min_doc_tokens", type=int, default=0); q.add_argument("--max_doc_tokens", type=int, default=0)
    q.add_argument("--exclude", default="")
    w = sub.add_parser("windows")
    w.add_argument("--src", nargs="+", required=True); w.add_argument("--seq_len", type=int, default=8192)
    w.add_argument("--holdout", type=int, default=4_194_304)
    sy = sub.add_parser("synth", help="write a synthetic Zipf stream")
    sy.add_argument("--out", required=True); sy.add_argument("--name", default="synthetic"); sy.add_argument("--tokens", type=int, default=10_000_000)
    sy.add_argument("--vocab", type=int, default=128256); sy.add_argument("--eos", type=int, default=128001)
    sy.add_argument("--mean_doc", type=int, default=2048); sy.add_argument("--seed", type=int, default=0); sy.add_argument("--zipf", type=float, default=1.1)
    a = ap.parse_args(argv)
    if a.cmd == "prepare":
        prepare(a.name, a.files, a.text_key, a.tokenizer, a.out, a.min_doc_tokens, a.bos, a.workers, a.clean)
    elif a.cmd == "prepare_grouped":
        prepare_grouped(a.name, a.files, a.text_key, a.group_key, a.order_key, a.tokenizer, a.out, a.min_group_tokens, a.workers)
    elif a.cmd == "filter":
        filter_stream(a.src, a.name, a.out, a.min_doc_tokens, a.max_doc_tokens, json.load(open(a.exclude)) if a.exclude else ())
    elif a.cmd == "unigram":
        c = unigram_counts(a.src, a.vocab, a.sample_tokens)
        with atomic_output(a.out) as fh:
            fh.write(c.tobytes())
        print(f"[data] unigram: {c.sum() / 1e9:.2f}B tokens counted, {int((c > 0).sum())} distinct ids -> {a.out}")
    elif a.cmd == "stats":
        text = json.dumps({os.path.basename(os.path.normpath(d)): length_stats(d) for d in a.src}, indent=2)
        if a.out:
            with open(a.out, "w") as fh:
                fh.write(text)
        print(text)
    elif a.cmd == "windows":
        for d in a.src:
            wv = doc_windows(d, a.seq_len, a.holdout)
            np.save(windows_path(d, a.seq_len, a.holdout), wv)
            print(f"[data] {d}: {len(wv)} windows -> {windows_path(d, a.seq_len, a.holdout)}", flush=True)
    elif a.cmd == "synth":
        from .synth import write_stream, zipf_tokens
        toks = zipf_tokens(a.tokens, a.vocab, a.seed, a.zipf, a.eos, a.mean_doc, exclude=(a.eos + 1,))
        print(write_stream(os.path.join(a.out, a.name), toks, a.eos, a.name, a.vocab))
