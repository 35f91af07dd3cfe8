"""Find the PG-19 test books inside prepared token streams.

Every document of at least ``--min_chars`` characters in a stream's parquet files is scored by the share of its word
13-grams (every ``--stride``-th; the measure of ``convert_dolma``) found among the test books.  Documents above
``--overlap`` are attributed to the book most of their hits come from, their index in the stream is verified against the
token file (first 32 tokens and length equal the tokenised text) and written to ``<out>/exclude_<name>.json`` for
``python -m dttt_b200.data filter --exclude``.  ``<out>/scan.json`` keeps every document above 0.05.

A stream's document index is its row's position over the parquet files in the order ``prepare`` read them, which holds
only when no document was dropped, regrouped or derived: other streams are refused.

    python -m dttt_b200.tools.data.pg19_overlap --out log/pg19_overlap --streams books=tokens/books_<hash> web=tokens/web_<hash>

Role of the reference's ``tools/pg19_overlap.py:1-151``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from multiprocessing import Pool
from typing import Dict, List, Optional

import numpy as np

from .decontam import BookSet

_BOOKS: Optional[BookSet] = None
_OPT = None
KEEP_ABOVE = 0.05


def scan_row_group(job):
    import pyarrow.parquet as pq
    name, path, rg = job
    texts = pq.ParquetFile(path).read_row_group(rg, columns=["text"]).column("text").to_pylist()
    hits, scored = [], 0
    for row, text in enumerate(texts):
        if not text or len(text) < _OPT.min_chars:
            continue
        scored += 1
        o, book = _BOOKS.best_book(text, _OPT.stride)
        if o > KEEP_ABOVE:
            hits.append({"file": os.path.basename(path), "rg": rg, "row": row, "chars": len(text), "overlap": round(o, 4), "book": book,
                         "head": text[:120].replace("\n", " ")})
    return name, len(texts), scored, hits


def document_ends(stream: np.ndarray, eos: int, block: int = 1 << 28) -> np.ndarray:
    return np.concatenate([s + np.flatnonzero(np.asarray(stream[s:s + block]) == eos) for s in range(0, len(stream), block)] or
                          [np.empty(0, np.int64)])


def verify_and_index(name: str, stream_dir: str, meta: dict, hits: List[dict], tokenizer) -> List[int]:
    """Stream indices of ``hits`` (in place: ``doc`` and ``tokens`` are added), each checked against the token file."""
    import pyarrow.parquet as pq
    files = {os.path.basename(f["path"]): pq.ParquetFile(f["path"]) for f in meta["files"]}
    first_row, n = {}, 0
    for f in meta["files"]:
        pf = files[os.path.basename(f["path"])]
        for rg in range(pf.num_row_groups):
            first_row[(os.path.basename(f["path"]), rg)] = n
            n += pf.metadata.row_group(rg).num_rows
    if n != meta["num_docs"]:
        raise SystemExit(f"{name}: {n} parquet rows but {meta['num_docs']} documents in the stream")
    if not hits:
        return []
    stream = np.memmap(os.path.join(stream_dir, "tokens.u32"), dtype="<u4", mode="r")
    eos = int(meta["tokenizer"]["eos_token_id"])
    ends = document_ends(stream, eos)
    if len(ends) != meta["num_docs"]:
        raise SystemExit(f"{name}: {len(ends)} end-of-document tokens but {meta['num_docs']} documents")
    out = []
    for h in hits:
        i = first_row[(h["file"], h["rg"])] + h["row"]
        text = files[h["file"]].read_row_group(h["rg"], columns=["text"]).column("text")[h["row"]].as_py()
        start = 0 if i == 0 else int(ends[i - 1]) + 1
        ids = tokenizer(text, add_special_tokens=False)["input_ids"]
        if np.asarray(stream[start:start + 32]).tolist() != ids[:32] or int(ends[i]) - start != len(ids):
            raise SystemExit(f"{name}: document {i} ({h['file']} row group {h['rg']} row {h['row']}) does not match its text")
        h.update(doc=i, tokens=len(ids))
        out.append(i)
    return out


def main(argv=None) -> int:
    global _BOOKS, _OPT
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.tools.data.pg19_overlap")
    ap.add_argument("--streams", nargs="+", required=True, help="NAME=STREAM_DIR (an output of `python -m dttt_b200.data prepare`)")
    ap.add_argument("--out", required=True)
    ap.add_argument("--pg19_test", default="bucket/data/raw/pg19_test/test.parquet")
    ap.add_argument("--tokenizer", default="configs/1b_e2e")
    ap.add_argument("--min_chars", type=int, default=8000)
    ap.add_argument("--stride", type=int, default=32)
    ap.add_argument("--overlap", type=float, default=0.2)
    ap.add_argument("--workers", type=int, default=16)
    _OPT = o = ap.parse_args(argv)
    import pyarrow.parquet as pq
    t0 = time.time()
    _BOOKS = BookSet.from_parquet(o.pg19_test)
    print(f"[pg19] {len(_BOOKS.names)} test books, {len(_BOOKS.hashes)} 13-grams ({time.time() - t0:.0f}s)", flush=True)
    streams: Dict[str, tuple] = {}
    jobs = []
    for spec in o.streams:
        name, d = spec.split("=", 1)
        meta = json.load(open(os.path.join(d, "meta.json")))
        if meta.get("dropped_docs") or meta.get("min_doc_tokens") or "derived_from" in meta or "group_key" in meta:
            raise SystemExit(f"{name}: documents were dropped, regrouped or derived; its indices are not parquet rows")
        streams[name] = (d, meta)
        for f in meta["files"]:
            jobs += [(name, f["path"], rg) for rg in range(pq.ParquetFile(f["path"]).num_row_groups)]
    res = {n: {"docs": 0, "scored": 0, "hits": []} for n in streams}
    it = Pool(o.workers).imap_unordered(scan_row_group, jobs) if o.workers > 1 else map(scan_row_group, jobs)
    for k, (name, n, scored, hits) in enumerate(it):
        r = res[name]
        r["docs"] += n; r["scored"] += scored; r["hits"] += hits
        if k % 500 == 0:
            print(f"[pg19] {k}/{len(jobs)} row groups ({time.time() - t0:.0f}s)", flush=True)
    from transformers import PreTrainedTokenizerFast
    tok = PreTrainedTokenizerFast.from_pretrained(o.tokenizer)
    os.makedirs(o.out, exist_ok=True)
    for name, (d, meta) in streams.items():
        r = res[name]
        r["hits"].sort(key=lambda h: (h["file"], h["rg"], h["row"]))
        big = [h for h in r["hits"] if h["overlap"] > o.overlap]
        excl = verify_and_index(name, d, meta, big, tok)
        with open(os.path.join(o.out, f"exclude_{name}.json"), "w") as fh:
            json.dump(sorted(excl), fh)
        r.update(stream=d, above=len(big), books=sorted({h["book"] for h in big if h["book"]}))
        for h in big:
            print(f"[pg19] {name}: doc {h['doc']} ({h['tokens']} tokens, overlap {h['overlap']:.3f}) <- {str(h['book'])[:60]}", flush=True)
        print(f"[pg19] {name}: {r['scored']} of {r['docs']} documents scored, {len(big)} above {o.overlap} from {len(r['books'])} books "
              f"-> {o.out}/exclude_{name}.json", flush=True)
    with open(os.path.join(o.out, "scan.json"), "w") as fh:
        json.dump({"min_chars": o.min_chars, "stride": o.stride, "overlap": o.overlap, "streams": res}, fh, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
