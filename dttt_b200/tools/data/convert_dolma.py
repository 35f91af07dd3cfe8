"""Dolma JSON lines (gzipped; the Common Pile's form, see ``download_common_pile``) to parquet for
``python -m dttt_b200.data prepare``: one parquet per input file with ``id``, ``title``, ``text`` and row groups of about
``--row_group_mb`` of text.  Documents of the evaluation books (the PG-19 test set, ``--pg19_test`` parquet) are removed:

    by id     a Project Gutenberg record whose ``metadata.url`` names a test book's number
    by text   a document whose share of word 13-grams (every ``--stride``-th) found in the test books exceeds ``--overlap``

Removed documents are listed in ``<out>/removed.jsonl``, the counts in ``<out>/summary.json``.  ``--group KEY:ORDER`` joins
consecutive records sharing ``KEY`` into one document ordered by ``ORDER`` (pages of a scanned volume), after the removal
page by page.

    python -m dttt_b200.tools.data.convert_dolma --src raw/common_pile/project_gutenberg --out raw/parquet/project_gutenberg

Role of the reference's ``tools/convert_dolma.py:1-190``.
"""
from __future__ import annotations

import argparse
import glob
import gzip
import json
import os
import sys
import time
from multiprocessing import Pool
from typing import Iterator, List, Optional

from .decontam import BookSet, gutenberg_number

_BOOKS: Optional[BookSet] = None
_OPT = None


def _order_key(v):
    v = str(v)
    return (0, int(v), "") if v.isdigit() else (1, 0, v)


def documents(lines: Iterator[str], group: Optional[tuple]) -> Iterator[dict]:
    """Records of a file as ``{"id", "title", "pages": [record, ...]}``; with ``group`` one document per run of equal KEY."""
    if not group:
        for line in lines:
            r = json.loads(line)
            yield {"id": str(r.get("id")), "title": str((r.get("metadata") or {}).get("title") or ""), "pages": [r]}
        return
    key, order = group
    run: List[dict] = []

    def emit():
        return {"id": str(run[0].get(key)), "title": str((run[0].get("metadata") or {}).get("title") or ""),
                "pages": sorted(run, key=lambda r: _order_key(r.get(order)))}
    for line in lines:
        r = json.loads(line)
        if run and r.get(key) != run[0].get(key):
            yield emit()
            run = []
        run.append(r)
    if run:
        yield emit()


def why_removed(page: dict, books: BookSet, stride: int, threshold: float) -> Optional[str]:
    gid = gutenberg_number(page)
    if gid is not None and gid in books.ids:
        return f"pg19_test id {gid}"
    o = books.overlap(page.get("text") or "", stride)
    return f"pg19_test 13-gram overlap {o:.3f}" if o > threshold else None


def convert_file(path: str) -> dict:
    import pyarrow as pa
    import pyarrow.parquet as pq
    o, books = _OPT, _BOOKS
    group = tuple(o.group.split(":")) if o.group else None
    dst = os.path.join(o.out, os.path.basename(path).replace(".json.gz", ".parquet"))
    schema = pa.schema([("id", pa.string()), ("title", pa.string()), ("text", pa.large_string())])
    stat = {"file": os.path.basename(path), "docs_in": 0, "docs_out": 0, "chars_in": 0, "chars_out": 0, "removed": []}
    buf, buf_chars = [], 0
    with pq.ParquetWriter(dst + ".tmp", schema, compression="zstd") as writer, gzip.open(path, "rt", encoding="utf-8") as fh:
        def flush():
            nonlocal buf, buf_chars
            if buf:
                writer.write_table(pa.table({k: [b[k] for b in buf] for k in ("id", "title", "text")}, schema=schema))
            buf, buf_chars = [], 0
        for doc in documents(fh, group):
            kept = []
            for page in doc["pages"]:
                text = page.get("text") or ""
                stat["docs_in"] += 1
                stat["chars_in"] += len(text)
                if len(text) < o.min_chars:
                    continue
                why = why_removed(page, books, o.stride, o.overlap)
                if why:
                    stat["removed"].append({"file": stat["file"], "id": str(page.get("id")), "title": (page.get("metadata") or {}).get("title"),
                                            "chars": len(text), "why": why})
                else:
                    kept.append(text)
            if not kept:
                continue
            text = "\n\n".join(kept)
            buf.append({"id": doc["id"], "title": doc["title"], "text": text})
            buf_chars += len(text)
            stat["docs_out"] += 1
            stat["chars_out"] += len(text)
            if buf_chars >= o.row_group_mb * 2 ** 20:
                flush()
        flush()
    os.replace(dst + ".tmp", dst)
    return stat


def main(argv=None) -> int:
    global _BOOKS, _OPT
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.tools.data.convert_dolma")
    ap.add_argument("--src", required=True, help="directory of *.json.gz (searched recursively)")
    ap.add_argument("--out", required=True)
    ap.add_argument("--pg19_test", default="bucket/data/raw/pg19_test/test.parquet")
    ap.add_argument("--stride", type=int, default=32)
    ap.add_argument("--overlap", type=float, default=0.2)
    ap.add_argument("--min_chars", type=int, default=0)
    ap.add_argument("--row_group_mb", type=float, default=64)
    ap.add_argument("--workers", type=int, default=16)
    ap.add_argument("--group", default="", help="KEY:ORDER")
    _OPT = o = ap.parse_args(argv)
    t0 = time.time()
    _BOOKS = BookSet.from_parquet(o.pg19_test) if os.path.exists(o.pg19_test) else BookSet([])
    print(f"[dolma] {len(_BOOKS.names)} evaluation books, {len(_BOOKS.hashes)} 13-grams ({time.time() - t0:.0f}s)", flush=True)
    files = sorted(glob.glob(os.path.join(o.src, "**", "*.json.gz"), recursive=True))
    if not files:
        print(f"no *.json.gz under {o.src}", file=sys.stderr)
        return 1
    os.makedirs(o.out, exist_ok=True)
    stats = []
    if o.workers > 1:
        with Pool(o.workers) as pool:                       # forked after the book set exists: it is shared, not copied
            for s in pool.imap_unordered(convert_file, files):
                stats.append(s)
                print(f"[dolma] {s['file']}: {s['docs_out']}/{s['docs_in']} documents, {len(s['removed'])} removed ({time.time() - t0:.0f}s)", flush=True)
    else:
        stats = [convert_file(f) for f in files]
    removed = [x for s in stats for x in s["removed"]]
    with open(os.path.join(o.out, "removed.jsonl"), "w") as fh:
        fh.writelines(json.dumps(x) + "\n" for x in removed)
    summary = {"src": o.src, "files": len(files), **{k: sum(s[k] for s in stats) for k in ("docs_in", "docs_out", "chars_in", "chars_out")},
               "removed": len(removed), "removed_by_id": sum(x["why"].startswith("pg19_test id") for x in removed),
               "stride": o.stride, "overlap": o.overlap, "min_chars": o.min_chars, "group": o.group}
    with open(os.path.join(o.out, "summary.json"), "w") as fh:
        json.dump(summary, fh, indent=1)
    print(f"[dolma] done: {json.dumps(summary)}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
