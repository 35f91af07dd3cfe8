"""Download sources of the Common Pile v0.1 (public-domain and openly licensed text) in their filtered form -- dolma
JSON lines, gzipped -- into ``<out>/<source>/`` and record the dataset revisions in ``<out>/manifest.json``.  Network
only; conversion to parquet and the evaluation books' removal are ``convert_dolma``.

    python -m dttt_b200.tools.data.download_common_pile --sources project_gutenberg,pre_1929_books --workers 4

Needs ``huggingface_hub`` and network access; exits with a message when either is missing.  Role of the reference's
``tools/download_common_pile.py:1-54``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

LONG_DOCUMENT_SOURCES = "project_gutenberg,pre_1929_books,library_of_congress,biodiversity_heritage_library,doab,arxiv_papers"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.tools.data.download_common_pile")
    ap.add_argument("--sources", default=LONG_DOCUMENT_SOURCES, help="comma-separated; the repository is common-pile/<name>_filtered")
    ap.add_argument("--out", default="bucket/data/raw/common_pile")
    ap.add_argument("--workers", type=int, default=4)
    ap.add_argument("--max_files", type=int, default=0, help="> 0: only a source's first files by name")
    a = ap.parse_args(argv)
    try:
        from huggingface_hub import HfApi, snapshot_download
    except ImportError:
        print("huggingface_hub is not installed: nothing downloaded", file=sys.stderr)
        return 2
    os.makedirs(a.out, exist_ok=True)
    man_path = os.path.join(a.out, "manifest.json")
    manifest = json.load(open(man_path)) if os.path.exists(man_path) else {}
    api = HfApi()
    for name in [s for s in a.sources.split(",") if s]:
        repo = f"common-pile/{name}_filtered"
        t0 = time.time()
        try:
            info = api.dataset_info(repo, files_metadata=True)
        except Exception as e:                                   # offline, unknown repository, rate limit
            print(f"[pile] {repo}: {type(e).__name__}: {e}", file=sys.stderr)
            return 3
        files = sorted((s for s in info.siblings if s.rfilename.endswith(".json.gz")), key=lambda s: s.rfilename)
        if a.max_files > 0:
            files = files[:a.max_files]
        size = sum(s.size or 0 for s in files)
        print(f"[pile] {name}: {len(files)} files, {size / 2 ** 30:.1f} GiB at revision {info.sha[:12]}", flush=True)
        snapshot_download(repo, repo_type="dataset", revision=info.sha, local_dir=os.path.join(a.out, name),
                          allow_patterns=[s.rfilename for s in files], max_workers=a.workers)
        manifest[name] = {"repo": repo, "revision": info.sha, "files": len(files), "bytes": size, "part": a.max_files > 0}
        with open(man_path, "w") as fh:
            json.dump(manifest, fh, indent=1)
        print(f"[pile] {name}: done in {time.time() - t0:.0f}s", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
