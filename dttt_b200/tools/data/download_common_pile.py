"""Fetch sources of the Common Pile v0.1 (public-domain and openly licensed text) in their filtered form: gzipped dolma
JSON lines, one directory per source under ``--out``, with a manifest that pins what was fetched.

    python -m dttt_b200.tools.data.download_common_pile --sources project_gutenberg,pre_1929_books --workers 4

The job is resumable file by file: every shard is fetched on its own (a thread pool of ``--workers``), its size is checked
against the repository's metadata, and the manifest (``<out>/manifest.json``: repository, pinned revision, shard list with
sizes, completeness) is rewritten after every source, so a second run only fetches what is missing.  Conversion to parquet
and the removal of the evaluation books are ``convert_dolma``'s job.  Needs ``huggingface_hub`` and a network; without
either the tool says so and exits non-zero.  It plays the part of the reference's ``tools/download_common_pile.py``.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import dataclasses
import json
import os
import sys
import time
from typing import Dict, List, Optional

# the long-document mix the 8k -> 128k stages are trained on
LONG_DOCUMENT_SOURCES = ("project_gutenberg", "pre_1929_books", "library_of_congress", "biodiversity_heritage_library", "doab",
                         "arxiv_papers")
SHARD_SUFFIX = ".json.gz"


@dataclasses.dataclass
class Shard:
    path: str
    nbytes: int


@dataclasses.dataclass
class SourcePlan:
    name: str
    repo: str
    revision: str
    shards: List[Shard]

    @property
    def nbytes(self) -> int:
        return sum(s.nbytes for s in self.shards)


def repository_of(source: str) -> str:
    return f"common-pile/{source}_filtered"


def plan_source(api, source: str, limit: int) -> SourcePlan:
    """Ask the hub which shards the source has at its current revision (``limit > 0``: the first ``limit`` by name)."""
    meta = api.dataset_info(repository_of(source), files_metadata=True)
    shards = sorted((Shard(f.rfilename, int(f.size or 0)) for f in meta.siblings if f.rfilename.endswith(SHARD_SUFFIX)),
                    key=lambda s: s.path)
    return SourcePlan(source, repository_of(source), meta.sha, shards[:limit] if limit > 0 else shards)


def missing_shards(plan: SourcePlan, root: str) -> List[Shard]:
    """Shards not on disk yet, or on disk with a size other than the repository's."""
    todo = []
    for s in plan.shards:
        local = os.path.join(root, plan.name, s.path)
        if not os.path.exists(local) or (s.nbytes and os.path.getsize(local) != s.nbytes):
            todo.append(s)
    return todo


def fetch(plan: SourcePlan, todo: List[Shard], root: str, workers: int, download) -> List[str]:
    """Download ``todo`` with a thread pool; returns the paths that failed (after the pool has drained)."""
    failed: List[str] = []

    def one(s: Shard) -> Optional[str]:
        try:
            download(repo_id=plan.repo, repo_type="dataset", revision=plan.revision, filename=s.path,
                     local_dir=os.path.join(root, plan.name))
            return None
        except Exception as e:                                   # network drop, rate limit, file withdrawn
            return f"{s.path}: {type(e).__name__}: {e}"

    with cf.ThreadPoolExecutor(max_workers=max(1, workers)) as pool:
        for err in pool.map(one, todo):
            if err:
                failed.append(err)
    return failed


def read_manifest(path: str) -> Dict[str, dict]:
    if os.path.exists(path):
        with open(path) as fh:
            return json.load(fh)
    return {}


def write_manifest(path: str, manifest: Dict[str, dict]) -> None:
    tmp = path + ".tmp"
    with open(tmp, "w") as fh:
        json.dump(manifest, fh, indent=1, sort_keys=True)
    os.replace(tmp, path)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.tools.data.download_common_pile")
    ap.add_argument("--sources", default=",".join(LONG_DOCUMENT_SOURCES), help="comma-separated source names (repository common-pile/<name>_filtered)")
    ap.add_argument("--out", default="bucket/data/raw/common_pile")
    ap.add_argument("--workers", type=int, default=4)
    ap.add_argument("--max_files", type=int, default=0, help="> 0: only the first shards of every source (a sample)")
    a = ap.parse_args(argv)
    try:
        from huggingface_hub import HfApi, hf_hub_download
    except ImportError:
        print("[pile] huggingface_hub is not installed: nothing fetched", file=sys.stderr)
        return 2
    os.makedirs(a.out, exist_ok=True)
    manifest_path = os.path.join(a.out, "manifest.json")
    manifest = read_manifest(manifest_path)
    api = HfApi()
    status = 0
    for source in filter(None, (s.strip() for s in a.sources.split(","))):
        started = time.time()
        try:
            plan = plan_source(api, source, a.max_files)
        except Exception as e:                                   # offline, unknown repository
            print(f"[pile] {repository_of(source)}: {type(e).__name__}: {e}", file=sys.stderr)
            return 3
        todo = missing_shards(plan, a.out)
        print(f"[pile] {source}: revision {plan.revision[:12]}, {len(plan.shards)} shards, {plan.nbytes / 2 ** 30:.1f} GiB, "
              f"{len(todo)} to fetch", flush=True)
        failed = fetch(plan, todo, a.out, a.workers, hf_hub_download) if todo else []
        for msg in failed:
            print(f"[pile]   failed {msg}", file=sys.stderr)
        still = missing_shards(plan, a.out)
        manifest[source] = {"repo": plan.repo, "revision": plan.revision, "sample": a.max_files > 0, "complete": not still,
                            "bytes": plan.nbytes, "shards": {s.path: s.nbytes for s in plan.shards}}
        write_manifest(manifest_path, manifest)
        print(f"[pile] {source}: {'complete' if not still else f'{len(still)} shards missing'} after {time.time() - started:.0f}s",
              flush=True)
        if still:
            status = 4
    return status


if __name__ == "__main__":
    sys.exit(main())
