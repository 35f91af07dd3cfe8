"""The offline analysis tools on a tiny run made by the training CLI: paired comparison of two runs' evaluation files,
reproduction check, likelihood bound, gradient-noise decomposition, and the statistics they share."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from util import ROOT
from dttt_b200.data.synth import write_stream, zipf_tokens


@pytest.fixture(scope="module")
def runs(tmp_path_factory):
    d = tmp_path_factory.mktemp("tools")
    for i, n in enumerate(("a", "b")):
        write_stream(str(d / "data" / n), zipf_tokens(120_000, 1024, seed=i, eos=1022, mean_doc=150), 1022, n, 1024)
    base = {"model_config": os.path.join(ROOT, "configs/tiny_baseline"), "data_root": str(d / "data"), "sources": "a=a:0.6,b=b:0.4",
            "seq_len": 256, "batch_size": 2, "grad_accum": 1, "steps": 3, "seed": 0, "lr": 0.001, "warmup_steps": 2,
            "inner_lr_warmup_steps": 0, "inner_task": "causal", "outer_shift": True, "cart_window": 32, "holdout": 20000,
            "eval_batches": 2, "eval_interval": 2, "eval_step0": False, "ckpt_interval": 2, "keep_checkpoints": 0, "log_interval": 1,
            "fused_ce_block": 0, "compute_dtype": "float32"}
    out = {}
    for name, lr in (("A", 0.001), ("B", 0.003)):
        cfg = dict(base, lr=lr, ckpt_dir=str(d / name), log_dir=str(d / name))
        (d / f"{name}.json").write_text(json.dumps(cfg))
        r = subprocess.run([sys.executable, "-m", "dttt_b200.train", "--config", str(d / f"{name}.json")], cwd=ROOT, capture_output=True,
                           text=True, timeout=900, env=dict(os.environ, OMP_NUM_THREADS="2"))
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
        (d / name / "train_main.log").write_text(r.stdout)
        out[name] = d / name
    return out


def _step_dir(run):
    return sorted(p for p in os.listdir(run) if p.startswith("step_"))[-1]


def test_evalstats_cluster_bootstrap_is_wider_for_correlated_clusters():
    from dttt_b200.tools import evalstats as S
    rng = np.random.default_rng(0)
    docs = np.repeat(np.arange(40), 5)
    x = rng.normal(size=40)[docs] + 0.1 * rng.normal(size=200)            # sequences of one document move together
    naive, clustered = S.weighted_se(x), S.cluster_se(x, docs)
    assert clustered > 1.5 * naive
    assert abs(S.cluster_se(x, np.arange(200)) - naive) < 0.2 * naive     # independent units: the two agree
    m, se_n, se_c = S.mix_stat(x, np.array(["s"] * 200), docs, {"s": 1.0})
    assert abs(m - x.mean()) < 1e-12 and se_c > se_n


def test_paired_diff_and_compare_eval(runs, capsys):
    from dttt_b200.tools import compare_eval, paired_diff
    files = sorted(f for f in os.listdir(runs["A"]) if f.startswith("eval_") and f.endswith(".npz"))
    assert files, os.listdir(runs["A"])
    step = int(files[-1][5:-4])
    assert paired_diff.main(["--step", str(step), f"A={runs['A']}", f"B={runs['B']}", "--n_boot", "200"]) == 0
    out = capsys.readouterr().out
    assert "| B - A |" in out and "cluster ±" in out and "per-source headline differences" in out
    assert compare_eval.main([str(runs["A"] / files[-1]), str(runs["B"] / files[-1])]) == 0
    out = capsys.readouterr().out
    assert "sources    identical" in out and "loss_1.0" in out


def test_elbo_eval_bound_and_pairing(runs, tmp_path):
    from dttt_b200.tools import elbo_eval
    ck = runs["A"] / _step_dir(runs["A"])
    assert elbo_eval.main(["--ckpt", str(ck), "--n_per_source", "2", "--n_t", "3", "--out", str(tmp_path / "elbo.npz")]) == 0
    d = np.load(tmp_path / "elbo.npz")
    assert d["ce"].shape == (3, 2, 4) and d["count"].shape == (3, 2, 4)
    assert np.all(np.diff(d["count"][:, 0].sum(-1)) > 0)                  # more masked tokens at higher noise levels
    assert np.array_equal(d["count"][:, 0], d["count"][:, 1])             # write on / off score the same masks
    assert np.all(np.isfinite(d["bound"])) and 3.0 < d["bound"][0] < 9.0


def test_grad_noise_decomposition(runs, tmp_path):
    from dttt_b200.tools import grad_noise
    ck = runs["A"] / _step_dir(runs["A"])
    assert grad_noise.main(["--ckpt", str(ck), "--n_seq", "3", "--n_masks", "2", "--out", str(tmp_path / "noise.json")]) == 0
    r = json.load(open(tmp_path / "noise.json"))
    t = r["views_1"]["total"]
    assert t["W"] > 0 and np.isfinite(t["D"]) and np.isfinite(t["G2"])
    assert set(r["views_1"]) >= {"embed", "prefix", "suffix", "total"}
    parts = sum(v["W"] for g, v in r["views_1"].items() if g != "total")
    assert abs(parts - t["W"]) < 1e-6 * abs(t["W"]) + 1e-12


def test_convert_dolma_removes_test_books_and_groups_pages(tmp_path):
    import gzip
    import pyarrow as pa
    import pyarrow.parquet as pq
    from dttt_b200.tools.data import convert_dolma
    rng = np.random.default_rng(0)
    words = lambda n, seed: " ".join(f"w{int(x)}" for x in np.random.default_rng(seed).integers(0, 5000, n))
    book = words(600, 1)
    pq.write_table(pa.table({"url": ["https://www.gutenberg.org/ebooks/4242"], "text": [book], "title": ["The Test Book"]}), tmp_path / "test.parquet")
    recs = [{"id": "a", "text": words(300, 2), "metadata": {"title": "fresh"}},
            {"id": "b", "text": "intro " + book[:2500] + " outro", "metadata": {"title": "copy of the book"}},
            {"id": "c", "text": words(50, 3), "metadata": {"title": "by id", "url": "https://www.gutenberg.org/ebooks/4242"}},
            {"id": "d", "text": words(200, 4), "metadata": {}}]
    (tmp_path / "src").mkdir()
    with gzip.open(tmp_path / "src" / "part0.json.gz", "wt") as fh:
        fh.writelines(json.dumps(r) + "\n" for r in recs)
    rc = convert_dolma.main(["--src", str(tmp_path / "src"), "--out", str(tmp_path / "out"), "--pg19_test", str(tmp_path / "test.parquet"),
                             "--stride", "4", "--workers", "1"])
    assert rc == 0
    t = pq.read_table(tmp_path / "out" / "part0.parquet")
    assert t.column("id").to_pylist() == ["a", "d"]
    removed = [json.loads(l) for l in open(tmp_path / "out" / "removed.jsonl")]
    assert {r["id"] for r in removed} == {"b", "c"} and any("id 4242" in r["why"] for r in removed)
    s = json.load(open(tmp_path / "out" / "summary.json"))
    assert s["docs_in"] == 4 and s["docs_out"] == 2 and s["removed_by_id"] == 1
    # pages of one volume become one document, in page order
    pages = [{"id": f"p{i}", "item_id": "vol1", "page_num": str(n), "text": f"page {n} " + words(30, 10 + n), "metadata": {}} for i, n in enumerate((2, 10, 1))]
    pages.append({"id": "q", "item_id": "vol2", "page_num": "1", "text": "other volume " + words(30, 99), "metadata": {}})
    (tmp_path / "src2").mkdir()
    with gzip.open(tmp_path / "src2" / "vols.json.gz", "wt") as fh:
        fh.writelines(json.dumps(r) + "\n" for r in pages)
    assert convert_dolma.main(["--src", str(tmp_path / "src2"), "--out", str(tmp_path / "out2"), "--pg19_test", str(tmp_path / "test.parquet"),
                               "--group", "item_id:page_num", "--workers", "1"]) == 0
    t = pq.read_table(tmp_path / "out2" / "vols.parquet")
    assert t.column("id").to_pylist() == ["vol1", "vol2"]
    txt = t.column("text").to_pylist()[0]
    assert txt.index("page 1 ") < txt.index("page 2 ") < txt.index("page 10 ")


def test_round_compare_sections(runs, tmp_path, capsys):
    from dttt_b200.tools import elbo_eval, round_compare
    for n in ("A", "B"):
        ck = runs[n] / _step_dir(runs[n])
        assert elbo_eval.main(["--ckpt", str(ck), "--n_per_source", "2", "--n_t", "2", "--out", str(runs[n] / "elbo.npz")]) == 0
    files = sorted(f for f in os.listdir(runs["A"]) if f.startswith("eval_") and f.endswith(".npz"))
    step = int(files[-1][5:-4])
    capsys.readouterr()
    assert round_compare.main(["--step", str(step), f"A={runs['A']}", f"B={runs['B']}", "--pairs", "B-A"]) == 0
    out = capsys.readouterr().out
    assert "## 8K" in out and "B - A" in out and "## bound" in out and "memory's part" in out


def test_memory_model_counts_kept_graphs_and_the_recomputation_they_save():
    from dttt_b200.tools import memory_model as mm
    c = mm._cfg(os.path.join(ROOT, "configs/b200_1b_8k"))
    base = mm.report(c, 8192, 2, 1, 1)
    kept = mm.report(c, 8192, 2, 1, 1, keep_prefix_layers=12, keep_suffix_chunks=8)
    assert base["kept_graphs_gib"] == 0 and base["hardware_gflop_per_token"] > base["model_gflop_per_token"]
    assert abs(kept["hardware_gflop_per_token"] - kept["model_gflop_per_token"]) < 1e-9          # nothing is recomputed
    assert 55 < kept["kept_graphs_gib"] < 80                                                      # measured: 70.7 GiB for two sequences
    half = mm.report(c, 8192, 2, 1, 1, keep_prefix_layers=6, keep_suffix_chunks=4)
    assert base["hardware_gflop_per_token"] > half["hardware_gflop_per_token"] > kept["hardware_gflop_per_token"]


def test_common_pile_fetch_is_resumable_against_a_fake_hub(tmp_path):
    """Plan -> missing -> fetch -> manifest with a stand-in hub: a second pass fetches only what is missing or has the wrong size."""
    import types
    from dttt_b200.tools.data import download_common_pile as dl
    files = {"a/000.json.gz": 10, "a/001.json.gz": 20, "README.md": 5, "a/002.json.gz": 30}
    api = types.SimpleNamespace(dataset_info=lambda repo, files_metadata: types.SimpleNamespace(
        sha="f" * 40, siblings=[types.SimpleNamespace(rfilename=k, size=v) for k, v in files.items()]))
    plan = dl.plan_source(api, "books", 0)
    assert plan.repo == "common-pile/books_filtered" and [s.path for s in plan.shards] == sorted(k for k in files if k.endswith(".gz"))
    assert plan.nbytes == 60 and len(dl.plan_source(api, "books", 2).shards) == 2
    calls = []

    def download(repo_id, repo_type, revision, filename, local_dir):
        calls.append(filename)
        if filename.endswith("001.json.gz") and calls.count(filename) == 1:
            raise OSError("connection reset")
        path = os.path.join(local_dir, filename)
        os.makedirs(os.path.dirname(path), exist_ok=True)
        with open(path, "wb") as fh:
            fh.write(b"x" * files[filename])

    root = str(tmp_path)
    failed = dl.fetch(plan, dl.missing_shards(plan, root), root, 2, download)
    assert len(failed) == 1 and "001" in failed[0]
    assert [s.path for s in dl.missing_shards(plan, root)] == ["a/001.json.gz"]
    with open(os.path.join(root, "books", "a/000.json.gz"), "wb") as fh:        # a truncated file counts as missing
        fh.write(b"x")
    todo = dl.missing_shards(plan, root)
    assert [s.path for s in todo] == ["a/000.json.gz", "a/001.json.gz"]
    assert dl.fetch(plan, todo, root, 2, download) == [] and dl.missing_shards(plan, root) == []
    man = os.path.join(root, "manifest.json")
    dl.write_manifest(man, {"books": {"revision": plan.revision}})
    assert dl.read_manifest(man)["books"]["revision"] == "f" * 40 and dl.read_manifest(os.path.join(root, "none.json")) == {}
