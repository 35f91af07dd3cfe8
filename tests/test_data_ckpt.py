import json
import os

import numpy as np
import pytest
import torch

from util import make_engine, tiny_model, tiny_train
from dttt_b200.ckpt import npystream as NS
from dttt_b200.ckpt import store as CK
from dttt_b200.data import prep
from dttt_b200.data.host_masks import MaskMaker, inner_mask_rule, split_perm
from dttt_b200.data.prefetch import Prefetcher
from dttt_b200.data.streams import Plant, Sampler, parse_sources
from dttt_b200.data.synth import write_stream, zipf_tokens


@pytest.fixture(scope="module")
def streams(tmp_path_factory):
    d = tmp_path_factory.mktemp("streams")
    for i, n in enumerate(("a", "b")):
        write_stream(str(d / n), zipf_tokens(150_000, 1024, seed=i, eos=1022, mean_doc=200), 1022, n, 1024)
    return str(d)


def test_zipf_stream_statistics():
    t = zipf_tokens(200_000, 1024, seed=0, eos=1022, mean_doc=200, exclude=(1023,))
    counts = np.bincount(t, minlength=1024)
    assert counts[1023] == 0 and 600 < counts[1022] < 1400                 # ~ n / mean_doc documents
    top = np.sort(counts[:1022])[::-1].astype(float)
    slope = np.polyfit(np.log(np.arange(1, 101)), np.log(top[:100]), 1)[0]
    assert -1.3 < slope < -0.9                                              # Zipf exponent ~ 1.1


def test_hosts_partition_the_global_batch_and_order_is_stateless(streams):
    src = parse_sources(f"a={streams}/a:0.7,b={streams}/b:0.3")
    full = Sampler(src, 256, 8, seed=3, holdout_tokens=20000)
    for step in (0, 7):
        parts = [Sampler(src, 256, 8, seed=3, rank=r, world=4, holdout_tokens=20000).batch(step) for r in range(4)]
        assert (np.concatenate(parts) == full.global_batch(step)).all()
    assert (Sampler(src, 256, 8, seed=3, holdout_tokens=20000).batch(5) == full.batch(5)).all()
    # 16 x 4 reads what 64 x 1 reads: the order depends on batch x accum only
    a = Sampler(src, 256, 4, seed=3, accum=2)
    b = Sampler(src, 256, 8, seed=3, accum=1)
    assert a.hash == b.hash and (np.concatenate([a.global_batch(2), a.global_batch(3)]) == b.global_batch(1)).all()


def test_data_hash_is_path_free_and_sensitive(streams, tmp_path):
    import shutil
    src = parse_sources(f"a={streams}/a:1.0")
    other = tmp_path / "elsewhere"
    shutil.copytree(f"{streams}/a", other / "a")
    h = Sampler(src, 256, 8, seed=3, holdout_tokens=1000).hash
    assert Sampler(parse_sources(f"a={other}/a:1.0"), 256, 8, seed=3, holdout_tokens=1000).hash == h
    assert Sampler(src, 256, 8, seed=4, holdout_tokens=1000).hash != h
    assert Sampler(src, 128, 8, seed=3, holdout_tokens=1000).hash != h
    assert Sampler(src, 256, 8, seed=3, holdout_tokens=1000, plant=Plant(0.5, 8, 16, 32, 2)).hash != h


def test_holdout_is_never_sampled_and_eval_starts_after_an_eos(streams):
    src = parse_sources(f"a={streams}/a:1.0")
    s = Sampler(src, 256, 4, seed=1, holdout_tokens=30000, eos=1022)
    mm = src[0].open()
    assert mm[int(s.eval_start[0]) - 1] == 1022 and s.eval_start[0] >= 150_000 - 30000
    assert s.n_seq[0] == (150_000 - 30000) // 256
    e = s.eval_batch(0, 0)
    assert (e[0] == np.asarray(mm[s.eval_start[0]:s.eval_start[0] + 256])).all()


def test_windows_and_filter(streams, tmp_path):
    w = prep.doc_windows(f"{streams}/a", 64, 10000)
    ln = prep.doc_lengths(f"{streams}/a")
    mm = np.memmap(f"{streams}/a/tokens.u32", dtype="<u4", mode="r")
    assert len(w) and all((np.asarray(mm[o:o + 64]) != 1022).all() for o in w[:50])         # a window never crosses a document
    assert ln.sum() == 150_000
    np.save(prep.windows_path(f"{streams}/a", 64, 10000), w)
    s = Sampler(parse_sources(f"a={streams}/a:1.0"), 64, 4, seed=0, holdout_tokens=10000, windows=[w])
    assert (s.batch(0) != 1022).all()
    f = prep.filter_stream(f"{streams}/a", "long", str(tmp_path), min_doc_tokens=300)
    assert (prep.doc_lengths(f) >= 300).all() and json.load(open(f + "/meta.json"))["num_docs"] == int((ln >= 300).sum())


def test_prefetcher_in_order_and_surfaces_errors(streams):
    s = Sampler(parse_sources(f"a={streams}/a:1.0"), 128, 4, seed=0)
    p = Prefetcher(s, 3, depth=2, pin=False)
    for step in (3, 4, 5):
        assert (p.get(step)[0] == s.batch(step)).all()
    with pytest.raises(RuntimeError, match="out of order"):
        p.get(9)
    p.close()

    class Broken:
        local, T = 1, 8

        def batch(self, step, out=None):
            raise OSError("disk gone")
    q = Prefetcher(Broken(), 0, pin=False)
    with pytest.raises(RuntimeError, match="prefetch thread failed"):
        q.get(0)


def test_host_masks_are_deterministic_and_skip_pad_eos():
    t = zipf_tokens(256, 512, seed=3, eos=500, mean_doc=40).astype(np.int64)
    uni = np.bincount(zipf_tokens(50000, 512, 9), minlength=512).astype(np.int64)
    for mode in ("rare", "docaware"):
        m = inner_mask_rule(t, mode, 64, 500, 500, uni, 0.5, 0.1, 1)
        assert (m == inner_mask_rule(t, mode, 64, 500, 500, uni, 0.5, 0.1, 1)).all() and not m[t == 500].any()
        assert (m.reshape(4, 64).sum(1) <= 32).all()
    p = split_perm(t, "random", 64, 500, 500, 0.5, uni, 0.1, 1)
    assert all(sorted(p[c * 64:(c + 1) * 64]) == list(range(c * 64, (c + 1) * 64)) for c in range(4))
    assert MaskMaker("random", 64, 500, 500).active is False and MaskMaker("rare", 64, 500, 500).active


def test_record_stream_parts_and_single_file(tmp_path):
    arrs = [np.random.randn(300, 17).astype(np.float32), np.asarray(7, np.int32), np.arange(50000, dtype=np.int64)]
    NS.write_records(str(tmp_path / "x.eqx"), arrs, max_bytes=50_000)
    assert len([f for f in os.listdir(tmp_path) if f.startswith("x.eqx.part")]) > 3
    for a, b in zip(arrs, NS.read_records(str(tmp_path / "x.eqx"))):
        assert a.dtype == b.dtype and (a == b).all()
    with open(tmp_path / "y.eqx", "wb") as fh:
        for a in arrs:
            np.save(fh, a)
    assert all((a == b).all() for a, b in zip(arrs, NS.read_records(str(tmp_path / "y.eqx"))))
    os.rename(tmp_path / "x.eqx.part002", tmp_path / "x.eqx.part009")
    with pytest.raises(ValueError, match="not contiguous"):
        NS.PartReader(str(tmp_path / "x.eqx"))


def test_checkpoint_bitwise_resume_prune_and_done_marker(tmp_path):
    ids = torch.randint(0, 120, (2, 32), generator=torch.Generator().manual_seed(0))
    e1 = make_engine()
    for s in range(3):
        e1.train_step(ids, s)
    ck = str(tmp_path / "ck")
    for s in (0, 1, 2):
        p = CK.save(ck, s, e1, "hash", keep=2, extra_state={"data_offset": 0})
    assert CK.complete_steps(ck) == ["step_00000001", "step_00000002"]
    os.remove(os.path.join(ck, "step_00000002", "DONE"))
    assert CK.latest_complete(ck).endswith("step_00000001")                   # a directory without DONE is ignored
    open(os.path.join(ck, "step_00000002", "DONE"), "w").write("ok\n")
    e2 = make_engine()
    CK.load_weights(p, e2); CK.load_opt(p, e2); e2.store.sync_compute()
    m1 = [e1.train_step(ids, s) for s in (3, 4)]
    m2 = [e2.train_step(ids, s) for s in (3, 4)]
    assert all(a["loss"] == b["loss"] and a["grad_norm"] == b["grad_norm"] for a, b in zip(m1, m2))
    assert torch.equal(e1.store.master, e2.store.master)
    st = CK.read_state(p)
    assert st["step"] == 2 and st["data_hash_version"] == 2 and st["data_offset"] == 0
    with pytest.raises(FileNotFoundError):
        CK.resolve_resume(ck, str(tmp_path / "nothing"))


def test_checkpoint_leaf_order_and_shapes_follow_the_reference_tree(tmp_path):
    e = make_engine(mc=tiny_model(inner_optimizer=True, mtp_head=True))
    p = CK.save(str(tmp_path / "ck"), 0, e, "h")
    recs = list(NS.read_records(os.path.join(p, "model.eqx")))
    names = list(e.spec)
    assert names[0] == "embed" and names[1] == "prefix.attn_norm.weight" and names[-1] == "final_norm.weight"
    assert names.index("prime_norm.weight") < names.index("fast_weight.gate.weight") < names.index("inner_precond.0.gate.weight") \
        < names.index("inner_step_log") < names.index("mtp_head.weight")
    assert [tuple(r.shape) for r in recs] == [tuple(s) for s, _ in e.spec.values()] and all(r.dtype == np.float32 for r in recs)
    opt = list(NS.read_records(os.path.join(p, "opt.eqx")))
    assert len(opt) == 2 * len(names) + 2 and opt[0].dtype == np.int32 and opt[-1].dtype == np.int32


def test_init_from_tolerates_new_heads_and_narrows_a_wider_fast_weight(tmp_path):
    wide = make_engine(mc=tiny_model(ttt_intermediate_size=96))
    p = CK.save(str(tmp_path / "ck"), 0, wide, "h")
    narrow = make_engine(mc=tiny_model(ttt_intermediate_size=48, mtp_head=True))
    before = narrow.store.gather_full("mtp_head.weight")
    logs = []
    CK.load_weights(p, narrow, logs.append)
    assert narrow.store.gather_full("fast_weight.gate.weight").shape[-1] == 48
    assert torch.equal(narrow.store.gather_full("mtp_head.weight"), before) and any("narrowed 96 -> 48" in l for l in logs)
    g = wide.store.gather_full("fast_weight.gate.weight").numpy()
    u = wide.store.gather_full("fast_weight.up.weight").numpy()
    d = wide.store.gather_full("fast_weight.down.weight").numpy()
    imp = np.linalg.norm(g, axis=1) * np.linalg.norm(u, axis=1) * np.linalg.norm(d, axis=2)
    keep = np.sort(np.argsort(-imp, axis=1)[:, :48], axis=1)
    assert np.allclose(narrow.store.gather_full("fast_weight.gate.weight").numpy()[0], g[0][:, keep[0]])
    with pytest.raises(ValueError, match="narrower"):
        CK.load_weights(CK.save(str(tmp_path / "ck2"), 0, narrow, "h"), make_engine(mc=tiny_model(ttt_intermediate_size=96)))


def test_prepare_tokenises_parquet_into_a_stream_once(tmp_path):
    """Raw parquet -> ``tokens.u32`` + ``meta.json`` with the shipped tokenizer: one EOS after every document, the directory is
    named by a hash of (files, tokenizer, options) so a second call does nothing, short documents are dropped on request, and
    the grouped form keeps the rows of a group adjacent and in order (a group is kept or dropped as a whole)."""
    import pyarrow as pa
    import pyarrow.parquet as pq
    from util import ROOT
    tokenizer = os.path.join(ROOT, "configs/1b_e2e")
    docs = [f"Document number {i}. " + "The quick brown fox jumps over the lazy dog. " * (i % 5 + 1) for i in range(23)]
    raw = str(tmp_path / "raw.parquet")
    pq.write_table(pa.table({"text": docs}), raw, row_group_size=10)
    out = prep.prepare("toy", [raw], "text", tokenizer, str(tmp_path / "tok"), workers=2)
    meta = json.load(open(os.path.join(out, "meta.json")))
    stream = np.fromfile(os.path.join(out, "tokens.u32"), dtype="<u4")
    eos = meta["tokenizer"]["eos_token_id"]
    assert meta["num_docs"] == 23 and meta["num_tokens"] == len(stream) and int((stream == eos).sum()) == 23 and stream[-1] == eos
    lengths = prep.doc_lengths(out)
    assert len(lengths) == 23 and int(lengths.sum()) == len(stream) and (np.diff(lengths[:5]) > 0).all()
    assert prep.prepare("toy", [raw], "text", tokenizer, str(tmp_path / "tok"), workers=2) == out          # already prepared
    longer = prep.prepare("toy", [raw], "text", tokenizer, str(tmp_path / "tok"), min_doc_tokens=40, workers=2)
    assert longer != out and json.load(open(os.path.join(longer, "meta.json")))["num_docs"] == int((lengths - 1 >= 40).sum())
    counts = prep.unigram_counts([out], 128256)
    assert counts.sum() == len(stream) and counts[eos] == 23
    pages = pa.table({"book": ["b", "a", "b", "a", "a"], "page": ["2", "1", "1", "3", "2"],
                      "text": ["b two.", "a one.", "b one.", "a three.", "a two."]})
    grouped_raw = str(tmp_path / "pages.parquet")
    pq.write_table(pages, grouped_raw)
    grouped = prep.prepare_grouped("books", [grouped_raw], "text", "book", "page", tokenizer, str(tmp_path / "tok"), 0, workers=1)
    gmeta = json.load(open(os.path.join(grouped, "meta.json")))
    assert gmeta["num_groups"] == 2 and gmeta["num_docs"] == 5 and len(prep.doc_lengths(grouped)) == 5      # pages stay documents
    from transformers import PreTrainedTokenizerFast
    tok = PreTrainedTokenizerFast.from_pretrained(tokenizer)
    text = tok.decode([int(t) for t in np.fromfile(os.path.join(grouped, "tokens.u32"), dtype="<u4") if t != eos])
    assert text.replace(" ", "") == "aone.atwo.athree.bone.btwo."                                           # groups and pages in order


def test_host_targets_match_recorded_vectors():
    """The ranking terms, the 3-gram hash and the shuffle seeding are a contract shared with the reference
    (src/ttt/inner_masks.py): the same tokens must give the same targets.  Vectors recorded from the loop-per-chunk statement."""
    toks = np.random.default_rng(7).integers(0, 40, 64)
    toks[5] = 39; toks[30] = 39; toks[40:44] = 38
    uni = np.random.default_rng(8).integers(1, 500, 40).astype(np.int64)
    m = inner_mask_rule(toks, "docaware", 16, 39, 38, uni, 0.5, 0.1, 3)
    assert "".join("1" if x else "0" for x in m) == "1110101010100001111010110101000000110110000011111110001011101000"
    p = split_perm(toks, "docaware", 16, 39, 38, 0.5, uni, 0.1, 3)
    assert p.tolist() == [3, 5, 7, 9, 11, 12, 13, 14, 1, 2, 6, 0, 4, 10, 15, 8, 19, 21, 24, 26, 28, 29, 30, 31, 18, 22, 25, 20, 23, 17,
                          16, 27, 32, 33, 36, 39, 40, 41, 42, 43, 37, 44, 47, 34, 46, 45, 35, 38, 51, 52, 53, 55, 59, 61, 62, 63, 54, 56,
                          57, 49, 50, 60, 58, 48]
    # a chunk of pads has no ranked target: the split order takes its targets from the end of the context
    pads = np.full(16, 38)
    q = split_perm(pads, "rare", 16, 39, 38, 0.5, uni, 0.1, 0)
    assert sorted(q.tolist()) == list(range(16)) and q[:8].tolist() == list(range(8))
