"""Every memory / speed lever is a layout change: the loss and the gradients must not move
(the reference's tests/test_exact_equivalence.py is the model for this file)."""
import dataclasses as dc

import pytest
import torch

from util import loss_and_grads, loss_config, make_engine, max_diff, tiny_model, tiny_train
from dttt_b200.ttt.scan import Batch
from dttt_b200.utils import rng

IDS = torch.randint(0, 120, (2, 32), generator=torch.Generator().manual_seed(0))


@pytest.mark.parametrize("task,shift", [("causal", True), ("mask", False)])
def test_remat_and_segments_do_not_change_loss_or_grads(task, shift):
    eng = make_engine(inner_task=task, outer_shift=shift)
    lc = loss_config(eng.tc)
    l0, g0, _ = loss_and_grads(eng, IDS, dc.replace(lc, remat=False))
    for variant in (dc.replace(lc, remat=True), dc.replace(lc, remat=True, keep_prefix_layers=1, keep_suffix_chunks=2), dc.replace(lc, segment_chunks=2),
                    dc.replace(lc, segment_chunks=2, keep_suffix_chunks=1),
                    dc.replace(lc, segment_chunks=2, remat=False),
                    dc.replace(lc, fused_ce_block=48)):
        l1, g1, _ = loss_and_grads(eng, IDS, variant)
        assert abs(l0 - l1) < 1e-6 and max_diff(g0, g1) < 1e-6
    assert all(v.abs().sum() > 0 for k, v in g0.items()), [k for k, v in g0.items() if v.abs().sum() == 0]


def test_nested_segment_regions_do_not_change_loss_or_grads(monkeypatch):
    from dttt_b200.ttt import scan
    eng = make_engine()
    lc = loss_config(eng.tc)
    l0, g0, _ = loss_and_grads(eng, IDS, dc.replace(lc, remat=False))
    monkeypatch.setattr(scan, "NEST_SEGMENTS_FROM", 2)                  # 4 chunks in segments of 2: every segment its own region
    for variant in (dc.replace(lc, segment_chunks=2), dc.replace(lc, segment_chunks=2, truncate_fast_weight=False, per_token=True)):
        l1, g1, _ = loss_and_grads(eng, IDS, variant)
        assert abs(l0 - l1) < 1e-6 and max_diff(g0, g1) < 1e-6


def test_second_order_is_alive_and_first_order_differs():
    eng = make_engine()
    lc = loss_config(eng.tc)
    l2, g2, _ = loss_and_grads(eng, IDS, lc)
    l1, g1, _ = loss_and_grads(eng, IDS, dc.replace(lc, second_order=False))
    assert abs(l1 - l2) < 1e-6                          # same forward
    assert max_diff(g1, g2) > 1e-4                      # the meta-gradient is a different gradient
    lt, gt, _ = loss_and_grads(eng, IDS, dc.replace(lc, segment_chunks=2, truncate_fast_weight=True))
    assert abs(lt - l2) < 1e-6 and max_diff(gt, g2) > 1e-6


def test_no_write_equals_zero_inner_lr_and_write_moves_w():
    eng = make_engine()
    lc = loss_config(eng.tc)
    la, _, sa = loss_and_grads(eng, IDS, dc.replace(lc, no_write=True))
    lb, _, sb = loss_and_grads(eng, IDS, dc.replace(lc, inner_lr=0.0))
    lw, _, sw = loss_and_grads(eng, IDS, lc)
    assert abs(la - lb) < 1e-6 and abs(la - lw) > 1e-6
    assert float(sw["ttt_drift_rel"]) > 0 and float(sb["ttt_drift_rel"]) == 0 and float(sw["inner_grad_norm"]) > 0


def test_row_keys_make_a_sequence_independent_of_its_batch():
    eng = make_engine()
    lc = dc.replace(loss_config(eng.tc), per_sequence=True)
    keys = rng.split(rng.key(3), 2)
    with torch.no_grad():
        from dttt_b200.ttt.scan import loss_fn
        _, s2 = loss_fn(eng.net(False), Batch(IDS), keys, 0, lc)
        _, s1 = loss_fn(eng.net(False), Batch(IDS[1:]), keys[1:], 0, lc)
    assert torch.allclose(s2["loss_by_seq"][1], s1["loss_by_seq"][0], atol=1e-5)


def test_grad_accumulation_is_one_large_batch():
    eng_a, eng_b = make_engine(batch_size=4), make_engine(batch_size=2, grad_accum=2)
    ids = torch.randint(0, 120, (4, 32), generator=torch.Generator().manual_seed(5))
    # the same masks for the same sequences: row keys through explicit batches
    keys = rng.split(rng.key(9), 4)
    from dttt_b200.models.blocks import Net
    from dttt_b200.parallel.store import ComputeWeights
    from dttt_b200.ttt.scan import loss_fn

    def grads(eng, parts):
        eng.store.zero_grad()
        wsum = 0.0
        for sl in parts:
            cw = ComputeWeights(eng.store)
            loss, st = loss_fn(Net(eng.mc, cw), Batch(ids[sl]), keys[sl], 0, loss_config(eng.tc))
            w = st["mask_count"] + 1e-6
            (loss * w).backward()
            cw.fold_grads()
            wsum += float(w)
        return {k: eng.store.grad_view(k) / wsum for k in eng.store.names()}
    g_full = grads(eng_a, [slice(0, 4)])
    g_acc = grads(eng_b, [slice(0, 2), slice(2, 4)])
    assert max_diff(g_full, g_acc) < 1e-6


@pytest.mark.parametrize("opt", [dict(outer_views=2), dict(self_prior=0.5), dict(window_drop=1.0, window_drop_until=10),
                                 dict(inner_views=2, inner_task="mask", outer_shift=False),
                                 dict(inner_views=2, inner_task="mask", outer_shift=False, inner_views_sequential=True),
                                 dict(inner_from_outer=True), dict(write_off=True, aux_causal_weight=0.5),
                                 dict(inner_update="sign"), dict(inner_update="muon2"), dict(inner_update_frac=0.5),
                                 dict(inner_cart=True, inner_task="mask", outer_shift=False), dict(time_reweighting="linear"),
                                 dict(reread_chunks=2, segment_chunks=2, score_from_chunk=2), dict(per_token=True, per_sequence=True)])
def test_options_run_and_remat_invariant(opt):
    eng = make_engine()
    lc = dc.replace(loss_config(eng.tc), **opt)
    l0, g0, st = loss_and_grads(eng, IDS, dc.replace(lc, remat=False))
    l1, g1, _ = loss_and_grads(eng, IDS, lc)
    assert abs(l0 - l1) < 1e-5 and torch.isfinite(torch.tensor(l0))
    if opt.get("inner_update") in ("sign", "muon2"):
        # these directions have near-singular second derivatives at small entries: a one-ulp difference between
        # the two passes rescales the dominant meta-gradient term, so only the direction is compared
        for k in g0:
            assert torch.nn.functional.cosine_similarity(g0[k].flatten(), g1[k].flatten(), dim=0) > 0.999, k
    else:
        assert max(float((g0[k] - g1[k]).abs().max() / (g0[k].abs().max() + 1e-6)) for k in g0) < 2e-4


def test_write_schemes_run():
    from dttt_b200.ttt.inner import WriteConfig
    for mc_kw, wc in ((dict(), WriteConfig(subchunks=2, subchunk_scale=0.5)), (dict(), WriteConfig(steps=2)),
                      (dict(), WriteConfig(norm_alpha=1.0, norm_cap=8.0)), (dict(), WriteConfig(surprise_gamma=0.5)),
                      (dict(), WriteConfig(subchunks=2, fast_frac=0.25, fast_decay=0.1)),
                      (dict(inner_kvb_head=True), WriteConfig(kvb_weight=0.1)),
                      (dict(inner_kvb_head=True), WriteConfig(kvb_weight=0.1, kvb_value="clean"))):
        eng = make_engine(mc=tiny_model(**mc_kw))
        lc = dc.replace(loss_config(eng.tc), write=wc)
        l0, g0, st = loss_and_grads(eng, IDS, dc.replace(lc, remat=False))
        l1, g1, _ = loss_and_grads(eng, IDS, lc)
        assert abs(l0 - l1) < 1e-5, wc
        assert max(float((g0[k] - g1[k]).abs().max() / (g0[k].abs().max() + 1e-6)) for k in g0) < 1e-3, wc
        assert float(st["ttt_drift_rel"]) > 0


def test_learned_write_controls_distill_mtp_feat_and_gdn():
    cases = [
        (dict(inner_lr_gate=True, inner_token_gate=True, inner_decay=0.01, inner_optimizer=True), dict()),
        (dict(inner_feat_head=True), dict(inner_feat="add")),
        (dict(mtp_head=True), dict(mtp=True)),
        (dict(), dict(distill=True, distill_topk=8)),
        (dict(memory="gdn", gdn_heads=2, gdn_head_dim=8, gdn_chunk=4), dict()),
        (dict(memory="gdn", gdn_heads=2, gdn_head_dim=8, gdn_chunk=8, gdn_conv=4, gdn_alternate=True), dict()),
        (dict(read_block=4), dict()), (dict(window_reach=1), dict()), (dict(suffix_len=3, suffix_plain_top=1), dict()),
        (dict(qk_norm=False, attention_bias=True, tie_word_embeddings=False), dict()),
    ]
    for mkw, lkw in cases:
        eng = make_engine(mc=tiny_model(**mkw))
        lc = dc.replace(loss_config(eng.tc), **lkw)
        l0, g0, st = loss_and_grads(eng, IDS, dc.replace(lc, remat=False))
        l1, g1, _ = loss_and_grads(eng, IDS, lc)
        assert abs(l0 - l1) < 1e-5, (mkw, lkw)
        assert max(float((g0[k] - g1[k]).abs().max() / (g0[k].abs().max() + 1e-6)) for k in g0) < 1e-3, (mkw, lkw)
        assert torch.isfinite(torch.tensor(l0))


def test_emulated_kernel_path_agrees_with_f32(monkeypatch):
    """The control flow a GPU run takes (custom autograd functions, in-place f32 gradient accumulation, staged
    second-order backward) on CPU bf16 tensors, against the plain f32 path."""
    from dttt_b200.ops import gemm
    monkeypatch.setattr(gemm, "EMULATE", True)
    mc = tiny_model(head_dim=16, hidden_size=64, intermediate_size=128)
    ids = torch.randint(0, 120, (2, 32), generator=torch.Generator().manual_seed(2))
    out = {}
    for dt in ("bfloat16", "float32"):
        eng = make_engine(mc=mc, compute_dtype=dt, fused_ce_block=64)
        out[dt] = loss_and_grads(eng, ids, loss_config(eng.tc))
    assert abs(out["bfloat16"][0] - out["float32"][0]) / out["float32"][0] < 0.02
    for k, g in out["float32"][1].items():
        gb = out["bfloat16"][1][k]
        cos = torch.nn.functional.cosine_similarity(g.flatten(), gb.flatten(), dim=0)
        assert cos > 0.97, (k, float(cos))
