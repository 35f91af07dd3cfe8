"""The GDN-memory model end to end, the visible window (``window_reach`` / ``window_drop``) and the self-prior read, on tiny random
models (the reference's tests/test_gdn_model.py and tests/test_window_self_prior.py check the same properties).

* GDN: the loss is finite, the state carries across chunks (inner rate 0 = the empty state = the no-memory twin differs from chunk 1
  on and not at chunk 0), the segmented scan equals the whole one, the new modules belong to the fast-weight parameter group;
* window: a model with ``window_reach`` 0 equals the full model under ``window_drop`` 1 (same weights, same draws) and differs from
  the full window; past ``window_drop_until`` the window is full again;
* self-prior: probability 0 is the plain scan, 0.5 changes the meta-gradient, and everything stays finite.
"""
import dataclasses as dc

import torch

from util import Batch, ComputeWeights, Net, loss_and_grads, loss_config, loss_fn, make_engine, max_diff, rng, tiny_model
from dttt_b200.optim import group_of


def _by_chunk(eng, lc, ids, step=3):
    net = Net(eng.mc, ComputeWeights(eng.store))
    with torch.no_grad():
        loss, stats = loss_fn(net, Batch(ids), rng.key(5), step, lc)
    return float(loss), stats["loss_by_chunk"].clone()


def test_gdn_memory_carries_across_chunks_and_segments_equal_the_whole():
    eng = make_engine(mc=tiny_model(memory="gdn", gdn_heads=2, gdn_head_dim=8, gdn_chunk=4, window_chunks=1))
    lc = loss_config(eng.tc)
    ids = torch.randint(1, 120, (2, 32), generator=torch.Generator().manual_seed(0))
    loss, with_memory = _by_chunk(eng, lc, ids)
    _, empty_state = _by_chunk(eng, dc.replace(lc, inner_lr=0.0), ids)
    assert torch.isfinite(torch.tensor(loss))
    assert torch.equal(with_memory[:1], empty_state[:1])                      # nothing has been written before chunk 0
    assert not torch.equal(with_memory[1:], empty_state[1:])                  # later chunks read what earlier ones wrote
    l_whole, g_whole, _ = loss_and_grads(eng, ids, lc)
    l_seg, g_seg, _ = loss_and_grads(eng, ids, dc.replace(lc, segment_chunks=2))
    assert abs(l_whole - l_seg) < 1e-6 and max_diff(g_whole, g_seg) < 1e-6
    gdn_leaves = [k for k in g_whole if k.startswith("gdn.")]
    assert gdn_leaves and all(group_of(k) == "fast_weight" for k in gdn_leaves)
    assert all(g_whole[k].abs().sum() > 0 for k in gdn_leaves), [k for k in gdn_leaves if g_whole[k].abs().sum() == 0]


def test_window_reach_zero_is_the_full_model_with_the_window_dropped():
    full = make_engine(mc=tiny_model(window_chunks=2))
    own_only = make_engine(mc=tiny_model(window_chunks=2, window_reach=0))
    for k in full.store.names():
        own_only.store.load_full(k, full.store.gather_full(k))
    own_only.store.sync_compute()
    ids = torch.randint(1, 120, (2, 32), generator=torch.Generator().manual_seed(1))
    lc = loss_config(full.tc)
    steps = 20
    dropped = dc.replace(lc, window_drop=1.0, window_drop_until=steps)
    a, a_chunks = _by_chunk(own_only, lc, ids)
    b, b_chunks = _by_chunk(full, dropped, ids, step=3)
    c, c_chunks = _by_chunk(full, lc, ids)
    assert abs(a - b) < 1e-6 and torch.allclose(a_chunks, b_chunks, atol=1e-6)
    assert abs(a - c) > 1e-5                                                   # the window matters
    d, _ = _by_chunk(full, dropped, ids, step=steps + 1)                       # past window_drop_until: the full window again
    assert abs(d - c) < 1e-6


def test_self_prior_zero_is_the_plain_scan_and_a_half_changes_the_meta_gradient():
    eng = make_engine()
    lc = loss_config(eng.tc)
    ids = torch.randint(1, 120, (2, 32), generator=torch.Generator().manual_seed(2))
    l0, g0, _ = loss_and_grads(eng, ids, lc)
    l_zero, g_zero, _ = loss_and_grads(eng, ids, dc.replace(lc, self_prior=0.0))
    assert l0 == l_zero and max_diff(g0, g_zero) == 0.0
    l_half, g_half, _ = loss_and_grads(eng, ids, dc.replace(lc, self_prior=0.5, window_drop=0.5, window_drop_until=100))
    assert all(torch.isfinite(v).all() for v in g_half.values()) and torch.isfinite(torch.tensor(l_half))
    l_one, g_one, _ = loss_and_grads(eng, ids, dc.replace(lc, self_prior=1.0))
    assert abs(l_one - l0) > 1e-7 and max_diff(g_one, g0) > 1e-7


def _loss_and_stats(eng, lc, ids, step=3):
    net = Net(eng.mc, ComputeWeights(eng.store))
    with torch.no_grad():
        loss, stats = loss_fn(net, Batch(ids), rng.key(5), step, lc)
    return float(loss), {k: v.clone() for k, v in stats.items()}


def test_write_off_keeps_the_inner_loss_but_never_moves_w_and_the_auxiliary_weight_adds_it():
    """The auxiliary-loss control (the reference's tests/test_aux_causal.py): ``write_off`` runs the inner stream for its
    cross-entropy only; ``aux_causal_weight`` adds that cross-entropy to the outer objective."""
    eng = make_engine(inner_task="causal", outer_shift=True)
    lc = loss_config(eng.tc)
    ids = torch.randint(1, 120, (2, 32), generator=torch.Generator().manual_seed(3))
    l_on, s_on = _loss_and_stats(eng, lc, ids)
    l_off, s_off = _loss_and_stats(eng, dc.replace(lc, write_off=True), ids)
    assert float(s_on["ttt_delta_norm"]) > 0 and float(s_off["ttt_delta_norm"]) == 0.0
    assert float(s_off["inner_loss"]) > 0 and torch.isfinite(s_off["inner_loss"])
    l_none, s_none = _loss_and_stats(eng, dc.replace(lc, no_write=True), ids)
    assert abs(l_off - l_none) < 1e-6                                          # reading W_0 either way
    for w in (0.5, 2.0):
        l_aux, s_aux = _loss_and_stats(eng, dc.replace(lc, write_off=True, aux_causal_weight=w), ids)
        assert abs((l_aux - l_off) - w * float(s_aux["inner_loss"])) < 1e-5, (w, l_aux, l_off, float(s_aux["inner_loss"]))
        assert abs(float(s_aux["main_loss"]) - l_off) < 1e-6


def test_the_shifted_outer_loss_scores_the_masked_targets_from_slot_one_on():
    """With ``outer_shift`` slot i predicts token i + 1: the first token of a sequence is never a target, so the scored count is
    the number of masked tokens after position 0 (the reference's tests/test_outer_shift.py, invariant 3)."""
    eng = make_engine(inner_task="causal", outer_shift=True, time_reweighting="none")
    lc = dc.replace(loss_config(eng.tc), per_token=True, per_sequence=True)
    ids = torch.randint(1, 120, (3, 32), generator=torch.Generator().manual_seed(4))
    keys = torch.stack([rng.fold_in(rng.key(9), j) for j in range(3)])
    net = Net(eng.mc, ComputeWeights(eng.store))
    with torch.no_grad():
        loss, st = loss_fn(net, Batch(ids), keys, 0, lc)
    scored = st["mask_by_token"] > 0.5
    assert torch.isfinite(loss) and float(st["mask_count"]) == float(scored.sum())
    assert torch.allclose(st["mask_by_seq"], scored.sum(1).float())
    assert not bool(scored[:, 0].any())                                        # per-token arrays are indexed by the TARGET token
    assert bool(scored[:, 1:].any())


def test_the_reread_layout_scores_the_same_tail_under_the_same_masks():
    """Re-read evaluation (the reference's tests/test_reread.py): the first n chunks run twice with the window restarted at the
    second pass and only the tail is scored; its outer masks are exactly those of the single pass, so the benefit of re-reading is a
    paired difference."""
    eng = make_engine(mc=tiny_model(window_chunks=2), seq_len=64)
    lc = dc.replace(loss_config(eng.tc), segment_chunks=2, score_from_chunk=2)
    ids = torch.randint(1, 120, (2, 64), generator=torch.Generator().manual_seed(0))
    keys = torch.stack([rng.fold_in(rng.key(9), j) for j in range(2)])
    net = Net(eng.mc, ComputeWeights(eng.store))
    with torch.no_grad():
        single, s1 = loss_fn(net, Batch(ids), keys, 3, lc)
        again, s2 = loss_fn(net, Batch(ids), keys, 3, dc.replace(lc, reread_chunks=2))
    assert torch.equal(s1["mask_by_chunk"], s2["mask_by_chunk"]) and float(s1["mask_by_chunk"][0]) == 0.0
    assert float(s1["mask_count"]) == float(s2["mask_count"])
    assert torch.isfinite(again) and float(again) != float(single)             # the memory has seen the first chunks twice
