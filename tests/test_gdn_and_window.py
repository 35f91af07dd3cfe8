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
