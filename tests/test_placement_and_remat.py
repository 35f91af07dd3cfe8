"""Fast weights in a subset of the suffix layers, and what the recompute regions keep.

* placement (the reference's tests/test_placement.py): a model whose second suffix layer is plain equals the default layout (a fast
  weight in every suffix layer) with that layer's post-norm scale set to zero: its memory term is then exactly zero whatever W,
  its inner gradient is zero (the clip norm is unchanged), so loss and shared gradients agree;
* regions (the reference's tests/test_remat_scan.py pins the memory half with XLA's memory analysis): the bytes that autograd
  saves for the backward, counted with saved-tensor hooks, drop under recompute regions and rise again with every layer / chunk
  step that ``keep_prefix_layers`` / ``keep_suffix_chunks`` exempts; values are covered by tests/test_objective_invariance.py.
"""
import dataclasses as dc

import torch

from util import Batch, ComputeWeights, Net, loss_and_grads, loss_config, loss_fn, make_engine, rng, tiny_model


def test_a_plain_suffix_layer_equals_a_fast_layer_with_a_zero_post_norm():
    a = make_engine(mc=tiny_model(suffix_len=2, fast_layers=(2,)))
    b = make_engine(mc=tiny_model(suffix_len=2))
    for k in a.store.names():
        va, vb = a.store.gather_full(k), b.store.gather_full(k).clone()
        if va.shape == vb.shape:
            vb.copy_(va)
        else:                                             # leading axis = fast layers: the first is shared, the second is the plain one
            vb[0].copy_(va[0])
            if k == "prime_post_norm.weight":
                vb[1].zero_()
        b.store.load_full(k, vb)
    b.store.sync_compute()
    ids = torch.randint(1, 120, (2, 32), generator=torch.Generator().manual_seed(4))
    la, ga, sa = loss_and_grads(a, ids, loss_config(a.tc))
    lb, gb, sb = loss_and_grads(b, ids, loss_config(b.tc))
    assert abs(la - lb) < 1e-6
    assert abs(float(sa["inner_grad_norm"]) - float(sb["inner_grad_norm"])) < 1e-6
    for k, g in ga.items():
        h = gb[k] if gb[k].shape == g.shape else gb[k][0:1]
        assert (g - h).abs().max().item() < 1e-6, k
    assert gb["fast_weight.gate.weight"][1].abs().max().item() == 0.0


def _saved_bytes(eng, lc, ids):
    seen = {}

    def pack(t):
        seen[(t.data_ptr(), tuple(t.shape))] = t.numel() * t.element_size()
        return t

    eng.store.zero_grad()
    net = Net(eng.mc, ComputeWeights(eng.store))
    with torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
        loss, _ = loss_fn(net, Batch(ids), rng.key(1), 0, lc)
    total = sum(seen.values())
    loss.backward()
    return total


def test_regions_keep_less_for_the_backward_and_the_keep_knobs_give_it_back():
    eng = make_engine(mc=tiny_model(num_hidden_layers=6, suffix_len=2), seq_len=64)
    lc = loss_config(eng.tc)
    ids = torch.randint(1, 120, (2, 64), generator=torch.Generator().manual_seed(5))
    full = _saved_bytes(eng, dc.replace(lc, remat=False), ids)
    regions = _saved_bytes(eng, dc.replace(lc, remat=True), ids)
    some = _saved_bytes(eng, dc.replace(lc, remat=True, keep_prefix_layers=2, keep_suffix_chunks=4), ids)
    everything = _saved_bytes(eng, dc.replace(lc, remat=True, keep_prefix_layers=4, keep_suffix_chunks=8), ids)
    assert regions < 0.5 * full, (regions, full)
    assert regions < some < everything, (regions, some, everything)
    assert everything >= 0.9 * full, (everything, full)
