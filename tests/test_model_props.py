"""Model and probe properties the reference checks one by one: initialisation statistics, the first loss near ln V, the
gradient-noise estimate of accumulated micro-batches, the recurrence / rarity / neighbour labels and the planted-recall
batches of the evaluation probes."""
import math

import numpy as np
import torch

from util import make_engine, tiny_model
from dttt_b200.eval import probes as PR
from dttt_b200.models import params as P


def test_init_statistics_are_stable_and_the_first_loss_is_near_ln_v():
    mc = tiny_model(hidden_size=64, intermediate_size=128)
    a, b = dict(P.iter_init(mc, 3)), dict(P.iter_init(mc, 3))
    assert all(torch.equal(a[k], b[k]) for k in a)                            # a function of (seed, leaf, layer) only
    assert not torch.equal(a["embed"], dict(P.iter_init(mc, 4))["embed"])
    for name, (shape, kind) in P.param_spec(mc).items():
        t = a[name]
        assert tuple(t.shape) == tuple(shape)
        if kind == "normal" and t.numel() > 2000:
            assert abs(t.std().item() / mc.initializer_range - 1) < 0.1 and abs(t.mean().item()) < 0.2 * mc.initializer_range, name
        if kind == "ones":
            assert torch.all(t == 1)
    # slicing the stacked leaves per layer draws the same values: layer l of a 4-layer model == layer l of a 3-layer prefix...
    eng = make_engine(batch_size=2)
    ids = torch.randint(0, 120, (2, 32), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        logits = eng.net(train=False).forward_logits(ids)
    ce = torch.nn.functional.cross_entropy(logits.flatten(0, 1), ids.flatten()).item()
    assert abs(ce - math.log(eng.mc.vocab_size)) < 0.3                         # an untrained model is uniform over the vocabulary


def test_grad_accumulation_reports_a_noise_scale():
    eng = make_engine(batch_size=2, grad_accum=3)
    ids = torch.randint(0, 120, (3, 2, 32), generator=torch.Generator().manual_seed(2))
    m = eng.train_step(ids, 0)
    assert "grad_noise_scale" in m and m["grad_norm_micro"] > 0
    # micro-batch gradients are noisier than their mean: |g_small|^2 > |g_full|^2 on average
    assert m["grad_norm_micro"] > 0.5 * m["grad_norm"]
    one = make_engine(batch_size=2).train_step(ids[0], 0)
    assert "grad_noise_scale" not in one


def test_recurrence_rarity_and_neighbour_labels():
    C, W = 8, 2
    doc = np.arange(100, 164)
    ctx = np.concatenate([np.arange(10, 30), doc])                            # a previous document, then ours
    seq_start = 20
    seq = ctx.copy()
    seq[seq_start + 40:seq_start + 44] = seq[seq_start + 2:seq_start + 6]     # 4-gram repeated 38 tokens later: beyond the window
    seq[seq_start + 50:seq_start + 54] = seq[seq_start + 44:seq_start + 48]   # and one 6 tokens later: within
    cls = PR.recurrence_classes(seq, seq_start, 64, np.array([0, seq_start]), C, W)
    assert cls[43] == 0 and cls[53] == 1 and cls[10] == 2
    counts = np.array([100, 50, 25, 10, 5, 0])
    bins = PR.rarity_bins(counts)
    assert bins[0] == 0 and bins[-1] == 2 and list(bins) == sorted(bins)
    scored = np.array([[True, False, True, True]])
    assert PR.neighbour_classes(scored).tolist() == [[2 + 0, 2 * 1 + 1, 2 * 0 + 1, 2 * 1 + 1]]


def test_planted_probe_batches_are_paired_and_scored_where_expected():
    C, W, L, cue = 8, 2, 6, 2
    g = np.random.default_rng(0)
    local = g.integers(3, 100, size=(3, 8 * C)).astype(np.int32)
    js = [5, 6, 7]
    beyond, lm_b = PR.planted_probe_batch(local, js, 12345, C, W, L, cue, "beyond", "alt")
    within, lm_w = PR.planted_probe_batch(local, js, 12345, C, W, L, cue, "within", "alt")
    none, lm_n = PR.planted_probe_batch(local, js, 12345, C, W, L, cue, "none", "alt")
    assert np.array_equal(lm_b, lm_w) and np.array_equal(lm_b, lm_n)          # the same scored slots in every placement
    assert np.array_equal(none, local)
    cs, ct, cw = PR.planted_chunks(8, W)
    assert (cs, ct, cw) == (1, W + 3, W + 2)
    for r in range(3):
        sc = np.flatnonzero(lm_b[r])
        assert len(sc) == (L - cue) // 2 and sc.min() >= ct * C and sc.max() < (ct + 1) * C
        b = sc.min() - cue - 1
        span = beyond[r, b:b + L]
        src = local[r, cs * C:(cs + 1) * C]
        assert any(np.array_equal(span, src[o:o + L]) for o in range(C - L + 1))          # the copy is a span of chunk 1
        assert any(np.array_equal(span, within[r, cw * C + o:cw * C + o + L]) for o in range(C - L + 1))
    blk, lm_blk = PR.planted_probe_batch(local, js, 12345, C, W, L, cue, "beyond", "block")
    assert lm_blk.sum(1).tolist() == [L - cue] * 3
