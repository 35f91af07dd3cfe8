"""Leak tests: a prediction never had access to what it predicts (the reference's tests/test_inner_task.py and
tests/test_outer_shift.py check the same properties on its model).

* objective level: changing a token of chunk c' leaves the loss of every chunk before c' bitwise unchanged (window attention,
  the clean stream's keys, the inner writes and the reads all look backwards only) and does change chunk c';
* inner stream, causal task: the inner objective restricted to slot i (which predicts token i + 1) is unchanged when the hidden
  state or the token of any slot j > i + 1 changes, and changes with slot i itself.
"""
import pytest
import torch

from util import Batch, ComputeWeights, Net, loss_config, loss_fn, make_engine, rng
from dttt_b200.ttt import inner as IN


def _chunk_losses(eng, lc, ids):
    net = Net(eng.mc, ComputeWeights(eng.store))
    with torch.no_grad():
        _, stats = loss_fn(net, Batch(ids), rng.key(7), 3, lc)
    return stats["loss_by_chunk"].clone(), stats["inner_loss"].clone()


@pytest.mark.parametrize("task,shift", [("causal", True), ("mask", False)])
def test_a_later_chunk_never_changes_an_earlier_chunks_loss(task, shift):
    eng = make_engine(inner_task=task, outer_shift=shift)
    lc = loss_config(eng.tc)
    C = eng.mc.chunk_size
    ids = torch.randint(1, 120, (2, 4 * C), generator=torch.Generator().manual_seed(0))
    base, _ = _chunk_losses(eng, lc, ids)
    for c in (1, 2, 3):
        flipped = ids.clone()
        flipped[:, c * C + C // 2] = (ids[:, c * C + C // 2] + 17) % 100 + 1          # a slot in the middle of chunk c
        got, _ = _chunk_losses(eng, lc, flipped)
        assert torch.equal(got[:c], base[:c]), (c, got, base)
        assert not torch.equal(got[c:], base[c:]), c


def test_the_causal_inner_slot_sees_nothing_after_its_target():
    eng = make_engine(inner_task="causal", outer_shift=True)
    net = eng.net(train=False)
    mc = eng.mc
    B, C, S = 2, mc.chunk_size, mc.suffix_len
    g = torch.Generator().manual_seed(1)
    h = torch.randn(B, C, mc.hidden_size, generator=g) * 0.5
    toks = torch.randint(1, 120, (B, C), generator=g)
    kv = [(torch.randn(B, mc.window_chunks * C, mc.num_key_value_heads, mc.head_dim, generator=g),
           torch.randn(B, mc.window_chunks * C, mc.num_key_value_heads, mc.head_dim, generator=g)) for _ in range(S)]
    pos = torch.arange(2 * C, 3 * C)[None].expand(B, C)
    W = [tuple(t.clone() for t in w) for w in net.template_fast(B)]

    def objective(hh, tt, slot):
        mask = torch.zeros(B, C)
        mask[:, slot] = 1.0
        tgt = torch.cat([tt[:, 1:], tt[:, -1:]], 1)                                  # slot i predicts token i + 1
        with torch.no_grad():
            return IN.inner_objective(W, net, hh, tgt, mask, kv, pos, 2, 0, pos_q=pos + 1, own="causal")[0]

    i = 3
    base = objective(h, toks, i)
    for j in range(i + 2, C):                                                         # strictly after the target
        h2, t2 = h.clone(), toks.clone()
        h2[:, j] += 1.0
        t2[:, j] = (toks[:, j] + 5) % 100 + 1
        assert torch.equal(objective(h2, t2, i), base), j
    t2 = toks.clone()
    t2[:, i + 1] = (toks[:, i + 1] + 5) % 100 + 1                                     # the label itself
    assert not torch.equal(objective(h, t2, i), base)
    for j in (0, i):                                                                  # visible slots do matter
        h2 = h.clone()
        h2[:, j] += 1.0
        assert not torch.equal(objective(h2, toks, i), base), j
