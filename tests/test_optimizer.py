"""The outer optimiser against a plain restatement of the reference's ``optax.chain(clip_by_global_norm, adamw(schedule, mask))``
(reference src/ttt/train.py:137-167): schedule, global-norm clip, decay mask by name, the fast-weight template's rate scale."""
import math
import re

import pytest
import torch

from util import make_engine
from dttt_b200.optim import lr_at


def test_schedule_warms_up_stays_flat_and_decays_linearly():
    kw = dict(lr=1e-3, end_lr=1e-4, warmup_steps=10, decay_start=100, decay_end=200)
    assert lr_at(0, **kw) == 0.0
    assert lr_at(5, **kw) == pytest.approx(5e-4)
    assert lr_at(10, **kw) == lr_at(99, **kw) == pytest.approx(1e-3)
    assert lr_at(150, **kw) == pytest.approx(5.5e-4)
    assert lr_at(200, **kw) == lr_at(10_000, **kw) == pytest.approx(1e-4)
    assert lr_at(50, 1e-3, 1e-4, 10) == pytest.approx(1e-3)                     # no decay window: flat for ever


@pytest.mark.parametrize("clip", [0.05, 1e9])
def test_steps_follow_the_restated_adamw(clip):
    eng = make_engine(lr=1e-2, end_lr=1e-3, warmup_steps=2, weight_decay=0.1, grad_clip=clip, fast_weight_lr_scale=0.25)
    st, opt = eng.store, eng.opt
    names = list(st.names())
    nd = re.compile(eng.tc.no_decay_pattern)
    p = {k: st.gather_full(k).clone() for k in names}
    m = {k: torch.zeros_like(v) for k, v in p.items()}
    v2 = {k: torch.zeros_like(v) for k, v in p.items()}
    gen = torch.Generator().manual_seed(0)
    for t in range(1, 4):
        grads = {k: torch.randn(p[k].shape, generator=gen) * 0.1 for k in names}
        st.zero_grad()
        for k in names:
            st.grad_view(k).copy_(grads[k])
        st.reduce_grads()
        out = opt.step()
        gnorm = math.sqrt(sum(float(g.pow(2).sum()) for g in grads.values()))
        assert out["grad_norm"] == pytest.approx(gnorm, rel=1e-5)
        factor = min(1.0, clip / gnorm)
        lr = lr_at(t - 1, 1e-2, 1e-3, 2)
        for k in names:
            g = grads[k] * factor
            m[k] = 0.9 * m[k] + 0.1 * g
            v2[k] = eng.tc.adam_b2 * v2[k] + (1 - eng.tc.adam_b2) * g * g
            upd = (m[k] / (1 - 0.9 ** t)) / ((v2[k] / (1 - eng.tc.adam_b2 ** t)).sqrt() + 1e-8)
            if not nd.search(k):
                upd = upd + 0.1 * p[k]
            scale = 0.25 if k.startswith("fast_weight.") else 1.0
            p[k] = p[k] - lr * scale * upd
            assert torch.allclose(st.gather_full(k), p[k], rtol=2e-5, atol=1e-7), (t, k)
    assert any(nd.search(k) for k in names) and any(not nd.search(k) for k in names)
    assert any(k.startswith("fast_weight.") for k in names)
