import numpy as np
import torch

from util import tiny_model
from dttt_b200.ops import reference as ref
from dttt_b200.ttt import objective as OBJ
from dttt_b200.utils import rng


def test_threefry_known_vector():
    a, b = rng.threefry2x32(torch.tensor(0x13198A2E), torch.tensor(0x03707344), torch.tensor(0x243F6A88), torch.tensor(0x85A308D3))
    assert (int(a), int(b)) == (0xC4923A9C, 0x483DF7A0)


def test_key_derivations_are_stateless_and_batched():
    k = rng.key(42)
    s = rng.split(k, 4)
    assert s.shape == (4, 2) and len({tuple(r.tolist()) for r in s}) == 4
    assert torch.equal(rng.split(k, 4)[:2], rng.split(k, 2))           # counter based: a prefix of a longer split
    kb = torch.stack([rng.fold_in(k, 3), rng.fold_in(k, 9)])
    assert torch.equal(rng.fold_in(k.expand(2, 2), torch.tensor([3, 9])), kb)
    u = rng.uniform(kb, (1000,))
    assert u.shape == (2, 1000) and 0 <= u.min() and u.max() < 1 and abs(u.mean() - 0.5) < 0.03
    assert torch.equal(u[1], rng.uniform(kb[1], (1000,)))
    n = rng.normal(k, (20000,))
    assert abs(n.mean()) < 0.03 and abs(n.std() - 1) < 0.03


def test_q_sample_row_keys_do_not_depend_on_batch_shape():
    ids = torch.randint(0, 100, (4, 64))
    keys = rng.split(rng.key(5), 4)
    x4, t4, m4 = OBJ.q_sample(keys, ids, None, 127)
    x2, t2, m2 = OBJ.q_sample(keys[1:3], ids[1:3], None, 127)
    assert torch.equal(x4[1:3], x2) and torch.equal(t4[1:3], t2)
    lm = torch.zeros(4, 64, dtype=torch.bool); lm[:, 10:20] = True
    _, _, m = OBJ.q_sample(rng.key(1), ids, lm, 127, t=torch.ones(4))
    assert torch.equal(m, lm)


def test_cart_band_correlate_matches_direct_sum():
    k = ref.cart_kernel(0.1, 16)
    assert k[16] == 0 and torch.isclose(k[17], torch.tensor(0.05)) and torch.isclose(k[18], torch.tensor(0.045))
    x = (torch.rand(3, 100) < 0.5).float()
    out = ref.band_correlate(x, k)
    direct = torch.zeros_like(out)
    for t in range(100):
        for d in range(-16, 17):
            if 0 <= t + d < 100:
                direct[:, t] += k[d + 16] * x[:, t + d]
    assert torch.allclose(out, direct, atol=1e-5)


def test_inner_masks_views_and_pads():
    mc = tiny_model()
    chunks = torch.randint(0, 100, (3, 5, 32)); chunks[..., -4:] = mc.pad_token_id
    keys = rng.split(rng.key(0), 15).reshape(3, 5, 2)
    x, m = OBJ.inner_masks(keys, chunks, -1.0, (0.5, 1.0), mc.mask_token_id, mc.pad_token_id)
    assert not m[..., -4:].any() and (x[m] == mc.mask_token_id).all() and (x[~m] == chunks[~m]).all()
    x2, m2 = OBJ.inner_masks(keys, chunks, -1.0, (0.5, 1.0), mc.mask_token_id, mc.pad_token_id, views=2)
    assert torch.equal(m2[..., 0, :], m) and (m2.sum(-2) == (chunks != mc.pad_token_id)).all()      # complementary
    _, m3 = OBJ.inner_masks(keys, chunks, 0.25, (0.5, 1.0), mc.mask_token_id, mc.pad_token_id)
    assert 0.15 < m3[..., :-4].float().mean() < 0.35
    _, m4 = OBJ.inner_masks(keys, chunks, -1.0, (0.2, 0.8), mc.mask_token_id, mc.pad_token_id, views=3, view_mode="strata")
    assert m4.shape == (3, 5, 3, 32)
    _, m5 = OBJ.inner_masks(keys, chunks, 0.5, (0.5, 1.0), mc.mask_token_id, mc.pad_token_id, span=4.0)
    assert m5.shape == (3, 5, 32)
