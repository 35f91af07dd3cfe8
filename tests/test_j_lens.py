"""Memory probes (tools.j_lens): the lens is the identity at the last layer, the first-order effect matches a finite
difference, a transplant at the slot's own inputs changes nothing, and the four probes run end to end on a tiny model."""
import argparse

import numpy as np
import pytest
import torch

ARGS = ["--random_init", "--model_config", "configs/tiny_smoke", "--synthetic", "200", "--n_per_source", "1"]


@pytest.fixture(scope="module")
def reader_ids():
    from dttt_b200.tools.j_lens import _cli
    ap = argparse.ArgumentParser()
    _cli.add_common(ap)
    a = ap.parse_args(ARGS + ["--seq_len", "512"])
    torch.manual_seed(0)
    return _cli.load(a)[:2]


def _read_setup(reader, ids, chunk=4):
    C = reader.C
    seq = torch.as_tensor(ids[:1])
    st, _ = reader.write_pass(seq, chunk)
    x = seq[:, chunk * C:(chunk + 1) * C]
    m = torch.zeros(1, C, dtype=torch.bool)
    m[0, 5::3] = True
    return st, x, m


def test_lens_is_identity_at_the_last_layer(reader_ids):
    from dttt_b200.tools.j_lens import core
    reader, ids = reader_ids
    st, x, m = _read_setup(reader, ids)
    L = reader.mc.num_hidden_layers
    J = core.fit_lens(reader, [(x, m, st)], ("out", L - 1), block=32)
    assert torch.allclose(J, torch.eye(J.shape[0]), atol=1e-5)
    J0 = core.fit_lens(reader, [(x, m, st)], ("out", 0), block=32)
    assert torch.isfinite(J0).all() and (J0 - torch.eye(J0.shape[0])).abs().max() > 1e-3


def test_direct_effect_matches_a_finite_difference(reader_ids):
    from dttt_b200.tools.j_lens import core
    reader, ids = reader_ids
    st, x, m = _read_setup(reader, ids)
    xm = torch.where(m, torch.full_like(x, reader.mc.mask_token_id), x)
    point = ("mem", 0)
    with torch.no_grad():
        _, cap = reader.forward(xm, st, capture=[("mem_part", 0)])
    mem = cap[("mem_part", 0)].float()
    d = core.direct_effect(reader, xm, st, point, mem)
    eps = 1e-3
    with torch.no_grad():
        lp = reader.unembed(reader.forward(xm, st, inject={point: eps * mem})[0])
        lm = reader.unembed(reader.forward(xm, st, inject={point: -eps * mem})[0])
    fd = (lp - lm) / (2 * eps)
    assert (d - fd).abs().max().item() < 2e-2 * fd.abs().max().item() + 1e-4


def test_transplant_at_own_inputs_is_a_no_op(reader_ids):
    from dttt_b200.tools.j_lens import core
    reader, ids = reader_ids
    st, x, m = _read_setup(reader, ids)
    xm = torch.where(m, torch.full_like(x, reader.mc.mask_token_id), x)
    S = reader.mc.suffix_len
    with torch.no_grad():
        h0, cap = reader.forward(xm, st, capture=[("mem_in", i) for i in range(S)])
    slots = torch.tensor([[3, 7, 11]])
    x_src = [torch.gather(cap[("mem_in", i)], 1, slots[..., None].expand(-1, -1, cap[("mem_in", i)].shape[-1]))
             for i in range(S) if ("mem_in", i) in cap]
    with torch.no_grad():
        h1, _ = reader.forward(xm, st, transplant=core.Transplant(slots, x_src))
    # only the first fast layer sees exactly its own input again; with one fast layer the read is unchanged
    if len(x_src) == 1:
        assert torch.allclose(h0, h1, atol=1e-5)
    else:
        assert torch.isfinite(h1).all()


def test_probes_run_end_to_end(tmp_path):
    from dttt_b200.tools.j_lens import context_learning, doc_switch, key_transplant, memory_distance
    assert key_transplant.main(ARGS + ["--seq_len", "512", "--length", "16", "--cue", "4", "--out", str(tmp_path / "kt.npz")]) == 0
    assert set(np.load(tmp_path / "kt.npz").files) >= set(key_transplant.VARIANTS)
    assert memory_distance.main(ARGS + ["--seq_len", "512", "--distances", "2,4", "--length", "16", "--cue", "4", "--out", str(tmp_path / "d.npz")]) == 0
    d = np.load(tmp_path / "d.npz")
    assert d["gain_copy"].shape == (1, 2, 6) and np.isfinite(d["ceiling"]).all()
    assert doc_switch.main(ARGS + ["--seq_len", "512", "--n_a", "3", "--n_b", "2", "--n_per_pair", "1", "--t", "0.5", "--out", str(tmp_path / "s.npz")]) == 0
    s = np.load(tmp_path / "s.npz")
    assert s["ce"].shape == (1, 1, 5, 3) and np.allclose(s["ce"][0, 0, 3, 1], s["ce"][0, 0, 3, 2])      # at the switch reset == off
    assert context_learning.main(ARGS + ["--seq_len", "640", "--targets", "8", "--tasks", "span,key1", "--out", str(tmp_path / "c.npz")]) == 0
    assert np.load(tmp_path / "c.npz")["recall"].shape == (1, 2, 1)
