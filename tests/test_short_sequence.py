"""Sequences shorter than the attention window: the window slots before the start of the sequence are never read, so a window of
three chunks gives the loss and the gradient of a window that just covers the sequence; segments shorter than the window are
refused (the window they would carry across the boundary is short).  The reference checks the same in tests/test_short_sequence.py."""
import dataclasses as dc

import pytest
import torch

from util import loss_and_grads, loss_config, make_engine, max_diff, tiny_model


@pytest.mark.parametrize("nc,covering", [(1, 1), (2, 1), (3, 2)])
@pytest.mark.parametrize("no_write", [False, True])
def test_a_window_longer_than_the_sequence_is_the_covering_window(nc, covering, no_write):
    C = 8
    ids = torch.randint(1, 110, (2, nc * C), generator=torch.Generator().manual_seed(1))
    res = {}
    for w in (3, covering):
        eng = make_engine(mc=tiny_model(window_chunks=w, chunk_size=C, suffix_len=1, num_hidden_layers=3), seq_len=nc * C)
        lc = dc.replace(loss_config(eng.tc), no_write=no_write)
        res[w] = loss_and_grads(eng, ids, lc)
    assert abs(res[3][0] - res[covering][0]) < 1e-6
    assert max_diff(res[3][1], res[covering][1]) < 1e-6


def test_segments_shorter_than_the_window_are_refused():
    eng = make_engine(mc=tiny_model(window_chunks=3, chunk_size=8))
    ids = torch.randint(1, 110, (2, 32), generator=torch.Generator().manual_seed(2))
    with pytest.raises(ValueError):
        loss_and_grads(eng, ids, dc.replace(loss_config(eng.tc), segment_chunks=2))
