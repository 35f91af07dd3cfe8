"""The read (stream A, and the extra outer views) and the clean pass (stream B) of a chunk step may go through the suffix in
one pass (``Net.suffix_forward_streams``) whenever they use the same memory.  It must be the same arithmetic: equal losses
and equal gradients to the stream-by-stream path, for the objective's variants that reach it."""
import pytest
import torch

from util import make_engine, tiny_model, tiny_train


def _step(flag, mc, tc):
    from dttt_b200.ttt import scan
    was = scan.STREAMS_TOGETHER
    scan.STREAMS_TOGETHER = flag
    try:
        eng = make_engine(mc=mc, tc=tc)
        ids = torch.randint(0, 100, (tc.batch_size, tc.seq_len), generator=torch.Generator().manual_seed(3))
        m = eng.train_step(ids, 0)
        return m, {k: eng.store.grad_view(k).clone() for k in eng.store.names()}
    finally:
        scan.STREAMS_TOGETHER = was


@pytest.mark.parametrize("mkw,tkw", [
    (dict(), dict()),
    (dict(), dict(outer_shift=False)),
    (dict(), dict(outer_views=2)),
    (dict(window_chunks=1), dict(inner_task="mask")),
    (dict(), dict(second_order=False)),
    (dict(inner_kvb_head=True), dict(inner_kvb_weight=0.1, inner_kvb_value="clean")),      # the clean pass also hands out (x, p_out)
])
def test_one_pass_for_read_and_clean_equals_stream_by_stream(mkw, tkw):
    mc, tc = tiny_model(**mkw), tiny_train(**tkw)
    a, ga = _step(True, mc, tc)
    b, gb = _step(False, mc, tc)
    assert a["finite"] == 1.0 and abs(a["loss"] - b["loss"]) < 1e-6 * max(1.0, abs(b["loss"]))
    for k in ga:
        scale = gb[k].abs().max().item() + 1e-12
        assert (ga[k] - gb[k]).abs().max().item() < 1e-5 * scale + 1e-9, k


def test_the_one_pass_path_is_taken():
    """(a spy on the method: the default configuration goes through it once per chunk)"""
    from dttt_b200.models.blocks import Net
    calls = []
    orig = Net.suffix_forward_streams

    def spy(self, *a, **k):
        calls.append(1)
        return orig(self, *a, **k)
    Net.suffix_forward_streams = spy
    try:
        mc, tc = tiny_model(), tiny_train()
        _step(True, mc, tc)
    finally:
        Net.suffix_forward_streams = orig
    assert len(calls) >= tc.seq_len // mc.chunk_size
