"""Decoding: sequential blocks == chunk-parallel logits; the write while decoding == the write while training;
determinism and every sampler option (the reference's tests/test_generate.py and test_write_schemes.py are the model)."""
import dataclasses as dc
import os

import pytest
import torch

from util import loss_config, make_engine, tiny_model
from dttt_b200 import generate as G
from dttt_b200.ckpt import store as CK
from dttt_b200.ttt import inner as IN
from dttt_b200.ttt.scan import Batch, loss_fn
from dttt_b200.utils import rng

IDS = torch.randint(0, 120, (2, 32), generator=torch.Generator().manual_seed(3))


def test_sequential_blocks_equal_chunk_parallel_logits():
    eng = make_engine()
    net = eng.net(train=False)
    C = eng.mc.chunk_size
    with torch.no_grad():
        full = net.forward_logits(IDS)
        state = G.init_state(net, 2)
        for c in range(IDS.shape[1] // C):
            pos = torch.arange(c * C, (c + 1) * C)[None].expand(2, C)
            logits = G.block_forward(net, IDS[:, c * C:(c + 1) * C], pos, state)[0]
            assert torch.allclose(logits, full[:, c * C:(c + 1) * C], atol=2e-4), c
            state = G.commit_block(net, IDS[:, c * C:(c + 1) * C], pos, state, rng.key(0), 0.0, 1.0, 0.75, 0, inner_task="causal")


@pytest.mark.parametrize("wc", [IN.WriteConfig(), IN.WriteConfig(subchunks=2, subchunk_scale=0.5), IN.WriteConfig(norm_alpha=1.0, norm_cap=8.0)])
def test_the_write_is_the_same_in_training_and_decoding(wc):
    eng = make_engine()
    net = eng.net(train=False)
    C = eng.mc.chunk_size
    lc = dc.replace(loss_config(eng.tc), write=wc)
    with torch.no_grad():
        _, st = loss_fn(net, Batch(IDS), rng.key(0), 0, lc)
        state = G.init_state(net, 2)
        for c in range(IDS.shape[1] // C):
            pos = torch.arange(c * C, (c + 1) * C)[None].expand(2, C)
            state = G.commit_block(net, IDS[:, c * C:(c + 1) * C], pos, state, rng.key(0), 1.0, 1.0, 0.75, 0, inner_task="causal", wc=wc)
        drift = IN.drift_stats(state.W, net.template_fast(2))
    assert abs(float(drift["ttt_delta_norm"]) - float(st["ttt_delta_norm"])) < 1e-4 * float(st["ttt_delta_norm"])


@pytest.mark.parametrize("opts,kw", [(G.DecodeOpts(), {}), (G.DecodeOpts(order="random"), dict(temperature=1.0)),
                                     (G.DecodeOpts(threshold=0.05), {}), (G.DecodeOpts(presence_penalty=1.0, priority="margin"), {}),
                                     (G.DecodeOpts(remask_loop=2, remask_k=3, priority="entropy"), dict(temperature=0.7)),
                                     (G.DecodeOpts(subblock=4), dict(outer_shift=True, inner_task="causal")),
                                     (G.DecodeOpts(), dict(inner_task="split", inner_mask_mode="random")),
                                     (G.DecodeOpts(), dict(inner_mask_mode="rare", inner_views=1))])
def test_generate_options_are_deterministic_and_keep_the_prompt(opts, kw):
    eng = make_engine()
    net = eng.net(train=False)
    prompt = IDS[0, :11]
    a = G.generate(net, prompt, 14, rng.key(5), steps=4, fused_ce_block=0, opts=opts, **kw)
    b = G.generate(net, prompt, 14, rng.key(5), steps=4, fused_ce_block=0, opts=opts, **kw)
    assert a.shape == (25,) and torch.equal(a, b) and torch.equal(a[:11], prompt)
    assert (a != eng.mc.mask_token_id).all()


def test_read_block_decoding_and_cli_from_a_checkpoint(tmp_path, capsys):
    eng = make_engine(mc=tiny_model(read_block=4))
    out = G.generate(eng.net(train=False), IDS[0, :5], 12, rng.key(1), steps=4, fused_ce_block=0, outer_shift=True, inner_task="causal")
    assert out.shape == (17,)
    plain = make_engine()
    d = CK.save(str(tmp_path / "ck"), 0, plain, "h")
    G.main(["--ckpt", d, "--prompt_ids", "5,6,7,8", "--max_new_tokens", "6", "--steps", "2", "--inner_task", "causal",
            "--outer_shift", "true"])
    printed = capsys.readouterr().out.strip().split(",")
    assert len(printed) == 6 and all(0 <= int(x) < 128 for x in printed)
