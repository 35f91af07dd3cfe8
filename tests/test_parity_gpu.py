"""Loss parity of the GPU path against the f32 CPU statement over a short training run.

The model is sized so that every hand-written kernel family is on the path: head dimension 64 and chunks of 128 (both
attention kernels and the second-order score kernel), a vocabulary that takes the fused linear + cross-entropy, the plain
inner step with its hand-written meta-gradient.  Both runs start from the same counter-RNG initialisation and see the same
batches and masks; after every optimiser step the unweighted masked-token cross-entropy on one fixed held-out batch is
recorded.  The two curves must stay within 1 % of each other at step 20 (the bar the reference sets for a
re-implementation) and the loss must have moved."""
import dataclasses as dc

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(device, dtype, steps, head_dim=64, qk_norm=False):
    from dttt_b200.engine import Engine
    from dttt_b200.ops import gemm, kernels
    from dttt_b200.schema import ModelConfig, TrainConfig
    from dttt_b200.ttt.scan import Batch
    from dttt_b200.utils import rng
    mc = ModelConfig(vocab_size=4096, hidden_size=256, intermediate_size=512, num_hidden_layers=3, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=head_dim, suffix_len=2, chunk_size=128, window_chunks=2, qk_norm=qk_norm,
                     mask_token_id=4095, pad_token_id=4094, eos_token_id=4094)
    tc = TrainConfig(seq_len=512, batch_size=4, steps=steps, lr=2e-3, end_lr=2e-3, warmup_steps=2, inner_lr_warmup_steps=0,
                     inner_task="causal", outer_shift=True, cart_window=64, fused_ce_block=2048, compute_dtype=dtype, seed=7)
    eng = Engine(mc, tc, device=torch.device(device))
    g = torch.Generator().manual_seed(1)
    # Zipf-like ids so that there is something to learn in 20 steps
    ranks = torch.arange(1, 4001, dtype=torch.float64)
    p = (ranks ** -1.1) / (ranks ** -1.1).sum()
    draw = lambda n: torch.multinomial(p, n, replacement=True, generator=g)
    held = draw(4 * 512).view(4, 512)
    t = (torch.arange(4, dtype=torch.float32) + 0.5) / 4
    lcfg = dc.replace(eng.lcfg, time_reweighting="none")
    keys = rng.split(rng.key(99), 4)
    curve = []
    n0 = gemm.LAUNCHES + kernels.LAUNCHES
    for s in range(steps):
        m = eng.train_step(draw(4 * 512).view(4, 512), s)
        assert m["finite"] == 1.0
        loss, _ = eng.eval_step(Batch(held, outer_t=t), keys, 0, lcfg)
        curve.append(float(loss))
    return curve, gemm.LAUNCHES + kernels.LAUNCHES - n0


def test_twenty_steps_bf16_kernels_track_the_f32_statement():
    from dttt_b200.ops import _lib
    steps = 20
    gpu, launches = _run("cuda", "bfloat16", steps)
    _lib.check_status()
    cpu, _ = _run("cpu", "float32", steps)
    assert launches > 1000                                        # the GPU run went through the hand-written kernels
    assert cpu[0] - cpu[-1] > 0.05                                # the model learned something, so the comparison means something
    for s, (a, b) in enumerate(zip(gpu, cpu)):
        assert abs(a - b) / b < (0.01 if s == steps - 1 else 0.02), (s, a, b)


def test_head_dimension_128_with_qk_norm_tracks_the_f32_statement():
    """The reference model's own geometry in small (heads of 128, QK-norm): forward `attn_fwd2_kernel<128>`, backward
    `attn_bwd128_kernel`, the second order on the row kernel.  Ten steps, 2 % at every step."""
    from dttt_b200.ops import _lib
    steps = 10
    gpu, launches = _run("cuda", "bfloat16", steps, head_dim=128, qk_norm=True)
    _lib.check_status()
    cpu, _ = _run("cpu", "float32", steps, head_dim=128, qk_norm=True)
    assert launches > 500
    for s_, (a, b) in enumerate(zip(gpu, cpu)):
        assert abs(a - b) / b < 0.02, (s_, a, b)
