import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from dttt_b200.engine import Engine, loss_config  # noqa: E402
from dttt_b200.models.blocks import Net  # noqa: E402
from dttt_b200.parallel.store import ComputeWeights  # noqa: E402
from dttt_b200.schema import ModelConfig, TrainConfig  # noqa: E402
from dttt_b200.ttt.scan import Batch, loss_fn  # noqa: E402
from dttt_b200.utils import rng  # noqa: E402


def tiny_model(**kw) -> ModelConfig:
    base = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=4, num_attention_heads=4,
                num_key_value_heads=2, head_dim=8, suffix_len=2, chunk_size=8, window_chunks=2, mask_token_id=127,
                pad_token_id=126, eos_token_id=126)
    base.update(kw)
    return ModelConfig(**base)


def tiny_train(**kw) -> TrainConfig:
    base = dict(compute_dtype="float32", fused_ce_block=0, cart_window=8, inner_task="causal", outer_shift=True, lr=1e-2,
                warmup_steps=2, inner_lr_warmup_steps=0, steps=20, seq_len=32, batch_size=2)
    base.update(kw)
    return TrainConfig(**base)


def make_engine(mc=None, tc=None, **tkw) -> Engine:
    return Engine(mc or tiny_model(), tc or tiny_train(**tkw), device=torch.device("cpu"))


def loss_and_grads(eng: Engine, ids, lc, key=None, step=0, batch=None):
    eng.store.zero_grad()
    cw = ComputeWeights(eng.store)
    net = Net(eng.mc, cw)
    loss, stats = loss_fn(net, batch or Batch(ids), rng.key(1) if key is None else key, step, lc)
    loss.backward()
    cw.fold_grads()
    return loss.item(), {k: eng.store.grad_view(k).clone() for k in eng.store.names()}, stats


def max_diff(a: dict, b: dict) -> float:
    return max((a[k] - b[k]).abs().max().item() for k in a)
