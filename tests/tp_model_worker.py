"""Worker of the tensor-parallel model test on GPUs: one gradient of the training loss (second order through the write)
with the trunk's projections split over 2 ranks and the fused all-gather / reduce-scatter GEMM kernels in the path; rank 0
saves the loss sum and the re-assembled gradients for comparison with a one-GPU run of the same model."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from dttt_b200.engine import Engine  # noqa: E402
from dttt_b200.ops import _lib  # noqa: E402
from dttt_b200.parallel.mesh import init_distributed, make_mesh  # noqa: E402
from dttt_b200.schema import ModelConfig, TrainConfig  # noqa: E402
from dttt_b200.ttt.scan import Batch  # noqa: E402
from dttt_b200.utils import rng  # noqa: E402


def configs(tp):
    mc = ModelConfig(vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=3, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=64, suffix_len=2, chunk_size=128, window_chunks=2, mask_token_id=2047,
                     pad_token_id=2046, eos_token_id=2046)
    tc = TrainConfig(seq_len=512, batch_size=2, steps=10, warmup_steps=2, inner_lr_warmup_steps=0, inner_task="causal", outer_shift=True,
                     cart_window=32, fused_ce_block=512, tp_size=tp)
    return mc, tc


def run(eng, out, tag, rank):
    ids = torch.randint(0, 2000, (2, 512), generator=torch.Generator().manual_seed(0))
    keys = rng.split(rng.key(11), 2)
    loss, w = eng.grad_of(Batch(ids), keys, 0, weight="sum")
    tot = torch.tensor([loss * w, w], dtype=torch.float64, device=eng.device)
    if dist.is_initialized():
        dist.all_reduce(tot)
    eng.store.reduce_grads()
    grads = {k: eng.store.gather_full(k, eng.store.grad_shard).cpu() for k in eng.store.names()}
    m = eng.train_step(ids, 0)
    torch.cuda.synchronize()
    _lib.check_status()
    if rank == 0:
        torch.save({"ce_sum": float(tot[0]), "count": float(tot[1]), "grads": grads, "finite": m["finite"]}, os.path.join(out, f"{tag}.pt"))


def main():
    out, tp = sys.argv[1], int(sys.argv[2])
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    if tp > 1:
        rank, world, local = init_distributed("nccl", timeout_s=120)
    else:
        rank, local = 0, 0
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    mc, tc = configs(tp)
    eng = Engine(mc, tc, make_mesh(0, tp, dev), dev)
    run(eng, out, f"tp{tp}", rank)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
