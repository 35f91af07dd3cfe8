"""Worker of the multi-GPU fused-collective test: trains a small model for a few steps on N GPUs (one rank each)
with the optimiser-step collectives either fused over peer memory or done by NCCL, and saves the parameters."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from dttt_b200.engine import Engine  # noqa: E402
from dttt_b200.parallel.mesh import init_distributed, make_mesh  # noqa: E402
from dttt_b200.schema import ModelConfig, TrainConfig  # noqa: E402


def main():
    out, mode = sys.argv[1], sys.argv[2]
    fused, shard = mode in ("1", "shard"), mode == "shard"
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world, local = init_distributed("nccl", timeout_s=120)
    dev = torch.device("cuda", local)
    mesh = make_mesh(0, 1, dev)
    mc = ModelConfig(vocab_size=2048, hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=32, suffix_len=2, chunk_size=64, window_chunks=2, qk_norm=True,
                     mask_token_id=2047, pad_token_id=2046, eos_token_id=2046)
    tc = TrainConfig(seq_len=256, batch_size=2 * world, steps=10, warmup_steps=2, inner_lr_warmup_steps=0, inner_task="causal",
                     outer_shift=True, cart_window=32, fused_ce_block=512, fused_comm=fused, shard_compute=shard)
    eng = Engine(mc, tc, mesh, dev)
    assert eng.store.fused == fused
    if shard:
        assert eng.store.sharded_names
        eng.store.forget_foreign_compute()             # whatever is not this rank's slice must come through the gather
    ids = torch.randint(0, 2000, (2 * world, 256), generator=torch.Generator().manual_seed(0))[2 * rank:2 * rank + 2]
    ms = [eng.train_step(ids, s) for s in range(3)]
    # the reduced gradient of the last step as the optimiser saw it (this rank's slice), gathered over the ranks
    gs = [torch.empty_like(eng.store.grad_shard) for _ in range(world)]
    dist.all_gather(gs, eng.store.grad_shard)
    full = {k: eng.store.gather_full(k).cpu() for k in eng.store.names()}
    lo = {k: eng.store.lo_view(k).float().cpu() for k in eng.store.names()}
    if rank == 0:
        from dttt_b200.parallel import wgather
        torch.save({"params": full, "lo": lo, "metrics": ms, "grad": torch.stack(gs).cpu(), "gather_launches": wgather.LAUNCHES},
                   os.path.join(out, f"fused{'shard' if shard else int(fused)}.pt"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
