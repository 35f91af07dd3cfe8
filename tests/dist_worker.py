"""Worker for the multi-process CPU tests (gloo): ``python dist_worker.py <case> <out_dir>`` under torchrun-style env."""
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from util import tiny_model, tiny_train  # noqa: E402
from dttt_b200.engine import Engine  # noqa: E402
from dttt_b200.parallel.mesh import init_distributed, make_mesh  # noqa: E402
from dttt_b200.ckpt import store as CK  # noqa: E402


def main():
    case, out = sys.argv[1], sys.argv[2]
    rank, world, _ = init_distributed("gloo", timeout_s=int(os.environ.get("TEST_TIMEOUT_S", "60")))
    fsdp = int(os.environ.get("TEST_FSDP", "0"))
    tp = int(os.environ.get("TEST_TP", "1"))
    mesh = make_mesh(fsdp, tp, torch.device("cpu"))
    mkw = dict(memory="gdn", gdn_heads=2, gdn_head_dim=8, gdn_conv=4, gdn_alternate=True, gdn_chunk=4) if os.environ.get("TEST_GDN") else {}
    tkw = dict(segment_chunks=2) if os.environ.get("TEST_SEGMENTS") else {}
    eng = Engine(tiny_model(**mkw), tiny_train(batch_size=4, fsdp_size=fsdp, tp_size=tp, **tkw), mesh, torch.device("cpu"))
    ids = torch.randint(0, 120, (4, 32), generator=torch.Generator().manual_seed(0))
    n = 4 // mesh.batch_ranks
    mine = ids[mesh.batch_index * n:(mesh.batch_index + 1) * n]
    if case == "train":
        ms = [eng.train_step(mine, s) for s in range(3)]
        full = {k: eng.store.gather_full(k) for k in eng.store.names()}
        d = CK.save(os.path.join(out, "ck"), 2, eng, "h")
        if rank == 0:
            torch.save({"metrics": ms, "params": full, "mesh": mesh.shape()}, os.path.join(out, "result.pt"))
    elif case == "tp_grads":
        # tensor parallel: the group's micro-batch is the whole `ids`; row-wise keys make the draws independent of the split
        from dttt_b200.ttt.scan import Batch
        from dttt_b200.utils import rng
        keys = rng.split(rng.key(11), 4)
        loss, w = eng.grad_of(Batch(ids), keys, 0, weight="sum")
        tot = torch.tensor([loss * w, w], dtype=torch.float64)
        dist.all_reduce(tot)
        eng.store.reduce_grads()
        grads = {k: eng.store.gather_full(k, eng.store.grad_shard) for k in eng.store.names()}
        import dataclasses as dc
        ev_loss, ev = eng.eval_step(Batch(ids), keys, 0, dc.replace(eng.lcfg, per_sequence=True))
        ms = [eng.train_step(ids, s) for s in range(2)]
        full = {k: eng.store.gather_full(k) for k in eng.store.names()}
        d = CK.save(os.path.join(out, "ck"), 1, eng, "h")
        if rank == 0:
            torch.save({"ce_sum": float(tot[0]), "count": float(tot[1]), "grads": grads, "metrics": ms, "params": full,
                        "ev_loss": float(ev_loss), "ev_by_seq": ev["loss_by_seq"], "ev_count": float(ev["mask_count"]),
                        "mesh": mesh.shape()}, os.path.join(out, "result.pt"))
    elif case == "tp_resume":
        # two steps, save, two more; a fresh engine of the same mesh restored from the checkpoint must take the same two steps
        for s in range(2):
            eng.train_step(ids, s)
        d = CK.save(os.path.join(out, "ck"), 2, eng, "h")
        moments = {k: (eng.store.gather_full(k, eng.opt.m), eng.store.gather_full(k, eng.opt.v)) for k in eng.store.names()}
        for s in range(2, 4):
            eng.train_step(ids, s)
        cont = {k: eng.store.gather_full(k) for k in eng.store.names()}
        eng2 = Engine(tiny_model(), tiny_train(batch_size=4, fsdp_size=fsdp, tp_size=tp), mesh, torch.device("cpu"))
        CK.load_weights(d, eng2)
        CK.load_opt(d, eng2)
        eng2.store.sync_compute()
        for s in range(2, 4):
            eng2.train_step(ids, s)
        resumed = {k: eng2.store.gather_full(k) for k in eng2.store.names()}
        if rank == 0:
            torch.save({"cont": cont, "resumed": resumed, "moments": moments, "mesh": mesh.shape()}, os.path.join(out, "result.pt"))
    elif case == "rank_exits":
        # rank 1 leaves between steps (no collective in flight); the others must get an error, not hang
        eng.train_step(mine, 0)
        if rank == 1:
            os._exit(7)
        t0 = time.time()
        try:
            eng.train_step(mine, 1)
            outcome = "no error"
        except Exception as e:                                    # noqa: BLE001
            outcome = type(e).__name__
        with open(os.path.join(out, f"rank{rank}.json"), "w") as fh:
            json.dump({"outcome": outcome, "seconds": time.time() - t0}, fh)
        os._exit(0)
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
