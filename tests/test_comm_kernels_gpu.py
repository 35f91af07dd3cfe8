"""The two optimiser-step collectives of ``csrc/comm_fused.cu`` on fixed buffers against ``torch``.

The kernels take a table of device pointers ("rank r's buffer as seen from this GPU") and never wait on a peer, so the
arithmetic can be checked on ONE device: the buffers of ``world`` ranks are ordinary allocations on it and every rank's
launch runs in turn.  (With several GPUs the same table holds CUDA-IPC pointers; ``tests/test_fused_comm_gpu.py`` runs that.)"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _table(tensors):
    return (ctypes.c_void_p * len(tensors))(*[ctypes.c_void_p(t.data_ptr()) for t in tensors])


@pytest.mark.parametrize("world", [1, 2, 4])
def test_reduce_scatter_sumsq_equals_sum_of_slices(world):
    from dttt_b200.parallel import symm
    torch.manual_seed(world)
    n_total, scale = 4096 * world, 0.25
    grads = [torch.randn(n_total, device="cuda") for _ in range(world)]
    n = n_total // world
    for me in range(world):
        out = torch.full((n,), float("nan"), device="cuda")
        sumsq = torch.zeros(1, device="cuda")
        symm.reduce_scatter_sumsq(_table(grads), world, me, me * n, n, scale, out, sumsq)
        # the kernel adds in ring order starting at its own copy
        want = torch.zeros(n, device="cuda")
        for k in range(world):
            want += grads[(me + k) % world][me * n:(me + 1) * n]
        want *= scale
        torch.cuda.synchronize()
        assert torch.equal(out, want), me
        assert abs(sumsq.item() - want.double().pow(2).sum().item()) < 1e-4 * want.double().pow(2).sum().item()


@pytest.mark.parametrize("world,bf16", [(1, True), (2, True), (4, True), (2, False)])
def test_adamw_allgather_updates_the_shard_and_every_copy(world, bf16):
    from dttt_b200.parallel import symm
    torch.manual_seed(7)
    n = 2048
    lr, b1, b2, eps, wd, gscale, t = 3e-3, 0.9, 0.95, 1e-8, 0.1, 0.5, 3
    bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t
    copies = [torch.zeros(n * world, device="cuda", dtype=torch.bfloat16 if bf16 else torch.float32) for _ in range(world)]
    for me in range(world):
        p, g = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
        m, v = 0.1 * torch.randn(n, device="cuda"), 0.01 * torch.rand(n, device="cuda")
        p0, m0, v0 = p.clone(), m.clone(), v.clone()
        symm.adamw_allgather(p, m, v, g, lr, b1, b2, eps, wd, bc1, bc2, gscale, _table(copies), world, me, me * n, bf16)
        torch.cuda.synchronize()
        x = g * gscale
        m_ref = b1 * m0 + (1 - b1) * x
        v_ref = b2 * v0 + (1 - b2) * x * x
        p_ref = p0 - lr * ((m_ref / bc1) / ((v_ref / bc2).sqrt() + eps) + wd * p0)
        assert torch.allclose(m, m_ref, rtol=1e-6, atol=1e-7) and torch.allclose(v, v_ref, rtol=1e-6, atol=1e-9)
        assert torch.allclose(p, p_ref, rtol=2e-6, atol=1e-7)
        for r in range(world):                                  # every rank's compute copy received this shard
            got = copies[r][me * n:(me + 1) * n]
            assert torch.equal(got, p.to(got.dtype)), (me, r)
    for r in range(world):                                      # and nothing outside the shards was touched
        assert copies[r].numel() == n * world
