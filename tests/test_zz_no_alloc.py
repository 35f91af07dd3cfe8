"""The allocation-free entry point of linear + cross-entropy (``dttt_linear_ce_fwd_static``): called through its exported
C symbol, twice in a row, against the ordinary entry point.  Collected last on purpose (it must hold after every other
test has used the device, and alone)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _sym():
    from dttt_b200.ops import _lib
    lib = _lib.lib()
    f = lib.dttt_linear_ce_fwd_static
    vp, ll, i = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
    f.restype = i
    f.argtypes = [vp, vp, vp, i, i, i, ll, ll, vp, vp, vp, vp, vp]
    e = lib.dttt_linear_ce_static_strerror
    e.restype = ctypes.c_char_p
    e.argtypes = [i]
    return f, e


def test_static_scratch_matches_ordinary_entry_point_twice():
    from dttt_b200.ops import _lib, kernels
    f, strerror = _sym()
    torch.manual_seed(11)
    N, K, V = 640, 512, 20000
    E = (torch.randn(V, K, device="cuda") * 0.05).to(torch.bfloat16)
    st = _lib.status_tensor("cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):
        h = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        y = torch.randint(0, V, (N,), device="cuda", dtype=torch.int32)
        tgt = torch.zeros(N, device="cuda")
        lse = torch.empty(N, device="cuda")
        nll = torch.empty(N, device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_stats().get("allocation.all.allocated", 0)
        free_before = torch.cuda.mem_get_info()[0]
        rc = f(h.data_ptr(), E.data_ptr(), y.data_ptr(), N, V, K, h.stride(0), E.stride(0), tgt.data_ptr(), lse.data_ptr(),
               nll.data_ptr(), st.data_ptr(), stream)
        assert rc == 0, strerror(rc)
        torch.cuda.synchronize()
        assert torch.cuda.memory_stats().get("allocation.all.allocated", 0) == before      # nothing went through torch's allocator
        if call == 1:
            # ... and nothing went to the driver behind its back either: once the first call has loaded the kernels, a call
            # leaves the device's free memory where it was (a raw cudaMalloc / cudaFree inside the library would move it)
            assert torch.cuda.mem_get_info()[0] == free_before
        _lib.check_status()
        lse_ref, nll_ref = kernels.linear_ce_fwd(h, E, y)
        torch.cuda.synchronize()
        assert (lse - lse_ref).abs().max().item() < 1e-4, call
        assert (nll - nll_ref).abs().max().item() < 1e-4, call
        logits = h.float() @ E.float().t()
        assert (lse - torch.logsumexp(logits, -1)).abs().max().item() < 2e-3


def test_static_scratch_refuses_oversize():
    f, strerror = _sym()
    h = torch.zeros(8, 64, device="cuda", dtype=torch.bfloat16)
    rc = f(h.data_ptr(), h.data_ptr(), 0, 8192, 131072, 64, 64, 64, 0, 0, 0, 0, None)
    assert rc == -10
    assert b"exceeds the fixed scratch" in strerror(rc)
