"""The CTA-pair GEMM (tcgen05 cta_group::2, ``csrc/gemm_pair_tcgen05.cu``) against f32 ``torch.matmul``: every operand
layout, ragged edges, batches, f32 accumulation into an existing buffer."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture()
def pair_on():
    from dttt_b200.ops import gemm
    old = gemm.PAIR, gemm.PAIR_MIN_N, gemm.PAIR_MIN_TILES
    gemm.PAIR, gemm.PAIR_MIN_N, gemm.PAIR_MIN_TILES = True, 256, 0
    yield gemm
    gemm.PAIR, gemm.PAIR_MIN_N, gemm.PAIR_MIN_TILES = old


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 512, 256), (1024, 2048, 2048), (384, 768, 192), (300, 520, 136), (2048, 8192, 2048)])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_pair_gemm_layouts(pair_on, M, N, K, ta, tb):
    from dttt_b200.ops import _lib
    gemm = pair_on
    torch.manual_seed(M + N + K)
    if (ta and M % 8) or (not tb and N % 8) or (not ta and K % 8) or (tb and K % 8):
        pytest.skip("row strides must be multiples of 8 elements")
    a = torch.randn((K, M) if ta else (M, K), device="cuda").to(torch.bfloat16)
    b = torch.randn((N, K) if tb else (K, N), device="cuda").to(torch.bfloat16)
    n0 = gemm.LAUNCHES
    c = gemm.gemm_raw(a, b, ta, tb)
    torch.cuda.synchronize()
    _lib.check_status()
    assert gemm.LAUNCHES == n0 + 1
    want = (a.float().t() if ta else a.float()) @ (b.float().t() if tb else b.float())
    err = (c.float() - want).abs().max().item()
    assert err < 0.02 * want.abs().max().item() + 0.05, err


def test_pair_gemm_batched_and_f32_accumulate(pair_on):
    from dttt_b200.ops import _lib
    gemm = pair_on
    torch.manual_seed(1)
    a = torch.randn(3, 512, 256, device="cuda").to(torch.bfloat16)
    b = torch.randn(3, 256, 768, device="cuda").to(torch.bfloat16)
    c = gemm.gemm_raw(a, b, False, False)
    assert (c.float() - a.float() @ b.float()).abs().max().item() < 0.5
    x = torch.randn(4096, 512, device="cuda").to(torch.bfloat16)
    g = torch.randn(4096, 1024, device="cuda").to(torch.bfloat16)
    acc = torch.randn(512, 1024, device="cuda")
    want = acc + 0.5 * (x.float().t() @ g.float())
    from dttt_b200.ops._lib import lib, status_tensor, stream_ptr
    import ctypes
    st = status_tensor(x.device)
    vp = ctypes.c_void_p
    # the accumulating epilogue is not routed to the pairs by default: call the entry point directly
    rc = lib().dttt_gemm_pair_bf16(vp(x.data_ptr()), vp(g.data_ptr()), vp(acc.data_ptr()), 512, 1024, 4096, 1, x.stride(0), g.stride(0),
                                   acc.stride(0), 0, 0, 0, 1, 1, 1, 1, 0.5, vp(st.data_ptr()), vp(stream_ptr()))
    assert rc == 0
    torch.cuda.synchronize()
    _lib.check_status()
    assert (acc - want).abs().max().item() < 1e-2 * want.abs().max().item()


def test_pair_gemm_matches_single_cta_kernel_bitwise_enough(pair_on):
    gemm = pair_on
    torch.manual_seed(2)
    a = torch.randn(2048, 2048, device="cuda").to(torch.bfloat16)
    b = torch.randn(2048, 4096, device="cuda").to(torch.bfloat16)
    c2 = gemm.gemm_raw(a, b, False, False)
    gemm.PAIR = False
    c1 = gemm.gemm_raw(a, b, False, False)
    assert (c1.float() - c2.float()).abs().max().item() < 0.26       # one bf16 ulp at the magnitude of the entries (~64)
