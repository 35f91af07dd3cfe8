"""Numerics of every hand-written kernel against a plain PyTorch f32 statement of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _status():
    yield
    from dttt_b200.ops import _lib
    torch.cuda.synchronize()
    _lib.check_status()


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-12)


@pytest.mark.parametrize("M,N,K,ta,tb,batch", [(256, 256, 128, 0, 0, 1), (300, 520, 200, 0, 1, 1), (384, 512, 256, 1, 0, 3),
                                              (512, 128, 512, 1, 1, 1), (2048, 2048, 1024, 0, 0, 2), (130, 72, 1032, 0, 1, 1)])
def test_gemm_layouts(M, N, K, ta, tb, batch):
    from dttt_b200.ops import gemm
    torch.manual_seed(0)
    lead = (batch,) if batch > 1 else ()
    a = torch.randn(*lead, *((K, M) if ta else (M, K)), device="cuda", dtype=torch.bfloat16)
    b = torch.randn(*lead, *((N, K) if tb else (K, N)), device="cuda", dtype=torch.bfloat16)
    c = gemm.gemm_raw(a, b, bool(ta), bool(tb))
    ref = (a.transpose(-1, -2) if ta else a).float() @ (b.transpose(-1, -2) if tb else b).float()
    assert _rel(c, ref) < 1e-2


@pytest.mark.parametrize("M,N,K,ta,tb,batch", [(512, 512, 256, 0, 0, 1), (300, 520, 200, 0, 1, 1), (384, 512, 256, 1, 0, 3),
                                              (640, 264, 512, 1, 1, 1), (2048, 2048, 1024, 0, 0, 2), (130, 272, 1032, 0, 1, 1),
                                              (4096, 1024, 2048, 1, 0, 1)])
def test_gemm_256_row_tiles(M, N, K, ta, tb, batch):
    """The 256 x 256 tile form (two row halves sharing every B tile) forced on, all four layouts, ragged edges, f32 accumulate."""
    from dttt_b200.ops import gemm
    torch.manual_seed(1)
    lead = (batch,) if batch > 1 else ()
    a = torch.randn(*lead, *((K, M) if ta else (M, K)), device="cuda", dtype=torch.bfloat16)
    b = torch.randn(*lead, *((N, K) if tb else (K, N)), device="cuda", dtype=torch.bfloat16)
    ref = (a.transpose(-1, -2) if ta else a).float() @ (b.transpose(-1, -2) if tb else b).float()
    gemm.set_tile_form(1)
    try:
        c = gemm.gemm_raw(a, b, bool(ta), bool(tb))
        acc = torch.ones(*lead, M, N, device="cuda", dtype=torch.float32)
        gemm.gemm_raw(a, b, bool(ta), bool(tb), torch.float32, out=acc, accumulate=True, alpha=0.5)
        gemm.gemm_raw(a, b, bool(ta), bool(tb), torch.float32, out=acc, accumulate=True, alpha=0.5)
    finally:
        gemm.set_tile_form(-1)
    assert _rel(c, ref) < 1e-2
    assert _rel(acc - 1.0, ref) < 1e-2


def test_gemm_f32_accumulate_and_views():
    from dttt_b200.ops import gemm
    torch.manual_seed(1)
    a = torch.randn(512, 640, device="cuda", dtype=torch.bfloat16)[:, :256]          # row stride 640
    b = torch.randn(256, 384, device="cuda", dtype=torch.bfloat16)
    out = torch.ones(512, 384, device="cuda")
    gemm.gemm_raw(a, b, False, False, torch.float32, out=out, accumulate=True, alpha=0.5)
    assert _rel(out, 1.0 + 0.5 * (a.float() @ b.float())) < 1e-5


@pytest.mark.parametrize("M,N,K,batch", [(1000, 520, 264, 1), (136, 96, 72, 1), (4096, 2048, 512, 1), (304, 264, 136, 3)])
@pytest.mark.parametrize("ta", [False, True])
def test_gemm_f32_accumulate_ragged_edges(M, N, K, batch, ta):
    """C += A B into f32 (the weight-gradient form: whole-line reductions staged through shared memory) with rows, columns and
    contraction lengths that are not multiples of the tile, twice into the same buffer, batched too."""
    from dttt_b200.ops import _lib, gemm
    torch.manual_seed(M + N)
    lead = (batch,) if batch > 1 else ()
    a = torch.randn(*lead, *((K, M) if ta else (M, K)), device="cuda").to(torch.bfloat16)
    b = torch.randn(*lead, K, N, device="cuda").to(torch.bfloat16)
    out = torch.full((*lead, M, N), 0.25, device="cuda")
    for _ in range(2):
        gemm.gemm_raw(a, b, ta, False, torch.float32, out=out, accumulate=True)
    torch.cuda.synchronize()
    _lib.check_status()
    want = 0.25 + 2.0 * ((a.transpose(-1, -2) if ta else a).float() @ b.float())
    assert _rel(out, want) < 1e-5


def test_mm_autograd_double_backward():
    from dttt_b200.ops import gemm
    torch.manual_seed(2)
    a = torch.randn(128, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = gemm.mm(a, b)
    (ga,) = torch.autograd.grad((y.float() ** 2).sum(), a, create_graph=True)
    (gb2,) = torch.autograd.grad(ga.float().pow(2).sum(), b)
    a32, b32 = a.detach().float().requires_grad_(), b.detach().float().requires_grad_()
    (ga_r,) = torch.autograd.grad(((a32 @ b32) ** 2).sum(), a32, create_graph=True)
    (gb2_r,) = torch.autograd.grad(ga_r.pow(2).sum(), b32)
    assert _rel(ga, ga_r) < 3e-2 and _rel(gb2, gb2_r) < 5e-2


@pytest.mark.parametrize("rows,D", [(1000, 2048), (77, 64), (4096, 128), (33, 8192), (3001, 2048), (1500, 1280), (1184, 1024)])
def test_rmsnorm(rows, D):
    from dttt_b200.ops import kernels, reference as ref
    torch.manual_seed(3)
    x = torch.randn(rows, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(D, device="cuda")).requires_grad_()
    y = kernels.rms_norm(x, w, 1e-6)
    g = torch.randn_like(y)
    dx, dw = torch.autograd.grad(y, (x, w), g)
    x32, w32 = x.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
    yr = ref.rms_norm(x32, w32, 1e-6)
    dxr, dwr = torch.autograd.grad(yr, (x32, w32), g.float())
    assert _rel(y, yr) < 1e-2 and _rel(dx, dxr) < 2e-2 and _rel(dw, dwr) < 2e-2


def test_rmsnorm_second_order_matches_reference():
    from dttt_b200.ops import kernels, reference as ref
    torch.manual_seed(4)
    x = torch.randn(64, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.ones(128, device="cuda", requires_grad=True)
    r = torch.randn(64, 128, device="cuda")
    y = kernels.rms_norm(x, w, 1e-6)
    (dx,) = torch.autograd.grad((y.float() * r).sum(), x, create_graph=True)
    (ddx,) = torch.autograd.grad(dx.float().pow(2).sum(), x)
    x32 = x.detach().float().requires_grad_()
    (dxr,) = torch.autograd.grad((ref.rms_norm(x32, w.detach(), 1e-6) * r).sum(), x32, create_graph=True)
    (ddxr,) = torch.autograd.grad(dxr.pow(2).sum(), x32)
    assert _rel(ddx, ddxr) < 0.1


def test_rope_table_follows_the_positions():
    """The cached (cos, sin) table is keyed on the position tensor: other positions of the same shape, and the same tensor
    edited in place, must not be served from it."""
    from dttt_b200.ops import kernels
    torch.manual_seed(6)
    x = torch.randn(500, 8, 64, device="cuda", dtype=torch.bfloat16)
    inv = (1.0 / (10000.0 ** (torch.arange(0, 32, device="cuda").float() / 32))).contiguous()
    pos = torch.randint(0, 100000, (500,), device="cuda")
    for _ in range(2):
        got = kernels._rope_run(x, pos, inv, 1.0)
        assert _rel(got, kernels._rope_ref(x.float(), pos, inv)) < 1e-2
    pos2 = torch.randint(0, 100000, (500,), device="cuda")
    assert _rel(kernels._rope_run(x, pos2, inv, -1.0), kernels._rope_ref(x.float(), -pos2, inv)) < 1e-2
    pos.add_(17)
    assert _rel(kernels._rope_run(x, pos, inv, 1.0), kernels._rope_ref(x.float(), pos, inv)) < 1e-2
    kernels._ROPE_TABLES.clear()


@pytest.mark.parametrize("d,heads", [(64, 8), (128, 4), (32, 3)])
def test_rope(d, heads):
    from dttt_b200.ops import functional as Fn, reference as ref
    torch.manual_seed(5)
    x = torch.randn(2, 300, heads, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    pos = torch.randint(0, 131072, (2, 300), device="cuda")
    scaling = (("factor", 16.0), ("high_freq_factor", 4.0), ("low_freq_factor", 1.0),
               ("original_max_position_embeddings", 8192), ("rope_type", "llama3"))
    y = Fn.rope(x, pos, d, 500000.0, scaling)
    g = torch.randn_like(y)
    (dx,) = torch.autograd.grad(y, x, g)
    x32 = x.detach().float().requires_grad_()
    cos, sin = ref.rope_cos_sin(pos, d, 500000.0, scaling)
    yr = ref.apply_rope(x32, cos, sin)
    (dxr,) = torch.autograd.grad(yr, x32, g.float())
    assert _rel(y, yr) < 1e-2 and _rel(dx, dxr) < 1e-2
    # the backward is itself differentiable (the rotation by the opposite angle): d<c, dx(g)>/dg = rope(c)
    g2 = g.clone().requires_grad_(True)
    (dx2,) = torch.autograd.grad(y, x, g2, create_graph=True)
    c = torch.randn_like(dx2)
    (gg,) = torch.autograd.grad(dx2, g2, c)
    assert _rel(gg, ref.apply_rope(c.float(), cos, sin)) < 1e-2


def test_swiglu():
    from dttt_b200.ops import kernels, reference as ref
    torch.manual_seed(6)
    g = torch.randn(513, 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    u = torch.randn(513, 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = kernels.swiglu(g, u)
    dy = torch.randn_like(y)
    dg, du = torch.autograd.grad(y, (g, u), dy)
    g32, u32 = g.detach().float().requires_grad_(), u.detach().float().requires_grad_()
    yr = ref.glu(g32, u32)
    dgr, dur = torch.autograd.grad(yr, (g32, u32), dy.float())
    assert _rel(y, yr) < 1e-2 and _rel(dg, dgr) < 2e-2 and _rel(du, dur) < 2e-2


def test_adamw_and_seq_ops():
    from dttt_b200.ops import kernels
    torch.manual_seed(7)
    n = 100_003
    p, m, v, g = (torch.randn(n, device="cuda") for _ in range(4))
    v = v.abs()
    p0, m0, v0 = p.clone(), m.clone(), v.clone()
    kernels.adamw(p, m, v, g, 1e-3, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05, 0.5)
    gg = g * 0.5
    mr = 0.9 * m0 + 0.1 * gg
    vr = 0.95 * v0 + 0.05 * gg * gg
    pr = p0 - 1e-3 * ((mr / 0.1) / ((vr / 0.05).sqrt() + 1e-8) + 0.1 * p0)
    assert _rel(p, pr) < 1e-5 and _rel(m, mr) < 1e-6 and _rel(v, vr) < 1e-6
    w = torch.randn(3, 700, 33, device="cuda")
    gb = torch.randn(3, 700, 33, device="cuda", dtype=torch.bfloat16)
    ss = kernels.seq_sumsq([w, gb])
    assert _rel(ss, w.pow(2).flatten(1).sum(1) + gb.float().pow(2).flatten(1).sum(1)) < 1e-4
    coef = torch.tensor([0.5, 1.0, 2.0], device="cuda")
    out, lo = kernels.seq_axpy(w, gb, coef, want_lo=True)
    refv = w - coef.view(3, 1, 1) * gb.float()
    assert _rel(out, refv) < 1e-6 and _rel(lo, refv) < 1e-2


@pytest.mark.parametrize("shape", [(3, 700, 33), (2, 256, 512)])          # odd sizes take the scalar kernels, aligned ones the 16-byte ones
def test_seq_kernels_scalar_and_vector_paths(shape):
    from dttt_b200.ops import kernels
    torch.manual_seed(17)
    B = shape[0]
    w, a = torch.randn(*shape, device="cuda"), torch.randn(*shape, device="cuda")
    for gdt in (torch.float32, torch.bfloat16):
        g = torch.randn(*shape, device="cuda").to(gdt)
        v1 = lambda t: t.view(B, 1, 1)
        coef, al, be = torch.rand(B, device="cuda"), torch.randn(B, device="cuda"), torch.randn(B, device="cuda")
        assert _rel(kernels.seq_sumsq([w, g]), w.pow(2).flatten(1).sum(1) + g.float().pow(2).flatten(1).sum(1)) < 1e-4
        out, lo = kernels.seq_axpy(w, g, coef, want_lo=True)
        assert _rel(out, w - v1(coef) * g.float()) < 1e-6 and _rel(lo, w - v1(coef) * g.float()) < 1e-2
        assert _rel(kernels.seq_dot([a, w], [g, g]), ((a + w) * g.float()).flatten(1).sum(1)) < 1e-3
        lc = kernels.seq_lincomb(a, g, al, be)
        assert lc.dtype == gdt and _rel(lc, v1(al) * a + v1(be) * g.float()) < (1e-6 if gdt == torch.float32 else 1e-2)
    n = 1 << 20
    p, m, v, g = (torch.randn(n, device="cuda") for _ in range(4))
    v = v.abs()
    p0, m0, v0 = p.clone(), m.clone(), v.clone()
    kernels.adamw(p, m, v, g, 1e-3, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05, 0.5)
    gg = g * 0.5
    mr, vr = 0.9 * m0 + 0.1 * gg, 0.95 * v0 + 0.05 * gg * gg
    assert _rel(p, p0 - 1e-3 * ((mr / 0.1) / ((vr / 0.05).sqrt() + 1e-8) + 0.1 * p0)) < 1e-5 and _rel(m, mr) < 1e-6 and _rel(v, vr) < 1e-6


def test_weighted_ce_matches_dense_with_grads():
    from dttt_b200.ops import ce as CE, reference as ref
    torch.manual_seed(8)
    N, H, V = 512, 256, 5000
    h = (0.5 * torch.randn(N, H, device="cuda")).to(torch.bfloat16).requires_grad_()
    E = (0.1 * torch.randn(V, H, device="cuda")).to(torch.bfloat16).requires_grad_()
    y = torch.randint(0, V, (N,), device="cuda")
    w = torch.rand(N, device="cuda")
    loss = CE.weighted_ce(h, E, y, w, 2048)
    gh, gE = torch.autograd.grad(loss, (h, E))
    h32, E32 = h.detach().float().requires_grad_(), E.detach().float().requires_grad_()
    lr = ref.weighted_ce_dense(h32, E32, y, w)
    ghr, gEr = torch.autograd.grad(lr, (h32, E32))
    assert abs(loss.item() - lr.item()) / lr.item() < 5e-3
    assert _rel(gh, ghr) < 3e-2 and _rel(gE, gEr) < 3e-2
    pt = CE.per_token_ce(h.detach(), E.detach(), y, 2048)
    assert _rel(pt, ref.per_token_ce_dense(h32.detach(), E32.detach(), y)) < 1e-2


@pytest.mark.parametrize("causal", [False, True])
def test_attention_window_staged(causal):
    from dttt_b200.ops import attention as A, reference as ref
    torch.manual_seed(9)
    n, C, nh, nkv, d, W = 2, 128, 8, 2, 64, 3
    q = torch.randn(n, C, nh, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(n, C, nkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(n, C, nkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    kw = torch.randn(n, W * C, nkv, d, device="cuda", dtype=torch.bfloat16)
    vw = torch.randn(n, W * C, nkv, d, device="cuda", dtype=torch.bfloat16)
    o = A.attend_window(q, k, v, kw, vw, 2, C, d ** -0.5, own="causal" if causal else "full")
    g = torch.randn_like(o)
    dq, dk, dv = torch.autograd.grad(o, (q, k, v), g)
    q32, k32, v32 = (t.detach().float().requires_grad_() for t in (q, k, v))
    K = torch.cat([kw[:, C:].float(), k32], 1)
    V = torch.cat([vw[:, C:].float(), v32], 1)
    om = A.own_mask_matrix(C, "causal", "cuda") if causal else None
    orf = ref.attend(q32, K, V, None, d ** -0.5, om)
    dqr, dkr, dvr = torch.autograd.grad(orf, (q32, k32, v32), g.float())
    assert _rel(o, orf) < 2e-2 and _rel(dq, dqr) < 3e-2 and _rel(dk, dkr) < 3e-2 and _rel(dv, dvr) < 3e-2
    # recorded backward (second order path) agrees with the first-order kernels
    o2 = A.attend_window(q, k, v, kw, vw, 2, C, d ** -0.5, own="causal" if causal else "full")
    (dq2,) = torch.autograd.grad(o2, q, g, create_graph=True)
    assert _rel(dq2, dqr) < 3e-2


def test_embedding_gather_and_f32_scatter():
    from dttt_b200.ops import kernels
    torch.manual_seed(21)
    V, H, n = 1000, 256, 5000
    table = torch.randn(V, H, device="cuda").to(torch.bfloat16)
    ids = torch.randint(0, V, (5, n // 5), device="cuda")
    ids[0, :300] = 7                                                       # a row hit many times (the mask token)
    out = kernels.embed_gather(table, ids)
    assert torch.equal(out, table[ids])
    dh = torch.randn(5, n // 5, H, device="cuda").to(torch.bfloat16)
    grad = torch.ones(V, H, device="cuda")
    kernels.embed_scatter_f32(dh, ids, grad)
    ref = torch.ones(V, H, device="cuda").index_add_(0, ids.flatten(), dh.float().flatten(0, 1))
    assert _rel(grad, ref) < 1e-5


def test_cart_band_and_threefry_match_the_host_statements():
    from dttt_b200.ops import kernels, reference as ref
    from dttt_b200.utils import rng
    torch.manual_seed(22)
    vis = (torch.rand(3, 2000, device="cuda") < 0.6)
    kern = torch.rand(2 * 512 + 1, device="cuda")
    assert _rel(kernels.cart_band(vis, kern), ref.band_correlate(vis.float(), kern)) < 1e-5
    keys = torch.stack([rng.key(5), rng.fold_in(rng.key(5), 3), rng.key(2 ** 40 + 17)]).cuda()
    u = kernels.threefry_uniform(keys, 1000)
    u_ref = torch.stack([rng.uniform(k.cpu(), (1000,)) for k in keys])
    assert torch.equal(u.cpu(), u_ref)
    th = torch.tensor([0.1, 0.5, 0.9], device="cuda")
    assert torch.equal(kernels.threefry_uniform(keys, 1000, th).cpu(), u_ref < th.cpu()[:, None])
