"""Host-side debug checks (``DTTT_DEBUG=1``, ``csrc/host_check.h``): every tensor map and peer range must lie inside one device
allocation.  The checks run on the host before a launch, so a violation is an error code, never a device fault."""
import ctypes
import os
import subprocess
import sys

import pytest
import torch

from util import ROOT

pytestmark = pytest.mark.gpu


def test_extent_check_accepts_inside_and_refuses_outside():
    from dttt_b200.ops import _lib
    _lib.register("dttt_debug_extent_check", ctypes.c_int, [ctypes.c_void_p, ctypes.c_longlong])
    fn = _lib.lib().dttt_debug_extent_check
    lib_alloc = ctypes.c_void_p()
    _lib.register("dttt_peer_alloc", ctypes.c_int, [ctypes.POINTER(ctypes.c_void_p), ctypes.c_longlong])
    _lib.register("dttt_peer_free", ctypes.c_int, [ctypes.c_void_p])
    assert _lib.lib().dttt_peer_alloc(ctypes.byref(lib_alloc), 1 << 20) == 0          # a cudaMalloc of exactly 1 MiB
    try:
        p = lib_alloc.value
        assert fn(ctypes.c_void_p(p), 1 << 20) == 0
        assert fn(ctypes.c_void_p(p + 4096), (1 << 20) - 4096) == 0
        assert fn(ctypes.c_void_p(p), (1 << 20) + 16) == -70                          # runs past the end
        assert fn(ctypes.c_void_p(p + (1 << 19)), (1 << 19) + 2) == -70
    finally:
        _lib.lib().dttt_peer_free(lib_alloc)


def test_small_cases_run_clean_with_the_checks_on():
    """GEMM (all layouts, batched, pair form), attention forward / backward in both forms and the second-order score kernel
    with the checks switched on: same results, no refusal."""
    code = r"""
import torch
from dttt_b200.ops import _lib, gemm, kernels
from dttt_b200.ops import attention as A
torch.manual_seed(0)
r = lambda *s: torch.randn(*s, device="cuda").to(torch.bfloat16)
for ta in (False, True):
    for tb in (False, True):
        a, b = r(*((320, 512) if ta else (512, 320))), r(*((384, 320) if tb else (320, 384)))
        y = gemm.gemm_raw(a, b, ta, tb)
        want = (a.t() if ta else a).float() @ (b.t() if tb else b).float()
        assert (y.float() - want).abs().max() < 0.05 * want.abs().max()
x, w = r(3, 256, 128), r(3, 128, 1024)
assert (gemm.gemm_raw(x, w, False, False).float() - x.float() @ w.float()).abs().max() < 0.5
q, k, v, g = r(2, 256, 4, 64), r(2, 512, 2, 64), r(2, 512, 2, 64), r(2, 256, 4, 64)
o, lse = kernels.attention_fwd(q, k, v, 0.125, "causal")
kernels.attention_bwd(g, q, k, v, o, lse, 0.125, "causal")
q5, k5, v5, g5 = r(1, 3, 512, 4, 128), r(1, 3, 512, 2, 128), r(1, 3, 512, 2, 128), r(1, 3, 512, 4, 128)
leaves = [t.requires_grad_(True) for t in (q5, k5, v5)]
o5, tk, tv = A.segment_attention(*leaves, None, 128, 2, 0, None, ("full", "full", "causal"), 128 ** -0.5)
torch.autograd.grad(o5, leaves, g5)
torch.cuda.synchronize()
_lib.check_status()
print("DEBUG_CHECKS_CLEAN")
"""
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, cwd=ROOT,
                       env=dict(os.environ, DTTT_DEBUG="1", PYTHONPATH=ROOT))
    assert r.returncode == 0 and "DEBUG_CHECKS_CLEAN" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
