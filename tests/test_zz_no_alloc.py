"""The allocation-free RMSNorm backward, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at the point where they
need the kernel (they sit inside an allocator callback, or only own raw pointers and a
stream), so ``tft_rmsnorm_bwd_noalloc`` keeps its scratch inside the library.  This test
loads the library on its own, calls that symbol twice in a row and checks both results
against the regular entry point, which gets its scratch from the caller, and against the
same formulas written in fp32 PyTorch.  It is collected last so a failure here never hides the
result of another test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _load():
    from torchft_b200.utils import build

    lib = ctypes.CDLL(str(build.kernels_lib_path()))
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.tft_rmsnorm_bwd_noalloc.argtypes = [P, P, P, P, P, P, P, I, I, I, P]
    lib.tft_rmsnorm_bwd_noalloc.restype = I
    lib.tft_rmsnorm_bwd_noalloc_max_dim.argtypes = []
    lib.tft_rmsnorm_bwd_noalloc_max_dim.restype = I
    lib.tft_rmsnorm_bwd.argtypes = [P, P, P, P, P, P, P, P, I, I, I, P]
    lib.tft_rmsnorm_bwd.restype = I
    lib.tft_rmsnorm_bwd_parts.argtypes = [I]
    lib.tft_rmsnorm_bwd_parts.restype = I
    return lib


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / max(b.float().abs().max().item(), 1e-6)


def test_noalloc_rmsnorm_bwd_matches_regular_entry_point_twice():
    lib = _load()
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.tft_rmsnorm_bwd_noalloc_max_dim() == 8192
    for call, (rows, dim) in enumerate([(700, 4096), (333, 2048)]):
        torch.manual_seed(call)
        dy = torch.randn(rows, dim, device="cuda").to(torch.bfloat16)
        x = torch.randn(rows, dim, device="cuda").to(torch.bfloat16)
        dres = torch.randn(rows, dim, device="cuda").to(torch.bfloat16)
        w = (1 + 0.1 * torch.randn(dim, device="cuda")).to(torch.bfloat16)
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5).contiguous()

        dx_ref, dw_ref = torch.empty_like(x), torch.empty_like(w)
        scratch = torch.empty(lib.tft_rmsnorm_bwd_parts(rows) * dim, dtype=torch.float32, device="cuda")
        rc = lib.tft_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(),
                                 dx_ref.data_ptr(), dw_ref.data_ptr(), scratch.data_ptr(), rows, dim, 0, stream)
        assert rc == 0

        dx, dw = torch.empty_like(x), torch.empty_like(w)
        rc = lib.tft_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(),
                                         dx.data_ptr(), dw.data_ptr(), rows, dim, 0, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(dx, dx_ref), f"call {call}: dx differs"
        # the two entry points split the rows over a different number of blocks, so the
        # weight gradient is summed in a different order
        assert _rel(dw, dw_ref) < 2e-2, f"call {call}: dw differs by {_rel(dw, dw_ref)}"
        # and both against plain fp32 PyTorch: y = x * rstd * w, differentiated by autograd
        xf = x.float().requires_grad_(True)
        wf = w.float().requires_grad_(True)
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
        y.backward(dy.float())
        assert _rel(dx, xf.grad + dres.float()) < 2e-2, f"call {call}: dx vs fp32 {_rel(dx, xf.grad + dres.float())}"
        assert _rel(dw, wf.grad) < 2e-2, f"call {call}: dw vs fp32 {_rel(dw, wf.grad)}"


def test_noalloc_rejects_oversized_rows():
    lib = _load()
    t = torch.zeros(16, device="cuda")
    rc = lib.tft_rmsnorm_bwd_noalloc(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), None, t.data_ptr(),
                                     t.data_ptr(), 4, 16384, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == -10
