"""The allocation-free LayerNorm-backward entry point (csrc/layernorm_noalloc.h), called through its exported C symbol.

Some hosts of the library may not allocate device memory while they run (pre-sized inference servers, real-time
loops, plug-ins under a foreign allocator); for them ``ffb_layernorm_bwd_noalloc`` keeps its scratch in a static
device array.  The test calls it with raw pointers, twice in a row (the array keeps the previous call's contents,
so the second call checks that it is cleared correctly), and compares dx / dgamma / dbeta with the regular entry
point ``ffb_layernorm_bwd`` on the same inputs and with the fp32 gradients of ``torch.nn.functional.layer_norm``; it
also checks that a row wider than the built-in capacity is refused.  Runs last in the suite (file name) and also on its own in a fresh process.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from fastfold_b200.ops import _lib
    lib = ctypes.CDLL(_lib.lib_path())
    P, L, I = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
    lib.ffb_layernorm_bwd_noalloc.argtypes = [P, P, P, P, P, P, P, P, L, I, I, P]
    lib.ffb_layernorm_bwd_noalloc.restype = I
    lib.ffb_layernorm_bwd.argtypes = [P, P, P, P, P, P, P, I, P, P, L, I, I, P]
    lib.ffb_layernorm_bwd.restype = I
    lib.ffb_layernorm_fwd.argtypes = [P, P, P, P, P, P, L, I, ctypes.c_float, I, P]
    lib.ffb_layernorm_fwd.restype = I
    return lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("dtype,code,tol", [(torch.bfloat16, 2, 1e-1), (torch.float32, 0, 1e-4)])
def test_noalloc_matches_regular_entry_point_twice(dtype, code, tol):
    lib = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (rows, C) in enumerate([(5000, 256), (777, 128)]):      # two calls in a row, different shapes
        torch.manual_seed(call)
        x = torch.randn(rows, C, device=dev, dtype=dtype)
        dy = torch.randn(rows, C, device=dev, dtype=dtype)
        gamma = (torch.randn(C, device=dev) * 0.3 + 1).to(dtype)
        beta = torch.zeros(C, device=dev, dtype=dtype)
        y = torch.empty_like(x)
        mean = torch.empty(rows, device=dev, dtype=torch.float32)
        rstd = torch.empty(rows, device=dev, dtype=torch.float32)
        assert lib.ffb_layernorm_fwd(_p(x), _p(gamma), _p(beta), _p(y), _p(mean), _p(rstd), rows, C, 1e-5, code, stream) == 0
        # regular entry point (caller-provided workspace)
        nblocks = 148
        part = torch.empty(nblocks * 2 * C, device=dev, dtype=torch.float32)
        dx_a, dg_a, db_a = torch.empty_like(x), torch.empty_like(gamma), torch.empty_like(gamma)
        assert lib.ffb_layernorm_bwd(_p(dy), _p(x), _p(gamma), _p(mean), _p(rstd), _p(dx_a), _p(part), nblocks, _p(dg_a), _p(db_a), rows, C,
                                     code, stream) == 0
        # allocation-free entry point: outputs are pre-allocated by the caller, nothing else is needed
        dx_b, dg_b, db_b = torch.empty_like(x), torch.empty_like(gamma), torch.empty_like(gamma)
        assert lib.ffb_layernorm_bwd_noalloc(_p(dy), _p(x), _p(gamma), _p(mean), _p(rstd), _p(dx_b), _p(dg_b), _p(db_b), rows, C, code,
                                             stream) == 0
        torch.cuda.synchronize()
        # independent oracle: autograd through torch's own LayerNorm in fp32 on the same (rounded) inputs
        xr = x.float().requires_grad_(True)
        gr = gamma.float().requires_grad_(True)
        br = beta.float().requires_grad_(True)
        torch.nn.functional.layer_norm(xr, (C,), gr, br, 1e-5).backward(dy.float())
        ref_tol = 5e-2 if dtype == torch.bfloat16 else 1e-3
        assert (dx_b.float() - xr.grad).abs().max().item() <= ref_tol * max(1.0, xr.grad.abs().max().item())
        assert (dg_b.float() - gr.grad).abs().max().item() <= ref_tol * max(1.0, gr.grad.abs().max().item())
        assert (db_b.float() - br.grad).abs().max().item() <= ref_tol * max(1.0, br.grad.abs().max().item())
        assert (dx_a.float() - dx_b.float()).abs().max().item() <= tol
        scale = max(1.0, dg_a.float().abs().max().item())
        assert (dg_a.float() - dg_b.float()).abs().max().item() <= tol * scale
        assert (db_a.float() - db_b.float()).abs().max().item() <= tol * max(1.0, db_a.float().abs().max().item())


def test_noalloc_rejects_rows_wider_than_capacity():
    lib = _lib()
    t = torch.zeros(8, device="cuda")
    rc = lib.ffb_layernorm_bwd_noalloc(_p(t), _p(t), _p(t), _p(t), _p(t), _p(t), _p(t), _p(t), 4, 2048, 0, ctypes.c_void_p(0))
    assert rc == -3
