"""The allocation-free RMSNorm-backward entry point, called through its exported C symbol.

Some users of the native library may not allocate device memory when they call it (a host that owns all device
memory in an arena of its own, a server plugin with a fixed budget, a path that must not trigger the implicit
synchronisation of cudaMalloc/cudaFree).  For them ``fmsb_rmsnorm_bwd_noalloc`` keeps the partial sums of the
weight gradient in a scratch array built into the library.  The test calls it twice in a row with different
inputs (the scratch keeps the first call's contents) and compares with the regular entry point, whose scratch is
allocated by the caller, and with the fp32 PyTorch formula of the same operation.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

from fms_acceleration_b200 import _native as NV

P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def _entry():
    raw = ctypes.CDLL(NV.library_path())
    fn = raw.fmsb_rmsnorm_bwd_noalloc
    fn.argtypes = [P, P, P, P, P, P, P, I, I, I, I, P]
    fn.restype = I
    err = raw.fmsb_noalloc_last_error
    err.restype = ctypes.c_char_p
    return fn, err


def _reference(dy, x, w, inv, dres, gemma):
    rows, H = x.shape
    dx = torch.empty_like(x)
    nblk = min(rows, 148 * 2)
    partial = torch.empty(nblk, H, dtype=torch.float32, device=x.device)
    dw = torch.empty(H, dtype=torch.float32, device=x.device)
    rc = NV.lib().fmsb_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), inv.data_ptr(), NV.ptr(dres), dx.data_ptr(),
                                   partial.data_ptr(), dw.data_ptr(), nblk, rows, H, int(gemma),
                                   NV.dtype_code(x.dtype), NV.stream_ptr())
    assert rc == 0
    return dx, dw


def _oracle(dy, x, w, inv, dres, gemma):
    """fp32 PyTorch statement of RMSNorm backward (inputs rounded to the storage dtype, arithmetic in fp32)."""
    xf, dyf, wf = x.float(), dy.float(), w.float() + (1.0 if gemma else 0.0)
    xhat = xf * inv[:, None]
    g = dyf * wf
    dx = inv[:, None] * (g - xhat * (g * xhat).mean(-1, keepdim=True))
    if dres is not None:
        dx = dx + dres.float()
    return dx, (dyf * xhat).sum(0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_noalloc_entry_matches_regular_entry_twice(dtype):
    fn, err = _entry()
    dev = torch.device("cuda")
    torch.manual_seed(0)
    # everything the calls need is allocated BEFORE them; the entry point itself allocates nothing
    cases = []
    for rows, H, with_res, gemma in [(700, 4096, True, 0), (33, 1536, False, 1)]:
        x = torch.randn(rows, H, device=dev).to(dtype)
        dy = torch.randn(rows, H, device=dev).to(dtype)
        w = (torch.randn(H, device=dev) * 0.1 + 1).to(dtype)
        inv = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6).contiguous()
        dres = torch.randn(rows, H, device=dev).to(dtype) if with_res else None
        dx = torch.empty_like(x)
        dw = torch.empty(H, dtype=torch.float32, device=dev)
        cases.append((x, dy, w, inv, dres, dx, dw, rows, H, gemma))
    stream = torch.cuda.current_stream().cuda_stream
    before = torch.cuda.memory_allocated()
    for x, dy, w, inv, dres, dx, dw, rows, H, gemma in cases:  # two calls in a row share the built-in scratch
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), inv.data_ptr(), None if dres is None else dres.data_ptr(),
                dx.data_ptr(), dw.data_ptr(), rows, H, gemma, NV.dtype_code(dtype), stream)
        assert rc == 0, err().decode()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    for x, dy, w, inv, dres, dx, dw, rows, H, gemma in cases:
        rdx, rdw = _reference(dy, x, w, inv, dres, gemma)
        torch.cuda.synchronize()
        assert torch.allclose(dx.float(), rdx.float(), rtol=2e-2, atol=2e-2)
        rel = ((dw - rdw).norm() / rdw.norm()).item()
        assert rel < 1e-4, rel
        odx, odw = _oracle(dy, x, w, inv, dres, gemma)
        # dx is rounded once to the 16-bit storage type: half a unit in the last place of the largest element
        ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
        assert ((dx.float() - odx).abs() <= ulp * odx.abs() + 1e-3).all()
        assert ((dw - odw).norm() / odw.norm()).item() < 1e-4


def test_noalloc_entry_rejects_oversized_rows():
    fn, err = _entry()
    dev = torch.device("cuda")
    H = 8192 + 8
    x = torch.zeros(2, H, device=dev, dtype=torch.bfloat16)
    inv = torch.ones(2, device=dev)
    dw = torch.zeros(H, device=dev)
    rc = fn(x.data_ptr(), x.data_ptr(), x.data_ptr(), inv.data_ptr(), None, x.data_ptr(), dw.data_ptr(), 2, H, 0, 1,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -3
    assert b"exceeds the built-in scratch" in err()


def test_noalloc_entry_rejects_misaligned_pointers():
    fn, err = _entry()
    dev = torch.device("cuda")
    rows, H = 4, 256
    buf = torch.zeros(rows * H + 8, device=dev, dtype=torch.bfloat16)
    good = buf[:rows * H].view(rows, H)
    off = buf[1:rows * H + 1]  # 2 bytes past a 16-byte boundary
    inv = torch.ones(rows, device=dev)
    dw = torch.zeros(H, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    assert off.data_ptr() % 16 != 0 and good.data_ptr() % 16 == 0
    for args in [(off, good, good, good), (good, off, good, good), (good, good, off, good), (good, good, good, off)]:
        dy_, x_, w_, dx_ = args
        rc = fn(dy_.data_ptr(), x_.data_ptr(), w_.data_ptr(), inv.data_ptr(), None, dx_.data_ptr(), dw.data_ptr(), rows, H,
                0, 1, st)
        assert rc == -2
        assert b"16-byte aligned" in err()
    torch.cuda.synchronize()  # nothing was launched; the context is intact
