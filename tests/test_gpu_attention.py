"""Varlen tcgen05 attention against an fp32 PyTorch oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from fms_acceleration_b200 import _native as NV
from fms_acceleration_b200.ops import attention as AT

DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)).item()


def _make(T, nh, nkv, d, lens, dtype, seed=0):
    torch.manual_seed(seed)
    assert sum(lens) == T
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    ds, de = AT.doc_bounds_from_cu_seqlens(cu, T)
    qkv = torch.randn(T, (nh + 2 * nkv) * d, device=DEV, dtype=dtype)
    return qkv, ds, de


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("lens", [[128], [300], [100, 156, 7, 249], [513, 1, 254]])
def test_attention_forward(dtype, d, lens):
    T = sum(lens)
    nh, nkv = 4, 2
    qkv, ds, de = _make(T, nh, nkv, d, lens, dtype)
    q = qkv[:, : nh * d].view(T, nh, d)
    k = qkv[:, nh * d: (nh + nkv) * d].view(T, nkv, d)
    v = qkv[:, (nh + nkv) * d:].view(T, nkv, d)
    o = AT.varlen_attention(q, k, v, ds, de)
    NV.check_status()
    ref = AT.attention_ref(q, k, v, ds)
    assert _rel(o, ref) < 1.5e-2


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("lens", [[256], [100, 156, 7, 249], [640, 129, 255]])
def test_attention_backward(d, lens):
    T = sum(lens)
    nh, nkv = 4, 2
    dtype = torch.bfloat16
    qkv, ds, de = _make(T, nh, nkv, d, lens, dtype, seed=1)
    q = qkv[:, : nh * d].reshape(T, nh, d).clone().requires_grad_()
    k = qkv[:, nh * d: (nh + nkv) * d].reshape(T, nkv, d).clone().requires_grad_()
    v = qkv[:, (nh + nkv) * d:].reshape(T, nkv, d).clone().requires_grad_()
    o = AT.varlen_attention(q, k, v, ds, de)
    g = torch.randn_like(o)
    o.backward(g)
    NV.check_status()
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = AT.attention_ref(qf, kf, vf, ds)
    ref.backward(g.float())
    assert _rel(q.grad, qf.grad) < 3e-2
    assert _rel(k.grad, kf.grad) < 3e-2
    assert _rel(v.grad, vf.grad) < 3e-2


@pytest.mark.parametrize("d,nh,nkv", [(128, 8, 2), (64, 6, 2)])
def test_backward_on_ragged_documents_against_fp32(d, nh, nkv):
    """Backward kernels against the fp32 PyTorch statement on a longer packed batch with ragged documents
    (tile-crossing, single-token and tail documents)."""
    lens = [700, 1, 129, 1023, 64, 131]
    T = sum(lens)
    qkv, ds, de = _make(T, nh, nkv, d, lens, torch.bfloat16, seed=5)
    q, k, v = qkv[:, : nh * d], qkv[:, nh * d: (nh + nkv) * d], qkv[:, (nh + nkv) * d:]
    scale = d ** -0.5
    o, lse = AT._fwd(q, k, v, ds, de, nh, nkv, d, scale)
    do = torch.randn_like(o)
    got = AT._bwd(q, k, v, o, lse, do, ds, de, nh, nkv, d, scale)
    NV.check_status()
    qf, kf, vf = (t.float().reshape(T, -1, d).requires_grad_() for t in (q, k, v))
    ref = AT.attention_ref(qf, kf, vf, ds, scale)
    ref.backward(do.float().reshape(T, nh, d))
    for a, r in zip(got, (qf.grad, kf.grad, vf.grad)):
        assert _rel(a.reshape(T, -1, d), r) < 3e-2


def test_backward_is_bitwise_reproducible():
    """No gradient is accumulated with atomics: two runs of the same backward give the same bits."""
    lens = [700, 129, 1, 450]
    T, nh, nkv, d = sum(lens), 8, 2, 128
    qkv, ds, de = _make(T, nh, nkv, d, lens, torch.bfloat16, seed=3)
    grads = []
    for _ in range(2):
        q = qkv[:, : nh * d].reshape(T, nh, d).clone().requires_grad_()
        k = qkv[:, nh * d: (nh + nkv) * d].reshape(T, nkv, d).clone().requires_grad_()
        v = qkv[:, (nh + nkv) * d:].reshape(T, nkv, d).clone().requires_grad_()
        o = AT.varlen_attention(q, k, v, ds, de)
        torch.manual_seed(11)
        o.backward(torch.randn_like(o))
        NV.check_status()
        grads.append((o.detach().clone(), q.grad.clone(), k.grad.clone(), v.grad.clone()))
    for a, b in zip(*grads):
        assert torch.equal(a, b)
