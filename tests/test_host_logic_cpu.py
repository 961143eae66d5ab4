"""Host-side decisions that steer the kernels, checked on the CPU: contraction splitting of weight-gradient GEMMs,
the one-concatenation column split of the Mamba2 mixer, slab ranges of the scan, and the CPU oracle of the
entering-state correction against the sequential recurrence."""
import torch

from fms_acceleration_b200.models.mamba2 import _SplitCols
from fms_acceleration_b200.ops import gemm as GM
from fms_acceleration_b200.ops import mamba as MB


def test_split_k_only_for_few_tiles_and_long_contractions():
    # plenty of tiles: never split
    assert GM._split_k(14336, 4096, 16384, 256) == 1
    # short contraction: never split
    assert GM._split_k(48, 4096, 512, 256) == 1
    for M, N, K in [(48, 4096, 16384), (6144, 48, 16384), (1536, 1536, 16384), (40, 1536, 16384), (1536, 512, 4096)]:
        bn = GM._pick_bn(N, True)
        s = GM._split_k(M, N, K, bn)
        tiles = -(-M // 128) * -(-N // bn)
        assert s > 1 and s & (s - 1) == 0, (M, N, K, s)
        assert K % (s * 64) == 0 and K // s >= GM.SPLIT_K_MIN
        assert tiles * s <= 2 * GM.SM_COUNT
    # a token count that only divides by 64 once cannot be split evenly
    assert GM._split_k(48, 4096, 64 * 33, 256) == 1


def test_split_cols_backward_is_the_slicing_backward():
    torch.manual_seed(0)
    t = torch.randn(7, 12, requires_grad=True)
    a, b, c = _SplitCols.apply(t, 5, 4, 3)
    assert a.shape == (7, 5) and b.shape == (7, 4) and c.shape == (7, 3)
    (a.sum() * 2 + (b * b).sum()).backward()          # c is unused: its block of the gradient is zero
    g = t.grad.clone()
    t.grad = None
    a2, b2 = t[:, :5], t[:, 5:9]
    (a2.sum() * 2 + (b2 * b2).sum()).backward()
    assert torch.equal(g, t.grad)
    assert torch.count_nonzero(g[:, 9:]) == 0


def test_slabs_cover_all_chunks_once():
    for nc, nh, Q in [(1, 4, 64), (32, 80, 256), (257, 8, 128)]:
        ranges = MB._slabs(nc, nh, Q)
        assert ranges[0][0] == 0 and ranges[-1][1] == nc
        assert all(a1 == b0 for (_, a1), (b0, _) in zip(ranges[:-1], ranges[1:]))
        assert all((c1 - c0) * nh * Q * Q * 4 <= max(MB.SLAB_BYTES, nh * Q * Q * 4) for c0, c1 in ranges)


def test_state_correction_oracle_equals_scan_with_initial_state():
    """y(h0) = y(0) + correction(h0): the identity context parallelism relies on, in fp64 on the CPU."""
    torch.manual_seed(1)
    T, nh, P, G, N = 48, 4, 8, 2, 16
    x = torch.randn(T, nh, P, dtype=torch.float64)
    dt = torch.rand(T, nh, dtype=torch.float64) * 0.1 + 0.01
    A = -(torch.rand(nh, dtype=torch.float64) + 0.5)
    B = torch.randn(T, G, N, dtype=torch.float64)
    C = torch.randn(T, G, N, dtype=torch.float64)
    D = torch.randn(nh, dtype=torch.float64)
    h0 = torch.randn(nh, P, N, dtype=torch.float64)
    y0, _ = MB.ssd_ref(x, dt, A, B, C, D, None)
    y1, _ = MB.ssd_ref(x, dt, A, B, C, D, h0)
    rep = nh // G
    Lg = torch.cumsum(dt * A[None, :], 0)
    Ch = C.repeat_interleave(rep, 1)
    corr = torch.exp(Lg)[:, :, None] * torch.einsum("thn,hpn->thp", Ch, h0)
    assert torch.allclose(y0 + corr, y1, rtol=1e-9, atol=1e-9)


def test_context_parallel_prefix_state_and_its_gradients():
    """The state entering rank r and the hand-written gradients sent back to the earlier ranks, against autograd."""
    from fms_acceleration_b200.parallel.context_parallel import prefix_state, prefix_state_grads

    torch.manual_seed(4)
    world, nh, P, N = 4, 3, 5, 7
    Fs = torch.randn(world, nh, P, N, dtype=torch.float64, requires_grad=True)
    lPs = (-torch.rand(world, nh, dtype=torch.float64)).requires_grad_()
    for r in range(1, world):
        h = prefix_state(Fs, lPs, r)
        # closed form: sum_j (prod_{j<i<r} P_i) F_j
        ref = sum(torch.exp(lPs[j + 1: r].sum(0))[:, None, None] * Fs[j] for j in range(r))
        assert torch.allclose(h.double(), ref.double(), rtol=1e-5, atol=1e-6)
        dh = torch.randn(nh, P, N, dtype=torch.float64)
        gF, glP = torch.autograd.grad((ref * dh).sum(), (Fs, lPs))
        dF, dlP = prefix_state_grads(dh, Fs.detach(), lPs.detach(), r, world)
        assert torch.allclose(dF.double(), gF, rtol=1e-4, atol=1e-5)
        assert torch.allclose(dlP.double(), glP, rtol=1e-4, atol=1e-5)
        assert torch.count_nonzero(dF[r:]) == 0 and torch.count_nonzero(dlP[r:]) == 0


def test_gemm_host_statement_of_the_kernel_contract():
    """On host tensors ``gemm`` is stated with torch operators: both operand orientations, the second operand pair,
    ``alpha`` / ``beta * c`` and an ``out`` buffer."""
    import torch

    from fms_acceleration_b200.ops.gemm import gemm

    torch.manual_seed(0)
    a, b = torch.randn(5, 7), torch.randn(3, 7)           # b is [N, K] unless b_mn
    assert torch.allclose(gemm(a, b), a @ b.t(), atol=1e-6)
    assert torch.allclose(gemm(a, b.t().contiguous(), b_mn=True), a @ b.t(), atol=1e-6)
    assert torch.allclose(gemm(a.t().contiguous(), b, a_mn=True), a @ b.t(), atol=1e-6)
    a2, b2, c = torch.randn(5, 2), torch.randn(3, 2), torch.randn(5, 3)
    want = 0.5 * (a @ b.t() + a2 @ b2.t()) + 2.0 * c
    out = torch.empty(5, 3)
    assert gemm(a, b, a2=a2, b2=b2, c=c, alpha=0.5, beta=2.0, out=out) is out
    assert torch.allclose(out, want, atol=1e-6)
    assert gemm(a.bfloat16(), b.bfloat16(), out_dtype=torch.float32).dtype == torch.float32
