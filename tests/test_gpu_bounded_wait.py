"""The device-side time-out path: a wait on a flag that nothing sets runs out of its (short) budget, records its
status code and returns; the context stays usable and the host turns the code into an exception."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_runs_out_and_reports():
    from fms_acceleration_b200 import _native as NV
    from fms_acceleration_b200.ops.gemm import gemm
    from fms_acceleration_b200.parallel import symm  # noqa: F401  (declares the comm entry points)

    dev = torch.device("cuda", 0)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    st = NV.status_word(dev)
    st[0] = 0
    budget = 20_000_000  # cycles: about ten milliseconds
    rc = NV.lib().fmsb_comm_wait_flag(flag.data_ptr(), 1, st.data_ptr(), budget, NV.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert int(st[0].item()) == 4  # kTimeoutPeerFlag
    with pytest.raises(NV.NativeError, match="4"):
        NV.check_status(dev)
    assert int(st[0].item()) == 0  # cleared by the check
    # a flag that is already at the epoch returns at once and reports nothing
    flag.fill_(1)
    NV.lib().fmsb_comm_wait_flag(flag.data_ptr(), 1, st.data_ptr(), budget, NV.stream_ptr())
    NV.check_status(dev)
    # the context is intact: a tensor-core kernel still runs and is right
    a = torch.randn(256, 128, device=dev, dtype=torch.bfloat16)
    b = torch.randn(64, 128, device=dev, dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    assert (gemm(a, b).float() - ref).abs().max() < 0.5
    NV.check_status(dev)
