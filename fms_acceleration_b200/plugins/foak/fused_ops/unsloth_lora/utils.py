"""Names of fms_acceleration_foak/fused_ops/unsloth_lora/utils.py:53-283."""
from fms_acceleration_b200.ops.gemm import gemm
from fms_acceleration_b200.ops.proj import _lora_parts, _unwrap
from fms_acceleration_b200.ops.quant import fast_dequantize, fast_gemv  # noqa: F401
from fms_acceleration_b200.plugins.foak.kernels.unsloth.utils import calculate_settings  # noqa: F401


def QUANT_STATE(W, base_layer=None):
    """The quantisation state that belongs to a packed weight (on the layer here, never on the tensor)."""
    if base_layer is not None and hasattr(base_layer, "quant_state"):
        return base_layer.quant_state()
    return getattr(W, "quant_state", None)


def get_lora_parameters(proj):
    """``(W, quant_state, bias, A, B, scaling, dropout)`` of a (possibly LoRA-wrapped, possibly 4-bit) projection;
    the four adapter entries are None for a bare layer or when the adapter is disabled or merged (the reference's
    tuple, fused_ops/unsloth_lora/utils.py:66-82)."""
    base, lora = _unwrap(proj)
    qs = base.quant_state() if hasattr(base, "quant_state") else None
    W = base.weight
    bias = getattr(base, "bias", None)
    if lora is None or getattr(lora, "disable_adapters", False) or getattr(lora, "merged", False):
        return W, qs, bias, None, None, None, None
    A, B, s = _lora_parts(lora)
    name = lora.active_adapters[0] if hasattr(lora, "active_adapters") else "default"
    drop = lora.lora_dropout[name] if hasattr(lora, "lora_dropout") else None
    return W, qs, bias, A, B, s, drop


def matmul_lora(X, W, W_quant, A, B, s, out=None, dropout=None):
    """``X W^T + s (dropout(X) A^T) B^T`` with ``W`` dense or 4-bit (``W_quant`` its state)."""
    Wd = fast_dequantize(W, W_quant) if W_quant is not None else W
    x2 = X.reshape(-1, X.shape[-1])
    cuda16 = x2.is_cuda and x2.dtype in (Wd.dtype,) and x2.dtype.itemsize == 2
    y = gemm(x2.contiguous(), Wd.contiguous(), out=out) if cuda16 else x2 @ Wd.to(x2.dtype).t()
    if A is not None:
        xd = dropout(x2) if dropout is not None else x2
        y = y + s * ((xd @ A.to(x2.dtype).t()) @ B.to(x2.dtype).t())
    return y.reshape(*X.shape[:-1], y.shape[-1])


def fast_linear_forward(proj, X, temp_lora=None, out=None):
    """Inference forward of a (LoRA-wrapped, possibly 4-bit) projection: ``X W^T (+ bias) + s (X A^T) B^T``
    (reference :209-247).  A few rows on a 4-bit base go through the fused dequantise+GEMM kernel."""
    W, qs, bias, A, B, s, _ = get_lora_parameters(proj)
    base, _lora = _unwrap(proj)
    rows = X.numel() // X.shape[-1]
    if qs is not None and X.is_cuda and rows <= 128:
        y = fast_gemv(X, base, qs)
        if A is not None:
            y = y + s * ((X @ A.to(X.dtype).t()) @ B.to(X.dtype).t())
    else:
        y = matmul_lora(X, W, qs, A, B, s)
    return y if bias is None else y + bias.to(y.dtype)
