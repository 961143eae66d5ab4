"""``calculate_settings`` of the reference (fms_acceleration_foak/kernels/unsloth/utils.py:19-28) picked a Triton block
size and warp count for a row width.  The CUDA kernels choose their own launch shapes; the function is kept for
callers that only want the numbers."""
MAX_FUSED_SIZE = 65536


def calculate_settings(n: int):
    block = 1
    while block < n:
        block <<= 1
    if block > MAX_FUSED_SIZE:
        raise RuntimeError(f"Cannot launch a kernel since n = {n} exceeds the maximum block size = {MAX_FUSED_SIZE}.")
    warps = 32 if block >= 32768 else 16 if block >= 8192 else 8 if block >= 2048 else 4
    return block, warps
