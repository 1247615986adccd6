"""CUDA compute gateway: grid / buffer validation (CPU) and NVRTC compile + dispatch (GPU)."""
import numpy as np
import pytest

from frankentorch_b200.ops.gateway import (BufferTooLarge, Gateway, GatewayError, Grid, MathMode, SizeOverflow,
                                           checked_byte_len, validate_buffer_size)


def test_grid_validation_matches_reference_rules():
    Grid.linear(4, 256).validate()
    Grid.grid_2d(2, 3, 16, 16).validate()
    with pytest.raises(GatewayError, match="zero extent"):
        Grid.linear(0, 32).validate()
    with pytest.raises(GatewayError, match="zero extent"):
        Grid((1, 1, 1), (32, 0, 1)).validate()
    big = 1 << 40
    with pytest.raises(SizeOverflow):
        Grid((big, big, 1), (1, 1, 1)).validate()
    with pytest.raises(SizeOverflow):
        Grid((big, 1, 1), (big, 1, 1)).validate()
    assert Grid.grid_2d(2, 3, 4, 5).threadgroup_count() == 6
    assert Grid.grid_2d(2, 3, 4, 5).threads_per_threadgroup_count() == 20


def test_buffer_size_checks():
    validate_buffer_size(16, 1024)
    with pytest.raises(GatewayError, match="zero-length"):
        validate_buffer_size(0, 1024)
    with pytest.raises(BufferTooLarge) as e:
        validate_buffer_size(2048, 1024)
    assert e.value.requested == 2048 and e.value.maximum == 1024
    assert checked_byte_len(10, 4, "x") == 40
    with pytest.raises(SizeOverflow):
        checked_byte_len(1 << 63, 4, "x")


SRC = r"""
extern "C" __global__ void saxpy(const float* x, float* y, const unsigned* n_and_a) {
  unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_and_a[0]) y[i] = 2.5f * x[i] + y[i];
}
"""


@pytest.mark.gpu
def test_compile_dispatch_readback(cuda_device):
    gw = Gateway.open()
    assert "B200" in gw.device_name() or gw.device_name()
    assert gw.max_threadgroup_memory() >= 48 * 1024
    assert not gw.has_unified_memory()
    lib = gw.library(SRC)
    pipe = lib.pipeline("saxpy")
    assert pipe.thread_execution_width() == 32 and pipe.max_threads_per_threadgroup() >= 256
    n = 1000
    x = np.arange(n, dtype=np.float32)
    y = np.ones(n, dtype=np.float32)
    bx, by, bn = gw.buffer_f32(x), gw.buffer_f32(y), gw.buffer_u32([n])
    gw.dispatch(pipe, [bx, by, bn], Grid.linear((n + 255) // 256, 256))
    out = np.empty(n, dtype=np.float32)
    by.read_f32(out)
    np.testing.assert_allclose(out, 2.5 * x + 1.0, rtol=0, atol=0)
    z = gw.buffer_zeroed(64)
    raw = np.full(64, 7, dtype=np.uint8)
    z.read_u8(raw)
    assert not raw.any()
    with pytest.raises(GatewayError, match="not found"):
        lib.pipeline("missing_kernel")
    with pytest.raises(GatewayError, match="failed to compile"):
        gw.library("this is not CUDA")
    with pytest.raises(GatewayError, match="exceeds the pipeline maximum"):
        gw.dispatch(pipe, [bx, by, bn], Grid.linear(1, 4096))
    with pytest.raises(GatewayError, match="zero-length"):
        gw.buffer_zeroed(0)
    fast = gw.library_with(SRC, MathMode.Fast)
    assert fast.mode is MathMode.Fast and fast.pipeline("saxpy").name == "saxpy"
