"""Kernels and sample factories for the compare tool tests (the shape of upstream's tools/backend_benchmark_kernels.py)."""
import baybridge_b200 as cute

POINTWISE_N = 65536


@cute.kernel(launch=cute.LaunchConfig(grid=(POINTWISE_N // 256, 1, 1), block=(256, 1, 1)))
def indexed_add_f32_kernel(src: cute.Tensor, other: cute.Tensor, dst: cute.Tensor):
    tidx, _, _ = cute.arch.thread_idx()
    bidx, _, _ = cute.arch.block_idx()
    bdim, _, _ = cute.arch.block_dim()
    idx = bidx * bdim + tidx
    dst[idx] = src[idx] + other[idx]


class _Shape:
    def __init__(self, shape, dtype):
        self.shape, self.dtype = shape, dtype

    def __dlpack__(self, stream=None):
        return "capsule"

    def __dlpack_device__(self):
        return (2, 0)

    def data_ptr(self):
        return 0


def shape_only_args():
    """Enough to trace and lower without a device."""
    return [_Shape((POINTWISE_N,), "float32") for _ in range(3)]


def device_args():
    """Device-resident DLPack run arguments (upstream tools/backend_benchmark_kernels.py:1805-1842)."""
    import torch

    src = torch.arange(POINTWISE_N, device="cuda", dtype=torch.float32)
    other = torch.full((POINTWISE_N,), 2.0, device="cuda", dtype=torch.float32)
    return {"run_args": [src, other, torch.zeros_like(src)], "result_indices": [2]}
