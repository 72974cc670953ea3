"""baybridge_b200 — a B200-native execution backend behind the baybridge kernel DSL.

``import baybridge_b200 as cute`` gives the slice of the upstream
``import baybridge as cute`` surface that the hot path uses (upstream
``__init__.py:1-170``): ``@kernel`` / ``@jit``, ``TensorSpec``, runtime tensors,
``from_dlpack``, the scalar and tensor-SSA DSL, ``gemm`` / ``rmsnorm`` /
``attention`` and ``compile(..., backend="b200")`` whose artifact launches
hand-written sm_100a kernels.  ``B200Backend`` also plugs into an unmodified
upstream checkout: ``baybridge.compile(k, ..., backend=B200Backend(),
target=baybridge.NvidiaTarget("sm_100a"))`` or, after
``install_into_upstream()``, ``backend="b200"``.
"""
from .errors import (
    BackendNotImplementedError,
    BaybridgeError,
    CompilationError,
    CudaDriverError,
    UnsupportedOperationError,
)
from .scalar_types import ElementType
from .portable_ir import (
    AddressSpace,
    KernelArgument,
    LaunchConfig,
    Layout,
    Operation,
    PortableKernelIR,
    ScalarSpec,
    TensorSpec,
)
from .host_values import (
    BFloat16,
    Boolean,
    Float16,
    Float32,
    Int,
    Int8,
    Int32,
    Int64,
    RuntimeScalar,
    RuntimeTensor,
    Shape,
    Tensor,
    TensorHandle,
    clone,
    from_dlpack,
    tensor,
    zeros,
)
from .trace import ReductionOp, ScalarValue, TensorValue
from .dsl import (
    KernelDefinition,
    KernelLaunch,
    acos, arch, asin, empty_like, full, full_like, ones_like, zeros_like, atan, atan2, attention, block_dim, block_idx, ceil, copy, cos, dim, erf, exp, exp2, floor,
    gemm, grid_dim, jit, kernel, lane_id, layernorm, load, log, log10, log2, make_copy_atom, make_tensor, math, maximum, minimum, mma,
    partition, partition_program, partition_thread, barrier, program_id, rmsnorm, round, rsqrt, sin, sqrt, store, thread_idx, trunc, where,
)
from . import nvgpu
from .targets import AMDTarget, NvidiaTarget
from .driver import (
    CompiledKernel,
    GenerateLineInfo,
    LoweredModule,
    compile,
    register_backend,
    registered_backends,
)
from .backend import B200Backend, install_into_upstream

TensorSSA = (Tensor, TensorValue)
__version__ = "0.1.0"
