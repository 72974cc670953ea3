"""Sample kernels of the hot path, shared by the benchmark, the build step, the golden-vector
generator and the parity tests.

Every kernel here is written once against a DSL module handle ``cute`` so that
the *same Python body* can be traced by the upstream package (when the golden
vectors are generated) and by ``baybridge_b200`` (everywhere else).  The
bodies follow the upstream samples: the indexed forms use the canonical
``block_idx * block_dim + thread_idx`` prefix of
``tools/backend_benchmark_kernels.py:691-697`` and the explicit-op kernels are
the one-liners of ``tests/test_backend_hipkittens_exec.py`` /
``tests/test_backend_hipkittens_exec_norm_attention.py``.
"""
from __future__ import annotations

from types import SimpleNamespace


def build_zoo(cute) -> SimpleNamespace:
    zoo = SimpleNamespace()

    # ---- config 1: rank-2 indexed f32 add, one thread per element -------------------------
    def make_indexed_add_2d(rows: int, cols: int, block: int = 256):
        @cute.kernel
        def indexed_add_2d_kernel(g_a: cute.Tensor, g_b: cute.Tensor, g_c: cute.Tensor):
            tidx, _, _ = cute.arch.thread_idx()
            bidx, _, _ = cute.arch.block_idx()
            bdim, _, _ = cute.arch.block_dim()
            i = bidx * bdim + tidx
            col = i % cols
            row = i // cols
            g_c[row, col] = g_a[row, col] + g_b[row, col]

        @cute.jit
        def indexed_add_2d(g_a: cute.Tensor, g_b: cute.Tensor, g_c: cute.Tensor):
            indexed_add_2d_kernel(g_a, g_b, g_c).launch(
                grid=((rows * cols + block - 1) // block, 1, 1), block=(block, 1, 1)
            )

        return indexed_add_2d

    zoo.make_indexed_add_2d = make_indexed_add_2d

    # ---- config 2: fused c = a*b + a, indexed and tensor-SSA forms ---------------------------
    def make_fused_mul_add_indexed(n: int, block: int = 256):
        @cute.kernel
        def fused_mul_add_kernel(a: cute.Tensor, b: cute.Tensor, c: cute.Tensor):
            tidx, _, _ = cute.arch.thread_idx()
            bidx, _, _ = cute.arch.block_idx()
            bdim, _, _ = cute.arch.block_dim()
            i = bidx * bdim + tidx
            c[i] = a[i] * b[i] + a[i]

        @cute.jit
        def fused_mul_add_indexed(a: cute.Tensor, b: cute.Tensor, c: cute.Tensor):
            fused_mul_add_kernel(a, b, c).launch(grid=((n + block - 1) // block, 1, 1), block=(block, 1, 1))

        return fused_mul_add_indexed

    zoo.make_fused_mul_add_indexed = make_fused_mul_add_indexed

    @cute.kernel
    def fused_mul_add_ssa(a: cute.Tensor, b: cute.Tensor, c: cute.Tensor):
        av = a.load()
        bv = b.load()
        c.store(av * bv + av)

    zoo.fused_mul_add_ssa = fused_mul_add_ssa

    # ---- reducing copy: dst = dst (op) src over whole tensors (upstream tests/test_backend_ptx_exec.py:227-302, 534-560) ----
    def make_copy_reduce(reduction: str, grid: int = 1, block: int = 1):
        import importlib

        nvgpu = importlib.import_module(cute.__name__ + ".nvgpu")
        kind = getattr(nvgpu.cpasync.ReductionOp, reduction.upper())

        @cute.kernel(launch=cute.LaunchConfig(grid=(grid, 1, 1), block=(block, 1, 1)))
        def copy_reduce_kernel(src: cute.Tensor, dst: cute.Tensor):
            atom = cute.make_copy_atom(nvgpu.cpasync.CopyReduceBulkTensorTileS2GOp(kind, nvgpu.tcgen05.CtaGroup.ONE), src.element_type)
            cute.copy(atom, src, dst)

        return copy_reduce_kernel

    zoo.make_copy_reduce = make_copy_reduce

    # ---- whole-tensor (tensor-SSA) families under the three launch shapes upstream's conformance kernels use ---------
    # (tests/test_backend_ptx_exec.py:430-1560: serial = one thread, parallel = one block, multiblock = a 2-D grid)
    launches = {"serial": ((1, 1, 1), (1, 1, 1)), "parallel": ((1, 1, 1), (64, 1, 1)), "multiblock": ((2, 2, 1), (2, 1, 1))}
    binary_ops = {
        "add": lambda a, b: a + b, "sub": lambda a, b: a - b, "mul": lambda a, b: a * b, "div": lambda a, b: a / b,
        "max": lambda a, b: cute.maximum(a, b), "min": lambda a, b: cute.minimum(a, b), "atan2": lambda a, b: cute.math.atan2(a, b),
        "bitand": lambda a, b: a & b, "bitor": lambda a, b: a | b, "bitxor": lambda a, b: a ^ b,
        "cmp_lt": lambda a, b: a < b, "cmp_eq": lambda a, b: a == b,
    }
    unary_ops = {
        "sqrt": cute.sqrt, "rsqrt": cute.rsqrt, "sin": cute.sin, "cos": cute.cos, "exp2": cute.exp2, "exp": cute.exp,
        "log2": cute.log2, "log": cute.log, "log10": cute.log10, "round": cute.round, "floor": cute.floor, "ceil": cute.ceil,
        "trunc": cute.trunc, "atan": cute.atan, "asin": cute.asin, "acos": cute.acos, "erf": cute.erf,
        "neg": lambda a: -a, "abs": lambda a: abs(a), "bitnot": lambda a: ~a,
    }
    zoo.launch_shapes = launches

    def _launch(shape: str):
        grid, block = launches[shape]
        return cute.LaunchConfig(grid=grid, block=block)

    def make_dense_binary(op: str, shape: str = "serial"):
        """``dst = lhs (op) rhs`` over whole tensors; operands of different shapes broadcast as upstream's tracer does."""
        body = binary_ops[op]

        @cute.kernel(launch=_launch(shape))
        def dense_binary_kernel(lhs: cute.Tensor, rhs: cute.Tensor, dst: cute.Tensor):
            dst.store(body(lhs.load(), rhs.load()))

        return dense_binary_kernel

    zoo.make_dense_binary = make_dense_binary

    def make_dense_unary(op: str, shape: str = "serial"):
        body = unary_ops[op]

        @cute.kernel(launch=_launch(shape))
        def dense_unary_kernel(src: cute.Tensor, dst: cute.Tensor):
            dst.store(body(src.load()))

        return dense_unary_kernel

    zoo.make_dense_unary = make_dense_unary

    def make_dense_scalar_binary(op: str, scalar: str = "f32", shape: str = "serial"):
        """``dst = src (op) alpha`` with ``alpha`` a kernel scalar parameter."""
        body = binary_ops[op]
        if scalar == "f32":
            @cute.kernel(launch=_launch(shape))
            def dense_scalar_binary_kernel(src: cute.Tensor, alpha: cute.Float32, dst: cute.Tensor):
                dst.store(body(src.load(), alpha))
        else:
            @cute.kernel(launch=_launch(shape))
            def dense_scalar_binary_kernel(src: cute.Tensor, alpha: cute.Int32, dst: cute.Tensor):
                dst.store(body(src.load(), alpha))

        return dense_scalar_binary_kernel

    zoo.make_dense_scalar_binary = make_dense_scalar_binary

    def make_dense_tensor_scalar_binary(op: str, shape: str = "serial"):
        """``dst = src (op) alpha[0]`` with ``alpha`` a one-element tensor."""
        body = binary_ops[op]

        @cute.kernel(launch=_launch(shape))
        def dense_tensor_scalar_binary_kernel(src: cute.Tensor, alpha: cute.Tensor, dst: cute.Tensor):
            dst.store(body(src.load(), alpha[0]))

        return dense_tensor_scalar_binary_kernel

    zoo.make_dense_tensor_scalar_binary = make_dense_tensor_scalar_binary

    def make_dense_select(form: str = "tensor", shape: str = "serial"):
        """``where`` over whole tensors: both branches tensors, or one branch a scalar parameter / a one-element tensor."""
        if form == "tensor":
            @cute.kernel(launch=_launch(shape))
            def dense_select_kernel(pred: cute.Tensor, lhs: cute.Tensor, rhs: cute.Tensor, dst: cute.Tensor):
                dst.store(cute.where(pred.load(), lhs.load(), rhs.load()))
        elif form == "scalar":
            @cute.kernel(launch=_launch(shape))
            def dense_select_kernel(pred: cute.Tensor, src: cute.Tensor, alpha: cute.Float32, dst: cute.Tensor):
                dst.store(cute.where(pred.load(), src.load(), alpha))
        else:
            @cute.kernel(launch=_launch(shape))
            def dense_select_kernel(pred: cute.Tensor, src: cute.Tensor, alpha: cute.Tensor, dst: cute.Tensor):
                dst.store(cute.where(pred.load(), alpha[0], src.load()))

        return dense_select_kernel

    zoo.make_dense_select = make_dense_select

    def make_dense_copy(shape: str = "serial"):
        @cute.kernel(launch=_launch(shape))
        def dense_copy_kernel(src: cute.Tensor, dst: cute.Tensor):
            cute.copy(src, dst)

        return dense_copy_kernel

    zoo.make_dense_copy = make_dense_copy

    def make_reduce(op: str, init, axis: str = "all", shape: str = "serial"):
        """``Tensor.reduce`` to a scalar (``dst[0]``), per row or per column (upstream tests/test_backend_ptx_exec.py:1949-2200)."""
        kind = getattr(cute.ReductionOp, op.upper())
        if axis == "all":
            @cute.kernel(launch=_launch(shape))
            def reduce_kernel(src: cute.Tensor, dst: cute.Tensor):
                dst[0] = src.reduce(kind, init, reduction_profile=0)
        else:
            profile = (None, 1) if axis == "rows" else (1, None)

            @cute.kernel(launch=_launch(shape))
            def reduce_kernel(src: cute.Tensor, dst: cute.Tensor):
                dst.store(src.load().reduce(kind, init, reduction_profile=profile))

        return reduce_kernel

    zoo.make_reduce = make_reduce

    # ---- rank-1 indexed binary family (upstream PTX conformance shape) --------------------------
    def make_indexed_binary(op: str, n: int, block: int = 128):
        def body(lhs, rhs):
            if op == "add":
                return lhs + rhs
            if op == "sub":
                return lhs - rhs
            if op == "mul":
                return lhs * rhs
            if op == "div":
                return lhs / rhs
            if op == "max":
                return cute.maximum(lhs, rhs)
            if op == "min":
                return cute.minimum(lhs, rhs)
            raise ValueError(op)

        @cute.kernel(launch=cute.LaunchConfig(grid=((n + block - 1) // block, 1, 1), block=(block, 1, 1)))
        def indexed_binary_kernel(src: cute.Tensor, other: cute.Tensor, dst: cute.Tensor):
            tidx, _, _ = cute.arch.thread_idx()
            bidx, _, _ = cute.arch.block_idx()
            bdim, _, _ = cute.arch.block_dim()
            idx = bidx * bdim + tidx
            dst[idx] = body(src[idx], other[idx])

        return indexed_binary_kernel

    zoo.make_indexed_binary = make_indexed_binary

    def make_indexed_unary(op: str, n: int, block: int = 128):
        @cute.kernel(launch=cute.LaunchConfig(grid=((n + block - 1) // block, 1, 1), block=(block, 1, 1)))
        def indexed_unary_kernel(src: cute.Tensor, dst: cute.Tensor):
            idx = cute.program_id("x") * cute.block_dim("x") + cute.thread_idx("x")
            value = cute.load(src, idx)
            if op == "neg":
                result = -value
            elif op == "abs":
                result = abs(value)
            elif op == "copy":
                result = value
            else:
                result = getattr(cute.math, op)(value)
            cute.store(result, dst, idx)

        return indexed_unary_kernel

    zoo.make_indexed_unary = make_indexed_unary

    # relu-like: compare → select, with a literal constant operand
    def make_indexed_clamp_scale(n: int, block: int = 128):
        @cute.kernel(launch=cute.LaunchConfig(grid=((n + block - 1) // block, 1, 1), block=(block, 1, 1)))
        def indexed_clamp_scale_kernel(src: cute.Tensor, dst: cute.Tensor, alpha: float):
            tidx, _, _ = cute.arch.thread_idx()
            bidx, _, _ = cute.arch.block_idx()
            bdim, _, _ = cute.arch.block_dim()
            idx = bidx * bdim + tidx
            value = src[idx]
            dst[idx] = cute.where(value > 0.0, value * alpha, 0.0)

        return indexed_clamp_scale_kernel

    zoo.make_indexed_clamp_scale = make_indexed_clamp_scale

    # over-provisioned grid guarded by a predicate (masked load / masked store)
    def make_indexed_masked_add(n: int, block: int = 128):
        grid = (n + block - 1) // block

        @cute.kernel(launch=cute.LaunchConfig(grid=(grid, 1, 1), block=(block, 1, 1)))
        def indexed_masked_add_kernel(src: cute.Tensor, other: cute.Tensor, dst: cute.Tensor):
            tidx, _, _ = cute.arch.thread_idx()
            bidx, _, _ = cute.arch.block_idx()
            bdim, _, _ = cute.arch.block_dim()
            idx = bidx * bdim + tidx
            inside = idx < n
            lhs = cute.load(src, idx, predicate=inside, else_value=0.0)
            rhs = cute.load(other, idx, predicate=inside, else_value=0.0)
            cute.store(lhs + rhs, dst, idx, predicate=inside)

        return indexed_masked_add_kernel

    zoo.make_indexed_masked_add = make_indexed_masked_add

    # zero padding: the load is guarded, the store is not, so elements past `valid` receive f(else_value)
    def make_indexed_padded_increment(n: int, valid: int, block: int = 128):
        @cute.kernel(launch=cute.LaunchConfig(grid=((n + block - 1) // block, 1, 1), block=(block, 1, 1)))
        def indexed_padded_increment_kernel(src: cute.Tensor, dst: cute.Tensor):
            tidx, _, _ = cute.arch.thread_idx()
            bidx, _, _ = cute.arch.block_idx()
            bdim, _, _ = cute.arch.block_dim()
            idx = bidx * bdim + tidx
            value = cute.load(src, idx, predicate=idx < valid, else_value=0.0)
            dst[idx] = value + 1.0

        return indexed_padded_increment_kernel

    zoo.make_indexed_padded_increment = make_indexed_padded_increment

    # reversed copy from an over-provisioned, unguarded grid: threads past n index outside both tensors
    def make_indexed_reverse(n: int, block: int = 128):
        @cute.kernel(launch=cute.LaunchConfig(grid=((n + block - 1) // block, 1, 1), block=(block, 1, 1)))
        def indexed_reverse_kernel(src: cute.Tensor, dst: cute.Tensor):
            tidx, _, _ = cute.arch.thread_idx()
            bidx, _, _ = cute.arch.block_idx()
            bdim, _, _ = cute.arch.block_dim()
            idx = bidx * bdim + tidx
            dst[n - 1 - idx] = src[idx]

        return indexed_reverse_kernel

    zoo.make_indexed_reverse = make_indexed_reverse

    # read-modify-write of one tensor: dst[i] = dst[i] + src[i]
    def make_indexed_accumulate(n: int, block: int = 128):
        @cute.kernel(launch=cute.LaunchConfig(grid=((n + block - 1) // block, 1, 1), block=(block, 1, 1)))
        def indexed_accumulate_kernel(src: cute.Tensor, dst: cute.Tensor):
            tidx, _, _ = cute.arch.thread_idx()
            bidx, _, _ = cute.arch.block_idx()
            bdim, _, _ = cute.arch.block_dim()
            idx = bidx * bdim + tidx
            dst[idx] = dst[idx] + src[idx]

        return indexed_accumulate_kernel

    zoo.make_indexed_accumulate = make_indexed_accumulate

    # tensor-SSA pointwise forms
    @cute.kernel
    def ssa_add(a: cute.Tensor, b: cute.Tensor, c: cute.Tensor):
        c.store(a.load() + b.load())

    zoo.ssa_add = ssa_add

    @cute.kernel
    def ssa_scale_shift(a: cute.Tensor, c: cute.Tensor):
        c.store(a.load() * 0.5 - 2.0)

    zoo.ssa_scale_shift = ssa_scale_shift

    @cute.kernel
    def ssa_exp_max(a: cute.Tensor, b: cute.Tensor, c: cute.Tensor):
        c.store(cute.maximum(cute.math.exp(a.load()), b.load()))

    zoo.ssa_exp_max = ssa_exp_max

    # ---- integer / predicate families of upstream's PTX conformance tests (tests/test_backend_ptx_exec.py:70-215) ----
    def make_indexed_bitwise(op: str, n: int, block: int = 64):
        @cute.kernel(launch=cute.LaunchConfig(grid=((n + block - 1) // block, 1, 1), block=(block, 1, 1)))
        def indexed_bitwise_kernel(a: cute.Tensor, b: cute.Tensor, c: cute.Tensor):
            tidx, _, _ = cute.arch.thread_idx()
            bidx, _, _ = cute.arch.block_idx()
            bdim, _, _ = cute.arch.block_dim()
            idx = bidx * bdim + tidx
            if op == "and":
                c[idx] = a[idx] & b[idx]
            elif op == "or":
                c[idx] = a[idx] | b[idx]
            elif op == "xor":
                c[idx] = a[idx] ^ b[idx]
            else:
                c[idx] = ~a[idx]

        return indexed_bitwise_kernel

    zoo.make_indexed_bitwise = make_indexed_bitwise

    def make_indexed_compare_select(n: int, block: int = 64):
        """mask[i] = a[i] < b[i] (an i1 tensor), then c[i] = mask[i] ? a[i] : b[i] read back from that tensor."""

        @cute.kernel(launch=cute.LaunchConfig(grid=((n + block - 1) // block, 1, 1), block=(block, 1, 1)))
        def indexed_compare_select_kernel(a: cute.Tensor, b: cute.Tensor, mask: cute.Tensor, c: cute.Tensor):
            tidx, _, _ = cute.arch.thread_idx()
            bidx, _, _ = cute.arch.block_idx()
            bdim, _, _ = cute.arch.block_dim()
            idx = bidx * bdim + tidx
            mask[idx] = a[idx] < b[idx]
            c[idx] = cute.where(mask[idx], a[idx], b[idx])

        return indexed_compare_select_kernel

    zoo.make_indexed_compare_select = make_indexed_compare_select

    # a one-element tensor used as a broadcast scalar (tests/test_backend_ptx_exec.py:195-201)
    def make_indexed_extent1_scalar(n: int, block: int = 64):
        @cute.kernel(launch=cute.LaunchConfig(grid=((n + block - 1) // block, 1, 1), block=(block, 1, 1)))
        def indexed_extent1_scalar_kernel(src: cute.Tensor, alpha: cute.Tensor, dst: cute.Tensor):
            tidx, _, _ = cute.arch.thread_idx()
            bidx, _, _ = cute.arch.block_idx()
            bdim, _, _ = cute.arch.block_dim()
            idx = bidx * bdim + tidx
            dst[idx] = src[idx] * alpha[0]

        return indexed_extent1_scalar_kernel

    zoo.make_indexed_extent1_scalar = make_indexed_extent1_scalar

    @cute.kernel
    def ssa_extent1_scalar(a: cute.Tensor, alpha: cute.Tensor, c: cute.Tensor):
        c.store(a.load() + alpha[0])

    zoo.ssa_extent1_scalar = ssa_extent1_scalar

    # rank-2 broadcasting: a row vector [1, C] and a column vector [R, 1] against [R, C]
    @cute.kernel
    def ssa_broadcast_row_col(a: cute.Tensor, row: cute.Tensor, col: cute.Tensor, c: cute.Tensor):
        c.store((a.load() + row.load()) * col.load())

    zoo.ssa_broadcast_row_col = ssa_broadcast_row_col

    # register tensors filled with constants (tests/test_backend_ptx_exec.py:2382-2393)
    @cute.kernel
    def factory_bundle(dst_zero: cute.Tensor, dst_one: cute.Tensor, dst_full: cute.Tensor):
        dst_zero.store(cute.zeros_like(dst_zero))
        dst_one.store(cute.ones_like(dst_one))
        dst_full.store(cute.full_like(dst_full, 7.0))

    zoo.factory_bundle = factory_bundle

    # several folds of one loaded tensor (tests/test_backend_ptx_exec.py:2370-2379)
    @cute.kernel
    def reduce_bundle_xor(src: cute.Tensor, dst_scalar: cute.Tensor, dst_rows: cute.Tensor, dst_cols: cute.Tensor):
        src_vec = src.load()
        dst_scalar[0] = src_vec.reduce(cute.ReductionOp.XOR, 0, reduction_profile=0)
        dst_rows.store(src_vec.reduce(cute.ReductionOp.XOR, 0, reduction_profile=(None, 1)))
        dst_cols.store(src_vec.reduce(cute.ReductionOp.XOR, 0, reduction_profile=(1, None)))

    zoo.reduce_bundle_xor = reduce_bundle_xor

    @cute.kernel
    def reduce_bundle_add(src: cute.Tensor, dst_scalar: cute.Tensor, dst_rows: cute.Tensor, dst_cols: cute.Tensor):
        src_vec = src.load()
        dst_scalar[0] = src_vec.reduce(cute.ReductionOp.ADD, 0.0, reduction_profile=0)
        dst_rows.store(src_vec.reduce(cute.ReductionOp.ADD, 0.0, reduction_profile=(None, 1)))
        dst_cols.store(src_vec.reduce(cute.ReductionOp.MAX, -1000.0, reduction_profile=(1, None)))

    zoo.reduce_bundle_add = reduce_bundle_add

    # a fold taken straight from the kernel argument, no explicit load (tests/test_backend_ptx_exec.py:2410-2412)
    @cute.kernel
    def reduce_argument_max(src: cute.Tensor, dst: cute.Tensor):
        dst[0] = src.reduce(cute.ReductionOp.MAX, -99, reduction_profile=0)

    zoo.reduce_argument_max = reduce_argument_max

    # ---- reductions (map, then fold) ----------------------------------------------------------------
    @cute.kernel
    def row_sum_of_squares(src: cute.Tensor, dst: cute.Tensor):
        v = src.load()
        dst.store((v * v).reduce(cute.ReductionOp.ADD, 0.0, reduction_profile=(None, 1)))

    zoo.row_sum_of_squares = row_sum_of_squares

    @cute.kernel
    def column_max(src: cute.Tensor, dst: cute.Tensor):
        dst.store(src.load().reduce(cute.ReductionOp.MAX, -1000.0, reduction_profile=(1, None)))

    zoo.column_max = column_max

    @cute.kernel
    def total_sum(src: cute.Tensor, dst: cute.Tensor):
        dst[0] = src.load().reduce(cute.ReductionOp.ADD, 1.0)

    zoo.total_sum = total_sum

    # ---- explicit single-op kernels ---------------------------------------------------------------
    @cute.kernel
    def gemm_abt(a: cute.Tensor, b: cute.Tensor, c: cute.Tensor):
        cute.gemm(a, b, c, transpose_b=True)

    zoo.gemm_abt = gemm_abt

    @cute.kernel
    def gemm_ab(a: cute.Tensor, b: cute.Tensor, c: cute.Tensor):
        cute.gemm(a, b, c)

    zoo.gemm_ab = gemm_ab

    @cute.kernel
    def gemm_atb(a: cute.Tensor, b: cute.Tensor, c: cute.Tensor):
        cute.gemm(a, b, c, transpose_a=True)

    zoo.gemm_atb = gemm_atb

    @cute.kernel
    def gemm_atbt(a: cute.Tensor, b: cute.Tensor, c: cute.Tensor):
        cute.gemm(a, b, c, transpose_a=True, transpose_b=True)

    zoo.gemm_atbt = gemm_atbt

    # a GEMM written per program: every program multiplies its own tiles of A and B into its tile of C
    def make_tiled_gemm(m: int, n: int, k: int, tile_m: int, tile_n: int, *, transpose_b: bool = True, block: int = 1):
        @cute.kernel(launch=cute.LaunchConfig(grid=(m // tile_m, n // tile_n, 1), block=(block, 1, 1)))
        def tiled_gemm_kernel(a: cute.Tensor, b: cute.Tensor, c: cute.Tensor):
            a_tile = cute.partition_program(a, (tile_m, k), axes=("x", "z"))
            if transpose_b:
                b_tile = cute.partition_program(b, (tile_n, k), axes=("y", "z"))
            else:
                b_tile = cute.partition_program(b, (k, tile_n), axes=("z", "y"))
            c_tile = cute.partition_program(c, (tile_m, tile_n), axes=("x", "y"))
            cute.gemm(a_tile, b_tile, c_tile, transpose_b=transpose_b)
            cute.barrier()

        return tiled_gemm_kernel

    zoo.make_tiled_gemm = make_tiled_gemm

    # tracing-only shapes of upstream's tests/test_api.py:6-36 (views, register accumulator, barrier, topology)
    @cute.kernel
    def api_vector_copy(src: cute.Tensor, dst: cute.Tensor):
        cute.copy(src, dst, vector_bytes=16)

    zoo.api_vector_copy = api_vector_copy

    @cute.jit(launch=cute.LaunchConfig(grid=(80, 1, 1), block=(256, 1, 1), shared_mem_bytes=4096))
    def api_tile_mma(a: cute.Tensor, b: cute.Tensor):
        a_tile = cute.partition(a, (16, 16))
        b_tile = cute.partition(b, (16, 16))
        cute.mma(a_tile, b_tile, tile=(16, 16, 16))
        cute.barrier()

    zoo.api_tile_mma = api_tile_mma

    @cute.kernel(launch=cute.LaunchConfig(grid=(120, 3, 1), block=(256, 1, 1)))
    def api_topology(src: cute.Tensor, dst: cute.Tensor):
        cute.program_id("x")
        cute.block_idx("y")
        cute.thread_idx("x")
        cute.block_dim("x")
        cute.grid_dim("y")
        cute.lane_id()
        cute.copy(src, dst)

    zoo.api_topology = api_topology

    def make_rmsnorm(epsilon: float | None = None):
        if epsilon is None:

            @cute.kernel
            def rmsnorm_default_eps(x: cute.Tensor, out: cute.Tensor, gamma: cute.Tensor):
                cute.rmsnorm(x, out, gamma)

            return rmsnorm_default_eps

        @cute.kernel
        def rmsnorm_kernel(x: cute.Tensor, out: cute.Tensor, gamma: cute.Tensor):
            cute.rmsnorm(x, out, gamma, epsilon=epsilon)

        return rmsnorm_kernel

    zoo.make_rmsnorm = make_rmsnorm

    @cute.kernel
    def layernorm_kernel(x: cute.Tensor, residual: cute.Tensor, out: cute.Tensor, out_resid: cute.Tensor,
                         weight: cute.Tensor, bias: cute.Tensor):
        cute.layernorm(x, residual, out, out_resid, weight, bias)

    zoo.layernorm_kernel = layernorm_kernel

    @cute.kernel
    def attention_full(q: cute.Tensor, k: cute.Tensor, v: cute.Tensor, out: cute.Tensor, lse: cute.Tensor):
        cute.attention(q, k, v, out, lse)

    zoo.attention_full = attention_full

    @cute.kernel
    def attention_causal(q: cute.Tensor, k: cute.Tensor, v: cute.Tensor, out: cute.Tensor, lse: cute.Tensor):
        cute.attention(q, k, v, out, lse, causal=True)

    zoo.attention_causal = attention_causal

    return zoo
