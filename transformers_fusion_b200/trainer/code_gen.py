"""Shape-specialised kernel source generator for sm_100a.

Given a kernel type and concrete sizes it emits a self-contained CUDA C++ translation unit (one ``extern "C"`` launcher
per kernel), checks it by compiling with nvcc for ``sm_100a`` (which works without a GPU), optionally loads the shared
object and runs it against a PyTorch statement of the same op, and keeps the result in a cache.  The generated kernels
are the memory-bound, shape-dependent ones (activation chains, norms, softmax, embedding, quantise / dequantise, a
shared-memory-tiled GEMM for odd small shapes): sizes are compile-time constants, loops are unrolled and loads are
vectorised to the widest width the size allows.  The tensor-core GEMM and attention kernels of the framework are
hand-written and are not produced here.

Reference counterpart: code_gen::CodeGenerator (include/quant/code_gen.h:14-200, src/trainer/code_gen.cpp), which emits
scalar / AVX2 / AVX-512 / NEON C++; the targets here are vector widths of CUDA loads instead of SIMD instruction sets."""
from __future__ import annotations

import ctypes
import enum
import hashlib
import os
import shutil
import subprocess
import tempfile
from dataclasses import dataclass, field
from typing import Dict, List, Optional


class KernelType(enum.IntEnum):
    GEMM = 0
    ATTENTION = 1
    RMS_NORM = 2
    LAYER_NORM = 3
    SOFTMAX = 4
    RELU = 5
    SILU = 6
    GELU = 7
    ADD = 8
    MUL = 9
    SCALE = 10
    RESIDUAL_ADD = 11
    EMBEDDING_LOOKUP = 12
    HEAD_PROJECTION = 13
    QUANTIZE_DEQUANTIZE = 14


class VectorWidth(enum.IntEnum):
    """Elements (bf16) per load: the counterpart of the reference's SIMD target."""
    SCALAR = 1
    V2 = 2
    V4 = 4
    V8 = 8


class UnrollLevel(enum.IntEnum):
    NONE = 0
    PARTIAL = 1
    FULL = 2


@dataclass
class KernelSpec:
    type: KernelType = KernelType.GEMM
    M: int = 0
    N: int = 0
    K: int = 0
    block_size: int = 256
    width: VectorWidth = VectorWidth.V8
    unroll: UnrollLevel = UnrollLevel.PARTIAL
    fused: bool = False
    scale: float = 1.0
    name: str = ""


@dataclass
class CodeTemplate:
    name: str
    description: str
    template_code: str
    placeholders: List[str]
    kernel_type: KernelType


@dataclass
class GeneratedKernel:
    spec: KernelSpec
    source_code: str = ""
    function_name: str = ""
    validated: bool = False
    compiled: bool = False
    benchmark_ms: float = 0.0
    error_message: str = ""
    so_path: str = ""


@dataclass
class SlowPath:
    op_name: str
    current_time_ms: float = 0.0
    target_time_ms: float = 0.0
    current_kernel: str = ""
    priority: int = 0


@dataclass
class CodeValidationResult:
    syntax_valid: bool = False
    compiles: bool = False
    runs: bool = False
    correctness_pass: bool = False
    max_error: float = 0.0
    error_message: str = ""
    runtime_ms: float = 0.0


_HEADER = '''#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#define GEN_API extern "C" __attribute__((visibility("default")))
__device__ __forceinline__ float gen_silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float gen_gelu(float x) { return 0.5f * x * (1.f + tanhf(0.7978845608f * (x + 0.044715f * x * x * x))); }
__device__ __forceinline__ float gen_warp_sum(float v) { for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(~0u, v, o); return v; }
__device__ __forceinline__ float gen_warp_max(float v) { for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(~0u, v, o)); return v; }
'''

_UNARY = {KernelType.RELU: "fmaxf(x, 0.f)", KernelType.SILU: "gen_silu(x)", KernelType.GELU: "gen_gelu(x)"}
_BINARY = {KernelType.ADD: "x + y", KernelType.MUL: "x * y", KernelType.RESIDUAL_ADD: "x + y"}


class CodeGenerator:
    def __init__(self, model=None, work_dir: Optional[str] = None):
        self.model = model
        self.kernels: Dict[str, GeneratedKernel] = {}
        self.templates: Dict[str, CodeTemplate] = {}
        self.slow_paths: List[SlowPath] = []
        self.work_dir = work_dir or tempfile.mkdtemp(prefix="tfb_codegen_")
        self._init_default_templates()

    def set_model(self, model): self.model = model

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _width_for(n: int, want: int) -> int:
        w = int(want)
        while w > 1 and n % w:
            w //= 2
        return w

    @staticmethod
    def make_function_name(spec: KernelSpec) -> str:
        dims = "_".join(str(d) for d in (spec.M, spec.N, spec.K) if d)
        return spec.name or f"gen_{spec.type.name.lower()}_{dims}_v{int(spec.width)}"

    def generate_includes(self, includes: List[str]) -> str:
        return "".join(f"#include <{i}>\n" for i in includes)

    def generate_unrolled_loop(self, var: str, start: int, end: int, unroll_factor: int, body: str) -> str:
        pragma = f"#pragma unroll {unroll_factor}\n" if unroll_factor > 1 else ""
        return f"{pragma}for (int {var} = {start}; {var} < {end}; ++{var}) {{\n{body}\n}}\n"

    def generate_vector_load(self, var: str, ptr: str, width: int) -> str:
        ty = {8: "uint4", 4: "uint2", 2: "uint32_t", 1: "uint16_t"}[width]
        return f"const {ty} {var} = *reinterpret_cast<const {ty}*>({ptr});"

    def generate_vector_store(self, ptr: str, var: str, width: int) -> str:
        ty = {8: "uint4", 4: "uint2", 2: "uint32_t", 1: "uint16_t"}[width]
        return f"*reinterpret_cast<{ty}*>({ptr}) = {var};"

    # ------------------------------------------------------------------ generators
    def _elementwise(self, fn: str, n: int, expr: str, binary: bool, width: int, block: int) -> str:
        w = self._width_for(n, width)
        ld = lambda name, p: (f"    __align__(16) __nv_bfloat16 {name}[{w}];\n"
                              f"    *reinterpret_cast<{self._vec_ty(w)}*>({name}) = *reinterpret_cast<const {self._vec_ty(w)}*>({p} + i);\n")
        body = ld("a", "A") + (ld("b", "B") if binary else "") + f"    __align__(16) __nv_bfloat16 o[{w}];\n#pragma unroll\n    for (int j = 0; j < {w}; ++j) {{\n" \
            f"      const float x = __bfloat162float(a[j]);{' const float y = __bfloat162float(b[j]);' if binary else ''}\n" \
            f"      o[j] = __float2bfloat16({expr});\n    }}\n" \
            f"    *reinterpret_cast<{self._vec_ty(w)}*>(O + i) = *reinterpret_cast<const {self._vec_ty(w)}*>(o);\n"
        args = "const __nv_bfloat16* __restrict__ A, " + ("const __nv_bfloat16* __restrict__ B, " if binary else "") + "__nv_bfloat16* __restrict__ O"
        call = "A, " + ("B, " if binary else "") + "O"
        grid = (n // w + block - 1) // block
        return (f"__global__ void __launch_bounds__({block}) {fn}_k({args}) {{\n"
                f"  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * {w}; i < {n}LL; i += (long long)gridDim.x * blockDim.x * {w}) {{\n"
                f"{body}  }}\n}}\n"
                f"GEN_API int {fn}({args.replace(' __restrict__', '')}, void* stream) {{\n"
                f"  {fn}_k<<<{min(grid, 148 * 8)}, {block}, 0, static_cast<cudaStream_t>(stream)>>>({call});\n  return int(cudaGetLastError());\n}}\n")

    @staticmethod
    def _vec_ty(w: int) -> str:
        return {8: "uint4", 4: "uint2", 2: "uint32_t", 1: "uint16_t"}[w]

    def generate_relu(self, n, width=VectorWidth.V8): return self._gen(KernelSpec(KernelType.RELU, N=n, width=width))
    def generate_silu(self, n, width=VectorWidth.V8): return self._gen(KernelSpec(KernelType.SILU, N=n, width=width))
    def generate_gelu(self, n, width=VectorWidth.V8): return self._gen(KernelSpec(KernelType.GELU, N=n, width=width))
    def generate_add(self, n, width=VectorWidth.V8): return self._gen(KernelSpec(KernelType.ADD, N=n, width=width))
    def generate_mul(self, n, width=VectorWidth.V8): return self._gen(KernelSpec(KernelType.MUL, N=n, width=width))
    def generate_residual_add(self, n, width=VectorWidth.V8): return self._gen(KernelSpec(KernelType.RESIDUAL_ADD, N=n, width=width))
    def generate_scale(self, n, scale_val, width=VectorWidth.V8): return self._gen(KernelSpec(KernelType.SCALE, N=n, width=width, scale=scale_val))
    def generate_rms_norm(self, dim, rows=1, width=VectorWidth.V8): return self._gen(KernelSpec(KernelType.RMS_NORM, M=rows, N=dim, width=width))
    def generate_layer_norm(self, dim, rows=1, width=VectorWidth.V8): return self._gen(KernelSpec(KernelType.LAYER_NORM, M=rows, N=dim, width=width))
    def generate_softmax(self, dim, rows=1, width=VectorWidth.V8): return self._gen(KernelSpec(KernelType.SOFTMAX, M=rows, N=dim, width=width))
    def generate_embedding_lookup(self, vocab_size, embed_dim, width=VectorWidth.V8):
        return self._gen(KernelSpec(KernelType.EMBEDDING_LOOKUP, M=vocab_size, N=embed_dim, width=width))
    def generate_gemm(self, M, N, K, width=VectorWidth.V8): return self._gen(KernelSpec(KernelType.GEMM, M=M, N=N, K=K, width=width))
    def generate_quantize_dequantize(self, n, bits=8, group=32):
        return self._gen(KernelSpec(KernelType.QUANTIZE_DEQUANTIZE, N=n, K=bits, M=group))

    def _row_kernel(self, fn: str, rows: int, dim: int, kind: str, width: int) -> str:
        w = self._width_for(dim, width)
        per_lane = (dim // w + 31) // 32
        pre, post, extra_args, extra_call = "", "", "", ""
        if kind == "rms":
            extra_args, extra_call = ", const __nv_bfloat16* W, float eps", ", W, eps"
            reduce = "float ss = 0.f;\n" + self._lane_loop(per_lane, w, dim, "ss += v * v;") + f"    ss = gen_warp_sum(ss);\n    const float r = rsqrtf(ss / {dim}.f + eps);\n"
            out = "v * r * __bfloat162float(W[c + j])"
        elif kind == "ln":
            extra_args, extra_call = ", const __nv_bfloat16* W, const __nv_bfloat16* Bv, float eps", ", W, Bv, eps"
            reduce = "float s = 0.f, ss = 0.f;\n" + self._lane_loop(per_lane, w, dim, "s += v; ss += v * v;") + \
                f"    s = gen_warp_sum(s) / {dim}.f; ss = gen_warp_sum(ss) / {dim}.f;\n    const float r = rsqrtf(ss - s * s + eps);\n"
            out = "(v - s) * r * __bfloat162float(W[c + j]) + __bfloat162float(Bv[c + j])"
        else:
            reduce = "float m = -3.0e38f;\n" + self._lane_loop(per_lane, w, dim, "m = fmaxf(m, v);") + "    m = gen_warp_max(m);\n    float s = 0.f;\n" + \
                self._lane_loop(per_lane, w, dim, "s += __expf(v - m);") + "    s = 1.f / gen_warp_sum(s);\n"
            out = "__expf(v - m) * s"
        write = self._lane_loop(per_lane, w, dim, f"y[(long long)row * {dim} + c + j] = __float2bfloat16({out});")
        return (f"__global__ void __launch_bounds__(256) {fn}_k(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int rows{extra_args}) {{\n"
                f"  const int lane = threadIdx.x & 31;\n  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;\n  if (row >= rows) return;\n"
                f"  const __nv_bfloat16* xr = x + (long long)row * {dim};\n    {reduce}{write}}}\n"
                f"GEN_API int {fn}(const __nv_bfloat16* x, __nv_bfloat16* y, int rows{extra_args}, void* stream) {{\n"
                f"  {fn}_k<<<(rows * 32 + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y, rows{extra_call});\n  return int(cudaGetLastError());\n}}\n")

    @staticmethod
    def _lane_loop(per_lane: int, w: int, dim: int, stmt: str) -> str:
        return (f"#pragma unroll\n    for (int i = 0; i < {per_lane}; ++i) {{\n      const int c = (i * 32 + lane) * {w};\n      if (c < {dim}) {{\n#pragma unroll\n"
                f"        for (int j = 0; j < {w}; ++j) {{ const float v = __bfloat162float(xr[c + j]); {stmt} }}\n      }}\n    }}\n")

    def _gemm(self, fn: str, M: int, N: int, K: int) -> str:
        return (f"// C[{M},{N}] = A[{M},{K}] * B[{N},{K}]^T, 32 x 32 tiles through shared memory, fp32 accumulation\n"
                f"__global__ void __launch_bounds__(1024) {fn}_k(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ B, __nv_bfloat16* __restrict__ C) {{\n"
                f"  __shared__ float sa[32][33], sb[32][33];\n  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;\n"
                f"  const int m = blockIdx.y * 32 + ty, n0 = blockIdx.x * 32;\n  float acc = 0.f;\n"
                f"  for (int k0 = 0; k0 < {K}; k0 += 32) {{\n"
                f"    sa[ty][tx] = (m < {M} && k0 + tx < {K}) ? __bfloat162float(A[(long long)m * {K} + k0 + tx]) : 0.f;\n"
                f"    sb[ty][tx] = (n0 + ty < {N} && k0 + tx < {K}) ? __bfloat162float(B[(long long)(n0 + ty) * {K} + k0 + tx]) : 0.f;\n"
                f"    __syncthreads();\n#pragma unroll\n    for (int k = 0; k < 32; ++k) acc += sa[ty][k] * sb[tx][k];\n    __syncthreads();\n  }}\n"
                f"  if (m < {M} && n0 + tx < {N}) C[(long long)m * {N} + n0 + tx] = __float2bfloat16(acc);\n}}\n"
                f"GEN_API int {fn}(const __nv_bfloat16* A, const __nv_bfloat16* B, __nv_bfloat16* C, void* stream) {{\n"
                f"  {fn}_k<<<dim3({(N + 31) // 32}, {(M + 31) // 32}), 1024, 0, static_cast<cudaStream_t>(stream)>>>(A, B, C);\n  return int(cudaGetLastError());\n}}\n")

    def _embedding(self, fn: str, V: int, H: int, width: int) -> str:
        w = self._width_for(H, width)
        return (f"__global__ void __launch_bounds__(256) {fn}_k(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ W, __nv_bfloat16* __restrict__ out, int T) {{\n"
                f"  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;\n  if (i >= (long long)T * {H // w}) return;\n"
                f"  const int t = int(i / {H // w}), c = int(i % {H // w}) * {w};\n  long long id = ids[t];\n  if (id < 0 || id >= {V}) id = 0;\n"
                f"  *reinterpret_cast<{self._vec_ty(w)}*>(out + (long long)t * {H} + c) = *reinterpret_cast<const {self._vec_ty(w)}*>(W + id * {H} + c);\n}}\n"
                f"GEN_API int {fn}(const long long* ids, const __nv_bfloat16* W, __nv_bfloat16* out, int T, void* stream) {{\n"
                f"  const long long n = (long long)T * {H // w};\n  {fn}_k<<<int((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(ids, W, out, T);\n  return int(cudaGetLastError());\n}}\n")

    def _qdq(self, fn: str, n: int, bits: int, group: int) -> str:
        qmax = (1 << (bits - 1)) - 1
        return (f"// symmetric {bits}-bit fake quantisation with one scale per {group} consecutive values (one warp lane group each)\n"
                f"__global__ void __launch_bounds__(256) {fn}_k(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y) {{\n"
                f"  const long long g = blockIdx.x * (long long)blockDim.x + threadIdx.x;\n  if (g >= {n // group}LL) return;\n  float amax = 0.f;\n"
                f"#pragma unroll 8\n  for (int j = 0; j < {group}; ++j) amax = fmaxf(amax, fabsf(__bfloat162float(x[g * {group} + j])));\n"
                f"  const float s = amax > 0.f ? amax / {qmax}.f : 1.f;\n"
                f"#pragma unroll 8\n  for (int j = 0; j < {group}; ++j) y[g * {group} + j] = __float2bfloat16(fminf(fmaxf(rintf(__bfloat162float(x[g * {group} + j]) / s), -{qmax}.f), {qmax}.f) * s);\n}}\n"
                f"GEN_API int {fn}(const __nv_bfloat16* x, __nv_bfloat16* y, void* stream) {{\n"
                f"  {fn}_k<<<{(n // group + 255) // 256}, 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y);\n  return int(cudaGetLastError());\n}}\n")

    def _attention(self, fn: str, S: int, D: int, H: int) -> str:
        """Causal self-attention for one fixed (sequence, head size, heads): a warp per (head, query), the head dimension
        spread over the lanes, keys visited in order with the running-maximum softmax so nothing of size S is stored."""
        if D % 32 or D > 256:
            raise ValueError("generated attention needs a head size that is a multiple of 32, at most 256")
        per = D // 32
        scale = repr(float(D) ** -0.5) + "f"
        ld = H * D
        return (f"// q, k, v, o: [{S}, {H} * {D}] bf16 rows (token-major); causal; softmax scale 1 / sqrt({D})\n"
                f"__global__ void __launch_bounds__(256) {fn}_k(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ o) {{\n"
                f"  const int lane = threadIdx.x & 31;\n  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;\n  if (w >= {S * H}) return;\n"
                f"  const int h = w % {H}, i = w / {H};\n  float qr[{per}], acc[{per}];\n"
                f"#pragma unroll\n  for (int c = 0; c < {per}; ++c) {{ qr[c] = __bfloat162float(q[(long long)i * {ld} + h * {D} + c * 32 + lane]) * {scale}; acc[c] = 0.f; }}\n"
                f"  float m = -3.0e38f, l = 0.f;\n  for (int j = 0; j <= i; ++j) {{\n    float s = 0.f;\n"
                f"#pragma unroll\n    for (int c = 0; c < {per}; ++c) s += qr[c] * __bfloat162float(k[(long long)j * {ld} + h * {D} + c * 32 + lane]);\n"
                f"    s = gen_warp_sum(s);\n    const float mn = fmaxf(m, s), corr = __expf(m - mn), p = __expf(s - mn);\n    l = l * corr + p;\n"
                f"#pragma unroll\n    for (int c = 0; c < {per}; ++c) acc[c] = acc[c] * corr + p * __bfloat162float(v[(long long)j * {ld} + h * {D} + c * 32 + lane]);\n"
                f"    m = mn;\n  }}\n  const float inv = 1.f / l;\n"
                f"#pragma unroll\n  for (int c = 0; c < {per}; ++c) o[(long long)i * {ld} + h * {D} + c * 32 + lane] = __float2bfloat16(acc[c] * inv);\n}}\n"
                f"GEN_API int {fn}(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v, __nv_bfloat16* o, void* stream) {{\n"
                f"  {fn}_k<<<{(S * H * 32 + 255) // 256}, 256, 0, static_cast<cudaStream_t>(stream)>>>(q, k, v, o);\n  return int(cudaGetLastError());\n}}\n")

    def generate_attention(self, seq_len: int, head_dim: int, num_heads: int, width=VectorWidth.SCALAR) -> str:
        """Source of a causal attention kernel for exactly this shape (small and odd shapes; the framework's own flash
        attention kernels serve the model shapes).  Reference counterpart: CodeGenerator::generate_attention
        (include/quant/code_gen.h:104)."""
        return self._gen(KernelSpec(KernelType.ATTENTION, M=seq_len, N=head_dim, K=num_heads, width=width))

    # ---- dispatch over weight formats (reference: generate_format_dispatch / generate_format_branch, code_gen.h:120-121)
    @staticmethod
    def _fmt_name(fmt) -> str:
        if isinstance(fmt, str):
            return fmt
        from ..quant import codec
        return codec.format_name(int(fmt)) if hasattr(codec, "format_name") else f"fmt{int(fmt)}"

    def generate_format_dispatch(self, op_name: str, formats) -> str:
        """A host function ``<op>_dispatch(format, x, w, y, n, stream)`` that switches on the format id and calls
        ``<op>_<FORMAT>`` for each of the given formats (-1 for any other id)."""
        from ..quant import codec
        cases = ""
        for f in formats:
            fid = codec.parse_format(f) if isinstance(f, str) else int(f)
            cases += f"    case {fid}: return {op_name}_{self._fmt_name(f)}(x, w, y, n, stream);\n"
        return (f"GEN_API int {op_name}_dispatch(int format, const void* x, const void* w, void* y, long long n, void* stream) {{\n"
                f"  switch (format) {{\n{cases}    default: return -1;\n  }}\n}}\n")

    def generate_format_branch(self, op_name: str, fmt, dim: int) -> str:
        """One branch of such a dispatch for plain absmax integer grids (``Q_2`` .. ``Q_8``): a kernel that expands ``dim``
        stored integers (one int8 each) with a per-32 scale and applies nothing else; ``<op>_<FORMAT>`` is its launcher."""
        name = self._fmt_name(fmt)
        return (f"__global__ void __launch_bounds__(256) {op_name}_{name}_k(const int8_t* __restrict__ w, const float* __restrict__ scale, __nv_bfloat16* __restrict__ y) {{\n"
                f"  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;\n  if (i >= {dim}LL) return;\n"
                f"  y[i] = __float2bfloat16(float(w[i]) * scale[i >> 5]);\n}}\n"
                f"GEN_API int {op_name}_{name}(const void* x, const void* w, void* y, long long n, void* stream) {{\n"
                f"  (void)n;\n  {op_name}_{name}_k<<<{(dim + 255) // 256}, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const int8_t*>(w), static_cast<const float*>(x), static_cast<__nv_bfloat16*>(y));\n"
                f"  return int(cudaGetLastError());\n}}\n")

    # ---- vector statement emitters (the reference's SIMD emitters, code_gen.h:125-129, for CUDA vector types: a "vector" is
    # an array of ``width`` floats in registers, loaded and stored through one wide bf16 access)
    def generate_simd_load(self, var: str, ptr: str, width: int) -> str:
        return (f"float {var}[{width}]; {{ __align__(16) __nv_bfloat16 t_[{width}]; *reinterpret_cast<{self._vec_ty(width)}*>(t_) = "
                f"*reinterpret_cast<const {self._vec_ty(width)}*>({ptr});\n#pragma unroll\n for (int j_ = 0; j_ < {width}; ++j_) {var}[j_] = __bfloat162float(t_[j_]); }}")

    def generate_simd_store(self, ptr: str, var: str, width: int) -> str:
        return (f"{{ __align__(16) __nv_bfloat16 t_[{width}];\n#pragma unroll\n for (int j_ = 0; j_ < {width}; ++j_) t_[j_] = __float2bfloat16({var}[j_]); "
                f"*reinterpret_cast<{self._vec_ty(width)}*>({ptr}) = *reinterpret_cast<const {self._vec_ty(width)}*>(t_); }}")

    def generate_simd_fma(self, dst: str, a: str, b: str, c: str, width: int = 8) -> str:
        return f"#pragma unroll\nfor (int j_ = 0; j_ < {width}; ++j_) {dst}[j_] = fmaf({a}[j_], {b}[j_], {c}[j_]);"

    def generate_simd_add(self, dst: str, a: str, b: str, width: int = 8) -> str:
        return f"#pragma unroll\nfor (int j_ = 0; j_ < {width}; ++j_) {dst}[j_] = {a}[j_] + {b}[j_];"

    def generate_simd_mul(self, dst: str, a: str, b: str, width: int = 8) -> str:
        return f"#pragma unroll\nfor (int j_ = 0; j_ < {width}; ++j_) {dst}[j_] = {a}[j_] * {b}[j_];"

    def generate_kernel_for_shape(self, spec: KernelSpec) -> str:
        fn, t = self.make_function_name(spec), spec.type
        if t in _UNARY:
            return self._elementwise(fn, spec.N, _UNARY[t], False, spec.width, spec.block_size)
        if t in _BINARY:
            return self._elementwise(fn, spec.N, _BINARY[t], True, spec.width, spec.block_size)
        if t == KernelType.SCALE:
            return self._elementwise(fn, spec.N, f"x * {float(spec.scale)!r}f", False, spec.width, spec.block_size)
        if t == KernelType.RMS_NORM:
            return self._row_kernel(fn, spec.M, spec.N, "rms", spec.width)
        if t == KernelType.LAYER_NORM:
            return self._row_kernel(fn, spec.M, spec.N, "ln", spec.width)
        if t == KernelType.SOFTMAX:
            return self._row_kernel(fn, spec.M, spec.N, "softmax", spec.width)
        if t in (KernelType.GEMM, KernelType.HEAD_PROJECTION):
            return self._gemm(fn, spec.M, spec.N, spec.K)
        if t == KernelType.EMBEDDING_LOOKUP:
            return self._embedding(fn, spec.M, spec.N, spec.width)
        if t == KernelType.QUANTIZE_DEQUANTIZE:
            return self._qdq(fn, spec.N, spec.K or 8, spec.M or 32)
        if t == KernelType.ATTENTION:
            return self._attention(fn, spec.M, spec.N, spec.K)
        raise ValueError(f"{t.name} kernels are hand-written in this framework and are not generated")

    def _gen(self, spec: KernelSpec) -> str:
        return self.generate_kernel_for_shape(spec)

    def generate_full_source(self, kernels: List[GeneratedKernel]) -> str:
        return _HEADER + "\n".join(k.source_code for k in kernels)

    def save_source(self, path: str, source: str) -> bool:
        with open(path, "w") as f:
            f.write(source)
        return True

    # ------------------------------------------------------------------ validation / compilation
    @staticmethod
    def _nvcc() -> Optional[str]:
        for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
            if c and os.path.exists(c):
                return c
        return None

    @staticmethod
    def syntax_ok(code: str) -> bool:
        depth = 0
        for ch in code:
            depth += ch == "{"
            depth -= ch == "}"
            if depth < 0:
                return False
        return depth == 0 and code.count("(") == code.count(")")

    def compile_code(self, code: str, shared: bool = True) -> str:
        """Compiles a full translation unit for sm_100a; returns the path of the shared object ('' on failure, with the
        compiler's message in ``last_error``)."""
        nvcc = self._nvcc()
        self.last_error = ""
        if nvcc is None:
            self.last_error = "nvcc not found"
            return ""
        h = hashlib.sha1(code.encode()).hexdigest()[:16]
        src, so = os.path.join(self.work_dir, f"gen_{h}.cu"), os.path.join(self.work_dir, f"gen_{h}.so")
        if not os.path.exists(so):
            self.save_source(src, code)
            r = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "--use_fast_math", "-shared",
                                "-Xcompiler", "-fPIC", "-o", so, src], capture_output=True, text=True)
            if r.returncode != 0:
                self.last_error = (r.stdout + r.stderr)[-2000:]
                return ""
        return so

    def validate(self, code: str) -> CodeValidationResult:
        res = CodeValidationResult(syntax_valid=self.syntax_ok(code))
        if not res.syntax_valid:
            res.error_message = "unbalanced braces or parentheses"
            return res
        full = code if code.lstrip().startswith("#include") else _HEADER + code
        res.compiles = bool(self.compile_code(full))
        res.error_message = getattr(self, "last_error", "")
        return res

    def generate_optimized_kernel(self, spec: KernelSpec) -> GeneratedKernel:
        fn = self.make_function_name(spec)
        k = GeneratedKernel(spec, self.generate_kernel_for_shape(spec), fn)
        k.validated = self.syntax_ok(k.source_code)
        k.so_path = self.compile_code(_HEADER + k.source_code) if k.validated else ""
        k.compiled = bool(k.so_path)
        k.error_message = getattr(self, "last_error", "")
        self.kernels[fn] = k
        return k

    def specialize_for_shape(self, type: KernelType, M: int, N: int, K: int) -> GeneratedKernel:
        return self.generate_optimized_kernel(KernelSpec(type, M, N, K))

    def run_test(self, kernel: GeneratedKernel) -> CodeValidationResult:
        """Loads the kernel and compares it with PyTorch on random data.  Needs a GPU; without one only the compile
        status is reported."""
        import torch
        res = CodeValidationResult(syntax_valid=kernel.validated, compiles=kernel.compiled)
        if not kernel.compiled or not torch.cuda.is_available():
            return res
        lib, s, t = ctypes.CDLL(kernel.so_path), kernel.spec, kernel.spec.type
        fn = getattr(lib, kernel.function_name)
        st = torch.cuda.current_stream().cuda_stream
        if t in _UNARY or t in _BINARY or t == KernelType.SCALE:
            a, b = torch.randn(s.N, device="cuda").bfloat16(), torch.randn(s.N, device="cuda").bfloat16()
            o = torch.empty_like(a)
            x, y = a.float(), b.float()
            ref = {KernelType.RELU: x.relu(), KernelType.SILU: torch.nn.functional.silu(x), KernelType.GELU: torch.nn.functional.gelu(x, approximate="tanh"),
                   KernelType.ADD: x + y, KernelType.MUL: x * y, KernelType.RESIDUAL_ADD: x + y, KernelType.SCALE: x * s.scale}[t]
            args = [ctypes.c_void_p(a.data_ptr())] + ([ctypes.c_void_p(b.data_ptr())] if t in _BINARY else []) + [ctypes.c_void_p(o.data_ptr()), ctypes.c_void_p(st)]
            rc = fn(*args)
        elif t == KernelType.ATTENTION:
            S, D, H = s.M, s.N, s.K
            q, k, v = (torch.randn(S, H * D, device="cuda").bfloat16() for _ in range(3))
            o = torch.empty_like(q)
            hm = lambda z: z.float().view(S, H, D).transpose(0, 1)
            ref = torch.nn.functional.scaled_dot_product_attention(hm(q), hm(k), hm(v), is_causal=True).transpose(0, 1).reshape(S, H * D)
            rc = fn(*(ctypes.c_void_p(z.data_ptr()) for z in (q, k, v, o)), ctypes.c_void_p(st))
        else:
            return res
        torch.cuda.synchronize()
        res.runs = rc == 0
        res.max_error = float((o.float() - ref).abs().max())
        res.correctness_pass = res.runs and res.max_error <= 0.02 * float(ref.abs().max()) + 1e-3
        return res

    # ------------------------------------------------------------------ slow paths / search
    def identify_slow_paths(self, timings_ms: Optional[Dict[str, float]] = None, roofline_ms: Optional[Dict[str, float]] = None,
                            threshold_ms: float = 1.0) -> List[SlowPath]:
        """Ops whose measured time exceeds ``threshold_ms`` and their bandwidth-roofline target, slowest first."""
        timings_ms, roofline_ms = timings_ms or {}, roofline_ms or {}
        out = [SlowPath(op, t, roofline_ms.get(op, t * 0.5), "", 0) for op, t in timings_ms.items() if t > threshold_ms]
        out.sort(key=lambda p: p.current_time_ms - p.target_time_ms, reverse=True)
        for i, p in enumerate(out):
            p.priority = len(out) - i
        self.slow_paths = out
        return out

    def improve_slow_path(self, path: SlowPath, n: int = 1 << 20) -> str:
        name = path.op_name.upper()
        t = KernelType[name] if name in KernelType.__members__ else KernelType.ADD
        return self.generate_kernel_for_shape(KernelSpec(t, N=n, M=1, width=VectorWidth.V8, unroll=UnrollLevel.FULL))

    def auto_optimize(self, type: KernelType = KernelType.SILU, n: int = 1 << 20, n_iterations: int = 4) -> List[GeneratedKernel]:
        """Generates the vector-width / block-size variants of one kernel, keeps those that compile, and (with a GPU) times
        them; the list comes back fastest first."""
        import torch
        cands = [(w, b) for w in (VectorWidth.V8, VectorWidth.V4, VectorWidth.V2) for b in (256, 128)][:n_iterations]
        out = []
        for w, b in cands:
            k = self.generate_optimized_kernel(KernelSpec(type, N=n, width=w, block_size=b, name=f"gen_{type.name.lower()}_{n}_v{int(w)}_b{b}"))
            if k.compiled and torch.cuda.is_available():
                r = self.run_test(k)
                if r.correctness_pass:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(5):
                        self.run_test(k)
                    e1.record()
                    torch.cuda.synchronize()
                    k.benchmark_ms = e0.elapsed_time(e1) / 5
            if k.compiled:
                out.append(k)
        out.sort(key=lambda k: k.benchmark_ms)
        return out

    # ------------------------------------------------------------------ templates
    def _init_default_templates(self):
        self.register_template(CodeTemplate("elementwise", "out[i] = f(in[i]) over N bf16 values",
                                            "__global__ void {{NAME}}(const __nv_bfloat16* x, __nv_bfloat16* y) {\n  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;\n"
                                            "  if (i < {{N}}LL) { const float v = __bfloat162float(x[i]); y[i] = __float2bfloat16({{EXPR}}); }\n}\n",
                                            ["NAME", "N", "EXPR"], KernelType.RELU))

    def register_template(self, t: CodeTemplate): self.templates[t.name] = t

    def apply_template(self, name: str, vars: Dict[str, str]) -> str:
        t = self.templates[name]
        missing = [p for p in t.placeholders if p not in vars]
        if missing:
            raise KeyError(f"template '{name}' needs {missing}")
        code = t.template_code
        for k, v in vars.items():
            code = code.replace("{{" + k + "}}", str(v))
        return code

    def get_available_templates(self) -> List[str]: return sorted(self.templates)
    def get_kernel(self, name: str) -> GeneratedKernel: return self.kernels[name]
    def get_all_kernels(self) -> List[GeneratedKernel]: return list(self.kernels.values())
    def clear_kernels(self): self.kernels.clear()
