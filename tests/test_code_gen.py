"""Kernel source generator: every generated kind compiles for sm_100a, names and vector widths follow the shape, broken
source is rejected with the compiler's message, templates substitute, slow paths are ranked."""
import pytest

from transformers_fusion_b200.trainer.code_gen import (CodeGenerator, CodeTemplate, KernelSpec, KernelType, SlowPath, VectorWidth)


def test_generated_kernels_compile(tmp_path):
    g = CodeGenerator(work_dir=str(tmp_path))
    if g._nvcc() is None:
        pytest.skip("nvcc not available")
    specs = [KernelSpec(KernelType.SILU, N=1 << 20), KernelSpec(KernelType.ADD, N=1004), KernelSpec(KernelType.SCALE, N=4096, scale=0.5),
             KernelSpec(KernelType.RMS_NORM, M=64, N=512), KernelSpec(KernelType.LAYER_NORM, M=64, N=768), KernelSpec(KernelType.SOFTMAX, M=8, N=1000),
             KernelSpec(KernelType.GEMM, M=70, N=50, K=96), KernelSpec(KernelType.EMBEDDING_LOOKUP, M=1000, N=256),
             KernelSpec(KernelType.QUANTIZE_DEQUANTIZE, N=4096, K=4, M=32)]
    ks = [g.generate_optimized_kernel(s) for s in specs]
    for k in ks:
        assert k.validated and k.compiled, (k.function_name, k.error_message)
    assert "uint4" in ks[0].source_code and "uint4" not in ks[1].source_code and "uint2" in ks[1].source_code   # 1004 = 4 * 251
    assert ks[0].function_name == "gen_silu_1048576_v8" and g.get_kernel("gen_silu_1048576_v8") is ks[0]
    full = g.generate_full_source(ks)
    assert full.count("GEN_API int") == len(ks) and g.validate(full).compiles
    assert len(g.get_all_kernels()) == len(ks)
    with pytest.raises(ValueError):
        g.generate_kernel_for_shape(KernelSpec(KernelType.ATTENTION, M=128, N=48, K=2))      # head size not a multiple of 32


def test_generated_attention_dispatch_and_vector_statements_compile(tmp_path):
    g = CodeGenerator(work_dir=str(tmp_path))
    if g._nvcc() is None:
        pytest.skip("nvcc not available")
    att = g.generate_optimized_kernel(KernelSpec(KernelType.ATTENTION, M=96, N=64, K=4))
    assert att.compiled, att.error_message
    assert "float qr[2], acc[2]" in att.source_code and g.generate_attention(96, 64, 4, VectorWidth.V8) == att.source_code
    # format dispatch: one branch per format plus the switch; the whole unit compiles
    branches = "".join(g.generate_format_branch("expand", f, 4096) for f in ("Q_4", "Q_8"))
    disp = g.generate_format_dispatch("expand", ["Q_4", "Q_8"])
    from transformers_fusion_b200.quant import codec
    assert f"case {codec.parse_format('Q_4')}: return expand_Q_4(" in disp and "default: return -1;" in disp
    assert g.validate(branches + disp).compiles, g.last_error
    # vector statement emitters compose into a kernel body
    body = "\n".join([g.generate_simd_load("a", "x + i", 8), g.generate_simd_load("b", "y + i", 8), "float c[8], d[8];",
                      g.generate_simd_mul("c", "a", "b", 8), g.generate_simd_add("d", "c", "a", 8), g.generate_simd_fma("d", "a", "b", "d", 8),
                      g.generate_simd_store("z + i", "d", 8)])
    kern = ("__global__ void vec_k(const __nv_bfloat16* x, const __nv_bfloat16* y, __nv_bfloat16* z, int n) {\n"
            "  const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 8;\n  if (i >= n) return;\n" + body + "\n}\n")
    assert g.validate(kern).compiles, g.last_error


def test_validation_rejects_broken_code(tmp_path):
    g = CodeGenerator(work_dir=str(tmp_path))
    bad = g.validate("__global__ void f() { int x = ; }")
    assert bad.syntax_valid and (g._nvcc() is None or (not bad.compiles and "error" in bad.error_message))
    assert not g.validate("void f() { {").syntax_valid


def test_templates_and_slow_paths(tmp_path):
    g = CodeGenerator(work_dir=str(tmp_path))
    code = g.apply_template("elementwise", {"NAME": "sq", "N": 128, "EXPR": "v * v"})
    assert "sq(" in code and "128LL" in code and "{{" not in code
    with pytest.raises(KeyError):
        g.apply_template("elementwise", {"NAME": "x"})
    g.register_template(CodeTemplate("noop", "", "// {{A}}", ["A"], KernelType.ADD))
    assert g.get_available_templates() == ["elementwise", "noop"]
    sp = g.identify_slow_paths({"silu": 3.0, "add": 0.2, "softmax": 5.0}, {"silu": 2.5, "softmax": 1.0})
    assert [p.op_name for p in sp] == ["softmax", "silu"] and sp[0].priority == 2
    assert "gen_silu" in g.improve_slow_path(sp[1])
    assert "#pragma unroll 4" in g.generate_unrolled_loop("i", 0, 16, 4, "x += i;")
    assert g._width_for(1000, 8) == 8 and g._width_for(1004, 8) == 4 and g._width_for(7, 8) == 1
