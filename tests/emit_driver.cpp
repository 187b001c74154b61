// Prints the host calls the B200 dispatchers emit for a fixed set of nodes (golden-text test driver).
#include <iostream>

#include "b200_emit.h"

using namespace docc_b200_plugin;

// A translation unit in the shape docc's CPPCodeGenerator produces (extern "C" entry, arrays and _s<i> shape symbols as
// arguments, one scope per library node in which LibraryNodeDispatcher::dispatch has declared the connector locals),
// with the node calls written by the same emitters the dispatchers use.
static void print_program(bool checked) {
    auto& o = std::cout;
    emit_include(o);
    o << "#include <math.h>\n#include <stdint.h>\n#include <stdio.h>\n#include <stdlib.h>\n";
    // BASELINE config 1 as add_gemm builds it, and config 2
    o << "extern \"C\" void matmul_op(double* a, double* b, double* _docc_ret_0, int64_t _s0, int64_t _s1, int64_t _s2) {\n{\n";
    o << "double* __A = a; double* __B = b; double* __C = _docc_ret_0; double __alpha = 1.0; double __beta = 0.0;\n";
    emit_gemm(o, 'd', 101, 111, 111, "_s0", "_s2", "_s1", "_s1", "_s2", "_s2", true, checked);
    o << "}\n}\n";
    o << "extern \"C\" void softmax_op(float* x, float* _docc_ret_0, int64_t _s0, int64_t _s1) {\n{\n";
    o << "float* X = x; float* Y = _docc_ret_0;\n";
    emit_softmax(o, 's', {"_s0", "_s1"}, {"1"}, true, checked);
    o << "}\n}\n";
    o << "extern \"C\" void conv_op(float* x, float* w, float* b, float* _docc_ret_0, int64_t _s0) {\n{\n";
    o << "float* X = x; float* W = w; float* B = b; float* Y = _docc_ret_0;\n";
    emit_conv(o, 's', {"_s0", "8", "12", "12"}, {"3", "3"}, {"1", "1"}, {"1", "1", "1", "1"}, {"1", "1"}, "16", "1", true, true, checked);
    o << "}\n}\n";
    o << "extern \"C\" void attn_op(float* q, float* k, float* v, float* _docc_ret_0, int64_t _s0, int64_t _s1, int64_t _s2, int64_t _s3) {\n{\n";
    o << "float* Q = q; float* K = k; float* V = v; float* O = _docc_ret_0;\n";
    emit_attention(o, 's', "_s0", "_s1", "_s2", "_s3", "32", 0.0, true, true, checked);
    o << "}\n}\n";
    o << "extern \"C\" void ln_erf_div_op(float* x, float* g, float* b, float* _docc_ret_0, int64_t _s0, int64_t _s1) {\n";
    o << "float* _tmp0 = (float*)malloc(sizeof(float) * _s0 * _s1); float* _tmp1 = (float*)malloc(sizeof(float) * _s0 * _s1);\n";
    o << "{\nfloat* X = x; float* G = g; float* B = b; float* Y = _tmp0;\n";
    emit_layernorm(o, 's', "_s0", "_s1", 1e-5, true, true, checked);
    o << "}\n{\nfloat* X = _tmp0; float* Y = _tmp1;\n";
    emit_unary(o, 's', 6, "(_s0) * (_s1)", true, checked);
    o << "}\n{\nfloat* A = _tmp1; float* B = x; float* C = _docc_ret_0;\n";
    emit_binary(o, 3, 's', "(_s0) * (_s1)", true, checked);
    o << "}\nfree(_tmp0); free(_tmp1);\n}\n";
    // an offloaded region: alloc + copy-in, device-resident nodes (no transfers), copy-out + free
    o << "extern \"C\" void offload_op(float* a, double* _docc_ret_0, double* _docc_ret_1, int64_t _s0, int64_t _s1) {\n";
    o << "float* __daisy_dev_a; double* __daisy_dev_c; double* __daisy_dev_m;\n{\n";
    emit_offload(o, true, true, false, false, "__daisy_dev_a", "a", "4 * _s0 * _s1", checked);
    o << "}\n{\n";
    emit_offload(o, true, false, false, false, "__daisy_dev_c", "", "8 * _s0 * _s1", checked);
    o << "}\n{\n";
    emit_offload(o, true, false, false, false, "__daisy_dev_m", "", "8 * _s0", checked);
    o << "}\n{\nfloat* X = __daisy_dev_a; double* Y = __daisy_dev_c;\n";
    emit_cast(o, 's', 'd', "(_s0) * (_s1)", false, checked);
    o << "}\n{\ndouble* X = __daisy_dev_c; double* Y = __daisy_dev_m;\n";
    emit_reduce(o, 3, 'd', {"_s0", "_s1"}, {"1"}, false, checked);
    o << "}\n{\n";
    emit_offload(o, false, false, true, true, "_docc_ret_0", "__daisy_dev_c", "8 * _s0 * _s1", checked);
    o << "}\n{\n";
    emit_offload(o, false, false, true, true, "_docc_ret_1", "__daisy_dev_m", "8 * _s0", checked);
    o << "}\n{\n";
    emit_offload(o, false, false, false, true, "", "__daisy_dev_a", "0", checked);
    o << "}\n}\n";
}

int main(int argc, char** argv) {
    const bool checked = argc > 1 && std::string(argv[1]) == "checked";
    if (argc > 1 && std::string(argv[1]) == "program") {
        print_program(argc > 2 && std::string(argv[2]) == "checked");
        return 0;
    }
    emit_include(std::cout);
    // GEMM fp64 row-major NN, symbolic m/n/k (BASELINE config 1 as add_gemm builds it)
    emit_gemm(std::cout, 'd', 101, 111, 111, "_s0", "_s2", "_s1", "_s1", "_s2", "_s2", true, checked);
    emit_gemm(std::cout, 's', 102, 112, 111, "m", "n", "k", "lda", "ldb", "ldc", false, checked);
    emit_matmul(std::cout, 'd', "2", "10", "10", "10", "10", "(10) * (10)", "10", "(10) * (10)", true, checked);
    emit_softmax(std::cout, 's', {"8192", "4096"}, {"1"}, true, checked);
    emit_reduce(std::cout, 3, 'd', {"_s0", "_s1", "_s2"}, {"0", "2"}, true, checked);
    emit_conv(std::cout, 's', {"32", "64", "56", "56"}, {"3", "3"}, {"1", "1"}, {"1", "1", "1", "1"}, {"1", "1"}, "128", "1", true,
              true, checked);
    emit_conv(std::cout, 'd', {"N", "C", "L"}, {"K"}, {"2"}, {"0", "0"}, {"1"}, "CO", "1", false, false, checked);
    // encoder-block attention (config 5: 16 heads of 64) with the default scale, and a causal one with an explicit scale
    emit_attention(std::cout, 'b', "32", "16", "512", "512", "64", 0.0, false, false, checked);
    emit_attention(std::cout, 's', "_s0", "_s1", "_s2", "_s3", "128", 0.125, true, true, checked);
    emit_layernorm(std::cout, 's', "(32) * (512)", "1024", 1e-5, true, false, checked);
    emit_layernorm(std::cout, 'b', "_s0", "_s1", 1e-6, false, true, checked);
    emit_unary(std::cout, 's', 6, "(_s0) * (_s1)", true, checked);    // ml::Erf
    emit_binary(std::cout, 3, 'd', "1000", true, checked);             // ml::Div
    emit_cast(std::cout, 's', 'b', "4096", false, checked);            // ml::Cast fp32 -> bf16
    // one CUDADataOffloadingNode each: alloc + copy-in, copy-out + free, alloc only, free only
    emit_offload(std::cout, true, true, false, false, "__daisy_dev_A", "A", "8 * m * k", checked);
    emit_offload(std::cout, false, false, true, true, "C", "__daisy_dev_C", "8 * m * n", checked);
    emit_offload(std::cout, true, false, false, false, "__daisy_dev_T", "", "4 * n", checked);
    emit_offload(std::cout, false, false, false, true, "__daisy_dev_T", "__daisy_dev_T", "4 * n", checked);
    emit_alloc(std::cout, "__daisy_dev_A", "8 * m * k", checked);
    emit_h2d(std::cout, "__daisy_dev_A", "A", "8 * m * k", checked);
    emit_d2h(std::cout, "C", "__daisy_dev_C", "8 * m * n", checked);
    emit_free(std::cout, "__daisy_dev_A", checked);
    return 0;
}
