// Text of the host calls that the B200 dispatchers write into docc's generated C++.
//
// Dependency-free on purpose: the dispatcher classes in b200_plugin.cpp (which need docc's headers)
// only collect node parameters as already-printed expressions and hand them to these functions, so
// the emitted text can be compiled and golden-tested without a docc build. `Stream` is anything with
// operator<< for strings (docc's codegen::PrettyPrinter, std::ostream).
//
// The connector locals used below (__A, __B, __C, __alpha, __beta / X, W, B, Y / A, B, Y) are the ones
// LibraryNodeDispatcher::dispatch has already declared when dispatch_code runs
// (sdfg/src/codegen/dispatchers/block_dispatcher.cpp:341-407).
#pragma once

#include <cstdlib>
#include <cstring>
#include <sstream>
#include <string>
#include <vector>

namespace docc_b200_plugin {

// Same switch and values as docc's CUDA error-check emitter: read at code-generation time
// (opt/src/targets/cuda/cuda.cpp:62-91).
inline bool debug_checks_enabled() {
    const char* v = std::getenv("DOCC_CUDA_DEBUG");
    return v && (std::strcmp(v, "1") == 0 || std::strcmp(v, "true") == 0);
}

template <class Stream> void emit_include(Stream& globals) { globals << "#include <docc_b200/rt.h>\n"; }

// Unchecked by default (as docc); with checks: print and exit like check_cuda_kernel_launch_errors.
template <class Stream> void emit_call(Stream& s, const std::string& name, const std::string& args, bool checked) {
    if (!checked) {
        s << name << "(" << args << ");\n";
        return;
    }
    s << "{\n";
    s << "    int __docc_b200_st = " << name << "(" << args << ");\n";
    s << "    if (__docc_b200_st != 0) {\n";
    s << "        fprintf(stderr, \"" << name << ": %s (%s)\\n\", docc_b200_strerror(__docc_b200_st), docc_b200_last_error());\n";
    s << "        exit(EXIT_FAILURE);\n";
    s << "    }\n";
    s << "}\n";
}

inline std::string join(const std::vector<std::string>& v) {
    std::string out;
    for (size_t i = 0; i < v.size(); i++) out += (i ? ", " : "") + v[i];
    return out;
}
inline std::string i64_array(const std::vector<std::string>& v) {
    return "(const int64_t[]){" + (v.empty() ? std::string("0") : join(v)) + "}";
}

// GEMMNode -> docc_b200_gemm. precision is BLAS_Precision's char, layout / trans are the enum values
// (blas_node.h:49-126), dimensions are printed symbolic expressions.
template <class Stream>
void emit_gemm(Stream& s, char precision, int layout, int trans_a, int trans_b, const std::string& m, const std::string& n,
               const std::string& k, const std::string& lda, const std::string& ldb, const std::string& ldc, bool with_transfers,
               bool checked) {
    std::ostringstream a;
    a << "'" << precision << "', " << layout << ", " << trans_a << ", " << trans_b << ", " << m << ", " << n << ", " << k
      << ", &__alpha, __A, " << lda << ", __B, " << ldb << ", &__beta, __C, " << ldc << ", " << (with_transfers ? 1 : 0);
    emit_call(s, "docc_b200_gemm", a.str(), checked);
}

// MatMulNode -> docc_b200_matmul (connectors A, B -> Y; batch strides are the products MatMulNode::expand
// derives from the shapes, matmul_node.cpp:353-489; 0 broadcasts an operand).
template <class Stream>
void emit_matmul(Stream& s, char precision, const std::string& batch, const std::string& m, const std::string& n,
                 const std::string& k, const std::string& lda, const std::string& stride_a, const std::string& ldb,
                 const std::string& stride_b, bool with_transfers, bool checked) {
    std::ostringstream a;
    a << "'" << precision << "', " << batch << ", " << m << ", " << n << ", " << k << ", A, " << lda << ", " << stride_a << ", B, "
      << ldb << ", " << stride_b << ", Y, " << n << ", (" << m << ") * (" << n << "), " << (with_transfers ? 1 : 0);
    emit_call(s, "docc_b200_matmul", a.str(), checked);
}

// SoftmaxNode / ReduceNode -> docc_b200_softmax / docc_b200_reduce (connectors X -> Y).
template <class Stream>
void emit_softmax(Stream& s, char precision, const std::vector<std::string>& shape, const std::vector<std::string>& axes,
                  bool with_transfers, bool checked) {
    std::ostringstream a;
    a << "'" << precision << "', " << shape.size() << ", " << i64_array(shape) << ", " << axes.size() << ", " << i64_array(axes)
      << ", X, Y, " << (with_transfers ? 1 : 0);
    emit_call(s, "docc_b200_softmax", a.str(), checked);
}
template <class Stream>
void emit_reduce(Stream& s, int op, char precision, const std::vector<std::string>& shape, const std::vector<std::string>& axes,
                 bool with_transfers, bool checked) {
    std::ostringstream a;
    a << op << ", '" << precision << "', " << shape.size() << ", " << i64_array(shape) << ", " << axes.size() << ", "
      << i64_array(axes) << ", X, Y, " << (with_transfers ? 1 : 0);
    emit_call(s, "docc_b200_reduce", a.str(), checked);
}

// ConvNode -> docc_b200_conv (connectors X, W, [B] -> Y). x_shape = [N, C_in, D0..]; pads = begins then ends.
template <class Stream>
void emit_conv(Stream& s, char precision, const std::vector<std::string>& x_shape, const std::vector<std::string>& kernel_shape,
               const std::vector<std::string>& strides, const std::vector<std::string>& pads,
               const std::vector<std::string>& dilations, const std::string& c_out, const std::string& group, bool has_bias,
               bool with_transfers, bool checked) {
    std::ostringstream a;
    a << "'" << precision << "', '" << precision << "', " << kernel_shape.size() << ", " << i64_array(x_shape) << ", "
      << i64_array(kernel_shape) << ", " << i64_array(strides) << ", " << i64_array(pads) << ", " << i64_array(dilations) << ", "
      << c_out << ", " << group << ", X, W, " << (has_bias ? "B" : "NULL") << ", Y, " << (with_transfers ? 1 : 0);
    emit_call(s, "docc_b200_conv", a.str(), checked);
}

// CUDADataOffloadingNode lifecycle -> pool / transfer calls (cuda_data_offloading_node.cpp:149-172).
template <class Stream> void emit_alloc(Stream& s, const std::string& dev_ptr, const std::string& bytes, bool checked) {
    emit_call(s, "docc_b200_malloc", "(void**)&" + dev_ptr + ", " + bytes, checked);
}
template <class Stream>
void emit_h2d(Stream& s, const std::string& dev_ptr, const std::string& host_ptr, const std::string& bytes, bool checked) {
    emit_call(s, "docc_b200_h2d", dev_ptr + ", " + host_ptr + ", " + bytes, checked);
}
template <class Stream>
void emit_d2h(Stream& s, const std::string& host_ptr, const std::string& dev_ptr, const std::string& bytes, bool checked) {
    emit_call(s, "docc_b200_d2h", host_ptr + ", " + dev_ptr + ", " + bytes, checked);
}
template <class Stream> void emit_free(Stream& s, const std::string& dev_ptr, bool checked) {
    emit_call(s, "docc_b200_free", dev_ptr, checked);
}

}  // namespace docc_b200_plugin
