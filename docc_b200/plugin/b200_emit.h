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
// `locals` (optional) are declarations the arguments refer to; they and the call then share one scope.
template <class Stream>
void emit_call(Stream& s, const std::string& name, const std::string& args, bool checked, const std::string& locals = "") {
    if (!checked) {
        if (locals.empty()) {
            s << name << "(" << args << ");\n";
        } else {
            s << "{\n" << locals << "    " << name << "(" << args << ");\n}\n";
        }
        return;
    }
    s << "{\n" << locals;
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
// A named local array of symbolic extents (a compound literal with run-time elements is not valid C++).
inline std::string i64_local(const std::string& name, const std::vector<std::string>& v) {
    return "    const int64_t " + name + "[] = {" + (v.empty() ? std::string("0") : join(v)) + "};\n";
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
    a << "'" << precision << "', " << shape.size() << ", __docc_b200_shape, " << axes.size() << ", __docc_b200_axes, X, Y, "
      << (with_transfers ? 1 : 0);
    emit_call(s, "docc_b200_softmax", a.str(), checked, i64_local("__docc_b200_shape", shape) + i64_local("__docc_b200_axes", axes));
}
template <class Stream>
void emit_reduce(Stream& s, int op, char precision, const std::vector<std::string>& shape, const std::vector<std::string>& axes,
                 bool with_transfers, bool checked) {
    std::ostringstream a;
    a << op << ", '" << precision << "', " << shape.size() << ", __docc_b200_shape, " << axes.size() << ", __docc_b200_axes, X, Y, "
      << (with_transfers ? 1 : 0);
    emit_call(s, "docc_b200_reduce", a.str(), checked, i64_local("__docc_b200_shape", shape) + i64_local("__docc_b200_axes", axes));
}

// ConvNode -> docc_b200_conv (connectors X, W, [B] -> Y). x_shape = [N, C_in, D0..]; pads = begins then ends.
template <class Stream>
void emit_conv(Stream& s, char precision, const std::vector<std::string>& x_shape, const std::vector<std::string>& kernel_shape,
               const std::vector<std::string>& strides, const std::vector<std::string>& pads,
               const std::vector<std::string>& dilations, const std::string& c_out, const std::string& group, bool has_bias,
               bool with_transfers, bool checked) {
    std::ostringstream a;
    a << "'" << precision << "', '" << precision << "', " << kernel_shape.size()
      << ", __docc_b200_x, __docc_b200_k, __docc_b200_strides, __docc_b200_pads, __docc_b200_dil, " << c_out << ", " << group
      << ", X, W, " << (has_bias ? "B" : "NULL") << ", Y, " << (with_transfers ? 1 : 0);
    emit_call(s, "docc_b200_conv", a.str(), checked,
              i64_local("__docc_b200_x", x_shape) + i64_local("__docc_b200_k", kernel_shape) + i64_local("__docc_b200_strides", strides) +
                  i64_local("__docc_b200_pads", pads) + i64_local("__docc_b200_dil", dilations));
}

// AttentionNode -> docc_b200_attention (connectors Q, K, V -> O; contiguous [B,H,S,D] operands, so all stride
// arguments are NULL). A scale <= 0 asks for 1/sqrt(head_dim), computed in the generated code.
template <class Stream>
void emit_attention(Stream& s, char precision, const std::string& batch, const std::string& heads, const std::string& seq_q,
                    const std::string& seq_kv, const std::string& head_dim, double scale, bool causal, bool with_transfers,
                    bool checked) {
    std::ostringstream a;
    a.precision(17);
    a << "'" << precision << "', " << batch << ", " << heads << ", " << seq_q << ", " << seq_kv << ", " << head_dim << ", ";
    if (scale > 0) a << "(float)" << scale;
    else a << "1.0f / sqrtf((float)(" << head_dim << "))";
    a << ", " << (causal ? 1 : 0) << ", Q, NULL, K, NULL, V, NULL, O, NULL, " << (with_transfers ? 1 : 0);
    emit_call(s, "docc_b200_attention", a.str(), checked);
}

// LayerNormNode -> docc_b200_layernorm (connectors X, [G, B] -> Y; rows = product of the leading dimensions).
template <class Stream>
void emit_layernorm(Stream& s, char precision, const std::string& rows, const std::string& cols, double eps, bool affine,
                    bool with_transfers, bool checked) {
    std::ostringstream a;
    a.precision(17);
    a << "'" << precision << "', " << rows << ", " << cols << ", X, " << (affine ? "G, B" : "NULL, NULL") << ", " << eps << ", Y, "
      << (with_transfers ? 1 : 0);
    emit_call(s, "docc_b200_layernorm", a.str(), checked);
}

// ElementWiseUnaryNode (Exp, Erf, Tanh, Sqrt, Sigmoid, ReLU, Abs; connectors X -> Y, elementwise_node.cpp:86-200)
// -> docc_b200_bias_act with the matching activation code, scale 1, no bias, no residual. `count` is the product of
// the node's shape; the call sees the tensor as one row.
template <class Stream>
void emit_unary(Stream& s, char precision, int act, const std::string& count, bool with_transfers, bool checked) {
    std::ostringstream a;
    a << "'" << precision << "', 1, " << count << ", X, 1.0f, NULL, " << act << ", NULL, Y, " << (with_transfers ? 1 : 0);
    emit_call(s, "docc_b200_bias_act", a.str(), checked);
}

// ElementWiseBinaryNode (Add, Sub, Mul, Div, Maximum, Minimum; connectors A, B -> C, elementwise_node.cpp:202-339)
// -> docc_b200_binary.
template <class Stream>
void emit_binary(Stream& s, int op, char precision, const std::string& count, bool with_transfers, bool checked) {
    std::ostringstream a;
    a << op << ", '" << precision << "', " << count << ", A, B, C, " << (with_transfers ? 1 : 0);
    emit_call(s, "docc_b200_binary", a.str(), checked);
}

// CastNode (connectors X -> Y) -> docc_b200_cast.
template <class Stream>
void emit_cast(Stream& s, char precision_in, char precision_out, const std::string& count, bool with_transfers, bool checked) {
    std::ostringstream a;
    a << "'" << precision_in << "', '" << precision_out << "', " << count << ", X, Y, " << (with_transfers ? 1 : 0);
    emit_call(s, "docc_b200_cast", a.str(), checked);
}

// One CUDADataOffloadingNode (cuda_data_offloading_node.cpp:139-173) in the order its dispatcher uses: allocation
// first, then the copy, then the release. `dst` / `src` are the node's output(0) / input(0) connector names.
template <class Stream>
void emit_offload(Stream& s, bool alloc, bool h2d, bool d2h, bool free_, const std::string& dst, const std::string& src,
                  const std::string& bytes, bool checked) {
    if (alloc) emit_call(s, "docc_b200_malloc", "(void**)&" + dst + ", " + bytes, checked);
    if (h2d) emit_call(s, "docc_b200_h2d", dst + ", " + src + ", " + bytes, checked);
    else if (d2h) emit_call(s, "docc_b200_d2h", dst + ", " + src + ", " + bytes, checked);
    if (free_) emit_call(s, "docc_b200_free", src, checked);
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
