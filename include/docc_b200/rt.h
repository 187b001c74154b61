/*
 * docc_b200 runtime — C ABI of the B200 (sm_100a) library-node kernels.
 *
 * This is the layer generated host code links against (next to -ldaisy_rtl,
 * python/bindings/py_structured_sdfg.cpp:529-541 in docc) and that a
 * LibraryNodeDispatcher for the B200 target emits calls into, in place of
 *   - the cuBLAS call sequence of opt/src/targets/cuda/blas/gemm.cpp:33-185,
 *   - the cudaMalloc/cudaMemcpy/cudaFree emitted by
 *     opt/src/targets/cuda/cuda_data_offloading_node.cpp:139-173,
 *   - the generic __global__ loop nests that Softmax / Conv / element-wise
 *     tensor nodes expand to (opt/src/targets/cuda/cuda_map_dispatcher.cpp:42-333).
 *
 * Conventions
 *   - Every entry returns an int status (DOCC_B200_OK == 0). Nothing here
 *     aborts the process; docc_b200_last_error() returns a thread-local
 *     detail string for the most recent failure on the calling thread.
 *   - Plain pointers and sizes only. Unless DOCC_B200_FLAG_HOST_PTRS is set,
 *     data pointers are device pointers of the current device.
 *   - With DOCC_B200_FLAG_HOST_PTRS the data pointers are host pointers; the
 *     call stages them through device memory (H2D, kernel, D2H) and returns
 *     after the result is back in host memory ("WithTransfers" in docc's
 *     vocabulary, cuda.h:20-26).
 *   - Device-pointer calls are asynchronous on the calling thread's stream
 *     (docc_b200_set_stream / docc_b200_get_stream); docc_b200_sync() waits.
 *   - Re-entrant: one context per (thread, device); the device-memory pool is
 *     guarded by a mutex.
 *   - Enum values for precision / layout / transpose are docc's own
 *     (sdfg/include/sdfg/data_flow/library_nodes/math/blas/blas_node.h:49-126).
 */
#ifndef DOCC_B200_RT_H
#define DOCC_B200_RT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
enum {
    DOCC_B200_OK = 0,
    DOCC_B200_ERR_INVALID_ARG = 1,   /* null pointer, negative size, bad enum, bad alignment */
    DOCC_B200_ERR_UNSUPPORTED = 2,   /* valid request that no kernel covers */
    DOCC_B200_ERR_CUDA = 3,          /* a CUDA runtime/driver call failed */
    DOCC_B200_ERR_OOM = 4,           /* device or pinned-host allocation failed / limit hit */
    DOCC_B200_ERR_NO_DEVICE = 5,     /* no usable sm_100 device */
    DOCC_B200_ERR_DEVICE_TIMEOUT = 6 /* a bounded device-side wait ran out (status word set by the kernel) */
};

/* ---- precision codes (BLAS_Precision, blas_node.h:49-55; 'b' is an extension) */
enum {
    DOCC_B200_PREC_H = 'h', /* fp16 storage, fp32 accumulate */
    DOCC_B200_PREC_S = 's', /* fp32 */
    DOCC_B200_PREC_D = 'd', /* fp64 */
    DOCC_B200_PREC_B = 'b'  /* bf16 storage, fp32 accumulate (no docc counterpart) */
};
/* BLAS_Layout (blas_node.h:113-116) and BLAS_Transpose (blas_node.h:77-81) */
enum { DOCC_B200_ROW_MAJOR = 101, DOCC_B200_COL_MAJOR = 102 };
enum { DOCC_B200_NO_TRANS = 111, DOCC_B200_TRANS = 112, DOCC_B200_CONJ_TRANS = 113 };

/* ---- flags ---------------------------------------------------------------- */
enum {
    DOCC_B200_FLAG_HOST_PTRS = 1,   /* data pointers are host memory: do the transfers */
    DOCC_B200_FLAG_FP32_EXACT = 2   /* fp32 contractions: use the FFMA kernels instead of split-bf16 tensor cores */
};

/* ---- activation / epilogue codes ------------------------------------------- */
enum {
    DOCC_B200_ACT_NONE = 0,
    DOCC_B200_ACT_GELU_ERF = 1,  /* 0.5*x*(1+erf(x/sqrt(2))) — what linalg.erf-based GELU lowers to */
    DOCC_B200_ACT_RELU = 2,
    DOCC_B200_ACT_TANH = 3,
    DOCC_B200_ACT_SIGMOID = 4,
    DOCC_B200_ACT_EXP = 5,
    DOCC_B200_ACT_ERF = 6,
    DOCC_B200_ACT_SQRT = 7,
    DOCC_B200_ACT_ABS = 8
};

/* ---- element-wise binary / reduce op codes ---------------------------------- */
enum { DOCC_B200_EW_ADD = 0, DOCC_B200_EW_SUB = 1, DOCC_B200_EW_MUL = 2, DOCC_B200_EW_DIV = 3,
       DOCC_B200_EW_MAX = 4, DOCC_B200_EW_MIN = 5 };
enum { DOCC_B200_RED_SUM = 0, DOCC_B200_RED_MAX = 1, DOCC_B200_RED_MIN = 2,
       DOCC_B200_RED_MEAN = 3, DOCC_B200_RED_STD = 4 };

/* ---- context, memory, transfers -------------------------------------------- */

/* Selects `device` for the calling thread and creates its context lazily.
 * Replaces the hard-coded cudaSetDevice(0) of
 * sdfg/src/codegen/code_generators/cpp_code_generator.cpp:191,218. */
int docc_b200_init(int device);
/* Releases the calling thread's pooled device memory and streams on the current device. */
int docc_b200_shutdown(void);
/* Number of visible CUDA devices (0 when there is none; never fails). */
int docc_b200_device_count(void);

/* Device allocation / free: 1:1 with the ALLOC / FREE lifecycle of
 * CUDADataOffloadingNode (cuda_data_offloading_node.cpp:149-158,166-172).
 * Backed by a size-bucketed, stream-ordered pool so repeated alloc/free pairs
 * around a node cost no cudaMalloc and no host synchronisation: free marks the
 * calling thread's stream, and whoever gets the block next (any thread, any
 * stream) is ordered after that mark on the device. Use a buffer only on the
 * stream that was current when it was allocated, or order the streams yourself. */
int docc_b200_malloc(void** dptr, size_t bytes);
int docc_b200_free(void* dptr);
/* H2D / D2H copies: the two transfer directions of CUDADataOffloadingNode
 * (cuda_data_offloading_node.cpp:159-165). Synchronous with respect to the
 * host buffer, ordered on the calling thread's stream. */
int docc_b200_h2d(void* dptr, const void* hptr, size_t bytes);
int docc_b200_d2h(void* hptr, const void* dptr, size_t bytes);
/* Pinned host memory for callers that want full-rate asynchronous transfers. */
int docc_b200_host_alloc(void** hptr, size_t bytes);
int docc_b200_host_free(void* hptr);
/* Caps the bytes the pool may hold from the driver (0 = no cap). Used by tests
 * to provoke DOCC_B200_ERR_OOM on the host without exhausting a GPU. */
int docc_b200_set_alloc_limit(size_t bytes);

/* Stream control. `stream` is a cudaStream_t; NULL restores the library's own
 * per-thread stream. CUDA's special handles cudaStreamLegacy ((cudaStream_t)0x1)
 * and cudaStreamPerThread ((cudaStream_t)0x2) name the default streams.
 * Replaces the implicit default stream of generated code.
 * The calling thread's library-owned workspaces (operand planes, block
 * intermediates) are ordered on one stream at a time: switching makes the new
 * stream wait, on the device, for the work queued on the old one. The old
 * stream must still exist when the switch is made. */
int docc_b200_set_stream(void* stream);
int docc_b200_get_stream(void** stream);
/* Waits for everything queued on the calling thread's stream
 * (cudaDeviceSynchronize in opt/src/targets/cuda/cuda.cpp:93-103). */
int docc_b200_sync(void);

const char* docc_b200_strerror(int status);
const char* docc_b200_last_error(void);
/* Number of kernels this library launched from the calling thread since the last reset. */
int64_t docc_b200_launch_count(int reset);
/* Self-test of the bounded-wait error path (no reference counterpart; docc's generated
 * kernels have no waits). Launches one warp that waits, for at most `limit_cycles` SM
 * clocks, on a shared-memory barrier nothing arrives at; the warp then gives up exactly
 * as the tensor-core kernels do: it sets the status word and returns. The following
 * docc_b200_sync() returns DOCC_B200_ERR_DEVICE_TIMEOUT once and clears the word. */
int docc_b200_selftest_wait_timeout(int64_t limit_cycles);

/* ---- GEMM -------------------------------------------------------------------
 * C[m x n] = alpha * op(A) * op(B) + beta * C, the GEMMNode contract
 * (gemm_node.h:16-87; parameters in the order of cblas_?gemm as emitted by
 * GEMMNodeDispatcher_BLAS, gemm_node.cpp:449-509, and of generate_kernel_gemm,
 * opt/src/targets/cuda/blas/gemm.cpp:131-185).
 * alpha/beta point to HOST scalars of the element type for 's'/'d' and to
 * float for 'h'/'b'. beta == 0 means C is not read (BLAS rule). */
int docc_b200_gemm(int prec, int layout, int transa, int transb,
                   int64_t m, int64_t n, int64_t k,
                   const void* alpha, const void* A, int64_t lda,
                   const void* B, int64_t ldb,
                   const void* beta, void* C, int64_t ldc, int flags);

/* Row-major fp32 GEMM C = alpha * op(A) * op(B) + beta * C on device pointers that allocates
 * nothing (no counterpart in the reference; docc's cuBLAS path allocates on every call).
 * For embedders that cannot allocate device memory once they are running: a host application
 * that gave the whole GPU to its own allocator at start-up, or a latency-critical loop that
 * cannot take the device-wide synchronisation of cudaMalloc / cudaFree. The bf16 hi/lo planes
 * of A and B live in a fixed 16 MiB array inside the library image (held by every GPU that
 * loads the library until the process exits), so 4 * (m + n) * roundup8(k) bytes must fit in
 * 16 MiB; larger problems return DOCC_B200_ERR_INVALID_ARG. k >= 1. `stream` is the
 * cudaStream_t to run on; the call returns once C is complete. All calls share the array
 * (it keeps the previous call's contents), so calls that overlap on the GPU race: serialise
 * them. The first call on a device looks up the array's device address and sets a kernel
 * attribute; make it before any stream capture. Same kernels and pass order as
 * docc_b200_gemm('s'), so results are identical to it. */
int docc_b200_gemm_f32_noalloc(int transa, int transb, int64_t m, int64_t n, int64_t k,
                               float alpha, const float* A, int64_t lda,
                               const float* B, int64_t ldb,
                               float beta, float* C, int64_t ldc, void* stream);

/* Batched row-major matmul Y[b] = A[b] * B[b]: the loop nest MatMulNode::expand
 * wraps around GEMMNode (matmul_node.cpp:286-544; lda = strides_a[-2], ldc = N,
 * :463-489). A batch stride of 0 broadcasts that operand. */
int docc_b200_matmul(int prec, int64_t batch, int64_t m, int64_t n, int64_t k,
                     const void* A, int64_t lda, int64_t batch_stride_a,
                     const void* B, int64_t ldb, int64_t batch_stride_b,
                     void* Y, int64_t ldy, int64_t batch_stride_y, int flags);

/* GEMM with a fused bandwidth epilogue (no docc counterpart as one node; it is
 * the fusion of GEMMNode with the element-wise tensor nodes of
 * elementwise_node.cpp:86-339 that follow it in a transformer block):
 *   Y = act(alpha * A*op(B) + bias[n]) + residual
 * Row-major. transb == DOCC_B200_TRANS reads B as [n x k] (torch Linear weight).
 * prec 's': fp32 in/out; 'd': fp64 in/out; 'b' / 'h': 16-bit in/out. The bias has the
 * element type of Y for 's' and 'd' and is fp32 for 16-bit operands; the residual has
 * the type of Y and at least m rows of n elements (row stride ldr >= n).
 * bias / residual may be NULL. */
int docc_b200_gemm_epilogue(int prec, int transb, int64_t m, int64_t n, int64_t k,
                            float alpha, const void* A, int64_t lda,
                            const void* B, int64_t ldb,
                            const void* bias, int act,
                            const void* residual, int64_t ldr,
                            void* Y, int64_t ldy, int flags);

/* ---- Softmax ------------------------------------------------------------------
 * Max-subtracted softmax over `axes` of a C-order tensor: SoftmaxNode
 * (softmax_node.h:9-53; expansion softmax_node.cpp:38-265). keepdims is always
 * false as in the node (softmax_node.cpp:31-33). prec 's', 'd', 'h' or 'b'. */
int docc_b200_softmax(int prec, int rank, const int64_t* shape,
                      int naxes, const int64_t* axes,
                      const void* X, void* Y, int flags);

/* ---- Reductions -----------------------------------------------------------------
 * Sum / Max / Min / Mean / Std over `axes` of a C-order tensor: ReduceNode and
 * its subclasses (reduce_node.cpp:122-345, sum_node.cpp:20-49, max_node.cpp:23-71,
 * mean_node.cpp:77-118, std_node.cpp:147-222). Y has the reduced axes removed. */
int docc_b200_reduce(int op, int prec, int rank, const int64_t* shape,
                     int naxes, const int64_t* axes,
                     const void* X, void* Y, int flags);

/* ---- Conv ------------------------------------------------------------------------
 * N-D cross-correlation in NC(D..) layout, the ConvNode contract
 * (conv_node.h:87-200, expansion conv_node.cpp:85-454):
 *   Y[n,oc,o..] = B[oc] + sum_{ic,k..} X[n, g*Cin/G + ic, o*s - p_begin + k*d] * W[oc, ic, k..]
 * x_shape = [N, C_in, D0..], k_shape = [k0..], pads = [begin0.., end0..].
 * Out-of-range taps contribute zero (the ONNX contract conv_node.h:9-22 cites).
 * prec_in 's' or 'b'/'h' (16-bit inputs), prec_out 's' or same as prec_in;
 * accumulation is fp32 ('d' in/out accumulates in fp64). Bias is of prec_out. */
int docc_b200_conv(int prec_in, int prec_out, int spatial_rank,
                   const int64_t* x_shape, const int64_t* k_shape,
                   const int64_t* strides, const int64_t* pads, const int64_t* dilations,
                   int64_t c_out, int64_t group,
                   const void* X, const void* W, const void* B_or_null, void* Y, int flags);

/* ---- Attention ----------------------------------------------------------------------
 * O = softmax(scale * Q K^T [+ causal mask]) V per (batch, head); flash-style, the
 * Sq x Skv score matrix never reaches HBM. No docc node exists; semantics are the
 * composition MatMulNode -> scale -> SoftmaxNode(axis -1) -> MatMulNode.
 * Element strides let Q/K/V/O live inside a packed projection output:
 * element (b,h,s,d) is at base + b*sb + h*sh + s*ss + d. Pass NULL strides for
 * contiguous [B,H,S,D]. prec 'b' or 'h' (fp32 accumulate) or 's'. Causal masking
 * aligns the last query with the last key (query i sees keys j <= i + Skv - Sq). */
int docc_b200_attention(int prec, int64_t B, int64_t H, int64_t Sq, int64_t Skv, int64_t D,
                        float scale, int causal,
                        const void* Q, const int64_t* q_strides /*[sb,sh,ss] or NULL*/,
                        const void* K, const int64_t* k_strides,
                        const void* V, const int64_t* v_strides,
                        void* O, const int64_t* o_strides, int flags);

/* ---- LayerNorm ---------------------------------------------------------------------
 * Y = (X - mean) / sqrt(var + eps) * gamma + beta over the last dimension, population
 * variance (the MeanNode / StdNode building blocks, mean_node.cpp:77-118,
 * std_node.cpp:147-222). gamma/beta are fp32 and may be NULL. prec 's', 'b' or 'h'. */
int docc_b200_layernorm(int prec, int64_t rows, int64_t cols,
                        const void* X, const void* gamma, const void* beta,
                        double eps, void* Y, int flags);

/* ---- element-wise -------------------------------------------------------------------
 * Y = act(scale * X + bias[col]) + residual over a [rows x cols] C-order tensor: the
 * fused form of the Add / Mul / Erf / Tanh / ... tensor nodes
 * (elementwise_node.cpp:86-339, elementwise_ops/). bias (fp32, per column) and
 * residual (same type and shape as X) may be NULL. */
int docc_b200_bias_act(int prec, int64_t rows, int64_t cols,
                       const void* X, float scale, const void* bias, int act,
                       const void* residual, void* Y, int flags);
/* Y = X1 (op) X2, same-shape binary tensor node (elementwise_ops/add_node.cpp etc.). */
int docc_b200_binary(int op, int prec, int64_t n, const void* X1, const void* X2, void* Y, int flags);
/* Y = cast(X): CastNode (elementwise_ops/cast_node.cpp). Types are precision codes. */
int docc_b200_cast(int prec_in, int prec_out, int64_t n, const void* X, void* Y, int flags);

/* ---- pre-LN transformer encoder block ----------------------------------------------
 * y = h + W2 gelu(W1 LN2(h) + b1) + b2,  h = x + Wo attn(LN1(x) Wqkv + bqkv) + bo
 * Convenience entry that chains the node kernels above on device with library-owned
 * workspaces (the "keep tensors device-resident across consecutive library nodes"
 * schedule that DataTransferMinimizationPass, loop_scheduling_pass.cpp:130-133, aims at).
 * Weights use the torch Linear layout [out_features x in_features]. prec 's' or 'b'
 * (weights and activations of that type; biases and LN parameters fp32). */
typedef struct {
    int64_t batch, seq, d_model, n_heads, d_ff;
    double eps;
    const void *ln1_g, *ln1_b, *w_qkv, *b_qkv, *w_o, *b_o;
    const void *ln2_g, *ln2_b, *w_1, *b_1, *w_2, *b_2;
} docc_b200_block_params;
int docc_b200_transformer_block(int prec, const docc_b200_block_params* p,
                                const void* X, void* Y, int flags);

#ifdef __cplusplus
}
#endif
#endif /* DOCC_B200_RT_H */
