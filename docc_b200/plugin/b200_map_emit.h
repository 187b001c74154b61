// Text of the sm_100a kernels and launches that the B200 map dispatcher writes for leftover element-wise maps:
// loop nests that are not library nodes and whose every access is `array[induction variable]`.
//
// docc's CUDA target turns such a map into a scalar kernel, one element per thread, guarded by `if (i < n)`
// (opt/src/targets/cuda/cuda_map_dispatcher.cpp:42-168, launch geometry 32 threads per block from
// opt/src/passes/scheduler/cuda_scheduler.cpp:13-70). These maps are HBM-bound, so what matters on B200 is the width
// of each access and the amount of data in flight: the kernel emitted here moves 16 bytes per access of the widest
// element type (narrower operands move proportionally less), walks the range with a grid-stride loop from a grid of
// at most 8 blocks of 256 threads per SM, and keeps the scalar form, chosen at launch, for operands that are not
// aligned for vector access. A scalar tail loop finishes ranges that are not a multiple of the vector width.
//
// Dependency-free like b200_emit.h: the dispatcher (b200_map_dispatcher.cpp, needs docc's headers) recognises the map,
// prints the tasklet body through docc's language extension and hands the pieces over as strings, so the emitted text
// can be golden-tested, compiled with nvcc for sm_100a and run against the same loop on the CPU without a docc build.
#pragma once

#include <sstream>
#include <string>
#include <vector>

namespace docc_b200_plugin {

struct MapOperand {
    std::string name;        // container name
    std::string ctype;       // element type as C text: "float", "double", "__nv_bfloat16", "int", ...
    int bytes;               // sizeof(ctype)
    bool also_read = false;  // outputs only: the map updates the container in place (reads the element it writes)
};

struct ElementwiseMap {
    std::string kernel_name;
    std::vector<MapOperand> inputs;    // read-only containers
    std::vector<MapOperand> outputs;   // written containers
    std::vector<MapOperand> scalars;   // passed by value (symbols, constants)
    std::string body;                  // C statements for one iteration
    std::string count;                 // iteration count as a C expression over the scalars
    // Two forms of `body`:
    //  * indvar empty: an operand's name denotes the element of the current iteration (`out = alpha * a + b;`)
    //  * indvar set:   the text docc's block dispatcher prints, `out[i] = alpha * a[i] + b[i];` with i = indvar. The kernel
    //    then declares, around the unchanged text, each container name as a pointer to the thread's vector registers and
    //    the induction variable as the lane index, so the same text serves the vector loop and the scalar tail.
    std::string indvar;
};

inline int map_vector_width(const ElementwiseMap& m) {
    int widest = 1;
    for (auto& o : m.inputs) widest = o.bytes > widest ? o.bytes : widest;
    for (auto& o : m.outputs) widest = o.bytes > widest ? o.bytes : widest;
    const int v = 16 / widest;
    return v < 1 ? 1 : v;
}

inline std::string map_parameters(const ElementwiseMap& m, bool restrict_qualified) {
    std::ostringstream s;
    const char* rq = restrict_qualified ? "* __restrict__ " : "* ";
    bool first = true;
    for (auto& o : m.inputs) {
        s << (first ? "" : ", ") << "const " << o.ctype << rq << o.name << "_ptr";
        first = false;
    }
    for (auto& o : m.outputs) {
        s << (first ? "" : ", ") << o.ctype << rq << o.name << "_ptr";
        first = false;
    }
    for (auto& o : m.scalars) {
        s << (first ? "" : ", ") << o.ctype << " " << o.name;
        first = false;
    }
    return s.str();
}

// The kernel: template parameter V = elements per thread and step (the vector width, or 1).
template <class Stream> void emit_map_kernel(Stream& s, const ElementwiseMap& m) {
    const bool indexed = !m.indvar.empty();
    s << "// element-wise map: 16-byte accesses of the widest operand, grid-stride loop, scalar tail\n";
    s << "#ifndef DOCC_B200_VEC_DEFINED\n#define DOCC_B200_VEC_DEFINED\n";
    s << "template <typename T, int V> struct alignas(sizeof(T) * V) docc_b200_vec { T v[V]; };\n#endif\n";
    s << "template <int V>\n__global__ void __launch_bounds__(256) " << m.kernel_name << "(";
    const std::string params = map_parameters(m, true);
    s << params << (params.empty() ? "" : ", ") << "long long __n) {\n";
    s << "    const long long __groups = __n / V;\n";
    s << "    const long long __stride = (long long)gridDim.x * blockDim.x;\n";
    s << "    for (long long __g = (long long)blockIdx.x * blockDim.x + threadIdx.x; __g < __groups; __g += __stride) {\n";
    for (auto& o : m.inputs)
        s << "        const docc_b200_vec<" << o.ctype << ", V> " << o.name << "_in = *reinterpret_cast<const docc_b200_vec<" << o.ctype
          << ", V>*>(" << o.name << "_ptr + __g * V);\n";
    for (auto& o : m.outputs) {
        s << "        docc_b200_vec<" << o.ctype << ", V> " << o.name << "_out";
        if (o.also_read) s << " = *reinterpret_cast<const docc_b200_vec<" << o.ctype << ", V>*>(" << o.name << "_ptr + __g * V)";
        s << ";\n";
    }
    if (indexed) {
        for (auto& o : m.inputs) s << "        const " << o.ctype << "* const " << o.name << " = " << o.name << "_in.v;\n";
        for (auto& o : m.outputs) s << "        " << o.ctype << "* const " << o.name << " = " << o.name << "_out.v;\n";
    }
    s << "#pragma unroll\n        for (int __e = 0; __e < V; __e++) {\n";
    if (indexed) {
        s << "            const int " << m.indvar << " = __e;\n";
        s << "            " << m.body << "\n";
    } else {
        for (auto& o : m.inputs) s << "            const " << o.ctype << " " << o.name << " = " << o.name << "_in.v[__e];\n";
        for (auto& o : m.outputs)
            s << "            " << o.ctype << " " << o.name << (o.also_read ? " = " + o.name + "_out.v[__e]" : "") << ";\n";
        s << "            " << m.body << "\n";
        for (auto& o : m.outputs) s << "            " << o.name << "_out.v[__e] = " << o.name << ";\n";
    }
    s << "        }\n";
    for (auto& o : m.outputs)
        s << "        *reinterpret_cast<docc_b200_vec<" << o.ctype << ", V>*>(" << o.name << "_ptr + __g * V) = " << o.name << "_out;\n";
    s << "    }\n";
    s << "    // tail: the last __n % V elements, one per thread of the first block\n";
    s << "    if (blockIdx.x == 0) {\n";
    if (indexed) {
        for (auto& o : m.inputs) s << "        const " << o.ctype << "* const " << o.name << " = " << o.name << "_ptr;\n";
        for (auto& o : m.outputs) s << "        " << o.ctype << "* const " << o.name << " = " << o.name << "_ptr;\n";
    }
    s << "        for (long long __i = __groups * V + threadIdx.x; __i < __n; __i += blockDim.x) {\n";
    if (indexed) {
        s << "            const long long " << m.indvar << " = __i;\n";
        s << "            " << m.body << "\n";
    } else {
        for (auto& o : m.inputs) s << "            const " << o.ctype << " " << o.name << " = " << o.name << "_ptr[__i];\n";
        for (auto& o : m.outputs)
            s << "            " << o.ctype << " " << o.name << (o.also_read ? " = " + o.name + "_ptr[__i]" : "") << ";\n";
        s << "            " << m.body << "\n";
        for (auto& o : m.outputs) s << "            " << o.name << "_ptr[__i] = " << o.name << ";\n";
    }
    s << "        }\n    }\n}\n";
}

// Host-side launcher, emitted into the same .cu file as the kernel (a template cannot be launched from another
// translation unit): `extern "C" void <kernel>_launch(device pointers..., scalars...)`. Picks the vector form when every
// operand is aligned for it, sizes the grid from the device's SM count, and launches on the stream of the runtime
// (docc_b200_get_stream) so that the kernel is ordered with the library-node calls around it.
template <class Stream> void emit_map_launcher(Stream& s, const ElementwiseMap& m) {
    const int V = map_vector_width(m);
    s << "extern \"C\" void " << m.kernel_name << "_launch(" << map_parameters(m, false) << ") {\n";
    s << "    const long long __n = (long long)(" << m.count << ");\n";
    s << "    if (__n <= 0) return;\n";
    s << "    void* __stream = 0;\n    docc_b200_get_stream(&__stream);\n";
    s << "    bool __vec = " << (V > 1 ? "true" : "false") << ";\n";
    auto align_check = [&](const MapOperand& o) {
        if (V > 1) s << "    __vec = __vec && ((unsigned long long)(" << o.name << "_ptr) % " << o.bytes * V << " == 0);\n";
    };
    for (auto& o : m.inputs) align_check(o);
    for (auto& o : m.outputs) align_check(o);
    s << "    int __sms = 0, __dev = 0;\n    cudaGetDevice(&__dev);\n    cudaDeviceGetAttribute(&__sms, cudaDevAttrMultiProcessorCount, __dev);\n";
    s << "    const long long __work = __vec ? (__n + " << V << " - 1) / " << V << " : __n;\n";
    s << "    long long __blocks = (__work + 255) / 256;\n";
    s << "    if (__blocks > 8LL * __sms) __blocks = 8LL * __sms;\n";
    std::ostringstream args;
    for (auto& o : m.inputs) args << o.name << "_ptr, ";
    for (auto& o : m.outputs) args << o.name << "_ptr, ";
    for (auto& o : m.scalars) args << o.name << ", ";
    args << "__n";
    s << "    if (__vec) " << m.kernel_name << "<" << V << "><<<(unsigned)__blocks, 256, 0, (cudaStream_t)__stream>>>(" << args.str() << ");\n";
    s << "    else " << m.kernel_name << "<1><<<(unsigned)__blocks, 256, 0, (cudaStream_t)__stream>>>(" << args.str() << ");\n";
    s << "}\n";
}

// Declaration of the launcher for the generated host file (globals stream).
template <class Stream> void emit_map_launcher_declaration(Stream& s, const ElementwiseMap& m) {
    s << "extern \"C\" void " << m.kernel_name << "_launch(" << map_parameters(m, false) << ");\n";
}

// The call in the generated host code. `dev_names[i]` is the variable holding operand i's device pointer (inputs first,
// then outputs); scalars are passed under their own names.
template <class Stream>
void emit_map_call(Stream& s, const ElementwiseMap& m, const std::vector<std::string>& dev_names) {
    s << m.kernel_name << "_launch(";
    bool first = true;
    for (auto& d : dev_names) {
        s << (first ? "" : ", ") << d;
        first = false;
    }
    for (auto& o : m.scalars) {
        s << (first ? "" : ", ") << o.name;
        first = false;
    }
    s << ");\n";
}

}  // namespace docc_b200_plugin
