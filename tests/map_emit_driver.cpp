// Prints a CUDA translation unit with the kernels and launches the B200 map dispatcher emits for four element-wise
// maps (golden-text test driver; the text is also compiled with nvcc for sm_100a and run against the same loops on the CPU).
// With the argument "cpu" it prints the same loop bodies as plain sequential C loops instead.
#include <iostream>
#include <string>

#include "b200_map_emit.h"

using namespace docc_b200_plugin;

static ElementwiseMap axpby() {
    ElementwiseMap m;
    m.kernel_name = "kernel_axpby_3";
    m.inputs = {{"a", "float", 4}, {"b", "float", 4}};
    m.outputs = {{"out", "float", 4}};
    m.scalars = {{"alpha", "float", 4}, {"_s0", "long long", 8}};
    m.body = "out = fmaf(alpha, a, b);";
    m.count = "_s0";
    return m;
}
static ElementwiseMap widen() {  // fp32 -> fp64 with arithmetic: the widest operand sets the vector width (2 elements)
    ElementwiseMap m;
    m.kernel_name = "kernel_widen_7";
    m.inputs = {{"x", "float", 4}};
    m.outputs = {{"y", "double", 8}};
    m.scalars = {{"_s0", "long long", 8}, {"_s1", "long long", 8}};
    m.body = "y = sqrt(fabs((double)x)) + 0.5;";
    m.count = "_s0 * _s1";
    return m;
}
static ElementwiseMap two_outputs() {  // 16-bit operands: eight elements per access
    ElementwiseMap m;
    m.kernel_name = "kernel_sumdiff_9";
    m.inputs = {{"p", "unsigned short", 2}, {"q", "unsigned short", 2}};
    m.outputs = {{"s", "unsigned short", 2}, {"d", "unsigned short", 2}};
    m.scalars = {{"_s0", "long long", 8}};
    m.body = "s = (unsigned short)(p + q); d = (unsigned short)(p - q);";
    m.count = "_s0";
    return m;
}

static ElementwiseMap scale_in_place() {  // body in the form docc's block dispatcher prints; updates its container in place
    ElementwiseMap m;
    m.kernel_name = "kernel_scale_12";
    m.inputs = {{"__daisy_cuda_w", "float", 4}};
    m.outputs = {{"__daisy_cuda_acc", "float", 4, true}};
    m.scalars = {{"lr", "float", 4}, {"N", "int", 4}};
    m.body = "{ float _in1 = __daisy_cuda_acc[i]; float _in2 = __daisy_cuda_w[i]; float _out = fmaf(-lr, _in2, _in1); __daisy_cuda_acc[i] = _out; }";
    m.count = "N";
    m.indvar = "i";
    return m;
}

static void cpu_loop(const ElementwiseMap& m, const std::string& entry, const std::string& params) {
    std::cout << "extern \"C\" void " << entry << "(" << params << ") {\n    const long long __n = (long long)(" << m.count << ");\n";
    if (!m.indvar.empty()) {
        for (auto& o : m.inputs) std::cout << "    const " << o.ctype << "* const " << o.name << " = " << o.name << "_ptr;\n";
        for (auto& o : m.outputs) std::cout << "    " << o.ctype << "* const " << o.name << " = " << o.name << "_ptr;\n";
        std::cout << "    for (long long " << m.indvar << " = 0; " << m.indvar << " < __n; " << m.indvar << "++) {\n        " << m.body << "\n    }\n}\n";
        return;
    }
    std::cout << "    for (long long __i = 0; __i < __n; __i++) {\n";
    for (auto& o : m.inputs) std::cout << "        const " << o.ctype << " " << o.name << " = " << o.name << "_ptr[__i];\n";
    for (auto& o : m.outputs) std::cout << "        " << o.ctype << " " << o.name << ";\n";
    std::cout << "        " << m.body << "\n";
    for (auto& o : m.outputs) std::cout << "        " << o.name << "_ptr[__i] = " << o.name << ";\n";
    std::cout << "    }\n}\n";
}

int main(int argc, char** argv) {
    const bool cpu = argc > 1 && std::string(argv[1]) == "cpu";
    const std::string p1 = "const float* a_ptr, const float* b_ptr, float* out_ptr, float alpha, long long _s0";
    const std::string p2 = "const float* x_ptr, double* y_ptr, long long _s0, long long _s1";
    const std::string p3 = "const unsigned short* p_ptr, const unsigned short* q_ptr, unsigned short* s_ptr, unsigned short* d_ptr, long long _s0";
    const std::string p4 = "const float* __daisy_cuda_w_ptr, float* __daisy_cuda_acc_ptr, float lr, int N";
    if (cpu) {
        std::cout << "#include <math.h>\n";
        cpu_loop(axpby(), "axpby_op", p1);
        cpu_loop(widen(), "widen_op", p2);
        cpu_loop(two_outputs(), "sumdiff_op", p3);
        cpu_loop(scale_in_place(), "scale_op", p4);
        return 0;
    }
    std::cout << "#include <cuda_runtime.h>\n#include <docc_b200/rt.h>\n";
    for (auto& m : {axpby(), widen(), two_outputs(), scale_in_place()}) {
        emit_map_kernel(std::cout, m);
        emit_map_launcher(std::cout, m);
    }
    // host entries in the shape of docc's generated code: device pointers of the offloaded containers, shape symbols
    std::cout << "extern \"C\" void axpby_op(" << p1 << ") {\n    ";
    emit_map_call(std::cout, axpby(), {"a_ptr", "b_ptr", "out_ptr"});
    std::cout << "}\nextern \"C\" void widen_op(" << p2 << ") {\n    ";
    emit_map_call(std::cout, widen(), {"x_ptr", "y_ptr"});
    std::cout << "}\nextern \"C\" void sumdiff_op(" << p3 << ") {\n    ";
    emit_map_call(std::cout, two_outputs(), {"p_ptr", "q_ptr", "s_ptr", "d_ptr"});
    std::cout << "}\nextern \"C\" void scale_op(" << p4 << ") {\n    ";
    emit_map_call(std::cout, scale_in_place(), {"__daisy_cuda_w_ptr", "__daisy_cuda_acc_ptr"});
    std::cout << "}\n";
    return 0;
}
