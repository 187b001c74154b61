// Prints the host calls the B200 dispatchers emit for a fixed set of nodes (golden-text test driver).
#include <iostream>

#include "b200_emit.h"

using namespace docc_b200_plugin;

int main(int argc, char** argv) {
    const bool checked = argc > 1 && std::string(argv[1]) == "checked";
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
    emit_alloc(std::cout, "__daisy_dev_A", "8 * m * k", checked);
    emit_h2d(std::cout, "__daisy_dev_A", "A", "8 * m * k", checked);
    emit_d2h(std::cout, "C", "__daisy_dev_C", "8 * m * n", checked);
    emit_free(std::cout, "__daisy_dev_A", checked);
    return 0;
}
