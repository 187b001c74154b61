// Implicit-GEMM convolution on the tcgen05 engine.
#include "conv.h"

namespace docc_b200 {

int conv_tc(Ctx*, const ConvTcProblem&, const void*, const void*, const float*, float*) {
    return set_error(DOCC_B200_ERR_UNSUPPORTED, "conv_tc: not available");
}

}  // namespace docc_b200
