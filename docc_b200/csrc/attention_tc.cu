// Flash attention on the tcgen05 engine.
#include "attention.h"

namespace docc_b200 {

int attention_tc(Ctx*, const AttnProblem&, const void*, const void*, const void*, void*) {
    return set_error(DOCC_B200_ERR_UNSUPPORTED, "attention_tc: not available");
}

}  // namespace docc_b200
