// gemm_f64_dmma.cu -- placeholder until the FP64 tensor-core kernel lands.
#include "common.cuh"
namespace ttb {
bool f64_dmma_eligible(const Problem &) { return false; }
int launch_f64_dmma(const Problem &) {
    set_error("f64 DMMA kernel not built");
    return TTB_EUNSUPPORTED;
}
}  // namespace ttb
