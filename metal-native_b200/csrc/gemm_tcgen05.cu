#include "mnq_common.cuh"
namespace mnq {
bool gemm_supported(const MatmulArgs&) { return false; }
int launch_gemm(const MatmulArgs&, const mnq_tuning*) { return fail(MNQ_NOT_IMPLEMENTED, "gemm path not built yet"); }
}
