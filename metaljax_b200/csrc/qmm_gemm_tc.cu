#include "qmm_internal.h"
namespace qmm {
bool gemm_tc_supports(const qmm_problem&) { return false; }
int launch_gemm_tc(const qmm_problem&, cudaStream_t) { return fail(QMM_ERR_UNSUPPORTED, "gemm_tc"); }
}
