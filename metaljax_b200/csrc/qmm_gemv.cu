#include "qmm_internal.h"
namespace qmm {
bool gemv_supports(const qmm_problem&) { return false; }
int launch_gemv(const qmm_problem&, cudaStream_t) { return fail(QMM_ERR_UNSUPPORTED, "gemv"); }
}
