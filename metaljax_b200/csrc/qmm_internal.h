// Internal declarations shared by the libqmm translation units.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qmm.h"

namespace qmm {

// Records `msg` (printf-style) as the calling thread's last error and returns `code`.
int fail(int code, const char* fmt, ...);

// Bumps the process-wide launch counter reported by qmm_launch_count().
void count_launch(int n = 1);

// Checks the CUDA runtime's sticky/launch error after a launch.
int check_launch(const char* what);

// Kernel families. Each validates nothing: `qmm_launch` has already done so.
int launch_simt(const qmm_problem& p, cudaStream_t stream);
int launch_gemv(const qmm_problem& p, cudaStream_t stream);
bool gemv_supports(const qmm_problem& p);
int launch_gemm_tc(const qmm_problem& p, cudaStream_t stream);
bool gemm_tc_supports(const qmm_problem& p);
// Reads (and clears) the tensor-core kernel's device status word; synchronizes the device.
int gemm_tc_status(int* out);

int launch_dequantize(const uint32_t* w, const void* scales, const void* biases, int table_dtype,
                      void* out, int out_dtype, int64_t rows, int64_t K, int group_size, int bits,
                      int mode, cudaStream_t stream);
int launch_pack_codes(const uint8_t* codes, uint32_t* out, int64_t rows, int64_t K, int bits,
                      cudaStream_t stream);

inline int elem_size(int e) {
  switch (e) {
    case QMM_BF16: case QMM_F16: return 2;
    case QMM_F32: case QMM_U32: case QMM_I32: return 4;
    case QMM_U8: return 1;
  }
  return 0;
}

}  // namespace qmm
