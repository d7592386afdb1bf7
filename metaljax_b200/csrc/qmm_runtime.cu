// Host-side helpers shared by the kernel launchers: tensor-map encoding through the driver
// entry point (no link-time dependency on libcuda), the device status word, device facts.
#include <cuda.h>

#include "qmm_internal.h"

namespace qmm {

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}
}  // namespace

int tensor_map_2d(void* map_out, int elem_kind, const void* base, uint64_t inner, uint64_t outer,
                  uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(QMM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  if (elem_kind == QMM_BF16) dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  else if (elem_kind == QMM_F16) dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  else if (elem_kind == QMM_U32) dt = CU_TENSOR_MAP_DATA_TYPE_UINT32;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(static_cast<CUtensorMap*>(map_out), dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(QMM_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return QMM_OK;
}

int* device_status_word() {
  static int* ptr = nullptr;  // one word per process, allocated on first use and kept
  if (!ptr) {
    if (cudaMalloc(&ptr, sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(ptr, 0, sizeof(int));
  }
  return ptr;
}

int device_sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

namespace {
thread_local const ScratchBlock* t_scratch = nullptr;
}

const ScratchBlock* scratch_override() { return t_scratch; }
void set_scratch_override(const ScratchBlock* block) { t_scratch = block; }

}  // namespace qmm
