// Host-side helpers shared by the kernel launchers: tensor-map encoding through the driver
// entry point (no link-time dependency on libcuda), the device status word, device facts.
#include <cuda.h>

#include <atomic>
#include <mutex>

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

int current_device() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    fail(QMM_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    return -1;
  }
  if (dev < 0 || dev >= kMaxDevices) {
    fail(QMM_ERR_DEVICE, "device ordinal %d is out of range", dev);
    return -1;
  }
  return dev;
}

namespace {
std::mutex g_device_mutex;
int* g_status_word[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};
std::atomic<long long> g_wait_limit{4000000000LL};
}  // namespace

int* device_status_word() {
  const int dev = current_device();
  if (dev < 0) return nullptr;
  std::lock_guard<std::mutex> lock(g_device_mutex);
  if (!g_status_word[dev]) {
    int* ptr = nullptr;
    if (cudaMalloc(&ptr, sizeof(int)) != cudaSuccess) return nullptr;
    count_alloc();
    cudaMemset(ptr, 0, sizeof(int));
    g_status_word[dev] = ptr;
  }
  return g_status_word[dev];
}

int read_status_word(int* out) {
  int* w = device_status_word();
  if (!w) return fail(QMM_ERR_CUDA, "no status word");
  cudaError_t e = cudaMemcpy(out, w, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "cudaMemcpy(status): %s", cudaGetErrorString(e));
  if (*out) cudaMemset(w, 0, sizeof(int));
  return QMM_OK;
}

int device_sm_count() {
  const int dev = current_device();
  if (dev < 0) return 148;
  std::lock_guard<std::mutex> lock(g_device_mutex);
  if (!g_sm_count[dev]) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    g_sm_count[dev] = n > 0 ? n : 148;
  }
  return g_sm_count[dev];
}

long long wait_limit_clocks() { return g_wait_limit.load(std::memory_order_relaxed); }
void set_wait_limit_clocks(long long clocks) { g_wait_limit.store(clocks, std::memory_order_relaxed); }

namespace {
thread_local const ScratchBlock* t_scratch = nullptr;
}

const ScratchBlock* scratch_override() { return t_scratch; }
void set_scratch_override(const ScratchBlock* block) { t_scratch = block; }

}  // namespace qmm

#if QMM_STEP_TRACING
namespace qmm {
namespace {
unsigned long long* g_trace_base = nullptr;
int64_t g_trace_blocks = 0, g_trace_next = 0;
int* g_trace_kinds = nullptr;
}  // namespace
unsigned long long* next_trace_block(int kind) {
  if (!g_trace_base || g_trace_next >= g_trace_blocks) return nullptr;
  if (g_trace_kinds) g_trace_kinds[g_trace_next] = kind;
  return g_trace_base + (g_trace_next++) * kTraceStamps * kTraceCtas;
}
}  // namespace qmm
// `buf`: device memory of blocks * 16 * 512 uint64, zeroed by the caller; `kinds`: host ints, one per block.
extern "C" void qmm_debug_set_trace(void* buf, int64_t blocks, int* kinds) {
  qmm::g_trace_base = static_cast<unsigned long long*>(buf);
  qmm::g_trace_blocks = blocks;
  qmm::g_trace_next = 0;
  qmm::g_trace_kinds = kinds;
}
extern "C" int64_t qmm_debug_trace_count() { return qmm::g_trace_next; }
#endif
