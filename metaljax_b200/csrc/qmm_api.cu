// C ABI of libqmm: argument validation, routing, and the DLPack-view front of every entry
// point declared in include/qmm.h. No kernel code lives here.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "qmm_internal.h"

namespace qmm {

namespace {
thread_local char g_error[512] = "";
std::atomic<uint64_t> g_launches{0};
std::atomic<uint64_t> g_allocs{0};
std::atomic<int> g_route_override{QMM_ROUTE_NONE};
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

void count_launch(int n) { g_launches.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }
void count_alloc(int n) { g_allocs.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }

int route_override() { return g_route_override.load(std::memory_order_relaxed); }

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return QMM_OK;
}

namespace {

// ---- tensor views -------------------------------------------------------------------------

int elem_of(const qmm_tensor* t) {
  if (t->dtype.lanes != 1) return -1;
  switch (t->dtype.code) {
    case 4: return t->dtype.bits == 16 ? QMM_BF16 : -1;
    case 2: return t->dtype.bits == 16 ? QMM_F16 : (t->dtype.bits == 32 ? QMM_F32 : -1);
    case 1: return t->dtype.bits == 8 ? QMM_U8 : (t->dtype.bits == 32 ? QMM_U32 : -1);
    case 0: return t->dtype.bits == 32 ? QMM_I32 : -1;
  }
  return -1;
}

bool is_float_elem(int e) { return e == QMM_BF16 || e == QMM_F16 || e == QMM_F32; }

// Row-major compact (a size-1 dimension may carry any stride).
bool is_compact(const qmm_tensor* t) {
  if (!t->strides) return true;
  int64_t expect = 1;
  for (int d = t->ndim - 1; d >= 0; --d) {
    if (t->shape[d] != 1 && t->strides[d] != expect) return false;
    expect *= t->shape[d];
  }
  return true;
}

void* data_of(const qmm_tensor* t) { return static_cast<char*>(t->data) + t->byte_offset; }

int64_t numel(const qmm_tensor* t) {
  int64_t n = 1;
  for (int d = 0; d < t->ndim; ++d) n *= t->shape[d];
  return n;
}

int check_view(const qmm_tensor* t, const char* name, int min_rank, int max_rank, bool on_device) {
  if (!t) return fail(QMM_ERR_NULL, "%s is NULL", name);
  if (t->ndim < min_rank || t->ndim > max_rank)
    return fail(QMM_ERR_SHAPE, "%s has rank %d, expected %d..%d", name, t->ndim, min_rank, max_rank);
  if (t->ndim > 0 && !t->shape) return fail(QMM_ERR_NULL, "%s has no shape", name);
  for (int d = 0; d < t->ndim; ++d)
    if (t->shape[d] < 0) return fail(QMM_ERR_SHAPE, "%s has a negative extent", name);
  if (!is_compact(t)) return fail(QMM_ERR_LAYOUT, "%s is not row-major contiguous", name);
  if (on_device) {
    if (t->device.device_type != 2)
      return fail(QMM_ERR_DEVICE, "%s is not a CUDA tensor (device type %d)", name,
                  t->device.device_type);
    if (numel(t) > 0 && !t->data) return fail(QMM_ERR_NULL, "%s has no data pointer", name);
    if (reinterpret_cast<uintptr_t>(data_of(t)) % 16)
      return fail(QMM_ERR_LAYOUT, "%s is not 16-byte aligned", name);
  }
  return QMM_OK;
}

int check_same_device(const qmm_tensor* a, const qmm_tensor* b, const char* name) {
  if (b && (a->device.device_type != b->device.device_type || a->device.device_id != b->device.device_id))
    return fail(QMM_ERR_DEVICE, "%s is on a different device than x", name);
  return QMM_OK;
}

int check_quant(int group_size, int bits, int mode) {
  if (mode == QMM_MODE_AFFINE) {
    if (bits != 4 && bits != 8) return fail(QMM_ERR_GROUP, "affine bits=%d (expected 4 or 8)", bits);
    if (group_size != 32 && group_size != 64 && group_size != 128)
      return fail(QMM_ERR_GROUP, "affine group_size=%d (expected 32, 64 or 128)", group_size);
  } else if (mode == QMM_MODE_MXFP4) {
    if (bits != 4 || group_size != 32)
      return fail(QMM_ERR_GROUP, "mxfp4 needs bits=4, group_size=32 (got %d, %d)", bits, group_size);
  } else {
    return fail(QMM_ERR_GROUP, "unknown mode %d", mode);
  }
  return QMM_OK;
}

// Shapes and types of the (w, scales, biases) triple: w [.., N, words], tables [.., N, K/gs].
// Returns K and N through the pointers.
int check_weight(const qmm_tensor* w, const qmm_tensor* scales, const qmm_tensor* biases,
                 int group_size, int bits, int mode, bool on_device, int64_t* K, int64_t* N,
                 int* table_dtype) {
  int rc;
  if ((rc = check_quant(group_size, bits, mode))) return rc;
  if ((rc = check_view(w, "w", 2, 3, on_device))) return rc;
  if ((rc = check_view(scales, "scales", 2, 3, on_device))) return rc;
  if (elem_of(w) != QMM_U32) return fail(QMM_ERR_DTYPE, "w must be uint32");
  const int64_t words = w->shape[w->ndim - 1];
  *N = w->shape[w->ndim - 2];
  if ((words * 32) % bits) return fail(QMM_ERR_SHAPE, "w row of %lld words at %d bits", (long long)words, bits);
  *K = words * 32 / bits;
  if (*K % group_size)
    return fail(QMM_ERR_GROUP, "K=%lld is not a multiple of group_size=%d", (long long)*K, group_size);
  const int st = elem_of(scales);
  if (mode == QMM_MODE_MXFP4) {
    if (st != QMM_U8) return fail(QMM_ERR_DTYPE, "mxfp4 scales must be uint8 (E8M0)");
    if (biases) return fail(QMM_ERR_GROUP, "mxfp4 takes no bias table");
  } else {
    if (!is_float_elem(st)) return fail(QMM_ERR_DTYPE, "affine scales must be bf16, f16 or f32");
    if (!biases) return fail(QMM_ERR_NULL, "affine mode needs a bias table");
    if ((rc = check_view(biases, "biases", 2, 3, on_device))) return rc;
    if (elem_of(biases) != st) return fail(QMM_ERR_DTYPE, "biases and scales differ in type");
    if (biases->ndim != scales->ndim) return fail(QMM_ERR_SHAPE, "biases and scales differ in rank");
    for (int d = 0; d < scales->ndim; ++d)
      if (biases->shape[d] != scales->shape[d])
        return fail(QMM_ERR_SHAPE, "biases and scales differ in shape");
  }
  *table_dtype = st;
  if (scales->ndim != w->ndim) return fail(QMM_ERR_SHAPE, "scales and w differ in rank");
  if (scales->shape[scales->ndim - 2] != *N || scales->shape[scales->ndim - 1] != *K / group_size)
    return fail(QMM_ERR_SHAPE, "scales are not [.., N=%lld, K/group_size=%lld]", (long long)*N,
                (long long)(*K / group_size));
  if (w->ndim == 3 && scales->shape[0] != w->shape[0])
    return fail(QMM_ERR_SHAPE, "scales and w differ in batch");
  return QMM_OK;
}

int validate_problem(const qmm_problem& p, bool pointers) {
  int rc;
  if (p.struct_size != sizeof(qmm_problem))
    return fail(QMM_ERR_UNSUPPORTED, "qmm_problem.struct_size=%u, library expects %zu", p.struct_size,
                sizeof(qmm_problem));
  if ((rc = check_quant(p.group_size, p.bits, p.mode))) return rc;
  if (!is_float_elem(p.x_dtype)) return fail(QMM_ERR_DTYPE, "x must be bf16, f16 or f32");
  if (!is_float_elem(p.y_dtype)) return fail(QMM_ERR_DTYPE, "y must be bf16, f16 or f32");
  if (p.mode == QMM_MODE_MXFP4 ? p.table_dtype != QMM_U8 : !is_float_elem(p.table_dtype))
    return fail(QMM_ERR_DTYPE, "table dtype %d does not fit mode %d", p.table_dtype, p.mode);
  if (p.batch < 0 || p.M < 0 || p.N < 0 || p.K < 0) return fail(QMM_ERR_SHAPE, "negative extent");
  if (p.K % p.group_size)
    return fail(QMM_ERR_GROUP, "K=%lld is not a multiple of group_size=%d", (long long)p.K, p.group_size);
  if ((p.lhs_idx != nullptr) != (p.rhs_idx != nullptr))
    return fail(QMM_ERR_NULL, "gather needs both lhs_idx and rhs_idx");
  if (p.group_sizes && p.lhs_idx) return fail(QMM_ERR_UNSUPPORTED, "ragged and gather are exclusive");
  if (p.num_weights < 0 || (p.lhs_idx && p.num_weights < 1 && pointers))
    return fail(QMM_ERR_SHAPE, "a gather needs num_weights (the number of experts behind w)");
  if (pointers && p.batch * p.M * p.N * p.K > 0) {
    if (!p.x || !p.w || !p.scales || !p.y) return fail(QMM_ERR_NULL, "a data pointer is NULL");
    if (p.mode == QMM_MODE_AFFINE && !p.biases) return fail(QMM_ERR_NULL, "affine mode needs biases");
    const void* ptrs[] = {p.x, p.w, p.scales, p.biases, p.y};
    for (const void* q : ptrs)
      if (reinterpret_cast<uintptr_t>(q) % 16) return fail(QMM_ERR_LAYOUT, "a data pointer is not 16-byte aligned");
    if ((p.x_batch_stride * elem_size(p.x_dtype)) % 16)
      return fail(QMM_ERR_LAYOUT, "x batches are not 16-byte aligned");
  }
  return QMM_OK;
}

int route_of(const qmm_problem& p) {
  if (p.batch == 0 || p.M == 0 || p.N == 0) return QMM_ROUTE_NONE;
  const int forced = g_route_override.load(std::memory_order_relaxed);
  if (forced == QMM_ROUTE_GEMV || forced == QMM_ROUTE_GEMV_FMMA) return gemv_supports(p) ? QMM_ROUTE_GEMV : -QMM_ERR_UNSUPPORTED;
  if (forced == QMM_ROUTE_GEMM_TC) return gemm_tc_supports(p) ? forced : -QMM_ERR_UNSUPPORTED;
  if (forced == QMM_ROUTE_SIMT) return forced;
  // More than 8 rows against a long K (the activations no longer fit next to the decode
  // kernel's rings) go to the tensor-core kernel, whose K split then fills the machine.
  const bool long_k = p.M > 8 && p.K >= 8192 && p.batch == 1 && !p.lhs_idx && gemm_tc_supports(p);
  if (gemv_supports(p) && !long_k) return QMM_ROUTE_GEMV;
  if (gemm_tc_supports(p)) return QMM_ROUTE_GEMM_TC;
  return QMM_ROUTE_SIMT;
}

int zero_fill(void* y, int64_t bytes, cudaStream_t stream) {
  if (bytes <= 0) return QMM_OK;
  cudaError_t e = cudaMemsetAsync(y, 0, static_cast<size_t>(bytes), stream);
  if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
  return QMM_OK;
}

int launch_problem(const qmm_problem& p, cudaStream_t stream) {
  if (p.K == 0 && p.batch * p.M * p.N > 0) {  // an empty contraction is a zero result
    const int64_t rows = p.group_sizes ? p.M : p.batch * p.M;
    return zero_fill(p.y, rows * p.N * elem_size(p.y_dtype), stream);
  }
  const int route = route_of(p);
  if (route < 0) return fail(-route, "the forced kernel family does not support this problem");
  switch (route) {
    case QMM_ROUTE_NONE: return QMM_OK;
    case QMM_ROUTE_GEMV: return launch_gemv(p, stream);
    case QMM_ROUTE_GEMM_TC: return launch_gemm_tc(p, stream);
    default: return launch_simt(p, stream);
  }
}

void init_problem(qmm_problem* p) {
  memset(p, 0, sizeof(*p));
  p->struct_size = sizeof(*p);
}

// x [M,K] | [B,M,K] against w [N,words] | [B,N,words]; y matches x.
int build_dense(const qmm_tensor* x, const qmm_tensor* w, const qmm_tensor* scales,
                const qmm_tensor* biases, const qmm_tensor* y, int transpose, int group_size,
                int bits, int mode, bool on_device, qmm_problem* p) {
  int rc;
  if (transpose != 1)
    return fail(QMM_ERR_UNSUPPORTED, "transpose=%d: only transpose=1 (y = x . w^T) is provided", transpose);
  int64_t K, N;
  int tdt;
  if ((rc = check_view(x, "x", 2, 3, on_device))) return rc;
  if ((rc = check_view(y, "y", 2, 3, on_device))) return rc;
  if ((rc = check_weight(w, scales, biases, group_size, bits, mode, on_device, &K, &N, &tdt))) return rc;
  if (on_device) {
    if ((rc = check_same_device(x, w, "w")) || (rc = check_same_device(x, scales, "scales")) ||
        (rc = check_same_device(x, biases, "biases")) || (rc = check_same_device(x, y, "y")))
      return rc;
  }
  const int xe = elem_of(x), ye = elem_of(y);
  if (!is_float_elem(xe)) return fail(QMM_ERR_DTYPE, "x must be bf16, f16 or f32");
  if (!is_float_elem(ye)) return fail(QMM_ERR_DTYPE, "y must be bf16, f16 or f32");
  if (x->shape[x->ndim - 1] != K)
    return fail(QMM_ERR_SHAPE, "x has K=%lld, the packed weight has K=%lld",
                (long long)x->shape[x->ndim - 1], (long long)K);
  const int64_t M = x->shape[x->ndim - 2];
  const int64_t B = x->ndim == 3 ? x->shape[0] : 1;
  if (y->ndim != x->ndim) return fail(QMM_ERR_SHAPE, "y and x differ in rank");
  if (y->shape[y->ndim - 1] != N || y->shape[y->ndim - 2] != M || (y->ndim == 3 && y->shape[0] != B))
    return fail(QMM_ERR_SHAPE, "y is not [%s M=%lld, N=%lld]", x->ndim == 3 ? "B," : "", (long long)M,
                (long long)N);
  if (w->ndim == 3 && (x->ndim != 3 || w->shape[0] != B))
    return fail(QMM_ERR_SHAPE, "a batched weight needs x with the same leading extent");
  init_problem(p);
  p->mode = mode; p->bits = bits; p->group_size = group_size;
  p->x_dtype = xe; p->table_dtype = tdt; p->y_dtype = ye;
  p->K = K; p->N = N;
  p->x = data_of(x); p->w = static_cast<const uint32_t*>(data_of(w));
  p->scales = data_of(scales); p->biases = biases ? data_of(biases) : nullptr;
  p->y = data_of(y);
  if (w->ndim == 3) {
    p->batch = B; p->M = M;
    p->x_batch_stride = M * K; p->y_batch_stride = M * N; p->w_batch_stride = N;
  } else {  // a shared weight: the batches of x are just more rows
    p->batch = 1; p->M = B * M;
    p->x_batch_stride = p->M * K; p->y_batch_stride = p->M * N; p->w_batch_stride = 0;
  }
  return QMM_OK;
}

}  // namespace
}  // namespace qmm

namespace qmm {
int check_problem(const qmm_problem& p) { return validate_problem(p, true); }
}  // namespace qmm

using namespace qmm;

// ---- the entry point that allocates nothing ------------------------------------------------
// The tensor-core kernel divides the K blocks of a short, narrow product among several CTAs and
// needs float32 scratch for their partial tiles. The ordinary entry points take that scratch
// from the stream-ordered allocator; this one takes it from a fixed block of device memory that
// is part of the library image, so that it can be called where allocating is not an option.
constexpr size_t kStaticScratchBytes = 8u << 20;      // 8 MiB: the stated maximum
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {

// Address of the block on the current device, looked up once per device. The last 256 bytes
// hold the status word of the calls made through this entry point (zero at load, like the
// whole block; nothing else in the block has to start at any particular value: every partial
// sum is written before it is read).
void* g_static_base[qmm::kMaxDevices] = {};     // the block's address on each device, once looked up

int static_scratch(qmm::ScratchBlock* out) {
  const int dev = qmm::current_device();
  if (dev < 0) return QMM_ERR_DEVICE;
  if (!g_static_base[dev]) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch);
    if (e != cudaSuccess || !ptr)
      return qmm::fail(QMM_ERR_CUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
    g_static_base[dev] = ptr;
  }
  out->ptr = g_static_base[dev];
  out->bytes = kStaticScratchBytes - 256;
  out->status = reinterpret_cast<int*>(static_cast<unsigned char*>(g_static_base[dev]) + kStaticScratchBytes - 256);
  return QMM_OK;
}

// Reads, and clears if set, the status word in the static block of the current device. Zero
// when the block has never been used there. A plain cudaMemcpy from the block: no allocation.
int read_static_status(int* out) {
  *out = 0;
  const int dev = qmm::current_device();
  if (dev < 0) return QMM_ERR_DEVICE;
  if (!g_static_base[dev]) return QMM_OK;
  int* word = reinterpret_cast<int*>(static_cast<unsigned char*>(g_static_base[dev]) + kStaticScratchBytes - 256);
  cudaError_t e = cudaMemcpy(out, word, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return qmm::fail(QMM_ERR_CUDA, "cudaMemcpy(static status): %s", cudaGetErrorString(e));
  if (*out) cudaMemset(word, 0, sizeof(int));
  return QMM_OK;
}

}  // namespace

extern "C" int qmm_quantized_matmul_static(const qmm_tensor* x, const qmm_tensor* w, const qmm_tensor* scales,
                                           const qmm_tensor* biases, qmm_tensor* y, int transpose, int group_size,
                                           int bits, int mode, void* stream) {
  using namespace qmm;
  qmm_problem p;
  int rc = build_dense(x, w, scales, biases, y, transpose, group_size, bits, mode, true, &p);
  if (rc) return rc;
  if ((rc = validate_problem(p, true))) return rc;
  if (p.K == 0 || p.batch * p.M * p.N == 0 || !gemm_tc_supports(p))
    return fail(QMM_ERR_UNSUPPORTED,
                "qmm_quantized_matmul_static runs the tensor-core kernel only: 16-bit activations, K >= 64, "
                "a non-empty product");
  ScratchBlock block;
  if ((rc = static_scratch(&block))) return rc;
  set_scratch_override(&block);
  rc = launch_gemm_tc(p, static_cast<cudaStream_t>(stream));
  set_scratch_override(nullptr);
  return rc;
}

extern "C" {

int qmm_version(void) { return QMM_VERSION; }

const char* qmm_last_error(void) { return g_error; }

int qmm_set_route_override(int route) {
  if (route < QMM_ROUTE_NONE || route > QMM_ROUTE_GEMV_FMMA) return fail(QMM_ERR_UNSUPPORTED, "unknown route %d", route);
  g_route_override.store(route, std::memory_order_relaxed);
  return QMM_OK;
}

int qmm_poll_status(int* status_out) {
  int st = 0, st_static = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
  int rc = read_status_word(&st);
  if (rc) return rc;
  if ((rc = read_static_status(&st_static))) return rc;
  if (!st) st = st_static;
  if (status_out) *status_out = st;
  if (st == QMM_DEVICE_BAD_INDEX) return fail(QMM_ERR_SHAPE, "a gather index was out of range (that pair used index 0)");
  if (st) return fail(QMM_ERR_TIMEOUT, "a device-side wait ran out (code %d)", st);
  return QMM_OK;
}

int qmm_poll_status_static(int* status_out) {
  int st = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
  int rc = read_static_status(&st);
  if (rc) return rc;
  if (status_out) *status_out = st;
  if (st) return fail(QMM_ERR_TIMEOUT, "a device-side wait of qmm_quantized_matmul_static ran out (code %d)", st);
  return QMM_OK;
}

int qmm_set_wait_limit(long long clocks) {
  if (clocks < 1000) return fail(QMM_ERR_UNSUPPORTED, "wait limit of %lld clocks is too short", clocks);
  set_wait_limit_clocks(clocks);
  return QMM_OK;
}

uint64_t qmm_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

uint64_t qmm_alloc_count(void) { return g_allocs.load(std::memory_order_relaxed); }

int qmm_launch(const qmm_problem* problem, void* stream) {
  if (!problem) return fail(QMM_ERR_NULL, "problem is NULL");
  int rc = validate_problem(*problem, true);
  if (rc) return rc;
  return launch_problem(*problem, static_cast<cudaStream_t>(stream));
}

int qmm_route(const qmm_problem* problem) {
  if (!problem) return -fail(QMM_ERR_NULL, "problem is NULL");
  int rc = validate_problem(*problem, false);
  if (rc) return -rc;
  const int route = route_of(*problem);
  if (route < 0) fail(-route, "the forced kernel family does not support this problem");
  return route;
}

int qmm_check_quantized_matmul(const qmm_tensor* x, const qmm_tensor* w, const qmm_tensor* scales,
                               const qmm_tensor* biases, const qmm_tensor* y, int transpose,
                               int group_size, int bits, int mode) {
  qmm_problem p;
  return build_dense(x, w, scales, biases, y, transpose, group_size, bits, mode, false, &p);
}

int qmm_quantized_matmul(const qmm_tensor* x, const qmm_tensor* w, const qmm_tensor* scales,
                         const qmm_tensor* biases, qmm_tensor* y, int transpose, int group_size,
                         int bits, int mode, void* stream) {
  qmm_problem p;
  int rc = build_dense(x, w, scales, biases, y, transpose, group_size, bits, mode, true, &p);
  if (rc) return rc;
  if ((rc = validate_problem(p, true))) return rc;
  return launch_problem(p, static_cast<cudaStream_t>(stream));
}

int qmm_gather_qmm(const qmm_tensor* x, const qmm_tensor* w, const qmm_tensor* scales,
                   const qmm_tensor* biases, const qmm_tensor* lhs_idx, const qmm_tensor* rhs_idx,
                   qmm_tensor* y, int transpose, int group_size, int bits, int mode, void* stream) {
  int rc;
  if (transpose != 1) return fail(QMM_ERR_UNSUPPORTED, "transpose=%d: only transpose=1 is provided", transpose);
  int64_t K, N;
  int tdt;
  if ((rc = check_view(x, "x", 3, 3, true))) return rc;
  if ((rc = check_view(y, "y", 3, 3, true))) return rc;
  if ((rc = check_view(lhs_idx, "lhs_idx", 1, 1, true))) return rc;
  if ((rc = check_view(rhs_idx, "rhs_idx", 1, 1, true))) return rc;
  if ((rc = check_weight(w, scales, biases, group_size, bits, mode, true, &K, &N, &tdt))) return rc;
  if (w->ndim != 3) return fail(QMM_ERR_SHAPE, "gather needs w [E, N, words]");
  if ((rc = check_same_device(x, w, "w")) || (rc = check_same_device(x, scales, "scales")) ||
      (rc = check_same_device(x, biases, "biases")) || (rc = check_same_device(x, y, "y")) ||
      (rc = check_same_device(x, lhs_idx, "lhs_idx")) || (rc = check_same_device(x, rhs_idx, "rhs_idx")))
    return rc;
  const int le = elem_of(lhs_idx), re = elem_of(rhs_idx);
  if ((le != QMM_U32 && le != QMM_I32) || (re != QMM_U32 && re != QMM_I32))
    return fail(QMM_ERR_DTYPE, "lhs_idx / rhs_idx must be 32-bit integers");
  const int64_t P = lhs_idx->shape[0];
  if (rhs_idx->shape[0] != P) return fail(QMM_ERR_SHAPE, "lhs_idx and rhs_idx differ in length");
  const int xe = elem_of(x), ye = elem_of(y);
  if (!is_float_elem(xe) || !is_float_elem(ye)) return fail(QMM_ERR_DTYPE, "x and y must be bf16, f16 or f32");
  if (x->shape[2] != K) return fail(QMM_ERR_SHAPE, "x has K=%lld, the packed weight has K=%lld",
                                    (long long)x->shape[2], (long long)K);
  const int64_t M = x->shape[1];
  if (y->shape[0] != P || y->shape[1] != M || y->shape[2] != N)
    return fail(QMM_ERR_SHAPE, "y is not [P=%lld, M=%lld, N=%lld]", (long long)P, (long long)M, (long long)N);
  qmm_problem p;
  init_problem(&p);
  p.mode = mode; p.bits = bits; p.group_size = group_size;
  p.x_dtype = xe; p.table_dtype = tdt; p.y_dtype = ye;
  p.batch = P; p.M = M; p.K = K; p.N = N;
  p.x = data_of(x); p.w = static_cast<const uint32_t*>(data_of(w));
  p.scales = data_of(scales); p.biases = biases ? data_of(biases) : nullptr; p.y = data_of(y);
  p.x_batch_stride = M * K; p.y_batch_stride = M * N; p.w_batch_stride = N;
  p.num_weights = static_cast<int32_t>(w->shape[0]);
  p.x_batches = x->shape[0];
  p.lhs_idx = static_cast<const int32_t*>(data_of(lhs_idx));
  p.rhs_idx = static_cast<const int32_t*>(data_of(rhs_idx));
  if ((rc = validate_problem(p, true))) return rc;
  return launch_problem(p, static_cast<cudaStream_t>(stream));
}

int qmm_ragged_dot(const qmm_tensor* x, const qmm_tensor* w, const qmm_tensor* scales,
                   const qmm_tensor* biases, const qmm_tensor* group_sizes, qmm_tensor* y,
                   int group_size, int bits, int mode, void* stream) {
  int rc;
  int64_t K, N;
  int tdt;
  if ((rc = check_view(x, "x", 2, 2, true))) return rc;
  if ((rc = check_view(y, "y", 2, 2, true))) return rc;
  if ((rc = check_view(group_sizes, "group_sizes", 1, 1, true))) return rc;
  if ((rc = check_weight(w, scales, biases, group_size, bits, mode, true, &K, &N, &tdt))) return rc;
  if (w->ndim != 3) return fail(QMM_ERR_SHAPE, "ragged_dot needs w [G, N, words]");
  if ((rc = check_same_device(x, w, "w")) || (rc = check_same_device(x, scales, "scales")) ||
      (rc = check_same_device(x, biases, "biases")) || (rc = check_same_device(x, y, "y")) ||
      (rc = check_same_device(x, group_sizes, "group_sizes")))
    return rc;
  if (elem_of(group_sizes) != QMM_I32) return fail(QMM_ERR_DTYPE, "group_sizes must be int32");
  if (group_sizes->shape[0] != w->shape[0])
    return fail(QMM_ERR_SHAPE, "group_sizes has %lld entries for %lld experts",
                (long long)group_sizes->shape[0], (long long)w->shape[0]);
  const int xe = elem_of(x), ye = elem_of(y);
  if (!is_float_elem(xe) || !is_float_elem(ye)) return fail(QMM_ERR_DTYPE, "x and y must be bf16, f16 or f32");
  if (x->shape[1] != K) return fail(QMM_ERR_SHAPE, "x has K=%lld, the packed weight has K=%lld",
                                    (long long)x->shape[1], (long long)K);
  if (y->shape[0] != x->shape[0] || y->shape[1] != N)
    return fail(QMM_ERR_SHAPE, "y is not [M=%lld, N=%lld]", (long long)x->shape[0], (long long)N);
  qmm_problem p;
  init_problem(&p);
  p.mode = mode; p.bits = bits; p.group_size = group_size;
  p.x_dtype = xe; p.table_dtype = tdt; p.y_dtype = ye;
  p.batch = w->shape[0]; p.M = x->shape[0]; p.K = K; p.N = N;
  p.x = data_of(x); p.w = static_cast<const uint32_t*>(data_of(w));
  p.scales = data_of(scales); p.biases = biases ? data_of(biases) : nullptr; p.y = data_of(y);
  p.w_batch_stride = N;
  p.group_sizes = static_cast<const int32_t*>(data_of(group_sizes));
  if ((rc = validate_problem(p, true))) return rc;
  return launch_problem(p, static_cast<cudaStream_t>(stream));
}

int qmm_ragged_mm(const qmm_tensor* x, const qmm_tensor* w, const qmm_tensor* group_sizes, qmm_tensor* y,
                  void* stream) {
  int rc;
  if ((rc = check_view(x, "x", 2, 2, true))) return rc;
  if ((rc = check_view(y, "y", 2, 2, true))) return rc;
  if ((rc = check_view(w, "w", 3, 3, true))) return rc;
  if ((rc = check_view(group_sizes, "group_sizes", 1, 1, true))) return rc;
  if ((rc = check_same_device(x, w, "w")) || (rc = check_same_device(x, y, "y")) ||
      (rc = check_same_device(x, group_sizes, "group_sizes")))
    return rc;
  if (elem_of(group_sizes) != QMM_I32) return fail(QMM_ERR_DTYPE, "group_sizes must be int32");
  const int xe = elem_of(x), ye = elem_of(y);
  if ((xe != QMM_BF16 && xe != QMM_F16) || elem_of(w) != xe)
    return fail(QMM_ERR_DTYPE, "ragged_mm: x and w must both be bf16 or both f16");
  if (!is_float_elem(ye)) return fail(QMM_ERR_DTYPE, "y must be bf16, f16 or f32");
  const int64_t K = w->shape[2], N = w->shape[1];
  if (group_sizes->shape[0] != w->shape[0])
    return fail(QMM_ERR_SHAPE, "group_sizes has %lld entries for %lld experts", (long long)group_sizes->shape[0],
                (long long)w->shape[0]);
  if (x->shape[1] != K) return fail(QMM_ERR_SHAPE, "x has K=%lld, the weight has K=%lld", (long long)x->shape[1], (long long)K);
  if (y->shape[0] != x->shape[0] || y->shape[1] != N)
    return fail(QMM_ERR_SHAPE, "y is not [M=%lld, N=%lld]", (long long)x->shape[0], (long long)N);
  qmm_problem p;
  init_problem(&p);
  p.mode = QMM_MODE_FLOAT; p.bits = 16; p.group_size = 64;      // (no groups: the kernel's K block)
  p.x_dtype = xe; p.table_dtype = xe; p.y_dtype = ye;
  p.batch = w->shape[0]; p.M = x->shape[0]; p.K = K; p.N = N;
  p.x = data_of(x); p.w = static_cast<const uint32_t*>(data_of(w)); p.y = data_of(y);
  p.w_batch_stride = N;
  p.group_sizes = static_cast<const int32_t*>(data_of(group_sizes));
  if (p.batch == 0 || p.M == 0 || p.N == 0) return QMM_OK;
  if (K == 0) return zero_fill(p.y, p.M * p.N * elem_size(ye), static_cast<cudaStream_t>(stream));
  if ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.w) | reinterpret_cast<uintptr_t>(p.y)) & 15)
    return fail(QMM_ERR_LAYOUT, "a data pointer is not 16-byte aligned");
  if (!gemm_tc_supports(p))
    return fail(QMM_ERR_UNSUPPORTED, "ragged_mm: K=%lld must be at least 64 and a multiple of 8, at most %d experts",
                (long long)K, 1024);
  return launch_gemm_tc(p, static_cast<cudaStream_t>(stream));
}

int qmm_dequantize(const qmm_tensor* w, const qmm_tensor* scales, const qmm_tensor* biases,
                   qmm_tensor* out, int group_size, int bits, int mode, void* stream) {
  int rc;
  int64_t K, N;
  int tdt;
  if ((rc = check_weight(w, scales, biases, group_size, bits, mode, true, &K, &N, &tdt))) return rc;
  if ((rc = check_view(out, "out", 2, 3, true))) return rc;
  if ((rc = check_same_device(w, scales, "scales")) || (rc = check_same_device(w, biases, "biases")) ||
      (rc = check_same_device(w, out, "out")))
    return rc;
  const int oe = elem_of(out);
  if (!is_float_elem(oe)) return fail(QMM_ERR_DTYPE, "out must be bf16, f16 or f32");
  if (out->ndim != w->ndim || out->shape[out->ndim - 1] != K || out->shape[out->ndim - 2] != N ||
      (w->ndim == 3 && out->shape[0] != w->shape[0]))
    return fail(QMM_ERR_SHAPE, "out is not [.., N=%lld, K=%lld]", (long long)N, (long long)K);
  const int64_t rows = (w->ndim == 3 ? w->shape[0] : 1) * N;
  return launch_dequantize(static_cast<const uint32_t*>(data_of(w)), data_of(scales),
                           biases ? data_of(biases) : nullptr, tdt, data_of(out), oe, rows, K,
                           group_size, bits, mode, static_cast<cudaStream_t>(stream));
}

int qmm_pack_codes(const qmm_tensor* codes, qmm_tensor* out, int bits, void* stream) {
  int rc;
  if (bits != 4 && bits != 8) return fail(QMM_ERR_GROUP, "pack_codes: bits=%d (expected 4 or 8)", bits);
  if ((rc = check_view(codes, "codes", 1, 4, true))) return rc;
  if ((rc = check_view(out, "out", 1, 4, true))) return rc;
  if ((rc = check_same_device(codes, out, "out"))) return rc;
  if (elem_of(codes) != QMM_U8) return fail(QMM_ERR_DTYPE, "codes must be uint8");
  if (elem_of(out) != QMM_U32) return fail(QMM_ERR_DTYPE, "out must be uint32");
  if (codes->ndim != out->ndim) return fail(QMM_ERR_SHAPE, "codes and out differ in rank");
  const int64_t K = codes->shape[codes->ndim - 1];
  const int per = 32 / bits;
  if (K % per) return fail(QMM_ERR_SHAPE, "pack_codes: K=%lld not a multiple of %d", (long long)K, per);
  if (out->shape[out->ndim - 1] != K / per) return fail(QMM_ERR_SHAPE, "out row is not K*bits/32 words");
  int64_t rows = 1;
  for (int d = 0; d + 1 < codes->ndim; ++d) {
    if (codes->shape[d] != out->shape[d]) return fail(QMM_ERR_SHAPE, "codes and out differ in shape");
    rows *= codes->shape[d];
  }
  return launch_pack_codes(static_cast<const uint8_t*>(data_of(codes)),
                           static_cast<uint32_t*>(data_of(out)), rows, K, bits,
                           static_cast<cudaStream_t>(stream));
}

}  // extern "C"
