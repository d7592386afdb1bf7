// Dispatch and combine of an expert-parallel mixture-of-experts block over peer memory.
//
// Every rank routes its own tokens; expert e lives on rank e / (experts / world). Instead of two
// rounds of all-to-all (sizes, then rows) with the sizes read back by the host in between, the
// ranks write straight into each other's memory (plain stores over NVLink into buffers every
// rank has mapped: torch symmetric memory in the Python host; no multimem, no TMA multicast):
//
//   counts    every rank stores its pairs-per-expert table into every rank as 8-byte units
//             {count, stamp}: data and "it has arrived" in one store
//   dispatch  with everybody's counts, a rank knows where each of its rows goes in the owner's
//             receive buffer -- rows are laid out (local expert, source rank, source order), which
//             is what the grouped product wants -- and stores the rows there, gathering them from
//             x by token index on the way; then it raises a flag on every rank
//   combine   after the expert products, a rank stores every result row back into its source's
//             return buffer at the row's position in the source's own sorted pair order
//
// The group sizes of the grouped product are computed on the device from the counts: nothing
// goes through the host, so the whole block can sit in a CUDA graph. Every wait is bounded and
// reports through the status word (code 110..112); a row that would fall outside a buffer is
// dropped and reported (QMM_DEVICE_BAD_INDEX). The reference is single-device: no counterpart.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qmm_ep.h"
#include "qmm_internal.h"

namespace qmm {
namespace {

constexpr int kEpThreads = 256;
constexpr int kEpMaxExperts = 256;
constexpr int kEpMaxWorld = 8;

struct EpParams {
  uint2* peer_counts[kEpMaxWorld];      // [world][experts] {count, stamp} on every rank
  uint32_t* peer_flags[kEpMaxWorld];    // [2][world] on every rank
  uint8_t* peer_recv[kEpMaxWorld];
  uint8_t* peer_ret[kEpMaxWorld];
  uint32_t* epoch;
  uint32_t* scratch;                    // [0] CTAs done (dispatch), [1] CTAs done (combine)
  int* status;
  long long spin_limit;
  int64_t capacity_rows, max_pairs, row_bytes;
  int rank, world, experts;
};

// This rank's counts to every rank (its row of their tables); starts a new call.
__global__ void ep_counts_kernel(const EpParams p, const int32_t* __restrict__ counts) {
  __shared__ uint32_t stamp;
  if (threadIdx.x == 0) {
    stamp = *p.epoch + 1;
    *p.epoch = stamp;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < p.world * p.experts; i += blockDim.x) {
    const int r = i / p.experts, e = i - r * p.experts;
    p.peer_counts[r][p.rank * p.experts + e] = make_uint2(static_cast<uint32_t>(counts[e]), stamp);
  }
}

// Everybody's counts into shared memory (bounded wait on the stamps). Returns false on a timeout.
__device__ bool load_counts(const EpParams& p, uint32_t stamp, int (*cnt)[kEpMaxExperts]) {
  const uint2* mine = p.peer_counts[p.rank];
  auto read = [&](int i) -> uint2 {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(mine + i) : "memory");
    return v;
  };
  bool ok = true;
  for (int i = threadIdx.x; i < p.world * p.experts; i += blockDim.x) {
    uint2 v = read(i);
    long long t0 = 0;
    int spins = 0;
    while (v.y != stamp) {
      if (++spins >= 64) {
        if (*reinterpret_cast<volatile int*>(p.status) != 0) { ok = false; break; }
        if (t0 == 0) t0 = clock64();
        else if (clock64() - t0 > p.spin_limit) {
          atomicCAS(p.status, 0, 110);
          ok = false;
          break;
        }
      }
      v = read(i);
    }
    cnt[i / p.experts][i % p.experts] = ok ? static_cast<int>(v.x) : 0;
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// Copies one row (16-byte pieces) with the whole CTA.
__device__ __forceinline__ void copy_row(uint8_t* dst, const uint8_t* src, int64_t row_bytes) {
  const int pieces = static_cast<int>(row_bytes / 16);
  for (int c = threadIdx.x; c < pieces; c += blockDim.x)
    reinterpret_cast<uint4*>(dst)[c] = __ldg(reinterpret_cast<const uint4*>(src) + c);
}

// The last CTA of a grid to get here raises flag `which` (stamped) on every rank.
__device__ void finish_and_flag(const EpParams& p, uint32_t stamp, int which) {
  __threadfence_system();
  __syncthreads();
  __shared__ int last;
  if (threadIdx.x == 0) {
    last = atomicAdd(&p.scratch[which], 1u) == gridDim.x - 1;
    if (last) p.scratch[which] = 0;
  }
  __syncthreads();
  if (last && threadIdx.x < p.world) {
    __threadfence_system();
    *reinterpret_cast<volatile uint32_t*>(&p.peer_flags[threadIdx.x][which * p.world + p.rank]) = stamp;
  }
}

// x rows (gathered by token) into the owners' receive buffers; the local group sizes.
__global__ void ep_dispatch_kernel(const EpParams p, const uint8_t* __restrict__ x, const int64_t* __restrict__ token_of_row,
                                   int64_t pairs, int64_t tokens, int32_t* __restrict__ group_sizes) {
  __shared__ int cnt[kEpMaxWorld][kEpMaxExperts];
  __shared__ int my_off[kEpMaxExperts + 1];        // first sorted row of this rank for expert e
  __shared__ int dest_base[kEpMaxExperts];         // where this rank's rows for expert e start in the owner's buffer
  const uint32_t stamp = *reinterpret_cast<volatile uint32_t*>(p.epoch);
  const int el = p.experts / p.world;
  const bool ok = load_counts(p, stamp, cnt);
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < p.experts; ++e) {
      my_off[e] = acc;
      acc += cnt[p.rank][e];
    }
    my_off[p.experts] = acc;
  }
  for (int e = threadIdx.x; e < p.experts; e += blockDim.x) {
    const int r = e / el, le = e - r * el;
    int base = 0;
    for (int l2 = 0; l2 < le; ++l2)
      for (int s = 0; s < p.world; ++s) base += cnt[s][r * el + l2];
    for (int s = 0; s < p.rank; ++s) base += cnt[s][e];
    dest_base[e] = base;
    if (blockIdx.x == 0 && r == p.rank) {
      int total = 0;
      for (int s = 0; s < p.world; ++s) total += cnt[s][e];
      group_sizes[le] = ok ? total : 0;
    }
  }
  __syncthreads();
  if (ok) {
    const int64_t mine = my_off[p.experts] < pairs ? my_off[p.experts] : pairs;
    for (int64_t i = blockIdx.x; i < mine; i += gridDim.x) {
      int lo = 0, hi = p.experts;                    // the expert e with my_off[e] <= i < my_off[e + 1]
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (my_off[mid] <= i) lo = mid; else hi = mid;
      }
      const int e = lo, r = e / el;
      const int64_t dst = dest_base[e] + (i - my_off[e]);
      int64_t tok = token_of_row[i];
      if (dst >= p.capacity_rows || tok < 0 || tok >= tokens) {
        if (threadIdx.x == 0) atomicCAS(p.status, 0, QMM_DEVICE_BAD_INDEX);
        continue;
      }
      copy_row(p.peer_recv[r] + dst * p.row_bytes, x + tok * p.row_bytes, p.row_bytes);
    }
  }
  finish_and_flag(p, stamp, 0);
}

// Result rows (receive order) back to their sources, at the pair's place in the source's sorted order.
__global__ void ep_combine_kernel(const EpParams p, const uint8_t* __restrict__ rows) {
  __shared__ int cnt[kEpMaxWorld][kEpMaxExperts];
  __shared__ int seg_start[kEpMaxExperts + 1];             // (local expert, source) segments of the receive order: `experts` of them
  __shared__ int src_off[kEpMaxWorld][kEpMaxExperts];     // first sorted row of source s for expert e
  const uint32_t stamp = *reinterpret_cast<volatile uint32_t*>(p.epoch);
  const int el = p.experts / p.world;
  const bool ok = load_counts(p, stamp, cnt);
  const int nseg = el * p.world;
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int le = 0; le < el; ++le)
      for (int s = 0; s < p.world; ++s) {
        seg_start[le * p.world + s] = acc;
        acc += cnt[s][p.rank * el + le];
      }
    seg_start[nseg] = acc;
  }
  if (threadIdx.x < p.world) {
    int acc = 0;
    for (int e = 0; e < p.experts; ++e) {
      src_off[threadIdx.x][e] = acc;
      acc += cnt[threadIdx.x][e];
    }
  }
  __syncthreads();
  if (ok) {
    const int64_t total = seg_start[nseg] < p.capacity_rows ? seg_start[nseg] : p.capacity_rows;
    for (int64_t q = blockIdx.x; q < total; q += gridDim.x) {
      int lo = 0, hi = nseg;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (seg_start[mid] <= q) lo = mid; else hi = mid;
      }
      const int le = lo / p.world, s = lo - le * p.world;
      const int64_t dst = src_off[s][p.rank * el + le] + (q - seg_start[lo]);
      if (dst >= p.max_pairs) {
        if (threadIdx.x == 0) atomicCAS(p.status, 0, QMM_DEVICE_BAD_INDEX);
        continue;
      }
      copy_row(p.peer_ret[s] + dst * p.row_bytes, rows + q * p.row_bytes, p.row_bytes);
    }
  }
  finish_and_flag(p, stamp, 1);
}

// Until every rank's flag `which` of this call has been raised here (bounded).
__global__ void ep_wait_kernel(const EpParams p, int which) {
  const uint32_t stamp = *reinterpret_cast<volatile uint32_t*>(p.epoch);
  if (threadIdx.x >= p.world) return;
  const volatile uint32_t* f = p.peer_flags[p.rank] + which * p.world + threadIdx.x;
  long long t0 = 0;
  int spins = 0;
  while (*f != stamp) {
    if (++spins >= 64) {
      if (*reinterpret_cast<volatile int*>(p.status) != 0) return;
      if (t0 == 0) t0 = clock64();
      else if (clock64() - t0 > p.spin_limit) {
        atomicCAS(p.status, 0, 111 + which);
        return;
      }
    }
  }
  __threadfence_system();
}

int fill_params(const qmm_ep_exchange* ex, int64_t row_bytes, EpParams* p) {
  if (!ex || !ex->peer_counts || !ex->peer_flags || !ex->peer_recv || !ex->peer_ret || !ex->epoch || !ex->scratch)
    return fail(QMM_ERR_NULL, "ep exchange: null pointer");
  if (ex->world < 1 || ex->world > kEpMaxWorld || ex->rank < 0 || ex->rank >= ex->world || ex->experts < ex->world ||
      ex->experts > kEpMaxExperts || ex->experts % ex->world)
    return fail(QMM_ERR_SHAPE, "ep exchange: world 1..8, experts a multiple of world, at most 256");
  if (row_bytes < 16 || row_bytes % 16 || ex->capacity_rows < 1 || ex->max_pairs < 1)
    return fail(QMM_ERR_SHAPE, "ep exchange: rows are multiples of 16 bytes, buffers hold at least one row");
  *p = EpParams{};
  for (int r = 0; r < ex->world; ++r) {
    if (!ex->peer_counts[r] || !ex->peer_flags[r] || !ex->peer_recv[r] || !ex->peer_ret[r])
      return fail(QMM_ERR_NULL, "ep exchange: bad peer pointer");
    if ((reinterpret_cast<uintptr_t>(ex->peer_recv[r]) | reinterpret_cast<uintptr_t>(ex->peer_ret[r]) |
         reinterpret_cast<uintptr_t>(ex->peer_counts[r])) & 15)
      return fail(QMM_ERR_LAYOUT, "ep exchange: buffers must be 16-byte aligned");
    p->peer_counts[r] = static_cast<uint2*>(ex->peer_counts[r]);
    p->peer_flags[r] = static_cast<uint32_t*>(ex->peer_flags[r]);
    p->peer_recv[r] = static_cast<uint8_t*>(ex->peer_recv[r]);
    p->peer_ret[r] = static_cast<uint8_t*>(ex->peer_ret[r]);
  }
  p->epoch = static_cast<uint32_t*>(ex->epoch);
  p->scratch = static_cast<uint32_t*>(ex->scratch);
  p->status = device_status_word();
  if (!p->status) return fail(QMM_ERR_CUDA, "could not allocate the device status word");
  p->spin_limit = wait_limit_clocks();
  p->capacity_rows = ex->capacity_rows;
  p->max_pairs = ex->max_pairs;
  p->row_bytes = row_bytes;
  p->rank = ex->rank; p->world = ex->world; p->experts = ex->experts;
  return QMM_OK;
}

}  // namespace
}  // namespace qmm

using namespace qmm;

extern "C" int qmm_ep_dispatch(const qmm_ep_exchange* ex, const void* x, int64_t tokens, int64_t row_bytes,
                               const int64_t* token_of_row, const int32_t* counts, int64_t pairs,
                               int32_t* group_sizes_out, void* stream) {
  EpParams p;
  int rc = fill_params(ex, row_bytes, &p);
  if (rc) return rc;
  if (!x || !token_of_row || !counts || !group_sizes_out) return fail(QMM_ERR_NULL, "ep dispatch: null pointer");
  if (pairs < 0 || pairs > ex->max_pairs || tokens < 0) return fail(QMM_ERR_SHAPE, "ep dispatch: more pairs than the return buffer holds");
  if (reinterpret_cast<uintptr_t>(x) & 15) return fail(QMM_ERR_LAYOUT, "ep dispatch: x must be 16-byte aligned");
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  ep_counts_kernel<<<1, kEpThreads, 0, st>>>(p, counts);
  int64_t grid = pairs < 1 ? 1 : pairs;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 8;
  if (grid > cap) grid = cap;
  ep_dispatch_kernel<<<static_cast<unsigned>(grid), kEpThreads, 0, st>>>(p, static_cast<const uint8_t*>(x), token_of_row, pairs,
                                                                       tokens, group_sizes_out);
  ep_wait_kernel<<<1, 32, 0, st>>>(p, 0);
  count_launch(3);
  return check_launch("ep dispatch kernels");
}

extern "C" int qmm_ep_combine(const qmm_ep_exchange* ex, const void* rows, int64_t row_bytes, void* stream) {
  EpParams p;
  int rc = fill_params(ex, row_bytes, &p);
  if (rc) return rc;
  if (!rows) return fail(QMM_ERR_NULL, "ep combine: null pointer");
  if (reinterpret_cast<uintptr_t>(rows) & 15) return fail(QMM_ERR_LAYOUT, "ep combine: rows must be 16-byte aligned");
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  int64_t grid = ex->capacity_rows;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 8;
  if (grid > cap) grid = cap;
  ep_combine_kernel<<<static_cast<unsigned>(grid), kEpThreads, 0, st>>>(p, static_cast<const uint8_t*>(rows));
  ep_wait_kernel<<<1, 32, 0, st>>>(p, 1);
  count_launch(2);
  return check_launch("ep combine kernels");
}
