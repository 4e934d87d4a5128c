// Bounds-checked accessors for debug builds (-DMTS_DEBUG_BOUNDS, build profile "debug-bounds").
//
// Kernels that compute an address from data (token ids, routing tables, peer slots) wrap the index in MTS_IN_BOUNDS.  In a
// release build the macro is the constant `true` and costs nothing.  In a debug build an index outside [0, limit) is
// recorded - kernel id, block, thread, index, limit - in a small per-translation-unit ring in device memory and the macro
// yields false, so the caller skips the access and carries on: nothing traps, the context stays usable, and the host reads
// the records afterwards (`ext.debug_bounds_report()`).  This is the stand-in for a memory checker on machines where none
// can be run.
#pragma once

#include <cuda_runtime.h>

namespace mts {
namespace dbg {

struct BoundsRecord {
  int kernel;        // one of the KERNEL_* ids below
  int block;
  int thread;
  int reserved;
  long long index;
  long long limit;
};

enum KernelId : int {
  KERNEL_EMBEDDING_FWD = 1, KERNEL_EMBEDDING_BWD = 2, KERNEL_MOE_GATHER = 3, KERNEL_MOE_COMBINE = 4, KERNEL_MOE_COMBINE_BWD = 5,
  KERNEL_EP_PUSH = 6, KERNEL_EP_PULL = 7, KERNEL_PLAN_PLACE = 8,
};

constexpr int kRingSize = 32;

// Host side (bindings.cpp): every translation unit that uses the macro registers a function that copies its ring out.
using Collector = int (*)(BoundsRecord* out, int max_records, bool reset);
void register_bounds_collector(Collector fn);

#ifdef MTS_DEBUG_BOUNDS
static __device__ BoundsRecord g_ring[kRingSize];
static __device__ unsigned g_count;

__device__ __forceinline__ bool in_bounds(int kernel, long long index, long long limit) {
  if (index >= 0 && index < limit) return true;
  const unsigned slot = atomicAdd(&g_count, 1u);
  if (slot < unsigned(kRingSize)) {
    BoundsRecord r;
    r.kernel = kernel; r.block = int(blockIdx.x); r.thread = int(threadIdx.x); r.reserved = 0; r.index = index; r.limit = limit;
    g_ring[slot] = r;
  }
  return false;
}

static int collect_bounds_of_this_unit(BoundsRecord* out, int max_records, bool reset) {
  unsigned count = 0;
  if (cudaMemcpyFromSymbol(&count, g_count, sizeof(count)) != cudaSuccess) return 0;
  int n = int(count < unsigned(kRingSize) ? count : unsigned(kRingSize));
  if (n > max_records) n = max_records;
  if (n > 0 && cudaMemcpyFromSymbol(out, g_ring, sizeof(BoundsRecord) * n) != cudaSuccess) n = 0;
  if (reset) {
    const unsigned zero = 0;
    cudaMemcpyToSymbol(g_count, &zero, sizeof(zero));
  }
  return n;
}

static const bool g_bounds_registered = (register_bounds_collector(&collect_bounds_of_this_unit), true);

#define MTS_IN_BOUNDS(kernel, index, limit) (::mts::dbg::in_bounds((kernel), (long long)(index), (long long)(limit)))
#else
#define MTS_IN_BOUNDS(kernel, index, limit) (true)
#endif

}  // namespace dbg
}  // namespace mts
