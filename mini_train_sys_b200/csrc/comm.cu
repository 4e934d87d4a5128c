// Collectives over NVLink / NVSwitch peer memory, written as ordinary kernels that load and store
// through peer-mapped pointers (and `multimem` on an NVLS multicast address where one is supplied).
// No NCCL call is involved once the buffers have been exchanged.
//
//   flags      every rank owns a `[channels][world]` array of 32-bit sequence numbers in symmetric memory.
//              A producer publishes epoch e by storing e into slot [channel][its rank] of every consumer
//              (st.release.sys); a consumer waits until its slots hold >= e (ld.acquire.sys).  Epochs only
//              grow, so a stale value can never satisfy a wait.  Every wait has a deadline, after which the
//              kernel records STATUS_WAIT_TIMEOUT in the status word and returns without touching data.
//   all-gather     pull: copy every peer's shard into the local full buffer.
//   reduce-scatter pull: sum the local slice of every peer's buffer (fp32), scale, accumulate sum of squares.
//                  multimem variant: one `multimem.ld_reduce` per 16 bytes does the sum inside the switch.
//   AdamW + push   update the local fp32 shard and store the new bf16 weights into every peer's replica, which
//                  turns "reduce-scatter, update, all-gather" into two kernels with no separate all-gather.
//   scalar sum     each rank deposits one float at every peer, then all sum the same values in the same order.
//
// The reference has no counterpart: it calls torch DDP / FSDP (NCCL) for all of this
// (minitrain/distributed/ddp.py:54-65, fsdp.py:128-153).
#include "comm.cuh"
#include "debug_bounds.cuh"
#include "ops.cuh"
#include "ptx_sm100.cuh"

#include <cuda_bf16.h>

namespace mts {

namespace {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Sequence number of this launch: the by-value number plus the per-step offset of graph replay (0 otherwise); 0 stays 0
// ("do not wait").
__device__ __forceinline__ uint32_t live_epoch(uint32_t epoch, const StepContext* ctx) {
  return epoch == 0u ? 0u : epoch + ctx->epoch_delta;
}

// true when *flag reached `epoch` before the deadline
__device__ __forceinline__ bool wait_epoch(const uint32_t* flag, uint32_t epoch, unsigned long long timeout_ns) {
  if (int32_t(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const unsigned long long t0 = global_timer_ns();
  while (int32_t(ld_acquire_sys(flag) - epoch) < 0) {
    if (global_timer_ns() - t0 > timeout_ns) return false;
    __nanosleep(64);
  }
  return true;
}

// Block-wide: the first `world` threads each wait for one peer, the verdict is shared with the whole block.
__device__ __forceinline__ bool block_wait_peers(const uint32_t* my_flags, int world, uint32_t epoch,
                                                 unsigned long long timeout_ns, int* status) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (int(threadIdx.x) < world && !wait_epoch(my_flags + threadIdx.x, epoch, timeout_ns)) {
    failed = 1;
    if (status != nullptr) atomicMax(status, STATUS_WAIT_TIMEOUT);
  }
  __syncthreads();
  return failed == 0;
}

__global__ void signal_kernel(PeerPtrs flag_bases, int channel, int world, int rank, uint32_t epoch, const StepContext* ctx) {
  epoch = live_epoch(epoch, ctx);
  const int peer = threadIdx.x;
  if (peer < world) {
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(flag_bases.p[peer]) + channel * world + rank, epoch);
  }
}

__global__ void wait_kernel(const uint32_t* my_flags, int channel, int world, uint32_t epoch, unsigned long long timeout_ns,
                            int* status, const StepContext* ctx) {
  epoch = live_epoch(epoch, ctx);
  block_wait_peers(my_flags + channel * world, world, epoch, timeout_ns, status);
}

// The copy kernels use CTAs of 128 threads with few registers: that is what fits on an SM beside a persistent GEMM CTA
// (320 threads x 168 registers and nearly all shared memory), so that a gather or a reduction on the side stream makes
// progress while the compute stream runs GEMMs instead of waiting for a whole SM to drain.
constexpr int kCopyThreads = 128;

// ---- all-gather (pull) ----
__global__ void __launch_bounds__(kCopyThreads)
allgather_pull_kernel(uint4* __restrict__ dst, PeerPtrs shards, long long shard_vec, int world, const uint32_t* my_flags,
                      int channel, uint32_t epoch, unsigned long long timeout_ns, int* status, const StepContext* ctx) {
  epoch = live_epoch(epoch, ctx);
  if (epoch != 0 && !block_wait_peers(my_flags + channel * world, world, epoch, timeout_ns, status)) return;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (int peer = 0; peer < world; ++peer) {
    const uint4* __restrict__ src = static_cast<const uint4*>(shards.p[peer]);
    uint4* __restrict__ out = dst + (long long)peer * shard_vec;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < shard_vec; i += 4 * stride) {      // four independent 16-byte loads in flight per thread
      const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
      out[i] = a; out[i + stride] = b; out[i + 2 * stride] = c; out[i + 3 * stride] = d;
    }
    for (; i < shard_vec; i += stride) out[i] = src[i];
  }
}

// ---- reduce-scatter (pull, fp32) ----
__device__ __forceinline__ void block_add_to(float v, float* out) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __shared__ float part[32];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < int(blockDim.x >> 5); ++w) s += part[w];
    if (s != 0.f) atomicAdd(out, s);
  }
}

__global__ void __launch_bounds__(kCopyThreads)
reduce_scatter_pull_kernel(float4* __restrict__ out, PeerPtrs bufs, long long slice_vec_offset, long long n_vec, int world,
                           float scale, float* __restrict__ sumsq, const uint32_t* my_flags, int channel, uint32_t epoch,
                           unsigned long long timeout_ns, int* status, const StepContext* ctx) {
  epoch = live_epoch(epoch, ctx);
  if (epoch != 0 && !block_wait_peers(my_flags + channel * world, world, epoch, timeout_ns, status)) return;
  float sq = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + stride < n_vec; i += 2 * stride) {                 // two positions x `world` peers of loads in flight
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
    for (int p = 0; p < world; ++p) {
      const float4* src = static_cast<const float4*>(bufs.p[p]) + slice_vec_offset;
      const float4 u = src[i], v = src[i + stride];
      a.x += u.x; a.y += u.y; a.z += u.z; a.w += u.w;
      b.x += v.x; b.y += v.y; b.z += v.z; b.w += v.w;
    }
    a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
    b.x *= scale; b.y *= scale; b.z *= scale; b.w *= scale;
    out[i] = a; out[i + stride] = b;
    sq += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
  }
  for (; i < n_vec; i += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < world; ++p) {
      const float4 v = static_cast<const float4*>(bufs.p[p])[slice_vec_offset + i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    out[i] = acc;
    sq += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  if (sumsq != nullptr) block_add_to(sq, sumsq);
}

// Same contract; the sum over ranks is done by the switch (NVLS) on a multicast address.
__global__ void __launch_bounds__(kCopyThreads)
reduce_scatter_multimem_kernel(float4* __restrict__ out, const float* __restrict__ mc_base, long long slice_vec_offset,
                               long long n_vec, int world, float scale, float* __restrict__ sumsq, const uint32_t* my_flags,
                               int channel, uint32_t epoch, unsigned long long timeout_ns, int* status, const StepContext* ctx) {
  epoch = live_epoch(epoch, ctx);
  if (epoch != 0 && !block_wait_peers(my_flags + channel * world, world, epoch, timeout_ns, status)) return;
  float sq = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (long long)gridDim.x * blockDim.x) {
    float4 acc;
    const float* addr = mc_base + 4 * (slice_vec_offset + i);
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(acc.x), "=f"(acc.y), "=f"(acc.z), "=f"(acc.w)
                 : "l"(addr)
                 : "memory");
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    out[i] = acc;
    sq += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  if (sumsq != nullptr) block_add_to(sq, sumsq);
}

// ---- AdamW on the local fp32 shard + push of the new low-precision weights to every replica ----
// Eight consecutive elements: update p, m, v in place and store the new weights into `world` replicas.
__device__ __forceinline__ void adamw_update8(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                              float* __restrict__ v, long long i, void* const* replicas, long long replica_elem_offset,
                                              int world, int push_bf16, float lr, float b1, float b2, float eps, float wd, float step,
                                              float inv_sqrt_bc2, float gs) {
  float pp[8], gg[8], mm[8], vv[8];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float4 a = reinterpret_cast<const float4*>(p)[2 * i + h], b = reinterpret_cast<const float4*>(g)[2 * i + h];
    const float4 c = reinterpret_cast<const float4*>(m)[2 * i + h], d = reinterpret_cast<const float4*>(v)[2 * i + h];
    pp[4 * h] = a.x; pp[4 * h + 1] = a.y; pp[4 * h + 2] = a.z; pp[4 * h + 3] = a.w;
    gg[4 * h] = b.x; gg[4 * h + 1] = b.y; gg[4 * h + 2] = b.z; gg[4 * h + 3] = b.w;
    mm[4 * h] = c.x; mm[4 * h + 1] = c.y; mm[4 * h + 2] = c.z; mm[4 * h + 3] = c.w;
    vv[4 * h] = d.x; vv[4 * h + 1] = d.y; vv[4 * h + 2] = d.z; vv[4 * h + 3] = d.w;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float grad = gg[j] * gs;
    mm[j] = b1 * mm[j] + (1.f - b1) * grad;
    vv[j] = b2 * vv[j] + (1.f - b2) * grad * grad;
    pp[j] = pp[j] * (1.f - lr * wd) - step * mm[j] / (sqrtf(vv[j]) * inv_sqrt_bc2 + eps);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    reinterpret_cast<float4*>(p)[2 * i + h] = make_float4(pp[4 * h], pp[4 * h + 1], pp[4 * h + 2], pp[4 * h + 3]);
    reinterpret_cast<float4*>(m)[2 * i + h] = make_float4(mm[4 * h], mm[4 * h + 1], mm[4 * h + 2], mm[4 * h + 3]);
    reinterpret_cast<float4*>(v)[2 * i + h] = make_float4(vv[4 * h], vv[4 * h + 1], vv[4 * h + 2], vv[4 * h + 3]);
  }
  if (push_bf16) {
    uint4 packed;
    uint32_t* w = &packed.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 h2 = __floats2bfloat162_rn(pp[2 * j], pp[2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&h2);
    }
    for (int r = 0; r < world; ++r)
      reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(replicas[r]) + replica_elem_offset)[i] = packed;
  } else {
    for (int r = 0; r < world; ++r) {
      float4* dst = reinterpret_cast<float4*>(static_cast<float*>(replicas[r]) + replica_elem_offset);
      dst[2 * i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
      dst[2 * i + 1] = make_float4(pp[4], pp[5], pp[6], pp[7]);
    }
  }
}

__global__ void __launch_bounds__(256)
adamw_push_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                  long long n, PeerPtrs replicas, long long replica_elem_offset, int world, int push_bf16, float lr, float b1,
                  float b2, float eps, float wd, float bc1, float bc2, const float* __restrict__ gscale_ptr, float static_scale,
                  const int* __restrict__ status) {
  // A wait that ran out earlier in this step left stale gradients behind: the whole update is skipped, so that weights and both
  // moments stay exactly as they were (weight decay and the momentum term would otherwise still move them).
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return;
  const float gs = (gscale_ptr != nullptr ? *gscale_ptr : 1.f) * static_scale;
  const float step = lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  const long long nvec = n / 8;   // the caller guarantees n % 8 == 0 and 32-byte aligned shards
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x)
    adamw_update8(p, g, m, v, i, replicas.p, replica_elem_offset, world, push_bf16, lr, b1, b2, eps, wd, step, inv_sqrt_bc2, gs);
}

// The same update over a table of segments in ONE launch: the segments of every unit of the model (a dozen units, two
// weight-decay groups) would otherwise be fifty launches of a few microseconds of work each.  Work is cut into chunks of
// kAdamChunk elements; a CTA finds the segment of a chunk by bisection over the chunk prefix stored in the table.
__global__ void __launch_bounds__(256)
adamw_push_table_kernel(const AdamWSegment* __restrict__ segs, int n_segs, long long total_chunks, float lr0, float lr1, float wd0,
                        float wd1, float b1, float b2, float eps, float bc1, float bc2, const float* __restrict__ gscale_ptr,
                        float static_scale, const int* __restrict__ status, const StepContext* __restrict__ ctx) {
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return;
  if (ctx->dynamic_adam != 0u) {     // graph replay: this step's learning rates and bias corrections come from device memory
    lr0 = ctx->lr0; lr1 = ctx->lr1; bc1 = ctx->bias_correction1; bc2 = ctx->bias_correction2;
  }
  const float gs = (gscale_ptr != nullptr ? *gscale_ptr : 1.f) * static_scale;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  for (long long chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    int lo = 0, hi = n_segs - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (segs[mid].chunk_begin <= chunk) lo = mid; else hi = mid - 1;
    }
    const AdamWSegment& sg = segs[lo];
    const long long i = (chunk - sg.chunk_begin) * (kAdamChunk / 8) + threadIdx.x;
    if (i * 8 < sg.n) {
      const float lr = sg.group == 0 ? lr0 : lr1, wd = sg.group == 0 ? wd0 : wd1;
      adamw_update8(sg.p, sg.g, sg.m, sg.v, i, sg.replicas, sg.replica_offset, sg.world, sg.push_bf16, lr, b1, b2, eps, wd,
                    lr / bc1, inv_sqrt_bc2, gs);
    }
  }
}

// ---- sum of one float per rank + clip coefficient (single block) ----
__global__ void scalar_allreduce_clip_kernel(const float* __restrict__ local_value, PeerPtrs slots, PeerPtrs flag_bases,
                                             const uint32_t* my_flags, int channel, int world, int rank, uint32_t epoch,
                                             unsigned long long timeout_ns, float max_norm, float extra_scale,
                                             float* __restrict__ coef_out, float* __restrict__ norm_out, int* status,
                                             const StepContext* ctx) {
  epoch = live_epoch(epoch, ctx);
  const int peer = threadIdx.x;
  if (peer < world) {
    // slot layout at every rank: [parity][world] so that consecutive steps never reuse a slot that is still being read
    static_cast<float*>(slots.p[peer])[(epoch & 1u) * world + rank] = *local_value;
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(flag_bases.p[peer]) + channel * world + rank, epoch);
  }
  if (!block_wait_peers(my_flags + channel * world, world, epoch, timeout_ns, status)) {
    if (threadIdx.x == 0) { *coef_out = 0.f; *norm_out = 0.f; }   // a failed step must not move the weights
    return;
  }
  if (threadIdx.x == 0) {
    const volatile float* mine = static_cast<const volatile float*>(slots.p[rank]) + (epoch & 1u) * world;
    float total = 0.f;
    for (int r = 0; r < world; ++r) total += mine[r];
    const float norm = sqrtf(total);
    *norm_out = norm;
    *coef_out = (max_norm > 0.f ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f) * extra_scale;
  }
}

int copy_grid(long long items, int threads, int max_ctas) {
  long long b = (items + threads - 1) / threads;
  if (b > max_ctas) b = max_ctas;
  return b < 1 ? 1 : int(b);
}

}  // namespace

cudaError_t launch_signal(const PeerPtrs& flag_bases, int channel, int world, int rank, unsigned epoch, cudaStream_t stream) {
  if (world > kMaxPeers) return cudaErrorInvalidValue;
  signal_kernel<<<1, 32, 0, stream>>>(flag_bases, channel, world, rank, epoch, step_context());
  ++g_launch_count;
  return cudaGetLastError();
}

cudaError_t launch_wait(const unsigned* my_flags, int channel, int world, unsigned epoch, unsigned long long timeout_ns,
                        int* status, cudaStream_t stream) {
  if (world > kMaxPeers) return cudaErrorInvalidValue;
  wait_kernel<<<1, 32, 0, stream>>>(my_flags, channel, world, epoch, timeout_ns, status, step_context());
  ++g_launch_count;
  return cudaGetLastError();
}

cudaError_t launch_allgather_pull(void* dst, const PeerPtrs& shards, long long shard_bytes, int world, const unsigned* my_flags,
                                  int channel, unsigned epoch, unsigned long long timeout_ns, int* status, int max_ctas,
                                  cudaStream_t stream) {
  if (world > kMaxPeers || shard_bytes % 16 != 0) return cudaErrorInvalidValue;
  const long long vec = shard_bytes / 16;
  allgather_pull_kernel<<<copy_grid(vec, kCopyThreads * 4, max_ctas), kCopyThreads, 0, stream>>>(
      static_cast<uint4*>(dst), shards, vec, world, my_flags, channel, epoch, timeout_ns, status, step_context());
  ++g_launch_count;
  return cudaGetLastError();
}

cudaError_t launch_reduce_scatter(float* out, const PeerPtrs& bufs, const float* multicast_base, long long slice_offset,
                                  long long n, int world, float scale, float* sumsq, const unsigned* my_flags, int channel,
                                  unsigned epoch, unsigned long long timeout_ns, int* status, int max_ctas, cudaStream_t stream) {
  if (world > kMaxPeers || n % 4 != 0 || slice_offset % 4 != 0) return cudaErrorInvalidValue;
  const int grid = copy_grid(n / 4, kCopyThreads * 2, max_ctas);
  if (multicast_base != nullptr)
    reduce_scatter_multimem_kernel<<<grid, kCopyThreads, 0, stream>>>(reinterpret_cast<float4*>(out), multicast_base, slice_offset / 4,
                                                             n / 4, world, scale, sumsq, my_flags, channel, epoch, timeout_ns, status, step_context());
  else
    reduce_scatter_pull_kernel<<<grid, kCopyThreads, 0, stream>>>(reinterpret_cast<float4*>(out), bufs, slice_offset / 4, n / 4, world,
                                                         scale, sumsq, my_flags, channel, epoch, timeout_ns, status, step_context());
  ++g_launch_count;
  return cudaGetLastError();
}

cudaError_t launch_adamw_push(const AdamWArgs& a, const PeerPtrs& replicas, long long replica_elem_offset, int world,
                              bool push_bf16, int max_ctas, const int* status, cudaStream_t stream) {
  if (world > kMaxPeers || a.n % 8 != 0) return cudaErrorInvalidValue;
  if (a.n == 0) return cudaSuccess;
  adamw_push_kernel<<<copy_grid(a.n / 8, 256, max_ctas), 256, 0, stream>>>(
      a.param, a.grad, a.exp_avg, a.exp_avg_sq, a.n, replicas, replica_elem_offset, world, push_bf16 ? 1 : 0, a.lr, a.beta1,
      a.beta2, a.eps, a.weight_decay, a.bias_correction1, a.bias_correction2, a.grad_scale, a.static_grad_scale, status);
  ++g_launch_count;
  return cudaGetLastError();
}

cudaError_t launch_adamw_push_table(const AdamWSegment* segs, int n_segs, long long total_chunks, float lr0, float lr1, float wd0,
                                    float wd1, float beta1, float beta2, float eps, float bc1, float bc2, const float* grad_scale,
                                    float static_scale, const int* status, int max_ctas, cudaStream_t stream) {
  if (n_segs <= 0 || total_chunks <= 0) return cudaSuccess;
  const int grid = int(total_chunks < max_ctas ? total_chunks : max_ctas);
  adamw_push_table_kernel<<<grid, 256, 0, stream>>>(segs, n_segs, total_chunks, lr0, lr1, wd0, wd1, beta1, beta2, eps, bc1, bc2,
                                                    grad_scale, static_scale, status, step_context());
  ++g_launch_count;
  return cudaGetLastError();
}

cudaError_t launch_scalar_allreduce_clip(const float* local_value, const PeerPtrs& slots, const PeerPtrs& flag_bases,
                                         const unsigned* my_flags, int channel, int world, int rank, unsigned epoch,
                                         unsigned long long timeout_ns, float max_norm, float extra_scale, float* coef_out,
                                         float* norm_out, int* status, cudaStream_t stream) {
  if (world > kMaxPeers) return cudaErrorInvalidValue;
  scalar_allreduce_clip_kernel<<<1, 32, 0, stream>>>(local_value, slots, flag_bases, my_flags, channel, world, rank, epoch,
                                                     timeout_ns, max_norm, extra_scale, coef_out, norm_out, status, step_context());
  ++g_launch_count;
  return cudaGetLastError();
}


// ---- expert-parallel exchange: rows pushed to the rank that owns their expert, results pulled back ---------------------
//
// Receive layout on every rank: `world` regions of `cap_rows` rows; region s belongs to source rank s, which fills slots
// 0 .. count_s - 1 in its own route order and posts count_s.  A route is (token, destination rank, slot, expert local to
// the destination).  One warp moves one row with 16-byte accesses; the destination pointer is the peer mapping of the
// receiver's buffer, so the dispatch IS the all-to-all: no staging buffer, no library call.
namespace {

__global__ void __launch_bounds__(256)
ep_push_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ route_token, const int* __restrict__ route_dest,
                    const int* __restrict__ route_slot, const int* __restrict__ route_expert, const float* __restrict__ route_scale,
                    int n_routes, int H, PeerPtrs recv_rows, PeerPtrs recv_expert, int src_rank, int cap_rows) {
  const int lane = threadIdx.x & 31;
  const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
  const int vec_per_row = H / 8;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < n_routes; r += warps_per_grid) {
    const int dest = route_dest[r];
    if (dest < 0) continue;
    if (!MTS_IN_BOUNDS(dbg::KERNEL_EP_PUSH, dest, kMaxPeers) || !MTS_IN_BOUNDS(dbg::KERNEL_EP_PUSH, route_slot[r], cap_rows)) continue;
    const long long dst_row = (long long)src_rank * cap_rows + route_slot[r];
    const uint4* src = reinterpret_cast<const uint4*>(x + (long long)route_token[r] * H);
    uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(recv_rows.p[dest]) + dst_row * H);
    const float scale = route_scale != nullptr ? route_scale[r] : 1.f;
    for (int v = lane; v < vec_per_row; v += 32) {
      uint4 q = src[v];
      if (route_scale != nullptr) {
        uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&w[k]);
          h = __floats2bfloat162_rn(__low2float(h) * scale, __high2float(h) * scale);
          w[k] = *reinterpret_cast<uint32_t*>(&h);
        }
        q = make_uint4(w[0], w[1], w[2], w[3]);
      }
      dst[v] = q;
    }
    if (lane == 0 && route_expert != nullptr) static_cast<int*>(recv_expert.p[dest])[dst_row] = route_expert[r];
  }
}

// out[t] = sum_k weight[t, k] * rows_of(dest(t, k))[me * cap + slot(t, k)], read through the peers' mappings.  `saved`
// (optional, [T * K, H]) keeps the pulled rows for the backward pass of the weights.
__global__ void __launch_bounds__(256)
ep_pull_combine_kernel(__nv_bfloat16* __restrict__ out, const int* __restrict__ token_dest, const int* __restrict__ token_slot,
                       const float* __restrict__ weight, int T, int K, int H, PeerPtrs rows, int my_rank, int cap_rows,
                       __nv_bfloat16* __restrict__ saved) {
  const int lane = threadIdx.x & 31;
  const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
  const int vec_per_row = H / 8;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps_per_grid) {
    for (int v = lane; v < vec_per_row; v += 32) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int k = 0; k < K; ++k) {
        const int dest = token_dest[t * K + k];
        uint4 q = make_uint4(0u, 0u, 0u, 0u);
        if (dest >= 0 && MTS_IN_BOUNDS(dbg::KERNEL_EP_PULL, dest, kMaxPeers) &&
            MTS_IN_BOUNDS(dbg::KERNEL_EP_PULL, token_slot[t * K + k], cap_rows)) {
          const long long row = (long long)my_rank * cap_rows + token_slot[t * K + k];
          q = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(rows.p[dest]) + row * H)[v];
        }
        if (saved != nullptr) reinterpret_cast<uint4*>(saved + ((long long)t * K + k) * H)[v] = q;
        const float w = weight != nullptr ? weight[t * K + k] : 1.f;
        const uint32_t ww[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&ww[j]);
          acc[2 * j] += w * __low2float(h);
          acc[2 * j + 1] += w * __high2float(h);
        }
      }
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        o[j] = *reinterpret_cast<uint32_t*>(&h);
      }
      reinterpret_cast<uint4*>(out + (long long)t * H)[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

__global__ void ep_post_counts_kernel(const int* __restrict__ counts, PeerPtrs recv_counts, int world, int src_rank) {
  const int d = threadIdx.x;
  if (d < world) static_cast<int*>(recv_counts.p[d])[src_rank] = counts[d];
}

}  // namespace

cudaError_t launch_ep_push_rows(const void* x, const int* route_token, const int* route_dest, const int* route_slot,
                                const int* route_expert, const float* route_scale, int n_routes, int H, const PeerPtrs& recv_rows,
                                const PeerPtrs& recv_expert, const int* counts, const PeerPtrs& recv_counts, int world, int src_rank,
                                int cap_rows, int max_ctas, cudaStream_t stream) {
  if (H % 8 != 0) return cudaErrorInvalidValue;
  if (counts != nullptr) ep_post_counts_kernel<<<1, 32, 0, stream>>>(counts, recv_counts, world, src_rank);
  if (n_routes > 0) {
    int grid = (n_routes + 7) / 8;
    if (grid > max_ctas) grid = max_ctas;
    ep_push_rows_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), route_token, route_dest, route_slot,
                                                 route_expert, route_scale, n_routes, H, recv_rows, recv_expert, src_rank, cap_rows);
  }
  return cudaGetLastError();
}

cudaError_t launch_ep_pull_combine(void* out, const int* token_dest, const int* token_slot, const float* weight, int T, int K, int H,
                                   const PeerPtrs& rows, int my_rank, int cap_rows, void* saved, int max_ctas, cudaStream_t stream) {
  if (H % 8 != 0) return cudaErrorInvalidValue;
  if (T <= 0) return cudaSuccess;
  int grid = (T + 7) / 8;
  if (grid > max_ctas) grid = max_ctas;
  ep_pull_combine_kernel<<<grid, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(out), token_dest, token_slot, weight, T, K, H, rows,
                                                  my_rank, cap_rows, static_cast<__nv_bfloat16*>(saved));
  return cudaGetLastError();
}

}  // namespace mts
