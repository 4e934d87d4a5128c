// Token embedding: row gather in forward, row scatter-add (fp32) in backward.
//
//   forward    out[t, :] = W[ids[t], :]           W fp32 or bf16 [V, H], out bf16 [T, H]; one warp per token, 16-byte accesses
//   backward   dW[ids[t], :] += dout[t, :] (fp32) vectorised fp32 reductions (red.global.add.v4.f32), straight into the flat
//              gradient buffer of a sharding engine or into a zeroed [V, H] buffer
//
// An id outside [0, V) cannot be made to index memory: the row is skipped (forward writes zeros) and the status word is
// raised to STATUS_BAD_ARGUMENT, which the host reads at its next status check.
// The reference uses nn.Embedding, i.e. the library gather and `embedding_dense_backward` (minitrain/model/transformer.py:30,76).
#include "debug_bounds.cuh"
#include "ops.cuh"
#include "ptx_sm100.cuh"

#include <cuda_bf16.h>

namespace mts {

namespace {

__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const long long* __restrict__ ids, const void* __restrict__ w, int w_bf16, __nv_bfloat16* __restrict__ out,
                     long long T, int V, int H, int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int vecs = H / 8;
  for (long long t = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    const long long id = ids[t];
    const bool ok = id >= 0 && id < V;
    if (!ok && lane == 0) {
      if (status != nullptr) atomicMax(status, STATUS_BAD_ARGUMENT);
      (void)MTS_IN_BOUNDS(dbg::KERNEL_EMBEDDING_FWD, id, V);      // bounds-checking builds also record which id it was
    }
    uint4* dst = reinterpret_cast<uint4*>(out + t * H);
    for (int v = lane; v < vecs; v += 32) {
      uint4 q = make_uint4(0u, 0u, 0u, 0u);
      if (ok) {
        if (w_bf16) {
          q = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(w) + id * H)[v];
        } else {
          const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(w) + id * H) + 2 * v;
          const float4 a = src[0], b = src[1];
          __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
          __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
          q = make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1), *reinterpret_cast<uint32_t*>(&p2),
                         *reinterpret_cast<uint32_t*>(&p3));
        }
      }
      dst[v] = q;
    }
  }
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__global__ void __launch_bounds__(256)
embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout, float* __restrict__ dw,
                     long long T, int V, int H, int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int vecs = H / 8;
  for (long long t = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    const long long id = ids[t];
    if (id < 0 || id >= V) {
      if (lane == 0) {
        if (status != nullptr) atomicMax(status, STATUS_BAD_ARGUMENT);
        (void)MTS_IN_BOUNDS(dbg::KERNEL_EMBEDDING_BWD, id, V);
      }
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(dout + t * H);
    float* dst = dw + id * H;
    for (int v = lane; v < vecs; v += 32) {
      const uint4 q = src[v];
      red_add_v4(dst + 8 * v, __uint_as_float(q.x << 16), __uint_as_float(q.x & 0xFFFF0000u), __uint_as_float(q.y << 16),
                 __uint_as_float(q.y & 0xFFFF0000u));
      red_add_v4(dst + 8 * v + 4, __uint_as_float(q.z << 16), __uint_as_float(q.z & 0xFFFF0000u), __uint_as_float(q.w << 16),
                 __uint_as_float(q.w & 0xFFFF0000u));
    }
  }
}

int token_grid(long long T) {
  long long blocks = (T + 7) / 8;                 // eight warps (tokens) per CTA
  const long long cap = (long long)device_sm_count() * 8;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : int(blocks);
}

}  // namespace

cudaError_t launch_embedding_fwd(const long long* ids, const void* w, bool w_bf16, void* out, long long T, int V, int H, int* status,
                                 cudaStream_t stream) {
  if (H % 8 != 0 || V <= 0) return cudaErrorInvalidValue;
  if (T <= 0) return cudaSuccess;
  embedding_fwd_kernel<<<token_grid(T), 256, 0, stream>>>(ids, w, w_bf16 ? 1 : 0, static_cast<__nv_bfloat16*>(out), T, V, H, status);
  ++g_launch_count;
  return cudaGetLastError();
}

cudaError_t launch_embedding_bwd(const long long* ids, const void* dout, float* dw, long long T, int V, int H, int* status,
                                 cudaStream_t stream) {
  if (H % 8 != 0 || V <= 0) return cudaErrorInvalidValue;
  if (T <= 0) return cudaSuccess;
  embedding_bwd_kernel<<<token_grid(T), 256, 0, stream>>>(ids, static_cast<const __nv_bfloat16*>(dout), dw, T, V, H, status);
  ++g_launch_count;
  return cudaGetLastError();
}

}  // namespace mts
