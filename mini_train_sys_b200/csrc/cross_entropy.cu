// Cross entropy over a [rows, vocab] logits matrix, one CTA per row.
//   forward : online (max, sum-exp) in one streaming pass -> lse; loss = lse - z[target]
//   backward: logits <- (exp(z - lse) - onehot) * scale, written in place (the second pass over a row
//             is served by the 126 MB L2 for the chunk sizes used by the fused linear-CE driver)
// Rows whose target is negative (-100) are ignored: zero loss, zero gradient, not counted.
// Reference counterpart: minitrain/kernels/triton/cross_entropy.py:68-163.
#include "ops.cuh"

#include <cuda_bf16.h>
#include <math_constants.h>

namespace mts {

namespace {

constexpr int kCeThreads = 256;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct MaxSum {
  float m, s;
  __device__ __forceinline__ void push(float z) {
    if (z > m) {
      s = s * __expf(m - z) + 1.f;
      m = z;
    } else {
      s += __expf(z - m);
    }
  }
  // N values at once: one maximum, at most one rescale of the running sum, then N independent exponentials in two
  // chains.  The element-at-a-time form carries (m, s) through a branch per element and is bound by that chain.
  template <int N>
  __device__ __forceinline__ void push_vec(const float (&z)[N]) {
    float vm = z[0];
#pragma unroll
    for (int j = 1; j < N; ++j) vm = fmaxf(vm, z[j]);
    if (vm > m) {
      s *= ex2f((m - vm) * kLog2e);      // m = -inf: the factor is 0 and s is 0
      m = vm;
    }
    const float mb = m == -CUDART_INF_F ? 0.f : -m * kLog2e;
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int j = 0; j < N; j += 2) {
      a += ex2f(fmaf(z[j], kLog2e, mb));
      b += ex2f(fmaf(z[j + 1], kLog2e, mb));
    }
    s += a + b;
  }
  __device__ __forceinline__ void merge(const MaxSum& o) {
    const float nm = fmaxf(m, o.m);
    if (nm == -CUDART_INF_F) return;
    s = s * __expf(m - nm) + o.s * __expf(o.m - nm);
    m = nm;
  }
};

// Visit every column of one row with 16-byte loads once the address is aligned.
template <typename T, typename F>
__device__ __forceinline__ void for_each_column(const T* row, int n, F&& f) {
  constexpr int per = 16 / sizeof(T);
  int head = int(((16 - (reinterpret_cast<uintptr_t>(row) & 15)) & 15) / sizeof(T));
  if (head > n) head = n;
  for (int c = threadIdx.x; c < head; c += blockDim.x) f(c, to_f<T>(row[c]));
  const int nvec = (n - head) / per;
  const uint4* body = reinterpret_cast<const uint4*>(row + head);
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 q = body[v];
    const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
    for (int j = 0; j < per; ++j) f(head + v * per + j, to_f<T>(e[j]));
  }
  for (int c = head + nvec * per + threadIdx.x; c < n; c += blockDim.x) f(c, to_f<T>(row[c]));
}

template <typename T>
__global__ void __launch_bounds__(kCeThreads)
ce_forward_kernel(const T* __restrict__ logits, long long ld, const long long* __restrict__ targets,
                  float* __restrict__ row_lse, float* __restrict__ stats, int vocab) {
  const long long r = blockIdx.x;
  const T* row = logits + r * ld;
  MaxSum acc{-CUDART_INF_F, 0.f};
  {
    constexpr int per = 16 / sizeof(T);
    int head = int(((16 - (reinterpret_cast<uintptr_t>(row) & 15)) & 15) / sizeof(T));
    if (head > vocab) head = vocab;
    for (int c = threadIdx.x; c < head; c += blockDim.x) acc.push(to_f<T>(row[c]));
    const int nvec = (vocab - head) / per;
    const uint4* body = reinterpret_cast<const uint4*>(row + head);
    int v = threadIdx.x;
    for (; v + int(blockDim.x) < nvec; v += 2 * blockDim.x) {      // two 16-byte loads in flight per thread
      const uint4 q0 = body[v], q1 = body[v + blockDim.x];
      float z[2 * per];
      const T* e0 = reinterpret_cast<const T*>(&q0);
      const T* e1 = reinterpret_cast<const T*>(&q1);
#pragma unroll
      for (int j = 0; j < per; ++j) { z[j] = to_f<T>(e0[j]); z[per + j] = to_f<T>(e1[j]); }
      acc.push_vec(z);
    }
    for (; v < nvec; v += blockDim.x) {
      const uint4 q = body[v];
      const T* e = reinterpret_cast<const T*>(&q);
      float z[per];
#pragma unroll
      for (int j = 0; j < per; ++j) z[j] = to_f<T>(e[j]);
      acc.push_vec(z);
    }
    for (int c = head + nvec * per + threadIdx.x; c < vocab; c += blockDim.x) acc.push(to_f<T>(row[c]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum other{__shfl_xor_sync(0xffffffffu, acc.m, o), __shfl_xor_sync(0xffffffffu, acc.s, o)};
    acc.merge(other);
  }
  __shared__ float sm[kCeThreads / 32], ss[kCeThreads / 32];
  if ((threadIdx.x & 31) == 0) {
    sm[threadIdx.x >> 5] = acc.m;
    ss[threadIdx.x >> 5] = acc.s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    MaxSum tot{sm[0], ss[0]};
    for (int w = 1; w < kCeThreads / 32; ++w) tot.merge(MaxSum{sm[w], ss[w]});
    const float lse = tot.m + __logf(tot.s);
    row_lse[r] = lse;
    const long long t = targets[r];
    if (t >= 0 && t < vocab) {
      atomicAdd(stats + 0, lse - to_f<T>(row[t]));
      atomicAdd(stats + 1, 1.f);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kCeThreads)
ce_backward_kernel(T* __restrict__ logits, long long ld, const long long* __restrict__ targets,
                   const float* __restrict__ row_lse, const float* __restrict__ valid_count,
                   const float* __restrict__ grad_scale, int vocab, int padded_vocab) {
  const long long r = blockIdx.x;
  T* row = logits + r * ld;
  const long long t = targets[r];
  const bool live = t >= 0 && t < vocab;
  const float scale = live ? (grad_scale != nullptr ? *grad_scale : 1.f) / fmaxf(*valid_count, 1.f) : 0.f;
  const float lse = row_lse[r];
  constexpr int per = 16 / sizeof(T);
  int head = int(((16 - (reinterpret_cast<uintptr_t>(row) & 15)) & 15) / sizeof(T));
  if (head > vocab) head = vocab;
  const float lse2 = -lse * kLog2e;
  auto grad = [&](int c, float z) -> float {
    float g = live ? ex2f(fmaf(z, kLog2e, lse2)) : 0.f;
    if (c == t) g -= 1.f;
    return g * scale;
  };
  for (int c = threadIdx.x; c < head; c += blockDim.x) row[c] = from_f<T>(grad(c, to_f<T>(row[c])));
  const int nvec = (vocab - head) / per;
  uint4* body = reinterpret_cast<uint4*>(row + head);
  const int t_vec = live && t >= head ? int((t - head) / per) : -1;     // the one vector that holds the target column
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    uint4 q = body[v];
    T* e = reinterpret_cast<T*>(&q);
    if (v == t_vec) {
#pragma unroll
      for (int j = 0; j < per; ++j) e[j] = from_f<T>(grad(head + v * per + j, to_f<T>(e[j])));
    } else {
#pragma unroll
      for (int j = 0; j < per; ++j) e[j] = from_f<T>((live ? ex2f(fmaf(to_f<T>(e[j]), kLog2e, lse2)) : 0.f) * scale);
    }
    body[v] = q;
  }
  for (int c = head + nvec * per + threadIdx.x; c < vocab; c += blockDim.x) row[c] = from_f<T>(grad(c, to_f<T>(row[c])));
  for (int c = vocab + threadIdx.x; c < padded_vocab; c += blockDim.x) row[c] = from_f<T>(0.f);
}

__global__ void count_valid_kernel(const long long* __restrict__ targets, long long n, float* __restrict__ out) {
  float local = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    local += targets[i] >= 0 ? 1.f : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
  if ((threadIdx.x & 31) == 0 && local != 0.f) atomicAdd(out, local);
}

}  // namespace

cudaError_t launch_ce_forward(const void* logits, long long ld, const long long* targets, float* row_lse, float* stats,
                              long long rows, int vocab, bool bf16, cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  if (bf16)
    ce_forward_kernel<__nv_bfloat16><<<unsigned(rows), kCeThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(logits), ld, targets, row_lse, stats, vocab);
  else
    ce_forward_kernel<float><<<unsigned(rows), kCeThreads, 0, stream>>>(static_cast<const float*>(logits), ld, targets,
                                                                         row_lse, stats, vocab);
  ++g_launch_count;
  return cudaGetLastError();
}

cudaError_t launch_ce_backward(void* logits, long long ld, const long long* targets, const float* row_lse,
                               const float* valid_count, const float* grad_scale, long long rows, int vocab,
                               int padded_vocab, bool bf16, cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  if (bf16)
    ce_backward_kernel<__nv_bfloat16><<<unsigned(rows), kCeThreads, 0, stream>>>(
        static_cast<__nv_bfloat16*>(logits), ld, targets, row_lse, valid_count, grad_scale, vocab, padded_vocab);
  else
    ce_backward_kernel<float><<<unsigned(rows), kCeThreads, 0, stream>>>(static_cast<float*>(logits), ld, targets, row_lse,
                                                                          valid_count, grad_scale, vocab, padded_vocab);
  ++g_launch_count;
  return cudaGetLastError();
}

cudaError_t launch_count_valid_targets(const long long* targets, long long n, float* out_count, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  long long blocks = (n + 255) / 256;
  if (blocks > 1024) blocks = 1024;
  count_valid_kernel<<<unsigned(blocks), 256, 0, stream>>>(targets, n, out_count);
  ++g_launch_count;
  return cudaGetLastError();
}

}  // namespace mts
