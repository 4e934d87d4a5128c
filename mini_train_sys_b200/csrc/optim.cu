// Optimizer-side kernels: fused AdamW over a flat fp32 shard (optionally refreshing a bf16 copy of
// the weights and applying a device-resident gradient scale such as the clip coefficient), the
// sum of squares used for the global gradient norm, and the clip coefficient itself.
// Reference counterpart: torch.optim.AdamW(fused=True) + clip_grad_norm_ (minitrain/train/optim.py:41-47,
// minitrain/train/trainer.py:63-83), which cost a host synchronisation per step.
#include "ops.cuh"

#include <cuda_bf16.h>

namespace mts {

namespace {

__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
             __nv_bfloat16* __restrict__ shadow, long long n, float lr, float b1, float b2, float eps, float wd,
             float bc1, float bc2, const float* __restrict__ gscale_ptr, float static_scale) {
  const float gs = (gscale_ptr != nullptr ? *gscale_ptr : 1.f) * static_scale;
  const float step = lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  const long long nvec = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float4 pp = reinterpret_cast<float4*>(p)[i];
    const float4 gg = reinterpret_cast<const float4*>(g)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float* pa = &pp.x; const float* ga = &gg.x; float* ma = &mm.x; float* va = &vv.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float grad = ga[j] * gs;
      ma[j] = b1 * ma[j] + (1.f - b1) * grad;
      va[j] = b2 * va[j] + (1.f - b2) * grad * grad;
      const float denom = sqrtf(va[j]) * inv_sqrt_bc2 + eps;
      pa[j] = pa[j] * (1.f - lr * wd) - step * ma[j] / denom;
    }
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (shadow != nullptr) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(pp.x, pp.y), hi = __floats2bfloat162_rn(pp.z, pp.w);
      uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
      reinterpret_cast<uint2*>(shadow)[i] = packed;
    }
  }
  // tail (n not a multiple of 4)
  const long long base = nvec * 4;
  if (blockIdx.x == 0 && threadIdx.x < n - base) {
    const long long i = base + threadIdx.x;
    const float grad = g[i] * gs;
    const float mi = b1 * m[i] + (1.f - b1) * grad;
    const float vi = b2 * v[i] + (1.f - b2) * grad * grad;
    m[i] = mi; v[i] = vi;
    const float np = p[i] * (1.f - lr * wd) - step * mi / (sqrtf(vi) * inv_sqrt_bc2 + eps);
    p[i] = np;
    if (shadow != nullptr) shadow[i] = __float2bfloat16(np);
  }
}

__global__ void __launch_bounds__(256)
sumsq_kernel(const float* __restrict__ x, long long n, float* __restrict__ out) {
  float acc = 0.f;
  const long long nvec = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const float4 q = reinterpret_cast<const float4*>(x)[i];
    acc += q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w;
  }
  if (blockIdx.x == 0 && threadIdx.x < n - nvec * 4) {
    const float t = x[nvec * 4 + threadIdx.x];
    acc += t * t;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ float part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < 8; ++w) s += part[w];
    atomicAdd(out, s);
  }
}

__global__ void clip_coef_kernel(const float* __restrict__ sumsq, float max_norm, float extra, float* __restrict__ coef,
                                 float* __restrict__ norm_out) {
  const float norm = sqrtf(*sumsq);
  if (norm_out != nullptr) *norm_out = norm;
  const float c = max_norm > 0.f ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
  *coef = c * extra;
}

}  // namespace

cudaError_t launch_adamw(const AdamWArgs& a, cudaStream_t stream) {
  if (a.n <= 0) return cudaSuccess;
  long long blocks = (a.n / 4 + 255) / 256;
  const long long cap = (long long)device_sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  adamw_kernel<<<unsigned(blocks), 256, 0, stream>>>(a.param, a.grad, a.exp_avg, a.exp_avg_sq,
                                                     static_cast<__nv_bfloat16*>(a.shadow_bf16), a.n, a.lr, a.beta1, a.beta2,
                                                     a.eps, a.weight_decay, a.bias_correction1, a.bias_correction2,
                                                     a.grad_scale, a.static_grad_scale);
  ++g_launch_count;
  return cudaGetLastError();
}

cudaError_t launch_sumsq(const float* x, long long n, float* out, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  long long blocks = (n / 4 + 255) / 256;
  const long long cap = (long long)device_sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  sumsq_kernel<<<unsigned(blocks), 256, 0, stream>>>(x, n, out);
  ++g_launch_count;
  return cudaGetLastError();
}

cudaError_t launch_clip_coef(const float* sumsq, float max_norm, float extra, float* coef, float* norm_out,
                             cudaStream_t stream) {
  clip_coef_kernel<<<1, 1, 0, stream>>>(sumsq, max_norm, extra, coef, norm_out);
  ++g_launch_count;
  return cudaGetLastError();
}

}  // namespace mts
