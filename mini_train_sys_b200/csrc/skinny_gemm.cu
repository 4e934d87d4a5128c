// Router projection: x[T, H] (bf16) times W[E, H] with a handful of experts (E = 4, 8 or 16).
//
// A 49,152 x 768 activation against 8 experts is 0.6 GFLOP over 75 MB: the work is reading x once.  The 256-wide tiles of
// the tcgen05 GEMM spend 32 us on it (1 / 32 of each tile is used); these kernels stay at the time of the read.  All
// arithmetic is fp32 FMA on exact bf16 inputs and fp32 (or bf16) weights, which is what the reference computes
// (fp32 F.linear outside autocast, minitrain/model/moe_router.py:64-73).
//
// Layout of the work: a lane owns COLS consecutive columns of a 32 * COLS wide column pass and keeps the E x COLS weights
// of that patch in registers while it walks over rows, so a weight is loaded once per (warp, pass), not once per row.
//   forward   per (row, pass) the lane's E partial sums are reduced over the warp with a halving exchange and added to a
//             warp-private accumulator in shared memory (fixed order: deterministic)
//   dx        out[row][cols] = sum_e g[row][e] * W[e][cols]
//   dW        acc[e][cols] += g[row][e] * x[row][cols] over the warp's rows; CTA partials meet in global memory and the last
//             CTA of a column pass adds them up in a fixed order (deterministic, no per-element atomics)
#include "ops.cuh"

#include <cuda_bf16.h>

namespace mts {

namespace {

constexpr int kRowsPerStep = 4;

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

template <int COLS>
__device__ __forceinline__ void load_x(const __nv_bfloat16* p, float (&v)[COLS]) {
  if constexpr (COLS == 8) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    v[0] = bf16_lo(q.x); v[1] = bf16_hi(q.x); v[2] = bf16_lo(q.y); v[3] = bf16_hi(q.y);
    v[4] = bf16_lo(q.z); v[5] = bf16_hi(q.z); v[6] = bf16_lo(q.w); v[7] = bf16_hi(q.w);
  } else {
    const uint2 q = *reinterpret_cast<const uint2*>(p);
    v[0] = bf16_lo(q.x); v[1] = bf16_hi(q.x); v[2] = bf16_lo(q.y); v[3] = bf16_hi(q.y);
  }
}

template <int E, int COLS>
__device__ __forceinline__ void load_w(const void* w, bool w_bf16, int H, int col, float (&r)[E][COLS]) {
#pragma unroll
  for (int e = 0; e < E; ++e) {
    if (w_bf16) {
      load_x<COLS>(static_cast<const __nv_bfloat16*>(w) + (long long)e * H + col, r[e]);
    } else {
      const float* src = static_cast<const float*>(w) + (long long)e * H + col;
#pragma unroll
      for (int c = 0; c < COLS; c += 4) {
        const float4 q = *reinterpret_cast<const float4*>(src + c);
        r[e][c] = q.x; r[e][c + 1] = q.y; r[e][c + 2] = q.z; r[e][c + 3] = q.w;
      }
    }
  }
}

// Sum of `v[e]` over the 32 lanes for every e, at the cost of E - 1 + (5 - log2 E) shuffles instead of 5 E: each halving
// step sends half of the values to the partner lane and keeps the other half.  Afterwards lane L holds the total of
// expert L >> (5 - log2 E) (all lanes that share those top bits hold the same total).
template <int E>
__device__ __forceinline__ float warp_reduce_by_expert(float (&v)[E], int lane) {
  int width = E;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    if (width > 1) {
      const int half = width >> 1;
      const bool upper = (lane & off) != 0;
#pragma unroll
      for (int i = 0; i < E / 2; ++i) {
        if (i < half) {
          const float send = upper ? v[i] : v[i + half];
          const float keep = upper ? v[i + half] : v[i];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
      }
      width = half;
    } else {
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
    }
  }
  return v[0];
}

constexpr int kFwdRows = 32;   // rows one warp accumulates before it writes them out
constexpr int kFwdStep = 8;    // of which this many are in flight at a time

// logits[T, E] (fp32).  A warp owns kFwdRows consecutive rows; for every column pass it keeps its E x COLS patch of the
// weights in registers, walks over its rows eight at a time (eight independent 16-byte loads in flight) and adds the
// per-row, per-expert sums into a private shared-memory accumulator; the order of additions is fixed, so the result is
// deterministic.
template <int E, int COLS>
__global__ void __launch_bounds__(256)
router_logits_fwd_kernel(const __nv_bfloat16* __restrict__ x, const void* __restrict__ w, int w_bf16, float* __restrict__ out,
                         int T, int H) {
  __shared__ float acc_sm[8][kFwdRows][E];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  constexpr int SPAN = 32 * COLS;
  constexpr int LOG2E = E == 4 ? 2 : (E == 8 ? 3 : 4);
  const int passes = (H + SPAN - 1) / SPAN;
  const int blocks = (T + kFwdRows - 1) / kFwdRows;
  float (*acc)[E] = acc_sm[warp];
  for (int blk = blockIdx.x * 8 + warp; blk < blocks; blk += gridDim.x * 8) {
    const int row0 = blk * kFwdRows;
    for (int i = lane; i < kFwdRows * E; i += 32) (&acc[0][0])[i] = 0.f;
    __syncwarp();
    for (int pass = 0; pass < passes; ++pass) {
      const int col = pass * SPAN + lane * COLS;
      const bool live = col < H;
      float wr[E][COLS];
      if (live) {
        load_w<E, COLS>(w, w_bf16 != 0, H, col, wr);
      } else {
#pragma unroll
        for (int e = 0; e < E; ++e)
#pragma unroll
          for (int c = 0; c < COLS; ++c) wr[e][c] = 0.f;
      }
      const int safe_col = live ? col : 0;
      for (int r = 0; r < kFwdRows; r += kFwdStep) {
        float xv[kFwdStep][COLS];
#pragma unroll
        for (int j = 0; j < kFwdStep; ++j) {
          const int row = row0 + r + j < T ? row0 + r + j : T - 1;
          load_x<COLS>(x + (long long)row * H + safe_col, xv[j]);
        }
#pragma unroll
        for (int j = 0; j < kFwdStep; ++j) {
          float part[E];
#pragma unroll
          for (int e = 0; e < E; ++e) {
            float a = 0.f;
#pragma unroll
            for (int c = 0; c < COLS; ++c) a = fmaf(xv[j][c], wr[e][c], a);
            part[e] = a;
          }
          const float total = warp_reduce_by_expert<E>(part, lane);
          if ((lane & ((32 >> LOG2E) - 1)) == 0) acc[r + j][lane >> (5 - LOG2E)] += total;
        }
      }
      __syncwarp();
    }
    for (int i = lane; i < kFwdRows * E; i += 32) {
      const long long idx = (long long)row0 * E + i;
      if (idx < (long long)T * E) out[idx] = (&acc[0][0])[i];
    }
    __syncwarp();
  }
}

// dx[T, H] (bf16) = g[T, E] (fp32) * W[E, H].  A warp keeps the weights of one column pass and walks over its rows, four
// rows per step so that four gradient rows are in flight.
template <int E, int COLS>
__global__ void __launch_bounds__(256)
router_logits_dx_kernel(const float* __restrict__ g, const void* __restrict__ w, int w_bf16, __nv_bfloat16* __restrict__ dx,
                        int T, int H) {
  const int lane = threadIdx.x & 31;
  const int warp_in_grid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  constexpr int SPAN = 32 * COLS;
  const int pass = blockIdx.y;
  const int col = pass * SPAN + lane * COLS;
  if (col >= H) return;
  float wr[E][COLS];
  load_w<E, COLS>(w, w_bf16 != 0, H, col, wr);
  for (int row0 = warp_in_grid * kRowsPerStep; row0 < T; row0 += warps * kRowsPerStep) {
    float gv[kRowsPerStep][E];
#pragma unroll
    for (int j = 0; j < kRowsPerStep; ++j) {
      const int row = row0 + j < T ? row0 + j : T - 1;
#pragma unroll
      for (int e = 0; e < E; e += 4) {
        const float4 q = *reinterpret_cast<const float4*>(g + (long long)row * E + e);
        gv[j][e] = q.x; gv[j][e + 1] = q.y; gv[j][e + 2] = q.z; gv[j][e + 3] = q.w;
      }
    }
#pragma unroll
    for (int j = 0; j < kRowsPerStep; ++j) {
      if (row0 + j >= T) break;
      uint32_t packed[COLS / 2];
#pragma unroll
      for (int c = 0; c < COLS; c += 2) {
        float a = 0.f, b = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) {
          a = fmaf(gv[j][e], wr[e][c], a);
          b = fmaf(gv[j][e], wr[e][c + 1], b);
        }
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        packed[c / 2] = *reinterpret_cast<uint32_t*>(&h);
      }
      __nv_bfloat16* dst = dx + (long long)(row0 + j) * H + col;
      if constexpr (COLS == 8) *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      else *reinterpret_cast<uint2*>(dst) = make_uint2(packed[0], packed[1]);
    }
  }
}

// dW[E, H] (fp32) = g^T x.  blockIdx.y = column pass; every warp accumulates its rows in registers (four rows in flight per
// step) and the CTA adds its eight warps up in shared memory.  The CTAs of a pass then meet in global memory: each writes its
// partial [E x SPAN] block, and the last one to arrive (a counter per pass) adds all of them up in a fixed order and writes
// the result, so the gradient is deterministic and nothing serialises on same-address atomics (one atomic per CTA instead of
// one per element: with 100 CTAs per pass the per-element version spent most of its 60 us queueing in L2).
template <int E, int COLS>
__global__ void __launch_bounds__(256)
router_logits_dw_kernel(const float* __restrict__ g, const __nv_bfloat16* __restrict__ x, float* __restrict__ dw,
                        float* __restrict__ partial, unsigned* __restrict__ arrivals, int T, int H) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warp_in_grid = blockIdx.x * 8 + warp;
  const int warps = gridDim.x * 8;
  constexpr int SPAN = 32 * COLS;
  const int col = blockIdx.y * SPAN + lane * COLS;
  const bool live = col < H;
  float acc[E][COLS];
#pragma unroll
  for (int e = 0; e < E; ++e)
#pragma unroll
    for (int c = 0; c < COLS; ++c) acc[e][c] = 0.f;
  if (live) {
    for (int row0 = warp_in_grid * kRowsPerStep; row0 < T; row0 += warps * kRowsPerStep) {
      float xv[kRowsPerStep][COLS], gv[kRowsPerStep][E];
#pragma unroll
      for (int j = 0; j < kRowsPerStep; ++j) {
        const bool ok = row0 + j < T;
        const int row = ok ? row0 + j : T - 1;
        load_x<COLS>(x + (long long)row * H + col, xv[j]);
#pragma unroll
        for (int e = 0; e < E; e += 4) {
          const float4 q = *reinterpret_cast<const float4*>(g + (long long)row * E + e);
          gv[j][e] = ok ? q.x : 0.f; gv[j][e + 1] = ok ? q.y : 0.f; gv[j][e + 2] = ok ? q.z : 0.f; gv[j][e + 3] = ok ? q.w : 0.f;
        }
      }
#pragma unroll
      for (int j = 0; j < kRowsPerStep; ++j)
#pragma unroll
        for (int e = 0; e < E; ++e)
#pragma unroll
          for (int c = 0; c < COLS; ++c) acc[e][c] = fmaf(gv[j][e], xv[j][c], acc[e][c]);
    }
  }
  __shared__ float part[E * SPAN];
  __shared__ int is_last;
  for (int i = threadIdx.x; i < E * SPAN; i += blockDim.x) part[i] = 0.f;
  __syncthreads();
  for (int w = 0; w < 8; ++w) {        // warps take turns: a fixed order of additions
    if (warp == w) {
#pragma unroll
      for (int e = 0; e < E; ++e)
#pragma unroll
        for (int c = 0; c < COLS; ++c) part[e * SPAN + lane * COLS + c] += acc[e][c];
    }
    __syncthreads();
  }
  float* mine = partial + ((long long)blockIdx.y * gridDim.x + blockIdx.x) * (E * SPAN);
  for (int i = threadIdx.x; i < E * SPAN; i += blockDim.x) mine[i] = part[i];
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(arrivals + blockIdx.y, 1u) == gridDim.x - 1 ? 1 : 0;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const float* base = partial + (long long)blockIdx.y * gridDim.x * (E * SPAN);
  for (int i = threadIdx.x; i < E * SPAN; i += blockDim.x) {
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    int b = 0;
    for (; b + 3 < int(gridDim.x); b += 4) {
      s0 += __ldcg(base + (long long)b * (E * SPAN) + i);
      s1 += __ldcg(base + (long long)(b + 1) * (E * SPAN) + i);
      s2 += __ldcg(base + (long long)(b + 2) * (E * SPAN) + i);
      s3 += __ldcg(base + (long long)(b + 3) * (E * SPAN) + i);
    }
    for (; b < int(gridDim.x); ++b) s0 += __ldcg(base + (long long)b * (E * SPAN) + i);
    const int e = i / SPAN, c = i - e * SPAN;
    const int gc = blockIdx.y * SPAN + c;
    if (gc < H) dw[(long long)e * H + gc] = (s0 + s1) + (s2 + s3);
  }
  if (threadIdx.x == 0) arrivals[blockIdx.y] = 0;     // ready for the next launch on this stream
}

template <int E, int COLS>
cudaError_t run_fwd(const void* x, const void* w, bool w_bf16, float* out, int T, int H, cudaStream_t stream) {
  const int grid = device_sm_count() * 4;
  router_logits_fwd_kernel<E, COLS><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), w, w_bf16 ? 1 : 0, out, T, H);
  return cudaGetLastError();
}

template <int E, int COLS>
cudaError_t run_dx(const float* g, const void* w, bool w_bf16, void* dx, int T, int H, cudaStream_t stream) {
  const int passes = (H + 32 * COLS - 1) / (32 * COLS);
  int gx = device_sm_count() * 4 / passes;
  if (gx < 1) gx = 1;
  router_logits_dx_kernel<E, COLS><<<dim3(gx, passes), 256, 0, stream>>>(g, w, w_bf16 ? 1 : 0, static_cast<__nv_bfloat16*>(dx), T, H);
  return cudaGetLastError();
}

template <int E, int COLS>
cudaError_t run_dw(const float* g, const void* x, float* dw, float* partial, unsigned* arrivals, int gx, int T, int H,
                   cudaStream_t stream) {
  const int passes = (H + 32 * COLS - 1) / (32 * COLS);
  router_logits_dw_kernel<E, COLS><<<dim3(gx, passes), 256, 0, stream>>>(g, static_cast<const __nv_bfloat16*>(x), dw, partial,
                                                                      arrivals, T, H);
  return cudaGetLastError();
}

}  // namespace

bool router_logits_supported(int E, int H) { return (E == 4 || E == 8 || E == 16) && H % 8 == 0 && H > 0; }

cudaError_t launch_router_logits_fwd(const void* x, const void* w, bool w_bf16, float* out, int T, int E, int H, cudaStream_t stream) {
  if (!router_logits_supported(E, H)) return cudaErrorInvalidValue;
  if (T <= 0) return cudaSuccess;
  ++g_launch_count;
  if (E == 4) return run_fwd<4, 8>(x, w, w_bf16, out, T, H, stream);
  if (E == 8) return run_fwd<8, 8>(x, w, w_bf16, out, T, H, stream);
  return run_fwd<16, 4>(x, w, w_bf16, out, T, H, stream);
}

cudaError_t launch_router_logits_dx(const float* g, const void* w, bool w_bf16, void* dx, int T, int E, int H, cudaStream_t stream) {
  if (!router_logits_supported(E, H)) return cudaErrorInvalidValue;
  if (T <= 0) return cudaSuccess;
  ++g_launch_count;
  if (E == 4) return run_dx<4, 8>(g, w, w_bf16, dx, T, H, stream);
  if (E == 8) return run_dx<8, 8>(g, w, w_bf16, dx, T, H, stream);
  return run_dx<16, 4>(g, w, w_bf16, dx, T, H, stream);
}

// Scratch of the weight-gradient kernel: `ctas_per_pass` partial blocks per column pass and one arrival counter per pass.
void router_logits_dw_plan(int E, int H, int* passes, int* ctas_per_pass, long long* partial_floats) {
  const int span = E == 16 ? 128 : 256;
  *passes = (H + span - 1) / span;
  int gx = device_sm_count() * 2 / *passes;
  if (gx < 1) gx = 1;
  *ctas_per_pass = gx;
  *partial_floats = (long long)*passes * gx * E * span;
}

cudaError_t launch_router_logits_dw(const float* g, const void* x, float* dw, float* partial, unsigned* arrivals, int T, int E, int H,
                                    cudaStream_t stream) {
  if (!router_logits_supported(E, H) || T <= 0) return cudaErrorInvalidValue;
  int passes = 0, gx = 0;
  long long floats = 0;
  router_logits_dw_plan(E, H, &passes, &gx, &floats);
  ++g_launch_count;
  if (E == 4) return run_dw<4, 8>(g, x, dw, partial, arrivals, gx, T, H, stream);
  if (E == 8) return run_dw<8, 8>(g, x, dw, partial, arrivals, gx, T, H, stream);
  return run_dw<16, 4>(g, x, dw, partial, arrivals, gx, T, H, stream);
}

}  // namespace mts
