// Top-k router post-processing (forward / backward), the routing plan for grouped GEMMs, and the
// gather / combine kernels around the expert GEMMs.
//
// Reference counterparts: minitrain/kernels/triton/router.py:61-259 (router),
// fused_moe_kernels.py:25-234 (histogram / prefix-sum / scatter) and :451-498 (weighted gather-sum).
// The plan here replaces the sort + associative scan by per-block counting: deterministic, token order
// is preserved inside every expert, and each expert segment is padded to a multiple of 256 rows so
// that GEMM tiles never straddle two experts and padding rows contribute exact zeros.
#include "ops.cuh"
#include "debug_bounds.cuh"

#include <cuda_bf16.h>
#include <math_constants.h>

namespace mts {

namespace {

constexpr int kMaxExperts = 64;
constexpr int kMaxTopK = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---------------- router forward: one thread per token ----------------
__global__ void __launch_bounds__(256)
router_forward_kernel(const float* __restrict__ logits, int T, int E, int K, int normalize, float* __restrict__ weights,
                      int* __restrict__ indices, float* __restrict__ row_lse, float* __restrict__ sums) {
  // sums: [0, E) probability mass per expert, [E] sum of lse^2, [E + 1] sum of entropies, [E + 2, 2E + 2) routes per expert
  extern __shared__ float block_sums[];   // [2E + 2]
  for (int i = threadIdx.x; i < 2 * E + 2; i += blockDim.x) block_sums[i] = 0.f;
  __syncthreads();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  float p[kMaxExperts];
  float lse = 0.f, ent = 0.f;
  const bool live = t < T;
  if (live) {
    float mx = -CUDART_INF_F;
    for (int e = 0; e < E; ++e) {
      p[e] = logits[(long long)t * E + e];
      mx = fmaxf(mx, p[e]);
    }
    float s = 0.f;
    for (int e = 0; e < E; ++e) s += __expf(p[e] - mx);
    lse = mx + __logf(s);
    for (int e = 0; e < E; ++e) {
      p[e] = __expf(p[e] - lse);
      ent -= p[e] * __logf(fmaxf(p[e], 1e-9f));
    }
    row_lse[t] = lse;
    // k rounds of arg-max with knockout; ties resolve to the lowest expert id
    float chosen_w[kMaxTopK];
    int chosen_i[kMaxTopK];
    unsigned long long taken = 0ull;
    float wsum = 0.f;
    for (int k = 0; k < K; ++k) {
      int best = -1;
      float bv = -1.f;
      for (int e = 0; e < E; ++e)
        if (!((taken >> e) & 1ull) && p[e] > bv) { bv = p[e]; best = e; }
      taken |= 1ull << best;
      chosen_w[k] = bv;
      chosen_i[k] = best;
      wsum += bv;
    }
    const float inv = normalize ? 1.f / fmaxf(wsum, 1.1920929e-07f) : 1.f;
    for (int k = 0; k < K; ++k) {
      weights[(long long)t * K + k] = chosen_w[k] * inv;
      indices[(long long)t * K + k] = chosen_i[k];
      atomicAdd(&block_sums[E + 2 + chosen_i[k]], 1.f);
    }
  }
  // CTA-level reduction of the statistics, then one atomic per value per CTA
  for (int e = 0; e < E; ++e) {
    const float v = warp_sum(live ? p[e] : 0.f);
    if ((threadIdx.x & 31) == 0) atomicAdd(&block_sums[e], v);
  }
  const float z = warp_sum(live ? lse * lse : 0.f);
  const float h = warp_sum(live ? ent : 0.f);
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(&block_sums[E], z);
    atomicAdd(&block_sums[E + 1], h);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * E + 2; i += blockDim.x) atomicAdd(sums + i, block_sums[i]);
}

// Load-balance figures of one routing decision from the per-expert route counts, one warp:
// out = [max count, min count, coefficient of variation of the load, max load / mean load, experts without a route,
//        load fraction of every expert ...].  (The framework-op form of the same numbers is a dozen launches and, through
// the histogram's size query, a host synchronisation per layer.)
__global__ void router_balance_kernel(const float* __restrict__ counts, int E, float n_routes, float* __restrict__ out) {
  const int lane = threadIdx.x;
  float mx = -CUDART_INF_F, mn = CUDART_INF_F, sum = 0.f, sq = 0.f, dead = 0.f;
  const float inv_routes = 1.f / fmaxf(n_routes, 1.f);
  for (int e = lane; e < E; e += 32) {
    const float c = counts[e];
    const float load = c * inv_routes;
    mx = fmaxf(mx, c); mn = fminf(mn, c);
    sum += load; sq += load * load;
    dead += c == 0.f ? 1.f : 0.f;
    out[5 + e] = load;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    sum += __shfl_xor_sync(0xffffffffu, sum, o);
    sq += __shfl_xor_sync(0xffffffffu, sq, o);
    dead += __shfl_xor_sync(0xffffffffu, dead, o);
  }
  if (lane == 0) {
    const float mean = sum / float(E);
    const float var = fmaxf(sq / float(E) - mean * mean, 0.f);
    out[0] = mx; out[1] = mn;
    out[2] = sqrtf(var) * float(E);            // std / (1 / E)
    out[3] = mx * inv_routes * float(E);       // max load / (1 / E)
    out[4] = dead;
  }
}

// ---------------- router backward ----------------
// mean_prob[e] = sum_t p[t,e] / T ; z = sum_t lse^2 / T ; w = top-k(p) (renormalised)
__global__ void __launch_bounds__(256)
router_backward_kernel(const float* __restrict__ logits, const float* __restrict__ row_lse, const int* __restrict__ indices,
                       const float* __restrict__ weights, const float* __restrict__ g_weights,
                       const float* __restrict__ g_mean_prob, const float* __restrict__ g_zloss, int T, int E, int K,
                       int normalize, float* __restrict__ g_logits) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const float lse = row_lse[t];
  const float inv_t = 1.f / float(T);
  float p[kMaxExperts], dp[kMaxExperts];
  for (int e = 0; e < E; ++e) {
    p[e] = __expf(logits[(long long)t * E + e] - lse);
    dp[e] = g_mean_prob != nullptr ? g_mean_prob[e] * inv_t : 0.f;
  }
  if (g_weights != nullptr) {
    float denom = 1.f, inner = 0.f;
    if (normalize) {
      float s = 0.f;
      for (int k = 0; k < K; ++k) {
        const int e = indices[(long long)t * K + k];
        if (e < 0) continue;                       // dropped route: no weight, no gradient
        s += p[e];
        inner += g_weights[(long long)t * K + k] * weights[(long long)t * K + k];
      }
      denom = fmaxf(s, 1.1920929e-07f);
    }
    for (int k = 0; k < K; ++k) {
      const int e = indices[(long long)t * K + k];
      if (e < 0) continue;
      const float g = g_weights[(long long)t * K + k];
      dp[e] += normalize ? (g - inner) / denom : g;
    }
  }
  float pd = 0.f;
  for (int e = 0; e < E; ++e) pd += p[e] * dp[e];
  const float zc = g_zloss != nullptr ? (*g_zloss) * 2.f * lse * inv_t : 0.f;
  for (int e = 0; e < E; ++e) g_logits[(long long)t * E + e] = p[e] * (dp[e] - pd + zc);
}

// ---------------- routing plan ----------------
constexpr int kPlanBlock = 1024;   // routes per CTA

// Pass 1: per-CTA expert histogram.
__global__ void __launch_bounds__(kPlanBlock)
plan_count_kernel(const int* __restrict__ indices, int n_routes, int E, int* __restrict__ block_counts) {
  __shared__ int hist[kMaxExperts];
  if (threadIdx.x < E) hist[threadIdx.x] = 0;
  __syncthreads();
  const int i = blockIdx.x * kPlanBlock + threadIdx.x;
  if (i < n_routes) {
    const int e = indices[i];
    if (e >= 0 && e < E) atomicAdd(&hist[e], 1);   // negative ids mark dropped routes / empty slots
  }
  __syncthreads();
  if (threadIdx.x < E) block_counts[blockIdx.x * E + threadIdx.x] = hist[threadIdx.x];
}

// Expert segments start on multiples of this many rows: two 128-row tiles, so that a 256-row work item of the
// two-CTA GEMM never straddles two experts.
constexpr int kSegmentPad = 256;

// Pass 2 (one CTA): exclusive scan over CTAs for every expert, padded expert offsets, tile -> expert map.
constexpr int kScanThreads = 1024;
__global__ void __launch_bounds__(kScanThreads)
plan_scan_kernel(int* __restrict__ block_counts, int n_blocks, int E, int capacity_rows, int* __restrict__ group_rows,
                 int* __restrict__ tile_group, int* __restrict__ meta) {
  __shared__ int totals[kMaxExperts];
  __shared__ int starts[kMaxExperts + 1];
  // one warp per expert, 32 CTAs' counts per step: a shuffle scan instead of a chain of n_blocks dependent loads
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  for (int e = warp; e < E; e += n_warps) {
    int run = 0;
    for (int base = 0; base < n_blocks; base += 32) {
      const int b = base + lane;
      const int c = b < n_blocks ? block_counts[b * E + e] : 0;
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      if (b < n_blocks) block_counts[b * E + e] = run + incl - c;     // becomes the CTA's offset inside the expert
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) totals[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int row = 0;
    for (int g = 0; g < E; ++g) {
      starts[g] = row;
      row += (totals[g] + kSegmentPad - 1) / kSegmentPad * kSegmentPad;
    }
    starts[E] = row;
    meta[0] = row / 128;
    meta[1] = row;
    meta[2] = row > capacity_rows ? 1 : 0;   // overflow flag (cannot happen when capacity = T*K + E*(kSegmentPad-1) rounded up)
  }
  __syncthreads();
  for (int q = threadIdx.x; q <= E; q += blockDim.x) group_rows[q] = starts[q];
  const int max_tiles = capacity_rows / 128;
  for (int tile = threadIdx.x; tile < max_tiles; tile += blockDim.x) {
    const int row = tile * 128;
    int g = E - 1;
    for (int q = 0; q < E; ++q)
      if (row >= starts[q] && row < starts[q + 1]) { g = q; break; }
    tile_group[tile] = g;
  }
}

// Pass 3: position of every route = expert start + CTA offset + rank among earlier routes of the CTA.
__global__ void __launch_bounds__(kPlanBlock)
plan_place_kernel(const int* __restrict__ indices, int n_routes, int K, int E, const int* __restrict__ block_counts,
                  const int* __restrict__ group_rows, int capacity_rows, int* __restrict__ row_token,
                  int* __restrict__ token_rows) {
  __shared__ int warp_hist[kPlanBlock / 32][kMaxExperts];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int i = blockIdx.x * kPlanBlock + threadIdx.x;
  int e = i < n_routes ? indices[i] : -1;
  if (e >= E) e = -1;
  for (int q = lane; q < E; q += 32) warp_hist[warp][q] = 0;
  __syncwarp();
  // rank inside the warp among lanes with the same expert
  const unsigned peers = __match_any_sync(0xffffffffu, e);
  const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (e >= 0 && rank_in_warp == 0) warp_hist[warp][e] = __popc(peers);
  __syncthreads();
  if (e >= 0) {
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_hist[w][e];
    const int row = group_rows[e] + block_counts[blockIdx.x * E + e] + before + rank_in_warp;
    if (row < capacity_rows) {
      row_token[row] = i / K;
      token_rows[i] = row;
    } else {
      token_rows[i] = -1;
    }
  } else if (i < n_routes) {
    token_rows[i] = -1;      // a dropped route has no row: the combine kernels skip it
  }
}

__global__ void fill_int_kernel(int* __restrict__ p, int value, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    p[i] = value;
}

// ---------------- gather / combine ----------------
__device__ __forceinline__ void bf16x8_to_float(const uint4& q, float (&v)[8]) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
    v[2 * i] = __low2float(h);
    v[2 * i + 1] = __high2float(h);
  }
}

__device__ __forceinline__ uint4 float_to_bf16x8(const float (&v)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// One warp per sorted row.
__global__ void __launch_bounds__(256)
moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_token, __nv_bfloat16* __restrict__ xs,
                  int H, const int* __restrict__ meta, int tokens) {
  const int live_rows = meta[1];
  const int lane = threadIdx.x & 31;
  for (int row = blockIdx.x * 8 + (threadIdx.x >> 5); row < live_rows; row += gridDim.x * 8) {
    const int tok = row_token[row];
    uint4* dst = reinterpret_cast<uint4*>(xs + (long long)row * H);
    if (tok >= 0 && MTS_IN_BOUNDS(dbg::KERNEL_MOE_GATHER, tok, tokens)) {
      const uint4* src = reinterpret_cast<const uint4*>(x + (long long)tok * H);
      for (int v = lane; v < H / 8; v += 32) dst[v] = src[v];
    } else {
      for (int v = lane; v < H / 8; v += 32) dst[v] = make_uint4(0, 0, 0, 0);
    }
  }
}

// One warp per token: out[t] = sum_k w[t,k] * y[row(t,k)].
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ token_rows,
                   const __nv_bfloat16* __restrict__ weights, __nv_bfloat16* __restrict__ out, int T, int K, int H, int y_rows) {
  const int lane = threadIdx.x & 31;
  for (int t = blockIdx.x * 8 + (threadIdx.x >> 5); t < T; t += gridDim.x * 8) {
    for (int v = lane; v < H / 8; v += 32) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int k = 0; k < K; ++k) {
        const int row = token_rows[(long long)t * K + k];
        if (row < 0 || !MTS_IN_BOUNDS(dbg::KERNEL_MOE_COMBINE, row, y_rows)) continue;
        const float w = weights != nullptr ? __bfloat162float(weights[(long long)t * K + k]) : 1.f;
        float val[8];
        bf16x8_to_float(reinterpret_cast<const uint4*>(y + (long long)row * H)[v], val);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += w * val[j];
      }
      reinterpret_cast<uint4*>(out + (long long)t * H)[v] = float_to_bf16x8(acc);
    }
  }
}

// One warp per sorted row: dys[r] = w * dout[token]; dweights[route] = <dout[token], y[r]>.
__global__ void __launch_bounds__(256)
moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y,
                       const int* __restrict__ row_token, const int* __restrict__ token_rows,
                       const __nv_bfloat16* __restrict__ weights, __nv_bfloat16* __restrict__ dys,
                       float* __restrict__ dweights, int K, int H, const int* __restrict__ meta, int tokens) {
  const int live_rows = meta[1];
  const int lane = threadIdx.x & 31;
  for (int row = blockIdx.x * 8 + (threadIdx.x >> 5); row < live_rows; row += gridDim.x * 8) {
    const int tok = row_token[row];
    uint4* dst = reinterpret_cast<uint4*>(dys + (long long)row * H);
    if (tok < 0 || !MTS_IN_BOUNDS(dbg::KERNEL_MOE_COMBINE_BWD, tok, tokens)) {
      for (int v = lane; v < H / 8; v += 32) dst[v] = make_uint4(0, 0, 0, 0);
      continue;
    }
    int route = -1;
    for (int k = 0; k < K; ++k)
      if (token_rows[(long long)tok * K + k] == row) route = tok * K + k;
    const float w = route >= 0 ? __bfloat162float(weights[route]) : 0.f;
    float dot = 0.f;
    for (int v = lane; v < H / 8; v += 32) {
      float g[8], yv[8];
      bf16x8_to_float(reinterpret_cast<const uint4*>(dout + (long long)tok * H)[v], g);
      bf16x8_to_float(reinterpret_cast<const uint4*>(y + (long long)row * H)[v], yv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dot += g[j] * yv[j];
        g[j] *= w;
      }
      dst[v] = float_to_bf16x8(g);
    }
    dot = warp_sum(dot);
    if (lane == 0 && route >= 0 && dweights != nullptr) dweights[route] = dot;
  }
}

// Per sorted row: the route it carries (t * K + k, or -1 on a padding row) and that route's weight (0 on padding rows).
// The grouped expert GEMMs read both in their SwiGLU epilogues.
__global__ void __launch_bounds__(256)
moe_row_meta_kernel(const int* __restrict__ row_token, const int* __restrict__ token_rows, const __nv_bfloat16* __restrict__ weights,
                    float* __restrict__ row_weight, int* __restrict__ row_slot, int rows, int K, int tokens) {
  for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < rows; row += gridDim.x * blockDim.x) {
    const int tok = row_token[row];
    int slot = -1;
    if (tok >= 0 && tok < tokens) {
      for (int k = 0; k < K; ++k)
        if (token_rows[(long long)tok * K + k] == row) slot = tok * K + k;
    }
    row_slot[row] = slot;
    row_weight[row] = slot >= 0 ? __bfloat162float(weights[slot]) : 0.f;
  }
}

int capped_grid(long long items, int per_block) {
  long long b = (items + per_block - 1) / per_block;
  const long long cap = (long long)device_sm_count() * 16;
  if (b > cap) b = cap;
  return b < 1 ? 1 : int(b);
}

}  // namespace

cudaError_t launch_router_forward(const float* logits, int T, int E, int K, bool normalize, float* weights, int* indices,
                                  float* row_lse, float* sums, float* balance, cudaStream_t stream) {
  if (E > kMaxExperts || K > kMaxTopK || K > E || T <= 0) return cudaErrorInvalidValue;
  router_forward_kernel<<<(T + 255) / 256, 256, sizeof(float) * (2 * E + 2), stream>>>(logits, T, E, K, normalize ? 1 : 0,
                                                                                       weights, indices, row_lse, sums);
  ++g_launch_count;
  if (balance != nullptr) {
    router_balance_kernel<<<1, 32, 0, stream>>>(sums + E + 2, E, float(T) * float(K), balance);
    ++g_launch_count;
  }
  return cudaGetLastError();
}

cudaError_t launch_router_backward(const float* logits, const float* row_lse, const int* indices, const float* weights,
                                   const float* g_weights, const float* g_mean_prob, const float* g_zloss, int T, int E,
                                   int K, bool normalize, float* g_logits, cudaStream_t stream) {
  if (E > kMaxExperts || K > kMaxTopK || T <= 0) return cudaErrorInvalidValue;
  router_backward_kernel<<<(T + 255) / 256, 256, 0, stream>>>(logits, row_lse, indices, weights, g_weights, g_mean_prob,
                                                              g_zloss, T, E, K, normalize ? 1 : 0, g_logits);
  ++g_launch_count;
  return cudaGetLastError();
}

size_t moe_plan_workspace_ints(int T, int K, int E) {
  const long long routes = (long long)T * K;
  return size_t((routes + kPlanBlock - 1) / kPlanBlock) * size_t(E);
}

cudaError_t launch_moe_plan(const int* indices, int T, int K, int E, int capacity_rows, int* row_token, int* token_rows,
                            int* tile_group, int* group_rows, int* meta, int* workspace, cudaStream_t stream) {
  if (E > kMaxExperts || capacity_rows % 128 != 0) return cudaErrorInvalidValue;
  const int routes = T * K;
  const int blocks = (routes + kPlanBlock - 1) / kPlanBlock;
  fill_int_kernel<<<capped_grid(capacity_rows, 256), 256, 0, stream>>>(row_token, -1, capacity_rows);
  plan_count_kernel<<<blocks, kPlanBlock, 0, stream>>>(indices, routes, E, workspace);
  plan_scan_kernel<<<1, kScanThreads, 0, stream>>>(workspace, blocks, E, capacity_rows, group_rows, tile_group, meta);
  plan_place_kernel<<<blocks, kPlanBlock, 0, stream>>>(indices, routes, K, E, workspace, group_rows, capacity_rows,
                                                      row_token, token_rows);
  g_launch_count += 4;
  return cudaGetLastError();
}

cudaError_t launch_moe_gather(const void* x, const int* row_token, void* x_sorted, int capacity_rows, int H,
                              const int* meta, int tokens, cudaStream_t stream) {
  if (H % 8 != 0) return cudaErrorInvalidValue;
  moe_gather_kernel<<<capped_grid(capacity_rows, 8), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), row_token, static_cast<__nv_bfloat16*>(x_sorted), H, meta, tokens);
  ++g_launch_count;
  return cudaGetLastError();
}

cudaError_t launch_moe_row_meta(const int* row_token, const int* token_rows, const void* weights, float* row_weight, int* row_slot,
                                int rows, int K, int tokens, cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  moe_row_meta_kernel<<<capped_grid(rows, 256), 256, 0, stream>>>(row_token, token_rows, static_cast<const __nv_bfloat16*>(weights),
                                                                  row_weight, row_slot, rows, K, tokens);
  ++g_launch_count;
  return cudaGetLastError();
}

cudaError_t launch_moe_combine(const void* y, const int* token_rows, const void* weights, void* out, int T, int K, int H,
                               int y_rows, cudaStream_t stream) {
  if (H % 8 != 0) return cudaErrorInvalidValue;
  moe_combine_kernel<<<capped_grid(T, 8), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(y), token_rows,
                                                            static_cast<const __nv_bfloat16*>(weights),
                                                            static_cast<__nv_bfloat16*>(out), T, K, H, y_rows);
  ++g_launch_count;
  return cudaGetLastError();
}

cudaError_t launch_moe_combine_bwd(const void* dout, const void* y, const int* row_token, const int* token_rows,
                                   const void* weights, void* dys, float* dweights, int T, int K, int H,
                                   int capacity_rows, const int* meta, cudaStream_t stream) {
  if (H % 8 != 0) return cudaErrorInvalidValue;
  moe_combine_bwd_kernel<<<capped_grid(capacity_rows, 8), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(y), row_token, token_rows,
      static_cast<const __nv_bfloat16*>(weights), static_cast<__nv_bfloat16*>(dys), dweights, K, H, meta, T);
  ++g_launch_count;
  return cudaGetLastError();
}

}  // namespace mts

// ---------------------------------------------------------------------------------------------------
// Allocation-free variant of the routing plan (declaration and contract: noalloc.h).
// Same kernels as launch_moe_plan; the only difference is where the histogram scratch lives.
// ---------------------------------------------------------------------------------------------------
#include "noalloc.h"

#include <cstdio>
#include <mutex>

namespace {

constexpr int kNoAllocMaxRoutes = 1 << 20;
constexpr int kNoAllocScratchInts = (kNoAllocMaxRoutes / mts::kPlanBlock) * mts::kMaxExperts;   // 65,536 ints = 256 KiB

// Lives in the library's device image.  In host code this name is only a handle for
// cudaGetSymbolAddress; it is never passed to a kernel directly.
static __device__ __align__(256) int g_plan_scratch[kNoAllocScratchInts];

constexpr int kMaxDevices = 64;
int* g_plan_scratch_addr[kMaxDevices] = {};
std::mutex g_plan_scratch_mutex;

// Device address of the scratch array on the current device (looked up once per device).
cudaError_t plan_scratch_for_current_device(int** out) {
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_plan_scratch_mutex);
  if (g_plan_scratch_addr[device] == nullptr) {
    void* addr = nullptr;
    err = cudaGetSymbolAddress(&addr, g_plan_scratch);
    if (err != cudaSuccess) return err;
    g_plan_scratch_addr[device] = static_cast<int*>(addr);
  }
  *out = g_plan_scratch_addr[device];
  return cudaSuccess;
}

}  // namespace

extern "C" int mts_moe_plan_noalloc(const int* indices, int tokens, int top_k, int experts, int capacity_rows,
                                    int* row_token, int* token_rows, int* tile_group, int* group_rows, int* meta,
                                    void* cuda_stream) {
  if (indices == nullptr || row_token == nullptr || token_rows == nullptr || tile_group == nullptr ||
      group_rows == nullptr || meta == nullptr || tokens <= 0 || top_k <= 0 || experts <= 0 || capacity_rows <= 0 ||
      capacity_rows % 128 != 0) {
    std::fprintf(stderr, "mts_moe_plan_noalloc: invalid argument (null pointer, non-positive size, or capacity_rows "
                         "not a multiple of 128)\n");
    return -2;
  }
  const long long routes = static_cast<long long>(tokens) * top_k;
  if (routes > kNoAllocMaxRoutes || experts > mts::kMaxExperts) {
    std::fprintf(stderr, "mts_moe_plan_noalloc: %lld routes / %d experts exceed the built-in scratch "
                         "(limit: %d routes, %d experts)\n", routes, experts, kNoAllocMaxRoutes, mts::kMaxExperts);
    return -1;
  }
  int* scratch = nullptr;
  const cudaError_t lookup = plan_scratch_for_current_device(&scratch);
  if (lookup != cudaSuccess) {
    std::fprintf(stderr, "mts_moe_plan_noalloc: scratch lookup failed: %s\n", cudaGetErrorString(lookup));
    return static_cast<int>(lookup);
  }
  const cudaError_t err = mts::launch_moe_plan(indices, tokens, top_k, experts, capacity_rows, row_token, token_rows,
                                               tile_group, group_rows, meta, scratch, static_cast<cudaStream_t>(cuda_stream));
  return static_cast<int>(err);
}
