// FlashAttention forward / backward for sm_100a (head_dim 64, bf16); interface in attention.cuh.
//
// Every CTA has 320 threads: warp 0 drives TMA, warp 1 issues tcgen05.mma, warps 2-9 do the softmax arithmetic on
// accumulators read from tensor memory, two threads per tile row: warps w and w + 4 share 32 rows and split the
// tile's columns between them, so every scheduler has four compute warps (two CTAs per SM) to hide the exp2 / TMEM
// latencies behind.  Probability / dS
// tiles that feed a second MMA are written to shared memory in the 128-byte swizzled K-major layout
// the UMMA descriptors expect.  Shared memory and TMEM budgets are sized for two CTAs per SM so one
// CTA's exponentials overlap the other's MMAs.
//
//   forward : 128 queries x 128 keys per step;  S = Q K^T -> softmax -> P V, running O in registers.
//   backward: two atomic-free sweeps.
//     dK/dV sweep: CTA owns 128 keys, streams 64-query tiles: S^T = K Q^T, dP^T = V dO^T,
//                  dV += P^T dO, dK += dS^T Q   (accumulators stay in TMEM for the whole sweep)
//     dQ sweep   : CTA owns 128 queries, streams 64-key tiles: S = Q K^T, dP = dO V^T, dQ += dS K
//
// Reference counterparts: vendored FlashAttention-2 sm80 kernels (minitrain/kernels/cuda_ext/csrc/
// third_party/flash_attn/src/flash_fwd_kernel.h:51-494, flash_bwd_kernel.h:80-841) and the Triton
// kernels in minitrain/kernels/triton/flash_attention.py:213-938.
#include "attention.cuh"
#include "ops.cuh"
#include "ptx_sm100.cuh"

#include <cudaTypedefs.h>
#include <cstdio>
#include <math_constants.h>
#include <mutex>

namespace mts {

const char* g_attn_last_error = "";

namespace {

constexpr int D = kAttnHeadDim;
constexpr int TILE128 = 128 * D * 2;   // bytes of a [128 x 64] bf16 tile
constexpr int TILE64 = 64 * D * 2;
constexpr int THREADS = 320;   // TMA warp, MMA warp, 2 x 4 compute warps (two threads per accumulator row)
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __host__ __forceinline__ uint32_t fmix32(uint32_t h) {
  h ^= h >> 16; h *= 0x85ebca6bu; h ^= h >> 13; h *= 0xc2b2ae35u; h ^= h >> 16;
  return h;
}

struct Dropout {
  uint32_t key;       // per (seed, batch*head)
  uint32_t thresh;    // drop when byte < thresh ; 0 disables
  float inv_keep;
  uint32_t words_per_row;
  __device__ __forceinline__ uint32_t word(uint32_t q, uint32_t kword) const {
    return fmix32(((q * words_per_row + kword) * 0x9E3779B1u) ^ key);
  }
  __device__ __forceinline__ bool keep(uint32_t q, uint32_t k) const {
    return ((word(q, k >> 2) >> ((k & 3u) * 8u)) & 0xFFu) >= thresh;
  }
};

__device__ __host__ __forceinline__ uint32_t dropout_key(unsigned long long seed, uint32_t bh) {
  return fmix32(uint32_t(seed) ^ fmix32(uint32_t(seed >> 32) + bh * 0x9E3779B9u));
}

__device__ __forceinline__ Dropout make_dropout(float p, unsigned long long seed, uint32_t bh, int S) {
  Dropout d;
  d.thresh = p > 0.f ? uint32_t(p * 256.f + 0.5f) : 0u;
  d.inv_keep = 1.f / (1.f - float(d.thresh) * (1.f / 256.f));
  d.key = dropout_key(seed, bh);
  d.words_per_row = uint32_t((S + 3) / 4);
  return d;
}

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// 16-byte chunk `chunk` (0..7) of row `row` in a 128-byte-swizzled tile with 128-byte rows
__device__ __forceinline__ void st_swizzled(uint8_t* tile, int row, int chunk, uint4 v) {
  *reinterpret_cast<uint4*>(tile + row * 128 + ((chunk ^ (row & 7)) << 4)) = v;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_addr, int kstep) {   // kstep: 16 contraction elements
  return make_smem_desc_sw128(tile_addr + kstep * 32, 16, 1024);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile_addr, int kstep) {  // tile = [K rows x 64], rows of 128 B
  return make_smem_desc_sw128(tile_addr + kstep * 2048, 8192, 1024);
}

__device__ __forceinline__ void epilogue_arrive(uint64_t* bar, int lane) {
  tc_fence_before_sync();
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

__device__ __forceinline__ void store_row64(__nv_bfloat16* dst, const float (&v)[64], float mul) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint4 q;
    q.x = pack2(v[8 * j + 0] * mul, v[8 * j + 1] * mul);
    q.y = pack2(v[8 * j + 2] * mul, v[8 * j + 3] * mul);
    q.z = pack2(v[8 * j + 4] * mul, v[8 * j + 5] * mul);
    q.w = pack2(v[8 * j + 6] * mul, v[8 * j + 7] * mul);
    reinterpret_cast<uint4*>(dst)[j] = q;
  }
}

// The same store for a gradient of rotated q / k rows: v is d(rotated row) at position `pos`; what is written is the gradient of
// the row before the half-split rotation, lo' = lo cos + hi sin, hi' = hi cos - lo sin (fp32, one rounding).
__device__ __forceinline__ void store_row64_unrotated(__nv_bfloat16* dst, const float (&v)[64], float mul,
                                                      const __nv_bfloat16* cos_row, const __nv_bfloat16* sin_row) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 cq = reinterpret_cast<const uint4*>(cos_row)[j], sq = reinterpret_cast<const uint4*>(sin_row)[j];
    const uint32_t cw[4] = {cq.x, cq.y, cq.z, cq.w}, sw[4] = {sq.x, sq.y, sq.z, sq.w};
    float lo[8], hi[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t cbits = (i & 1) ? (cw[i >> 1] & 0xFFFF0000u) : (cw[i >> 1] << 16);
      const uint32_t sbits = (i & 1) ? (sw[i >> 1] & 0xFFFF0000u) : (sw[i >> 1] << 16);
      const float c = __uint_as_float(cbits) * mul, sn = __uint_as_float(sbits) * mul;
      const float a = v[8 * j + i], b = v[32 + 8 * j + i];
      lo[i] = a * c + b * sn;
      hi[i] = b * c - a * sn;
    }
    uint4 q;
    q.x = pack2(lo[0], lo[1]); q.y = pack2(lo[2], lo[3]); q.z = pack2(lo[4], lo[5]); q.w = pack2(lo[6], lo[7]);
    reinterpret_cast<uint4*>(dst)[j] = q;
    q.x = pack2(hi[0], hi[1]); q.y = pack2(hi[2], hi[3]); q.z = pack2(hi[4], hi[5]); q.w = pack2(hi[6], hi[7]);
    reinterpret_cast<uint4*>(dst)[4 + j] = q;
  }
}

// Optional phase trace of CTA (0, 0) of the forward kernel (build with -DMTS_ATTN_TRACE): slot 8*j+k of
// g_attn_trace receives clock64() when the softmax warp (k = 0..5) or the MMA thread (slot 4096 + 8*j + k)
// passes phase k of key tile j.  Compiled out by default.
#ifdef MTS_ATTN_TRACE
__device__ long long g_attn_trace[8192];
#define MTS_TRACE(slot) do { if (blockIdx.x == 0 && blockIdx.y == 0 && lane == 0) g_attn_trace[(slot)] = clock64(); } while (0)
#else
#define MTS_TRACE(slot) do { } while (0)
#endif

struct Params {
  __nv_bfloat16 *o, *dq, *dk, *dv;
  long long o_sb, o_sh, o_ss, dq_sb, dq_sh, dq_ss, dk_sb, dk_sh, dk_ss, dv_sb, dv_sh, dv_ss;
  float* lse;
  const float* delta;
  int B, H, S, causal;
  float scale, dropout_p;
  unsigned long long seed;
  const StepContext* ctx;   // seed is salted with ctx->salt (0 outside graph replay)
  int* status;
  const __nv_bfloat16 *rope_cos, *rope_sin;   // backward: un-rotate dQ / dK while storing them (nullptr = store as is)
};

// Work order of the persistent kernels.  A (batch, head) with T tiles along the CTA's own axis is cut into ceil(T / 2) pairs
// (tile T-1-i, tile i): under a causal mask a pair costs the same whatever i is, so handing pair g to CTA g % grid balances the
// CTAs without a queue, and CTAs that run at the same time work on the same or neighbouring (batch, head): the K / V (or Q /
// dO) tiles they stream are read from DRAM once and found in L2 by the others.  Slot `seq` of a CTA is the first (seq even) or
// second (seq odd) tile of its (seq / 2)-th pair; the middle tile of an odd T is a pair of one.
struct WorkItem { int tile, bh; bool valid, done; };
__device__ __forceinline__ WorkItem work_item(int seq, int T, int BH) {
  const int per_bh = (T + 1) >> 1;
  const long long pair = (long long)blockIdx.x + (long long)(seq >> 1) * gridDim.x;
  WorkItem w;
  w.done = pair >= (long long)per_bh * BH;
  w.bh = int(pair / per_bh);
  const int i = int(pair % per_bh);
  w.tile = (seq & 1) ? i : T - 1 - i;
  w.valid = !((seq & 1) && i == T - 1 - i);
  return w;
}

// =====================================================================================================
// forward
// =====================================================================================================
constexpr int FWD_SMEM = TILE128 /*Q*/ + TILE128 /*K*/ + 2 * TILE128 /*V x 2*/ + 2 * TILE128 /*P*/ + 1024;

// Persistent: the grid is two CTAs per SM and every CTA walks the work items (query tile, batch * head) it owns, in the
// order work_item() gives.  Barriers and tensor memory are set up once; the loader runs ahead into the next item (its Q as soon
// as the last Q K^T of the current item has been issued, its K / V as their buffers free up) and the MMA warp computes the
// next item's first scores while the softmax warps write the current item's output, so the latency of an item's first
// loads and the write-out of its last rows are no longer paid once per 128 query rows.  O is double-buffered in tensor
// memory (columns 128..191 and 192..255) so that the next item's first P V does not wait for that write-out.
template <bool DROPOUT>
__global__ void __launch_bounds__(THREADS, 2)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + TILE128;          // one K tile: it is free again as soon as its Q K^T has run, a whole softmax before the next is needed
  uint8_t* sV = smem + 2 * TILE128;      // two V tiles: a V tile is held until its P V has run, at the end of its key tile
  uint8_t* sP = smem + 4 * TILE128;

  __shared__ __align__(8) uint64_t q_full, q_free, k_full, k_empty, v_full[2], v_empty[2], s_full, s_free, p_ready, pv_full, o_free[2], pair_bar[4];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_word;
  __shared__ float pair_val[2][2][128];   // [exchange parity][column half][row]: what the two threads of a row tell each other

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_q_tiles = (p.S + 127) / 128;
  const int n_k_tiles = n_q_tiles;
  const int BH = p.B * p.H;
  if (warp == 0) MTS_TRACE(8000);

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1); mbar_init(&q_free, 1);
    mbar_init(&k_full, 1); mbar_init(&k_empty, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
    mbar_init(&s_full, 1); mbar_init(&s_free, 8); mbar_init(&p_ready, 8); mbar_init(&pv_full, 1);
    mbar_init(&o_free[0], 8); mbar_init(&o_free[1], 8);
    for (int i = 0; i < 4; ++i) mbar_init(&pair_bar[i], 2);
    abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 0) { tmem_alloc(&tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_s = tmem_slot, tmem_o = tmem_slot + 128;
  volatile int* abort_ptr = &abort_word;
  if (warp == 0) MTS_TRACE(8001);

  if (warp == 0) {
    if (lane == 0) {
      int kt = 0;            // key tiles loaded so far, over all items (K and V counted alike)
      int n = 0;             // items started by this CTA
      bool ok = true;
      for (int seq = 0; ok; ++seq) {
        const WorkItem w = work_item(seq, n_q_tiles, BH);
        if (w.done) break;
        if (!w.valid) continue;
        const int q_tile = w.tile, bh = w.bh, b = bh / p.H, h = bh % p.H;
        const int n_kv = p.causal ? min(n_k_tiles, q_tile + 1) : n_k_tiles;
        if (n < 20) MTS_TRACE(7800 + 8 * n + 0);
        if (n > 0 && !mbar_wait(&q_free, (n - 1) & 1, abort_ptr)) break;      // the previous item's Q K^T are all issued and done
        if (n < 20) MTS_TRACE(7800 + 8 * n + 1);
        mbar_expect_tx(&q_full, TILE128);
        tma_load_4d(sQ, &tm_q, &q_full, 0, q_tile * 128, h, b);
        for (int j = 0; j < n_kv; ++j, ++kt) {
          if (!mbar_wait(&k_empty, (kt & 1) ^ 1, abort_ptr)) { ok = false; break; }
          mbar_expect_tx(&k_full, TILE128);
          tma_load_4d(sK, &tm_k, &k_full, 0, j * 128, h, b);
          const int vs = kt & 1;
          if (!mbar_wait(&v_empty[vs], ((kt >> 1) & 1) ^ 1, abort_ptr)) { ok = false; break; }
          mbar_expect_tx(&v_full[vs], TILE128);
          tma_load_4d(sV + vs * TILE128, &tm_v, &v_full[vs], 0, j * 128, h, b);
        }
        ++n;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, 64, false, true);
      // Descriptors are built once: a 16-wide contraction step adds 2 (32 B) to a K-major descriptor and 128 (2048 B) to
      // an MN-major one; the two V tiles and the two halves of P lie TILE128 bytes (1024 descriptor units) apart.
      const uint64_t qd = desc_kmajor(smem_u32(sQ), 0), pd = desc_kmajor(smem_u32(sP), 0);
      const uint64_t kd = desc_kmajor(smem_u32(sK), 0), v_m = desc_mnmajor(smem_u32(sV), 0);
      constexpr uint64_t kSlot = TILE128 >> 4;
      int tiles = 0;         // key tiles whose scores have been issued, over all items (parity of s_full / s_free)
      int pvs = 0;           // key tiles whose P V has been issued (parity of p_ready / pv_full)
      int n = 0;
      bool ok = true;
      for (int seq = 0; ok; ++seq) {
        const WorkItem w = work_item(seq, n_q_tiles, BH);
        if (w.done) break;
        if (!w.valid) continue;
        const int q_tile = w.tile;
        const int n_kv = p.causal ? min(n_k_tiles, q_tile + 1) : n_k_tiles;
        const uint32_t tmem_pv = tmem_o + 64u * uint32_t(n & 1);
        // S_j = Q K_j^T.  The softmax warps copy S into registers right away, so S_{j+1} is issued before
        // waiting for P_j: the tensor core computes the next scores while the exponentials of tile j run.
        auto issue_scores = [&](int j) -> bool {
          if (!mbar_wait_hot(&k_full, tiles & 1, abort_ptr)) return false;
          if (!mbar_wait_hot(&s_free, (tiles & 1) ^ 1, abort_ptr)) return false;
          tc_fence_after_sync();
          umma_bf16_ss(tmem_s, qd, kd, idesc_s, 0u);
          umma_bf16_ss(tmem_s, qd + 2, kd + 2, idesc_s, 1u);
          umma_bf16_ss(tmem_s, qd + 4, kd + 4, idesc_s, 1u);
          umma_bf16_ss(tmem_s, qd + 6, kd + 6, idesc_s, 1u);
          umma_commit(&s_full);
          umma_commit(&k_empty);
          if (j == n_kv - 1) umma_commit(&q_free);       // Q may be replaced by the next item's
          ++tiles;
          return true;
        };
        if (n < 20) MTS_TRACE(7600 + 8 * n + 0);
        if (!mbar_wait(&q_full, n & 1, abort_ptr)) break;
        if (n < 20) MTS_TRACE(7600 + 8 * n + 1);
        if (!issue_scores(0)) break;
        if (n < 20) MTS_TRACE(7600 + 8 * n + 2);
        for (int j = 0; j < n_kv; ++j, ++pvs) {
          const int vs = pvs & 1;
          if (n == 0) MTS_TRACE(4096 + 8 * j + 0);
          if (j + 1 < n_kv && !issue_scores(j + 1)) { ok = false; break; }
          if (n == 0) MTS_TRACE(4096 + 8 * j + 1);
          if (!mbar_wait_hot(&p_ready, pvs & 1, abort_ptr)) { ok = false; break; }
          if (n == 0) MTS_TRACE(4096 + 8 * j + 2);
          // the write-out of the item that used this O buffer two items ago has read it
          if (j == 0 && n >= 2 && !mbar_wait_hot(&o_free[n & 1], ((n >> 1) - 1) & 1, abort_ptr)) { ok = false; break; }
          if (!mbar_wait_hot(&v_full[vs], (pvs >> 1) & 1, abort_ptr)) { ok = false; break; }
          tc_fence_after_sync();
          const uint64_t vm = v_m + vs * kSlot;
          umma_bf16_ss(tmem_pv, pd, vm, idesc_pv, j != 0 ? 1u : 0u);
          umma_bf16_ss(tmem_pv, pd + 2, vm + 128, idesc_pv, 1u);
          umma_bf16_ss(tmem_pv, pd + 4, vm + 256, idesc_pv, 1u);
          umma_bf16_ss(tmem_pv, pd + 6, vm + 384, idesc_pv, 1u);
          umma_bf16_ss(tmem_pv, pd + kSlot, vm + 512, idesc_pv, 1u);
          umma_bf16_ss(tmem_pv, pd + kSlot + 2, vm + 640, idesc_pv, 1u);
          umma_bf16_ss(tmem_pv, pd + kSlot + 4, vm + 768, idesc_pv, 1u);
          umma_bf16_ss(tmem_pv, pd + kSlot + 6, vm + 896, idesc_pv, 1u);
          umma_commit(&pv_full);
          if (n == 0) MTS_TRACE(4096 + 8 * j + 3);
          umma_commit(&v_empty[vs]);
        }
        ++n;
      }
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;             // the 32 tensor-memory lanes (tile rows) this warp may read
    const int half = (warp - 2) >> 2;         // key columns 64 * half .. + 63 of every tile; output columns 32 * half .. + 31
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const float scale_log2 = p.scale * LOG2E;
    uint8_t* const p_half = sP + half * TILE128;
    // The two threads of a row exchange one float per tile (their half-row maximum) and one per item (their half-row sum)
    // through shared memory; an mbarrier with two arrivals (one per warp) orders the exchange and inherits the bounded wait.
    int pair_phase = 0;
    auto exchange = [&](float mine, float& other) -> bool {
      const int parity = pair_phase & 1;
      pair_val[parity][half][r] = mine;
      __syncwarp();
      if (lane == 0) mbar_arrive(&pair_bar[quarter]);
      if (!mbar_wait_warp(&pair_bar[quarter], parity, abort_ptr, lane)) return false;
      ++pair_phase;
      __syncwarp();                             // lane 0 observed the phase: order the other lanes' reads behind it
      other = pair_val[parity][half ^ 1][r];
      return true;
    };
    // Running maximum m (log2 units, may lag the true maximum by up to kRescaleSlack), running sum l of this thread's columns.
    // O stays in tensor memory: every P V MMA accumulates into it, and it is only read back and rescaled when
    // the maximum of some row of this warp moved by more than the slack (stale maxima keep exp2 arguments
    // below 2^slack, which fp32 sums and bf16 probabilities hold without loss).
    constexpr float kRescaleSlack = 8.f;
    int tiles = 0;           // key tiles processed, over all items: parity of s_full / pv_full
    int n = 0;
    bool ok = true;
    for (int seq = 0; ok; ++seq) {
      const WorkItem w = work_item(seq, n_q_tiles, BH);
      if (w.done) break;
      if (!w.valid) continue;
      const int q_tile = w.tile, bh = w.bh, b = bh / p.H, h = bh % p.H;
      const int n_kv = p.causal ? min(n_k_tiles, q_tile + 1) : n_k_tiles;
      const int q0 = q_tile * 128, q_row = q0 + r;
      const uint32_t tmem_pv = tmem_o + 64u * uint32_t(n & 1);
      const Dropout drop = make_dropout(p.dropout_p, p.seed + p.ctx->salt * kSaltMultiplier, uint32_t(bh), p.S);
      float m = -CUDART_INF_F, l = 0.f;
      if (warp == 2 && n < 60) MTS_TRACE(7000 + 8 * n + 0);
      for (int j = 0; j < n_kv; ++j, ++tiles) {
        if (!mbar_wait_warp(&s_full, tiles & 1, abort_ptr, lane)) { ok = false; break; }
        if (warp == 2 && n == 0) MTS_TRACE(8 * j + 0);
        if (warp == 2 && n < 60 && j == 0) MTS_TRACE(7000 + 8 * n + 1);
        tc_fence_after_sync();
        const int k0 = j * 128 + half * 64;
        const bool need_mask = (p.causal && k0 + 63 > q0) || (k0 + 64 > p.S);
        uint32_t s0[32], s1[32];
        tmem_ld_32x32(tmem_s + lane_base + half * 64, s0);
        tmem_ld_32x32(tmem_s + lane_base + half * 64 + 32, s1);
        tmem_ld_wait();
        epilogue_arrive(&s_free, lane);            // S is in registers: the next Q K^T may overwrite it
        if (warp == 2 && n == 0) MTS_TRACE(8 * j + 1);
        if (need_mask) {       // one uniform branch around the loop (diagonal and ragged tiles only); selects inside, no branches
          const int last = min(p.S - 1, p.causal ? q_row : 0x7fffffff) - k0;    // last column of this thread's 64 that is kept
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            s0[i] = i > last ? __float_as_uint(-CUDART_INF_F) : s0[i];
            s1[i] = i + 32 > last ? __float_as_uint(-CUDART_INF_F) : s1[i];
          }
        }
        float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};   // four independent max chains
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          mx4[0] = fmaxf(mx4[0], __uint_as_float(s0[i]));
          mx4[1] = fmaxf(mx4[1], __uint_as_float(s0[16 + i]));
          mx4[2] = fmaxf(mx4[2], __uint_as_float(s1[i]));
          mx4[3] = fmaxf(mx4[3], __uint_as_float(s1[16 + i]));
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])), mx_other;
        if (!exchange(mx, mx_other)) { ok = false; break; }
        mx = fmaxf(mx, mx_other);
        if (warp == 2 && n == 0) MTS_TRACE(8 * j + 4);
        const float m_tile = mx * scale_log2;
        float alpha = 1.f;
        bool grow = false;
        if (j == 0) {
          // the last P V of the previous item was awaited before its write-out: P is free, and this item's O buffer is
          // handed over by the MMA warp (it waits for the write-out that last read it)
          m = m_tile == -CUDART_INF_F ? 0.f : m_tile;
        } else {
          // previous P V must be complete: its P tile is about to be overwritten and O may be rescaled
          if (!mbar_wait_warp(&pv_full, (tiles - 1) & 1, abort_ptr, lane)) { ok = false; break; }
          tc_fence_after_sync();
          if (warp == 2 && n == 0) MTS_TRACE(8 * j + 5);
          grow = m_tile > m + kRescaleSlack;        // the same decision in both threads of a row: m and m_tile are shared
          if (__any_sync(0xffffffffu, grow)) {
            if (grow) { alpha = ex2(m - m_tile); m = m_tile; l *= alpha; }
#pragma unroll 1
            for (int c = 2 * half; c < 2 * half + 2; ++c) {   // rare path: this thread's 32 of the 64 output columns
              uint32_t oo[16];
              tmem_ld_32x16(tmem_pv + lane_base + c * 16, oo);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) oo[i] = __float_as_uint(__uint_as_float(oo[i]) * alpha);
              tmem_st_32x16(tmem_pv + lane_base + c * 16, oo);
            }
            tmem_st_wait();
          }
        }
        float rowsum[8];                          // eight independent partial sums: one accumulator would chain 64 dependent adds
#pragma unroll
        for (int i = 0; i < 8; ++i) rowsum[i] = 0.f;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t (&rr)[32] = c == 0 ? s0 : s1;
#pragma unroll
          for (int g = 0; g < 4; ++g) {            // eight probabilities at a time: exp, dropout, pack, store
            float e[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              e[i] = ex2(fmaf(__uint_as_float(rr[8 * g + i]), scale_log2, -m));   // masked entries are -inf -> 0
              rowsum[i] += e[i];
            }
            if (DROPOUT) {
#pragma unroll
              for (int w = 0; w < 2; ++w) {
                const uint32_t bits = drop.word(uint32_t(q_row), uint32_t(k0 + c * 32 + 8 * g + 4 * w) >> 2);
#pragma unroll
                for (int t = 0; t < 4; ++t)
                  e[4 * w + t] = ((bits >> (8 * t)) & 0xFFu) >= drop.thresh ? e[4 * w + t] : 0.f;   // 1 / keep: applied to O at the end
              }
            }
            uint4 q4;
            q4.x = pack2(e[0], e[1]); q4.y = pack2(e[2], e[3]); q4.z = pack2(e[4], e[5]); q4.w = pack2(e[6], e[7]);
            st_swizzled(p_half, r, c * 4 + g, q4);
          }
        }
        l += ((rowsum[0] + rowsum[1]) + (rowsum[2] + rowsum[3])) + ((rowsum[4] + rowsum[5]) + (rowsum[6] + rowsum[7]));
        if (warp == 2 && n == 0) MTS_TRACE(8 * j + 2);
        fence_proxy_async_smem();                  // P (generic-proxy stores) -> visible to the tensor core
        epilogue_arrive(&p_ready, lane);
        if (warp == 2 && n == 0) MTS_TRACE(8 * j + 3);
      }
      if (!ok) break;
      if (warp == 2 && n < 60) MTS_TRACE(7000 + 8 * n + 2);
      float l_other = 0.f;
      if (!exchange(l, l_other)) { ok = false; break; }
      if (!mbar_wait_warp(&pv_full, (tiles - 1) & 1, abort_ptr, lane)) { ok = false; break; }
      tc_fence_after_sync();
      if (warp == 2 && n < 60) MTS_TRACE(7000 + 8 * n + 3);
      l += l_other;
      uint32_t rr[32];
      tmem_ld_32x32(tmem_pv + lane_base + half * 32, rr);
      tmem_ld_wait();
      epilogue_arrive(&o_free[n & 1], lane);       // O is in registers: the buffer may take the item after the next
      if (warp == 2 && n < 60) MTS_TRACE(7000 + 8 * n + 4);
      if (q_row < p.S) {
        const float inv_l = l > 0.f ? (DROPOUT ? drop.inv_keep : 1.f) / l : 0.f;
        __nv_bfloat16* dst = p.o + (long long)b * p.o_sb + (long long)h * p.o_sh + (long long)q_row * p.o_ss + half * 32;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          uint4 q;
          q.x = pack2(__uint_as_float(rr[8 * jj + 0]) * inv_l, __uint_as_float(rr[8 * jj + 1]) * inv_l);
          q.y = pack2(__uint_as_float(rr[8 * jj + 2]) * inv_l, __uint_as_float(rr[8 * jj + 3]) * inv_l);
          q.z = pack2(__uint_as_float(rr[8 * jj + 4]) * inv_l, __uint_as_float(rr[8 * jj + 5]) * inv_l);
          q.w = pack2(__uint_as_float(rr[8 * jj + 6]) * inv_l, __uint_as_float(rr[8 * jj + 7]) * inv_l);
          reinterpret_cast<uint4*>(dst)[jj] = q;
        }
        if (half == 0) p.lse[((long long)bh) * p.S + q_row] = (m + log2f(l)) * LN2;
      }
      if (warp == 2 && n < 60) MTS_TRACE(7000 + 8 * n + 5);
      ++n;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && abort_word != 0) {
    __nanosleep(50000);   // bounded grace period for bulk copies still in flight
    if (p.status != nullptr) atomicMax(p.status, abort_word);
  }
  __syncthreads();
  if (warp == 0) MTS_TRACE(8003);
  if (warp == 0) tmem_dealloc(tmem_slot, 256);
}

// =====================================================================================================
// backward, sweep 1: dK / dV.  CTA = 128 keys; streams 64-query tiles.
// =====================================================================================================
constexpr int BWD_KV_SMEM = 2 * TILE128 /*K,V*/ + 4 * TILE64 /*Q,dO x 2 stages*/ + 2 * TILE128 /*P^T, dS^T*/ + 2048 /*lse, delta*/ + 1024;

template <bool DROPOUT>
__global__ void __launch_bounds__(THREADS, 2)
flash_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tm_q64, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do64, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + TILE128;
  uint8_t* sQ = smem + 2 * TILE128;                 // 2 stages x 8 KB
  uint8_t* sDO = smem + 2 * TILE128 + 2 * TILE64;   // 2 stages x 8 KB
  uint8_t* sP = smem + 2 * TILE128 + 4 * TILE64;    // [128 keys x 64 q]
  uint8_t* sDS = sP + TILE128;
  uint8_t* sStats = sDS + TILE128;                  // 8 warps x 256 B

  __shared__ __align__(8) uint64_t kv_full, qd_full[2], qd_empty[2], st_full, st_free, pds_ready, pds_free, acc_full;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_word;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_k_tiles = (p.S + 127) / 128;
  const int k_tile = int(blockIdx.x);   // early key tiles see the most queries and are scheduled first
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int k0 = k_tile * 128;
  const int n_q64 = (p.S + 63) / 64;
  const int first_q = p.causal ? k0 / 64 : 0;
  const int n_iter = n_q64 - first_q;
  (void)n_k_tiles;

  if (threadIdx.x == 0) {
    mbar_init(&kv_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&qd_full[i], 1); mbar_init(&qd_empty[i], 1); }
    mbar_init(&st_full, 1); mbar_init(&st_free, 8); mbar_init(&pds_ready, 8); mbar_init(&pds_free, 1); mbar_init(&acc_full, 1);
    abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 0) { tmem_alloc(&tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t t_st = tmem_slot, t_dp = tmem_slot + 64, t_dv = tmem_slot + 128, t_dk = tmem_slot + 192;
  volatile int* abort_ptr = &abort_word;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&kv_full, 2 * TILE128);
      tma_load_4d(sK, &tm_k, &kv_full, 0, k0, h, b);
      tma_load_4d(sV, &tm_v, &kv_full, 0, k0, h, b);
      for (int i = 0; i < n_iter; ++i) {
        const int s = i & 1;
        if (!mbar_wait(&qd_empty[s], ((i >> 1) & 1) ^ 1, abort_ptr)) break;
        mbar_expect_tx(&qd_full[s], 2 * TILE64);
        tma_load_4d(sQ + s * TILE64, &tm_q64, &qd_full[s], 0, (first_q + i) * 64, h, b);
        tma_load_4d(sDO + s * TILE64, &tm_do64, &qd_full[s], 0, (first_q + i) * 64, h, b);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_st = make_idesc_bf16(128, 64, false, false);   // [128 keys x 64 q], both K-major
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, 64, false, true);   // B = [q rows x 64 d] read MN-major
      // This one thread feeds the tensor core, so its instruction stream is kept short: every descriptor is built once;
      // a 16-wide contraction step adds 2 (32 B) to a K-major descriptor and 128 (2048 B) to an MN-major one, and the
      // second Q / dO stage lies TILE64 bytes (512 descriptor units) after the first.
      const uint64_t kd = desc_kmajor(smem_u32(sK), 0), vd = desc_kmajor(smem_u32(sV), 0);
      const uint64_t pd = desc_kmajor(smem_u32(sP), 0), dsd = desc_kmajor(smem_u32(sDS), 0);
      const uint64_t qk0 = desc_kmajor(smem_u32(sQ), 0), dok0 = desc_kmajor(smem_u32(sDO), 0);
      const uint64_t qm0 = desc_mnmajor(smem_u32(sQ), 0), dom0 = desc_mnmajor(smem_u32(sDO), 0);
      constexpr uint64_t kStage = TILE64 >> 4;
      // S^T_i = K Q_i^T and dP^T_i = V dO_i^T.  The compute warps copy both to registers early in their iteration, so the
      // scores of tile i+1 are issued before waiting for P^T_i / dS^T_i and run while tile i is being processed.
      auto issue_scores = [&](int i) -> bool {
        const int s = i & 1;
        if (!mbar_wait_hot(&qd_full[s], (i >> 1) & 1, abort_ptr)) return false;
        if (!mbar_wait_hot(&st_free, (i & 1) ^ 1, abort_ptr)) return false;
        tc_fence_after_sync();
        const uint64_t q = qk0 + s * kStage, d_o = dok0 + s * kStage;
        umma_bf16_ss(t_st, kd, q, idesc_st, 0u);
        umma_bf16_ss(t_st, kd + 2, q + 2, idesc_st, 1u);
        umma_bf16_ss(t_st, kd + 4, q + 4, idesc_st, 1u);
        umma_bf16_ss(t_st, kd + 6, q + 6, idesc_st, 1u);
        umma_bf16_ss(t_dp, vd, d_o, idesc_st, 0u);
        umma_bf16_ss(t_dp, vd + 2, d_o + 2, idesc_st, 1u);
        umma_bf16_ss(t_dp, vd + 4, d_o + 4, idesc_st, 1u);
        umma_bf16_ss(t_dp, vd + 6, d_o + 6, idesc_st, 1u);
        umma_commit(&st_full);
        return true;
      };
      bool ok = mbar_wait(&kv_full, 0, abort_ptr);
      ok = ok && (n_iter <= 0 || issue_scores(0));
      for (int i = 0; i < n_iter && ok; ++i) {
        const int s = i & 1;
        MTS_TRACE(4096 + 8 * i + 0);
        if (i + 1 < n_iter && !issue_scores(i + 1)) break;
        MTS_TRACE(4096 + 8 * i + 1);
        if (!mbar_wait_hot(&pds_ready, i & 1, abort_ptr)) break;
        MTS_TRACE(4096 + 8 * i + 2);
        tc_fence_after_sync();
        const uint64_t qm = qm0 + s * kStage, dom = dom0 + s * kStage;
        const uint32_t acc = i != 0 ? 1u : 0u;
        umma_bf16_ss(t_dv, pd, dom, idesc_acc, acc);
        umma_bf16_ss(t_dv, pd + 2, dom + 128, idesc_acc, 1u);
        umma_bf16_ss(t_dv, pd + 4, dom + 256, idesc_acc, 1u);
        umma_bf16_ss(t_dv, pd + 6, dom + 384, idesc_acc, 1u);
        umma_bf16_ss(t_dk, dsd, qm, idesc_acc, acc);
        umma_bf16_ss(t_dk, dsd + 2, qm + 128, idesc_acc, 1u);
        umma_bf16_ss(t_dk, dsd + 4, qm + 256, idesc_acc, 1u);
        umma_bf16_ss(t_dk, dsd + 6, qm + 384, idesc_acc, 1u);
        umma_commit(&qd_empty[s]);
        umma_commit(&pds_free);
        MTS_TRACE(4096 + 8 * i + 3);
      }
      umma_commit(&acc_full);
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;
    const int c = (warp - 2) >> 2;               // this thread's 32 of the tile's 64 query columns
    const int r = quarter * 32 + lane;           // key row inside the tile
    const int key = k0 + r;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const float scale_log2 = p.scale * LOG2E;
    const Dropout drop = make_dropout(p.dropout_p, p.seed + p.ctx->salt * kSaltMultiplier, uint32_t(bh), p.S);
    const float* lse_bh = p.lse + (long long)bh * p.S;
    const float* delta_bh = p.delta + (long long)bh * p.S;
    const uint32_t keep_shift = uint32_t(key & 3) * 8u;
    float* stats = reinterpret_cast<float*>(sStats) + (warp - 2) * 64;   // [lse 32 | delta 32] of this warp's query columns
    float pre[2];
    auto fetch_stats = [&](int qb0) {
      const int qa = qb0 + c * 32 + lane;
      pre[0] = qa < p.S ? lse_bh[qa] * LOG2E : 0.f;
      pre[1] = qa < p.S ? delta_bh[qa] : 0.f;
    };
    if (n_iter > 0) fetch_stats(first_q * 64);
    bool ok = true;
    for (int i = 0; i < n_iter; ++i) {
      const int qbase = (first_q + i) * 64;
      // lse / delta of this warp's 32 queries of the tile: staged in a 256-byte area private to the warp and read back as
      // float4 broadcasts (every lane reads the same address), 16 loads per 32 queries instead of 64 shuffles.  The
      // values were fetched from global memory one iteration ahead, so their latency is not on this path.
      stats[lane] = pre[0];
      stats[32 + lane] = pre[1];
      if (i + 1 < n_iter) fetch_stats(qbase + 64);
      __syncwarp();
      if (warp == 2) MTS_TRACE(8 * i + 0);
      if (!mbar_wait_warp(&st_full, i & 1, abort_ptr, lane)) { ok = false; break; }
      if (warp == 2) MTS_TRACE(8 * i + 1);
      tc_fence_after_sync();
      const bool need_mask = (p.causal && qbase < k0 + 127) || (qbase + 64 > p.S) || (k0 + 128 > p.S);
      {
        uint32_t rs[32], rd[32];
        tmem_ld_32x32(t_st + lane_base + c * 32, rs);
        tmem_ld_32x32(t_dp + lane_base + c * 32, rd);
        tmem_ld_wait();
        if (warp == 2) MTS_TRACE(8 * i + 2);
        // this warp's columns are in registers: once all eight warps say so the MMA warp starts the next query tile's scores
        epilogue_arrive(&st_free, lane);
        const float4* lse4 = reinterpret_cast<const float4*>(stats);
        const float4* del4 = reinterpret_cast<const float4*>(stats + 32);
        // The loops below are written one operation at a time over all 32 columns so that the latency of each
        // exp2 / multiply is covered by independent work of the same warp.
        float e[32];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 l4 = lse4[g];
          e[4 * g + 0] = ex2(fmaf(__uint_as_float(rs[4 * g + 0]), scale_log2, -l4.x));
          e[4 * g + 1] = ex2(fmaf(__uint_as_float(rs[4 * g + 1]), scale_log2, -l4.y));
          e[4 * g + 2] = ex2(fmaf(__uint_as_float(rs[4 * g + 2]), scale_log2, -l4.z));
          e[4 * g + 3] = ex2(fmaf(__uint_as_float(rs[4 * g + 3]), scale_log2, -l4.w));
        }
        if (need_mask) {       // selects on two per-thread bounds, no per-element branches
          const int col0 = qbase + c * 32;
          const int first = p.causal ? key - col0 : -0x7fffffff;   // queries before the key are masked
          const int end = key < p.S ? p.S - col0 : 0;              // queries past the sequence; a key past it masks its whole row
#pragma unroll
          for (int j = 0; j < 32; ++j) e[j] = (j < first || j >= end) ? 0.f : e[j];
        }
        uint32_t pa[16], pb[16];
        if (DROPOUT) {
          // Keep bits: one hashed word covers four consecutive keys of one query, i.e. the four lanes of a quad.
          // Each lane hashes the words of 8 of the 32 queries and the quad exchanges them by shuffle.
          uint32_t words[8];
#pragma unroll
          for (int t = 0; t < 8; ++t)
            words[t] = drop.word(uint32_t(qbase + c * 32 + 4 * t + (lane & 3)), uint32_t(key) >> 2);
          const int quad = lane & 28;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const float4 d4 = del4[g];
            const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
            float pv[4], ds[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const uint32_t w = __shfl_sync(0xffffffffu, words[g], quad | u);
              const bool kept = ((w >> keep_shift) & 0xFFu) >= drop.thresh;
              pv[u] = kept ? e[4 * g + u] : 0.f;                                    // 1 / keep: applied to dV at the end
              const float dp = kept ? __uint_as_float(rd[4 * g + u]) * drop.inv_keep : 0.f;
              ds[u] = e[4 * g + u] * (dp - dl[u]);                                   // softmax scale: applied to dK at the end
            }
            pa[2 * g] = pack2(pv[0], pv[1]); pa[2 * g + 1] = pack2(pv[2], pv[3]);
            pb[2 * g] = pack2(ds[0], ds[1]); pb[2 * g + 1] = pack2(ds[2], ds[3]);
          }
        } else {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const float4 d4 = del4[g];
            const float ds0 = e[4 * g + 0] * (__uint_as_float(rd[4 * g + 0]) - d4.x);
            const float ds1 = e[4 * g + 1] * (__uint_as_float(rd[4 * g + 1]) - d4.y);
            const float ds2 = e[4 * g + 2] * (__uint_as_float(rd[4 * g + 2]) - d4.z);
            const float ds3 = e[4 * g + 3] * (__uint_as_float(rd[4 * g + 3]) - d4.w);
            pa[2 * g] = pack2(e[4 * g + 0], e[4 * g + 1]); pa[2 * g + 1] = pack2(e[4 * g + 2], e[4 * g + 3]);
            pb[2 * g] = pack2(ds0, ds1); pb[2 * g + 1] = pack2(ds2, ds3);
          }
        }
        if (warp == 2) MTS_TRACE(8 * i + 3);
        // the previous tile's dV / dK MMAs must have read P^T / dS^T before they are overwritten
        if (!mbar_wait_warp(&pds_free, (i & 1) ^ 1, abort_ptr, lane)) { ok = false; break; }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          st_swizzled(sP, r, c * 4 + g, make_uint4(pa[4 * g], pa[4 * g + 1], pa[4 * g + 2], pa[4 * g + 3]));
          st_swizzled(sDS, r, c * 4 + g, make_uint4(pb[4 * g], pb[4 * g + 1], pb[4 * g + 2], pb[4 * g + 3]));
        }
        if (warp == 2) MTS_TRACE(8 * i + 4);
      }
      fence_proxy_async_smem();
      epilogue_arrive(&pds_ready, lane);
    }
    if (ok && mbar_wait_warp(&acc_full, 0, abort_ptr, lane)) {
      tc_fence_after_sync();
      // the two threads of a key row share the write-out: one takes dV, the other dK
      float acc[64];
      const uint32_t t_src = c == 0 ? t_dv : t_dk;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t rr[32];
        tmem_ld_32x32(t_src + lane_base + cc * 32, rr);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[cc * 32 + j] = __uint_as_float(rr[j]);
      }
      if (key < p.S && c == 0) {
        store_row64(p.dv + (long long)b * p.dv_sb + (long long)h * p.dv_sh + (long long)key * p.dv_ss, acc,
                    DROPOUT ? drop.inv_keep : 1.f);
      } else if (key < p.S) {
        __nv_bfloat16* dst = p.dk + (long long)b * p.dk_sb + (long long)h * p.dk_sh + (long long)key * p.dk_ss;
        if (p.rope_cos != nullptr) store_row64_unrotated(dst, acc, p.scale, p.rope_cos + (long long)key * 64, p.rope_sin + (long long)key * 64);
        else store_row64(dst, acc, p.scale);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && abort_word != 0) {
    __nanosleep(50000);   // bounded grace period for bulk copies still in flight
    if (p.status != nullptr) atomicMax(p.status, abort_word);
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_slot, 256);
}

// =====================================================================================================
// backward, sweep 2: dQ.  CTA = 128 queries; streams 64-key tiles.
// =====================================================================================================
constexpr int BWD_Q_SMEM = 2 * TILE128 /*Q,dO*/ + 4 * TILE64 /*K,V x 2 stages*/ + TILE128 /*dS*/ + 1024;

template <bool DROPOUT>
__global__ void __launch_bounds__(THREADS, 2)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k64,
                    const __grid_constant__ CUtensorMap tm_v64, const __grid_constant__ CUtensorMap tm_do, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = smem + TILE128;
  uint8_t* sK = smem + 2 * TILE128;
  uint8_t* sV = smem + 2 * TILE128 + 2 * TILE64;
  uint8_t* sDS = smem + 2 * TILE128 + 4 * TILE64;    // [128 q x 64 keys]

  __shared__ __align__(8) uint64_t qd_full, kv_full[2], kv_empty[2], st_full, st_free, ds_ready, ds_free, acc_full;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_word;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_q_tiles = (p.S + 127) / 128;
  const int q_tile = n_q_tiles - 1 - int(blockIdx.x);
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int q0 = q_tile * 128;
  const int n_k64 = (p.S + 63) / 64;
  const int n_iter = p.causal ? min(n_k64, (q0 + 127) / 64 + 1) : n_k64;

  if (threadIdx.x == 0) {
    mbar_init(&qd_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    mbar_init(&st_full, 1); mbar_init(&st_free, 8); mbar_init(&ds_ready, 8); mbar_init(&ds_free, 1); mbar_init(&acc_full, 1);
    abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 0) { tmem_alloc(&tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t t_s = tmem_slot, t_dp = tmem_slot + 64, t_dq = tmem_slot + 128;
  volatile int* abort_ptr = &abort_word;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&qd_full, 2 * TILE128);
      tma_load_4d(sQ, &tm_q, &qd_full, 0, q0, h, b);
      tma_load_4d(sDO, &tm_do, &qd_full, 0, q0, h, b);
      for (int i = 0; i < n_iter; ++i) {
        const int s = i & 1;
        if (!mbar_wait(&kv_empty[s], ((i >> 1) & 1) ^ 1, abort_ptr)) break;
        mbar_expect_tx(&kv_full[s], 2 * TILE64);
        tma_load_4d(sK + s * TILE64, &tm_k64, &kv_full[s], 0, i * 64, h, b);
        tma_load_4d(sV + s * TILE64, &tm_v64, &kv_full[s], 0, i * 64, h, b);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 64, false, false);
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, 64, false, true);
      // descriptors built once (see the dK / dV sweep for the arithmetic on them)
      const uint64_t qd = desc_kmajor(smem_u32(sQ), 0), dod = desc_kmajor(smem_u32(sDO), 0), dsd = desc_kmajor(smem_u32(sDS), 0);
      const uint64_t kk0 = desc_kmajor(smem_u32(sK), 0), vk0 = desc_kmajor(smem_u32(sV), 0), km0 = desc_mnmajor(smem_u32(sK), 0);
      constexpr uint64_t kStage = TILE64 >> 4;
      auto issue_scores = [&](int i) -> bool {
        const int s = i & 1;
        if (!mbar_wait_hot(&kv_full[s], (i >> 1) & 1, abort_ptr)) return false;
        if (!mbar_wait_hot(&st_free, (i & 1) ^ 1, abort_ptr)) return false;
        tc_fence_after_sync();
        const uint64_t k = kk0 + s * kStage, v = vk0 + s * kStage;
        umma_bf16_ss(t_s, qd, k, idesc_s, 0u);
        umma_bf16_ss(t_s, qd + 2, k + 2, idesc_s, 1u);
        umma_bf16_ss(t_s, qd + 4, k + 4, idesc_s, 1u);
        umma_bf16_ss(t_s, qd + 6, k + 6, idesc_s, 1u);
        umma_bf16_ss(t_dp, dod, v, idesc_s, 0u);
        umma_bf16_ss(t_dp, dod + 2, v + 2, idesc_s, 1u);
        umma_bf16_ss(t_dp, dod + 4, v + 4, idesc_s, 1u);
        umma_bf16_ss(t_dp, dod + 6, v + 6, idesc_s, 1u);
        umma_commit(&st_full);
        return true;
      };
      bool ok = mbar_wait(&qd_full, 0, abort_ptr);
      ok = ok && (n_iter <= 0 || issue_scores(0));
      for (int i = 0; i < n_iter && ok; ++i) {
        const int s = i & 1;
        MTS_TRACE(6144 + 8 * i + 0);
        if (i + 1 < n_iter && !issue_scores(i + 1)) break;   // next scores run while dS of this tile is being formed
        MTS_TRACE(6144 + 8 * i + 1);
        if (!mbar_wait_hot(&ds_ready, i & 1, abort_ptr)) break;
        MTS_TRACE(6144 + 8 * i + 2);
        tc_fence_after_sync();
        const uint64_t km = km0 + s * kStage;
        umma_bf16_ss(t_dq, dsd, km, idesc_dq, i != 0 ? 1u : 0u);
        umma_bf16_ss(t_dq, dsd + 2, km + 128, idesc_dq, 1u);
        umma_bf16_ss(t_dq, dsd + 4, km + 256, idesc_dq, 1u);
        umma_bf16_ss(t_dq, dsd + 6, km + 384, idesc_dq, 1u);
        umma_commit(&kv_empty[s]);
        umma_commit(&ds_free);
        MTS_TRACE(6144 + 8 * i + 3);
      }
      umma_commit(&acc_full);
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;
    const int c = (warp - 2) >> 2;               // this thread's 32 of the tile's 64 key columns
    const int r = quarter * 32 + lane;
    const int q_row = q0 + r;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const float scale_log2 = p.scale * LOG2E;
    const Dropout drop = make_dropout(p.dropout_p, p.seed + p.ctx->salt * kSaltMultiplier, uint32_t(bh), p.S);
    const float lse2 = q_row < p.S ? p.lse[(long long)bh * p.S + q_row] * LOG2E : 0.f;
    const float delta = q_row < p.S ? p.delta[(long long)bh * p.S + q_row] : 0.f;
    bool ok = true;
    for (int i = 0; i < n_iter; ++i) {
      const int kbase = i * 64;
      if (warp == 2) MTS_TRACE(2048 + 8 * i + 0);
      if (!mbar_wait_warp(&st_full, i & 1, abort_ptr, lane)) { ok = false; break; }
      if (warp == 2) MTS_TRACE(2048 + 8 * i + 1);
      tc_fence_after_sync();
      const bool need_mask = (p.causal && kbase + 63 > q0) || (kbase + 64 > p.S) || (q0 + 128 > p.S);
      {
        uint32_t rs[32], rd[32];
        tmem_ld_32x32(t_s + lane_base + c * 32, rs);
        tmem_ld_32x32(t_dp + lane_base + c * 32, rd);
        tmem_ld_wait();
        if (warp == 2) MTS_TRACE(2048 + 8 * i + 2);
        epilogue_arrive(&st_free, lane);   // S / dP are in registers: the next scores may be issued once all eight warps say so
        float ds[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) ds[j] = ex2(fmaf(__uint_as_float(rs[j]), scale_log2, -lse2));   // probabilities first
        if (need_mask) {      // one uniform branch around the whole loop; selects on one per-thread bound inside
          const int last = q_row < p.S ? min(p.S - 1, p.causal ? q_row : 0x7fffffff) - (kbase + c * 32) : -1;
#pragma unroll
          for (int j = 0; j < 32; ++j) ds[j] = j > last ? 0.f : ds[j];
        }
        if (DROPOUT) {
#pragma unroll
          for (int w = 0; w < 8; ++w) {
            const uint32_t bits = drop.word(uint32_t(q_row), uint32_t(kbase + c * 32 + 4 * w) >> 2);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const bool kept = ((bits >> (8 * t)) & 0xFFu) >= drop.thresh;
              const float dp = kept ? __uint_as_float(rd[4 * w + t]) * drop.inv_keep : 0.f;
              ds[4 * w + t] = ds[4 * w + t] * (dp - delta);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) ds[j] = ds[j] * (__uint_as_float(rd[j]) - delta);   // softmax scale: applied to dQ at the end
        }
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) pk[j] = pack2(ds[2 * j], ds[2 * j + 1]);
        if (warp == 2) MTS_TRACE(2048 + 8 * i + 3);
        // the previous tile's dQ MMAs must have read dS before it is overwritten
        if (!mbar_wait_warp(&ds_free, (i & 1) ^ 1, abort_ptr, lane)) { ok = false; break; }
#pragma unroll
        for (int g = 0; g < 4; ++g) st_swizzled(sDS, r, c * 4 + g, make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]));
        if (warp == 2) MTS_TRACE(2048 + 8 * i + 4);
      }
      fence_proxy_async_smem();
      epilogue_arrive(&ds_ready, lane);
    }
    if (ok && mbar_wait_warp(&acc_full, 0, abort_ptr, lane)) {
      tc_fence_after_sync();
      // write-out shared by the two threads of a query row: output columns 16 c .. + 15 and 32 + 16 c .. + 15, the pairs the
      // rotary un-rotation couples
      uint32_t lo[16], hi[16];
      tmem_ld_32x16(t_dq + lane_base + 16 * c, lo);
      tmem_ld_32x16(t_dq + lane_base + 32 + 16 * c, hi);
      tmem_ld_wait();
      if (q_row < p.S) {
        __nv_bfloat16* dst = p.dq + (long long)b * p.dq_sb + (long long)h * p.dq_sh + (long long)q_row * p.dq_ss;
        const bool rot = p.rope_cos != nullptr;
        const __nv_bfloat16* cos_row = rot ? p.rope_cos + (long long)q_row * 64 : nullptr;
        const __nv_bfloat16* sin_row = rot ? p.rope_sin + (long long)q_row * 64 : nullptr;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          float a8[8], b8[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) { a8[i] = __uint_as_float(lo[8 * j + i]) * p.scale; b8[i] = __uint_as_float(hi[8 * j + i]) * p.scale; }
          if (rot) {      // gradient of the row before the half-split rotation: lo' = lo cos + hi sin, hi' = hi cos - lo sin
            const uint4 cq = reinterpret_cast<const uint4*>(cos_row)[2 * c + j], sq = reinterpret_cast<const uint4*>(sin_row)[2 * c + j];
            const uint32_t cw[4] = {cq.x, cq.y, cq.z, cq.w}, sw[4] = {sq.x, sq.y, sq.z, sq.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float cs = __uint_as_float((i & 1) ? (cw[i >> 1] & 0xFFFF0000u) : (cw[i >> 1] << 16));
              const float sn = __uint_as_float((i & 1) ? (sw[i >> 1] & 0xFFFF0000u) : (sw[i >> 1] << 16));
              const float x = a8[i], y = b8[i];
              a8[i] = x * cs + y * sn;
              b8[i] = y * cs - x * sn;
            }
          }
          uint4 q;
          q.x = pack2(a8[0], a8[1]); q.y = pack2(a8[2], a8[3]); q.z = pack2(a8[4], a8[5]); q.w = pack2(a8[6], a8[7]);
          reinterpret_cast<uint4*>(dst)[2 * c + j] = q;
          q.x = pack2(b8[0], b8[1]); q.y = pack2(b8[2], b8[3]); q.z = pack2(b8[4], b8[5]); q.w = pack2(b8[6], b8[7]);
          reinterpret_cast<uint4*>(dst)[4 + 2 * c + j] = q;
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && abort_word != 0) {
    __nanosleep(50000);   // bounded grace period for bulk copies still in flight
    if (p.status != nullptr) atomicMax(p.status, abort_word);
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_slot, 256);
}

// ---- delta = rowsum(dO * O): 8 threads per row ----
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ o, long long o_sb, long long o_sh, long long o_ss,
                  const __nv_bfloat16* __restrict__ d_o, long long d_sb, long long d_sh, long long d_ss,
                  float* __restrict__ delta, int B, int H, int S) {
  const long long rows = (long long)B * H * S;
  const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
  const int part = threadIdx.x & 7;
  float acc = 0.f;
  if (row < rows) {
    const int s = int(row % S);
    const int h = int((row / S) % H);
    const int b = int(row / ((long long)S * H));
    const uint4 a = *reinterpret_cast<const uint4*>(o + b * o_sb + h * o_sh + s * o_ss + part * 8);
    const uint4 g = *reinterpret_cast<const uint4*>(d_o + b * d_sb + h * d_sh + s * d_ss + part * 8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&aw[i]);
      const __nv_bfloat162 y = *reinterpret_cast<const __nv_bfloat162*>(&gw[i]);
      acc += __low2float(x) * __low2float(y) + __high2float(x) * __high2float(y);
    }
  }
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  acc += __shfl_xor_sync(0xffffffffu, acc, 4);
  if (row < rows && part == 0) delta[row] = acc;
}

__global__ void dropout_mask_kernel(unsigned char* __restrict__ keep, int BH, int S, float p, unsigned long long seed) {
  const long long total = (long long)BH * S * S;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int k = int(i % S);
    const int q = int((i / S) % S);
    const int bh = int(i / ((long long)S * S));
    const Dropout d = make_dropout(p, seed, uint32_t(bh), S);
    keep[i] = d.thresh == 0u || d.keep(uint32_t(q), uint32_t(k)) ? 1 : 0;
  }
}

// ---- host ----
PFN_cuTensorMapEncodeTiled_v12000 attn_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  });
  return fn;
}

// Driver entry points need a current context; see the note in gemm_sm100.cu.
void attn_ensure_context_current() {
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

bool encode_bhsd(CUtensorMap* map, const StridedBHSD& t, int B, int H, int S, int box_rows) {
  attn_ensure_context_current();
  auto fn = attn_encode_fn();
  if (fn == nullptr) { g_attn_last_error = "cuTensorMapEncodeTiled entry point not found"; return false; }
  if ((reinterpret_cast<uintptr_t>(t.ptr) & 15) != 0 || t.sb % 8 != 0 || t.sh % 8 != 0 || t.ss % 8 != 0) {
    g_attn_last_error = "attention operand is not 16-byte aligned in every row";
    return false;
  }
  const cuuint64_t dims[4] = {cuuint64_t(D), cuuint64_t(S), cuuint64_t(H), cuuint64_t(B)};
  const cuuint64_t strides[3] = {cuuint64_t(t.ss) * 2, cuuint64_t(t.sh) * 2, cuuint64_t(t.sb) * 2};
  const cuuint32_t box[4] = {cuuint32_t(D), cuuint32_t(box_rows), 1u, 1u};
  const cuuint32_t elem[4] = {1u, 1u, 1u, 1u};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, t.ptr, dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    static char msg[200];
    snprintf(msg, sizeof(msg), "cuTensorMapEncodeTiled (4-D) error %d: B=%d H=%d S=%d strides=(%lld,%lld,%lld) box_rows=%d",
             int(r), B, H, S, t.sb, t.sh, t.ss, box_rows);
    g_attn_last_error = msg;
    return false;
  }
  return true;
}

Params make_params(const AttentionArgs& a) {
  Params p{};
  p.o = static_cast<__nv_bfloat16*>(a.o.ptr); p.o_sb = a.o.sb; p.o_sh = a.o.sh; p.o_ss = a.o.ss;
  p.dq = static_cast<__nv_bfloat16*>(a.dq.ptr); p.dq_sb = a.dq.sb; p.dq_sh = a.dq.sh; p.dq_ss = a.dq.ss;
  p.dk = static_cast<__nv_bfloat16*>(a.dk.ptr); p.dk_sb = a.dk.sb; p.dk_sh = a.dk.sh; p.dk_ss = a.dk.ss;
  p.dv = static_cast<__nv_bfloat16*>(a.dv.ptr); p.dv_sb = a.dv.sb; p.dv_sh = a.dv.sh; p.dv_ss = a.dv.ss;
  p.lse = a.lse; p.delta = a.delta;
  p.B = a.B; p.H = a.H; p.S = a.S; p.causal = a.causal;
  p.scale = a.scale; p.dropout_p = a.dropout_p; p.seed = a.seed; p.ctx = step_context(); p.status = a.status;
  if (p.ctx == nullptr) { g_attn_last_error = "step context allocation failed"; }
  p.rope_cos = static_cast<const __nv_bfloat16*>(a.rope_cos);
  p.rope_sin = static_cast<const __nv_bfloat16*>(a.rope_sin);
  return p;
}

template <typename K>
cudaError_t set_smem(K kernel, int bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

// cudaFuncSetAttribute applies to the current device only: remember per device ordinal which launchers have raised their
// shared-memory limit (a process that drives several GPUs would otherwise launch with the default limit on all but the first).
bool* attr_done_slot(bool (&flags)[64]) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  return &flags[dev];
}

}  // namespace

cudaError_t launch_flash_fwd(const AttentionArgs& a) {
  g_attn_last_error = "";
  if (a.B <= 0 || a.H <= 0 || a.S <= 0 || (long long)a.B * a.H > 65535) { g_attn_last_error = "bad attention extents"; return cudaErrorInvalidValue; }
  CUtensorMap tq, tk, tv;
  if (!encode_bhsd(&tq, a.q, a.B, a.H, a.S, 128) || !encode_bhsd(&tk, a.k, a.B, a.H, a.S, 128) ||
      !encode_bhsd(&tv, a.v, a.B, a.H, a.S, 128))
    return cudaErrorInvalidValue;
  static bool done_on[64] = {};
  bool* done = attr_done_slot(done_on);
  if (done == nullptr) { g_attn_last_error = "unexpected device ordinal"; return cudaErrorInvalidDevice; }
  if (!*done) {
    cudaError_t e = set_smem(flash_fwd_kernel<false>, FWD_SMEM);
    if (e == cudaSuccess) e = set_smem(flash_fwd_kernel<true>, FWD_SMEM);
    if (e != cudaSuccess) return e;
    *done = true;
  }
  const long long pairs = (long long)(((a.S + 127) / 128 + 1) / 2) * a.B * a.H;      // see work_item()
  const int grid = int(pairs < 2LL * device_sm_count() ? pairs : 2LL * device_sm_count());     // two resident CTAs per SM
  (void)cudaGetLastError();
  // the dropout arithmetic is compiled into an instantiation of its own: p = 0 runs (evaluation, most fine-tuning) carry none of it
  if (a.dropout_p > 0.f) flash_fwd_kernel<true><<<grid, THREADS, FWD_SMEM, a.stream>>>(tq, tk, tv, make_params(a));
  else flash_fwd_kernel<false><<<grid, THREADS, FWD_SMEM, a.stream>>>(tq, tk, tv, make_params(a));
  ++g_launch_count;
  return cudaGetLastError();
}

cudaError_t launch_flash_bwd(const AttentionArgs& a) {
  g_attn_last_error = "";
  if (a.B <= 0 || a.H <= 0 || a.S <= 0 || (long long)a.B * a.H > 65535) { g_attn_last_error = "bad attention extents"; return cudaErrorInvalidValue; }
  CUtensorMap tq128, tq64, tk128, tk64, tv128, tv64, tdo128, tdo64;
  if (!encode_bhsd(&tq128, a.q, a.B, a.H, a.S, 128) || !encode_bhsd(&tq64, a.q, a.B, a.H, a.S, 64) ||
      !encode_bhsd(&tk128, a.k, a.B, a.H, a.S, 128) || !encode_bhsd(&tk64, a.k, a.B, a.H, a.S, 64) ||
      !encode_bhsd(&tv128, a.v, a.B, a.H, a.S, 128) || !encode_bhsd(&tv64, a.v, a.B, a.H, a.S, 64) ||
      !encode_bhsd(&tdo128, a.d_o, a.B, a.H, a.S, 128) || !encode_bhsd(&tdo64, a.d_o, a.B, a.H, a.S, 64))
    return cudaErrorInvalidValue;
  static bool done_on[64] = {};
  bool* done = attr_done_slot(done_on);
  if (done == nullptr) { g_attn_last_error = "unexpected device ordinal"; return cudaErrorInvalidDevice; }
  if (!*done) {
    cudaError_t e = set_smem(flash_bwd_dkdv_kernel<false>, BWD_KV_SMEM);
    if (e == cudaSuccess) e = set_smem(flash_bwd_dkdv_kernel<true>, BWD_KV_SMEM);
    if (e == cudaSuccess) e = set_smem(flash_bwd_dq_kernel<false>, BWD_Q_SMEM);
    if (e == cudaSuccess) e = set_smem(flash_bwd_dq_kernel<true>, BWD_Q_SMEM);
    if (e != cudaSuccess) return e;
    *done = true;
  }
  (void)cudaGetLastError();
  const long long rows = (long long)a.B * a.H * a.S;
  attn_delta_kernel<<<unsigned((rows * 8 + 255) / 256), 256, 0, a.stream>>>(
      static_cast<const __nv_bfloat16*>(a.o.ptr), a.o.sb, a.o.sh, a.o.ss, static_cast<const __nv_bfloat16*>(a.d_o.ptr),
      a.d_o.sb, a.d_o.sh, a.d_o.ss, a.delta, a.B, a.H, a.S);
  const Params p = make_params(a);
  const dim3 grid((a.S + 127) / 128, a.B * a.H);
  if (a.dropout_p > 0.f) {
    flash_bwd_dkdv_kernel<true><<<grid, THREADS, BWD_KV_SMEM, a.stream>>>(tq64, tk128, tv128, tdo64, p);
    flash_bwd_dq_kernel<true><<<grid, THREADS, BWD_Q_SMEM, a.stream>>>(tq128, tk64, tv64, tdo128, p);
  } else {
    flash_bwd_dkdv_kernel<false><<<grid, THREADS, BWD_KV_SMEM, a.stream>>>(tq64, tk128, tv128, tdo64, p);
    flash_bwd_dq_kernel<false><<<grid, THREADS, BWD_Q_SMEM, a.stream>>>(tq128, tk64, tv64, tdo128, p);
  }
  g_launch_count += 3;
  return cudaGetLastError();
}

#ifdef MTS_ATTN_TRACE
cudaError_t copy_attention_trace(long long* host, int n) {
  return cudaMemcpyFromSymbol(host, g_attn_trace, sizeof(long long) * n);
}
#endif

cudaError_t launch_dropout_keep_mask(unsigned char* keep, int BH, int S, float dropout_p, unsigned long long seed,
                                     cudaStream_t stream) {
  dropout_mask_kernel<<<device_sm_count() * 8, 256, 0, stream>>>(keep, BH, S, dropout_p, seed);
  ++g_launch_count;
  return cudaGetLastError();
}

}  // namespace mts
