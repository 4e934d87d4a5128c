// Persistent, warp-specialised tcgen05 GEMM for sm_100a (see gemm_sm100.cuh for the interface).
//
// CTA = 320 threads: warp 0 issues TMA loads into a shared-memory ring, warp 1 issues tcgen05.mma
// (fp32 accumulators in tensor memory), warps 2-9 drain the accumulator (tcgen05.ld, four 32-column
// chunks in flight per warp; two warps share each 32-lane quarter and split its columns) and run the
// epilogue.  Two 256-column accumulators ping-pong, so the epilogue of tile i overlaps the MMAs of
// tile i+1.  One CTA per SM, tiles assigned round-robin.
//
// Two instantiations:
//   single  one CTA per 128 x 256 tile (cta_group::1), 4 stages of 48 KB.
//   pair    a cluster of two CTAs per 256 x 256 tile (cta_group::2): each CTA stages its 128 rows of A and
//           its 128 rows of B (6 stages of 32 KB), the leader CTA issues 256 x 256 x 16 MMAs that read both
//           shared memories and write both tensor memories, and each CTA runs the epilogue of its own 128
//           rows.  Per FLOP this moves one third less data from L2 than the single form, which is what
//           bounds the single form on the 768-wide contractions of the model.  No load is multicast:
//           every TMA copy has one destination CTA and only its completion bytes go to the leader's mbarrier.
//
// Reference counterpart: the Triton grouped-GEMM kernels of minitrain/kernels/triton/fused_moe_kernels.py
// (:264-437, :500-828) and the cuBLAS-backed nn.Linear layers; none of them has an sm_100 path.
#include "gemm_sm100.cuh"
#include "ptx_sm100.cuh"

#include <cudaTypedefs.h>
#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <mutex>

namespace mts {

std::atomic<unsigned long long> g_launch_count{0};
const char* g_last_error = "";

#ifdef MTS_GEMM_TRACE
// Phase trace of CTA 0 (debug builds only): clock64 stamps, 8 slots per tile, globals from slot 4000.
__device__ long long g_gemm_trace[4096];
#define GTRACE(slot) do { if (blockIdx.x == 0 && (slot) < 4096) g_gemm_trace[(slot)] = clock64(); } while (0)
cudaError_t copy_gemm_trace(long long* host, int n) { return cudaMemcpyFromSymbol(host, g_gemm_trace, sizeof(long long) * n); }
#else
#define GTRACE(slot) do {} while (0)
#endif

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr int NUM_THREADS = 320;   // producer warp, MMA warp, 8 epilogue warps
constexpr int EPI_WARPS = 8;
constexpr int EPI_STAGE_BYTES = 32 * 128;   // one 32-row x 128-byte box per epilogue warp, 128-byte swizzled
constexpr int ACC_COLS = 256;
constexpr int TMEM_COLS = 512;
constexpr int MN_BLOCK_BYTES = BK * 128;  // one 64-wide MN block of an MN-major operand: BK rows of 128 B

template <bool PAIR>
struct Cfg {
  static constexpr int STAGES = PAIR ? 6 : 4;
  static constexpr int TILE_M = PAIR ? 256 : 128;        // rows of one work item
  static constexpr int B_ROWS = PAIR ? 128 : 256;        // rows of B staged by one CTA
  static constexpr int B_BYTES = B_ROWS * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr size_t SMEM_BYTES = size_t(RING_BYTES) + EPI_WARPS * EPI_STAGE_BYTES + 1024;
};

struct KernelParams {
  int M, N, K;
  int mode, epilogue;
  int a_mn, b_mn;
  void* out;
  long long ldo;
  int out_fp32, accumulate, atomic_out;
  void* aux;
  long long ld_aux;
  const int* tile_group;
  const int* num_row_tiles;
  const int* group_rows;
  int num_groups;
  int k_splits;      // GROUPED_K: every group's row range is cut into this many parts, each a work item that adds into the group's output
  int b_group_stride_rows;
  long long out_group_stride;
  int tiles_m, tiles_n;
  int* status;
  const int* gather_a;   // pair kernels only: row r of A (K-major, grouped-M) or contraction row k of A (MN-major, grouped-K) is row
  const int* gather_b;   // gather[r] of the tensor behind the map (negative: a zero row); same for B (MN-major, grouped-K)
  int gather_a_rows, gather_b_rows;   // extents of those tensors: the index used for "no row"
  const float* row_scale;   // SwiGLU epilogues: weight of every output row (route weight; 0 on padding rows) or null
  const int* row_slot;      // SwiGLU backward: where the row's weight gradient goes (index into row_grad; negative: nowhere)
  float* row_grad;          // SwiGLU backward: += sum_i acc[r, i] * silu(gate) * up, the gradient of row_scale
  int tma_store;     // epilogue writes through shared memory and TMA stores / reduce-adds (else per-lane global stores)
  int diag_no_loads; // timing diagnostic: after the ring's first fill the producer only signals, nothing is copied
};

struct Tile {
  int a_coord;     // K-major: first row of A; MN-major: first MN column of A
  int b_coord;     // same for B (first 128-row half when K-major)
  int b_coord2;    // second 128-row half of B (K-major only)
  int k_begin;     // first contraction index
  int k_blocks;    // number of BK blocks
  int b_k_offset;  // added to the contraction coordinate of an MN-major B (stacked experts)
  int c_row, c_col;
  long long out_offset;
  int out_group;   // third coordinate of the output tensor map
  int row_limit, col_limit;
};

// `tiles_m` counts work items of TILE_M rows; `num_row_tiles` and `tile_group` always count 128-row tiles.
template <int TILE_M>
__device__ __forceinline__ int live_tiles(const KernelParams& p) {
  if (p.mode == GEMM_GROUPED_M) {
    int rows = (*p.num_row_tiles + TILE_M / 128 - 1) / (TILE_M / 128);
    rows = rows < p.tiles_m ? rows : p.tiles_m;
    return rows * p.tiles_n;
  }
  if (p.mode == GEMM_GROUPED_K) return p.num_groups * p.k_splits * p.tiles_m * p.tiles_n;
  return p.tiles_m * p.tiles_n;
}

template <int TILE_M>
__device__ __forceinline__ Tile decode_tile(const KernelParams& p, int t) {
  Tile o;
  o.b_k_offset = 0;
  o.out_offset = 0;
  o.out_group = 0;
  if (p.mode == GEMM_GROUPED_K) {
    const int per = p.tiles_m * p.tiles_n;
    const int part = t / per;                       // (group, split), splits of one group adjacent
    const int r = t - part * per;
    const int mt = r / p.tiles_n, nt = r - mt * p.tiles_n;
    const int g = part / p.k_splits, sp = part - g * p.k_splits;
    int k0 = p.group_rows[g], k1 = p.group_rows[g + 1];
    if (p.k_splits > 1) {                           // equal parts, whole k-blocks each; the last ones may be empty
      const int blocks = (k1 - k0 + BK - 1) / BK;
      const int per_split = (blocks + p.k_splits - 1) / p.k_splits;
      const int lo = k0 + sp * per_split * BK, hi = lo + per_split * BK;
      k0 = lo < k1 ? lo : k1;
      k1 = hi < k1 ? hi : k1;
    }
    o.a_coord = mt * TILE_M;
    o.b_coord = nt * BN;
    o.b_coord2 = o.b_coord + 128;
    o.k_begin = k0;
    o.k_blocks = (k1 - k0 + BK - 1) / BK;
    o.c_row = mt * TILE_M;
    o.c_col = nt * BN;
    o.out_offset = (long long)g * p.out_group_stride;
    o.out_group = p.out_group_stride > 0 ? g : 0;
    o.row_limit = p.M;
    o.col_limit = p.N;
    return o;
  }
  const int mt = t / p.tiles_n, nt = t - mt * p.tiles_n;
  o.a_coord = mt * TILE_M;
  o.k_begin = 0;
  o.k_blocks = (p.K + BK - 1) / BK;
  o.c_row = mt * TILE_M;
  o.c_col = nt * BN;
  o.row_limit = p.M;
  o.col_limit = p.N;
  o.b_coord = nt * BN;
  o.b_coord2 = o.b_coord + 128;
  if (p.mode == GEMM_GROUPED_M) {
    const int g = p.tile_group[mt * (TILE_M / 128)];   // a 256-row work item needs segments padded to 256 rows
    if (p.b_mn) {
      o.b_k_offset = g * p.b_group_stride_rows;
    } else if (p.epilogue == EPI_SWIGLU) {
      o.b_coord = g * p.b_group_stride_rows + nt * 128;          // gate rows
      o.b_coord2 = g * p.b_group_stride_rows + p.N / 2 + nt * 128;  // up rows
    } else {
      o.b_coord += g * p.b_group_stride_rows;
      o.b_coord2 = o.b_coord + 128;
    }
    if (p.epilogue == EPI_SWIGLU) {
      o.c_col = nt * 128;
      o.col_limit = p.N / 2;
    }
  }
  return o;
}

// ---- epilogue helpers -------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void store_row_bf16(__nv_bfloat16* dst, const float (&v)[32], int valid_cols) {
  if (valid_cols >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 q;
      q.x = pack_bf16(v[8 * j + 0], v[8 * j + 1]);
      q.y = pack_bf16(v[8 * j + 2], v[8 * j + 3]);
      q.z = pack_bf16(v[8 * j + 4], v[8 * j + 5]);
      q.w = pack_bf16(v[8 * j + 6], v[8 * j + 7]);
      reinterpret_cast<uint4*>(dst)[j] = q;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid_cols) dst[j] = __float2bfloat16(v[j]);
  }
}

__device__ __forceinline__ void store_row_f32(float* dst, float (&v)[32], int valid_cols, int accumulate, int atomic) {
  if (atomic) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid_cols) atomicAdd(dst + j, v[j]);
    return;
  }
  if (valid_cols >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float4 q = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      if (accumulate) {
        const float4 old = reinterpret_cast<const float4*>(dst)[j];
        q.x += old.x; q.y += old.y; q.z += old.z; q.w += old.w;
      }
      reinterpret_cast<float4*>(dst)[j] = q;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid_cols) dst[j] = accumulate ? dst[j] + v[j] : v[j];
  }
}

__device__ __forceinline__ void regs_to_float(const uint32_t (&r)[32], float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
}

// sigmoid(x) = 0.5 tanh(x / 2) + 0.5: one MUFU instruction and two FMA-pipe ones.  The form 1 / (1 + exp(-x)) costs an
// exponential, a full-precision division (about ten instructions) and made the SwiGLU epilogues, not the MMA, the bound
// of the expert GEMMs.  tanh.approx is good to about 2^-11, inside the bf16 rounding of everything these epilogues store.
__device__ __forceinline__ float sigmoidf_fast(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return fmaf(0.5f, t, 0.5f);
}

// ---- staging for TMA stores: rows of 128 bytes, 16-byte chunk j of row r lives at chunk (j ^ (r & 7)) ----
__device__ __forceinline__ void stage_chunk(uint8_t* stage, int row, int j, uint4 q) {
  *reinterpret_cast<uint4*>(stage + row * 128 + ((j ^ (row & 7)) << 4)) = q;
}

__device__ __forceinline__ void stage_row_bf16(uint8_t* stage, int row, int j0, const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 q;
    q.x = pack_bf16(v[8 * j + 0], v[8 * j + 1]);
    q.y = pack_bf16(v[8 * j + 2], v[8 * j + 3]);
    q.z = pack_bf16(v[8 * j + 4], v[8 * j + 5]);
    q.w = pack_bf16(v[8 * j + 6], v[8 * j + 7]);
    stage_chunk(stage, row, j0 + j, q);
  }
}

__device__ __forceinline__ void stage_row_f32(uint8_t* stage, int row, const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint4 q;
    q.x = __float_as_uint(v[4 * j + 0]);
    q.y = __float_as_uint(v[4 * j + 1]);
    q.z = __float_as_uint(v[4 * j + 2]);
    q.w = __float_as_uint(v[4 * j + 3]);
    stage_chunk(stage, row, j, q);
  }
}

// Warp-collective: the staging box may be rewritten once the TMA unit has read what the previous flush handed over.
// Waiting here, right before the next write, instead of right after the flush lets the math of the next box run while
// the unit drains the last one.
__device__ __forceinline__ void stage_acquire(int lane) {
  if (lane == 0) tma_store_wait_read<0>();
  __syncwarp();
}

// Warp-collective: publish the staged box and hand it to the TMA unit.  The box belongs to the unit until stage_acquire.
__device__ __forceinline__ void flush_box(const CUtensorMap* map, const uint8_t* stage, int col, int row0, int group, bool reduce,
                                          int lane) {
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    if (reduce) tma_reduce_add_3d(map, stage, col, row0, group);
    else tma_store_3d(map, stage, col, row0, group);
    tma_store_commit();
  }
}

// The SwiGLU pre-activations saved by the forward epilogue are read by nothing but the backward epilogue, so they live in a
// layout of their own: [rows / 32][ld / 8][32 rows][8 values].  The 16 bytes that lane r (row r of a 32-row block) owns of
// column chunk q sit between those of lanes r - 1 and r + 1, so every per-row access of a warp is one 512-byte transaction
// (row-major, the same access touched 32 lines and ran at an eighth of the L1 rate, which bounded the whole GEMM).
__device__ __forceinline__ long long aux_chunk(long long row, int col, long long ld) {     // element offset; col % 8 == 0
  return (((row >> 5) * (ld >> 3) + (col >> 3)) * 32 + (row & 31)) * 8;
}

__device__ __forceinline__ void aux_store32(__nv_bfloat16* aux, long long row, int col, long long ld, const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 q;
    q.x = pack_bf16(v[8 * j + 0], v[8 * j + 1]); q.y = pack_bf16(v[8 * j + 2], v[8 * j + 3]);
    q.z = pack_bf16(v[8 * j + 4], v[8 * j + 5]); q.w = pack_bf16(v[8 * j + 6], v[8 * j + 7]);
    *reinterpret_cast<uint4*>(aux + aux_chunk(row, col + 8 * j, ld)) = q;
  }
}

// 32 saved gate values and 32 saved up values of one row, as packed bf16 (four 16-byte loads each).
__device__ __forceinline__ void aux_load32(const __nv_bfloat16* aux, long long row, int gate_col, int up_col, long long ld,
                                           uint4 (&pg)[4], uint4 (&pu)[4]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    pg[j] = __ldg(reinterpret_cast<const uint4*>(aux + aux_chunk(row, gate_col + 8 * j, ld)));
    pu[j] = __ldg(reinterpret_cast<const uint4*>(aux + aux_chunk(row, up_col + 8 * j, ld)));
  }
}

__device__ __forceinline__ void prefetch_l2(const void* ptr) { asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr)); }

template <int OFF>
__device__ __forceinline__ void unpack_bf16x8(const uint4& q, float (&v)[32]) {
  v[OFF + 0] = __uint_as_float(q.x << 16); v[OFF + 1] = __uint_as_float(q.x & 0xFFFF0000u);
  v[OFF + 2] = __uint_as_float(q.y << 16); v[OFF + 3] = __uint_as_float(q.y & 0xFFFF0000u);
  v[OFF + 4] = __uint_as_float(q.z << 16); v[OFF + 5] = __uint_as_float(q.z & 0xFFFF0000u);
  v[OFF + 6] = __uint_as_float(q.w << 16); v[OFF + 7] = __uint_as_float(q.w & 0xFFFF0000u);
}

// ---- the kernel ---------------------------------------------------------------------------------
// EPI (the epilogue) is a template parameter so that every instantiation holds one epilogue only: with all three behind a
// run-time switch the register allocation of each was that of the largest.
template <bool PAIR, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    const __grid_constant__ CUtensorMap tm_out, const __grid_constant__ CUtensorMap tm_aux, const KernelParams p) {
  using C = Cfg<PAIR>;
  constexpr int STAGES = C::STAGES;
  constexpr int STAGE_BYTES = C::STAGE_BYTES;
  constexpr int TILE_M = C::TILE_M;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  __shared__ __align__(8) uint64_t full_bar[STAGES];    // pair: only the leader's are used
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];        // pair: only the leader's are used
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_word;
  __shared__ int loads_issued, loads_consumed;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;   // 0 = leader
  const int worker = PAIR ? int(blockIdx.x >> 1) : int(blockIdx.x);
  const int workers = PAIR ? int(gridDim.x >> 1) : int(gridDim.x);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], PAIR ? 2 * EPI_WARPS : EPI_WARPS);  // one arrive per epilogue warp (of both CTAs)
    }
    abort_word = 0;
    loads_issued = 0;
    loads_consumed = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }
  if (warp == 0) {
    if (PAIR) {
      tmem_alloc_pair(&tmem_slot, TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&tmem_slot, TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the peer's barriers exist before anything is signalled on them
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abort_ptr = &abort_word;

  const int total = live_tiles<TILE_M>(p);
#ifdef MTS_GEMM_TRACE
  if (threadIdx.x == 0 && blockIdx.x == 0) { g_gemm_trace[4000] = clock64(); g_gemm_trace[4001] = (long long)global_timer_ns(); }
#endif

  if (warp == 0) {
    // ================= TMA producer (in a pair: each CTA loads its own halves) =================
    // One thread; its instruction stream per k-block is kept short because the ring's refill latency rides on it.  With a
    // gathered operand all 32 lanes take part: every lane fetches four rows per k-block with one tile::gather4 copy, lane 0
    // still posts the byte count and loads the other operand.
    const bool gathers = PAIR && (p.gather_a != nullptr || p.gather_b != nullptr);
    if (lane == 0 || gathers) {
      int it = 0, s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int tj = 0;
      const uint32_t full0 = PAIR ? map_to_cta(smem_u32(&full_bar[0]), 0) : smem_u32(&full_bar[0]);
      const uint32_t ring0 = PAIR ? map_to_cta(smem_u32(smem), rank) : smem_u32(smem);
      for (int tile = worker; tile < total && ok; tile += workers, ++tj) {
        const Tile t = decode_tile<TILE_M>(p, tile);
        const int a_coord = t.a_coord + int(rank) * 128;
        const int b_coord = PAIR ? (B_MN ? t.b_coord + int(rank) * 128 : (rank == 0 ? t.b_coord : t.b_coord2)) : t.b_coord;
        GTRACE(8 * tj + 6);
        int k = t.k_begin;
        // K-major gathered A (grouped-M): the same 128 rows for every k-block of the tile, four per lane
        int4 rows_a = make_int4(0, 0, 0, 0);
        if (gathers && !A_MN && p.gather_a != nullptr) {
          rows_a = *reinterpret_cast<const int4*>(p.gather_a + a_coord + 4 * lane);
          rows_a.x = rows_a.x < 0 ? p.gather_a_rows : rows_a.x; rows_a.y = rows_a.y < 0 ? p.gather_a_rows : rows_a.y;
          rows_a.z = rows_a.z < 0 ? p.gather_a_rows : rows_a.z; rows_a.w = rows_a.w < 0 ? p.gather_a_rows : rows_a.w;
        }
        // MN-major gathered operands (grouped-K): four contraction rows per lane and k-block, fetched one k-block ahead
        const int sub = lane & 15, blk = lane >> 4;      // rows 4 * sub .. + 3 of 64-column block blk
        int4 next_a = make_int4(0, 0, 0, 0), next_b = make_int4(0, 0, 0, 0);
        if (gathers && A_MN && p.gather_a != nullptr && t.k_blocks > 0) next_a = *reinterpret_cast<const int4*>(p.gather_a + k + 4 * sub);
        if (gathers && B_MN && p.gather_b != nullptr && t.k_blocks > 0) next_b = *reinterpret_cast<const int4*>(p.gather_b + k + 4 * sub);
        for (int kb = 0; kb < t.k_blocks; ++kb, ++it, k += BK) {
          int4 cur_a = next_a, cur_b = next_b;
          if (gathers && kb + 1 < t.k_blocks) {
            if (A_MN && p.gather_a != nullptr) next_a = *reinterpret_cast<const int4*>(p.gather_a + k + BK + 4 * sub);
            if (B_MN && p.gather_b != nullptr) next_b = *reinterpret_cast<const int4*>(p.gather_b + k + BK + 4 * sub);
          }
          if (!mbar_wait_hot(&empty_bar[s], ph ^ 1, abort_ptr)) { ok = false; break; }
          if (p.diag_no_loads && it >= STAGES) {
            if (rank == 0 && lane == 0) mbar_arrive(&full_bar[s]);
          } else if (PAIR) {
            const uint32_t bar = full0 + s * 8;
            const uint32_t a_sm = ring0 + s * STAGE_BYTES, b_sm = a_sm + A_BYTES;
            const bool ga = gathers && p.gather_a != nullptr, gb = gathers && p.gather_b != nullptr;
            if (lane == 0) {
              if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);   // both CTAs' bytes
              if (!ga) {
                if (A_MN) {
                  tma_load_2d_pair(a_sm, &tm_a, bar, a_coord, k);
                  tma_load_2d_pair(a_sm + MN_BLOCK_BYTES, &tm_a, bar, a_coord + 64, k);
                } else {
                  tma_load_2d_pair(a_sm, &tm_a, bar, k, a_coord);
                }
              }
              if (!gb) {
                if (B_MN) {
                  tma_load_2d_pair(b_sm, &tm_b, bar, b_coord, k + t.b_k_offset);
                  tma_load_2d_pair(b_sm + MN_BLOCK_BYTES, &tm_b, bar, b_coord + 64, k + t.b_k_offset);
                } else {
                  tma_load_2d_pair(b_sm, &tm_b, bar, k, b_coord);
                }
              }
            }
            if (ga) {
              if (A_MN) {
                const int none = p.gather_a_rows;
                tma_gather4_pair(a_sm + blk * MN_BLOCK_BYTES + sub * 512, &tm_a, bar, a_coord + 64 * blk, cur_a.x < 0 ? none : cur_a.x,
                                 cur_a.y < 0 ? none : cur_a.y, cur_a.z < 0 ? none : cur_a.z, cur_a.w < 0 ? none : cur_a.w);
              } else {
                tma_gather4_pair(a_sm + lane * 512, &tm_a, bar, k, rows_a.x, rows_a.y, rows_a.z, rows_a.w);
              }
            }
            if (gb) {     // MN-major only (checked on the host)
              const int none = p.gather_b_rows;
              tma_gather4_pair(b_sm + blk * MN_BLOCK_BYTES + sub * 512, &tm_b, bar, b_coord + 64 * blk, cur_b.x < 0 ? none : cur_b.x,
                               cur_b.y < 0 ? none : cur_b.y, cur_b.z < 0 ? none : cur_b.z, cur_b.w < 0 ? none : cur_b.w);
            }
          } else {
            uint8_t* a_dst = smem + s * STAGE_BYTES;
            uint8_t* b_dst = a_dst + A_BYTES;
            mbar_expect_tx(&full_bar[s], STAGE_BYTES);
            if (A_MN) {
              tma_load_2d(a_dst, &tm_a, &full_bar[s], a_coord, k);
              tma_load_2d(a_dst + MN_BLOCK_BYTES, &tm_a, &full_bar[s], a_coord + 64, k);
            } else {
              tma_load_2d(a_dst, &tm_a, &full_bar[s], k, a_coord);
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(b_dst + j * MN_BLOCK_BYTES, &tm_b, &full_bar[s], b_coord + 64 * j, k + t.b_k_offset);
            } else {
              tma_load_2d(b_dst, &tm_b, &full_bar[s], k, t.b_coord);
              tma_load_2d(b_dst + 128 * 128, &tm_b, &full_bar[s], k, t.b_coord2);
            }
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (lane == 0) loads_issued = it;
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================= MMA issuer (in a pair: the leader CTA only) =================
    // One thread feeds the tensor core: four MMAs per k-block take 4 x 128 cycles of pipe time, so everything this
    // thread executes between them (wait, fence, descriptors, commit, loop) has to stay well below that.
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(TILE_M, BN, A_MN, B_MN);
      // descriptors differ between stages and K steps only in the 14-bit start-address field (16-byte units)
      const uint64_t a_tmpl = A_MN ? make_smem_desc_sw128(0, MN_BLOCK_BYTES, 1024) : make_smem_desc_sw128(0, 16, 1024);
      const uint64_t b_tmpl = B_MN ? make_smem_desc_sw128(0, MN_BLOCK_BYTES, 1024) : make_smem_desc_sw128(0, 16, 1024);
      constexpr uint32_t a_step = (A_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4;
      constexpr uint32_t b_step = (B_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4;
      const uint32_t ring16 = (smem_u32(smem) & 0x3FFFF) >> 4;
      const uint32_t empty_local = PAIR ? map_to_cta(smem_u32(&empty_bar[0]), 0) : smem_u32(&empty_bar[0]);
      const uint32_t empty_peer = PAIR ? map_to_cta(smem_u32(&empty_bar[0]), 1) : 0u;
      const uint32_t accfull_local = PAIR ? map_to_cta(smem_u32(&acc_full[0]), 0) : smem_u32(&acc_full[0]);
      const uint32_t accfull_peer = PAIR ? map_to_cta(smem_u32(&acc_full[0]), 1) : 0u;
      int it = 0, acc_it = 0, s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = worker; tile < total && ok; tile += workers) {
        const Tile t = decode_tile<TILE_M>(p, tile);
        if (t.k_blocks == 0) continue;
        const int buf = acc_it & 1;
        const uint32_t acc_ph = (acc_it >> 1) & 1;
        GTRACE(8 * acc_it + 0);
        if (!mbar_wait_hot(&acc_empty[buf], acc_ph ^ 1, abort_ptr)) { ok = false; break; }
        GTRACE(8 * acc_it + 1);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * ACC_COLS;
        uint32_t accumulate = 0;
        for (int kb = 0; kb < t.k_blocks; ++kb, ++it) {
          if (!mbar_wait_hot(&full_bar[s], ph, abort_ptr)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a16 = ring16 + s * (STAGE_BYTES >> 4);
          const uint64_t ad = a_tmpl | a16, bd = b_tmpl | (a16 + (A_BYTES >> 4));
          if (PAIR) {
            umma_bf16_ss_pair(d_tmem, ad, bd, idesc, accumulate);
            umma_bf16_ss_pair(d_tmem, ad + a_step, bd + b_step, idesc, 1u);
            umma_bf16_ss_pair(d_tmem, ad + 2 * a_step, bd + 2 * b_step, idesc, 1u);
            umma_bf16_ss_pair(d_tmem, ad + 3 * a_step, bd + 3 * b_step, idesc, 1u);
            umma_commit_pair(empty_local + s * 8);   // frees the stage in both CTAs once these MMAs have read it
            umma_commit_pair(empty_peer + s * 8);
          } else {
            umma_bf16_ss(d_tmem, ad, bd, idesc, accumulate);
            umma_bf16_ss(d_tmem, ad + a_step, bd + b_step, idesc, 1u);
            umma_bf16_ss(d_tmem, ad + 2 * a_step, bd + 2 * b_step, idesc, 1u);
            umma_bf16_ss(d_tmem, ad + 3 * a_step, bd + 3 * b_step, idesc, 1u);
            umma_commit(&empty_bar[s]);
          }
          accumulate = 1u;
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        GTRACE(8 * acc_it + 2);
        if (PAIR) {
          umma_commit_pair(accfull_local + buf * 8);
          umma_commit_pair(accfull_peer + buf * 8);
        } else {
          umma_commit(&acc_full[buf]);
        }
        ++acc_it;
      }
      loads_consumed = it;
    }
    __syncwarp();
  } else {
    // ================= epilogue: warps 2..9; warp w drains TMEM lane quarter (w & 3), column half (w - 2) / 4 =======
    const int quarter = warp & 3;
    const int half_id = (warp - 2) >> 2;
    const int row_in_tile = int(rank) * 128 + quarter * 32 + lane;
    const uint32_t acc_empty_addr[2] = {PAIR ? map_to_cta(smem_u32(&acc_empty[0]), 0) : 0u,
                                        PAIR ? map_to_cta(smem_u32(&acc_empty[1]), 0) : 0u};
    uint8_t* stage = smem + C::RING_BYTES + (warp - 2) * EPI_STAGE_BYTES;
    const bool aux_vec = p.aux != nullptr && (reinterpret_cast<uintptr_t>(p.aux) & 15) == 0 && (p.ld_aux & 7) == 0 && (p.N & 7) == 0;
    int acc_it = 0;
    bool ok = true;
    for (int tile = worker; tile < total && ok; tile += workers) {
      const Tile t = decode_tile<TILE_M>(p, tile);
      const int row = t.c_row + row_in_tile;
      const int row0 = row - lane;                 // first row of this warp's 32-row box
      const bool row_ok = row < t.row_limit;
      // SwiGLU epilogues of the routed experts: this row's route weight (0 on padding rows) and, in backward, where the
      // gradient of that weight is accumulated
      const float wrow = (p.row_scale != nullptr && EPI != EPI_STORE && row_ok) ? __ldg(p.row_scale + row) : 1.f;
      float wgrad_part = 0.f;
      if (t.k_blocks == 0) {
        // nothing was contracted: the product is zero
        if (p.tma_store && EPI == EPI_STORE && !p.accumulate && !p.atomic_out) {
          float z[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) z[j] = 0.f;
          stage_acquire(lane);
          if (p.out_fp32) stage_row_f32(stage, lane, z);
          else { stage_row_bf16(stage, lane, 0, z); stage_row_bf16(stage, lane, 4, z); }
          const int step = p.out_fp32 ? 32 : 64;
          for (int col = t.c_col + half_id * 128; col < t.c_col + half_id * 128 + 128; col += step)
            if (col < t.col_limit && row0 < t.row_limit) flush_box(&tm_out, stage, col, row0, t.out_group, false, lane);
        } else if (EPI == EPI_STORE && !p.accumulate && !p.atomic_out && row_ok) {
          float z[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) z[j] = 0.f;
          for (int c = half_id * 4; c < half_id * 4 + 4; ++c) {
            const int col = t.c_col + c * 32;
            const int valid = t.col_limit - col;
            if (valid <= 0) break;
            if (p.out_fp32) store_row_f32(reinterpret_cast<float*>(p.out) + t.out_offset + (long long)row * p.ldo + col, z, valid, 0, 0);
            else store_row_bf16(reinterpret_cast<__nv_bfloat16*>(p.out) + t.out_offset + (long long)row * p.ldo + col, z, valid);
          }
        }
        continue;
      }
      // SwiGLU backward reads the saved [gate | up] values of its rows, 32 columns at a time.  The first chunk is fetched
      // into registers before the accumulator is awaited, so that its latency hides behind the MMA; the lines of the
      // other chunks are pulled into L2 meanwhile, and each is loaded one chunk ahead of its use.
      uint4 cg[4], cu[4];
      bool swb_fast = false;
      if (p.tma_store && EPI == EPI_SWIGLU_BWD) {
        const int colw = t.c_col + half_id * 128;
        const __nv_bfloat16* pre = reinterpret_cast<const __nv_bfloat16*>(p.aux);
        swb_fast = row0 < t.row_limit && aux_vec && colw + 128 <= p.N;
        if (swb_fast) {
          aux_load32(pre, row, colw, p.N + colw, p.ld_aux, cg, cu);
          // this warp's 128 gate columns are one contiguous 8 KB run of the blocked layout, and so are its up columns:
          // 64 lines each, two per lane
          const char* g_run = reinterpret_cast<const char*>(pre + aux_chunk(row0, colw, p.ld_aux));
          const char* u_run = reinterpret_cast<const char*>(pre + aux_chunk(row0, p.N + colw, p.ld_aux));
          prefetch_l2(g_run + 128 * lane); prefetch_l2(g_run + 128 * (lane + 32));
          prefetch_l2(u_run + 128 * lane); prefetch_l2(u_run + 128 * (lane + 32));
        }
      }
      const int buf = acc_it & 1;
      const uint32_t acc_ph = (acc_it >> 1) & 1;
      if (warp == 2 && lane == 0) GTRACE(8 * acc_it + 3);
      if (!mbar_wait_warp(&acc_full[buf], acc_ph, abort_ptr, lane)) { ok = false; break; }
      if (warp == 2 && lane == 0) GTRACE(8 * acc_it + 4);
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + buf * ACC_COLS;
      bool released = false;
      // the accumulator buffer goes back to the MMA warp as soon as its values are in registers
      auto release_acc = [&]() {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if (PAIR) mbar_arrive_cluster(acc_empty_addr[buf]);
          else mbar_arrive(&acc_empty[buf]);
        }
        released = true;
      };

      if (p.tma_store && EPI == EPI_STORE) {
        uint32_t r0[32], r1[32], r2[32], r3[32];
        const int c0 = half_id * 4;
        tmem_ld_32x32(taddr + (c0 + 0) * 32, r0);
        tmem_ld_32x32(taddr + (c0 + 1) * 32, r1);
        tmem_ld_32x32(taddr + (c0 + 2) * 32, r2);
        tmem_ld_32x32(taddr + (c0 + 3) * 32, r3);
        tmem_ld_wait();
        release_acc();
        const bool box_rows = row0 < t.row_limit;
        const bool reduce = p.accumulate || p.atomic_out;
        const int col0 = t.c_col + c0 * 32;
        float v[32];
        if (p.out_fp32) {
          stage_acquire(lane); regs_to_float(r0, v); stage_row_f32(stage, lane, v);
          if (box_rows && col0 < t.col_limit) flush_box(&tm_out, stage, col0, row0, t.out_group, reduce, lane);
          stage_acquire(lane); regs_to_float(r1, v); stage_row_f32(stage, lane, v);
          if (box_rows && col0 + 32 < t.col_limit) flush_box(&tm_out, stage, col0 + 32, row0, t.out_group, reduce, lane);
          stage_acquire(lane); regs_to_float(r2, v); stage_row_f32(stage, lane, v);
          if (box_rows && col0 + 64 < t.col_limit) flush_box(&tm_out, stage, col0 + 64, row0, t.out_group, reduce, lane);
          stage_acquire(lane); regs_to_float(r3, v); stage_row_f32(stage, lane, v);
          if (box_rows && col0 + 96 < t.col_limit) flush_box(&tm_out, stage, col0 + 96, row0, t.out_group, reduce, lane);
        } else {
          stage_acquire(lane);
          regs_to_float(r0, v); stage_row_bf16(stage, lane, 0, v);
          regs_to_float(r1, v); stage_row_bf16(stage, lane, 4, v);
          if (box_rows && col0 < t.col_limit) flush_box(&tm_out, stage, col0, row0, t.out_group, false, lane);
          stage_acquire(lane);
          regs_to_float(r2, v); stage_row_bf16(stage, lane, 0, v);
          regs_to_float(r3, v); stage_row_bf16(stage, lane, 4, v);
          if (box_rows && col0 + 64 < t.col_limit) flush_box(&tm_out, stage, col0 + 64, row0, t.out_group, false, lane);
        }
      } else if (p.tma_store && EPI == EPI_SWIGLU) {
        const int half = p.N / 2;
        uint32_t rg0[32], ru0[32], rg1[32], ru1[32];
        const int c0 = half_id * 2;
        tmem_ld_32x32(taddr + c0 * 32, rg0);
        tmem_ld_32x32(taddr + 128 + c0 * 32, ru0);
        tmem_ld_32x32(taddr + (c0 + 1) * 32, rg1);
        tmem_ld_32x32(taddr + 128 + (c0 + 1) * 32, ru1);
        tmem_ld_wait();
        release_acc();
        const bool box_ok = row0 < t.row_limit && t.c_col + c0 * 32 < half;
        const int col0 = t.c_col + c0 * 32;
        float g0[32], g1[32], u[32];
        regs_to_float(rg0, g0);
        regs_to_float(rg1, g1);
        if (p.aux != nullptr && box_ok) {          // whole 32-row blocks: rows past the segment's end are padding of the buffer
          __nv_bfloat16* pre = reinterpret_cast<__nv_bfloat16*>(p.aux);
          aux_store32(pre, row, col0, p.ld_aux, g0);
          aux_store32(pre, row, col0 + 32, p.ld_aux, g1);
          regs_to_float(ru0, u); aux_store32(pre, row, half + col0, p.ld_aux, u);
          regs_to_float(ru1, u); aux_store32(pre, row, half + col0 + 32, p.ld_aux, u);
        }
        regs_to_float(ru0, u);
#pragma unroll
        for (int j = 0; j < 32; ++j) g0[j] = g0[j] * sigmoidf_fast(g0[j]) * (u[j] * wrow);
        regs_to_float(ru1, u);
#pragma unroll
        for (int j = 0; j < 32; ++j) g1[j] = g1[j] * sigmoidf_fast(g1[j]) * (u[j] * wrow);
        stage_acquire(lane);
        stage_row_bf16(stage, lane, 0, g0); stage_row_bf16(stage, lane, 4, g1);
        if (box_ok) flush_box(&tm_out, stage, col0, row0, 0, false, lane);
      } else if (p.tma_store) {  // EPI_SWIGLU_BWD
        // Four 32-column chunks; registers hold one chunk at a time (accumulator, saved gate / up, results), the packed
        // d(up) of an even chunk, which waits for its own box, and the packed saved values of the next chunk.
        const __nv_bfloat16* pre = reinterpret_cast<const __nv_bfloat16*>(p.aux);
        uint4 keep[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int c = half_id * 4 + k;
          const int col = t.c_col + c * 32;
          uint32_t r[32];
          float g[32], u[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          if (k == 3) release_acc();
          if (swb_fast) {
            unpack_bf16x8<0>(cg[0], g); unpack_bf16x8<8>(cg[1], g); unpack_bf16x8<16>(cg[2], g); unpack_bf16x8<24>(cg[3], g);
            unpack_bf16x8<0>(cu[0], u); unpack_bf16x8<8>(cu[1], u); unpack_bf16x8<16>(cu[2], u); unpack_bf16x8<24>(cu[3], u);
            if (k < 3) aux_load32(pre, row, col + 32, p.N + col + 32, p.ld_aux, cg, cu);   // in flight during the math below
          } else if (row0 < t.row_limit && aux_vec && col < p.N) {      // tiles that reach past N: chunk by chunk
            uint4 tg[4], tu[4];
            aux_load32(pre, row, col, p.N + col, p.ld_aux, tg, tu);
            unpack_bf16x8<0>(tg[0], g); unpack_bf16x8<8>(tg[1], g); unpack_bf16x8<16>(tg[2], g); unpack_bf16x8<24>(tg[3], g);
            unpack_bf16x8<0>(tu[0], u); unpack_bf16x8<8>(tu[1], u); unpack_bf16x8<16>(tu[2], u); unpack_bf16x8<24>(tu[3], u);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) { g[j] = 0.f; u[j] = 0.f; }
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) {             // g <- d gate, u <- d up
            const float acc = __uint_as_float(r[j]);
            const float d = acc * wrow;
            const float sg = sigmoidf_fast(g[j]);
            const float silu = g[j] * sg;
            wgrad_part = fmaf(acc, silu * u[j], wgrad_part);
            const float dgate = d * u[j] * (sg + silu * (1.f - sg));
            u[j] = d * silu;
            g[j] = dgate;
          }
          if ((k & 1) == 0) {
            stage_acquire(lane);
            stage_row_bf16(stage, lane, 0, g);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              keep[j].x = pack_bf16(u[8 * j + 0], u[8 * j + 1]); keep[j].y = pack_bf16(u[8 * j + 2], u[8 * j + 3]);
              keep[j].z = pack_bf16(u[8 * j + 4], u[8 * j + 5]); keep[j].w = pack_bf16(u[8 * j + 6], u[8 * j + 7]);
            }
          } else {
            const int col0 = col - 32;
            const bool box_ok = row0 < t.row_limit && col0 < p.N;
            stage_row_bf16(stage, lane, 4, g);
            if (box_ok) flush_box(&tm_out, stage, col0, row0, 0, false, lane);
            stage_acquire(lane);
#pragma unroll
            for (int j = 0; j < 4; ++j) stage_chunk(stage, lane, j, keep[j]);
            stage_row_bf16(stage, lane, 4, u);
            if (box_ok) flush_box(&tm_out, stage, p.N + col0, row0, 0, false, lane);
          }
        }
      } else if (EPI == EPI_STORE) {
        // this warp's four chunks: one TMEM round trip
        uint32_t r0[32], r1[32], r2[32], r3[32];
        const int c0 = half_id * 4;
        tmem_ld_32x32(taddr + (c0 + 0) * 32, r0);
        tmem_ld_32x32(taddr + (c0 + 1) * 32, r1);
        tmem_ld_32x32(taddr + (c0 + 2) * 32, r2);
        tmem_ld_32x32(taddr + (c0 + 3) * 32, r3);
        tmem_ld_wait();
        auto put = [&](uint32_t (&r)[32], int c) {
          float v[32];
          regs_to_float(r, v);
          const int col = t.c_col + c * 32;
          const int valid = t.col_limit - col;
          if (row_ok && valid > 0) {
            if (p.out_fp32)
              store_row_f32(reinterpret_cast<float*>(p.out) + t.out_offset + (long long)row * p.ldo + col, v, valid,
                            p.accumulate, p.atomic_out);
            else
              store_row_bf16(reinterpret_cast<__nv_bfloat16*>(p.out) + t.out_offset + (long long)row * p.ldo + col, v, valid);
          }
        };
        put(r0, c0); put(r1, c0 + 1); put(r2, c0 + 2); put(r3, c0 + 3);
      } else if (EPI == EPI_SWIGLU) {
        const int half = p.N / 2;
        uint32_t rg0[32], ru0[32], rg1[32], ru1[32];
        const int c0 = half_id * 2;
        tmem_ld_32x32(taddr + c0 * 32, rg0);
        tmem_ld_32x32(taddr + 128 + c0 * 32, ru0);
        tmem_ld_32x32(taddr + (c0 + 1) * 32, rg1);
        tmem_ld_32x32(taddr + 128 + (c0 + 1) * 32, ru1);
        tmem_ld_wait();
        auto put = [&](uint32_t (&rg)[32], uint32_t (&ru)[32], int c) {
          float g[32], u[32];
          regs_to_float(rg, g);
          regs_to_float(ru, u);
          const int col = t.c_col + c * 32;
          const int valid = half - col;
          if (row_ok && valid > 0) {
            if (p.aux != nullptr) {                 // N % 256 == 0 for this epilogue: chunks are whole
              __nv_bfloat16* pre = reinterpret_cast<__nv_bfloat16*>(p.aux);
              aux_store32(pre, row, col, p.ld_aux, g);
              aux_store32(pre, row, half + col, p.ld_aux, u);
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) g[j] = g[j] * sigmoidf_fast(g[j]) * (u[j] * wrow);
            store_row_bf16(reinterpret_cast<__nv_bfloat16*>(p.out) + (long long)row * p.ldo + col, g, valid);
          }
        };
        put(rg0, ru0, c0); put(rg1, ru1, c0 + 1);
      } else {  // EPI_SWIGLU_BWD: accumulator = d(post); aux = saved [gate | up]; out = [d gate | d up]
#pragma unroll 1
        for (int cc = 0; cc < 4; cc += 2) {
          uint32_t ra[32], rb[32];
          const int c0 = half_id * 4 + cc;
          tmem_ld_32x32(taddr + c0 * 32, ra);
          tmem_ld_32x32(taddr + (c0 + 1) * 32, rb);
          tmem_ld_wait();
          auto put = [&](uint32_t (&r)[32], int c) {
            float d[32], g[32], u[32];
            regs_to_float(r, d);
            const int col = t.c_col + c * 32;
            const int valid = p.N - col;
            if (row_ok && valid > 0) {
              uint4 tg[4], tu[4];
              aux_load32(reinterpret_cast<const __nv_bfloat16*>(p.aux), row, col, p.N + col, p.ld_aux, tg, tu);
              unpack_bf16x8<0>(tg[0], g); unpack_bf16x8<8>(tg[1], g); unpack_bf16x8<16>(tg[2], g); unpack_bf16x8<24>(tg[3], g);
              unpack_bf16x8<0>(tu[0], u); unpack_bf16x8<8>(tu[1], u); unpack_bf16x8<16>(tu[2], u); unpack_bf16x8<24>(tu[3], u);
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float s = sigmoidf_fast(g[j]);
                const float silu = g[j] * s;
                if (j < valid) wgrad_part = fmaf(d[j], silu * u[j], wgrad_part);
                const float dd = d[j] * wrow;
                const float dgate = dd * u[j] * (s + silu * (1.f - s));
                u[j] = dd * silu;     // d up
                g[j] = dgate;         // d gate
              }
              __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (long long)row * p.ldo;
              store_row_bf16(o + col, g, valid);
              store_row_bf16(o + p.N + col, u, valid);
            }
          };
          put(ra, c0); put(rb, c0 + 1);
        }
      }
      if (EPI == EPI_SWIGLU_BWD && p.row_grad != nullptr && p.row_slot != nullptr && row_ok) {
        const int slot = __ldg(p.row_slot + row);
        if (slot >= 0) atomicAdd(p.row_grad + slot, wgrad_part);     // eight partial sums per row (column halves x N tiles)
      }
      if (warp == 2 && lane == 0) GTRACE(8 * acc_it + 5);
      if (!released) release_acc();
      ++acc_it;
    }
  }

  // ---- teardown: every thread arrives here, also after an abort ----
  if (p.tma_store && warp >= 2 && lane == 0) tma_store_wait<0>();   // this thread's bulk stores have been written
  tc_fence_before_sync();
  __syncthreads();
#ifdef MTS_GEMM_TRACE
  if (threadIdx.x == 0 && blockIdx.x == 0) { g_gemm_trace[4002] = clock64(); g_gemm_trace[4003] = (long long)global_timer_ns(); }
#endif
  if (threadIdx.x == 0 && abort_word != 0) {
    // Loads that were issued but never consumed may still be in flight: give them a bounded
    // chance to land before shared memory is released.
    if (PAIR) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);   // 0.2 ms: far longer than any copy takes
    } else {
      for (int i = loads_consumed; i < loads_issued; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        for (int spin = 0; spin < (1 << 20) && !mbar_test(&full_bar[s], ph); ++spin) {
        }
      }
    }
    if (p.status != nullptr) atomicMax(p.status, abort_word);
  }
  __syncthreads();
  if (PAIR) cluster_sync_all();   // neither CTA leaves while the other may still signal its barriers or read its tiles
  if (warp == 0) {
    if (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- host side ------------------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
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

// 2-D bf16 tensor [rows, cols] (cols contiguous), box = [box_rows, 64 cols], 128-byte swizzle.
// The tensor-map encoder is a driver entry point and needs a current context.  Worker threads (the
// autograd engine's, for one) may reach this code before any runtime call has bound the primary
// context to them, so bind it once per thread.
void ensure_context_current() {
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

bool encode_bf16_2d(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  ensure_context_current();
  auto fn = encode_fn();
  if (fn == nullptr) { g_last_error = "cuTensorMapEncodeTiled entry point not found"; return false; }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld * 2) % 16 != 0 || rows <= 0 || cols <= 0) {
    g_last_error = "operand base/pitch not 16-byte aligned or empty";
    return false;
  }
  const cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(ld) * 2};
  const cuuint32_t box[2] = {64u, cuuint32_t(box_rows)};
  const cuuint32_t elem[2] = {1u, 1u};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    static char msg[160];
    snprintf(msg, sizeof(msg), "cuTensorMapEncodeTiled error %d (rows=%lld cols=%lld ld=%lld box_rows=%d)", int(r),
             (long long)rows, (long long)cols, (long long)ld, box_rows);
    g_last_error = msg;
  }
  return r == CUDA_SUCCESS;
}

// Output view [groups, rows, cols] (cols contiguous, row pitch `ld`, group pitch `group_stride` elements) cut into boxes of
// 32 rows x 128 bytes with the 128-byte swizzle the epilogue stages in.  Returns false when the view cannot be described.
bool encode_out_3d(CUtensorMap* map, const void* base, bool fp32, int64_t cols, int64_t rows, int64_t groups, int64_t ld,
                   int64_t group_stride) {
  ensure_context_current();
  auto fn = encode_fn();
  const int64_t es = fp32 ? 4 : 2;
  if (fn == nullptr || base == nullptr || (reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld * es) % 16 != 0 || cols <= 0 ||
      rows <= 0 || groups <= 0)
    return false;
  if (groups > 1 && (group_stride * es) % 16 != 0) return false;
  const int64_t gs = groups > 1 ? group_stride : rows * ld;
  const cuuint64_t dims[3] = {cuuint64_t(cols), cuuint64_t(rows), cuuint64_t(groups)};
  const cuuint64_t strides[2] = {cuuint64_t(ld * es), cuuint64_t(gs * es)};
  const cuuint32_t box[3] = {cuuint32_t(128 / es), 32u, 1u};
  const cuuint32_t elem[3] = {1u, 1u, 1u};
  const CUresult r = fn(map, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base),
                        dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return dev >= 0 && dev < 64 ? dev : 0;
}

int sm_count() {       // per device: a process may drive several
  static int n[64] = {};
  const int dev = current_device();
  if (n[dev] == 0) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
  return n[dev];
}

}  // namespace

cudaError_t launch_gemm_sm100(const GemmArgs& a) {
  CUtensorMap tm_a, tm_b;
  // a gathered operand is fetched four rows at a time by index (tile::gather4): its map describes boxes of one row
  g_last_error = "gathered operands need the paired kernel; B (and A in grouped-K) must be MN-major, A K-major only in grouped-M";
  if ((a.gather_a != nullptr || a.gather_b != nullptr) && !a.pair) return cudaErrorInvalidValue;
  if (a.gather_b != nullptr && !(a.b_mn_major && a.mode == GEMM_GROUPED_K)) return cudaErrorInvalidValue;
  if (a.gather_a != nullptr && !((a.a_mn_major && a.mode == GEMM_GROUPED_K) || (!a.a_mn_major && a.mode == GEMM_GROUPED_M)))
    return cudaErrorInvalidValue;
  g_last_error = "";
  if (!encode_bf16_2d(&tm_a, a.a, a.a_rows, a.a_cols, a.lda, a.gather_a != nullptr ? 1 : (a.a_mn_major ? 64 : 128))) return cudaErrorInvalidValue;
  if (!encode_bf16_2d(&tm_b, a.b, a.b_rows, a.b_cols, a.ldb, a.gather_b != nullptr ? 1 : (a.b_mn_major ? 64 : 128))) return cudaErrorInvalidValue;

  KernelParams p{};
  p.M = int(a.M); p.N = int(a.N); p.K = int(a.K);
  p.mode = a.mode; p.epilogue = a.epilogue;
  p.a_mn = a.a_mn_major; p.b_mn = a.b_mn_major;
  p.out = a.out; p.ldo = a.ldo; p.out_fp32 = a.out_fp32; p.accumulate = a.accumulate; p.atomic_out = a.atomic_out;
  p.aux = a.aux; p.ld_aux = a.ld_aux;
  p.tile_group = a.tile_group; p.num_row_tiles = a.num_row_tiles; p.group_rows = a.group_rows;
  p.num_groups = a.num_groups;
  p.k_splits = a.k_splits > 1 ? a.k_splits : 1;
  p.b_group_stride_rows = int(a.b_group_stride_rows);
  p.out_group_stride = a.out_group_stride;
  p.status = a.status;
  p.gather_a = a.gather_a; p.gather_b = a.gather_b;
  p.gather_a_rows = int(a.a_rows); p.gather_b_rows = int(a.b_rows);
  p.row_scale = a.row_scale; p.row_slot = a.row_slot; p.row_grad = a.row_grad;
  const bool pair = a.pair != 0;
  // epilogue through shared memory + TMA when every output view can be described by a tensor map
  CUtensorMap tm_out, tm_aux;
  static const int env_tma_store = [] { const char* e = getenv("MTS_GEMM_TMA_STORE"); return e ? atoi(e) : 1; }();
  {
    const int64_t out_cols = a.epilogue == EPI_SWIGLU ? a.N / 2 : (a.epilogue == EPI_SWIGLU_BWD ? 2 * a.N : a.N);
    const int64_t groups = (a.mode == GEMM_GROUPED_K && a.out_group_stride > 0) ? a.num_groups : 1;
    // TMA stores clip at 16-byte granularity: the view is widened to the next 16-byte boundary when the row pitch has the
    // room (those pad columns then receive exact zeros), otherwise the per-lane store path is used.
    const int64_t per16 = a.out_fp32 ? 4 : 8;
    int64_t map_cols = (out_cols + per16 - 1) / per16 * per16;
    bool ok = env_tma_store != 0 && (map_cols == out_cols || (map_cols <= a.ldo && a.epilogue == EPI_STORE && !a.accumulate && !a.atomic_out));
    ok = ok && encode_out_3d(&tm_out, a.out, a.out_fp32 != 0, map_cols, a.M, groups, a.ldo, a.out_group_stride);
    if (ok) tm_aux = tm_out;     // spare map slot: the saved pre-activations are written with plain coalesced stores
    if (!ok) { tm_out = tm_a; tm_aux = tm_a; }
    p.tma_store = ok ? 1 : 0;
  }
  static const int env_noload = [] { const char* e = getenv("MTS_GEMM_DIAG_NOLOAD"); return e ? atoi(e) : 0; }();
  p.diag_no_loads = env_noload;
  const int tile_m = pair ? 256 : 128;
  p.tiles_m = int((a.M + tile_m - 1) / tile_m);
  p.tiles_n = int((a.N + BN - 1) / BN);
  g_last_error = "inconsistent epilogue arguments";
  if (a.epilogue == EPI_SWIGLU && (a.N % 256 != 0 || a.mode != GEMM_GROUPED_M || a.b_mn_major)) return cudaErrorInvalidValue;
  if (a.epilogue == EPI_SWIGLU_BWD && (a.aux == nullptr || a.N % 32 != 0)) return cudaErrorInvalidValue;
  // saved pre-activations: blocked layout of 32-row x 8-value chunks (see aux_chunk), addressed with 16-byte accesses
  if (a.aux != nullptr && ((reinterpret_cast<uintptr_t>(a.aux) & 15) != 0 || a.ld_aux % 8 != 0)) return cudaErrorInvalidValue;
  if (a.atomic_out && !a.out_fp32) return cudaErrorInvalidValue;
  if (p.k_splits > 1 && (a.mode != GEMM_GROUPED_K || !a.atomic_out)) return cudaErrorInvalidValue;   // parts add into one output
  g_last_error = "";

  long long total = (long long)p.tiles_m * p.tiles_n;
  if (a.mode == GEMM_GROUPED_K) total *= (long long)a.num_groups * p.k_splits;
  if (total <= 0) return cudaSuccess;
  int workers = pair ? sm_count() / 2 : sm_count();
  if (a.sm_limit > 0 && a.sm_limit < workers * (pair ? 2 : 1)) workers = pair ? (a.sm_limit / 2 > 0 ? a.sm_limit / 2 : 1) : a.sm_limit;
  if (total < workers) workers = int(total);

  using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const KernelParams);
#define MTS_GEMM_EPI(P, A, B) {gemm_tcgen05_kernel<P, A, B, EPI_STORE>, gemm_tcgen05_kernel<P, A, B, EPI_SWIGLU>, \
                              gemm_tcgen05_kernel<P, A, B, EPI_SWIGLU_BWD>}
  static const KernelFn kernels[2][2][2][3] = {
      {{MTS_GEMM_EPI(false, false, false), MTS_GEMM_EPI(false, false, true)},
       {MTS_GEMM_EPI(false, true, false), MTS_GEMM_EPI(false, true, true)}},
      {{MTS_GEMM_EPI(true, false, false), MTS_GEMM_EPI(true, false, true)},
       {MTS_GEMM_EPI(true, true, false), MTS_GEMM_EPI(true, true, true)}}};
#undef MTS_GEMM_EPI
  static_assert(EPI_STORE == 0 && EPI_SWIGLU == 1 && EPI_SWIGLU_BWD == 2, "the kernel table is indexed by the epilogue code");
  static bool attr_set_on[64] = {};          // cudaFuncSetAttribute applies to the current device only
  bool& attr_set = attr_set_on[current_device()];
  if (!attr_set) {
    for (int i = 0; i < 24; ++i) {
      const bool pr = (i / 12) & 1;
      cudaError_t e = cudaFuncSetAttribute(kernels[pr][(i / 6) & 1][(i / 3) & 1][i % 3], cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           int(pr ? Cfg<true>::SMEM_BYTES : Cfg<false>::SMEM_BYTES));
      if (e != cudaSuccess) return e;
    }
    attr_set = true;
  }
  if (a.epilogue < 0 || a.epilogue > 2) return cudaErrorInvalidValue;
  const KernelFn kernel = kernels[pair ? 1 : 0][a.a_mn_major ? 1 : 0][a.b_mn_major ? 1 : 0][a.epilogue];
  (void)cudaGetLastError();   // do not attribute an earlier sticky error to this launch
  cudaError_t launch_err;
  if (pair) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(workers) * 2u);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = Cfg<true>::SMEM_BYTES;
    cfg.stream = a.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    launch_err = cudaLaunchKernelEx(&cfg, kernel, tm_a, tm_b, tm_out, tm_aux, p);
  } else {
    kernel<<<workers, NUM_THREADS, Cfg<false>::SMEM_BYTES, a.stream>>>(tm_a, tm_b, tm_out, tm_aux, p);
    launch_err = cudaGetLastError();
  }
  ++g_launch_count;
  if (launch_err != cudaSuccess) g_last_error = "kernel launch failed";
  return launch_err;
}

}  // namespace mts
