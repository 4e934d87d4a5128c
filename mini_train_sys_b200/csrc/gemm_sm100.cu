// Persistent, warp-specialised tcgen05 GEMM for sm_100a (see gemm_sm100.cuh for the interface).
//
// CTA = 192 threads: warp 0 issues TMA loads into a 4-stage shared-memory ring, warp 1 issues
// tcgen05.mma (128 x 256 x 16 per instruction, fp32 accumulators in tensor memory), warps 2-5 drain
// the accumulator (tcgen05.ld) and run the epilogue.  Two 256-column accumulators ping-pong, so
// the epilogue of tile i overlaps the MMAs of tile i+1.  One CTA per SM, tiles assigned round-robin.
//
// Reference counterpart: the Triton grouped-GEMM kernels of minitrain/kernels/triton/fused_moe_kernels.py
// (:264-437, :500-828) and the cuBLAS-backed nn.Linear layers; none of them has an sm_100 path.
#include "gemm_sm100.cuh"
#include "ptx_sm100.cuh"

#include <cudaTypedefs.h>
#include <cstdio>
#include <mutex>

namespace mts {

unsigned long long g_launch_count = 0;
const char* g_last_error = "";

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int ACC_COLS = 256;
constexpr int TMEM_COLS = 512;
constexpr int MN_BLOCK_BYTES = BK * 128;  // one 64-wide MN block of an MN-major operand: BK rows of 128 B
constexpr size_t SMEM_BYTES = size_t(STAGES) * STAGE_BYTES + 1024;

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
  int b_group_stride_rows;
  long long out_group_stride;
  int tiles_m, tiles_n;
  int* status;
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
  int row_limit, col_limit;
};

__device__ __forceinline__ int live_tiles(const KernelParams& p) {
  if (p.mode == GEMM_GROUPED_M) {
    int rows = *p.num_row_tiles;
    rows = rows < p.tiles_m ? rows : p.tiles_m;
    return rows * p.tiles_n;
  }
  if (p.mode == GEMM_GROUPED_K) return p.num_groups * p.tiles_m * p.tiles_n;
  return p.tiles_m * p.tiles_n;
}

__device__ __forceinline__ Tile decode_tile(const KernelParams& p, int t) {
  Tile o;
  o.b_k_offset = 0;
  o.out_offset = 0;
  if (p.mode == GEMM_GROUPED_K) {
    const int per = p.tiles_m * p.tiles_n;
    const int g = t / per;
    const int r = t - g * per;
    const int mt = r / p.tiles_n, nt = r - mt * p.tiles_n;
    const int k0 = p.group_rows[g], k1 = p.group_rows[g + 1];
    o.a_coord = mt * BM;
    o.b_coord = nt * BN;
    o.b_coord2 = o.b_coord + 128;
    o.k_begin = k0;
    o.k_blocks = (k1 - k0 + BK - 1) / BK;
    o.c_row = mt * BM;
    o.c_col = nt * BN;
    o.out_offset = (long long)g * p.out_group_stride;
    o.row_limit = p.M;
    o.col_limit = p.N;
    return o;
  }
  const int mt = t / p.tiles_n, nt = t - mt * p.tiles_n;
  o.a_coord = mt * BM;
  o.k_begin = 0;
  o.k_blocks = (p.K + BK - 1) / BK;
  o.c_row = mt * BM;
  o.c_col = nt * BN;
  o.row_limit = p.M;
  o.col_limit = p.N;
  o.b_coord = nt * BN;
  o.b_coord2 = o.b_coord + 128;
  if (p.mode == GEMM_GROUPED_M) {
    const int g = p.tile_group[mt];
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

__device__ __forceinline__ void load_row_bf16(const __nv_bfloat16* src, float (&v)[32], int valid_cols) {
  if (valid_cols >= 32 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 q = reinterpret_cast<const uint4*>(src)[j];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
        v[8 * j + 2 * i] = __low2float(h);
        v[8 * j + 2 * i + 1] = __high2float(h);
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = j < valid_cols ? __bfloat162float(src[j]) : 0.f;
  }
}

__device__ __forceinline__ void regs_to_float(const uint32_t (&r)[32], float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
}

__device__ __forceinline__ float sigmoidf_fast(float x) { return 1.f / (1.f + __expf(-x)); }

// ---- the kernel ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    const KernelParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_word;
  __shared__ int loads_issued, loads_consumed;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);  // one arrive per epilogue warp
    }
    abort_word = 0;
    loads_issued = 0;
    loads_consumed = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }
  if (warp == 0) {
    tmem_alloc(&tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abort_ptr = &abort_word;

  const int total = live_tiles(p);

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const Tile t = decode_tile(p, tile);
        for (int kb = 0; kb < t.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_ptr)) { ok = false; break; }
          uint8_t* a_dst = smem + s * STAGE_BYTES;
          uint8_t* b_dst = a_dst + A_BYTES;
          const int k = t.k_begin + kb * BK;
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          if (p.a_mn) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(a_dst + j * MN_BLOCK_BYTES, &tm_a, &full_bar[s], t.a_coord + 64 * j, k);
          } else {
            tma_load_2d(a_dst, &tm_a, &full_bar[s], k, t.a_coord);
          }
          if (p.b_mn) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(b_dst + j * MN_BLOCK_BYTES, &tm_b, &full_bar[s], t.b_coord + 64 * j, k + t.b_k_offset);
          } else {
            tma_load_2d(b_dst, &tm_b, &full_bar[s], k, t.b_coord);
            tma_load_2d(b_dst + 128 * 128, &tm_b, &full_bar[s], k, t.b_coord2);
          }
        }
      }
      loads_issued = it;
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================= MMA issuer =================
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, p.a_mn != 0, p.b_mn != 0);
      int it = 0, acc_it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const Tile t = decode_tile(p, tile);
        if (t.k_blocks == 0) continue;
        const int buf = acc_it & 1;
        const uint32_t acc_ph = (acc_it >> 1) & 1;
        if (!mbar_wait(&acc_empty[buf], acc_ph ^ 1, abort_ptr)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * ACC_COLS;
        for (int kb = 0; kb < t.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_ptr)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t a_desc = p.a_mn ? make_smem_desc_sw128(a_addr + k * (UMMA_K * 128), MN_BLOCK_BYTES, 1024)
                                           : make_smem_desc_sw128(a_addr + k * (UMMA_K * 2), 16, 1024);
            const uint64_t b_desc = p.b_mn ? make_smem_desc_sw128(b_addr + k * (UMMA_K * 128), MN_BLOCK_BYTES, 1024)
                                           : make_smem_desc_sw128(b_addr + k * (UMMA_K * 2), 16, 1024);
            umma_bf16_ss(d_tmem, a_desc, b_desc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
        }
        if (!ok) break;
        umma_commit(&acc_full[buf]);
        ++acc_it;
      }
      loads_consumed = it;
    }
    __syncwarp();
  } else {
    // ================= epilogue (warps 2..5 -> TMEM lane quarters 2,3,0,1) =================
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    int acc_it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
      const Tile t = decode_tile(p, tile);
      const int row = t.c_row + row_in_tile;
      const bool row_ok = row < t.row_limit;
      if (t.k_blocks == 0) {
        // nothing was contracted: the product is zero
        if (p.epilogue == EPI_STORE && !p.accumulate && !p.atomic_out && row_ok) {
          float z[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) z[j] = 0.f;
          for (int c = 0; c < BN / 32; ++c) {
            const int col = t.c_col + c * 32;
            const int valid = t.col_limit - col;
            if (valid <= 0) break;
            if (p.out_fp32) store_row_f32(reinterpret_cast<float*>(p.out) + t.out_offset + (long long)row * p.ldo + col, z, valid, 0, 0);
            else store_row_bf16(reinterpret_cast<__nv_bfloat16*>(p.out) + t.out_offset + (long long)row * p.ldo + col, z, valid);
          }
        }
        continue;
      }
      const int buf = acc_it & 1;
      const uint32_t acc_ph = (acc_it >> 1) & 1;
      if (!mbar_wait_warp(&acc_full[buf], acc_ph, abort_ptr, lane)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + buf * ACC_COLS;

      if (p.epilogue == EPI_STORE) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          float v[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
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
        }
      } else if (p.epilogue == EPI_SWIGLU) {
        const int half = p.N / 2;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t rg[32], ru[32];
          float g[32], u[32];
          tmem_ld_32x32(taddr + c * 32, rg);
          tmem_ld_32x32(taddr + 128 + c * 32, ru);
          tmem_ld_wait();
          regs_to_float(rg, g);
          regs_to_float(ru, u);
          const int col = t.c_col + c * 32;
          const int valid = half - col;
          if (row_ok && valid > 0) {
            if (p.aux != nullptr) {
              __nv_bfloat16* pre = reinterpret_cast<__nv_bfloat16*>(p.aux) + (long long)row * p.ld_aux;
              store_row_bf16(pre + col, g, valid);
              store_row_bf16(pre + half + col, u, valid);
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) g[j] = g[j] * sigmoidf_fast(g[j]) * u[j];
            store_row_bf16(reinterpret_cast<__nv_bfloat16*>(p.out) + (long long)row * p.ldo + col, g, valid);
          }
        }
      } else {  // EPI_SWIGLU_BWD: accumulator = d(post); aux = saved [gate | up]; out = [d gate | d up]
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          float d[32], g[32], u[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          regs_to_float(r, d);
          const int col = t.c_col + c * 32;
          const int valid = p.N - col;
          if (row_ok && valid > 0) {
            const __nv_bfloat16* pre = reinterpret_cast<const __nv_bfloat16*>(p.aux) + (long long)row * p.ld_aux;
            load_row_bf16(pre + col, g, valid);
            load_row_bf16(pre + p.N + col, u, valid);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float s = sigmoidf_fast(g[j]);
              const float silu = g[j] * s;
              const float dgate = d[j] * u[j] * (s + silu * (1.f - s));
              u[j] = d[j] * silu;   // d up
              g[j] = dgate;         // d gate
            }
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (long long)row * p.ldo;
            store_row_bf16(o + col, g, valid);
            store_row_bf16(o + p.N + col, u, valid);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
      ++acc_it;
    }
  }

  // ---- teardown: every thread arrives here, also after an abort ----
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && abort_word != 0) {
    // Loads that were issued but never consumed may still be in flight: give them a bounded
    // chance to land before shared memory is released.
    for (int i = loads_consumed; i < loads_issued; ++i) {
      const int s = i % STAGES;
      const uint32_t ph = (i / STAGES) & 1;
      for (int spin = 0; spin < (1 << 20) && !mbar_test(&full_bar[s], ph); ++spin) {
      }
    }
    if (p.status != nullptr) atomicMax(p.status, abort_word);
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
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

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

}  // namespace

cudaError_t launch_gemm_sm100(const GemmArgs& a) {
  CUtensorMap tm_a, tm_b;
  if (!encode_bf16_2d(&tm_a, a.a, a.a_rows, a.a_cols, a.lda, a.a_mn_major ? 64 : 128)) return cudaErrorInvalidValue;
  if (!encode_bf16_2d(&tm_b, a.b, a.b_rows, a.b_cols, a.ldb, a.b_mn_major ? 64 : 128)) return cudaErrorInvalidValue;

  KernelParams p{};
  p.M = int(a.M); p.N = int(a.N); p.K = int(a.K);
  p.mode = a.mode; p.epilogue = a.epilogue;
  p.a_mn = a.a_mn_major; p.b_mn = a.b_mn_major;
  p.out = a.out; p.ldo = a.ldo; p.out_fp32 = a.out_fp32; p.accumulate = a.accumulate; p.atomic_out = a.atomic_out;
  p.aux = a.aux; p.ld_aux = a.ld_aux;
  p.tile_group = a.tile_group; p.num_row_tiles = a.num_row_tiles; p.group_rows = a.group_rows;
  p.num_groups = a.num_groups;
  p.b_group_stride_rows = int(a.b_group_stride_rows);
  p.out_group_stride = a.out_group_stride;
  p.status = a.status;
  p.tiles_m = int((a.M + BM - 1) / BM);
  p.tiles_n = int((a.N + BN - 1) / BN);
  g_last_error = "inconsistent epilogue arguments";
  if (a.epilogue == EPI_SWIGLU && (a.N % 256 != 0 || a.mode != GEMM_GROUPED_M || a.b_mn_major)) return cudaErrorInvalidValue;
  if (a.epilogue == EPI_SWIGLU_BWD && a.aux == nullptr) return cudaErrorInvalidValue;
  if (a.atomic_out && !a.out_fp32) return cudaErrorInvalidValue;
  g_last_error = "";

  long long total = (long long)p.tiles_m * p.tiles_n;
  if (a.mode == GEMM_GROUPED_K) total *= a.num_groups;
  if (total <= 0) return cudaSuccess;
  int ctas = sm_count();
  if (a.sm_limit > 0 && a.sm_limit < ctas) ctas = a.sm_limit;
  if (total < ctas) ctas = int(total);

  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM_BYTES));
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  (void)cudaGetLastError();   // do not attribute an earlier sticky error to this launch
  gemm_tcgen05_kernel<<<ctas, NUM_THREADS, SMEM_BYTES, a.stream>>>(tm_a, tm_b, p);
  ++g_launch_count;
  const cudaError_t launch_err = cudaGetLastError();
  if (launch_err != cudaSuccess) g_last_error = "kernel launch failed";
  return launch_err;
}

}  // namespace mts
