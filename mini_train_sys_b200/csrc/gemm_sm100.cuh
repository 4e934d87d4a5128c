// Host-visible interface of the tcgen05 GEMM family (implemented in gemm_sm100.cu).
//
//   D[M, N] (+)= A * B^T      bf16 inputs, fp32 accumulation in tensor memory
//
// Each operand is described by how its contraction dimension lies in memory:
//   K-major  : stored [rows, K] with K contiguous        (activations in a forward pass, weights [out, in])
//   MN-major : stored [K, rows] with the rows contiguous (what dgrad / wgrad see without any transpose)
//
// Scheduling modes:
//   GEMM_DENSE     one problem.
//   GEMM_GROUPED_M rows of A / D are grouped by expert in 128-row aligned segments; the expert of each
//                  128-row tile comes from `tile_group`; B is the experts' weights stacked along rows.
//   GEMM_GROUPED_K one output per group; the contraction runs over that group's row range
//                  [group_rows[g], group_rows[g+1]) of A and B (both MN-major).  With `atomic_out` all
//                  groups add into the same output, which is how split-K wgrad is expressed; with `k_splits` > 1
//                  every group's range is cut further and the parts add into that group's output (pre-zeroed).
//
// Epilogues:
//   EPI_STORE       D -> out (bf16 or fp32; optional accumulate; optional fp32 atomic add).  When N is not a multiple of
//                   16 bytes' worth of elements and the row pitch has room, the columns between N and that boundary
//                   are overwritten with zeros (the store goes through TMA, which clips at 16-byte granularity).
//   EPI_SWIGLU      the 256 accumulator columns are [128 gate | 128 up] of one expert:
//                   out = silu(gate) * up (bf16, [M, N/2]); aux (optional) receives gate/up (bf16, [M, N])
//   EPI_SWIGLU_BWD  accumulator = d(post) ; aux holds the saved gate/up; out = [d gate | d up] (bf16, [M, 2*N])
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace mts {

enum GemmMode : int { GEMM_DENSE = 0, GEMM_GROUPED_M = 1, GEMM_GROUPED_K = 2 };
enum GemmEpilogue : int { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_SWIGLU_BWD = 2 };

struct GemmArgs {
  // operands (bf16).  `a_rows`/`b_rows` are the extents of the stored 2-D arrays [rows, cols], row-major,
  // with leading dimension `lda`/`ldb` in elements (must be a multiple of 8).
  const void* a = nullptr;
  const void* b = nullptr;
  int64_t a_rows = 0, a_cols = 0, lda = 0;
  int64_t b_rows = 0, b_cols = 0, ldb = 0;
  int a_mn_major = 0, b_mn_major = 0;

  // problem: DENSE M,N,K.  GROUPED_M: M = row capacity (multiple of 128), N,K per expert.
  // GROUPED_K: M,N = output dims per group, K unused.
  int64_t M = 0, N = 0, K = 0;
  int mode = GEMM_DENSE;
  int epilogue = EPI_STORE;

  // output
  void* out = nullptr;
  int64_t ldo = 0;
  int out_fp32 = 0;
  int accumulate = 0;   // out += D (non-atomic read-modify-write)
  int atomic_out = 0;   // fp32 red.add into out
  void* aux = nullptr;  // EPI_SWIGLU: optional pre-activation store; EPI_SWIGLU_BWD: saved pre-activation
  int64_t ld_aux = 0;

  // grouping
  const int* tile_group = nullptr;   // GROUPED_M: group id of every 128-row tile
  const int* num_row_tiles = nullptr;  // GROUPED_M: device scalar, number of live 128-row tiles
  const int* group_rows = nullptr;   // GROUPED_K: [groups + 1] row offsets (multiples of 64)
  int num_groups = 1;
  int k_splits = 1;                  // GROUPED_K with atomic_out: cut every group's rows into this many work items (load balance)
  int64_t b_group_stride_rows = 0;   // GROUPED_M: rows of stacked B per group
  int64_t out_group_stride = 0;      // GROUPED_K: elements between consecutive group outputs (0 with atomic_out)

  // Operands gathered by row index (paired kernel only).  `gather_a`: grouped-M with a K-major A - output row r reads row
  // gather_a[r] of the tensor `a`; grouped-K with an MN-major A - contraction row k reads row gather_a[k].  `gather_b`: grouped-K,
  // MN-major B, same meaning.  A negative index is a row of zeros.  Index arrays have one entry per row of the padded layout.
  const int* gather_a = nullptr;
  const int* gather_b = nullptr;
  // SwiGLU epilogues: optional weight per output row.  EPI_SWIGLU: out = weight * silu(gate) * up.  EPI_SWIGLU_BWD: the
  // accumulator is the gradient of that weighted output, so d(gate, up) use weight * accumulator, and the gradient of the
  // weight, sum_i acc * silu(gate) * up, is added to row_grad[row_slot[row]] (rows with a negative slot add nothing).
  const float* row_scale = nullptr;
  const int* row_slot = nullptr;
  float* row_grad = nullptr;

  int pair = 0;                      // 1: two-CTA clusters on 256 x 256 tiles (GROUPED_M then needs 256-row aligned segments)
  int* status = nullptr;             // device int: receives a KernelStatus on failure
  int sm_limit = 0;                  // cap on CTAs (0 = all SMs)
  cudaStream_t stream = nullptr;
};

// Returns cudaSuccess or the launch / descriptor error.
cudaError_t launch_gemm_sm100(const GemmArgs& args);

// Number of kernels launched through this library since load (the benchmark reports it).
extern std::atomic<unsigned long long> g_launch_count;
// Human-readable reason of the most recent launch_gemm_sm100 failure ("" when none).
extern const char* g_last_error;

}  // namespace mts
