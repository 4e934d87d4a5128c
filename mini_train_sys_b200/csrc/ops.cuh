// Launchers of the non-GEMM sm_100a kernels (raw pointers + stream; no framework types).
// Each returns the launch error; all increment mts::g_launch_count.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace mts {

extern std::atomic<unsigned long long> g_launch_count;
int device_sm_count();

// Values that change with every optimizer step but must not be baked into kernel arguments, so that a whole step can be
// replayed from a CUDA graph: kernels read them from this per-device block, the host rewrites it before each replay.
// All zeros (the state outside graph replay) reproduces the by-value behaviour exactly.
struct StepContext {
  unsigned long long salt;      // mixed into every dropout seed (fused dropout + residual, attention dropout)
  unsigned int epoch_delta;     // added to the sequence number of every peer-flag signal / wait
  unsigned int dynamic_adam;    // 1: the table-driven AdamW takes the four values below instead of its arguments
  float lr0, lr1, bias_correction1, bias_correction2;
  unsigned int reserved[8];
};
constexpr unsigned long long kSaltMultiplier = 0x9E3779B97F4A7C15ull;
// Device pointer of the calling thread's current device; allocated (zero-filled) on first use, never freed.
StepContext* step_context();
// Rewrite the block on `stream` (a one-thread kernel: the values travel as launch arguments, so consecutive steps never race
// on a host staging buffer).
cudaError_t launch_set_step_context(unsigned long long salt, unsigned int epoch_delta, unsigned int dynamic_adam, float lr0, float lr1,
                                    float bias_correction1, float bias_correction2, cudaStream_t stream);

// ---- elementwise.cu ----
cudaError_t launch_rmsnorm_fwd(const void* x, const float* w, void* y, float* rstd, long long rows, int H, float eps,
                               bool bf16, cudaStream_t stream);
cudaError_t launch_rmsnorm_bwd(const void* dy, const void* x, const float* w, const float* rstd, const void* dres, void* dx,
                               float* dw, long long rows, int H, bool bf16, cudaStream_t stream);
cudaError_t launch_rope(const void* in, void* out, const void* cosp, const void* sinp, int B, int Hh, int S, int D,
                        long long sb, long long sh, long long ss, long long osb, long long osh, long long oss,
                        bool backward, bool bf16, cudaStream_t stream);
cudaError_t launch_swiglu_fwd(const void* g, const void* u, void* out, long long n, bool bf16, cudaStream_t stream);
cudaError_t launch_swiglu_bwd(const void* dy, const void* g, const void* u, void* dg, void* du, long long n, bool bf16,
                              cudaStream_t stream);
// out = residual + dropout(y) (residual may be null: out = dropout(y)); keep pattern = f(seed, element index), p quantised to 1/256.
cudaError_t launch_dropout_add(const void* y, const void* residual, void* out, long long n, float p, unsigned long long seed,
                               bool bf16, cudaStream_t stream);
cudaError_t launch_cast_f32_to_bf16(const float* src, void* dst, long long n, cudaStream_t stream);

// ---- cross_entropy.cu ----
// Per-row loss/lse over `vocab` columns of a [rows, ld] logits matrix; targets < 0 are ignored.
// stats[0] += sum of row losses, stats[1] += number of valid rows (both fp32, caller zeroes them).
cudaError_t launch_ce_forward(const void* logits, long long ld, const long long* targets, float* row_lse,
                              float* stats, long long rows, int vocab, bool bf16, cudaStream_t stream);
// In place: logits <- (softmax - onehot) * (*grad_scale) * (1 / valid_count[0]); columns in [vocab, ld_valid)
// are zeroed so that a padded matrix can feed a GEMM.
cudaError_t launch_ce_backward(void* logits, long long ld, const long long* targets, const float* row_lse,
                               const float* valid_count, const float* grad_scale, long long rows, int vocab,
                               int padded_vocab, bool bf16, cudaStream_t stream);
cudaError_t launch_count_valid_targets(const long long* targets, long long n, float* out_count, cudaStream_t stream);

// ---- router_moe.cu ----
// Softmax over E experts, top-k (k <= 8) with optional renormalisation, and the batch statistics.
// sums[0..E) += per-expert probability sums, sums[E] += sum(lse^2), sums[E+1] += sum(entropy).
cudaError_t launch_router_forward(const float* logits, int T, int E, int K, bool normalize, float* weights, int* indices,
                                  float* row_lse, float* sums, float* balance, cudaStream_t stream);
cudaError_t launch_router_backward(const float* logits, const float* row_lse, const int* indices, const float* weights,
                                   const float* g_weights, const float* g_mean_prob, const float* g_zloss, int T, int E,
                                   int K, bool normalize, float* g_logits, cudaStream_t stream);

// Routing plan for grouped GEMMs.  Rows of every expert form a segment padded to a multiple of 128.
//   row_token[r]  : source token of sorted row r, or -1 for a padding row       (capacity rows)
//   token_rows[i] : sorted row of route i = t * K + k                            (T*K)
//   tile_group[j] : expert of 128-row tile j                                     (capacity / 128)
//   meta[0] = live 128-row tiles, meta[1] = live rows; group_rows[e] = first row of expert e (E + 1)
cudaError_t launch_moe_plan(const int* indices, int T, int K, int E, int capacity_rows, int* row_token, int* token_rows,
                            int* tile_group, int* group_rows, int* meta, int* workspace, cudaStream_t stream);
size_t moe_plan_workspace_ints(int T, int K, int E);

// x_sorted[r] = x[row_token[r]] (zeros for padding); only rows below meta[1] are written, plus zero fill
// up to `capacity_rows` when `zero_tail` is set.
// `tokens` = rows of x (the extent source indices are checked against in bounds-checking builds).
cudaError_t launch_moe_gather(const void* x, const int* row_token, void* x_sorted, int capacity_rows, int H,
                              const int* meta, int tokens, cudaStream_t stream);
// row_slot[r] = route (t * K + k) carried by sorted row r or -1; row_weight[r] = weights[route] (bf16 in, fp32 out) or 0
cudaError_t launch_moe_row_meta(const int* row_token, const int* token_rows, const void* weights, float* row_weight, int* row_slot,
                                int rows, int K, int tokens, cudaStream_t stream);
// out[t] = sum_k w[t,k] * y[token_rows[t,k]]   (w may be null -> unweighted sum)
cudaError_t launch_moe_combine(const void* y, const int* token_rows, const void* weights, void* out, int T, int K, int H,
                               int y_rows, cudaStream_t stream);
// Backward of combine: dys[r] = w * dout[token] ; dweights[t,k] = <dout[t], y[row]> (fp32)
cudaError_t launch_moe_combine_bwd(const void* dout, const void* y, const int* row_token, const int* token_rows,
                                   const void* weights, void* dys, float* dweights, int T, int K, int H,
                                   int capacity_rows, const int* meta, cudaStream_t stream);

// ---- embedding.cu: out[t] = W[ids[t]] (bf16 out; W fp32 or bf16) and dW[ids[t]] += dout[t] (fp32 reductions) ----
// Ids outside [0, V) are skipped and raise STATUS_BAD_ARGUMENT in `status` (may be null).
cudaError_t launch_embedding_fwd(const long long* ids, const void* w, bool w_bf16, void* out, long long T, int V, int H, int* status,
                                 cudaStream_t stream);
cudaError_t launch_embedding_bwd(const long long* ids, const void* dout, float* dw, long long T, int V, int H, int* status,
                                 cudaStream_t stream);

// ---- skinny_gemm.cu: router projection x[T, H] (bf16) x W[E, H] (fp32 or bf16), E in {4, 8, 16}, fp32 arithmetic ----
bool router_logits_supported(int E, int H);
cudaError_t launch_router_logits_fwd(const void* x, const void* w, bool w_bf16, float* out, int T, int E, int H, cudaStream_t stream);
// dx[T, H] (bf16) = g[T, E] W
cudaError_t launch_router_logits_dx(const float* g, const void* w, bool w_bf16, void* dx, int T, int E, int H, cudaStream_t stream);
// dw[E, H] (fp32) = g^T x.  `partial` (floats, size from router_logits_dw_plan) and `arrivals` (one zeroed counter per column pass;
// the kernel leaves them zeroed) are scratch; launches that share them must not overlap.
void router_logits_dw_plan(int E, int H, int* passes, int* ctas_per_pass, long long* partial_floats);
cudaError_t launch_router_logits_dw(const float* g, const void* x, float* dw, float* partial, unsigned* arrivals, int T, int E, int H,
                                    cudaStream_t stream);

// ---- optim.cu ----
struct AdamWArgs {
  float* param;          // fp32 master weights
  const float* grad;     // fp32 gradients
  float* exp_avg;
  float* exp_avg_sq;
  void* shadow_bf16;     // optional bf16 copy refreshed with the new weights
  long long n;
  float lr, beta1, beta2, eps, weight_decay;
  float bias_correction1, bias_correction2;   // 1 - beta^t
  const float* grad_scale;   // optional device scalar multiplied into every gradient (clip coefficient / world)
  float static_grad_scale;
};
cudaError_t launch_adamw(const AdamWArgs& args, cudaStream_t stream);
// sum of squares of a fp32 buffer accumulated into *out (fp32, caller zeroes)
cudaError_t launch_sumsq(const float* x, long long n, float* out, cudaStream_t stream);
// *coef = min(1, max_norm / (sqrt(*sumsq) + 1e-6)) * extra ; norm_out = sqrt(sumsq)
cudaError_t launch_clip_coef(const float* sumsq, float max_norm, float extra, float* coef, float* norm_out,
                             cudaStream_t stream);

}  // namespace mts
