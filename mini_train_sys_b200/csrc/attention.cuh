// FlashAttention for sm_100a, head_dim 64, bf16, self-attention (Sq == Sk), optional causal mask and
// dropout.  Implemented in attention.cu with tcgen05 MMAs (accumulators in tensor memory) and TMA
// loads through 4-D tensor maps, so q/k/v may be arbitrary [B, H, S, D] views with unit inner stride.
//
// Saved for backward: O and the natural-log row log-sum-exp `lse[B, H, S]` (no probabilities).
// Dropout is a stateless function of (seed, batch*head, query, key); `dropout_keep_mask` materialises
// the same pattern for tests.  The drop probability is quantised to p_eff = round(p * 256) / 256 and
// kept values are scaled by 1 / (1 - p_eff).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace mts {

struct StridedBHSD {
  void* ptr;
  long long sb, sh, ss;   // element strides of batch, head, sequence (inner stride is 1)
};

struct AttentionArgs {
  StridedBHSD q, k, v, o;      // bf16
  StridedBHSD d_o, dq, dk, dv; // bf16 (backward only)
  float* lse;                  // [B, H, S]
  float* delta;                // [B, H, S] rowsum(dO * O) (backward scratch)
  int B, H, S;
  int causal;
  float scale;                 // 1 / sqrt(D)
  float dropout_p;
  unsigned long long seed;
  int* status;
  cudaStream_t stream;
  // Backward only, optional: bf16 RoPE tables [>= S, 64] (two identical halves).  When set, dQ and dK are rotated back
  // (the gradient of the half-split rotation applied to q and k before the forward) in the epilogues that write them.
  const void* rope_cos = nullptr;
  const void* rope_sin = nullptr;
};

constexpr int kAttnHeadDim = 64;

cudaError_t launch_flash_fwd(const AttentionArgs& a);
cudaError_t launch_flash_bwd(const AttentionArgs& a);
// keep[b*h, q, k] as uint8 (1 = kept)
cudaError_t launch_dropout_keep_mask(unsigned char* keep, int BH, int S, float dropout_p, unsigned long long seed,
                                     cudaStream_t stream);
extern const char* g_attn_last_error;
#ifdef MTS_ATTN_TRACE
cudaError_t copy_attention_trace(long long* host, int n);   // clock64 phase stamps of CTA 0 (trace-attention build profile)
#endif

}  // namespace mts
