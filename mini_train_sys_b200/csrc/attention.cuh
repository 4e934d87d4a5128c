// FlashAttention kernels for sm_100a (implemented in attention.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace mts {

struct AttentionArgs {
  // q, k, v, o: bf16 [B, H, S, D] addressed through element strides (innermost stride 1)
  const void* q; const void* k; const void* v; void* o;
  long long q_sb, q_sh, q_ss, k_sb, k_sh, k_ss, v_sb, v_sh, v_ss, o_sb, o_sh, o_ss;
  float* lse;            // [B, H, S] natural-log sum-exp of the scaled scores
  int B, H, S, D;
  int causal;
  float scale;
  float dropout_p;
  unsigned long long seed;
  int* status;
  cudaStream_t stream;
};

}  // namespace mts
