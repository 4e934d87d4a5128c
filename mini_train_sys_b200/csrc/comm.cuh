// Peer-memory collectives for sm_100a (implemented in comm.cu): flag signalling with bounded waits,
// pull all-gather, pull / multimem reduce-scatter, AdamW fused with the push of the updated weights,
// and a scalar all-reduce that also produces the gradient-clipping coefficient.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "ops.cuh"

namespace mts {

constexpr int kMaxPeers = 16;

// One pointer per rank (peer-mapped addresses of the same symmetric allocation), passed by value.
struct PeerPtrs {
  void* p[kMaxPeers];
};

cudaError_t launch_signal(const PeerPtrs& flag_bases, int channel, int world, int rank, unsigned epoch, cudaStream_t stream);
cudaError_t launch_wait(const unsigned* my_flags, int channel, int world, unsigned epoch, unsigned long long timeout_ns,
                        int* status, cudaStream_t stream);
// `epoch == 0` skips the wait (single-rank use and tests of the copy itself).
cudaError_t launch_allgather_pull(void* dst, const PeerPtrs& shards, long long shard_bytes, int world, const unsigned* my_flags,
                                  int channel, unsigned epoch, unsigned long long timeout_ns, int* status, int max_ctas,
                                  cudaStream_t stream);
// out[i] = scale * sum_r bufs[r][slice_offset + i]; *sumsq += sum(out^2).  With `multicast_base` the sum is a
// multimem.ld_reduce on the NVLS multicast mapping of the same buffers.
cudaError_t launch_reduce_scatter(float* out, const PeerPtrs& bufs, const float* multicast_base, long long slice_offset,
                                  long long n, int world, float scale, float* sumsq, const unsigned* my_flags, int channel,
                                  unsigned epoch, unsigned long long timeout_ns, int* status, int max_ctas, cudaStream_t stream);
// `status` (optional): the device's status word; when it is non-zero at launch the kernel changes nothing.
cudaError_t launch_adamw_push(const AdamWArgs& args, const PeerPtrs& replicas, long long replica_elem_offset, int world,
                              bool push_bf16, int max_ctas, const int* status, cudaStream_t stream);
// One row of the table behind launch_adamw_push_table: a run of a unit's local shard with one weight-decay group.
constexpr int kAdamChunk = 2048;   // elements per CTA pass (256 threads x 8)
struct AdamWSegment {
  float* p; const float* g; float* m; float* v;   // start of the run in the fp32 shard buffers
  long long n;                // elements, a multiple of 8
  long long chunk_begin;      // number of chunks in all earlier rows
  long long replica_offset;   // element offset of the run inside every replica
  void* replicas[kMaxPeers];  // low-precision destinations (the rank's own shard buffer, or every peer's replica)
  int world;                  // how many of them
  int group;                  // 0: decayed parameters (lr0, wd0), 1: the rest (lr1, wd1)
  int push_bf16;
  int reserved;
};
cudaError_t launch_adamw_push_table(const AdamWSegment* segs, int n_segs, long long total_chunks, float lr0, float lr1, float wd0,
                                    float wd1, float beta1, float beta2, float eps, float bc1, float bc2, const float* grad_scale,
                                    float static_scale, const int* status, int max_ctas, cudaStream_t stream);
cudaError_t launch_scalar_allreduce_clip(const float* local_value, const PeerPtrs& slots, const PeerPtrs& flag_bases,
                                         const unsigned* my_flags, int channel, int world, int rank, unsigned epoch,
                                         unsigned long long timeout_ns, float max_norm, float extra_scale, float* coef_out,
                                         float* norm_out, int* status, cudaStream_t stream);

// Expert-parallel exchange over peer memory (see comm.cu): rows are stored straight into the owning rank's receive regions, results
// are read back through the peers' mappings and combined.  `counts` (optional, [world]) is posted to every peer's `recv_counts[src]`.
cudaError_t launch_ep_push_rows(const void* x, const int* route_token, const int* route_dest, const int* route_slot,
                                const int* route_expert, const float* route_scale, int n_routes, int H, const PeerPtrs& recv_rows,
                                const PeerPtrs& recv_expert, const int* counts, const PeerPtrs& recv_counts, int world, int src_rank,
                                int cap_rows, int max_ctas, cudaStream_t stream);
cudaError_t launch_ep_pull_combine(void* out, const int* token_dest, const int* token_slot, const float* weight, int T, int K, int H,
                                   const PeerPtrs& rows, int my_rank, int cap_rows, void* saved, int max_ctas, cudaStream_t stream);

}  // namespace mts
