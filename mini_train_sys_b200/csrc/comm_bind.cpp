// Python bindings of the peer-memory collectives.  Peer pointers arrive as integer lists (one per rank)
// obtained from the symmetric-memory rendezvous; everything else is an ordinary CUDA tensor.
#include <ATen/cuda/CUDAContext.h>
#include <cmath>
#include <cstring>
#include <tuple>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "comm.cuh"

namespace {

using torch::Tensor;

cudaStream_t cur() { return at::cuda::getCurrentCUDAStream().stream(); }

mts::PeerPtrs to_ptrs(const std::vector<int64_t>& v) {
  TORCH_CHECK(!v.empty() && v.size() <= size_t(mts::kMaxPeers), "between 1 and ", mts::kMaxPeers, " peers are supported");
  mts::PeerPtrs out{};
  for (size_t i = 0; i < v.size(); ++i) {
    TORCH_CHECK(v[i] != 0 && (v[i] & 15) == 0, "peer pointers must be non-null and 16-byte aligned");
    out.p[i] = reinterpret_cast<void*>(v[i]);
  }
  return out;
}

void ok(cudaError_t e, const char* what) { TORCH_CHECK(e == cudaSuccess, what, " failed: ", cudaGetErrorString(e)); }

const unsigned* flags_ptr(const Tensor& flags, int64_t channel, int64_t world) {
  TORCH_CHECK(flags.is_cuda() && flags.scalar_type() == at::kInt && flags.is_contiguous(), "flags must be contiguous int32");
  TORCH_CHECK(channel >= 0 && (channel + 1) * world <= flags.numel(), "flag channel out of range");
  return reinterpret_cast<const unsigned*>(flags.data_ptr<int>());
}

void comm_signal(const std::vector<int64_t>& flag_bases, int64_t channel, int64_t rank, int64_t epoch, const Tensor& like) {
  c10::cuda::CUDAGuard guard(like.device());
  ok(mts::launch_signal(to_ptrs(flag_bases), int(channel), int(flag_bases.size()), int(rank), unsigned(epoch), cur()), "signal");
}

void comm_wait(const Tensor& flags, int64_t channel, int64_t world, int64_t epoch, double timeout_ms, Tensor status) {
  c10::cuda::CUDAGuard guard(flags.device());
  ok(mts::launch_wait(flags_ptr(flags, channel, world), int(channel), int(world), unsigned(epoch),
                      (unsigned long long)(timeout_ms * 1e6), status.data_ptr<int>(), cur()), "wait");
}

void comm_allgather(Tensor dst, const std::vector<int64_t>& shard_ptrs, int64_t shard_bytes, const Tensor& flags, int64_t channel,
                    int64_t epoch, double timeout_ms, Tensor status, int64_t max_ctas) {
  const int64_t world = int64_t(shard_ptrs.size());
  TORCH_CHECK(dst.is_cuda() && dst.is_contiguous() && dst.numel() * dst.element_size() >= shard_bytes * world, "dst too small");
  TORCH_CHECK(shard_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(dst.data_ptr()) & 15) == 0, "16-byte alignment required");
  c10::cuda::CUDAGuard guard(dst.device());
  ok(mts::launch_allgather_pull(dst.data_ptr(), to_ptrs(shard_ptrs), shard_bytes, int(world), flags_ptr(flags, channel, world),
                                int(channel), unsigned(epoch), (unsigned long long)(timeout_ms * 1e6), status.data_ptr<int>(),
                                int(max_ctas), cur()), "allgather");
}

void comm_reduce_scatter(Tensor out, const std::vector<int64_t>& buf_ptrs, int64_t multicast_ptr, int64_t slice_offset,
                         double scale, const c10::optional<Tensor>& sumsq, const Tensor& flags, int64_t channel, int64_t epoch,
                         double timeout_ms, Tensor status, int64_t max_ctas) {
  const int64_t world = int64_t(buf_ptrs.size());
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kFloat && out.is_contiguous(), "out must be contiguous fp32");
  TORCH_CHECK(out.numel() % 4 == 0 && slice_offset % 4 == 0 && (reinterpret_cast<uintptr_t>(out.data_ptr()) & 15) == 0,
              "reduce-scatter slices must be multiples of 4 floats and 16-byte aligned");
  float* sq = (sumsq.has_value() && sumsq->defined()) ? sumsq->data_ptr<float>() : nullptr;
  c10::cuda::CUDAGuard guard(out.device());
  ok(mts::launch_reduce_scatter(out.data_ptr<float>(), to_ptrs(buf_ptrs), reinterpret_cast<const float*>(multicast_ptr),
                                slice_offset, out.numel(), int(world), float(scale), sq, flags_ptr(flags, channel, world),
                                int(channel), unsigned(epoch), (unsigned long long)(timeout_ms * 1e6), status.data_ptr<int>(),
                                int(max_ctas), cur()), "reduce_scatter");
}

void comm_adamw_push(Tensor param, const Tensor& grad, Tensor exp_avg, Tensor exp_avg_sq, const std::vector<int64_t>& replica_ptrs,
                     int64_t replica_elem_offset, bool push_bf16, double lr, double beta1, double beta2, double eps,
                     double weight_decay, int64_t step, const c10::optional<Tensor>& grad_scale, double static_scale,
                     int64_t max_ctas, const c10::optional<Tensor>& status) {
  TORCH_CHECK(param.is_cuda() && param.scalar_type() == at::kFloat && param.is_contiguous() && param.numel() % 8 == 0,
              "param shard must be contiguous fp32 with a multiple of 8 elements");
  TORCH_CHECK(grad.scalar_type() == at::kFloat && grad.is_contiguous() && grad.numel() == param.numel() &&
                  exp_avg.numel() == param.numel() && exp_avg_sq.numel() == param.numel(), "state size mismatch");
  for (const void* ptr : {param.data_ptr(), grad.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr()})
    TORCH_CHECK((reinterpret_cast<uintptr_t>(ptr) & 15) == 0, "adamw buffers must be 16-byte aligned");
  TORCH_CHECK(replica_elem_offset % 8 == 0, "replica offset must be a multiple of 8 elements");
  c10::cuda::CUDAGuard guard(param.device());
  mts::AdamWArgs a{};
  a.param = param.data_ptr<float>(); a.grad = grad.data_ptr<float>();
  a.exp_avg = exp_avg.data_ptr<float>(); a.exp_avg_sq = exp_avg_sq.data_ptr<float>();
  a.shadow_bf16 = nullptr; a.n = param.numel();
  a.lr = float(lr); a.beta1 = float(beta1); a.beta2 = float(beta2); a.eps = float(eps); a.weight_decay = float(weight_decay);
  a.bias_correction1 = float(1.0 - std::pow(beta1, double(step)));
  a.bias_correction2 = float(1.0 - std::pow(beta2, double(step)));
  a.grad_scale = (grad_scale.has_value() && grad_scale->defined()) ? grad_scale->data_ptr<float>() : nullptr;
  a.static_grad_scale = float(static_scale);
  const int* status_ptr = (status.has_value() && status->defined()) ? status->data_ptr<int>() : nullptr;
  ok(mts::launch_adamw_push(a, to_ptrs(replica_ptrs), replica_elem_offset, int(replica_ptrs.size()), push_bf16, int(max_ctas),
                            status_ptr, cur()), "adamw_push");
}

// rows: [p, g, m, v, n, replica_offset, group, push_bf16, replica pointers...] (addresses as integers).  Returns the table as a
// device byte tensor and the total number of chunks.
std::tuple<Tensor, int64_t> comm_adamw_table(const std::vector<std::vector<int64_t>>& rows, const Tensor& like) {
  std::vector<mts::AdamWSegment> host(rows.size());
  int64_t chunks = 0;
  for (size_t i = 0; i < rows.size(); ++i) {
    const auto& r = rows[i];
    TORCH_CHECK(r.size() >= 9 && r.size() <= 8 + size_t(mts::kMaxPeers), "adamw table row: 8 fields + 1..16 replica pointers");
    mts::AdamWSegment sg{};
    sg.p = reinterpret_cast<float*>(r[0]); sg.g = reinterpret_cast<const float*>(r[1]);
    sg.m = reinterpret_cast<float*>(r[2]); sg.v = reinterpret_cast<float*>(r[3]);
    sg.n = r[4]; sg.replica_offset = r[5]; sg.group = int(r[6]); sg.push_bf16 = int(r[7]);
    TORCH_CHECK(sg.n > 0 && sg.n % 8 == 0 && sg.replica_offset % 8 == 0, "adamw table: runs must be multiples of 8 elements");
    for (int64_t a : {r[0], r[1], r[2], r[3]}) TORCH_CHECK(a != 0 && (a & 15) == 0, "adamw table: 16-byte aligned buffers");
    sg.world = int(r.size() - 8);
    for (int k = 0; k < sg.world; ++k) {
      TORCH_CHECK(r[8 + k] != 0 && (r[8 + k] & 15) == 0, "adamw table: replica pointers must be 16-byte aligned");
      sg.replicas[k] = reinterpret_cast<void*>(r[8 + k]);
    }
    sg.chunk_begin = chunks;
    chunks += (sg.n + mts::kAdamChunk - 1) / mts::kAdamChunk;
    host[i] = sg;
  }
  Tensor cpu = torch::empty({int64_t(host.size() * sizeof(mts::AdamWSegment))}, torch::dtype(torch::kUInt8));
  std::memcpy(cpu.data_ptr(), host.data(), host.size() * sizeof(mts::AdamWSegment));
  return {cpu.to(like.device()), chunks};
}

void comm_adamw_push_table(const Tensor& table, int64_t n_segs, int64_t total_chunks, double lr0, double lr1, double wd0, double wd1,
                           double beta1, double beta2, double eps, int64_t step, const c10::optional<Tensor>& grad_scale,
                           double static_scale, const c10::optional<Tensor>& status, int64_t max_ctas) {
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == at::kByte && table.is_contiguous() &&
                  table.numel() == n_segs * int64_t(sizeof(mts::AdamWSegment)), "adamw table has the wrong size");
  c10::cuda::CUDAGuard guard(table.device());
  const float* gs = (grad_scale.has_value() && grad_scale->defined()) ? grad_scale->data_ptr<float>() : nullptr;
  const int* st = (status.has_value() && status->defined()) ? status->data_ptr<int>() : nullptr;
  ok(mts::launch_adamw_push_table(reinterpret_cast<const mts::AdamWSegment*>(table.data_ptr()), int(n_segs), total_chunks, float(lr0),
                                  float(lr1), float(wd0), float(wd1), float(beta1), float(beta2), float(eps),
                                  float(1.0 - std::pow(beta1, double(step))), float(1.0 - std::pow(beta2, double(step))), gs,
                                  float(static_scale), st, int(max_ctas), cur()), "adamw_push_table");
}

void comm_norm_clip(const Tensor& local_sumsq, const std::vector<int64_t>& slot_ptrs, const std::vector<int64_t>& flag_bases,
                    const Tensor& flags, int64_t channel, int64_t rank, int64_t epoch, double timeout_ms, double max_norm,
                    double extra_scale, Tensor coef, Tensor norm, Tensor status) {
  const int64_t world = int64_t(slot_ptrs.size());
  TORCH_CHECK(flag_bases.size() == slot_ptrs.size(), "peer lists differ in length");
  c10::cuda::CUDAGuard guard(local_sumsq.device());
  ok(mts::launch_scalar_allreduce_clip(local_sumsq.data_ptr<float>(), to_ptrs(slot_ptrs), to_ptrs(flag_bases),
                                       flags_ptr(flags, channel, world), int(channel), int(world), int(rank), unsigned(epoch),
                                       (unsigned long long)(timeout_ms * 1e6), float(max_norm), float(extra_scale),
                                       coef.data_ptr<float>(), norm.data_ptr<float>(), status.data_ptr<int>(), cur()), "norm_clip");
}


// rows of `x` (bf16 [T, H]) go to the receive regions of the ranks that own their experts; see comm.cu for the layout
void ep_push_rows(const Tensor& x, const Tensor& route_token, const Tensor& route_dest, const Tensor& route_slot,
                  const c10::optional<Tensor>& route_expert, const c10::optional<Tensor>& route_scale,
                  const std::vector<int64_t>& recv_rows, const std::vector<int64_t>& recv_expert, const c10::optional<Tensor>& counts,
                  const std::vector<int64_t>& recv_counts, int64_t src_rank, int64_t cap_rows, int64_t max_ctas) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.is_contiguous() && x.size(1) % 8 == 0,
              "x must be a contiguous bf16 matrix with a multiple of 8 columns");
  auto ints = [](const Tensor& t, const char* n) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous(), n, " must be contiguous int32");
    return t.data_ptr<int>();
  };
  const int64_t n = route_token.numel();
  TORCH_CHECK(route_dest.numel() == n && route_slot.numel() == n, "route arrays disagree");
  const int* expert = nullptr;
  if (route_expert.has_value() && route_expert->defined()) { TORCH_CHECK(route_expert->numel() == n, "route_expert size"); expert = ints(*route_expert, "route_expert"); }
  const float* scale = nullptr;
  if (route_scale.has_value() && route_scale->defined()) {
    TORCH_CHECK(route_scale->is_cuda() && route_scale->scalar_type() == at::kFloat && route_scale->is_contiguous() && route_scale->numel() == n,
                "route_scale must be contiguous fp32, one per route");
    scale = route_scale->data_ptr<float>();
  }
  const int* cnt = nullptr;
  if (counts.has_value() && counts->defined()) { TORCH_CHECK(counts->numel() >= int64_t(recv_rows.size()), "counts size"); cnt = ints(*counts, "counts"); }
  c10::cuda::CUDAGuard guard(x.device());
  ok(mts::launch_ep_push_rows(x.data_ptr(), ints(route_token, "route_token"), ints(route_dest, "route_dest"), ints(route_slot, "route_slot"),
                              expert, scale, int(n), int(x.size(1)), to_ptrs(recv_rows), expert ? to_ptrs(recv_expert) : mts::PeerPtrs{},
                              cnt, cnt ? to_ptrs(recv_counts) : mts::PeerPtrs{}, int(recv_rows.size()), int(src_rank), int(cap_rows),
                              int(max_ctas), cur()), "ep_push_rows");
}

void ep_pull_combine(Tensor out, const Tensor& token_dest, const Tensor& token_slot, const c10::optional<Tensor>& weight,
                     const std::vector<int64_t>& rows, int64_t my_rank, int64_t cap_rows, const c10::optional<Tensor>& saved, int64_t max_ctas) {
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.dim() == 2 && out.is_contiguous() && out.size(1) % 8 == 0,
              "out must be a contiguous bf16 matrix with a multiple of 8 columns");
  TORCH_CHECK(token_dest.is_cuda() && token_dest.scalar_type() == at::kInt && token_dest.is_contiguous() && token_dest.dim() == 2 &&
                  token_dest.size(0) == out.size(0) && token_slot.sizes() == token_dest.sizes() && token_slot.scalar_type() == at::kInt &&
                  token_slot.is_contiguous(), "token_dest / token_slot must be contiguous int32 [T, K]");
  const float* w = nullptr;
  if (weight.has_value() && weight->defined()) {
    TORCH_CHECK(weight->is_cuda() && weight->scalar_type() == at::kFloat && weight->is_contiguous() && weight->sizes() == token_dest.sizes(),
                "weight must be contiguous fp32 [T, K]");
    w = weight->data_ptr<float>();
  }
  void* keep = nullptr;
  if (saved.has_value() && saved->defined()) {
    TORCH_CHECK(saved->scalar_type() == at::kBFloat16 && saved->is_contiguous() && saved->numel() == token_dest.numel() * out.size(1), "saved size");
    keep = saved->data_ptr();
  }
  c10::cuda::CUDAGuard guard(out.device());
  ok(mts::launch_ep_pull_combine(out.data_ptr(), token_dest.data_ptr<int>(), token_slot.data_ptr<int>(), w, int(out.size(0)),
                                 int(token_dest.size(1)), int(out.size(1)), to_ptrs(rows), int(my_rank), int(cap_rows), keep, int(max_ctas),
                                 cur()), "ep_pull_combine");
}

}  // namespace

void bind_comm(pybind11::module_& m) {
  m.def("ep_push_rows", &ep_push_rows);
  m.def("ep_pull_combine", &ep_pull_combine);
  m.def("comm_signal", &comm_signal);
  m.def("comm_wait", &comm_wait);
  m.def("comm_allgather", &comm_allgather);
  m.def("comm_reduce_scatter", &comm_reduce_scatter);
  m.def("comm_adamw_push", &comm_adamw_push);
  m.def("comm_adamw_table", &comm_adamw_table);
  m.def("comm_adamw_push_table", &comm_adamw_push_table);
  m.def("comm_norm_clip", &comm_norm_clip);
}
