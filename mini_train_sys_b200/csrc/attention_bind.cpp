// Python bindings of the FlashAttention kernels: capability checks duplicated at the C++ boundary,
// output allocation ([B, S, H, D] storage returned as a [B, H, S, D] view), stream selection.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "attention.cuh"

namespace {

using torch::Tensor;

mts::StridedBHSD view_of(const Tensor& t) { return {t.data_ptr(), t.stride(0), t.stride(1), t.stride(2)}; }

void check_qkv(const Tensor& t, const char* name, int64_t B, int64_t H, int64_t S) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16, name, " must be a bf16 CUDA tensor");
  TORCH_CHECK(t.dim() == 4 && t.size(0) == B && t.size(1) == H && t.size(2) == S && t.size(3) == mts::kAttnHeadDim,
              name, " must be [B, H, S, 64]");
  TORCH_CHECK(t.stride(3) == 1, name, " must have a contiguous last dimension");
  TORCH_CHECK(t.stride(0) % 8 == 0 && t.stride(1) % 8 == 0 && t.stride(2) % 8 == 0 &&
                  (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, name, " rows must be 16-byte aligned");
}

mts::AttentionArgs base_args(const Tensor& q, const Tensor& k, const Tensor& v, bool causal, double dropout_p, int64_t seed) {
  const int64_t B = q.size(0), H = q.size(1), S = q.size(2);
  TORCH_CHECK(B > 0 && H > 0 && S > 0 && B * H <= 65535, "unsupported attention extents");
  TORCH_CHECK(dropout_p >= 0.0 && dropout_p < 1.0, "dropout_p must be in [0, 1)");
  check_qkv(q, "q", B, H, S);
  check_qkv(k, "k", B, H, S);
  check_qkv(v, "v", B, H, S);
  mts::AttentionArgs a{};
  a.q = view_of(q); a.k = view_of(k); a.v = view_of(v);
  a.B = int(B); a.H = int(H); a.S = int(S);
  a.causal = causal;
  a.scale = 1.0f / std::sqrt(float(mts::kAttnHeadDim));
  a.dropout_p = float(dropout_p);
  a.seed = static_cast<unsigned long long>(seed);
  a.status = nullptr;
  a.stream = at::cuda::getCurrentCUDAStream().stream();
  return a;
}

Tensor alloc_bhsd(const Tensor& like) {   // [B, S, H, D] storage viewed as [B, H, S, D]
  return torch::empty({like.size(0), like.size(2), like.size(1), like.size(3)}, like.options()).transpose(1, 2);
}

std::vector<Tensor> flash_fwd(const Tensor& q, const Tensor& k, const Tensor& v, bool causal, double dropout_p, int64_t seed,
                              const Tensor& status) {
  c10::cuda::CUDAGuard guard(q.device());
  mts::AttentionArgs a = base_args(q, k, v, causal, dropout_p, seed);
  Tensor o = alloc_bhsd(q);
  Tensor lse = torch::empty({q.size(0), q.size(1), q.size(2)}, q.options().dtype(torch::kFloat));
  a.o = view_of(o);
  a.lse = lse.data_ptr<float>();
  a.status = status.data_ptr<int>();
  const cudaError_t e = mts::launch_flash_fwd(a);
  TORCH_CHECK(e == cudaSuccess, "flash_fwd failed: ", cudaGetErrorString(e), " (", mts::g_attn_last_error, ")");
  return {o, lse};
}

std::vector<Tensor> flash_bwd(const Tensor& d_o, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o,
                              const Tensor& lse, bool causal, double dropout_p, int64_t seed, const Tensor& status,
                              const c10::optional<Tensor>& dq_out, const c10::optional<Tensor>& dk_out,
                              const c10::optional<Tensor>& dv_out, const c10::optional<Tensor>& rope_cos,
                              const c10::optional<Tensor>& rope_sin) {
  c10::cuda::CUDAGuard guard(q.device());
  mts::AttentionArgs a = base_args(q, k, v, causal, dropout_p, seed);
  if (rope_cos.has_value() && rope_cos->defined()) {
    // q and k were rotated before the forward: dQ / dK come back un-rotated from the kernels that produce them
    TORCH_CHECK(rope_sin.has_value() && rope_sin->defined(), "rope_cos needs rope_sin");
    for (const Tensor* t : {&*rope_cos, &*rope_sin})
      TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kBFloat16 && t->dim() == 2 && t->is_contiguous() &&
                  t->size(0) >= q.size(2) && t->size(1) == 64, "rope tables must be contiguous bf16 [>= S, 64]");
    a.rope_cos = rope_cos->data_ptr();
    a.rope_sin = rope_sin->data_ptr();
  }
  check_qkv(o, "o", q.size(0), q.size(1), q.size(2));
  check_qkv(d_o, "d_o", q.size(0), q.size(1), q.size(2));
  TORCH_CHECK(lse.is_cuda() && lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.numel() == q.size(0) * q.size(1) * q.size(2),
              "lse must be contiguous fp32 [B, H, S]");
  auto pick = [&](const c10::optional<Tensor>& given, const char* name) {
    if (given.has_value() && given->defined()) {
      check_qkv(*given, name, q.size(0), q.size(1), q.size(2));
      return *given;
    }
    return alloc_bhsd(q);
  };
  Tensor dq = pick(dq_out, "dq"), dk = pick(dk_out, "dk"), dv = pick(dv_out, "dv");
  Tensor delta = torch::empty_like(lse);
  a.o = view_of(o); a.d_o = view_of(d_o); a.dq = view_of(dq); a.dk = view_of(dk); a.dv = view_of(dv);
  a.lse = lse.data_ptr<float>();
  a.delta = delta.data_ptr<float>();
  a.status = status.data_ptr<int>();
  const cudaError_t e = mts::launch_flash_bwd(a);
  TORCH_CHECK(e == cudaSuccess, "flash_bwd failed: ", cudaGetErrorString(e), " (", mts::g_attn_last_error, ")");
  return {dq, dk, dv};
}

Tensor dropout_keep_mask(int64_t BH, int64_t S, double dropout_p, int64_t seed, const Tensor& like) {
  c10::cuda::CUDAGuard guard(like.device());
  Tensor keep = torch::empty({BH, S, S}, like.options().dtype(torch::kUInt8));
  const cudaError_t e = mts::launch_dropout_keep_mask(keep.data_ptr<unsigned char>(), int(BH), int(S), float(dropout_p),
                                                      static_cast<unsigned long long>(seed), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(e == cudaSuccess, "dropout_keep_mask failed: ", cudaGetErrorString(e));
  return keep;
}

}  // namespace

void bind_attention(pybind11::module_& m) {
  m.def("flash_fwd", &flash_fwd);
  m.def("flash_bwd", &flash_bwd, pybind11::arg("d_o"), pybind11::arg("q"), pybind11::arg("k"), pybind11::arg("v"), pybind11::arg("o"),
        pybind11::arg("lse"), pybind11::arg("causal"), pybind11::arg("dropout_p"), pybind11::arg("seed"), pybind11::arg("status"),
        pybind11::arg("dq_out") = pybind11::none(), pybind11::arg("dk_out") = pybind11::none(),
        pybind11::arg("dv_out") = pybind11::none(), pybind11::arg("rope_cos") = pybind11::none(),
        pybind11::arg("rope_sin") = pybind11::none());
  m.def("dropout_keep_mask", &dropout_keep_mask);
}
