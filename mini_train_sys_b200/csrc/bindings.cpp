// Python bindings: validate tensors, pick the current CUDA stream, call the raw launchers.
// Every check that could otherwise become a device fault (dtype, contiguity, alignment, extents)
// happens here, before anything is launched.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "attention.cuh"
#include "debug_bounds.cuh"
#include "comm.cuh"
#include "gemm_sm100.cuh"
#include "ops.cuh"

namespace mts {
namespace dbg {
namespace {
std::vector<Collector>& collectors() {
  static std::vector<Collector> list;      // built on first use: registration happens during static initialisation
  return list;
}
}  // namespace
void register_bounds_collector(Collector fn) { collectors().push_back(fn); }
}  // namespace dbg
}  // namespace mts

namespace {

using torch::Tensor;

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_launch(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, what, " failed: ", cudaGetErrorString(e));
}

bool is_bf16(const Tensor& t) { return t.scalar_type() == at::kBFloat16; }

void check_act(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kFloat, name, " must be bf16 or fp32");
}

void check_rowmajor_2d(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 2, name, " must be a 2-D CUDA tensor");
  TORCH_CHECK(t.stride(1) == 1, name, " must have a contiguous last dimension");
}

// One status word per device, zeroed at creation; kernels raise it with atomicMax.
Tensor& status_word(int device) {
  static std::vector<Tensor> words(64);
  TORCH_CHECK(device >= 0 && device < 64, "unexpected device index");
  if (!words[device].defined())
    words[device] = torch::zeros({4}, torch::dtype(torch::kInt32).device(torch::kCUDA, device));
  return words[device];
}

// ---------------- embedding ----------------
void check_embedding(const Tensor& ids, int64_t H) {
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous(), "ids must be contiguous int64 on the device");
  TORCH_CHECK(H % 8 == 0, "embedding width must be a multiple of 8");
}

Tensor embedding_fwd(const Tensor& ids, const Tensor& w) {
  TORCH_CHECK(w.is_cuda() && w.dim() == 2 && w.is_contiguous() && (w.scalar_type() == at::kFloat || is_bf16(w)),
              "embedding weight must be contiguous fp32 or bf16 [V, H]");
  check_embedding(ids, w.size(1));
  TORCH_CHECK((reinterpret_cast<uintptr_t>(w.data_ptr()) & 15) == 0, "embedding weight must be 16-byte aligned");
  c10::cuda::CUDAGuard guard(w.device());
  auto shape = ids.sizes().vec();
  shape.push_back(w.size(1));
  Tensor out = torch::empty(shape, w.options().dtype(torch::kBFloat16));
  check_launch(mts::launch_embedding_fwd(reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()), w.data_ptr(), is_bf16(w),
                                         out.data_ptr(), ids.numel(), int(w.size(0)), int(w.size(1)),
                                         status_word(w.get_device()).data_ptr<int>(), cur_stream()), "embedding_fwd");
  return out;
}

// dw (fp32 [V, H], contiguous) += scatter of dout's rows; the caller decides whether dw starts at zero.
void embedding_bwd(const Tensor& ids, const Tensor& dout, Tensor dw) {
  TORCH_CHECK(dw.is_cuda() && dw.dim() == 2 && dw.is_contiguous() && dw.scalar_type() == at::kFloat, "dw must be contiguous fp32 [V, H]");
  check_embedding(ids, dw.size(1));
  TORCH_CHECK(dout.is_cuda() && is_bf16(dout) && dout.is_contiguous() && dout.numel() == ids.numel() * dw.size(1),
              "dout must be contiguous bf16 with one row per id");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(dw.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(dout.data_ptr()) & 15) == 0,
              "embedding gradient buffers must be 16-byte aligned");
  c10::cuda::CUDAGuard guard(dw.device());
  check_launch(mts::launch_embedding_bwd(reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()), dout.data_ptr(),
                                         dw.data_ptr<float>(), ids.numel(), int(dw.size(0)), int(dw.size(1)),
                                         status_word(dw.get_device()).data_ptr<int>(), cur_stream()), "embedding_bwd");
}

// ---------------- router projection (skinny GEMM) ----------------
void check_router_operands(const Tensor& x, const Tensor& w) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.is_contiguous(), "x must be contiguous bf16 [T, H]");
  TORCH_CHECK(w.is_cuda() && w.dim() == 2 && w.is_contiguous() && w.size(1) == x.size(1) &&
                  (w.scalar_type() == at::kFloat || w.scalar_type() == at::kBFloat16), "w must be contiguous fp32 or bf16 [E, H]");
  TORCH_CHECK(mts::router_logits_supported(int(w.size(0)), int(w.size(1))), "router projection: E must be 4, 8 or 16 and H a multiple of 8");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(w.data_ptr()) & 15) == 0,
              "router projection operands must be 16-byte aligned");
}

bool router_logits_ok(int64_t experts, int64_t hidden) { return mts::router_logits_supported(int(experts), int(hidden)); }

Tensor router_logits_fwd(const Tensor& x, const Tensor& w) {
  check_router_operands(x, w);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = torch::empty({x.size(0), w.size(0)}, x.options().dtype(torch::kFloat));
  check_launch(mts::launch_router_logits_fwd(x.data_ptr(), w.data_ptr(), is_bf16(w), out.data_ptr<float>(), int(x.size(0)),
                                             int(w.size(0)), int(w.size(1)), cur_stream()), "router_logits_fwd");
  return out;
}

// g: fp32 [T, E] gradient of the logits.  Returns (dx bf16 [T, H] or undefined, dw fp32 [E, H] or undefined).
std::vector<Tensor> router_logits_bwd(const Tensor& g, const Tensor& x, const Tensor& w, bool need_dx, bool need_dw) {
  check_router_operands(x, w);
  TORCH_CHECK(g.is_cuda() && g.scalar_type() == at::kFloat && g.is_contiguous() && g.dim() == 2 && g.size(0) == x.size(0) &&
                  g.size(1) == w.size(0), "g must be contiguous fp32 [T, E]");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor dx, dw;
  const int T = int(x.size(0)), E = int(w.size(0)), H = int(w.size(1));
  if (need_dx && T > 0) {
    dx = torch::empty_like(x);
    check_launch(mts::launch_router_logits_dx(g.data_ptr<float>(), w.data_ptr(), is_bf16(w), dx.data_ptr(), T, E, H, cur_stream()),
                 "router_logits_dx");
  }
  if (need_dw) {
    dw = torch::empty({w.size(0), w.size(1)}, x.options().dtype(torch::kFloat));
    if (T == 0) {
      dw.zero_();
    } else {
      int passes = 0, gx = 0;
      long long floats = 0;
      mts::router_logits_dw_plan(E, H, &passes, &gx, &floats);
      Tensor partial = torch::empty({floats}, dw.options());
      // one counter array per device, zeroed once: the kernel resets what it used (launches on one stream are ordered)
      static std::vector<Tensor> counters(64);
      Tensor& arrivals = counters[x.get_device()];
      if (!arrivals.defined()) arrivals = torch::zeros({64}, x.options().dtype(torch::kInt));
      TORCH_CHECK(passes <= 64, "router projection: too many column passes");
      check_launch(mts::launch_router_logits_dw(g.data_ptr<float>(), x.data_ptr(), dw.data_ptr<float>(), partial.data_ptr<float>(),
                                                reinterpret_cast<unsigned*>(arrivals.data_ptr<int>()), T, E, H, cur_stream()),
                   "router_logits_dw");
    }
  }
  return {dx, dw};
}

// ---------------- memory-bound ops ----------------
std::vector<Tensor> rmsnorm_fwd(const Tensor& x, const Tensor& w, double eps) {
  check_act(x, "x");
  TORCH_CHECK(x.is_contiguous(), "x must be contiguous");
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kFloat && w.is_contiguous(), "weight must be contiguous fp32");
  const int64_t H = x.size(-1);
  TORCH_CHECK(w.numel() == H && H % 8 == 0, "hidden size must match the weight and be a multiple of 8");
  const int64_t rows = x.numel() / H;
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty_like(x);
  Tensor rstd = torch::empty({rows}, x.options().dtype(torch::kFloat));
  check_launch(mts::launch_rmsnorm_fwd(x.data_ptr(), w.data_ptr<float>(), y.data_ptr(), rstd.data_ptr<float>(), rows, int(H),
                                       float(eps), is_bf16(x), cur_stream()), "rmsnorm_fwd");
  return {y, rstd};
}

// dres (optional): gradient of the residual branch with the shape of x; the result is dx + dres.
// dw_out (optional): fp32 [H] destination of the weight gradient (a slot of a flat gradient buffer); it is overwritten.
std::vector<Tensor> rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd, bool need_dw,
                                const c10::optional<Tensor>& dres, const c10::optional<Tensor>& dw_out) {
  check_act(x, "x");
  const bool fuse_res = dres.has_value() && dres->defined() && is_bf16(x);
  if (dres.has_value() && dres->defined())
    TORCH_CHECK(dres->scalar_type() == x.scalar_type() && dres->is_contiguous() && dres->numel() == x.numel() && dres->is_cuda(),
                "dres must match x");
  TORCH_CHECK(dy.scalar_type() == x.scalar_type() && dy.is_contiguous() && x.is_contiguous(), "dy/x mismatch");
  const int64_t H = x.size(-1);
  TORCH_CHECK(H % 8 == 0 && H <= 1024, "rmsnorm backward supports hidden sizes up to 1024 (multiple of 8)");
  const int64_t rows = x.numel() / H;
  c10::cuda::CUDAGuard guard(x.device());
  Tensor dx = torch::empty_like(x);
  Tensor dw;
  if (need_dw && dw_out.has_value() && dw_out->defined()) {
    TORCH_CHECK(dw_out->is_cuda() && dw_out->scalar_type() == at::kFloat && dw_out->is_contiguous() && dw_out->numel() == H,
                "dw_out must be a contiguous fp32 CUDA tensor of H elements");
    dw = *dw_out;
    dw.zero_();
  } else if (need_dw) {
    dw = torch::zeros({H}, x.options().dtype(torch::kFloat));
  }
  check_launch(mts::launch_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr<float>(), rstd.data_ptr<float>(),
                                       fuse_res ? dres->data_ptr() : nullptr, dx.data_ptr(),
                                       need_dw ? dw.data_ptr<float>() : nullptr, rows, int(H), is_bf16(x), cur_stream()),
               "rmsnorm_bwd");
  if (dres.has_value() && dres->defined() && !fuse_res) dx.add_(*dres);
  return {dx, dw};
}

// x: [B, Hh, S, D] view (any strides, unit inner stride) -> contiguous [B, Hh, S, D], or into `out`
// (same shape, any 16-byte aligned strides) when one is given.
Tensor rope(const Tensor& x, const Tensor& cosv, const Tensor& sinv, bool backward, const c10::optional<Tensor>& out_opt) {
  check_act(x, "x");
  TORCH_CHECK(x.dim() == 4 && x.stride(3) == 1, "rope expects [B, H, S, D] with a contiguous last dimension");
  const int64_t B = x.size(0), Hh = x.size(1), S = x.size(2), D = x.size(3);
  TORCH_CHECK(D % 16 == 0, "head_dim must be a multiple of 16");
  TORCH_CHECK(cosv.scalar_type() == x.scalar_type() && sinv.scalar_type() == x.scalar_type(), "cos/sin dtype mismatch");
  TORCH_CHECK(cosv.is_contiguous() && sinv.is_contiguous() && cosv.size(0) >= S && cosv.size(1) == D, "bad cos/sin tables");
  const int64_t vec = is_bf16(x) ? 8 : 4;
  auto aligned = [vec](const Tensor& t) {
    return t.stride(0) % vec == 0 && t.stride(1) % vec == 0 && t.stride(2) % vec == 0 && t.stride(3) == 1 &&
           (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0;
  };
  TORCH_CHECK(aligned(x), "rope input must be 16-byte aligned in every row");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out;
  if (out_opt.has_value() && out_opt->defined()) {
    out = *out_opt;
    TORCH_CHECK(out.sizes() == x.sizes() && out.scalar_type() == x.scalar_type() && out.is_cuda() && aligned(out),
                "rope output must match the input shape/dtype and be 16-byte aligned in every row");
  } else {
    out = torch::empty({B, Hh, S, D}, x.options());
  }
  check_launch(mts::launch_rope(x.data_ptr(), out.data_ptr(), cosv.data_ptr(), sinv.data_ptr(), int(B), int(Hh), int(S), int(D),
                                x.stride(0), x.stride(1), x.stride(2), out.stride(0), out.stride(1), out.stride(2), backward,
                                is_bf16(x), cur_stream()), "rope");
  return out;
}

Tensor swiglu_fwd(const Tensor& g, const Tensor& u) {
  check_act(g, "gate");
  TORCH_CHECK(g.is_contiguous() && u.is_contiguous() && g.sizes() == u.sizes() && g.scalar_type() == u.scalar_type() &&
                  g.numel() % 8 == 0, "swiglu needs contiguous same-shaped inputs with numel % 8 == 0");
  c10::cuda::CUDAGuard guard(g.device());
  Tensor out = torch::empty_like(g);
  check_launch(mts::launch_swiglu_fwd(g.data_ptr(), u.data_ptr(), out.data_ptr(), g.numel(), is_bf16(g), cur_stream()), "swiglu_fwd");
  return out;
}

std::vector<Tensor> swiglu_bwd(const Tensor& dy, const Tensor& g, const Tensor& u) {
  TORCH_CHECK(dy.is_contiguous() && g.is_contiguous() && u.is_contiguous() && dy.scalar_type() == g.scalar_type(), "bad inputs");
  c10::cuda::CUDAGuard guard(g.device());
  Tensor dg = torch::empty_like(g), du = torch::empty_like(u);
  check_launch(mts::launch_swiglu_bwd(dy.data_ptr(), g.data_ptr(), u.data_ptr(), dg.data_ptr(), du.data_ptr(), g.numel(), is_bf16(g),
                                      cur_stream()), "swiglu_bwd");
  return {dg, du};
}

// out = residual + dropout(y); with an undefined residual: out = dropout(y) (this is also the backward of the y branch)
Tensor dropout_add(const Tensor& y, const c10::optional<Tensor>& residual, double p, int64_t seed) {
  check_act(y, "y");
  TORCH_CHECK(y.is_contiguous() && y.numel() % 8 == 0, "dropout_add needs a contiguous tensor with numel % 8 == 0");
  const bool has_res = residual.has_value() && residual->defined();
  if (has_res)
    TORCH_CHECK(residual->is_contiguous() && residual->sizes() == y.sizes() && residual->scalar_type() == y.scalar_type(),
                "residual must match y");
  c10::cuda::CUDAGuard guard(y.device());
  Tensor out = torch::empty_like(y);
  check_launch(mts::launch_dropout_add(y.data_ptr(), has_res ? residual->data_ptr() : nullptr, out.data_ptr(), y.numel(), float(p),
                                       static_cast<unsigned long long>(seed), is_bf16(y), cur_stream()), "dropout_add");
  return out;
}

Tensor cast_bf16(const Tensor& src) {
  TORCH_CHECK(src.is_cuda() && src.scalar_type() == at::kFloat && src.is_contiguous(), "cast_bf16 expects contiguous fp32");
  c10::cuda::CUDAGuard guard(src.device());
  Tensor dst = torch::empty(src.sizes(), src.options().dtype(torch::kBFloat16));
  check_launch(mts::launch_cast_f32_to_bf16(src.data_ptr<float>(), dst.data_ptr(), src.numel(), cur_stream()), "cast");
  return dst;
}

void cast_bf16_into(const Tensor& src, Tensor dst) {
  TORCH_CHECK(src.is_cuda() && src.scalar_type() == at::kFloat && src.is_contiguous(), "cast expects contiguous fp32");
  TORCH_CHECK(dst.is_cuda() && dst.scalar_type() == at::kBFloat16 && dst.is_contiguous() && dst.numel() == src.numel(), "bad dst");
  c10::cuda::CUDAGuard guard(src.device());
  check_launch(mts::launch_cast_f32_to_bf16(src.data_ptr<float>(), dst.data_ptr(), src.numel(), cur_stream()), "cast");
}

// ---------------- GEMM ----------------
void gemm(const Tensor& a, const Tensor& b, Tensor out, int64_t M, int64_t N, int64_t K, bool a_mn, bool b_mn, int64_t mode,
          int64_t epilogue, bool accumulate, bool atomic_out, const c10::optional<Tensor>& aux,
          const c10::optional<Tensor>& tile_group, const c10::optional<Tensor>& num_row_tiles,
          const c10::optional<Tensor>& group_rows, int64_t num_groups, int64_t b_group_stride_rows, int64_t out_group_stride,
          int64_t ldo, int64_t sm_limit, bool pair, int64_t k_splits, const c10::optional<Tensor>& gather_a,
          const c10::optional<Tensor>& gather_b, const c10::optional<Tensor>& row_scale, const c10::optional<Tensor>& row_slot,
          const c10::optional<Tensor>& row_grad) {
  check_rowmajor_2d(a, "a");
  check_rowmajor_2d(b, "b");
  TORCH_CHECK(is_bf16(a) && is_bf16(b), "GEMM operands must be bf16");
  TORCH_CHECK(a.stride(0) % 8 == 0 && b.stride(0) % 8 == 0, "operand leading dimensions must be multiples of 8");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(a.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(b.data_ptr()) & 15) == 0,
              "operands must be 16-byte aligned");
  TORCH_CHECK(out.is_cuda() && (out.scalar_type() == at::kBFloat16 || out.scalar_type() == at::kFloat), "bad output dtype");
  TORCH_CHECK(M > 0 && N > 0, "empty problem");
  c10::cuda::CUDAGuard guard(a.device());
  mts::GemmArgs g;
  g.a = a.data_ptr(); g.a_rows = a.size(0); g.a_cols = a.size(1); g.lda = a.stride(0);
  g.b = b.data_ptr(); g.b_rows = b.size(0); g.b_cols = b.size(1); g.ldb = b.stride(0);
  g.a_mn_major = a_mn; g.b_mn_major = b_mn;
  g.M = M; g.N = N; g.K = K; g.mode = int(mode); g.epilogue = int(epilogue);
  g.out = out.data_ptr(); g.ldo = ldo; g.out_fp32 = out.scalar_type() == at::kFloat;
  g.accumulate = accumulate; g.atomic_out = atomic_out;
  if (aux.has_value() && aux->defined()) {
    // storage for the saved pre-activations; the kernels lay it out in 32-row blocks of their own
    TORCH_CHECK(is_bf16(*aux) && aux->dim() == 2 && aux->is_contiguous() && aux->size(0) % 32 == 0 && aux->size(1) % 8 == 0,
                "aux must be a contiguous bf16 matrix with a multiple of 32 rows and of 8 columns");
    g.aux = aux->data_ptr(); g.ld_aux = aux->stride(0);
  }
  auto int_ptr = [](const c10::optional<Tensor>& t) -> const int* {
    if (!t.has_value() || !t->defined()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->is_contiguous(), "index tensors must be contiguous int32");
    return t->data_ptr<int>();
  };
  g.tile_group = int_ptr(tile_group); g.num_row_tiles = int_ptr(num_row_tiles); g.group_rows = int_ptr(group_rows);
  if (mode == mts::GEMM_GROUPED_M) {
    TORCH_CHECK(g.tile_group && g.num_row_tiles, "grouped-M needs tile_group and num_row_tiles");
    TORCH_CHECK(M % 128 == 0 && tile_group->numel() >= M / 128, "grouped-M capacity must be a multiple of 128");
    TORCH_CHECK(!a_mn, "grouped-M expects a K-major A operand");
    TORCH_CHECK(!pair || M % 256 == 0, "grouped-M on CTA pairs needs a row capacity that is a multiple of 256");
  }
  if (mode == mts::GEMM_GROUPED_K) {
    TORCH_CHECK(g.group_rows && group_rows->numel() >= num_groups + 1, "grouped-K needs group_rows[groups + 1]");
    TORCH_CHECK(a_mn && b_mn, "grouped-K expects MN-major operands");
  }
  TORCH_CHECK(k_splits >= 1 && k_splits <= 64, "k_splits out of range");
  TORCH_CHECK(k_splits == 1 || (mode == mts::GEMM_GROUPED_K && atomic_out), "k_splits needs grouped-K with atomic_out");
  g.k_splits = int(k_splits);
  g.num_groups = int(num_groups); g.b_group_stride_rows = b_group_stride_rows; g.out_group_stride = out_group_stride;
  // extents that the epilogue may touch must lie inside `out`
  const int64_t out_rows = (mode == mts::GEMM_GROUPED_K) ? M : M;
  const int64_t out_cols = epilogue == mts::EPI_SWIGLU ? N / 2 : (epilogue == mts::EPI_SWIGLU_BWD ? 2 * N : N);
  const int64_t groups_out = (mode == mts::GEMM_GROUPED_K && out_group_stride > 0) ? num_groups : 1;
  TORCH_CHECK(ldo >= out_cols, "output leading dimension too small");
  TORCH_CHECK((groups_out - 1) * out_group_stride + (out_rows - 1) * ldo + out_cols <= out.numel(), "output buffer too small");
  if (g.aux) {
    const int64_t aux_cols = epilogue == mts::EPI_SWIGLU ? N : 2 * N;
    TORCH_CHECK(aux->size(0) >= M && aux->size(1) >= aux_cols, "aux buffer too small");
  }
  g.gather_a = int_ptr(gather_a); g.gather_b = int_ptr(gather_b);
  if (g.gather_a != nullptr) {
    const int64_t need = (mode == mts::GEMM_GROUPED_M) ? M : 0;      // grouped-K: one entry per contraction row of the padded layout
    TORCH_CHECK(gather_a->numel() >= need && gather_a->numel() % 4 == 0 && (reinterpret_cast<uintptr_t>(g.gather_a) & 15) == 0,
                "gather_a must cover the padded rows, in multiples of 4, 16-byte aligned");
  }
  if (g.gather_b != nullptr)
    TORCH_CHECK(gather_b->numel() % 4 == 0 && (reinterpret_cast<uintptr_t>(g.gather_b) & 15) == 0, "gather_b must be 16-byte aligned");
  if (row_scale.has_value() && row_scale->defined()) {
    TORCH_CHECK(row_scale->is_cuda() && row_scale->scalar_type() == at::kFloat && row_scale->is_contiguous() && row_scale->numel() >= M,
                "row_scale must be contiguous fp32 with one entry per output row");
    g.row_scale = row_scale->data_ptr<float>();
  }
  if (row_slot.has_value() && row_slot->defined()) {
    TORCH_CHECK(row_grad.has_value() && row_grad->defined() && row_grad->is_cuda() && row_grad->scalar_type() == at::kFloat &&
                    row_grad->is_contiguous(), "row_slot needs a contiguous fp32 row_grad");
    TORCH_CHECK(row_slot->numel() >= M, "row_slot must have one entry per output row");
    g.row_slot = int_ptr(row_slot);
    g.row_grad = row_grad->data_ptr<float>();
  }
  g.status = status_word(a.get_device()).data_ptr<int>();
  g.sm_limit = int(sm_limit);
  g.pair = pair ? 1 : 0;
  g.stream = cur_stream();
  const cudaError_t gemm_err = mts::launch_gemm_sm100(g);
  TORCH_CHECK(gemm_err == cudaSuccess, "tcgen05 gemm failed: ", cudaGetErrorString(gemm_err), " (", mts::g_last_error, ")");
}

// ---------------- cross entropy ----------------
void ce_forward(const Tensor& logits, const Tensor& targets, Tensor row_lse, Tensor stats, int64_t vocab) {
  check_rowmajor_2d(logits, "logits");
  check_act(logits, "logits");
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kLong && targets.is_contiguous() && targets.numel() == logits.size(0),
              "targets must be contiguous int64 with one entry per row");
  TORCH_CHECK(vocab <= logits.size(1) && row_lse.numel() >= logits.size(0) && stats.numel() >= 2, "bad ce buffers");
  TORCH_CHECK(row_lse.scalar_type() == at::kFloat && stats.scalar_type() == at::kFloat, "lse/stats must be fp32");
  c10::cuda::CUDAGuard guard(logits.device());
  check_launch(mts::launch_ce_forward(logits.data_ptr(), logits.stride(0), reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()), row_lse.data_ptr<float>(),
                                      stats.data_ptr<float>(), logits.size(0), int(vocab), is_bf16(logits), cur_stream()), "ce_forward");
}

void ce_backward(Tensor logits, const Tensor& targets, const Tensor& row_lse, const Tensor& valid_count,
                 const c10::optional<Tensor>& grad_scale, int64_t vocab) {
  check_rowmajor_2d(logits, "logits");
  check_act(logits, "logits");
  TORCH_CHECK(targets.scalar_type() == at::kLong && targets.is_contiguous() && targets.numel() == logits.size(0), "bad targets");
  c10::cuda::CUDAGuard guard(logits.device());
  const float* gs = (grad_scale.has_value() && grad_scale->defined()) ? grad_scale->data_ptr<float>() : nullptr;
  check_launch(mts::launch_ce_backward(logits.data_ptr(), logits.stride(0), reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()), row_lse.data_ptr<float>(),
                                       valid_count.data_ptr<float>(), gs, logits.size(0), int(vocab), int(logits.size(1)),
                                       is_bf16(logits), cur_stream()), "ce_backward");
}

void count_valid(const Tensor& targets, Tensor out) {
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kLong && targets.is_contiguous(), "bad targets");
  c10::cuda::CUDAGuard guard(targets.device());
  check_launch(mts::launch_count_valid_targets(reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()), targets.numel(), out.data_ptr<float>(), cur_stream()), "count_valid");
}

// ---------------- router / MoE ----------------
std::vector<Tensor> router_forward(const Tensor& logits, int64_t K, bool normalize) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.scalar_type() == at::kFloat && logits.is_contiguous(),
              "router logits must be a contiguous 2-D fp32 CUDA tensor");
  const int64_t T = logits.size(0), E = logits.size(1);
  TORCH_CHECK(E <= 64 && K <= 8 && K <= E && T > 0, "router supports up to 64 experts and top-8");
  c10::cuda::CUDAGuard guard(logits.device());
  auto f32 = logits.options();
  Tensor w = torch::empty({T, K}, f32), idx = torch::empty({T, K}, f32.dtype(torch::kInt32));
  // sums: [E] probability mass, sum lse^2, sum entropy, [E] routes per expert; balance: 5 load-balance figures + [E] load fractions
  Tensor lse = torch::empty({T}, f32), sums = torch::zeros({2 * E + 2}, f32), balance = torch::empty({5 + E}, f32);
  check_launch(mts::launch_router_forward(logits.data_ptr<float>(), int(T), int(E), int(K), normalize, w.data_ptr<float>(),
                                          idx.data_ptr<int>(), lse.data_ptr<float>(), sums.data_ptr<float>(),
                                          balance.data_ptr<float>(), cur_stream()), "router_forward");
  return {w, idx, lse, sums, balance};
}

Tensor router_backward(const Tensor& logits, const Tensor& lse, const Tensor& idx, const Tensor& w,
                       const c10::optional<Tensor>& g_w, const c10::optional<Tensor>& g_mp, const c10::optional<Tensor>& g_z,
                       bool normalize) {
  const int64_t T = logits.size(0), E = logits.size(1), K = idx.size(1);
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor out = torch::empty_like(logits);
  auto opt = [](const c10::optional<Tensor>& t) -> const float* {
    if (!t.has_value() || !t->defined()) return nullptr;
    TORCH_CHECK(t->scalar_type() == at::kFloat && t->is_contiguous(), "router grads must be contiguous fp32");
    return t->data_ptr<float>();
  };
  check_launch(mts::launch_router_backward(logits.data_ptr<float>(), lse.data_ptr<float>(), idx.data_ptr<int>(), w.data_ptr<float>(),
                                           opt(g_w), opt(g_mp), opt(g_z), int(T), int(E), int(K), normalize, out.data_ptr<float>(),
                                           cur_stream()), "router_backward");
  return out;
}

int64_t moe_capacity_rows(int64_t T, int64_t K, int64_t E) { return ((T * K + E * 255) + 255) / 256 * 256; }   // segments padded to 256 rows

// returns row_token[cap], token_rows[T*K], tile_group[cap/128], group_rows[E+1], meta[4]
std::vector<Tensor> moe_plan(const Tensor& indices, int64_t E) {
  TORCH_CHECK(indices.is_cuda() && indices.dim() == 2 && indices.scalar_type() == at::kInt && indices.is_contiguous(),
              "expert indices must be contiguous int32 [T, K]");
  const int64_t T = indices.size(0), K = indices.size(1);
  const int64_t cap = moe_capacity_rows(T, K, E);
  c10::cuda::CUDAGuard guard(indices.device());
  auto i32 = indices.options();
  Tensor row_token = torch::empty({cap}, i32), token_rows = torch::empty({T * K}, i32);
  Tensor tile_group = torch::empty({cap / 128}, i32), group_rows = torch::empty({E + 1}, i32), meta = torch::zeros({4}, i32);
  Tensor ws = torch::empty({int64_t(mts::moe_plan_workspace_ints(int(T), int(K), int(E))) + 1}, i32);
  check_launch(mts::launch_moe_plan(indices.data_ptr<int>(), int(T), int(K), int(E), int(cap), row_token.data_ptr<int>(),
                                    token_rows.data_ptr<int>(), tile_group.data_ptr<int>(), group_rows.data_ptr<int>(),
                                    meta.data_ptr<int>(), ws.data_ptr<int>(), cur_stream()), "moe_plan");
  return {row_token, token_rows, tile_group, group_rows, meta};
}

void moe_gather(const Tensor& x, const Tensor& row_token, Tensor xs, const Tensor& meta) {
  TORCH_CHECK(is_bf16(x) && x.is_contiguous() && is_bf16(xs) && xs.is_contiguous() && x.size(1) == xs.size(1) && x.size(1) % 8 == 0, "bad gather tensors");
  TORCH_CHECK(xs.size(0) >= row_token.numel(), "sorted buffer smaller than the plan capacity");
  c10::cuda::CUDAGuard guard(x.device());
  check_launch(mts::launch_moe_gather(x.data_ptr(), row_token.data_ptr<int>(), xs.data_ptr(), int(row_token.numel()), int(x.size(1)),
                                      meta.data_ptr<int>(), int(x.size(0)), cur_stream()), "moe_gather");
}

std::vector<Tensor> moe_row_meta(const Tensor& row_token, const Tensor& token_rows, const Tensor& weights, int64_t K) {
  TORCH_CHECK(row_token.is_cuda() && row_token.scalar_type() == at::kInt && row_token.is_contiguous(), "row_token must be contiguous int32");
  TORCH_CHECK(token_rows.is_cuda() && token_rows.scalar_type() == at::kInt && token_rows.is_contiguous() && K > 0 &&
                  token_rows.numel() % K == 0, "token_rows must be contiguous int32 [T * K]");
  TORCH_CHECK(is_bf16(weights) && weights.is_contiguous() && weights.numel() == token_rows.numel(), "weights must be contiguous bf16 [T * K]");
  c10::cuda::CUDAGuard guard(row_token.device());
  Tensor row_weight = torch::empty({row_token.numel()}, row_token.options().dtype(torch::kFloat));
  Tensor row_slot = torch::empty({row_token.numel()}, row_token.options());
  check_launch(mts::launch_moe_row_meta(row_token.data_ptr<int>(), token_rows.data_ptr<int>(), weights.data_ptr(), row_weight.data_ptr<float>(),
                                        row_slot.data_ptr<int>(), int(row_token.numel()), int(K), int(token_rows.numel() / K), cur_stream()),
               "moe_row_meta");
  return {row_weight, row_slot};
}

void moe_combine(const Tensor& y, const Tensor& token_rows, const c10::optional<Tensor>& weights, Tensor out, int64_t K) {
  TORCH_CHECK(is_bf16(y) && y.is_contiguous() && is_bf16(out) && out.is_contiguous() && y.size(1) == out.size(1), "bad combine tensors");
  const void* w = nullptr;
  if (weights.has_value() && weights->defined()) {
    TORCH_CHECK(is_bf16(*weights) && weights->is_contiguous() && weights->numel() == out.size(0) * K, "weights must be bf16 [T, K]");
    w = weights->data_ptr();
  }
  TORCH_CHECK(token_rows.numel() == out.size(0) * K, "token_rows must have T*K entries");
  c10::cuda::CUDAGuard guard(y.device());
  check_launch(mts::launch_moe_combine(y.data_ptr(), token_rows.data_ptr<int>(), w, out.data_ptr(), int(out.size(0)), int(K),
                                       int(out.size(1)), int(y.size(0)), cur_stream()), "moe_combine");
}

void moe_combine_bwd(const Tensor& dout, const Tensor& y, const Tensor& row_token, const Tensor& token_rows, const Tensor& weights,
                     Tensor dys, Tensor dweights, const Tensor& meta, int64_t K) {
  TORCH_CHECK(is_bf16(dout) && dout.is_contiguous() && is_bf16(y) && y.is_contiguous() && is_bf16(dys) && dys.is_contiguous(), "bad tensors");
  TORCH_CHECK(is_bf16(weights) && weights.is_contiguous() && dweights.scalar_type() == at::kFloat && dweights.is_contiguous(), "bad weights");
  TORCH_CHECK(dys.size(0) >= row_token.numel() && y.size(0) >= row_token.numel(), "sorted buffers smaller than the plan capacity");
  c10::cuda::CUDAGuard guard(y.device());
  check_launch(mts::launch_moe_combine_bwd(dout.data_ptr(), y.data_ptr(), row_token.data_ptr<int>(), token_rows.data_ptr<int>(),
                                           weights.data_ptr(), dys.data_ptr(), dweights.data_ptr<float>(), int(dout.size(0)), int(K),
                                           int(dout.size(1)), int(row_token.numel()), meta.data_ptr<int>(), cur_stream()), "moe_combine_bwd");
}

// ---------------- optimizer ----------------
void adamw_step(Tensor param, const Tensor& grad, Tensor exp_avg, Tensor exp_avg_sq, const c10::optional<Tensor>& shadow, double lr,
                double beta1, double beta2, double eps, double weight_decay, int64_t step, const c10::optional<Tensor>& grad_scale,
                double static_scale) {
  TORCH_CHECK(param.is_cuda() && param.scalar_type() == at::kFloat && param.is_contiguous(), "param must be contiguous fp32");
  TORCH_CHECK(grad.scalar_type() == at::kFloat && grad.is_contiguous() && grad.numel() == param.numel(), "grad mismatch");
  TORCH_CHECK(exp_avg.numel() == param.numel() && exp_avg_sq.numel() == param.numel(), "state mismatch");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(param.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(grad.data_ptr()) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(exp_avg.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(exp_avg_sq.data_ptr()) & 15) == 0,
              "adamw buffers must be 16-byte aligned");
  c10::cuda::CUDAGuard guard(param.device());
  mts::AdamWArgs a{};
  a.param = param.data_ptr<float>(); a.grad = grad.data_ptr<float>();
  a.exp_avg = exp_avg.data_ptr<float>(); a.exp_avg_sq = exp_avg_sq.data_ptr<float>();
  a.shadow_bf16 = nullptr;
  if (shadow.has_value() && shadow->defined()) {
    TORCH_CHECK(is_bf16(*shadow) && shadow->is_contiguous() && shadow->numel() == param.numel() &&
                    (reinterpret_cast<uintptr_t>(shadow->data_ptr()) & 7) == 0, "bad bf16 shadow");
    a.shadow_bf16 = shadow->data_ptr();
  }
  a.n = param.numel(); a.lr = float(lr); a.beta1 = float(beta1); a.beta2 = float(beta2); a.eps = float(eps);
  a.weight_decay = float(weight_decay);
  a.bias_correction1 = float(1.0 - std::pow(beta1, double(step)));
  a.bias_correction2 = float(1.0 - std::pow(beta2, double(step)));
  a.grad_scale = (grad_scale.has_value() && grad_scale->defined()) ? grad_scale->data_ptr<float>() : nullptr;
  a.static_grad_scale = float(static_scale);
  check_launch(mts::launch_adamw(a, cur_stream()), "adamw");
}

void sumsq(const Tensor& x, Tensor out) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.is_contiguous() && out.scalar_type() == at::kFloat, "sumsq expects fp32");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0, "sumsq input must be 16-byte aligned");
  c10::cuda::CUDAGuard guard(x.device());
  check_launch(mts::launch_sumsq(x.data_ptr<float>(), x.numel(), out.data_ptr<float>(), cur_stream()), "sumsq");
}

void clip_coef(const Tensor& sumsq_in, double max_norm, double extra, Tensor coef, Tensor norm_out) {
  c10::cuda::CUDAGuard guard(sumsq_in.device());
  check_launch(mts::launch_clip_coef(sumsq_in.data_ptr<float>(), float(max_norm), float(extra), coef.data_ptr<float>(),
                                     norm_out.data_ptr<float>(), cur_stream()), "clip_coef");
}

// Out-of-range indices recorded by a bounds-checking build since the last reset: rows of
// (kernel id, block, thread, index, limit).  Always empty in a release build.  Synchronises the device.
std::vector<std::vector<int64_t>> debug_bounds_report(bool reset) {
  std::vector<std::vector<int64_t>> rows;
  cudaDeviceSynchronize();
  for (auto fn : mts::dbg::collectors()) {
    mts::dbg::BoundsRecord buf[mts::dbg::kRingSize];
    const int n = fn(buf, mts::dbg::kRingSize, reset);
    for (int i = 0; i < n; ++i) rows.push_back({buf[i].kernel, buf[i].block, buf[i].thread, buf[i].index, buf[i].limit});
  }
  return rows;
}

#ifdef MTS_ATTN_TRACE
// clock64 phase stamps of the first work item of CTA 0 (trace-attention build profile only)
Tensor attention_trace() {
  Tensor out = torch::zeros({8192}, torch::dtype(torch::kInt64));
  check_launch(mts::copy_attention_trace(reinterpret_cast<long long*>(out.data_ptr<int64_t>()), 8192), "attention trace");
  return out;
}
#endif

bool debug_bounds_enabled() {
#ifdef MTS_DEBUG_BOUNDS
  return true;
#else
  return false;
#endif
}

// The per-device StepContext block as an int32 tensor (a view of device memory owned by the extension; see ops.cuh for the
// layout: salt lo/hi, epoch_delta, dynamic_adam, then lr0, lr1, bias corrections as float bits).
Tensor step_context_tensor(int64_t device) {
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
  mts::StepContext* ctx = mts::step_context();
  TORCH_CHECK(ctx != nullptr, "could not allocate the step context");
  return torch::from_blob(ctx, {int64_t(sizeof(mts::StepContext) / 4)}, torch::dtype(torch::kInt32).device(torch::kCUDA, device));
}

void set_step_context(int64_t device, int64_t salt, int64_t epoch_delta, bool dynamic_adam, double lr0, double lr1, double bc1, double bc2) {
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
  check_launch(mts::launch_set_step_context(static_cast<unsigned long long>(salt), static_cast<unsigned int>(epoch_delta),
                                            dynamic_adam ? 1u : 0u, float(lr0), float(lr1), float(bc1), float(bc2), cur_stream()),
               "set_step_context");
}

int64_t launch_count() { return int64_t(mts::g_launch_count); }

Tensor status_tensor(int64_t device) { return status_word(int(device)); }

}  // namespace

void bind_attention(pybind11::module_& m);
void bind_comm(pybind11::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd, py::arg("dy"), py::arg("x"), py::arg("w"), py::arg("rstd"), py::arg("need_dw"),
        py::arg("dres") = py::none(), py::arg("dw_out") = py::none());
  m.def("rope", &rope);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("dropout_add", &dropout_add);
  m.def("cast_bf16", &cast_bf16);
  m.def("cast_bf16_into", &cast_bf16_into);
  m.def("gemm", &gemm);
  m.def("ce_forward", &ce_forward);
  m.def("ce_backward", &ce_backward);
  m.def("count_valid", &count_valid);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("router_logits_ok", &router_logits_ok);
  m.def("router_logits_fwd", &router_logits_fwd);
  m.def("router_logits_bwd", &router_logits_bwd);
  m.def("router_forward", &router_forward);
  m.def("router_backward", &router_backward);
  m.def("moe_capacity_rows", &moe_capacity_rows);
  m.def("moe_plan", &moe_plan);
  m.def("moe_gather", &moe_gather);
  m.def("moe_row_meta", &moe_row_meta);
  m.def("moe_combine", &moe_combine);
  m.def("moe_combine_bwd", &moe_combine_bwd);
  m.def("adamw_step", &adamw_step);
  m.def("sumsq", &sumsq);
  m.def("clip_coef", &clip_coef);
  m.def("launch_count", &launch_count);
  m.def("step_context_tensor", &step_context_tensor);
  m.def("set_step_context", &set_step_context);
  m.def("debug_bounds_report", &debug_bounds_report, py::arg("reset") = true);
  #ifdef MTS_ATTN_TRACE
  m.def("attention_trace", &attention_trace);
#endif
  m.def("debug_bounds_enabled", &debug_bounds_enabled);
  m.def("status_tensor", &status_tensor);
  bind_attention(m);
  bind_comm(m);
}
