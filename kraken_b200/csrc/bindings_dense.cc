// Bindings of the dense-parameter path (fused dense step, DCT compression).
#include <c10/cuda/CUDAStream.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "cuda/dense_kernels.h"
#include "cuda/mlp_gemm.h"

namespace py = pybind11;
using namespace kb;

namespace {

cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

void check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

template <typename T>
T* optr(const c10::optional<torch::Tensor>& t) {
  return (t.has_value() && t->defined() && t->numel() > 0) ? reinterpret_cast<T*>(t->data_ptr()) : nullptr;
}

cu::SymHost sym_from(const std::vector<uintptr_t>& bases, int rank) {
  cu::SymHost s{};
  TORCH_CHECK(bases.size() <= static_cast<size_t>(cu::kMaxWorldHost), "too many ranks");
  for (size_t i = 0; i < bases.size(); ++i) s.base[i] = reinterpret_cast<void*>(bases[i]);
  s.rank = rank;
  s.world = static_cast<int>(bases.size());
  return s;
}

}  // namespace

void bind_dense(py::module_& m) {
  py::class_<cu::DenseLayout>(m, "DenseLayout")
      .def(py::init<>())
      .def_readwrite("grad", &cu::DenseLayout::grad)
      .def_readwrite("param", &cu::DenseLayout::param)
      .def_readwrite("flag_grad", &cu::DenseLayout::flag_grad)
      .def_readwrite("flag_done", &cu::DenseLayout::flag_done)
      .def_readwrite("coo_cnt", &cu::DenseLayout::coo_cnt)
      .def_readwrite("coo_idx", &cu::DenseLayout::coo_idx)
      .def_readwrite("coo_val", &cu::DenseLayout::coo_val);
  m.attr("DENSE_CHUNK") = cu::kDenseChunk;
  m.attr("DENSE_CTRL_INTS") = cu::kDenseCtrlInts;

  m.def("dense_step",
        [](const std::vector<uintptr_t>& bases, int rank, const cu::DenseLayout& lay, const torch::Tensor& ctrl,
           int64_t n_pad, const c10::optional<torch::Tensor>& s0, const c10::optional<torch::Tensor>& s1,
           const c10::optional<torch::Tensor>& s2, const c10::optional<torch::Tensor>& acc,
           const torch::Tensor& chunk_table, const torch::Tensor& table_steps, const torch::Tensor& table_active,
           const OptimPOD& optim, const torch::Tensor& lr, float grad_scale, bool use_coo, uint32_t spin) {
          TORCH_CHECK(n_pad % (static_cast<int64_t>(bases.size()) * cu::kDenseChunk) == 0,
                      "n_pad must be a multiple of world * 256");
          TORCH_CHECK(chunk_table.numel() == n_pad / cu::kDenseChunk, "chunk_table has the wrong size");
          TORCH_CHECK(!use_coo || optr<float>(acc) != nullptr, "COO mode needs the accumulator");
          TORCH_CHECK(ctrl.is_cuda() && ctrl.scalar_type() == torch::kInt32 && ctrl.numel() >= cu::kDenseCtrlInts,
                      "ctrl must be an int32 CUDA tensor of at least ", cu::kDenseCtrlInts, " elements");
          cu::dense_step(sym_from(bases, rank), lay, reinterpret_cast<cu::DenseCtrl*>(ctrl.data_ptr()), n_pad,
                         optr<float>(s0), optr<float>(s1), optr<float>(s2), optr<float>(acc),
                         chunk_table.data_ptr<int>(), table_steps.data_ptr<int>(), table_active.data_ptr<uint8_t>(),
                         static_cast<int>(table_steps.numel()), optim, lr.data_ptr<float>(), grad_scale,
                         use_coo ? 1 : 0, spin, cur_stream());
          check_launch("dense_step");
        });
  m.def("dct_accumulate", [](const torch::Tensor& grad, const torch::Tensor& residual) {
    TORCH_CHECK(grad.numel() == residual.numel(), "grad and residual differ in size");
    cu::dct_accumulate(grad.data_ptr<float>(), residual.data_ptr<float>(), grad.numel(), cur_stream());
    check_launch("dct_accumulate");
  });
  m.def("dct_select_tau", [](const torch::Tensor& x, int64_t k, const torch::Tensor& hist,
                             const torch::Tensor& prefix_state, const torch::Tensor& tau) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kFloat32 && x.is_contiguous(), "x must be CUDA f32");
    TORCH_CHECK(k >= 1 && k <= x.numel(), "k out of range");
    TORCH_CHECK(hist.numel() >= 1024 && prefix_state.numel() >= 2, "radix scratch too small");
    cu::dct_select_tau(x.data_ptr<float>(), x.numel(), k, reinterpret_cast<uint32_t*>(hist.data_ptr()),
                       reinterpret_cast<uint32_t*>(prefix_state.data_ptr()), tau.data_ptr<float>(), cur_stream());
    check_launch("dct_select_tau");
  });
  m.def("dct_compact", [](const std::vector<uintptr_t>& bases, int rank, const cu::DenseLayout& lay, int64_t n_pad,
                          const torch::Tensor& residual, const torch::Tensor& tau, const torch::Tensor& chunk_table) {
    cu::dct_compact(sym_from(bases, rank), lay, n_pad, residual.data_ptr<float>(), tau.data_ptr<float>(),
                    chunk_table.data_ptr<int>(), cur_stream());
    check_launch("dct_compact");
  });
  m.def("dct_threshold_dense", [](const torch::Tensor& grad, const torch::Tensor& residual, const torch::Tensor& tau,
                                  const torch::Tensor& chunk_table) {
    cu::dct_threshold_dense(grad.data_ptr<float>(), residual.data_ptr<float>(), grad.numel(), tau.data_ptr<float>(),
                            chunk_table.data_ptr<int>(), cur_stream());
    check_launch("dct_threshold_dense");
  });

  // ---------------- tcgen05 Linear layers (bf16 in, fp32 accumulate)
  auto bf = [](const torch::Tensor& t) { return reinterpret_cast<const __nv_bfloat16*>(t.data_ptr()); };
  auto need_bf16 = [](const torch::Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16 && t.dim() == 2 && t.stride(1) == 1, name,
                " must be a 2-D CUDA bf16 tensor with unit inner stride");
  };
  m.def("linear_forward", [bf, need_bf16](const torch::Tensor& x, const torch::Tensor& w,
                                          const c10::optional<torch::Tensor>& bias, bool relu, const torch::Tensor& y,
                                          const torch::Tensor& status, const c10::optional<torch::Tensor>& mask_out) {
    need_bf16(x, "x");
    need_bf16(w, "w");
    need_bf16(y, "y");
    const int M = x.size(0), K = x.size(1), N = w.size(0);
    TORCH_CHECK(w.size(1) == K && y.size(0) == M && y.size(1) == N, "linear_forward: shape mismatch");
    uint16_t* mp = nullptr;
    int ldm = 0;
    if (mask_out.has_value()) {
      TORCH_CHECK(mask_out->is_cuda() && mask_out->scalar_type() == torch::kInt16 && mask_out->dim() == 2 &&
                      mask_out->stride(1) == 1 && mask_out->size(0) * 16 >= N && mask_out->size(1) >= M,
                  "mask_out must be a CUDA int16 tensor [ceil(N / 16), >= M]");
      mp = reinterpret_cast<uint16_t*>(mask_out->data_ptr());
      ldm = mask_out->stride(0);
    }
    const int rc = cu::linear_forward(bf(x), x.stride(0), bf(w), w.stride(0), optr<float>(bias),
                                      reinterpret_cast<__nv_bfloat16*>(y.data_ptr()), y.stride(0), M, N, K, relu, mp, ldm,
                                      status.data_ptr<int>(), cur_stream());
    TORCH_CHECK(rc == 0, "linear_forward: cannot encode the TMA descriptors (pitches must be multiples of 8)");
  }, py::arg("x"), py::arg("w"), py::arg("bias"), py::arg("relu"), py::arg("y"), py::arg("status"),
     py::arg("mask_out") = py::none());
  m.def("linear_dgrad", [bf, need_bf16](const torch::Tensor& dy, const torch::Tensor& wt,
                                        const c10::optional<torch::Tensor>& h, const torch::Tensor& dx,
                                        const torch::Tensor& status, const c10::optional<torch::Tensor>& mask) {
    need_bf16(dy, "dy");
    need_bf16(wt, "wt");
    need_bf16(dx, "dx");
    const int M = dy.size(0), N = dy.size(1), K = wt.size(0);
    TORCH_CHECK(wt.size(1) == N && dx.size(0) == M && dx.size(1) == K, "linear_dgrad: shape mismatch");
    const __nv_bfloat16* hp = nullptr;
    int ldh = 0;
    if (h.has_value()) {
      need_bf16(*h, "h");
      TORCH_CHECK(h->size(0) == M && h->size(1) == K, "linear_dgrad: mask shape mismatch");
      hp = bf(*h);
      ldh = h->stride(0);
    }
    const uint16_t* mp = nullptr;
    int ldm = 0;
    if (mask.has_value()) {
      TORCH_CHECK(mask->is_cuda() && mask->scalar_type() == torch::kInt16 && mask->dim() == 2 && mask->stride(1) == 1 &&
                      mask->size(0) * 16 >= K && mask->size(1) >= M,
                  "mask must be a CUDA int16 tensor [ceil(K / 16), >= M]");
      mp = reinterpret_cast<const uint16_t*>(mask->data_ptr());
      ldm = mask->stride(0);
    }
    const int rc = cu::linear_dgrad(bf(dy), dy.stride(0), bf(wt), wt.stride(0), hp, ldh, mp, ldm,
                                    reinterpret_cast<__nv_bfloat16*>(dx.data_ptr()), dx.stride(0), M, N, K,
                                    status.data_ptr<int>(), cur_stream());
    TORCH_CHECK(rc == 0, "linear_dgrad: cannot encode the TMA descriptors (pitches must be multiples of 8)");
  }, py::arg("dy"), py::arg("wt"), py::arg("h"), py::arg("dx"), py::arg("status"), py::arg("mask") = py::none());
  m.def("linear_wgrad", [bf, need_bf16](const torch::Tensor& dy, const torch::Tensor& x, const torch::Tensor& dw,
                                        const torch::Tensor& status) {
    need_bf16(dy, "dy");
    need_bf16(x, "x");
    TORCH_CHECK(dw.is_cuda() && dw.scalar_type() == torch::kFloat32 && dw.dim() == 2 && dw.stride(1) == 1,
                "dw must be a 2-D CUDA f32 tensor");
    const int M = dy.size(0), N = dy.size(1), K = x.size(1);
    TORCH_CHECK(x.size(0) == M && dw.size(0) == N && dw.size(1) == K, "linear_wgrad: shape mismatch");
    const int rc = cu::linear_wgrad(bf(dy), dy.stride(0), bf(x), x.stride(0), dw.data_ptr<float>(), dw.stride(0), M,
                                    N, K, status.data_ptr<int>(), cur_stream());
    TORCH_CHECK(rc == 0, "linear_wgrad: cannot encode the TMA descriptors (pitches must be multiples of 8)");
  });
  m.def("gemm_set_tuning", &cu::gemm_set_tuning, py::arg("variant") = 0, py::arg("n_tiles") = 0);
  m.def("colsum_bf16", [bf, need_bf16](const torch::Tensor& dy, const torch::Tensor& db) {
    need_bf16(dy, "dy");
    TORCH_CHECK(db.is_cuda() && db.scalar_type() == torch::kFloat32 && db.numel() >= dy.size(1), "db too small");
    cu::colsum_bf16(bf(dy), dy.stride(0), dy.size(0), dy.size(1), db.data_ptr<float>(), cur_stream());
    check_launch("colsum_bf16");
  });
  m.def("rowdot_forward", [bf, need_bf16](const torch::Tensor& x, const torch::Tensor& w,
                                          const c10::optional<torch::Tensor>& bias, const torch::Tensor& y,
                                          const c10::optional<torch::Tensor>& addend) {
    need_bf16(x, "x");
    TORCH_CHECK(w.is_cuda() && w.scalar_type() == torch::kFloat32 && w.is_contiguous() && w.numel() == x.size(1),
                "w must be a contiguous CUDA f32 vector of K elements");
    TORCH_CHECK(y.scalar_type() == torch::kFloat32 && y.numel() == x.size(0) && (x.stride(0) % 2) == 0, "bad y / pitch");
    TORCH_CHECK(!addend.has_value() || (addend->is_cuda() && addend->scalar_type() == torch::kFloat32 &&
                                        addend->is_contiguous() && addend->numel() == x.size(0)),
                "addend must be a contiguous CUDA f32 vector of M elements");
    cu::rowdot_forward(bf(x), x.stride(0), w.data_ptr<float>(), optr<float>(bias), optr<float>(addend), x.size(0),
                       x.size(1), y.data_ptr<float>(), cur_stream());
    check_launch("rowdot_forward");
  }, py::arg("x"), py::arg("w"), py::arg("bias"), py::arg("y"), py::arg("addend") = py::none());
  m.def("rowdot_backward", [bf, need_bf16](const torch::Tensor& x, const torch::Tensor& w, const torch::Tensor& dy,
                                           bool relu_mask, const c10::optional<torch::Tensor>& dx,
                                           const torch::Tensor& dw, const c10::optional<torch::Tensor>& db) {
    need_bf16(x, "x");
    TORCH_CHECK(dy.is_cuda() && dy.scalar_type() == torch::kFloat32 && dy.is_contiguous() && dy.numel() == x.size(0),
                "dy must be a contiguous CUDA f32 vector of M elements");
    TORCH_CHECK(dw.scalar_type() == torch::kFloat32 && dw.is_contiguous() && dw.numel() == x.size(1), "bad dw");
    __nv_bfloat16* dxp = nullptr;
    int lddx = 0;
    if (dx.has_value()) {
      need_bf16(*dx, "dx");
      TORCH_CHECK(dx->size(0) == x.size(0) && dx->size(1) == x.size(1) && (dx->stride(0) % 2) == 0, "bad dx");
      dxp = reinterpret_cast<__nv_bfloat16*>(dx->data_ptr());
      lddx = dx->stride(0);
    }
    cu::rowdot_backward(bf(x), x.stride(0), w.data_ptr<float>(), dy.data_ptr<float>(), x.size(0), x.size(1), relu_mask,
                        dxp, lddx, dw.data_ptr<float>(), optr<float>(db), cur_stream());
    check_launch("rowdot_backward");
  });
  m.def("cast_w_wt", [](const torch::Tensor& w) {
    TORCH_CHECK(w.is_cuda() && w.scalar_type() == torch::kFloat32 && w.dim() == 2 && w.is_contiguous(),
                "w must be a contiguous 2-D CUDA f32 tensor");
    const int N = w.size(0), K = w.size(1);
    torch::Tensor w16 = torch::empty({N, K}, w.options().dtype(torch::kBFloat16));
    torch::Tensor wt16 = torch::empty({K, N}, w.options().dtype(torch::kBFloat16));
    cu::cast_w_wt(w.data_ptr<float>(), N, K, reinterpret_cast<__nv_bfloat16*>(w16.data_ptr()),
                  reinterpret_cast<__nv_bfloat16*>(wt16.data_ptr()), cur_stream());
    check_launch("cast_w_wt");
    return std::make_pair(w16, wt16);
  });
}
