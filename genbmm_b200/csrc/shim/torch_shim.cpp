// Thin PyTorch binding over the C ABI of libgenbmm_b200.so for the dense operators.
//
// It stands where the reference's pybind module does (matmul_cuda.cpp:65-172): CHECK_CUDA / CHECK_CONTIGUOUS
// with the same messages, outputs allocated here, then one call into the kernels.  Unlike the reference it
// sets a device guard for the tensors' device and launches on torch's current stream.  It also holds the four
// operators as C++ autograd functions (genmul.py:11-103 are Python ones), so that one call of
// genbmm_b200.logbmm costs one trip from Python instead of an autograd.Function written in Python plus three
// to six ctypes calls.  Everything numerical happens behind include/genbmm_b200.h; this file launches nothing
// itself.  The ctypes binding (genbmm_b200/_native.py) remains as the fallback when this module is not built.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime_api.h>
#include <torch/extension.h>

#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "genbmm_b200.h"

namespace {

using torch::Tensor;
using torch::autograd::AutogradContext;
using torch::autograd::variable_list;

void* stream_of(const Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

void check_status(int st, const char* what) {
  TORCH_CHECK(st == GBMM_OK, what, " failed: ", gbmm_status_string(st), " (status ", st, ")");
}

// matmul_cuda.cpp:65-67, same words
void check_input(const Tensor& x, const char* name) {
  TORCH_CHECK(x.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(x.is_contiguous(), name, " must be contiguous");
}

void check_pair(const Tensor& a, const Tensor& b) {
  check_input(a, "a");
  check_input(b, "b");
  TORCH_CHECK(a.dim() == 3 && b.dim() == 3 && a.size(0) == b.size(0) && a.size(2) == b.size(1),
              "expected a:(B,M,K) and b:(B,K,N), got ", a.sizes(), " and ", b.sizes());
  TORCH_CHECK(a.device() == b.device(), "a and b must be on the same device");
  TORCH_CHECK(a.scalar_type() == b.scalar_type(), "b must be ", a.scalar_type(), " (got ", b.scalar_type(), ")");
}

// half / bfloat16 are computed in float32; float32 and float64 as they are
Tensor widen(const Tensor& x, const char* name) {
  const auto t = x.scalar_type();
  if (t == torch::kFloat32 || t == torch::kFloat64) return x;
  if (t == torch::kFloat16 || t == torch::kBFloat16) return x.to(torch::kFloat32);
  TORCH_CHECK(false, name, ": dtype ", t, " is not supported");
  return x;
}

const char* env_or(const char* name, const char* fallback) {
  const char* v = std::getenv(name);
  return v ? v : fallback;
}

enum LogPath { PATH_EXACT = 0, PATH_FP32 = 1, PATH_TENSOR = 2 };

// Which kernels logbmm uses (genbmm_b200/genmul.py `_log_path` states the same rule for the Python binding).
LogPath log_path(int64_t M, int64_t K, int64_t N) {
  const char* mode = env_or("GENBMM_B200_LOGBMM", "auto");
  if (K == 0 || M == 0 || N == 0 || !std::strcmp(mode, "exact")) return PATH_EXACT;
  if (!std::strcmp(mode, "fp32") || !std::strcmp(mode, "fast")) return PATH_FP32;
  if (!std::strcmp(mode, "tensor")) return PATH_TENSOR;
  return M * K * N >= 128LL * 128 * 64 ? PATH_TENSOR : PATH_EXACT;
}

bool keep_factors(const Tensor& a, const Tensor& b) {
  const char* mode = env_or("GENBMM_B200_KEEP_FACTORS", "auto");
  if (!std::strcmp(mode, "0")) return false;
  if (!std::strcmp(mode, "1")) return true;
  const int64_t nbytes = 16 * (a.numel() + b.numel());
  if (nbytes <= (1LL << 30)) return true;
  size_t free_b = 0, total_b = 0;
  if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) return false;
  return (int64_t)free_b >= 4 * nbytes;
}

Tensor bytes(int64_t n, const Tensor& like) {
  return torch::empty({n < 256 ? 256 : n}, like.options().dtype(torch::kUInt8));
}

// ---- plain calls: what `_genbmm.forward` / `_genbmm.backward` are in the reference ------------------------

// -> [out, aux]; aux = maxes (mode 0, only if want_maxes) or the int32 indices
std::vector<Tensor> dense_forward(const Tensor& a, const Tensor& b, int64_t mode, const c10::optional<Tensor>& u_in,
                                  bool want_maxes) {
  check_pair(a, b);
  TORCH_CHECK(mode >= 0 && mode <= 3, "unknown mode ", mode);
  TORCH_CHECK(a.scalar_type() == torch::kFloat32 || a.scalar_type() == torch::kFloat64, "a must be float32 or float64");
  const c10::cuda::CUDAGuard guard(a.device());
  const int64_t B = a.size(0), M = a.size(1), K = a.size(2), N = b.size(2);
  Tensor out = torch::empty({B, M, N}, a.options());
  Tensor aux, u;
  if (mode == GBMM_MODE_LOG) {
    if (want_maxes) aux = torch::empty_like(out);
  } else {
    aux = torch::empty({B, M, N}, a.options().dtype(torch::kInt32));
  }
  if (mode == GBMM_MODE_SAMPLE) {
    u = u_in.has_value() && u_in->defined() ? *u_in : torch::rand({B, M, N}, a.options());
    check_input(u, "u");
    TORCH_CHECK(u.scalar_type() == a.scalar_type() && u.sizes() == out.sizes(), "u must have shape ", out.sizes());
  }
  void* aux_p = aux.defined() ? aux.data_ptr() : nullptr;
  if (a.scalar_type() == torch::kFloat64) {
    check_status(gbmm_dense_forward_f64((int)mode, a.data_ptr<double>(), b.data_ptr<double>(),
                                        u.defined() ? u.data_ptr<double>() : nullptr, out.data_ptr<double>(), aux_p, B,
                                        M, K, N, stream_of(a)),
                 "gbmm_dense_forward_f64");
    return {out, aux};
  }
  const int64_t nbytes = gbmm_dense_forward_workspace_bytes((int)mode, B, M, K, N);
  Tensor ws;
  if (nbytes > 0) ws = bytes(nbytes, a);
  check_status(gbmm_dense_forward_f32((int)mode, a.data_ptr<float>(), b.data_ptr<float>(),
                                      u.defined() ? u.data_ptr<float>() : nullptr, out.data_ptr<float>(), aux_p, B, M,
                                      K, N, ws.defined() ? ws.data_ptr() : nullptr, ws.defined() ? ws.numel() : 0,
                                      stream_of(a)),
               "gbmm_dense_forward_f32");
  return {out, aux};
}

// -> [grad_a, grad_b]; mode 0: part = the forward's out; modes 1-3: part = the int32 indices
std::vector<Tensor> dense_backward(const Tensor& a, const Tensor& b, const Tensor& grad, const Tensor& part_in,
                                   int64_t mode) {
  check_pair(a, b);
  check_input(grad, "grad_output");
  const c10::cuda::CUDAGuard guard(a.device());
  const int64_t B = a.size(0), M = a.size(1), K = a.size(2), N = b.size(2);
  TORCH_CHECK(grad.dim() == 3 && grad.size(0) == B && grad.size(1) == M && grad.size(2) == N &&
                  grad.scalar_type() == a.scalar_type(),
              "grad_output must have shape (", B, ", ", M, ", ", N, ") and a's dtype");
  Tensor part = part_in;
  if (mode != GBMM_MODE_LOG && part.scalar_type() != torch::kInt32) part = part.to(torch::kInt32);
  check_input(part, "part");
  TORCH_CHECK(part.sizes() == grad.sizes(), "part must have shape ", grad.sizes());
  Tensor ga = torch::empty_like(a), gb = torch::empty_like(b);
  const void* pf = mode == GBMM_MODE_LOG ? part.data_ptr() : nullptr;
  const void* ix = mode == GBMM_MODE_LOG ? nullptr : part.data_ptr();
  if (a.scalar_type() == torch::kFloat64) {
    check_status(gbmm_dense_backward_f64((int)mode, a.data_ptr<double>(), b.data_ptr<double>(), grad.data_ptr<double>(),
                                         static_cast<const double*>(pf), ix, ga.data_ptr<double>(),
                                         gb.data_ptr<double>(), B, M, K, N, stream_of(a)),
                 "gbmm_dense_backward_f64");
  } else {
    check_status(gbmm_dense_backward_f32((int)mode, a.data_ptr<float>(), b.data_ptr<float>(), grad.data_ptr<float>(),
                                         static_cast<const float*>(pf), ix, ga.data_ptr<float>(), gb.data_ptr<float>(),
                                         B, M, K, N, stream_of(a)),
                 "gbmm_dense_backward_f32");
  }
  return {ga, gb};
}

// -> [out, rowmax, colmax, flags, factors or undefined]
std::vector<Tensor> logbmm_fast_forward(const Tensor& a, const Tensor& b, bool tensor_cores, bool keep) {
  check_pair(a, b);
  TORCH_CHECK(a.scalar_type() == torch::kFloat32, "a must be float32");
  const c10::cuda::CUDAGuard guard(a.device());
  const int64_t B = a.size(0), M = a.size(1), K = a.size(2), N = b.size(2);
  Tensor out = torch::empty({B, M, N}, a.options());
  Tensor rowmax = torch::empty({B, M}, a.options()), colmax = torch::empty({B, N}, a.options());
  const int64_t nf = gbmm_logbmm_flag_count(B, M, N);
  Tensor flags = torch::empty({nf < 1 ? 1 : nf}, a.options().dtype(torch::kInt32));
  Tensor ws = bytes(tensor_cores ? gbmm_logbmm_tc_workspace_bytes(0, B, M, K, N)
                                 : gbmm_logbmm_workspace_bytes(0, B, M, K, N), a);
  auto fn = tensor_cores ? gbmm_logbmm_tc_forward_f32 : gbmm_logbmm_forward_f32;
  check_status(fn(a.data_ptr<float>(), b.data_ptr<float>(), out.data_ptr<float>(), rowmax.data_ptr<float>(),
                  colmax.data_ptr<float>(), flags.data_ptr<int32_t>(), ws.data_ptr(), ws.numel(), B, M, K, N,
                  stream_of(a)),
               "gbmm_logbmm_forward_f32");
  return {out, rowmax, colmax, flags, (tensor_cores && keep) ? ws : Tensor()};
}

std::vector<Tensor> logbmm_fast_backward(const Tensor& a, const Tensor& b, const Tensor& grad, const Tensor& out,
                                         const Tensor& rowmax, const Tensor& colmax, const Tensor& flags,
                                         bool tensor_cores, const Tensor& factors) {
  check_pair(a, b);
  check_input(grad, "grad_output");
  const c10::cuda::CUDAGuard guard(a.device());
  const int64_t B = a.size(0), M = a.size(1), K = a.size(2), N = b.size(2);
  TORCH_CHECK(grad.sizes() == out.sizes() && grad.scalar_type() == torch::kFloat32, "grad_output must have shape ",
              out.sizes());
  Tensor ga = torch::empty_like(a), gb = torch::empty_like(b);
  Tensor ws = bytes(tensor_cores ? gbmm_logbmm_tc_workspace_bytes(1, B, M, K, N)
                                 : gbmm_logbmm_workspace_bytes(1, B, M, K, N), a);
  int st;
  if (tensor_cores) {
    st = gbmm_logbmm_tc_backward_f32(a.data_ptr<float>(), b.data_ptr<float>(), grad.data_ptr<float>(),
                                     out.data_ptr<float>(), rowmax.data_ptr<float>(), colmax.data_ptr<float>(),
                                     flags.data_ptr<int32_t>(), ga.data_ptr<float>(), gb.data_ptr<float>(),
                                     factors.defined() ? factors.data_ptr() : nullptr, ws.data_ptr(), ws.numel(), B, M,
                                     K, N, stream_of(a));
  } else {
    st = gbmm_logbmm_backward_f32(a.data_ptr<float>(), b.data_ptr<float>(), grad.data_ptr<float>(),
                                  out.data_ptr<float>(), rowmax.data_ptr<float>(), colmax.data_ptr<float>(),
                                  flags.data_ptr<int32_t>(), ga.data_ptr<float>(), gb.data_ptr<float>(), ws.data_ptr(),
                                  ws.numel(), B, M, K, N, stream_of(a));
  }
  check_status(st, "gbmm_logbmm_backward_f32");
  return {ga, gb};
}

// ---- the operators as autograd functions ------------------------------------------------------------------

// First-order gradients of logbmm as a differentiable node (genmul.py:11-24): its backward is the second order.
struct LogMatMulBack : public torch::autograd::Function<LogMatMulBack> {
  // aux = {rowmax, colmax, flags, factors} after a factorised forward, empty after the exact one
  static variable_list forward(AutogradContext* ctx, const Tensor& a, const Tensor& b, const Tensor& grad,
                               const Tensor& part, const variable_list& aux, int64_t path) {
    ctx->save_for_backward({a, b, grad, part});
    std::vector<Tensor> g;
    if (path == PATH_EXACT)
      g = dense_backward(a, b, grad, part, GBMM_MODE_LOG);
    else
      g = logbmm_fast_backward(a, b, grad, part, aux[0], aux[1], aux[2], path == PATH_TENSOR, aux[3]);
    return {g[0], g[1]};
  }

  static variable_list backward(AutogradContext* ctx, variable_list h) {
    const auto saved = ctx->get_saved_variables();
    const Tensor &a = saved[0], &b = saved[1], &grad = saved[2], &part = saved[3];
    TORCH_CHECK(a.scalar_type() == torch::kFloat32,
                "logbmm: second-order gradients are implemented for float32 inputs only");
    const c10::cuda::CUDAGuard guard(a.device());
    const int64_t B = a.size(0), M = a.size(1), K = a.size(2), N = b.size(2);
    Tensor h_a = h[0].defined() ? h[0].to(torch::kFloat32).contiguous() : torch::zeros_like(a);
    Tensor h_b = h[1].defined() ? h[1].to(torch::kFloat32).contiguous() : torch::zeros_like(b);
    Tensor d_a = torch::empty_like(a), d_b = torch::empty_like(b), d_g = torch::empty_like(grad);
    if (B == 0 || M == 0 || K == 0 || N == 0) {
      d_a.zero_(); d_b.zero_(); d_g.zero_();
    } else {
      check_status(gbmm_dense_backbackward_f32(a.data_ptr<float>(), b.data_ptr<float>(), grad.data_ptr<float>(),
                                               part.data_ptr<float>(), h_a.data_ptr<float>(), h_b.data_ptr<float>(),
                                               d_a.data_ptr<float>(), d_b.data_ptr<float>(), d_g.data_ptr<float>(), B,
                                               M, K, N, stream_of(a)),
                   "gbmm_dense_backbackward_f32");
    }
    return {d_a, d_b, d_g, Tensor(), Tensor(), Tensor()};
  }
};

struct LogMatMul : public torch::autograd::Function<LogMatMul> {
  static Tensor forward(AutogradContext* ctx, const Tensor& a_in, const Tensor& b_in) {
    const Tensor a = widen(a_in, "a"), b = widen(b_in, "b");
    check_pair(a, b);
    const int64_t M = a.size(1), K = a.size(2), N = b.size(2);
    LogPath path = a.scalar_type() == torch::kFloat64 ? PATH_EXACT : log_path(M, K, N);
    Tensor out;
    variable_list aux;
    if (path == PATH_EXACT) {
      out = dense_forward(a, b, GBMM_MODE_LOG, c10::nullopt, false)[0];
    } else {
      auto r = logbmm_fast_forward(a, b, path == PATH_TENSOR, path == PATH_TENSOR && keep_factors(a, b));
      out = r[0];
      aux = {r[1], r[2], r[3], r[4]};
    }
    ctx->save_for_backward({a, b, out});
    ctx->saved_data["path"] = (int64_t)path;
    ctx->saved_data["aux"] = aux;
    ctx->saved_data["ta"] = (int64_t)a_in.scalar_type();
    ctx->saved_data["tb"] = (int64_t)b_in.scalar_type();
    return out.to(a_in.scalar_type());
  }

  static variable_list backward(AutogradContext* ctx, variable_list g) {
    const auto saved = ctx->get_saved_variables();
    const Tensor &a = saved[0], &b = saved[1], &out = saved[2];
    const auto aux = ctx->saved_data["aux"].toTensorVector();
    const int64_t path = ctx->saved_data["path"].toInt();
    auto r = LogMatMulBack::apply(a, b, g[0].contiguous().to(a.scalar_type()), out, aux, path);
    return {r[0].to((c10::ScalarType)ctx->saved_data["ta"].toInt()),
            r[1].to((c10::ScalarType)ctx->saved_data["tb"].toInt())};
  }
};

// max / sample / prodmax (genmul.py:50-97): forward saves the indices, backward routes the cotangent
template <int MODE>
struct IndexRouted : public torch::autograd::Function<IndexRouted<MODE>> {
  static Tensor forward(AutogradContext* ctx, const Tensor& a_in, const Tensor& b_in, const c10::optional<Tensor>& u) {
    const Tensor a = widen(a_in, "a"), b = widen(b_in, "b");
    check_pair(a, b);
    Tensor out, idx;
    const int64_t B = a.size(0), M = a.size(1), K = a.size(2), N = b.size(2);
    if (MODE == GBMM_MODE_SAMPLE && a.scalar_type() == torch::kFloat32 && K > 0 && log_path(M, K, N) == PATH_TENSOR) {
      // the logsumexp from the factorised tensor-core forward, then only the inverse-CDF pass
      const c10::cuda::CUDAGuard guard(a.device());
      Tensor uu = u.has_value() && u->defined() ? *u : torch::rand({B, M, N}, a.options());
      check_input(uu, "u");
      TORCH_CHECK(uu.scalar_type() == a.scalar_type() && uu.dim() == 3 && uu.size(0) == B && uu.size(1) == M &&
                      uu.size(2) == N, "u must have shape (", B, ", ", M, ", ", N, ")");
      out = logbmm_fast_forward(a, b, true, false)[0];
      idx = torch::empty({B, M, N}, a.options().dtype(torch::kInt32));
      check_status(gbmm_dense_sample_pick_f32(a.data_ptr<float>(), b.data_ptr<float>(), uu.data_ptr<float>(),
                                              out.data_ptr<float>(), idx.data_ptr<int32_t>(), B, M, K, N, stream_of(a)),
                   "gbmm_dense_sample_pick_f32");
    } else {
      auto r = dense_forward(a, b, MODE, u, false);
      out = r[0];
      idx = r[1];
    }
    ctx->save_for_backward({a, b, idx});
    ctx->saved_data["ta"] = (int64_t)a_in.scalar_type();
    ctx->saved_data["tb"] = (int64_t)b_in.scalar_type();
    return out.to(a_in.scalar_type());
  }

  static variable_list backward(AutogradContext* ctx, variable_list g) {
    const auto saved = ctx->get_saved_variables();
    const Tensor &a = saved[0], &b = saved[1], &idx = saved[2];
    auto r = dense_backward(a, b, g[0].contiguous().to(a.scalar_type()), idx, MODE);
    return {r[0].to((c10::ScalarType)ctx->saved_data["ta"].toInt()),
            r[1].to((c10::ScalarType)ctx->saved_data["tb"].toInt()), Tensor()};
  }
};

Tensor logbmm(const Tensor& a, const Tensor& b) { return LogMatMul::apply(a, b); }
Tensor maxbmm(const Tensor& a, const Tensor& b) { return IndexRouted<GBMM_MODE_MAX>::apply(a, b, c10::nullopt); }
Tensor prodmaxbmm(const Tensor& a, const Tensor& b) {
  return IndexRouted<GBMM_MODE_PRODMAX>::apply(a, b, c10::nullopt);
}
Tensor samplebmm(const Tensor& a, const Tensor& b, const c10::optional<Tensor>& u) {
  return IndexRouted<GBMM_MODE_SAMPLE>::apply(a, b, u);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "PyTorch binding of libgenbmm_b200.so: the dense semiring operators as C++ autograd functions";
  m.def("logbmm", &logbmm, "log-semiring batched matrix product (differentiable twice)");
  m.def("maxbmm", &maxbmm, "max-plus batched matrix product");
  m.def("prodmaxbmm", &prodmaxbmm, "product-max batched matrix product");
  m.def("samplebmm", &samplebmm, "logsumexp value, one-hot sampled gradient", py::arg("a"), py::arg("b"),
        py::arg("u") = py::none());
  m.def("forward", &dense_forward, "_genbmm.forward(a, b, mode) -> [out, aux]", py::arg("a"), py::arg("b"),
        py::arg("mode"), py::arg("u") = py::none(), py::arg("want_maxes") = true);
  m.def("backward", &dense_backward, "-> [grad_a, grad_b]");
  m.def("abi_version", []() { return gbmm_abi_version(); });
}
