// Python entry points of the model-side kernels (fused batch normalisation).
// They run on the caller's current CUDA stream like any torch op.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <tuple>

#include "../kernels/kernels.h"

namespace hvd {

namespace {

void CheckActivations(const at::Tensor& t, const char* what) {
  TORCH_CHECK(t.is_cuda(), what, " must be a CUDA tensor");
  TORCH_CHECK(t.dim() == 4, what, " must be 4-D (N, C, H, W)");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kHalf, what,
              " must be bfloat16 or float16");
  TORCH_CHECK(t.is_contiguous(at::MemoryFormat::ChannelsLast), what,
              " must be contiguous in channels_last memory format");
}

const float* FloatPtrOrNull(const c10::optional<at::Tensor>& t, int64_t channels, const char* what) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() &&
                  t->numel() == channels,
              what, " must be a contiguous float32 CUDA vector with one entry per channel");
  return t->data_ptr<float>();
}

}  // namespace

void BindModelOps(py::module_& m) {
  m.def("bn_supported", [](int64_t rows, int64_t channels) {
    return kern::BatchNormSupported(rows, static_cast<int>(channels));
  });
  // (x, residual?, weight?, bias?, running_mean?, running_var?, momentum, eps, relu)
  //   -> (y, save_mean, save_invstd)
  m.def("bn_forward", [](const at::Tensor& x, const c10::optional<at::Tensor>& residual,
                         const c10::optional<at::Tensor>& weight,
                         const c10::optional<at::Tensor>& bias,
                         c10::optional<at::Tensor> running_mean,
                         c10::optional<at::Tensor> running_var, double momentum, double eps,
                         bool relu) {
    CheckActivations(x, "x");
    const int64_t C = x.size(1), M = x.numel() / C;
    TORCH_CHECK(kern::BatchNormSupported(M, static_cast<int>(C)),
                "fused batch norm does not support ", C, " channels");
    const void* res = nullptr;
    if (residual.has_value() && residual->defined()) {
      CheckActivations(*residual, "residual");
      TORCH_CHECK(residual->sizes() == x.sizes() && residual->scalar_type() == x.scalar_type(),
                  "residual must match x");
      res = residual->data_ptr();
    }
    c10::cuda::CUDAGuard guard(x.device());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    at::Tensor y = at::empty_like(x, x.options(), at::MemoryFormat::ChannelsLast);
    auto fopt = x.options().dtype(at::kFloat);
    at::Tensor mean = at::empty({C}, fopt), invstd = at::empty({C}, fopt);
    at::Tensor sums = at::zeros({2 * C}, x.options().dtype(at::kDouble));
    float* rm = nullptr;
    float* rv = nullptr;
    if (running_mean.has_value() && running_mean->defined()) {
      rm = const_cast<float*>(FloatPtrOrNull(running_mean, C, "running_mean"));
      rv = const_cast<float*>(FloatPtrOrNull(running_var, C, "running_var"));
      TORCH_CHECK(rv != nullptr, "running_var must accompany running_mean");
    }
    cudaError_t err = kern::LaunchBatchNormForward(
        x.data_ptr(), res, y.data_ptr(), M, static_cast<int>(C),
        x.scalar_type() == at::kBFloat16, sums.data_ptr<double>(),
        FloatPtrOrNull(weight, C, "weight"), FloatPtrOrNull(bias, C, "bias"),
        static_cast<float>(eps), static_cast<float>(momentum), mean.data_ptr<float>(),
        invstd.data_ptr<float>(), rm, rv, relu, stream);
    TORCH_CHECK(err == cudaSuccess, "fused batch norm forward: ", cudaGetErrorString(err));
    return std::make_tuple(y, mean, invstd);
  });
  // (dy, y, x, weight?, save_mean, save_invstd, relu, want_dresidual)
  //   -> (dx, dresidual or None, dweight, dbias)
  m.def("bn_backward", [](const at::Tensor& dy, const at::Tensor& y, const at::Tensor& x,
                          const c10::optional<at::Tensor>& weight, const at::Tensor& save_mean,
                          const at::Tensor& save_invstd, bool relu, bool want_dresidual) {
    CheckActivations(x, "x");
    CheckActivations(dy, "dy");
    if (relu) CheckActivations(y, "y");
    TORCH_CHECK(dy.sizes() == x.sizes() && dy.scalar_type() == x.scalar_type(), "dy must match x");
    const int64_t C = x.size(1), M = x.numel() / C;
    c10::cuda::CUDAGuard guard(x.device());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    at::Tensor dx = at::empty_like(x, x.options(), at::MemoryFormat::ChannelsLast);
    at::Tensor dres;
    if (want_dresidual) dres = at::empty_like(x, x.options(), at::MemoryFormat::ChannelsLast);
    auto fopt = x.options().dtype(at::kFloat);
    at::Tensor dweight = at::empty({C}, fopt), dbias = at::empty({C}, fopt);
    at::Tensor sums = at::zeros({2 * C}, x.options().dtype(at::kDouble));
    cudaError_t err = kern::LaunchBatchNormBackward(
        dy.data_ptr(), relu ? y.data_ptr() : nullptr, x.data_ptr(), dx.data_ptr(),
        want_dresidual ? dres.data_ptr() : nullptr, M, static_cast<int>(C),
        x.scalar_type() == at::kBFloat16, sums.data_ptr<double>(),
        FloatPtrOrNull(weight, C, "weight"), save_mean.data_ptr<float>(),
        save_invstd.data_ptr<float>(), dweight.data_ptr<float>(), dbias.data_ptr<float>(), relu,
        stream);
    TORCH_CHECK(err == cudaSuccess, "fused batch norm backward: ", cudaGetErrorString(err));
    return std::make_tuple(dx, want_dresidual ? c10::optional<at::Tensor>(dres) : c10::nullopt,
                           dweight, dbias);
  });
}

}  // namespace hvd
