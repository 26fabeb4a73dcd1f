// Python entry points of the model-side kernels (fused batch normalisation).
// They run on the caller's current CUDA stream like any torch op.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstring>
#include <map>
#include <mutex>
#include <tuple>
#include <vector>

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

// Zero-filled scratch for the batch-norm reductions without a fill launch per
// call: slices are handed out from a per-stream pool that is cleared with one
// memset whenever it has been used up. Slices are consumed in stream order
// and the memset is queued behind their consumers, so a slice is zero when
// the kernel that was given it runs.
double* ZeroedDoubles(int64_t count, const at::Tensor& like, cudaStream_t stream) {
  struct Pool {
    at::Tensor buf;
    int64_t used = 0;
  };
  constexpr int64_t POOL_DOUBLES = 1 << 20;  // 8 MB
  static std::mutex mu;
  static std::map<std::pair<int, cudaStream_t>, Pool> pools;
  TORCH_CHECK(count <= POOL_DOUBLES, "batch norm scratch request too large");
  std::lock_guard<std::mutex> lock(mu);
  Pool& p = pools[{like.get_device(), stream}];
  if (!p.buf.defined()) {
    p.buf = at::zeros({POOL_DOUBLES}, like.options().dtype(at::kDouble));
    p.used = 0;
  }
  const int64_t need = (count + 31) / 32 * 32;  // 256-byte slices
  if (p.used + need > POOL_DOUBLES) {
    cudaMemsetAsync(p.buf.data_ptr(), 0, POOL_DOUBLES * sizeof(double), stream);
    p.used = 0;
  }
  double* out = p.buf.data_ptr<double>() + p.used;
  p.used += need;
  return out;
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
    double* sums = ZeroedDoubles(2 * C, x, stream);
    float* rm = nullptr;
    float* rv = nullptr;
    if (running_mean.has_value() && running_mean->defined()) {
      rm = const_cast<float*>(FloatPtrOrNull(running_mean, C, "running_mean"));
      rv = const_cast<float*>(FloatPtrOrNull(running_var, C, "running_var"));
      TORCH_CHECK(rv != nullptr, "running_var must accompany running_mean");
    }
    cudaError_t err = kern::LaunchBatchNormForward(
        x.data_ptr(), res, y.data_ptr(), M, static_cast<int>(C),
        x.scalar_type() == at::kBFloat16, sums,
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
    double* sums = ZeroedDoubles(2 * C, x, stream);
    cudaError_t err = kern::LaunchBatchNormBackward(
        dy.data_ptr(), relu ? y.data_ptr() : nullptr, x.data_ptr(), dx.data_ptr(),
        want_dresidual ? dres.data_ptr() : nullptr, M, static_cast<int>(C),
        x.scalar_type() == at::kBFloat16, sums,
        FloatPtrOrNull(weight, C, "weight"), save_mean.data_ptr<float>(),
        save_invstd.data_ptr<float>(), dweight.data_ptr<float>(), dbias.data_ptr<float>(), relu,
        stream);
    TORCH_CHECK(err == cudaSuccess, "fused batch norm backward: ", cudaGetErrorString(err));
    return std::make_tuple(dx, want_dresidual ? c10::optional<at::Tensor>(dres) : c10::nullopt,
                           dweight, dbias);
  });

  // ---- max pooling 3x3 / stride 2 / padding 1 (channels-last, 16-bit) -------
  m.def("maxpool3s2_supported", [](int64_t channels) {
    return kern::MaxPool3s2Supported(static_cast<int>(channels));
  });
  // x -> (y, idx): idx holds one byte per output element (winning window position).
  m.def("maxpool3s2_forward", [](const at::Tensor& x) {
    CheckActivations(x, "x");
    const int64_t N = x.size(0), C = x.size(1), H = x.size(2), W = x.size(3);
    TORCH_CHECK(kern::MaxPool3s2Supported(static_cast<int>(C)),
                "fused max pooling needs a channel count that is a multiple of 8");
    const int64_t Ho = (H + 2 - 3) / 2 + 1, Wo = (W + 2 - 3) / 2 + 1;
    c10::cuda::CUDAGuard guard(x.device());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    at::Tensor y = at::empty({N, C, Ho, Wo}, x.options(), at::MemoryFormat::ChannelsLast);
    at::Tensor idx = at::empty({N, Ho, Wo, C}, x.options().dtype(at::kByte));
    cudaError_t err = kern::LaunchMaxPool3s2Forward(
        x.data_ptr(), y.data_ptr(), idx.data_ptr<uint8_t>(), static_cast<int>(N),
        static_cast<int>(H), static_cast<int>(W), static_cast<int>(C),
        x.scalar_type() == at::kBFloat16, stream);
    TORCH_CHECK(err == cudaSuccess, "fused max pooling forward: ", cudaGetErrorString(err));
    return std::make_tuple(y, idx);
  });
  // (dy, idx, H, W) -> dx
  m.def("maxpool3s2_backward", [](const at::Tensor& dy, const at::Tensor& idx, int64_t H,
                                  int64_t W) {
    CheckActivations(dy, "dy");
    const int64_t N = dy.size(0), C = dy.size(1);
    TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kByte && idx.is_contiguous() &&
                    idx.numel() == dy.numel(),
                "idx must be the byte tensor returned by maxpool3s2_forward");
    TORCH_CHECK(dy.size(2) == (H + 2 - 3) / 2 + 1 && dy.size(3) == (W + 2 - 3) / 2 + 1,
                "dy does not match the pooled size of an input of ", H, " x ", W);
    c10::cuda::CUDAGuard guard(dy.device());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    at::Tensor dx = at::empty({N, C, H, W}, dy.options(), at::MemoryFormat::ChannelsLast);
    cudaError_t err = kern::LaunchMaxPool3s2Backward(
        dy.data_ptr(), idx.data_ptr<uint8_t>(), dx.data_ptr(), static_cast<int>(N),
        static_cast<int>(H), static_cast<int>(W), static_cast<int>(C),
        dy.scalar_type() == at::kBFloat16, stream);
    TORCH_CHECK(err == cudaSuccess, "fused max pooling backward: ", cudaGetErrorString(err));
    return dx;
  });

  // ---- multi-tensor SGD ------------------------------------------------------
  // Builds the device-side tensor list for sgd_step: (descriptor bytes on the
  // device, number of tensors, number of chunks). Parameters, gradients and
  // momentum buffers must be fp32 CUDA tensors with one memory layout per
  // triple; bufs may be empty (no momentum).
  m.def("sgd_plan", [](const std::vector<at::Tensor>& params,
                       const std::vector<at::Tensor>& grads,
                       const std::vector<at::Tensor>& bufs, int64_t chunk_elems) {
    const size_t n = params.size();
    TORCH_CHECK(n > 0 && grads.size() == n && (bufs.empty() || bufs.size() == n),
                "sgd_plan: list lengths differ");
    TORCH_CHECK(chunk_elems > 0 && chunk_elems % 4 == 0, "chunk_elems must be a multiple of 4");
    std::vector<int64_t> chunk_start;
    std::vector<int32_t> chunk_tensor;
    for (size_t i = 0; i < n; ++i) {
      const at::Tensor& p = params[i];
      const at::Tensor& g = grads[i];
      TORCH_CHECK(p.is_cuda() && p.scalar_type() == at::kFloat && g.is_cuda() &&
                      g.scalar_type() == at::kFloat && g.device() == p.device(),
                  "sgd_plan: parameters and gradients must be fp32 tensors on one GPU");
      TORCH_CHECK(p.is_non_overlapping_and_dense() && g.sizes() == p.sizes() &&
                      g.strides() == p.strides(),
                  "sgd_plan: a gradient does not share its parameter's memory layout");
      if (!bufs.empty())
        TORCH_CHECK(bufs[i].is_cuda() && bufs[i].scalar_type() == at::kFloat &&
                        bufs[i].sizes() == p.sizes() && bufs[i].strides() == p.strides(),
                    "sgd_plan: a momentum buffer does not share its parameter's layout");
      for (int64_t s = 0; s < p.numel(); s += chunk_elems) {
        chunk_start.push_back(s);
        chunk_tensor.push_back(static_cast<int32_t>(i));
      }
    }
    const size_t nc = chunk_start.size();
    const size_t bytes = n * 32 + nc * 8 + nc * 4;
    at::Tensor host = at::empty({static_cast<int64_t>(bytes)},
                                at::TensorOptions().dtype(at::kByte).pinned_memory(true));
    char* h = static_cast<char*>(host.data_ptr());
    void** hp = reinterpret_cast<void**>(h);
    for (size_t i = 0; i < n; ++i) {
      hp[i] = params[i].data_ptr();
      hp[n + i] = grads[i].data_ptr();
      hp[2 * n + i] = bufs.empty() ? nullptr : bufs[i].data_ptr();
      reinterpret_cast<int64_t*>(h + n * 24)[i] = params[i].numel();
    }
    std::memcpy(h + n * 32, chunk_start.data(), nc * 8);
    std::memcpy(h + n * 32 + nc * 8, chunk_tensor.data(), nc * 4);
    c10::cuda::CUDAGuard guard(params[0].device());
    at::Tensor dev = at::empty({static_cast<int64_t>(bytes)},
                               params[0].options().dtype(at::kByte));
    dev.copy_(host, /*non_blocking=*/true);
    return std::make_tuple(dev, static_cast<int64_t>(n), static_cast<int64_t>(nc));
  });
  m.def("sgd_step", [](const at::Tensor& plan, int64_t n, int64_t n_chunks, int64_t chunk_elems,
                       bool has_bufs, double lr, double momentum, double dampening,
                       double weight_decay, bool nesterov, bool first_step, bool maximize) {
    TORCH_CHECK(plan.is_cuda() && plan.scalar_type() == at::kByte &&
                    plan.numel() == n * 32 + n_chunks * 12,
                "sgd_step: not a plan made by sgd_plan");
    c10::cuda::CUDAGuard guard(plan.device());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    char* d = static_cast<char*>(plan.data_ptr());
    kern::SgdTensors t;
    t.n = static_cast<int>(n);
    t.params = reinterpret_cast<float* const*>(d);
    t.grads = reinterpret_cast<const float* const*>(d + n * 8);
    t.bufs = has_bufs ? reinterpret_cast<float* const*>(d + n * 16) : nullptr;
    t.counts = reinterpret_cast<const int64_t*>(d + n * 24);
    t.n_chunks = static_cast<int>(n_chunks);
    t.chunk_start = reinterpret_cast<const int64_t*>(d + n * 32);
    t.chunk_tensor = reinterpret_cast<const int32_t*>(d + n * 32 + n_chunks * 8);
    t.chunk_elems = chunk_elems;
    cudaError_t err = kern::LaunchFusedSgd(
        t, static_cast<float>(lr), static_cast<float>(momentum), static_cast<float>(dampening),
        static_cast<float>(weight_decay), nesterov, first_step, maximize, stream);
    TORCH_CHECK(err == cudaSuccess, "fused SGD: ", cudaGetErrorString(err));
  });
}

}  // namespace hvd
