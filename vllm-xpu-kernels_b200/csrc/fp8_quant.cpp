// Torch-facing launchers of the fp8 activation-quantisation ops (namespace `_C`).
// Counterparts in the reference: csrc/quantization/fp8/fp8_quant.cpp:135-250.
#include <ATen/core/Tensor.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include "dispatch_utils.h"
#include "kvcache_b200.h"
#include "ops.h"

namespace {

struct QuantArgs {
  int in_dtype, fp8_dtype;
  cudaStream_t stream;
};

int fp8_code(const char* op, c10::ScalarType t) {
  if (t == c10::ScalarType::Float8_e4m3fn) return KVC_KV_FP8_E4M3;
  if (t == c10::ScalarType::Float8_e5m2) return KVC_KV_FP8_E5M2;
  TORCH_CHECK(false, op, ": result must be float8_e4m3fn or float8_e5m2, got ", t);
}

void check_pair(const char* op, const at::Tensor& out, const at::Tensor& input) {
  TORCH_CHECK(input.is_cuda(), op, ": input must be a CUDA tensor (this build has no CPU path)");
  TORCH_CHECK(out.device() == input.device(), op, ": result and input must be on the same device");
  TORCH_CHECK(input.is_contiguous() && out.is_contiguous(), op, ": result and input must be contiguous");
  TORCH_CHECK(out.numel() >= input.numel(), op, ": result is smaller than input");
}

void check_scale(const char* op, const at::Tensor& scale, const at::Tensor& input, int64_t need) {
  TORCH_CHECK(scale.device() == input.device() && scale.scalar_type() == at::kFloat && scale.is_contiguous() &&
                  scale.numel() >= need,
              op, ": scale must be a contiguous float32 tensor on input's device with at least ", need, " element(s)");
}

void check_rc(const char* op, int rc) { TORCH_CHECK(rc == KVC_OK, op, ": ", kvc_last_error()); }

}  // namespace

void static_scaled_fp8_quant(at::Tensor& out, at::Tensor const& input, at::Tensor const& scale) {
  constexpr const char* op = "static_scaled_fp8_quant";
  check_pair(op, out, input);
  check_scale(op, scale, input, 1);
  const int in = vllm::kvc_in_dtype_of(input.scalar_type());
  const int f8 = fp8_code(op, out.scalar_type());
  const c10::cuda::CUDAGuard guard(input.device());
  check_rc(op, kvc_static_scaled_fp8_quant(out.data_ptr(), input.data_ptr(), static_cast<const float*>(scale.data_ptr()),
                                           input.numel(), in, f8, c10::cuda::getCurrentCUDAStream().stream()));
}

void dynamic_scaled_fp8_quant(at::Tensor& out, at::Tensor const& input, at::Tensor& scale) {
  constexpr const char* op = "dynamic_scaled_fp8_quant";
  check_pair(op, out, input);
  check_scale(op, scale, input, 1);
  const int in = vllm::kvc_in_dtype_of(input.scalar_type());
  const int f8 = fp8_code(op, out.scalar_type());
  const c10::cuda::CUDAGuard guard(input.device());
  check_rc(op, kvc_dynamic_scaled_fp8_quant(out.data_ptr(), input.data_ptr(), static_cast<float*>(scale.data_ptr()),
                                            input.numel(), in, f8, c10::cuda::getCurrentCUDAStream().stream()));
}

void dynamic_per_token_scaled_fp8_quant(at::Tensor& out, at::Tensor const& input, at::Tensor& scales,
                                        std::optional<at::Tensor> const& scale_ub) {
  constexpr const char* op = "dynamic_per_token_scaled_fp8_quant";
  check_pair(op, out, input);
  TORCH_CHECK(input.dim() >= 1, op, ": input must have at least one dim");
  const int64_t hidden = input.size(-1);
  const int64_t tokens = hidden == 0 ? 0 : input.numel() / hidden;
  check_scale(op, scales, input, tokens);
  const float* ub = nullptr;
  if (scale_ub.has_value()) {
    check_scale(op, scale_ub.value(), input, 1);
    ub = static_cast<const float*>(scale_ub.value().data_ptr());
  }
  const int in = vllm::kvc_in_dtype_of(input.scalar_type());
  const int f8 = fp8_code(op, out.scalar_type());
  const c10::cuda::CUDAGuard guard(input.device());
  check_rc(op, kvc_dynamic_per_token_scaled_fp8_quant(out.data_ptr(), input.data_ptr(),
                                                      static_cast<float*>(scales.data_ptr()), ub, tokens, hidden, in,
                                                      f8, c10::cuda::getCurrentCUDAStream().stream()));
}
