// Torch-facing launchers of the two KV-cache write ops.
//
// Each function reads sizes and strides off its tensors (what the reference does in
// csrc/cache.cpp:409-434 and :461-489), validates what the kernels rely on, pins the
// device and stream, and hands plain pointers to the CUDA library's C ABI.  There is no
// CPU path: tensors that are not on a CUDA device are rejected.
#include <ATen/core/Tensor.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include "dispatch_utils.h"
#include "kvcache_b200.h"
#include "ops.h"

namespace {

struct CommonArgs {
  int64_t num_tokens, num_heads, head_size;
  int in_dtype, kv_dtype;
  const float* k_scale;
  const float* v_scale;
};

CommonArgs check_common(const char* op, const at::Tensor& key, const at::Tensor& value,
                        const at::Tensor& key_cache, const at::Tensor& value_cache,
                        const at::Tensor& slot_mapping, const std::string& kv_cache_dtype,
                        const at::Tensor& k_scale, const at::Tensor& v_scale) {
  CommonArgs a{};
  a.kv_dtype = vllm::kvc_kv_dtype_of(kv_cache_dtype);
  a.in_dtype = vllm::kvc_in_dtype_of(key.scalar_type());
  TORCH_CHECK(key.is_cuda(), op, ": key must be a CUDA tensor (this build has no CPU path)");
  const auto dev = key.device();
  TORCH_CHECK(value.device() == dev && key_cache.device() == dev && value_cache.device() == dev &&
                  slot_mapping.device() == dev,
              op, ": key, value, key_cache, value_cache and slot_mapping must be on the same device");
  TORCH_CHECK(value.scalar_type() == key.scalar_type(), op, ": key and value must have the same dtype");
  TORCH_CHECK(key.dim() == 3 && value.dim() == 3, op, ": key and value must be [num_tokens, num_heads, head_size]");
  TORCH_CHECK(key.size(1) == value.size(1) && key.size(2) == value.size(2), op,
              ": key and value must agree in num_heads and head_size");
  TORCH_CHECK((key.size(2) <= 1 || key.stride(2) == 1) && (value.size(2) <= 1 || value.stride(2) == 1), op,
              ": the last dim of key and value must be contiguous");
  TORCH_CHECK(slot_mapping.scalar_type() == at::kLong, op, ": slot_mapping must be int64");
  TORCH_CHECK(slot_mapping.dim() == 1 && (slot_mapping.size(0) <= 1 || slot_mapping.stride(0) == 1), op,
              ": slot_mapping must be a contiguous 1-D tensor");
  a.num_tokens = slot_mapping.size(0);  // not key.size(0): padded batches pass a shorter slot_mapping
  TORCH_CHECK(a.num_tokens <= key.size(0) && a.num_tokens <= value.size(0), op,
              ": slot_mapping is longer than key/value");
  a.num_heads = key.size(1);
  a.head_size = key.size(2);
  TORCH_CHECK(key_cache.scalar_type() == value_cache.scalar_type(), op,
              ": key_cache and value_cache must have the same dtype");
  TORCH_CHECK(vllm::kvc_cache_dtype_ok(key_cache.scalar_type(), key.scalar_type(), a.kv_dtype), op,
              ": cache dtype ", key_cache.scalar_type(), " does not match kv_cache_dtype '", kv_cache_dtype,
              "' for ", key.scalar_type(), " inputs");
  if (a.kv_dtype != KVC_KV_AUTO) {
    TORCH_CHECK(k_scale.device() == dev && v_scale.device() == dev, op,
                ": k_scale and v_scale must be on key's device (they are read by the kernel)");
    TORCH_CHECK(k_scale.scalar_type() == at::kFloat && v_scale.scalar_type() == at::kFloat, op,
                ": k_scale and v_scale must be float32");
    TORCH_CHECK(k_scale.numel() >= 1 && v_scale.numel() >= 1, op, ": k_scale and v_scale must hold one value");
    a.k_scale = static_cast<const float*>(k_scale.data_ptr());
    a.v_scale = static_cast<const float*>(v_scale.data_ptr());
  }
  return a;
}

void check_rc(const char* op, int rc) { TORCH_CHECK(rc == KVC_OK, op, ": ", kvc_last_error()); }

}  // namespace

void reshape_and_cache(at::Tensor& key, at::Tensor& value, at::Tensor& key_cache, at::Tensor& value_cache,
                       at::Tensor& slot_mapping, const std::string& kv_cache_dtype, at::Tensor& k_scale,
                       at::Tensor& v_scale) {
  constexpr const char* op = "reshape_and_cache";
  const CommonArgs a =
      check_common(op, key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype, k_scale, v_scale);
  TORCH_CHECK(key_cache.dim() == 5 && value_cache.dim() == 4, op,
              ": key_cache must be [num_blocks, H, D/x, block_size, x] and value_cache [num_blocks, H, D, block_size]");
  const int64_t block_size = key_cache.size(3);
  const int64_t x = key_cache.size(4);
  TORCH_CHECK(x > 0 && a.head_size % x == 0, op, ": head_size must be a multiple of x = key_cache.size(4)");
  TORCH_CHECK(key_cache.size(1) == a.num_heads && key_cache.size(2) * x == a.head_size, op,
              ": key_cache shape does not match key");
  TORCH_CHECK(value_cache.size(0) == key_cache.size(0) && value_cache.size(1) == a.num_heads &&
                  value_cache.size(2) == a.head_size && value_cache.size(3) == block_size,
              op, ": value_cache shape does not match key_cache / value");
  TORCH_CHECK(key_cache.is_contiguous() && value_cache.is_contiguous(), op, ": paged caches must be contiguous");

  const c10::cuda::CUDAGuard guard(key.device());
  const cudaStream_t stream = c10::cuda::getCurrentCUDAStream().stream();
  check_rc(op, kvc_reshape_and_cache(key.data_ptr(), value.data_ptr(), key_cache.data_ptr(),
                                     value_cache.data_ptr(), slot_mapping.data_ptr<int64_t>(), a.num_tokens,
                                     a.num_heads, a.head_size, block_size, x, key.stride(0), key.stride(1),
                                     value.stride(0), value.stride(1), a.in_dtype, a.kv_dtype, a.k_scale,
                                     a.v_scale, stream));
}

void reshape_and_cache_flash(at::Tensor& key, at::Tensor& value, at::Tensor& key_cache,
                             at::Tensor& value_cache, at::Tensor& slot_mapping,
                             const std::string& kv_cache_dtype, at::Tensor& k_scale, at::Tensor& v_scale) {
  constexpr const char* op = "reshape_and_cache_flash";
  const CommonArgs a =
      check_common(op, key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype, k_scale, v_scale);
  TORCH_CHECK(key_cache.dim() == 4 && value_cache.dim() == 4, op,
              ": caches must be [num_blocks, block_size, num_heads, head_size]");
  TORCH_CHECK(key_cache.size(2) == a.num_heads && key_cache.size(3) == a.head_size, op,
              ": key_cache shape does not match key");
  TORCH_CHECK(value_cache.sizes() == key_cache.sizes(), op, ": value_cache shape does not match key_cache");
  TORCH_CHECK(a.head_size <= 1 || (key_cache.stride(3) == 1 && value_cache.stride(3) == 1), op,
              ": the last dim of the caches must be contiguous");
  // The reference checks stride(0) only (csrc/cache.cpp:480) and then uses key_cache's
  // strides for both caches; requiring all three to agree makes that assumption safe.
  TORCH_CHECK(key_cache.stride(0) == value_cache.stride(0) && key_cache.stride(1) == value_cache.stride(1) &&
                  key_cache.stride(2) == value_cache.stride(2),
              op, ": key_cache and value_cache must have the same strides");

  const c10::cuda::CUDAGuard guard(key.device());
  const cudaStream_t stream = c10::cuda::getCurrentCUDAStream().stream();
  check_rc(op, kvc_reshape_and_cache_flash(
                   key.data_ptr(), value.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
                   slot_mapping.data_ptr<int64_t>(), a.num_tokens, a.num_heads, a.head_size, key_cache.size(1),
                   key.stride(0), key.stride(1), value.stride(0), value.stride(1), key_cache.stride(0),
                   key_cache.stride(1), key_cache.stride(2), a.in_dtype, a.kv_dtype, a.k_scale, a.v_scale,
                   stream));
}
