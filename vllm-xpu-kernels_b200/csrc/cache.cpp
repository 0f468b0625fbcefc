// Torch-facing launchers of the KV-cache ops (two K/V writes, the MLA write, the gather).
//
// Each function reads sizes and strides off its tensors (what the reference does in
// csrc/cache.cpp:409-434, :461-489, :513-550 and :576-638), validates what the kernels rely on, pins the
// device and stream, and hands plain pointers to the CUDA library's C ABI.  There is no
// CPU path: tensors that are not on a CUDA device are rejected.
#include <ATen/core/Tensor.h>
#include <ATen/ops/zeros.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <cstdlib>

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

// Opt-in debugging (KVC_DEBUG_SLOTS=1): count slots >= num_slots on the device and fail before the
// scatter is launched.  It allocates and synchronises, so it is off by default and must not be
// used under CUDA-graph capture.  The reference performs no such check.
void debug_check_slots(const char* op, const at::Tensor& slot_mapping, int64_t num_slots, cudaStream_t stream) {
  static const bool enabled = [] {
    const char* e = std::getenv("KVC_DEBUG_SLOTS");
    return e != nullptr && e[0] != '\0' && e[0] != '0';
  }();
  if (!enabled || slot_mapping.size(0) == 0) return;
  at::Tensor bad = at::zeros({1}, slot_mapping.options());
  check_rc(op, kvc_count_bad_slots(slot_mapping.data_ptr<int64_t>(), slot_mapping.size(0), num_slots,
                                   bad.data_ptr<int64_t>(), stream));
  const int64_t n = bad.item<int64_t>();
  TORCH_CHECK(n == 0, op, ": ", n, " entries of slot_mapping are >= num_blocks * block_size = ", num_slots);
}

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
  debug_check_slots(op, slot_mapping, key_cache.size(0) * block_size, stream);
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
  debug_check_slots(op, slot_mapping, key_cache.size(0) * key_cache.size(1), stream);
  check_rc(op, kvc_reshape_and_cache_flash(
                   key.data_ptr(), value.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
                   slot_mapping.data_ptr<int64_t>(), a.num_tokens, a.num_heads, a.head_size, key_cache.size(1),
                   key.stride(0), key.stride(1), value.stride(0), value.stride(1), key_cache.stride(0),
                   key_cache.stride(1), key_cache.stride(2), a.in_dtype, a.kv_dtype, a.k_scale, a.v_scale,
                   stream));
}

void concat_and_cache_mla(at::Tensor& kv_c, at::Tensor& k_pe, at::Tensor& kv_cache, at::Tensor& slot_mapping,
                          const std::string& kv_cache_dtype, at::Tensor& scale) {
  constexpr const char* op = "concat_and_cache_mla";
  const int kv = vllm::kvc_kv_dtype_of(kv_cache_dtype);
  const int in = vllm::kvc_in_dtype_of(kv_c.scalar_type());
  TORCH_CHECK(kv_c.is_cuda(), op, ": kv_c must be a CUDA tensor (this build has no CPU path)");
  const auto dev = kv_c.device();
  TORCH_CHECK(k_pe.device() == dev && kv_cache.device() == dev && slot_mapping.device() == dev, op,
              ": kv_c, k_pe, kv_cache and slot_mapping must be on the same device");
  TORCH_CHECK(k_pe.scalar_type() == kv_c.scalar_type(), op, ": kv_c and k_pe must have the same dtype");
  TORCH_CHECK(kv_c.dim() == 2 && k_pe.dim() == 2 && kv_cache.dim() == 3, op,
              ": expected kv_c [T, R], k_pe [T, P], kv_cache [num_blocks, block_size, R + P]");
  const int64_t kv_lora_rank = kv_c.size(1), pe_dim = k_pe.size(1);
  TORCH_CHECK(kv_cache.size(2) == kv_lora_rank + pe_dim, op, ": kv_cache.size(2) must be kv_lora_rank + pe_dim");
  TORCH_CHECK((kv_lora_rank <= 1 || kv_c.stride(1) == 1) && (pe_dim <= 1 || k_pe.stride(1) == 1) &&
                  (kv_cache.size(2) <= 1 || kv_cache.stride(2) == 1),
              op, ": the last dim of kv_c, k_pe and kv_cache must be contiguous");
  TORCH_CHECK(slot_mapping.scalar_type() == at::kLong && slot_mapping.dim() == 1 &&
                  (slot_mapping.size(0) <= 1 || slot_mapping.stride(0) == 1),
              op, ": slot_mapping must be a contiguous 1-D int64 tensor");
  const int64_t num_tokens = slot_mapping.size(0);  // may be shorter than kv_c (padded batches)
  TORCH_CHECK(num_tokens <= kv_c.size(0) && num_tokens <= k_pe.size(0), op, ": slot_mapping is longer than kv_c/k_pe");
  TORCH_CHECK(vllm::kvc_cache_dtype_ok(kv_cache.scalar_type(), kv_c.scalar_type(), kv), op, ": cache dtype ",
              kv_cache.scalar_type(), " does not match kv_cache_dtype '", kv_cache_dtype, "' for ",
              kv_c.scalar_type(), " inputs");
  const float* scale_ptr = nullptr;
  if (kv != KVC_KV_AUTO) {
    TORCH_CHECK(scale.device() == dev && scale.scalar_type() == at::kFloat && scale.numel() >= 1, op,
                ": scale must be a float32 tensor on kv_c's device (it is read by the kernel)");
    scale_ptr = static_cast<const float*>(scale.data_ptr());
  }
  const c10::cuda::CUDAGuard guard(dev);
  const cudaStream_t stream = c10::cuda::getCurrentCUDAStream().stream();
  debug_check_slots(op, slot_mapping, kv_cache.size(0) * kv_cache.size(1), stream);
  check_rc(op, kvc_concat_and_cache_mla(kv_c.data_ptr(), k_pe.data_ptr(), kv_cache.data_ptr(),
                                        slot_mapping.data_ptr<int64_t>(), num_tokens, kv_lora_rank, pe_dim,
                                        kv_cache.size(1), kv_c.stride(0), k_pe.stride(0), kv_cache.stride(0),
                                        kv_cache.stride(1), in, kv, scale_ptr, stream));
}

void gather_cache(at::Tensor const& src_cache, at::Tensor const& dst, at::Tensor const& block_table,
                  at::Tensor const& cu_seq_lens, int64_t batch_size, std::optional<at::Tensor> seq_starts) {
  constexpr const char* op = "gather_cache";
  TORCH_CHECK(src_cache.is_cuda(), op, ": src_cache must be a CUDA tensor (this build has no CPU path)");
  // the reference's checks and messages (csrc/cache.cpp:589-610, :624-626)
  TORCH_CHECK(block_table.dtype() == at::kInt, "block_table must be int32");
  TORCH_CHECK(cu_seq_lens.dtype() == at::kInt, "cu_seq_lens must be int32");
  if (seq_starts.has_value()) TORCH_CHECK(seq_starts.value().dtype() == at::kInt, "seq_starts must be int32");
  TORCH_CHECK(src_cache.device() == dst.device(), "src_cache and dst must be on the same device");
  TORCH_CHECK(src_cache.device() == block_table.device(), "src_cache and block_table must be on the same device");
  TORCH_CHECK(src_cache.device() == cu_seq_lens.device(), "src_cache and cu_seq_lens must be on the same device");
  if (seq_starts.has_value())
    TORCH_CHECK(src_cache.device() == seq_starts.value().device(), "src_cache and seq_starts must be on the same device");
  TORCH_CHECK(src_cache.dtype() == dst.dtype(), "src_cache and dst must have the same dtype");
  // what the kernel additionally relies on
  TORCH_CHECK(src_cache.dim() >= 3 && dst.dim() >= 2, op, ": expected src_cache [num_blocks, block_size, entries...] and dst [tot_tokens, entries...]");
  TORCH_CHECK(block_table.dim() == 2 && (block_table.size(1) <= 1 || block_table.stride(1) == 1), op,
              ": block_table must be [batch, blocks] with a contiguous last dim");
  TORCH_CHECK(cu_seq_lens.dim() == 1 && cu_seq_lens.is_contiguous() && cu_seq_lens.size(0) >= batch_size + 1, op,
              ": cu_seq_lens must be a contiguous [batch_size + 1] tensor");
  TORCH_CHECK(batch_size >= 0 && block_table.size(0) >= batch_size, op, ": block_table has fewer rows than batch_size");
  if (seq_starts.has_value())
    TORCH_CHECK(seq_starts.value().is_contiguous() && seq_starts.value().numel() >= batch_size, op,
                ": seq_starts must be a contiguous [batch_size] tensor");
  int64_t entry_size = 1;
  for (int64_t d = 2; d < src_cache.dim(); ++d) entry_size *= src_cache.size(d);
  int64_t dst_entry = 1;
  for (int64_t d = 1; d < dst.dim(); ++d) dst_entry *= dst.size(d);
  TORCH_CHECK(dst_entry == entry_size, op, ": dst rows and cache entries differ in size");
  TORCH_CHECK(src_cache[0][0].is_contiguous() && (dst.size(0) == 0 || dst[0].is_contiguous()), op,
              ": cache entries and dst rows must be contiguous");
  const int64_t width = src_cache.element_size();
  TORCH_CHECK(width == 1 || width == 2 || width == 4, "Unsupported data type width: ", width * 8);

  const c10::cuda::CUDAGuard guard(src_cache.device());
  const cudaStream_t stream = c10::cuda::getCurrentCUDAStream().stream();
  check_rc(op, kvc_gather_cache(src_cache.data_ptr(), dst.data_ptr(), block_table.data_ptr<int32_t>(),
                                cu_seq_lens.data_ptr<int32_t>(),
                                seq_starts.has_value() ? seq_starts.value().data_ptr<int32_t>() : nullptr,
                                batch_size, dst.size(0), src_cache.size(1), entry_size, width, block_table.stride(0),
                                src_cache.stride(0), src_cache.stride(1), dst.stride(0), stream));
}
