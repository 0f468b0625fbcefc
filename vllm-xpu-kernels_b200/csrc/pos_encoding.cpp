// Torch-facing launchers of the rotary embedding (namespace `_C`, the reference's schema) and of its
// fusion with the flash-layout cache write (namespace `_C_cache_ops`, an addition of this library).
// Counterpart in the reference: csrc/pos_encoding_kernels.cpp:165-286.
#include <ATen/core/Tensor.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include "dispatch_utils.h"
#include "kvcache_b200.h"
#include "ops.h"

namespace {

struct RopeView {
  int64_t heads = 0, stride_t = 0, stride_h = 0;
};

// Heads and strides of a query/key tensor whose first `lead` dims index tokens:
// [.., heads, head_size] or flat [.., heads * head_size] (pos_encoding_kernels.cpp:196-211 there).
RopeView rope_view(const char* op, const at::Tensor& t, int64_t head_size, int64_t lead) {
  TORCH_CHECK(t.dim() == lead + 1 || t.dim() == lead + 2, op,
              ": query/key must be [.., heads, head_size] or [.., heads * head_size]");
  TORCH_CHECK(t.size(-1) <= 1 || t.stride(-1) == 1, op, ": the last dim of query/key must be contiguous");
  // The kernel addresses a token as index * stride(seq dim): with [batch, seq, ...] the batch dim has
  // to continue the seq dim.  The reference assumes it (pos_encoding_kernels.cpp:205-207).
  TORCH_CHECK(lead == 1 || t.size(0) <= 1 || t.stride(0) == t.size(1) * t.stride(1), op,
              ": [batch, seq, ...] tensors must be contiguous across batch and seq");
  RopeView v;
  v.stride_t = t.stride(lead - 1);
  if (t.dim() == lead + 2) {
    TORCH_CHECK(t.size(-1) == head_size, op, ": last dim of query/key must be head_size");
    v.heads = t.size(-2);
    v.stride_h = t.stride(-2);
  } else {
    TORCH_CHECK(t.size(-1) % head_size == 0, op, ": hidden size of query/key is not a multiple of head_size");
    v.heads = t.size(-1) / head_size;
    v.stride_h = head_size;
  }
  return v;
}

struct RopeArgs {
  int64_t num_tokens, rot_dim, max_position;
  RopeView q, k;
  int in_dtype;
};

RopeArgs check_rope(const char* op, const at::Tensor& positions, const at::Tensor& query,
                    const std::optional<at::Tensor>& key, int64_t head_size, const at::Tensor& cos_sin_cache) {
  TORCH_CHECK(query.is_cuda(), op, ": query must be a CUDA tensor (this build has no CPU path)");
  TORCH_CHECK(positions.device() == query.device() && cos_sin_cache.device() == query.device() &&
                  (!key.has_value() || key->device() == query.device()),
              op, ": all tensors must be on query's device");
  const int64_t lead = positions.dim();
  TORCH_CHECK(lead == 1 || lead == 2, "positions must have shape [num_tokens] or [batch_size, seq_len]");
  TORCH_CHECK(positions.scalar_type() == at::kLong && positions.is_contiguous(), op,
              ": positions must be a contiguous int64 tensor");
  TORCH_CHECK(head_size > 0, op, ": head_size must be positive");
  TORCH_CHECK(query.dim() > lead && (!key.has_value() || key->dim() > lead), op, ": query/key have too few dims");
  if (lead == 1) {
    TORCH_CHECK(query.size(0) == positions.size(0) && (!key.has_value() || key->size(0) == positions.size(0)),
                "query, key and positions must have the same number of tokens");
  } else {
    TORCH_CHECK(query.size(0) == positions.size(0) && (!key.has_value() || key->size(0) == positions.size(0)) &&
                    query.size(1) == positions.size(1) && (!key.has_value() || key->size(1) == positions.size(1)),
                "query, key and positions must have the same batch_size and seq_len");
  }
  TORCH_CHECK(!key.has_value() || key->scalar_type() == query.scalar_type(), op,
              ": query and key must have the same dtype");
  TORCH_CHECK(cos_sin_cache.dim() == 2 && cos_sin_cache.is_contiguous() &&
                  cos_sin_cache.scalar_type() == query.scalar_type(),
              op, ": cos_sin_cache must be a contiguous [max_position, rot_dim] tensor of query's dtype");
  RopeArgs a;
  a.num_tokens = positions.numel();
  a.rot_dim = cos_sin_cache.size(1);
  a.max_position = cos_sin_cache.size(0);
  a.q = rope_view(op, query, head_size, lead);
  if (key.has_value()) a.k = rope_view(op, *key, head_size, lead);
  TORCH_CHECK(!key.has_value() || a.k.heads == 0 || a.q.heads % a.k.heads == 0, op,
              ": the number of query heads must be a multiple of the number of key heads");
  a.in_dtype = vllm::kvc_in_dtype_of(query.scalar_type());
  return a;
}

}  // namespace

void rotary_embedding(at::Tensor& positions, at::Tensor& query, std::optional<at::Tensor> key, int64_t head_size,
                      at::Tensor& cos_sin_cache, bool is_neox) {
  constexpr const char* op = "rotary_embedding";
  const RopeArgs a = check_rope(op, positions, query, key, head_size, cos_sin_cache);
  const c10::cuda::CUDAGuard guard(query.device());
  const int rc = kvc_rotary_embedding(
      positions.data_ptr<int64_t>(), query.data_ptr(), key.has_value() ? key->data_ptr() : nullptr,
      cos_sin_cache.data_ptr(), a.num_tokens, a.q.heads, a.k.heads, head_size, a.rot_dim, a.max_position,
      a.q.stride_t, a.q.stride_h, a.k.stride_t, a.k.stride_h, is_neox ? 1 : 0, a.in_dtype,
      c10::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == KVC_OK, op, ": ", kvc_last_error());
}

void rotary_embedding_and_cache_flash(at::Tensor& positions, at::Tensor& query, at::Tensor& key, at::Tensor& value,
                                      int64_t head_size, at::Tensor& cos_sin_cache, bool is_neox,
                                      at::Tensor& key_cache, at::Tensor& value_cache, at::Tensor& slot_mapping,
                                      const std::string& kv_cache_dtype, at::Tensor& k_scale, at::Tensor& v_scale,
                                      bool write_back_key) {
  constexpr const char* op = "rotary_embedding_and_cache_flash";
  const RopeArgs a = check_rope(op, positions, query, std::optional<at::Tensor>(key), head_size, cos_sin_cache);
  const int kv = vllm::kvc_kv_dtype_of(kv_cache_dtype);
  const auto dev = query.device();
  TORCH_CHECK(value.device() == dev && key_cache.device() == dev && value_cache.device() == dev &&
                  slot_mapping.device() == dev,
              op, ": all tensors must be on query's device");
  TORCH_CHECK(value.dim() == 3 && value.size(0) == a.num_tokens && value.size(1) == a.k.heads &&
                  value.size(2) == head_size && (head_size <= 1 || value.stride(2) == 1) &&
                  value.scalar_type() == query.scalar_type(),
              op, ": value must be [num_tokens, num_kv_heads, head_size] of query's dtype, last dim contiguous");
  TORCH_CHECK(slot_mapping.dim() == 1 && slot_mapping.scalar_type() == at::kLong && slot_mapping.is_contiguous() &&
                  slot_mapping.size(0) <= a.num_tokens,
              op, ": slot_mapping must be a contiguous int64 vector no longer than positions");
  for (const at::Tensor* c : {&key_cache, &value_cache}) {
    TORCH_CHECK(c->dim() == 4 && c->size(2) == a.k.heads && c->size(3) == head_size &&
                    (head_size <= 1 || c->stride(3) == 1),
                op, ": caches must be [num_blocks, block_size, num_kv_heads, head_size], last dim contiguous");
    TORCH_CHECK(vllm::kvc_cache_dtype_ok(c->scalar_type(), query.scalar_type(), kv), op,
                ": cache dtype does not fit kv_cache_dtype ", kv_cache_dtype);
  }
  TORCH_CHECK(key_cache.sizes() == value_cache.sizes() && key_cache.strides() == value_cache.strides(), op,
              ": key_cache and value_cache must have the same shape and strides");
  if (kv != KVC_KV_AUTO) {
    for (const at::Tensor* s : {&k_scale, &v_scale})
      TORCH_CHECK(s->device() == dev && s->scalar_type() == at::kFloat && s->numel() >= 1, op,
                  ": k_scale and v_scale must be float32 tensors on query's device");
  }
  const c10::cuda::CUDAGuard guard(dev);
  const int rc = kvc_rotary_embedding_and_cache_flash(
      positions.data_ptr<int64_t>(), query.data_ptr(), key.data_ptr(), value.data_ptr(), cos_sin_cache.data_ptr(),
      key_cache.data_ptr(), value_cache.data_ptr(), slot_mapping.data_ptr<int64_t>(), a.num_tokens,
      slot_mapping.size(0), a.q.heads, a.k.heads, head_size, a.rot_dim, a.max_position, key_cache.size(1),
      a.q.stride_t, a.q.stride_h, a.k.stride_t, a.k.stride_h, value.stride(0), value.stride(1), key_cache.stride(0),
      key_cache.stride(1), key_cache.stride(2), is_neox ? 1 : 0, write_back_key ? 1 : 0, a.in_dtype, kv,
      kv != KVC_KV_AUTO ? static_cast<const float*>(k_scale.data_ptr()) : nullptr,
      kv != KVC_KV_AUTO ? static_cast<const float*>(v_scale.data_ptr()) : nullptr,
      c10::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == KVC_OK, op, ": ", kvc_last_error());
}
