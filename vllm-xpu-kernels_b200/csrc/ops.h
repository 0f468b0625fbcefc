// C++ entry points registered with the PyTorch dispatcher.  Signatures are the ones the
// reference declares in csrc/ops.h:41-59, so the schemas in torch_bindings.cpp bind
// without adapters.
#pragma once
#include <ATen/core/Tensor.h>

#include <optional>
#include <string>

// Paged layout: key_cache [num_blocks, H, D/x, block_size, x], value_cache [num_blocks, H, D, block_size].
void reshape_and_cache(at::Tensor& key, at::Tensor& value, at::Tensor& key_cache, at::Tensor& value_cache,
                       at::Tensor& slot_mapping, const std::string& kv_cache_dtype, at::Tensor& k_scale,
                       at::Tensor& v_scale);

// Flash (NHD) layout: caches [num_blocks, block_size, H, D], possibly strided views.
void reshape_and_cache_flash(at::Tensor& key, at::Tensor& value, at::Tensor& key_cache,
                             at::Tensor& value_cache, at::Tensor& slot_mapping,
                             const std::string& kv_cache_dtype, at::Tensor& k_scale, at::Tensor& v_scale);

// MLA: cache entry = kv_c row followed by k_pe row; kv_cache [num_blocks, block_size, kv_lora_rank + pe_dim].
void concat_and_cache_mla(at::Tensor& kv_c, at::Tensor& k_pe, at::Tensor& kv_cache, at::Tensor& slot_mapping,
                          const std::string& kv_cache_dtype, at::Tensor& scale);

// Inverse direction: paged entries -> dense [tot_tokens, entry...] through block_table / cu_seq_lens.
void gather_cache(at::Tensor const& src_cache, at::Tensor const& dst, at::Tensor const& block_table,
                  at::Tensor const& cu_seq_lens, int64_t batch_size, std::optional<at::Tensor> seq_starts);

// fp8 activation quantisation (namespace `_C`; the reference's csrc/ops.h + fp8_quant.cpp:135-250).
void static_scaled_fp8_quant(at::Tensor& out, at::Tensor const& input, at::Tensor const& scale);
void dynamic_scaled_fp8_quant(at::Tensor& out, at::Tensor const& input, at::Tensor& scale);
void dynamic_per_token_scaled_fp8_quant(at::Tensor& out, at::Tensor const& input, at::Tensor& scales,
                                        std::optional<at::Tensor> const& scale_ub);

// Rotary position embedding, in place (namespace `_C`; the reference's csrc/ops.h:33-39 and
// pos_encoding_kernels.cpp:165-286).
void rotary_embedding(at::Tensor& positions, at::Tensor& query, std::optional<at::Tensor> key, int64_t head_size,
                      at::Tensor& cos_sin_cache, bool is_neox);

// rotary_embedding followed by reshape_and_cache_flash(key, value, ...) in one pass (namespace
// `_C_cache_ops`; the reference has no such op).
void rotary_embedding_and_cache_flash(at::Tensor& positions, at::Tensor& query, at::Tensor& key, at::Tensor& value,
                                      int64_t head_size, at::Tensor& cos_sin_cache, bool is_neox,
                                      at::Tensor& key_cache, at::Tensor& value_cache, at::Tensor& slot_mapping,
                                      const std::string& kv_cache_dtype, at::Tensor& k_scale, at::Tensor& v_scale,
                                      bool write_back_key);
