// Registers the KV-cache ops under torch.ops._C_cache_ops, and the fp8 quantisation ops and the rotary
// embedding under torch.ops._C.
//
// Schema strings are the public interface vLLM's attention backends call and are kept
// character-compatible with the reference's csrc/torch_bindings.cpp:61-64, :67-88, :107-112, :116-122,
// :127-133 and :136-139;
// the implementations are bound for CUDA tensors.  Ops returning () need no meta kernel.
// Only the `_C_cache_ops` namespace of the reference's `_C` module is provided by this library.
#include <torch/library.h>

#include "core/registration.h"
#include "ops.h"

#ifndef TORCH_EXTENSION_NAME
#define TORCH_EXTENSION_NAME _C
#endif

// Namespace `_C`: only the rotary embedding and the fp8 quantisation ops of the reference's much
// larger set (csrc/torch_bindings.cpp:61-64 and :67-88 there).
KVC_TORCH_LIBRARY(TORCH_EXTENSION_NAME, m) {
  m.def(
      "rotary_embedding(Tensor positions, Tensor! query,"
      "                 Tensor!? key, int head_size,"
      "                 Tensor cos_sin_cache, bool is_neox) -> ()");
  m.def("static_scaled_fp8_quant(Tensor! result, Tensor input, Tensor scale) -> ()");
  m.def("dynamic_scaled_fp8_quant(Tensor! result, Tensor input, Tensor! scale) -> ()");
  m.def(
      "dynamic_per_token_scaled_fp8_quant(Tensor! result, Tensor input, "
      "Tensor! scale, Tensor? scale_ub) -> ()");
}

KVC_TORCH_LIBRARY_IMPL(TORCH_EXTENSION_NAME, CUDA, m) {
  m.impl("rotary_embedding", &rotary_embedding);
  m.impl("static_scaled_fp8_quant", &static_scaled_fp8_quant);
  m.impl("dynamic_scaled_fp8_quant", &dynamic_scaled_fp8_quant);
  m.impl("dynamic_per_token_scaled_fp8_quant", &dynamic_per_token_scaled_fp8_quant);
}

KVC_TORCH_LIBRARY(KVC_PP_CAT(TORCH_EXTENSION_NAME, _cache_ops), m) {
  m.def(
      "reshape_and_cache(Tensor key, Tensor value,"
      "                  Tensor! key_cache, Tensor! value_cache,"
      "                  Tensor slot_mapping,"
      "                  str kv_cache_dtype,"
      "                  Tensor k_scale, Tensor v_scale) -> ()");
  m.def(
      "reshape_and_cache_flash(Tensor key, Tensor value,"
      "                        Tensor! key_cache,"
      "                        Tensor! value_cache,"
      "                        Tensor slot_mapping,"
      "                        str kv_cache_dtype,"
      "                        Tensor k_scale, Tensor v_scale) -> ()");
  m.def(
      "concat_and_cache_mla(Tensor kv_c, Tensor k_pe,"
      "                     Tensor! kv_cache,"
      "                     Tensor slot_mapping,"
      "                     str kv_cache_dtype,"
      "                     Tensor scale) -> ()");
  m.def(
      "gather_cache(Tensor src_cache, Tensor! dst, Tensor block_table, "
      "Tensor cu_seq_lens, int batch_size, Tensor? seq_starts) -> ()");
  // Not in the reference: rotary_embedding + reshape_and_cache_flash in one pass over the key.
  m.def(
      "rotary_embedding_and_cache_flash(Tensor positions, Tensor! query, Tensor! key, Tensor value,"
      "                                 int head_size, Tensor cos_sin_cache, bool is_neox,"
      "                                 Tensor! key_cache, Tensor! value_cache, Tensor slot_mapping,"
      "                                 str kv_cache_dtype, Tensor k_scale, Tensor v_scale,"
      "                                 bool write_back_key=True) -> ()");
}

KVC_TORCH_LIBRARY_IMPL(KVC_PP_CAT(TORCH_EXTENSION_NAME, _cache_ops), CUDA, m) {
  m.impl("reshape_and_cache", &reshape_and_cache);
  m.impl("reshape_and_cache_flash", &reshape_and_cache_flash);
  m.impl("concat_and_cache_mla", &concat_and_cache_mla);
  m.impl("gather_cache", &gather_cache);
  m.impl("rotary_embedding_and_cache_flash", &rotary_embedding_and_cache_flash);
}

KVC_DEFINE_EMPTY_PYMODULE(TORCH_EXTENSION_NAME)
