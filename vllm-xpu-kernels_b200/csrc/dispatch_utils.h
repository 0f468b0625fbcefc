// Type keys of the KV-cache write path.
//
// The reference selects a kernel instance from (key.scalar_type(), kv_cache_dtype string)
// with DISPATCH_BY_KV_CACHE_DTYPE (csrc/quantization/fp8/quant_utils.h:136-173) and keeps
// generic AT_DISPATCH wrappers in csrc/dispatch_utils.h.  Here the template selection
// happens inside the CUDA library, behind the C ABI, so this header only translates torch
// types to the library's integer keys: inputs bf16 / fp16 / fp32, cache stores "auto" /
// fp8_e4m3 / fp8_e5m2.  Error texts match the reference's.
#pragma once
#include <c10/core/ScalarType.h>
#include <c10/util/Exception.h>

#include <string>

#include "kvcache_b200.h"

namespace vllm {

// key/value dtype -> KVC_IN_*   (quant_utils.h:138-146: Float, Half, BFloat16)
inline int kvc_in_dtype_of(c10::ScalarType t) {
  switch (t) {
    case c10::ScalarType::BFloat16: return KVC_IN_BF16;
    case c10::ScalarType::Half: return KVC_IN_F16;
    case c10::ScalarType::Float: return KVC_IN_F32;
    default: TORCH_CHECK(false, "Unsupported input type of kv cache: ", t);
  }
}

// "auto" | "fp8" | "fp8_e4m3" | "fp8_e5m2" -> KVC_KV_*   (quant_utils.h:137, :148, :160, :171)
inline int kvc_kv_dtype_of(const std::string& s) {
  int kv = KVC_KV_AUTO;
  TORCH_CHECK(kvc_parse_kv_cache_dtype(s.c_str(), &kv) == KVC_OK, "Unsupported data type of kv cache: ", s);
  return kv;
}

// Does a cache tensor of dtype `cache` fit the store mode?  "auto" stores key's dtype;
// fp8 modes store one byte per element and accept the torch fp8 dtype as well as a raw
// uint8 buffer (the reference reinterpret_casts data_ptr: csrc/cache.cpp:389-407).
inline bool kvc_cache_dtype_ok(c10::ScalarType cache, c10::ScalarType key, int kv) {
  if (kv == KVC_KV_AUTO) return cache == key;
  if (cache == c10::ScalarType::Byte) return true;
  return kv == KVC_KV_FP8_E4M3 ? cache == c10::ScalarType::Float8_e4m3fn
                               : cache == c10::ScalarType::Float8_e5m2;
}

}  // namespace vllm
