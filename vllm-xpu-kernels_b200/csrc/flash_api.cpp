// Torch-facing launcher of the paged decode attention, registered under `_vllm_fa2_C` like the
// reference's attention op.  Counterpart in the reference: mha_varlen_fwd, csrc/flash_attn/flash_api.cpp:10-176
// (decode branch :124-165) and its schema :179-193.  Both branches are served: one query token per sequence
// (decode) and several, with the causal mask and sliding windows; the non-paged form runs as a cache of
// one-token blocks.  alibi, softcap, dropout and the softmax output are refused.
#include <ATen/core/Tensor.h>
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <vector>

#include "core/registration.h"
#include "dispatch_utils.h"
#include "kvcache_b200.h"

namespace {

void paged_decode_impl(const char* op, const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache,
                       at::Tensor& out, const at::Tensor& seqused_k, const at::Tensor& block_table,
                       int64_t max_seqlen_k, double softmax_scale, const std::optional<at::Tensor>& sink, int kv,
                       const std::optional<at::Tensor>& k_descale, const std::optional<at::Tensor>& v_descale,
                       const std::optional<at::Tensor>& cu_seqlens_q, int64_t max_seqlen_q, bool causal,
                       int64_t window_left, int64_t window_right) {
  TORCH_CHECK(q.is_cuda(), op, ": query must be a CUDA tensor (this build has no CPU path)");
  const auto dev = q.device();
  const auto qt = q.scalar_type();
  TORCH_CHECK(qt == at::kHalf || qt == at::kBFloat16, "VLLM Kernel XPU only supports fp16 and bf16 type");
  TORCH_CHECK(q.dim() == 3, "query must be in ragged format");
  TORCH_CHECK(q.stride(-1) == 1 && k_cache.stride(-1) == 1 && v_cache.stride(-1) == 1,
              "Input tensor must have contiguous last dimension");
  TORCH_CHECK(k_cache.device() == dev && v_cache.device() == dev && out.device() == dev &&
                  seqused_k.device() == dev && block_table.device() == dev,
              op, ": all tensors must be on query's device");
  TORCH_CHECK(k_cache.dim() == 4 && v_cache.sizes() == k_cache.sizes() && v_cache.strides() == k_cache.strides(), op,
              ": caches must be [num_blocks, block_size, num_kv_heads, head_size] with common strides");
  TORCH_CHECK(k_cache.size(3) == q.size(2), op, ": head_size of query and caches differ");
  TORCH_CHECK(vllm::kvc_cache_dtype_ok(k_cache.scalar_type(), qt, kv) && v_cache.scalar_type() == k_cache.scalar_type(),
              kv == KVC_KV_AUTO ? "query and key must have the same dtype" : "cache dtype does not fit kv_cache_dtype");
  TORCH_CHECK(block_table.scalar_type() == at::kInt, "page_table must have dtype torch.int32");
  TORCH_CHECK(block_table.dim() == 2 && block_table.stride(-1) == 1, "page_table must have contiguous last dimension");
  const int64_t num_seqs = seqused_k.numel();
  TORCH_CHECK(seqused_k.scalar_type() == at::kInt && seqused_k.is_contiguous() && seqused_k.dim() == 1, op,
              ": seqused_k must be a contiguous int32 vector with one entry per sequence");
  TORCH_CHECK(block_table.size(0) == num_seqs, op, ": block_table must have one row per sequence");
  const int32_t* cu_q = nullptr;
  if (cu_seqlens_q.has_value()) {
    TORCH_CHECK(cu_seqlens_q->device() == dev && cu_seqlens_q->scalar_type() == at::kInt &&
                    cu_seqlens_q->is_contiguous() && cu_seqlens_q->numel() == num_seqs + 1,
                "cu_seqlens_q must have dtype torch.int32 and one entry per sequence plus one");
    cu_q = cu_seqlens_q->data_ptr<int32_t>();
  } else {
    TORCH_CHECK(q.size(0) == num_seqs && max_seqlen_q == 1, op, ": without cu_seqlens_q every sequence has one query token");
  }
  TORCH_CHECK(out.scalar_type() == qt && out.sizes() == q.sizes() && out.stride(-1) == 1, op,
              ": out must have query's shape and dtype");
  const void* sink_ptr = nullptr;
  if (sink.has_value()) {
    TORCH_CHECK(sink->device() == dev && sink->scalar_type() == qt && sink->is_contiguous() &&
                    sink->numel() == q.size(1),
                op, ": softmax_sink must be a contiguous [num_heads] tensor of query's dtype");
    sink_ptr = sink->data_ptr();
  }
  const float* kd = nullptr;
  const float* vd = nullptr;
  if (kv != KVC_KV_AUTO) {  // per-tensor: the first element of each descale tensor
    for (const auto* d : {&k_descale, &v_descale}) {
      TORCH_CHECK(!d->has_value() || ((*d)->device() == dev && (*d)->scalar_type() == at::kFloat && (*d)->numel() >= 1),
                  op, ": k_descale / v_descale must be float32 tensors on query's device");
    }
    if (k_descale.has_value()) kd = static_cast<const float*>(k_descale->data_ptr());
    if (v_descale.has_value()) vd = static_cast<const float*>(v_descale->data_ptr());
  }
  const int in = vllm::kvc_in_dtype_of(qt);
  const c10::cuda::CUDAGuard guard(dev);
  const int64_t ws_bytes = kvc_paged_attention_workspace_bytes(num_seqs, q.size(0), max_seqlen_q, q.size(1),
                                                               k_cache.size(2), q.size(2), max_seqlen_k, in, kv);
  at::Tensor ws;
  if (ws_bytes > 0) ws = at::empty({ws_bytes}, q.options().dtype(at::kByte));
  const int rc = kvc_paged_attention(
      out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr<int32_t>(),
      seqused_k.data_ptr<int32_t>(), cu_q, sink_ptr, kd, vd, ws_bytes > 0 ? ws.data_ptr() : nullptr, ws_bytes, num_seqs,
      q.size(0), max_seqlen_q, q.size(1), k_cache.size(2), q.size(2), k_cache.size(1), block_table.stride(0),
      max_seqlen_k, q.stride(0), q.stride(1), out.stride(0), out.stride(1), k_cache.stride(0), k_cache.stride(1),
      k_cache.stride(2), static_cast<float>(softmax_scale), causal ? 1 : 0, window_left, window_right, in, kv,
      c10::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == KVC_OK, op, ": ", kvc_last_error());
}

// Argument list of the reference (csrc/flash_attn/flash_api.cpp:10-33).
std::vector<at::Tensor> mha_varlen_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                       std::optional<at::Tensor> out_, const at::Tensor& cu_seqlens_q,
                                       const at::Tensor& cu_seqlens_k, std::optional<at::Tensor> seqused_k,
                                       std::optional<at::Tensor> leftpad_k_, std::optional<at::Tensor> block_table_,
                                       std::optional<at::Tensor> alibi_slopes_, int64_t max_seqlen_q,
                                       int64_t max_seqlen_k, double p_dropout, double softmax_scale,
                                       std::optional<at::Tensor> softmax_sink_, bool zero_tensors, bool is_causal,
                                       int64_t window_size_left, int64_t window_size_right, double softcap,
                                       bool return_softmax, std::optional<at::Generator> gen_) {
  constexpr const char* op = "varlen_fwd";
  (void)zero_tensors;
  (void)gen_;
  TORCH_CHECK(!alibi_slopes_.has_value() && !leftpad_k_.has_value() && softcap == 0.0 && p_dropout == 0.0 &&
                  !return_softmax,
              op, ": alibi_slopes, leftpad_k, softcap, dropout and return_softmax are not supported");
  TORCH_CHECK(cu_seqlens_q.scalar_type() == at::kInt, "cu_seqlens_q must have dtype torch.int32");
  // The reference op's rule (csrc/flash_attn/flash_api.cpp:94 and csrc/xpu/attn/xe_2/fmha_xe2.cpp:99-106 there): a
  // side is open only when it is -1, every other pair is a window -- (0, 0) is the diagonal, (-1, 0) a causal
  // band -- and under the causal mask the right side counts as 0, which the kernels' min() of both ends gives.
  TORCH_CHECK(window_size_left >= -1 && window_size_right >= -1, op, ": a window side is -1 (open) or >= 0");
  const int64_t wl = window_size_left, wr = window_size_right;
  at::Tensor out = out_.has_value() ? *out_ : at::empty(q.sizes(), q.options());
  if (block_table_.has_value()) {
    TORCH_CHECK(seqused_k.has_value(), op, ": seqused_k is needed with a block_table");
    paged_decode_impl(op, q, k, v, out, *seqused_k, *block_table_, max_seqlen_k, softmax_scale, softmax_sink_,
                      KVC_KV_AUTO, std::nullopt, std::nullopt, cu_seqlens_q, max_seqlen_q, is_causal, wl, wr);
  } else {
    // Non-paged form: k, v are [total_k, heads, head_size], sequence s owning rows cu_seqlens_k[s] ..
    // cu_seqlens_k[s+1].  That is a cache of one-token blocks with the table block_table[s][j] = cu_seqlens_k[s] + j.
    TORCH_CHECK(k.dim() == 3 && v.dim() == 3, op, ": without a block_table key and value are [total_k, heads, head_size]");
    TORCH_CHECK(cu_seqlens_k.scalar_type() == at::kInt && cu_seqlens_k.is_contiguous() &&
                    cu_seqlens_k.numel() == cu_seqlens_q.numel() && cu_seqlens_k.device() == q.device(),
                "cu_seqlens_k must have dtype torch.int32");
    const int64_t num_seqs = cu_seqlens_k.numel() - 1;
    const int64_t total_k = k.size(0);
    at::Tensor starts = cu_seqlens_k.slice(0, 0, num_seqs);
    at::Tensor lens = cu_seqlens_k.slice(0, 1, num_seqs + 1) - starts;
    at::Tensor table = (starts.unsqueeze(1) + at::arange(std::max<int64_t>(max_seqlen_k, 1), starts.options()).unsqueeze(0))
                           .clamp_max(std::max<int64_t>(total_k - 1, 0))
                           .contiguous();
    at::Tensor k4 = k.unsqueeze(1), v4 = v.unsqueeze(1);
    paged_decode_impl(op, q, k4, v4, out, lens.contiguous(), table, max_seqlen_k, softmax_scale, softmax_sink_,
                      KVC_KV_AUTO, std::nullopt, std::nullopt, cu_seqlens_q, max_seqlen_q, is_causal, wl, wr);
  }
  return {out, at::empty({0}, q.options().dtype(at::kFloat))};
}

// Shapes and dtypes only (meta tensors): what tracing and fake-tensor propagation need of an op that returns
// tensors.
std::vector<at::Tensor> mha_varlen_fwd_meta(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                            std::optional<at::Tensor> out_, const at::Tensor& cu_seqlens_q,
                                            const at::Tensor& cu_seqlens_k, std::optional<at::Tensor> seqused_k,
                                            std::optional<at::Tensor> leftpad_k_,
                                            std::optional<at::Tensor> block_table_,
                                            std::optional<at::Tensor> alibi_slopes_, int64_t max_seqlen_q,
                                            int64_t max_seqlen_k, double p_dropout, double softmax_scale,
                                            std::optional<at::Tensor> softmax_sink_, bool zero_tensors, bool is_causal,
                                            int64_t window_size_left, int64_t window_size_right, double softcap,
                                            bool return_softmax, std::optional<at::Generator> gen_) {
  at::Tensor out = out_.has_value() ? *out_ : at::empty(q.sizes(), q.options());
  return {out, at::empty({0}, q.options().dtype(at::kFloat))};
}

// Not in the reference: the same decode over a cache stored as fp8 bytes, with the descales its interface
// names (vllm_xpu_kernels/flash_attn_interface.py:46-49 there) but does not implement.
void paged_decode_attention(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache, at::Tensor& out,
                            const at::Tensor& seqused_k, const at::Tensor& block_table, int64_t max_seqlen_k,
                            double softmax_scale, std::optional<at::Tensor> softmax_sink,
                            const std::string& kv_cache_dtype, std::optional<at::Tensor> k_descale,
                            std::optional<at::Tensor> v_descale, std::optional<at::Tensor> cu_seqlens_q,
                            int64_t max_seqlen_q, bool is_causal, int64_t window_size_left,
                            int64_t window_size_right) {
  TORCH_CHECK(window_size_left >= -1 && window_size_right >= -1,
              "paged_decode_attention: a window side is -1 (open) or >= 0");
  paged_decode_impl("paged_decode_attention", q, k_cache, v_cache, out, seqused_k, block_table, max_seqlen_k,
                    softmax_scale, softmax_sink, vllm::kvc_kv_dtype_of(kv_cache_dtype), k_descale, v_descale,
                    cu_seqlens_q, max_seqlen_q, is_causal, window_size_left, window_size_right);
}

}  // namespace

KVC_TORCH_LIBRARY(_vllm_fa2_C, m) {
  m.def(
      "varlen_fwd(Tensor q, Tensor k, Tensor v, Tensor!? out, Tensor "
      "cu_seqlens_q, "
      "Tensor cu_seqlens_k, Tensor? seqused_k, Tensor? leftpad_k, Tensor? "
      "block_table, Tensor? alibi_slopes, "
      "int max_seqlen_q, int max_seqlen_k, float p_dropout, float "
      "softmax_scale, Tensor? softmax_sink, bool zero_tensors, "
      "bool is_causal, int window_size_left, int window_size_right, float "
      "softcap, bool return_softmax, "
      "Generator? gen) -> Tensor[]");
  m.def(
      "paged_decode_attention(Tensor q, Tensor k_cache, Tensor v_cache, Tensor! out, Tensor seqused_k, "
      "Tensor block_table, int max_seqlen_k, float softmax_scale, Tensor? softmax_sink, str kv_cache_dtype, "
      "Tensor? k_descale, Tensor? v_descale, Tensor? cu_seqlens_q=None, int max_seqlen_q=1, bool is_causal=False, "
      "int window_size_left=-1, int window_size_right=-1) -> ()");
}

KVC_TORCH_LIBRARY_IMPL(_vllm_fa2_C, Meta, m) { m.impl("varlen_fwd", &mha_varlen_fwd_meta); }

KVC_TORCH_LIBRARY_IMPL(_vllm_fa2_C, CUDA, m) {
  m.impl("varlen_fwd", &mha_varlen_fwd);
  m.impl("paged_decode_attention", &paged_decode_attention);
}
