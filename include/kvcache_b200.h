/*
 * kvcache_b200 -- C ABI of the B200 (sm_100a) paged KV-cache write kernels.
 *
 * The reference plugin exposes this path only through the PyTorch dispatcher
 * (there is no C interface in it).  Each entry point below carries, as plain
 * pointers, sizes and strides, exactly what the reference's host launcher
 * reads off its at::Tensor arguments before it submits the device kernel, so
 * a binding written in any language can stand where that launcher stands.
 * Citations are file:line inside the reference project.
 *
 * Conventions
 *   - All data pointers are DEVICE pointers on the current CUDA device unless a
 *     parameter says "host".  Strides are in ELEMENTS of the tensor's dtype.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 *     stream).  Calls only enqueue work: no allocation, no host
 *     synchronisation, no reads of device memory on the host.  They are
 *     therefore legal during CUDA-graph stream capture.
 *   - k_scale / v_scale point to one fp32 value each in DEVICE memory and are
 *     read by the kernel (csrc/cache.cpp:161-162).  They are ignored, and may
 *     be NULL, when kv_dtype is KVC_KV_AUTO.
 *   - Return value: KVC_OK or a KVC_ERR_* code; kvc_last_error() then returns
 *     a message (thread-local, valid until the next failing call on the thread).
 *   - Tokens whose slot is negative are skipped (csrc/cache.cpp:49, :145).
 *     Slots >= num_blocks*block_size and duplicate slots are undefined
 *     behaviour, as in the reference; kvc_count_bad_slots() is the debug check.
 *   - Environment (read once per process): KVC_PREFETCH_CTAS=<n> sets how many CTAs of
 *     a scatter launch prefetch their inputs into L2 before waiting for the preceding
 *     kernel (default: half of one resident wave; 0 disables);
 *     KVC_TEST_MAX_ITEMS_PER_LAUNCH=<n> lowers the work-item limit at which
 *     kvc_reshape_and_cache_flash splits a batch into several launches (test hook).
 *     (The torch op layer additionally honours KVC_DEBUG_SLOTS=1: validate slot_mapping
 *     with kvc_count_bad_slots before every scatter, synchronising; debugging only.)
 *   - fp8 stores compute float(x) / scale in IEEE fp32 (correctly rounded),
 *     then round to nearest even onto the fp8 grid and saturate at the largest
 *     finite value (448 for e4m3, 57344 for e5m2); NaN becomes 0x7F.
 */
#ifndef KVCACHE_B200_H_
#define KVCACHE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define KVC_API __attribute__((visibility("default")))
#else
#define KVC_API
#endif

/* dtype of key/value (the reference dispatches on key.scalar_type():
 * csrc/quantization/fp8/quant_utils.h:136-173) */
enum { KVC_IN_F32 = 0, KVC_IN_F16 = 1, KVC_IN_BF16 = 2 };

/* what the cache stores; mirrors Fp8KVCacheDataType
 * (csrc/quantization/fp8/quant_utils.h:10-14).  AUTO = same dtype as key. */
enum { KVC_KV_AUTO = 0, KVC_KV_FP8_E4M3 = 1, KVC_KV_FP8_E5M2 = 2 };

enum {
  KVC_OK = 0,
  KVC_ERR_INVALID_ARG = 1, /* NULL pointer, negative size, head_size % x != 0, ... */
  KVC_ERR_UNSUPPORTED = 2, /* unknown dtype code or kv_cache_dtype string */
  KVC_ERR_CUDA = 3,        /* a CUDA runtime call failed; message holds cudaGetErrorString */
  KVC_ERR_TOO_LARGE = 4    /* request exceeds a fixed capacity of the entry point */
};

/* Library version: major*10000 + minor*100 + patch. */
KVC_API int kvc_version(void);

/* Message of the last failing call on this thread ("" if none). */
KVC_API const char* kvc_last_error(void);

/*
 * Maps the reference's kv_cache_dtype string to a KVC_KV_* code:
 * "auto" -> AUTO, "fp8" and "fp8_e4m3" -> FP8_E4M3, "fp8_e5m2" -> FP8_E5M2
 * (csrc/quantization/fp8/quant_utils.h:137, :148, :160).  Any other string
 * fails with KVC_ERR_UNSUPPORTED and the reference's message
 * "Unsupported data type of kv cache: <s>" (quant_utils.h:171).
 */
KVC_API int kvc_parse_kv_cache_dtype(const char* s, int* kv_dtype_out);

/*
 * Replaces the host launcher + kernel of `reshape_and_cache_flash`
 * (csrc/cache.cpp:461-489 host, :105-189 kernel; schema
 * csrc/torch_bindings.cpp:116-124; prototype csrc/ops.h:51-59).
 *
 *   key, value    [>= num_tokens, num_heads, head_size], last dim contiguous;
 *                 *_stride_t = stride(0), *_stride_h = stride(1)
 *                 (reference reads stride(0) only and assumes stride(1) ==
 *                 head_size: cache.cpp:475-476)
 *   key_cache,    [num_blocks, block_size, num_heads, head_size] views sharing
 *   value_cache   block_stride = stride(0), page_stride = stride(1),
 *                 head_stride = stride(2) (cache.cpp:477-480); last dim
 *                 contiguous.  Element type: key's dtype (AUTO) or 1 byte (fp8).
 *   slot_mapping  int64 [num_tokens]; num_tokens is ITS length, which may be
 *                 smaller than key's first dim (cache.cpp:470).
 */
KVC_API int kvc_reshape_and_cache_flash(const void* key, const void* value, void* key_cache,
                                        void* value_cache, const int64_t* slot_mapping,
                                        int64_t num_tokens, int64_t num_heads, int64_t head_size,
                                        int64_t block_size, int64_t key_stride_t, int64_t key_stride_h,
                                        int64_t value_stride_t, int64_t value_stride_h,
                                        int64_t block_stride, int64_t page_stride, int64_t head_stride,
                                        int in_dtype, int kv_dtype, const float* k_scale,
                                        const float* v_scale, void* stream);

/*
 * Replaces the host launcher + kernel of `reshape_and_cache`
 * (csrc/cache.cpp:409-434 host, :13-103 kernel; schema
 * csrc/torch_bindings.cpp:107-113; prototype csrc/ops.h:41-49).
 *
 *   key_cache     contiguous [num_blocks, num_heads, head_size/x, block_size, x]
 *   value_cache   contiguous [num_blocks, num_heads, head_size, block_size]
 *   x             key_cache.size(4) (cache.cpp:422); must divide head_size
 * All index arithmetic is 64-bit (the reference's is 32-bit: cache.cpp:48-67).
 * fp8 modes DIVIDE by the scale, like the flash op.
 */
KVC_API int kvc_reshape_and_cache(const void* key, const void* value, void* key_cache, void* value_cache,
                                  const int64_t* slot_mapping, int64_t num_tokens, int64_t num_heads,
                                  int64_t head_size, int64_t block_size, int64_t x, int64_t key_stride_t,
                                  int64_t key_stride_h, int64_t value_stride_t, int64_t value_stride_h,
                                  int in_dtype, int kv_dtype, const float* k_scale, const float* v_scale,
                                  void* stream);

/*
 * Replaces the host launcher + kernel of `concat_and_cache_mla`
 * (csrc/cache.cpp:513-550 host, :191-269 kernel; schema
 * csrc/torch_bindings.cpp:127-133).
 *
 *   kv_c      [>= num_tokens, kv_lora_rank], last dim contiguous, kv_c_stride = stride(0)
 *   k_pe      [>= num_tokens, pe_dim],       last dim contiguous, k_pe_stride = stride(0)
 *   kv_cache  [num_blocks, block_size, kv_lora_rank + pe_dim] with block_stride =
 *             stride(0), entry_stride = stride(1); entry = kv_c row then k_pe row
 *   scale     one fp32 value in DEVICE memory, used for both halves (fp8 modes)
 * fp8 modes store rne_saturate(float(x) / scale), the rule of the K/V ops and of
 * upstream vLLM; the reference's SYCL kernel multiplies (cache.cpp:240-244) in a
 * branch its own test cannot reach.  Index arithmetic is 64-bit (reference: int).
 */
KVC_API int kvc_concat_and_cache_mla(const void* kv_c, const void* k_pe, void* kv_cache,
                                     const int64_t* slot_mapping, int64_t num_tokens,
                                     int64_t kv_lora_rank, int64_t pe_dim, int64_t block_size,
                                     int64_t kv_c_stride, int64_t k_pe_stride, int64_t block_stride,
                                     int64_t entry_stride, int in_dtype, int kv_dtype, const float* scale,
                                     void* stream);

/*
 * Replaces the host launcher + kernel of `gather_cache`
 * (csrc/cache.cpp:576-638 host, :271-382 kernel; schema
 * csrc/torch_bindings.cpp:136-139): for every sequence b < batch_size and every
 * j < cu_seq_lens[b+1] - cu_seq_lens[b],
 *   dst[cu_seq_lens[b] + j] = src_cache[block_table[b][seq_starts[b]/block_size + j/block_size]][j % block_size]
 * (seq_starts may be NULL = all zero).  A plain byte copy of entry_size elements
 * of elem_size 1, 2 or 4 bytes; strides in elements.  Only rows below
 * min(num_dst_rows, cu_seq_lens[batch_size]) are written, so the launch is
 * sized from dst's row count and never reads the token total on the host.
 * block_table, cu_seq_lens and seq_starts are int32 DEVICE arrays.
 */
KVC_API int kvc_gather_cache(const void* src_cache, void* dst, const int32_t* block_table,
                             const int32_t* cu_seq_lens, const int32_t* seq_starts, int64_t batch_size,
                             int64_t num_dst_rows, int64_t block_size, int64_t entry_size, int64_t elem_size,
                             int64_t block_table_stride, int64_t cache_block_stride,
                             int64_t cache_entry_stride, int64_t dst_entry_stride, void* stream);

/*
 * Same operation as kvc_reshape_and_cache_flash for callers whose key, value
 * and slot_mapping live in HOST memory (pinned memory makes the copies
 * asynchronous).  The rows are copied into device staging buffers owned by the
 * library (one set per device, grown with cudaMalloc when a call needs more,
 * so the first call and any growing call must not happen during stream
 * capture), then scattered by the same kernel.  key/value rows are
 * [num_tokens, num_heads*head_size] with *_stride_t elements between tokens.
 * The caches and the two scales stay DEVICE pointers.  Work on `stream` is
 * ordered; calls on different streams must not overlap, they share the staging.
 * No counterpart in the reference: its callers always hold device tensors.
 */
KVC_API int kvc_reshape_and_cache_flash_host(const void* host_key, const void* host_value,
                                             void* key_cache, void* value_cache,
                                             const int64_t* host_slot_mapping, int64_t num_tokens,
                                             int64_t num_heads, int64_t head_size, int64_t block_size,
                                             int64_t key_stride_t, int64_t value_stride_t,
                                             int64_t block_stride, int64_t page_stride,
                                             int64_t head_stride, int in_dtype, int kv_dtype,
                                             const float* k_scale, const float* v_scale, void* stream);

/*
 * Variant of kvc_reshape_and_cache_flash_host that never allocates.  It has no
 * counterpart in the reference.
 *
 * Who needs it: processes in which, by the time the cache is being written, the
 * serving framework has already claimed the GPU's free memory for its own pool
 * (vLLM sizes the KV cache from whatever is left), so that a late cudaMalloc by
 * a helper library can fail or eat into that budget; and callers on a latency
 * path that must not meet the device-wide synchronisation cudaMalloc/cudaFree
 * imply.  For them the device staging of key, value and slot_mapping is a fixed
 * area of KVC_NOALLOC_STAGING_BYTES inside the library's own device image:
 * every GPU that loads the library holds that much until the process exits,
 * whether or not this entry point is ever called.  "Loads" is meant literally:
 * under the CUDA runtime's default lazy loading the library's device image
 * reaches a GPU with the first kernel launch or symbol lookup of the library on
 * that GPU, and it is that moment that reserves the area.  A process that is
 * going to hand all free memory to a pool must therefore make its first call of
 * this entry point on each device (or any other call of this library on that
 * device) BEFORE it sizes the pool; if the very first use came afterwards, the
 * load itself could fail for lack of memory and the call would return
 * KVC_ERR_CUDA.  From then on no call changes the amount of free memory.
 *
 * Limit: 2 * round256(num_tokens*num_heads*head_size*elem_size)
 *        + round256(8*num_tokens) must not exceed KVC_NOALLOC_STAGING_BYTES
 * (e.g. 4088 tokens of 8 x 128 bf16).  A larger batch fails with
 * KVC_ERR_TOO_LARGE and a message that states both numbers; nothing is enqueued.
 *
 * The call uses no cudaMalloc, cudaFree or other allocating routine.  The first
 * call on each device looks up the area's device address (cudaGetSymbolAddress,
 * with that device current) and remembers it; make that first call outside of
 * any stream capture.  All calls on a device share the one area and it keeps
 * whatever the last call left in it: each call overwrites every byte it later
 * reads, so nothing needs clearing, but two calls whose work overlaps on the GPU
 * (different streams without ordering) race on it.  Arguments, semantics and
 * results are otherwise those of kvc_reshape_and_cache_flash_host.
 */
#define KVC_NOALLOC_STAGING_BYTES (16 * 1024 * 1024)
KVC_API int kvc_reshape_and_cache_flash_host_noalloc(
    const void* host_key, const void* host_value, void* key_cache, void* value_cache,
    const int64_t* host_slot_mapping, int64_t num_tokens, int64_t num_heads, int64_t head_size,
    int64_t block_size, int64_t key_stride_t, int64_t value_stride_t, int64_t block_stride,
    int64_t page_stride, int64_t head_stride, int in_dtype, int kv_dtype, const float* k_scale,
    const float* v_scale, void* stream);

/* Frees the staging buffers of kvc_reshape_and_cache_flash_host on the current device. */
KVC_API int kvc_release_staging(void);

/*
 * fp8 activation quantisation (the reference's csrc/quantization/fp8/fp8_quant.cpp;
 * schemas csrc/torch_bindings.cpp:67-88).  Element rule, from
 * csrc/quantization/fp8/quant_utils.h:80-91 with an inverted scale:
 *     byte = rne_fp8( fmax(-M, fmin(float(x) * (1.0f / scale), M)) ),  M = 448 | 57344.
 * That is a product with a rounded reciprocal -- the rule the reference's tests pin
 * (tests/test_fp8_quant.py:20-38) -- not the correctly rounded division of the cache ops.
 * in_dtype: KVC_IN_*; fp8_dtype: KVC_KV_FP8_E4M3 or KVC_KV_FP8_E5M2.  Inputs and
 * outputs are contiguous.
 *
 * kvc_static_scaled_fp8_quant            fp8_quant.cpp:135-164: `scale` is given (device fp32).
 * kvc_dynamic_scaled_fp8_quant           fp8_quant.cpp:166-203: first *scale = max(*scale,
 *                                        absmax(x) / M) (atomic; the caller zero-initialises
 *                                        *scale, as the reference's wrapper does), then as static.
 * kvc_dynamic_per_token_scaled_fp8_quant fp8_quant.cpp:205-250: per row of hidden_size elements,
 *                                        scales[t] = max(min(absmax_t, *scale_ub) / M, 1/(512 M))
 *                                        (scale_ub may be NULL), then the row is quantised with it.
 */
KVC_API int kvc_static_scaled_fp8_quant(void* out, const void* input, const float* scale, int64_t num_elems,
                                        int in_dtype, int fp8_dtype, void* stream);
KVC_API int kvc_dynamic_scaled_fp8_quant(void* out, const void* input, float* scale, int64_t num_elems,
                                         int in_dtype, int fp8_dtype, void* stream);
KVC_API int kvc_dynamic_per_token_scaled_fp8_quant(void* out, const void* input, float* scales,
                                                   const float* scale_ub, int64_t num_tokens,
                                                   int64_t hidden_size, int in_dtype, int fp8_dtype,
                                                   void* stream);

/*
 * Rotary position embedding, in place.  Replaces rotary_embedding of the reference: host launcher
 * csrc/pos_encoding_kernels.cpp:165-286, device code :9-162, prototype csrc/ops.h:33-39, schema
 * csrc/torch_bindings.cpp:61-65.
 *
 *   positions      int64 [num_tokens]
 *   query          [num_tokens, num_heads, head_size]; token stride query_stride_t, head stride
 *                  query_stride_h (elements), last dim contiguous; a flat [num_tokens, heads * head_size]
 *                  tensor is the case query_stride_h == head_size
 *   key            the same with num_kv_heads, or NULL (then num_kv_heads is ignored)
 *   cos_sin_cache  contiguous [max_position, rot_dim] of the tensors' type: row p holds rot_dim/2 cosines,
 *                  then rot_dim/2 sines
 *
 * For every token t, head h and i < rot_dim/2, with c = cos_sin_cache[positions[t]][i] and
 * s = cos_sin_cache[positions[t]][rot_dim/2 + i]:
 *     x' = x*c - y*s,   y' = y*c + x*s
 * where (x, y) = elements (i, rot_dim/2 + i) of the head when is_neox, else (2i, 2i+1); each product
 * and the sum are rounded to the tensors' type (three roundings, no fused multiply-add), which is what
 * the torch expression of the reference's tests/ops/rotary_embedding_op.py:11-30 computes.  Elements at
 * and above rot_dim are not touched.  A token whose position is outside [0, max_position) is left
 * unrotated (the reference would read outside the table).  The reference takes one head stride, from
 * query, for both tensors (pos_encoding_kernels.cpp:209-211); here key has its own.
 */
KVC_API int kvc_rotary_embedding(const int64_t* positions, void* query, void* key, const void* cos_sin_cache,
                                 int64_t num_tokens, int64_t num_heads, int64_t num_kv_heads, int64_t head_size,
                                 int64_t rot_dim, int64_t max_position, int64_t query_stride_t,
                                 int64_t query_stride_h, int64_t key_stride_t, int64_t key_stride_h, int is_neox,
                                 int in_dtype, void* stream);

/*
 * No counterpart in the reference: kvc_rotary_embedding followed by kvc_reshape_and_cache_flash of the
 * rotated key and the value, in one pass, so that the key rows are read from HBM once and there is one
 * launch instead of two.  Results are bit-identical to the two calls in sequence.
 *
 *   tokens [0, num_slot_tokens) have a slot in slot_mapping (negative = skip); tokens from there to
 *   num_tokens are rotated only.  value and the caches are as in kvc_reshape_and_cache_flash.
 *   write_back_key == 0 leaves `key` as it was (un-rotated) and only the cache receives the rotated
 *   rows: for callers whose attention reads keys from the cache alone.
 *
 * Needs 16-byte access everywhere (pointers, strides, rot_dim/2 or rot_dim, head_size - rot_dim in
 * whole 16-byte vectors); otherwise KVC_ERR_UNSUPPORTED, and the two separate calls do the job.
 */
KVC_API int kvc_rotary_embedding_and_cache_flash(
    const int64_t* positions, void* query, void* key, const void* value, const void* cos_sin_cache, void* key_cache,
    void* value_cache, const int64_t* slot_mapping, int64_t num_tokens, int64_t num_slot_tokens, int64_t num_heads,
    int64_t num_kv_heads, int64_t head_size, int64_t rot_dim, int64_t max_position, int64_t block_size,
    int64_t query_stride_t, int64_t query_stride_h, int64_t key_stride_t, int64_t key_stride_h,
    int64_t value_stride_t, int64_t value_stride_h, int64_t block_stride, int64_t page_stride, int64_t head_stride,
    int is_neox, int write_back_key, int in_dtype, int kv_dtype, const float* k_scale, const float* v_scale,
    void* stream);

/*
 * Paged decode attention: one query token per sequence against its cached keys and values.
 * Replaces the decode branch of mha_varlen_fwd of the reference (csrc/flash_attn/flash_api.cpp:124-165:
 * paged, max_seqlen_q == 1, no window; op schema :179-193), and extends it to caches stored as fp8,
 * which the reference leaves unimplemented (vllm_xpu_kernels/flash_attn_interface.py:77-82).
 *
 *   out, query     [num_seqs, num_heads, head_size], fp16 or bf16 (q_dtype: KVC_IN_F16 / KVC_IN_BF16),
 *                  strides in elements, last dim contiguous, rows 16-byte aligned
 *   key_cache,     [num_blocks, block_size, num_kv_heads, head_size] views with common strides
 *   value_cache    (block_stride, page_stride, head_stride, in elements), as written by
 *                  kvc_reshape_and_cache_flash: kv_dtype KVC_KV_AUTO = the query's type, KVC_KV_FP8_* = bytes
 *   block_table    int32 [num_seqs, block_table_stride]: block of tokens [i*block_size, (i+1)*block_size)
 *   seq_lens       int32 [num_seqs]: cached tokens per sequence (0 gives a zero row)
 *   sink           NULL, or [num_heads] of the query's type: an extra logit that only enters the softmax
 *                  denominator (flash_api.cpp:27, "softmax_sink")
 *   k_descale,     NULL (= 1), or device fp32 scalars: a stored key element k means k * k_descale, the
 *   v_descale      inverse of the k_scale / v_scale division of the cache write; ignored for KVC_KV_AUTO
 *   max_seq_len    host-side upper bound of seq_lens (the reference's max_seqlen_k); sizes the split
 *   workspace      device scratch of kvc_paged_decode_workspace_bytes(same sizes and types) bytes, 16-byte
 *                  aligned; may be NULL when that function returns 0 (it needs a current CUDA device)
 *   softmax_scale  positive; the descales are positive too
 *
 *   out[s][h] = sum_j softmax_j(softmax_scale * q[s][h] . K[s][j][h / g]) * V[s][j][h / g],  g = num_heads /
 *   num_kv_heads.  Products run on fp16/bf16 tensor-core tiles with fp32 accumulation; probabilities are
 *   rounded to the 16-bit type before they meet V, as in the reference's torch statement
 *   (tests/flash_attn/test_flash_attn_varlen_func.py:27-110).  Floating point: results agree with that
 *   statement within its own tolerance, atol = rtol = 1e-2.  head_size 64, 128, 192 or 256.
 */
KVC_API int64_t kvc_paged_decode_workspace_bytes(int64_t num_seqs, int64_t num_heads, int64_t num_kv_heads,
                                                 int64_t head_size, int64_t max_seq_len, int q_dtype, int kv_dtype);

/*
 * The same over several query tokens per sequence (a chunk of a prefill, speculative tokens) and with sliding
 * windows: what mha_varlen_fwd routes to the reference's chunked-prefill kernel (csrc/flash_attn/
 * flash_api.cpp:105-123: max_seqlen_q > 1 or local attention).  Its non-paged form is the case block_size = 1
 * with block_table[s][j] = cu_seqlens_k[s] + j.
 *
 *   query, out     [total_q, num_heads, head_size]; sequence s owns tokens cu_seqlens_q[s] .. cu_seqlens_q[s+1]
 *   cu_seqlens_q   int32 [num_seqs + 1] on the device; NULL means one token per sequence (the decode call above)
 *   max_seqlen_q   host-side upper bound of the query lengths (sizes the grid)
 *   causal         the query tokens are the last q_len positions of their sequence; with causal != 0 the i-th
 *                  of them sees the first seq_lens[s] - q_len + i + 1 cached tokens, else all seq_lens[s]
 *                  (tests/flash_attn/test_flash_attn_varlen_func.py:79-80, :99-100 of the reference).  A row that
 *                  sees no token gives zeros.
 *   window_left,   sliding window: the query token at position pos sees cached positions pos - window_left ..
 *   window_right   pos + window_right; -1 leaves a side open (test_flash_attn_varlen_func.py:81-95)
 *
 * Sequences with at most 16 (token, head) rows per kv head run on the decode kernel, the others on a second
 * kernel launched beside it.  With head size 128 (or 64 over a 16-bit cache) and some sequence of more than 64 rows per kv head that
 * second kernel runs on the tcgen05 tensor cores: persistent CTAs own two tiles of 128 rows that share every
 * key/value tile; queries, keys, values and results move by TMA tile copies (power-of-two block sizes of at
 * least 8 tokens; other block sizes take a one-tile variant with ordinary asynchronous copies); both products
 * are tcgen05.mma with scores, probabilities and accumulators in tensor memory; fp8 caches are widened to fp16
 * in shared memory.  Head sizes 192 and 256 (one CTA per SM) and fp8 caches of head size 64 take the one-tile
 * variant as well.  Calls whose longest run has at most 64 rows per kv head take the mma.sync kernel in which a
 * CTA owns 64 rows.  In such a mixed call the decode part is not split over the sequence.  At most 65535 sequences per call.
 *
 * kvc_paged_attention_device_status waits for the device's earlier work and reads the tcgen05 kernel's status
 * word: 0 = fine; 1 = a bounded wait on an mbarrier gave up (results of that call are then undefined; the
 * kernel still ran to its end and freed its tensor memory); 2 = its shared-memory window was not 1024-byte
 * aligned (nothing was computed).  The word stays raised until kvc_paged_attention_clear_device_status
 * (which also waits for the device's earlier work) puts it back to 0.
 *
 * kvc_paged_attention_plan tells the launch shape kvc_paged_attention will use for the same arguments (any of
 * the four outputs may be NULL): sequence splits, tiles per split, tokens per tile, and the workspace that shape
 * needs.  It knows the window; its workspace figure is never above kvc_paged_attention_workspace_bytes', which
 * does not, because a windowed call never uses more splits than the same call without the window would.
 *
 * kvc_selftest_bounded_wait_gives_up runs the give-up path of the kernel's bounded waits on purpose: one CTA
 * allocates tensor memory, waits on an mbarrier that nothing arrives on for `tries` tries of about 20 us each
 * (1..5000), gives up, frees its tensor memory and raises the status word to 1.  No counterpart in the reference
 * (its kernels have no bounded waits); it exists so that the path a stuck product or copy would take is one that
 * has run.
 */
KVC_API int kvc_paged_attention_plan(int64_t num_seqs, int64_t total_q, int64_t max_seqlen_q, int64_t num_heads,
                                     int64_t num_kv_heads, int64_t head_size, int64_t max_seq_len, int causal,
                                     int64_t window_left, int64_t window_right, int q_dtype, int kv_dtype,
                                     int32_t* splits, int32_t* tiles_per_split, int32_t* tile_tokens,
                                     int64_t* workspace_bytes);
KVC_API int kvc_paged_attention_clear_device_status(void);
KVC_API int kvc_selftest_bounded_wait_gives_up(int64_t tries, void* stream);
KVC_API int64_t kvc_paged_attention_workspace_bytes(int64_t num_seqs, int64_t total_q, int64_t max_seqlen_q,
                                                    int64_t num_heads, int64_t num_kv_heads, int64_t head_size,
                                                    int64_t max_seq_len, int q_dtype, int kv_dtype);
KVC_API int kvc_paged_attention(void* out, const void* query, const void* key_cache, const void* value_cache,
                                const int32_t* block_table, const int32_t* seq_lens, const int32_t* cu_seqlens_q,
                                const void* sink, const float* k_descale, const float* v_descale, void* workspace,
                                int64_t workspace_bytes, int64_t num_seqs, int64_t total_q, int64_t max_seqlen_q,
                                int64_t num_heads, int64_t num_kv_heads, int64_t head_size, int64_t block_size,
                                int64_t block_table_stride, int64_t max_seq_len, int64_t query_stride_t,
                                int64_t query_stride_h, int64_t out_stride_t, int64_t out_stride_h,
                                int64_t block_stride, int64_t page_stride, int64_t head_stride, float softmax_scale,
                                int causal, int64_t window_left, int64_t window_right, int q_dtype, int kv_dtype,
                                void* stream);
KVC_API int kvc_paged_attention_device_status(int* status);
KVC_API int kvc_paged_decode_attention(void* out, const void* query, const void* key_cache, const void* value_cache,
                                       const int32_t* block_table, const int32_t* seq_lens, const void* sink,
                                       const float* k_descale, const float* v_descale, void* workspace,
                                       int64_t workspace_bytes, int64_t num_seqs, int64_t num_heads,
                                       int64_t num_kv_heads, int64_t head_size, int64_t block_size,
                                       int64_t block_table_stride, int64_t max_seq_len, int64_t query_stride_t,
                                       int64_t query_stride_h, int64_t out_stride_t, int64_t out_stride_h,
                                       int64_t block_stride, int64_t page_stride, int64_t head_stride,
                                       float softmax_scale, int q_dtype, int kv_dtype, void* stream);

/*
 * Debug aid the reference lacks: counts entries of slot_mapping that are
 * >= num_slots (negative entries are legal padding and not counted) into
 * *bad_count, a DEVICE int64 the caller owns; the kernel overwrites it.
 */
KVC_API int kvc_count_bad_slots(const int64_t* slot_mapping, int64_t num_tokens, int64_t num_slots,
                                int64_t* bad_count, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KVCACHE_B200_H_ */
