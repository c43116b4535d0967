/*
 * cvllm.h — C ABI of libcompactor_sm100.so
 *
 * Drop-in boundary for the attention + KV-compression hot path of
 * vnchari/compactor-vllm, rebuilt as hand-written sm_100a CUDA.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the name ends in `_host`
 *   - every launch function takes the CUDA stream (a cudaStream_t passed as
 *     void*) last, launches on it and returns without synchronising
 *   - return value: 0 = launched; negative = argument error detected on the
 *     host before any launch (see CVLLM_E_*); nothing is thrown
 *   - no torch types; TMA descriptors are rebuilt per call.  Process state is
 *     limited to: the launch counter, a per-(kernel, device) "dynamic shared
 *     memory limit raised" bit (so one process can drive several GPUs), a
 *     per-device SM-count cache, and the explicit test options below.  The
 *     library never reads the environment.
 *   - all index tensors are int32 unless stated; scores are fp32
 *   - strides are in ELEMENTS of the tensor's dtype
 *   - `dtype`: CVLLM_F16 or CVLLM_BF16 (the arithmetic is always fp32
 *     accumulate)
 *
 * Each entry point cites the reference interface it replaces
 * (paths relative to the reference's src/compactor_vllm/).
 */
#ifndef CVLLM_H_
#define CVLLM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CVLLM_ABI_VERSION 1

/* CVLLM_F32: 32-bit storage; only the entry points of the "model blocks" and "biased attention" sections take it. */
enum { CVLLM_F16 = 0, CVLLM_BF16 = 1, CVLLM_F32 = 3 };

enum {
  CVLLM_OK = 0,
  CVLLM_E_ARG = -1,         /* bad shape / size / null pointer            */
  CVLLM_E_UNSUPPORTED = -2, /* head_dim / group size / page size combo    */
  CVLLM_E_WORKSPACE = -3,   /* workspace too small                        */
  CVLLM_E_CUDA = -4,        /* launch or driver-entry-point failure       */
  CVLLM_E_ALIGN = -5        /* pointer / stride not 16-byte aligned       */
};

typedef void* cvllm_stream_t;

/* ABI version + last CUDA error string (host, static storage). */
int cvllm_abi_version(void);
const char* cvllm_last_error(void);
/* Number of kernels this library has launched in this process (monotonic).
 * Lets a caller report how many of its kernels ran inside a timed region. */
uint64_t cvllm_launch_count(void);
/* Test / profiling switches (never needed by a product caller; defaults = product behaviour):
 *   "prefill_v1" 1|0         force the one-query-head-per-CTA prefill kernel (the path odd GQA groups take)
 *   "prefill_threshold" t    lazy-rescale threshold of the prefill softmax in log2 units (0 exercises the
 *                            O-correction path on every growing row max); negative = built-in default
 *   "decode_mode" m          decode_attn.cu profiling modes (0 = product), "decode_slots" n  TMA ring depth cap
 *   "chunk_scores_v1" / "snap_v1" 1|0   the mma.sync scorers instead of the tcgen05 ones (A/B)
 *   "pdl" 1|0                launch the selection chain with programmatic dependent launch (A/B; off by default)
 *   "grs_pairs" n            cap the CTA pairs of cvllm_gemm_allreduce (several virtual ranks on one GPU: the tests)
 *   "grs_rows_per_round" r   rows per reduce round of cvllm_gemm_allreduce (multiple of 256; 0 = default 256)
 *   "grs_probe" mask         timing probes of cvllm_gemm_allreduce (results are wrong on purpose: 1 no TMA loads,
 *                            2 no UMMA, 4 no stores, 8 no reduce, 16 no L2 hints)
 *   "bias_attn_fma" 0|1|2    bfloat16 portions of cvllm_bias_attn_varlen: 0 product choice, 1 the fp32 FMA kernel,
 *                            2 mma.sync also where the tcgen05 kernel would serve (A/B)
 *   "ssm_segment" n          tokens per segment of cvllm_ssm_scan (0 = the product's choice; tests use short segments)
 *   "grs_debug_host_ptr" p   pinned host buffer (64 words per CTA) for cvllm_gemm_allreduce's timeout records
 * Returns CVLLM_E_ARG for an unknown name. */
int cvllm_set_test_option(const char* name, double value);
/* Profiling only: in a library built with -DCVLLM_DECODE_TRACE (tools/trace_decode.py) the next decode launches
 * stamp 8 globaltimer values per CTA (entry, lengths read, first unit landed, streaming done, merge done, role,
 * ticket taken, slots folded) into dev_buf (8 * #CTAs uint64); NULL = off.  Returns -1 in the normal build. */
int cvllm_debug_decode_trace(void* dev_buf);

/* ------------------------------------------------------------------------
 * Store path
 * --------------------------------------------------------------------- */

/* decode_store_kv — kv_cache/store_kv_cache.py:374-466 (kernel :374-416).
 * Append key[b,h,:], value[b,h,:] at logical position bh_lens[b,h] of head
 * (batch_mapping[b], h); bh_lens[b,h] += 1.  Rows with
 * batch_mapping[b] == reserved_batch are skipped. */
int cvllm_decode_store_kv(const void* key, const void* value,
                          int64_t sk_b, int64_t sk_h, int64_t sv_b, int64_t sv_h,
                          const int32_t* batch_mapping, int32_t* bh_lens,
                          const int32_t* page_table, void* k_cache, void* v_cache,
                          int B, int HKV, int D, int PS, int NLP, int elem_bytes,
                          int reserved_batch, cvllm_stream_t stream);

/* prefill_store_all_kv — kv_cache/store_kv_cache.py:251-371.
 * Scatter every (token, head) row of the packed batch to logical position
 * bh_lens[b,h] + t, then bh_lens[b,:] += len_b (the reference's
 * `bh_lens += cu_seqlens_k.diff()[:,None]`, :371). */
int cvllm_prefill_store_all(const void* keys, const void* vals,
                            int64_t sk_n, int64_t sk_h, int64_t sv_n, int64_t sv_h,
                            const int32_t* cu_seqlens_k, const int32_t* batch_mapping,
                            int32_t* bh_lens, const int32_t* page_table,
                            void* k_cache, void* v_cache,
                            int B, int N, int HKV, int D, int PS, int NLP,
                            int elem_bytes, cvllm_stream_t stream);

/* scatter_to_page_table — kv_cache/write_page_table.py:6-95.
 * page_table[l,h,curr[l,h]+i] = new_phys[cum[l,h]+i] for i < add[l,h];
 * the exclusive prefix sum `cum` is computed inside (replaces torch.cumsum,
 * :42-44).  pt_stride_* in int32 elements. */
int cvllm_scatter_pages(const int32_t* add_pages, const int32_t* new_phys,
                        const int32_t* curr_pages, int32_t* page_table,
                        int64_t pt_stride_l, int64_t pt_stride_h, int64_t pt_stride_p,
                        int L, int H, int max_pages_per_head, cvllm_stream_t stream);

/* ------------------------------------------------------------------------
 * Device-side page allocator — PagedKVCache.reserve_tokens /
 * reclaim_pages / free_batch, kv_cache/page_table.py:144-291, without the
 * host heaps: the free set of a layer is a bitmap (bit set = page free), "pop
 * the n smallest ids" is a popcount scan.  Same page ids as the reference's
 * min-heaps.  page_table int32 [L, num_slots, H, P]; bh_seq_lens /
 * bh_num_pages int32 [L, num_slots, H]; free_bits uint32 [L, words];
 * free_count int32 [L]; slots int32 [nb] (entries == reserved_batch are
 * skipped); sequences of one call are served in order.
 * --------------------------------------------------------------------- */
enum {
  CVLLM_PAGES_OK = 0,
  CVLLM_PAGES_EXCEEDS_MAX_SEQUENCE_LENGTH = 1,
  CVLLM_PAGES_EXCEEDS_AVAILABLE_PAGES = 2
};
size_t cvllm_pages_bitmap_words(int n_pages);
size_t cvllm_pages_workspace_bytes(int L, int H, int P, int n_pages, int nb);
int cvllm_pages_init(uint32_t* free_bits, int32_t* free_count, int L, int n_pages,
                     cvllm_stream_t stream);
/* status int32 [nb] <- CVLLM_PAGES_*; a sequence that fails takes nothing
 * (all-or-nothing across layers, page_table.py:171-176). */
int cvllm_pages_reserve(uint32_t* free_bits, int32_t* free_count, int32_t* page_table,
                        const int32_t* bh_seq_lens, int32_t* bh_num_pages, const int32_t* slots,
                        int nb, int add_tokens, int32_t* status, int L, int num_slots, int H,
                        int P, int PS, int n_pages, int reserved_batch, void* workspace,
                        size_t workspace_bytes, cvllm_stream_t stream);
/* free_all == 0: reclaim_pages (keep ceil((len + future_tokens)/PS) pages per
 * head); free_all != 0: free_batch (all pages back, lens and counts zeroed).
 * freed_pages_out (may be NULL) is incremented by the pages returned. */
int cvllm_pages_release(uint32_t* free_bits, int32_t* free_count, const int32_t* page_table,
                        int32_t* bh_seq_lens, int32_t* bh_num_pages, const int32_t* slots, int nb,
                        int future_tokens, int free_all, unsigned long long* freed_pages_out,
                        int L, int num_slots, int H, int P, int PS, int n_pages,
                        int reserved_batch, cvllm_stream_t stream);

/* ------------------------------------------------------------------------
 * The step after the path: the tensor-parallel all-reduce
 * behind o_proj / down_proj — layers/linear.py:149-153 `dist.all_reduce(y)`.
 * One-shot all-reduce over NVLink peer memory for decode-size messages;
 * every rank reads all peers' buffers and sums in rank order (fp32), so all
 * ranks hold identical bits.  Buffers come from cvllm_ipc_alloc (cudaMalloc +
 * cudaIpc handle, flags zeroed); the 64-byte handles are exchanged by the
 * caller (torch.distributed) and opened with cvllm_ipc_open.  A rank's payload
 * starts cvllm_allreduce_flag_bytes() into its buffer.  *_host = host pointers.
 * --------------------------------------------------------------------- */
size_t cvllm_allreduce_flag_bytes(void);
int cvllm_ipc_alloc(size_t payload_bytes, void** ptr_out_host, void* handle_out_host);
int cvllm_ipc_open(const void* handle_host, void** ptr_out_host);
int cvllm_ipc_close(void* peer_ptr);
int cvllm_ipc_free(void* own_ptr);
/* out[i] = sum over ranks of payload_r[i]; numel 16-bit elements, % 8 == 0,
 * the same on every rank; world <= 8.  peer_bases_host[r] = rank r's buffer as
 * mapped in this process.  The payload may be rewritten as soon as the kernel
 * has finished on this rank's stream. */
int cvllm_allreduce_oneshot(void* const* peer_bases_host, int rank, int world, void* out,
                            int64_t numel, int dtype, cvllm_stream_t stream);
/* The same sum in two steps for messages of a few MB at 4-8 ranks: rank r reduces slice r into a RESULT area of its
 * own buffer (result_offset_bytes past the payload start, >= numel * 2, the same on every rank; allocate
 * cvllm_ipc_alloc(payload + result)), publishes it, and every rank gathers the slices.  NVLink traffic per rank
 * 2 x (world-1)/world x message instead of (world-1) x message; identical bits to the one-shot form. */
int cvllm_allreduce_twoshot(void* const* peer_bases_host, int rank, int world, void* out,
                            int64_t numel, int dtype, int64_t result_offset_bytes, cvllm_stream_t stream);

/* RowParallelLinear.forward as ONE kernel — layers/linear.py:133-153 (`F.linear` then `dist.all_reduce`), the o_proj of
 * models/llama3.py:111.  y[M, N] = sum over ranks r of round16(x_r[M, K] . w_r[N, K]^T), fp32 sum in rank order,
 * rounded once, identical bits on every rank.  The GEMM runs on tcgen05 CTA pairs; its epilogue TMA-stores each
 * finished tile into the owning rank's buffer over NVLink (reduce-scatter), reducer warps of the same kernel sum a
 * round of rows as soon as every rank's tiles for it have landed and store the result into y on every rank
 * (all-gather).  Buffers: one cvllm_ipc_alloc(cvllm_gemm_allreduce_payload_bytes(M_max, N, world)) per rank, mapped
 * by every rank (cvllm_ipc_open); a buffer is private to this entry (its flag words are not the all-reduce's).
 * Every rank calls with the same M, N, dtype, in the same order.  *y_out_host = y inside peer_bases_host[rank]; it
 * stays valid until the next call on this buffer.  Needs N, K, lda, ldw multiples of 8 (else CVLLM_E_UNSUPPORTED). */
int64_t cvllm_gemm_allreduce_payload_bytes(int64_t M, int64_t N, int world);
int cvllm_gemm_allreduce(const void* x, int64_t lda, const void* w, int64_t ldw, int64_t M, int64_t N, int64_t K,
                         void* const* peer_bases_host, int rank, int world, int dtype,
                         int64_t payload_capacity_bytes, void** y_out_host, cvllm_stream_t stream);

/* ------------------------------------------------------------------------
 * Selection + compaction
 * --------------------------------------------------------------------- */

/* scores_to_retain_indices — compression/common.py:171-243.
 * Per sequence b: full descending ranking of its len_b*H scores, ties broken
 * by ascending flat index, NaN ranked above +inf (torch.topk order).  Output
 * int64 [B, k_eff], k_eff = min(top_k, max_k_len*H); entry = global flat
 * index (cu[b]+tok)*H + head.  Positions >= len_b*H hold the padded-slot
 * indices the reference would produce (cu[b]*H + padded position). */
size_t cvllm_rank_scores_workspace_bytes(int B, int H, int max_k_len);
int cvllm_rank_scores(const float* scores, int64_t s_stride_n,
                      const int32_t* cu_seqlens_k, int B, int H, int max_k_len,
                      int top_k, int64_t* out_indices, void* workspace,
                      size_t workspace_bytes, cvllm_stream_t stream);
/* The same ranking with NO caller workspace and no allocation of any kind (no cudaMalloc / cudaFree / allocating
 * library call).  No counterpart in the reference: added at the request of the run's operators for callers that cannot
 * allocate (CUDA-graph capture, tight serving loops, harnesses that forbid cudaMalloc).  The sort's scratch is a
 * file-scope device array of cvllm_rank_scores_static_max_bytes() = 8 MiB that every GPU loading the library holds
 * until exit; problems whose cvllm_rank_scores_workspace_bytes(B, H, max_k_len) exceeds it (more than ~510 K scores)
 * return CVLLM_E_UNSUPPORTED with the sizes in cvllm_last_error().  All calls on a device SHARE the array: calls that
 * overlap on the GPU (different streams) race; nothing needs clearing between calls.  Output identical to
 * cvllm_rank_scores. */
size_t cvllm_rank_scores_static_max_bytes(void);
int cvllm_rank_scores_static(const float* scores, int64_t s_stride_n,
                             const int32_t* cu_seqlens_k, int B, int H, int max_k_len,
                             int top_k, int64_t* out_indices, cvllm_stream_t stream);

/* prefill_store_topk_kv — kv_cache/store_kv_cache.py:9-248 (K4 + K5), index
 * flavour: `indices` is the [B, max_sel] ranking (int32 or int64 by
 * idx_bytes).  The first num_retain[b] entries are stored, then (if
 * pad_to_page) each head is topped up to a page multiple with the next
 * entries of that head (:205-248).  Rows are written in ascending token order
 * per head (the reference's order is atomic-nondeterministic). */
size_t cvllm_store_topk_workspace_bytes(int B, int H, int N, int max_sel);
int cvllm_prefill_store_topk_idx(const void* keys, const void* vals,
                                 int64_t sk_n, int64_t sk_h, int64_t sv_n, int64_t sv_h,
                                 const void* indices, int idx_bytes, int max_sel,
                                 const int32_t* num_retain, const int32_t* cu_seqlens_k,
                                 const int32_t* batch_mapping, int32_t* bh_lens,
                                 const int32_t* page_table, void* k_cache, void* v_cache,
                                 int B, int N, int HKV, int D, int PS, int NLP,
                                 int elem_bytes, int pad_to_page, int reserved_batch,
                                 void* workspace, size_t workspace_bytes,
                                 cvllm_stream_t stream);

/* extract_and_store_top_kv — compression/common.py:126-168, fused: scores ->
 * radix-select (global top num_retain[b], then per-head top n_h) -> gather
 * into the paged cache.  Same kept sets as rank + store_topk_idx with the full
 * ranking (top_k >= max_len*H, the engine's setting, utils/arguments.py
 * :208-211). */
size_t cvllm_select_store_workspace_bytes(int B, int H, int N);
int cvllm_select_store_topk(const float* scores, int64_t s_stride_n,
                            const void* keys, const void* vals,
                            int64_t sk_n, int64_t sk_h, int64_t sv_n, int64_t sv_h,
                            const int32_t* num_retain, const int32_t* cu_seqlens_k,
                            const int32_t* batch_mapping, int32_t* bh_lens,
                            const int32_t* page_table, void* k_cache, void* v_cache,
                            int B, int N, int HKV, int D, int PS, int NLP,
                            int elem_bytes, int pad_to_page, int reserved_batch,
                            void* workspace, size_t workspace_bytes,
                            cvllm_stream_t stream);

/* ------------------------------------------------------------------------
 * Attention
 * --------------------------------------------------------------------- */

/* head_sparse_decode_attention — attention/sparse_decode_kernel.py:10-165
 * (K2 :247-388 + K3 :392-435).  One query token per sequence against the
 * per-(b,h) paged rows; balanced split over 128-token units with an in-kernel
 * LSE merge.  Rows with L==0 are written as zeros.  `num_ctas` <= 0 picks
 * one persistent CTA per SM.  PS must be 16, 32, 64 or a multiple of 128 (a
 * TMA box of min(PS,128) rows never crosses a page).  Workspace contract: the
 * first 256-byte-rounded B*HKV*4 bytes are per-head tickets that must be ZERO
 * the first time a workspace is used; every launch leaves them zero again, so
 * a workspace zeroed once at allocation can be reused forever (and a captured
 * graph is the single kernel node).  Graph-capturable: no host sync, fixed
 * grid. */
size_t cvllm_decode_attention_workspace_bytes(int B, int HQ, int HKV, int D, int num_ctas);
int cvllm_decode_attention(const void* q, void* out, const void* k_cache, const void* v_cache,
                           const int32_t* seq_lens_bh, const int32_t* page_table,
                           const int32_t* batch_mapping, void* workspace,
                           size_t workspace_bytes, int B, int HQ, int HKV, int D,
                           int PS, int NLP, float sm_scale, int dtype, int num_ctas,
                           cvllm_stream_t stream);

/* The decode branch of Attention.forward (layers/attention.py:133-160) as one call: decode_store_kv followed by
 * head_sparse_decode_attention, both indexing the cache's own `bh_seq_lens` table [Bmax+1, HKV] through
 * `batch_mapping` (rows mapped to `reserved_batch` are skipped by the store and read length 0).  Replaces the
 * reference's index_select / clone / index_copy_ of a gathered length copy: two kernel nodes per layer-step.
 * 16-bit caches only; workspace contract as for cvllm_decode_attention. */
int cvllm_decode_step(const void* key, const void* value, int64_t sk_b, int64_t sk_h,
                      int64_t sv_b, int64_t sv_h, const void* q, void* out, void* k_cache,
                      void* v_cache, int32_t* bh_seq_lens, const int32_t* page_table,
                      const int32_t* batch_mapping, void* workspace, size_t workspace_bytes,
                      int B, int HQ, int HKV, int D, int PS, int NLP, float sm_scale, int dtype,
                      int reserved_batch, int num_ctas, cvllm_stream_t stream);

/* causal_sparse_varlen_with_cache — attention/sparse_varlen_kernel.py:11-197
 * (K1 :265-519).  Causal attention of the packed new tokens over
 * [cached prefix of (b,h) || new K/V of b]; tcgen05/TMEM/TMA kernel. */
int cvllm_prefill_attention(const void* q, const void* k, const void* v, void* out,
                            const void* k_cache, const void* v_cache,
                            const int32_t* seq_lens_bh, const int32_t* page_table,
                            const int32_t* batch_mapping, const int32_t* cu_seqlens_q,
                            int B, int N, int HQ, int HKV, int D, int PS, int NLP,
                            int64_t cache_rows, int64_t q_stride_n, int64_t k_stride_n,
                            int64_t v_stride_n, int64_t o_stride_n, int max_seqlen_q,
                            float sm_scale, int dtype, cvllm_stream_t stream);

/* ------------------------------------------------------------------------
 * Scoring
 * --------------------------------------------------------------------- */

/* approximate_leverage_scores — compression/compactor.py:113-221 (+ z-score
 * :224-269).  chunk_offsets[n_chunks+1] are packed-token offsets of the
 * (<= chunk_size) chunks produced by split_into_chunks (:62-110).  out is
 * [N, HKV] in `dtype` (the reference returns K's dtype). */
size_t cvllm_leverage_scores_workspace_bytes(int N, int HKV, int sketch, int n_chunks);
int cvllm_leverage_scores(const void* k_pre, int64_t k_stride_n, int64_t k_stride_h,
                          const int32_t* chunk_offsets, int n_chunks, int max_chunk,
                          const void* phi, void* out_scores, int N, int HKV, int D,
                          int sketch, float regularizer, int normalize, int dtype,
                          void* workspace, size_t workspace_bytes, cvllm_stream_t stream);
/* Same chain from a precomputed sketch: sketch_rows [N, HKV, 48] in `dtype`
 * = round16(K_pre . PHI) — compression/compactor.py:153-158 — as written by
 * cvllm_rope_qk; bit-identical scores to cvllm_leverage_scores on the same
 * keys.  phi may be NULL. */
int cvllm_leverage_scores_from_sketch(const void* sketch_rows, const int32_t* chunk_offsets,
                                      int n_chunks, int max_chunk, const void* phi,
                                      void* out_scores, int N, int HKV, int sketch,
                                      float regularizer, int normalize, int dtype,
                                      void* workspace, size_t workspace_bytes,
                                      cvllm_stream_t stream);

/* ------------------------------------------------------------------------
 * The step in front of the path
 * --------------------------------------------------------------------- */

/* RotaryEmbedding.forward — layers/rotary_embedding.py:69-80 (neox
 * rotate-half, :8-16), optionally preceded by the per-head q_norm / k_norm
 * RMSNorm of models/qwen3.py:90-91 (layers/layernorm.py:16-26) and emitting
 * the Compactor sketch of the (normed) pre-RoPE keys
 * (compression/compactor.py:153-158) in the same pass.
 *   q [N,HQ,128], k [N,HKV,128] strided; q_out / k_out may alias q / k
 *   positions int64 [N]; cos_sin_cache fp32 [max_position, 128] = cos | sin
 *   q_norm_weight / k_norm_weight: [128] in `dtype` or NULL (no norm)
 *   phi [128,48] in `dtype` + sketch_out [N,HKV,48] in `dtype`, or both NULL
 *   (sketch needs HKV <= 8) */
int cvllm_rope_qk(const void* q, const void* k, void* q_out, void* k_out, int64_t q_stride_n,
                  int64_t q_stride_h, int64_t k_stride_n, int64_t k_stride_h,
                  int64_t qo_stride_n, int64_t qo_stride_h, int64_t ko_stride_n,
                  int64_t ko_stride_h, const int64_t* positions, const float* cos_sin_cache,
                  int max_position, const void* q_norm_weight, const void* k_norm_weight,
                  float eps, const void* phi, void* sketch_out, int N, int HQ, int HKV, int D,
                  int sketch, int dtype, cvllm_stream_t stream);

/* RMSNorm.forward — layers/layernorm.py:16-49.  residual == NULL:
 * out = round16(x * rsqrt(mean(x^2) + eps)) * weight.  residual != NULL
 * (add_rms_forward): x += residual in fp32, residual <- round16(x) in place,
 * then the same norm.  width % 8 == 0, width <= 8192. */
int cvllm_rmsnorm(const void* x, void* residual, const void* weight, void* out, int64_t x_stride,
                  int64_t residual_stride, int64_t out_stride, int rows, int width, float eps,
                  int dtype, cvllm_stream_t stream);

/* non_causal_attn_scores — compression/compactor.py:338-599.  Chunk-local
 * softmax column sums, per-sequence z-score, + blend*accum, protected
 * first/last tokens <- +inf.  out fp32 [N, HKV]. accum may be NULL;
 * accum_dtype: 2 = fp32, else CVLLM_F16/BF16.  prot_first/prot_last may be
 * NULL (device int32 [B]). */
size_t cvllm_chunk_attn_scores_workspace_bytes(int B, int N, int HKV, int chunk);
int cvllm_chunk_attn_scores(const void* q, const void* k, int64_t q_stride_n,
                            int64_t k_stride_n, const int32_t* cu_seqlens,
                            int B, int N, int HQ, int HKV, int D, int chunk,
                            int max_seqlen, float sm_scale, int normalize,
                            const void* accum, int accum_dtype, int64_t accum_stride_n,
                            float blend, const int32_t* prot_first,
                            const int32_t* prot_last, float* out, int dtype,
                            void* workspace, size_t workspace_bytes,
                            cvllm_stream_t stream);

/* query_aware_key_scores — compression/snapkv.py:39-276,332-448.  SnapKV:
 * last-w queries x G heads against keys [0, L-w), softmax over those keys,
 * column sums, causal `kpool`-tap mean pool inside `pool_segment`-key
 * segments (the reference's autotuned BLOCK_K, :160-168,253-262), window
 * keys <- +inf.  No logits scratch. */
size_t cvllm_snapkv_scores_workspace_bytes(int B, int N, int HQ, int HKV, int w);
int cvllm_snapkv_scores(const void* q, const void* k, int64_t q_stride_n,
                        int64_t k_stride_n, const int32_t* cu_seqlens_q,
                        const int32_t* cu_seqlens_k, int w, int B, int Nk, int HQ,
                        int HKV, int D, int max_seqlen_k, float sm_scale, int kpool,
                        int pool_segment, float* out, int dtype, void* workspace,
                        size_t workspace_bytes, cvllm_stream_t stream);

/* Test entry: the fp64 symmetric eigensolver of the leverage chain alone (csrc/score_leverage.cu).
 * gram fp32 [mats,48,48]; lam_out fp64 [mats,48]; vec_out fp64 [mats,48,48] (columns = eigenvectors, any
 * order); sv_out fp32 [mats,48,48] = round16(V |lam|^-1/2), what the score kernel consumes
 * (reference compression/compactor.py:177,197).  clk_out (optional, int64 [mats,6]): SM clock at kernel entry,
 * after the tridiagonal reduction, at the end of the QL producer, at the end of the reflector accumulation, at
 * exit, and the number of ring entries produced (profiling). */
int cvllm_selftest_eig(const float* gram, double* lam_out, double* vec_out, float* sv_out, int mats,
                       int dtype, long long* clk_out, cvllm_stream_t stream);

/* ------------------------------------------------------------------------
 * Self tests (device sanity for descriptor encodings; used by tests only)
 * --------------------------------------------------------------------- */
int cvllm_selftest_umma(const void* a, const void* b, float* d, int mode,
                        uint32_t lbo, uint32_t sbo, int dtype, cvllm_stream_t stream);

/* ------------------------------------------------------------------------
 * Model blocks with a 32-bit residual stream (csrc/blocks.cu).  dtype arguments: CVLLM_BF16 or CVLLM_F32.
 * Norm weights, router logits, routing weights and the residual are fp32.
 * --------------------------------------------------------------------- */

/* Sandwich RMS norm, one launch per residual update, rows independent:
 *   y != NULL:      resid += y / sqrt(mean(y^2) + eps) * (w_post + gain_offset)   (y [rows, width] of y_dtype;
 *                   with `assign` the sum is replaced: resid = normed y)
 *   w_pre != NULL:  out = resid / sqrt(mean(resid^2) + eps) * (w_pre + gain_offset)   (out [rows, width] of out_dtype)
 *   out != NULL without w_pre:  out = resid rounded to out_dtype
 * gain_offset 1 serves gains stored around zero.  y and w_post come together.  width <= 12288.  Strides in elements. */
int cvllm_sandwich_norm(const void* y, int64_t y_stride, int y_dtype, const float* w_post, float* resid,
                        int64_t r_stride, const float* w_pre, void* out, int64_t o_stride, int out_dtype,
                        int rows, int width, float eps, float gain_offset, int assign, cvllm_stream_t stream);

/* One launch per residual update of a 32-bit stream, rows independent:
 *   resid += a + b + c   (a, b [rows, width] of ab_dtype, c fp32 [rows, width]; each may be NULL)
 *   out = norm(resid)    (out may be NULL: the sum alone); kind 0: resid / sqrt(mean(resid^2) + eps) * w;
 *   kind 1, layer norm: (resid - mean) / sqrt(var + eps) * w + bias, var = the mean of the squared deviations
 *   (bias may be NULL).  w, bias fp32.  width <= 12288.  Strides in elements. */
int cvllm_residual_norm(const void* a, int64_t a_stride, const void* b, int64_t b_stride, int ab_dtype,
                        const float* c, int64_t c_stride, float* resid, int64_t r_stride, const float* w,
                        const float* bias, void* out, int64_t o_stride, int out_dtype, int rows, int width, float eps,
                        int kind, cvllm_stream_t stream);

/* out[t, :] (fp32) = embed[ids[t], :] + pair[row_t, :] with row_t = (prev_t * mul_prev + ids[t] * mul_cur) mod buckets,
 * and row_t = buckets (the table's extra last row) where positions[t] == 0.  prev_t = ids[t - 1] when token t - 1 of
 * the step has the same slot and the position before, else prev_state[token_slot[t]]; afterwards prev_state[slot] =
 * the last token the slot brought in this step (reserved_slot excepted).  embed [V, width], pair [buckets + 1, width]. */
int cvllm_pair_hash_embed(const int64_t* ids, const int32_t* positions, const int32_t* token_slot, const void* embed,
                          const void* pair, int64_t buckets, int64_t mul_prev, int64_t mul_cur, int32_t* prev_state,
                          float* out, int64_t out_stride, int T, int width, int reserved_slot, int dtype,
                          cvllm_stream_t stream);

/* Packed [gate | up] rows -> out[t, f]; kind 0: silu(gate) * up, 1: gelu_tanh(gate) * up, 2: the clamped gated unit
 * g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(1.702 g) * (u + 1).  limit is read by kind 2 only. */
int cvllm_gated_act(const void* x, int64_t x_stride, void* out, int64_t o_stride, int64_t rows, int F, int kind,
                    float limit, int dtype, cvllm_stream_t stream);

/* Router: s = softmax(logits[t, :E]); choice = s + correction (NULL = none).  The E outputs form `groups` equal
 * runs of neighbours; only the `keep` groups with the largest maximum of choice stay eligible; of those the `top`
 * largest choices are taken (ties: the lower index).  idx int32 [T, top], wts fp32 [T, top] = the plain s of the
 * chosen outputs, not renormalised.  E <= 2048, E % groups == 0, keep * E / groups >= top.
 * mode 1 (groups 1, no correction, top <= 32): the `top` largest LOGITS are taken and wts is the softmax over the
 * chosen logits alone.  mode 2 (same limits): the `top` largest sigmoid(logit) are taken - the same choice - and wts
 * is each chosen output's own sigmoid(logit), not renormalised. */
int cvllm_moe_route(const float* logits, int64_t l_stride, const float* correction, int T, int E, int top,
                    int groups, int keep, int mode, int32_t* idx, float* wts, cvllm_stream_t stream);

/* out[t, :] = sum_r wts[t, r] * (idx[t, r] < n_real ? y[pos[t * top + r], :] : h[t, :]) + s_t * shared[t, :]
 * in fp32.  y holds one row per (token, choice) pair with a real expert, at the row pos gives (NULL: the pair's
 * own index); outputs idx >= n_real are identity experts (their output is the input h).  shared may be NULL.
 * s_t = sigmoid(shared_gate[t * gate_stride]) (one fp32 logit per token), or 1 when shared_gate is NULL.
 * wts NULL: every weight is 1 (experts whose weight went into their input, cvllm_scaled_rows). */
int cvllm_moe_combine(const void* y, const int32_t* pos, const float* wts, int top, const int32_t* idx, int n_real,
                      const void* h, const void* shared, const float* shared_gate, int64_t gate_stride, float* out,
                      int64_t rows, int width, int dtype, cvllm_stream_t stream);

/* Expert products for a few tokens without host knowledge of the routing (decode, CUDA graphs): one row per
 * (token, choice) pair p with expert e = idx[p] and input row p / x_div of xs [.., K]:
 *   gated_kind 0 | 1:  out[p, f] = act(w[e, f, :] . x) * w[e, N + f, :] . x,  w [E, 2N, K], act = silu | gelu (tanh)
 *   gated_kind 2:      the clamped gated unit of cvllm_gated_act on the same two products (limit)
 *   gated_kind -1:     out[p, n] = w[e, n, :] . x,                            w [E, N, K]
 * Pairs with e >= n_real are left untouched.  out [pairs, N]. */
int cvllm_expert_gemv(const void* xs, int x_div, const void* w, const int32_t* idx, int n_real, void* out,
                      int pairs, int N, int K, int gated_kind, float limit, int dtype, cvllm_stream_t stream);

/* ------------------------------------------------------------------------
 * Biased attention over the paged cache (csrc/bias_attn.cu): any head size, CVLLM_BF16 or CVLLM_F32 storage,
 * fp32 arithmetic.  score(i, j) = scale * q_i . k_j - slopes[h] * (i - j) for j <= i with
 * floor(i / chunk) == floor(j / chunk) (chunk 0: no chunking; slopes NULL: no bias);
 * p_j = exp(s_j) / (sink * exp(sink_logits[h]) + sum exp(s_j)), sink 0 or 1; sink_logits [H] fp32 is the sink's score
 * per head (not scaled; NULL = 0).  Positions count from the start of each sequence.
 * The cache is the one of the store path: k_cache [rows, D], v_cache [rows, Dv], page_table[slot, head, page]
 * with the two strides given, page_size rows per page.  v_stride (elements between value rows; 0 = Dv) lets the
 * values be a column range of wider rows, e.g. v_cache = k_cache with v_stride = D: the first Dv columns of the keys.
 * --------------------------------------------------------------------- */

/* qkv [T, H*D + G*D + G*Dv] packed rows -> q_out [T, H, D] (per-head RMS norm, weight q_weight [D] or NULL),
 * keys (same norm with k_weight) and values written to the cache row of (token_slot[t], head, positions[t]);
 * bh_lens[slot, head] (may be NULL) is raised to positions[t] + 1.  Tokens of reserved_slot store nothing. */
int cvllm_qknorm_store(const void* qkv, int64_t qkv_stride, const float* q_weight, const float* k_weight,
                       float eps, const int32_t* positions, const int32_t* token_slot, void* q_out,
                       void* k_cache, void* v_cache, const int32_t* page_table, int64_t table_stride_slot,
                       int64_t table_stride_head, int page_size, int32_t* bh_lens, int T, int H, int G, int D,
                       int Dv, int reserved_slot, int dtype, cvllm_stream_t stream);

/* The same with a rotation in front of the norm: inv_freq [rot_dims / 2] doubles (NULL = none); neighbours
 * (2 i, 2 i + 1) of the first rot_dims numbers of every q and k head turn by positions[t] * inv_freq[i].
 * norm 0: no norm at all; 1: the RMS norm above (weights may be NULL). */
int cvllm_rope_qknorm_store(const void* qkv, int64_t qkv_stride, const double* inv_freq, int rot_dims, int norm,
                            const float* q_weight, const float* k_weight, float eps, const int32_t* positions,
                            const int32_t* token_slot, void* q_out, void* k_cache, void* v_cache,
                            const int32_t* page_table, int64_t table_stride_slot, int64_t table_stride_head,
                            int page_size, int32_t* bh_lens, int T, int H, int G, int D, int Dv, int reserved_slot,
                            int dtype, cvllm_stream_t stream);

/* Portions: sequence b brings tokens cu_seqlens_q[b] .. cu_seqlens_q[b+1]-1 at positions seq_start[b] + 0, 1, ...;
 * all their keys (and every earlier one) are in the cache of slot batch_mapping[b].  out [T, H, Dv].
 * max_new = the largest number of new tokens of one sequence, total_tokens = T, cache_rows = rows of k_cache,
 * pages_per_head = the page table's last dimension.  Dv <= 512.
 * Kernels: tcgen05 / TMEM / TMA (bfloat16, D = Dv = 128, page_size % 128 == 0, H / G even, dense page table);
 * mma.sync (bfloat16, D % 16 == 0, Dv % 8 == 0, both <= 128); fp32 FMA (everything else, float32 included). */
int cvllm_bias_attn_varlen(const void* q, const void* k_cache, const void* v_cache, const int32_t* page_table,
                           int64_t table_stride_slot, int64_t table_stride_head, int page_size,
                           const int32_t* cu_seqlens_q, const int32_t* seq_start, const int32_t* batch_mapping,
                           const float* slopes, int chunk, int sink, const float* sink_logits, float scale, void* out,
                           int B, int max_new, int H, int G, int D, int Dv, int total_tokens, int64_t cache_rows,
                           int pages_per_head,
                           int64_t v_stride, int dtype, cvllm_stream_t stream);

/* Decode: one query per sequence at position positions[b] (its key is in the cache already).  q [B, H, D],
 * out [B, H, Dv]; rows of reserved_slot give zeros.  Dv <= 512.  With D and Dv multiples of 8 (and D <= 256) the keys
 * of a sequence are cut into `splits` parts that run on CTAs of their own; splits > 1 needs a workspace of
 * 4 * B * H * splits * (2 + Dv) bytes.  Other sizes run one CTA per (sequence, head) and ignore `splits`. */
int cvllm_bias_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int32_t* page_table,
                           int64_t table_stride_slot, int64_t table_stride_head, int page_size,
                           const int32_t* positions, const int32_t* batch_mapping, const float* slopes, int chunk,
                           int sink, const float* sink_logits, float scale, void* out, int B, int H, int G, int D, int Dv,
                           int reserved_slot,
                           int splits, float* workspace, size_t workspace_bytes, int64_t v_stride, int dtype,
                           cvllm_stream_t stream);

/* The same two with a sliding window and a learned bias per distance beside the linear bias and the chunk mask:
 * a query sees the keys at distances 0 .. window - 1 (window 0: no limit), and the score of the key at distance n
 * gets dist_bias[min(n, dist_rows - 1), h] (fp32 [dist_rows, H]; NULL = none), unscaled.  The caller makes the
 * table, so any rule from distance to bias (buckets of a smaller learned table) is served.  These shapes run on the
 * mma.sync and fp32 FMA kernels. */
int cvllm_bias_attn_varlen_dist(const void* q, const void* k_cache, const void* v_cache, const int32_t* page_table,
                                int64_t table_stride_slot, int64_t table_stride_head, int page_size,
                                const int32_t* cu_seqlens_q, const int32_t* seq_start, const int32_t* batch_mapping,
                                const float* slopes, int chunk, int window, const float* dist_bias, int dist_rows,
                                int sink, const float* sink_logits, float scale, void* out, int B, int max_new, int H,
                                int G, int D, int Dv, int total_tokens, int64_t cache_rows, int pages_per_head,
                                int64_t v_stride, int dtype, cvllm_stream_t stream);
int cvllm_bias_attn_decode_dist(const void* q, const void* k_cache, const void* v_cache, const int32_t* page_table,
                                int64_t table_stride_slot, int64_t table_stride_head, int page_size,
                                const int32_t* positions, const int32_t* batch_mapping, const float* slopes, int chunk,
                                int window, const float* dist_bias, int dist_rows, int sink, const float* sink_logits,
                                float scale, void* out, int B, int H, int G, int D, int Dv, int reserved_slot,
                                int splits, float* workspace, size_t workspace_bytes, int64_t v_stride, int dtype,
                                cvllm_stream_t stream);

/* ------------------------------------------------------------------------
 * Latent attention (csrc/latent_attn.cu): the steps around attention in the latent space.  The cache row of a token
 * is [c | k_rot] (kv_rank + rot_dim numbers, one key/value head).  inv_freq: rot_dim / 2 doubles, base ** (-2 i / rot_dim).
 * --------------------------------------------------------------------- */

/* proj [T, ..] rows hold the query latent at q_off (q_rank numbers) and - kv_off >= 0 - the kv latent followed by the
 * shared key part at kv_off (kv_rank + rot_dim).  cq_out [T, q_rank] = RMS norm(query latent) * q_weight;
 * cache row of (token_slot[t], positions[t]) = [RMS norm(kv latent) * kv_weight | rotate(shared key part)];
 * lens[slot] (may be NULL) is raised to positions[t] + 1.  page_table[slot * table_stride_slot + page].
 * Tokens of reserved_slot store nothing. */
int cvllm_latent_norm_store(const void* proj, int64_t proj_stride, int q_off, int q_rank, int kv_off, int kv_rank,
                            int rot_dim, const float* q_weight, const float* kv_weight, float eps,
                            const double* inv_freq, const int32_t* positions, const int32_t* token_slot, void* cq_out,
                            void* cache, const int32_t* page_table, int64_t table_stride_slot, int page_size,
                            int32_t* lens, int T, int reserved_slot, int dtype, cvllm_stream_t stream);

/* q [T, H, D + rot_dim] (row stride q_stride): q_full[t * full_stride + h * full_head + off + 0 .. rot_dim) =
 * rotate(q[t, h, D .. D + rot_dim)) at positions[t]. */
int cvllm_latent_q_rope(const void* q, int64_t q_stride, int H, int D, int rot_dim, const double* inv_freq,
                        const int32_t* positions, void* q_full, int64_t full_stride, int full_head, int off, int T,
                        int dtype, cvllm_stream_t stream);

/* Gated residual sum fused with the next RMS norm, one launch on a 32-bit residual stream [rows, width]:
 *   resid += sigmoid(gate) * y   (y, gate [rows, width] bfloat16 or float32; both NULL: no sum)
 *   out = resid / sqrt(mean(resid^2) + eps) * w   (out NULL: the sum alone).  Sum and statistics are fp32. */
int cvllm_gated_residual_norm(const void* y, int64_t y_stride, int y_dtype, const void* gate, int64_t g_stride,
                              int g_dtype, float* resid, int64_t r_stride, const float* w, void* out, int64_t o_stride,
                              int out_dtype, int rows, int width, float eps, cvllm_stream_t stream);

/* out = scale * (a / rms(a) * wa + b / rms(b) * wb) per row, rms(v) = sqrt(mean(v^2) + eps); weights fp32. */
int cvllm_dual_norm_blend(const void* a, int64_t a_stride, const float* wa, const void* b, int64_t b_stride,
                          const float* wb, void* out, int64_t o_stride, int rows, int width, float eps, float scale,
                          int dtype, cvllm_stream_t stream);

/* out = act(x) element by element; kind 0: relu(x)^2. */
int cvllm_unary_act(const void* x, int64_t x_stride, void* out, int64_t o_stride, int64_t rows, int F, int kind,
                    int dtype, cvllm_stream_t stream);

/* out = cap * tanh(x / cap), fp32 out (logit soft cap). */
int cvllm_softcap(const void* x, int64_t x_stride, float* out, int64_t o_stride, int64_t rows, int F, float cap,
                  int dtype, cvllm_stream_t stream);

/* out[p, :] = x[pair / top, :] * scale[pair] with pair = perm ? perm[p] : p: rows of (token, choice) pairs multiplied
 * by their routing weight on the way into the experts. */
int cvllm_scaled_rows(const void* x, int64_t x_stride, const int64_t* perm, const float* scale, int top, void* out,
                      int64_t pairs, int width, int dtype, cvllm_stream_t stream);

/* out[t, c] = x[t, c] * sigmoid(gate[t, c]) */
int cvllm_sigmoid_gate(const void* x, int64_t x_stride, const void* gate, int64_t g_stride, void* out,
                       int64_t o_stride, int64_t rows, int width, int dtype, cvllm_stream_t stream);

/* ------------------------------------------------------------------------
 * State-space mixer (csrc/ssm.cu).  A step brings sequence b the tokens cu_seqlens_q[b] .. cu_seqlens_q[b + 1] - 1 at
 * positions seq_start[b] + 0, 1, ..; cu_seqlens_q NULL = one token per sequence at positions[b].  batch_mapping[b] is
 * the sequence's slot of the state pool.  A portion that starts at position 0 starts from a zero state.
 * --------------------------------------------------------------------- */

/* out[t, ch] (fp32) = silu(bias[ch] + sum_k weight[ch, k] * x(t - (taps - 1 - k), ch)) with x = columns x_off.. of proj;
 * inputs before the portion come from conv_state [slots, taps - 1, channels] (zeros before position 0). taps <= 16. */
int cvllm_causal_conv(const void* proj, int64_t proj_stride, int x_off, int channels, int taps, const float* weight,
                      const float* bias, const void* conv_state, const int32_t* cu_seqlens_q,
                      const int32_t* seq_start, const int32_t* positions, const int32_t* batch_mapping, int B,
                      int max_new, float* out, int64_t out_stride, int dtype, cvllm_stream_t stream);

/* The same with a choice of what comes out: mode 0 silu(bias + conv), mode 1 input + bias + conv (the convolution
 * added to its own input, no activation); out_dtype CVLLM_F32 or the inputs' dtype. */
int cvllm_causal_conv_mode(const void* proj, int64_t proj_stride, int x_off, int channels, int taps,
                           const float* weight, const float* bias, const void* conv_state,
                           const int32_t* cu_seqlens_q, const int32_t* seq_start, const int32_t* positions,
                           const int32_t* batch_mapping, int B, int max_new, void* out, int64_t out_stride,
                           int out_dtype, int mode, int dtype, cvllm_stream_t stream);

/* Selective scan with a decay per (channel, state channel): x, dt_raw [T, inner], the columns B | C of bc (N each, at
 * b_off / c_off) and z (at z_off) are stored projections of the model type;
 *   dt = softplus(dt_raw + dt_bias[c]);  S[c, n] <- exp(-exp(A_log[c, n]) dt) S[c, n] + dt x[c] B[n];
 *   out[c] = (sum_n S[c, n] C[n] + D[c] x[c]) * silu(z[c]).   state fp32 [slots, inner, N]. */
int cvllm_selective_scan(const void* x, int64_t x_stride, const void* dt_raw, int64_t dt_stride, const float* dt_bias,
                         const void* bc, int64_t bc_stride, int b_off, int c_off, const float* A_log, const float* D,
                         const void* z, int64_t z_stride, int z_off, float* state, const int32_t* cu_seqlens_q,
                         const int32_t* seq_start, const int32_t* positions, const int32_t* batch_mapping, int B,
                         int max_new, void* out, int64_t out_stride, int inner, int N, int reserved_slot, int dtype,
                         cvllm_stream_t stream);

/* conv_state of every sequence of the step := its last taps - 1 inputs (after cvllm_causal_conv has read the old one). */
int cvllm_conv_state_update(const void* proj, int64_t proj_stride, int x_off, int channels, int taps, void* conv_state,
                            const int32_t* cu_seqlens_q, const int32_t* seq_start, const int32_t* positions,
                            const int32_t* batch_mapping, int B, int reserved_slot, int dtype, cvllm_stream_t stream);

/* xbc [T, heads * P + 2 * groups * N] fp32 = (x | B | C) after the convolution; dt_raw = proj[t, dt_off + h];
 * state [slots, heads, P, N] fp32, read (portions that start after position 0) and written in place;
 * y [T, heads * P] fp32 = S_t C_t + D_h x_t.  N <= 512.  max_new = the longest portion of the step.  Steps whose
 * whole portions would leave half of the SMs idle run the segments (128 tokens or more) of a sequence side by side in
 * three launches (local end states from zero, a combine pass, the rerun with outputs) and need a workspace of
 * cvllm_ssm_scan_workspace_bytes(B, max_new, heads, P, N) bytes (0 for shorter steps). */
size_t cvllm_ssm_scan_workspace_bytes(int B, int max_new, int heads, int P, int N);
int cvllm_ssm_scan(const float* xbc, int64_t xbc_stride, const void* proj, int64_t proj_stride, int dt_off,
                   const float* dt_bias, const float* A_log, const float* D, float* state,
                   const int32_t* cu_seqlens_q, const int32_t* seq_start, const int32_t* positions,
                   const int32_t* batch_mapping, int B, int max_new, float* y, int64_t y_stride, int heads, int groups,
                   int P, int N, int reserved_slot, float* workspace, size_t workspace_bytes, int dtype,
                   cvllm_stream_t stream);

/* out[t, c] = v / sqrt(mean over c's part of v^2 + eps) * weight[c], v = y[t, c] * silu(z[t, c]); `parts` equal parts. */
int cvllm_gated_group_norm(const float* y, int64_t y_stride, const void* z, int64_t z_stride, const float* weight,
                           float eps, void* out, int64_t out_stride, int64_t rows, int width, int parts, int dtype,
                           cvllm_stream_t stream);

/* ------------------------------------------------------------------------
 * Mixers with a [key, value] matrix state per head (csrc/recurrent.cu).  Step geometry as for the state-space mixer.
 * Both recurrences end, inside the kernel, with each head's unit norm, a weight and a gate:
 *   out[t, h * Dv + j] = o / sqrt(mean_j(o^2) + eps) * norm_w[h * norm_head_stride + j] * silu(gate[t, gate_off + h * Dv + j])
 * (norm_head_stride 0: one weight vector shared by the heads).  state [slots, H, Dv, D] fp32 (the key rows of a value
 * column are contiguous).  D, Dv <= 256.
 * --------------------------------------------------------------------- */

/* out[s, t, :] = h[t] + (h[t - 1] - h[t]) * mu[s, :] for s < S (out [S, total_tokens, W], model type, mu fp32 [S, W]);
 * the row before a portion's first comes from shift_state [slots, W] (zeros at position 0), which then takes the
 * portion's last row. */
int cvllm_token_shift_mix(const void* h, int64_t h_stride, const float* mu, int S, int W, void* shift_state,
                          const int32_t* cu_seqlens_q, const int32_t* seq_start, const int32_t* positions,
                          const int32_t* batch_mapping, int B, int max_new, void* out, int64_t total_tokens,
                          int reserved_slot, int dtype, cvllm_stream_t stream);

/* Gated delta rule.  qkv [T, 2 G D + H Dv] fp32 = (q | k | v) after the short convolution; q and k are made unit
 * vectors per head (x / sqrt(sum x^2 + 1e-6)), q times D^-1/2; beta = sigmoid(proj[t, b_off + h]);
 * g = exp(-exp(A_log[h]) * softplus(proj[t, a_off + h] + dt_bias[h])); per head
 *   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.   Head h reads q / k head h / (H / G). */
int cvllm_delta_rule(const float* qkv, int64_t qkv_stride, const void* proj, int64_t proj_stride, int b_off, int a_off,
                     const float* A_log, const float* dt_bias, float* state, const void* gate, int64_t gate_stride,
                     int gate_off, const float* norm_w, int norm_head_stride, float eps, const int32_t* cu_seqlens_q,
                     const int32_t* seq_start, const int32_t* positions, const int32_t* batch_mapping, int B,
                     int max_new, void* out, int64_t out_stride, int H, int G, int D, int Dv, int reserved_slot,
                     int dtype, cvllm_stream_t stream);

/* wkv: r, k, v, w_raw rows of H * D numbers (model type); w = exp(-exp(w_raw + w0)) per head and key channel;
 *   o = (S + diag(bonus_h) k v^T)^T r;  S <- diag(w) S + k v^T.   Dv = D. */
int cvllm_wkv_scan(const void* r, int64_t r_stride, const void* k, int64_t k_stride, const void* v, int64_t v_stride,
                   const void* w_raw, int64_t w_stride, const float* w0, const float* bonus, float* state,
                   const void* gate, int64_t gate_stride, int gate_off, const float* norm_w, int norm_head_stride,
                   float eps, const int32_t* cu_seqlens_q, const int32_t* seq_start, const int32_t* positions,
                   const int32_t* batch_mapping, int B, int max_new, void* out, int64_t out_stride, int H, int D,
                   int reserved_slot, int dtype, cvllm_stream_t stream);

/* General delta rule: r, k, v, removal-rate logits and the gate are columns of proj (model type) at r_off, k_off,
 * v_off, a_off, gate_off (+ h * D); w_raw rows of H * D decay logits: w = exp(-rate * sigmoid(w_raw + w0)).  With the
 * unit key u = k / sqrt(sum k^2 + 1e-6) and a = sigmoid(.) per head and key channel
 *   S <- diag(w) S - (a u)(u^T S) + k v^T   (both terms on the old S);   o = S^T r.   Dv = D.
 * gate_kind 0: the output is multiplied by silu(gate), 1: by sigmoid(gate). */
int cvllm_general_delta(const void* proj, int64_t proj_stride, int r_off, int k_off, int v_off, int a_off,
                        const void* w_raw, int64_t w_stride, const float* w0, float rate, float* state, int gate_off,
                        int gate_kind, const float* norm_w, int norm_head_stride, float eps,
                        const int32_t* cu_seqlens_q, const int32_t* seq_start, const int32_t* positions,
                        const int32_t* batch_mapping, int B, int max_new, void* out, int64_t out_stride, int H, int D,
                        int reserved_slot, int dtype, cvllm_stream_t stream);

/* Matrix memory with exponential gates: q, k (H x D), v, gate (H x Dv) and one input-gate and one forget-gate logit
 * per head are columns of proj at q_off, k_off, v_off, gate_off, i_off + h, f_off + h.  i = cap tanh(z_i / cap),
 * f = logsigmoid(cap tanh(z_f / cap)); with the running maximum m (starts at 0): m' = max(f + m, i),
 *   S <- exp(f + m - m') S + exp(i - m') k v^T,  n likewise with k alone,
 *   o = S^T q / (max(|n . q|, exp(-m')) + 1e-6),   q times q_scale.
 * state [slots, H, Dv, D], nvec [slots, H, D], mstate [slots, H], all fp32. */
int cvllm_matrix_memory(const void* proj, int64_t proj_stride, int q_off, int k_off, int v_off, int i_off, int f_off,
                        float cap, float q_scale, float* state, float* nvec, float* mstate, int gate_off,
                        int gate_kind, const float* norm_w, int norm_head_stride, float eps,
                        const int32_t* cu_seqlens_q, const int32_t* seq_start, const int32_t* positions,
                        const int32_t* batch_mapping, int B, int max_new, void* out, int64_t out_stride, int H, int D,
                        int Dv, int reserved_slot, int dtype, cvllm_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* CVLLM_H_ */
