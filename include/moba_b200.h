/* C ABI of libmoba_b200.so: the sm_100a MoBA sparse-attention kernels.
 *
 * Every entry point takes raw device pointers, explicit sizes and a CUDA stream, allocates
 * nothing, never synchronises the host, and returns an int status (MOBA_OK or a MOBA_ERR_*).
 * The caller owns every buffer, so a sequence of calls can be captured in a CUDA graph, and the
 * entry points of this header keep no mutable state between calls (moba_prefill_route_static, which
 * says so, is the one exception).  Profiling and self-test hooks, which do keep process-wide
 * state, are declared apart in moba_b200_debug.h.
 */
#ifndef MOBA_B200_H_
#define MOBA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  MOBA_OK = 0,
  MOBA_ERR_INVALID = 1,     /* an argument violates the documented contract            */
  MOBA_ERR_CUDA = 2,        /* a CUDA runtime call or launch failed                      */
  MOBA_ERR_WORKSPACE = 3,   /* the workspace passed is smaller than *_workspace_bytes()  */
  MOBA_ERR_UNSUPPORTED = 4  /* shape outside the compiled envelope                       */
};

/* Human-readable text for a status code (static storage). */
const char* moba_status_string(int status);

/* sizeof the descriptor structs below as the library was compiled (which = 0: moba_prefill_desc, 1: moba_cache_desc;
 * 0 otherwise), so that a binding in another language can check its mirror of them when it loads the library. No
 * counterpart in the reference, whose operators take tensors. */
size_t moba_abi_sizeof(int which);

/* ---------------------------------------------------------------------------------------------
 * Prefill: MoBA attention over a packed (varlen) batch, forward and backward.
 *
 * Replaces the device work behind opt_gqa_cuda (src/moba_opt/grouped_attention.py:29-99 of the
 * reference): routing (:48-71), expert packing (:76-94), the two FlashAttention calls and the LSE
 * merge of OptMixedAttention.forward (src/moba_opt/mixed_attention.py:43-139, ops/merge.cu:27-288)
 * and OptMixedAttention.backward (mixed_attention.py:141-225).
 *
 * Layout: q [T,Hq,D], k/v [T,Hkv,D] bf16 (fp16 with MOBA_INPUT_FP16) with element strides given in the descriptor (last
 * dimension contiguous, strides multiples of 8 elements, base pointers 16-byte aligned);
 * out [T,Hq,D] in the input format, contiguous; lse [T,Hq] fp32 (natural log).
 * The int32 metadata arrays are device pointers built by the host from cu_seqlens:
 *   chunk_start[n+1], chunk_seq[n], chunk_local[n]   (chunking of src/moba_opt/diagnostic.py:30-80)
 *   qtile_chunk/qtile_tok0/qtile_local[num_qtiles]   128-token query tiles that never cross a chunk;
 *                                                    qtile_local = chunk_local * ceil(C/128) + tile in chunk
 *   self_pairs[num_self_pairs]                       first tile of every pair of consecutive query tiles of a
 *                                                    chunk (tiles 2i and 2i+1 of the chunk; the second may be
 *                                                    missing), by decreasing causal work
 *   kv_order[num_qtiles]                             the same tiles seen as key blocks, earliest chunk of a
 *                                                    sequence first (those are routed to most often)
 * remote_k = min(topk-1, number of routable chunks); remote_k == 0 selects nothing (the caller
 * expresses the dense fallback of grouped_attention.py:41-46 by passing chunk_size >= max_seqlen).
 */
#define MOBA_ROUTE_BF16_MEANS 1
#define MOBA_BWD_DETERMINISTIC 2
#define MOBA_INPUT_FP16 4

typedef struct moba_prefill_desc {
  int32_t total_tokens, num_seqs, hq, hkv, dim, chunk_size, remote_k;
  int32_t num_chunks, num_qtiles, max_tiles_per_seq, max_chunks_per_seq;
  int32_t flags; /* MOBA_ROUTE_BF16_MEANS: round chunk means to the input format (route_precision='upstream');
                    MOBA_BWD_DETERMINISTIC: dQ summed in 64-bit fixed point, bit-repeatable (needs the larger scratch
                    moba_prefill_bwd_scratch_bytes reports for a descriptor with the flag set);
                    MOBA_INPUT_FP16: q, k, v, dout, out and the gradients are IEEE half instead of bf16 (both are
                    accepted by baseline_adapter.py:13); everything else about the call is the same */
  int32_t num_self_pairs, reserved0;
  int64_t q_stride_t, q_stride_h, k_stride_t, k_stride_h, v_stride_t, v_stride_h;
  const int32_t* cu_seqlens;
  const int32_t* chunk_start;
  const int32_t* chunk_seq;
  const int32_t* chunk_local;
  const int32_t* qtile_chunk;
  const int32_t* qtile_tok0;
  const int32_t* qtile_local;
  const int32_t* self_pairs;
  const int32_t* kv_order;
} moba_prefill_desc;

/* Bytes of the state kept from forward to backward (route lists written by moba_prefill_route, followed by
 * packed operand tiles written by moba_prefill_fwd) and of the routing scratch. The state is required for
 * every call, also when remote_k == 0. */
size_t moba_prefill_route_state_bytes(const moba_prefill_desc* d);
size_t moba_prefill_route_scratch_bytes(const moba_prefill_desc* d);

/* Routing (grouped_attention.py:48-94, route_precision='fp32', stable_routes=True). The route state
 * starts with sel[T,Hq,remote_k] int32: global chunk ids per (token, query head), ascending, -1 padded. */
int moba_prefill_route(const moba_prefill_desc* d, const void* q, const void* k, void* route_state, void* scratch,
                       size_t scratch_bytes, void* stream);

/* Routing without a caller-provided scratch buffer. This entry point has no counterpart in the
 * reference. It is for callers that cannot allocate device memory themselves (all memory reserved by
 * one pool at start-up, cudaMalloc forbidden on the request path, or a language binding that only
 * holds tensors it was given): the routing scratch is a fixed array of
 * MOBA_ROUTE_STATIC_SCRATCH_BYTES inside the library, held on every GPU that loads the library until
 * the process exits. Same inputs, outputs and results as moba_prefill_route; it allocates nothing.
 *   - Returns MOBA_ERR_WORKSPACE when moba_prefill_route_scratch_bytes(d) exceeds the array.
 *   - The first call on each device looks up the array's device address (with that device current);
 *     make that first call before starting any stream capture.  The address is remembered per device
 *     ordinal for the life of the process: a process that destroys its CUDA context and creates a new
 *     one must not call this entry point again afterwards (a new context may place the array elsewhere).
 *   - All calls on a device share the one array: two calls whose kernels may overlap on the GPU
 *     (different streams, no ordering between them) race. Order them, or use moba_prefill_route. */
#define MOBA_ROUTE_STATIC_SCRATCH_BYTES (8u << 20)
size_t moba_prefill_route_static_capacity(void);
int moba_prefill_route_static(const moba_prefill_desc* d, const void* q, const void* k, void* route_state, void* stream);

/* Forward attention + LSE merge (mixed_attention.py:43-139). status: device uint32 error bits (0 = clean). */
size_t moba_prefill_fwd_scratch_bytes(const moba_prefill_desc* d);
int moba_prefill_fwd(const moba_prefill_desc* d, const void* q, const void* k, const void* v, const void* route_state,
                     void* scratch, size_t scratch_bytes, void* out, float* lse, unsigned* status, void* stream);

/* Backward (mixed_attention.py:141-225): gradients of out w.r.t. q, k, v with the route held fixed.
 * dq [T,Hq,D], dk/dv [T,Hkv,D] in the input format, contiguous.  dK, dV are bit-repeatable; dQ is summed over key blocks with FP32
 * reductions in arrival order unless d->flags has MOBA_BWD_DETERMINISTIC (the reference's deterministic=True,
 * mixed_attention.py:185,220), which sums 64-bit fixed-point values instead: about twice the backward kernel's time and a
 * scratch twice the size. */
size_t moba_prefill_bwd_scratch_bytes(const moba_prefill_desc* d);
int moba_prefill_bwd(const moba_prefill_desc* d, const void* q, const void* k, const void* v, const void* out,
                     const float* lse, const void* dout, const void* route_state, void* scratch, size_t scratch_bytes,
                     void* dq, void* dk, void* dv, unsigned* status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Decode: paged KV cache, block routing and attention for single-token queries.
 *
 * Replaces the Triton kernels behind PagedKVCache / PreparedDecode of the reference
 * (src/moba_opt/ops/paged_decode.py:11-144, src/moba_opt/ops/prepared_decode.py:7-94) and the
 * torch.topk of src/moba_opt/kv_cache.py:208-223. The cache pools stay owned by the caller:
 *   k_cache, v_cache [num_pages, page_size, hkv, dim] 16-bit    table   [batch_slots, table_width] int32 (-1 unmapped)
 *   means [batch_slots, max_chunks, hkv, dim] 16-bit             lengths [batch_slots] int32
 * dim must be a multiple of 8 (<= 256). All functions enqueue on `stream` and return.
 */
#define MOBA_CACHE_FP16 1

typedef struct moba_cache_desc {
  int32_t batch_slots, max_seq_len, page_size, num_pages, table_width, chunk_size, max_chunks, hkv, dim;
  int32_t flags; /* MOBA_CACHE_FP16: pools, means, q, k, v and out are IEEE half instead of bf16 (the reference's cache
                    takes both, src/moba_opt/kv_cache.py:65); the fused q/k/v projection input of
                    moba_decode_step_begin is bf16 only */
  void* k_cache;
  void* v_cache;
  int32_t* table;
  int32_t* lengths;
  void* means;
} moba_cache_desc;

/* Per-step metadata (ops/prepared_decode.py:7-20): for row i with sequence ids[i], write
 * table[ids[i]][delta[i]] = delta[rows+i] when delta[i] >= 0 (idempotent), then
 * append != 0: positions[i] = lengths[ids[i]]++ ; append == 0: positions[i] = lengths[ids[i]] - 1. */
int moba_decode_metadata(const moba_cache_desc* c, const int32_t* ids, int32_t* positions, const int32_t* delta, int rows,
                         int append, void* stream);

/* Applies host-planned changes to the device copies of the page table and the lengths, the changed entries only
 * (the reference re-uploads the whole [batch, width] table and the lengths on every append and reset,
 * src/moba_opt/kv_cache.py:112-126): edits [n][3] = (sequence, logical page, physical page), then
 * lengths[ids[j]] = lengths_new[j] for j < m.  clear_rows != 0 (with n == 0) unmaps the whole row of every listed
 * sequence first: a reset. */
int moba_cache_update(const moba_cache_desc* c, const int32_t* edits, int n, const int32_t* ids, const int32_t* lengths_new, int m,
                      int clear_rows, void* stream);

/* Scatter k, v [tokens, hkv, dim] (contiguous) to (table[token_seq[t]][token_pos[t]/page], token_pos[t]%page)
 * (ops/paged_decode.py:11-23). */
int moba_decode_append(const moba_cache_desc* c, const void* k, const void* v, const int32_t* token_seq,
                       const int32_t* token_pos, int tokens, unsigned* status, void* stream);

/* Chunk means, FP32 sum / chunk_size rounded to the cache's format (ops/paged_decode.py:27-44). predicated == 0: item i is
 * (seqs[i], chunk chunk_or_pos[i]). predicated != 0: chunk_or_pos holds the position of the token just
 * appended to seqs[i]; the mean of its chunk is written only if that token completed the chunk
 * (ops/prepared_decode.py:24-41). */
int moba_decode_means(const moba_cache_desc* c, const int32_t* seqs, const int32_t* chunk_or_pos, int items, int predicated,
                      unsigned* status, void* stream);

/* Prefill hand-off: appends whole prompts, k, v [tokens, hkv, dim] packed by cu_seqlens [num_seqs + 1], to sequences
 * seqs[i] at positions start[i] .. and writes the mean of every chunk the append completes, in one launch and one
 * pass over K (the reference appends per layer with cache.append after the prefill attention, examples/full_qwen2.py:109,
 * kv_cache.py:172-191: a scatter over per-token index arrays, then a second pass for the means).  The page table must
 * already map the new positions.  max_chunks_touched >= the largest number of chunks one sequence's new tokens fall
 * into.  Means are bit-identical to moba_decode_means. */
int moba_prefill_to_cache(const moba_cache_desc* c, const void* k, const void* v, const int32_t* seqs, const int32_t* start,
                          const int32_t* cu_seqlens, int num_seqs, int max_chunks_touched, unsigned* status, void* stream);

/* Copies a step's q, k, v into the fixed buffers a captured step reads (prepared_decode.py:150-176 of the reference
 * does three tensor copies), as one launch.  Sizes in bytes, multiples of 16, pointers 16-byte aligned
 * (MOBA_ERR_UNSUPPORTED otherwise: copy some other way); a size of 0 skips that tensor. */
int moba_decode_stage_inputs(void* q_dst, const void* q_src, size_t q_bytes, void* k_dst, const void* k_src, size_t k_bytes,
                             void* v_dst, const void* v_src, size_t v_bytes, void* stream);

/* First launch of an appending decode step: moba_decode_metadata (append != 0), moba_decode_append of one token per
 * row and the predicated moba_decode_means in one launch, one CTA per row (ops/prepared_decode.py:7-41 are three
 * kernels).  With qkv == NULL, k and v [rows, hkv, dim] are inputs.  With qkv [rows, (hq + 2 hkv) * dim] (the fused
 * projection of the new token), the launch also applies the rotate-half rotary embedding with cos, sin [rows, dim]
 * to the query and key heads and writes q [rows, hq, dim], k, v [rows, hkv, dim] before appending.
 * positions is read before it is written (the previous step's position is a hint for the page of the new token): it is
 * in/out, must be readable memory, and may hold anything before the first step (the hint is range-checked). */
int moba_decode_step_begin(const moba_cache_desc* c, const int32_t* ids, int32_t* positions, const int32_t* delta, int rows,
                           int hq, const void* qkv, const void* cosv, const void* sinv, void* q, void* k, void* v,
                           unsigned* status, void* stream);

/* Routing (ops/paged_decode.py:48-64 scores; ops/prepared_decode.py:45-55,78-94 selection): q [rows,hq,dim];
 * scores [rows,hq,width] fp32 (may be null), -inf for chunks not completed before the query's chunk;
 * selected [rows,hq,1+remote] int32 = (pos/chunk_size, picks in descending score order with the lowest chunk
 * winning exact ties, -1 padding). Also writes the per-(row, kv head) union of attended chunks for
 * moba_decode_attend: u_chunk/u_mask [rows,hkv,umax], u_count [rows,hkv], umax = moba_decode_union_capacity(). */
int moba_decode_union_capacity(int hq, int hkv, int remote, int width);
int moba_decode_route(const moba_cache_desc* c, const void* q, const int32_t* ids, const int32_t* positions, int rows, int hq,
                      int remote, int width, float* scores, int32_t* selected, int32_t* u_chunk, uint32_t* u_mask,
                      int32_t* u_count, void* stream);

/* Attention (ops/paged_decode.py:68-112): per (row, query head) softmax over the tokens <= positions[row] of the
 * listed chunks (selected != null, slots = 1+remote) or of the whole prefix (selected == null, slots =
 * max_chunks); out [rows,hq,dim] in the cache's format, lse [rows,hq] fp32 natural log. The workspace starts with one int32
 * counter per (row, kv head) that must be zero before the first call; the kernel leaves it zero. */
size_t moba_decode_attend_workspace_bytes(const moba_cache_desc* c, int rows, int hq, int slots);
int moba_decode_attend(const moba_cache_desc* c, const void* q, const int32_t* ids, const int32_t* positions, int rows, int hq,
                       const int32_t* selected, int slots, const int32_t* u_chunk, const uint32_t* u_mask,
                       const int32_t* u_count, int umax, void* workspace, size_t workspace_bytes, void* out, float* lse,
                       unsigned* status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Standalone merge operator: replaces merge_forward of the reference (src/moba_opt/ops/bindings.cpp:6-22,
 * wrapper src/moba_opt/ops/merge_cuda.py:32-60, kernels ops/merge.cu:27-288) for callers that hold the self
 * branch and the scattered remote contributions themselves; the prefill path merges in its own epilogue.
 *   self_out [rows, dim], self_lse [rows]; remote_out [remote_rows, dim], remote_lse [remote_rows];
 *   mapping [remote_rows] int64: the row each contribution belongs to; at most kmax (<= 32) per row.
 *   dtype: 0 = bf16, 1 = fp32, 2 = fp16 (of self_out, remote_out and out); LSE is fp32 natural log.
 * Contributions are reduced in ascending index order, so the result is bit-repeatable. status bits: 2 = a
 * mapping entry was out of range (skipped), 4 = a row had more than kmax contributions (the excess is skipped). */
size_t moba_merge_scratch_bytes(long long rows, int kmax);
int moba_merge_forward(const void* self_out, const float* self_lse, const void* remote_out, const float* remote_lse,
                       const int64_t* mapping, long long rows, long long remote_rows, int dim, int kmax, int dtype,
                       void* scratch, size_t scratch_bytes, void* out, float* lse, unsigned* status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Layer glue of the full-model decode step (no reference counterpart: examples/full_qwen2.py of the reference
 * leaves these operations to the Hugging Face modules).  bf16 tensors, rows contiguous; arithmetic rounds to
 * bf16 wherever those modules do, so the fused step reproduces their bits.
 *   moba_add_rmsnorm  h_out = h_in + delta (delta and h_out may be null), y = weight * rmsnorm(h_out)
 *   moba_rope_split   qkv [rows, (hq + 2 hk) * dim] -> q, k with rotate-half rotary embedding (cos, sin [rows, dim]), v
 *   moba_silu_mul     gate_up [rows, 2 ffn] (gate then up) -> out [rows, ffn] = silu(gate) * up */
int moba_add_rmsnorm(const void* h_in, const void* delta, const void* weight, float eps, long long rows, int hidden, void* h_out,
                     void* y, void* stream);
int moba_rope_split(const void* qkv, const void* cosv, const void* sinv, long long rows, int hq, int hk, int dim, void* q, void* k,
                    void* v, void* stream);
int moba_silu_mul(const void* gate_up, long long rows, int ffn, void* out, void* stream);

/* Inputs of a decode step in one launch: h [rows, hidden] = embedding[tokens[i]] and the rotary table of each row's
 * position, cos / sin [rows, dim] = cos / sin(positions[i] * inv_freq[d mod dim/2]) * scaling, FP32 arithmetic rounded
 * to bf16 (the default-type rotary module of Hugging Face, which the reference's session calls:
 * examples/full_qwen2.py:160-170).  tokens int64, positions int32, both on the device. */
int moba_decode_step_inputs(const int64_t* tokens, const void* embedding, int hidden, const int32_t* positions,
                            const float* inv_freq, float scaling, int dim, long long rows, void* h, void* cosv, void* sinv,
                            void* stream);

/* Greedy token of a decode step: index of the largest of n bf16 logits, the lowest index among equal maxima (NaN never
 * wins), written as int64 to out.  workspace: moba_argmax_workspace_bytes() bytes, 16-byte aligned, zeroed once
 * before the first call (the kernel leaves it ready for the next); logits 16-byte aligned.  The reference takes
 * logits.argmax on the host side of its greedy loop (scripts/evaluate_full_model.py:283-288). */
size_t moba_argmax_workspace_bytes(void);
int moba_argmax_bf16(const void* logits, int n, void* workspace, size_t workspace_bytes, int64_t* out, void* stream);

/* Linear layer of a one-token decode step: y [n] = weight [n, k] x (+ bias), bf16 in and out, FP32 accumulation; the
 * weight is read once with all loads of a thread in flight, which is what bounds a batch-1 step.
 *   input: either x [k], or h_in [k] with norm_weight [k] (then x = norm_weight * rmsnorm(h_in + delta, eps), delta
 *          may be null, and h_out, if given, receives h_in + delta: the residual add and the RMSNorm that precede the
 *          projection in the layer run inside the same launch; h_out must not be h_in or delta - every CTA re-reads
 *          those while one writes h_out - and equal pointers are refused with MOBA_ERR_INVALID);
 *   epilogue 0: y [n] = W x + bias (bias may be null);
 *   epilogue 1: weight is [2 n, k], gate rows then up rows, y [n] = silu(gate) * up (no bias).
 * k a multiple of 8, at most 16384 (8192 with epilogue 1); weight and x 16-byte aligned.  No reference counterpart
 * (the reference's session calls the Hugging Face modules: examples/full_qwen2.py:76-90, 160-190). */
int moba_decode_linear(const void* x, const void* h_in, const void* delta, const void* norm_weight, float eps, void* h_out,
                       const void* weight, const void* bias, int k, int n, int epilogue, void* y, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOBA_B200_H_ */
