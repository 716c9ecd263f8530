/*
 * hkb -- C ABI of the B200 (sm_100a) paged-KV hot path: the KV-cache write
 * (reshape_and_cache) and paged GQA decode attention over block tables, with
 * split-KV partials and an LSE merge.
 *
 * This is the boundary a host binds to (ctypes, cffi, cgo, JNI ...). It takes
 * plain pointers and sizes only: no C++ types, no torch types, no exceptions.
 *
 * Conventions that hold for every entry point
 *   - every pointer is a BORROWED DEVICE pointer of the current CUDA device,
 *     valid until the stream reaches the launch; the library allocates and
 *     frees nothing;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 *     stream); launches are asynchronous and never synchronise with the host;
 *     hkb_reshape_and_cache, hkb_paged_decode and hkb_merge can be captured into
 *     a CUDA graph;
 *   - the return value is an hkb_status: 0 on success, a negative code for a
 *     refused argument (nothing was launched), HKB_ERR_CUDA for a CUDA launch
 *     error. Nothing aborts and nothing throws;
 *   - re-entrant: the only state is a per-device read-only attribute cache -- except where an
 *     entry point says otherwise (hkb_paged_decode_static shares one built-in array a device;
 *     hkb_decode_step with `arrivals` keeps counters in the caller's array).
 *   - strides are in ELEMENTS of the tensor's own type; head_dim is contiguous.
 *
 * What each entry point stands in for in hk-dsl (paths are the reference's):
 * see the comment above each declaration.
 */
#ifndef HKB_H_
#define HKB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HKB_VERSION 122 /* major*100 + minor */

/* KV element types (kv_dtype). Queries, new K/V rows and outputs are bf16, except with HKB_KV_F16. */
#define HKB_KV_BF16 0
#define HKB_KV_FP8_E4M3 1
/* float16 throughout: the cache, the new K/V rows, the query and the output are all fp16 (a model
 * served in float16; the reference's `_f16` kernel variants, python/hk/ops/paged.py:706-729). */
#define HKB_KV_F16 2

typedef enum {
  HKB_OK = 0,
  HKB_ERR_NULL = -1,        /* a required pointer is NULL */
  HKB_ERR_HEAD_DIM = -2,    /* head_dim not one of 64, 128, 256 */
  HKB_ERR_BLOCK_SIZE = -3,  /* block_size not a positive multiple of 16 */
  HKB_ERR_GROUP = -4,       /* q heads not a multiple of kv heads, or group > 16 */
  HKB_ERR_DTYPE = -5,       /* kv_dtype not HKB_KV_* */
  HKB_ERR_STRIDE = -6,      /* a stride breaks 16-byte alignment of a row */
  HKB_ERR_ALIGN = -7,       /* a base pointer is not 16-byte aligned */
  HKB_ERR_SPLITS = -8,      /* num_splits < 1, > HKB_MAX_SPLITS, or scratch missing */
  HKB_ERR_SIZE = -9,        /* a count is negative or a grid limit is exceeded */
  HKB_ERR_SCALE = -10,      /* fp8 cache without k_scale / v_scale */
  HKB_ERR_UNSUPPORTED = -11,/* a combination this build has no kernel for */
  HKB_ERR_STATIC_SCRATCH = -12, /* the split partials would not fit the library's built-in scratch */
  HKB_ERR_CUDA = -100       /* CUDA reported an error at launch (see hkb_last_cuda_error) */
} hkb_status;

#define HKB_MAX_SPLITS 256
#define HKB_MAX_GROUP 16

/*
 * One paged cache tensor (K or V) by base pointer and strides, so the same
 * kernels read hk's head-major pages (blocks, kv_heads, block, head_dim), vLLM's
 * (blocks, block, kv_heads, head_dim) views, and K|V side by side in one tensor
 * (python/hk/integration/vllm_backend.py:603-611, vllm_prefill.py:599-628).
 */
typedef struct {
  void* ptr;
  int64_t stride_block; /* elements between consecutive blocks */
  int64_t stride_token; /* elements between consecutive tokens of a block */
  int64_t stride_head;  /* elements between consecutive kv heads */
  int64_t num_blocks;   /* blocks in the pool; page ids are clamped to it */
} hkb_cache_t;

/*
 * The KV-cache write. For every token t with slot = slot_mapping[t] >= 0 (and
 * below num_blocks*block_size): cache[slot / block_size, slot % block_size, h, :]
 * = key[t, h, :] (value likewise); a negative slot -- a CUDA graph's padding
 * token -- is skipped. bf16 caches take the bits unchanged; fp8-e4m3 caches take
 * RNE(float(x) / scale) saturated to +-448. Duplicate live slots in one call race.
 *
 * Replaces: vllm._custom_ops.reshape_and_cache_flash as called from
 * python/hk/integration/vllm_backend.py:582-599 (argument order pinned by
 * tests/hk/engines/test_vllm_contract.py:271-277); same semantics as the torch
 * scatter of tests/hk/gpu/test_vllm_backend_decode.py:44-49 and the DSL scatter
 * of examples/09_kv_scatter.py:20-25.
 *
 * key/value: [num_tokens, num_kv_heads, head_dim] bf16 with the given token and
 * head strides. slot_mapping: int64 (slot_is_i64 != 0) or int32. k_scale/v_scale:
 * device pointers to one float each (required for fp8, ignored for bf16).
 */
int hkb_reshape_and_cache(const void* key, const void* value,
                          int64_t key_stride_tok, int64_t key_stride_head,
                          int64_t val_stride_tok, int64_t val_stride_head,
                          hkb_cache_t k_cache, hkb_cache_t v_cache,
                          const void* slot_mapping, int slot_is_i64,
                          int num_tokens, int num_kv_heads, int head_dim, int block_size,
                          int kv_dtype, const float* k_scale, const float* v_scale,
                          void* stream);

/*
 * The decode walk: one CTA per (sequence, kv head, kv split). Sequence i reads
 * tokens [0, seq_lens[i]) through block_table[i, :], query head h reads kv head
 * h / (num_q_heads / num_kv_heads).
 *
 *   num_splits == 1: writes out[i, h, :] = softmax(q k^T * scale) v as bf16.
 *   num_splits  > 1: split s of sequence i covers a contiguous range of 16-token
 *     tiles and writes its NORMALISED partial to part_out[(i*num_splits+s), h, :]
 *     (fp32) and part_lse[(i*num_splits+s), h] = natural-log sum-exp of its scaled
 *     scores (-inf for a split with no tokens); hkb_merge folds them.
 *
 * seq_lens[i] <= 0 (a padded request) reads no KV and answers zeros. If q_start
 * is not NULL it is cu_seqlens_q (num_seqs+1 int32): sequence i's query row is
 * q_start[i], and a sequence with q_start[i+1] <= q_start[i] writes nothing.
 * fp8 caches are dequantised in the load: k_scale multiplies the scores and
 * v_scale the output.
 *
 * Replaces: paged_decode_fused_kernel / paged_decode_split_kernel
 * (python/hk/ops/paged.py:498-667, 171-280), paged_decode.walk_kernel
 * (python/hk/ops/paged_decode.py:61-440) and paged_cdna.decode_kernel
 * (python/hk/ops/paged_cdna.py:113-393), as launched from
 * python/hk/integration/vllm_backend.py:222-232 and vllm_prefill.py:1042-1065.
 *
 * q/out: [rows, num_q_heads, head_dim] bf16. block_table: int32, table_stride
 * elements per row, max_pages valid columns. scale: softmax scale.
 */
int hkb_paged_decode(void* out, int64_t out_stride_tok, int64_t out_stride_head,
                     const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                     hkb_cache_t k_cache, hkb_cache_t v_cache,
                     const int32_t* block_table, int64_t table_stride, int max_pages,
                     const int32_t* seq_lens, const int32_t* q_start,
                     int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                     int block_size, float scale, int kv_dtype,
                     const float* k_scale, const float* v_scale,
                     int num_splits, float* part_out, float* part_lse,
                     void* stream);

/*
 * The walk of hkb_paged_decode with stages left out, for attribution measurements: time it with
 * one stage missing and the difference to the whole walk is what the stage costs. `ablate` is a
 * mask: 1 page-table reads, 2 the K copies, 4 the V copies, 8 the q.K products, 16 the softmax
 * (maximum, exponential, sum), 32 the p.V products; the masks built are each bit alone, 2|4 (no
 * copies) and 8|16|32 (no math); 0 is hkb_paged_decode itself. Only the headline shape is built
 * (head_dim 128, bf16 cache, a GQA group of 4 to 8, num_splits > 1): anything else answers
 * HKB_ERR_UNSUPPORTED. What it writes into part_out / part_lse is meaningless.
 *
 * Replaces: the `ablate=` switches of the reference's fused walk (python/hk/ops/paged.py:524-533)
 * and the table tools/hk-bench/paged_attrib.py builds from them.
 */
int hkb_paged_decode_ablate(void* out, int64_t out_stride_tok, int64_t out_stride_head,
                            const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                            hkb_cache_t k_cache, hkb_cache_t v_cache,
                            const int32_t* block_table, int64_t table_stride, int max_pages,
                            const int32_t* seq_lens, const int32_t* q_start,
                            int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                            int block_size, float scale, int kv_dtype,
                            const float* k_scale, const float* v_scale,
                            int num_splits, float* part_out, float* part_lse, int ablate, void* stream);

/*
 * The LSE merge: out[i, h, :] = sum_p w_p * part_out[p, i, h, :] / sum_p w_p with
 * w_p = exp(part_lse[p, i, h] - max_p part_lse). A part whose lse is -inf is
 * never read (its memory may hold anything); if every part is -inf the answer is
 * zero. Also folds the partials of several GPUs after an all-gather: a part is
 * then one rank's (out, lse). If out_lse is not NULL the merged natural-log lse
 * is written to out_lse[i, h]. out_is_f32 says what `out` holds: 0 bf16, 1 fp32 (so a
 * rank's local merge can feed a second, cross-GPU merge), 2 fp16.
 *
 * part_out element (p, i, h, d) is at p*part_stride_p + i*part_stride_seq +
 * h*head_dim + d; part_lse (p, i, h) at p*lse_stride_p + i*lse_stride_seq + h.
 * seq_lens may be NULL; otherwise sequences with seq_lens[i] <= 0 answer zeros.
 * q_start as in hkb_paged_decode.
 *
 * Replaces: paged_merge_kernel / _merge_splits (python/hk/ops/paged.py:394-495),
 * the torch merge_splits (paged.py:283-317), paged_decode.merge_kernel_def
 * (python/hk/ops/paged_decode.py:443-537), paged_cdna.merge_kernel
 * (python/hk/ops/paged_cdna.py:439-560).
 */
int hkb_merge(void* out, int64_t out_stride_tok, int64_t out_stride_head, int out_is_f32,
              float* out_lse,
              const float* part_out, int64_t part_stride_p, int64_t part_stride_seq,
              const float* part_lse, int64_t lse_stride_p, int64_t lse_stride_seq,
              int num_parts, int num_seqs, int num_q_heads, int head_dim,
              const int32_t* seq_lens, const int32_t* q_start, void* stream);

/*
 * Paged prefill: causal attention of each request's new tokens over its paged KV cache
 * (cached prefix + the new tokens, already written by hkb_reshape_and_cache). Request r has
 * q_start[r+1] - q_start[r] query rows and seq_lens[r] tokens in the cache; its query row i
 * sits at position seq_lens[r] - q_len + i and sees keys 0..that position.
 *
 * `work` is a device array of num_work (request, first row) int32 pairs, one a query tile of
 * hkb_prefill_tile_rows(num_q_heads, num_kv_heads) rows (the host builds it: query lengths
 * are host values in a prefill step; put long tiles first). Rows of requests that are not in
 * the work list are not written. bf16 caches, or fp8-e4m3 with per-tensor k_scale / v_scale
 * (device pointers to one float each). num_tokens: the rows q and out hold
 * (q_start[last request + 1] at least): the tensor-memory kernel fetches query tiles with TMA and
 * must know where the tensor ends.
 *
 * Replaces: paged_prefill_kernel and its work list (python/hk/ops/paged_prefill.py:59-620,
 * 879-968) as launched from python/hk/integration/vllm_backend.py:667-698.
 */
int hkb_paged_prefill(void* out, int64_t out_stride_tok, int64_t out_stride_head,
                      const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                      hkb_cache_t k_cache, hkb_cache_t v_cache,
                      const int32_t* block_table, int64_t table_stride, int max_pages,
                      const int32_t* seq_lens, const int32_t* q_start,
                      const int32_t* work, int num_work, int num_tokens,
                      int num_q_heads, int num_kv_heads, int head_dim, int block_size,
                      float scale, int kv_dtype, const float* k_scale, const float* v_scale,
                      void* stream);

/*
 * One decode step -- the cache write of the step's new token of every sequence, the walk
 * and the merge -- in fewer launches than hkb_reshape_and_cache + hkb_paged_decode +
 * hkb_merge: two (the walk writes the new rows itself; then the merge kernel), or one when
 * `arrivals` is given (the walk also folds the partials). Where the shape does not allow it
 * (one split, more than 2048 sequences) the three separate launches run. `out` holds the
 * final bf16 answer either way, and the cache holds the new rows. Every refusal -- the cache
 * write's, the walk's and the merge's -- is returned before the first launch.
 *
 * key / value: the new rows, bf16, one row a sequence (row of sequence i = q_start[i], or i
 * when q_start is NULL -- the row of its query; with q_start, row i must belong to sequence
 * i, as in a decode-only batch), strides in elements; slot_mapping[row] is where the row
 * goes, and must address position seq_lens[i] - 1 of sequence i (what a decode step's slot
 * mapping is) or be negative (skipped). key == value == NULL: the cache is already written.
 *
 * The ring of the walk that owns a sequence's last tile writes the new row into the cache
 * before it fetches that tile; no other ring of that kv head reads the tile.
 *
 * arrivals (optional): hkb_arrivals_bytes(num_seqs, num_kv_heads) bytes of int32 counters,
 * ZERO before the first call; every call leaves them zero. One array a stream: two steps in
 * flight at once must not share it (nor the scratch). With it the ring that finishes the last
 * outstanding piece of a sequence folds its partials -- no ring waits for another -- as a
 * two-level tree of 16-way folds, so results may differ from hkb_merge's in the last fp32
 * bits when a sequence has more than 16 pieces (identical otherwise). One warp folds where
 * the merge kernel uses a grid: measured on B200 this form is slower than the merge launch
 * it saves except for small, evenly cut batches, which is why it is opt-in.
 *
 * Replaces: the backend's decode step, _update_cache + two launches
 * (python/hk/integration/vllm_backend.py:582-599, 700-729); joining them is what
 * docs/history/17-the-decode-step-captured-whole.md:181-188 leaves as future work.
 */
int hkb_decode_step(void* out, int64_t out_stride_tok, int64_t out_stride_head,
                    const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                    const void* key, const void* value,
                    int64_t key_stride_tok, int64_t key_stride_head,
                    int64_t val_stride_tok, int64_t val_stride_head,
                    const void* slot_mapping, int slot_is_i64,
                    hkb_cache_t k_cache, hkb_cache_t v_cache,
                    const int32_t* block_table, int64_t table_stride, int max_pages,
                    const int32_t* seq_lens, const int32_t* q_start,
                    int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                    int block_size, float scale, int kv_dtype,
                    const float* k_scale, const float* v_scale,
                    int num_splits, float* part_out, float* part_lse, int32_t* arrivals, void* stream);

/*
 * The same step for ONE RANK of a KV axis cut across GPUs: the walk over this rank's tokens
 * (writing the step's new rows if key / value are given -- the rank that holds the sequence's
 * last position passes them, the others pass NULL) and a merge of its splits that leaves the
 * rank's RECORD instead of the final answer: rec_out[i, h, :] the normalised fp32 partial
 * (contiguous, num_seqs x num_q_heads x head_dim) and rec_lse[i, h] its natural-log sum-exp
 * (-inf where the rank holds no token of sequence i). Records of all ranks, gathered, are folded
 * by hkb_merge with one part a rank. Two launches; num_splits >= 2 (the record is written by the
 * merge). rec_out == NULL (and rec_lse NULL): the walk alone, one launch -- the partials stay in
 * part_out / part_lse for the caller to fold (hkb_kvsplit_push). Everything else as hkb_decode_step.
 *
 * Replaces nothing in the reference, which cuts the KV axis inside one GPU only
 * (python/hk/ops/paged.py:171-194); it is that cut carried one level up.
 */
int hkb_decode_step_record(float* rec_out, float* rec_lse,
                           const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                           const void* key, const void* value,
                           int64_t key_stride_tok, int64_t key_stride_head,
                           int64_t val_stride_tok, int64_t val_stride_head,
                           const void* slot_mapping, int slot_is_i64,
                           hkb_cache_t k_cache, hkb_cache_t v_cache,
                           const int32_t* block_table, int64_t table_stride, int max_pages,
                           const int32_t* seq_lens, const int32_t* q_start,
                           int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                           int block_size, float scale, int kv_dtype,
                           const float* k_scale, const float* v_scale,
                           int num_splits, float* part_out, float* part_lse, void* stream);

/*
 * hkb_paged_decode over caches in vLLM's older "x-split" layout, read in place
 * (no copy, no re-layout): K is (blocks, kv_heads, head_dim / 8, block_size, 8)
 * and V is (blocks, kv_heads, head_dim, block_size) -- V^T -- of 16-bit elements,
 * everything inside a block contiguous; `*_stride_block` is elements between
 * blocks. head_dim 128, bf16 or fp16 caches, num_splits >= 2 (the balanced tile
 * stream), at most HKB_STREAM_MAX_SEQS sequences; anything else is
 * HKB_ERR_UNSUPPORTED / HKB_ERR_SPLITS / HKB_ERR_SIZE before a launch. Partials
 * as in hkb_paged_decode; hkb_merge folds them.
 * Replaces: python/hk/ops/paged_prefill.py:768-772 (`rocm_views`, the strided
 * views the reference's kernels read that layout through) and the decode over
 * them, `_rocm_decode` (python/hk/integration/vllm_prefill.py:1332-1356).
 */
int hkb_paged_decode_xsplit(void* out, int64_t out_stride_tok, int64_t out_stride_head,
                            const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                            const void* k_cache, int64_t k_stride_block,
                            const void* v_cache, int64_t v_stride_block, int64_t num_blocks,
                            const int32_t* block_table, int64_t table_stride, int max_pages,
                            const int32_t* seq_lens, const int32_t* q_start,
                            int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                            int block_size, float scale, int kv_dtype,
                            int num_splits, float* part_out, float* part_lse, void* stream);

/*
 * The exchange step of a KV axis cut across the GPUs of one box, over peer memory instead of a
 * collective. Every rank allocates a gather buffer (hkb_exchange_gather_bytes) and a state block
 * (hkb_exchange_state_bytes, ZERO before the first step) in memory that every other rank has mapped
 * (CUDA IPC, or torch's symmetric memory); `gather[r]` / `state[r]` are rank r's two buffers as
 * mapped in THIS process (for r == rank: the rank's own).
 *
 * A step, on one stream, the same on every rank:
 *   hkb_paged_decode(..., num_splits >= 2, part_out, part_lse)   the walk, partials in local scratch
 *   hkb_kvsplit_push(x, part_out, part_lse, num_splits, ...)     folds the rank's splits and stores its
 *                                                               record (normalised fp32 out, natural-log
 *                                                               lse) into every rank's gather buffer,
 *                                                               then raises its flag on every rank
 *   hkb_kvsplit_merge(x, out, ..., spin_limit)                   waits for every rank's flag of this
 *                                                               step, folds the records into `out`
 * No host value changes between steps (the step counter lives in the state block), so the three
 * launches can be captured and replayed. The wait is bounded: a flag polled `spin_limit` times (about
 * 0.1 us a poll) without arriving sets the error word -- the last int32 of the rank's state block -- to
 * 1 + the rank that was missing, the CTA skips its fold and the kernel returns; `out` is then not
 * valid and the host decides (the ranks' step counters are out of step after a miss: zero the state
 * blocks on every rank before going on). Ranks must make the same calls in the same order.
 * At most 8 ranks. Plain peer stores: no multicast, no multimem.
 *
 * Replaces nothing in the reference (its KV split stays inside one GPU,
 * python/hk/ops/paged.py:171-194); it is what ncclAllGather + hkb_merge do for this path, as two kernels.
 */
typedef struct {
  int world, rank;
  void* gather[8];
  void* state[8];
} hkb_exchange_t;

size_t hkb_exchange_gather_bytes(int world, int num_seqs, int num_q_heads, int head_dim);
size_t hkb_exchange_state_bytes(void);
int hkb_kvsplit_push(hkb_exchange_t x, const float* part_out, const float* part_lse, int num_splits,
                     int num_seqs, int num_q_heads, int head_dim, void* stream);
int hkb_kvsplit_merge(hkb_exchange_t x, void* out, int64_t out_stride_tok, int64_t out_stride_head, int out_kind,
                      int num_seqs, int num_q_heads, int head_dim, int spin_limit, void* stream);

/*
 * hkb_kvsplit_push and hkb_kvsplit_merge in one launch: a CTA a (sequence, head) folds the
 * rank's splits, stores its row of the record into every rank, raises the row's own flag on
 * every rank, waits (at most spin_limit polls a rank; a miss sets the error word, skips the
 * row and returns) for the same row of every rank and folds them into `out`. The state
 * blocks must be hkb_exchange_state_bytes_rows(num_seqs, num_q_heads) bytes (the 20 words of
 * hkb_exchange_state_bytes, then a flag a (parity, rank, row)), zeroed once. Do not mix the
 * two forms on one state block within a step. No counterpart in the reference (as above).
 */
size_t hkb_exchange_state_bytes_rows(int num_seqs, int num_q_heads);
int hkb_kvsplit_exchange(hkb_exchange_t x, const float* part_out, const float* part_lse, int num_splits,
                         void* out, int64_t out_stride_tok, int64_t out_stride_head, int out_kind,
                         int num_seqs, int num_q_heads, int head_dim, int spin_limit, void* stream);

/* Bytes of the arrival counters hkb_decode_step takes. */
size_t hkb_arrivals_bytes(int num_seqs, int num_kv_heads);

/* Query tokens one work item of hkb_paged_prefill covers: 256 rows divided by the heads of the
 * GQA group a CTA serves (32 for a group of 8, 64 for 4, 128 for 2, 256 for 1); 0 if the head
 * counts are not a valid GQA shape. */
int hkb_prefill_tile_rows(int num_q_heads, int num_kv_heads);

/* 1 if hkb_paged_prefill runs its tcgen05 / tensor-memory kernel for this head size and cache
 * type (head_dim 128: bf16, fp16, or fp8-e4m3 widened to f16 on its way into shared memory), 0 if
 * the mma.sync kernel (other head sizes, or HKB_PREFILL_MMA_SYNC=1 in the environment, the
 * comparison arm). Like the reference, which picks
 * its contraction form per architecture and shape (python/hk/ops/paged_prefill.py:59-120). */
int hkb_prefill_uses_tcgen05(int head_dim, int kv_dtype);

/*
 * hkb_paged_prefill on a traced build of the tensor-memory kernel (head_dim 128, a bf16 cache, a
 * GQA group of 4, 16-byte-aligned query rows; HKB_ERR_UNSUPPORTED otherwise): besides the answer,
 * every CTA -- index kv_head * num_work + work item -- writes 32 uint64 cycle counters to
 * `trace` (device memory, num_work * num_kv_heads * 32 entries): softmax warps of query tile g at
 * 8 g + {0 waiting for scores, 1 TMEM loads and maximum, 2 exponentials, 3 waiting for the
 * previous product / rescale, 4 P store and arrive, 5 epilogue}; MMA warp at 16 + {0 wait for Q,
 * 1 wait for K, 2 issue of the first q.K, 3 wait for V, 4 / 6 wait for P of tile 0 / 1, 5 issue of
 * p.V and of the next block's q.K};
 * producer w (0 K, 1 V) at 24 + 4 w + {0 wait for a free slot, 1 issue of copies, 2 wait for
 * copies to land}; 31 the CTA's whole time. A measurement aid with no counterpart in the reference
 * (which attributes time by ablation, python/hk/ops/paged.py:524-533).
 */
int hkb_paged_prefill_trace(void* out, int64_t out_stride_tok, int64_t out_stride_head,
                            const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                            hkb_cache_t k_cache, hkb_cache_t v_cache,
                            const int32_t* block_table, int64_t table_stride, int max_pages,
                            const int32_t* seq_lens, const int32_t* q_start,
                            const int32_t* work, int num_work, int num_tokens,
                            int num_q_heads, int num_kv_heads, int head_dim, int block_size,
                            float scale, int kv_dtype, const float* k_scale, const float* v_scale,
                            unsigned long long* trace, void* stream);

/* The tensor-memory prefill kernel bounds every wait on a barrier; a wait that ran out leaves a
 * code here (0: none; 1..7: which wait) instead of hanging the GPU. Reads the word back from the
 * current device (this synchronises); `clear` != 0 resets it. -1 if the read failed. */
int hkb_prefill_tc_error(int clear);

/*
 * Bytes of the scratch array built into the library for hkb_paged_decode_static (below).
 */
#define HKB_STATIC_SCRATCH_BYTES (8u << 20)

/*
 * The split decode for callers that have no device memory to give and no way to get any:
 * the same walk + merge as hkb_paged_decode followed by hkb_merge, but the split partials
 * live in a fixed array inside the library instead of caller-owned scratch, and the call
 * itself allocates and frees nothing (no cudaMalloc, no cudaFree, no allocating library
 * routine). It has no counterpart in the reference, whose routes always own their scratch.
 *
 * Who needs it: a binding that only ever holds the pointers its engine handed it -- a cgo /
 * JNI / N-API caller with no allocator bridge -- and a serving loop that runs after the engine
 * has given the whole GPU to its KV-cache pool, where a late cudaMalloc fails or stalls.
 *
 * Arguments are those of hkb_paged_decode without part_out / part_lse; `out` receives the
 * final bf16 answer. num_splits == 1 needs no partials and is passed straight through.
 *
 * Limits and rules:
 *   - the partials need hkb_scratch_bytes(num_seqs, num_q_heads, head_dim, num_splits) bytes;
 *     more than HKB_STATIC_SCRATCH_BYTES is refused with HKB_ERR_STATIC_SCRATCH and nothing
 *     is launched -- use fewer splits or the caller-scratch entry points;
 *   - the array costs HKB_STATIC_SCRATCH_BYTES of device memory on every GPU that loads the
 *     library, from load until the process exits;
 *   - the FIRST call on each device looks the array's device address up (with that device
 *     current); make that first call before any stream capture begins;
 *   - every call on a device shares the one array and finds the previous call's partials in
 *     it. Nothing in it has to start at zero: each call first rewrites the lse of every slot
 *     it may read (a value, or -inf for "unused") and never reads a slot marked unused. Two
 *     calls that overlap on the GPU (different streams, or threads on one device) race on the
 *     array: serialise them.
 */
int hkb_paged_decode_static(void* out, int64_t out_stride_tok, int64_t out_stride_head,
                            const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                            hkb_cache_t k_cache, hkb_cache_t v_cache,
                            const int32_t* block_table, int64_t table_stride, int max_pages,
                            const int32_t* seq_lens, const int32_t* q_start,
                            int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                            int block_size, float scale, int kv_dtype,
                            const float* k_scale, const float* v_scale,
                            int num_splits, void* stream);

/*
 * Split planner: how many ways to cut the KV axis so that num_seqs*num_kv_heads
 * CTAs fill sm_count SMs; a power of two, at most max_tiles (16-token tiles of
 * the longest sequence the engine allows) and HKB_MAX_SPLITS. A function of host
 * values only, so a captured graph's plan is right for every replay.
 * Replaces: plan_splits (python/hk/ops/paged.py:877-914) and decode_splits
 * (python/hk/integration/vllm_backend.py:137-151).
 */
int hkb_plan_splits(int num_seqs, int num_kv_heads, int max_tiles, int sm_count);

/* Bytes of (part_out, part_lse) scratch for a split decode, part_out first;
 * part_lse starts at hkb_scratch_lse_offset. Replaces fused_scratch
 * (python/hk/ops/paged.py:733-743). */
size_t hkb_scratch_bytes(int num_seqs, int num_q_heads, int head_dim, int num_splits);
size_t hkb_scratch_lse_offset(int num_seqs, int num_q_heads, int head_dim, int num_splits);

/* 1 if the walk of a GQA group of `group` query heads a kv head runs on tensor-core (mma) tiles,
 * 0 if on CUDA cores: bf16 caches from a group of 4, fp8-e4m3 always (measured on B200; the
 * environment's HKB_MMA_MIN_GROUP = 1..8 overrides both). The reference picks its own contraction
 * form per architecture the same way (python/hk/ops/paged.py:498-547). */
int hkb_walk_uses_mma(int group, int kv_dtype);

/*
 * A read-only streaming probe: one launch reads `bytes` of `buf` once with 16-byte loads (a
 * persistent grid of ctas_per_sm x SMs CTAs of 256 threads, loads_in_flight = 1, 2, 4, 8 or 16
 * independent loads a thread) and writes nothing (`sink`, 4 device bytes, is only there to keep
 * the loads alive). The caller times it, rotates buffers larger than L2 and sweeps the two
 * parameters; the best figure is the read ceiling the decode walk is held to beside the copy peak.
 * Replaces: tools/hk-bench/hbm_probe.hip:1-134.
 */
int hkb_hbm_read_probe(const void* buf, size_t bytes, int ctas_per_sm, int loads_in_flight, void* sink,
                       void* stream);

/* SM count of CUDA device `device` (-1 = current), cached; <= 0 on error. */
int hkb_sm_count(int device);

/* A sentence for a status code; never NULL. */
const char* hkb_strerror(int code);

/* The last CUDA error code seen by this thread inside the library (cudaError_t). */
int hkb_last_cuda_error(void);

/* HKB_VERSION of the built library. */
int hkb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* HKB_H_ */
