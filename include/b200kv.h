/*
 * b200kv — C ABI of the paged-KV attention path for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers, sizes and strides (in
 * ELEMENTS of the pointed-to type unless a name ends in _bytes) and a CUDA
 * stream passed as void* (a cudaStream_t; NULL = the legacy default stream).
 * Nothing here allocates or frees device memory, synchronises the device, or
 * keeps a pointer after the call returns (the one exception is documented on
 * the entry point itself).  All launches are asynchronous on `stream`.
 *
 * Return value: 0 on success, otherwise one of the B200KV_E* codes below;
 * b200kv_strerror() turns a code into text.  Arguments are validated on the
 * host BEFORE anything is launched, so a non-zero return means nothing ran.
 *
 * Device-side index checks: kernels bounds-check every index they read from
 * device memory before using it: slots and page ids against the pool, table
 * rows (row_ids / req_ids) against table_rows, lengths against the table's
 * width.  An out-of-range index is never dereferenced; the access (or the
 * whole sequence, for a bad row or length) is skipped and, when `status` is
 * not NULL, the first offending code is recorded in *status (a device int32
 * the caller zeroes beforehand and may read back whenever it is willing to
 * synchronise).
 *
 * Stream ordering: kernels are launched with programmatic stream serialisation
 * (programmatic dependent launch).  Each kernel touches q / K / V / the pool /
 * new rows / slot_mapping / workspaces / outputs only after the previous
 * kernel in the stream has completed, but the decode kernel plans its work
 * (reads seq_lens, row_ids and the page table) before that point, overlapping
 * the tail of the previous kernel.  Those three metadata arrays must therefore
 * not be produced by the kernel launched IMMEDIATELY before a decode entry
 * point on the same stream -- or that call passes B200KV_DECODE_SERIALIZED,
 * which launches it as an ordinary, fully ordered kernel.  Anything earlier
 * (copies, other kernels) is ordered as usual.
 *
 * The reference project (lite_llama, Python + Triton-Ascend) has no native
 * interface; each function below names the reference Python operator whose
 * device work it replaces, as file:line inside that project.
 */
#ifndef B200KV_H_
#define B200KV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200KV_VERSION 200

/* ---- host-side return codes ------------------------------------------- */
#define B200KV_OK              0
#define B200KV_EINVAL          1  /* NULL pointer, negative size, bad enum      */
#define B200KV_EUNSUPPORTED    2  /* head_dim / page_size / group size not built */
#define B200KV_EALIGN          3  /* pointer or stride not 16-byte aligned       */
#define B200KV_EWORKSPACE      4  /* workspace too small                         */
#define B200KV_ECUDA           5  /* a CUDA runtime call failed (see last error) */
#define B200KV_ETOOLARGE       6  /* size beyond a documented fixed maximum      */

/* ---- device-side status codes written to *status ---------------------- */
#define B200KV_DEV_OK            0
#define B200KV_DEV_BAD_SLOT      101  /* slot_mapping entry outside the pool     */
#define B200KV_DEV_BAD_PAGE      102  /* table entry outside the pool            */
#define B200KV_DEV_BAD_LENGTH    103  /* negative length or length > table width */
#define B200KV_DEV_WAIT_TIMEOUT  104  /* a bounded device-side wait ran out      */

/* ---- table kinds ------------------------------------------------------- */
/* BLOCK: table[row][p] = physical page id of logical page p.
 * TOKEN: table[row][t] = physical token slot of logical token t, where the
 *        page_size slots of one page are consecutive and page-aligned (what
 *        the reference's PagedReqTokensManager writes,
 *        lite_llama/executor/paged_attention.py:116-147,346-358).  Only
 *        entries at t % page_size == 0 are read. */
#define B200KV_TABLE_BLOCK 0
#define B200KV_TABLE_TOKEN 1
/* DENSE (prefill only): no table; logical token t of request r is slot
 * q_start[r] + t of k_base / v_base, i.e. K/V are packed exactly like Q. */
#define B200KV_TABLE_DENSE 2

int b200kv_version(void);
const char* b200kv_strerror(int code);
/* Text of the last CUDA error seen by this library on the calling thread. */
const char* b200kv_last_cuda_error(void);

/*
 * KV append: pool[slots[i], r, :] = kv_values[i, r, :] for r in [0, n_rows).
 * Replaces update_kv_buffer (lite_llama/kernels/update_kv_buffer.py:47-81,
 * kernel :7-43).  Pure 16-byte-vector copy, bit-exact.
 *   kv_values  fp16 [n_tokens, n_rows, head_dim], row-contiguous inside a token,
 *              token stride src_tok_stride
 *   slots      int32 [n_tokens]  (the slot_mapping / cur_select_index)
 *   pool       fp16 [pool_tokens, n_rows, head_dim], token stride pool_tok_stride
 *   n_rows     2 * kv_heads (K heads first, then V heads)
 * n_tokens == 0 is a no-op.  Duplicate slots in one call race (last writer
 * wins, as in the reference).
 */
int b200kv_kv_append(const void* kv_values, int64_t n_tokens, int64_t src_tok_stride,
                     const int32_t* slots,
                     void* pool, int64_t pool_tokens, int64_t pool_tok_stride,
                     int n_rows, int head_dim,
                     int32_t* status, void* stream);

/*
 * Same scatter with K and V given separately ([n_tokens, kv_heads, head_dim]
 * each), so the caller need not materialise torch.cat([xk, xv], dim=-2)
 * (lite_llama/models/qwen3.py:29,62) first.
 */
int b200kv_kv_append_split(const void* k_values, const void* v_values,
                           int64_t n_tokens, int64_t k_tok_stride, int64_t v_tok_stride,
                           const int32_t* slots,
                           void* pool, int64_t pool_tokens, int64_t pool_tok_stride,
                           int kv_heads, int head_dim,
                           int32_t* status, void* stream);

/*
 * Attention prologue in one launch: per-head RMSNorm of Q and K, rotary
 * embedding of Q and K, and the scatter of K (normalised, rotated) and V (as
 * is) into the pool.  Replaces, for one layer,
 *   skip_rmsnorm(xq, None, q_norm_weight), skip_rmsnorm(xk, None, k_norm_weight)
 *       lite_llama/models/qwen3.py:122-123, kernel lite_llama/kernels/skip_rmsnorm.py:118-144
 *   rope_emb_forward(xq, xk, cos, sin)
 *       lite_llama/models/qwen3.py:125-126, kernel lite_llama/kernels/rope_emb.py:6-87
 *   torch.cat([xk, xv], dim=-2) + update_kv_buffer
 *       lite_llama/models/qwen3.py:62-65 (decode), :29-32 (prefill)
 *   q, q_out    fp16 [n_tokens, q_heads, head_dim]; q_out may be q (in place)
 *   kv          fp16 [n_tokens, 2*kv_heads, head_dim]: the kv_proj output, K heads first
 *   q_weight, k_weight  fp16 [head_dim] or NULL (NULL: that norm is skipped, as
 *               for models without QK-norm, lite_llama/models/qwen2.py)
 *   cos, sin    fp16 rows per token, token stride cs_tok_stride; only the first
 *               head_dim/2 entries of a row are read (rope_emb.py:41-44)
 *   slots, pool as for b200kv_kv_append
 * Strides are in elements and must be multiples of 8; pointers 16-byte aligned;
 * head_dim 64 or 128.  V rows and slots not named are bit-exact; Q and K follow
 * the reference kernels' rounding (fp32 statistics, fp16(x*rrms)*w in fp16,
 * rotation in fp32 rounded once).  n_tokens == 0 is a no-op.
 */
int b200kv_qk_norm_rope_append(const void* q, void* q_out, int64_t q_tok_stride,
                               int64_t q_out_tok_stride,
                               const void* kv, int64_t kv_tok_stride,
                               const void* q_weight, const void* k_weight, float eps,
                               const void* cos, const void* sin, int64_t cs_tok_stride,
                               const int32_t* slots,
                               void* pool, int64_t pool_tokens, int64_t pool_tok_stride,
                               int64_t n_tokens, int q_heads, int kv_heads, int head_dim,
                               int32_t* status, void* stream);

/*
 * Decode-step batch metadata on the device.  For every sequence b of the batch
 * (table row r = req_ids[b], or b when req_ids is NULL), with pos = seq_lens[b]:
 *   slots[b]     = block_table[r][pos / page_size] * page_size + pos % page_size
 *   token_table[r][pos] = slots[b]            (when token_table is not NULL)
 *   seq_lens[b]  = pos + 1
 * i.e. what the reference computes on the host, request by request, before each
 * decode step: extend_req (lite_llama/executor/paged_attention.py:313-359) and
 * batch_metadata (:287-311), called from extend_paged_requests /
 * activate_paged_decode_batch (lite_llama/executor/model_executor.py:893-931).
 * The page for position pos must already be in the block table (the host
 * allocates it when a page boundary is crossed); page_counts, when not NULL,
 * gives the pages present per table row and lets the kernel refuse
 * (B200KV_DEV_BAD_LENGTH, nothing written for that sequence) instead of
 * reading a stale entry.  Integer work, bit-exact.
 */
int b200kv_decode_advance(const int32_t* req_ids, void* seq_lens, int seq_lens_i64,
                          int32_t* slots,
                          const int32_t* block_table, int64_t block_row_stride,
                          int table_rows, int table_pages, const int32_t* page_counts,
                          int32_t* token_table, int64_t token_row_stride, int token_cols,
                          int batch, int page_size, int64_t pool_pages,
                          int32_t* status, void* stream);

/*
 * table[offsets[i]] = values[i] for i in [0, n): a few entries of a device table (block table,
 * token table, page counts) that changed on the host.  offsets_host and values_host are HOST
 * arrays; they are copied into the launch arguments, so they may be reused as soon as the call
 * returns and nothing crosses PCIe as a separate copy.  Replaces the small per-request
 * host-to-device writes of the reference's extend_req / alloc_req
 * (lite_llama/executor/paged_attention.py:209-212, :354-357).  Offsets are element offsets into
 * `table` (table_elems elements); one outside it is refused with B200KV_EINVAL and nothing is
 * launched.  Any n; 96 entries go into one launch.
 */
int b200kv_table_patch(int32_t* table, int64_t table_elems,
                       const int64_t* offsets_host, const int32_t* values_host, int64_t n,
                       void* stream);

/*
 * req_to_token_indexs[b_req_idx[i]][b_seq_len[i] - 1] = select_index[i] for i in [0, n).
 * Replaces update_kv_index (lite_llama/kernels/update_kv_index.py:42-74, kernel :6-38), the
 * token-table write of the non-paged decode path
 * (lite_llama/executor/model_executor.py:958-967).  Strides in elements.  An index outside
 * the table sets B200KV_DEV_BAD_LENGTH and skips that entry.  Bit-exact.
 */
int b200kv_update_kv_index(int32_t* req_to_token_indexs, int64_t row_stride, int64_t col_stride,
                           int rows, int cols,
                           const int32_t* b_req_idx, const void* b_seq_len, int seq_lens_i64,
                           const int32_t* select_index, int n,
                           int32_t* status, void* stream);

/*
 * Bytes of scratch that the decode entry points need for a batch of `batch`
 * sequences on the CURRENT device: B200KV_DECODE_COUNTER_BYTES of arrival
 * counters followed by the split-KV partial outputs and their log-sum-exp.
 * Depends on the device's SM count.  Returns 0 on bad input.
 *
 * The counters (one per sequence and KV head, at the start of the workspace
 * whatever the shape) must be ZERO when a decode call starts.  Every call
 * leaves them at zero again, so the caller clears the first
 * B200KV_DECODE_COUNTER_BYTES once, after allocating the workspace
 * (cudaMemsetAsync), and never again -- unless a call ended with
 * B200KV_DEV_WAIT_TIMEOUT in *status, after which they must be cleared anew.
 * Calls that may overlap on the GPU need separate workspaces.
 */
#define B200KV_DECODE_COUNTER_BYTES (256u << 10)
size_t b200kv_decode_workspace_bytes(int batch, int q_heads, int kv_heads, int head_dim);

/* flags of the decode entry points */
#define B200KV_DECODE_SERIALIZED 1  /* no programmatic overlap with the previous kernel:
                                       seq_lens / row_ids / table may come straight from it */

/*
 * Paged flash-decoding: one query token per sequence attends to that
 * sequence's whole paged context.  Replaces flash_decoding
 * (lite_llama/kernels/flashdecoding.py:295-342; stage 1 :6-138, stage 2
 * :199-267).  ONE launch: a persistent split-KV kernel in which each CTA
 * serves one KV head together with its whole GQA query group; the CTA that
 * delivers the last partial of a sequence merges that sequence's partials
 * (log-sum-exp weights) and writes its output rows.
 *   q          fp16 [batch, q_heads, head_dim]; strides q_stride_b, q_stride_h
 *   k_base     fp16 K view of the pool, element (t, h, d) at
 *              k_base + t*kv_tok_stride + h*kv_head_stride + d
 *   v_base     likewise for V (same strides)
 *   pool_tokens number of token slots addressable from k_base / v_base
 *   table      int32 [table_rows, table_cols], row stride table_row_stride,
 *              kind B200KV_TABLE_*
 *   row_ids    int32 [batch] table row of each sequence, or NULL = 0..batch-1
 *              (the reference indexes rows by batch position,
 *              lite_llama/kernels/flashdecoding.py:48,85); a row outside
 *              [0, table_rows) sets B200KV_DEV_BAD_LENGTH and that sequence
 *              is treated as empty
 *   seq_lens   int32 or int64 [batch] (seq_lens_i64 selects); length 0 gives
 *              an all-zero output row; a length above max_seq_len is clamped
 *              and reported
 *   scale      natural softmax scale (1/sqrt(head_dim)); softmax is base e
 *   max_seq_len host upper bound of the lengths; must fit the table's width
 *   workspace  see b200kv_decode_workspace_bytes (counters zeroed once)
 *   out        fp16 [batch, q_heads, head_dim]; strides out_stride_b, out_stride_h
 *   flags      0 or B200KV_DECODE_SERIALIZED
 * Supported: head_dim 128, page_size 16, q_heads/kv_heads in [1,16], batch <= 4096,
 * batch * kv_heads <= B200KV_DECODE_COUNTER_BYTES / 4.
 */
int b200kv_paged_decode(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                        const void* k_base, const void* v_base,
                        int64_t kv_tok_stride, int64_t kv_head_stride, int64_t pool_tokens,
                        const int32_t* table, int64_t table_row_stride, int table_kind,
                        int table_rows, int64_t table_cols,
                        const int32_t* row_ids,
                        const void* seq_lens, int seq_lens_i64,
                        int batch, int q_heads, int kv_heads, int head_dim, int page_size,
                        float scale, int64_t max_seq_len,
                        void* workspace, size_t workspace_bytes,
                        void* out, int64_t out_stride_b, int64_t out_stride_h,
                        int flags, int32_t* status, void* stream);

/*
 * One decode step of one layer in one launch: the KV append of the step's new
 * token of every sequence, then paged flash-decoding over the context that
 * includes it.  Same result as b200kv_kv_append(new_kv, batch, ..., slots, pool)
 * followed by b200kv_paged_decode(...): update_kv_buffer then flash_decoding in
 * Attention.token_forward (lite_llama/models/qwen3.py:62-74).  The pool rows
 * are written bit-exactly.
 *   new_k, new_v  fp16 [batch, kv_heads, head_dim] each, token strides
 *              new_k_tok_stride / new_v_tok_stride: the step's new K and V row of
 *              every sequence.  For one combined [batch, 2*kv_heads, head_dim]
 *              tensor (K heads first) pass new_v = new_k + kv_heads*head_dim and
 *              the same stride twice
 *   slots      int32 [batch] slot_mapping; slots[b] must be the slot of the LAST
 *              token of sequence b, i.e. position seq_lens[b] - 1 of its table
 *              row (seq_lens already counts the new token).  A slot outside the
 *              pool is skipped, one that is not that position is still written;
 *              both set B200KV_DEV_BAD_SLOT
 *   k_base, v_base  as for b200kv_paged_decode, but written to
 * new_k / new_v and slots may come from the kernel launched immediately before; the
 * rule for seq_lens / row_ids / table stands.  Sequences of length 0 append
 * nothing.
 */
int b200kv_append_paged_decode(const void* new_k, const void* new_v,
                               int64_t new_k_tok_stride, int64_t new_v_tok_stride,
                               const int32_t* slots,
                               const void* q, int64_t q_stride_b, int64_t q_stride_h,
                               void* k_base, void* v_base,
                               int64_t kv_tok_stride, int64_t kv_head_stride, int64_t pool_tokens,
                               const int32_t* table, int64_t table_row_stride, int table_kind,
                               int table_rows, int64_t table_cols,
                               const int32_t* row_ids,
                               const void* seq_lens, int seq_lens_i64,
                               int batch, int q_heads, int kv_heads, int head_dim, int page_size,
                               float scale, int64_t max_seq_len,
                               void* workspace, size_t workspace_bytes,
                               void* out, int64_t out_stride_b, int64_t out_stride_h,
                               int flags, int32_t* status, void* stream);

/*
 * Tuning overrides of the decode launch (no counterpart in the reference); a
 * value of 0 restores the automatic choice.  Process-wide, not thread-safe
 * against concurrent decode calls.
 *   B200KV_OPT_DECODE_TEAMS       upper bound on the teams (CTAs per KV head) of a launch
 *   B200KV_OPT_DECODE_PIECE_COST  pages of streaming that ending a piece is charged with
 */
#define B200KV_OPT_DECODE_TEAMS       1
#define B200KV_OPT_DECODE_PIECE_COST  2
int b200kv_set_option(int option, int64_t value);

/*
 * Paged flash-decoding for callers that cannot allocate device memory.
 * (No counterpart in the reference: its decode operator allocates its partial
 * buffers with torch on every call.)
 *
 * Identical to b200kv_paged_decode in arguments, semantics and results, except
 * that there is no workspace argument: the arrival counters and the split-KV
 * partials go to a fixed array of B200KV_STATIC_SCRATCH_BYTES that is part of
 * the library image on every GPU that loads it.  Meant for hosts that have no
 * way to get device memory when the call is made -- a server whose device
 * budget was handed to one arena at start-up and which treats any later
 * cudaMalloc as an error, a plug-in whose memory is owned by the embedding
 * application, a real-time loop that cannot risk the device-wide stall an
 * allocation or free can cause.  The call path contains no cudaMalloc /
 * cudaFree and no allocating library call.
 *
 * Limits and rules:
 *  - the batch must be small enough that b200kv_decode_workspace_bytes() for it
 *    is <= B200KV_STATIC_SCRATCH_BYTES; larger batches are refused with
 *    B200KV_ETOOLARGE before anything is launched (split the batch, or use
 *    b200kv_paged_decode with a caller-owned workspace);
 *  - the first call on each device looks up the array's device address (with
 *    that device current) and should be made before any stream capture begins;
 *  - all calls on one device share the one array, which keeps whatever the last
 *    call left there.  The array starts zero-filled and every call returns the
 *    counters to zero; the partials need no clearing (each is written before it
 *    is read).  Two calls whose kernels may overlap on the GPU -- different
 *    streams without an ordering between them -- race on it.
 */
#define B200KV_STATIC_SCRATCH_BYTES (8u << 20)
int b200kv_paged_decode_static_scratch(
    const void* q, int64_t q_stride_b, int64_t q_stride_h,
    const void* k_base, const void* v_base,
    int64_t kv_tok_stride, int64_t kv_head_stride, int64_t pool_tokens,
    const int32_t* table, int64_t table_row_stride, int table_kind,
    int table_rows, int64_t table_cols,
    const int32_t* row_ids,
    const void* seq_lens, int seq_lens_i64,
    int batch, int q_heads, int kv_heads, int head_dim, int page_size,
    float scale, int64_t max_seq_len,
    void* out, int64_t out_stride_b, int64_t out_stride_h,
    int flags, int32_t* status, void* stream);

/*
 * Packed no-pad causal prefill over paged KV with history: query row i of
 * request r sits at logical position ctx_r + i and sees keys 0..ctx_r+i of
 * that request's table row.  Replaces paged_chunk_flash_attention
 * (lite_llama/kernels/paged_chunk_flashattention.py:227-327, kernel :58-176,
 * torch statement :179-222) and, with ctx = 0, flash_attention2_no_pad
 * (lite_llama/kernels/flashattention2_nopad.py:171-221) once the chunk's own
 * K/V have been appended to the pool.  Tensor-core (tcgen05 / TMEM) kernel.
 *   q          fp16 [total_q, q_heads, head_dim] packed; strides q_stride_t, q_stride_h
 *   table      int32 [table_rows, table_cols] (ignored for B200KV_TABLE_DENSE)
 *   req_ids    int32 [batch] table row of each request, or NULL = 0..batch-1; a
 *              request whose row is outside the table, or whose ctx + q length
 *              exceeds the table's width, is skipped (B200KV_DEV_BAD_LENGTH)
 *   q_start    int32 [batch] first packed row of each request
 *   ctx_lens, q_lens  int32 or int64 [batch] (lens_i64 selects)
 *   max_q_len  host upper bound of q_lens (sizes the launch only)
 *   scale_log2 softmax scale already multiplied by log2(e), as the reference's
 *              callers pass it (lite_llama/models/qwen3.py:296)
 */
int b200kv_paged_prefill(const void* q, int64_t q_stride_t, int64_t q_stride_h,
                         const void* k_base, const void* v_base,
                         int64_t kv_tok_stride, int64_t kv_head_stride, int64_t pool_tokens,
                         const int32_t* table, int64_t table_row_stride, int table_kind,
                         int table_rows, int64_t table_cols,
                         const int32_t* req_ids, const int32_t* q_start,
                         const void* ctx_lens, const void* q_lens, int lens_i64,
                         int batch, int64_t total_q, int64_t max_q_len,
                         int q_heads, int kv_heads, int head_dim, int page_size,
                         float scale_log2,
                         void* out, int64_t out_stride_t, int64_t out_stride_h,
                         int32_t* status, void* stream);

/*
 * Self-test of the bounded device-side wait every pipelined kernel here relies
 * on (no counterpart in the reference).  Launches one small CTA that waits on
 * two mbarriers for at most limit_ns (1 ns .. 1 s) each: the first receives its
 * arrival, the second never does.  On return (after synchronising the stream)
 * result[0] == 1 (the first wait completed), result[1] == 0 (the second gave up)
 * and *status == B200KV_DEV_WAIT_TIMEOUT.  Nothing faults or hangs: this is how
 * a lost copy or a missing producer surfaces in the real kernels (limit ~2 s).
 *   result  device int32[2];  status  device int32 (zeroed by the caller) or NULL
 */
int b200kv_selftest_bounded_wait(uint64_t limit_ns, int32_t* result, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200KV_H_ */
