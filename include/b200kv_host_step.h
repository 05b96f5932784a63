/*
 * b200kv host-buffer decode steps — C ABI.
 *
 * The same step as b200kv_append_paged_decode (include/b200kv.h: KV append by slot_mapping +
 * paged flash-decoding + merge, one launch), for a caller whose per-step tensors live in HOST
 * memory: the query rows, the step's new K/V rows, the sequence lengths and the slot_mapping go
 * in through pinned staging that this object owns, the attention output comes back the same way.
 * In the reference these five tensors are torch tensors already on the device when
 * the decode attention runs (lite_llama/models/qwen3.py:53-75 takes xq / xk / xv from the layer's
 * projections, lite_llama/executor/model_executor.py:943-972 builds the slots and lengths); a binding
 * that keeps its activations on the host (a C or Go serving loop driving the library over FFI)
 * has no torch to move them, and pays a copy in, a launch and a copy out per step.  This object
 * makes that ONE call per step and overlaps the three across steps:
 *
 *   - `depth` slots, each with pinned host staging and device staging of its own;
 *   - three streams (copy-in, compute, copy-out) and three events per slot, so that step i+1's
 *     inputs cross PCIe while step i computes and step i's result returns while step i+1
 *     computes; the steps themselves run in submission order on the compute stream;
 *   - submit() enqueues copy-in -> kernel -> copy-out for one slot and returns at once;
 *     wait() blocks until that slot's result is in its host buffer.  A slot's host buffers may
 *     be rewritten once wait() on it has returned;
 *   - with more than one slot, submit() starts the slot's copy-in at once but leaves its kernel
 *     launch to the next submit(), flush() or wait(): by then the inputs have landed, the launch
 *     needs no cross-stream wait and follows the previous step's kernel directly (programmatic
 *     dependent launch overlaps its planning with that kernel's tail).  An argument error of a
 *     step is therefore reported by the call that launches it.
 *
 * The KV pool, the page (or token) table and the optional row ids stay DEVICE memory: they are
 * the engine's resident state, not per-step inputs.  A handle is bound to the device that was
 * current at create time and is not thread-safe.
 */
#ifndef B200KV_HOST_STEP_H_
#define B200KV_HOST_STEP_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/*
 * depth: 1..8 slots.  max_batch, q_heads, kv_heads, head_dim size the staging (fp16 rows) and the
 * split-KV workspace.  Returns B200KV_OK and the handle in *out, else an error code (B200KV_EINVAL,
 * B200KV_EUNSUPPORTED for a shape the decode kernel is not built for, B200KV_ECUDA).
 */
int b200kv_host_steps_create(int depth, int max_batch, int q_heads, int kv_heads, int head_dim,
                             void** out);
void b200kv_host_steps_destroy(void* steps);

/*
 * The pinned host buffers of `slot` for a step of `batch` sequences (1..max_batch):
 *   q        fp16 [batch, q_heads, head_dim]        in
 *   new_k    fp16 [batch, kv_heads, head_dim]       in
 *   new_v    fp16 [batch, kv_heads, head_dim]       in
 *   seq_lens int32 [batch]  (lengths INCLUDING the step's new token)   in
 *   slots    int32 [batch]  (slot_mapping of the new token)            in
 *   out      fp16 [batch, q_heads, head_dim]        out
 * The inputs are packed back to back (16-byte aligned) so that one copy moves them.  Pointers
 * stay valid until destroy; their layout depends on `batch` only.
 */
int b200kv_host_steps_buffers(void* steps, int slot, int batch, void** q, void** new_k, void** new_v,
                              int32_t** seq_lens, int32_t** slots, void** out);

/*
 * Enqueue one step on `slot`: copy the slot's inputs in, run the fused append + decode on the
 * device pool (k_base / v_base, strides in ELEMENTS as in b200kv_append_paged_decode), copy the
 * output back.  table / row_ids / status are device pointers; flags as for b200kv_paged_decode.
 * The slot must not have a step in flight (call b200kv_host_steps_wait first when reusing it).
 */
int b200kv_host_steps_submit(void* steps, int slot, int batch, void* k_base, void* v_base,
                             int64_t kv_tok_stride, int64_t kv_head_stride, int64_t pool_tokens,
                             const int32_t* table, int64_t table_row_stride, int table_kind,
                             int table_rows, int64_t table_cols, const int32_t* row_ids,
                             int page_size, float scale, int64_t max_seq_len, int flags,
                             int32_t* status);

/*
 * The same with the resident state registered once: bind() remembers a pool / table / row-id /
 * page-size / scale set and returns its index (>= 0; a negated B200KV_E* code on error), and
 * submit_bound() names it.  A serving loop binds each layer's pool once and then passes seven
 * scalars per step.  Bindings live as long as the handle; the memory they name must too.
 */
int b200kv_host_steps_bind(void* steps, void* k_base, void* v_base, int64_t kv_tok_stride,
                           int64_t kv_head_stride, int64_t pool_tokens, const int32_t* table,
                           int64_t table_row_stride, int table_kind, int table_rows, int64_t table_cols,
                           const int32_t* row_ids, int page_size, float scale);
int b200kv_host_steps_submit_bound(void* steps, int slot, int batch, int binding, int64_t max_seq_len,
                                   int flags, int32_t* status);

/* Launch the step that the last submit left pending, if any (wait() does the same for its own slot, and for
 * another slot's step once that step's inputs have landed). */
int b200kv_host_steps_flush(void* steps);

/* Block until the slot's last submitted step has delivered its output to the host buffer. */
int b200kv_host_steps_wait(void* steps, int slot);

/*
 * Wait for everything in flight and return the handle to its initial state (arrival counters of
 * the split-KV workspace zeroed).  Needed only after the status word reported
 * B200KV_DEV_WAIT_TIMEOUT: a launch that gave up on a wait may leave a counter short of wrapping.
 */
int b200kv_host_steps_reset(void* steps);

/* The compute stream (a cudaStream_t), for a caller that orders other device work against the steps. */
void* b200kv_host_steps_stream(void* steps);

#ifdef __cplusplus
}
#endif

#endif  /* B200KV_HOST_STEP_H_ */
