// Internal host-side declarations shared by the .cu files and the C-ABI shim.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace b200kv {

// SM count of the current device (cached per device); <= 0 on failure.
int device_sm_count();
// cudaGetLastError() -> B200KV_OK / B200KV_ECUDA, remembering the message.
int check_launch();
int record_cuda_error(cudaError_t e);

int kv_append(const void* kv_values, int64_t n_tokens, int64_t src_tok_stride, const int32_t* slots,
              void* pool, int64_t pool_tokens, int64_t pool_tok_stride, int n_rows, int head_dim,
              int32_t* status, cudaStream_t stream);
int kv_append_split(const void* k_values, const void* v_values, int64_t n_tokens,
                    int64_t k_tok_stride, int64_t v_tok_stride, const int32_t* slots, void* pool,
                    int64_t pool_tokens, int64_t pool_tok_stride, int kv_heads, int head_dim,
                    int32_t* status, cudaStream_t stream);

struct PrologueArgs {
  const void* q;
  void* q_out;
  int64_t q_tok_stride, q_out_tok_stride;
  const void* kv;
  int64_t kv_tok_stride;
  const void* q_weight;
  const void* k_weight;
  float eps;
  const void* cos;
  const void* sin;
  int64_t cs_tok_stride;
  const int32_t* slots;
  void* pool;
  int64_t pool_tokens, pool_tok_stride;
  int64_t n_tokens;
  int q_heads, kv_heads, head_dim;
  int32_t* status;
};
int qk_norm_rope_append(const PrologueArgs& a, cudaStream_t stream);

struct AdvanceArgs {
  const int32_t* req_ids;
  void* seq_lens;
  int seq_lens_i64;
  int32_t* slots;
  const int32_t* block_table;
  int64_t block_row_stride;
  int table_pages;
  const int32_t* page_counts;
  int32_t* token_table;
  int64_t token_row_stride;
  int token_cols;
  int batch, table_rows, page_size;
  int64_t pool_pages;
  int32_t* status;
};
int decode_advance(const AdvanceArgs& a, cudaStream_t stream);
// table[offsets[i]] = values[i]; offsets / values are HOST arrays, passed to the kernel as arguments.
int table_patch(int32_t* table, int64_t elems, const int64_t* offsets_host, const int32_t* values_host,
                int64_t n, cudaStream_t stream);
int update_kv_index(int32_t* table, int64_t row_stride, int64_t col_stride, int rows, int cols,
                    const int32_t* req_ids, const void* seq_lens, int seq_lens_i64,
                    const int32_t* select_index, int n, int32_t* status, cudaStream_t stream);

struct DecodeArgs {
  const void* q;
  int64_t q_stride_b, q_stride_h;
  const void* k_base;
  const void* v_base;
  int64_t kv_tok_stride, kv_head_stride, pool_tokens;
  const int32_t* table;
  int64_t table_row_stride;
  int table_kind;
  int table_rows;
  int64_t table_cols;
  const int32_t* row_ids;
  const void* seq_lens;
  int seq_lens_i64;
  const void* new_k;           // fused append: nullptr = none
  const void* new_v;
  int64_t new_k_tok_stride, new_v_tok_stride;
  const int32_t* slots;
  int batch, q_heads, kv_heads, head_dim, page_size;
  float scale;
  int64_t max_seq_len;
  void* workspace;
  size_t workspace_bytes;
  void* out;
  int64_t out_stride_b, out_stride_h;
  int flags;
  int32_t* status;
};
size_t decode_workspace_bytes(int batch, int q_heads, int kv_heads, int head_dim);
int set_decode_option(int option, int64_t value);
int paged_decode(const DecodeArgs& a, cudaStream_t stream);
// Same, with the split-KV scratch in a fixed device array owned by the library (args.workspace ignored).
int paged_decode_static_scratch(const DecodeArgs& args, cudaStream_t stream);

struct PrefillArgs {
  const void* q;
  int64_t q_stride_t, q_stride_h;
  const void* k_base;
  const void* v_base;
  int64_t kv_tok_stride, kv_head_stride, pool_tokens;
  const int32_t* table;
  int64_t table_row_stride;
  int table_kind;
  int table_rows;
  int64_t table_cols;
  const int32_t* req_ids;
  const int32_t* q_start;
  const void* ctx_lens;
  const void* q_lens;
  int lens_i64;
  int batch;
  int64_t total_q, max_q_len;
  int q_heads, kv_heads, head_dim, page_size;
  float scale_log2;
  void* out;
  int64_t out_stride_t, out_stride_h;
  int32_t* status;
};
int paged_prefill(const PrefillArgs& a, cudaStream_t stream);
int wait_selftest(uint64_t limit_ns, int32_t* result, int32_t* status, cudaStream_t stream);

}  // namespace b200kv
