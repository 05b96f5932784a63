// extern "C" surface of libb200kv.so: argument marshalling only, see include/b200kv.h.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>

#include "b200kv.h"
#include "launch.h"

namespace b200kv {

namespace {
thread_local char g_last_cuda_error[256] = "";
}

int record_cuda_error(cudaError_t e) {
  if (e == cudaSuccess) return B200KV_OK;
  std::snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s: %s", cudaGetErrorName(e),
                cudaGetErrorString(e));
  return B200KV_ECUDA;
}

int check_launch() { return record_cuda_error(cudaGetLastError()); }

int device_sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    record_cuda_error(cudaGetLastError());
    return -1;
  }
  if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
  int sms = 0;
  cudaError_t e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) {
    record_cuda_error(e);
    return -1;
  }
  if (dev >= 0 && dev < 64) cached[dev] = sms;
  return sms;
}

}  // namespace b200kv

extern "C" {

int b200kv_version(void) { return B200KV_VERSION; }

const char* b200kv_strerror(int code) {
  switch (code) {
    case B200KV_OK: return "ok";
    case B200KV_EINVAL: return "invalid argument (null pointer, negative size or bad enum)";
    case B200KV_EUNSUPPORTED: return "unsupported head_dim, page_size or query-group size";
    case B200KV_EALIGN: return "pointer or stride is not suitably aligned";
    case B200KV_EWORKSPACE: return "workspace too small";
    case B200KV_ECUDA: return "CUDA runtime error";
    case B200KV_ETOOLARGE: return "size exceeds a fixed maximum of this entry point";
    case B200KV_DEV_BAD_SLOT: return "device: slot_mapping entry outside the KV pool";
    case B200KV_DEV_BAD_PAGE: return "device: page/token table entry outside the KV pool";
    case B200KV_DEV_BAD_LENGTH: return "device: sequence length negative or above the stated maximum";
    case B200KV_DEV_WAIT_TIMEOUT: return "device: bounded wait ran out";
    default: return "unknown b200kv code";
  }
}

const char* b200kv_last_cuda_error(void) { return b200kv::g_last_cuda_error; }

int b200kv_kv_append(const void* kv_values, int64_t n_tokens, int64_t src_tok_stride,
                     const int32_t* slots, void* pool, int64_t pool_tokens, int64_t pool_tok_stride,
                     int n_rows, int head_dim, int32_t* status, void* stream) {
  return b200kv::kv_append(kv_values, n_tokens, src_tok_stride, slots, pool, pool_tokens,
                           pool_tok_stride, n_rows, head_dim, status,
                           static_cast<cudaStream_t>(stream));
}

int b200kv_kv_append_split(const void* k_values, const void* v_values, int64_t n_tokens,
                           int64_t k_tok_stride, int64_t v_tok_stride, const int32_t* slots,
                           void* pool, int64_t pool_tokens, int64_t pool_tok_stride, int kv_heads,
                           int head_dim, int32_t* status, void* stream) {
  return b200kv::kv_append_split(k_values, v_values, n_tokens, k_tok_stride, v_tok_stride, slots,
                                 pool, pool_tokens, pool_tok_stride, kv_heads, head_dim, status,
                                 static_cast<cudaStream_t>(stream));
}

int b200kv_qk_norm_rope_append(const void* q, void* q_out, int64_t q_tok_stride,
                               int64_t q_out_tok_stride, const void* kv, int64_t kv_tok_stride,
                               const void* q_weight, const void* k_weight, float eps,
                               const void* cos, const void* sin, int64_t cs_tok_stride,
                               const int32_t* slots, void* pool, int64_t pool_tokens,
                               int64_t pool_tok_stride, int64_t n_tokens, int q_heads,
                               int kv_heads, int head_dim, int32_t* status, void* stream) {
  b200kv::PrologueArgs a{};
  a.q = q;
  a.q_out = q_out;
  a.q_tok_stride = q_tok_stride;
  a.q_out_tok_stride = q_out_tok_stride;
  a.kv = kv;
  a.kv_tok_stride = kv_tok_stride;
  a.q_weight = q_weight;
  a.k_weight = k_weight;
  a.eps = eps;
  a.cos = cos;
  a.sin = sin;
  a.cs_tok_stride = cs_tok_stride;
  a.slots = slots;
  a.pool = pool;
  a.pool_tokens = pool_tokens;
  a.pool_tok_stride = pool_tok_stride;
  a.n_tokens = n_tokens;
  a.q_heads = q_heads;
  a.kv_heads = kv_heads;
  a.head_dim = head_dim;
  a.status = status;
  return b200kv::qk_norm_rope_append(a, static_cast<cudaStream_t>(stream));
}

int b200kv_decode_advance(const int32_t* req_ids, void* seq_lens, int seq_lens_i64, int32_t* slots,
                          const int32_t* block_table, int64_t block_row_stride, int table_rows,
                          int table_pages, const int32_t* page_counts, int32_t* token_table,
                          int64_t token_row_stride, int token_cols, int batch, int page_size,
                          int64_t pool_pages, int32_t* status, void* stream) {
  b200kv::AdvanceArgs a{};
  a.req_ids = req_ids;
  a.seq_lens = seq_lens;
  a.seq_lens_i64 = seq_lens_i64;
  a.slots = slots;
  a.block_table = block_table;
  a.block_row_stride = block_row_stride;
  a.table_rows = table_rows;
  a.table_pages = table_pages;
  a.page_counts = page_counts;
  a.token_table = token_table;
  a.token_row_stride = token_row_stride;
  a.token_cols = token_cols;
  a.batch = batch;
  a.page_size = page_size;
  a.pool_pages = pool_pages;
  a.status = status;
  return b200kv::decode_advance(a, static_cast<cudaStream_t>(stream));
}

int b200kv_table_patch(int32_t* table, int64_t table_elems, const int64_t* offsets_host,
                       const int32_t* values_host, int64_t n, void* stream) {
  return b200kv::table_patch(table, table_elems, offsets_host, values_host, n, static_cast<cudaStream_t>(stream));
}

int b200kv_update_kv_index(int32_t* req_to_token_indexs, int64_t row_stride, int64_t col_stride,
                           int rows, int cols, const int32_t* b_req_idx, const void* b_seq_len,
                           int seq_lens_i64, const int32_t* select_index, int n, int32_t* status,
                           void* stream) {
  return b200kv::update_kv_index(req_to_token_indexs, row_stride, col_stride, rows, cols, b_req_idx,
                                 b_seq_len, seq_lens_i64, select_index, n, status,
                                 static_cast<cudaStream_t>(stream));
}

size_t b200kv_decode_workspace_bytes(int batch, int q_heads, int kv_heads, int head_dim) {
  return b200kv::decode_workspace_bytes(batch, q_heads, kv_heads, head_dim);
}

namespace {
b200kv::DecodeArgs decode_args(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* k_base,
                               const void* v_base, int64_t kv_tok_stride, int64_t kv_head_stride,
                               int64_t pool_tokens, const int32_t* table, int64_t table_row_stride,
                               int table_kind, int table_rows, int64_t table_cols, const int32_t* row_ids,
                               const void* seq_lens, int seq_lens_i64, int batch, int q_heads, int kv_heads,
                               int head_dim, int page_size, float scale, int64_t max_seq_len, void* out,
                               int64_t out_stride_b, int64_t out_stride_h, int flags, int32_t* status) {
  b200kv::DecodeArgs a{};
  a.q = q;
  a.q_stride_b = q_stride_b;
  a.q_stride_h = q_stride_h;
  a.k_base = k_base;
  a.v_base = v_base;
  a.kv_tok_stride = kv_tok_stride;
  a.kv_head_stride = kv_head_stride;
  a.pool_tokens = pool_tokens;
  a.table = table;
  a.table_row_stride = table_row_stride;
  a.table_kind = table_kind;
  a.table_rows = table_rows;
  a.table_cols = table_cols;
  a.row_ids = row_ids;
  a.seq_lens = seq_lens;
  a.seq_lens_i64 = seq_lens_i64;
  a.batch = batch;
  a.q_heads = q_heads;
  a.kv_heads = kv_heads;
  a.head_dim = head_dim;
  a.page_size = page_size;
  a.scale = scale;
  a.max_seq_len = max_seq_len;
  a.out = out;
  a.out_stride_b = out_stride_b;
  a.out_stride_h = out_stride_h;
  a.flags = flags;
  a.status = status;
  return a;
}
}  // namespace

int b200kv_set_option(int option, int64_t value) { return b200kv::set_decode_option(option, value); }

int b200kv_paged_decode(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* k_base,
                        const void* v_base, int64_t kv_tok_stride, int64_t kv_head_stride,
                        int64_t pool_tokens, const int32_t* table, int64_t table_row_stride,
                        int table_kind, int table_rows, int64_t table_cols, const int32_t* row_ids,
                        const void* seq_lens, int seq_lens_i64, int batch, int q_heads, int kv_heads,
                        int head_dim, int page_size, float scale, int64_t max_seq_len, void* workspace,
                        size_t workspace_bytes, void* out, int64_t out_stride_b, int64_t out_stride_h,
                        int flags, int32_t* status, void* stream) {
  b200kv::DecodeArgs a = decode_args(q, q_stride_b, q_stride_h, k_base, v_base, kv_tok_stride, kv_head_stride,
                                     pool_tokens, table, table_row_stride, table_kind, table_rows, table_cols,
                                     row_ids, seq_lens, seq_lens_i64, batch, q_heads, kv_heads, head_dim,
                                     page_size, scale, max_seq_len, out, out_stride_b, out_stride_h, flags,
                                     status);
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  return b200kv::paged_decode(a, static_cast<cudaStream_t>(stream));
}

int b200kv_append_paged_decode(const void* new_k, const void* new_v, int64_t new_k_tok_stride,
                               int64_t new_v_tok_stride, const int32_t* slots,
                               const void* q, int64_t q_stride_b, int64_t q_stride_h, void* k_base,
                               void* v_base, int64_t kv_tok_stride, int64_t kv_head_stride,
                               int64_t pool_tokens, const int32_t* table, int64_t table_row_stride,
                               int table_kind, int table_rows, int64_t table_cols, const int32_t* row_ids,
                               const void* seq_lens, int seq_lens_i64, int batch, int q_heads,
                               int kv_heads, int head_dim, int page_size, float scale,
                               int64_t max_seq_len, void* workspace, size_t workspace_bytes, void* out,
                               int64_t out_stride_b, int64_t out_stride_h, int flags, int32_t* status,
                               void* stream) {
  if (batch > 0 && (new_k == nullptr || new_v == nullptr || slots == nullptr)) return B200KV_EINVAL;
  b200kv::DecodeArgs a = decode_args(q, q_stride_b, q_stride_h, k_base, v_base, kv_tok_stride, kv_head_stride,
                                     pool_tokens, table, table_row_stride, table_kind, table_rows, table_cols,
                                     row_ids, seq_lens, seq_lens_i64, batch, q_heads, kv_heads, head_dim,
                                     page_size, scale, max_seq_len, out, out_stride_b, out_stride_h, flags,
                                     status);
  a.new_k = new_k;
  a.new_v = new_v;
  a.new_k_tok_stride = new_k_tok_stride;
  a.new_v_tok_stride = new_v_tok_stride;
  a.slots = slots;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  return b200kv::paged_decode(a, static_cast<cudaStream_t>(stream));
}

int b200kv_paged_decode_static_scratch(
    const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* k_base, const void* v_base,
    int64_t kv_tok_stride, int64_t kv_head_stride, int64_t pool_tokens, const int32_t* table,
    int64_t table_row_stride, int table_kind, int table_rows, int64_t table_cols, const int32_t* row_ids,
    const void* seq_lens, int seq_lens_i64, int batch, int q_heads, int kv_heads, int head_dim,
    int page_size, float scale, int64_t max_seq_len, void* out, int64_t out_stride_b,
    int64_t out_stride_h, int flags, int32_t* status, void* stream) {
  b200kv::DecodeArgs a = decode_args(q, q_stride_b, q_stride_h, k_base, v_base, kv_tok_stride, kv_head_stride,
                                     pool_tokens, table, table_row_stride, table_kind, table_rows, table_cols,
                                     row_ids, seq_lens, seq_lens_i64, batch, q_heads, kv_heads, head_dim,
                                     page_size, scale, max_seq_len, out, out_stride_b, out_stride_h, flags,
                                     status);
  return b200kv::paged_decode_static_scratch(a, static_cast<cudaStream_t>(stream));
}

int b200kv_paged_prefill(const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* k_base,
                         const void* v_base, int64_t kv_tok_stride, int64_t kv_head_stride,
                         int64_t pool_tokens, const int32_t* table, int64_t table_row_stride,
                         int table_kind, int table_rows, int64_t table_cols, const int32_t* req_ids,
                         const int32_t* q_start,
                         const void* ctx_lens, const void* q_lens, int lens_i64, int batch,
                         int64_t total_q, int64_t max_q_len, int q_heads, int kv_heads, int head_dim,
                         int page_size, float scale_log2, void* out, int64_t out_stride_t,
                         int64_t out_stride_h, int32_t* status, void* stream) {
  b200kv::PrefillArgs a{};
  a.q = q;
  a.q_stride_t = q_stride_t;
  a.q_stride_h = q_stride_h;
  a.k_base = k_base;
  a.v_base = v_base;
  a.kv_tok_stride = kv_tok_stride;
  a.kv_head_stride = kv_head_stride;
  a.pool_tokens = pool_tokens;
  a.table = table;
  a.table_row_stride = table_row_stride;
  a.table_kind = table_kind;
  a.table_rows = table_rows;
  a.table_cols = table_cols;
  a.req_ids = req_ids;
  a.q_start = q_start;
  a.ctx_lens = ctx_lens;
  a.q_lens = q_lens;
  a.lens_i64 = lens_i64;
  a.batch = batch;
  a.total_q = total_q;
  a.max_q_len = max_q_len;
  a.q_heads = q_heads;
  a.kv_heads = kv_heads;
  a.head_dim = head_dim;
  a.page_size = page_size;
  a.scale_log2 = scale_log2;
  a.out = out;
  a.out_stride_t = out_stride_t;
  a.out_stride_h = out_stride_h;
  a.status = status;
  return b200kv::paged_prefill(a, static_cast<cudaStream_t>(stream));
}

int b200kv_selftest_bounded_wait(uint64_t limit_ns, int32_t* result, int32_t* status, void* stream) {
  return b200kv::wait_selftest(limit_ns, result, status, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
