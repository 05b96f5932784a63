// Decode-step batch metadata on the device: advance every sequence of the batch by one token
// and derive the slot its new K/V row goes to, from the block table that is already resident.
//
// Per decode step the reference does this on the host, one request at a time
// (lite_llama/executor/model_executor.py:913-931 -> paged_attention.py:313-359 extend_req, then
// :287-311 batch_metadata): bump the length, write the new token-table entry to the device, then
// build and copy b_req_idx / b_seq_len / cur_select_index.  Here the host only allocates a page
// when a sequence crosses a page boundary (1 step in page_size); lengths, slots and the new
// token-table entries are produced by one tiny kernel and never cross PCIe, so a captured decode
// step can be replayed with no host-to-device copy at all.
//
// One thread per sequence; integer work, a few hundred bytes of traffic: latency-bound by design.
#include "common.cuh"
#include "launch.h"

namespace b200kv {

namespace {

struct AdvanceParams {
  const int32_t* req_ids;      // nullptr: row b of the tables is sequence b
  void* seq_lens;              // in: length before the step; out: length including the new token
  int seq_lens_i64;
  int32_t* slots;              // out: slot of the new token
  const int32_t* block_table;
  int64_t block_row_stride;
  int table_pages;             // columns of the block table
  const int32_t* page_counts;  // nullptr or pages allocated per table row
  int32_t* token_table;        // nullptr or the per-token slot table to extend
  int64_t token_row_stride;
  int token_cols;
  int batch, table_rows, page_size;
  int64_t pool_pages;
  int32_t* status;
};

__global__ void __launch_bounds__(128) decode_advance_kernel(AdvanceParams p) {
  cudaGridDependencySynchronize();
  cudaTriggerProgrammaticLaunchCompletion();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= p.batch) return;
  const int row = p.req_ids ? p.req_ids[b] : b;
  const int64_t pos = load_len(p.seq_lens, p.seq_lens_i64, b);   // index of the new token
  // A refused sequence gets slot -1 (the append and the prologue skip negative slots); left alone,
  // slots[b] would still name the previous step's row and the next append would overwrite it.
  if (row < 0 || row >= p.table_rows || pos < 0) {
    set_status(p.status, B200KV_DEV_BAD_LENGTH);
    p.slots[b] = -1;
    return;
  }
  const int64_t page_idx = pos / p.page_size;
  if (page_idx >= p.table_pages || (p.page_counts && page_idx >= p.page_counts[row]) ||
      (p.token_table && pos >= p.token_cols)) {
    set_status(p.status, B200KV_DEV_BAD_LENGTH);   // no page reserved for the new token
    p.slots[b] = -1;
    return;
  }
  const int64_t page = p.block_table[row * p.block_row_stride + page_idx];
  if (page < 0 || page >= p.pool_pages) {
    set_status(p.status, B200KV_DEV_BAD_PAGE);
    p.slots[b] = -1;
    return;
  }
  const int32_t slot = static_cast<int32_t>(page * p.page_size + (pos - page_idx * p.page_size));
  p.slots[b] = slot;
  if (p.token_table) p.token_table[row * p.token_row_stride + pos] = slot;
  if (p.seq_lens_i64)
    reinterpret_cast<int64_t*>(p.seq_lens)[b] = pos + 1;
  else
    reinterpret_cast<int32_t*>(p.seq_lens)[b] = static_cast<int32_t>(pos + 1);
}

// table[req_ids[i]][seq_lens[i] - 1] = select_index[i]: the token-table write of the reference's
// non-paged decode path (lite_llama/kernels/update_kv_index.py:6-38).
struct IndexParams {
  int32_t* table;
  int64_t row_stride, col_stride;
  int rows, cols;
  const int32_t* req_ids;
  const void* seq_lens;
  int seq_lens_i64;
  const int32_t* select_index;
  int n;
  int32_t* status;
};

__global__ void __launch_bounds__(128) update_kv_index_kernel(IndexParams p) {
  cudaGridDependencySynchronize();
  cudaTriggerProgrammaticLaunchCompletion();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= p.n) return;
  const int row = p.req_ids[i];
  const int64_t col = load_len(p.seq_lens, p.seq_lens_i64, i) - 1;
  if (row < 0 || row >= p.rows || col < 0 || col >= p.cols) {
    set_status(p.status, B200KV_DEV_BAD_LENGTH);
    return;
  }
  p.table[row * p.row_stride + col * p.col_stride] = p.select_index[i];
}

// A handful of table entries changed on the host (a sequence crossed a page boundary, a request
// was admitted): the (offset, value) pairs travel as kernel ARGUMENTS, so there is no staging
// buffer to keep alive and no host-to-device copy to order, just one small launch.
constexpr int kPatchMax = 96;
struct PatchParams {
  int32_t* table;
  int64_t elems;
  int n;
  int64_t off[kPatchMax];
  int32_t val[kPatchMax];
};

__global__ void __launch_bounds__(kPatchMax) table_patch_kernel(const __grid_constant__ PatchParams p) {
  cudaGridDependencySynchronize();
  cudaTriggerProgrammaticLaunchCompletion();
  const int i = threadIdx.x;
  if (i >= p.n) return;
  const int64_t off = p.off[i];
  if (off >= 0 && off < p.elems) p.table[off] = p.val[i];
}

}  // namespace

int table_patch(int32_t* table, int64_t elems, const int64_t* offsets_host, const int32_t* values_host,
                int64_t n, cudaStream_t stream) {
  if (n < 0 || elems <= 0) return B200KV_EINVAL;
  if (n == 0) return B200KV_OK;
  if (!table || !offsets_host || !values_host) return B200KV_EINVAL;
  for (int64_t i = 0; i < n; ++i)
    if (offsets_host[i] < 0 || offsets_host[i] >= elems) return B200KV_EINVAL;   // nothing launched
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  for (int64_t done = 0; done < n; done += kPatchMax) {
    PatchParams p{};
    p.table = table;
    p.elems = elems;
    p.n = static_cast<int>(n - done < kPatchMax ? n - done : kPatchMax);
    for (int i = 0; i < p.n; ++i) {
      p.off[i] = offsets_host[done + i];
      p.val[i] = values_host[done + i];
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(kPatchMax);
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, table_patch_kernel, p);
    if (e != cudaSuccess) return record_cuda_error(e);
  }
  return check_launch();
}

int update_kv_index(int32_t* table, int64_t row_stride, int64_t col_stride, int rows, int cols,
                    const int32_t* req_ids, const void* seq_lens, int seq_lens_i64,
                    const int32_t* select_index, int n, int32_t* status, cudaStream_t stream) {
  if (n < 0 || rows <= 0 || cols <= 0) return B200KV_EINVAL;
  if (n == 0) return B200KV_OK;
  if (!table || !req_ids || !seq_lens || !select_index) return B200KV_EINVAL;
  IndexParams p{table, row_stride, col_stride, rows, cols, req_ids, seq_lens, seq_lens_i64,
                select_index, n, status};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>((n + 127) / 128));
  cfg.blockDim = dim3(128);
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, update_kv_index_kernel, p);
  if (e != cudaSuccess) return record_cuda_error(e);
  return check_launch();
}

int decode_advance(const AdvanceArgs& a, cudaStream_t stream) {
  if (a.batch < 0 || a.table_rows <= 0 || a.table_pages <= 0 || a.page_size <= 0 || a.pool_pages <= 0)
    return B200KV_EINVAL;
  if (a.batch == 0) return B200KV_OK;
  if (!a.seq_lens || !a.slots || !a.block_table || a.block_row_stride < a.table_pages) return B200KV_EINVAL;
  if (a.token_table && (a.token_cols <= 0 || a.token_row_stride < a.token_cols)) return B200KV_EINVAL;
  if (a.pool_pages * a.page_size > INT32_MAX) return B200KV_ETOOLARGE;   // slots are int32
  AdvanceParams p{};
  p.req_ids = a.req_ids;
  p.seq_lens = a.seq_lens;
  p.seq_lens_i64 = a.seq_lens_i64;
  p.slots = a.slots;
  p.block_table = a.block_table;
  p.block_row_stride = a.block_row_stride;
  p.table_pages = a.table_pages;
  p.page_counts = a.page_counts;
  p.token_table = a.token_table;
  p.token_row_stride = a.token_row_stride;
  p.token_cols = a.token_cols;
  p.batch = a.batch;
  p.table_rows = a.table_rows;
  p.page_size = a.page_size;
  p.pool_pages = a.pool_pages;
  p.status = a.status;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>((a.batch + 127) / 128));
  cfg.blockDim = dim3(128);
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, decode_advance_kernel, p);
  if (e != cudaSuccess) return record_cuda_error(e);
  return check_launch();
}

}  // namespace b200kv
