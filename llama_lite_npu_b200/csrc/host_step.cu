// Decode steps whose per-step tensors live in host memory: pinned staging, three streams, one call
// per step.  See include/b200kv_host_step.h for the contract.
#include <cuda_runtime.h>

#include <new>
#include <vector>

#include "b200kv.h"
#include "b200kv_host_step.h"
#include "launch.h"

namespace b200kv {
namespace {

constexpr int kMaxDepth = 8;

struct Layout {
  size_t q, new_k, new_v, lens, slots, in_bytes, out_bytes;
};

inline size_t align16(size_t x) { return (x + 15) & ~size_t(15); }

Layout layout_for(int batch, int q_heads, int kv_heads, int head_dim) {
  Layout l;
  const size_t q_bytes = size_t(batch) * q_heads * head_dim * 2;
  const size_t kv_bytes = size_t(batch) * kv_heads * head_dim * 2;
  l.q = 0;
  l.new_k = align16(q_bytes);
  l.new_v = align16(l.new_k + kv_bytes);
  l.lens = align16(l.new_v + kv_bytes);
  l.slots = align16(l.lens + size_t(batch) * 4);
  l.in_bytes = align16(l.slots + size_t(batch) * 4);
  l.out_bytes = q_bytes;
  return l;
}

struct Slot {
  char* h_in = nullptr;
  char* h_out = nullptr;
  char* d_in = nullptr;
  char* d_out = nullptr;
  cudaEvent_t in_done = nullptr;    // the slot's inputs are on the device
  cudaEvent_t step_done = nullptr;  // the slot's kernel has finished
  cudaEvent_t out_done = nullptr;   // the slot's result is in h_out
  DecodeArgs args{};                // of the slot's submitted step
  size_t out_bytes = 0;
  bool idle = true;                 // no step of this slot can still be in flight (never used, or waited for)
};

// The resident state a step runs on (pool, table, row ids, scale), registered once.
struct Binding {
  void* k_base;
  void* v_base;
  int64_t kv_tok_stride, kv_head_stride, pool_tokens;
  const int32_t* table;
  int64_t table_row_stride;
  int table_kind, table_rows;
  int64_t table_cols;
  const int32_t* row_ids;
  int page_size;
  float scale;
};

struct HostSteps {
  std::vector<Binding> bindings;
  int device = -1;
  int depth = 0;
  int max_batch = 0, q_heads = 0, kv_heads = 0, head_dim = 0;
  Layout cap;
  Slot slot[kMaxDepth];
  cudaStream_t s_in = nullptr, s_run = nullptr, s_out = nullptr;
  void* workspace = nullptr;
  size_t workspace_bytes = 0;
  int pending = -1;                 // slot whose step is submitted but not launched yet

  ~HostSteps() {
    // Nothing of this object may still be in flight when its memory goes.
    if (s_in) cudaStreamSynchronize(s_in);
    if (s_run) cudaStreamSynchronize(s_run);
    if (s_out) cudaStreamSynchronize(s_out);
    for (int i = 0; i < kMaxDepth; ++i) {
      Slot& s = slot[i];
      if (s.h_in) cudaFreeHost(s.h_in);
      if (s.h_out) cudaFreeHost(s.h_out);
      if (s.d_in) cudaFree(s.d_in);
      if (s.d_out) cudaFree(s.d_out);
      if (s.in_done) cudaEventDestroy(s.in_done);
      if (s.step_done) cudaEventDestroy(s.step_done);
      if (s.out_done) cudaEventDestroy(s.out_done);
    }
    if (workspace) cudaFree(workspace);
    if (s_in) cudaStreamDestroy(s_in);
    if (s_run) cudaStreamDestroy(s_run);
    if (s_out) cudaStreamDestroy(s_out);
  }
};

#define HS_TRY(call)                                      \
  do {                                                    \
    cudaError_t e_ = (call);                              \
    if (e_ != cudaSuccess) return record_cuda_error(e_);  \
  } while (0)

int build(HostSteps& h) {
  HS_TRY(cudaGetDevice(&h.device));
  HS_TRY(cudaStreamCreateWithFlags(&h.s_in, cudaStreamNonBlocking));
  HS_TRY(cudaStreamCreateWithFlags(&h.s_run, cudaStreamNonBlocking));
  HS_TRY(cudaStreamCreateWithFlags(&h.s_out, cudaStreamNonBlocking));
  for (int i = 0; i < h.depth; ++i) {
    Slot& s = h.slot[i];
    HS_TRY(cudaHostAlloc(reinterpret_cast<void**>(&s.h_in), h.cap.in_bytes, cudaHostAllocDefault));
    HS_TRY(cudaHostAlloc(reinterpret_cast<void**>(&s.h_out), h.cap.out_bytes, cudaHostAllocDefault));
    HS_TRY(cudaMalloc(reinterpret_cast<void**>(&s.d_in), h.cap.in_bytes));
    HS_TRY(cudaMalloc(reinterpret_cast<void**>(&s.d_out), h.cap.out_bytes));
    HS_TRY(cudaEventCreateWithFlags(&s.in_done, cudaEventDisableTiming));
    HS_TRY(cudaEventCreateWithFlags(&s.step_done, cudaEventDisableTiming));
    HS_TRY(cudaEventCreateWithFlags(&s.out_done, cudaEventDisableTiming));
  }
  h.workspace_bytes = decode_workspace_bytes(h.max_batch, h.q_heads, h.kv_heads, h.head_dim);
  if (h.workspace_bytes == 0) return B200KV_ETOOLARGE;   // more (sequence, KV head) pairs than arrival counters
  HS_TRY(cudaMalloc(&h.workspace, h.workspace_bytes));
  // the piece counters at the head of the workspace start at zero and return to zero after a launch
  HS_TRY(cudaMemsetAsync(h.workspace, 0, h.workspace_bytes, h.s_run));
  HS_TRY(cudaStreamSynchronize(h.s_run));
  return B200KV_OK;
}

// Make `stream` wait for `event` unless the event has already happened (then no dependency is
// needed, and a kernel launched next keeps its programmatic edge to the kernel before it).
inline cudaError_t wait_unless_done(cudaStream_t stream, cudaEvent_t event) {
  const cudaError_t q = cudaEventQuery(event);
  if (q == cudaSuccess) return cudaSuccess;
  if (q != cudaErrorNotReady) return q;
  return cudaStreamWaitEvent(stream, event, 0);
}

// Launch the step that the last submit left pending: kernel on the compute stream, result copy on
// the copy-out stream.
int launch_pending(HostSteps& h) {
  if (h.pending < 0) return B200KV_OK;
  Slot& s = h.slot[h.pending];
  h.pending = -1;
  // after its inputs have landed and after the slot's previous result has left d_out
  HS_TRY(wait_unless_done(h.s_run, s.in_done));
  if (!s.idle) HS_TRY(wait_unless_done(h.s_run, s.out_done));
  s.idle = false;
  const int rc = paged_decode(s.args, h.s_run);
  if (rc != B200KV_OK) return rc;
  HS_TRY(cudaEventRecord(s.step_done, h.s_run));
  HS_TRY(cudaStreamWaitEvent(h.s_out, s.step_done, 0));
  HS_TRY(cudaMemcpyAsync(s.h_out, s.d_out, s.out_bytes, cudaMemcpyDeviceToHost, h.s_out));
  HS_TRY(cudaEventRecord(s.out_done, h.s_out));
  return B200KV_OK;
}

inline HostSteps* handle(void* p, int slot) {
  HostSteps* h = static_cast<HostSteps*>(p);
  if (h == nullptr || slot < 0 || slot >= h->depth) return nullptr;
  return h;
}

}  // namespace
}  // namespace b200kv

extern "C" {

int b200kv_host_steps_create(int depth, int max_batch, int q_heads, int kv_heads, int head_dim, void** out) {
  using namespace b200kv;
  if (out == nullptr) return B200KV_EINVAL;
  *out = nullptr;
  if (depth < 1 || depth > kMaxDepth || max_batch < 1 || q_heads < 1 || kv_heads < 1 || head_dim < 1 ||
      q_heads % kv_heads != 0)
    return B200KV_EINVAL;
  if (head_dim != 128) return B200KV_EUNSUPPORTED;
  const int group = q_heads / kv_heads;
  if (group > 16) return B200KV_EUNSUPPORTED;
  HostSteps* h = new (std::nothrow) HostSteps();
  if (h == nullptr) return B200KV_EINVAL;
  h->depth = depth;
  h->max_batch = max_batch;
  h->q_heads = q_heads;
  h->kv_heads = kv_heads;
  h->head_dim = head_dim;
  h->cap = layout_for(max_batch, q_heads, kv_heads, head_dim);
  const int rc = build(*h);
  if (rc != B200KV_OK) {
    delete h;
    return rc;
  }
  *out = h;
  return B200KV_OK;
}

void b200kv_host_steps_destroy(void* steps) { delete static_cast<b200kv::HostSteps*>(steps); }

int b200kv_host_steps_buffers(void* steps, int slot, int batch, void** q, void** new_k, void** new_v,
                              int32_t** seq_lens, int32_t** slots, void** out) {
  using namespace b200kv;
  HostSteps* h = handle(steps, slot);
  if (h == nullptr || batch < 1 || batch > h->max_batch) return B200KV_EINVAL;
  const Layout l = layout_for(batch, h->q_heads, h->kv_heads, h->head_dim);
  const Slot& s = h->slot[slot];
  if (q) *q = s.h_in + l.q;
  if (new_k) *new_k = s.h_in + l.new_k;
  if (new_v) *new_v = s.h_in + l.new_v;
  if (seq_lens) *seq_lens = reinterpret_cast<int32_t*>(s.h_in + l.lens);
  if (slots) *slots = reinterpret_cast<int32_t*>(s.h_in + l.slots);
  if (out) *out = s.h_out;
  return B200KV_OK;
}

}  // extern "C"

namespace b200kv {
namespace {

int submit_step(HostSteps* h, int slot, int batch, const Binding& bd, int64_t max_seq_len, int flags,
                int32_t* status) {
  if (batch < 1 || batch > h->max_batch) return B200KV_EINVAL;
  if (bd.k_base == nullptr || bd.v_base == nullptr || bd.table == nullptr || status == nullptr) return B200KV_EINVAL;
  if (h->pending == slot) return B200KV_EINVAL;   // the slot's previous step has not even been launched
  int dev = -1;
  HS_TRY(cudaGetDevice(&dev));
  if (dev != h->device) return B200KV_EINVAL;
  const Layout l = layout_for(batch, h->q_heads, h->kv_heads, h->head_dim);
  Slot& s = h->slot[slot];

  // Inputs first: the staging on the device is free once the kernel that last read it has finished
  // (known without asking when the host has already waited for the slot's result).
  if (!s.idle) HS_TRY(wait_unless_done(h->s_in, s.step_done));
  HS_TRY(cudaMemcpyAsync(s.d_in, s.h_in, l.in_bytes, cudaMemcpyHostToDevice, h->s_in));
  HS_TRY(cudaEventRecord(s.in_done, h->s_in));

  // Then the step submitted BEFORE this one: its inputs have had a whole submission to land, so
  // its launch usually needs no wait on the copy stream and follows its predecessor directly.
  const int rc = launch_pending(*h);
  if (rc != B200KV_OK) return rc;

  DecodeArgs& a = s.args;
  a = DecodeArgs{};
  const int64_t q_row = int64_t(h->q_heads) * h->head_dim;
  const int64_t kv_row = int64_t(h->kv_heads) * h->head_dim;
  a.q = s.d_in + l.q;
  a.q_stride_b = q_row;
  a.q_stride_h = h->head_dim;
  a.k_base = bd.k_base;
  a.v_base = bd.v_base;
  a.kv_tok_stride = bd.kv_tok_stride;
  a.kv_head_stride = bd.kv_head_stride;
  a.pool_tokens = bd.pool_tokens;
  a.table = bd.table;
  a.table_row_stride = bd.table_row_stride;
  a.table_kind = bd.table_kind;
  a.table_rows = bd.table_rows;
  a.table_cols = bd.table_cols;
  a.row_ids = bd.row_ids;
  a.seq_lens = s.d_in + l.lens;
  a.seq_lens_i64 = 0;
  a.new_k = s.d_in + l.new_k;
  a.new_v = s.d_in + l.new_v;
  a.new_k_tok_stride = kv_row;
  a.new_v_tok_stride = kv_row;
  a.slots = reinterpret_cast<const int32_t*>(s.d_in + l.slots);
  a.batch = batch;
  a.q_heads = h->q_heads;
  a.kv_heads = h->kv_heads;
  a.head_dim = h->head_dim;
  a.page_size = bd.page_size;
  a.scale = bd.scale;
  a.max_seq_len = max_seq_len;
  a.workspace = h->workspace;
  a.workspace_bytes = h->workspace_bytes;
  a.out = s.d_out;
  a.out_stride_b = q_row;
  a.out_stride_h = h->head_dim;
  a.flags = flags;
  a.status = status;
  s.out_bytes = l.out_bytes;
  h->pending = slot;
  if (h->depth == 1) return launch_pending(*h);   // nothing to overlap with
  return B200KV_OK;
}

}  // namespace
}  // namespace b200kv

extern "C" {

int b200kv_host_steps_submit(void* steps, int slot, int batch, void* k_base, void* v_base,
                             int64_t kv_tok_stride, int64_t kv_head_stride, int64_t pool_tokens,
                             const int32_t* table, int64_t table_row_stride, int table_kind,
                             int table_rows, int64_t table_cols, const int32_t* row_ids, int page_size,
                             float scale, int64_t max_seq_len, int flags, int32_t* status) {
  using namespace b200kv;
  HostSteps* h = handle(steps, slot);
  if (h == nullptr) return B200KV_EINVAL;
  const Binding bd{k_base,     v_base,     kv_tok_stride, kv_head_stride, pool_tokens, table, table_row_stride,
                   table_kind, table_rows, table_cols,    row_ids,        page_size,   scale};
  return submit_step(h, slot, batch, bd, max_seq_len, flags, status);
}

int b200kv_host_steps_bind(void* steps, void* k_base, void* v_base, int64_t kv_tok_stride,
                           int64_t kv_head_stride, int64_t pool_tokens, const int32_t* table,
                           int64_t table_row_stride, int table_kind, int table_rows, int64_t table_cols,
                           const int32_t* row_ids, int page_size, float scale) {
  using namespace b200kv;
  HostSteps* h = static_cast<HostSteps*>(steps);
  if (h == nullptr || k_base == nullptr || v_base == nullptr || table == nullptr) return -B200KV_EINVAL;
  if (h->bindings.size() >= 65536) return -B200KV_ETOOLARGE;
  h->bindings.push_back(Binding{k_base, v_base, kv_tok_stride, kv_head_stride, pool_tokens, table,
                                table_row_stride, table_kind, table_rows, table_cols, row_ids, page_size, scale});
  return static_cast<int>(h->bindings.size()) - 1;
}

int b200kv_host_steps_submit_bound(void* steps, int slot, int batch, int binding, int64_t max_seq_len,
                                   int flags, int32_t* status) {
  using namespace b200kv;
  HostSteps* h = handle(steps, slot);
  if (h == nullptr || binding < 0 || binding >= static_cast<int>(h->bindings.size())) return B200KV_EINVAL;
  return submit_step(h, slot, batch, h->bindings[binding], max_seq_len, flags, status);
}

int b200kv_host_steps_flush(void* steps) {
  using namespace b200kv;
  HostSteps* h = static_cast<HostSteps*>(steps);
  if (h == nullptr) return B200KV_EINVAL;
  return launch_pending(*h);
}

int b200kv_host_steps_wait(void* steps, int slot) {
  using namespace b200kv;
  HostSteps* h = handle(steps, slot);
  if (h == nullptr) return B200KV_EINVAL;
  // A host that blocks here is not about to submit.  The pending step goes out now if it is this
  // slot's own (it must), or if its inputs have already landed (then its launch needs no
  // cross-stream wait and nothing is gained by holding it back).
  if (h->pending >= 0 &&
      (h->pending == slot || cudaEventQuery(h->slot[h->pending].in_done) == cudaSuccess)) {
    const int rc = launch_pending(*h);
    if (rc != B200KV_OK) return rc;
  }
  HS_TRY(cudaEventSynchronize(h->slot[slot].out_done));
  h->slot[slot].idle = true;
  return B200KV_OK;
}

int b200kv_host_steps_reset(void* steps) {
  using namespace b200kv;
  HostSteps* h = static_cast<HostSteps*>(steps);
  if (h == nullptr) return B200KV_EINVAL;
  const int rc = launch_pending(*h);
  HS_TRY(cudaStreamSynchronize(h->s_in));
  HS_TRY(cudaStreamSynchronize(h->s_run));
  HS_TRY(cudaStreamSynchronize(h->s_out));
  for (int i = 0; i < h->depth; ++i) h->slot[i].idle = true;
  // the arrival counters at the head of the workspace: a launch that gave up on a wait may have
  // left some of them short of wrapping back to zero
  HS_TRY(cudaMemsetAsync(h->workspace, 0, B200KV_DECODE_COUNTER_BYTES, h->s_run));
  HS_TRY(cudaStreamSynchronize(h->s_run));
  return rc;
}

void* b200kv_host_steps_stream(void* steps) {
  b200kv::HostSteps* h = static_cast<b200kv::HostSteps*>(steps);
  return h ? h->s_run : nullptr;
}

}  // extern "C"
