// KV append: scatter freshly computed K/V rows into the paged fp16 pool by slot_mapping.
//
// Device work of update_kv_buffer in the reference
// (lite_llama/kernels/update_kv_buffer.py:7-43): pool[slots[i]] = kv_values[i].
// A token row is n_rows*head_dim halves (4 KB for 8 KV heads of 128); a warp moves one row
// as 16-byte vectors, consecutive lanes on consecutive vectors, eight loads in flight per lane, so
// both the read and the write are fully coalesced 128-byte lines.  HBM-bound copy:
// algorithmic bytes = 2 * n_tokens * row_bytes + 4 * n_tokens.
#include "common.cuh"
#include "launch.h"

namespace b200kv {

namespace {

constexpr int kAppendThreads = 256;
constexpr int kAppendUnroll = 8;

struct AppendParams {
  const uint4* src0;       // combined [n, rows, d] or K [n, kvh, d]
  const uint4* src1;       // V when split, else unused
  int64_t src0_tok_vec;    // token stride of src0 in 16-byte vectors
  int64_t src1_tok_vec;
  const int32_t* slots;
  uint4* pool;
  int64_t pool_tokens;
  int64_t pool_tok_vec;    // token stride of the pool in 16-byte vectors
  int64_t n_tokens;
  int vec_per_token;       // 16-byte vectors per token row
  int vec_split;           // vectors that come from src0 (== vec_per_token when not split)
  int32_t* status;
};

__global__ void __launch_bounds__(kAppendThreads) kv_append_kernel(AppendParams p) {
  // Programmatic dependent launch: this kernel has no prologue worth overlapping, so it waits
  // for the previous kernel first and only then lets its own dependent start its prologue.
  cudaGridDependencySynchronize();
  cudaTriggerProgrammaticLaunchCompletion();
  // One warp per token row: 32 lanes x kAppendUnroll independent 16-byte loads cover 4 KB (a row
  // of 8 KV heads) in one round trip; the slot is read in parallel with the row, not before it.
  const int lane = threadIdx.x & 31;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * (kAppendThreads / 32);
  int64_t tok = static_cast<int64_t>(blockIdx.x) * (kAppendThreads / 32) + (threadIdx.x >> 5);
  for (; tok < p.n_tokens; tok += warps) {
    const int64_t slot = __ldg(p.slots + tok);
    const bool slot_ok = slot >= 0 && slot < p.pool_tokens;
    if (!slot_ok && lane == 0) set_status(p.status, B200KV_DEV_BAD_SLOT);
    const uint4* s0 = p.src0 + tok * p.src0_tok_vec;
    // V half of a split source, indexed by the row's vector number (never used when not split)
    const uint4* s1 = p.src1 ? p.src1 + tok * p.src1_tok_vec - p.vec_split : s0;
    uint4* dst = p.pool + (slot_ok ? slot : 0) * p.pool_tok_vec;
    for (int c0 = 0; c0 < p.vec_per_token; c0 += 32 * kAppendUnroll) {
      uint4 v[kAppendUnroll];
#pragma unroll
      for (int u = 0; u < kAppendUnroll; ++u) {
        const int c = c0 + u * 32 + lane;
        if (c < p.vec_per_token) v[u] = __ldg(c < p.vec_split ? s0 + c : s1 + c);
      }
      if (slot_ok) {
#pragma unroll
        for (int u = 0; u < kAppendUnroll; ++u) {
          const int c = c0 + u * 32 + lane;
          if (c < p.vec_per_token) dst[c] = v[u];
        }
      }
    }
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int launch_append(AppendParams p, cudaStream_t stream) {
  if (p.n_tokens == 0) return B200KV_OK;
  const int sms = device_sm_count();
  if (sms <= 0) return B200KV_ECUDA;
  int64_t blocks = (p.n_tokens + kAppendThreads / 32 - 1) / (kAppendThreads / 32);   // a warp per token
  const int64_t cap = static_cast<int64_t>(sms) * 8;  // 8 resident CTAs of 256 threads per SM
  if (blocks > cap) blocks = cap;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(blocks));
  cfg.blockDim = dim3(kAppendThreads);
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kv_append_kernel, p);
  if (e != cudaSuccess) return record_cuda_error(e);
  return check_launch();
}

}  // namespace

int kv_append(const void* kv_values, int64_t n_tokens, int64_t src_tok_stride, const int32_t* slots,
              void* pool, int64_t pool_tokens, int64_t pool_tok_stride, int n_rows, int head_dim,
              int32_t* status, cudaStream_t stream) {
  if (n_tokens < 0 || n_rows <= 0 || head_dim <= 0 || pool_tokens < 0) return B200KV_EINVAL;
  if (n_tokens == 0) return B200KV_OK;
  if (!kv_values || !slots || !pool) return B200KV_EINVAL;
  const int64_t row_elems = static_cast<int64_t>(n_rows) * head_dim;
  if (row_elems % 8 != 0 || src_tok_stride % 8 != 0 || pool_tok_stride % 8 != 0) return B200KV_EALIGN;
  if (!aligned16(kv_values) || !aligned16(pool)) return B200KV_EALIGN;
  if (src_tok_stride < row_elems || pool_tok_stride < row_elems) return B200KV_EINVAL;
  AppendParams p{};
  p.src0 = static_cast<const uint4*>(kv_values);
  p.src1 = nullptr;
  p.src0_tok_vec = src_tok_stride / 8;
  p.src1_tok_vec = 0;
  p.slots = slots;
  p.pool = static_cast<uint4*>(pool);
  p.pool_tokens = pool_tokens;
  p.pool_tok_vec = pool_tok_stride / 8;
  p.n_tokens = n_tokens;
  p.vec_per_token = static_cast<int>(row_elems / 8);
  p.vec_split = p.vec_per_token;
  p.status = status;
  return launch_append(p, stream);
}

int kv_append_split(const void* k_values, const void* v_values, int64_t n_tokens,
                    int64_t k_tok_stride, int64_t v_tok_stride, const int32_t* slots, void* pool,
                    int64_t pool_tokens, int64_t pool_tok_stride, int kv_heads, int head_dim,
                    int32_t* status, cudaStream_t stream) {
  if (n_tokens < 0 || kv_heads <= 0 || head_dim <= 0 || pool_tokens < 0) return B200KV_EINVAL;
  if (n_tokens == 0) return B200KV_OK;
  if (!k_values || !v_values || !slots || !pool) return B200KV_EINVAL;
  const int64_t half_elems = static_cast<int64_t>(kv_heads) * head_dim;
  if (half_elems % 8 != 0 || k_tok_stride % 8 != 0 || v_tok_stride % 8 != 0 ||
      pool_tok_stride % 8 != 0)
    return B200KV_EALIGN;
  if (!aligned16(k_values) || !aligned16(v_values) || !aligned16(pool)) return B200KV_EALIGN;
  if (k_tok_stride < half_elems || v_tok_stride < half_elems || pool_tok_stride < 2 * half_elems)
    return B200KV_EINVAL;
  AppendParams p{};
  p.src0 = static_cast<const uint4*>(k_values);
  p.src1 = static_cast<const uint4*>(v_values);
  p.src0_tok_vec = k_tok_stride / 8;
  p.src1_tok_vec = v_tok_stride / 8;
  p.slots = slots;
  p.pool = static_cast<uint4*>(pool);
  p.pool_tokens = pool_tokens;
  p.pool_tok_vec = pool_tok_stride / 8;
  p.n_tokens = n_tokens;
  p.vec_per_token = static_cast<int>(2 * half_elems / 8);
  p.vec_split = static_cast<int>(half_elems / 8);
  p.status = status;
  return launch_append(p, stream);
}

}  // namespace b200kv
