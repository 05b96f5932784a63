// Attention prologue in one launch: per-head RMSNorm of Q and K, rotary embedding of Q and K,
// and the scatter of K and V into the paged fp16 pool by slot_mapping.
//
// It stands for four steps of the reference's attention layer
// (lite_llama/models/qwen3.py:122-126 then :62-65):
//   skip_rmsnorm(xq, None, q_norm_weight)   lite_llama/kernels/skip_rmsnorm.py:118-144
//   skip_rmsnorm(xk, None, k_norm_weight)
//   rope_emb_forward(xq, xk, cos, sin)      lite_llama/kernels/rope_emb.py:6-87
//   update_kv_buffer(cat(xk, xv), slots)    lite_llama/kernels/update_kv_buffer.py:7-43
// K never exists in its normalised form outside the pool and no [n, 2*KH, D] tensor is built.
//
// Rounding follows the reference kernels where it is observable: the norm takes fp32 statistics,
// rounds x*rrms to fp16 and multiplies by the fp16 weight in fp16; the rotation is evaluated in
// fp32 from those fp16 values and rounded once.
//
// A head row of D halves is handled by D/16 lanes: each lane owns 8 consecutive elements of the
// first half and the 8 elements D/2 further on, which are exactly the pairs the rotation
// mixes, so the only cross-lane traffic is the sum of squares.  All global accesses are 16-byte
// vectors, and a warp touches 2 x 128 contiguous bytes of each of its rows.  HBM-bound:
// algorithmic bytes per token = 2*H*D*2 (Q read + write) + 2*KH*D*2 (K, V read)
// + 2*KH*D*2 (pool write) + D*2 (cos, sin first halves) + 4 (slot).
#include "common.cuh"
#include "launch.h"

namespace b200kv {

namespace {

constexpr int kPrologueThreads = 256;

struct PrologueParams {
  const __half* q;
  __half* q_out;
  int64_t q_tok_stride, q_out_tok_stride;
  const __half* kv;
  int64_t kv_tok_stride;
  const __half* q_weight;   // nullptr: no norm on Q
  const __half* k_weight;   // nullptr: no norm on K
  const __half* cos;
  const __half* sin;
  int64_t cs_tok_stride;
  const int32_t* slots;
  __half* pool;
  int64_t pool_tokens, pool_tok_stride;
  int64_t n_tokens;
  int q_heads, kv_heads;
  float eps;
  int32_t* status;
};

struct Vec8 {
  float v[8];
};

__device__ __forceinline__ Vec8 unpack8(const uint4& u) {
  Vec8 r;
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    r.v[2 * i] = f.x;
    r.v[2 * i + 1] = f.y;
  }
  return r;
}

__device__ __forceinline__ uint4 pack8(const Vec8& x) {
  uint4 u;
  u.x = pack_half2(x.v[0], x.v[1]);
  u.y = pack_half2(x.v[2], x.v[3]);
  u.z = pack_half2(x.v[4], x.v[5]);
  u.w = pack_half2(x.v[6], x.v[7]);
  return u;
}

template <int D>
__global__ void __launch_bounds__(kPrologueThreads) qk_prologue_kernel(PrologueParams p) {
  constexpr int kLanes = D / 16;            // lanes per head row
  constexpr int kRowsPerWarp = 32 / kLanes;
  constexpr int kHalf = D / 2;
  cudaGridDependencySynchronize();
  cudaTriggerProgrammaticLaunchCompletion();

  const int lane = threadIdx.x & 31;
  const int sub = lane % kLanes;            // position inside the row
  const int rows_per_token = p.q_heads + 2 * p.kv_heads;
  const int64_t total_rows = p.n_tokens * rows_per_token;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * kPrologueThreads + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * kPrologueThreads) >> 5;

  for (int64_t base = warp * kRowsPerWarp; base < total_rows; base += n_warps * kRowsPerWarp) {
    const int64_t row = base + lane / kLanes;
    const bool live = row < total_rows;     // rows are padded to whole warps; dead lanes still shuffle
    const int64_t tok = live ? row / rows_per_token : 0;
    const int h = live ? static_cast<int>(row - tok * rows_per_token) : 0;
    const bool is_q = h < p.q_heads;
    const bool is_v = h >= p.q_heads + p.kv_heads;

    const __half* src = is_q ? p.q + tok * p.q_tok_stride + static_cast<int64_t>(h) * D
                             : p.kv + tok * p.kv_tok_stride + static_cast<int64_t>(h - p.q_heads) * D;
    uint4 ua = make_uint4(0, 0, 0, 0), ub = ua;
    if (live) {
      ua = __ldg(reinterpret_cast<const uint4*>(src + sub * 8));
      ub = __ldg(reinterpret_cast<const uint4*>(src + kHalf + sub * 8));
    }

    __half* dst = nullptr;
    if (live) {
      if (is_q) {
        dst = p.q_out + tok * p.q_out_tok_stride + static_cast<int64_t>(h) * D;
      } else {
        const int64_t slot = __ldg(p.slots + tok);
        if (slot < 0 || slot >= p.pool_tokens) {
          set_status(p.status, B200KV_DEV_BAD_SLOT);
        } else {
          dst = p.pool + slot * p.pool_tok_stride + static_cast<int64_t>(h - p.q_heads) * D;
        }
      }
    }

    // Sum of squares over the row.  The row's kLanes lanes are consecutive, so xor-shuffles below
    // kLanes stay inside it; every lane of the warp takes part (V rows and dead lanes too), which
    // keeps the shuffle outside any divergent branch.
    Vec8 a = unpack8(ua), b = unpack8(ub);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += a.v[i] * a.v[i] + b.v[i] * b.v[i];
#pragma unroll
    for (int m = 1; m < kLanes; m <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);

    if (!is_v) {
      const __half* w = is_q ? p.q_weight : p.k_weight;
      if (w != nullptr) {
        const float rrms = 1.0f / sqrtf(ss * (1.0f / D) + p.eps);
        const uint4 wa_u = __ldg(reinterpret_cast<const uint4*>(w + sub * 8));
        const uint4 wb_u = __ldg(reinterpret_cast<const uint4*>(w + kHalf + sub * 8));
        const __half* wa = reinterpret_cast<const __half*>(&wa_u);
        const __half* wb = reinterpret_cast<const __half*>(&wb_u);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          a.v[i] = __half2float(__hmul(__float2half_rn(a.v[i] * rrms), wa[i]));
          b.v[i] = __half2float(__hmul(__float2half_rn(b.v[i] * rrms), wb[i]));
        }
      }
      const __half* crow = p.cos + tok * p.cs_tok_stride + sub * 8;
      const __half* srow = p.sin + tok * p.cs_tok_stride + sub * 8;
      const Vec8 c = unpack8(__ldg(reinterpret_cast<const uint4*>(crow)));
      const Vec8 s = unpack8(__ldg(reinterpret_cast<const uint4*>(srow)));
      Vec8 oa, ob;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        oa.v[i] = a.v[i] * c.v[i] - b.v[i] * s.v[i];
        ob.v[i] = b.v[i] * c.v[i] + a.v[i] * s.v[i];
      }
      ua = pack8(oa);
      ub = pack8(ob);
    }
    if (dst != nullptr) {
      *reinterpret_cast<uint4*>(dst + sub * 8) = ua;
      *reinterpret_cast<uint4*>(dst + kHalf + sub * 8) = ub;
    }
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <int D>
int launch(const PrologueParams& p, cudaStream_t stream) {
  constexpr int kRowsPerBlock = (kPrologueThreads / 32) * (32 / (D / 16));
  const int64_t total_rows = p.n_tokens * (p.q_heads + 2 * p.kv_heads);
  const int sms = device_sm_count();
  if (sms <= 0) return B200KV_ECUDA;
  int64_t blocks = (total_rows + kRowsPerBlock - 1) / kRowsPerBlock;
  const int64_t cap = static_cast<int64_t>(sms) * 8;   // 8 resident CTAs of 256 threads per SM
  if (blocks > cap) blocks = cap;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(blocks));
  cfg.blockDim = dim3(kPrologueThreads);
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, qk_prologue_kernel<D>, p);
  if (e != cudaSuccess) return record_cuda_error(e);
  return check_launch();
}

}  // namespace

int qk_norm_rope_append(const PrologueArgs& a, cudaStream_t stream) {
  if (a.n_tokens < 0 || a.q_heads <= 0 || a.kv_heads <= 0 || a.pool_tokens < 0) return B200KV_EINVAL;
  if (a.head_dim != 64 && a.head_dim != 128) return B200KV_EUNSUPPORTED;
  if (a.n_tokens == 0) return B200KV_OK;
  if (!a.q || !a.q_out || !a.kv || !a.cos || !a.sin || !a.slots || !a.pool) return B200KV_EINVAL;
  if (!(a.eps >= 0.f)) return B200KV_EINVAL;
  const int64_t d = a.head_dim;
  if (a.q_tok_stride % 8 || a.q_out_tok_stride % 8 || a.kv_tok_stride % 8 || a.cs_tok_stride % 8 ||
      a.pool_tok_stride % 8)
    return B200KV_EALIGN;
  if (!aligned16(a.q) || !aligned16(a.q_out) || !aligned16(a.kv) || !aligned16(a.cos) ||
      !aligned16(a.sin) || !aligned16(a.pool) || (a.q_weight && !aligned16(a.q_weight)) ||
      (a.k_weight && !aligned16(a.k_weight)))
    return B200KV_EALIGN;
  if (a.q_tok_stride < a.q_heads * d || a.q_out_tok_stride < a.q_heads * d ||
      a.kv_tok_stride < 2 * a.kv_heads * d || a.pool_tok_stride < 2 * a.kv_heads * d ||
      a.cs_tok_stride < d / 2)
    return B200KV_EINVAL;
  PrologueParams p{};
  p.q = static_cast<const __half*>(a.q);
  p.q_out = static_cast<__half*>(a.q_out);
  p.q_tok_stride = a.q_tok_stride;
  p.q_out_tok_stride = a.q_out_tok_stride;
  p.kv = static_cast<const __half*>(a.kv);
  p.kv_tok_stride = a.kv_tok_stride;
  p.q_weight = static_cast<const __half*>(a.q_weight);
  p.k_weight = static_cast<const __half*>(a.k_weight);
  p.cos = static_cast<const __half*>(a.cos);
  p.sin = static_cast<const __half*>(a.sin);
  p.cs_tok_stride = a.cs_tok_stride;
  p.slots = a.slots;
  p.pool = static_cast<__half*>(a.pool);
  p.pool_tokens = a.pool_tokens;
  p.pool_tok_stride = a.pool_tok_stride;
  p.n_tokens = a.n_tokens;
  p.q_heads = a.q_heads;
  p.kv_heads = a.kv_heads;
  p.eps = a.eps;
  p.status = a.status;
  return a.head_dim == 128 ? launch<128>(p, stream) : launch<64>(p, stream);
}

}  // namespace b200kv
