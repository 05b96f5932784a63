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
  int n_tokens;
  int q_heads, kv_heads;
  int groups_per_token;     // ceil((q_heads + 2*kv_heads) / rows per warp)
  int step_tok, step_grp;   // (warps in the grid) / and % groups_per_token
  float eps;
  int32_t* status;
};

__device__ __forceinline__ float2 h2f(uint32_t u) {
  return __half22float2(*reinterpret_cast<const __half2*>(&u));
}

// One 16-byte slice (8 halves) of a row: x*rrms rounded to fp16, times the fp16 weight in fp16.
__device__ __forceinline__ void norm8(float (&x)[8], float rrms, const uint4& w) {
  const uint32_t* wp = reinterpret_cast<const uint32_t*>(&w);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 y = __floats2half2_rn(x[2 * i] * rrms, x[2 * i + 1] * rrms);
    const float2 f = __half22float2(__hmul2(y, *reinterpret_cast<const __half2*>(wp + i)));
    x[2 * i] = f.x;
    x[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&x)[8]) {
  const uint32_t* p = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = h2f(p[i]);
    x[2 * i] = f.x;
    x[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
  return make_uint4(pack_half2(x[0], x[1]), pack_half2(x[2], x[3]), pack_half2(x[4], x[5]),
                    pack_half2(x[6], x[7]));
}

// A warp takes one "group" of 32/kLanes consecutive head rows of ONE token per iteration, so the
// token's slot, cos and sin are the same for the whole warp, and walks (token, group) pairs with
// precomputed steps: no division in the loop.
template <int D>
__global__ void __launch_bounds__(kPrologueThreads) qk_prologue_kernel(PrologueParams p) {
  constexpr int kLanes = D / 16;            // lanes per head row
  constexpr int kRowsPerWarp = 32 / kLanes;
  constexpr int kHalf = D / 2;
  cudaGridDependencySynchronize();
  cudaTriggerProgrammaticLaunchCompletion();

  const int lane = threadIdx.x & 31;
  const int sub = lane % kLanes;            // position inside the row: fixed for the thread
  const int rows_per_token = p.q_heads + 2 * p.kv_heads;
  const unsigned warp = (blockIdx.x * kPrologueThreads + threadIdx.x) >> 5;
  int tok = static_cast<int>(warp / static_cast<unsigned>(p.groups_per_token));
  int grp = static_cast<int>(warp % static_cast<unsigned>(p.groups_per_token));

  // The thread's slice of both norm weights never changes: keep it in registers.
  uint4 wq0, wq1, wk0, wk1;
  wq0 = wq1 = wk0 = wk1 = make_uint4(0, 0, 0, 0);
  if (p.q_weight != nullptr) {
    wq0 = __ldg(reinterpret_cast<const uint4*>(p.q_weight + sub * 8));
    wq1 = __ldg(reinterpret_cast<const uint4*>(p.q_weight + kHalf + sub * 8));
  }
  if (p.k_weight != nullptr) {
    wk0 = __ldg(reinterpret_cast<const uint4*>(p.k_weight + sub * 8));
    wk1 = __ldg(reinterpret_cast<const uint4*>(p.k_weight + kHalf + sub * 8));
  }

  for (; tok < p.n_tokens;) {
    const int h = grp * kRowsPerWarp + lane / kLanes;
    const bool live = h < rows_per_token;   // the last group of a token may be ragged
    const int kind = h < p.q_heads ? 0 : (h < p.q_heads + p.kv_heads ? 1 : 2);   // Q, K, V row
    const int64_t t = tok;

    uint4 ua = make_uint4(0, 0, 0, 0), ub = ua, uc = ua, us = ua;
    __half* dst = nullptr;
    if (live) {
      const __half* src = kind == 0 ? p.q + t * p.q_tok_stride + h * D
                                    : p.kv + t * p.kv_tok_stride + (h - p.q_heads) * D;
      ua = __ldg(reinterpret_cast<const uint4*>(src + sub * 8));
      ub = __ldg(reinterpret_cast<const uint4*>(src + kHalf + sub * 8));
      if (kind != 2) {
        uc = __ldg(reinterpret_cast<const uint4*>(p.cos + t * p.cs_tok_stride + sub * 8));
        us = __ldg(reinterpret_cast<const uint4*>(p.sin + t * p.cs_tok_stride + sub * 8));
      }
      if (kind == 0) {
        dst = p.q_out + t * p.q_out_tok_stride + h * D;
      } else {
        const int64_t slot = __ldg(p.slots + tok);
        if (slot < 0 || slot >= p.pool_tokens) {
          set_status(p.status, B200KV_DEV_BAD_SLOT);
        } else {
          dst = p.pool + slot * p.pool_tok_stride + (h - p.q_heads) * D;
        }
      }
    }

    // Sum of squares over the row.  The row's kLanes lanes are consecutive, so xor-shuffles below
    // kLanes stay inside it; every lane of the warp takes part (V rows and dead lanes too), which
    // keeps the shuffle outside any divergent branch.
    float a[8], b[8];
    unpack8(ua, a);
    unpack8(ub, b);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += a[i] * a[i] + b[i] * b[i];
#pragma unroll
    for (int m = 1; m < kLanes; m <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);

    if (kind != 2) {
      if ((kind == 0 ? p.q_weight : p.k_weight) != nullptr) {
        // correctly rounded sqrt and divide: the fast-math forms would move more values across
        // an fp16 rounding boundary than the summation order already does
        const float rrms = __fdiv_rn(1.0f, __fsqrt_rn(ss * (1.0f / D) + p.eps));
        norm8(a, rrms, kind == 0 ? wq0 : wk0);
        norm8(b, rrms, kind == 0 ? wq1 : wk1);
      }
      float c[8], s[8];
      unpack8(uc, c);
      unpack8(us, s);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float x1 = a[i], x2 = b[i];
        a[i] = x1 * c[i] - x2 * s[i];
        b[i] = x2 * c[i] + x1 * s[i];
      }
      ua = pack8(a);
      ub = pack8(b);
    }
    if (dst != nullptr) {
      *reinterpret_cast<uint4*>(dst + sub * 8) = ua;
      *reinterpret_cast<uint4*>(dst + kHalf + sub * 8) = ub;
    }

    tok += p.step_tok;
    grp += p.step_grp;
    if (grp >= p.groups_per_token) {
      grp -= p.groups_per_token;
      ++tok;
    }
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <int D>
int launch(PrologueParams p, cudaStream_t stream) {
  constexpr int kRowsPerWarp = 32 / (D / 16);
  constexpr int kWarpsPerBlock = kPrologueThreads / 32;
  p.groups_per_token = (p.q_heads + 2 * p.kv_heads + kRowsPerWarp - 1) / kRowsPerWarp;
  const int64_t groups = static_cast<int64_t>(p.n_tokens) * p.groups_per_token;
  const int sms = device_sm_count();
  if (sms <= 0) return B200KV_ECUDA;
  int64_t blocks = (groups + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const int64_t cap = static_cast<int64_t>(sms) * 8;   // grid-stride above 8 CTAs of 256 threads per SM
  if (blocks > cap) blocks = cap;
  const int64_t n_warps = blocks * kWarpsPerBlock;
  p.step_tok = static_cast<int>(n_warps / p.groups_per_token);
  p.step_grp = static_cast<int>(n_warps % p.groups_per_token);
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
  if (a.n_tokens > (1 << 30)) return B200KV_ETOOLARGE;
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
  p.n_tokens = static_cast<int>(a.n_tokens);
  p.q_heads = a.q_heads;
  p.kv_heads = a.kv_heads;
  p.eps = a.eps;
  p.status = a.status;
  return a.head_dim == 128 ? launch<128>(p, stream) : launch<64>(p, stream);
}

}  // namespace b200kv
