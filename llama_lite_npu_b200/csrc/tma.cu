// cuTensorMapEncodeTiled is a driver-API entry point; it is resolved through the runtime
// (cudaGetDriverEntryPoint) so the library links against libcudart only.
#include "tma.h"

#include <cstdio>
#include <cstring>
#include <mutex>

#include "b200kv.h"
#include "common.cuh"
#include "launch.h"

namespace b200kv {

namespace {
// One CTA, 64 threads.  Barrier A gets its single arrival (the wait on it must succeed);
// barrier B never does (the wait on it must give up after limit_ns and report it).
__global__ void wait_selftest_kernel(uint64_t limit_ns, int32_t* result, int32_t* status) {
  __shared__ uint64_t bars[2];
  const uint32_t a = smem_u32(&bars[0]), b = smem_u32(&bars[1]);
  if (threadIdx.x == 0) {
    mbar_init(a, 1);
    mbar_init(b, 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 32) mbar_arrive(a);
  const bool got_a = mbar_wait_limit(a, 0, limit_ns);
  const bool got_b = mbar_wait_limit(b, 0, limit_ns);
  if (!got_b) set_status(status, B200KV_DEV_WAIT_TIMEOUT);
  if (threadIdx.x == 0) {
    result[0] = got_a ? 1 : 0;
    result[1] = got_b ? 1 : 0;
  }
}
}  // namespace

int wait_selftest(uint64_t limit_ns, int32_t* result, int32_t* status, cudaStream_t stream) {
  if (!result || limit_ns == 0 || limit_ns > 1000000000ull) return B200KV_EINVAL;
  wait_selftest_kernel<<<1, 64, 0, stream>>>(limit_ns, result, status);
  return check_launch();
}

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess) {
      record_cuda_error(e != cudaSuccess ? e : cudaErrorSymbolNotFound);
      return static_cast<EncodeTiledFn>(nullptr);
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

}  // namespace

int encode_kv_tensor_map(CUtensorMap* out, const void* base, int64_t pool_tokens,
                         int64_t tok_stride, int64_t head_stride, int n_heads, int head_dim,
                         int box_tokens) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return B200KV_ECUDA;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return B200KV_EALIGN;
  if ((tok_stride * 2) % 16 != 0 || (head_stride * 2) % 16 != 0) return B200KV_EALIGN;
  if (pool_tokens <= 0 || n_heads <= 0 || head_dim % 64 != 0 || box_tokens <= 0 || box_tokens > 256)
    return B200KV_EINVAL;
  // Dimensions fastest first: d, head, token.
  const cuuint64_t gdim[3] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(n_heads),
                              static_cast<cuuint64_t>(pool_tokens)};
  const cuuint64_t gstride[2] = {static_cast<cuuint64_t>(head_stride) * 2,
                                 static_cast<cuuint64_t>(tok_stride) * 2};
  const cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(box_tokens)};
  const cuuint32_t estride[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), gdim, gstride,
                  box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    record_cuda_error(cudaErrorInvalidValue);
    return B200KV_ECUDA;
  }
  return B200KV_OK;
}

namespace {
struct MapKey {
  const void* base;
  int64_t pool_tokens, tok_stride, head_stride;
  int n_heads, head_dim, box_tokens, pad;
};
struct MapEntry {
  MapKey key;
  bool used;
  CUtensorMap map;
};
constexpr int kMapCacheSize = 256;   // direct-mapped; a collision just re-encodes
MapEntry g_map_cache[kMapCacheSize];
std::mutex g_map_mutex;
}  // namespace

int cached_kv_tensor_map(CUtensorMap* out, const void* base, int64_t pool_tokens,
                         int64_t tok_stride, int64_t head_stride, int n_heads, int head_dim,
                         int box_tokens) {
  MapKey key{base, pool_tokens, tok_stride, head_stride, n_heads, head_dim, box_tokens, 0};
  uint64_t h = reinterpret_cast<uintptr_t>(base) >> 4;
  h ^= static_cast<uint64_t>(pool_tokens) * 0x9E3779B97F4A7C15ull;
  h ^= static_cast<uint64_t>(tok_stride) * 0xC2B2AE3D27D4EB4Full + static_cast<uint64_t>(box_tokens);
  h ^= h >> 29;
  MapEntry& e = g_map_cache[h % kMapCacheSize];
  {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    if (e.used && std::memcmp(&e.key, &key, sizeof(MapKey)) == 0) {
      *out = e.map;
      return B200KV_OK;
    }
  }
  const int rc = encode_kv_tensor_map(out, base, pool_tokens, tok_stride, head_stride, n_heads, head_dim,
                                      box_tokens);
  if (rc != B200KV_OK) return rc;
  std::lock_guard<std::mutex> lock(g_map_mutex);
  e.key = key;
  e.map = *out;
  e.used = true;
  return B200KV_OK;
}

}  // namespace b200kv
