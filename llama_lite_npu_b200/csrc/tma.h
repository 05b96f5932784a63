// Host-side construction of TMA tensor maps for the paged KV pool, and the device-side
// mbarrier / bulk-tensor-copy primitives the kernels use (sm_100a inline PTX).
#pragma once

#include <cuda.h>  // CUtensorMap and its enums only; the encoder is resolved at run time
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200kv {

// Tensor map over one K or V view of a pool: element (d, head, token) at
// base + token*tok_stride + head*head_stride + d (fp16 elements).  The box is
// 64 halves x 1 head x box_tokens tokens, written to shared memory as box_tokens rows of
// 128 bytes with the 128-byte swizzle (16-byte chunk index XOR row%8), so one page of one
// head is fetched by two copies (d in [0,64) and [64,128)).  Returns B200KV_OK or an error.
int encode_kv_tensor_map(CUtensorMap* out, const void* base, int64_t pool_tokens,
                         int64_t tok_stride, int64_t head_stride, int n_heads, int head_dim,
                         int box_tokens);

// Same map through a small per-process cache keyed by every argument: encoding costs a driver
// call, and a serving loop passes the same few pool views (one per layer) on every step.
int cached_kv_tensor_map(CUtensorMap* out, const void* base, int64_t pool_tokens,
                         int64_t tok_stride, int64_t head_stride, int n_heads, int head_dim,
                         int box_tokens);

#ifdef __CUDACC__
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
// Make freshly initialised barriers visible to the async (TMA) proxy.
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking test of a barrier phase (for a thread that polls several barriers in turn).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Wait for a barrier phase, but never for longer than ~2 s: a wait that runs out returns false
// and the caller records B200KV_DEV_WAIT_TIMEOUT and leaves.  No wait in this library spins
// without such a bound.
constexpr uint64_t kWaitLimitNs = 2000000000ull;
// Same wait with an explicit limit (used by the self-test with a limit of a few milliseconds).
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
  const uint64_t t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > limit_ns) return false;
  }
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  // Fast path: a few thousand hardware-suspended tries without touching the clock (reading
  // %globaltimer costs far more than a try, and almost every wait ends here).
#pragma unroll 1
  for (int i = 0; i < 4096; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > kWaitLimitNs) return false;
  }
}
// 3-D tiled bulk tensor copy global -> shared of this CTA, completion counted in bytes on `bar`.
// The innermost coordinate c0 times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4, %5}], [%2], %6;\n"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2),
        "l"(policy)
      : "memory");
}
// Same box, but only brought into L2 (no shared-memory destination, no completion to wait for).
__device__ __forceinline__ void tma_prefetch_l2_3d(const CUtensorMap* map, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global [%0, {%1, %2, %3}];\n"
               :
               : "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
#endif  // __CUDACC__

}  // namespace b200kv
