// Packed causal prefill over paged KV with history, on the 5th-generation tensor cores.
//
// Replaces paged_chunk_flash_attention of the reference
// (lite_llama/kernels/paged_chunk_flashattention.py:227-327; Triton kernel :58-176, torch
// statement :179-222) and, with zero history over dense K/V, flash_attention2_no_pad
// (lite_llama/kernels/flashattention2_nopad.py:171-221): query row i of request r sits at
// logical position ctx_r + i and attends to keys 0 .. ctx_r + i of that request.
//
// One CTA = one (request, 128-row query tile, query head).  Six warps:
//   warp 4  producer : TMA (cp.async.bulk.tensor) of the Q tile once, then of the K and V pages of
//                      each 64-key tile into a 2-stage ring; pages come through the block/token
//                      table, each page of one head is two 16-row x 128-byte swizzled boxes;
//   warp 5  MMA      : one lane issues tcgen05.mma: S = Q K^T (M128 N64 K16 x 8) into TMEM, and,
//                      once the softmax warps have published P, O += P V (M128 N128 K16 x 4) into
//                      a second TMEM region; tcgen05.commit signals mbarriers;
//   warps 0-3 softmax: thread i owns query row i = TMEM lane i: tcgen05.ld of its S row, causal
//                      mask, online softmax in the log2 domain (exp2), P rounded to fp16 and
//                      written to shared memory in the UMMA K-major 128-byte-swizzled layout; O
//                      accumulates in TMEM and is rescaled only when the row maximum has grown
//                      by more than a factor 2^8 since the last rescale.
// S for tile j+1 is issued as soon as the softmax warps have read S_j, so the tensor core works
// while they exponentiate; two CTAs per SM (112 KB of shared memory, 256 TMEM columns each)
// interleave their phases.  Operands are fp16, accumulation fp32, P is rounded to fp16 before
// P V as in the reference (:166, :220), output fp16.  Tensor-bound:
// flops = 4 * 128 * sum over (query, visible key) pairs, per query head.
//
// Every wait is an mbarrier try-wait bounded by ~2 s of %globaltimer; a wait that runs out sets
// B200KV_DEV_WAIT_TIMEOUT, and every warp still reaches the common exit where TMEM is freed.
#include "common.cuh"
#include "launch.h"
#include "tma.h"

namespace b200kv {

namespace {

constexpr int kD = 128;
constexpr int kPS = 16;
constexpr int kBM = 128;             // query rows per CTA
constexpr int kBN = 64;              // keys per pipeline tile
constexpr int kTilePages = kBN / kPS;
constexpr int kStages = 2;
constexpr int kSoftmaxWarps = 4;
constexpr int kProducerWarp = 4;
constexpr int kMmaWarp = 5;
constexpr int kThreads = 6 * 32;
constexpr int kQBytes = kBM * kD * 2;          // 32 KB: [2 d-chunks][128 rows][128 B]
constexpr int kKBytes = kBN * kD * 2;          // 16 KB: [2 d-chunks][64 keys][128 B]
constexpr int kVBytes = kKBytes;
constexpr int kPBytes = kBM * kBN * 2;         // 16 KB: [128 rows][128 B]
constexpr int kHalfPage = kPS * 128;           // one TMA box: 16 rows x 128 B
constexpr int kTmemCols = 256;                 // S at column 0 (64 used), O at column 128
constexpr int kTmemPV = 128;
constexpr int kSmemBytes = kQBytes + kStages * (kKBytes + kVBytes) + kPBytes + 128;

// tcgen05 instruction descriptor, kind::f16: fp16 A/B, fp32 accumulate.
//   bits [4,6) D format (1 = f32), [7,10) A format (0 = f16), [10,13) B format (0 = f16),
//   bit 15 A major (0 = K), bit 16 B major (0 = K, 1 = MN), [17,23) N >> 3, [24,29) M >> 4.
constexpr uint32_t make_idesc(int m, int n, int b_mn_major) {
  return (1u << 4) | (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}
constexpr uint32_t kIdescS = make_idesc(kBM, kBN, 0);
constexpr uint32_t kIdescPV = make_idesc(kBM, kD, 1);

// Shared-memory matrix descriptor for 128-byte-swizzled operands: start address >> 4 in bits
// [0,14), leading byte offset >> 4 in [16,30), stride byte offset >> 4 in [32,46), descriptor
// version 1 in [46,48), layout type SWIZZLE_128B (2) in [61,64).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

struct PrefillParams {
  const int32_t* table;
  int64_t table_row_stride;
  int table_kind;
  const int32_t* req_ids;
  const int32_t* q_start;
  const void* ctx_lens;
  const void* q_lens;
  int lens_i64;
  int batch;
  int64_t total_q, pool_tokens;
  int q_heads, group;
  float scale_log2;
  __half* out;
  int64_t out_stride_t, out_stride_h;
  int32_t* status;
  int tiles_m;
};

__global__ void __launch_bounds__(kThreads, 2)
paged_prefill_kernel(PrefillParams p, const __grid_constant__ CUtensorMap qmap,
                     const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;

  // ---- which tile is this? (heavy query tiles first) -----------------------------------------
  const int head = blockIdx.x;
  const int mt = p.tiles_m - 1 - static_cast<int>(blockIdx.y);
  const int b = blockIdx.z;
  int64_t q_len = load_len(p.q_lens, p.lens_i64, b);
  int64_t ctx = load_len(p.ctx_lens, p.lens_i64, b);
  if (q_len < 0 || ctx < 0) {
    set_status(p.status, B200KV_DEV_BAD_LENGTH);
    return;
  }
  const int64_t row0 = static_cast<int64_t>(mt) * kBM;  // first query row of the tile in its request
  if (row0 >= q_len) return;
  const int rows = static_cast<int>(q_len - row0 < kBM ? q_len - row0 : kBM);
  const int64_t q_tok0 = static_cast<int64_t>(__ldg(p.q_start + b)) + row0;  // packed row of tile row 0
  if (q_tok0 < 0 || q_tok0 + rows > p.total_q) {
    set_status(p.status, B200KV_DEV_BAD_LENGTH);
    return;
  }
  const int64_t kv_len = ctx + row0 + rows;               // keys visible to the tile's last row
  const int n_tiles = static_cast<int>((kv_len + kBN - 1) / kBN);
  const int64_t n_pages = (kv_len + kPS - 1) / kPS;
  const int kv_head = head / p.group;
  const int table_row = p.req_ids ? __ldg(p.req_ids + b) : b;

  // ---- shared memory carve-up -----------------------------------------------------------------
  const uint32_t sm_q = smem_u32(smem);
  const uint32_t sm_k = sm_q + kQBytes;                     // [stage][16 KB]
  const uint32_t sm_v = sm_k + kStages * kKBytes;           // [stage][16 KB]
  const uint32_t sm_p = sm_v + kStages * kVBytes;
  const uint32_t sm_bar = sm_p + kPBytes;
  const uint32_t bar_q = sm_bar;
  const uint32_t bar_kfull = sm_bar + 8;                    // [2]
  const uint32_t bar_vfull = sm_bar + 24;                   // [2]
  const uint32_t bar_kvempty = sm_bar + 40;                 // [2]
  const uint32_t bar_sfull = sm_bar + 56;
  const uint32_t bar_sfree = sm_bar + 64;
  const uint32_t bar_pfull = sm_bar + 72;
  const uint32_t bar_pvfull = sm_bar + 80;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + (sm_bar - sm_q) + 96);
  if ((sm_q & 1023u) != 0) {  // swizzled boxes and UMMA descriptors assume 1024-byte alignment
    set_status(p.status, B200KV_DEV_BAD_PAGE);
    return;
  }

  if (tid == 0) {
    mbar_init(bar_q, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar_kfull + 8 * i, 1);
      mbar_init(bar_vfull + 8 * i, 1);
      mbar_init(bar_kvempty + 8 * i, 1);
    }
    mbar_init(bar_sfull, 1);
    mbar_init(bar_sfree, kSoftmaxWarps * 32);
    mbar_init(bar_pfull, kSoftmaxWarps * 32);
    mbar_init(bar_pvfull, 1);
    fence_barrier_init();
  }
  if (warp == kMmaWarp) {  // TMEM allocation is a warp-wide operation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                     smem_u32(tmem_slot)),
                 "n"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  cudaGridDependencySynchronize();  // q and the pool belong to earlier kernels until here
  cudaTriggerProgrammaticLaunchCompletion();

  if (warp == kProducerWarp) {
    // ============================== TMA producer ============================================
    const uint64_t policy_kv = l2_evict_first_policy();
    if (lane == 0) {
      prefetch_tensormap(&qmap);
      prefetch_tensormap(&kmap);
      prefetch_tensormap(&vmap);
      mbar_arrive_expect_tx(bar_q, kQBytes);
      // Rows past this request's q_len are the next request's rows (or zero fill past the end);
      // their results are never stored.
      tma_load_3d(sm_q, &qmap, bar_q, 0, head, static_cast<int>(q_tok0), policy_kv);
      tma_load_3d(sm_q + kQBytes / 2, &qmap, bar_q, 64, head, static_cast<int>(q_tok0), policy_kv);
    }
    const int my_page = lane >> 2;   // lanes 0..15: page of the tile
    const int my_part = lane & 3;    // K low, K high, V low, V high half of head_dim
    const bool is_v = (my_part & 2) != 0;
    const int32_t* trow = p.table + static_cast<int64_t>(table_row) * p.table_row_stride;
    const int64_t dense0 = static_cast<int64_t>(__ldg(p.q_start + b));
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j % kStages;
      if (j >= kStages && !mbar_wait_bounded(bar_kvempty + 8 * st, ((j / kStages) - 1) & 1)) {
        set_status(p.status, B200KV_DEV_WAIT_TIMEOUT);
        break;
      }
      const int64_t page0 = static_cast<int64_t>(j) * kTilePages;
      const int np = static_cast<int>(n_pages - page0 < kTilePages ? n_pages - page0 : kTilePages);
      if (lane == 0) {
        mbar_arrive_expect_tx(bar_kfull + 8 * st, np * 2 * kHalfPage);
        mbar_arrive_expect_tx(bar_vfull + 8 * st, np * 2 * kHalfPage);
      }
      __syncwarp();
      if (lane < 4 * np) {
        const int64_t lp = page0 + my_page;
        int64_t slot;
        if (p.table_kind == B200KV_TABLE_BLOCK) slot = static_cast<int64_t>(__ldg(trow + lp)) * kPS;
        else if (p.table_kind == B200KV_TABLE_TOKEN) slot = static_cast<int64_t>(__ldg(trow + lp * kPS));
        else slot = dense0 + lp * kPS;   // dense packed K/V: token t of the request at q_start + t
        if (slot < 0 || slot >= p.pool_tokens) {
          set_status(p.status, B200KV_DEV_BAD_PAGE);
          slot = 0;  // never dereference a bad entry: report it and read page 0 instead
        }
        const uint32_t dst = (is_v ? sm_v + st * kVBytes : sm_k + st * kKBytes) +
                             (my_part & 1) * (kKBytes / 2) + my_page * kHalfPage;
        tma_load_3d(dst, is_v ? &vmap : &kmap, (is_v ? bar_vfull : bar_kfull) + 8 * st,
                    (my_part & 1) * 64, kv_head, static_cast<int>(slot), policy_kv);
      }
    }
  } else if (warp == kMmaWarp) {
    // ============================== MMA issuer ==============================================
    if (lane == 0) {
      bool ok = mbar_wait_bounded(bar_q, 0);
      const uint32_t tmem_s = tmem_base;
      const uint32_t tmem_pv = tmem_base + kTmemPV;
      auto issue_s = [&](int j) {
        const int st = j % kStages;
        if (!mbar_wait_bounded(bar_kfull + 8 * st, (j / kStages) & 1)) return false;
        if (j > 0 && !mbar_wait_bounded(bar_sfree, (j - 1) & 1)) return false;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks) {
          const uint64_t a = smem_desc(sm_q + (ks >> 2) * (kQBytes / 2) + (ks & 3) * 32, 16, 1024);
          const uint64_t bd =
              smem_desc(sm_k + st * kKBytes + (ks >> 2) * (kKBytes / 2) + (ks & 3) * 32, 16, 1024);
          umma_f16(tmem_s, a, bd, kIdescS, ks > 0 ? 1u : 0u);
        }
        umma_commit(bar_sfull);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int st = j % kStages;
        if (j + 1 < n_tiles) ok = issue_s(j + 1);   // S of the next tile overlaps this tile's softmax
        if (!ok) break;
        if (!mbar_wait_bounded(bar_pfull, j & 1) || !mbar_wait_bounded(bar_vfull + 8 * st, (j / kStages) & 1)) {
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < kBN / 16; ++ks) {
          const uint64_t a = smem_desc(sm_p + ks * 32, 16, 1024);
          // V tile is MN-major for B: 64 head_dim values contiguous (128 B), next 64 at +8 KB (LBO),
          // 8-key groups 1024 B apart (SBO); a K step of 16 keys advances 16 rows = 2048 B.
          const uint64_t bd = smem_desc(sm_v + st * kVBytes + ks * 2048, kVBytes / 2, 1024);
          umma_f16(tmem_pv, a, bd, kIdescPV, (j > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(bar_pvfull);
        umma_commit(bar_kvempty + 8 * st);
      }
      if (!ok) set_status(p.status, B200KV_DEV_WAIT_TIMEOUT);
    }
  } else {
    // ============================== softmax warps ===========================================
    // O accumulates in TMEM.  The running maximum used to scale P and O (m_used) is only moved
    // when the true row maximum has grown by more than 8 (a factor 256, harmless for fp16 P and
    // fp32 accumulation): then O and l are rescaled once; otherwise a tile costs no pass over O.
    const int row = tid;                                   // query row of the tile = TMEM lane
    const uint32_t t_lane = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t tmem_o = tmem_base + t_lane + kTmemPV;
    const int64_t q_pos = ctx + row0 + row;                // logical position of this query row
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      if (!mbar_wait_bounded(bar_sfull, j & 1)) { ok = false; break; }
      tc_fence_after();
      uint32_t sr[2][32];
      tmem_ld32(tmem_base + t_lane + 0, sr[0]);
      tmem_ld32(tmem_base + t_lane + 32, sr[1]);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(bar_sfree);                              // S_j is in registers: S_{j+1} may start
      const int64_t key0 = static_cast<int64_t>(j) * kBN;
      const bool need_mask = key0 + kBN - 1 > ctx + row0;  // tile reaches past the first row's diagonal
      float sv[kBN];
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < kBN; ++c) {
        float sc = __uint_as_float(sr[c >> 5][c & 31]) * p.scale_log2;
        if (need_mask && key0 + c > q_pos) sc = -INFINITY;
        sv[c] = sc;
        mx = fmaxf(mx, sc);
      }
      // P_{j-1} and O are free once PV_{j-1} has completed.
      if (j > 0 && !mbar_wait_bounded(bar_pvfull, (j - 1) & 1)) { ok = false; break; }
      const bool grow = mx > m_used + 8.f;                 // also true on the first tile (m_used = -inf)
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = grow ? mx : m_used;
        const float alpha = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_new);
        l_run *= alpha;
        m_used = m_new;
        if (j > 0) {                                       // rescale this warp's 32 rows of O
          tc_fence_after();
#pragma unroll
          for (int q4 = 0; q4 < kD / 32; ++q4) {
            uint32_t ov[32];
            tmem_ld32(tmem_o + q4 * 32, ov);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tmem_st32(tmem_o + q4 * 32, ov);
          }
          tmem_st_wait();
          tc_fence_before();
        }
      }
      const float msub = (m_used == -INFINITY) ? 0.f : m_used;
      float rs = 0.f;
      // P row -> shared memory, UMMA K-major layout with the 128-byte swizzle: row r at r*128 B,
      // its eight 16-byte chunks XOR-ed with r % 8.
      const uint32_t prow = sm_p + row * 128;
#pragma unroll
      for (int ch = 0; ch < kBN / 8; ++ch) {
        uint32_t pk[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p0 = fast_exp2(sv[ch * 8 + 2 * e] - msub);
          const float p1 = fast_exp2(sv[ch * 8 + 2 * e + 1] - msub);
          rs += p0 + p1;
          pk[e] = pack_half2(p0, p1);
        }
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};\n" ::"r"(prow + ((ch ^ (row & 7)) << 4)),
                     "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3])
                     : "memory");
      }
      l_run += rs;
      if (j == n_tiles - 1) {
        // Keys past kv_len in the last tile were either not loaded or lie in never-written pool
        // slots; their P is 0 but 0 * NaN would still poison the row, so zero those V rows.
        const int st = j % kStages;
        const int valid = static_cast<int>(kv_len - key0);
        if (valid < kBN) {
          if (!mbar_wait_bounded(bar_vfull + 8 * st, (j / kStages) & 1)) { ok = false; break; }
          for (int i = tid; i < (kBN - valid) * 16; i += kSoftmaxWarps * 32) {
            const int r = valid + (i >> 4);
            const int c = i & 15;
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n" ::"r"(
                             sm_v + st * kVBytes + (c >> 3) * (kVBytes / 2) + r * 128 + ((c & 7) << 4)),
                         "r"(0)
                         : "memory");
          }
        }
      }
      fence_proxy_async_smem();                            // P (and V fix-ups) visible to the tensor core
      mbar_arrive(bar_pfull);
    }
    if (ok && !mbar_wait_bounded(bar_pvfull, (n_tiles - 1) & 1)) ok = false;
    if (!ok) set_status(p.status, B200KV_DEV_WAIT_TIMEOUT);
    if (ok) {
      tc_fence_after();
      const float inv = 1.f / l_run;
      __half* op = p.out + (q_tok0 + row) * p.out_stride_t + static_cast<int64_t>(head) * p.out_stride_h;
#pragma unroll
      for (int q4 = 0; q4 < kD / 32; ++q4) {
        uint32_t ov[32];
        tmem_ld32(tmem_o + q4 * 32, ov);                   // warp-collective: every lane takes part
        tmem_ld_wait();
        if (row < rows) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint4 v;
            v.x = pack_half2(__uint_as_float(ov[c * 8 + 0]) * inv, __uint_as_float(ov[c * 8 + 1]) * inv);
            v.y = pack_half2(__uint_as_float(ov[c * 8 + 2]) * inv, __uint_as_float(ov[c * 8 + 3]) * inv);
            v.z = pack_half2(__uint_as_float(ov[c * 8 + 4]) * inv, __uint_as_float(ov[c * 8 + 5]) * inv);
            v.w = pack_half2(__uint_as_float(ov[c * 8 + 6]) * inv, __uint_as_float(ov[c * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(op + q4 * 32 + c * 8) = v;
          }
        }
      }
      tc_fence_before();
    }
  }

  // ---- common exit: every warp gets here (all waits above are bounded) ----------------------
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "n"(kTmemCols)
                 : "memory");
  }
}

// Tensor map over packed Q: element (d, head, token) at q + token*stride_t + head*stride_h + d;
// box = 64 halves x 1 head x 128 tokens (one half of a query tile), 128-byte swizzle.
int encode_q_tensor_map(CUtensorMap* out, const void* q, int64_t total_q, int64_t stride_t,
                        int64_t stride_h, int heads) {
  return encode_kv_tensor_map(out, q, total_q, stride_t, stride_h, heads, kD, kBM);
}

}  // namespace

int paged_prefill(const PrefillArgs& a, cudaStream_t stream) {
  if (a.batch < 0 || a.total_q < 0 || a.max_q_len < 0 || a.q_heads <= 0 || a.kv_heads <= 0)
    return B200KV_EINVAL;
  if (a.batch == 0 || a.total_q == 0 || a.max_q_len == 0) return B200KV_OK;
  if (!a.q || !a.k_base || !a.v_base || !a.q_start || !a.ctx_lens || !a.q_lens || !a.out)
    return B200KV_EINVAL;
  if (a.table_kind != B200KV_TABLE_BLOCK && a.table_kind != B200KV_TABLE_TOKEN &&
      a.table_kind != B200KV_TABLE_DENSE)
    return B200KV_EINVAL;
  if (a.table_kind != B200KV_TABLE_DENSE && !a.table) return B200KV_EINVAL;
  if (a.head_dim != kD || a.page_size != kPS) return B200KV_EUNSUPPORTED;
  if (a.q_heads % a.kv_heads != 0) return B200KV_EUNSUPPORTED;
  if (a.batch > 65535 || a.q_heads > 65535 * 16) return B200KV_ETOOLARGE;
  if (a.pool_tokens <= 0 || a.pool_tokens > (int64_t{1} << 31) - 1 || a.total_q > (int64_t{1} << 31) - 1)
    return B200KV_ETOOLARGE;
  if ((reinterpret_cast<uintptr_t>(a.out) & 15u) != 0 || a.out_stride_t % 8 != 0 || a.out_stride_h % 8 != 0)
    return B200KV_EALIGN;

  CUtensorMap qmap, kmap, vmap;
  int rc = encode_q_tensor_map(&qmap, a.q, a.total_q, a.q_stride_t, a.q_stride_h, a.q_heads);
  if (rc != B200KV_OK) return rc;
  rc = encode_kv_tensor_map(&kmap, a.k_base, a.pool_tokens, a.kv_tok_stride, a.kv_head_stride,
                            a.kv_heads, kD, kPS);
  if (rc != B200KV_OK) return rc;
  rc = encode_kv_tensor_map(&vmap, a.v_base, a.pool_tokens, a.kv_tok_stride, a.kv_head_stride,
                            a.kv_heads, kD, kPS);
  if (rc != B200KV_OK) return rc;

  PrefillParams p{};
  p.table = a.table;
  p.table_row_stride = a.table_row_stride;
  p.table_kind = a.table_kind;
  p.req_ids = a.req_ids;
  p.q_start = a.q_start;
  p.ctx_lens = a.ctx_lens;
  p.q_lens = a.q_lens;
  p.lens_i64 = a.lens_i64;
  p.batch = a.batch;
  p.total_q = a.total_q;
  p.pool_tokens = a.pool_tokens;
  p.q_heads = a.q_heads;
  p.group = a.q_heads / a.kv_heads;
  p.scale_log2 = a.scale_log2;
  p.out = static_cast<__half*>(a.out);
  p.out_stride_t = a.out_stride_t;
  p.out_stride_h = a.out_stride_h;
  p.status = a.status;
  p.tiles_m = static_cast<int>((a.max_q_len + kBM - 1) / kBM);
  if (p.tiles_m > 65535) return B200KV_ETOOLARGE;

  static bool attr_done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return record_cuda_error(cudaGetLastError());
  if (dev < 0 || dev >= 64 || !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(paged_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBytes);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev >= 0 && dev < 64) attr_done[dev] = true;
  }
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(a.q_heads), static_cast<unsigned>(p.tiles_m),
                     static_cast<unsigned>(a.batch));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, paged_prefill_kernel, p, qmap, kmap, vmap);
  if (e != cudaSuccess) return record_cuda_error(e);
  return check_launch();
}

}  // namespace b200kv
