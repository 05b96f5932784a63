// Packed causal prefill over paged KV with history, on the 5th-generation tensor cores.
//
// Replaces paged_chunk_flash_attention of the reference
// (lite_llama/kernels/paged_chunk_flashattention.py:227-327; Triton kernel :58-176, torch
// statement :179-222) and, with zero history over dense K/V, flash_attention2_no_pad
// (lite_llama/kernels/flashattention2_nopad.py:171-221): query row i of request r sits at
// logical position ctx_r + i and attends to keys 0 .. ctx_r + i of that request.
//
// One CTA = one (request, 128-row query tile, PAIR of query heads of one GQA group): the two
// heads are two 128 x 128 query tiles with identical causal structure that share every K/V tile,
// so K/V cross L2 -> shared memory once for both and the tensor core always has the other tile's
// MMAs to run while one tile is in its softmax.  A CTA then does a SECOND query tile of the same
// request and heads: tile t-1-k (many key tiles) is followed by tile k (few), which balances the
// causal work across CTAs and lets the second tile's Q / K / V loads, barriers and TMEM be ready
// while the first one drains.  Ten warps, one CTA per SM:
//   warp 8  producer : TMA (cp.async.bulk.tensor) of both Q tiles once, then of the K and V pages
//                      of each 128-key tile into a 3-slot ring of 32 KB slots in which K runs one
//                      tile ahead of V (K_0 K_1 V_0 K_2 V_1 ...), the order in which the tensor
//                      core finishes with them; pages come through the block/token table (entry
//                      fetched one item ahead), each page of one head is two 16-row x 128-byte
//                      swizzled boxes, one per lane;
//   warp 9  MMA      : one lane issues tcgen05.mma.cta_group::1.kind::f16, always as M128 N128 K16
//                      (the per-instruction cost of tcgen05.mma is nearly flat in N, so small-N
//                      instructions waste the tensor pipe): S_g = Q_g K^T (8 instructions) into
//                      TMEM, for key tile j+1 as soon as softmax group g holds S_g of tile j in
//                      registers (so it runs under that softmax), and O_g += P_g V (8
//                      instructions) once the group has published P_g; descriptors are built once
//                      and only their address field advances; tcgen05.commit signals mbarriers;
//   warps 0-3 / 4-7  : softmax group 0 / 1: thread i owns query row i = TMEM lane i of its tile:
//                      tcgen05.ld of its whole 128-column S row, causal mask on diagonal
//                      tiles only, online softmax in the log2 domain (3-input max, packed f32x2
//                      FFMA/ADD, exp2), P rounded to fp16 and written to shared memory in the UMMA
//                      K-major 128-byte-swizzled layout; O accumulates in TMEM and is rescaled only
//                      when the row maximum has grown by more than a factor 2^8 since the last
//                      rescale.
// TMEM: 512 columns (S_0, S_1, O_0, O_1: 128 each).  Shared memory: 2 x 32 KB Q, 2 x 32 KB P,
// 3 x 32 KB K/V ring.  Operands are fp16, accumulation fp32, P is rounded to fp16 before P V as
// in the reference (:166, :220), output fp16.  Tensor-bound:
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
constexpr int kBM = 128;             // query rows per tile
constexpr int kQBoxRows = 16;        // query rows per TMA box: 8 boxes per head_dim half of a tile, one per lane
constexpr int kBN = 128;             // keys per pipeline tile
constexpr int kTilePages = kBN / kPS;
constexpr int kSlots = 3;            // 32 KB ring slots shared by K and V tiles
constexpr int kGroups = 2;           // query tiles (heads) per CTA
constexpr int kGroupWarps = 4;       // softmax warps per tile
constexpr int kProducerWarp = kGroups * kGroupWarps;
constexpr int kMmaWarp = kProducerWarp + 1;
constexpr int kThreads = (kMmaWarp + 1) * 32;
constexpr int kQBytes = kBM * kD * 2;          // 32 KB: [2 d-chunks][128 rows][128 B]
constexpr int kTileBytes = kBN * kD * 2;       // 32 KB: K or V tile, [2 d-chunks][128 keys][128 B]
constexpr int kPBytes = kBM * kBN * 2;         // 32 KB: [2 key-chunks][128 rows][128 B]
constexpr int kHalfPage = kPS * 128;           // one TMA box: 16 rows x 128 B
constexpr int kTmemCols = 512;
constexpr int kTmemS = 0;                      // S_0 at 0, S_1 at 128
constexpr int kTmemO = 256;                    // O_0 at 256, O_1 at 384
constexpr int kBarBytes = 256;
constexpr int kSmemBytes = kGroups * (kQBytes + kPBytes) + kSlots * kTileBytes + kBarBytes;

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

// Packed fp32 pairs (sm_100 f32x2 arithmetic) and the 3-input maximum.
__device__ __forceinline__ uint64_t pack_u32x2(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  return pack_u32x2(__float_as_uint(lo), __float_as_uint(hi));
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  uint32_t a, b;
  asm("mov.b64 {%0, %1}, %2;\n" : "=r"(a), "=r"(b) : "l"(v));
  lo = __uint_as_float(a);
  hi = __uint_as_float(b);
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

struct PrefillParams {
  const int32_t* table;
  int64_t table_row_stride;
  int table_kind;
  int table_rows;
  int64_t table_tokens;   // positions a table row can name (dense: tokens addressable from K/V)
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

__global__ void __launch_bounds__(kThreads, 1)
paged_prefill_kernel(PrefillParams p, const __grid_constant__ CUtensorMap qmap,
                     const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;

  // ---- which work item is this? (heavy query tiles first) ------------------------------------
  const int pairs_per_group = (p.group + 1) / 2;
  const int kv_head = static_cast<int>(blockIdx.x) / pairs_per_group;
  const int pair = static_cast<int>(blockIdx.x) - kv_head * pairs_per_group;
  const int head0 = kv_head * p.group + 2 * pair;          // query head of tile 0; tile 1 is head0 + 1
  const bool active1 = (2 * pair + 1) < p.group;            // an odd group leaves its last head alone
  // A CTA takes up to TWO query tiles of its request, one after the other: tile t_b-1-k (many key
  // tiles) and tile k (few), so every CTA of a request does about the same work, and the second
  // tile's Q / K / V loads, barrier set-up and TMEM are already there when the first one drains.
  const int pair_k = static_cast<int>(blockIdx.y);
  const int b = blockIdx.z;
  const int64_t q_len = load_len(p.q_lens, p.lens_i64, b);
  const int64_t ctx = load_len(p.ctx_lens, p.lens_i64, b);
  // Every early exit below still makes the programmatic-launch calls, so that a dependent kernel
  // can rely on "my predecessor waited for its own predecessor".
  auto leave_early = [] {
    cudaGridDependencySynchronize();
    cudaTriggerProgrammaticLaunchCompletion();
  };
  const int table_row = p.req_ids ? __ldg(p.req_ids + b) : b;
  // A stale length or request id must not become a read outside the table: such a request is
  // reported and skipped.
  if (q_len < 0 || ctx < 0 || q_len > p.total_q || ctx > p.table_tokens || ctx + q_len > p.table_tokens ||
      (p.table_kind != B200KV_TABLE_DENSE && (table_row < 0 || table_row >= p.table_rows))) {
    set_status(p.status, B200KV_DEV_BAD_LENGTH);
    leave_early();
    return;
  }
  const int t_b = static_cast<int>((q_len + kBM - 1) / kBM);   // query tiles of the request
  if (pair_k > t_b - 1 - pair_k) {                              // also q_len == 0
    leave_early();
    return;
  }
  const int n_work = pair_k < t_b - 1 - pair_k ? 2 : 1;
  const int64_t q_start_b = static_cast<int64_t>(__ldg(p.q_start + b));
  struct Work {
    int64_t row0;      // first query row of the tile in its request
    int rows;          // rows of the tile that exist
    int64_t q_tok0;    // packed row of tile row 0
    int64_t kv_len;    // keys visible to the tile's last row
    int64_t n_pages;
    int n_tiles;       // 128-key tiles
  };
  auto work_of = [&](int w) {
    Work k;
    k.row0 = static_cast<int64_t>(w == 0 ? t_b - 1 - pair_k : pair_k) * kBM;
    k.rows = static_cast<int>(q_len - k.row0 < kBM ? q_len - k.row0 : kBM);
    k.q_tok0 = q_start_b + k.row0;
    k.kv_len = ctx + k.row0 + k.rows;
    k.n_tiles = static_cast<int>((k.kv_len + kBN - 1) / kBN);
    k.n_pages = (k.kv_len + kPS - 1) / kPS;
    return k;
  };
  const Work work0 = work_of(0), work1 = work_of(n_work - 1);
  if (work0.q_tok0 < 0 || work0.q_tok0 + work0.rows > p.total_q || work1.q_tok0 < 0) {
    set_status(p.status, B200KV_DEV_BAD_LENGTH);
    leave_early();
    return;
  }

  // ---- shared memory carve-up -----------------------------------------------------------------
  const uint32_t sm_q = smem_u32(smem);                     // [group][32 KB]
  const uint32_t sm_p = sm_q + kGroups * kQBytes;           // [group][32 KB]
  const uint32_t sm_ring = sm_p + kGroups * kPBytes;        // [kSlots][32 KB]: K_0 V_0 K_1 V_1 ...
  const uint32_t sm_bar = sm_ring + kSlots * kTileBytes;
  const uint32_t bar_q = sm_bar;                            // 1
  const uint32_t bar_full = sm_bar + 8;                     // [kSlots]  TMA bytes landed
  const uint32_t bar_empty = bar_full + 8 * kSlots;         // [kSlots]  MMAs that read the slot completed
  const uint32_t bar_sfull = bar_empty + 8 * kSlots;        // [kGroups] S_g of a tile is in TMEM
  const uint32_t bar_pfull = bar_sfull + 8 * kGroups;       // [kGroups] P_g of a tile is in shared memory
  const uint32_t bar_pvfull = bar_pfull + 8 * kGroups;      // [kGroups] O_g += P_g V of a tile completed
  const uint32_t bar_sfree = bar_pvfull + 8 * kGroups;      // [kGroups] S_g of a tile is in registers
  const uint32_t bar_qfree = bar_sfree + 8 * kGroups;       // every S of a query tile has completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + (bar_qfree + 8 - sm_q));
  static_assert(8 + 2 * 8 * kSlots + 4 * 8 * kGroups + 8 + 8 <= kBarBytes, "barrier area too small");
  if ((sm_q & 1023u) != 0) {  // swizzled boxes and UMMA descriptors assume 1024-byte alignment
    set_status(p.status, B200KV_DEV_BAD_PAGE);
    leave_early();
    return;
  }

  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_qfree, 1);
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, 1);
    }
    for (int g = 0; g < kGroups; ++g) {
      mbar_init(bar_sfull + 8 * g, 1);
      mbar_init(bar_pfull + 8 * g, kGroupWarps * 32);
      mbar_init(bar_pvfull + 8 * g, 1);
      mbar_init(bar_sfree + 8 * g, kGroupWarps * 32);
    }
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
  // Ring order: K runs one tile ahead of V, K_0 K_1 V_0 K_2 V_1 ... K_{T-1} V_{T-2} V_{T-1}, which is
  // also the order in which the tensor core finishes with the tiles (S of tile j+1 is issued
  // before P V of tile j).  Item n lives in slot n % kSlots.
  // A query tile with T key tiles uses 2T consecutive ring items starting at `base`; barrier
  // phases simply keep counting across the CTA's query tiles.
  auto pos_k = [](int base, int t) { return base + (t == 0 ? 0 : 2 * t - 1); };
  auto pos_v = [](int base, int T, int t) { return base + (t == T - 1 ? 2 * T - 1 : 2 * t + 2); };
  cudaGridDependencySynchronize();  // q and the pool belong to earlier kernels until here
  cudaTriggerProgrammaticLaunchCompletion();

  if (warp == kProducerWarp) {
    // ============================== TMA producer ============================================
    // Ring items alternate K_0, V_0, K_1, V_1, ...; item n lives in slot n % kSlots.  A K or V
    // tile is 8 pages x 2 head_dim halves = 16 boxes, one per lane 0..15.
    const uint64_t policy = l2_evict_first_policy();
    if (lane == 0) {
      prefetch_tensormap(&qmap);
      prefetch_tensormap(&kmap);
      prefetch_tensormap(&vmap);
    }
    const int my_page = lane >> 1;   // lanes 0..15: page of the tile
    const int my_half = lane & 1;    // low / high half of head_dim
    const int32_t* trow = p.table + static_cast<int64_t>(table_row) * p.table_row_stride;
    bool ok = true;
    int item_base = 0;
    for (int w = 0; ok && w < n_work; ++w) {
      const Work wk = w ? work1 : work0;
      const int n_tiles = wk.n_tiles;
      const int64_t n_pages = wk.n_pages;
      // ---- both Q tiles of this query tile (the previous one's S MMAs must be done with them)
      if (w > 0 && !mbar_wait_bounded(bar_qfree, (w - 1) & 1)) {
        set_status(p.status, B200KV_DEV_WAIT_TIMEOUT);
        break;
      }
      if (lane == 0) mbar_arrive_expect_tx(bar_q, (active1 ? 2 : 1) * kQBytes);
      __syncwarp();
      {
        // A query tile's rows are a whole token row apart in memory, so a box is 16 rows and every
        // lane issues one: lane = 16 * head of the pair + 8 * head_dim half + row group.  Rows past
        // this request's q_len are the next request's rows (or zero fill past the end); their
        // results are never stored.
        const int qh = lane >> 4, qhalf = (lane >> 3) & 1, qg = lane & 7;
        if (qh == 0 || active1)
          tma_load_3d(sm_q + qh * kQBytes + qhalf * (kQBytes / 2) + qg * (kQBoxRows * 128), &qmap, bar_q,
                      qhalf * 64, head0 + qh, static_cast<int>(wk.q_tok0) + qg * kQBoxRows, policy);
      }
      // Raw table entry of this lane's page of a tile (0 when the page does not exist).
      auto fetch_id = [&](int j) -> int32_t {
        const int64_t lp = static_cast<int64_t>(j) * kTilePages + my_page;
        if (lane >= 16 || j >= n_tiles || lp >= n_pages || p.table_kind == B200KV_TABLE_DENSE) return 0;
        return __ldg(trow + (p.table_kind == B200KV_TABLE_BLOCK ? lp : lp * kPS));
      };
      // Item n of the ring order above: which tile, and K or V.
      auto item_tile = [n_tiles](int n, bool& is_v) {
        if (n == 0) { is_v = false; return 0; }
        if (n == 2 * n_tiles - 1) { is_v = true; return n_tiles - 1; }
        is_v = (n & 1) == 0;
        return is_v ? (n - 2) / 2 : (n + 1) / 2;
      };
      bool v_cur;
      int t_cur = item_tile(0, v_cur);
      int32_t id_cur = fetch_id(t_cur);
      for (int nl = 0; ok && nl < 2 * n_tiles; ++nl) {
        bool v_next = false;
        const int t_next = nl + 1 < 2 * n_tiles ? item_tile(nl + 1, v_next) : n_tiles;
        const int32_t id_next = fetch_id(t_next);   // in flight while this item is issued
        const int64_t page0 = static_cast<int64_t>(t_cur) * kTilePages;
        const int np = static_cast<int>(n_pages - page0 < kTilePages ? n_pages - page0 : kTilePages);
        const int64_t lp = page0 + my_page;
        int64_t slot;
        if (p.table_kind == B200KV_TABLE_BLOCK) slot = static_cast<int64_t>(id_cur) * kPS;
        else if (p.table_kind == B200KV_TABLE_TOKEN) slot = static_cast<int64_t>(id_cur);
        else slot = q_start_b + lp * kPS;   // dense packed K/V: token t of the request at q_start + t
        if (lane < 2 * np && (slot < 0 || slot >= p.pool_tokens)) {
          set_status(p.status, B200KV_DEV_BAD_PAGE);
          slot = 0;  // never dereference a bad entry: report it and read page 0 instead
        }
        const uint32_t dst_off = my_half * (kTileBytes / 2) + my_page * kHalfPage;
        const int n = item_base + nl;
        const int sl = n % kSlots;
        if (n >= kSlots && !mbar_wait_bounded(bar_empty + 8 * sl, ((n / kSlots) - 1) & 1)) {
          set_status(p.status, B200KV_DEV_WAIT_TIMEOUT);
          ok = false;
          break;
        }
        if (lane == 0) mbar_arrive_expect_tx(bar_full + 8 * sl, np * 2 * kHalfPage);
        __syncwarp();
        if (lane < 2 * np)
          tma_load_3d(sm_ring + sl * kTileBytes + dst_off, v_cur ? &vmap : &kmap, bar_full + 8 * sl, my_half * 64,
                      kv_head, static_cast<int>(slot), policy);
        t_cur = t_next;
        v_cur = v_next;
        id_cur = id_next;
      }
      item_base += 2 * n_tiles;
    }
  } else if (warp == kMmaWarp) {
    // ============================== MMA issuer ==============================================
    if (lane == 0) {
      bool ok = true;
      // Descriptors are built once; per instruction only the 14-bit start-address field (bytes
      // >> 4, shared-memory addresses fit without carry) is advanced by a compile-time constant.
      // K is the K-major B operand of S; V is the MN-major B operand of P V: 64 head_dim values
      // contiguous (128 B), the next 64 at +16 KB (LBO), 8-key groups 1024 B apart (SBO), a K step
      // of 16 keys advances 2048 B.
      const uint64_t dq0 = smem_desc(sm_q, 16, 1024), dq1 = smem_desc(sm_q + kQBytes, 16, 1024);
      const uint64_t dp0 = smem_desc(sm_p, 16, 1024), dp1 = smem_desc(sm_p + kPBytes, 16, 1024);
      const uint64_t dk_base = smem_desc(sm_ring, 16, 1024);
      const uint64_t dv_base = smem_desc(sm_ring, kTileBytes / 2, 1024);
      constexpr uint64_t kSlotStep = kTileBytes >> 4;
      constexpr uint64_t kChunkStep = (kTileBytes / 2) >> 4;   // second 64-wide chunk of an operand tile

      int tile_base = 0, item_base = 0, n_tiles = 0;   // of the query tile being issued
      auto issue_s = [&](int g, int j) {            // S_g = Q_g K_j^T : 8 x (M128 N128 K16)
        const uint64_t kd = dk_base + static_cast<uint64_t>(pos_k(item_base, j) % kSlots) * kSlotStep;
        const uint64_t qd = g ? dq1 : dq0;
        const uint32_t d_s = tmem_base + kTmemS + g * kBN;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks) {
          const uint64_t off = static_cast<uint64_t>((ks >> 2) * kChunkStep + (ks & 3) * 2);
          if (ks == 0) umma_f16(d_s, qd + off, kd + off, kIdescS, 0u);
          else umma_f16(d_s, qd + off, kd + off, kIdescS, 1u);
        }
        umma_commit(bar_sfull + 8 * g);
      };
      auto issue_pv = [&](int g, int j) {           // O_g += P_g V_j : 8 x (M128 N128 K16)
        const uint64_t vd = dv_base + static_cast<uint64_t>(pos_v(item_base, n_tiles, j) % kSlots) * kSlotStep;
        const uint64_t pd = g ? dp1 : dp0;
        const uint32_t d_o = tmem_base + kTmemO + g * kD;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < kBN / 16; ++ks) {
          const uint64_t a = pd + static_cast<uint64_t>((ks >> 2) * kChunkStep + (ks & 3) * 2);
          const uint64_t bd = vd + static_cast<uint64_t>(ks * (2048 >> 4));
          if (ks == 0) umma_f16(d_o, a, bd, kIdescPV, j > 0 ? 1u : 0u);
          else umma_f16(d_o, a, bd, kIdescPV, 1u);
        }
        umma_commit(bar_pvfull + 8 * g);
      };
      const int ng = active1 ? 2 : 1;
      // Tensor-core order within a query tile: S0_0 S1_0 | S0_1 S1_1 PV0_0 PV1_0 | S0_2 S1_2 PV0_1
      // PV1_1 | ...  The S of key tile j+1 is issued as soon as the softmax group holds S of tile j in
      // registers, so it runs under that softmax and the group does not wait for its next S.
      //
      // This thread paces the CTA (the tensor core idles whenever it is not issuing), and a barrier
      // test costs it a few hundred cycles even when the phase is long complete.  So the three
      // barriers a step depends on are tested together (independent instructions, one latency)
      // and only the ones that were not ready are waited for.
      for (int w = 0; ok && w < n_work; ++w) {
        n_tiles = (w ? work1 : work0).n_tiles;
        // ---- first S of the query tile: its Q, its K_0, and (second tile) the S registers of the
        // previous tile's last key tile
        ok = mbar_wait_bounded(bar_q, w & 1);
        const int pk0 = pos_k(item_base, 0);
        if (ok) ok = mbar_wait_bounded(bar_full + 8 * (pk0 % kSlots), (pk0 / kSlots) & 1);
        for (int g = 0; ok && g < ng; ++g) {
          if (w > 0) ok = mbar_wait_bounded(bar_sfree + 8 * g, (tile_base - 1) & 1);
          if (ok) issue_s(g, 0);
        }
        if (!ok) break;
        umma_commit(bar_empty + 8 * (pk0 % kSlots));        // K_0: both S issued
        if (n_tiles == 1) umma_commit(bar_qfree);           // the Q tiles may be replaced
        for (int j = 0; ok && j < n_tiles; ++j) {
          const uint32_t par = (tile_base + j) & 1;         // phase of the per-key-tile barriers
          if (j + 1 < n_tiles) {
            const int pk = pos_k(item_base, j + 1);
            const uint32_t b_k = bar_full + 8 * (pk % kSlots), par_k = (pk / kSlots) & 1;
            const bool r_k = mbar_test_wait(b_k, par_k);
            const bool r_0 = mbar_test_wait(bar_sfree, par);
            const bool r_1 = ng > 1 ? mbar_test_wait(bar_sfree + 8, par) : true;
            if (!r_k && !mbar_wait_bounded(b_k, par_k)) { ok = false; break; }
            if (!r_0 && !mbar_wait_bounded(bar_sfree, par)) { ok = false; break; }
            issue_s(0, j + 1);
            if (ng > 1) {
              if (!r_1 && !mbar_wait_bounded(bar_sfree + 8, par)) { ok = false; break; }
              issue_s(1, j + 1);
            }
            umma_commit(bar_empty + 8 * (pk % kSlots));     // K_{j+1}: both S issued
            if (j + 2 == n_tiles) umma_commit(bar_qfree);   // that was the query tile's last S
          }
          const int pv = pos_v(item_base, n_tiles, j);
          const uint32_t b_v = bar_full + 8 * (pv % kSlots), par_v = (pv / kSlots) & 1;
          const bool r_v = mbar_test_wait(b_v, par_v);
          const bool r_0 = mbar_test_wait(bar_pfull, par);
          const bool r_1 = ng > 1 ? mbar_test_wait(bar_pfull + 8, par) : true;
          if (!r_v && !mbar_wait_bounded(b_v, par_v)) { ok = false; break; }
          if (!r_0 && !mbar_wait_bounded(bar_pfull, par)) { ok = false; break; }
          issue_pv(0, j);
          if (ng > 1) {
            if (!r_1 && !mbar_wait_bounded(bar_pfull + 8, par)) { ok = false; break; }
            issue_pv(1, j);
          }
          umma_commit(bar_empty + 8 * (pv % kSlots));       // V_j: both P V issued
        }
        tile_base += n_tiles;
        item_base += 2 * n_tiles;
      }
      if (!ok) set_status(p.status, B200KV_DEV_WAIT_TIMEOUT);
    }
  } else {
    // ============================== softmax warps ===========================================
    // O accumulates in TMEM.  The running maximum used to scale P and O (m_used) is only moved
    // when the true row maximum has grown by more than 8 (a factor 256, harmless for fp16 P and
    // fp32 accumulation): then O and l are rescaled once; otherwise a tile costs no pass over O.
    // A thread holds its whole 128-column S row in registers: one TMEM round trip per tile.
    const int g = warp / kGroupWarps;                      // which query tile (head) of the pair
    const int gtid = tid - g * kGroupWarps * 32;
    const int row = gtid;                                  // query row of the tile = TMEM lane
    const bool active = (g == 0) || active1;
    const uint32_t t_lane = static_cast<uint32_t>((warp % kGroupWarps) * 32) << 16;
    const uint32_t tmem_s = tmem_base + t_lane + kTmemS + g * kBN;
    const uint32_t tmem_o = tmem_base + t_lane + kTmemO + g * kD;
    const uint32_t my_p = sm_p + g * kPBytes;
    const uint32_t b_sfull = bar_sfull + 8 * g, b_pfull = bar_pfull + 8 * g, b_pvfull = bar_pvfull + 8 * g;
    bool ok = true;
    int tile_base = 0, item_base = 0;
    // A warp whose wait ran out (ok == false) stops computing but keeps visiting its query tiles,
    // so that it still meets the other warps of its group at the two named barriers of each
    // read-out: nobody is left waiting at a barrier for a warp that has gone.
    for (int w = 0; active && w < n_work; ++w) {
    const Work wk = w ? work1 : work0;
    const int n_tiles = wk.n_tiles;
    const int64_t row0 = wk.row0, kv_len = wk.kv_len;
    const int64_t q_pos = ctx + row0 + row;                // logical position of this query row
    float m_used = -INFINITY, l_run = 0.f;
    for (int j = 0; ok && j < n_tiles; ++j) {
      const uint32_t par = (tile_base + j) & 1;            // phase of the per-key-tile barriers
      if (!mbar_wait_bounded(b_sfull, par)) { ok = false; break; }
      tc_fence_after();
      const int64_t key0 = static_cast<int64_t>(j) * kBN;
      // Only tiles that reach past the first row's diagonal need the causal mask (warp-uniform).
      const bool need_mask = key0 + kBN - 1 > ctx + row0;
      const int lim = static_cast<int>(q_pos - key0 < kBN ? q_pos - key0 : kBN);  // keys c <= lim visible
      // The whole 128-column S row in one TMEM round trip (four loads in flight, one wait).
      uint32_t sr[4][32];
      tmem_ld32(tmem_s + 0, sr[0]);
      tmem_ld32(tmem_s + 32, sr[1]);
      tmem_ld32(tmem_s + 64, sr[2]);
      tmem_ld32(tmem_s + 96, sr[3]);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(bar_sfree + 8 * g);                      // S_g may be overwritten by the next tile's S
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < kBN; ++c)
          if (c > lim) sr[c >> 5][c & 31] = 0xff800000u;   // -inf
      }
      // Row maximum of the RAW scores (the scale is positive), two new elements per instruction.
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four independent chains
#pragma unroll
      for (int c = 0; c < kBN; c += 2)
        mx4[(c >> 1) & 3] = max3(mx4[(c >> 1) & 3], __uint_as_float(sr[c >> 5][c & 31]),
                                 __uint_as_float(sr[(c + 1) >> 5][(c + 1) & 31]));
      float mx = fmaxf(max3(mx4[0], mx4[1], mx4[2]), mx4[3]);
      mx *= p.scale_log2;
      // P_g and O_g are free once the P V MMAs of tile j-1 have completed (they were issued
      // before this tile's S, so this wait is normally already satisfied).
      if (j > 0 && !mbar_wait_bounded(b_pvfull, par ^ 1)) { ok = false; break; }
      const bool grow = mx > m_used + 8.f;                 // also true on the first tile (m_used = -inf)
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = grow ? mx : m_used;
        const float alpha = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_new);
        l_run *= alpha;
        m_used = m_new;
        if (j > 0) {                                       // rescale this warp's 32 rows of O
          tc_fence_after();
#pragma unroll 1
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
      // p = 2^(s * scale - m): one packed FFMA per two elements, then exp2, packed row sums.
      const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
      const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2);
      const uint64_t negm2 = pack_f32x2(neg_m, neg_m);
      uint64_t rs2[2] = {pack_f32x2(0.f, 0.f), pack_f32x2(0.f, 0.f)};
      // P row -> shared memory, UMMA K-major layout with the 128-byte swizzle: 64-key chunk h is a
      // [128 rows][128 B] block, row r at r*128 B, its eight 16-byte pieces XOR-ed with r % 8.
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t prow = my_p + h * (kPBytes / 2) + row * 128;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = h * 64 + ch * 8 + 2 * e;
            const uint64_t x2 =
                fma_f32x2(pack_u32x2(sr[c >> 5][c & 31], sr[(c + 1) >> 5][(c + 1) & 31]), scale2, negm2);
            float x0, x1;
            unpack_f32x2(x2, x0, x1);
            const float p0 = fast_exp2(x0);
            const float p1 = fast_exp2(x1);
            rs2[e & 1] = add_f32x2(rs2[e & 1], pack_f32x2(p0, p1));
            pk[e] = pack_half2(p0, p1);
          }
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};\n" ::"r"(prow + ((ch ^ (row & 7)) << 4)),
                       "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3])
                       : "memory");
        }
      }
      {
        float a0, a1, b0, b1;
        unpack_f32x2(rs2[0], a0, a1);
        unpack_f32x2(rs2[1], b0, b1);
        l_run += (a0 + a1) + (b0 + b1);
      }
      if (j == n_tiles - 1) {
        // Keys past kv_len in the last tile were either not loaded or lie in never-written pool
        // slots; their P is 0 but 0 * NaN would still poison the row, so zero those V rows.  Each
        // group does the whole clean-up before publishing its own P, which is what its own P V
        // waits for; the two groups write the same zeros.
        const int item = pos_v(item_base, n_tiles, j);
        const int sl = item % kSlots;
        const int valid = static_cast<int>(kv_len - key0);
        if (valid < kBN) {
          if (!mbar_wait_bounded(bar_full + 8 * sl, (item / kSlots) & 1)) { ok = false; break; }
          for (int i = gtid; i < (kBN - valid) * 16; i += kGroupWarps * 32) {
            const int r = valid + (i >> 4);
            const int c = i & 15;
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n" ::"r"(
                             sm_ring + sl * kTileBytes + (c >> 3) * (kTileBytes / 2) + r * 128 + ((c & 7) << 4)),
                         "r"(0)
                         : "memory");
          }
        }
      }
      fence_proxy_async_smem();                            // P (and V fix-ups) visible to the tensor core
      mbar_arrive(b_pfull);
    }
    // ---- the query tile's rows: O / l, once its last P V has completed -----------------------
    if (ok && !mbar_wait_bounded(b_pvfull, (tile_base + n_tiles - 1) & 1)) ok = false;
    {
      tc_fence_after();
      const float inv = 1.f / l_run;
      const int rows = wk.rows;
      // O / l -> fp16, staged through the group's (now idle) P buffer so that the global stores are
      // whole 256-byte rows: written straight from the registers, a warp's 16-byte stores would
      // land in 32 different rows (16 KB apart) and the read-out took ~6 000 cycles per query tile.
      // Staging layout: row r at r * 256 B, its sixteen 16-byte chunks XOR-ed with r % 16 (no
      // bank conflicts either way).
      uint32_t ov[4][32];                                  // the S registers are dead here
#pragma unroll
      for (int q4 = 0; q4 < kD / 32; ++q4) tmem_ld32(tmem_o + q4 * 32, ov[q4]);   // warp-collective, all in flight
      tmem_ld_wait();
#pragma unroll
      for (int q4 = 0; q4 < kD / 32; ++q4) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t v0 = pack_half2(__uint_as_float(ov[q4][c * 8 + 0]) * inv, __uint_as_float(ov[q4][c * 8 + 1]) * inv);
          const uint32_t v1 = pack_half2(__uint_as_float(ov[q4][c * 8 + 2]) * inv, __uint_as_float(ov[q4][c * 8 + 3]) * inv);
          const uint32_t v2 = pack_half2(__uint_as_float(ov[q4][c * 8 + 4]) * inv, __uint_as_float(ov[q4][c * 8 + 5]) * inv);
          const uint32_t v3 = pack_half2(__uint_as_float(ov[q4][c * 8 + 6]) * inv, __uint_as_float(ov[q4][c * 8 + 7]) * inv);
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};\n" ::"r"(
                           my_p + row * 256 + (((q4 * 4 + c) ^ (row & 15)) << 4)),
                       "r"(v0), "r"(v1), "r"(v2), "r"(v3)
                       : "memory");
        }
      }
      asm volatile("bar.sync %0, %1;\n" ::"r"(2 + g), "n"(kGroupWarps * 32) : "memory");
      __half* obase = p.out + wk.q_tok0 * p.out_stride_t + static_cast<int64_t>(head0 + g) * p.out_stride_h;
#pragma unroll 4
      for (int it = 0; it < kBM * 16 / (kGroupWarps * 32); ++it) {
        const int idx = it * (kGroupWarps * 32) + gtid;    // half a warp per row
        const int r = idx >> 4, c = idx & 15;
        if (ok && r < rows) {
          uint4 v;
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n"
                       : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                       : "r"(my_p + r * 256 + ((c ^ (r & 15)) << 4)));
          *reinterpret_cast<uint4*>(obase + static_cast<int64_t>(r) * p.out_stride_t + c * 8) = v;
        }
      }
      // the P buffer goes back to the next query tile's softmax only when everybody has read it
      asm volatile("bar.sync %0, %1;\n" ::"r"(2 + g), "n"(kGroupWarps * 32) : "memory");
      tc_fence_before();
    }
    tile_base += n_tiles;
    item_base += 2 * n_tiles;
    }  // query tiles of this CTA
    if (!ok) set_status(p.status, B200KV_DEV_WAIT_TIMEOUT);
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
// box = 64 halves x 1 head x 16 tokens (an eighth of one half of a query tile), 128-byte swizzle.
int encode_q_tensor_map(CUtensorMap* out, const void* q, int64_t total_q, int64_t stride_t,
                        int64_t stride_h, int heads) {
  return cached_kv_tensor_map(out, q, total_q, stride_t, stride_h, heads, kD, kQBoxRows);
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
  if (a.table_kind != B200KV_TABLE_DENSE &&
      (!a.table || a.table_rows <= 0 || a.table_cols <= 0 || a.table_row_stride < a.table_cols))
    return B200KV_EINVAL;
  if (a.table_kind != B200KV_TABLE_DENSE && a.req_ids == nullptr && a.batch > a.table_rows) return B200KV_EINVAL;
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
  rc = cached_kv_tensor_map(&kmap, a.k_base, a.pool_tokens, a.kv_tok_stride, a.kv_head_stride,
                            a.kv_heads, kD, kPS);
  if (rc != B200KV_OK) return rc;
  rc = cached_kv_tensor_map(&vmap, a.v_base, a.pool_tokens, a.kv_tok_stride, a.kv_head_stride,
                            a.kv_heads, kD, kPS);
  if (rc != B200KV_OK) return rc;

  PrefillParams p{};
  p.table = a.table;
  p.table_row_stride = a.table_row_stride;
  p.table_kind = a.table_kind;
  p.table_rows = a.table_rows;
  p.table_tokens = a.table_kind == B200KV_TABLE_DENSE ? a.pool_tokens
                   : a.table_cols * (a.table_kind == B200KV_TABLE_BLOCK ? kPS : 1);
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
  if (p.tiles_m > 2 * 65535) return B200KV_ETOOLARGE;

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
  // x: (KV head, pair of query heads of its group), adjacent so a group's CTAs share K/V in L2.
  cfg.gridDim = dim3(static_cast<unsigned>(a.kv_heads * ((p.group + 1) / 2)),
                     static_cast<unsigned>((p.tiles_m + 1) / 2), static_cast<unsigned>(a.batch));
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
