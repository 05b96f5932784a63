// Paged flash-decoding for B200: one persistent split-KV launch that also merges its partials
// and, when asked, performs the step's KV append.
//
// Replaces flash_decoding of the reference (lite_llama/kernels/flashdecoding.py:295-342):
// stage 1 there launches one program per (sequence, QUERY head, 128-token partition), so
// every K/V byte is fetched once per query head of its group; stage 2 merges partitions.
//
// Here the unit of work is a KV head: a CTA owns one KV head and serves all G = Hq/Hkv
// query heads of its group from a single pass over that head's K/V pages, so each K/V
// byte leaves HBM once.  Scheduling is a static "flat page line" decomposition:
//
//   * all sequences' pages are laid end to end (NP = sum_b ceil(L_b / 16) pages);
//   * the launch has `nteams` teams of Hkv CTAs; team i takes the contiguous range
//     [i*U/nteams, (i+1)*U/nteams) of that line and CTA k of the team handles KV head k over
//     it, so every CTA has the same work whatever the length mix, and the Hkv CTAs of a team
//     sweep the same token rows (one 2*Hkv*128-half pool row holds all heads of a token) at
//     the same time.  The line is measured in units, U = NP + piece_cost per non-empty
//     sequence: ending a piece costs a CTA about that many pages of streaming, and a cut
//     inside a sequence's extra units snaps to the start of the sequence;
//   * a team's range may cover the tail of one sequence, several whole sequences and the
//     head of another: each such "piece" yields either the final fp16 output (piece ==
//     whole sequence) or an fp32 partial (normalised output + log2-domain log-sum-exp) in
//     slot team + b of the workspace.  The CTA that delivers the LAST partial of a (sequence,
//     KV head) -- found with a wrapping atomic counter that is back at zero when the launch
//     ends -- merges all of them (stage 2 of the reference, flashdecoding.py:199-267) and
//     writes the fp16 rows, so the whole decode is ONE launch;
//   * optionally the step's KV append is part of the same launch: the CTA whose range holds
//     the last page of a sequence writes that sequence's new K and V row of its head into the
//     pool (update_kv_buffer of the reference, update_kv_buffer.py:47-81) right before it
//     fetches that page.
//
// Pipeline inside a CTA (5 warps, 2 CTAs per SM): tiles of 64 tokens (4 pages; K and V rows
// of 256 B each) flow through a 3-deep ring of 32 KB stages that keeps running across piece
// boundaries.  Warp 4 is the producer: it fetches page-table entries four tiles ahead, waits
// for a stage's "empty" mbarrier, arms its "full" mbarrier with the byte count and issues the
// tile's 16 TMA copies (cp.async.bulk.tensor, 16 rows x 128 B boxes with the 128-byte swizzle,
// so ldmatrix is conflict-free), one per lane.  Warps 0..3 are consumers: warp w owns page w
// (tokens [16w, 16w+16)) of every tile: S^T = K Q^T and O^T += V^T P^T run on mma.sync
// m16n8k16 (fp16 in, fp32 accumulate) with the tokens as the M rows and the G query heads as
// the N columns; per-warp online-softmax states are merged through shared memory at the end
// of a piece (named barriers among the four consumer warps; the next sequence's Q is
// requested before the merge so that its latency hides under it).  No CTA-wide barrier in the
// steady state; every mbarrier wait is time-bounded, and a consumer warp whose wait ran out
// keeps walking its tiles without computing, so it still meets the other warps at every named
// barrier and the arrival counters end at zero.
// The kernel is HBM-bound: algorithmic bytes per token per KV head = 2 (K,V) * 128 * 2 B.
#include <climits>

#include "common.cuh"
#include "launch.h"
#include "tma.h"

namespace b200kv {

namespace {

constexpr int kD = 128;
constexpr int kPS = 16;
constexpr int kTileTok = 64;
constexpr int kTilePages = kTileTok / kPS;
constexpr int kConsumerWarps = 4;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = (kConsumerWarps + 1) * 32;  // + one producer warp
constexpr int kScanThreads = 128;
constexpr int kRowBytes = kD * 2;
constexpr int kPageBytes = kPS * kRowBytes;       // one page of one head, K or V: 4 KB
constexpr int kTileBytes = kTileTok * kRowBytes;  // one of K or V
constexpr int kStageBytes = 2 * kTileBytes;
constexpr int kCtasPerSm = 2;
constexpr int kStagesRows8 = 3;
constexpr int kL2PrefetchTiles = 2;   // tiles prefetched into L2 before the dependency wait (<= kLead)
constexpr int kMinPagesPerTeam = 4;   // a team is not worth launching for fewer pages
// Ending a piece (merging the four warps' state, writing the rows, restarting on another
// sequence) costs a CTA about as much as streaming this many pages.  The page line is therefore
// split in UNITS: every non-empty sequence counts its pages plus this constant, so that teams
// with more sequence boundaries get fewer pages; a team boundary that falls inside a sequence's
// extra units snaps to the start of that sequence.
constexpr int kDefaultPieceCost = 8;
// Pages per CTA (by the host's length bound) below which the cut is tuned for short ranges;
// measured on KV-head shards of 32 sequences of 1-4 k tokens (1, 2, 4, 8 KV heads per GPU).
constexpr int kMediumRangePages = 128;
constexpr int kShortRangePages = 64;
constexpr int kShortRangePieceCost = 16;
// The first bytes of the workspace hold one arrival counter per (sequence, KV head).
constexpr size_t kCounterBytes = B200KV_DECODE_COUNTER_BYTES;
constexpr int64_t kMaxCounters = static_cast<int64_t>(kCounterBytes / sizeof(unsigned));

struct DecodeParams {
  const __half* q;
  int64_t q_stride_b, q_stride_h;
  __half* k_base;
  __half* v_base;
  int64_t kv_tok_stride, kv_head_stride, pool_tokens;
  const int32_t* table;
  int64_t table_row_stride;
  int table_kind;
  int table_rows;
  const int32_t* row_ids;
  const void* seq_lens;
  int seq_lens_i64;
  int batch, q_heads, kv_heads, group;
  float scale_log2;
  int64_t max_seq_len;
  int nteams;
  int piece_cost;
  // fused KV append (new_k == nullptr: none): pool[slots[b]] = (new_k[b], new_v[b]) for this CTA's head
  const __half* new_k;        // [batch][kv_heads][128], token stride new_k_tok_stride
  const __half* new_v;
  int64_t new_k_tok_stride, new_v_tok_stride;
  const int32_t* slots;
  float* part_o;        // [nslots][kv_heads][ROWS][128]
  float* part_lse;      // [nslots][kv_heads][ROWS]
  unsigned* piece_ctr;  // [batch][kv_heads], zero between launches
  __half* out;
  int64_t out_stride_b, out_stride_h;
  int32_t* status;
};

// Length of sequence b as every part of the kernel sees it: clamped to [0, max_seq_len] (the
// host made sure max_seq_len fits the table's width), and 0 when its table row does not exist,
// so a stale length or request id can never turn into a read outside the table.
__device__ __forceinline__ int seq_len_checked(const DecodeParams& p, int b) {
  int64_t len = load_len(p.seq_lens, p.seq_lens_i64, b);
  if (len < 0) {
    set_status(p.status, B200KV_DEV_BAD_LENGTH);
    len = 0;
  } else if (len > p.max_seq_len) {
    set_status(p.status, B200KV_DEV_BAD_LENGTH);
    len = p.max_seq_len;
  }
  if (p.row_ids != nullptr) {
    const int row = __ldg(p.row_ids + b);
    if (row < 0 || row >= p.table_rows) {
      set_status(p.status, B200KV_DEV_BAD_LENGTH);
      len = 0;
    }
  }
  return static_cast<int>(len);
}
__device__ __forceinline__ int pages_of(int len) { return (len + kPS - 1) / kPS; }

// Number of teams that actually get work for NP pages (host launched `nteams`).
__device__ __forceinline__ int effective_teams(int nteams, int64_t np_total) {
  int64_t t = np_total / kMinPagesPerTeam;
  if (t > nteams) t = nteams;
  if (t < 1) t = 1;
  return static_cast<int>(t);
}
__device__ __forceinline__ int64_t team_begin(int team, int nteams_eff, int64_t total) {
  return (static_cast<int64_t>(team) * total) / nteams_eff;
}
// Team whose range holds position x (0 <= x < total).
__device__ __forceinline__ int team_of(int64_t x, int nteams_eff, int64_t total) {
  return static_cast<int>(((x + 1) * nteams_eff - 1) / total);
}

struct Tile {
  int b;        // sequence (batch position)
  int row;      // table row of that sequence
  int page0;    // first logical page of the tile
  int npages;   // pages in the tile (1..4)
  int ntok;     // valid tokens in the tile
  int np;       // pages of the whole sequence
  int len;      // tokens of the whole sequence
  int64_t units0;  // unit position of the sequence's start on the line
  bool first;   // first tile of its piece
  bool last;    // last tile of its piece
  bool whole;   // the piece is the whole sequence
};

// Walks the tiles of flat page range [flat, flat_end) in order.  Producer and consumer each
// own one walker; both visit exactly the same tiles.
struct Walker {
  int b;
  int64_t flat, flat_end;
  int page, piece_begin, piece_end, np, len, row;
  int kseq;   // non-empty sequences before b

  __device__ __forceinline__ void enter(const DecodeParams& p, int seq, int first_page) {
    b = seq;
    len = seq_len_checked(p, b);
    np = pages_of(len);
    row = p.row_ids ? __ldg(p.row_ids + b) : b;
    page = piece_begin = first_page;
    const int64_t room = flat_end - flat;
    piece_end = (np - first_page <= room) ? np : first_page + static_cast<int>(room);
  }
  __device__ __forceinline__ bool next(const DecodeParams& p, Tile& t) {
    if (flat >= flat_end) return false;
    if (page == piece_end) {
      int nb = b + 1;
      while (nb < p.batch && pages_of(seq_len_checked(p, nb)) == 0) ++nb;
      if (nb >= p.batch) {  // cannot happen for consistent lengths; stop rather than overrun
        flat = flat_end;
        return false;
      }
      ++kseq;
      enter(p, nb, 0);
    }
    t.b = b;
    t.row = row;
    t.page0 = page;
    t.npages = min(kTilePages, piece_end - page);
    const int tok_end = min(len, (page + t.npages) * kPS);
    t.ntok = tok_end - page * kPS;
    t.np = np;
    t.len = len;
    t.units0 = (flat - page) + static_cast<int64_t>(p.piece_cost) * kseq;
    t.first = (page == piece_begin);
    t.last = (page + t.npages == piece_end);
    t.whole = (piece_begin == 0 && piece_end == np);
    page += t.npages;
    flat += t.npages;
    return true;
  }
};

// What the producer needs to issue one tile.  The table entries are kept RAW (undecoded and
// unchecked) so that nothing depends on the loaded values until the tile is issued, kLead
// tiles after the loads were started: the table latency is off the producer's critical path.
// A tile that holds the last page of its sequence also carries this lane's 16 bytes of the
// sequence's new K (lanes 0..15) or V (lanes 16..31) row when the append is fused.
constexpr int kLead = 4;
struct Fetch {
  int ntok;    // valid tokens of the tile; 0 = no tile
  int npages;  // pages of the tile
  int32_t id[kTilePages];
  int app_b;         // >= 0: the tile ends this sequence, whose new row is written before the tile is fetched
  int app_off;       // offset of that row inside the sequence's last page
  int32_t app_slot;  // slot_mapping entry of that row
  uint32_t app_row0, app_row1, app_row2, app_row3;   // this lane's 16 bytes of the row
};

// This lane's 16 bytes of the new row of sequence f.app_b, and the slot it goes to.  The new rows
// and the slot_mapping usually come from the kernel launched just before this one, so they are
// only read after the dependency wait.
__device__ __forceinline__ void load_new_row(const DecodeParams& p, Fetch& f, int head, int lane) {
  f.app_slot = __ldg(p.slots + f.app_b);
  const __half* src = (lane < 16 ? p.new_k + static_cast<int64_t>(f.app_b) * p.new_k_tok_stride
                                 : p.new_v + static_cast<int64_t>(f.app_b) * p.new_v_tok_stride) +
                      static_cast<int64_t>(head) * kD + (lane & 15) * 8;
  const uint4 v = __ldcg(reinterpret_cast<const uint4*>(src));
  f.app_row0 = v.x;
  f.app_row1 = v.y;
  f.app_row2 = v.z;
  f.app_row3 = v.w;
}

__device__ __forceinline__ void fetch_next(const DecodeParams& p, Walker& w, Fetch& f, int head, int lane,
                                           bool after_wait) {
  Tile t;
  f.ntok = 0;
  f.npages = 0;
  f.app_b = -1;
  f.app_off = 0;
  f.app_slot = -1;
  f.app_row0 = f.app_row1 = f.app_row2 = f.app_row3 = 0u;
#pragma unroll
  for (int i = 0; i < kTilePages; ++i) f.id[i] = 0;
  if (!w.next(p, t)) return;
  f.ntok = t.ntok;
  f.npages = t.npages;
  const int32_t* rowp = p.table + static_cast<int64_t>(t.row) * p.table_row_stride;
#pragma unroll
  for (int i = 0; i < kTilePages; ++i) {
    if (i < t.npages) {
      const int64_t lp = t.page0 + i;
      f.id[i] = __ldg(rowp + (p.table_kind == B200KV_TABLE_BLOCK ? lp : lp * kPS));
    }
  }
  if (p.new_k != nullptr && t.page0 + t.npages == t.np) {
    f.app_b = t.b;
    f.app_off = (t.len - 1) & (kPS - 1);
    if (after_wait) load_new_row(p, f, head, lane);
  }
}

// Programmatic dependent launch, used by every kernel of this library the same way: whatever
// a kernel does BEFORE this call may overlap the tail of the previous kernel in the stream, so
// it must only read launch metadata (lengths, row ids, page table) that an earlier, already
// completed operation produced.  Every thread of every CTA makes this call on every path, early
// exits included, and a kernel releases its own dependents only after its own wait: when a
// dependent's prologue runs, everything two or more kernels back has completed.
__device__ __forceinline__ void pdl_wait_then_trigger() {
  cudaGridDependencySynchronize();
  cudaTriggerProgrammaticLaunchCompletion();
}

// Transpose an 8x8 matrix of b16 held in mma-fragment layout (lane l: row l/4, cols 2(l%4)..+1).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
  return d;
}

// Shared-memory image of one page of one head as the two TMA boxes leave it: two blocks of
// 16 rows x 128 B (head_dim halves [0,64) and [64,128)), each row's 16-byte chunks XOR-swizzled
// with row % 8.  Byte offset of chunk c (0..15 across the 256-byte head row) of token row r.
__device__ __forceinline__ uint32_t page_chunk_off(int r, int c) {
  return static_cast<uint32_t>(((c >> 3) << 11) + (r << 7) + (((c & 7) ^ (r & 7)) << 4));
}

__device__ __forceinline__ void consumer_bar() {
  asm volatile("bar.sync 1, %0;\n" ::"n"(kConsumerThreads) : "memory");
}

// Merge the `npieces` partials of (sequence b, KV head `head`) held in slots t_first + b ...:
// out = sum_p 2^(lse_p - M) o_p / sum_p 2^(lse_p - M).  Run by the 128 consumer threads of the CTA
// that delivered the last partial; everything it reads was written by other CTAs, so the loads go
// past L1, and the whole merge costs about three memory round trips whatever the piece count:
//   A. thread (piece j, row r) fetches lse[j][r] (128 / ROWS pieces per sweep) into shared memory
//      and the row maxima are reduced with shuffles and one pass through shared memory;
//   B. the same threads turn their entries into weights 2^(lse - M) in place and reduce the row sums;
//   C. thread = output column: the partial outputs are loaded kMergeBatch pieces at a time, every
//      load of a batch issued before any arithmetic (the first batch before step A even), and
//      weighted with the shared-memory weights.
// `wbuf` (npieces * ROWS floats) and `red` (2 * 4 * ROWS floats) are shared-memory scratch that
// nobody else uses between the surrounding consumer barriers.
constexpr int kMergeBatch = 6;
template <int ROWS>
__device__ __forceinline__ void merge_pieces(const DecodeParams& p, int b, int head, int t_first,
                                             int npieces, int tid, float* wbuf, float* red) {
  constexpr int kPerSweep = kConsumerThreads / ROWS;
  const int my_r = tid % ROWS;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  auto slot_of = [&](int pc) { return (static_cast<int64_t>(t_first + pc) + b) * p.kv_heads + head; };
  auto load_batch = [&](float (&ov)[kMergeBatch][8], int r0, int p0) {
#pragma unroll
    for (int j = 0; j < kMergeBatch; ++j) {
      if (p0 + j < npieces) {   // the same for every thread of the CTA
        const int64_t slot = slot_of(p0 + j);
#pragma unroll
        for (int r = 0; r < 8; ++r) ov[j][r] = __ldcg(p.part_o + (slot * ROWS + r0 + r) * kD + tid);
      } else {
#pragma unroll
        for (int r = 0; r < 8; ++r) ov[j][r] = 0.f;
      }
    }
  };
  // The first batch of partial outputs needs no weights to be requested: its loads are issued
  // now and are in flight under steps A and B.
  float first[kMergeBatch][8];
  load_batch(first, 0, 0);
  // ---- A: log-sum-exp values -> shared memory, row maxima --------------------------------------
  float m = -INFINITY;
  for (int j = tid / ROWS; j < npieces; j += kPerSweep) {
    const float v = __ldcg(p.part_lse + slot_of(j) * ROWS + my_r);
    wbuf[j * ROWS + my_r] = v;
    m = fmaxf(m, v);
  }
#pragma unroll
  for (int d = ROWS; d < 32; d <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
  if (lane < ROWS) red[warp * ROWS + lane] = m;
  consumer_bar();
  const float M = fmaxf(fmaxf(red[my_r], red[ROWS + my_r]), fmaxf(red[2 * ROWS + my_r], red[3 * ROWS + my_r]));
  // ---- B: weights in place, row sums --------------------------------------------------------------
  float sum = 0.f;
  for (int j = tid / ROWS; j < npieces; j += kPerSweep) {
    const float w = fast_exp2(wbuf[j * ROWS + my_r] - M);
    wbuf[j * ROWS + my_r] = w;
    sum += w;
  }
#pragma unroll
  for (int d = ROWS; d < 32; d <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
  float* red_sum = red + kConsumerWarps * ROWS;
  if (lane < ROWS) red_sum[warp * ROWS + lane] = sum;
  consumer_bar();
  // ---- C: weighted sum of the partial outputs, thread = column -----------------------------------
  auto add_batch = [&](float (&acc)[8], const float (&ov)[kMergeBatch][8], int r0, int p0) {
#pragma unroll
    for (int j = 0; j < kMergeBatch; ++j) {
      if (p0 + j < npieces) {
        const float4 w0 = *reinterpret_cast<const float4*>(wbuf + (p0 + j) * ROWS + r0);
        const float4 w1 = *reinterpret_cast<const float4*>(wbuf + (p0 + j) * ROWS + r0 + 4);
        acc[0] += w0.x * ov[j][0]; acc[1] += w0.y * ov[j][1]; acc[2] += w0.z * ov[j][2]; acc[3] += w0.w * ov[j][3];
        acc[4] += w1.x * ov[j][4]; acc[5] += w1.y * ov[j][5]; acc[6] += w1.z * ov[j][6]; acc[7] += w1.w * ov[j][7];
      }
    }
  };
#pragma unroll 1
  for (int r0 = 0; r0 < ROWS && r0 < p.group; r0 += 8) {
    float acc[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[r] = 0.f;
    if (r0 == 0) add_batch(acc, first, 0, 0);
#pragma unroll 1
    for (int p0 = (r0 == 0 ? kMergeBatch : 0); p0 < npieces; p0 += kMergeBatch) {
      float ov[kMergeBatch][8];
      load_batch(ov, r0, p0);
      add_batch(acc, ov, r0, p0);
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      if (r0 + r < p.group) {
        const float L = red_sum[r0 + r] + red_sum[ROWS + r0 + r] + red_sum[2 * ROWS + r0 + r] + red_sum[3 * ROWS + r0 + r];
        p.out[static_cast<int64_t>(b) * p.out_stride_b +
              (static_cast<int64_t>(head) * p.group + r0 + r) * p.out_stride_h + tid] =
            __float2half_rn(acc[r] / L);
      }
    }
  }
}

// Kernel structure: warp 4 is the producer (walks the page line, waits for a free stage, arms
// its "full" mbarrier with the byte count and issues the tile's 16 TMA copies from 16 lanes);
// warps 0..3 are consumers (wait "full", compute their page of the tile, arrive on "empty").
//
// MMA roles: the 16 tokens a consumer warp owns (exactly one page) are the M rows, the (padded)
// query heads of the group the N columns.  S^T[tok, head] = K[tok, d] . Q^T[d, head] takes K as
// the A operand straight from shared memory; P^T is transposed in registers (movmatrix) into the
// B operand of O^T[d, head] += V^T[d, tok] . P^T[tok, head], whose A operand is V read with
// ldmatrix.trans.  With N = 8 a group of up to 8 query heads wastes no tensor work; ROWS = 16
// uses two N blocks.
template <int ROWS, int STAGES>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
paged_decode_kernel(DecodeParams p, const __grid_constant__ CUtensorMap kmap,
                    const __grid_constant__ CUtensorMap vmap) {
  static_assert(ROWS == 8 || ROWS == 16, "query-group heads are padded to 8 or 16");
  constexpr int NB = ROWS / 8;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* stages = smem;
  float* merge_o = reinterpret_cast<float*>(smem + STAGES * kStageBytes);  // [4][128][ROWS]
  float* merge_ml = merge_o + kConsumerWarps * kD * ROWS;                  // [4][ROWS][2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(merge_ml + kConsumerWarps * ROWS * 2);
  int* arrival = reinterpret_cast<int*>(bars + 2 * STAGES);  // [0] pieces to merge (0 = not the last arrival), [2] everybody else had arrived already
  int* scan = reinterpret_cast<int*>(merge_o);  // start-up only: [kScanThreads + 1] page prefix

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int team = blockIdx.x / p.kv_heads;
  const int head = blockIdx.x - team * p.kv_heads;
  const uint32_t stage_base = smem_u32(stages);
  const uint32_t bar_full = smem_u32(bars);                 // [STAGES]
  const uint32_t bar_empty = bar_full + 8 * STAGES;         // [STAGES]
  if ((stage_base & 1023u) != 0) {  // the swizzled TMA boxes need 1024-byte aligned stages
    set_status(p.status, B200KV_DEV_BAD_PAGE);
    pdl_wait_then_trigger();
    return;
  }
  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, kConsumerWarps);
    }
    fence_barrier_init();
  }

  // ---- where does this team's range start and end? -----------------------------------------
  // Thread t < 128 sums the units (pages + piece_cost per non-empty sequence) and the non-empty
  // sequences of [t*per, (t+1)*per); scans over the 128 sums give the totals and the chunk holding
  // a boundary, then a short linear walk finds the sequence.
  int* scan_k = scan + kScanThreads + 1;   // non-empty sequences, same indexing
  int* scan_lo = scan_k + kScanThreads + 1;  // fewest / most pages of a non-empty sequence per thread,
  int* scan_hi = scan_lo + kScanThreads + 1; // reduced into entry [0]
  const int per = (p.batch + kScanThreads - 1) / kScanThreads;
  if (tid < kScanThreads) {
    int sum = 0, cnt = 0, lo_np = INT_MAX, hi_np = 0;
    const int lo = tid * per;
    const int hi = min(p.batch, lo + per);
    for (int b = lo; b < hi; ++b) {
      const int np = pages_of(seq_len_checked(p, b));
      sum += np + (np > 0 ? p.piece_cost : 0);
      cnt += np > 0;
      if (np > 0) {
        lo_np = min(lo_np, np);
        hi_np = max(hi_np, np);
      }
    }
    scan[tid + 1] = sum;
    scan_k[tid + 1] = cnt;
    scan_lo[tid + 1] = lo_np;
    scan_hi[tid + 1] = hi_np;
    if (tid == 0) scan[0] = scan_k[0] = 0;
  }
  __syncthreads();
  if (warp == 2 || warp == 3) {  // fewest / most pages over the 128 entries
    int* arr = warp == 2 ? scan_lo : scan_hi;
    int v = arr[1 + lane * 4];
#pragma unroll
    for (int i = 1; i < 4; ++i) v = warp == 2 ? min(v, arr[1 + lane * 4 + i]) : max(v, arr[1 + lane * 4 + i]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const int o = __shfl_xor_sync(0xffffffffu, v, d);
      v = warp == 2 ? min(v, o) : max(v, o);
    }
    if (lane == 0) arr[0] = v;
  }
  if (warp < 2) {  // inclusive scans of [1..128] by one warp each, 4 values per lane
    int* arr = warp == 0 ? scan : scan_k;
    int v[4];
    int run = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      run += arr[1 + lane * 4 + i];
      v[i] = run;
    }
    int incl = run;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += o;
    }
    const int excl = incl - run;
#pragma unroll
    for (int i = 0; i < 4; ++i) arr[1 + lane * 4 + i] = v[i] + excl;
  }
  __syncthreads();
  const int64_t units_total = scan[kScanThreads];
  const int nonempty_total = scan_k[kScanThreads];
  const int64_t np_total = units_total - static_cast<int64_t>(p.piece_cost) * nonempty_total;
  int nteams_eff = effective_teams(p.nteams, np_total);
  // Sequences of one length whose count divides into about as many groups as there are teams: one
  // team per group of k whole sequences.  Every piece is then a whole sequence — nothing is
  // published, counted or merged — at the price of leaving up to a quarter of the CTA slots empty,
  // which the streaming rate survives.
  if (nonempty_total > 0 && scan_lo[0] == scan_hi[0]) {
    const int k = (nonempty_total + p.nteams - 1) / p.nteams;   // sequences per team
    const int groups = nonempty_total / k;
    if (groups * k == nonempty_total && 4 * groups >= 3 * p.nteams) nteams_eff = groups;
  }
  const bool any_empty = nonempty_total < p.batch;

  // Unit position x -> (sequence, page inside it, flat page index).  Positions inside a sequence's
  // piece_cost extra units map to its first page.
  int start_b = 0, start_page = 0, start_k = 0;
  int64_t r_begin = 0, r_end = 0;
  if (np_total > 0 && team < nteams_eff) {
#pragma unroll 1
    for (int side = 0; side < 2; ++side) {
      const int64_t x = team_begin(team + side, nteams_eff, units_total);
      int64_t flat = np_total;
      int sb = 0, sp = 0, sk = 0;
      if (x < units_total) {
        int lo = 0, hi = kScanThreads - 1;   // last chunk whose unit prefix <= x
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (scan[mid] <= x) lo = mid; else hi = mid - 1;
        }
        int64_t acc = scan[lo];
        sk = scan_k[lo];
        int64_t pages_before = acc - static_cast<int64_t>(p.piece_cost) * sk;
        int b = lo * per;
        for (; b < p.batch; ++b) {   // ends before the batch does when the lengths are consistent
          const int np = pages_of(seq_len_checked(p, b));
          const int w = np + (np > 0 ? p.piece_cost : 0);
          if (acc + w > x) break;
          acc += w;
          pages_before += np;
          sk += np > 0;
        }
        if (b < p.batch) {
          const int64_t o = x - acc - p.piece_cost;
          sb = b;
          sp = o > 0 ? static_cast<int>(o) : 0;
          flat = pages_before + sp;
        }
      }
      if (side == 0) {
        start_b = sb;
        start_page = sp;
        start_k = sk;
        r_begin = flat;
      } else {
        r_end = flat;
      }
    }
  }
  const bool has_range = r_end > r_begin;   // false also for a range wholly inside a sequence's extra units
  __syncthreads();  // the scan scratch aliases the merge buffer; barrier inits are visible

  // ================================= producer warp ==========================================
  // All 32 lanes walk the page line in lock step (cheap, uniform); lane 0 arms the stage's
  // "full" barrier with the byte count, then lanes 0..15 each issue ONE of the tile's copies:
  // lane = 4*page + {K low half, K high half, V low half, V high half}.
  if (warp == kConsumerWarps) {
    if (!has_range) {
      pdl_wait_then_trigger();
      return;
    }
    if (lane == 0) {
      prefetch_tensormap(&kmap);
      prefetch_tensormap(&vmap);
    }
    const uint64_t policy = l2_evict_first_policy();
    Walker prod;
    prod.flat = r_begin;
    prod.flat_end = r_end;
    prod.kseq = start_k;
    prod.enter(p, start_b, start_page);
    Fetch fq[kLead];
#pragma unroll
    for (int i = 0; i < kLead; ++i) fetch_next(p, prod, fq[i], head, lane, false);
    const int my_page = lane >> 2;
    const int my_part = lane & 3;
    const CUtensorMap* my_map = (my_part & 2) ? &vmap : &kmap;
    // Pull the first tiles towards L2 while the previous kernel is still finishing: L2 is the
    // point of coherence, so rows that kernel writes afterwards are still seen by the real loads.
#pragma unroll
    for (int i = 0; i < kL2PrefetchTiles; ++i) {
      const Fetch& f = fq[i];
      if (lane < 4 * f.npages) {
        int32_t id = f.id[0];
#pragma unroll
        for (int k = 1; k < kTilePages; ++k) id = (my_page == k) ? f.id[k] : id;
        const int64_t slot = (p.table_kind == B200KV_TABLE_BLOCK) ? static_cast<int64_t>(id) * kPS
                                                                  : static_cast<int64_t>(id);
        if (slot >= 0 && slot + kPS <= p.pool_tokens)
          tma_prefetch_l2_3d(my_map, (my_part & 1) * 64, head, static_cast<int>(slot));
      }
    }
    pdl_wait_then_trigger();  // the pool and the new rows may have been written by the previous kernel
#pragma unroll
    for (int i = 0; i < kLead; ++i)
      if (fq[i].app_b >= 0) load_new_row(p, fq[i], head, lane);
    const uint32_t my_off = my_page * kPageBytes + (my_part & 1) * (kPageBytes / 2) +
                            ((my_part & 2) ? kTileBytes : 0);
    for (int it = 0;; ++it) {
      const Fetch f = fq[0];
      if (f.ntok == 0) break;
      const int st = it % STAGES;
      if (f.app_b >= 0) {
        // Fused append: this tile holds the last page of its sequence, whose newest row is not in
        // the pool yet.  Lanes 0..15 write the K row of this head, lanes 16..31 the V row, 16 bytes
        // each; the proxy fence orders these generic stores before the bulk copies issued below.
        int32_t last_id = f.id[0];
#pragma unroll
        for (int i = 1; i < kTilePages; ++i) last_id = (f.npages - 1 == i) ? f.id[i] : last_id;
        const int64_t want = ((p.table_kind == B200KV_TABLE_BLOCK) ? static_cast<int64_t>(last_id) * kPS
                                                                    : static_cast<int64_t>(last_id)) + f.app_off;
        const int64_t slot = f.app_slot;
        if (slot < 0 || slot >= p.pool_tokens) {
          set_status(p.status, B200KV_DEV_BAD_SLOT);   // never dereferenced
        } else {
          if (slot != want) set_status(p.status, B200KV_DEV_BAD_SLOT);   // not this sequence's last position
          __half* dst = (lane < 16 ? p.k_base : p.v_base) + slot * p.kv_tok_stride +
                        static_cast<int64_t>(head) * p.kv_head_stride + (lane & 15) * 8;
          *reinterpret_cast<uint4*>(dst) = make_uint4(f.app_row0, f.app_row1, f.app_row2, f.app_row3);
        }
        asm volatile("fence.proxy.async.global;\n" ::: "memory");
        __syncwarp();
      }
      if (it >= STAGES && !mbar_wait_bounded(bar_empty + 8 * st, ((it / STAGES) - 1) & 1)) {
        set_status(p.status, B200KV_DEV_WAIT_TIMEOUT);
        break;  // consumers run into their own bounded waits and stop computing too
      }
      const uint32_t full = bar_full + 8 * st;
      if (lane == 0)
        mbar_arrive_expect_tx(full, static_cast<uint32_t>(f.npages) * (2 * kPageBytes));
      __syncwarp();
      if (lane < 4 * f.npages) {
        int32_t id = f.id[0];
#pragma unroll
        for (int i = 1; i < kTilePages; ++i) id = (my_page == i) ? f.id[i] : id;
        int64_t slot = (p.table_kind == B200KV_TABLE_BLOCK) ? static_cast<int64_t>(id) * kPS
                                                            : static_cast<int64_t>(id);
        if (slot < 0 || slot + kPS > p.pool_tokens) {
          // never dereference a bad entry: report it and read page 0 instead
          set_status(p.status, B200KV_DEV_BAD_PAGE);
          slot = 0;
        }
        tma_load_3d(stage_base + st * kStageBytes + my_off, my_map, full, (my_part & 1) * 64, head,
                    static_cast<int>(slot), policy);
      }
#pragma unroll
      for (int i = 0; i + 1 < kLead; ++i) fq[i] = fq[i + 1];
      fetch_next(p, prod, fq[kLead - 1], head, lane, true);
    }
    return;
  }

  // ================================= consumer warps =========================================
  pdl_wait_then_trigger();  // q, the workspace and out belong to earlier kernels until here
  if (team == 0 && any_empty) {
    // No keys: the output rows are defined as zero, and nobody else writes them.
    for (int b = 0; b < p.batch; ++b) {
      if (seq_len_checked(p, b) != 0) continue;
      for (int g = 0; g < p.group; ++g)
        p.out[static_cast<int64_t>(b) * p.out_stride_b +
              (static_cast<int64_t>(head) * p.group + g) * p.out_stride_h + tid] = __float2half_rn(0.f);
    }
  }
  if (!has_range) return;

  Walker cons;
  cons.flat = r_begin;
  cons.flat_end = r_end;
  cons.kseq = start_k;
  cons.enter(p, start_b, start_page);

  uint32_t qf[NB][8][2];  // Q^T as mma B fragments: 8 k-steps of 16 along head_dim
  float o[8][NB][4];      // O^T accumulator: 8 M blocks of 16 along head_dim
  float m_run[NB][2], l_run[NB][2];  // per head column (2 per N block per lane)
  const int frow = lane >> 2;        // fragment row: token (S^T) or head_dim (O^T) within 8
  const int fcol = (lane & 3) * 2;   // fragment column pair: head within the N block
  const int mi = lane >> 3;          // which 8x8 matrix of an ldmatrix.x4 this lane addresses
  const int lrow = lane & 7;

  // Q of one sequence as B fragments.  The next sequence's Q is requested when a piece ends, so
  // that its latency hides under the merge of that piece instead of in front of the next tile.
  uint32_t qn[NB][8][2];
  int qn_b = -1;
  auto load_q = [&](int b, uint32_t (&dst)[NB][8][2]) {
    const __half* qb = p.q + static_cast<int64_t>(b) * p.q_stride_b +
                       static_cast<int64_t>(head) * p.group * p.q_stride_h + fcol;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const int hq = nb * 8 + frow;  // B fragment column n = lane / 4
      const bool hok = hq < p.group;
      const __half* qh = qb + static_cast<int64_t>(hq) * p.q_stride_h;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        dst[nb][ks][0] = hok ? __ldg(reinterpret_cast<const uint32_t*>(qh + ks * 16)) : 0u;
        dst[nb][ks][1] = hok ? __ldg(reinterpret_cast<const uint32_t*>(qh + ks * 16 + 8)) : 0u;
      }
    }
  };

  bool alive = true;   // false once a wait of this warp ran out: keep walking, stop computing
  unsigned seen_arrivals = 0;   // thread 0: the piece counter as seen at the start of a piece's last tile
  Tile t;
  for (int it = 0; cons.next(p, t); ++it) {
    if (t.first) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) o[j][nb][0] = o[j][nb][1] = o[j][nb][2] = o[j][nb][3] = 0.f;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        m_run[nb][0] = m_run[nb][1] = -INFINITY;
        l_run[nb][0] = l_run[nb][1] = 0.f;
      }
      if (qn_b == t.b) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            qf[nb][ks][0] = qn[nb][ks][0];
            qf[nb][ks][1] = qn[nb][ks][1];
          }
      } else {
        load_q(t.b, qf);
      }
    }

    // Last tile of a partial piece: look at the sequence's arrival counter now (the answer is
    // needed only after this tile's arithmetic).  If every other piece has already arrived, this
    // CTA is going to be the one that merges, and its own hand-over needs neither the publishing
    // fence nor the counter's round trip.
    if (tid == 0 && t.last && !t.whole) {
      asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];\n"
                   : "=r"(seen_arrivals)
                   : "l"(p.piece_ctr + static_cast<int64_t>(t.b) * p.kv_heads + head)
                   : "memory");
    }
    const int st = it % STAGES;
    if (alive && !mbar_wait_bounded(bar_full + 8 * st, (it / STAGES) & 1)) {
      set_status(p.status, B200KV_DEV_WAIT_TIMEOUT);
      alive = false;
    }

    const int wtok = alive ? t.ntok - warp * kPS : 0;  // valid tokens of this warp's page (may be <= 0)
    if (wtok > 0) {
      const uint32_t kpage = stage_base + st * kStageBytes + warp * kPageBytes;
      const uint32_t vpage = kpage + kTileBytes;
      if (wtok < kPS) {
        // Last page of a sequence: its rows past the length were never written and may hold
        // anything (NaN included); zero them in V so that P = 0 really contributes nothing.
        for (int i = lane; i < (kPS - wtok) * 16; i += 32) {
          const int r = wtok + (i >> 4);
          const int c = i & 15;
          asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n" ::"r"(vpage + page_chunk_off(r, c)),
                       "r"(0)
                       : "memory");
        }
        fence_proxy_async_smem();  // these generic-proxy writes precede the next TMA refill
        __syncwarp();
      }
      // ---- S^T = K Q^T over this warp's 16 tokens ---------------------------------------------
      float s[NB][4];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
      {
        const int kr = ((mi & 1) << 3) + lrow;  // token row this lane addresses
        const int csel = mi >> 1;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          uint32_t ka[4];
          ldmatrix_x4(ka, kpage + page_chunk_off(kr, 2 * ks + csel));
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) mma_16816(s[nb], ka, qf[nb][ks][0], qf[nb][ks][1]);
        }
      }
      // ---- online softmax per head column (log2 domain) ---------------------------------------
      const bool ok0 = frow < wtok;
      const bool ok1 = (frow + 8) < wtok;
      float alpha[NB][2];
      uint32_t pb[NB][2];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        float pr[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float s0 = ok0 ? s[nb][h] * p.scale_log2 : -INFINITY;
          const float s1 = ok1 ? s[nb][h + 2] * p.scale_log2 : -INFINITY;
          float mx = fmaxf(s0, s1);
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
          const float m_new = fmaxf(m_run[nb][h], mx);
          const float msub = (m_new == -INFINITY) ? 0.f : m_new;
          alpha[nb][h] = fast_exp2(m_run[nb][h] - msub);
          m_run[nb][h] = m_new;
          pr[h] = fast_exp2(s0 - msub);
          pr[h + 2] = fast_exp2(s1 - msub);
          l_run[nb][h] = l_run[nb][h] * alpha[nb][h] + pr[h] + pr[h + 2];
        }
        // P^T[tok, head] -> B fragment [k = tok, n = head]
        pb[nb][0] = movmatrix_trans(pack_half2(pr[0], pr[1]));
        pb[nb][1] = movmatrix_trans(pack_half2(pr[2], pr[3]));
      }
      // ---- O^T = alpha * O^T + V^T P^T --------------------------------------------------------
      {
        const int vr = ((mi >> 1) << 3) + lrow;
        const int csel = mi & 1;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint32_t va[4];
          ldmatrix_x4_trans(va, vpage + page_chunk_off(vr, 2 * j + csel));
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            float(&acc)[4] = o[j][nb];
            acc[0] *= alpha[nb][0];
            acc[1] *= alpha[nb][1];
            acc[2] *= alpha[nb][0];
            acc[3] *= alpha[nb][1];
            mma_16816(acc, va, pb[nb][0], pb[nb][1]);
          }
        }
      }
    }
    // This warp is done with the stage: hand it back to the producer.
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_empty + 8 * st);

    if (t.last) {
      // ---- merge the four warps' (m, l, O) and emit the piece --------------------------------
      if (cons.flat < cons.flat_end) {   // another piece follows: it starts the next non-empty sequence
        int nb_seq = t.b + 1;
        while (nb_seq < p.batch && pages_of(seq_len_checked(p, nb_seq)) == 0) ++nb_seq;
        if (nb_seq < p.batch) {
          load_q(nb_seq, qn);
          qn_b = nb_seq;
        }
      }
      // the merge buffer is shared by the four consumer warps: named barrier 1 (128 threads)
      // before it is rewritten and again before it is read
      consumer_bar();
      float* mo = merge_o + warp * kD * ROWS;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float l = l_run[nb][h];
          l += __shfl_xor_sync(0xffffffffu, l, 4);
          l += __shfl_xor_sync(0xffffffffu, l, 8);
          l += __shfl_xor_sync(0xffffffffu, l, 16);
          if (frow == 0) {
            float* ml = merge_ml + (warp * ROWS + nb * 8 + fcol + h) * 2;
            ml[0] = m_run[nb][h];
            ml[1] = l;
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int d0 = j * 16 + frow;
          *reinterpret_cast<float2*>(mo + d0 * ROWS + nb * 8 + fcol) = make_float2(o[j][nb][0], o[j][nb][1]);
          *reinterpret_cast<float2*>(mo + (d0 + 8) * ROWS + nb * 8 + fcol) =
              make_float2(o[j][nb][2], o[j][nb][3]);
        }
      }
      // (thread 0, partial pieces) had every other piece of the sequence arrived when this piece's
      // last tile began?  The flag rides on the barrier below.
      const int64_t u0 = t.units0 + p.piece_cost;
      const int t_first = team_of(u0, nteams_eff, units_total);
      const int t_last = team_of(u0 + t.np - 1, nteams_eff, units_total);
      const int npieces = t_last - t_first + 1;
      if (tid == 0 && !t.whole) {
        const bool others_in = seen_arrivals == static_cast<unsigned>(npieces - 1);
        if (others_in) __threadfence();   // acquire: their published rows come before what follows
        arrival[2] = others_in ? 1 : 0;
      }
      consumer_bar();
      const int64_t slot = (static_cast<int64_t>(team) + t.b) * p.kv_heads + head;
      // Thread = output column; its ROWS values of a warp's O are contiguous in the merge buffer
      // (vector loads), the (m, l) pairs are broadcast loads, and all rows are merged in registers.
#pragma unroll 1
      for (int r0 = 0; r0 < ROWS; r0 += 8) {   // eight rows at a time keeps the registers modest
        float M[8], L[8], acc[8];
        float mw[kConsumerWarps][8], lw[kConsumerWarps][8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          M[r] = -INFINITY;
          L[r] = acc[r] = 0.f;
        }
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) {
#pragma unroll
          for (int r2 = 0; r2 < 4; ++r2) {
            const float4 v = *reinterpret_cast<const float4*>(merge_ml + (w * ROWS + r0 + 2 * r2) * 2);
            mw[w][2 * r2] = v.x;
            lw[w][2 * r2] = v.y;
            mw[w][2 * r2 + 1] = v.z;
            lw[w][2 * r2 + 1] = v.w;
            M[2 * r2] = fmaxf(M[2 * r2], v.x);
            M[2 * r2 + 1] = fmaxf(M[2 * r2 + 1], v.z);
          }
        }
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) {
          const float4 v0 = *reinterpret_cast<const float4*>(merge_o + (w * kD + tid) * ROWS + r0);
          const float4 v1 = *reinterpret_cast<const float4*>(merge_o + (w * kD + tid) * ROWS + r0 + 4);
          const float ov[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            const float sc = (mw[w][r] == -INFINITY) ? 0.f : fast_exp2(mw[w][r] - M[r]);
            L[r] += sc * lw[w][r];
            acc[r] += sc * ov[r];
          }
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          if (r0 + r < p.group) {
            const float val = acc[r] / L[r];
            if (t.whole) {
              p.out[static_cast<int64_t>(t.b) * p.out_stride_b +
                    (static_cast<int64_t>(head) * p.group + r0 + r) * p.out_stride_h + tid] =
                  __float2half_rn(val);
            } else {
              p.part_o[(slot * ROWS + r0 + r) * kD + tid] = val;
              if (tid == 0) p.part_lse[slot * ROWS + r0 + r] = M[r] + log2f(L[r]);
            }
          }
        }
      }
      if (!t.whole) {
        // A partial: publish it, count it, and merge the sequence if it was the last one to arrive.
        // The counter wraps to zero on the last arrival, so it needs no reset between launches.
        unsigned* ctr = p.piece_ctr + static_cast<int64_t>(t.b) * p.kv_heads + head;
        if (arrival[2] != 0) {
          // Everybody else had arrived before this piece's last tile: nobody waits for this
          // partial but this CTA itself, which reads it back through L2 in the merge (a barrier,
          // not a fence, orders that).  The count still has to wrap the counter to zero.
          consumer_bar();
          if (tid == 0) atomicInc(ctr, static_cast<unsigned>(npieces - 1));
          merge_pieces<ROWS>(p, t.b, head, t_first, npieces, tid, merge_o, merge_ml);
        } else {
          __threadfence();
          consumer_bar();
          if (tid == 0) {
            const unsigned old = atomicInc(ctr, static_cast<unsigned>(npieces - 1));
            const bool last_arrival = old == static_cast<unsigned>(npieces - 1);
            arrival[0] = last_arrival ? npieces : 0;
            // Acquire side of the hand-over, paid by the merging CTA only: this thread saw the other
            // pieces' counts; the fence orders their published rows before everything that follows,
            // and the named barrier below extends that to the other 127 threads.
            if (last_arrival) __threadfence();
          }
          consumer_bar();
          if (arrival[0] > 0) merge_pieces<ROWS>(p, t.b, head, t_first, npieces, tid, merge_o, merge_ml);
        }
      }
    }
  }
}

inline int rows_for_group(int group) { return group <= 8 ? 8 : 16; }
inline int max_teams(int sms, int kv_heads) {
  const int t = (sms * kCtasPerSm) / kv_heads;
  return t < 1 ? 1 : t;
}
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Tuning overrides (b200kv_set_option): 0 = automatic.
int g_option_teams = 0;
int g_option_piece_cost = 0;

template <int ROWS, int STAGES>
int launch_decode(const DecodeParams& p, const CUtensorMap& kmap, const CUtensorMap& vmap,
                  bool programmatic, cudaStream_t stream) {
  constexpr int smem = STAGES * kStageBytes + kConsumerWarps * ROWS * kD * 4 +
                       kConsumerWarps * ROWS * 2 * 4 + (2 * STAGES + 2) * 8;
  static bool attr_done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return record_cuda_error(cudaGetLastError());
  if (dev < 0 || dev >= 64 || !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(paged_decode_kernel<ROWS, STAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev >= 0 && dev < 64) attr_done[dev] = true;
  }
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(p.nteams * p.kv_heads));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = programmatic ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, paged_decode_kernel<ROWS, STAGES>, p, kmap, vmap);
  if (e != cudaSuccess) return record_cuda_error(e);
  return check_launch();
}

}  // namespace

int set_decode_option(int option, int64_t value) {
  if (value < 0 || value > 65535) return B200KV_EINVAL;
  switch (option) {
    case B200KV_OPT_DECODE_TEAMS: g_option_teams = static_cast<int>(value); return B200KV_OK;
    case B200KV_OPT_DECODE_PIECE_COST: g_option_piece_cost = static_cast<int>(value); return B200KV_OK;
    default: return B200KV_EINVAL;
  }
}

size_t decode_workspace_bytes(int batch, int q_heads, int kv_heads, int head_dim) {
  if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim != kD) return 0;
  if (q_heads % kv_heads != 0 || q_heads / kv_heads > 16) return 0;
  if (static_cast<int64_t>(batch) * kv_heads > kMaxCounters) return 0;
  const int sms = device_sm_count();
  if (sms <= 0) return 0;
  const int rows = rows_for_group(q_heads / kv_heads);
  const size_t nslots = static_cast<size_t>(max_teams(sms, kv_heads)) + static_cast<size_t>(batch);
  const size_t po = align_up(nslots * kv_heads * rows * kD * sizeof(float), 256);
  const size_t pl = align_up(nslots * kv_heads * rows * sizeof(float), 256);
  return kCounterBytes + po + pl;
}

int paged_decode(const DecodeArgs& a, cudaStream_t stream) {
  if (a.batch < 0 || a.q_heads <= 0 || a.kv_heads <= 0 || a.max_seq_len < 0) return B200KV_EINVAL;
  if (a.batch == 0) return B200KV_OK;
  if (!a.q || !a.k_base || !a.v_base || !a.table || !a.seq_lens || !a.out || !a.workspace)
    return B200KV_EINVAL;
  if (a.table_kind != B200KV_TABLE_BLOCK && a.table_kind != B200KV_TABLE_TOKEN) return B200KV_EINVAL;
  if (a.head_dim != kD || a.page_size != kPS) return B200KV_EUNSUPPORTED;
  if (a.q_heads % a.kv_heads != 0) return B200KV_EUNSUPPORTED;
  const int group = a.q_heads / a.kv_heads;
  if (group > 16) return B200KV_EUNSUPPORTED;
  if (a.batch > 4096) return B200KV_ETOOLARGE;
  if (static_cast<int64_t>(a.batch) * a.kv_heads > kMaxCounters) return B200KV_ETOOLARGE;
  if (a.max_seq_len > (int64_t{1} << 30)) return B200KV_ETOOLARGE;
  // The table must hold every row and every position the lengths can name.
  if (a.table_rows <= 0 || a.table_cols <= 0 || a.table_row_stride < a.table_cols) return B200KV_EINVAL;
  if (a.row_ids == nullptr && a.batch > a.table_rows) return B200KV_EINVAL;
  const int64_t width_tokens = a.table_cols * (a.table_kind == B200KV_TABLE_BLOCK ? kPS : 1);
  if (a.max_seq_len > width_tokens) return B200KV_EINVAL;
  if ((a.new_k == nullptr) != (a.slots == nullptr) || (a.new_k == nullptr) != (a.new_v == nullptr))
    return B200KV_EINVAL;
  if (a.flags & ~B200KV_DECODE_SERIALIZED) return B200KV_EINVAL;
  auto mis = [](const void* ptr, uintptr_t al) { return (reinterpret_cast<uintptr_t>(ptr) & (al - 1)) != 0; };
  if (mis(a.k_base, 16) || mis(a.v_base, 16) || mis(a.q, 4) || mis(a.out, 8) || mis(a.workspace, 16))
    return B200KV_EALIGN;
  if (a.kv_tok_stride % 8 != 0 || a.kv_head_stride % 8 != 0) return B200KV_EALIGN;
  if (a.q_stride_b % 2 != 0 || a.q_stride_h % 2 != 0) return B200KV_EALIGN;
  if (a.out_stride_b % 4 != 0 || a.out_stride_h % 4 != 0) return B200KV_EALIGN;
  if (a.new_k != nullptr) {
    if (mis(a.new_k, 16) || mis(a.new_v, 16) || a.new_k_tok_stride % 8 != 0 || a.new_v_tok_stride % 8 != 0)
      return B200KV_EALIGN;
    if (a.new_k_tok_stride < static_cast<int64_t>(a.kv_heads) * kD ||
        a.new_v_tok_stride < static_cast<int64_t>(a.kv_heads) * kD)
      return B200KV_EINVAL;
  }
  const size_t need = decode_workspace_bytes(a.batch, a.q_heads, a.kv_heads, a.head_dim);
  if (need == 0) return B200KV_ECUDA;
  if (a.workspace_bytes < need) return B200KV_EWORKSPACE;

  const int sms = device_sm_count();
  const int rows = rows_for_group(group);
  const int teams_cap = max_teams(sms, a.kv_heads);
  // Do not launch more teams than the page bound can feed.
  const int64_t pages_bound = static_cast<int64_t>(a.batch) * ((a.max_seq_len + kPS - 1) / kPS);
  int64_t teams = pages_bound / kMinPagesPerTeam;
  if (teams > teams_cap) teams = teams_cap;
  int piece_cost = kDefaultPieceCost;
  if (teams == teams_cap && pages_bound < static_cast<int64_t>(kMediumRangePages) * teams_cap) {
    // Ranges of a few dozen pages per CTA (KV-head shards of a modest batch): most pieces are
    // partial ones, whose ends cost more (publish, count, maybe merge), so they weigh more
    // against the pages when the line is cut.
    piece_cost = kShortRangePieceCost;
    if (pages_bound < static_cast<int64_t>(kShortRangePages) * teams_cap) {
      // Shorter still: the launch is latency-bound rather than bandwidth-bound.  Seven eighths of
      // the CTA slots stream as fast, leave slots free for the next launch's CTAs to do their
      // planning under this launch's tail, and cut every sequence in fewer pieces.
      teams = (7 * static_cast<int64_t>(teams_cap)) / 8;
    }
  }
  if (g_option_teams > 0 && teams > g_option_teams) teams = g_option_teams;
  if (teams < 1) teams = 1;
  if (g_option_piece_cost > 0) piece_cost = g_option_piece_cost;

  DecodeParams p{};
  p.q = static_cast<const __half*>(a.q);
  p.q_stride_b = a.q_stride_b;
  p.q_stride_h = a.q_stride_h;
  p.k_base = static_cast<__half*>(const_cast<void*>(a.k_base));
  p.v_base = static_cast<__half*>(const_cast<void*>(a.v_base));
  p.kv_tok_stride = a.kv_tok_stride;
  p.kv_head_stride = a.kv_head_stride;
  p.pool_tokens = a.pool_tokens;
  p.table = a.table;
  p.table_row_stride = a.table_row_stride;
  p.table_kind = a.table_kind;
  p.table_rows = a.table_rows;
  p.row_ids = a.row_ids;
  p.seq_lens = a.seq_lens;
  p.seq_lens_i64 = a.seq_lens_i64;
  p.batch = a.batch;
  p.q_heads = a.q_heads;
  p.kv_heads = a.kv_heads;
  p.group = group;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.max_seq_len = a.max_seq_len;
  p.nteams = static_cast<int>(teams);
  p.piece_cost = piece_cost;
  p.new_k = static_cast<const __half*>(a.new_k);
  p.new_v = static_cast<const __half*>(a.new_v);
  p.new_k_tok_stride = a.new_k_tok_stride;
  p.new_v_tok_stride = a.new_v_tok_stride;
  p.slots = a.slots;
  const size_t nslots = static_cast<size_t>(teams_cap) + static_cast<size_t>(a.batch);
  uint8_t* ws = static_cast<uint8_t*>(a.workspace);
  p.piece_ctr = reinterpret_cast<unsigned*>(ws);
  p.part_o = reinterpret_cast<float*>(ws + kCounterBytes);
  p.part_lse = reinterpret_cast<float*>(ws + kCounterBytes +
                                        align_up(nslots * a.kv_heads * rows * kD * sizeof(float), 256));
  p.out = static_cast<__half*>(a.out);
  p.out_stride_b = a.out_stride_b;
  p.out_stride_h = a.out_stride_h;
  p.status = a.status;

  // TMA views of the K and V halves of the pool (d, head, token); one box = 16 token rows of
  // 64 halves, i.e. half a page of one head.
  CUtensorMap kmap, vmap;
  int rc = cached_kv_tensor_map(&kmap, a.k_base, a.pool_tokens, a.kv_tok_stride, a.kv_head_stride,
                                a.kv_heads, kD, kPS);
  if (rc != B200KV_OK) return rc;
  rc = cached_kv_tensor_map(&vmap, a.v_base, a.pool_tokens, a.kv_tok_stride, a.kv_head_stride,
                            a.kv_heads, kD, kPS);
  if (rc != B200KV_OK) return rc;
  const bool programmatic = (a.flags & B200KV_DECODE_SERIALIZED) == 0;
  if (rows == 8) return launch_decode<8, kStagesRows8>(p, kmap, vmap, programmatic, stream);
  return launch_decode<16, 2>(p, kmap, vmap, programmatic, stream);
}

// ---- decode on library-owned scratch (no allocation anywhere on the call path) -----------------
//
// Some hosts cannot hand us a workspace because they cannot obtain device memory at call time at
// all: a serving process that gave its whole device budget to one arena at start-up and treats a
// later cudaMalloc as a fault; a plug-in whose device memory is accounted for by the embedding
// application; code running where the CUDA allocator must not be entered (a latency-critical
// loop that cannot afford the device-wide synchronisation cudaMalloc / cudaFree imply).  For them
// the split-KV partials and the arrival counters live in this file-scope device array instead.
// Every GPU that loads the library holds these bytes until the process exits, which is why the
// size is modest and fixed.  The array starts zero-filled, which is the state the counters need.
constexpr size_t kStaticScratchBytes = B200KV_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

int paged_decode_static_scratch(const DecodeArgs& args, cudaStream_t stream) {
  if (args.batch < 0) return B200KV_EINVAL;
  if (args.batch == 0) return B200KV_OK;
  const size_t need = decode_workspace_bytes(args.batch, args.q_heads, args.kv_heads, args.head_dim);
  if (need > kStaticScratchBytes) return B200KV_ETOOLARGE;  // need == 0: rejected below with its own code
  // In host code `g_decode_scratch` is only a handle for the symbol, not an address the GPU
  // understands; the device address is asked for once per device, with that device current.
  static void* scratch_of_device[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return record_cuda_error(cudaGetLastError());
  if (dev < 0 || dev >= 64) return B200KV_EUNSUPPORTED;
  if (scratch_of_device[dev] == nullptr) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_decode_scratch);
    if (e != cudaSuccess || ptr == nullptr) return record_cuda_error(e != cudaSuccess ? e : cudaErrorInvalidSymbol);
    scratch_of_device[dev] = ptr;
  }
  DecodeArgs a = args;
  a.workspace = scratch_of_device[dev];
  a.workspace_bytes = kStaticScratchBytes;
  return paged_decode(a, stream);
}

}  // namespace b200kv
