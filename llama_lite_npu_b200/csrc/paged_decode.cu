// Paged flash-decoding for B200: persistent split-KV kernel + log-sum-exp merge.
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
//   * the launch has `nteams` teams of Hkv CTAs; team i takes the contiguous page range
//     [i*NP/nteams, (i+1)*NP/nteams) and CTA k of the team handles KV head k over it, so
//     every CTA streams the same number of bytes (+-1 page) whatever the length mix, and
//     the Hkv CTAs of a team sweep the same token rows (one 2*Hkv*128-half pool row holds
//     all heads of a token) at the same time;
//   * a team's range may cover the tail of one sequence, several whole sequences and the
//     head of another: each such "piece" yields either the final fp16 output (piece ==
//     whole sequence) or an fp32 partial (normalised output + log2-domain log-sum-exp) in
//     slot team + b of the workspace, merged afterwards by decode_combine_kernel.
//
// Pipeline inside a CTA (128 threads, 4 warps, 2 CTAs per SM): tiles of 64 tokens (4
// pages; K and V rows of 256 B each) are staged through a 3-deep cp.async ring of 32 KB
// stages that keeps running across piece boundaries; shared-memory rows are XOR-swizzled
// in 16-byte chunks so ldmatrix is conflict-free.  Warp w owns tokens [16w, 16w+16) of
// every tile: S = Q K^T and O += P V run on mma.sync m16n8k16 (fp16 in, fp32 accumulate)
// with the G query heads as the M rows; per-warp online-softmax states are merged through
// shared memory at the end of a piece.  The kernel is HBM-bound: algorithmic bytes per
// token per KV head = 2 (K,V) * 128 * 2 B.
#include "common.cuh"
#include "launch.h"

namespace b200kv {

namespace {

constexpr int kD = 128;
constexpr int kPS = 16;
constexpr int kTileTok = 64;
constexpr int kTilePages = kTileTok / kPS;
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kRowBytes = kD * 2;
constexpr int kTileBytes = kTileTok * kRowBytes;  // one of K or V
constexpr int kStageBytes = 2 * kTileBytes;
constexpr int kCtasPerSm = 2;
constexpr int kMinPagesPerTeam = 8;
constexpr int kCombineThreads = 256;

struct DecodeParams {
  const __half* q;
  int64_t q_stride_b, q_stride_h;
  const __half* k_base;
  const __half* v_base;
  int64_t kv_tok_stride, kv_head_stride, pool_tokens;
  const int32_t* table;
  int64_t table_row_stride;
  int table_kind;
  const int32_t* row_ids;
  const void* seq_lens;
  int seq_lens_i64;
  int batch, q_heads, kv_heads, group;
  float scale_log2;
  int64_t max_seq_len;
  int nteams;
  float* part_o;    // [nslots][kv_heads][ROWS][128]
  float* part_lse;  // [nslots][kv_heads][ROWS]
  __half* out;
  int64_t out_stride_b, out_stride_h;
  int32_t* status;
};

__device__ __forceinline__ int seq_len_checked(const DecodeParams& p, int b) {
  int64_t len = load_len(p.seq_lens, p.seq_lens_i64, b);
  if (len < 0) {
    set_status(p.status, B200KV_DEV_BAD_LENGTH);
    len = 0;
  } else if (len > p.max_seq_len) {
    set_status(p.status, B200KV_DEV_BAD_LENGTH);
    len = p.max_seq_len;
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
__device__ __forceinline__ int64_t team_begin(int team, int nteams_eff, int64_t np_total) {
  return (static_cast<int64_t>(team) * np_total) / nteams_eff;
}
// Team whose range holds flat page x (0 <= x < np_total).
__device__ __forceinline__ int team_of(int64_t x, int nteams_eff, int64_t np_total) {
  return static_cast<int>(((x + 1) * nteams_eff - 1) / np_total);
}

struct Tile {
  int b;        // sequence (batch position)
  int row;      // table row of that sequence
  int page0;    // first logical page of the tile
  int npages;   // pages in the tile (1..4)
  int ntok;     // valid tokens in the tile
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
      enter(p, nb, 0);
    }
    t.b = b;
    t.row = row;
    t.page0 = page;
    t.npages = min(kTilePages, piece_end - page);
    const int tok_end = min(len, (page + t.npages) * kPS);
    t.ntok = tok_end - page * kPS;
    t.first = (page == piece_begin);
    t.last = (page + t.npages == piece_end);
    t.whole = (piece_begin == 0 && piece_end == np);
    page += t.npages;
    flat += t.npages;
    return true;
  }
};

// Token slot of the first row of each page of a tile, or -1 (zero-fill) when the tile has no
// such page or the table entry is out of range.
__device__ __forceinline__ void load_page_bases(const DecodeParams& p, const Tile& t, bool valid,
                                                int64_t (&base)[kTilePages]) {
#pragma unroll
  for (int i = 0; i < kTilePages; ++i) {
    base[i] = -1;
    if (valid && i < t.npages) {
      const int lp = t.page0 + i;
      const int32_t* rowp = p.table + static_cast<int64_t>(t.row) * p.table_row_stride;
      int64_t s = (p.table_kind == B200KV_TABLE_BLOCK)
                      ? static_cast<int64_t>(__ldg(rowp + lp)) * kPS
                      : static_cast<int64_t>(__ldg(rowp + static_cast<int64_t>(lp) * kPS));
      if (s < 0 || s + kPS > p.pool_tokens) {
        set_status(p.status, B200KV_DEV_BAD_PAGE);
        s = -1;
      }
      base[i] = s;
    }
  }
}

// Issue the cp.async copies of one tile (K then V) for KV head `head` into a stage.
__device__ __forceinline__ void issue_tile(const DecodeParams& p, int head, int ntok,
                                           const int64_t (&base)[kTilePages], uint32_t stage_smem,
                                           uint64_t policy) {
  const int tid = threadIdx.x;
  const int c = tid & 15;        // 16-byte chunk inside the 256-byte row
  const int r0 = tid >> 4;       // rows r0, r0+8, ..., r0+56
  const __half* kh = p.k_base + static_cast<int64_t>(head) * p.kv_head_stride + c * 8;
  const __half* vh = p.v_base + static_cast<int64_t>(head) * p.kv_head_stride + c * 8;
#pragma unroll
  for (int j = 0; j < kTileTok / 8; ++j) {
    const int r = r0 + 8 * j;
    const int64_t pb = base[j >> 1];  // page of row r is r / 16 == j / 2
    const bool ok = (r < ntok) && (pb >= 0);
    const int64_t off = ok ? (pb + (r & (kPS - 1))) * p.kv_tok_stride : 0;
    const uint32_t dst = stage_smem + r * kRowBytes + ((c ^ (r & 7)) << 4);
    cp_async_16_hint(dst, kh + off, ok ? 16 : 0, policy);
    cp_async_16_hint(dst + kTileBytes, vh + off, ok ? 16 : 0, policy);
  }
}

template <int ROWS, int STAGES>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) paged_decode_split_kernel(DecodeParams p) {
  static_assert(ROWS == 8 || ROWS == 16, "query-group rows are padded to 8 or 16");
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* stages = smem;
  float* merge_o = reinterpret_cast<float*>(smem + STAGES * kStageBytes);  // [4][ROWS][128]
  float* merge_ml = merge_o + kWarps * ROWS * kD;                          // [4][ROWS][2]
  int* scan = reinterpret_cast<int*>(merge_o);  // start-up only: [kThreads + 1] page prefix

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int team = blockIdx.x / p.kv_heads;
  const int head = blockIdx.x - team * p.kv_heads;

  // ---- where does this team's page range start? -------------------------------------------
  // Thread t sums the pages of sequences [t*per, (t+1)*per); an exclusive scan over the 128
  // sums gives NP and the chunk holding the range start, then a short linear walk finds it.
  const int per = (p.batch + kThreads - 1) / kThreads;
  {
    int s = 0;
    const int lo = tid * per;
    const int hi = min(p.batch, lo + per);
    for (int b = lo; b < hi; ++b) s += pages_of(seq_len_checked(p, b));
    scan[tid + 1] = s;
    if (tid == 0) scan[0] = 0;
  }
  __syncthreads();
  if (warp == 0) {  // inclusive scan of scan[1..128] by one warp, 4 values per lane
    int v[4];
    int run = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      run += scan[1 + lane * 4 + i];
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
    for (int i = 0; i < 4; ++i) scan[1 + lane * 4 + i] = v[i] + excl;
  }
  __syncthreads();
  const int64_t np_total = scan[kThreads];
  const int nteams_eff = effective_teams(p.nteams, np_total);
  if (np_total == 0 || team >= nteams_eff) return;
  const int64_t r_begin = team_begin(team, nteams_eff, np_total);
  const int64_t r_end = team_begin(team + 1, nteams_eff, np_total);

  int start_b, start_page;
  {
    // last chunk whose prefix <= r_begin
    int lo = 0, hi = kThreads - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (scan[mid] <= r_begin) lo = mid; else hi = mid - 1;
    }
    int64_t acc = scan[lo];
    int b = lo * per;
    for (;;) {
      const int np = pages_of(seq_len_checked(p, b));
      if (acc + np > r_begin) break;
      acc += np;
      ++b;
    }
    start_b = b;
    start_page = static_cast<int>(r_begin - acc);
  }
  __syncthreads();  // the scan scratch aliases the merge buffer

  const uint64_t policy = l2_evict_first_policy();
  const uint32_t stage_base = smem_u32(stages);

  Walker prod, cons;
  prod.flat = cons.flat = r_begin;
  prod.flat_end = cons.flat_end = r_end;
  prod.enter(p, start_b, start_page);
  cons.enter(p, start_b, start_page);

  // ---- prologue: STAGES-1 tiles in flight, plus the page ids of the next one -----------------
  Tile pend;
  int64_t pend_base[kTilePages];
  bool pend_valid = prod.next(p, pend);
  load_page_bases(p, pend, pend_valid, pend_base);
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (pend_valid) issue_tile(p, head, pend.ntok, pend_base, stage_base + s * kStageBytes, policy);
    cp_async_commit();
    pend_valid = prod.next(p, pend);
    load_page_bases(p, pend, pend_valid, pend_base);
  }

  // ---- per-piece state -------------------------------------------------------------------------
  uint32_t qf[8][4];   // Q as mma A fragments: 8 k-steps of 16 along head_dim
  float o[16][4];      // O accumulator: 16 n-blocks of 8 along head_dim
  float m_run[2], l_run[2];
  const int qrow0 = lane >> 2;
  const int qcol = (lane & 3) * 2;

  Tile t;
  int it = 0;
  while (cons.next(p, t)) {
    if (t.first) {
#pragma unroll
      for (int nb = 0; nb < 16; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f;
      m_run[0] = m_run[1] = -INFINITY;
      l_run[0] = l_run[1] = 0.f;
      const __half* qb = p.q + static_cast<int64_t>(t.b) * p.q_stride_b +
                         static_cast<int64_t>(head) * p.group * p.q_stride_h;
      const bool r0ok = qrow0 < p.group;
      const bool r1ok = (ROWS == 16) && (qrow0 + 8 < p.group);
      const __half* q0 = qb + static_cast<int64_t>(qrow0) * p.q_stride_h + qcol;
      const __half* q1 = qb + static_cast<int64_t>(qrow0 + 8) * p.q_stride_h + qcol;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        qf[ks][0] = r0ok ? __ldg(reinterpret_cast<const uint32_t*>(q0 + ks * 16)) : 0u;
        qf[ks][2] = r0ok ? __ldg(reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8)) : 0u;
        qf[ks][1] = r1ok ? __ldg(reinterpret_cast<const uint32_t*>(q1 + ks * 16)) : 0u;
        qf[ks][3] = r1ok ? __ldg(reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8)) : 0u;
      }
    }

    cp_async_wait<STAGES - 2>();
    __syncthreads();
    {  // refill the stage freed by the previous iteration
      const int ps = (it + STAGES - 1) % STAGES;
      if (pend_valid) issue_tile(p, head, pend.ntok, pend_base, stage_base + ps * kStageBytes, policy);
      cp_async_commit();
      pend_valid = prod.next(p, pend);
      load_page_bases(p, pend, pend_valid, pend_base);
    }

    const int wtok0 = warp * 16;
    if (wtok0 < t.ntok) {
      const uint32_t ks_smem = stage_base + (it % STAGES) * kStageBytes;
      const uint32_t vs_smem = ks_smem + kTileBytes;
      // ---- S = Q K^T over this warp's 16 tokens -----------------------------------------------
      float s[2][4];
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
      {
        const int ktok = wtok0 + ((lane >> 4) << 3) + (lane & 7);
        const uint32_t krow = ks_smem + ktok * kRowBytes;
        const int kx = ktok & 7;
        const int csel = (lane >> 3) & 1;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          uint32_t kb[4];
          ldmatrix_x4(kb, krow + (((2 * ks + csel) ^ kx) << 4));
          mma_16816(s[0], qf[ks], kb[0], kb[1]);
          mma_16816(s[1], qf[ks], kb[2], kb[3]);
        }
      }
      // ---- online softmax (log2 domain) -----------------------------------------------------
      // With 8 padded rows the accumulator halves e = 2,3 (rows 8..15) carry no query head.
      constexpr int kE = (ROWS == 8) ? 2 : 4;
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        const int col = wtok0 + nb * 8 + qcol;
#pragma unroll
        for (int e = 0; e < kE; ++e) {
          const bool ok = (col + (e & 1)) < t.ntok;
          s[nb][e] = ok ? s[nb][e] * p.scale_log2 : -INFINITY;
          mx[e >> 1] = fmaxf(mx[e >> 1], s[nb][e]);
        }
      }
      float alpha[2] = {1.f, 1.f}, msub[2] = {0.f, 0.f};
#pragma unroll
      for (int r = 0; r < kE / 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_run[r], mx[r]);
        msub[r] = (m_new == -INFINITY) ? 0.f : m_new;
        alpha[r] = fast_exp2(m_run[r] - msub[r]);
        m_run[r] = m_new;
      }
      uint32_t pf[4];
      {
        float pr[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        float rs[2] = {0.f, 0.f};
#pragma unroll
        for (int nb = 0; nb < 2; ++nb)
#pragma unroll
          for (int e = 0; e < kE; ++e) {
            pr[nb][e] = fast_exp2(s[nb][e] - msub[e >> 1]);
            rs[e >> 1] += pr[nb][e];
          }
        l_run[0] = l_run[0] * alpha[0] + rs[0];
        l_run[1] = l_run[1] * alpha[1] + rs[1];
        pf[0] = pack_half2(pr[0][0], pr[0][1]);
        pf[1] = pack_half2(pr[0][2], pr[0][3]);
        pf[2] = pack_half2(pr[1][0], pr[1][1]);
        pf[3] = pack_half2(pr[1][2], pr[1][3]);
      }
      // ---- O = alpha * O + P V ----------------------------------------------------------------
      {
        const int vtok = wtok0 + (((lane >> 3) & 1) << 3) + (lane & 7);
        const uint32_t vrow = vs_smem + vtok * kRowBytes;
        const int vx = vtok & 7;
        const int csel = lane >> 4;
#pragma unroll
        for (int jp = 0; jp < 8; ++jp) {
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, vrow + (((2 * jp + csel) ^ vx) << 4));
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float(&acc)[4] = o[2 * jp + h];
            acc[0] *= alpha[0];
            acc[1] *= alpha[0];
            acc[2] *= alpha[1];
            acc[3] *= alpha[1];
            mma_16816(acc, pf, vb[2 * h], vb[2 * h + 1]);
          }
        }
      }
    }

    if (t.last) {
      // ---- merge the four warps' (m, l, O) and emit the piece --------------------------------
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
      }
      float* mo = merge_o + warp * ROWS * kD;
#pragma unroll
      for (int nb = 0; nb < 16; ++nb) {
        const int col = nb * 8 + qcol;
        *reinterpret_cast<float2*>(mo + qrow0 * kD + col) = make_float2(o[nb][0], o[nb][1]);
        if (ROWS == 16)
          *reinterpret_cast<float2*>(mo + (qrow0 + 8) * kD + col) = make_float2(o[nb][2], o[nb][3]);
      }
      if ((lane & 3) == 0) {
        float* ml = merge_ml + warp * ROWS * 2;
        ml[qrow0 * 2 + 0] = m_run[0];
        ml[qrow0 * 2 + 1] = l_run[0];
        if (ROWS == 16) {
          ml[(qrow0 + 8) * 2 + 0] = m_run[1];
          ml[(qrow0 + 8) * 2 + 1] = l_run[1];
        }
      }
      __syncthreads();
      const int64_t slot = (static_cast<int64_t>(team) + t.b) * p.kv_heads + head;
      for (int r = 0; r < p.group; ++r) {
        float mw[kWarps], M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
          mw[w] = merge_ml[(w * ROWS + r) * 2];
          M = fmaxf(M, mw[w]);
        }
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
          const float sc = (mw[w] == -INFINITY) ? 0.f : fast_exp2(mw[w] - M);
          L += sc * merge_ml[(w * ROWS + r) * 2 + 1];
          acc += sc * merge_o[(w * ROWS + r) * kD + tid];
        }
        const float val = acc / L;
        if (t.whole) {
          p.out[static_cast<int64_t>(t.b) * p.out_stride_b +
                (static_cast<int64_t>(head) * p.group + r) * p.out_stride_h + tid] = __float2half_rn(val);
        } else {
          p.part_o[(slot * ROWS + r) * kD + tid] = val;
          if (tid == 0) p.part_lse[slot * ROWS + r] = M + log2f(L);
        }
      }
      // the next write to the merge buffer is at least one __syncthreads away (loop top)
    }
    ++it;
  }
  cp_async_wait<0>();
}

// Merge the split partials of each sequence: out = sum_p 2^(lse_p - M) o_p / sum_p 2^(lse_p - M)
// (stage 2 of the reference, lite_llama/kernels/flashdecoding.py:199-267).  One CTA per
// sequence, one warp per query head at a time; lanes hold the pieces' log-sum-exp values and
// reduce them with warp shuffles, then every lane accumulates four output columns.
template <int ROWS>
__global__ void __launch_bounds__(kCombineThreads) decode_combine_kernel(DecodeParams p) {
  __shared__ long long red[2][kCombineThreads / 32];
  const int b = blockIdx.x;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;

  long long before = 0, total = 0;
  for (int i = tid; i < p.batch; i += kCombineThreads) {
    const int np = pages_of(seq_len_checked(p, i));
    total += np;
    if (i < b) before += np;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    before += __shfl_xor_sync(0xffffffffu, before, d);
    total += __shfl_xor_sync(0xffffffffu, total, d);
  }
  if (lane == 0) {
    red[0][warp] = before;
    red[1][warp] = total;
  }
  __syncthreads();
  before = total = 0;
#pragma unroll
  for (int w = 0; w < kCombineThreads / 32; ++w) {
    before += red[0][w];
    total += red[1][w];
  }

  const int len = seq_len_checked(p, b);
  if (len == 0) {  // no keys: the output row is defined as zero
    for (int i = tid; i < p.q_heads * kD; i += kCombineThreads) {
      const int h = i / kD;
      p.out[static_cast<int64_t>(b) * p.out_stride_b + static_cast<int64_t>(h) * p.out_stride_h +
            (i - h * kD)] = __float2half_rn(0.f);
    }
    return;
  }
  const int np = pages_of(len);
  const int nteams_eff = effective_teams(p.nteams, total);
  const int t_first = team_of(before, nteams_eff, total);
  const int t_last = team_of(before + np - 1, nteams_eff, total);
  const int npieces = t_last - t_first + 1;
  if (npieces == 1) return;  // the split kernel already wrote the final row

  for (int hq = warp; hq < p.q_heads; hq += kCombineThreads / 32) {
    const int kvh = hq / p.group;
    const int g = hq - kvh * p.group;
    float M = -INFINITY;
    for (int p0 = 0; p0 < npieces; p0 += 32) {
      const int pc = p0 + lane;
      if (pc < npieces) {
        const int64_t slot = (static_cast<int64_t>(t_first + pc) + b) * p.kv_heads + kvh;
        M = fmaxf(M, p.part_lse[slot * ROWS + g]);
      }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, d));
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float wsum = 0.f;
    for (int p0 = 0; p0 < npieces; p0 += 32) {
      const int pc = p0 + lane;
      float w = 0.f;
      if (pc < npieces) {
        const int64_t slot = (static_cast<int64_t>(t_first + pc) + b) * p.kv_heads + kvh;
        w = fast_exp2(p.part_lse[slot * ROWS + g] - M);
      }
      wsum += w;
      const int cnt = min(32, npieces - p0);
      for (int j = 0; j < cnt; ++j) {
        const float wj = __shfl_sync(0xffffffffu, w, j);
        const int64_t slot = (static_cast<int64_t>(t_first + p0 + j) + b) * p.kv_heads + kvh;
        const float4 ov =
            *reinterpret_cast<const float4*>(p.part_o + (slot * ROWS + g) * kD + lane * 4);
        acc.x += wj * ov.x;
        acc.y += wj * ov.y;
        acc.z += wj * ov.z;
        acc.w += wj * ov.w;
      }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, d);
    const float inv = 1.f / wsum;
    __half2 h01 = __floats2half2_rn(acc.x * inv, acc.y * inv);
    __half2 h23 = __floats2half2_rn(acc.z * inv, acc.w * inv);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&h01);
    pk.y = *reinterpret_cast<uint32_t*>(&h23);
    *reinterpret_cast<uint2*>(p.out + static_cast<int64_t>(b) * p.out_stride_b +
                              static_cast<int64_t>(hq) * p.out_stride_h + lane * 4) = pk;
  }
}

inline int rows_for_group(int group) { return group <= 8 ? 8 : 16; }
inline int max_teams(int sms, int kv_heads) {
  const int t = (sms * kCtasPerSm) / kv_heads;
  return t < 1 ? 1 : t;
}
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

template <int ROWS, int STAGES>
int launch_decode(const DecodeParams& p, cudaStream_t stream) {
  constexpr int smem = STAGES * kStageBytes + kWarps * ROWS * kD * 4 + kWarps * ROWS * 2 * 4;
  static bool attr_done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return record_cuda_error(cudaGetLastError());
  if (dev < 0 || dev >= 64 || !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(paged_decode_split_kernel<ROWS, STAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev >= 0 && dev < 64) attr_done[dev] = true;
  }
  paged_decode_split_kernel<ROWS, STAGES>
      <<<static_cast<unsigned>(p.nteams * p.kv_heads), kThreads, smem, stream>>>(p);
  int rc = check_launch();
  if (rc != B200KV_OK) return rc;
  decode_combine_kernel<ROWS><<<static_cast<unsigned>(p.batch), kCombineThreads, 0, stream>>>(p);
  return check_launch();
}

}  // namespace

size_t decode_workspace_bytes(int batch, int q_heads, int kv_heads, int head_dim) {
  if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim != kD) return 0;
  if (q_heads % kv_heads != 0 || q_heads / kv_heads > 16) return 0;
  const int sms = device_sm_count();
  if (sms <= 0) return 0;
  const int rows = rows_for_group(q_heads / kv_heads);
  const size_t nslots = static_cast<size_t>(max_teams(sms, kv_heads)) + static_cast<size_t>(batch);
  const size_t po = align_up(nslots * kv_heads * rows * kD * sizeof(float), 256);
  const size_t pl = align_up(nslots * kv_heads * rows * sizeof(float), 256);
  return po + pl;
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
  if (a.max_seq_len > (int64_t{1} << 30)) return B200KV_ETOOLARGE;
  auto mis = [](const void* ptr, uintptr_t al) { return (reinterpret_cast<uintptr_t>(ptr) & (al - 1)) != 0; };
  if (mis(a.k_base, 16) || mis(a.v_base, 16) || mis(a.q, 4) || mis(a.out, 8) || mis(a.workspace, 16))
    return B200KV_EALIGN;
  if (a.kv_tok_stride % 8 != 0 || a.kv_head_stride % 8 != 0) return B200KV_EALIGN;
  if (a.q_stride_b % 2 != 0 || a.q_stride_h % 2 != 0) return B200KV_EALIGN;
  if (a.out_stride_b % 4 != 0 || a.out_stride_h % 4 != 0) return B200KV_EALIGN;
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
  if (teams < 1) teams = 1;

  DecodeParams p{};
  p.q = static_cast<const __half*>(a.q);
  p.q_stride_b = a.q_stride_b;
  p.q_stride_h = a.q_stride_h;
  p.k_base = static_cast<const __half*>(a.k_base);
  p.v_base = static_cast<const __half*>(a.v_base);
  p.kv_tok_stride = a.kv_tok_stride;
  p.kv_head_stride = a.kv_head_stride;
  p.pool_tokens = a.pool_tokens;
  p.table = a.table;
  p.table_row_stride = a.table_row_stride;
  p.table_kind = a.table_kind;
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
  const size_t nslots = static_cast<size_t>(teams_cap) + static_cast<size_t>(a.batch);
  p.part_o = static_cast<float*>(a.workspace);
  p.part_lse = reinterpret_cast<float*>(static_cast<uint8_t*>(a.workspace) +
                                        align_up(nslots * a.kv_heads * rows * kD * sizeof(float), 256));
  p.out = static_cast<__half*>(a.out);
  p.out_stride_b = a.out_stride_b;
  p.out_stride_h = a.out_stride_h;
  p.status = a.status;

  if (rows == 8) return launch_decode<8, 3>(p, stream);
  return launch_decode<16, 2>(p, stream);
}

}  // namespace b200kv
