// FBLA compressed-KV decode for sm_100a: coarse pass (+ the BF16 windows), select, refine, merge.
//
// Semantics follow the reference's decode (attention/fbla/src/fbla_kernels.cuh:315-359 qhat, :479-533 coarse blocks,
// :866-920 select, :1036-1072 refine, :1270-1294 merge): per (query, group) int8 qhat, 16-token P blocks of integers
// p = round(255 * 2^(s - max)), coarse cells decoded at their midpoint, blocks with 2^(lse_j - R) > tau corrected by
// (full - coarse). The structure is new:
//   * a persistent grid, one CTA per SM; every warp owns a contiguous range of the flattened list of closed
//     (virtual head, group) units and a private 2-stage ring in shared memory that whole groups (8 records + 1 KiB
//     metadata) are streamed into by 1-D bulk asynchronous copies completing on mbarriers (all waits bounded);
//   * scores and values are integer tensor-core products taken straight from the packed records (fbla_frag.cuh):
//     tokens on M for S^T = K_codes qhat^T, channels on M for O^T = V_codes^T P^T, both P blocks of a record pair
//     in the 8 columns of one product; the instruction count per byte no longer grows with the GQA ratio;
//   * one extra warp per CTA serves the BF16 sink / open windows with plain loads and FP32 FMAs.
// Reduction orders are fixed by (warp, unit) ranges alone, so outputs are bit-reproducible run to run.
#pragma once
#include "fbla_frag.cuh"
#include "fbla_kernels.h"

namespace fbla {

constexpr int PSTRIDE = FBLA_K_PSTRIDE;  // floats of one partial row: o[128], m, l, 2 pad (coarse); o[128], dl, 3 pad (refine)
constexpr int SLICE = FBLA_K_SLICE;      // sub-blocks per select slice

// Streaming warps per CTA and ring slots per warp, per coarse bit width. A slot holds one record pair (32 tokens);
// the group's metadata has two slots of its own. NP <= 4 (one group of lookahead) keeps two metadata slots enough.
#ifndef FBLA_RW
#define FBLA_RW 12   /* refine warps per CTA */
#endif
#ifndef FBLA_RNST
#define FBLA_RNST 2  /* refine ring stages per warp */
#endif
// Eight warps per CTA leave a thread 255 registers, which the coarse loop needs to run without spills. Measured on B200
// with streaming + window warps (decode batch 8 x 16K 4+2 / batch 1 x 128K 3+3 / 4+2, us per step):
// 10 + 2 warps (168 registers) 135.5 / 80.3 / 78.1; 8 + 2: 121.3 / 81.0 / 65.2; 7 + 1: 121.7 / 76.3 / 63.5; 6 + 2: 131.6 / 84.3 / 68.6.
// FBLA_CW*: the streaming warps of that fixed split; a CTA has one warp more (CoarseShape::TOTAL).
#ifndef FBLA_CW4
#define FBLA_CW4 7
#endif
#ifndef FBLA_CW3
#define FBLA_CW3 7
#endif
#ifndef FBLA_NP
#define FBLA_NP 2
#endif
#ifndef FBLA_PPC
#define FBLA_PPC 2  // record pairs per chunk (one bulk copy, one barrier wait)
#endif
template <int CB> struct CoarseShape {
  static constexpr int WARPS = CB == 4 ? FBLA_CW4 : FBLA_CW3, TOTAL = WARPS + 1;
  static constexpr int NP = FBLA_NP;
  static constexpr int PPC = FBLA_PPC, CPG = 4 / FBLA_PPC;  // pairs per chunk, chunks per group
  static constexpr int PAIR_BYTES = 2 * record_bytes(CB), CHUNK_BYTES = FBLA_PPC * PAIR_BYTES;
  static constexpr int GROUP_BYTES = SBG * record_bytes(CB);
};
static_assert(FBLA_RNST == 2, "the refine pass keeps the metadata of two groups");
static_assert(FBLA_NP >= 2 && FBLA_NP * FBLA_PPC <= 4 && 4 % FBLA_PPC == 0, "ring slots per warp: at most one group of lookahead");

// ---- where a batch row's tokens put its units -----------------------------------------------------------------------
struct Row { int tokens, groups, g0, closed, na, exact; };  // g0: the first closed group processed; na: sink sub-blocks
__device__ __forceinline__ Row row_of(const fbla_k_decode &a, int b) {
  Row r;
  r.tokens = (a.length ? FBLA_POS::ro(a.length + (a.lstride ? b : 0)) : 0) + a.tokens;
  r.groups = (r.tokens + G - 1) / G;
  int first = 1, last = r.groups - 1, win = 3;  // closed groups [first, last); the whole cache: 1 .. groups - 2
  if (a.shard_on) { first = a.sh_first; last = min(last, a.sh_first + a.sh_count); win = a.sh_windows; }
  r.g0 = first;
  r.closed = max(last - first, 0);
  r.na = !(win & 1) ? 0 : r.groups == 1 ? (r.tokens + S - 1) / S : (r.groups >= 2 ? SBG : 0);
  // the open window: the last group's tokens; a cache of one group is read through its sink window unless only the open one is asked for
  const int no = !(win & 2) ? 0 : r.groups >= 2 ? (r.tokens - G * (r.groups - 1) + S - 1) / S : (win & 1) ? 0 : (r.tokens + S - 1) / S;
  r.exact = r.na + no;  // BF16 sub-blocks: the sink's, then the open group's
  return r;
}
// Flattened unit lists. Closed groups: row b contributes hpr * closed(b) units, head-major. BF16 sub-blocks likewise.
// A cursor walks one list; every warp builds its own from the row lengths (no shared state, no limit on the batch).
struct Cursor {
  int b, hir, i, n;  // batch row, virtual head within the row, index within the head's n units
};
// the group of closed-group cursor c
__device__ __forceinline__ int group_of(const fbla_k_decode &a, const Cursor &c) { return row_of(a, c.b).g0 + c.i; }
template <bool EXACT>
__device__ __forceinline__ int units_of(const Row &r) { return EXACT ? r.exact : r.closed; }

// (one length for every batch row: closed forms, no loop over the batch)
template <bool EXACT>
__device__ __forceinline__ long long total_units(const fbla_k_decode &a, int hpr) {
  if (!a.lstride) return (long long)a.batch * hpr * units_of<EXACT>(row_of(a, 0));
  long long t = 0;
  for (int b = 0; b < a.batch; ++b) t += (long long)hpr * units_of<EXACT>(row_of(a, b));
  return t;
}
// the cursor of flattened unit u (u < total)
template <bool EXACT>
__device__ __forceinline__ Cursor locate(const fbla_k_decode &a, int hpr, long long u) {
  Cursor c{0, 0, 0, 0};
  if (!a.lstride) {
    const int n = units_of<EXACT>(row_of(a, 0)), h = (int)(u / n);
    c.b = h / hpr; c.hir = h - c.b * hpr; c.i = (int)(u - (long long)h * n); c.n = n;
    return c;
  }
  for (int b = 0; b < a.batch; ++b) {
    const int n = units_of<EXACT>(row_of(a, b));
    const long long span = (long long)hpr * n;
    if (u < span) { c.b = b; c.hir = (int)(u / n); c.i = (int)(u % n); c.n = n; return c; }
    u -= span;
  }
  c.b = a.batch;
  return c;
}
template <bool EXACT>
__device__ __forceinline__ void advance(const fbla_k_decode &a, int hpr, Cursor &c) {
  if (++c.i < c.n) return;
  c.i = 0;
  if (++c.hir < hpr) return;
  c.hir = 0;
  for (++c.b; c.b < a.batch; ++c.b) {
    c.n = units_of<EXACT>(row_of(a, c.b));
    if (c.n) return;
  }
}
// first flattened unit of virtual head vh, and the head's unit count
template <bool EXACT>
__device__ __forceinline__ long long head_offset(const fbla_k_decode &a, int hpr, int vh, int &n) {
  if (!a.lstride) { n = units_of<EXACT>(row_of(a, 0)); return (long long)vh * n; }
  const int bq = vh / hpr, hir = vh - bq * hpr;
  long long off = 0;
  for (int b = 0; b < bq; ++b) off += (long long)hpr * units_of<EXACT>(row_of(a, b));
  n = units_of<EXACT>(row_of(a, bq));
  return off + (long long)hir * n;
}
__device__ __forceinline__ long long ceil_div(long long a, long long b) { return (a + b - 1) / b; }

// q row (batch b, virtual head hir = kh * vg + j, query qi) in q / out
__device__ __forceinline__ int q_row(const fbla_k_decode &a, int b, int hir, int qi) {
  const int kh = hir / a.vg, j = hir - kh * a.vg;
  return b * a.q_heads + kh * (a.q_heads / a.kv_heads) + j * a.qg + qi;
}

// ---- per-group query quantization (the definition of include/mlops_fbla.h) --------------------------------------------
// Lane l holds channels 4 l .. 4 l + 3: km = the lane's 16 metadata bytes of K (4 bases, 4 steps), q4 = its 4 q values.
// Returns the lane's qhat word (quantize_query also writes it to qst_row[l]) and, through the references, the
// warp-uniform sq, qb (= sl q . base), qsum (= sum qhat).
__device__ __forceinline__ uint32_t quantize_query_word(uint4 km, float4 q4, float sl, float &sq, float &qb, float &qsum) {
  const float kb[4] = {bf_lo(km.x), bf_hi(km.x), bf_lo(km.y), bf_hi(km.y)}, ks[4] = {bf_lo(km.z), bf_hi(km.z), bf_lo(km.w), bf_hi(km.w)};
  const float qf[4] = {q4.x, q4.y, q4.z, q4.w};
  float z[4], amax = 0.f, dot = 0.f;
#pragma unroll
  for (int x = 0; x < 4; ++x) { z[x] = __fmul_rn(qf[x], ks[x]); amax = fmaxf(amax, fabsf(z[x])); dot = fmaf(qf[x], kb[x], dot); }
  amax = __uint_as_float(__reduce_max_sync(FULL, __float_as_uint(amax)));  // amax >= 0: the bit patterns order as the values
  // r = fl(127 / amax), correctly rounded: reciprocal seed, one Newton step, quotient and its residual correction
  float rc;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rc) : "f"(amax));
  rc = fmaf(fmaf(-amax, rc, 1.f), rc, rc);
  const float q0 = __fmul_rn(127.f, rc);
  const float r = amax > 0.f ? fmaf(fmaf(-amax, q0, 127.f), rc, q0) : 0.f;
  uint32_t word = 0;
#pragma unroll
  for (int x = 0; x < 4; ++x)  // rint(z r) in the low mantissa bits: one rounding of the exact product
    word |= (__float_as_uint(fmaf(z[x], r, MAGICF)) & 255u) << (8 * x);
  sq = __fmul_rn(amax, __fmul_rn(sl, 1.f / 127.f));
  qb = __fmul_rn(warp_sum(dot), sl);
  qsum = (float)__reduce_add_sync(FULL, __dp4a((int)word, 0x01010101, 0));  // the exact integer sum of the codes
  return word;
}
__device__ __forceinline__ void quantize_query(uint4 km, float4 q4, float sl, uint32_t *qst_row, int lane, float &sq, float &qb, float &qsum) {
  qst_row[lane] = quantize_query_word(km, q4, sl, sq, qb, qsum);
}

// ---- shared memory of the coarse kernel ---------------------------------------------------------------------------------
template <int CB> struct __align__(128) StreamWarp {
  uint8_t pair[CoarseShape<CB>::NP][CoarseShape<CB>::CHUNK_BYTES];  // ring of chunks (PPC record pairs each)
  uint8_t meta[2][1024];                                           // metadata of the group in progress and of the next
  uint8_t qst[8 * QST_ROW];  // qhat rows (rows >= QG stay zero)
  uint8_t pst[128];          // P bytes of a record pair: [block parity][query 0..3][16 tokens]
  uint64_t bar_pair[CoarseShape<CB>::NP], bar_meta[2];
  // The partial rows of the first and the last virtual head of the warp's run, which neighbouring warps of the CTA may
  // share: they are folded into one row per (CTA, virtual head) before they leave the CTA. stage_vh: the rows' virtual
  // heads (-1: no such row).
  float stage[2][4][FBLA_K_PSTRIDE];
  int stage_vh[2];
};
struct __align__(16) ExactWarp {
  uint16_t q[8][D + 8];   // the virtual head's queries in BF16 (rows >= QG: zero); rows 272 bytes apart: 16-byte aligned, conflict-free
  uint16_t v[S][D + 8];   // the sub-block's V rows
  uint16_t p[8][S];       // P as BF16 integers: [query][token]
};
// (every warp has streaming buffers; a warp that serves windows keeps its ExactWarp in the buffers it does not stream
// into yet, or at all)
template <int CB> struct CoarseSmem {
  StreamWarp<CB> w[CoarseShape<CB>::TOTAL];
};
static_assert(sizeof(CoarseSmem<3>) + 128 <= 227 * 1024 && sizeof(CoarseSmem<4>) + 128 <= 227 * 1024, "one CTA's shared memory");
static_assert(sizeof(ExactWarp) <= sizeof(StreamWarp<3>) && sizeof(ExactWarp) <= sizeof(StreamWarp<4>), "a window warp's state fits a streaming warp's");

// ---- the coarse pass's work, split over its warps --------------------------------------------------------------------------
// Streaming units are the closed groups of all virtual heads, flattened; window units the 16-token sub-blocks of the
// BF16 sink / open windows, flattened. Either way of dealing them depends on the lengths alone and leaves no empty warp
// between two that serve a head: the readers (slots_of) take every slot from the first to the last warp of a head as
// written.
// Split by the lengths (short contexts, FBLA_K_DEAL_LENGTHS): of a CTA's warps the last xw serve windows and the others stream, and
// each kind's units are dealt in equal contiguous runs over its warps of all CTAs. xw is the windows' share of all units
// by cost (a sub-block 3 eighths of a group at these lengths), at least one warp for the windows and one for the groups
// if there are any. The host asks for it when the windows are a large part of the work: short contexts
// at large batch (batch 256 x 512 tokens: 638 -> 352 us per step, batch 32 x 4096: 182 -> 166).
//
// FBLA_K_DEAL_FIXED (contexts in between): the same with xw = 1, whatever the lengths.
//
// FBLA_K_DEAL_COST (long contexts): no warp is set aside. All units form one list, window sub-blocks first, then the groups, each
// with a cost in eighths of a group's time: a window sub-block, on its BF16 tensor-core products, costs half a group
// (measured, batch 1 x 128K tokens, us per step with costs 2 / 3 / 4 / 6 / 10: 3+3 67.9 / 69.8 / 66.0 / 66.3 / -, 4+2
// 64.6 / 60.6 / 55.9 / - / 59.3; what matters most is that a share is a whole number of groups: with 57 instead of 56
// eighths one warp in eight streams 8 groups instead of 7). Every warp of the grid takes the units whose cost interval
// starts inside its equal share [w P, (w + 1) P) of the total, serves its window sub-blocks and then streams its
// groups. A share is at least one unit's cost, so consecutive units lie in the same or in consecutive warps. At batch 1
// and 128K tokens a warp then streams 7 groups instead of 8.
struct Deal { long long S, X, P; int wc; };  // groups, window sub-blocks, cost share per warp, cost of a window sub-block
constexpr int GROUP_COST = 8, WINDOW_COST = 4, WINDOW_COST_SHORT = 3;  // a warp's time for a group / a window sub-block, in eighths of a group
__device__ __forceinline__ Deal deal_of(const fbla_k_decode &a, int hpr) {
  Deal d;
  d.S = total_units<false>(a, hpr);
  d.X = total_units<true>(a, hpr);
  d.wc = WINDOW_COST;
  // (a whole number of groups per share: every streaming warp then takes the same number of groups)
  d.P = GROUP_COST * max(1ll, ceil_div(GROUP_COST * d.S + d.wc * d.X, (long long)GROUP_COST * a.coarse_ctas * a.coarse_warps));
  return d;
}
// the units of warp w: window sub-blocks [xlo, xhi), groups [lo, hi)
__device__ __forceinline__ void deal_range(const Deal &d, long long w, long long &xlo, long long &xhi, long long &lo, long long &hi) {
  const long long c0 = w * d.P, c1 = c0 + d.P, wx = d.wc * d.X;
  xlo = min(d.X, ceil_div(c0, (long long)d.wc)); xhi = min(d.X, ceil_div(c1, (long long)d.wc));
  lo = c0 <= wx ? 0 : min(d.S, ceil_div(c0 - wx, (long long)GROUP_COST));
  hi = c1 <= wx ? 0 : min(d.S, ceil_div(c1 - wx, (long long)GROUP_COST));
}
struct Split { int sw, xw; };  // streaming / window warps per CTA
__device__ __forceinline__ Split split_of(const fbla_k_decode &a, int hpr) {
  const int total = (a.cb == 4 ? FBLA_CW4 : FBLA_CW3) + 1;
  if (a.deal == FBLA_K_DEAL_FIXED) return Split{total - 1, 1};
  const long long S = GROUP_COST * total_units<false>(a, hpr), W = WINDOW_COST_SHORT * total_units<true>(a, hpr);  // in eighths of a group's time
  const int xw = S == 0 ? total : max(1, min(total - 1, (int)((2 * total * W + S + W) / (2 * (S + W)))));
  return Split{total - xw, xw};
}

// Programmatic dependent launch: the next pass of a decode is launched while this one still runs (hiding its launch
// latency) and waits here until the previous pass has completed and its writes are visible.
__device__ __forceinline__ void wait_previous_pass() { if (FBLA_STREAM_LAUNCH) asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void allow_next_pass() { if (FBLA_STREAM_LAUNCH) asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void report(const fbla_k_decode &a, int pass) {
  if (a.status) { atomicCAS(a.status, 0, pass); a.status[1] = FBLA_POS::x(); }
}

// ---- the BF16 windows ---------------------------------------------------------------------------------------------------
// Unit = one 16-token sub-block of the sink (first) or the open window, on BF16 tensor-core products with FP32 sums:
//   S^T[16 tokens x 8 queries] = K[16 x 128] Q^T        (mma.sync m16n8k16, 8 steps over the channels)
//   O^T[128 channels x 8 queries] += V^T[128 x 16] P^T  (8 tiles of 16 channels; P: the same integer block, exact in BF16)
// Scores s = sl * (q . k): BF16 products are exact in FP32, so only the order of the sums differs from a chain of FMAs.
// Thread (gid, tig) of a product holds rows gid, gid + 8 and columns 2 tig, 2 tig + 1 of its result. The channels are
// taken in the order that lets a lane load 16 bytes of a K row (its 8 channels of a 32-channel round serve two steps);
// the query fragments use the same order. V^T fragments come from shared memory through ldmatrix.trans.
__device__ __forceinline__ void mma_bf16_k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(row)) : "memory");
}
// one window sub-block's rows in registers: 16 bytes of the K rows of tokens gid and gid + 8 per 32-channel round, and the
// lane's share of the 16 V rows (256 x 16 bytes over the warp)
struct WindowTile {
  uint4 ka[4], kb[4];
  uint4 v[8];
  int count;  // attended tokens of the sub-block (1 .. 16)
};
// the window sub-blocks [lo, hi) of the flattened list; the partial rows go to window slot xw + virtual head
template <int QG>
__device__ void exact_range(const fbla_k_decode &a, ExactWarp &sm, int lane, long long lo, long long hi, int xw) {
  const int hpr = a.kv_heads * a.vg;
  if (lo >= hi) return;
  const int slot0 = a.coarse_ctas * a.coarse_warps + a.batch * hpr;  // after the coarse slots
  const int gid = lane >> 2, tig = lane & 3;
  Cursor c = locate<true>(a, hpr, lo);
  int cur_vh = -1;
  float m[2], l[2], o[8][4];  // queries 2 tig + e; o[tile]: channels 16 tile + gid (.0, .1), + 8 (.2, .3) x the two queries
  auto flush = [&]() {
    float *p = a.part + (size_t)(slot0 + xw + cur_vh) * QG * PSTRIDE;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int qi = 2 * tig + e;
      if (qi < QG) {
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
          p[qi * PSTRIDE + 16 * mt + gid] = o[mt][e];
          p[qi * PSTRIDE + 16 * mt + gid + 8] = o[mt][2 + e];
        }
        if (gid == 0) { p[qi * PSTRIDE + D] = m[e]; p[qi * PSTRIDE + D + 1] = l[e]; }
      }
    }
  };
  // all loads of a sub-block at once (the next sub-block's are issued before the current one is computed)
  auto load = [&](const Cursor &cu, WindowTile &w) {
    const Row r = row_of(a, cu.b);
    const bool sink = cu.i < r.na;
    const int j = sink ? cu.i : cu.i - r.na;  // sub-block within its window
    const int window = sink ? (r.groups == 1 ? r.tokens : G) : r.tokens - G * (r.groups - 1);
    w.count = min(window - j * S, S);
    const size_t eh = (size_t)((cu.b * hpr + cu.hir) / a.vg) * G * D;
    const uint16_t *ek = (sink ? a.c.sink_k : a.c.open_k) + eh + (size_t)j * S * D, *ev = (sink ? a.c.sink_v : a.c.open_v) + eh + (size_t)j * S * D;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int r4 = 0; r4 < 4; ++r4) {  // channels 32 r4 + 8 tig .. + 7 of tokens gid, gid + 8
      w.ka[r4] = gid < w.count ? __ldcg(reinterpret_cast<const uint4 *>(ek + (size_t)gid * D + 32 * r4 + 8 * tig)) : zero;
      w.kb[r4] = gid + 8 < w.count ? __ldcg(reinterpret_cast<const uint4 *>(ek + (size_t)(gid + 8) * D + 32 * r4 + 8 * tig)) : zero;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {  // 16-byte piece 32 i + lane of the 16 x 256 bytes: row (32 i + lane) / 16
      const int row = 2 * i + (lane >> 4);
      w.v[i] = row < w.count ? __ldcg(reinterpret_cast<const uint4 *>(ev + (size_t)row * D) + (lane & 15)) : zero;
    }
  };
  for (int i = lane; i < 8 * (D + 8) / 2; i += 32) reinterpret_cast<uint32_t *>(&sm.q[0][0])[i] = 0u;
  WindowTile cur, nxt;
  load(c, cur);
  for (long long u = lo; u < hi; ++u) {
    const int vh = c.b * hpr + c.hir;
    if (vh != cur_vh) {
      if (cur_vh >= 0) flush();
      cur_vh = vh;
      __syncwarp();
#pragma unroll
      for (int qi = 0; qi < QG; ++qi)
        *reinterpret_cast<uint2 *>(&sm.q[qi][4 * lane]) = __ldg(reinterpret_cast<const uint2 *>(a.q + (size_t)q_row(a, c.b, c.hir, qi) * D) + lane);
      m[0] = m[1] = -FBLA_INF; l[0] = l[1] = 0.f;
#pragma unroll
      for (int mt = 0; mt < 8; ++mt) o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f;
    }
    __syncwarp();  // (the queries are in place; the previous sub-block's V rows and P have been read)
#pragma unroll
    for (int i = 0; i < 8; ++i) *reinterpret_cast<uint4 *>(&sm.v[2 * i + (lane >> 4)][8 * (lane & 15)]) = cur.v[i];
    // scores
    float x[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r4 = 0; r4 < 4; ++r4) {
      const uint4 qq = *reinterpret_cast<const uint4 *>(&sm.q[gid][32 * r4 + 8 * tig]);
      mma_bf16_k16(x, cur.ka[r4].x, cur.kb[r4].x, cur.ka[r4].y, cur.kb[r4].y, qq.x, qq.y);
      mma_bf16_k16(x, cur.ka[r4].z, cur.kb[r4].z, cur.ka[r4].w, cur.kb[r4].w, qq.z, qq.w);
    }
    const int count = cur.count;
    advance<true>(a, hpr, c);
    if (u + 1 < hi) load(c, nxt);
    // x[2 r + e]: token gid + 8 r, query 2 tig + e
    float al[2], w[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const float s0 = gid < count ? __fmul_rn(x[e], a.sl) : -FBLA_INF, s1 = gid + 8 < count ? __fmul_rn(x[2 + e], a.sl) : -FBLA_INF;
      float mb = fmaxf(s0, s1);
#pragma unroll
      for (int off = 4; off <= 16; off <<= 1) mb = fmaxf(mb, __shfl_xor_sync(FULL, mb, off));
      const float mn = fmaxf(m[e], mb);
      al[e] = ex2(m[e] - mn); w[e] = ex2(mb - mn);  // (2^-inf = 0; mb is finite: token 0 of a unit always exists)
      m[e] = mn;
      // the integer p as an exact float: (p + 1.5 * 2^23) - 1.5 * 2^23; its BF16 form is its upper half
      const float p0 = fmaf(ex2(s0 - mb), 255.f, MAGICF) - MAGICF, p1 = fmaf(ex2(s1 - mb), 255.f, MAGICF) - MAGICF;
      sm.p[2 * tig + e][gid] = (uint16_t)(__float_as_uint(p0) >> 16);
      sm.p[2 * tig + e][gid + 8] = (uint16_t)(__float_as_uint(p1) >> 16);
      float sp = p0 + p1;
#pragma unroll
      for (int off = 4; off <= 16; off <<= 1) sp += __shfl_xor_sync(FULL, sp, off);
      l[e] = fmaf(al[e], l[e], w[e] * sp);
    }
    __syncwarp();
    // values: P^T fragments (tokens 2 tig, 2 tig + 1 and + 8 of query gid), V^T fragments per 16-channel tile
    const uint32_t pb0 = *reinterpret_cast<const uint32_t *>(&sm.p[gid][2 * tig]), pb1 = *reinterpret_cast<const uint32_t *>(&sm.p[gid][2 * tig + 8]);
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
      uint32_t va[4];  // matrices: (tokens 0-7, channels 16 mt ..), (0-7, + 8), (8-15, ..), (8-15, + 8)
      ldmatrix_x4_trans(va, &sm.v[8 * (lane >> 4) + (lane & 7)][16 * mt + 8 * ((lane >> 3) & 1)]);
      float y[4] = {0.f, 0.f, 0.f, 0.f};
      mma_bf16_k16(y, va[0], va[1], va[2], va[3], pb0, pb1);
      o[mt][0] = fmaf(al[0], o[mt][0], w[0] * y[0]); o[mt][1] = fmaf(al[1], o[mt][1], w[1] * y[1]);
      o[mt][2] = fmaf(al[0], o[mt][2], w[0] * y[2]); o[mt][3] = fmaf(al[1], o[mt][3], w[1] * y[3]);
    }
    cur = nxt;
  }
  flush();
}
// window warp xw of nxw: an equal contiguous run of the sub-blocks
template <int QG>
__device__ __forceinline__ void exact_warp(const fbla_k_decode &a, ExactWarp &sm, int lane, int xw, int nxw) {
  const long long total = total_units<true>(a, a.kv_heads * a.vg), per = ceil_div(total, nxw), lo = (long long)xw * per;
  exact_range<QG>(a, sm, lane, lo, min(total, lo + per), xw);
}

// ---- one closed group on the tensor cores ----------------------------------------------------------------------------------
// The warp's running softmax of its current virtual head. Thread (gid, tig): channels 4 (8 u + gid) + cc, u, cc = 0..3,
// of queries qe = 2 (tig & 1) + e, e = 0, 1, summed over the sub-blocks of parity tig >> 1 only: the two parities'
// threads are added when the partial is written.
struct Run {
  float m[2], l[2];
  float2 o[4][4];  // (.x, .y) = queries e = 0, 1
};
template <int QG> __device__ __forceinline__ bool query_valid(int tig, int e) { return 2 * (tig & 1) + e < QG; }

// The warp's stream of record pairs: chunk p = CPG k + i holds pairs PPC i .. of the k-th group of the warp's range, in ring
// slot p % NP (its (p / NP)-th use); the group's metadata travels with chunk 0 into metadata slot k & 1. All lanes carry the
// (warp-uniform) state; lane 0 issues the copies.
template <int CB> struct Ring {
  using Sh = CoarseShape<CB>;
  StreamWarp<CB> &w;
  const fbla_k_decode &a;
  int hpr, lane;
  Cursor fc;                           // the group of the next chunk to issue
  int issued, chunks;                  // chunks issued / in the warp's range
  const uint8_t *src_pair, *src_meta;  // that group's records and metadata
  __device__ __forceinline__ void point() {
    const int bh = (fc.b * hpr + fc.hir) / a.vg;
    const size_t unit = (size_t)bh * a.hs + (size_t)group_of(a, fc) * a.gs;
    src_pair = a.c.coarse + unit * Sh::GROUP_BYTES;
    src_meta = reinterpret_cast<const uint8_t *>(a.c.meta) + unit * 1024;
  }
  __device__ __forceinline__ void issue_next() {
    if (issued >= chunks) return;
    const int i = issued % Sh::CPG, slot = issued % Sh::NP, ms = (issued / Sh::CPG) & 1;
    if (lane == 0) {  // (the slot's earlier reads have completed: their values were consumed before the __syncwarp above)
      if (i == 0) {
        mbar_expect_tx(&w.bar_meta[ms], 1024);
        bulk_g2s(w.meta[ms], src_meta, 1024, &w.bar_meta[ms]);
      }
      mbar_expect_tx(&w.bar_pair[slot], Sh::CHUNK_BYTES);
      bulk_g2s(w.pair[slot], src_pair + i * Sh::CHUNK_BYTES, Sh::CHUNK_BYTES, &w.bar_pair[slot]);
    }
    ++issued;
    if (i == Sh::CPG - 1 && issued < chunks) { advance<false>(a, hpr, fc); point(); }
  }
  // false: a bounded wait gave up
  __device__ __forceinline__ bool wait_meta(int k) { return __all_sync(FULL, mbar_wait_bounded(&w.bar_meta[k & 1], (uint32_t)((k >> 1) & 1))); }
  __device__ __forceinline__ bool wait_pair(int p) { return __all_sync(FULL, mbar_wait_bounded(&w.bar_pair[p % Sh::NP], (uint32_t)((p / Sh::NP) & 1))); }
};

// Group k of the warp's range. Returns false if a bounded wait gave up.
template <int CB, int FB, int QG>
__device__ __forceinline__ bool coarse_group(Ring<CB> &ring, int k, const float4 (&q4)[QG], float sl, int lane, Run &run,
                                             float *lse_group /* [8 sub-blocks][QG] of this (virtual head, group) */) {
  constexpr int RB = record_bytes(CB);
  constexpr float HOFF = .5f * ((1 << FB) - 1);
  StreamWarp<CB> &sm = ring.w;
  const int gid = lane >> 2, tig = lane & 3;
  const bool odd = tig >> 1;  // threads tig >= 2 accumulate the odd sub-block of every pair (columns 4..7 of the value products)
  if (!ring.wait_meta(k)) return false;
  const uint8_t *meta = sm.meta[k & 1];
  // qhat of every query; c0 / sqc of the thread's two score columns
  float c0[2] = {0.f, 0.f}, sqc[2] = {0.f, 0.f};
  {
    const uint4 km = lds128(meta + 16 * lane);
#pragma unroll
    for (int qi = 0; qi < QG; ++qi) {
      float sq, qb, qsum;
      quantize_query(km, q4[qi], sl, reinterpret_cast<uint32_t *>(sm.qst + QST_ROW * qi), lane, sq, qb, qsum);
      const float c = fmaf(__fmul_rn(sq, HOFF), qsum, qb), s2 = __fmul_rn(sq, (float)(1 << FB));
      if (qi == 2 * (tig & 1)) { c0[0] = c; sqc[0] = s2; }
      if (qi == 2 * (tig & 1) + 1) { c0[1] = c; sqc[1] = s2; }
    }
  }
  __syncwarp();
  uint32_t B[8];
  qhat_frag<CB>(sm.qst, gid, tig, B);
  // the group's sums in code units, relative to the running maximum run.m: A = sum w y, Bs = sum w sum p
  float2 A[4][4], Bs = make_float2(0.f, 0.f);
#pragma unroll
  for (int u = 0; u < 4; ++u)
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) A[u][cc] = make_float2(0.f, 0.f);
  const float2 sqc2 = make_float2(sqc[0], sqc[1]), c02 = make_float2(c0[0], c0[1]);
  // Software pipeline over the group's four record pairs: the scores of pair J + 1 (stage A: shared loads, score products,
  // sub-block maxima) are issued before the softmax and value products of pair J (stage B), so that each stage's
  // latencies are covered by the other's instructions.
  struct Scores { float s[2][4], mb[2][2]; };
  // stage A of pair J: scores s[par][i], i = (token gid, column 2 tig), (gid, 2 tig + 1), (gid + 8, 2 tig), (gid + 8, 2 tig + 1)
  // (only columns < QG, i.e. threads tig < 2, are queries; the others multiply zero rows of qst), and their maxima
  auto stage_a = [&](int J, Scores &sc) -> bool {
    const int p = CoarseShape<CB>::CPG * k + J / CoarseShape<CB>::PPC;  // the pair's chunk
    if (J % CoarseShape<CB>::PPC == 0 && !ring.wait_pair(p)) return false;
    const uint8_t *ra = sm.pair[p % CoarseShape<CB>::NP] + (J % CoarseShape<CB>::PPC) * CoarseShape<CB>::PAIR_BYTES, *rb = ra + RB;
#pragma unroll
    for (int par = 0; par < 2; ++par) {
      float x[4];
      qk_tile<CB>(par ? rb : ra, gid, tig, B, x);
      const float2 s01 = __ffma2_rn(sqc2, make_float2(x[0], x[1]), c02), s23 = __ffma2_rn(sqc2, make_float2(x[2], x[3]), c02);
      sc.s[par][0] = s01.x; sc.s[par][1] = s01.y; sc.s[par][2] = s23.x; sc.s[par][3] = s23.y;
    }
#pragma unroll
    for (int par = 0; par < 2; ++par)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float v = fmaxf(sc.s[par][e], sc.s[par][2 + e]);
        v = fmaxf(v, __shfl_xor_sync(FULL, v, 4));
        v = fmaxf(v, __shfl_xor_sync(FULL, v, 8));
        v = fmaxf(v, __shfl_xor_sync(FULL, v, 16));
        sc.mb[par][e] = v;
      }
    return true;
  };
  // stage B of pair J: sub-blocks 2 J (parity 0) and 2 J + 1 (parity 1)
  auto stage_b = [&](int J, const Scores &sc) {
    const int p = CoarseShape<CB>::CPG * k + J / CoarseShape<CB>::PPC;
    const uint8_t *ra = sm.pair[p % CoarseShape<CB>::NP] + (J % CoarseShape<CB>::PPC) * CoarseShape<CB>::PAIR_BYTES, *rb = ra + RB;
    // the thread's own sub-block 2 J + (tig >> 1) of queries 2 (tig & 1) + e, and the pair's maximum (the same value in
    // both parities' threads, so their running maxima stay equal)
    float mbj[2], mp[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const float other = __shfl_xor_sync(FULL, sc.mb[1][e], 2);
      mbj[e] = odd ? other : sc.mb[0][e];
      const float pm = fmaxf(sc.mb[0][e], sc.mb[1][e]), pmo = __shfl_xor_sync(FULL, pm, 2);
      mp[e] = odd ? pmo : pm;
    }
    // the running maximum moves only when a pair exceeds it by more than 2^8 (weights stay <= 2^8; the rescale is rare)
    const bool grow = mp[0] > run.m[0] + 8.f || mp[1] > run.m[1] + 8.f;
    if (__any_sync(FULL, grow)) {
      float alv[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float mn = mp[e] > run.m[e] + 8.f ? mp[e] : run.m[e], al = ex2(run.m[e] - mn);  // (2^-inf = 0 on the first group)
        run.m[e] = mn;
        run.l[e] *= al;
        alv[e] = al;
      }
      const float2 al2 = make_float2(alv[0], alv[1]);
      Bs = __fmul2_rn(Bs, al2);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) { run.o[u][cc] = __fmul2_rn(run.o[u][cc], al2); A[u][cc] = __fmul2_rn(A[u][cc], al2); }
    }
    if (tig < 2) {  // P bytes: pst[parity][query][token]
#pragma unroll
      for (int par = 0; par < 2; ++par)
#pragma unroll
        for (int e = 0; e < 2; ++e)
          if (query_valid<QG>(tig, e)) {
            const int qe = 2 * tig + e;
            sm.pst[(par * 4 + qe) * 16 + gid] = (uint8_t)__float_as_uint(fmaf(ex2(sc.s[par][e] - sc.mb[par][e]), 255.f, MAGICF));
            sm.pst[(par * 4 + qe) * 16 + gid + 8] = (uint8_t)__float_as_uint(fmaf(ex2(sc.s[par][2 + e] - sc.mb[par][e]), 255.f, MAGICF));
          }
    }
    __syncwarp();
    // column gid of the value products: gid < 4: parity 0, query gid, k block = tokens 4 tig ..; gid >= 4: parity 1
    const uint32_t pw = lds32(sm.pst + 4 * lane);
    const uint32_t b0 = gid < 4 ? pw : 0u, b1 = gid < 4 ? 0u : pw;
    const float2 wj = make_float2(ex2(mbj[0] - run.m[0]), ex2(mbj[1] - run.m[1]));
    {  // sum p of both sub-blocks, every column: a product with an all-ones A
      uint32_t d[4];
      mma_u8u8_k32_from(d, 0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u, b0, b1, MAGIC);
      const float2 sp = isum2(d[0], d[1]);
      Bs = __ffma2_rn(wj, sp, Bs);
      if (gid == 0) {
        if (query_valid<QG>(tig, 0)) lse_group[(2 * J + (tig >> 1)) * QG + 2 * (tig & 1)] = mbj[0] + lg2(sp.x);
        if (query_valid<QG>(tig, 1)) lse_group[(2 * J + (tig >> 1)) * QG + 2 * (tig & 1) + 1] = mbj[1] + lg2(sp.y);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      uint32_t va[4], vb[4];
      v_slots<CB>(ra, 8 * u + gid, tig, va);
      v_slots<CB>(rb, 8 * u + gid, tig, vb);
      uint32_t d01[4], d23[4];
      mma_u8u8_k32_from(d01, va[0], va[1], vb[0], vb[1], b0, b1, MAGIC);  // rows gid: channel cc 0, gid + 8: cc 1
      mma_u8u8_k32_from(d23, va[2], va[3], vb[2], vb[3], b0, b1, MAGIC);  // cc 2, cc 3
      A[u][0] = __ffma2_rn(wj, isum2(d01[0], d01[1]), A[u][0]);
      A[u][1] = __ffma2_rn(wj, isum2(d01[2], d01[3]), A[u][1]);
      A[u][2] = __ffma2_rn(wj, isum2(d23[0], d23[1]), A[u][2]);
      A[u][3] = __ffma2_rn(wj, isum2(d23[2], d23[3]), A[u][3]);
    }
    __syncwarp();  // pst is free; after a chunk's last pair its slot is too
    if (J % CoarseShape<CB>::PPC == CoarseShape<CB>::PPC - 1) ring.issue_next();  // refill the slot with the chunk NP ahead
  };
#pragma unroll 1
  for (int J = 0; J < SBG / 2; ++J) {
    Scores sc;
    if (!stage_a(J, sc)) return false;
    stage_b(J, sc);
  }
  // fold the group into the running softmax: o += vs' A + vb' B, coarse cell midpoints folded into vb'
  run.l[0] += Bs.x; run.l[1] += Bs.y;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const uint4 vm = lds128(meta + 512 + 16 * (8 * u + gid));
    const float vb[4] = {bf_lo(vm.x), bf_hi(vm.x), bf_lo(vm.y), bf_hi(vm.y)}, vs[4] = {bf_lo(vm.z), bf_hi(vm.z), bf_lo(vm.w), bf_hi(vm.w)};
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      const float vbp = fmaf(vs[cc], HOFF, vb[cc]), vsp = __fmul_rn(vs[cc], (float)(1 << FB) * v_unscale<CB>(cc));
      run.o[u][cc] = __fadd2_rn(run.o[u][cc], __ffma2_rn(splat(vsp), A[u][cc], __fmul2_rn(splat(vbp), Bs)));
    }
  }
  return true;
}

// ---- the coarse kernel -------------------------------------------------------------------------------------------------
template <int QG> __device__ __forceinline__ void reset(Run &r) {
  r.m[0] = r.m[1] = -FBLA_INF; r.l[0] = r.l[1] = 0.f;
#pragma unroll
  for (int u = 0; u < 4; ++u)
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) r.o[u][cc] = make_float2(0.f, 0.f);
}
// one partial row set: threads tig and tig ^ 2 hold the two sub-block parities of the same (channel, query) sums
template <int QG> __device__ __forceinline__ void write_partial(float *p, const Run &r, int lane, bool correction) {
  const int gid = lane >> 2, tig = lane & 3;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const float l = r.l[e] + __shfl_xor_sync(FULL, r.l[e], 2);
    const int qe = 2 * tig + e;
    float *row = p + qe * PSTRIDE;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float4 v;
      const float o0 = e ? r.o[u][0].y : r.o[u][0].x, o1 = e ? r.o[u][1].y : r.o[u][1].x;
      const float o2 = e ? r.o[u][2].y : r.o[u][2].x, o3 = e ? r.o[u][3].y : r.o[u][3].x;
      v.x = o0 + __shfl_xor_sync(FULL, o0, 2);
      v.y = o1 + __shfl_xor_sync(FULL, o1, 2);
      v.z = o2 + __shfl_xor_sync(FULL, o2, 2);
      v.w = o3 + __shfl_xor_sync(FULL, o3, 2);
      if (tig < 2 && qe < QG) *reinterpret_cast<float4 *>(row + 4 * (8 * u + gid)) = v;
    }
    if (tig < 2 && qe < QG && gid == 0) {
      if (correction) row[D] = l;
      else { row[D] = r.m[e]; row[D + 1] = l; }
    }
  }
}


// dst (scratch) = the staged row set `own` merged with the first staged row sets of the next `more` warps (`next` points at
// the first of them, the following ones lie one StreamWarp further each): per query the usual log-sum-exp merge of
// (m, l, o[128]), taken in warp order. Lane l owns channels 4 l .. 4 l + 3.
template <int QG, class W>
__device__ __forceinline__ void fold_rows(float *dst, const float *own, const float *next, int more, int lane, size_t warp_stride_floats) {
#pragma unroll
  for (int qi = 0; qi < QG; ++qi) {
    const float *p = own + qi * PSTRIDE;
    float4 o = *reinterpret_cast<const float4 *>(p + 4 * lane);
    float m = p[D], l = p[D + 1];
    for (int x = 0; x < more; ++x) {
      const float *n = next + (size_t)x * warp_stride_floats + qi * PSTRIDE;
      const float4 o2 = *reinterpret_cast<const float4 *>(n + 4 * lane);
      const float m2 = n[D], l2 = n[D + 1];
      const float mn = fmaxf(m, m2), sa = ex2(m - mn), sb = ex2(m2 - mn);
      o.x = fmaf(o.x, sa, o2.x * sb); o.y = fmaf(o.y, sa, o2.y * sb); o.z = fmaf(o.z, sa, o2.z * sb); o.w = fmaf(o.w, sa, o2.w * sb);
      l = fmaf(l, sa, l2 * sb);
      m = mn;
    }
    float *d = dst + qi * PSTRIDE;
    *reinterpret_cast<float4 *>(d + 4 * lane) = o;
    if (lane == 0) { d[D] = m; d[D + 1] = l; }
  }
}

// DEAL: how the work is dealt to the warps (FBLA_K_DEAL_*, the host's choice in fbla_k_decode::deal; one build per way, so
// that none carries the others' code)
template <int CB, int FB, int QG, int DEAL>
__device__ __forceinline__ void coarse_item(const fbla_k_decode &a, uint8_t *smem_raw) {
  using Sh = CoarseShape<CB>;
  allow_next_pass();
  smem_raw += (128u - (smem_u32(smem_raw) & 127u)) & 127u;  // (an executor's storage is 16-byte aligned; an offset keeps the pointer's address space known)
  CoarseSmem<CB> &sm = *reinterpret_cast<CoarseSmem<CB> *>(smem_raw);
  const int lane = FBLA_POS::tid() & 31, warp = FBLA_POS::tid() >> 5;
  if (FBLA_POS::x() == 0 && FBLA_POS::tid() == 0 && a.status && !a.status_cleared) { a.status[0] = 0; a.status[1] = 0; }
  const int hpr = a.kv_heads * a.vg;
  int sw = Sh::TOTAL;                 // streaming warps of this CTA
  long long gw, lo, hi;               // the warp's index among the grid's streaming warps and its run of the flattened groups
  if (DEAL != FBLA_K_DEAL_COST) {  // the CTA's last xw warps serve windows, the others stream
    const Split sp = DEAL == FBLA_K_DEAL_LENGTHS ? split_of(a, hpr) : Split{Sh::WARPS, 1};
    sw = sp.sw;
    if (warp >= sw) {
      exact_warp<QG>(a, *reinterpret_cast<ExactWarp *>(&sm.w[warp]), lane, FBLA_POS::x() * sp.xw + (warp - sw), FBLA_POS::nx() * sp.xw);
      return;
    }
    const long long total = total_units<false>(a, hpr), per = ceil_div(total, (long long)FBLA_POS::nx() * sw);
    gw = (long long)FBLA_POS::x() * sw + warp;
    lo = gw * per;
    hi = min(total, lo + per);
  } else {  // the warp's share of all units by cost: its window sub-blocks first, then its groups
    const Deal d = deal_of(a, hpr);
    long long xlo, xhi;
    gw = (long long)FBLA_POS::x() * sw + warp;
    deal_range(d, gw, xlo, xhi, lo, hi);
    exact_range<QG>(a, *reinterpret_cast<ExactWarp *>(&sm.w[warp]), lane, xlo, xhi, (int)gw);
    __syncwarp();
  }
  StreamWarp<CB> &w = sm.w[warp];
  for (int i = lane; i < (int)sizeof(w.qst) / 4; i += 32) reinterpret_cast<uint32_t *>(w.qst)[i] = 0u;
  reinterpret_cast<uint32_t *>(w.pst)[lane] = 0u;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < Sh::NP; ++s) mbar_init(&w.bar_pair[s], 1);
    mbar_init(&w.bar_meta[0], 1);
    mbar_init(&w.bar_meta[1], 1);
    mbar_init_fence();
  }
  __syncwarp();

  // (before leaving, a warp invalidates its barriers: an executor may run another item on this CTA, whose initialisation
  // then meets no live barrier object)
  auto retire = [&]() {
    __syncwarp();
    if (lane == 0) {
#pragma unroll
      for (int s = 0; s < Sh::NP; ++s) mbar_inval(&w.bar_pair[s]);
      mbar_inval(&w.bar_meta[0]);
      mbar_inval(&w.bar_meta[1]);
    }
  };
  // a.fold (few virtual heads, each spread over many warps): one partial row per (CTA, virtual head), slot cta + vh. Rows
  // of virtual heads that lie wholly inside the warp's run go straight to the scratch; the run's first and last virtual
  // head may continue in the neighbouring warps, so their rows are staged in shared memory and folded below, in warp order
  // (a fixed order: the result is reproducible bit for bit). Otherwise: one row per (warp, virtual head), slot gw + vh.
  const int cta = FBLA_POS::x();
  int first_vh = -1, cur_vh = -1;
  bool ok = true;
  if (lo < hi) {
    Cursor cc = locate<false>(a, hpr, lo);
    Ring<CB> ring{w, a, hpr, lane, cc, 0, (int)(Sh::CPG * (hi - lo)), nullptr, nullptr};
    ring.point();
#pragma unroll
    for (int s = 0; s < Sh::NP; ++s) ring.issue_next();
    Run run;
    float4 q4[QG];
    for (long long u = lo; u < hi; ++u, advance<false>(a, hpr, cc)) {
      const int vh = cc.b * hpr + cc.hir;
      if (vh != cur_vh) {
        if (cur_vh >= 0)
          write_partial<QG>(!a.fold ? a.part + (size_t)(gw + cur_vh) * QG * PSTRIDE
                            : cur_vh == first_vh ? &w.stage[0][0][0] : a.part + (size_t)(cta + cur_vh) * QG * PSTRIDE, run, lane, false);
        if (cur_vh < 0) first_vh = vh;
        cur_vh = vh;
        reset<QG>(run);
#pragma unroll
        for (int qi = 0; qi < QG; ++qi) {
          const uint2 qw = __ldg(reinterpret_cast<const uint2 *>(a.q + (size_t)q_row(a, cc.b, cc.hir, qi) * D) + lane);
          q4[qi] = make_float4(bf_lo(qw.x), bf_hi(qw.x), bf_lo(qw.y), bf_hi(qw.y));
        }
      }
      if (!coarse_group<CB, FB, QG>(ring, (int)(u - lo), q4, a.sl, lane, run, a.lse + ((size_t)vh * a.nblocks + (size_t)group_of(a, cc) * SBG) * QG)) {
        if (lane == 0) report(a, 1);
        ok = false;
        break;
      }
    }
    if (ok) write_partial<QG>(!a.fold ? a.part + (size_t)(gw + cur_vh) * QG * PSTRIDE : &w.stage[cur_vh == first_vh ? 0 : 1][0][0], run, lane, false);
  }
  if (!a.fold) {  // one row per (warp, virtual head), already in the scratch
    if (ok) retire();
    return;
  }
  if (ok) retire();  // (after a wait that gave up a copy may still be in flight: the barriers stay as they are)
  if (lane == 0) {
    w.stage_vh[0] = ok ? first_vh : -1;
    w.stage_vh[1] = ok && cur_vh != first_vh ? cur_vh : -1;
  }
  // every streaming warp of the CTA has staged its rows
  asm volatile("bar.sync 1, %0;" ::"r"(32 * sw) : "memory");
  // Row r of this warp is folded here unless an earlier warp does it: the first row belongs to the first warp that
  // touched its virtual head, the last row (a later virtual head) always to this warp. The rows that continue it are
  // the first rows of the following warps, as long as those warps stay inside the same virtual head.
#pragma unroll 1
  for (int r = 0; r < 2; ++r) {
    const int v = w.stage_vh[r];
    if (v < 0) continue;
    if (r == 0 && warp > 0) {
      const StreamWarp<CB> &prev = sm.w[warp - 1];
      const int prev_last = prev.stage_vh[1] >= 0 ? prev.stage_vh[1] : prev.stage_vh[0];
      if (prev_last == v) continue;
    }
    if (r == 0 && w.stage_vh[1] >= 0) {  // the virtual head ends inside this warp's run: nothing to fold
      fold_rows<QG, StreamWarp<CB>>(a.part + (size_t)(cta + v) * QG * PSTRIDE, &w.stage[0][0][0], nullptr, 0, lane, 0);
      continue;
    }
    int more = 0;
    for (int x = warp + 1; x < sw && sm.w[x].stage_vh[0] == v; ++x) {
      ++more;
      if (sm.w[x].stage_vh[1] >= 0) break;
    }
    fold_rows<QG, StreamWarp<CB>>(a.part + (size_t)(cta + v) * QG * PSTRIDE, &w.stage[r][0][0], warp + 1 < sw ? &sm.w[warp + 1].stage[0][0][0] : nullptr, more, lane, sizeof(StreamWarp<CB>) / sizeof(float));
  }
}

// ---- which partial slots belong to a virtual head ------------------------------------------------------------------------
struct Slots { int c0, c1, x0, x1; };  // coarse CTAs (a.fold) or warps c0..c1 (slot c + vh), window warps x0..x1 (slot tw + vheads + x + vh); empty if c1 < c0
__device__ __forceinline__ Slots slots_of(const fbla_k_decode &a, int vh) {
  const int hpr = a.kv_heads * a.vg;
  Slots s{0, -1, 0, -1};
  int n;
  if (a.deal == FBLA_K_DEAL_COST) {  // a unit belongs to the warp whose cost share holds the start of its cost interval (deal_range)
    const Deal d = deal_of(a, hpr);
    long long off = head_offset<false>(a, hpr, vh, n);
    if (n > 0) {
      const long long div = d.P * (a.fold ? a.coarse_warps : 1);  // (a.fold: one row per CTA = coarse_warps consecutive warps)
      s.c0 = (int)((d.wc * d.X + GROUP_COST * off) / div);
      s.c1 = (int)((d.wc * d.X + GROUP_COST * (off + n - 1)) / div);
    }
    off = head_offset<true>(a, hpr, vh, n);
    if (n > 0) { s.x0 = (int)(d.wc * off / d.P); s.x1 = (int)(d.wc * (off + n - 1) / d.P); }
    return s;
  }
  const Split sp = split_of(a, hpr);
  long long off = head_offset<false>(a, hpr, vh, n);
  if (n > 0) { const long long per = ceil_div(total_units<false>(a, hpr), (long long)a.coarse_ctas * sp.sw) * (a.fold ? sp.sw : 1); s.c0 = (int)(off / per); s.c1 = (int)((off + n - 1) / per); }
  off = head_offset<true>(a, hpr, vh, n);
  if (n > 0) { const long long per = ceil_div(total_units<true>(a, hpr), (long long)a.coarse_ctas * sp.xw); s.x0 = (int)(off / per); s.x1 = (int)((off + n - 1) / per); }
  return s;
}
__device__ __forceinline__ const float *coarse_slot(const fbla_k_decode &a, int w, int vh, int qi) {
  return a.part + ((size_t)(w + vh) * a.qg + qi) * PSTRIDE;
}
__device__ __forceinline__ const float *window_slot(const fbla_k_decode &a, int x, int vh, int qi) {
  const int base = a.coarse_ctas * a.coarse_warps + a.batch * a.kv_heads * a.vg;
  return a.part + ((size_t)(base + x + vh) * a.qg + qi) * PSTRIDE;
}

// ---- select: R = log2 of the row's coarse mass; the sub-blocks holding more than tau of it for some query ------------
template <int QG>
__device__ __forceinline__ void select_item(const fbla_k_decode &a, uint8_t *smem_raw) {
  __shared__ float R[4];
  __shared__ int wc[8];
  const int lane = FBLA_POS::tid() & 31, warp = FBLA_POS::tid() >> 5, vh = FBLA_POS::y(), slice = FBLA_POS::x();
  const int hpr = a.kv_heads * a.vg;
  allow_next_pass();
  const Row row = row_of(a, vh / hpr);
  const Slots s = slots_of(a, vh);
  wait_previous_pass();
  // the slice's sub-block masses first (they do not depend on R): a thread takes four consecutive sub-blocks, so its loads
  // are contiguous and all in flight together
  const int mine0 = slice * SLICE + warp * (SLICE / 8) + 4 * lane, first = SBG * row.g0, hi = SBG * (row.g0 + row.closed);
  float x[4][QG];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int sb = mine0 + i;
    const bool closed = a.phase != 1 && sb >= first && sb < hi;
    const float *p = a.lse + ((size_t)vh * a.nblocks + (closed ? sb : 0)) * QG;
#pragma unroll
    for (int qi = 0; qi < QG; ++qi) x[i][qi] = closed ? __ldcg(p + qi) : -FBLA_INF;
  }
  if (a.phase == 2) {  // the rows' (global) log2 mass is given
    if (FBLA_POS::tid() < QG) R[FBLA_POS::tid()] = __ldcg(a.row_r + vh * QG + FBLA_POS::tid());
  } else if (warp < QG) {  // R of query `warp`: one pass over the head's partial (m, l), merged online, then across lanes
    const int nc = s.c1 - s.c0 + 1, nx = s.x1 - s.x0 + 1, n = nc + nx;
    float mx = -FBLA_INF, ls = 0.f;
    for (int i0 = 0; i0 < n; i0 += 128) {  // four rows per lane at a time, their loads all in flight before the first is used
      float mm[4], ll[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = i0 + 32 * j + lane;
        mm[j] = -FBLA_INF; ll[j] = 0.f;
        if (i < n) {
          const float *p = i < nc ? coarse_slot(a, s.c0 + i, vh, warp) : window_slot(a, s.x0 + i - nc, vh, warp);
          mm[j] = __ldcg(p + D); ll[j] = __ldcg(p + D + 1);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (mm[j] != -FBLA_INF) {
          const float mn = fmaxf(mx, mm[j]);
          ls = fmaf(ls, ex2(mx - mn), ll[j] * ex2(mm[j] - mn));
          mx = mn;
        }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float m2 = __shfl_xor_sync(FULL, mx, o), l2 = __shfl_xor_sync(FULL, ls, o);
      const float mn = fmaxf(mx, m2);
      // (lanes pair up symmetrically: both compute the same sum in the same order of magnitudes)
      const float a1 = mx == -FBLA_INF ? 0.f : ls * ex2(mx - mn), a2 = m2 == -FBLA_INF ? 0.f : l2 * ex2(m2 - mn);
      ls = (lane & o) ? a2 + a1 : a1 + a2;
      mx = mn;
    }
    const float r = mx + lg2(ls);  // (-inf for a shard that holds nothing of this row)
    if (!lane) { R[warp] = r; if (!slice) a.row_r[vh * QG + warp] = r; }
  }
  if (a.phase == 1) return;  // only the local mass was asked for
  __syncthreads();
  // The thread's selected sub-blocks become items (sub-block << 4) | query mask; their place in the slice's list:
  // an inclusive scan of the per-thread counts over the warp, and the warps' totals through shared memory.
  int masks[4], kept = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    masks[i] = 0;
#pragma unroll
    for (int qi = 0; qi < QG; ++qi) masks[i] |= (x[i][qi] - R[qi] > a.log2_tau ? 1 : 0) << qi;
    kept += masks[i] != 0;
  }
  int upto = kept;  // selected by lanes 0 .. lane of this warp
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int below = __shfl_up_sync(FULL, upto, o);
    if (lane >= o) upto += below;
  }
  if (lane == 31) wc[warp] = upto;
  __syncthreads();
  int before = 0, total = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w) { if (w < warp) before += wc[w]; total += wc[w]; }
  int *dst = a.items + ((size_t)vh * a.nslices + slice) * SLICE + before + (upto - kept);
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (masks[i]) *dst++ = ((mine0 + i) << 4) | masks[i];
  if (!FBLA_POS::tid()) a.counts[(size_t)vh * a.nslices + slice] = total;
}

// ---- refine: full - coarse of every selected sub-block ----------------------------------------------------------------------
template <int CB, int FB> struct RefineShape {
  static constexpr int WARPS = FBLA_RW, NST = FBLA_RNST;
  static constexpr int RC = record_bytes(CB), RF = record_bytes(FB);
  static constexpr int STAGE = RC + RF;
};
template <int CB, int FB> struct __align__(128) RefineWarp {
  uint8_t stage[RefineShape<CB, FB>::NST][RefineShape<CB, FB>::STAGE];
  uint8_t meta[2][1024];  // the metadata of the two groups that items in flight can belong to (NST = 2: the item in work and one ahead)
  uint8_t qst[8 * QST_ROW];
  uint8_t pst[128];  // rows 0..3: P under the full scores, rows 4..7: under the coarse scores; 16 tokens each
  uint64_t bar[RefineShape<CB, FB>::NST];
};

template <int CB, int FB, int QG>
__device__ __forceinline__ void refine_item(const fbla_k_decode &a, uint8_t *smem_raw) {
  using Sh = RefineShape<CB, FB>;
  constexpr float HOFF = .5f * ((1 << FB) - 1);
  smem_raw += (128u - (smem_u32(smem_raw) & 127u)) & 127u;  // (an executor's storage is 16-byte aligned; an offset keeps the pointer's address space known)
  RefineWarp<CB, FB> *ws = reinterpret_cast<RefineWarp<CB, FB> *>(smem_raw);
  int *pre = reinterpret_cast<int *>(smem_raw + sizeof(RefineWarp<CB, FB>) * Sh::WARPS);  // [entries + 1]
  __shared__ int chunk_sum[256];
  const int lane = FBLA_POS::tid() & 31, warp = FBLA_POS::tid() >> 5, gid = lane >> 2, tig = lane & 3;
  const int hpr = a.kv_heads * a.vg, vheads = a.batch * hpr, entries = vheads * a.nslices;
  allow_next_pass();
  wait_previous_pass();
  // exclusive prefix of the slices' counts: pre[e], e = vh * nslices + slice
  {
    const int per = (entries + 255) / 256, e0 = FBLA_POS::tid() * per, e1 = min(entries, e0 + per);
    int sum = 0;
    for (int e = e0; e < e1; ++e) sum += __ldcg(a.counts + e);
    if (FBLA_POS::tid() < 256) chunk_sum[FBLA_POS::tid()] = sum;  // (threads past 256 own no entries)
    __syncthreads();
    if (warp == 0) {
      int run = 0;
      for (int i0 = 0; i0 < 256; i0 += 32) {
        const int v = chunk_sum[i0 + lane];
        int x = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(FULL, x, o); x += lane >= o ? y : 0; }
        chunk_sum[i0 + lane] = run + x - v;
        run += __shfl_sync(FULL, x, 31);
      }
      if (!lane) pre[entries] = run;
    }
    __syncthreads();
    int acc = FBLA_POS::tid() < 256 ? chunk_sum[FBLA_POS::tid()] : 0;
    for (int e = e0; e < e1; ++e) { pre[e] = acc; acc += __ldcg(a.counts + e); }
    __syncthreads();
    if (FBLA_POS::x() == 0)  // for the merge: the first item of every virtual head, and the total
      for (int v = FBLA_POS::tid(); v <= vheads; v += 32 * Sh::WARPS) a.item_off[v] = pre[v * a.nslices];
  }
  const int total = pre[entries];
  const long long rw = (long long)FBLA_POS::nx() * Sh::WARPS;
  const int per = (int)ceil_div(total, rw), gw = FBLA_POS::x() * Sh::WARPS + warp;
  const int lo = gw * per, hi = min(total, lo + per);
  if (lo >= hi) return;
  RefineWarp<CB, FB> &w = ws[warp];
  for (int i = lane; i < (int)sizeof(w.qst) / 4; i += 32) reinterpret_cast<uint32_t *>(w.qst)[i] = 0u;
  reinterpret_cast<uint32_t *>(w.pst)[lane] = 0u;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < Sh::NST; ++s) mbar_init(&w.bar[s], 1);
    mbar_init_fence();
  }
  __syncwarp();
  // entry of item lo: the last e with pre[e] <= lo
  int fe;
  {
    int l = 0, h = entries;  // pre[l] <= lo < pre[h]
    while (h - l > 1) { const int mid = (l + h) >> 1; if (pre[mid] <= lo) l = mid; else h = mid; }
    fe = l;
  }
  // The warp's items are read 32 at a time, one per lane (lane i: item base + i, with its entry), and handed out by
  // shuffles: the per-item loads of the list would otherwise sit, one dependent round trip to L2 each, in front of every
  // copy that is issued and every item that is decoded.
  int win_base = lo, win_it = 0, win_e = fe;
  auto load_window = [&](int base, int e_start) {
    win_base = base;
    const int k = base + lane;
    int e = e_start;
    if (k < hi) {
      while (pre[e + 1] <= k) ++e;
      win_it = __ldcg(a.items + (size_t)e * SLICE + (k - pre[e]));
    }
    win_e = e;
  };
  auto item_at = [&](int k, int &e) {  // item k of the window (warp-uniform k): its entry and value
    e = __shfl_sync(FULL, win_e, k - win_base);
    return __shfl_sync(FULL, win_it, k - win_base);
  };
  load_window(lo, fe);
  long long issued_unit = -1;  // (lane 0) the (virtual head, group) of the last item issued, and which metadata buffer it uses
  int issued_par = 1;
  auto issue = [&](int it, int e, int s) {  // lane 0
    const int vh = e / a.nslices, bh = vh / a.vg, sb = it >> 4;
    const size_t unit = (size_t)bh * a.hs + (size_t)(sb / SBG) * a.gs, rec = unit * SBG + sb % SBG;
    const long long vu = (long long)vh * a.nblocks + sb / SBG;
    const bool fresh = vu != issued_unit;  // the group's metadata travels with its first item only
    mbar_expect_tx(&w.bar[s], Sh::STAGE + (fresh ? 1024 : 0));
    bulk_g2s(w.stage[s], a.c.coarse + rec * Sh::RC, Sh::RC, &w.bar[s]);
    bulk_g2s(w.stage[s] + Sh::RC, a.c.fine + rec * Sh::RF, Sh::RF, &w.bar[s]);
    if (fresh) {
      issued_unit = vu; issued_par ^= 1;
      bulk_g2s(w.meta[issued_par], reinterpret_cast<const uint8_t *>(a.c.meta) + unit * 1024, 1024, &w.bar[s]);
    }
  };
#pragma unroll
  for (int s = 0; s < Sh::NST; ++s)
    if (lo + s < hi) {
      int e;
      const int first = item_at(lo + s, e);
      if (lane == 0) issue(first, e, s);
    }
  Run run;  // m unused: corrections are already in units of 2^-R
  float2 Ag[4][4], Bg = make_float2(0.f, 0.f);  // the current group's sums in code units, (.x, .y) = queries e = 0, 1
#pragma unroll
  for (int u = 0; u < 4; ++u)
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) Ag[u][cc] = make_float2(0.f, 0.f);
  float4 q4[QG];
  float Rq[2] = {0.f, 0.f}, c0[2] = {0.f, 0.f}, sqc[2] = {0.f, 0.f}, sqf[2] = {0.f, 0.f}, qbf[2] = {0.f, 0.f};
  uint32_t B[8];
  int cur_vh = -1, cur_par = 1;
  long long cur_unit = -1, cur_unit2 = -1;  // cur_unit is also reset when the virtual head changes; cur_unit2 follows the groups only
  for (int k = lo; k < hi; ++k) {
    const int s = (k - lo) % Sh::NST;
    if (k + Sh::NST >= win_base + 32) {  // the window moves on before an item beyond it is asked for
      int e0;
      item_at(k, e0);
      load_window(k, e0);
    }
    int ce;
    const int it = item_at(k, ce), vh = ce / a.nslices, sb = it >> 4;
    if (vh != cur_vh) {
      if (cur_vh >= 0) write_partial<QG>(a.dpart + (size_t)(gw + cur_vh) * QG * PSTRIDE, run, lane, true);
      cur_vh = vh; cur_unit = -1;
      reset<QG>(run);
      const int b = vh / hpr, hir = vh - b * hpr;
#pragma unroll
      for (int qi = 0; qi < QG; ++qi) {
        const uint2 qw = __ldg(reinterpret_cast<const uint2 *>(a.q + (size_t)q_row(a, b, hir, qi) * D) + lane);
        q4[qi] = make_float4(bf_lo(qw.x), bf_hi(qw.x), bf_lo(qw.y), bf_hi(qw.y));
      }
#pragma unroll
      for (int e = 0; e < 2; ++e) Rq[e] = query_valid<QG>(tig, e) ? __ldcg(a.row_r + vh * QG + 2 * (tig & 1) + e) : 0.f;
    }
    const bool ok = mbar_wait_bounded(&w.bar[s], ((k - lo) / Sh::NST) & 1);
    if (!__all_sync(FULL, ok)) {
      if (lane == 0) report(a, 3);
      return;
    }
    const uint8_t *crec = w.stage[s], *frec = crec + Sh::RC;
    const long long unit = (long long)vh * a.nblocks + sb / SBG;
    if (unit != cur_unit2) { cur_unit2 = unit; cur_par ^= 1; }  // (the same sequence of groups as the issuing side)
    const uint8_t *meta = w.meta[cur_par];
    if (unit != cur_unit) {  // the group's qhat: the same function of the same inputs as the coarse pass
      cur_unit = unit;
      __syncwarp();
      const uint4 km = lds128(meta + 16 * lane);
#pragma unroll
      for (int qi = 0; qi < QG; ++qi) {
        float sq, qb, qsum;
        quantize_query(km, q4[qi], a.sl, reinterpret_cast<uint32_t *>(w.qst + QST_ROW * qi), lane, sq, qb, qsum);
        const float c = fmaf(__fmul_rn(sq, HOFF), qsum, qb), s2 = __fmul_rn(sq, (float)(1 << FB));
#pragma unroll
        for (int e = 0; e < 2; ++e)
          if (qi == 2 * (tig & 1) + e) { c0[e] = c; sqc[e] = s2; sqf[e] = sq; qbf[e] = qb; }
      }
      __syncwarp();
      qhat_frag<CB>(w.qst, gid, tig, B);
    }
    float xh[4], xl[4];
    qk_tile<CB>(crec, gid, tig, B, xh);
    qk_tile<FB>(frec, gid, tig, B, xl);
    // columns 2 tig + e (tig < 2: queries): coarse and full scores of tokens gid, gid + 8
    float mc[2], mf[2], sc[2][2], sf[2][2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        sc[e][r] = fmaf(sqc[e], xh[2 * r + e], c0[e]);
        sf[e][r] = fmaf(sqf[e], fmaf((float)(1 << FB), xh[2 * r + e], xl[2 * r + e]), qbf[e]);
      }
      float vc = fmaxf(sc[e][0], sc[e][1]), vf = fmaxf(sf[e][0], sf[e][1]);
#pragma unroll
      for (int o = 4; o <= 16; o <<= 1) { vc = fmaxf(vc, __shfl_xor_sync(FULL, vc, o)); vf = fmaxf(vf, __shfl_xor_sync(FULL, vf, o)); }
      mc[e] = vc; mf[e] = vf;
    }
    if (tig < 2) {
#pragma unroll
      for (int e = 0; e < 2; ++e)
        if (query_valid<QG>(tig, e)) {
          const int qe = 2 * tig + e;
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            w.pst[qe * 16 + gid + 8 * r] = (uint8_t)__float_as_uint(fmaf(ex2(sf[e][r] - mf[e]), 255.f, MAGICF));
            w.pst[(4 + qe) * 16 + gid + 8 * r] = (uint8_t)__float_as_uint(fmaf(ex2(sc[e][r] - mc[e]), 255.f, MAGICF));
          }
        }
    }
    __syncwarp();
    // Value products: column gid < 4: query gid under the full scores, gid >= 4: query gid - 4 under the coarse ones.
    // Thread (gid, tig) reads columns 2 tig + e: tig < 2 holds the full-score sums of queries 2 tig + e, tig >= 2 the
    // coarse-score sums of queries 2 (tig - 2) + e.
    const bool cset = tig >> 1;
    const uint32_t b0 = lds32(w.pst + 4 * lane);
    float wgt[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const float mco = __shfl_xor_sync(FULL, mc[e], 2);
      const bool on = query_valid<QG>(tig, e) && ((it >> (2 * (tig & 1) + e)) & 1);
      wgt[e] = on ? (cset ? -ex2(mco - Rq[e]) : ex2(mf[e] - Rq[e])) : 0.f;
    }
    {
      const float2 wgt2 = make_float2(wgt[0], wgt[1]);
      {  // sum p of the thread's two columns: a product with an all-ones A
        uint32_t d[4];
        mma_u8u8_k16_from(d, 0x01010101u, 0x01010101u, b0, MAGIC);
        Bg = __ffma2_rn(wgt2, isum2(d[0], d[1]), Bg);
      }
      // the group's weighted code sums: full-score threads add w (2^FB h + f), coarse-score threads -w 2^FB h
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint32_t vh4[4], vl4[4];
        v_slots<CB>(crec, 8 * u + gid, tig, vh4);
        v_slots<FB>(frec, 8 * u + gid, tig, vl4);
        uint32_t h01[4], h23[4], l01[4], l23[4];
        mma_u8u8_k16_from(h01, vh4[0], vh4[1], b0, MAGIC);
        mma_u8u8_k16_from(h23, vh4[2], vh4[3], b0, MAGIC);
        mma_u8u8_k16_from(l01, vl4[0], vl4[1], b0, MAGIC);
        mma_u8u8_k16_from(l23, vl4[2], vl4[3], b0, MAGIC);
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const float ch_ = (float)(1 << FB) * v_unscale<CB>(cc), cl_ = cset ? 0.f : v_unscale<FB>(cc);
          const uint32_t *hh = cc < 2 ? h01 : h23, *ll = cc < 2 ? l01 : l23;
          const float2 yh = isum2(hh[2 * (cc & 1)], hh[2 * (cc & 1) + 1]), yl = isum2(ll[2 * (cc & 1)], ll[2 * (cc & 1) + 1]);
          Ag[u][cc] = __ffma2_rn(wgt2, __ffma2_rn(splat(ch_), yh, __fmul2_rn(splat(cl_), yl)), Ag[u][cc]);
        }
      }
      // the group's last item of this warp: apply the V affine once (coarse cells at their midpoint)
      bool last = k + 1 >= hi;
      if (!last) {
        int pe;
        const int nx = item_at(k + 1, pe);
        last = pe / a.nslices != vh || (nx >> 4) / SBG != sb / SBG;
      }
      if (last) {
        run.l[0] += Bg.x; run.l[1] += Bg.y;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint4 vm = lds128(meta + 512 + 16 * (8 * u + gid));
          const float vb[4] = {bf_lo(vm.x), bf_hi(vm.x), bf_lo(vm.y), bf_hi(vm.y)}, vs[4] = {bf_lo(vm.z), bf_hi(vm.z), bf_lo(vm.w), bf_hi(vm.w)};
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            const float vbx = cset ? fmaf(vs[cc], HOFF, vb[cc]) : vb[cc];
            run.o[u][cc] = __fadd2_rn(run.o[u][cc], __ffma2_rn(splat(vs[cc]), Ag[u][cc], __fmul2_rn(splat(vbx), Bg)));
            Ag[u][cc] = make_float2(0.f, 0.f);
          }
        }
        Bg = make_float2(0.f, 0.f);
      }
    }
    __syncwarp();
    if (k + Sh::NST < hi) {
      int ne;
      const int ahead = item_at(k + Sh::NST, ne);
      if (lane == 0) { fence_async_smem(); issue(ahead, ne, s); }
    }
  }
  write_partial<QG>(a.dpart + (size_t)(gw + cur_vh) * QG * PSTRIDE, run, lane, true);
  __syncwarp();
  if (lane == 0) {  // (as the coarse pass: no live barrier is left behind for the CTA's next item)
#pragma unroll
    for (int s = 0; s < Sh::NST; ++s) mbar_inval(&w.bar[s]);
  }
}

// ---- merge: out = (sum 2^(m_c - R) o_c + sum do) / (sum 2^(m_c - R) l_c + sum dl), BF16 ---------------------------------
// One CTA per output row (virtual head, query): thread (c4, sl) sums the partial rows sl, sl + 16, ... of channels
// 4 c4 .. 4 c4 + 3, the sixteen sums of a channel are then added in a fixed order.
template <int QG>
__device__ __forceinline__ void merge_item(const fbla_k_decode &a, uint8_t *smem_raw) {
  constexpr int NS = 16, MJ = 6;  // row slices of the CTA; rows a thread has in flight (two CTAs share an SM's registers)
  __shared__ float4 so[NS][32];
  __shared__ float sl_[NS];
  __shared__ Slots ss;
  const int vh = FBLA_POS::x() / QG, qi = FBLA_POS::x() % QG, c4 = FBLA_POS::tid() & 31, sl = FBLA_POS::tid() >> 5;
  const int hpr = a.kv_heads * a.vg, vheads = a.batch * hpr, b = vh / hpr, hir = vh - b * hpr;
  if (FBLA_POS::tid() == 0) ss = slots_of(a, vh);  // (from the lengths alone: before the previous pass has completed)
  __syncthreads();
  wait_previous_pass();
  const Slots s = ss;
  // every load that does not depend on another is issued here, ahead of the rows: the head's range of correction rows,
  // the row's mass, the status word
  const int it0 = __ldcg(a.item_off + vh), it1 = __ldcg(a.item_off + vh + 1), total = __ldcg(a.item_off + vheads);
  const float Rq = __ldcg(a.row_r + vh * QG + qi);
  const int status = a.status ? __ldcg(a.status) : 0;
  float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
  float L = 0.f;
  const int nc = s.c1 - s.c0 + 1, nx = s.x1 - s.x0 + 1, n = nc + nx;
  // (a long sequence at a small batch gives a head some tens of partial rows and a few hundred correction rows: NS * MJ
  // rows of the CTA in flight keep the number of dependent round trips to memory small; the summation order is fixed
  // by the loops alone)
  for (int i0 = sl; i0 < n; i0 += NS * MJ) {
    float m[MJ], l[MJ];
    float4 o[MJ];
#pragma unroll
    for (int j = 0; j < MJ; ++j) {
      const int i = min(i0 + NS * j, n - 1);
      const float *p = i < nc ? coarse_slot(a, s.c0 + i, vh, qi) : window_slot(a, s.x0 + i - nc, vh, qi);
      m[j] = __ldcg(p + D); l[j] = __ldcg(p + D + 1); o[j] = __ldcg(reinterpret_cast<const float4 *>(p) + c4);
    }
#pragma unroll
    for (int j = 0; j < MJ; ++j)
      if (i0 + NS * j < n) {
        const float e = m[j] == -FBLA_INF ? 0.f : ex2(m[j] - Rq);
        L = fmaf(e, l[j], L);
        O.x = fmaf(e, o[j].x, O.x); O.y = fmaf(e, o[j].y, O.y); O.z = fmaf(e, o[j].z, O.z); O.w = fmaf(e, o[j].w, O.w);
      }
  }
  int w0 = 0, w1 = -1;  // the refine warps whose runs of items met this head
  if (it1 > it0) {
    const int per = (int)ceil_div(total, (long long)a.refine_ctas * a.refine_warps);
    w0 = it0 / per; w1 = (it1 - 1) / per;
  }
  for (int i0 = w0 + sl; i0 <= w1; i0 += NS * MJ) {  // (one correction row per refine warp that met the head)
    float l[MJ];
    float4 o[MJ];
#pragma unroll
    for (int j = 0; j < MJ; ++j) {
      const float *p = a.dpart + ((size_t)(min(i0 + NS * j, w1) + vh) * QG + qi) * PSTRIDE;
      l[j] = __ldcg(p + D); o[j] = __ldcg(reinterpret_cast<const float4 *>(p) + c4);
    }
#pragma unroll
    for (int j = 0; j < MJ; ++j)
      if (i0 + NS * j <= w1) { L += l[j]; O.x += o[j].x; O.y += o[j].y; O.z += o[j].z; O.w += o[j].w; }
  }
  so[sl][c4] = O;
  if (c4 == 0) sl_[sl] = L;
  __syncthreads();
  if (FBLA_POS::tid() < D) {
    const int ch = FBLA_POS::tid();
    const float *col = reinterpret_cast<const float *>(so) + ch;  // so as [NS][128] floats
    float os[NS];
#pragma unroll
    for (int x = 0; x < NS; ++x) os[x] = col[x * D];
#pragma unroll
    for (int w = 1; w < NS; w <<= 1)  // pairwise: ((0 + 1) + (2 + 3)) + ...
#pragma unroll
      for (int x = 0; x < NS; x += 2 * w) os[x] += os[x + w];
    float ls[NS];
#pragma unroll
    for (int x = 0; x < NS; ++x) ls[x] = sl_[x];
#pragma unroll
    for (int w = 1; w < NS; w <<= 1)
#pragma unroll
      for (int x = 0; x < NS; x += 2 * w) ls[x] += ls[x + w];
    const float Os = os[0], Ls = ls[0];
    const size_t row = (size_t)q_row(a, b, hir, qi);
    // a pass of this call reported a wait that gave up: some partial rows were never written, so the row is NaN, not a
    // plausible number (every pass has completed by now, so every report is visible)
    const bool failed = status != 0;
    const float nan = __int_as_float(0x7fc00000);
    if (a.out_partial) {  // a shard's share of the row, in units of 2^-R: summed over the shards before the division
      a.out_partial[row * PSTRIDE + ch] = failed ? nan : Os;
      if (ch == 0) a.out_partial[row * PSTRIDE + D] = failed ? nan : Ls;
    } else {
      a.out[row * D + ch] = failed ? (uint16_t)0x7fc0 : f32_to_bf16(__fdividef(Os, Ls));
    }
  }
}


}  // namespace fbla
