// Causal prefill attention over the compressed cache on Blackwell tensor cores: tcgen05.mma with TMEM accumulators.
//
// Semantics: the reference's DP4A prefill (attention/fbla/src/fbla_prefill.cuh:389-705) -- the row at position p attends
// to 0..p: group 0 (sink) and its own group in BF16, closed groups 1..own-1 through their full 6-bit codes with the
// per-(row, group) int8 qhat, 16-token integer P blocks p = round(255 * 2^(s - max_block)) everywhere.
//
// One CTA = two tiles of 128 query rows of one KV head (row r = position r / qg, query r % qg) x a sequence of "passes",
// one per 128-token group the rows attend to. Per pass and tile, two tensor-core products with FP32 accumulators in
// tensor memory:
//   S[128 rows x 128 tokens]  = Qop[rows x 128 ch] . Kop[tokens x 128 ch]^T
//   O[128 rows x 128 ch]     += P'[rows x 128 tokens] . V'[ch x 128 tokens]^T
// Closed group: Qop = qhat (integers in [-127, 127]) and Kop = the 6-bit codes, both as FP16 -- products and the FP32
// sums (< 2^24) are exact, so S is the reference's integer dot product; BF16 group: Qop = q, Kop = k in BF16 (exact
// products, FP32 sums). P' = fp16(w_j p_t): the integer P block times its block weight 2^(m_j - m_row); V' =
// fp16(base + step * code) (closed) or fp16(v) (BF16), so O accumulates across ALL passes in tensor memory and is read
// once, at the end. The two FP16 roundings (relative 2^-11, zero mean) are the only deviations from the reference's
// arithmetic; they stay far inside the 2e-3 output tolerance.
//
// Warps 0-15: the rows. Softmax: two threads per row (warps w and w + 8 share a tensor-memory lane quadrant; warps 0-3,
// 8-11: tile 0); qhat: lane-per-channel-chunk over the tile's rows. Warps 16-19: operands, shared by both tiles: unpack the
// group's records (bulk-copied raw into shared memory) into the Kop / V' tiles. Warp 20: allocates tensor memory; its
// lane 0 issues the bulk copies and the products, which complete on mbarriers. P' is written over qhat (dead once S is complete). Operand tiles are K-major with the 128-byte swizzle
// (8-row x 128-byte atoms, 16-byte chunk c of row r at c ^ (r % 8)).
// What bounds it: per (row, group) the reference's semantics need ~130 exp2 and the requantisation of the row's 128
// query channels on the CUDA cores; the tensor-core share of a pass is about as long as its exp2 share alone.
// Every wait is bounded: on a timeout the thread raises a flag, everybody drains, tensor memory is freed, the kernel
// returns and the host sees fbla_k_attend_tc_status() != 0.
#pragma once
#include "fbla_tc.cuh"
#include "fbla_kernels.h"
#include <cuda_fp16.h>

namespace fbla {
namespace tc {

constexpr int ROWS = 128;                 // rows of a tile
constexpr int CTA_ROWS = 2 * ROWS;
#ifndef FBLA_PF_PRODUCERS
#define FBLA_PF_PRODUCERS 4  /* operand warps. Measured: 4 (21 warps, 80 registers, 28 bytes of spills) 336.5 TFLOP/s; 3 (96 registers, none) 324.8 */
#endif
constexpr int PRODUCERS = FBLA_PF_PRODUCERS, PT = 32 * PRODUCERS;  // operand warps and threads
constexpr int PRODUCER_WARP0 = 16, ISSUER_WARP = 16 + PRODUCERS;  // warps 0-15: rows
constexpr int THREADS = (17 + PRODUCERS) * 32;
constexpr int SLAB = ROWS * 128;          // bytes of one K slab (128 rows x 128 bytes): 64 FP16 / BF16 of the K extent
constexpr int TILE = 2 * SLAB;            // a [128 x 128] 16-bit operand tile: 32 KiB
constexpr int RAW = 8 * 3072;              // a raw group: 8 coarse + 8 fine records, 3072 bytes per pair in both formats
constexpr uint32_t WAIT_LIMIT = 1u << 18;

__device__ int g_status = 0;  // nonzero: a bounded wait gave up in some launch since the last read

struct __align__(1024) Smem {
  uint8_t q[2][TILE];   // Qop of BF16 passes: the rows' q, BF16
  uint8_t qp[2][TILE];  // Qop of closed passes: qhat as FP16 (at the very end: staging of the output rows)
  uint8_t k[TILE];      // Kop
  uint8_t v[TILE];      // V'
  uint8_t raw[RAW];     // the group's coarse records, then its fine records
  uint8_t meta[2][1024];  // the metadata of closed pass c in buffer c % 2, fetched two passes ahead
  float qscale[2][2][128], qbias[2][2][128];  // [pass parity][tile][row]: the pass's score scale and bias (from the quantising lanes to the row's threads)
  float ex2[2][128][2];  // exchange between the two threads of a row: pass maximum, final sum
  uint64_t bar_raw, bar_meta[2], bar_k, bar_v, bar_q[2], bar_s[2], bar_p[2], bar_o[2];
  uint32_t tmem_base;
  int abort;
};

static_assert(sizeof(Smem) + 1024 <= 232448, "operand tiles exceed the shared memory of an SM");

// ---- operand descriptors of this kernel's tiles ---------------------------------------------------------------------------
__device__ __forceinline__ uint64_t smem_desc(const void *tile_base, int slab, int kstep) { return smem_desc_at(tile_base, slab * SLAB + kstep * 32); }
__device__ __forceinline__ bool wait(Smem &sm, uint64_t *bar, uint32_t parity) {
  if (try_wait_hint(bar, parity)) return true;
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (*reinterpret_cast<volatile int *>(&sm.abort)) return false;
    if (try_wait_hint(bar, parity)) return true;
  }
  *reinterpret_cast<volatile int *>(&sm.abort) = 1;
  atomicExch(&g_status, 1);
  return false;
}

// V' tile row (= O column) of channel ch: 32 (ch % 4) + ch / 4, so that the 32 lanes of a record (4 channels each) write
// rows with all residues mod 8 -- conflict-free under the swizzle; the epilogue undoes it
__device__ __forceinline__ int vrow(int ch) { return 32 * (ch & 3) + (ch >> 2); }
// byte address of the 16-byte chunk holding K-extent element k0 (a multiple of 8) of tile row r
__device__ __forceinline__ uint8_t *chunk_at(uint8_t *tile, int r, int k0) {
  const int slab = k0 >> 6, c = (k0 & 63) >> 3;
  return tile + slab * SLAB + r * 128 + ((c ^ (r & 7)) << 4);
}

// ---- record unpacking (the slot maps of include/mlops_fbla.h) --------------------------------------------------------------
template <int BITS> __device__ __forceinline__ void lane_words(const uint8_t *rec, int tensor, int lane, uint32_t *W) {
#pragma unroll
  for (int w = 0; w < 2 * BITS; ++w) W[w] = lds32(rec + word_offset(BITS, tensor, lane, w));
}
// four small unsigned integers (bytes of x, each < 1024) as two packed FP16 pairs: 0x6400 | b is 1024 + b
__device__ __forceinline__ uint2 bytes_to_half4(uint32_t x) {
  const uint32_t lo = __byte_perm(x, 0x64646464u, 0x7170), hi = __byte_perm(x, 0x64646464u, 0x7372);  // (b1 | 0x64 << 8) << 16 | b0 | 0x64 << 8
  const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6400));
  const __half2 a = __hsub2(*reinterpret_cast<const __half2 *>(&lo), bias), b = __hsub2(*reinterpret_cast<const __half2 *>(&hi), bias);
  return make_uint2(*reinterpret_cast<const uint32_t *>(&a), *reinterpret_cast<const uint32_t *>(&b));
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&h);
}

// FP16 pairs (code as FP16) * step + base, one rounding
__device__ __forceinline__ uint32_t hfma2_bits(uint32_t code2, __half2 step, __half2 base) {
  const __half2 r = __hfma2(*reinterpret_cast<const __half2 *>(&code2), step, base);
  return *reinterpret_cast<const uint32_t *>(&r);
}
__device__ __forceinline__ float2 bf2(uint32_t w) { return make_float2(bf_lo(w), bf_hi(w)); }
// pairs of FP32 operations: the packed FP32x2 instructions of sm_100
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }

template <int CB, int FB>
__device__ __forceinline__ void attend_tc_item(const fbla_k_prefill &a, uint8_t *smem_raw) {
  smem_raw += (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;  // (an offset, not a rebuilt pointer: the address space stays known)
  Smem &sm = *reinterpret_cast<Smem *>(smem_raw);
  constexpr int RC = record_bytes(CB), RF = record_bytes(FB);
  const int tid = FBLA_POS::tid(), warp = tid >> 5, lane = tid & 31;
  const int bh = FBLA_POS::y(), b = bh / a.kv_heads, kh = bh - b * a.kv_heads, qg = a.q_heads / a.kv_heads;
  const int n0 = (a.length ? FBLA_POS::ro(a.length + (a.lstride ? b : 0)) : 0) + a.n0;
  const int count = a.dcount ? FBLA_POS::ro(a.dcount) : a.count, n1 = n0 + count;
  // the last tiles attend to the most groups: they are taken first, so that the grid's tail is made of short CTAs
  const int rows = count * qg, r0 = (FBLA_POS::nx() - 1 - FBLA_POS::x()) * CTA_ROWS;
  if (r0 >= rows || rows < a.tc_min_rows) return;  // (CTA-uniform; a short device count is the warp-per-row pass's work)
  const int last_row = min(r0 + CTA_ROWS, rows) - 1;
  const int own_min = (n0 + r0 / qg) / G, own_max = (n0 + last_row / qg) / G;
  // passes: closed groups 1 .. own_max - 1, then the BF16 groups: 0 and the rows' own groups
  const int n_closed = max(own_max - 1, 0), own_lo = max(own_min, 1);
  const int n_pass = n_closed + 1 + max(own_max - own_lo + 1, 0);
  auto pass_group = [&](int n, bool &closed) {
    closed = n < n_closed;
    return closed ? 1 + n : n == n_closed ? 0 : own_lo + (n - n_closed - 1);
  };

  if (tid == 0) {
    mbar_init(&sm.bar_raw, 1); mbar_init(&sm.bar_meta[0], 1); mbar_init(&sm.bar_meta[1], 1); mbar_init(&sm.bar_k, PT); mbar_init(&sm.bar_v, PT);
    for (int x = 0; x < 2; ++x) { mbar_init(&sm.bar_q[x], 256); mbar_init(&sm.bar_s[x], 1); mbar_init(&sm.bar_p[x], 256); mbar_init(&sm.bar_o[x], 1); }
    sm.abort = 0;
    mbar_init_fence();
  }
  if (warp == ISSUER_WARP) {  // all 512 columns of tensor memory: S of tile x at 128 x, O at 256 + 128 x
    // (the allocation permit is kept: an executor may run further tensor-core items on this CTA, and a CTA that has given
    // its permit up may not allocate again)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(512) : "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const size_t head = (size_t)bh * a.hs, eh = (size_t)bh * G * D, ih = (size_t)bh * a.count * D;
  // the BF16 row of position tp: the chunk, the sink window, or the window of the group that was open before the chunk
  auto token_row = [&](int tp, const uint16_t *in, const uint16_t *sink, const uint16_t *open) -> const uint16_t * {
    return tp >= n0 ? in + ih + (size_t)(tp - n0) * D : tp < G ? sink + eh + (size_t)tp * D : open + eh + (size_t)(tp - (n0 - 1) / G * G) * D;
  };

  if (warp == ISSUER_WARP) {
    // ================= issuer: bulk copies of the raw groups, the products =================
    if (lane == 0) {
      auto fetch = [&](int g) {
        const size_t unit = head + (size_t)g * a.gs;
        mbar_expect_tx(&sm.bar_raw, SBG * (RC + RF));
        bulk_g2s(sm.raw, a.c.coarse + unit * SBG * RC, SBG * RC, &sm.bar_raw);
        bulk_g2s(sm.raw + SBG * RC, a.c.fine + unit * SBG * RF, SBG * RF, &sm.bar_raw);
      };
      auto fetch_meta = [&](int c) {  // closed pass c = group 1 + c: 1 KiB, two passes ahead of its use
        mbar_expect_tx(&sm.bar_meta[c & 1], 1024);
        bulk_g2s(sm.meta[c & 1], reinterpret_cast<const uint8_t *>(a.c.meta) + (head + (size_t)(1 + c) * a.gs) * 1024, 1024, &sm.bar_meta[c & 1]);
      };
      if (n_closed > 0) { fetch(1); fetch_meta(0); }
      if (n_closed > 1) fetch_meta(1);
      for (int n = 0; n < n_pass; ++n) {
        bool closed;
        pass_group(n, closed);
        const uint32_t ph = n & 1, idesc = closed ? IDESC_F16 : IDESC_BF16;
        // Both tiles' S first, then both tiles' O: the tiles run in step (holding tile 1 back by half a pass, so that one
        // tile quantises while the other exponentiates, measured slower: each tile then waits for the other's operands)
        bool ok = wait(sm, &sm.bar_k, ph);
        for (int x = 0; x < 2 && ok; ++x) {
          if (!(ok = wait(sm, &sm.bar_q[x], ph))) break;
          tc_fence_after();
          const uint8_t *qop = closed ? sm.qp[x] : sm.q[x];
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) mma_f16(tmem + 128 * x, smem_desc(qop, kk >> 2, kk & 3), smem_desc(sm.k, kk >> 2, kk & 3), idesc, kk > 0);
          mma_commit(&sm.bar_s[x]);
        }
        if (!ok || !wait(sm, &sm.bar_v, ph)) break;
        if (n + 1 < n_closed) fetch(2 + n);  // the raw buffer has been consumed: the next closed group's records
        if (n + 2 < n_closed) fetch_meta(n + 2);  // (this pass's metadata has been consumed too)
        for (int x = 0; x < 2 && ok; ++x) {
          if (!(ok = wait(sm, &sm.bar_p[x], ph))) break;
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)  // P' of token block kk: eight columns inside the tile's S columns (see the row threads)
            mma_f16_ts(tmem + 256 + 128 * x, tmem + 128 * x + 64 * (kk >> 2) + 8 * (kk & 3), smem_desc(sm.v, kk >> 2, kk & 3), IDESC_F16, n > 0 || kk > 0);
          mma_commit(&sm.bar_o[x]);
        }
        if (!ok) break;
      }
    }
  } else if (warp >= PRODUCER_WARP0) {
    // ================= operand producers =================
    const int pt = tid - 32 * PRODUCER_WARP0;  // 0 .. PT - 1
    const int l = pt & 31;
    int raw_uses = 0;
    for (int n = 0; n < n_pass; ++n) {
      bool closed;
      const int g = pass_group(n, closed);
      const uint32_t prev = (n - 1) & 1;
      // ---- Kop (free once both tiles' S of the previous pass are complete) ----
      if (n > 0 && (!wait(sm, &sm.bar_s[0], prev) || !wait(sm, &sm.bar_s[1], prev))) break;
      if (closed) {
        if (!wait(sm, &sm.bar_meta[n & 1], (uint32_t)(n >> 1) & 1u)) break;
        if (!wait(sm, &sm.bar_raw, raw_uses++ & 1)) break;
      }
      if (closed) {
        // (record j, lane l): token 16 j + l % 16, channels 64 (l / 16) + 4 s + byte: one 128-byte row of slab l / 16
#pragma unroll 1
        for (int j = pt >> 5; j < SBG; j += PRODUCERS) {
          uint32_t Wc[2 * CB], Wf[2 * FB];
          lane_words<CB>(sm.raw + j * RC, 0, l, Wc);
          lane_words<FB>(sm.raw + SBG * RC + j * RF, 0, l, Wf);
          const int tok = 16 * j + (l & 15);
#pragma unroll
          for (int s2 = 0; s2 < 8; ++s2) {
            const uint2 x = bytes_to_half4((slot_value<CB>(Wc, 2 * s2) << FB) | slot_value<FB>(Wf, 2 * s2));
            const uint2 y = bytes_to_half4((slot_value<CB>(Wc, 2 * s2 + 1) << FB) | slot_value<FB>(Wf, 2 * s2 + 1));
            *reinterpret_cast<uint4 *>(chunk_at(sm.k, tok, 64 * (l >> 4) + 8 * s2)) = make_uint4(x.x, x.y, y.x, y.y);
          }
        }
      } else {
        for (int e = pt; e < G * 16; e += PT) {  // BF16 group g: K rows as they are
          const int tk = e >> 4, c = e & 15, tp = g * G + tk;
          const uint4 kw = tp < n1 ? __ldcg(reinterpret_cast<const uint4 *>(token_row(tp, a.k, a.c.sink_k, a.c.open_k)) + c) : make_uint4(0u, 0u, 0u, 0u);
          *reinterpret_cast<uint4 *>(chunk_at(sm.k, tk, 8 * c)) = kw;
        }
      }
      fence_async_smem();
      mbar_arrive(&sm.bar_k);
      // ---- V' (free once both tiles' O products of the previous pass are complete) ----
      if (n > 0 && (!wait(sm, &sm.bar_o[0], prev) || !wait(sm, &sm.bar_o[1], prev))) break;
      if (closed) {
        // (record j, lane l): channels 4 l + cc, tokens 16 j + 4 quad + byte, value base + step * code in FP16 arithmetic
        const uint4 vm = lds128(sm.meta[n & 1] + 512 + 16 * l);
        const __half2 vb[4] = {__float2half2_rn(bf_lo(vm.x)), __float2half2_rn(bf_hi(vm.x)), __float2half2_rn(bf_lo(vm.y)), __float2half2_rn(bf_hi(vm.y))};
        const __half2 vs[4] = {__float2half2_rn(bf_lo(vm.z)), __float2half2_rn(bf_hi(vm.z)), __float2half2_rn(bf_lo(vm.w)), __float2half2_rn(bf_hi(vm.w))};
#pragma unroll 1
        for (int j = pt >> 5; j < SBG; j += PRODUCERS) {
          uint32_t Wc[2 * CB], Wf[2 * FB];
          lane_words<CB>(sm.raw + j * RC, 1, l, Wc);
          lane_words<FB>(sm.raw + SBG * RC + j * RF, 1, l, Wf);
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t h[8];
#pragma unroll
            for (int quad = 0; quad < 4; ++quad) {
              const uint2 c4 = bytes_to_half4((slot_value<CB>(Wc, v_slot_of(CB, cc, quad)) << FB) | slot_value<FB>(Wf, v_slot_of(FB, cc, quad)));
              h[2 * quad] = hfma2_bits(c4.x, vs[cc], vb[cc]);
              h[2 * quad + 1] = hfma2_bits(c4.y, vs[cc], vb[cc]);
            }
            *reinterpret_cast<uint4 *>(chunk_at(sm.v, 32 * cc + l, 16 * j)) = make_uint4(h[0], h[1], h[2], h[3]);
            *reinterpret_cast<uint4 *>(chunk_at(sm.v, 32 * cc + l, 16 * j + 8)) = make_uint4(h[4], h[5], h[6], h[7]);
          }
        }
      } else {
        for (int e = pt; e < G * 16; e += PT) {  // V rows converted to FP16 and transposed (tokens along the K extent)
          const int tk = e >> 4, c = e & 15, tp = g * G + tk;
          const uint4 vw = tp < n1 ? __ldcg(reinterpret_cast<const uint4 *>(token_row(tp, a.v, a.c.sink_v, a.c.open_v)) + c) : make_uint4(0u, 0u, 0u, 0u);
          const uint32_t w4[4] = {vw.x, vw.y, vw.z, vw.w};
#pragma unroll
          for (int x = 0; x < 8; ++x) {
            const float f = (x & 1) ? bf_hi(w4[x >> 1]) : bf_lo(w4[x >> 1]);
            *reinterpret_cast<__half *>(chunk_at(sm.v, vrow(8 * c + x), tk & ~7) + 2 * (tk & 7)) = __float2half_rn(f);
          }
        }
      }
      fence_async_smem();
      mbar_arrive(&sm.bar_v);
    }
  } else {
    // ================= row threads: qhat, softmax, P', output =================
    // Softmax: two threads per row (warps w and w + 8 share a tensor-memory lane quadrant): thread hf owns tokens
    // 64 hf .. + 63 of S and P' (slab hf of the P' tile) and O columns 64 hf .. + 63; the pair meets on a named barrier to
    // exchange the pass maximum. qhat: a different map -- a warp takes 16 rows of its tile, two rows at a time: lane
    // (c = lane % 16, lane / 16) holds channels 8 c .. + 7 of one row, with the group's steps and bases of those channels
    // in registers for the whole pass; max |z| and the bias dot product are reduced over the 16 lanes of a row. That
    // keeps shared-memory traffic (the limiter of a thread-per-row quantiser, which re-reads steps and bases per row)
    // at one load and one store per row chunk. A thread never leaves the pass loop early: after an abort every wait
    // returns at once, so both threads of a pair still reach every named barrier.
    const int hf = warp >> 3, X = (warp >> 2) & 1, r = 32 * (warp & 3) + lane, R = r0 + ROWS * X + r;
    const int pair_bar = 1 + (warp & 7);
    auto pair_sync = [&] { asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory"); };
    const bool valid = R < rows;
    const int i = valid ? R / qg : 0, hq = kh * qg + (valid ? R - i * qg : 0), pos = n0 + i, own = pos / G;
    const int tile_last = min(r0 + ROWS * X + ROWS, rows) - 1;                 // the tile's last row, if it has any
    const int tile_own = tile_last >= r0 + ROWS * X ? (n0 + tile_last / qg) / G : -1;  // closed group g concerns the tile iff g < tile_own
    // quantiser lane: chunk qc of rows qrow0 + 2 it, it = 0 .. 7 (qrow0 % 8 is 0 or 1, so (row % 8) = (2 it) | (qrow0 & 1))
    const int qc = lane & 15, qrow0 = 16 * ((warp & 3) + 4 * hf) + (lane >> 4);
    const uint32_t qoff = (qc >> 3) * SLAB + qrow0 * 128, qcx = (uint32_t)((qc & 7) ^ (qrow0 & 1)) << 4;
    const uint32_t qmask = (lane & 16) ? 0xffff0000u : 0x0000ffffu;
    // the rows' q into the BF16 Q tile (rows past the end: zeros), by the same map
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int rowq = qrow0 + 2 * it, Rq = r0 + ROWS * X + rowq;
      uint4 w = make_uint4(0u, 0u, 0u, 0u);
      if (Rq < rows) {
        const int iq = Rq / qg;
        w = __ldg(reinterpret_cast<const uint4 *>(a.q + ((size_t)(b * a.q_heads + kh * qg + (Rq - iq * qg)) * a.count + iq) * D) + qc);
      }
      *reinterpret_cast<uint4 *>(sm.q[X] + qoff + 2 * it * 128 + (qcx ^ (((2 * it) & 7) << 4))) = w;
    }
    float m_run = -FBLA_INF, l_run = 0.f;  // l_run: this thread's tokens only
    const uint32_t lane_base = (uint32_t)(32 * (warp & 3)) << 16;
    const uint32_t tmem_s = tmem + 128 * X + 64 * hf + lane_base, tmem_o = tmem + 256 + 128 * X + 64 * hf + lane_base;
    bool ok = true;
    // Qop of pass np into the qhat tile (free once the S product of pass np - 1 is complete), then the tile's arrival for it
    auto prepare = [&](int np) {
      bool closed;
      const int g = pass_group(np, closed);
      if (closed) {
        // the group's metadata (fetched two passes ahead; it is replaced only after both tiles have arrived for this pass)
        ok &= __all_sync(FULL, wait(sm, &sm.bar_meta[np & 1], (uint32_t)(np >> 1) & 1u));
        if (g < tile_own) {
      // qhat for this group: z = q * step_K, r = fl(127 / max|z|), rint(z r) written as FP16; four rows per batch, with
      // every load ahead of the arithmetic and every store behind it, so that the rows' dependency chains overlap
      // K bases and steps of channels 8 qc .. 8 qc + 7: per four channels, four BF16 bases then four BF16 steps
      const uint4 ma = lds128(sm.meta[np & 1] + 32 * qc), mb = lds128(sm.meta[np & 1] + 32 * qc + 16);
      const float4 b0 = make_float4(bf_lo(ma.x), bf_hi(ma.x), bf_lo(ma.y), bf_hi(ma.y)), s0 = make_float4(bf_lo(ma.z), bf_hi(ma.z), bf_lo(ma.w), bf_hi(ma.w));
      const float4 b1 = make_float4(bf_lo(mb.x), bf_hi(mb.x), bf_lo(mb.y), bf_hi(mb.y)), s1 = make_float4(bf_lo(mb.z), bf_hi(mb.z), bf_lo(mb.w), bf_hi(mb.w));
      const float2 mg = splat(MAGICF), ng = splat(-MAGICF);
      const float sl127 = __fmul_rn(a.sl, 1.f / 127.f);
      const bool h3 = lane & 8;
#pragma unroll
      for (int bt = 0; bt < 4; ++bt) {  // two rows per batch; their z = q * step stay in registers for the second sweep
        float2 z[2][4];
        uint32_t off[2];
        float amax[2], dot[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {  // the lane's share of max |z| and of the bias dot product
          const int it = 2 * bt + k;
          off[k] = qoff + 2 * it * 128 + (qcx ^ (((2 * it) & 7) << 4));
          const uint4 qv = *reinterpret_cast<const uint4 *>(sm.q[X] + off[k]);
          const float2 q0 = bf2(qv.x), q1 = bf2(qv.y), q2 = bf2(qv.z), q3 = bf2(qv.w);
          z[k][0] = mul2(q0, make_float2(s0.x, s0.y)); z[k][1] = mul2(q1, make_float2(s0.z, s0.w));
          z[k][2] = mul2(q2, make_float2(s1.x, s1.y)); z[k][3] = mul2(q3, make_float2(s1.z, s1.w));
          amax[k] = fmaxf(fmaxf(fmaxf(fabsf(z[k][0].x), fabsf(z[k][0].y)), fmaxf(fabsf(z[k][1].x), fabsf(z[k][1].y))),
                          fmaxf(fmaxf(fabsf(z[k][2].x), fabsf(z[k][2].y)), fmaxf(fabsf(z[k][3].x), fabsf(z[k][3].y))));
          float2 d2 = fma2(q0, make_float2(b0.x, b0.y), mul2(q1, make_float2(b0.z, b0.w)));
          d2 = fma2(q2, make_float2(b1.x, b1.y), fma2(q3, make_float2(b1.z, b1.w), d2));
          dot[k] = d2.x + d2.y;
        }
        // over the 16 lanes of a row: the maxima by reductions (nonnegative floats order as integers), the dot products by
        // a merging butterfly that leaves row b3 of the batch in the lanes with bit 3 = b3
#pragma unroll
        for (int k = 0; k < 2; ++k) amax[k] = __uint_as_float(__reduce_max_sync(qmask, __float_as_uint(amax[k])));
        float dsum = (h3 ? dot[1] : dot[0]) + __shfl_xor_sync(FULL, h3 ? dot[0] : dot[1], 8);
        dsum += __shfl_xor_sync(FULL, dsum, 4);
        dsum += __shfl_xor_sync(FULL, dsum, 2);
        dsum += __shfl_xor_sync(FULL, dsum, 1);
        if (!(lane & 7)) sm.qbias[np & 1][X][qrow0 + 2 * (2 * bt + ((lane >> 3) & 1))] = __fmul_rn(dsum, a.sl);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const float am = amax[k];
          float rc;
          asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rc) : "f"(am));
          rc = fmaf(fmaf(-am, rc, 1.f), rc, rc);
          const float q0_ = __fmul_rn(127.f, rc);
          // rint(z r) as the exact float (t - 1.5 * 2^23), then FP16 (an integer of magnitude <= 127: exact)
          const float2 rr2 = splat(am > 0.f ? fmaf(fmaf(-am, q0_, 127.f), rc, q0_) : 0.f);
          const float2 t0 = add2(fma2(z[k][0], rr2, mg), ng), t1 = add2(fma2(z[k][1], rr2, mg), ng);
          const float2 t2 = add2(fma2(z[k][2], rr2, mg), ng), t3 = add2(fma2(z[k][3], rr2, mg), ng);
          *reinterpret_cast<uint4 *>(sm.qp[X] + off[k]) = make_uint4(pack_half2(t0.x, t0.y), pack_half2(t1.x, t1.y), pack_half2(t2.x, t2.y), pack_half2(t3.x, t3.y));
          if (qc == 0) sm.qscale[np & 1][X][qrow0 + 2 * (2 * bt + k)] = __fmul_rn(am, sl127);
        }
      }
        }
      }
      fence_async_smem();
      mbar_arrive(&sm.bar_q[X]);
    };
    prepare(0);
    // Per pass: the softmax of S(n), whose P' goes back into tensor memory over the S columns it came from -- row r in lane
    // r, tokens 2 c and 2 c + 1 of this thread's 64 in column c of its 64 S columns, so the O product takes P' as its
    // tensor-memory operand and no shared memory is written -- then Qop of pass n + 1, while the O product of pass n runs.
    // Products execute in the order they were issued: S(n + 1) overwrites P'(n) only after O(n) has read it.
    for (int n = 0; n < n_pass; ++n) {
      bool closed;
      const int g = pass_group(n, closed);
      const bool include = valid && (closed ? g < own : (g == 0 || g == own));
      const bool any = __any_sync(FULL, include);
      // S(n) is complete, and with it every product issued before: O of pass n - 1 is stable
      ok &= __all_sync(FULL, wait(sm, &sm.bar_s[X], n & 1));
      tc_fence_after();
      // softmax of the row over the pass's 128 tokens, by 16-token blocks; P' = fp16(2^(m_block - m_row) p)
      const int lim = (include ? (closed ? G : pos - g * G) : -1) - 64 * hf;  // this thread's tokens 0 .. lim are attended
      const float mul1 = closed ? sm.qscale[n & 1][X][r] : a.sl, add1 = closed ? sm.qbias[n & 1][X][r] : 0.f;  // score = mul x + add, monotonic in x (mul >= 0)
      // sweep 1: the block maxima, from the raw sums
      float mbk[4];
      if (any) {
#pragma unroll
        for (int cq = 0; cq < 2; ++cq) {
          uint32_t x[32];
          tmem_ld32(tmem_s + 32 * cq, x);
#pragma unroll
          for (int hb = 0; hb < 2; ++hb) {
            const int t0 = 32 * cq + 16 * hb;
            float xm = -FBLA_INF;
            if (lim >= t0 + 15) {
#pragma unroll
              for (int t = 0; t < 16; t += 2) xm = fmaxf(xm, fmaxf(__uint_as_float(x[16 * hb + t]), __uint_as_float(x[16 * hb + t + 1])));
            } else {
#pragma unroll
              for (int t = 0; t < 16; ++t) if (t0 + t <= lim) xm = fmaxf(xm, __uint_as_float(x[16 * hb + t]));
            }
            mbk[2 * cq + hb] = xm == -FBLA_INF ? -FBLA_INF : fmaf(mul1, xm, add1);  // -inf: a block without attended tokens
          }
        }
        sm.ex2[X][r][hf] = fmaxf(fmaxf(mbk[0], mbk[1]), fmaxf(mbk[2], mbk[3]));
      }
      pair_sync();
      if (!any) {  // (warp-uniform, and the same in both warps of the pair) nothing to attend: P' = 0
        const uint32_t zero[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_st8(tmem_s + 8 * c, zero);
      } else {
        const float2 e = *reinterpret_cast<const float2 *>(&sm.ex2[X][r][0]);
        const float mp = fmaxf(e.x, e.y);
        // the row's running maximum moves only when a block exceeds it by more than 2^8 (rare): its sums and its O row in
        // tensor memory are rescaled. Tensor-memory accesses are warp-wide, so the whole warp takes part (rows that do
        // not move scale by 1); both threads of a row decide alike and each rescales its own 64 columns.
        const bool need = mp > m_run + 8.f;
        if (__any_sync(FULL, need)) {
          const float al = need ? ex2(m_run - mp) : 1.f;  // 0 on the row's first attended block
          if (n > 0) {
#pragma unroll 1
            for (int oc = 0; oc < 2; ++oc) {
              uint32_t o[32];
              tmem_ld32(tmem_o + 32 * oc, o);
#pragma unroll
              for (int z = 0; z < 32; ++z) o[z] = __float_as_uint(__uint_as_float(o[z]) * al);
              tmem_st32(tmem_o + 32 * oc, o);
            }
          }
          if (need) { l_run *= al; m_run = mp; }
        }
        // sweep 2: the integer P blocks times their weights
        const float2 mul = splat(mul1), c255 = splat(255.f), mg = splat(MAGICF), ng = splat(-MAGICF);
        float2 lacc = make_float2(0.f, 0.f);
#pragma unroll
        for (int cq = 0; cq < 2; ++cq) {
          uint32_t x[32];
          tmem_ld32(tmem_s + 32 * cq, x);
#pragma unroll
          for (int hb = 0; hb < 2; ++hb) {
            const int t0 = 32 * cq + 16 * hb;
            const float mb = mbk[2 * cq + hb];
            // score - block maximum in one step: mul x + (add - m_block)
            const float2 addm = splat(mb == -FBLA_INF ? add1 : add1 - mb), w2 = splat(mb == -FBLA_INF ? 0.f : ex2(mb - m_run));
            float2 sc[8];
#pragma unroll
            for (int t = 0; t < 8; ++t)
              sc[t] = fma2(make_float2(__uint_as_float(x[16 * hb + 2 * t]), __uint_as_float(x[16 * hb + 2 * t + 1])), mul, addm);
            if (lim < t0 + 15) {  // the causal edge (or a row that does not attend to this group)
#pragma unroll
              for (int t = 0; t < 8; ++t) {
                if (t0 + 2 * t > lim) sc[t].x = -FBLA_INF;
                if (t0 + 2 * t + 1 > lim) sc[t].y = -FBLA_INF;
              }
            }
            uint32_t h[8];
            float2 acc = make_float2(0.f, 0.f);
#pragma unroll
            for (int t = 0; t < 8; ++t) {
              const float2 pf = add2(fma2(make_float2(ex2(sc[t].x), ex2(sc[t].y)), c255, mg), ng);
              acc = add2(acc, pf);
              const float2 pw = mul2(pf, w2);
              h[t] = pack_half2(pw.x, pw.y);
            }
            lacc = fma2(acc, w2, lacc);
            tmem_st8(tmem_s + 16 * cq + 8 * hb, h);  // (over S columns this thread has already taken into registers)
          }
        }
        l_run += lacc.x + lacc.y;
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&sm.bar_p[X]);
      if (n + 1 < n_pass) prepare(n + 1);
    }
    ok &= __all_sync(FULL, wait(sm, &sm.bar_o[X], (n_pass - 1) & 1));
    tc_fence_after();
    pair_sync();  // (the partner has read the last pass's exchange)
    sm.ex2[X][r][hf] = l_run;
    pair_sync();
    {
      // O column 32 cc + l is channel 4 l + cc: through the row's (now free) P' row as BF16 in channel order, then out.
      // This thread: O columns 64 hf .. + 63 (cc = 2 hf, 2 hf + 1); then it copies chunks 8 hf .. + 7 of the row.
      const float inv = 1.f / (sm.ex2[X][r][0] + sm.ex2[X][r][1]);
      uint16_t *stage = reinterpret_cast<uint16_t *>(sm.qp[X] + r * 256);  // 256 bytes per row, private to the pair
#pragma unroll 1
      for (int cu = 0; cu < 2; ++cu) {
        const int cc = 2 * hf + cu;
        uint32_t o[32];
        tmem_ld32(tmem_o + 32 * cu, o);
#pragma unroll
        for (int l = 0; l < 32; ++l)  // channel 4 l + cc: 16-byte chunk l / 2 of the row, stored at chunk (l / 2) ^ (r % 16)
          stage[8 * ((l >> 1) ^ (r & 15)) + 4 * (l & 1) + cc] = f32_to_bf16(__uint_as_float(o[l]) * inv);
      }
      pair_sync();
      if (valid) {  // (after a wait that gave up: NaN, so that the failure shows in the caller's data)
        uint16_t *orow = a.out + (size_t)(b * a.q_heads + hq) * a.out_hs + (size_t)i * a.out_ts;
        const uint4 nan4 = make_uint4(0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u);
#pragma unroll
        for (int c = 8 * hf; c < 8 * hf + 8; ++c) reinterpret_cast<uint4 *>(orow)[c] = ok ? reinterpret_cast<const uint4 *>(stage)[c ^ (r & 15)] : nan4;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == ISSUER_WARP) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
  if (tid == 0) {  // no live barrier object is left behind: an executor may run another item on this CTA next
    mbar_inval(&sm.bar_raw); mbar_inval(&sm.bar_meta[0]); mbar_inval(&sm.bar_meta[1]); mbar_inval(&sm.bar_k); mbar_inval(&sm.bar_v);
    for (int x = 0; x < 2; ++x) { mbar_inval(&sm.bar_q[x]); mbar_inval(&sm.bar_s[x]); mbar_inval(&sm.bar_p[x]); mbar_inval(&sm.bar_o[x]); }
  }
}

}  // namespace tc
}  // namespace fbla
