// Register fragments of the integer tensor-core products, built straight from packed records in shared memory.
//
// A record (one plane, 16 tokens) is staged in shared memory byte for byte as it lies in the cache. The products run
// with TOKENS on the M axis for scores (S^T = K_codes x qhat^T) and CHANNELS on the M axis for values
// (O^T = V_codes^T x P^T), so a record's "slot" -- four codes in the four bytes of a 32-bit word -- is exactly one
// A-fragment register once it is masked; nothing is ever unpacked to bytes in memory. A mask leaves the codes times a
// fixed power of two ("class"); products of one class go to their own s32 accumulator (scores) or their own row
// (values) and the factor is folded into the FP32 epilogue.
//
// Thread T of a warp: gid = T / 4 (fragment row / column), tig = T % 4 (k block). Scores: thread (gid, tig) supplies,
// for tokens gid and gid + 8, the slots whose word index is tig. Values: it supplies token quad tig of the channels of
// record lanes 8 u + gid, u = 0..3.
#pragma once
#include "fbla_device.cuh"

namespace fbla {

__device__ __forceinline__ void mma_u8u8_k16_from(uint32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0, uint32_t c) {
  asm("mma.sync.aligned.m16n8k16.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a0), "r"(a1), "r"(b0), "r"(c));
}
__device__ __forceinline__ void mma_u8u8_k16(uint32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm("mma.sync.aligned.m16n8k16.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(b0));
}

// ---- qhat fragments -------------------------------------------------------------------------------------------------
// qst: 8 rows (fragment columns: queries, rows >= QG zero) of 128 s8 codes in channel order, row stride QST_ROW bytes
// (36 words: 4 * gid + word is then conflict-free over a warp).
constexpr int QST_ROW = 144;
__device__ __forceinline__ uint32_t qword(const uint8_t *qst, int gid, int w) { return lds32(qst + QST_ROW * gid + 4 * w); }

// B[8]: the qhat words matching the A slots of kfrag<BITS> below (pairs: k blocks tig and 4 + tig of one product)
template <int BITS> __device__ __forceinline__ void qhat_frag(const uint8_t *qst, int gid, int tig, uint32_t (&B)[8]) {
  if (BITS == 3) {
    const int e = ((tig & 1) ? 10 : 4) + (tig >> 1);
    B[0] = qword(qst, gid, tig);      B[1] = qword(qst, gid, 16 + tig);       // slots tig (bits 0-2)
    B[2] = qword(qst, gid, 6 + tig);  B[3] = qword(qst, gid, 22 + tig);       // slots 6 + tig (bits 3-5, class x8)
    B[4] = qword(qst, gid, 12 + tig); B[5] = qword(qst, gid, 28 + tig);       // slots 12 + tig (split over two words)
    B[6] = qword(qst, gid, e);        B[7] = qword(qst, gid, 16 + e);         // slots 4, 5 (even tig) / 10, 11 (odd tig)
  } else {  // 4 and 2 bits: word 4 m + tig, m = 0..7 (m < 4: channels 0..63, m >= 4: 64..127)
#pragma unroll
    for (int m = 0; m < 8; ++m) B[m] = qword(qst, gid, 4 * m + tig);
  }
}

// ---- scores: x[i] = sum_c qhat[c] * plane_value[token][c], i = (gid, 2 tig), (gid, 2 tig + 1), (gid + 8, 2 tig), (gid + 8, 2 tig + 1)
template <int BITS> __device__ __forceinline__ void qk_tile(const uint8_t *rec, int gid, int tig, const uint32_t (&B)[8], float (&x)[4]) {
  const uint8_t *p0 = rec + 16 * gid + 4 * tig, *p1 = p0 + 128;  // tokens gid, gid + 8
  if (BITS == 4) {
    const uint32_t a = lds32(p0), a8 = lds32(p1), b = lds32(p0 + 512), b8 = lds32(p1 + 512);          // half 0: W[tig], W[4 + tig]
    const uint32_t c = lds32(p0 + 256), c8 = lds32(p1 + 256), d = lds32(p0 + 768), d8 = lds32(p1 + 768);  // half 1
    constexpr uint32_t L = 0x0f0f0f0fu, H = 0xf0f0f0f0u;
    uint32_t lo[4], hi[4];
    mma_u8s8_k32_from(lo, a & L, a8 & L, b & L, b8 & L, B[0], B[1], MAGIC);
    mma_u8s8_k32_from(hi, a & H, a8 & H, b & H, b8 & H, B[2], B[3], MAGIC);
    mma_u8s8_k32(lo, c & L, c8 & L, d & L, d8 & L, B[4], B[5]);
    mma_u8s8_k32(hi, c & H, c8 & H, d & H, d8 & H, B[6], B[7]);
    const float2 x01 = __ffma2_rn(isum2(hi[0], hi[1]), splat(1.f / 16), isum2(lo[0], lo[1]));
    const float2 x23 = __ffma2_rn(isum2(hi[2], hi[3]), splat(1.f / 16), isum2(lo[2], lo[3]));
    x[0] = x01.x; x[1] = x01.y; x[2] = x23.x; x[3] = x23.y;
  } else if (BITS == 2) {
    const uint32_t a = lds32(p0), a8 = lds32(p1), c = lds32(p0 + 256), c8 = lds32(p1 + 256);
    uint32_t acc[4][4];
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const uint32_t M = 0x03030303u << (2 * m);
      mma_u8s8_k32_from(acc[m], a & M, a8 & M, c & M, c8 & M, B[m], B[4 + m], MAGIC);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
      x[i] = fmaf(isum(acc[3][i]), 1.f / 64, fmaf(isum(acc[2][i]), 1.f / 16, fmaf(isum(acc[1][i]), 1.f / 4, isum(acc[0][i]))));
  } else {
    const int sh = 4 + (tig & 1), se = 3 * (tig & 1);
    const uint8_t *q0 = rec + 1024 + 16 * gid + 4 * (tig >> 1), *q1 = q0 + 128;  // W[4 + tig / 2]: half 0, half 1 at + 8
    const uint32_t a = lds32(p0), a8 = lds32(p1), c = lds32(p0 + 256), c8 = lds32(p1 + 256);
    const uint32_t e = lds32(q0), e8 = lds32(q1), f = lds32(q0 + 8), f8 = lds32(q1 + 8);
    constexpr uint32_t L = 0x07070707u, M = 0x38383838u, T2 = 0x03030303u, T1 = 0x04040404u;
    uint32_t lo[4], mid[4];
    mma_u8s8_k32_from(lo, a & L, a8 & L, c & L, c8 & L, B[0], B[1], MAGIC);
    mma_u8s8_k32_from(mid, a & M, a8 & M, c & M, c8 & M, B[2], B[3], MAGIC);
    mma_u8s8_k32(lo, ((a >> 6) & T2) | ((e >> sh) & T1), ((a8 >> 6) & T2) | ((e8 >> sh) & T1),
                 ((c >> 6) & T2) | ((f >> sh) & T1), ((c8 >> 6) & T2) | ((f8 >> sh) & T1), B[4], B[5]);
    mma_u8s8_k32(lo, (e >> se) & L, (e8 >> se) & L, (f >> se) & L, (f8 >> se) & L, B[6], B[7]);
    const float2 x01 = __ffma2_rn(isum2(mid[0], mid[1]), splat(1.f / 8), isum2(lo[0], lo[1]));
    const float2 x23 = __ffma2_rn(isum2(mid[2], mid[3]), splat(1.f / 8), isum2(lo[2], lo[3]));
    x[0] = x01.x; x[1] = x01.y; x[2] = x23.x; x[3] = x23.y;
  }
}

// ---- values ---------------------------------------------------------------------------------------------------------
// The four masked slot words (channels 4 l + 0..3 of record lane l, token quad tig) of a BITS-plane record's V half.
// Channel cc carries the factor 1 / v_unscale<BITS>(cc).
template <int BITS> __device__ __forceinline__ void v_slots(const uint8_t *rec, int l, int tig, uint32_t (&v)[4]) {
  if (BITS == 4) {
    const uint2 y = lds64(rec + 1024 + 512 * (tig >> 1) + 16 * l + 8 * (tig & 1));
    v[0] = y.x & 0x0f0f0f0fu; v[1] = y.y & 0x0f0f0f0fu; v[2] = y.x & 0xf0f0f0f0u; v[3] = y.y & 0xf0f0f0f0u;
  } else if (BITS == 2) {
    const uint32_t w = lds32(rec + 512 + 16 * l + 4 * tig);
    v[0] = w & 0x03030303u; v[1] = w & 0x0c0c0c0cu; v[2] = w & 0x30303030u; v[3] = w & 0xc0c0c0c0u;
  } else {
    const uint32_t w = lds32(rec + 512 + 16 * l + 4 * tig);
    const uint2 y = lds64(rec + 1280 + 8 * l);
    const uint32_t wt = (tig >> 1) ? y.y : y.x;  // W[4 + tig / 2]: the top bit of slot 12 + tig
    const uint32_t ws = (tig & 1) ? y.y : y.x;   // W[4 + tig % 2]: slot 4 + tig (tig < 2) or 10 + tig - 2
    v[0] = w & 0x07070707u;
    v[1] = w & 0x38383838u;
    v[2] = (ws >> (3 * (tig >> 1))) & 0x07070707u;
    v[3] = ((w >> 6) & 0x03030303u) | ((wt >> (4 + (tig & 1))) & 0x04040404u);
  }
}
template <int BITS> __host__ __device__ constexpr float v_unscale(int cc) {
  return BITS == 4 ? (cc < 2 ? 1.f : 1.f / 16) : BITS == 2 ? (cc == 0 ? 1.f : cc == 1 ? 1.f / 4 : cc == 2 ? 1.f / 16 : 1.f / 64)
                                                            : (cc == 1 ? 1.f / 8 : 1.f);
}

}  // namespace fbla
