// The attention inputs of new tokens, fused: per head the optional RMSNorm of q and k, the rotary embedding in the
// reference's exact-phase arithmetic, q written for the decode (or the chunk's q / k / v written as the prefill takes
// them), and -- for the one-token step -- k and v stored into the cache's BF16 windows.
//
// Replaces qkv_item / qkv_chunk_item / norm_rope (attention/fbla/src/fbla_qkv.cuh:32-170) and the rotation arithmetic
// of positional/rope/src/rope.cuh:19-37,67-70. Every FP32 step is spelled with explicit round-to-nearest intrinsics
// in the order that defines the result:
//   RMSNorm: a lane holds elements 2 l, 2 l + 1, 64 + 2 l, 65 + 2 l of the head; s = x0 x0, then three FMAs, then the
//     xor butterfly 16 .. 1; r = rsqrt_rn(s / 128 + eps); y = bf16(bf16(x r) w).
//   Phase of position m for frequency f (in turns, f = fh + fl, g = frac(2^16 f) = gh + gl): m = 2^16 a + b,
//     t = frac(a g) + frac(b f) with each product's rounding error recovered by an FMA, reduced to [-1/2, 1/2];
//     (cos, sin) = sincospi(2 t) times the attention factor.
//   Rotation of the pair (i, i + 64): y1 = fma(x1, c, -x2 s), y2 = fma(x2, c, x1 s), one rounding to BF16.
// HBM-bound and tiny (a few KB per head); one CTA per (batch row, KV head) or per (8 positions, KV head).
#pragma once
#include "fbla_device.cuh"
#include "fbla_kernels.h"

namespace fbla {

__device__ __forceinline__ float frac_of_product(float x, float hi, float lo) {  // frac(x (hi + lo)), x an integer below 2^16
  const float p = __fmul_rn(x, hi), err = __fmaf_rn(x, hi, -p);
  return __fadd_rn(__fsub_rn(p, rintf(p)), __fmaf_rn(x, lo, err));
}
__device__ __forceinline__ float2 cos_sin_at(int pos, float4 f, float att) {
  const float a = (float)(pos >> 16), b = (float)(pos & 0xffff);
  const float t = __fadd_rn(frac_of_product(a, f.z, f.w), frac_of_product(b, f.x, f.y));
  float s, c;
  sincospif(__fmul_rn(2.f, __fsub_rn(t, rintf(t))), &s, &c);
  return make_float2(__fmul_rn(c, att), __fmul_rn(s, att));
}

// One head vector through the optional RMSNorm and the rotation. A lane owns the two rotation pairs (2 l, 64 + 2 l) and
// (2 l + 1, 65 + 2 l): `first` = elements 2 l, 2 l + 1, `second` = elements 64 + 2 l, 65 + 2 l, each pair of BF16 in one
// word. cs[i] = (cos, sin) of pair i. Returns the lane's two output words in the same arrangement.
struct LaneQuad { float a0, a1, b0, b1; };  // a: elements 2 l, 2 l + 1; b: their partners 64 further on
__device__ __forceinline__ LaneQuad unpack_quad(uint32_t first, uint32_t second) { return LaneQuad{bf_lo(first), bf_hi(first), bf_lo(second), bf_hi(second)}; }
__device__ __forceinline__ float round_through_bf16(float x) { return bf16_to_f32(f32_to_bf16(x)); }

template <bool NORM>
__device__ __forceinline__ uint2 norm_rotate(const uint16_t *x, const uint16_t *w, float eps, const float2 *cs, int lane) {
  const uint32_t *xw = reinterpret_cast<const uint32_t *>(x);
  LaneQuad v = unpack_quad(__ldg(xw + lane), __ldg(xw + 32 + lane));
  if (NORM) {
    // sum of squares: the lane's four terms chained through FMAs in element order, then the xor butterfly from 16 down
    float sq = __fmaf_rn(v.b1, v.b1, __fmaf_rn(v.b0, v.b0, __fmaf_rn(v.a1, v.a1, __fmul_rn(v.a0, v.a0))));
    for (int stride = 16; stride > 0; stride >>= 1) sq = __fadd_rn(sq, __shfl_xor_sync(FULL, sq, stride));
    const float inv_rms = __frsqrt_rn(__fadd_rn(__fmul_rn(sq, 1.f / D), eps));
    const uint32_t *ww = reinterpret_cast<const uint32_t *>(w);
    const LaneQuad g = unpack_quad(__ldg(ww + lane), __ldg(ww + 32 + lane));
    // two roundings to BF16, as a BF16 norm layer gives: the normalised value, then its product with the weight
    v.a0 = round_through_bf16(__fmul_rn(round_through_bf16(__fmul_rn(v.a0, inv_rms)), g.a0));
    v.a1 = round_through_bf16(__fmul_rn(round_through_bf16(__fmul_rn(v.a1, inv_rms)), g.a1));
    v.b0 = round_through_bf16(__fmul_rn(round_through_bf16(__fmul_rn(v.b0, inv_rms)), g.b0));
    v.b1 = round_through_bf16(__fmul_rn(round_through_bf16(__fmul_rn(v.b1, inv_rms)), g.b1));
  }
  // (a, b) -> (a cos - b sin, b cos + a sin): the sine product rounded first, then one FMA, then BF16
  const float2 p0 = cs[2 * lane], p1 = cs[2 * lane + 1];
  const uint32_t ra0 = f32_to_bf16(__fmaf_rn(v.a0, p0.x, __fmul_rn(-v.b0, p0.y))), rb0 = f32_to_bf16(__fmaf_rn(v.b0, p0.x, __fmul_rn(v.a0, p0.y)));
  const uint32_t ra1 = f32_to_bf16(__fmaf_rn(v.a1, p1.x, __fmul_rn(-v.b1, p1.y))), rb1 = f32_to_bf16(__fmaf_rn(v.b1, p1.x, __fmul_rn(v.a1, p1.y)));
  return make_uint2(ra0 | ra1 << 16, rb0 | rb1 << 16);
}

// ---- one token per sequence: q to q_out, k and v into the windows (the group the position closes has been quantized by
// the close pass launched before this kernel) -----------------------------------------------------------------------------
template <bool NORM>
__device__ __forceinline__ void qkv_token_item(const fbla_k_token &a, uint8_t *smem_raw) {
  __shared__ float2 cs[64];
  const int bh = FBLA_POS::x(), b = bh / a.kv_heads, kh = bh - b * a.kv_heads, qg = a.q_heads / a.kv_heads;
  const int pos = FBLA_POS::ro(a.length + (a.lstride ? b : 0)) + a.n0, lane = FBLA_POS::tid() & 31, warp = FBLA_POS::tid() >> 5;
  if (FBLA_POS::tid() < 64) cs[FBLA_POS::tid()] = cos_sin_at(pos, __ldg(reinterpret_cast<const float4 *>(a.freq) + FBLA_POS::tid()), a.att);
  __syncthreads();
  const size_t eh = (size_t)bh * G * D;
  const int row = pos % G;
  for (int t = warp; t < qg + 2; t += 8) {  // tasks: the KV head's q heads, k, v
    if (t < qg) {
      const uint2 y = norm_rotate<NORM>(a.q + (int64_t)b * a.batch_stride + (int64_t)kh * a.q_group_stride + (size_t)t * D, a.q_norm, a.eps, cs, lane);
      uint32_t *o = reinterpret_cast<uint32_t *>(a.q_out + ((size_t)b * a.q_heads + kh * qg + t) * D);
      o[lane] = y.x; o[32 + lane] = y.y;
    } else {
      const bool isk = t == qg;
      uint2 y;
      if (isk) y = norm_rotate<NORM>(a.k + (int64_t)b * a.batch_stride + (int64_t)kh * a.kv_group_stride, a.k_norm, a.eps, cs, lane);
      else {
        const uint32_t *x = reinterpret_cast<const uint32_t *>(a.v + (int64_t)b * a.batch_stride + (int64_t)kh * a.kv_group_stride);
        y = make_uint2(__ldg(x + lane), __ldg(x + 32 + lane));
      }
      uint32_t *open = reinterpret_cast<uint32_t *>((isk ? a.c.open_k : a.c.open_v) + eh + (size_t)row * D);
      open[lane] = y.x; open[32 + lane] = y.y;
      if (pos < G) {
        uint32_t *sink = reinterpret_cast<uint32_t *>((isk ? a.c.sink_k : a.c.sink_v) + eh + (size_t)row * D);
        sink[lane] = y.x; sink[32 + lane] = y.y;
      }
    }
  }
  if (row == 0)  // the token opens a group: rows 1 .. 127 of both open windows are cleared
    for (int e = FBLA_POS::tid(); e < 2 * (G - 1) * 16; e += 256) {
      const int x = e >= (G - 1) * 16, r = e - x * (G - 1) * 16;
      reinterpret_cast<uint4 *>((x ? a.c.open_v : a.c.open_k) + eh + D)[r] = make_uint4(0u, 0u, 0u, 0u);
    }
}

// ---- a prefill chunk: the projection's rows [count][row_stride] -> q [q_heads][max_count][128], k / v [kv_heads][max_count][128]
constexpr int TOK = 8;  // positions per CTA
template <bool NORM>
__device__ __forceinline__ void qkv_chunk_item(const fbla_k_token &a, uint8_t *smem_raw) {
  __shared__ float2 cs[TOK][64];
  const int kh = FBLA_POS::y(), qg = a.q_heads / a.kv_heads, lane = FBLA_POS::tid() & 31, warp = FBLA_POS::tid() >> 5;
  const int base = FBLA_POS::ro(a.length) + a.n0, n = FBLA_POS::ro(a.dcount), i0 = FBLA_POS::x() * TOK, rows = max(0, min(TOK, n - i0));
  for (int e = FBLA_POS::tid(); e < rows * 64; e += 256)
    cs[e >> 6][e & 63] = cos_sin_at(base + i0 + (e >> 6), __ldg(reinterpret_cast<const float4 *>(a.freq) + (e & 63)), a.att);
  __syncthreads();
  const int per = qg + 2;
  for (int task = warp; task < rows * per; task += 8) {
    const int r = task / per, i = i0 + r, t = task - r * per;
    if (t < qg) {
      const uint2 y = norm_rotate<NORM>(a.q + (int64_t)i * a.batch_stride + (int64_t)kh * a.q_group_stride + (size_t)t * D, a.q_norm, a.eps, cs[r], lane);
      uint32_t *o = reinterpret_cast<uint32_t *>(a.q_out + (((size_t)kh * qg + t) * a.max_count + i) * D);
      o[lane] = y.x; o[32 + lane] = y.y;
    } else if (t == qg) {
      const uint2 y = norm_rotate<NORM>(a.k + (int64_t)i * a.batch_stride + (int64_t)kh * a.kv_group_stride, a.k_norm, a.eps, cs[r], lane);
      uint32_t *o = reinterpret_cast<uint32_t *>(a.k_out + ((size_t)kh * a.max_count + i) * D);
      o[lane] = y.x; o[32 + lane] = y.y;
    } else {
      const uint32_t *x = reinterpret_cast<const uint32_t *>(a.v + (int64_t)i * a.batch_stride + (int64_t)kh * a.kv_group_stride);
      uint32_t *o = reinterpret_cast<uint32_t *>(a.v_out + ((size_t)kh * a.max_count + i) * D);
      o[lane] = __ldg(x + lane); o[32 + lane] = __ldg(x + 32 + lane);
    }
  }
}

}  // namespace fbla

