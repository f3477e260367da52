// Causal prefill attention over the compressed cache, CUDA-core version: one warp per query row.
//
// Semantics (the reference's DP4A prefill, attention/fbla/src/fbla_prefill.cuh:389-705): the row at position p attends
// to 0..p -- group 0 (sink) and its own group in BF16 from the windows / the chunk, closed groups 1..own-1 through
// their full 6-bit codes (coarse << FB | fine) with the per-(row, group) int8 qhat, 16-token integer P blocks
// everywhere. This kernel is the simple, obviously-correct form of that definition (each lane is the record lane of
// the same number, integer dot products by DP4A); it is the fallback the tensor-core prefill is checked against
// and the path taken for shapes the tensor-core kernel does not cover.
#pragma once
#include "fbla_device.cuh"
#include "fbla_kernels.h"

namespace fbla {

template <int BITS> __device__ __forceinline__ void load_words(const uint8_t *rec, int tensor, int lane, uint32_t *W) {
#pragma unroll
  for (int w = 0; w < 2 * BITS; ++w) W[w] = __ldcg(reinterpret_cast<const uint32_t *>(rec + word_offset(BITS, tensor, lane, w)));
}

struct RowState { float m, l, o[4]; };

// one 16-token block given the lane's score (lanes t and t + 16 hold token t's) and a functor for sum_t p_t v[t][4 lane + cc]
template <class PV> __device__ __forceinline__ void block_update(RowState &st, float s, uint8_t *pst, int lane, PV pv) {
  float mb = s;
#pragma unroll
  for (int o = 8; o; o >>= 1) mb = fmaxf(mb, __shfl_xor_sync(FULL, mb, o));
  if (mb == -FBLA_INF) return;  // (warp-uniform: every token masked)
  if (lane < 16) pst[lane] = (uint8_t)__float_as_uint(fmaf(ex2(s - mb), 255.f, MAGICF));
  __syncwarp();
  const uint4 pw = *reinterpret_cast<const uint4 *>(pst);
  const uint32_t P[4] = {pw.x, pw.y, pw.z, pw.w};
  const float sp = (float)(__dp4a(P[0], 0x01010101u, 0u) + __dp4a(P[1], 0x01010101u, 0u) + __dp4a(P[2], 0x01010101u, 0u) + __dp4a(P[3], 0x01010101u, 0u));
  float y[4];
  pv(P, y);
  const float mn = fmaxf(st.m, mb), al = ex2(st.m - mn), w = ex2(mb - mn);
  st.m = mn;
  st.l = fmaf(al, st.l, w * sp);
#pragma unroll
  for (int cc = 0; cc < 4; ++cc) st.o[cc] = fmaf(al, st.o[cc], w * y[cc]);
  __syncwarp();
}

template <int CB, int FB>
__device__ __forceinline__ void attend_rows_item(const fbla_k_prefill &a, uint8_t *smem_raw) {
  __shared__ __align__(16) float qs[8][D];
  __shared__ __align__(16) uint32_t qh[8][32];
  __shared__ __align__(16) uint8_t pst[8][16];
  const int lane = FBLA_POS::tid() & 31, warp = FBLA_POS::tid() >> 5;
  const int bh = FBLA_POS::y(), b = bh / a.kv_heads, kh = bh - b * a.kv_heads, qg = a.q_heads / a.kv_heads;
  const int n0 = (a.length ? FBLA_POS::ro(a.length + (a.lstride ? b : 0)) : 0) + a.n0;
  const int count = a.dcount ? FBLA_POS::ro(a.dcount) : a.count, n1 = n0 + count;
  const int r = FBLA_POS::x() * 8 + warp;
  if (r >= count * qg || (a.tc_min_rows && count * qg >= a.tc_min_rows)) return;  // (a long device count is the tensor-core pass's work)
  const int i = r / qg, hq = kh * qg + (r - i * qg), pos = n0 + i, own = pos / G;
  const size_t eh = (size_t)bh * G * D, ih = (size_t)bh * a.count * D;
  {
    const uint2 w = __ldg(reinterpret_cast<const uint2 *>(a.q + ((size_t)(b * a.q_heads + hq) * a.count + i) * D) + lane);
    *reinterpret_cast<float4 *>(&qs[warp][4 * lane]) = make_float4(bf_lo(w.x), bf_hi(w.x), bf_lo(w.y), bf_hi(w.y));
  }
  __syncwarp();
  RowState st{-FBLA_INF, 0.f, {0.f, 0.f, 0.f, 0.f}};
  const int t = lane & 15, h = lane >> 4;

  // the BF16 row of position tp: the chunk, the sink window, or the window of the group that was open before the chunk
  auto row_of = [&](int tp, const uint16_t *in, const uint16_t *sink, const uint16_t *open) -> const uint16_t * {
    return tp >= n0 ? in + ih + (size_t)(tp - n0) * D : tp < G ? sink + eh + (size_t)tp * D : open + eh + (size_t)(tp - (n0 - 1) / G * G) * D;
  };
  auto exact_group = [&](int g) {
    for (int j = 0; j < SBG; ++j) {
      const int t0 = g * G + j * S;
      if (t0 > pos || t0 >= n1) break;
      const int tp = t0 + t;
      float x = 0.f;
      if (tp <= pos) {
        const uint4 *kp = reinterpret_cast<const uint4 *>(row_of(tp, a.k, a.c.sink_k, a.c.open_k) + 64 * h);
#pragma unroll
        for (int e8 = 0; e8 < 8; ++e8) {
          const uint4 w = __ldcg(kp + e8);
          const float kv[8] = {bf_lo(w.x), bf_hi(w.x), bf_lo(w.y), bf_hi(w.y), bf_lo(w.z), bf_hi(w.z), bf_lo(w.w), bf_hi(w.w)};
#pragma unroll
          for (int e = 0; e < 8; ++e) x = fmaf(qs[warp][64 * h + 8 * e8 + e], kv[e], x);
        }
      }
      x += __shfl_xor_sync(FULL, x, 16);
      const float s = tp <= pos ? __fmul_rn(x, a.sl) : -FBLA_INF;
      block_update(st, s, pst[warp], lane, [&](const uint32_t (&P)[4], float (&y)[4]) {
        y[0] = y[1] = y[2] = y[3] = 0.f;
        for (int tt = 0; tt < S; ++tt) {
          if (t0 + tt > pos) break;
          const uint2 vw = __ldcg(reinterpret_cast<const uint2 *>(row_of(t0 + tt, a.v, a.c.sink_v, a.c.open_v)) + lane);
          const float p = (float)((P[tt >> 2] >> (8 * (tt & 3))) & 255u);
          y[0] = fmaf(p, bf_lo(vw.x), y[0]); y[1] = fmaf(p, bf_hi(vw.x), y[1]);
          y[2] = fmaf(p, bf_lo(vw.y), y[2]); y[3] = fmaf(p, bf_hi(vw.y), y[3]);
        }
      });
    }
  };

  exact_group(0);
  if (own > 0) exact_group(own);
  for (int g = own - 1; g >= 1; --g) {  // closed groups, newest first
    const size_t unit = (size_t)bh * a.hs + (size_t)g * a.gs;
    const uint8_t *meta = reinterpret_cast<const uint8_t *>(a.c.meta) + unit * 1024;
    const uint4 km = __ldcg(reinterpret_cast<const uint4 *>(meta) + lane);
    const uint4 vm = __ldcg(reinterpret_cast<const uint4 *>(meta + 512) + lane);
    // qhat of the row for this group (lane: channels 4 lane ..)
    float sq, qb;
    {
      const float4 q4 = *reinterpret_cast<const float4 *>(&qs[warp][4 * lane]);
      const float kb[4] = {bf_lo(km.x), bf_hi(km.x), bf_lo(km.y), bf_hi(km.y)}, ks[4] = {bf_lo(km.z), bf_hi(km.z), bf_lo(km.w), bf_hi(km.w)};
      const float qf[4] = {q4.x, q4.y, q4.z, q4.w};
      float z[4], amax = 0.f, dot = 0.f;
#pragma unroll
      for (int x = 0; x < 4; ++x) { z[x] = __fmul_rn(qf[x], ks[x]); amax = fmaxf(amax, fabsf(z[x])); dot = fmaf(qf[x], kb[x], dot); }
      amax = warp_max(amax);
      float rc;
      asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rc) : "f"(amax));
      rc = fmaf(fmaf(-amax, rc, 1.f), rc, rc);
      const float q0 = __fmul_rn(127.f, rc), rr = amax > 0.f ? fmaf(fmaf(-amax, q0, 127.f), rc, q0) : 0.f;
      uint32_t word = 0;
#pragma unroll
      for (int x = 0; x < 4; ++x) word |= (__float_as_uint(fmaf(z[x], rr, MAGICF)) & 255u) << (8 * x);
      __syncwarp();
      qh[warp][lane] = word;
      sq = __fmul_rn(amax, __fmul_rn(a.sl, 1.f / 127.f));
      qb = __fmul_rn(warp_sum(dot), a.sl);
      __syncwarp();
    }
    const float vb[4] = {bf_lo(vm.x), bf_hi(vm.x), bf_lo(vm.y), bf_hi(vm.y)}, vs[4] = {bf_lo(vm.z), bf_hi(vm.z), bf_lo(vm.w), bf_hi(vm.w)};
    float Ag[4] = {0.f, 0.f, 0.f, 0.f}, Bg = 0.f;  // the group's sum w y (code units) and sum w sum p, relative to mg
    float mg = -FBLA_INF;
    for (int j = 0; j < SBG; ++j) {
      const uint8_t *rc_ = a.c.coarse + (unit * SBG + j) * record_bytes(CB), *rf_ = a.c.fine + (unit * SBG + j) * record_bytes(FB);
      uint32_t Wc[2 * CB], Wf[2 * FB];
      load_words<CB>(rc_, 0, lane, Wc);
      load_words<FB>(rf_, 0, lane, Wf);
      int acc = 0;
#pragma unroll
      for (int s = 0; s < 16; ++s) acc = __dp4a((int)((slot_value<CB>(Wc, s) << FB) | slot_value<FB>(Wf, s)), (int)qh[warp][16 * h + s], acc);
      float x = (float)acc;
      x += __shfl_xor_sync(FULL, x, 16);
      const float s = fmaf(sq, x, qb);
      float mb = s;
#pragma unroll
      for (int o = 8; o; o >>= 1) mb = fmaxf(mb, __shfl_xor_sync(FULL, mb, o));
      if (lane < 16) pst[warp][lane] = (uint8_t)__float_as_uint(fmaf(ex2(s - mb), 255.f, MAGICF));
      __syncwarp();
      const uint4 pw = *reinterpret_cast<const uint4 *>(pst[warp]);
      const uint32_t P[4] = {pw.x, pw.y, pw.z, pw.w};
      const float sp = (float)(__dp4a(P[0], 0x01010101u, 0u) + __dp4a(P[1], 0x01010101u, 0u) + __dp4a(P[2], 0x01010101u, 0u) + __dp4a(P[3], 0x01010101u, 0u));
      load_words<CB>(rc_, 1, lane, Wc);
      load_words<FB>(rf_, 1, lane, Wf);
      float y[4];
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t sum = 0;
#pragma unroll
        for (int quad = 0; quad < 4; ++quad)
          sum = __dp4a((slot_value<CB>(Wc, v_slot_of(CB, cc, quad)) << FB) | slot_value<FB>(Wf, v_slot_of(FB, cc, quad)), P[quad], sum);
        y[cc] = (float)sum;
      }
      const float mn = fmaxf(mg, mb), al = ex2(mg - mn), w = ex2(mb - mn);
      mg = mn;
      Bg = fmaf(al, Bg, w * sp);
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) Ag[cc] = fmaf(al, Ag[cc], w * y[cc]);
      __syncwarp();
    }
    const float mn = fmaxf(st.m, mg), al = ex2(st.m - mn), be = ex2(mg - mn);
    st.m = mn;
    st.l = fmaf(al, st.l, be * Bg);
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) st.o[cc] = fmaf(al, st.o[cc], be * fmaf(vs[cc], Ag[cc], vb[cc] * Bg));
  }
  const float inv = 1.f / st.l;
  const uint32_t w0 = f32_to_bf16(st.o[0] * inv) | (uint32_t)f32_to_bf16(st.o[1] * inv) << 16;
  const uint32_t w1 = f32_to_bf16(st.o[2] * inv) | (uint32_t)f32_to_bf16(st.o[3] * inv) << 16;
  uint16_t *orow = a.out + (size_t)(b * a.q_heads + hq) * a.out_hs + (size_t)i * a.out_ts;
  reinterpret_cast<uint2 *>(orow)[lane] = make_uint2(w0, w1);
}

}  // namespace fbla

