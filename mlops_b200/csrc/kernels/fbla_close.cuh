// Quantize-on-write ("close") and the BF16 window update ("finish") of the FBLA cache, sm_100a.
//
// close: one CTA per (group the chunk closes, KV head). The group's 128 x 128 BF16 tiles of K and V are staged in shared
// memory with 128-bit coalesced loads (each token row comes from the chunk, the sink window or the old open window),
// thread c owns channel c of one tensor: min / max over the 128 tokens, BF16 base (rounded down) and step (rounded up),
// the 6-bit codes; then every thread assembles whole 32-bit words of the coarse and fine records from the code tile
// and stores them, together with the 1 KiB metadata. HBM-bound: 64 KiB read, 25 KiB written per (head, group).
// Replaces the reference's close_kernel / finish_kernel (attention/fbla/src/fbla_prefill.cuh:63-164); results are
// bit-identical by construction of the FP32 steps (no contraction: explicit round-to-nearest intrinsics).
#pragma once
#include "fbla_device.cuh"
#include "fbla_kernels.h"

namespace fbla {

// x rounded to BF16 toward -inf (up false) or +inf (up true)
__device__ __forceinline__ uint16_t bf16_directed(float x, bool up) {
  uint16_t u = f32_to_bf16(x);
  const float y = bf16_to_f32(u);
  if (up ? y < x : y > x) {
    if (y > 0.f) u = up ? u + 1 : u - 1;
    else if (y < 0.f) u = up ? u - 1 : u + 1;
    else u = up ? 0x0001 : 0x8001;
  }
  return u;
}

constexpr int ROW = D + 8;  // padded BF16 row (elements): 272 bytes, keeps 16-byte alignment, spreads banks

struct CloseSmem {
  uint16_t x[2][G][ROW];  // [K, V][token][channel] BF16
  uint8_t code[2][G][D];  // 6-bit codes
};

// the code of (tensor, sub-block j, lane l, slot s, byte b) of a BITS-plane record
template <int BITS>
__device__ __forceinline__ uint32_t code_of(const CloseSmem &sm, int tensor, int j, int l, int s, int b) {
  return tensor ? sm.code[1][16 * j + 4 * v_quad(BITS, s) + b][4 * l + v_chan(BITS, s)]
                : sm.code[0][16 * j + (l & 15)][64 * (l >> 4) + 4 * s + b];
}

// word w of (tensor, lane) of sub-block j's record in a BITS-plane; PART(code) extracts the plane's bits
template <int BITS, int SHIFT, int MASK>
__device__ __forceinline__ uint32_t record_word(const CloseSmem &sm, int tensor, int j, int l, int w) {
  uint32_t word = 0;
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    auto part = [&](int s) -> uint32_t { return (code_of<BITS>(sm, tensor, j, l, s, b) >> SHIFT) & MASK; };
    uint32_t byte;
    if (BITS == 4) byte = part(w) | part(w + 8) << 4;
    else if (BITS == 2) byte = part(w) | part(4 + w) << 2 | part(8 + w) << 4 | part(12 + w) << 6;
    else if (w < 4) byte = part(w) | part(w + 6) << 3 | (part(12 + w) & 3u) << 6;
    else byte = part(w) | part(w + 6) << 3 | (part(12 + 2 * (w - 4)) >> 2) << 6 | (part(13 + 2 * (w - 4)) >> 2) << 7;
    word |= byte << (8 * b);
  }
  return word;
}

template <int BITS, int SHIFT, int MASK>
__device__ __forceinline__ void write_plane(const CloseSmem &sm, uint8_t *plane_unit) {
  constexpr int WPL = 2 * BITS;          // words per (tensor, lane)
  constexpr int NW = SBG * 2 * 32 * WPL;  // words of the group's 8 records
  for (int i = FBLA_POS::tid(); i < NW; i += 256) {
    const int w = i % WPL, l = (i / WPL) % 32, tensor = (i / (WPL * 32)) % 2, j = i / (WPL * 64);
    const uint32_t word = record_word<BITS, SHIFT, MASK>(sm, tensor, j, l, w);
    *reinterpret_cast<uint32_t *>(plane_unit + (size_t)j * record_bytes(BITS) + word_offset(BITS, tensor, l, w)) = word;
  }
}

template <int CB, int FB>
__device__ __forceinline__ void close_item(const fbla_k_prefill &a, uint8_t *smem_raw) {
  CloseSmem &sm = *reinterpret_cast<CloseSmem *>(smem_raw);
  const int bh = FBLA_POS::y(), b = bh / a.kv_heads;
  const int n0 = (a.length ? FBLA_POS::ro(a.length + (a.lstride ? b : 0)) : 0) + a.n0;
  const int count = a.dcount ? FBLA_POS::ro(a.dcount) : a.count;
  const int g = (n0 == 0 ? 0 : (n0 - 1) / G) + (int)FBLA_POS::x();
  if (g >= (n0 + count - 1) / G) return;  // the chunk does not close this group

  const size_t eh = (size_t)bh * G * D, ih = (size_t)bh * a.count * D;
  // stage the 2 x 128 rows
  for (int i = FBLA_POS::tid(); i < 2 * G * 16; i += 256) {
    const int x = i >> 11, t = (i >> 4) & 127, qd = i & 15, pos = g * G + t;
    const uint16_t *row = pos >= n0 ? (x ? a.v : a.k) + ih + (size_t)(pos - n0) * D
                        : pos < G   ? (x ? a.c.sink_v : a.c.sink_k) + eh + (size_t)pos * D
                                    : (x ? a.c.open_v : a.c.open_k) + eh + (size_t)(pos - (n0 - 1) / G * G) * D;
    *reinterpret_cast<uint4 *>(&sm.x[x][t][8 * qd]) = *(reinterpret_cast<const uint4 *>(row) + qd);
  }
  __syncthreads();
  const size_t unit = (size_t)bh * a.hs + (size_t)g * a.gs;
  {
    const int x = FBLA_POS::tid() >> 7, c = FBLA_POS::tid() & 127;
    float lo = FBLA_INF, hi = -FBLA_INF;
#pragma unroll 8
    for (int t = 0; t < G; ++t) { const float e = bf16_to_f32(sm.x[x][t][c]); lo = fminf(lo, e); hi = fmaxf(hi, e); }
    const uint16_t ub = bf16_directed(lo, false);
    const float base = bf16_to_f32(ub);
    const uint16_t us = bf16_directed(__fmul_rn(__fsub_rn(hi, base), 1.f / 63.f), true);
    const float step = bf16_to_f32(us), inv = step > 0.f ? __frcp_rn(step) : 0.f;
#pragma unroll 8
    for (int t = 0; t < G; ++t) {
      const float r = rintf(__fmul_rn(__fsub_rn(bf16_to_f32(sm.x[x][t][c]), base), inv));
      sm.code[x][t][c] = (uint8_t)fminf(fmaxf(r, 0.f), 63.f);
    }
    uint16_t *meta = a.c.meta + unit * 512;
    meta[256 * x + 8 * (c >> 2) + (c & 3)] = ub;
    meta[256 * x + 8 * (c >> 2) + 4 + (c & 3)] = us;
  }
  __syncthreads();
  write_plane<CB, FB, (1 << CB) - 1>(sm, a.c.coarse + unit * SBG * record_bytes(CB));
  write_plane<FB, 0, (1 << FB) - 1>(sm, a.c.fine + unit * SBG * record_bytes(FB));
}

// finish: the sink window takes the chunk's positions < 128, the open window the tokens of the newest group; a fresh
// open group's unused rows are cleared. One CTA per KV head.
__device__ __forceinline__ void finish_item(const fbla_k_prefill &a, uint8_t *smem_raw) {
  const int bh = FBLA_POS::x(), b = bh / a.kv_heads;
  const int n0 = (a.length ? FBLA_POS::ro(a.length + (a.lstride ? b : 0)) : 0) + a.n0;
  const int n1 = n0 + (a.dcount ? FBLA_POS::ro(a.dcount) : a.count), gl = (n1 - 1) / G;
  const bool fresh = n0 == 0 || (n0 - 1) / G != gl;
  const size_t eh = (size_t)bh * G * D, ih = (size_t)bh * a.count * D;
  for (int x = 0; x < 2; ++x) {
    const uint4 *in = reinterpret_cast<const uint4 *>((x ? a.v : a.k) + ih);
    uint4 *open = reinterpret_cast<uint4 *>((x ? a.c.open_v : a.c.open_k) + eh);
    uint4 *sink = reinterpret_cast<uint4 *>((x ? a.c.sink_v : a.c.sink_k) + eh);
    for (int e = FBLA_POS::tid(); e < G * 16; e += 256) {
      const int t = e >> 4, pos = gl * G + t;
      if (pos >= n0 && pos < n1) open[e] = in[(size_t)(pos - n0) * 16 + (e & 15)];
      else if (fresh && pos >= n1) open[e] = make_uint4(0u, 0u, 0u, 0u);
      if (t >= n0 && t < n1) sink[e] = in[(size_t)(t - n0) * 16 + (e & 15)];
    }
  }
}

}  // namespace fbla

