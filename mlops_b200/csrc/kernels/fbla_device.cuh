// Device-side building blocks shared by the FBLA kernels (sm_100a): BF16 and special-function helpers, the legacy
// warp-level integer tensor-core instruction, 1-D bulk asynchronous copies with mbarrier completion and BOUNDED waits,
// and the packed-record format as compile-time traits.
#pragma once
#ifdef __CUDACC_RTC__  // compiled at run time inside an executor's own kernels: no host headers
typedef unsigned char uint8_t;
typedef signed char int8_t;
typedef unsigned short uint16_t;
typedef unsigned int uint32_t;
typedef int int32_t;
typedef unsigned long long uint64_t;
typedef long long int64_t;
typedef unsigned long long uintptr_t;
typedef unsigned long size_t;
#else
#include <cuda_runtime.h>
#include <stdint.h>
#endif

namespace fbla {

// Where a CTA stands in its pass. The library's own kernels are launched one CTA per item and read the hardware's
// registers (GridPos); an executor that runs the passes' items from kernels of its own (include/mlops_fbla_items.h)
// defines mlops_fbla::Pos with the same members and FBLA_POS to name it before including the item bodies.
//   x y z nx ny nz: the item's coordinates in the pass's grid; tid: the thread within the item's CTA;
//   ro(p): the read of a device length or count (at most once per call site);
struct GridPos {
  static __device__ __forceinline__ int x() { return blockIdx.x; }
  static __device__ __forceinline__ int y() { return blockIdx.y; }
  static __device__ __forceinline__ int z() { return blockIdx.z; }
  static __device__ __forceinline__ int nx() { return gridDim.x; }
  static __device__ __forceinline__ int ny() { return gridDim.y; }
  static __device__ __forceinline__ int nz() { return gridDim.z; }
  static __device__ __forceinline__ int tid() { return threadIdx.x; }
  static __device__ __forceinline__ int ro(const int *p) { return __ldg(p); }
};
#ifndef FBLA_POS
#define FBLA_POS ::fbla::GridPos
#endif
// programmatic dependent launch is used by the library's own stream launches only
template <class A, class B> struct same_type { static constexpr bool value = false; };
template <class A> struct same_type<A, A> { static constexpr bool value = true; };
#define FBLA_STREAM_LAUNCH (::fbla::same_type<FBLA_POS, ::fbla::GridPos>::value)
#define FBLA_INF (__int_as_float(0x7f800000))

constexpr int D = 128;    // head dimension
constexpr int G = 128;    // tokens per group
constexpr int S = 16;     // tokens per sub-block (one record, one P block)
constexpr int SBG = 8;    // sub-blocks per group
constexpr uint32_t FULL = 0xffffffffu;
constexpr uint32_t MAGIC = 0x4B400000u;  // bits of 1.5 * 2^23: an s32 accumulator started here reads, as FP32, 1.5 * 2^23 + sum
constexpr float MAGICF = 12582912.f;

__host__ __device__ constexpr int record_bytes(int bits) { return 2 * bits * 256; }

// ---- scalar helpers -------------------------------------------------------------------------------------------
__device__ __forceinline__ float bf16_to_f32(uint16_t x) { return __uint_as_float((uint32_t)x << 16); }
__device__ __forceinline__ uint16_t f32_to_bf16(float x) {  // round to nearest even, NaN canonical
  uint32_t u = __float_as_uint(x);
  if ((u & 0x7fffffffu) > 0x7f800000u) u = 0x7fc00000u;
  return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
// two BF16 packed in a word -> two floats
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ float ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float lg2(float x) { float y; asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float isum(uint32_t acc) { return __uint_as_float(acc) - MAGICF; }  // exact for |sum| < 2^22

// packed pairs of FP32 (FADD2 / FMUL2 / FFMA2 of sm_100: two lanes of arithmetic per instruction)
__device__ __forceinline__ float2 isum2(uint32_t a, uint32_t b) {
  return __fadd2_rn(make_float2(__uint_as_float(a), __uint_as_float(b)), make_float2(-MAGICF, -MAGICF));
}
__device__ __forceinline__ float2 splat(float x) { return make_float2(x, x); }

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o; o >>= 1) x = fmaxf(x, __shfl_xor_sync(FULL, x, o));
  return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o; o >>= 1) x += __shfl_xor_sync(FULL, x, o);
  return x;
}

// ---- integer tensor-core products (warp-wide, operands in registers) ------------------------------------------
// D[16 x 8] (s32) += A[16 x 32] (u8, row-major) * B[32 x 8] (s8 or u8, column-major). Thread T = 4 * gid + tig holds
//   a0: row gid,   k 4 tig .. 4 tig + 3     a1: row gid + 8, same k     a2 / a3: the same rows, k + 16
//   b0: k 4 tig .. + 3, column gid          b1: k + 16, column gid
//   d0: (gid, 2 tig)  d1: (gid, 2 tig + 1)  d2: (gid + 8, 2 tig)  d3: (gid + 8, 2 tig + 1)
__device__ __forceinline__ void mma_u8s8_k32(uint32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// the same products starting from the constant c in every accumulator (D = A B + c): no register moves to set D up
__device__ __forceinline__ void mma_u8s8_k32_from(uint32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1, uint32_t c) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c));
}
__device__ __forceinline__ void mma_u8u8_k32_from(uint32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1, uint32_t c) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c));
}
__device__ __forceinline__ void mma_u8u8_k32(uint32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- mbarrier + bulk asynchronous copy (global -> this CTA's shared memory) -------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint64_t *bar) {  // the word may then be re-initialised (the next item on this CTA) or reused
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {  // make the initialised barriers visible to the copy engine
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity, at most `limit` polls. Returns false if it gave up: the caller records
// an error status and leaves; nothing here can spin forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, uint32_t limit = (1u << 24)) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// order this thread's earlier generic-proxy accesses of shared memory before later asynchronous-proxy ones
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// bytes: a multiple of 16; both addresses 16-byte aligned
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ uint32_t lds32(const uint8_t *p) { return *reinterpret_cast<const uint32_t *>(p); }
__device__ __forceinline__ uint2 lds64(const uint8_t *p) { return *reinterpret_cast<const uint2 *>(p); }
__device__ __forceinline__ uint4 lds128(const uint8_t *p) { return *reinterpret_cast<const uint4 *>(p); }

// ---- the packed record format, as the slot maps of include/mlops_fbla.h ------------------------------------------
// V slot s of a BITS-plane -> channel (0..3 within the lane's four) and token quad
__host__ __device__ constexpr int v_chan(int bits, int s) {
  return bits == 4 ? (s < 8 ? s % 2 : 2 + s % 2) : bits == 2 ? s / 4 : s < 4 ? 0 : s < 6 ? 2 : s < 10 ? 1 : s < 12 ? 2 : 3;
}
__host__ __device__ constexpr int v_quad(int bits, int s) {
  return bits == 4 ? (s < 8 ? s / 2 : (s - 8) / 2) : bits == 2 ? s % 4 : s < 4 ? s : s < 6 ? s - 4 : s < 10 ? s - 6 : s < 12 ? s - 8 : s - 12;
}
// byte offset of word w of lane l of tensor t (0 K, 1 V) in a BITS-plane record
__host__ __device__ constexpr int word_offset(int bits, int t, int l, int w) {
  return bits == 4 ? 1024 * t + (w < 4 ? 16 * l + 4 * w : 512 + 16 * l + 4 * (w - 4))
       : bits == 2 ? 512 * t + 16 * l + 4 * w
       : w < 4 ? 512 * t + 16 * l + 4 * w
       : t ? 1280 + 8 * l + 4 * (w - 4) : 1024 + 16 * (l % 16) + 8 * (l / 16) + 4 * (w - 4);
}

// the four codes of slot s of a lane's words W[0 .. 2 BITS - 1] of one tensor, one code per byte, unscaled
template <int BITS> __device__ __forceinline__ uint32_t slot_value(const uint32_t *W, int s) {
  if (BITS == 4) return s < 8 ? W[s] & 0x0f0f0f0fu : (W[s - 8] >> 4) & 0x0f0f0f0fu;
  if (BITS == 2) return (W[s & 3] >> (2 * (s >> 2))) & 0x03030303u;
  if (s < 6) return W[s] & 0x07070707u;
  if (s < 12) return (W[s - 6] >> 3) & 0x07070707u;
  const int r = s - 12;
  return ((W[r] >> 6) & 0x03030303u) | ((W[4 + (r >> 1)] >> (4 + (r & 1))) & 0x04040404u);
}
// the V slot holding channel cc (of the lane's four) and token quad `quad`: the inverse of (v_chan, v_quad)
__host__ __device__ constexpr int v_slot_of(int bits, int cc, int quad) {
  return bits == 4 ? (cc < 2 ? 2 * quad + cc : 8 + 2 * quad + (cc - 2))
       : bits == 2 ? 4 * cc + quad
       : cc == 0 ? quad : cc == 1 ? 6 + quad : cc == 2 ? (quad < 2 ? 4 + quad : 8 + quad) : 12 + quad;
}

}  // namespace fbla
