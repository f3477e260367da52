// The thin C ABI between the C++ host layer (validation, geometry, dispatch) and the CUDA kernels: plain structs of
// pointers and sizes, one launcher per pass. The host layer fills these; nothing here validates.
#pragma once
#include "fbla_device.cuh"  /* fixed-width integers; under run-time compilation no host header is available */
#ifndef __CUDACC_RTC__
#include <stddef.h>
#define FBLA_HOST_API(decl) decl
#else
#define FBLA_HOST_API(decl)  /* launchers exist only in the library */
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
  uint8_t *coarse, *fine;
  uint16_t *meta, *sink_k, *sink_v, *open_k, *open_v;
} fbla_k_cache;

// ---- decode -------------------------------------------------------------------------------------------------------
// Virtual heads: a KV head with r = q_heads / kv_heads queries is served as vg = r / qg virtual heads of qg in {1, 2, 4}
// queries each (virtual head vh = kv_head_linear * vg + j owns queries j * qg .. j * qg + qg - 1 of its KV head).
// Scratch arrays (all written before they are read; no initial contents needed):
//   lse    [VH][nblocks][qg]  float  log2 mass of every closed sub-block under the coarse scores
//   part   [2 TW + 2 VH][qg][132] float  (o[128], m, l) partials: slot w + vh for streaming warp (or, folded, CTA) w,
//          coarse_ctas * coarse_warps + VH + x + vh for window warp x; TW = coarse_ctas * coarse_warps
//   dpart  [RW + VH][qg][129] float  (dl, do[128]) corrections of refine warp w at slot w + vh
//   row_r  [VH][qg]           float  log2 of the row's total coarse mass
//   counts [VH][nslices]      int    selected sub-blocks per slice of 1024 sub-blocks
//   items  [VH][nslices][1024] int   (sub-block << 4) | query mask, in sub-block order
//   item_off [VH * nslices + 1] int  exclusive prefix of counts (written by the refine pass for the merge)
//   status [4]                int    0 ok; nonzero: a bounded wait gave up (which pass, which CTA)
typedef struct {
  fbla_k_cache c;
  const uint16_t *q;
  uint16_t *out;
  float *lse, *part, *dpart, *row_r;
  int *counts, *items, *item_off, *status;
  const int *length;  // NULL, or device lengths: tokens of batch row b = length[b * lstride] + tokens
  int lstride;
  int batch, q_heads, kv_heads, tokens;
  int nblocks, nslices;  // layout of lse / items: sub-blocks and slices per head at the capacity
  int hs, gs;            // units between KV heads and between groups
  int qg, vg;            // queries per virtual head, virtual heads per KV head
  int cb, fb;            // plane bits
  int coarse_ctas, coarse_warps;  // persistent coarse CTAs and their warps (8): how the work is dealt to them is `deal`
  int refine_ctas, refine_warps;  // RW = refine_ctas * refine_warps
  float sl, log2_tau;
  // Sequence shards (one GPU's part of a long context); shard_on 0: the whole cache. A shard processes the closed groups
  // [sh_first, sh_first + sh_count) of its local cache, the BF16 sink window if sh_windows & 1, the open window if & 2.
  // phase 0: a whole decode. phase 1: coarse pass, then only the rows' local log2 mass into row_r. phase 2: select with
  // the given (global) row_r, refine, and the rows' unnormalised sums (o[128], l, relative to row_r) into out_partial.
  int shard_on, sh_first, sh_count, sh_windows, phase;
  float *out_partial;  // [rows][FBLA_K_PSTRIDE] floats (phase 2)
  int status_cleared;  // 1: the launcher zeroes the status word on the stream before the first pass; 0: CTA 0 of the coarse pass does
  short fold;          // 1: the coarse pass leaves one partial row per (CTA, virtual head) instead of one per (warp, virtual head)
  short deal;          // how the coarse pass's warps share the work, FBLA_K_DEAL_*
} fbla_k_decode;
#define FBLA_K_DEAL_LENGTHS 0 /* a CTA's warps are split between windows and groups by the rows' lengths (short contexts) */
#define FBLA_K_DEAL_FIXED 1   /* seven warps of a CTA stream groups, the eighth serves windows */
#define FBLA_K_DEAL_COST 2    /* every warp takes an equal cost share of windows and groups (long contexts) */

#define FBLA_K_PSTRIDE 132 /* floats of one partial row: o[128], then (m, l) or (dl) and padding */
#define FBLA_K_SLICE 1024  /* sub-blocks per select slice */

FBLA_HOST_API(cudaError_t fbla_k_decode_launch(const fbla_k_decode *a, cudaStream_t stream);)
// One pass of a decode alone (0 coarse, 1 select, 2 refine, 3 merge) as an ordinary launch, for timing the passes one by
// one; `a` as fbla_k_decode_launch takes it (e.g. the argument blob of a decode plan). Valid after one whole decode has
// run on the device.
FBLA_HOST_API(cudaError_t fbla_k_decode_pass_launch(const fbla_k_decode *a, int pass, cudaStream_t stream);)
// chooses the split of the coarse CTAs' warps for rows of about `tokens` tokens (after fbla_k_decode_shape; the scratch layout holds either)
FBLA_HOST_API(void fbla_k_decode_split(fbla_k_decode *a, long long tokens);)
// the same choice for a shape given by its numbers (pure host arithmetic: no device is touched): deal and fold as fbla_k_decode_split sets them
FBLA_HOST_API(void fbla_k_decode_split_of(int cb, int batch, int kv_heads, int vg, long long tokens, int *deal, int *fold);)
// out[row][ch] = bf16(partial[row][ch] / partial[row][128]) for rows rows of FBLA_K_PSTRIDE floats
// total[i] = log2 sum over shards of 2^mass[s][i]
FBLA_HOST_API(cudaError_t fbla_k_total_mass_launch(const float *mass, float *total, int shards, int rows, cudaStream_t stream);)
FBLA_HOST_API(cudaError_t fbla_k_combine_launch(const float *partial, uint16_t *out, int rows, cudaStream_t stream);)
// the most (virtual head, slice) entries one decode may have: the refine pass keeps their prefix sums in shared memory
FBLA_HOST_API(long long fbla_k_refine_entry_limit(int cb);)
// occupancy-derived launch shape for the current device; fills coarse_ctas .. refine_warps from cb / qg
FBLA_HOST_API(cudaError_t fbla_k_decode_shape(fbla_k_decode *a);)

// ---- the exchanges of a sequence-sharded decode as stores into the peers' memory (kernels/fbla_link.cu) -------------------
#define FBLA_K_MAX_RANKS 8
typedef struct {
  void *peer[FBLA_K_MAX_RANKS];  // the base of every rank's mailbox, as this rank addresses it (peer[rank]: its own)
  int rank, world, rows;         // rows = batch * q_heads
  unsigned spin_limit;           // polls (64 ns apart) before a wait for a peer gives up
} fbla_k_link;
// Byte offsets inside a mailbox (the same on every rank). epoch: the step counter; status: 0, or which wait gave up
// (1 masses, 2 sums, + 16 * the silent rank); *_flag[s], *_in[s]: the stamp and the data rank s stored here.
typedef struct {
  size_t epoch, status, mass_flag, part_flag, mass_in, local_mass, total, part_in, local_part, bytes;
} fbla_k_mailbox;
static inline __host__ __device__ fbla_k_mailbox fbla_k_mailbox_of(int world, int rows) {
  fbla_k_mailbox m;
  size_t at = 0;
  m.epoch = at; at += 16;
  m.status = at; at += 240;
  m.mass_flag = at; at += 256;
  m.part_flag = at; at += 256;
  m.mass_in = at; at += ((size_t)world * rows * 4 + 255) / 256 * 256;
  m.local_mass = at; at += ((size_t)rows * 4 + 255) / 256 * 256;
  m.total = at; at += ((size_t)rows * 4 + 255) / 256 * 256;
  m.part_in = at; at += ((size_t)world * rows * FBLA_K_PSTRIDE * 4 + 255) / 256 * 256;
  m.local_part = at; at += ((size_t)rows * FBLA_K_PSTRIDE * 4 + 255) / 256 * 256;
  m.bytes = at;
  return m;
}
FBLA_HOST_API(cudaError_t fbla_k_link_push_mass(const fbla_k_link *L, cudaStream_t stream);)
FBLA_HOST_API(cudaError_t fbla_k_link_gather_mass(const fbla_k_link *L, cudaStream_t stream);)
FBLA_HOST_API(cudaError_t fbla_k_link_push_partial(const fbla_k_link *L, cudaStream_t stream);)
FBLA_HOST_API(cudaError_t fbla_k_link_combine(const fbla_k_link *L, uint16_t *out, cudaStream_t stream);)

// ---- prefill: close the chunk's groups, attention, update the BF16 windows --------------------------------------------
typedef struct {
  fbla_k_cache c;
  const uint16_t *q, *k, *v;  // q NULL: append only
  uint16_t *out;
  int64_t out_hs;             // elements between q heads of out
  int out_ts;                 // elements between positions of out
  const int *length;          // NULL, or the chunk starts at length[row * lstride] + n0
  const int *dcount;          // NULL, or the chunk's token count on the device (count is then its ceiling)
  int lstride;
  int batch, q_heads, kv_heads, n0, count;
  int hs, gs;
  int cb, fb;
  float sl;
  // 0: the attention pass serves every count. > 0 (a chunk whose count lives on the device): the attention is two
  // passes and the count decides on the device which of them works -- the tensor-core pass when count * queries per KV
  // head >= tc_min_rows, the warp-per-row pass below that -- so that a device-count call takes the kernel the host-count
  // call of the same chunk takes and the two stay bit-identical.
  int tc_min_rows;
} fbla_k_prefill;

// close_blocks: grid x of the close pass (groups the chunk can close); 0 skips it
FBLA_HOST_API(cudaError_t fbla_k_close_launch(const fbla_k_prefill *a, int close_blocks, cudaStream_t stream);)
FBLA_HOST_API(cudaError_t fbla_k_finish_launch(const fbla_k_prefill *a, cudaStream_t stream);)
// Attention of the chunk's rows: the tensor-core kernel (tcgen05, 128 rows per CTA), or -- for chunks of fewer than
// FBLA_K_TC_MIN_ROWS rows, or when the environment variable MLOPS_FBLA_PREFILL=rows asks for it -- one warp per row.
// fbla_k_attend_plan splits a chunk's attention into its one or two passes (two when the count is on the device and
// its ceiling reaches the tensor-core kernel, see tc_min_rows): args[i] / tensor[i] for pass i; returns their number.
FBLA_HOST_API(int fbla_k_attend_plan(const fbla_k_prefill *a, fbla_k_prefill args[2], int tensor[2]);)
FBLA_HOST_API(cudaError_t fbla_k_attend_launch(const fbla_k_prefill *a, cudaStream_t stream);)  // every pass of the plan
FBLA_HOST_API(cudaError_t fbla_k_attend_rows_launch(const fbla_k_prefill *a, cudaStream_t stream);)
FBLA_HOST_API(cudaError_t fbla_k_attend_tc_launch(const fbla_k_prefill *a, cudaStream_t stream);)
// 1 if a bounded wait of the tensor-core kernel gave up since the last call (and clears it), 0 if not, -1 on a CUDA
// error. A CTA whose wait gave up also writes NaN to every output row it owns, so the failure shows in the data.
FBLA_HOST_API(int fbla_k_attend_tc_status(void);)
#define FBLA_K_TC_MIN_ROWS 64

// ---- fused QKV step: RMSNorm + rotary embedding of new tokens (+ the window stores of the one-token step) ------------------
typedef struct {
  fbla_k_cache c;                 // token step only
  const uint16_t *q, *k, *v;      // the projection's output
  int64_t batch_stride, q_group_stride, kv_group_stride;  // elements; batch_stride is the row stride of a chunk
  const uint16_t *q_norm, *k_norm;  // both or neither
  const float *freq;              // 64 x (fh, fl, gh, gl)
  float eps, att;
  const int *length, *dcount;
  int lstride, n0, max_count;
  int batch, q_heads, kv_heads;
  uint16_t *q_out, *k_out, *v_out;
} fbla_k_token;
FBLA_HOST_API(cudaError_t fbla_k_qkv_token_launch(const fbla_k_token *a, cudaStream_t stream);)
FBLA_HOST_API(cudaError_t fbla_k_qkv_chunk_launch(const fbla_k_token *a, cudaStream_t stream);)

// ---- what an executor needs to run a pass from kernels of its own (include/mlops_fbla_items.h) ---------------------------
typedef struct {
  int gx, gy, gz;    // the grid of the equivalent launch: one item per CTA
  int threads;       // the exact CTA size
  int smem_bytes;    // shared memory to hand the entry (includes the slack entries use to re-align a 16-byte aligned pointer)
  int regs;          // registers per thread of this library's kernel
  char entry[96];    // the device function (kernels/*.cuh), called as entry(args, shared memory)
} fbla_k_pass;
FBLA_HOST_API(cudaError_t fbla_k_decode_passes(const fbla_k_decode *a, fbla_k_pass info[4]);)  // coarse, select, refine, merge
FBLA_HOST_API(cudaError_t fbla_k_close_pass(const fbla_k_prefill *a, int close_blocks, fbla_k_pass *info);)
FBLA_HOST_API(cudaError_t fbla_k_finish_pass(const fbla_k_prefill *a, fbla_k_pass *info);)
FBLA_HOST_API(cudaError_t fbla_k_attend_rows_pass(const fbla_k_prefill *a, fbla_k_pass *info);)
FBLA_HOST_API(cudaError_t fbla_k_attend_tc_pass(const fbla_k_prefill *a, fbla_k_pass *info);)
FBLA_HOST_API(cudaError_t fbla_k_qkv_token_pass(const fbla_k_token *a, fbla_k_pass *info);)
FBLA_HOST_API(cudaError_t fbla_k_qkv_chunk_pass(const fbla_k_token *a, fbla_k_pass *info);)

#ifdef __cplusplus
}
#endif
