/* FBLA compressed-KV attention for NVIDIA B200 (sm_100a): the C interface.
 *
 * This header is ABI-identical to the interface of mlops-attention 0.4.0 (reference: attention/include/mlops_fbla.h:1-189):
 * the same type names, field order and sizes, enum values, function names and argument orders, so a program written
 * against that header links against this library unchanged. The text below is a restatement; the layout facts it
 * gives are the contract the kernels and the tests are written from.
 *
 * Model. Head dimension 128. The tokens of one KV head form groups of 128. A group that is complete and has been
 * followed by at least one more token is "closed": every element x of K and of V is stored as a 6-bit code c with
 *     x ~ base[channel] + c * step[channel],        c in 0..63,
 * base = the channel's minimum over the group rounded down to BF16, step = fl32((max - base) * fl32(1/63)) rounded up
 * to BF16, c = clamp(rint(fl32(fl32(x - base) * fl32(1/step))), 0, 63) (c = 0 where step is 0). The code is split in
 * two planes: the coarse plane keeps the top CB bits (h = c >> FB), the fine plane the low FB bits (f = c & (2^FB-1));
 * CB+FB is 3+3 or 4+2. An element read without its fine bits decodes to the middle of its coarse cell,
 * base + step * (2^FB * h + (2^FB - 1) / 2). Group 0 (the attention sink) and the newest group (still filling) are
 * additionally kept as BF16 and are always read as BF16.
 *
 * Decode reads all coarse planes once, and the fine planes only of those 16-token sub-blocks whose share of a
 * query's softmax mass (estimated from the coarse scores) exceeds tau. Scores use a per-(query, group) int8 query:
 * z = q * step_K (exact in FP32), qhat = rint(z * fl32(127 / max|z|)), sq = max|z| * sl / 127, sl = fl32(scale*log2 e):
 *     score(log2 units) = sq * (qhat . code) + sl * (q . base_K).
 * Softmax weights are formed per 16-token sub-block as integers p = round(255 * 2^(s - max_block)).
 */
#ifndef MLOPS_FBLA_H
#define MLOPS_FBLA_H

#include <stddef.h>
#include <stdint.h>

#ifdef MLOPS_FBLA_NO_CUDA_RUNTIME /* host tools that only need the types (the CPU oracle, ctypes mirrors) */
typedef struct CUstream_st *cudaStream_t;
#else
#include <cuda_runtime.h>
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* reference: mlops_fbla.h:29 */
enum { MLOPS_FBLA_HEAD_DIM = 128, MLOPS_FBLA_GROUP = 128, MLOPS_FBLA_SUBBLOCK = 16 };

/* reference: mlops_fbla.h:37-45 */
typedef enum {
  MLOPS_FBLA_3P3 = 0, /* 3 coarse + 3 fine bits; default tau 3e-4 */
  MLOPS_FBLA_4P2 = 1  /* 4 coarse + 2 fine bits; default tau 1e-3 */
} mlops_fbla_format;
typedef enum {
  MLOPS_FBLA_OK = 0,
  MLOPS_FBLA_INVALID_VALUE = 1,
  MLOPS_FBLA_CUDA_ERROR = 2
} mlops_fbla_status;

/* The cache of one attention layer (reference: mlops_fbla.h:47-73). All pointers are device memory owned by the caller.
 *
 * coarse / fine: one record per 16-token sub-block, 2*bits*256 bytes (bits = CB resp. FB: 1536, 2048 or 1024 bytes),
 *   holding K and V of the sub-block's 16 tokens. 32 lanes own a record; lane l owns, per tensor, 16 slots of 4 codes:
 *     K: lane l = token l%16, slot s, byte b  -> channel 64*(l/16) + 4*s + b
 *     V: lane l = channels 4l..4l+3, slot s, byte b -> channel 4l + c(s), token 4*j(s) + b with (c, j) =
 *        4 bit: s<8: (s%2, s/2); s>=8: (2 + s%2, (s-8)/2)      2 bit: s = 4m+k: (m, k)
 *        3 bit: s=0..3: (0, s); s=4,5: (2, s-4); s=6..9: (1, s-6); s=10,11: (2, s-8); s=12..15: (3, s-12)
 *   A lane's 16 slots of one tensor occupy 2*bits 32-bit words W[], packed per byte position:
 *     4 bit: slot s<8 in bits 0-3 of W[s]; slot 8+k in bits 4-7 of W[k]
 *     2 bit: slot 4m+k in bits 2m..2m+1 of W[k]
 *     3 bit: slot s<6 in bits 0-2 of W[s]; slot 6+k (k<6) in bits 3-5 of W[k]; slot 12+r: code bits 0-1 in bits 6-7
 *            of W[r], code bit 2 in bit 6 + r%2 of W[4 + r/2]
 *   Byte offset of word w of lane l inside the record:
 *     4 bit: K w<4: 16l+4w; K w>=4: 512+16l+4(w-4); V: the same + 1024
 *     2 bit: K: 16l+4w; V: 512+16l+4w
 *     3 bit: w<4: K 16l+4w, V 512+16l+4w; w=4,5: K 1024 + 16(l%16) + 8(l/16) + 4(w-4), V 1280 + 8l + 4(w-4)
 * meta: 512 BF16 (1 KiB) per group: lane l's K base[4] then step[4] for channels 4l..4l+3 at byte 16l; V's at 512+16l.
 * exact_sink_* / exact_open_*: [batch, kv_heads, 128, 128] BF16; the open group's tokens are rows 0..n-1.
 * Unit placement: the 8 records (planes) / the KiB (meta) of (head h = b*kv_heads + kh, group g) is unit number
 *   h*head_stride + g*group_stride; the defaults (0, 0) mean head_stride = groups of the capacity, group_stride = 1.
 * tc_images: optional persistent prefill images of the reference's mma.sync prefill; this library keeps none
 *   (mlops_fbla_images_bytes returns 0) and ignores the pointer beyond checking its alignment. */
typedef struct {
  uint8_t *coarse, *fine;
  uint16_t *meta;
  uint16_t *exact_sink_k, *exact_sink_v, *exact_open_k, *exact_open_v;
  uint8_t *tc_images;
} mlops_fbla_cache;

/* reference: mlops_fbla.h:75-88 */
typedef struct {
  int batch, q_heads, kv_heads, tokens;
  float scale;   /* 0: 1/sqrt(128) */
  float tau;     /* refinement threshold on a sub-block's share of the softmax mass; 0: the format's default */
  mlops_fbla_format format;
  int capacity;  /* tokens the planes and metadata are laid out for; 0: tokens */
  int head_stride, group_stride; /* units between KV heads / groups; 0, 0: the capacity's dense layout */
  /* prefill output placement (BF16 elements): element (q head h, position i) at h*out_head_stride + i*out_token_stride;
   * 0, 0: [batch, q_heads, count, 128]. Both nonzero requires batch 1 and multiples of 8. */
  int64_t out_head_stride, out_token_stride;
  int length_stride; /* the *_at calls: 0 = one device length for all batch rows, 1 = length[b] per row */
} mlops_fbla_config;

/* reference: mlops_fbla.h:111-116 */
typedef struct {
  size_t coarse, fine, meta;
  size_t exact; /* each of the four exact planes */
  size_t images;
} mlops_fbla_sizes;

/* Bytes of scratch one decode of cfg needs on the current device; 0 for an invalid cfg. The scratch needs no
 * initial contents and may be reused by later calls that fit. reference: mlops_fbla.h:93 */
size_t mlops_fbla_decode_scratch_bytes(const mlops_fbla_config *cfg);

/* One query per q head: q, output [batch, q_heads, 128] BF16. Work is enqueued on `stream`; no host
 * synchronisation. tokens <= 2^26. One call handles at most about 27 500 (virtual head, slice of 16 384 tokens) pairs --
 * batch * kv_heads * max(1, q_heads / kv_heads / 4) * ceil(tokens / 16384) -- beyond which it returns
 * MLOPS_FBLA_INVALID_VALUE ("split the batch"): a limit of this library, not of the reference.
 * A device-side wait that gives up (not seen on a healthy device) turns the affected output rows into NaN.
 * reference: mlops_fbla.h:98-100 */
mlops_fbla_status mlops_fbla_decode(const mlops_fbla_config *cfg, const uint16_t *q,
                                    const mlops_fbla_cache *cache, uint16_t *output,
                                    void *scratch, size_t scratch_bytes, cudaStream_t stream);

/* Bytes of mlops_fbla_cache.tc_images on the current device. This library keeps no images: always 0.
 * reference: mlops_fbla.h:104 */
size_t mlops_fbla_images_bytes(const mlops_fbla_config *cfg);

/* Allocation sizes of a cache for cfg (batch, kv_heads, format, capacity or tokens, strides). Returns 1 and fills
 * *out, or 0 (out untouched) for an invalid cfg. reference: mlops_fbla.h:117 */
int mlops_fbla_cache_sizes(const mlops_fbla_config *cfg, mlops_fbla_sizes *out);

/* Scratch of mlops_fbla_decode_at for cfg->capacity (> 0). per_head (the reference: CTAs per head the partials are laid
 * out for) only enlarges the answer here -- per_head further partial rows per head, so a larger per_head never gives a
 * smaller scratch -- because this library's passes are persistent grids whose shape it does not change.
 * reference: mlops_fbla.h:122 */
size_t mlops_fbla_decode_scratch_bytes_for(const mlops_fbla_config *cfg, int per_head);

/* Append `count` tokens k, v [batch, kv_heads, count, 128] BF16 to a cache holding cfg->tokens tokens: groups that
 * become closed are quantized into the planes and metadata, the sink and open windows take their BF16 rows.
 * With q != NULL (q, output [batch, q_heads, count, 128] BF16) also returns causal attention of the new positions:
 * position tokens+i attends to 0..tokens+i, closed groups through their full 6-bit codes, the sink group and the
 * position's own group in BF16. reference: mlops_fbla.h:130-132 */
mlops_fbla_status mlops_fbla_prefill(const mlops_fbla_config *cfg, int count, const uint16_t *q,
                                     const uint16_t *k, const uint16_t *v, const mlops_fbla_cache *cache,
                                     uint16_t *output, cudaStream_t stream);

/* As mlops_fbla_prefill with the start (*length + cfg->tokens) and *count read on the device when the kernels run;
 * launches are sized by max_count alone. cfg->capacity > 0. reference: mlops_fbla.h:142-144 */
mlops_fbla_status mlops_fbla_prefill_at(const mlops_fbla_config *cfg, const int *length, const int *count, int max_count,
                                        const uint16_t *q, const uint16_t *k, const uint16_t *v,
                                        const mlops_fbla_cache *cache, uint16_t *output, cudaStream_t stream);

/* Decode with the cache length *length (+ cfg->tokens) read on the device; cfg->capacity > 0 sizes the launches and
 * the scratch. reference: mlops_fbla.h:151-153 */
mlops_fbla_status mlops_fbla_decode_at(const mlops_fbla_config *cfg, const int *length, const uint16_t *q,
                                       const mlops_fbla_cache *cache, uint16_t *output, void *scratch, size_t scratch_bytes,
                                       cudaStream_t stream);
/* One token per KV head (k, v [batch, kv_heads, 128]) appended at position *length + cfg->tokens.
 * reference: mlops_fbla.h:154-155 */
mlops_fbla_status mlops_fbla_append_at(const mlops_fbla_config *cfg, const int *length, const uint16_t *k, const uint16_t *v,
                                       const mlops_fbla_cache *cache, cudaStream_t stream);

/* The attention inputs of new tokens as the model's projection leaves them. q head h of KV head g = h / (q_heads /
 * kv_heads) of batch row b starts at q + b * batch_stride + g * q_group_stride + (h % (q_heads / kv_heads)) * 128; k and
 * v of KV head g at k / v + b * batch_stride + g * kv_group_stride (strides in elements; BF16, 128 per head; 4-byte
 * aligned). q_norm / k_norm: a head's RMSNorm weights (128 BF16 each), or both NULL for no norm; eps is the norm's.
 * freq: device, 64 x 4 floats per rotary pair (i, i + 64), each frequency f = inv_freq / 2 pi split as (fh, fl) with
 * fh = float(f), fl = float(f - fh), and g = frac(65536 f) split the same way (gh, gl). attention_factor 0 means 1.
 * q_out [batch, q_heads, 128] BF16: the q that mlops_fbla_decode_at takes. 96 bytes. reference: mlops_fbla.h:157-167 */
typedef struct {
  const uint16_t *q, *k, *v;
  int64_t batch_stride, q_group_stride, kv_group_stride;
  const uint16_t *q_norm, *k_norm;
  float eps;
  const float *freq;
  float attention_factor;
  uint16_t *q_out;
} mlops_fbla_token;

/* One decode step's attention inputs at the device length (position *length + cfg->tokens; per-row lengths with
 * cfg->length_stride 1): per head the RMSNorm of q and k (FP32 sum of squares, 1 / sqrt(mean + eps) rounded to nearest,
 * x r rounded to BF16, times the weight rounded to BF16), the rotary embedding (phase reduced exactly, one rounding to
 * BF16), q to token->q_out, k and v appended to the cache as mlops_fbla_append_at does. cfg->capacity > 0; launches do
 * not depend on the length. reference: mlops_fbla.h:169-173 */
mlops_fbla_status mlops_fbla_qkv_at(const mlops_fbla_config *cfg, const int *length, const mlops_fbla_token *token,
                                    const mlops_fbla_cache *cache, cudaStream_t stream);

/* The attention inputs of a prefill chunk of *count (<= max_count) tokens at the device length: token->q / k / v point
 * at row 0 of the projection's [count][token->batch_stride] BF16 rows (group strides as for one token); per position
 * the RMSNorm of q and k and the rotary embedding at *length + cfg->tokens + i; written as mlops_fbla_prefill_at takes
 * them: q_out [q_heads, max_count, 128], k_out, v_out [kv_heads, max_count, 128] BF16 (token->q_out unused). Batch 1;
 * rows past *count are not written; launches depend on neither *length nor *count. reference: mlops_fbla.h:175-181 */
mlops_fbla_status mlops_fbla_qkv_prefill_at(const mlops_fbla_config *cfg, const int *length, const int *count, int max_count,
                                            const mlops_fbla_token *token, uint16_t *q_out, uint16_t *k_out, uint16_t *v_out,
                                            cudaStream_t stream);

/* Decode without a caller-provided scratch, for callers that cannot allocate device memory (an engine whose allocator
 * is closed after start-up, a plugin host that forbids cudaMalloc, a real-time loop): the scratch is a 32 MiB array
 * inside the library image, held by every GPU that loads the library until the process exits. Same arguments and
 * results as mlops_fbla_decode otherwise. Configurations whose scratch (mlops_fbla_decode_scratch_bytes) exceeds
 * mlops_fbla_decode_static_scratch_limit() are rejected with MLOPS_FBLA_INVALID_VALUE. The first call on a device
 * looks the array's device address up and should come before any stream capture; all calls on a device share the
 * array, so calls that overlap on the GPU race (keep them on one stream). Error text: mlops_fbla_decode_static_error().
 * This entry point has no counterpart in the reference interface. */
mlops_fbla_status mlops_fbla_decode_static(const mlops_fbla_config *cfg, const uint16_t *q, const mlops_fbla_cache *cache,
                                           uint16_t *output, cudaStream_t stream);
size_t mlops_fbla_decode_static_scratch_limit(void);
const char *mlops_fbla_decode_static_error(void);
/* Optional, once per device at start-up (that device current), before the caller takes its memory arena and before any
 * capture: makes the driver load this library's module on the device -- which is when the 32 MiB array and the kernels'
 * code get their device memory -- and looks the array's address up. Launches nothing. No counterpart in the reference. */
mlops_fbla_status mlops_fbla_decode_static_prepare(void);

/* reference: mlops_fbla.h:185-186 */
const char *mlops_fbla_status_string(mlops_fbla_status status);
const char *mlops_fbla_last_error(void); /* thread-local; "" after a successful call */

#ifdef __cplusplus
}
#endif
#endif /* MLOPS_FBLA_H */
