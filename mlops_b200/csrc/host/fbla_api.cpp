// Host layer of the FBLA library: checks a call's arguments, lays out the decode scratch, fills the kernels' plain
// argument structures and enqueues the passes on the caller's stream. It accepts and rejects what the reference's host
// code accepts and rejects and returns the same status codes (attention/fbla/src/fbla.cu:62-80 shape rules, :90-138
// decode, :193-268 prefill, :307-382 fused QKV step, :408-430 size queries) behind the same C interface
// (include/mlops_fbla.h); the wording of the messages is this library's own. Nothing here allocates or synchronises;
// the only state is per host thread (the last message, a per-device cache of launch attributes), so any number of
// host threads may call in at once.
#include "../../../include/mlops_fbla.h"
#include "../../../include/mlops_fbla_shard.h"
#include "../../../include/mlops_fbla_items.h"
#include "../kernels/fbla_kernels.h"

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>

namespace {

constexpr int kGroup = MLOPS_FBLA_GROUP, kBlocksPerGroup = MLOPS_FBLA_GROUP / MLOPS_FBLA_SUBBLOCK, kHeadDim = MLOPS_FBLA_HEAD_DIM;
constexpr long long kTokenLimit = 1ll << 26;

// ---- the calling thread's last message ------------------------------------------------------------------------------------
thread_local char g_message[256] = "";

// "<function>: <what is wrong>", status INVALID_VALUE
mlops_fbla_status refuse(const char *function, const char *format, ...) {
  const int used = snprintf(g_message, sizeof g_message, "%s: ", function);
  va_list args;
  va_start(args, format);
  if (used >= 0 && (size_t)used < sizeof g_message) vsnprintf(g_message + used, sizeof g_message - (size_t)used, format, args);
  va_end(args);
  return MLOPS_FBLA_INVALID_VALUE;
}
mlops_fbla_status device_failure(const char *function, cudaError_t error) {
  snprintf(g_message, sizeof g_message, "%s: CUDA reports \"%s\"", function, cudaGetErrorString(error));
  return MLOPS_FBLA_CUDA_ERROR;
}
mlops_fbla_status accepted() {
  g_message[0] = '\0';
  return MLOPS_FBLA_OK;
}

// ---- small predicates ---------------------------------------------------------------------------------------------------------
bool on_boundary(const void *pointer, uintptr_t bytes) { return reinterpret_cast<uintptr_t>(pointer) % bytes == 0; }
template <size_t N> bool all_on_boundary(const void *const (&pointers)[N], uintptr_t bytes) {
  for (const void *p : pointers)
    if (!on_boundary(p, bytes)) return false;
  return true;
}
size_t padded(size_t bytes) { return (bytes + 255) / 256 * 256; }  // scratch arrays start on 256-byte boundaries
bool known_format(const mlops_fbla_config *c) { return c->format == MLOPS_FBLA_3P3 || c->format == MLOPS_FBLA_4P2; }
int coarse_bits(const mlops_fbla_config *c) { return c->format == MLOPS_FBLA_3P3 ? 3 : 4; }
int fine_bits(const mlops_fbla_config *c) { return c->format == MLOPS_FBLA_3P3 ? 3 : 2; }
// unit strides: give both or neither
bool unit_strides_consistent(const mlops_fbla_config *c) {
  const bool none = c->head_stride == 0 && c->group_stride == 0, both = c->head_stride > 0 && c->group_stride > 0;
  return none || both;
}
// output strides: neither, or both as positive multiples of 8 elements (16-byte rows) for a single batch row
bool output_strides_usable(const mlops_fbla_config *c) {
  const long long hs = c->out_head_stride, ts = c->out_token_stride;
  if (hs == 0 && ts == 0) return true;
  if (hs <= 0 || ts <= 0 || c->batch != 1) return false;
  return hs % 8 == 0 && ts % 8 == 0 && ts < (1ll << 30);
}
bool heads_consistent(const mlops_fbla_config *c) {
  return c->batch > 0 && c->q_heads > 0 && c->kv_heads > 0 && c->q_heads % c->kv_heads == 0;
}
// A KV head with `ratio` queries is served as virtual heads of 4, 2 or 1 queries: the ratio itself up to 4 (3 -> 1),
// beyond that the largest of 4, 2, 1 that divides it.
int queries_per_virtual_head(int ratio) {
  if (ratio == 1 || ratio == 2 || ratio == 4) return ratio;
  return ratio % 4 == 0 ? 4 : ratio % 2 == 0 ? 2 : 1;
}
// softmax scale times log2(e): scores live in the log2 domain
float log2_scale(const mlops_fbla_config *c) {
  const float natural = c->scale == 0.f ? 1.f / sqrtf((float)kHeadDim) : c->scale;
  return natural * 1.4426950408889634f;
}
bool all_cache_arrays_given(const mlops_fbla_cache *k) {
  const void *const arrays[] = {k->coarse, k->fine, k->meta, k->exact_sink_k, k->exact_sink_v, k->exact_open_k, k->exact_open_v};
  for (const void *p : arrays)
    if (!p) return false;
  return true;
}
fbla_k_cache kernel_cache(const mlops_fbla_cache *k) {
  return fbla_k_cache{k->coarse, k->fine, k->meta, k->exact_sink_k, k->exact_sink_v, k->exact_open_k, k->exact_open_v};
}
long long groups_of(long long tokens) { return (tokens + kGroup - 1) / kGroup; }

// ---- decode scratch ------------------------------------------------------------------------------------------------------------
// Byte offsets of the arrays fbla_kernels.h describes, in this order, inside the caller's scratch.
struct ScratchMap {
  size_t lse, part, dpart, row_r, counts, items, item_off, status, bytes;
  int nblocks, nslices;
};
// `shape`: the launch shape on the current device; `tokens`: what the layout has room for; extra_rows: partial rows per
// virtual head beyond the shape's own (the per_head of the size query)
ScratchMap map_scratch(const mlops_fbla_config *c, long long tokens, const fbla_k_decode &shape, int extra_rows) {
  ScratchMap m{};
  const int ratio = c->q_heads / c->kv_heads, qg = queries_per_virtual_head(ratio);
  const size_t vheads = (size_t)c->batch * c->kv_heads * (ratio / qg);
  m.nblocks = (int)(groups_of(tokens) * kBlocksPerGroup);
  m.nslices = (m.nblocks + FBLA_K_SLICE - 1) / FBLA_K_SLICE;
  if (m.nslices < 1) m.nslices = 1;
  const size_t row_bytes = (size_t)qg * FBLA_K_PSTRIDE * sizeof(float);
  // partial rows: coarse slot (writer + virtual head) for up to coarse_warps writers per CTA, the same again for the
  // window warps; corrections: refine slot (warp + virtual head)
  const size_t coarse_rows = 2 * ((size_t)shape.coarse_ctas * shape.coarse_warps + vheads) + (size_t)extra_rows * vheads;
  const size_t refine_rows = (size_t)shape.refine_ctas * shape.refine_warps + vheads;
  size_t at = 0;
  auto take = [&at](size_t bytes) { const size_t here = at; at += padded(bytes); return here; };
  m.lse = take(vheads * m.nblocks * qg * sizeof(float));
  m.part = take(coarse_rows * row_bytes);
  m.dpart = take(refine_rows * row_bytes);
  m.row_r = take(vheads * qg * sizeof(float));
  m.counts = take(vheads * m.nslices * sizeof(int));
  m.items = take(vheads * m.nslices * FBLA_K_SLICE * sizeof(int));
  m.item_off = take((vheads + 1) * sizeof(int));
  m.status = take(16);
  m.bytes = at;
  return m;
}
// c->tokens here is the token count the LAYOUT is made for
bool decode_shape_acceptable(const mlops_fbla_config *c) {
  if (!c || !heads_consistent(c) || !unit_strides_consistent(c)) return false;
  if (c->tokens <= 0 || c->tokens > kTokenLimit) return false;
  return c->capacity == 0 || c->capacity >= c->tokens;
}
size_t scratch_size(const mlops_fbla_config *layout, int extra_rows) {
  fbla_k_decode shape{};
  shape.cb = coarse_bits(layout);
  if (fbla_k_decode_shape(&shape) != cudaSuccess) return 0;
  return map_scratch(layout, layout->tokens, shape, extra_rows).bytes;
}

// Checks a decode and fills the kernels' arguments. `length` non-null: a device-length call, laid out by cfg->capacity.
// `out` may be null when the caller is one of the shard passes (wants_output false).
mlops_fbla_status make_decode(const char *fn, const mlops_fbla_config *c, const int *length, const uint16_t *q, const mlops_fbla_cache *k,
                              uint16_t *out, bool wants_output, void *scratch, size_t scratch_bytes, fbla_k_decode &a) {
  if (!c || !q || !k || !scratch || (wants_output && !out)) return refuse(fn, "a required pointer is null");
  const bool device_length = length != nullptr;
  mlops_fbla_config layout = *c;
  if (device_length) layout.tokens = c->capacity;
  if (!decode_shape_acceptable(&layout) || (device_length && c->tokens < 0))
    return refuse(fn, "needs batch, q_heads, kv_heads > 0 with kv_heads dividing q_heads; %s; at most 2^26 tokens; capacity 0 or no "
                      "smaller than tokens; head_stride and group_stride given together or not at all",
                  device_length ? "capacity > 0 and a token offset >= 0" : "tokens > 0");
  if (!known_format(c)) return refuse(fn, "format %d is neither MLOPS_FBLA_3P3 nor MLOPS_FBLA_4P2", (int)c->format);
  if (!(c->scale >= 0.f) || !(c->tau >= 0.f)) return refuse(fn, "scale and tau may not be negative or NaN");
  if (!all_cache_arrays_given(k)) return refuse(fn, "the cache lacks one of its seven arrays");
  const void *const wide[] = {q, out, scratch, k->coarse, k->fine, k->meta, k->exact_sink_k, k->exact_sink_v, k->exact_open_k, k->exact_open_v};
  if (!all_on_boundary(wide, 16)) return refuse(fn, "q, output, scratch and the cache arrays have to start on 16-byte boundaries");
  if (!on_boundary(length, 4)) return refuse(fn, "the device length has to start on a 4-byte boundary");
  if (c->length_stride != 0 && !(c->length_stride == 1 && device_length))
    return refuse(fn, "length_stride %d: only 0, or 1 together with a device length", c->length_stride);

  a = fbla_k_decode{};
  a.cb = coarse_bits(c);
  a.fb = fine_bits(c);
  const cudaError_t shape_error = fbla_k_decode_shape(&a);
  if (shape_error != cudaSuccess) return device_failure(fn, shape_error);
  const ScratchMap m = map_scratch(&layout, layout.tokens, a, 0);
  if (scratch_bytes < m.bytes) return refuse(fn, "the scratch is %zu bytes but this decode takes %zu", scratch_bytes, m.bytes);
  const int ratio = c->q_heads / c->kv_heads;
  a.qg = queries_per_virtual_head(ratio);
  a.vg = ratio / a.qg;
  // the refine pass keeps one prefix entry per (virtual head, slice of 16 384 tokens) in shared memory
  const long long entries = (long long)c->batch * c->kv_heads * a.vg * m.nslices, entry_limit = fbla_k_refine_entry_limit(a.cb);
  if (entries > entry_limit)
    return refuse(fn, "batch * kv_heads * virtual heads * slices of 16384 tokens = %lld is more than the %lld one call handles: split the batch",
                  entries, entry_limit);
  a.c = kernel_cache(k);
  a.q = q;
  a.out = out;
  char *const base = static_cast<char *>(scratch);
  a.lse = reinterpret_cast<float *>(base + m.lse);
  a.part = reinterpret_cast<float *>(base + m.part);
  a.dpart = reinterpret_cast<float *>(base + m.dpart);
  a.row_r = reinterpret_cast<float *>(base + m.row_r);
  a.counts = reinterpret_cast<int *>(base + m.counts);
  a.items = reinterpret_cast<int *>(base + m.items);
  a.item_off = reinterpret_cast<int *>(base + m.item_off);
  a.status = reinterpret_cast<int *>(base + m.status);
  a.length = length;
  a.lstride = c->length_stride;
  a.batch = c->batch;
  a.q_heads = c->q_heads;
  a.kv_heads = c->kv_heads;
  a.tokens = c->tokens;
  a.nblocks = m.nblocks;
  a.nslices = m.nslices;
  const long long room = c->capacity ? c->capacity : c->tokens;
  a.hs = c->head_stride ? c->head_stride : (int)groups_of(room);
  a.gs = c->group_stride ? c->group_stride : 1;
  a.sl = log2_scale(c);
  // Which coarse kernel runs is decided by the cache's room where it has one, for host and device lengths alike: both
  // calls on one cache then run the same kernels and return the same bits.
  fbla_k_decode_split(&a, room);
  const float threshold = c->tau != 0.f ? c->tau : (c->format == MLOPS_FBLA_3P3 ? 3e-4f : 1e-3f);
  a.log2_tau = log2f(threshold);
  return MLOPS_FBLA_OK;
}
mlops_fbla_status enqueue_decode(const char *fn, fbla_k_decode &a, cudaStream_t stream) {
  a.status_cleared = 1;  // the launcher zeroes the status word on the stream, ahead of the first pass
  const cudaError_t e = fbla_k_decode_launch(&a, stream);
  return e == cudaSuccess ? accepted() : device_failure(fn, e);
}
mlops_fbla_status run_decode(const char *fn, const mlops_fbla_config *c, const int *length, const uint16_t *q, const mlops_fbla_cache *k,
                             uint16_t *out, void *scratch, size_t scratch_bytes, cudaStream_t stream) {
  fbla_k_decode a;
  const mlops_fbla_status st = make_decode(fn, c, length, q, k, out, true, scratch, scratch_bytes, a);
  return st == MLOPS_FBLA_OK ? enqueue_decode(fn, a, stream) : st;
}

// ---- prefill family ---------------------------------------------------------------------------------------------------------------
// what every chunk call checks after its shape: layout options, format, scale, the cache, alignments
mlops_fbla_status check_chunk_operands(const char *fn, const mlops_fbla_config *c, const uint16_t *q, const uint16_t *k, const uint16_t *v,
                                       const mlops_fbla_cache *cache, uint16_t *out) {
  if (!output_strides_usable(c))
    return refuse(fn, "out_head_stride / out_token_stride: leave both 0, or give both as positive multiples of 8 (token stride below 2^30) "
                      "with batch 1");
  if (!known_format(c)) return refuse(fn, "format %d is neither MLOPS_FBLA_3P3 nor MLOPS_FBLA_4P2", (int)c->format);
  if (!(c->scale >= 0.f)) return refuse(fn, "scale may not be negative or NaN");
  if (!all_cache_arrays_given(cache)) return refuse(fn, "the cache lacks one of its seven arrays");
  const void *const wide[] = {q, k, v, out, cache->coarse, cache->fine, cache->meta, cache->exact_sink_k, cache->exact_sink_v,
                              cache->exact_open_k, cache->exact_open_v};
  if (!all_on_boundary(wide, 16)) return refuse(fn, "q, k, v, output and the cache arrays have to start on 16-byte boundaries");
  if (!on_boundary(cache->tc_images, 128)) return refuse(fn, "tc_images has to start on a 128-byte boundary");
  return MLOPS_FBLA_OK;
}
void fill_chunk(const mlops_fbla_config *c, int count, long long room, const uint16_t *q, const uint16_t *k, const uint16_t *v,
                const mlops_fbla_cache *cache, uint16_t *out, fbla_k_prefill &a) {
  a.c = kernel_cache(cache);
  a.q = q;
  a.k = k;
  a.v = v;
  a.out = out;
  a.out_hs = c->out_head_stride ? c->out_head_stride : (int64_t)count * kHeadDim;  // default: [batch, q_heads, count, 128]
  a.out_ts = c->out_token_stride ? (int)c->out_token_stride : kHeadDim;
  a.batch = c->batch;
  a.q_heads = c->q_heads;
  a.kv_heads = c->kv_heads;
  a.n0 = c->tokens;
  a.count = count;
  a.hs = c->head_stride ? c->head_stride : (int)groups_of(room);
  a.gs = c->group_stride ? c->group_stride : 1;
  a.cb = coarse_bits(c);
  a.fb = fine_bits(c);
  a.sl = log2_scale(c);
}
// The passes in the order that keeps them correct: closing groups reads the windows as they were, the attention reads
// them too, and only then are the windows rewritten.
mlops_fbla_status enqueue_chunk(const char *fn, const fbla_k_prefill &a, int closable_groups, cudaStream_t stream) {
  cudaError_t e = fbla_k_close_launch(&a, closable_groups, stream);
  if (e == cudaSuccess && a.q) e = fbla_k_attend_launch(&a, stream);
  if (e == cudaSuccess) e = fbla_k_finish_launch(&a, stream);
  return e == cudaSuccess ? accepted() : device_failure(fn, e);
}
// device-length chunk (prefill_at, append_at and their plans)
mlops_fbla_status make_chunk_at(const char *fn, const mlops_fbla_config *c, const int *length, const int *device_count, int max_count,
                                const uint16_t *q, const uint16_t *k, const uint16_t *v, const mlops_fbla_cache *cache, uint16_t *out,
                                fbla_k_prefill &a) {
  if (!c || !length || !cache || !k || !v) return refuse(fn, "a required pointer is null");
  if (q && !out) return refuse(fn, "queries were given but no output to write their attention to");
  const bool shape_ok = heads_consistent(c) && unit_strides_consistent(c) && c->tokens >= 0 && max_count > 0 && c->capacity > 0 &&
                        c->capacity <= kTokenLimit && (long long)c->tokens + max_count <= c->capacity;
  if (!shape_ok)
    return refuse(fn, "needs batch, q_heads, kv_heads > 0 with kv_heads dividing q_heads; a token offset >= 0; max_count > 0; "
                      "offset + max_count within a capacity of at most 2^26; head_stride and group_stride given together or not at all");
  if (c->length_stride != 0 && !(c->length_stride == 1 && !q && !device_count))
    return refuse(fn, "length_stride %d: per-row lengths (1) exist for the one-token append only", c->length_stride);
  const mlops_fbla_status st = check_chunk_operands(fn, c, q, k, v, cache, out);
  if (st != MLOPS_FBLA_OK) return st;
  if (!on_boundary(length, 4) || !on_boundary(device_count, 4)) return refuse(fn, "the device length and count have to start on 4-byte boundaries");
  a = fbla_k_prefill{};
  fill_chunk(c, max_count, c->capacity, q, k, v, cache, out, a);
  a.length = length;
  a.dcount = device_count;
  a.lstride = c->length_stride;
  return MLOPS_FBLA_OK;
}
mlops_fbla_status run_chunk_at(const char *fn, const mlops_fbla_config *c, const int *length, const int *device_count, int max_count,
                               const uint16_t *q, const uint16_t *k, const uint16_t *v, const mlops_fbla_cache *cache, uint16_t *out,
                               cudaStream_t stream) {
  fbla_k_prefill a;
  const mlops_fbla_status st = make_chunk_at(fn, c, length, device_count, max_count, q, k, v, cache, out, a);
  // wherever it starts, a chunk of max_count tokens completes at most max_count / 128 + 1 groups
  return st == MLOPS_FBLA_OK ? enqueue_chunk(fn, a, max_count / kGroup + 1, stream) : st;
}

}  // namespace

extern "C" {

size_t mlops_fbla_decode_scratch_bytes(const mlops_fbla_config *c) {
  return decode_shape_acceptable(c) && known_format(c) ? scratch_size(c, 0) : 0;
}

// per_head: partial rows per virtual head an executor wants room for on top of this library's own launch shape. The
// plans always use the library's persistent grid; a larger per_head only enlarges the answer, never shrinks it.
size_t mlops_fbla_decode_scratch_bytes_for(const mlops_fbla_config *c, int per_head) {
  if (!c || per_head < 0 || c->capacity <= 0) return 0;
  mlops_fbla_config layout = *c;
  layout.tokens = c->capacity;
  return decode_shape_acceptable(&layout) && known_format(c) ? scratch_size(&layout, per_head) : 0;
}

mlops_fbla_status mlops_fbla_decode(const mlops_fbla_config *c, const uint16_t *q, const mlops_fbla_cache *k, uint16_t *out,
                                    void *scratch, size_t scratch_bytes, cudaStream_t stream) {
  return run_decode("mlops_fbla_decode", c, nullptr, q, k, out, scratch, scratch_bytes, stream);
}

mlops_fbla_status mlops_fbla_decode_at(const mlops_fbla_config *c, const int *length, const uint16_t *q, const mlops_fbla_cache *k,
                                       uint16_t *out, void *scratch, size_t scratch_bytes, cudaStream_t stream) {
  constexpr const char *fn = "mlops_fbla_decode_at";
  if (!length) return refuse(fn, "the device length pointer is null");
  if (c && c->capacity <= 0) return refuse(fn, "a device-length decode is laid out by capacity, which has to be positive");
  return run_decode(fn, c, length, q, k, out, scratch, scratch_bytes, stream);
}

size_t mlops_fbla_images_bytes(const mlops_fbla_config *) { return 0; }  // no persistent prefill images in this library

int mlops_fbla_cache_sizes(const mlops_fbla_config *c, mlops_fbla_sizes *out) {
  if (!c || !out || !heads_consistent(c) || !unit_strides_consistent(c) || !known_format(c)) return 0;
  const long long room = c->capacity ? c->capacity : c->tokens;
  if (room <= 0 || (c->capacity != 0 && c->capacity < c->tokens)) return 0;
  const size_t heads = (size_t)c->batch * c->kv_heads, groups = (size_t)groups_of(room);
  const size_t head_step = c->head_stride ? (size_t)c->head_stride : groups, group_step = c->group_stride ? (size_t)c->group_stride : 1;
  const size_t units = (heads - 1) * head_step + (groups - 1) * group_step + 1;  // up to the last unit any (head, group) maps to
  out->coarse = units * kBlocksPerGroup * (size_t)(512 * coarse_bits(c));
  out->fine = units * kBlocksPerGroup * (size_t)(512 * fine_bits(c));
  out->meta = units * 1024;
  out->exact = heads * kGroup * kHeadDim * sizeof(uint16_t);
  out->images = 0;
  return 1;
}

mlops_fbla_status mlops_fbla_prefill(const mlops_fbla_config *c, int count, const uint16_t *q, const uint16_t *k, const uint16_t *v,
                                     const mlops_fbla_cache *cache, uint16_t *out, cudaStream_t stream) {
  constexpr const char *fn = "mlops_fbla_prefill";
  if (!c || !cache || !k || !v) return refuse(fn, "a required pointer is null");
  if (q && !out) return refuse(fn, "queries were given but no output to write their attention to");
  const long long end = (long long)c->tokens + count;
  const bool shape_ok = heads_consistent(c) && unit_strides_consistent(c) && c->tokens >= 0 && count > 0 && end <= kTokenLimit &&
                        (c->capacity == 0 || c->capacity >= end);
  if (!shape_ok)
    return refuse(fn, "needs batch, q_heads, kv_heads > 0 with kv_heads dividing q_heads; tokens >= 0; count > 0; tokens + count within the "
                      "capacity (when one is given) and 2^26; head_stride and group_stride given together or not at all");
  const mlops_fbla_status st = check_chunk_operands(fn, c, q, k, v, cache, out);
  if (st != MLOPS_FBLA_OK) return st;
  fbla_k_prefill a{};
  fill_chunk(c, count, c->capacity ? c->capacity : end, q, k, v, cache, out, a);
  // groups completed by this chunk: those whose last token lies before `end` and that were still open before it
  const int first_open = c->tokens == 0 ? 0 : (c->tokens - 1) / kGroup, last_open = (int)((end - 1) / kGroup);
  return enqueue_chunk(fn, a, last_open - first_open, stream);
}

mlops_fbla_status mlops_fbla_prefill_at(const mlops_fbla_config *c, const int *length, const int *count, int max_count, const uint16_t *q,
                                        const uint16_t *k, const uint16_t *v, const mlops_fbla_cache *cache, uint16_t *out,
                                        cudaStream_t stream) {
  constexpr const char *fn = "mlops_fbla_prefill_at";
  if (!count) return refuse(fn, "a required pointer is null");
  return run_chunk_at(fn, c, length, count, max_count, q, k, v, cache, out, stream);
}

mlops_fbla_status mlops_fbla_append_at(const mlops_fbla_config *c, const int *length, const uint16_t *k, const uint16_t *v,
                                       const mlops_fbla_cache *cache, cudaStream_t stream) {
  return run_chunk_at("mlops_fbla_append_at", c, length, nullptr, 1, nullptr, k, v, cache, nullptr, stream);
}

// ---- fused QKV step (reference rules: attention/fbla/src/fbla.cu:307-400) ----------------------------------------------------
static mlops_fbla_status fill_token_common(const char *fn, const mlops_fbla_token *t, fbla_k_token &a) {
  if ((t->q_norm == nullptr) != (t->k_norm == nullptr)) return refuse(fn, "give the norm weights of q and k both or neither");
  if (!(t->eps >= 0.f) || !(t->attention_factor >= 0.f)) return refuse(fn, "eps and attention_factor may not be negative or NaN");
  a.q = t->q;
  a.k = t->k;
  a.v = t->v;
  a.batch_stride = t->batch_stride;
  a.q_group_stride = t->q_group_stride;
  a.kv_group_stride = t->kv_group_stride;
  a.q_norm = t->q_norm;
  a.k_norm = t->k_norm;
  a.freq = t->freq;
  a.eps = t->eps;
  a.att = t->attention_factor == 0.f ? 1.f : t->attention_factor;
  return MLOPS_FBLA_OK;
}

static mlops_fbla_status make_token_step(const mlops_fbla_config *c, const int *length, const mlops_fbla_token *t, const mlops_fbla_cache *cache,
                                         fbla_k_prefill &closing, fbla_k_token &a) {
  constexpr const char *fn = "mlops_fbla_qkv_at";
  if (!c || !length || !t || !cache || !t->q || !t->k || !t->v || !t->freq || !t->q_out) return refuse(fn, "a required pointer is null");
  if (!heads_consistent(c) || !unit_strides_consistent(c) || c->tokens < 0 || c->capacity <= 0)
    return refuse(fn, "needs batch, q_heads, kv_heads > 0 with kv_heads dividing q_heads; a token offset >= 0; capacity > 0; "
                      "head_stride and group_stride given together or not at all");
  if (!known_format(c)) return refuse(fn, "format %d is neither MLOPS_FBLA_3P3 nor MLOPS_FBLA_4P2", (int)c->format);
  a = fbla_k_token{};
  const mlops_fbla_status st = fill_token_common(fn, t, a);
  if (st != MLOPS_FBLA_OK) return st;
  if (!all_cache_arrays_given(cache)) return refuse(fn, "the cache lacks one of its seven arrays");
  const void *const wide[] = {cache->coarse, cache->fine, cache->meta, cache->exact_sink_k, cache->exact_sink_v, cache->exact_open_k,
                              cache->exact_open_v, t->freq};
  if (!all_on_boundary(wide, 16)) return refuse(fn, "the cache arrays and freq have to start on 16-byte boundaries");
  const void *const narrow[] = {length, t->q, t->k, t->v, t->q_norm, t->k_norm, t->q_out};
  if (!all_on_boundary(narrow, 4)) return refuse(fn, "the device length and the token's tensors have to start on 4-byte boundaries");
  const int64_t strides[] = {t->batch_stride, t->q_group_stride, t->kv_group_stride};
  for (const int64_t stride : strides) {
    if (stride % 2) return refuse(fn, "an odd stride: head rows are read as 4-byte words, strides have to be even");
    if (stride < 0 || stride > INT32_MAX) return refuse(fn, "strides lie between 0 and 2^31 - 1 elements");
  }
  if (!on_boundary(cache->tc_images, 128)) return refuse(fn, "tc_images has to start on a 128-byte boundary");
  if (c->length_stride != 0 && c->length_stride != 1) return refuse(fn, "length_stride %d: only 0 or 1", c->length_stride);
  // a position that is a multiple of 128 completes the previous group: it is quantized from the open window first
  closing = fbla_k_prefill{};
  fill_chunk(c, 1, c->capacity, nullptr, nullptr, nullptr, cache, nullptr, closing);
  closing.length = length;
  closing.lstride = c->length_stride;
  a.c = closing.c;
  a.length = length;
  a.lstride = c->length_stride;
  a.n0 = c->tokens;
  a.max_count = 1;
  a.batch = c->batch;
  a.q_heads = c->q_heads;
  a.kv_heads = c->kv_heads;
  a.q_out = t->q_out;
  return MLOPS_FBLA_OK;
}
mlops_fbla_status mlops_fbla_qkv_at(const mlops_fbla_config *c, const int *length, const mlops_fbla_token *t, const mlops_fbla_cache *cache,
                                    cudaStream_t stream) {
  fbla_k_prefill closing;
  fbla_k_token a;
  const mlops_fbla_status st = make_token_step(c, length, t, cache, closing, a);
  if (st != MLOPS_FBLA_OK) return st;
  cudaError_t e = fbla_k_close_launch(&closing, 1, stream);
  if (e == cudaSuccess) e = fbla_k_qkv_token_launch(&a, stream);
  return e == cudaSuccess ? accepted() : device_failure("mlops_fbla_qkv_at", e);
}

static mlops_fbla_status make_token_chunk(const mlops_fbla_config *c, const int *length, const int *count, int max_count, const mlops_fbla_token *t,
                                          uint16_t *q_out, uint16_t *k_out, uint16_t *v_out, fbla_k_token &a) {
  constexpr const char *fn = "mlops_fbla_qkv_prefill_at";
  if (!c || !length || !count || !t || !t->q || !t->k || !t->v || !t->freq || !q_out || !k_out || !v_out)
    return refuse(fn, "a required pointer is null");
  const bool shape_ok = c->batch == 1 && c->kv_heads > 0 && c->q_heads > 0 && c->q_heads % c->kv_heads == 0 && c->tokens >= 0 && max_count > 0 &&
                        c->capacity > 0 && (long long)c->tokens + max_count <= c->capacity;
  if (!shape_ok)
    return refuse(fn, "works on batch 1 with q_heads, kv_heads > 0 (kv_heads dividing q_heads), a token offset >= 0, max_count > 0 and "
                      "offset + max_count within the capacity");
  a = fbla_k_token{};
  const mlops_fbla_status st = fill_token_common(fn, t, a);
  if (st != MLOPS_FBLA_OK) return st;
  const bool strides_ok = t->batch_stride >= kHeadDim && t->batch_stride % 2 == 0 && t->q_group_stride >= 0 && t->q_group_stride % 2 == 0 &&
                          t->kv_group_stride >= 0 && t->kv_group_stride % 2 == 0;
  if (!strides_ok) return refuse(fn, "batch_stride is the stride between projection rows: even and at least one head (128); the group strides even, >= 0");
  const void *const wide[] = {q_out, k_out, v_out, t->freq};
  if (!all_on_boundary(wide, 16)) return refuse(fn, "q_out, k_out, v_out and freq have to start on 16-byte boundaries");
  const void *const narrow[] = {length, count, t->q, t->k, t->v, t->q_norm, t->k_norm};
  if (!all_on_boundary(narrow, 4)) return refuse(fn, "length, count and the projection's tensors have to start on 4-byte boundaries");
  a.length = length;
  a.dcount = count;
  a.n0 = c->tokens;
  a.max_count = max_count;
  a.batch = 1;
  a.q_heads = c->q_heads;
  a.kv_heads = c->kv_heads;
  a.q_out = q_out;
  a.k_out = k_out;
  a.v_out = v_out;
  return MLOPS_FBLA_OK;
}
mlops_fbla_status mlops_fbla_qkv_prefill_at(const mlops_fbla_config *c, const int *length, const int *count, int max_count, const mlops_fbla_token *t,
                                            uint16_t *q_out, uint16_t *k_out, uint16_t *v_out, cudaStream_t stream) {
  fbla_k_token a;
  const mlops_fbla_status st = make_token_chunk(c, length, count, max_count, t, q_out, k_out, v_out, a);
  if (st != MLOPS_FBLA_OK) return st;
  const cudaError_t e = fbla_k_qkv_chunk_launch(&a, stream);
  return e == cudaSuccess ? accepted() : device_failure("mlops_fbla_qkv_prefill_at", e);
}

// ---- sequence shards (include/mlops_fbla_shard.h) ------------------------------------------------------------------------
static mlops_fbla_status apply_shard(const char *fn, const mlops_fbla_shard *sh, fbla_k_decode &a) {
  if (!sh || sh->group_first < 0 || sh->group_count < 0 || (sh->windows & ~3))
    return refuse(fn, "the shard descriptor needs group_first >= 0, group_count >= 0 and windows within 0..3");
  a.shard_on = 1;
  a.sh_first = sh->group_first;
  a.sh_count = sh->group_count;
  a.sh_windows = sh->windows;
  return MLOPS_FBLA_OK;
}

mlops_fbla_status mlops_fbla_shard_mass(const mlops_fbla_config *c, const mlops_fbla_shard *sh, const uint16_t *q, const mlops_fbla_cache *k,
                                        float *row_mass, void *scratch, size_t scratch_bytes, cudaStream_t stream) {
  constexpr const char *fn = "mlops_fbla_shard_mass";
  if (!row_mass || !on_boundary(row_mass, 16)) return refuse(fn, "row_mass has to be a device pointer on a 16-byte boundary");
  fbla_k_decode a;
  mlops_fbla_status st = make_decode(fn, c, nullptr, q, k, nullptr, false, scratch, scratch_bytes, a);
  if (st == MLOPS_FBLA_OK) st = apply_shard(fn, sh, a);
  if (st != MLOPS_FBLA_OK) return st;
  a.phase = 1;
  a.row_r = row_mass;
  return enqueue_decode(fn, a, stream);
}

mlops_fbla_status mlops_fbla_shard_partial(const mlops_fbla_config *c, const mlops_fbla_shard *sh, const uint16_t *q, const mlops_fbla_cache *k,
                                           const float *row_mass_total, float *partial, void *scratch, size_t scratch_bytes,
                                           cudaStream_t stream) {
  constexpr const char *fn = "mlops_fbla_shard_partial";
  if (!row_mass_total || !partial || !on_boundary(row_mass_total, 16) || !on_boundary(partial, 16))
    return refuse(fn, "row_mass_total and partial have to be device pointers on 16-byte boundaries");
  fbla_k_decode a;
  mlops_fbla_status st = make_decode(fn, c, nullptr, q, k, nullptr, false, scratch, scratch_bytes, a);
  if (st == MLOPS_FBLA_OK) st = apply_shard(fn, sh, a);
  if (st != MLOPS_FBLA_OK) return st;
  a.phase = 2;
  a.row_r = const_cast<float *>(row_mass_total);
  a.out_partial = partial;
  return enqueue_decode(fn, a, stream);
}

size_t mlops_fbla_shard_mailbox_bytes(int world, int rows) {
  if (world <= 0 || world > MLOPS_FBLA_SHARD_MAX_RANKS || rows <= 0) return 0;
  return fbla_k_mailbox_of(world, rows).bytes;
}

static mlops_fbla_status make_link(const char *fn, const mlops_fbla_shard_link *link, int rows, fbla_k_link &L) {
  if (!link || !link->mailboxes || link->world <= 0 || link->world > MLOPS_FBLA_SHARD_MAX_RANKS || link->rank < 0 || link->rank >= link->world)
    return refuse(fn, "the link needs 1 <= world <= %d, 0 <= rank < world and the list of mailboxes", MLOPS_FBLA_SHARD_MAX_RANKS);
  L = fbla_k_link{};
  for (int p = 0; p < link->world; ++p) {
    if (!link->mailboxes[p] || !on_boundary(link->mailboxes[p], 256)) return refuse(fn, "mailbox %d is null or not on a 256-byte boundary", p);
    L.peer[p] = link->mailboxes[p];
  }
  L.rank = link->rank;
  L.world = link->world;
  L.rows = rows;
  L.spin_limit = link->wait_polls ? link->wait_polls : (1u << 22);
  return MLOPS_FBLA_OK;
}

mlops_fbla_status mlops_fbla_shard_step(const mlops_fbla_config *c, const mlops_fbla_shard *sh, const mlops_fbla_shard_link *link, const uint16_t *q,
                                        const mlops_fbla_cache *k, uint16_t *output, void *scratch, size_t scratch_bytes, cudaStream_t stream) {
  constexpr const char *fn = "mlops_fbla_shard_step";
  if (!output || !on_boundary(output, 16)) return refuse(fn, "output has to be a device pointer on a 16-byte boundary");
  if (!c) return refuse(fn, "a required pointer is null");
  fbla_k_link L;
  mlops_fbla_status st = make_link(fn, link, c->batch * c->q_heads, L);
  fbla_k_decode mass_pass, sum_pass;
  if (st == MLOPS_FBLA_OK) st = make_decode(fn, c, nullptr, q, k, nullptr, false, scratch, scratch_bytes, mass_pass);
  if (st == MLOPS_FBLA_OK) st = apply_shard(fn, sh, mass_pass);
  if (st != MLOPS_FBLA_OK) return st;
  const fbla_k_mailbox M = fbla_k_mailbox_of(L.world, L.rows);
  char *own = static_cast<char *>(L.peer[L.rank]);
  sum_pass = mass_pass;
  mass_pass.phase = 1;  // coarse pass; the rows' local masses
  mass_pass.row_r = reinterpret_cast<float *>(own + M.local_mass);
  mass_pass.status_cleared = 1;
  sum_pass.phase = 2;   // select with the common masses, refine, the shard's sums
  sum_pass.row_r = reinterpret_cast<float *>(own + M.total);
  sum_pass.out_partial = reinterpret_cast<float *>(own + M.local_part);
  sum_pass.status_cleared = 1;
  cudaError_t e = fbla_k_decode_launch(&mass_pass, stream);
  if (e == cudaSuccess) e = fbla_k_link_push_mass(&L, stream);
  if (e == cudaSuccess) e = fbla_k_link_gather_mass(&L, stream);
  if (e == cudaSuccess) e = fbla_k_decode_launch(&sum_pass, stream);
  if (e == cudaSuccess) e = fbla_k_link_push_partial(&L, stream);
  if (e == cudaSuccess) e = fbla_k_link_combine(&L, output, stream);
  return e == cudaSuccess ? accepted() : device_failure(fn, e);
}

int mlops_fbla_shard_link_status(const mlops_fbla_shard_link *link, int rows, cudaStream_t stream) {
  fbla_k_link L;
  if (make_link("mlops_fbla_shard_link_status", link, rows, L) != MLOPS_FBLA_OK) return -1;
  int word = 0;
  const char *own = static_cast<const char *>(L.peer[L.rank]);
  if (cudaMemcpyAsync(&word, own + fbla_k_mailbox_of(L.world, L.rows).status, sizeof word, cudaMemcpyDeviceToHost, stream) != cudaSuccess) return -1;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return -1;
  accepted();
  return word;
}

mlops_fbla_status mlops_fbla_shard_total_mass(int shards, int rows, const float *gathered, float *row_mass_total, cudaStream_t stream) {
  constexpr const char *fn = "mlops_fbla_shard_total_mass";
  if (shards <= 0 || rows <= 0 || !gathered || !row_mass_total) return refuse(fn, "needs shards > 0, rows > 0 and both device pointers");
  const cudaError_t e = fbla_k_total_mass_launch(gathered, row_mass_total, shards, rows, stream);
  return e == cudaSuccess ? accepted() : device_failure(fn, e);
}

mlops_fbla_status mlops_fbla_shard_combine(int rows, const float *partial_sum, uint16_t *output, cudaStream_t stream) {
  constexpr const char *fn = "mlops_fbla_shard_combine";
  if (rows <= 0 || !partial_sum || !output || !on_boundary(partial_sum, 16) || !on_boundary(output, 16))
    return refuse(fn, "needs rows > 0 and both device pointers on 16-byte boundaries");
  const cudaError_t e = fbla_k_combine_launch(partial_sum, output, rows, stream);
  return e == cudaSuccess ? accepted() : device_failure(fn, e);
}

// ---- work items (include/mlops_fbla_items.h; reference: attention/fbla/src/fbla_kernels.cuh:1446-1510 plan builders,
// attention/fbla/src/fbla.cu:587-810 access ranges) -------------------------------------------------------------------------
extern "C++" {
namespace {
// geometry slots of this library beyond the shared ones: 3 = item_off offset, 4 = status offset (decode scratch);
// 3 = the chunk's ceiling (prefill family)
template <class A> bool fill_pass(mlops_fbla_items &p, int kind, const fbla_k_pass &k, const char *args_type, const A &args) {
  static_assert(sizeof(A) <= MLOPS_FBLA_ITEM_ARGS_BYTES, "argument structure exceeds the blob");
  memset(&p, 0, sizeof p);
  p.kind = kind; p.items = k.gx * k.gy * k.gz; p.threads = k.threads; p.smem_bytes = k.smem_bytes; p.regs = k.regs; p.arch = 100;
  snprintf(p.entry, sizeof p.entry, "%s", k.entry);
  snprintf(p.args_type, sizeof p.args_type, "%s", args_type);
  p.args_bytes = (int)sizeof(A);
  memcpy(p.args.bytes, &args, sizeof(A));
  p.geom[MLOPS_FBLA_GEOM_GRID_X] = k.gx; p.geom[MLOPS_FBLA_GEOM_GRID_Y] = k.gy; p.geom[MLOPS_FBLA_GEOM_GRID_Z] = k.gz;
  return true;
}
void cache_geom(mlops_fbla_items &p, int hs, int gs, long long capacity, int cb, int fb) {
  p.geom[MLOPS_FBLA_GEOM_HEAD_STRIDE] = hs; p.geom[MLOPS_FBLA_GEOM_GROUP_STRIDE] = gs;
  p.geom[MLOPS_FBLA_GEOM_CAPACITY_GROUPS] = groups_of(capacity);
  p.geom[MLOPS_FBLA_GEOM_COARSE_BYTES] = 2 * cb * 256; p.geom[MLOPS_FBLA_GEOM_FINE_BYTES] = 2 * fb * 256;
}
int plan_fail(const cudaError_t e, const char *fn) {
  device_failure(fn, e);
  return -1;
}

struct Ranges {
  mlops_fbla_item_range *out;
  int max, n;
  void add(int arg, int write, long long offset, long long bytes, long long stride = 0, int rows = 1) {
    if (bytes <= 0 || rows <= 0) return;
    if (n < max) out[n] = mlops_fbla_item_range{arg, write, offset, bytes, rows > 1 ? stride : bytes, rows};
    ++n;
  }
};
// the units of KV head h (all groups the layout holds): records and metadata
void head_units(Ranges &r, const mlops_fbla_items &p, int h, int write, bool coarse, bool fine, bool meta) {
  const long long hs = p.geom[MLOPS_FBLA_GEOM_HEAD_STRIDE], gs = p.geom[MLOPS_FBLA_GEOM_GROUP_STRIDE], cg = p.geom[MLOPS_FBLA_GEOM_CAPACITY_GROUPS];
  const long long uc = kBlocksPerGroup * p.geom[MLOPS_FBLA_GEOM_COARSE_BYTES], uf = kBlocksPerGroup * p.geom[MLOPS_FBLA_GEOM_FINE_BYTES];
  if (coarse) r.add(MLOPS_FBLA_ARG_COARSE, write, h * hs * uc, uc, gs * uc, (int)cg);
  if (fine) r.add(MLOPS_FBLA_ARG_FINE, write, h * hs * uf, uf, gs * uf, (int)cg);
  if (meta) r.add(MLOPS_FBLA_ARG_META, write, h * hs * 1024, 1024, gs * 1024, (int)cg);
}
void head_windows(Ranges &r, int h, int write, bool sink, bool open) {
  const long long w = (long long)kGroup * kHeadDim * 2;
  if (sink) { r.add(MLOPS_FBLA_ARG_SINK_K, write, h * w, w); r.add(MLOPS_FBLA_ARG_SINK_V, write, h * w, w); }
  if (open) { r.add(MLOPS_FBLA_ARG_OPEN_K, write, h * w, w); r.add(MLOPS_FBLA_ARG_OPEN_V, write, h * w, w); }
}
}  // namespace
}  // extern "C++"

int mlops_fbla_decode_at_items(const mlops_fbla_config *c, const int *length, const uint16_t *q, const mlops_fbla_cache *k, uint16_t *out,
                               void *scratch, size_t scratch_bytes, int /*per_head: see mlops_fbla_decode_scratch_bytes_for*/, mlops_fbla_items *passes, int max) {
  constexpr const char *fn = "mlops_fbla_decode_at_items";
  if (!length) { refuse(fn, "the device length pointer is null"); return -1; }
  if (c && c->capacity <= 0) { refuse(fn, "a device-length decode is laid out by capacity, which has to be positive"); return -1; }
  fbla_k_decode a;
  if (make_decode(fn, c, length, q, k, out, true, scratch, scratch_bytes, a) != MLOPS_FBLA_OK) return -1;
  if (max == 0) { accepted(); return 4; }
  if (!passes || max < 4) { refuse(fn, "the plan has 4 passes: `max` is too small or `passes` is null"); return -1; }
  fbla_k_pass info[4];
  const cudaError_t e = fbla_k_decode_passes(&a, info);
  if (e != cudaSuccess) return plan_fail(e, fn);
  const int kinds[4] = {MLOPS_FBLA_ITEM_COARSE, MLOPS_FBLA_ITEM_SELECT, MLOPS_FBLA_ITEM_REFINE, MLOPS_FBLA_ITEM_MERGE};
  const char *base = static_cast<const char *>(scratch);
  for (int i = 0; i < 4; ++i) {
    mlops_fbla_items &p = passes[i];
    fill_pass(p, kinds[i], info[i], "fbla_k_decode", a);
    cache_geom(p, a.hs, a.gs, c->capacity, a.cb, a.fb);
    p.geom[MLOPS_FBLA_GEOM_LSE] = (const char *)a.lse - base; p.geom[MLOPS_FBLA_GEOM_PART] = (const char *)a.part - base;
    p.geom[MLOPS_FBLA_GEOM_DPART] = (const char *)a.dpart - base; p.geom[MLOPS_FBLA_GEOM_ROW_LSE] = (const char *)a.row_r - base;
    p.geom[MLOPS_FBLA_GEOM_ITEMS] = (const char *)a.items - base; p.geom[MLOPS_FBLA_GEOM_COUNTS] = (const char *)a.counts - base;
    p.geom[3] = (const char *)a.item_off - base; p.geom[4] = (const char *)a.status - base;
  }
  accepted();
  return 4;
}

static int prefill_items(const char *fn, const mlops_fbla_config *c, const int *length, const int *count, int max_count, const uint16_t *q,
                         const uint16_t *k, const uint16_t *v, const mlops_fbla_cache *cache, uint16_t *out, mlops_fbla_items *passes, int max) {
  fbla_k_prefill a;
  if (make_chunk_at(fn, c, length, count, max_count, q, k, v, cache, out, a) != MLOPS_FBLA_OK) return -1;
  fbla_k_prefill parts[2];
  int tc[2];
  const int np = q ? fbla_k_attend_plan(&a, parts, tc) : 0, n = 2 + np;  // close, the attention's one or two passes, finish
  if (max == 0) { accepted(); return n; }
  if (!passes || max < n) { refuse(fn, "the plan has %d passes: `max` is too small or `passes` is null", n); return -1; }
  fbla_k_pass info;
  int at = 0;
  cudaError_t e = fbla_k_close_pass(&a, max_count / kGroup + 1, &info);
  if (e != cudaSuccess) return plan_fail(e, fn);
  fill_pass(passes[at++], MLOPS_FBLA_ITEM_CLOSE, info, "fbla_k_prefill", a);
  if (q) {
    for (int i = 0; i < np; ++i) {
      e = tc[i] ? fbla_k_attend_tc_pass(&parts[i], &info) : fbla_k_attend_rows_pass(&parts[i], &info);
      if (e != cudaSuccess) return plan_fail(e, fn);
      fill_pass(passes[at++], tc[i] ? MLOPS_FBLA_ITEM_TC : MLOPS_FBLA_ITEM_STREAM, info, "fbla_k_prefill", parts[i]);
    }
  }
  e = fbla_k_finish_pass(&a, &info);
  if (e != cudaSuccess) return plan_fail(e, fn);
  fill_pass(passes[at++], MLOPS_FBLA_ITEM_FINISH, info, "fbla_k_prefill", a);
  for (int i = 0; i < at; ++i) { cache_geom(passes[i], a.hs, a.gs, c->capacity, a.cb, a.fb); passes[i].geom[3] = max_count; }
  accepted();
  return at;
}

int mlops_fbla_prefill_at_items(const mlops_fbla_config *c, const int *length, const int *count, int max_count, const uint16_t *q, const uint16_t *k,
                                const uint16_t *v, const mlops_fbla_cache *cache, uint16_t *out, mlops_fbla_items *passes, int max) {
  if (!count) { refuse("mlops_fbla_prefill_at_items", "a required pointer is null"); return -1; }
  return prefill_items("mlops_fbla_prefill_at_items", c, length, count, max_count, q, k, v, cache, out, passes, max);
}

int mlops_fbla_append_at_items(const mlops_fbla_config *c, const int *length, const uint16_t *k, const uint16_t *v, const mlops_fbla_cache *cache,
                               mlops_fbla_items *passes, int max) {
  return prefill_items("mlops_fbla_append_at_items", c, length, nullptr, 1, nullptr, k, v, cache, nullptr, passes, max);
}

int mlops_fbla_qkv_at_items(const mlops_fbla_config *c, const int *length, const mlops_fbla_token *t, const mlops_fbla_cache *cache,
                            mlops_fbla_items *passes, int max) {
  constexpr const char *fn = "mlops_fbla_qkv_at_items";
  fbla_k_prefill cl;
  fbla_k_token a;
  if (make_token_step(c, length, t, cache, cl, a) != MLOPS_FBLA_OK) return -1;
  if (max == 0) { accepted(); return 2; }
  if (!passes || max < 2) { refuse(fn, "the plan has 2 passes: `max` is too small or `passes` is null"); return -1; }
  fbla_k_pass info;
  cudaError_t e = fbla_k_close_pass(&cl, 1, &info);
  if (e != cudaSuccess) return plan_fail(e, fn);
  fill_pass(passes[0], MLOPS_FBLA_ITEM_CLOSE, info, "fbla_k_prefill", cl);
  e = fbla_k_qkv_token_pass(&a, &info);
  if (e != cudaSuccess) return plan_fail(e, fn);
  fill_pass(passes[1], MLOPS_FBLA_ITEM_QKV, info, "fbla_k_token", a);
  for (int i = 0; i < 2; ++i) { cache_geom(passes[i], cl.hs, cl.gs, c->capacity, cl.cb, cl.fb); passes[i].geom[3] = 1; }
  accepted();
  return 2;
}

int mlops_fbla_qkv_prefill_at_items(const mlops_fbla_config *c, const int *length, const int *count, int max_count, const mlops_fbla_token *t,
                                    uint16_t *q_out, uint16_t *k_out, uint16_t *v_out, mlops_fbla_items *passes, int max) {
  constexpr const char *fn = "mlops_fbla_qkv_prefill_at_items";
  fbla_k_token a;
  if (make_token_chunk(c, length, count, max_count, t, q_out, k_out, v_out, a) != MLOPS_FBLA_OK) return -1;
  if (max == 0) { accepted(); return 1; }
  if (!passes || max < 1) { refuse(fn, "the plan has 1 pass: `max` is too small or `passes` is null"); return -1; }
  fbla_k_pass info;
  const cudaError_t e = fbla_k_qkv_chunk_pass(&a, &info);
  if (e != cudaSuccess) return plan_fail(e, fn);
  fill_pass(passes[0], MLOPS_FBLA_ITEM_QKV_CHUNK, info, "fbla_k_token", a);
  passes[0].geom[3] = max_count;
  accepted();
  return 1;
}

int mlops_fbla_item_call(const mlops_fbla_items *p, char *out, size_t capacity) {
  if (!p || !out || p->kind < MLOPS_FBLA_ITEM_CLOSE || p->kind > MLOPS_FBLA_ITEM_QKV_CHUNK || !p->entry[0]) return -1;
  const int n = snprintf(out, capacity,
                         "mlops_fbla::position(item, %lld, %lld, %lld); __syncthreads(); "
                         "%s(*reinterpret_cast<const %s *>(args), reinterpret_cast<unsigned char *>(sm));",
                         p->geom[0], p->geom[1], p->geom[2], p->entry, p->args_type);
  return n < 0 || (size_t)n >= capacity ? -1 : n;
}

int mlops_fbla_item_access(const mlops_fbla_items *passes, int npasses, int pass, int item, mlops_fbla_item_range *ranges, int max) {
  if (!passes || pass < 0 || pass >= npasses || max < 0 || (max > 0 && !ranges)) return -1;
  const mlops_fbla_items &p = passes[pass];
  if (item < 0 || item >= p.items) return -1;
  Ranges r{ranges, max, 0};
  const int x = item % (int)p.geom[0], y = (item / (int)p.geom[0]) % (int)p.geom[1];
  const long long row = kHeadDim * 2;  // bytes of one head vector
  if (p.kind >= MLOPS_FBLA_ITEM_COARSE && p.kind <= MLOPS_FBLA_ITEM_MERGE) {
    fbla_k_decode a;
    memcpy(&a, p.args.bytes, sizeof a);
    const int heads = a.batch * a.kv_heads, hpr = a.kv_heads * a.vg, vheads = a.batch * hpr;
    const long long lse = p.geom[MLOPS_FBLA_GEOM_LSE], part = p.geom[MLOPS_FBLA_GEOM_PART], dpart = p.geom[MLOPS_FBLA_GEOM_DPART];
    const long long row_r = p.geom[MLOPS_FBLA_GEOM_ROW_LSE], items = p.geom[MLOPS_FBLA_GEOM_ITEMS], counts = p.geom[MLOPS_FBLA_GEOM_COUNTS];
    const long long item_off = p.geom[3], status = p.geom[4];
    r.add(MLOPS_FBLA_ARG_LENGTH, 0, 0, 4, 4, a.lstride ? a.batch : 1);
    if (p.kind == MLOPS_FBLA_ITEM_COARSE || p.kind == MLOPS_FBLA_ITEM_REFINE) {
      // a persistent CTA's unit range depends on the device length: every head's units are the envelope
      r.add(MLOPS_FBLA_ARG_Q, 0, 0, (long long)a.batch * a.q_heads * row);
      for (int h = 0; h < heads; ++h) head_units(r, p, h, 0, true, p.kind == MLOPS_FBLA_ITEM_REFINE, true);
    }
    if (p.kind == MLOPS_FBLA_ITEM_COARSE) {
      for (int h = 0; h < heads; ++h) head_windows(r, h, 0, true, true);
      r.add(MLOPS_FBLA_ARG_SCRATCH, 1, lse, part - lse);
      r.add(MLOPS_FBLA_ARG_SCRATCH, 1, part, dpart - part);
      r.add(MLOPS_FBLA_ARG_SCRATCH, 1, status, 16);
    } else if (p.kind == MLOPS_FBLA_ITEM_SELECT) {
      const long long per = (long long)a.nblocks * a.qg * 4;
      r.add(MLOPS_FBLA_ARG_SCRATCH, 0, lse + y * per, per);
      r.add(MLOPS_FBLA_ARG_SCRATCH, 0, part, dpart - part);
      r.add(MLOPS_FBLA_ARG_SCRATCH, 1, row_r + (long long)y * a.qg * 4, a.qg * 4);
      r.add(MLOPS_FBLA_ARG_SCRATCH, 1, counts + ((long long)y * a.nslices + x) * 4, 4);
      r.add(MLOPS_FBLA_ARG_SCRATCH, 1, items + ((long long)y * a.nslices + x) * FBLA_K_SLICE * 4, FBLA_K_SLICE * 4);
    } else if (p.kind == MLOPS_FBLA_ITEM_REFINE) {
      r.add(MLOPS_FBLA_ARG_SCRATCH, 0, row_r, (long long)vheads * a.qg * 4);
      r.add(MLOPS_FBLA_ARG_SCRATCH, 0, counts, (long long)vheads * a.nslices * 4);
      r.add(MLOPS_FBLA_ARG_SCRATCH, 0, items, (long long)vheads * a.nslices * FBLA_K_SLICE * 4);
      r.add(MLOPS_FBLA_ARG_SCRATCH, 1, dpart, row_r - dpart);
      if (x == 0) r.add(MLOPS_FBLA_ARG_SCRATCH, 1, item_off, (long long)(vheads + 1) * 4);
      r.add(MLOPS_FBLA_ARG_SCRATCH, 1, status, 16);
    } else {
      const int vh = item / a.qg, qi = item % a.qg, b = vh / hpr, hir = vh % hpr;
      const long long qrow = (long long)b * a.q_heads + (hir / a.vg) * (a.qg * a.vg) + (hir % a.vg) * a.qg + qi;
      r.add(MLOPS_FBLA_ARG_SCRATCH, 0, part, dpart - part);
      r.add(MLOPS_FBLA_ARG_SCRATCH, 0, dpart, row_r - dpart);
      r.add(MLOPS_FBLA_ARG_SCRATCH, 0, row_r + (long long)vh * a.qg * 4, a.qg * 4);
      r.add(MLOPS_FBLA_ARG_SCRATCH, 0, item_off, (long long)(vheads + 1) * 4);
      r.add(MLOPS_FBLA_ARG_OUT, 1, qrow * row, row);
    }
  } else if (p.kind == MLOPS_FBLA_ITEM_QKV || p.kind == MLOPS_FBLA_ITEM_QKV_CHUNK) {
    fbla_k_token a;
    memcpy(&a, p.args.bytes, sizeof a);
    const int qg = a.q_heads / a.kv_heads;
    r.add(MLOPS_FBLA_ARG_TFREQ, 0, 0, 64 * 16);
    if (a.q_norm) { r.add(MLOPS_FBLA_ARG_TQN, 0, 0, row); r.add(MLOPS_FBLA_ARG_TKN, 0, 0, row); }
    if (p.kind == MLOPS_FBLA_ITEM_QKV) {
      const int b = x / a.kv_heads, kh = x % a.kv_heads;
      r.add(MLOPS_FBLA_ARG_LENGTH, 0, 0, 4, 4, a.lstride ? a.batch : 1);
      r.add(MLOPS_FBLA_ARG_TQ, 0, (b * a.batch_stride + kh * a.q_group_stride) * 2, qg * row);
      r.add(MLOPS_FBLA_ARG_TK, 0, (b * a.batch_stride + kh * a.kv_group_stride) * 2, row);
      r.add(MLOPS_FBLA_ARG_TV, 0, (b * a.batch_stride + kh * a.kv_group_stride) * 2, row);
      r.add(MLOPS_FBLA_ARG_TQ_OUT, 1, ((long long)b * a.q_heads + kh * qg) * row, qg * row);
      head_windows(r, x, 1, true, true);
    } else {
      const long long i0 = 8LL * x, rows = a.max_count - i0 < 8 ? a.max_count - i0 : 8;
      r.add(MLOPS_FBLA_ARG_LENGTH, 0, 0, 4);
      r.add(MLOPS_FBLA_ARG_COUNT, 0, 0, 4);
      r.add(MLOPS_FBLA_ARG_TQ, 0, (i0 * a.batch_stride + y * a.q_group_stride) * 2, qg * row, a.batch_stride * 2, (int)rows);
      r.add(MLOPS_FBLA_ARG_TK, 0, (i0 * a.batch_stride + y * a.kv_group_stride) * 2, row, a.batch_stride * 2, (int)rows);
      r.add(MLOPS_FBLA_ARG_TV, 0, (i0 * a.batch_stride + y * a.kv_group_stride) * 2, row, a.batch_stride * 2, (int)rows);
      r.add(MLOPS_FBLA_ARG_Q, 1, (((long long)y * qg) * a.max_count + i0) * row, rows * row, a.max_count * row, qg);
      r.add(MLOPS_FBLA_ARG_K, 1, ((long long)y * a.max_count + i0) * row, rows * row);
      r.add(MLOPS_FBLA_ARG_V, 1, ((long long)y * a.max_count + i0) * row, rows * row);
    }
  } else {
    fbla_k_prefill a;
    memcpy(&a, p.args.bytes, sizeof a);
    const int qg = a.q_heads / a.kv_heads;
    const int h = p.kind == MLOPS_FBLA_ITEM_FINISH ? x : y, b = h / a.kv_heads, kh = h % a.kv_heads;  // the KV head of the item
    const long long chunk = (long long)a.count * row;
    if (a.length) r.add(MLOPS_FBLA_ARG_LENGTH, 0, 0, 4, 4, a.lstride ? a.batch : 1);
    if (a.dcount) r.add(MLOPS_FBLA_ARG_COUNT, 0, 0, 4);
    if (a.k) { r.add(MLOPS_FBLA_ARG_K, 0, h * chunk, chunk); r.add(MLOPS_FBLA_ARG_V, 0, h * chunk, chunk); }
    if (p.kind == MLOPS_FBLA_ITEM_CLOSE) {  // which group closes depends on the device length: the head's units are the envelope
      head_windows(r, h, 0, true, true);
      head_units(r, p, h, 1, true, true, true);
    } else if (p.kind == MLOPS_FBLA_ITEM_FINISH) {
      head_windows(r, h, 1, true, true);
    } else {
      head_units(r, p, h, 0, true, true, true);
      head_windows(r, h, 0, true, true);
      for (int t = 0; t < qg; ++t) {
        const long long hq = (long long)b * a.q_heads + kh * qg + t;
        r.add(MLOPS_FBLA_ARG_Q, 0, hq * chunk, chunk);
        r.add(MLOPS_FBLA_ARG_OUT, 1, hq * a.out_hs * 2, row, (long long)a.out_ts * 2, a.count);
      }
    }
  }
  return r.n;
}

const char *mlops_fbla_status_string(mlops_fbla_status status) {
  switch (status) {
    case MLOPS_FBLA_OK: return "ok";
    case MLOPS_FBLA_INVALID_VALUE: return "invalid value";
    case MLOPS_FBLA_CUDA_ERROR: return "CUDA error";
  }
  return "unknown status";
}

const char *mlops_fbla_last_error(void) { return g_message; }

}  // extern "C"
