// Host layer of the FBLA library: argument validation, cache / scratch geometry and dispatch to the CUDA passes.
// It mirrors the accept / reject behaviour and the status codes of the reference's host code
// (attention/fbla/src/fbla.cu:16-20 error text, :62-80 shape rules, :90-138 decode preparation, :193-268 prefill
// rules, :408-430 size queries) behind the same C interface (include/mlops_fbla.h). It allocates nothing, never
// synchronises, and keeps only per-thread state (last error, device attribute cache), so calls may come from many
// host threads at once.
#include "../../../include/mlops_fbla.h"
#include "../../../include/mlops_fbla_shard.h"
#include "../../../include/mlops_fbla_items.h"
#include "../kernels/fbla_kernels.h"

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>

namespace {

constexpr int G = MLOPS_FBLA_GROUP, SBG = MLOPS_FBLA_GROUP / MLOPS_FBLA_SUBBLOCK, D = MLOPS_FBLA_HEAD_DIM;
constexpr long long MAX_TOKENS = 1ll << 26;

thread_local char error_buf[256] = {0};
mlops_fbla_status fail(mlops_fbla_status st, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buf, sizeof(error_buf) - 1, fmt, ap);
  va_end(ap);
  return st;
}
mlops_fbla_status ok() { error_buf[0] = 0; return MLOPS_FBLA_OK; }
bool aligned(const void *p, size_t n) { return (reinterpret_cast<uintptr_t>(p) & (n - 1)) == 0; }
size_t up256(size_t n) { return (n + 255) & ~(size_t)255; }
bool valid_format(const mlops_fbla_config *c) { return c->format == MLOPS_FBLA_3P3 || c->format == MLOPS_FBLA_4P2; }
bool valid_strides(const mlops_fbla_config *c) {
  return (c->head_stride == 0 && c->group_stride == 0) || (c->head_stride > 0 && c->group_stride > 0);
}
bool valid_out_layout(const mlops_fbla_config *c) {
  if (c->out_head_stride == 0 && c->out_token_stride == 0) return true;
  return c->out_head_stride > 0 && c->out_token_stride > 0 && c->out_token_stride < (1ll << 30) && c->out_head_stride % 8 == 0 &&
         c->out_token_stride % 8 == 0 && c->batch == 1;
}
// queries served together per virtual KV head for r queries per KV head: r for 1, 2, 4, else the largest of 4, 2, 1 dividing r
int decode_group(int r) { return r == 1 || r == 2 || r == 4 ? r : r % 4 == 0 ? 4 : r % 2 == 0 ? 2 : 1; }
float scale_log2(const mlops_fbla_config *c) {
  const float scale = c->scale == 0.f ? 1.f / sqrtf((float)D) : c->scale;
  return scale * 1.4426950408889634f;
}
bool cache_complete(const mlops_fbla_cache *k) {
  return k->coarse && k->fine && k->meta && k->exact_sink_k && k->exact_sink_v && k->exact_open_k && k->exact_open_v;
}
fbla_k_cache kcache(const mlops_fbla_cache *k) {
  return fbla_k_cache{k->coarse, k->fine, k->meta, k->exact_sink_k, k->exact_sink_v, k->exact_open_k, k->exact_open_v};
}

// ---- decode scratch ------------------------------------------------------------------------------------------------
struct Layout {
  size_t lse, part, dpart, row_r, counts, items, item_off, status, bytes;
  int nblocks, nslices;
};
// shape: the launch shape of the current device (fbla_k_decode_shape); tokens: the layout's token count
bool decode_layout(const mlops_fbla_config *c, long long tokens, const fbla_k_decode &shape, Layout &L) {
  const int r = c->q_heads / c->kv_heads, qg = decode_group(r), vg = r / qg;
  const size_t vheads = (size_t)c->batch * c->kv_heads * vg;
  const long long groups = (tokens + G - 1) / G;
  L.nblocks = (int)(groups * SBG);
  L.nslices = (int)((L.nblocks + FBLA_K_SLICE - 1) / FBLA_K_SLICE);
  if (L.nslices < 1) L.nslices = 1;
  // (shape.coarse_warps: the streaming warps of the fixed 7 + 1 split; a CTA has one warp more, and the split by the
  // lengths can put all but one of them on either kind of work)
  const size_t tw = (size_t)shape.coarse_ctas * (shape.coarse_warps + 1), xw = tw;
  const size_t rw = (size_t)shape.refine_ctas * shape.refine_warps;
  const size_t row = (size_t)qg * FBLA_K_PSTRIDE * sizeof(float);
  L.lse = 0;
  L.part = L.lse + up256(vheads * L.nblocks * qg * sizeof(float));
  L.dpart = L.part + up256((tw + xw + 2 * vheads) * row);
  L.row_r = L.dpart + up256((rw + vheads) * row);
  L.counts = L.row_r + up256(vheads * qg * sizeof(float));
  L.items = L.counts + up256(vheads * L.nslices * sizeof(int));
  L.item_off = L.items + up256(vheads * L.nslices * FBLA_K_SLICE * sizeof(int));
  L.status = L.item_off + up256((vheads + 1) * sizeof(int));
  L.bytes = L.status + 256;
  return true;
}
bool valid_decode_shape(const mlops_fbla_config *c) {  // c->tokens: the layout's
  if (!c || c->batch <= 0 || c->q_heads <= 0 || c->kv_heads <= 0 || c->tokens <= 0 || !valid_strides(c)) return false;
  if (c->q_heads % c->kv_heads) return false;
  if (c->capacity != 0 && c->capacity < c->tokens) return false;
  return c->tokens <= MAX_TOKENS;
}
size_t scratch_bytes_of(const mlops_fbla_config *lc) {
  fbla_k_decode shape{};
  shape.cb = lc->format == MLOPS_FBLA_3P3 ? 3 : 4;
  if (fbla_k_decode_shape(&shape) != cudaSuccess) return 0;
  Layout L;
  decode_layout(lc, lc->tokens, shape, L);
  return L.bytes;
}

// validates a decode and fills the kernels' arguments (out may be null when need_out is false: the shard passes)
mlops_fbla_status prepare_decode(const char *fn, const mlops_fbla_config *c, const int *length, const uint16_t *q, const mlops_fbla_cache *k,
                                 uint16_t *out, bool need_out, void *scratch, size_t scratch_bytes, fbla_k_decode &a) {
  const bool by_capacity = length != nullptr;
  if (!c || !k || !q || (need_out && !out) || !scratch) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: null argument", fn);
  mlops_fbla_config lc = *c;
  if (by_capacity) lc.tokens = c->capacity;
  if (!valid_decode_shape(&lc) || (by_capacity && c->tokens < 0))
    return fail(MLOPS_FBLA_INVALID_VALUE, "%s: batch, heads and tokens must be positive (device length: capacity positive, tokens >= 0), "
                "q_heads a multiple of kv_heads, tokens <= 2^26, capacity 0 or >= tokens, strides both 0 or both positive", fn);
  if (!valid_format(c)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: invalid format", fn);
  if (!(c->scale >= 0.f) || !(c->tau >= 0.f)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: scale and tau must be nonnegative", fn);
  if (!cache_complete(k)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: every cache pointer is required", fn);
  const void *ptrs[] = {q, out, scratch, k->coarse, k->fine, k->meta, k->exact_sink_k, k->exact_sink_v, k->exact_open_k, k->exact_open_v};
  for (const void *p : ptrs)
    if (!aligned(p, 16)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: pointers must be 16-byte aligned", fn);
  if (!aligned(length, 4)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: length must be 4-byte aligned", fn);
  if ((c->length_stride != 0 && c->length_stride != 1) || (c->length_stride && !length))
    return fail(MLOPS_FBLA_INVALID_VALUE, "%s: length_stride is 0, or 1 with a device length", fn);

  a = fbla_k_decode{};
  a.cb = c->format == MLOPS_FBLA_3P3 ? 3 : 4;
  a.fb = c->format == MLOPS_FBLA_3P3 ? 3 : 2;
  cudaError_t e = fbla_k_decode_shape(&a);
  if (e != cudaSuccess) return fail(MLOPS_FBLA_CUDA_ERROR, "%s: %s", fn, cudaGetErrorString(e));
  Layout L;
  decode_layout(&lc, lc.tokens, a, L);
  if (scratch_bytes < L.bytes) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: scratch has %zu bytes, need %zu", fn, scratch_bytes, L.bytes);
  const int r = c->q_heads / c->kv_heads;
  a.qg = decode_group(r);
  a.vg = r / a.qg;
  if ((long long)c->batch * c->kv_heads * a.vg * L.nslices > 36000)
    return fail(MLOPS_FBLA_INVALID_VALUE, "%s: batch * kv_heads * virtual heads * slices of 16384 tokens exceeds 36000 (split the batch)", fn);
  a.c = kcache(k);
  a.q = q; a.out = out;
  char *base = static_cast<char *>(scratch);
  a.lse = reinterpret_cast<float *>(base + L.lse);
  a.part = reinterpret_cast<float *>(base + L.part);
  a.dpart = reinterpret_cast<float *>(base + L.dpart);
  a.row_r = reinterpret_cast<float *>(base + L.row_r);
  a.counts = reinterpret_cast<int *>(base + L.counts);
  a.items = reinterpret_cast<int *>(base + L.items);
  a.item_off = reinterpret_cast<int *>(base + L.item_off);
  a.status = reinterpret_cast<int *>(base + L.status);
  a.length = length;
  a.lstride = c->length_stride;
  a.batch = c->batch; a.q_heads = c->q_heads; a.kv_heads = c->kv_heads; a.tokens = c->tokens;
  a.nblocks = L.nblocks; a.nslices = L.nslices;
  const long long cap = c->capacity ? c->capacity : c->tokens;
  a.hs = c->head_stride ? c->head_stride : (int)((cap + G - 1) / G);
  a.gs = c->group_stride ? c->group_stride : 1;
  a.sl = scale_log2(c);
  // (by the cache's capacity where it has one, for host and device lengths alike: the two calls then run the same
  // kernels on the same cache and give bit-identical outputs)
  fbla_k_decode_split(&a, c->capacity ? c->capacity : c->tokens);
  const float tau = c->tau != 0.f ? c->tau : c->format == MLOPS_FBLA_3P3 ? 3e-4f : 1e-3f;
  a.log2_tau = log2f(tau);
  return MLOPS_FBLA_OK;
}
mlops_fbla_status launch_decode(const char *fn, const fbla_k_decode &a, cudaStream_t stream) {
  const cudaError_t e = fbla_k_decode_launch(&a, stream);
  if (e != cudaSuccess) return fail(MLOPS_FBLA_CUDA_ERROR, "%s: %s", fn, cudaGetErrorString(e));
  return ok();
}
mlops_fbla_status decode(const char *fn, const mlops_fbla_config *c, const int *length, const uint16_t *q, const mlops_fbla_cache *k,
                         uint16_t *out, void *scratch, size_t scratch_bytes, cudaStream_t stream) {
  fbla_k_decode a;
  const mlops_fbla_status st = prepare_decode(fn, c, length, q, k, out, true, scratch, scratch_bytes, a);
  return st != MLOPS_FBLA_OK ? st : launch_decode(fn, a, stream);
}

// ---- prefill ------------------------------------------------------------------------------------------------------------
mlops_fbla_status prefill_common(const char *fn, const mlops_fbla_config *c, const uint16_t *q, const uint16_t *k, const uint16_t *v,
                                 const mlops_fbla_cache *x, uint16_t *out) {
  if (!valid_out_layout(c))
    return fail(MLOPS_FBLA_INVALID_VALUE, "%s: out_head_stride and out_token_stride both positive multiples of 8 (batch 1) or both 0", fn);
  if (!valid_format(c)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: invalid format", fn);
  if (!(c->scale >= 0.f)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: scale must be nonnegative", fn);
  if (!cache_complete(x)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: every cache pointer is required", fn);
  const void *ptrs[] = {k, v, q, out, x->coarse, x->fine, x->meta, x->exact_sink_k, x->exact_sink_v, x->exact_open_k, x->exact_open_v};
  for (const void *p : ptrs)
    if (!aligned(p, 16)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: pointers must be 16-byte aligned", fn);
  if (!aligned(x->tc_images, 128)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: tc_images must be 128-byte aligned", fn);
  return MLOPS_FBLA_OK;
}
void fill_prefill(const mlops_fbla_config *c, int count, long long capacity, const uint16_t *q, const uint16_t *k, const uint16_t *v,
                  const mlops_fbla_cache *x, uint16_t *out, fbla_k_prefill &a) {
  a.c = kcache(x);
  a.q = q; a.k = k; a.v = v; a.out = out;
  a.out_hs = c->out_head_stride ? c->out_head_stride : (int64_t)count * D;
  a.out_ts = c->out_token_stride ? (int)c->out_token_stride : D;
  a.batch = c->batch; a.q_heads = c->q_heads; a.kv_heads = c->kv_heads;
  a.n0 = c->tokens; a.count = count;
  a.hs = c->head_stride ? c->head_stride : (int)((capacity + G - 1) / G);
  a.gs = c->group_stride ? c->group_stride : 1;
  a.cb = c->format == MLOPS_FBLA_3P3 ? 3 : 4;
  a.fb = c->format == MLOPS_FBLA_3P3 ? 3 : 2;
  a.sl = scale_log2(c);
}
mlops_fbla_status run_prefill(const char *fn, const fbla_k_prefill &a, int close_blocks, cudaStream_t stream) {
  // order: close reads the old windows, the attention reads them too, finish overwrites them last
  cudaError_t e = fbla_k_close_launch(&a, close_blocks, stream);
  if (e == cudaSuccess && a.q) e = fbla_k_attend_launch(&a, stream);
  if (e == cudaSuccess) e = fbla_k_finish_launch(&a, stream);
  if (e != cudaSuccess) return fail(MLOPS_FBLA_CUDA_ERROR, "%s: %s", fn, cudaGetErrorString(e));
  return ok();
}
mlops_fbla_status prefill_at_prepare(const char *fn, const mlops_fbla_config *c, const int *length, const int *dcount, int max_count,
                             const uint16_t *q, const uint16_t *k, const uint16_t *v, const mlops_fbla_cache *cache, uint16_t *out,
                             fbla_k_prefill &a) {
  if (!c || !length || !cache || !k || !v) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: null argument", fn);
  if (q && !out) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: q needs output", fn);
  if (c->batch <= 0 || c->kv_heads <= 0 || c->q_heads <= 0 || c->q_heads % c->kv_heads || c->tokens < 0 || c->capacity <= 0 ||
      (long long)c->tokens + max_count > c->capacity || max_count <= 0 || c->capacity > MAX_TOKENS || !valid_strides(c))
    return fail(MLOPS_FBLA_INVALID_VALUE, "%s: batch, heads, max_count and capacity must be positive, tokens >= 0, tokens + max_count <= "
                "capacity <= 2^26, q_heads a multiple of kv_heads, strides both 0 or both positive", fn);
  if ((c->length_stride != 0 && c->length_stride != 1) || (c->length_stride && (q || dcount)))
    return fail(MLOPS_FBLA_INVALID_VALUE, "%s: length_stride is 0 (1 only for the one-token append)", fn);
  const mlops_fbla_status st = prefill_common(fn, c, q, k, v, cache, out);
  if (st != MLOPS_FBLA_OK) return st;
  if (!aligned(length, 4) || !aligned(dcount, 4)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: length and count must be 4-byte aligned", fn);
  a = fbla_k_prefill{};
  fill_prefill(c, max_count, c->capacity, q, k, v, cache, out, a);
  a.length = length; a.dcount = dcount; a.lstride = c->length_stride;
  return MLOPS_FBLA_OK;
}
mlops_fbla_status prefill_at(const char *fn, const mlops_fbla_config *c, const int *length, const int *dcount, int max_count,
                             const uint16_t *q, const uint16_t *k, const uint16_t *v, const mlops_fbla_cache *cache, uint16_t *out,
                             cudaStream_t stream) {
  fbla_k_prefill a;
  const mlops_fbla_status st = prefill_at_prepare(fn, c, length, dcount, max_count, q, k, v, cache, out, a);
  // a chunk of at most max_count tokens starting anywhere closes at most max_count / 128 + 1 groups
  return st != MLOPS_FBLA_OK ? st : run_prefill(fn, a, max_count / G + 1, stream);
}

}  // namespace

extern "C" {

size_t mlops_fbla_decode_scratch_bytes(const mlops_fbla_config *c) {
  if (!valid_decode_shape(c) || !valid_format(c)) return 0;
  return scratch_bytes_of(c);
}

size_t mlops_fbla_decode_scratch_bytes_for(const mlops_fbla_config *c, int per_head) {
  if (!c || c->capacity <= 0 || per_head < 0) return 0;
  mlops_fbla_config lc = *c;
  lc.tokens = c->capacity;
  if (!valid_decode_shape(&lc) || !valid_format(c)) return 0;
  return scratch_bytes_of(&lc);
}

mlops_fbla_status mlops_fbla_decode(const mlops_fbla_config *c, const uint16_t *q, const mlops_fbla_cache *k, uint16_t *out,
                                    void *scratch, size_t scratch_bytes, cudaStream_t stream) {
  return decode("mlops_fbla_decode", c, nullptr, q, k, out, scratch, scratch_bytes, stream);
}

mlops_fbla_status mlops_fbla_decode_at(const mlops_fbla_config *c, const int *length, const uint16_t *q, const mlops_fbla_cache *k,
                                       uint16_t *out, void *scratch, size_t scratch_bytes, cudaStream_t stream) {
  if (!length) return fail(MLOPS_FBLA_INVALID_VALUE, "mlops_fbla_decode_at: null length");
  if (c && c->capacity <= 0) return fail(MLOPS_FBLA_INVALID_VALUE, "mlops_fbla_decode_at: capacity must be positive");
  return decode("mlops_fbla_decode_at", c, length, q, k, out, scratch, scratch_bytes, stream);
}

size_t mlops_fbla_images_bytes(const mlops_fbla_config *) { return 0; }

int mlops_fbla_cache_sizes(const mlops_fbla_config *c, mlops_fbla_sizes *out) {
  if (!c || !out || c->batch <= 0 || c->q_heads <= 0 || c->kv_heads <= 0 || c->q_heads % c->kv_heads || !valid_strides(c)) return 0;
  if (!valid_format(c)) return 0;
  const long long tokens = c->capacity ? c->capacity : c->tokens;
  if (tokens <= 0 || (c->capacity && c->capacity < c->tokens)) return 0;
  const size_t heads = (size_t)c->batch * c->kv_heads, groups = (size_t)((tokens + G - 1) / G);
  const size_t hs = c->head_stride ? (size_t)c->head_stride : groups, gs = c->group_stride ? (size_t)c->group_stride : 1;
  const size_t units = (heads - 1) * hs + (groups - 1) * gs + 1;
  const bool three = c->format == MLOPS_FBLA_3P3;
  out->coarse = units * SBG * (three ? 1536 : 2048);
  out->fine = units * SBG * (three ? 1536 : 1024);
  out->meta = units * 1024;
  out->exact = heads * G * D * sizeof(uint16_t);
  out->images = 0;
  return 1;
}

mlops_fbla_status mlops_fbla_prefill(const mlops_fbla_config *c, int count, const uint16_t *q, const uint16_t *k, const uint16_t *v,
                                     const mlops_fbla_cache *cache, uint16_t *out, cudaStream_t stream) {
  constexpr const char *fn = "mlops_fbla_prefill";
  if (!c || !cache || !k || !v) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: null argument", fn);
  if (q && !out) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: q needs output", fn);
  const long long n1 = (long long)c->tokens + count;
  if (c->batch <= 0 || c->q_heads <= 0 || c->kv_heads <= 0 || c->tokens < 0 || count <= 0 || !valid_strides(c) || c->q_heads % c->kv_heads ||
      !(c->capacity == 0 || c->capacity >= n1) || n1 > MAX_TOKENS)
    return fail(MLOPS_FBLA_INVALID_VALUE, "%s: batch, heads and count must be positive, tokens >= 0, q_heads a multiple of kv_heads, "
                "tokens + count <= capacity (0: tokens + count) and <= 2^26, strides both 0 or both positive", fn);
  const mlops_fbla_status st = prefill_common(fn, c, q, k, v, cache, out);
  if (st != MLOPS_FBLA_OK) return st;
  fbla_k_prefill a{};
  fill_prefill(c, count, c->capacity ? c->capacity : n1, q, k, v, cache, out, a);
  const int g_first = c->tokens == 0 ? 0 : (c->tokens - 1) / G, g_end = (int)((n1 - 1) / G);
  return run_prefill(fn, a, g_end - g_first, stream);
}

mlops_fbla_status mlops_fbla_prefill_at(const mlops_fbla_config *c, const int *length, const int *count, int max_count, const uint16_t *q,
                                        const uint16_t *k, const uint16_t *v, const mlops_fbla_cache *cache, uint16_t *out,
                                        cudaStream_t stream) {
  if (!count) return fail(MLOPS_FBLA_INVALID_VALUE, "mlops_fbla_prefill_at: null argument");
  return prefill_at("mlops_fbla_prefill_at", c, length, count, max_count, q, k, v, cache, out, stream);
}

mlops_fbla_status mlops_fbla_append_at(const mlops_fbla_config *c, const int *length, const uint16_t *k, const uint16_t *v,
                                       const mlops_fbla_cache *cache, cudaStream_t stream) {
  return prefill_at("mlops_fbla_append_at", c, length, nullptr, 1, nullptr, k, v, cache, nullptr, stream);
}

// ---- fused QKV step (reference: attention/fbla/src/fbla.cu:307-400) ---------------------------------------------------------
static mlops_fbla_status token_common(const char *fn, const mlops_fbla_token *t, fbla_k_token &a) {
  if (!t->q_norm != !t->k_norm) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: q_norm and k_norm both or neither", fn);
  if (!(t->eps >= 0.f) || !(t->attention_factor >= 0.f)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: eps and attention_factor nonnegative", fn);
  a.q = t->q; a.k = t->k; a.v = t->v;
  a.batch_stride = t->batch_stride; a.q_group_stride = t->q_group_stride; a.kv_group_stride = t->kv_group_stride;
  a.q_norm = t->q_norm; a.k_norm = t->k_norm; a.freq = t->freq; a.eps = t->eps;
  a.att = t->attention_factor == 0.f ? 1.f : t->attention_factor;
  return MLOPS_FBLA_OK;
}

static mlops_fbla_status qkv_at_prepare(const mlops_fbla_config *c, const int *length, const mlops_fbla_token *t, const mlops_fbla_cache *cache,
                                        fbla_k_prefill &cl, fbla_k_token &a) {
  constexpr const char *fn = "mlops_fbla_qkv_at";
  if (!c || !length || !t || !cache || !t->q || !t->k || !t->v || !t->freq || !t->q_out) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: null argument", fn);
  if (c->batch <= 0 || c->kv_heads <= 0 || c->q_heads <= 0 || c->q_heads % c->kv_heads || c->tokens < 0 || c->capacity <= 0 || !valid_strides(c))
    return fail(MLOPS_FBLA_INVALID_VALUE, "%s: batch and heads must be positive, q_heads a multiple of kv_heads, tokens >= 0, capacity positive, "
                "strides both 0 or both positive", fn);
  if (!valid_format(c)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: invalid format", fn);
  a = fbla_k_token{};
  mlops_fbla_status st = token_common(fn, t, a);
  if (st != MLOPS_FBLA_OK) return st;
  if (!cache_complete(cache)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: every cache pointer is required", fn);
  const void *p16[] = {cache->coarse, cache->fine, cache->meta, cache->exact_sink_k, cache->exact_sink_v, cache->exact_open_k, cache->exact_open_v, t->freq};
  for (const void *p : p16)
    if (!aligned(p, 16)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: cache pointers and freq must be 16-byte aligned", fn);
  const void *p4[] = {length, t->q, t->k, t->v, t->q_norm, t->k_norm, t->q_out};
  for (const void *p : p4)
    if (!aligned(p, 4)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: length and the token's pointers must be 4-byte aligned", fn);
  if (t->batch_stride % 2 || t->q_group_stride % 2 || t->kv_group_stride % 2)
    return fail(MLOPS_FBLA_INVALID_VALUE, "%s: strides must be even (4-byte rows)", fn);
  if (t->batch_stride < 0 || t->q_group_stride < 0 || t->kv_group_stride < 0 || t->batch_stride > INT32_MAX || t->q_group_stride > INT32_MAX ||
      t->kv_group_stride > INT32_MAX)
    return fail(MLOPS_FBLA_INVALID_VALUE, "%s: strides are nonnegative and below 2^31", fn);
  if (!aligned(cache->tc_images, 128)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: tc_images must be 128-byte aligned", fn);
  if (c->length_stride != 0 && c->length_stride != 1) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: length_stride is 0 or 1", fn);
  // the group that the position closes (when it is a multiple of 128) is quantized from the open window first
  cl = fbla_k_prefill{};
  fill_prefill(c, 1, c->capacity, nullptr, nullptr, nullptr, cache, nullptr, cl);
  cl.length = length; cl.lstride = c->length_stride;
  a.c = cl.c; a.length = length; a.lstride = c->length_stride; a.n0 = c->tokens; a.max_count = 1;
  a.batch = c->batch; a.q_heads = c->q_heads; a.kv_heads = c->kv_heads; a.q_out = t->q_out;
  return MLOPS_FBLA_OK;
}
mlops_fbla_status mlops_fbla_qkv_at(const mlops_fbla_config *c, const int *length, const mlops_fbla_token *t, const mlops_fbla_cache *cache,
                                    cudaStream_t stream) {
  fbla_k_prefill cl;
  fbla_k_token a;
  const mlops_fbla_status st = qkv_at_prepare(c, length, t, cache, cl, a);
  if (st != MLOPS_FBLA_OK) return st;
  cudaError_t e = fbla_k_close_launch(&cl, 1, stream);
  if (e == cudaSuccess) e = fbla_k_qkv_token_launch(&a, stream);
  if (e != cudaSuccess) return fail(MLOPS_FBLA_CUDA_ERROR, "mlops_fbla_qkv_at: %s", cudaGetErrorString(e));
  return ok();
}

static mlops_fbla_status qkv_chunk_prepare(const mlops_fbla_config *c, const int *length, const int *count, int max_count, const mlops_fbla_token *t,
                                           uint16_t *q_out, uint16_t *k_out, uint16_t *v_out, fbla_k_token &a) {
  constexpr const char *fn = "mlops_fbla_qkv_prefill_at";
  if (!c || !length || !count || !t || !t->q || !t->k || !t->v || !t->freq || !q_out || !k_out || !v_out)
    return fail(MLOPS_FBLA_INVALID_VALUE, "%s: null argument", fn);
  if (c->batch != 1 || c->kv_heads <= 0 || c->q_heads <= 0 || c->q_heads % c->kv_heads || c->tokens < 0 || max_count <= 0 || c->capacity <= 0 ||
      (long long)c->tokens + max_count > c->capacity)
    return fail(MLOPS_FBLA_INVALID_VALUE, "%s: batch 1, positive heads (q_heads a multiple of kv_heads), tokens >= 0, max_count > 0, "
                "tokens + max_count <= capacity", fn);
  a = fbla_k_token{};
  mlops_fbla_status st = token_common(fn, t, a);
  if (st != MLOPS_FBLA_OK) return st;
  if (t->batch_stride < D || t->batch_stride % 2 || t->q_group_stride % 2 || t->kv_group_stride % 2 || t->q_group_stride < 0 || t->kv_group_stride < 0)
    return fail(MLOPS_FBLA_INVALID_VALUE, "%s: the row stride (batch_stride) and the group strides must be even, the row at least 128", fn);
  const void *p16[] = {q_out, k_out, v_out, t->freq};
  for (const void *p : p16)
    if (!aligned(p, 16)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: outputs and freq must be 16-byte aligned", fn);
  const void *p4[] = {length, count, t->q, t->k, t->v, t->q_norm, t->k_norm};
  for (const void *p : p4)
    if (!aligned(p, 4)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: length, count and the projection's pointers must be 4-byte aligned", fn);
  a.length = length; a.dcount = count; a.n0 = c->tokens; a.max_count = max_count;
  a.batch = 1; a.q_heads = c->q_heads; a.kv_heads = c->kv_heads;
  a.q_out = q_out; a.k_out = k_out; a.v_out = v_out;
  return MLOPS_FBLA_OK;
}
mlops_fbla_status mlops_fbla_qkv_prefill_at(const mlops_fbla_config *c, const int *length, const int *count, int max_count, const mlops_fbla_token *t,
                                            uint16_t *q_out, uint16_t *k_out, uint16_t *v_out, cudaStream_t stream) {
  fbla_k_token a;
  const mlops_fbla_status st = qkv_chunk_prepare(c, length, count, max_count, t, q_out, k_out, v_out, a);
  if (st != MLOPS_FBLA_OK) return st;
  const cudaError_t e = fbla_k_qkv_chunk_launch(&a, stream);
  if (e != cudaSuccess) return fail(MLOPS_FBLA_CUDA_ERROR, "mlops_fbla_qkv_prefill_at: %s", cudaGetErrorString(e));
  return ok();
}

// ---- sequence shards (include/mlops_fbla_shard.h) ------------------------------------------------------------------------
static mlops_fbla_status shard_args(const char *fn, const mlops_fbla_shard *sh, fbla_k_decode &a) {
  if (!sh || sh->group_first < 0 || sh->group_count < 0 || (sh->windows & ~3))
    return fail(MLOPS_FBLA_INVALID_VALUE, "%s: shard needs group_first >= 0, group_count >= 0, windows in 0..3", fn);
  a.shard_on = 1; a.sh_first = sh->group_first; a.sh_count = sh->group_count; a.sh_windows = sh->windows;
  return MLOPS_FBLA_OK;
}

mlops_fbla_status mlops_fbla_shard_mass(const mlops_fbla_config *c, const mlops_fbla_shard *sh, const uint16_t *q, const mlops_fbla_cache *k,
                                        float *row_mass, void *scratch, size_t scratch_bytes, cudaStream_t stream) {
  constexpr const char *fn = "mlops_fbla_shard_mass";
  if (!row_mass || !aligned(row_mass, 16)) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: row_mass must be a 16-byte aligned device pointer", fn);
  fbla_k_decode a;
  mlops_fbla_status st = prepare_decode(fn, c, nullptr, q, k, nullptr, false, scratch, scratch_bytes, a);
  if (st == MLOPS_FBLA_OK) st = shard_args(fn, sh, a);
  if (st != MLOPS_FBLA_OK) return st;
  a.phase = 1;
  a.row_r = row_mass;
  return launch_decode(fn, a, stream);
}

mlops_fbla_status mlops_fbla_shard_partial(const mlops_fbla_config *c, const mlops_fbla_shard *sh, const uint16_t *q, const mlops_fbla_cache *k,
                                           const float *row_mass_total, float *partial, void *scratch, size_t scratch_bytes,
                                           cudaStream_t stream) {
  constexpr const char *fn = "mlops_fbla_shard_partial";
  if (!row_mass_total || !partial || !aligned(row_mass_total, 16) || !aligned(partial, 16))
    return fail(MLOPS_FBLA_INVALID_VALUE, "%s: row_mass_total and partial must be 16-byte aligned device pointers", fn);
  fbla_k_decode a;
  mlops_fbla_status st = prepare_decode(fn, c, nullptr, q, k, nullptr, false, scratch, scratch_bytes, a);
  if (st == MLOPS_FBLA_OK) st = shard_args(fn, sh, a);
  if (st != MLOPS_FBLA_OK) return st;
  a.phase = 2;
  a.row_r = const_cast<float *>(row_mass_total);
  a.out_partial = partial;
  return launch_decode(fn, a, stream);
}

mlops_fbla_status mlops_fbla_shard_total_mass(int shards, int rows, const float *gathered, float *row_mass_total, cudaStream_t stream) {
  constexpr const char *fn = "mlops_fbla_shard_total_mass";
  if (shards <= 0 || rows <= 0 || !gathered || !row_mass_total) return fail(MLOPS_FBLA_INVALID_VALUE, "%s: shards and rows must be positive, pointers non-null", fn);
  const cudaError_t e = fbla_k_total_mass_launch(gathered, row_mass_total, shards, rows, stream);
  if (e != cudaSuccess) return fail(MLOPS_FBLA_CUDA_ERROR, "%s: %s", fn, cudaGetErrorString(e));
  return ok();
}

mlops_fbla_status mlops_fbla_shard_combine(int rows, const float *partial_sum, uint16_t *output, cudaStream_t stream) {
  constexpr const char *fn = "mlops_fbla_shard_combine";
  if (rows <= 0 || !partial_sum || !output || !aligned(partial_sum, 16) || !aligned(output, 16))
    return fail(MLOPS_FBLA_INVALID_VALUE, "%s: rows must be positive, pointers 16-byte aligned", fn);
  const cudaError_t e = fbla_k_combine_launch(partial_sum, output, rows, stream);
  if (e != cudaSuccess) return fail(MLOPS_FBLA_CUDA_ERROR, "%s: %s", fn, cudaGetErrorString(e));
  return ok();
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
  p.geom[MLOPS_FBLA_GEOM_CAPACITY_GROUPS] = (capacity + G - 1) / G;
  p.geom[MLOPS_FBLA_GEOM_COARSE_BYTES] = 2 * cb * 256; p.geom[MLOPS_FBLA_GEOM_FINE_BYTES] = 2 * fb * 256;
}
int plan_fail(const cudaError_t e, const char *fn) {
  fail(MLOPS_FBLA_CUDA_ERROR, "%s: %s", fn, cudaGetErrorString(e));
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
  const long long uc = SBG * p.geom[MLOPS_FBLA_GEOM_COARSE_BYTES], uf = SBG * p.geom[MLOPS_FBLA_GEOM_FINE_BYTES];
  if (coarse) r.add(MLOPS_FBLA_ARG_COARSE, write, h * hs * uc, uc, gs * uc, (int)cg);
  if (fine) r.add(MLOPS_FBLA_ARG_FINE, write, h * hs * uf, uf, gs * uf, (int)cg);
  if (meta) r.add(MLOPS_FBLA_ARG_META, write, h * hs * 1024, 1024, gs * 1024, (int)cg);
}
void head_windows(Ranges &r, int h, int write, bool sink, bool open) {
  const long long w = (long long)G * D * 2;
  if (sink) { r.add(MLOPS_FBLA_ARG_SINK_K, write, h * w, w); r.add(MLOPS_FBLA_ARG_SINK_V, write, h * w, w); }
  if (open) { r.add(MLOPS_FBLA_ARG_OPEN_K, write, h * w, w); r.add(MLOPS_FBLA_ARG_OPEN_V, write, h * w, w); }
}
}  // namespace
}  // extern "C++"

int mlops_fbla_decode_at_items(const mlops_fbla_config *c, const int *length, const uint16_t *q, const mlops_fbla_cache *k, uint16_t *out,
                               void *scratch, size_t scratch_bytes, int /*per_head*/, mlops_fbla_items *passes, int max) {
  constexpr const char *fn = "mlops_fbla_decode_at_items";
  if (!length) { fail(MLOPS_FBLA_INVALID_VALUE, "%s: null length", fn); return -1; }
  if (c && c->capacity <= 0) { fail(MLOPS_FBLA_INVALID_VALUE, "%s: capacity must be positive", fn); return -1; }
  fbla_k_decode a;
  if (prepare_decode(fn, c, length, q, k, out, true, scratch, scratch_bytes, a) != MLOPS_FBLA_OK) return -1;
  if (max == 0) { ok(); return 4; }
  if (!passes || max < 4) { fail(MLOPS_FBLA_INVALID_VALUE, "%s: room for 4 passes is needed", fn); return -1; }
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
  ok();
  return 4;
}

static int prefill_items(const char *fn, const mlops_fbla_config *c, const int *length, const int *count, int max_count, const uint16_t *q,
                         const uint16_t *k, const uint16_t *v, const mlops_fbla_cache *cache, uint16_t *out, mlops_fbla_items *passes, int max) {
  fbla_k_prefill a;
  if (prefill_at_prepare(fn, c, length, count, max_count, q, k, v, cache, out, a) != MLOPS_FBLA_OK) return -1;
  const int n = q ? 3 : 2;
  if (max == 0) { ok(); return n; }
  if (!passes || max < n) { fail(MLOPS_FBLA_INVALID_VALUE, "%s: room for %d passes is needed", fn, n); return -1; }
  fbla_k_pass info;
  int at = 0, tensor = 0;
  cudaError_t e = fbla_k_close_pass(&a, max_count / G + 1, &info);
  if (e != cudaSuccess) return plan_fail(e, fn);
  fill_pass(passes[at++], MLOPS_FBLA_ITEM_CLOSE, info, "fbla_k_prefill", a);
  if (q) {
    e = fbla_k_attend_pass(&a, &info, &tensor);
    if (e != cudaSuccess) return plan_fail(e, fn);
    fill_pass(passes[at++], tensor ? MLOPS_FBLA_ITEM_TC : MLOPS_FBLA_ITEM_STREAM, info, "fbla_k_prefill", a);
  }
  e = fbla_k_finish_pass(&a, &info);
  if (e != cudaSuccess) return plan_fail(e, fn);
  fill_pass(passes[at++], MLOPS_FBLA_ITEM_FINISH, info, "fbla_k_prefill", a);
  for (int i = 0; i < at; ++i) { cache_geom(passes[i], a.hs, a.gs, c->capacity, a.cb, a.fb); passes[i].geom[3] = max_count; }
  ok();
  return at;
}

int mlops_fbla_prefill_at_items(const mlops_fbla_config *c, const int *length, const int *count, int max_count, const uint16_t *q, const uint16_t *k,
                                const uint16_t *v, const mlops_fbla_cache *cache, uint16_t *out, mlops_fbla_items *passes, int max) {
  if (!count) { fail(MLOPS_FBLA_INVALID_VALUE, "mlops_fbla_prefill_at_items: null argument"); return -1; }
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
  if (qkv_at_prepare(c, length, t, cache, cl, a) != MLOPS_FBLA_OK) return -1;
  if (max == 0) { ok(); return 2; }
  if (!passes || max < 2) { fail(MLOPS_FBLA_INVALID_VALUE, "%s: room for 2 passes is needed", fn); return -1; }
  fbla_k_pass info;
  cudaError_t e = fbla_k_close_pass(&cl, 1, &info);
  if (e != cudaSuccess) return plan_fail(e, fn);
  fill_pass(passes[0], MLOPS_FBLA_ITEM_CLOSE, info, "fbla_k_prefill", cl);
  e = fbla_k_qkv_token_pass(&a, &info);
  if (e != cudaSuccess) return plan_fail(e, fn);
  fill_pass(passes[1], MLOPS_FBLA_ITEM_QKV, info, "fbla_k_token", a);
  for (int i = 0; i < 2; ++i) { cache_geom(passes[i], cl.hs, cl.gs, c->capacity, cl.cb, cl.fb); passes[i].geom[3] = 1; }
  ok();
  return 2;
}

int mlops_fbla_qkv_prefill_at_items(const mlops_fbla_config *c, const int *length, const int *count, int max_count, const mlops_fbla_token *t,
                                    uint16_t *q_out, uint16_t *k_out, uint16_t *v_out, mlops_fbla_items *passes, int max) {
  constexpr const char *fn = "mlops_fbla_qkv_prefill_at_items";
  fbla_k_token a;
  if (qkv_chunk_prepare(c, length, count, max_count, t, q_out, k_out, v_out, a) != MLOPS_FBLA_OK) return -1;
  if (max == 0) { ok(); return 1; }
  if (!passes || max < 1) { fail(MLOPS_FBLA_INVALID_VALUE, "%s: room for 1 pass is needed", fn); return -1; }
  fbla_k_pass info;
  const cudaError_t e = fbla_k_qkv_chunk_pass(&a, &info);
  if (e != cudaSuccess) return plan_fail(e, fn);
  fill_pass(passes[0], MLOPS_FBLA_ITEM_QKV_CHUNK, info, "fbla_k_token", a);
  passes[0].geom[3] = max_count;
  ok();
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
  const long long row = D * 2;  // bytes of one head vector
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

const char *mlops_fbla_last_error(void) { return error_buf; }

}  // extern "C"
