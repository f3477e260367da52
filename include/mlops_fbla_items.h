/* FBLA work items: a call described as ordered passes of independent items, for an executor that runs them from kernels
 * of its own instead of this library's stream launches. ABI-identical restatement of the reference's
 * attention/include/mlops_fbla_items.h (same enums, struct layouts, function names and argument orders); the passes,
 * entries and argument blobs it returns describe THIS library's kernels.
 *
 * A plan builder takes the arguments of the equally named call, validates them the same way, and writes up to `max`
 * passes, returning their number (-1 and mlops_fbla_last_error() on bad arguments; max = 0 only counts). Plans are for
 * the current device; building one allocates nothing and launches nothing.
 *
 * Pass: `items` independent items; item i is the CTA (x, y, z) of the grid geom[0..2] of the equivalent launch,
 * x = i % geom[0], y = (i / geom[0]) % geom[1], z = i / (geom[0] * geom[1]). `threads` is the exact CTA size,
 * `smem_bytes` the shared memory the executor hands the entry (16-byte aligned is enough: entries re-align inside and
 * the size includes the slack), `regs` the registers per thread of this library's kernel, `arch` the virtual
 * architecture to compile the entries for (100: compute_100a). `args` is the pass's device argument structure
 * (`args_type`, `args_bytes` bytes, unused bytes zero): the entry's first argument is a 16-byte aligned device copy.
 * `entry` names the device function (include/mlops_fbla_items.cuh) called as entry(args, shared_memory_pointer).
 *
 * Order and dependencies: passes run in order; an item depends on items of earlier passes exactly where their
 * mlops_fbla_item_access ranges overlap (read after write, write after read, write after write). Ranges whose place
 * depends on a device length or count are envelopes over every allowed value and may overlap inside a pass; the bytes
 * actually stored by the items of one pass are disjoint. The executor provides GPU-scope release / acquire ordering
 * between dependent items; entries contain CTA barriers but no waits on other CTAs. An entry that uses tensor memory
 * allocates and frees it inside the call.
 *
 * reference: attention/include/mlops_fbla_items.h:3-8 (purpose), :14-35 (enums), :37-44 (ranges), :46-53 (geom slots),
 * :55-83 (pass contract), :85-116 (functions). */
#ifndef MLOPS_FBLA_ITEMS_H
#define MLOPS_FBLA_ITEMS_H

#include "mlops_fbla.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Pass kinds (values as the reference's). This library emits: CLOSE (one group the chunk may close, x, of KV head y),
 * STREAM (8 query rows of KV head y on CUDA cores: chunks of fewer than 64 rows), TC (256 query rows of KV head y on
 * tcgen05 tensor cores; no split pieces, no TC_MERGE pass, no TRANSCODE: this library keeps no images; a prefill plan whose
 * count lives on the device and may reach 64 rows has a TC and a STREAM pass, of which the count activates one), FINISH (one KV
 * head's windows), COARSE / REFINE (CTA x of the persistent pass), SELECT (slice x of virtual head y), MERGE (one output
 * row), QKV (one (batch, KV head)), QKV_CHUNK (8 positions x of KV head y). */
enum { MLOPS_FBLA_ITEM_CLOSE = 1, MLOPS_FBLA_ITEM_TRANSCODE, MLOPS_FBLA_ITEM_STREAM, MLOPS_FBLA_ITEM_TC,
       MLOPS_FBLA_ITEM_TC_MERGE, MLOPS_FBLA_ITEM_FINISH, MLOPS_FBLA_ITEM_COARSE, MLOPS_FBLA_ITEM_SELECT,
       MLOPS_FBLA_ITEM_REFINE, MLOPS_FBLA_ITEM_MERGE, MLOPS_FBLA_ITEM_QKV, MLOPS_FBLA_ITEM_QKV_CHUNK };

/* The call argument a range is relative to. */
enum {
  MLOPS_FBLA_ARG_Q = 0, MLOPS_FBLA_ARG_K, MLOPS_FBLA_ARG_V, MLOPS_FBLA_ARG_OUT,
  MLOPS_FBLA_ARG_COARSE, MLOPS_FBLA_ARG_FINE, MLOPS_FBLA_ARG_META, MLOPS_FBLA_ARG_SINK_K, MLOPS_FBLA_ARG_SINK_V,
  MLOPS_FBLA_ARG_OPEN_K, MLOPS_FBLA_ARG_OPEN_V, MLOPS_FBLA_ARG_IMAGES,
  MLOPS_FBLA_ARG_SCRATCH,
  MLOPS_FBLA_ARG_LENGTH, MLOPS_FBLA_ARG_COUNT,
  MLOPS_FBLA_ARG_TQ, MLOPS_FBLA_ARG_TK, MLOPS_FBLA_ARG_TV,
  MLOPS_FBLA_ARG_TQN, MLOPS_FBLA_ARG_TKN, MLOPS_FBLA_ARG_TFREQ, MLOPS_FBLA_ARG_TQ_OUT,
  MLOPS_FBLA_ARG_PART_ML, MLOPS_FBLA_ARG_PART_O
};

/* `rows` runs of `bytes` bytes, `stride` bytes apart, from `offset`, relative to argument `arg`; write: 0 read, 1 store. */
typedef struct {
  int arg, write;
  long long offset, bytes, stride;
  int rows;
} mlops_fbla_item_range;

/* Geometry slots shared by all kinds; LSE .. COUNTS are byte offsets of the decode scratch arrays. */
enum {
  MLOPS_FBLA_GEOM_GRID_X = 0, MLOPS_FBLA_GEOM_GRID_Y, MLOPS_FBLA_GEOM_GRID_Z,
  MLOPS_FBLA_GEOM_HEAD_STRIDE = 20, MLOPS_FBLA_GEOM_GROUP_STRIDE, MLOPS_FBLA_GEOM_CAPACITY_GROUPS,
  MLOPS_FBLA_GEOM_COARSE_BYTES, MLOPS_FBLA_GEOM_FINE_BYTES,
  MLOPS_FBLA_GEOM_LSE, MLOPS_FBLA_GEOM_PART, MLOPS_FBLA_GEOM_DPART, MLOPS_FBLA_GEOM_ROW_LSE,
  MLOPS_FBLA_GEOM_ITEMS, MLOPS_FBLA_GEOM_COUNTS
};

#define MLOPS_FBLA_ITEM_ARGS_BYTES 256
typedef struct {
  int kind, items, threads, smem_bytes, regs, arch;
  char entry[160], args_type[48];
  int args_bytes;
  union { long long align; unsigned char bytes[MLOPS_FBLA_ITEM_ARGS_BYTES]; } args;
  long long geom[32];
} mlops_fbla_items;

int mlops_fbla_prefill_at_items(const mlops_fbla_config *cfg, const int *length, const int *count, int max_count,
                                const uint16_t *q, const uint16_t *k, const uint16_t *v, const mlops_fbla_cache *cache,
                                uint16_t *output, mlops_fbla_items *passes, int max);
int mlops_fbla_append_at_items(const mlops_fbla_config *cfg, const int *length, const uint16_t *k, const uint16_t *v,
                               const mlops_fbla_cache *cache, mlops_fbla_items *passes, int max);
/* per_head does not change the plan: the passes always use the stream call's persistent launch shape and scratch layout
 * (a scratch sized with mlops_fbla_decode_scratch_bytes_for(cfg, per_head) for any per_head >= 0 is large enough). */
int mlops_fbla_decode_at_items(const mlops_fbla_config *cfg, const int *length, const uint16_t *q,
                               const mlops_fbla_cache *cache, uint16_t *output, void *scratch, size_t scratch_bytes,
                               int per_head, mlops_fbla_items *passes, int max);
int mlops_fbla_qkv_at_items(const mlops_fbla_config *cfg, const int *length, const mlops_fbla_token *token,
                            const mlops_fbla_cache *cache, mlops_fbla_items *passes, int max);
/* One QKV_CHUNK pass; reads are relative to token->q / k / v (ARG_TQ / TK / TV), writes to q_out / k_out / v_out (ARG_Q / K / V). */
int mlops_fbla_qkv_prefill_at_items(const mlops_fbla_config *cfg, const int *length, const int *count, int max_count,
                                    const mlops_fbla_token *token, uint16_t *q_out, uint16_t *k_out, uint16_t *v_out,
                                    mlops_fbla_items *passes, int max);

/* For an executor that generates its kernels' source: the statements that run item `item` of pass p on its CTA, as a C
 * string of at most `capacity` bytes (returns its length, -1 if it does not fit or the kind is unknown). They name
 * `args` (the aligned device copy of the blob), `item` and `sm` (the shared memory), call
 * mlops_fbla::position(item, nx, ny, nz) and a CTA barrier, then the entry. The executor defines mlops_fbla::Pos
 * (static x y z nx ny nz tid, and ro(const int *) for reads of the device length / count) and mlops_fbla::position
 * before including mlops_fbla_items.cuh. */
int mlops_fbla_item_call(const mlops_fbla_items *p, char *out, size_t capacity);

/* The ranges item `item` of pass `pass` reads and writes, at most max of them; returns their total number (max = 0 with
 * ranges NULL only counts); -1 for NULL passes, an item or pass out of range, max < 0, or NULL ranges with max > 0. */
int mlops_fbla_item_access(const mlops_fbla_items *passes, int npasses, int pass, int item, mlops_fbla_item_range *ranges,
                           int max);

#ifdef __cplusplus
}
#endif
#endif /* MLOPS_FBLA_ITEMS_H */
