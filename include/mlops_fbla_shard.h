/* Sequence-sharded decode: one long context split over several GPUs of a box.
 *
 * No counterpart in the reference (it is single-GPU; attention/fbla/src has no multi-device code). The reference's
 * decode is a sum over sub-blocks weighted by 2^(m - R), R the log2 of the row's total coarse mass; that sum splits
 * over GPUs if every GPU uses the same R. So a sharded decode is two local passes with one small exchange after each:
 *
 *   1. mlops_fbla_shard_mass     coarse pass over the shard; writes the rows' LOCAL log2 mass (-inf if the shard
 *                                holds nothing of a row)                                  -> row_mass [batch * q_heads]
 *      exchange A (caller)       R_total[i] = log2 sum_shards 2^row_mass[i]                  (all-gather of 4 B per row)
 *   2. mlops_fbla_shard_partial  select with R_total, refine, and the shard's share of every row in units of 2^-R_total
 *                                                       -> partial [batch * q_heads][MLOPS_FBLA_PARTIAL_STRIDE] floats:
 *                                                          o[0..127], then l at index 128
 *      exchange B (caller)       element-wise sum of `partial` over the shards               (all-reduce of 528 B per row)
 *   3. mlops_fbla_shard_combine  output = bf16(o / l)
 *
 * Each shard is an ordinary mlops_fbla_cache holding a contiguous run of whole 128-token groups of the sequence (its
 * cfg->tokens is the LOCAL token count), written by mlops_fbla_prefill like any cache. The shard descriptor says which
 * of its local groups take part as closed (quantized) groups and whether its BF16 windows are the sequence's sink /
 * open group: first shard: windows = 1, closed groups 1 ..; middle shards: windows = 0, closed groups 0 ..; last
 * shard: windows = 2, its last group open. A shard whose last group must count as closed needs one more token after
 * it in its local cache (the first token of the next shard), exactly as a group closes in a growing cache.
 * The row order of row_mass / partial is internal but identical on every shard of the same configuration; the
 * caller only adds them up. Scratch: mlops_fbla_decode_scratch_bytes(cfg) per shard, kept between pass 1 and pass 2.
 */
#ifndef MLOPS_FBLA_SHARD_H
#define MLOPS_FBLA_SHARD_H

#include "mlops_fbla.h"

#ifdef __cplusplus
extern "C" {
#endif

enum { MLOPS_FBLA_PARTIAL_STRIDE = 132 };

typedef struct {
  int group_first, group_count; /* local closed groups [group_first, group_first + group_count) */
  int windows;                  /* bit 0: the local sink window is the sequence's; bit 1: the local open window is */
} mlops_fbla_shard;

mlops_fbla_status mlops_fbla_shard_mass(const mlops_fbla_config *cfg, const mlops_fbla_shard *shard, const uint16_t *q,
                                        const mlops_fbla_cache *cache, float *row_mass, void *scratch, size_t scratch_bytes,
                                        cudaStream_t stream);
mlops_fbla_status mlops_fbla_shard_partial(const mlops_fbla_config *cfg, const mlops_fbla_shard *shard, const uint16_t *q,
                                           const mlops_fbla_cache *cache, const float *row_mass_total, float *partial,
                                           void *scratch, size_t scratch_bytes, cudaStream_t stream);
/* ---- the whole step with the exchanges done by the GPUs themselves ---------------------------------------------------------
 * Instead of two host-launched collectives the ranks store their few KB straight into each other's memory (NVLink peer
 * stores, one release flag per exchange, bounded acquire polls on the receiving side; mlops_b200/csrc/kernels/fbla_link.cu).
 * Every rank owns a "mailbox" of mlops_fbla_shard_mailbox_bytes(world, batch * q_heads) bytes that all ranks can address
 * (symmetric / peer-mapped memory: cudaIpc handles, cuMemMap, torch's symmetric memory ...), zero-filled ONCE before the
 * first step and after that touched only by these calls. `mailboxes` lists the `world` base addresses as THIS rank sees
 * them (mailboxes[rank] its own). mlops_fbla_shard_step enqueues one decode step -- nine kernel launches, no host
 * synchronisation, no allocation; it can be captured in a CUDA graph -- and leaves the full output on every rank (the
 * ranks add the shards' sums in rank order, so all hold the same bits). All ranks must make the same sequence of calls.
 * A peer that never arrives: after wait_polls polls (64 ns apart; 0 = about a quarter of a second) the wait gives up, the
 * output rows become NaN and mlops_fbla_shard_link_status reports which exchange and which rank (0 = healthy). */
enum { MLOPS_FBLA_SHARD_MAX_RANKS = 8 };
typedef struct {
  int rank, world;          /* world <= MLOPS_FBLA_SHARD_MAX_RANKS */
  void *const *mailboxes;   /* host array of `world` device pointers, 256-byte aligned */
  unsigned wait_polls;
} mlops_fbla_shard_link;

size_t mlops_fbla_shard_mailbox_bytes(int world, int rows);
mlops_fbla_status mlops_fbla_shard_step(const mlops_fbla_config *cfg, const mlops_fbla_shard *shard, const mlops_fbla_shard_link *link,
                                        const uint16_t *q, const mlops_fbla_cache *cache, uint16_t *output, void *scratch,
                                        size_t scratch_bytes, cudaStream_t stream);
/* reads this rank's status word (synchronises with `stream` first): 0, or 1 / 2 (the mass / the sum exchange gave up) + 16 * rank */
int mlops_fbla_shard_link_status(const mlops_fbla_shard_link *link, int rows, cudaStream_t stream);

/* exchange A's arithmetic: gathered [shards][rows] local masses -> row_mass_total [rows] */
mlops_fbla_status mlops_fbla_shard_total_mass(int shards, int rows, const float *gathered, float *row_mass_total, cudaStream_t stream);
mlops_fbla_status mlops_fbla_shard_combine(int rows, const float *partial_sum, uint16_t *output, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MLOPS_FBLA_SHARD_H */
