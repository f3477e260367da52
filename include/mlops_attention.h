/* Umbrella header of libmlops_attention for B200: what a program written against the reference package includes
 * (reference: attention/include/mlops_attention.h:6-13 -- the package's version macro and its one attention family).
 * MLOPS_ATTENTION_VERSION names the interface version this library implements, so `#if`/string checks made against the
 * reference keep working. mlops_fbla.h: the FBLA compressed-KV cache, prefill and decode; the work-item plans
 * (mlops_fbla_items.h) and the sequence shards (mlops_fbla_shard.h, an addition of this library) are included on demand. */
#ifndef MLOPS_ATTENTION_H
#define MLOPS_ATTENTION_H

#define MLOPS_ATTENTION_VERSION "0.4.0"

#include "mlops_fbla.h"

#endif /* MLOPS_ATTENTION_H */
