/* C ABI of the batched KV-cache decode attention (libmoe_b200.so, sm_100a).
 *
 * Replaces, for many sequences at once, the attention arithmetic of
 * MultiHeadAttention::forward_cached (reference attention.rs:344-398): rotate the new queries and keys
 * (rope.rs:170-225, rotate-half pairing of channel j with j + head_dim / 2), append the new keys and
 * values to each sequence's cache (KvCache::append, attention.rs:65-78: post-RoPE rows of
 * kv_heads * head_dim values), then for every new row softmax(q . K^T / sqrt(head_dim)) V over the
 * positions it may see (head_scores, attention.rs:1100-1130; accumulate_head_output, :1133-1160; query
 * head h reads key/value head h / (num_heads / kv_heads)).  The projections around it (query, key,
 * value, output Linear layers) stay with the caller, as they do for the MoE layer.
 *
 * The reference decodes one sequence per call; here `sequences` caches advance together, each with its
 * own length.  All pointers are device pointers unless said otherwise.  Status codes are the moe_status
 * values of moe_b200.h.
 */
#ifndef KV_ATTENTION_B200_H
#define KV_ATTENTION_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct kv_cache kv_cache_t;

typedef struct {
  int32_t sequences;    /* caches that advance together */
  int32_t num_heads;    /* query heads */
  int32_t kv_heads;     /* key/value heads; num_heads is a multiple (attention.rs:178) */
  int32_t head_dim;     /* 8, 16, 32, 64, 128 or 256 */
  int32_t capacity;     /* positions per sequence (KvCache::with_capacity, attention.rs:39-48) */
  int32_t max_seq_len;  /* length of the RoPE tables (rope.rs:71-97); capacity <= max_seq_len */
  float rope_base;      /* 10000.0 in the reference's configs */
  int32_t rope;         /* 0: no rotation (rope_enabled == false) */
  int32_t precision;    /* MOE_PRECISION_F32 (0) or MOE_PRECISION_BF16 (1): type of q, k, v, out and of the cache */
  int32_t device;
} kv_cache_config_t;

/* KvCache::with_capacity for `sequences` sequences.  InvalidConfig for the shapes the reference refuses
 * (attention.rs:173-186, rope.rs:72-76) and for head_dim values the kernels do not cover. */
int32_t kv_cache_create(const kv_cache_config_t* config, kv_cache_t** out);
void kv_cache_destroy(kv_cache_t* cache);
const char* kv_cache_last_error(const kv_cache_t* cache);

/* KvCache::clear (attention.rs:58-62) for every sequence, or for one when sequence >= 0. */
int32_t kv_cache_clear(kv_cache_t* cache, int32_t sequence, void* stream);

/* KvCache::len of every sequence into host memory (read from the device; synchronises the stream).
 * The capacity checks of the calls below use a host copy of the lengths that every call keeps up to
 * date; a step replayed from a captured CUDA graph advances the device lengths only, and this call
 * brings the host copy back in line.  A replayed step that no longer fits is caught on the device: for a
 * sequence whose cache cannot take the step's rows the kernels store nothing, leave its length alone, write
 * zeros as its merged heads and mark it; the other sequences of the call proceed.  This call reports such a
 * mark as MOE_INVALID_INPUT ("SequenceTooLong", attention.rs:364-371) once and clears it; kv_cache_clear /
 * kv_cache_truncate of the sequence clear it too. */
int32_t kv_cache_lengths(kv_cache_t* cache, int32_t* lengths_host, void* stream);

/* forward_cached without the projections, for sequences first_sequence .. first_sequence + n_sequences - 1
 * (all of them for a decode step, one of them for the prefill of a new request).
 * q [n_sequences * rows_per_sequence, num_heads * head_dim], k and v [same rows, kv_heads * head_dim],
 * rows of one sequence adjacent (row = j * rows_per_sequence + i for the j-th sequence of the range);
 * row i of a sequence sits at position len + i and sees positions 0 ..= len + i.  q, k and v are the
 * projections BEFORE rotation (`project`, attention.rs:920-944, rotates queries and keys; here the call
 * does).  q is scratch: one kernel path rotates it in place, the other rotates in registers and leaves it
 * alone, so its contents after the call are unspecified; k and v are read only.
 * merged [rows, num_heads * head_dim] is the input of the output projection.
 * SequenceTooLong -> MOE_INVALID_INPUT when a cache would pass its capacity (rope.rs:194-200); nothing
 * is appended in that case. */
int32_t kv_attention_forward_cached(kv_cache_t* cache, int32_t first_sequence, int32_t n_sequences, void* q,
                                    const void* k, const void* v, int32_t rows_per_sequence, void* merged,
                                    void* stream);

/* Drops the newest positions of a sequence (all sequences when sequence < 0) so that `length` remain;
 * a length above the current one is InvalidInput.  Used to replay a decode step at a fixed history. */
int32_t kv_cache_truncate(kv_cache_t* cache, int32_t sequence, int32_t length, void* stream);

/* Read-only views for tests and for handing a cache back: keys / values of one sequence,
 * [len, kv_heads * head_dim] as f32, into host memory. */
int32_t kv_cache_read(kv_cache_t* cache, int32_t sequence, float* keys_host, float* values_host, void* stream);

#ifdef __cplusplus
}
#endif
#endif
