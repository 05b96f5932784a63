/*
 * b200kv prefix cache — host-side C ABI (no GPU work, no CUDA calls).
 *
 * The page-level prefix cache a paged-KV executor keeps beside its page pool: which physical
 * pages hold the K/V of a prompt (or of a page-aligned prefix of it) that was prefilled before.
 * Replaces the two OrderedDict caches of the reference executor and the loops over them
 * (lite_llama/executor/model_executor.py:293-303 the tables, :547-568 exact lookup, :570-620
 * longest-prefix lookup with the parent-fingerprint chain :622-625, :627-656 block store with
 * LRU eviction, :658-683 exact store with LRU eviction).
 *
 * Two tables, both least-recently-used with a fixed capacity:
 *   exact : whole prompt                     -> (pages, token count, first generated token)
 *   block : (fingerprint of the blocks before it, the page_size tokens of one block)
 *                                            -> (one page, tokens up to and including the block)
 * The cache never touches the page pool.  It tells its caller which references to take and to
 * drop, in order, and the caller applies them to its reference counts
 * (PagedKVCacheManager.add_ref / free, lite_llama/executor/paged_attention.py:85-105).
 *
 * Token ids and page ids are int64.  A handle is not thread-safe; the reference drives its
 * caches from the single scheduler thread (lite_llama/server.py:457-469).
 */
#ifndef B200KV_PREFIX_CACHE_H_
#define B200KV_PREFIX_CACHE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* NULL on bad arguments (page_size, capacities must be positive). */
void* b200kv_prefix_cache_create(int page_size, int64_t max_exact_entries, int64_t max_block_entries);
void b200kv_prefix_cache_destroy(void* cache);

/* Entries currently held: which = 0 exact table, 1 block table.  -1 on a bad argument. */
int64_t b200kv_prefix_cache_entries(const void* cache, int which);

/*
 * Exact lookup (model_executor.py:558-562, :587-590).  On a hit the entry becomes the most
 * recently used, its pages are copied to pages_out (capacity pages_cap) and the return value is
 * their number; *num_tokens_out and *first_token_out receive the stored values.
 * Returns -1 on a miss, -2 when pages_cap is too small (nothing touched), -3 on a bad argument.
 */
int64_t b200kv_prefix_cache_lookup_exact(void* cache, const int64_t* tokens, int64_t n_tokens,
                                         int64_t* pages_out, int64_t pages_cap,
                                         int64_t* num_tokens_out, int64_t* first_token_out);

/*
 * Longest page-aligned prefix through the block table (model_executor.py:597-612): full
 * blocks are looked up in order, each under the fingerprint of the chain before it, until the
 * first miss; every block found becomes the most recently used.  Returns the number of pages
 * matched (0 = no block matched) and writes them to pages_out; *matched_tokens_out is the token
 * count stored with the last matched block.  -2 when pages_cap is too small, -3 bad argument.
 */
int64_t b200kv_prefix_cache_lookup_blocks(void* cache, const int64_t* tokens, int64_t n_tokens,
                                          int64_t* pages_out, int64_t pages_cap,
                                          int64_t* matched_tokens_out);

/*
 * Remember a finished prompt (store_paged_request_prefix + _store_paged_prompt_blocks,
 * model_executor.py:658-683, :627-656): pages[0 .. n_pages) are the request's pages in logical
 * order, num_tokens its token count, first_token the first token generated after the prompt.
 * If the prompt is already in the exact table nothing changes and 0 is returned.  Otherwise the
 * reference changes the caller must make are recorded, in the reference's order:
 *   +1 on every page of the request (the exact entry's reference),
 *   per full block not yet in the block table: +1 on its page, then -1 on the page of every
 *     block entry evicted to make room,
 *   then -1 on every page of every exact entry evicted to make room;
 * the return value is their number, to be read with b200kv_prefix_cache_ref_ops.
 * -3 on a bad argument.
 */
int64_t b200kv_prefix_cache_store(void* cache, const int64_t* tokens, int64_t n_tokens,
                                  const int64_t* pages, int64_t n_pages,
                                  int64_t num_tokens, int64_t first_token);

/*
 * The reference changes recorded by the last store: pages_out[i] gets delta_out[i] (+1 / -1),
 * i in order.  Returns the number written, or -2 when cap is too small.
 */
int64_t b200kv_prefix_cache_ref_ops(const void* cache, int64_t* pages_out, int32_t* delta_out, int64_t cap);

/* Drop every entry; the pages the cache held a reference on are recorded as -1 operations
 * (read them with b200kv_prefix_cache_ref_ops).  Returns their number. */
int64_t b200kv_prefix_cache_clear(void* cache);

#ifdef __cplusplus
}
#endif
#endif /* B200KV_PREFIX_CACHE_H_ */
