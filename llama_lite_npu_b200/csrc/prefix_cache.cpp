// Host-side prefix cache of the paged-KV executor: exact-prompt table and block table with a
// parent-fingerprint chain, both least-recently-used.  C++17, no CUDA.  See
// include/b200kv_prefix_cache.h for the contract and the reference code it replaces
// (lite_llama/executor/model_executor.py:547-683).
//
// Layout: each table is a doubly linked list in recency order (front = oldest) plus a hash index
// from a 64-bit fingerprint to list nodes; equal fingerprints are resolved by comparing the stored
// tokens, so a fingerprint collision costs a comparison, never a wrong hit.  A block's key is the
// fingerprint of the chain before it together with its own tokens; the fingerprint that the next
// block chains on is the hash of exactly that pair.
#include <cstdint>
#include <cstring>
#include <list>
#include <new>
#include <unordered_map>
#include <utility>
#include <vector>

#include "b200kv_prefix_cache.h"

namespace {

constexpr uint64_t kRootFingerprint = 0x6b32303062766b70ull;   // "no parent"

inline uint64_t mix64(uint64_t x) {
  x ^= x >> 30;
  x *= 0xbf58476d1ce4e5b9ull;
  x ^= x >> 27;
  x *= 0x94d049bb133111ebull;
  x ^= x >> 31;
  return x;
}

uint64_t fingerprint(uint64_t parent, const int64_t* tokens, int64_t n) {
  uint64_t h = mix64(parent ^ (static_cast<uint64_t>(n) * 0x9e3779b97f4a7c15ull));
  for (int64_t i = 0; i < n; ++i) h = mix64(h ^ (static_cast<uint64_t>(tokens[i]) + 0x9e3779b97f4a7c15ull + (h << 6)));
  return h;
}

struct ExactEntry {
  uint64_t fp;
  std::vector<int64_t> tokens;
  std::vector<int64_t> pages;
  int64_t num_tokens;
  int64_t first_token;
};

struct BlockEntry {
  uint64_t fp;       // fingerprint of (parent, tokens): the next block's parent
  uint64_t parent;
  std::vector<int64_t> tokens;
  int64_t page;
  int64_t token_count;
};

struct RefOp {
  int64_t page;
  int32_t delta;
};

class PrefixCache {
 public:
  PrefixCache(int page_size, int64_t max_exact, int64_t max_block)
      : page_size_(page_size), max_exact_(max_exact), max_block_(max_block) {}

  int64_t entries(int which) const {
    return which == 0 ? static_cast<int64_t>(exact_.size()) : static_cast<int64_t>(block_.size());
  }

  std::list<ExactEntry>::iterator find_exact(uint64_t fp, const int64_t* tokens, int64_t n) {
    auto range = exact_index_.equal_range(fp);
    for (auto it = range.first; it != range.second; ++it) {
      const ExactEntry& e = *it->second;
      if (static_cast<int64_t>(e.tokens.size()) == n &&
          (n == 0 || std::memcmp(e.tokens.data(), tokens, sizeof(int64_t) * n) == 0))
        return it->second;
    }
    return exact_.end();
  }

  std::list<BlockEntry>::iterator find_block(uint64_t fp, uint64_t parent, const int64_t* tokens) {
    auto range = block_index_.equal_range(fp);
    for (auto it = range.first; it != range.second; ++it) {
      const BlockEntry& e = *it->second;
      if (e.parent == parent && std::memcmp(e.tokens.data(), tokens, sizeof(int64_t) * page_size_) == 0)
        return it->second;
    }
    return block_.end();
  }

  int64_t lookup_exact(const int64_t* tokens, int64_t n, int64_t* pages_out, int64_t cap, int64_t* num_tokens,
                       int64_t* first_token) {
    auto it = find_exact(fingerprint(kRootFingerprint, tokens, n), tokens, n);
    if (it == exact_.end()) return -1;
    const int64_t np = static_cast<int64_t>(it->pages.size());
    if (np > cap) return -2;
    exact_.splice(exact_.end(), exact_, it);   // most recently used; iterators stay valid
    if (np > 0) std::memcpy(pages_out, it->pages.data(), sizeof(int64_t) * np);
    *num_tokens = it->num_tokens;
    *first_token = it->first_token;
    return np;
  }

  int64_t lookup_blocks(const int64_t* tokens, int64_t n, int64_t* pages_out, int64_t cap, int64_t* matched_tokens) {
    const int64_t blocks = n / page_size_;
    if (blocks > cap) return -2;
    uint64_t parent = kRootFingerprint;
    int64_t found = 0;
    *matched_tokens = 0;
    for (int64_t b = 0; b < blocks; ++b) {
      const int64_t* bt = tokens + b * page_size_;
      const uint64_t fp = fingerprint(parent, bt, page_size_);
      auto it = find_block(fp, parent, bt);
      if (it == block_.end()) break;
      block_.splice(block_.end(), block_, it);
      pages_out[found++] = it->page;
      *matched_tokens = it->token_count;
      parent = fp;
    }
    return found;
  }

  int64_t store(const int64_t* tokens, int64_t n, const int64_t* pages, int64_t n_pages, int64_t num_tokens,
                int64_t first_token) {
    ops_.clear();
    const uint64_t fp = fingerprint(kRootFingerprint, tokens, n);
    if (find_exact(fp, tokens, n) != exact_.end()) return 0;
    for (int64_t i = 0; i < n_pages; ++i) ops_.push_back({pages[i], +1});
    exact_.push_back(ExactEntry{fp, std::vector<int64_t>(tokens, tokens + n),
                                std::vector<int64_t>(pages, pages + n_pages), num_tokens, first_token});
    exact_index_.emplace(fp, std::prev(exact_.end()));

    // the prompt's full blocks, each chained on the fingerprint of the blocks before it
    int64_t blocks = n / page_size_;
    if (blocks > n_pages) blocks = n_pages;
    uint64_t parent = kRootFingerprint;
    for (int64_t b = 0; b < blocks; ++b) {
      const int64_t* bt = tokens + b * page_size_;
      const uint64_t bfp = fingerprint(parent, bt, page_size_);
      auto it = find_block(bfp, parent, bt);
      if (it != block_.end()) {
        block_.splice(block_.end(), block_, it);
      } else {
        ops_.push_back({pages[b], +1});
        block_.push_back(BlockEntry{bfp, parent, std::vector<int64_t>(bt, bt + page_size_), pages[b],
                                    (b + 1) * static_cast<int64_t>(page_size_)});
        block_index_.emplace(bfp, std::prev(block_.end()));
        while (static_cast<int64_t>(block_.size()) > max_block_) evict_block();
      }
      parent = bfp;
    }
    while (static_cast<int64_t>(exact_.size()) > max_exact_) evict_exact();
    return static_cast<int64_t>(ops_.size());
  }

  int64_t clear() {
    ops_.clear();
    while (!block_.empty()) evict_block();
    while (!exact_.empty()) evict_exact();
    return static_cast<int64_t>(ops_.size());
  }

  const std::vector<RefOp>& ops() const { return ops_; }

 private:
  void evict_block() {
    auto victim = block_.begin();
    auto range = block_index_.equal_range(victim->fp);
    for (auto it = range.first; it != range.second; ++it)
      if (it->second == victim) {
        block_index_.erase(it);
        break;
      }
    ops_.push_back({victim->page, -1});
    block_.erase(victim);
  }
  void evict_exact() {
    auto victim = exact_.begin();
    auto range = exact_index_.equal_range(victim->fp);
    for (auto it = range.first; it != range.second; ++it)
      if (it->second == victim) {
        exact_index_.erase(it);
        break;
      }
    for (int64_t p : victim->pages) ops_.push_back({p, -1});
    exact_.erase(victim);
  }

  int page_size_;
  int64_t max_exact_, max_block_;
  std::list<ExactEntry> exact_;
  std::unordered_multimap<uint64_t, std::list<ExactEntry>::iterator> exact_index_;
  std::list<BlockEntry> block_;
  std::unordered_multimap<uint64_t, std::list<BlockEntry>::iterator> block_index_;
  std::vector<RefOp> ops_;
};

inline PrefixCache* as_cache(void* p) { return static_cast<PrefixCache*>(p); }

}  // namespace

extern "C" {

void* b200kv_prefix_cache_create(int page_size, int64_t max_exact_entries, int64_t max_block_entries) {
  if (page_size <= 0 || max_exact_entries <= 0 || max_block_entries <= 0) return nullptr;
  return new (std::nothrow) PrefixCache(page_size, max_exact_entries, max_block_entries);
}

void b200kv_prefix_cache_destroy(void* cache) { delete as_cache(cache); }

int64_t b200kv_prefix_cache_entries(const void* cache, int which) {
  if (cache == nullptr || (which != 0 && which != 1)) return -1;
  return static_cast<const PrefixCache*>(cache)->entries(which);
}

int64_t b200kv_prefix_cache_lookup_exact(void* cache, const int64_t* tokens, int64_t n_tokens, int64_t* pages_out,
                                         int64_t pages_cap, int64_t* num_tokens_out, int64_t* first_token_out) {
  if (cache == nullptr || n_tokens < 0 || (n_tokens > 0 && tokens == nullptr) || pages_cap < 0 ||
      (pages_cap > 0 && pages_out == nullptr) || num_tokens_out == nullptr || first_token_out == nullptr)
    return -3;
  return as_cache(cache)->lookup_exact(tokens, n_tokens, pages_out, pages_cap, num_tokens_out, first_token_out);
}

int64_t b200kv_prefix_cache_lookup_blocks(void* cache, const int64_t* tokens, int64_t n_tokens, int64_t* pages_out,
                                          int64_t pages_cap, int64_t* matched_tokens_out) {
  if (cache == nullptr || n_tokens < 0 || (n_tokens > 0 && tokens == nullptr) || pages_cap < 0 ||
      (pages_cap > 0 && pages_out == nullptr) || matched_tokens_out == nullptr)
    return -3;
  return as_cache(cache)->lookup_blocks(tokens, n_tokens, pages_out, pages_cap, matched_tokens_out);
}

int64_t b200kv_prefix_cache_store(void* cache, const int64_t* tokens, int64_t n_tokens, const int64_t* pages,
                                  int64_t n_pages, int64_t num_tokens, int64_t first_token) {
  if (cache == nullptr || n_tokens < 0 || n_pages < 0 || (n_tokens > 0 && tokens == nullptr) ||
      (n_pages > 0 && pages == nullptr))
    return -3;
  return as_cache(cache)->store(tokens, n_tokens, pages, n_pages, num_tokens, first_token);
}

int64_t b200kv_prefix_cache_ref_ops(const void* cache, int64_t* pages_out, int32_t* delta_out, int64_t cap) {
  if (cache == nullptr) return -3;
  const auto& ops = static_cast<const PrefixCache*>(cache)->ops();
  const int64_t n = static_cast<int64_t>(ops.size());
  if (n > cap || (n > 0 && (pages_out == nullptr || delta_out == nullptr))) return -2;
  for (int64_t i = 0; i < n; ++i) {
    pages_out[i] = ops[i].page;
    delta_out[i] = ops[i].delta;
  }
  return n;
}

int64_t b200kv_prefix_cache_clear(void* cache) {
  if (cache == nullptr) return -3;
  return as_cache(cache)->clear();
}

}  // extern "C"
