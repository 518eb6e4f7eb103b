// Greedy longest-match byte tokenizer over the RWKV vocabulary: the host-side native counterpart of the Python
// trie in data/tokenizers/rwkv_tokenizer.py (the reference's tokenizer, rwkvtune/data/tokenizers/rwkv_tokenizer.py:5-47
// and :111-120, walks a tree of Python objects byte by byte).  Host code only: no kernel is launched from this file.
//
// Layout: the root has a direct 256-entry child table; every other edge (node, byte) -> child lives in one
// open-addressing hash table keyed by node * 256 + byte, so inserting a token later (special tokens are added at
// run time) costs no rebuild.  Encoding walks the longest match from each position: one table probe per byte.
// rwkv_trie_encode_batch splits a list of texts over std::threads; every text is independent.
#include <atomic>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#define RWKV_API extern "C" __attribute__((visibility("default")))

namespace {

struct Trie {
  std::vector<int32_t> value;          // token id that ends at this node, or -1
  int32_t root_child[256];
  std::vector<uint64_t> keys;          // node * 256 + byte, or EMPTY
  std::vector<int32_t> vals;           // child node
  size_t used = 0;
  static constexpr uint64_t EMPTY = ~0ull;

  Trie() : value(1, -1), keys(1u << 16, EMPTY), vals(1u << 16, 0) {
    for (int i = 0; i < 256; ++i) root_child[i] = -1;
  }

  static size_t hash(uint64_t k) {
    k ^= k >> 33;
    k *= 0xff51afd7ed558ccdull;
    k ^= k >> 33;
    return (size_t)k;
  }

  void grow() {
    std::vector<uint64_t> old_keys(keys.size() * 2, EMPTY);
    std::vector<int32_t> old_vals(vals.size() * 2, 0);
    old_keys.swap(keys);
    old_vals.swap(vals);
    const size_t mask = keys.size() - 1;
    for (size_t i = 0; i < old_keys.size(); ++i) {
      if (old_keys[i] == EMPTY) continue;
      size_t h = hash(old_keys[i]) & mask;
      while (keys[h] != EMPTY) h = (h + 1) & mask;
      keys[h] = old_keys[i];
      vals[h] = old_vals[i];
    }
  }

  inline int32_t child(int32_t node, uint8_t b) const {
    if (node == 0) return root_child[b];
    const uint64_t k = (uint64_t)node * 256 + b;
    const size_t mask = keys.size() - 1;
    size_t h = hash(k) & mask;
    while (true) {
      const uint64_t cur = keys[h];
      if (cur == k) return vals[h];
      if (cur == EMPTY) return -1;
      h = (h + 1) & mask;
    }
  }

  int32_t add_child(int32_t node, uint8_t b) {
    const int32_t fresh = (int32_t)value.size();
    value.push_back(-1);
    if (node == 0) {
      root_child[b] = fresh;
      return fresh;
    }
    if ((used + 1) * 2 > keys.size()) grow();
    const uint64_t k = (uint64_t)node * 256 + b;
    const size_t mask = keys.size() - 1;
    size_t h = hash(k) & mask;
    while (keys[h] != EMPTY) h = (h + 1) & mask;
    keys[h] = k;
    vals[h] = fresh;
    ++used;
    return fresh;
  }

  void insert(const uint8_t* tok, int len, int32_t id) {
    int32_t node = 0;
    for (int i = 0; i < len; ++i) {
      int32_t c = child(node, tok[i]);
      if (c < 0) c = add_child(node, tok[i]);
      node = c;
    }
    value[node] = id;
  }

  // Returns the number of ids written, or -1 - offset of the first byte that no token covers.
  int64_t encode(const uint8_t* src, int64_t n, int32_t* out) const {
    int64_t i = 0, count = 0;
    while (i < n) {
      int32_t node = 0, best = -1;
      int64_t j = i, best_end = i;
      while (j < n) {
        node = child(node, src[j]);
        if (node < 0) break;
        ++j;
        const int32_t v = value[node];
        if (v >= 0) {
          best = v;
          best_end = j;
        }
      }
      if (best < 0) return -1 - i;
      out[count++] = best;
      i = best_end;
    }
    return count;
  }
};

}  // namespace

RWKV_API void* rwkv_trie_create() { return new Trie(); }

RWKV_API void rwkv_trie_destroy(void* handle) { delete static_cast<Trie*>(handle); }

RWKV_API int rwkv_trie_insert(void* handle, const uint8_t* tok, int len, int id) {
  if (handle == nullptr || tok == nullptr || len <= 0 || id < 0) return 1;
  static_cast<Trie*>(handle)->insert(tok, len, id);
  return 0;
}

// Bulk insert: `blob` holds the tokens back to back, token t spans [offsets[t], offsets[t + 1]).
RWKV_API int rwkv_trie_insert_many(void* handle, const uint8_t* blob, const int64_t* offsets, const int32_t* ids, int count) {
  if (handle == nullptr || blob == nullptr || offsets == nullptr || ids == nullptr || count < 0) return 1;
  Trie* t = static_cast<Trie*>(handle);
  for (int i = 0; i < count; ++i) {
    const int64_t len = offsets[i + 1] - offsets[i];
    if (len <= 0 || ids[i] < 0) return 1;
    t->insert(blob + offsets[i], (int)len, ids[i]);
  }
  return 0;
}

RWKV_API int64_t rwkv_trie_nodes(void* handle) { return handle ? (int64_t)static_cast<Trie*>(handle)->value.size() : 0; }

// `out` needs room for n ids (a token covers at least one byte).
RWKV_API int64_t rwkv_trie_encode(void* handle, const uint8_t* src, int64_t n, int32_t* out) {
  if (handle == nullptr || (n > 0 && (src == nullptr || out == nullptr))) return INT64_MIN;
  return static_cast<const Trie*>(handle)->encode(src, n, out);
}

// Text t spans blob[offsets[t], offsets[t + 1]); its ids go to out + offsets[t] (same offsets: at most one id per
// byte) and counts[t] receives their number, or -1 - offset of the uncovered byte inside that text.
RWKV_API int rwkv_trie_encode_batch(void* handle, const uint8_t* blob, const int64_t* offsets, int n_texts, int32_t* out,
                                    int64_t* counts, int n_threads) {
  if (handle == nullptr || offsets == nullptr || counts == nullptr || n_texts < 0) return 1;
  const Trie* t = static_cast<const Trie*>(handle);
  if (n_threads < 1) n_threads = 1;
  if (n_threads > n_texts) n_threads = n_texts > 0 ? n_texts : 1;
  std::atomic<int> next{0};
  auto work = [&]() {
    while (true) {
      const int i = next.fetch_add(1);
      if (i >= n_texts) break;
      counts[i] = t->encode(blob + offsets[i], offsets[i + 1] - offsets[i], out + offsets[i]);
    }
  };
  if (n_threads == 1) {
    work();
    return 0;
  }
  std::vector<std::thread> pool;
  pool.reserve(n_threads);
  for (int k = 0; k < n_threads; ++k) pool.emplace_back(work);
  for (auto& th : pool) th.join();
  return 0;
}
