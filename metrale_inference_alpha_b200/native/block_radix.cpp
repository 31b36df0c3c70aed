// Host runtime, part 1: KV block allocator (free list + per-block reference counts, block 0
// reserved as the null block) and the radix prefix index over whole blocks of token ids with
// per-adapter roots, LRU leaf eviction and optional recurrent-state snapshot ids.
//
// Same contract as the Python classes in cache/block_pool.py and cache/radix.py (which remain the
// behavioural oracle in the differential tests); this is the serving-path implementation: an
// admission pass over a few hundred waiting requests walks the tree for every prompt, which is
// pointer chasing that does not belong in an interpreter. Role of the reference's
// crates/cache/src/{paged_kv_cache.rs,radix_tree/*.rs}.
//
// C ABI, no exceptions across the boundary: every function returns a count or a negative error.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <unordered_map>
#include <vector>

namespace {

struct Allocator {
  std::vector<int32_t> refcount;
  std::vector<int32_t> free_list;
  explicit Allocator(int32_t n) : refcount(n, 0) {
    refcount[0] = 1 << 30;
    for (int32_t b = n - 1; b >= 1; --b) free_list.push_back(b);
  }
};

// FNV-1a over one block of token ids: the child key. Collisions are resolved by comparing the ids.
inline uint64_t hash_chunk(const int32_t* t, int n) {
  uint64_t h = 1469598103934665603ull;
  for (int i = 0; i < n; ++i) {
    h ^= static_cast<uint32_t>(t[i]);
    h *= 1099511628211ull;
  }
  return h;
}

struct Node {
  std::vector<int32_t> key;
  int32_t block = 0;
  Node* parent = nullptr;
  int64_t last_use = 0;
  int64_t snapshot = -1;
  std::unordered_multimap<uint64_t, std::unique_ptr<Node>> children;
};

struct Radix {
  Allocator* alloc;
  int32_t block_size;
  bool needs_snapshot;
  int64_t clock = 0;
  int64_t num_nodes = 0, hits = 0, queries = 0, hit_tokens = 0;
  std::map<int64_t, std::unique_ptr<Node>> roots;   // adapter id -> root
  std::vector<int64_t> evicted_snapshots;            // drained by the caller after evict()

  Node* root(int64_t adapter) {
    auto it = roots.find(adapter);
    if (it == roots.end()) it = roots.emplace(adapter, std::make_unique<Node>()).first;
    return it->second.get();
  }
  Node* child(Node* n, const int32_t* chunk) const {
    auto range = n->children.equal_range(hash_chunk(chunk, block_size));
    for (auto it = range.first; it != range.second; ++it)
      if (std::memcmp(it->second->key.data(), chunk, sizeof(int32_t) * block_size) == 0) return it->second.get();
    return nullptr;
  }
  void collect_leaves(Node* n, std::vector<Node*>& out) const {
    for (auto& kv : n->children) {
      Node* c = kv.second.get();
      if (c->children.empty()) out.push_back(c);
      else collect_leaves(c, out);
    }
  }
  void remove(Node* leaf) {
    Node* p = leaf->parent;
    auto range = p->children.equal_range(hash_chunk(leaf->key.data(), block_size));
    for (auto it = range.first; it != range.second; ++it)
      if (it->second.get() == leaf) { p->children.erase(it); break; }
    --num_nodes;
  }
};

int32_t release(Allocator* a, const int32_t* blocks, int32_t n, int32_t* released) {
  int32_t r = 0;
  for (int32_t i = 0; i < n; ++i) {
    int32_t b = blocks[i];
    if (b == 0) continue;
    if (b < 0 || b >= static_cast<int32_t>(a->refcount.size()) || a->refcount[b] <= 0) return -2;
    if (--a->refcount[b] == 0) {
      a->free_list.push_back(b);
      if (released) released[r] = b;
      ++r;
    }
  }
  return r;
}

}  // namespace

extern "C" {

// ---------------------------------------------------------------- allocator
void* mrt_alloc_create(int32_t num_blocks) { return num_blocks >= 2 ? new Allocator(num_blocks) : nullptr; }
void mrt_alloc_destroy(void* h) { delete static_cast<Allocator*>(h); }
int32_t mrt_alloc_num_free(void* h) { return static_cast<int32_t>(static_cast<Allocator*>(h)->free_list.size()); }
int32_t mrt_alloc_refcount(void* h, int32_t b) { return static_cast<Allocator*>(h)->refcount[b]; }

// returns n, or -1 when fewer than n blocks are free (nothing is taken)
int32_t mrt_alloc_take(void* h, int32_t n, int32_t* out) {
  auto* a = static_cast<Allocator*>(h);
  if (n > static_cast<int32_t>(a->free_list.size())) return -1;
  for (int32_t i = 0; i < n; ++i) {
    out[i] = a->free_list.back();
    a->free_list.pop_back();
    a->refcount[out[i]] = 1;
  }
  return n;
}

// returns 0, or -2 when a block is free (reference on a block nobody owns)
int32_t mrt_alloc_incref(void* h, const int32_t* blocks, int32_t n) {
  auto* a = static_cast<Allocator*>(h);
  for (int32_t i = 0; i < n; ++i)
    if (blocks[i] < 0 || blocks[i] >= static_cast<int32_t>(a->refcount.size()) || a->refcount[blocks[i]] <= 0) return -2;
  for (int32_t i = 0; i < n; ++i) ++a->refcount[blocks[i]];
  return 0;
}

// drops one reference per block; writes the blocks that became free; returns their count or -2 (double free)
int32_t mrt_alloc_release(void* h, const int32_t* blocks, int32_t n, int32_t* released) {
  return release(static_cast<Allocator*>(h), blocks, n, released);
}

// ---------------------------------------------------------------- radix index
void* mrt_radix_create(void* alloc, int32_t block_size, int32_t needs_snapshot) {
  auto* r = new Radix();
  r->alloc = static_cast<Allocator*>(alloc);
  r->block_size = block_size;
  r->needs_snapshot = needs_snapshot != 0;
  return r;
}
void mrt_radix_destroy(void* h) { delete static_cast<Radix*>(h); }

// Longest cached prefix in whole blocks, never the whole prompt (limit = min(max_tokens, n-1)).
// Takes a reference on every returned block. Returns the number of blocks; *snapshot = id or -1.
int32_t mrt_radix_match(void* h, const int32_t* tokens, int32_t n, int64_t adapter, int32_t max_tokens,
                        int32_t* out_blocks, int64_t* snapshot) {
  auto* r = static_cast<Radix*>(h);
  ++r->queries;
  const int32_t bs = r->block_size;
  int32_t limit = n - 1;
  if (max_tokens >= 0 && max_tokens < limit) limit = max_tokens;
  std::vector<Node*> path;
  Node* node = r->root(adapter);
  for (int32_t i = 0; i + bs <= n; i += bs) {
    if (static_cast<int32_t>(path.size() + 1) * bs > limit) break;
    Node* nxt = r->child(node, tokens + i);
    if (!nxt) break;
    path.push_back(nxt);
    node = nxt;
  }
  *snapshot = -1;
  if (r->needs_snapshot) {
    while (!path.empty() && path.back()->snapshot < 0) path.pop_back();
    if (!path.empty()) *snapshot = path.back()->snapshot;
  }
  const int64_t now = ++r->clock;
  int32_t k = 0;
  for (Node* p : path) {
    p->last_use = now;
    out_blocks[k++] = p->block;
    ++r->alloc->refcount[p->block];
  }
  if (k) {
    ++r->hits;
    r->hit_tokens += static_cast<int64_t>(k) * bs;
  }
  return k;
}

// Publish the full blocks of a sequence; snapshots are (token_count, id) pairs. Returns adopted blocks.
int32_t mrt_radix_insert(void* h, const int32_t* tokens, int32_t n, const int32_t* blocks, int32_t nblocks,
                         int64_t adapter, const int64_t* snap_pos, const int64_t* snap_id, int32_t nsnap) {
  auto* r = static_cast<Radix*>(h);
  const int32_t bs = r->block_size;
  Node* node = r->root(adapter);
  const int64_t now = ++r->clock;
  int32_t adopted = 0;
  for (int32_t i = 0, c = 0; i + bs <= n && c < nblocks; i += bs, ++c) {
    Node* nxt = r->child(node, tokens + i);
    if (!nxt) {
      auto nn = std::make_unique<Node>();
      nn->key.assign(tokens + i, tokens + i + bs);
      nn->block = blocks[c];
      nn->parent = node;
      nxt = nn.get();
      node->children.emplace(hash_chunk(tokens + i, bs), std::move(nn));
      ++r->alloc->refcount[blocks[c]];
      ++r->num_nodes;
      ++adopted;
    }
    nxt->last_use = now;
    for (int32_t s = 0; s < nsnap; ++s)
      if (snap_pos[s] == static_cast<int64_t>(c + 1) * bs && nxt->snapshot < 0) nxt->snapshot = snap_id[s];
    node = nxt;
  }
  return adopted;
}

// Evict leaves that only the tree references, least recently used first, until `want` blocks went
// back to the allocator. One pass takes the current leaves in LRU order; parents exposed by the
// pass are considered in the next one.
int32_t mrt_radix_evict(void* h, int32_t want) {
  auto* r = static_cast<Radix*>(h);
  int32_t freed = 0;
  while (freed < want) {
    std::vector<Node*> leaves, cands;
    for (auto& kv : r->roots) r->collect_leaves(kv.second.get(), leaves);
    for (Node* l : leaves)
      if (r->alloc->refcount[l->block] == 1) cands.push_back(l);
    if (cands.empty()) break;
    std::stable_sort(cands.begin(), cands.end(), [](const Node* a, const Node* b) { return a->last_use < b->last_use; });
    for (Node* n : cands) {
      if (freed >= want) break;
      if (n->snapshot >= 0) r->evicted_snapshots.push_back(n->snapshot);
      int32_t b = n->block;
      freed += release(r->alloc, &b, 1, nullptr);
      r->remove(n);
    }
  }
  return freed;
}

// blocks that only the tree holds
int32_t mrt_radix_evictable(void* h) {
  auto* r = static_cast<Radix*>(h);
  struct Rec {
    static void walk(const Radix* r, const Node* n, int32_t& count) {
      for (auto& kv : n->children) {
        if (r->alloc->refcount[kv.second->block] == 1) ++count;
        walk(r, kv.second.get(), count);
      }
    }
  };
  int32_t count = 0;
  for (auto& kv : r->roots) Rec::walk(r, kv.second.get(), count);
  return count;
}

int32_t mrt_radix_drain_evicted_snapshots(void* h, int64_t* out, int32_t cap) {
  auto* r = static_cast<Radix*>(h);
  int32_t n = 0;
  while (n < cap && !r->evicted_snapshots.empty()) {
    out[n++] = r->evicted_snapshots.back();
    r->evicted_snapshots.pop_back();
  }
  return n;
}

// stats[0..4] = nodes, queries, hits, hit_tokens, clock
void mrt_radix_stats(void* h, int64_t* stats) {
  auto* r = static_cast<Radix*>(h);
  stats[0] = r->num_nodes; stats[1] = r->queries; stats[2] = r->hits; stats[3] = r->hit_tokens; stats[4] = r->clock;
}

void mrt_radix_clear(void* h) {
  auto* r = static_cast<Radix*>(h);
  struct Rec {
    static void drop(Radix* r, Node* n) {
      for (auto& kv : n->children) {
        Node* c = kv.second.get();
        drop(r, c);
        int32_t b = c->block;
        release(r->alloc, &b, 1, nullptr);
        if (c->snapshot >= 0) r->evicted_snapshots.push_back(c->snapshot);
      }
      n->children.clear();
    }
  };
  for (auto& kv : r->roots) Rec::drop(r, kv.second.get());
  r->num_nodes = 0;
}

}  // extern "C"
