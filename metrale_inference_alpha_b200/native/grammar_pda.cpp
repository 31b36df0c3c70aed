// Host runtime, part 4: pushdown matcher for compiled grammars (EBNF / regex / JSON Schema /
// structural tags, compiled in Python to per-rule NFAs whose edges are byte ranges, rule
// references and epsilons) and its whole-vocabulary token mask.
//
// State = a sorted set of items (node, frame); a frame is an interned (return node, parent) pair,
// so ambiguous parses share stack tails. A call whose return node can only end the caller reuses
// the caller's frame (tail call), which keeps right-recursive automata at constant depth.
//
// Mask fill walks the vocabulary in byte-lexicographic order with a stack of states, one per
// prefix length: a token re-uses the states of the prefix it shares with its predecessor, and
// when a byte is refused every following token with that prefix is skipped without being walked.
// Masks are memoised per state (item set incl. frame identities), which is what repeats inside
// strings, numbers and free text. Role of the reference's crates/grammar matcher + bitmask fill.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <unordered_map>
#include <vector>

#include "vocab.h"

namespace {

enum : int32_t { E_EPS = 0, E_BYTES = 1, E_RULE = 2 };

struct Grammar {
  std::vector<int32_t> edge_begin, kind, a, b, to, fin, rule_start;
  int32_t root = 0;
};

using Item = uint64_t;                     // node << 32 | (frame + 1)
inline Item mk(int32_t node, int32_t frame) { return (uint64_t(uint32_t(node)) << 32) | uint32_t(frame + 1); }
inline int32_t node_of(Item it) { return int32_t(it >> 32); }
inline int32_t frame_of(Item it) { return int32_t(uint32_t(it)) - 1; }

struct Frame { int32_t ret, parent; };

struct VecHash {
  size_t operator()(const std::vector<Item>& v) const {
    uint64_t h = 1469598103934665603ull;
    for (Item x : v) { h ^= x; h *= 1099511628211ull; h ^= h >> 29; }
    return size_t(h);
  }
};

struct Pda {
  const Grammar* g = nullptr;
  std::vector<Frame> frames;
  std::unordered_map<uint64_t, int32_t> intern;
  std::vector<Item> items;
  std::vector<std::vector<Item>> history;
  std::unordered_map<std::vector<Item>, std::vector<uint8_t>, VecHash> mask_cache;
  const MrtVocab* cache_vocab = nullptr;
  int32_t cache_eos = -2, cache_len = -1;
  int64_t cache_hits = 0, cache_misses = 0;
  // scratch
  std::vector<Item> todo;

  int32_t frame(int32_t ret, int32_t parent) {
    const uint64_t k = (uint64_t(uint32_t(ret)) << 32) | uint32_t(parent + 1);
    auto it = intern.find(k);
    if (it != intern.end()) return it->second;
    const int32_t f = int32_t(frames.size());
    frames.push_back({ret, parent});
    intern.emplace(k, f);
    return f;
  }

  // closes `seed` under epsilons, calls and returns; result sorted and unique
  void closure(std::vector<Item>& seed, std::vector<Item>& out) {
    out.clear();
    todo.assign(seed.begin(), seed.end());
    // small sets dominate: linear membership test, switching to sort + unique at the end
    while (!todo.empty()) {
      const Item it = todo.back();
      todo.pop_back();
      bool dup = false;
      if (out.size() <= 24) {
        for (Item x : out) if (x == it) { dup = true; break; }
      } else {
        dup = std::find(out.begin(), out.end(), it) != out.end();
      }
      if (dup) continue;
      out.push_back(it);
      const int32_t n = node_of(it), f = frame_of(it);
      for (int32_t e = g->edge_begin[n]; e < g->edge_begin[n + 1]; ++e) {
        const int32_t k = g->kind[e];
        if (k == E_EPS) {
          todo.push_back(mk(g->to[e], f));
        } else if (k == E_RULE) {
          const int32_t t = g->to[e];
          todo.push_back(mk(g->rule_start[g->a[e]], (g->fin[t] & 2) ? f : frame(t, f)));
        }
      }
      if ((g->fin[n] & 1) && f >= 0) todo.push_back(mk(frames[f].ret, frames[f].parent));
    }
    std::sort(out.begin(), out.end());
  }

  bool step(const std::vector<Item>& cur, uint8_t c, std::vector<Item>& scratch, std::vector<Item>& out) {
    scratch.clear();
    for (Item it : cur) {
      const int32_t n = node_of(it);
      for (int32_t e = g->edge_begin[n]; e < g->edge_begin[n + 1]; ++e)
        if (g->kind[e] == E_BYTES && g->a[e] <= c && c <= g->b[e])
          scratch.push_back(mk(g->to[e], frame_of(it)));
    }
    if (scratch.empty()) { out.clear(); return false; }
    closure(scratch, out);
    return true;
  }

  void reset() {
    frames.clear();
    intern.clear();
    history.clear();
    mask_cache.clear();
    std::vector<Item> seed{mk(g->rule_start[g->root], -1)};
    closure(seed, items);
  }

  bool complete() const {
    for (Item it : items)
      if (frame_of(it) < 0 && (g->fin[node_of(it)] & 1)) return true;
    return false;
  }

  // atomic: all bytes or nothing
  bool feed(const uint8_t* p, int64_t n) {
    std::vector<Item> cur = items, nxt, scratch;
    for (int64_t i = 0; i < n; ++i) {
      if (!step(cur, p[i], scratch, nxt)) return false;
      cur.swap(nxt);
    }
    items.swap(cur);
    return true;
  }
};

void sort_vocab(MrtVocab* v) {
  if (!v->sorted.empty() || v->n == 0) return;
  std::vector<int32_t> ids(v->n);
  std::iota(ids.begin(), ids.end(), 0);
  auto len = [&](int32_t t) { return v->offsets[t + 1] - v->offsets[t]; };
  std::sort(ids.begin(), ids.end(), [&](int32_t x, int32_t y) {
    const int64_t lx = len(x), ly = len(y);
    const int c = std::memcmp(v->bytes.data() + v->offsets[x], v->bytes.data() + v->offsets[y], size_t(std::min(lx, ly)));
    if (c != 0) return c < 0;
    if (lx != ly) return lx < ly;
    return x < y;
  });
  v->lcp.assign(v->n, 0);
  for (int32_t i = 1; i < v->n; ++i) {
    const int32_t x = ids[i - 1], y = ids[i];
    const int64_t m = std::min(len(x), len(y));
    const uint8_t* px = v->bytes.data() + v->offsets[x];
    const uint8_t* py = v->bytes.data() + v->offsets[y];
    int64_t k = 0;
    while (k < m && px[k] == py[k]) ++k;
    v->lcp[i] = int32_t(k);
  }
  v->sorted.swap(ids);
}

}  // namespace

extern "C" {

void* mrt_pda_grammar_create(int32_t n_nodes, const int32_t* edge_begin, int32_t n_edges, const int32_t* kind,
                             const int32_t* a, const int32_t* b, const int32_t* to, const int32_t* fin,
                             int32_t n_rules, const int32_t* rule_start, int32_t root) {
  if (n_nodes <= 0 || n_rules <= 0 || root < 0 || root >= n_rules || edge_begin[n_nodes] != n_edges) return nullptr;
  for (int32_t e = 0; e < n_edges; ++e) {
    if (to[e] < 0 || to[e] >= n_nodes) return nullptr;
    if (kind[e] == E_RULE && (a[e] < 0 || a[e] >= n_rules)) return nullptr;
  }
  for (int32_t r = 0; r < n_rules; ++r)
    if (rule_start[r] < 0 || rule_start[r] >= n_nodes) return nullptr;
  auto* g = new Grammar();
  g->edge_begin.assign(edge_begin, edge_begin + n_nodes + 1);
  g->kind.assign(kind, kind + n_edges);
  g->a.assign(a, a + n_edges);
  g->b.assign(b, b + n_edges);
  g->to.assign(to, to + n_edges);
  g->fin.assign(fin, fin + n_nodes);
  g->rule_start.assign(rule_start, rule_start + n_rules);
  g->root = root;
  return g;
}
void mrt_pda_grammar_destroy(void* g) { delete static_cast<Grammar*>(g); }

void* mrt_pda_create(void* grammar) {
  auto* p = new Pda();
  p->g = static_cast<const Grammar*>(grammar);
  p->reset();
  return p;
}
void mrt_pda_destroy(void* p) { delete static_cast<Pda*>(p); }
void mrt_pda_reset(void* p) { static_cast<Pda*>(p)->reset(); }
int32_t mrt_pda_complete(void* p) { return static_cast<Pda*>(p)->complete() ? 1 : 0; }
int32_t mrt_pda_feed(void* p, const uint8_t* bytes, int32_t n) { return static_cast<Pda*>(p)->feed(bytes, n) ? 1 : 0; }

// accepts one token and remembers the previous state for rollback; 0 = refused (state unchanged)
int32_t mrt_pda_advance(void* h, void* vocab, int32_t tok) {
  auto* p = static_cast<Pda*>(h);
  const auto* v = static_cast<const MrtVocab*>(vocab);
  if (tok < 0 || tok >= v->n) return 0;
  std::vector<Item> before = p->items;
  if (!p->feed(v->bytes.data() + v->offsets[tok], v->offsets[tok + 1] - v->offsets[tok])) return 0;
  p->history.push_back(std::move(before));
  return 1;
}

int32_t mrt_pda_rollback(void* h, int32_t n) {
  auto* p = static_cast<Pda*>(h);
  int32_t done = 0;
  while (done < n && !p->history.empty()) {
    p->items.swap(p->history.back());
    p->history.pop_back();
    ++done;
  }
  return done;
}

void mrt_pda_stats(void* h, int64_t* out4) {
  auto* p = static_cast<Pda*>(h);
  out4[0] = int64_t(p->items.size());
  out4[1] = int64_t(p->frames.size());
  out4[2] = p->cache_hits;
  out4[3] = p->cache_misses;
}

// mask[t] = 1 when token t may come next; eos (>= 0) is legal exactly when the grammar may end.
// Tokens without bytes are never legal. Returns the number of legal tokens.
int32_t mrt_pda_fill_mask(void* h, void* vocab, int32_t eos, uint8_t* mask, int32_t mask_len) {
  auto* p = static_cast<Pda*>(h);
  auto* v = static_cast<MrtVocab*>(vocab);
  sort_vocab(v);
  if (p->cache_vocab != v || p->cache_eos != eos || p->cache_len != mask_len) {
    p->mask_cache.clear();
    p->cache_vocab = v;
    p->cache_eos = eos;
    p->cache_len = mask_len;
  }
  auto hit = p->mask_cache.find(p->items);
  if (hit != p->mask_cache.end()) {
    ++p->cache_hits;
    std::memcpy(mask, hit->second.data(), size_t(mask_len));
    int32_t legal = 0;
    for (int32_t i = 0; i < mask_len; ++i) legal += mask[i];
    return legal;
  }
  ++p->cache_misses;
  std::memset(mask, 0, size_t(mask_len));
  int32_t legal = 0;
  std::vector<std::vector<Item>> st(1, p->items);      // st[d] = state after d bytes of the walked prefix
  std::vector<Item> scratch;
  int32_t valid = 0;                                    // st[0..valid] belong to a prefix of the current token
  bool dead = false;                                    // the byte after that prefix was refused
  for (int32_t i = 0; i < v->n; ++i) {
    const int32_t tok = v->sorted[i];
    const int64_t off = v->offsets[tok], len = v->offsets[tok + 1] - off;
    const int32_t share = v->lcp[i];
    if (dead && share > valid) continue;                // still under the refused prefix
    dead = false;
    valid = std::min(valid, share);
    if (len == 0 || tok == eos || tok >= mask_len) continue;
    int32_t d = valid;
    for (; d < len; ++d) {
      if (int32_t(st.size()) < d + 2) st.emplace_back();
      if (!p->step(st[d], v->bytes[off + d], scratch, st[d + 1])) {
        dead = true;
        break;
      }
    }
    valid = d;
    if (!dead) { mask[tok] = 1; ++legal; }
  }
  if (eos >= 0 && eos < mask_len && p->complete()) { mask[eos] = 1; ++legal; }
  if (p->mask_cache.size() >= 512) p->mask_cache.clear();
  p->mask_cache.emplace(p->items, std::vector<uint8_t>(mask, mask + mask_len));
  return legal;
}

}  // extern "C"
