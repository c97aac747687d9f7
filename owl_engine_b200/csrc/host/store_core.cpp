// Host-side core of the KV store: content-addressed block chains, the prefix tree with
// leaf-LRU eviction, page reference counts and carriers (device / host / disk).
//
// A block is `block_tokens` consecutive tokens; its identity is hash(parent_hash, tokens, tag), so
// equal prefixes of different requests map to the same chain. The tree holds one reference on a
// page it indexes; sequences that use a page hold their own references. A node can only be
// evicted (or demoted to a slower carrier) when it is a leaf among device-resident nodes and no
// sequence references its page. This file is pure bookkeeping: it never touches device memory;
// the engine executes the moves it plans at step boundaries.
//
// Reference counterpart: crates/store/src/kv/{mod,tree,chain,slot}.rs, leg.rs (carriers), id.rs.
#include <cstdint>
#include <cstring>
#include <cmath>
#include <list>
#include <unordered_map>
#include <vector>

#define API extern "C" __attribute__((visibility("default")))

namespace {

inline uint64_t mix(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

enum Carrier : int8_t { DEVICE = 0, HOST = 1, DISK = 2 };

struct Node {
  uint64_t hash, parent;
  int32_t page;        // device page (carrier DEVICE), host slot (HOST) or -1 (DISK)
  int8_t carrier;
  uint64_t tag;        // e.g. image fingerprint, 0 for text
  uint64_t last_use;
  int32_t children;    // children of any carrier
  int32_t dev_children;// children that are device resident
  std::list<uint64_t>::iterator lru_it;
  bool in_lru;
  double crf;          // LRFU: combined recency / frequency value at crf_tick (every use adds 1, age halves it every 1/lambda ticks)
  uint64_t crf_tick;
};

struct Store {
  int n_pages, block_tokens;
  std::vector<int32_t> free_pages;
  std::vector<int32_t> refs;          // per device page
  std::unordered_map<uint64_t, Node> nodes;
  std::list<uint64_t> lru;            // device-resident evictable candidates, front = oldest
  uint64_t tick = 0;
  uint64_t hits = 0, lookups = 0, evictions = 0, published = 0;
  double lambda = -1.0;               // < 0: plain LRU order of the candidate list; >= 0: LRFU with this decay

  // LRFU order without a clock: value(now) = crf * 2^(-lambda (now - crf_tick)), so log2(crf) + lambda * crf_tick orders
  // the candidates the same way at every `now`.
  double lrfu_key(const Node& n) const { return std::log2(n.crf > 0 ? n.crf : 1e-300) + lambda * (double)n.crf_tick; }

  void touch(Node& n) {
    n.last_use = ++tick;
    n.crf = 1.0 + n.crf * std::exp2(-(lambda >= 0 ? lambda : 0.05) * (double)(tick - n.crf_tick));
    n.crf_tick = tick;
    if (n.in_lru) { lru.erase(n.lru_it); n.in_lru = false; }
    maybe_enlist(n);
  }
  // a device node is an eviction candidate when it has no device-resident children
  void maybe_enlist(Node& n) {
    if (n.carrier == DEVICE && n.dev_children == 0 && !n.in_lru) {
      lru.push_back(n.hash);
      n.lru_it = std::prev(lru.end());
      n.in_lru = true;
    }
  }
  void delist(Node& n) {
    if (n.in_lru) { lru.erase(n.lru_it); n.in_lru = false; }
  }
};

}  // namespace

// Victim order of owl_kv_evict: lambda < 0 = least recently used leaf first; lambda >= 0 = LRFU (0 = pure frequency,
// large = recency only).
API void owl_kv_set_policy(void* h, double lambda) { static_cast<Store*>(h)->lambda = lambda; }

API void* owl_kv_new(int n_pages, int block_tokens) {
  Store* s = new Store();
  s->n_pages = n_pages;
  s->block_tokens = block_tokens;
  s->refs.assign(n_pages, 0);
  for (int i = n_pages - 1; i >= 0; --i) s->free_pages.push_back(i);
  return s;
}
API void owl_kv_free(void* h) { delete static_cast<Store*>(h); }

API uint64_t owl_kv_hash(uint64_t parent, const int32_t* toks, int n, uint64_t tag) {
  uint64_t hsh = mix(parent ^ 0x9E3779B97F4A7C15ull) ^ mix(tag + 0x51ED270B7F4A7C15ull);
  for (int i = 0; i < n; ++i) hsh = mix(hsh ^ ((uint64_t)(uint32_t)toks[i] + 0x9E3779B97F4A7C15ull + ((uint64_t)i << 32)));
  return hsh ? hsh : 1;   // 0 is reserved for "no parent"
}

// Hashes of the consecutive full blocks of a token sequence; returns the number of blocks.
API int owl_kv_chain(const int32_t* toks, int n_tokens, int block_tokens, uint64_t root, const uint64_t* tags,
                     uint64_t* out) {
  const int nb = n_tokens / block_tokens;
  uint64_t parent = root;
  for (int b = 0; b < nb; ++b) {
    parent = owl_kv_hash(parent, toks + (size_t)b * block_tokens, block_tokens, tags ? tags[b] : 0);
    out[b] = parent;
  }
  return nb;
}

API int owl_kv_free_pages(void* h) { return (int)static_cast<Store*>(h)->free_pages.size(); }

// Allocate n device pages with one reference each (all or nothing). Returns n or 0.
API int owl_kv_alloc(void* h, int n, int32_t* out) {
  Store* s = static_cast<Store*>(h);
  if ((int)s->free_pages.size() < n) return 0;
  for (int i = 0; i < n; ++i) {
    out[i] = s->free_pages.back();
    s->free_pages.pop_back();
    s->refs[out[i]] = 1;
  }
  return n;
}
API void owl_kv_ref(void* h, const int32_t* pages, int n) {
  Store* s = static_cast<Store*>(h);
  for (int i = 0; i < n; ++i) s->refs[pages[i]]++;
}
API void owl_kv_unref(void* h, const int32_t* pages, int n) {
  Store* s = static_cast<Store*>(h);
  for (int i = 0; i < n; ++i) {
    if (--s->refs[pages[i]] == 0) s->free_pages.push_back(pages[i]);
  }
}
API int owl_kv_refcount(void* h, int page) { return static_cast<Store*>(h)->refs[page]; }

// Longest prefix of `hashes` present in the tree. pages_out / carrier_out describe each matched
// block; device-resident matches get one extra page reference (the caller now uses them).
API int owl_kv_match(void* h, const uint64_t* hashes, int n, int32_t* pages_out, int8_t* carrier_out) {
  Store* s = static_cast<Store*>(h);
  s->lookups++;
  int m = 0;
  for (; m < n; ++m) {
    auto it = s->nodes.find(hashes[m]);
    if (it == s->nodes.end()) break;
    Node& nd = it->second;
    pages_out[m] = nd.page;
    carrier_out[m] = nd.carrier;
    if (nd.carrier == DEVICE) s->refs[nd.page]++;
    s->touch(nd);
  }
  if (m) s->hits++;
  return m;
}

// Register blocks (already written on the device) in the tree; the tree takes its own reference.
// Blocks whose hash is already present are skipped (their page is not adopted). Returns the
// number of newly indexed blocks.
API int owl_kv_publish(void* h, const uint64_t* hashes, const int32_t* pages, int n, uint64_t root,
                       const uint64_t* tags) {
  Store* s = static_cast<Store*>(h);
  int added = 0;
  uint64_t parent = root;
  for (int i = 0; i < n; ++i) {
    auto it = s->nodes.find(hashes[i]);
    if (it == s->nodes.end()) {
      Node nd{};
      nd.hash = hashes[i]; nd.parent = parent; nd.page = pages[i]; nd.carrier = DEVICE;
      nd.tag = tags ? tags[i] : 0; nd.children = 0; nd.dev_children = 0; nd.in_lru = false;
      s->refs[pages[i]]++;
      auto ins = s->nodes.emplace(hashes[i], nd).first;
      auto pit = s->nodes.find(parent);
      if (pit != s->nodes.end()) {
        pit->second.children++;
        pit->second.dev_children++;
        s->delist(pit->second);
      }
      s->touch(ins->second);
      ++added;
      s->published++;
    } else {
      s->touch(it->second);
    }
    parent = hashes[i];
  }
  return added;
}

// Pick up to `max` victims (oldest evictable device leaves whose page only the tree references)
// until `need` pages would be free. `mode`: 0 = drop (node removed), 1 = demote (node stays with
// carrier HOST and page = -1 until owl_kv_set_carrier assigns its host slot). The tree's page
// reference is released in both modes. Returns the number of victims.
API int owl_kv_evict(void* h, int need, int mode, int32_t* pages_out, uint64_t* hashes_out, int max) {
  Store* s = static_cast<Store*>(h);
  int got = 0;
  auto it = s->lru.begin();
  while (it != s->lru.end() && got < max && (int)s->free_pages.size() < need) {
    if (s->lambda >= 0) {
      // LRFU: the candidate of least combined value (a block hit often stays although it was not hit last)
      auto best = s->lru.end();
      double best_key = 0;
      for (auto c = s->lru.begin(); c != s->lru.end(); ++c) {
        const Node& cn = s->nodes.find(*c)->second;
        if (s->refs[cn.page] > 1) continue;
        const double k = s->lrfu_key(cn);
        if (best == s->lru.end() || k < best_key) { best = c; best_key = k; }
      }
      if (best == s->lru.end()) break;
      it = best;
    }
    auto nit = s->nodes.find(*it);
    Node& nd = nit->second;
    if (s->refs[nd.page] > 1) { ++it; continue; }   // in use by a sequence
    pages_out[got] = nd.page;
    hashes_out[got] = nd.hash;
    ++got;
    it = s->lru.erase(it);
    nd.in_lru = false;
    const int32_t page = nd.page;
    auto pit = s->nodes.find(nd.parent);
    if (pit != s->nodes.end()) {
      pit->second.dev_children--;
      if (mode == 0) pit->second.children--;
      s->maybe_enlist(pit->second);
    }
    if (mode == 0 && nd.children == 0) {
      s->nodes.erase(nit);
    } else {
      nd.carrier = HOST;   // also the fate of an interior node dropped from the device
      nd.page = -1;
    }
    if (--s->refs[page] == 0) s->free_pages.push_back(page);
    s->evictions++;
    it = s->lru.begin();   // the parent may have become a candidate: rescan (pinned entries are skipped again)
  }
  return got;
}

// Move a node between carriers (after the engine executed the copy). For carrier DEVICE `slot` is
// a device page the caller allocated (the tree adopts one reference).
API int owl_kv_set_carrier(void* h, uint64_t hash, int carrier, int slot) {
  Store* s = static_cast<Store*>(h);
  auto it = s->nodes.find(hash);
  if (it == s->nodes.end()) return -1;
  Node& nd = it->second;
  const bool was_dev = nd.carrier == DEVICE;
  nd.carrier = (int8_t)carrier;
  nd.page = slot;
  if (carrier == DEVICE && !was_dev) {
    s->refs[slot]++;
    auto pit = s->nodes.find(nd.parent);
    if (pit != s->nodes.end()) { pit->second.dev_children++; s->delist(pit->second); }
    s->touch(nd);
  }
  return 0;
}

// Insert a node that lives below the device (restart adoption of the disk tier's index, or a block written by another
// process): carrier HOST with its slot, or DISK. Parents must be adopted before their children for the child counts to
// be right; a node whose parent is unknown is still inserted (it can only be reached through a chain that matches the
// parent first, so it stays unreachable until the parent arrives). Returns 1 when inserted, 0 when the hash was known.
API int owl_kv_adopt(void* h, uint64_t hash, uint64_t parent, int carrier, int slot, uint64_t tag) {
  Store* s = static_cast<Store*>(h);
  if (carrier == DEVICE || hash == 0 || s->nodes.count(hash)) return 0;
  Node nd{};
  nd.hash = hash; nd.parent = parent; nd.page = slot; nd.carrier = (int8_t)carrier; nd.tag = tag;
  nd.children = 0; nd.dev_children = 0; nd.in_lru = false; nd.last_use = ++s->tick;
  s->nodes.emplace(hash, nd);
  auto pit = s->nodes.find(parent);
  if (pit != s->nodes.end()) pit->second.children++;
  return 1;
}

// Remove a non-device node for good (tier overflow). Fails (-1) when it still has children.
API int owl_kv_forget(void* h, uint64_t hash) {
  Store* s = static_cast<Store*>(h);
  auto it = s->nodes.find(hash);
  if (it == s->nodes.end() || it->second.carrier == DEVICE || it->second.children > 0) return -1;
  auto pit = s->nodes.find(it->second.parent);
  if (pit != s->nodes.end()) pit->second.children--;
  s->nodes.erase(it);
  return 0;
}

API int owl_kv_node(void* h, uint64_t hash, int32_t* page, int8_t* carrier, uint64_t* tag, uint64_t* parent) {
  Store* s = static_cast<Store*>(h);
  auto it = s->nodes.find(hash);
  if (it == s->nodes.end()) return -1;
  *page = it->second.page; *carrier = it->second.carrier; *tag = it->second.tag; *parent = it->second.parent;
  return 0;
}

// stats: [nodes, device_nodes, free_pages, lookups, hits, evictions, published, lru_len]
API void owl_kv_stats(void* h, uint64_t* out) {
  Store* s = static_cast<Store*>(h);
  uint64_t dev = 0;
  for (auto& kv : s->nodes) dev += kv.second.carrier == DEVICE;
  out[0] = s->nodes.size(); out[1] = dev; out[2] = s->free_pages.size(); out[3] = s->lookups; out[4] = s->hits;
  out[5] = s->evictions; out[6] = s->published; out[7] = s->lru.size();
}

// All node hashes of a carrier (for dumps / restart index). Returns the count written.
API int owl_kv_list(void* h, int carrier, uint64_t* out, int max) {
  Store* s = static_cast<Store*>(h);
  int n = 0;
  for (auto& kv : s->nodes)
    if (carrier < 0 || kv.second.carrier == carrier) {
      if (n < max) out[n] = kv.first;
      ++n;
    }
  return n;
}
