// KV block allocation for the scheduler: a free list, and a radix trie over token ids that lets
// requests share the blocks of a common prompt prefix (prefix caching).
//
// Behaviour follows the reference's Rust allocator (backends/v3/src/block_allocator.rs:7-221,
// backends/v3/src/radix.rs:20-600): block 0 is reserved for the health-check request, an
// allocation covers `tokens` tokens with whole blocks, a prefix hit re-uses the trie's blocks and
// pins them (reference count) until the request is freed, freeing a request inserts the blocks of
// its prompt into the trie and returns the rest (decode blocks, and blocks that duplicate what a
// concurrent request inserted first) to the free list, and when the free list runs dry the least
// recently used unpinned leaves are evicted, partially if that suffices.
//
// The implementation is a plain pointer-free arena (`std::vector<Node>` + free slots) driven from
// the single scheduler thread; it needs no locking.
#pragma once
#include <algorithm>
#include <cstdint>
#include <map>
#include <optional>
#include <set>
#include <stdexcept>
#include <unordered_map>
#include <vector>

namespace sched {

struct BlockAllocation {
  uint64_t allocation_id = 0;
  std::vector<uint32_t> blocks;
  std::vector<uint32_t> slots;
  uint32_t prefix_len = 0;   // tokens whose KV is already in the cache
};

class RadixTrie {
 public:
  explicit RadixTrie(uint32_t block_size) : bs_(block_size) {
    nodes_.push_back(Node{});   // root
    nodes_[0].alive = true;
  }

  // Longest cached prefix of `key` in whole blocks: appends its blocks and returns the deepest node.
  int find(const std::vector<uint32_t>& key, std::vector<uint32_t>& blocks) {
    ++clock_;
    int node = 0;
    size_t pos = 0;
    while (pos + bs_ <= key.size()) {
      auto it = nodes_[node].children.find(block_hash(key, pos));
      if (it == nodes_[node].children.end()) break;
      int child = it->second;
      Node& c = nodes_[child];
      const size_t shared = shared_blocks(c.key, key, pos);
      if (shared == 0) break;
      touch(child);
      blocks.insert(blocks.end(), c.blocks.begin(), c.blocks.begin() + shared);
      pos += shared * bs_;
      node = child;
      if (shared < c.blocks.size()) break;   // partial edge match: stop here
    }
    return node;
  }

  void incref(int node) {
    while (node != 0) {
      Node& n = nodes_[node];
      if (n.ref_count++ == 0) leaves_.erase({n.last_accessed, node});
      node = n.parent;
    }
  }

  void decref(int node) {
    while (node != 0) {
      Node& n = nodes_[node];
      if (n.ref_count == 0) throw std::runtime_error("radix: decref of an unpinned node");
      if (--n.ref_count == 0 && n.children.empty()) leaves_.insert({n.last_accessed, node});
      node = n.parent;
    }
  }

  // Inserts `key` (length a multiple of the block size) backed by `blocks`.  Returns how many
  // leading tokens were already present (their blocks in `blocks` are duplicates the caller owns).
  size_t insert(const std::vector<uint32_t>& key, const std::vector<uint32_t>& blocks) {
    ++clock_;
    if (key.size() != blocks.size() * bs_) throw std::runtime_error("radix: key/blocks length mismatch");
    int node = 0;
    size_t pos = 0;
    while (pos < key.size()) {
      auto it = nodes_[node].children.find(block_hash(key, pos));
      if (it == nodes_[node].children.end()) {
        add_child(node, key, blocks, pos);
        return pos;
      }
      int child = it->second;
      const size_t shared = shared_blocks(nodes_[child].key, key, pos);
      if (shared == 0) {   // hash collision with different tokens: keep the existing entry
        return pos;
      }
      touch(child);
      if (shared < nodes_[child].blocks.size()) {
        child = split(child, shared);
      }
      pos += shared * bs_;
      node = child;
    }
    return pos;
  }

  // Frees at least `n_blocks` blocks from unpinned leaves, least recently used first.
  std::vector<uint32_t> evict(size_t n_blocks) {
    std::vector<uint32_t> freed;
    while (freed.size() < n_blocks && !leaves_.empty()) {
      auto it = leaves_.begin();
      int id = it->second;
      Node& n = nodes_[id];
      const size_t want = n_blocks - freed.size();
      if (n.blocks.size() > want) {
        // partial eviction: drop blocks from the tail of the edge
        const size_t keep = n.blocks.size() - want;
        freed.insert(freed.end(), n.blocks.begin() + keep, n.blocks.end());
        n.blocks.resize(keep);
        n.key.resize(keep * bs_);
        break;
      }
      freed.insert(freed.end(), n.blocks.begin(), n.blocks.end());
      leaves_.erase(it);
      remove_node(id);
    }
    return freed;
  }

  size_t cached_blocks() const {
    size_t n = 0;
    for (const auto& nd : nodes_)
      if (nd.alive) n += nd.blocks.size();
    return n;
  }
  size_t live_nodes() const {
    size_t n = 0;
    for (const auto& nd : nodes_) n += nd.alive;
    return n;
  }
  uint32_t ref_count(int node) const { return nodes_[node].ref_count; }
  int parent(int node) const { return nodes_[node].parent; }
  size_t arena_size() const { return nodes_.size(); }
  bool alive(int node) const { return nodes_[node].alive; }

  // invariant check used by the tests
  bool check() const {
    for (size_t i = 1; i < nodes_.size(); ++i) {
      const Node& n = nodes_[i];
      if (!n.alive) continue;
      if (n.key.size() != n.blocks.size() * bs_ || n.blocks.empty()) return false;
      const bool is_leaf = n.children.empty() && n.ref_count == 0;
      if (is_leaf != (leaves_.count({n.last_accessed, static_cast<int>(i)}) == 1)) return false;
      for (const auto& kv : n.children)
        if (!nodes_[kv.second].alive || nodes_[kv.second].parent != static_cast<int>(i)) return false;
    }
    return true;
  }

 private:
  struct Node {
    std::vector<uint32_t> key;
    std::vector<uint32_t> blocks;
    std::unordered_map<uint64_t, int> children;
    int parent = 0;
    uint32_t ref_count = 0;
    uint64_t last_accessed = 0;
    bool alive = false;
  };

  uint64_t block_hash(const std::vector<uint32_t>& key, size_t pos) const {
    uint64_t h = 1469598103934665603ull;
    for (size_t i = 0; i < bs_; ++i) {
      h ^= key[pos + i];
      h *= 1099511628211ull;
    }
    return h;
  }
  size_t shared_blocks(const std::vector<uint32_t>& edge, const std::vector<uint32_t>& key, size_t pos) const {
    size_t n = 0;
    const size_t max_blocks = std::min(edge.size(), key.size() - pos) / bs_;
    while (n < max_blocks && std::equal(edge.begin() + n * bs_, edge.begin() + (n + 1) * bs_, key.begin() + pos + n * bs_))
      ++n;
    return n;
  }
  void touch(int id) {
    Node& n = nodes_[id];
    const bool leaf = n.children.empty() && n.ref_count == 0;
    if (leaf) leaves_.erase({n.last_accessed, id});
    n.last_accessed = clock_;
    if (leaf) leaves_.insert({n.last_accessed, id});
  }
  int new_node() {
    if (!free_ids_.empty()) {
      int id = free_ids_.back();
      free_ids_.pop_back();
      nodes_[id] = Node{};
      nodes_[id].alive = true;
      return id;
    }
    nodes_.push_back(Node{});
    nodes_.back().alive = true;
    return static_cast<int>(nodes_.size()) - 1;
  }
  void add_child(int parent, const std::vector<uint32_t>& key, const std::vector<uint32_t>& blocks, size_t pos) {
    Node& p0 = nodes_[parent];
    if (parent != 0 && p0.children.empty() && p0.ref_count == 0) leaves_.erase({p0.last_accessed, parent});
    int id = new_node();
    Node& n = nodes_[id];
    n.key.assign(key.begin() + pos, key.end());
    n.blocks.assign(blocks.begin() + pos / bs_, blocks.end());
    n.parent = parent;
    n.last_accessed = clock_;
    nodes_[parent].children[block_hash(key, pos)] = id;
    leaves_.insert({n.last_accessed, id});
  }
  // Cuts the edge of `id` after `nblocks` blocks.  The node keeps its id and becomes the deeper half (so
  // holders that pinned `id` release both halves when they walk up from it, as the reference's
  // split_node does, backends/v3/src/radix.rs:473-506); a new node takes the first `nblocks` blocks
  // and the place of `id` under its parent.  Returns the new (upper) node.
  int split(int id, size_t nblocks) {
    const int head = new_node();   // may grow the arena: take references afterwards
    Node& n = nodes_[id];
    Node& h = nodes_[head];
    h.key.assign(n.key.begin(), n.key.begin() + nblocks * bs_);
    h.blocks.assign(n.blocks.begin(), n.blocks.begin() + nblocks);
    h.parent = n.parent;
    h.ref_count = n.ref_count;   // every pin of the lower half passes through the upper half
    h.last_accessed = n.last_accessed;
    nodes_[n.parent].children[block_hash(h.key, 0)] = head;   // same first block: replaces `id`
    n.key.erase(n.key.begin(), n.key.begin() + nblocks * bs_);
    n.blocks.erase(n.blocks.begin(), n.blocks.begin() + nblocks);
    n.parent = head;
    h.children[block_hash(n.key, 0)] = id;
    // `id` keeps its children, pins and position in the leaf set; the upper half has a child and is no leaf
    return head;
  }
  void remove_node(int id) {
    Node& n = nodes_[id];
    int parent = n.parent;
    Node& p = nodes_[parent];
    p.children.erase(block_hash(n.key, 0));
    n.alive = false;
    n.key.clear();
    n.blocks.clear();
    free_ids_.push_back(id);
    if (parent != 0 && p.children.empty() && p.ref_count == 0) leaves_.insert({p.last_accessed, parent});
  }

  uint32_t bs_;
  uint64_t clock_ = 0;
  std::vector<Node> nodes_;
  std::vector<int> free_ids_;
  std::set<std::pair<uint64_t, int>> leaves_;   // unpinned leaves ordered by last access
};

class BlockAllocator {
 public:
  BlockAllocator(uint32_t num_blocks, uint32_t block_size, bool prefix_caching, std::optional<uint32_t> window = {})
      : bs_(block_size), prefix_caching_(prefix_caching), window_(window), trie_(block_size) {
    // block 0 is reserved for the shard liveness probe
    for (uint32_t b = num_blocks; b-- > 1;) free_.push_back(b);
  }

  size_t free_blocks() const { return free_.size(); }
  RadixTrie& trie() { return trie_; }
  size_t live_allocations() const { return live_.size(); }

  // Structural invariants of the trie plus the pin accounting: every node's reference count equals the
  // number of live allocations whose pinned path passes through it (so it is 0 everywhere once nothing
  // is live and every cached block can be evicted again).
  bool check() const {
    if (!trie_.check()) return false;
    std::vector<uint32_t> expect(trie_.arena_size(), 0);
    for (const auto& kv : live_) {
      if (!prefix_caching_ || !kv.second.has_prompt) continue;
      for (int node = kv.second.node; node != 0; node = trie_.parent(node)) ++expect[node];
    }
    for (size_t i = 1; i < expect.size(); ++i)
      if (trie_.alive(static_cast<int>(i)) && trie_.ref_count(static_cast<int>(i)) != expect[i]) return false;
    return true;
  }

  // Allocate blocks for `tokens` tokens; `prompt` (token ids) enables prefix re-use.
  std::optional<BlockAllocation> allocate(uint32_t tokens, const std::vector<uint32_t>* prompt) {
    BlockAllocation a;
    int node = 0;
    if (prefix_caching_ && prompt != nullptr) {
      node = trie_.find(*prompt, a.blocks);
      trie_.incref(node);
    }
    a.prefix_len = static_cast<uint32_t>(a.blocks.size()) * bs_;
    uint32_t want_tokens = tokens;
    if (window_ && !prefix_caching_) want_tokens = std::min(tokens, *window_);   // blocks are re-used cyclically
    const uint32_t total_blocks = (want_tokens + bs_ - 1) / bs_;
    const size_t suffix = total_blocks > a.blocks.size() ? total_blocks - a.blocks.size() : 0;
    if (free_.size() < suffix) {
      auto got = trie_.evict(suffix - free_.size());
      free_.insert(free_.end(), got.begin(), got.end());
    }
    if (free_.size() < suffix) {
      if (node != 0 || prefix_caching_) trie_.decref(node);
      return std::nullopt;
    }
    for (size_t i = 0; i < suffix; ++i) {
      a.blocks.push_back(free_.back());
      free_.pop_back();
    }
    a.slots.reserve(static_cast<size_t>(tokens));
    if (window_ && !prefix_caching_) {
      // sliding window: positions beyond the window wrap around the allocated blocks
      for (uint32_t t = 0; t < tokens; ++t) {
        const uint32_t w = t % (static_cast<uint32_t>(a.blocks.size()) * bs_);
        a.slots.push_back(a.blocks[w / bs_] * bs_ + w % bs_);
      }
    } else {
      for (uint32_t b : a.blocks)
        for (uint32_t s = 0; s < bs_; ++s) a.slots.push_back(b * bs_ + s);
    }
    a.allocation_id = next_id_++;
    live_[a.allocation_id] = Live{node, a.prefix_len, prompt ? *prompt : std::vector<uint32_t>{}, prompt != nullptr};
    return a;
  }

  // `computed_tokens`: how many prompt tokens have their KV written.  Only those blocks may enter the
  // prefix cache: a request that was pushed back before it ran, or whose prefill failed or was cut
  // short, passes what it knows to be computed (0 if nothing) and the rest goes back to the free list.
  void free(const std::vector<uint32_t>& blocks, uint64_t allocation_id, uint32_t computed_tokens = UINT32_MAX) {
    auto it = live_.find(allocation_id);
    if (it == live_.end()) throw std::runtime_error("allocator: unknown allocation id");
    Live l = std::move(it->second);
    live_.erase(it);
    if (!prefix_caching_ || !l.has_prompt) {
      free_.insert(free_.end(), blocks.begin(), blocks.end());
      return;
    }
    trie_.decref(l.node);
    // only whole prompt blocks can be shared; the last prompt token's block may be partial
    const size_t aligned_blocks =
        std::min(std::min<size_t>(l.prompt.size(), computed_tokens) / bs_, blocks.size());
    size_t already = l.cached_prefix / bs_;
    if (aligned_blocks > 0) {
      std::vector<uint32_t> key(l.prompt.begin(), l.prompt.begin() + aligned_blocks * bs_);
      std::vector<uint32_t> kb(blocks.begin(), blocks.begin() + aligned_blocks);
      const size_t present = trie_.insert(key, kb) / bs_;
      // blocks in [cached_prefix, present) duplicate what another request inserted in the meantime
      for (size_t i = already; i < std::min(present, aligned_blocks); ++i) free_.push_back(blocks[i]);
    }
    for (size_t i = std::max(aligned_blocks, already); i < blocks.size(); ++i) free_.push_back(blocks[i]);
  }

 private:
  struct Live {
    int node;
    uint32_t cached_prefix;
    std::vector<uint32_t> prompt;
    bool has_prompt;
  };
  uint32_t bs_;
  bool prefix_caching_;
  std::optional<uint32_t> window_;
  RadixTrie trie_;
  std::vector<uint32_t> free_;
  std::unordered_map<uint64_t, Live> live_;
  uint64_t next_id_ = 1;
};

}  // namespace sched
