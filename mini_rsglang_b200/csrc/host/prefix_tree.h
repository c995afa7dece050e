// Prefix sharing: which full pages of keys and values spell which tokens.
//
// A tree of pages.  Every node stands for one full page of tokens that follows its parent's pages, and holds
// the physical page (one per page group) in which some request left the keys and values of exactly those
// tokens after exactly that prefix.  A request whose prompt begins with the same tokens reads those pages
// instead of computing them again.  Nodes are found by (parent, tokens of the page) in a hash table; there
// are no compressed edges, so nothing is ever split.  A request pins the path it reads (every node from its
// deepest match to the root); nodes that nobody pins can be evicted, leaves first, least recently used first.
//
// The tree only keeps the books: the manager counts a page reference for every page the tree holds and gives
// the pages of evicted nodes back to their pools.
//
// Reference: the `PrefixCache` trait and `RadixCache` of crates/cache/src/lib.rs:15-240 (lookup, insert, pin,
// unpin, evictable_pages, evict, resident_pages; page-aligned keys; least-recently-used leaves go first).
#pragma once
#include <cstdint>
#include <set>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace mrs {

class PrefixTree {
public:
    PrefixTree(int page_size, int groups);

    // The deepest node whose path spells the full pages of tokens[0, n) (0 = the root: nothing matched).
    // `pages[g]` gets the path's physical pages of group g, first page first.  Every node on the way counts
    // as used now.
    int lookup(const int32_t* tokens, int64_t n, std::vector<std::vector<int32_t>>* pages);
    // Makes the path for the full pages of tokens[0, n) exist.  Pages of new nodes are taken from
    // `tables[g][logical page]`; `retained` gets (group, page) of every page the tree holds from now on.
    // Returns the deepest node of the path.  Where a node exists already it keeps its own pages.
    int insert(const int32_t* tokens, int64_t n, const std::vector<std::vector<int32_t>>& tables,
               std::vector<std::pair<int, int32_t>>* retained);
    void pin(int node);                // the node and all its ancestors
    void unpin(int node);
    int64_t evictable_nodes() const { return unpinned_; }      // each holds one page in every group
    int64_t resident_nodes() const { return (int64_t)live_; }
    // Evicts up to `count` unpinned nodes, leaves first, least recently used first; `released` gets their
    // (group, page).  Returns how many went.
    int64_t evict(int64_t count, std::vector<std::pair<int, int32_t>>* released);
    void resident(std::vector<std::pair<int, int32_t>>* out) const;
    int depth(int node) const;         // pages on the path to the node
    bool pinned(int node) const { return nodes_[(size_t)node].pins > 0; }
    // Empty when the books are sound (counters match the nodes, leaves are where the eviction order says).
    std::string check() const;

private:
    struct Node {
        int parent = 0;
        std::vector<int32_t> tokens;      // the page's tokens
        std::vector<int32_t> pages;       // per group
        int64_t pins = 0;
        int64_t children = 0;
        uint64_t tick = 0;
        bool live = false;
    };
    uint64_t key_of(int parent, const int32_t* tokens) const;
    int child(int parent, const int32_t* tokens) const;
    void touch(int node);
    void set_evictable(int node, bool on);
    int page_size_, groups_;
    std::vector<Node> nodes_;             // [0] is the root
    std::vector<int> vacant_;
    std::unordered_multimap<uint64_t, int> index_;
    std::set<std::pair<uint64_t, int>> leaves_;      // unpinned nodes without children, by (tick, node)
    int64_t unpinned_ = 0;
    size_t live_ = 0;
    uint64_t clock_ = 0;
};

}  // namespace mrs
