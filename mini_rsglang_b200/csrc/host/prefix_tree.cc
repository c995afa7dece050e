#include "prefix_tree.h"

#include <algorithm>
#include <sstream>
#include <stdexcept>
#include <string>

namespace mrs {

PrefixTree::PrefixTree(int page_size, int groups) : page_size_(page_size), groups_(groups) {
    if (page_size <= 0 || groups <= 0) throw std::invalid_argument("empty prefix tree geometry");
    nodes_.emplace_back();
    nodes_[0].live = true;
}

uint64_t PrefixTree::key_of(int parent, const int32_t* tokens) const {
    uint64_t h = 0x9E3779B97F4A7C15ull ^ (uint64_t)(uint32_t)parent;
    for (int i = 0; i < page_size_; ++i) {
        h ^= (uint64_t)(uint32_t)tokens[i] + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
        h *= 0xFF51AFD7ED558CCDull;
    }
    return h;
}

int PrefixTree::child(int parent, const int32_t* tokens) const {
    auto range = index_.equal_range(key_of(parent, tokens));
    for (auto it = range.first; it != range.second; ++it) {
        const Node& n = nodes_[(size_t)it->second];
        if (n.parent == parent && std::equal(n.tokens.begin(), n.tokens.end(), tokens)) return it->second;
    }
    return -1;
}

// A node is in the eviction order while nobody pins it and it has no children.
void PrefixTree::set_evictable(int node, bool on) {
    if (node == 0) return;
    const Node& n = nodes_[(size_t)node];
    if (on) leaves_.insert({n.tick, node});
    else leaves_.erase({n.tick, node});
}

void PrefixTree::touch(int node) {
    Node& n = nodes_[(size_t)node];
    const bool listed = n.pins == 0 && n.children == 0;
    if (listed) set_evictable(node, false);
    n.tick = clock_;
    if (listed) set_evictable(node, true);
}

int PrefixTree::lookup(const int32_t* tokens, int64_t n, std::vector<std::vector<int32_t>>* pages) {
    ++clock_;
    if (pages) pages->assign((size_t)groups_, {});
    int node = 0;
    for (int64_t at = 0; at + page_size_ <= n; at += page_size_) {
        const int next = child(node, tokens + at);
        if (next < 0) break;
        node = next;
        touch(node);
        if (pages)
            for (int g = 0; g < groups_; ++g) (*pages)[(size_t)g].push_back(nodes_[(size_t)node].pages[(size_t)g]);
    }
    return node;
}

int PrefixTree::insert(const int32_t* tokens, int64_t n, const std::vector<std::vector<int32_t>>& tables,
                       std::vector<std::pair<int, int32_t>>* retained) {
    ++clock_;
    int node = 0;
    int64_t logical = 0;
    for (int64_t at = 0; at + page_size_ <= n; at += page_size_, ++logical) {
        int next = child(node, tokens + at);
        if (next < 0) {
            for (int g = 0; g < groups_; ++g)
                if ((int64_t)tables[(size_t)g].size() <= logical || tables[(size_t)g][(size_t)logical] < 0)
                    throw std::logic_error("a page to be shared does not exist");
            if (vacant_.empty()) {
                next = (int)nodes_.size();
                nodes_.emplace_back();
            } else {
                next = vacant_.back();
                vacant_.pop_back();
            }
            Node& fresh = nodes_[(size_t)next];
            fresh = Node();
            fresh.parent = node;
            fresh.tokens.assign(tokens + at, tokens + at + page_size_);
            fresh.pages.resize((size_t)groups_);
            for (int g = 0; g < groups_; ++g) {
                fresh.pages[(size_t)g] = tables[(size_t)g][(size_t)logical];
                if (retained) retained->push_back({g, fresh.pages[(size_t)g]});
            }
            fresh.tick = clock_;
            fresh.live = true;
            index_.insert({key_of(node, tokens + at), next});
            Node& parent = nodes_[(size_t)node];
            if (node != 0 && parent.pins == 0 && parent.children == 0) set_evictable(node, false);
            parent.children += 1;
            ++live_;
            ++unpinned_;
            set_evictable(next, true);
        } else {
            touch(next);
        }
        node = next;
    }
    return node;
}

void PrefixTree::pin(int node) {
    for (int id = node; id != 0; id = nodes_[(size_t)id].parent) {
        Node& n = nodes_[(size_t)id];
        if (!n.live) throw std::logic_error("pin of a node that is gone");
        if (n.pins == 0) {
            if (n.children == 0) set_evictable(id, false);
            --unpinned_;
        }
        n.pins += 1;
    }
}

void PrefixTree::unpin(int node) {
    for (int id = node; id != 0; id = nodes_[(size_t)id].parent) {
        Node& n = nodes_[(size_t)id];
        if (!n.live || n.pins <= 0) throw std::logic_error("unpin without a pin");
        n.pins -= 1;
        if (n.pins == 0) {
            ++unpinned_;
            if (n.children == 0) set_evictable(id, true);
        }
    }
}

int64_t PrefixTree::evict(int64_t count, std::vector<std::pair<int, int32_t>>* released) {
    int64_t gone = 0;
    while (gone < count && !leaves_.empty()) {
        const int id = leaves_.begin()->second;
        leaves_.erase(leaves_.begin());
        Node& n = nodes_[(size_t)id];
        auto range = index_.equal_range(key_of(n.parent, n.tokens.data()));
        for (auto it = range.first; it != range.second; ++it)
            if (it->second == id) {
                index_.erase(it);
                break;
            }
        if (released)
            for (int g = 0; g < groups_; ++g) released->push_back({g, n.pages[(size_t)g]});
        const int parent = n.parent;
        n = Node();
        vacant_.push_back(id);
        --live_;
        --unpinned_;
        ++gone;
        Node& p = nodes_[(size_t)parent];
        p.children -= 1;
        if (parent != 0 && p.children == 0 && p.pins == 0) set_evictable(parent, true);      // now a leaf itself
    }
    return gone;
}

void PrefixTree::resident(std::vector<std::pair<int, int32_t>>* out) const {
    for (size_t id = 1; id < nodes_.size(); ++id)
        if (nodes_[id].live)
            for (int g = 0; g < groups_; ++g) out->push_back({g, nodes_[id].pages[(size_t)g]});
}

int PrefixTree::depth(int node) const {
    int d = 0;
    for (int id = node; id != 0; id = nodes_[(size_t)id].parent) ++d;
    return d;
}

std::string PrefixTree::check() const {
    std::ostringstream bad;
    int64_t unpinned = 0;
    size_t live = 0, listed = 0;
    std::vector<int64_t> children(nodes_.size(), 0);
    for (size_t id = 1; id < nodes_.size(); ++id) {
        const Node& n = nodes_[id];
        if (!n.live) continue;
        ++live;
        if (n.parent < 0 || (size_t)n.parent >= nodes_.size() || !nodes_[(size_t)n.parent].live) {
            bad << "prefix node " << id << " hangs on a node that is gone; ";
            continue;
        }
        children[(size_t)n.parent] += 1;
        if (n.pins == 0) ++unpinned;
        if (n.parent != 0 && nodes_[(size_t)n.parent].pins < n.pins) bad << "prefix node " << id << " is pinned more often than its parent; ";
        if (child(n.parent, n.tokens.data()) != (int)id) bad << "prefix node " << id << " is not found under its tokens; ";
    }
    for (size_t id = 1; id < nodes_.size(); ++id) {
        const Node& n = nodes_[id];
        if (!n.live) continue;
        if (children[id] != n.children) bad << "prefix node " << id << " counts " << n.children << " children, has " << children[id] << "; ";
        const bool should = n.pins == 0 && children[id] == 0;
        const bool is = leaves_.count({n.tick, (int)id}) != 0;
        if (should != is) bad << "prefix node " << id << (should ? " is missing from" : " is wrongly in") << " the eviction order; ";
        listed += is;
    }
    if (listed != leaves_.size()) bad << "the eviction order holds nodes that are gone; ";
    if (unpinned != unpinned_) bad << "prefix tree counts " << unpinned_ << " unpinned nodes, has " << unpinned << "; ";
    if (live != live_) bad << "prefix tree counts " << live_ << " nodes, has " << live << "; ";
    return bad.str();
}

}  // namespace mrs
