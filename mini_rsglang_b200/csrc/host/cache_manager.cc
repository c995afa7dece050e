#include "cache_manager.h"

#include <algorithm>
#include <sstream>
#include <stdexcept>

namespace mrs {

PagePool::PagePool(int64_t count) : refs_((size_t)count, 0) {
    free_.reserve((size_t)count);
    for (int64_t p = count - 1; p >= 0; --p) free_.push_back((int32_t)p);
}

int32_t PagePool::allocate() {
    if (free_.empty()) throw std::logic_error("page pool empty: reserved page capacity violated");
    const int32_t p = free_.back();
    free_.pop_back();
    if (refs_[(size_t)p] != 0) throw std::logic_error("free list held a page in use");
    refs_[(size_t)p] = 1;
    return p;
}

void PagePool::retain(int32_t page) {
    if (page < 0 || (size_t)page >= refs_.size() || refs_[(size_t)page] <= 0)
        throw std::logic_error("retain of a page that nobody holds");
    refs_[(size_t)page] += 1;
}

void PagePool::release(int32_t page) {
    if (page < 0 || (size_t)page >= refs_.size() || refs_[(size_t)page] <= 0)
        throw std::logic_error("double page release");
    if (--refs_[(size_t)page] == 0) free_.push_back(page);
}

static int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

CacheManager::CacheManager(std::vector<GroupSpec> groups, int page_size, int max_slots, bool prefix_cache)
    : groups_(std::move(groups)), page_size_(page_size), max_slots_(max_slots) {
    if (groups_.empty() || page_size <= 0 || max_slots <= 0) throw std::invalid_argument("empty cache geometry");
    for (const auto& g : groups_) {
        if (g.num_pages <= 0 || g.num_pages > INT32_MAX) throw std::invalid_argument("invalid page count");
        if (g.kind == GroupKind::Window && g.window <= 0) throw std::invalid_argument("window group needs a window");
        pools_.emplace_back(g.num_pages);
    }
    reserved_.assign(groups_.size(), 0);
    for (int s = max_slots - 1; s >= 0; --s) free_slots_.push_back(s);
    if (prefix_cache) {
        for (const auto& g : groups_)
            if (g.kind != GroupKind::Full) throw std::invalid_argument("prefix sharing needs groups that keep all keys");
        tree_ = std::make_unique<PrefixTree>(page_size, (int)groups_.size());
    }
}

// Evicts up to `nodes` pages that only the tree holds (one page a group each) and gives them back.
int64_t CacheManager::evict(int64_t nodes) {
    if (!tree_ || nodes <= 0) return 0;
    std::vector<std::pair<int, int32_t>> released;
    const int64_t gone = tree_->evict(nodes, &released);
    for (const auto& [g, page] : released) pools_[(size_t)g].release(page);
    return gone;
}

int64_t CacheManager::clear_idle_cache() { return evict(INT64_MAX); }

// The first logical page that a query at `next_position` (or any later one) can still read.
int64_t CacheManager::first_needed_page(int g, int64_t next_position) const {
    if (groups_[g].kind == GroupKind::Full) return 0;
    // a query at position p reads keys (p - window, p]; the earliest later query is next_position
    const int64_t first_key = std::max<int64_t>(0, next_position - groups_[g].window + 1);
    return first_key / page_size_;
}

int64_t CacheManager::worst_case_pages(int g, int64_t tokens, int64_t max_step) const {
    const int64_t all = ceil_div(tokens, page_size_);
    if (groups_[g].kind == GroupKind::Full) return all;
    // before a step of n tokens from position s the pages from first_needed_page(s) to the one of
    // s + n - 1 are live: at most window - 1 + max_step keys, which touch at most this many pages
    const int64_t span = (int64_t)groups_[g].window - 1 + std::max<int64_t>(1, max_step);
    return std::min(all, ceil_div(span, page_size_) + 1);
}

// What is still promised to a request in group g: enough to reach its worst case, but never more
// than the logical pages it has yet to make.
void CacheManager::settle_promise(Lease& lease, int g) {
    if (lease.promise[g] == 0) return;
    const int64_t to_make = lease.promised_pages - (int64_t)lease.tables[g].size();
    const int64_t target = std::max<int64_t>(0, std::min(lease.promise[g] - lease.held[g], to_make));
    reserved_[g] += target - lease.reserved[g];
    lease.reserved[g] = target;
}

int CacheManager::open(int64_t request, int64_t reserve_tokens, int64_t max_step) {
    if (leases_.count(request)) return kDuplicate;
    if (reserve_tokens < 0) return kInvalid;
    std::vector<int64_t> need(groups_.size(), 0);
    if (reserve_tokens > 0) {
        for (size_t g = 0; g < groups_.size(); ++g) {
            need[g] = worst_case_pages((int)g, reserve_tokens, max_step);
            if (need[g] > pools_[g].total()) return kTooLarge;
        }
        for (size_t g = 0; g < groups_.size(); ++g)
            if (pools_[g].free_count() + evictable_pages() < reserved_[g] + need[g]) return kNoRoom;
    }
    if (free_slots_.empty()) return kNoSlot;
    Lease lease;
    lease.request = request;
    lease.slot = free_slots_.back();
    free_slots_.pop_back();
    lease.tables.resize(groups_.size());
    lease.first_live.assign(groups_.size(), 0);
    lease.held.assign(groups_.size(), 0);
    lease.reserved = need;
    lease.promise = need;
    lease.promised_pages = ceil_div(reserve_tokens, page_size_);
    for (size_t g = 0; g < groups_.size(); ++g) reserved_[g] += need[g];
    const int slot = lease.slot;
    leases_.emplace(request, std::move(lease));
    return slot;
}

int CacheManager::open_prompt(int64_t request, const int32_t* prompt, int64_t prompt_len, int64_t reserve_tokens,
                              int64_t max_step, int64_t* shared_tokens) {
    if (shared_tokens) *shared_tokens = 0;
    if (!tree_) return open(request, reserve_tokens, max_step);
    if (leases_.count(request)) return kDuplicate;
    if (reserve_tokens < prompt_len || prompt_len <= 0 || !prompt) return kInvalid;
    const int64_t all = ceil_div(reserve_tokens, page_size_);
    for (size_t g = 0; g < groups_.size(); ++g)
        if (all > pools_[g].total()) return kTooLarge;
    if (free_slots_.empty()) return kNoSlot;
    std::vector<std::vector<int32_t>> found;
    const int node = tree_->lookup(prompt, prompt_len - 1, &found);
    tree_->pin(node);                       // what this request reads must not count as room
    const int64_t shared = (int64_t)found[0].size();
    for (size_t g = 0; g < groups_.size(); ++g)
        if (pools_[g].free_count() + evictable_pages() < reserved_[g] + (all - shared)) {
            tree_->unpin(node);
            return kNoRoom;
        }
    Lease lease;
    lease.request = request;
    lease.slot = free_slots_.back();
    free_slots_.pop_back();
    lease.tables = std::move(found);
    lease.first_live.assign(groups_.size(), 0);
    lease.held.assign(groups_.size(), shared);
    lease.reserved.assign(groups_.size(), all - shared);
    lease.promise.assign(groups_.size(), all);
    lease.promised_pages = all;
    lease.node = node;
    lease.shared_tokens = shared * page_size_;
    lease.length = lease.shared_tokens;
    for (size_t g = 0; g < groups_.size(); ++g) {
        for (int32_t page : lease.tables[g]) pools_[g].retain(page);
        reserved_[g] += all - shared;
    }
    if (shared_tokens) *shared_tokens = lease.shared_tokens;
    const int slot = lease.slot;
    leases_.emplace(request, std::move(lease));
    return slot;
}

int CacheManager::publish(int64_t request, const int32_t* tokens, int64_t computed) {
    if (!tree_) return kOk;
    auto it = leases_.find(request);
    if (it == leases_.end()) return kUnknown;
    Lease& lease = it->second;
    if (computed > lease.length || computed < 0 || !tokens) return kInvalid;
    std::vector<std::pair<int, int32_t>> retained;
    const int node = tree_->insert(tokens, computed, lease.tables, &retained);
    for (const auto& [g, page] : retained) pools_[(size_t)g].retain(page);
    tree_->pin(node);                       // the new path first, so that no node of both paths is ever unpinned
    tree_->unpin(lease.node);
    lease.node = node;
    return kOk;
}

int CacheManager::extend(int64_t request, int64_t new_length) {
    auto it = leases_.find(request);
    if (it == leases_.end()) return kUnknown;
    Lease& lease = it->second;
    if (new_length < lease.length) return kInvalid;
    const int64_t pages = ceil_div(new_length, page_size_);
    // First see whether every group can give what is asked: a refusal changes nothing.
    int64_t short_of = 0;              // pages that the pools lack and the prefix tree may give back
    for (size_t g = 0; g < groups_.size(); ++g) {
        const int64_t take = std::max<int64_t>(0, pages - (int64_t)lease.tables[g].size());
        const int64_t promised_to_others = reserved_[g] - lease.reserved[g];
        if (pools_[g].free_count() + evictable_pages() - promised_to_others < take) return kNoRoom;
        short_of = std::max(short_of, take - pools_[g].free_count());
    }
    evict(short_of);
    for (size_t g = 0; g < groups_.size(); ++g) {
        auto& table = lease.tables[g];
        while ((int64_t)table.size() < pages) {
            table.push_back(pools_[g].allocate());
            lease.held[g] += 1;
            if (lease.reserved[g] > 0) {
                lease.reserved[g] -= 1;
                reserved_[g] -= 1;
            }
        }
        settle_promise(lease, (int)g);
    }
    lease.length = new_length;
    return kOk;
}

int CacheManager::trim(int64_t request, int64_t computed) {
    auto it = leases_.find(request);
    if (it == leases_.end()) return kUnknown;
    Lease& lease = it->second;
    if (computed > lease.length) return kInvalid;
    int freed = 0;
    for (size_t g = 0; g < groups_.size(); ++g) {
        if (groups_[g].kind != GroupKind::Window) continue;
        auto& table = lease.tables[g];
        const int64_t keep_from = std::min<int64_t>(first_needed_page((int)g, computed), (int64_t)table.size());
        for (int64_t p = lease.first_live[g]; p < keep_from; ++p) {
            if (table[(size_t)p] >= 0) {
                pools_[g].release(table[(size_t)p]);
                table[(size_t)p] = -1;
                lease.held[g] -= 1;
                ++freed;
            }
        }
        lease.first_live[g] = std::max(lease.first_live[g], keep_from);
        settle_promise(lease, (int)g);
    }
    return freed;
}

int CacheManager::close(int64_t request) {
    auto it = leases_.find(request);
    if (it == leases_.end()) return kUnknown;
    Lease& lease = it->second;
    for (size_t g = 0; g < groups_.size(); ++g) {
        for (int32_t page : lease.tables[g])
            if (page >= 0) pools_[g].release(page);
        reserved_[g] -= lease.reserved[g];
    }
    if (tree_) tree_->unpin(lease.node);
    free_slots_.push_back(lease.slot);
    leases_.erase(it);
    return kOk;
}

const Lease* CacheManager::find(int64_t request) const {
    auto it = leases_.find(request);
    return it == leases_.end() ? nullptr : &it->second;
}

std::string CacheManager::check() const {
    std::ostringstream bad;
    for (size_t g = 0; g < groups_.size(); ++g) {
        const auto& pool = pools_[g];
        std::vector<int32_t> expected((size_t)pool.total(), 0);
        std::vector<char> in_tree((size_t)pool.total(), 0);
        if (tree_) {
            std::vector<std::pair<int, int32_t>> resident;
            tree_->resident(&resident);
            for (const auto& [group, page] : resident) {
                if (group != (int)g) continue;
                if (page < 0 || page >= pool.total()) { bad << "group " << g << ": the prefix tree holds page " << page << " outside the pool; "; continue; }
                if (in_tree[(size_t)page]) bad << "group " << g << ": the prefix tree holds page " << page << " twice; ";
                in_tree[(size_t)page] = 1;
                expected[(size_t)page] += 1;
            }
        }
        int64_t promised = 0;
        for (const auto& [id, lease] : leases_) {
            promised += lease.reserved[g];
            int64_t held = 0;
            for (int32_t page : lease.tables[g]) held += page >= 0;
            if (held != lease.held[g]) bad << "group " << g << ": request " << id << " counts " << lease.held[g] << " pages, its table has " << held << "; ";
            if (lease.promise[g] > 0 && lease.promised_pages >= (int64_t)lease.tables[g].size() && held + lease.reserved[g] > lease.promise[g]) bad << "group " << g << ": request " << id << " holds and is promised more than its worst case; ";
            for (size_t p = 0; p < lease.tables[g].size(); ++p) {
                const int32_t page = lease.tables[g][p];
                if (page < 0) continue;
                if (page >= pool.total()) { bad << "group " << g << ": request " << id << " holds page " << page << " outside the pool; "; continue; }
                if ((int64_t)p < lease.first_live[g]) bad << "group " << g << ": request " << id << " holds logical page " << p << " below its live range; ";
                expected[(size_t)page] += 1;
            }
        }
        if (promised != reserved_[g]) bad << "group " << g << ": promises " << reserved_[g] << " != sum over requests " << promised << "; ";
        if (reserved_[g] > pool.free_count() + evictable_pages()) bad << "group " << g << ": more pages promised than free; ";
        std::vector<char> in_free((size_t)pool.total(), 0);
        for (int32_t page : pool.free_list()) {
            if (page < 0 || page >= pool.total()) { bad << "group " << g << ": free list holds page " << page << "; "; continue; }
            if (in_free[(size_t)page]) bad << "group " << g << ": page " << page << " freed twice; ";
            in_free[(size_t)page] = 1;
        }
        for (int64_t page = 0; page < pool.total(); ++page) {
            const int32_t refs = pool.refs()[(size_t)page];
            if (refs != expected[(size_t)page]) bad << "group " << g << ": page " << page << " has " << refs << " holders on record, " << expected[(size_t)page] << " in the tables; ";
            if (expected[(size_t)page] > 1 && !in_tree[(size_t)page]) bad << "group " << g << ": page " << page << " held twice; ";
            if ((refs == 0) != (in_free[(size_t)page] != 0)) bad << "group " << g << ": page " << page << (refs == 0 ? " lost (neither held nor free); " : " both held and free; ");
        }
    }
    std::vector<char> slot_used((size_t)max_slots_, 0);
    for (int s : free_slots_) {
        if (s < 0 || s >= max_slots_ || slot_used[(size_t)s]) bad << "slot " << s << " twice in the free list; ";
        else slot_used[(size_t)s] = 1;
    }
    for (const auto& [id, lease] : leases_) {
        if (lease.slot < 0 || lease.slot >= max_slots_ || slot_used[(size_t)lease.slot]) bad << "request " << id << " shares or lacks its slot " << lease.slot << "; ";
        else slot_used[(size_t)lease.slot] = 1;
    }
    for (int s = 0; s < max_slots_; ++s)
        if (!slot_used[(size_t)s]) bad << "slot " << s << " lost; ";
    if (tree_) {
        bad << tree_->check();
        for (const auto& [id, lease] : leases_) {
            if (!tree_->pinned(lease.node) && lease.node != 0) bad << "request " << id << " reads a prefix that is not pinned; ";
            if ((int64_t)tree_->depth(lease.node) * page_size_ < lease.shared_tokens) bad << "request " << id << " pins less than it shares; ";
        }
    }
    return bad.str();
}

}  // namespace mrs
