// Paged cache manager: who holds which page.  Host only; it never sees a device pointer
// (as in the reference, docs/architecture.md:95).
//
// Layers with the same need share a *group*: its own pool of pages and, for every open
// request, its own block table.  A "full" group keeps every key of a request; a "window" group
// keeps only the pages that the last `window` positions still touch and gives the others
// back while the request runs.  Beside the pages, every open request holds one *state slot*:
// an index into per-request arrays of fixed size (recurrent state, sampler state).
//
// Reference: PagePool, PageLease and CacheManager of crates/cache/src/lib.rs:242-410
// (reservation at admission, allocation on extend, release, integrity check).  Prefix
// sharing (`prefix_tree.h`) is an option of the manager: a request opened with its prompt
// reads the full pages that an earlier request left for the same tokens, and what it computes
// itself is shared in turn once its prompt is in the cache.  Pages that only the tree holds
// count as room: they are evicted, least recently used first, when a pool runs short.
#pragma once
#include <cstdint>
#include <string>
#include <unordered_map>
#include <memory>
#include <vector>

#include "prefix_tree.h"

namespace mrs {

enum class GroupKind : int { Full = 0, Window = 1 };

struct GroupSpec {
    GroupKind kind;
    int window;          // positions a query may look back (Window groups); 0 for Full
    int64_t num_pages;   // size of this group's pool
};

class PagePool {
public:
    explicit PagePool(int64_t count);
    int64_t total() const { return (int64_t)refs_.size(); }
    int64_t free_count() const { return (int64_t)free_.size(); }
    int32_t allocate();              // precondition: free_count() > 0
    void retain(int32_t page);       // one more holder of a page that is held
    void release(int32_t page);      // throws on a page that is not held
    const std::vector<int32_t>& refs() const { return refs_; }
    const std::vector<int32_t>& free_list() const { return free_; }
private:
    std::vector<int32_t> refs_;
    std::vector<int32_t> free_;      // LIFO; page 0 is handed out first
};

struct Lease {
    int64_t request = 0;
    int slot = -1;                               // state slot
    int64_t length = 0;                          // tokens covered by extend() so far
    std::vector<std::vector<int32_t>> tables;    // per group: logical page -> physical page, -1 once given back
    std::vector<int64_t> first_live;             // per group: first logical page still held
    std::vector<int64_t> held;                   // per group: pages held now
    std::vector<int64_t> reserved;               // per group: pages promised but not yet taken
    std::vector<int64_t> promise;                // per group: most pages it was promised to hold at once (0: none)
    int64_t promised_pages = 0;                  // logical pages the promise covers (ceil(reserve_tokens / page_size))
    int node = 0;                                // prefix sharing: the deepest node of the tree that this request pins
    int64_t shared_tokens = 0;                   // tokens it found in shared pages when it was opened
};

// Result codes of the calls below (negative = refusal, nothing changed).
enum : int {
    kOk = 0,
    kNoRoom = -1,        // does not fit now; may fit later
    kTooLarge = -2,      // can never fit this pool
    kUnknown = -3,       // no such request
    kDuplicate = -4,     // request id already open
    kNoSlot = -5,        // every state slot is taken
    kInvalid = -6,
};

class CacheManager {
public:
    // `prefix_cache`: share full pages between requests with the same first tokens (every group must keep
    // all keys: a window group cannot be shared).
    CacheManager(std::vector<GroupSpec> groups, int page_size, int max_slots, bool prefix_cache = false);

    int page_size() const { return page_size_; }
    int num_groups() const { return (int)groups_.size(); }
    int64_t total_pages(int g) const { return pools_[g].total(); }
    int64_t free_pages(int g) const { return pools_[g].free_count(); }
    int64_t reserved_pages(int g) const { return reserved_[g]; }
    bool prefix_cache() const { return tree_ != nullptr; }
    // Pages that only the prefix tree holds (evicted when room is needed), and all pages it holds.
    int64_t evictable_pages() const { return tree_ ? tree_->evictable_nodes() : 0; }
    int64_t cached_pages() const { return tree_ ? tree_->resident_nodes() : 0; }
    int free_slots() const { return (int)free_slots_.size(); }
    int open_requests() const { return (int)leases_.size(); }

    // Pages a request of `tokens` tokens holds at most in group g, when no step brings more than
    // `max_step` tokens of it.
    int64_t worst_case_pages(int g, int64_t tokens, int64_t max_step) const;

    // Opens a request and takes a state slot.  With reserve_tokens > 0 the worst-case pages of a
    // request of that many tokens are promised to it (it can then never run out); the request is
    // refused with kNoRoom if the promise cannot be kept now, kTooLarge if never.
    int open(int64_t request, int64_t reserve_tokens, int64_t max_step);
    // The same for a request whose prompt is known, with prefix sharing: the full pages that the tree has for
    // the prompt's first tokens (all but the last token, which is always computed: its logits are wanted)
    // become the first pages of the request, read only; `shared_tokens` gets how many tokens they hold, and
    // the request's length starts there.  Without a tree this is open().
    int open_prompt(int64_t request, const int32_t* prompt, int64_t prompt_len, int64_t reserve_tokens,
                    int64_t max_step, int64_t* shared_tokens);
    // The first `computed` tokens of the request (`tokens`) are in its pages: their full pages are shared
    // from now on.  Nothing without a tree.
    int publish(int64_t request, const int32_t* tokens, int64_t computed);
    // Evicts every page that only the tree holds; returns how many nodes went.
    int64_t clear_idle_cache();
    // Makes the pages for positions [0, new_length) exist (window groups: only those still
    // needed).  kNoRoom if a pool is empty; then nothing is changed.
    int extend(int64_t request, int64_t new_length);
    // After `computed` tokens are in the cache: window groups give back the pages that no later
    // query can reach.
    int trim(int64_t request, int64_t computed);
    // Gives everything back: pages, promises, the slot.
    int close(int64_t request);

    const Lease* find(int64_t request) const;
    // Every invariant: no page lost, held twice or freed twice; promises add up.  Empty string = sound.
    std::string check() const;

private:
    int64_t first_needed_page(int g, int64_t next_position) const;
    void settle_promise(Lease& lease, int g);
    int64_t evict(int64_t nodes);
    std::unique_ptr<PrefixTree> tree_;
    std::vector<GroupSpec> groups_;
    std::vector<PagePool> pools_;
    std::vector<int64_t> reserved_;
    int page_size_;
    int max_slots_;
    std::vector<int> free_slots_;
    std::unordered_map<int64_t, Lease> leases_;
};

}  // namespace mrs
