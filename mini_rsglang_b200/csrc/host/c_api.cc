// C interface of the host library, loaded from Python with ctypes.  Handles are opaque
// pointers; every call returns a code (>= 0 success) and leaves a message for the last
// failure in thread-local storage.
#include <cstring>
#include <algorithm>
#include <exception>
#include <stdexcept>
#include <string>

#include "cache_manager.h"
#include "scheduler.h"

#define API extern "C" __attribute__((visibility("default")))

static thread_local std::string g_error;
static const int kException = -100;

template <typename F>
static int guarded(F f) {
    try {
        return f();
    } catch (const std::exception& e) {
        g_error = e.what();
        return kException;
    }
}

API const char* mrs_last_error() { return g_error.c_str(); }

// ----------------------------------------------------------------------------- cache manager
static void* cache_create(int n_groups, const int* kinds, const int* windows, const int64_t* num_pages, int page_size,
                          int max_slots, bool prefix_cache) {
    try {
        std::vector<mrs::GroupSpec> groups;
        for (int g = 0; g < n_groups; ++g)
            groups.push_back({kinds[g] == 1 ? mrs::GroupKind::Window : mrs::GroupKind::Full, windows[g], num_pages[g]});
        return new mrs::CacheManager(std::move(groups), page_size, max_slots, prefix_cache);
    } catch (const std::exception& e) {
        g_error = e.what();
        return nullptr;
    }
}
API void* mrs_cache_create(int n_groups, const int* kinds, const int* windows, const int64_t* num_pages,
                           int page_size, int max_slots) {
    return cache_create(n_groups, kinds, windows, num_pages, page_size, max_slots, false);
}
// The same with prefix sharing between requests (every group must keep all keys).
API void* mrs_cache_create_sharing(int n_groups, const int* kinds, const int* windows, const int64_t* num_pages,
                                   int page_size, int max_slots) {
    return cache_create(n_groups, kinds, windows, num_pages, page_size, max_slots, true);
}
API void mrs_cache_destroy(void* c) { delete static_cast<mrs::CacheManager*>(c); }
API int mrs_cache_open(void* c, int64_t request, int64_t reserve_tokens, int64_t max_step) {
    return guarded([&] { return static_cast<mrs::CacheManager*>(c)->open(request, reserve_tokens, max_step); });
}
// Opens a request whose prompt is known; with prefix sharing `shared_tokens` gets the tokens found in shared pages.
API int mrs_cache_open_prompt(void* c, int64_t request, const int32_t* prompt, int64_t prompt_len, int64_t reserve_tokens,
                              int64_t max_step, int64_t* shared_tokens) {
    return guarded([&] {
        return static_cast<mrs::CacheManager*>(c)->open_prompt(request, prompt, prompt_len, reserve_tokens, max_step, shared_tokens);
    });
}
API int mrs_cache_publish(void* c, int64_t request, const int32_t* tokens, int64_t computed) {
    return guarded([&] { return static_cast<mrs::CacheManager*>(c)->publish(request, tokens, computed); });
}
API int64_t mrs_cache_clear_idle(void* c) {
    try {
        return static_cast<mrs::CacheManager*>(c)->clear_idle_cache();
    } catch (const std::exception& e) {
        g_error = e.what();
        return kException;
    }
}
API int mrs_cache_shares_prefixes(void* c) { return static_cast<mrs::CacheManager*>(c)->prefix_cache() ? 1 : 0; }
API int64_t mrs_cache_cached_pages(void* c) { return static_cast<mrs::CacheManager*>(c)->cached_pages(); }
API int64_t mrs_cache_evictable_pages(void* c) { return static_cast<mrs::CacheManager*>(c)->evictable_pages(); }
API int mrs_cache_extend(void* c, int64_t request, int64_t new_length) {
    return guarded([&] { return static_cast<mrs::CacheManager*>(c)->extend(request, new_length); });
}
API int mrs_cache_trim(void* c, int64_t request, int64_t computed) {
    return guarded([&] { return static_cast<mrs::CacheManager*>(c)->trim(request, computed); });
}
API int mrs_cache_close(void* c, int64_t request) {
    return guarded([&] { return static_cast<mrs::CacheManager*>(c)->close(request); });
}
// Copies the block table of (request, group) into out (capacity cap); returns its length, or < 0.
API int mrs_cache_table(void* c, int64_t request, int group, int32_t* out, int cap) {
    return guarded([&]() -> int {
        auto* m = static_cast<mrs::CacheManager*>(c);
        const mrs::Lease* lease = m->find(request);
        if (!lease) return mrs::kUnknown;
        if (group < 0 || group >= m->num_groups()) return mrs::kInvalid;
        const auto& table = lease->tables[(size_t)group];
        if ((int)table.size() > cap) return mrs::kInvalid;
        if (!table.empty()) std::memcpy(out, table.data(), table.size() * sizeof(int32_t));     // an empty table has no data to point at
        return (int)table.size();
    });
}
API int mrs_cache_slot(void* c, int64_t request) {
    const mrs::Lease* lease = static_cast<mrs::CacheManager*>(c)->find(request);
    return lease ? lease->slot : mrs::kUnknown;
}
API int64_t mrs_cache_length(void* c, int64_t request) {
    const mrs::Lease* lease = static_cast<mrs::CacheManager*>(c)->find(request);
    return lease ? lease->length : (int64_t)mrs::kUnknown;
}
API int64_t mrs_cache_free_pages(void* c, int g) { return static_cast<mrs::CacheManager*>(c)->free_pages(g); }
API int64_t mrs_cache_total_pages(void* c, int g) { return static_cast<mrs::CacheManager*>(c)->total_pages(g); }
API int64_t mrs_cache_reserved_pages(void* c, int g) { return static_cast<mrs::CacheManager*>(c)->reserved_pages(g); }
API int64_t mrs_cache_worst_case_pages(void* c, int g, int64_t tokens, int64_t max_step) {
    return static_cast<mrs::CacheManager*>(c)->worst_case_pages(g, tokens, max_step);
}
API int mrs_cache_free_slots(void* c) { return static_cast<mrs::CacheManager*>(c)->free_slots(); }
API int mrs_cache_open_requests(void* c) { return static_cast<mrs::CacheManager*>(c)->open_requests(); }
// Writes the integrity report into msg (capacity cap); returns 0 when the manager is sound.
API int mrs_cache_check(void* c, char* msg, int cap) {
    const std::string report = static_cast<mrs::CacheManager*>(c)->check();
    if (cap > 0) {
        std::strncpy(msg, report.c_str(), (size_t)cap - 1);
        msg[cap - 1] = 0;
    }
    return report.empty() ? 0 : 1;
}

// --------------------------------------------------------------------------------- scheduler
API void* mrs_sched_create(void* cache, int64_t max_seq_len, int64_t prefill_budget, int max_running, int max_waiting,
                           const int32_t* eos, int n_eos, int policy, int64_t vocab_size) {
    try {
        return new mrs::Scheduler(static_cast<mrs::CacheManager*>(cache), max_seq_len, prefill_budget, max_running,
                                  max_waiting, std::vector<int32_t>(eos, eos + n_eos),
                                  policy == 1 ? mrs::Policy::Alternate : mrs::Policy::Mixed, vocab_size);
    } catch (const std::exception& e) {
        g_error = e.what();
        return nullptr;
    }
}
API void mrs_sched_destroy(void* s) { delete static_cast<mrs::Scheduler*>(s); }
API int mrs_sched_submit(void* s, int64_t id, const int32_t* tokens, int n, int64_t max_tokens, int ignore_eos) {
    return guarded([&] {
        mrs::Submission sub{id, std::vector<int32_t>(tokens, tokens + n), max_tokens, ignore_eos != 0};
        return static_cast<mrs::Scheduler*>(s)->submit(std::move(sub), &g_error);
    });
}
API int mrs_sched_cancel(void* s, int64_t id) { return static_cast<mrs::Scheduler*>(s)->cancel(id) ? 1 : 0; }
API int mrs_sched_idle(void* s) { return static_cast<mrs::Scheduler*>(s)->idle() ? 1 : 0; }
API int mrs_sched_waiting(void* s) { return static_cast<mrs::Scheduler*>(s)->waiting(); }
API int mrs_sched_running(void* s) { return static_cast<mrs::Scheduler*>(s)->running(); }
// Plans the next step.  Arrays have capacity cap; returns the number of sequences, or < 0.
API int mrs_sched_plan(void* s, int64_t* requests, int32_t* slots, int64_t* start_pos, int64_t* counts,
                       int32_t* sample, int cap) {
    return guarded([&]() -> int {
        const auto& plan = static_cast<mrs::Scheduler*>(s)->plan();
        if ((int)plan.size() > cap) throw std::length_error("plan larger than the caller's arrays");
        for (size_t i = 0; i < plan.size(); ++i) {
            requests[i] = plan[i].request;
            slots[i] = plan[i].slot;
            start_pos[i] = plan[i].start_pos;
            counts[i] = plan[i].count;
            sample[i] = plan[i].sample ? 1 : 0;
        }
        return (int)plan.size();
    });
}
// Copies the tokens of every sequence of the last plan, in the plan's order; returns their number, or < 0.
API int64_t mrs_sched_plan_tokens(void* s, int32_t* out, int64_t cap) {
    try {
        auto* sched = static_cast<mrs::Scheduler*>(s);
        int64_t n = 0;
        for (const auto& p : sched->last_plan()) {
            const mrs::Running* r = sched->find(p.request);
            if (!r || p.start_pos < 0 || p.start_pos + p.count > (int64_t)r->tokens.size()) return mrs::kInvalid;
            if (n + p.count > cap) return mrs::kInvalid;
            if (p.count > 0) std::memcpy(out + n, r->tokens.data() + p.start_pos, (size_t)p.count * sizeof(int32_t));
            n += p.count;
        }
        return n;
    } catch (const std::exception& e) {
        g_error = e.what();
        return kException;
    }
}
// Copies tokens [start, start + count) of a running request.
API int mrs_sched_tokens(void* s, int64_t request, int64_t start, int64_t count, int32_t* out) {
    return guarded([&]() -> int {
        const mrs::Running* r = static_cast<mrs::Scheduler*>(s)->find(request);
        if (!r) return mrs::kUnknown;
        if (start < 0 || count < 0 || start + count > (int64_t)r->tokens.size()) return mrs::kInvalid;
        if (count > 0) std::memcpy(out, r->tokens.data() + start, (size_t)count * sizeof(int32_t));
        return (int)count;
    });
}
API int mrs_sched_commit(void* s, const int32_t* sampled, int n) {
    return guarded([&] {
        static_cast<mrs::Scheduler*>(s)->commit(std::vector<int32_t>(sampled, sampled + n));
        return 0;
    });
}
// The values of tokens that were committed as unknown (-1): (request, token) pairs.
API int mrs_sched_resolve(void* s, const int64_t* requests, const int32_t* tokens, int n) {
    return guarded([&] {
        static_cast<mrs::Scheduler*>(s)->resolve(std::vector<int64_t>(requests, requests + n),
                                                 std::vector<int32_t>(tokens, tokens + n));
        return 0;
    });
}
API int mrs_sched_fail(void* s, int reason) {
    return guarded([&] {
        static_cast<mrs::Scheduler*>(s)->fail(static_cast<mrs::Finish>(reason));
        return 0;
    });
}
// Requests that ended since the last call; at most cap are written and returned, the rest stay for the next call.
static int drain(void* s, int64_t* requests, int32_t* reasons, int64_t* prompt_tokens, int64_t* completion_tokens,
                 int64_t* cached_tokens, int cap) {
    return guarded([&]() -> int {
        const auto pending = static_cast<mrs::Scheduler*>(s)->drain_finished((size_t)std::max(cap, 0));
        const int n = (int)pending.size();
        for (int i = 0; i < n; ++i) {
            requests[i] = pending[(size_t)i].request;
            reasons[i] = (int)pending[(size_t)i].reason;
            prompt_tokens[i] = pending[(size_t)i].prompt_tokens;
            completion_tokens[i] = pending[(size_t)i].completion_tokens;
            if (cached_tokens) cached_tokens[i] = pending[(size_t)i].cached_tokens;
        }
        return n;
    });
}
API int mrs_sched_drain(void* s, int64_t* requests, int32_t* reasons, int64_t* prompt_tokens,
                        int64_t* completion_tokens, int cap) {
    return drain(s, requests, reasons, prompt_tokens, completion_tokens, nullptr, cap);
}
// The same with the prompt tokens that each request found in shared pages.
API int mrs_sched_drain_cached(void* s, int64_t* requests, int32_t* reasons, int64_t* prompt_tokens,
                               int64_t* completion_tokens, int64_t* cached_tokens, int cap) {
    return drain(s, requests, reasons, prompt_tokens, completion_tokens, cached_tokens, cap);
}
API int64_t mrs_sched_cached_tokens(void* s) { return static_cast<mrs::Scheduler*>(s)->counters().cached_tokens; }
API void mrs_sched_counters(void* s, int64_t* out9) {
    const mrs::Counters& c = static_cast<mrs::Scheduler*>(s)->counters();
    const int64_t values[9] = {c.submitted, c.completed, c.cancelled, c.failed, c.prompt_tokens,
                               c.generated_tokens, c.prefill_batches, c.decode_batches, c.mixed_batches};
    std::memcpy(out9, values, sizeof(values));
}
