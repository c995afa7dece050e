#include "scheduler.h"

#include <algorithm>
#include <stdexcept>

namespace mrs {

Scheduler::Scheduler(CacheManager* cache, int64_t max_seq_len, int64_t prefill_budget, int max_running,
                     int max_waiting, std::vector<int32_t> eos, Policy policy, int64_t vocab_size)
    : cache_(cache), max_seq_len_(max_seq_len), prefill_budget_(prefill_budget), max_running_(max_running),
      max_waiting_(max_waiting), eos_(std::move(eos)), policy_(policy), vocab_size_(vocab_size) {
    if (!cache || max_seq_len <= 0 || prefill_budget <= 0 || max_running <= 0 || max_waiting <= 0)
        throw std::invalid_argument("runtime limits must be positive");
}

int Scheduler::submit(Submission s, std::string* why) {
    auto refuse = [&](int code, const char* text) {
        if (why) *why = text;
        return code;
    };
    if (s.tokens.empty()) return refuse(kInvalid, "prompt must contain valid nonempty token IDs");
    for (int32_t t : s.tokens)
        if (t < 0 || t >= vocab_size_) return refuse(kInvalid, "prompt must contain valid nonempty token IDs");
    if (s.max_tokens <= 0) return refuse(kInvalid, "top_k and max_tokens must be positive");
    const int64_t length = (int64_t)s.tokens.size() + s.max_tokens;
    if (length > max_seq_len_) return refuse(kInvalid, "prompt + max_tokens exceeds context limit");
    for (int g = 0; g < cache_->num_groups(); ++g)
        if (cache_->worst_case_pages(g, length, prefill_budget_) > cache_->total_pages(g))
            return refuse(kTooLarge, "request exceeds total KV capacity");
    for (const auto& w : waiting_)
        if (w.id == s.id) return refuse(kInvalid, "duplicate request id");
    for (const auto& r : running_)
        if (r.input.id == s.id) return refuse(kInvalid, "duplicate request id");
    if ((int)waiting_.size() >= max_waiting_) return refuse(kNoRoom, "waiting queue is full");
    counters_.submitted += 1;
    waiting_.push_back(std::move(s));
    return kOk;
}

bool Scheduler::cancel(int64_t request) {
    for (auto& r : running_)
        if (r.input.id == request) { r.cancel = true; return true; }
    for (auto it = waiting_.begin(); it != waiting_.end(); ++it)
        if (it->id == request) {
            finished_.push_back({request, Finish::Cancelled, (int64_t)it->tokens.size(), 0});
            counters_.cancelled += 1;
            waiting_.erase(it);
            return true;
        }
    return false;
}

void Scheduler::finish(size_t index, Finish reason) {
    Running& r = running_[index];
    finished_.push_back({r.input.id, reason, r.prompt_len, r.generated, r.cached});
    switch (reason) {
        case Finish::Stop: case Finish::Length: counters_.completed += 1; break;
        case Finish::Cancelled: counters_.cancelled += 1; break;
        case Finish::Error: counters_.failed += 1; break;
    }
    // a request that ended by itself leaves what it generated behind as well: a next turn that begins with
    // this one's prompt and answer reads both (reference: terminal(), crates/runtime/src/scheduler.rs:94-96)
    if (reason == Finish::Stop || reason == Finish::Length) cache_->publish(r.input.id, r.tokens.data(), r.computed);
    cache_->close(r.input.id);
    running_.erase(running_.begin() + (std::ptrdiff_t)index);
}

void Scheduler::admit() {
    while ((int)running_.size() < max_running_ && !waiting_.empty()) {
        const Submission& front = waiting_.front();
        const int64_t length = (int64_t)front.tokens.size() + front.max_tokens;
        int64_t shared = 0;
        const int slot = cache_->open_prompt(front.id, front.tokens.data(), (int64_t)front.tokens.size(), length,
                                             prefill_budget_, &shared);
        if (slot < 0) break;   // the head of the queue waits, and so do those behind it
        Running r;
        r.computed = r.cached = shared;
        counters_.cached_tokens += shared;
        r.input = std::move(waiting_.front());
        waiting_.pop_front();
        r.tokens = r.input.tokens;
        r.prompt_len = (int64_t)r.tokens.size();
        r.slot = slot;
        counters_.prompt_tokens += r.prompt_len;
        running_.push_back(std::move(r));
    }
}

const std::vector<PlannedSequence>& Scheduler::plan() {
    plan_.clear();
    plan_index_.clear();
    for (size_t i = running_.size(); i-- > 0;)
        if (running_[i].cancel) finish(i, Finish::Cancelled);
    admit();
    bool any_prefill = false, any_decode = false;
    for (const auto& r : running_)
        if (!r.length_reached) (r.computed < r.prompt_len ? any_prefill : any_decode) = true;
    if (!any_prefill && !any_decode) return plan_;
    bool take_prefill = true, take_decode = true;
    if (policy_ == Policy::Alternate) {
        const bool decode_step = any_decode && (!any_prefill || prefer_decode_);
        take_decode = decode_step;
        take_prefill = !decode_step;
        prefer_decode_ = !decode_step;
    }
    int64_t budget = prefill_budget_;
    bool planned_prefill = false, planned_decode = false;
    if (take_decode) {
        for (size_t i = 0; i < running_.size() && budget > 0; ++i) {
            Running& r = running_[i];
            if (r.computed < r.prompt_len || r.length_reached) continue;
            if (cache_->extend(r.input.id, r.computed + 1) != kOk)
                throw std::logic_error("a running request ran out of promised pages");
            plan_.push_back({r.input.id, r.slot, r.computed, 1, true});
            plan_index_.push_back(i);
            if (policy_ == Policy::Mixed) budget -= 1;
            planned_decode = true;
        }
    }
    if (take_prefill) {
        for (size_t i = 0; i < running_.size() && budget > 0; ++i) {
            Running& r = running_[i];
            if (r.computed >= r.prompt_len) continue;
            const int64_t n = std::min(budget, r.prompt_len - r.computed);
            budget -= n;
            if (cache_->extend(r.input.id, r.computed + n) != kOk)
                throw std::logic_error("a running request ran out of promised pages");
            plan_.push_back({r.input.id, r.slot, r.computed, n, r.computed + n >= r.prompt_len});
            plan_index_.push_back(i);
            planned_prefill = true;
        }
    }
    if (planned_prefill && planned_decode) counters_.mixed_batches += 1;
    else if (planned_prefill) counters_.prefill_batches += 1;
    else if (planned_decode) counters_.decode_batches += 1;
    return plan_;
}

const Running* Scheduler::find(int64_t request) const {
    for (const auto& r : running_)
        if (r.input.id == request) return &r;
    return nullptr;
}

// Whether a request whose newest token is `token` ends with it, and why.
bool Scheduler::ends_with(Running& r, int32_t token, Finish* reason) const {
    if (r.cancel) *reason = Finish::Cancelled;
    else if (!r.input.ignore_eos && std::find(eos_.begin(), eos_.end(), token) != eos_.end()) *reason = Finish::Stop;
    else if (r.generated >= r.input.max_tokens) *reason = Finish::Length;
    else return false;
    return true;
}

void Scheduler::commit(const std::vector<int32_t>& sampled) {
    size_t expected = 0;
    for (const auto& p : plan_) expected += p.sample;
    if (sampled.size() != expected) throw std::invalid_argument("runner output IDs do not match sampled batch");
    std::vector<std::pair<size_t, Finish>> ending;
    size_t next = 0;
    for (size_t j = 0; j < plan_.size(); ++j) {
        // by its id: a request may have ended between plan() and commit() (resolve() of the step before)
        size_t index = plan_index_[j];
        if (index >= running_.size() || running_[index].input.id != plan_[j].request) {
            for (index = 0; index < running_.size(); ++index)
                if (running_[index].input.id == plan_[j].request) break;
        }
        if (index == running_.size()) {
            next += plan_[j].sample;
            continue;
        }
        Running& r = running_[index];
        const bool prompt_was_open = r.computed < r.prompt_len;
        r.computed = plan_[j].start_pos + plan_[j].count;
        cache_->trim(r.input.id, r.computed);
        if (prompt_was_open && r.computed >= r.prompt_len)      // the prompt is in the cache: others may read its pages
            cache_->publish(r.input.id, r.tokens.data(), r.prompt_len);
        if (!plan_[j].sample) continue;
        const int32_t token = sampled[next++];
        if (r.unknown) throw std::logic_error("a second token of a request was committed before the first was resolved");
        r.tokens.push_back(token);
        r.generated += 1;
        counters_.generated_tokens += 1;
        if (token == kUnknownToken) {
            r.unknown = true;
            r.length_reached = r.generated >= r.input.max_tokens;
            continue;
        }
        Finish reason;
        if (ends_with(r, token, &reason)) ending.push_back({index, reason});
    }
    std::sort(ending.begin(), ending.end(), [](const auto& a, const auto& b) { return a.first < b.first; });
    size_t removed = 0;
    for (auto& [index, reason] : ending) finish(index - removed++, reason);
    plan_.clear();
    plan_index_.clear();
}

void Scheduler::resolve(const std::vector<int64_t>& requests, const std::vector<int32_t>& tokens) {
    if (requests.size() != tokens.size()) throw std::invalid_argument("resolve: as many tokens as requests");
    for (size_t k = 0; k < requests.size(); ++k) {
        size_t index = 0;
        for (; index < running_.size(); ++index)
            if (running_[index].input.id == requests[k]) break;
        if (index == running_.size()) continue;                  // ended meanwhile
        Running& r = running_[index];
        if (!r.unknown) throw std::logic_error("resolve: the request has no unknown token");
        if (tokens[k] < 0 || tokens[k] >= vocab_size_) throw std::invalid_argument("resolve: token outside the vocabulary");
        r.tokens.back() = tokens[k];
        r.unknown = false;
        Finish reason;
        if (ends_with(r, tokens[k], &reason)) finish(index, reason);
    }
}

void Scheduler::fail(Finish reason) {
    while (!running_.empty()) finish(0, reason);
    while (!waiting_.empty()) {
        finished_.push_back({waiting_.front().id, reason, (int64_t)waiting_.front().tokens.size(), 0});
        (reason == Finish::Error ? counters_.failed : counters_.cancelled) += 1;
        waiting_.pop_front();
    }
    plan_.clear();
    plan_index_.clear();
}

std::vector<Finished> Scheduler::drain_finished(size_t at_most) {
    const size_t n = std::min(at_most, finished_.size());
    std::vector<Finished> out(finished_.begin(), finished_.begin() + (std::ptrdiff_t)n);
    finished_.erase(finished_.begin(), finished_.begin() + (std::ptrdiff_t)n);
    return out;
}

}  // namespace mrs
