// Continuous-batching scheduler: admits requests, cuts prompts into portions under a token
// budget, decodes, finishes and frees.  It decides; the caller runs the model.  One step is
//     plan()  ->  the caller runs the batch and samples  ->  commit(tokens)
// and a failed step is answered with fail(), which finishes every request and frees every page.
//
// Reference: Scheduler of crates/runtime/src/scheduler.rs:33-360 (FIFO admission with a
// worst-case page reservation, head-of-line waiting, `prefill_budget`, finish reasons).  The
// reference alternates steps of prompt portions with steps of decoded tokens; here one step
// holds both (decoded tokens first, prompt portions in what is left of the budget), and the
// reference's alternation is kept as a policy for comparison.
//
// When pages run out: a request is admitted only if the pages of its whole life (prompt +
// max_tokens) can be promised to it, so a running request never lacks a page; a request that
// does not fit now waits at the head of the queue and holds back those behind it; one that can
// never fit is refused when it is submitted.  Nothing is preempted, swapped or recomputed.
//
// With prefix sharing in the cache manager a request is admitted with its prompt: what the tree has of the
// prompt's first pages is not computed again (`computed` starts behind them; the last prompt token is always
// computed), and when a request's prompt is in the cache its full pages are published for those that follow;
// a request that ends by a stop token or by its length publishes what it generated too
// (reference: acquire / publish, crates/runtime/src/scheduler.rs:94-96, 174, 283).
#pragma once
#include <cstdint>
#include <deque>
#include <string>
#include <vector>

#include "cache_manager.h"

namespace mrs {

enum class Policy : int { Mixed = 0, Alternate = 1 };
enum class Finish : int { Stop = 0, Length = 1, Cancelled = 2, Error = 3 };

struct Submission {
    int64_t id;
    std::vector<int32_t> tokens;   // the prompt
    int64_t max_tokens;
    bool ignore_eos;
};

struct Running {
    Submission input;
    std::vector<int32_t> tokens;   // prompt and generated tokens
    int64_t prompt_len = 0;
    int64_t computed = 0;          // tokens whose keys and values are in the cache
    int64_t generated = 0;
    int64_t cached = 0;            // prompt tokens found in shared pages at admission
    int slot = -1;
    bool cancel = false;
    bool unknown = false;          // its last token was committed before its value was known (kUnknownToken)
    bool length_reached = false;   // ... and was its last by max_tokens: the request ends when the value arrives
};

// A sampled token whose value the caller does not know yet (the step that samples it is still running): commit()
// takes it in a value's place, resolve() brings the value.
constexpr int32_t kUnknownToken = -1;

struct PlannedSequence {
    int64_t request;
    int slot;
    int64_t start_pos;
    int64_t count;                 // tokens of this step: tokens[start_pos, start_pos + count)
    bool sample;                   // the last of them yields the request's next token
};

struct Finished {
    int64_t request;
    Finish reason;
    int64_t prompt_tokens;
    int64_t completion_tokens;
    int64_t cached_tokens = 0;
};

struct Counters {
    int64_t submitted = 0, completed = 0, cancelled = 0, failed = 0;
    int64_t prompt_tokens = 0, generated_tokens = 0, cached_tokens = 0;
    int64_t prefill_batches = 0, decode_batches = 0, mixed_batches = 0;
};

class Scheduler {
public:
    Scheduler(CacheManager* cache, int64_t max_seq_len, int64_t prefill_budget, int max_running,
              int max_waiting, std::vector<int32_t> eos, Policy policy, int64_t vocab_size);

    // kOk, or kInvalid (empty prompt, id outside the vocabulary, too long for max_seq_len,
    // max_tokens < 1, duplicate id), kTooLarge (can never fit the pool), kNoRoom (queue full).
    int submit(Submission s, std::string* why);
    bool cancel(int64_t request);        // takes effect at the next plan() or commit()
    bool idle() const { return waiting_.empty() && running_.empty(); }
    int waiting() const { return (int)waiting_.size(); }
    int running() const { return (int)running_.size(); }

    // Builds the next batch (cancelled requests are finished first, then requests are admitted).
    // An empty plan means there is nothing to run.
    const std::vector<PlannedSequence>& plan();
    const std::vector<PlannedSequence>& last_plan() const { return plan_; }
    const Running* find(int64_t request) const;

    // One token per planned sequence with sample == true, in plan order.
    // Throws std::invalid_argument when the count differs.
    // A token may be kUnknownToken: the caller has queued the step and goes on before it has read what was
    // sampled.  The request then counts as one token further (its next step decodes that token, which the
    // caller takes from the device), but whether it ends is decided when resolve() brings the value: until
    // then it is planned as if it went on, except that a request at its max_tokens is not planned again.  At
    // most one token of a request is unknown at a time.  A request that has ended since the plan (by resolve()
    // or a cancel) is passed over, its token dropped.
    void commit(const std::vector<int32_t>& sampled);
    // The values of tokens committed as unknown: (request, token) in any order.  Each request is finished
    // here if the token ends it (stop token, max_tokens reached, cancelled); a request that is gone is skipped.
    void resolve(const std::vector<int64_t>& requests, const std::vector<int32_t>& tokens);
    // The step failed (or the engine shuts down): every request ends with `reason`, pages freed.
    void fail(Finish reason);
    // Requests that ended since the last call (by cancel, plan, commit or fail), in the order they ended.
    std::vector<Finished> drain_finished(size_t at_most = (size_t)-1);

    const Counters& counters() const { return counters_; }

private:
    void finish(size_t index, Finish reason);
    bool ends_with(Running& r, int32_t token, Finish* reason) const;
    void admit();
    CacheManager* cache_;
    int64_t max_seq_len_, prefill_budget_;
    int max_running_, max_waiting_;
    std::vector<int32_t> eos_;
    Policy policy_;
    int64_t vocab_size_;
    bool prefer_decode_ = true;
    std::deque<Submission> waiting_;
    std::vector<Running> running_;
    std::vector<PlannedSequence> plan_;
    std::vector<size_t> plan_index_;
    std::vector<Finished> finished_;
    Counters counters_;
};

}  // namespace mrs
