// Continuous-batching scheduler: admits requests, cuts prompts into portions
// under a token budget, puts single decoded tokens beside them, finishes and
// frees.  It decides; it runs nothing.  Each tick is plan() -> (the engine runs
// the step and samples) -> commit().
//
// What is mirrored from the reference's slot scheduler (src/batching.rs):
// FIFO admission (:283-328), max_new_tokens == 0 finishes at once (:287-290),
// an end-of-sequence token ends the request and is part of its output
// (:353-360), abort drops a request and what it holds (:264-269), an empty
// prompt is refused at submit (:248-250).  The reference prefills a whole
// prompt inside admit and fails every request when pages run out
// (src/server/engine.rs:317-321); here prompts are cut into portions and a
// request is pre-empted instead (see plan()).
#pragma once
#include <cstdint>
#include <deque>
#include <map>
#include <set>
#include <string>
#include <vector>

#include "cache_manager.hpp"

namespace dlm {

struct SchedulerConfig {
    int max_step_tokens = 2048;   // token budget of a step
    int max_step_requests = 64;   // rows of a step (and live requests)
    int max_context = 4096;       // prompt + generated tokens of one request
    int vocab_size = 0;           // token ids >= vocab are refused at submit; 0: no check
};

struct PlannedItem {
    int64_t id = 0;
    int slot = -1;
    int start = 0;                 // tokens of this request already in the cache
    std::vector<int32_t> tokens;   // the tokens this step runs
    bool sample = false;           // the last of them is the request's newest token
};

struct Plan {
    std::vector<PlannedItem> items;      // decode rows first, then prompt portions
    std::vector<int64_t> preempted;      // requests sent back to the queue in this plan
    std::vector<int64_t> failed;         // requests that can never fit; finished with an error
};

struct FinishedRequest {
    int64_t id = 0;
    std::vector<int32_t> output;   // generated tokens (end-of-sequence included)
    std::string reason;            // "length", "eos", "abort", "cache"
};

struct SchedulerStats {
    long steps = 0, prompt_tokens = 0, decode_tokens = 0, preemptions = 0, finished = 0;
};

class Scheduler {
public:
    Scheduler(CacheManager* cache, SchedulerConfig cfg);

    // Throws std::invalid_argument for an empty prompt, a token outside the
    // vocabulary, an id in use, or a prompt that leaves no room in the context.
    // max_new_tokens is clamped to what the context leaves.
    void submit(int64_t id, std::vector<int32_t> prompt, int max_new_tokens, std::vector<int32_t> eos);
    bool abort(int64_t id);

    bool has_work() const { return !waiting_.empty() || !running_.empty() || !done_.empty(); }
    int num_waiting() const { return (int)waiting_.size(); }
    int num_running() const { return (int)running_.size(); }

    // Decides the next step and takes its pages.  Order of decisions:
    //  1. every running request whose next portion is one token (a decode row), oldest first;
    //     if its page cannot be had, the most recently admitted running request is pre-empted
    //     (its pages freed, its tokens kept, put back at the head of the queue to be
    //     recomputed) until it can, or until it is itself the one pre-empted;
    //  2. running requests still in their prompt, oldest first: a portion of
    //     min(what is left, what the budget leaves, what the free pages hold);
    //  3. waiting requests in arrival order while a slot, a row and budget are left and the
    //     pool holds the first portion besides one spare page per running request.
    // A request that is alone and still cannot grow is finished with reason "cache".
    Plan plan();

    // `sampled` holds one token for every planned item with sample == true, in order.
    // Returns the requests that ended with this step.
    std::vector<FinishedRequest> commit(const Plan& plan, const std::vector<int32_t>& sampled);
    // Requests that ended without a step (max_new_tokens == 0, abort, cache failure).
    std::vector<FinishedRequest> drain_finished();

    const SchedulerStats& stats() const { return stats_; }
    // Output so far of a live request (empty if unknown).
    std::vector<int32_t> output_of(int64_t id) const;

private:
    struct Req {
        int64_t id = 0;
        std::vector<int32_t> tokens;   // prompt + generated
        int prompt_len = 0;
        int max_new = 0;
        std::set<int32_t> eos;
        int computed = 0;              // tokens whose keys and values are in the cache
        int slot = -1;
        long admitted_at = -1;         // order of admission among running requests
    };
    void finish(Req& r, const std::string& reason);
    void preempt(Req& r, Plan& plan);

    CacheManager* cache_;
    SchedulerConfig cfg_;
    std::deque<int64_t> waiting_;
    std::vector<int64_t> running_;     // in order of admission
    std::map<int64_t, Req> reqs_;
    std::vector<FinishedRequest> done_;
    SchedulerStats stats_;
    long admit_counter_ = 0;
};

}  // namespace dlm
