#include "scheduler.hpp"

#include <algorithm>
#include <stdexcept>

namespace dlm {

Scheduler::Scheduler(CacheManager* cache, SchedulerConfig cfg) : cache_(cache), cfg_(cfg) {
    if (!cache_) throw std::invalid_argument("scheduler needs a cache manager");
    if (cfg_.max_step_tokens <= 0) throw std::invalid_argument("max_step_tokens must be > 0");
    if (cfg_.max_step_requests <= 0) throw std::invalid_argument("max_step_requests must be > 0");
    if (cfg_.max_context <= 0) throw std::invalid_argument("max_context must be > 0");
}

void Scheduler::submit(int64_t id, std::vector<int32_t> prompt, int max_new_tokens, std::vector<int32_t> eos) {
    if (reqs_.count(id)) throw std::invalid_argument("request id " + std::to_string(id) + " is already in use");
    if (prompt.empty()) throw std::invalid_argument("empty prompt");
    if (max_new_tokens < 0) throw std::invalid_argument("max_new_tokens must be >= 0");
    for (int32_t t : prompt) {
        if (t < 0 || (cfg_.vocab_size > 0 && t >= cfg_.vocab_size))
            throw std::invalid_argument("token id " + std::to_string(t) + " is outside the vocabulary of " +
                                        std::to_string(cfg_.vocab_size));
    }
    if ((int)prompt.size() >= cfg_.max_context && max_new_tokens > 0)
        throw std::invalid_argument("prompt of " + std::to_string(prompt.size()) +
                                    " tokens leaves no room in a context of " + std::to_string(cfg_.max_context));
    Req r;
    r.id = id;
    r.prompt_len = (int)prompt.size();
    r.tokens = std::move(prompt);
    r.max_new = std::min(max_new_tokens, cfg_.max_context - r.prompt_len);
    r.eos.insert(eos.begin(), eos.end());
    if (r.max_new <= 0) {
        done_.push_back({id, {}, "length"});
        ++stats_.finished;
        return;
    }
    reqs_.emplace(id, std::move(r));
    waiting_.push_back(id);
}

void Scheduler::finish(Req& r, const std::string& reason) {
    if (r.slot >= 0) cache_->close(r.slot);
    FinishedRequest f;
    f.id = r.id;
    f.output.assign(r.tokens.begin() + r.prompt_len, r.tokens.end());
    f.reason = reason;
    done_.push_back(std::move(f));
    ++stats_.finished;
    const int64_t id = r.id;
    running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
    waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
    reqs_.erase(id);
}

bool Scheduler::abort(int64_t id) {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) return false;
    finish(it->second, "abort");
    return true;
}

void Scheduler::preempt(Req& r, Plan& plan) {
    cache_->close(r.slot);
    r.slot = -1;
    r.computed = 0;
    r.admitted_at = -1;
    running_.erase(std::remove(running_.begin(), running_.end(), r.id), running_.end());
    waiting_.push_front(r.id);
    plan.preempted.push_back(r.id);
    ++stats_.preemptions;
}

Plan Scheduler::plan() {
    Plan plan;
    int budget = cfg_.max_step_tokens;
    int rows = 0;
    std::set<int64_t> planned;

    auto youngest_unplanned = [&]() -> int64_t {
        for (auto it = running_.rbegin(); it != running_.rend(); ++it)
            if (!planned.count(*it)) return *it;
        return -1;
    };
    // Makes room for `n` more tokens of `r` by pre-empting younger requests.  Returns false
    // when `r` itself had to go (pre-empted, or failed because it was alone).
    auto make_room = [&](Req& r, int n) -> bool {
        while (!cache_->can_append({{r.slot, n}})) {
            const int64_t victim = youngest_unplanned();
            if (victim < 0 || victim == r.id) {
                if (running_.size() == 1) {
                    plan.failed.push_back(r.id);
                    finish(r, "cache");
                } else {
                    preempt(r, plan);
                }
                return false;
            }
            preempt(reqs_.at(victim), plan);
        }
        return true;
    };

    // 1. decode rows, oldest first
    {
        const std::vector<int64_t> snapshot = running_;
        for (int64_t id : snapshot) {
            auto it = reqs_.find(id);
            if (it == reqs_.end() || it->second.slot < 0) continue;   // gone or pre-empted meanwhile
            Req& r = it->second;
            if ((int)r.tokens.size() - r.computed != 1) continue;
            if (budget < 1 || rows >= cfg_.max_step_requests) break;
            if (!make_room(r, 1)) continue;
            cache_->append({{r.slot, 1}});
            PlannedItem item;
            item.id = id; item.slot = r.slot; item.start = r.computed;
            item.tokens = {r.tokens.back()};
            item.sample = true;
            plan.items.push_back(std::move(item));
            planned.insert(id);
            --budget; ++rows;
        }
    }
    // 2. running requests still in their prompt, oldest first
    {
        const std::vector<int64_t> snapshot = running_;
        for (int64_t id : snapshot) {
            auto it = reqs_.find(id);
            if (it == reqs_.end() || it->second.slot < 0) continue;
            Req& r = it->second;
            const int pending = (int)r.tokens.size() - r.computed;
            if (pending <= 1 || planned.count(id)) continue;
            if (budget < 1 || rows >= cfg_.max_step_requests) break;
            int n = cache_->max_appendable(r.slot, std::min(pending, budget));
            if (n == 0) {
                if (!plan.items.empty()) continue;      // others make progress; wait for their pages
                if (!make_room(r, 1)) continue;         // nobody would move: the oldest must
                n = cache_->max_appendable(r.slot, std::min(pending, budget));
                if (n == 0) continue;
            }
            cache_->append({{r.slot, n}});
            PlannedItem item;
            item.id = id; item.slot = r.slot; item.start = r.computed;
            item.tokens.assign(r.tokens.begin() + r.computed, r.tokens.begin() + r.computed + n);
            item.sample = (r.computed + n == (int)r.tokens.size());
            plan.items.push_back(std::move(item));
            planned.insert(id);
            budget -= n; ++rows;
        }
    }
    // 3. admission, in arrival order; not in a step that had to pre-empt
    while (plan.preempted.empty() && !waiting_.empty() && budget > 0 && rows < cfg_.max_step_requests &&
           (int)running_.size() < cfg_.max_step_requests && cache_->free_slots() > 0) {
        Req& r = reqs_.at(waiting_.front());
        const int pending = (int)r.tokens.size() - r.computed;
        const int slot = cache_->open();
        const int reserve = (int)running_.size();
        int n = cache_->max_appendable(slot, std::min(pending, budget), reserve);
        // Beside running requests a prompt is admitted only if all of it fits in what is free now: a prompt
        // that gets its first portion and then has to give its pages back is computed twice.
        if (n > 0 && !running_.empty() && cache_->max_appendable(slot, pending, reserve) < pending) n = 0;
        if (n == 0) {
            cache_->close(slot);
            if (running_.empty() && plan.items.empty()) {   // an empty engine cannot hold one token of it
                plan.failed.push_back(r.id);
                finish(r, "cache");
                continue;
            }
            break;
        }
        waiting_.pop_front();
        r.slot = slot;
        r.admitted_at = admit_counter_++;
        running_.push_back(r.id);
        cache_->append({{slot, n}});
        PlannedItem item;
        item.id = r.id; item.slot = slot; item.start = 0;
        item.tokens.assign(r.tokens.begin(), r.tokens.begin() + n);
        item.sample = (n == (int)r.tokens.size());
        plan.items.push_back(std::move(item));
        planned.insert(r.id);
        budget -= n; ++rows;
    }
    return plan;
}

std::vector<FinishedRequest> Scheduler::commit(const Plan& plan, const std::vector<int32_t>& sampled) {
    size_t k = 0;
    size_t want = 0;
    for (auto& item : plan.items) want += item.sample ? 1 : 0;
    if (sampled.size() != want)
        throw std::invalid_argument("commit: expected " + std::to_string(want) + " sampled tokens, got " +
                                    std::to_string(sampled.size()));
    if (!plan.items.empty()) ++stats_.steps;
    for (auto& item : plan.items) {
        auto it = reqs_.find(item.id);
        if (it == reqs_.end()) { if (item.sample) ++k; continue; }   // aborted between plan and commit
        Req& r = it->second;
        const int n = (int)item.tokens.size();
        if (item.start < r.prompt_len) stats_.prompt_tokens += std::min(n, r.prompt_len - item.start);
        r.computed = item.start + n;
        if (!item.sample) continue;
        const int32_t tok = sampled[k++];
        r.tokens.push_back(tok);
        ++stats_.decode_tokens;
        const int generated = (int)r.tokens.size() - r.prompt_len;
        if (r.eos.count(tok)) finish(r, "eos");
        else if (generated >= r.max_new) finish(r, "length");
    }
    return drain_finished();
}

std::vector<FinishedRequest> Scheduler::drain_finished() {
    std::vector<FinishedRequest> out;
    out.swap(done_);
    return out;
}

std::vector<int32_t> Scheduler::output_of(int64_t id) const {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) return {};
    return std::vector<int32_t>(it->second.tokens.begin() + it->second.prompt_len, it->second.tokens.end());
}

}  // namespace dlm
