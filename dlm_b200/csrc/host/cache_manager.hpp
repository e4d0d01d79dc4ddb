// Page-pool bookkeeping for the key/value cache, and state slots.
//
// The manager owns no device memory.  It hands out page ids and slot ids; the
// Python side keeps the tensors those ids index.  Layers with the same cache
// needs form a *group*; each group has a pool of pages of its own and each
// request has one block table per group.  A group either keeps every key
// (window == 0) or only the last `window` positions; in the second case a page
// goes back to the pool as soon as no later query can see any of its positions.
//
// Behaviour mirrored from the reference's bookkeeping (src/cache/paged.rs):
// a LIFO free list that hands out low ids first (:117-126); growth that is
// atomic, so a failed request for pages changes nothing (:164-190); all of a
// request's pages given back at once when it ends (:193-197).
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace dlm {

struct GroupSpec {
    int page_size = 16;   // tokens per page
    int window = 0;       // 0: keep all keys; W > 0: a query at p sees keys j with p - j < W
    int num_pages = 0;    // pages in this group's pool
};

struct GroupStats {
    int total_pages = 0;
    int used_pages = 0;
    int free_pages = 0;
    int high_water = 0;   // most pages ever in use at once
};

struct CacheExhausted : std::runtime_error {
    int group, requested, free_pages, total_pages;
    CacheExhausted(int g, int req, int fr, int tot)
        : std::runtime_error("KV cache exhausted in group " + std::to_string(g) + ": requested " +
                             std::to_string(req) + " pages, " + std::to_string(fr) + " free of " +
                             std::to_string(tot)),
          group(g), requested(req), free_pages(fr), total_pages(tot) {}
};

// One (request, tokens) pair of a step, as the metadata packer sees it.
struct StepItem {
    int slot = -1;
    std::vector<int32_t> tokens;   // the next tokens of this request
    std::vector<int32_t> want;     // places among `tokens` whose logits are wanted
};

// Sizes of the packed metadata of a step (all counts in int32 elements).
struct StepLayout {
    int num_tokens = 0, num_requests = 0, num_wanted = 0, num_groups = 0;
    int max_q_len = 0, max_kv_len = 0;
    int num_single = 0;            // requests with exactly one token in this step
    std::vector<int> table_width;  // per group
    // offsets into the int32 buffer
    int off_tokens = 0, off_positions = 0, off_token_req = 0, off_cu_q = 0, off_kv_len = 0,
        off_state_slot = 0, off_logit_rows = 0;
    std::vector<int> off_slots, off_table;   // per group
    int total = 0;
};

class CacheManager {
public:
    CacheManager(std::vector<GroupSpec> groups, int num_slots);

    int num_groups() const { return (int)groups_.size(); }
    int num_slots() const { return (int)slots_.size(); }
    int free_slots() const { return (int)free_slots_.size(); }
    const GroupSpec& group(int g) const { return groups_.at(g); }

    // A request takes a state slot for its lifetime.  Returns -1 when none is free.
    int open();
    // Gives back the slot and every page the request still holds.
    void close(int slot);
    bool is_open(int slot) const;
    int length(int slot) const;

    // Pages each group would have to take from its pool to append n tokens to
    // `slot` now (pages a window has passed are counted as given back first).
    std::vector<int> pages_needed(int slot, int n) const;
    // Most tokens (<= n) that can be appended to `slot` with the pages free now
    // minus `reserve` pages kept back in every group.
    int max_appendable(int slot, int n, int reserve = 0) const;
    // Atomic over all pairs: either every request grows, or nothing changes and
    // CacheExhausted is thrown.  Window pages that no later query can see are
    // given back before new pages are taken.
    void append(const std::vector<std::pair<int, int>>& slot_and_n);
    bool can_append(const std::vector<std::pair<int, int>>& slot_and_n) const;

    // Block table of a request in one group, indexed by logical page; -1 marks a
    // page that was given back (or not yet taken).
    const std::vector<int32_t>& table(int slot, int g) const;
    GroupStats stats(int g) const;
    int free_pages(int g) const { return (int)free_[g].size(); }

    // Step metadata.  `plan_layout` sizes the buffer; `pack` fills it.  `pad_requests` > items.size() adds
    // rows that belong to nobody, so that steps of different numbers of requests share one layout (one
    // recorded graph): such a row brings one token (id 0, position 0), holds one key, writes it to the sink
    // page (the page after the pool's last, which the tensors have and the pool never hands out), uses the
    // sink state slot (index num_slots), and wants its logits like any row; the caller ignores them.  The
    // lengths of the requests must already include this step's tokens (append
    // first).  `min_table_width` > 0 forces a fixed width (for replayed graphs).
    StepLayout plan_layout(const std::vector<StepItem>& items, int min_table_width = 0, int pad_requests = 0) const;
    void pack(const std::vector<StepItem>& items, const StepLayout& lay, int32_t* out) const;

    // Consistency check used by tests: every page is either free or held by
    // exactly one request; returns a description of the first fault, or "".
    std::string check() const;

private:
    struct Slot {
        bool open = false;
        int length = 0;
        std::vector<std::vector<int32_t>> tables;   // per group, by logical page
        std::vector<int> first_live;                // per group: first logical page not given back
    };
    // first logical page that a query at position >= next_pos can still see
    int first_needed_page(int g, int next_pos) const;

    std::vector<GroupSpec> groups_;
    std::vector<std::vector<int32_t>> free_;   // per group LIFO
    std::vector<int> high_water_;
    std::vector<Slot> slots_;
    std::vector<int> free_slots_;
};

}  // namespace dlm
