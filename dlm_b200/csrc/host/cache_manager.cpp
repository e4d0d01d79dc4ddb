#include "cache_manager.hpp"

#include <algorithm>
#include <sstream>

namespace dlm {

namespace {
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline int align4(int x) { return (x + 3) & ~3; }
}  // namespace

CacheManager::CacheManager(std::vector<GroupSpec> groups, int num_slots) : groups_(std::move(groups)) {
    if (num_slots <= 0) throw std::invalid_argument("num_slots must be > 0");
    for (size_t g = 0; g < groups_.size(); ++g) {
        const GroupSpec& s = groups_[g];
        if (s.page_size <= 0) throw std::invalid_argument("page_size must be > 0");
        if (s.window < 0) throw std::invalid_argument("window must be >= 0");
        if (s.num_pages < 0) throw std::invalid_argument("num_pages must be >= 0");
        std::vector<int32_t> fl(s.num_pages);
        // low ids are handed out first: the stack's top is page 0
        for (int i = 0; i < s.num_pages; ++i) fl[i] = s.num_pages - 1 - i;
        free_.push_back(std::move(fl));
        high_water_.push_back(0);
    }
    slots_.resize(num_slots);
    for (int i = num_slots - 1; i >= 0; --i) free_slots_.push_back(i);
}

int CacheManager::open() {
    if (free_slots_.empty()) return -1;
    int s = free_slots_.back();
    free_slots_.pop_back();
    Slot& sl = slots_[s];
    sl.open = true;
    sl.length = 0;
    sl.tables.assign(groups_.size(), {});
    sl.first_live.assign(groups_.size(), 0);
    return s;
}

bool CacheManager::is_open(int slot) const {
    return slot >= 0 && slot < (int)slots_.size() && slots_[slot].open;
}

void CacheManager::close(int slot) {
    if (!is_open(slot)) throw std::invalid_argument("close: slot " + std::to_string(slot) + " is not open");
    Slot& sl = slots_[slot];
    for (size_t g = 0; g < groups_.size(); ++g) {
        for (int32_t p : sl.tables[g])
            if (p >= 0) free_[g].push_back(p);
        sl.tables[g].clear();
    }
    sl.open = false;
    sl.length = 0;
    free_slots_.push_back(slot);
}

int CacheManager::length(int slot) const {
    if (!is_open(slot)) throw std::invalid_argument("length: slot " + std::to_string(slot) + " is not open");
    return slots_[slot].length;
}

int CacheManager::first_needed_page(int g, int next_pos) const {
    const GroupSpec& s = groups_[g];
    if (s.window == 0) return 0;
    int lo = next_pos - s.window + 1;
    if (lo < 0) lo = 0;
    return lo / s.page_size;
}

std::vector<int> CacheManager::pages_needed(int slot, int n) const {
    if (!is_open(slot)) throw std::invalid_argument("pages_needed: slot is not open");
    if (n < 0) throw std::invalid_argument("pages_needed: n must be >= 0");
    const Slot& sl = slots_[slot];
    std::vector<int> need(groups_.size(), 0);
    for (size_t g = 0; g < groups_.size(); ++g) {
        const int ps = groups_[g].page_size;
        const int have = (int)sl.tables[g].size();
        const int total = ceil_div(sl.length + n, ps);
        int take = std::max(0, total - have);
        int give = 0;
        if (n > 0) {
            const int upto = std::min(first_needed_page((int)g, sl.length), have);
            for (int i = sl.first_live[g]; i < upto; ++i)
                if (sl.tables[g][i] >= 0) ++give;
        }
        need[g] = take - give;
    }
    return need;
}

bool CacheManager::can_append(const std::vector<std::pair<int, int>>& slot_and_n) const {
    std::vector<long> sum(groups_.size(), 0);
    for (auto& sn : slot_and_n) {
        auto need = pages_needed(sn.first, sn.second);
        for (size_t g = 0; g < groups_.size(); ++g) sum[g] += need[g];
    }
    for (size_t g = 0; g < groups_.size(); ++g)
        if (sum[g] > (long)free_[g].size()) return false;
    return true;
}

int CacheManager::max_appendable(int slot, int n, int reserve) const {
    if (n <= 0) return 0;
    auto fits = [&](int m) {
        auto need = pages_needed(slot, m);
        for (size_t g = 0; g < groups_.size(); ++g)
            if (need[g] > (int)free_[g].size() - reserve) return false;
        return true;
    };
    if (fits(n)) return n;
    int lo = 0, hi = n;   // fits(lo) is true for lo == 0 only if nothing is needed; treat 0 as the floor
    while (hi - lo > 1) {
        int mid = lo + (hi - lo) / 2;
        if (fits(mid)) lo = mid; else hi = mid;
    }
    return lo;
}

void CacheManager::append(const std::vector<std::pair<int, int>>& slot_and_n) {
    // check first, so that a failure leaves everything as it was
    std::vector<long> sum(groups_.size(), 0);
    for (auto& sn : slot_and_n) {
        auto need = pages_needed(sn.first, sn.second);
        for (size_t g = 0; g < groups_.size(); ++g) sum[g] += need[g];
    }
    for (size_t g = 0; g < groups_.size(); ++g)
        if (sum[g] > (long)free_[g].size())
            throw CacheExhausted((int)g, (int)sum[g], (int)free_[g].size(), groups_[g].num_pages);
    // give back what windows have passed, for every request of the step, before any page is taken
    for (auto& sn : slot_and_n) {
        if (sn.second <= 0) continue;
        Slot& sl = slots_[sn.first];
        for (size_t g = 0; g < groups_.size(); ++g) {
            const int upto = std::min(first_needed_page((int)g, sl.length), (int)sl.tables[g].size());
            for (int i = sl.first_live[g]; i < upto; ++i) {
                if (sl.tables[g][i] >= 0) {
                    free_[g].push_back(sl.tables[g][i]);
                    sl.tables[g][i] = -1;
                }
            }
            if (upto > sl.first_live[g]) sl.first_live[g] = upto;
        }
    }
    for (auto& sn : slot_and_n) {
        if (sn.second <= 0) continue;
        Slot& sl = slots_[sn.first];
        sl.length += sn.second;
        for (size_t g = 0; g < groups_.size(); ++g) {
            const int total = ceil_div(sl.length, groups_[g].page_size);
            while ((int)sl.tables[g].size() < total) {
                if (free_[g].empty()) throw std::logic_error("free list ran dry after a passed check");
                sl.tables[g].push_back(free_[g].back());
                free_[g].pop_back();
            }
            const int used = groups_[g].num_pages - (int)free_[g].size();
            if (used > high_water_[g]) high_water_[g] = used;
        }
    }
}

const std::vector<int32_t>& CacheManager::table(int slot, int g) const {
    if (!is_open(slot)) throw std::invalid_argument("table: slot is not open");
    return slots_[slot].tables.at(g);
}

GroupStats CacheManager::stats(int g) const {
    GroupStats st;
    st.total_pages = groups_.at(g).num_pages;
    st.free_pages = (int)free_[g].size();
    st.used_pages = st.total_pages - st.free_pages;
    st.high_water = high_water_[g];
    return st;
}

StepLayout CacheManager::plan_layout(const std::vector<StepItem>& items, int min_table_width, int pad_requests) const {
    StepLayout lay;
    lay.num_groups = (int)groups_.size();
    lay.num_requests = (int)items.size();
    const int padded = std::max(0, pad_requests - (int)items.size());
    lay.num_requests += padded;
    lay.num_tokens += padded;
    lay.num_single += padded;
    lay.num_wanted += padded;
    if (padded > 0) {
        lay.max_q_len = std::max(lay.max_q_len, 1);
        lay.max_kv_len = std::max(lay.max_kv_len, 1);
    }
    lay.table_width.assign(groups_.size(), 1);
    for (auto& it : items) {
        if (!is_open(it.slot)) throw std::invalid_argument("step item names a slot that is not open");
        const int q = (int)it.tokens.size();
        if (q <= 0) throw std::invalid_argument("step item without tokens");
        const int kv = slots_[it.slot].length;
        if (kv < q) throw std::invalid_argument("step item has more tokens than its request holds (append first)");
        for (int w : it.want)
            if (w < 0 || w >= q) throw std::invalid_argument("wanted place is outside the item's tokens");
        lay.num_tokens += q;
        if (q == 1) ++lay.num_single;
        lay.num_wanted += (int)it.want.size();
        lay.max_q_len = std::max(lay.max_q_len, q);
        lay.max_kv_len = std::max(lay.max_kv_len, kv);
        for (size_t g = 0; g < groups_.size(); ++g)
            lay.table_width[g] = std::max(lay.table_width[g], (int)slots_[it.slot].tables[g].size());
    }
    for (size_t g = 0; g < groups_.size(); ++g) {
        lay.table_width[g] = align4(lay.table_width[g]);
        if (min_table_width > 0) {
            if (lay.table_width[g] > align4(min_table_width))
                throw std::invalid_argument("a request needs a wider block table than the fixed width");
            lay.table_width[g] = align4(min_table_width);
        }
    }
    int off = 0;
    auto take = [&](int n) { int o = off; off += align4(n); return o; };
    lay.off_tokens = take(lay.num_tokens);
    lay.off_positions = take(lay.num_tokens);
    lay.off_token_req = take(lay.num_tokens);
    lay.off_cu_q = take(lay.num_requests + 1);
    lay.off_kv_len = take(lay.num_requests);
    lay.off_state_slot = take(lay.num_requests);
    lay.off_logit_rows = take(lay.num_wanted);
    for (size_t g = 0; g < groups_.size(); ++g) {
        lay.off_slots.push_back(take(lay.num_tokens));
        lay.off_table.push_back(take(lay.num_requests * lay.table_width[g]));
    }
    lay.total = off;
    return lay;
}

void CacheManager::pack(const std::vector<StepItem>& items, const StepLayout& lay, int32_t* out) const {
    std::fill(out, out + lay.total, 0);
    int t = 0, w = 0;
    for (int r = 0; r < (int)items.size(); ++r) {
        const StepItem& it = items[r];
        const Slot& sl = slots_[it.slot];
        const int q = (int)it.tokens.size();
        const int start = sl.length - q;
        out[lay.off_cu_q + r] = t;
        out[lay.off_kv_len + r] = sl.length;
        out[lay.off_state_slot + r] = it.slot;
        for (int wi : it.want) out[lay.off_logit_rows + w++] = t + wi;
        for (size_t g = 0; g < groups_.size(); ++g) {
            const int width = lay.table_width[g];
            int32_t* row = out + lay.off_table[g] + r * width;
            const auto& tab = sl.tables[g];
            for (int i = 0; i < width; ++i) row[i] = i < (int)tab.size() ? tab[i] : -1;
            const int ps = groups_[g].page_size;
            for (int j = 0; j < q; ++j) {
                const int pos = start + j;
                const int page = tab[pos / ps];
                if (page < 0) throw std::logic_error("a new token's page was already given back");
                out[lay.off_slots[g] + t + j] = page * ps + pos % ps;
            }
        }
        for (int j = 0; j < q; ++j) {
            out[lay.off_tokens + t + j] = it.tokens[j];
            out[lay.off_positions + t + j] = start + j;
            out[lay.off_token_req + t + j] = r;
        }
        t += q;
    }
    // rows that belong to nobody (see plan_layout)
    for (int r = (int)items.size(); r < lay.num_requests; ++r) {
        out[lay.off_cu_q + r] = t;
        out[lay.off_kv_len + r] = 1;
        out[lay.off_state_slot + r] = (int)slots_.size();
        out[lay.off_logit_rows + w++] = t;
        for (size_t g = 0; g < groups_.size(); ++g) {
            const int width = lay.table_width[g];
            int32_t* row = out + lay.off_table[g] + r * width;
            for (int i = 0; i < width; ++i) row[i] = -1;
            row[0] = groups_[g].num_pages;
            out[lay.off_slots[g] + t] = groups_[g].num_pages * groups_[g].page_size;
        }
        out[lay.off_tokens + t] = 0;
        out[lay.off_positions + t] = 0;
        out[lay.off_token_req + t] = r;
        ++t;
    }
    out[lay.off_cu_q + lay.num_requests] = t;
}

std::string CacheManager::check() const {
    for (size_t g = 0; g < groups_.size(); ++g) {
        std::vector<int> owner(groups_[g].num_pages, 0);
        for (int32_t p : free_[g]) {
            if (p < 0 || p >= groups_[g].num_pages) return "free list holds an id outside the pool";
            if (owner[p]++) return "page " + std::to_string(p) + " of group " + std::to_string(g) + " is free twice";
        }
        for (size_t s = 0; s < slots_.size(); ++s) {
            if (!slots_[s].open) continue;
            for (int32_t p : slots_[s].tables[g]) {
                if (p < 0) continue;
                if (p >= groups_[g].num_pages) return "a table holds an id outside the pool";
                if (owner[p]++)
                    return "page " + std::to_string(p) + " of group " + std::to_string(g) + " is held twice";
            }
        }
        for (int p = 0; p < groups_[g].num_pages; ++p)
            if (!owner[p]) return "page " + std::to_string(p) + " of group " + std::to_string(g) + " is lost";
    }
    std::vector<int> seen(slots_.size(), 0);
    for (int s : free_slots_) if (seen[s]++) return "slot free twice";
    for (size_t s = 0; s < slots_.size(); ++s)
        if (!slots_[s].open && !seen[s]) return "slot " + std::to_string(s) + " is lost";
    return "";
}

}  // namespace dlm
