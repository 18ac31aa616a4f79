// Host runtime of the engine: the page pool, per-request block tables for
// groups of layers with different needs, state slots, and the
// continuous-batching scheduler above them.
//
// Shape of the reference it restates (not its code):
//   crates/ai-engine-candle/src/paged/block_table.rs:5-59  — LIFO free list that hands
//     out low ids first, ceil(n / page) pages for n tokens, growth that takes all
//     pages or none, release of every page, locate(pos) = (table[pos / P], pos % P);
//   crates/ai-engine-candle/src/paged/engine.rs:62-237 — admit while a sequence slot is
//     free, one token per running sequence per step, finish on EOS or max_tokens,
//     give pages back on finish.
// Beyond it: several page groups (all keys / a window of keys) with pages of
// their own, pages given back once a window has passed them, prompts cut into
// portions under a token budget and batched with decoded tokens, and
// preemption (recompute later) instead of failing a request when pages run out.
#pragma once
#include <algorithm>
#include <cstdint>
#include <deque>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace aie {

// ---------------------------------------------------------------------------
class PagePool {
 public:
    explicit PagePool(int num_pages) : held_(num_pages, 0) {
        if (num_pages < 0) throw std::invalid_argument("PagePool: negative page count");
        free_.reserve(num_pages);
        for (int i = num_pages - 1; i >= 0; --i) free_.push_back(i);  // low ids leave first
    }
    int num_pages() const { return (int)held_.size(); }
    int free_count() const { return (int)free_.size(); }
    int in_use() const { return num_pages() - free_count(); }
    int high_water() const { return high_water_; }
    long long total_allocations() const { return total_allocs_; }
    bool is_held(int id) const { return id >= 0 && id < num_pages() && held_[id]; }

    // n pages or none
    bool alloc(int n, std::vector<int>& out) {
        if (n < 0) throw std::invalid_argument("PagePool::alloc: negative count");
        if (n > (int)free_.size()) return false;
        for (int i = 0; i < n; ++i) {
            int id = free_.back();
            free_.pop_back();
            held_[id] = 1;
            out.push_back(id);
        }
        total_allocs_ += n;
        high_water_ = std::max(high_water_, in_use());
        return true;
    }
    void release(int id) {
        if (id < 0 || id >= num_pages()) throw std::out_of_range("PagePool::release: page id " + std::to_string(id) + " outside the pool");
        if (!held_[id]) throw std::logic_error("PagePool::release: page " + std::to_string(id) + " freed twice");
        held_[id] = 0;
        free_.push_back(id);
    }

 private:
    std::vector<int> free_;
    std::vector<uint8_t> held_;
    int high_water_ = 0;
    long long total_allocs_ = 0;
};

// ---------------------------------------------------------------------------
struct GroupSpec {
    int page_size = 16;   // tokens per page
    int num_pages = 0;    // pages of this group's pool
    int window = 0;       // 0: every key is kept; w > 0: a query at p reads keys in (p - w, p]
};

struct SeqTable {
    std::vector<int> pages;  // by page index (pos / page_size); -1 once given back
    int first_live = 0;      // pages [first_live, pages.size()) are held
};

class CacheManager {
 public:
    CacheManager(std::vector<GroupSpec> groups, int max_seqs, int max_pages_per_seq)
        : groups_(std::move(groups)), max_seqs_(max_seqs), max_pages_per_seq_(max_pages_per_seq),
          slot_used_(max_seqs, 0) {
        if (max_seqs <= 0) throw std::invalid_argument("CacheManager: max_seqs must be positive");
        for (auto& g : groups_) {
            if (g.page_size <= 0) throw std::invalid_argument("CacheManager: page_size must be positive");
            if (g.window < 0) throw std::invalid_argument("CacheManager: negative window");
            pools_.emplace_back(g.num_pages);
            tables_.emplace_back(max_seqs);
        }
        for (int i = max_seqs - 1; i >= 0; --i) free_slots_.push_back(i);
    }
    int num_groups() const { return (int)groups_.size(); }
    const GroupSpec& group(int g) const { return groups_.at(g); }
    const PagePool& pool(int g) const { return pools_.at(g); }
    int max_seqs() const { return max_seqs_; }
    int max_pages_per_seq() const { return max_pages_per_seq_; }
    int free_slots() const { return (int)free_slots_.size(); }
    bool slot_live(int slot) const { return slot >= 0 && slot < max_seqs_ && slot_used_[slot]; }

    // a state slot (also the row of the request's block tables); -1 when none is free
    int admit() {
        if (free_slots_.empty()) return -1;
        int s = free_slots_.back();
        free_slots_.pop_back();
        slot_used_[s] = 1;
        return s;
    }

    // pages that ensure(slot, n_tokens) would take from group g
    int pages_missing(int g, int slot, int n_tokens) const {
        const auto& t = tables_[g][slot];
        int need_end = (n_tokens + groups_[g].page_size - 1) / groups_[g].page_size;
        return std::max(0, need_end - (int)t.pages.size());
    }

    // Most tokens (<= want) that slot can hold with the pages now free in every group.
    int tokens_that_fit(int slot, int want) const {
        check_slot(slot);
        int fit = want;
        for (int g = 0; g < num_groups(); ++g) {
            const auto& t = tables_[g][slot];
            long long cap = ((long long)t.pages.size() + pools_[g].free_count()) * groups_[g].page_size;
            cap = std::min<long long>(cap, (long long)max_pages_per_seq_ * groups_[g].page_size);
            fit = (int)std::min<long long>(fit, cap);
        }
        return std::max(fit, 0);
    }

    // Pages for tokens [0, n_tokens) in every group, or nothing at all.
    bool ensure(int slot, int n_tokens) {
        check_slot(slot);
        for (int g = 0; g < num_groups(); ++g) {
            int need_end = (n_tokens + groups_[g].page_size - 1) / groups_[g].page_size;
            if (need_end > max_pages_per_seq_) return false;
            if (pages_missing(g, slot, n_tokens) > pools_[g].free_count()) return false;
        }
        for (int g = 0; g < num_groups(); ++g) {
            int miss = pages_missing(g, slot, n_tokens);
            if (miss) pools_[g].alloc(miss, tables_[g][slot].pages);
        }
        return true;
    }

    // `computed` tokens are in the cache and every later query sits at >= computed:
    // window groups give back the pages that no later query can read.
    int advance(int slot, int computed) {
        check_slot(slot);
        int released = 0;
        for (int g = 0; g < num_groups(); ++g) {
            const int w = groups_[g].window;
            if (w <= 0) continue;
            const int first_key = std::max(0, computed - w + 1);
            auto& t = tables_[g][slot];
            const int stop = std::min<int>(first_key / groups_[g].page_size, (int)t.pages.size());
            for (int i = t.first_live; i < stop; ++i) {
                pools_[g].release(t.pages[i]);
                t.pages[i] = -1;
                ++released;
            }
            t.first_live = std::max(t.first_live, stop);
        }
        return released;
    }

    // every page of the request goes back; the slot stays taken
    void release_pages(int slot) {
        check_slot(slot);
        for (int g = 0; g < num_groups(); ++g) {
            auto& t = tables_[g][slot];
            for (int i = t.first_live; i < (int)t.pages.size(); ++i) pools_[g].release(t.pages[i]);
            t.pages.clear();
            t.first_live = 0;
        }
    }

    void finish(int slot) {
        release_pages(slot);
        slot_used_[slot] = 0;
        free_slots_.push_back(slot);
    }

    const std::vector<int>& pages(int g, int slot) const { return tables_.at(g).at(slot).pages; }
    int first_live(int g, int slot) const { return tables_.at(g).at(slot).first_live; }

    // rows of block tables for a batch: out[i * width + j] = page j of slots[i], -1 beyond
    void fill_block_table(int g, const int* slots, int n, int width, int32_t* out) const {
        for (int i = 0; i < n; ++i) {
            int32_t* row = out + (size_t)i * width;
            std::fill(row, row + width, -1);
            if (slots[i] < 0) continue;   // padding row
            check_slot(slots[i]);
            const auto& p = tables_[g][slots[i]].pages;
            const int m = std::min<int>(width, (int)p.size());
            for (int j = 0; j < m; ++j) row[j] = p[j];
        }
    }

    // Throws when a page is lost, held twice, or held while marked free.
    void check_invariants() const {
        for (int g = 0; g < num_groups(); ++g) {
            std::vector<int> owner(pools_[g].num_pages(), -1);
            int held = 0;
            for (int s = 0; s < max_seqs_; ++s) {
                const auto& t = tables_[g][s];
                if (!slot_used_[s] && !t.pages.empty())
                    throw std::logic_error("free slot " + std::to_string(s) + " still has pages");
                for (int i = 0; i < (int)t.pages.size(); ++i) {
                    const int p = t.pages[i];
                    if (i < t.first_live) {
                        if (p != -1) throw std::logic_error("page behind the window still listed");
                        continue;
                    }
                    if (p < 0 || p >= pools_[g].num_pages()) throw std::logic_error("table holds a page id outside the pool");
                    if (owner[p] != -1) throw std::logic_error("page " + std::to_string(p) + " held twice (slots " + std::to_string(owner[p]) + " and " + std::to_string(s) + ")");
                    if (!pools_[g].is_held(p)) throw std::logic_error("page " + std::to_string(p) + " is in a table and on the free list");
                    owner[p] = s;
                    ++held;
                }
            }
            if (held != pools_[g].in_use())
                throw std::logic_error("group " + std::to_string(g) + ": " + std::to_string(pools_[g].in_use() - held) + " pages lost (held by no request, not free)");
        }
    }

 private:
    void check_slot(int slot) const {
        if (slot < 0 || slot >= max_seqs_ || !slot_used_[slot])
            throw std::logic_error("CacheManager: slot " + std::to_string(slot) + " is not live");
    }
    std::vector<GroupSpec> groups_;
    int max_seqs_, max_pages_per_seq_;
    std::vector<PagePool> pools_;
    std::vector<std::vector<SeqTable>> tables_;  // [group][slot]
    std::vector<int> free_slots_;
    std::vector<uint8_t> slot_used_;
};

// ---------------------------------------------------------------------------
struct StepEntry {
    long long id;
    int slot;
    int start;      // tokens [start, start + n_tokens) of the request run in this step
    int n_tokens;
    bool sample;    // the portion ends at the last known token: its logits are wanted
};

struct StepPlan {
    std::vector<StepEntry> entries;
    std::vector<long long> preempted;  // ids put back in the queue in this call
    std::vector<long long> admitted;
};

struct SchedulerStats {
    long long steps = 0, prompt_tokens = 0, decode_tokens = 0, preemptions = 0, admitted = 0, finished = 0;
};

class Scheduler {
 public:
    Scheduler(CacheManager* cache, int max_num_seqs, int max_num_batched_tokens, int max_seq_len)
        : cache_(cache), max_num_seqs_(max_num_seqs), budget_(max_num_batched_tokens), max_seq_len_(max_seq_len) {
        if (max_num_batched_tokens <= 0) throw std::invalid_argument("Scheduler: token budget must be positive");
        if (max_num_seqs <= 0) throw std::invalid_argument("Scheduler: max_num_seqs must be positive");
    }

    // "" when queued; otherwise why the request can never run
    // (crates/ai-engine-candle/src/paged/engine.rs:190-201 rejects max_tokens == 0 and over-long prompts)
    std::string add(long long id, int prompt_len, int max_new) {
        if (reqs_.count(id)) return "request id already in use";
        if (prompt_len <= 0) return "empty prompt";
        if (max_new <= 0) return "max_tokens must be positive";
        if (prompt_len > max_seq_len_)
            return "prompt exceeds max context (" + std::to_string(prompt_len) + " > " + std::to_string(max_seq_len_) + ")";
        const int most = std::min(prompt_len + max_new - 1, max_seq_len_);  // tokens ever cached
        for (int g = 0; g < cache_->num_groups(); ++g) {
            const auto& gs = cache_->group(g);
            int held = most;
            if (gs.window > 0) held = std::min(most, gs.window + 2 * gs.page_size + std::min(budget_, most));
            const int pages = (held + gs.page_size - 1) / gs.page_size;
            if (pages > gs.num_pages || (most + gs.page_size - 1) / gs.page_size > cache_->max_pages_per_seq())
                return "request can never fit the cache (" + std::to_string(most) + " tokens need " + std::to_string(pages) + " pages of group " + std::to_string(g) + ", pool has " + std::to_string(gs.num_pages) + ")";
        }
        Req r;
        r.id = id; r.prompt_len = prompt_len; r.max_new = max_new; r.total = prompt_len;
        reqs_[id] = r;
        waiting_.push_back(id);
        return "";
    }

    bool has_work() const { return !waiting_.empty() || !running_.empty(); }
    int num_running() const { return (int)running_.size(); }
    int num_waiting() const { return (int)waiting_.size(); }
    const SchedulerStats& stats() const { return stats_; }

    StepPlan schedule() {
        StepPlan plan;
        int budget = budget_;
        bool preempted_any = false;
        // 1. decoded tokens of running requests, in admission order; 2. their prompt portions
        for (int pass = 0; pass < 2; ++pass) {
            for (size_t i = 0; i < running_.size();) {
                Req& r = reqs_.at(running_[i]);
                const int remaining = r.total - r.computed;
                const bool is_decode = remaining == 1 && r.generated > 0;
                if ((pass == 0) != is_decode || r.scheduled || budget == 0) { ++i; continue; }
                int n = std::min(remaining, budget);
                bool ok = false;
                while (true) {
                    if (cache_->ensure(r.slot, r.computed + n)) { ok = true; break; }
                    if (!is_decode) {   // a smaller portion may still fit
                        int fit = cache_->tokens_that_fit(r.slot, r.computed + n) - r.computed;
                        if (fit > 0 && cache_->ensure(r.slot, r.computed + fit)) { n = fit; ok = true; break; }
                    }
                    // pages ran out: the request admitted last gives way and is recomputed later
                    long long victim = running_.back();
                    preempt(victim, plan, budget);
                    preempted_any = true;
                    if (victim == r.id) break;
                }
                if (!ok) continue;   // r itself left running_: index i now names the next one
                Req& rr = reqs_.at(running_[i]);
                rr.scheduled = true;
                plan.entries.push_back({rr.id, rr.slot, rr.computed, n, rr.computed + n == rr.total});
                budget -= n;
                ++i;
            }
        }
        // 3. admit from the queue (FIFO; preempted requests wait at its front)
        while (!preempted_any && !waiting_.empty() && (int)running_.size() < max_num_seqs_ && budget > 0) {
            Req& r = reqs_.at(waiting_.front());
            int slot = cache_->admit();
            if (slot < 0) break;
            int n = std::min(r.total, budget);
            if (!cache_->ensure(slot, n)) {
                int fit = cache_->tokens_that_fit(slot, n);
                if (fit <= 0 || !cache_->ensure(slot, fit)) { cache_->finish(slot); break; }
                n = fit;
            }
            waiting_.pop_front();
            r.slot = slot; r.computed = 0; r.scheduled = true;
            running_.push_back(r.id);
            plan.admitted.push_back(r.id);
            ++stats_.admitted;
            plan.entries.push_back({r.id, slot, 0, n, n == r.total});
            budget -= n;
        }
        for (auto& e : plan.entries) reqs_.at(e.id).scheduled = false;
        if (!plan.entries.empty()) ++stats_.steps;
        return plan;
    }

    // The step ran: its tokens are in the cache; windows give pages back.
    void commit(const StepPlan& plan) {
        for (const auto& e : plan.entries) {
            auto it = reqs_.find(e.id);
            if (it == reqs_.end()) continue;
            Req& r = it->second;
            if (r.slot != e.slot || r.computed != e.start) throw std::logic_error("Scheduler::commit: plan does not match request " + std::to_string(e.id));
            r.computed += e.n_tokens;
            if (e.n_tokens == 1 && r.generated > 0 && e.sample) ++stats_.decode_tokens; else stats_.prompt_tokens += e.n_tokens;
            cache_->advance(r.slot, r.computed);
        }
    }

    // A token was sampled for `id`.  `stop`: the caller saw an end condition (EOS).
    // Returns true when the request is finished (its pages and slot are free again).
    bool on_token(long long id, bool stop) {
        Req& r = reqs_.at(id);
        r.total += 1;
        r.generated += 1;
        if (stop || r.generated >= r.max_new || r.total > max_seq_len_) {
            finish(id);
            return true;
        }
        return false;
    }

    void finish(long long id) {
        auto it = reqs_.find(id);
        if (it == reqs_.end()) return;
        Req& r = it->second;
        if (r.slot >= 0) {
            cache_->finish(r.slot);
            running_.erase(std::find(running_.begin(), running_.end(), id));
        } else {
            auto w = std::find(waiting_.begin(), waiting_.end(), id);
            if (w != waiting_.end()) waiting_.erase(w);
        }
        reqs_.erase(it);
        ++stats_.finished;
    }

    int computed(long long id) const { return reqs_.at(id).computed; }
    int generated(long long id) const { return reqs_.at(id).generated; }
    int slot(long long id) const { return reqs_.at(id).slot; }
    std::vector<long long> running() const { return running_; }
    std::vector<long long> waiting() const { return {waiting_.begin(), waiting_.end()}; }

 private:
    struct Req {
        long long id = 0;
        int prompt_len = 0, max_new = 0;
        int total = 0;      // known tokens: prompt + sampled so far
        int computed = 0;   // of these, in the cache
        int generated = 0;
        int slot = -1;
        bool scheduled = false;
    };

    void preempt(long long id, StepPlan& plan, int& budget) {
        Req& r = reqs_.at(id);
        for (auto it = plan.entries.begin(); it != plan.entries.end(); ++it)
            if (it->id == id) { budget += it->n_tokens; plan.entries.erase(it); break; }
        cache_->finish(r.slot);
        r.slot = -1; r.computed = 0; r.scheduled = false;
        running_.erase(std::find(running_.begin(), running_.end(), id));
        waiting_.push_front(id);
        plan.preempted.push_back(id);
        ++stats_.preemptions;
    }

    CacheManager* cache_;
    int max_num_seqs_, budget_, max_seq_len_;
    std::unordered_map<long long, Req> reqs_;
    std::vector<long long> running_;   // admission order
    std::deque<long long> waiting_;
    SchedulerStats stats_;
};

}  // namespace aie
