#include "scheduler.h"

#include <algorithm>

namespace axon {

Scheduler::Scheduler(CacheManager* cache, SchedulerConfig cfg) : cache_(cache), cfg_(cfg) {
    if (!cache_) throw SchedulerError("the scheduler needs a cache manager");
    if (cfg_.max_running <= 0) throw SchedulerError("max_running must be positive");
    if (cfg_.max_running > cache_->max_slots())
        throw SchedulerError("max_running " + std::to_string(cfg_.max_running) + " exceeds the cache's " +
                             std::to_string(cache_->max_slots()) + " slots");
    if (cfg_.max_batch_tokens < cfg_.max_running)
        throw SchedulerError("the token budget must hold one decode token per running request");
    if (cfg_.prefill_chunk < 0) throw SchedulerError("prefill_chunk cannot be negative");
}

Request& Scheduler::get(int64_t id) {
    auto it = requests_.find(id);
    if (it == requests_.end()) throw SchedulerError("request " + std::to_string(id) + " is unknown");
    return it->second;
}

const Request& Scheduler::request(int64_t id) const {
    auto it = requests_.find(id);
    if (it == requests_.end()) throw SchedulerError("request " + std::to_string(id) + " is unknown");
    return it->second;
}

void Scheduler::add(int64_t id, std::vector<int32_t> prompt, int max_new, std::vector<int32_t> stop) {
    if (requests_.count(id)) throw SchedulerError("request " + std::to_string(id) + " exists already");
    if (prompt.empty()) throw SchedulerError("a request needs at least one prompt token");
    if (max_new < 1) throw SchedulerError("a request must ask for at least one token");
    const long long total = (long long)prompt.size() + max_new;
    if (total > cache_->max_positions())
        throw SchedulerError("prompt " + std::to_string(prompt.size()) + " + " + std::to_string(max_new) +
                             " tokens exceed the context of " + std::to_string(cache_->max_positions()));
    if (!cache_->could_ever_hold((int)total))
        throw SchedulerError("request " + std::to_string(id) + " needs more pages than the whole pool has");
    Request r;
    r.id = id;
    r.prompt_len = (int)prompt.size();
    r.tokens = std::move(prompt);
    r.max_new = max_new;
    r.stop = std::move(stop);
    r.arrival = ++clock_;
    requests_.emplace(id, std::move(r));
    waiting_.push_back(id);
}

void Scheduler::abort(int64_t id) {
    Request& r = get(id);
    if (r.slot >= 0) {
        cache_->close_slot(r.slot);
        running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
    } else {
        waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
    }
    r.slot = -1;
    r.phase = Phase::Finished;
    r.finish = Finish::Aborted;
}

bool Scheduler::idle() const { return waiting_.empty() && running_.empty(); }

void Scheduler::to_waiting(Request& r) {
    cache_->close_slot(r.slot);
    running_.erase(std::remove(running_.begin(), running_.end(), r.id), running_.end());
    r.slot = -1;
    r.fed = 0;
    r.phase = Phase::Waiting;
    ++r.preemptions;
    // back in line by arrival, so an old request is fed again before younger ones
    auto it = waiting_.begin();
    while (it != waiting_.end() && requests_.at(*it).arrival < r.arrival) ++it;
    waiting_.insert(it, r.id);
}

bool Scheduler::preempt_youngest(int64_t grower) {
    if (running_.empty()) return false;
    // running_ is kept by arrival: the youngest is last; the oldest never yields
    const int64_t victim = running_.back();
    if (running_.size() == 1 || victim == running_.front()) return false;
    (void)grower;
    to_waiting(get(victim));
    cache_->flush();
    return true;
}

int Scheduler::feedable(const Request& r, int want) const {
    // leave one page per decoding request for its growth (src/serve/engine.rs:1798-1813)
    int decoding = 0;
    for (int64_t id : running_)
        if (requests_.at(id).phase == Phase::Decode) ++decoding;
    const int reach = cache_->coverable(r.slot, decoding);
    return std::max(0, std::min(want, reach - r.fed));
}

Plan Scheduler::plan() {
    std::vector<int64_t> preempted;
    for (;;) {
        Plan p;
        cache_->flush();
        int budget = cfg_.max_batch_tokens;

        // 1. every decoding request gets room for its next row, oldest first
        const std::vector<int64_t> order = running_;
        for (int64_t id : order) {
            Request& r = get(id);
            if (r.phase != Phase::Decode || r.slot < 0) continue;
            if (budget == 0) break;
            while (r.slot >= 0 && !cache_->reserve(r.slot, r.fed + 1)) {
                const int64_t victim = running_.back();
                if (!preempt_youngest(id))
                    throw SchedulerError("stuck: request " + std::to_string(id) + " cannot grow and nobody can yield");
                preempted.push_back(victim);
            }
            if (r.slot < 0) continue;  // it was the youngest itself
            PlanEntry e;
            e.id = id;
            e.slot = r.slot;
            e.start = r.fed;
            e.tokens.assign(r.tokens.begin() + r.fed, r.tokens.end());
            e.want_logits = true;
            budget -= (int)e.tokens.size();
            p.n_tokens += (int)e.tokens.size();
            p.entries.push_back(std::move(e));
        }
        // drop entries of requests preempted after they were planned
        p.entries.erase(std::remove_if(p.entries.begin(), p.entries.end(),
                                       [&](const PlanEntry& e) { return requests_.at(e.id).slot != e.slot; }),
                        p.entries.end());
        p.n_tokens = 0;
        for (const PlanEntry& e : p.entries) p.n_tokens += (int)e.tokens.size();

        auto feed = [&](Request& r) {
            const int remaining = (int)r.tokens.size() - r.fed;
            int want = std::min(remaining, budget);
            if (cfg_.prefill_chunk > 0) want = std::min(want, cfg_.prefill_chunk);
            const int n = feedable(r, want);
            if (n <= 0) return;
            if (!cache_->reserve(r.slot, r.fed + n)) return;
            PlanEntry e;
            e.id = r.id;
            e.slot = r.slot;
            e.start = r.fed;
            e.tokens.assign(r.tokens.begin() + r.fed, r.tokens.begin() + r.fed + n);
            e.want_logits = (r.fed + n == (int)r.tokens.size());
            budget -= n;
            p.n_tokens += n;
            p.entries.push_back(std::move(e));
        };

        // 2. prompts that are being fed, oldest first
        for (int64_t id : running_) {
            if (budget == 0) break;
            Request& r = get(id);
            if (r.phase == Phase::Prefill) feed(r);
        }
        // 3. admit waiting requests in arrival order while a slot and the pages are there
        while (!waiting_.empty() && budget > 0 && (int)running_.size() < cfg_.max_running) {
            Request& r = get(waiting_.front());
            const int slot = cache_->open_slot();
            if (slot < 0) break;
            const int spare = (int)running_.size();  // headroom: a page for each request already running
            bool fits = true;
            for (int g = 0; g < cache_->n_groups(); ++g)
                if (cache_->free_pages(g) - cache_->pages_needed(g, slot, (int)r.tokens.size() + 1) < spare) fits = false;
            if (!fits) {
                cache_->close_slot(slot);
                break;  // first come first served: nobody jumps the queue
            }
            waiting_.pop_front();
            r.slot = slot;
            r.fed = 0;
            r.phase = Phase::Prefill;
            auto it = running_.begin();
            while (it != running_.end() && requests_.at(*it).arrival < r.arrival) ++it;
            running_.insert(it, r.id);
            feed(r);
        }

        if (!p.entries.empty() || idle()) {
            p.preempted = preempted;
            return p;
        }
        // Nothing could run although requests exist: prompts hold pages and none can go on.
        // The youngest gives its pages up; the oldest alone always fits (checked by add()).
        if (running_.size() > 1) {
            preempted.push_back(running_.back());
            preempt_youngest(running_.back());
            continue;
        }
        if (running_.empty() && !waiting_.empty())
            throw SchedulerError("stuck: request " + std::to_string(waiting_.front()) + " cannot be admitted into an empty cache");
        throw SchedulerError("stuck: request " + std::to_string(running_.front()) + " cannot go on");
    }
}

std::vector<Done> Scheduler::commit(const Plan& plan, const std::map<int64_t, int32_t>& picked) {
    std::vector<Done> done;
    for (const PlanEntry& e : plan.entries) {
        auto it = requests_.find(e.id);
        if (it == requests_.end() || it->second.slot != e.slot || it->second.phase == Phase::Finished) continue;
        Request& r = it->second;
        const int end = e.start + (int)e.tokens.size();
        cache_->commit(r.slot, end);
        r.fed = end;
        if (!e.want_logits) continue;
        auto pk = picked.find(e.id);
        if (pk == picked.end()) throw SchedulerError("no token was reported for request " + std::to_string(e.id));
        const int32_t tok = pk->second;
        Finish fin = Finish::None;
        if (std::find(r.stop.begin(), r.stop.end(), tok) != r.stop.end()) {
            fin = Finish::Stop;  // a stop token is not emitted (src/serve/engine.rs:2151-2169)
        } else {
            r.tokens.push_back(tok);
            ++r.generated;
            r.phase = Phase::Decode;
            if (r.generated >= r.max_new) fin = Finish::Length;
        }
        if (fin != Finish::None) {
            cache_->close_slot(r.slot);
            running_.erase(std::remove(running_.begin(), running_.end(), r.id), running_.end());
            r.slot = -1;
            r.phase = Phase::Finished;
            r.finish = fin;
            done.push_back({r.id, fin});
        }
    }
    return done;
}

std::vector<Done> Scheduler::commit_in_order(const Plan& plan, const int32_t* picks, int n_picks) {
    std::map<int64_t, int32_t> picked;
    int k = 0;
    for (const PlanEntry& e : plan.entries) {
        if (!e.want_logits) continue;
        if (k >= n_picks) throw SchedulerError("fewer tokens were reported than the plan's entries wanted");
        picked[e.id] = picks[k++];
    }
    if (k != n_picks) throw SchedulerError("more tokens were reported than the plan's entries wanted");
    return commit(plan, picked);
}

std::vector<int32_t> Scheduler::take_output(int64_t id) {
    Request& r = get(id);
    std::vector<int32_t> out(r.tokens.begin() + r.prompt_len, r.tokens.end());
    if (r.phase == Phase::Finished) requests_.erase(id);
    return out;
}

}  // namespace axon
