// The continuous-batching scheduler: which tokens of which requests run in the
// next step.  It decides; it runs no model.  The step function executes a plan and
// the caller reports the tokens picked from the wanted logits back with commit().
//
// Shape of one iteration, after the reference's Batch::step (src/serve/engine.rs:
// 1999-2181): running requests first get room for their next row (grow), then
// prompts are fed in portions under a token budget, oldest request first.
// When pages run out the youngest request holding a slot gives everything up and
// is fed again from position 0 later (preemption by recompute); the oldest request
// never yields (src/serve/engine.rs:2191-2276).
#pragma once

#include <cstdint>
#include <deque>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "cache_manager.h"

namespace axon {

struct SchedulerError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

struct SchedulerConfig {
    int max_batch_tokens = 2048;  // tokens per step: decode rows first, prompt portions after
    int max_running = 16;         // requests holding a slot at once (the reference's 16 slots)
    int prefill_chunk = 0;        // most prompt tokens of one request per step; 0 = the budget
};

enum class Phase { Waiting, Prefill, Decode, Finished };
enum class Finish { None, Stop, Length, Aborted };

struct Request {
    int64_t id = 0;
    std::vector<int32_t> tokens;  // prompt, then what was generated
    int prompt_len = 0;
    int max_new = 0;
    std::vector<int32_t> stop;
    Phase phase = Phase::Waiting;
    Finish finish = Finish::None;
    int slot = -1;
    int fed = 0;        // positions of `tokens` that are in the cache
    int generated = 0;  // tokens decided so far
    uint64_t arrival = 0;
    int preemptions = 0;
};

struct PlanEntry {
    int64_t id = 0;
    int slot = -1;
    int start = 0;                // cache position of the first token
    std::vector<int32_t> tokens;  // what to run
    bool want_logits = false;     // the logits after the last token decide the next token
};

struct Plan {
    std::vector<PlanEntry> entries;
    std::vector<int64_t> preempted;  // requests that gave their pages up while planning
    int n_tokens = 0;
};

struct Done {
    int64_t id;
    Finish finish;
};

class Scheduler {
public:
    Scheduler(CacheManager* cache, SchedulerConfig cfg);

    // Queue a request.  Throws when it could never run: an empty prompt, more
    // positions than the cache allows, or more pages than the whole pool has.
    void add(int64_t id, std::vector<int32_t> prompt, int max_new, std::vector<int32_t> stop);
    void abort(int64_t id);

    Plan plan();
    // `picked`: for every entry of the plan that wanted logits, the token chosen from them.
    std::vector<Done> commit(const Plan& plan, const std::map<int64_t, int32_t>& picked);
    // The same with the picks in the order of the plan's entries that wanted logits.
    std::vector<Done> commit_in_order(const Plan& plan, const int32_t* picks, int n_picks);

    bool idle() const;  // nothing waiting, nothing running
    int n_waiting() const { return (int)waiting_.size(); }
    int n_running() const { return (int)running_.size(); }
    const Request& request(int64_t id) const;
    // Generated tokens of a request (stop token excluded); forgets a finished request.
    std::vector<int32_t> take_output(int64_t id);
    const SchedulerConfig& config() const { return cfg_; }

private:
    Request& get(int64_t id);
    bool preempt_youngest(int64_t grower);  // false: nobody else to take pages from
    void to_waiting(Request& r);
    int feedable(const Request& r, int want) const;

    CacheManager* cache_;
    SchedulerConfig cfg_;
    std::map<int64_t, Request> requests_;
    std::deque<int64_t> waiting_;   // by arrival
    std::vector<int64_t> running_;  // hold a slot (Prefill or Decode), by arrival
    uint64_t clock_ = 0;
};

}  // namespace axon
