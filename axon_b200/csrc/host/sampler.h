// The sampler's host half: top-p, min-p, temperature and the seeded draw over the
// candidates the device selected (repeat penalty and top-k happen there).
//
// Order and rules follow the reference (src/sample.rs:1-30): penalty -> top-k ->
// top-p -> min-p -> temperature -> draw, one uniform number per decided token from
// xoshiro256** seeded through splitmix64 (src/sample.rs:202-242).
#pragma once

#include <array>
#include <cstdint>
#include <vector>

namespace axon {

struct SampleConfig {
    float temp = 0.8f;            // > 0 (0 is greedy and never builds a sampler)
    int top_k = 40;               // 0 = off (every token)
    float top_p = 0.9f;           // >= 1 = off
    float min_p = 0.0f;           // 0 = off
    float repeat_penalty = 1.1f;  // 1 = off
    int repeat_last_n = 64;       // tokens the penalty looks back over; 0 = off
    uint64_t seed = 0;
};

class Rng {
public:
    explicit Rng(uint64_t seed);
    uint64_t next_u64();
    double uniform();  // [0, 1), 53 bits
    std::array<uint64_t, 4> state() const { return s_; }

private:
    std::array<uint64_t, 4> s_;
};

// How many of the candidates (best first) survive top-p then min-p: at least 1.
int kept(const SampleConfig& c, const float* logits, int n);
// The token that `u` in [0, 1) picks from the candidates.
int pick_at(const SampleConfig& c, const float* logits, const int32_t* ids, int n, double u);
// The distinct ids among the last `last_n` of `recent`, ascending.
std::vector<int32_t> penalty_ids(const std::vector<int32_t>& recent, int last_n);

class Sampler {
public:
    explicit Sampler(SampleConfig c) : cfg_(c), rng_(c.seed) {}
    const SampleConfig& config() const { return cfg_; }
    double uniform() { return rng_.uniform(); }
    // Takes exactly one number from the generator, always.
    int pick(const float* logits, const int32_t* ids, int n) { return pick_at(cfg_, logits, ids, n, rng_.uniform()); }

private:
    SampleConfig cfg_;
    Rng rng_;
};

}  // namespace axon
