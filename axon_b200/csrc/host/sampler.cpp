#include "sampler.h"

#include <algorithm>
#include <cmath>

namespace axon {

namespace {
uint64_t splitmix(uint64_t& s) {
    s += 0x9e3779b97f4a7c15ull;
    uint64_t z = s;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}
uint64_t rotl(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }
}  // namespace

Rng::Rng(uint64_t seed) {
    uint64_t s = seed;
    for (auto& v : s_) v = splitmix(s);
}

uint64_t Rng::next_u64() {
    const uint64_t r = rotl(s_[1] * 5, 7) * 9;
    const uint64_t t = s_[1] << 17;
    s_[2] ^= s_[0];
    s_[3] ^= s_[1];
    s_[1] ^= s_[2];
    s_[0] ^= s_[3];
    s_[2] ^= t;
    s_[3] = rotl(s_[3], 45);
    return r;
}

double Rng::uniform() { return (double)(next_u64() >> 11) * (1.0 / 9007199254740992.0); }

int kept(const SampleConfig& c, const float* logits, int n_in) {
    int n = 0;
    while (n < n_in && !std::isnan(logits[n])) ++n;
    const double l0 = (double)logits[0];
    if (n <= 1 || !std::isfinite(l0)) return 1;
    if (c.top_p < 1.0f) {
        // the smallest prefix whose softmax (temperature 1) mass reaches top_p
        std::vector<double> e(n);
        double z = 0.0;
        for (int i = 0; i < n; ++i) {
            e[i] = std::exp((double)logits[i] - l0);
            z += e[i];
        }
        double cum = 0.0;
        int keep = n;
        for (int i = 0; i < n; ++i) {
            cum += e[i] / z;
            if (cum >= (double)c.top_p) {
                keep = i + 1;
                break;
            }
        }
        n = keep;
    }
    if (c.min_p > 0.0f) {
        // p_i >= min_p * p_max, on logits: l_i >= l_0 + ln(min_p)
        const double lo = l0 + std::log((double)c.min_p);
        int keep = 0;
        while (keep < n && (double)logits[keep] >= lo) ++keep;
        n = std::max(keep, 1);
    }
    return n;
}

int pick_at(const SampleConfig& c, const float* logits, const int32_t* ids, int n_in, double u) {
    const int n = kept(c, logits, n_in);
    if (n == 1) return ids[0];
    const double l0 = (double)logits[0], t = (double)c.temp;
    std::vector<double> w(n);
    double z = 0.0;
    for (int i = 0; i < n; ++i) {
        w[i] = std::exp(((double)logits[i] - l0) / t);
        z += w[i];
    }
    // inverse CDF: the first i whose cumulative weight passes u * total; never a
    // zero-weight index
    const double target = std::min(u * z, std::nextafter(z, 0.0));
    double cum = 0.0;
    int last = 0;
    for (int i = 0; i < n; ++i) {
        if (w[i] > 0.0) last = i;
        cum += w[i];
        if (target < cum) return ids[i];
    }
    return ids[last];
}

std::vector<int32_t> penalty_ids(const std::vector<int32_t>& recent, int last_n) {
    const size_t n = recent.size();
    const size_t from = (last_n >= 0 && (size_t)last_n < n) ? n - (size_t)last_n : 0;
    std::vector<int32_t> w(recent.begin() + from, recent.end());
    std::sort(w.begin(), w.end());
    w.erase(std::unique(w.begin(), w.end()), w.end());
    return w;
}

}  // namespace axon
