// Seeded input generator shared by the tests and the benchmark's CPU-baseline leg.
// TEST INFRASTRUCTURE ONLY (see matmul_oracle.h).
//
// The workload definitions draw every tensor of a configuration from ONE
// std::mt19937 seeded with 0, in a fixed order, each tensor filled in memory
// order (column-major, minibatch outermost), with libstdc++'s
// std::uniform_real_distribution<float> or std::normal_distribution<float>.
// Those distributions are implementation-defined, so the generator is C++
// compiled against the same libstdc++ on every machine rather than a Python
// re-implementation.
#include <cstdint>
#include <random>

extern "C" {

// kind[i] == 0: uniform on [p0[i], p1[i]);  kind[i] == 1: normal(mean p0[i], sd p1[i]).
void oracle_mt19937_draw(std::uint32_t seed, int ntensors, const int *kind, const float *p0,
                         const float *p1, const std::uint64_t *count, float **out) {
  std::mt19937 rng(seed);
  for (int t = 0; t < ntensors; ++t) {
    float *dst = out[t];
    if (kind[t] == 0) {
      std::uniform_real_distribution<float> dist(p0[t], p1[t]);
      for (std::uint64_t i = 0; i < count[t]; ++i) dst[i] = dist(rng);
    } else {
      std::normal_distribution<float> dist(p0[t], p1[t]);
      for (std::uint64_t i = 0; i < count[t]; ++i) dst[i] = dist(rng);
    }
  }
}

}  // extern "C"
