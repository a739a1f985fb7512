// CPU check of the rule that cuts a minibatch over the shards of a device group
// (primitiv_b200/device/batch_partition.h): for every shard count 1..16 and batch size 1..600 the
// ranges tile the batch in order without gaps, differ in size by at most one, and owner() inverts
// range().  Prints "ok <cases>" and exits 0, or the first violation and exits 1.
#include <cstdint>
#include <cstdio>

#include "batch_partition.h"

namespace bp = primitiv::devices::batch_partition;

int main() {
  unsigned long cases = 0;
  for (std::uint32_t g = 1; g <= 16; ++g) {
    for (std::uint32_t batch = 1; batch <= 600; ++batch) {
      const std::uint32_t n = bp::active(g, batch);
      if (batch == 1) {
        for (std::uint32_t r = 0; r < g; ++r) {
          std::uint32_t lo, hi;
          bp::range(g, 1, r, &lo, &hi);
          if (n != g || lo != 0 || hi != 1) { std::printf("replica rule broken: g %u r %u\n", g, r); return 1; }
        }
        ++cases;
        continue;
      }
      if (n != (batch < g ? batch : g)) { std::printf("active: g %u batch %u -> %u\n", g, batch, n); return 1; }
      std::uint32_t next = 0, smallest = batch, largest = 0;
      for (std::uint32_t r = 0; r < n; ++r) {
        std::uint32_t lo, hi;
        bp::range(g, batch, r, &lo, &hi);
        if (lo != next || hi <= lo) { std::printf("gap or empty: g %u batch %u r %u [%u,%u)\n", g, batch, r, lo, hi); return 1; }
        next = hi;
        if (hi - lo < smallest) smallest = hi - lo;
        if (hi - lo > largest) largest = hi - lo;
        for (std::uint32_t i = lo; i < hi; ++i)
          if (bp::owner(g, batch, i) != r) { std::printf("owner: g %u batch %u item %u\n", g, batch, i); return 1; }
      }
      if (next != batch || largest - smallest > 1) { std::printf("cover / balance: g %u batch %u\n", g, batch); return 1; }
      if (batch % g == 0) {  // the cut of functions::batch::split when it divides
        std::uint32_t lo, hi;
        bp::range(g, batch, g - 1, &lo, &hi);
        if (lo != (g - 1) * (batch / g) || hi != batch) { std::printf("even cut: g %u batch %u\n", g, batch); return 1; }
      }
      ++cases;
    }
  }
  std::printf("ok %lu\n", cases);
  return 0;
}
