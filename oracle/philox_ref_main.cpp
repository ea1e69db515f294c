// Prints word 0 of the reference's own Philox4x32-10 for the Philox
// known-answer fixture.  Compiled against the reference header where it lies
// (see Makefile, target _ref/philox_ref); the header itself is not copied.
//
// usage: philox_ref <seed> <first_counter> <count>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "src/custom_kernels/cuda/philox.h"

int main(int argc, char** argv) {
  if (argc != 4) return 2;
  const uint64_t seed = strtoull(argv[1], nullptr, 0);
  const uint64_t first = strtoull(argv[2], nullptr, 0);
  const uint64_t count = strtoull(argv[3], nullptr, 0);
  for (uint64_t i = 0; i < count; ++i) {
    aether::Philox4 counter = {{static_cast<uint32_t>(first + i), 0u, 0u, 0u}};
    aether::Philox4 out = aether::Philox4x32(counter, static_cast<uint32_t>(seed),
                                             static_cast<uint32_t>(seed >> 32));
    printf("%u\n", out.v[0]);
  }
  return 0;
}
