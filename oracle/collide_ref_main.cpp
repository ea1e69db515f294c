// Runs the reference's own inline collision functions (selection count, random
// words, pair collision) over a binary case file and writes the results, for
// the collision golden fixture.  Compiled against the reference headers where
// they lie (see Makefile, target _ref/collide_ref); no reference source is
// copied.  The per-cell loop is this harness's own: the reference keeps its
// loop in a .cu test, which does not compile without a GPU toolchain target.
//
// usage: collide_ref <in.bin> <out.bin>
// in : int32 num_cells, int32 padded, float selection_factor, float coefficient,
//      float exponent, uint64 seed, uint64 step, int32 cell_start[C+1],
//      float sigma_g_max[C], float velocity[3*padded]
// out: float velocity[3*padded], float sigma_g_max[C], int32 collisions[C]
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <vector>

#include "src/custom_kernels/cuda/dsmc_collide_tma.h"

int main(int argc, char** argv) {
  if (argc != 3) return 2;
  FILE* in = fopen(argv[1], "rb");
  if (!in) return 3;
  int32_t num_cells = 0, padded = 0;
  float factor = 0, coefficient = 0, exponent = 0;
  uint64_t seed = 0, step = 0;
  bool ok = fread(&num_cells, 4, 1, in) == 1 && fread(&padded, 4, 1, in) == 1 &&
            fread(&factor, 4, 1, in) == 1 && fread(&coefficient, 4, 1, in) == 1 &&
            fread(&exponent, 4, 1, in) == 1 && fread(&seed, 8, 1, in) == 1 &&
            fread(&step, 8, 1, in) == 1;
  if (!ok) return 4;
  std::vector<int32_t> cell_start(num_cells + 1);
  std::vector<float> sigma(num_cells), velocity(3 * static_cast<size_t>(padded));
  ok = fread(cell_start.data(), 4, cell_start.size(), in) == cell_start.size() &&
       fread(sigma.data(), 4, sigma.size(), in) == sigma.size() &&
       fread(velocity.data(), 4, velocity.size(), in) == velocity.size();
  fclose(in);
  if (!ok) return 4;
  aether::dsmc::CollideParams p;
  p.num_particles = cell_start[num_cells];
  p.padded_particles = padded;
  p.num_cells = num_cells;
  p.selection_factor = factor;
  p.gas = aether::dsmc::VhsGas{coefficient, exponent};
  p.seed = seed;
  p.step = step;
  std::vector<int32_t> collisions(num_cells, 0);
  for (int cell = 0; cell < num_cells; ++cell) {
    const int start = cell_start[cell], count = cell_start[cell + 1] - start;
    const float majorant = sigma[cell];
    const int selections = aether::dsmc::NtcSelections(
        count, majorant, factor,
        aether::UniformFloat(aether::dsmc::CollisionRandom(cell, aether::dsmc::kCellDraw, p).v[0]));
    float observed = 0.0f;
    for (int pair = 0; pair < selections; ++pair) {
      const size_t i = static_cast<size_t>(start) + 2 * pair;
      float a[3], b[3];
      for (int c = 0; c < 3; ++c) {
        a[c] = velocity[c * static_cast<size_t>(padded) + i];
        b[c] = velocity[c * static_cast<size_t>(padded) + i + 1];
      }
      float sigma_g = 0.0f;
      if (aether::dsmc::CollidePair(a, b, majorant, p.gas,
                                    aether::dsmc::CollisionRandom(cell, static_cast<uint32_t>(pair), p),
                                    &sigma_g)) {
        for (int c = 0; c < 3; ++c) {
          velocity[c * static_cast<size_t>(padded) + i] = a[c];
          velocity[c * static_cast<size_t>(padded) + i + 1] = b[c];
        }
        ++collisions[cell];
      }
      observed = std::max(observed, sigma_g);
    }
    sigma[cell] = std::max(majorant, observed);
  }
  FILE* out = fopen(argv[2], "wb");
  if (!out) return 5;
  fwrite(velocity.data(), 4, velocity.size(), out);
  fwrite(sigma.data(), 4, sigma.size(), out);
  fwrite(collisions.data(), 4, collisions.size(), out);
  fclose(out);
  return 0;
}
