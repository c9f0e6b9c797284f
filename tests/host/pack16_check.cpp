// Host check of the half-wise pack arithmetic (onebitsparsemul_b200/csrc/pack16.h) against the element-wise rules
// it must agree with: the 2:4 magnitude mask of mask24.h and the group encoder of formats.h. Prints three counts
// of disagreements (mask, metadata, signs) over seeded random chunks rich in ties, zeros, infinities and NaNs.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#define __device__
#define __forceinline__ inline
#include "mask24.h"
#undef __forceinline__
#define OB_HD inline
#include "formats.h"
#include "pack16.h"

static bool nonzero(uint16_t v) { return (v & 0x7fff) != 0; }
static bool positive(uint16_t v, unsigned lim) { const unsigned mag = v & 0x7fff; return !(v & 0x8000) && mag != 0 && mag <= lim; }
static uint16_t draw() {
  const int r = rand() % 10;
  if (r < 3) return rand() & 0xffff;
  if (r < 5) return (rand() & 1) << 15;                                   // +-0
  if (r < 6) return 0x7c00 | ((rand() & 1) << 15);                        // +-inf (fp16)
  if (r < 7) return 0x7c00 | (rand() & 0x3ff) | ((rand() & 1) << 15);     // NaN or inf
  if (r < 9) return (0x3c00 + (rand() & 3)) | ((rand() & 1) << 15);       // ties
  return rand() & 0x8003;                                                 // subnormals
}

int main(int argc, char** argv) {
  const long iters = argc > 1 ? atol(argv[1]) : 1000000;
  srand(7);
  long bad_mask = 0, bad_meta = 0, bad_signs = 0;
  for (long it = 0; it < iters; ++it) {
    uint16_t e[16];
    for (int t = 0; t < 16; ++t) e[t] = draw();
    const bool bf = it & 1, domask = !bf && (it & 2);
    const unsigned lim = bf ? 0x7f80 : 0x7c00;
    uint16_t ref[16];
    memcpy(ref, e, 32);
    uint32_t x[8];
    memcpy(x, e, 32);
    if (domask) {
      for (int g = 0; g < 4; ++g) {
        const unsigned keep = ob_keep_mask4(&ref[4 * g]);
        uint32_t k0, k1;
        ob_keep_group2(x[2 * g], x[2 * g + 1], k0, k1);
        const unsigned got = ((k0 >> 15) & 1) | (((k0 >> 31) & 1) << 1) | (((k1 >> 15) & 1) << 2) | (((k1 >> 31) & 1) << 3);
        if (got != keep) ++bad_mask;
        for (int t = 0; t < 4; ++t)
          if (!((keep >> t) & 1)) ref[4 * g + t] = ob_dropped_value(ref[4 * g + t]);
        ob_mask_group2(x[2 * g], x[2 * g + 1]);
      }
      if (memcmp(x, ref, 32)) { ++bad_mask; memcpy(x, ref, 32); }
    }
    unsigned meta = 0, signs = 0;
    for (int g = 0; g < 4; ++g) {
      const unsigned nib = ob_encode_group(nonzero(ref[4 * g]), nonzero(ref[4 * g + 1]), nonzero(ref[4 * g + 2]), nonzero(ref[4 * g + 3]));
      meta |= nib << (4 * g);
      const int i0 = nib & 3, i1 = nib >> 2;
      const uint16_t v0 = i0 == 0 ? ref[4 * g] : i0 == 1 ? ref[4 * g + 1] : ref[4 * g + 2];
      const uint16_t v1 = i1 == 1 ? ref[4 * g + 1] : i1 == 2 ? ref[4 * g + 2] : ref[4 * g + 3];
      signs |= (positive(v0, lim) ? 1u : 0u) << (2 * g);
      signs |= (positive(v1, lim) ? 1u : 0u) << (2 * g + 1);
    }
    uint32_t s0, s1;
    if (ob_encode_chunk16(x, bf ? 0x007f007fu : 0x03ff03ffu, s0, s1) != meta) ++bad_meta;
    const unsigned even = (signs & 1) | ((signs >> 1) & 2) | ((signs >> 2) & 4) | ((signs >> 3) & 8);
    const unsigned odd = ((signs >> 1) & 1) | ((signs >> 2) & 2) | ((signs >> 3) & 4) | ((signs >> 4) & 8);
    if (ob_plane_to_nibble(s0) != even || ob_plane_to_nibble(s1) != odd) ++bad_signs;
  }
  printf("%ld %ld %ld\n", bad_mask, bad_meta, bad_signs);
  return (bad_mask || bad_meta || bad_signs) ? 1 : 0;
}
