/* CPU oracle, second restatement: bfp8/bfp4 pack and unpack at the byte level, in plain C.
 * TEST INFRASTRUCTURE ONLY: tests load the shared object built from this file to cross-check the
 * NumPy oracle and the CUDA kernels. The product never links or loads it.
 *
 * It follows the reference's own C fragments (paths inside the baretile project):
 *   nibble rounding        baretile/kernels.py:1074-1081
 *   bfp8 rounding          baretile/kernels.py:1108-1114
 *   run -> exponent+values baretile/kernels.py:1130-1138
 *   bfp4 tile loop         baretile/kernels.py:1547-1563
 *   decode                 baretile/kernels.py:1497-1512, baretile/tensor.py:1095-1104
 * A tile is 1024 datums as four row-major 16x16 faces; a run is 16 consecutive datums.
 */
#include <stdint.h>
#include <stddef.h>

static unsigned nibble_of(unsigned b, unsigned top) {
  unsigned e = b >> 7 & 255, shift = top - e, m = (b & 127) | (e ? 128u : 0u);
  unsigned q = shift < 4 ? (m + (16u << shift)) >> (shift + 5) : 0;
  if (q > 7) q = 7;
  return q ? (b >> 15 & 1) << 3 | q : 0;
}

/* fmt: 8 or 4. in: n tiles of 1024 bf16 bit patterns. out: n tiles of 1088 or 576 bytes. */
int oracle_pack(int fmt, const uint16_t *in, uint8_t *out, size_t n) {
  if (fmt != 8 && fmt != 4) return 1;
  size_t tb = fmt == 8 ? 1088 : 576;
  for (size_t t = 0; t < n; t++) {
    const uint16_t *v = in + t * 1024;
    uint8_t *o = out + t * tb;
    for (unsigned r = 0; r < 64; r++) {
      unsigned top = 0;
      for (unsigned k = 0; k < 16; k++) { unsigned e = v[16 * r + k] >> 7 & 255; if (e > top) top = e; }
      o[r] = (uint8_t)top;
      for (unsigned k = 0; k < 16; k++) {
        unsigned b = v[16 * r + k];
        if (fmt == 8) {
          unsigned e = b >> 7 & 255, m = (b & 127) | (e ? 128u : 0u), shift = top - e < 8 ? top - e : 8;
          unsigned q = (m + (1u << shift)) >> (shift + 1);
          if (q > 127) q = 127;
          o[64 + 16 * r + k] = (uint8_t)(q ? (b >> 15) << 7 | q : 0);
        } else if (k % 2 == 0) {
          o[64 + 8 * r + k / 2] = (uint8_t)(nibble_of(b, top) | nibble_of(v[16 * r + k + 1], top) << 4);
        }
      }
    }
  }
  return 0;
}

int oracle_unpack(int fmt, const uint8_t *in, uint16_t *out, size_t n) {
  if (fmt != 8 && fmt != 4) return 1;
  size_t tb = fmt == 8 ? 1088 : 576;
  for (size_t t = 0; t < n; t++) {
    const uint8_t *i = in + t * tb;
    for (unsigned q = 0; q < 1024; q++) {
      unsigned x = fmt == 8 ? i[64 + q] : ((unsigned)(i[64 + q / 2] >> (4 * (q % 2))) & 15u) << 4;
      unsigned e = i[q / 16], v = x >> 7 ? 0xff80u : 0u;
      if (x & 127) {
        unsigned m = (x & 127) << 1, shift = 0;
        while (!(m & 128)) { m <<= 1; shift++; }
        v = (x >> 7) << 15 | ((e - shift) & 255) << 7 | (m & 126);
      }
      out[t * 1024 + q] = (uint16_t)v;
    }
  }
  return 0;
}
