// The streaming layout of block-float weights (what Tensor.columns() produces on this backend).
//
// A matrix of tr x tc tiles is stored as runs of kPanel tile columns. Inside a run the tiles go tile row by
// tile row, the run's tiles of one tile row side by side, so the tiles a CTA needs for consecutive K are one
// contiguous range. Inside a tile the 64 exponent bytes still come first, then the values, but both are
// permuted so that each lane of a warp fetches exactly the bytes of its MMA fragment with 128-bit loads, and the
// values are recoded, one to one, from sign and magnitude to offset binary:
//
//   exponents  position t*16 + face*4 + j             holds the exponent of datum row k = 4t + kk of face `face`,
//              j = 0, 2, 1, 3 for kk = 0, 1, 2, 3: a lane's word then has the exponents of its first k pair in bytes
//              0 and 2 and of its second pair in bytes 1 and 3, so one mask and one multiply-add turn each pair
//              into two bf16 scale lanes (scale_pair below)
//   bfp8       position 64 + h*512 + lane*16 + fs*8 + ns*4 + j
//              holds datum (k = 16h + 4t + kk, n = 16fs + 2g + ns), lane = 4g + t, as the byte 128 + v, where v
//              is the datum's signed 7-bit integer (the byte 0x80, "minus zero", which the packer never writes,
//              becomes 0 so that the recoding is one to one)
//   bfp4       position 64 + lane*16 + h*8 + fs*4 + j
//              holds the byte with datums (k = 16h + 4t + kk, n = 16fs + 2g) in its low nibble and (.., n + 1) in
//              its high nibble, each as 8 + v (the nibble 8 becomes 0)
//
// with face = 2h + fs, k the row (input channel) and n the column (output channel) inside the tile, and j the
// byte of the lane's word as above. Why offset binary: a byte zero-extended into a 16-bit lane IS the bf16 number
// byte * 2^-133 (subnormals run straight on into the first normal binade), so one mask or byte-permute per
// register puts two weights into bf16 lanes, and one packed fused multiply-add per register, with the face row's
// power of two and minus the offset times it, makes them the exact signed weights. Sign and magnitude would need a
// second mask and a permute per register, on the pipe the dequantisation saturates.
// Reading back (bt_relayout with to_stream = 0) restores every canonical byte: nothing is lost, duplicated or padded.
#pragma once
#include <cstddef>
#include <cstdint>
#include "../../include/baretile_b200.h"

namespace bt {

constexpr int kPanel = 4;  // tile columns in a run

// Position in the streamed tile of canonical byte c.
template <int FMT>
__host__ __device__ inline int stream_pos(int c) {
  if (c < 64) return (c % 16 / 4) * 16 + (c / 16) * 4 + ((c & 1) << 1 | (c >> 1 & 1));
  int i = c - 64;
  if (FMT == BT_BFP8) {
    int face = i / 256, k = i / 16 % 16, n = i % 16;
    int lane = (n / 2) * 4 + k / 4;
    return 64 + (face / 2) * 512 + lane * 16 + (face % 2) * 8 + (n % 2) * 4 + ((k & 1) << 1 | (k >> 1 & 1));
  }
  int face = i / 128, k = i / 8 % 16, g = i % 8;
  int lane = g * 4 + k / 4;
  return 64 + lane * 16 + (face / 2) * 8 + (face % 2) * 4 + ((k & 1) << 1 | (k >> 1 & 1));
}

// Sign and magnitude (sign in the top bit of BITS bits) <-> offset binary, one to one on all 2^BITS codes.
template <int BITS>
__host__ __device__ inline uint32_t to_offset(uint32_t b) {
  const uint32_t half = 1u << (BITS - 1), q = b & (half - 1);
  return b & half ? (q ? half - q : 0u) : half + q;
}
template <int BITS>
__host__ __device__ inline uint32_t from_offset(uint32_t u) {
  const uint32_t half = 1u << (BITS - 1);
  return u == 0 ? half : u >= half ? u - half : half | (half - u);
}
// A value byte (not an exponent) of a tile, canonical -> streamed coding and back.
template <int FMT>
__host__ __device__ inline uint32_t stream_code(uint32_t b) {
  return FMT == BT_BFP8 ? to_offset<8>(b) : to_offset<4>(b & 15) | to_offset<4>(b >> 4) << 4;
}
template <int FMT>
__host__ __device__ inline uint32_t canonical_code(uint32_t u) {
  return FMT == BT_BFP8 ? from_offset<8>(u) : from_offset<4>(u & 15) | from_offset<4>(u >> 4) << 4;
}

// The same recoding of four value bytes at once, canonical -> streamed. Per byte (per nibble for bfp4) the result is
// offset + q for a positive code and, for a negative one, (offset - q) without its top bit: offset - q for q = 1..,
// and 0 for "minus zero". No byte's (nibble's) subtraction borrows from its neighbour, since offset - q is never
// negative, so plain 32-bit arithmetic does for all lanes. `neg` is all ones in the bytes (nibbles) whose sign is set;
// on the device one byte permute in its sign-replicating form makes it.
template <int FMT>
__host__ __device__ inline uint32_t stream_code_word(uint32_t w) {
  if (FMT == BT_BFP8) {
    const uint32_t q = w & 0x7F7F7F7Fu;
    uint32_t neg;
#ifdef __CUDA_ARCH__
    asm("prmt.b32 %0, %1, 0, 0xBA98;" : "=r"(neg) : "r"(w));
#else
    neg = (w >> 7 & 0x01010101u) * 0xFFu;
#endif
    return ((q | 0x80808080u) & ~neg) | ((0x80808080u - q) & 0x7F7F7F7Fu & neg);
  }
  const uint32_t q = w & 0x77777777u, neg = (w >> 3 & 0x11111111u) * 0xFu;
  return ((q | 0x88888888u) & ~neg) | ((0x88888888u - q) & 0x77777777u & neg);
}

// And back, streamed -> canonical, four value bytes at once. Per byte (per nibble): offset + q becomes q, offset - q
// becomes sign | q (0x80 - u without its top bit, then the sign), and 0 becomes "minus zero", the sign alone, which
// the same expression gives (0x80 - 0 without its top bit is 0).
template <int FMT>
__host__ __device__ inline uint32_t canonical_code_word(uint32_t u) {
  if (FMT == BT_BFP8) {
    const uint32_t q = u & 0x7F7F7F7Fu;
    uint32_t pos;                                   // all ones in the bytes that hold a positive code (top bit set)
#ifdef __CUDA_ARCH__
    asm("prmt.b32 %0, %1, 0, 0xBA98;" : "=r"(pos) : "r"(u));
#else
    pos = (u >> 7 & 0x01010101u) * 0xFFu;
#endif
    return (q & pos) | ((((0x80808080u - q) & 0x7F7F7F7Fu) | 0x80808080u) & ~pos);
  }
  const uint32_t q = u & 0x77777777u, pos = (u >> 3 & 0x11111111u) * 0xFu;
  return (q & pos) | ((((0x88888888u - q) & 0x77777777u) | 0x88888888u) & ~pos);
}

#ifdef __CUDACC__
// bf16 lanes 2^(e - 64) for two exponent bytes of a lane's exponent word `ew`: bytes 0 and 2 (HI = 0, the lane's
// first k pair) or bytes 1 and 3 (HI = 1, its second pair). e << 7 is the exponent field, 0x1F80 = 63 << 7 the bias
// shift. Written as multiply-adds so that they run on the FMA pipe, which the dequantisation leaves mostly idle.
template <int HI>
__device__ __forceinline__ uint32_t scale_pair(uint32_t ew) {
  uint32_t s;
  if (HI) asm("mad.hi.u32 %0, %1, 0x80000000, 0x1F801F80;" : "=r"(s) : "r"(ew & 0xFF00FF00u));   // (bytes >> 1) + bias
  else asm("mad.lo.u32 %0, %1, 128, 0x1F801F80;" : "=r"(s) : "r"(ew & 0x00FF00FFu));
  return s;
}
#endif

// Index, in tiles, of tile (ti, tj) of a tr x tc matrix in the streamed order.
__host__ __device__ inline size_t stream_tile_index(int ti, int tj, int tr, int tc) {
  int run = tj / kPanel, width = tc - run * kPanel < kPanel ? tc - run * kPanel : kPanel;
  return (size_t)run * kPanel * tr + (size_t)ti * width + tj % kPanel;
}

}  // namespace bt
