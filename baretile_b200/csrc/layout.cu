// Tile layout and block-float conversion kernels: the byte and integer work either side of the matmul.
// All of it is HBM-bound; every kernel moves 16 bytes per thread per access and touches each byte once.
#include "common.cuh"
#include "stream_layout.cuh"

using namespace bt;

namespace {

constexpr int kThreads = 256;
inline unsigned blocks_for(size_t items) { return (unsigned)((items + kThreads - 1) / kThreads); }

// ---- tilize / untilize ------------------------------------------------------------------------------------
// One thread moves half a run: 8 consecutive datums of a face row (16 bytes of bf16, 32 of fp32).
// Datum (r, c) of a tile is at (r / 16 * 2 + c / 16) * 256 + r % 16 * 16 + c % 16.
// WIDE: every row of the row-major side starts on a 16-byte boundary and cols is a multiple of 8, so the 8 datums
// move as whole 16-byte words.
template <typename T, bool WIDE>
__global__ void tilize_kernel(const T *__restrict__ src, T *__restrict__ dst, int batch, int rows, int cols, int tr, int tc) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;          // half-run index in the tiled image
  size_t total = (size_t)batch * tr * tc * 128;
  if (i >= total) return;
  size_t tile = i / 128;
  int h = (int)(i % 128), face = h / 32, r16 = h % 32 / 2, c8 = h % 2 * 8;
  int b = (int)(tile / ((size_t)tr * tc)), ti = (int)(tile / tc % tr), tj = (int)(tile % tc);
  int r = ti * 32 + face / 2 * 16 + r16, c0 = tj * 32 + face % 2 * 16 + c8;
  if (rows == 1) r = 0;                                              // a single row fills its tile
  __align__(16) T out[8];
  const T *row = src + ((size_t)b * rows + r) * cols;
  if (WIDE) {
#pragma unroll
    for (int k = 0; k < (int)(sizeof(out) / 16); k++)
      reinterpret_cast<uint4 *>(out)[k] = r < rows && c0 < cols ? reinterpret_cast<const uint4 *>(row + c0)[k] : make_uint4(0, 0, 0, 0);
  } else {
#pragma unroll
    for (int k = 0; k < 8; k++) {
      int c = cols == 1 ? 0 : c0 + k;                                // a single column repeats
      out[k] = (r < rows && c < cols) ? row[c] : T(0);
    }
  }
  uint4 *o = reinterpret_cast<uint4 *>(dst + i * 8);
#pragma unroll
  for (int k = 0; k < (int)(sizeof(out) / 16); k++) o[k] = reinterpret_cast<const uint4 *>(out)[k];
}

template <typename T, bool WIDE>
__global__ void untilize_kernel(const T *__restrict__ src, T *__restrict__ dst, int batch, int rows, int cols, int tr, int tc) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t total = (size_t)batch * tr * tc * 128;
  if (i >= total) return;
  size_t tile = i / 128;
  int h = (int)(i % 128), face = h / 32, r16 = h % 32 / 2, c8 = h % 2 * 8;
  int b = (int)(tile / ((size_t)tr * tc)), ti = (int)(tile / tc % tr), tj = (int)(tile % tc);
  int r = ti * 32 + face / 2 * 16 + r16, c0 = tj * 32 + face % 2 * 16 + c8;
  if (r >= rows) return;
  __align__(16) T in[8];
#pragma unroll
  for (int k = 0; k < (int)(sizeof(in) / 16); k++) reinterpret_cast<uint4 *>(in)[k] = reinterpret_cast<const uint4 *>(src + i * 8)[k];
  T *row = dst + ((size_t)b * rows + r) * cols;
  if (WIDE) {
    if (c0 < cols) {
#pragma unroll
      for (int k = 0; k < (int)(sizeof(in) / 16); k++) reinterpret_cast<uint4 *>(row + c0)[k] = reinterpret_cast<const uint4 *>(in)[k];
    }
  } else {
#pragma unroll
    for (int k = 0; k < 8; k++)
      if (c0 + k < cols) row[c0 + k] = in[k];
  }
}

// The wide case of both, for matrices of at least 8 tile columns: four half runs to a thread, all four loads issued
// before the first store (with 16 bytes in flight per thread an SM cannot hold enough threads to keep HBM busy), and no
// division: blockIdx.x is the tile row, blockIdx.z the matrix of the batch, and blockIdx.y * 1024 + k * 256 +
// threadIdx.x, k = 0..3, the half run within the tile row.
template <typename T, bool TILIZE>
__global__ void __launch_bounds__(kThreads) tile_wide_kernel(const T *__restrict__ src, T *__restrict__ dst, int batch, int rows, int cols, int tr, int tc) {
  constexpr int W = (int)sizeof(T) * 8 / 16;                           // 16-byte words of a half run
  const int ti = blockIdx.x;
  for (int b = blockIdx.z; b < batch; b += gridDim.z)
    for (int chunk = blockIdx.y; chunk * 1024 < tc * 128; chunk += gridDim.y) {
      uint4 v[4][W];
      const uint4 *from[4];
      uint4 *to[4];
      bool read[4], write[4];
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const int x = chunk * 1024 + k * kThreads + threadIdx.x, tj = x >> 7, h = x & 127, face = h / 32, r16 = h % 32 / 2, c8 = h % 2 * 8;
        int r = ti * 32 + face / 2 * 16 + r16;
        const int c0 = tj * 32 + face % 2 * 16 + c8;
        if (TILIZE && rows == 1) r = 0;                                // a single row fills its tile
        const bool inside = tj < tc, there = inside && r < rows && c0 < cols;
        const size_t rowmajor = ((size_t)b * rows + (there ? r : 0)) * cols + (there ? c0 : 0), tiled = (((size_t)b * tr + ti) * tc + (inside ? tj : 0)) * 1024 + h * 8;
        from[k] = reinterpret_cast<const uint4 *>(src + (TILIZE ? rowmajor : tiled));
        to[k] = reinterpret_cast<uint4 *>(dst + (TILIZE ? tiled : rowmajor));
        read[k] = there, write[k] = TILIZE ? inside : there;
      }
#pragma unroll
      for (int k = 0; k < 4; k++)
#pragma unroll
        for (int j = 0; j < W; j++) v[k][j] = read[k] ? from[k][j] : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int k = 0; k < 4; k++)
        if (write[k]) {
#pragma unroll
          for (int j = 0; j < W; j++) to[k][j] = v[k][j];
        }
    }
}
template <typename T, bool TILIZE>
void launch_tile_wide(const T *src, T *dst, int batch, int rows, int cols, int tr, int tc, cudaStream_t st) {
  const dim3 grid((unsigned)tr, (unsigned)min((tc * 128 + 1023) / 1024, 65535), (unsigned)min(batch, 65535));
  tile_wide_kernel<T, TILIZE><<<grid, kThreads, 0, st>>>(src, dst, batch, rows, cols, tr, tc);
}

// Many small matrices in one launch (a decode step's inputs on their way in, its results on their way out): the table
// travels by value with the launch, item k owns the half runs [first[k], first[k + 1]), and each thread does what a
// thread of tilize_kernel / untilize_kernel does for one matrix (batch 1). One launch instead of one per matrix: for
// matrices of a few tiles the launch is the cost.
constexpr int kManyMax = 64;
struct ManyArgs {
  const void *src[kManyMax];
  void *dst[kManyMax];
  int rows[kManyMax], cols[kManyMax], first[kManyMax + 1];
  int n;
};
template <typename T, bool TILIZE>
__global__ void many_kernel(const ManyArgs a) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= a.first[a.n]) return;
  int k = 0;
#pragma unroll
  for (int step = kManyMax / 2; step > 0; step /= 2)                   // the last item whose first half run is not past i
    if (k + step < a.n && i >= a.first[k + step]) k += step;
  const int rows = a.rows[k], cols = a.cols[k], tc = (cols + 31) / 32, h = i - a.first[k];
  const int tile = h / 128, in = h % 128, face = in / 32, r16 = in % 32 / 2, c8 = in % 2 * 8;
  int r = tile / tc * 32 + face / 2 * 16 + r16;
  const int c0 = tile % tc * 32 + face % 2 * 16 + c8;
  constexpr int W = (int)sizeof(T) * 8 / 16;                           // 16-byte words of a half run
  // rows that start on a 16-byte boundary and hold a multiple of 8 datums move as whole 16-byte words
  const bool wide = cols % 8 == 0 && (reinterpret_cast<uintptr_t>(TILIZE ? a.src[k] : a.dst[k]) & 15) == 0;
  __align__(16) T v[8];
  if (TILIZE) {
    if (rows == 1) r = 0;                                              // a single row fills its tile
    const T *row = static_cast<const T *>(a.src[k]) + (size_t)r * cols;
    if (wide) {
#pragma unroll
      for (int j = 0; j < W; j++) reinterpret_cast<uint4 *>(v)[j] = r < rows && c0 < cols ? reinterpret_cast<const uint4 *>(row + c0)[j] : make_uint4(0, 0, 0, 0);
    } else {
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const int c = cols == 1 ? 0 : c0 + j;                          // a single column repeats
        v[j] = (r < rows && c < cols) ? row[c] : T(0);
      }
    }
    uint4 *o = reinterpret_cast<uint4 *>(static_cast<T *>(a.dst[k]) + (size_t)h * 8);
#pragma unroll
    for (int j = 0; j < W; j++) o[j] = reinterpret_cast<const uint4 *>(v)[j];
  } else {
    if (r >= rows) return;
#pragma unroll
    for (int j = 0; j < W; j++) reinterpret_cast<uint4 *>(v)[j] = reinterpret_cast<const uint4 *>(static_cast<const T *>(a.src[k]) + (size_t)h * 8)[j];
    T *row = static_cast<T *>(a.dst[k]) + (size_t)r * cols;
    if (wide) {
      if (c0 < cols) {
#pragma unroll
        for (int j = 0; j < W; j++) reinterpret_cast<uint4 *>(row + c0)[j] = reinterpret_cast<const uint4 *>(v)[j];
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; j++)
        if (c0 + j < cols) row[c0 + j] = v[j];
    }
  }
}

// fp32 bits -> bf16 bits, round to nearest even; a NaN keeps a quiet payload.
__global__ void round_bf16_kernel(const uint32_t *__restrict__ src, uint16_t *__restrict__ dst, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint32_t b = src[i];
  dst[i] = (b & 0x7FFFFFFFu) > 0x7F800000u ? (uint16_t)(b >> 16 | 0x40) : (uint16_t)((b + 0x7FFFu + (b >> 16 & 1)) >> 16);
}

// ---- pack ---------------------------------------------------------------------------------------------------
// One thread packs one run: the 16 datums of a face row share their largest exponent field.
// bfp8: q = min((m + (1 << s)) >> (s + 1), 127) with s = min(top - e, 8); byte = q ? sign << 7 | q : 0.
// bfp4: q = s < 4 ? min((m + (16 << s)) >> (s + 5), 7) : 0; nibble = q ? sign << 3 | q : 0, even datum low.
// Packs the run in w (16 bf16 values, two to a word) into `values` (16 bytes for bfp8, the first 8 for bfp4) and
// returns the shared exponent.
template <int FMT>
__device__ __forceinline__ uint32_t pack_run(const uint32_t (&w)[8], uint32_t (&values)[4]) {
  // the largest exponent field of the 16 values: both halves of a word at once
  uint32_t both = w[0] & 0x7F807F80u;
#pragma unroll
  for (int k = 1; k < 8; k++) both = __vmaxu2(both, w[k] & 0x7F807F80u);
  const uint32_t top = max(both & 0xFFFFu, both >> 16) >> 7;
  if (top >= 9u && top < 255u) {
    // The rounding on the multiply-add pipe, which this kernel otherwise leaves idle while the integer pipe is what
    // bounds it: the magnitude kept is floor(|x| * 2^(133 - top) + 1/2) for bfp8 (2^(129 - top) for bfp4), and adding
    // 2^23 with rounding toward zero leaves that integer in the low byte. Equal to the integer formula below for every
    // bf16 pattern whenever the run's largest exponent field is 9..254 (checked exhaustively on the host); runs of
    // tiny numbers and runs with an infinity or a NaN take the integer formula itself. What follows the rounding
    // works on four values to a word: gather the magnitudes, clamp the one that can exceed the format (128 to 127, or 8
    // to 7), bring the sign bits over, and leave no sign on a zero magnitude (mag + 0x7F sets a byte's top bit exactly
    // when mag is not 0, and no byte carries into the next).
    const float scale = __uint_as_float(((FMT == BT_BFP8 ? 260u : 256u) - top) << 23);
    uint32_t bytes[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t a = w[2 * i], b = w[2 * i + 1];
      auto kept = [&](uint32_t bits) { return __float_as_uint(__fadd_rz(fmaf(fabsf(__uint_as_float(bits)), scale, 0.5f), 8388608.f)); };
      const uint32_t lo = __byte_perm(kept(a << 16), kept(a & 0xFFFF0000u), 0x4040), hi = __byte_perm(kept(b << 16), kept(b & 0xFFFF0000u), 0x4040);
      uint32_t mag = __byte_perm(lo, hi, 0x5410);
      const uint32_t sign = __byte_perm(a, b, 0x7531) & 0x80808080u;
      if (FMT == BT_BFP8) {
        mag -= mag >> 7 & 0x01010101u;
        bytes[i] = mag | (sign & (mag + 0x7F7F7F7Fu));
      } else {
        mag -= mag >> 3 & 0x01010101u;
        bytes[i] = mag | (sign >> 4 & (mag + 0x07070707u));
      }
    }
    if (FMT == BT_BFP8) {
#pragma unroll
      for (int i = 0; i < 4; i++) values[i] = bytes[i];
    } else {
      // four nibbles out of four bytes: b0 | b1 << 4 | b2 << 8 | b3 << 12
      auto squeeze = [](uint32_t v) {
        v = (v | v >> 4) & 0x00FF00FFu;
        return (v | v >> 8) & 0xFFFFu;
      };
      values[0] = squeeze(bytes[0]) | squeeze(bytes[1]) << 16;
      values[1] = squeeze(bytes[2]) | squeeze(bytes[3]) << 16;
      values[2] = values[3] = 0;
    }
    return top;
  }
  uint32_t q[16];
#pragma unroll
  for (int k = 0; k < 16; k++) {
    uint32_t b = (w[k / 2] >> (16 * (k % 2))) & 0xFFFFu, e = b >> 7 & 255u, m = (b & 127u) | (e ? 128u : 0u), d = top - e;
    if (FMT == BT_BFP8) {
      uint32_t s = min(d, 8u), v = min((m + (1u << s)) >> (s + 1), 127u);
      q[k] = v ? (b >> 15) << 7 | v : 0u;
    } else {
      uint32_t s = min(d, 4u), v = d < 4 ? min((m + (16u << s)) >> (s + 5), 7u) : 0u;
      q[k] = v ? (b >> 15) << 3 | v : 0u;
    }
  }
  if (FMT == BT_BFP8) {
#pragma unroll
    for (int i = 0; i < 4; i++) values[i] = q[4 * i] | q[4 * i + 1] << 8 | q[4 * i + 2] << 16 | q[4 * i + 3] << 24;
  } else {
#pragma unroll
    for (int i = 0; i < 2; i++)
      values[i] = q[8 * i] | q[8 * i + 1] << 4 | q[8 * i + 2] << 8 | q[8 * i + 3] << 12 | q[8 * i + 4] << 16 | q[8 * i + 5] << 20 | q[8 * i + 6] << 24 | q[8 * i + 7] << 28;
    values[2] = values[3] = 0;
  }
  return top;
}

// A thread packs two neighbouring runs: 64 bytes in with four 128-bit loads, the two exponents as one 16-bit store,
// the values as 32 (bfp8) or 16 (bfp4) bytes. (A tile has 64 runs, so a pair never straddles two tiles.)
template <int FMT>
__global__ void pack_kernel(const uint4 *__restrict__ src, uint8_t *__restrict__ dst, size_t pairs) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pairs) return;
  uint4 q[4];
#pragma unroll
  for (int k = 0; k < 4; k++) q[k] = src[4 * i + k];
  uint32_t v[2][4], top[2];
#pragma unroll
  for (int k = 0; k < 2; k++) {
    const uint32_t w[8] = {q[2 * k].x, q[2 * k].y, q[2 * k].z, q[2 * k].w, q[2 * k + 1].x, q[2 * k + 1].y, q[2 * k + 1].z, q[2 * k + 1].w};
    top[k] = pack_run<FMT>(w, v[k]);
  }
  constexpr size_t TB = tile_bytes(FMT);
  uint8_t *tile = dst + i / 32 * TB;
  int r = (int)(i % 32) * 2;
  *reinterpret_cast<uint16_t *>(tile + r) = (uint16_t)(top[0] | top[1] << 8);
  if (FMT == BT_BFP8) {
#pragma unroll
    for (int k = 0; k < 2; k++) *reinterpret_cast<uint4 *>(tile + 64 + (r + k) * 16) = make_uint4(v[k][0], v[k][1], v[k][2], v[k][3]);
  } else {
    *reinterpret_cast<uint4 *>(tile + 64 + r * 8) = make_uint4(v[0][0], v[0][1], v[1][0], v[1][1]);
  }
}

// ---- put: rows of x into rows of a tensor, in place (the packer's other user: a block-float KV cache) ----------
// One thread moves one run: the 16 datums of row i of x in one face of one tile column, to row ids[i] of the
// destination. Into a block float the run is packed exactly as a cast packs it. A row whose place is past the
// destination's last tile row is skipped; when several rows of x go to the same place the last one wins, so a
// thread whose place comes up again later in ids leaves its run alone. Distinct rows touch distinct bytes (a run's
// exponent, its values), so nothing is read back or merged. A destination of one logical row keeps that row in all
// 32 rows of its tile, so there every place inside the tile writes all 32 (and the last such row of x wins).
// ids is an int32 row in tile layout: place i is datum (0, i % 32) of tile i / 32.
// With many rows the search for a later row to the same place is what costs (every thread looks at every later
// place), so a caller may lend an int per row of the destination's tile rows: a first pass leaves there, for each
// place, the last row of x that goes to it (the array starts at -1), and the copy compares instead of searching.
__global__ void put_last_kernel(const int *__restrict__ ids, int n, int dst_tr, int single, int *__restrict__ last) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int p = ids[(size_t)(i / 32) * 1024 + (i % 32 / 16) * 256 + i % 16];
  if (p < 0 || p / 32 >= dst_tr) return;
  atomicMax(last + (single ? 0 : p), i);
}

template <int FMT>   // BT_BFP8, BT_BFP4, or an item size in bytes (2, 4 coded as -2, -4) for a plain copy
__global__ void put_kernel(uint8_t *__restrict__ dst, const uint8_t *__restrict__ x, const int *__restrict__ ids, int batch, int n, int tc,
                           int dst_tr, int x_tr, int single, const int *__restrict__ last) {
  const size_t unit = (size_t)blockIdx.x * blockDim.x + threadIdx.x;          // ((b * n + i) * tc + j) * 2 + f
  if (unit >= (size_t)batch * n * tc * 2) return;
  const int f = (int)(unit % 2), j = (int)(unit / 2 % tc), i = (int)(unit / 2 / tc % n), b = (int)(unit / 2 / tc / n);
  auto place = [&](int r) { return ids[(size_t)(r / 32) * 1024 + (r % 32 / 16) * 256 + r % 16]; };
  const int p = place(i);
  if (p < 0 || p / 32 >= dst_tr) return;
  if (last) {
    if (last[single ? 0 : p] != i) return;
  } else {
    for (int later = i + 1; later < n; later++) {
      const int q = place(later);
      if (single ? (unsigned)q < 32u : q == p) return;
    }
  }
  constexpr int ITEM = FMT < 0 ? -FMT : 2;                                    // bytes of a datum of x
  const size_t at_x = (size_t)((i % 32 / 16) * 2 + f) * 256 + (i % 16) * 16;  // first datum of the run in x's tile
  const uint8_t *src = x + (((size_t)b * x_tr + i / 32) * tc + j) * (1024 * ITEM) + at_x * ITEM;
  const size_t tile = ((size_t)b * dst_tr + p / 32) * tc + j;
  constexpr int BFP = FMT < 0 ? BT_BFP8 : FMT, TB = tile_bytes(BFP);
  uint4 raw[4];
  uint32_t v[4], top = 0;
  if (FMT < 0) {
#pragma unroll
    for (int k = 0; k < ITEM; k++) raw[k] = reinterpret_cast<const uint4 *>(src)[k];
  } else {
    const uint4 lo = reinterpret_cast<const uint4 *>(src)[0], hi = reinterpret_cast<const uint4 *>(src)[1];
    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    top = pack_run<BFP>(w, v);
  }
  for (int r = single ? 0 : p % 32, end = single ? 32 : r + 1; r < end; r++) {
    const int run = ((r / 16) * 2 + f) * 16 + r % 16;                         // which of the destination tile's 64 runs
    if (FMT < 0) {
      uint4 *to = reinterpret_cast<uint4 *>(dst + tile * (1024 * ITEM) + (size_t)run * 16 * ITEM);
#pragma unroll
      for (int k = 0; k < ITEM; k++) to[k] = raw[k];
    } else {
      uint8_t *t = dst + tile * TB;
      t[run] = (uint8_t)top;
      if (BFP == BT_BFP8) *reinterpret_cast<uint4 *>(t + 64 + run * 16) = make_uint4(v[0], v[1], v[2], v[3]);
      else *reinterpret_cast<uint2 *>(t + 64 + run * 8) = make_uint2(v[0], v[1]);
    }
  }
}

// ---- unpack --------------------------------------------------------------------------------------------------
// x = value byte (bfp4: nibble << 4). A zero magnitude is 0, or -inf (0xFF80) with the sign set. Otherwise the
// magnitude is normalised: m = (x & 127) << 1, s = 8 - bit_length(m), bf16 = sign | ((e - s) mod 256) << 7 | (m << s) & 0x7E.
__device__ __forceinline__ uint32_t decode_bfp(uint32_t x, uint32_t e) {
  uint32_t mag = x & 127u;
  if (!mag) return x >> 7 ? 0xFF80u : 0u;
  uint32_t m = mag << 1, s = __clz(m) - 24;     // 8 - bit_length(m)
  return (x >> 7) << 15 | ((e - s) & 255u) << 7 | ((m << s) & 0x7Eu);
}

// One run: the exponent byte e and the 16 value bytes in xb, four to a word (bfp4: each nibble moved to the top of a
// byte of its own), to 16 bf16 values in o, two to a word.
__device__ __forceinline__ void unpack_run(uint32_t e, const uint32_t (&xb)[4], uint32_t (&o)[8]) {
  if (e >= 7u && e <= 247u) {
    // The same values on the multiply-add pipe: a magnitude of up to 7 bits times 2^(e - 133) is exact in fp32 and needs
    // no rounding to bf16, so its upper half IS the normalised bf16 the integer formula builds (equal for every byte
    // whenever the exponent byte is 7..247, checked exhaustively on the host; outside that range the formula's
    // exponent wraps or overflows, and the formula itself runs). A byte permute puts a magnitude under 0x4B000000, the
    // float 2^23 + mag. What a sign adds is worked out four values to a word: `top`, the upper byte of a value's bf16,
    // gets 0x80 for a negative value and 0xFF for a signed zero magnitude, which reads as -inf, 0xFF80; `low`, the
    // lower byte, 0x80 for a signed zero (mag + 0x7F sets a byte's top bit exactly when mag is not 0); one byte permute
    // per pair of values interleaves them. (Asking the run first whether it has a signed zero at all, which a packer
    // never writes, and filling in only then, was slower: the branch costs more than the operations it saves.)
    const float scale = __uint_as_float((e - 6u) << 23);
#pragma unroll
    for (int k = 0; k < 8; k++) {
      const uint32_t x = xb[k / 2], mags = x & 0x7F7F7F7Fu;
      const uint32_t low = x & ~(mags + 0x7F7F7F7Fu) & 0x80808080u, top = (x & 0x80808080u) | (low - (low >> 7));
      const uint32_t a = k % 2 ? __byte_perm(mags, 0x4B000000u, 0x7442) : __byte_perm(mags, 0x4B000000u, 0x7440);
      const uint32_t b = k % 2 ? __byte_perm(mags, 0x4B000000u, 0x7443) : __byte_perm(mags, 0x4B000000u, 0x7441);
      const float fa = (__uint_as_float(a) - 8388608.f) * scale, fb = (__uint_as_float(b) - 8388608.f) * scale;
      const uint32_t both = __byte_perm(__float_as_uint(fa), __float_as_uint(fb), 0x7632);
      o[k] = both | (k % 2 ? __byte_perm(top, low, 0x3726) : __byte_perm(top, low, 0x1504));
    }
  } else {
#pragma unroll
    for (int k = 0; k < 8; k++) {
      const uint32_t lo = xb[k / 2] >> (16 * (k % 2)) & 255u, hi = xb[k / 2] >> (16 * (k % 2) + 8) & 255u;
      o[k] = decode_bfp(lo, e) | decode_bfp(hi, e) << 16;
    }
  }
}

// A thread unpacks one run: 64 consecutive bytes of a warp's output per store instruction pair (two runs to a thread,
// which serves the packer well, spreads a warp's stores over twice the lines and was slower here).
template <int FMT>
__global__ void unpack_kernel(const uint8_t *__restrict__ src, uint4 *__restrict__ dst, size_t runs) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= runs) return;
  constexpr size_t TB = tile_bytes(FMT);
  const uint8_t *tile = src + i / 64 * TB;
  int r = (int)(i % 64);
  uint32_t e = tile[r], xb[4], o[8];
  if (FMT == BT_BFP8) {
    uint4 v = *reinterpret_cast<const uint4 *>(tile + 64 + r * 16);
    xb[0] = v.x, xb[1] = v.y, xb[2] = v.z, xb[3] = v.w;
  } else {
    uint2 v = *reinterpret_cast<const uint2 *>(tile + 64 + r * 8);
    const uint32_t w[2] = {v.x, v.y};
#pragma unroll
    for (int k = 0; k < 2; k++) {
      const uint32_t even = (w[k] & 0x0F0F0F0Fu) << 4, odd = w[k] & 0xF0F0F0F0u;
      xb[2 * k] = __byte_perm(even, odd, 0x5140), xb[2 * k + 1] = __byte_perm(even, odd, 0x7362);
    }
  }
  unpack_run(e, xb, o);
  dst[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// ---- canonical <-> streaming layout ---------------------------------------------------------------------------
// Canonical -> streaming, the direction every weight takes once, without shared memory or barriers. The permutation
// moves bytes only inside a tile, and inside a tile only between the four datum rows 4t..4t+3 of a face (64
// contiguous bytes for bfp8, 32 for bfp4) and the pieces of the lanes 4g + t, g = 0..7. So one thread takes the
// rows 4t..4t+3 of a pair of faces (bfp8) or of all four faces (bfp4) with eight 128-bit loads, transposes them in
// registers with byte permutes, recodes a word at a time and writes the eight 16-byte pieces of the lanes 4g + t.
// The thread of datum rows 4t.. also writes the tile's exponent piece t: one word of each face's exponents, its bytes
// in the order 0, 2, 1, 3. blockIdx.y is the run of tile columns; a thread's unit is (tile of the run, h, t).
template <int FMT>
__global__ void __launch_bounds__(256) to_stream_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, int tr, int tc) {
  constexpr int TB = tile_bytes(FMT), UNITS = FMT == BT_BFP8 ? 8 : 4;
  const int run = blockIdx.y, tj0 = run * kPanel, width = min(kPanel, tc - tj0);
  const unsigned long long u = (unsigned long long)blockIdx.x * 256 + threadIdx.x;
  const uint32_t local = (uint32_t)(u / UNITS), v = (uint32_t)(u % UNITS), tl = v % 4;
  if (local >= (uint32_t)tr * width) return;
  const uint32_t ti = width == kPanel ? local / kPanel : local / width, tj = tj0 + (local - ti * width);
  const uint8_t *in = src + ((size_t)ti * tc + tj) * TB;
  uint8_t *out = dst + ((size_t)run * kPanel * tr + local) * TB;
  uint4 a[8];
  if (FMT == BT_BFP8) {
    const uint8_t *rows = in + 64 + (v / 4) * 512 + tl * 64;                 // face 2h, datum rows 4t..4t+3; face 2h + 1 is 256 further
#pragma unroll
    for (int i = 0; i < 8; i++) a[i] = *reinterpret_cast<const uint4 *>(rows + (i / 4) * 256 + (i % 4) * 16);
  } else {
    const uint8_t *rows = in + 64 + tl * 32;                                 // face f 128 further each
#pragma unroll
    for (int i = 0; i < 8; i++) a[i] = *reinterpret_cast<const uint4 *>(rows + (i / 2) * 128 + (i % 2) * 16);
  }
  if (FMT == BT_BFP4 || v < 4) {
    uint32_t e[4];
#pragma unroll
    for (int face = 0; face < 4; face++) e[face] = __byte_perm(*reinterpret_cast<const uint32_t *>(in + face * 16 + tl * 4), 0u, 0x3120);
    *reinterpret_cast<uint4 *>(out + tl * 16) = make_uint4(e[0], e[1], e[2], e[3]);
  }
  // four bytes b of the words r0..r3 (datum rows kk = 0..3) as one word in the order kk = 0, 2, 1, 3: lo takes byte
  // 2 * PAIR of each, hi byte 2 * PAIR + 1
  auto gather = [](uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3, bool upper, uint32_t &lo, uint32_t &hi) {
    const uint32_t x = upper ? __byte_perm(r0, r2, 0x7362) : __byte_perm(r0, r2, 0x5140), y = upper ? __byte_perm(r1, r3, 0x7362) : __byte_perm(r1, r3, 0x5140);
    lo = stream_code_word<FMT>(__byte_perm(x, y, 0x5410)), hi = stream_code_word<FMT>(__byte_perm(x, y, 0x7632));
  };
  if (FMT == BT_BFP8) {
    uint8_t *pieces = out + 64 + (v / 4) * 512 + tl * 16;                    // the piece of lane 4g + t is g * 64 further
#pragma unroll
    for (int m = 0; m < 4; m++) {                                            // word m of a row holds the channels of g = 2m and 2m + 1
      uint32_t w[2][4];
#pragma unroll
      for (int fs = 0; fs < 2; fs++) {
        const uint32_t r[4] = {(&a[4 * fs].x)[m], (&a[4 * fs + 1].x)[m], (&a[4 * fs + 2].x)[m], (&a[4 * fs + 3].x)[m]};
        gather(r[0], r[1], r[2], r[3], false, w[0][2 * fs], w[0][2 * fs + 1]);
        gather(r[0], r[1], r[2], r[3], true, w[1][2 * fs], w[1][2 * fs + 1]);
      }
#pragma unroll
      for (int odd = 0; odd < 2; odd++) *reinterpret_cast<uint4 *>(pieces + (2 * m + odd) * 64) = make_uint4(w[odd][0], w[odd][1], w[odd][2], w[odd][3]);
    }
  } else {
    uint8_t *pieces = out + 64 + tl * 16;
    uint32_t w[8][4];                                                        // [g][face]
#pragma unroll
    for (int face = 0; face < 4; face++)
#pragma unroll
      for (int m = 0; m < 2; m++) {                                          // word m of a row holds the bytes of g = 4m..4m+3
        const uint32_t r0 = m ? a[2 * face].y : a[2 * face].x, r1 = m ? a[2 * face].w : a[2 * face].z;
        const uint32_t r2 = m ? a[2 * face + 1].y : a[2 * face + 1].x, r3 = m ? a[2 * face + 1].w : a[2 * face + 1].z;
        gather(r0, r1, r2, r3, false, w[4 * m][face], w[4 * m + 1][face]);
        gather(r0, r1, r2, r3, true, w[4 * m + 2][face], w[4 * m + 3][face]);
      }
#pragma unroll
    for (int g = 0; g < 8; g++) *reinterpret_cast<uint4 *>(pieces + g * 64) = make_uint4(w[g][0], w[g][1], w[g][2], w[g][3]);
  }
}

// Streaming -> canonical, the mirror image: the same thread takes the eight pieces of the lanes 4g + t, decodes a word
// at a time, undoes the transposition and writes the datum rows 4t..4t+3 (and the exponent words of t).
template <int FMT>
__global__ void __launch_bounds__(256) from_stream_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, int tr, int tc) {
  constexpr int TB = tile_bytes(FMT), UNITS = FMT == BT_BFP8 ? 8 : 4;
  const int run = blockIdx.y, tj0 = run * kPanel, width = min(kPanel, tc - tj0);
  const unsigned long long u = (unsigned long long)blockIdx.x * 256 + threadIdx.x;
  const uint32_t local = (uint32_t)(u / UNITS), v = (uint32_t)(u % UNITS), tl = v % 4;
  if (local >= (uint32_t)tr * width) return;
  const uint32_t ti = width == kPanel ? local / kPanel : local / width, tj = tj0 + (local - ti * width);
  const uint8_t *in = src + ((size_t)run * kPanel * tr + local) * TB;
  uint8_t *out = dst + ((size_t)ti * tc + tj) * TB;
  const uint8_t *pieces = in + 64 + (FMT == BT_BFP8 ? (v / 4) * 512 : 0) + tl * 16;   // the piece of lane 4g + t is g * 64 further
  uint4 p[8], a[8];
#pragma unroll
  for (int g = 0; g < 8; g++) p[g] = *reinterpret_cast<const uint4 *>(pieces + g * 64);
  if (FMT == BT_BFP4 || v < 4) {
    const uint4 e = *reinterpret_cast<const uint4 *>(in + tl * 16);
    const uint32_t w[4] = {e.x, e.y, e.z, e.w};
#pragma unroll
    for (int face = 0; face < 4; face++) *reinterpret_cast<uint32_t *>(out + face * 16 + tl * 4) = __byte_perm(w[face], 0u, 0x3120);
  }
  // the inverse of to_stream_kernel's gather: four words that each hold one byte of the datum rows kk = 0, 2, 1, 3
  // (bytes 0..3 of the rows' word in w0..w3) back to the four rows' words
  auto scatter = [](uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    w0 = canonical_code_word<FMT>(w0), w1 = canonical_code_word<FMT>(w1), w2 = canonical_code_word<FMT>(w2), w3 = canonical_code_word<FMT>(w3);
    const uint32_t t = __byte_perm(w0, w1, 0x5140), t2 = __byte_perm(w2, w3, 0x5140), s = __byte_perm(w0, w1, 0x7362), s2 = __byte_perm(w2, w3, 0x7362);
    r0 = __byte_perm(t, t2, 0x5410), r2 = __byte_perm(t, t2, 0x7632), r1 = __byte_perm(s, s2, 0x5410), r3 = __byte_perm(s, s2, 0x7632);
  };
  if (FMT == BT_BFP8) {
#pragma unroll
    for (int m = 0; m < 4; m++)                                              // word m of a row holds the channels of g = 2m and 2m + 1
#pragma unroll
      for (int fs = 0; fs < 2; fs++) {
        const uint32_t e0 = fs ? p[2 * m].z : p[2 * m].x, e1 = fs ? p[2 * m].w : p[2 * m].y;
        const uint32_t o0 = fs ? p[2 * m + 1].z : p[2 * m + 1].x, o1 = fs ? p[2 * m + 1].w : p[2 * m + 1].y;
        scatter(e0, e1, o0, o1, (&a[4 * fs].x)[m], (&a[4 * fs + 1].x)[m], (&a[4 * fs + 2].x)[m], (&a[4 * fs + 3].x)[m]);
      }
    uint8_t *rows = out + 64 + (v / 4) * 512 + tl * 64;                      // face 2h, datum rows 4t..4t+3; face 2h + 1 is 256 further
#pragma unroll
    for (int i = 0; i < 8; i++) *reinterpret_cast<uint4 *>(rows + (i / 4) * 256 + (i % 4) * 16) = a[i];
  } else {
#pragma unroll
    for (int face = 0; face < 4; face++)
#pragma unroll
      for (int m = 0; m < 2; m++) {                                          // word m of a row holds the bytes of g = 4m..4m+3
        uint32_t r0, r1, r2, r3;
        scatter((&p[4 * m].x)[face], (&p[4 * m + 1].x)[face], (&p[4 * m + 2].x)[face], (&p[4 * m + 3].x)[face], r0, r1, r2, r3);
        if (m == 0) a[2 * face].x = r0, a[2 * face].z = r1, a[2 * face + 1].x = r2, a[2 * face + 1].z = r3;
        else a[2 * face].y = r0, a[2 * face].w = r1, a[2 * face + 1].y = r2, a[2 * face + 1].w = r3;
      }
    uint8_t *rows = out + 64 + tl * 32;                                      // face f 128 further each
#pragma unroll
    for (int i = 0; i < 8; i++) *reinterpret_cast<uint4 *>(rows + (i / 2) * 128 + (i % 2) * 16) = a[i];
  }
}

int check_shape(const char *what, int batch, int rows, int cols) {
  BT_REQUIRE(batch > 0 && rows > 0 && cols > 0, "%s: tensor dimensions must be positive: %d x %d x %d", what, batch, rows, cols);
  return BT_OK;
}

}  // namespace

extern "C" {

int bt_tilize(int device, int itemsize, uint64_t src, uint64_t dst, int batch, int rows, int cols, uint64_t stream) {
  if (int s = check_shape("bt_tilize", batch, rows, cols)) return s;
  BT_REQUIRE(itemsize == 2 || itemsize == 4, "bt_tilize: itemsize must be 2 or 4, not %d", itemsize);
  BT_REQUIRE(src && dst, "bt_tilize: null device address");
  if (int s = use_device(device)) return s;
  int tr = (rows + 31) / 32, tc = (cols + 31) / 32;
  size_t items = (size_t)batch * tr * tc * 128;
  const bool wide = cols % 8 == 0 && src % 16 == 0 && dst % 16 == 0;
  const unsigned blocks = blocks_for(items);
  cudaStream_t st = as_stream(stream);
  if (wide && tc >= 8) {
    if (itemsize == 2) launch_tile_wide<uint16_t, true>(as_ptr<uint16_t>(src), as_ptr<uint16_t>(dst), batch, rows, cols, tr, tc, st);
    else launch_tile_wide<uint32_t, true>(as_ptr<uint32_t>(src), as_ptr<uint32_t>(dst), batch, rows, cols, tr, tc, st);
    return launched("tile_wide_kernel");
  }
  if (itemsize == 2) {
    if (wide) tilize_kernel<uint16_t, true><<<blocks, kThreads, 0, st>>>(as_ptr<uint16_t>(src), as_ptr<uint16_t>(dst), batch, rows, cols, tr, tc);
    else tilize_kernel<uint16_t, false><<<blocks, kThreads, 0, st>>>(as_ptr<uint16_t>(src), as_ptr<uint16_t>(dst), batch, rows, cols, tr, tc);
  } else {
    if (wide) tilize_kernel<uint32_t, true><<<blocks, kThreads, 0, st>>>(as_ptr<uint32_t>(src), as_ptr<uint32_t>(dst), batch, rows, cols, tr, tc);
    else tilize_kernel<uint32_t, false><<<blocks, kThreads, 0, st>>>(as_ptr<uint32_t>(src), as_ptr<uint32_t>(dst), batch, rows, cols, tr, tc);
  }
  return launched("tilize_kernel");
}

int bt_untilize(int device, int itemsize, uint64_t src, uint64_t dst, int batch, int rows, int cols, uint64_t stream) {
  if (int s = check_shape("bt_untilize", batch, rows, cols)) return s;
  BT_REQUIRE(itemsize == 2 || itemsize == 4, "bt_untilize: itemsize must be 2 or 4, not %d", itemsize);
  BT_REQUIRE(src && dst, "bt_untilize: null device address");
  if (int s = use_device(device)) return s;
  int tr = (rows + 31) / 32, tc = (cols + 31) / 32;
  size_t items = (size_t)batch * tr * tc * 128;
  const bool wide = cols % 8 == 0 && src % 16 == 0 && dst % 16 == 0;
  const unsigned blocks = blocks_for(items);
  cudaStream_t st = as_stream(stream);
  if (wide && tc >= 8) {
    if (itemsize == 2) launch_tile_wide<uint16_t, false>(as_ptr<uint16_t>(src), as_ptr<uint16_t>(dst), batch, rows, cols, tr, tc, st);
    else launch_tile_wide<uint32_t, false>(as_ptr<uint32_t>(src), as_ptr<uint32_t>(dst), batch, rows, cols, tr, tc, st);
    return launched("tile_wide_kernel");
  }
  if (itemsize == 2) {
    if (wide) untilize_kernel<uint16_t, true><<<blocks, kThreads, 0, st>>>(as_ptr<uint16_t>(src), as_ptr<uint16_t>(dst), batch, rows, cols, tr, tc);
    else untilize_kernel<uint16_t, false><<<blocks, kThreads, 0, st>>>(as_ptr<uint16_t>(src), as_ptr<uint16_t>(dst), batch, rows, cols, tr, tc);
  } else {
    if (wide) untilize_kernel<uint32_t, true><<<blocks, kThreads, 0, st>>>(as_ptr<uint32_t>(src), as_ptr<uint32_t>(dst), batch, rows, cols, tr, tc);
    else untilize_kernel<uint32_t, false><<<blocks, kThreads, 0, st>>>(as_ptr<uint32_t>(src), as_ptr<uint32_t>(dst), batch, rows, cols, tr, tc);
  }
  return launched("untilize_kernel");
}

static int many(const char *what, bool tilize, int device, int itemsize, int n, const uint64_t *src, const uint64_t *dst, const int *rows, const int *cols,
                uint64_t stream) {
  BT_REQUIRE(itemsize == 2 || itemsize == 4, "%s: itemsize must be 2 or 4, not %d", what, itemsize);
  BT_REQUIRE(n > 0 && src && dst && rows && cols, "%s: null table or no matrices", what);
  if (int s = use_device(device)) return s;
  for (int at = 0; at < n; at += kManyMax) {
    ManyArgs a{};
    a.n = min(kManyMax, n - at);
    for (int k = 0; k < a.n; k++) {
      if (int s = check_shape(what, 1, rows[at + k], cols[at + k])) return s;
      BT_REQUIRE(src[at + k] && dst[at + k] && (tilize ? dst : src)[at + k] % 16 == 0, "%s: matrix %d: null address or tiles not 16-byte aligned", what, at + k);
      a.src[k] = as_ptr<void>(src[at + k]), a.dst[k] = as_ptr<void>(dst[at + k]), a.rows[k] = rows[at + k], a.cols[k] = cols[at + k];
      const long long halves = (long long)((rows[at + k] + 31) / 32) * ((cols[at + k] + 31) / 32) * 128;
      BT_REQUIRE(a.first[k] + halves < (1ll << 31), "%s: too much for one launch: put large matrices through the single-matrix call", what);
      a.first[k + 1] = a.first[k] + (int)halves;
    }
    const unsigned blocks = blocks_for((size_t)a.first[a.n]);
    cudaStream_t st = as_stream(stream);
    if (itemsize == 2) {
      if (tilize) many_kernel<uint16_t, true><<<blocks, kThreads, 0, st>>>(a);
      else many_kernel<uint16_t, false><<<blocks, kThreads, 0, st>>>(a);
    } else {
      if (tilize) many_kernel<uint32_t, true><<<blocks, kThreads, 0, st>>>(a);
      else many_kernel<uint32_t, false><<<blocks, kThreads, 0, st>>>(a);
    }
    if (int s = launched("many_kernel")) return s;
  }
  return BT_OK;
}

int bt_tilize_many(int device, int itemsize, int n, const uint64_t *src, const uint64_t *dst, const int *rows, const int *cols, uint64_t stream) {
  return many("bt_tilize_many", true, device, itemsize, n, src, dst, rows, cols, stream);
}

int bt_untilize_many(int device, int itemsize, int n, const uint64_t *src, const uint64_t *dst, const int *rows, const int *cols, uint64_t stream) {
  return many("bt_untilize_many", false, device, itemsize, n, src, dst, rows, cols, stream);
}

int bt_round_bf16(int device, uint64_t src_f32, uint64_t dst_bf16, size_t count, uint64_t stream) {
  BT_REQUIRE(src_f32 && dst_bf16 && count, "bt_round_bf16: null device address or zero count");
  if (int s = use_device(device)) return s;
  round_bf16_kernel<<<blocks_for(count), kThreads, 0, as_stream(stream)>>>(as_ptr<uint32_t>(src_f32), as_ptr<uint16_t>(dst_bf16), count);
  return launched("round_bf16_kernel");
}

int bt_pack_bfp(int device, int fmt, uint64_t src, uint64_t dst, size_t ntiles, uint64_t stream) {
  BT_REQUIRE(fmt == BT_BFP8 || fmt == BT_BFP4, "bt_pack_bfp: format must be bfp8 (8) or bfp4 (4), not %d", fmt);
  BT_REQUIRE(src && dst && ntiles, "bt_pack_bfp: null device address or zero tiles");
  BT_REQUIRE(src % 16 == 0 && dst % 16 == 0, "bt_pack_bfp: tiles must be 16-byte aligned");
  if (int s = use_device(device)) return s;
  size_t pairs = ntiles * 32;
  if (fmt == BT_BFP8) pack_kernel<BT_BFP8><<<blocks_for(pairs), kThreads, 0, as_stream(stream)>>>(as_ptr<uint4>(src), as_ptr<uint8_t>(dst), pairs);
  else pack_kernel<BT_BFP4><<<blocks_for(pairs), kThreads, 0, as_stream(stream)>>>(as_ptr<uint4>(src), as_ptr<uint8_t>(dst), pairs);
  return launched("pack_kernel");
}

int bt_unpack_bfp(int device, int fmt, uint64_t src, uint64_t dst, size_t ntiles, uint64_t stream) {
  BT_REQUIRE(fmt == BT_BFP8 || fmt == BT_BFP4, "bt_unpack_bfp: format must be bfp8 (8) or bfp4 (4), not %d", fmt);
  BT_REQUIRE(src && dst && ntiles, "bt_unpack_bfp: null device address or zero tiles");
  BT_REQUIRE(src % 16 == 0 && dst % 16 == 0, "bt_unpack_bfp: tiles must be 16-byte aligned");
  if (int s = use_device(device)) return s;
  size_t runs = ntiles * 64;
  if (fmt == BT_BFP8) unpack_kernel<BT_BFP8><<<blocks_for(runs), kThreads, 0, as_stream(stream)>>>(as_ptr<uint8_t>(src), as_ptr<uint4>(dst), runs);
  else unpack_kernel<BT_BFP4><<<blocks_for(runs), kThreads, 0, as_stream(stream)>>>(as_ptr<uint8_t>(src), as_ptr<uint4>(dst), runs);
  return launched("unpack_kernel");
}

int bt_put(int device, int fmt, uint64_t dst, uint64_t x, uint64_t ids, int batch, int n, int dst_rows, int cols, uint64_t scratch, uint64_t stream) {
  BT_REQUIRE(fmt == BT_BFP8 || fmt == BT_BFP4 || fmt == BT_BF16 || fmt == BT_FP32 || fmt == BT_INT32, "bt_put: unknown format %d", fmt);
  BT_REQUIRE(dst && x && ids && dst != x && dst != ids && dst % 16 == 0 && x % 16 == 0, "bt_put: needs 16-byte aligned tensors, x and ids apart from dst");
  if (int s = check_shape("bt_put", batch, n, cols)) return s;
  BT_REQUIRE(dst_rows > 0, "bt_put: the destination has no rows");
  if (int s = use_device(device)) return s;
  const int tc = (cols + 31) / 32, dst_tr = (dst_rows + 31) / 32, x_tr = (n + 31) / 32;
  const size_t units = (size_t)batch * n * tc * 2;
  const unsigned blocks = blocks_for(units);
  uint8_t *d = as_ptr<uint8_t>(dst);
  const uint8_t *s8 = as_ptr<uint8_t>(x);
  const int *places = as_ptr<int>(ids);
  cudaStream_t st = as_stream(stream);
  int *last = as_ptr<int>(scratch);
  if (last) {
    BT_REQUIRE(scratch % 4 == 0, "bt_put: the scratch holds ints");
    BT_CUDA(cudaMemsetAsync(last, 0xFF, (size_t)dst_tr * 32 * sizeof(int), st));
    put_last_kernel<<<blocks_for((size_t)n), kThreads, 0, st>>>(places, n, dst_tr, dst_rows == 1, last);
    if (int s = launched("put_last_kernel")) return s;
  }
  if (fmt == BT_BFP8) put_kernel<BT_BFP8><<<blocks, kThreads, 0, st>>>(d, s8, places, batch, n, tc, dst_tr, x_tr, dst_rows == 1, last);
  else if (fmt == BT_BFP4) put_kernel<BT_BFP4><<<blocks, kThreads, 0, st>>>(d, s8, places, batch, n, tc, dst_tr, x_tr, dst_rows == 1, last);
  else if (fmt == BT_BF16) put_kernel<-2><<<blocks, kThreads, 0, st>>>(d, s8, places, batch, n, tc, dst_tr, x_tr, dst_rows == 1, last);
  else put_kernel<-4><<<blocks, kThreads, 0, st>>>(d, s8, places, batch, n, tc, dst_tr, x_tr, dst_rows == 1, last);
  return launched("put_kernel");
}

int bt_relayout(int device, int fmt, int to_stream, int tile_rows, int tile_cols, uint64_t src, uint64_t dst, uint64_t stream) {
  BT_REQUIRE(fmt == BT_BFP8 || fmt == BT_BFP4, "bt_relayout: format must be bfp8 (8) or bfp4 (4), not %d", fmt);
  BT_REQUIRE(tile_rows > 0 && tile_cols > 0, "bt_relayout: tile counts must be positive: %d x %d", tile_rows, tile_cols);
  BT_REQUIRE((long long)tile_rows * tile_cols < (1ll << 31), "bt_relayout: too many tiles for one launch");
  const int runs = (tile_cols + kPanel - 1) / kPanel;
  BT_REQUIRE(runs <= 65535, "bt_relayout: at most %d tile columns in one launch, not %d", 65535 * kPanel, tile_cols);
  BT_REQUIRE(src && dst && src != dst && src % 16 == 0 && dst % 16 == 0, "bt_relayout: needs distinct 16-byte aligned buffers");
  if (int s = use_device(device)) return s;
  cudaStream_t st = as_stream(stream);
  const uint8_t *s8 = as_ptr<uint8_t>(src);
  uint8_t *d8 = as_ptr<uint8_t>(dst);
  const unsigned long long units = (unsigned long long)tile_rows * min(kPanel, tile_cols) * (fmt == BT_BFP8 ? 8 : 4);
  const dim3 grid((unsigned)((units + 255) / 256), (unsigned)runs);
  if (fmt == BT_BFP8 && to_stream) to_stream_kernel<BT_BFP8><<<grid, 256, 0, st>>>(s8, d8, tile_rows, tile_cols);
  else if (to_stream) to_stream_kernel<BT_BFP4><<<grid, 256, 0, st>>>(s8, d8, tile_rows, tile_cols);
  else if (fmt == BT_BFP8) from_stream_kernel<BT_BFP8><<<grid, 256, 0, st>>>(s8, d8, tile_rows, tile_cols);
  else from_stream_kernel<BT_BFP4><<<grid, 256, 0, st>>>(s8, d8, tile_rows, tile_cols);
  return launched(to_stream ? "to_stream_kernel" : "from_stream_kernel");
}

}  // extern "C"
