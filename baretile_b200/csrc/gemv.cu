// Decode matmul for up to 32 token rows: out = epilogue(alpha * x @ W + add), W block-float in streaming layout,
// and a queue of such matmuls run by ONE launch.
//
// The work is bound by HBM: every packed weight byte is read once, by a bulk (TMA) copy into a ring of
// shared-memory stages, and dequantised in registers on its way into a bf16 MMA with fp32 accumulators.
//
// A queue. In decode one matmul's result is the next one's x, so between two of them the GPU has nothing to read
// unless the next weights are already on their way. The kernel therefore takes a list of matmuls (up to kQueueMax
// per launch) and runs them in order with the same persistent CTAs. The weight warp of a CTA walks the whole list:
// weight copies depend on nothing and go out as soon as the ring has room, across the boundary between two matmuls.
// Only x waits: the x warp copies a matmul's activations once every CTA has reported the matmuls it depends on
// finished (a counter per matmul in global memory, read with acquire semantics; the host works out the dependences
// from the buffer addresses, and matmuls that do not depend on one another overlap, two in flight at most). While
// that report travels, the ring fills with the next weights.
//
// Decomposition ("stream-K"). A weight matrix is cut into sub-panels of 4 tile columns (one run of the streaming
// layout). A unit is one tile row of one sub-panel. Units are numbered sub-panel by sub-panel and dealt out in
// contiguous ranges to the CTAs (two per SM): equal shares of all CTAs, so every SM streams the same number of bytes
// whatever the shape, or, where that keeps most CTAs busy, shares cut so that ranges end where sub-panels end. A
// sub-panel that several CTAs share is finished by the CTA that holds its last tile row: the others write
// their fp32 partial sums to scratch and bump a counter; the owner, which takes that sub-panel last, waits for the
// counter (with a limit), adds the partials in CTA order, so results do not depend on timing, and runs the
// epilogue. Contributors never wait, so the owner's wait always ends; it is bounded all the same.
//
// Inside a CTA: warps 8 and 9 are the producers. Warp 8 waits for room in the ring, announces the stage's weight
// bytes to the stage's mbarrier and issues one bulk copy per weight matrix; warp 9 does the same for the stage's x
// tiles once the matmuls this one depends on are finished. Stages are as large as the matmul's kind wants and follow
// one another through the ring's bytes; 16 mbarrier pairs go round with them. The 8 consumer
// warps form a 2 x 4 grid: warp (ck, cc) takes column cc of the sub-panel; for one weight matrix ck picks every
// other tile row of the stage (the two halves are added through shared memory when the sub-panel ends), for a
// gate/up pair ck picks the matrix (the up half is handed to the gate warp for the epilogue). A weight tile is
// four 16x16 faces; a face is one m16n8k16 MMA with the face's 16 output channels as the MMA's rows, 16 input
// channels as its K and up to 8 tokens as its columns. The 16 weights of a face row share an exponent e; how the
// packed bytes become exact bf16 weights times 2^(e - 197) is described at tile_mma; the epilogue multiplies the
// sums by 2^64.
#include "common.cuh"
#include "ptx.cuh"
#include "stream_layout.cuh"
#include <cstring>
#include <mutex>

using namespace bt;

namespace {

constexpr int kWC = kPanel;                 // tile columns of a sub-panel = one run of the streaming layout
constexpr int kCW = 8;                      // consumer warps per CTA
constexpr int kThreads = (kCW + 2) * 32;    // plus the two producer warps
constexpr int kOcc = 2;                     // CTAs per SM
constexpr int kBars = 16;                   // stages in the ring at most: mbarriers that go round with the stages
constexpr int kMaxCtas = 320;
constexpr int kMaxSubPanels = 16384;
constexpr int kQueueMax = 32;               // matmuls per launch; longer lists take several launches
constexpr uint32_t kSpinLimit = 1u << 14;   // attempts of up to 100 us each (mbarriers) or 32-64 ns polls x 32 (counters)

// Shared memory of a CTA.
constexpr int kSmFull = 0, kSmEmpty = 128;  // mbarriers: a stage's weights and x have landed; it is free again
constexpr int kSmHeld = 256;                // uint32[2][kBars]: ring bytes of each stage in the ring, as each producer warp noted them
constexpr int kSmArgVal = 512;              // float[4][32]: best value per column warp and token
constexpr int kSmArgIdx = 512 + 512;        // int[4][32]: and its channel
constexpr int kSmRed = 1536;                // 4 KiB: 8 accumulators per lane handed from warps ck = 1 to warps ck = 0
constexpr int kSmRing = kSmRed + 4096;
constexpr int kSmemBytes = (228 * 1024 / kOcc - 1024) / 128 * 128;   // an SM's shared memory less the runtime's 1 KiB per CTA
constexpr int kRingBytes = kSmemBytes - kSmRing;
static_assert(kSmRing % 128 == 0 && kRingBytes % 128 == 0, "stages are 128-byte aligned");

// Scratch layout (byte offsets into the caller's workspace). Two matmuls of a queue may be in flight at once, so
// what a matmul uses while it runs exists twice (a set for even and one for odd positions in the queue).
constexpr size_t kWsError = 0;                                   // int: set to nonzero when a wait gave up
constexpr size_t kWsOpsDone = 8;                                 // int[kQueueMax]: CTAs that finished each matmul of the launch
constexpr size_t kWsSets = 256;                                  // the sets start here
constexpr size_t kSetPanelsDone = 0;                             // int: sub-panels finished (argmax epilogue)
constexpr size_t kSetKeys = 256;                                 // u64[32]: per token the best (value, column) so far (argmax epilogue)
constexpr size_t kSetCounters = 512;                             // int[kMaxSubPanels]: CTAs arrived at a sub-panel
constexpr size_t kSetPartials = kSetCounters + 4 * kMaxSubPanels;
constexpr size_t kSlotFloatsMax = 8 * 32 * 32;                   // 8 warps x up to 32 accumulators x 32 lanes
constexpr size_t kSetBytes = kSetPartials + (size_t)kMaxCtas * kSlotFloatsMax * 4;
constexpr int kSets = 2;                                         // matmuls of a queue in flight at most
constexpr size_t kWsBytes = kWsSets + kSets * kSetBytes;

// The shape of a stage for one kind of matmul: format, one matrix or a gate/up pair, token groups of 8 rows.
struct Geometry {
  int tb;        // bytes of a packed tile
  int t;         // tile rows a warp takes per stage
  int ups;       // units (tile rows) per stage
  int matrix;    // bytes of one matrix's part of a stage
  int w_bytes;   // all weights of a stage; the x tiles follow
  int xb;        // bytes of an x tile staged: its first half (token rows 0-15) or all of it
  int stage;     // bytes of a stage
};
__host__ __device__ constexpr int stage_rows_per_warp(int fmt, int tg) { return tg == 1 && fmt == BT_BFP4 ? 4 : 2; }
__host__ __device__ constexpr Geometry geometry(int fmt, bool pair, int tg) {
  Geometry g{};
  g.tb = tile_bytes(fmt), g.t = stage_rows_per_warp(fmt, tg);
  g.ups = pair ? g.t : 2 * g.t;
  g.matrix = g.ups * kWC * g.tb;
  g.w_bytes = (pair ? 2 : 1) * g.matrix;
  g.xb = tg == 4 ? 2048 : 1024;
  g.stage = g.w_bytes + g.ups * g.xb;
  return g;
}
static_assert(geometry(BT_BFP8, false, 1).stage % 128 == 0 && geometry(BT_BFP4, false, 4).stage % 128 == 0 && geometry(BT_BFP4, true, 4).stage % 128 == 0,
              "stages keep the ring 128-byte aligned");

// One matmul of the queue, as the kernel sees it.
struct GemvParams {
  const uint8_t *x;
  const uint8_t *w[2];
  const uint16_t *add;
  void *out;
  float *arg_val;
  int *arg_idx;
  float alpha;
  int arg_base, M, KT, TC, epi, out_fp32;
  int fmt, pair, tg;
  int wait_for;               // the matmul of the launch that must be complete before this one starts; -1: none
  int turn;                   // CTA c takes the unit range (c + turn) % CTAs
  int per;                    // units per range when ranges are cut to fit the sub-panels; 0: equal shares of all CTAs
};

// What a matmul uses while it runs: the count of finished sub-panels and the per-token best keys (argmax), the
// arrivals per sub-panel (all zero before first use; the kernel leaves them zero) and one slot of partial sums per CTA.
struct Scratch {
  int *panels_done, *counters;
  unsigned long long *keys;   // per token the best (value, column) so far, as an ordered key; zero: nothing yet
  float *partials;
};

// What one launch gets: the matmuls and the scratch they share: a wait-gave-up flag, the counts of CTAs that
// finished each matmul (zero before first use; the kernel leaves them zero) and one or two sets of running scratch.
struct Queue {
  int n;
  int sets;                   // kSets: matmuls take the sets in turn, and as many may be in flight; 1: one after the other
  int *error, *ops_done;
  Scratch set[kSets];
  int slot_floats;            // floats between two CTAs' slots of partial sums
  GemvParams op[kQueueMax];
};


// Where range b of `ctas` starts: equal shares, or with `per` > 0 shares of exactly `per` units (the last one shorter).
__host__ __device__ __forceinline__ long long range_start(long long units, int b, int ctas, int per) {
  return per > 0 ? min((long long)b * per, units) : units * b / ctas;
}
// The CTA whose (non-empty) range holds unit u.
__device__ __forceinline__ int cta_of(long long u, long long units, int ctas, int per) {
  if (per > 0) return (int)(u / per);
  int b = (int)(u * ctas / units);
  while (b + 1 < ctas && range_start(units, b + 1, ctas, 0) <= u) b++;
  while (b > 0 && range_start(units, b, ctas, 0) > u) b--;
  return b;
}

// One weight tile times the staged x tile. `tile`, `ex` and `xs` are shared-memory addresses that already include
// the lane's own offsets: tile = tile base + 16 * lane; ex = tile base + 16 * t, where the lane's exponents are;
// xs = x tile base + 32 * g + 8 * t (g = lane / 4, t = lane % 4).
//
// A weight byte (offset binary, see stream_layout.cuh) zero-extended into a 16-bit lane is the bf16 number
// byte * 2^-133, so a mask (bytes 0 and 2 of a word: the lane's first k pair) or a byte-permute (bytes 1 and 3: its
// second pair) makes a register of two weights, and one packed fused multiply-add with the face row's power of two
// s = 2^(e - 64) and with -offset * 2^-133 * s turns it into the exact signed weights times 2^(e - 197); the
// epilogue multiplies the sums by 2^64. An all-zero run has e = 0: both products underflow to zero, as they should.
//
// bfp8: a face (16 k x 16 n) is one MMA, rows g and g + 8 of it the channels 2g and 2g + 1; acc[fs][tg] collects
// face column fs. bfp4: a byte holds two channels of the same k, low and high nibble. The whole byte as a weight,
// 16 * high + low, goes into one MMA ("both", acc[0]), the masked low nibble into another ("low", acc[1]); rows g of
// these MMAs are the byte of channels (2g, 2g + 1) of face column 0, rows g + 8 that of face column 1. When a
// sub-panel's sums are complete, 16 * high = both - low (settle below; a nibble q is worth 16 q). Sixteen registers of weights per tile either
// way, for half as many loaded bytes.
constexpr uint32_t kByteLanes = 0x00FF00FFu, kNibbleLanes = 0x000F000Fu, kOddBytes = 0x4341u;
constexpr uint32_t kMinus128 = 0x80808080u;   // two bf16 lanes of -128 * 2^-133 = -2^-126
constexpr uint32_t kMinus136 = 0x80888088u;   // -(128 + 8) * 2^-133: offset of a byte made of two offset nibbles
constexpr uint32_t kMinus8 = 0x80088008u;     // -8 * 2^-133
template <int FMT, int TG>
__device__ __forceinline__ void tile_mma(uint32_t tile, uint32_t ex, uint32_t xs, float (&acc)[2][TG][4]) {
  const uint4 ev = lds128(ex);
  const uint32_t ee[4] = {ev.x, ev.y, ev.z, ev.w};
  uint2 bx[2][TG];
#pragma unroll
  for (int h = 0; h < 2; h++) {
#pragma unroll
    for (int tg = 0; tg < TG; tg++) bx[h][tg] = lds64(xs + (tg >> 1) * 1024 + h * 512 + (tg & 1) * 256);
  }
  uint4 wv[2];
  if (FMT == BT_BFP8) wv[0] = lds128(tile + 64), wv[1] = lds128(tile + 64 + 512);
  else wv[0] = lds128(tile + 64), wv[1] = wv[0];
  uint32_t s[4][2];   // scales of face 2h + fs, first and second k pair
#pragma unroll
  for (int f = 0; f < 4; f++) s[f][0] = scale_pair<0>(ee[f]), s[f][1] = scale_pair<1>(ee[f]);
#pragma unroll
  for (int h = 0; h < 2; h++) {
    if (FMT == BT_BFP8) {
#pragma unroll
      for (int fs = 0; fs < 2; fs++) {
        const int f = 2 * h + fs;
        const uint32_t w0 = fs ? wv[h].z : wv[h].x, w1 = fs ? wv[h].w : wv[h].y;   // channels 2g and 2g + 1
        const uint32_t n01 = mul_bf16x2(s[f][0], kMinus128), n23 = mul_bf16x2(s[f][1], kMinus128);
        const uint32_t a0 = fma_bf16x2(w0 & kByteLanes, s[f][0], n01), a1 = fma_bf16x2(w1 & kByteLanes, s[f][0], n01);
        const uint32_t a2 = fma_bf16x2(prmt(w0, 0u, kOddBytes), s[f][1], n23), a3 = fma_bf16x2(prmt(w1, 0u, kOddBytes), s[f][1], n23);
#pragma unroll
        for (int tg = 0; tg < TG; tg++) mma_bf16(acc[fs][tg], a0, a1, a2, a3, bx[h][tg].x, bx[h][tg].y);
      }
    } else {
      const uint32_t w0 = h ? wv[0].z : wv[0].x, w1 = h ? wv[0].w : wv[0].y;       // face columns 0 and 1
      const uint32_t b0 = w0 & kByteLanes, b1 = w1 & kByteLanes, b2 = prmt(w0, 0u, kOddBytes), b3 = prmt(w1, 0u, kOddBytes);
      const uint32_t s0 = s[2 * h][0], s1 = s[2 * h + 1][0], s2 = s[2 * h][1], s3 = s[2 * h + 1][1];
      {
        const uint32_t a0 = fma_bf16x2(b0, s0, mul_bf16x2(s0, kMinus136)), a1 = fma_bf16x2(b1, s1, mul_bf16x2(s1, kMinus136));
        const uint32_t a2 = fma_bf16x2(b2, s2, mul_bf16x2(s2, kMinus136)), a3 = fma_bf16x2(b3, s3, mul_bf16x2(s3, kMinus136));
#pragma unroll
        for (int tg = 0; tg < TG; tg++) mma_bf16(acc[0][tg], a0, a1, a2, a3, bx[h][tg].x, bx[h][tg].y);
      }
      {
        const uint32_t a0 = fma_bf16x2(w0 & kNibbleLanes, s0, mul_bf16x2(s0, kMinus8)), a1 = fma_bf16x2(w1 & kNibbleLanes, s1, mul_bf16x2(s1, kMinus8));
        const uint32_t a2 = fma_bf16x2(b2 & kNibbleLanes, s2, mul_bf16x2(s2, kMinus8)), a3 = fma_bf16x2(b3 & kNibbleLanes, s3, mul_bf16x2(s3, kMinus8));
#pragma unroll
        for (int tg = 0; tg < TG; tg++) mma_bf16(acc[1][tg], a0, a1, a2, a3, bx[h][tg].x, bx[h][tg].y);
      }
    }
  }
}

// bfp4: from ("both", "low") sums to the arrangement the rest of the kernel uses, acc[face column][tg][j] for
// channel 2g and [2 + j] for channel 2g + 1. "both" and "low" hold face column 0 in [0], [1] and face column 1 in
// [2], [3]. Linear, so it may run on partial sums.
template <int FMT, int TG>
__device__ __forceinline__ void settle(float (&acc)[2][TG][4]) {
  if (FMT != BT_BFP4) return;
#pragma unroll
  for (int tg = 0; tg < TG; tg++) {
    float both[4], low[4];
#pragma unroll
    for (int i = 0; i < 4; i++) both[i] = acc[0][tg][i], low[i] = acc[1][tg][i];
#pragma unroll
    for (int fs = 0; fs < 2; fs++) {
#pragma unroll
      for (int j = 0; j < 2; j++) acc[fs][tg][j] = 16.f * low[2 * fs + j], acc[fs][tg][2 + j] = both[2 * fs + j] - low[2 * fs + j];
    }
  }
}

__device__ __forceinline__ float silu(float v) { return __fdividef(v, 1.0f + __expf(-v)); }
__device__ __forceinline__ uint32_t bf16_half_up(float v) { return (__float_as_uint(v) + 0x8000u) >> 16; }
__device__ __forceinline__ float bf16_value(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
// a beats b: larger value, or the same value at a lower column; -0 equals 0; a NaN never wins
__device__ __forceinline__ bool beats(float av, int ai, float bv, int bi) { return av > bv || (av == bv && ai < bi); }
// (value, column) as one number whose order is `beats`: larger value first, then the lower column. Zero is reserved
// for "nothing yet"; no value maps to it, since a NaN is never offered and -inf maps to 0x007FFFFF in the upper half.
__device__ __forceinline__ unsigned long long pick_key(float v, int column) {
  uint32_t b = __float_as_uint(v == 0.f ? 0.f : v);
  b ^= b >> 31 ? 0xFFFFFFFFu : 0x80000000u;
  return (unsigned long long)b << 32 | (0xFFFFFFFFu - (uint32_t)column);
}


// The epilogue of one finished tile column. Lane (g, t) holds, for each channel group ng and token group tg,
// tokens 8 tg + 2t + j (j = 0, 1) and channels 16 ng + 2g + {0, 1}: acc[ng][tg][j] and [2 + j].
// For a gate/up pair `acc` holds the gate sums and `up` the up sums in the same arrangement.
template <int TG, bool PAIR>
__device__ __forceinline__ void finish_column(const GemvParams &p, const float (&acc)[2][TG][4], const float (&up)[2][TG][4], int col, int cc,
                                              int lane, float *arg_v, int *arg_i) {
  const int g = lane >> 2, t = lane & 3;
  const float unscale = 18446744073709551616.f * p.alpha;  // 2^64: the weights entered the MMA scaled by 2^-64
  float best_v[TG][2];
  int best_i[TG][2];
#pragma unroll
  for (int tg = 0; tg < TG; tg++) best_v[tg][0] = best_v[tg][1] = -INFINITY, best_i[tg][0] = best_i[tg][1] = 0x7FFFFFFF;
#pragma unroll
  for (int ng = 0; ng < 2; ng++) {
#pragma unroll
    for (int tg = 0; tg < 4; tg++) {
      constexpr int kLast = TG - 1;
      const int tgs = tg < TG ? tg : 0;  // a one-row result repeats across its tile: every row shows token 0
#pragma unroll
      for (int j = 0; j < 2; j++) {
        const int m = 8 * tg + 2 * t + j, at = ((m >> 4) * 2 + ng) * 256 + (m & 15) * 16 + 2 * g;
        const bool valid = p.M == 1 || (tg <= kLast && m < p.M);
        float v0 = acc[ng][tgs][j] * unscale, v1 = acc[ng][tgs][2 + j] * unscale;
        if (p.add) {
          const uint32_t a = *reinterpret_cast<const uint32_t *>(p.add + (size_t)col * 1024 + at);
          v0 += bf16_value((uint16_t)a), v1 += bf16_value((uint16_t)(a >> 16));
        }
        if (p.epi == BT_EPI_RELU) v0 = fmaxf(v0, 0.f), v1 = fmaxf(v1, 0.f);
        else if (p.epi == BT_EPI_SILU) v0 = silu(v0), v1 = silu(v1);
        else if (PAIR) v0 = silu(v0) * (up[ng][tgs][j] * unscale), v1 = silu(v1) * (up[ng][tgs][2 + j] * unscale);
        if (p.epi == BT_EPI_ARGMAX) {
          if (tg <= kLast && m < p.M) {
            const int n0 = col * 32 + 16 * ng + 2 * g;
            if (beats(v0, n0, best_v[tgs][j], best_i[tgs][j])) best_v[tgs][j] = v0, best_i[tgs][j] = n0;
            if (beats(v1, n0 + 1, best_v[tgs][j], best_i[tgs][j])) best_v[tgs][j] = v1, best_i[tgs][j] = n0 + 1;
          }
          continue;
        }
        if (p.out_fp32 == 2) {
          // row-major fp32, only the rows there are: partial sums on their way to an all-reduce
          if (tg <= kLast && m < p.M) *reinterpret_cast<float2 *>(static_cast<float *>(p.out) + (size_t)m * (p.TC * 32) + col * 32 + 16 * ng + 2 * g) = make_float2(v0, v1);
          continue;
        }
        if (!valid) v0 = v1 = 0.f;
        if (p.out_fp32) *reinterpret_cast<float2 *>(static_cast<float *>(p.out) + (size_t)col * 1024 + at) = make_float2(v0, v1);
        else *reinterpret_cast<uint32_t *>(static_cast<uint16_t *>(p.out) + (size_t)col * 1024 + at) = bf16_half_up(v0) | bf16_half_up(v1) << 16;
      }
    }
  }
  if (p.epi == BT_EPI_ARGMAX) {
    // best over this column's 32 channels: combine the lanes that hold the same tokens (same t)
#pragma unroll
    for (int tg = 0; tg < 4; tg++) {
#pragma unroll
      for (int j = 0; j < 2; j++) {
        float v = -INFINITY;
        int i = 0x7FFFFFFF;
        if (tg < TG) v = best_v[tg < TG ? tg : 0][j], i = best_i[tg < TG ? tg : 0][j];
#pragma unroll
        for (int d = 4; d < 32; d <<= 1) {
          const float ov = __shfl_xor_sync(0xFFFFFFFFu, v, d);
          const int oi = __shfl_xor_sync(0xFFFFFFFFu, i, d);
          if (beats(ov, oi, v, i)) v = ov, i = oi;
        }
        if (g == 0) arg_v[cc * 32 + 8 * tg + 2 * t + j] = v, arg_i[cc * 32 + 8 * tg + 2 * t + j] = i;
      }
    }
  }
}

// The unit ranges of a CTA in the order it takes them. A sub-panel that several CTAs share is finished by the CTA
// that holds its last tile row (its owner); the others hand it their partial sums through global memory. So a CTA
// first takes the sub-panel its range ends in (it is that one's first contributor, and the owner will not need the
// sums for a while), then the sub-panels it has whole, and last the sub-panel its range starts in, which it owns:
// by then the other contributors have long signalled, or are finishing at the same moment.
struct Segments {
  long long a[3], b[3];
  int n;
};
__device__ __forceinline__ Segments segments_of(long long u0, long long u1, int KT) {
  Segments s;
  s.n = 0;
  for (int i = 0; i < 3; i++) s.a[i] = s.b[i] = 0;
  if (u0 >= u1) return s;
  const long long head_end = min(u1, (u0 / KT + 1) * KT);            // end of the sub-panel the range starts in
  const bool head_partial = u0 % KT != 0 || head_end - u0 < KT;
  const long long tail_start = (u1 / KT) * KT;                       // start of the sub-panel the range ends in
  const bool tail_partial = u1 % KT != 0 && tail_start >= head_end;  // a tail that is not the head itself
  long long mid_a = head_partial ? head_end : u0, mid_b = tail_partial ? tail_start : u1;
  if (tail_partial) s.a[s.n] = tail_start, s.b[s.n++] = u1;
  if (mid_b > mid_a) s.a[s.n] = mid_a, s.b[s.n++] = mid_b;
  if (head_partial) s.a[s.n] = u0, s.b[s.n++] = head_end;
  return s;
}

// Where the next stage goes, kept in step by the three parties of a CTA: stages follow one another through the
// ring's bytes (a stage that would run past the end starts over at 0) and through the kBars mbarrier pairs.
struct Ring {
  uint32_t off;     // where the next stage would start
  uint32_t bar;     // byte offset of its mbarriers among their kind: 8 * (stages so far % kBars)
  uint32_t parity;  // the phase to wait for: (stages so far / kBars) & 1
  __device__ __forceinline__ uint32_t place(uint32_t bytes) {       // byte offset of the next stage
    if (off + bytes > kRingBytes) off = 0;
    const uint32_t at = off;
    off += bytes;
    return at;
  }
  __device__ __forceinline__ void advance() {
    bar = (bar + 8) & (8 * kBars - 1);
    if (bar == 0) parity ^= 1;
  }
};

// A CTA's stages of one matmul, in order: sub-panel, first tile row and number of tile rows of each. Everything
// is a scalar with a fixed place, so the walk lives in registers.
struct Walk {
  int KT, ups, segs;                       // segments left, this one included
  int sp, kt, left;                        // where the next stage starts, and the tile rows left in this segment
  int sp1, kt1, left1, sp2, kt2, left2;    // the segments after this one
  __device__ __forceinline__ void start(const Segments &s, int kt_count, int units_per_stage) {
    KT = kt_count, ups = units_per_stage, segs = s.n;
    sp = (int)(s.a[0] / KT), kt = (int)(s.a[0] % KT), left = (int)(s.b[0] - s.a[0]);
    sp1 = (int)(s.a[1] / KT), kt1 = (int)(s.a[1] % KT), left1 = (int)(s.b[1] - s.a[1]);
    sp2 = (int)(s.a[2] / KT), kt2 = (int)(s.a[2] % KT), left2 = (int)(s.b[2] - s.a[2]);
  }
  __device__ __forceinline__ bool more() const { return segs > 0; }
  __device__ __forceinline__ int rows() const { return min(min(ups, left), KT - kt); }
  // past `n` tile rows that end at the sub-panel's end or at the segment's
  __device__ __forceinline__ void skip(int n) { next(n); }
  __device__ __forceinline__ void next(int n) {
    left -= n, kt += n;
    if (kt == KT) kt = 0, sp++;
    if (left == 0) segs--, sp = sp1, kt = kt1, left = left1, sp1 = sp2, kt1 = kt2, left1 = left2;
  }
};

// ---- producers: two warps walk the whole queue ---------------------------------------------------------------
// Warp 8 copies weights, warp 9 copies x. Both follow the same stages through the ring and wait for the same room
// (the oldest stage in the ring freed by the consumers), each keeping its own books, so neither waits for the other.
// Weights never depend on an earlier matmul: their copies go out as soon as the ring has room, lane 0 announcing
// the bytes and lanes 0 and 1 issuing one bulk copy per weight matrix. x is the result of an earlier matmul: the x
// warp waits (with a limit) until every CTA has reported the matmuls it depends on finished, then copies each stage's
// x tiles: whole with one bulk copy for more than 16 token rows, else the first half of each tile (token rows 0-15),
// one copy per tile issued from as many lanes at once (an asynchronous copy costs its issuer some 250 cycles
// whatever its size, which rules out copying row by row). While the x warp waits, the weight warp fills the ring.
template <bool WEIGHTS>
__device__ __forceinline__ void produce(const Queue &q, uint8_t *smem, uint32_t sbase, int cta, int ctas) {
  const uint32_t full0 = sbase + kSmFull, empty0 = sbase + kSmEmpty, ring0 = sbase + kSmRing;
  volatile uint32_t *held = reinterpret_cast<volatile uint32_t *>(smem + kSmHeld) + (WEIGHTS ? 0 : kBars);   // ring bytes of each stage in the ring
  const int lane = threadIdx.x & 31;
  Ring ring{0, 0, 0};
  uint32_t count = 0, oldest = 0, used = 0;   // stages placed; first stage not yet known to be free; ring bytes held from there on
  for (int i = 0; i < q.n; i++) {
    const GemvParams &p = q.op[i];
    const Geometry g = geometry(p.fmt, p.pair != 0, p.tg);
    const int KT = p.KT, nw = p.pair ? 2 : 1;
    const long long units = (long long)((p.TC + kWC - 1) / kWC) * KT;
    const int active = p.per > 0 ? (int)((units + p.per - 1) / p.per) : (int)min((long long)ctas, units);   // the other ranges are empty
    const int me = (cta + p.turn) % ctas;                    // the range this CTA takes in this matmul
    if (me >= active) continue;
    Walk walk;
    walk.start(segments_of(range_start(units, me, active, p.per), range_start(units, me + 1, active, p.per), KT), KT, g.ups);
    const uint8_t *w = p.w[lane < nw ? lane : 0];
    bool gate = !WEIGHTS;                 // the x warp has yet to wait for the matmul before this one
    for (int stage_no = 0; walk.more(); stage_no++) {
      const int n = walk.rows(), sp = walk.sp, kt = walk.kt;
      walk.next(n);
      // room: the stage's bytes plus what is skipped when it starts over at the ring's beginning
      const uint32_t need = g.stage + (ring.off + g.stage > kRingBytes ? kRingBytes - ring.off : 0);
      for (uint32_t spins = 0; used + need > kRingBytes || count - oldest == kBars;) {
        // looking in a loop rather than sleeping in the instruction: a sleeper is woken some hundreds of ns late, and
        // this latency is on the ring's critical path; the two producer warps are 2 of 20, so the polls are cheap
        int ok = 0;
        if (lane == 0) ok = mbar_test(empty0 + 8 * (oldest % kBars), (oldest / kBars) & 1);
        if (__shfl_sync(0xFFFFFFFFu, ok, 0)) {
          used -= held[oldest % kBars], oldest++;
        } else if (++spins > kSpinLimit * 4096) {
          if (lane == 0) atomicExch(q.error, 1);
          break;
        }
      }
      const uint32_t b = count % kBars, stage = ring0 + ring.place(g.stage);
      if (lane == 0) held[b] = need;
      if (WEIGHTS) {
        const int width = min(kWC, p.TC - sp * kWC);
        const uint32_t bytes = n * width * g.tb;
        if (lane == 0) mbar_expect_tx(full0 + 8 * b, nw * bytes);
        __syncwarp();
        if (lane < nw) bulk_g2s(stage + lane * g.matrix, w + ((size_t)sp * kWC * KT + (size_t)kt * width) * g.tb, bytes, full0 + 8 * b);
      } else {
        if (gate) {
          // x may be the result of the launch before this one, or of an earlier matmul of this one: the host has
          // worked out the last matmul this one must see finished, by every CTA
          int ok = 1;
          if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");     // returns when the previous launch is complete and visible
            if (p.wait_for >= 0) {
              uint32_t spins = 0;
              while (ld_acquire_gpu(q.ops_done + p.wait_for) < ctas) {
                if (++spins > kSpinLimit * 32) { ok = 0; break; }
                __nanosleep(32);
              }
            }
          }
          if (!__shfl_sync(0xFFFFFFFFu, ok, 0) && lane == 0) atomicExch(q.error, 5);
          // x was written with ordinary stores (by other CTAs of this launch, or by the launch before) and is about to
          // be read by bulk copies: order what the acquire made visible before the asynchronous proxy's reads
          fence_proxy_async();
          gate = false;
        }
        if (p.tg == 4) {
          if (lane == 0) {
            mbar_expect_tx(full0 + 8 * b, n * 2048);
            bulk_g2s(stage + g.w_bytes, p.x + (size_t)kt * 2048, n * 2048, full0 + 8 * b);
          }
        } else {
          // up to 16 token rows: the first half of each x tile, one copy per tile from as many lanes
          if (lane == 0) mbar_expect_tx(full0 + 8 * b, n * 1024);
          __syncwarp();
          if (lane < n) bulk_g2s(stage + g.w_bytes + lane * 1024, p.x + (size_t)(kt + lane) * 2048, 1024, full0 + 8 * b);
        }
      }
      used += need, count++;
    }
  }
}

// ---- consumers: one matmul of the queue -------------------------------------------------------------------------
template <int FMT, int TG, bool PAIR>
__device__ __forceinline__ void consume(const Queue &q, const GemvParams &p, const Scratch &sc, Ring &ring, uint8_t *smem, uint32_t sbase, int cta, int ctas) {
  constexpr Geometry G = geometry(FMT, PAIR, TG);
  constexpr int ACC = 8 * TG;                                  // accumulator floats per lane
  const uint32_t full0 = sbase + kSmFull, empty0 = sbase + kSmEmpty;
  float *arg_v = reinterpret_cast<float *>(smem + kSmArgVal);
  int *arg_i = reinterpret_cast<int *>(smem + kSmArgIdx);
  float *red = reinterpret_cast<float *>(smem + kSmRed);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, ck = warp >> 2, cc = warp & 3, tl = lane & 3;
  const int KT = p.KT, subpanels = (p.TC + kWC - 1) / kWC;
  const long long units = (long long)subpanels * KT;
  const int active = p.per > 0 ? (int)((units + p.per - 1) / p.per) : (int)min((long long)ctas, units);   // the other ranges are empty
  // The ranges go round the CTAs from matmul to matmul: the CTAs that finish shared sub-panels have more to do than
  // the others, and it should not be the same ones every time.
  const int me = (cta + p.turn) % ctas;
  if (me >= active) return;
  Walk walk;
  walk.start(segments_of(range_start(units, me, active, p.per), range_start(units, me + 1, active, p.per), KT), KT, G.ups);

  float acc[2][TG][4];
// accumulator i of the lane, with i a compile-time constant after unrolling, so that acc stays in registers
#define ACC_OF(a, i) a[(i) / (4 * TG)][(i) / 4 % TG][(i) % 4]
#pragma unroll
  for (int i = 0; i < ACC; i++) ACC_OF(acc, i) = 0.f;

  // shared-memory addresses of this lane's pieces, relative to a stage: its 16 bytes of a tile's values, its exponents
  // and its rows of an x tile
  const uint32_t matrix0 = sbase + kSmRing + (PAIR ? ck * G.matrix : 0);
  const uint32_t lane_tile = matrix0 + lane * 16, lane_ex = matrix0 + tl * 16, lane_x = sbase + kSmRing + G.w_bytes + lane * 8;
  const bool mine = PAIR || ck == 0;       // this warp holds sums when a sub-panel ends
  const int slab = PAIR ? warp : cc;       // and this is their place in a slot of partial sums
  bool first_stage = true;
  int stage_no = 0;
  const int TC = p.TC;
  uint32_t slot = 0;
  // A stage: find its place in the ring and wait for its weights and x; when done with it, free it.
  auto stage_begin = [&]() {
    slot = ring.place(G.stage);
    if (!mbar_wait(full0 + ring.bar, ring.parity, kSpinLimit)) atomicExch(q.error, 2);
    first_stage = false;
  };
  auto stage_end = [&]() {
    __syncwarp();
    mbar_arrive_if(empty0 + ring.bar, lane == 0);
    ring.advance();
    stage_no++;
  };
  while (walk.more()) {
    // one piece: the rest of this sub-panel's share of the range, as whole stages and then what is left
    const int sp = walk.sp, col = sp * kWC + cc, done_sp = sp, width = min(kWC, TC - sp * kWC);
    int todo = min(walk.left, KT - walk.kt);
    walk.skip(todo);
    const bool last_stage = !walk.more();
    {
      if (width == kWC) {
        // full stages of a full run: every offset is a compile-time constant
        for (; todo >= G.ups; todo -= G.ups) {
          stage_begin();
#pragma unroll
          for (int j = 0; j < G.t; j++) {
            const uint32_t row = PAIR ? j : 2 * j + ck, o = slot + (row * kWC + cc) * G.tb;
            tile_mma<FMT, TG>(lane_tile + o, lane_ex + o, lane_x + slot + row * G.xb, acc);
          }
          stage_end();
        }
      }
      while (todo > 0) {
        const int n = min(G.ups, todo);
        todo -= n;
        stage_begin();
        if (col < TC) {
#pragma unroll
          for (int j = 0; j < G.t; j++) {
            const int row = PAIR ? j : 2 * j + ck;
            if (row < n) {
              const uint32_t o = slot + (row * width + cc) * G.tb;
              tile_mma<FMT, TG>(lane_tile + o, lane_ex + o, lane_x + slot + row * G.xb, acc);
            }
          }
        }
        stage_end();
      }

      // ---- this CTA is done with sub-panel done_sp: add the k halves, combine with other CTAs, run the epilogue ----
      settle<FMT, TG>(acc);
      if (!PAIR) {
        // eight accumulators per lane at a time go through the 4 KiB buffer
#pragma unroll
        for (int r = 0; r < TG; r++) {
          if (r > 0) named_barrier(1, kCW * 32);
          if (ck == 1) {
#pragma unroll
            for (int i = 0; i < 8; i++) red[(cc * 8 + i) * 32 + lane] = ACC_OF(acc, 8 * r + i);
          }
          named_barrier(1, kCW * 32);
          if (ck == 0) {
#pragma unroll
            for (int i = 0; i < 8; i++) ACC_OF(acc, 8 * r + i) += red[(cc * 8 + i) * 32 + lane];
          }
        }
      }
      const int first = cta_of((long long)done_sp * KT, units, active, p.per), last = cta_of((long long)(done_sp + 1) * KT - 1, units, active, p.per);
      const bool finish = me == last;         // the owner finishes the sub-panel; the others only contribute
      if (first != last) {
        int *counter = sc.counters + done_sp;
        if (!finish) {
          // a contributor has one shared sub-panel that it does not own, so one slot per CTA is enough
          if (mine) {
            float4 *slot = reinterpret_cast<float4 *>(sc.partials + (size_t)me * q.slot_floats) + (size_t)slab * (ACC / 4) * 32;
#pragma unroll
            for (int i = 0; i < ACC / 4; i++)
              slot[i * 32 + lane] = make_float4(ACC_OF(acc, 4 * i), ACC_OF(acc, 4 * i + 1), ACC_OF(acc, 4 * i + 2), ACC_OF(acc, 4 * i + 3));
          }
          // the barrier orders every warp's stores before thread 0's fence, which releases them with the count
          named_barrier(1, kCW * 32);
          if (threadIdx.x == 0) {
            fence_gpu();
            atomicAdd(counter, 1);
          }
        } else {
          // wait, with a limit, until the last - first other contributors have signalled
          if (threadIdx.x == 0) {
            uint32_t spins = 0;
            while (*reinterpret_cast<volatile int *>(counter) < last - first) {
              if (++spins > kSpinLimit * 32) { atomicExch(q.error, 3); break; }
              __nanosleep(64);
            }
            *counter = 0;                      // ready for the next matmul
            fence_gpu();                       // what follows the barrier, in any warp, sees the contributors' sums
          }
          named_barrier(1, kCW * 32);
          if (mine) {
            // this CTA's own sums first, then the others' in CTA order: the result does not depend on timing
            constexpr int BATCH = ACC <= 8 ? 5 : ACC <= 16 ? 3 : 2;   // contributors whose loads are in flight together
            for (int c0 = first; c0 < last; c0 += BATCH) {
              float4 v[BATCH][ACC / 4];
#pragma unroll
              for (int j = 0; j < BATCH; j++) {
                const float4 *slot = reinterpret_cast<const float4 *>(sc.partials + (size_t)(c0 + j) * q.slot_floats) + (size_t)slab * (ACC / 4) * 32;
#pragma unroll
                for (int i = 0; i < ACC / 4; i++) v[j][i] = c0 + j < last ? __ldcg(slot + i * 32 + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
              }
#pragma unroll
              for (int j = 0; j < BATCH; j++) {
#pragma unroll
                for (int i = 0; i < ACC / 4; i++)
                  ACC_OF(acc, 4 * i) += v[j][i].x, ACC_OF(acc, 4 * i + 1) += v[j][i].y, ACC_OF(acc, 4 * i + 2) += v[j][i].z, ACC_OF(acc, 4 * i + 3) += v[j][i].w;
              }
            }
          }
        }
      }
      if (finish) {
        if (PAIR) {
          // the up warp hands its sums to the gate warp of the same column
          float up[2][TG][4];
#pragma unroll
          for (int r = 0; r < TG; r++) {        // eight accumulators per lane at a time
            if (r > 0) named_barrier(1, kCW * 32);
            if (ck == 1) {
#pragma unroll
              for (int i = 0; i < 8; i++) red[(cc * 8 + i) * 32 + lane] = ACC_OF(acc, 8 * r + i);
            }
            named_barrier(1, kCW * 32);
#pragma unroll
            for (int i = 0; i < 8; i++) ACC_OF(up, 8 * r + i) = red[(cc * 8 + i) * 32 + lane];
          }
          if (ck == 0 && col < TC) finish_column<TG, true>(p, acc, up, col, cc, lane, arg_v, arg_i);
        } else if (ck == 0 && col < TC) {
          finish_column<TG, false>(p, acc, acc, col, cc, lane, arg_v, arg_i);
        }
        if (!PAIR && p.epi == BT_EPI_ARGMAX) {
          // the sub-panel's best per token, then, in the last sub-panel to finish, the best over all sub-panels in order
          named_barrier(1, kCW * 32);
          const int wcols = min(kWC, TC - done_sp * kWC);
          if (warp == 0) {
            float v = arg_v[lane];
            int i = arg_i[lane];
            for (int c = 1; c < wcols; c++)
              if (beats(arg_v[c * 32 + lane], arg_i[c * 32 + lane], v, i)) v = arg_v[c * 32 + lane], i = arg_i[c * 32 + lane];
            // offer it to the token's key: a maximum over all sub-panels whatever the order they finish in, so the last
            // one to finish has the answer at hand instead of a pass over every sub-panel's candidates
            if (lane < p.M && i != 0x7FFFFFFF) atomicMax(sc.keys + lane, pick_key(v, i));
            __syncwarp();
            int is_last = 0;
            if (lane == 0) {
              fence_gpu();
              is_last = atomicAdd(sc.panels_done, 1) == subpanels - 1;
            }
            is_last = __shfl_sync(0xFFFFFFFFu, is_last, 0);
            if (is_last) {
              // turns the keys into the answer and leaves the scratch as it found it
              fence_gpu();
              if (lane < p.M) {
                const unsigned long long key = atomicExch(sc.keys + lane, 0ull);
                uint32_t b = (uint32_t)(key >> 32);
                b ^= b >> 31 ? 0x80000000u : 0xFFFFFFFFu;
                p.arg_val[lane] = key ? __uint_as_float(b) : -INFINITY;
                p.arg_idx[lane] = (key ? (int)(0xFFFFFFFFu - (uint32_t)key) : 0x7FFFFFFF) + p.arg_base;
              }
              if (lane == 0) *sc.panels_done = 0;
            }
          }
        }
      }
      // the next sub-panel must not overwrite `red` or the argmax staging while a slower warp still reads them
      named_barrier(1, kCW * 32);
#pragma unroll
      for (int i = 0; i < ACC; i++) ACC_OF(acc, i) = 0.f;
    }
  }
#undef ACC_OF
}

__global__ void __launch_bounds__(kThreads, kOcc) gemv_queue_kernel(const __grid_constant__ Queue q) {
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const int warp = threadIdx.x >> 5, cta = blockIdx.x, ctas = gridDim.x;
  // The next launch in the stream may start as soon as there is room for its CTAs: what it does before its own
  // griddepcontrol.wait (set up, prefetch weights) does not depend on this launch.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int s = 0; s < kBars; s++) {
      mbar_init(sbase + kSmFull + 8 * s, 2);        // the announcements of the weight bytes and of the x bytes
      mbar_init(sbase + kSmEmpty + 8 * s, kCW);
    }
    mbar_fence_init();
  }
  __syncthreads();
  if (warp >= kCW) {
    if (warp == kCW) produce<true>(q, smem, sbase, cta, ctas);
    else produce<false>(q, smem, sbase, cta, ctas);
    return;
  }
  Ring ring{0, 0, 0};
  for (int i = 0; i < q.n; i++) {
    const GemvParams &p = q.op[i];
    const Scratch &sc = q.set[i % q.sets];
    const int kind = (p.fmt == BT_BFP4 ? 6 : 0) + (p.pair ? 3 : 0) + (p.tg == 1 ? 0 : p.tg == 2 ? 1 : 2);
    switch (kind) {
      case 0: consume<BT_BFP8, 1, false>(q, p, sc, ring, smem, sbase, cta, ctas); break;
      case 1: consume<BT_BFP8, 2, false>(q, p, sc, ring, smem, sbase, cta, ctas); break;
      case 2: consume<BT_BFP8, 4, false>(q, p, sc, ring, smem, sbase, cta, ctas); break;
      case 3: consume<BT_BFP8, 1, true>(q, p, sc, ring, smem, sbase, cta, ctas); break;
      case 4: consume<BT_BFP8, 2, true>(q, p, sc, ring, smem, sbase, cta, ctas); break;
      case 5: consume<BT_BFP8, 4, true>(q, p, sc, ring, smem, sbase, cta, ctas); break;
      case 6: consume<BT_BFP4, 1, false>(q, p, sc, ring, smem, sbase, cta, ctas); break;
      case 7: consume<BT_BFP4, 2, false>(q, p, sc, ring, smem, sbase, cta, ctas); break;
      case 8: consume<BT_BFP4, 4, false>(q, p, sc, ring, smem, sbase, cta, ctas); break;
      case 9: consume<BT_BFP4, 1, true>(q, p, sc, ring, smem, sbase, cta, ctas); break;
      case 10: consume<BT_BFP4, 2, true>(q, p, sc, ring, smem, sbase, cta, ctas); break;
      default: consume<BT_BFP4, 4, true>(q, p, sc, ring, smem, sbase, cta, ctas); break;
    }
    // Report this CTA done with matmul i: its results and partial sums are visible to the whole GPU before the count
    // moves. A CTA without work in a matmul reports at once, which is harmless: the count of matmul i is complete
    // only when the CTAs that do have work got their x, that is when matmul i - 1 was complete. The last report of
    // the last matmul finds every producer past its last look at the counts, and zeroes them for the next launch.
    // The counts are shared with the launch before this one, which may still be running (this launch may start
    // early): a CTA without work in the first matmul must not report before that launch is complete.
    named_barrier(1, kCW * 32);
    if (threadIdx.x == 0) {
      fence_gpu();
      if (i == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
      if (atomicAdd(q.ops_done + i, 1) == ctas - 1 && i == q.n - 1)
        for (int j = 0; j < q.n; j++) q.ops_done[j] = 0;
    }
  }
}

// ---- host side ---------------------------------------------------------------------------------------------------

int check_op(const char *who, int index, const bt_gemv_op &o) {
  BT_REQUIRE(o.fmt == BT_BFP8 || o.fmt == BT_BFP4, "%s: matmul %d: weights must be bfp8 (8) or bfp4 (4), not %d", who, index, o.fmt);
  BT_REQUIRE(o.epilogue >= BT_EPI_NONE && o.epilogue <= BT_EPI_ARGMAX, "%s: matmul %d: unknown epilogue %d", who, index, o.epilogue);
  BT_REQUIRE(o.M >= 1 && o.M <= 32, "%s: matmul %d: takes 1 to 32 rows of x, not %d", who, index, o.M);
  BT_REQUIRE(o.K > 0 && o.N > 0 && o.K % 32 == 0 && o.N % 32 == 0, "%s: matmul %d: K and N must be positive multiples of 32: %d x %d", who, index, o.K, o.N);
  BT_REQUIRE((o.N / 32 + kWC - 1) / kWC <= kMaxSubPanels, "%s: matmul %d: N = %d is past the %d columns one matmul handles", who, index, o.N,
             kMaxSubPanels * kWC * 32);
  BT_REQUIRE(o.x && o.w && o.x % 16 == 0 && o.w % 16 == 0, "%s: matmul %d: x and w must be 16-byte aligned device addresses", who, index);
  BT_REQUIRE((o.epilogue == BT_EPI_GLU) == (o.w2 != 0) && o.w2 % 16 == 0, "%s: matmul %d: w2 goes with the GLU epilogue, and only with it", who, index);
  BT_REQUIRE(o.add % 4 == 0, "%s: matmul %d: the addend must be 4-byte aligned", who, index);
  if (o.epilogue == BT_EPI_ARGMAX) BT_REQUIRE(o.arg_val && o.arg_idx, "%s: matmul %d: the argmax epilogue needs arg_val and arg_idx", who, index);
  else BT_REQUIRE(o.out && o.out % 8 == 0 && (o.out_dtype == BT_BF16 || o.out_dtype == BT_FP32 || o.out_dtype == BT_FP32_ROWS), "%s: matmul %d: needs an 8-byte aligned bf16 or fp32 result", who, index);
  return BT_OK;
}

// The byte ranges a matmul reads (besides its weights, which no matmul writes) and writes.
struct Range {
  uint64_t a, b;
  bool meets(const Range &o) const { return a < o.b && o.a < b; }
};
int ranges_read(const bt_gemv_op &o, Range *r) {
  int n = 0;
  r[n++] = {o.x, o.x + (uint64_t)(o.K / 32) * 2048};
  if (o.add) r[n++] = {o.add, o.add + (uint64_t)(o.N / 32) * 2048};
  return n;
}
int ranges_written(const bt_gemv_op &o, Range *r) {
  int n = 0;
  if (o.epilogue == BT_EPI_ARGMAX) r[n++] = {o.arg_val, o.arg_val + 4ull * o.M}, r[n++] = {o.arg_idx, o.arg_idx + 4ull * o.M};
  else if (o.out_dtype == BT_FP32_ROWS) r[n++] = {o.out, o.out + 4ull * o.M * o.N};
  else r[n++] = {o.out, o.out + (uint64_t)(o.N / 32) * (o.out_dtype == BT_FP32 ? 4096 : 2048)};
  return n;
}
// `later` must not start before `earlier` is complete: it reads or writes what `earlier` writes, or writes what it reads.
bool depends(const bt_gemv_op &later, const bt_gemv_op &earlier) {
  Range lr[2], lw[2], er[2], ew[2];
  const int nlr = ranges_read(later, lr), nlw = ranges_written(later, lw), ner = ranges_read(earlier, er), new_ = ranges_written(earlier, ew);
  for (int i = 0; i < new_; i++) {
    for (int j = 0; j < nlr; j++) if (ew[i].meets(lr[j])) return true;
    for (int j = 0; j < nlw; j++) if (ew[i].meets(lw[j])) return true;
  }
  for (int i = 0; i < ner; i++)
    for (int j = 0; j < nlw; j++) if (er[i].meets(lw[j])) return true;
  return false;
}

// The last earlier matmul of a launch that matmul `i` of it (ops[i]; the launch starts at ops[0]) must not overtake:
// one whose result it reads (x, the addend) or whose buffers it writes, or that reads what it writes; and, because
// the running scratch exists `sets` times, the matmul `sets` places before it. -1: none.
int wait_for(const bt_gemv_op *ops, int i, int sets) {
  int w = i - sets;
  for (int e = i - 1; e > w && e >= 0; e--)
    if (depends(ops[i], ops[e])) w = e;
  return w < 0 ? -1 : w;
}

// Units per CTA such that range boundaries fall on sub-panel boundaries (a share that divides a sub-panel's K tiles,
// or a whole number of sub-panels), when that keeps enough of the CTAs busy; else 0: equal shares of all CTAs, whose
// ranges straddle sub-panels. With fitted shares a CTA has one piece per matmul instead of up to three, and a
// sub-panel's partial sums come from fewer CTAs. That is worth idle CTAs only while ranges are short and the hand-over
// of partial sums weighs against the streaming: up to kShortRange units per CTA a fitted share is taken if it keeps
// 70 % of the CTAs busy (inside a queue the CTAs left without a share go on to the next matmul), beyond that only if it
// keeps 97 % busy. The choice depends on the shape only, never on a matmul's place in a queue: the way the sums are
// grouped, and with it the last bit of a result, must not change with how matmuls are batched.
constexpr int kShortRange = 96;
int aligned_share(int KT, int subpanels, int ctas, int least_busy_percent) {
  const long long units = (long long)subpanels * KT;
  const int least = (int)((units + ctas - 1) / ctas);
  for (int d = least; d <= 4 * least && d <= units; d++) {
    if (KT % d != 0 && d % KT != 0) continue;
    const long long busy = (units + d - 1) / d;
    return busy * 100 >= (long long)(least <= kShortRange ? least_busy_percent : 97) * ctas ? d : 0;
  }
  return 0;
}

// Whether the last thing this library queued, on any stream, before the current entry-point call was a matmul launch
// on `stream`; and the note that one is being queued now. Entry points stamp g_calls when they select their device.
bool follows_matmul(uint64_t stream) {
  static std::mutex lock;
  static struct { uint64_t stream, stamp; } last[64] = {};
  std::lock_guard<std::mutex> hold(lock);
  const uint64_t now = g_calls.load(std::memory_order_relaxed);
  int slot = -1, spare = 0;
  for (int i = 0; i < 64; i++) {
    if (last[i].stamp && last[i].stream == stream) slot = i;
    if (last[i].stamp < last[spare].stamp) spare = i;
  }
  const bool yes = slot >= 0 && last[slot].stamp + 1 == now;
  if (slot < 0) slot = spare;
  last[slot].stream = stream, last[slot].stamp = now;
  return yes;
}

// Argument checks and the launches shared by the entry points. `scratch` carries the scratch pointers.
int enqueue(const char *who, int device, int n, const bt_gemv_op *ops, const Queue &scratch, uint64_t stream) {
  BT_REQUIRE(n >= 1 && ops, "%s: needs at least one matmul", who);
  for (int i = 0; i < n; i++)
    if (int s = check_op(who, i, ops[i])) return s;
  if (int s = use_device(device)) return s;
  int sms = 0;
  BT_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  // The CTAs of a launch wait for one another, so all of them must fit on the GPU at once.
  static int resident[64] = {};
  if (!resident[device & 63]) {
    BT_CUDA(cudaFuncSetAttribute(gemv_queue_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    int per_sm = 0;
    BT_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv_queue_kernel, kThreads, kSmemBytes));
    if (per_sm < 1) return fail(BT_DEVICE, "%s: the matmul kernel does not fit an SM of device %d", who, device);
    resident[device & 63] = min(per_sm, kOcc);
  }
  const int ctas = min(sms * resident[device & 63], kMaxCtas);
  for (int base = 0; base < n; base += kQueueMax) {
    Queue q = scratch;
    q.n = min(kQueueMax, n - base);
    for (int i = 0; i < q.n; i++) {
      const bt_gemv_op &o = ops[base + i];
      GemvParams &p = q.op[i];
      p.x = as_ptr<uint8_t>(o.x), p.w[0] = as_ptr<uint8_t>(o.w), p.w[1] = as_ptr<uint8_t>(o.w2), p.add = as_ptr<uint16_t>(o.add);
      p.out = as_ptr<void>(o.out), p.arg_val = as_ptr<float>(o.arg_val), p.arg_idx = as_ptr<int>(o.arg_idx);
      p.alpha = o.alpha, p.arg_base = o.arg_base, p.M = o.M, p.KT = o.K / 32, p.TC = o.N / 32, p.epi = o.epilogue, p.out_fp32 = o.out_dtype == BT_FP32 ? 1 : o.out_dtype == BT_FP32_ROWS ? 2 : 0;
      p.fmt = o.fmt, p.pair = o.epilogue == BT_EPI_GLU, p.tg = o.M <= 8 ? 1 : o.M <= 16 ? 2 : 4;
      p.wait_for = wait_for(ops + base, i, scratch.sets);
      p.turn = (int)(((long long)(base + i) * 101) % ctas);
      p.per = aligned_share(p.KT, (p.TC + kWC - 1) / kWC, ctas, 70);
    }
    // Programmatic dependent launch: this grid may begin while the previous launch of the stream is still finishing.
    // It only sets up and prefetches weights until its x warps pass griddepcontrol.wait. Weights read that early must
    // be in place, so the launch overlaps its predecessor only when that was a matmul launch of this file too (which
    // never writes weights): anything else this library queued in between (a cast, a relayout, a copy, a memset)
    // turns the overlap off for the next matmul launch.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas), cfg.blockDim = dim3(kThreads), cfg.dynamicSmemBytes = kSmemBytes, cfg.stream = as_stream(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = base > 0 || follows_matmul(stream) ? 1 : 0;
    BT_CUDA(cudaLaunchKernelEx(&cfg, gemv_queue_kernel, q));
    if (int st = launched("gemv_queue_kernel")) return st;
  }
  return BT_OK;
}

Scratch scratch_at(unsigned char *set) {
  Scratch s;
  s.panels_done = reinterpret_cast<int *>(set + kSetPanelsDone), s.counters = reinterpret_cast<int *>(set + kSetCounters);
  s.keys = reinterpret_cast<unsigned long long *>(set + kSetKeys);
  s.partials = reinterpret_cast<float *>(set + kSetPartials);
  return s;
}

Queue workspace_scratch(uint64_t work) {
  Queue q{};
  unsigned char *base = as_ptr<unsigned char>(work);
  q.error = reinterpret_cast<int *>(base + kWsError), q.ops_done = reinterpret_cast<int *>(base + kWsOpsDone);
  q.sets = kSets;
  for (int s = 0; s < kSets; s++) q.set[s] = scratch_at(base + kWsSets + s * kSetBytes);
  q.slot_floats = (int)kSlotFloatsMax;
  return q;
}

}  // namespace

// ---- the entry point that allocates nothing -------------------------------------------------------------------
// Scratch for bt_gemv_bfp_static lives in this array, inside the library's device image, so a caller that may
// not allocate device memory still has somewhere for the kernel's counters and partial sums. Every device that
// loads the library holds these bytes until the process exits. The layout mirrors the caller-provided workspace
// at reduced limits: up to 8 rows of x, up to kStaticSubPanels sub-panels of 4 tile columns.
namespace {
constexpr int kStaticSubPanels = 4096;                                  // N <= 4096 * 4 * 32 = 524288 columns
constexpr size_t kStaticSlotFloats = 8 * 8 * 32;                        // 8 warps, 8 accumulators per lane
constexpr size_t kStKeys = 256;
constexpr size_t kStCounters = 512;
constexpr size_t kStControlBytes = kStCounters + 4 * (size_t)kStaticSubPanels;   // what must be zero when a call starts
constexpr size_t kStPartials = kStControlBytes;
constexpr size_t kStaticBytes = kStPartials + (size_t)kMaxCtas * kStaticSlotFloats * 4;   // about 2.6 MB
}  // namespace
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

extern "C" {

int bt_gemv_workspace_bytes(int device, size_t *bytes) {
  BT_REQUIRE(bytes, "bt_gemv_workspace_bytes: null result");
  (void)device;
  *bytes = kWsBytes;
  return BT_OK;
}

int bt_gemv_queue(int device, int n, const bt_gemv_op *ops, uint64_t work, size_t work_bytes, uint64_t stream) {
  BT_REQUIRE(work && work % 16 == 0 && work_bytes >= kWsBytes, "bt_gemv_queue: needs %zu bytes of 16-byte aligned scratch, got %zu", kWsBytes, work_bytes);
  return enqueue("bt_gemv_queue", device, n, ops, workspace_scratch(work), stream);
}

int bt_gemv_queue_plan(int n, const bt_gemv_op *ops, int *waits) {
  BT_REQUIRE(n >= 1 && ops && waits, "bt_gemv_queue_plan: needs at least one matmul and somewhere for the answer");
  for (int i = 0; i < n; i++)
    if (int s = check_op("bt_gemv_queue_plan", i, ops[i])) return s;
  for (int i = 0; i < n; i++) {
    const int base = i / kQueueMax * kQueueMax, w = wait_for(ops + base, i - base, kSets);
    waits[i] = w < 0 ? -1 : base + w;
  }
  return BT_OK;
}

int bt_gemv_bfp(int device, int fmt, int epilogue, int M, int K, int N, uint64_t x, uint64_t w, uint64_t w2, uint64_t add,
                float alpha, uint64_t out, int out_dtype, uint64_t arg_val, uint64_t arg_idx, int arg_base, uint64_t work,
                size_t work_bytes, uint64_t stream) {
  BT_REQUIRE(work && work % 16 == 0 && work_bytes >= kWsBytes, "bt_gemv_bfp: needs %zu bytes of 16-byte aligned scratch, got %zu", kWsBytes, work_bytes);
  const bt_gemv_op op = {fmt, epilogue, M, K, N, out_dtype, arg_base, alpha, x, w, w2, add, out, arg_val, arg_idx};
  return enqueue("bt_gemv_bfp", device, 1, &op, workspace_scratch(work), stream);
}

// The device address of g_static_scratch on `device`, looked up once per device. In host code the array's name is
// only a handle for the runtime, not an address a kernel could use, so the address comes from
// cudaGetSymbolAddress, asked with that device current.
static int static_scratch(int device, unsigned char **base) {
  static unsigned char *bases[64] = {};
  BT_REQUIRE(device >= 0 && device < 64, "bt_gemv_bfp_static: device %d is out of range", device);
  if (!bases[device]) {
    if (int s = use_device(device)) return s;
    void *ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || !ptr) return fail(BT_DEVICE, "bt_gemv_bfp_static: no address for the built-in scratch on device %d: %s", device, cudaGetErrorString(e));
    bases[device] = static_cast<unsigned char *>(ptr);
  }
  *base = bases[device];
  return BT_OK;
}

int bt_gemv_bfp_static(int device, int fmt, int epilogue, int M, int K, int N, uint64_t x, uint64_t w, uint64_t w2, uint64_t add,
                       float alpha, uint64_t out, int out_dtype, uint64_t arg_val, uint64_t arg_idx, int arg_base, uint64_t stream) {
  BT_REQUIRE(M <= 8, "bt_gemv_bfp_static: the built-in scratch holds up to 8 rows of x, not %d; use bt_gemv_bfp with your own scratch", M);
  BT_REQUIRE(N <= kStaticSubPanels * 128, "bt_gemv_bfp_static: the built-in scratch holds up to %d columns, not %d; use bt_gemv_bfp with your own scratch",
             kStaticSubPanels * 128, N);
  const bt_gemv_op op = {fmt, epilogue, M, K, N, out_dtype, arg_base, alpha, x, w, w2, add, out, arg_val, arg_idx};
  if (int s = check_op("bt_gemv_bfp_static", 0, op)) return s;
  unsigned char *base = nullptr;
  if (int s = static_scratch(device, &base)) return s;
  if (int s = use_device(device)) return s;
  // the array keeps whatever the last call left: the arrival counters must start at zero. The wait-gave-up word at
  // its start is left alone, so that it stays until bt_gemv_check(device, 0, ...) reads it.
  BT_CUDA(cudaMemsetAsync(base + kWsOpsDone, 0, kStControlBytes - kWsOpsDone, as_stream(stream)));
  Queue scratch{};
  scratch.error = reinterpret_cast<int *>(base + kWsError), scratch.ops_done = reinterpret_cast<int *>(base + kWsOpsDone);
  scratch.sets = 1;
  scratch.set[0].panels_done = reinterpret_cast<int *>(base + 192), scratch.set[0].counters = reinterpret_cast<int *>(base + kStCounters);
  scratch.set[0].keys = reinterpret_cast<unsigned long long *>(base + kStKeys);
  scratch.set[0].partials = reinterpret_cast<float *>(base + kStPartials);
  scratch.slot_floats = (int)kStaticSlotFloats;
  return enqueue("bt_gemv_bfp_static", device, 1, &op, scratch, stream);
}

// Nonzero once a bounded wait inside a launch that used this scratch gave up; the results of that launch are
// then unreliable. Reads the flag back (synchronising the stream) and, if it was set, clears it together with the
// counters a launch that gave up may have left half-counted, so that the next launch starts clean. `work` = 0 means
// the built-in scratch of bt_gemv_bfp_static on `device`.
int bt_gemv_check(int device, uint64_t work, uint64_t stream, int *error) {
  BT_REQUIRE(error, "bt_gemv_check: null result");
  unsigned char *base = as_ptr<unsigned char>(work);
  if (!work) {
    if (int s = static_scratch(device, &base)) return s;
  }
  if (int s = use_device(device)) return s;
  BT_CUDA(cudaMemcpyAsync(error, base + kWsError, 4, cudaMemcpyDeviceToHost, as_stream(stream)));
  BT_CUDA(cudaStreamSynchronize(as_stream(stream)));
  if (*error) {
    if (!work) BT_CUDA(cudaMemsetAsync(base, 0, kStControlBytes, as_stream(stream)));
    else {
      BT_CUDA(cudaMemsetAsync(base, 0, kWsSets, as_stream(stream)));
      for (int s = 0; s < kSets; s++)
        BT_CUDA(cudaMemsetAsync(base + kWsSets + s * kSetBytes, 0, kSetCounters + 4 * (size_t)kMaxSubPanels, as_stream(stream)));
    }
  }
  return BT_OK;
}

}  // extern "C"
