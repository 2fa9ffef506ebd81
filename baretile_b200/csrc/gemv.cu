// Decode matmul for up to 32 token rows: out = epilogue(alpha * x @ W + add), W block-float in streaming layout.
//
// The kernel is bound by HBM: every packed weight byte is read once, by a bulk (TMA) copy into a ring of
// shared-memory stages, and dequantised in registers on its way into a bf16 MMA with fp32 accumulators.
//
// Decomposition ("stream-K"). The weight matrix is cut into sub-panels of WC tile columns. A unit is one tile
// row of one sub-panel (WC tiles). Units are numbered sub-panel by sub-panel and dealt out in equal contiguous
// ranges to one persistent CTA per SM, so every SM streams the same number of bytes whatever the shape. A
// sub-panel that several CTAs share is finished by the CTA that holds its last tile row: the others write their
// fp32 partial sums to scratch and bump a counter; the owner, which takes that sub-panel last, waits for the
// counter (with a limit), adds the partials in CTA order, so results do not depend on timing, and runs the
// epilogue. Contributors never wait, so the owner's wait always ends; it is bounded all the same.
//
// Inside a CTA: warp 16 is the producer. One of its lanes waits for a free stage and announces the stage's bytes
// to the stage's mbarrier; then each lane issues one bulk copy (a run of weights, or a piece of an x tile). The 16 consumer
// warps form a WC x KS grid: warp (ck, cc) takes column cc of the sub-panel and every KS-th tile row of the
// stage, so x tiles in shared memory serve WC warps. A weight tile is four 16x16 faces; a face is one
// m16n8k16 MMA with the face's 16 output channels as the MMA's rows, 16 input channels as its K and up to 8
// tokens as its columns. The 16 weights of a face row share an exponent e: the lane builds bf16 lanes
// (sign << 15 | magnitude), i.e. +-q * 2^-133 as a bf16 subnormal, and multiplies by 2^(e - 64) as a packed bf16
// multiply, which gives q * 2^(e - 133) * 2^-64 exactly; the epilogue multiplies the sums by 2^64.
#include "common.cuh"
#include "ptx.cuh"
#include "stream_layout.cuh"
#include "tmap.cuh"
#include <cstring>

using namespace bt;

namespace {

constexpr int kConsumerWarps = 16;
constexpr int kMaxStages = 8;
constexpr int kMaxCtas = 320;
constexpr int kMaxSubPanels = 16384;
constexpr uint32_t kSpinLimit = 1u << 14;   // attempts of up to 100 us each (mbarriers) or 64 ns polls x 32 (counters)
constexpr int kSmemBudget = 225 * 1024;

// Scratch layout (byte offsets into the caller's workspace).
constexpr size_t kWsError = 0;                                   // int: set to nonzero when a wait gave up
constexpr size_t kWsPanelsDone = 4;                              // int: sub-panels finished (argmax epilogue)
constexpr size_t kWsCounters = 256;                              // int[kMaxSubPanels]: CTAs arrived at a sub-panel
constexpr size_t kWsArgVal = kWsCounters + 4 * kMaxSubPanels;    // float[kMaxSubPanels][32]
constexpr size_t kWsArgIdx = kWsArgVal + 4 * 32 * kMaxSubPanels; // int[kMaxSubPanels][32]
constexpr size_t kWsPartials = kWsArgIdx + 4 * 32 * kMaxSubPanels;
constexpr size_t kSlotFloatsMax = 2 * 16 * 2 * 4 * 4 * 32;       // NW * WC * 2 * TG * 4 * 32 at its largest
constexpr size_t kWsBytes = kWsPartials + (size_t)kMaxCtas * kSlotFloatsMax * 4;

struct GemvParams {
  const uint8_t *x;
  const uint8_t *w[2];
  const uint16_t *add;
  void *out;
  float *arg_val;
  int *arg_idx;
  // scratch, zero before first use: a wait-gave-up flag, sub-panels finished (argmax), CTAs arrived per sub-panel,
  // per-sub-panel argmax candidates, and one slot of partial sums per CTA
  int *error, *panels_done, *counters, *part_idx;
  float *part_val, *partials;
  float alpha;
  int arg_base, M, KT, TC, epi, out_fp32, nstages;
  unsigned long long *trace;  // when set: 8 timestamps per CTA (debugging aid)
};

template <int FMT, int NW, int TG, int WC>
struct Config {
  // Two CTAs of 8 consumer warps (plus the producer warp) share an SM, so that a CTA that is starting up, combining
  // partial sums or belongs to the next launch overlaps with one that streams. The widest accumulators (32 rows of a
  // gate/up pair) take one CTA of 12 warps per SM, which leaves each thread 128 registers.
  static constexpr int OCC = WC == 12 ? 1 : 2;
  static constexpr int CW = WC == 12 ? 12 : 8;
  static constexpr int THREADS = (CW + 1) * 32;
  static constexpr int KS = CW / WC;                             // k-slices: warps sharing a column
  static constexpr int T = NW == 2 ? 1 : (FMT == BT_BFP4 && TG == 1 ? 4 : 2);   // tile rows a warp takes per stage
  static constexpr int UPS = KS * T;                             // units (tile rows) per stage
  static constexpr int TB = tile_bytes(FMT);
  static constexpr int XB = TG == 1 ? 512 : TG == 2 ? 1024 : 2048;  // bytes of an x tile staged: rows 0-7, 0-15 or all 32
  static constexpr int W_BYTES = UPS * NW * WC * TB;
  static constexpr int STAGE = (W_BYTES + UPS * XB + 127) / 128 * 128;
  static constexpr int ACC = NW * 2 * TG * 4;                    // accumulator floats per lane
  static constexpr int SLAB = WC * ACC * 32 * 4;                 // one k-slice's accumulators, all columns
  static constexpr int RED_SLABS = KS > 1 ? (24576 / SLAB < 1 ? 1 : 24576 / SLAB < KS - 1 ? 24576 / SLAB : KS - 1) : 0;
  static constexpr int RED = RED_SLABS * SLAB;                   // cross-warp reduction buffer
  static constexpr int FIXED = 4352 + RED;                       // barriers, flags, argmax staging, reduction buffer
  static constexpr size_t SLOT = (size_t)WC * ACC * 32;          // floats in one partial slot
};

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#ifdef BT_GEMV_TRACE
#define BT_TRACE(slot, cond) do { if (p.trace && (cond)) p.trace[blockIdx.x * 8 + (slot)] = global_ns(); } while (0)
#else
#define BT_TRACE(slot, cond) do { } while (0)
#endif

__device__ __forceinline__ long long range_start(long long units, int b, int ctas) { return units * b / ctas; }
__device__ __forceinline__ int cta_of(long long u, long long units, int ctas) {
  int b = (int)(u * ctas / units);
  while (b + 1 < ctas && range_start(units, b + 1, ctas) <= u) b++;
  while (b > 0 && range_start(units, b, ctas) > u) b--;
  return b;
}

// bf16 lanes 2^(e + 63 - 127) for two exponent bytes of `ew` (bytes 0,1 for HI = 0; bytes 2,3 for HI = 1).
template <int HI>
__device__ __forceinline__ uint32_t scale_pair(uint32_t ew) {
  return prmt(ew, 0u, HI ? 0x4342u : 0x4140u) * 128u + 0x1F801F80u;
}

// One weight tile times the staged x tile, added into acc[ng][tg][4]. `tile` and `xs` are shared-memory addresses
// that already include the lane's own offsets: tile = tile base + 16 * lane; xs = x tile base + 32 * g + 8 * t
// (g = lane / 4, t = lane % 4); `ex` = tile base + 16 * t, where the lane's exponents are.
template <int FMT, int TG>
__device__ __forceinline__ void tile_mma(uint32_t tile, uint32_t ex, uint32_t xs, float (&acc)[2][TG][4]) {
  const uint4 ev = lds128(ex);
  const uint32_t ee[4] = {ev.x, ev.y, ev.z, ev.w};
  uint4 wv[2];
  if (FMT == BT_BFP8) wv[0] = lds128(tile + 64), wv[1] = lds128(tile + 64 + 512);
  else wv[0] = lds128(tile + 64), wv[1] = wv[0];
  uint2 bx[2][TG];
#pragma unroll
  for (int h = 0; h < 2; h++) {
#pragma unroll
    for (int tg = 0; tg < TG; tg++) bx[h][tg] = lds64(xs + (TG == 1 ? h * 256 : (tg >> 1) * 1024 + h * 512 + (tg & 1) * 256));
  }
#pragma unroll
  for (int h = 0; h < 2; h++) {
#pragma unroll
    for (int fs = 0; fs < 2; fs++) {
      const uint32_t ew = ee[2 * h + fs];
      const uint32_t s01 = scale_pair<0>(ew), s23 = scale_pair<1>(ew);
      uint32_t m0, s0, m1, s1;  // magnitude and sign bytes of MMA rows g (channel 2g) and g + 8 (channel 2g + 1)
      if (FMT == BT_BFP8) {
        const uint32_t w0 = fs ? wv[h].z : wv[h].x, w1 = fs ? wv[h].w : wv[h].y;
        m0 = w0 & 0x7F7F7F7Fu, s0 = w0 & 0x80808080u, m1 = w1 & 0x7F7F7F7Fu, s1 = w1 & 0x80808080u;
      } else {
        const uint32_t wb = h ? (fs ? wv[0].w : wv[0].z) : (fs ? wv[0].y : wv[0].x), wl = wb << 4;
        m0 = wl & 0x70707070u, s0 = wl & 0x80808080u, m1 = wb & 0x70707070u, s1 = wb & 0x80808080u;
      }
      const uint32_t a0 = mul_bf16x2(prmt(m0, s0, 0x5140u), s01), a1 = mul_bf16x2(prmt(m1, s1, 0x5140u), s01);
      const uint32_t a2 = mul_bf16x2(prmt(m0, s0, 0x7362u), s23), a3 = mul_bf16x2(prmt(m1, s1, 0x7362u), s23);
#pragma unroll
      for (int tg = 0; tg < TG; tg++) mma_bf16(acc[fs][tg], a0, a1, a2, a3, bx[h][tg].x, bx[h][tg].y);
    }
  }
}

__device__ __forceinline__ float silu(float v) { return __fdividef(v, 1.0f + __expf(-v)); }
__device__ __forceinline__ uint32_t bf16_half_up(float v) { return (__float_as_uint(v) + 0x8000u) >> 16; }
__device__ __forceinline__ float bf16_value(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
// a beats b: larger value, or the same value at a lower column; -0 equals 0; a NaN never wins
__device__ __forceinline__ bool beats(float av, int ai, float bv, int bi) { return av > bv || (av == bv && ai < bi); }


// The epilogue of one finished tile column. Lane (g, t) holds, for each channel group ng and token group tg,
// tokens 8 tg + 2t + j (j = 0, 1) and channels 16 ng + 2g + {0, 1}: acc[..][ng][tg][j] and [2 + j].
template <int NW, int TG>
__device__ __forceinline__ void finish_column(const GemvParams &p, const float (&acc)[NW][2][TG][4], int col, int cc, int lane,
                                              float *arg_v, int *arg_i) {
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
        float v0 = acc[0][ng][tgs][j] * unscale, v1 = acc[0][ng][tgs][2 + j] * unscale;
        if (p.add) {
          const uint32_t a = *reinterpret_cast<const uint32_t *>(p.add + (size_t)col * 1024 + at);
          v0 += bf16_value((uint16_t)a), v1 += bf16_value((uint16_t)(a >> 16));
        }
        if (p.epi == BT_EPI_RELU) v0 = fmaxf(v0, 0.f), v1 = fmaxf(v1, 0.f);
        else if (p.epi == BT_EPI_SILU) v0 = silu(v0), v1 = silu(v1);
        else if (NW == 2) v0 = silu(v0) * (acc[NW - 1][ng][tgs][j] * unscale), v1 = silu(v1) * (acc[NW - 1][ng][tgs][2 + j] * unscale);
        if (p.epi == BT_EPI_ARGMAX) {
          if (tg <= kLast && m < p.M) {
            const int n0 = col * 32 + 16 * ng + 2 * g;
            if (beats(v0, n0, best_v[tgs][j], best_i[tgs][j])) best_v[tgs][j] = v0, best_i[tgs][j] = n0;
            if (beats(v1, n0 + 1, best_v[tgs][j], best_i[tgs][j])) best_v[tgs][j] = v1, best_i[tgs][j] = n0 + 1;
          }
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

template <int FMT, int NW, int TG, int WC>
__global__ void __launch_bounds__((Config<FMT, NW, TG, WC>::THREADS), (Config<FMT, NW, TG, WC>::OCC)) gemv_kernel(const GemvParams p, const __grid_constant__ CUtensorMap xmap) {
  using C = Config<FMT, NW, TG, WC>;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t full0 = sbase, empty0 = sbase + 64;
  int *flags = reinterpret_cast<int *>(smem + 128);               // [0], [1]: last-arriver verdicts
  float *arg_v = reinterpret_cast<float *>(smem + 256);           // [16][32] best value per column warp and token
  int *arg_i = reinterpret_cast<int *>(smem + 256 + 2048);        // [16][32] and its channel
  float *red = reinterpret_cast<float *>(smem + 4352);
  constexpr int kStageBase = (C::FIXED + 127) / 128 * 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ctas = gridDim.x, cta = blockIdx.x, KT = p.KT;
  const int subpanels = (p.TC + WC - 1) / WC;
  const long long units = (long long)subpanels * KT;
  const long long u0 = range_start(units, cta, ctas), u1 = range_start(units, cta + 1, ctas);
  const Segments seg = segments_of(u0, u1, KT);
  int *error = p.error;

  BT_TRACE(0, threadIdx.x == 0);
  // The next launch in the stream may start as soon as there is room for its CTAs: what it does before its own
  // griddepcontrol.wait (set up, prefetch weights) does not depend on this launch.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.nstages; s++) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, C::CW);
    }
    mbar_fence_init();
  }
  __syncthreads();
  BT_TRACE(1, threadIdx.x == 0);

  if (warp == C::CW) {
    // ---- producer: lane 0 waits for the stage to be free and announces its bytes; then one lane per copy issues it.
    // A bulk copy costs the issuing warp on the order of a hundred cycles whatever its size, so a stage is a few
    // large copies: one per run of weights, and one for the stage's x tiles (a tiled TMA box that picks the rows
    // the MMAs need out of each tile, or for 32 rows the tiles as they are).
    constexpr int RPS = WC / kPanel;             // runs of the streamed layout in a sub-panel
    int s = 0;                 // the stage to fill next
    uint32_t round = 0;        // how many times the ring has wrapped
    // Weights never depend on the launch before this one, x (the previous layer's result) does. So the first pass
    // over the ring issues only the weight copies and notes the x copies; then the warp waits for the previous launch
    // to finish (griddepcontrol.wait) and issues the noted x copies. From there on a stage gets both at once.
    bool released = false;
    int noted = 0, noted_kt[kMaxStages], noted_n[kMaxStages];
    auto copy_x = [&](int stage_index, int kt, int n) {
      const uint32_t bar = full0 + 8 * stage_index, xs = sbase + kStageBase + stage_index * C::STAGE + C::W_BYTES;
      if (TG == 4) bulk_g2s(xs, p.x + (size_t)kt * 2048, n * 2048, bar);
      else tma_load_3d(xs, &xmap, 0, 0, kt, bar);   // tiles past the last read as zeros
    };
    auto release = [&]() {
      asm volatile("griddepcontrol.wait;" ::: "memory");
      if (lane == NW * RPS)
        for (int i = 0; i < noted; i++) copy_x(i, noted_kt[i], noted_n[i]);
      released = true;
    };
    for (int q = 0; q < seg.n; q++) {
      int sp = (int)(seg.a[q] / KT), kt = (int)(seg.a[q] % KT);
      for (int left = (int)(seg.b[q] - seg.a[q]); left > 0;) {
        const int n = min(min(C::UPS, left), KT - kt);
        if (!released && round > 0) release();
        const uint32_t bar = full0 + 8 * s, stage = sbase + kStageBase + s * C::STAGE;
        if (lane == 0) {
          if (round > 0 && !mbar_wait(empty0 + 8 * s, (round - 1) & 1, kSpinLimit)) atomicExch(error, 1);
          mbar_expect_tx(bar, n * NW * min(WC, p.TC - sp * WC) * C::TB + (TG == 4 ? n : C::UPS) * C::XB);
        }
        __syncwarp();
        if (lane < NW * RPS) {
          const int m = lane / RPS, r = lane % RPS, run = sp * RPS + r, width = min(kPanel, p.TC - run * kPanel);
          if (width > 0)
            bulk_g2s(stage + (m * RPS + r) * C::UPS * kPanel * C::TB, p.w[m] + ((size_t)run * kPanel * KT + (size_t)kt * width) * C::TB,
                     n * width * C::TB, bar);
        }
        if (released) {
          if (lane == NW * RPS) copy_x(s, kt, n);
        } else {
          noted_kt[noted] = kt, noted_n[noted] = n, noted++;
        }
        left -= n, kt += n;
        if (kt == KT) kt = 0, sp++;
        if (++s == p.nstages) s = 0, round++;
      }
    }
    if (!released) release();
    BT_TRACE(5, lane == 0);
    return;
  }

  // ---- consumers ----
  const int ck = warp / WC, cc = warp % WC;
  constexpr int RPS = WC / kPanel;
  const int warp_tile = ((cc / kPanel) * C::UPS * kPanel + cc % kPanel) * C::TB;   // this warp's column inside a stage
  float acc[NW][2][TG][4];
// accumulator i of the lane, with i a compile-time constant after unrolling, so that acc stays in registers
#define ACC_AT(i) acc[(i) / (8 * TG)][(i) / (4 * TG) % 2][(i) / 4 % TG][(i) % 4]
#pragma unroll
  for (int i = 0; i < C::ACC; i++) ACC_AT(i) = 0.f;

  const int g = lane >> 2, tl = lane & 3;
  // shared-memory addresses of this lane's pieces, relative to a stage: its 16 bytes of a tile's values, its exponents
  // and its rows of an x tile
  const uint32_t lane_tile = sbase + kStageBase + warp_tile + lane * 16, lane_ex = sbase + kStageBase + warp_tile + tl * 16;
  const uint32_t lane_x = sbase + kStageBase + C::W_BYTES + g * 32 + tl * 8;
  int s = 0;
  uint32_t round = 0;
  bool first_stage = true;
  for (int q = 0; q < seg.n; q++) {
    int sp = (int)(seg.a[q] / KT), kt = (int)(seg.a[q] % KT);
    for (int left = (int)(seg.b[q] - seg.a[q]); left > 0;) {
      const int n = min(min(C::UPS, left), KT - kt);
      if (!mbar_wait(full0 + 8 * s, round & 1, kSpinLimit)) atomicExch(error, 2);
      BT_TRACE(2, threadIdx.x == 0 && first_stage);
      first_stage = false;
      const int col = sp * WC + cc;
      if (col < p.TC) {
        const int width = min(kPanel, p.TC - (sp * RPS + cc / kPanel) * kPanel);   // tiles of a tile row in this run
        if (n == C::UPS && width == kPanel) {
          // a full stage of a full run: every offset is a compile-time constant
          const uint32_t so = s * C::STAGE + ck * (kPanel * C::TB), xo = s * C::STAGE + ck * C::XB;
#pragma unroll
          for (int j = 0; j < C::T; j++) {
#pragma unroll
            for (int m = 0; m < NW; m++) {
              constexpr int kMatrix = RPS * C::UPS * kPanel * C::TB;
              const uint32_t o = so + m * kMatrix + j * (C::KS * kPanel * C::TB);
              tile_mma<FMT, TG>(lane_tile + o, lane_ex + o, lane_x + xo + j * (C::KS * C::XB), acc[m]);
            }
          }
        } else {
          const uint32_t so = s * C::STAGE + ck * width * C::TB, xo = s * C::STAGE + ck * C::XB;
#pragma unroll 1
          for (int j = 0; j < C::T; j++) {                      // this warp's tile rows of the stage: ck, ck + KS, ...
            if (ck + j * C::KS < n) {
#pragma unroll
              for (int m = 0; m < NW; m++) {
                const uint32_t o = so + (m * RPS * C::UPS * kPanel + j * C::KS * width) * C::TB;
                tile_mma<FMT, TG>(lane_tile + o, lane_ex + o, lane_x + xo + j * C::KS * C::XB, acc[m]);
              }
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * s);
      if (++s == p.nstages) s = 0, round++;
      left -= n, kt += n;
      BT_TRACE(3, threadIdx.x == 0 && q == seg.n - 1 && left == 0);
      if (left != 0 && kt != KT) continue;
      const int done_sp = sp;
      if (kt == KT) kt = 0, sp++;

      // ---- this CTA is done with sub-panel sp: reduce over k-slices, combine with other CTAs, run the epilogue ----
      if (C::KS > 1) {
        for (int r0 = 1; r0 < C::KS; r0 += C::RED_SLABS) {       // as many k-slices at a time as the buffer holds
          if (ck >= r0 && ck < r0 + C::RED_SLABS) {
#pragma unroll
            for (int i = 0; i < C::ACC; i++) red[(((ck - r0) * WC + cc) * C::ACC + i) * 32 + lane] = ACC_AT(i);
          }
          named_barrier(1, C::CW * 32);
          if (ck == 0) {
            for (int r = r0; r < min(C::KS, r0 + C::RED_SLABS); r++) {
#pragma unroll
              for (int i = 0; i < C::ACC; i++) ACC_AT(i) += red[(((r - r0) * WC + cc) * C::ACC + i) * 32 + lane];
            }
          }
          if (r0 + C::RED_SLABS < C::KS) named_barrier(1, C::CW * 32);
        }
      }
      BT_TRACE(6, threadIdx.x == 0 && q == seg.n - 1 && left == 0);
      const int first = cta_of((long long)done_sp * KT, units, ctas), last = cta_of((long long)(done_sp + 1) * KT - 1, units, ctas);
      const bool finish = cta == last;        // the owner finishes the sub-panel; the others only contribute
      if (first != last) {
        float *partials = p.partials;
        int *counter = p.counters + done_sp;
        if (!finish) {
          // a contributor has one shared sub-panel that it does not own, so one slot per CTA is enough
          if (ck == 0) {
            float4 *slot = reinterpret_cast<float4 *>(partials + (size_t)cta * C::SLOT) + (size_t)cc * (C::ACC / 4) * 32;
#pragma unroll
            for (int i = 0; i < C::ACC / 4; i++)
              slot[i * 32 + lane] = make_float4(ACC_AT(4 * i), ACC_AT(4 * i + 1), ACC_AT(4 * i + 2), ACC_AT(4 * i + 3));
            __threadfence();
          }
          named_barrier(1, C::CW * 32);
          if (threadIdx.x == 0) atomicAdd(counter, 1);
        } else {
          // wait, with a limit, until the last - first other contributors have signalled
          if (threadIdx.x == 0) {
            uint32_t spins = 0;
            while (*reinterpret_cast<volatile int *>(counter) < last - first) {
              if (++spins > kSpinLimit * 32) { atomicExch(error, 3); break; }
              __nanosleep(64);
            }
            *counter = 0;                      // ready for the next launch
          }
          named_barrier(1, C::CW * 32);
          if (ck == 0) {
            __threadfence();
            // this CTA's own sums first, then the others' in CTA order: the result does not depend on timing
            constexpr int BATCH = C::ACC <= 16 ? 4 : C::ACC <= 32 ? 2 : 1;   // contributors whose loads are in flight together
            for (int c0 = first; c0 < last; c0 += BATCH) {
              float4 v[BATCH][C::ACC / 4];
#pragma unroll
              for (int j = 0; j < BATCH; j++) {
                const float4 *slot = reinterpret_cast<const float4 *>(partials + (size_t)(c0 + j) * C::SLOT) + (size_t)cc * (C::ACC / 4) * 32;
#pragma unroll
                for (int i = 0; i < C::ACC / 4; i++) v[j][i] = c0 + j < last ? __ldcg(slot + i * 32 + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
              }
#pragma unroll
              for (int j = 0; j < BATCH; j++) {
#pragma unroll
                for (int i = 0; i < C::ACC / 4; i++)
                  ACC_AT(4 * i) += v[j][i].x, ACC_AT(4 * i + 1) += v[j][i].y, ACC_AT(4 * i + 2) += v[j][i].z, ACC_AT(4 * i + 3) += v[j][i].w;
              }
            }
          }
        }
      }

      BT_TRACE(7, threadIdx.x == 0 && q == seg.n - 1 && left == 0);
      if (finish && ck == 0 && col < p.TC) finish_column<NW, TG>(p, acc, col, cc, lane, arg_v, arg_i);
      if (p.epi == BT_EPI_ARGMAX && finish) {
        // the sub-panel's best per token, then, in the last sub-panel to finish, the best over all sub-panels in order
        named_barrier(1, C::CW * 32);
        float *part_v = p.part_val;
        int *part_i = p.part_idx;
        const int wcols = min(WC, p.TC - done_sp * WC);
        if (warp == 0) {
          float v = arg_v[lane];
          int i = arg_i[lane];
          for (int c = 1; c < wcols; c++)
            if (beats(arg_v[c * 32 + lane], arg_i[c * 32 + lane], v, i)) v = arg_v[c * 32 + lane], i = arg_i[c * 32 + lane];
          part_v[done_sp * 32 + lane] = v, part_i[done_sp * 32 + lane] = i;
          __threadfence();
        }
        named_barrier(1, C::CW * 32);
        int *done = p.panels_done;
        if (threadIdx.x == 0) flags[1] = atomicAdd(done, 1) == subpanels - 1;
        named_barrier(1, C::CW * 32);
        if (flags[1]) {
          __threadfence();
          if (warp == 0 && lane < p.M) {
            float v = -INFINITY;
            int i = 0x7FFFFFFF;
            for (int qq = 0; qq < subpanels; qq++) {
              const float ov = __ldcg(part_v + qq * 32 + lane);
              const int oi = __ldcg(part_i + qq * 32 + lane);
              if (beats(ov, oi, v, i)) v = ov, i = oi;
            }
            p.arg_val[lane] = v, p.arg_idx[lane] = i + p.arg_base;
          }
          if (threadIdx.x == 0) *done = 0;
        }
      }
      // the next sub-panel's reduction must not overwrite `red` or the flags while a slower warp still reads them
      if (C::KS > 1 || p.epi == BT_EPI_ARGMAX) named_barrier(1, C::CW * 32);
#pragma unroll
      for (int i = 0; i < C::ACC; i++) ACC_AT(i) = 0.f;
    }
  }
  BT_TRACE(4, threadIdx.x == 0);
#undef ACC_AT
}

// ---- host side: pick a configuration, size shared memory, launch ----

int g_wc[3] = {4, 4, 4};  // tile columns per sub-panel for 1, 2 and 4 token groups
int g_stages = 0;          // 0: as many as fit
unsigned long long *g_trace = nullptr;

template <int FMT, int NW, int TG, int WC>
int launch(const GemvParams &base, int sms, cudaStream_t stream) {
  using C = Config<FMT, NW, TG, WC>;
  GemvParams p = base;
  constexpr int kBudget = kSmemBudget / C::OCC - (C::OCC > 1 ? 1024 : 0);     // the runtime keeps 1 KiB per resident CTA
  int fit = (kBudget - (C::FIXED + 127) / 128 * 128) / C::STAGE;
  p.nstages = min(kMaxStages, g_stages > 0 ? min(g_stages, fit) : fit);
  if (p.nstages < 2) return fail(BT_DEVICE, "bt_gemv_bfp: a stage of %d bytes leaves room for %d stages", C::STAGE, p.nstages);
  const int smem = (C::FIXED + 127) / 128 * 128 + p.nstages * C::STAGE;
  static bool configured[64] = {};
  int device = 0;
  BT_CUDA(cudaGetDevice(&device));
  if (!configured[device & 63]) {
    BT_CUDA(cudaFuncSetAttribute(gemv_kernel<FMT, NW, TG, WC>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBudget));
    configured[device & 63] = true;
  }
  const long long units = (long long)((p.TC + WC - 1) / WC) * p.KT;
  const int ctas = (int)min((long long)min(sms * C::OCC, kMaxCtas), units);
  // x as (8 TG rows x 32 bytes, 2 faces, K tiles): a box picks the rows the MMAs read out of UPS consecutive tiles
  alignas(64) CUtensorMap xmap;
  memset(&xmap, 0, sizeof xmap);
  if (TG < 4) {
    const uint64_t dims[3] = {(uint64_t)(64 * TG), 2, (uint64_t)p.KT}, strides[2] = {512, 2048};
    const uint32_t box[3] = {(uint32_t)(64 * TG), 2, (uint32_t)C::UPS};
    if (int st = make_tmap(&xmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, p.x, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE)) return st;
  }
  // Programmatic dependent launch: this grid may begin while the previous launch of the stream is still finishing.
  // It only sets up and prefetches weights until its producer warps pass griddepcontrol.wait.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas), cfg.blockDim = dim3(C::THREADS), cfg.dynamicSmemBytes = smem, cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  BT_CUDA(cudaLaunchKernelEx(&cfg, gemv_kernel<FMT, NW, TG, WC>, p, xmap));
  return launched("gemv_kernel");
}

template <int FMT, int NW, int TG>
int launch_wc(const GemvParams &p, int wc, int sms, cudaStream_t stream) {
  if constexpr (NW == 2 && TG == 4) {
    return launch<FMT, NW, TG, 12>(p, sms, stream);   // the widest accumulators: see Config::CW
  } else {
    if (wc == 8) return launch<FMT, NW, TG, 8>(p, sms, stream);
    return launch<FMT, NW, TG, 4>(p, sms, stream);
  }
}

template <int FMT, int NW>
int launch_tg(const GemvParams &p, int wc_force, int sms, cudaStream_t stream) {
  if (p.M <= 8) return launch_wc<FMT, NW, 1>(p, wc_force ? wc_force : g_wc[0], sms, stream);
  if (p.M <= 16) return launch_wc<FMT, NW, 2>(p, wc_force ? wc_force : g_wc[1], sms, stream);
  return launch_wc<FMT, NW, 4>(p, wc_force ? wc_force : g_wc[2], sms, stream);
}

}  // namespace

// ---- the entry point that allocates nothing -------------------------------------------------------------------
// Scratch for bt_gemv_bfp_static lives in this array, inside the library's device image, so a caller that may
// not allocate device memory still has somewhere for the kernel's counters and partial sums. Every device that
// loads the library holds these bytes until the process exits. The layout mirrors the caller-provided workspace
// at reduced limits: up to 8 rows of x, up to kStaticSubPanels sub-panels of 4 tile columns.
namespace {
constexpr int kStaticSubPanels = 4096;                                  // N <= 4096 * 4 * 32 = 524288 columns
constexpr size_t kStaticSlotFloats = 4 * 16 * 32;                       // WC = 4, up to 16 accumulators per lane
constexpr size_t kStCounters = 256;
constexpr size_t kStControlBytes = kStCounters + 4 * (size_t)kStaticSubPanels;   // what must be zero when a call starts
constexpr size_t kStArgVal = kStControlBytes;
constexpr size_t kStArgIdx = kStArgVal + 4 * 32 * (size_t)kStaticSubPanels;
constexpr size_t kStPartials = kStArgIdx + 4 * 32 * (size_t)kStaticSubPanels;
constexpr size_t kStaticBytes = kStPartials + (size_t)kMaxCtas * kStaticSlotFloats * 4;   // about 3.1 MB
}  // namespace
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

extern "C" {

int bt_gemv_workspace_bytes(int device, size_t *bytes) {
  BT_REQUIRE(bytes, "bt_gemv_workspace_bytes: null result");
  (void)device;
  *bytes = kWsBytes;
  return BT_OK;
}

// Tuning knobs for experiments: tile columns per sub-panel (4, 8 or 16) for up to 8, 16 and 32 token rows, and the
// number of pipeline stages (0 = as many as fit). Values of 0 keep the current setting.
int bt_gemv_tune(int wc_m8, int wc_m16, int wc_m32, int stages) {
  const int wc[3] = {wc_m8, wc_m16, wc_m32};
  for (int i = 0; i < 3; i++) {
    BT_REQUIRE(wc[i] == 0 || wc[i] == 4 || wc[i] == 8, "bt_gemv_tune: sub-panel width must be 4 or 8, not %d", wc[i]);
    if (wc[i]) g_wc[i] = wc[i];
  }
  BT_REQUIRE(stages >= 0 && stages <= kMaxStages, "bt_gemv_tune: stages must be 0..%d", kMaxStages);
  g_stages = stages;
  return BT_OK;
}

// Argument checks and the launch shared by the entry points. `scratch` carries the scratch pointers; wc_force, when
// nonzero, fixes the sub-panel width.
static int gemv_common(const char *who, int device, int fmt, int epilogue, int M, int K, int N, uint64_t x, uint64_t w, uint64_t w2,
                       uint64_t add, float alpha, uint64_t out, int out_dtype, uint64_t arg_val, uint64_t arg_idx, int arg_base,
                       const GemvParams &scratch, int wc_force, uint64_t stream) {
  BT_REQUIRE(fmt == BT_BFP8 || fmt == BT_BFP4, "%s: weights must be bfp8 (8) or bfp4 (4), not %d", who, fmt);
  BT_REQUIRE(epilogue >= BT_EPI_NONE && epilogue <= BT_EPI_ARGMAX, "%s: unknown epilogue %d", who, epilogue);
  BT_REQUIRE(M >= 1 && M <= 32, "%s: takes 1 to 32 rows of x, not %d", who, M);
  BT_REQUIRE(K > 0 && N > 0 && K % 32 == 0 && N % 32 == 0, "%s: K and N must be positive multiples of 32: %d x %d", who, K, N);
  BT_REQUIRE(x && w && x % 16 == 0 && w % 16 == 0, "%s: x and w must be 16-byte aligned device addresses", who);
  BT_REQUIRE((epilogue == BT_EPI_GLU) == (w2 != 0) && w2 % 16 == 0, "%s: w2 goes with the GLU epilogue, and only with it", who);
  BT_REQUIRE(add % 4 == 0, "%s: the addend must be 4-byte aligned", who);
  if (epilogue == BT_EPI_ARGMAX) BT_REQUIRE(arg_val && arg_idx, "%s: the argmax epilogue needs arg_val and arg_idx", who);
  else BT_REQUIRE(out && out % 8 == 0 && (out_dtype == BT_BF16 || out_dtype == BT_FP32), "%s: needs an 8-byte aligned bf16 or fp32 result", who);
  if (int s = use_device(device)) return s;
  int sms = 0;
  BT_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  GemvParams p = scratch;
  p.x = as_ptr<uint8_t>(x), p.w[0] = as_ptr<uint8_t>(w), p.w[1] = as_ptr<uint8_t>(w2), p.add = as_ptr<uint16_t>(add);
  p.out = as_ptr<void>(out), p.arg_val = as_ptr<float>(arg_val), p.arg_idx = as_ptr<int>(arg_idx);
  p.trace = g_trace;
  p.alpha = alpha, p.arg_base = arg_base, p.M = M, p.KT = K / 32, p.TC = N / 32, p.epi = epilogue, p.out_fp32 = out_dtype == BT_FP32;
  cudaStream_t st = as_stream(stream);
  if (fmt == BT_BFP8) return epilogue == BT_EPI_GLU ? launch_tg<BT_BFP8, 2>(p, wc_force, sms, st) : launch_tg<BT_BFP8, 1>(p, wc_force, sms, st);
  return epilogue == BT_EPI_GLU ? launch_tg<BT_BFP4, 2>(p, wc_force, sms, st) : launch_tg<BT_BFP4, 1>(p, wc_force, sms, st);
}

int bt_gemv_bfp(int device, int fmt, int epilogue, int M, int K, int N, uint64_t x, uint64_t w, uint64_t w2, uint64_t add,
                float alpha, uint64_t out, int out_dtype, uint64_t arg_val, uint64_t arg_idx, int arg_base, uint64_t work,
                size_t work_bytes, uint64_t stream) {
  BT_REQUIRE(work && work % 16 == 0 && work_bytes >= kWsBytes, "bt_gemv_bfp: needs %zu bytes of 16-byte aligned scratch, got %zu", kWsBytes, work_bytes);
  BT_REQUIRE(N <= 0 || (N / 32 + 3) / 4 <= kMaxSubPanels, "bt_gemv_bfp: N = %d is past the %d columns one launch handles", N, kMaxSubPanels * 128);
  GemvParams scratch{};
  scratch.error = as_ptr<int>(work + kWsError), scratch.panels_done = as_ptr<int>(work + kWsPanelsDone), scratch.counters = as_ptr<int>(work + kWsCounters);
  scratch.part_val = as_ptr<float>(work + kWsArgVal), scratch.part_idx = as_ptr<int>(work + kWsArgIdx), scratch.partials = as_ptr<float>(work + kWsPartials);
  return gemv_common("bt_gemv_bfp", device, fmt, epilogue, M, K, N, x, w, w2, add, alpha, out, out_dtype, arg_val, arg_idx, arg_base, scratch, 0, stream);
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
  unsigned char *base = nullptr;
  if (int s = static_scratch(device, &base)) return s;
  if (int s = use_device(device)) return s;
  // the array keeps whatever the last call left: flags and arrival counters must start at zero
  BT_CUDA(cudaMemsetAsync(base, 0, kStControlBytes, as_stream(stream)));
  GemvParams scratch{};
  scratch.error = reinterpret_cast<int *>(base), scratch.panels_done = reinterpret_cast<int *>(base + 4);
  scratch.counters = reinterpret_cast<int *>(base + kStCounters);
  scratch.part_val = reinterpret_cast<float *>(base + kStArgVal), scratch.part_idx = reinterpret_cast<int *>(base + kStArgIdx);
  scratch.partials = reinterpret_cast<float *>(base + kStPartials);
  return gemv_common("bt_gemv_bfp_static", device, fmt, epilogue, M, K, N, x, w, w2, add, alpha, out, out_dtype, arg_val, arg_idx, arg_base, scratch,
                     4, stream);
}

// Debugging aid: when `buffer` is nonzero, every later launch writes 8 nanosecond timestamps per CTA into it (kernel
// start, barriers ready, first stage arrived, last stage consumed, kernel end, last copy issued). 0 turns it off.
int bt_gemv_trace(uint64_t buffer) {
  g_trace = as_ptr<unsigned long long>(buffer);
  return BT_OK;
}

// Nonzero once a bounded wait inside a launch that used this scratch gave up; the results of that launch are
// then unreliable. Reads the flag back (synchronising the stream) and clears it.
int bt_gemv_check(int device, uint64_t work, uint64_t stream, int *error) {
  BT_REQUIRE(work && error, "bt_gemv_check: null argument");
  if (int s = use_device(device)) return s;
  BT_CUDA(cudaMemcpyAsync(error, as_ptr<void>(work + kWsError), 4, cudaMemcpyDeviceToHost, as_stream(stream)));
  BT_CUDA(cudaStreamSynchronize(as_stream(stream)));
  if (*error) BT_CUDA(cudaMemsetAsync(as_ptr<void>(work + kWsError), 0, 4, as_stream(stream)));
  return BT_OK;
}

}  // extern "C"
