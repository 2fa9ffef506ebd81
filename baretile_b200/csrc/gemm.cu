// Prefill matmul for many token rows: out = epilogue(alpha * x @ W + add), W block-float in streaming layout.
//
// With hundreds of rows the contraction is dense and belongs on the 5th-generation tensor cores. What bounds it on
// one SM is shared-memory bandwidth, not the tensor pipe: every MMA reads its A and B slabs from shared memory while
// TMA writes the next x tiles and the dequantising warps write the next expanded weights. So two CTAs on neighbouring
// SMs work as a pair (a cluster of two, tcgen05 cta_group::2): one MMA of 256 rows x 256 columns takes 128 rows of
// x from each CTA and 128 weight columns from each CTA, so each CTA stages, expands and feeds only half of the
// weights, and each B slab is read from shared memory once for 256 rows instead of once for every 128.
//
// A pair computes a block of 512 (or, for few rows, 256) rows x 256 MMA columns; each CTA holds its rows' fp32
// accumulators in tensor memory (two halves of 256 columns). For a gate/up pair the 256 MMA columns are 128 columns
// of Wg (CTA 0) next to the same 128 columns of Wu (CTA 1), and the epilogue writes silu(gate) * up for 128 columns.
//
// Per 64-deep K block, in each CTA:
//   warp 0   (producer)  TMA-loads its 128 x 64 tiles of x (row-major bf16, 128-byte swizzle), whose bytes complete
//                        directly on the LEADER CTA's "full" barrier (a cta_group::2 load; the leader arms the barrier
//                        for both CTAs' bytes), and bulk-copies its 8 packed weight tiles (one run of the streaming
//                        layout, two tile rows) into a ring.
//   warps 2-9 (dequant)  each takes one packed tile, expands it to exact bf16 in registers the way the decode kernel
//                        does (a mask or byte permute, then a packed multiply-add with the face row's power of two),
//                        and stores it into the B tile in the K-major 128-byte-swizzled layout the MMA reads. The
//                        weights carry a factor 2^-64, undone in the epilogue. When its tile is stored and fenced
//                        for the tensor core, the warp arrives on the leader CTA's "full" barrier (17 arrivals in
//                        all: 8 warps of each CTA and the leader's producer).
//   warp 1   (MMA)       in the leader CTA one lane issues 2 x 4 tcgen05.mma (256 x 256 x 16 each) and commits to
//                        both CTAs; the commit frees the stage for both producers and all dequant warps.
// After the last K block the dequant warps become the epilogue: tcgen05.ld brings 32 rows x 32 columns per warp into
// registers, the addend and the activation are applied, and bf16 (rounded half up) or fp32 goes out in tile layout.
// N needs no alignment (a last run of fewer than 4 tile columns is staged tile row by tile row, a missing run is
// skipped); K is a multiple of 32 (an odd last tile row issues half the MMAs of a K block).
// Every wait is bounded and reports through the error word instead of hanging; both CTAs meet at a cluster barrier
// before either frees its tensor memory or exits, so neither signals a barrier of a CTA that has gone.
#include "common.cuh"
#include "ptx.cuh"
#include "stream_layout.cuh"
#include "tmap.cuh"
#include <cstring>

using namespace bt;

namespace {

constexpr int kBK = 64;                                  // K block
constexpr int kStagesAB = 3, kStagesP = 4;             // four stages of x and weights measured the same as three
constexpr int kDequantWarps = 8;
constexpr int kThreads = (2 + kDequantWarps) * 32;
constexpr uint32_t kWaitLimit = 1u << 14;                // attempts of up to 100 us each

constexpr int kABytes = 128 * 128;                       // one 128-row half of this CTA's x for a K block
constexpr int kBBytes = 128 * 128;                       // this CTA's 128 expanded weight columns for a K block
constexpr int kStageAB = 2 * kABytes + kBBytes;          // 48 KiB

struct GemmParams {
  const uint8_t *w[2];       // packed weights by columns; w[1] only for the gate/up pair
  const uint16_t *add;       // addend tiles (bf16), or null
  size_t add_row_stride;     // datums from one tile row of the addend to the next; 0 when the addend is one row
  void *out;
  int *error;
  float alpha;
  int M, KT, TC, epi, out_fp32, pair;
  int row_blocks;            // blocks of 512 rows
  int whole;                 // pairs of CTAs that take a whole block of 512 rows x 256 MMA columns; the pairs after them
};                           // take half a block (256 rows) each, so that the last wave of the grid is a short one

template <int FMT>
struct Layout {
  static constexpr int TB = tile_bytes(FMT);
  static constexpr int P_STAGE = 8 * TB;                  // packed tiles of one K block: 2 tile rows x 4 tile columns
  static constexpr int AB0 = 1024;                        // barriers and the tensor-memory address live below
  static constexpr int P0 = AB0 + kStagesAB * kStageAB;
  static constexpr int BYTES = P0 + kStagesP * P_STAGE;
};

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp32 accumulator, bf16 A and B, both K-major, N = 256, M = 256 (128 rows in each CTA).
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);

__device__ __forceinline__ float silu(float v) { return __fdividef(v, 1.0f + __expf(-v)); }
__device__ __forceinline__ uint32_t bf16_half_up(float v) { return (__float_as_uint(v) + 0x8000u) >> 16; }

// Expand one packed tile (streaming layout, shared address `tile`) to bf16 and store it as rows [32 c, 32 c + 32) and
// K columns [32 j, 32 j + 32) of the B tile at shared address `b` (K-major, 128-byte rows, 128-byte swizzle: the
// 16-byte chunk index of a row is XORed with the row's index modulo 8). Weights are stored in offset binary: a byte
// (or a masked nibble) zero-extended into a 16-bit lane is the bf16 number code * 2^-133, and one packed fused
// multiply-add with the face row's power of two, minus the offset times it, makes it the exact signed weight
// times 2^(e - 197). A nibble q is worth 16 q: a high nibble stays where it is in its byte (16 * code), a low nibble
// takes 16 times the scale.
template <int FMT>
__device__ __forceinline__ void expand_tile(uint32_t tile, uint32_t b, int c, int j, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const uint4 ev = lds128(tile + t * 16);
  const uint32_t ee[4] = {ev.x, ev.y, ev.z, ev.w};
  uint4 wv[2];
  if (FMT == BT_BFP8) wv[0] = lds128(tile + 64 + lane * 16), wv[1] = lds128(tile + 64 + 512 + lane * 16);
  else wv[0] = lds128(tile + 64 + lane * 16), wv[1] = wv[0];
#pragma unroll
  for (int h = 0; h < 2; h++) {
#pragma unroll
    for (int fs = 0; fs < 2; fs++) {
      const uint32_t ew = ee[2 * h + fs];
      const uint32_t s01 = scale_pair<0>(ew), s23 = scale_pair<1>(ew);
      uint32_t a0, a1, a2, a3;   // channels 2g (a0, a2) and 2g + 1 (a1, a3), four consecutive k each
      if (FMT == BT_BFP8) {
        const uint32_t w0 = fs ? wv[h].z : wv[h].x, w1 = fs ? wv[h].w : wv[h].y;
        const uint32_t n01 = mul_bf16x2(s01, 0x80808080u), n23 = mul_bf16x2(s23, 0x80808080u);   // -128 * 2^-133 * scale
        a0 = fma_bf16x2(w0 & 0x00FF00FFu, s01, n01), a1 = fma_bf16x2(w1 & 0x00FF00FFu, s01, n01);
        a2 = fma_bf16x2(prmt(w0, 0u, 0x4341u), s23, n23), a3 = fma_bf16x2(prmt(w1, 0u, 0x4341u), s23, n23);
      } else {
        const uint32_t wb = h ? (fs ? wv[0].w : wv[0].z) : (fs ? wv[0].y : wv[0].x), wo = prmt(wb, 0u, 0x4341u);
        const uint32_t t01 = mul_bf16x2(s01, 0x41804180u), t23 = mul_bf16x2(s23, 0x41804180u);   // 16 * scale: a nibble q is worth 16 q
        const uint32_t n01 = mul_bf16x2(t01, 0x80088008u), n23 = mul_bf16x2(t23, 0x80088008u);   // -8 * 2^-133 * 16 * scale
        a0 = fma_bf16x2(wb & 0x000F000Fu, t01, n01), a1 = fma_bf16x2(wb & 0x00F000F0u, s01, n01);
        a2 = fma_bf16x2(wo & 0x000F000Fu, t23, n23), a3 = fma_bf16x2(wo & 0x00F000F0u, s23, n23);
      }
      const int n0 = 32 * c + 16 * fs + 2 * g;                       // even, so n0 and n0 + 1 share an 8-row group
      const int chunk = 4 * j + 2 * h + (t >> 1);                    // 16-byte chunk of k = 32 j + 16 h + 4 t
      const uint32_t group = b + (n0 >> 3) * 1024 + (t & 1) * 8;
      sts64(group + (n0 & 7) * 128 + ((chunk ^ (n0 & 7)) << 4), a0, a2);
      sts64(group + ((n0 + 1) & 7) * 128 + ((chunk ^ ((n0 + 1) & 7)) << 4), a1, a3);
    }
  }
}

template <int FMT>
__global__ void __launch_bounds__(kThreads, 1) gemm_kernel(const GemmParams p, const __grid_constant__ CUtensorMap amap) {
  using L = Layout<FMT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);   // swizzled tiles want 1024-byte alignment
  const uint32_t sb = smem_u32(smem);
  const uint32_t full0 = sb, empty0 = sb + 32, pfull0 = sb + 96, pempty0 = sb + 128, acc_full = sb + 160, tmem_slot = sb + 176;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                          // 0: the leader, which issues the MMAs
  const int KB = (p.KT + 1) / 2;                                    // K blocks of 64; the last may hold one tile row
  const int pair_id = blockIdx.x >> 1;
  const int block = pair_id < p.whole ? pair_id : p.whole + ((pair_id - p.whole) >> 1);   // blocks go down the rows first
  const int bc = block / p.row_blocks;                              // block column: 128 output columns (pair) or 256
  const int pair_m0 = (block % p.row_blocks) * 512 + (pair_id < p.whole ? 0 : ((pair_id - p.whole) & 1) * 256);   // first row of the pair's rows
  const int MH = pair_id < p.whole && pair_m0 + 256 < p.M ? 2 : 1;  // halves of 256 rows this pair computes
  if (pair_m0 >= p.M) return;                                       // (both CTAs of the pair: nothing here)
  const int run = p.pair ? bc : 2 * bc + (int)rank;                 // this CTA's run of 4 tile columns
  const int width = min(kPanel, p.TC - run * kPanel);               // tile columns it really has; <= 0: none
  const uint8_t *wsrc = (p.pair ? p.w[rank] : p.w[0]) + (size_t)run * kPanel * p.KT * L::TB;
  auto row0 = [&](int mh) { return pair_m0 + (2 * mh + (int)rank) * 128; };   // first row of this CTA's half mh
  auto a_tile = [&](int s, int mh) { return sb + L::AB0 + s * kStageAB + mh * kABytes; };
  auto b_tile = [&](int s) { return sb + L::AB0 + s * kStageAB + 2 * kABytes; };
  auto p_stage = [&](int ps) { return sb + L::P0 + ps * L::P_STAGE; };
  auto wait = [&](uint32_t bar, uint32_t parity, int code) {
    if (!mbar_wait(bar, parity, kWaitLimit)) atomicExch(p.error, code);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStagesAB; s++) mbar_init(full0 + 8 * s, 1 + 2 * kDequantWarps), mbar_init(empty0 + 8 * s, 1);
    for (int s = 0; s < kStagesP; s++) mbar_init(pfull0 + 8 * s, 1), mbar_init(pempty0 + 8 * s, kDequantWarps);
    mbar_init(acc_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  cluster_sync();                                                   // the peer's barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t *>(smem + 176);

  if (warp == 0) {
    // ---- producer ----
    if (lane == 0) {
      const uint32_t leader_full = map_to_cta(full0, 0);
      auto packed = [&](int kb) {           // the K block's packed tiles of this CTA's run: up to 2 tile rows x 4 tiles
        if (width <= 0) return;
        const int ps = kb % kStagesP, rows = min(2, p.KT - 2 * kb);
        if (kb >= kStagesP) wait(pempty0 + 8 * ps, (kb / kStagesP - 1) & 1, 11);
        mbar_expect_tx(pfull0 + 8 * ps, rows * width * L::TB);
        const uint8_t *src = wsrc + (size_t)(2 * kb) * width * L::TB;
        if (width == kPanel) bulk_g2s(p_stage(ps), src, rows * kPanel * L::TB, pfull0 + 8 * ps);
        else
          for (int j = 0; j < rows; j++) bulk_g2s(p_stage(ps) + j * kPanel * L::TB, src + (size_t)j * width * L::TB, width * L::TB, pfull0 + 8 * ps);
      };
      for (int kb = 0; kb < min(KB, kStagesP - 1); kb++) packed(kb);
      for (int kb = 0; kb < KB; kb++) {
        if (kb + kStagesP - 1 < KB) packed(kb + kStagesP - 1);
        const int s = kb % kStagesAB;
        if (kb >= kStagesAB) wait(empty0 + 8 * s, (kb / kStagesAB - 1) & 1, 12);
        // the x tiles of BOTH CTAs complete on the leader's barrier, which the leader arms for all of them
        if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * MH * kABytes);
        for (int mh = 0; mh < MH; mh++) tma_load_2d_pair(a_tile(s, mh), &amap, kb * kBK, row0(mh), leader_full + 8 * s);   // past M or K: zeros
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the leader CTA alone ----
    if (lane == 0 && rank == 0) {
      for (int kb = 0; kb < KB; kb++) {
        const int s = kb % kStagesAB, steps = 2 * min(2, p.KT - 2 * kb);       // 16-deep MMAs in this K block
        wait(full0 + 8 * s, (kb / kStagesAB) & 1, 13);
        tc_fence_after();
        for (int mh = 0; mh < MH; mh++)
          for (int kk = 0; kk < steps; kk++)
            umma_bf16_pair(tmem + mh * 256, smem_desc(a_tile(s, mh) + kk * 32), smem_desc(b_tile(s) + kk * 32), kIdesc, (kb | kk) != 0);
        umma_commit_pair(empty0 + 8 * s);
      }
      umma_commit_pair(acc_full);
    }
  } else {
    // ---- dequant warps, then the epilogue ----
    const int d = warp - 2, c = d & 3, j = d >> 2;                  // this warp's tile column and tile row in a K block
    const uint32_t leader_full0 = map_to_cta(full0, 0);
    for (int kb = 0; kb < KB; kb++) {
      const int ps = kb % kStagesP, s = kb % kStagesAB;
      if (width > 0) wait(pfull0 + 8 * ps, (kb / kStagesP) & 1, 14);
      if (kb >= kStagesAB) wait(empty0 + 8 * s, (kb / kStagesAB - 1) & 1, 15);
      tc_fence_after();
      if (c < width && 2 * kb + j < p.KT) expand_tile<FMT>(p_stage(ps) + (j * kPanel + c) * L::TB, b_tile(s), c, j, lane);
      fence_async_shared();
      __syncwarp();
      if (lane == 0) {
        if (width > 0) mbar_arrive(pempty0 + 8 * ps);
        mbar_arrive_cluster(leader_full0 + 8 * s);
      }
    }
    wait(acc_full, 0, 16);
    tc_fence_after();
    const int q = warp & 3, ch = d >> 2;                            // tensor-memory lane quarter; column half
    const float unscale = 18446744073709551616.f * p.alpha;         // 2^64: the weights were expanded times 2^-64
    const int out_cols = p.pair ? 128 : 256, chunks = out_cols / 64;  // 32-column chunks for this warp
    const int tile_rows = (p.M + 31) / 32;
#pragma unroll 1
    for (int mh = 0; mh < MH; mh++) {
      const int row = row0(mh) + 32 * q + lane, tr = row >> 5;
      if (tr >= tile_rows) continue;                                // the whole warp is past the tensor's tile rows
#pragma unroll 1
      for (int cc = 0; cc < chunks; cc++) {
        const int col = ch * (out_cols / 2) + 32 * cc;              // first output column of the chunk, within the block
        const int tcol = bc * (out_cols / 32) + (col >> 5);         // its tile column
        if (tcol >= p.TC) continue;
        uint32_t v[32], u[32];
        tmem_ld32(tmem + ((uint32_t)(32 * q) << 16) + mh * 256 + col, v);
        if (p.pair) tmem_ld32(tmem + ((uint32_t)(32 * q) << 16) + mh * 256 + 128 + col, u);
        tmem_ld_wait();
        const int in_tile = ((row >> 4) & 1) * 512 + (row & 15) * 16;    // datum index of (row, 0) in the tile
        float f[32];
        if (p.add) {
          const uint16_t *a = p.add + (size_t)tr * p.add_row_stride + (size_t)tcol * 1024 + (p.add_row_stride ? in_tile : 0);
#pragma unroll
          for (int fcol = 0; fcol < 2; fcol++)
#pragma unroll
            for (int i = 0; i < 2; i++) {
              const uint4 w4 = reinterpret_cast<const uint4 *>(a + fcol * 256)[i];
              const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
              for (int k = 0; k < 4; k++) f[16 * fcol + 8 * i + 2 * k] = __uint_as_float(w[k] << 16), f[16 * fcol + 8 * i + 2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
            }
        }
#pragma unroll
        for (int i = 0; i < 32; i++) {
          float x = __uint_as_float(v[i]) * unscale;
          if (p.add) x += f[i];
          if (p.pair) x = silu(x) * (__uint_as_float(u[i]) * unscale);
          else if (p.epi == BT_EPI_RELU) x = fmaxf(x, 0.f);
          else if (p.epi == BT_EPI_SILU) x = silu(x);
          f[i] = row < p.M ? x : 0.f;
        }
        const size_t tile = (size_t)tr * p.TC + tcol;
        if (p.out_fp32) {
          float *o = static_cast<float *>(p.out) + tile * 1024 + in_tile;
#pragma unroll
          for (int fcol = 0; fcol < 2; fcol++)
#pragma unroll
            for (int i = 0; i < 4; i++)
              reinterpret_cast<float4 *>(o + fcol * 256)[i] = make_float4(f[16 * fcol + 4 * i], f[16 * fcol + 4 * i + 1], f[16 * fcol + 4 * i + 2], f[16 * fcol + 4 * i + 3]);
        } else {
          uint16_t *o = static_cast<uint16_t *>(p.out) + tile * 1024 + in_tile;
#pragma unroll
          for (int fcol = 0; fcol < 2; fcol++)
#pragma unroll
            for (int i = 0; i < 2; i++) {
              uint32_t w[4];
#pragma unroll
              for (int k = 0; k < 4; k++) w[k] = bf16_half_up(f[16 * fcol + 8 * i + 2 * k]) | bf16_half_up(f[16 * fcol + 8 * i + 2 * k + 1]) << 16;
              reinterpret_cast<uint4 *>(o + fcol * 256)[i] = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();                                                   // neither CTA frees or leaves while the other may still use it
  if (warp == 1) tmem_dealloc_pair(tmem, 512);
}

}  // namespace

extern "C" {

int bt_gemm_bfp(int device, int fmt, int epilogue, int M, int K, int N, uint64_t a, uint64_t w, uint64_t w2, uint64_t add, int add_rows,
                float alpha, uint64_t out, int out_dtype, uint64_t work, uint64_t stream) {
  BT_REQUIRE(fmt == BT_BFP8 || fmt == BT_BFP4, "bt_gemm_bfp: weights must be bfp8 (8) or bfp4 (4), not %d", fmt);
  BT_REQUIRE(epilogue >= BT_EPI_NONE && epilogue <= BT_EPI_GLU, "bt_gemm_bfp: the epilogue is none, relu, silu or glu, not %d", epilogue);
  const bool pair = epilogue == BT_EPI_GLU;
  BT_REQUIRE(M >= 1 && K > 0 && N > 0 && K % 32 == 0, "bt_gemm_bfp: needs M >= 1, N >= 1 and K a positive multiple of 32: %d x %d x %d", M, K, N);
  BT_REQUIRE(a && w && out && work && a % 16 == 0 && w % 16 == 0 && out % 16 == 0, "bt_gemm_bfp: needs 16-byte aligned device addresses");
  BT_REQUIRE(pair == (w2 != 0) && w2 % 16 == 0, "bt_gemm_bfp: w2 goes with the GLU epilogue, and only with it");
  BT_REQUIRE(add % 16 == 0 && (!add || add_rows == 1 || add_rows == M), "bt_gemm_bfp: the addend is 16-byte aligned and has 1 or M rows, not %d", add_rows);
  BT_REQUIRE(out_dtype == BT_BF16 || out_dtype == BT_FP32, "bt_gemm_bfp: results are bf16 or fp32");
  if (int s = use_device(device)) return s;
  alignas(64) CUtensorMap amap;
  const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M}, strides[1] = {(uint64_t)K * 2};
  const uint32_t box[2] = {kBK, 128};
  if (int s = make_tmap(&amap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, as_ptr<void>(a), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return s;
  GemmParams p{};
  p.w[0] = as_ptr<uint8_t>(w), p.w[1] = as_ptr<uint8_t>(w2), p.add = as_ptr<uint16_t>(add), p.out = as_ptr<void>(out), p.error = as_ptr<int>(work);
  p.alpha = alpha, p.M = M, p.KT = K / 32, p.TC = (N + 31) / 32, p.epi = epilogue, p.out_fp32 = out_dtype == BT_FP32, p.pair = pair;
  p.add_row_stride = add && add_rows > 1 ? (size_t)p.TC * 1024 : 0;
  const int runs = (p.TC + kPanel - 1) / kPanel, columns = pair ? runs : (runs + 1) / 2;
  p.row_blocks = (M + 511) / 512;
  // One pair of CTAs per pair of SMs is resident. When the blocks do not fill the last wave, the blocks of that wave
  // are cut in two, so that it takes half as long (as long as the halves still fit in one wave).
  int sms = 0;
  BT_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  const int blocks = p.row_blocks * columns, slots = sms / 2 > 0 ? sms / 2 : 1, last = blocks % slots;
  p.whole = blocks >= slots && last > 0 && 2 * last <= slots && M > 256 ? blocks - last : blocks;
  const int pairs = p.whole + 2 * (blocks - p.whole);
  static bool configured[64] = {};
  if (!configured[device & 63]) {
    BT_CUDA(cudaFuncSetAttribute(gemm_kernel<BT_BFP8>, cudaFuncAttributeMaxDynamicSharedMemorySize, Layout<BT_BFP8>::BYTES + 1024));
    BT_CUDA(cudaFuncSetAttribute(gemm_kernel<BT_BFP4>, cudaFuncAttributeMaxDynamicSharedMemorySize, Layout<BT_BFP4>::BYTES + 1024));
    configured[device & 63] = true;
  }
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = (fmt == BT_BFP8 ? Layout<BT_BFP8>::BYTES : Layout<BT_BFP4>::BYTES) + 1024;
  cfg.stream = as_stream(stream);
  cfg.attrs = attr, cfg.numAttrs = 1;
  if (fmt == BT_BFP8) BT_CUDA(cudaLaunchKernelEx(&cfg, gemm_kernel<BT_BFP8>, p, amap));
  else BT_CUDA(cudaLaunchKernelEx(&cfg, gemm_kernel<BT_BFP4>, p, amap));
  return launched("gemm_kernel");
}

}  // extern "C"
