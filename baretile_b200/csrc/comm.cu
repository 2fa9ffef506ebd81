// Exchanges between the GPUs of one box for layers that are split over them: raw NCCL collectives on the caller's
// stream, so that they queue in order with the matmul launches, and the small kernels either side of them.
//
// The reference has no collective backend: its only transport between chips is a point-to-point tensor copy over
// Ethernet (Tensor.to, baretile/tensor.py:708-726; link_kernel, baretile/kernels.py:1316-1372). The partitioning
// these entry points serve follows the shapes of the path instead:
//   gate/up   split over N: every rank computes SiLU(x Wg) * (x Wu) for its own tile columns; bt_allgather on the
//             bf16 tile buffers rebuilds the [M, N] activations in tile layout as they are (tile columns of a tile
//             row are contiguous, so the ranks' buffers one after another ARE the full tensor's tile row).
//   down      split over K: every rank writes its fp32 partial sums row-major (BT_FP32_ROWS), bt_allreduce_sum adds
//             them over the ranks, bt_round_tilize rounds the sums once to bf16 tiles.
//   LM head   split over the vocabulary: every rank's matmul reduces its logits to (max, first global index) per
//             row; bt_allgather collects the ranks' 256-byte candidate blocks and bt_argmax_combine applies the
//             reference's tie rule (topk_kernel, baretile/kernels.py:1173-1231).
// NCCL is loaded on first use (dlopen), so a process that never shards needs no NCCL at all.
//
// The down projection's exchange also exists without NCCL, as ONE kernel over peer memory (bt_peer_*): every rank
// owns a buffer that the other ranks map through CUDA IPC (NVLink loads and stores, no multicast). The matmul writes
// its fp32 partial rows into the rank's own buffer; bt_peer_allreduce_round then tells every peer "my rows of step e
// are there" (a flag in the PEER's buffer), waits, with a limit, for the peers' flags in its own, and adds the ranks'
// rows straight from their memories in rank order (so every rank gets the same bits), rounds half up and writes bf16
// tiles: the all-reduce, the rounding and the tilizing in one launch, bound by a flag's flight over NVLink and one
// round of peer loads instead of a collective's set-up. The rows alternate between two halves of the buffer from step
// to step: a rank can be at most one step ahead of a peer (it needs the peer's flag of the step it is in), so the
// half it overwrites was read by everyone two steps ago, and no second barrier is needed.
#include "common.cuh"
#include <dlfcn.h>
#include <nccl.h>

using namespace bt;

namespace {

struct Nccl {
  void *lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

int nccl(Nccl **out) {
  static Nccl n;
  if (!n.lib) {
    void *lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    if (!lib) return fail(BT_DEVICE, "NCCL is not available: %s", dlerror());
#define BT_SYM(field, name)                                                        \
    n.field = reinterpret_cast<decltype(n.field)>(dlsym(lib, name));               \
    if (!n.field) return fail(BT_DEVICE, "NCCL lacks %s: %s", name, dlerror());
    BT_SYM(GetUniqueId, "ncclGetUniqueId") BT_SYM(CommInitRank, "ncclCommInitRank") BT_SYM(CommDestroy, "ncclCommDestroy")
    BT_SYM(AllGather, "ncclAllGather") BT_SYM(AllReduce, "ncclAllReduce") BT_SYM(GetErrorString, "ncclGetErrorString")
#undef BT_SYM
    n.lib = lib;
  }
  *out = &n;
  return BT_OK;
}

#define BT_NCCL(n, call)                                                                         \
  do {                                                                                           \
    ncclResult_t r_ = (call);                                                                    \
    if (r_ != ncclSuccess) return fail(BT_DEVICE, "%s: %s", #call, (n)->GetErrorString(r_));     \
  } while (0)

// a beats b: larger value, or the same value at a lower index; -0 equals 0; a NaN never wins
__device__ __forceinline__ bool beats(float av, int ai, float bv, int bi) { return av > bv || (av == bv && ai < bi); }

// blocks: per rank 32 fp32 values then 32 int32 indices (what the matmul's pick writes with arg_idx = arg_val + 32).
__global__ void argmax_combine_kernel(const float *__restrict__ blocks, int world, int rows, float *__restrict__ out_val, int *__restrict__ out_idx) {
  const int m = threadIdx.x;
  if (m >= rows) return;
  float bv = -INFINITY;
  int bi = 0x7FFFFFFF;
  for (int r = 0; r < world; r++) {
    const float v = blocks[r * 64 + m];
    const int i = reinterpret_cast<const int *>(blocks)[r * 64 + 32 + m];
    if (beats(v, i, bv, bi)) bv = v, bi = i;
  }
  out_val[m] = bv, out_idx[m] = bi;
}

// fp32 row-major (rows x cols) -> bf16 tiles of one tile row (rows <= 32), rounded half up like a matmul result
// (docs/compiler.md, "Matmul precision"); rows past `rows` are zero, a single row fills its tile.
__global__ void round_tilize_kernel(const float *__restrict__ src, uint16_t *__restrict__ dst, int rows, int cols) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;   // datum index in the tiled image
  const size_t total = (size_t)((cols + 31) / 32) * 1024;
  if (i >= total) return;
  const int tile = (int)(i / 1024), in = (int)(i % 1024), face = in / 256, r = face / 2 * 16 + in % 256 / 16, c = tile * 32 + face % 2 * 16 + in % 16;
  const int row = rows == 1 ? 0 : r;
  float v = 0.f;
  if (row < rows && c < cols) v = src[(size_t)row * cols + c];
  dst[i] = (uint16_t)((__float_as_uint(v) + 0x8000u) >> 16);
}

// ---- the exchange over peer memory ---------------------------------------------------------------------------
constexpr int kPeerMax = 8;                  // ranks of one box
constexpr size_t kPeerFlags = 0;             // int[kPeerMax]: flags[r] = the last step rank r has announced to this rank
constexpr size_t kPeerError = 256;           // int: a wait for a peer's flag gave up
constexpr size_t kPeerData = BT_PEER_DATA;   // the rows start here
constexpr uint32_t kPeerSpins = 1u << 22;    // polls of about 250 ns: about a second

struct PeerArgs {
  uint8_t *peer[kPeerMax];                   // every rank's buffer as mapped on this device; peer[rank] is the local one
  size_t data;                               // byte offset of this step's rows in every buffer
  uint16_t *dst;
  int rank, world, step, rows, cols;
};

__device__ __forceinline__ int ld_acquire_sys(const int *p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int *p, int v) { asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ float4 ld_volatile_f4(const float *p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

// rows x cols fp32 row-major in every rank's buffer -> their sum, in rank order, as bf16 tiles of one tile row
// (rows <= 32, cols a multiple of 32; rows past `rows` zero, a single row fills its tile).
__global__ void __launch_bounds__(256) peer_allreduce_round_kernel(const PeerArgs a) {
  __shared__ int gave_up;
  if (threadIdx.x == 0) gave_up = 0;
  // this rank's rows were written by the launch before this one in the stream: they are complete and in this GPU's
  // memory, where a peer's loads will find them; announce them to every peer, once
  if (blockIdx.x == 0 && threadIdx.x < a.world && (int)threadIdx.x != a.rank) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<int *>(a.peer[threadIdx.x] + kPeerFlags) + a.rank, a.step);
  }
  __syncthreads();
  if (threadIdx.x < a.world && (int)threadIdx.x != a.rank) {
    const int *flag = reinterpret_cast<const int *>(a.peer[a.rank] + kPeerFlags) + threadIdx.x;
    uint32_t spins = 0;
    while (ld_acquire_sys(flag) - a.step < 0) {                     // steps only grow; the difference survives a wrap
      if (++spins > kPeerSpins) { gave_up = 1; break; }
      __nanosleep(200);
    }
  }
  __syncthreads();
  if (gave_up) {
    if (threadIdx.x == 0) atomicExch(reinterpret_cast<int *>(a.peer[a.rank] + kPeerError), 1);
    return;                                                          // the result stays as it was; the host reads the word
  }
  const int quads = a.cols / 32 * 256;                               // 4 datums each: a tile is 256 quads
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += gridDim.x * blockDim.x) {
    const int tile = i / 256, in = i % 256 * 4, face = in / 256, r = face / 2 * 16 + in % 256 / 16, c = tile * 32 + face % 2 * 16 + in % 16;
    const int row = a.rows == 1 ? 0 : r;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row < a.rows) {
      float4 v[kPeerMax];
#pragma unroll
      for (int k = 0; k < kPeerMax; k++)
        if (k < a.world) v[k] = ld_volatile_f4(reinterpret_cast<const float *>(a.peer[k] + a.data) + (size_t)row * a.cols + c);
#pragma unroll
      for (int k = 0; k < kPeerMax; k++)
        if (k < a.world) sum.x += v[k].x, sum.y += v[k].y, sum.z += v[k].z, sum.w += v[k].w;
    }
    const uint32_t lo = ((__float_as_uint(sum.x) + 0x8000u) >> 16) | ((__float_as_uint(sum.y) + 0x8000u) & 0xFFFF0000u);
    const uint32_t hi = ((__float_as_uint(sum.z) + 0x8000u) >> 16) | ((__float_as_uint(sum.w) + 0x8000u) & 0xFFFF0000u);
    *reinterpret_cast<uint2 *>(a.dst + (size_t)tile * 1024 + in) = make_uint2(lo, hi);
  }
}

// The vocabulary-split pick the same way: this rank's block (32 fp32 values then 32 int32 indices, as the matmul's
// fused pick leaves them) is stored into slot `rank` of every rank's buffer, this rank's included, then the step is
// announced; when every rank's step is here, the blocks in the local buffer are combined with the reference's tie
// rule. One CTA. The slots alternate between two halves of the buffer from step to step, like the rows above.
struct PeerPickArgs {
  uint8_t *peer[kPeerMax];
  size_t data;
  const uint32_t *mine;
  float *out_val;
  int *out_idx;
  int rank, world, step, rows;
};
__global__ void __launch_bounds__(kPeerMax * 64) peer_argmax_combine_kernel(const PeerPickArgs a) {
  __shared__ int gave_up;
  const int to = threadIdx.x / 64, word = threadIdx.x % 64;
  if (threadIdx.x == 0) gave_up = 0;
  if (to < a.world) {
    volatile uint32_t *slot = reinterpret_cast<volatile uint32_t *>(a.peer[to] + a.data) + a.rank * 64;
    slot[word] = a.mine[word];
    __threadfence_system();                                          // the block before the flag, as the peer sees them
  }
  __syncthreads();
  if (threadIdx.x < a.world && (int)threadIdx.x != a.rank) st_release_sys(reinterpret_cast<int *>(a.peer[threadIdx.x] + kPeerFlags) + a.rank, a.step);
  if (threadIdx.x < a.world && (int)threadIdx.x != a.rank) {
    const int *flag = reinterpret_cast<const int *>(a.peer[a.rank] + kPeerFlags) + threadIdx.x;
    uint32_t spins = 0;
    while (ld_acquire_sys(flag) - a.step < 0) {
      if (++spins > kPeerSpins) { gave_up = 1; break; }
      __nanosleep(200);
    }
  }
  __syncthreads();
  if (gave_up) {
    if (threadIdx.x == 0) atomicExch(reinterpret_cast<int *>(a.peer[a.rank] + kPeerError), 1);
    return;
  }
  const int m = threadIdx.x;
  if (m >= a.rows) return;
  const volatile float *blocks = reinterpret_cast<const volatile float *>(a.peer[a.rank] + a.data);
  float bv = -INFINITY;
  int bi = 0x7FFFFFFF;
  for (int r = 0; r < a.world; r++) {
    const float v = blocks[r * 64 + m];
    const int i = reinterpret_cast<const volatile int *>(blocks)[r * 64 + 32 + m];
    if (beats(v, i, bv, bi)) bv = v, bi = i;
  }
  a.out_val[m] = bv, a.out_idx[m] = bi;
}

}  // namespace

extern "C" {

int bt_comm_unique_id(void *id, size_t bytes) {
  BT_REQUIRE(id && bytes >= sizeof(ncclUniqueId), "bt_comm_unique_id: needs %zu bytes for the id", sizeof(ncclUniqueId));
  Nccl *n;
  if (int s = nccl(&n)) return s;
  BT_NCCL(n, n->GetUniqueId(static_cast<ncclUniqueId *>(id)));
  return BT_OK;
}

int bt_comm_init(int device, int rank, int world, const void *id, uint64_t *comm) {
  BT_REQUIRE(id && comm && world >= 1 && rank >= 0 && rank < world, "bt_comm_init: rank %d of %d", rank, world);
  Nccl *n;
  if (int s = nccl(&n)) return s;
  if (int s = use_device(device)) return s;
  ncclUniqueId uid;
  memcpy(&uid, id, sizeof uid);
  ncclComm_t c = nullptr;
  BT_NCCL(n, n->CommInitRank(&c, world, uid, rank));
  *comm = reinterpret_cast<uint64_t>(c);
  return BT_OK;
}

int bt_comm_destroy(uint64_t comm) {
  Nccl *n;
  if (int s = nccl(&n)) return s;
  if (comm) BT_NCCL(n, n->CommDestroy(reinterpret_cast<ncclComm_t>(comm)));
  return BT_OK;
}

int bt_allgather(int device, uint64_t comm, uint64_t src, uint64_t dst, size_t bytes, uint64_t stream) {
  BT_REQUIRE(comm && src && dst && bytes, "bt_allgather: null argument");
  Nccl *n;
  if (int s = nccl(&n)) return s;
  if (int s = use_device(device)) return s;
  BT_NCCL(n, n->AllGather(as_ptr<void>(src), as_ptr<void>(dst), bytes, ncclUint8, reinterpret_cast<ncclComm_t>(comm), as_stream(stream)));
  return BT_OK;
}

int bt_allreduce_sum(int device, uint64_t comm, uint64_t buf_f32, size_t count, uint64_t stream) {
  BT_REQUIRE(comm && buf_f32 && count, "bt_allreduce_sum: null argument");
  Nccl *n;
  if (int s = nccl(&n)) return s;
  if (int s = use_device(device)) return s;
  BT_NCCL(n, n->AllReduce(as_ptr<void>(buf_f32), as_ptr<void>(buf_f32), count, ncclFloat32, ncclSum, reinterpret_cast<ncclComm_t>(comm), as_stream(stream)));
  return BT_OK;
}

int bt_argmax_combine(int device, uint64_t blocks, int world, int rows, uint64_t out_val, uint64_t out_idx, uint64_t stream) {
  BT_REQUIRE(blocks && out_val && out_idx && world >= 1 && rows >= 1 && rows <= 32, "bt_argmax_combine: %d ranks x %d rows", world, rows);
  if (int s = use_device(device)) return s;
  argmax_combine_kernel<<<1, 32, 0, as_stream(stream)>>>(as_ptr<float>(blocks), world, rows, as_ptr<float>(out_val), as_ptr<int>(out_idx));
  return launched("argmax_combine_kernel");
}

int bt_round_tilize(int device, uint64_t src_f32_rows, uint64_t dst_bf16_tiles, int rows, int cols, uint64_t stream) {
  BT_REQUIRE(src_f32_rows && dst_bf16_tiles && rows >= 1 && rows <= 32 && cols >= 1, "bt_round_tilize: %d x %d (one tile row)", rows, cols);
  if (int s = use_device(device)) return s;
  const size_t total = (size_t)((cols + 31) / 32) * 1024;
  round_tilize_kernel<<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>(as_ptr<float>(src_f32_rows), as_ptr<uint16_t>(dst_bf16_tiles), rows, cols);
  return launched("round_tilize_kernel");
}

int bt_peer_open(int device, uint64_t comm, int rank, int world, size_t bytes, uint64_t *peers, uint64_t stream) {
  BT_REQUIRE(comm && peers && world >= 1 && world <= kPeerMax && rank >= 0 && rank < world && bytes > 0, "bt_peer_open: rank %d of %d (up to %d ranks)", rank, world, kPeerMax);
  Nccl *n;
  if (int s = nccl(&n)) return s;
  if (int s = use_device(device)) return s;
  cudaStream_t st = as_stream(stream);
  uint8_t *mine = nullptr, *handles = nullptr;
  const size_t total = kPeerData + bytes;
  BT_CUDA(cudaMalloc(&mine, total));
  BT_CUDA(cudaMemsetAsync(mine, 0, kPeerData, st));
  cudaIpcMemHandle_t h, all[kPeerMax];
  BT_CUDA(cudaIpcGetMemHandle(&h, mine));
  BT_CUDA(cudaMalloc(&handles, sizeof h * world));
  BT_CUDA(cudaMemcpyAsync(handles + sizeof h * rank, &h, sizeof h, cudaMemcpyHostToDevice, st));
  BT_NCCL(n, n->AllGather(handles + sizeof h * rank, handles, sizeof h, ncclUint8, reinterpret_cast<ncclComm_t>(comm), st));
  BT_CUDA(cudaMemcpyAsync(all, handles, sizeof h * world, cudaMemcpyDeviceToHost, st));
  BT_CUDA(cudaStreamSynchronize(st));
  BT_CUDA(cudaFree(handles));
  for (int r = 0; r < world; r++) {
    void *p = mine;
    if (r != rank) BT_CUDA(cudaIpcOpenMemHandle(&p, all[r], cudaIpcMemLazyEnablePeerAccess));
    peers[r] = reinterpret_cast<uint64_t>(p);
  }
  // nobody signals before everybody has zeroed its flags and mapped the others: one more collective as the barrier
  int *token = reinterpret_cast<int *>(mine + kPeerError + 64);
  BT_NCCL(n, n->AllReduce(token, token, 1, ncclInt32, ncclSum, reinterpret_cast<ncclComm_t>(comm), st));
  BT_CUDA(cudaStreamSynchronize(st));
  return BT_OK;
}

int bt_peer_close(int device, uint64_t comm, int rank, int world, const uint64_t *peers, uint64_t stream) {
  BT_REQUIRE(comm && peers && world >= 1 && world <= kPeerMax && rank >= 0 && rank < world && peers[rank], "bt_peer_close: rank %d of %d", rank, world);
  Nccl *n;
  if (int s = nccl(&n)) return s;
  if (int s = use_device(device)) return s;
  // Collective: a rank must not free its rows while a slower peer's last kernel still reads them. The all-reduce is
  // queued behind this rank's kernels and completes only when every rank has queued, and so got past, its own.
  int *token = reinterpret_cast<int *>(as_ptr<uint8_t>(peers[rank]) + kPeerError + 64);
  BT_NCCL(n, n->AllReduce(token, token, 1, ncclInt32, ncclSum, reinterpret_cast<ncclComm_t>(comm), as_stream(stream)));
  BT_CUDA(cudaStreamSynchronize(as_stream(stream)));
  for (int r = 0; r < world; r++)
    if (r != rank && peers[r]) BT_CUDA(cudaIpcCloseMemHandle(as_ptr<void>(peers[r])));
  BT_CUDA(cudaFree(as_ptr<void>(peers[rank])));
  return BT_OK;
}

int bt_peer_allreduce_round(int device, int rank, int world, const uint64_t *peers, size_t offset, int step, int rows, int cols, uint64_t dst_bf16_tiles,
                            uint64_t stream) {
  BT_REQUIRE(peers && dst_bf16_tiles && world >= 1 && world <= kPeerMax && rank >= 0 && rank < world, "bt_peer_allreduce_round: rank %d of %d", rank, world);
  BT_REQUIRE(rows >= 1 && rows <= 32 && cols >= 32 && cols % 32 == 0 && offset % 16 == 0 && step > 0, "bt_peer_allreduce_round: %d x %d rows at offset %zu, step %d", rows, cols, offset, step);
  if (int s = use_device(device)) return s;
  PeerArgs a{};
  for (int r = 0; r < world; r++) {
    BT_REQUIRE(peers[r], "bt_peer_allreduce_round: rank %d's buffer is not mapped", r);
    a.peer[r] = as_ptr<uint8_t>(peers[r]);
  }
  a.data = kPeerData + offset, a.dst = as_ptr<uint16_t>(dst_bf16_tiles), a.rank = rank, a.world = world, a.step = step, a.rows = rows, a.cols = cols;
  const int quads = cols / 32 * 256, blocks = min(148, (quads + 255) / 256);
  peer_allreduce_round_kernel<<<blocks, 256, 0, as_stream(stream)>>>(a);
  return launched("peer_allreduce_round_kernel");
}

int bt_peer_argmax_combine(int device, int rank, int world, const uint64_t *peers, size_t offset, int step, int rows, uint64_t block, uint64_t out_val,
                           uint64_t out_idx, uint64_t stream) {
  BT_REQUIRE(peers && block && out_val && out_idx && world >= 1 && world <= kPeerMax && rank >= 0 && rank < world, "bt_peer_argmax_combine: rank %d of %d", rank, world);
  BT_REQUIRE(rows >= 1 && rows <= 32 && offset % 16 == 0 && step > 0 && block % 4 == 0, "bt_peer_argmax_combine: %d rows at offset %zu, step %d", rows, offset, step);
  if (int s = use_device(device)) return s;
  PeerPickArgs a{};
  for (int r = 0; r < world; r++) {
    BT_REQUIRE(peers[r], "bt_peer_argmax_combine: rank %d's buffer is not mapped", r);
    a.peer[r] = as_ptr<uint8_t>(peers[r]);
  }
  a.data = kPeerData + offset, a.mine = as_ptr<uint32_t>(block), a.out_val = as_ptr<float>(out_val), a.out_idx = as_ptr<int>(out_idx);
  a.rank = rank, a.world = world, a.step = step, a.rows = rows;
  peer_argmax_combine_kernel<<<1, kPeerMax * 64, 0, as_stream(stream)>>>(a);
  return launched("peer_argmax_combine_kernel");
}

int bt_peer_check(int device, int rank, const uint64_t *peers, uint64_t stream, int *error) {
  BT_REQUIRE(peers && error && rank >= 0 && rank < kPeerMax && peers[rank], "bt_peer_check: null argument");
  if (int s = use_device(device)) return s;
  uint8_t *mine = as_ptr<uint8_t>(peers[rank]);
  BT_CUDA(cudaMemcpyAsync(error, mine + kPeerError, 4, cudaMemcpyDeviceToHost, as_stream(stream)));
  BT_CUDA(cudaStreamSynchronize(as_stream(stream)));
  if (*error) BT_CUDA(cudaMemsetAsync(mine + kPeerError, 0, 4, as_stream(stream)));
  return BT_OK;
}

}  // extern "C"
