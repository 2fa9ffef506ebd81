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

}  // extern "C"
