/* C-ABI of libbaretile_b200.so: the B200 backend for baretile's block-float matmul path.
 *
 * The reference reaches its device through a ctypes-loaded C library with explicit argtypes
 * (baretile/pci.py:52-63: libttsim_init, libttsim_pci_mem_rd_bytes/wr_bytes, libttsim_clock). This
 * header is the matching boundary for a CUDA device: plain pointers and sizes, no C++ or torch types.
 * Each entry point names the reference interface it stands in for (paths inside the baretile project).
 *
 * Conventions
 *   - Every function returns a status: BT_OK, or an error whose text bt_last_error() gives.
 *     Host code maps BT_BAD_ARGUMENT -> ValueError, BT_DEVICE -> RuntimeError, BT_TIMEOUT -> TimeoutError,
 *     BT_NO_MEMORY -> MemoryError, as the reference raises them (docs/api.md:51-62).
 *   - Device addresses and stream/event handles travel as uint64_t.
 *   - Work is queued on the given stream and runs in order, asynchronously, like launches on the
 *     reference's command ring (baretile/runtime.py:680-771). bt_stream_sync waits.
 *   - The library never frees or allocates device memory behind the caller's back: only
 *     bt_malloc / bt_free do.
 *   - Tensors are in tile layout: 32x32 tiles in row order, each tile four row-major 16x16 faces
 *     (baretile/tensix.py:6-9). A bfp tile is 64 exponent bytes followed by its values
 *     (baretile/tensix.py:14-20): 1088 bytes for bfp8, 576 for bfp4.
 */
#ifndef BARETILE_B200_H
#define BARETILE_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { BT_OK = 0, BT_BAD_ARGUMENT = 1, BT_DEVICE = 2, BT_TIMEOUT = 3, BT_NO_MEMORY = 4 };
enum { BT_BF16 = 0, BT_FP32 = 1, BT_INT32 = 2, BT_BFP8 = 8, BT_BFP4 = 4 };            /* storage formats */
enum { BT_FP32_ROWS = 16 };   /* a matmul result as fp32 ROW-MAJOR [M, N] instead of tiles (only rows < M are written) */
enum { BT_EPI_NONE = 0, BT_EPI_RELU = 1, BT_EPI_SILU = 2, BT_EPI_GLU = 3, BT_EPI_ARGMAX = 4 };

typedef struct bt_device_info {
  char name[64];
  int sm_count, cc_major, cc_minor, l2_bytes;
  uint64_t memory_bytes;
  int max_shared_bytes, clock_khz;
} bt_device_info;

/* Text of the calling thread's last error. */
const char *bt_last_error(void);

/* ---- device, memory, streams, events: stand in for pci.open_device / Chip / Runtime
 *      (baretile/pci.py:453-463, baretile/chip.py:75-83, baretile/runtime.py:543-923) ---- */
int bt_device_count(int *count);                       /* pci.Sim.chips / find_cards */
int bt_device_info_get(int device, bt_device_info *out); /* Chip telemetry (chip.py:22-31) */
int bt_malloc(int device, size_t bytes, uint64_t *ptr);  /* the DRAM a Runtime carves (runtime.py:791-812) */
int bt_free(int device, uint64_t ptr);
int bt_host_alloc(size_t bytes, void **ptr);           /* the runtime's host DMA page (runtime.py:548-600) */
int bt_host_free(void *ptr);
int bt_stream_create(int device, uint64_t *stream);    /* the command ring */
int bt_stream_destroy(int device, uint64_t stream);
int bt_stream_sync(int device, uint64_t stream, int timeout_ms); /* Runtime.wait(timeout) (runtime.py:858-880) */
int bt_stream_query(int device, uint64_t stream, int *done);     /* Runtime.finished (runtime.py:837) */
int bt_h2d(int device, uint64_t dst, const void *src, size_t bytes, uint64_t stream); /* Chip.write / upload_kernel */
int bt_d2h(int device, void *dst, uint64_t src, size_t bytes, uint64_t stream);       /* Chip.read / readback_kernel */
int bt_d2d(int device, uint64_t dst, uint64_t src, size_t bytes, uint64_t stream);    /* copy_kernel (kernels.py:1051) */
int bt_memset(int device, uint64_t dst, int value, size_t bytes, uint64_t stream);    /* zeros_kernel (kernels.py:1439) */
int bt_event_create(int device, uint64_t *event);      /* dispatcher timestamps (runtime.py:773-786) */
int bt_event_destroy(int device, uint64_t event);
int bt_event_record(int device, uint64_t event, uint64_t stream);
int bt_event_elapsed_ms(int device, uint64_t start, uint64_t end, float *ms);
/* What is queued on `stream` after this call runs only once the work recorded by `event` is done; the host does not
 * wait. With bt_event_record it lets copies on a second stream run beside the kernels of the first (the reference
 * overlaps its host DMA with running kernels the same way: uploads go through the PCIe window while the dispatcher
 * drains the command ring, baretile/runtime.py:734-771). Inside bt_graph_begin / bt_graph_end it forks and joins
 * branches of the recorded graph. */
int bt_stream_wait_event(int device, uint64_t stream, uint64_t event);

/* ---- replay: tensor.jit / Recording (baretile/tensor.py:1171-1293, baretile/runtime.py:725-732) ----
 * Between bt_graph_begin and bt_graph_end the launches queued on the stream are recorded instead of run;
 * bt_graph_launch replays the recording with one call, as the reference replays a block of commands with one
 * doorbell write. Recorded launches keep the addresses they were queued with. */
int bt_graph_begin(int device, uint64_t stream);
int bt_graph_end(int device, uint64_t stream, uint64_t *graph);
int bt_graph_launch(int device, uint64_t graph, uint64_t stream);
int bt_graph_destroy(int device, uint64_t graph);

/* ---- layout: Tensor.frombytes / Tensor.tobytes (baretile/tensor.py:107-135, :159-193) ----
 * Row-major (batch, rows, cols) of itemsize-byte values <-> tiles. Padding is zero; a dimension of
 * size 1 repeats across its tile. itemsize is 2 or 4. */
int bt_tilize(int device, int itemsize, uint64_t src, uint64_t dst, int batch, int rows, int cols, uint64_t stream);
int bt_untilize(int device, int itemsize, uint64_t src, uint64_t dst, int batch, int rows, int cols, uint64_t stream);
/* The same for n small matrices (batch 1 each) in one launch: a decode step's inputs and results, where a launch
 * per matrix would cost more than the work. src, dst, rows, cols are host arrays of n entries. */
int bt_tilize_many(int device, int itemsize, int n, const uint64_t *src, const uint64_t *dst, const int *rows, const int *cols, uint64_t stream);
int bt_untilize_many(int device, int itemsize, int n, const uint64_t *src, const uint64_t *dst, const int *rows, const int *cols, uint64_t stream);
/* fp32 -> bf16, round to nearest even, NaN kept quiet: tensix.round_bf16 (baretile/tensix.py:240-242). */
int bt_round_bf16(int device, uint64_t src_f32, uint64_t dst_bf16, size_t count, uint64_t stream);

/* ---- block-float pack / unpack ----
 * bt_pack_bfp: Tensor.cast("bfp8" | "bfp4") (baretile/tensor.py:581-596): the packer's bfp8 rounding
 * (baretile/kernels.py:1108-1114, baretile/models/gpt2.py:19-30) and bfp4_kernel
 * (baretile/kernels.py:1074-1081, :1527-1567). src: ntiles bf16 tiles; dst: ntiles bfp tiles.
 * bt_unpack_bfp: the unpacker's conversion, storage_kernel (baretile/kernels.py:1483-1525) and
 * tensor._bf16s (baretile/tensor.py:1095-1104). */
int bt_pack_bfp(int device, int fmt, uint64_t src, uint64_t dst, size_t ntiles, uint64_t stream);
int bt_unpack_bfp(int device, int fmt, uint64_t src, uint64_t dst, size_t ntiles, uint64_t stream);

/* Tensor.put / put_kernel (baretile/tensor.py:224-241, baretile/kernels.py:1083-1168): rows of x written in place into
 * the rows of dst that ids names, e.g. new keys and values into a KV cache. dst: batch matrices of dst_rows x cols in
 * tile layout, format fmt. x: batch matrices of n x cols, bf16 when dst is a block float (each run of 16 is then
 * rounded exactly as bt_pack_bfp rounds it), else dst's format. ids: an int32 row of n places in tile layout. A
 * place past dst's last tile row is skipped (one in the padding of the last tile row is written there); of several
 * rows to one place the last wins. A dst of one row keeps it in all 32 rows of its tile, as every one-row tensor
 * does. x and ids must not overlap dst: the caller copies an aliased one first (Tensor.put does).
 * scratch: 0, or room for one int per row of dst's tile rows (32 * ceil(dst_rows / 32) ints), used to find the last
 * row for each place in one pass; without it every row searches all later places, which is fine for a few hundred
 * rows and quadratic beyond. */
int bt_put(int device, int fmt, uint64_t dst, uint64_t x, uint64_t ids, int batch, int n, int dst_rows, int cols, uint64_t scratch,
           uint64_t stream);

/* Tensor.columns() / columns_kernel (baretile/tensor.py:598-611, baretile/kernels.py:1455-1481): a pure
 * byte permutation of a (tile_rows x tile_cols) block-float matrix into the layout the matmul streams.
 * Runs of 4 tile columns; inside a run, tile row by tile row; inside a tile, exponents then values,
 * both ordered for one 128-bit load per lane, value bytes recoded one to one from sign and magnitude to offset
 * binary. to_stream = 0 undoes it, byte for byte. One launch takes up to 262140 tile columns. */
int bt_relayout(int device, int fmt, int to_stream, int tile_rows, int tile_cols, uint64_t src, uint64_t dst,
                uint64_t stream);

/* ---- the matmul: fused_kernel's decode paths (baretile/kernels.py:216-253, :543-584) ----
 * out[M, N] = epilogue(alpha * (x[M, K] @ W[K, N]) + add), M <= 32.
 *   x      bf16 tiles, one tile row (K/32 tiles).  K and N are multiples of 32.
 *   w, w2  block-float weights in streaming layout (bt_relayout). w2 only for BT_EPI_GLU:
 *          out = silu(x @ w) * (x @ w2) (baretile/models/llama.py:179-183).
 *   add    0, or bf16 tiles of an (M or 1) x N addend, added before the activation
 *          (baretile/kernels.py:593-599).
 *   out    bf16 or fp32 tiles (out_dtype), rows past M zero (or, with BT_FP32_ROWS, fp32 row-major [M, N]: the form
 *          an all-reduce of partial sums wants); or with BT_EPI_ARGMAX nothing, and
 *          arg_val[M] (fp32) / arg_idx[M] (int32) receive each row's largest value and its first
 *          column (topk_kernel's tie rule, baretile/kernels.py:1173-1231), index + arg_base.
 *   work   scratch of at least bt_gemv_workspace_bytes() bytes, zeroed once before first use;
 *          launches that share it go on one stream (where they may overlap at their edges: a launch
 *          fetches weights while the one before it finishes, and touches the scratch only after it).
 *          That overlap happens only behind another matmul launch of this library: after any other call of
 *          this library (a cast, a relayout, a copy) the launch starts once everything before it is complete.
 *          Work queued on the stream by other means and writing the weights needs a synchronisation of the
 *          caller's before the matmul.
 * Products are exact, sums are fp32, outputs round half up to bf16 like the packer
 * (docs/compiler.md, "Matmul precision"). */
int bt_gemv_workspace_bytes(int device, size_t *bytes);
int bt_gemv_bfp(int device, int fmt, int epilogue, int M, int K, int N, uint64_t x, uint64_t w, uint64_t w2,
                uint64_t add, float alpha, uint64_t out, int out_dtype, uint64_t arg_val, uint64_t arg_idx,
                int arg_base, uint64_t work, size_t work_bytes, uint64_t stream);
/* ---- a queue of matmuls in one launch: the command ring the dispatcher drains (baretile/runtime.py:734-771,
 * the resident dispatcher :369-446) ----
 * Runs ops[0..n), each exactly as bt_gemv_bfp would, as one kernel (one per 32 matmuls), with the results a
 * one-after-the-other run gives: a matmul may read what any earlier one wrote (its x, its addend), as in a decode
 * step where each result feeds the next, and the library works out from the addresses which earlier matmuls each
 * one has to wait for (bt_gemv_queue_plan shows the answer). Between two matmuls the GPU keeps streaming: the
 * weights of the next ones are fetched while the previous one finishes, only x waits, and matmuls that do not
 * depend on one another overlap (two in flight at most). The weights (w, w2) must not be written by an earlier
 * matmul of the same call or by the launch right before it in the stream. The fields of bt_gemv_op are
 * bt_gemv_bfp's arguments of the same names. */
typedef struct bt_gemv_op {
  int fmt, epilogue, M, K, N, out_dtype, arg_base;
  float alpha;
  uint64_t x, w, w2, add, out, arg_val, arg_idx;
} bt_gemv_op;
int bt_gemv_queue(int device, int n, const bt_gemv_op *ops, uint64_t work, size_t work_bytes, uint64_t stream);
/* What bt_gemv_queue would make each matmul wait for, without touching a device: waits[i] receives the index of the
 * last earlier matmul that ops[i] must see finished before it starts, or -1 when it only waits for the launch
 * before it. A matmul waits for the latest earlier one whose result it reads (x, add) or whose result buffers it
 * writes or that reads what it writes, and never runs more than two places ahead of a matmul still in flight; a
 * list longer than 32 is cut into launches of 32, and the first matmul of a launch waits for the whole launch
 * before it (-1). */
int bt_gemv_queue_plan(int n, const bt_gemv_op *ops, int *waits);
/* ---- the matmul: fused_kernel's prefill grid (baretile/kernels.py:205-215, :470-506, grid_parts :18-39) ----
 * out[M, N] = epilogue(alpha * (a[M, K] @ W[K, N]) + add) for many rows, on the tcgen05 tensor cores with fp32
 * accumulators in tensor memory, two CTAs to an MMA. The weights are expanded from block float to exact bf16
 * inside the kernel.
 *   a      bf16, ROW-MAJOR [M, K] (bt_untilize of the tile-layout tensor, over whole tiles: K a multiple of 32,
 *          columns past the tensor's own holding zeros).
 *   w, w2  block-float weights in streaming layout; w2 only for BT_EPI_GLU (out = silu(a @ w + add) * (a @ w2)).
 *          N is the tensor's own column count, any positive number.
 *   add    0, or bf16 tiles of an addend of add_rows (M or 1) x N, added before the activation.
 *   out    bf16 or fp32 tiles, rows past M zero.
 *   work   the matmul scratch (bt_gemv_workspace_bytes): only its error word is used. */
int bt_gemm_bfp(int device, int fmt, int epilogue, int M, int K, int N, uint64_t a, uint64_t w, uint64_t w2, uint64_t add,
                int add_rows, float alpha, uint64_t out, int out_dtype, uint64_t work, uint64_t stream);

/* The same matmul for callers that cannot allocate device memory: it has no counterpart in the reference.
 * Some embedders of this library run where cudaMalloc is off limits -- inside another framework's capture or
 * allocator-owned region, in a process whose memory budget was handed out in full at start-up, or in a plug-in
 * that is only ever given its input and output buffers. For them the scratch that bt_gemv_bfp takes from the
 * caller sits in a fixed array inside the library's device image (about 2.6 MB on every GPU that loads the
 * library, held until the process exits). The call allocates and frees nothing, on the host side either.
 * Limits, rejected with BT_BAD_ARGUMENT: M <= 8 rows of x, N <= 524288 columns. Inputs and outputs are the
 * caller's, exactly as for bt_gemv_bfp. The first call on a device looks the array's address up (one runtime
 * query); make that first call outside any stream capture. All calls on a device share the one array and each
 * call first clears the counters it keeps there, so two calls whose kernels overlap on the GPU (different
 * streams) race: keep them on one stream or serialise them. The word that records a wait that gave up is not cleared
 * by a call: it stays until bt_gemv_check(device, 0, stream, &error) reads it. */
int bt_gemv_bfp_static(int device, int fmt, int epilogue, int M, int K, int N, uint64_t x, uint64_t w, uint64_t w2,
                       uint64_t add, float alpha, uint64_t out, int out_dtype, uint64_t arg_val, uint64_t arg_idx,
                       int arg_base, uint64_t stream);
/* Nonzero in *error once a bounded wait inside a launch that used this scratch gave up (its results are then
 * unreliable): the counterpart of Runtime.wait's timeout report (baretile/runtime.py:866-876). Synchronises the
 * stream; if the flag was set, clears it and the counters that launch may have left half-counted. work = 0 asks
 * about the built-in scratch of bt_gemv_bfp_static on that device. */
int bt_gemv_check(int device, uint64_t work, uint64_t stream, int *error);
/* ---- exchanges between the GPUs of one box, for layers split over them ----
 * The reference has no collectives; its transport between chips is the point-to-point copy of Tensor.to
 * (baretile/tensor.py:708-726) over link_kernel (baretile/kernels.py:1316-1372). These entry points carry what the
 * split layers of this path need instead, as NCCL collectives queued on the caller's stream (NCCL is loaded on first
 * use; a process that never calls them needs none).
 *   bt_comm_unique_id   128 bytes that one rank makes and hands to the others by any means.
 *   bt_comm_init        every rank, with its device current: joins the communicator of `world` ranks.
 *   bt_allgather        `bytes` from every rank into dst, ranks one after another. On bf16 tile buffers of [M, N/world]
 *                       column slices this yields the [M, N] tensor in tile layout as it is (gate/up split over N).
 *   bt_allreduce_sum    in-place sum of `count` fp32 over the ranks (down projection split over K: BT_FP32_ROWS partial
 *                       sums), then bt_round_tilize rounds [rows, cols] fp32 row-major to bf16 tiles of one tile row,
 *                       half up like every matmul result.
 *   bt_argmax_combine   the greedy pick over a vocabulary split across ranks: `blocks` holds, per rank, 32 fp32
 *                       values then 32 int32 global indices (a matmul's pick with arg_idx = arg_val + 128 bytes,
 *                       gathered by bt_allgather of 256 bytes); per row the larger value wins, of equal values the
 *                       lower index (topk_kernel's tie rule, baretile/kernels.py:1228-1231). */
int bt_comm_unique_id(void *id, size_t bytes);
int bt_comm_init(int device, int rank, int world, const void *id, uint64_t *comm);
int bt_comm_destroy(uint64_t comm);
int bt_allgather(int device, uint64_t comm, uint64_t src, uint64_t dst, size_t bytes, uint64_t stream);
int bt_allreduce_sum(int device, uint64_t comm, uint64_t buf_f32, size_t count, uint64_t stream);
int bt_round_tilize(int device, uint64_t src_f32_rows, uint64_t dst_bf16_tiles, int rows, int cols, uint64_t stream);

/* ---- the down projection's exchange as one kernel over peer memory (no counterpart in the reference, like the
 * collectives above) ----
 * bt_peer_open gives every rank a buffer of BT_PEER_DATA + bytes that the other ranks of the box map through CUDA IPC
 * (the handles go round the communicator); peers[r] receives rank r's buffer as an address on this device,
 * peers[rank] the rank's own. Collective: every rank calls it, with the same bytes. The first BT_PEER_DATA bytes
 * are the library's (flags, an error word); the caller's rows live behind them.
 * bt_peer_allreduce_round(step): every rank has written rows x cols fp32, row-major, at BT_PEER_DATA + offset of its
 * own buffer (a matmul with out_dtype BT_FP32_ROWS does); the kernel announces them to the peers, waits (about a
 * second at most) for theirs, adds all ranks' rows in rank order straight from their memories, rounds half up and
 * writes bf16 tiles of one tile row to dst. step grows by one per call, on every rank alike, starting at 1; the
 * caller alternates offset between two halves of the buffer from step to step (a rank is never more than one
 * step ahead of a peer, so the half it overwrites has been read by all). bt_peer_check reads (and clears) the word a
 * wait that gave up sets. bt_peer_close is collective too: it waits until every rank has got past its kernels that read
 * the others' rows, then unmaps and frees. */
#define BT_PEER_DATA 4096
int bt_peer_open(int device, uint64_t comm, int rank, int world, size_t bytes, uint64_t *peers, uint64_t stream);
int bt_peer_close(int device, uint64_t comm, int rank, int world, const uint64_t *peers, uint64_t stream);
int bt_peer_allreduce_round(int device, int rank, int world, const uint64_t *peers, size_t offset, int step, int rows, int cols,
                            uint64_t dst_bf16_tiles, uint64_t stream);
/* The vocabulary-split pick over peer memory: `block` is this rank's 256 bytes as the matmul's fused pick leaves
 * them (32 fp32 values, then 32 int32 indices); they go into slot `rank` (256 bytes each, from BT_PEER_DATA + offset)
 * of every rank's buffer, and when every rank's block of this step is here they are combined as bt_argmax_combine
 * combines them. The buffer holds 2 x world x 256 bytes: offset alternates between its halves from step to step. */
int bt_peer_argmax_combine(int device, int rank, int world, const uint64_t *peers, size_t offset, int step, int rows, uint64_t block,
                           uint64_t out_val, uint64_t out_idx, uint64_t stream);
int bt_peer_check(int device, int rank, const uint64_t *peers, uint64_t stream, int *error);
int bt_argmax_combine(int device, uint64_t blocks, int world, int rows, uint64_t out_val, uint64_t out_idx, uint64_t stream);
/* Number of GPU kernels this library has launched on behalf of the calling process. */
int bt_launch_count(uint64_t *count);

#ifdef __cplusplus
}
#endif
#endif
