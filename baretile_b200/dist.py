"""Layers too large for one GPU: the block-float matmul path sharded over the GPUs of one box.

One process per GPU (torchrun). On GPUs the exchanges are NCCL collectives behind the library's C-ABI (bt_allgather,
bt_allreduce_sum, bt_argmax_combine), queued on the runtime's stream between the matmul launches; the same rules as
plain host functions over `torch.distributed` (gloo) are what the CPU tests run. The reference has no collective backend -- its only inter-chip transport is a point-to-point tensor copy
over Ethernet (`Tensor.to`, baretile/tensor.py:708-726) -- so the partitioning here follows the shapes of the path:

  gate/up   W[K, N] split over N in whole tile columns; x is replicated; SiLU(x Wg) * (x Wu) is local to a rank;
            an all-gather rebuilds the [M, N] activations (or none, when the down projection that follows is split
            over the same range of its K).
  down      W[K, N] split over K; each rank multiplies its slice of the activations and the fp32 partial sums are
            all-reduced, then rounded to bf16 once.
  LM head   W[K, V] split over the vocabulary; each rank's kernel reduces its logits to (max, first index) per row,
            with the index already global; the ranks all-gather those pairs and apply the reference's tie rule
            (larger value wins, of equal values the lower index; topk_kernel, baretile/kernels.py:1173-1231).

The functions in the first half are pure host logic and work on any backend; the classes in the second half drive
the CUDA kernels and the collectives through the C-ABI on the runtime's stream.
"""
import torch
import torch.distributed as dist


def split_tiles(extent, world, rank):
  """[start, end) of rank's share when `extent` (a multiple of 32) is cut into `world` contiguous ranges of whole
  32-wide tiles, as evenly as the tile count allows."""
  if extent % 32: raise ValueError(f"sharded extents are multiples of 32, not {extent}")
  if not 0 <= rank < world: raise ValueError(f"rank {rank} of {world}")
  tiles = extent // 32
  if tiles < world: raise ValueError(f"{tiles} tiles cannot be split {world} ways")
  return 32 * (tiles * rank // world), 32 * (tiles * (rank + 1) // world)


def combine_argmax(values, indices):
  """Per row, the best of each rank's candidate: values and indices are [world, M]. The larger value wins; of equal
  values the lower index; -0 equals 0; a NaN never wins. A handful of whole-array operations whatever the world size."""
  values, indices = torch.as_tensor(values), torch.as_tensor(indices)
  values = torch.nan_to_num(values, nan=float("-inf"), posinf=float("inf"), neginf=float("-inf"))
  best_v = values.max(dim=0).values
  far = torch.iinfo(indices.dtype).max
  best_i = torch.where(values == best_v, indices, torch.full_like(indices, far)).min(dim=0).values
  return best_v, best_i


def all_gather_columns(local, sizes=None, group=None):
  """[M, n_local] on each rank -> [M, sum n] on every rank, ranks' columns in rank order. `sizes` lists every rank's
  column count when they differ."""
  world = dist.get_world_size(group)
  if sizes is None: sizes = [local.shape[1]] * world
  if len(set(sizes)) == 1:
    out = torch.empty((world * local.shape[0], local.shape[1]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, local.contiguous(), group=group)     # ranks' blocks one after another
    return out.view(world, *local.shape).permute(1, 0, 2).reshape(local.shape[0], -1)
  widest = max(sizes)                                # unequal shares: pad to the widest, gather, trim
  padded = torch.zeros((local.shape[0], widest), dtype=local.dtype, device=local.device)
  padded[:, :local.shape[1]] = local
  out = torch.empty((world * local.shape[0], widest), dtype=local.dtype, device=local.device)
  dist.all_gather_into_tensor(out, padded, group=group)
  out = out.view(world, local.shape[0], widest)
  return torch.cat([out[r, :, :n] for r, n in enumerate(sizes)], dim=1)


def all_reduce_sum(partial, group=None):
  """Sum fp32 partial results over the ranks, in place."""
  dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
  return partial


def gather_argmax(values, indices, group=None):
  """Each rank's per-row (max, global index) -> the global pick on every rank. The payload is 8 bytes per row."""
  world = dist.get_world_size(group)
  pair = torch.stack([values.to(torch.float32), indices.to(torch.int32).view(torch.float32)], dim=-1).contiguous()
  out = torch.empty((world * pair.shape[0], 2), dtype=pair.dtype, device=pair.device)
  dist.all_gather_into_tensor(out, pair, group=group)
  out = out.view(world, pair.shape[0], 2)
  return combine_argmax(out[..., 0], out[..., 1].contiguous().view(torch.int32))


# ---- the sharded layers on GPUs -----------------------------------------------------------------------------------
# Everything below goes through the C-ABI on the runtime's stream: matmul launches, NCCL collectives (bt_allgather,
# bt_allreduce_sum) and the small kernels either side of them, with no torch operation on the data path.

BT_PEER_DATA = 4096   # bytes the library keeps at the start of a peer buffer (include/baretile_b200.h)


class Comm:
  """The ranks' NCCL communicator behind the C-ABI (bt_comm_init). `exchange(bytes)` hands rank 0's bytes to every
  rank: by default over torch.distributed (any backend), which is only used for this one hand-shake."""
  def __init__(self, rt, rank, world, exchange=None):
    import ctypes
    from baretile_b200 import _lib
    self.rt, self.rank, self.world = rt, rank, world
    uid = ctypes.create_string_buffer(128)
    if rank == 0: _lib.call("bt_comm_unique_id", uid, 128)
    if exchange is None:
      def exchange(data):
        box = [data]
        dist.broadcast_object_list(box, src=0)
        return box[0]
    uid = ctypes.create_string_buffer(exchange(uid.raw), 128)
    handle = ctypes.c_uint64()
    _lib.call("bt_comm_init", rt.device, rank, world, uid, ctypes.byref(handle))
    self.handle = handle.value
    self.opened = []

  def open_peers(self, size):
    """A buffer of BT_PEER_DATA + size bytes on every rank, mapped on all of them (bt_peer_open): the ranks' addresses
    as a ctypes array for the peer entry points. Collective: every rank calls it with the same size."""
    import ctypes
    from baretile_b200 import _lib
    peers = (ctypes.c_uint64 * self.world)()
    _lib.call("bt_peer_open", self.rt.device, self.handle, self.rank, self.world, size, peers, self.rt.stream)
    self.opened.append(peers)
    return peers

  def close(self):
    from baretile_b200 import _lib
    for peers in self.opened: _lib.call("bt_peer_close", self.rt.device, self.handle, self.rank, self.world, peers, self.rt.stream)
    self.opened = []
    if self.handle: _lib.lib().bt_comm_destroy(self.handle)
    self.handle = 0


class ShardedMLP:
  """SwiGLU MLP over the ranks: gate/up split over N, down split over K.

  `wg`, `wu` are this rank's [K, N/world] column slices and `wd` its [N/world, K_out] row slice, as block-float
  Tensors by columns. forward(x) takes the replicated bf16 activations [M, K] (M <= 32) and returns the [M, K_out]
  result as a bf16 Tensor on every rank: the gate/up pair and the down projection leave as one queue launch, the down
  projection writes fp32 partial sums row-major, one all-reduce adds them over the ranks and one small kernel rounds
  them to bf16 tiles. With gather=True the gate/up result is also all-gathered to [M, N], as a stand-alone
  column-parallel layer would do (the tile buffers of the ranks, one after another, are the full tensor's tile row);
  the down projection needs only the rank's own slice either way.
  With peer=True the all-reduce and the rounding are one kernel over peer memory instead (bt_peer_allreduce_round): the
  partial sums go into a buffer the other ranks map, alternating between its two halves from step to step."""
  def __init__(self, rt, wg, wu, wd, comm, peer=False):
    self.rt, self.wg, self.wu, self.wd, self.comm = rt, wg, wu, wd, comm
    self.half = 4 * 32 * wd.cols
    self.peers, self.step = (comm.open_peers(2 * self.half) if peer else None), 0
    self.partial = None if peer else rt.dram_alloc(self.half)
    self.gathered = None

  def forward(self, x, gather=False):
    import ctypes
    from baretile_b200.tensor import Tensor, FMT_CODE
    rt, m = self.rt, x.rows
    out = Tensor(rt, m, self.wd.cols)
    self.step += 1
    offset = (self.step & 1) * self.half
    partial = self.partial if self.peers is None else self.peers[self.comm.rank] + BT_PEER_DATA + offset
    with rt.queue():
      h = ((x @ self.wg).silu() * (x @ self.wu)).realize()              # [M, N/world] bf16 tiles
      rt.launch("bt_gemv_bfp", (FMT_CODE[self.wd.dtype], 0, m, h.cols, self.wd.cols, h.addr, self.wd.addr, 0, 0, ctypes.c_float(1.0),
                                partial, 16, 0, 0, 0, rt.work, rt.work_bytes), name="matmul down partial")
    if gather:
      if self.gathered is None or self.gathered.cols != h.cols * self.comm.world: self.gathered = Tensor(rt, 32, h.cols * self.comm.world)
      rt.launch("bt_allgather", (self.comm.handle, h.addr, self.gathered.addr, h.tiles * 2048), name="all-gather")
    if self.peers is not None:
      rt.launch("bt_peer_allreduce_round", (self.comm.rank, self.comm.world, self.peers, offset, self.step, m, self.wd.cols, out.addr), name="peer all-reduce")
    else:
      rt.launch("bt_allreduce_sum", (self.comm.handle, self.partial, m * self.wd.cols), name="all-reduce")
      rt.launch("bt_round_tilize", (self.partial, out.addr, m, self.wd.cols), name="round")
    self.h = h                                                         # its memory is read by the launches above
    return out


class ShardedHead:
  """Greedy pick over a vocabulary split across the ranks: `w` is this rank's [K, V/world] slice by columns and
  `base` the global index of its first column. pick(x) queues the matmul with its fused pick, the all-gather of the
  ranks' 256-byte candidate blocks and the combining kernel, and returns the device address of the result: M fp32
  values followed, 128 bytes in, by M int32 indices, identical on every rank. read() brings them to the host."""
  def __init__(self, rt, w, base, comm, peer=False):
    self.rt, self.w, self.base, self.comm = rt, w, base, comm
    self.mine, self.all, self.out = rt.dram_alloc(256), rt.dram_alloc(256 * comm.world), rt.dram_alloc(256)
    self.half = 256 * comm.world
    self.peers, self.step = (comm.open_peers(2 * self.half) if peer else None), 0     # peer=True: the exchange over peer memory

  def pick(self, x):
    import ctypes
    from baretile_b200.tensor import FMT_CODE
    rt, m = self.rt, x.rows
    rt.launch("bt_gemv_bfp", (FMT_CODE[self.w.dtype], 4, m, x.cols, self.w.cols, x.addr, self.w.addr, 0, 0, ctypes.c_float(1.0), 0, 0,
                              self.mine, self.mine + 128, self.base, rt.work, rt.work_bytes), name="matmul pick")
    if self.peers is not None:
      self.step += 1
      rt.launch("bt_peer_argmax_combine", (self.comm.rank, self.comm.world, self.peers, (self.step & 1) * self.half, self.step, m, self.mine,
                                           self.out, self.out + 128), name="peer combine")
      return self.out
    rt.launch("bt_allgather", (self.comm.handle, self.mine, self.all, 256), name="all-gather")
    rt.launch("bt_argmax_combine", (self.all, self.comm.world, m, self.out, self.out + 128), name="combine")
    return self.out

  def read(self, m):
    import numpy as np
    raw = self.rt.download(self.out, 256)
    return np.frombuffer(raw[:4 * m], np.float32).copy(), np.frombuffer(raw[128:128 + 4 * m], np.int32).copy()
