"""Layers too large for one GPU: the block-float matmul path sharded over the GPUs of one box.

One process per GPU (torchrun); `torch.distributed` carries the exchanges, NCCL over NVLink on GPUs and gloo in the
CPU tests. The reference has no collective backend -- its only inter-chip transport is a point-to-point tensor copy
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
the CUDA kernels through the Tensor API and share the runtime's stream with the collectives.
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

def _stream(rt):
  """The runtime's CUDA stream as a torch stream, so collectives queue in order with the kernels."""
  return torch.cuda.ExternalStream(rt.stream, device=torch.device("cuda", rt.device))


def _rows(rt, t, dtype):
  """A realized Tensor's values as a row-major torch tensor on the runtime's stream (fp32 or bf16)."""
  out = torch.empty((t.rows, t.cols), dtype=dtype, device=torch.device("cuda", rt.device))
  rt.launch("bt_untilize", (out.element_size(), t.addr, out.data_ptr(), 1, t.rows, t.cols), name="readback")
  return out


def _tensor(rt, rows, dtype="bf16"):
  """A row-major torch tensor (bf16, or fp32 to be rounded to bf16) as a bf16 Tensor in tile layout."""
  from baretile_b200.tensor import Tensor
  t = Tensor(rt, rows.shape[0], rows.shape[1], dtype=dtype)
  src = rows.contiguous()
  if src.dtype == torch.float32:
    half = torch.empty(src.shape, dtype=torch.bfloat16, device=src.device)
    rt.launch("bt_round_bf16", (src.data_ptr(), half.data_ptr(), src.numel()), name="round")
    src = half
  rt.launch("bt_tilize", (2, src.data_ptr(), t.addr, 1, t.rows, t.cols), name="upload")
  t._keep = (rows, src)    # the launches above read these buffers
  return t


class ShardedMLP:
  """SwiGLU MLP over the ranks of a process group: gate/up split over N, down split over K.

  `wg`, `wu` are this rank's [K, N/world] column slices and `wd` its [N/world, K_out] row slice, as block-float
  Tensors by columns. forward(x) takes the replicated bf16 activations [M, K] (M <= 32) and returns the [M, K_out]
  result as a bf16 Tensor on every rank. With gather=True the gate/up result is all-gathered to [M, N] first, as a
  stand-alone column-parallel layer would do, and the rank then multiplies its own slice of it; with gather=False
  the local slice feeds the down projection directly (column-parallel into row-parallel needs no exchange)."""
  def __init__(self, rt, wg, wu, wd, group=None):
    self.rt, self.wg, self.wu, self.wd, self.group = rt, wg, wu, wd, group
    self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)

  def forward(self, x, gather=True):
    rt = self.rt
    with torch.cuda.stream(_stream(rt)):
      h = ((x @ self.wg).silu() * (x @ self.wu)).realize()              # [M, N/world] bf16, one launch
      if gather:
        full = all_gather_columns(_rows(rt, h, torch.bfloat16), group=self.group)
        n = h.cols
        h = _tensor(rt, full[:, self.rank * n:(self.rank + 1) * n])
      partial = _rows(rt, h.matmul(self.wd, dtype="fp32").realize(), torch.float32)
      return _tensor(rt, all_reduce_sum(partial, self.group))


class ShardedHead:
  """Greedy pick over a vocabulary split across the ranks: `w` is this rank's [K, V/world] slice by columns and
  `base` the global index of its first column. pick(x) returns (values[M] fp32, indices[M] int32) torch tensors,
  identical on every rank."""
  def __init__(self, rt, w, base, group=None):
    self.rt, self.w, self.base, self.group = rt, w, base, group

  def pick(self, x):
    from baretile_b200.tensor import _launch_matmul, _linear
    rt, m = self.rt, x.rows
    dev = torch.device("cuda", rt.device)
    vals, ids = torch.empty(32, dtype=torch.float32, device=dev), torch.empty(32, dtype=torch.int32, device=dev)
    with torch.cuda.stream(_stream(rt)):
      _launch_matmul(rt, _linear(x @ self.w), "argmax", None, m, arg=(vals.data_ptr(), ids.data_ptr()), arg_base=self.base)
      return gather_argmax(vals[:m], ids[:m], self.group)
