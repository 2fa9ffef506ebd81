"""The block-float matmul with its fused epilogues on the GPU against the oracle's fp32 NumPy matmul over the same
dequantised weights. Tolerance (stated by the task): max relative error 1e-2 for bf16 results, where relative error
is max |got - ref| / max |ref| (docs/workload.md:141). fp32 results are held to 1e-4. Argmax indices are exact."""
import ctypes
import numpy as np
import pytest
from oracle import bfp_oracle as o
from helpers import acts, bf16, check_matmul, upload, weights

pytestmark = pytest.mark.gpu
TOL_BF16, TOL_FP32 = 1e-2, 1e-4


def run(rt, x, w, fmt, epilogue="none", w2=None, dtype=None, columns=True, add=None, alpha=None):
  """Build the Tensor expression the way a model would, realize it, and return (result, oracle reference)."""
  tx, tw = upload(rt, x), upload(rt, w).cast(fmt)
  if columns: tw = tw.columns()
  wd = o.dequant(w, fmt)
  y = tx.matmul(tw, dtype=dtype)
  ref = x.astype(np.float32) @ wd
  if alpha is not None: y, ref = y * alpha, ref * np.float32(alpha)
  if add is not None: y, ref = y + upload(rt, add), ref + add
  if epilogue == "relu": y, ref = y.relu(), np.maximum(ref, 0)
  elif epilogue == "silu": y, ref = y.silu(), o.silu(ref)
  elif epilogue == "glu":
    tw2 = upload(rt, w2).cast(fmt)
    if columns: tw2 = tw2.columns()
    y, ref = y.silu() * tx.matmul(tw2, dtype=dtype), o.silu(ref) * (x.astype(np.float32) @ o.dequant(w2, fmt))
  rt.log = []
  got = y.realize()
  rt.wait()
  names, rt.log = [name for *_, name in rt.log], None
  # one matmul launch with the epilogue fused (up to 32 rows: the decode kernel; more: the tensor-core kernel after
  # x is laid out by rows); a B not yet by columns is first laid out, once
  many = x.shape[0] > 32
  assert sum(n.startswith("prefill" if many else "matmul") for n in names) == 1 and len(names) <= 1 + many + (0 if columns else 2), names
  out = got.numpy()
  if epilogue in ("none", "relu"):   # every element within 2^-8 of sum |x||w| (+ |addend|): the reference's per-element bound
    check_matmul(out, x, wd, ref, TOL_BF16 if dtype != "fp32" else TOL_FP32, addend=add, alpha=alpha if alpha is not None else 1.0)
  return out, ref


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_exact_small_integers(rt, fmt):
  # weights and activations that both formats hold exactly: the result equals integer arithmetic (test/test_kernels.py:637-651)
  k, n = 64, 64
  x = np.array([[float((r * 7 + c * 3) % 3 - 1) for c in range(k)] for r in range(32)], np.float32)
  w = np.array([[float((r * 5 + c) % 3 - 1) for c in range(n)] for r in range(k)], np.float32)
  got, ref = run(rt, x, w, fmt, dtype="fp32")
  assert np.array_equal(got, x @ w) and np.array_equal(ref, x @ w)
  eye = np.eye(64, dtype=np.float32)
  xr = bf16(np.random.default_rng(1).uniform(-8, 8, (32, 64)))
  got, _ = run(rt, xr, eye, fmt)
  assert np.array_equal(got, xr)                                   # A @ I == A pins the tile and fragment layout
  ones = np.full((1, 1024), 1 / 32, np.float32)
  got, _ = run(rt, ones, np.full((1024, 64), 1 / 32, np.float32), fmt)
  assert np.array_equal(got, np.ones((1, 64), np.float32))          # test/test_kernels.py:783-800


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 17, 32])
def test_rows(rt, fmt, m):
  rng = np.random.default_rng(m)
  x, w = acts(rng, m, 1024), weights(rng, 1024, 736)               # 23 tile columns: ragged sub-panels and runs
  got, ref = run(rt, x, w, fmt)
  check_matmul(got, x, None, ref, TOL_BF16)
  got, ref = run(rt, x, w, fmt, dtype="fp32")
  check_matmul(got, x, None, ref, TOL_FP32)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("epilogue", ["relu", "silu", "glu"])
@pytest.mark.parametrize("m", [1, 8, 32])
def test_epilogues(rt, fmt, epilogue, m):
  rng = np.random.default_rng(3)
  x, w, w2 = acts(rng, m, 512), weights(rng, 512, 1536), weights(rng, 512, 1536)
  got, ref = run(rt, x, w, fmt, epilogue, w2)
  check_matmul(got, x, None, ref, TOL_BF16)
  if epilogue == "relu": assert (got >= 0).all() and (got == 0).any()


def test_config0_smollm_mlp(rt):
  # the reference's CPU-runnable case: relu(x[32,576] @ W[576,1536]) with W bfp8, seed 0
  rng = np.random.default_rng(0)
  x, w = bf16(rng.normal(0, 1, (32, 576))), bf16(rng.normal(0, 0.02, (576, 1536)))
  for columns in (True, False):
    got, ref = run(rt, x, w, "bfp8", "relu", columns=columns)
    check_matmul(got, x, None, ref, TOL_BF16)
    packed = o.bf16_floats(o.bf16_half_up(ref))                    # the packer's rounding of the fp32 reference
    assert np.abs(got - packed).max() <= 2.0 ** -7 * np.abs(ref).max()


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_addend_and_scale(rt, fmt):
  rng = np.random.default_rng(5)
  x, w = acts(rng, 8, 256), weights(rng, 256, 416)
  bias, resid = bf16(rng.normal(0, 1, (1, 416))), bf16(rng.normal(0, 1, (8, 416)))
  for add in (bias, resid):
    got, ref = run(rt, x, w, fmt, "relu", add=add)
    check_matmul(got, x, None, ref, TOL_BF16)
  got, ref = run(rt, x, w, fmt, alpha=0.5, add=bias, dtype="fp32")
  check_matmul(got, x, None, ref, TOL_FP32)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_more_than_one_tile_row(rt, fmt):
  rng = np.random.default_rng(9)
  x, w = acts(rng, 70, 256), weights(rng, 256, 160)
  got, ref = run(rt, x, w, fmt, "relu")
  check_matmul(got, x, None, ref, TOL_BF16)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("k,n", [(4096, 4096), (4096, 14336), (14336, 4096)])
def test_llama_shapes(rt, fmt, k, n):
  # the benchmark's decode shapes at full size, with the x20 channels; M = 8 and the fused gate/up pair at M = 1
  rng = np.random.default_rng(k + n)
  x, w = acts(rng, 8, k), weights(rng, k, n)
  got, ref = run(rt, x, w, fmt)
  check_matmul(got, x, None, ref, TOL_BF16)
  again, _ = run(rt, x, w, fmt)
  assert np.array_equal(got, again)                                 # partial sums combine in a fixed order
  if n == 14336:
    x1, w2 = acts(rng, 1, k), weights(rng, k, n)
    got, ref = run(rt, x1, w, fmt, "glu", w2)
    check_matmul(got, x1, None, ref, TOL_BF16)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_every_configuration(rt, fmt):
  # each group of row counts, one matrix and the gate/up pair, on shapes with ragged sub-panels and short ranges
  rng = np.random.default_rng(13)
  w, w2 = weights(rng, 2048, 1184), weights(rng, 2048, 1184)
  for m in (2, 16, 32):
    x = acts(rng, m, 2048)
    got, ref = run(rt, x, w, fmt, "glu", w2)
    check_matmul(got, x, None, ref, TOL_BF16)
    got, ref = run(rt, x, w, fmt, dtype="fp32")
    check_matmul(got, x, None, ref, TOL_FP32)


def _layer_chain(rt, x, layers):
  """x through a chain of dependent matmuls: each layer is (gate, up, down) Tensors; returns every layer's output."""
  outs, h = [], x
  for wg, wu, wd in layers:
    a = ((h @ wg).silu() * (h @ wu)).realize()
    h = (a @ wd).relu().realize()
    outs += [a, h]
  return outs


@pytest.mark.parametrize("m", [1, 8, 20])
def test_queue_equals_separate_launches(rt, m):
  # a chain where every matmul reads the one before it, mixed formats: one queue launch gives the same bits as one
  # launch per matmul, and matches the oracle
  rng = np.random.default_rng(31 + m)
  shapes = [(512, 1536, "bfp8"), (512, 736, "bfp4"), (512, 1536, "bfp4"), (512, 2048, "bfp8")]
  host = [(weights(rng, k, n) * 2, weights(rng, k, n) * 2, weights(rng, n, 512) * 2, fmt) for k, n, fmt in shapes]
  layers = [tuple(upload(rt, w).cast(fmt).columns() for w in (wg, wu, wd)) for wg, wu, wd, fmt in host]
  x = acts(rng, m, 512)
  tx = upload(rt, x)
  separate = [t.numpy() for t in _layer_chain(rt, tx, layers)]
  rt.log = []
  with rt.queue(): queued = _layer_chain(rt, tx, layers)
  rt.wait()
  log, rt.log = rt.log, None
  assert len(log) == 2 * len(layers) and all(kernel == "bt_gemv_bfp" for kernel, *_ in log)
  for got, want in zip(queued, separate): assert np.array_equal(got.numpy(), want)
  h = x
  for (wg, wu, wd, fmt), a, out in zip(host, separate[0::2], separate[1::2]):
    ref = o.silu(h @ o.dequant(wg, fmt)) * (h @ o.dequant(wu, fmt))
    check_matmul(a, h, None, ref, TOL_BF16)
    check_matmul(out, a, None, np.maximum(a @ o.dequant(wd, fmt), 0), TOL_BF16)
    h = out


def test_queue_longer_than_one_launch(rt):
  # 40 dependent matmuls: more than one kernel's worth (32), so the list is cut and the second kernel waits for the first
  rng = np.random.default_rng(5)
  w = upload(rt, bf16(np.eye(256, dtype=np.float32) * 1.0)).cast("bfp8").columns()
  x = acts(rng, 4, 256)
  h = upload(rt, x)
  from baretile_b200 import _lib
  before, count = ctypes.c_uint64(), ctypes.c_uint64()
  _lib.call("bt_launch_count", ctypes.byref(before))
  with rt.queue():
    for _ in range(40): h = (h @ w).realize()
  rt.wait()
  _lib.call("bt_launch_count", ctypes.byref(count))
  assert count.value - before.value == 2
  assert np.array_equal(h.numpy(), x)                               # x @ I, forty times


def test_queue_of_independent_matmuls(rt):
  # matmuls that do not read one another's results may overlap inside the launch (two in flight); some do depend
  # (the last reads the first one's result; a dropped result's memory is handed to a later one), which the library
  # works out from the addresses
  rng = np.random.default_rng(41)
  cases = [(1, 1024, 736, "bfp8"), (8, 512, 2048, "bfp4"), (20, 1024, 736, "bfp4"), (3, 2048, 512, "bfp8"), (16, 512, 1024, "bfp8"), (1, 512, 4096, "bfp4")]
  host = [(acts(rng, m, k), weights(rng, k, n), fmt) for m, k, n, fmt in cases]
  dev = [(upload(rt, x), upload(rt, w).cast(fmt).columns()) for x, w, fmt in host]
  w_last = weights(rng, 736, 512)
  tw_last = upload(rt, w_last).cast("bfp8").columns()
  def run():
    dropped = (dev[1][0] @ dev[1][1]).realize()
    del dropped                                              # the allocator hands this memory to a matmul below
    outs = [(x @ w).realize() for x, w in dev]
    outs.append((outs[0] @ tw_last).relu().realize())        # reads the first result
    return outs
  separate = [t.numpy() for t in run()]
  for _ in range(3):
    with rt.queue(): queued = run()
    rt.wait()
    for got, want in zip(queued, separate): assert np.array_equal(got.numpy(), want)
  for (x, w, fmt), got in zip(host, separate): check_matmul(got, x, None, x @ o.dequant(w, fmt), TOL_BF16)
  check_matmul(separate[-1], separate[0], None, np.maximum(separate[0] @ o.dequant(w_last, "bfp8"), 0), TOL_BF16)


def test_queue_random_programs(rt):
  # random lists of matmuls, some reading earlier results, mixed formats, row counts, pairs and epilogues: one queue
  # launch must give the bits that one launch per matmul gives, whatever overlaps inside
  rng = np.random.default_rng(77)
  dims = [256, 512, 736, 1024]
  weights_by_shape = {}
  def weight(k, n, fmt):
    key = (k, n, fmt, int(rng.integers(2)))
    if key not in weights_by_shape: weights_by_shape[key] = upload(rt, weights(rng, k, n) * 2).cast(fmt).columns()
    return weights_by_shape[key]
  for program in range(12):
    m = int(rng.choice([1, 2, 8, 9, 16, 17, 32]))
    steps, width = [], int(rng.choice(dims))
    x0 = upload(rt, acts(rng, m, width))
    for _ in range(int(rng.integers(3, 14))):
      src = int(rng.integers(-1, len(steps)))          # -1: the program's input, else an earlier result
      k = width if src < 0 else steps[src][2]
      n, fmt, kind = int(rng.choice(dims)), str(rng.choice(["bfp8", "bfp4"])), str(rng.choice(["none", "relu", "silu", "glu"]))
      steps.append((src, (weight(k, n, fmt), weight(k, n, fmt) if kind == "glu" else None, kind), n))
    def run():
      outs = []
      for src, (w, w2, kind), _ in steps:
        x = x0 if src < 0 else outs[src]
        y = x @ w
        y = y.relu() if kind == "relu" else y.silu() if kind == "silu" else y.silu() * (x @ w2) if kind == "glu" else y
        outs.append(y.realize())
      return outs
    separate = [t.numpy() for t in run()]
    with rt.queue(): queued = run()
    rt.wait()
    for i, (got, want) in enumerate(zip(queued, separate)): assert np.array_equal(got.numpy(), want, equal_nan=True), (program, i, m, steps[i][0], steps[i][1][2])


def test_queue_with_addend_scale_fp32_and_pick(rt):
  # the other epilogues inside one queue: an addend that is an earlier result, a scale, an fp32 result, the greedy pick
  rng = np.random.default_rng(9)
  m, k, n = 5, 512, 1024
  x, w1, w2, wv = acts(rng, m, k), weights(rng, k, n), weights(rng, k, n), weights(rng, n, 4000 // 32 * 32)
  tx, t1, t2, tv = upload(rt, x), upload(rt, w1).cast("bfp8").columns(), upload(rt, w2).cast("bfp4").columns(), upload(rt, wv).cast("bfp8").columns()
  def run():
    a = (tx @ t1).realize()
    b = ((tx @ t2) * 0.5 + a).relu().realize()                     # reads a as its addend
    c = b.matmul(tv, dtype="fp32").realize()
    values, ids = (b @ tv).topk(1)
    return a, b, c, values, ids
  separate = [t.numpy() for t in run()]
  with rt.queue(): queued = run()
  rt.wait()
  for got, want in zip(queued, separate): assert np.array_equal(got.numpy(), want)
  a, b = separate[0], separate[1]
  check_matmul(b, x, None, np.maximum(0.5 * (x @ o.dequant(w2, "bfp4")) + a, 0), TOL_BF16)
  assert np.array_equal(separate[4][:, 0], o.argmax(separate[2]))


def test_queue_is_flushed_by_a_read(rt):
  # reading a result back inside the block sends what was collected first
  rng = np.random.default_rng(6)
  x, w = acts(rng, 2, 256), weights(rng, 256, 256)
  tx, tw = upload(rt, x), upload(rt, w).cast("bfp8").columns()
  with rt.queue():
    y = (tx @ tw).realize()
    got = y.numpy()
    z = (y @ tw).realize()
  check_matmul(got, x, None, x @ o.dequant(w, "bfp8"), TOL_BF16)
  check_matmul(z.numpy(), got, None, got @ o.dequant(w, "bfp8"), TOL_BF16)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("m", [1, 4, 8])
def test_fused_argmax(rt, fmt, m):
  rng = np.random.default_rng(21 + m)
  x, w = acts(rng, m, 1024), weights(rng, 1024, 4000 // 32 * 32)
  tx, tw = upload(rt, x), upload(rt, w).cast(fmt).columns()
  values, ids = (tx @ tw).topk(1)
  logits = x.astype(np.float32) @ o.dequant(w, fmt)
  want = o.argmax(logits)
  got_ids, got_vals = np.array(ids.tolist())[:, 0], np.array(values.tolist())[:, 0]
  full = tx.matmul(tw, dtype="fp32").realize().numpy()              # the same accumulators, written out
  assert np.array_equal(got_ids, o.argmax(full))                    # exact against the kernel's own fp32 logits
  assert np.array_equal(got_vals, full.max(-1))
  gap = np.sort(logits, -1)[:, -1] - np.sort(logits, -1)[:, -2]
  near = gap <= 2.0 ** -8 * (np.abs(x) @ np.abs(o.dequant(w, fmt))).max(-1)
  assert np.array_equal(got_ids[~near], want[~near])                # and against the oracle except at stated near-ties


def test_argmax_ties_take_the_first_column(rt):
  x = np.zeros((4, 64), np.float32)
  x[:, 0] = 1
  w = np.zeros((64, 2048), np.float32)
  w[0, [5, 700, 1999]] = 2.0                                        # three equal maxima, in different sub-panels
  w[0, 3] = -0.0
  tx, tw = upload(rt, x), upload(rt, w).cast("bfp8").columns()
  values, ids = (tx @ tw).topk(1)
  assert np.array(ids.tolist())[:, 0].tolist() == [5, 5, 5, 5] and np.array(values.tolist())[:, 0].tolist() == [2.0] * 4
  values, ids = (tx @ upload(rt, np.zeros((64, 2048), np.float32)).cast("bfp4")).topk(1)
  assert np.array(ids.tolist())[:, 0].tolist() == [0, 0, 0, 0]      # all equal: column 0


def test_unsupported_expressions_raise(rt):
  from baretile_b200.tensor import Tensor
  x, w = Tensor.zeros(rt, 8, 64), Tensor.zeros(rt, 64, 64)
  with pytest.raises(ValueError, match="block-float"): x @ w                      # bf16 B is outside this path
  with pytest.raises(ValueError, match="columns to match"): x @ Tensor.zeros(rt, 32, 64, dtype="bfp8")
  with pytest.raises(ValueError, match="this backend runs"): x.relu().realize()
  with pytest.raises(ValueError, match="fidelity"): x.matmul(w.cast("bfp8"), fidelity=5)
  with pytest.raises(ValueError): (x @ w.cast("bfp8")).topk(2)
  rt.wait()


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("m", [1, 5, 16, 32])
def test_results_stay_inside_their_tiles(rt, fmt, m):
  # Guard regions either side of the result (the reference's canary trick, test/test_kernels.py:665-680): the kernel
  # writes the result's tiles and nothing else; token rows past M are zero, and a one-row result fills its tile.
  from baretile_b200 import _lib
  rng = np.random.default_rng(17 + m)
  k, n = 512, 736
  x, w = acts(rng, m, k), weights(rng, k, n)
  tx, tw = upload(rt, x), upload(rt, w).cast(fmt).columns()
  guard, size = 4096, (n // 32) * 2048
  buf = rt.dram_alloc(size + 2 * guard)
  try:
    _lib.call("bt_memset", rt.device, buf, 0xA5, size + 2 * guard, rt.stream)
    _lib.call("bt_gemv_bfp", rt.device, int(fmt[3]), 0, m, k, n, tx.addr, tw.addr, 0, 0, ctypes.c_float(1.0), buf + guard, 0, 0, 0, 0,
              rt.work, rt.work_bytes, rt.stream)
    rt.wait()
    raw = np.frombuffer(rt.download(buf, size + 2 * guard), np.uint8)
  finally: rt.dram_free(buf)
  assert (raw[:guard] == 0xA5).all() and (raw[-guard:] == 0xA5).all()
  tiles = np.frombuffer(raw[guard:-guard].tobytes(), np.uint16).reshape(-1, 1024)
  full = o.bf16_floats(o.untilize(tiles, 1, 32, n)[0])              # all 32 rows of the tile row
  ref = x.astype(np.float32) @ o.dequant(w, fmt)
  check_matmul(full[:m], x, o.dequant(w, fmt), ref, TOL_BF16)
  if m == 1: assert (full == full[0]).all()                         # a single row repeats across its tile
  else: assert not full[m:].any()                                   # rows past M are zero


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_matmul_right_after_its_weights_were_written(rt, fmt):
  # cast, columns() and the matmul queued back to back on a large matrix: the matmul's early weight fetches must not
  # overtake the kernels that write the weights (the launch only overlaps a preceding matmul launch)
  rng = np.random.default_rng(3)
  k, n = 4096, 14336
  x, w = acts(rng, 8, k), weights(rng, k, n)
  tx, tb = upload(rt, x), upload(rt, w)
  warm = (tx @ upload(rt, weights(rng, k, 512)).cast(fmt).columns()).realize()    # a matmul launch right before
  y = (tx @ tb.cast(fmt).columns()).realize()                      # pack, relayout and matmul with nothing in between
  rt.wait()
  check_matmul(y.numpy(), x, o.dequant(w, fmt), x @ o.dequant(w, fmt), TOL_BF16)
  del warm


def _tiled(rt, block, reps_k, reps_n, fmt, scales=None):
  """A big weight matrix made of a seeded block repeated reps_k x reps_n times (column copy i scaled by scales[i]), as a
  Tensor in streaming layout, and the dequantised values of one row of blocks. Runs of 16 never straddle a block
  (its width is a multiple of 16), so the block's packed values are the big matrix' packed values; only one row of
  blocks crosses the bus, the others are copies made on the device (tile rows are contiguous in tile layout)."""
  from baretile_b200.tensor import Tensor
  scales = scales if scales is not None else [1.0] * reps_n
  cols = [bf16(block * s) for s in scales]
  row = np.concatenate(cols, axis=1)
  wd_row = np.concatenate([o.dequant(c, fmt) for c in cols], axis=1)
  first = upload(rt, row)
  k, n = block.shape[0] * reps_k, row.shape[1]
  full = Tensor(rt, k, n)
  for r in range(reps_k): rt.launch("bt_d2d", (full.addr + r * first.tiles * 2048, first.addr, first.tiles * 2048), name="copy")
  return full.cast(fmt).columns(), wd_row


def _folded(x, reps_k):
  """x @ tile(B, (reps_k, 1)) = (sum of x's reps_k column blocks) @ B: the activations folded onto one row of blocks, in float64."""
  m, k = x.shape
  return x.astype(np.float64).reshape(m, reps_k, k // reps_k)


@pytest.mark.parametrize("k,n", [(4096, 4096), (4096, 14336), (14336, 4096)])
@pytest.mark.parametrize("m", [1, 32])
def test_llama_shapes_other_row_counts(rt, k, n, m):
  # configs[1] at M = 1 and M = 32 on the three full shapes (M = 8 is test_llama_shapes)
  rng = np.random.default_rng(k + n + m)
  x, w = acts(rng, m, k), weights(rng, k, n)
  for fmt in ("bfp8", "bfp4"):
    got, ref = run(rt, x, w, fmt)
    check_matmul(got, x, None, ref, TOL_BF16)


@pytest.mark.parametrize("m", [1, 4, 16])
def test_llama70b_layer_shapes(rt, m):
  # configs[3] on one GPU at full size: gate/up [8192, 28672] bfp4 fused, then down [28672, 8192] bfp4
  rng = np.random.default_rng(70 + m)
  bg, bu, bd = weights(rng, 1024, 1024), weights(rng, 1024, 1024), weights(rng, 1024, 1024)
  x = acts(rng, m, 8192)
  tx = upload(rt, x)
  (tg, dg), (tu, du), (td, dd) = _tiled(rt, bg, 8, 28, "bfp4"), _tiled(rt, bu, 8, 28, "bfp4"), _tiled(rt, bd, 28, 8, "bfp4")
  h = ((tx @ tg).silu() * (tx @ tu)).realize()
  y = (h @ td).realize()
  hg = h.numpy()
  xf = _folded(x, 8).sum(1)
  ref_h = o.silu((xf @ dg).astype(np.float32)) * (xf @ du).astype(np.float32)
  check_matmul(hg, x, None, ref_h, TOL_BF16)
  hf = _folded(hg, 28)
  check_matmul(y.numpy(), None, None, hf.sum(1) @ dd, TOL_BF16)
  room = np.abs(hf).sum(1) @ np.abs(dd)                             # the per-element bound, 2^-8 of sum |h||w|
  assert (np.abs(y.numpy() - hf.sum(1) @ dd) <= 2.0 ** -8 * room * (1 + 2.0 ** -10)).all()


@pytest.mark.parametrize("m", [1, 4, 8])
def test_lm_head_pick_full_size(rt, m):
  # configs[4] on one GPU: x[M, 8192] @ W[8192, 128256] bfp8 with the fused greedy pick; the index is exact against
  # the kernel's own fp32 logits everywhere, and against the oracle outside the stated near-ties
  rng = np.random.default_rng(400 + m)
  block = weights(rng, 1024, 2672)                                 # 48 copies side by side make the 128256 columns
  tw, wd = _tiled(rt, block, 8, 48, "bfp8", scales=[1 + i / 64 for i in range(48)])
  x = acts(rng, m, 8192)
  tx = upload(rt, x)
  values, ids = (tx @ tw).topk(1)
  got_ids, got_vals = np.array(ids.tolist())[:, 0], np.array(values.tolist())[:, 0]
  full = tx.matmul(tw, dtype="fp32").realize().numpy()
  assert np.array_equal(got_ids, o.argmax(full)) and np.array_equal(got_vals, full.max(-1))
  xf = _folded(x, 8)
  logits = xf.sum(1) @ wd
  assert o.rel_err(full, logits) <= TOL_FP32
  top2 = np.sort(logits, -1)[:, -2:]
  near = top2[:, 1] - top2[:, 0] <= 2.0 ** -8 * (np.abs(xf).sum(1) @ np.abs(wd)).max(-1)
  assert np.array_equal(got_ids[~near], o.argmax(logits)[~near]), ("near ties at rows", np.nonzero(near)[0].tolist())
