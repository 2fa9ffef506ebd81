"""The tensor-core (tcgen05) matmul for many rows against the oracle's fp32 NumPy matmul over the same dequantised
weights: max relative error 1e-2 for bf16 results, 1e-4 for fp32 results (relative error as in docs/workload.md:141)."""
import numpy as np
import pytest
from oracle import bfp_oracle as o
from helpers import acts, bf16, check_matmul, upload, weights

pytestmark = pytest.mark.gpu


def deq(w, fmt):
  """The oracle's dequantised weights for any N: columns padded with zeros to whole tiles, as the tensor stores them."""
  pad = -w.shape[1] % 32
  return o.dequant(np.pad(w, ((0, 0), (0, pad))), fmt)[:, :w.shape[1]]


def run(rt, x, w, fmt, epilogue="none", w2=None, dtype=None, add=None, alpha=None):
  tx, tw = upload(rt, x), upload(rt, w).cast(fmt).columns()
  y, ref = tx.matmul(tw, dtype=dtype), x.astype(np.float32) @ deq(w, fmt)
  if alpha is not None: y, ref = y * alpha, ref * np.float32(alpha)
  if add is not None: y, ref = y + upload(rt, add), ref + add
  if epilogue == "relu": y, ref = y.relu(), np.maximum(ref, 0)
  elif epilogue == "silu": y, ref = y.silu(), o.silu(ref)
  elif epilogue == "glu":
    y, ref = y.silu() * tx.matmul(upload(rt, w2).cast(fmt).columns(), dtype=dtype), o.silu(ref) * (x.astype(np.float32) @ deq(w2, fmt))
  rt.log = []
  got = y.realize()
  rt.wait()
  names, rt.log = [n for *_, n in rt.log], None
  assert sum(n.startswith("prefill") for n in names) == 1, names    # the tensor-core kernel ran, once, not the decode loop
  out = got.numpy()
  if epilogue in ("none", "relu"):   # every element within 2^-8 of sum |x||w| (+ |addend|): the reference's per-element bound
    check_matmul(out, x, deq(w, fmt), ref, 1e-2 if dtype != "fp32" else 1e-4, addend=add, alpha=alpha if alpha is not None else 1.0)
  return out, ref


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_exact_integers_pin_the_operand_layouts(rt, fmt):
  # small integers are exact in both formats and in fp32 sums: any misplaced row, column or k shows up
  rng = np.random.default_rng(1)
  x = rng.integers(-2, 3, (256, 128)).astype(np.float32)
  w = rng.integers(-1, 2, (128, 256)).astype(np.float32)
  got, ref = run(rt, x, w, fmt, dtype="fp32")
  assert np.array_equal(got, x @ w)
  eye = np.zeros((256, 256), np.float32)
  eye[np.arange(256), np.arange(256)] = 1
  xr = bf16(rng.uniform(-8, 8, (200, 256)))
  got, _ = run(rt, xr, eye, fmt)
  assert np.array_equal(got, xr)                                   # A @ I == A, with a ragged last block of rows


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("m", [33, 128, 300, 512])
def test_rows(rt, fmt, m):
  rng = np.random.default_rng(m)
  x, w = acts(rng, m, 1024), weights(rng, 1024, 512)
  got, ref = run(rt, x, w, fmt)
  check_matmul(got, x, None, ref, 1e-2)
  got, ref = run(rt, x, w, fmt, "relu", dtype="fp32")
  check_matmul(got, x, None, ref, 1e-4)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_gate_up_pair(rt, fmt):
  rng = np.random.default_rng(4)
  x, w, w2 = acts(rng, 384, 512), weights(rng, 512, 640), weights(rng, 512, 640)
  got, ref = run(rt, x, w, fmt, "glu", w2)
  check_matmul(got, x, None, ref, 1e-2)


def test_config2_shapes_reduced_rows(rt):
  # the prefill configuration's weights at full size (4096 x 14336 gate/up in bfp8, 14336 x 4096 down in bfp4), 256 rows
  rng = np.random.default_rng(2)
  x = acts(rng, 256, 4096)
  wg, wu = weights(rng, 4096, 14336), weights(rng, 4096, 14336)
  got, ref = run(rt, x, wg, "bfp8", "glu", wu)
  check_matmul(got, x, None, ref, 1e-2)
  h = bf16(ref)
  wd = weights(rng, 14336, 4096)
  got, ref = run(rt, h, wd, "bfp4")
  check_matmul(got, h, None, ref, 1e-2)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_addend_and_scale(rt, fmt):
  # a bias row and a residual of M rows, added before the activation; a scale; fp32 results
  rng = np.random.default_rng(5)
  x, w = acts(rng, 300, 256), weights(rng, 256, 512)
  bias, resid = bf16(rng.normal(0, 1, (1, 512))), bf16(rng.normal(0, 1, (300, 512)))
  for add in (bias, resid):
    got, ref = run(rt, x, w, fmt, "relu", add=add)
    check_matmul(got, x, None, ref, 1e-2)
    got, ref = run(rt, x, w, fmt, "silu", add=add)
    check_matmul(got, x, None, ref, 1e-2)
  got, ref = run(rt, x, w, fmt, alpha=0.5, add=resid, dtype="fp32")
  check_matmul(got, x, None, ref, 1e-4)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("k,n", [(96, 96), (160, 1000), (1024, 416), (80, 130), (64, 32), (32, 4128)])
def test_shapes_that_are_not_whole_blocks(rt, fmt, k, n):
  # a last run of fewer than four tile columns, a block column with one run, an odd last tile row of K, and K and N
  # that are not whole tiles: all through the one kernel, exact on small integers and within tolerance on weights
  rng = np.random.default_rng(k * 7 + n)
  xi, wi = rng.integers(-2, 3, (70, k)).astype(np.float32), rng.integers(-1, 2, (k, n)).astype(np.float32)
  got, _ = run(rt, xi, wi, fmt, dtype="fp32")
  assert np.array_equal(got, xi @ wi)
  x, w, w2 = acts(rng, 300, k), weights(rng, k, n, stress=False), weights(rng, k, n, stress=False)
  add = bf16(rng.normal(0, 1, (300, n)))
  got, ref = run(rt, x, w, fmt, "relu", add=add)
  check_matmul(got, x, None, ref, 1e-2)
  got, ref = run(rt, x, w, fmt, "glu", w2)
  check_matmul(got, x, None, ref, 1e-2)


def test_results_stay_inside_their_tiles(rt):
  # the tensors either side of a result in device memory keep their bytes (ragged rows and columns included)
  from baretile_b200.tensor import Tensor
  from helpers import raw_tiles
  rng = np.random.default_rng(9)
  x, w = acts(rng, 70, 96), weights(rng, 96, 130, stress=False)
  tx, tw = upload(rt, x), upload(rt, w).cast("bfp8").columns()
  before = upload(rt, np.full((32, 32), 3.0, np.float32))
  y = (tx @ tw).realize()
  after = upload(rt, np.full((32, 32), 5.0, np.float32))
  y2 = (tx @ tw).relu().realize()
  assert np.all(before.numpy() == 3.0) and np.all(after.numpy() == 5.0)
  assert np.array_equal(np.maximum(y.numpy(), 0), y2.numpy())
  tiles = raw_tiles(rt, y).view(np.uint16).reshape(3, 5, 1024)
  full = o.untilize(tiles.reshape(15, 1024), 1, 96, 160)[0]
  assert not full[70:].any() and not full[:, 130:].any()            # rows past M and columns past N are zero
