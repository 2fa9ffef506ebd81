"""The tensor-core (tcgen05) matmul for many rows against the oracle's fp32 NumPy matmul over the same dequantised
weights: max relative error 1e-2 for bf16 results, 1e-4 for fp32 results (relative error as in docs/workload.md:141)."""
import numpy as np
import pytest
from oracle import bfp_oracle as o
from helpers import acts, bf16, check_matmul, upload, weights

pytestmark = pytest.mark.gpu


def run(rt, x, w, fmt, epilogue="none", w2=None, dtype=None):
  tx, tw = upload(rt, x), upload(rt, w).cast(fmt).columns()
  y, ref = tx.matmul(tw, dtype=dtype), x.astype(np.float32) @ o.dequant(w, fmt)
  if epilogue == "relu": y, ref = y.relu(), np.maximum(ref, 0)
  elif epilogue == "silu": y, ref = y.silu(), o.silu(ref)
  elif epilogue == "glu":
    y, ref = y.silu() * tx.matmul(upload(rt, w2).cast(fmt).columns(), dtype=dtype), o.silu(ref) * (x.astype(np.float32) @ o.dequant(w2, fmt))
  rt.log = []
  got = y.realize()
  rt.wait()
  names, rt.log = [n for *_, n in rt.log], None
  assert any(n.startswith("prefill") for n in names), names       # the tensor-core kernel ran, not the decode loop
  return got.numpy(), ref


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
