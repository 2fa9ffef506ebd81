"""Helpers shared by the GPU tests: seeded inputs of the benchmark's distributions and oracle-side references."""
import numpy as np
from oracle import bfp_oracle as o


def bf16(a):
  """Round to bf16 (nearest even) and back to float32."""
  return o.bf16_floats(o.bf16_bits(np.asarray(a, np.float32)))


def weights(rng, k, n, stress=True):
  """N(0, 0.02) weights with 1% of the input channels scaled by 20, which stresses the shared exponents."""
  w = rng.normal(0, 0.02, (k, n)).astype(np.float32)
  if stress and k >= 100: w[rng.choice(k, k // 100, replace=False)] *= 20
  return bf16(w)


def acts(rng, m, k): return bf16(rng.normal(0, 1, (m, k)))


def upload(rt, a, dtype="bf16"):
  """A float32 array that already holds bf16 values -> Tensor, without going through Python lists."""
  from baretile_b200.tensor import Tensor
  a = np.ascontiguousarray(a, np.float32)
  rows, cols = a.shape[-2:]
  batch = a.shape[0] if a.ndim == 3 else 1
  if dtype == "bf16": return Tensor.frombytes(rt, rows, cols, o.bf16_bits(a).tobytes(), batch, "bf16")
  return Tensor.frombytes(rt, rows, cols, a.astype(np.int32 if dtype == "int32" else np.float32).tobytes(), batch, dtype)


def raw_tiles(rt, t):
  """The tensor's storage bytes as a (tiles, tile_bytes) array."""
  from baretile_b200.tensix import tile_bytes
  rt.wait()
  tb = tile_bytes(t.dtype)
  return np.frombuffer(rt.download(t.addr, t.tiles * tb), np.uint8).reshape(t.tiles, tb)


def check_matmul(got, x, wd, ref, tol=1e-2, addend=None, alpha=1.0):
  """The two bounds the reference uses: max relative error (docs/workload.md:141) within tol, and, when the
  dequantised weights wd are given (a linear or ReLU result: a 1-Lipschitz epilogue), every element within
  2^-8 of sum |x||w| (+ |addend|), the bound of test/test_kernels.py:745: half a bf16 step of the largest value
  the sum could have, which covers the one rounding of the result; accumulation is fp32 over exact products."""
  got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
  assert got.shape == ref.shape, (got.shape, ref.shape)
  assert np.isfinite(got).all()
  err = o.rel_err(got, ref)
  assert err <= tol, err
  if wd is not None and x is not None:
    room = abs(alpha) * (np.abs(np.asarray(x, np.float64)) @ np.abs(np.asarray(wd, np.float64)))
    if addend is not None: room = room + np.abs(np.asarray(addend, np.float64))
    over = np.abs(got - ref) - 2.0 ** -8 * room * (1 + 2.0 ** -10) - 1e-30
    assert (over <= 0).all(), (float(over.max()), np.unravel_index(over.argmax(), over.shape))
  return err
