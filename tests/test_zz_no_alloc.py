"""The matmul entry point for hosts that cannot allocate device memory (bt_gemv_bfp_static).

Who needs it: code embedded where cudaMalloc is not allowed or not possible -- inside a framework's stream capture,
in a process that handed out its whole memory budget at start-up, or in a plug-in that is only given input and output
buffers. The variant keeps the kernel's scratch (arrival counters, partial sums, argmax candidates) in a fixed array
inside the library instead of taking it from the caller. This file is collected last on purpose, so that a run that
stops at the first failure has already run every other test.

It calls the entry point through the C-ABI twice in a row on different inputs and checks each result against the
ordinary entry point's: the two run the same kernel with the same work split, so the results are required to be equal
bit for bit, which is inside the 1e-2 relative tolerance the other matmul tests use."""
import ctypes
import numpy as np
import pytest
from oracle import bfp_oracle as o
from helpers import acts, upload, weights

pytestmark = pytest.mark.gpu


def both(rt, x, w, fmt, epilogue, w2=None):
  """(result through bt_gemv_bfp_static, result through bt_gemv_bfp), each as float32 arrays."""
  from baretile_b200 import _lib
  from baretile_b200.tensor import Tensor
  m, k = x.shape
  n = w.shape[1]
  tx = upload(rt, x)
  tw = upload(rt, w).cast(fmt).columns()
  tw2 = upload(rt, w2).cast(fmt).columns() if w2 is not None else None
  code = {"none": 0, "relu": 1, "glu": 3}[epilogue]
  outs = []
  for static in (True, False):
    out = Tensor.zeros(rt, m, n)
    args = (rt.device, int(fmt[3]), code, m, k, n, tx.addr, tw.addr, tw2.addr if tw2 else 0, 0, ctypes.c_float(1.0), out.addr, 0, 0, 0, 0)
    if static: _lib.call("bt_gemv_bfp_static", *args, rt.stream)
    else: _lib.call("bt_gemv_bfp", *args, rt.work, rt.work_bytes, rt.stream)
    rt.wait()
    outs.append(out.numpy())
  return outs


def test_static_scratch_matches_twice_in_a_row(rt):
  rng = np.random.default_rng(77)
  for call, (m, k, n, fmt, epilogue) in enumerate(((8, 2048, 2208, "bfp8", "relu"), (3, 4096, 1536, "bfp4", "glu"))):
    x, w = acts(rng, m, k), weights(rng, k, n)
    w2 = weights(rng, k, n) if epilogue == "glu" else None
    got, want = both(rt, x, w, fmt, epilogue, w2)
    assert np.array_equal(got, want), (call, o.rel_err(got, want))
    ref = o.matmul(x, o.dequant(w, fmt), epilogue, o.dequant(w2, fmt) if w2 is not None else None)
    assert o.rel_err(got, ref) <= 1e-2, call


def test_static_scratch_pick_and_its_error_word(rt):
  # the greedy pick through the built-in scratch, twice, against the ordinary entry point; and the word that records a
  # wait that gave up is readable for the built-in scratch too (work = 0) and reads zero after clean runs
  from baretile_b200 import _lib
  rng = np.random.default_rng(9)
  m, k, n = 5, 1024, 4000 // 32 * 32
  flat = rt.dram_alloc(1024)
  try:
    for call in range(2):
      x, w = acts(rng, m, k), weights(rng, k, n)
      tx, tw = upload(rt, x), upload(rt, w).cast("bfp8").columns()
      picks = []
      for static in (True, False):
        _lib.call("bt_memset", rt.device, flat, 0xFF, 1024, rt.stream)
        args = (rt.device, 8, 4, m, k, n, tx.addr, tw.addr, 0, 0, ctypes.c_float(1.0), 0, 0, flat, flat + 512, 7)
        if static: _lib.call("bt_gemv_bfp_static", *args, rt.stream)
        else: _lib.call("bt_gemv_bfp", *args, rt.work, rt.work_bytes, rt.stream)
        rt.wait()
        raw = rt.download(flat, 1024)
        picks.append((np.frombuffer(raw[:4 * m], np.float32).copy(), np.frombuffer(raw[512:512 + 4 * m], np.int32).copy()))
      assert np.array_equal(picks[0][0], picks[1][0]) and np.array_equal(picks[0][1], picks[1][1]), call
      logits = tx.matmul(tw, dtype="fp32").realize().numpy()
      assert np.array_equal(picks[0][1] - 7, o.argmax(logits)) and np.array_equal(picks[0][0], logits.max(-1))
    error = ctypes.c_int(-1)
    _lib.call("bt_gemv_check", rt.device, 0, rt.stream, ctypes.byref(error))
    assert error.value == 0
  finally: rt.dram_free(flat)


def test_static_scratch_rejects_what_it_cannot_hold(rt):
  from baretile_b200 import _lib
  with pytest.raises(ValueError, match="up to 8 rows"):
    _lib.call("bt_gemv_bfp_static", rt.device, 8, 0, 9, 64, 64, 256, 256, 0, 0, ctypes.c_float(1.0), 256, 0, 0, 0, 0, rt.stream)
  with pytest.raises(ValueError, match="columns"):
    _lib.call("bt_gemv_bfp_static", rt.device, 8, 0, 1, 64, 1 << 20, 256, 256, 0, 0, ctypes.c_float(1.0), 256, 0, 0, 0, 0, rt.stream)
  rt.wait()
