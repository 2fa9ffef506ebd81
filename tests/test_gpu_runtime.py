"""The runtime mirror on the GPU: ordering, waiting, closing, memory reuse and error reporting without faults."""
import ctypes
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_open_and_describe():
  from baretile_b200 import pci
  from baretile_b200.chip import Chip
  with pytest.raises(ValueError, match="there are"): pci.open_device(1 << 20)
  chip = Chip(pci.open_device(0))
  t = chip.telemetry()
  assert t["sm_count"] > 0 and t["memory_bytes"] > 1 << 30 and len(chip.tensix) == t["sm_count"]


def test_alloc_free_reuse_and_close(rt):
  from baretile_b200.tensor import Tensor
  used = dict(rt.used)
  junk = Tensor.of(rt, np.random.default_rng(3).integers(1, 9, (2, 70, 100)).tolist(), "int32")
  at = junk.addr
  del junk
  z = Tensor.zeros(rt, 70, 100, 2, "int32")
  assert z.addr == at and not np.array(z.tolist()).any()             # freed memory is reused, and zeros overwrites it
  del z
  assert rt.used == used
  with pytest.raises(MemoryError, match="bytes free in DRAM"): rt.dram_alloc(1 << 50)
  rt.wait()
  with pytest.raises(ValueError, match="never queued"): rt.wait(launch=rt.launches + 5)


def test_profile_names(rt):
  from baretile_b200.tensor import Tensor
  since = rt.launches
  Tensor.zeros(rt, 32, 32)
  Tensor.zeros(rt, 32, 32)
  rows = rt.profile(since)
  assert rows[0][0] == "zeros" and rows[0][1] == 2


def test_second_runtime_replaces_the_first():
  # a new Runtime on the chip closes the old one; its tensors can no longer run (baretile/runtime.py:593-598)
  from baretile_b200 import pci
  from baretile_b200.chip import Chip
  from baretile_b200.runtime import Runtime
  from baretile_b200.tensor import Tensor
  chip = Chip(pci.open_device(0))
  a = Runtime(chip, timing=True)
  x = Tensor.zeros(a, 32, 32)
  since = a.launches
  Tensor.zeros(a, 64, 64)
  assert a.profile(since)[0][2] >= 0
  b = Runtime(chip)
  assert a.closed and not b.closed
  with pytest.raises(RuntimeError, match="closed"): x.tolist()
  with pytest.raises(RuntimeError, match="closed"): Tensor.zeros(a, 1, 1)
  b.close(); b.close()
  assert b.closed
