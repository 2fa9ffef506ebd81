"""Open a device: the CUDA stand-in for the reference's device openers (baretile/pci.py:33-106 Sim, :453-463
open_device). Device n is CUDA device n of this process."""
import ctypes
from baretile_b200 import _lib


class Cuda:
  """One CUDA device, opened. The slot the reference fills with Sim, Kmd or Card."""
  def __init__(self, index):
    self.index, info = index, _lib.DeviceInfo()
    _lib.call("bt_device_info_get", index, ctypes.byref(info))
    self.name, self.sm_count, self.cc = info.name.decode(), info.sm_count, (info.cc_major, info.cc_minor)
    self.memory_bytes, self.l2_bytes, self.clock_khz, self.max_shared_bytes = info.memory_bytes, info.l2_bytes, info.clock_khz, info.max_shared_bytes
    if self.cc[0] != 10:
      raise RuntimeError(f"not a B200-class device: {self.name} has compute capability {self.cc[0]}.{self.cc[1]}, and the kernels are built for sm_100a")

  @staticmethod
  def chips():
    n = ctypes.c_int()
    _lib.call("bt_device_count", ctypes.byref(n))
    return list(range(n.value))


def open_device(n=0):
  """Open CUDA device n (reference: baretile/pci.py:453-463, same error for an index out of range)."""
  found = Cuda.chips()
  if not 0 <= n < len(found): raise ValueError(f"open_device({n}): there are {len(found)} chips")
  return Cuda(found[n])
