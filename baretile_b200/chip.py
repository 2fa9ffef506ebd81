"""Raw access to a device's memory and its description: the part of the reference's Chip that the matmul path and
its tests use (baretile/chip.py:7-83: read, write, read32, write32, telemetry; `tensix`, `banks`, `aiclk`).
NoC windows, ARC messages and Ethernet have no counterpart on a GPU."""
import ctypes
from baretile_b200 import _lib


class Chip:
  def __init__(self, pci):
    self.pci, self.device = pci, pci.index
    self.taken = {}                       # runtimes open on this chip
    self.aiclk = pci.clock_khz // 1000    # MHz, as the reference reports its AI clock
    self.tensix = [(sm, 0) for sm in range(pci.sm_count)]   # the workers: one per SM
    self.banks = [0]                      # HBM is one address space

  def read(self, addr, n):
    """n bytes of device memory at addr (blocking). Reference: Chip.read (baretile/chip.py:75)."""
    if addr < 0 or n < 0: raise ValueError("addresses and transfer sizes must be nonnegative")
    buf = ctypes.create_string_buffer(n)
    _lib.call("bt_d2h", self.device, ctypes.cast(buf, ctypes.c_void_p), addr, n, 0)
    _lib.call("bt_stream_sync", self.device, 0, -1)
    return buf.raw

  def write(self, addr, data):
    """Write bytes at addr (blocking). Reference: Chip.write (baretile/chip.py:76-82)."""
    data = bytes(data)
    if addr < 0: raise ValueError("addresses and transfer sizes must be nonnegative")
    _lib.call("bt_h2d", self.device, addr, ctypes.cast(ctypes.c_char_p(data), ctypes.c_void_p), len(data), 0)
    _lib.call("bt_stream_sync", self.device, 0, -1)

  def read32(self, addr): return int.from_bytes(self.read(addr, 4), "little")
  def write32(self, addr, val): self.write(addr, val.to_bytes(4, "little"))

  def telemetry(self):
    p = self.pci
    return {"name": p.name, "sm_count": p.sm_count, "memory_bytes": p.memory_bytes, "l2_bytes": p.l2_bytes, "clock_mhz": self.aiclk}
