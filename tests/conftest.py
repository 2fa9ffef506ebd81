"""Shared fixtures. Tests marked `gpu` need a B200 and the built CUDA library; everything else runs on CPU."""
import ctypes, pathlib, subprocess, sys
import numpy as np
import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path: sys.path.insert(0, str(ROOT))


def pytest_configure(config):
  config.addinivalue_line("markers", "gpu: needs a CUDA device (B200) and the built libbaretile_b200.so")


@pytest.fixture(scope="session")
def golden():
  return np.load(ROOT / "tests" / "golden" / "bfp_golden.npz")


@pytest.fixture(scope="session")
def c_oracle():
  """The C restatement of pack/unpack, built on demand with gcc."""
  so = ROOT / "oracle" / "_build" / "libbfp_oracle.so"
  if not so.exists(): subprocess.run(["make", "-C", str(ROOT / "oracle")], check=True, capture_output=True)
  lib = ctypes.CDLL(str(so))
  for f in (lib.oracle_pack, lib.oracle_unpack):
    f.argtypes, f.restype = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t], ctypes.c_int
  def pack(tiles, fmt):
    tiles = np.ascontiguousarray(tiles, np.uint16).reshape(-1, 1024)
    out = np.zeros((len(tiles), 1088 if fmt == "bfp8" else 576), np.uint8)
    assert lib.oracle_pack(int(fmt[3]), tiles.ctypes.data, out.ctypes.data, len(tiles)) == 0
    return out
  def unpack(tiles, fmt):
    tiles = np.ascontiguousarray(tiles, np.uint8).reshape(-1, 1088 if fmt == "bfp8" else 576)
    out = np.zeros((len(tiles), 1024), np.uint16)
    assert lib.oracle_unpack(int(fmt[3]), tiles.ctypes.data, out.ctypes.data, len(tiles)) == 0
    return out
  return type("COracle", (), {"pack": staticmethod(pack), "unpack": staticmethod(unpack)})


@pytest.fixture(scope="session")
def rt():
  """One runtime on CUDA device 0 for the GPU tests."""
  from baretile_b200 import pci
  from baretile_b200.chip import Chip
  from baretile_b200.runtime import Runtime
  runtime = Runtime(Chip(pci.open_device(0)))
  yield runtime
  runtime.close()
