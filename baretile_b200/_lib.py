"""ctypes binding of libbaretile_b200.so (declared in include/baretile_b200.h).

The reference binds its device library the same way: ctypes.CDLL with explicit argtypes and restype
(baretile/pci.py:52-63). Status codes become the exceptions the reference raises for the same conditions
(docs/api.md:51-62): bad argument -> ValueError, device or state -> RuntimeError, timeout -> TimeoutError,
out of memory -> MemoryError."""
import ctypes, os, pathlib

PATH = pathlib.Path(os.environ.get("BARETILE_B200_LIB") or pathlib.Path(__file__).resolve().parent / "libbaretile_b200.so")
u64, i32, f32, size_t, vp = ctypes.c_uint64, ctypes.c_int, ctypes.c_float, ctypes.c_size_t, ctypes.c_void_p


class DeviceInfo(ctypes.Structure):
  _fields_ = [("name", ctypes.c_char * 64), ("sm_count", i32), ("cc_major", i32), ("cc_minor", i32), ("l2_bytes", i32),
              ("memory_bytes", u64), ("max_shared_bytes", i32), ("clock_khz", i32)]


class GemvOp(ctypes.Structure):
  """bt_gemv_op: one matmul of a bt_gemv_queue call; the fields are bt_gemv_bfp's arguments of the same names."""
  _fields_ = [("fmt", i32), ("epilogue", i32), ("M", i32), ("K", i32), ("N", i32), ("out_dtype", i32), ("arg_base", i32), ("alpha", f32),
              ("x", u64), ("w", u64), ("w2", u64), ("add", u64), ("out", u64), ("arg_val", u64), ("arg_idx", u64)]


SIGNATURES = {
  "bt_device_count": [ctypes.POINTER(i32)],
  "bt_device_info_get": [i32, ctypes.POINTER(DeviceInfo)],
  "bt_malloc": [i32, size_t, ctypes.POINTER(u64)],
  "bt_free": [i32, u64],
  "bt_host_alloc": [size_t, ctypes.POINTER(vp)],
  "bt_host_free": [vp],
  "bt_stream_create": [i32, ctypes.POINTER(u64)],
  "bt_stream_destroy": [i32, u64],
  "bt_stream_sync": [i32, u64, i32],
  "bt_stream_query": [i32, u64, ctypes.POINTER(i32)],
  "bt_h2d": [i32, u64, vp, size_t, u64],
  "bt_d2h": [i32, vp, u64, size_t, u64],
  "bt_d2d": [i32, u64, u64, size_t, u64],
  "bt_memset": [i32, u64, i32, size_t, u64],
  "bt_event_create": [i32, ctypes.POINTER(u64)],
  "bt_event_destroy": [i32, u64],
  "bt_event_record": [i32, u64, u64],
  "bt_event_elapsed_ms": [i32, u64, u64, ctypes.POINTER(f32)],
  "bt_stream_wait_event": [i32, u64, u64],
  "bt_graph_begin": [i32, u64],
  "bt_graph_end": [i32, u64, ctypes.POINTER(u64)],
  "bt_graph_launch": [i32, u64, u64],
  "bt_graph_destroy": [i32, u64],
  "bt_tilize": [i32, i32, u64, u64, i32, i32, i32, u64],
  "bt_untilize": [i32, i32, u64, u64, i32, i32, i32, u64],
  "bt_tilize_many": [i32, i32, i32, ctypes.POINTER(u64), ctypes.POINTER(u64), ctypes.POINTER(i32), ctypes.POINTER(i32), u64],
  "bt_untilize_many": [i32, i32, i32, ctypes.POINTER(u64), ctypes.POINTER(u64), ctypes.POINTER(i32), ctypes.POINTER(i32), u64],
  "bt_round_bf16": [i32, u64, u64, size_t, u64],
  "bt_pack_bfp": [i32, i32, u64, u64, size_t, u64],
  "bt_unpack_bfp": [i32, i32, u64, u64, size_t, u64],
  "bt_put": [i32, i32, u64, u64, u64, i32, i32, i32, i32, u64, u64],
  "bt_relayout": [i32, i32, i32, i32, i32, u64, u64, u64],
  "bt_gemv_workspace_bytes": [i32, ctypes.POINTER(size_t)],
  "bt_gemv_bfp": [i32, i32, i32, i32, i32, i32, u64, u64, u64, u64, f32, u64, i32, u64, u64, i32, u64, size_t, u64],
  "bt_gemm_bfp": [i32, i32, i32, i32, i32, i32, u64, u64, u64, u64, i32, f32, u64, i32, u64, u64],
  "bt_gemv_bfp_static": [i32, i32, i32, i32, i32, i32, u64, u64, u64, u64, f32, u64, i32, u64, u64, i32, u64],
  "bt_gemv_check": [i32, u64, u64, ctypes.POINTER(i32)],
  "bt_gemv_queue": [i32, i32, ctypes.POINTER(GemvOp), u64, size_t, u64],
  "bt_gemv_queue_plan": [i32, ctypes.POINTER(GemvOp), ctypes.POINTER(i32)],
  "bt_comm_unique_id": [vp, size_t],
  "bt_comm_init": [i32, i32, i32, vp, ctypes.POINTER(u64)],
  "bt_comm_destroy": [u64],
  "bt_allgather": [i32, u64, u64, u64, size_t, u64],
  "bt_allreduce_sum": [i32, u64, u64, size_t, u64],
  "bt_round_tilize": [i32, u64, u64, i32, i32, u64],
  "bt_argmax_combine": [i32, u64, i32, i32, u64, u64, u64],
  "bt_peer_open": [i32, u64, i32, i32, size_t, ctypes.POINTER(u64), u64],
  "bt_peer_close": [i32, u64, i32, i32, ctypes.POINTER(u64), u64],
  "bt_peer_allreduce_round": [i32, i32, i32, ctypes.POINTER(u64), size_t, i32, i32, i32, u64, u64],
  "bt_peer_argmax_combine": [i32, i32, i32, ctypes.POINTER(u64), size_t, i32, i32, u64, u64, u64, u64],
  "bt_peer_check": [i32, i32, ctypes.POINTER(u64), u64, ctypes.POINTER(i32)],
  "bt_launch_count": [ctypes.POINTER(u64)],
}

ERRORS = {1: ValueError, 2: RuntimeError, 3: TimeoutError, 4: MemoryError}
_lib = None


def lib():
  """The loaded library. Raises if it was not built: this backend has no other way to compute."""
  global _lib
  if _lib is None:
    if not PATH.exists():
      raise RuntimeError(f"{PATH} is missing: build it with `make -C {PATH.parent / 'csrc'}` (needs nvcc, sm_100a); "
                         "baretile_b200 has no CPU fallback")
    loaded = ctypes.CDLL(str(PATH))
    for name, argtypes in SIGNATURES.items():
      f = getattr(loaded, name)
      f.argtypes, f.restype = argtypes, i32
    loaded.bt_last_error.argtypes, loaded.bt_last_error.restype = [], ctypes.c_char_p
    _lib = loaded
  return _lib


def check(status):
  """Raise the exception that matches a nonzero status, with the library's message."""
  if status: raise ERRORS.get(status, RuntimeError)(lib().bt_last_error().decode(errors="replace"))


def call(name, *args): check(getattr(lib(), name)(*args))
