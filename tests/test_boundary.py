"""The C-ABI boundary and the host-side mirror, without a GPU: the library loads and exports every symbol the header
declares, the Python bindings agree with the header, and argument checks run before anything touches a device."""
import ctypes, pathlib, re, subprocess, sys
import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "baretile_b200.h").read_text()


def declared():
  code = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
  return {m.group(2): m.group(3) for m in re.finditer(r"\b(int|const char \*)\s*(bt_\w+)\s*\(([^;]*)\)\s*;", code)}


@pytest.fixture(scope="module")
def built():
  so = ROOT / "baretile_b200" / "libbaretile_b200.so"
  if not so.exists():
    run = subprocess.run(["make", "-C", str(ROOT / "baretile_b200" / "csrc"), "-j4"], capture_output=True, text=True)
    assert run.returncode == 0, run.stderr[-2000:]
  return so


def test_library_exports_every_declared_symbol(built):
  lib, names = ctypes.CDLL(str(built)), declared()
  assert len(names) >= 25
  for name in names: assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_bindings_match_header(built):
  from baretile_b200 import _lib
  names = declared()
  for name, argtypes in _lib.SIGNATURES.items():
    assert name in names, f"{name} is bound but not declared"
    params = [p for p in names[name].split(",") if p.strip() and p.strip() != "void"]
    assert len(params) == len(argtypes), (name, names[name])
  assert set(names) - set(_lib.SIGNATURES) == {"bt_last_error"}
  _lib.lib()


def test_argument_checks_need_no_device(built):
  from baretile_b200 import _lib
  n = ctypes.c_int(-1)
  _lib.call("bt_device_count", ctypes.byref(n))
  assert n.value >= 0
  with pytest.raises(ValueError, match="bfp8"): _lib.call("bt_pack_bfp", 0, 3, 256, 512, 1, 0)
  with pytest.raises(ValueError, match="1 to 32 rows"): _lib.call("bt_gemv_bfp", 0, 8, 0, 40, 64, 64, 256, 256, 0, 0, 1.0, 256, 0, 0, 0, 0, 256, 1 << 30, 0)
  with pytest.raises(ValueError, match="multiples of 32"): _lib.call("bt_gemv_bfp", 0, 8, 0, 8, 60, 64, 256, 256, 0, 0, 1.0, 256, 0, 0, 0, 0, 256, 1 << 30, 0)
  with pytest.raises(ValueError, match="GLU"): _lib.call("bt_gemv_bfp", 0, 8, 3, 8, 64, 64, 256, 256, 0, 0, 1.0, 256, 0, 0, 0, 0, 256, 1 << 30, 0)
  op = _lib.GemvOp(fmt=8, epilogue=0, M=8, K=64, N=60, out_dtype=0, alpha=1.0, x=256, w=256, out=256)
  with pytest.raises(ValueError, match="matmul 0: K and N"): _lib.call("bt_gemv_queue", 0, 1, ctypes.byref(op), 256, 1 << 30, 0)
  with pytest.raises(ValueError, match="at least one"): _lib.call("bt_gemv_queue", 0, 0, ctypes.byref(op), 256, 1 << 30, 0)
  assert b"at least one" in _lib.lib().bt_last_error()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
  from baretile_b200 import _lib
  monkeypatch.setattr(_lib, "_lib", None)
  monkeypatch.setattr(_lib, "PATH", tmp_path / "libbaretile_b200.so")
  with pytest.raises(RuntimeError, match="no CPU fallback"): _lib.lib()


def test_tensor_checks_without_a_device():
  # bad calls raise ValueError before any allocation, also under python -O (reference: test/test_kernels.py:370-389)
  code = """
from baretile_b200.tensor import Tensor
class Runtime:
  def check(self): pass
  def dram_alloc(self, size): return 0
  def dram_free(self, addr): pass
rt = Runtime()
x, y = Tensor(rt, 2, 3), Tensor(rt, 2, 3)
for bad in (lambda: x @ y, lambda: x + Tensor(rt, 3, 2), lambda: Tensor.frombytes(rt, 1, 1, bytes(2), dtype="bfp8"),
            lambda: Tensor(rt, 0, 1), lambda: Tensor(rt, 1, 1, dtype="float64"), lambda: Tensor.of(rt, [[1, 2], [3]]),
            lambda: x.cast("int32") @ y, lambda: x.columns(), lambda: x.topk(1)):
  try: bad()
  except ValueError: continue
  raise SystemExit("no ValueError")
print("all raised")
"""
  run = subprocess.run([sys.executable, "-O", "-c", code], capture_output=True, text=True, timeout=120, cwd=ROOT)
  assert run.returncode == 0 and run.stdout.strip() == "all raised", run.stdout + run.stderr


def test_hole_allocator_merges():
  from baretile_b200.runtime import _merge_holes
  holes = [(512, 256), (0, 256), (256, 256), (2048, 64)]
  _merge_holes(holes)
  assert holes == [(0, 768), (2048, 64)]


def test_queue_plan_follows_the_addresses(built):
  # which earlier matmul each one of a queue waits for: worked out on the host from the buffers, no device needed
  from baretile_b200 import _lib
  def op(x, out, m=8, k=512, n=1024, add=0, fmt=8, epilogue=0):
    return _lib.GemvOp(fmt=fmt, epilogue=epilogue, M=m, K=k, N=n, out_dtype=0, alpha=1.0, x=x, w=0x100000, w2=0x200000 if epilogue == 3 else 0, add=add, out=out)
  def plan(ops):
    arr, waits = (_lib.GemvOp * len(ops))(*ops), (ctypes.c_int * len(ops))()
    _lib.call("bt_gemv_queue_plan", len(ops), arr, waits)
    return list(waits)
  A, B, C, D, E = (0x1000000 * i for i in range(1, 6))
  # a chain: every matmul reads the one before it
  assert plan([op(A, B), op(B, C, k=1024), op(C, D, k=1024), op(D, E, k=1024)]) == [-1, 0, 1, 2]
  # independent matmuls: only the limit of two in flight holds them back
  assert plan([op(A, B), op(A, C), op(A, D), op(A, E)]) == [-1, -1, 0, 1]
  # the addend is read too; a result buffer is not overwritten while an earlier matmul may still read or write it
  assert plan([op(A, B), op(A, C, add=B)]) == [-1, 0]
  assert plan([op(A, B), op(C, A)]) == [-1, 0]                       # writes what the first one reads
  assert plan([op(A, B), op(C, B)]) == [-1, 0]                       # writes what the first one writes
  assert plan([op(A, B), op(A + 512 * 64, C, k=32)]) == [-1, -1]      # reads A's tiles past the first one's 16: no overlap with B
  assert plan([op(A, B), op(B + 2048 * 31, C, k=32)]) == [-1, 0]      # the last tile of B
  assert plan([op(A, B), op(B + 2048 * 32, C, k=32)]) == [-1, -1]     # just past B
  # a list longer than one launch: the 33rd matmul starts a new launch and waits for all of the first
  many = [op(A, B + 0x10000 * i) for i in range(34)]
  waits = plan(many)
  assert waits[:3] == [-1, -1, 0] and waits[31] == 29 and waits[32] == -1 and waits[33] == -1
  with pytest.raises(ValueError, match="matmul 1: takes 1 to 32 rows"): plan([op(A, B), op(A, C, m=33)])


def test_queue_collects_matmuls_and_flushes_in_order(monkeypatch):
  # host logic of Runtime.queue(): matmuls are collected, anything else that needs the stream sends them first, the
  # block's end sends the rest; the C-ABI calls are captured instead of made, so no device is needed
  from baretile_b200 import _lib, runtime
  calls = []
  def fake_call(name, *args):
    if name == "bt_gemv_queue":
      n, arr = args[1], args[2]
      calls.append((name, [(arr[i].fmt, arr[i].epilogue, arr[i].M, arr[i].K, arr[i].N, arr[i].x, arr[i].w, arr[i].w2, arr[i].add, arr[i].out, arr[i].out_dtype,
                            arr[i].arg_val, arr[i].arg_idx, arr[i].arg_base, round(arr[i].alpha, 3)) for i in range(n)]))
    else: calls.append((name, args))
  monkeypatch.setattr(_lib, "call", fake_call)
  rt = runtime.Runtime.__new__(runtime.Runtime)
  rt.active, rt.device, rt.stream, rt.launches, rt.sent, rt.log, rt.pending, rt.timing, rt.work, rt.work_bytes = True, 0, 7, 0, {}, None, None, False, 4096, 1 << 20
  rt.sides, rt.unjoined, rt.side = [], [], None
  def matmul(x, out, epilogue=0, w2=0, alpha=1.0):
    rt.launch("bt_gemv_bfp", (8, epilogue, 4, 512, 1024, x, 0x1000, w2, 0, ctypes.c_float(alpha), out, 0, 0, 0, 0, rt.work, rt.work_bytes), name="matmul")
  matmul(0x10, 0x20)                                                  # outside a queue: sent at once
  assert [c[0] for c in calls] == ["bt_gemv_bfp"]
  calls.clear()
  with rt.queue():
    matmul(0x10, 0x20)
    matmul(0x20, 0x30, epilogue=3, w2=0x2000, alpha=0.5)
    assert calls == []                                               # nothing has left yet
    rt.launch("bt_untilize", (2, 0x30, 0x40, 1, 4, 1024), name="readback")
    matmul(0x40, 0x50)
  assert [c[0] for c in calls] == ["bt_gemv_queue", "bt_untilize", "bt_gemv_queue"]
  assert calls[0][1] == [(8, 0, 4, 512, 1024, 0x10, 0x1000, 0, 0, 0x20, 0, 0, 0, 0, 1.0), (8, 3, 4, 512, 1024, 0x20, 0x1000, 0x2000, 0, 0x30, 0, 0, 0, 0, 0.5)]
  assert len(calls[2][1]) == 1 and calls[2][1][0][5] == 0x40
  assert rt.launches == 5 and rt.pending is None
  calls.clear()
  with pytest.raises(KeyError):
    with rt.queue():
      matmul(0x10, 0x20)
      raise KeyError("the block fails")
  assert calls == [] and rt.pending is None                          # a failed block sends nothing


def test_beside_blocks_fork_from_the_stream_and_join_it_again(monkeypatch):
  # host logic of Runtime.beside(): a block's copies go to a stream of its own that starts behind what the runtime has
  # queued; the runtime's later launches do not wait for it until join(); the C-ABI calls are captured, no device needed
  from baretile_b200 import _lib, runtime
  calls, made = [], iter(range(100, 200))
  def fake_call(name, *args):
    if name in ("bt_stream_create", "bt_event_create"): args[-1]._obj.value = next(made)
    calls.append((name, args))
  monkeypatch.setattr(_lib, "call", fake_call)
  rt = runtime.Runtime.__new__(runtime.Runtime)
  rt.active, rt.device, rt.stream, rt.launches, rt.sent, rt.log, rt.pending, rt.timing, rt.work, rt.work_bytes = True, 0, 7, 0, {}, None, None, False, 4096, 1 << 20
  rt.sides, rt.unjoined, rt.side, rt.recording = [], [], None, None
  buf = (ctypes.c_char * 64)()
  with rt.beside(): rt.upload_async(0x1000, buf)
  with rt.beside(): rt.download_async(buf, 0x2000)
  rt.launch("bt_untilize", (2, 0x30, 0x40, 1, 4, 1024), name="readback")
  (s1, f1, d1), (s2, f2, d2) = rt.sides
  assert len({7, s1, s2}) == 3 and rt.stream == 7 and rt.unjoined == [d1, d2]
  order = [(n, a) for n, a in calls if n not in ("bt_stream_create", "bt_event_create")]
  assert [n for n, _ in order] == ["bt_event_record", "bt_stream_wait_event", "bt_h2d", "bt_event_record",
                                   "bt_event_record", "bt_stream_wait_event", "bt_d2h", "bt_event_record", "bt_untilize"]
  assert order[0][1] == (0, f1, 7) and order[1][1] == (0, s1, f1) and order[2][1][-1] == s1 and order[3][1] == (0, d1, s1)
  assert order[4][1] == (0, f2, 7) and order[5][1] == (0, s2, f2) and order[6][1][-1] == s2 and order[7][1] == (0, d2, s2)
  assert order[8][1][-1] == 7                                         # the runtime's own launch did not wait for either
  calls.clear()
  rt.join()
  assert calls == [("bt_stream_wait_event", (0, 7, d1)), ("bt_stream_wait_event", (0, 7, d2))] and rt.unjoined == []
  with pytest.raises(RuntimeError, match="own stream"):
    with rt.beside(): rt.launch("bt_gemv_bfp", (8, 0, 4, 512, 1024, 0x10, 0x1000, 0, 0, ctypes.c_float(1.0), 0x20, 0, 0, 0, 0, rt.work, rt.work_bytes))
  assert rt.stream == 7 and rt.side is None                           # the failed block gave the stream back
  rt.join()
  calls.clear()
  with rt.beside():
    with pytest.raises(RuntimeError, match="already open"):
      with rt.beside(): pass
    with pytest.raises(RuntimeError, match="inside a beside block"): rt.join()


def test_newer_entry_points_refuse_bad_arguments_before_any_device_work(built):
  """Argument checks come first in every entry point: they raise ValueError on a box without a GPU too."""
  import ctypes
  from baretile_b200 import _lib
  f = ctypes.c_float(1.0)
  # prefill matmul: K in whole tiles, w2 only with the gate/up epilogue, an addend of 1 or M rows
  with pytest.raises(ValueError, match="multiple of 32"): _lib.call("bt_gemm_bfp", 0, 8, 0, 64, 40, 64, 256, 256, 0, 0, 0, f, 256, 0, 256, 0)
  with pytest.raises(ValueError, match="w2 goes with"): _lib.call("bt_gemm_bfp", 0, 8, 0, 64, 64, 64, 256, 256, 256, 0, 0, f, 256, 0, 256, 0)
  with pytest.raises(ValueError, match="1 or M rows"): _lib.call("bt_gemm_bfp", 0, 8, 0, 64, 64, 64, 256, 256, 0, 256, 7, f, 256, 0, 256, 0)
  # put: formats, distinct aligned tensors
  with pytest.raises(ValueError, match="unknown format"): _lib.call("bt_put", 0, 3, 256, 512, 768, 1, 1, 32, 32, 0, 0)
  with pytest.raises(ValueError, match="apart from dst"): _lib.call("bt_put", 0, 8, 256, 256, 768, 1, 1, 32, 32, 0, 0)
  # the streaming layout: one launch takes up to 65535 runs of 4 tile columns; and an event to wait for must exist
  with pytest.raises(ValueError, match="tile columns in one launch"): _lib.call("bt_relayout", 0, 8, 1, 1, 4 * 65535 + 1, 256, 512, 0)
  with pytest.raises(ValueError, match="null event"): _lib.call("bt_stream_wait_event", 0, 0, 0)
  # many small matrices: a table is needed
  with pytest.raises(ValueError, match="no matrices"): _lib.call("bt_tilize_many", 0, 2, 0, None, None, None, None, 0)
  with pytest.raises(ValueError, match="itemsize"): _lib.call("bt_untilize_many", 0, 3, 1, None, None, None, None, 0)
  # the exchange over peer memory: ranks of one box, one tile row of whole tiles, steps from 1
  peers = (ctypes.c_uint64 * 2)(256, 512)
  with pytest.raises(ValueError, match="rank"): _lib.call("bt_peer_allreduce_round", 0, 2, 2, peers, 0, 1, 4, 64, 256, 0)
  with pytest.raises(ValueError, match="step"): _lib.call("bt_peer_allreduce_round", 0, 0, 2, peers, 0, 0, 4, 64, 256, 0)
  with pytest.raises(ValueError, match="rows at offset"): _lib.call("bt_peer_allreduce_round", 0, 0, 2, peers, 0, 1, 33, 64, 256, 0)
  with pytest.raises(ValueError, match="up to 8 ranks"): _lib.call("bt_peer_open", 0, 1, 0, 9, 1024, peers, 0)
  with pytest.raises(ValueError, match="rows at offset"): _lib.call("bt_peer_argmax_combine", 0, 0, 2, peers, 0, 1, 40, 256, 256, 512, 0)
