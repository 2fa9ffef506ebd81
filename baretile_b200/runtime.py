"""Queue work on a device: the CUDA stand-in for the reference's Runtime (baretile/runtime.py:543-923).

The reference's Runtime owns a rectangle of workers, a command ring in host memory, a DRAM hole allocator with
deferred frees, and per-launch timing records. Here one CUDA stream plays the ring (launches run in order,
asynchronously; `wait` blocks), device memory comes from arenas carved by the same first-fit hole allocator
(64-byte granularity there, 256 here), and timing records are CUDA events. Frees need no deferral: every access
to device memory is queued on the runtime's stream, so memory released now is reused only by work queued later.
"""
import collections, ctypes, time
from baretile_b200 import _lib

ALIGN = 256            # allocation granularity in bytes
ARENA = 1 << 30        # device memory is taken from the driver in pieces of at least this size
TIMES = 1024           # launches whose timing records are kept (baretile/runtime.py: TIMES)


class Bound(int):
  """A launch argument that a replay can replace, such as the address of a jit input; key names it in a binding
  (baretile/runtime.py:476-482). Adding a byte offset keeps it bound: a replay then points that far into the new
  allocation."""
  def __new__(cls, value, key, offset=0):
    self = super().__new__(cls, value)
    self.key, self.offset = key, offset
    return self
  def __add__(self, other):
    if isinstance(other, int) and not isinstance(other, Bound): return Bound(int(self) + other, self.key, self.offset + other)
    return int(self) + int(other)
  __radd__ = __add__
  def rebind(self, binding):
    """The argument's value under `binding` (key -> address); its recorded value when the key is missing."""
    return binding[self.key] + self.offset if self.key in binding else int(self)


def _merge_holes(holes, starts=()):
  """Join adjacent holes, but never across the start of an arena: two arenas that happen to be neighbours in the
  address space are separate allocations of the driver, and one copy or tensor must not span both."""
  holes.sort()
  merged = []
  for addr, room in holes:
    if merged and merged[-1][0] + merged[-1][1] == addr and addr not in starts: merged[-1] = (merged[-1][0], merged[-1][1] + room)
    else: merged.append((addr, room))
  holes[:] = merged


class Recording:
  """Launches recorded once and replayed with one call: the reference's Recording / tensor.jit
  (baretile/tensor.py:1171-1293), which replays a block of commands with one doorbell write. Here the block is a
  CUDA graph, and matmuls that follow one another in it become one queue launch (see Runtime.queue). Recorded
  launches keep their addresses, so the tensors they use must stay alive. Memory that is released while recording
  (a temporary of a launch: staging for an upload, the flat scratch of a pick) is used by every replay, so the
  recording keeps it out of the allocator until close().

      with rt.record() as step: y = (x @ w).relu().realize()      # runs once, like any launches
      step.replay()                                                # and again
  """
  def __init__(self, rt): self.rt, self.graph, self.count, self.held, self.launches = rt, None, 0, [], None
  def __enter__(self):
    self.rt.check()
    if self.rt.recording is not None: raise RuntimeError("a recording is already in progress on this runtime")
    self.rt.flush()
    self.rt.join()
    self.rt._sides(SIDES)                                   # streams and events are made before the capture starts
    self.first = self.rt.launches
    _lib.call("bt_graph_begin", self.rt.device, self.rt.stream)
    self.outer, self.rt.pending = self.rt.pending, []
    self.rt.recording = self
    self.outer_log, self.rt.log = self.rt.log, []          # what is launched meanwhile, for replays with a binding
    return self
  def __exit__(self, kind, *_):
    graph = ctypes.c_uint64()
    try:
      try:
        if kind is None: self.rt.flush()
      finally:
        try: self.rt.join()                                  # every branch comes back to the stream before the capture ends
        except Exception:
          if kind is None: raise
        self.launches, self.rt.log = self.rt.log, self.outer_log
        if self.outer_log is not None: self.outer_log.extend(self.launches)
        self.rt.pending, self.rt.recording = self.outer, None
        _lib.call("bt_graph_end", self.rt.device, self.rt.stream, ctypes.byref(graph))
    except Exception:
      if kind is None: raise
      return
    self.graph, self.count = graph.value, self.rt.launches - self.first
    # what was recorded also runs once, as it would have without the recording (the reference's Recording logs launches
    # that execute as usual): the results exist when the block ends
    _lib.call("bt_graph_launch", self.rt.device, self.graph, self.rt.stream)
  def replay(self, binding=None):
    """Queue the recorded launches again. Without a binding they replay as recorded, with one call. `binding` maps
    a Bound argument's key to its value for this replay (an argument whose key is missing keeps its recorded value,
    baretile/tensor.py:1194-1214): the launches are then queued again one by one with the new values, the matmuls
    among them still leaving as one queue launch."""
    self.rt.check()
    if self.graph is None: raise RuntimeError("nothing was recorded")
    if self.rt.recording is not None: raise RuntimeError("cannot replay while recording on the same runtime")
    if not binding:
      _lib.call("bt_graph_launch", self.rt.device, self.graph, self.rt.stream)
      self.rt.launches += self.count
      return
    with self.rt.queue():
      for kernel, args, units, name in self.launches:
        self.rt.launch(kernel, tuple(a.rebind(binding) if isinstance(a, Bound) else a for a in args), units, name)
  send = replay                          # the reference's name for it
  def close(self):
    """Drop the recording and hand the memory it kept back to the allocator."""
    if self.graph is not None and self.rt.active: _lib.lib().bt_graph_destroy(self.rt.device, self.graph)
    self.graph = None
    held, self.held = self.held, []
    for addr, size in held:
      if self.rt.active:
        self.rt.holes.append((addr, size))
        _merge_holes(self.rt.holes, {a for a, _ in self.rt.arenas})


class Queue:
  """Inside `with rt.queue():` matmuls of up to 32 rows are collected instead of launched, and go out together as
  one bt_gemv_queue launch when the block ends or when anything else needs the stream (another kind of launch, a
  copy, wait). The kernel runs them in order and keeps streaming weights across the boundaries between them, which
  is what a chain of dependent decode matmuls needs. The reference queues commands in a ring that its dispatcher
  drains without the host (baretile/runtime.py:734-771); this is the same idea for the path's matmuls."""
  def __init__(self, rt): self.rt = rt
  def __enter__(self):
    self.rt.check()
    self.outer = self.rt.pending
    if self.outer is None: self.rt.pending = []
    return self
  def __exit__(self, kind, *_):
    try:
      if kind is None: self.rt.flush()
    finally:
      if self.outer is None: self.rt.pending = None


SIDES = 4   # streams a runtime keeps for work that runs beside its own


class Beside:
  """Inside `with rt.beside():` copies (and layout launches) are queued on a stream of their own: they start once
  everything queued on the runtime before the block is done, and run BESIDE what the runtime queues after the block,
  until the runtime joins them again: at the next wait(), at the end of a recording, or at join(). Each block gets a
  stream of its own, so two blocks also run beside one another. This is how the copies of a step's inputs and of the
  previous step's results cross the bus while the current step computes (the reference's host DMA likewise runs while
  its dispatcher drains the command ring, baretile/runtime.py:734-771). Matmuls stay on the runtime's own stream: they
  share its scratch.

      with rt.record() as step:
        with rt.beside(): rt.upload_async(next_in, host_in)        # the next step's inputs
        with rt.beside(): rt.download_async(host_out, last_out)    # the last step's results
        ...                                                        # this step's launches
  """
  def __init__(self, rt): self.rt = rt
  def __enter__(self):
    rt = self.rt
    rt.check()
    if rt.side is not None: raise RuntimeError("a beside block is already open on this runtime")
    rt.flush()
    if len(rt.unjoined) >= SIDES: raise RuntimeError(f"at most {SIDES} beside blocks between two joins")
    stream, fork, done = rt._sides(len(rt.unjoined) + 1)[len(rt.unjoined)]
    _lib.call("bt_event_record", rt.device, fork, rt.stream)
    _lib.call("bt_stream_wait_event", rt.device, stream, fork)
    self.done, rt.side, rt.stream = done, rt.stream, stream
    return self
  def __exit__(self, *_):
    rt = self.rt
    stream, rt.stream, rt.side = rt.stream, rt.side, None
    _lib.call("bt_event_record", rt.device, self.done, stream)
    rt.unjoined.append(self.done)


class Runtime:
  """Run kernels on one CUDA device, in order. A new Runtime on a chip closes the chip's older runtime, as an
  overlapping rectangle does in the reference (baretile/runtime.py:593-598). Close a runtime to release its
  memory; a closed runtime cannot be reused."""
  def __init__(self, chip, start=None, end=None, ring=1 << 20, timing=False):
    if ring < 64 or ring & (ring - 1): raise ValueError("ring size must be a power of two, at least 64 bytes")
    self.chip, self.device, self.launches = chip, chip.device, 0
    self.cores = list(chip.tensix)
    self.grid = (list(range(len(self.cores))), [0])
    self.start, self.end = start or self.cores[0], end or self.cores[-1]
    self.active, self.timing = False, timing
    self.holes, self.used, self.arenas = [], {}, []
    self.sent = {}                                   # launch number % TIMES -> (name, start event, end event)
    self.numbers = {}                                # 1 x 1 tensors of Python numbers, made once
    self.log = None
    self.pending = None      # matmuls collected for one queue launch (a list while queueing)
    self.recording = None    # the Recording in progress, which keeps what is freed meanwhile
    self.sides, self.unjoined, self.side = [], [], None   # (stream, fork event, done event) of beside blocks; their done events not yet joined; the own stream while a block is open
    self.stream = ctypes.c_uint64()
    for other in list(chip.taken.values()): other.close()
    _lib.call("bt_stream_create", self.device, ctypes.byref(self.stream))
    self.stream = self.stream.value
    self.active = True
    chip.taken[id(self)] = self
    try:
      size = ctypes.c_size_t()
      _lib.call("bt_gemv_workspace_bytes", self.device, ctypes.byref(size))
      self.work_bytes = size.value
      self.work = self.dram_alloc(self.work_bytes)
      _lib.call("bt_memset", self.device, self.work, 0, self.work_bytes, self.stream)
      self.flag = self.host_alloc(4)     # page-locked: wait() has the scratch's error word copied here ahead of its one sync
    except BaseException:
      self.close()
      raise

  # ---- lifetime ----
  def check(self):
    """Reject work after explicit shutdown or takeover by another runtime (baretile/runtime.py:645-647)."""
    if not self.active: raise RuntimeError("runtime is closed or was replaced by an overlapping runtime")

  def close(self):
    """Finish queued work and release the device memory. Closing twice is harmless (baretile/runtime.py:649-653)."""
    if not self.active: return
    self.active = False
    try: _lib.call("bt_stream_sync", self.device, self.stream, 2000)
    except (TimeoutError, RuntimeError): pass
    for _, start, end in self.sent.values():
      for e in (start, end):
        if e: _lib.lib().bt_event_destroy(self.device, e)
    self.sent.clear()
    if self.side is not None: self.stream, self.side = self.side, None
    for stream, fork, done in self.sides:
      try: _lib.call("bt_stream_sync", self.device, stream, 2000)
      except (TimeoutError, RuntimeError): pass
      _lib.lib().bt_stream_destroy(self.device, stream)
      for e in (fork, done): _lib.lib().bt_event_destroy(self.device, e)
    self.sides, self.unjoined = [], []
    for ptr in getattr(self, "pinned", []): _lib.lib().bt_host_free(ptr)
    self.pinned = []
    for addr, _ in self.arenas: _lib.lib().bt_free(self.device, addr)
    self.arenas, self.holes = [], []
    self.used.clear()
    _lib.lib().bt_stream_destroy(self.device, self.stream)
    self.chip.taken.pop(id(self), None)

  @property
  def closed(self): return not self.active
  def __enter__(self): self.check(); return self
  def __exit__(self, *_): self.close()
  def __del__(self):
    try: self.close()
    except Exception: pass

  # ---- launches ----
  def launch(self, kernel, args=(), units=None, name=""):
    """Queue a kernel: here `kernel` is the name of a C-ABI entry point and `args` its arguments after the device
    and before the stream (reference: a compiled kernel image and its words, baretile/runtime.py:680-697). `units`
    is accepted for parity; the entry point sizes its own grid."""
    self.check()
    if units is not None and not 1 <= int(units) < 2**32: raise ValueError("launch units must be in [1, 2**32 - 1]")
    if self.side is not None and kernel in ("bt_gemv_bfp", "bt_gemv_queue", "bt_gemm_bfp"):
      raise RuntimeError("a matmul uses the runtime's scratch and runs on its own stream, not in a beside block")
    if self.log is not None: self.log.append((kernel, args, units, name))
    if self.pending is not None and kernel == "bt_gemv_bfp":
      self.pending.append(args)
      self._count(name or kernel, 0, 0)
      return
    self.flush()
    start = end = 0
    if self.timing:
      start, end = ctypes.c_uint64(), ctypes.c_uint64()
      _lib.call("bt_event_create", self.device, ctypes.byref(start))
      _lib.call("bt_event_create", self.device, ctypes.byref(end))
      start, end = start.value, end.value
      _lib.call("bt_event_record", self.device, start, self.stream)
    _lib.call(kernel, self.device, *args, self.stream)
    if self.timing: _lib.call("bt_event_record", self.device, end, self.stream)
    self._count(name or kernel, start, end)

  def _count(self, name, start, end):
    self.launches += 1
    old = self.sent.pop(self.launches % TIMES, None)
    if old:
      for e in old[1:]:
        if e: _lib.lib().bt_event_destroy(self.device, e)
    self.sent[self.launches % TIMES] = (name, start, end)

  def queue(self): return Queue(self)

  def beside(self): return Beside(self)

  def _sides(self, n):
    """At least n streams for beside blocks, each with the two events that fork it from and join it to the own stream."""
    while len(self.sides) < n:
      made = [ctypes.c_uint64() for _ in range(3)]
      _lib.call("bt_stream_create", self.device, ctypes.byref(made[0]))
      for e in made[1:]: _lib.call("bt_event_create", self.device, ctypes.byref(e))
      self.sides.append(tuple(m.value for m in made))
    return self.sides

  def join(self):
    """What is queued from here on runs after the work of every beside block so far."""
    if self.side is not None: raise RuntimeError("join inside a beside block")
    done, self.unjoined = self.unjoined, []
    for e in done: _lib.call("bt_stream_wait_event", self.device, self.stream, e)

  def flush(self):
    """Send the matmuls collected so far as one queue launch."""
    if not self.pending: return
    ops, self.pending = self.pending, []
    arr = (_lib.GemvOp * len(ops))()
    for o, (fmt, epi, m, k, n, x, w, w2, add, alpha, out, out_dtype, arg_val, arg_idx, arg_base, _work, _bytes) in zip(arr, ops):
      o.fmt, o.epilogue, o.M, o.K, o.N, o.out_dtype, o.arg_base, o.alpha = fmt, epi, m, k, n, out_dtype, arg_base, getattr(alpha, "value", alpha)
      o.x, o.w, o.w2, o.add, o.out, o.arg_val, o.arg_idx = x, w, w2, add, out, arg_val, arg_idx
    _lib.call("bt_gemv_queue", self.device, len(ops), arr, self.work, self.work_bytes, self.stream)

  def wait(self, timeout=60, launch=None):
    """Block until the queued launches are done (baretile/runtime.py:858-880). On timeout raise TimeoutError; the
    runtime stays usable. Also raises RuntimeError if a kernel reported that one of its bounded waits gave up."""
    self.check()
    if launch is not None and launch > self.launches:
      raise ValueError(f"launch {launch} was never queued; the last one queued is {self.launches}")
    self.flush()
    self.join()
    # the word a wait that gave up sets is the first of the scratch: its copy is queued behind the work and arrives with
    # the one synchronisation (a separate check afterwards costs a second round trip on every wait)
    _lib.call("bt_d2h", self.device, ctypes.addressof(self.flag), self.work, 4, self.stream)
    _lib.call("bt_stream_sync", self.device, self.stream, int(timeout * 1000))
    if int.from_bytes(self.flag.raw, "little", signed=True):
      error = ctypes.c_int()
      _lib.call("bt_gemv_check", self.device, self.work, self.stream, ctypes.byref(error))     # reads it again and resets the counters
      raise RuntimeError(f"a matmul launch gave up on a bounded wait (code {error.value}); its results are unreliable")

  def finished(self):
    done = ctypes.c_int()
    _lib.call("bt_stream_query", self.device, self.stream, ctypes.byref(done))
    return self.launches if done.value else max(self.launches - 1, 0)

  def profile(self, since):
    """Wait, then [(name, launches, microseconds, None)] for the launches after `since`, grouped by name, longest
    first (baretile/runtime.py:773-786 returns cycles and NoC bytes). Times need Runtime(timing=True)."""
    self.wait()
    if self.launches - since > TIMES: raise ValueError(f"{self.launches - since} launches to profile, but only the last {TIMES} are kept")
    totals = collections.defaultdict(lambda: [0, 0.0])
    for n in range(since + 1, self.launches + 1):
      if n % TIMES not in self.sent: continue   # a replayed launch has no record of its own
      name, start, end = self.sent[n % TIMES]
      ms = ctypes.c_float()
      if start: _lib.call("bt_event_elapsed_ms", self.device, start, end, ctypes.byref(ms))
      totals[name][0] += 1
      totals[name][1] += ms.value * 1e3
    return sorted(((name, n, us if self.timing else None, None) for name, (n, us) in totals.items()), key=lambda r: -(r[2] or 0))

  # ---- device memory ----
  def dram_alloc(self, size):
    """First free hole that is big enough (baretile/runtime.py:791-812); a new arena from the driver when none is."""
    self.check()
    size = max(ALIGN, -(-size // ALIGN) * ALIGN)
    for attempt in range(2):
      for i, (addr, room) in enumerate(self.holes):
        if room >= size:
          self.holes[i:i + 1] = [(addr + size, room - size)] if room > size else []
          self.used[addr] = size
          return addr
      if attempt: break
      arena, addr = max(size, ARENA), ctypes.c_uint64()
      try: _lib.call("bt_malloc", self.device, arena, ctypes.byref(addr))
      except MemoryError: raise MemoryError(f"no {size} bytes free in DRAM") from None
      self.arenas.append((addr.value, arena))
      self.holes.append((addr.value, arena))
    raise MemoryError(f"no {size} bytes free in DRAM")

  def dram_free(self, addr):
    """Release an allocation (baretile/runtime.py:814-820). Work already queued may still use it; work queued
    later may reuse it, which the stream's ordering makes safe."""
    if not self.active: return
    size = self.used.pop(addr, None)
    if size is None: return
    if self.recording is not None:   # a replay will use this memory again
      self.recording.held.append((addr, size))
      return
    self.holes.append((addr, size))
    _merge_holes(self.holes, {a for a, _ in self.arenas})

  def record(self): return Recording(self)

  # ---- host <-> device ----
  def host_alloc(self, size):
    """Page-locked host memory as a ctypes byte array: the reference's host DMA page (baretile/runtime.py:548-600).
    Copies from and to it are asynchronous."""
    ptr = ctypes.c_void_p()
    _lib.call("bt_host_alloc", size, ctypes.byref(ptr))
    buf = (ctypes.c_char * size).from_address(ptr.value)
    self.pinned = getattr(self, "pinned", [])
    self.pinned.append(ptr.value)
    return buf

  def upload_async(self, addr, buf, n=None):
    """Queue a copy from page-locked host memory to device memory; returns at once."""
    self.check()
    self.flush()
    _lib.call("bt_h2d", self.device, addr, ctypes.addressof(buf), len(buf) if n is None else n, self.stream)

  def download_async(self, buf, addr, n=None):
    """Queue a copy from device memory into page-locked host memory; wait() before reading it."""
    self.check()
    self.flush()
    _lib.call("bt_d2h", self.device, ctypes.addressof(buf), addr, len(buf) if n is None else n, self.stream)

  def layout_many(self, tilize, items, itemsize=2):
    """Queue ONE launch that brings many small matrices from row-major order into tile layout (tilize) or back:
    items = [(src address, dst address, rows, cols), ...]. For a decode step's inputs and results, where a launch per
    matrix costs more than the work (bt_tilize_many / bt_untilize_many)."""
    n = len(items)
    src, dst = (ctypes.c_uint64 * n)(*(int(i[0]) for i in items)), (ctypes.c_uint64 * n)(*(int(i[1]) for i in items))
    rows, cols = (ctypes.c_int * n)(*(i[2] for i in items)), (ctypes.c_int * n)(*(i[3] for i in items))
    self.launch("bt_tilize_many" if tilize else "bt_untilize_many", (itemsize, n, src, dst, rows, cols), name="upload" if tilize else "readback")

  def upload(self, addr, data):
    """Copy host bytes to device memory at addr, in order with the queued launches."""
    self.check()
    data = bytes(data) if not isinstance(data, (bytes, bytearray)) else data
    buf = (ctypes.c_char * len(data)).from_buffer_copy(data)
    self.flush()
    _lib.call("bt_h2d", self.device, addr, ctypes.cast(buf, ctypes.c_void_p), len(data), self.stream)
    _lib.call("bt_stream_sync", self.device, self.stream, -1)   # buf is pageable and short-lived

  def download(self, addr, n):
    """n bytes of device memory at addr, after the queued launches."""
    self.check()
    buf = ctypes.create_string_buffer(n)
    self.flush()
    _lib.call("bt_d2h", self.device, ctypes.cast(buf, ctypes.c_void_p), addr, n, self.stream)
    _lib.call("bt_stream_sync", self.device, self.stream, -1)
    return buf.raw
