"""Tensors on the B200 backend: the part of the reference's Tensor (baretile/tensor.py:25-1299) that the block-float
matmul path uses, with the same names, argument meaning and errors.

A Tensor is a batch of matrices in tile layout in device memory, or an unrealized expression. The expressions this
backend runs are the ones the path is made of:

    act(alpha * (x @ W) + addend)          act in {identity, relu, silu}
    (x @ Wg).silu() * (x @ Wu)             the gate/up pair of an MLP
    (x @ W).topk(1)                        greedy pick fused into the LM-head matmul

with x bf16 and W bfp8 or bfp4. `realize` turns one such expression into one kernel launch (the reference fuses the
same trees in kernels.fused_kernel, baretile/kernels.py:41-727). Anything else raises ValueError.
"""
import array, ctypes, math, operator
from baretile_b200 import _lib
from baretile_b200.tensix import BFP, FMT_CODE, ITEMSIZE, tile_bytes

DIMS = 5
FIDELITY = 4   # accepted for parity; products are always exact here (baretile/tensor.py:12)
EPILOGUE = {"none": 0, "relu": 1, "silu": 2, "glu": 3, "argmax": 4}


def _shape(shape):
  if not 1 <= len(shape) <= DIMS: raise ValueError(f"a tensor needs one to {DIMS} dimensions")
  shape = tuple(map(operator.index, shape))
  if any(n <= 0 for n in shape): raise ValueError(f"tensor dimensions must be positive: {shape}")
  return (1,) * (3 - len(shape)) + shape


class Tensor:
  """A batch of matrices, shape (batch, rows, cols), stored as 32 x 32 tiles in row order with matrices one after
  another; partial tiles pad with zeros and a dimension of size 1 repeats across its tile (baretile/tensor.py:26-36).
  Formats: bf16, fp32, int32, bfp8, bfp4."""
  def __init__(self, rt, rows, cols, op=None, srcs=(), batch=1, dtype="bf16"):
    self.addr = None
    batch, rows, cols = _shape((batch, rows, cols))
    if dtype not in (*ITEMSIZE, *BFP): raise ValueError(f"unknown tensor dtype: {dtype}")
    if any(s.rt is not rt for s in srcs if isinstance(s, Tensor)): raise ValueError("tensor operands must use the same runtime")
    rt.check()
    self.rt, self.rows, self.cols, self.batch, self.op, self.srcs, self.dtype = rt, rows, cols, batch, op, srcs, dtype
    self.lead = (batch,)
    self.tr, self.tc = -(-rows // 32), -(-cols // 32)
    self.tiles, self.owner, self.runs = batch * self.tr * self.tc, None, None
    self._stream = None          # this block-float matrix in streaming layout, made on first use as a matmul's B
    self.addr = None if op else self._alloc()

  def _alloc(self): return self.rt.dram_alloc(self.tiles * tile_bytes(self.dtype))
  def __del__(self):
    if getattr(self, "addr", None) is not None and self.owner is None:
      try: self.rt.dram_free(self.addr)
      except Exception: pass

  @property
  def shape(self): return (*self.lead, self.rows, self.cols)
  def _same_runtime(self, *xs):
    if any(x.rt is not self.rt for x in xs): raise ValueError("tensor operands must use the same runtime")

  # ---- construction ----
  @classmethod
  def full(cls, rt, rows, cols, value, dtype="bf16"): return cls.of(rt, [[value] * cols for _ in range(rows)], dtype)

  @classmethod
  def zeros(cls, rt, rows, cols, batch=1, dtype="bf16"):
    """Zeros in any storage format, block floats included: all-zero bytes are zeros in each (test/test_kernels.py:351-368)."""
    t = cls(rt, rows, cols, batch=batch, dtype=dtype)
    rt.launch("bt_memset", (t.addr, 0, t.tiles * tile_bytes(dtype)), name="zeros")
    return t

  @classmethod
  def of(cls, rt, data, dtype="bf16"):
    """From rows of numbers, or a list of those for a batch. bf16 rounds to nearest even (baretile/tensor.py:88-104)."""
    if not len(data) or not len(data[0]): raise ValueError("tensor data must be nonempty")
    matrices = data if isinstance(data[0][0], (list, tuple)) else [data]
    if matrices and isinstance(matrices[0][0], (list, tuple)) and len(matrices[0][0]) and isinstance(matrices[0][0][0], (list, tuple)):
      raise ValueError("this backend takes at most three dimensions")
    rows, cols = len(matrices[0]), len(matrices[0][0])
    if not cols or any(len(m) != rows or any(len(row) != cols for row in m) for m in matrices):
      raise ValueError("tensor data must be nonempty rectangular matrices of the same shape")
    values = array.array("i" if dtype == "int32" else "f", [v for m in matrices for row in m for v in row])
    return cls.frombytes(rt, rows, cols, values, len(matrices), dtype, _round=dtype == "bf16")

  @classmethod
  def frombytes(cls, rt, rows, cols, data, batch=1, dtype="bf16", _round=False):
    """Upload little-endian values in row-major order, matrices one after another, and convert to tile layout on
    the device (baretile/tensor.py:107-135). Block floats are not uploaded: upload bf16, then cast."""
    if dtype in BFP: raise ValueError("upload as bf16, then cast on the chip to a block-float format")
    if dtype not in ITEMSIZE: raise ValueError(f"unknown tensor dtype: {dtype}")
    batch, rows, cols = _shape((batch, rows, cols))
    n, data = ITEMSIZE[dtype], memoryview(data).cast("B")
    count = batch * rows * cols
    if len(data) != (4 if _round else n) * count: raise ValueError(f"{len(data)} bytes for {batch} x {rows} x {cols} of {dtype}")
    t = cls(rt, rows, cols, batch=batch, dtype=dtype)
    stage = rt.dram_alloc(len(data) + (2 * count if _round else 0))
    try:
      rt.upload(stage, data)
      src = stage
      if _round:   # fp32 values to bf16 bits on the device, to nearest even
        src = stage + len(data)
        rt.launch("bt_round_bf16", (stage, src, count), name="round")
      rt.launch("bt_tilize", (n, src, t.addr, batch, rows, cols), name="upload")
    finally: rt.dram_free(stage)
    return t

  # ---- readback ----
  def tobytes(self):
    """Row-major bytes in the format frombytes accepts; block floats read back as their bf16 values
    (baretile/tensor.py:159-193)."""
    x = self.realize()
    rt, n = self.rt, 2 if self.dtype in BFP else ITEMSIZE[self.dtype]
    size = n * self.batch * self.rows * self.cols
    flat, held, tiles = rt.dram_alloc(size), [], x.addr
    try:
      if self.dtype in BFP:
        if x.runs:   # streamed layout back to tile order
          held.append(rt.dram_alloc(self.tiles * tile_bytes(self.dtype)))
          self._relayout(tiles, held[-1], to_stream=0)
          tiles = held[-1]
        held.append(rt.dram_alloc(self.tiles * 2048))
        rt.launch("bt_unpack_bfp", (FMT_CODE[self.dtype], tiles, held[-1], self.tiles), name="storage")
        tiles = held[-1]
      rt.launch("bt_untilize", (n, tiles, flat, self.batch, self.rows, self.cols), name="readback")
      return rt.download(flat, size)
    finally:
      for a in (flat, *held): rt.dram_free(a)

  def tolist(self):
    """Rows of numbers, or a list of them for a batch (baretile/tensor.py:195-204)."""
    raw = self.tobytes()
    if self.dtype == "bf16" or self.dtype in BFP:
      raw = array.array("I", [b << 16 for b in array.array("H", raw)]).tobytes()
    values = array.array("i" if self.dtype == "int32" else "f", raw).tolist()
    m = [[values[(b * self.rows + r) * self.cols:(b * self.rows + r + 1) * self.cols] for r in range(self.rows)]
         for b in range(self.batch)]
    return m if self.batch > 1 else m[0]

  def numpy(self):
    """The values as a NumPy float32 (or int32) array of this tensor's shape. A convenience for tests and models."""
    import numpy as np
    raw = self.tobytes()
    if self.dtype == "bf16" or self.dtype in BFP: a = (np.frombuffer(raw, np.uint16).astype(np.uint32) << 16).view(np.float32)
    else: a = np.frombuffer(raw, np.int32 if self.dtype == "int32" else np.float32)
    return a.reshape(self.shape if self.batch > 1 else (self.rows, self.cols))

  # ---- formats ----
  def _relayout(self, src, dst, to_stream):
    per = self.tr * self.tc * tile_bytes(self.dtype)
    for b in range(self.batch):
      self.rt.launch("bt_relayout", (FMT_CODE[self.dtype], to_stream, self.tr, self.tc, src + b * per, dst + b * per), name="columns")

  def cast(self, dtype):
    """Convert storage format (baretile/tensor.py:581-596). bf16 -> bfp8 / bfp4 packs each run of 16 values along a
    row around its largest exponent; a block float -> bf16 decodes exactly."""
    if dtype not in (*ITEMSIZE, *BFP): raise ValueError(f"unknown tensor dtype: {dtype}")
    if dtype == self.dtype and not self.runs: return self
    x = self.realize()
    if self.dtype in BFP:
      out, src, held = Tensor(self.rt, self.rows, self.cols, batch=self.batch), x.addr, None
      if x.runs:
        held = self.rt.dram_alloc(self.tiles * tile_bytes(self.dtype))
        self._relayout(src, held, to_stream=0)
        src = held
      self.rt.launch("bt_unpack_bfp", (FMT_CODE[self.dtype], src, out.addr, self.tiles), name="storage")
      if held is not None: self.rt.dram_free(held)
      return out.cast(dtype)
    if dtype in BFP:
      if self.dtype != "bf16": raise ValueError(f"a block float is cast from bf16, not {self.dtype}")
      out = Tensor(self.rt, self.rows, self.cols, batch=self.batch, dtype=dtype)
      self.rt.launch("bt_pack_bfp", (FMT_CODE[dtype], x.addr, out.addr, self.tiles), name=dtype)
      return out
    raise ValueError(f"this backend casts between bf16 and block floats, not {self.dtype} to {dtype}")

  def columns(self):
    """Store the matrix the way matmul streams its B (baretile/tensor.py:598-611). Here: runs of 4 tile columns,
    tile row by tile row, each tile's bytes ordered for the kernel's loads. A pure permutation; it reads back as
    it was."""
    if self.dtype not in BFP:
      raise ValueError(f"columns lays out a matmul's B, which is a block float on this backend, not {self.dtype}")
    if self.runs: return self
    x = self.realize()
    out = Tensor(self.rt, self.rows, self.cols, batch=self.batch, dtype=self.dtype)
    out.runs = (-(-self.tc // 4), self.tr, 0)
    self._relayout(x.addr, out.addr, to_stream=1)
    return out

  def put(self, ids, x):
    """Write x into the rows selected by ids, in place: how models update KV caches without changing the shape of a
    decode step (baretile/tensor.py:224-241). For a block-float destination x is bf16 and is rounded as in cast."""
    self._same_runtime(ids, x)
    if not (ids.dtype == "int32" and ids.shape[:2] == (1, 1) and ids.cols == x.rows):
      raise ValueError("put needs ids as an int32 row, with one position for each row of x")
    if not ((x.batch, x.cols) == (self.batch, self.cols) and x.dtype == ("bf16" if self.dtype in BFP else self.dtype)):
      raise ValueError(f"put needs rows of the cache's batch and width, "
                       f"bf16 for a block float: {x.shape} {x.dtype} into {self.shape} {self.dtype}")
    if self.runs: raise ValueError("put writes a tensor in tile order, not one laid out by columns")
    x, ids = x.realize(), ids.realize()
    if 2 * x.rows + self.tr > 2**17: raise ValueError("put has too many rows")   # the reference's bound, kept
    self.realize()
    self._stream = None                     # a copy by columns made earlier no longer matches
    held = []                               # x or ids that is the tensor itself is copied first, as the reference does
    def apart(t):
      if t.addr != self.addr: return t.addr
      size = t.tiles * tile_bytes(t.dtype)
      held.append(self.rt.dram_alloc(size))
      self.rt.launch("bt_d2d", (held[-1], t.addr, size), name="copy")
      return held[-1]
    try:
      scratch = 0
      if x.rows > 64:                       # beyond a few rows: one int per row of the tile rows, to find each place's last row in one pass
        held.append(self.rt.dram_alloc(4 * 32 * self.tr))
        scratch = held[-1]
      self.rt.launch("bt_put", (FMT_CODE[self.dtype], self.addr, apart(x), apart(ids), self.batch, x.rows, self.rows, self.cols, scratch), name="put")
    finally:
      for a in held: self.rt.dram_free(a)
    return self

  def float(self): return self.cast("fp32")
  def bfloat16(self): return self.cast("bf16")

  # ---- expressions ----
  def _node(self, op, srcs, rows=None, cols=None, dtype=None):
    return Tensor(self.rt, rows or self.rows, cols or self.cols, op, srcs, self.batch, dtype or self.dtype)
  def relu(self): return self._node("relu", (self,))
  def silu(self): return self._node("silu", (self,))
  def __mul__(self, x):
    if isinstance(x, (int, float)): return self._node("scale", (self, float(x)))
    self._same_runtime(x)
    if x.shape != self.shape: raise ValueError(f"cannot broadcast {self.shape} with {x.shape}")
    return self._node("mul", (self, x))
  __rmul__ = __mul__
  def __add__(self, x):
    if not isinstance(x, Tensor): raise ValueError("this backend adds tensors, not numbers")
    self._same_runtime(x)
    if x.cols != self.cols or x.rows not in (1, self.rows) or x.batch != self.batch: raise ValueError(f"cannot broadcast {self.shape} with {x.shape}")
    return self._node("add", (self, x))
  __radd__ = __add__

  def __matmul__(self, x): return self.matmul(x)
  def matmul(self, x, dtype=None, fidelity=None, index=None):
    """self @ x with fp32 accumulation (baretile/tensor.py:738-795). self is bf16, x is bfp8 or bfp4."""
    self._same_runtime(x)
    fidelity = FIDELITY if fidelity is None else operator.index(fidelity)
    if not 1 <= fidelity <= 4: raise ValueError("matmul fidelity must be between one and four phases")
    if index is not None: raise ValueError("matmul by index is not on this backend's path")
    if "int32" in (self.dtype, x.dtype): raise ValueError(f"matmul needs floats, since the FPU has no int32: {self.dtype} @ {x.dtype}")
    if not (self.cols == x.rows and self.batch == x.batch == 1):
      raise ValueError(f"matmul needs A's columns to match B's rows, and single matrices: {self.shape} @ {x.shape}")
    if self.dtype != "bf16" or x.dtype not in BFP:
      raise ValueError(f"this backend multiplies bf16 A by a block-float B, not {self.dtype} @ {x.dtype}")
    if dtype not in (None, "bf16", "fp32"): raise ValueError(f"matmul results are bf16 or fp32, not {dtype}")
    if self.cols == 1: raise ValueError(f"this backend's matmul needs more than one column of A: {self.shape} @ {x.shape}")
    return self._node("matmul", (self, x), cols=x.cols, dtype=dtype or "bf16")

  def topk(self, k, parts=1, labels=None):
    """(values, int32 indices) of the largest entry in each row; of equal values the first column wins
    (baretile/tensor.py:686-706). Here k is 1 and self is a matmul expression: the pick is fused into the kernel's
    epilogue and compares the fp32 accumulators."""
    if operator.index(k) != 1 or parts != 1 or labels is not None: raise ValueError("this backend's topk is the fused k = 1 pick")
    e = _linear(self)
    if e is None: raise ValueError("this backend's topk takes a matmul expression")
    values, ids = Tensor(self.rt, self.rows, 1, dtype="fp32"), Tensor(self.rt, self.rows, 1, dtype="int32")
    flat = self.rt.dram_alloc(512)
    try:
      _launch_matmul(self.rt, e, "argmax", None, self.rows, arg=(flat, flat + 256))
      self.rt.launch("bt_tilize", (4, flat, values.addr, 1, self.rows, 1), name="topk")
      self.rt.launch("bt_tilize", (4, flat + 256, ids.addr, 1, self.rows, 1), name="topk")
    finally: self.rt.dram_free(flat)
    return values, ids

  def realize(self, into=None):
    """Compute an unrealized expression with one launch and keep the result (baretile/tensor.py:466-524)."""
    self.rt.check()
    if self.op is None: return self
    if into is not None: raise ValueError("realize(into=) is not on this backend's path")
    plan = _plan(self)
    if plan is None:
      raise ValueError(f"this backend runs act(alpha * (x @ W) + addend) and (x @ Wg).silu() * (x @ Wu); got {_describe(self)}")
    epilogue, e = plan
    self.addr = self._alloc()
    _launch_matmul(self.rt, e, epilogue, self, self.rows)
    self.op, self.srcs = None, ()
    return self


# ---- jit ----------------------------------------------------------------------------------------------------------

def jit(f):
  """Run f normally on the first call, record the second call's launches, then replay them: later calls queue the
  same launches with the new inputs' addresses and skip f's Python code (baretile/tensor.py:1220-1293). Inputs are
  realized tensors whose shapes and dtypes stay fixed; the result reuses its buffer, so the next call overwrites it.
  f must not read tensors back to the host."""
  import functools
  from baretile_b200.runtime import Bound
  signature, rec, out = None, None, None
  @functools.wraps(f)
  def run(*xs):
    nonlocal signature, rec, out
    if not xs or not all(isinstance(x, Tensor) for x in xs): raise ValueError("jit inputs must be tensors, with at least one input")
    rt = xs[0].rt
    if any(x.rt is not rt for x in xs): raise ValueError("jit inputs must use the same runtime")
    if signature is None:
      result = f(*xs).realize()
      signature = [(x.rt, x.shape, x.dtype, x.runs) for x in xs]
      return result
    if len(xs) != len(signature): raise ValueError(f"jit expected {len(signature)} inputs, got {len(xs)}")
    for x, (runtime, shape, dtype, runs) in zip(xs, signature):
      if x.rt is not runtime: raise ValueError("jit inputs must use the recorded runtime")
      if (x.shape, x.dtype) != (shape, dtype): raise ValueError(f"a jit input is {x.shape} {x.dtype}, where the first call had {shape} {dtype}")
      if x.runs != runs: raise ValueError("a jit input by columns must keep the layout it was recorded with")
    xs = [x.realize() for x in xs]
    if rec is None:
      ins = []
      for i, x in enumerate(xs):       # stand-ins at the inputs' places, under addresses bound to their positions
        t = Tensor.__new__(Tensor)
        t.__dict__.update(x.__dict__)
        t.addr, t.owner, t._stream = Bound(x.addr, i), x, None
        ins.append(t)
      with rt.record() as rec: out = f(*ins).realize()
      return out
    rec.replay({i: x.addr for i, x in enumerate(xs)})
    return out
  return run


# ---- expression matching -------------------------------------------------------------------------------------------

def _describe(t):
  if not isinstance(t, Tensor): return repr(t)
  return t.dtype if t.op is None else f"{t.op}({', '.join(_describe(s) for s in t.srcs)})"


def _linear(t):
  """alpha * (x @ w) + addend as a dict, or None."""
  if t.op == "matmul": return dict(x=t.srcs[0], w=t.srcs[1], alpha=1.0, add=None, dtype=t.dtype)
  if t.op == "scale":
    e = _linear(t.srcs[0])
    if e is None or e["add"] is not None: return None
    return dict(e, alpha=e["alpha"] * t.srcs[1])
  if t.op == "add":
    for a, b in (t.srcs, t.srcs[::-1]):
      e = _linear(a) if a.op else None
      if e is not None and e["add"] is None and b.dtype == "bf16": return dict(e, add=b)
  return None


def _plan(t):
  if t.op in ("relu", "silu"):
    e = _linear(t.srcs[0])
    return None if e is None else (t.op, e)
  if t.op == "mul":
    for a, b in (t.srcs, t.srcs[::-1]):
      if a.op == "silu" and a.srcs[0].op == "matmul" and b.op == "matmul":
        g, u = a.srcs[0], b
        if g.srcs[0] is u.srcs[0] and g.srcs[1].dtype == u.srcs[1].dtype and g.srcs[1].shape == u.srcs[1].shape:
          return "glu", dict(x=g.srcs[0], w=g.srcs[1], w2=u.srcs[1], alpha=1.0, add=None, dtype=t.dtype)
    return None
  e = _linear(t)
  return None if e is None else ("none", e)


def _streamed(w):
  """w in streaming layout: itself if columns() made it, else a relaid copy made once and kept with w."""
  w = w.realize()
  if w.runs: return w
  if w._stream is None: w._stream = w.columns()
  return w._stream


def _launch_matmul(rt, e, epilogue, out, rows, arg=(0, 0), arg_base=0):
  x, w = e["x"].realize(), _streamed(e["w"])
  w2 = _streamed(e["w2"]) if e.get("w2") is not None else None
  add = e["add"].realize() if e["add"] is not None else None
  # both kernels work on whole tiles: the padding of x, of the weights and of the addend is zero, and so is the result's
  fmt, K, N = FMT_CODE[w.dtype], x.tc * 32, w.tc * 32
  if epilogue == "argmax" and w.cols % 32: raise ValueError("the fused pick needs N in multiples of 32 (a padding column's zero could win)")
  out_dtype = FMT_CODE[out.dtype] if out is not None else 0
  osize = tile_bytes(out.dtype) if out is not None else 0
  name = f"matmul {w.dtype} {epilogue}"
  if epilogue == "argmax" and rows > 32: raise ValueError("the fused pick takes up to 32 rows")
  if rows > 32 and epilogue != "argmax":
    # many rows: the tensor-core kernel, which reads x row-major, whole tiles wide
    flat = rt.dram_alloc(2 * rows * K)
    try:
      rt.launch("bt_untilize", (2, x.addr, flat, 1, rows, K), name="rows")
      rt.launch("bt_gemm_bfp", (fmt, EPILOGUE[epilogue], rows, K, w.cols, flat, w.addr, w2.addr if w2 else 0, add.addr if add else 0,
                                add.rows if add else 0, ctypes.c_float(e["alpha"]), out.addr, out_dtype, rt.work), name=f"prefill {w.dtype} {epilogue}")
    finally: rt.dram_free(flat)
    return
  for i in range(0, rows, 32):   # one launch per tile row of x; each streams W once
    m, tr = min(32, rows - i), i // 32
    rt.launch("bt_gemv_bfp", (fmt, EPILOGUE[epilogue], m, K, N, x.addr + tr * x.tc * 2048, w.addr, w2.addr if w2 else 0,
                              (add.addr + (tr * add.tc * 2048 if add.rows > 1 else 0)) if add else 0, ctypes.c_float(e["alpha"]),
                              (out.addr + tr * out.tc * osize) if out is not None else 0, out_dtype, arg[0], arg[1], arg_base,
                              rt.work, rt.work_bytes), name=name)
