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


def _chain(rt, tx, layers, head):
  """x through gate/up pairs and down projections, each reading the one before it, then the greedy pick of a head."""
  h = tx
  for wg, wu, wd in layers:
    a = ((h @ wg).silu() * (h @ wu)).realize()
    h = (a @ wd).relu().realize()
  values, ids = (h @ head).topk(1)
  return h, values, ids


def test_record_and_replay(rt):
  # a recorded dependent chain (with a pick, whose scratch is a temporary) replays bit for bit like plain launches,
  # also after its input changed in place and after later allocations took whatever memory was free
  # (baretile/tensor.py:1171-1293: a Recording replays a block of commands with one doorbell write)
  from helpers import acts, upload, weights
  from baretile_b200.tensor import Tensor
  rng = np.random.default_rng(101)
  host = [(weights(rng, 512, 1024) * 2, weights(rng, 512, 1024) * 2, weights(rng, 1024, 512) * 2) for _ in range(3)]
  layers = [tuple(upload(rt, w).cast(fmt).columns() for w in ws) for ws, fmt in zip(host, ("bfp8", "bfp4", "bfp8"))]
  head = upload(rt, weights(rng, 512, 2016)).cast("bfp8").columns()
  xs = [acts(rng, 4, 512) for _ in range(3)]
  tx = upload(rt, xs[0])
  want = []
  for x in xs:                                                     # plain launches, one input after the other
    h, values, ids = _chain(rt, upload(rt, x), layers, head)
    want.append((h.numpy(), values.numpy(), ids.numpy()))
  used_before = set(rt.used)
  with rt.record() as step:
    h, values, ids = _chain(rt, tx, layers, head)
  assert step.held, "the pick's scratch was released while recording and must stay with the recording"
  later = [Tensor.zeros(rt, 64, 512) for _ in range(8)]            # takes free memory: must not be what a replay writes
  for x, (wh, wv, wi) in zip(xs, want):
    staged = upload(rt, x)
    rt.launch("bt_d2d", (tx.addr, staged.addr, tx.tiles * 2048), name="copy")   # new input, same address
    step.replay()
    rt.wait()
    assert np.array_equal(h.numpy(), wh) and np.array_equal(values.numpy(), wv) and np.array_equal(ids.numpy(), wi)
  assert all(not np.array(t.tolist()).any() for t in later[:2])    # and a replay wrote nothing into the later tensors
  step.close()
  del h, values, ids, later, staged
  assert set(rt.used) - used_before <= {tx.addr}


def test_wait_times_out_and_the_runtime_stays_usable(rt):
  # Runtime.wait(timeout) raises TimeoutError while work is still queued (baretile/runtime.py:858-876); nothing hangs:
  # the queued work is a few long memsets, and a later wait finds them done
  from baretile_b200.tensor import Tensor
  size = 2 << 30
  big = rt.dram_alloc(size)
  try:
    for _ in range(6): rt.launch("bt_memset", (big, 0, size), name="zeros")
    with pytest.raises(TimeoutError, match="did not finish"): rt.wait(timeout=0.0001)
    rt.wait()
    assert not np.array(Tensor.zeros(rt, 32, 32).tolist()).any()
  finally: rt.dram_free(big)


def test_bounded_wait_for_an_earlier_matmul_reports_instead_of_hanging(rt):
  # A wait inside the matmul kernel that cannot be met gives up after its limit and sets the error word, which
  # Runtime.wait turns into RuntimeError; the kernel ends normally and the runtime keeps working. The wait is made
  # unmeetable on the host: a matmul of a queue takes its x only when every CTA has reported the matmul two places
  # before it finished, and that count (one int per matmul of a launch, from byte 8 of the workspace: kWsOpsDone in
  # csrc/gemv.cu) starts far below zero for the first matmul, so the third one's x warp never sees it complete.
  from helpers import acts, upload, weights
  from oracle import bfp_oracle as o
  rng = np.random.default_rng(5)
  x, w = acts(rng, 4, 4096), weights(rng, 4096, 512)               # 4 sub-panels, each shared by many CTAs
  tx, tw = upload(rt, x), upload(rt, w).cast("bfp8").columns()
  def three():
    with rt.queue(): return [(tx @ tw).realize() for _ in range(3)]
  good = [y.numpy() for y in three()]
  rt.wait()
  rt.upload(rt.work + 8, bytes((ctypes.c_int * 1)(-1000)))
  ys = three()
  with pytest.raises(RuntimeError, match="gave up on a bounded wait"): rt.wait()
  rt.wait()                                                        # the flag was read and cleared, the counts reset
  again = [y.numpy() for y in three()]
  assert all(np.array_equal(a, g) for a, g in zip(again, good))
  assert o.rel_err(good[0], x @ o.dequant(w, "bfp8")) <= 1e-2
  del ys


def test_bounded_wait_for_partial_sums_reports_instead_of_hanging(rt):
  # A wait inside the matmul kernel that cannot be met gives up after its limit and sets the error word, which
  # Runtime.wait turns into RuntimeError; the kernel ends normally and the runtime keeps working. The wait is made
  # unmeetable on the host: the arrival counters of the matrix' sub-panels in the scratch start far below zero, so
  # a sub-panel's owner never sees its contributors arrive. Offsets: the first scratch set starts at byte 256 of the
  # workspace and its counters (one int per sub-panel of 4 tile columns) 512 bytes further (kWsSets, kSetCounters in
  # csrc/gemv.cu).
  from helpers import acts, upload, weights
  from oracle import bfp_oracle as o
  rng = np.random.default_rng(5)
  x, w = acts(rng, 4, 4096), weights(rng, 4096, 512)               # 4 sub-panels, each shared by many CTAs
  tx, tw = upload(rt, x), upload(rt, w).cast("bfp8").columns()
  good = (tx @ tw).realize().numpy()
  rt.wait()
  counters = rt.work + 256 + 512
  poisoned = (ctypes.c_int * 4)(*([-1000] * 4))
  rt.upload(counters, bytes(poisoned))
  y = (tx @ tw).realize()
  with pytest.raises(RuntimeError, match="gave up on a bounded wait"): rt.wait()
  rt.wait()                                                        # the flag was read and cleared, the counters reset
  again = (tx @ tw).realize().numpy()
  assert np.array_equal(again, good)
  assert o.rel_err(good, x @ o.dequant(w, "bfp8")) <= 1e-2
  del y


def test_replay_with_bound_arguments_and_jit(rt):
  # a recorded chain whose input address is a Bound argument replays on other tensors (baretile/runtime.py:476-482,
  # baretile/tensor.py:1194-1214), and tensor.jit does the same by itself from its third call on
  from helpers import acts, upload, weights
  from baretile_b200.runtime import Bound
  from baretile_b200.tensor import Tensor, jit
  rng = np.random.default_rng(55)
  host = [(weights(rng, 512, 1024) * 2, weights(rng, 512, 1024) * 2, weights(rng, 1024, 512) * 2) for _ in range(2)]
  layers = [tuple(upload(rt, w).cast("bfp8").columns() for w in ws) for ws in host]
  head = upload(rt, weights(rng, 512, 1024)).cast("bfp8").columns()
  def f(x):
    h = x
    for wg, wu, wd in layers:
      a = ((h @ wg).silu() * (h @ wu)).realize()
      h = (a @ wd).relu().realize()
    return h
  xs = [upload(rt, acts(rng, 4, 512)) for _ in range(4)]
  want = [f(x).numpy() for x in xs]
  # by hand: record on a stand-in whose address is bound to the key "x", replay on each input
  stand_in = Tensor.__new__(Tensor)
  stand_in.__dict__.update(xs[0].__dict__)
  stand_in.addr, stand_in.owner = Bound(xs[0].addr, "x"), xs[0]
  with rt.record() as step: out = f(stand_in)
  assert any(isinstance(a, Bound) for _, args, _, _ in step.launches for a in args)
  for x, w in zip(xs, want):
    step.replay({"x": x.addr})
    rt.wait()
    assert np.array_equal(out.numpy(), w)
  step.replay()                                                      # no binding: as recorded, on xs[0]
  rt.wait()
  assert np.array_equal(out.numpy(), want[0])
  step.close()
  # jit: the first call runs f, the second records, later ones replay with the new input's address
  fast = jit(f)
  for x, w in zip(xs, want): assert np.array_equal(fast(x).numpy(), w)
  with pytest.raises(ValueError, match="where the first call had"): fast(upload(rt, acts(rng, 5, 512)))


def test_copies_beside_a_recorded_step(rt):
  # Runtime.beside(): while step s computes on buffer set s % 2, the inputs of step s + 1 go into the other set and
  # the results of step s - 1 come out of it, as branches of the step's recording. Every step has its own input, so a
  # copy that ran too early or too late shows as a wrong result.
  import ctypes
  from helpers import acts, upload, weights
  from oracle import bfp_oracle as o
  from baretile_b200.tensor import Tensor
  rng = np.random.default_rng(77)
  m, k, n, steps = 4, 512, 1024, 7
  w = upload(rt, weights(rng, k, n)).cast("bfp8").columns()
  xs = [acts(rng, m, k) for _ in range(steps)]
  want = [o.bf16_bits((upload(rt, x) @ w).relu().numpy()).tobytes() for x in xs]
  host_in, host_out = [rt.host_alloc(m * k * 2) for _ in range(2)], [rt.host_alloc(m * n * 2) for _ in range(2)]
  stage_in, stage_out = [rt.dram_alloc(m * k * 2) for _ in range(2)], [rt.dram_alloc(m * n * 2) for _ in range(2)]
  tx = Tensor(rt, m, k)
  def put(buf, x): ctypes.memmove(ctypes.addressof(buf), o.bf16_bits(x).tobytes(), m * k * 2)
  def recorded(b):
    with rt.record() as g:
      with rt.beside(): rt.upload_async(stage_in[1 - b], host_in[1 - b])
      with rt.beside(): rt.download_async(host_out[1 - b], stage_out[1 - b])
      rt.layout_many(True, [(stage_in[b], tx.addr, m, k)])
      y = (tx @ w).relu().realize()
      rt.layout_many(False, [(y.addr, stage_out[b], m, n)])
    assert not rt.unjoined
    return g, y
  put(host_in[0], xs[0]); put(host_in[1], xs[0])
  rt.upload_async(stage_in[0], host_in[0])
  pipe = [recorded(0), recorded(1)]                                  # each also runs once, on whatever the buffers hold
  rt.wait()
  try:
    rt.upload_async(stage_in[0], host_in[0])
    for s in range(steps):
      if s + 1 < steps: put(host_in[(s + 1) % 2], xs[s + 1])          # the caller's part: the next input, before the replay
      pipe[s % 2][0].replay()
      rt.wait()
      if s: assert bytes(host_out[(s - 1) % 2]) == want[s - 1], s      # the previous step's result is here now
    rt.download_async(host_out[(steps - 1) % 2], stage_out[(steps - 1) % 2])
    rt.wait()
    assert bytes(host_out[(steps - 1) % 2]) == want[steps - 1]
    # outside a recording: a copy beside a long launch, joined by wait()
    big = rt.dram_alloc(256 << 20)
    rt.launch("bt_memset", (big, 0, 256 << 20), name="zeros")
    with rt.beside(): rt.download_async(host_out[0], stage_out[(steps - 1) % 2])
    assert len(rt.unjoined) == 1
    rt.wait()
    assert not rt.unjoined and bytes(host_out[0]) == want[steps - 1]
    rt.dram_free(big)
  finally:
    for g, _ in pipe: g.close()
    for addr in stage_in + stage_out: rt.dram_free(addr)
