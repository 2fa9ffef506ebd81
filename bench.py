"""Benchmark of the block-float matmul path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--reference PATH]

Workload at every N (per GPU): the decode GEMV sweep on Llama-3-8B-shaped random weights: K x N in {4096x4096,
4096x14336, 14336x4096}, bfp8 and bfp4, M in {1, 8, 32} rows of bf16 activations, plus the fused gate/up pair
silu(x Wg) * (x Wu) at 4096x14336. One step is one pass over these 24 matmuls, which do not read one another's
results and leave as one bt_gemv_queue launch. Every matmul streams its own weight buffers and a pass touches about
410 MB of distinct weights, more than three times the L2, so no matmul finds its weights cached. Weights are N(0, 0.02) with 1% of input channels scaled by 20; activations are N(0, 1); seeds fixed.

The metric is achieved HBM GB/s: algorithmic bytes (packed weight tiles + bf16 x + bf16 result) per step over the
step's time. `value` is measured with the inputs resident in HBM (the step recorded once and replayed as a CUDA
graph, timed with CUDA events on the launching stream). `e2e` is the same step through the public Tensor API with
host buffers: every matmul's activations are copied from page-locked host memory, tilized, multiplied, untilized and
copied back inside the timed region (recorded once with Runtime.record() and replayed, then waited for); the copy of
the next step's inputs and of the previous step's results run beside the step's kernels (Runtime.beside), and the
same steps one after the other are reported as `e2e.serial_ms_per_step`. With N > 1 every rank runs the same sweep on its own GPU (weak scaling, no
data-path collective), times are the maximum over ranks, and the sharded configurations that do exchange data are
measured separately (`config.sharded`).

Beside the headline, in `config`: `chain`, a Llama-3-8B decode layer chain (o-proj 4096x4096 -> fused gate/up
4096x14336 -> down 14336x4096, every matmul reading the one before it, 32 layers with their own weights) as queue
launches, which is what a decode step pays at the boundaries between dependent matmuls; `byte_kernels`, the pack,
unpack, relayout and tilize kernels on a 4096x14336 matrix against the same HBM peak; `prefill`, configs[2] on the
tensor cores; `big`, one large matmul (Llama-3-70B gate shape) alone.

--impl reference times the reference's CPU path on a bounded sample: NumPy block-float rounding + fp32 matmul. With
--reference PATH (a checkout of the reference) the rounding is the reference's own gpt2.bfp (kind "reference"); without,
its restatement in oracle/bfp_oracle.py (kind "port").
"""
import argparse, ctypes, hashlib, json, os, statistics, subprocess, sys, threading, time
import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = [(4096, 4096), (4096, 14336), (14336, 4096)]
FORMATS = ["bfp8", "bfp4"]
ROWS = [1, 8, 32]
TILE = {"bfp8": 1088, "bfp4": 576}


def cases():
  """(K, N, fmt, M, pair) for the sweep, ordered so that a weight buffer is reused only after all others were read."""
  out = []
  for m in ROWS:
    for fmt in FORMATS:
      for k, n in SHAPES: out.append((k, n, fmt, m, False))
      out.append((4096, 14336, fmt, m, True))
  return out


def algorithmic_bytes(k, n, fmt, m, pair):
  """Packed weight tiles read once, bf16 x read once, bf16 result written once."""
  return (k // 32) * (n // 32) * TILE[fmt] * (2 if pair else 1) + 2 * m * k + 2 * m * n


def peaks():
  try:
    with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f: return json.load(f)["hbm_gbs"], "measured"
  except Exception: return 6650.0, "fallback"


def rounded(rng, shape, scale, stress=False):
  from oracle import bfp_oracle as o
  a = rng.normal(0, scale, shape).astype(np.float32)
  if stress: a[rng.choice(shape[0], shape[0] // 100, replace=False)] *= 20
  return o.bf16_bits(a)


class Clocks:
  """Samples nvidia-smi while the timed region runs."""
  QUERY = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
  def __init__(self, index):
    self.rows, self.proc = [], None
    try:
      self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                                   stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
      threading.Thread(target=self._read, daemon=True).start()
    except OSError: pass
  def _read(self):
    for line in self.proc.stdout: self.rows.append([c.strip() for c in line.split(",")])
  def stop(self):
    if self.proc is None: return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
    time.sleep(0.15)
    self.proc.terminate()
    rows = [r for r in self.rows if len(r) == 6 and r[0].isdigit()]
    if not rows: return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    reasons = [n for i, n in enumerate(names) if any(r[2 + i] == "Active" for r in rows)]
    return {"sm_mhz": statistics.median(int(r[0]) for r in rows), "sm_max_mhz": int(rows[0][1]), "reasons": reasons, "samples": len(rows)}


def reference_bfp(path):
  """The block-float rounding the CPU leg uses: the reference's own gpt2.bfp when a checkout is given, else the oracle's
  restatement of it. Returns (function(values, dtype) -> values, kind)."""
  from oracle import bfp_oracle as o
  if path:
    sys.path.insert(0, path)
    from baretile.models import gpt2
    return (lambda a, dtype: np.asarray(gpt2.bfp(a, dtype), np.float32)), "reference"
  return (lambda a, dtype: o.bfp_values(a, dtype).astype(np.float32)), "port"


def cpu_sample(path=None):
  """The reference's CPU path (NumPy block-float rounding + fp32 matmul, baretile/models/gpt2.py:19-30 and
  baretile/models/llama.py:19-33,500-510) on a bounded sample of the sweep: 4096 x 14336, both formats, M = 1 and 8.
  Timed three ways: the rounding alone (the packer's CPU counterpart), the matmul on already dequantised weights, and
  both together, which is what the GB/s figure is quoted on; and configs[0] (SmolLM MLP shape) as a time."""
  from oracle import bfp_oracle as o
  bfp, kind = reference_bfp(path)
  rng = np.random.default_rng(0)
  k, n = 4096, 14336
  w = o.bf16_floats(rounded(rng, (k, n), 0.02, True))
  total, t_pack, t_mm = 0, 0.0, 0.0
  for m in (1, 8):
    x = o.bf16_floats(rounded(rng, (m, k), 1.0))
    for fmt in FORMATS:
      t0 = time.perf_counter()
      wd = np.concatenate([bfp(w[i:i + 1024], fmt) for i in range(0, k, 1024)])   # unpack: the weights as the values the format holds
      t1 = time.perf_counter()
      o.matmul(x, wd, "none")
      t2 = time.perf_counter()
      t_pack, t_mm = t_pack + t1 - t0, t_mm + t2 - t1
      total += algorithmic_bytes(k, n, fmt, m, False)
  x0, w0 = o.bf16_floats(rounded(rng, (32, 576), 1.0)), o.bf16_floats(rounded(rng, (576, 1536), 0.02))
  t0 = time.perf_counter()
  for _ in range(20): o.matmul(x0, bfp(w0, "bfp8"), "relu")
  cfg0_ms = (time.perf_counter() - t0) / 20 * 1e3
  dt = t_pack + t_mm
  detail = {"kind": kind, "pack_Mvalues_per_s": round(4 * k * n / t_pack / 1e6, 1), "matmul_on_dequantised_GBps": round(total / t_mm / 1e9, 3),
            "dequant_plus_matmul_GBps": round(total / dt / 1e9, 3), "config0_relu_32x576x1536_bfp8_ms": round(cfg0_ms, 3)}
  return total / dt / 1e9, dt, f"4096x14336 bfp8+bfp4, M=1 and 8: NumPy block-float rounding + fp32 matmul, {dt:.1f} s", detail


def run_reference(args, rank):
  if rank != 0: return
  values, seconds = [], []
  for _ in range(max(1, min(args.warmup, 1))): cpu_sample(args.reference)
  for _ in range(args.steps):
    v, dt, sample, detail = cpu_sample(args.reference)
    values.append(v); seconds.append(dt)
  v = statistics.mean(values)
  print(json.dumps({"impl": "reference", "metric": "decode GEMV achieved HBM GB/s (bfp8/bfp4, Llama-3-8B shapes)", "value": v, "unit": "GB/s",
                    "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(seconds),
                    "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 x bfp8/bfp4, fp32 accumulate", "data": "synthetic",
                    "config": {"workload": "decode-gemv-sweep (configs[1]), bounded sample", "sample": sample, "cpu_detail": detail},
                    "cpu_baseline": {"value": v, "unit": "GB/s", "cores": os.cpu_count(), "kind": detail["kind"], "sample": sample},
                    "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def recorded_traffic():
  """DRAM read + write bytes of one 24-matmul launch, from the ncu capture summarised in profiles/: valid only for the
  kernel source it was taken from, so the file names that source's hash; None when the source has changed since."""
  try:
    with open(os.path.join(ROOT, "profiles", "gemv_queue_kernel_sweep_traffic.json")) as f: rec = json.load(f)
    with open(os.path.join(ROOT, "baretile_b200", "csrc", "gemv.cu"), "rb") as f: sha = hashlib.sha256(f.read()).hexdigest()
    return rec["dram_bytes_per_launch"] if rec["gemv_cu_sha256"] == sha else None
  except Exception: return None


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=20)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
  ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
  ap.add_argument("--reference", default="", help="a checkout of the reference: the CPU leg then uses its own gpt2.bfp")
  ap.add_argument("--no-extras", action="store_true", help="headline and end-to-end only (profiling captures)")
  ap.add_argument("--quick", action="store_true", help="4096x4096 only (profiling captures)")
  ap.add_argument("--only", default="", help="run one case of the sweep, as KxN:fmt:M:pair, e.g. 4096x14336:bfp8:8:0 (profiling captures)")
  ap.add_argument("--prefill-rows", type=int, default=2048, help="rows of the prefill leg; 0 skips it")
  ap.add_argument("--prefill-only", action="store_true", help="of the legs beside the headline, only the prefill one (profiling captures)")
  args = ap.parse_args()
  rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
  if args.impl == "reference": return run_reference(args, rank)
  args.warmup = max(args.warmup, 3)

  from baretile_b200 import _lib, pci
  from baretile_b200.chip import Chip
  from baretile_b200.runtime import Runtime
  from baretile_b200.tensor import Tensor
  dist = None
  # stdout carries the one JSON line and nothing else: whatever libraries print there meanwhile (NCCL announces its
  # version when it starts) goes to stderr
  sys.stdout.flush()
  json_out = os.fdopen(os.dup(1), "w")
  os.dup2(2, 1)
  if world > 1:
    import torch, torch.distributed as dist
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
  rt = Runtime(Chip(pci.open_device(local)))
  dev = rt.device

  # ---- inputs: one weight buffer per (shape, format, role), activations per case ----
  rng = np.random.default_rng(1234 + rank)
  todo = [c for c in cases() if not args.quick or (c[0], c[1]) == (4096, 4096)]
  if args.only:
    shape, fmt, m, pair = args.only.split(":")
    k, n = map(int, shape.split("x"))
    todo = [(k, n, fmt, int(m), bool(int(pair)))]
  weights, work = {}, []
  sources = {}
  def weight(k, n, fmt, role):
    if (k, n, fmt, role) not in weights:
      bits = rounded(rng, (k, n), 0.02, True).tobytes()
      if (k, n) == (4096, 4096): sources[k, n, fmt, role] = bits          # kept for the check against the oracle below
      weights[k, n, fmt, role] = Tensor.frombytes(rt, k, n, bits).cast(fmt).columns()
    return weights[k, n, fmt, role]
  for k, n, fmt, m, pair in todo:
    xh = rounded(rng, (m, k), 1.0)
    x = Tensor.frombytes(rt, m, k, xh.tobytes())
    w = weight(k, n, fmt, "gate" if pair else "w")
    w2 = weight(k, n, fmt, "up") if pair else None
    work.append(dict(k=k, n=n, fmt=fmt, m=m, pair=pair, x=x, xh=xh, w=w, w2=w2, bytes=algorithmic_bytes(k, n, fmt, m, pair),
                     w_source=sources.get((k, n, fmt, "w"))))
  rt.wait()
  step_bytes = sum(c["bytes"] for c in work)

  def expression(c): return (c["x"] @ c["w"]).silu() * (c["x"] @ c["w2"]) if c["pair"] else c["x"] @ c["w"]

  # ---- resident: record the step once, replay it ----
  def kernels_launched():
    n = ctypes.c_uint64()
    _lib.call("bt_launch_count", ctypes.byref(n))
    return n.value
  outs, rt.log = [], []
  kernels_before = kernels_launched()
  with rt.record() as step:
    for c in work: outs.append(expression(c).realize())
    rt.flush()                                 # the queue launch leaves here, into the recording
    kernels_in_recording = kernels_launched() - kernels_before   # (counted before the block's end runs the recording once)
  recorded, rt.log = rt.log, None            # (entry point, arguments) of each launch, to time them one by one below
  assert len(recorded) == len(work) == step.count      # the recording sends them as one queue launch
  def barrier():
    rt.wait()
    if dist is not None: dist.barrier()
  ev = [ctypes.c_uint64() for _ in range(2)]
  for e in ev: _lib.call("bt_event_create", dev, ctypes.byref(e))
  def timed(fn, steps):
    barrier()
    _lib.call("bt_event_record", dev, ev[0], rt.stream)
    for _ in range(steps): fn()
    _lib.call("bt_event_record", dev, ev[1], rt.stream)
    rt.wait()
    ms = ctypes.c_float()
    _lib.call("bt_event_elapsed_ms", dev, ev[0], ev[1], ctypes.byref(ms))
    if dist is not None:
      import torch
      t = torch.tensor([ms.value], device="cuda")
      dist.all_reduce(t, op=dist.ReduceOp.MAX)
      return t.item()
    return ms.value
  for _ in range(args.warmup): step.replay()
  clocks = Clocks(local) if rank == 0 else None
  kernels_per_step = kernels_in_recording    # a replay launches what the recording captured: one kernel per 32 matmuls
  ms = timed(step.replay, args.steps)
  ms_per_step = ms / args.steps
  value = world * step_bytes / (ms_per_step * 1e-3) / 1e9

  # ---- what the replays computed is what the oracle computes: one replayed result per format ----
  from oracle import bfp_oracle as o
  checked = {}
  for c, y in zip(work, outs):
    if c["fmt"] in checked or c["pair"] or c["k"] != 4096 or c["n"] != 4096: continue
    wd = o.bf16_floats(np.frombuffer(c["w_source"], np.uint16).reshape(c["k"], c["n"]))
    ref = o.bf16_floats(c["xh"]).astype(np.float32) @ o.dequant(wd, c["fmt"])
    checked[c["fmt"]] = round(o.rel_err(y.numpy(), ref), 5)
    assert checked[c["fmt"]] <= 1e-2, ("replayed result differs from the oracle", c, checked)

  # ---- per-launch durations, for the roofline: events around every launch of a plain (not replayed) step ----
  pairs = [(ctypes.c_uint64(), ctypes.c_uint64()) for _ in work]
  for a, b in pairs:
    _lib.call("bt_event_create", dev, ctypes.byref(a)); _lib.call("bt_event_create", dev, ctypes.byref(b))
  per = [[] for _ in work]
  # a copy to host memory long enough that the launches below queue up behind it (a read: a memset would leave the L2
  # full of dirty lines, and their write-back would slow the launches that follow it)
  blocker_bytes = 64 << 20
  blocker, blocker_host = rt.dram_alloc(blocker_bytes), rt.host_alloc(blocker_bytes)
  for rep in range(args.warmup + max(5, min(args.steps, 20))):
    rt.download_async(blocker_host, blocker)
    for (a, b), (kernel, kargs, _, _) in zip(pairs, recorded):
      _lib.call("bt_event_record", dev, a, rt.stream)
      _lib.call(kernel, dev, *kargs, rt.stream)
      _lib.call("bt_event_record", dev, b, rt.stream)
    rt.wait()
    if rep < args.warmup: continue
    for i, (a, b) in enumerate(pairs):
      t = ctypes.c_float()
      _lib.call("bt_event_elapsed_ms", dev, a, b, ctypes.byref(t))
      per[i].append(t.value)
  peak, peak_kind = peaks()
  # DRAM read + write bytes of one 24-matmul launch, from an ncu capture of this command; it belongs to the full sweep only
  traffic = recorded_traffic() if len(work) == 24 and world == 1 else None
  table, total_t = [], 0.0
  for c, ts in zip(work, per):
    t = statistics.median(ts)
    total_t += t
    table.append({"K": c["k"], "N": c["n"], "fmt": c["fmt"], "M": c["m"], "pair": c["pair"], "us": round(t * 1e3, 2),
                  "GBps": round(c["bytes"] / (t * 1e-3) / 1e9, 1), "frac": round(c["bytes"] / (t * 1e-3) / 1e9 / peak, 3)})
  per_launch_sum = step_bytes / (total_t * 1e-3) / 1e9      # each launch bracketed by its own events: a few us pessimistic each
  achieved = step_bytes / (ms_per_step * 1e-3) / 1e9         # average over the launches of the timed region
  rt.dram_free(blocker)

  # ---- end to end: host buffers in, host buffers out, through the Tensor API ----
  # One page-locked buffer holds every matmul's x (row-major bf16), another receives every result; each crosses the
  # bus as one copy per step. Offsets are rounded to 256 bytes.
  def offsets(sizes):
    at, out = 0, []
    for s in sizes: out.append(at); at += -(-s // 256) * 256
    return out, at
  in_at, in_bytes = offsets([c["xh"].nbytes for c in work])
  out_at, out_bytes = offsets([2 * c["m"] * c["n"] for c in work])
  host_in, host_out = [rt.host_alloc(in_bytes) for _ in range(2)], [rt.host_alloc(out_bytes) for _ in range(2)]
  for buf in host_in:
    for at, c in zip(in_at, work): ctypes.memmove(ctypes.addressof(buf) + at, c["xh"].ctypes.data, c["xh"].nbytes)
  stage_in, stage_out = [rt.dram_alloc(in_bytes) for _ in range(2)], [rt.dram_alloc(out_bytes) for _ in range(2)]
  for addr, n in [(a, in_bytes) for a in stage_in] + [(a, out_bytes) for a in stage_out]: rt.launch("bt_memset", (addr, 0, n), name="zeros")   # the gaps between matrices too
  def time_steps(step, after=None):
    """Host wall clock per step over the timed steps (max over ranks); `after` runs once inside the timed region."""
    for s in range(args.warmup): step(s)
    barrier()
    t0 = time.perf_counter()
    for s in range(args.warmup, args.warmup + args.steps): step(s)
    if after: after()
    per_step = (time.perf_counter() - t0) / args.steps
    if dist is not None:
      import torch
      t = torch.tensor([per_step], device="cuda")
      dist.all_reduce(t, op=dist.ReduceOp.MAX)
      per_step = t.item()
    return per_step
  # One step after the other. The step is recorded once (the copies from and to the page-locked buffers, one layout
  # kernel each way and the queue launch: five nodes) and replayed: what the reference's tensor.jit does for a decode
  # step. The caller writes its inputs into the page-locked buffer before a replay and reads the results from the
  # other after wait().
  with rt.record() as serial:
    rt.upload_async(stage_in[0], host_in[0])
    rt.layout_many(True, [(stage_in[0] + at, c["x"].addr, c["m"], c["k"]) for c, at in zip(work, in_at)])       # one launch for all x
    ys = [expression(c).realize() for c in work]
    rt.layout_many(False, [(y.addr, stage_out[0] + at, c["m"], c["n"]) for c, y, at in zip(work, ys, out_at)])  # and one for all results
    rt.download_async(host_out[0], stage_out[0])
  def serial_step(s):
    serial.replay()
    rt.wait()
  serial_s = time_steps(serial_step)
  expected = bytes(host_out[0])
  # The same steps with the bus busy beside the kernels (Runtime.beside): while step s computes on buffer set s % 2, the
  # inputs of step s + 1 are copied into the other set and the results of step s - 1 are copied out of it. One
  # recording per set: two branches of one copy each and the step's three launches, replayed in turn and waited for
  # every step. Every step's inputs cross the bus and every step's results reach the host inside the timed region;
  # a result is in the caller's hands one step later, and the last one after a copy of its own (timed too).
  def overlapped(b):
    with rt.record() as g:
      with rt.beside(): rt.upload_async(stage_in[1 - b], host_in[1 - b])
      with rt.beside(): rt.download_async(host_out[1 - b], stage_out[1 - b])
      rt.layout_many(True, [(stage_in[b] + at, c["x"].addr, c["m"], c["k"]) for c, at in zip(work, in_at)])
      out = [expression(c).realize() for c in work]
      rt.layout_many(False, [(y.addr, stage_out[b] + at, c["m"], c["n"]) for c, y, at in zip(work, out, out_at)])
    return g, out
  rt.upload_async(stage_in[0], host_in[0])
  pipe = [overlapped(0), overlapped(1)]
  rt.wait()
  for buf in host_out: ctypes.memset(ctypes.addressof(buf), 0, out_bytes)
  def pipe_step(s):
    pipe[s % 2][0].replay()
    rt.wait()
  def drain():
    last = (args.warmup + args.steps - 1) % 2
    rt.download_async(host_out[last], stage_out[last])
    rt.wait()
  e2e_s = time_steps(pipe_step, drain)
  if args.warmup + args.steps >= 2 and any(bytes(buf) != expected for buf in host_out):
    raise SystemExit("the overlapped end-to-end steps did not return the bytes the step-by-step ones did")
  e2e = world * step_bytes / e2e_s / 1e9
  clock = clocks.stop() if clocks else None

  extras = world == 1 and not args.quick and not args.only and not args.no_extras
  decode_extras = extras and not args.prefill_only

  # ---- a decode layer chain: every matmul reads the one before it (what a decode step pays at the boundaries) ----
  chain = None
  if decode_extras:
    chain = []
    layers = 32
    for fmt in FORMATS:
      base = [weight(4096, 4096, fmt, "w"), weight(4096, 14336, fmt, "gate"), weight(4096, 14336, fmt, "up"), weight(14336, 4096, fmt, "w")]
      stack = []
      for _ in range(layers):                       # every layer streams its own copy: 32 layers are 3.5 to 6.6 GB of weights
        copies = []
        for b in base:
          t = Tensor(rt, b.rows, b.cols, dtype=fmt)
          t.runs = b.runs
          rt.launch("bt_d2d", (t.addr, b.addr, b.tiles * TILE[fmt]), name="copy")
          copies.append(t)
        stack.append(copies)
      chain_bytes = layers * sum(b.tiles * TILE[fmt] for b in base)
      for m in (1, 8):
        h0 = Tensor.frombytes(rt, m, 4096, rounded(rng, (m, 4096), 1.0).tobytes())
        with rt.record() as chain_step:
          h = h0
          with rt.queue():
            for wo, wg, wu, wd in stack:
              a = (h @ wo).realize()
              g = ((a @ wg).silu() * (a @ wu)).realize()
              h = (g @ wd).realize()
        for _ in range(2): chain_step.replay()
        reps = 3
        cms = timed(chain_step.replay, reps) / reps
        chain.append({"fmt": fmt, "M": m, "matmuls": 3 * layers, "us_per_matmul": round(cms * 1e3 / (3 * layers), 2), "GBps": round(chain_bytes / (cms * 1e-3) / 1e9, 1),
                      "frac": round(chain_bytes / (cms * 1e-3) / 1e9 / peak, 3)})
        chain_step.close()
        del h, a, g, h0
      del stack

  # ---- one large matmul alone (Llama-3-70B gate shape, 8192 x 28672): the kernel without the boundaries ----
  big = None
  if decode_extras:
    big = []
    for fmt in FORMATS:
      src = weight(4096, 14336, fmt, "gate")
      ws = []
      for _ in range(3):                              # three copies taken in turn: none finds its bytes in L2
        t = Tensor(rt, 8192, 28672, dtype=fmt)
        t.runs = (-(-t.tc // 4), t.tr, 0)
        for part in range(4): rt.launch("bt_d2d", (t.addr + part * src.tiles * TILE[fmt], src.addr, src.tiles * TILE[fmt]), name="copy")
        ws.append(t)
      for m in (1, 8):
        xb = Tensor.frombytes(rt, m, 8192, rounded(rng, (m, 8192), 1.0).tobytes())
        with rt.record() as big_step:
          ys = [(xb @ w).realize() for w in ws]
        for _ in range(2): big_step.replay()
        reps = 5
        bms = timed(big_step.replay, reps) / (reps * len(ws))
        nbytes = algorithmic_bytes(8192, 28672, fmt, m, False)
        big.append({"K": 8192, "N": 28672, "fmt": fmt, "M": m, "us": round(bms * 1e3, 2), "GBps": round(nbytes / (bms * 1e-3) / 1e9, 1), "frac": round(nbytes / (bms * 1e-3) / 1e9 / peak, 3)})
        big_step.close()
        del ys, xb
      del ws

  # ---- the byte kernels either side of the matmul, on a 4096 x 14336 matrix, against the same HBM peak ----
  byte_kernels = None
  if decode_extras:
    byte_kernels = []
    k, n = 4096, 14336
    values = k * n
    flats = [rt.dram_alloc(2 * values) for _ in range(3)]
    tiles = [Tensor(rt, k, n) for _ in range(3)]
    for f in flats: rt.launch("bt_d2d", (f, weights[k, n, "bfp8", "w"].addr, values), name="copy")    # any bytes will do for a layout kernel
    def time_kernel(name, bytes_per_value, launches):
      for fn in launches: fn()
      reps = 4
      kms = timed(lambda: [fn() for fn in launches], reps) / (reps * len(launches))
      gbps = bytes_per_value * values / (kms * 1e-3) / 1e9
      byte_kernels.append({"kernel": name, "bytes_per_value": bytes_per_value, "us": round(kms * 1e3, 1), "GBps": round(gbps, 1), "frac": round(gbps / peak, 3)})
    time_kernel("tile_wide_kernel<bf16, tilize>", 4.0, [lambda f=f, t=t: rt.launch("bt_tilize", (2, f, t.addr, 1, k, n), name="upload") for f, t in zip(flats, tiles)])
    for t, bits in zip(tiles, range(3)): rt.launch("bt_tilize", (2, flats[0], t.addr, 1, k, n), name="upload")
    real = Tensor.frombytes(rt, k, n, rounded(rng, (k, n), 0.02, True).tobytes())
    for t in tiles: rt.launch("bt_d2d", (t.addr, real.addr, 2 * values), name="copy")
    for fmt in FORMATS:
      tb = TILE[fmt] / 1024
      packed = [Tensor(rt, k, n, dtype=fmt) for _ in range(3)]
      streamed = [Tensor(rt, k, n, dtype=fmt) for _ in range(3)]
      code = int(fmt[3])
      time_kernel(f"pack_kernel<{fmt}>", 2 + tb, [lambda t=t, q=q: rt.launch("bt_pack_bfp", (code, t.addr, q.addr, t.tiles), name=fmt) for t, q in zip(tiles, packed)])
      time_kernel(f"to_stream_kernel<{fmt}>", 2 * tb, [lambda q=q, z=z: rt.launch("bt_relayout", (code, 1, q.tr, q.tc, q.addr, z.addr), name="columns") for q, z in zip(packed, streamed)])
      time_kernel(f"unpack_kernel<{fmt}>", 2 + tb, [lambda t=t, q=q: rt.launch("bt_unpack_bfp", (code, q.addr, t.addr, t.tiles), name="storage") for t, q in zip(tiles, packed)])
      del packed, streamed
    for f in flats: rt.dram_free(f)
    del tiles, real

  # ---- the prefill configuration (configs[2]) on the tensor cores: reported beside the headline, 1 GPU ----
  prefill = None
  if extras and args.prefill_rows > 0:
    M = args.prefill_rows
    xp = Tensor.frombytes(rt, M, 4096, rounded(rng, (M, 4096), 1.0).tobytes())
    wg, wu, wd = weight(4096, 14336, "bfp8", "gate"), weight(4096, 14336, "bfp8", "up"), weight(14336, 4096, "bfp4", "w")
    def prefill_step():
      h = ((xp @ wg).silu() * (xp @ wu)).realize()
      return (h @ wd).realize()
    for _ in range(3): prefill_step()
    reps = max(3, min(args.steps, 10))
    pms = timed(prefill_step, reps) / reps
    flops = 3 * 2 * M * 4096 * 14336
    try:
      with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f: pk = json.load(f)
    except Exception: pk = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
    prefill = {"rows": M, "workload": "configs[2]: x[rows,4096] @ (Wg,Wu)[4096,14336] bfp8 with fused SiLU-gate, then @ Wd[14336,4096] bfp4; bf16 out",
               "TFLOPs": round(flops / (pms * 1e-3) / 1e12, 1), "ms": round(pms, 4), "bound": "tensor",
               "frac_of_burst_peak": round(flops / (pms * 1e-3) / 1e12 / pk["bf16_tflops"], 3),
               "frac_of_sustained_peak": round(flops / (pms * 1e-3) / 1e12 / pk["bf16_tflops_sustained"], 3),
               "includes": "the row-major copy of x and of h that feeds the TMA loads (2 small launches per step)"}

  # ---- the sharded configurations (configs[3], configs[4]): layers split over the ranks, with their exchanges ----
  # Every rank holds its slice of the weights; the matmul launches, the NCCL collectives and the combining kernels
  # are queued through the C-ABI on the runtime's stream. Times are CUDA events, the maximum over ranks; `ideal_us`
  # is the rank's packed weight bytes at the measured HBM peak (the exchanges are latency, not bandwidth).
  sharded = None
  if dist is not None:
    from baretile_b200 import dist as bd
    comm = bd.Comm(rt, rank, world)
    def tiled(rows, cols, seed):      # bf16 bits of a rows x cols matrix, a 1024 x 1024 N(0, 0.02) block repeated
      block = rounded(np.random.default_rng(seed), (1024, 1024), 0.02, True)
      return np.tile(block, (-(-rows // 1024), -(-cols // 1024)))[:rows, :cols]
    def shard(rows, cols, seed, fmt): return Tensor.frombytes(rt, rows, cols, np.ascontiguousarray(tiled(rows, cols, seed)).tobytes()).cast(fmt).columns()
    K3, N3, V4 = 8192, 28672, 128256
    a, b = bd.split_tiles(N3, world, rank)
    slices = (shard(K3, b - a, 1, "bfp4"), shard(K3, b - a, 2, "bfp4"), shard(b - a, K3, 3, "bfp4"))
    mlp = bd.ShardedMLP(rt, *slices, comm)
    # the same layers with their exchange as one kernel over peer memory (CUDA IPC between the ranks' processes): a
    # box where that cannot be set up still reports everything else
    peer_error = None
    try: mlp_peer = bd.ShardedMLP(rt, *slices, comm, peer=True)
    except Exception as e: mlp_peer, peer_error = None, f"{type(e).__name__}: {e}"[:200]
    va, vb = bd.split_tiles(V4, world, rank)
    head = bd.ShardedHead(rt, shard(K3, vb - va, 4, "bfp8"), va, comm)
    try: head_peer = bd.ShardedHead(rt, head.w, va, comm, peer=True) if peer_error is None else None
    except Exception as e: head_peer, peer_error = None, f"{type(e).__name__}: {e}"[:200]
    mlp_bytes, head_bytes = 3 * (K3 // 32) * (N3 // 32) * TILE["bfp4"], (K3 // 32) * (V4 // 32) * TILE["bfp8"]
    sharded = {"ranks": world, "mlp": [], "head": [],
               "mlp_ideal_us": round(mlp_bytes / world / peak / 1e3, 1), "head_ideal_us": round(head_bytes / world / peak / 1e3, 1)}
    def median_us(fn):
      for _ in range(5): fn()
      return round(statistics.median(timed(fn, 10) / 10 for _ in range(7)) * 1e3, 1)   # a median: the first collective of a size may set up connections, and eight ranks' hosts disturb one another
    for m in (1, 4, 16):
      xs = Tensor.frombytes(rt, m, K3, rounded(rng, (m, K3), 1.0).tobytes())
      for gather in (True, False):
        us = median_us(lambda: mlp.forward(xs, gather=gather))
        sharded["mlp"].append({"M": m, "all_gather": gather, "exchange": "nccl all-reduce + rounding kernel", "us": us, "GBps_all_ranks": round(mlp_bytes / us / 1e3, 1)})
      if mlp_peer is not None:
        us = median_us(lambda: mlp_peer.forward(xs))
        sharded["mlp"].append({"M": m, "all_gather": False, "exchange": "one kernel over peer memory", "us": us, "GBps_all_ranks": round(mlp_bytes / us / 1e3, 1)})
    for m in (1, 4, 8):
      xs = Tensor.frombytes(rt, m, K3, rounded(rng, (m, K3), 1.0).tobytes())
      us = median_us(lambda: head.pick(xs))
      sharded["head"].append({"M": m, "exchange": "nccl all-gather + combining kernel", "us": us, "GBps_all_ranks": round(head_bytes / us / 1e3, 1)})
      if head_peer is not None:
        us = median_us(lambda: head_peer.pick(xs))
        sharded["head"].append({"M": m, "exchange": "one kernel over peer memory", "us": us, "GBps_all_ranks": round(head_bytes / us / 1e3, 1)})
    sharded["note"] = ("configs[3]: gate/up [8192,28672] bfp4 split over N, down [28672,8192] split over K: one queue launch, then either an "
                       "NCCL all-reduce of fp32 partial sums and a rounding kernel (with or without the all-gather of the gate/up result) or one "
                       "kernel that adds the ranks' partial rows from peer memory, rounds and tiles; configs[4]: LM head "
                       "[8192,128256] bfp8 split over the vocabulary: fused pick, then an all-gather of 256 bytes per rank and a combining kernel, "
                       "or one kernel that stores the rank's block into every peer's memory and combines")
    if peer_error is not None: sharded["peer_memory"] = "unavailable: " + peer_error
    rt.wait()
    comm.close()

  if dist is not None: dist.barrier()
  if rank == 0:
    line = {"metric": "decode GEMV achieved HBM GB/s (bfp8/bfp4, Llama-3-8B shapes)", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 x bfp8/bfp4, fp32 accumulate", "data": "synthetic",
            "config": {"workload": "decode-gemv-sweep (configs[1]): K x N in {4096x4096, 4096x14336, 14336x4096} x {bfp8, bfp4} x M in {1, 8, 32} + fused gate/up pair",
                       "matmuls_per_step": len(work), "launches_per_step": kernels_per_step, "bytes_per_step": step_bytes, "l2": "a step reads 410 MB of distinct weights (> 3x L2); no buffer is reused within 2x L2 of traffic",
                       "timing": "CUDA events on the launching stream around K replays of the recorded step; max over ranks",
                       "replay_vs_oracle_rel_err": checked,
                       "chain": chain, "chain_note": "Llama-3-8B decode layers, o-proj -> fused gate/up -> down, each reading the one before it, 32 layers of distinct weights, as bt_gemv_queue launches of 32; frac is of the same HBM peak",
                       "big": big, "byte_kernels": byte_kernels, "prefill": prefill, "sharded": sharded},
            "clocks": clock,
            "e2e": {"value": round(e2e, 1), "unit": "GB/s", "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes,
                    "ms_per_step": round(e2e_s * 1e3, 3), "serial_ms_per_step": round(serial_s * 1e3, 3),
                    "how": "host wall clock; every step copies its inputs from page-locked memory and its results back; the copies of the next step's inputs and of the previous step's results run beside the step's kernels (Runtime.beside), each step is waited for; serial_ms_per_step is one step after the other"},
            "gpu_launches": world * args.steps * kernels_per_step,   # the whole job, like value: every rank launches its own
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 3), "traffic": traffic,
                         "of": peak_kind, "kernel": "gemv_queue_kernel: a step is one launch that runs the 24 matmuls in order; bytes per launch / launch duration averaged over the event-timed region",
                         "per_launch_events_GBps": round(per_launch_sum, 1),
                         "frac_of_spec_8TBps": round(achieved / 8000, 3)},
            "cases": table}
    if not args.no_cpu:
      v, dt, sample, detail = cpu_sample(args.reference)
      line["cpu_baseline"] = {"value": round(v, 3), "unit": "GB/s", "cores": os.cpu_count(), "kind": detail["kind"], "sample": sample, "detail": detail}
    json_out.write(json.dumps(line) + "\n")
    json_out.flush()
  rt.close()
  if dist is not None: dist.destroy_process_group()


if __name__ == "__main__":
  main()
