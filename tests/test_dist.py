"""The multi-GPU host logic on CPU: two gloo ranks shard the oracle's matmuls the way the GPU ranks shard the kernels
(N-split gate/up with all-gather, K-split down with all-reduce, vocabulary-split argmax with a gathered tie-break),
and a rank that leaves is detected by a short collective timeout instead of a hang."""
import datetime, os, socket, sys
import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port():
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


def run_ranks(fn, world=2, timeout=60, **kw):
  port = free_port()
  ctx = mp.get_context("spawn")
  q = ctx.SimpleQueue()
  procs = [ctx.Process(target=_entry, args=(fn, r, world, port, q, kw)) for r in range(world)]
  for p in procs: p.start()
  for p in procs: p.join(timeout)
  for p in procs:
    if p.is_alive(): p.kill(); pytest.fail("a rank did not finish")
  results = {}
  while not q.empty():
    r, value = q.get()
    results[r] = value
  return results


def _entry(fn, rank, world, port, q, kw):
  sys.path.insert(0, ROOT)
  dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                          timeout=datetime.timedelta(seconds=kw.pop("pg_timeout", 30)))
  try: q.put((rank, fn(rank, world, **kw)))
  except Exception as e: q.put((rank, f"raised {type(e).__name__}"))
  finally:
    try: dist.destroy_process_group()
    except Exception: pass


def _inputs(m, k, n):
  from oracle import bfp_oracle as o
  rng = np.random.default_rng(3)
  bf = lambda a: o.bf16_floats(o.bf16_bits(a))
  return bf(rng.normal(0, 1, (m, k))), bf(rng.normal(0, 0.02, (k, n))), bf(rng.normal(0, 0.02, (k, n))), bf(rng.normal(0, 0.02, (n, k)))


def _mlp(rank, world, gather):
  from oracle import bfp_oracle as o
  from baretile_b200 import dist as bd
  x, wg, wu, wd = _inputs(4, 256, 1184)                       # 37 tile columns: the ranks' shares differ
  a, b = bd.split_tiles(1184, world, rank)
  sizes = [np.subtract(*bd.split_tiles(1184, world, r)[::-1]) for r in range(world)]
  h = o.matmul(x, o.dequant(wg, "bfp4")[:, a:b], "glu", o.dequant(wu, "bfp4")[:, a:b])
  h = o.bf16_floats(o.bf16_half_up(h))                        # the kernel writes bf16
  if gather:
    full = bd.all_gather_columns(torch.from_numpy(h), sizes=[int(s) for s in sizes]).numpy()
    h = full[:, a:b]
  partial = torch.from_numpy(o.matmul(h, o.dequant(wd, "bfp4")[a:b]))
  return bd.all_reduce_sum(partial).numpy()


@pytest.mark.parametrize("gather", [True, False])
def test_sharded_mlp_matches_unsharded(gather):
  from oracle import bfp_oracle as o
  x, wg, wu, wd = _inputs(4, 256, 1184)
  h = o.bf16_floats(o.bf16_half_up(o.matmul(x, o.dequant(wg, "bfp4"), "glu", o.dequant(wu, "bfp4"))))
  want = o.matmul(h, o.dequant(wd, "bfp4"))
  got = run_ranks(_mlp, gather=gather)
  assert set(got) == {0, 1}
  for r in (0, 1): assert o.rel_err(got[r], want) < 1e-5, r
  assert np.array_equal(got[0], got[1])


def _head(rank, world):
  from oracle import bfp_oracle as o
  from baretile_b200 import dist as bd
  rng = np.random.default_rng(9)
  logits = rng.normal(0, 1, (5, 4096)).astype(np.float32)
  logits[0, [100, 3000]] = 9.0                                # a tie across the ranks: the lower index wins
  logits[1, [2500, 2600]] = 9.0                               # a tie inside rank 1
  logits[2, :] = 0.0                                          # all equal: index 0
  logits[2, 7] = -0.0
  a, b = bd.split_tiles(4096, world, rank)
  local = logits[:, a:b]
  idx = o.argmax(local)
  v, i = bd.gather_argmax(torch.from_numpy(local[np.arange(5), idx]), torch.from_numpy((idx + a).astype(np.int32)))
  return v.numpy(), i.numpy(), o.argmax(logits), logits.max(-1)


def test_vocabulary_split_argmax_is_index_exact():
  got = run_ranks(_head)
  for r in (0, 1):
    v, i, want_i, want_v = got[r]
    assert i.tolist() == want_i.tolist() and np.array_equal(v, want_v), r
  assert got[0][1][:3].tolist() == [100, 2500, 0]


def test_split_and_combine_rules():
  from baretile_b200 import dist as bd
  for extent, world in ((28672, 8), (128256, 8), (1184, 3), (64, 2)):
    ranges = [bd.split_tiles(extent, world, r) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == extent
    assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:])) and all(s % 32 == 0 and e % 32 == 0 for s, e in ranges)
  assert bd.split_tiles(128256, 8, 3) == (3 * 16032, 4 * 16032)
  with pytest.raises(ValueError): bd.split_tiles(100, 2, 0)
  with pytest.raises(ValueError): bd.split_tiles(32, 2, 0)
  v, i = bd.combine_argmax([[1.0, 5.0, 0.0], [1.0, 4.0, -0.0], [2.0, 5.0, 0.0]], [[7, 9, 3], [2, 1, 1], [8, 4, 5]])
  assert v.tolist() == [2.0, 5.0, 0.0] and i.tolist() == [8, 4, 1]


def _leaver(rank, world):
  # rank 1 leaves between steps, with nothing in flight; rank 0's next collective ends with an error, not a hang
  from baretile_b200 import dist as bd
  t = torch.ones(4)
  bd.all_reduce_sum(t)
  if rank == 1: return "left"
  bd.all_reduce_sum(t)
  return "finished"


def test_a_rank_that_leaves_is_detected():
  got = run_ranks(_leaver, pg_timeout=5, timeout=90)
  assert got[1] == "left" and got[0].startswith("raised"), got
