"""Run under torchrun with one rank per GPU: the sharded MLP and the vocabulary-split greedy pick on real GPUs,
checked on every rank against the oracle's unsharded fp32 NumPy result. Prints one 'ok' line per rank."""
import ctypes, os, sys
import numpy as np
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
  from oracle import bfp_oracle as o
  from helpers import acts, upload, weights
  from baretile_b200 import _lib, dist as bd, pci
  from baretile_b200.chip import Chip
  from baretile_b200.runtime import Runtime
  rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
  dist.init_process_group("gloo")                                   # only hands the communicator's id round
  rt = Runtime(Chip(pci.open_device(local)))
  comm = bd.Comm(rt, rank, world)
  rng = np.random.default_rng(42)                                   # the same inputs on every rank
  k, n, vocab = 1024, 2048 * world // 2 if world > 2 else 2048, 4096 * max(1, world // 2)
  for m in (1, 4, 16):
    x = acts(rng, m, k)
    wg, wu, wd = weights(rng, k, n), weights(rng, k, n), weights(rng, n, k)
    a, b = bd.split_tiles(n, world, rank)
    tx = upload(rt, x)
    mine = (upload(rt, wg[:, a:b]).cast("bfp4").columns(), upload(rt, wu[:, a:b]).cast("bfp4").columns(), upload(rt, wd[a:b]).cast("bfp4").columns())
    mlp = bd.ShardedMLP(rt, *mine, comm)
    h = o.bf16_floats(o.bf16_half_up(o.matmul(x, o.dequant(wg, "bfp4"), "glu", o.dequant(wu, "bfp4"))))
    want = o.matmul(h, o.dequant(wd, "bfp4"))
    for gather in (True, False):
      got = mlp.forward(tx, gather=gather).numpy()
      err = o.rel_err(got, want)
      assert err <= 1e-2, (rank, m, gather, err)
      if gather:                                                    # the gathered activations are the unsharded ones
        full = mlp.gathered.numpy()[:m]
        assert o.rel_err(full, h) <= 1e-2, (rank, m, o.rel_err(full, h))
    # the same layer with the exchange as one kernel over peer memory: several steps in a row (the rows alternate
    # between the two halves of the peer buffer), the same bits on every rank, and no wait that gave up
    peer = bd.ShardedMLP(rt, *mine, comm, peer=True)
    for step in range(5):
      got = peer.forward(upload(rt, x * (step + 1))).numpy()
      err = o.rel_err(got, o.matmul(o.bf16_floats(o.bf16_half_up(o.matmul(x * (step + 1), o.dequant(wg, "bfp4"), "glu", o.dequant(wu, "bfp4")))), o.dequant(wd, "bfp4")))
      assert err <= 1e-2, (rank, m, step, err)
      everyone = [None] * world
      dist.all_gather_object(everyone, got.tobytes())
      assert all(b == everyone[0] for b in everyone), (rank, m, step)
    gave_up = ctypes.c_int(-1)
    _lib.call("bt_peer_check", rt.device, rank, peer.peers, rt.stream, ctypes.byref(gave_up))
    assert gave_up.value == 0
    # LM head: vocabulary split, index-exact against the unsharded fp32 logits of the same kernels' arithmetic
    wv = weights(rng, k, vocab)
    wv[:, 5] = wv[:, vocab - 7]                                     # equal columns on the first and the last rank: a tie
    va, vb = bd.split_tiles(vocab, world, rank)
    head = bd.ShardedHead(rt, upload(rt, wv[:, va:vb]).cast("bfp8").columns(), va, comm)
    head.pick(tx)
    vals, got_ids = head.read(m)
    logits = x.astype(np.float32) @ o.dequant(wv, "bfp8")
    ref = o.argmax(logits)
    gap = np.sort(logits, -1)[:, -1] - np.sort(logits, -1)[:, -2]
    near = (gap <= 2.0 ** -8 * (np.abs(x) @ np.abs(o.dequant(wv, "bfp8"))).max(-1)) & (gap > 0)
    assert np.array_equal(got_ids[~near], ref[~near]), (rank, m, got_ids, ref)
    assert o.rel_err(vals, logits.max(-1)) < 1e-3
    # the same pick with the exchange over peer memory: the same answer, bit for bit, step after step
    head_p = bd.ShardedHead(rt, head.w, va, comm, peer=True)
    for step in range(3):
      head_p.pick(tx)
      vals_p, ids_p = head_p.read(m)
      assert np.array_equal(ids_p, got_ids) and np.array_equal(vals_p, vals), (rank, m, step, ids_p, got_ids)
    _lib.call("bt_peer_check", rt.device, rank, head_p.peers, rt.stream, ctypes.byref(gave_up))
    assert gave_up.value == 0
  rt.wait()
  every = [None] * world
  dist.all_gather_object(every, "ok")
  print(f"rank {rank} of {world}: ok", flush=True)
  comm.close()
  rt.close()
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
