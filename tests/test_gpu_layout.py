"""Tile layout, block-float pack/unpack and the streaming layout on the GPU, bit for bit against the oracle and
the reference's golden outputs. Every call goes through the C-ABI (via the Runtime/Tensor mirror)."""
import numpy as np
import pytest
from oracle import bfp_oracle as o
from helpers import bf16, raw_tiles, upload, weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["a", "b", "row", "col", "one", "x"])
def test_tilize_matches_reference_image(rt, golden, name):
  from baretile_b200.tensor import Tensor
  a, want = golden[f"tile_{name}_in"], golden[f"tile_{name}"]
  dtype = "bf16" if a.dtype == np.uint16 else "fp32"
  t = Tensor.frombytes(rt, a.shape[1], a.shape[2], a.tobytes(), a.shape[0], dtype)
  got = raw_tiles(rt, t).view(a.dtype)
  assert np.array_equal(got, want)
  assert t.tobytes() == a.tobytes()          # and back: what frombytes took is what tobytes gives


def test_of_rounds_to_nearest_even(rt):
  from baretile_b200.tensor import Tensor
  vals = [[1.0, 1.00390625, 1.01171875, -1.00390625, 3.0e38, 1e-40, float("inf"), 0.1]]
  t = Tensor.of(rt, vals)
  want = o.bf16_floats(o.round_bf16_bits(np.array(vals, np.float32)))
  assert np.array_equal(t.numpy().view(np.uint32), want.view(np.uint32))
  assert Tensor.of(rt, [[1, 2], [3, 4]], "int32").tolist() == [[1, 2], [3, 4]]
  assert Tensor.of(rt, [[[1.5, 2.5]], [[3.5, 4.5]]], "fp32").tolist() == [[[1.5, 2.5]], [[3.5, 4.5]]]


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("case", ["spread", "weights", "cache", "corner"])
def test_pack_golden(rt, golden, c_oracle, fmt, case):
  # the cast's bytes are the oracle's, and what reads back are the reference's gpt2.bfp values (test/test_models.py:587-593)
  a = golden[f"bfp_{case}_in"]
  t = upload(rt, bf16(a)).cast(fmt)
  tiles = o.tilize(o.bf16_bits(a))
  want = o.pack_tiles(tiles, fmt)
  assert np.array_equal(raw_tiles(rt, t), want)
  assert np.array_equal(raw_tiles(rt, t), c_oracle.pack(tiles, fmt))
  top = np.repeat((o.bf16_bits(a) >> 7 & 255).reshape(a.shape[0], -1, 16).max(-1), 16, axis=1)
  ok = top >= 8   # below, the reference's decoder wraps the exponent and gpt2.bfp does not; no reference test pins either
  assert np.array_equal(t.numpy().astype(np.float64)[ok], golden[f"bfp_{case}_{fmt}"][ok])


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_pack_unpack_random(rt, fmt):
  rng = np.random.default_rng(7)
  for shape in ((70, 100), (1, 70), (256, 512), (33, 31)):
    a = bf16(rng.normal(0, 1, shape) * np.exp(rng.normal(0, 2, shape)))
    t = upload(rt, a).cast(fmt)
    tiles = o.tilize(o.bf16_bits(a))
    packed = o.pack_tiles(tiles, fmt)
    assert np.array_equal(raw_tiles(rt, t), packed), shape
    back = t.cast("bf16")
    assert np.array_equal(raw_tiles(rt, back).view(np.uint16), o.unpack_tiles(packed, fmt)), shape
  w = weights(rng, 512, 256)
  assert np.array_equal(upload(rt, w).cast(fmt).numpy(), o.dequant(w, fmt))


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_decode_golden_bytes(rt, golden, fmt):
  # arbitrary tile bytes, including -0 (reads as -inf) and tiny shared exponents, decode as tensor._bf16s does
  from baretile_b200.tensor import Tensor
  tiles = golden[f"dec_{fmt}_in"]
  t = Tensor(rt, 32, 32 * len(tiles), dtype=fmt)
  rt.upload(t.addr, tiles.tobytes())
  back = t.cast("bf16")
  assert np.array_equal(raw_tiles(rt, back).view(np.uint16), golden[f"dec_{fmt}"])


def test_zeros_and_known_answers(rt):
  from baretile_b200.tensor import Tensor
  for dtype in ("bf16", "fp32", "int32", "bfp8", "bfp4"):
    z = Tensor.zeros(rt, 70, 100, 2, dtype)
    assert not raw_tiles(rt, z).any() and not np.array(z.tolist()).any(), dtype
    if dtype in ("bfp8", "bfp4"):
      cast = Tensor.frombytes(rt, 70, 100, bytes(2 * 2 * 70 * 100), 2).cast(dtype)
      assert np.array_equal(raw_tiles(rt, cast), raw_tiles(rt, z)), dtype
      neg = upload(rt, np.full((32, 32), -0.0, np.float32)).cast(dtype)      # -0 packs without a sign
      assert not raw_tiles(rt, neg).any(), dtype
      two = np.zeros((32, 32), np.float32)
      two[:, 0], two[:, 1] = 2, 3
      dec = raw_tiles(rt, upload(rt, two).cast(dtype).cast("bf16")).view(np.uint16).reshape(4, 16, 16)
      assert np.all(dec[[0, 2], :, :2] == [0x4000, 0x4040]), dtype           # test/test_kernels.py:2098-2103


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("shape", [(32, 32), (96, 160), (64, 512), (128, 1184), (64, 96)])
def test_columns_is_a_permutation_that_reads_back(rt, fmt, shape):
  rng = np.random.default_rng(11)
  w = weights(rng, *shape)
  t = upload(rt, w).cast(fmt)
  c = t.columns()
  tr, tc = shape[0] // 32, shape[1] // 32
  assert np.array_equal(raw_tiles(rt, c).reshape(-1), o.to_stream(raw_tiles(rt, t), fmt, tr, tc))
  assert np.array_equal(c.numpy(), t.numpy())                                  # reads back as it was
  assert np.array_equal(raw_tiles(rt, c.cast("bf16")), raw_tiles(rt, t.cast("bf16")))


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("tiles", [(1, 1), (3, 5), (2, 8), (5, 3), (17, 6)])
def test_relayout_of_arbitrary_bytes(rt, fmt, tiles):
  # every byte value in every kind of place, the "minus zero" codes a packer never writes included: to the streaming
  # layout as the oracle lays it out, and back to the very bytes
  from baretile_b200 import _lib
  from baretile_b200.tensix import tile_bytes
  from baretile_b200.tensor import FMT_CODE
  tr, tc = tiles
  n = tr * tc * tile_bytes(fmt)
  raw = np.random.default_rng(tr * 100 + tc).integers(0, 256, n, dtype=np.uint8)
  raw[:256] = np.arange(256)
  a, b, c = (rt.dram_alloc(n) for _ in range(3))
  try:
    rt.upload(a, raw.tobytes())
    rt.launch("bt_relayout", (FMT_CODE[fmt], 1, tr, tc, a, b), name="columns")
    rt.launch("bt_relayout", (FMT_CODE[fmt], 0, tr, tc, b, c), name="columns")
    rt.wait()
    streamed = np.frombuffer(rt.download(b, n), np.uint8)
    assert np.array_equal(streamed, o.to_stream(raw, fmt, tr, tc))
    assert np.array_equal(np.frombuffer(rt.download(c, n), np.uint8), raw)
  finally:
    for addr in (a, b, c): rt.dram_free(addr)


def test_bad_arguments_raise(rt):
  from baretile_b200 import _lib
  from baretile_b200.tensor import Tensor
  used = dict(rt.used)
  for data in ([], [[]], [[1, 2], [3], [4, 5, 6]]):
    with pytest.raises(ValueError, match="nonempty|rectangular"): Tensor.of(rt, data)
  for rows, cols, batch in ((0, 1, 1), (1, -1, 1), (1, 1, 0)):
    with pytest.raises(ValueError, match="positive"): Tensor(rt, rows, cols, batch=batch)
  with pytest.raises(ValueError, match="dtype"): Tensor(rt, 1, 1, dtype="float64")
  with pytest.raises(ValueError, match="bytes"): Tensor.frombytes(rt, 1, 2, bytes(2))
  with pytest.raises(ValueError, match="upload as bf16"): Tensor.frombytes(rt, 1, 1, bytes(2), dtype="bfp8")
  assert rt.used == used                       # nothing was allocated for the rejected inputs
  with pytest.raises(ValueError): _lib.call("bt_pack_bfp", rt.device, 7, 256, 256, 1, rt.stream)
  with pytest.raises(ValueError): _lib.call("bt_tilize", rt.device, 3, 256, 256, 1, 1, 1, rt.stream)
  with pytest.raises(ValueError): _lib.call("bt_gemv_bfp", rt.device, 8, 0, 33, 64, 64, 256, 256, 0, 0, 1.0, 256, 0, 0, 0, 0, rt.work, rt.work_bytes, rt.stream)
  rt.wait()                                    # the runtime is still usable


def test_many_small_matrices_in_one_launch(rt):
  # bt_tilize_many / bt_untilize_many give, per matrix, exactly what the single-matrix calls give; more than 64
  # matrices take several launches; ragged shapes, single rows and single columns included
  from baretile_b200.tensor import Tensor
  rng = np.random.default_rng(12)
  shapes = [(1, 4096), (8, 96), (32, 32), (5, 70), (33, 31), (1, 1), (70, 1), (17, 1000)] * 9          # 72 matrices
  host = [o.bf16_bits(rng.normal(0, 1, s).astype(np.float32)) for s in shapes]
  flat = [rt.dram_alloc(h.nbytes) for h in host]
  for a, h in zip(flat, host): rt.upload(a, h.tobytes())
  ts = [Tensor(rt, r, c) for r, c in shapes]
  for t in ts: rt.launch("bt_memset", (t.addr, 0xFF, t.tiles * 2048), name="junk")
  rt.layout_many(True, [(a, t.addr, t.rows, t.cols) for a, t in zip(flat, ts)])
  for t, h in zip(ts, host):
    assert np.array_equal(raw_tiles(rt, t).view(np.uint16), o.tilize(h[None])), t.shape
  back = [rt.dram_alloc(h.nbytes) for h in host]
  rt.layout_many(False, [(t.addr, b, t.rows, t.cols) for t, b in zip(ts, back)])
  rt.wait()
  for b, h in zip(back, host): assert rt.download(b, h.nbytes) == h.tobytes()
  for a in flat + back: rt.dram_free(a)
  with pytest.raises(ValueError, match="no matrices"): rt.layout_many(True, [])
