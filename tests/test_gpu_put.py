"""put on the GPU: rows written in place into bf16, fp32, int32, bfp8 and bfp4 tensors, storage bytes bit for bit
against the oracle's restatement of the reference's put_kernel. Every call goes through the C-ABI (bt_put)."""
import numpy as np
import pytest
from oracle import bfp_oracle as o
from helpers import bf16, raw_tiles, upload, weights, acts

pytestmark = pytest.mark.gpu


def ids_of(rt, places):
  from baretile_b200.tensor import Tensor
  return Tensor.frombytes(rt, 1, len(places), np.asarray(places, np.int32).tobytes(), 1, "int32")


def stored(a, dtype):
  """Storage bytes the oracle expects for row-major values a in a plain format."""
  t = o.tilize(o.bf16_bits(a)) if dtype == "bf16" else o.tilize(np.asarray(a, np.int32 if dtype == "int32" else np.float32))
  return t.view(np.uint8).reshape(t.shape[0], -1)


@pytest.mark.parametrize("dtype", ["bf16", "fp32", "int32"])
def test_scattered_rows_later_one_wins(rt, dtype):
  # 70 rows of a batch of 3 into 200 places over seven tile rows, out of order, one place twice
  rng = np.random.default_rng(23)
  cache, x = rng.normal(0, 1, (3, 200, 96)), rng.normal(0, 1, (3, 70, 96))
  if dtype == "int32": cache, x = np.rint(cache * 1000), np.rint(x * 1000)
  cache, x = (bf16(a) if dtype == "bf16" else a.astype(np.float32) for a in (cache, x))
  places = [int(p) for p in rng.permutation(200)[:70]]
  places[40] = places[7]
  t = upload(rt, cache, dtype)
  assert t.put(ids_of(rt, places), upload(rt, x, dtype)) is t
  assert np.array_equal(raw_tiles(rt, t), o.put(stored(cache, dtype), places, stored(x, dtype), dtype, 3, 200))
  for i, p in enumerate(places): cache[:, p] = x[:, i]
  assert np.array_equal(t.numpy().astype(np.float32), cache)


def test_prompt_rows_in_order_into_an_empty_cache(rt):
  from baretile_b200.tensor import Tensor
  rng = np.random.default_rng(24)
  kv, rows = Tensor.zeros(rt, 64, 64, batch=3), bf16(rng.normal(0, 1, (3, 40, 64)))
  kv.put(ids_of(rt, range(5, 45)), upload(rt, rows))
  got = kv.numpy()
  assert np.array_equal(got[:, 5:45], rows) and not got[:, :5].any() and not got[:, 45:].any()


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_block_float_cache_rounds_as_cast(rt, fmt):
  # one row, rows in two tiles, a prompt filling a tile, the edges: each run of 16 lands as cast packs it
  from baretile_b200.tensor import Tensor
  rng = np.random.default_rng(16)
  cache = Tensor.zeros(rt, 96, 64, batch=4, dtype=fmt)
  tiles = np.zeros((4 * 3 * 2, o.tile_bytes(fmt)), np.uint8)
  want = np.zeros((4, 96, 64), np.float32)
  for places in ([5], [33, 34, 70], list(range(32, 64)), [0, 95]):
    x = bf16(rng.normal(0, 2, (4, len(places), 64)) * 10.0 ** rng.integers(-3, 3, (4, len(places), 1)))
    cache.put(ids_of(rt, places), upload(rt, x))
    tiles = o.put(tiles, places, stored(x, "bf16"), fmt, 4, 96)
    assert np.array_equal(raw_tiles(rt, cache), tiles), (fmt, places)
    want[:, places] = upload(rt, x).cast(fmt).numpy()
    assert np.array_equal(cache.numpy(), want), (fmt, places)


@pytest.mark.parametrize("fmt", ["bf16", "bfp8", "bfp4"])
def test_places_outside_are_skipped_and_padding_is_written(rt, fmt):
  from baretile_b200.tensor import Tensor
  rng = np.random.default_rng(25)
  t = Tensor.zeros(rt, 70, 32, dtype=fmt)
  x = bf16(rng.normal(0, 1, (1, 5, 32)))
  places = [96, -1, 75, 2, 2**31 - 1]       # tile row 3 does not exist; 75 is padding of the last tile row
  t.put(ids_of(rt, places), upload(rt, x))
  zero = np.zeros((3, o.tile_bytes(fmt)), np.uint8)
  want = o.put(zero, places, stored(x, "bf16"), fmt, 1, 70)
  assert np.array_equal(raw_tiles(rt, t), want) and want[2].any()        # the padding row is stored, in tile row 2
  got = t.numpy()
  assert got[2].any() and not np.delete(got, 2, axis=0).any()            # and is not a row of the tensor


@pytest.mark.parametrize("dtype", ["bf16", "fp32", "int32", "bfp8", "bfp4"])
def test_single_row_destination_fills_its_tile(rt, dtype):
  # the reference's known answer (test/test_kernels.py:2095-2103): 2 and 3 read back as 0x4000 and 0x4040 in every row
  from baretile_b200.tensor import Tensor
  xd = "bf16" if dtype in o.BFP else dtype
  x = Tensor.zeros(rt, 1, 2, dtype=dtype)
  x.put(Tensor.of(rt, [[0]], "int32"), Tensor.of(rt, [[2, 3]], xd))
  raw = raw_tiles(rt, x)
  assert np.array_equal(raw, o.put(np.zeros_like(raw), [0], stored(np.array([[[2, 3]]]), xd), dtype, 1, 1))
  if dtype in o.BFP:
    assert np.all(o.unpack_tiles(raw, dtype).reshape(4, 16, 16)[[0, 2], :, :2] == [0x4000, 0x4040])
  else:
    rows = o.untilize(raw.view({"bf16": np.uint16, "fp32": np.float32, "int32": np.int32}[dtype]), 1, 32, 2)[0]
    assert np.array_equal(o.bf16_floats(rows) if dtype == "bf16" else rows, np.tile([2, 3], (32, 1)))
  # two rows of x to a one-row tensor: the later one is what stays
  y = Tensor.zeros(rt, 1, 40, dtype=dtype)
  rows = np.arange(80, dtype=np.float32).reshape(1, 2, 40)
  y.put(ids_of(rt, [3, 31]), upload(rt, rows, xd))
  assert np.array_equal(raw_tiles(rt, y), o.put(np.zeros((2, o.tile_bytes(dtype)), np.uint8), [3, 31], stored(rows, xd), dtype, 1, 1))


def test_put_of_a_tensor_into_itself(rt):
  # x and ids that are the destination are copied first (test/test_kernels.py:2083-2090)
  a = np.arange(64, dtype=np.float32).reshape(64, 1)
  x = upload(rt, a, "fp32")
  x.put(ids_of(rt, list(range(32, 64)) + list(range(32))), x)
  assert np.array_equal(x.numpy(), np.concatenate([a[32:], a[:32]]))


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_long_prompt_into_a_large_cache(rt, fmt):
  # 2048 rows of 8 heads x 128 into places 1000.. of a 4096-row cache: the rest stays, the rows equal their cast
  from baretile_b200.tensor import Tensor
  rng = np.random.default_rng(26)
  cache = Tensor.zeros(rt, 4096, 128, batch=8, dtype=fmt)
  x = bf16(rng.normal(0, 1, (8, 2048, 128)) * np.exp(rng.normal(0, 1, (8, 2048, 1))))
  cache.put(ids_of(rt, range(1000, 3048)), upload(rt, x))
  got = cache.numpy()
  assert np.array_equal(got[:, 1000:3048], upload(rt, x).cast(fmt).numpy())
  assert not got[:, :1000].any() and not got[:, 3048:].any()
  want = o.put(np.zeros((8 * 128 * 4, o.tile_bytes(fmt)), np.uint8), range(1000, 3048), stored(x, "bf16"), fmt, 8, 4096)
  assert np.array_equal(raw_tiles(rt, cache), want)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_matmul_sees_rows_put_into_its_weights(rt, fmt):
  # a tensor that has served as a matmul's B (and so has a copy by columns) is read afresh after a put
  rng = np.random.default_rng(27)
  w, x = weights(rng, 256, 192), acts(rng, 4, 256)
  wt, xt = upload(rt, w).cast(fmt), upload(rt, x)
  before = (xt @ wt).numpy()
  rows = weights(rng, 3, 192, stress=False) * 50
  wt.put(ids_of(rt, [0, 100, 255]), upload(rt, rows))
  after = (xt @ wt).numpy()
  assert np.array_equal(after, (xt @ upload(rt, wt.numpy()).cast(fmt)).numpy()) and not np.array_equal(before, after)


def test_bad_arguments_raise(rt):
  from baretile_b200.tensor import Tensor
  from baretile_b200.runtime import Runtime
  t, x = Tensor.zeros(rt, 64, 32), Tensor.zeros(rt, 2, 32)
  with pytest.raises(ValueError, match="int32 row"): t.put(Tensor.zeros(rt, 1, 2), x)
  with pytest.raises(ValueError, match="int32 row"): t.put(Tensor.zeros(rt, 1, 3, dtype="int32"), x)
  with pytest.raises(ValueError, match="batch and width"): t.put(Tensor.zeros(rt, 1, 2, dtype="int32"), Tensor.zeros(rt, 2, 64))
  with pytest.raises(ValueError, match="bf16 for a block float"):
    Tensor.zeros(rt, 64, 32, dtype="bfp8").put(Tensor.zeros(rt, 1, 2, dtype="int32"), Tensor.zeros(rt, 2, 32, dtype="fp32"))
  with pytest.raises(ValueError, match="too many rows"):
    Tensor.zeros(rt, 32, 32).put(Tensor.zeros(rt, 1, 2**16, dtype="int32"), Tensor.zeros(rt, 2**16, 32))


@pytest.mark.parametrize("dtype", ["bf16", "bfp8"])
def test_many_rows_with_repeated_places(rt, dtype):
  # more rows than places, so most places come several times and the last row to each wins: the one-pass search for
  # each place's last row (used beyond a few rows) against the oracle, which applies the rows in order
  from baretile_b200.tensor import Tensor
  rng = np.random.default_rng(28)
  n, rows = 700, 200
  x = bf16(rng.normal(0, 1, (2, n, 64)))
  places = [int(p) for p in rng.integers(-3, rows + 40, n)]            # some negative, some past the last tile row
  t = Tensor.zeros(rt, rows, 64, batch=2, dtype=dtype)
  t.put(ids_of(rt, places), upload(rt, x))
  zero = np.zeros((2 * 7 * 2, o.tile_bytes(dtype)), np.uint8)
  assert np.array_equal(raw_tiles(rt, t), o.put(zero, places, stored(x, "bf16"), dtype, 2, rows))
  one = Tensor.zeros(rt, 1, 64, dtype=dtype)                           # a one-row destination: the last row into the tile wins
  y = bf16(rng.normal(0, 1, (1, 100, 64)))
  where = [int(p) for p in rng.integers(0, 40, 100)]
  one.put(ids_of(rt, where), upload(rt, y))
  assert np.array_equal(raw_tiles(rt, one), o.put(np.zeros((2, o.tile_bytes(dtype)), np.uint8), where, stored(y, "bf16"), dtype, 1, 1))
