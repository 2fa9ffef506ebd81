"""CPU oracle for the block-float matmul path. TEST INFRASTRUCTURE ONLY.

This is a NumPy restatement of the reference's algorithms for tile layout, bfp8/bfp4 packing and
unpacking, rows put in place into a cache, the fp32 matmul with its epilogues and the stable argmax. Only tests, the smoke check
and the benchmark's CPU-baseline leg import it; the product (baretile_b200) never does.

Parity pin: every function here is checked against outputs of the reference's own Python code
(gpt2.bfp, gpt2.bf16_bits, tensor._bf16s, tensix.round_bf16, Tensor.frombytes), captured as the
fixtures under tests/golden/ by tests/golden/make_golden.py, and against the independent C
restatement in bfp_oracle.c.

Each function cites the reference file:line it follows (paths inside the baretile project).
"""
import numpy as np

TILE = 32
FACE = 16
BFP = {"bfp8": 1024, "bfp4": 512}            # value bytes per tile   (baretile/tensix.py:19)
ITEMSIZE = {"bf16": 2, "fp32": 4, "int32": 4}  # (baretile/tensix.py:14)


def tile_bytes(dtype):
  """Bytes of one 32x32 tile: 64 exponents + values for block floats (baretile/tensix.py:20)."""
  return 64 + BFP[dtype] if dtype in BFP else 1024 * ITEMSIZE[dtype]


def at(r, c):
  """Index of datum (r, c) in a tile of four row-major 16x16 faces (baretile/tensix.py:6-9, :668)."""
  return (r // 16 * 2 + c // 16) * 256 + r % 16 * 16 + c % 16


def bf16_bits(a):
  """fp32 -> bf16 bits, round to nearest even, as uploads do (baretile/models/gpt2.py:14-16)."""
  b = np.asarray(a, np.float32).view(np.uint32)
  return ((b + 0x7FFF + (b >> 16 & 1)) >> 16).astype(np.uint16)


def round_bf16_bits(a):
  """fp32 -> bf16 bits like Tensor.of: RNE, but a NaN keeps a quiet payload (baretile/tensix.py:240-242)."""
  b = np.asarray(a, np.float32).view(np.uint32).astype(np.uint64)
  rne = (b + 0x7FFF + (b >> 16 & 1)) >> 16
  nan = (b & 0x7FFFFFFF) > 0x7F800000
  return np.where(nan, b >> 16 | 0x40, rne).astype(np.uint16)


def bf16_floats(bits):
  """bf16 bits -> fp32 values (baretile/models/gpt2.py:17)."""
  return (np.asarray(bits).astype(np.uint32) << 16).view(np.float32)


def bf16_half_up(a):
  """fp32 -> bf16 bits the way the packer rounds results: (bits + 0x8000) >> 16
  (test/conftest.py:11-13 with packer=True; docs/compiler.md 'Matmul precision')."""
  b = np.asarray(a, np.float32).view(np.uint32).astype(np.uint64)
  return ((b + 0x8000) >> 16).astype(np.uint16)


def bfp_values(a, dtype="bfp8"):
  """Values after rounding to a block-float format, runs of 16 along the last axis
  (baretile/models/gpt2.py:19-30)."""
  bits = bf16_bits(a).astype(np.uint32)
  s, e = bits >> 15, bits >> 7 & 255
  m = (bits & 127) | np.where(e != 0, 128, 0).astype(np.uint32)
  runs = lambda x: x.reshape(*x.shape[:-1], -1, 16)
  top = runs(e).max(-1, keepdims=True)
  shift = np.minimum(top - runs(e), 8)
  q = np.minimum((runs(m) + (1 << shift)) >> (shift + 1), 127)
  if dtype == "bfp4": q = np.minimum((runs(m) + (16 << shift)) >> (shift + 5), 7) << 4
  return (np.where(runs(s), -1.0, 1.0) * q * 2.0 ** (top.astype(np.int64) - 133)).reshape(np.shape(a))


# ---- tile layout --------------------------------------------------------------------------------

def tilize(a):
  """Row-major (batch, rows, cols) array -> tiles in row order, matrices consecutive, each tile as four
  16x16 faces. Partial tiles pad with zeros; a dimension of size 1 repeats across its tile
  (baretile/tensor.py:107-135; the bank interleave at :129-131 is a Tenstorrent artefact and is not
  reproduced: tile i sits at byte i * tile_bytes)."""
  a = np.asarray(a)
  if a.ndim == 2: a = a[None]
  batch, rows, cols = a.shape
  tr, tc = -(-rows // 32), -(-cols // 32)
  full = np.zeros((batch, tr * 32, tc * 32), a.dtype)
  if rows == 1: full[:, :32, :cols] = a            # a single row fills its tile (tensor.py:120)
  else: full[:, :rows, :cols] = a
  if cols == 1: full[:, :, :32] = full[:, :, :1]   # a single column repeats 32 times (tensor.py:122)
  t = full.reshape(batch, tr, 2, 16, tc, 2, 16)    # b, tr, face row, r, tc, face col, c
  return np.ascontiguousarray(t.transpose(0, 1, 4, 2, 5, 3, 6)).reshape(batch * tr * tc, 1024)


def untilize(tiles, batch, rows, cols):
  """Inverse of tilize: tiles -> (batch, rows, cols) (baretile/tensor.py:181-193)."""
  tr, tc = -(-rows // 32), -(-cols // 32)
  t = np.asarray(tiles).reshape(batch, tr, tc, 2, 2, 16, 16).transpose(0, 1, 3, 5, 2, 4, 6)
  return np.ascontiguousarray(t.reshape(batch, tr * 32, tc * 32)[:, :rows, :cols])


# ---- pack / unpack at the byte level ---------------------------------------------------------------

def pack_tiles(tiles_bf16, dtype):
  """bf16 tiles (n, 1024) uint16 -> block-float tiles (n, tile_bytes) uint8.

  A run is a row of a face: 16 consecutive datums of the tile. Exponent byte n of the tile belongs to
  run n (baretile/kernels.py:1130-1138). bfp8 (kernels.py:1108-1114): top = largest exponent field,
  m = mantissa | hidden bit, shift = min(top - e, 8), q = min((m + (1 << shift)) >> (shift + 1), 127),
  byte = q ? sign << 7 | q : 0. bfp4 (kernels.py:1074-1081, :1547-1563): q = shift < 4 ?
  (m + (16 << shift)) >> (shift + 5) : 0, clamped to 7, nibble = q ? sign << 3 | q : 0, the even
  datum in the low nibble."""
  b = np.asarray(tiles_bf16, np.uint16).reshape(-1, 64, 16).astype(np.uint32)
  s, e = b >> 15, b >> 7 & 255
  m = (b & 127) | np.where(e != 0, 128, 0).astype(np.uint32)
  top = e.max(-1, keepdims=True)
  d = top - e
  if dtype == "bfp8":
    shift = np.minimum(d, 8)
    q = np.minimum((m + (1 << shift)) >> (shift + 1), 127)
    vals = np.where(q != 0, s << 7 | q, 0).astype(np.uint8).reshape(-1, 1024)
  else:
    sh = np.minimum(d, 4)  # shifts of 4 or more give 0 below
    q = np.where(d < 4, (m + (16 << sh)) >> (sh + 5), 0)
    q = np.minimum(q, 7)
    nib = np.where(q != 0, s << 3 | q, 0).astype(np.uint8).reshape(-1, 512, 2)
    vals = nib[:, :, 0] | nib[:, :, 1] << 4
  return np.concatenate([top.reshape(-1, 64).astype(np.uint8), vals], axis=1)


def unpack_tiles(tiles, dtype):
  """Block-float tiles (n, tile_bytes) uint8 -> bf16 tiles (n, 1024) uint16, as the unpacker converts
  them (baretile/tensor.py:1095-1104; baretile/kernels.py:1497-1512). A zero magnitude is 0, or -inf
  (0xFF80) with the sign set; otherwise the magnitude is normalised and the exponent wraps mod 256."""
  t = np.asarray(tiles, np.uint8).reshape(-1, tile_bytes(dtype))
  e = np.repeat(t[:, :64].astype(np.int64), 16, axis=1)
  if dtype == "bfp8": x = t[:, 64:].astype(np.int64)
  else:
    v = t[:, 64:].astype(np.int64)
    x = np.stack([v & 15, v >> 4], axis=2).reshape(-1, 1024) << 4
  mag = x & 127
  m = mag << 1
  bl = np.zeros_like(m)
  for k in range(8): bl = np.where(m >> k != 0, k + 1, bl)   # bit_length
  shift = 8 - bl
  out = (x >> 7) << 15 | ((e - shift) % 256) << 7 | ((m << np.maximum(shift, 0)) & 0x7E)
  return np.where(mag == 0, np.where(x >> 7 != 0, 0xFF80, 0), out).astype(np.uint16)


# ---- put: rows written in place, the way a KV cache takes them --------------------------------------

def put(dst_tiles, places, x_tiles, dtype, batch, dst_rows):
  """Rows of x into the rows of a tensor that `places` names, on storage bytes; returns the new tiles.

  dst_tiles: (batch * tr * tc, tile_bytes(dtype)) uint8. x_tiles: (batch * xr * tc, tile_bytes(xd)) uint8 with
  xd = bf16 when dtype is a block float, else dtype. places: n ints, one for each row of x.
  Follows put_kernel (baretile/kernels.py:1083-1168): rows go first to last, so a later row to the same place
  wins (:1097-1098); a place whose tile row is past the tensor's last is skipped, one in the padding of the last
  tile row is written there (:1099-1100, the test `place / 32 < tr` at :1147 on unsigned places, so a negative
  place is skipped too); a row is two runs of 16, the left and right face of each tile column (:1107-1111);
  into a block float a run is packed as a cast packs it: its exponent byte, then its values (:1126-1135); a
  tensor of one logical row takes the row into all 32 rows of its tile (:1111, `a[15] == 1`)."""
  bfp = dtype in BFP
  item = 2 if bfp else ITEMSIZE[dtype]
  n = len(places)
  dst = np.array(dst_tiles, np.uint8)
  tr, xr = -(-dst_rows // 32), -(-n // 32)
  tc = dst.shape[0] // (batch * tr)
  dst = dst.reshape(batch, tr, tc, -1)
  x = np.asarray(x_tiles, np.uint8).reshape(batch * xr * tc, -1)
  if bfp: x = pack_tiles(x.view(np.uint16), dtype)     # runs pack independently, so a tile packs run by run
  x = x.reshape(batch, xr, tc, -1)
  per = BFP[dtype] // 64 if bfp else 16 * item           # value bytes of a run
  first = 64 if bfp else 0
  for i, p in enumerate(int(p) & 0xFFFFFFFF for p in places):
    if p // 32 >= tr: continue
    for r in (range(32) if dst_rows == 1 else (p % 32,)):
      for f in range(2):
        a, b = at(i % 32, 16 * f) // 16, at(r, 16 * f) // 16   # the run in x's tile, in the tensor's tile
        if bfp: dst[:, p // 32, :, b] = x[:, i // 32, :, a]
        dst[:, p // 32, :, first + b * per:first + (b + 1) * per] = x[:, i // 32, :, first + a * per:first + (a + 1) * per]
  return dst.reshape(batch * tr * tc, -1)


# ---- streaming layout (the B200 backend's own `columns()` layout) ---------------------------------------

PANEL = 4  # tile columns per run


def stream_perm(dtype):
  """Byte permutation inside one tile for the streaming layout: position p of the streamed tile holds
  canonical byte stream_perm[p] (recoded, see stream_code). It is defined by this backend (the reference's
  columns() is likewise a rearrangement that reads back unchanged, baretile/kernels.py:1455-1481).

  Exponents: position t*16 + face*4 + j holds the exponent of run face*16 + 4t + kk, j = 0, 2, 1, 3 for
  kk = 0, 1, 2, 3.
  bfp8 values: position 64 + h*512 + lane*16 + fs*8 + ns*4 + j, with lane = g*4 + t, holds datum
  (k = 16h + 4t + kk, n = 16fs + 2g + ns). bfp4 values: position 64 + lane*16 + h*8 + fs*4 + j holds the
  byte with datums (k = 16h + 4t + kk, n = 16fs + 2g) and (…, n + 1)."""
  perm = np.zeros(tile_bytes(dtype), np.int64)
  for t in range(4):
    for face in range(4):
      for kk in range(4): perm[t * 16 + face * 4 + (0, 2, 1, 3)[kk]] = face * 16 + 4 * t + kk
  for h in range(2):
    for g in range(8):
      for t in range(4):
        lane = g * 4 + t
        for fs in range(2):
          for kk in range(4):
            k, j = 16 * h + 4 * t + kk, (0, 2, 1, 3)[kk]
            if dtype == "bfp8":
              for ns in range(2):
                perm[64 + h * 512 + lane * 16 + fs * 8 + ns * 4 + j] = 64 + at(k, 16 * fs + 2 * g + ns)
            else:
              perm[64 + lane * 16 + h * 8 + fs * 4 + j] = 64 + at(k, 16 * fs + 2 * g) // 2
  assert sorted(perm.tolist()) == list(range(tile_bytes(dtype)))
  return perm


def _offset_tables(bits):
  """Sign and magnitude (sign in the top bit) -> offset binary half + v, one to one: the code "minus zero",
  which the packer never writes, takes the one spare offset code, 0."""
  half = 1 << (bits - 1)
  fwd = np.zeros(1 << bits, np.uint8)
  for b in range(1 << bits):
    q = b & (half - 1)
    fwd[b] = (half - q if q else 0) if b & half else half + q
  assert sorted(fwd.tolist()) == list(range(1 << bits))
  return fwd, np.argsort(fwd).astype(np.uint8)


def stream_code(values, dtype, back=False):
  """Value bytes of tiles, canonical coding -> the streaming layout's offset binary (bfp8: 128 + v per byte;
  bfp4: 8 + v per nibble), or back."""
  v = np.asarray(values, np.uint8)
  if dtype == "bfp8": return _offset_tables(8)[1 if back else 0][v]
  t = _offset_tables(4)[1 if back else 0]
  return t[v & 15] | t[v >> 4] << 4


def to_stream(tiles, dtype, tr, tc):
  """Canonical block-float tiles of one (tr x tc)-tile matrix -> streaming layout: runs of PANEL tile
  columns; inside a run, tile row by tile row, the run's tiles of that row side by side, each tile's
  value bytes recoded by stream_code and all its bytes permuted by stream_perm."""
  t = np.asarray(tiles, np.uint8).reshape(tr, tc, tile_bytes(dtype)).copy()
  t[:, :, 64:] = stream_code(t[:, :, 64:], dtype)
  t = t[:, :, stream_perm(dtype)]
  return np.concatenate([t[:, p:p + PANEL].reshape(-1) for p in range(0, tc, PANEL)])


def from_stream(data, dtype, tr, tc):
  tb, out, off = tile_bytes(dtype), np.zeros((tr, tc, tile_bytes(dtype)), np.uint8), 0
  inv = np.argsort(stream_perm(dtype))
  data = np.asarray(data, np.uint8).reshape(-1)
  for p in range(0, tc, PANEL):
    w = min(PANEL, tc - p)
    out[:, p:p + w] = data[off:off + tr * w * tb].reshape(tr, w, tb)[:, :, inv]
    off += tr * w * tb
  out[:, :, 64:] = stream_code(out[:, :, 64:], dtype, back=True)
  return out.reshape(tr * tc, tb)


# ---- the matmul with its epilogues, and the argmax ----------------------------------------------------

def silu(a):
  """a / (1 + exp(-a)) (baretile/models/llama.py:25; baretile/tensor.py:652-653)."""
  a = np.asarray(a, np.float32)
  return a / (1 + np.exp(-a))


def dequant(w, dtype):
  """fp32 values a weight matrix holds once cast to dtype (baretile/models/llama.py:500-510)."""
  w = np.asarray(w, np.float32)
  if dtype == "bf16": return bf16_floats(bf16_bits(w))
  return np.concatenate([bfp_values(w[i:i + 1024], dtype).astype(np.float32) for i in range(0, len(w), 1024)])


def matmul(x, w_deq, epilogue="none", w2_deq=None):
  """fp32 x @ w over already dequantised weights with the fused epilogue
  (baretile/models/llama.py:19-33, :174-183): 'none', 'relu', 'silu', 'glu' = silu(x@w) * (x@w2)."""
  x = np.asarray(x, np.float32)
  y = x @ np.asarray(w_deq, np.float32)
  if epilogue == "relu": return np.maximum(y, 0)
  if epilogue == "silu": return silu(y)
  if epilogue == "glu": return silu(y) * (x @ np.asarray(w2_deq, np.float32))
  if epilogue != "none": raise ValueError(epilogue)
  return y


def argmax(y):
  """Per-row index of the largest value; of equal values the first column wins, and -0 equals 0
  (np.argsort(-x, kind='stable')[..., 0]: baretile/models/llama.py:20, test/test_kernels.py:2044;
  tie rule of topk_kernel, baretile/kernels.py:1173-1231)."""
  return np.argsort(-np.asarray(y), axis=-1, kind="stable")[..., 0]


def rel_err(got, ref):
  """max |got - ref| / max(max |ref|, 1e-6) (docs/workload.md:141)."""
  got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
  return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-6))
