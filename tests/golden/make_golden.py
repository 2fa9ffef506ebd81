"""Generate the golden fixtures in this directory by running the reference's own Python code.

Run it where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/baretile-checkout

It imports baretile from that checkout (pure Python, no device needed for these functions) and stores
inputs with the reference's outputs in bfp_golden.npz:
  * gpt2.bf16_bits / tensix.round_bf16 on edge values,
  * gpt2.bfp (bfp8 and bfp4) on the inputs of the reference's own tests (seed 5, wide exponent spread),
    on N(0, 0.02) weights with x20 channels, and on corner runs (zeros, -0, tiny negatives, clamps),
  * tensor._bf16s decoding random and corner block-float tiles,
  * Tensor.frombytes tile images, captured through a stand-in runtime that records the bank writes.
The tests compare the oracle (oracle/bfp_oracle.py, oracle/bfp_oracle.c) with these arrays, so the
fixtures travel to machines that do not have the reference.
"""
import pathlib, struct, sys
import numpy as np


def main(ref):
  sys.path.insert(0, ref)
  from baretile import bh, tensix, tensor
  from baretile.models import gpt2
  out = {}
  rng = np.random.default_rng(5)

  # bf16 rounding: random fp32 bit patterns plus ties, infinities and NaNs
  bits = np.concatenate([rng.integers(0, 2**32, 4096, dtype=np.uint64).astype(np.uint32),
                         np.array([0, 0x80000000, 0x3F808000, 0x3F818000, 0x3F807FFF, 0x3F808001, 0x7F800000, 0xFF800000,
                                   0x7FC00000, 0x7F800001, 0xFFFFFFFF, 0x7F7FFFFF, 0x00000001, 0x00800000], np.uint32)])
  out["round_in"] = bits
  out["round_bf16"] = np.array([tensix.round_bf16(int(b)) for b in bits], np.uint32)
  finite = bits[np.isfinite(bits.view(np.float32))]
  out["bits_in"] = finite
  out["bf16_bits"] = gpt2.bf16_bits(finite.view(np.float32))

  # gpt2.bfp: the reference tests' own input (test/test_models.py:587-593), weights, and corners
  cases = {
    "spread": rng.normal(0, 1, (64, 96)) * np.exp(rng.normal(0, 2, (64, 96))),
    "weights": np.random.default_rng(0).normal(0, 0.02, (96, 128)),
    "cache": np.random.default_rng(16).normal(0, 2, (8, 64)) * 10.0 ** np.random.default_rng(17).integers(-3, 3, (8, 1)),
  }
  cases["weights"][np.random.default_rng(1).choice(96, 3, replace=False)] *= 20
  corner = np.zeros((16, 32), np.float32)
  corner[1, :16] = -0.0
  corner[2, :4] = [1.0, -1.0, 0.0, -0.0]
  corner[3, :16] = [1.0] + [2.0 ** -k for k in range(1, 16)]
  corner[4, :16] = [-1.0] + [-(2.0 ** -k) * 1.5 for k in range(1, 16)]
  corner[5, :16] = np.float32(1.9921875)            # all-ones mantissa: rounds up and clamps
  corner[6, :16] = [255.0, 254.0, 127.5, 127.0, 1.0, 0.5, 0.25, 3.0, -255.0, -254.5, 64.0, 65.0, 66.0, 67.0, 68.0, 69.0]
  corner[7, :16] = [1e-30, -1e-30, 1e-32, 0, 1e-31, 3e-31, 1e-38, -1e-38, 1e-39, 0, 0, 0, 0, 0, 0, 1e-30]
  corner[8, 16:] = [3e38, -3e38, 1e38, 1.0, 2e38, 1.5e38, 1e37, 1e36, 0, 0, 0, 0, 0, 0, 0, -1e38]
  corner[9, :16] = [1.0, 0.0625, 0.06, 0.07, 0.03125, 0.03, 0.04, 0.015625, 0.0078125, 0.00390625, 0.001, 0.002, 0.5, 0.75, 0.875, 0.9375]
  cases["corner"] = corner
  for name, a in cases.items():
    a = np.asarray(a, np.float32)
    out[f"bfp_{name}_in"] = a
    for fmt in ("bfp8", "bfp4"): out[f"bfp_{name}_{fmt}"] = gpt2.bfp(a, fmt).astype(np.float64)

  # tensor._bf16s: decode tiles (random bytes with exponents away from the wrap, then all byte values, then wrap cases)
  for fmt in ("bfp8", "bfp4"):
    tb = tensix.tile_bytes(fmt)
    tiles = rng.integers(0, 256, (6, tb), dtype=np.uint16).astype(np.uint8)
    tiles[:4, :64] = rng.integers(8, 250, (4, 64))
    tiles[4, 64:64 + 256] = np.arange(256) if fmt == "bfp8" else np.resize(np.arange(256), 256)
    tiles[5, :64] = rng.integers(0, 8, 64)              # tiny shared exponents: the decoder wraps mod 256
    out[f"dec_{fmt}_in"] = tiles
    out[f"dec_{fmt}"] = np.stack([np.frombuffer(tensor._bf16s(bytes(t), fmt), np.uint16) for t in tiles])

  # Tensor.frombytes: the tile image it writes, with the bank interleave undone
  class FakeChip:
    def __init__(self): self.banks = {}
    def write(self, x, y, addr, data, start=None): self.banks[(x, y)] = bytes(data)
  class FakeRuntime:
    def __init__(self): self.chip, self.back = FakeChip(), bytearray(1 << 21)
    def check(self): pass
    def dram_alloc(self, size): return 0
    def dram_free(self, addr): pass
  tensor.DMA_UPLOAD = 1 << 40   # always the BAR path, which the fake chip records
  for name, (batch, rows, cols, dtype) in {"a": (1, 70, 100, "bf16"), "b": (2, 33, 40, "fp32"), "row": (1, 1, 70, "bf16"),
                                           "col": (1, 40, 1, "bf16"), "one": (1, 1, 1, "fp32"), "x": (1, 32, 576, "bf16")}.items():
    n = tensix.ITEMSIZE[dtype]
    vals = rng.integers(1, 2 ** (8 * n) - 1, batch * rows * cols, dtype=np.uint64).astype(np.uint16 if n == 2 else np.uint32)
    rt = FakeRuntime()
    t = tensor.Tensor.frombytes(rt, rows, cols, vals.tobytes(), batch, dtype)
    tb = tensix.tile_bytes(dtype)
    banks = [rt.chip.banks[bh.DRAM[b]] for b in range(len(bh.DRAM))]
    image = b"".join(banks[i % 8][i // 8 * tb:(i // 8 + 1) * tb] for i in range(t.tiles))
    out[f"tile_{name}_in"] = vals.reshape(batch, rows, cols)
    out[f"tile_{name}"] = np.frombuffer(image, vals.dtype).reshape(t.tiles, 1024)
    del t

  path = pathlib.Path(__file__).with_name("bfp_golden.npz")
  np.savez_compressed(path, **out)
  print(f"wrote {path} ({path.stat().st_size} bytes, {len(out)} arrays)")


if __name__ == "__main__":
  if len(sys.argv) != 2: raise SystemExit(__doc__)
  main(sys.argv[1])
