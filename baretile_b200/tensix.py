"""Storage formats of the path, with the reference's names (baretile/tensix.py:6-20, :240-242).

A 32x32 tile has four row-major 16x16 faces: datum (r, c) is at (r // 16 * 2 + c // 16) * 256 + r % 16 * 16 + c % 16.
A block-float tile is 64 exponent bytes, one per face row, then the values: a sign and 7 magnitude bits worth
m * 2^(e - 133) in bfp8; a sign and 3 bits, two to a byte with the first in the low nibble, in bfp4."""
import struct

ITEMSIZE = {"bf16": 2, "fp32": 4, "int32": 4}
BFP = {"bfp8": 1024, "bfp4": 512}
FMT_CODE = {"bf16": 0, "fp32": 1, "int32": 2, "bfp8": 8, "bfp4": 4}   # the C-ABI's format numbers


def tile_bytes(dtype): return 64 + BFP[dtype] if dtype in BFP else 1024 * ITEMSIZE[dtype]
def at(r, c): return (r // 16 * 2 + c // 16) * 256 + r % 16 * 16 + c % 16


def round_bf16(bits):
  """fp32 bits to bf16 bits: round to nearest even; infinities stay and a NaN keeps a quiet payload."""
  if bits & 0x7FFFFFFF > 0x7F800000: return bits >> 16 | 0x40
  return (bits + 0x7FFF + (bits >> 16 & 1)) >> 16


def to_bf16(x): return round_bf16(struct.unpack("<I", struct.pack("<f", x))[0])
def from_bf16(b): return struct.unpack("<f", struct.pack("<I", b << 16))[0]
