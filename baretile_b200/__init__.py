"""baretile_b200: a B200 (sm_100a) backend for baretile's block-float matmul path.

It keeps baretile's own surface for that path (baretile/tensor.py, baretile/runtime.py, baretile/chip.py,
baretile/pci.py in the reference): `Runtime(Chip(pci.open_device(n)))`, `Tensor.of(rt, ...)`, `.cast("bfp8")`,
`.columns()`, `@`, `.relu()`, `.silu()`, `*`, `.tolist()`. The work runs in hand-written CUDA kernels inside
libbaretile_b200.so, reached through ctypes. There is no CPU fallback: importing a module that needs the
library raises if it has not been built.
"""
__version__ = "0.1.0"
