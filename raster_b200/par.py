"""`par/dp4a` (src/raster/par.clj:421-440): 4-way signed int8 dot-accumulate.

Lane 0 is the low byte of each int32.  Host reference of the primitive the
device kernels use (`__dp4a` / the int8 tensor-core tile)."""


def _s8(v: int, shift: int) -> int:
    b = (v >> shift) & 0xFF
    return b - 256 if b >= 128 else b


def dp4a(a: int, b: int, acc: int) -> int:
    a &= 0xFFFFFFFF
    b &= 0xFFFFFFFF
    return acc + sum(_s8(a, s) * _s8(b, s) for s in (0, 8, 16, 24))
