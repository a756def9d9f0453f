"""Shard plans of the quantized matmul: which slab of a weight matrix a rank owns.

The reference has no weight sharding; this extends its placement vocabulary
(src/raster/compiler/passes/placement.clj:21-89: a plan is data attached to a
value and resolved to ``:cuda:N`` devices) with a split across the GPUs of one box:

* column split -- rank r owns output rows ``[r*out/P, (r+1)*out/P)``: a contiguous slab of the
  codes and of the scales in both host layouts (row-major and the 8-row stream layout of
  src/raster/compiler/backend/cpu/quant.clj:317-326, as long as ``out/P`` is a multiple of 8);
  x is replicated, the per-rank outputs are all-gathered.
* row split -- rank r owns K blocks ``[r*nb/P, (r+1)*nb/P)`` of every row; x is sliced on the
  same 32-element block boundaries (the activation quantizer works per block, so slicing
  changes no code or scale), the per-rank partial products are summed.

Everything here is host arithmetic on numpy arrays in the reference's layouts; the device side
is ``Context.bind_weight(..., split=, rank=, nranks=)`` and ``TpEndpoint``.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from . import _lib as L

BLOCK = 32


@dataclass(frozen=True)
class ShardPlan:
    """{:split :column|:row :ranks P :devices [...] :collective :all-gather|:all-reduce}"""
    split: str
    ranks: int
    devices: tuple = field(default_factory=tuple)

    def __post_init__(self):
        if self.split not in ("column", "row"):
            raise ValueError(f"unknown split {self.split!r}")
        if self.ranks < 1:
            raise ValueError("ranks must be >= 1")
        if self.devices and len(self.devices) != self.ranks:
            raise ValueError("one device per rank")

    @property
    def collective(self) -> str:
        return "all-gather" if self.split == "column" else "all-reduce"

    @property
    def split_code(self) -> int:
        return L.SPLIT_COLUMN if self.split == "column" else L.SPLIT_ROW

    def as_map(self) -> dict:
        return {"split": self.split, "ranks": self.ranks, "devices": list(self.devices),
                "collective": self.collective}


def check(plan: ShardPlan, out: int, in_: int, layout: int = L.LAYOUT_ROWMAJOR) -> None:
    """The divisibility rules; raises ValueError with the failing rule."""
    if in_ % BLOCK:
        raise ValueError(f"in = {in_} is not a multiple of {BLOCK}")
    if plan.split == "column":
        q = 8 if layout == L.LAYOUT_STREAM8 else 1
        if out % (plan.ranks * q):
            raise ValueError(f"column split: out = {out} not divisible by {plan.ranks * q}")
    else:
        if (in_ // BLOCK) % plan.ranks:
            raise ValueError(f"row split: in/32 = {in_ // BLOCK} not divisible by {plan.ranks}")


def shard_shape(plan: ShardPlan, out: int, in_: int) -> tuple:
    """(out, in) of one rank's matrix."""
    return (out // plan.ranks, in_) if plan.split == "column" else (out, in_ // plan.ranks)


def row_range(plan: ShardPlan, rank: int, out: int) -> tuple:
    if plan.split != "column":
        return (0, out)
    n = out // plan.ranks
    return (rank * n, (rank + 1) * n)


def k_range(plan: ShardPlan, rank: int, in_: int) -> tuple:
    if plan.split != "row":
        return (0, in_)
    n = in_ // plan.ranks
    return (rank * n, (rank + 1) * n)


def shard_rowmajor(plan: ShardPlan, rank: int, codes, scales, out: int, in_: int, bits: int):
    """One rank's dense (codes, scales) in the row-major host layout.

    4-bit rows hold 16 bytes per block (byte j: element j low nibble, element j + 16 high), so a
    K slice on block boundaries is a byte slice of each row in both widths."""
    check(plan, out, in_)
    row_bytes = in_ * bits // 8
    c = np.ascontiguousarray(codes).view(np.uint8).reshape(out, row_bytes)
    s = np.ascontiguousarray(scales, dtype=np.float32).reshape(out, in_ // BLOCK)
    r0, r1 = row_range(plan, rank, out)
    k0, k1 = k_range(plan, rank, in_)
    cb0, cb1 = k0 * bits // 8, k1 * bits // 8
    return (np.ascontiguousarray(c[r0:r1, cb0:cb1]).reshape(-1),
            np.ascontiguousarray(s[r0:r1, k0 // BLOCK:k1 // BLOCK]).reshape(-1))


def shard_kquant(plan: ShardPlan, rank: int, enc: dict, out: int, in_: int) -> dict:
    """One rank's arrays of a Q4_K (keys wq, da, db, aq, bq) or Q6_K (wq, sc, ds) matrix, row-major [out, in].

    Every array holds a fixed number of entries per row and super-block of 256 elements (Q4_K: 128 code
    bytes, one da and db, eight aq and bq; Q6_K: 256 code bytes, sixteen sc, one ds), so a column split is a
    slice of rows and a row split a slice of whole super-blocks in every row; the activation quantizer
    q8_K works per super-block, so each rank quantizes its own slice of x exactly as the whole would be."""
    check(plan, out, in_)
    if in_ % 256 or (plan.split == "row" and (in_ // 256) % plan.ranks):
        raise ValueError(f"K-quant shards are cut at super-blocks of 256: in = {in_}, ranks = {plan.ranks}")
    r0, r1 = row_range(plan, rank, out)
    k0, k1 = k_range(plan, rank, in_)
    per_sb = ({"wq": 128, "da": 1, "db": 1, "aq": 8, "bq": 8} if "da" in enc else {"wq": 256, "sc": 16, "ds": 1})
    nsb = in_ // 256
    part = {}
    for key, n in per_sb.items():
        a = np.ascontiguousarray(enc[key]).reshape(out, nsb, n)
        part[key] = np.ascontiguousarray(a[r0:r1, k0 // 256:k1 // 256]).reshape(-1)
    return part


def slice_activations(plan: ShardPlan, rank: int, x, M: int, in_: int):
    """x [M, in] -> the columns this rank multiplies (all of them for a column split)."""
    xa = np.ascontiguousarray(x).reshape(M, in_)
    k0, k1 = k_range(plan, rank, in_)
    return np.ascontiguousarray(xa[:, k0:k1]).reshape(-1)


def combine(plan: ShardPlan, parts, M: int):
    """The collective on host arrays: parts[r] = rank r's [M, out_r] result."""
    ps = [np.asarray(p, dtype=np.float32).reshape(M, -1) for p in parts]
    if plan.split == "column":
        return np.concatenate(ps, axis=1)
    acc = ps[0].copy()
    for p in ps[1:]:          # rank order, f32: the order the device kernel uses
        acc += p
    return acc


def exchange_bytes(plan: ShardPlan, M: int, out: int) -> int:
    """Bytes one rank sends to each peer per call (f32 results)."""
    return 4 * M * (out // plan.ranks if plan.split == "column" else out)
