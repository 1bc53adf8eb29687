"""Kernel choice by measurement, kept in a database with the reference's schema.

The reference picks between registered kernels either by priority or from a SQLite ``KernelCache`` table keyed by the
kernel context's identifier (``KernelCacheManager``: ``src/nnfusion/engine/cache/manager.hpp:16-70``, table created in
``manager.cpp:54-65``; ``FetchBasedSelector`` / ``ProfilingBasedKernelSelector``:
``src/nnfusion/engine/pass/graph/kernel_selection.cpp:20-73,301-390``).  Here the same table records, per
``DequantDot`` node shape, which of this library's two kernels to run and with which split-K factor, instead of the
built-in rule (small-M kernel up to 16 rows, automatic split).

* identifier: operator type, then the shapes of inputs and outputs joined with ``,`` / ``;``, then the dtypes --
  the recipe of ``KernelContext::generate_identifier`` (``src/nnfusion/core/kernels/kernel_emitter.cpp:415-503``);
* ``Function`` holds the launch choice as json (``{"kernel": .., "split_k": ..}``), ``Miscs`` the measured times as
  ``{"external_profile": {"time": {<device>: microseconds}}}`` the way the reference's profile fields are laid out,
  ``Tags`` the comma-joined tag set, ``Source`` is ``"nnf_b200"``;
* ``fetch_with_tags`` returns the fastest matching entry for the device, like the reference's.
"""
from __future__ import annotations

import hashlib
import json
import os
import sqlite3
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Set

from . import _lib as L

DEVICE_TYPE = "CUDA_GPU"
SOURCE = "nnf_b200"

_SCHEMA = """
CREATE TABLE IF NOT EXISTS KernelCache(
   Key        TEXT NOT NULL,
   Identifier TEXT NOT NULL,
   OpType     TEXT NOT NULL,
   Attributes TEXT DEFAULT "",
   Source     TEXT DEFAULT "External",
   DeviceType TEXT NOT NULL,
   Function   TEXT NOT NULL,
   Tags       TEXT DEFAULT "",
   Miscs      TEXT DEFAULT "",
   PRIMARY KEY(Key)
   );
"""

_DT_NAME = {L.F32: "float", L.F16: "half"}


def identifier(M: int, N: int, K: int, w_bits: int, group: int, x_dtype: int, scale_dtype: int, y_dtype: int,
               dual: bool = False) -> str:
    """``DequantDot`` + input shapes (x, wq, scale, zp [, second set]) ; output shape + dtypes."""
    G = K // group
    wq = [N, K // 2 if w_bits == 4 else K]
    zp = [N, (G + 1) // 2 if w_bits == 4 else G]
    ins = [[M, K], wq, [N, G], zp] * 1 + ([wq, [N, G], zp] if dual else [])
    shapes = ";".join(",".join(str(d) for d in s) for s in ins) + ";" + f"{M},{N}"
    # element_type::c_type_string() spells uint8 tensors "uint8_t" (src/nnfusion/common/type/element_type.cpp:35)
    dts = [_DT_NAME[x_dtype], "uint8_t", _DT_NAME[scale_dtype], "uint8_t"] + \
        (["uint8_t", _DT_NAME[scale_dtype], "uint8_t"] if dual else []) + [_DT_NAME[y_dtype]]
    return "DequantDot" + shapes + "".join(dts)


@dataclass
class KernelEntry:
    identifier: str
    function: dict                       # {"kernel": NNF_B200_KERNEL_*, "split_k": int}
    op_type: str = "DequantDot"
    attributes: dict = field(default_factory=dict)
    source: str = SOURCE
    device_type: str = DEVICE_TYPE
    tags: Set[str] = field(default_factory=set)
    miscs: dict = field(default_factory=dict)
    key: str = ""

    def make_key(self) -> str:
        text = self.identifier + self.device_type + json.dumps(self.function, sort_keys=True) + ",".join(sorted(self.tags))
        return hashlib.sha1(text.encode()).hexdigest()

    def time_us(self, device: str) -> Optional[float]:
        return self.miscs.get("external_profile", {}).get("time", {}).get(device)


class KernelCacheManager:
    def __init__(self, path: Optional[str] = None):
        self.path = path or os.path.join(os.path.expanduser("~"), ".cache", "nnfusion", "kernel_cache.db")
        d = os.path.dirname(self.path)
        if d:
            os.makedirs(d, exist_ok=True)
        self.db = sqlite3.connect(self.path)
        self.db.execute(_SCHEMA)
        self.db.commit()

    def close(self) -> None:
        self.db.close()

    def insert_kernel_entry(self, e: KernelEntry, overwrite: bool = False) -> bool:
        e.key = e.key or e.make_key()
        row = (e.key, e.identifier, e.op_type, json.dumps(e.attributes), e.source, e.device_type,
               json.dumps(e.function), ",".join(sorted(e.tags)), json.dumps(e.miscs))
        try:
            self.db.execute(("INSERT OR REPLACE" if overwrite else "INSERT") +
                            " INTO KernelCache VALUES (?,?,?,?,?,?,?,?,?)", row)
        except sqlite3.IntegrityError:
            return False                  # same key already there and overwrite not asked for
        self.db.commit()
        return True

    def fetch_all(self, ident: str, device_type: str = DEVICE_TYPE) -> List[KernelEntry]:
        rows = self.db.execute(
            "SELECT Key, Identifier, OpType, Attributes, Source, DeviceType, Function, Tags, Miscs FROM KernelCache "
            "WHERE (Identifier = ?) AND (DeviceType = ?);", (ident, device_type)).fetchall()
        return [KernelEntry(key=r[0], identifier=r[1], op_type=r[2], attributes=json.loads(r[3] or "{}"), source=r[4],
                            device_type=r[5], function=json.loads(r[6]), tags=set(t for t in r[7].split(",") if t),
                            miscs=json.loads(r[8] or "{}")) for r in rows]

    def fetch_with_tags(self, ident: str, device_type: str, tags: Iterable[str], device: str) -> Optional[KernelEntry]:
        """The fastest entry (on ``device``) whose tag set equals ``tags``; entries without a time lose."""
        want = set(tags)
        best, best_t = None, float("inf")
        for e in self.fetch_all(ident, device_type):
            if e.tags != want:
                continue
            t = e.time_us(device)
            t = 1048576.0 if t is None else t     # the reference's default for "no profile"
            if t < best_t:
                best, best_t = e, t
        return best


def tune(db: KernelCacheManager, ident: str, candidates: List[dict], measure: Callable[[dict], Optional[float]],
         device: str, tags: Iterable[str] = ("fast",)) -> Optional[KernelEntry]:
    """Measure every candidate launch choice (``measure`` returns microseconds, or None when the library refuses the
    combination), store them all, return the fastest."""
    for fn in candidates:
        t = measure(fn)
        if t is None:
            continue
        db.insert_kernel_entry(KernelEntry(identifier=ident, function=dict(fn), tags=set(tags),
                                           miscs={"external_profile": {"time": {device: float(t)}}}), overwrite=True)
    return db.fetch_with_tags(ident, DEVICE_TYPE, tags, device)


def default_candidates(M: int) -> List[dict]:
    """Both kernels where they apply, and a few split-K factors for the small-M one."""
    out = []
    if M <= 16:
        out += [{"kernel": L.KERNEL_GEMV, "split_k": s} for s in (0, 1, 2, 3, 4, 6, 8)]
    if M >= 1:
        out.append({"kernel": L.KERNEL_GEMM, "split_k": 0})
    return out


def measure_on_gpu(op_factory: Callable[[dict], "object"], x, repeats: int = 50) -> Callable[[dict], Optional[float]]:
    """``measure`` for :func:`tune`: builds the node with the candidate's choice and times it with CUDA events."""
    import torch

    from .linear import NNFB200Error

    def measure(fn: dict) -> Optional[float]:
        try:
            op = op_factory(fn)
            y = op(x)
            for _ in range(5):
                op(x, out=y)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(repeats):
                op(x, out=y)
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) * 1e3 / repeats
        except NNFB200Error:
            return None

    return measure
