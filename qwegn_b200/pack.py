"""QWP1 pack reader and verbatim plane upload.

File layout (Scripts/quantize/pack.py:115-316 of the reference; Swift reader
Sources/Foundation/QWQuant/QWPack.swift:36-147): b"QWP1", a little-endian u64 header length, padding to 256, the
planes (quantized planes 16 KiB aligned, raw planes 256-byte aligned) and, at the very end of the file, that many
bytes of JSON: {"provenance": {...}, "tensors": {name: {"shape", "hq4_off" | "raw_off", "kind", "experts",
"e_hq4", "hq": {"bits", "group"}}}}.  Planes are copied to the device unchanged
(Sources/Foundation/QWLoad/PlaneIO.swift:64-198): the kernels read the pack's own block layout.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from typing import Dict, Optional

import numpy as np

from .gemm import CONTAINERS, ContainerKind, QWGemmError, incumbentHQ4G32, rotatedHQ

MAGIC = b"QWP1"


@dataclass(frozen=True)
class QWQTensorEntry:
    """One entry of the pack index (QWQuantTypes.swift:69-149)."""
    name: str
    shape: tuple
    offset: int
    nbytes: int
    kind: str                      # "blocks", "bf16" or "f32"
    container: Optional[ContainerKind]
    experts: int = 0
    expert_bytes: int = 0


class Pack:
    """QWQuant.Pack: memory-mapped QWP1 file."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        if self._mm[:4] != MAGIC:
            raise QWGemmError(2, f"{path}: not a QWP1 pack")
        (hlen,) = struct.unpack("<Q", self._mm[4:12])
        if hlen <= 0 or hlen > len(self._mm) - 12:
            raise QWGemmError(2, f"{path}: header length {hlen} is outside the file")
        header = json.loads(bytes(self._mm[len(self._mm) - hlen:]).decode("utf-8"))
        self.provenance = header.get("provenance", {})
        self.entries: Dict[str, QWQTensorEntry] = {}
        for name, t in header["tensors"].items():
            shape = tuple(int(v) for v in t["shape"])
            if "raw_off" in t:
                kind = t.get("kind", "bf16")
                esz = 2 if kind == "bf16" else 4
                n = int(np.prod(shape)) if shape else 1
                self.entries[name] = QWQTensorEntry(name, shape, int(t["raw_off"]), n * esz, kind, None)
                continue
            if "hq4_off" not in t:
                continue   # planar legacy kinds have no GEMM consumer
            hq = t.get("hq")
            if hq and hq.get("vq"):
                continue   # vector-quantized formats are outside this path
            cont = rotatedHQ(int(hq["bits"]), int(hq["group"])) if hq else incumbentHQ4G32
            rows = int(np.prod(shape[:-1]))
            k = shape[-1]
            if k % cont.group:
                raise QWGemmError(2, f"{name}: k={k} is not a multiple of group {cont.group}")
            nbytes = rows * cont.row_bytes(k)
            experts = int(t.get("experts", 0))
            if experts and int(t["e_hq4"]) * experts != nbytes:
                raise QWGemmError(2, f"{name}: expert slab size does not match its shape")
            off = int(t["hq4_off"])
            if off + nbytes > len(self._mm) - hlen:
                raise QWGemmError(2, f"{name}: plane runs past the end of the planes")
            self.entries[name] = QWQTensorEntry(name, shape, off, nbytes, "blocks", cont, experts, int(t.get("e_hq4", 0)))

    def plane(self, name: str) -> np.ndarray:
        """The tensor's bytes as they are in the file (uint8 view of the mapping)."""
        e = self.entries[name]
        return np.frombuffer(self._mm, dtype=np.uint8, count=e.nbytes, offset=e.offset)

    def raw_f32(self, name: str) -> np.ndarray:
        e = self.entries[name]
        if e.kind == "f32":
            return np.frombuffer(self._mm, dtype="<f4", count=e.nbytes // 4, offset=e.offset).reshape(e.shape)
        if e.kind == "bf16":
            u = np.frombuffer(self._mm, dtype="<u2", count=e.nbytes // 2, offset=e.offset).astype(np.uint32) << 16
            return u.view(np.float32).reshape(e.shape)
        raise QWGemmError(2, f"{name} is a quantized plane")

    def load(self, hal, name: str):
        """PlaneIO.loadBatch for one tensor: copy the plane verbatim into device memory and wrap it in a weight view.
        A 3-D expert stack [E, N, K] becomes one view of E * N rows (expert e at row e * N)."""
        import torch
        from .gemm import QWWeightView
        e = self.entries[name]
        if e.kind != "blocks":
            raise QWGemmError(2, f"{name} is not a quantized plane")
        host = torch.from_numpy(np.array(self.plane(name)))   # one host copy out of the mapping
        dev = host.to(hal.device)
        rows = int(np.prod(e.shape[:-1]))
        return QWWeightView(dev, rows, e.shape[-1], e.container)

    def close(self):
        self._mm.close()
        self._f.close()
