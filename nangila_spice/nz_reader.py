"""Pure-Python reader of ``.nz`` waveform files (container versions 1 and 2; layout in
``csrc/spice/nz.hpp``). API counterpart: ``nangila-spice/src/nangila_spice/nz_reader.py``."""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np


@dataclass
class NzHeader:
    version: int
    num_nodes: int
    num_points: int
    t_start: float
    t_end: float
    error_bound: float
    node_names: list[str] = field(default_factory=list)


@dataclass
class NzWaveform:
    header: NzHeader
    time: np.ndarray
    signals: dict[str, np.ndarray]
    predicted_blocks: int = 0
    raw_blocks: int = 0
    file_bytes: int = 0

    @property
    def node_names(self) -> list[str]:
        return self.header.node_names

    @property
    def num_points(self) -> int:
        return int(len(self.time))

    def voltage(self, node: str, time: "float | None" = None) -> float:
        """Voltage of ``node`` at the sample nearest to ``time`` (the last sample when no time is given)."""
        if node not in self.signals:
            raise KeyError(f"no net '{node}' in the file; it holds {', '.join(self.node_names[:8])}{' ...' if len(self.node_names) > 8 else ''}")
        values = self.signals[node]
        if len(values) == 0:
            return 0.0
        if time is None:
            return float(values[-1])
        i = int(np.searchsorted(self.time, time))
        if i <= 0:
            return float(values[0])
        if i >= len(self.time):
            return float(values[-1])
        return float(values[i] if abs(self.time[i] - time) < abs(time - self.time[i - 1]) else values[i - 1])

    @property
    def compression_ratio(self) -> float:
        raw = 8 * self.header.num_points * (self.header.num_nodes + 1)
        return raw / self.file_bytes if self.file_bytes else 1.0

    def summary(self) -> str:
        h = self.header
        return (f".nz v{h.version}: {h.num_nodes} nets x {h.num_points} points, t = {h.t_start:.3e} .. {h.t_end:.3e} s, bound {h.error_bound:.1e} V, "
                f"{self.predicted_blocks} predicted / {self.raw_blocks} raw blocks, {self.compression_ratio:.1f}x smaller than raw")


def read_nz(path: str) -> NzWaveform:
    with open(path, "rb") as f:
        return read_nz_bytes(f.read())


def read_nz_bytes(data: bytes) -> NzWaveform:
    if data[:4] != b"NZWF":
        raise ValueError("not a .nz file (bad magic)")
    pos = 4
    version, nodes, points = struct.unpack_from("<HII", data, pos)
    pos += 10
    if version not in (1, 2):
        raise ValueError(f"unsupported .nz version {version}")
    t_start, t_end, bound = struct.unpack_from("<ddd", data, pos)
    pos += 24
    names = []
    for _ in range(nodes):
        (ln,) = struct.unpack_from("<H", data, pos)
        pos += 2
        names.append(data[pos:pos + ln].decode())
        pos += ln
    time = np.frombuffer(data, dtype="<f8", count=points, offset=pos).copy()
    pos += 8 * points
    (nblocks,) = struct.unpack_from("<I", data, pos)
    pos += 4
    out = np.zeros((nodes, points))
    predicted = raw = 0
    for _ in range(nblocks):
        kind = data[pos]
        node, start, count = struct.unpack_from("<III", data, pos + 1)
        pos += 13
        if node >= nodes or start + count > points:
            raise ValueError("block outside the waveform")
        if kind == 2:
            out[node, start:start + count] = np.frombuffer(data, dtype="<f8", count=count, offset=pos)
            pos += 8 * count
            raw += 1
            continue
        if kind != 1:
            raise ValueError(f"unknown block type {kind}")
        base, grad, scale = struct.unpack_from("<ddd", data, pos)
        pos += 24
        res = np.frombuffer(data, dtype="<i2", count=count, offset=pos).astype(np.float64) * scale
        pos += 2 * count
        predicted += 1
        r = out[node, start:start + count]
        t = time[start:start + count]
        for i in range(count):
            if version >= 2:
                p = base if i == 0 else (base + grad * (t[1] - t[0]) if i == 1 else 2.0 * r[i - 1] - r[i - 2])
            else:
                p = base + grad * (t[i] - t[0])
                if i >= 2:
                    p += 0.25 * (r[i - 2] - 2.0 * r[i - 1] + p)
            r[i] = p + res[i]
    hdr = NzHeader(version, nodes, points, t_start, t_end, bound, names)
    return NzWaveform(hdr, time, {n: out[i] for i, n in enumerate(names)}, predicted, raw, len(data))
