"""Text-level SPICE netlist model for the Python front end: devices with named terminals,
subcircuit definitions and flattening. The numeric netlist the solver runs comes from the native
parser (``Netlist.to_native``), which also applies engineering suffixes, models and PVT scaling.

API counterpart: ``nangila-spice/src/nangila_spice/parser.py:15-223`` of the reference.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional

TERMINALS = {"R": 2, "C": 2, "L": 2, "V": 2, "I": 2, "D": 2, "M": 4, "Q": 3, "J": 3, "E": 4, "G": 4}


@dataclass
class Device:
    """One circuit element: name, type letter, terminal nets in card order, ``key=value`` parameters
    and the model (or subcircuit) name where the card has one."""
    name: str
    dev_type: str
    nodes: list[str] = field(default_factory=list)
    params: dict[str, str] = field(default_factory=dict)
    model: Optional[str] = None
    value: Optional[str] = None


@dataclass
class Subcircuit:
    name: str
    ports: list[str] = field(default_factory=list)
    devices: list[Device] = field(default_factory=list)


@dataclass
class Netlist:
    title: str = ""
    devices: list[Device] = field(default_factory=list)
    subcircuits: dict[str, Subcircuit] = field(default_factory=dict)
    global_nodes: set[str] = field(default_factory=set)
    directives: list[str] = field(default_factory=list)
    source_path: Optional[str] = None
    source_text: Optional[str] = None

    @property
    def num_devices(self) -> int:
        return len(self.devices)

    @property
    def num_nodes(self) -> int:
        nets = set()
        for d in self.devices:
            nets.update(d.nodes)
        return len(nets)

    def flatten(self) -> "Netlist":
        """Expands every ``X`` instance; inner nets and device names get the instance path as prefix
        (``X1.n3``), ports map to the nets of the instance line, ground and global nets stay global."""
        flat = Netlist(title=self.title, global_nodes=set(self.global_nodes), directives=list(self.directives),
                       source_path=self.source_path, source_text=self.source_text)
        for dev in self.devices:
            if dev.dev_type == "X":
                self._expand(dev, "", {}, flat.devices, 0)
            else:
                flat.devices.append(dev)
        return flat

    def _expand(self, inst: Device, prefix: str, outer: dict[str, str], out: list[Device], depth: int) -> None:
        if depth > 64:
            raise RecursionError(f"subcircuit nesting deeper than 64 at {inst.name}")
        sub = self.subcircuits.get((inst.model or "").upper())
        if sub is None:
            raise KeyError(f"unknown subcircuit '{inst.model}' on {inst.name}")
        if len(sub.ports) != len(inst.nodes):
            raise ValueError(f"{inst.name}: {len(inst.nodes)} nets for {len(sub.ports)} ports of {sub.name}")
        path = f"{prefix}.{inst.name}" if prefix else inst.name   # instance names keep their case, as the reference's do ("X1.internal")
        mapping = {p.lower(): self._resolve(n, prefix, outer) for p, n in zip(sub.ports, inst.nodes)}
        for d in sub.devices:
            if d.dev_type == "X":
                self._expand(d, path, mapping, out, depth + 1)
            else:
                out.append(Device(name=f"{path}.{d.name}", dev_type=d.dev_type,
                                  nodes=[self._resolve(n, path, mapping) for n in d.nodes], params=dict(d.params),
                                  model=d.model, value=d.value))

    def _resolve(self, net: str, prefix: str, mapping: dict[str, str]) -> str:
        n = net.lower()
        if n in ("0", "gnd") or n in self.global_nodes:
            return "0" if n in ("0", "gnd") else n
        if n in mapping:
            return mapping[n]
        return f"{prefix}.{n}" if prefix else n

    def tran(self) -> Optional[tuple]:
        """``(step, stop)`` in seconds from the deck's ``.tran`` card, or ``None`` when it has none."""
        from . import _native

        for d in self.directives:
            tok = re.sub(r"[(),]", " ", d).split()
            if tok and tok[0].upper() == ".TRAN" and len(tok) >= 3:
                step, stop = _native.parse_scaled(tok[1]), _native.parse_scaled(tok[2])
                if step and stop and step > 0 and stop > 0:
                    return float(step), float(stop)
        return None

    def to_native(self, process: str = "TT", vdd: float = 1.8, temp: float = 27.0) -> dict:
        """The numeric, flattened netlist (the partition-file form) from the native parser."""
        from . import _native

        if self.source_text is None:
            raise ValueError("netlist was not read from SPICE text")
        js, warnings = _native.parse_spice(self.source_text, Path(self.source_path or "netlist").name, process, vdd, temp)
        out = json.loads(js)
        out["warnings"] = list(warnings)
        return out


_VALUE_LIKE = re.compile(r"^([+-]?(\d|\.\d)|[{']|.*=|(DC|AC|PULSE|SIN|PWL|EXP)$)", re.IGNORECASE)


def _first_line_is_card(letter: str, line: str, deck: str = "") -> bool:
    """Whether the first line of a deck is an element rather than a title (same rule as the native parser): it starts
    with an element letter and has the shape of that card: nothing but values and parameters after the nodes of a
    two-terminal element; for a diode, a MOSFET or a sub-circuit call the model / sub-circuit it names is defined in the
    deck ("Diode bridge rectifier circuit" has the field count of a diode card)."""
    tok = re.sub(r"[(),]", " ", line).split()
    if len(tok) < 3 or len(tok[0]) < 2 or not tok[0][1].isalnum():
        return False
    if letter in "RCLVI":
        return len(tok) >= 4 and all(_VALUE_LIKE.match(t) for t in tok[3:])

    def defines(directive: str, name: str) -> bool:
        return re.search(rf"^\s*\{directive}\s+{re.escape(name)}(\s|$)", deck, re.IGNORECASE | re.MULTILINE) is not None

    if letter == "D":
        return len(tok) >= 4 and defines(".model", tok[3])
    if letter == "M":
        return len(tok) >= 6 and defines(".model", tok[5])
    if letter == "X":
        plain = [t for t in tok[1:] if "=" not in t]
        return len(plain) >= 2 and defines(".subckt", plain[-1])
    return letter in "QJEG" and len(tok) >= 4


def _statements(text: str) -> list[str]:
    out: list[str] = []
    first = True
    for raw in text.splitlines():
        line = raw.split(";")[0].split("$")[0].strip()
        if not line:
            first = False
            continue
        if line.startswith("*"):
            first = False
            continue
        if first:
            first = False
            head = line[0].upper()
            if not (head == "." or _first_line_is_card(head, line, text)):
                out.append("*TITLE* " + line)
                continue
        if line.startswith("+"):
            if out:
                out[-1] += " " + line[1:].strip()
            continue
        out.append(line)
    return out


def _parse_device_line(line: str) -> Optional[Device]:
    tok = line.replace("(", " ").replace(")", " ").replace(",", " ").split()
    if len(tok) < 3:
        return None
    name, kind = tok[0], tok[0][0].upper()
    params = {}
    plain = []
    for t in tok[1:]:
        if "=" in t and not t.startswith("="):
            k, v = t.split("=", 1)
            params[k.lower()] = v
        else:
            plain.append(t)
    if kind == "X":
        if len(plain) < 2:
            return None
        return Device(name=name, dev_type="X", nodes=plain[:-1], params=params, model=plain[-1])
    nterm = TERMINALS.get(kind)
    if nterm is None or len(plain) < nterm:
        return None
    rest = plain[nterm:]
    dev = Device(name=name, dev_type=kind, nodes=plain[:nterm], params=params)
    if kind in ("M", "D", "Q", "J"):
        dev.model = rest[0] if rest else None
    elif rest:
        dev.value = " ".join(rest)
    return dev


def parse_netlist_text(text: str, path: Optional[str] = None) -> Netlist:
    nl = Netlist(source_path=path, source_text=text)
    current: Optional[Subcircuit] = None
    for st in _statements(text):
        if st.startswith("*TITLE* "):
            nl.title = st[8:]
            continue
        head = st.split()[0].upper()
        if head == ".SUBCKT":
            tok = st.split()
            ports = [t for t in tok[2:] if "=" not in t and t.upper() != "PARAMS:"]
            current = Subcircuit(name=tok[1].upper(), ports=ports)
            continue
        if head == ".ENDS":
            if current is not None:
                nl.subcircuits[current.name] = current
            current = None
            continue
        if head == ".GLOBAL":
            nl.global_nodes.update(t.lower() for t in st.split()[1:])
            continue
        if head == ".END":
            break
        if head.startswith("."):
            nl.directives.append(st)
            continue
        dev = _parse_device_line(st)
        if dev is None:
            continue
        (current.devices if current is not None else nl.devices).append(dev)
    return nl


def parse_netlist(filepath: str) -> Netlist:
    """Reads a ``.sp`` / ``.cir`` file."""
    p = Path(filepath)
    if not p.exists():
        raise FileNotFoundError(filepath)
    text = p.read_text()
    if re.search(r"^\s*\.(include|inc|lib)\b", text, re.IGNORECASE | re.MULTILINE):
        from . import _native

        text = _native.expand_includes(text, str(p.parent), str(p))  # model cards and sub-circuits kept in other files
    return parse_netlist_text(text, str(p))
