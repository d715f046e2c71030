"""Netlist partitioning.

Nets (not devices) are assigned to partitions; every partition then receives each element that
injects current into one of its nets, and the foreign nets of those elements become ghost nodes.
An element on the cut therefore appears in both neighbouring partitions, which is what the block
relaxation of the partitioned solver needs to converge to the single-matrix solution. Nets held by
an ideal source to ground (supplies, stimulus) are replicated with their source instead of being
shared, and nets tied together by a floating voltage source or by a feedback loop are kept in one
partition.

API counterpart: ``nangila-spice/src/nangila_spice/partitioner.py:33-410`` of the reference
(METIS / spectral / recursive bisection over the device graph). ``pymetis`` is optional here as
there; the built-in methods are recursive spectral bisection and a breadth-first ordering split.
"""
from __future__ import annotations

import json
from collections import deque
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

from .graph import detect_feedback_loops
from .parser import Netlist


@dataclass
class Partition:
    partition_id: int
    device_names: list[str] = field(default_factory=list)
    internal_nodes: set[str] = field(default_factory=set)
    boundary_nodes: set[str] = field(default_factory=set)
    num_devices: int = 0
    netlist: Optional[dict] = None  # the partition file (native JSON form)

    @property
    def ghost_count(self) -> int:
        return len(self.boundary_nodes)


@dataclass
class PartitionResult:
    partitions: list[Partition] = field(default_factory=list)
    total_cut_edges: int = 0
    total_boundary_nodes: int = 0
    method: str = "unknown"
    feedback_groups_enforced: int = 0
    balance_ratio: float = 0.0
    net_assignment: dict[str, int] = field(default_factory=dict)

    def summary(self) -> str:
        sizes = [p.num_devices for p in self.partitions] or [0]
        return "\n".join([
            f"Partitioner: {self.method}",
            f"  Partitions: {len(self.partitions)}",
            f"  Devices:    {sum(sizes)} (min={min(sizes)}, max={max(sizes)}, avg={sum(sizes) / len(sizes):.1f})",
            f"  Balance:    {self.balance_ratio:.2f}x",
            f"  Boundary:   {self.total_boundary_nodes} ghost nodes",
            f"  Cut edges:  {self.total_cut_edges}",
            f"  Constraints: {self.feedback_groups_enforced} feedback groups enforced",
        ])

    def partition_files(self) -> list[str]:
        return [json.dumps(p.netlist) for p in self.partitions]


# ---- element helpers (native JSON form) -----------------------------------------------------------

def _kind(el: dict) -> str:
    return next(iter(el))


def _terminals(el: dict) -> list[int]:
    """All nets an element touches (0 = ground included)."""
    k, b = _kind(el), next(iter(el.values()))
    if k in ("Resistor", "Capacitor", "Inductor"):
        return [b["a"], b["b"]]
    if k in ("VoltageSource", "CurrentSource"):
        return [b["pos"], b["neg"]]
    if k == "Diode":
        return [b["p"], b["n"]]
    if k == "Mosfet":
        return [b["d"], b["g"], b["s"], b["b"]]
    if k == "GhostSource":
        return [b["node"]]
    raise ValueError(f"unknown element kind {k}")


def _current_terminals(el: dict) -> list[int]:
    """Nets whose KCL row the element contributes to."""
    if _kind(el) == "Mosfet":
        b = el["Mosfet"]
        return [b["d"], b["s"]]
    return _terminals(el)


def _remap(el: dict, m: dict[int, int]) -> dict:
    k, b = _kind(el), dict(next(iter(el.values())))
    g = lambda n: 0 if n == 0 else m[n]  # noqa: E731
    if k in ("Resistor", "Capacitor", "Inductor"):
        b["a"], b["b"] = g(b["a"]), g(b["b"])
    elif k in ("VoltageSource", "CurrentSource"):
        b["pos"], b["neg"] = g(b["pos"]), g(b["neg"])
    elif k == "Diode":
        b["p"], b["n"] = g(b["p"]), g(b["n"])
        if "model" in b:
            b["model"] = dict(b["model"], node_p=b["p"], node_n=b["n"])
    elif k == "Mosfet":
        b["d"], b["g"], b["s"] = g(b["d"]), g(b["g"]), g(b["s"])
        b["b"] = m.get(b["b"], 0) if b["b"] else 0
        if "model" in b:
            b["model"] = dict(b["model"], node_d=b["d"], node_g=b["g"], node_s=b["s"])
    return {k: b}


class _UnionFind:
    def __init__(self, n: int):
        self.p = list(range(n))

    def find(self, x: int) -> int:
        while self.p[x] != x:
            self.p[x] = self.p[self.p[x]]
            x = self.p[x]
        return x

    def union(self, a: int, b: int) -> None:
        ra, rb = self.find(a), self.find(b)
        if ra != rb:
            self.p[rb] = ra


# ---- graph partitioning of the net graph ------------------------------------------------------------

def _bfs_order(adj: list[dict[int, float]], nodes: list[int]) -> list[int]:
    """Breadth-first order from a pseudo-peripheral node, component by component."""
    inside = set(nodes)
    seen: set[int] = set()
    order: list[int] = []

    def bfs(start: int) -> list[int]:
        out, q = [start], deque([start])
        local = {start}
        while q:
            u = q.popleft()
            for v in adj[u]:
                if v in inside and v not in local and v not in seen:
                    local.add(v)
                    out.append(v)
                    q.append(v)
        return out

    for s in nodes:
        if s in seen:
            continue
        far = bfs(s)[-1]
        comp = bfs(far)
        seen.update(comp)
        order.extend(comp)
    return order


def _fiedler_split(adj: list[dict[int, float]], nodes: list[int], left_share: float) -> tuple[list[int], list[int]]:
    """Splits `nodes` by the Fiedler vector of the weighted Laplacian of the induced subgraph."""
    n = len(nodes)
    if n <= 2:
        cut = max(1, int(round(n * left_share)))
        return nodes[:cut], nodes[cut:]
    index = {v: i for i, v in enumerate(nodes)}
    order: Optional[list[int]] = None
    try:
        import scipy.sparse as sp
        import scipy.sparse.linalg as spla

        rows, cols, vals = [], [], []
        for v in nodes:
            for u, w in adj[v].items():
                if u in index:
                    rows.append(index[v])
                    cols.append(index[u])
                    vals.append(w)
        a = sp.csr_matrix((vals, (rows, cols)), shape=(n, n))
        ncomp, labels = sp.csgraph.connected_components(a, directed=False)
        if ncomp > 1:
            order = [nodes[i] for i in np.argsort(labels, kind="stable")]
        else:
            lap = sp.diags(np.asarray(a.sum(axis=1)).ravel()) - a
            if n <= 400:
                w, vec = np.linalg.eigh(lap.toarray())
                f = vec[:, 1]
            else:
                w, vec = spla.eigsh(lap.tocsc(), k=2, sigma=-1e-3, which="LM", tol=1e-4)
                f = vec[:, int(np.argsort(w)[1])]
            order = [nodes[i] for i in np.argsort(f, kind="stable")]
    except Exception:
        order = None
    if order is None:
        order = _bfs_order(adj, nodes)
    cut = min(n - 1, max(1, int(round(n * left_share))))
    return order[:cut], order[cut:]


def _recursive_bisect(adj: list[dict[int, float]], nodes: list[int], k: int, first: int, out: dict[int, int], spectral: bool) -> None:
    if k <= 1 or len(nodes) <= 1:
        for v in nodes:
            out[v] = first
        return
    kl = k // 2
    if spectral:
        left, right = _fiedler_split(adj, nodes, kl / k)
    else:
        order = _bfs_order(adj, nodes)
        cut = min(len(order) - 1, max(1, int(round(len(order) * kl / k))))
        left, right = order[:cut], order[cut:]
    _recursive_bisect(adj, left, kl, first, out, spectral)
    _recursive_bisect(adj, right, k - kl, first + kl, out, spectral)


def _partition_metis(adj: list[dict[int, float]], nodes: list[int], k: int) -> dict[int, int]:
    import pymetis

    index = {v: i for i, v in enumerate(nodes)}
    adjacency = [[index[u] for u in adj[v] if u in index] for v in nodes]
    _, membership = pymetis.part_graph(k, adjacency=adjacency)
    return {v: int(membership[i]) for i, v in enumerate(nodes)}


# ---- main entry points --------------------------------------------------------------------------------

def partition_flat(flat: dict, k: int, method: str = "auto", feedback_nets: Optional[list[set[str]]] = None,
                   keep_channels: bool = True) -> PartitionResult:
    """Partitions a numeric netlist (native JSON form as a dict) into ``k`` partition files. With ``keep_channels``
    nets joined by a transistor channel always land in the same partition (fewer than ``k`` partitions result when
    the deck has fewer channel-connected components than that)."""
    from . import _native

    if k <= 0:
        raise ValueError(f"k must be positive, got {k}")
    n = int(flat["num_nodes"])
    names = list(flat.get("node_names") or [f"node_{i + 1}" for i in range(n)])
    elements = flat["elements"]
    # nets held by an ideal source to ground are replicated, not partitioned
    held: set[int] = set()
    for el in elements:
        if _kind(el) == "VoltageSource":
            b = el["VoltageSource"]
            if b["neg"] == 0 and b["pos"] > 0:
                held.add(b["pos"])
            elif b["pos"] == 0 and b["neg"] > 0:
                held.add(b["neg"])
    uf = _UnionFind(n + 1)
    for el in elements:
        if _kind(el) == "VoltageSource":
            b = el["VoltageSource"]
            if b["pos"] > 0 and b["neg"] > 0:
                uf.union(b["pos"], b["neg"])
    # Channel-connected components stay whole: the drain and source of a transistor are coupled in both
    # directions through the channel conductance, and internal nets of a series stack carry no capacitance
    # at all, so block relaxation across such a cut converges slowly or not at all. A cut through a gate
    # is one-directional (no gate current in the level-1 model) and relaxes in one sweep.
    if keep_channels:
        for el in elements:
            if _kind(el) == "Mosfet":
                b = el["Mosfet"]
                if b["d"] > 0 and b["s"] > 0 and b["d"] not in held and b["s"] not in held:
                    uf.union(b["d"], b["s"])
    enforced = 0
    name_to_net = {nm: i + 1 for i, nm in enumerate(names)}
    for group in feedback_nets or []:
        ids = [name_to_net[g] for g in group if g in name_to_net and name_to_net[g] not in held]
        for a in ids[1:]:
            uf.union(ids[0], a)
        enforced += 1 if len(ids) > 1 else 0
    free = [v for v in range(1, n + 1) if v not in held]
    reps = sorted({uf.find(v) for v in free})
    members: dict[int, list[int]] = {r: [] for r in reps}
    for v in free:
        members[uf.find(v)].append(v)
    adj: list[dict[int, float]] = [dict() for _ in range(n + 1)]
    for el in elements:
        t = [uf.find(x) for x in _terminals(el) if x > 0 and x not in held]
        # with whole channels a transistor only contributes its gate edge, the cheapest place to cut
        w = (1.0 if keep_channels else 10.0) if _kind(el) == "Mosfet" else 5.0
        for i in range(len(t)):
            for j in range(i + 1, len(t)):
                if t[i] != t[j]:
                    adj[t[i]][t[j]] = adj[t[i]].get(t[j], 0.0) + w
                    adj[t[j]][t[i]] = adj[t[j]].get(t[i], 0.0) + w
    k_eff = max(1, min(k, len(reps)))
    if method == "auto":
        try:
            import pymetis  # noqa: F401

            method = "metis"
        except ImportError:
            method = "spectral" if len(reps) <= 50_000 else "bisect"
    rep_part: dict[int, int] = {}
    if k_eff == 1:
        rep_part = {r: 0 for r in reps}
    elif method == "metis":
        rep_part = _partition_metis(adj, reps, k_eff)
    elif method in ("spectral", "bisect"):
        _recursive_bisect(adj, reps, k_eff, 0, rep_part, spectral=(method == "spectral"))
    else:
        raise ValueError(f"Unknown method: {method}. Use 'metis', 'spectral', 'bisect' or 'auto'.")
    owner = {v: rep_part[uf.find(v)] for v in free}

    result = PartitionResult(method=method, feedback_groups_enforced=enforced)
    result.net_assignment = {names[v - 1]: p for v, p in owner.items()}
    ic = {int(node): float(val) for node, val in flat.get("initial_conditions", [])}
    # one pass over the elements: which partitions take each (every partition that owns one of its current-carrying
    # terminals), and which sources hold which replicated net
    cut_elements = 0
    chosen_by_part: list[list[int]] = [[] for _ in range(k_eff)]
    terminals = [_terminals(el) for el in elements]
    holders: dict[int, list[int]] = {}
    for idx, el in enumerate(elements):
        ps = {owner[x] for x in _current_terminals(el) if x in owner}
        cut_elements += 1 if len(ps) > 1 else 0
        for p in ps:
            chosen_by_part[p].append(idx)
        if "VoltageSource" in el:
            b = el["VoltageSource"]
            if b["neg"] == 0 and b["pos"] in held:
                holders.setdefault(b["pos"], []).append(idx)
            elif b["pos"] == 0 and b["neg"] in held:
                holders.setdefault(b["neg"], []).append(idx)
    own_by_part: list[list[int]] = [[] for _ in range(k_eff)]
    for v in free:
        own_by_part[owner[v]].append(v)
    for p in range(k_eff):
        own = own_by_part[p]
        chosen = chosen_by_part[p]
        touched: list[int] = []
        seen = set(own)
        for idx in chosen:
            for x in terminals[idx]:
                if x > 0 and x not in seen:
                    seen.add(x)
                    touched.append(x)
        local_held = [x for x in touched if x in held]
        ghosts = [x for x in touched if x not in held]
        # sources that hold a replicated net come along
        have = set(chosen)
        for x in local_held:
            for idx in holders.get(x, ()):
                if idx not in have:
                    have.add(idx)
                    chosen.append(idx)
        chosen.sort()
        order = own + local_held + ghosts
        local = {v: i + 1 for i, v in enumerate(order)}
        part_json = {
            "name": f"{flat.get('name', 'netlist')}#p{p}",
            "num_nodes": len(order),
            "elements": [_remap(elements[i], local) for i in chosen],
            "ghost_map": [[int(_native.net_name_hash(names[v - 1])), local[v], int(owner[v])] for v in ghosts],
            "node_names": [names[v - 1] for v in order],
            "initial_conditions": [[local[v], ic[v]] for v in order if v in ic],
        }
        part = Partition(partition_id=p, device_names=[f"e{i}" for i in chosen], internal_nodes={names[v - 1] for v in own},
                         boundary_nodes={names[v - 1] for v in ghosts}, num_devices=len(chosen), netlist=part_json)
        result.partitions.append(part)
    sizes = [pt.num_devices for pt in result.partitions]
    result.balance_ratio = max(sizes) / (sum(sizes) / len(sizes)) if sum(sizes) else 0.0
    result.total_boundary_nodes = sum(pt.ghost_count for pt in result.partitions)
    result.total_cut_edges = cut_elements
    return result


def partition_netlist(netlist: Netlist, k: int, method: str = "auto", imbalance_tolerance: float = 1.05,
                      process: str = "TT", vdd: float = 1.8, temp: float = 27.0) -> PartitionResult:
    """Partitions a parsed netlist into ``k`` parts; ``result.partitions[i].netlist`` is the partition
    file for solver node ``i``. ``imbalance_tolerance`` is accepted for compatibility: the built-in
    methods split at the balanced point of their ordering."""
    del imbalance_tolerance
    if k <= 0:
        raise ValueError(f"k must be positive, got {k}")
    flat_text = netlist.flatten()
    dev_by_name = {d.name: d for d in flat_text.devices}
    groups = []
    for g in detect_feedback_loops(flat_text):  # the loops only: the star-expansion graph is not needed to partition
        nets: set[str] = set()
        for name in g:
            d = dev_by_name.get(name)
            if d is not None and len(d.nodes) >= 3:
                nets.update(x.lower() for x in (d.nodes[0], d.nodes[1]))
        groups.append(nets)
    flat = netlist.to_native(process, vdd, temp)
    result = partition_flat(flat, k, method, groups)
    # device names of the text-level netlist, by position (the native parser keeps card order)
    cards = [d for d in flat_text.devices if d.dev_type in "RCLVIDM"]
    if len(cards) == len(flat["elements"]):
        for part in result.partitions:
            part.device_names = [cards[int(n[1:])].name for n in part.device_names]
    return result
