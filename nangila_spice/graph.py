"""Circuit graph for partitioning: star expansion of the netlist hypergraph (one graph node per net,
one per device, an edge per terminal) and detection of feedback loops that must not be cut.

API counterpart: ``nangila-spice/src/nangila_spice/graph.py:30-215`` of the reference. Feedback
detection differs by design: instead of cross-coupled pairs plus three-device cycles, the loops are
the strongly connected components of the directed signal-flow graph (gate net -> drain / source
nets of every MOSFET), which finds latches and ring oscillators of any length and ignores passive
ladders.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import networkx as nx

from .parser import Device, Netlist

SUPPLY_NETS = {"0", "gnd", "vdd", "vss", "vcc", "vdd!", "gnd!"}


@dataclass
class CircuitGraph:
    graph: nx.Graph = field(default_factory=nx.Graph)
    net_nodes: set[str] = field(default_factory=set)
    device_nodes: set[str] = field(default_factory=set)
    feedback_groups: list[set[str]] = field(default_factory=list)

    @property
    def num_nets(self) -> int:
        return len(self.net_nodes)

    @property
    def num_devices(self) -> int:
        return len(self.device_nodes)

    @property
    def num_edges(self) -> int:
        return self.graph.number_of_edges()


def _connection_weight(device: Device, net_name: str) -> int:
    """Cutting a MOSFET gate connection is expensive (10), a supply connection cheap (1), the rest 5."""
    if device.dev_type == "M" and len(device.nodes) >= 2 and net_name == device.nodes[1]:
        return 10
    if net_name.lower() in SUPPLY_NETS:
        return 1
    return 5


def detect_feedback_loops(netlist: Netlist) -> list[set[str]]:
    """Sets of device names that form a signal loop (each set should stay in one partition)."""
    flow = nx.DiGraph()
    drivers: dict[str, list[str]] = {}
    for d in netlist.devices:
        if d.dev_type == "M" and len(d.nodes) >= 3:
            gate = d.nodes[1].lower()
            for out in (d.nodes[0].lower(), d.nodes[2].lower()):
                if out in SUPPLY_NETS or gate in SUPPLY_NETS:
                    continue
                flow.add_edge(gate, out)
                drivers.setdefault(out, []).append(d.name)
    groups: list[set[str]] = []
    gate_of = {d.name: d.nodes[1].lower() for d in netlist.devices if d.dev_type == "M" and len(d.nodes) >= 3}
    for comp in nx.strongly_connected_components(flow):
        if len(comp) < 2:
            continue
        devs = {name for net in comp for name in drivers.get(net, []) if gate_of.get(name) in comp}
        if len(devs) >= 2:
            groups.append(devs)
    return _merge_overlapping_groups(groups)


def _merge_overlapping_groups(groups: list[set[str]]) -> list[set[str]]:
    merged: list[set[str]] = []
    for g in groups:
        g = set(g)
        keep = []
        for m in merged:
            if m & g:
                g |= m
            else:
                keep.append(m)
        keep.append(g)
        merged = keep
    return merged


def build_circuit_graph(netlist: Netlist) -> CircuitGraph:
    """Device nodes are named ``D:<name>``, net nodes ``N:<net>``."""
    cg = CircuitGraph()
    for device in netlist.devices:
        dev_id = f"D:{device.name}"
        cg.graph.add_node(dev_id, ntype="device", dev_type=device.dev_type)
        cg.device_nodes.add(dev_id)
        for net in device.nodes:
            net_id = f"N:{net.lower()}"
            if net_id not in cg.net_nodes:
                cg.graph.add_node(net_id, ntype="net")
                cg.net_nodes.add(net_id)
            w = _connection_weight(device, net)
            if cg.graph.has_edge(dev_id, net_id):
                cg.graph[dev_id][net_id]["weight"] += w
            else:
                cg.graph.add_edge(dev_id, net_id, weight=w)
    cg.feedback_groups = detect_feedback_loops(netlist)
    return cg
