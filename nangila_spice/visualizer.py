"""Pictures of a partitioning: Graphviz DOT text (always), an image when matplotlib is installed.
Counterpart of the reference's ``visualizer.py`` (``visualize_partitions``, visualizer.py:49-196), which draws with
matplotlib only and returns nothing without it."""
from __future__ import annotations

from typing import Optional, Union

from .graph import CircuitGraph, build_circuit_graph
from .parser import Netlist
from .partitioner import PartitionResult

_COLOURS = ["#4e79a7", "#f28e2b", "#e15759", "#76b7b2", "#59a14f", "#edc948", "#b07aa1", "#ff9da7", "#9c755f", "#bab0ac"]


def _graph_of(circuit: Union[Netlist, CircuitGraph]) -> CircuitGraph:
    """The device / net graph of a netlist (flattened first), or the graph itself when one is handed over."""
    if isinstance(circuit, CircuitGraph):
        return circuit
    return build_circuit_graph(circuit.flatten())


def partition_dot(circuit: Union[Netlist, CircuitGraph], result: PartitionResult, title: Optional[str] = None, show_nets: bool = True) -> str:
    """DOT text: nets coloured by owning partition, devices as boxes (coloured when all their nets have one owner),
    connections that cross a partition boundary dashed. ``show_nets=False`` leaves the nets out and joins devices that
    share one directly, which reads better on large circuits."""
    cg = _graph_of(circuit)
    owner = {n.lower(): p for n, p in result.net_assignment.items()}

    def colour(p):
        return _COLOURS[p % len(_COLOURS)] if p is not None else "#dddddd"

    def owners_of(dev):
        return {owner.get(x[2:]) for x in cg.graph[dev] if x.startswith("N:")} - {None}

    lines = ["graph partitions {", "  node [style=filled, fontsize=9];"]
    if title:
        lines.append(f'  label="{title}"; labelloc=t;')
    if show_nets:
        for net in sorted(cg.net_nodes):
            lines.append(f'  "{net}" [label="{net[2:]}", shape=ellipse, fillcolor="{colour(owner.get(net[2:]))}"];')
    for dev in sorted(cg.device_nodes):
        own = owners_of(dev)
        lines.append(f'  "{dev}" [label="{dev[2:]}", shape=box, fillcolor="{colour(next(iter(own))) if len(own) == 1 else "#ffffff"}"];')
    if show_nets:
        for a, b in cg.graph.edges():
            d, n = (a, b) if a.startswith("D:") else (b, a)
            lines.append(f'  "{d}" -- "{n}" [style={"dashed" if len(owners_of(d)) > 1 else "solid"}];')
    else:
        seen = set()
        for net in sorted(cg.net_nodes):
            if owner.get(net[2:]) is None:
                continue  # supplies and other replicated nets would join everything to everything
            devs = sorted(cg.graph[net])
            for i in range(len(devs) - 1):
                pair = (devs[i], devs[i + 1])
                if pair not in seen:
                    seen.add(pair)
                    crossing = len(owners_of(devs[i]) | owners_of(devs[i + 1])) > 1
                    lines.append(f'  "{devs[i]}" -- "{devs[i + 1]}" [style={"dashed" if crossing else "solid"}];')
    lines.append("}")
    return "\n".join(lines)


def visualize_partitions(circuit: Union[Netlist, CircuitGraph], result: PartitionResult, output_path: Optional[str] = None,
                         title: Optional[str] = None, show_nets: bool = True, figsize: tuple = (12, 8), max_nodes: int = 400) -> str:
    """Writes ``output_path``: ``.dot`` text, or an image (any other suffix) drawn with matplotlib and a networkx layout
    when matplotlib is installed and the graph has at most ``max_nodes`` nodes; otherwise the DOT text goes to the same
    name with ``.dot``. Returns the path written, or the DOT text when no path is given. ``circuit`` is a parsed netlist
    or its ``CircuitGraph`` (the reference's first argument)."""
    dot = partition_dot(circuit, result, title=title, show_nets=show_nets)
    if output_path is None:
        return dot
    if not output_path.endswith(".dot"):
        try:
            import matplotlib

            matplotlib.use("Agg")
            import matplotlib.pyplot as plt
            import networkx as nx

            cg = _graph_of(circuit)
            graph = cg.graph if show_nets else cg.graph.subgraph(cg.device_nodes | {n for n in cg.net_nodes if n[2:] in
                                                                                   {k.lower() for k in result.net_assignment}})
            if graph.number_of_nodes() <= max_nodes:
                owner = {n.lower(): p for n, p in result.net_assignment.items()}
                pos = nx.spring_layout(graph, seed=0)
                colours = []
                for node in graph.nodes():
                    p = owner.get(node[2:]) if node.startswith("N:") else None
                    colours.append(_COLOURS[p % len(_COLOURS)] if p is not None else "#dddddd")
                fig = plt.figure(figsize=figsize)
                nx.draw(graph, pos, node_color=colours, node_size=60, width=0.5)
                if title:
                    fig.suptitle(title)
                fig.savefig(output_path, dpi=120)
                plt.close(fig)
                return output_path
        except Exception:
            pass
        output_path = output_path.rsplit(".", 1)[0] + ".dot"
    with open(output_path, "w") as f:
        f.write(dot)
    return output_path
