"""Pictures of a partitioning: Graphviz DOT text (always), an image when matplotlib is installed.
Counterpart of the reference's ``visualizer.py`` (``visualize_partitions``)."""
from __future__ import annotations

from typing import Optional

from .graph import build_circuit_graph
from .parser import Netlist
from .partitioner import PartitionResult

_COLOURS = ["#4e79a7", "#f28e2b", "#e15759", "#76b7b2", "#59a14f", "#edc948", "#b07aa1", "#ff9da7", "#9c755f", "#bab0ac"]


def partition_dot(netlist: Netlist, result: PartitionResult) -> str:
    """DOT text: nets coloured by owning partition, devices as boxes, ghost copies dashed."""
    flat = netlist.flatten()
    cg = build_circuit_graph(flat)
    owner = {n.lower(): p for n, p in result.net_assignment.items()}
    lines = ["graph partitions {", "  node [style=filled, fontsize=9];"]
    for net in sorted(cg.net_nodes):
        name = net[2:]
        p = owner.get(name)
        colour = _COLOURS[p % len(_COLOURS)] if p is not None else "#dddddd"
        lines.append(f'  "{net}" [label="{name}", shape=ellipse, fillcolor="{colour}"];')
    for dev in sorted(cg.device_nodes):
        lines.append(f'  "{dev}" [label="{dev[2:]}", shape=box, fillcolor="#ffffff"];')
    for a, b in cg.graph.edges():
        d, n = (a, b) if a.startswith("D:") else (b, a)
        nets = [x for x in cg.graph[d] if x.startswith("N:")]
        owners = {owner.get(x[2:]) for x in nets} - {None}
        style = "dashed" if len(owners) > 1 else "solid"
        lines.append(f'  "{d}" -- "{n}" [style={style}];')
    lines.append("}")
    return "\n".join(lines)


def visualize_partitions(netlist: Netlist, result: PartitionResult, output_path: Optional[str] = None, max_nodes: int = 400) -> str:
    """Writes ``output_path`` (``.dot`` text, or ``.png`` via matplotlib + networkx layout when
    available and the graph is small enough). Returns the path written, or the DOT text when no
    path is given."""
    dot = partition_dot(netlist, result)
    if output_path is None:
        return dot
    if output_path.endswith(".png"):
        try:
            import matplotlib

            matplotlib.use("Agg")
            import matplotlib.pyplot as plt
            import networkx as nx

            cg = build_circuit_graph(netlist.flatten())
            if cg.graph.number_of_nodes() <= max_nodes:
                owner = {n.lower(): p for n, p in result.net_assignment.items()}
                pos = nx.spring_layout(cg.graph, seed=0)
                colours = []
                for node in cg.graph.nodes():
                    p = owner.get(node[2:]) if node.startswith("N:") else None
                    colours.append(_COLOURS[p % len(_COLOURS)] if p is not None else "#dddddd")
                fig = plt.figure(figsize=(8, 6))
                nx.draw(cg.graph, pos, node_color=colours, node_size=60, width=0.5)
                fig.savefig(output_path, dpi=120)
                plt.close(fig)
                return output_path
        except Exception:
            pass
        output_path = output_path[:-4] + ".dot"
    with open(output_path, "w") as f:
        f.write(dot)
    return output_path
