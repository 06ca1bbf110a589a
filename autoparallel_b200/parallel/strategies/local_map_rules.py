"""Strategies for ``local_map`` higher-order nodes (filled in by the collectives module)."""
import torch.fx as fx


def is_local_map_node(node: fx.Node) -> bool:
    t = node.target
    return node.op == "call_function" and type(t).__name__ in ("LocalMapHOP", "LocalMapBackwardHOP", "LocalMapAOTExportModule")


def local_map_options(mesh, node, strats):
    raise NotImplementedError("local_map nodes are not supported yet")
