"""Pickling stage ``GraphModule``s by their node list instead of by generated source
(reference pippy/_IR.py:407-491).  The default ``GraphModule`` pickle re-traces generated code, which breaks on very
long graphs; this form is for shipping a stage to another process, not for long-term storage.
"""
from __future__ import annotations

from typing import Any, Dict, List

import torch
import torch.fx as fx


class _NodeReference:
    def __init__(self, name: str):
        self.name = name


class _OpReference:
    """A ``torch.ops`` overload named by namespace, op and overload (the objects themselves do not pickle)."""

    def __init__(self, qualified: str, overload: str):
        self.qualified, self.overload = qualified, overload

    def resolve(self):
        ns, name = self.qualified.split("::")
        packet = getattr(getattr(torch.ops, ns), name)
        return getattr(packet, self.overload) if self.overload else packet


def _encode_target(target):
    if isinstance(target, torch._ops.OpOverload):
        return _OpReference(target._schema.name, target._overloadname)
    if isinstance(target, torch._ops.OpOverloadPacket):
        return _OpReference(target._qualified_op_name, "")
    return target


class _LinearNodeList:
    """A graph flattened into a list of plain records; node arguments that refer to other nodes become
    :class:`_NodeReference`."""

    def __init__(self, nodes: fx.node.Node):
        self.records: List[Dict[str, Any]] = []
        for n in nodes:
            def ref(a):
                return _NodeReference(a.name) if isinstance(a, fx.Node) else a

            self.records.append({
                "op": n.op, "name": n.name, "target": _encode_target(n.target),
                "args": fx.node.map_arg(n.args, ref), "kwargs": fx.node.map_arg(n.kwargs, ref), "type": n.type,
            })

    def to_graph(self) -> fx.Graph:
        graph = fx.Graph()
        env: Dict[str, fx.Node] = {}

        def deref(a):
            return env[a.name] if isinstance(a, _NodeReference) else a

        for rec in self.records:
            args = fx.node.map_aggregate(rec["args"], deref)
            kwargs = fx.node.map_aggregate(rec["kwargs"], deref)
            target = rec["target"].resolve() if isinstance(rec["target"], _OpReference) else rec["target"]
            if rec["op"] == "output":
                node = graph.output(args[0])
            else:
                node = graph.create_node(rec["op"], target, args, kwargs, rec["name"], rec["type"])
            env[rec["name"]] = node
        return graph


def _direct_serialization_deserialize(body: Dict[str, Any], nodes: _LinearNodeList) -> fx.GraphModule:
    class _Root(torch.nn.Module):
        def __init__(self, state):
            super().__init__()
            self.__dict__ = state

    root = _Root(body)
    return fx.GraphModule(root, nodes.to_graph())


def _direct_serialization_reduce(self: fx.GraphModule):
    body = dict(self.__dict__)
    for key in ("_graph", "_code", "_lineno_map", "_prologue_start", "meta", "_tracer_cls", "_tracer_extras",
                "_replace_hooks", "_create_node_hooks", "_erase_node_hooks", "_deepcopy_hooks"):
        body.pop(key, None)
    return (_direct_serialization_deserialize, (body, _LinearNodeList(self.graph.nodes)))


def enable_direct_serialization(gm: fx.GraphModule) -> fx.GraphModule:
    """Makes ``pickle`` use the node-list form for this module's class."""
    gm.__class__.__reduce__ = _direct_serialization_reduce
    return gm
