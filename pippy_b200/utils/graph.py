"""Graph utilities used by the traced front-end."""
from __future__ import annotations

import torch
import torch.fx as fx


def modify_graph_op_device(gm: torch.nn.Module, new_device: torch.device) -> None:
    """Rewrites the ``device=`` argument burned into factory ops at trace time (for example
    ``torch.ones(..., device=x.device)`` traced on CPU) so the stage can run on ``new_device``; recurses into nested
    graph modules (reference pippy/_utils.py:56-88)."""
    modified = False
    if isinstance(gm, fx.GraphModule):
        for node in gm.graph.nodes:
            if node.op == "call_function":
                if "device" in node.kwargs and node.kwargs["device"] != new_device:
                    node.update_kwarg("device", new_device)
                    modified = True
                # positional device arguments of aten ops, e.g. aten._to_copy / aten.to.device
                new_args = []
                changed = False
                for a in node.args:
                    if isinstance(a, torch.device) and a != new_device:
                        new_args.append(new_device)
                        changed = True
                    else:
                        new_args.append(a)
                if changed:
                    node.args = tuple(new_args)
                    modified = True
        if modified:
            gm.recompile()
    for child in gm.children():
        inner = getattr(child, "graph_module", None)
        if isinstance(child, fx.GraphModule):
            modify_graph_op_device(child, new_device)
        elif isinstance(inner, fx.GraphModule):
            modify_graph_op_device(inner, new_device)
