"""Graph rewrites: dead-code elimination and the fusion pass.

The fusion pass reproduces the reference's three rewrites
(src/flag_dnn/graph/passes/fusion.py:40-160) with the same preconditions and
the same statistics keys, and adds two the reference cannot express: a
per-channel multiply between the convolution and the bias (a BatchNorm folded
into scale and bias) is absorbed into the fused node as a fourth input, and a
residual block's tail, relu(conv(...) + shortcut), becomes one node whose add
and ReLU run in the convolution's epilogue.
"""
from __future__ import annotations

from .ir import Graph, OpNode


def eliminate_dead_nodes(graph: Graph) -> int:
    removed = 0
    changed = True
    while changed:
        changed = False
        for node in list(graph.nodes):
            if all(graph.num_users(v) == 0 for v in node.outputs):
                graph.remove_nodes([node.id])
                removed += 1
                changed = True
    return removed


def apply_fusion_pass(graph: Graph) -> Graph:
    stats = graph.attrs.setdefault("fusion", {})
    rules = (
        (_fuse_conv_bias_relu, "conv2d_bias_activation_fused"),
        (_fold_conv_scale_bias, "conv2d_scale_bias_folded"),
        (_fold_conv_bias, "conv2d_bias_folded"),
        (_fuse_bias_relu, "bias_activation_fused"),
        (_fuse_conv_add_relu, "conv2d_residual_activation_fused"),
    )
    changed = True
    while changed:
        changed = False
        for rule, key in rules:  # long patterns first
            if rule(graph):
                stats[key] = stats.get(key, 0) + 1
                changed = True
                break
    return graph


def _single_use_producer(graph: Graph, value_id: int, op_type: str):
    node = graph.producer(value_id)
    if node is None or node.op_type != op_type:
        return None
    if len(node.outputs) != 1 or graph.num_users(value_id) != 1:
        return None
    return node


def _channel_scale_input(graph: Graph, mul_node: OpNode, conv_out_channels: int):
    """The non-conv operand of `conv * scale` if it is a per-channel vector.

    The captured ``mul`` broadcasts like ``torch.mul``: against a [N, K, H, W] convolution output only
    shapes (K, 1, 1) and (1, K, 1, 1) multiply along the channels.  A plain (K,) vector broadcasts along
    W, so it is a per-channel scale only in the degenerate case K == 1 (a one-element vector).
    """
    if len(mul_node.inputs) != 2:
        return None
    scale_id = mul_node.inputs[1]
    shape = tuple(graph.values[scale_id].spec.shape)
    k = conv_out_channels
    if shape in ((k, 1, 1), (1, k, 1, 1)) or (k == 1 and shape == (1,)):
        return scale_id
    return None


def _match_conv_chain(graph: Graph, bias_node: OpNode):
    """bias_add <- [mul <-] conv2d (no bias yet); returns (conv, mul_or_None, scale_id_or_None)."""
    if len(bias_node.inputs) != 2 or len(bias_node.outputs) != 1:
        return None
    upstream = bias_node.inputs[0]
    mul_node = _single_use_producer(graph, upstream, "mul")
    scale_id = None
    if mul_node is not None:
        conv_node = _single_use_producer(graph, mul_node.inputs[0], "conv2d")
        if conv_node is None:
            return None
        k = graph.values[conv_node.outputs[0]].spec.shape[1]
        scale_id = _channel_scale_input(graph, mul_node, k)
        if scale_id is None:
            return None
    else:
        conv_node = _single_use_producer(graph, upstream, "conv2d")
        if conv_node is None:
            return None
    if len(conv_node.inputs) != 2:
        return None
    return conv_node, mul_node, scale_id


def _fuse_conv_bias_relu(graph: Graph) -> bool:
    """conv2d -> [mul(scale) ->] bias_add -> relu | gelu.  The ReLU form is the reference's rule
    (src/flag_dnn/graph/passes/fusion.py:40-83); the GELU form has no counterpart there (the reference
    leaves conv2d(+bias) and gelu as two nodes) and becomes a fused_conv2d_bias_gelu node."""
    for act in list(graph.nodes):
        if act.op_type not in ("relu", "gelu") or len(act.inputs) != 1 or len(act.outputs) != 1:
            continue
        bias_node = _single_use_producer(graph, act.inputs[0], "bias_add")
        if bias_node is None:
            continue
        match = _match_conv_chain(graph, bias_node)
        if match is None:
            continue
        conv_node, mul_node, scale_id = match
        attrs = dict(conv_node.attrs)
        attrs.update(act.attrs)
        attrs["activation"] = act.op_type
        inputs = [conv_node.inputs[0], conv_node.inputs[1], bias_node.inputs[1]]
        doomed = [conv_node.id, bias_node.id, act.id]
        if mul_node is not None:
            inputs.append(scale_id)
            doomed.append(mul_node.id)
        kind = "fused_conv2d_bias_relu" if act.op_type == "relu" else "fused_conv2d_bias_gelu"
        fused = OpNode(id=graph.new_node_id(), op_type=kind, inputs=inputs,
                       outputs=list(act.outputs), attrs=attrs, name=kind)
        graph.replace_nodes_with(doomed, fused)
        return True
    return False


def _redirect(graph: Graph, old_value: int, new_value: int) -> None:
    if old_value in graph.outputs:
        graph.outputs = [new_value if v == old_value else v for v in graph.outputs]
        graph.values[new_value].spec = graph.values[new_value].spec.as_output()
    for user in graph.users(old_value):
        user.inputs = [new_value if v == old_value else v for v in user.inputs]


def _fold_conv_scale_bias(graph: Graph) -> bool:
    """conv2d -> mul(scale) -> bias_add with no ReLU (pre-residual convolutions)."""
    for bias_node in list(graph.nodes):
        if bias_node.op_type != "bias_add":
            continue
        match = _match_conv_chain(graph, bias_node)
        if match is None or match[1] is None:
            continue
        conv_node, mul_node, scale_id = match
        conv_out = conv_node.outputs[0]
        conv_node.inputs = [conv_node.inputs[0], conv_node.inputs[1], bias_node.inputs[1], scale_id]
        _redirect(graph, bias_node.outputs[0], conv_out)
        graph.remove_nodes([mul_node.id, bias_node.id])
        return True
    return False


def _fold_conv_bias(graph: Graph) -> bool:
    for bias_node in list(graph.nodes):
        if bias_node.op_type != "bias_add":
            continue
        match = _match_conv_chain(graph, bias_node)
        if match is None or match[1] is not None:
            continue
        conv_node = match[0]
        conv_out = conv_node.outputs[0]
        conv_node.inputs = [conv_node.inputs[0], conv_node.inputs[1], bias_node.inputs[1]]
        _redirect(graph, bias_node.outputs[0], conv_out)
        graph.remove_nodes([bias_node.id])
        return True
    return False


def _fuse_bias_relu(graph: Graph) -> bool:
    """bias_add -> relu | gelu (src/flag_dnn/graph/passes/fusion.py:129-160)."""
    for act in list(graph.nodes):
        if act.op_type not in ("relu", "gelu") or len(act.inputs) != 1 or len(act.outputs) != 1:
            continue
        bias_node = _single_use_producer(graph, act.inputs[0], "bias_add")
        if bias_node is None:
            continue
        attrs = dict(bias_node.attrs)
        attrs.update(act.attrs)
        attrs["activation"] = act.op_type
        kind = "fused_bias_relu" if act.op_type == "relu" else "fused_bias_gelu"
        fused = OpNode(id=graph.new_node_id(), op_type=kind, inputs=list(bias_node.inputs),
                       outputs=list(act.outputs), attrs=attrs, name=kind)
        graph.replace_nodes_with([bias_node.id, act.id], fused)
        return True
    return False


def _fuse_conv_add_relu(graph: Graph) -> bool:
    """relu(add(conv2d(...), shortcut)) -> fused_conv2d_bias_add_relu(x, w, shortcut[, bias[, scale]]).

    Runs after the folding rules (it is last in the rule list), so the convolution already carries
    its bias and scale.  The shortcut must have exactly the convolution's output shape and dtype.
    """
    for act in list(graph.nodes):
        if act.op_type != "relu" or len(act.inputs) != 1 or len(act.outputs) != 1:
            continue
        add_node = _single_use_producer(graph, act.inputs[0], "add")
        if add_node is None or len(add_node.inputs) != 2 or add_node.attrs.get("alpha", 1) != 1:
            continue
        for conv_slot in (0, 1):
            conv_value, other = add_node.inputs[conv_slot], add_node.inputs[1 - conv_slot]
            conv_node = _single_use_producer(graph, conv_value, "conv2d")
            if conv_node is None or conv_value == other:
                continue
            conv_spec, other_spec = graph.values[conv_value].spec, graph.values[other].spec
            if tuple(conv_spec.shape) != tuple(other_spec.shape) or conv_spec.dtype != other_spec.dtype:
                continue
            attrs = dict(conv_node.attrs)
            attrs["activation"] = "relu"
            inputs = [conv_node.inputs[0], conv_node.inputs[1], other] + list(conv_node.inputs[2:])
            fused = OpNode(id=graph.new_node_id(), op_type="fused_conv2d_bias_add_relu", inputs=inputs,
                           outputs=list(act.outputs), attrs=attrs, name="fused_conv2d_bias_add_relu")
            # the fused node stands where the add stood: both of its producers come before that
            graph.nodes.insert(graph.nodes.index(add_node), fused)
            for vid in fused.outputs:
                graph.values[vid].producer = fused.id
            graph.remove_nodes([conv_node.id, add_node.id, act.id])
            return True
    return False
