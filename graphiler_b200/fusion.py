"""Additional fusion patterns for a compiled MP-DFG.

The reference's optimizer (python/graphiler/mpdfg_optimizer.py:4-16; src/optimizer/fusion.cpp:24-141) knows
three fusions: broadcast + add -> ``gsddmm_u_add_v_mul_alpha``, broadcast + mul + SpMMEdge ->
``gspmm_{src,dst}_mul_e_sum`` and BroadcastXType + bmm -> ``SegmentMM*``.  At its highest level the example
models still materialise (E, F) intermediates: RGCN and HGT gather node rows to edges in front of the edge-typed
linear, multiply the (E, F) message by its per-edge weight before the segment sum, HGT forms the attention score
with ``aten::mul`` + ``aten::sum`` on two gathered (E, F) tensors, and GAT runs SDDMM, activation, softmax and
SpMM as four operators.

``extra_fusion`` rewrites the TorchScript graph of an already optimised MP-DFG, in place, with four more
patterns whose targets this library registers next to the reference's fifteen operators:

  SegmentMMEdge(BroadcastSrcNode(x, g), w, g)                         -> SegmentMMEdgeSrc(x, w, g)
  sum(mul(BroadcastSrcNode(a, g), BroadcastDstNode(b, g)), [1], True) -> gsddmm_u_dot_v(a, b, 1, g)
  sum(mul(e, BroadcastDstNode(b, g)), [1], True)                      -> gsddmm_e_dot_v(e, b, 1, g)
  SpMMEdge(mul(a, b), ..., g)                                         -> SpMMEdgeMul(a, b, g)
  gspmm_src_mul_e_sum(z, SegmentSoftmax(leaky_relu[_](gsddmm_u_add_v_mul_alpha(l, r, _, g), s), 1, None, g), ..., g)
                                                                      -> gat_fused(l, r, z, s, g)

A pattern is applied only when every intermediate value it removes has no other reader and all operators
involved name the same graph handle.  Shapes are unknown at rewrite time, so the two targets that could meet
shapes their kernels do not cover (``gsddmm_e_dot_v``, ``SpMMEdgeMul``) take the unfused route at run time
instead of raising.

    mpdfg = mpdfg_builder(message, reduce, update, opt_level=2)     # the reference's own call
    graphiler_b200.fusion.extra_fusion(mpdfg)                       # counts of applied patterns
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

_OPS = "my_ops::"


def _graph_of(obj):
    fwd = getattr(obj, "forward", obj)
    return getattr(fwd, "graph", fwd)


def _produced_by(value, kind: str):
    node = value.node()
    return node if node.kind() == kind else None


def _same_node(a, b) -> bool:
    # Python wrappers of one IR node are distinct objects: compare the ids of the values they define
    return a.outputsSize() > 0 and b.outputsSize() > 0 and a.outputsAt(0).unique() == b.outputsAt(0).unique()


def _only_reader(value, reader) -> bool:
    uses = value.uses()
    return len(uses) == 1 and _same_node(uses[0].user, reader)


def _const(value):
    node = value.node()
    if node.kind() != "prim::Constant":
        raise LookupError
    return value.toIValue()


def _is_const(value, expected) -> bool:
    try:
        got = _const(value)
    except LookupError:
        return False
    return got is expected if expected is None or isinstance(expected, bool) else got == expected


def _int_list(value) -> Optional[List[int]]:
    node = value.node()
    if node.kind() == "prim::ListConstruct":
        try:
            return [int(_const(v)) for v in node.inputs()]
        except (LookupError, TypeError):
            return None
    try:
        got = _const(value)
    except LookupError:
        return None
    return list(got) if isinstance(got, (list, tuple)) else None


def _is_tensor(value) -> bool:
    return value.type().kind() == "TensorType"


def _replace(graph, old_node, kind: str, inputs) -> None:
    new = graph.create(kind, list(inputs), 1)
    new.insertBefore(old_node)
    new.output().setType(old_node.output().type())
    old_node.output().replaceAllUsesWith(new.output())
    old_node.destroy()


def _erase_dead(*nodes) -> None:
    """Destroy, consumer first, those of ``nodes`` whose results nobody reads any more.  Dead-code elimination keeps
    custom operators (registered without alias information, so possibly side-effecting in its eyes); the ones a
    pattern has just bypassed are known to be pure or to write only into the bypassed chain."""
    for node in nodes:
        if all(len(o.uses()) == 0 for o in node.outputs()):
            node.destroy()


def _handle(node):
    return list(node.inputs())[-1]


def _same_handle(*nodes) -> bool:
    first = _handle(nodes[0]).unique()
    return all(_handle(n).unique() == first for n in nodes[1:])


def _fuse_gather_into_typed_linear(graph) -> int:
    done = 0
    for node in list(graph.nodes()):
        if node.kind() != _OPS + "SegmentMMEdge":
            continue
        x, w, g = node.inputs()
        src = _produced_by(x, _OPS + "BroadcastSrcNode")
        if src is None or not _same_handle(node, src):
            continue
        _replace(graph, node, _OPS + "SegmentMMEdgeSrc", [list(src.inputs())[0], w, g])
        _erase_dead(src)
        done += 1
    return done


def _fuse_dot(graph) -> Dict[str, int]:
    done = {"gsddmm_u_dot_v": 0, "gsddmm_e_dot_v": 0}
    for node in list(graph.nodes()):
        if node.kind() != "aten::sum":
            continue
        ins = list(node.inputs())
        if len(ins) != 4 or _int_list(ins[1]) != [1] or not _is_const(ins[2], True) or not _is_const(ins[3], None):
            continue
        mul = _produced_by(ins[0], "aten::mul")
        if mul is None or not _only_reader(ins[0], node):
            continue
        a, b = list(mul.inputs())
        if not (_is_tensor(a) and _is_tensor(b)):
            continue
        for left, right in ((a, b), (b, a)):
            dst = _produced_by(right, _OPS + "BroadcastDstNode")
            if dst is None:
                continue
            g = _handle(dst)
            one = graph.insertConstant(1)
            one.node().moveBefore(node)
            src = _produced_by(left, _OPS + "BroadcastSrcNode")
            if src is not None and _same_handle(src, dst):
                _replace(graph, node, _OPS + "gsddmm_u_dot_v", [list(src.inputs())[0], list(dst.inputs())[0], one, g])
                _erase_dead(mul, src, dst)
                done["gsddmm_u_dot_v"] += 1
            else:
                _replace(graph, node, _OPS + "gsddmm_e_dot_v", [left, list(dst.inputs())[0], one, g])
                _erase_dead(mul, dst)
                done["gsddmm_e_dot_v"] += 1
            break
    return done


def _fuse_weighted_segment_sum(graph) -> int:
    done = 0
    for node in list(graph.nodes()):
        if node.kind() != _OPS + "SpMMEdge":
            continue
        ins = list(node.inputs())
        mul = _produced_by(ins[0], "aten::mul")
        if mul is None or not _only_reader(ins[0], node):
            continue
        a, b = list(mul.inputs())
        if not (_is_tensor(a) and _is_tensor(b)):
            continue
        _replace(graph, node, _OPS + "SpMMEdgeMul", [a, b, ins[-1]])
        done += 1
    return done


def _fuse_attention(graph) -> int:
    done = 0
    for node in list(graph.nodes()):
        if node.kind() != _OPS + "gspmm_src_mul_e_sum":
            continue
        ins = list(node.inputs())
        z, alpha = ins[0], ins[1]
        soft = _produced_by(alpha, _OPS + "SegmentSoftmax")
        if soft is None or not _only_reader(alpha, node) or not _same_handle(node, soft):
            continue
        s_in = list(soft.inputs())
        if not _is_const(s_in[1], 1):
            continue
        act = s_in[0].node()
        if act.kind() not in ("aten::leaky_relu_", "aten::leaky_relu", "aten::relu", "aten::relu_"):
            continue
        if not _only_reader(s_in[0], soft):
            continue
        a_in = list(act.inputs())
        add = _produced_by(a_in[0], _OPS + "gsddmm_u_add_v_mul_alpha")
        if add is None or not _only_reader(a_in[0], act) or not _same_handle(node, add):
            continue
        if act.kind().startswith("aten::relu"):
            slope = graph.insertConstant(0.0)
            slope.node().moveBefore(node)
        else:
            slope = a_in[1]
            if slope.type().kind() != "FloatType":
                continue
        l, r = list(add.inputs())[:2]
        _replace(graph, node, _OPS + "gat_fused", [l, r, z, slope, ins[-1]])
        _erase_dead(soft, act, add)
        done += 1
    return done


def extra_fusion(mpdfg) -> Dict[str, int]:
    """Apply the added patterns to ``mpdfg`` (an ``MPDFG`` of the reference's wrapper, a scripted function, or a
    ``torch.Graph``) in place and return how often each target was emitted."""
    graph = _graph_of(mpdfg)
    counts = {"SegmentMMEdgeSrc": _fuse_gather_into_typed_linear(graph)}
    counts.update(_fuse_dot(graph))
    counts["SpMMEdgeMul"] = _fuse_weighted_segment_sum(graph)
    counts["gat_fused"] = _fuse_attention(graph)
    torch._C._jit_pass_dce(graph)
    torch._C._jit_pass_lint(graph)
    return counts
