"""torch.compile backend: `torch.compile(model, backend="omarchy_mac_torch")`.

Dynamo captures the model and AOTAutograd lowers it to aten graphs for forward and backward. FX passes then rewrite
those graphs to the fused `omt::` ops, and the graph runs op by op on the device:

  1. training BatchNorm2d followed by ReLU            -> omt.bn_relu_train
     training BatchNorm2d, + identity branch, ReLU    -> omt.bn_add_relu_train (the tail of a residual block)
  2. threshold_backward -> native_batch_norm_backward -> omt.bn_relu_backward (ReLU mask folded into the BN backward)
     the same where the masked gradient also feeds the identity branch -> omt.bn_add_relu_backward
  3. conv -> [eval BatchNorm] -> [ReLU]               -> omt.conv_act / omt.conv_bn_act_eval
     conv -> training BatchNorm [+ identity] [ReLU]   -> omt.conv_bn_train (batch statistics reduced in the conv epilogue)
  +  add(convolution_backward(...)[0], g) with g a gradient nobody else reads -> omt.conv_backward_acc (the input
     gradient is accumulated into g by the conv epilogue: the joins of residual branches in the backward graph)

  4. chains of elementwise ops (add/mul/relu/sigmoid/hardswish/..., their backward forms, scalars folded in) that only
     feed one another                                   -> omt.fused_pointwise (one kernel, one pass over memory)

  6. num_batches_tracked + 1 of all BatchNorm layers -> one aten._foreach_add (one launch instead of one per layer)

  5. _log_softmax -> nll_loss_forward (what F.cross_entropy lowers to) -> omt.softmax_nll, and in the backward graph
     nll_loss_backward -> _log_softmax_backward_data -> omt.softmax_nll_backward: the loss is two launches per step

These are passes 1-4 of the reference's omarchy_mac_torch/compile.py:69-161, 256-336. Its pass 4 generates shader source
for every chain; here the chain is encoded as a small program string that one ahead-of-time interpreter kernel runs
(csrc/pointwise.cu). Every fused op has a composite definition in plain aten ops, so a rewritten graph is always
correct, on any device. OMARCHY_MAC_TORCH_COMPILE_DEBUG=1 prints what each pass did."""

import math
import operator
import os

import torch
from torch._dynamo import register_backend
from torch._dynamo.backends.common import aot_autograd
from torch.fx import Node

from omarchy_mac_torch_b200.native import DEVICE

aten = torch.ops.aten
omt = torch.ops.omt
_DEBUG = os.environ.get("OMARCHY_MAC_TORCH_COMPILE_DEBUG", "0") == "1"
_ANY_DEVICE = False  # tests flip this to exercise the passes on CPU graphs through the composite implementations


def _meta(n):
    return n.meta.get("val") if isinstance(n, Node) else None


def _f32_4d(n):
    v = _meta(n)
    return (isinstance(v, torch.Tensor) and v.dtype == torch.float32 and v.dim() == 4 and (_ANY_DEVICE or v.device.type == DEVICE))


def _is(n, target):
    return isinstance(n, Node) and n.op == "call_function" and n.target is target


def _items(n):
    """index -> getitem node, for a node with tuple output"""
    return {u.args[1]: u for u in n.users if _is(u, operator.getitem)}


def _sole_user(n):
    users = list(n.users)
    return users[0] if len(users) == 1 else None


def _getitem_after(graph, anchor, src, index, meta):
    with graph.inserting_before(anchor):
        node = graph.call_function(operator.getitem, (src, index))
    node.meta = dict(meta)
    return node


def _swap_tuple_node(graph, old, new):
    """Re-point every getitem of `old` at `new` (same indices) and drop `old`."""
    for idx, gi in _items(old).items():
        gi.replace_all_uses_with(_getitem_after(graph, gi, new, idx, gi.meta))
        graph.erase_node(gi)
    graph.erase_node(old)


def fuse_bn_relu(graph):
    done = 0
    for bn in list(graph.nodes):
        if not _is(bn, aten._native_batch_norm_legit_functional.default):
            continue
        x, w, b, rm, rv, training, momentum, eps = bn.args[:8]
        if not training or None in (w, b, rm, rv) or not _f32_4d(x):
            continue
        y = _items(bn).get(0)
        relu = _sole_user(y) if y is not None else None
        if not _is(relu, aten.relu.default):
            continue
        with graph.inserting_before(bn):
            fused = graph.call_function(omt.bn_relu_train.default, (x, w, b, rm, rv, momentum, eps))
        relu.replace_all_uses_with(_getitem_after(graph, relu, fused, 0, relu.meta))
        graph.erase_node(relu)
        graph.erase_node(y)
        _swap_tuple_node(graph, bn, fused)
        done += 1
    return done


def _same_shape(a, b):
    va, vb = _meta(a), _meta(b)
    return isinstance(va, torch.Tensor) and isinstance(vb, torch.Tensor) and va.shape == vb.shape and va.dtype == vb.dtype


def fuse_bn_add_relu(graph):
    """bn(x) + other -> relu, with the BatchNorm output and the sum used nowhere else."""
    done = 0
    for bn in list(graph.nodes):
        if not _is(bn, aten._native_batch_norm_legit_functional.default):
            continue
        x, w, b, rm, rv, training, momentum, eps = bn.args[:8]
        if not training or None in (w, b, rm, rv) or not _f32_4d(x):
            continue
        y = _items(bn).get(0)
        add = _sole_user(y) if y is not None else None
        if not _is(add, aten.add.Tensor) or len(add.args) != 2 or add.kwargs.get("alpha", 1) != 1:
            continue
        other = add.args[1] if add.args[0] is y else add.args[0]
        if other is y or not isinstance(other, Node) or not _same_shape(other, y):
            continue
        relu = _sole_user(add)
        if not _is(relu, aten.relu.default):
            continue
        # `other` may be computed after the BatchNorm (a downsample branch): the fused node goes where the add was, so every
        # other consumer of the BatchNorm's outputs (batch statistics, running statistics) has to come after that point
        order = {n: i for i, n in enumerate(graph.nodes)}
        rest = {idx: gi for idx, gi in _items(bn).items() if idx != 0}
        if any(order[u] < order[add] for gi in rest.values() for u in gi.users):
            continue
        with graph.inserting_before(add):
            fused = graph.call_function(omt.bn_add_relu_train.default, (x, other, w, b, rm, rv, momentum, eps))
        relu.replace_all_uses_with(_getitem_after(graph, relu, fused, 0, relu.meta))
        for idx, gi in rest.items():
            gi.replace_all_uses_with(_getitem_after(graph, relu, fused, idx, gi.meta))
        for dead in [relu, add, y] + list(rest.values()) + [bn]:
            graph.erase_node(dead)
        done += 1
    return done


def fuse_bn_add_relu_backward(graph):
    """native_batch_norm_backward of a ReLU-masked gradient whose masked form is used elsewhere too (the identity branch)."""
    done = 0
    for bw in list(graph.nodes):
        if not _is(bw, aten.native_batch_norm_backward.default):
            continue
        g, x, w, _rm, _rv, mean, invstd, train, _eps, mask = bw.args[:10]
        if not train or w is None or not _f32_4d(x):
            continue
        if not (_is(g, aten.threshold_backward.default) and g.args[2] == 0 and len(g.users) > 1):
            continue
        gout, y = g.args[0], g.args[1]
        if not _same_shape(y, x):
            continue
        with graph.inserting_before(g):
            fused = graph.call_function(omt.bn_add_relu_backward.default, (gout, x, y, w, mean, invstd, list(mask)))
        with graph.inserting_after(fused):
            dres = graph.call_function(operator.getitem, (fused, 3))
        dres.meta = dict(g.meta)
        for idx, gi in _items(bw).items():
            gi.replace_all_uses_with(_getitem_after(graph, gi, fused, idx, gi.meta))
            graph.erase_node(gi)
        graph.erase_node(bw)
        g.replace_all_uses_with(dres)
        graph.erase_node(g)
        done += 1
    return done


def fuse_bn_relu_backward(graph):
    done = 0
    for bw in list(graph.nodes):
        if not _is(bw, aten.native_batch_norm_backward.default):
            continue
        g, x, w, _rm, _rv, mean, invstd, train, _eps, mask = bw.args[:10]
        if not train or w is None or not _f32_4d(x):
            continue
        if not (_is(g, aten.threshold_backward.default) and g.args[2] == 0 and len(g.users) == 1):
            continue
        gout, y = g.args[0], g.args[1]
        with graph.inserting_before(bw):
            fused = graph.call_function(omt.bn_relu_backward.default, (gout, x, y, w, mean, invstd, list(mask)))
        _swap_tuple_node(graph, bw, fused)
        graph.erase_node(g)
        done += 1
    return done


def _fresh_gradient(n):
    """A tensor this graph produced for exactly one consumer, so it may be accumulated into in place."""
    if not (_is(n, operator.getitem) and len(n.users) == 1):
        return False
    src, idx = n.args
    return ((_is(src, omt.bn_add_relu_backward.default) and idx == 3) or (_is(src, aten.convolution_backward.default) and idx == 0)
            or (_is(src, omt.conv_backward_acc.default) and idx == 0) or (_is(src, omt.bn_relu_backward.default) and idx == 0)
            or (_is(src, omt.bn_add_relu_backward.default) and idx == 0))


def fuse_dgrad_accumulate(graph):
    done = 0
    for add in list(graph.nodes):
        if not _is(add, aten.add.Tensor) or len(add.args) != 2 or add.kwargs.get("alpha", 1) != 1:
            continue
        for a, b in ((add.args[0], add.args[1]), (add.args[1], add.args[0])):
            if not (_is(a, operator.getitem) and a.args[1] == 0 and len(a.users) == 1 and _is(a.args[0], aten.convolution_backward.default)):
                continue
            cb = a.args[0]
            gy, x, w, _bias_sizes, stride, padding, dilation, transposed, _outpad, groups, mask = cb.args[:11]
            if transposed or groups != 1 or list(dilation) != [1, 1] or not mask[0] or mask[2] or not _f32_4d(x):
                continue
            if len(set(stride)) != 1 or len(set(padding)) != 1 or a is b or not _fresh_gradient(b) or not _same_shape(a, b):
                continue
            order = {n: i for i, n in enumerate(graph.nodes)}
            others = {idx: gi for idx, gi in _items(cb).items() if idx != 0}
            if any(order[u] < order[add] for gi in others.values() for u in gi.users):
                continue
            with graph.inserting_before(add):
                fused = graph.call_function(omt.conv_backward_acc.default, (gy, x, w, b, list(stride), list(padding), bool(mask[1])))
            add.replace_all_uses_with(_getitem_after(graph, add, fused, 0, add.meta))
            for idx, gi in others.items():
                if idx == 1:
                    gi.replace_all_uses_with(_getitem_after(graph, add, fused, 1, gi.meta))
            for dead in [add, a] + list(others.values()) + [cb]:
                graph.erase_node(dead)
            done += 1
            break
    return done


def _dense_conv(n):
    if not _is(n, aten.convolution.default):
        return False
    x, w, _b, stride, padding, dilation, transposed, _outpad, groups = n.args[:9]
    wv = _meta(w)
    return (_f32_4d(x) and not transposed and groups == 1 and list(dilation) == [1, 1] and wv is not None and wv.shape[2] == wv.shape[3]
            and len(set(stride)) == 1 and len(set(padding)) == 1)


def fuse_conv_epilogues(graph):
    done = 0
    for conv in list(graph.nodes):
        if not _dense_conv(conv):
            continue
        x, w, b, stride, padding = conv.args[:5]
        nxt = _sole_user(conv)
        if nxt is None:
            continue
        if _is(nxt, aten._native_batch_norm_legit_no_training.default) and nxt.args[0] is conv:
            _, bw, bb, rm, rv, _mom, eps = nxt.args[:7]
            outs = _items(nxt)
            if None in (bw, bb, rm, rv) or set(outs) != {0}:
                continue
            y = outs[0]
            relu = _sole_user(y)
            act = 1 if _is(relu, aten.relu.default) else 0
            last = relu if act else y
            with graph.inserting_before(conv):
                fused = graph.call_function(omt.conv_bn_act_eval.default, (x, w, b, bw, bb, rm, rv, eps, list(stride), list(padding), act))
            fused.meta = dict(last.meta)
            last.replace_all_uses_with(fused)
            for dead in ([relu] if act else []) + [y, nxt, conv]:
                graph.erase_node(dead)
            done += 1
        elif _is(nxt, aten.relu.default):
            with graph.inserting_before(conv):
                fused = graph.call_function(omt.conv_act.default, (x, w, b, list(stride), list(padding), 1))
            fused.meta = dict(nxt.meta)
            nxt.replace_all_uses_with(fused)
            graph.erase_node(nxt)
            graph.erase_node(conv)
            done += 1
    return done


def fuse_conv_bn_train(graph):
    """A dense conv whose output feeds a training BatchNorm (already rewritten to omt.bn_relu_train / omt.bn_add_relu_train by
    the passes above, or still the plain aten op): one op, so that the conv epilogue can reduce the batch statistics. The
    conv output stays an output of the fused op (the backward graph keeps it)."""
    done = 0
    for bn in list(graph.nodes):
        if _is(bn, omt.bn_relu_train.default):
            x, res, (w, b, rm, rv, momentum, eps), act = bn.args[0], None, bn.args[1:7], 1
        elif _is(bn, omt.bn_add_relu_train.default):
            x, res, (w, b, rm, rv, momentum, eps), act = bn.args[0], bn.args[1], bn.args[2:8], 1
        elif _is(bn, aten._native_batch_norm_legit_functional.default):
            x, res, (w, b, rm, rv, training, momentum, eps), act = bn.args[0], None, bn.args[1:8], 0
            if not training or None in (w, b, rm, rv):
                continue
        else:
            continue
        if not _dense_conv(x) or res is x:
            continue
        order = {n: i for i, n in enumerate(graph.nodes)}
        if any(order[u] < order[bn] for u in x.users):  # every other reader of the conv output has to come after the fused op
            continue
        cx, cw, cb, stride, padding = x.args[:5]
        with graph.inserting_before(bn):
            fused = graph.call_function(omt.conv_bn_train.default, (cx, cw, cb, list(stride), list(padding), res, w, b, rm, rv, momentum, eps, act))
            yconv = graph.call_function(operator.getitem, (fused, 0))
        yconv.meta = dict(x.meta)
        for idx, gi in _items(bn).items():
            gi.replace_all_uses_with(_getitem_after(graph, bn, fused, idx + 1, gi.meta))
            graph.erase_node(gi)
        graph.erase_node(bn)
        x.replace_all_uses_with(yconv)
        graph.erase_node(x)
        done += 1
    return done


# ---- pass 4: pointwise chains ----------------------------------------------------------------------------------------------
# aten op -> (mnemonic of csrc/ext/fused.cpp's program text, operand builder). The builder gets the call's positional
# operands (already turned into operand tokens) and kwargs and returns the three operand tokens of the instruction;
# `lit(x)` interns a number. Same op coverage as the reference's table (compile.py:176-222) plus the hard-swish family.
def _pw_table():
    def binary_alpha(a, kw, lit):
        return a[0], a[1], lit(kw.get("alpha", 1))

    def binary(a, kw, lit):
        return a[0], a[1], a[0]

    def unary(a, kw, lit):
        return a[0], a[0], a[0]

    def clamp(a, kw, lit):
        lo = a[1] if len(a) > 1 and a[1] is not None else lit(-math.inf)
        hi = a[2] if len(a) > 2 and a[2] is not None else lit(math.inf)
        return a[0], lo, hi

    def gelu(name):
        return lambda kw: name + ("_tanh" if kw.get("approximate", "none") == "tanh" else "")

    t = {
        aten.add.Tensor: ("add", binary_alpha), aten.sub.Tensor: ("sub", binary_alpha), aten.add.Scalar: ("add", binary_alpha),
        aten.sub.Scalar: ("sub", binary_alpha), aten.rsub.Scalar: ("rsub", binary_alpha),
        aten.mul.Tensor: ("mul", binary), aten.div.Tensor: ("div", binary), aten.mul.Scalar: ("mul", binary), aten.div.Scalar: ("div", binary),
        aten.maximum.default: ("max", binary), aten.minimum.default: ("min", binary), aten.pow.Tensor_Scalar: ("pow", binary),
        aten.sigmoid_backward.default: ("sigmoid_bwd", binary), aten.tanh_backward.default: ("tanh_bwd", binary),
        aten.silu_backward.default: ("silu_bwd", binary), aten.hardswish_backward.default: ("hardswish_bwd", binary),
        aten.hardsigmoid_backward.default: ("hardsigmoid_bwd", binary),
        aten.threshold_backward.default: ("threshold_bwd", lambda a, kw, lit: (a[0], a[1], a[2])),
        aten.clamp.default: ("clamp", clamp),
        aten.gelu.default: (gelu("gelu"), unary), aten.gelu_backward.default: (lambda kw: gelu("gelu")(kw) + "_bwd", binary),
    }
    for op, name in ((aten.neg, "neg"), (aten.relu, "relu"), (aten.exp, "exp"), (aten.log, "log"), (aten.sqrt, "sqrt"), (aten.rsqrt, "rsqrt"),
                     (aten.reciprocal, "recip"), (aten.abs, "abs"), (aten.tanh, "tanh"), (aten.sigmoid, "sigmoid"), (aten.silu, "silu"),
                     (aten.hardswish, "hardswish"), (aten.hardsigmoid, "hardsigmoid")):
        t[op.default] = (name, unary)
    return t


_PW = _pw_table()
_PW_KWARGS = {aten.gelu.default: {"approximate"}, aten.gelu_backward.default: {"approximate"}}
_PW_MAX_INPUTS, _PW_MAX_INSTR, _PW_MAX_LITERALS = 6, 24, 24  # limits of the interpreter kernel (include/omt_b200.h)
_PW_SCALAR_ONLY = {aten.pow.Tensor_Scalar: (1,), aten.threshold_backward.default: (2,), aten.clamp.default: (1, 2)}  # operands that must be numbers


def _f32_dev(n):
    v = _meta(n)
    return isinstance(v, torch.Tensor) and v.dtype == torch.float32 and (_ANY_DEVICE or v.device.type == DEVICE)


def _pointwise_ok(n):
    if n.op != "call_function" or n.target not in _PW or not _f32_dev(n) or _meta(n).dim() > 8 or _meta(n).numel() == 0:
        return False
    for k, a in enumerate(n.args):
        if isinstance(a, Node):
            if not _f32_dev(a) or k in _PW_SCALAR_ONLY.get(n.target, ()):
                return False
        elif isinstance(a, bool) or not (isinstance(a, (int, float)) or a is None):
            return False
        elif a is None and n.target is not aten.clamp.default:
            return False
    return set(n.kwargs) <= (_PW_KWARGS.get(n.target, set()) | {"alpha"}) and not isinstance(n.kwargs.get("alpha", 1), Node)


def fuse_pointwise(graph):
    """Greedy chains: a node joins the group of a producer whose only user it is and whose shape it has (so nothing but the
    chain's last value leaves it), as long as the group stays within the kernel's limits."""
    group_of, groups = {}, []
    for n in graph.nodes:
        if not _pointwise_ok(n):
            continue
        shape = tuple(_meta(n).shape)
        target = None
        for a in n.args:
            if isinstance(a, Node) and a in group_of and len(a.users) == 1 and tuple(_meta(a).shape) == shape:
                target = group_of[a]
                break
        if target is not None:
            g = groups[target]
            external = {a for m in g + [n] for a in m.args if isinstance(a, Node) and a not in g and a is not n}
            if len(external) > _PW_MAX_INPUTS or len(g) + 1 > _PW_MAX_INSTR:
                target = None
        if target is None:
            groups.append([n])
            group_of[n] = len(groups) - 1
        else:
            groups[target].append(n)
            group_of[n] = target
    done = 0
    for g in groups:
        if len(g) < 2:
            continue
        members, inputs, literals, instrs = set(g), [], [], []

        def lit(v):
            v = float(v)
            text = "nan" if math.isnan(v) else ("inf" if v == math.inf else ("-inf" if v == -math.inf else v.hex()))
            if text not in literals:
                literals.append(text)
            return f"#{literals.index(text)}"

        for m in g:
            for a in m.args:
                if isinstance(a, Node) and a not in members and a not in inputs:
                    inputs.append(a)
        token = {a: f"v{i}" for i, a in enumerate(inputs)}
        for j, m in enumerate(g):
            name, build = _PW[m.target]
            if callable(name):
                name = name(m.kwargs)
            ops = [token[a] if isinstance(a, Node) else (None if a is None else lit(a)) for a in m.args]
            a, b, c = build(ops, m.kwargs, lit)
            instrs.append(f"{name},{a},{b},{c}")
            token[m] = f"t{j}"
        if len(literals) > _PW_MAX_LITERALS or not inputs:
            continue
        program = f"pw1|{len(inputs)}|{';'.join(instrs)}|{','.join(literals)}"
        last = g[-1]
        with graph.inserting_before(last):
            fused = graph.call_function(omt.fused_pointwise.default, (program, list(inputs)))
        fused.meta = dict(last.meta)
        last.replace_all_uses_with(fused)
        for m in reversed(g):
            graph.erase_node(m)
        done += 1
    return done


def _f32_2d(n):
    v = _meta(n)
    return isinstance(v, torch.Tensor) and v.dtype == torch.float32 and v.dim() == 2 and (_ANY_DEVICE or v.device.type == DEVICE)


def fuse_softmax_nll(graph):
    """Pass 5: the two halves of F.cross_entropy on a [batch, classes] matrix, forward and backward."""
    done = 0
    order = {n: i for i, n in enumerate(graph.nodes)}
    for nll in list(graph.nodes):
        if _is(nll, aten.nll_loss_forward.default):
            lp, target, weight, reduction, ignore = nll.args[:5]
            if not (_is(lp, aten._log_softmax.default) and _f32_2d(lp) and lp.args[1] in (1, -1) and not lp.args[2]):
                continue
            # the fused op takes the place of _log_softmax (other readers of logp, e.g. the copy saved for backward, may come
            # before nll_loss_forward), so its other operands must exist by then
            if any(isinstance(a, Node) and order[a] > order[lp] for a in (target, weight)):
                continue
            with graph.inserting_before(lp):
                fused = graph.call_function(omt.softmax_nll.default, (lp.args[0], target, weight, reduction, ignore))
            items = _items(nll)
            for idx, new_idx in ((0, 0), (1, 2)):
                gi = items.get(idx)
                if gi is not None:
                    gi.replace_all_uses_with(_getitem_after(graph, gi, fused, new_idx, gi.meta))
                    graph.erase_node(gi)
            graph.erase_node(nll)
            lp.replace_all_uses_with(_getitem_after(graph, lp, fused, 1, lp.meta))
            graph.erase_node(lp)
            done += 1
        elif _is(nll, aten.nll_loss_backward.default):
            g, lp, target, weight, reduction, ignore, tw = nll.args[:7]
            user = _sole_user(nll)
            # nll_loss_backward is the gradient of logp; when the only reader is a _log_softmax_backward_data taking it as its
            # gradient, that op's `output` operand is logp itself (possibly through detach nodes): the chain rule of the pair
            if not (_is(user, aten._log_softmax_backward_data.default) and user.args[0] is nll and _f32_2d(lp) and _meta(user.args[1]) is not None
                    and _meta(user.args[1]).shape == _meta(lp).shape and user.args[2] in (1, -1) and user.args[3] == torch.float32):
                continue
            with graph.inserting_before(user):
                fused = graph.call_function(omt.softmax_nll_backward.default, (g, lp, target, weight, reduction, ignore, tw))
            fused.meta = dict(user.meta)
            user.replace_all_uses_with(fused)
            graph.erase_node(user)
            graph.erase_node(nll)
            done += 1
    return done


def fuse_step_counters(graph):
    """Pass 6: `num_batches_tracked + 1` of every BatchNorm layer (an int64 scalar graph input each) as one _foreach_add."""
    adds = []
    for n in graph.nodes:
        if not (_is(n, aten.add.Tensor) and len(n.args) == 2 and n.args[1] == 1 and not n.kwargs):
            continue
        src, v = n.args[0], _meta(n.args[0])
        if (isinstance(src, Node) and src.op == "placeholder" and isinstance(v, torch.Tensor) and v.dtype == torch.int64 and v.dim() == 0
                and (_ANY_DEVICE or v.device.type == DEVICE)):
            adds.append(n)
    if len(adds) < 2:
        return 0
    with graph.inserting_before(adds[0]):  # every operand is a graph input, so the first add's place is as good as any
        fused = graph.call_function(aten._foreach_add.Scalar, ([n.args[0] for n in adds], 1))
    for i, n in enumerate(adds):
        n.replace_all_uses_with(_getitem_after(graph, n, fused, i, n.meta))
        graph.erase_node(n)
    return len(adds)


def rewrite(gm):
    """Apply the passes to a GraphModule in place; returns {pass: rewrites}."""
    g = gm.graph
    stats = {"bn_relu": fuse_bn_relu(g), "bn_add_relu": fuse_bn_add_relu(g), "bn_relu_backward": fuse_bn_relu_backward(g),
             "bn_add_relu_backward": fuse_bn_add_relu_backward(g), "conv_epilogue": fuse_conv_epilogues(g),
             "conv_bn_train": fuse_conv_bn_train(g), "dgrad_accumulate": fuse_dgrad_accumulate(g)}
    stats["softmax_nll"] = fuse_softmax_nll(g)
    stats["step_counters"] = fuse_step_counters(g)
    stats["pointwise"] = fuse_pointwise(g)
    g.eliminate_dead_code()
    g.lint()
    gm.recompile()
    return stats


def _compile(gm, example_inputs):
    stats = rewrite(gm)
    if _DEBUG:
        print("[omarchy-mac-torch compile]", stats)
    from functorch.compile import make_boxed_func
    return make_boxed_func(gm.forward)


backend = aot_autograd(fw_compiler=_compile, bw_compiler=_compile, inference_compiler=_compile)


def compile_regions(model, regions=None):
    """Compile a model region by region instead of as one graph, in place, and return the model.

    A whole model compiled at once has ONE backward graph, so every parameter's gradient becomes visible to autograd hooks
    when that graph ends: a data-parallel wrapper that reduces gradient buckets from such hooks (omarchy_mac_torch_b200.dp)
    could only start its all-reduces after the last backward kernel. Compiled region by region (for a residual network: the
    stem and a few groups of blocks), the backward graphs run one after the other and each region's gradients arrive as soon
    as its own graph is done, so the reductions of the last layers' buckets run underneath the backward of the earlier
    layers. The rewrites of this backend never cross a block boundary, so nothing is lost; every region costs a fraction of a
    millisecond of host time per step, which is why the regions are a handful and not every block.

    `regions` lists (parent module, child name) pairs and (nn.Sequential, (start, stop)) pairs, the latter covering the
    Sequential completely and in order; by default the model's own `compile_regions()` method supplies them. Parameter
    names do not change."""
    if regions is None:
        regions = model.compile_regions()
    groups = {}
    for parent, what in regions:
        if isinstance(what, str):
            child = getattr(parent, what)
            if isinstance(child, torch.nn.Sequential):  # as one slice over the whole of it (below)
                groups.setdefault(id(child), (child, []))[1].append((0, len(child), torch.compile(torch.nn.Sequential(*list(child)), backend=DEVICE)))
            else:  # the module stays where it is, under its name; its forward runs compiled
                fn = torch.compile(type(child).forward, backend=DEVICE)
                child.forward = (lambda *a, _m=child, _f=fn, **k: _f(_m, *a, **k))
        else:
            start, stop = what
            groups.setdefault(id(parent), (parent, []))[1].append((start, stop, torch.compile(torch.nn.Sequential(*list(parent)[start:stop]), backend=DEVICE)))
    for parent, parts in groups.values():
        parts.sort(key=lambda p: p[0])
        assert parts[0][0] == 0 and parts[-1][1] == len(parent) and all(a[1] == b[0] for a, b in zip(parts, parts[1:])), \
            "the slices must cover the Sequential completely and in order"
        chain = [p[2] for p in parts]

        def forward(x, chain=chain):
            for part in chain:
                x = part(x)
            return x
        parent.forward = forward  # the children stay registered under their own names; only the call path changes
    return model
try:
    register_backend(name=DEVICE)(backend)
except Exception:  # already registered (module re-import)
    pass
