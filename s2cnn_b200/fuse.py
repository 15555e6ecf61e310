"""``fuse(model)``: route a model written with the reference's plain calls through the fused kernels.

Models built on the reference look like examples/mnist/run.py:55-98 - convolution modules,
``F.relu`` between them, ``so3_integrate`` before the linear head - either as a hand-written
``forward`` or as an ``nn.Sequential``.  Written that way every layer boundary is a tensor in
memory.  ``fuse`` traces the model once (``torch.fx``; the convolution modules are leaves,
``so3_integrate`` is recorded as one call), finds the chains below and rewrites them into the
keyword arguments of this package's modules that select the fused kernels; everything else in the
model is left as traced.  The result computes the same function.

    conv_a -> relu -> SO3Convolution b     conv_a(x, relu_so3_fft=b.b_out); b(.., input_spectrum=True)
                                           (synthesis, bias, ReLU and the next analysis in one kernel)
    conv -> BatchNorm3d (eval mode)        conv(x, channel_scale=s, bias=t): the normalisation is a
                                           per-channel affine map, folded into the kernel's spectrum
                                           and the bias (training-mode BatchNorm is left alone)
    SO3Convolution -> relu -> so3_integrate    conv(x, relu_integrate=True)
    relu -> SO3Convolution                 conv(x, relu_input=True)   (ReLU applied while loading)
    relu -> so3_integrate                  so3_relu_integrate(x)

A chain is only rewritten when the intermediate tensor has no other consumer and the sizes are
ones the fused kernels take (2 b <= 32, non-increasing bandwidth); otherwise it stays as it is.
"""
import sys
from operator import getitem as _getitem

import torch
import torch.fx
import torch.nn.functional as F

from .soft.s2_conv import S2Convolution
from .soft.so3_conv import SO3Convolution, SO3Shortcut
from .soft.so3_integrate import so3_integrate, so3_relu_integrate

_LEAVES = (S2Convolution, SO3Convolution, SO3Shortcut)
_RELU_FUNCTIONS = (torch.relu, F.relu, torch.nn.functional.relu, torch.relu_)


class _Tracer(torch.fx.Tracer):
    def is_leaf_module(self, m, qualname):
        return isinstance(m, _LEAVES) or super().is_leaf_module(m, qualname)


class _RecordedCalls:
    """While tracing, every binding of the given functions in any imported module's namespace
    (``from s2cnn_b200 import so3_integrate``, ``S.so3_integrate``, ...) is replaced by a stand-in
    that records ONE call node instead of being traced into (their bodies look at tensor sizes)."""

    def __init__(self, *functions):
        self.functions = functions
        self.patched = []

    @staticmethod
    def _stand_in(fn):
        def call(*args, **kwargs):
            for a in args:
                if isinstance(a, torch.fx.Proxy):
                    return a.tracer.create_proxy("call_function", fn, args, kwargs)
            return fn(*args, **kwargs)
        return call

    def __enter__(self):
        stand_ins = {id(f): self._stand_in(f) for f in self.functions}
        for mod in list(sys.modules.values()):
            ns = getattr(mod, "__dict__", None)
            if not isinstance(ns, dict):
                continue
            for name, value in list(ns.items()):
                if id(value) in stand_ins and any(value is f for f in self.functions):
                    self.patched.append((ns, name, value))
                    ns[name] = stand_ins[id(value)]
        return self

    def __exit__(self, *exc):
        for ns, name, value in self.patched:
            ns[name] = value
        self.patched = []
        return False


_OWN_KEYWORDS = {"relu_input", "relu_integrate", "input_spectrum", "relu_so3_fft", "channel_scale",
                 "bias"}


def _fold_batchnorm(conv_bias, mean, var, weight, bias, eps):
    """Eval-mode BatchNorm3d after a convolution with bias b:  ((y + b) - mean) / sqrt(var + eps) *
    weight + bias  =  y * s + (b * s + bias - mean * s): the per-channel scale for the kernel's
    spectrum and the bias that replaces the layer's own."""
    s = torch.rsqrt(var + eps)
    if weight is not None:
        s = s * weight
    shift = -mean * s
    if bias is not None:
        shift = shift + bias
    return s, conv_bias * s.view(1, -1, 1, 1, 1) + shift.view(1, -1, 1, 1, 1)


def _is_relu(node, modules):
    if node.op == "call_function" and node.target in _RELU_FUNCTIONS:
        return len(node.args) >= 1
    if node.op == "call_method" and node.target in ("relu", "relu_"):
        return True
    if node.op == "call_module" and isinstance(modules.get(node.target), torch.nn.ReLU):
        return True
    return False


def _conv(node, modules, kinds):
    """The convolution module a node calls with one positional argument (and at most the keywords
    this rewrite itself adds), else None."""
    if node.op != "call_module":
        return None
    m = modules.get(node.target)
    if isinstance(m, kinds) and len(node.args) == 1 and set(node.kwargs) <= _OWN_KEYWORDS:
        return m
    return None


def _is_integrate(node):
    return node.op == "call_function" and node.target is so3_integrate


def _only_user(node):
    users = list(node.users)
    return users[0] if len(users) == 1 else None


def fuse(model):
    """Returns a ``torch.fx.GraphModule`` sharing ``model``'s parameters in which the chains listed
    in the module docstring run through the fused kernels.  ``model`` itself is not modified."""
    tracer = _Tracer()
    with _RecordedCalls(so3_integrate, so3_relu_integrate):
        graph = tracer.trace(model)
    modules = dict(model.named_modules())
    # eval-mode BatchNorm3d right after a convolution: fold it into the layer
    for node in list(graph.nodes):
        bn = modules.get(node.target) if node.op == "call_module" else None
        if not isinstance(bn, torch.nn.BatchNorm3d) or bn.training or bn.running_mean is None:
            continue
        src = node.args[0] if node.args else None
        if not isinstance(src, torch.fx.Node) or len(src.users) != 1:
            continue
        conv = _conv(src, modules, (S2Convolution, SO3Convolution))
        if conv is None or src.kwargs:
            continue
        with graph.inserting_before(src):
            attr = lambda mod_name, name: graph.get_attr(mod_name + "." + name)  # noqa: E731
            weight = attr(node.target, "weight") if bn.affine else None
            bias = attr(node.target, "bias") if bn.affine else None
            folded = graph.call_function(_fold_batchnorm, (
                attr(src.target, "bias"), attr(node.target, "running_mean"),
                attr(node.target, "running_var"), weight, bias, bn.eps))
            scale = graph.call_function(_getitem, (folded, 0))
            new_bias = graph.call_function(_getitem, (folded, 1))
        src.kwargs = {"channel_scale": scale, "bias": new_bias}
        node.replace_all_uses_with(src)
        graph.erase_node(node)
    for node in list(graph.nodes):
        if not _is_relu(node, modules):
            continue
        src = node.args[0] if node.args else None
        if not isinstance(src, torch.fx.Node):
            continue
        dst = _only_user(node)
        if dst is None:
            continue
        if len(src.users) > 1:
            continue   # someone else reads the pre-activation tensor (or an in-place ReLU's result)
        producer = _conv(src, modules, (S2Convolution, SO3Convolution))
        producer_ok = producer is not None and _only_user(src) is node
        consumer = _conv(dst, modules, (SO3Convolution,))
        if consumer is not None and dst.args[0] is not node:
            consumer = None
        if consumer is not None:
            if (producer_ok and not src.kwargs.get("relu_so3_fft") and
                    not src.kwargs.get("relu_integrate") and producer.b_out == consumer.b_in and
                    2 * producer.b_out <= 32 and consumer.b_out <= producer.b_out):
                # synthesis + bias + ReLU + the next layer's analysis in one kernel
                src.kwargs = dict(src.kwargs, relu_so3_fft=consumer.b_out)
                dst.args = (src,)
                dst.kwargs = dict(dst.kwargs, input_spectrum=True)
                graph.erase_node(node)
            elif 2 * consumer.b_in <= 32:
                dst.args = (src,)
                dst.kwargs = dict(dst.kwargs, relu_input=True)
                graph.erase_node(node)
            continue
        if _is_integrate(dst) and dst.args[0] is node:
            if (producer_ok and isinstance(producer, SO3Convolution) and 2 * producer.b_out <= 32
                    and not src.kwargs.get("relu_so3_fft")):
                src.kwargs = dict(src.kwargs, relu_integrate=True)
                dst.replace_all_uses_with(src)
                graph.erase_node(dst)
                graph.erase_node(node)
            else:
                with graph.inserting_before(dst):
                    new = graph.call_function(so3_relu_integrate, (src,))
                dst.replace_all_uses_with(new)
                graph.erase_node(dst)
                graph.erase_node(node)
    graph.lint()
    fused = torch.fx.GraphModule(tracer.root, graph, class_name="Fused" + type(model).__name__)
    fused.train(model.training)
    return fused


__all__ = ["fuse"]
