"""``torch.compile(backend="docc")`` front end, the surface docc exposes in ``docc.torch``
(mlir/docc/torch/__init__.py:335-441): ``set_backend_options``, ``compile_torch``, ``TorchProgram``
and a dynamo backend registered under the name ``"docc"``.

The reference exports the FX graph through torch-mlir to linalg-on-tensors and translates that to
SDFG library nodes (mlir/lib/Target/SDFG/LinalgToSDFGTranslator.cpp:354-454). torch-mlir is not part
of this environment, and several operations of the target configurations have no translation in the
reference at all (batched matmul, conv padding and bias, Linear bias, softmax/LayerNorm/GELU as single
nodes, attention). This module lowers the dynamo FX graph directly: every tensor operation becomes
one library node of ``docc_b200.nodes`` (Linear → GEMM with fused bias/activation/residual epilogue,
``scaled_dot_product_attention`` → Attention node, ``conv2d`` → Conv node, ...), shape operations stay
views, and anything outside that set raises — there is no eager fallback.

Unlike the reference (which forces every input to CPU numpy, mlir/docc/torch/__init__.py:251-266),
CUDA tensors are consumed in place; CPU tensors are staged to the device once per call and results are
returned on the inputs' device.
"""
from __future__ import annotations

import math
import operator
from typing import Callable, Dict, List

import torch
import torch.nn.functional as F

from .. import nodes as N
from .. import ops

__all__ = ["set_backend_options", "compile_torch", "TorchProgram"]

_CUDA_TARGETS = ("cuda", "b200")

# Global options of the backend, same keys and defaults as the reference.
_backend_options = {"target": "none", "category": "server"}


def set_backend_options(target: str = "none", category: str = "server"):
    """Configure ``torch.compile(backend="docc")`` (call before compiling)."""
    _backend_options["target"] = target
    _backend_options["category"] = category


class UnsupportedGraph(NotImplementedError):
    pass


def _check_target(target: str) -> None:
    if target not in _CUDA_TARGETS:
        raise NotImplementedError(
            f"target {target!r}: this package provides the cuda target only; docc's CPU targets are not re-implemented "
            "and there is no host fallback")


def _dispatch(node: N.LibraryNode, *inputs):
    """Runs one library node through the dispatcher registry on positional inputs."""
    env = {f"_in{i}": v for i, v in enumerate(inputs)}
    node.inputs = [f"_in{i}" if v is not None else None for i, v in enumerate(inputs)]
    node.outputs = ["_out"]
    N.B200LibraryNodeMapper(with_transfers=False).try_map(node)
    N.LibraryNodeDispatcherRegistry.instance().dispatch(node, env)
    return env["_out"]


def _contig(t):
    return t if t.is_contiguous() else t.contiguous()


def _f32(t):
    return t if t is None or t.dtype == torch.float32 else ops.cast(_contig(t), torch.float32)


_ACT = {"gelu": ops.ACT_GELU_ERF, "relu": ops.ACT_RELU, "tanh": ops.ACT_TANH, "sigmoid": ops.ACT_SIGMOID, "exp": ops.ACT_EXP,
        "erf": ops.ACT_ERF, "sqrt": ops.ACT_SQRT, "abs": ops.ACT_ABS}


# ---- lowering of single operations -----------------------------------------------------------------
def _linear(x, w, bias=None, act=ops.ACT_NONE, residual=None):
    if residual is not None:
        # The epilogue reads the residual as a full [.., out_features] tensor of the output type. An addend that
        # broadcasts (a bias-like vector, a [1, S, d] table) or has another type goes through the add node instead.
        out_shape = tuple(x.shape[:-1]) + (w.shape[0],)
        if not isinstance(residual, torch.Tensor) or tuple(residual.shape) != out_shape or residual.dtype != x.dtype:
            return _binary("add")(_linear(x, w, bias, act), residual)
    node = N.LinearNode(act=act, has_bias=bias is not None, has_residual=residual is not None)
    if bias is not None:  # the epilogue reads the bias in the output type for fp32 / fp64 and as fp32 for 16-bit layers
        bias = _contig(bias) if x.dtype == torch.float64 and bias.dtype == torch.float64 else (
            ops.cast(_contig(bias), torch.float64) if x.dtype == torch.float64 else _f32(bias))
    return _dispatch(node, _contig(x), _contig(w), bias, _contig(residual) if residual is not None else None)


def _matmul(a, b):
    if a.dim() == 2 and b.dim() == 2:
        prec = {torch.float64: "d", torch.float32: "s", torch.float16: "h", torch.bfloat16: "b"}[a.dtype]
        ta = (not a.is_contiguous()) and a.t().is_contiguous()
        tb = (not b.is_contiguous()) and b.t().is_contiguous()
        node = N.GEMMNode(precision=prec, trans_a=ta, trans_b=tb)
        return _dispatch(node, a.t() if ta else _contig(a), b.t() if tb else _contig(b))
    if a.dim() < 2 or b.dim() < 2:
        raise UnsupportedGraph("vector operands of matmul")
    return _dispatch(N.MatMulNode(), _contig(a), _contig(b))


def _softmax(x, dim=-1, _stacklevel=3, dtype=None):
    if dtype is not None and dtype != x.dtype:
        raise UnsupportedGraph("softmax with a dtype= conversion")
    return _dispatch(N.SoftmaxNode(axes=[dim]), _contig(x))


def _conv2d(x, w, bias=None, stride=1, padding=0, dilation=1, groups=1):
    pair = lambda v: [v, v] if isinstance(v, int) else list(v)
    if isinstance(padding, str):
        raise UnsupportedGraph("string padding modes")
    p = pair(padding)
    node = N.ConvNode(strides=pair(stride), pads=[p[0], p[1], p[0], p[1]], dilations=pair(dilation), group=groups)
    if bias is not None and x.dtype in (torch.bfloat16, torch.float16):
        bias = _f32(bias)  # 16-bit convolutions produce fp32 (fp32 accumulate); cast back below
    y = _dispatch(node, _contig(x), _contig(w), _contig(bias) if bias is not None else None)
    return y if y.dtype == x.dtype else ops.cast(y, x.dtype)


def _sdpa(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, enable_gqa=False):
    if attn_mask is not None or dropout_p != 0.0 or enable_gqa:
        raise UnsupportedGraph("attention masks, dropout and grouped-query attention")
    B, H, Sq, D = q.shape
    Skv = k.shape[2]
    if is_causal and Sq != Skv:
        # torch aligns the causal mask with the first key, the kernels with the last one; the two agree only for Sq == Skv
        raise UnsupportedGraph("is_causal with different query and key lengths")
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    # Output is laid out [B, S, H, D] so that the transpose(1, 2).reshape(B, S, H*D) that follows in a
    # transformer block is a view; Q/K/V are consumed through their strides (no .contiguous() copies).
    o_mem = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
    o = o_mem.permute(0, 2, 1, 3)

    def strides(t):
        if t.stride(3) != 1:
            return None
        return ops._arr((t.stride(0), t.stride(1), t.stride(2)))

    sq, sk, sv = strides(q), strides(k), strides(v)
    if sq is None or sk is None or sv is None:
        q, k, v = _contig(q), _contig(k), _contig(v)
        sq, sk, sv = strides(q), strides(k), strides(v)
    ops.call("docc_b200_attention", ops._prec(q), B, H, Sq, Skv, D, float(scale), int(bool(is_causal)), ops._ptr(q), sq,
             ops._ptr(k), sk, ops._ptr(v), sv, ops._ptr(o_mem), strides(o), 0)
    return o


def _layer_norm(x, normalized_shape, weight=None, bias=None, eps=1e-5):
    if len(tuple(normalized_shape)) != 1:
        raise UnsupportedGraph("layer_norm over more than the last dimension")
    node = N.LayerNormNode(eps=eps, has_affine=weight is not None)
    return _dispatch(node, _contig(x), _f32(weight), _f32(bias))


def _unary(kind):
    def fn(x, *args, **kwargs):
        if kind == "gelu" and kwargs.get("approximate", "none") != "none":
            raise UnsupportedGraph("tanh-approximated GELU")
        return ops.bias_act(_contig(x), act=_ACT[kind])

    return fn


def _binary(kind):
    def fn(a, b, *args, **kwargs):
        if kwargs.get("alpha", 1) != 1:
            raise UnsupportedGraph("alpha on add/sub")
        if kwargs.get("rounding_mode") is not None:
            raise UnsupportedGraph("div with a rounding mode")
        if kwargs.get("out") is not None:
            raise UnsupportedGraph("out= arguments")
        ta, tb = isinstance(a, torch.Tensor), isinstance(b, torch.Tensor)
        if ta and tb:
            if a.shape == b.shape and a.dtype == b.dtype:
                if kind == "add":
                    return ops.bias_act(_contig(a), residual=_contig(b))  # works for every precision
                if a.dtype in (torch.float32, torch.float64):
                    return ops.binary({"sub": ops.EW_SUB, "mul": ops.EW_MUL, "div": ops.EW_DIV}[kind], _contig(a), _contig(b))
            if kind == "add" and b.dim() == 1 and b.shape[0] == a.shape[-1]:
                return ops.bias_act(_contig(a), bias=_f32(b))
            if kind == "add" and a.dim() == 1 and a.shape[0] == b.shape[-1]:
                return ops.bias_act(_contig(b), bias=_f32(a))
            raise UnsupportedGraph(f"{kind} with broadcasting between {tuple(a.shape)} and {tuple(b.shape)}")
        if ta and not tb:
            if kind == "mul":
                return ops.bias_act(_contig(a), scale=float(b))
            if kind == "div":
                return ops.bias_act(_contig(a), scale=1.0 / float(b))
        if tb and not ta and kind == "mul":
            return ops.bias_act(_contig(b), scale=float(a))
        if not ta and not tb:
            return {"add": operator.add, "sub": operator.sub, "mul": operator.mul, "div": operator.truediv}[kind](a, b)
        raise UnsupportedGraph(f"{kind} of a tensor and a scalar")

    return fn


_FUNCTIONS: Dict[object, Callable] = {
    F.linear: _linear, torch._C._nn.linear: _linear,
    torch.matmul: _matmul, operator.matmul: _matmul, torch.mm: _matmul, torch.bmm: _matmul,
    F.softmax: _softmax, torch.softmax: _softmax,
    F.conv2d: _conv2d, torch.conv2d: _conv2d,
    F.scaled_dot_product_attention: _sdpa, torch._C._nn.scaled_dot_product_attention: _sdpa,
    F.layer_norm: _layer_norm,
    F.gelu: _unary("gelu"), torch._C._nn.gelu: _unary("gelu"), F.relu: _unary("relu"), torch.relu: _unary("relu"),
    torch.tanh: _unary("tanh"), F.tanh: _unary("tanh"), torch.sigmoid: _unary("sigmoid"), F.sigmoid: _unary("sigmoid"),
    torch.exp: _unary("exp"), torch.erf: _unary("erf"), torch.sqrt: _unary("sqrt"), torch.abs: _unary("abs"),
    operator.add: _binary("add"), torch.add: _binary("add"),
    operator.sub: _binary("sub"), torch.sub: _binary("sub"),
    operator.mul: _binary("mul"), torch.mul: _binary("mul"),
    operator.truediv: _binary("div"), torch.div: _binary("div"),
    operator.getitem: lambda x, idx: x[idx],
    torch.transpose: lambda x, a, b: x.transpose(a, b), torch.permute: lambda x, dims: x.permute(dims),
    torch.reshape: lambda x, shape: x.reshape(shape), torch.flatten: lambda x, *a, **k: x.flatten(*a, **k),
    torch.chunk: lambda x, *a, **k: x.chunk(*a, **k), torch.split: lambda x, *a, **k: x.split(*a, **k),
    torch.unbind: lambda x, *a, **k: x.unbind(*a, **k),
}

_INPLACE_FUNCTIONS = {operator.iadd: "add", operator.imul: "mul", operator.isub: "sub", operator.itruediv: "div"}
_INPLACE_METHODS = {"add_": "add", "mul_": "mul", "sub_": "sub", "div_": "div"}

# tensor methods that only change metadata (views); .contiguous() materialises through a copy
_VIEW_METHODS = {"view", "reshape", "transpose", "permute", "flatten", "unsqueeze", "squeeze", "t", "size", "chunk", "split",
                 "unbind", "contiguous", "expand", "unflatten", "dim"}
_METHODS: Dict[str, Callable] = {
    "softmax": _softmax, "matmul": _matmul, "mm": _matmul, "bmm": _matmul,
    "add": _binary("add"), "mul": _binary("mul"), "sub": _binary("sub"), "div": _binary("div"),
    "relu": _unary("relu"), "tanh": _unary("tanh"), "sigmoid": _unary("sigmoid"), "exp": _unary("exp"),
}


class _Lowered:
    """An FX graph lowered to a list of steps over a value table."""

    def __init__(self, gm: torch.fx.GraphModule):
        self.gm = gm
        self.steps: List[tuple] = []
        self.placeholders: List[str] = []
        self.output = None
        self.n_library_nodes = 0
        self._lower()

    def _lower(self):
        graph = self.gm.graph
        users = {n: list(n.users) for n in graph.nodes}
        fused = set()
        for n in graph.nodes:
            if n in fused:
                continue
            if n.op == "placeholder":
                self.placeholders.append(n.name)
            elif n.op == "get_attr":
                self.steps.append(("attr", n.name, n.target))
            elif n.op == "call_function":
                fn = _FUNCTIONS.get(n.target)
                if fn is None and n.target in _INPLACE_FUNCTIONS:
                    fn = self._inplace(n, _INPLACE_FUNCTIONS[n.target])
                if fn is None and getattr(n.target, "__module__", "") in ("_operator", "operator", "builtins", "math"):
                    # shape arithmetic on Python / symbolic integers (dynamic shapes): host scalars, not tensor work
                    self.steps.append(("scalar", n.name, n.target, n.args, dict(n.kwargs)))
                    continue
                if fn is None:
                    raise UnsupportedGraph(f"operation {n.target} has no library node on this path")
                args, kwargs, out_name = n.args, dict(n.kwargs), n.name
                # peephole fusions into the GEMM epilogue: linear -> gelu/relu/tanh, linear -> + residual
                if fn is _linear and len(users[n]) == 1:
                    u = users[n][0]
                    tgt = _FUNCTIONS.get(u.target) if u.op == "call_function" else None
                    act_of = {id(_FUNCTIONS[F.gelu]): ops.ACT_GELU_ERF, id(_FUNCTIONS[F.relu]): ops.ACT_RELU,
                              id(_FUNCTIONS[torch.tanh]): ops.ACT_TANH}
                    if tgt is not None and id(tgt) in act_of and u.kwargs.get("approximate", "none") == "none" and len(u.args) == 1:
                        kwargs["act"] = act_of[id(tgt)]
                        out_name = u.name
                        fused.add(u)
                    elif tgt is _FUNCTIONS[operator.add] and len(u.args) == 2 and not u.kwargs:
                        other = u.args[1] if u.args[0] is n else u.args[0]
                        if isinstance(other, torch.fx.Node) and other is not n and self._defined_before(other, n):
                            kwargs["residual"] = other
                            out_name = u.name
                            fused.add(u)
                self.steps.append(("call", out_name, fn, args, kwargs))
                self.n_library_nodes += 1
            elif n.op == "call_method":
                if n.target in _INPLACE_METHODS:
                    self.steps.append(("call", n.name, self._inplace(n, _INPLACE_METHODS[n.target]), n.args, dict(n.kwargs)))
                elif n.target in _METHODS:
                    self.steps.append(("call", n.name, _METHODS[n.target], n.args, dict(n.kwargs)))
                elif n.target in _VIEW_METHODS:
                    self.steps.append(("method", n.name, n.target, n.args, dict(n.kwargs)))
                elif n.target in ("float", "double", "half", "bfloat16", "to", "type"):
                    self.steps.append(("cast", n.name, n.target, n.args, dict(n.kwargs)))
                else:
                    raise UnsupportedGraph(f"tensor method {n.target} has no library node on this path")
            elif n.op == "call_module":
                raise UnsupportedGraph("un-inlined module call; compile with dynamo's default inlining")
            elif n.op == "output":
                self.output = n.args[0]

    @staticmethod
    def _inplace(n: torch.fx.Node, kind: str):
        """``x += y`` / ``x.add_(y)`` on a value this graph produced: the node's result stands for the updated tensor
        in every later use, so computing it out of place is equivalent. On a graph input or parameter the caller would
        have to see the update, which this path does not do."""
        dst = n.args[0] if n.args else None
        if not isinstance(dst, torch.fx.Node) or dst.op in ("placeholder", "get_attr"):
            raise UnsupportedGraph(f"in-place {kind} on a graph input or parameter")
        return _binary(kind)

    @staticmethod
    def _defined_before(a: torch.fx.Node, b: torch.fx.Node) -> bool:
        for n in b.graph.nodes:
            if n is a:
                return True
            if n is b:
                return False
        return False

    def run(self, *inputs):
        vals: Dict[str, object] = dict(zip(self.placeholders, inputs))

        def load(a):
            if isinstance(a, torch.fx.Node):
                return vals[a.name]
            if isinstance(a, (tuple, list)):
                return type(a)(load(x) for x in a)
            if isinstance(a, dict):
                return {k: load(v) for k, v in a.items()}
            return a

        for step in self.steps:
            kind = step[0]
            if kind == "attr":
                obj = self.gm
                for part in step[2].split("."):
                    obj = getattr(obj, part)
                vals[step[1]] = obj
            elif kind == "call":
                _, name, fn, args, kwargs = step
                vals[name] = fn(*load(args), **load(kwargs))
            elif kind == "scalar":
                _, name, fn, args, kwargs = step
                largs, lkwargs = load(args), load(kwargs)
                if any(isinstance(a, torch.Tensor) for a in list(largs) + list(lkwargs.values())):
                    raise UnsupportedGraph(f"operation {fn} on tensors has no library node on this path")
                vals[name] = fn(*largs, **lkwargs)
            elif kind == "method":
                _, name, meth, args, kwargs = step
                largs = load(args)
                vals[name] = getattr(largs[0], meth)(*largs[1:], **load(kwargs))
            elif kind == "cast":
                _, name, meth, args, kwargs = step
                largs = load(args)
                x = largs[0]
                dtype = {"float": torch.float32, "double": torch.float64, "half": torch.float16, "bfloat16": torch.bfloat16}.get(meth)
                if dtype is None:
                    cand = [a for a in list(largs[1:]) + list(load(kwargs).values()) if isinstance(a, torch.dtype)]
                    if not cand:
                        raise UnsupportedGraph(".to() without a dtype")
                    dtype = cand[0]
                vals[name] = x if x.dtype == dtype else ops.cast(_contig(x), dtype)
        return load(self.output)


class TorchProgram:
    """Compiled form of a torch model or FX graph (the reference's TorchProgram,
    mlir/docc/torch/__init__.py:31-329): lowers on first call, then replays the lowered steps."""

    def __init__(self, model, example_input=None, target: str = "none", category: str = "server"):
        self.model = model
        self.example_input = example_input
        self.target = target
        self.category = category
        self._lowered = None
        self._compiled = None
        self._param_cache: Dict[int, tuple] = {}

    # parameters living on the host are staged once and reused until they are modified in place
    def _to_device(self, t, device):
        if not isinstance(t, torch.Tensor) or t.is_cuda:
            return t
        if not isinstance(t, torch.nn.Parameter):
            return t.detach().to(device)
        hit = self._param_cache.get(id(t))
        if hit is not None and hit[0] == t._version and hit[1].device == device:
            return hit[1]
        d = t.detach().to(device)
        self._param_cache[id(t)] = (t._version, d)
        return d

    def _run_graph(self, gm, *args):
        _check_target(self.target)
        if self._lowered is None:
            self._lowered = _Lowered(gm)
        if not torch.cuda.is_available():
            raise RuntimeError("docc backend (cuda target): no CUDA device is available and there is no CPU fallback")
        device = next((a.device for a in args if isinstance(a, torch.Tensor) and a.is_cuda), torch.device("cuda", torch.cuda.current_device()))
        all_cpu = all(not a.is_cuda for a in args if isinstance(a, torch.Tensor))
        ops.init(device.index or 0)
        ops.set_stream(torch.cuda.current_stream(device).cuda_stream)
        with torch.no_grad():
            dev_args = [self._to_device(a, device) for a in args]
            out = self._lowered.run(*dev_args)
        back = (lambda t: t.cpu() if isinstance(t, torch.Tensor) else t) if all_cpu else (lambda t: t)
        if isinstance(out, (tuple, list)):
            return type(out)(back(o) for o in out)
        return back(out)

    def __call__(self, *args):
        if isinstance(self.model, torch.fx.GraphModule):
            return self._run_graph(self.model, *args)
        if self._compiled is None:
            _check_target(self.target)
            program = self

            def backend(gm, example_inputs):
                inner = TorchProgram(gm, target=program.target, category=program.category)

                def fn(*a):
                    r = inner(*a)
                    return r if isinstance(r, (tuple, list)) else (r,)

                program._inner = inner
                return fn

            self._compiled = torch.compile(self.model, backend=backend)
        return self._compiled(*args)

    @property
    def n_library_nodes(self) -> int:
        inner = getattr(self, "_inner", self)
        return inner._lowered.n_library_nodes if inner._lowered is not None else 0


def compile_torch(model, example_input, target: str = "none", category: str = "server") -> TorchProgram:
    return TorchProgram(model, example_input=example_input, target=target, category=category)


def _docc_backend(gm: "torch.fx.GraphModule", example_inputs):
    """Called by torch.compile(backend="docc"): lowers the FX graph to library nodes."""
    program = TorchProgram(gm, example_input=tuple(example_inputs), target=_backend_options["target"],
                           category=_backend_options["category"])
    _check_target(program.target)

    def compiled_fn(*args):
        result = program(*args)
        return result if isinstance(result, (tuple, list)) else (result,)

    compiled_fn.program = program
    return compiled_fn


def _register_backend():
    try:
        import torch._dynamo

        torch._dynamo.register_backend(name="docc")(_docc_backend)
    except Exception:
        pass


_register_backend()
