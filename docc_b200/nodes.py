"""Library nodes, target mapping and dispatch — the host-side mirror of docc's node API.

Mirrors, for the hot path only, what docc keeps in
``sdfg/include/sdfg/data_flow/library_nodes/math/{blas,tensor}`` and
``sdfg/include/sdfg/codegen/dispatchers/node_dispatcher_registry.h``:

* a node carries a ``code`` (``"GEMM"``, ``"ml::MatMul"``, ``"ml::Softmax"``, ``"ml::Conv"`` — the
  strings of ``gemm_node.h:14``, ``matmul_node.h:49``, ``softmax_node.h:9``, ``conv_node.h:48``), an
  ``implementation_type`` (free string, ``library_node.h:73,82``), named input / output connectors
  and its parameters;
* ``B200LibraryNodeMapper.try_map`` plays the role of ``CudaLibraryNodeRewriter``
  (``opt/src/passes/offloading/cuda_library_node_rewriter_pass.cpp:12-54``) / ``EtLibNodeMapper``
  (``targets/et/src/et/et_lib_node_mapper.cpp:10-25``): it flips the implementation type to one of
  the B200 keys *before* expansion, so the node reaches code generation whole;
* ``LibraryNodeDispatcherRegistry`` maps ``"<code>::<implementation type>"`` to a dispatcher
  factory, first registration wins (``node_dispatcher_registry.h:188-194``). A dispatcher here does
  not print C++: it issues the call into the C ABI that docc's generated host code would contain.

Dispatch operates on an environment ``{container name -> array}`` where arrays are numpy arrays
(host pointers, the "WithTransfers" flavour) or torch CUDA tensors (device pointers).
"""
from __future__ import annotations

import threading
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

from . import ops

IMPL_NONE = "NONE"
IMPL_BLAS = "BLAS"  # blas_node.h: ImplementationType_BLAS
IMPL_B200_WITH_TRANSFERS = "B200WithTransfers"
IMPL_B200_WITHOUT_TRANSFERS = "B200WithoutTransfers"

CODE_GEMM = "GEMM"
CODE_MATMUL = "ml::MatMul"
CODE_SOFTMAX = "ml::Softmax"
CODE_CONV = "ml::Conv"
CODE_REDUCE = {"sum": "ml::Sum", "max": "ml::Max", "min": "ml::Min", "mean": "ml::Mean", "std": "ml::Std"}
CODE_ELEMENTWISE = "ml::Elementwise"
CODE_ATTENTION = "ml::Attention"  # no docc counterpart
CODE_LAYERNORM = "ml::LayerNorm"  # no docc counterpart
CODE_LINEAR = "ml::Linear"  # GEMM fused with its element-wise consumers; no docc counterpart
CODE_CAST = "ml::Cast"


class InvalidSDFGException(ValueError):
    """Same role as sdfg::InvalidSDFGException: a node that violates its contract."""


@dataclass
class LibraryNode:
    code: str = ""
    inputs: List[str] = field(default_factory=list)  # connector -> container name, in connector order
    outputs: List[str] = field(default_factory=list)
    implementation_type: str = IMPL_NONE
    element_id: int = 0

    input_connectors: Sequence[str] = ()
    output_connectors: Sequence[str] = ()

    def validate(self) -> None:
        if len(self.outputs) != len(self.output_connectors):
            raise InvalidSDFGException(f"{self.code}: expected outputs {list(self.output_connectors)}")

    def flop(self, env=None) -> Optional[int]:
        return None

    def to_json(self) -> dict:
        d = {"type": "library_node", "code": self.code, "implementation_type": self.implementation_type,
             "inputs": list(self.inputs), "outputs": list(self.outputs), "element_id": self.element_id}
        d.update(self._params())
        return d

    def _params(self) -> dict:
        return {}

    def key(self) -> str:
        return f"{self.code}::{self.implementation_type}"


@dataclass
class GEMMNode(LibraryNode):
    """C = alpha*op(A)*op(B) + beta*C (gemm_node.h:16-87). Connectors __A, __B, __C -> __C; alpha and
    beta are node constants here (docc wires them through __alpha / __beta connectors)."""

    precision: str = "d"
    layout: int = ops.ROW_MAJOR
    trans_a: bool = False
    trans_b: bool = False
    alpha: float = 1.0
    beta: float = 0.0
    code: str = CODE_GEMM
    implementation_type: str = IMPL_BLAS
    input_connectors: Sequence[str] = ("__A", "__B", "__C")
    output_connectors: Sequence[str] = ("__C",)

    def validate(self) -> None:
        super().validate()
        if self.precision not in ("h", "s", "d", "b"):
            raise InvalidSDFGException("Invalid BLAS_Precision value")
        if len(self.inputs) not in (2, 3):
            raise InvalidSDFGException("GEMMNode requires __A and __B (and optionally __C)")

    def _mnk(self, env):
        a, b = env[self.inputs[0]], env[self.inputs[1]]
        m, k = (a.shape[1], a.shape[0]) if self.trans_a else a.shape
        n = b.shape[0] if self.trans_b else b.shape[1]
        return m, n, k

    def flops(self, env, alpha_non_zero=True, alpha_non_ident=True, beta_non_zero=True, beta_non_ident=True) -> int:
        """GEMMNode::flops (gemm_node.cpp:341-356): every term is multiplied by the condition it depends on.
        mn*k multiplies and mn*(k-1) additions of the product if alpha != 0; mn multiplies for the alpha scaling if
        alpha is neither 0 nor 1; mn multiplies for the beta scaling if beta is neither 0 nor 1; mn additions of the
        scaled C if beta != 0."""
        m, n, k = self._mnk(env)
        res = m * n
        mul_ops = res * k * int(alpha_non_zero) + res * int(alpha_non_ident and alpha_non_zero) + res * int(beta_non_ident and beta_non_zero)
        add_ops = res * (k - 1) * int(alpha_non_zero) + res * int(beta_non_zero)
        return mul_ops + add_ops

    def flop(self, env=None) -> Optional[int]:
        # GEMMNode::flop (gemm_node.cpp:337-339): all four conditions true, 2mnk + 2mn
        if env is None:
            return None
        return self.flops(env)

    def flop_for_constants(self, env) -> int:
        """The count for this node's own alpha and beta (they are node constants here, so the conditions are known)."""
        return self.flops(env, self.alpha != 0.0, self.alpha != 1.0, self.beta != 0.0, self.beta != 1.0)

    def _params(self) -> dict:
        return {"precision": self.precision, "layout": self.layout, "trans_a": self.trans_a, "trans_b": self.trans_b,
                "alpha": self.alpha, "beta": self.beta}


@dataclass
class MatMulNode(LibraryNode):
    """N-D batched matmul Y[..., M, N] = A[..., M, K] B[..., K, N] (matmul_node.cpp:25-70)."""

    code: str = CODE_MATMUL
    input_connectors: Sequence[str] = ("A", "B")
    output_connectors: Sequence[str] = ("Y",)


@dataclass
class SoftmaxNode(LibraryNode):
    """Max-subtracted softmax over ``axes``; keepdims must be false (softmax_node.cpp:21-34)."""

    axes: Sequence[int] = (-1,)
    keepdims: bool = False
    code: str = CODE_SOFTMAX
    input_connectors: Sequence[str] = ("X",)
    output_connectors: Sequence[str] = ("Y",)

    def validate(self) -> None:
        super().validate()
        if self.keepdims:
            raise InvalidSDFGException("Unsupported attribute on library node: softmax")

    def _params(self) -> dict:
        return {"axes": list(self.axes), "keepdims": self.keepdims}


@dataclass
class ReduceNode(LibraryNode):
    """Sum / Max / Min / Mean / Std over ``axes`` (reduce_node.cpp:122-345 and subclasses)."""

    op: str = "sum"
    axes: Sequence[int] = (-1,)
    keepdims: bool = False
    input_connectors: Sequence[str] = ("X",)
    output_connectors: Sequence[str] = ("Y",)

    def __post_init__(self):
        if self.op not in CODE_REDUCE:
            raise InvalidSDFGException(f"unknown reduction {self.op}")
        self.code = CODE_REDUCE[self.op]

    def _params(self) -> dict:
        return {"op": self.op, "axes": list(self.axes), "keepdims": self.keepdims}


@dataclass
class ConvNode(LibraryNode):
    """ONNX-style N-D cross-correlation, NC(D..) layout (conv_node.h:87-200). Connectors X, W, [B] -> Y."""

    strides: Sequence[int] = ()
    pads: Sequence[int] = ()  # begin..., end...
    dilations: Sequence[int] = ()
    group: int = 1
    code: str = CODE_CONV
    input_connectors: Sequence[str] = ("X", "W", "B")
    output_connectors: Sequence[str] = ("Y",)

    def validate(self) -> None:
        super().validate()
        if len(self.inputs) < 2:
            raise InvalidSDFGException("ConvNode requires X and W inputs")

    def _params(self) -> dict:
        return {"strides": list(self.strides), "pads": list(self.pads), "dilations": list(self.dilations), "group": self.group}


@dataclass
class ElementwiseNode(LibraryNode):
    """Unary / binary tensor node (elementwise_node.cpp:86-339): ``kind`` is a binary op name
    (add, sub, mul, div, max, min), a unary function name (exp, tanh, erf, sqrt, abs, sigmoid, relu,
    gelu), or ``scale`` (multiply by the constant ``value``)."""

    kind: str = "add"
    value: float = 1.0
    code: str = CODE_ELEMENTWISE
    input_connectors: Sequence[str] = ("A", "B")
    output_connectors: Sequence[str] = ("Y",)

    def _params(self) -> dict:
        return {"kind": self.kind, "value": self.value}


@dataclass
class CastNode(LibraryNode):
    dtype: str = "float32"
    code: str = CODE_CAST
    input_connectors: Sequence[str] = ("X",)
    output_connectors: Sequence[str] = ("Y",)

    def _params(self) -> dict:
        return {"dtype": self.dtype}


@dataclass
class LinearNode(LibraryNode):
    """Y = act(X W^T + bias) + residual: a GEMM with its element-wise consumers folded into the epilogue."""

    act: int = ops.ACT_NONE
    has_bias: bool = False
    has_residual: bool = False
    code: str = CODE_LINEAR
    input_connectors: Sequence[str] = ("X", "W", "B", "R")
    output_connectors: Sequence[str] = ("Y",)

    def _params(self) -> dict:
        return {"act": self.act, "has_bias": self.has_bias, "has_residual": self.has_residual}


@dataclass
class AttentionNode(LibraryNode):
    scale: Optional[float] = None
    causal: bool = False
    code: str = CODE_ATTENTION
    input_connectors: Sequence[str] = ("Q", "K", "V")
    output_connectors: Sequence[str] = ("O",)

    def _params(self) -> dict:
        return {"scale": self.scale, "causal": self.causal}


@dataclass
class LayerNormNode(LibraryNode):
    eps: float = 1e-5
    has_affine: bool = True
    code: str = CODE_LAYERNORM
    input_connectors: Sequence[str] = ("X", "G", "B")
    output_connectors: Sequence[str] = ("Y",)

    def _params(self) -> dict:
        return {"eps": self.eps, "has_affine": self.has_affine}


# ---- target mapping -------------------------------------------------------------------------------
class B200LibraryNodeMapper:
    """Picks the implementation type for nodes the B200 runtime executes. Everything it does not
    recognise is left untouched (and will fail at dispatch: there is no expansion to loop nests)."""

    MAPPED = {CODE_GEMM, CODE_MATMUL, CODE_SOFTMAX, CODE_CONV, CODE_ELEMENTWISE, CODE_ATTENTION, CODE_LAYERNORM, CODE_LINEAR,
              CODE_CAST, *CODE_REDUCE.values()}

    def __init__(self, with_transfers: bool = True):
        self.impl = IMPL_B200_WITH_TRANSFERS if with_transfers else IMPL_B200_WITHOUT_TRANSFERS

    def try_map(self, node: LibraryNode) -> bool:
        if node.code in self.MAPPED:
            node.implementation_type = self.impl
            return True
        return False


# ---- dispatcher registry ------------------------------------------------------------------------------
Dispatcher = Callable[[LibraryNode, dict], None]


class LibraryNodeDispatcherRegistry:
    """``"<code>::<implementation type>"`` -> dispatcher. First registration wins; registration is
    guarded by a lock, look-ups are lock free (node_dispatcher_registry.h:188-202)."""

    _instance = None

    def __init__(self):
        self._lock = threading.Lock()
        self._table: Dict[str, Dispatcher] = {}

    @classmethod
    def instance(cls) -> "LibraryNodeDispatcherRegistry":
        if cls._instance is None:
            cls._instance = cls()
            register_b200_plugin(cls._instance)
        return cls._instance

    def register_library_node_dispatcher(self, key: str, dispatcher: Dispatcher) -> bool:
        with self._lock:
            if key in self._table:
                return False
            self._table[key] = dispatcher
            return True

    def get_library_node_dispatcher(self, key: str) -> Optional[Dispatcher]:
        return self._table.get(key)

    def dispatch(self, node: LibraryNode, env: dict) -> None:
        fn = self.get_library_node_dispatcher(node.key())
        if fn is None:
            raise InvalidSDFGException(f"no dispatcher registered for library node {node.key()}")
        node.validate()
        fn(node, env)


_UNARY_ACT = {"gelu": ops.ACT_GELU_ERF, "relu": ops.ACT_RELU, "tanh": ops.ACT_TANH, "sigmoid": ops.ACT_SIGMOID,
              "exp": ops.ACT_EXP, "erf": ops.ACT_ERF, "sqrt": ops.ACT_SQRT, "abs": ops.ACT_ABS}
_BINARY = {"add": ops.EW_ADD, "sub": ops.EW_SUB, "mul": ops.EW_MUL, "div": ops.EW_DIV, "max": ops.EW_MAX, "min": ops.EW_MIN}
_REDUCE = {"sum": ops.RED_SUM, "max": ops.RED_MAX, "min": ops.RED_MIN, "mean": ops.RED_MEAN, "std": ops.RED_STD}


def _as2d(x):
    return x.reshape(-1, x.shape[-1]) if x.ndim != 2 else x


def _gemm(node: GEMMNode, env: dict) -> None:
    a, b = env[node.inputs[0]], env[node.inputs[1]]
    c = env.get(node.inputs[2]) if len(node.inputs) > 2 and node.beta != 0.0 else None
    env[node.outputs[0]] = ops.gemm(a, b, c, alpha=node.alpha, beta=node.beta, transa=node.trans_a, transb=node.trans_b,
                                    layout=node.layout)


def _matmul(node: MatMulNode, env: dict) -> None:
    env[node.outputs[0]] = ops.matmul(env[node.inputs[0]], env[node.inputs[1]])


def _softmax(node: SoftmaxNode, env: dict) -> None:
    env[node.outputs[0]] = ops.softmax(env[node.inputs[0]], list(node.axes))


def _reduce(node: ReduceNode, env: dict) -> None:
    x = env[node.inputs[0]]
    y = ops.reduce(_REDUCE[node.op], x, list(node.axes))
    if node.keepdims:
        norm = sorted(a % x.ndim for a in node.axes)
        y = y.reshape(tuple(1 if d in norm else s for d, s in enumerate(x.shape)))
    env[node.outputs[0]] = y


def _conv(node: ConvNode, env: dict) -> None:
    x, w = env[node.inputs[0]], env[node.inputs[1]]
    b = env[node.inputs[2]] if len(node.inputs) > 2 and node.inputs[2] is not None else None
    env[node.outputs[0]] = ops.conv(x, w, b, strides=list(node.strides) or None, pads=list(node.pads) or None,
                                    dilations=list(node.dilations) or None, group=node.group)


def _elementwise(node: ElementwiseNode, env: dict) -> None:
    a = env[node.inputs[0]]
    if node.kind in _BINARY:
        env[node.outputs[0]] = ops.binary(_BINARY[node.kind], a, env[node.inputs[1]])
    elif node.kind == "scale":
        env[node.outputs[0]] = ops.bias_act(a, scale=node.value)
    elif node.kind in _UNARY_ACT:
        env[node.outputs[0]] = ops.bias_act(a, act=_UNARY_ACT[node.kind])
    else:
        raise InvalidSDFGException(f"unknown element-wise kind {node.kind}")


def _cast(node: CastNode, env: dict) -> None:
    x = env[node.inputs[0]]
    if ops._is_torch(x):
        import torch

        env[node.outputs[0]] = ops.cast(x, getattr(torch, node.dtype))
    else:
        env[node.outputs[0]] = ops.cast(x, node.dtype)


def _linear(node: LinearNode, env: dict) -> None:
    x, w = env[node.inputs[0]], env[node.inputs[1]]
    bias = env[node.inputs[2]] if node.has_bias else None
    res = env[node.inputs[3]] if node.has_residual else None
    env[node.outputs[0]] = ops.linear(x, w, bias, node.act, res)


def _attention(node: AttentionNode, env: dict) -> None:
    q, k, v = (env[n] for n in node.inputs[:3])
    env[node.outputs[0]] = ops.attention(q, k, v, node.scale, node.causal)


def _layernorm(node: LayerNormNode, env: dict) -> None:
    x = env[node.inputs[0]]
    g = env[node.inputs[1]] if node.has_affine and len(node.inputs) > 1 else None
    b = env[node.inputs[2]] if node.has_affine and len(node.inputs) > 2 else None
    env[node.outputs[0]] = ops.layernorm(x, g, b, node.eps)


def register_b200_plugin(registry: LibraryNodeDispatcherRegistry) -> None:
    """The ``register_plugin(plugins::Context&)`` of a docc target (targets/et/src/et/target.cpp:21-36)."""
    table = {CODE_GEMM: _gemm, CODE_MATMUL: _matmul, CODE_SOFTMAX: _softmax, CODE_CONV: _conv,
             CODE_ELEMENTWISE: _elementwise, CODE_CAST: _cast, CODE_LINEAR: _linear, CODE_ATTENTION: _attention,
             CODE_LAYERNORM: _layernorm}
    for code in CODE_REDUCE.values():
        table[code] = _reduce
    for code, fn in table.items():
        for impl in (IMPL_B200_WITH_TRANSFERS, IMPL_B200_WITHOUT_TRANSFERS):
            registry.register_library_node_dispatcher(f"{code}::{impl}", fn)


@dataclass
class Program:
    """A straight-line schedule of library nodes over named containers: what is left of an SDFG on
    this path once every tensor operation is a library node."""

    arguments: List[str]
    nodes: List[LibraryNode]
    results: List[str]
    constants: Dict[str, object] = field(default_factory=dict)

    def map_to_target(self, with_transfers: bool) -> int:
        mapper = B200LibraryNodeMapper(with_transfers)
        return sum(1 for n in self.nodes if mapper.try_map(n))

    def run(self, *args):
        if len(args) != len(self.arguments):
            raise TypeError(f"expected {len(self.arguments)} arguments, got {len(args)}")
        env = dict(self.constants)
        env.update(zip(self.arguments, args))
        registry = LibraryNodeDispatcherRegistry.instance()
        for node in self.nodes:
            registry.dispatch(node, env)
        out = [env[r] for r in self.results]
        return out[0] if len(out) == 1 else tuple(out)

    def loop_report(self) -> dict:
        """Shape of StructuredSDFG.loop_report(): on this path nothing is left as a loop."""
        return {"library_nodes": len(self.nodes), "maps": 0, "fors": 0}

    def to_json(self) -> dict:
        return {"arguments": self.arguments, "results": self.results, "nodes": [n.to_json() for n in self.nodes]}
