"""Reader for docc's SDFG JSON wire format: executes the library nodes of a dumped SDFG through the C ABI.

docc writes a structured SDFG as JSON (``JSONSerializer::serialize``, sdfg/src/serializer/json_serializer.cpp:63-113):
``name``, ``containers`` (name -> type), ``arguments`` (ordered names), ``root`` (a ``sequence`` whose ``children`` are
``block`` / ``sequence`` / ``for`` / ``map`` / ``if_else`` / ``while`` / ``return`` elements, :191-343). A block carries a
``dataflow`` object with ``nodes`` (``access_node``, ``constant_node``, ``tasklet``, ``library_node``; :115-159) and
``edges`` (``src``, ``dst`` element ids, ``src_conn``, ``dst_conn``, ``subset``, ``base_type``; :161-186). A library node
carries ``code``, ``implementation_type`` and the fields of its own serializer (GEMM: gemm_node.cpp:387-405; MatMul:
matmul_node.cpp; Conv: conv_node.cpp:552-647; reductions and Softmax: ``shape``, ``axes``, ``keepdims``; element-wise
nodes: ``shape``), with every symbolic expression printed as a string.

This reader covers the part of that format the math path needs: straight-line sequences of blocks whose dataflow
consists of access nodes, constant nodes and library nodes with whole-container memlets (empty ``subset``). Anything
else (tasklets, loops, branches, partial memlets) raises :class:`UnsupportedSdfg` naming the element, so a caller can fall
back to docc's own code generation for that SDFG. Containers are flat buffers, as in docc's generated code: every node
views its operands with the shape it carries.
"""
from __future__ import annotations

import ast
import json
import math
import operator
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np

from . import nodes as N
from . import ops


class UnsupportedSdfg(NotImplementedError):
    """The SDFG contains an element this reader does not execute."""


# ---- symbolic expressions --------------------------------------------------------------------------------------
# SymEngine prints integers, symbols, + - * / ** and a few functions; shapes and leading dimensions are integer
# valued, so division is exact or floor division of non-negative operands.
_BINOPS = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul, ast.FloorDiv: operator.floordiv,
           ast.Mod: operator.mod, ast.Pow: operator.pow}
_FUNCS: Dict[str, Callable] = {
    "max": max, "Max": max, "min": min, "Min": min, "floor": math.floor, "ceiling": math.ceil, "abs": abs,
    "idiv": lambda a, b: a // b, "imod": lambda a, b: a % b, "iabs": abs,
}


def evaluate(expr, symbols: Optional[Dict[str, int]] = None) -> int:
    """Value of a symbolic expression string (``symbolic::parse`` syntax) under ``symbols``."""
    if isinstance(expr, (int, np.integer)):
        return int(expr)
    symbols = symbols or {}

    def ev(node):
        if isinstance(node, ast.Expression):
            return ev(node.body)
        if isinstance(node, ast.Constant) and isinstance(node.value, (int, float)):
            return node.value
        if isinstance(node, ast.Name):
            if node.id not in symbols:
                raise KeyError(f"symbol {node.id!r} has no value")
            return symbols[node.id]
        if isinstance(node, ast.UnaryOp) and isinstance(node.op, (ast.USub, ast.UAdd)):
            v = ev(node.operand)
            return -v if isinstance(node.op, ast.USub) else v
        if isinstance(node, ast.BinOp):
            a, b = ev(node.left), ev(node.right)
            if isinstance(node.op, ast.Div):
                q = a / b
                return int(q) if float(q).is_integer() else q
            if type(node.op) in _BINOPS:
                return _BINOPS[type(node.op)](a, b)
        if isinstance(node, ast.Call) and isinstance(node.func, ast.Name) and node.func.id in _FUNCS and not node.keywords:
            return _FUNCS[node.func.id](*[ev(a) for a in node.args])
        raise UnsupportedSdfg(f"expression {expr!r}: unsupported syntax")

    value = ev(ast.parse(str(expr).replace("^", "**"), mode="eval"))
    if isinstance(value, float):
        if not value.is_integer():
            raise UnsupportedSdfg(f"expression {expr!r} is not integer valued ({value})")
        value = int(value)
    return int(value)


# ---- types --------------------------------------------------------------------------------------------------------
# types::PrimitiveType in declaration order (sdfg/include/sdfg/types/type.h): the serializer writes the enum value
_PRIMITIVE = {1: "bool", 2: "int8", 3: "int16", 4: "int32", 5: "int64", 7: "uint8", 8: "uint16", 9: "uint32", 10: "uint64",
              12: "float16", 13: "bfloat16", 14: "float32", 15: "float64"}
_PRECISION_DTYPE = {"h": "float16", "s": "float32", "d": "float64", "b": "bfloat16"}


def element_dtype(type_json: dict) -> Optional[str]:
    """numpy-style dtype name of the scalar at the bottom of a (pointer / array / tensor) type, if it is a primitive."""
    t = type_json
    while isinstance(t, dict):
        kind = t.get("type")
        if kind == "scalar":
            return _PRIMITIVE.get(int(t.get("primitive_type", -1)))
        t = t.get("pointee_type") or t.get("element_type") or t.get("reference_type")
    return None


# ---- plan --------------------------------------------------------------------------------------------------------
@dataclass
class Step:
    """One library node with its operands bound to container names and its shapes still symbolic."""

    element_id: int
    code: str
    fields: dict
    inputs: Dict[str, object]  # connector -> container name (str) or ("const", text)
    outputs: Dict[str, str]    # connector -> container name


_UNARY = {"ml::Exp": "exp", "ml::Erf": "erf", "ml::Tanh": "tanh", "ml::Sqrt": "sqrt", "ml::Sigmoid": "sigmoid",
          "ml::ReLU": "relu", "ml::Abs": "abs"}
_BINARY = {"ml::Add": "add", "ml::Sub": "sub", "ml::Mul": "mul", "ml::Div": "div", "ml::Maximum": "max", "ml::Minimum": "min"}
_REDUCE = {"ml::Sum": "sum", "ml::Max": "max", "ml::Min": "min", "ml::Mean": "mean", "ml::Std": "std"}
SUPPORTED_CODES = {"GEMM", "ml::MatMul", "ml::Softmax", "ml::Conv", "ml::Cast", *_UNARY, *_BINARY, *_REDUCE}


def _block_steps(block: dict) -> List[Step]:
    flow = block["dataflow"]
    by_id = {n["element_id"]: n for n in flow["nodes"]}
    for n in flow["nodes"]:
        if n["type"] == "tasklet":
            raise UnsupportedSdfg(f"tasklet {n['element_id']} ({n.get('code')}): scalar code is left to docc's code generator")
        if n["type"] == "library_node" and n["code"] not in SUPPORTED_CODES:
            raise UnsupportedSdfg(f"library node {n['element_id']} with code {n['code']!r}")
    steps: Dict[int, Step] = {}
    succ: Dict[int, List[int]] = {i: [] for i in by_id}
    indeg = {i: 0 for i in by_id}
    for e in flow["edges"]:
        if e.get("subset"):
            raise UnsupportedSdfg(f"edge {e['element_id']}: memlet with a subset {e['subset']}")
        src, dst = by_id[e["src"]], by_id[e["dst"]]
        succ[e["src"]].append(e["dst"])
        indeg[e["dst"]] += 1
        if dst["type"] == "library_node":
            st = steps.setdefault(dst["element_id"], Step(dst["element_id"], dst["code"], dst, {}, {}))
            if src["type"] == "access_node":
                st.inputs[e["dst_conn"]] = src["data"]
            elif src["type"] == "constant_node":
                st.inputs[e["dst_conn"]] = ("const", src["data"])
            else:
                raise UnsupportedSdfg(f"edge {e['element_id']}: library node fed by a {src['type']}")
        if src["type"] == "library_node":
            if dst["type"] != "access_node":
                raise UnsupportedSdfg(f"edge {e['element_id']}: library node writes to a {dst['type']}")
            st = steps.setdefault(src["element_id"], Step(src["element_id"], src["code"], src, {}, {}))
            st.outputs[e["src_conn"]] = dst["data"]
    # dataflow order (Kahn), element ids break ties
    ready = sorted(i for i, d in indeg.items() if d == 0)
    order: List[int] = []
    while ready:
        i = ready.pop(0)
        order.append(i)
        for j in succ[i]:
            indeg[j] -= 1
            if indeg[j] == 0:
                ready.append(j)
                ready.sort()
    if len(order) != len(by_id):
        raise UnsupportedSdfg("dataflow graph has a cycle")
    return [steps[i] for i in order if i in steps]


def _sequence_steps(seq: dict) -> List[Step]:
    out: List[Step] = []
    for child in seq.get("children", []):
        kind = child.get("type")
        if kind == "block":
            out.extend(_block_steps(child))
        elif kind == "sequence":
            out.extend(_sequence_steps(child))
        elif kind == "return":
            continue
        else:
            raise UnsupportedSdfg(f"control-flow element {child.get('element_id')} of type {kind!r}")
    return out


# ---- execution -----------------------------------------------------------------------------------------------------
def _flat(x):
    return x.reshape(-1)


def _view(x, shape: Sequence[int]):
    n = int(np.prod(shape)) if len(shape) else 1
    flat = _flat(x)
    if flat.shape[0] < n:
        raise ValueError(f"container holds {flat.shape[0]} elements, node needs {n}")
    return flat[:n].reshape(tuple(shape))


def _store(env: dict, name: str, value) -> None:
    """Writes a node result into its container: into the caller's buffer when there is one, else binds the new array."""
    if name in env and env[name] is not None and not isinstance(env[name], (int, float)):
        dst = _flat(env[name])
        src = _flat(value)
        if dst.shape[0] < src.shape[0]:
            raise ValueError(f"container {name!r} is too small for the result")
        if ops._is_torch(dst):
            dst[: src.shape[0]].copy_(src)
        elif isinstance(dst, np.ndarray):
            dst[: src.shape[0]] = src
        else:
            raise UnsupportedSdfg(f"container {name!r}: results can be written into numpy arrays and torch tensors only")
    else:
        env[name] = value


@dataclass
class SdfgJsonProgram:
    """An executable view of a dumped SDFG: ``run(*arguments)`` in ``sdfg['arguments']`` order."""

    name: str
    arguments: List[str]
    containers: Dict[str, dict]
    steps: List[Step]
    nodes_run: List[str] = field(default_factory=list)

    def library_nodes(self) -> List[str]:
        return [s.code for s in self.steps]

    def _operand(self, env: dict, ref):
        if isinstance(ref, tuple):  # constant node
            return float(ref[1])
        if ref not in env:
            raise KeyError(f"container {ref!r} is read before anything wrote it")
        return env[ref]

    def run(self, *args, symbols: Optional[Dict[str, int]] = None):
        """Executes the library nodes. Arrays are numpy arrays (host path with transfers), CUDA torch tensors or
        ``ops.DeviceArray``; integer arguments become symbol values. Returns the dict of containers written."""
        if len(args) != len(self.arguments):
            raise TypeError(f"{self.name}: expected {len(self.arguments)} arguments, got {len(args)}")
        env: dict = {}
        sym: Dict[str, int] = dict(symbols or {})
        for name, value in zip(self.arguments, args):
            if isinstance(value, (int, np.integer)):
                sym[name] = int(value)
            env[name] = value
        written: Dict[str, object] = {}
        registry = N.LibraryNodeDispatcherRegistry.instance()
        self.nodes_run = []
        for st in self.steps:
            f = st.fields
            ev = lambda e: evaluate(e, sym)  # noqa: E731
            shape = [ev(d) for d in f.get("shape", [])]
            local: dict = {}
            node = None
            if st.code == "GEMM":
                self._gemm(st, env, sym, written)
                self.nodes_run.append(st.code)
                continue
            if st.code == "ml::MatMul":
                a = _view(self._operand(env, st.inputs["A"]), [ev(d) for d in f["shape_a"]])
                b = _view(self._operand(env, st.inputs["B"]), [ev(d) for d in f["shape_b"]])
                if ev(f.get("offset_a", 0)) or ev(f.get("offset_b", 0)):
                    raise UnsupportedSdfg(f"MatMul {st.element_id}: operand offsets")
                local = {"A": a, "B": b}
                node = N.MatMulNode(inputs=["A", "B"], outputs=["Y"])
            elif st.code == "ml::Softmax":
                local = {"X": _view(self._operand(env, st.inputs["X"]), shape)}
                node = N.SoftmaxNode(inputs=["X"], outputs=["Y"], axes=[int(a) for a in f["axes"]], keepdims=bool(f.get("keepdims", False)))
            elif st.code in _REDUCE:
                local = {"X": _view(self._operand(env, st.inputs["X"]), shape)}
                node = N.ReduceNode(inputs=["X"], outputs=["Y"], op=_REDUCE[st.code], axes=[int(a) for a in f["axes"]],
                                    keepdims=bool(f.get("keepdims", False)))
            elif st.code == "ml::Conv":
                kshape = [ev(d) for d in f["kernel_shape"]]
                c_out, group = ev(f["output_channels"]), ev(f.get("group", 1))
                local = {"X": _view(self._operand(env, st.inputs["X"]), shape),
                         "W": _view(self._operand(env, st.inputs["W"]), [c_out, shape[1] // group] + kshape)}
                ins = ["X", "W"]
                if "B" in st.inputs:
                    local["B"] = _view(self._operand(env, st.inputs["B"]), [c_out])
                    ins.append("B")
                node = N.ConvNode(inputs=ins, outputs=["Y"], strides=[ev(d) for d in f["strides"]], pads=[ev(d) for d in f["pads"]],
                                  dilations=[ev(d) for d in f["dilations"]], group=group)
            elif st.code in _UNARY:
                local = {"A": _view(self._operand(env, st.inputs["X"]), shape)}
                node = N.ElementwiseNode(inputs=["A"], outputs=["Y"], kind=_UNARY[st.code])
            elif st.code in _BINARY:
                local = {"A": _view(self._operand(env, st.inputs["A"]), shape), "B": _view(self._operand(env, st.inputs["B"]), shape)}
                node = N.ElementwiseNode(inputs=["A", "B"], outputs=["Y"], kind=_BINARY[st.code])
            elif st.code == "ml::Cast":
                target = _PRIMITIVE.get(int(f["target_type"]))
                if target is None:
                    raise UnsupportedSdfg(f"Cast {st.element_id}: target type {f['target_type']}")
                local = {"X": _view(self._operand(env, st.inputs["X"]), shape)}
                node = N.CastNode(inputs=["X"], outputs=["Y"], dtype=target)
            else:  # pragma: no cover - guarded by SUPPORTED_CODES
                raise UnsupportedSdfg(st.code)
            N.B200LibraryNodeMapper(with_transfers=isinstance(next(iter(local.values())), np.ndarray)).try_map(node)
            registry.dispatch(node, local)
            out_name = next(iter(st.outputs.values()))
            _store(env, out_name, local["Y"])
            written[out_name] = env[out_name]
            self.nodes_run.append(st.code)
        return written

    def _gemm(self, st: Step, env: dict, sym: dict, written: dict) -> None:
        """GEMM on flat buffers with leading dimensions, as generated code calls BLAS (gemm_node.cpp:441-520)."""
        f = st.fields
        ev = lambda e: evaluate(e, sym)  # noqa: E731
        m, n, k = ev(f["m"]), ev(f["n"]), ev(f["k"])
        lda, ldb, ldc = ev(f["lda"]), ev(f["ldb"]), ev(f["ldc"])
        prec = f["precision"]
        prec = chr(prec) if isinstance(prec, int) else str(prec)
        layout, ta, tb = int(f["layout"]), int(f["trans_a"]) != ops.NO_TRANS, int(f["trans_b"]) != ops.NO_TRANS
        a, b = self._operand(env, st.inputs["__A"]), self._operand(env, st.inputs["__B"])
        alpha = self._scalar(env, st.inputs.get("__alpha", ("const", "1.0")))
        beta = self._scalar(env, st.inputs.get("__beta", ("const", "0.0")))
        c_name = st.outputs["__C"]
        row_major = layout == ops.ROW_MAJOR
        c_rows = m if row_major else n
        if env.get(c_name) is None:
            if beta != 0.0:
                raise KeyError(f"GEMM {st.element_id}: beta != 0 but container {c_name!r} holds nothing")
            env[c_name] = ops._empty(_flat(a), (c_rows * ldc,), None)
        c = env[c_name]
        want = _PRECISION_DTYPE.get(prec)
        have = str(getattr(_flat(a), "dtype", "")).replace("torch.", "")
        if want is None or have != want:
            raise TypeError(f"GEMM {st.element_id}: precision {prec!r} but operand of type {have}")
        ops.gemm_strided(prec, layout, ta, tb, m, n, k, alpha, _flat(a), lda, _flat(b), ldb, beta, _flat(c), ldc)
        written[c_name] = c

    def _scalar(self, env: dict, ref) -> float:
        v = self._operand(env, ref)
        if isinstance(v, (int, float)):
            return float(v)
        return float(np.asarray(v.cpu() if ops._is_torch(v) else v).reshape(-1)[0])


def load(source) -> SdfgJsonProgram:
    """``source``: a path to a dumped ``<name>.json``, a JSON string, or the parsed dict."""
    if isinstance(source, dict):
        j = source
    else:
        text = str(source)
        if text.lstrip().startswith("{"):
            j = json.loads(text)
        else:
            with open(text) as fh:
                j = json.load(fh)
    for key in ("name", "containers", "arguments", "root"):
        if key not in j:
            raise ValueError(f"not an SDFG dump: missing {key!r}")
    if j["root"].get("type") != "sequence":
        raise ValueError("not a structured SDFG: root is not a sequence")
    return SdfgJsonProgram(name=j["name"], arguments=list(j["arguments"]), containers=dict(j["containers"]), steps=_sequence_steps(j["root"]))
