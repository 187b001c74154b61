"""``@native`` front end: the entry point docc exposes as ``docc.python.native``
(python/docc/python/python_program.py:713-747), for the subset of Python that lowers to the
library nodes of the hot path.

The reference parses the function's AST into an SDFG, where ``a @ b`` becomes a GEMM node
(python/docc/python/functions/numpy.py:256-479,1869-1980), ``scipy.special.softmax`` a Softmax
node (functions/scipy.py:61-124), reductions and element-wise numpy calls tensor nodes. This
module does the same walk over the AST, per call signature, and produces a ``nodes.Program``: a
straight-line schedule of library nodes. Scheduling for the ``cuda`` target maps every node to the
B200 runtime (no expansion into loop nests) and keeps intermediates on the device between the one
H2D per argument and the one D2H per result.

Only ``target="cuda"`` (alias ``"b200"``) is provided here. The CPU targets (``none``,
``sequential``, ``openmp``) belong to docc itself; asking for them raises instead of silently
computing on the host.
"""
from __future__ import annotations

import ast
import inspect
import textwrap
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np

from .. import nodes as N
from .. import ops

__all__ = ["native", "PythonProgram", "register_target_overrides", "install_docc_overrides"]

_CUDA_TARGETS = ("cuda", "b200")
_target_overrides: Dict[str, Tuple[object, object]] = {}


def register_target_overrides(name, schedule_fn, compile_fn):
    """Same hook as docc's ``register_target_overrides`` (python/docc/python/target_registry.py:22-43):
    ``schedule_fn(program, category, options)`` and ``compile_fn(program, ...)`` replace the built-in steps."""
    _target_overrides[name] = (schedule_fn, compile_fn)


def install_docc_overrides() -> bool:
    """When docc itself is importable, registers a ``"b200"`` target with it through docc's own hook
    (``register_target_overrides``, python/docc/python/target_registry.py:22-43). Returns False when docc is
    not installed.

    * ``schedule_fn(sdfg, category, options)`` forwards to ``sdfg.schedule("b200", category, remote_tuning)``: in a
      docc built with the B200 plugin that branch runs ``b200_scheduling_passes`` (the library-node mapper), the way
      the ``etsoc`` branch runs ``et_scheduling_passes`` (python/bindings/py_structured_sdfg.cpp:302-348).
    * ``compile_fn(sdfg, output_folder, instrumentation_mode, capture_args, options)`` calls the binding exactly as
      it is declared, ``_compile(output_folder, target, instrumentation_mode, capture_args)``
      (python/bindings/bindings.cpp:166-172). That signature has no room for extra flags, and the stock driver only
      adds target flags for the names it knows (py_structured_sdfg.cpp:486-550), so the header and the runtime reach
      the compiler through its environment (``CPATH`` for ``#include <docc_b200/rt.h>``, ``LIBRARY_PATH`` for the
      linker), and ``libdocc_b200_rt.so`` is loaded into the process with global visibility first so that the
      generated library's ``docc_b200_*`` references resolve when ``CompiledSDFG`` opens it with ``ctypes.CDLL``.
      A docc rebuilt with the plugin passes the same flags itself (``b200_get_host_additional_compile_args`` /
      ``b200_get_host_additional_link_args``); the environment route is then redundant and harmless.
    """
    try:
        from docc.python import target_registry  # type: ignore
    except Exception:
        return False
    import ctypes
    import os

    from ..build import INCLUDE, LIB_DIR, LIB_PATH

    def schedule_fn(sdfg, category, options=None):
        sdfg.schedule("b200", category, bool((options or {}).get("remote_tuning", False)))

    def _prepend(var, value):
        old = os.environ.get(var)
        os.environ[var] = value if not old else value + os.pathsep + old
        return old

    def compile_fn(sdfg, output_folder, instrumentation_mode, capture_args, options=None):
        ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        saved = {var: _prepend(var, val) for var, val in (("CPATH", INCLUDE), ("LIBRARY_PATH", LIB_DIR))}
        try:
            return sdfg._compile(output_folder, "b200", instrumentation_mode, capture_args)
        finally:
            for var, old in saved.items():
                if old is None:
                    os.environ.pop(var, None)
                else:
                    os.environ[var] = old

    target_registry.register_target_overrides("b200", schedule_fn, compile_fn)
    return True


@dataclass
class _Sym:
    """A tensor-valued name during AST translation: container name, shape, dtype."""

    name: str
    shape: Tuple[int, ...]
    dtype: np.dtype
    transposed_of: Optional["_Sym"] = None  # set for `x.T` of a 2-D tensor: folded into the consuming GEMM

    @property
    def ndim(self):
        return len(self.shape)


class UnsupportedSyntax(NotImplementedError):
    pass


_UNARY_NUMPY = {"exp": "exp", "tanh": "tanh", "sqrt": "sqrt", "abs": "abs", "absolute": "abs"}
_BINARY_NUMPY = {"add": "add", "subtract": "sub", "multiply": "mul", "divide": "div", "maximum": "max", "minimum": "min"}
_REDUCE_NUMPY = {"sum": "sum", "max": "max", "amax": "max", "min": "min", "amin": "min", "mean": "mean", "std": "std"}
_BINOPS = {ast.Add: "add", ast.Sub: "sub", ast.Mult: "mul", ast.Div: "div"}


class _Builder(ast.NodeVisitor):
    """Walks a function body and emits library nodes (the role of docc's ASTParser + handlers)."""

    def __init__(self, arg_names: List[str], args):
        self.env: Dict[str, object] = {}
        self.nodes: List[N.LibraryNode] = []
        self.results: List[str] = []
        self.counter = 0
        self.tensor_args: List[str] = []
        for name, value in zip(arg_names, args):
            if isinstance(value, np.ndarray):
                self.env[name] = _Sym(name, tuple(value.shape), value.dtype)
                self.tensor_args.append(name)
            else:
                self.env[name] = value  # python scalar: a compile-time constant of this specialisation

    # -- helpers --------------------------------------------------------------------------------
    def fresh(self, shape, dtype) -> _Sym:
        self.counter += 1
        return _Sym(f"_tmp{self.counter}", tuple(int(s) for s in shape), np.dtype(dtype))

    def emit(self, node: N.LibraryNode, out: _Sym) -> _Sym:
        node.outputs = [out.name]
        node.element_id = len(self.nodes)
        self.nodes.append(node)
        return out

    def materialise(self, v):
        if isinstance(v, _Sym) and v.transposed_of is not None:
            raise UnsupportedSyntax("a transposed view may only be used as a matmul operand")
        return v

    @staticmethod
    def dotted(node) -> str:
        parts = []
        while isinstance(node, ast.Attribute):
            parts.append(node.attr)
            node = node.value
        if isinstance(node, ast.Name):
            parts.append(node.id)
        return ".".join(reversed(parts))

    # -- statements -------------------------------------------------------------------------------
    def visit_FunctionDef(self, fn):
        for stmt in fn.body:
            if isinstance(stmt, ast.Expr) and isinstance(stmt.value, ast.Constant):
                continue  # docstring
            if isinstance(stmt, ast.Assign):
                if len(stmt.targets) != 1 or not isinstance(stmt.targets[0], ast.Name):
                    raise UnsupportedSyntax("only `name = expression` assignments are supported")
                self.env[stmt.targets[0].id] = self.visit(stmt.value)
            elif isinstance(stmt, ast.Return):
                value = stmt.value
                items = value.elts if isinstance(value, ast.Tuple) else [value]
                for item in items:
                    v = self.materialise(self.visit(item))
                    if not isinstance(v, _Sym):
                        raise UnsupportedSyntax("only tensors can be returned")
                    self.results.append(v.name)
                return
            else:
                raise UnsupportedSyntax(f"statement {type(stmt).__name__} is outside the supported subset")
        raise UnsupportedSyntax("function does not return a tensor")

    # -- expressions -------------------------------------------------------------------------------
    def visit_Name(self, node):
        if node.id not in self.env:
            raise UnsupportedSyntax(f"unknown name {node.id}")
        return self.env[node.id]

    def visit_Constant(self, node):
        return node.value

    def visit_UnaryOp(self, node):
        v = self.visit(node.operand)
        if isinstance(node.op, ast.USub):
            if isinstance(v, _Sym):
                return self.emit(N.ElementwiseNode(inputs=[self.materialise(v).name], kind="scale", value=-1.0), self.fresh(v.shape, v.dtype))
            return -v
        raise UnsupportedSyntax("unary operator")

    def visit_Attribute(self, node):
        if node.attr == "T":
            v = self.visit(node.value)
            if isinstance(v, _Sym) and v.ndim == 2:
                return _Sym(v.name, (v.shape[1], v.shape[0]), v.dtype, transposed_of=v)
        raise UnsupportedSyntax(f"attribute {self.dotted(node)}")

    def visit_BinOp(self, node):
        a, b = self.visit(node.left), self.visit(node.right)
        if isinstance(node.op, ast.MatMult):
            return self.matmul(a, b)
        kind = _BINOPS.get(type(node.op))
        if kind is None:
            raise UnsupportedSyntax(f"operator {type(node.op).__name__}")
        return self.binary(kind, a, b)

    def visit_Call(self, node):
        name = self.dotted(node.func)
        base = name.split(".")[-1]
        args = [self.visit(a) for a in node.args]
        kwargs = {k.arg: self.visit(k.value) for k in node.keywords}
        if name in ("np.matmul", "numpy.matmul", "np.dot", "numpy.dot"):
            return self.matmul(args[0], args[1])
        if name in ("scipy.special.softmax", "special.softmax", "softmax"):
            x = self.materialise(args[0])
            axis = kwargs.get("axis", args[1] if len(args) > 1 else None)
            axes = list(range(x.ndim)) if axis is None else ([axis] if np.isscalar(axis) else list(axis))
            return self.emit(N.SoftmaxNode(inputs=[x.name], axes=axes), self.fresh(x.shape, x.dtype))
        if name in ("scipy.special.erf", "special.erf"):
            x = self.materialise(args[0])
            return self.emit(N.ElementwiseNode(inputs=[x.name], kind="erf"), self.fresh(x.shape, x.dtype))
        if name.startswith(("np.", "numpy.")) and base in _UNARY_NUMPY:
            x = self.materialise(args[0])
            return self.emit(N.ElementwiseNode(inputs=[x.name], kind=_UNARY_NUMPY[base]), self.fresh(x.shape, x.dtype))
        if name.startswith(("np.", "numpy.")) and base in _BINARY_NUMPY:
            return self.binary(_BINARY_NUMPY[base], args[0], args[1])
        if name.startswith(("np.", "numpy.")) and base in _REDUCE_NUMPY:
            x = self.materialise(args[0])
            axis = kwargs.get("axis", args[1] if len(args) > 1 else None)
            keepdims = bool(kwargs.get("keepdims", False))
            axes = list(range(x.ndim)) if axis is None else ([axis] if np.isscalar(axis) else list(axis))
            norm = sorted(a % x.ndim for a in axes)
            shape = tuple((1 if d in norm else s) for d, s in enumerate(x.shape) if keepdims or d not in norm)
            return self.emit(N.ReduceNode(inputs=[x.name], op=_REDUCE_NUMPY[base], axes=axes, keepdims=keepdims),
                             self.fresh(shape, x.dtype))
        if name in ("np.transpose", "numpy.transpose") and len(args) == 1 and isinstance(args[0], _Sym) and args[0].ndim == 2:
            v = args[0]
            return _Sym(v.name, (v.shape[1], v.shape[0]), v.dtype, transposed_of=v)
        raise UnsupportedSyntax(f"call to {name} is outside the supported subset")

    # -- node construction ----------------------------------------------------------------------------
    def matmul(self, a, b):
        if not (isinstance(a, _Sym) and isinstance(b, _Sym)):
            raise UnsupportedSyntax("matmul of non-tensors")
        if a.dtype != b.dtype:
            raise UnsupportedSyntax("matmul operands must have the same element type")
        # integer element types are rejected by MatMulNode::expand (matmul_node.cpp:338-341)
        if a.dtype.kind != "f":
            raise N.InvalidSDFGException("matmul: integer element types are not supported")
        ta, tb = a.transposed_of is not None, b.transposed_of is not None
        if a.ndim == 2 and b.ndim == 2:
            if a.shape[1] != b.shape[0]:
                raise N.InvalidSDFGException(f"matmul: shapes {a.shape} and {b.shape} do not align")
            prec = {"float64": "d", "float32": "s", "float16": "h"}[a.dtype.name]
            # what add_gemm builds: GEMM(BLAS, RowMajor, alpha = 1, beta = 0) (py_structured_sdfg_builder.cpp:677-712)
            node = N.GEMMNode(inputs=[a.name, b.name], precision=prec, trans_a=ta, trans_b=tb)
            return self.emit(node, self.fresh((a.shape[0], b.shape[1]), a.dtype))
        if ta or tb:
            raise UnsupportedSyntax("transposed operands of a batched matmul")
        if a.ndim == 1 or b.ndim == 1:
            raise UnsupportedSyntax("vector operands (DOT / GEMV) are not library nodes of this path")
        if a.shape[-1] != b.shape[-2]:
            raise N.InvalidSDFGException(f"matmul: shapes {a.shape} and {b.shape} do not align")
        batch = np.broadcast_shapes(a.shape[:-2], b.shape[:-2])
        return self.emit(N.MatMulNode(inputs=[a.name, b.name]), self.fresh(tuple(batch) + (a.shape[-2], b.shape[-1]), a.dtype))

    def binary(self, kind, a, b):
        a, b = self.materialise(a), self.materialise(b)
        if isinstance(a, _Sym) and isinstance(b, _Sym):
            if a.shape == b.shape and a.dtype == b.dtype:
                return self.emit(N.ElementwiseNode(inputs=[a.name, b.name], kind=kind), self.fresh(a.shape, a.dtype))
            raise UnsupportedSyntax("broadcasting between tensors of different shape")
        if isinstance(a, _Sym) and np.isscalar(b):
            if kind == "mul":
                return self.emit(N.ElementwiseNode(inputs=[a.name], kind="scale", value=float(b)), self.fresh(a.shape, a.dtype))
            if kind == "div":
                return self.emit(N.ElementwiseNode(inputs=[a.name], kind="scale", value=1.0 / float(b)), self.fresh(a.shape, a.dtype))
            raise UnsupportedSyntax("tensor +/- scalar")
        if np.isscalar(a) and isinstance(b, _Sym) and kind == "mul":
            return self.binary("mul", b, a)
        if np.isscalar(a) and np.isscalar(b):
            return {"add": a + b, "sub": a - b, "mul": a * b, "div": a / b}[kind]
        raise UnsupportedSyntax("operand combination")


class PythonProgram:
    """Callable wrapper around a Python function, specialised per argument signature
    (same role and constructor arguments as docc's PythonProgram, python_program.py:100-157)."""

    def __init__(self, func, target="none", category="server", instrumentation_mode=None, capture_args=None,
                 remote_tuning=False):
        self.func = func
        self.name = func.__name__
        self.target = target
        self.category = category
        self.instrumentation_mode = instrumentation_mode
        self.capture_args = capture_args
        self.remote_tuning = remote_tuning
        self.cache: Dict[str, N.Program] = {}
        self.last_program: Optional[N.Program] = None

    def _signature_key(self, args) -> str:
        parts = []
        for a in args:
            if isinstance(a, np.ndarray):
                parts.append(f"{a.dtype.name}{list(a.shape)}")
            else:
                parts.append(f"{type(a).__name__}:{a!r}")
        return "|".join(parts)

    def compile(self, *args) -> N.Program:
        if self.target not in _CUDA_TARGETS and self.target not in _target_overrides:
            raise NotImplementedError(
                f"target {self.target!r}: this package provides the cuda target only; docc's CPU targets are not "
                "re-implemented and there is no host fallback")
        key = self._signature_key(args)
        if key in self.cache:
            return self.cache[key]
        try:
            source = textwrap.dedent(inspect.getsource(self.func))
        except OSError as exc:
            raise UnsupportedSyntax(f"the source of {self.name} is not available for translation") from exc
        tree = ast.parse(source)
        fn = next(n for n in ast.walk(tree) if isinstance(n, ast.FunctionDef) and n.name == self.func.__name__)
        arg_names = [a.arg for a in fn.args.args]
        if len(arg_names) != len(args):
            raise TypeError(f"{self.name} takes {len(arg_names)} arguments, got {len(args)}")
        builder = _Builder(arg_names, args)
        builder.visit_FunctionDef(fn)
        program = N.Program(arguments=builder.tensor_args, nodes=builder.nodes, results=builder.results)
        for node in program.nodes:
            node.validate()
        if self.target in _target_overrides and _target_overrides[self.target][0] is not None:
            _target_overrides[self.target][0](program, self.category, {})
        else:
            program.map_to_target(with_transfers=False)  # schedule(): intermediates stay on the device
        self.cache[key] = program
        return program

    def __call__(self, *args):
        args = [np.ascontiguousarray(a) if isinstance(a, np.ndarray) else a for a in args]
        program = self.compile(*args)
        self.last_program = program
        tensors = [a for a in args if isinstance(a, np.ndarray)]
        dev = [ops.DeviceArray.from_numpy(a) for a in tensors]  # one H2D per argument
        out = program.run(*dev)
        outs = out if isinstance(out, tuple) else (out,)
        host = tuple(o.to_numpy() for o in outs)  # one D2H per result
        return host[0] if len(host) == 1 else host


def native(func=None, *, target="none", category="server", instrumentation_mode=None, capture_args=None, remote_tuning=False):
    """Decorator with the signature of ``docc.python.native``.

        @native(target="cuda")
        def f(a, b):
            return a @ b
    """
    def wrap(f):
        return PythonProgram(f, target=target, category=category, instrumentation_mode=instrumentation_mode,
                             capture_args=capture_args, remote_tuning=remote_tuning)

    return wrap if func is None else wrap(func)
