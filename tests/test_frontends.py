"""Front ends: ``@native`` (docc.python.native) and ``torch.compile(backend="docc")`` (docc.torch).
CPU tests check the translation into library nodes; GPU tests run the reference's own test programs
(python/tests/python/functions/numpy/test_linalg.py, .../scipy/test_scipy_softmax.py,
mlir/integration/torch/test_matmul.py, test_linear.py, test_conv2d.py) end to end."""
import numpy as np
import pytest
import scipy.special
import torch
import torch.nn as nn
import torch.nn.functional as F

import docc_b200.torch as docc_torch
from conftest import relerr
from docc_b200 import nodes
from docc_b200.python import UnsupportedSyntax, native


# ---- translation (no GPU) ------------------------------------------------------------------------------
def test_matmul_operator_becomes_a_blas_gemm_node():
    @native(target="cuda")
    def matmul_op(a, b):
        return a @ b

    prog = matmul_op.compile(np.zeros((10, 10)), np.zeros((10, 10)))
    assert [n.code for n in prog.nodes] == ["GEMM"]
    g = prog.nodes[0]
    # add_gemm: precision from dtype, RowMajor, NoTrans, alpha 1, beta 0 (py_structured_sdfg_builder.cpp:677-712)
    assert (g.precision, g.layout, g.trans_a, g.trans_b, g.alpha, g.beta) == ("d", 101, False, False, 1.0, 0.0)
    assert g.implementation_type == nodes.IMPL_B200_WITHOUT_TRANSFERS  # mapped, not expanded
    assert prog.loop_report() == {"library_nodes": 1, "maps": 0, "fors": 0}


def test_softmax_and_chain_translation():
    @native(target="cuda")
    def f(a, b):
        c = np.matmul(a, b.T)
        return scipy.special.softmax(c, axis=0) * 0.5

    prog = f.compile(np.zeros((4, 6), dtype=np.float32), np.zeros((5, 6), dtype=np.float32))
    assert [n.code for n in prog.nodes] == ["GEMM", "ml::Softmax", "ml::Elementwise"]
    assert prog.nodes[0].trans_b and prog.nodes[0].precision == "s"
    assert list(prog.nodes[1].axes) == [0]
    js = prog.to_json()
    assert js["nodes"][1]["code"] == "ml::Softmax" and js["results"] == [prog.nodes[2].outputs[0]]


def test_batched_matmul_and_reductions_translate():
    @native(target="cuda")
    def f(a, b):
        return np.sum(a @ b, axis=1)

    prog = f.compile(np.zeros((2, 10, 10)), np.zeros((2, 10, 10)))
    assert [n.code for n in prog.nodes] == ["ml::MatMul", "ml::Sum"]


def test_unsupported_python_and_targets_raise():
    @native(target="cuda")
    def loop(a):
        for i in range(3):
            a = a @ a
        return a

    with pytest.raises(UnsupportedSyntax):
        loop.compile(np.zeros((2, 2)))

    @native  # default target "none": a CPU target of docc, not provided here
    def g(a):
        return a @ a

    with pytest.raises(NotImplementedError):
        g(np.zeros((2, 2)))

    @native(target="cuda")
    def ints(a):
        return a @ a

    with pytest.raises(nodes.InvalidSDFGException):
        ints.compile(np.zeros((2, 2), dtype=np.int64))


def test_softmax_keepdims_is_rejected_like_the_node():
    with pytest.raises(nodes.InvalidSDFGException):
        nodes.SoftmaxNode(inputs=["x"], outputs=["y"], keepdims=True).validate()


def test_registry_first_registration_wins():
    reg = nodes.LibraryNodeDispatcherRegistry()
    assert reg.register_library_node_dispatcher("GEMM::X", lambda n, e: None)
    assert not reg.register_library_node_dispatcher("GEMM::X", lambda n, e: 1 / 0)
    with pytest.raises(nodes.InvalidSDFGException):
        reg.dispatch(nodes.GEMMNode(inputs=["a", "b"], outputs=["c"], implementation_type="Y"), {})


def test_install_docc_overrides_calls_the_bindings_as_they_are_declared(monkeypatch, tmp_path):
    """A stand-in ``docc.python.target_registry`` records what gets registered; a stand-in SDFG records how the hooks
    call it. ``_compile`` is bound as (output_folder, target, instrumentation_mode, capture_args) and ``schedule`` as
    (target, category, remote_tuning) (python/bindings/bindings.cpp:157-172); the hooks themselves are invoked with
    the argument lists of python/docc/python/python_program.py:289-314."""
    import sys
    import types

    import docc_b200.python as dpy
    from docc_b200 import build

    registered = {}
    docc, pkg, reg = types.ModuleType("docc"), types.ModuleType("docc.python"), types.ModuleType("docc.python.target_registry")
    reg.register_target_overrides = lambda name, schedule_fn, compile_fn=None: registered.update({name: (schedule_fn, compile_fn)})
    docc.python, pkg.target_registry = pkg, reg
    for name, mod in (("docc", docc), ("docc.python", pkg), ("docc.python.target_registry", reg)):
        monkeypatch.setitem(sys.modules, name, mod)
    assert dpy.install_docc_overrides() is True
    schedule_fn, compile_fn = registered["b200"]

    class FakeSDFG:
        def __init__(self):
            self.calls = []

        def schedule(self, target, category, remote_tuning=False):  # exactly the bound parameters
            self.calls.append(("schedule", target, category, remote_tuning))

        def _compile(self, output_folder, target, instrumentation_mode="", capture_args=False):
            import os

            self.calls.append(("_compile", output_folder, target, instrumentation_mode, capture_args))
            self.env = (os.environ.get("CPATH", ""), os.environ.get("LIBRARY_PATH", ""))
            return output_folder + "/libx.so"

    sdfg = FakeSDFG()
    schedule_fn(sdfg, "server", {"remote_tuning": False})
    monkeypatch.setenv("CPATH", "/somewhere/else")
    monkeypatch.delenv("LIBRARY_PATH", raising=False)
    assert compile_fn(sdfg, str(tmp_path), "ols", True, {}) == str(tmp_path) + "/libx.so"
    assert sdfg.calls == [("schedule", "b200", "server", False), ("_compile", str(tmp_path), "b200", "ols", True)]
    # the header and the library were on the compiler's search paths during the call, and only during the call
    import os

    assert sdfg.env[0].split(os.pathsep)[0] == build.INCLUDE and "/somewhere/else" in sdfg.env[0]
    assert sdfg.env[1] == build.LIB_DIR
    assert os.environ["CPATH"] == "/somewhere/else" and "LIBRARY_PATH" not in os.environ


class Block(nn.Module):
    def __init__(self, d=64, heads=4, dff=128):
        super().__init__()
        self.h = heads
        self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.fc1, self.fc2 = nn.Linear(d, dff), nn.Linear(dff, d)

    def forward(self, x):
        B, S, d = x.shape
        qkv = self.qkv(self.ln1(x)).view(B, S, 3, self.h, d // self.h)
        q, k, v = qkv[:, :, 0].transpose(1, 2), qkv[:, :, 1].transpose(1, 2), qkv[:, :, 2].transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, S, d)
        x = x + self.proj(a)
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x))))


def lower_on_cpu(model, *inputs):
    captured = {}

    def backend(gm, example_inputs):
        captured["lowered"] = docc_torch._Lowered(gm)
        return gm.forward

    torch._dynamo.reset()
    torch.compile(model, backend=backend)(*inputs)
    return captured["lowered"]


def test_transformer_block_lowers_with_fused_epilogues():
    low = lower_on_cpu(Block(), torch.randn(2, 8, 64))
    calls = [s for s in low.steps if s[0] == "call"]
    fns = [s[2].__name__ for s in calls]
    assert fns.count("_linear") == 4 and fns.count("_sdpa") == 1 and fns.count("_layer_norm") == 2
    fused = [s[4] for s in calls if s[2].__name__ == "_linear"]
    assert sum(1 for k in fused if k.get("act")) == 1  # fc1 -> GELU
    assert sum(1 for k in fused if k.get("residual") is not None) == 2  # proj + x, fc2 + x
    assert "gelu" not in " ".join(fns) and not any(s[2].__name__ == "fn" and False for s in calls)


def test_linear_plus_broadcast_addend_is_not_folded_into_the_epilogue(monkeypatch):
    # The epilogue's residual is a full [.., out] tensor of the output type. `linear(x) + pos` with a broadcasting or
    # differently typed addend must run as linear followed by the add node, never hand the short buffer to the kernel.
    seen = []
    monkeypatch.setattr(docc_torch, "_dispatch", lambda node, *inputs: seen.append((node, inputs)) or torch.zeros(2, 8, 16))
    added = []
    monkeypatch.setattr(docc_torch, "_binary", lambda kind: (lambda a, b: added.append((kind, tuple(b.shape), b.dtype)) or a))
    x, w = torch.randn(2, 8, 4), torch.randn(16, 4)
    for other in (torch.randn(16), torch.randn(1, 8, 16), torch.randn(2, 8, 16, dtype=torch.float64)):
        seen.clear(), added.clear()
        docc_torch._linear(x, w, None, residual=other)
        assert len(seen) == 1 and not seen[0][0].has_residual and seen[0][1][3] is None
        assert added == [("add", tuple(other.shape), other.dtype)]
    seen.clear(), added.clear()
    docc_torch._linear(x, w, None, residual=torch.randn(2, 8, 16))  # exact shape and type: fused
    assert seen[0][0].has_residual and not added


def test_frontend_refuses_semantics_it_would_get_wrong():
    class CausalCross(nn.Module):
        def forward(self, q, k):
            return F.scaled_dot_product_attention(q, k, k, is_causal=True)

    low = lower_on_cpu(CausalCross(), torch.randn(1, 1, 4, 8), torch.randn(1, 1, 6, 8))
    sdpa = next(s for s in low.steps if s[0] == "call")
    with pytest.raises(docc_torch.UnsupportedGraph):
        sdpa[2](torch.randn(1, 1, 4, 8), torch.randn(1, 1, 6, 8), torch.randn(1, 1, 6, 8), is_causal=True)
    with pytest.raises(docc_torch.UnsupportedGraph):
        docc_torch._softmax(torch.randn(2, 2), -1, dtype=torch.float64)
    with pytest.raises(docc_torch.UnsupportedGraph):
        docc_torch._binary("div")(torch.randn(2), torch.randn(2), rounding_mode="floor")

    class InPlaceOnInput(nn.Module):
        def forward(self, x, y):
            x += y
            return x

    with pytest.raises(Exception) as e:
        lower_on_cpu(InPlaceOnInput(), torch.randn(3), torch.randn(3))
    assert "in-place" in str(e.value)

    class InPlaceOnIntermediate(nn.Module):
        def forward(self, x, y):
            z = x * y
            z += y
            return z

    low = lower_on_cpu(InPlaceOnIntermediate(), torch.randn(3), torch.randn(3))
    assert sum(1 for s in low.steps if s[0] == "call") == 2


def test_unsupported_torch_op_raises_instead_of_falling_back():
    class M(nn.Module):
        def forward(self, x):
            return torch.cumsum(x, dim=0)

    with pytest.raises(Exception) as e:
        lower_on_cpu(M(), torch.randn(3, 3))
    assert "no library node" in str(e.value)


def test_backend_is_registered_and_refuses_cpu_targets():
    assert "docc" in torch._dynamo.list_backends(None)
    docc_torch.set_backend_options(target="none")
    torch._dynamo.reset()
    with pytest.raises(Exception) as e:
        torch.compile(nn.Linear(4, 4), backend="docc")(torch.randn(2, 4))
    assert "cuda target only" in str(e.value)


# ---- end to end on the GPU -----------------------------------------------------------------------------------
@pytest.mark.gpu
def test_native_reference_programs(rt):
    @native(target="cuda")
    def matmul_op(a, b):
        return a @ b

    a, b = np.random.rand(10, 10), np.random.rand(10, 10)
    assert np.allclose(matmul_op(a, b), a @ b)  # test_linalg.py:5-14
    a32, b32 = a.astype(np.float32), b.astype(np.float32)
    assert np.allclose(matmul_op(a32, b32), a32 @ b32, rtol=1e-4)
    ab, bb = np.random.rand(2, 10, 10), np.random.rand(2, 10, 10)
    assert np.allclose(matmul_op(ab, bb), ab @ bb)  # test_linalg.py:49-58

    @native(target="cuda")
    def chained(a, b, c):
        return (a @ b) @ c

    assert np.allclose(chained(a, b, a), (a @ b) @ a)

    @native(target="cuda")
    def softmax_simple(A):
        return scipy.special.softmax(A, axis=0)

    @native(target="cuda")
    def softmax_all(A):
        return scipy.special.softmax(A)

    A = np.random.rand(10, 10)
    assert np.allclose(softmax_simple(A), scipy.special.softmax(A, axis=0))  # test_scipy_softmax.py:8-24
    assert np.allclose(softmax_all(A), scipy.special.softmax(A))  # test_scipy_softmax.py:27-44


@pytest.mark.gpu
def test_native_config1_and_config2(rt):
    @native(target="cuda")
    def gemm(a, b):
        return a @ b

    rng = np.random.RandomState(0)
    a, b = rng.rand(1000, 1000), rng.rand(1000, 1000)
    assert relerr(gemm(a, b), a @ b) <= 1e-12

    @native(target="cuda")
    def softmax(x):
        return scipy.special.softmax(x, axis=-1)

    torch.manual_seed(1)
    x = (3 * torch.randn(1024, 4096)).numpy()
    assert relerr(softmax(x), scipy.special.softmax(x.astype(np.float64), axis=-1)) <= 1e-4


@pytest.fixture
def docc_cuda():
    docc_torch.set_backend_options(target="cuda", category="server")
    torch._dynamo.reset()
    yield
    docc_torch.set_backend_options(target="none", category="server")


@pytest.mark.gpu
def test_torch_backend_reference_integration_cases(rt, docc_cuda):
    torch.manual_seed(815)  # mlir/integration/torch/conftest.py:5-8
    lin = nn.Linear(10, 5, bias=False)
    x = torch.randn(4, 10)
    assert torch.allclose(torch.compile(lin, backend="docc")(x), lin(x), rtol=1e-4, atol=1e-5)  # test_linear.py

    class MatMul(nn.Module):
        def forward(self, a, b):
            return torch.matmul(a, b)

    a, b = torch.randn(16, 32), torch.randn(32, 8)
    assert torch.allclose(torch.compile(MatMul(), backend="docc")(a, b), a @ b, rtol=1e-4, atol=1e-4)  # test_matmul.py

    conv = nn.Conv2d(3, 16, kernel_size=3, bias=False)
    img = torch.randn(1, 3, 32, 32)
    assert torch.allclose(torch.compile(conv, backend="docc")(img), conv(img), rtol=1e-4, atol=1e-5)  # test_conv2d.py:30-49
    # the cases the reference skips: bias and padding
    conv_b = nn.Conv2d(3, 16, kernel_size=3, padding=1, bias=True)
    assert torch.allclose(torch.compile(conv_b, backend="docc")(img), conv_b(img), rtol=1e-4, atol=1e-5)


@pytest.mark.gpu
def test_torch_backend_transformer_block(rt, docc_cuda):
    torch.manual_seed(4)
    model = Block(128, 4, 256).eval()
    x = torch.randn(2, 64, 128)
    ref = model(x)
    out = torch.compile(model, backend="docc")(x)
    assert relerr(out.detach().numpy(), ref.detach().numpy()) <= 1e-4
    mb, xb = Block(128, 2, 256).eval().cuda().bfloat16(), torch.randn(2, 128, 128).cuda().bfloat16()
    ref = mb(xb)
    out = torch.compile(mb, backend="docc")(xb)
    assert out.is_cuda and relerr(out.detach().float().cpu().numpy(), ref.detach().float().cpu().numpy()) <= 2e-2


@pytest.mark.gpu
def test_torch_backend_linear_plus_position_table_and_fp64_bias(rt, docc_cuda):
    class WithPos(nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = nn.Linear(32, 48)
            self.pos = nn.Parameter(torch.randn(1, 6, 48))
            self.vec = nn.Parameter(torch.randn(48))

        def forward(self, x):
            return (self.lin(x) + self.pos) if x.dim() == 3 else (self.lin(x) + self.vec)

    torch.manual_seed(9)
    m = WithPos().eval()
    x2 = torch.randn(5, 32)
    assert torch.allclose(torch.compile(m, backend="docc")(x2), m(x2), rtol=1e-4, atol=1e-5)
    x3 = torch.randn(4, 6, 32)
    torch._dynamo.reset()
    with pytest.raises(Exception) as e:  # [1, S, d] broadcast: refused by the add node, never read out of bounds
        torch.compile(m, backend="docc")(x3)
    assert "broadcasting" in str(e.value)
    torch._dynamo.reset()
    m64 = nn.Linear(24, 40).double().eval()
    x64 = torch.randn(7, 24, dtype=torch.float64)
    assert torch.allclose(torch.compile(m64, backend="docc")(x64), m64(x64), rtol=1e-12, atol=1e-12)


@pytest.mark.gpu
def test_compile_torch_entry_point(rt):
    model = nn.Sequential(nn.Linear(32, 64), nn.GELU(), nn.Linear(64, 16)).eval()
    x = torch.randn(8, 32)
    prog = docc_torch.compile_torch(model, x, target="cuda")
    assert torch.allclose(prog(x), model(x), rtol=1e-4, atol=1e-5)


def test_gemm_flop_terms_follow_the_alpha_and_beta_conditions():
    """GEMMNode::flops (gemm_node.cpp:341-356) multiplies each term by the condition it depends on; flop() is the
    all-true case, 2mnk + 2mn."""
    m, n, k = 7, 5, 3
    env = {"a": np.zeros((m, k)), "b": np.zeros((k, n))}
    g = nodes.GEMMNode(inputs=["a", "b"], outputs=["c"])
    res = m * n
    assert g.flop(env) == 2 * m * n * k + 2 * m * n
    assert g.flop() is None
    # alpha == 0: no product, no alpha scaling; the beta terms stay
    assert g.flops(env, alpha_non_zero=False) == 2 * res
    # alpha == 1: the product without the scaling multiply
    assert g.flops(env, alpha_non_ident=False) == res * k + res * (k - 1) + 2 * res
    # beta == 0: neither the scaling of C nor its addition
    assert g.flops(env, beta_non_zero=False) == res * k + res * (k - 1) + res
    # beta == 1: C is added unscaled
    assert g.flops(env, beta_non_ident=False) == res * k + res * (k - 1) + res + res
    # plain product (alpha 1, beta 0), the case the front ends emit: 2mnk - mn
    plain = nodes.GEMMNode(inputs=["a", "b"], outputs=["c"], alpha=1.0, beta=0.0)
    assert plain.flop_for_constants(env) == 2 * m * n * k - res
    assert nodes.GEMMNode(inputs=["a", "b"], outputs=["c"], alpha=0.5, beta=2.0).flop_for_constants(env) == g.flop(env)
    # transposed operands read their extents the other way round
    env_t = {"a": np.zeros((k, m)), "b": np.zeros((n, k))}
    assert nodes.GEMMNode(inputs=["a", "b"], outputs=["c"], trans_a=True, trans_b=True).flop(env_t) == g.flop(env)
