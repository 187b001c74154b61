"""Reader for docc's SDFG JSON dumps (docc_b200/sdfg_json.py): planning on CPU, execution against the oracle on a GPU.

The fixtures under tests/golden/sdfg_*.json are written by tests/golden/make_sdfg_json.py after the field names of
docc's JSONSerializer and node serializers."""
import json
import os

import numpy as np
import pytest

from conftest import ROOT, relerr
from docc_b200 import sdfg_json
from oracle import oracle

GOLDEN = os.path.join(ROOT, "tests", "golden")


def fixture(name):
    return os.path.join(GOLDEN, name + ".json")


def test_expressions():
    ev = sdfg_json.evaluate
    assert ev("1000") == 1000
    assert ev("_s0*_s1", {"_s0": 3, "_s1": 5}) == 15
    assert ev("2 + _s0", {"_s0": 7}) == 9
    assert ev("(_s0 + 2 - 3)/1 + 1", {"_s0": 9}) == 9
    assert ev("idiv(_s0 + 2*1 - 1*(3 - 1) - 1, 2) + 1", {"_s0": 9}) == 5  # conv output extent, stride 2
    assert ev("max(_s0, 4)", {"_s0": 2}) == 4
    assert ev("_s0**2", {"_s0": 4}) == 16
    assert ev(12) == 12
    with pytest.raises(KeyError):
        ev("_s3 + 1", {})
    with pytest.raises(sdfg_json.UnsupportedSdfg):
        ev("_s0 / 2", {"_s0": 3})  # not integer valued
    with pytest.raises(sdfg_json.UnsupportedSdfg):
        ev("__import__('os')")


def test_plan_gemm_softmax():
    prog = sdfg_json.load(fixture("sdfg_gemm_softmax"))
    assert prog.name == "gemm_softmax"
    assert prog.arguments == ["A", "B", "Y", "_s0", "_s1", "_s2"]
    assert prog.library_nodes() == ["GEMM", "ml::Softmax"]
    gemm, softmax = prog.steps
    assert gemm.inputs["__A"] == "A" and gemm.inputs["__B"] == "B" and gemm.outputs == {"__C": "tmp"}
    assert gemm.inputs["__alpha"] == ("const", "1.0") and gemm.inputs["__beta"] == ("const", "0.0")
    assert softmax.inputs == {"X": "tmp"} and softmax.outputs == {"Y": "Y"}
    assert sdfg_json.element_dtype(prog.containers["A"]) == "float64"
    assert sdfg_json.element_dtype(prog.containers["_s0"]) == "int64"


def test_plan_orders_by_dataflow_not_by_position():
    with open(fixture("sdfg_conv_relu")) as fh:
        j = json.load(fh)
    for block in j["root"]["children"]:
        block["dataflow"]["nodes"].reverse()
        block["dataflow"]["edges"].reverse()
    prog = sdfg_json.load(j)
    assert prog.library_nodes() == ["ml::Conv", "ml::ReLU"]
    assert prog.steps[0].inputs == {"X": "X", "W": "W", "B": "Bias"}


def test_unsupported_elements_are_refused():
    with pytest.raises(sdfg_json.UnsupportedSdfg, match="tasklet"):
        sdfg_json.load(fixture("sdfg_scalar_code"))
    with open(fixture("sdfg_gemm_softmax")) as fh:
        j = json.load(fh)
    j["root"]["children"][0]["dataflow"]["edges"][0]["subset"] = ["i"]
    with pytest.raises(sdfg_json.UnsupportedSdfg, match="subset"):
        sdfg_json.load(j)
    with open(fixture("sdfg_gemm_softmax")) as fh:
        j = json.load(fh)
    j["root"]["children"].append({"type": "for", "element_id": 999, "indvar": "i", "init": "0", "condition": "i < 4", "update": "1 + i",
                                  "root": {"type": "sequence", "element_id": 1000, "children": [], "transitions": []}})
    with pytest.raises(sdfg_json.UnsupportedSdfg, match="for"):
        sdfg_json.load(j)
    with pytest.raises(ValueError, match="not an SDFG dump"):
        sdfg_json.load({"name": "x"})


@pytest.mark.gpu
def test_run_gemm_softmax_host_and_device(rt):
    import torch

    prog = sdfg_json.load(fixture("sdfg_gemm_softmax"))
    rng = np.random.RandomState(11)
    m, n, k = 37, 50, 29
    a, b = rng.rand(m, k), rng.rand(k, n)
    ref = oracle.softmax(oracle.gemm(a, b), [1])
    y = np.zeros((m, n))
    written = prog.run(a.ravel(), b.ravel(), y.ravel(), m, n, k)  # flat host buffers, as generated code passes them
    assert prog.nodes_run == ["GEMM", "ml::Softmax"] and set(written) == {"tmp", "Y"}
    assert relerr(y, ref) <= 1e-12
    ya = torch.zeros(m * n, dtype=torch.float64, device="cuda")
    prog.run(torch.from_numpy(a).cuda().reshape(-1), torch.from_numpy(b).cuda().reshape(-1), ya, m, n, k)
    assert relerr(ya.cpu().numpy().reshape(m, n), ref) <= 1e-12


@pytest.mark.gpu
def test_run_conv_relu(rt):
    prog = sdfg_json.load(fixture("sdfg_conv_relu"))
    rng = np.random.RandomState(12)
    nb = 3
    x = rng.randn(nb, 4, 9, 10).astype(np.float32)
    w = rng.randn(6, 4, 3, 3).astype(np.float32)
    bias = rng.randn(6).astype(np.float32)
    ref = np.maximum(oracle.conv(x, w, bias, pads=[1, 1, 1, 1]), 0)
    y = np.zeros((nb, 6, 9, 10), np.float32)
    prog.run(x.ravel(), w.ravel(), bias, y.ravel(), nb)
    assert relerr(y, ref) <= 1e-4


@pytest.mark.gpu
def test_run_matmul_add_mean_cast(rt):
    prog = sdfg_json.load(fixture("sdfg_matmul_add_mean_cast"))
    assert prog.library_nodes() == ["ml::MatMul", "ml::Add", "ml::Mean", "ml::Cast"]
    rng = np.random.RandomState(13)
    nb = 5
    a = rng.randn(nb, 8, 16).astype(np.float32)
    b = rng.randn(16, 12).astype(np.float32)
    c = rng.randn(nb, 8, 12).astype(np.float32)
    summed = oracle.binary(0, oracle.matmul(a, b), c)  # binary op 0 = add
    ref = oracle.reduce(oracle.RED_MEAN, summed, [2]).astype(np.float64)
    y = np.zeros((nb, 8))
    prog.run(a.ravel(), b.ravel(), c.ravel(), y.ravel(), nb)
    assert y.dtype == np.float64 and relerr(y, ref) <= 1e-4
