"""Writes tests/golden/sdfg_gemm_softmax.json and sdfg_conv_relu.json: SDFG dumps in docc's JSON wire format, built
field by field after ``JSONSerializer`` (sdfg/src/serializer/json_serializer.cpp:63-113 top level, :115-186 dataflow
nodes and edges, :188-199 block, :317-343 sequence, :355-430 types) and the node serializers (GEMM gemm_node.cpp:387-405,
Softmax / reductions ``shape`` ``axes`` ``keepdims``, Conv conv_node.cpp:552-600, element-wise nodes ``shape``).
docc itself cannot be built or imported in this environment, so the files are hand-assembled; run this script to
regenerate them."""
import json
import os

HERE = os.path.dirname(os.path.abspath(__file__))
DEBUG = {"has": False, "filename": "", "function": "", "start_line": 0, "start_column": 0, "end_line": 0, "end_column": 0}
STORAGE = {"value": "CPU_Stack", "allocation": "Unmanaged", "deallocation": "Unmanaged"}


def scalar(primitive):
    return {"type": "scalar", "primitive_type": primitive, "storage_type": STORAGE, "initializer": "", "alignment": 0}


def pointer(primitive):
    return {"type": "pointer", "pointee_type": scalar(primitive), "storage_type": STORAGE, "initializer": "", "alignment": 0}


class Builder:
    def __init__(self, name):
        self.j = {"name": name, "element_counter": 0, "type": "CPU", "return_type": scalar(0), "structures": [], "containers": {},
                  "arguments": [], "externals": [], "metadata": {}, "root": None}
        self.counter = 0
        self.blocks = []

    def eid(self):
        self.counter += 1
        return self.counter

    def container(self, name, type_json, argument=False):
        self.j["containers"][name] = type_json
        if argument:
            self.j["arguments"].append(name)

    def block(self, nodes, edges):
        self.blocks.append({"type": "block", "element_id": self.eid(), "debug_info": DEBUG,
                            "dataflow": {"type": "dataflow", "nodes": nodes, "edges": edges}})

    def access(self, data):
        return {"element_id": self.eid(), "debug_info": DEBUG, "type": "access_node", "data": data}

    def constant(self, data, primitive):
        return {"element_id": self.eid(), "debug_info": DEBUG, "type": "constant_node", "data": data, "data_type": scalar(primitive)}

    def library(self, code, **fields):
        d = {"element_id": self.eid(), "debug_info": DEBUG, "type": "library_node", "implementation_type": "NONE", "code": code}
        d.update(fields)
        return d

    def edge(self, src, src_conn, dst, dst_conn, base_type):
        return {"element_id": self.eid(), "debug_info": DEBUG, "src": src["element_id"], "dst": dst["element_id"],
                "src_conn": src_conn, "dst_conn": dst_conn, "subset": [], "base_type": base_type}

    def finish(self):
        self.j["root"] = {"type": "sequence", "element_id": self.eid(), "debug_info": DEBUG, "children": self.blocks,
                          "transitions": [{"type": "transition", "element_id": self.eid(), "debug_info": DEBUG, "assignments": []}
                                          for _ in self.blocks]}
        self.j["element_counter"] = self.counter
        return self.j


DOUBLE, FLOAT, INT64 = 15, 14, 5


def gemm_softmax():
    """Y = softmax(A @ B, axis=1): GEMM (BLAS, RowMajor 101, NoTrans 111) into a transient, then Softmax."""
    b = Builder("gemm_softmax")
    for name in ("A", "B"):
        b.container(name, pointer(DOUBLE), argument=True)
    b.container("Y", pointer(DOUBLE), argument=True)
    for sym in ("_s0", "_s1", "_s2"):
        b.container(sym, scalar(INT64), argument=True)
    b.container("tmp", pointer(DOUBLE))
    a, bb, c_out = b.access("A"), b.access("B"), b.access("tmp")
    one, zero = b.constant("1.0", DOUBLE), b.constant("0.0", DOUBLE)
    g = b.library("GEMM", precision=ord("d"), layout=101, trans_a=111, trans_b=111, m="_s0", n="_s1", k="_s2",
                  lda="_s2", ldb="_s1", ldc="_s1")
    g["implementation_type"] = "BLAS"
    b.block([a, bb, c_out, one, zero, g],
            [b.edge(a, "void", g, "__A", pointer(DOUBLE)), b.edge(bb, "void", g, "__B", pointer(DOUBLE)),
             b.edge(one, "void", g, "__alpha", scalar(DOUBLE)), b.edge(zero, "void", g, "__beta", scalar(DOUBLE)),
             b.edge(g, "__C", c_out, "void", pointer(DOUBLE))])
    t_in, y = b.access("tmp"), b.access("Y")
    sm = b.library("ml::Softmax", shape=["_s0", "_s1"], axes=[1], keepdims=False)
    b.block([t_in, y, sm], [b.edge(t_in, "void", sm, "X", pointer(DOUBLE)), b.edge(sm, "Y", y, "void", pointer(DOUBLE))])
    return b.finish()


def conv_relu():
    """Y = relu(conv2d(X, W) + bias), fp32, [N, C, H, W] with symbolic batch."""
    b = Builder("conv_relu")
    for name in ("X", "W", "Bias", "Y"):
        b.container(name, pointer(FLOAT), argument=True)
    b.container("_s0", scalar(INT64), argument=True)
    b.container("t0", pointer(FLOAT))
    x, w, bias, t0 = b.access("X"), b.access("W"), b.access("Bias"), b.access("t0")
    conv = b.library("ml::Conv", shape=["_s0", "4", "9", "10"], kernel_shape=["3", "3"], strides=["1", "1"],
                     pads=["1", "1", "1", "1"], dilations=["1", "1"], output_channels="6", group="1")
    b.block([x, w, bias, t0, conv],
            [b.edge(x, "void", conv, "X", pointer(FLOAT)), b.edge(w, "void", conv, "W", pointer(FLOAT)),
             b.edge(bias, "void", conv, "B", pointer(FLOAT)), b.edge(conv, "Y", t0, "void", pointer(FLOAT))])
    t_in, y = b.access("t0"), b.access("Y")
    relu = b.library("ml::ReLU", shape=["_s0", "6", "9", "10"])
    b.block([t_in, y, relu], [b.edge(t_in, "void", relu, "X", pointer(FLOAT)), b.edge(relu, "Y", y, "void", pointer(FLOAT))])
    return b.finish()


def matmul_add_mean_cast():
    """Y = float64(mean(A @ B + C, axis=2)): batched MatMul with a broadcast right operand, Add, Mean, Cast."""
    b = Builder("matmul_add_mean_cast")
    for name in ("A", "B", "C"):
        b.container(name, pointer(FLOAT), argument=True)
    b.container("Y", pointer(DOUBLE), argument=True)
    b.container("_s0", scalar(INT64), argument=True)
    for name in ("t0", "t1", "t2"):
        b.container(name, pointer(FLOAT))
    a, bb, t0 = b.access("A"), b.access("B"), b.access("t0")
    mm = b.library("ml::MatMul", shape_a=["_s0", "8", "16"], shape_b=["16", "12"], strides_a=["128", "16", "1"], strides_b=["12", "1"],
                   offset_a="0", offset_b="0")
    b.block([a, bb, t0, mm], [b.edge(a, "void", mm, "A", pointer(FLOAT)), b.edge(bb, "void", mm, "B", pointer(FLOAT)),
                              b.edge(mm, "Y", t0, "void", pointer(FLOAT))])
    t0_in, c, t1 = b.access("t0"), b.access("C"), b.access("t1")
    add = b.library("ml::Add", shape=["_s0", "8", "12"])
    b.block([t0_in, c, t1, add], [b.edge(t0_in, "void", add, "A", pointer(FLOAT)), b.edge(c, "void", add, "B", pointer(FLOAT)),
                                  b.edge(add, "C", t1, "void", pointer(FLOAT))])
    t1_in, t2 = b.access("t1"), b.access("t2")
    mean = b.library("ml::Mean", shape=["_s0", "8", "12"], axes=[2], keepdims=False)
    b.block([t1_in, t2, mean], [b.edge(t1_in, "void", mean, "X", pointer(FLOAT)), b.edge(mean, "Y", t2, "void", pointer(FLOAT))])
    t2_in, y = b.access("t2"), b.access("Y")
    cast = b.library("ml::Cast", shape=["_s0", "8"], target_type=DOUBLE)
    b.block([t2_in, y, cast], [b.edge(t2_in, "void", cast, "X", pointer(FLOAT)), b.edge(cast, "Y", y, "void", pointer(DOUBLE))])
    return b.finish()


def with_tasklet():
    """A block with a scalar tasklet: outside what the reader executes."""
    b = Builder("scalar_code")
    b.container("a", scalar(DOUBLE), argument=True)
    b.container("b", scalar(DOUBLE), argument=True)
    a, out = b.access("a"), b.access("b")
    t = {"element_id": b.eid(), "debug_info": DEBUG, "type": "tasklet", "code": 0, "inputs": ["_in"], "output": "_out"}
    b.block([a, out, t], [b.edge(a, "void", t, "_in", scalar(DOUBLE)), b.edge(t, "_out", out, "void", scalar(DOUBLE))])
    return b.finish()


if __name__ == "__main__":
    for name, fn in (("sdfg_gemm_softmax", gemm_softmax), ("sdfg_conv_relu", conv_relu), ("sdfg_matmul_add_mean_cast", matmul_add_mean_cast),
                     ("sdfg_scalar_code", with_tasklet)):
        with open(os.path.join(HERE, name + ".json"), "w") as fh:
            json.dump(fn(), fh, indent=1, sort_keys=True)
            fh.write("\n")
        print("wrote", name + ".json")
