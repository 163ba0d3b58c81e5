"""Extracts the reference's own known-answer tests for the conv2d/linear hot path into
``reference_known_answers.json``.

Run in a container where the reference checkout is present:
    python tests/golden/make_golden.py /path/to/ferrox
The numbers are read from the reference's Rust unit tests as text (nothing is retyped):
  src/ops/mod.rs            relu/sigmoid/tanh/add/mul/matmul/transpose/sum/mean/softmax/conv2d tests
  src/backend/tensor.rs     test_matmul_operation, activations, sum/mean
  src/nn/optim/sgd.rs       test_sgd_basic_step
The JSON is committed so the tests run where the reference checkout is absent.
"""
import json
import os
import re
import sys

NUM = r"-?\d+(?:\.\d*)?(?:[eE][-+]?\d+)?(?:f32|f64)?"
ARR = re.compile(r"(?:vec!|&)?\[\s*((?:" + NUM + r"\s*,?\s*)+)\]")


def body(text, fn_name):
    m = re.search(r"fn\s+" + re.escape(fn_name) + r"\s*\(\)\s*\{", text)
    if not m:
        raise KeyError(fn_name)
    start = m.end()
    nxt = text.find("#[test]", start)
    return text[start: nxt if nxt >= 0 else len(text)]


def arrays(src):
    out = []
    src = re.sub(r"//[^\n]*", "", src)
    for m in ARR.finditer(src):
        inner = m.group(1)
        vals = [float(re.sub(r"f32|f64", "", t)) for t in re.findall(NUM, inner)]
        out.append(vals)
    return out


def main(ref):
    ops = open(os.path.join(ref, "src/ops/mod.rs")).read()
    ten = open(os.path.join(ref, "src/backend/tensor.rs")).read()
    sgd = open(os.path.join(ref, "src/nn/optim/sgd.rs")).read()
    G = {}

    def unary(name, fn, op):
        a = arrays(body(ops, fn))
        G[name] = {"source": f"src/ops/mod.rs::{fn}", "op": op, "input": a[0], "shape": a[1],
                   "expected": a[2]}

    unary("relu_activation", "relu_activation", "relu")
    unary("sigmoid_activation", "sigmoid_activation", "sigmoid")
    unary("tanh_activation", "tanh_activation", "tanh")
    G["relu_activation"]["tol"] = 1e-6
    G["sigmoid_activation"]["tol"] = 1e-4
    G["tanh_activation"]["tol"] = 1e-4

    a = arrays(body(ops, "matrix_multiply"))
    G["matrix_multiply"] = {"source": "src/ops/mod.rs::matrix_multiply", "a": a[0], "b": a[1],
                            "shape": a[2], "expected": a[3], "tol": 1e-6}
    a = arrays(body(ops, "matrix_transpose"))
    G["matrix_transpose"] = {"source": "src/ops/mod.rs::matrix_transpose", "input": a[0], "rows": 2, "cols": 3,
                             "shape": a[1], "expected": a[2], "tol": 1e-6}
    a = arrays(body(ops, "sum_all_elements"))
    G["sum_all_elements"] = {"source": "src/ops/mod.rs::sum_all_elements", "input": a[0], "rows": 2, "cols": 2,
                             "expected": a[-1], "tol": 1e-6}
    a = arrays(body(ops, "sum_along_axes"))
    G["sum_along_axes"] = {"source": "src/ops/mod.rs::sum_along_axes", "input": a[0], "rows": 2, "cols": 2,
                           "axes": [int(v) for v in a[1]], "expected": a[3], "tol": 1e-6}
    a = arrays(body(ops, "mean_all_elements"))
    G["mean_all_elements"] = {"source": "src/ops/mod.rs::mean_all_elements", "input": a[0], "rows": 2, "cols": 2,
                              "expected": a[-1], "tol": 1e-6}
    a = arrays(body(ops, "mean_along_axes"))
    G["mean_along_axes"] = {"source": "src/ops/mod.rs::mean_along_axes", "input": a[0], "rows": 2, "cols": 2,
                            "axes": [int(v) for v in a[1]], "expected": a[3], "tol": 1e-6}
    a = arrays(body(ops, "softmax_last_axis"))
    G["softmax_last_axis"] = {"source": "src/ops/mod.rs::softmax_last_axis", "input": a[0], "rows": 2, "cols": 3,
                              "axis": 1, "expected": a[2], "tol": 1e-3}
    a = arrays(body(ops, "softmax_first_axis"))
    G["softmax_first_axis"] = {"source": "src/ops/mod.rs::softmax_first_axis", "input": a[0], "rows": 2, "cols": 2,
                               "axis": 0, "expected": a[2], "tol": 1e-3}

    a = arrays(body(ops, "conv2d_simple_forward"))
    G["conv2d_simple_forward"] = {"source": "src/ops/mod.rs::conv2d_simple_forward", "x": a[0], "x_shape": [1, 1, 2, 2],
                                  "w": a[1], "w_shape": [1, 1, 2, 2], "stride": [1, 1], "pad": [0, 0],
                                  "y_shape": [int(v) for v in a[2]], "expected": a[3], "tol": 1e-5}
    a = arrays(body(ops, "conv2d_test"))
    G["conv2d_test"] = {"source": "src/ops/mod.rs::conv2d_test", "x": a[0], "x_shape": [1, 3, 5, 5],
                        "w": a[1], "w_shape": [4, 3, 3, 3], "stride": [1, 1], "pad": [1, 1],
                        "y_shape": [int(v) for v in a[3]], "expected": a[2], "tol": 1e-3}
    a = arrays(body(ops, "conv2d_edge_cases"))
    G["conv2d_edge_cases"] = {"source": "src/ops/mod.rs::conv2d_edge_cases", "x": a[0], "x_shape": [1, 1, 2, 2],
                              "w": a[1], "w_shape": [1, 1, 1, 1], "stride": [1, 1], "pad": [0, 0],
                              "y_shape": [int(v) for v in a[3]], "expected": a[2], "tol": 1e-6}
    # shape-only conv tests of the reference: (x_shape, w_shape, stride, pad, y_shape)
    G["conv2d_shape_only"] = {
        "source": "src/ops/mod.rs::conv2d_{different_strides,with_padding,same_padding,multiple_channels,batch_processing,larger_kernel}",
        "cases": [
            [[1, 1, 4, 4], [1, 1, 2, 2], [2, 2], [0, 0], [1, 1, 2, 2]],
            [[1, 1, 3, 3], [1, 1, 2, 2], [1, 1], [1, 1], [1, 1, 4, 4]],
            [[1, 1, 5, 5], [1, 1, 3, 3], [1, 1], [1, 1], [1, 1, 5, 5]],
            [[1, 3, 2, 2], [2, 3, 2, 2], [1, 1], [0, 0], [1, 2, 1, 1]],
            [[2, 1, 2, 2], [1, 1, 2, 2], [1, 1], [0, 0], [2, 1, 1, 1]],
            [[1, 1, 6, 6], [1, 1, 5, 5], [1, 1], [0, 0], [1, 1, 2, 2]],
        ]}
    for i, fn in enumerate(["conv2d_different_strides", "conv2d_with_padding", "conv2d_same_padding",
                            "conv2d_multiple_channels", "conv2d_batch_processing", "conv2d_larger_kernel"]):
        b = body(ops, fn)
        ys = [v for v in arrays(b) if len(v) == 4 and all(float(t).is_integer() for t in v)]
        assert [int(t) for t in ys[-1]] == G["conv2d_shape_only"]["cases"][i][4], (fn, ys)

    a = arrays(body(ten, "test_matmul_operation"))
    G["test_matmul_operation"] = {"source": "src/backend/tensor.rs::test_matmul_operation", "a": a[0], "b": a[2],
                                  "shape": [2, 2], "expected": [4.0, 6.0, 10.0, 12.0], "tol": 0.0}
    assert a[1] == [2.0, 2.0] and a[0] == [1.0, 2.0, 3.0, 4.0]
    G["test_sigmoid_activation"] = {"source": "src/backend/tensor.rs::test_sigmoid_activation",
                                    "input": arrays(body(ten, "test_sigmoid_activation"))[0],
                                    "checks": "y[0]==0.5 within 1e-6; y[1]>0.99; y[2]<0.01"}
    G["test_tanh_activation"] = {"source": "src/backend/tensor.rs::test_tanh_activation",
                                 "input": arrays(body(ten, "test_tanh_activation"))[0],
                                 "checks": "|y[0]|<1e-6; y[1]>0.99; y[2]<-0.99"}
    G["test_relu_activation"] = {"source": "src/backend/tensor.rs::test_relu_activation",
                                 "input": arrays(body(ten, "test_relu_activation"))[0],
                                 "expected": [0.0, 0.0, 3.0], "tol": 0.0}
    G["test_sum_reduction"] = {"source": "src/backend/tensor.rs::test_sum_reduction",
                               "input": arrays(body(ten, "test_sum_reduction"))[0], "expected": [10.0], "tol": 0.0}
    G["test_mean_reduction"] = {"source": "src/backend/tensor.rs::test_mean_reduction",
                                "input": arrays(body(ten, "test_mean_reduction"))[0], "expected": [5.0], "tol": 0.0}
    a = arrays(body(sgd, "test_sgd_basic_step"))
    G["test_sgd_basic_step"] = {"source": "src/nn/optim/sgd.rs::test_sgd_basic_step", "param": a[0], "grad": a[2],
                                "lr": 0.1, "expected": [1.9], "tol": 1e-6}
    a = arrays(body(ops, "test_global_avgpool2d_forward"))
    G["test_global_avgpool2d_forward"] = {"source": "src/ops/mod.rs::test_global_avgpool2d_forward", "input": a[0],
                                          "x_shape": [1, 1, 4, 4], "y_shape": [int(v) for v in a[2]], "expected": a[1], "tol": 1e-4}
    cops = open(os.path.join(ref, "src/backend/cuda/ops.rs")).read()
    b = body(cops, "test_bias_broadcasting")
    bias = [float(re.sub(r"f32|f64", "", str(re.findall(r"let bias_data = vec!\[(" + NUM + r")\]", b)[0])))]
    target = [int(v) for v in re.findall(r"broadcast_to\(&mut bias_tensor, &\[(\d+)\]\)", b)]
    rep = re.search(r"vec!\[(" + NUM + r");\s*(\d+)\]", b)
    G["test_bias_broadcasting"] = {"source": "src/backend/cuda/ops.rs::test_bias_broadcasting", "input": bias, "in_shape": [1],
                                   "target_shape": target,
                                   "expected": [float(re.sub(r"f32|f64", "", rep.group(1)))] * int(rep.group(2)), "tol": 1e-6}
    b = body(ten, "test_transpose_operation")
    G["test_transpose_operation"] = {"source": "src/backend/tensor.rs::test_transpose_operation", "input": arrays(b)[0],
                                     "shape": [2, 3], "expected_shape": [3, 2]}
    b = body(ten, "test_broadcast_to")
    G["test_broadcast_to"] = {"source": "src/backend/tensor.rs::test_broadcast_to", "input": arrays(b)[0], "in_shape": [2],
                              "target_shape": [3, 2]}
    # element-wise add / mul (gradient accumulation and the mask products of the backward rules)
    for name, op in (("add_operation", "add"), ("mul_operation", "mul")):
        a = arrays(body(ops, name))
        G[name] = {"source": f"src/ops/mod.rs::{name}", "op": op, "a": a[0], "b": a[1], "shape": a[2], "expected": a[3],
                   "tol": 1e-6}
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_known_answers.json")
    with open(out, "w") as f:
        json.dump(G, f, indent=1)
    print("wrote", out, "with", len(G), "entries")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of the reference repository>")
    main(sys.argv[1])
