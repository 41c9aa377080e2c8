"""Extract the reference's own known-answer vectors for the backward path.

Run once in a container that has the apache/singa sources:

    python tests/golden/make_golden.py /path/to/singa > /dev/null

It READS the reference's test files as text (nothing is executed or imported)
and writes ``tests/golden/reference_vectors.json`` next to this script.  Each
entry records the file and line range it was taken from.  The tests replay the
vectors against the CPU oracle (no GPU) and against the CUDA path (GPU).
"""
import ast
import json
import os
import re
import sys

NUM = r"[-+]?(?:\d+\.\d*|\.\d+|\d+)(?:[eE][-+]?\d+)?"


def lines(root, rel, lo, hi):
    with open(os.path.join(root, rel)) as f:
        return "".join(f.readlines()[lo - 1:hi])


def c_array(text, name):
    """Values of ``const <type> name[...] = {...};`` inside text."""
    m = re.search(r"\b%s\s*\[[^\]]*\]\s*=\s*\{([^}]*)\}" % re.escape(name), text)
    if not m:
        raise KeyError(name)
    return [float(v) for v in re.findall(NUM, m.group(1).replace("f,", ",").replace("f}", "}"))]


def expects(text, ptr):
    """(index -> value) from EXPECT_NEAR/EXPECT_EQ/EXPECT_FLOAT_EQ lines that
    compare a literal with ptr[i], in either argument order."""
    out = {}
    pat1 = re.compile(r"EXPECT_(?:NEAR|EQ|FLOAT_EQ)\(\s*(%s)f?\s*,\s*%s\[(\d+)\]" % (NUM, re.escape(ptr)))
    pat2 = re.compile(r"EXPECT_(?:NEAR|EQ|FLOAT_EQ)\(\s*%s\[(\d+)\]\s*,\s*(%s)f?" % (re.escape(ptr), NUM))
    for v, i in pat1.findall(text):
        out[int(i)] = float(v)
    for i, v in pat2.findall(text):
        out[int(i)] = float(v)
    return [out[i] for i in range(len(out))]


def py_func_literals(root, rel, func):
    """All list/number literals assigned inside a python function, by name."""
    with open(os.path.join(root, rel)) as f:
        tree = ast.parse(f.read())
    found = {}

    def numeric(node):
        try:
            return ast.literal_eval(node)
        except Exception:
            return None

    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == func:
            for sub in ast.walk(node):
                if isinstance(sub, ast.Assign) and isinstance(sub.targets[0], ast.Name):
                    name = sub.targets[0].id
                    val = sub.value
                    lit = numeric(val)
                    if lit is None:
                        # np.array(<literal>, ...).reshape(...) -> the literal
                        cands = [n for n in ast.walk(val)
                                 if isinstance(n, (ast.List, ast.Tuple))
                                 and numeric(n) is not None]
                        if cands:   # first in source order = np.array's argument
                            cands.sort(key=lambda n: (n.lineno, n.col_offset))
                            lit = numeric(cands[0])
                    if lit is not None:
                        found.setdefault(name, lit)
            found["_lines"] = [node.lineno, node.end_lineno]
    return found


def main(root):
    g = {}

    # --- softmax cross entropy (logits 0.1 everywhere -> p = 0.25) ----------
    rel = "test/singa/test_cross_entropy.cc"
    t = lines(root, rel, 28, 112)
    bwd = lines(root, rel, 76, 94)
    g["cross_entropy"] = {
        "source": rel + ":36-38,54-56,83-90",
        "logits": c_array(t, "pdat"), "shape": [2, 4],
        "int_target": [int(v) for v in c_array(t, "tdat")],
        "array_target": [int(v) for v in c_array(t, "tary")],
        "loss_is_minus_log_of": 0.25,
        "grad": expects(bwd, "gdat"),
    }

    # --- cuDNN batch-norm forward + backward, shape (1,2,4,4) ----------------
    rel = "test/singa/test_cudnn_batchnorm.cc"
    f = lines(root, rel, 44, 115)
    b = lines(root, rel, 117, 229)
    g["batchnorm"] = {
        "source": rel + ":44-115 (forward), :117-229 (backward)",
        "note": "expected values were produced with cuDNN-7 semantics: "
                "epsilon = CUDNN_BN_MIN_EPSILON = 1e-5; tolerance 1e-4",
        "shape": [1, 2, 4, 4], "eps": 1e-5, "tol": 1e-4,
        "x": c_array(f, "x"), "scale": c_array(f, "alpha_"), "bias": c_array(f, "beta_"),
        "y": expects(f, "outptr"),
        "bwd_x": c_array(b, "x"), "bwd_dy": c_array(b, "dy"),
        "bwd_scale": c_array(b, "alpha_"),
        "dx": expects(b, "dxptr"), "dscale": expects(b, "dbnScaleptr"),
        "dbias": expects(b, "dbnBiasptr"),
    }

    # --- cuDNN max pooling 2x2 stride 1 on 3x3 -------------------------------
    rel = "test/singa/test_cudnn_pooling.cc"
    f = lines(root, rel, 55, 85)
    b = lines(root, rel, 87, 130)
    g["maxpool_cudnn"] = {
        "source": rel + ":55-85 (forward), :87-130 (backward)",
        "x_shape": [1, 1, 3, 3], "kernel": [2, 2], "stride": [1, 1], "pad": [0, 0],
        "x": c_array(f, "x"), "y": expects(f, "outptr1"),
        "dy": c_array(b, "dy"), "dx": expects(b, "dx"),
    }

    # --- python API goldens: BN backward (eps 1e-5), max / avg pooling -------
    rel = "test/python/test_api.py"
    lit = py_func_literals(root, rel, "test_batchnorm_backward_dnnl")
    g["batchnorm_api"] = {
        "source": rel + ":%d-%d" % tuple(lit["_lines"]),
        "shape": [lit["N"], lit["C"], lit["H"], lit["W"]], "eps": 1e-5,
        "x": lit["data"], "dy": lit["data"], "scale": [1] * lit["C"],
        "dx": lit["dx_truth"], "decimal": 6,
    }
    lit = py_func_literals(root, rel, "test_batchnorm_training_gpu")
    g["batchnorm_training_api"] = {
        "source": rel + ":31-54 (numpy model), %d-%d" % tuple(lit["_lines"]),
        "x": lit["x_0"], "x_shape": [2, 2, 2, 2], "scale": lit["s_0"], "bias": lit["b_0"],
        "running_mean": lit["rm_0"], "running_var": lit["rv_0"], "momenta": [0.0, 1.0, 0.2],
        "random_case": {"shape": [10, 10, 20, 20], "momentum": 0.2},
        "decimals": {"y": 4, "batch_mean": 6, "running_mean": 6, "saved_inv_std": 3, "running_var": 4},
    }
    lit = py_func_literals(root, rel, "test_dnnl_pooling_max")
    g["maxpool_api"] = {
        "source": rel + ":%d-%d" % tuple(lit["_lines"]),
        "x_shape": [lit["N"], lit["C"], lit["H"], lit["W"]], "kernel": [2, 2],
        "stride": [1, 1], "pad": [0, 0], "x": lit["data"], "dy": lit["dy0"],
        "y": lit["y1"], "dx": lit["dx1"],
    }
    lit = py_func_literals(root, rel, "test_dnnl_pooling_avg")
    g["avgpool_api"] = {
        "source": rel + ":%d-%d" % tuple(lit["_lines"]),
        "x_shape": [lit["N"], lit["C"], lit["H"], lit["W"]], "kernel": [2, 2],
        "stride": [1, 1], "pad": [0, 0], "x": lit["data"], "dy": lit["dy0"],
        "y": lit["y1"], "dx": lit["dx1"],
    }

    # --- ReLU forward/backward (python operation test) -----------------------
    rel = "test/python/test_operation.py"
    lit = py_func_literals(root, rel, "_Relu_helper")
    g["relu"] = {
        "source": rel + ":%d-%d" % tuple(lit["_lines"]),
        "x": lit["X"], "shape": [3, 2], "dy": "ones",
        "rule": "y = max(x,0); dx = (x > 0) * dy",
    }

    # --- SGD one-step values (closed forms stated in the test) ---------------
    g["sgd"] = {
        "source": "test/python/test_opt.py:96-107,180-213",
        "cases": [
            {"name": "const_lr", "w": 0.1, "g": 0.1, "lr": 0.1, "momentum": 0.0,
             "weight_decay": 0.0, "steps": 1, "expect": "w - 0.1*g"},
            {"name": "momentum", "w": 0.1, "g": 0.01, "lr": 0.1, "momentum": 0.9,
             "weight_decay": 0.0, "steps": 2,
             "expect": "step1: w-0.1*g ; step2: w1-0.1*(g+0.9*g)"},
            {"name": "weight_decay", "w": 0.1, "g": 0.01, "lr": 0.1, "momentum": 0.0,
             "weight_decay": 0.2, "steps": 1, "expect": "w - 0.1*(g+0.2*w)"},
        ],
        "shape": [2, 3],
    }

    # --- distributed tests: constant inputs, all six modes -------------------
    g["dist"] = {
        "source": "test/python/test_dist.py:37-121",
        "grad": 1.0, "param": 10.0, "lr": 0.1, "expect_param": 9.9,
        "modes": ["all_reduce", "fused_all_reduce", "all_reduce_half",
                  "fused_all_reduce_half", "sparsification_threshold_0.05",
                  "sparsification_topK_1.0"],
        "shape": [10, 10],
    }

    # --- tensor math fixtures and small known answers (CUDA variants of the tests)
    tm = "test/singa/test_tensor_math.cc"
    fixture = lines(root, tm, 40, 43)
    g["tensor_math"] = {
        "source": tm + ":41-42 (fixture), :87-100 (ReLU), :856-864 (L2), :952-967 (MultColumn), "
                       ":1016-1047 (MultRow, DivRow), :1049-1082 (SumRows, SumColumns), :1084-1097 (strided Exp), "
                       ":1161-1173 (RowMax), :1254-1283 (SoftPlus, SoftSign)",
        "dat1": c_array(fixture, "dat1"), "dat2": c_array(fixture, "dat2"), "shape": [3, 2],
        "relu_shift": 2.0, "relu_expect_first3": expects(lines(root, tm, 87, 100), "dptr1"),
        "mult_column_x": c_array(lines(root, tm, 952, 967), "x"),
        "mult_row_x": c_array(lines(root, tm, 1016, 1031), "x"),
        "div_row_x": c_array(lines(root, tm, 1033, 1047), "x"),
        "row_max_in": c_array(lines(root, tm, 1161, 1173), "data1"),
        "row_max_expect": expects(lines(root, tm, 1161, 1173), "dptr1"),
        "soft_in": c_array(lines(root, tm, 1254, 1267), "data"),
        "softsign_expect": expects(lines(root, tm, 1269, 1283), "dptr"),
        # strided Exp: a (3,2) reshaped to (1,3,2) written through the (1,2,0) transpose of a (2,1,3)
        # tensor; the test checks y[0], y[2], y[4] = exp(dat1[0]), exp(dat1[4]), exp(dat1[3])
        "exp_stride_checks": [[0, 0], [2, 4], [4, 3]],
    }

    # --- cuDNN softmax layer tests: row softmax of a literal input, 1-D and 2-D
    sm = "test/singa/test_cudnn_softmax.cc"
    g["softmax_cudnn"] = {
        "source": sm + ":44-68 (1-D), :104-132 (2-D); expectation = exp(x) / sum(exp(x)) per row",
        "x": c_array(lines(root, sm, 44, 68), "x"), "shapes": [[1, 6], [2, 3]],
    }

    # --- AsType float <-> int on CUDA
    tc = "test/singa/test_tensor.cc"
    g["astype"] = {
        "source": tc + ":73-110; test/python/test_tensor.py:405-425 (uniform(-5, 5) floats truncate toward zero)",
        "float_in": c_array(lines(root, tc, 73, 90), "data"),
        "int_expect": expects(lines(root, tc, 73, 90), "dptr2"),
        "int_in": [int(v) for v in c_array(lines(root, tc, 92, 110), "data")],
        "float_expect": expects(lines(root, tc, 92, 110), "dptr2"),
    }

    # --- legacy Dense backward on CUDA: bias gradient = column sums of dy
    dn = "test/singa/test_dense.cc"
    g["dense_bias_grad"] = {
        "source": dn + ":176-242",
        "dy": c_array(lines(root, dn, 176, 242), "dy"), "shape": [3, 3],
    }

    # --- SoftMax(axis): shapes and the 2-D view each axis maps to
    cases = re.findall(r"_run_test\(dev, (\[[^\]]*\]), (-?\d+), (\[[^\]]*\])\)", lines(root, "test/python/test_api.py", 204, 244))
    g["softmax_axis"] = {
        "source": "test/python/test_api.py:204-244 (inputs uniform[0,1) + 1000, compared with a 2-D numpy softmax)",
        "cases": [[json.loads(a), int(b), json.loads(c)] for a, b, c in cases],
    }

    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.json")
    with open(out, "w") as f:
        json.dump(g, f, indent=1)
    print("wrote", out)


def launcher_symbols():
    """Mangled names of the `singa::cuda::*` launchers (those taking a stream)
    exported by the reference's math_kernel.cu once compiled here
    (oracle/ref_build.py -> oracle/_ref/libref_cuda.so), one per line: the
    symbol contract of the drop-in launcher library."""
    import subprocess
    here = os.path.dirname(os.path.abspath(__file__))
    lib = os.path.join(os.path.dirname(os.path.dirname(here)), "oracle", "_ref", "libref_cuda.so")
    if not os.path.exists(lib):
        print("skipped launcher symbols:", lib, "not built")
        return
    rows = subprocess.run(["nm", "-D", "--defined-only", lib], capture_output=True, text=True, check=True).stdout
    names = sorted(r.split()[2] for r in rows.splitlines()
                   if "_ZN5singa4cuda" in r and "P11CUstream_st" in r and r.split()[1] == "T")
    out = os.path.join(here, "singa_cuda_launcher_symbols.txt")
    with open(out, "w") as f:
        f.write("\n".join(names) + "\n")
    print("wrote", out, len(names))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
    launcher_symbols()
