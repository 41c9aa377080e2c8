"""Pins the CPU oracle to the reference's own known-answer vectors
(tests/golden/reference_vectors.json, extracted by tests/golden/make_golden.py).
Runs without a GPU."""
import numpy as np


def test_cross_entropy_golden(golden, oracle):
    g = golden["cross_entropy"]
    logits = np.array(g["logits"], np.float32).reshape(g["shape"])
    p = oracle.softmax(logits)
    np.testing.assert_allclose(p, 0.25, rtol=1e-6)
    want = np.float32(-np.log(g["loss_is_minus_log_of"]))
    for t in (np.array(g["int_target"], np.int32),
              np.array(g["array_target"], np.int32).reshape(g["shape"])):
        loss = oracle.cross_entropy_fwd(p, t)
        np.testing.assert_allclose(loss, want, rtol=1e-6)
        grad = oracle.softmax_cross_entropy_bwd(p, t)
        np.testing.assert_allclose(grad.ravel(), np.array(g["grad"], np.float32), rtol=1e-6)


def test_batchnorm_cudnn_golden(golden, oracle):
    g = golden["batchnorm"]
    x = np.array(g["x"], np.float32).reshape(g["shape"])
    mean, invstd = oracle.bn_stats(x, eps=g["eps"])
    scale = np.array(g["scale"], np.float32)
    bias = np.array(g["bias"], np.float32)
    y = (x - mean.reshape(1, -1, 1, 1)) * invstd.reshape(1, -1, 1, 1) \
        * scale.reshape(1, -1, 1, 1) + bias.reshape(1, -1, 1, 1)
    np.testing.assert_allclose(y.ravel(), g["y"], atol=g["tol"])

    xb = np.array(g["bwd_x"], np.float32).reshape(g["shape"])
    dy = np.array(g["bwd_dy"], np.float32).reshape(g["shape"])
    mean, invstd = oracle.bn_stats(xb, eps=g["eps"])
    dx, ds, db = oracle.bn_backward(dy, xb, np.array(g["bwd_scale"], np.float32), mean, invstd)
    np.testing.assert_allclose(dx.ravel(), g["dx"], atol=g["tol"])
    np.testing.assert_allclose(ds, g["dscale"], atol=g["tol"])
    np.testing.assert_allclose(db, g["dbias"], atol=g["tol"])


def test_batchnorm_api_golden(golden, oracle):
    # dy == x, so dx is purely the epsilon term: a sharp test of the formula.
    g = golden["batchnorm_api"]
    x = np.array(g["x"], np.float32).reshape(g["shape"])
    mean, invstd = oracle.bn_stats(x, eps=g["eps"])
    dx, _, _ = oracle.bn_backward(x.copy(), x, np.array(g["scale"], np.float32), mean, invstd)
    np.testing.assert_array_almost_equal(dx, np.array(g["dx"], np.float32), decimal=g["decimal"])


def test_bn_saved_invstd_has_no_epsilon_in_api_model(oracle):
    # test/python/test_api.py:52-54 models resultSaveInvVariance as 1/sqrt(var).
    rng = np.random.default_rng(0)
    x = rng.random((10, 10, 20, 20), dtype=np.float32)
    mean, invstd = oracle.bn_stats(x, eps=0.0)
    np.testing.assert_allclose(mean, x.mean(axis=(0, 2, 3)), rtol=1e-5)
    np.testing.assert_allclose(invstd, 1 / np.sqrt(x.var(axis=(0, 2, 3))), rtol=1e-4)


def test_pooling_goldens(golden, oracle):
    g = golden["maxpool_cudnn"]
    x = np.array(g["x"], np.float32).reshape(g["x_shape"])
    y = oracle.maxpool_forward(x, g["kernel"], g["stride"], g["pad"])
    assert y.ravel().tolist() == g["y"]
    dy = np.array(g["dy"], np.float32).reshape(y.shape)
    dx = oracle.maxpool_backward(dy, x, g["kernel"], g["stride"], g["pad"])
    assert dx.ravel().tolist() == np.array(g["dx"], np.float32).tolist()

    g = golden["maxpool_api"]
    x = np.array(g["x"], np.float32).reshape(g["x_shape"])
    y = oracle.maxpool_forward(x, g["kernel"], g["stride"], g["pad"])
    np.testing.assert_array_equal(y, np.array(g["y"], np.float32))
    dy = np.array(g["dy"], np.float32).reshape(y.shape)
    dx = oracle.maxpool_backward(dy, x, g["kernel"], g["stride"], g["pad"])
    np.testing.assert_array_equal(dx, np.array(g["dx"], np.float32))

    g = golden["avgpool_api"]
    x = np.array(g["x"], np.float32).reshape(g["x_shape"])
    y = oracle.avgpool_forward(x, g["kernel"], g["stride"], g["pad"])
    np.testing.assert_allclose(y, np.array(g["y"], np.float32), rtol=1e-6)
    dy = np.array(g["dy"], np.float32).reshape(y.shape)
    dx = oracle.avgpool_backward(dy, x.shape, g["kernel"], g["stride"], g["pad"])
    np.testing.assert_allclose(dx, np.array(g["dx"], np.float32), rtol=1e-6)


def test_relu_golden(golden, oracle):
    g = golden["relu"]
    x = np.array(g["x"], np.float32).reshape(g["shape"])
    dy = np.ones(g["shape"], np.float32)
    np.testing.assert_array_equal(oracle.relu(x), np.maximum(x, 0))
    np.testing.assert_array_equal(oracle.relu_backward(dy, x), (x > 0).astype(np.float32) * dy)
    # CUDA conventions at the edges: x == 0 and x == -0 give exactly +0.
    e = np.array([0.0, -0.0, 1e-45, -1e-45], np.float32)
    assert oracle.relu_backward(np.ones(4, np.float32), e).tolist() == [0.0, 0.0, 1.0, 0.0]
    assert not np.signbit(oracle.relu(e)).any()
    # fp16 backward keeps the gradient at x == 0 (math_kernel.cu:261-271)
    h = oracle.relu_backward_f16(np.ones(3, np.float16), np.array([0.0, -1.0, 2.0], np.float16))
    assert h.tolist() == [1.0, 0.0, 1.0]


def test_sgd_goldens(golden, oracle):
    for case in golden["sgd"]["cases"]:
        shape = golden["sgd"]["shape"]
        w = np.full(shape, case["w"], np.float32)
        g0 = np.full(shape, case["g"], np.float32)
        buf = np.zeros(shape, np.float32) if case["momentum"] else None
        lr = case["lr"]
        if case["name"] == "const_lr":
            want = w - np.float32(lr) * g0
            oracle.sgd_update(w, g0.copy(), buf, lr)
            np.testing.assert_array_almost_equal(w, want, decimal=5)
        elif case["name"] == "weight_decay":
            want = w - np.float32(lr) * (g0 + np.float32(0.2) * w)
            oracle.sgd_update(w, g0.copy(), buf, lr, weight_decay=case["weight_decay"])
            np.testing.assert_array_almost_equal(w, want, decimal=5)
        else:
            w1 = w - np.float32(lr) * g0
            oracle.sgd_update(w, g0.copy(), buf, lr, momentum=0.9)
            np.testing.assert_array_almost_equal(w, w1, decimal=5)
            w2 = w1 - np.float32(lr) * (g0 + g0 * np.float32(0.9))
            oracle.sgd_update(w, g0.copy(), buf, lr, momentum=0.9)
            np.testing.assert_array_almost_equal(w, w2, decimal=5)


def test_sum_rows_columns(oracle):
    # test/singa/test_tensor_math.cc:775-803: SumRows sums over rows (one value
    # per column), SumColumns over columns.
    rng = np.random.default_rng(1)
    m = (rng.random((3, 2), dtype=np.float32) * 10)
    np.testing.assert_allclose(oracle.sum_rows(m), m.sum(axis=0), rtol=1e-6)
    np.testing.assert_allclose(oracle.sum_columns(m), m.sum(axis=1), rtol=1e-6)
    dy = rng.standard_normal((4, 3, 5, 5), dtype=np.float32)
    np.testing.assert_allclose(oracle.conv_bias_backward(dy), dy.sum(axis=(0, 2, 3)), rtol=1e-5, atol=1e-6)


def test_batchnorm_training_api_golden(golden, oracle):
    """test_api.py:31-54, 107-161: batch mean and saved inverse std (no epsilon)
    of the training-mode forward, which is what the backward consumes."""
    g = golden["batchnorm_training_api"]
    x = np.array(g["x"], np.float32).reshape(g["x_shape"])
    mean, invstd = oracle.bn_stats(x)
    x64 = x.astype(np.float64)
    np.testing.assert_array_almost_equal(mean, x64.mean(axis=(0, 2, 3)), decimal=6)
    np.testing.assert_array_almost_equal(invstd, 1.0 / np.sqrt(x64.var(axis=(0, 2, 3))), decimal=3)
    np.testing.assert_allclose(mean, [5.5, 11.0])
    np.testing.assert_allclose(invstd, [1.0 / 4.5, 1.0 / 9.0], rtol=1e-6)


def test_tensor_math_fixture_goldens(golden, oracle):
    """The reference's tensor-math fixture (test_tensor_math.cc): ReLU of the
    shifted fixture, SumRows / SumColumns, and the legacy Dense bias gradient
    (test_dense.cc: column sums of dy)."""
    g = golden["tensor_math"]
    a = np.array(g["dat1"], np.float32)
    r = oracle.relu(a - np.float32(g["relu_shift"]))
    np.testing.assert_array_equal(r[:3], np.array(g["relu_expect_first3"], np.float32))
    m = a.reshape(g["shape"])
    np.testing.assert_array_equal(oracle.sum_rows(m), np.array([9.0, 12.0], np.float32))      # 1+3+5, 2+4+6
    np.testing.assert_array_equal(oracle.sum_columns(m), np.array([3.0, 7.0, 11.0], np.float32))
    d = golden["dense_bias_grad"]
    dy = np.array(d["dy"], np.float32).reshape(d["shape"])
    np.testing.assert_array_equal(oracle.sum_rows(dy), np.array([6.0, 6.0, 6.0], np.float32))


def test_softmax_cudnn_layer_golden(golden, oracle):
    g = golden["softmax_cudnn"]
    for shape in g["shapes"]:
        x = np.array(g["x"], np.float32).reshape(shape)
        e = np.exp(x.astype(np.float64))
        np.testing.assert_allclose(oracle.softmax(x), e / e.sum(axis=1, keepdims=True), rtol=1e-6)


def test_softmax_axis_goldens(golden, oracle):
    """test_api.py:204-244: SoftMax(axis) equals a 2-D softmax of the reshaped
    input (rows = product of the leading axes)."""
    rng = np.random.default_rng(0)
    for shape, axis, two_d in golden["softmax_axis"]["cases"]:
        x = (rng.random(shape) + 1000).astype(np.float32)
        x2 = x.reshape(two_d)
        e = np.exp(x2 - x2.max())
        want = (e / e.sum(axis=1, keepdims=True)).reshape(shape)
        ax = axis % len(shape)
        rows = int(np.prod(shape[:ax])) if ax else 1
        assert [rows, x.size // rows] == two_d
        got = oracle.softmax(x.reshape(rows, -1)).reshape(shape)
        np.testing.assert_array_almost_equal(got, want)


def test_dist_constant_golden(golden):
    # test/python/test_dist.py: grad=1, param=10 -> 10 - 0.1 in all six modes.
    from oracle import comm
    g = golden["dist"]
    for world in (1, 2, 4):
        grads = [np.full(g["shape"], g["grad"], np.float32).ravel() for _ in range(world)]
        outs = {
            "all_reduce": comm.allreduce_sum(grads),
            "all_reduce_half": comm.allreduce_half(grads),
            "threshold": comm.sparse_threshold_step(grads, None, 0.05)[0],
            "topk": comm.sparse_topk_step(grads, None, 1.0)[0],
            "threshold_corr": comm.sparse_threshold_step(grads, [np.zeros_like(x) for x in grads], 0.05)[0],
            "topk_corr": comm.sparse_topk_step(grads, [np.zeros_like(x) for x in grads], 1.0)[0],
        }
        for name, red in outs.items():
            upd = comm.divide_by_world(red, world)
            param = np.full_like(upd, g["param"]) - np.float32(g["lr"]) * upd
            np.testing.assert_array_almost_equal(param, g["expect_param"], decimal=5, err_msg=name)
