"""Runs a fixed battery of operations on singa::Tensor objects through one CUDA
build of apache/singa's core (variant "reference" = its own CUDA back end,
"sgb" = this repository's replacement back end) and saves every result.
Launched twice by tests/test_singa_types_gpu.py, once per variant; the two
result files must agree.  usage: singa_core_worker.py <variant> <out.npz>"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle.ref_cuda import Core      # noqa: E402


def main(variant, out_path):
    core = Core(variant)
    L = core.L
    rng = np.random.default_rng(42)
    R = {}
    f32 = lambda *s: rng.standard_normal(s).astype(np.float32)

    # ---- elementwise
    a, b = f32(257, 129), f32(257, 129)
    b[::5] = 0.0
    ta, tb = core.tensor(a), core.tensor(b)
    R["relu"] = core.numpy(core.call("rs_relu", ta))
    R["relu_backward"] = core.numpy(core.call("rs_relu_backward", ta, tb))
    for name in ("add", "sub", "eltwise_mult"):
        R[name] = core.numpy(core.call("rs_" + name, ta, tb))
    pos = np.abs(f32(257, 129)) + np.float32(0.5)
    tp = core.tensor(pos)
    R["div"] = core.numpy(core.call("rs_div", ta, tp))
    # transposed views: (129, 257)^T + dense, dense + transposed, both transposed
    c = f32(129, 257)
    tcT = core.call("rs_transpose", core.tensor(c))
    R["add_transposed_left"] = core.numpy(core.call("rs_add", tcT, ta))
    R["add_transposed_right"] = core.numpy(core.call("rs_add", ta, tcT))
    R["mul_both_transposed"] = core.numpy(core.call("rs_eltwise_mult", tcT, tcT))
    for op in range(10):
        src = tp if op in (1, 2) else ta                      # log / sqrt need positive input
        R["unary_%d" % op] = core.numpy(core.call("rs_unary", op, src))
    R["exp_of_transposed"] = core.numpy(core.call("rs_unary", 0, tcT))
    for op in range(5):
        R["compare_%d" % op] = core.numpy(core.call("rs_compare_scalar", op, tb, C.c_float(0.0)))
    t2 = core.tensor(a)
    L.rs_mult_scalar_inplace(t2, C.c_float(0.37))
    L.rs_div_scalar_inplace(t2, C.c_float(3.0))
    L.rs_add_inplace(t2, tb)
    R["scalar_chain"] = core.numpy(t2)

    # ---- reductions
    m = f32(256, 4096)
    tm = core.tensor(m)
    R["sum_axis0"] = core.numpy(core.call("rs_sum_axis", tm, 0))
    R["sum_axis1"] = core.numpy(core.call("rs_sum_axis", tm, 1))
    R["sum_all"] = core.numpy(core.call("rs_sum_all", core.tensor(f32(4096))))
    R["row_max"] = core.numpy(core.call("rs_row_max", tm))
    R["l1_l2"] = np.array([L.rs_l1(tm), L.rs_l2(tm)], np.float32)
    v_col, v_row = core.tensor(f32(256)), core.tensor(f32(4096))
    t3 = core.tensor(m)
    L.rs_mult_column(v_col, t3)
    L.rs_mult_row(v_row, t3)
    L.rs_add_row(v_row, t3)
    R["row_column_ops"] = core.numpy(t3)

    # ---- loss head
    logits = (f32(32, 1000) * np.float32(3)).astype(np.float32)
    labels = rng.integers(0, 1000, 32).astype(np.int32)
    tl, tt = core.tensor(logits), core.tensor(labels)
    p = core.call("rs_softmax", tl)
    R["softmax"] = core.numpy(p)
    # the two loss functions get one and the same probability matrix in both
    # variants (the soft-max above agrees only to rounding), so they compare exactly
    e = np.exp(logits - logits.max(axis=1, keepdims=True))
    pf = core.tensor((e / e.sum(axis=1, keepdims=True)).astype(np.float32))
    R["cross_entropy"] = core.numpy(core.call("rs_cross_entropy_fwd", pf, tt))
    R["softmax_ce_bwd"] = core.numpy(core.call("rs_softmax_cross_entropy_bwd", pf, tt))
    half = core.call("rs_tensor_as_type", tl, 1)
    R["f32_f16_f32"] = core.numpy(core.call("rs_tensor_as_type", half, 0))
    R["f32_i32_f32"] = core.numpy(core.call("rs_tensor_as_type", core.call("rs_tensor_as_type", tl, 2), 0))

    # ---- optimizer chain and contractions
    prm, grd, mom = core.tensor(f32(5000)), core.tensor(f32(5000) * np.float32(1e-2)), core.tensor(np.zeros(5000, np.float32))
    for _ in range(2):
        L.rs_sgd(prm, grd, mom, C.c_float(0.05), C.c_float(0.9), C.c_float(1e-5))
    R["sgd_param"], R["sgd_moment"] = core.numpy(prm), core.numpy(mom)
    A, B = core.tensor(f32(64, 128)), core.tensor(f32(128, 32))
    R["mult"] = core.numpy(core.call("rs_mult", A, B))
    R["mult_transposed"] = core.numpy(core.call("rs_mult", core.call("rs_transpose", A), core.tensor(f32(64, 16))))

    # ---- batch normalisation (spatial and per-activation) and pooling
    for tag, shape in (("bn4d", (8, 16, 14, 14)), ("bn4d_odd", (4, 8, 7, 7)), ("bn2d", (32, 64))):
        x = f32(*shape) * np.float32(1.5) + np.float32(0.2)
        ch = shape[1]
        tx = core.tensor(x)
        h = C.c_void_p(L.rs_bn_handle_new(C.c_float(0.9), tx))
        scale, bias = core.tensor(f32(ch) * np.float32(0.1) + np.float32(1)), core.tensor(f32(ch))
        rm, rv = core.tensor(np.zeros(ch, np.float32)), core.tensor(np.ones(ch, np.float32))
        y, mean, invstd = core.three("rs_bn_forward_training", h, tx, scale, bias, rm, rv)
        R[tag + "_y"], R[tag + "_mean"], R[tag + "_invstd"] = core.numpy(y), core.numpy(mean), core.numpy(invstd)
        dy = core.tensor(f32(*shape) * np.float32(1e-2))
        dx, ds, db = core.three("rs_bn_backward", h, dy, tx, scale, mean, invstd)
        R[tag + "_dx"], R[tag + "_dscale"], R[tag + "_dbias"] = core.numpy(dx), core.numpy(ds), core.numpy(db)
    for tag, shape, k, s, pd, is_max in (("maxpool", (4, 8, 28, 28), 3, 2, 1, 1), ("maxpool2", (4, 8, 24, 24), 2, 2, 0, 1),
                                         ("avgpool", (4, 16, 7, 7), 7, 1, 0, 0)):
        x = f32(*shape)
        tx = core.tensor(x)
        h = C.c_void_p(L.rs_pool_handle_new(tx, k, k, s, s, pd, pd, is_max))
        y = core.call("rs_pool_forward", h, tx)
        R[tag + "_y"] = core.numpy(y)
        dy = core.tensor(rng.standard_normal(R[tag + "_y"].shape).astype(np.float32))
        R[tag + "_dx"] = core.numpy(core.call("rs_pool_backward", h, dy, tx, y))
    dyc = f32(6, 32, 24, 24)              # drawn in both variants: the random stream must stay aligned
    if variant == "sgb":
        R["conv_bias_backward"] = core.numpy(core.call("rs_conv_bias_backward", core.tensor(dyc),
                                                       core.tensor(np.zeros(32, np.float32))))
        R["conv_bias_backward_want"] = dyc.astype(np.float64).sum((0, 2, 3)).astype(np.float32)

    # ---- communicator, one rank: sums of a single contribution
    idb = C.create_string_buffer(L.rs_nccl_id_bytes())
    L.rs_nccl_id_new(idb)
    comm = C.c_void_p(L.rs_comm_new(0, 1, idb, 4194304))
    g1, g2 = f32(100000), f32(33333)
    t1, t2c = core.tensor(g1), core.tensor(g2)
    L.rs_comm_synch(comm, t1)
    L.rs_comm_wait(comm)
    R["comm_synch"] = core.numpy(t1)
    arr = (C.c_void_p * 2)(t1, t2c)
    one = (C.c_void_p * 1)(t1)
    two = (C.c_void_p * 1)(t2c)
    L.rs_comm_fused_synch(comm, one, 1, 0)
    L.rs_comm_fused_synch(comm, two, 1, 0)
    L.rs_comm_fused_synch(comm, arr, 2, 1)
    L.rs_comm_wait(comm)
    R["comm_fused_a"], R["comm_fused_b"] = core.numpy(t1), core.numpy(t2c)
    L.rs_comm_fused_synch_half(comm, one, 1, 0)
    L.rs_comm_fused_synch_half(comm, two, 1, 0)
    L.rs_comm_fused_synch_half(comm, arr, 2, 1)
    L.rs_comm_wait(comm)
    R["comm_fused_half_a"], R["comm_fused_half_b"] = core.numpy(t1), core.numpy(t2c)
    t4 = core.tensor(g2)
    L.rs_comm_synch_half(comm, t4)
    L.rs_comm_wait(comm)
    R["comm_synch_half"] = core.numpy(t4)
    # top-K with residual: values spread over +-3 so that the integer-truncated keys differ
    g3 = (f32(200000) * np.float32(3)).astype(np.float32)
    t5, acc = core.tensor(g3), core.tensor(np.zeros(200000, np.float32))
    L.rs_comm_sparsification(comm, t5, acc, C.c_float(0.01), 1)
    L.rs_comm_wait(comm)
    L.rs_sync()
    R["comm_topk_dense"], R["comm_topk_residual"] = core.numpy(t5), core.numpy(acc)
    L.rs_comm_free(comm)
    np.savez(out_path, **R)
    print("worker %s: %d results" % (variant, len(R)))


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
