"""Trains a small MLP for a few steps with apache/singa's UNMODIFIED Python
layer (model.Model, layer.Linear / ReLU / SoftMaxCrossEntropy, autograd,
opt.SGD or opt.DistOpt) on top of the pybind11 `singa_wrap` of this repository
(singa_b200/adapter), and saves losses and parameters for the caller to check
against a numpy statement of the same steps.

usage: reference_python_worker.py <cpp|sgb> <out.npz> [plain|dist|dist_half|dist_partial|dist_topk|dist_threshold]
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from singa_b200.adapter import py_compat   # noqa: E402


def main(variant, out_path, mode):
    if variant == "sgb":
        # torch ships a newer NCCL under the same soname: it must be loaded
        # before the extension module pulls in the system one
        import torch  # noqa: F401
    py_compat.use(variant)
    from singa import device, layer, model, opt, singa_wrap, tensor
    if variant == "sgb":
        dev = device.create_cuda_gpu_on(0)
    else:
        dev = device.get_default_device()
    rng = np.random.default_rng(0)
    B, D, H, K = 32, 48, 64, 10

    class MLP(model.Model):
        def __init__(self):
            super().__init__()
            self.l1 = layer.Linear(H)
            self.relu = layer.ReLU()
            self.l2 = layer.Linear(K)
            self.loss = layer.SoftMaxCrossEntropy()

        def forward(self, x):
            return self.l2(self.relu(self.l1(x)))

        def train_one_batch(self, x, y):
            out = self.forward(x)
            loss = self.loss(out, y)
            if mode == "plain" or mode == "dist":
                self.optimizer(loss)
            elif mode == "dist_half":
                self.optimizer.backward_and_update_half(loss)
            elif mode == "dist_partial":
                self.optimizer.backward_and_partial_update(loss)
            elif mode == "dist_topk":
                self.optimizer.backward_and_sparse_update(loss, topK=True, spars=1.0)
            elif mode == "dist_threshold":
                self.optimizer.backward_and_sparse_update(loss, topK=False, spars=0.0)
            return out, loss

        def set_optimizer(self, o):
            self.optimizer = o

    m = MLP()
    sgd = opt.SGD(lr=0.05, momentum=0.9)
    if mode == "plain":
        m.set_optimizer(sgd)
    else:
        m.set_optimizer(opt.DistOpt(sgd, nccl_id=singa_wrap.NcclIdHolder(), local_rank=0, world_size=1))
    x_np = rng.standard_normal((B, D)).astype(np.float32)
    y_np = rng.integers(0, K, B).astype(np.int32)
    x = tensor.Tensor((B, D), dev)
    x.copy_from_numpy(x_np)
    y = tensor.Tensor((B,), dev, tensor.int32)
    y.copy_from_numpy(y_np)
    m.compile([x], is_train=True, use_graph=False, sequential=False)
    params0 = {k: tensor.to_numpy(v).copy() for k, v in m.get_params().items()}
    losses = []
    for _ in range(3):
        _, loss = m(x, y)
        losses.append(float(tensor.to_numpy(loss).ravel()[0]))
    dev.Sync()
    params = {k: tensor.to_numpy(v).copy() for k, v in m.get_params().items()}
    out = {"x": x_np, "y": y_np, "losses": np.array(losses, np.float64)}
    for k, v in params0.items():
        out["init:" + k] = v
    for k, v in params.items():
        out["final:" + k] = v
    np.savez(out_path, **out)
    print("worker %s/%s: losses %s" % (variant, mode, ["%.5f" % l for l in losses]))


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2], sys.argv[3] if len(sys.argv) > 3 else "plain")
