"""MNIST classifier: 784-30-10 MLP with Sigmoid, SGD (reference: example/mnist/main.cc, dataset.cc:60-80).

Reads the IDX files (``train-images-idx3-ubyte`` / ``train-labels-idx1-ubyte``) from ``--dataset``;
without it, trains on a synthetic set of the same shape.
"""
import argparse
import os
import struct
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def read_idx(path: str) -> np.ndarray:
    with open(path, "rb") as f:
        zero, dtype_code, ndim = struct.unpack(">HBB", f.read(4))
        if zero != 0 or dtype_code != 0x08:
            raise ValueError(f"not an unsigned-byte IDX file: {path}")
        dims = struct.unpack(">" + "I" * ndim, f.read(4 * ndim))
        return np.frombuffer(f.read(), dtype=np.uint8).reshape(dims)


class MNISTDataset:
    def __init__(self, root: str = "", train: bool = True, n_synth: int = 2048):
        prefix = "train" if train else "t10k"
        if root:
            self.images = read_idx(os.path.join(root, f"{prefix}-images-idx3-ubyte")).astype(np.float32) / 255.0
            self.labels = read_idx(os.path.join(root, f"{prefix}-labels-idx1-ubyte")).astype(np.int64)
        else:
            g = np.random.default_rng(0)
            self.labels = g.integers(0, 10, n_synth).astype(np.int64)
            centers = g.normal(0.5, 0.5, (10, 784)).astype(np.float32)
            self.images = (centers[self.labels] + g.normal(0, 0.2, (n_synth, 784))).astype(np.float32).reshape(-1, 28, 28)

    def Size(self):
        return len(self.labels)

    def __getitem__(self, i):
        return torch.from_numpy(self.images[i].reshape(784)), torch.tensor(self.labels[i])


def main(argv=None):
    from infinitrain_b200 import nn
    from infinitrain_b200.data import DataLoader
    from infinitrain_b200.optim import SGD

    ap = argparse.ArgumentParser()
    ap.add_argument("--dataset", default="")
    ap.add_argument("--bs", type=int, default=64)
    ap.add_argument("--num_epoch", type=int, default=1)
    ap.add_argument("--lr", type=float, default=0.5)
    ap.add_argument("--device", default="cpu")
    args = ap.parse_args(argv)
    dev = torch.device(args.device)
    model = nn.Sequential(nn.Linear(784, 30), nn.Sigmoid(), nn.Linear(30, 10)).to(dev)
    opt = SGD(model.Parameters(), args.lr, fused=False)
    ds = MNISTDataset(args.dataset)
    loss_fn = nn.CrossEntropyLoss()
    first = last = None
    for epoch in range(args.num_epoch):
        for i, (x, y) in enumerate(DataLoader(ds, args.bs)):
            opt.ZeroGrad()
            loss = loss_fn(model(x.to(dev)), y.to(dev))
            loss.backward()
            opt.Step()
            first = loss.item() if first is None else first
            last = loss.item()
            if i % 10 == 0:
                print(f"epoch {epoch} batch {i} loss {last:.4f}")
    print(f"final loss {last:.4f} (first {first:.4f})")
    return 0 if last < first else 1


if __name__ == "__main__":
    sys.exit(main())
