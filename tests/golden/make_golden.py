"""Generates tests/golden/*.npz: small seeded inputs with outputs of the formulations the
reference's own tests use as their oracle, evaluated in float64 with PyTorch on the CPU:

  * cdist    : torch.cdist(a, b, p) for p in {1.0, 1.3, 2.0}, L=2 batches
               (tests/test_cdist.py:75 of the reference compares against exactly this)
  * gradient : the einsum pair of tests/test_cdist_grad.py:43-49 for p = 2

The reference package itself cannot be imported here (it needs cuda.core, lmdb and a
GPU), so these vectors come from its test oracle, not from its kernels.

    python tests/golden/make_golden.py
"""
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def cdist_vectors():
    g = torch.Generator().manual_seed(1234)
    L, M, N, K = 2, 37, 29, 19
    a = torch.randn(L, M, K, generator=g, dtype=torch.float32)
    b = torch.randn(L, N, K, generator=g, dtype=torch.float32)
    out = {"a": a.numpy(), "b": b.numpy()}
    for p in (1.0, 1.3, 2.0):
        mode = "donot_use_mm_for_euclid_dist"
        ref = torch.cdist(a.double(), b.double(), p=p, compute_mode=mode)
        out[f"cdist_p{p}"] = ref.numpy()
    np.savez_compressed(os.path.join(HERE, "cdist_small.npz"), **out)


def grad_vectors():
    g = torch.Generator().manual_seed(4321)
    L, K, M, N, O = 2, 23, 21, 18, 5
    a = torch.randn(L, K, M, generator=g, dtype=torch.float32)
    b = torch.randn(L, N, K, generator=g, dtype=torch.float32)
    c = torch.randn(L, O, K, generator=g, dtype=torch.float32)
    d = torch.randn(L, N, M, generator=g, dtype=torch.float32)
    coefs, kernel_matrix = c.double(), a.double()
    x, z = b.double().permute(0, 2, 1), d.double().permute(0, 2, 1)
    left = torch.einsum('bli,bij,bjd->bljd', coefs, kernel_matrix, z)
    right = torch.einsum('bli,bij,bid->bljd', coefs, kernel_matrix, x)
    ref = (left - right).permute(0, 1, 3, 2).contiguous()   # (L, O, N, M)
    np.savez_compressed(os.path.join(HERE, "grad_small.npz"), a=a.numpy(), b=b.numpy(), c=c.numpy(), d=d.numpy(),
                        grad_p2=ref.numpy())


if __name__ == "__main__":
    cdist_vectors()
    grad_vectors()
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))
