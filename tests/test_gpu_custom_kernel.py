"""The reference's extension contract on the GPU: a user-defined ``Kernel`` that implements only ``compute`` gets
working ``mmv`` / ``dmmv`` / ``kernel(X1, X2)`` (falkon/kernels/kernel.py:462-505).  Same kernel, shapes, seeds and
assertions as the reference's own test of that contract (falkon/tests/test_custom_kernel.py:14-98: a scaled
linear kernel on Uniform[0,1) data, n = 2000, m = 1500, d = 10, t = 5, seeds 92-95).  Such kernels run block by block
through their own ``compute`` and library GEMMs (falkon_b200/mmv_ops/generic.py); the fused CUDA kernels serve the
built-in distance kernels only.
"""
import numpy as np
import pytest
import torch

from falkon_b200 import FalkonOptions
from falkon_b200.kernels import Kernel

pytestmark = pytest.mark.gpu

n, m, d, t = 2000, 1500, 10, 5


def _uniform(rows, cols, seed):
    return torch.from_numpy(np.random.default_rng(seed).random((rows, cols)).astype(np.float32))


class ScaledLinearKernel(Kernel):
    def __init__(self, lengthscale, options=None):
        super().__init__("scaled_linear", options)
        self.lengthscale = torch.as_tensor(lengthscale)

    def compute(self, X1, X2, out, diag, **kwargs):
        scale = self.lengthscale.to(device=X1.device, dtype=X1.dtype)
        if diag:
            out.copy_(torch.sum(X1 * scale * X2, dim=-1))
            return out
        return torch.matmul(X1 * scale, X2.T, out=out)


def _dense(A, B, scale):
    return (A.double() * scale) @ B.double().T


@pytest.mark.parametrize("where", ["cuda", "cpu"])
def test_products_of_a_user_defined_kernel(where):
    A, B, v, w = _uniform(n, d, 92), _uniform(m, d, 93), _uniform(m, t, 94), _uniform(n, t, 95)
    A, B, v, w = (x.to(where) for x in (A, B, v, w))
    k = ScaledLinearKernel(3.0)
    K = _dense(A, B, 3.0)
    out = k.mmv(A, B, v)
    assert out.device == A.device
    torch.testing.assert_close(out.double(), K @ v.double(), rtol=1e-4, atol=1e-3)
    given = torch.empty(n, t, device=where)
    assert k.mmv(A, B, v, out=given).data_ptr() == given.data_ptr()
    torch.testing.assert_close(given.double(), K @ v.double(), rtol=1e-4, atol=1e-3)
    want = K.T @ (K @ v.double() + w.double())
    torch.testing.assert_close(k.dmmv(A, B, v, w).double(), want, rtol=1e-4, atol=1e-1)
    given = torch.empty(m, t, device=where)
    k.dmmv(A, B, v, w, out=given)
    torch.testing.assert_close(given.double(), want, rtol=1e-4, atol=1e-1)
    torch.testing.assert_close(k.dmmv(A, B, None, w).double(), K.T @ w.double(), rtol=1e-4, atol=1e-2)
    torch.testing.assert_close(k(A, B).double(), K, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(k(A, A, diag=True).double(), torch.diagonal(_dense(A, A, 3.0)), rtol=1e-5, atol=1e-5)


def test_user_defined_kernel_under_a_memory_budget():
    A, B, v, w = (x.cuda() for x in (_uniform(n, d, 92), _uniform(m, d, 93), _uniform(m, t, 94), _uniform(n, t, 95)))
    k = ScaledLinearKernel(3.0)
    K = _dense(A, B, 3.0)
    tight = FalkonOptions(max_gpu_mem=2 * 2**20)  # 2 MiB: blocks of about 300 rows
    torch.testing.assert_close(k.mmv(A, B, v, opt=tight).double(), K @ v.double(), rtol=1e-4, atol=1e-3)
    torch.testing.assert_close(k.dmmv(A, B, v, w, opt=tight).double(), K.T @ (K @ v.double() + w.double()),
                               rtol=1e-4, atol=1e-1)
    with pytest.raises(MemoryError):
        k.mmv(A, B, v, opt=FalkonOptions(max_gpu_mem=1024))
