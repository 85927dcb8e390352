"""GPU: the tcgen05 / tensor-memory helpers against a plain matrix product."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [16, 64, 128, 256])
def test_umma_tile_product(backend, n):
    be = backend
    rng = np.random.default_rng(n)
    a = rng.normal(size=(128, 64)).astype(np.float16)
    b = rng.normal(size=(n, 64)).astype(np.float16)
    ab, bb, cb = be.from_host(a), be.from_host(b), be.alloc(128 * n * 4)
    be._check(be._lib.infr_cuda_umma_selftest(be._ctx, ab.handle, bb.handle, cb.handle, n))
    got = be.download(cb, np.float32).reshape(128, n)
    want = a.astype(np.float32) @ b.astype(np.float32).T
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-3)
