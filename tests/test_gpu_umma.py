"""The tcgen05 helpers of the library (csrc/umma.cuh) against numpy: D = A B^T with fp16 operands holding small integers
(every product and partial sum is exact in fp32, so the comparison is bit-exact), for both storage orders of the core
matrices in shared memory, for the A operand in tensor memory, and several K."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    from qwental_b200.gpu import Gpu
    g = Gpu()
    yield g
    g.close()


@pytest.mark.parametrize("K", [16, 64, 128])
@pytest.mark.parametrize("order", [0, 1, 2])
def test_umma_f16_matches_numpy(gpu, K, order):
    from qwental_b200.layers import u32
    if order == 2 and K % 32:
        pytest.skip("the tensor-memory form of the self-test stores 32 K values at a time")
    rng = np.random.default_rng(K + order)
    A = rng.integers(-15, 16, (128, K)).astype(np.float16)
    B = rng.integers(-8, 9, (16, K)).astype(np.float16)
    a, b, out = gpu.buf_from(A), gpu.buf_from(B), gpu.buf(128 * 16 * 4).zero()
    bt = gpu.batch()
    bt.kernel(gpu.compile("umma_test", "umma_test")).buf(0, a).buf(1, b).buf(2, out).bytes(3, u32(K, order)).dispatch((1,), (128,))
    bt.end()
    got = out.download(np.float32, 128 * 16).reshape(128, 16)
    ref = A.astype(np.float32) @ B.astype(np.float32).T
    assert np.array_equal(got, ref)
