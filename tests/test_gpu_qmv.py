"""GPU parity of the quantized matvec kernels, through the C ABI (qw_gpu.h batches).

dq_test and qmv_gg must be bit-exact against the CPU oracle; qmv_mma must be within fp16 tolerance of the FP64
product of the exactly decoded weights, and every batched row must be bit-identical to the same row alone."""
import numpy as np
import pytest

from oracle import oracle as orc
from qwental_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    from qwental_b200.gpu import Gpu
    g = Gpu()
    yield g
    g.close()


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def run_dq(gpu, qtype, W, K):
    k = gpu.compile("dq_test", "dq_test_%d" % qtype, DQ_TEST=qtype)
    N = W.shape[0]
    wb, yb = gpu.buf_from(W), gpu.buf(N * K * 4)
    gpu.batch().kernel(k).buf(0, wb).buf(1, yb).bytes(2, np.array([K, W.shape[1]], np.uint32)).dispatch((N,), (32,)).end()
    return yb.download(np.float32, N * K).reshape(N, K)


def run_qmv(gpu, family, qtype, W, K, x, f32=True):
    N, B = W.shape[0], x.shape[0]
    k = gpu.compile(family, "%s_%d_%d_%d" % (family, qtype, K, int(f32)), GF=qtype, KD=K, NB=64, YT_F32=int(f32))
    wb, xb = gpu.buf_from(W), gpu.buf_from(x)
    yb = gpu.buf(B * N * (4 if f32 else 2)).zero()
    args = np.array([N, K, N, B], np.uint32)
    gpu.batch().kernel(k).buf(0, wb).buf(3, xb).buf(4, yb).bytes(5, args).dispatch(((N + 7) // 8,), (256,)).end()
    return yb.download(np.float32 if f32 else np.float16, B * N).reshape(B, N)


def test_dq_golden_bit_exact(gpu, golden):
    assert np.array_equal(bits(run_dq(gpu, 21, golden["iq3s_raw"], 2048)), bits(golden["iq3s_ref"]))
    assert np.array_equal(bits(run_dq(gpu, 21, golden["edge_raw"], 256)), bits(golden["edge_ref"]))
    assert np.array_equal(bits(run_dq(gpu, 8, golden["q8_raw"], 2048)), bits(golden["q8_ref"]))


@pytest.mark.parametrize("qtype,N,K", [(21, 4096, 2048), (21, 64, 4096), (8, 256, 2048)])
def test_dq_random_bit_exact_vs_oracle(gpu, qtype, N, K):
    W = synth.quant_rows(np.random.default_rng(7), qtype, N, K)
    assert np.array_equal(bits(run_dq(gpu, qtype, W, K)), bits(orc.dq_rows(qtype, W, K)))


# config 0 of the benchmark: W 4096 x 2048 IQ3_S, x 2048 fp16, batch 1, fp32 accumulate, seed 0
@pytest.mark.parametrize("qtype,N,K,B", [(21, 4096, 2048, 1), (21, 512, 4096, 4), (8, 1024, 2048, 3), (21, 40, 256, 9)])
def test_qmv_gg_bit_exact_vs_canonical_oracle(gpu, qtype, N, K, B):
    rng = np.random.default_rng(0)
    W = synth.quant_rows(rng, qtype, N, K)
    x = synth.acts_fp16(rng, B, K)
    y = run_qmv(gpu, "qmv_gg", qtype, W, K, x)
    assert np.array_equal(bits(y), bits(orc.qmv_canon(qtype, W, K, x)))


# config 1: ragged batched matvec shapes (reduced row counts for lm_head so the oracle finishes in seconds)
@pytest.mark.parametrize("qtype,N,K", [(21, 5120, 2048), (21, 2048, 4096), (8, 4096, 2048), (21, 12352, 2048)])
@pytest.mark.parametrize("B", [1, 4, 8, 16, 17, 40, 64])
def test_qmv_mma_close_to_fp64_and_rows_independent_of_batch(gpu, qtype, N, K, B):
    rng = np.random.default_rng(1)
    W = synth.quant_rows(rng, qtype, N, K)
    x = synth.acts_fp16(rng, B, K)
    y = run_qmv(gpu, "qmv_mma", qtype, W, K, x)
    ref = orc.qmv_f64(qtype, W, K, x)
    # tolerance: fp16 products are exact, fp32 accumulation over K terms: 2e-5 of the output scale
    assert np.abs(y - ref).max() <= 2e-5 * np.abs(ref).max()
    # each row alone gives the same bits (batched == alone)
    for b in sorted({0, B // 2, B - 1}):
        ya = run_qmv(gpu, "qmv_mma", qtype, W, K, x[b:b + 1])
        assert np.array_equal(bits(ya[0]), bits(y[b]))


def test_qmv_mma_fp16_output_and_top1(gpu):
    rng = np.random.default_rng(2)
    W = synth.q8_0_rows(rng, 8192, 2048)
    x = synth.acts_fp16(rng, 16, 2048)
    y32 = run_qmv(gpu, "qmv_mma", 8, W, 2048, x, f32=True)
    y16 = run_qmv(gpu, "qmv_mma", 8, W, 2048, x, f32=False)
    assert np.array_equal(y16, y32.astype(np.float16))
    ref = orc.qmv_f64(8, W, 2048, x)
    assert np.array_equal(y32.argmax(1), ref.argmax(1))


def test_bad_arguments_fail_the_batch_not_the_device(gpu):
    from qwental_b200.gpu import GpuError
    k = gpu.compile("qmv_mma", "qmv_bad", GF=21, KD=2048, NB=8, YT_F32=1)
    wb, xb, yb = gpu.buf(880 * 16), gpu.buf(4096), gpu.buf(64)
    with pytest.raises(GpuError):  # y too small for N = 16 rows of fp32
        gpu.batch().kernel(k).buf(0, wb).buf(3, xb).buf(4, yb).bytes(5, np.array([16, 2048, 16, 2], np.uint32)).dispatch((2,), (256,)).end()
    # the device is still usable
    W = synth.iq3s_rows(np.random.default_rng(3), 16, 2048)
    assert np.array_equal(bits(run_dq(gpu, 21, W, 2048)), bits(orc.dq_rows(21, W, 2048)))
