"""Single-precision operands on the tensor cores as tf32: parity with the oracle (which multiplies
in full fp32) within the tolerance stated for tf32 contractions, rel 2e-2 on the outputs, and the
exact generic path behind `tf32=0` within the fp32 pointwise tolerance."""
import numpy as np
import pytest

from ocannl_b200 import workloads as W
from tests.parity import compare, run_device, run_oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(2, 256, 256, 256), (1, 200, 136, 200), (3, 128, 512, 64), (1, 384, 48, 1000),
                                   (2, 300, 200, 72), (1, 520, 264, 40), (1, 1024, 1024, 1024)])
def test_einsum_bias_gelu_tf32(device, shape):
    """Config 3's routine with fp32 operands: K-major A, N-major B (the transposed smem form of the
    tf32 kind), ragged M / N / K through the tensor maps' zero fill, CTA pairs from M >= 256."""
    b, m, n, k = shape
    ir = W.einsum_gelu(b, m, n, k, in_prec="single", y_prec="single")
    inputs = W.einsum_gelu_inputs(b, m, n, k, in_prec="single")
    want = run_oracle(ir, inputs)
    got, info = run_device(device, ir, inputs)
    assert info["stages"][0]["kind"] == "gemm" and "tf32" in info["stages"][0]["note"], info
    # a product of two tf32-truncated operands is off by up to 2^-9 relative; a sum of K such
    # products of N(0, 1) values by about 2^-10 sqrt(K): the absolute part follows sqrt(K)
    compare(ir, got, want, rtol=2e-2, atol=2e-3 * np.sqrt(k))
    got2, info2 = run_device(device, ir, inputs, options="tf32=0")
    assert all(s["kind"] != "gemm" for s in info2["stages"])
    compare(ir, got2, want, rtol=2e-5, atol=1e-5 * np.sqrt(k))


@pytest.mark.parametrize("options,rtol,atol", [(None, 2e-2, 2e-2), ("tf32=0", 1e-5, 1e-5)])
def test_makemore_forward_fp32_weights(device, options, rtol, atol):
    """Config 2 with fp32 weights: the logits layer (4096 x 27 x 200) is a tf32 contraction with the
    log-softmax pieces in its epilogue by default, exact generic kernels with tf32=0; the guarded
    gather is bit-exact either way."""
    ir = W.makemore_forward(wprec="single")
    ids, onehot = W.makemore_inputs()
    ids[5, 1], ids[6, 2], ids[7, 0] = -1.0, 27.0, 1.5
    inputs = dict(W.makemore_params(), input_batch=ids, target_batch=onehot)
    want = run_oracle(ir, inputs)
    got, info = run_device(device, ir, inputs, options=options)
    assert any("tf32" in (s["note"] or "") for s in info["stages"]) == (options is None)
    compare(ir, got, want, rtol=rtol, atol=atol, exact=["embed"])


def test_mlp_training_fp32(device):
    """Config 5's update routine with fp32 weights and activations on a 512-row shard: forward,
    dW (both operands M/N-major, batch axis contracted, split over K) and dX as tf32 contractions."""
    rows = 512
    ir = W.mlp_train_update(rows=rows, wprec="single")
    x, onehot = W.mlp_inputs(rows=rows, xprec="single")
    inputs = dict(W.mlp_params(wprec="single"), x=x, labels=onehot)
    want = run_oracle(ir, inputs)
    got, info = run_device(device, ir, inputs)
    assert sum("tf32" in (s["note"] or "") for s in info["stages"]) >= 6, info
    for t in ir.params():
        w_ = want[t.ident].astype(np.float64).reshape(-1)
        g_ = got[t.ident].astype(np.float64).reshape(-1)
        if t.ident.endswith("_grad"):
            # An activation within tf32's rounding of zero passes its relu gate on one side only (a few
            # in ten thousand do); each such gate switches one whole element of an activation
            # gradient and one whole term of every gradient behind it.  With the exact kernels
            # (tf32=0) the same comparison gives 5e-7.  A gradient is therefore compared as a tensor,
            # relative error in the 2-norm, with the allowance the bf16 tests give gate switches.
            assert np.linalg.norm(g_ - w_) <= 5e-2 * np.linalg.norm(w_), (t.ident, np.linalg.norm(g_ - w_), np.linalg.norm(w_))
        else:
            scale = float(np.abs(w_).max())
            bad = np.abs(g_ - w_) > 2e-2 * np.abs(w_) + 2e-2 * max(scale, 1e-30)
            assert not bad.any(), (t.ident, int(bad.sum()), w_.size, scale)
