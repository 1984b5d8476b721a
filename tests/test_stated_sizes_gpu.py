"""Parity at the sizes the benchmark configurations state (the other parity tests use reduced
shapes).  The oracle is the single-threaded cc restatement, so the largest contractions are checked
on sampled rows and columns: the host slices A's rows and B's columns, the oracle computes exactly
those outputs over the full K, and they are compared with the same positions of the device result."""
import numpy as np
import pytest

from ocannl_b200 import backend as bk
from ocannl_b200 import workloads as W
from tests.parity import compare, run_device, run_oracle

pytestmark = pytest.mark.gpu

# Absolute tolerances beside rel 2e-2 (the stated tolerance of bf16 contractions).  z is an fp32 sum
# of K products summed in another order: 2e-3 at K = 1024, growing with sqrt(K).  y runs the
# composed GELU in bf16, one rounding per operation: where `1 + tanh(..)` nearly cancels (z between
# -4 and -1), a one-unit flip of the rounded tanh (2^-8 for values in [0.5, 1)) moves y by
# 0.5 |z| 2^-8, up to 8e-3, on the rare elements where the two sides round apart.
ATOL_Z, ATOL_Y = 2e-3, 8e-3


def test_einsum_gelu_1024_full(device):
    """Config 3 at batch 8, M = N = K = 1024: every element of z (fp32) and y (bf16) against the
    oracle (17 GFLOP on one host core)."""
    ir = W.einsum_gelu(8, 1024, 1024, 1024)
    inputs = W.einsum_gelu_inputs(8, 1024, 1024, 1024)
    want = run_oracle(ir, inputs)
    got, info = run_device(device, ir, inputs)
    assert info["stages"][0]["kind"] == "gemm" and len(info["stages"]) == 1, info
    compare(ir, got, want, rtol=2e-2, atol=ATOL_Z, only=["z"])
    compare(ir, got, want, rtol=2e-2, atol=ATOL_Y, only=["y"])


def _sample_positions(n, tile, inside):
    """Positions `inside` (offsets within a tile) of every tile of extent `tile` along an axis of n."""
    return np.array(sorted({t * tile + o for t in range(n // tile) for o in inside if t * tile + o < n}))


@pytest.mark.parametrize("n", [4096, 8192])
def test_einsum_gelu_large_sampled(device, n):
    """Config 3 at batch 8, M = N = K = 4096 and 8192 (the sizes the contraction roofline is quoted
    on).  Sampled rows: the first and last row of each 128-row half of every 256-row CTA-pair
    tile (so both CTAs of every pair, and the edge between them); sampled columns: first, last
    and the 32-column chunk edges of every 256-column tile.  Every output tile of every batch
    index -- first and last tile, every wave of the persistent grid -- therefore holds checked
    positions, each over the full K."""
    batch = 8
    ir = W.einsum_gelu(batch, n, n, n)
    code = bk.Code(ir)
    rt = bk.Context(device).link(code)
    info = rt.info()
    assert [s["kind"] for s in info["stages"]] == ["gemm"] and "CTA pair" in info["stages"][0]["note"], info
    rows = _sample_positions(n, 256, (0, 127, 128, 255))
    cols = _sample_positions(n, 256, (0, 31, 32, 255))
    if n == 8192:                      # halve the sample, keep every tile covered
        rows, cols = rows[::2], cols[1::2]
    a_rows = np.empty((batch, len(rows), n), np.uint16)
    b_cols = np.empty((batch, n, len(cols)), np.uint16)
    pa, oa, _ = rt.context.arrays["a"]
    pb, ob, _ = rt.context.arrays["b"]
    for b in range(batch):
        # one batch block at a time keeps the host's working set near 1 GB at n = 8192
        blk = W.store("bfloat16", np.random.default_rng(600 + b).standard_normal((n, n), np.float32))
        a_rows[b] = blk[rows]
        device.from_host(pa, oa + b * blk.nbytes, blk)
        device.await_()
        blk = W.store("bfloat16", np.random.default_rng(700 + b).standard_normal((n, n), np.float32))
        b_cols[b] = blk[:, cols]
        device.from_host(pb, ob + b * blk.nbytes, blk)
        device.await_()
    bias = np.random.default_rng(8).standard_normal(n).astype(np.float32)
    rt.context.from_host("bias", bias)
    rt.run()
    device.await_()
    # the oracle on the slices: same routine, M = len(rows), N = len(cols), full K
    small = W.einsum_gelu(batch, len(rows), len(cols), n)
    want = run_oracle(small, {"a": a_rows, "b": b_cols, "bias": bias[cols]})
    pz, oz, _ = rt.context.arrays["z"]
    py, oy, _ = rt.context.arrays["y"]
    got_z = np.empty((batch, len(rows), len(cols)), np.float32)
    got_y = np.empty((batch, len(rows), len(cols)), np.uint16)
    zrow = np.empty(n, np.float32)
    yrow = np.empty(n, np.uint16)
    for b in range(batch):
        for i, r in enumerate(rows):
            device.to_host(pz, oz + 4 * ((b * n + int(r)) * n), zrow)
            device.to_host(py, oy + 2 * ((b * n + int(r)) * n), yrow)
            device.await_()
            got_z[b, i] = zrow[cols]
            got_y[b, i] = yrow[cols]
    compare(small, {"z": got_z, "y": got_y}, want, rtol=2e-2, atol=ATOL_Z * np.sqrt(n / 1024.0), only=["z"])
    compare(small, {"z": got_z, "y": got_y}, want, rtol=2e-2, atol=ATOL_Y, only=["y"])
    pools = {p for p, _, _ in rt.context.arrays.values()}
    rt.free()
    code.free()
    for p in pools:
        device.free_pool(p)


@pytest.mark.parametrize("act", ["gelu", "relu"])
def test_decoder_full_width_reduced_batch(device, act):
    """Config 4 at its stated width -- 6 layers, d_model 512, 8 heads of 64, FFN 2048, sequence
    256, vocabulary 27 -- on a batch of 2 sequences instead of 64 (the batch axis only repeats the
    same per-sequence work; 21 GFLOP on the oracle's one core)."""
    ir = W.transformer_forward(batch=2, act=act)
    inputs = dict(W.transformer_params(), **W.transformer_inputs(batch=2))
    want = run_oracle(ir, inputs)
    got, info = run_device(device, ir, inputs)
    kinds = [s["kind"] for s in info["stages"]]
    assert kinds.count("attention") == 6, kinds       # q.k^T, softmax and attn.v of a layer are one launch
    assert kinds.count("gemm") + 2 * kinds.count("attention") >= 6 * 7, kinds
    compare(ir, got, want, rtol=2e-2, atol=2e-2)


def test_mlp_forward_8192_rows(device):
    """Config 5 forward at the benchmarked shard size: 8192 rows through 784-1024-1024-10, every
    node against the oracle, and the mean cross-entropy loss to 1e-3 relative."""
    ir = W.mlp_forward(rows=8192)
    x, onehot = W.mlp_inputs(rows=8192)
    inputs = dict(W.mlp_params(), x=x, labels=onehot)
    want = run_oracle(ir, inputs)
    got, info = run_device(device, ir, inputs)
    # The logits sum 1024 products of a bf16 activation (up to ~10, so one unit in its last place
    # is up to 2^-5) and a weight (up to 0.08): an activation that rounds to the neighbouring bf16
    # value on one side moves a logit by up to 2.5e-3, several of them more.  The absolute part of
    # the tolerance is therefore 2e-2 of the node's largest magnitude; the relative part stays 2e-2.
    for t in ir.params():
        scale = float(np.abs(W.load(t.prec, want[t.ident]).astype(np.float64)).max())
        compare(ir, got, want, rtol=2e-2, atol=max(2e-3, 2e-2 * scale) if t.ident in ("logits", "exp_vals", "sum_exp", "max_l") else 2e-3,
                only=[t.ident])
    assert abs(float(got["loss"][0]) - float(want["loss"][0])) <= 1e-3 * abs(float(want["loss"][0]))
