"""Device parity: every routine runs through the C ABI on the GPU and on the CPU oracle
(the restated cc backend) from identical seeded inputs.

Tolerances (the ones the north star states): fp32 pointwise rel 1e-5; bf16 contractions
rel 2e-2 with fp32 accumulation; index work (the gather) bit-exact."""
import numpy as np
import pytest

from ocannl_b200 import workloads as W
from tests.golden.golden_routines import GOLDEN, n3_fwd
from tests.parity import compare, run_device, run_oracle

pytestmark = pytest.mark.gpu


def test_golden_routines_on_device(device):
    for name, mk in GOLDEN.items():
        ir = mk()
        rng = np.random.default_rng(1)
        inputs = {}
        for t in ir.params():
            if t.prec == "half":
                inputs[t.ident] = rng.normal(0, 1, t.dims).astype(np.float16)
            elif t.prec == "bfloat16":
                inputs[t.ident] = W.f32_to_bf16_bits(rng.normal(0, 1, t.dims).astype(np.float32))
            elif t.prec == "byte":
                inputs[t.ident] = np.ones(t.dims, np.uint8)
            else:
                inputs[t.ident] = rng.normal(0, 1, t.dims).astype(np.float32)
        want = run_oracle(ir, inputs)
        got, _ = run_device(device, ir, inputs)
        for t in ir.params():
            assert np.array_equal(got[t.ident].view(np.uint8), want[t.ident].view(np.uint8)), (name, t.ident)


@pytest.mark.parametrize("prec", ["bfloat16", "half", "single"])
@pytest.mark.parametrize("options", ["fuse=0", "fuse=0 pairs=0", None])
def test_pointwise_arithmetic_bits(device, prec, options):
    """Every exactly-rounded operation of the pointwise tables, in the pair form (packed 16-bit add,
    sub, mul, min, max, one packed rounding per float pair) and in the one-element form, gives the
    bits the cc restatement gives: the packed instructions round the exact result once, the
    reference rounds a float result, and for operands of the format these coincide.  Half is
    compared with a tolerance: the reference's C text writes half arithmetic on native `_Float16`
    values (its conversion macros are the identity then), so how often a chain of half operations
    is rounded is the host compiler's choice (gcc keeps float intermediates unless the CPU has
    half arithmetic), while the device rounds after every operation as the cc backend's rule says."""
    from ocannl_b200.low_level import Routine, Seq, Set, loops, binop, un, where, fma
    r = Routine("pointwise_" + prec)
    a = r.tn("a", prec, [96, 64], read_only=True)
    b = r.tn("b", prec, [96, 64], read_only=True)
    c = r.tn("c", "single", [96, 64], read_only=True)
    outs = {}
    body = []
    exprs = {
        "add": lambda x, y, z: x + y, "sub": lambda x, y, z: x - y, "mul": lambda x, y, z: x * y,
        "div": lambda x, y, z: x / y, "max": lambda x, y, z: binop("max", x, y), "min": lambda x, y, z: binop("min", x, y),
        "neg_relu": lambda x, y, z: un("relu", -x) + un("relu", y), "gate": lambda x, y, z: binop("relu_gate", x, y),
        "where": lambda x, y, z: where(binop("lt", x, y), x, y), "fma": lambda x, y, z: fma(x, y, x),
        "mixed": lambda x, y, z: (x * z + y) * 0.5 - z, "cube": lambda x, y, z: x ** 3.0 + y ** 2.0,
        "sqrt_recip": lambda x, y, z: un("sqrt", x * x) + un("recip", y),
    }
    for name, f in exprs.items():
        t = r.tn("o_" + name, prec, [96, 64])
        outs[name] = t
        i, j = r.syms(2)
        body.append(loops([(i, 96), (j, 64)], Set(t, (i, j), f(a[i, j], b[i, j], c[i, j]))))
    r.body = Seq(body)
    rng = np.random.default_rng(11)
    va = rng.normal(0, 1, (96, 64)).astype(np.float32)
    vb = rng.normal(0, 3, (96, 64)).astype(np.float32)
    vb[np.abs(vb) < 1e-3] = 1.0
    va[0, :8] = [0.0, -0.0, 1.0, -1.0, 65504.0, 1e-7, 3.0e38, -3.0e38]        # zeros, format edges
    vb[0, :8] = [0.0, 1.0, -1.0, 2.0 ** -14, 65504.0, 1e-7, 3.0e38, 1.0]
    vc = rng.normal(0, 1, (96, 64)).astype(np.float32)
    inputs = {"a": W.store(prec, va), "b": W.store(prec, vb), "c": vc}
    want = run_oracle(r, inputs)
    got, info = run_device(device, r, inputs, options=options)
    if options == "fuse=0":
        assert all("pairs" in (s["note"] or "") for s in info["stages"]), info
    elif options is None:      # thirteen small stages: one single-block kernel
        assert len(info["stages"]) == 1, info
    for name, t in outs.items():
        g = np.ascontiguousarray(got[t.ident]).view(np.uint16 if prec != "single" else np.uint32)
        w_ = np.ascontiguousarray(want[t.ident]).view(np.uint16 if prec != "single" else np.uint32)
        if name in ("div", "sqrt_recip", "cube") or prec == "half":
            # libm / division / multiplication chains: last-bit tolerance; half: see the docstring
            gv = W.load(prec, got[t.ident]).astype(np.float64)
            wv = W.load(prec, want[t.ident]).astype(np.float64)
            rtol = {"single": 1e-5, "half": 4e-3}.get(prec, 8e-3)       # fp32: the pointwise tolerance; 16-bit: 1-2 units
            fin = np.isfinite(wv)
            scale = float(np.abs(wv[fin & (np.abs(wv) < 1e30)]).max())  # sums of terms of either sign: absolute part
            ok = np.isclose(gv, wv, rtol=rtol, atol=rtol * scale * (1e-2 if prec == "single" else 1.0), equal_nan=True) | (gv == wv)
            assert ok.all(), (name, np.argwhere(~ok)[:4])
        else:
            same = (g == w_) | (np.isnan(W.load(prec, got[t.ident])) & np.isnan(W.load(prec, want[t.ident])))
            assert same.all(), (name, np.argwhere(~same)[:4], g[~same][:4], w_[~same][:4])


def test_pair_form_falls_back_on_element_aligned_bindings(device):
    """A pair-form stage reads 16-bit elements two at a time.  A node bound one element into its
    pool -- which the reference's allocator may do, it aligns to the element size only
    (arrayjit/lib/backends.ml:22-51) -- links all the same: the statement is re-planned in the
    one-element form, and the values are right."""
    from ocannl_b200 import backend as bk
    from ocannl_b200.low_level import Routine, Seq, Set, loops
    r = Routine("scale2")
    x = r.tn("x", "bfloat16", [64, 32], read_only=True)
    y = r.tn("y", "bfloat16", [64, 32])
    i, j = r.syms(2)
    r.body = Seq([loops([(i, 64), (j, 32)], Set(y, (i, j), x[i, j] + x[i, j]))])
    pool = device.alloc_pool(1 << 16)
    xs = W.f32_to_bf16_bits(np.random.default_rng(3).normal(0, 1, (64, 32)).astype(np.float32))
    code = bk.Code(r)
    assert any((s["note"] or "").endswith("pairs") for s in code.info()["stages"])
    for x_off, paired in ((2, False), (4096, True), (6, False)):
        arrays = {"x": (pool, x_off, x), "y": (pool, 8192, y)}
        rt = bk.Context(device, dict(arrays)).link(code)
        assert any((s["note"] or "").endswith("pairs") for s in rt.info()["stages"]) == paired
        rt.context.from_host("x", xs)
        rt.run()
        got = W.bf16_bits_to_f32(rt.context.to_host("y"))
        assert np.array_equal(got, W.bf16_bits_to_f32(W.f32_to_bf16_bits(2 * W.bf16_bits_to_f32(xs))))
        rt.free()
    with pytest.raises(bk.B200Error, match="element size"):
        bk.Context(device, {"x": (pool, 1, x), "y": (pool, 8192, y)}).link(code)
    device.free_pool(pool)


def test_uploads_on_second_stream_keep_order(device):
    """With b200_set_async_uploads the copies run on their own stream; launches queued after a copy
    still see its data, and a copy queued after a launch does not overwrite what the launch reads."""
    ir = W.mlp_forward(rows=256)
    x, onehot = W.mlp_inputs(rows=256)
    x2, onehot2 = W.mlp_inputs(rows=256, seed=77, label_seed=78)
    params = W.mlp_params()
    want = [run_oracle(ir, dict(params, x=a, labels=b))["loss"] for a, b in ((x, onehot), (x2, onehot2))]
    from ocannl_b200 import backend as bk
    code = bk.Code(ir)
    rt = bk.Context(device).link(code)
    device.set_async_uploads(True)
    try:
        for k, v in params.items():
            rt.context.from_host(k, v)
        px, ox, _ = rt.context.arrays["x"]
        pl, ol, _ = rt.context.arrays["labels"]
        ps, os_, _ = rt.context.arrays["loss"]
        h = [(bk.PinnedBuffer(a.shape, a.dtype), bk.PinnedBuffer(b.shape, b.dtype)) for a, b in ((x, onehot), (x2, onehot2))]
        for (ha, hb), (a, b) in zip(h, ((x, onehot), (x2, onehot2))):
            ha.array[...] = a
            hb.array[...] = b
        out = [bk.PinnedBuffer((1,), np.float32) for _ in range(6)]
        for i in range(6):       # alternate the two batches through ONE input buffer, no host sync in between
            ha, hb = h[i % 2]
            device.from_host(px, ox, ha.array)
            device.from_host(pl, ol, hb.array)
            rt.run()
            device.to_host(ps, os_, out[i].array)
        device.await_()
        for i in range(6):
            np.testing.assert_allclose(out[i].array[0], want[i % 2][0], rtol=2e-2)
        assert abs(float(want[0][0]) - float(want[1][0])) > 1e-4     # the two batches are told apart
    finally:
        device.set_async_uploads(False)


@pytest.mark.parametrize("prec", ["single", "double", "bfloat16", "half", "int32"])
@pytest.mark.parametrize("variant,count,options", [("light", 5, None), ("crypto", 1000, "fuse=0"), ("light", 70001, None)])
def test_threefry_uniform_bits(device, prec, variant, count, options):
    """Random numbers are integer work: seed and counter widening, threefry4x32 (2-round and
    20-round), the vector and the one-value uniform conversions agree bit for bit."""
    ir = n3_fwd(prec, count, variant, scalar_too=prec != "int32")
    want = run_oracle(ir, {})
    got, _ = run_device(device, ir, {}, options=options)
    for t in ir.params():
        assert np.array_equal(np.ascontiguousarray(got[t.ident]).view(np.uint8),
                              np.ascontiguousarray(want[t.ident]).view(np.uint8)), t.ident
    if prec == "single" and variant == "light":     # test/operations/test_threefry4x32.ml:37-45
        assert ["%.4g" % v for v in got["n3"][:5]] == ["0.4638", "0.7325", "0.5608", "0.5066", "0.5019"]


@pytest.mark.parametrize("options", [None, "fuse=0"])
@pytest.mark.parametrize("graph", [False, True])
def test_moons_training_steps(device, graph, options):
    """Config 1: forward + backprop + SGD, five steps over different batches; parameters,
    gradients, activations and the loss agree with the cc restatement to rel 1e-5."""
    ir = W.moons_train_step()
    x, y = W.moons_inputs()
    inputs = dict(W.moons_params(), moons_flat=x, moons_classes=y)
    statics = [{"i1": b, "i2": s} for s, b in enumerate([0, 1, 7, 50, 3])]
    want = run_oracle(ir, inputs, statics)
    got, info = run_device(device, ir, inputs, statics, options=options, graph=graph)
    assert (len(info["stages"]) == 1) == (options is None)       # one fused launch by default
    compare(ir, got, want, rtol=1e-5, atol=1e-6)
    assert abs(float(got["scalar_loss"][0])) > 0


def test_moons_static_index_errors(device):
    from ocannl_b200 import backend as bk
    ir = W.moons_train_step()
    code = bk.Code(ir)
    rt = bk.Context(device).link(code)
    with pytest.raises(bk.UserError):
        rt.run(i1=51, i2=0)          # range is 0..50
    with pytest.raises(bk.UserError):
        rt.run(i1=-1, i2=0)
    rt.run(i1=0, i2=0)
    device.await_()
    rt.free()


@pytest.mark.parametrize("wprec", ["single", "bfloat16"])
@pytest.mark.parametrize("options", [None, "gemm=0 coop=0"])
def test_makemore_forward(device, wprec, options):
    """Config 2 at full size (batch 4096).  The gathered embedding is index work: bit-exact,
    including ids that are negative, too large or fractional (they gather 0)."""
    ir = W.makemore_forward(wprec=wprec)
    ids, onehot = W.makemore_inputs()
    ids[0, 0], ids[1, 1], ids[2, 2] = -1.0, 27.0, 1.5
    inputs = {k: W.store(wprec, v) for k, v in W.makemore_params().items()}
    inputs.update(input_batch=ids, target_batch=onehot)
    want = run_oracle(ir, inputs)
    if wprec == "single":      # exact fp32 arithmetic here; the tf32 form of the logits layer has its own test
        options = "tf32=0" if options is None else options + " tf32=0"
    got, info = run_device(device, ir, inputs, options=options)
    if wprec == "single":
        compare(ir, got, want, rtol=1e-5, atol=1e-5, exact=["embed"])
    else:
        compare(ir, got, want, rtol=2e-2, atol=2e-2, exact=["embed"])


@pytest.mark.parametrize("shape", [(2, 256, 256, 256), (1, 200, 136, 200), (3, 128, 512, 64), (1, 384, 48, 1000),
                                   # ragged CTA-pair tiles: the second CTA of the last pair is partly / wholly beyond M,
                                   # a last column tile of 8, a single partial k block
                                   (2, 300, 200, 72), (1, 520, 264, 40)])
@pytest.mark.parametrize("y_prec", ["bfloat16", "single"])
def test_einsum_bias_gelu(device, shape, y_prec):
    """Config 3 shapes (`b|m,k ; b|k,n => b|m,n`, bias, composed GELU) on the tensor-core path,
    including ragged M/N/K that exercise the zero-filled tile edges.  bf16 operands, fp32
    accumulation: rel 2e-2 (outputs) as the tolerance for bf16 contractions."""
    b, m, n, k = shape
    ir = W.einsum_gelu(b, m, n, k, y_prec=y_prec)
    inputs = W.einsum_gelu_inputs(b, m, n, k)
    want = run_oracle(ir, inputs)
    got, info = run_device(device, ir, inputs)
    assert info["stages"][0]["kind"] == "gemm", info
    compare(ir, got, want, rtol=2e-2, atol=2e-3)
    # same routine on the generic path: the two device paths agree with the oracle alike
    got2, info2 = run_device(device, ir, inputs, options="gemm=0")
    assert all(s["kind"] != "gemm" for s in info2["stages"])
    compare(ir, got2, want, rtol=2e-2, atol=2e-3)


@pytest.mark.parametrize("rows", [256, 1000])
def test_mlp_forward_bf16(device, rows):
    """Config 5 forward (784-1024-1024-10, bf16 weights and activations, fp32 accumulation
    and loss) on a shard of `rows` rows."""
    ir = W.mlp_forward(rows=rows)
    x, onehot = W.mlp_inputs(rows=rows)
    inputs = dict(W.mlp_params(), x=x, labels=onehot)
    want = run_oracle(ir, inputs)
    got, info = run_device(device, ir, inputs)
    kinds = [s["kind"] for s in info["stages"]]
    assert kinds[:2] == ["gemm", "gemm"], info
    compare(ir, got, want, rtol=2e-2, atol=2e-3)


@pytest.mark.parametrize("act,options", [("gelu", None), ("relu", "attn=0"), ("gelu", "fuse=0 pairs=0"),
                                         ("gelu", "attn=0 fuse=0 pairs=0")])
def test_decoder_only_forward(device, act, options):
    """Config 4 at reduced width (2 sequences of 128 tokens, 2 layers, 2 heads of 64, d_model 128):
    every stage of the decoder block — batched strided q.k^T and attn.v contractions on the
    tensor-core path, masked softmax, layer norm, residual epilogues — against the cc restatement.
    The reference's own tests pin only shapes for these blocks, so the oracle is the only pin."""
    cfg = dict(batch=2, seq=128, layers=2, d_model=128, heads=2, d_head=64, d_ff=256)
    ir = W.transformer_forward(act=act, **cfg)
    inputs = dict(W.transformer_params(layers=2, d_model=128, heads=2, d_head=64, d_ff=256),
                  **W.transformer_inputs(batch=2, seq=128))
    want = run_oracle(ir, inputs)
    got, info = run_device(device, ir, inputs, options=options)
    kinds = [s["kind"] for s in info["stages"]]
    notes = [s["note"] or "" for s in info["stages"]]
    fused_attention = "attn=0" not in (options or "")
    if "fuse=0" not in (options or ""):   # layer norm (and, apart from the fused attention stage, softmax) chains: one warp-per-row kernel each
        assert sum("one warp per row" in n for n in notes) >= 2 * (2 if fused_attention else 3), notes
    else:
        assert not any("row-fused" in n or "pairs" in n for n in notes), notes
    # q, k, v, q.k^T, attn.v, w_o, ffn, ffn_out per layer; the fused attention stage holds q.k^T and attn.v
    assert kinds.count("attention") == (2 if fused_attention else 0), kinds
    assert kinds.count("gemm") + 2 * kinds.count("attention") >= 2 * 7, kinds
    gemms = [s for s in info["stages"] if s["kind"] == "gemm"]
    if not fused_attention:
        assert any(s["batch"] == 4 and not s["b_kmajor"] for s in gemms)      # attn.v: (b, h) batch, v is n-major
    compare(ir, got, want, rtol=2e-2, atol=2e-2)


def test_moons_large_batch_split_reductions(device):
    """Batch 512: the bias / weight gradient accumulations (reduced loop outermost) run with
    the serial loop split over a 32x32 block; sums are re-associated, hence rel 1e-4 on the
    gradients that add 512 terms."""
    ir = W.moons_train_step(n_batches=2, batch=512)
    x, y = W.moons_inputs(n_points=1024, batch=512)
    inputs = dict(W.moons_params(), moons_flat=x, moons_classes=y)
    statics = [{"i1": 0, "i2": 0}, {"i1": 1, "i2": 1}]
    want = run_oracle(ir, inputs, statics)
    got, info = run_device(device, ir, inputs, statics)
    assert any("split" in s["note"] for s in info["stages"]), info
    compare(ir, got, want, rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("rows,options", [(512, None), (512, "splitk=0 pairs=0"), (1024, None)])
def test_mlp_train_update_and_sgd(device, rows, options):
    """Config 5 (ii) on a 512-row shard: forward, backprop (dW with both operands m/n-major and
    the batch axis contracted, dX with an n-major weight operand, beta = 0 into zeroed
    gradients) and the SGD routine, against the cc restatement."""
    from ocannl_b200 import backend as bk
    ir = W.mlp_train_update(rows=rows)
    x, onehot = W.mlp_inputs(rows=rows)
    inputs = dict(W.mlp_params(), x=x, labels=onehot)
    want = run_oracle(ir, inputs)
    got, info = run_device(device, ir, inputs, options=options)
    gemms = [s for s in info["stages"] if s["kind"] == "gemm"]
    if options is None:       # the weight gradients are few tiles over a long K: split, added with reductions
        assert any("split_k" in s["note"] for s in gemms), [s["note"] for s in gemms]
    else:
        assert not any("split_k" in s["note"] for s in gemms)
    assert len(gemms) >= 6 and any(not s["a_kmajor"] and not s["b_kmajor"] for s in gemms), info
    # Gradients are sums over 512 rows of products of bf16 values.  Upstream activation
    # gradients are themselves ROUNDED to bf16 after an fp32 accumulation whose order differs
    # between the two paths, so a few of them land on the neighbouring bf16 value and the
    # difference is carried into the sums: compare against each gradient's own scale.
    for t in ir.params():
        if t.ident.endswith("_grad") and t.prec == "single":
            scale = float(np.abs(want[t.ident]).max())
            np.testing.assert_allclose(got[t.ident], want[t.ident], rtol=2e-2, atol=5e-2 * scale + 1e-9, err_msg=t.ident)
    compare(ir, got, want, rtol=2e-2, atol=2e-3, only=["h1", "h2", "logits", "loss", "exp_vals"])
    # the optimizer routine on top of the oracle's gradients
    sgd = W.mlp_sgd()
    sin = {k: want[k] for k in [p for p in W.MLP_PARAM_NAMES] + [p + "_grad" for p in W.MLP_PARAM_NAMES]}
    sin["learning_rate"] = np.float32([0.01])
    want2 = run_oracle(sgd, sin)
    got2, _ = run_device(device, sgd, sin)
    compare(sgd, got2, want2, rtol=1e-2, atol=1e-6)


@pytest.mark.parametrize("stride,prec", [(1, "single"), (2, "single"), (1, "bfloat16")])
@pytest.mark.parametrize("options", [None, "coop=0 fuse=0"])
def test_convolution_layer_with_gradients(device, stride, prec, options):
    """Convolution as a contraction over affine positions (`stride * oh + kh`), with a padded
    input node (margins reset by constant loops, the copy shifted by the margin), bias, relu,
    a squared-error loss and the kernel / bias / input gradients.  The input gradient is an
    accumulation whose written position moves with the output and kernel loops: with the
    default options it is spread over threads with atomic adds, with `coop=0` only the batch
    and channel loops are parallel.  fp32 throughout (bf16 nodes: products and sums in float,
    results rounded): accumulation order differs, rel 1e-4 against each node's scale."""
    ir = W.conv2d_update(stride=stride, prec=prec)
    inputs = W.conv2d_inputs(stride=stride, prec=prec)
    want = run_oracle(ir, inputs)
    got, info = run_device(device, ir, inputs, options=options)
    notes = [s["note"] or "" for s in info["stages"]]
    assert any("scatter accumulation" in n for n in notes) == (options is None), notes
    lowp = prec != "single"
    for name in ("x_padded", "y", "loss", "z_grad", "bias_grad", "kernel_grad", "x_padded_grad"):
        w = W.load(prec, want[name]) if want[name].dtype == np.uint16 else want[name]
        g = W.load(prec, got[name]) if got[name].dtype == np.uint16 else got[name]
        scale = float(np.abs(w).max())
        np.testing.assert_allclose(g, w, rtol=2e-2 if lowp else 1e-4, atol=(2e-2 if lowp else 1e-5) * scale, err_msg=name)
    if stride == 1:     # the margins of the padded node hold zeros, the inside the input
        xp = got["x_padded"]
        assert not xp[:, 0].any() and not xp[:, -1].any() and not xp[:, :, 0].any() and not xp[:, :, -1].any()
        assert np.array_equal(xp[:, 1:-1, 1:-1], inputs["x"])


@pytest.mark.parametrize("kwargs", [dict(momentum=0.9, weight_decay=1e-4, nesterov=True), dict(momentum=0.9),
                                    dict(weight_decay=1e-2)])
@pytest.mark.parametrize("options", [None, "fuse=0 pairs=0"])
def test_sgd_with_momentum_and_weight_decay(device, kwargs, options):
    """`Train.sgd_one` (lib/train.ml:76-88) with momentum, Nesterov correction and weight decay on
    the MLP's parameters (bf16) with fp32 gradients, two steps so that the momentum node
    carries state.  Pointwise fp32 / bf16 arithmetic in the reference's order: the fp32 state
    nodes agree to rel 1e-6, the bf16 parameters bit for bit up to one unit in the last place
    where the rounded product lr * delta straddles a rounding boundary."""
    dims = (64, 48, 32, 10)
    ir = W.mlp_sgd(dims=dims, **kwargs)
    g = np.random.default_rng(41)
    inputs = {"learning_rate": np.float32([0.05])}
    for t in ir.params():
        if t.ident.endswith("_grad"):
            inputs[t.ident] = g.standard_normal(t.dims).astype(np.float32)
        elif t.ident.endswith(("_sgd_delta", "_sgd_momentum")):
            inputs[t.ident] = np.zeros(t.dims, np.float32)
        elif t.ident != "learning_rate":
            inputs[t.ident] = W.store("bfloat16", g.standard_normal(t.dims).astype(np.float32))
    want = run_oracle(ir, inputs, statics=({}, {}))
    got, info = run_device(device, ir, inputs, statics=({}, {}), options=options)
    for t in ir.params():
        w, d = want[t.ident], got[t.ident]
        if t.prec == "bfloat16":
            assert np.abs(w.astype(np.int32) - d.astype(np.int32)).max() <= 1, t.ident
            assert (w != d).mean() < 0.01, t.ident
        else:
            np.testing.assert_allclose(d, w, rtol=1e-6, atol=1e-7, err_msg=t.ident)


@pytest.mark.parametrize("options", [None, "fuse=0 pairs=0 coop=0"])
def test_edge_shapes_empty_loops_and_single_elements(device, options):
    """Edge cases of the loop forms: extents of one with fixed indices, odd extents (no pair
    form, ragged last block), a loop that starts past zero, an assignment outside any loop and a
    reduction over a single element.  Integer and fp32 nodes bit for bit, bf16 bit for bit (one
    operation per element)."""
    from ocannl_b200.low_level import Comment, Const, For, Get, Routine, Seq, Set, binop, loops
    r = Routine("edge_shapes")
    a = r.tn("a", "single", [7, 13], read_only=True)
    h = r.tn("h", "bfloat16", [7, 13], read_only=True)
    out = r.tn("out", "single", [7, 13])
    outh = r.tn("outh", "bfloat16", [7, 13])
    untouched = r.tn("untouched", "single", [5])
    one = r.tn("one", "single", [1, 1])
    tail = r.tn("tail", "int32", [9])
    rowsum = r.tn("rowsum", "single", [7])
    i, j, k, l, m, n, p, q = r.syms(8)
    body = [Comment("edge fwd"),
            loops([(j, 7), (k, 13)], Set(out, (j, k), a[j, k] * 2.0 + a[j, 12 - 12])),       # odd extents, a fixed index
            loops([(l, 7), (m, 13)], Set(outh, (l, m), h[l, m] + h[l, 0])),
            Set(one, (0, 0), a[6, 12] - 1.0),                                                 # no loop at all
            For(n, 4, 8, Set(tail, (n,), Const(7.0, "int32"))),                               # starts past zero
            loops([(p, 7)], Set(rowsum, (p,), W.reduce_scope(r, "n_rs", "single", [(q, 1)], lambda: a[p, q], op="add", orig=(p,)))),
            Comment("end")]
    r.body = Seq(body)
    g = np.random.default_rng(51)
    inputs = {"a": g.standard_normal((7, 13)).astype(np.float32),
              "h": W.store("bfloat16", g.standard_normal((7, 13)).astype(np.float32)),
              "untouched": np.full(5, -1.0, np.float32), "tail": np.arange(9, dtype=np.int32)}
    want = run_oracle(r, inputs)
    got, info = run_device(device, r, inputs, options=options)
    for name in ("out", "outh", "untouched", "one", "tail", "rowsum"):
        assert np.array_equal(got[name], want[name]), (name, got[name], want[name])
    assert np.array_equal(got["untouched"], inputs["untouched"]) and got["tail"].tolist() == [0, 1, 2, 3, 7, 7, 7, 7, 7]


def test_routine_without_statements(device):
    """A routine whose body holds only comments compiles to no stages and runs as a no-op; so
    does a loop with `to_ < from_` (device only: the reference's C text compares an unsigned
    counter with the bound, so it has no zero-iteration loops and never emits one)."""
    from ocannl_b200.low_level import Comment, Const, For, Routine, Seq, Set
    r = Routine("nothing_to_do")
    keep = r.tn("keep", "single", [4])
    r.body = Seq([Comment("nothing fwd"), Comment("end")])
    got, info = run_device(device, r, {"keep": np.float32([1, 2, 3, 4])})
    assert info["stages"] == [] and got["keep"].tolist() == [1, 2, 3, 4]
    r = Routine("empty_loop")
    keep = r.tn("keep", "single", [4])
    (i,) = r.syms(1)
    r.body = Seq([Comment("empty fwd"), For(i, 0, -1, Set(keep, (i,), Const(9.0, "single"))), Comment("end")])
    got, info = run_device(device, r, {"keep": np.float32([1, 2, 3, 4])})
    assert got["keep"].tolist() == [1, 2, 3, 4], (got, info)
