"""Host logic of the stage planner, checked without a GPU: `b200_compile` is device independent,
so the plan (which stages exist, what each one is) can be read back from `b200_code_info`."""
from ocannl_b200 import backend as bk
from ocannl_b200 import workloads as W
import pytest


def _plan(ir, options=None):
    code = bk.Code(ir, options)
    try:
        return code.info()["stages"]
    finally:
        code.free()


def test_mlp_forward_plan():
    st = _plan(W.mlp_forward(rows=8192))
    notes = [s["note"] or "" for s in st]
    # three launches: the softmax pieces (row max, exponentials, row sum) and the mean cross-entropy
    # run in the epilogue of the logits contraction, whose 10-wide rows fit one epilogue chunk
    assert [s["kind"] for s in st] == ["gemm", "gemm", "gemm"], notes
    # 8192 x 1024 layers: CTA pairs on 256 x 256 tiles; the 10-wide logits: one CTA per 128 x 16 tile
    assert "CTA pair" in notes[0] and "256x256x64" in notes[0] and "CTA pair" in notes[1]
    assert "128x16x64" in notes[2] and "CTA pair" not in notes[2]
    assert "4 whole-row assignments in the epilogue (the last one a grid-wide sum)" in notes[2]
    # without contraction kernels the same statements are generic stages
    off = _plan(W.mlp_forward(rows=8192), "gemm=0")
    assert all(s["kind"] == "generic" for s in off) and len(off) >= 4


def test_training_plan_split_k_and_dropped_zero_outs():
    st = _plan(W.mlp_train_update(rows=8192))
    notes = [s["note"] or "" for s in st]
    # seven gradient nodes are zeroed by the routine; the two activation gradients are then
    # overwritten completely (beta = 0 contraction, promoted accumulation): their zero_outs go
    assert sum(s["kind"] == "memset" for s in st) == 5, notes
    split = [n for n in notes if "split_k" in n]
    assert len(split) == 2 and all("split_k=4" in n for n in split), notes     # dW1, dW2: 16 pair tiles each
    assert any("outer loop of 10 kept in registers" in n for n in notes), notes  # dW_out
    assert any("slices per output group (atomic adds)" in n for n in notes), notes
    assert any(n.endswith("pairs") for n in notes), notes
    off = [s["note"] or "" for s in _plan(W.mlp_train_update(rows=8192), "splitk=0 pairs=0")]
    assert not any("split_k" in n or n.endswith("pairs") for n in off), off


def test_decoder_plan_fuses_softmax_and_layer_norm():
    small = dict(batch=2, seq=128, layers=2, d_model=128, heads=2, d_head=64, d_ff=256)
    # without the fused attention stage: softmax + 2 layer norms per layer, each a 4-stage warp-per-row kernel
    st = _plan(W.transformer_forward(**small), "attn=0")
    notes = [s["note"] or "" for s in st]
    assert sum("row-fused 4 stages, one warp per row" in n for n in notes) == 2 * 3, notes
    unfused = _plan(W.transformer_forward(**small), "attn=0 fuse=0")
    assert len(unfused) == len(st) + 2 * 3 * 3
    # the (head, d) columns of the q / k / v projections are one contiguous n axis: stored through the staging tile
    code = bk.Code(W.transformer_forward(**small))
    try:
        first_gemm = [i for i, s in enumerate(st) if s["kind"] == "gemm"][0]
        assert "b200_stage[" in code.source(first_gemm)
    finally:
        code.free()


def test_decoder_plan_takes_the_attention_chain_as_one_stage():
    small = dict(batch=2, seq=128, layers=2, d_model=128, heads=2, d_head=64, d_ff=256)
    apart = _plan(W.transformer_forward(**small), "attn=0")
    st = _plan(W.transformer_forward(**small))
    attn = [s for s in st if s["kind"] == "attention"]
    assert len(attn) == 2, [s["kind"] for s in st]
    # scores contraction + softmax kernel + weights . values contraction become one launch per layer;
    # one more stage packs the (read-only) mask to bits, once for both layers
    assert len(st) == len(apart) - 2 * 2 + 1
    assert sum("one bit per element" in s["note"] for s in st) == 1
    assert all("3 of the 3 row nodes written" in s["note"] for s in attn)     # the context holds every node
    # routine-local intermediates that nobody reads are not written, and get no scratch
    local = _plan(W.transformer_forward(attn_nodes="local", **small))
    assert all("0 of the 3 row nodes written" in s["note"] for s in local if s["kind"] == "attention")
    # forms the fused kernel does not cover stay with the separate stages: 96 keys, a head dimension of 32
    assert not any(s["kind"] == "attention" for s in _plan(W.transformer_forward(batch=2, seq=96, layers=1, d_model=128, heads=2, d_head=64, d_ff=256)))
    assert not any(s["kind"] == "attention" for s in _plan(W.transformer_forward(batch=2, seq=128, layers=1, d_model=64, heads=2, d_head=32, d_ff=256)))


def test_random_number_routine_plan():
    from tests.golden.golden_routines import n3_fwd
    st = _plan(n3_fwd("single", 100000, "light"), "fuse=0")
    assert all(s["kind"] == "generic" and s["total"] == 100000 for s in st), st     # every loop parallel, the vector store too


def test_convolution_plan_affine_positions():
    """A convolution layer with its gradients (affine positions `stride * o + k`, a padded node
    written past its margin): no stage is taken for a tensor-core contraction (affine operands
    are not strided tiles), the shifted copy into the padded node runs in parallel, and the
    input gradient, whose written position moves with four serial loops, is spread over threads
    with atomic adds instead of running as 32 threads."""
    st = _plan(W.conv2d_update(stride=1), "fuse=0")
    notes = [s["note"] or "" for s in st]
    assert all(s["kind"] != "gemm" for s in st), notes
    copy = [s for s in st if s["kind"] == "generic" and s["total"] in (4 * 16 * 16 * 8, 4 * 16 * 16 * 4)]
    assert copy, st
    scatter = [s for s in st if "scatter accumulation" in (s["note"] or "")]
    assert len(scatter) == 1 and scatter[0]["total"] == 4 * 16 * 16 * 3 * 3 * 8, notes
    assert any("slices per output group" in n for n in notes), notes      # kernel and bias gradients
    off = [s["note"] or "" for s in _plan(W.conv2d_update(stride=1), "coop=0")]
    assert not any("scatter" in n for n in off), off


def test_momentum_sgd_is_one_launch_per_parameter():
    """delta, momentum, Nesterov correction and the parameter update of one parameter share their
    loops and meet only at one position: a pointwise chain (one kernel, pair form)."""
    st = _plan(W.mlp_sgd(momentum=0.9, weight_decay=1e-4, nesterov=True))
    notes = [s["note"] or "" for s in st]
    assert sum("pointwise chain of 4 stages, pairs" in n for n in notes) == 2, notes   # w1, w2; the small ones share a block
    assert len(st) == 4, notes
    assert len(_plan(W.mlp_sgd(momentum=0.9, weight_decay=1e-4, nesterov=True), "fuse=0")) == 5 * 4


def test_plan_pool_segments_layout():
    """Element-size alignment, in order, a new pool when the cap would be passed
    (arrayjit/lib/backends.ml:22-51)."""
    where, sizes = bk.plan_pool_segments([(20, 2), (8, 4), (6, 2), (100, 4)], cap=64 + 40)
    assert where == [(0, 0), (0, 20), (0, 28), (1, 0)] and sizes == [34, 100]
    where, sizes = bk.plan_pool_segments([(3, 1), (8, 8), (2, 2)])
    assert where == [(0, 0), (0, 8), (0, 16)] and sizes == [18]
    with pytest.raises(bk.UserError, match="per-pool cap"):
        bk.plan_pool_segments([(200, 4)], cap=100)
    assert bk.plan_pool_segments([]) == ([], [])


def test_range_checked_build_wraps_every_node_pointer():
    """`bounds=1`: generic kernels only, each node pointer shadowed by a checked proxy of the node's
    size, the device status word as a last parameter."""
    ir = W.mlp_train_update(rows=64, dims=(32, 64, 64, 10))
    code = bk.Code(ir, "bounds=1")
    try:
        st = code.info()["stages"]
        assert all(s["kind"] in ("generic", "memset") for s in st), st
        src = code.source(-1)
        kernels = src.count('extern "C" __global__')
        assert kernels >= 1 and src.count("unsigned int* b200_status)") == kernels
        assert "const b200_checked<const unsigned short> x = {x__p, 2048ull, b200_status" in src
    finally:
        code.free()


def test_contraction_epilogues_use_the_copy_engine_where_the_layout_allows():
    """Outputs that are regular [batch.., m, n] arrays with 16-byte row strides leave as TMA stores, a
    residual arrives by TMA loads; ten- or 27-column rows (40 / 108 bytes) keep the plain stores."""
    def sources(ir):
        code = bk.Code(ir)
        try:
            return [(s, code.source(i)) for i, s in enumerate(code.info()["stages"]) if s["kind"] == "gemm"]
        finally:
            code.free()

    mlp = sources(W.mlp_forward(rows=8192))
    assert len(mlp) == 3
    assert all("b200_tma_store_4d_nc(b200_omap0" in src for _, src in mlp[:2])          # the two hidden layers
    assert "b200_omap0" not in mlp[2][1]                                                 # logits: rows of 10 floats
    dec = sources(W.transformer_forward(batch=8, layers=1))
    with_residual = [src for _, src in dec if "b200_imap0" in src]
    assert len(with_residual) == 2                                                       # w_o and the second feed-forward contraction
    assert all("b200_tma_load_4d(b200_smem_addr(b200_es.ltile), b200_imap0" in src for src in with_residual)
    assert dec[-1][0]["n"] == 27 and "b200_omap" not in dec[-1][1]                        # the head: rows of 27 floats
    # partial tiles that are added to the output (split-K) do not go through the copy engine
    train = sources(W.mlp_train_update(rows=8192))
    split = [src for s, src in train if "split_k" in s["note"]]
    assert split and all("b200_omap" not in src for src in split)


def test_attention_stage_writes_a_local_node_that_a_later_statement_reads():
    """A routine-local node of the attention chain is left unwritten only when nothing after the chain
    reads it: here the weights are read by one more statement, the scores and exponentials are not."""
    from ocannl_b200.low_level import Set, loops
    ir = W.attention(2, 2, 128, 128, row_mode="local")
    attn = [t for t in ir.tnodes if t.ident == "attn"][0]
    twice = ir.tn("twice", "bfloat16", [2, 128, 2, 128])
    b, s, h, t = ir.syms(4)
    ir.body.items.append(loops([(b, 2), (s, 128), (h, 2), (t, 128)], Set(twice, (b, s, h, t), attn[b, s, h, t] + attn[b, s, h, t])))
    st = _plan(ir)
    notes = [x["note"] for x in st if x["kind"] == "attention"]
    assert notes and "1 of the 3 row nodes written" in notes[0], [x["note"] for x in st]
