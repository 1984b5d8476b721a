"""The fused attention stage against the oracle: the six statements of `multi_head_attention`
(lib/nn_blocks.ml:222-236, softmax of :137-143) run as one kernel must leave in every node the
context holds what the six separate loop nests leave there.

Tolerances.  Scores are sums of 64 products of bf16 values accumulated in fp32 on both sides in a
different order: rel 1e-5 + abs 1e-5 * sqrt(64).  Exponentials and sums inherit the hardware `exp`
(2 ulp) and the summation order: rel 2e-4.  The weights are quotients of two values that were
rounded to bf16 / half first (the cc backend's rule): each operand may land on the other side of a
rounding boundary, which moves the quotient by up to two units in the last place of the format:
rel 2.2 * 2^-7 for bf16 (2.2 * 2^-10 for half).  The output sums up to 256 such weights times values of magnitude ~1:
rel 2e-2 with an absolute part of 2e-2 (the north star's bf16 contraction tolerance)."""
import numpy as np
import pytest

from ocannl_b200 import backend as bk
from tests import routines as R
from tests.parity import compare, run_device, run_oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    return bk.Device(0)


def _check(device, ir, inputs, options=None, expect_fused=True, prec="bfloat16"):
    got, info = run_device(device, ir, inputs, options=options)
    kinds = [s["kind"] for s in info["stages"]]
    assert ("attention" in kinds) == expect_fused, kinds
    want = run_oracle(ir, inputs)
    names = {t.ident for t in ir.params()}
    lowp = 2.0 ** -7 if prec == "bfloat16" else 2.0 ** -10
    for group, rtol, atol in ((["scores"], 1e-5, 8e-5), (["max"], 1e-5, 8e-5), (["exp_vals", "sum_exp"], 2e-4, 1e-30),
                              (["attn"], 2.2 * lowp, 1e-30), (["av"], 2e-2, 2e-2)):
        only = [g for g in group if g in names]
        if only:
            compare(ir, got, want, rtol, atol, only=only)
    return info


@pytest.mark.parametrize("keys", [64, 128, 256])
def test_self_attention_all_nodes_kept(device, keys):
    ir = R.attention(2, 3, keys, keys)
    _check(device, ir, R.attention_inputs(2, 3, keys, keys))


def test_unfused_form_agrees(device):
    ir = R.attention(2, 2, 128, 128)
    _check(device, ir, R.attention_inputs(2, 2, 128, 128), options="attn=0", expect_fused=False)


def test_ragged_queries_and_other_key_count(device):
    # 320 queries: the third tile of 128 holds 64 rows; 128 keys
    ir = R.attention(1, 2, 320, 128)
    _check(device, ir, R.attention_inputs(1, 2, 320, 128))


def test_without_mask_and_half_precision(device):
    ir = R.attention(1, 4, 256, 256, prec="half", mask=False)
    inputs = R.attention_inputs(1, 4, 256, 256, prec="half")
    inputs.pop("mask")
    _check(device, ir, inputs, prec="half")


def test_single_precision_output(device):
    ir = R.attention(1, 1, 128, 64, out_prec="single")
    _check(device, ir, R.attention_inputs(1, 1, 128, 64))


def test_routine_local_rows_are_not_written(device):
    # the intermediate nodes are routine-local and nobody reads them afterwards: only `av` leaves the kernel
    ir = R.attention(2, 4, 256, 256, row_mode="local")
    inputs = R.attention_inputs(2, 4, 256, 256)
    info = _check(device, ir, inputs)
    note = [s["note"] for s in info["stages"] if s["kind"] == "attention"][0]
    assert "0 of the 3 row nodes written" in note
    # and the same routine through the separate stages
    _check(device, ir, inputs, options="attn=0", expect_fused=False)


def test_two_runs_in_a_row_and_graph_replay(device):
    ir = R.attention(2, 2, 256, 256)
    inputs = R.attention_inputs(2, 2, 256, 256)
    want = run_oracle(ir, inputs)
    got, _ = run_device(device, ir, inputs, statics=({}, {}, {}), graph=True)
    compare(ir, got, want, 2e-2, 2e-2, only=["av"])
    compare(ir, got, want, 1e-5, 8e-5, only=["scores"])


def test_operands_off_the_16_byte_grid_fall_back_to_the_separate_stages(device):
    """Under the reference's packing a three-element node ahead of q, k and v leaves them 6 bytes off
    the 16-byte grid: no tensor map can describe them, the statements are planned again without the
    fused stage (and without the tensor-core contractions) at link, and the results do not change."""
    ir = R.attention(1, 2, 128, 128, odd_first=True)
    inputs = R.attention_inputs(1, 2, 128, 128)
    inputs["odd"] = np.zeros(3, np.uint16)
    want = run_oracle(ir, inputs)
    code = bk.Code(ir)
    assert any(s["kind"] == "attention" for s in code.info()["stages"])
    rt = bk.Context(device, packing="reference").link(code)
    assert not any(s["kind"] in ("attention", "gemm") for s in rt.info()["stages"]), rt.info()
    for name, v in inputs.items():
        rt.context.from_host(name, v)
    rt.run()
    device.await_()
    got = {t.ident: rt.context.to_host(t.ident) for t in ir.params()}
    rt.free()
    code.free()
    for p in {p for p, _, _ in rt.context.arrays.values()}:
        device.free_pool(p)
    compare(ir, got, want, 1e-5, 8e-5, only=["scores", "max"])
    compare(ir, got, want, 2e-2, 2e-2, only=["av"])


def test_local_weights_with_a_later_reader_are_written(device):
    """Routine-local intermediate nodes, but one more statement reads the weights after the chain: the
    fused stage must write that node (into the routine's scratch) and only that one."""
    from ocannl_b200.low_level import Set, loops
    ir = R.attention(2, 2, 128, 128, row_mode="local")
    attn = [t for t in ir.tnodes if t.ident == "attn"][0]
    twice = ir.tn("twice", "bfloat16", [2, 128, 2, 128])
    b, s, h, t = ir.syms(4)
    ir.body.items.append(loops([(b, 2), (s, 128), (h, 2), (t, 128)], Set(twice, (b, s, h, t), attn[b, s, h, t] + attn[b, s, h, t])))
    inputs = R.attention_inputs(2, 2, 128, 128)
    got, info = run_device(device, ir, inputs)
    note = [s_["note"] for s_ in info["stages"] if s_["kind"] == "attention"][0]
    assert "1 of the 3 row nodes written" in note
    want = run_oracle(ir, inputs)
    compare(ir, got, want, 2.2 * 2.0 ** -7, 1e-30, only=["twice"])
    compare(ir, got, want, 2e-2, 2e-2, only=["av"])
