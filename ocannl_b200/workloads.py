"""The benchmark configurations as lowered routines plus their seeded synthetic inputs.

No OCaml frontend runs here, so each routine is assembled by hand in the forms the
reference's lowering produces (`Assignments.to_low_level`, arrayjit/lib/assignments.ml:311-488,
followed by inlining and FMA formation, arrayjit/lib/low_level.ml:750-1150,1631-1634):

  * a contraction read once by a pointwise consumer is a virtual accumulator inside the
    consumer's assignment (`v := 0; for k { v := fma(a, b, v) }`);
  * anything read more than once per position, every parameter gradient and every routine
    output is a materialised node updated in place;
  * loop order is the LHS axes (batch, output, input) followed by the contracted axes, and
    back-propagation keeps the forward loop order.

Models follow lib/nn_blocks.ml (`mlp` :119-126 — hidden layers `relu(w*x + b)`, linear output
without bias; `softmax` :137-143) and the training programs test/training/moons_demo.ml:42-59
and test/training/mlp_names.ml:153-168.  Inputs are seeded numpy (PCG64) draws with the
shapes and value ranges of the reference's datasets, which are not available offline.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Sequence, Tuple

import numpy as np

from .low_level import (Affine, Comment, Const, EmbedIndex, For, Get, GetDynamic, GetLocal, LocalScope, Routine, Scalar, Seq,
                        Set, SetLocal, Tnode, Unop, ZeroOut, binop, fma, loops, un, where)

NEG_INF = float("-inf")


# ------------------------------------------------------------------ bf16 helpers (host side)
def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even on the bit pattern (arrayjit/lib/builtins.c:620-627)."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return ((u >> 16) & 0xFFFF).astype(np.uint16)


def bf16_bits_to_f32(h: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(h, np.uint16).astype(np.uint32) << 16).view(np.float32)


def store(prec: str, a: np.ndarray) -> np.ndarray:
    """Host array in the storage type of `prec`."""
    if prec == "bfloat16":
        return f32_to_bf16_bits(a)
    if prec == "half":
        return np.asarray(a, np.float16)
    return np.asarray(a, {"single": np.float32, "double": np.float64}[prec])


def load(prec: str, a: np.ndarray) -> np.ndarray:
    """Host array of storage type `prec` as float32/float64 values."""
    if prec == "bfloat16":
        return bf16_bits_to_f32(a)
    if prec == "half":
        return np.asarray(a, np.float32)
    return a


# ------------------------------------------------------------------ lowering helpers
def reduce_scope(r: Routine, name: str, prec: str, red: Sequence[Tuple[str, int]], term: Callable[[], Scalar],
                 op: str = "fma", orig=()) -> LocalScope:
    """`v { v := neutral; for k.. { v := op(v, term) } }` — the inlined form of a virtual
    accumulation (golden: test/einsum/inline_permuted_view-c_fwd.ll.expected)."""
    vt = r.tn(name, prec, [1], mode="virtual")
    sid = r.scope(vt)
    if op == "fma":
        a, b = term()
        step = SetLocal(sid, fma(a, b, GetLocal(sid)))
        init = 0.0
    elif op == "add":
        step = SetLocal(sid, binop("add", GetLocal(sid), term()))
        init = 0.0
    elif op == "max":
        step = SetLocal(sid, binop("max", GetLocal(sid), term()))
        init = NEG_INF
    else:
        raise ValueError(op)
    body = Seq([SetLocal(sid, Const(init, prec)), loops(red, step)])
    return LocalScope(sid, body, tuple(orig))


def gelu_tanh(z: Scalar) -> Scalar:
    """0.5*z*(1 + tanh(0.7978845608*(z + 0.044715*z^3))) composed from the reference's
    primitives (`*.`, `+`, `**.`, `tanh`); GELU itself is not a reference op."""
    z3 = binop("pow", z, 3.0)
    inner = 0.7978845608 * (z + 0.044715 * z3)
    return (0.5 * z) * (1.0 + un("tanh", inner))


# ------------------------------------------------------------------ config 1: half-moons MLP, train step
def moons_inputs(n_points=1024, batch=20, seed=1):
    """Two interleaved unit half-circles with N(0, 0.1) noise per coordinate; labels +1 / -1.
    The upper one is (cos t, sin t); the lower one is the mirrored half-circle moved to
    (1 - cos t, 0.5 - sin t), i.e. centred one unit to the right and half a unit below the
    first one's top.  Angles are uniform on [0, pi]; points are shuffled, then viewed as
    [n_batches, batch, 2]."""
    rng = np.random.default_rng(seed)
    half = n_points // 2
    t = rng.uniform(0.0, math.pi, n_points)
    x = np.empty((n_points, 2), np.float32)
    y = np.empty((n_points, 1), np.float32)
    x[:half, 0] = np.cos(t[:half]); x[:half, 1] = np.sin(t[:half]); y[:half] = 1.0
    x[half:, 0] = 1.0 - np.cos(t[half:]); x[half:, 1] = 0.5 - np.sin(t[half:]); y[half:] = -1.0
    x += rng.normal(0.0, 0.1, x.shape).astype(np.float32)
    perm = rng.permutation(n_points)
    x, y = x[perm], y[perm]
    nb = n_points // batch
    return (np.ascontiguousarray(x[:nb * batch].reshape(nb, batch, 2)),
            np.ascontiguousarray(y[:nb * batch].reshape(nb, batch, 1)))


def moons_params(seed=2, hid=16):
    rng = np.random.default_rng(seed)
    u = lambda *s: rng.uniform(-1.0, 1.0, s).astype(np.float32)
    return {"w1": u(hid, 2), "b1": u(hid), "w2": u(hid, hid), "b2": u(hid), "w3": u(1, hid)}


def moons_train_step(n_batches=51, batch=20, hid=16, steps=4080, weight_decay=1e-4) -> Routine:
    """One routine = forward + zero grads + backprop + SGD (`Asgns.sequence [update; sgd]`,
    test/training/moons_demo.ml:63-72; lib/train.ml:61-90) of the 2->16->16->1 ReLU MLP with
    the hinge loss relu(1 - y*mlp(x)) averaged over the batch."""
    r = Routine("moons_sgd_step")
    i_batch = r.static_sym(n_batches)
    i_step = r.static_sym(None)
    B, H = batch, hid
    flat = r.tn("moons_flat", "single", [n_batches, B, 2], read_only=True)
    cls = r.tn("moons_classes", "single", [n_batches, B, 1], read_only=True)
    w1, b1 = r.tn("w1", "single", [H, 2]), r.tn("b1", "single", [H])
    w2, b2 = r.tn("w2", "single", [H, H]), r.tn("b2", "single", [H])
    w3 = r.tn("w3", "single", [1, H])
    h1, h2 = r.tn("h1", "single", [B, H]), r.tn("h2", "single", [B, H])
    margin = r.tn("margin_loss", "single", [B, 1])
    loss = r.tn("scalar_loss", "single", [1])
    lr = r.tn("learning_rate", "single", [1])
    grads = {p.ident: r.tn(p.ident + "_grad", "single", p.dims) for p in (w1, b1, w2, b2, w3)}
    loc = lambda n, d: r.tn(n, "single", d, mode="local", zero_init=True)
    g_margin, g_f = loc("margin_loss_grad", [B, 1]), loc("mlp_grad", [B, 1])
    g_h2, g_z2, g_h1, g_z1 = loc("h2_grad", [B, H]), loc("z2_grad", [B, H]), loc("h1_grad", [B, H]), loc("z1_grad", [B, H])
    g_loss = loc("scalar_loss_grad", [1])
    body: List = [Comment("scalar_loss forward and gradient update")]
    # ---- forward
    b, o, i = r.syms(3)
    body.append(loops([(b, B), (o, H)], Set(h1, (b, o), un("relu", b1[o] + reduce_scope(
        r, "n_w1x", "single", [(i, 2)], lambda: (w1[o, i], flat[i_batch, b, i]), orig=(b, o))))))
    b, o, i = r.syms(3)
    body.append(loops([(b, B), (o, H)], Set(h2, (b, o), un("relu", b2[o] + reduce_scope(
        r, "n_w2h", "single", [(i, H)], lambda: (w2[o, i], h1[b, i]), orig=(b, o))))))
    b, i = r.syms(2)
    body.append(loops([(b, B)], Set(margin, (b, 0), un("relu", 1.0 - cls[i_batch, b, 0] * reduce_scope(
        r, "mlp_out", "single", [(i, H)], lambda: (w3[0, i], h2[b, i]), orig=(b, 0))))))
    b = r.sym()
    body.append(Set(loss, (0,), reduce_scope(r, "n_sum", "single", [(b, B)], lambda: margin[b, 0], op="add") / float(B)))
    # ---- zero grads and backprop
    body.append(Comment("zero grads and backprop"))
    for g in list(grads.values()) + [g_margin, g_f, g_h2, g_z2, g_h1, g_z1, g_loss]:
        body.append(ZeroOut(g))
    body.append(Set(g_loss, (0,), Const(1.0)))
    b = r.sym()
    body.append(loops([(b, B)], Set(g_margin, (b, 0), g_margin[b, 0] + g_loss[0] / float(B))))
    b = r.sym()
    body.append(loops([(b, B)], Set(g_f, (b, 0), g_f[b, 0] - cls[i_batch, b, 0] * binop(
        "relu_gate", margin[b, 0], g_margin[b, 0]))))
    b, i = r.syms(2)
    body.append(loops([(b, B), (i, H)], Set(grads["w3"], (0, i), fma(g_f[b, 0], h2[b, i], grads["w3"][0, i]))))
    b, i = r.syms(2)
    body.append(loops([(b, B), (i, H)], Set(g_h2, (b, i), fma(w3[0, i], g_f[b, 0], g_h2[b, i]))))

    def layer_backward(g_h, h, g_z, w, gw, gb, x_get, g_x, in_dim):
        bb, oo = r.syms(2)
        body.append(loops([(bb, B), (oo, H)], Set(g_z, (bb, oo), g_z[bb, oo] + binop("relu_gate", h[bb, oo], g_h[bb, oo]))))
        bb, oo = r.syms(2)
        body.append(loops([(bb, B), (oo, H)], Set(gb, (oo,), gb[oo] + g_z[bb, oo])))
        bb, oo, ii = r.syms(3)
        body.append(loops([(bb, B), (oo, H), (ii, in_dim)],
                          Set(gw, (oo, ii), fma(g_z[bb, oo], x_get(bb, ii), gw[oo, ii]))))
        if g_x is not None:
            bb, oo, ii = r.syms(3)
            body.append(loops([(bb, B), (oo, H), (ii, in_dim)],
                              Set(g_x, (bb, ii), fma(w[oo, ii], g_z[bb, oo], g_x[bb, ii]))))

    layer_backward(g_h2, h2, g_z2, w2, grads["w2"], grads["b2"], lambda bb, ii: h1[bb, ii], g_h1, H)
    layer_backward(g_h1, h1, g_z1, w1, grads["w1"], grads["b1"], lambda bb, ii: flat[i_batch, bb, ii], None, 2)
    # ---- sgd_update with weight decay; the learning rate decays linearly with step_n
    body.append(Comment("sgd_update"))
    body.append(Set(lr, (0,), (0.1 * ((2.0 * steps) - Scalar_from_index(i_step))) / float(steps)))
    for p in (w1, b1, w2, b2, w3):
        syms = r.syms(len(p.dims))
        idx = tuple(0 if d == 1 else s for s, d in zip(syms, p.dims))
        nest = [(s, d) for s, d in zip(syms, p.dims) if d != 1]
        upd = Get(p, idx) - lr[0] * fma(Const(weight_decay), Get(p, idx), Get(grads[p.ident], idx))
        body.append(loops(nest, Set(p, idx, upd)))
    body.append(Comment("end"))
    r.body = Seq(body)
    return r


def Scalar_from_index(sym: str) -> Scalar:
    """`!@step_n`: the static index embedded as a number."""
    return EmbedIndex(sym)


def moons_step_numpy(P: Dict[str, np.ndarray], x: np.ndarray, y: np.ndarray, step: int, steps=4080, wd=1e-4):
    """Float64 numpy statement of the same training step, used as an independent
    cross-check of the hand-lowered routine (not as the parity oracle)."""
    P = {k: v.astype(np.float64) for k, v in P.items()}
    B = x.shape[0]
    z1 = x @ P["w1"].T + P["b1"]; h1 = np.maximum(z1, 0)
    z2 = h1 @ P["w2"].T + P["b2"]; h2 = np.maximum(z2, 0)
    f = h2 @ P["w3"].T
    m = np.maximum(1 - y * f, 0)
    loss = m.sum() / B
    gf = -(y * (m > 0)) / B
    g = {"w3": gf.T @ h2}
    gz2 = (gf @ P["w3"]) * (h2 > 0)
    g["b2"] = gz2.sum(0); g["w2"] = gz2.T @ h1
    gz1 = (gz2 @ P["w2"]) * (h1 > 0)
    g["b1"] = gz1.sum(0); g["w1"] = gz1.T @ x
    lr = 0.1 * (2 * steps - step) / steps
    new = {k: P[k] - lr * (wd * P[k] + g[k]) for k in P}
    return new, loss


# ------------------------------------------------------------------ config 2: makemore char MLP forward
def makemore_inputs(batch=4096, block=3, vocab=27, seed=3, target_seed=5):
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, vocab, (batch, block)).astype(np.float32)
    tg = np.random.default_rng(target_seed).integers(0, vocab, batch)
    onehot = np.zeros((batch, vocab), np.float32)
    onehot[np.arange(batch), tg] = 1.0
    return ids, onehot


def makemore_params(vocab=27, block=3, embed=10, hid=200, seed=4):
    rng = np.random.default_rng(seed)
    n = lambda fan_in, *s: (rng.normal(0.0, 1.0, s) / math.sqrt(fan_in)).astype(np.float32)
    return {"c": n(vocab, embed, vocab), "w1": n(block * embed, hid, block, embed), "b1": n(block * embed, hid),
            "w2": n(hid, vocab, hid), "b2": n(hid, vocab)}


def makemore_forward(batch=4096, block=3, vocab=27, embed=10, hid=200, wprec="single") -> Routine:
    """Inference forward of the character MLP of test/training/mlp_names.ml:153-168:
    embedding gather (the one-hot contraction rewritten by `rewrite_one_hot_reductions`,
    arrayjit/lib/low_level.ml:2158-2329) -> tanh(sum_{s,e} emb*w1 + b1) -> logits ->
    max-subtracted log-softmax cross-entropy against one-hot targets, mean over the batch."""
    r = Routine("makemore_fwd_" + wprec)
    B = batch
    ids = r.tn("input_batch", "single", [B, block], read_only=True)
    tgt = r.tn("target_batch", "single", [B, vocab], read_only=True)
    c = r.tn("c", wprec, [embed, vocab], read_only=True)
    w1 = r.tn("w1", wprec, [hid, block, embed], read_only=True)
    b1 = r.tn("b1", wprec, [hid], read_only=True)
    w2 = r.tn("w2", wprec, [vocab, hid], read_only=True)
    b2 = r.tn("b2", wprec, [vocab], read_only=True)
    emb = r.tn("embed", wprec, [B, block, embed])
    hidden = r.tn("hidden", wprec, [B, hid])
    logits = r.tn("logits", "single", [B, vocab])
    max_l = r.tn("max_l", "single", [B, 1])
    shifted = r.tn("shifted", "single", [B, vocab])
    lse = r.tn("lse", "single", [B, 1])
    nll = r.tn("nll", "single", [1])
    batch_loss = r.tn("batch_loss", "single", [1])
    body: List = [Comment("batch_loss fwd")]
    # gather: where(-1 < id && id < vocab && id == trunc(id), c[e, (uint32)id], 0), guard in double
    b, s, e = r.syms(3)
    idv = lambda: Get(ids, (b, s))
    D = "double"
    lower = binop("lt", Const(-1.0, D), _as(idv(), D))
    upper = binop("lt", _as(idv(), D), Const(float(vocab), D))
    integral = binop("eq", _as(idv(), D), Unop("trunc", _as(idv(), D), D))
    guard = _force(binop("and", _force(binop("and", _force(lower, D), _force(upper, D)), D), _force(integral, D)), D)
    gather = GetDynamic(c, (e, 0), 1, idv())
    body.append(loops([(b, B), (s, block), (e, embed)], Set(emb, (b, s, e), where(guard, gather, Const(0.0, wprec)))))
    # hidden = tanh(sum_{s,e} emb*w1 + b1); contraction accumulates in single
    b, h, s, e = r.syms(4)
    body.append(loops([(b, B), (h, hid)], Set(hidden, (b, h), un("tanh", reduce_scope(
        r, "n_hid", "single", [(s, block), (e, embed)], lambda: (emb[b, s, e], w1[h, s, e]), orig=(b, h)) + b1[h]))))
    b, v, h = r.syms(3)
    body.append(loops([(b, B), (v, vocab)], Set(logits, (b, v), reduce_scope(
        r, "n_logit", "single", [(h, hid)], lambda: (w2[v, h], hidden[b, h]), orig=(b, v)) + b2[v])))
    b, v = r.syms(2)
    body.append(loops([(b, B)], Set(max_l, (b, 0), reduce_scope(
        r, "n_max", "single", [(v, vocab)], lambda: logits[b, v], op="max"))))
    b, v = r.syms(2)
    body.append(loops([(b, B), (v, vocab)], Set(shifted, (b, v), logits[b, v] - max_l[b, 0])))
    b, v = r.syms(2)
    body.append(loops([(b, B)], Set(lse, (b, 0), un("log", reduce_scope(
        r, "n_sumexp", "single", [(v, vocab)], lambda: un("exp", shifted[b, v]), op="add")))))
    b, v = r.syms(2)
    body.append(Set(nll, (0,), un("neg", reduce_scope(
        r, "n_nll", "single", [(b, B), (v, vocab)], lambda: tgt[b, v] * (shifted[b, v] - lse[b, 0]), op="add"))))
    body.append(Set(batch_loss, (0,), nll[0] / float(B)))
    body.append(Comment("end"))
    r.body = Seq(body)
    return r


def _as(s: Scalar, prec: str) -> Scalar:
    return s


def _force(s: Scalar, prec: str) -> Scalar:
    """Pins the argument precision recorded for a heterogeneous consumer (the guard of
    `build_guarded_gather` is typed double throughout, low_level.ml:2193-2215)."""
    s.prec = prec
    return s


def makemore_forward_numpy(P, ids, onehot):
    P = {k: v.astype(np.float64) for k, v in P.items()}
    idx = ids.astype(np.int64)
    emb = np.transpose(P["c"][:, idx], (1, 2, 0))                 # [B, block, embed]
    hidden = np.tanh(np.einsum("bse,hse->bh", emb, P["w1"]) + P["b1"])
    logits = hidden @ P["w2"].T + P["b2"]
    sh = logits - logits.max(1, keepdims=True)
    lse = np.log(np.exp(sh).sum(1, keepdims=True))
    return -(onehot * (sh - lse)).sum() / ids.shape[0], logits


# ------------------------------------------------------------------ config 3: batched einsum + bias + GELU
def einsum_gelu(batch=8, M=1024, N=1024, K=1024, in_prec="bfloat16", y_prec="bfloat16") -> Routine:
    """`b|m,k ; b|k,n => b|m,n` through `+*`, bias add and a composed tanh-GELU.  The
    contraction result is read once (by the bias add) so it is a virtual fp32 accumulator
    inside `z`'s assignment; `z` is read three times by the GELU chain and is therefore
    materialised (fp32), `y` is the routine output."""
    r = Routine("einsum_gelu_%dx%dx%dx%d" % (batch, M, N, K))
    a = r.tn("a", in_prec, [batch, M, K], read_only=True)
    bm = r.tn("b", in_prec, [batch, K, N], read_only=True)
    bias = r.tn("bias", "single", [N], read_only=True)
    z = r.tn("z", "single", [batch, M, N])
    y = r.tn("y", y_prec, [batch, M, N])
    ib, im, in_, ik = r.syms(4)
    s1 = loops([(ib, batch), (im, M), (in_, N)], Set(z, (ib, im, in_), reduce_scope(
        r, "n_ab", "single", [(ik, K)], lambda: (a[ib, im, ik], bm[ib, ik, in_]), orig=(ib, im, in_)) + bias[in_]))
    jb, jm, jn = r.syms(3)
    s2 = loops([(jb, batch), (jm, M), (jn, N)], Set(y, (jb, jm, jn), gelu_tanh(z[jb, jm, jn])))
    r.body = Seq([Comment("y fwd"), s1, s2, Comment("end")])
    return r


def einsum_gelu_inputs(batch, M, N, K, in_prec="bfloat16"):
    a = np.random.default_rng(6).standard_normal((batch, M, K), np.float32)
    b = np.random.default_rng(7).standard_normal((batch, K, N), np.float32)
    bias = np.random.default_rng(8).standard_normal(N).astype(np.float32)
    return {"a": store(in_prec, a), "b": store(in_prec, b), "bias": bias}


# ------------------------------------------------------------------ config 5: data-parallel MLP 784-1024-1024-10
def mlp_params(dims=(784, 1024, 1024, 10), seed=22, wprec="bfloat16"):
    """U(-1,1)*sqrt(6/(fan_in+fan_out)) weights, the same on every shard; hidden-layer biases."""
    rng = np.random.default_rng(seed)
    P = {}
    n_layers = len(dims) - 1
    for l in range(n_layers):
        fi, fo = dims[l], dims[l + 1]
        name = "w_out" if l == n_layers - 1 else "w%d" % (l + 1)
        P[name] = store(wprec, (rng.uniform(-1, 1, (fo, fi)) * math.sqrt(6.0 / (fi + fo))).astype(np.float32))
        if l < n_layers - 1:
            P["b%d" % (l + 1)] = store(wprec, (rng.uniform(-1, 1, fo) * math.sqrt(6.0 / (fi + fo))).astype(np.float32))
    return P


def mlp_inputs(rows=8192, in_dim=784, classes=10, seed=20, label_seed=21, xprec="bfloat16"):
    x = np.random.default_rng(seed).standard_normal((rows, in_dim), np.float32)
    lab = np.random.default_rng(label_seed).integers(0, classes, rows)
    onehot = np.zeros((rows, classes), np.float32)
    onehot[np.arange(rows), lab] = 1.0
    return store(xprec, x), onehot


def mlp_forward(rows=8192, dims=(784, 1024, 1024, 10), wprec="bfloat16", with_loss=True) -> Routine:
    """Forward of `Nn_blocks.mlp` (lib/nn_blocks.ml:108,119-126: hidden `relu(w*x + b)`, linear
    output without bias) with bf16 weights/activations and fp32 accumulation, followed by the
    softmax cross-entropy mean loss of lib/nn_blocks.ml:137-143 against one-hot labels."""
    r = Routine("mlp_fwd_%d" % rows)
    x = r.tn("x", wprec, [rows, dims[0]], read_only=True)
    labels = r.tn("labels", "single", [rows, dims[-1]], read_only=True)
    n_layers = len(dims) - 1
    body: List = [Comment("mlp fwd")]
    h = x
    for l in range(n_layers):
        fi, fo = dims[l], dims[l + 1]
        last = l == n_layers - 1
        w = r.tn("w_out" if last else "w%d" % (l + 1), wprec, [fo, fi], read_only=True)
        ib, io, ii = r.syms(3)
        hin = h
        acc = lambda: reduce_scope(r, "n_mm%d" % l, "single", [(ii, fi)], lambda: (w[io, ii], hin[ib, ii]), orig=(ib, io))
        if last:
            out = r.tn("logits", "single", [rows, fo])
            body.append(loops([(ib, rows), (io, fo)], Set(out, (ib, io), acc())))
        else:
            b = r.tn("b%d" % (l + 1), wprec, [fo], read_only=True)
            out = r.tn("h%d" % (l + 1), wprec, [rows, fo])
            body.append(loops([(ib, rows), (io, fo)], Set(out, (ib, io), un("relu", acc() + b[io]))))
        h = out
    if with_loss:
        C = dims[-1]
        logits = h
        max_l = r.tn("max_l", "single", [rows, 1])
        expv = r.tn("exp_vals", "single", [rows, C])
        ssum = r.tn("sum_exp", "single", [rows, 1])
        loss = r.tn("loss", "single", [1])
        ib, ic = r.syms(2)
        body.append(loops([(ib, rows)], Set(max_l, (ib, 0), reduce_scope(
            r, "n_max", "single", [(ic, C)], lambda: logits[ib, ic], op="max"))))
        ib, ic = r.syms(2)
        body.append(loops([(ib, rows), (ic, C)], Set(expv, (ib, ic), un("exp", logits[ib, ic] - max_l[ib, 0]))))
        ib, ic = r.syms(2)
        body.append(loops([(ib, rows)], Set(ssum, (ib, 0), reduce_scope(
            r, "n_sum", "single", [(ic, C)], lambda: expv[ib, ic], op="add"))))
        ib, ic = r.syms(2)
        body.append(Set(loss, (0,), un("neg", reduce_scope(
            r, "n_ce", "single", [(ib, rows), (ic, C)],
            lambda: labels[ib, ic] * un("log", expv[ib, ic] / ssum[ib, 0]), op="add")) / float(rows)))
    body.append(Comment("end"))
    r.body = Seq(body)
    return r


# ------------------------------------------------------------------ data-parallel regression step
def linreg_update(batch: int) -> Routine:
    """`Train.grad_update` of the sum-over-batch squared error ((w *. x) - y)^2 of
    test/training/data_parallel.ml:44-51: forward, zero grads, backprop.  `w` has one element."""
    r = Routine("linreg_update_%d" % batch)
    x = r.tn("x", "single", [batch, 1], read_only=True)
    y = r.tn("y", "single", [batch, 1], read_only=True)
    w = r.tn("w", "single", [1])
    g = r.tn("w_grad", "single", [1])
    loss = r.tn("loss", "single", [1])
    b = r.sym()
    diff = lambda bb: (w[0] * x[bb, 0]) - y[bb, 0]
    fwd = Set(loss, (0,), reduce_scope(r, "n_sq", "single", [(b, batch)], lambda: diff(b) * diff(b), op="add"))
    b2 = r.sym()
    bwd = loops([(b2, batch)], Set(g, (0,), g[0] + ((diff(b2) * x[b2, 0]) + (diff(b2) * x[b2, 0]))))
    r.body = Seq([Comment("loss forward and gradient update"), fwd, ZeroOut(g), bwd, Comment("end")])
    return r


def linreg_sgd() -> Routine:
    """`Train.sgd_update` without momentum or weight decay (lib/train.ml:76-90): w =- lr * w.grad."""
    r = Routine("linreg_sgd")
    w = r.tn("w", "single", [1])
    g = r.tn("w_grad", "single", [1], read_only=True)
    lr = r.tn("learning_rate", "single", [1], read_only=True)
    r.body = Seq([Comment("w param sgd step"), Set(w, (0,), w[0] - lr[0] * g[0]), Comment("end")])
    return r


# ------------------------------------------------------------------ config 4: decoder-only transformer forward
def transformer_params(layers=6, d_model=512, heads=8, d_head=64, d_ff=2048, vocab=27, seed=10, wprec="bfloat16"):
    """Xavier-normal weights (sigma = sqrt(2/(fan_in+fan_out))), gamma = 1, beta = 0, zero biases
    except the FFN bias which is drawn like the weights."""
    rng = np.random.default_rng(seed)

    def xavier(shape, fan_in, fan_out):
        return store(wprec, (rng.standard_normal(shape) * math.sqrt(2.0 / (fan_in + fan_out))).astype(np.float32))

    P = {"tok_embed": xavier((d_model, vocab), vocab, d_model), "pos": xavier((d_model,), 1, d_model),
         "w_head": xavier((vocab, d_model), d_model, vocab)}
    for l in range(layers):
        p = "l%d_" % l
        for n in ("w_q", "w_k", "w_v"):
            P[p + n] = xavier((heads, d_head, d_model), d_model, heads * d_head)
        P[p + "w_o"] = xavier((d_model, heads, d_head), heads * d_head, d_model)
        P[p + "ffn_w"] = xavier((d_ff, d_model), d_model, d_ff)
        P[p + "ffn_b"] = xavier((d_ff,), d_model, d_ff)
        P[p + "ffn_w_out"] = xavier((d_model, d_ff), d_ff, d_model)
        for ln in ("ln1_", "ln2_"):
            P[p + ln + "gamma"] = np.ones(d_model, np.float32)
            P[p + ln + "beta"] = np.zeros(d_model, np.float32)
    return P


def transformer_inputs(batch=64, seq=256, vocab=27, seed=9):
    tok = np.random.default_rng(seed).integers(0, vocab, (batch, seq))
    onehot = np.zeros((batch, seq, vocab), np.float32)
    onehot[np.arange(batch)[:, None], np.arange(seq)[None, :], tok] = 1.0
    mask = (np.arange(seq)[:, None] >= np.arange(seq)[None, :]).astype(np.float32)   # s >= t
    return {"tokens": store("bfloat16", onehot), "mask": mask}


def transformer_forward(batch=64, seq=256, layers=6, d_model=512, heads=8, d_head=64, d_ff=2048, vocab=27,
                        wprec="bfloat16", act="gelu", eps=1e-5, attn_nodes="ctx") -> Routine:
    """Forward of `Nn_blocks.decoder_only` (lib/nn_blocks.ml:274-296): per layer masked
    multi-head attention (:209-236: q/k/v projections, scores `s | h d ; t | h d => s | t -> h`
    scaled by 1/sqrt(d), `where mask scores -1e9`, softmax over t as in :137-143, `attn +* v`,
    `w_o`), residual, layer_norm as written in :251-258 (`(x - sum_d x) / d`, summed squares),
    FFN (`mlp` with one hidden layer, :119-126), residual, layer_norm; then a linear head.
    bf16 weights and activations, fp32 accumulators, fp32 softmax and layer-norm statistics.
    `attn_nodes` is the memory class of the attention chain's intermediate nodes (scores, max,
    exponentials, sum, weights): "ctx" when the context holds them, "local" when they are
    routine-local (the class `C_syntax.compile_proc` gives a node that one routine alone uses)."""
    r = Routine("decoder_fwd_b%d_s%d_l%d" % (batch, seq, layers))
    AM = attn_nodes
    B, S, D, H, E, F, V = batch, seq, d_model, heads, d_head, d_ff, vocab
    P = wprec
    tokens = r.tn("tokens", P, [B, S, V], read_only=True)
    mask = r.tn("mask", "single", [S, S], read_only=True)
    tok_embed = r.tn("tok_embed", P, [D, V], read_only=True)
    pos = r.tn("pos", P, [D], read_only=True)
    body: List = [Comment("logits fwd")]
    x = r.tn("x0", P, [B, S, D])
    b, s, d, v = r.syms(4)
    body.append(loops([(b, B), (s, S), (d, D)], Set(x, (b, s, d), reduce_scope(
        r, "n_emb", "single", [(v, V)], lambda: (tok_embed[d, v], tokens[b, s, v]), orig=(b, s, d)) + pos[d])))

    def layer_norm(pref, src, out):
        ssum = r.tn(pref + "sum", "single", [B, S, 1])
        cen = r.tn(pref + "centered", "single", [B, S, D])
        std = r.tn(pref + "std", "single", [B, S, 1])
        gamma = r.tn(pref + "gamma", "single", [D], read_only=True)
        beta = r.tn(pref + "beta", "single", [D], read_only=True)
        bb, ss, dd = r.syms(3)
        body.append(loops([(bb, B), (ss, S)], Set(ssum, (bb, ss, 0), reduce_scope(
            r, pref + "n_sum", "single", [(dd, D)], lambda: src[bb, ss, dd], op="add"))))
        bb, ss, dd = r.syms(3)
        body.append(loops([(bb, B), (ss, S), (dd, D)], Set(cen, (bb, ss, dd), (src[bb, ss, dd] - ssum[bb, ss, 0]) / float(D))))
        bb, ss, dd = r.syms(3)
        body.append(loops([(bb, B), (ss, S)], Set(std, (bb, ss, 0), un("sqrt", reduce_scope(
            r, pref + "n_var", "single", [(dd, D)], lambda: cen[bb, ss, dd] * cen[bb, ss, dd], op="add") + eps))))
        bb, ss, dd = r.syms(3)
        body.append(loops([(bb, B), (ss, S), (dd, D)], Set(out, (bb, ss, dd),
                                                            (gamma[dd] * (cen[bb, ss, dd] / std[bb, ss, 0])) + beta[dd])))

    for l in range(layers):
        p = "l%d_" % l
        wq, wk, wv = (r.tn(p + n, P, [H, E, D], read_only=True) for n in ("w_q", "w_k", "w_v"))
        wo = r.tn(p + "w_o", P, [D, H, E], read_only=True)
        q, k, vv = (r.tn(p + n, P, [B, S, H, E]) for n in ("q", "k", "v"))
        for w, out in ((wq, q), (wk, k), (wv, vv)):
            b, s, h, e, i = r.syms(5)
            xin = x
            body.append(loops([(b, B), (s, S), (h, H), (e, E)], Set(out, (b, s, h, e), reduce_scope(
                r, out.ident + "_mm", "single", [(i, D)], lambda: (w[h, e, i], xin[b, s, i]), orig=(b, s, h, e)))))
        scores = r.tn(p + "scores", "single", [B, S, H, S], mode=AM)
        b, s, h, t, e = r.syms(5)
        body.append(loops([(b, B), (s, S), (h, H), (t, S)], Set(scores, (b, s, h, t), where(
            mask[s, t],
            reduce_scope(r, p + "qk", "single", [(e, E)], lambda: (q[b, s, h, e], k[b, t, h, e]), orig=(b, s, h, t))
            / math.sqrt(E), Const(-1e9)))))
        mx = r.tn(p + "max", "single", [B, S, H, 1], mode=AM)
        b, s, h, t = r.syms(4)
        body.append(loops([(b, B), (s, S), (h, H)], Set(mx, (b, s, h, 0), reduce_scope(
            r, p + "n_max", "single", [(t, S)], lambda: scores[b, s, h, t], op="max"))))
        ex = r.tn(p + "exp_vals", "single", [B, S, H, S], mode=AM)
        b, s, h, t = r.syms(4)
        body.append(loops([(b, B), (s, S), (h, H), (t, S)], Set(ex, (b, s, h, t), un("exp", scores[b, s, h, t] - mx[b, s, h, 0]))))
        sm = r.tn(p + "sum_exp", "single", [B, S, H, 1], mode=AM)
        b, s, h, t = r.syms(4)
        body.append(loops([(b, B), (s, S), (h, H)], Set(sm, (b, s, h, 0), reduce_scope(
            r, p + "n_sumexp", "single", [(t, S)], lambda: ex[b, s, h, t], op="add"))))
        attn = r.tn(p + "attn", P, [B, S, H, S], mode=AM)
        b, s, h, t = r.syms(4)
        body.append(loops([(b, B), (s, S), (h, H), (t, S)], Set(attn, (b, s, h, t), ex[b, s, h, t] / sm[b, s, h, 0])))
        av = r.tn(p + "av", P, [B, S, H, E])
        b, s, h, e, t = r.syms(5)
        body.append(loops([(b, B), (s, S), (h, H), (e, E)], Set(av, (b, s, h, e), reduce_scope(
            r, p + "n_av", "single", [(t, S)], lambda: (attn[b, s, h, t], vv[b, t, h, e]), orig=(b, s, h, e)))))
        r1 = r.tn(p + "res1", P, [B, S, D])
        b, s, o, h, e = r.syms(5)
        xin = x
        body.append(loops([(b, B), (s, S), (o, D)], Set(r1, (b, s, o), xin[b, s, o] + reduce_scope(
            r, p + "n_wo", "single", [(h, H), (e, E)], lambda: (wo[o, h, e], av[b, s, h, e]), orig=(b, s, o)))))
        x1 = r.tn(p + "x1", P, [B, S, D])
        layer_norm(p + "ln1_", r1, x1)
        fw = r.tn(p + "ffn_w", P, [F, D], read_only=True)
        fb = r.tn(p + "ffn_b", P, [F], read_only=True)
        fwo = r.tn(p + "ffn_w_out", P, [D, F], read_only=True)
        hid = r.tn(p + "ffn_h", P, [B, S, F])
        b, s, j, i = r.syms(4)
        pre = lambda: reduce_scope(r, p + "n_ffn", "single", [(i, D)], lambda: (fw[j, i], x1[b, s, i]), orig=(b, s, j)) + fb[j]
        if act == "relu":
            body.append(loops([(b, B), (s, S), (j, F)], Set(hid, (b, s, j), un("relu", pre()))))
        else:
            # the pre-activation is read three times by the composed GELU: materialised
            z = r.tn(p + "ffn_z", "single", [B, S, F])
            body.append(loops([(b, B), (s, S), (j, F)], Set(z, (b, s, j), pre())))
            b2, s2, j2 = r.syms(3)
            body.append(loops([(b2, B), (s2, S), (j2, F)], Set(hid, (b2, s2, j2), gelu_tanh(z[b2, s2, j2]))))
        r2 = r.tn(p + "res2", P, [B, S, D])
        b, s, o, j = r.syms(4)
        body.append(loops([(b, B), (s, S), (o, D)], Set(r2, (b, s, o), x1[b, s, o] + reduce_scope(
            r, p + "n_ffo", "single", [(j, F)], lambda: (fwo[o, j], hid[b, s, j]), orig=(b, s, o)))))
        x2 = r.tn(p + "x2", P, [B, S, D])
        layer_norm(p + "ln2_", r2, x2)
        x = x2
    w_head = r.tn("w_head", P, [V, D], read_only=True)
    logits = r.tn("logits", "single", [B, S, V])
    b, s, v, d = r.syms(4)
    xin = x
    body.append(loops([(b, B), (s, S), (v, V)], Set(logits, (b, s, v), reduce_scope(
        r, "n_head", "single", [(d, D)], lambda: (w_head[v, d], xin[b, s, d]), orig=(b, s, v)))))
    body.append(Comment("end"))
    r.body = Seq(body)
    return r


# ------------------------------------------------------------------ attention chain
def attention(batch: int, heads: int, queries: int, keys: int, prec: str = "bfloat16", mask: bool = True,
              row_mode: str = "ctx", out_prec: str = None, d_head: int = 64, odd_first: bool = False) -> Routine:
    """The six statements `multi_head_attention` lowers to (lib/nn_blocks.ml:222-236 with the softmax
    of :137-143), on q [b, s, h, e], k and v [b, t, h, e]: scaled scores (masked by `where` when
    `mask`), row max, exponentials, row sum, weights, weights . values.  `row_mode` is the memory
    class of the five intermediate nodes ("ctx": kept by the context, "local": routine-local).
    `odd_first` declares a three-element node ahead of the operands, so that an allocator that aligns
    to the element size only (the reference's) places everything behind it off the 16-byte grid."""
    r = Routine("attention_b%d_h%d_s%d_t%d" % (batch, heads, queries, keys))
    B, H, S, T, E = batch, heads, queries, keys, d_head
    if odd_first:
        r.tn("odd", prec, [3], read_only=True)
    q = r.tn("q", prec, [B, S, H, E], read_only=True)
    k = r.tn("k", prec, [B, T, H, E], read_only=True)
    v = r.tn("v", prec, [B, T, H, E], read_only=True)
    m = r.tn("mask", "single", [S, T], read_only=True) if mask else None
    scores = r.tn("scores", "single", [B, S, H, T], mode=row_mode)
    mx = r.tn("max", "single", [B, S, H, 1], mode=row_mode)
    ex = r.tn("exp_vals", "single", [B, S, H, T], mode=row_mode)
    sm = r.tn("sum_exp", "single", [B, S, H, 1], mode=row_mode)
    w = r.tn("attn", prec, [B, S, H, T], mode=row_mode)
    av = r.tn("av", out_prec or prec, [B, S, H, E])
    body = []
    b, s, h, t, e = r.syms(5)
    qk = reduce_scope(r, "qk", "single", [(e, E)], lambda: (q[b, s, h, e], k[b, t, h, e]), orig=(b, s, h, t)) / math.sqrt(E)
    body.append(loops([(b, B), (s, S), (h, H), (t, T)], Set(scores, (b, s, h, t), where(m[s, t], qk, Const(-1e9)) if mask else qk)))
    b, s, h, t = r.syms(4)
    body.append(loops([(b, B), (s, S), (h, H)], Set(mx, (b, s, h, 0), reduce_scope(
        r, "n_max", "single", [(t, T)], lambda: scores[b, s, h, t], op="max"))))
    b, s, h, t = r.syms(4)
    body.append(loops([(b, B), (s, S), (h, H), (t, T)], Set(ex, (b, s, h, t), un("exp", scores[b, s, h, t] - mx[b, s, h, 0]))))
    b, s, h, t = r.syms(4)
    body.append(loops([(b, B), (s, S), (h, H)], Set(sm, (b, s, h, 0), reduce_scope(
        r, "n_sumexp", "single", [(t, T)], lambda: ex[b, s, h, t], op="add"))))
    b, s, h, t = r.syms(4)
    body.append(loops([(b, B), (s, S), (h, H), (t, T)], Set(w, (b, s, h, t), ex[b, s, h, t] / sm[b, s, h, 0])))
    b, s, h, e, t = r.syms(5)
    body.append(loops([(b, B), (s, S), (h, H), (e, E)], Set(av, (b, s, h, e), reduce_scope(
        r, "n_av", "single", [(t, T)], lambda: (w[b, s, h, t], v[b, t, h, e]), orig=(b, s, h, e)))))
    r.body = Seq(body)
    return r


def attention_inputs(batch: int, heads: int, queries: int, keys: int, prec: str = "bfloat16", seed: int = 31, d_head: int = 64):
    rng = np.random.default_rng(seed)
    out = {n: store(prec, rng.standard_normal(shape).astype(np.float32))
           for n, shape in (("q", (batch, queries, heads, d_head)), ("k", (batch, keys, heads, d_head)),
                            ("v", (batch, keys, heads, d_head)))}
    # a causal band shifted so that every row keeps at least one key, plus a few holes
    s_idx, t_idx = np.arange(queries)[:, None], np.arange(keys)[None, :]
    mask = (t_idx <= (s_idx * keys) // max(queries, 1)).astype(np.float32)
    mask[rng.integers(0, queries, 16), rng.integers(0, keys, 16)] = 0.0
    mask[:, 0] = 1.0
    out["mask"] = mask
    return out


# ------------------------------------------------------------------ config 5 (ii): forward + backward, SGD
def mlp_train_update(rows=8192, dims=(784, 1024, 1024, 10), wprec="bfloat16") -> Routine:
    """`Train.grad_update` of the softmax cross-entropy MLP (lib/train.ml:61-73): forward, zero
    grads, backprop.  bf16 weights, activations and activation gradients; parameter gradients
    and the gradients that are accumulated over a contracted axis are fp32 (so that the
    contraction result nodes are fp32, as the tensor-core path requires).  Back-propagation
    keeps the forward loop order (b, o, i): dW reduces over the outermost loop, dX over the
    middle one."""
    r = Routine("mlp_update_%d" % rows)
    n_layers = len(dims) - 1
    x = r.tn("x", wprec, [rows, dims[0]], read_only=True)
    labels = r.tn("labels", "single", [rows, dims[-1]], read_only=True)
    body: List = [Comment("loss forward and gradient update")]
    W_, Bv, H = [], [], [x]
    for l in range(n_layers):
        fi, fo = dims[l], dims[l + 1]
        last = l == n_layers - 1
        w = r.tn("w_out" if last else "w%d" % (l + 1), wprec, [fo, fi], read_only=True)
        W_.append(w)
        ib, io, ii = r.syms(3)
        hin = H[-1]
        acc = lambda: reduce_scope(r, "n_mm%d" % l, "single", [(ii, fi)], lambda: (w[io, ii], hin[ib, ii]), orig=(ib, io))
        if last:
            out = r.tn("logits", "single", [rows, fo])
            body.append(loops([(ib, rows), (io, fo)], Set(out, (ib, io), acc())))
            Bv.append(None)
        else:
            b = r.tn("b%d" % (l + 1), wprec, [fo], read_only=True)
            Bv.append(b)
            out = r.tn("h%d" % (l + 1), wprec, [rows, fo])
            body.append(loops([(ib, rows), (io, fo)], Set(out, (ib, io), un("relu", acc() + b[io]))))
        H.append(out)
    C = dims[-1]
    logits = H[-1]
    max_l = r.tn("max_l", "single", [rows, 1])
    expv = r.tn("exp_vals", "single", [rows, C])
    ssum = r.tn("sum_exp", "single", [rows, 1])
    loss = r.tn("loss", "single", [1])
    ib, ic = r.syms(2)
    body.append(loops([(ib, rows)], Set(max_l, (ib, 0), reduce_scope(r, "n_max", "single", [(ic, C)], lambda: logits[ib, ic], op="max"))))
    ib, ic = r.syms(2)
    body.append(loops([(ib, rows), (ic, C)], Set(expv, (ib, ic), un("exp", logits[ib, ic] - max_l[ib, 0]))))
    ib, ic = r.syms(2)
    body.append(loops([(ib, rows)], Set(ssum, (ib, 0), reduce_scope(r, "n_sum", "single", [(ic, C)], lambda: expv[ib, ic], op="add"))))
    ib, ic = r.syms(2)
    body.append(Set(loss, (0,), un("neg", reduce_scope(
        r, "n_ce", "single", [(ib, rows), (ic, C)], lambda: labels[ib, ic] * un("log", expv[ib, ic] / ssum[ib, 0]), op="add")) / float(rows)))
    # ---- zero grads and backprop
    body.append(Comment("zero grads and backprop"))
    gW = [r.tn(w.ident + "_grad", "single", w.dims) for w in W_]
    gB = [r.tn(b.ident + "_grad", "single", b.dims) if b is not None else None for b in Bv]
    dH = [None] + [r.tn("h%d_grad" % l, "single", [rows, dims[l]]) for l in range(1, n_layers)]
    for g in gW + [g for g in gB if g is not None] + [d for d in dH if d is not None]:
        body.append(ZeroOut(g))
    dz = r.tn("logits_grad", wprec, [rows, C])
    ib, ic = r.syms(2)
    body.append(loops([(ib, rows), (ic, C)], Set(dz, (ib, ic), (expv[ib, ic] / ssum[ib, 0] - labels[ib, ic]) / float(rows))))
    for l in reversed(range(n_layers)):
        fi, fo = dims[l], dims[l + 1]
        w, gw, hin = W_[l], gW[l], H[l]
        if gB[l] is not None:
            ib, io = r.syms(2)
            body.append(loops([(ib, rows), (io, fo)], Set(gB[l], (io,), gB[l][io] + dz[ib, io])))
        ib, io, ii = r.syms(3)
        dzz = dz
        body.append(loops([(ib, rows), (io, fo), (ii, fi)], Set(gw, (io, ii), fma(dzz[ib, io], hin[ib, ii], gw[io, ii]))))
        if l > 0:
            ib, io, ii = r.syms(3)
            body.append(loops([(ib, rows), (io, fo), (ii, fi)], Set(dH[l], (ib, ii), fma(w[io, ii], dzz[ib, io], dH[l][ib, ii]))))
            ndz = r.tn("z%d_grad" % l, wprec, [rows, fi])
            ib, ii = r.syms(2)
            body.append(loops([(ib, rows), (ii, fi)], Set(ndz, (ib, ii), binop("relu_gate", hin[ib, ii], dH[l][ib, ii]))))
            dz = ndz
    body.append(Comment("end"))
    r.body = Seq(body)
    return r


def mlp_sgd(dims=(784, 1024, 1024, 10), wprec="bfloat16", momentum=0.0, weight_decay=0.0, nesterov=False) -> Routine:
    """`Train.sgd_update` (lib/train.ml:76-91) per parameter: `sgd_delta =: p.grad + weight_decay * p`;
    with momentum `sgd_momentum =: momentum * sgd_momentum + sgd_delta` and then
    `sgd_delta =+ momentum * sgd_momentum` (Nesterov) or `sgd_delta =: sgd_momentum`; last
    `p =- learning_rate * sgd_delta`.  Without momentum `sgd_delta` is read once and is inlined
    into the parameter's assignment; with momentum it and `sgd_momentum` are fp32 nodes and the
    three or four assignments are separate loop nests over the parameter's axes."""
    tag = "" if momentum == 0.0 and weight_decay == 0.0 else "_m%g_wd%g%s" % (momentum, weight_decay, "_nesterov" if nesterov else "")
    r = Routine("mlp_sgd" + tag.replace(".", "p").replace("-", "n"))
    lr = r.tn("learning_rate", "single", [1], read_only=True)
    n_layers = len(dims) - 1
    body: List = [Comment("sgd_update")]
    for l in range(n_layers):
        fi, fo = dims[l], dims[l + 1]
        last = l == n_layers - 1
        names = [("w_out" if last else "w%d" % (l + 1), [fo, fi])] + ([] if last else [("b%d" % (l + 1), [fo])])
        for name, d in names:
            p = r.tn(name, wprec, d)
            g = r.tn(name + "_grad", "single", d, read_only=True)
            nest = lambda: (lambda syms: (list(zip(syms, d)), tuple(syms)))(r.syms(len(d)))
            delta = lambda idx: (Get(g, idx) + float(weight_decay) * Get(p, idx)) if weight_decay != 0.0 else Get(g, idx)
            if momentum > 0.0:
                sd = r.tn(name + "_sgd_delta", "single", d)
                sm = r.tn(name + "_sgd_momentum", "single", d)
                lp, idx = nest()
                body.append(loops(lp, Set(sd, idx, delta(idx))))
                lp, idx = nest()
                body.append(loops(lp, Set(sm, idx, float(momentum) * Get(sm, idx) + Get(sd, idx))))
                lp, idx = nest()
                if nesterov:
                    body.append(loops(lp, Set(sd, idx, Get(sd, idx) + float(momentum) * Get(sm, idx))))
                else:
                    body.append(loops(lp, Set(sd, idx, Get(sm, idx))))
                lp, idx = nest()
                body.append(loops(lp, Set(p, idx, Get(p, idx) - lr[0] * Get(sd, idx))))
            else:
                lp, idx = nest()
                body.append(loops(lp, Set(p, idx, Get(p, idx) - lr[0] * delta(idx))))
    body.append(Comment("end"))
    r.body = Seq(body)
    return r


MLP_PARAM_NAMES = ("w1", "b1", "w2", "b2", "w_out")


# ------------------------------------------------------------------ convolution as a contraction with affine indices
def conv2d_update(batch=4, size=16, cin=8, cout=16, kernel=3, stride=1, prec="single") -> Routine:
    """A `same`-padded (stride 1) or `valid` strided 2-d convolution layer with bias and relu,
    its squared-error loss and the gradients of kernel, bias and input, in the forms the
    reference lowers `conv2d` to (lib/nn_blocks.ml:418-428): the input position of an output
    position is the affine index `stride * oh + kh`, a
    padded node carries its margins in its dimensions, accesses to it are shifted by the left
    margin (`apply_padding_offset`, arrayjit/lib/assignments.ml:202-219) and the margins are reset by loops of constant assignments before the node is filled
    (`reset_padding_regions`, assignments.ml:281-297)."""
    pad = (kernel - 1) // 2 if stride == 1 else 0
    out = size if stride == 1 else (size - kernel) // stride + 1
    padded = size + 2 * pad
    r = Routine("conv2d_update_b%d_s%d_c%d_%d_k%d_st%d_%s" % (batch, size, cin, cout, kernel, stride, prec))
    x = r.tn("x", prec, [batch, size, size, cin], read_only=True)
    xp = r.tn("x_padded", prec, [batch, padded, padded, cin])
    kw_ = r.tn("kernel", prec, [cout, kernel, kernel, cin], read_only=True)
    bias = r.tn("bias", prec, [cout], read_only=True)
    y = r.tn("y", prec, [batch, out, out, cout])
    target = r.tn("target", prec, [batch, out, out, cout], read_only=True)
    loss = r.tn("loss", "single", [1])
    body: List = [Comment("conv fwd")]
    if pad:
        body.append(Comment("reset padding margins of x_padded to 0"))
        ib, ih, iw, ic = r.syms(4)
        for lo, hi in ((0, pad - 1), (padded - pad, padded - 1)):
            body.append(For(ib, 0, batch - 1, For(ih, lo, hi, For(iw, 0, padded - 1, For(ic, 0, cin - 1,
                        Set(xp, (ib, ih, iw, ic), Const(0.0, prec)))))))
            ib, ih, iw, ic = r.syms(4)
            body.append(For(ib, 0, batch - 1, For(ih, pad, padded - pad - 1, For(iw, lo, hi, For(ic, 0, cin - 1,
                        Set(xp, (ib, ih, iw, ic), Const(0.0, prec)))))))
            ib, ih, iw, ic = r.syms(4)
    ib, ih, iw, ic = r.syms(4)
    body.append(loops([(ib, batch), (ih, size), (iw, size), (ic, cin)],
                      Set(xp, (ib, Affine(((1, ih),), pad), Affine(((1, iw),), pad), ic), x[ib, ih, iw, ic])))
    ib, oh, ow, co, kh, kw, ci = r.syms(7)
    src = lambda: xp[ib, Affine(((stride, oh), (1, kh))), Affine(((stride, ow), (1, kw))), ci]
    body.append(loops([(ib, batch), (oh, out), (ow, out), (co, cout)], Set(y, (ib, oh, ow, co), un("relu", bias[co] + reduce_scope(
        r, "n_conv", "single", [(kh, kernel), (kw, kernel), (ci, cin)], lambda: (kw_[co, kh, kw, ci], src()),
        orig=(ib, oh, ow, co))))))
    ib, oh, ow, co = r.syms(4)
    diff = lambda: y[ib, oh, ow, co] - target[ib, oh, ow, co]
    body.append(Set(loss, (0,), reduce_scope(r, "n_sq", "single", [(ib, batch), (oh, out), (ow, out), (co, cout)],
                                            lambda: (diff(), diff())) / float(batch)))
    body.append(Comment("zero grads and backprop"))
    gk = r.tn("kernel_grad", "single", kw_.dims)
    gb = r.tn("bias_grad", "single", bias.dims)
    gx = r.tn("x_padded_grad", "single", xp.dims)
    dz = r.tn("z_grad", prec, y.dims)
    for g in (gk, gb, gx):
        body.append(ZeroOut(g))
    ib, oh, ow, co = r.syms(4)
    body.append(loops([(ib, batch), (oh, out), (ow, out), (co, cout)], Set(dz, (ib, oh, ow, co), binop(
        "relu_gate", y[ib, oh, ow, co], (y[ib, oh, ow, co] - target[ib, oh, ow, co]) * (2.0 / batch)))))
    ib, oh, ow, co = r.syms(4)
    body.append(loops([(ib, batch), (oh, out), (ow, out), (co, cout)], Set(gb, (co,), gb[co] + dz[ib, oh, ow, co])))
    ib, oh, ow, co, kh, kw, ci = r.syms(7)
    nest = [(ib, batch), (oh, out), (ow, out), (co, cout), (kh, kernel), (kw, kernel), (ci, cin)]
    body.append(loops(nest, Set(gk, (co, kh, kw, ci), fma(dz[ib, oh, ow, co], src(), gk[co, kh, kw, ci]))))
    ib, oh, ow, co, kh, kw, ci = r.syms(7)
    nest = [(ib, batch), (oh, out), (ow, out), (co, cout), (kh, kernel), (kw, kernel), (ci, cin)]
    at = (ib, Affine(((stride, oh), (1, kh))), Affine(((stride, ow), (1, kw))), ci)
    body.append(loops(nest, Set(gx, at, fma(kw_[co, kh, kw, ci], dz[ib, oh, ow, co], Get(gx, at)))))
    body.append(Comment("end"))
    r.body = Seq(body)
    return r


def conv2d_inputs(batch=4, size=16, cin=8, cout=16, kernel=3, stride=1, prec="single"):
    out = size if stride == 1 else (size - kernel) // stride + 1
    g = np.random.default_rng(31)
    return {"x": store(prec, g.standard_normal((batch, size, size, cin), np.float32)),
            "kernel": store(prec, (g.standard_normal((cout, kernel, kernel, cin), np.float32) / math.sqrt(kernel * kernel * cin)).astype(np.float32)),
            "bias": store(prec, 0.1 * g.standard_normal(cout).astype(np.float32)),
            "target": store(prec, g.standard_normal((batch, out, out, cout), np.float32))}
