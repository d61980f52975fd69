"""CPU tests of the oracle (oracle/fdeep_oracle.cpp).

The reference cannot be built here and holds no golden vectors, so the oracle is cross-checked
against independent PyTorch CPU operators (float64 where possible) and hand-computed cases, and
against the committed fixtures under tests/golden/ (regression pin).
"""
import glob
import json
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from fdeep_b200 import model_writer as mw
from oracle import OracleModel
from util import assert_close, model_text

HERE = os.path.dirname(os.path.abspath(__file__))


def tf_same_pad(size, k, s, d=1):
    ek = (k - 1) * d + 1
    total = max(ek - s, 0) if size % s == 0 else max(ek - size % s, 0)
    return total // 2, total - total // 2


def run_oracle(js, inputs):
    return OracleModel(json_text=model_text(js)).predict(inputs)


@pytest.mark.parametrize("k,s,d,pad,cin,cout,h,w", [
    (3, 1, 1, "same", 3, 8, 9, 11), (3, 2, 1, "same", 4, 6, 10, 7), (1, 1, 1, "valid", 8, 16, 5, 5),
    (1, 2, 1, "valid", 8, 4, 9, 9), (7, 2, 1, "valid", 3, 8, 23, 23), (3, 1, 2, "same", 4, 4, 12, 12),
    (5, 3, 1, "same", 2, 3, 14, 13), (3, 1, 1, "valid", 5, 7, 6, 8), (2, 2, 1, "same", 3, 3, 7, 7),
])
def test_conv2d_against_torch(k, s, d, pad, cin, cout, h, w):
    rng = np.random.default_rng(k * 100 + s * 10 + d + h)
    kernel = rng.normal(size=(k, k, cin, cout)).astype(np.float32)
    bias = rng.normal(size=cout).astype(np.float32)
    x = rng.normal(size=(h, w, cin)).astype(np.float32)
    b = mw.ModelBuilder("m")
    i = b.input([h, w, cin])
    o = mw.conv2d(b, i, "c", kernel, bias, strides=s, padding=pad, dilation=d)
    oh = -(-h // s) if pad == "same" else -(-(h - ((k - 1) * d + 1) + 1) // s)
    ow = -(-w // s) if pad == "same" else -(-(w - ((k - 1) * d + 1) + 1) // s)
    got = run_oracle(b.to_json([o], [[oh, ow, cout]]), [x])[0]
    xt = torch.from_numpy(x).double().permute(2, 0, 1)[None]
    if pad == "same":
        pt, pb = tf_same_pad(h, k, s, d)
        pl, pr = tf_same_pad(w, k, s, d)
        xt = F.pad(xt, (pl, pr, pt, pb))
    want = F.conv2d(xt, torch.from_numpy(kernel).double().permute(3, 2, 0, 1), torch.from_numpy(bias).double(), stride=s, dilation=d)
    want = want[0].permute(1, 2, 0).numpy().astype(np.float32)
    assert_close(got, want, "conv2d", rel=1e-4)


@pytest.mark.parametrize("s,pad,h,w,c", [(1, "same", 8, 9, 6), (2, "valid", 9, 9, 4), (2, "same", 10, 7, 3)])
def test_depthwise_against_torch(s, pad, h, w, c):
    rng = np.random.default_rng(7 + s + h)
    kernel = rng.normal(size=(3, 3, c, 1)).astype(np.float32)
    bias = rng.normal(size=c).astype(np.float32)
    x = rng.normal(size=(h, w, c)).astype(np.float32)
    b = mw.ModelBuilder("m")
    i = b.input([h, w, c])
    o = mw.depthwise_conv2d(b, i, "d", kernel, bias, strides=s, padding=pad)
    oh = -(-h // s) if pad == "same" else (h - 3) // s + 1
    ow = -(-w // s) if pad == "same" else (w - 3) // s + 1
    got = run_oracle(b.to_json([o], [[oh, ow, c]]), [x])[0]
    xt = torch.from_numpy(x).double().permute(2, 0, 1)[None]
    if pad == "same":
        pt, pb = tf_same_pad(h, 3, s)
        pl, pr = tf_same_pad(w, 3, s)
        xt = F.pad(xt, (pl, pr, pt, pb))
    wt = torch.from_numpy(kernel).double().permute(2, 3, 0, 1)  # (C,1,kh,kw)
    want = F.conv2d(xt, wt, torch.from_numpy(bias).double(), stride=s, groups=c)[0].permute(1, 2, 0).numpy().astype(np.float32)
    assert_close(got, want, "depthwise", rel=1e-4)


@pytest.mark.parametrize("kind,p,s,pad,h,w", [("max", 2, 2, "valid", 8, 8), ("max", 3, 2, "same", 9, 10), ("avg", 3, 2, "same", 9, 10),
                                                ("avg", 2, 2, "valid", 7, 9), ("max", 3, 1, "same", 5, 5), ("avg", 3, 1, "same", 5, 6)])
def test_pooling_against_torch(kind, p, s, pad, h, w):
    rng = np.random.default_rng(3 + p + h)
    c = 5
    x = rng.normal(size=(h, w, c)).astype(np.float32)
    b = mw.ModelBuilder("m")
    i = b.input([h, w, c])
    o = (mw.max_pool2d if kind == "max" else mw.avg_pool2d)(b, i, "p", p, s, pad)
    oh = -(-h // s) if pad == "same" else (h - p) // s + 1
    ow = -(-w // s) if pad == "same" else (w - p) // s + 1
    got = run_oracle(b.to_json([o], [[oh, ow, c]]), [x])[0]
    xt = torch.from_numpy(x).double().permute(2, 0, 1)[None]
    pt = pb = pl = pr = 0
    if pad == "same":
        pt, pb = tf_same_pad(h, p, s)
        pl, pr = tf_same_pad(w, p, s)
    if kind == "max":
        want = F.max_pool2d(F.pad(xt, (pl, pr, pt, pb), value=-1e30), p, s)
    else:  # divide by the number of taps inside the tensor (average_pooling_3d_layer.hpp:34-41)
        ssum = F.avg_pool2d(F.pad(xt, (pl, pr, pt, pb)), p, s, divisor_override=1)
        cnt = F.avg_pool2d(F.pad(torch.ones_like(xt), (pl, pr, pt, pb)), p, s, divisor_override=1)
        want = ssum / cnt
    want = want[0].permute(1, 2, 0).numpy().astype(np.float32)
    assert_close(got, want, "pool", rel=1e-4)


def test_dense_bn_layernorm_softmax_against_torch():
    rng = np.random.default_rng(11)
    x = rng.normal(size=(6, 12)).astype(np.float32)
    W = rng.normal(size=(12, 9)).astype(np.float32)
    bias = rng.normal(size=9).astype(np.float32)
    mean, var = rng.normal(size=9).astype(np.float32), rng.uniform(0.5, 1.5, 9).astype(np.float32)
    gamma, beta = rng.normal(size=9).astype(np.float32), rng.normal(size=9).astype(np.float32)
    g2, b2 = rng.normal(size=9).astype(np.float32), rng.normal(size=9).astype(np.float32)
    b = mw.ModelBuilder("m")
    i = b.input([6, 12])
    d = mw.dense(b, i, "d", W, bias, "relu")
    n = mw.batch_norm(b, d, "bn", mean, var, gamma, beta, eps=1e-3)
    ln = mw.layer_norm(b, n, "ln", g2, b2, eps=1e-5)
    sm = mw.activation(b, ln, "sm", "softmax")
    outs = run_oracle(b.to_json([d, n, ln, sm], [[6, 9]] * 4), [x])
    xt = torch.from_numpy(x).double()
    td = torch.relu(xt @ torch.from_numpy(W).double() + torch.from_numpy(bias).double())
    tn = (td - torch.from_numpy(mean).double()) / torch.sqrt(torch.from_numpy(var).double() + 1e-3) * torch.from_numpy(gamma).double() + torch.from_numpy(beta).double()
    tl = F.layer_norm(tn, (9,), torch.from_numpy(g2).double(), torch.from_numpy(b2).double(), eps=1e-5)
    ts = torch.softmax(tl, dim=-1)
    for got, want, name in zip(outs, (td, tn, tl, ts), ("dense", "bn", "ln", "softmax")):
        assert_close(got, want.numpy().astype(np.float32), name, rel=1e-4)


def norms_model():
    """RMS, unit and group normalisation on one (5, 6, 8) input; returns (json, input, float64 expectations)."""
    rng = np.random.default_rng(21)
    x = rng.normal(size=(5, 6, 8)).astype(np.float32)
    scale = rng.normal(size=8).astype(np.float32)
    gamma, beta = rng.normal(size=8).astype(np.float32), rng.normal(size=8).astype(np.float32)
    b = mw.ModelBuilder("norms")
    i = b.input([5, 6, 8])
    rms = b.add("RMSNormalization", "rms", {"axis": [-1], "epsilon": 1e-6}, i, {"scale": scale})
    unit = b.add("UnitNormalization", "unit", {"axis": [-1]}, i)
    grp = b.add("GroupNormalization", "grp", {"groups": 4, "axis": -1, "epsilon": 1e-3, "center": True, "scale": True}, i,
                {"gamma": gamma, "beta": beta})
    grp1 = b.add("GroupNormalization", "grp_plain", {"groups": 1, "axis": -1, "epsilon": 1e-3, "center": False, "scale": False}, i)
    js = b.to_json([rms, unit, grp, grp1], [[5, 6, 8]] * 4)
    xd = x.astype(np.float64)
    want_rms = xd / np.sqrt((xd ** 2).mean(-1, keepdims=True) + 1e-6) * scale
    want_unit = xd / np.sqrt(np.maximum((xd ** 2).sum(-1, keepdims=True), np.finfo(np.float32).eps))
    g = xd.reshape(5, 6, 4, 2)
    m, v = g.mean(axis=(0, 1, 3), keepdims=True), g.var(axis=(0, 1, 3), keepdims=True)
    want_grp = ((g - m) / np.sqrt(v + 1e-3)).reshape(5, 6, 8) * gamma + beta
    want_grp1 = (xd - xd.mean()) / np.sqrt(xd.var() + 1e-3)
    return js, x, [want_rms, want_unit, want_grp, want_grp1]


def test_rms_unit_group_normalisation_against_numpy():
    js, x, wants = norms_model()
    outs = run_oracle(js, [x])
    for got, want, name in zip(outs, wants, ("rms", "unit", "group", "group_plain")):
        assert_close(got, want.astype(np.float32), name, rel=1e-5)


def test_lstm_against_torch():
    rng = np.random.default_rng(5)
    T, Fdim, U = 7, 5, 6
    W = rng.normal(size=(Fdim, 4 * U)).astype(np.float32) * 0.4
    Uw = rng.normal(size=(U, 4 * U)).astype(np.float32) * 0.4
    bias = rng.normal(size=4 * U).astype(np.float32) * 0.1
    x = rng.normal(size=(T, Fdim)).astype(np.float32)
    b = mw.ModelBuilder("m")
    i = b.input([T, Fdim])
    seq, h, c = mw.lstm(b, i, "l", W, Uw, bias, return_sequences=True, return_state=True)
    got = run_oracle(b.to_json([seq, h, c], [[T, U], [U], [U]]), [x])
    lstm = torch.nn.LSTM(Fdim, U, batch_first=True).double()
    with torch.no_grad():
        lstm.weight_ih_l0.copy_(torch.from_numpy(W.T).double())
        lstm.weight_hh_l0.copy_(torch.from_numpy(Uw.T).double())
        lstm.bias_ih_l0.copy_(torch.from_numpy(bias).double())
        lstm.bias_hh_l0.zero_()
        out, (hn, cn) = lstm(torch.from_numpy(x).double()[None])
    assert_close(got[0], out[0].numpy().astype(np.float32), "lstm seq", rel=1e-4)
    assert_close(got[1], hn[0, 0].numpy().astype(np.float32), "lstm h", rel=1e-4)
    assert_close(got[2], cn[0, 0].numpy().astype(np.float32), "lstm c", rel=1e-4)


def test_gru_reset_after_against_torch():
    rng = np.random.default_rng(6)
    T, Fdim, U = 6, 4, 5
    W = rng.normal(size=(Fdim, 3 * U)).astype(np.float32) * 0.4   # Keras order z, r, h
    Uw = rng.normal(size=(U, 3 * U)).astype(np.float32) * 0.4
    bias = rng.normal(size=(2, 3 * U)).astype(np.float32) * 0.1
    x = rng.normal(size=(T, Fdim)).astype(np.float32)
    b = mw.ModelBuilder("m")
    i = b.input([T, Fdim])
    seq = mw.gru(b, i, "g", W, Uw, bias.reshape(-1), reset_after=True, return_sequences=True)
    got = run_oracle(b.to_json([seq], [[T, U]]), [x])[0]

    def reorder(m):  # Keras z, r, h -> torch r, z, n
        z, r, h = np.split(m, 3, axis=-1)
        return np.concatenate([r, z, h], axis=-1)
    gru = torch.nn.GRU(Fdim, U, batch_first=True).double()
    with torch.no_grad():
        gru.weight_ih_l0.copy_(torch.from_numpy(reorder(W).T).double())
        gru.weight_hh_l0.copy_(torch.from_numpy(reorder(Uw).T).double())
        gru.bias_ih_l0.copy_(torch.from_numpy(reorder(bias[0])).double())
        gru.bias_hh_l0.copy_(torch.from_numpy(reorder(bias[1])).double())
        out, _ = gru(torch.from_numpy(x).double()[None])
    assert_close(got, out[0].numpy().astype(np.float32), "gru", rel=1e-4)


def gru_plain_model(T=6, Fdim=4, U=8, seed=16):
    """GRU with reset_after=False (one bias of 3U, reset gate applied to h before the candidate product),
    with the numpy result of the Keras recurrence in float64."""
    rng = np.random.default_rng(seed)
    W = rng.normal(size=(Fdim, 3 * U)).astype(np.float32) * 0.4   # Keras order z, r, h
    Uw = rng.normal(size=(U, 3 * U)).astype(np.float32) * 0.4
    bias = rng.normal(size=3 * U).astype(np.float32) * 0.1
    x = rng.normal(size=(T, Fdim)).astype(np.float32)
    b = mw.ModelBuilder("m")
    i = b.input([T, Fdim])
    seq = mw.gru(b, i, "g", W, Uw, bias, reset_after=False, return_sequences=True)
    js = b.to_json([seq], [[T, U]])
    sig = lambda v: 1.0 / (1.0 + np.exp(-v))
    h = np.zeros(U)
    want = []
    for t in range(T):
        xp = x[t].astype(np.float64) @ W + bias
        z = sig(xp[:U] + h @ Uw[:, :U])
        r = sig(xp[U:2 * U] + h @ Uw[:, U:2 * U])
        hh = np.tanh(xp[2 * U:] + (r * h) @ Uw[:, 2 * U:])
        h = z * h + (1 - z) * hh
        want.append(h)
    return js, x, np.array(want)


def test_gru_without_reset_after_against_numpy():
    js, x, want = gru_plain_model()
    got = run_oracle(js, [x])[0]
    assert_close(got, want.astype(np.float32), "gru reset_after=False", rel=1e-4)


def lstm_weights(rng, Fdim, U):
    return (rng.normal(size=(Fdim, 4 * U)).astype(np.float32) * 0.4, rng.normal(size=(U, 4 * U)).astype(np.float32) * 0.4,
            rng.normal(size=4 * U).astype(np.float32) * 0.1)


def torch_lstm(x, layers, bidirectional=False):
    """float64 torch LSTM with Keras weights: `layers` is a list of (W, U, b) per layer, or per layer a pair
    of them (forward, backward) when bidirectional.  Gate order i, f, c, o is the same in both."""
    first = layers[0][0] if bidirectional else layers[0]
    m = torch.nn.LSTM(first[0].shape[0], first[1].shape[0], num_layers=len(layers), batch_first=True, bidirectional=bidirectional).double()
    with torch.no_grad():
        for li, layer in enumerate(layers):
            for suffix, (W, U, b) in zip(("", "_reverse"), layer if bidirectional else (layer,)):
                getattr(m, f"weight_ih_l{li}{suffix}").copy_(torch.from_numpy(W.T).double())
                getattr(m, f"weight_hh_l{li}{suffix}").copy_(torch.from_numpy(U.T).double())
                getattr(m, f"bias_ih_l{li}{suffix}").copy_(torch.from_numpy(b).double())
                getattr(m, f"bias_hh_l{li}{suffix}").zero_()
        out, (hn, cn) = m(torch.from_numpy(x).double()[None])
    return out[0].numpy(), hn[:, 0].numpy(), cn[:, 0].numpy()


def bidirectional_models(T=7, Fdim=5, U=8, seed=21):
    """One input, five Bidirectional(LSTM) heads: concat with sequences, and concat / sum / mul / ave of the
    last states; returns the model, an input and the float64 torch results."""
    rng = np.random.default_rng(seed)
    fw, bw = lstm_weights(rng, Fdim, U), lstm_weights(rng, Fdim, U)
    x = rng.normal(size=(T, Fdim)).astype(np.float32)
    b = mw.ModelBuilder("m")
    i = b.input([T, Fdim])
    outs = [mw.bidirectional(b, i, "bi_seq", "LSTM", fw, bw, "concat", return_sequences=True)]
    shapes = [[T, 2 * U]]
    for mode in ("concat", "sum", "mul", "ave"):
        outs.append(mw.bidirectional(b, i, "bi_" + mode, "LSTM", fw, bw, mode))
        shapes.append([2 * U] if mode == "concat" else [U])
    seq, hn, _ = torch_lstm(x, [(fw, bw)], bidirectional=True)
    f, r = hn[0], hn[1]
    wants = [seq, np.concatenate([f, r]), f + r, f * r, (f + r) / 2]
    return b.to_json(outs, shapes), x, wants


def test_bidirectional_lstm_against_torch():
    js, x, wants = bidirectional_models()
    outs = run_oracle(js, [x])
    for got, want, name in zip(outs, wants, ("seq", "concat", "sum", "mul", "ave")):
        assert_close(got, want.astype(np.float32), "bidirectional " + name, rel=1e-4)


def stacked_rnn_model(T=6, Fdim=5, U=8, seed=22, return_sequences=True):
    rng = np.random.default_rng(seed)
    l0, l1 = lstm_weights(rng, Fdim, U), lstm_weights(rng, U, U)
    x = rng.normal(size=(T, Fdim)).astype(np.float32)
    b = mw.ModelBuilder("m")
    i = b.input([T, Fdim])
    stacked = mw.rnn(b, i, "stack", [("LSTMCell",) + l0 + (None,), ("LSTMCell",) + l1 + (None,)], return_sequences=return_sequences)
    single = mw.rnn(b, i, "single", [("LSTMCell",) + l0 + (None,)], return_sequences=False, return_state=True)
    seq2, hn2, _ = torch_lstm(x, [l0, l1])
    _, hn1, cn1 = torch_lstm(x, [l0])
    js = b.to_json([stacked] + list(single), [[T, U] if return_sequences else [U], [U], [U], [U]])
    return js, x, [seq2 if return_sequences else hn2[1], hn1[0], hn1[0], cn1[0]]


@pytest.mark.parametrize("return_sequences", [True, False])
def test_rnn_of_cells_against_torch(return_sequences):
    js, x, wants = stacked_rnn_model(return_sequences=return_sequences)
    outs = run_oracle(js, [x])
    for got, want, name in zip(outs, wants, ("stacked", "single out", "single h", "single c")):
        assert_close(got, want.astype(np.float32), "rnn " + name, rel=1e-4)


def np_softmax(s):
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def attention_zoo(Tq=5, Tk=7, D=6, Dv=4, seed=31):
    """Attention (dot with and without scale, concat), AdditiveAttention (no scale, vector scale), with separate
    key inputs and without; returns the model, the inputs (query, value, key) and float64 numpy results."""
    rng = np.random.default_rng(seed)
    q, v, k = (rng.normal(size=s).astype(np.float32) for s in ((Tq, D), (Tk, Dv), (Tk, D)))
    v_same = rng.normal(size=(Tk, D)).astype(np.float32)
    svec = rng.normal(size=D).astype(np.float32)
    b = mw.ModelBuilder("m")
    iq, iv, ik, ivs = b.input([Tq, D]), b.input([Tk, Dv]), b.input([Tk, D]), b.input([Tk, D])
    outs = [mw.attention(b, iq, iv, "dot_plain", k=ik),
            mw.attention(b, iq, iv, "dot_scaled", k=ik, scale=0.37),
            mw.attention(b, iq, ivs, "dot_two_inputs"),
            mw.attention(b, iq, iv, "concat", k=ik, score_mode="concat", scale=0.8, concat_score_weight=1.7),
            mw.additive_attention(b, iq, iv, "add_plain", k=ik),
            mw.additive_attention(b, iq, iv, "add_scaled", k=ik, scale=svec)]
    shapes = [[Tq, Dv], [Tq, Dv], [Tq, D], [Tq, Dv], [Tq, Dv], [Tq, Dv]]
    Q, V, K, VS = (a.astype(np.float64) for a in (q, v, k, v_same))
    pair = np.tanh(Q[:, None, :] + K[None, :, :])
    wants = [np_softmax(Q @ K.T) @ V, np_softmax(0.37 * (Q @ K.T)) @ V, np_softmax(Q @ VS.T) @ VS,
             np_softmax(1.7 * np.tanh(0.8 * (Q[:, None, :] + K[None, :, :])).sum(-1)) @ V,
             np_softmax(pair.sum(-1)) @ V, np_softmax((pair * svec).sum(-1)) @ V]
    return b.to_json(outs, shapes), [q, v, k, v_same], wants


def test_attention_layers_against_numpy():
    js, xs, wants = attention_zoo()
    outs = run_oracle(js, xs)
    for i, (got, want) in enumerate(zip(outs, wants)):
        assert_close(got, want.astype(np.float32), f"attention {i}", rel=1e-4)


def gqa_model(Tq=4, Tk=6, dim=8, Hq=4, Hkv=2, hd=3, out_dim=5, use_bias=True, use_gate=False, seed=41):
    rng = np.random.default_rng(seed)
    q, x = rng.normal(size=(Tq, dim)).astype(np.float32), rng.normal(size=(Tk, dim)).astype(np.float32)
    def kern(*shape):
        return rng.normal(size=shape).astype(np.float32) * 0.4
    heads = [Hq, Hkv] + ([Hq] if use_gate else []) + [Hkv]
    weights = []
    for h in heads:
        weights.append(kern(dim, h, hd))
        if use_bias:
            weights.append(kern(h, hd))
    weights.append(kern(Hq, hd, out_dim))
    if use_bias:
        weights.append(kern(out_dim))
    b = mw.ModelBuilder("m")
    iq, ix = b.input([Tq, dim]), b.input([Tk, dim])
    o = mw.grouped_query_attention(b, iq, ix, "gqa", weights, hd, Hq, Hkv, use_bias, use_gate)
    f = 2 if use_bias else 1
    W = [w.astype(np.float64) for w in weights]
    def proj(inp, idx):
        r = np.einsum("td,dhc->thc", inp.astype(np.float64), W[f * idx])
        return r + W[f * idx + 1] if use_bias else r
    Q, K, V = proj(q, 0), proj(x, 1), proj(x, 3 if use_gate else 2)
    attn = np.zeros((Tq, Hq, hd))
    for h in range(Hq):
        hk = h // (Hq // Hkv)
        attn[:, h] = np_softmax(Q[:, h] @ K[:, hk].T / np.sqrt(hd)) @ V[:, hk]
    if use_gate:
        attn = attn / (1 + np.exp(-proj(q, 2)))
    oi = f * (4 if use_gate else 3)
    want = np.einsum("thc,hco->to", attn, W[oi]) + (W[oi + 1] if use_bias else 0)
    return b.to_json([o], [[Tq, out_dim]]), [q, x], want


@pytest.mark.parametrize("use_bias,use_gate,Hkv", [(True, False, 2), (False, True, 1), (True, True, 4)])
def test_grouped_query_attention_against_numpy(use_bias, use_gate, Hkv):
    js, xs, want = gqa_model(use_bias=use_bias, use_gate=use_gate, Hkv=Hkv)
    assert_close(run_oracle(js, xs)[0], want.astype(np.float32), "gqa", rel=1e-4)


def prelu_model(H=5, W=4, C=6, seed=51):
    """PReLU with a full alpha, alpha shared over the two spatial axes, and on a rank-1 tensor."""
    rng = np.random.default_rng(seed)
    x, x1 = rng.normal(size=(H, W, C)).astype(np.float32), rng.normal(size=(C,)).astype(np.float32)
    a_full, a_ch, a1 = (rng.uniform(0.05, 0.5, size=s).astype(np.float32) for s in ((H, W, C), (1, 1, C), (C,)))
    b = mw.ModelBuilder("m")
    i, i1 = b.input([H, W, C]), b.input([C])
    outs = [mw.prelu(b, i, "full", a_full), mw.prelu(b, i, "per_channel", a_ch, shared_axes=[1, 2]), mw.prelu(b, i1, "vector", a1)]
    wants = [np.where(x > 0, x, a_full * x), np.where(x > 0, x, a_ch * x), np.where(x1 > 0, x1, a1 * x1)]
    return b.to_json(outs, [[H, W, C], [H, W, C], [C]]), [x, x1], wants


def test_prelu_against_numpy():
    js, xs, wants = prelu_model()
    for got, want in zip(run_oracle(js, xs), wants):
        assert_close(got, want, "prelu", rel=1e-6)


EINSUM_CASES = [
    # equation, input shape, kernel shape, bias axes, activation
    ("ab,bc->ac", (6,), (6, 4), None, None),
    ("abc,cd->abd", (5, 6), (6, 4), "d", "relu"),
    ("abc,cde->abde", (5, 6), (6, 3, 4), "de", None),
    ("abcd,cde->abe", (5, 3, 4), (3, 4, 7), "e", None),
    ("abc,cd->abd", (5, 6), (6, 4), "bd", None),       # bias over the sequence axis too
    ("abc,bcd->abd", (5, 6), (5, 6, 4), "d", None),    # one kernel slice per sequence position
    ("abc,dc->abd", (5, 6), (4, 6), None, "tanh"),     # kernel stored output-major
    ("abcd,abcde->abe", (2, 3, 4), (1, 2, 3, 4, 5), "e", None),
]


def einsum_model(case, seed=61):
    eq, in_shape, k_shape, bias_axes, act = case
    rng = np.random.default_rng(seed)
    x = rng.normal(size=in_shape).astype(np.float32)
    kernel = rng.normal(size=k_shape).astype(np.float32) * 0.4
    lhs, rest = eq.split(",")
    kch, rhs = rest.split("->")
    sizes = dict(zip(lhs, (1,) + tuple(in_shape)))
    sizes.update(zip(kch, k_shape))
    out_shape = [sizes[c] for c in rhs[1:]]
    bias = None
    want = np.einsum(eq, x.astype(np.float64)[None], kernel.astype(np.float64))
    if bias_axes:
        chars = [c for c in rhs if c in bias_axes]
        bias = rng.normal(size=[sizes[c] for c in chars]).astype(np.float32)
        want = want + bias.astype(np.float64).reshape([sizes[c] if c in chars else 1 for c in rhs])
    if act == "relu":
        want = np.maximum(want, 0)
    elif act == "tanh":
        want = np.tanh(want)
    b = mw.ModelBuilder("m")
    i = b.input(list(in_shape))
    o = mw.einsum_dense(b, i, "ed", eq, kernel, out_shape, bias, bias_axes, act)
    return b.to_json([o], [out_shape]), x, want[0]


@pytest.mark.parametrize("case", EINSUM_CASES, ids=[c[0] + (c[3] or "") for c in EINSUM_CASES])
def test_einsum_dense_against_numpy(case):
    js, x, want = einsum_model(case)
    got = run_oracle(js, [x])[0]
    assert got.shape == want.shape
    assert_close(got, want.astype(np.float32), "einsum " + case[0], rel=1e-4)


CONV3D_CASES = [
    # in (D, H, W, C), kernel (kd, kh, kw), Cout, strides, padding, dilation, transposed
    ((5, 6, 7, 3), (3, 3, 3), 4, 1, "valid", 1, False),
    ((5, 6, 7, 3), (3, 3, 3), 4, 1, "same", 1, False),
    ((6, 7, 9, 2), (3, 2, 3), 5, (2, 1, 2), "same", 1, False),
    ((7, 8, 9, 2), (2, 3, 3), 3, 2, "valid", 1, False),
    ((7, 8, 9, 2), (2, 3, 2), 3, 1, "valid", (2, 1, 2), False),
    ((3, 4, 5, 3), (3, 3, 3), 4, 2, "valid", 1, True),
    ((3, 4, 5, 3), (3, 3, 3), 4, 2, "same", 1, True),
    ((3, 4, 5, 2), (2, 3, 4), 3, (1, 2, 2), "same", 1, True),
    ((4, 4, 4, 2), (3, 3, 3), 3, 1, "valid", 1, True),
    # channels a multiple of 4: on the device these run without a patch matrix (filter taps walk the input slices)
    ((5, 6, 7, 4), (3, 3, 3), 8, 1, "same", 1, False),
    ((6, 9, 10, 8), (3, 2, 3), 12, (2, 1, 2), "same", 1, False),
    ((7, 8, 9, 4), (2, 3, 3), 6, 2, "valid", 1, False),
    ((7, 8, 9, 4), (2, 3, 2), 8, 1, "valid", (2, 1, 2), False),
    ((3, 20, 24, 36), (3, 3, 3), 40, 1, "same", 1, False),
    # transposed with channels a multiple of 4: one implicit product per output phase on the device (the output depth
    # must be a multiple of the depth stride: the fourth case keeps the patch matrix)
    ((3, 4, 5, 4), (3, 3, 3), 8, 2, "same", 1, True),
    ((3, 4, 5, 8), (2, 3, 4), 4, (1, 2, 2), "same", 1, True),
    ((4, 4, 4, 4), (2, 2, 2), 8, 2, "valid", 1, True),
    ((4, 4, 4, 4), (3, 3, 3), 4, 2, "valid", 1, True),
    ((4, 5, 6, 4), (3, 3, 3), 8, 1, "valid", 1, True),
    ((5, 9, 11, 16), (4, 4, 4), 12, 2, "same", 1, True),
]


def conv3d_model(case, seed=71):
    """Conv3D / Conv3DTranspose with the result of torch's float64 convolution.  SAME padding is applied by hand:
    TensorFlow's split for the forward layer; for the transposed layer the full output is cropped at
    (k - 1) - (k - 1) // 2 - ((s - 1) - (s - 1) // 2), where the reference's spread-and-pad form starts."""
    in_shape, ks, cout, strides, padding, dilation, transposed = case
    st = [strides] * 3 if isinstance(strides, int) else list(strides)
    dl = [dilation] * 3 if isinstance(dilation, int) else list(dilation)
    rng = np.random.default_rng(seed)
    cin = in_shape[3]
    x = rng.normal(size=in_shape).astype(np.float32)
    kernel = (rng.normal(size=ks + ((cout, cin) if transposed else (cin, cout))) * 0.3).astype(np.float32)
    bias = rng.normal(size=cout).astype(np.float32)
    b = mw.ModelBuilder("m")
    i = b.input(list(in_shape))
    o = mw.conv3d(b, i, "c3", kernel, bias, strides, padding, dilation, "linear", transposed)
    xt = torch.from_numpy(x).double().permute(3, 0, 1, 2)[None]
    if not transposed:
        wt = torch.from_numpy(kernel).double().permute(4, 3, 0, 1, 2)
        if padding == "same":
            pads = []
            for n, k, s_, d in reversed(list(zip(in_shape[:3], ks, st, dl))):
                ek = (k - 1) * d + 1
                total = max(ek - s_, 0) if n % s_ == 0 else max(ek - n % s_, 0)
                pads += [total // 2, total - total // 2]
            xt = F.pad(xt, pads)
        y = F.conv3d(xt, wt, torch.from_numpy(bias).double(), stride=st, dilation=dl)
    else:
        wt = torch.from_numpy(kernel).double().permute(4, 3, 0, 1, 2)  # (Cin, Cout, kd, kh, kw)
        y = F.conv_transpose3d(xt, wt, torch.from_numpy(bias).double(), stride=st)
        if padding == "same":
            sl = [slice(None), slice(None)]
            for n, k, s_ in zip(in_shape[:3], ks, st):
                c0 = (k - 1) - (k - 1) // 2 - ((s_ - 1) - (s_ - 1) // 2)
                sl.append(slice(c0, c0 + n * s_))
            y = y[tuple(sl)]
    want = y[0].permute(1, 2, 3, 0).numpy()
    return b.to_json([o], [list(want.shape)]), x, want


@pytest.mark.parametrize("case", CONV3D_CASES, ids=[f"{'T' if c[6] else 'C'}{c[1]}s{c[3]}{c[4]}d{c[5]}".replace(" ", "") for c in CONV3D_CASES])
def test_conv3d_against_torch(case):
    js, x, want = conv3d_model(case)
    got = run_oracle(js, [x])[0]
    assert got.shape == want.shape, (got.shape, want.shape)
    assert_close(got, want.astype(np.float32), "conv3d", rel=1e-4)


CONV2D_TRANSPOSE_CASES = [
    # in (H, W, C), kernel (kh, kw), Cout, strides, padding
    ((5, 6, 4), (3, 3), 8, 2, "same"),
    ((5, 6, 4), (3, 3), 8, 2, "valid"),
    ((4, 7, 8), (4, 4), 4, 2, "same"),
    ((6, 5, 4), (2, 2), 12, 2, "valid"),
    ((5, 4, 4), (5, 5), 4, 3, "same"),
    ((7, 6, 8), (3, 3), 8, 1, "same"),
    ((5, 9, 4), (3, 4), 8, (2, 1), "valid"),
    ((6, 6, 4), (5, 3), 4, (3, 2), "same"),
    ((40, 37, 16), (4, 4), 24, 2, "same"),
    ((9, 8, 6), (3, 3), 5, 2, "same"),      # channels not a multiple of 4: the gathered form on the device
    ((5, 5, 4), (1, 1), 4, 2, "valid"),     # a kernel shorter than the stride: phases without taps
]


def conv2d_transpose_model(case, seed=73):
    """Conv2DTranspose with the result of torch's float64 transposed convolution; for SAME padding the full output is
    cropped where the reference's spread-and-pad form starts (convolution.hpp:443-469), as in conv3d_model."""
    in_shape, ks, cout, strides, padding = case
    st = [strides] * 2 if isinstance(strides, int) else list(strides)
    rng = np.random.default_rng(seed)
    cin = in_shape[2]
    x = rng.normal(size=in_shape).astype(np.float32)
    kernel = (rng.normal(size=ks + (cout, cin)) * 0.3).astype(np.float32)
    bias = rng.normal(size=cout).astype(np.float32)
    b = mw.ModelBuilder("m")
    i = b.input(list(in_shape))
    o = mw.conv2d_transpose(b, i, "ct", kernel, bias, strides, padding)
    xt = torch.from_numpy(x).double().permute(2, 0, 1)[None]
    wt = torch.from_numpy(kernel).double().permute(3, 2, 0, 1)  # (Cin, Cout, kh, kw)
    y = F.conv_transpose2d(xt, wt, torch.from_numpy(bias).double(), stride=st)
    if padding == "same":
        sl = [slice(None), slice(None)]
        for n, k, s_ in zip(in_shape[:2], ks, st):
            c0 = (k - 1) - (k - 1) // 2 - ((s_ - 1) - (s_ - 1) // 2)
            sl.append(slice(c0, c0 + n * s_))
        y = y[tuple(sl)]
    want = y[0].permute(1, 2, 0).numpy()
    return b.to_json([o], [list(want.shape)]), x, want


@pytest.mark.parametrize("case", CONV2D_TRANSPOSE_CASES, ids=[f"{c[0]}k{c[1]}s{c[3]}{c[4]}".replace(" ", "") for c in CONV2D_TRANSPOSE_CASES])
def test_conv2d_transpose_against_torch(case):
    js, x, want = conv2d_transpose_model(case)
    got = run_oracle(js, [x])[0]
    assert got.shape == want.shape, (got.shape, want.shape)
    assert_close(got, want.astype(np.float32), "conv2d transpose", rel=1e-4)


def preprocessing_model(H=5, W=6, C=3, seed=81):
    """Rescaling, Normalization (per channel, one statistic, inverted, along the width) and UpSampling (1-D, 2-D nearest
    and bilinear) with float64 numpy results.  Bilinear follows Keras' half-pixel rule with edge clamping."""
    rng = np.random.default_rng(seed)
    x = rng.normal(size=(H, W, C)).astype(np.float32)
    seq = rng.normal(size=(W, C)).astype(np.float32)
    mean_c, var_c = rng.normal(size=C).astype(np.float32), rng.uniform(0.2, 2.0, size=C).astype(np.float32)
    mean_w, var_w = rng.normal(size=W).astype(np.float32), rng.uniform(0.2, 2.0, size=W).astype(np.float32)
    mean_1, var_1 = np.array([0.3], np.float32), np.array([1.7], np.float32)
    b = mw.ModelBuilder("m")
    i, i2 = b.input([H, W, C]), b.input([W, C])
    outs = [mw.rescaling(b, i, "rescale", 1.0 / 127.5, -1.0),
            mw.normalization(b, i, "norm_c", mean_c, var_c),
            mw.normalization(b, i, "norm_all", mean_1, var_1, axis=None),
            mw.normalization(b, i, "norm_inv", mean_c, var_c, invert=True),
            mw.normalization(b, i, "norm_w", mean_w, var_w, axis=2),
            mw.upsampling1d(b, i2, "up1", 3),
            mw.upsampling2d(b, i, "up_nearest", (2, 3)),
            mw.upsampling2d(b, i, "up_bilinear", (2, 3), "bilinear")]
    X = x.astype(np.float64)
    def bilinear(a, sy, sx):
        Ho, Wo = a.shape[0] * sy, a.shape[1] * sx
        yy = np.clip((np.arange(Ho) + 0.5) / sy - 0.5, 0, None)
        xx = np.clip((np.arange(Wo) + 0.5) / sx - 0.5, 0, None)
        y0, x0 = np.floor(yy).astype(int), np.floor(xx).astype(int)
        y1, x1 = np.minimum(y0 + 1, a.shape[0] - 1), np.minimum(x0 + 1, a.shape[1] - 1)
        wy1 = np.where(y1 > y0, yy - y0, 0.0)[:, None, None]
        wx1 = np.where(x1 > x0, xx - x0, 0.0)[None, :, None]
        top = a[y0][:, x0] * (1 - wx1) + a[y0][:, x1] * wx1
        bot = a[y1][:, x0] * (1 - wx1) + a[y1][:, x1] * wx1
        return top * (1 - wy1) + bot * wy1
    wants = [X / 127.5 - 1.0, (X - mean_c) / np.sqrt(var_c.astype(np.float64)), (X - 0.3) / np.sqrt(np.float64(var_1[0])),
             mean_c + X * np.sqrt(var_c.astype(np.float64)), (X - mean_w[None, :, None]) / np.sqrt(var_w.astype(np.float64))[None, :, None],
             np.repeat(seq.astype(np.float64), 3, axis=0), np.repeat(np.repeat(X, 2, axis=0), 3, axis=1), bilinear(X, 2, 3)]
    shapes = [[H, W, C]] * 5 + [[W * 3, C], [H * 2, W * 3, C], [H * 2, W * 3, C]]
    return b.to_json(outs, shapes), [x, seq], wants


def test_preprocessing_and_upsampling_against_numpy():
    js, xs, wants = preprocessing_model()
    names = ("rescale", "norm_c", "norm_all", "norm_inv", "norm_w", "up1", "up_nearest", "up_bilinear")
    for got, want, name in zip(run_oracle(js, xs), wants, names):
        assert got.shape == want.shape, name
        assert_close(got, want.astype(np.float32), name, rel=2e-6)


def repeat_crop_upsample3d_model(D=3, H=7, W=9, C=4, seed=83):
    """RepeatVector, CenterCrop (even and odd excess) and UpSampling3D (nearest) with numpy results."""
    rng = np.random.default_rng(seed)
    vol = rng.normal(size=(D, H, W, C)).astype(np.float32)
    img = rng.normal(size=(H, W, C)).astype(np.float32)
    vec = rng.normal(size=(C * 5,)).astype(np.float32)
    b = mw.ModelBuilder("m")
    iv, ii, ic = b.input([D, H, W, C]), b.input([H, W, C]), b.input([C * 5])
    outs = [mw.repeat_vector(b, ic, "repeat", 6),
            mw.center_crop(b, ii, "crop_even", H - 2, W - 4),
            mw.center_crop(b, ii, "crop_odd", H - 3, W - 1),
            mw.center_crop(b, iv, "crop_vol", H - 1, W - 5),
            mw.upsampling3d(b, iv, "up3", (2, 3, 2)),
            mw.upsampling3d(b, iv, "up3_one", (1, 1, 3))]
    def crop(a, h, w):
        t, l = (a.shape[-3] - h) // 2, (a.shape[-2] - w) // 2
        return a[..., t:t + h, l:l + w, :]
    wants = [np.tile(vec, (6, 1)), crop(img, H - 2, W - 4), crop(img, H - 3, W - 1), crop(vol, H - 1, W - 5),
             np.repeat(np.repeat(np.repeat(vol, 2, axis=0), 3, axis=1), 2, axis=2), np.repeat(vol, 3, axis=2)]
    shapes = [list(w.shape) for w in wants]
    return b.to_json(outs, shapes), [vol, img, vec], wants


def test_repeat_crop_upsample3d_against_numpy():
    js, xs, wants = repeat_crop_upsample3d_model()
    for got, want, name in zip(run_oracle(js, xs), wants, ("repeat", "crop_even", "crop_odd", "crop_vol", "up3", "up3_one")):
        assert got.shape == want.shape, name
        assert np.array_equal(got, want), name


def time_distributed_model(T=5, F=6, U=4, H=7, W=8, C=3, Co=5, seed=85):
    """TimeDistributed(Dense, relu) on (T, F) and TimeDistributed(Conv2D 3x3 same, stride 2) on (T, H, W, C), with
    float64 torch results of the wrapped layer applied to every time slice."""
    rng = np.random.default_rng(seed)
    seq = rng.normal(size=(T, F)).astype(np.float32)
    clip = rng.normal(size=(T, H, W, C)).astype(np.float32)
    kd, bd = rng.normal(size=(F, U)).astype(np.float32), rng.normal(size=U).astype(np.float32)
    kc, bc = (rng.normal(size=(3, 3, C, Co)) * 0.3).astype(np.float32), rng.normal(size=Co).astype(np.float32)
    b = mw.ModelBuilder("m")
    i1, i2 = b.input([T, F]), b.input([T, H, W, C])
    outs = [mw.time_distributed_dense(b, i1, "td_dense", kd, bd, "relu"),
            mw.time_distributed_conv2d(b, i2, "td_conv", kc, bc, strides=1, padding="valid")]
    want_d = np.maximum(seq.astype(np.float64) @ kd.astype(np.float64) + bd, 0.0)
    xt = torch.from_numpy(clip).double().permute(0, 3, 1, 2)
    wt = torch.from_numpy(kc).double().permute(3, 2, 0, 1)
    want_c = F_conv(xt, wt, torch.from_numpy(bc).double()).permute(0, 2, 3, 1).numpy()
    return b.to_json(outs, [list(want_d.shape), list(want_c.shape)]), [seq, clip], [want_d, want_c]


def F_conv(x, w, bias):
    return F.conv2d(x, w, bias)


def test_time_distributed_against_torch():
    js, xs, wants = time_distributed_model()
    for got, want, name in zip(run_oracle(js, xs), wants, ("td_dense", "td_conv")):
        assert got.shape == want.shape, name
        assert_close(got, want.astype(np.float32), name, rel=1e-5)


def test_multi_head_attention_against_torch():
    rng = np.random.default_rng(9)
    Tq, Tk, dim, H, dk = 3, 5, 8, 2, 4
    ws = []
    for _ in range(3):
        ws += [rng.normal(size=(dim, H, dk)).astype(np.float32) * 0.5, rng.normal(size=(H, dk)).astype(np.float32) * 0.1]
    ws += [rng.normal(size=(H, dk, dim)).astype(np.float32) * 0.5, rng.normal(size=dim).astype(np.float32) * 0.1]
    q = rng.normal(size=(Tq, dim)).astype(np.float32)
    v = rng.normal(size=(Tk, dim)).astype(np.float32)
    b = mw.ModelBuilder("m")
    qi, vi = b.input([Tq, dim]), b.input([Tk, dim])
    o = mw.multi_head_attention(b, qi, vi, "mha", ws, H, dk)
    got = run_oracle(b.to_json([o], [[Tq, dim]]), [q, v])[0]
    t = [torch.from_numpy(w).double() for w in ws]
    qt, vt = torch.from_numpy(q).double(), torch.from_numpy(v).double()
    Q = torch.einsum("td,dhk->htk", qt, t[0]) + t[1][:, None, :]
    K = torch.einsum("td,dhk->htk", vt, t[2]) + t[3][:, None, :]
    V = torch.einsum("td,dhk->htk", vt, t[4]) + t[5][:, None, :]
    A = F.scaled_dot_product_attention(Q[None], K[None], V[None])[0]      # (H, Tq, dk)
    want = torch.einsum("htk,hkd->td", A, t[6]) + t[7]
    assert_close(got, want.numpy().astype(np.float32), "mha", rel=1e-4)


def test_hand_computed_cases():
    # 2x2 input, 2x2 'valid' kernel of ones, bias 0.5 -> one output = sum + 0.5
    b = mw.ModelBuilder("m")
    i = b.input([2, 2, 1])
    o = mw.conv2d(b, i, "c", np.ones((2, 2, 1, 1), np.float32), np.array([0.5], np.float32))
    got = run_oracle(b.to_json([o], [[1, 1, 1]]), [np.array([[[1.], [2.]], [[3.], [4.]]], np.float32)])[0]
    assert got.shape == (1, 1, 1) and got[0, 0, 0] == 10.5
    # ReLU with max_value 6, slope 0.1, threshold 1 (relu_layer.hpp:40-46)
    b = mw.ModelBuilder("m")
    i = b.input([4])
    o = mw.relu(b, i, "r", max_value=6.0, negative_slope=0.1, threshold=1.0)
    got = run_oracle(b.to_json([o], [[4]]), [np.array([-1.0, 0.5, 3.0, 7.0], np.float32)])[0]
    np.testing.assert_allclose(got, np.array([-0.2, -0.05, 3.0, 6.0], np.float32), rtol=1e-6)
    # average pooling 'same' divides by the valid count: corner of a 2x2 window at the border
    b = mw.ModelBuilder("m")
    i = b.input([3, 3, 1])
    o = mw.avg_pool2d(b, i, "p", 2, 2, "same")
    x = np.arange(9, dtype=np.float32).reshape(3, 3, 1)
    got = run_oracle(b.to_json([o], [[2, 2, 1]]), [x])[0]
    np.testing.assert_allclose(got[..., 0], np.array([[2.0, 3.5], [6.5, 8.0]], np.float32))
    # embedding truncates float ids
    b = mw.ModelBuilder("m")
    i = b.input([3])
    o = mw.embedding(b, i, "e", np.arange(8, dtype=np.float32).reshape(4, 2))
    got = run_oracle(b.to_json([o], [[3, 2]]), [np.array([0.0, 3.9, 1.2], np.float32)])[0]
    np.testing.assert_array_equal(got, np.array([[0, 1], [6, 7], [2, 3]], np.float32))


def test_oracle_errors_mirror_the_reference():
    js = mw.build_small_cnn()
    m = OracleModel(json_text=model_text(js))
    with pytest.raises(RuntimeError):
        m.predict([np.zeros((31, 32, 3), np.float32)])  # wrong input shape (model.hpp:137-139)
    bad = json.loads(model_text(js))
    bad["image_data_format"] = "channels_first"
    with pytest.raises(RuntimeError, match="channels_last"):
        OracleModel(json_text=json.dumps(bad))
    bad = json.loads(model_text(js))
    bad["architecture"]["config"]["layers"][1]["class_name"] = "NoSuchLayer"
    with pytest.raises(RuntimeError, match="unknown layer type"):
        OracleModel(json_text=json.dumps(bad))
    b = mw.ModelBuilder("m")
    i = b.input([2])
    o = mw.embedding(b, i, "e", np.zeros((4, 2), np.float32))
    m = OracleModel(json_text=model_text(b.to_json([o], [[2, 2]])))
    with pytest.raises(RuntimeError, match="strictly less"):
        m.predict([np.array([1.0, 4.0], np.float32)])


def test_predict_multi_matches_predict_and_keeps_order():
    js = mw.build_small_cnn()
    m = OracleModel(json_text=model_text(js))
    x = mw.inputs_small_cnn(6)
    multi = m.predict_multi([[x[i]] for i in range(6)], threads=3)
    for i in range(6):
        np.testing.assert_array_equal(multi[i][0], m.predict([x[i]])[0])


def test_golden_fixtures():
    """Committed fixtures (tests/golden/make_golden.py): model JSON + inputs + oracle outputs."""
    files = sorted(glob.glob(os.path.join(HERE, "golden", "*.npz")))
    assert files, "no golden fixtures found"
    for f in files:
        z = np.load(f, allow_pickle=False)
        text = bytes(z["model_json"]).decode()
        m = OracleModel(json_text=text)
        n_in, n_out, ns = int(z["n_in"]), int(z["n_out"]), int(z["n_samples"])
        for s in range(ns):
            outs = m.predict([z[f"in_{s}_{i}"] for i in range(n_in)])
            for o in range(n_out):
                assert_close(outs[o], z[f"out_{s}_{o}"], f"{os.path.basename(f)} sample {s} output {o}", rel=1e-6)
        m.run_tests(1e-5)  # the embedded self test, like load_model(verify=true) with the tests' epsilon


# ---------------------------------------------------------------------------------------------------------
# Layer classes beyond the benchmark configurations: Resizing, Dot, adaptive pooling, the remaining
# activation classes, the preprocessing look-ups, and the augmentation names that pass through.
# ---------------------------------------------------------------------------------------------------------
def more_layers_model(H=9, W=7, C=3):
    """One model exercising the classes above; returns (json, inputs, expected outputs from numpy / torch in float64
    where an independent formula exists, else None)."""
    import torch
    rng = np.random.default_rng(41)
    b = mw.ModelBuilder("more_layers")
    img = b.input([H, W, C])
    vec_a = b.input([5, 6])
    vec_b = b.input([6, 4])
    ids = b.input([7])
    x_img = rng.normal(size=(H, W, C)).astype(np.float32)
    x_a = rng.normal(size=(5, 6)).astype(np.float32)
    x_b = rng.normal(size=(6, 4)).astype(np.float32)
    x_ids = np.array([3, 0, 12, 7, 3, 9, 100], np.float32)
    outs, shapes, wants = [], [], []
    t = torch.from_numpy(x_img.astype(np.float64)).permute(2, 0, 1)[None]

    def add(ref, shape, want):
        outs.append(ref); shapes.append(shape); wants.append(want)

    # Resizing: bilinear and nearest against torch's half-pixel interpolation, area against adaptive averaging where the
    # target divides the input, plus an upscale and the cropping form
    add(mw.resizing(b, img, "rs_bilinear", 13, 10, "bilinear"), [13, 10, C],
        torch.nn.functional.interpolate(t, size=(13, 10), mode="bilinear", align_corners=False)[0].permute(1, 2, 0).numpy())
    add(mw.resizing(b, img, "rs_nearest", 2 * H, 2 * W, "nearest"), [2 * H, 2 * W, C], np.repeat(np.repeat(x_img, 2, axis=0), 2, axis=1).astype(np.float64))
    add(mw.resizing(b, img, "rs_area", 3, W, "area"), [3, W, C], x_img.astype(np.float64).reshape(3, H // 3, W, C).mean(axis=1) if H % 3 == 0 else None)
    add(mw.resizing(b, img, "rs_area_up", 12, 9, "area"), [12, 9, C], None)
    add(mw.resizing(b, img, "rs_crop", 4, 6, "bilinear", crop_to_aspect_ratio=True), [4, 6, C], None)
    add(mw.center_crop(b, img, "cc_small_input", H + 3, W + 5), [H + 3, W + 5, C], None)
    # Dot: matrix product, the same normalised, and a contraction of the first axes
    add(mw.dot(b, [vec_a, vec_b], "dot_mm", [2, 1]), [5, 4], x_a.astype(np.float64) @ x_b.astype(np.float64))
    na = x_a.astype(np.float64) / np.sqrt((x_a.astype(np.float64) ** 2).sum(axis=1, keepdims=True))
    nb = x_b.astype(np.float64) / np.sqrt((x_b.astype(np.float64) ** 2).sum(axis=0, keepdims=True))
    add(mw.dot(b, [vec_a, vec_b], "dot_norm", [2, 1], normalize=True), [5, 4], na @ nb)
    add(mw.dot(b, [img, img], "dot_first", 1), [W, C, W, C], np.einsum("hwc,hxd->wcxd", x_img.astype(np.float64), x_img.astype(np.float64)))
    # adaptive pooling against torch
    add(mw.adaptive_pooling(b, img, "ap_avg2", "AdaptiveAveragePooling2D", [4, 3]), [4, 3, C],
        torch.nn.functional.adaptive_avg_pool2d(t, (4, 3))[0].permute(1, 2, 0).numpy())
    add(mw.adaptive_pooling(b, img, "ap_max2", "AdaptiveMaxPooling2D", [5, 7]), [5, 7, C],
        torch.nn.functional.adaptive_max_pool2d(t, (5, 7))[0].permute(1, 2, 0).numpy())
    add(mw.adaptive_pooling(b, vec_a, "ap_avg1", "AdaptiveAveragePooling1D", 2), [2, 6],
        torch.nn.functional.adaptive_avg_pool1d(torch.from_numpy(x_a.astype(np.float64)).T[None], 2)[0].T.numpy())
    # activation classes
    xa = x_a.astype(np.float64)
    add(mw.activation_layer(b, vec_a, "act_threshold", "Threshold", threshold=0.2, default_value=-3.0), [5, 6], np.where(xa > 0.2, xa, -3.0))
    add(mw.activation_layer(b, vec_a, "act_hard_shrink", "HardShrink", threshold=0.5), [5, 6], np.where(np.abs(xa) > 0.5, xa, 0.0))
    add(mw.activation_layer(b, vec_a, "act_soft_shrink", "SoftShrink", threshold=0.5), [5, 6],
        np.where(xa > 0.5, xa - 0.5, np.where(xa < -0.5, xa + 0.5, 0.0)))
    add(mw.activation_layer(b, vec_a, "act_sparse_plus", "SparsePlus"), [5, 6], np.where(xa <= -1, 0.0, np.where(xa < 1, 0.25 * (xa + 1) ** 2, xa)))
    add(mw.activation_layer(b, vec_a, "act_squareplus", "Squareplus", b=4.0), [5, 6], (xa + np.sqrt(xa * xa + 4.0)) / 2)
    add(mw.dense(b, vec_a, "dense_soft_shrink", rng.normal(size=(6, 3)).astype(np.float32), None, "sparse_plus"), [5, 3], None)
    # augmentation layers pass through
    add(mw.activation_layer(b, mw.activation_layer(b, vec_a, "aug_a", "RandAugment"), "aug_b", "RandomFlip"), [5, 6], xa)
    # preprocessing look-ups
    add(mw.discretization(b, vec_a, "disc", [-1.0, -0.25, 0.0, 0.5]), [5, 6], np.searchsorted(np.array([-1.0, -0.25, 0.0, 0.5]), xa, side="right").astype(np.float64))
    vocab = [12, 3, 7, 40]
    add(mw.integer_lookup(b, ids, "lookup", vocab), [7], np.array([vocab.index(int(v)) + 1 if int(v) in vocab else 0 for v in x_ids], np.float64))
    add(mw.integer_lookup(b, ids, "lookup_mask", vocab, mask_token=0), [7],
        np.array([0 if int(v) == 0 else (vocab.index(int(v)) + 2 if int(v) in vocab else 1) for v in x_ids], np.float64))
    small_ids = b.input([4])
    x_small = np.array([2.0, 5.7, 2.2, 0.0], np.float32)
    add(mw.category_encoding(b, small_ids, "cat_multi", 8, "multi_hot"), [8], np.array([1, 0, 1, 0, 0, 1, 0, 0], np.float64))
    add(mw.category_encoding(b, small_ids, "cat_count", 8, "count"), [8], np.array([1, 0, 2, 0, 0, 1, 0, 0], np.float64))
    one_id = b.input([1])
    add(mw.category_encoding(b, one_id, "cat_one", 5, "one_hot"), [5], np.array([0, 0, 0, 1, 0], np.float64))
    return b.to_json(outs, shapes), [x_img, x_a, x_b, x_ids, x_small, np.array([3.0], np.float32)], wants


def test_more_layer_classes_against_numpy_and_torch(built_library):
    js, xs, wants = more_layers_model()
    got = OracleModel(json_text=model_text(js)).predict(xs)
    assert len(got) == len(wants)
    for k, (g, w) in enumerate(zip(got, wants)):
        assert np.isfinite(g).all(), f"output {k}"
        if w is not None:
            assert g.shape == w.shape, f"output {k}: {g.shape} != {w.shape}"
            np.testing.assert_allclose(g, w, rtol=2e-5, atol=2e-6, err_msg=f"output {k}")


def test_category_encoding_rejects_values_outside(built_library):
    b = mw.ModelBuilder("m")
    i = b.input([3])
    js = b.to_json([mw.category_encoding(b, i, "cat", 4, "count")], [[4]])
    m = OracleModel(json_text=model_text(js))
    m.predict([np.array([0.0, 3.9, 1.0], np.float32)])
    with pytest.raises(RuntimeError, match="num_tokens"):
        m.predict([np.array([0.0, 4.0, 1.0], np.float32)])


def test_restatement_against_the_reference_itself(built_library):
    """When the reference could be compiled (oracle/build_ref.py found Eigen and FunctionalPlus), the restatement must
    agree with it on every golden fixture: this is what pins the oracle.  Skipped where the reference is not built."""
    import build_ref
    exe = build_ref.build(verbose=False)
    if exe is None:
        pytest.skip("the reference is not built here (Eigen 3.4.0 / FunctionalPlus 0.2.24 missing): parity stays unpinned")
    assert build_ref.compare_golden(exe) == 0


def test_double_precision_arbiter_agrees_with_the_fp32_oracle(built_library):
    """The oracle built with real = double (the reference's FDEEP_FLOAT_TYPE = double) is the arbiter that separates
    fp32 rounding noise from real differences: on every golden fixture and on reduced versions of the benchmark
    models the fp32 oracle must sit within 1e-5 of it (same algorithms, same weights, only the arithmetic type differs)."""
    from util import arbiter_outputs, oracle_outputs, worst_relative
    cases = []
    for f in sorted(glob.glob(os.path.join(HERE, "golden", "*.npz"))):
        z = np.load(f, allow_pickle=False)
        n_in, ns = int(z["n_in"]), int(z["n_samples"])
        cases.append((os.path.basename(f), bytes(z["model_json"]).decode(), [[z[f"in_{s}_{i}"] for i in range(n_in)] for s in range(ns)]))
    x = mw.inputs_resnet50(2, size=64)
    cases.append(("resnet50/64px", model_text(mw.build_resnet50(size=64, width=16, classes=10, top="linear")), [[x[i]] for i in range(2)]))
    x = mw.inputs_small_cnn(8)
    cases.append(("small_cnn", model_text(mw.build_small_cnn()), [[x[i]] for i in range(8)]))
    for name, text, samples in cases:
        a, b = oracle_outputs(text, samples), arbiter_outputs(text, samples)
        for s in range(len(samples)):
            for o in range(len(a[s])):
                assert b[s][o].dtype == np.float64
                w = worst_relative(a[s][o], b[s][o])
                assert w <= 1e-5, f"{name} sample {s} output {o}: fp32 oracle is {w:.2e} from the double-precision one"


# ---------------------------------------------------------------------------------------------------------
# Convolutional LSTM (conv_lstm_2d_layer.hpp): the oracle against a float64 torch loop.
# ---------------------------------------------------------------------------------------------------------
def conv_lstm_case(rank, T, spatial, cin, filters, kernel, strides=1, padding="same", dilation=1, return_sequences=True,
                   return_state=False, activation="tanh", recurrent_activation="sigmoid", use_bias=True, seed=3):
    """Returns (json, input, expected outputs) for one ConvLSTM1D/2D layer; the expectation is a plain float64 loop over the
    time steps with torch's conv2d (gates i, f, c, o; Keras' definition of the layer)."""
    import torch
    import torch.nn.functional as F
    rng = np.random.default_rng(seed)
    ks = (kernel,) * rank if isinstance(kernel, int) else tuple(kernel)
    k_in = (rng.normal(size=ks + (cin, 4 * filters)) * 0.3).astype(np.float32)
    k_rec = (rng.normal(size=ks + (filters, 4 * filters)) * 0.3).astype(np.float32)
    bias = (rng.normal(size=(4 * filters,)) * 0.2).astype(np.float32) if use_bias else None
    sp = (spatial,) * rank if isinstance(spatial, int) else tuple(spatial)
    x = rng.normal(size=(T,) + sp + (cin,)).astype(np.float32)
    b = mw.ModelBuilder("conv_lstm")
    i = b.input([T, *sp, cin])
    refs = mw.conv_lstm(b, i, "cl", k_in, k_rec, bias, strides=strides, padding=padding, dilation=dilation,
                        return_sequences=return_sequences, return_state=return_state, activation=activation,
                        recurrent_activation=recurrent_activation)
    refs = refs if isinstance(refs, list) else [refs]

    def as4(k):  # (kh, kw, Cin, Cout) -> torch (Cout, Cin, kh, kw)
        if k.ndim == 3:
            k = k[None]
        return torch.tensor(k.astype(np.float64)).permute(3, 2, 0, 1)
    st = (1, strides) if rank == 1 and isinstance(strides, int) else ((strides, strides) if isinstance(strides, int) else tuple(strides))
    dl = (1, dilation) if rank == 1 and isinstance(dilation, int) else ((dilation, dilation) if isinstance(dilation, int) else tuple(dilation))
    kh, kw = (1, ks[0]) if rank == 1 else ks
    acts = {"tanh": torch.tanh, "sigmoid": torch.sigmoid, "relu": torch.relu,
            "hard_sigmoid": lambda v: torch.clamp(v / 6.0 + 0.5, 0.0, 1.0)}
    act, ract = acts[activation], acts[recurrent_activation]

    def conv(img, w, bias_, stride, dil, pad):  # img (H, W, C) float64
        H, W = img.shape[0], img.shape[1]
        t = img.permute(2, 0, 1)[None]
        if pad == "same":  # TensorFlow's rule: total = max((ceil(n/s)-1)*s + (k-1)*d + 1 - n, 0), smaller half first
            ph = max((-(-H // stride[0]) - 1) * stride[0] + (kh - 1) * dil[0] + 1 - H, 0)
            pw = max((-(-W // stride[1]) - 1) * stride[1] + (kw - 1) * dil[1] + 1 - W, 0)
            t = F.pad(t, (pw // 2, pw - pw // 2, ph // 2, ph - ph // 2))
        r = F.conv2d(t, w, bias_, stride=stride, dilation=dil)
        return r[0].permute(1, 2, 0)
    wi, wr = as4(k_in), as4(k_rec)
    bt = torch.tensor(bias.astype(np.float64)) if bias is not None else None
    xt = torch.tensor(x.astype(np.float64))
    if rank == 1:
        xt = xt[:, None]
    h = c = None
    seq = []
    for t in range(T):
        z = conv(xt[t], wi, bt, st, dl, padding)
        if h is None:
            h = torch.zeros(z.shape[0], z.shape[1], filters, dtype=torch.float64)
            c = torch.zeros_like(h)
        z = z + conv(h, wr, None, (1, 1), (1, 1), "same")
        zi, zf, zc, zo = torch.split(z, filters, dim=-1)
        c = ract(zf) * c + ract(zi) * act(zc)
        h = ract(zo) * act(c)
        seq.append(h)

    def state(v):
        return (v[0] if rank == 1 else v).numpy()
    wants = [np.stack([state(v) for v in seq]) if return_sequences else state(h)]
    if return_state:
        wants += [state(h), state(c)]
    js = b.to_json(refs, [list(w.shape) for w in wants])
    return js, x, wants


CONV_LSTM_CASES = [
    dict(rank=2, T=4, spatial=(6, 5), cin=3, filters=4, kernel=3, padding="same", return_sequences=True, return_state=True),
    dict(rank=2, T=3, spatial=(9, 8), cin=2, filters=5, kernel=(3, 2), strides=2, padding="valid", return_sequences=False),
    dict(rank=2, T=3, spatial=(7, 7), cin=3, filters=3, kernel=3, dilation=2, padding="same", return_sequences=True, use_bias=False,
         activation="relu", recurrent_activation="hard_sigmoid"),
    dict(rank=1, T=5, spatial=11, cin=4, filters=6, kernel=3, padding="same", return_sequences=True),
    dict(rank=1, T=4, spatial=12, cin=3, filters=4, kernel=4, strides=2, padding="valid", return_sequences=False, return_state=True),
    dict(rank=2, T=1, spatial=(4, 4), cin=1, filters=2, kernel=1, padding="valid", return_sequences=True),
]


@pytest.mark.parametrize("case", range(len(CONV_LSTM_CASES)))
def test_oracle_conv_lstm_matches_float64_loop(built_library, case):
    js, x, wants = conv_lstm_case(**CONV_LSTM_CASES[case])
    got = run_oracle(js, [x])
    assert len(got) == len(wants)
    for g, w in zip(got, wants):
        assert g.shape == w.shape
        np.testing.assert_allclose(g, w, rtol=2e-5, atol=2e-6)
