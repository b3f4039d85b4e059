"""One NeoML transformer encoder layer written as the sequence of IMathEngine calls its layers make
(CTransformerEncoderLayer, post-norm: NeoML/src/Dnn/Layers/TransformerLayer.cpp:249-329; attention
MultiheadAttentionLayer.cpp:261-378; layer norm ObjectNormalizationLayer.cpp:190-241; GELU in its default
sigmoid-approximation form, ActivationDesc.h:86-100).  `e` is any object with the method names of oracle_lib
(the plain-C oracle, the reference CPU engine, or the B200 engine behind the shim), so the same call sequence runs on
the checker and on the device; tensors stay whatever type `e` works on (numpy arrays or torch CUDA tensors)."""
import numpy as np

import cases

MULTIPLY, NEG_MULTIPLY, ADD_VALUE, ADD, ELTWISE_MUL, SIGMOID, SQRT, INV = 6, 7, 8, 3, 5, 10, 11, 12


def make_weights(seed: int, hidden: int, ffn: int, std: float = 0.02):
    w = {}
    for i, name in enumerate(("q", "k", "v", "o")):
        w[name + ".w"] = cases.normal(seed + 2 * i, (hidden, hidden), std)
        w[name + ".b"] = cases.uniform(seed + 2 * i + 1, (hidden,), -0.1, 0.1)
    w["ffn1.w"], w["ffn1.b"] = cases.normal(seed + 10, (ffn, hidden), std), cases.uniform(seed + 11, (ffn,), -0.1, 0.1)
    w["ffn2.w"], w["ffn2.b"] = cases.normal(seed + 12, (hidden, ffn), std), cases.uniform(seed + 13, (hidden,), -0.1, 0.1)
    for i, name in enumerate(("norm1", "norm2")):
        w[name + ".scale"] = cases.uniform(seed + 20 + 2 * i, (hidden,), 0.5, 1.5)
        w[name + ".bias"] = cases.uniform(seed + 21 + 2 * i, (hidden,), -0.2, 0.2)
    return w


def _linear(e, x, rows, w, b):
    y = e.multiply_matrix_by_transposed_matrix(x.reshape(rows, w.shape[1]), w)
    return e.add_vector_to_matrix_rows(1, y.reshape(-1), rows, w.shape[0], b)


def _layer_norm(e, x, rows, width, scale, bias, eps=1e-5):
    neg_mean = e.vector_op(NEG_MULTIPLY, e.sum_matrix_columns(x, rows, width), None, 1.0 / width)
    t = e.add_vector_to_matrix_columns(x, rows, width, neg_mean)
    t = e.vector_op(ELTWISE_MUL, t, t)
    inv = e.vector_op(MULTIPLY, e.sum_matrix_columns(t, rows, width), None, 1.0 / width)
    inv = e.vector_op(INV, e.vector_op(SQRT, e.vector_op(ADD_VALUE, inv, None, eps)))
    norm = e.add_vector_to_matrix_columns(x, rows, width, neg_mean)
    norm = e.multiply_diag_matrix_by_matrix(inv, rows, norm, width)
    out = e.multiply_matrix_by_diag_matrix(1, norm, rows, width, scale, 0)
    return e.add_vector_to_matrix_rows(1, out, rows, width, bias)


def encoder_layer(e, x, w, mask, batch: int, seq: int, hidden: int, heads: int):
    """x: flat [batch*seq*hidden]; mask: flat [seq*seq], 1 = blocked (multiplied by -1e9 and added to the scores,
    as CMultiheadAttentionLayer does).  Returns the flat layer output."""
    d = hidden // heads
    rows = batch * seq
    q = _linear(e, x, rows, w["q.w"], w["q.b"])
    k = _linear(e, x, rows, w["k.w"], w["k.b"])
    v = _linear(e, x, rows, w["v.w"], w["v.b"])
    q = e.transpose_matrix(batch, q, seq, 1, heads, d)            # [B,S,heads,d] -> [B,heads,S,d]
    v = e.transpose_matrix(batch, v, seq, 1, heads, d)
    kt = e.transpose_matrix(batch, k, seq, 1, hidden, 1)          # [B,S,hidden] -> [B,heads*d,S]
    scores = e.multiply_matrix_by_matrix(q.reshape(batch * heads, seq, d), kt.reshape(batch * heads, d, seq))
    scores = e.vector_op(MULTIPLY, scores.reshape(-1), None, 1.0 / float(np.sqrt(d)))
    blocked = e.vector_op(MULTIPLY, mask, None, -1e9)
    scores = e.add_vector_to_matrix_rows(1, scores, batch * heads, seq * seq, blocked)
    probs = e.matrix_softmax_by_rows(scores, batch * heads * seq, seq)
    ctx = e.multiply_matrix_by_matrix(probs.reshape(batch * heads, seq, seq), v.reshape(batch * heads, seq, d))
    ctx = e.transpose_matrix(batch, ctx.reshape(-1), heads, 1, seq, d)   # [B,heads,S,d] -> [B,S,heads,d]
    attn = _linear(e, ctx, rows, w["o.w"], w["o.b"])
    y = _layer_norm(e, e.vector_op(ADD, x, attn), rows, hidden, w["norm1.scale"], w["norm1.bias"])
    h = _linear(e, y, rows, w["ffn1.w"], w["ffn1.b"])
    gate = e.vector_op(SIGMOID, e.vector_op(MULTIPLY, h, None, 1.702))
    h = e.vector_op(ELTWISE_MUL, h, gate)
    o = _linear(e, h, rows, w["ffn2.w"], w["ffn2.b"])
    return _layer_norm(e, e.vector_op(ADD, y, o), rows, hidden, w["norm2.scale"], w["norm2.bias"])


def make_inputs(seed: int, batch: int, seq: int, hidden: int):
    x = cases.normal(seed, (batch * seq * hidden,), 1.0)
    # a causal mask (1 above the diagonal = blocked): every row keeps at least one open position
    mask = np.triu(np.ones((seq, seq), np.float32), k=1).reshape(-1)
    return x, mask
