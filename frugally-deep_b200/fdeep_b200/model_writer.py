"""Keras-free writer for frugally-deep's converted-JSON model format.

The reference produces these files with keras_export/convert_model.py
(model_to_fdeep_json, convert_model.py:971-1001), which needs Keras/TensorFlow.
This module writes the same on-disk contract from numpy alone: a Keras-3 style
functional ``architecture`` plus ``trainable_params`` in the exporter's weight
layouts (convert_model.py:197-236, 429-470, 600-631), floats encoded as
little-endian float32 -> base64 -> 1024-character chunks (convert_model.py:187-194).

It also holds the builders for the five benchmark workloads (small CNN,
ResNet-50, MobileNetV2, text LSTM, GPT-2-small-shaped incremental decoder)
with seeded synthetic weights.  No pretrained weights and no dataset items are
involved anywhere.
"""
from __future__ import annotations

import base64
import hashlib
import json
from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np


def encode_floats(arr: np.ndarray) -> List[str]:
    """float32 bytes -> base64 -> 1024-char chunks (convert_model.py:187-194)."""
    s = base64.b64encode(np.ascontiguousarray(arr, dtype=np.float32).tobytes()).decode("ascii")
    return [s[i:i + 1024] for i in range(0, len(s), 1024)] or [""]


def show_tensor(arr: np.ndarray) -> dict:
    """Test-case tensor: shape without the batch dim + encoded values (convert_model.py:58-65)."""
    return {"shape": list(arr.shape), "values": encode_floats(arr.reshape(-1))}


Ref = Tuple[str, int, int]  # (layer name, node index, tensor index)


class ModelBuilder:
    """Accumulates layers of a functional model and emits the fdeep JSON dict."""

    def __init__(self, name: str = "model"):
        self.name = name
        self.layers: List[dict] = []
        self.params: Dict[str, dict] = {}
        self.inputs: List[Ref] = []
        self.input_shapes: List[list] = []
        self._layer_index: Dict[str, dict] = {}
        self._hash = hashlib.sha256()

    # -- graph construction -------------------------------------------------
    def input(self, shape: Sequence[Optional[int]], name: Optional[str] = None) -> Ref:
        name = name or f"input_{len(self.inputs)}"
        layer = {
            "class_name": "InputLayer",
            "name": name,
            "config": {"batch_shape": [None] + list(shape), "dtype": "float32", "name": name},
            "inbound_nodes": [],
        }
        self.layers.append(layer)
        self._layer_index[name] = layer
        ref = (name, 0, 0)
        self.inputs.append(ref)
        self.input_shapes.append(list(shape))
        return ref

    def add(self, class_name: str, name: str, config: dict,
            inputs: Union[Ref, Sequence[Ref]], params: Optional[dict] = None,
            n_outputs: int = 1) -> Union[Ref, List[Ref]]:
        """Add a layer application.  Calling it again with an existing ``name``
        adds another inbound node to the same (shared) layer."""
        if isinstance(inputs, tuple) and len(inputs) == 3 and isinstance(inputs[0], str):
            arg_list = [self._tensor_arg(inputs)]
        else:
            arg_list = [[self._tensor_arg(r) for r in inputs]]
        node = {"args": arg_list, "kwargs": {}}
        if name in self._layer_index:
            layer = self._layer_index[name]
            layer["inbound_nodes"].append(node)
        else:
            cfg = dict(config)
            cfg.setdefault("name", name)
            layer = {"class_name": class_name, "name": name, "config": cfg, "inbound_nodes": [node]}
            self.layers.append(layer)
            self._layer_index[name] = layer
            if params:
                enc = {}
                for k, v in params.items():
                    enc[k] = self._encode_param(v)
                self.params[name] = enc
            self._hash.update(name.encode("ascii"))
        node_idx = len(layer["inbound_nodes"]) - 1
        if n_outputs == 1:
            return (name, node_idx, 0)
        return [(name, node_idx, i) for i in range(n_outputs)]

    def _encode_param(self, v):
        if isinstance(v, np.ndarray):
            self._hash.update(np.ascontiguousarray(v, dtype=np.float32).tobytes())
            return encode_floats(v.reshape(-1))
        if isinstance(v, (list, tuple)) and v and isinstance(v[0], np.ndarray):
            return [self._encode_param(a) for a in v]
        return v  # plain json (shape lists, scalars)

    @staticmethod
    def _tensor_arg(ref: Ref) -> dict:
        return {"class_name": "__keras_tensor__",
                "config": {"keras_history": [ref[0], int(ref[1]), int(ref[2])]}}

    # -- emission -----------------------------------------------------------
    def to_json(self, outputs: Sequence[Ref], output_shapes: Sequence[Sequence[Optional[int]]],
                tests: Optional[List[dict]] = None) -> dict:
        def conn(r: Ref):
            return [r[0], int(r[1]), int(r[2])]
        in_l = [conn(r) for r in self.inputs]
        out_l = [conn(r) for r in outputs]
        arch = {
            "class_name": "Functional",
            "config": {
                "name": self.name,
                "layers": self.layers,
                # Keras writes a single connection as a flat triple.
                "input_layers": in_l[0] if len(in_l) == 1 else in_l,
                "output_layers": out_l[0] if len(out_l) == 1 else out_l,
            },
        }
        out = {
            "architecture": arch,
            "image_data_format": "channels_last",
            "input_shapes": [list(s) for s in self.input_shapes],
            "output_shapes": [list(s) for s in output_shapes],
            "trainable_params": self.params,
            "hash": self._hash.hexdigest(),
        }
        if tests:
            out["tests"] = tests
        return out


def write_json(model_json: dict, path: str) -> None:
    with open(path, "w") as f:
        json.dump(model_json, f, allow_nan=False, separators=(",", ":"))


# ---------------------------------------------------------------------------
# Seeded initialisers (numpy PCG64; drawn in layer order, weights before biases)
# ---------------------------------------------------------------------------
class Init:
    def __init__(self, seed: int):
        self.rng = np.random.default_rng(seed)

    def glorot_uniform(self, shape, fan_in, fan_out):
        lim = np.sqrt(6.0 / (fan_in + fan_out))
        return self.rng.uniform(-lim, lim, size=shape).astype(np.float32)

    def he_normal(self, shape, fan_in):
        std = np.sqrt(2.0 / fan_in)
        x = self.rng.normal(0.0, 1.0, size=shape)
        bad = np.abs(x) > 2.0
        while bad.any():  # truncate to +-2 sigma by resampling
            x[bad] = self.rng.normal(0.0, 1.0, size=int(bad.sum()))
            bad = np.abs(x) > 2.0
        return (x * std).astype(np.float32)

    def normal(self, shape, std, mean=0.0):
        return self.rng.normal(mean, std, size=shape).astype(np.float32)

    def uniform(self, shape, lo, hi):
        return self.rng.uniform(lo, hi, size=shape).astype(np.float32)

    def orthogonal(self, rows, cols):
        a = self.rng.normal(0.0, 1.0, size=(max(rows, cols), min(rows, cols)))
        q, r = np.linalg.qr(a)
        q = q * np.sign(np.diag(r))
        if rows < cols:
            q = q.T
        return q[:rows, :cols].astype(np.float32)


# ---------------------------------------------------------------------------
# Layer helpers: Keras weights in, exporter layouts out
# ---------------------------------------------------------------------------
def _pair(v):
    return [v, v] if isinstance(v, int) else list(v)


def conv2d(b: ModelBuilder, x: Ref, name: str, kernel: np.ndarray, bias: Optional[np.ndarray],
           strides=1, padding="valid", dilation=1, activation="linear") -> Ref:
    """kernel in Keras layout (kh, kw, Cin, Cout); stored as (Cout, kh, kw, Cin)."""
    kh, kw, _, cout = kernel.shape
    cfg = {"filters": int(cout), "kernel_size": [int(kh), int(kw)], "strides": _pair(strides),
           "padding": padding, "data_format": "channels_last", "dilation_rate": _pair(dilation),
           "groups": 1, "activation": activation, "use_bias": bias is not None}
    params = {"weights": np.moveaxis(kernel, [0, 1, 2, 3], [1, 2, 3, 0])}
    if bias is not None:
        params["bias"] = bias
    return b.add("Conv2D", name, cfg, x, params)


def conv2d_transpose(b: ModelBuilder, x: Ref, name: str, kernel: np.ndarray, bias: Optional[np.ndarray], strides=1, padding="valid",
                     activation="linear") -> Ref:
    """Conv2DTranspose with the kernel in Keras layout (kh, kw, Cout, Cin); stored as (Cout, kh, kw, Cin)."""
    kh, kw, cout, _ = kernel.shape
    cfg = {"filters": int(cout), "kernel_size": [int(kh), int(kw)], "strides": _pair(strides), "padding": padding,
           "data_format": "channels_last", "dilation_rate": [1, 1], "groups": 1, "activation": activation, "use_bias": bias is not None}
    params = {"weights": np.ascontiguousarray(np.moveaxis(kernel, [0, 1, 2, 3], [1, 2, 0, 3]))}
    if bias is not None:
        params["bias"] = bias
    return b.add("Conv2DTranspose", name, cfg, x, params)


def _triple(v):
    return [int(v)] * 3 if isinstance(v, int) else [int(a) for a in v]


def conv3d(b: ModelBuilder, x: Ref, name: str, kernel: np.ndarray, bias: Optional[np.ndarray], strides=1, padding="valid",
           dilation=1, activation="linear", transposed=False) -> Ref:
    """Conv3D with the kernel in Keras layout (kd, kh, kw, Cin, Cout), or Conv3DTranspose with (kd, kh, kw, Cout, Cin);
    both are stored as (Cout, kd, kh, kw, Cin) (convert_model.py:227-236)."""
    kd, kh, kw = kernel.shape[:3]
    cout = kernel.shape[3] if transposed else kernel.shape[4]
    cfg = {"filters": int(cout), "kernel_size": [int(kd), int(kh), int(kw)], "strides": _triple(strides), "padding": padding,
           "data_format": "channels_last", "dilation_rate": _triple(dilation), "groups": 1, "activation": activation,
           "use_bias": bias is not None}
    order = [1, 2, 3, 0, 4] if transposed else [1, 2, 3, 4, 0]
    params = {"weights": np.ascontiguousarray(np.moveaxis(kernel, [0, 1, 2, 3, 4], order))}
    if bias is not None:
        params["bias"] = bias
    return b.add("Conv3DTranspose" if transposed else "Conv3D", name, cfg, x, params)


def depthwise_conv2d(b: ModelBuilder, x: Ref, name: str, kernel: np.ndarray,
                     bias: Optional[np.ndarray], strides=1, padding="valid",
                     activation="linear") -> Ref:
    """kernel in Keras layout (kh, kw, C, 1); stored as (C, kh, kw, 1)."""
    kh, kw, _, _ = kernel.shape
    cfg = {"kernel_size": [int(kh), int(kw)], "strides": _pair(strides), "padding": padding,
           "data_format": "channels_last", "dilation_rate": [1, 1], "depth_multiplier": 1,
           "activation": activation, "use_bias": bias is not None}
    params = {"slice_weights": np.moveaxis(kernel, [0, 1, 2, 3], [1, 2, 0, 3])}
    if bias is not None:
        params["bias"] = bias
    return b.add("DepthwiseConv2D", name, cfg, x, params)


def dense(b: ModelBuilder, x: Ref, name: str, kernel: np.ndarray, bias: Optional[np.ndarray],
          activation="linear") -> Ref:
    cfg = {"units": int(kernel.shape[1]), "activation": activation, "use_bias": bias is not None}
    params = {"weights": kernel}
    if bias is not None:
        params["bias"] = bias
    return b.add("Dense", name, cfg, x, params)


def batch_norm(b: ModelBuilder, x: Ref, name: str, mean, var, gamma=None, beta=None,
               eps=1e-3, axis=-1) -> Ref:
    cfg = {"axis": axis, "momentum": 0.99, "epsilon": float(eps),
           "center": beta is not None, "scale": gamma is not None}
    params = {"moving_mean": mean, "moving_variance": var}
    if gamma is not None:
        params["gamma"] = gamma
    if beta is not None:
        params["beta"] = beta
    return b.add("BatchNormalization", name, cfg, x, params)


def layer_norm(b: ModelBuilder, x: Ref, name: str, gamma, beta, eps=1e-5, axis=-1) -> Ref:
    cfg = {"axis": [axis] if isinstance(axis, int) else list(axis), "epsilon": float(eps),
           "center": beta is not None, "scale": gamma is not None}
    params = {}
    if gamma is not None:
        params["gamma"] = gamma
    if beta is not None:
        params["beta"] = beta
    return b.add("LayerNormalization", name, cfg, x, params)


def activation(b: ModelBuilder, x: Ref, name: str, kind: str) -> Ref:
    return b.add("Activation", name, {"activation": kind}, x)


def relu(b: ModelBuilder, x: Ref, name: str, max_value=None, negative_slope=0.0, threshold=0.0) -> Ref:
    cfg = {"max_value": max_value, "negative_slope": float(negative_slope), "threshold": float(threshold)}
    return b.add("ReLU", name, cfg, x)


def zero_pad2d(b: ModelBuilder, x: Ref, name: str, pad) -> Ref:
    return b.add("ZeroPadding2D", name, {"padding": [list(pad[0]), list(pad[1])],
                                         "data_format": "channels_last"}, x)


def max_pool2d(b, x, name, pool, strides, padding="valid") -> Ref:
    return b.add("MaxPooling2D", name, {"pool_size": _pair(pool), "strides": _pair(strides),
                                        "padding": padding, "data_format": "channels_last"}, x)


def avg_pool2d(b, x, name, pool, strides, padding="valid") -> Ref:
    return b.add("AveragePooling2D", name, {"pool_size": _pair(pool), "strides": _pair(strides),
                                            "padding": padding, "data_format": "channels_last"}, x)


def global_avg_pool2d(b, x, name, keepdims=False) -> Ref:
    return b.add("GlobalAveragePooling2D", name, {"data_format": "channels_last", "keepdims": keepdims}, x)


def add_layers(b, xs: Sequence[Ref], name) -> Ref:
    return b.add("Add", name, {}, list(xs))


def concat(b, xs: Sequence[Ref], name, axis=-1) -> Ref:
    return b.add("Concatenate", name, {"axis": axis}, list(xs))


def embedding(b, x, name, table: np.ndarray) -> Ref:
    cfg = {"input_dim": int(table.shape[0]), "output_dim": int(table.shape[1])}
    return b.add("Embedding", name, cfg, x, {"weights": table})


def lstm(b, x, name, w, u, bias, return_sequences=False, return_state=False,
         activation="tanh", recurrent_activation="sigmoid"):
    units = u.shape[0]
    cfg = {"units": int(units), "activation": activation, "recurrent_activation": recurrent_activation,
           "use_bias": bias is not None, "return_sequences": return_sequences,
           "return_state": return_state, "go_backwards": False, "stateful": False, "unroll": False}
    params = {"weights": w, "recurrent_weights": u}
    if bias is not None:
        params["bias"] = bias
    return b.add("LSTM", name, cfg, x, params, n_outputs=3 if return_state else 1)


def conv_lstm(b, x, name, kernel: np.ndarray, recurrent_kernel: np.ndarray, bias: Optional[np.ndarray], strides=1, padding="valid",
              dilation=1, return_sequences=False, return_state=False, activation="tanh", recurrent_activation="sigmoid") -> Ref:
    """ConvLSTM1D (kernels (kw, Cin, 4F)) or ConvLSTM2D (kernels (kh, kw, Cin, 4F)), Keras layouts; gates ordered i, f, c, o.
    Stored as (4F, kh, kw, Cin) like the converter's _prepare_conv_lstm_kernel (keras_export/convert_model.py:639-646)."""
    rank = kernel.ndim - 2
    assert rank in (1, 2) and recurrent_kernel.ndim == kernel.ndim
    filters = recurrent_kernel.shape[-2]

    def stored(k):
        if k.ndim == 3:
            k = k[None]
        return np.moveaxis(k, [0, 1, 2, 3], [1, 2, 3, 0])

    one = (lambda v: [v] if isinstance(v, int) else list(v)) if rank == 1 else _pair
    cfg = {"filters": int(filters), "kernel_size": [int(d) for d in kernel.shape[:rank]], "strides": one(strides), "padding": padding,
           "data_format": "channels_last", "dilation_rate": one(dilation), "activation": activation,
           "recurrent_activation": recurrent_activation, "use_bias": bias is not None, "return_sequences": return_sequences,
           "return_state": return_state, "go_backwards": False, "stateful": False, "unroll": False}
    params = {"weights": stored(kernel), "recurrent_weights": stored(recurrent_kernel)}
    if bias is not None:
        params["bias"] = bias
    return b.add("ConvLSTM%dD" % rank, name, cfg, x, params, n_outputs=3 if return_state else 1)


def gru(b, x, name, w, u, bias, reset_after=True, return_sequences=False, return_state=False,
        activation="tanh", recurrent_activation="sigmoid"):
    units = u.shape[0]
    cfg = {"units": int(units), "activation": activation, "recurrent_activation": recurrent_activation,
           "use_bias": bias is not None, "return_sequences": return_sequences,
           "return_state": return_state, "reset_after": reset_after,
           "go_backwards": False, "stateful": False, "unroll": False}
    params = {"weights": w, "recurrent_weights": u}
    if bias is not None:
        params["bias"] = bias
    return b.add("GRU", name, cfg, x, params, n_outputs=2 if return_state else 1)


def bidirectional(b, x, name, wrapped, forward, backward, merge_mode="concat", return_sequences=False,
                  reset_after=True, activation="tanh", recurrent_activation="sigmoid"):
    """Bidirectional wrapper (convert_model.py:710-737): `forward` and `backward` are (kernel, recurrent
    kernel, bias or None) of the two directions; `wrapped` is "LSTM", "GRU" or "SimpleRNN"."""
    units = forward[1].shape[0]
    inner = {"units": int(units), "activation": activation, "recurrent_activation": recurrent_activation,
             "use_bias": forward[2] is not None, "return_sequences": return_sequences, "return_state": False,
             "reset_after": reset_after, "go_backwards": False, "stateful": False, "unroll": False}
    cfg = {"merge_mode": merge_mode, "layer": {"class_name": wrapped, "config": inner}}
    params = {"forward_weights": forward[0], "forward_recurrent_weights": forward[1],
              "backward_weights": backward[0], "backward_recurrent_weights": backward[1]}
    if forward[2] is not None:
        params["forward_bias"] = forward[2]
        params["backward_bias"] = backward[2]
    return b.add("Bidirectional", name, cfg, x, params)


def rnn(b, x, name, cells, return_sequences=False, return_state=False):
    """keras.layers.RNN around one cell or a StackedRNNCells (convert_model.py:675-707).  `cells` is a list
    of (cell class, kernel, recurrent kernel, bias or None, extra cell config); parameters of cell i of a
    stack are stored under the prefix `cell{i}_`."""
    def cell_json(cls, u, bias, extra):
        c = {"units": int(u.shape[0]), "activation": "tanh", "recurrent_activation": "sigmoid", "use_bias": bias is not None}
        c.update(extra or {})
        return {"class_name": cls, "config": c}
    params = {}
    if len(cells) == 1:
        cls, w, u, bias, extra = cells[0]
        cell = cell_json(cls, u, bias, extra)
        prefixes = [""]
    else:
        cell = {"class_name": "StackedRNNCells",
                "config": {"cells": [cell_json(cls, u, bias, extra) for cls, w, u, bias, extra in cells]}}
        prefixes = [f"cell{i}_" for i in range(len(cells))]
    for pre, (cls, w, u, bias, extra) in zip(prefixes, cells):
        params[pre + "weights"] = w
        params[pre + "recurrent_weights"] = u
        if bias is not None:
            params[pre + "bias"] = bias
    cfg = {"cell": cell, "return_sequences": return_sequences, "return_state": return_state,
           "go_backwards": False, "stateful": False, "unroll": False}
    last = cells[-1][0]
    n_out = 1 if not return_state else (3 if last == "LSTMCell" else 2)
    return b.add("RNN", name, cfg, x, params, n_outputs=n_out)


def multi_head_attention(b, q: Ref, v: Ref, name, weights: List[np.ndarray], num_heads, key_dim,
                         value_dim=None, use_bias=True, k: Optional[Ref] = None) -> Ref:
    """weights in Keras order: Q kernel (dim,H,key_dim), Q bias (H,key_dim), K.., V.., O kernel
    (H,value_dim,out), O bias (out) (convert_model.py:600-607)."""
    cfg = {"num_heads": int(num_heads), "key_dim": int(key_dim),
           "value_dim": int(value_dim if value_dim is not None else key_dim),
           "use_bias": use_bias, "output_shape": None, "attention_axes": None, "dropout": 0.0}
    params = {"weight_shapes": [list(map(int, w.shape)) for w in weights],
              "weights": [w for w in weights]}
    ins = [q, v] if k is None else [q, v, k]
    # Keras serialises mha(query, value[, key]) positionally: args is a flat list.
    node = {"args": [ModelBuilder._tensor_arg(r) for r in ins], "kwargs": {}}
    cfgc = dict(cfg)
    cfgc["name"] = name
    layer = {"class_name": "MultiHeadAttention", "name": name, "config": cfgc, "inbound_nodes": [node]}
    b.layers.append(layer)
    b._layer_index[name] = layer
    b.params[name] = {k_: b._encode_param(v_) for k_, v_ in params.items()}
    b._hash.update(name.encode("ascii"))
    return (name, 0, 0)


def attention(b, q: Ref, v: Ref, name, k: Optional[Ref] = None, score_mode="dot", scale=None, concat_score_weight=None) -> Ref:
    """keras.layers.Attention([query, value(, key)]); `scale` and `concat_score_weight` are stored as plain
    numbers (convert_model.py:581-589)."""
    cfg = {"use_scale": scale is not None, "score_mode": score_mode, "dropout": 0.0}
    params = {}
    if scale is not None:
        params["scale"] = float(scale)
    if score_mode == "concat":
        params["concat_score_weight"] = float(concat_score_weight)
    return b.add("Attention", name, cfg, [q, v] if k is None else [q, v, k], params)


def additive_attention(b, q: Ref, v: Ref, name, k: Optional[Ref] = None, scale: Optional[np.ndarray] = None) -> Ref:
    """keras.layers.AdditiveAttention; `scale` is a vector over the feature axis (convert_model.py:592-597)."""
    cfg = {"use_scale": scale is not None, "dropout": 0.0}
    return b.add("AdditiveAttention", name, cfg, [q, v] if k is None else [q, v, k], {"scale": scale} if scale is not None else None)


def grouped_query_attention(b, q: Ref, v: Ref, name, weights: List[np.ndarray], head_dim, num_query_heads, num_key_value_heads,
                            use_bias=True, use_gate=False, k: Optional[Ref] = None) -> Ref:
    """weights in Keras order: Q kernel (dim,Hq,d), K (dim,Hkv,d), [gate (dim,Hq,d)], V (dim,Hkv,d), out (Hq,d,out),
    each followed by its bias when use_bias (convert_model.py:610-615)."""
    cfg = {"head_dim": int(head_dim), "num_query_heads": int(num_query_heads), "num_key_value_heads": int(num_key_value_heads),
           "use_bias": use_bias, "use_gate": use_gate, "dropout": 0.0, "name": name}
    params = {"weight_shapes": [list(map(int, w.shape)) for w in weights], "weights": [w for w in weights]}
    ins = [q, v] if k is None else [q, v, k]
    node = {"args": [ModelBuilder._tensor_arg(r) for r in ins], "kwargs": {}}
    layer = {"class_name": "GroupedQueryAttention", "name": name, "config": cfg, "inbound_nodes": [node]}
    b.layers.append(layer)
    b._layer_index[name] = layer
    b.params[name] = {k_: b._encode_param(v_) for k_, v_ in params.items()}
    b._hash.update(name.encode("ascii"))
    return (name, 0, 0)


def prelu(b, x: Ref, name, alpha: np.ndarray, shared_axes=None) -> Ref:
    """PReLU with its alpha flattened (convert_model.py:481-489); shared_axes as Keras counts them (1 = height)."""
    return b.add("PReLU", name, {"shared_axes": list(shared_axes) if shared_axes else None}, x, {"alpha": alpha})


def einsum_dense(b, x: Ref, name, equation, kernel: np.ndarray, output_shape, bias: Optional[np.ndarray] = None,
                 bias_axes: Optional[str] = None, activation: Optional[str] = None) -> Ref:
    """keras.layers.EinsumDense (convert_model.py:502-515): `equation` includes the batch letter, `output_shape`
    excludes it; the bias has its axes in the order of the output letters."""
    cfg = {"equation": equation, "output_shape": list(output_shape), "bias_axes": bias_axes, "activation": activation or "linear"}
    params = {"kernel": kernel, "kernel_shape": [int(d) for d in kernel.shape]}
    if bias is not None:
        params["bias"] = bias
        params["bias_shape"] = [int(d) for d in bias.shape]
    return b.add("EinsumDense", name, cfg, x, params)


def rescaling(b, x: Ref, name, scale, offset=0.0) -> Ref:
    return b.add("Rescaling", name, {"scale": float(scale), "offset": float(offset)}, x)


def normalization(b, x: Ref, name, mean: np.ndarray, variance: np.ndarray, axis=-1, invert=False) -> Ref:
    """keras.layers.Normalization with adapted statistics; axis None = one mean / variance for everything."""
    cfg = {"axis": [] if axis is None else [int(axis)], "invert": bool(invert)}
    return b.add("Normalization", name, cfg, x, {"mean": mean.reshape(-1), "variance": variance.reshape(-1)})


def upsampling1d(b, x: Ref, name, size) -> Ref:
    return b.add("UpSampling1D", name, {"size": int(size)}, x)


def upsampling3d(b, x: Ref, name, size=2) -> Ref:
    size = [int(size)] * 3 if np.isscalar(size) else [int(v) for v in size]
    return b.add("UpSampling3D", name, {"size": size, "data_format": "channels_last"}, x)


def time_distributed(b, x: Ref, name, inner_class: str, inner_cfg: dict, inner_params: dict, input_rank: int, output_rank: int) -> Ref:
    """keras.layers.TimeDistributed(layer): the wrapped layer's parameters sit under the wrapper's name, next to the
    ranks of the wrapper's input and output (convert_model.py: td_input_len / td_output_len)."""
    inner = {"class_name": inner_class, "config": dict(inner_cfg, name=name + "_inner")}
    params = dict(inner_params)
    params["td_input_len"] = np.array([input_rank], np.float32)
    params["td_output_len"] = np.array([output_rank], np.float32)
    return b.add("TimeDistributed", name, {"layer": inner}, x, params)


def time_distributed_dense(b, x: Ref, name, kernel: np.ndarray, bias: Optional[np.ndarray], activation="linear",
                           input_rank=2, output_rank=2) -> Ref:
    cfg = {"units": int(kernel.shape[1]), "activation": activation, "use_bias": bias is not None}
    params = {"weights": kernel}
    if bias is not None:
        params["bias"] = bias
    return time_distributed(b, x, name, "Dense", cfg, params, input_rank, output_rank)


def time_distributed_conv2d(b, x: Ref, name, kernel: np.ndarray, bias: Optional[np.ndarray], strides=1, padding="valid",
                            activation="linear") -> Ref:
    """TimeDistributed(Conv2D) on (T, H, W, C); kernel in Keras layout (kh, kw, Cin, Cout)."""
    kh, kw, _, cout = kernel.shape
    cfg = {"filters": int(cout), "kernel_size": [int(kh), int(kw)], "strides": _pair(strides), "padding": padding,
           "data_format": "channels_last", "dilation_rate": [1, 1], "groups": 1, "activation": activation, "use_bias": bias is not None}
    params = {"weights": np.moveaxis(kernel, [0, 1, 2, 3], [1, 2, 3, 0])}
    if bias is not None:
        params["bias"] = bias
    return time_distributed(b, x, name, "Conv2D", cfg, params, 4, 4)


def repeat_vector(b, x: Ref, name, n) -> Ref:
    return b.add("RepeatVector", name, {"n": int(n)}, x)


def center_crop(b, x: Ref, name, height, width) -> Ref:
    return b.add("CenterCrop", name, {"height": int(height), "width": int(width), "data_format": "channels_last"}, x)


def resizing(b, x: Ref, name, height, width, interpolation="bilinear", crop_to_aspect_ratio=False) -> Ref:
    return b.add("Resizing", name, {"height": int(height), "width": int(width), "interpolation": interpolation,
                                    "crop_to_aspect_ratio": bool(crop_to_aspect_ratio), "data_format": "channels_last"}, x)


def dot(b, xs: Sequence[Ref], name, axes, normalize=False) -> Ref:
    """axes: one axis or a pair, counted as Keras does (the batch axis is 0, so 1 is a sample's first axis)."""
    return b.add("Dot", name, {"axes": list(axes) if isinstance(axes, (list, tuple)) else int(axes), "normalize": bool(normalize)}, list(xs))


def adaptive_pooling(b, x: Ref, name, kind, output_size) -> Ref:
    """kind: 'AdaptiveAveragePooling2D', 'AdaptiveMaxPooling1D', ..."""
    size = list(output_size) if isinstance(output_size, (list, tuple)) else int(output_size)
    return b.add(kind, name, {"output_size": size, "data_format": "channels_last"}, x)


def activation_layer(builder, x: Ref, name, class_name, **config) -> Ref:
    """A parameter-free activation layer class (Threshold, HardShrink, SoftShrink, SparsePlus, Squareplus, ...)."""
    return builder.add(class_name, name, dict(config), x)


def discretization(b, x: Ref, name, bin_boundaries) -> Ref:
    return b.add("Discretization", name, {"bin_boundaries": [float(v) for v in bin_boundaries], "output_mode": "int"}, x)


def integer_lookup(b, x: Ref, name, vocabulary, mask_token=None) -> Ref:
    return b.add("IntegerLookup", name, {"vocabulary": [int(v) for v in vocabulary], "num_oov_indices": 1, "output_mode": "int",
                                         "mask_token": None if mask_token is None else int(mask_token), "invert": False}, x)


def category_encoding(b, x: Ref, name, num_tokens, output_mode="multi_hot") -> Ref:
    return b.add("CategoryEncoding", name, {"num_tokens": int(num_tokens), "output_mode": output_mode}, x)


def upsampling2d(b, x: Ref, name, size=2, interpolation="nearest") -> Ref:
    return b.add("UpSampling2D", name, {"size": _pair(size), "data_format": "channels_last", "interpolation": interpolation}, x)


# ---------------------------------------------------------------------------
# Workload builders
# ---------------------------------------------------------------------------
def build_small_cnn(seed: int = 0, size: int = 32) -> dict:
    """Input 32x32x3 -> Conv2D(32,3x3,same,relu) -> MaxPool2D(2) -> Conv2D(64,3x3,same,relu)
    -> BatchNormalization -> GlobalAveragePooling2D -> Dense(128,relu) -> Dense(10,softmax)."""
    ini = Init(seed)
    b = ModelBuilder("small_cnn")
    x = b.input([size, size, 3], "input_image")
    x = conv2d(b, x, "conv_a", ini.glorot_uniform((3, 3, 3, 32), 27, 288), np.zeros(32, np.float32),
               padding="same", activation="relu")
    x = max_pool2d(b, x, "pool_a", 2, 2)
    x = conv2d(b, x, "conv_b", ini.glorot_uniform((3, 3, 32, 64), 288, 576), np.zeros(64, np.float32),
               padding="same", activation="relu")
    x = batch_norm(b, x, "bn_b", ini.normal(64, 0.1), ini.uniform(64, 0.5, 1.5),
                   gamma=np.ones(64, np.float32), beta=np.zeros(64, np.float32), eps=1e-3)
    x = global_avg_pool2d(b, x, "gap")
    x = dense(b, x, "fc_a", ini.glorot_uniform((64, 128), 64, 128), np.zeros(128, np.float32), "relu")
    x = dense(b, x, "fc_b", ini.glorot_uniform((128, 10), 128, 10), np.zeros(10, np.float32), "softmax")
    return b.to_json([x], [[10]])


def build_resnet50(seed: int = 0, size: int = 224, width: int = 64, classes: int = 1000,
                   blocks: Sequence[int] = (3, 4, 6, 3), top: str = "softmax") -> dict:
    """Keras-applications ResNet50 (v1) topology: stride on the first 1x1 of each stage, conv
    bias on, BatchNormalization eps 1.001e-5.  He-normal weights; BN mean/var mildly random so
    that BatchNormalization is not a no-op.  ``top="linear"`` leaves out the final softmax, which
    saturates with random weights and would hide differences in a parity test."""
    ini = Init(seed)
    b = ModelBuilder("resnet50")
    eps = 1.001e-5

    def conv_bn(x, name, cin, cout, k, stride=1, padding="valid", act=True):
        w = ini.he_normal((k, k, cin, cout), k * k * cin)
        bias = ini.normal(cout, 0.01)
        x = conv2d(b, x, name + "_conv", w, bias, strides=stride, padding=padding)
        x = batch_norm(b, x, name + "_bn", ini.normal(cout, 0.05), ini.uniform(cout, 0.8, 1.2),
                       gamma=ini.uniform(cout, 0.9, 1.1), beta=ini.normal(cout, 0.05), eps=eps)
        if act:
            x = activation(b, x, name + "_relu", "relu")
        return x

    def block(x, name, cin, f, stride, conv_shortcut):
        if conv_shortcut:
            sc = conv_bn(x, name + "_0", cin, 4 * f, 1, stride, act=False)
        else:
            sc = x
        y = conv_bn(x, name + "_1", cin, f, 1, stride)
        y = conv_bn(y, name + "_2", f, f, 3, 1, padding="same")
        y = conv_bn(y, name + "_3", f, 4 * f, 1, act=False)
        y = add_layers(b, [sc, y], name + "_add")
        return activation(b, y, name + "_out", "relu")

    x = b.input([size, size, 3], "input_image")
    x = zero_pad2d(b, x, "conv1_pad", ((3, 3), (3, 3)))
    x = conv_bn(x, "conv1", 3, width, 7, 2)
    x = zero_pad2d(b, x, "pool1_pad", ((1, 1), (1, 1)))
    x = max_pool2d(b, x, "pool1_pool", 3, 2)
    cin = width
    for si, n in enumerate(blocks):
        f = width * (2 ** si)
        for bi in range(n):
            stride = 2 if (bi == 0 and si > 0) else 1
            x = block(x, f"conv{si + 2}_block{bi + 1}", cin, f, stride, bi == 0)
            cin = 4 * f
    x = global_avg_pool2d(b, x, "avg_pool")
    x = dense(b, x, "predictions", ini.he_normal((cin, classes), cin), ini.normal(classes, 0.01), top)
    return b.to_json([x], [[classes]])


def build_mobilenetv2(seed: int = 0, size: int = 224, classes: int = 1000, alpha: float = 1.0,
                      last: int = 1280) -> dict:
    """Keras-applications MobileNetV2 topology (alpha=1.0): Conv 3x3/2 -> 17 inverted-residual
    blocks (expand 1x1 -> BN -> ReLU6 -> DW 3x3 -> BN -> ReLU6 -> project 1x1 -> BN [+Add]) ->
    Conv 1x1 -> BN -> ReLU6 -> GAP -> Dense softmax; no conv bias; BN eps 1e-3."""
    ini = Init(seed)
    b = ModelBuilder("mobilenetv2")

    def make_div(v, d=8):
        nv = max(d, int(v + d / 2) // d * d)
        if nv < 0.9 * v:
            nv += d
        return nv

    def bn(x, name, c):
        return batch_norm(b, x, name, ini.normal(c, 0.05), ini.uniform(c, 0.8, 1.2),
                          gamma=ini.uniform(c, 0.9, 1.1), beta=ini.normal(c, 0.05), eps=1e-3)

    x = b.input([size, size, 3], "input_image")
    c0 = make_div(32 * alpha)
    x = conv2d(b, x, "Conv1", ini.he_normal((3, 3, 3, c0), 27), None, strides=2, padding="same")
    x = bn(x, "bn_Conv1", c0)
    x = relu(b, x, "Conv1_relu", max_value=6.0)
    cin = c0
    spec = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1),
            (6, 160, 3, 2), (6, 320, 1, 1)]
    bid = 0
    for t, c, n, s in spec:
        cout = make_div(c * alpha)
        for i in range(n):
            stride = s if i == 0 else 1
            pre = f"block_{bid}_" if bid else "expanded_conv_"
            inp = x
            y = x
            if bid:
                y = conv2d(b, y, pre + "expand", ini.he_normal((1, 1, cin, t * cin), cin), None)
                y = bn(y, pre + "expand_BN", t * cin)
                y = relu(b, y, pre + "expand_relu", max_value=6.0)
            ce = t * cin if bid else cin
            if stride == 2:
                y = zero_pad2d(b, y, pre + "pad", ((0, 1), (0, 1)))
            y = depthwise_conv2d(b, y, pre + "depthwise", ini.he_normal((3, 3, ce, 1), 9), None,
                                 strides=stride, padding="same" if stride == 1 else "valid")
            y = bn(y, pre + "depthwise_BN", ce)
            y = relu(b, y, pre + "depthwise_relu", max_value=6.0)
            y = conv2d(b, y, pre + "project", ini.he_normal((1, 1, ce, cout), ce), None)
            y = bn(y, pre + "project_BN", cout)
            if cin == cout and stride == 1:
                y = add_layers(b, [inp, y], pre + "add")
            x = y
            cin = cout
            bid += 1
    cl = make_div(last * alpha) if alpha > 1.0 else last
    x = conv2d(b, x, "Conv_1", ini.he_normal((1, 1, cin, cl), cin), None)
    x = bn(x, "Conv_1_bn", cl)
    x = relu(b, x, "out_relu", max_value=6.0)
    x = global_avg_pool2d(b, x, "global_average_pooling2d")
    x = dense(b, x, "predictions", ini.he_normal((cl, classes), cl), ini.normal(classes, 0.01), "softmax")
    return b.to_json([x], [[classes]])


def build_text_lstm(seed: int = 0, vocab: int = 20000, dim: int = 128, units: int = 512,
                    seq_len: Optional[int] = 200) -> dict:
    """Embedding(vocab, dim) -> LSTM(units, return_sequences) -> LSTM(units) -> Dense(1, sigmoid).
    Glorot-uniform kernels, orthogonal recurrent kernels, unit forget bias."""
    ini = Init(seed)
    b = ModelBuilder("text_lstm")
    x = b.input([seq_len], "token_ids")
    x = embedding(b, x, "embed", ini.uniform((vocab, dim), -0.05, 0.05))

    def lstm_params(fin):
        w = ini.glorot_uniform((fin, 4 * units), fin, 4 * units)
        u = np.concatenate([ini.orthogonal(units, units) for _ in range(4)], axis=1)
        bias = np.zeros(4 * units, np.float32)
        bias[units:2 * units] = 1.0
        return w, u, bias

    w, u, bi = lstm_params(dim)
    x = lstm(b, x, "lstm_a", w, u, bi, return_sequences=True)
    w, u, bi = lstm_params(units)
    x = lstm(b, x, "lstm_b", w, u, bi, return_sequences=False)
    x = dense(b, x, "head", ini.glorot_uniform((units, 1), units, 1), np.zeros(1, np.float32), "sigmoid")
    return b.to_json([x], [[1]])


def build_gpt2_step(seed: int = 0, vocab: int = 50257, ctx: int = 1024, dim: int = 768,
                    layers: int = 12, heads: int = 12, ffn: int = 3072, first: bool = False) -> dict:
    """GPT-2-small-shaped decoder as a one-token *incremental* graph.

    The reference's MultiHeadAttention has no mask (multi_head_attention_layer.hpp:98-110), so
    causal attention is expressed with T_q = 1: inputs are token_id (1), pos_id (1) and, unless
    ``first``, one ``past_l`` (None, dim) tensor per block holding the LayerNorm'd block inputs of
    the earlier positions.  Block l computes x_ln = LN(x); kv = Concatenate(axis=1)([past_l, x_ln]);
    x += MHA(query=x_ln, value=kv); x += Dense(gelu(Dense(LN(x)))).  Outputs: logits (1, vocab) and
    the ``layers`` x_ln rows (1, dim) which the caller appends to its past tensors.
    ``first=True`` builds the graph for position 0 (no past inputs, kv = x_ln).  Both graphs are
    built from the same seed, so they carry identical weights."""
    ini = Init(seed)
    b = ModelBuilder("gpt2_first" if first else "gpt2_step")
    tok = b.input([1], "token_id")
    pos = b.input([1], "pos_id")
    pasts = []
    if not first:
        for l in range(layers):
            pasts.append(b.input([None, dim], f"past_{l}"))
    te = embedding(b, tok, "wte", ini.normal((vocab, dim), 0.02))
    pe = embedding(b, pos, "wpe", ini.normal((ctx, dim), 0.02))
    x = add_layers(b, [te, pe], "embed_add")
    hd = dim // heads
    outs = []
    for l in range(layers):
        g1, b1 = np.ones(dim, np.float32), np.zeros(dim, np.float32)
        xl = layer_norm(b, x, f"h{l}_ln1", g1, b1, eps=1e-5)
        outs.append(xl)
        kv = xl if first else concat(b, [pasts[l], xl], f"h{l}_kv", axis=1)
        ws = []
        for _ in range(3):
            ws.append(ini.normal((dim, heads, hd), 0.02))
            ws.append(np.zeros((heads, hd), np.float32))
        ws.append(ini.normal((heads, hd, dim), 0.02))
        ws.append(np.zeros(dim, np.float32))
        a = multi_head_attention(b, xl, kv, f"h{l}_attn", ws, heads, hd)
        x = add_layers(b, [x, a], f"h{l}_res1")
        xm = layer_norm(b, x, f"h{l}_ln2", np.ones(dim, np.float32), np.zeros(dim, np.float32), eps=1e-5)
        m = dense(b, xm, f"h{l}_fc", ini.normal((dim, ffn), 0.02), np.zeros(ffn, np.float32), "gelu")
        m = dense(b, m, f"h{l}_proj", ini.normal((ffn, dim), 0.02), np.zeros(dim, np.float32))
        x = add_layers(b, [x, m], f"h{l}_res2")
    x = layer_norm(b, x, "ln_f", np.ones(dim, np.float32), np.zeros(dim, np.float32), eps=1e-5)
    logits = dense(b, x, "lm_head", ini.normal((dim, vocab), 0.02), None)
    return b.to_json([logits] + outs, [[1, vocab]] + [[1, dim]] * layers)


# ---------------------------------------------------------------------------
# Seeded synthetic inputs for the workloads
# ---------------------------------------------------------------------------
def inputs_small_cnn(n: int, seed: int = 1, size: int = 32) -> np.ndarray:
    return np.random.default_rng(seed).uniform(0.0, 1.0, size=(n, size, size, 3)).astype(np.float32)


def inputs_resnet50(n: int, seed: int = 1, size: int = 224) -> np.ndarray:
    return np.random.default_rng(seed).normal(0.0, 1.0, size=(n, size, size, 3)).astype(np.float32)


def inputs_mobilenetv2(n: int, seed: int = 1, size: int = 224) -> np.ndarray:
    return np.random.default_rng(seed).uniform(-1.0, 1.0, size=(n, size, size, 3)).astype(np.float32)


def inputs_text_lstm(n: int, seed: int = 1, vocab: int = 20000, seq_len: int = 200) -> np.ndarray:
    return np.random.default_rng(seed).integers(1, vocab, size=(n, seq_len)).astype(np.float32)


def inputs_gpt2_prompts(n: int, seed: int = 1, vocab: int = 50257, prompt_len: int = 32) -> np.ndarray:
    return np.random.default_rng(seed).integers(0, vocab, size=(n, prompt_len)).astype(np.float32)
