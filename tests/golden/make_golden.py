"""Generates the golden fixtures in this folder:  python tests/golden/make_golden.py

Each fixture is one .npz holding a small converted-JSON model (with an embedded `tests` entry, so the
load-time self test is exercised too), seeded inputs for a few samples, and the outputs of the CPU
oracle.  The reference itself cannot be run where these were made (Eigen and FunctionalPlus are not
available), so these vectors pin the oracle and the CUDA engine to each other and guard against
regressions; they are not outputs of the reference.
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "frugally-deep_b200"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))

from fdeep_b200 import model_writer as mw  # noqa: E402
from oracle import OracleModel  # noqa: E402


def text_of(js):
    return json.dumps(js, allow_nan=False, separators=(",", ":"))


def save(name, build_fn, samples):
    """build_fn(tests) -> model json; samples: list of input lists."""
    plain = text_of(build_fn(None))
    m = OracleModel(json_text=plain)
    outs = [m.predict(s) for s in samples]
    tests = [{"inputs": [mw.show_tensor(a) for a in samples[0]], "outputs": [mw.show_tensor(o) for o in outs[0]]}]
    text = text_of(build_fn(tests))
    arrays = {"model_json": np.frombuffer(text.encode(), dtype=np.uint8), "n_in": np.int64(len(samples[0])),
              "n_out": np.int64(len(outs[0])), "n_samples": np.int64(len(samples))}
    for s, (ins, os_) in enumerate(zip(samples, outs)):
        for i, a in enumerate(ins):
            arrays[f"in_{s}_{i}"] = np.asarray(a, np.float32)
        for o, a in enumerate(os_):
            arrays[f"out_{s}_{o}"] = a
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrays)
    print(name, os.path.getsize(path), "bytes")


def cnn_tiny(tests):
    ini = mw.Init(0)
    b = mw.ModelBuilder("cnn_tiny")
    x = b.input([12, 12, 3])
    x = mw.conv2d(b, x, "conv_a", ini.glorot_uniform((3, 3, 3, 8), 27, 72), ini.normal(8, 0.1), padding="same", activation="relu")
    x = mw.max_pool2d(b, x, "pool_a", 2, 2)
    x = mw.conv2d(b, x, "conv_b", ini.glorot_uniform((3, 3, 8, 16), 72, 144), np.zeros(16, np.float32), padding="same", activation="relu")
    x = mw.batch_norm(b, x, "bn_b", ini.normal(16, 0.1), ini.uniform(16, 0.5, 1.5), np.ones(16, np.float32), np.zeros(16, np.float32))
    x = mw.global_avg_pool2d(b, x, "gap")
    x = mw.dense(b, x, "fc_a", ini.glorot_uniform((16, 16), 16, 16), ini.normal(16, 0.1), "relu")
    x = mw.dense(b, x, "fc_b", ini.glorot_uniform((16, 5), 16, 5), ini.normal(5, 0.1), "softmax")
    return b.to_json([x], [[5]], tests)


def resnet_tiny(tests):
    js = mw.build_resnet50(seed=2, size=32, width=4, classes=5, blocks=(1, 2, 1, 1))
    if tests:
        js["tests"] = tests
    return js


def inverted_residual_tiny(tests):
    ini = mw.Init(3)
    b = mw.ModelBuilder("mb_tiny")

    def bn(x, name, c):
        return mw.batch_norm(b, x, name, ini.normal(c, 0.05), ini.uniform(c, 0.8, 1.2), ini.uniform(c, 0.9, 1.1), ini.normal(c, 0.05))
    x = b.input([17, 17, 3])
    x = mw.conv2d(b, x, "stem", ini.he_normal((3, 3, 3, 8), 27), None, strides=2, padding="same")
    x = mw.relu(b, bn(x, "stem_bn", 8), "stem_relu", max_value=6.0)
    for i, stride in enumerate((1, 2, 1)):
        inp = x
        y = mw.conv2d(b, x, f"b{i}_expand", ini.he_normal((1, 1, 8, 24), 8), None)
        y = mw.relu(b, bn(y, f"b{i}_expand_bn", 24), f"b{i}_expand_relu", max_value=6.0)
        if stride == 2:
            y = mw.zero_pad2d(b, y, f"b{i}_pad", ((0, 1), (0, 1)))
        y = mw.depthwise_conv2d(b, y, f"b{i}_dw", ini.he_normal((3, 3, 24, 1), 9), None, strides=stride,
                                padding="same" if stride == 1 else "valid")
        y = mw.relu(b, bn(y, f"b{i}_dw_bn", 24), f"b{i}_dw_relu", max_value=6.0)
        y = bn(mw.conv2d(b, y, f"b{i}_project", ini.he_normal((1, 1, 24, 8), 24), None), f"b{i}_project_bn", 8)
        x = mw.add_layers(b, [inp, y], f"b{i}_add") if stride == 1 else y
    x = mw.global_avg_pool2d(b, x, "gap")
    x = mw.dense(b, x, "fc", ini.he_normal((8, 4), 8), ini.normal(4, 0.01), "softmax")
    return b.to_json([x], [[4]], tests)


def lstm_tiny(tests):
    js = mw.build_text_lstm(seed=4, vocab=50, dim=8, units=12, seq_len=6)
    if tests:
        js["tests"] = tests
    return js


def gpt2_tiny(first):
    def fn(tests):
        js = mw.build_gpt2_step(seed=5, vocab=37, ctx=16, dim=16, layers=2, heads=2, ffn=32, first=first)
        if tests:
            js["tests"] = tests
        return js
    return fn


def misc_ops(tests):
    ini = mw.Init(6)
    b = mw.ModelBuilder("misc_ops")
    img = b.input([9, 10, 4], "img")
    seq = b.input([7, 5], "seq")
    # image branch
    a = mw.avg_pool2d(b, img, "avg_same", 3, 2, "same")                       # (5,5,4)
    m = mw.max_pool2d(b, img, "max_same", 3, 2, "same")                       # (5,5,4)
    cat = mw.concat(b, [a, m], "cat_depth", axis=-1)                          # (5,5,8)
    sep = b.add("SeparableConv2D", "sep", {"filters": 6, "kernel_size": [3, 3], "strides": [1, 1], "padding": "same",
                                           "dilation_rate": [1, 1], "depth_multiplier": 1, "activation": "swish", "use_bias": True},
                cat, {"slice_weights": np.moveaxis(ini.he_normal((3, 3, 8, 1), 9), [0, 1, 2, 3], [1, 2, 0, 3]),
                      "stack_weights": np.moveaxis(ini.he_normal((1, 1, 8, 6), 8), [0, 1, 2, 3], [1, 2, 3, 0]),
                      "bias": ini.normal(6, 0.1)})                            # (5,5,6)
    tr = b.add("Conv2DTranspose", "deconv", {"filters": 3, "kernel_size": [3, 3], "strides": [2, 2], "padding": "same",
                                             "dilation_rate": [1, 1], "activation": "linear", "use_bias": True},
               sep, {"weights": np.moveaxis(ini.he_normal((3, 3, 3, 6), 54), [0, 1, 2, 3], [1, 2, 0, 3]), "bias": ini.normal(3, 0.1)})  # (10,10,3)
    crop = b.add("Cropping2D", "crop", {"cropping": [[1, 0], [0, 0]]}, tr)    # (9,10,3)
    pad = mw.zero_pad2d(b, crop, "pad", ((1, 2), (0, 1)))                     # (12,11,3)
    gmp = b.add("GlobalMaxPooling2D", "gmp", {"keepdims": False}, pad)        # (3)
    dil = mw.conv2d(b, img, "dilated", ini.he_normal((3, 3, 4, 5), 36), ini.normal(5, 0.1), padding="same", dilation=2, activation="elu")
    mx = b.add("Maximum", "maxi", {}, [dil, dil])
    mul = b.add("Multiply", "mul", {}, [mx, b.add("Reshape", "gate", {"target_shape": [1, 1, 5]},
                                                  mw.dense(b, b.add("GlobalAveragePooling2D", "gap2", {"keepdims": False}, dil), "gate_fc",
                                                           ini.glorot_uniform((5, 5), 5, 5), ini.normal(5, 0.1), "sigmoid"))])  # broadcast
    flat = b.add("Flatten", "flat", {}, mul)                                  # (450)
    head = mw.dense(b, flat, "head", ini.glorot_uniform((450, 4), 450, 4), ini.normal(4, 0.1), "tanh")
    # sequence branch
    c1 = b.add("Conv1D", "causal", {"filters": 6, "kernel_size": [3], "strides": [1], "padding": "causal", "dilation_rate": [2],
                                    "activation": "relu", "use_bias": True},
               seq, {"weights": np.moveaxis(ini.he_normal((3, 5, 6), 15), [0, 1, 2], [1, 2, 0]), "bias": ini.normal(6, 0.1)})  # (7,6)
    g = mw.gru(b, c1, "gru", ini.glorot_uniform((6, 12), 6, 12), ini.orthogonal(4, 12), ini.normal(24, 0.1).reshape(-1),
               reset_after=True, return_sequences=True)                       # (7,4)
    perm = b.add("Permute", "perm", {"dims": [2, 1]}, g)                      # (4,7)
    ln = mw.layer_norm(b, perm, "ln", ini.uniform(7, 0.9, 1.1), ini.normal(7, 0.1))
    sub = b.add("Subtract", "sub", {}, [ln, perm])
    avg = b.add("Average", "avg", {}, [sub, ln, perm])
    gelu = mw.activation(b, avg, "gelu", "gelu")
    return b.to_json([gmp, head, gelu], [[3], [4], [4, 7]], tests)


def main():
    rng = np.random.default_rng(123)
    save("cnn_tiny", cnn_tiny, [[rng.uniform(0, 1, (12, 12, 3)).astype(np.float32)] for _ in range(3)])
    save("resnet_tiny", resnet_tiny, [[rng.normal(0, 1, (32, 32, 3)).astype(np.float32)] for _ in range(2)])
    save("inverted_residual_tiny", inverted_residual_tiny, [[rng.uniform(-1, 1, (17, 17, 3)).astype(np.float32)] for _ in range(3)])
    save("lstm_tiny", lstm_tiny, [[rng.integers(1, 50, 6).astype(np.float32)] for _ in range(3)])
    save("gpt2_first_tiny", gpt2_tiny(True), [[np.array([float(t)], np.float32), np.array([0.0], np.float32)] for t in (3, 17)])
    save("gpt2_step_tiny", gpt2_tiny(False),
         [[np.array([float(t)], np.float32), np.array([float(s)], np.float32)] + [rng.normal(0, 1, (s, 16)).astype(np.float32) for _ in range(2)]
          for t, s in ((5, 1), (11, 4), (30, 9))])
    save("misc_ops", misc_ops, [[rng.normal(0, 1, (9, 10, 4)).astype(np.float32), rng.normal(0, 1, (7, 5)).astype(np.float32)] for _ in range(2)])


if __name__ == "__main__":
    main()
