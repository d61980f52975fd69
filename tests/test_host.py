"""CPU tests of the host side: the C-ABI library loads and exports what include/fdeep_b200.h declares,
the loader and the plan compiler (shape inference, epilogue fusion, memory plan) behave like the
reference's loader and graph walk, and the engine refuses to run without a CUDA device."""
import json
import os
import re

import numpy as np
import pytest

import fdeep_b200
from fdeep_b200 import model_writer as mw
from fdeep_b200.capi import EXPORTS
from util import model_text

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(built_library):
    header = open(os.path.join(ROOT, "include", "fdeep_b200.h")).read()
    declared = sorted(set(re.findall(r"\b(fdk_[a-z_0-9]+)\s*\(", header)))
    assert declared, "no declarations found in the header"
    lib = fdeep_b200.load_library()
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/fdeep_b200.h but not exported"
    assert sorted(EXPORTS) == declared


def test_no_cuda_device_fails_loudly(built_library):
    if fdeep_b200.device_count() > 0:
        pytest.skip("a CUDA device is present")
    with pytest.raises(fdeep_b200.FdeepError, match="no CUDA device"):
        fdeep_b200.read_model_from_string(model_text(mw.build_small_cnn()))


def test_plan_small_cnn_fuses_activation_and_batchnorm(built_library):
    txt = fdeep_b200.plan_describe(model_text(mw.build_small_cnn()), [[32, 32, 3]])
    lines = txt.strip().split("\n")
    assert lines[0].startswith("arena_elems_per_sample=")
    assert "flops_per_sample=11225600" in lines[0]  # 5.613 MMAC per sample
    assert lines[1] == "output 0 (10)"
    ops = [l.split()[0] for l in lines[2:]]
    assert ops == ["conv", "pool", "conv", "gpool", "gemm", "gemm", "softmax"]
    conv_b = [l for l in lines if " conv_b " in l][0]
    assert "act1" in conv_b and "affine" in conv_b  # Conv2D(relu) -> BatchNormalization in one epilogue


def test_plan_resnet_block_fuses_bn_add_relu(built_library):
    txt = fdeep_b200.plan_describe(model_text(mw.build_resnet50(size=64, width=16, classes=10)), [[64, 64, 3]])
    lines = txt.strip().split("\n")
    # every block ends in one conv op carrying bias, BN affine, residual add and ReLU
    fused = [l for l in lines if "residual" in l]
    assert len(fused) == 16
    for l in fused:
        assert "bias" in l and "affine" in l and "act1" in l
    assert not any(l.startswith(("binary", "affine", "unary")) for l in lines[2:])
    assert lines[-1].startswith("softmax predictions out=(10)")


def test_plan_full_resnet50_flops(built_library):
    txt = fdeep_b200.plan_describe(model_text(mw.build_resnet50()), [[224, 224, 3]])
    flops = int(re.search(r"flops_per_sample=(\d+)", txt).group(1))
    assert abs(flops - 2 * 3.858e9) / (2 * 3.858e9) < 0.01  # 3.858 GMAC per image


def test_plan_variable_shapes_and_memory_reuse(built_library):
    js = mw.build_gpt2_step(vocab=101, ctx=16, dim=32, layers=2, heads=4, ffn=64)
    t3 = fdeep_b200.plan_describe(model_text(js), [[1], [1], [3, 32], [3, 32]])
    t9 = fdeep_b200.plan_describe(model_text(js), [[1], [1], [9, 32], [9, 32]])
    assert "concat h0_kv out=(4, 32)" in t3 and "concat h0_kv out=(10, 32)" in t9
    for l in t3.split("\n"):
        m = re.search(r"off=(-?\d+)", l)
        if m:
            assert int(m.group(1)) >= 0 and int(m.group(1)) % 64 == 0  # 256-byte aligned arena offsets
    # liveness-based reuse keeps the arena well below the sum of all intermediates
    arena = int(re.search(r"arena_elems_per_sample=(\d+)", t3).group(1))
    total = sum(int(x) for x in re.findall(r"elems=(\d+)", t3))
    assert arena < total


def test_loader_and_shape_errors_mirror_the_reference(built_library):
    js = mw.build_small_cnn()
    text = model_text(js)
    with pytest.raises(fdeep_b200.FdeepError, match="Invalid inputs shape"):
        fdeep_b200.plan_describe(text, [[31, 32, 3]])
    with pytest.raises(fdeep_b200.FdeepError, match="Invalid number of input tensors"):
        fdeep_b200.plan_describe(text, [[32, 32, 3], [1]])
    bad = json.loads(text)
    bad["image_data_format"] = "channels_first"
    with pytest.raises(fdeep_b200.FdeepError, match="only channels_last data format supported"):
        fdeep_b200.plan_describe(json.dumps(bad), [[32, 32, 3]])
    bad = json.loads(text)
    bad["architecture"]["config"]["layers"][1]["class_name"] = "NoSuchLayer"
    with pytest.raises(fdeep_b200.FdeepError, match="unknown layer type: NoSuchLayer"):
        fdeep_b200.plan_describe(json.dumps(bad), [[32, 32, 3]])
    bad = json.loads(text)
    bad["architecture"]["config"]["layers"][1]["inbound_nodes"][0]["args"][0]["config"]["keras_history"][0] = "ghost"
    with pytest.raises(fdeep_b200.FdeepError, match="dangling layer reference: ghost"):
        fdeep_b200.plan_describe(json.dumps(bad), [[32, 32, 3]])
    with pytest.raises(fdeep_b200.FdeepError, match="json parse error"):
        fdeep_b200.plan_describe("{not json", [[32, 32, 3]])
    bad = json.loads(text)
    bad["architecture"]["config"]["layers"][1]["config"]["activation"] = "mystery"
    with pytest.raises(fdeep_b200.FdeepError, match="unknown activation type: mystery"):
        fdeep_b200.plan_describe(json.dumps(bad), [[32, 32, 3]])


def test_plain_number_weight_arrays_are_accepted(built_library):
    """decode_floats also reads plain JSON number arrays (import_model.hpp:279-282)."""
    b = mw.ModelBuilder("m")
    i = b.input([3])
    o = mw.dense(b, i, "d", np.eye(3, dtype=np.float32), np.zeros(3, np.float32))
    js = json.loads(model_text(b.to_json([o], [[3]])))
    js["trainable_params"]["d"]["weights"] = [1.0, 0.0, 0.0, 0.0, 1.0, 0.0, 0.0, 0.0, 1.0]
    assert "gemm d out=(3)" in fdeep_b200.plan_describe(json.dumps(js), [[3]])


def test_nested_model_and_shared_layer(built_library):
    """Nested Functional models get their parameters under '<outer>_' (import_model.hpp:404-409,1941);
    a layer applied twice has two inbound nodes (node.hpp:66-74)."""
    inner = mw.ModelBuilder("inner")
    ii = inner.input([4], "inner_in")
    io = mw.dense(inner, ii, "inner_fc", np.ones((4, 2), np.float32), np.zeros(2, np.float32), "relu")
    inner_js = inner.to_json([io], [[2]])
    outer = mw.ModelBuilder("outer")
    a = outer.input([4], "a")
    bb = outer.input([4], "b")
    shared_a = mw.dense(outer, a, "shared", np.eye(4, dtype=np.float32), np.zeros(4, np.float32))
    shared_b = mw.dense(outer, bb, "shared", np.eye(4, dtype=np.float32), np.zeros(4, np.float32))
    s = mw.add_layers(outer, [shared_a, shared_b], "sum")
    sub_layer = dict(inner_js["architecture"])
    sub_layer["name"] = "inner"
    sub_layer["inbound_nodes"] = [{"args": [mw.ModelBuilder._tensor_arg(s)], "kwargs": {}}]
    outer.layers.append(sub_layer)
    outer.params["inner_inner_fc"] = inner_js["trainable_params"]["inner_fc"]
    js = outer.to_json([("inner", 1, 0)], [[2]])
    txt = fdeep_b200.plan_describe(model_text(js), [[4], [4]])
    assert txt.count("gemm shared") == 2 and "gemm inner_fc out=(2)" in txt


def test_plan_of_tiny_models_has_exact_flops(built_library):
    """Two- and three-layer graphs (the tensor list of the plan compiler grows while shapes are in use)."""
    ini = mw.Init(9)
    for n_layers in (1, 2, 3, 5):
        b = mw.ModelBuilder("tiny")
        x = b.input([4])
        width, flops = 4, 0
        for i in range(n_layers):
            x = mw.dense(b, x, f"fc{i}", ini.glorot_uniform((width, 8), width, 8), ini.normal(8, 0.1), "relu")
            flops += 2 * width * 8
            width = 8
        text = model_text(b.to_json([x], [[8]]))
        listing = fdeep_b200.plan_describe(text, [[4]])
        assert f"flops_per_sample={flops}\n" in listing, listing


def test_plan_of_recurrent_wrappers(built_library):
    """Bidirectional becomes two recurrent operations and a merge; a stack of cells becomes one recurrent
    operation per cell.  FLOPs: 2 T g U (F + U) per recurrent layer."""
    from test_oracle import bidirectional_models, stacked_rnn_model
    js, x, _ = bidirectional_models(T=7, Fdim=5, U=8)
    listing = fdeep_b200.plan_describe(model_text(js), [[7, 5]])
    assert listing.count("lstm") == 10, listing       # five heads, two directions each
    assert f"flops_per_sample={10 * 2 * 7 * 4 * 8 * (5 + 8)}\n" in listing, listing
    js, x, _ = stacked_rnn_model(T=6, Fdim=5, U=8)
    listing = fdeep_b200.plan_describe(model_text(js), [[6, 5]])
    assert listing.count("lstm") == 3, listing
    assert f"flops_per_sample={2 * 6 * 4 * 8 * (2 * (5 + 8) + (8 + 8))}\n" in listing, listing


def test_plan_of_attention_variants(built_library):
    from test_oracle import attention_zoo, gqa_model, prelu_model
    js, xs, _ = attention_zoo()
    listing = fdeep_b200.plan_describe(model_text(js), [list(a.shape) for a in xs])
    assert listing.count("attn") == 6, listing
    js, xs, _ = gqa_model(use_gate=True)
    listing = fdeep_b200.plan_describe(model_text(js), [list(a.shape) for a in xs])
    assert listing.count("mha") == 1, listing
    js, xs, _ = prelu_model()
    listing = fdeep_b200.plan_describe(model_text(js), [list(a.shape) for a in xs])
    assert listing.count("prelu") == 3, listing


def test_plan_of_einsum_dense(built_library):
    """Equations of the form X S, S O -> X O become the matrix product; the others the general contraction."""
    from test_oracle import EINSUM_CASES, einsum_model
    kinds = []
    for case in EINSUM_CASES:
        js, x, _ = einsum_model(case)
        listing = fdeep_b200.plan_describe(model_text(js), [list(x.shape)])
        kinds.append("gemm" if "gemm" in listing else "einsum" if "einsum" in listing else "?")
    assert kinds == ["gemm", "gemm", "gemm", "gemm", "einsum", "einsum", "einsum", "einsum"], kinds


def test_plan_of_conv3d(built_library):
    """Each case plans as one patch-matrix + product operation with 2 * rows * K * N contraction FLOPs."""
    from test_oracle import CONV3D_CASES, conv3d_model
    for case in CONV3D_CASES:
        js, x, want = conv3d_model(case)
        listing = fdeep_b200.plan_describe(model_text(js), [list(x.shape)])
        assert "conv3d" in listing, listing
        in_shape, ks, cout, strides, padding, dilation, transposed = case
        dl = [dilation] * 3 if isinstance(dilation, int) else list(dilation)
        k = int(np.prod([(a - 1) * d + 1 for a, d in zip(ks, dl)])) * in_shape[3]
        rows = int(np.prod(want.shape[:3]))
        assert f"flops_per_sample={2 * rows * k * cout}\n" in listing, listing
        assert (" implicit" in listing) == (not transposed and in_shape[3] % 4 == 0), listing
        st = [strides] * 3 if isinstance(strides, int) else list(strides)
        phases = transposed and in_shape[3] % 4 == 0 and cout % 4 == 0 and want.shape[0] % st[0] == 0 and all(k_ >= s_ for k_, s_ in zip(ks, st))
        assert (" phases" in listing) == phases, listing


def test_plan_of_conv2d_transpose(built_library):
    """A transposed convolution with 4 | input channels plans as per-phase implicit products (no patch matrix in the
    arena); other channel counts and kernels shorter than the stride keep the gathered form."""
    from test_oracle import CONV2D_TRANSPOSE_CASES, conv2d_transpose_model
    for case in CONV2D_TRANSPOSE_CASES:
        js, x, want = conv2d_transpose_model(case)
        listing = fdeep_b200.plan_describe(model_text(js), [list(x.shape)])
        in_shape, ks, cout, strides, padding = case
        st = [strides] * 2 if isinstance(strides, int) else list(strides)
        phases = in_shape[2] % 4 == 0 and cout % 4 == 0 and all(k >= s_ for k, s_ in zip(ks, st))
        assert (" phases" if phases else " im2col") in listing, listing


def test_transposed_phase_arithmetic(tmp_path):
    """The (filter tap, input index) pairs of every output position of a transposed convolution, from the per-phase
    formula of the loader and executor against the reference's spread-pad-convolve definition (convolution.hpp:443-469),
    for kernels 1-7, strides 1-4, both paddings and inputs of 1-9 samples (a host program, tests/cpp/transposed_phases.cpp)."""
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        pytest.skip("no host compiler")
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    exe = str(tmp_path / "transposed_phases")
    cmd = ["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "frugally-deep_b200", "csrc"), "-I", cuda_inc,
           os.path.join(ROOT, "tests", "cpp", "transposed_phases.cpp"), "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.startswith("ok"), r.stdout + r.stderr


def test_plan_of_preprocessing_layers(built_library):
    from test_oracle import preprocessing_model
    js, xs, _ = preprocessing_model()
    listing = fdeep_b200.plan_describe(model_text(js), [list(a.shape) for a in xs])
    assert listing.count("normalize") == 4 and listing.count("upsample") == 3 and listing.count("unary") == 1, listing


def test_plan_of_conv_lstm(built_library):
    """The plan of a convolutional LSTM holds, per time step, the input convolution, the recurrent convolution of the previous
    hidden state (none at the first step) and one gate kernel."""
    from test_oracle import CONV_LSTM_CASES, conv_lstm_case
    for case in CONV_LSTM_CASES:
        js, x, wants = conv_lstm_case(**case)
        txt = fdeep_b200.plan_describe(model_text(js), [list(x.shape)])
        assert txt.count("convlstm_cell") == case["T"], txt
