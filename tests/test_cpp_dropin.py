"""The drop-in C++ header (frugally-deep_b200/include/fdeep/fdeep.hpp): a program written against the
reference's public API (the shape of its test/readme_example_main.cpp) compiles as C++14 against the
header and the shared library; on a GPU it loads a model file, runs the embedded self test, predicts and
prints what the oracle computes."""
import json
import os
import re
import subprocess

import numpy as np
import pytest

from fdeep_b200 import model_writer as mw
from util import model_text

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
PKG = os.path.join(ROOT, "frugally-deep_b200")


def compile_example(built_library, out_dir, name="readme_example"):
    exe = os.path.join(str(out_dir), name)
    cmd = ["g++", "-std=c++14", "-O1", "-Wall", "-I", os.path.join(PKG, "include"), os.path.join(HERE, "cpp", name + ".cpp"),
           "-o", exe, "-L", PKG, "-lfdeep_b200", "-Wl,-rpath," + PKG, "-pthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def dense_model(tests=None):
    ini = mw.Init(9)
    b = mw.ModelBuilder("readme_model")
    x = b.input([4])
    x = mw.dense(b, x, "hidden", ini.glorot_uniform((4, 8), 4, 8), ini.normal(8, 0.1), "relu")
    x = mw.dense(b, x, "out", ini.glorot_uniform((8, 3), 8, 3), ini.normal(3, 0.1), "softmax")
    return b.to_json([x], [[3]], tests)


def test_example_compiles_as_cpp14(built_library, tmp_path):
    compile_example(built_library, tmp_path)
    compile_example(built_library, tmp_path, "device_chain")
    compile_example(built_library, tmp_path, "bench_dropin")


@pytest.mark.gpu
def test_two_models_chain_on_the_device(built_library, tmp_path):
    """Device-resident fdeep::tensor: the results of one model feed the next without a copy through host memory
    (checked with the library's transfer counters), and every value equals the host path's bit for bit."""
    exe = compile_example(built_library, tmp_path, "device_chain")
    ini = mw.Init(4)
    a = mw.ModelBuilder("stage_a")
    x = a.input([12, 12, 3])
    x = mw.conv2d(a, x, "conv", ini.he_normal((3, 3, 3, 8), 27), ini.normal(8, 0.1), strides=1, padding="same", activation="relu")
    x = mw.global_avg_pool2d(a, x, "gap")
    x = mw.dense(a, x, "fc", ini.glorot_uniform((8, 16), 8, 16), ini.normal(16, 0.1), "tanh")
    ja = a.to_json([x], [[16]])
    b = mw.ModelBuilder("stage_b")
    y = b.input([16])
    y = mw.dense(b, y, "h", ini.glorot_uniform((16, 32), 16, 32), ini.normal(32, 0.1), "relu")
    y = mw.dense(b, y, "out", ini.glorot_uniform((32, 5), 32, 5), ini.normal(5, 0.1), "softmax")
    jb = b.to_json([y], [[5]])
    pa, pb = os.path.join(str(tmp_path), "a.json"), os.path.join(str(tmp_path), "b.json")
    for path, js in ((pa, ja), (pb, jb)):
        with open(path, "w") as f:
            json.dump(js, f)
    r = subprocess.run([exe, pa, pb], capture_output=True, text=True, timeout=300, env=dict(os.environ, FDEEP_B200_DEVICES="0"))
    assert r.returncode == 0, f"exit {r.returncode}: {r.stdout}{r.stderr}"
    assert "device chain ok" in r.stdout


@pytest.mark.gpu
def test_example_runs_and_matches_oracle(built_library, tmp_path):
    from oracle import OracleModel
    exe = compile_example(built_library, tmp_path)
    x = np.array([1, 2, 3, 4], np.float32)
    want = OracleModel(json_text=model_text(dense_model())).predict([x])[0]
    tests = [{"inputs": [mw.show_tensor(x)], "outputs": [mw.show_tensor(want)]}]
    path = os.path.join(str(tmp_path), "readme_model.json")
    with open(path, "w") as f:
        json.dump(dense_model(tests), f)
    r = subprocess.run([exe, path], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    shown = re.search(r"\[\[\[\[\[\[[^\n]*", r.stdout).group(0)
    got = np.array([float(v) for v in re.findall(r"-?\d+\.\d+", shown)], np.float32)
    np.testing.assert_allclose(got, want.reshape(-1), atol=6e-5)  # printed with four decimals
    assert f"class {int(np.argmax(want))} name readme_model" in r.stdout
    assert "test_speed" in r.stdout
