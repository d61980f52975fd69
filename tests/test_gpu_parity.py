"""GPU parity tests: the CUDA engine, called through the C ABI, against the CPU oracle on the same
seeded inputs, against the committed golden fixtures, and through size-independent properties at the
benchmark sizes.  Tolerance: 1e-4 relative per output with a floor for near-zero outputs (util.py),
plus the reference's own 1e-4 absolute rule through the embedded self tests."""
import glob
import json
import os

import numpy as np
import pytest

import fdeep_b200
from fdeep_b200 import model_writer as mw
from util import assert_close, model_text, oracle_outputs

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
PATHS = [pytest.param(False, id="ffma"), pytest.param(True, id="tcgen05")]


def load(js_or_text, tensor_cores, verify=False):
    text = js_or_text if isinstance(js_or_text, str) else model_text(js_or_text)
    return fdeep_b200.read_model_from_string(text, verify=verify, tensor_cores=tensor_cores), text


def check_against_oracle(js, samples, tensor_cores, what, rel=1e-4):
    m, text = load(js, tensor_cores)
    got = m.predict_multi(samples)
    want = oracle_outputs(text, samples)
    assert len(got) == len(want)
    for s, (g, w) in enumerate(zip(got, want)):
        assert len(g) == len(w)
        for o, (a, b) in enumerate(zip(g, w)):
            assert_close(a, b, f"{what} sample {s} output {o}", rel=rel)
    return m, got


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_golden_fixtures(built_library, tensor_cores):
    files = sorted(glob.glob(os.path.join(HERE, "golden", "*.npz")))
    assert files
    for f in files:
        z = np.load(f, allow_pickle=False)
        text = bytes(z["model_json"]).decode()
        # verify=True runs the embedded self test on the GPU like fdeep::load_model does
        m = fdeep_b200.read_model_from_string(text, verify=True, verify_epsilon=1e-4, tensor_cores=tensor_cores)
        n_in, n_out, ns = int(z["n_in"]), int(z["n_out"]), int(z["n_samples"])
        samples = [[z[f"in_{s}_{i}"] for i in range(n_in)] for s in range(ns)]
        got = m.predict_multi(samples)
        for s in range(ns):
            for o in range(n_out):
                assert_close(got[s][o], z[f"out_{s}_{o}"], f"{os.path.basename(f)} sample {s} output {o}")


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_small_cnn_full_config(built_library, tensor_cores):
    """Config 1 as specified: 1024 inputs U[0,1) through predict_multi."""
    x = mw.inputs_small_cnn(1024)
    m, got = check_against_oracle(mw.build_small_cnn(), [[x[i]] for i in range(1024)], tensor_cores, "small_cnn")
    sums = np.array([g[0].sum() for g in got])
    np.testing.assert_allclose(sums, 1.0, atol=1e-5)
    assert m.launch_count() > 0


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_resnet50_reduced(built_library, tensor_cores):
    js = mw.build_resnet50(size=64, width=16, classes=10, top="linear")
    x = mw.inputs_resnet50(6, size=64)
    check_against_oracle(js, [[x[i]] for i in range(6)], tensor_cores, "resnet50/64px")


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_resnet50_full_size(built_library, tensor_cores):
    """ResNet-50 at 224x224x3 with the benchmark's weights: two images against the oracle, then
    batch-size independence on a larger batch (the oracle would take too long there)."""
    js = mw.build_resnet50(top="linear")  # logits: the softmax of random weights saturates
    x = mw.inputs_resnet50(18)
    m, got = check_against_oracle(js, [[x[i]] for i in range(2)], tensor_cores, "resnet50/224px")
    big = m.predict_batch([x])[0]
    assert big.shape == (18, 1000)
    np.testing.assert_array_equal(big[0], got[0][0])  # same arithmetic whatever the batch
    np.testing.assert_array_equal(big[1], got[1][0])
    single = m.predict([x[17]])[0]
    np.testing.assert_array_equal(big[17], single)


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_mobilenetv2(built_library, tensor_cores):
    js = mw.build_mobilenetv2(size=96, classes=16)
    x = mw.inputs_mobilenetv2(4, size=96)
    check_against_oracle(js, [[x[i]] for i in range(4)], tensor_cores, "mobilenetv2/96px")
    js = mw.build_mobilenetv2()
    x = mw.inputs_mobilenetv2(2)
    check_against_oracle(js, [[x[i]] for i in range(2)], tensor_cores, "mobilenetv2/224px")


@pytest.mark.parametrize("kind", ["max", "avg"])
def test_pooling_2d_shapes(built_library, kind):
    """Max and average pooling on the shapes the TMA-staged kernel takes (2 x 2 / 2 and 3 x 3 / 1, 2 with every window
    inside the tensor, or inside a frame of explicit zeros folded in from a ZeroPadding2D layer: those zeros count) and on
    shapes that stay with the general kernel (SAME padding, where clipped taps are skipped; other windows; few channels),
    several samples each, against the oracle."""
    rng = np.random.default_rng(11)
    pool = mw.max_pool2d if kind == "max" else mw.avg_pool2d
    cases = [(32, 32, 32, 2, 2, "valid", 0), (57, 55, 36, 3, 2, "valid", 0), (30, 29, 64, 3, 1, "valid", 0), (112, 112, 64, 3, 2, "valid", 1),
             (15, 17, 8, 2, 2, "valid", 1), (9, 10, 40, 3, 2, "same", 0), (7, 7, 16, 2, 2, "same", 0), (20, 20, 12, 4, 2, "valid", 0),
             (13, 13, 4, 3, 2, "valid", 0)]
    for (h, w, c, p_, s_, pad, frame) in cases:
        b = mw.ModelBuilder("pool")
        i = b.input([h, w, c])
        x = i
        hh, ww = h, w
        if frame:
            x = mw.zero_pad2d(b, x, "zp", ((frame, frame), (frame, frame)))
            hh, ww = h + 2 * frame, w + 2 * frame
        o = pool(b, x, "p", p_, s_, pad)
        oh = -(-hh // s_) if pad == "same" else (hh - p_) // s_ + 1
        ow = -(-ww // s_) if pad == "same" else (ww - p_) // s_ + 1
        js = b.to_json([o], [[oh, ow, c]])
        samples = [[(rng.normal(size=(h, w, c)) - 0.5).astype(np.float32)] for _ in range(3)]
        check_against_oracle(js, samples, True, f"{kind} pool {h}x{w}x{c} window {p_} stride {s_} {pad} frame {frame}", rel=1e-6)


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_errors_against_the_double_precision_arbiter(built_library, tensor_cores):
    """The engine and the fp32 oracle both measured against the oracle built in double precision (the reference's
    FDEEP_FLOAT_TYPE = double): on the benchmark models at reduced sizes the engine's error against that arbiter stays
    below 1e-4 and is of the size of the fp32 CPU arithmetic's own error (at most ten times it, or 1e-5), so what
    separates the engine from the fp32 oracle in the other tests is rounding noise, not a different result."""
    from util import arbiter_outputs, worst_relative
    cases = []
    x = mw.inputs_small_cnn(16)
    cases.append(("small_cnn", mw.build_small_cnn(), [[x[i]] for i in range(16)]))
    x = mw.inputs_resnet50(3, size=64)
    cases.append(("resnet50/64px", mw.build_resnet50(size=64, width=16, classes=10, top="linear"), [[x[i]] for i in range(3)]))
    x = mw.inputs_mobilenetv2(2, size=96)
    cases.append(("mobilenetv2/96px", mw.build_mobilenetv2(size=96, classes=16), [[x[i]] for i in range(2)]))
    ids = mw.inputs_text_lstm(3, vocab=500, seq_len=24)
    cases.append(("text_lstm", mw.build_text_lstm(vocab=500, dim=32, units=64, seq_len=24), [[ids[i]] for i in range(3)]))
    cfg = dict(vocab=307, ctx=48, dim=128, layers=3, heads=4, ffn=256)
    tok = mw.inputs_gpt2_prompts(4, vocab=307, prompt_len=1)
    cases.append(("gpt2 first position", mw.build_gpt2_step(first=True, **cfg),
                  [[tok[i, :1].astype(np.float32), np.zeros(1, np.float32)] for i in range(4)]))
    for name, js, samples in cases:
        m, text = load(js, tensor_cores)
        got = m.predict_multi(samples)
        cpu = oracle_outputs(text, samples)
        truth = arbiter_outputs(text, samples)
        e_gpu = max(worst_relative(got[s][o], truth[s][o]) for s in range(len(samples)) for o in range(len(truth[s])))
        e_cpu = max(worst_relative(cpu[s][o], truth[s][o]) for s in range(len(samples)) for o in range(len(truth[s])))
        assert e_gpu <= 1e-4, f"{name}: engine is {e_gpu:.2e} from the double-precision result"
        assert e_gpu <= max(10.0 * e_cpu, 1e-5), f"{name}: engine error {e_gpu:.2e} against fp32 CPU error {e_cpu:.2e}"


@pytest.mark.parametrize("h,w,c,stride,pad,act", [
    (9, 11, 8, 1, "same", "linear"), (17, 13, 36, 2, "same", "relu"), (30, 30, 40, 1, "valid", "relu6"), (15, 16, 100, 2, "valid", "linear"),
    (56, 56, 144, 1, "same", "relu6"), (57, 55, 96, 2, "same", "relu6"), (7, 7, 320, 1, "same", "relu"), (3, 3, 64, 1, "same", "linear"),
    (29, 31, 4, 1, "same", "relu"), (14, 14, 20, 2, "same", "tanh")])
def test_depthwise_3x3_shapes(built_library, h, w, c, stride, pad, act):
    """Depthwise 3 x 3 on the shapes the TMA-staged kernel tiles in different ways (channel counts that are not multiples
    of 32, images smaller and larger than a tile, both strides and paddings, zero padding folded in from a ZeroPadding2D
    layer, bias / BatchNormalization / residual / activation in the epilogue) and on shapes that fall back to the general
    kernel (fewer than 8 channels): the engine against the oracle and against torch in float64."""
    import torch
    import torch.nn.functional as F
    from test_oracle import tf_same_pad
    rng = np.random.default_rng(h * 100 + w + c)
    kernel = rng.normal(size=(3, 3, c, 1)).astype(np.float32)
    bias = rng.normal(size=c).astype(np.float32)
    b = mw.ModelBuilder("dw")
    i = b.input([h, w, c])
    x = i
    extra = pad == "valid" and stride == 2
    if extra:
        x = mw.zero_pad2d(b, x, "zp", ((0, 1), (0, 1)))   # MobileNet's stride-2 blocks pad like this
    keras_act = {"relu6": "linear"}.get(act, act)
    o = mw.depthwise_conv2d(b, x, "d", kernel, bias, strides=stride, padding=pad, activation=keras_act)
    hh, ww = (h + 1, w + 1) if extra else (h, w)
    oh = -(-hh // stride) if pad == "same" else (hh - 3) // stride + 1
    ow = -(-ww // stride) if pad == "same" else (ww - 3) // stride + 1
    mean, var = rng.normal(size=c).astype(np.float32), rng.uniform(0.5, 2.0, size=c).astype(np.float32)
    gamma, beta = rng.normal(size=c).astype(np.float32), rng.normal(size=c).astype(np.float32)
    o = mw.batch_norm(b, o, "bn", mean, var, gamma, beta)
    if act == "relu6":
        o = mw.relu(b, o, "r6", max_value=6.0)
    if stride == 1 and pad == "same":
        o = mw.add_layers(b, [o, i], "res")
    js = b.to_json([o], [[oh, ow, c]])
    samples = [[rng.normal(size=(h, w, c)).astype(np.float32)] for _ in range(5)]
    m, got = check_against_oracle(js, samples, True, f"depthwise {h}x{w}x{c} s{stride} {pad}", rel=2e-5)
    xt = torch.from_numpy(samples[0][0]).double().permute(2, 0, 1)[None]
    if extra:
        xt = F.pad(xt, (0, 1, 0, 1))
    if pad == "same":
        pt, pb = tf_same_pad(hh, 3, stride)
        pl, pr = tf_same_pad(ww, 3, stride)
        xt = F.pad(xt, (pl, pr, pt, pb))
    y = F.conv2d(xt, torch.from_numpy(kernel).double().permute(2, 3, 0, 1), torch.from_numpy(bias).double(), stride=stride, groups=c)
    y = {"linear": lambda v: v, "relu6": lambda v: v, "relu": torch.relu, "tanh": torch.tanh}[act](y)
    inv = torch.from_numpy(gamma).double() / torch.sqrt(torch.from_numpy(var).double() + 1e-3)
    y = y * inv[None, :, None, None] + (torch.from_numpy(beta).double() - torch.from_numpy(mean).double() * inv)[None, :, None, None]
    if act == "relu6":
        y = torch.clamp(y, 0.0, 6.0)
    if stride == 1 and pad == "same":
        y = y + torch.from_numpy(samples[0][0]).double().permute(2, 0, 1)[None]
    np.testing.assert_allclose(got[0][0], y[0].permute(1, 2, 0).numpy(), rtol=1e-4, atol=2e-5)


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_text_lstm(built_library, tensor_cores):
    js = mw.build_text_lstm(vocab=500, dim=32, units=64, seq_len=20)
    x = mw.inputs_text_lstm(16, vocab=500, seq_len=20)
    check_against_oracle(js, [[x[i]] for i in range(16)], tensor_cores, "text_lstm/reduced")
    js = mw.build_text_lstm()  # config 4 as specified, a few sequences
    x = mw.inputs_text_lstm(4)
    check_against_oracle(js, [[x[i]] for i in range(4)], tensor_cores, "text_lstm/full")


def greedy_decode(predict_first, predict_step, prompts, new_tokens, layers):
    """Greedy loop over the incremental graphs: consume the prompt token by token, then generate."""
    n = prompts.shape[0]
    pasts = [[None] * layers for _ in range(n)]
    logits_log, tokens = [[] for _ in range(n)], [[] for _ in range(n)]
    total = prompts.shape[1] + new_tokens
    cur = prompts[:, 0].copy()
    for pos in range(total - 1):
        samples = []
        for s in range(n):
            base = [np.array([cur[s]], np.float32), np.array([float(pos)], np.float32)]
            samples.append(base if pos == 0 else base + pasts[s])
        outs = predict_first(samples) if pos == 0 else predict_step(samples)
        for s in range(n):
            logits = outs[s][0]
            for l in range(layers):
                row = outs[s][1 + l]
                pasts[s][l] = row if pos == 0 else np.concatenate([pasts[s][l], row], axis=0)
            logits_log[s].append(logits)
            if pos + 1 < prompts.shape[1]:
                cur[s] = prompts[s, pos + 1]
            else:
                cur[s] = float(np.argmax(logits[0]))
                tokens[s].append(int(cur[s]))
    return logits_log, tokens


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_gpt2_incremental_decode(built_library, tensor_cores):
    from oracle import OracleModel
    cfg = dict(vocab=211, ctx=64, dim=64, layers=3, heads=4, ffn=128)
    first_js, step_js = mw.build_gpt2_step(first=True, **cfg), mw.build_gpt2_step(first=False, **cfg)
    prompts = mw.inputs_gpt2_prompts(3, vocab=211, prompt_len=5)
    mf, tf = load(first_js, tensor_cores)
    ms, ts = load(step_js, tensor_cores)
    of, os_ = OracleModel(json_text=tf), OracleModel(json_text=ts)
    g_logits, g_tok = greedy_decode(mf.predict_multi, ms.predict_multi, prompts, 8, cfg["layers"])
    o_logits, o_tok = greedy_decode(lambda s: of.predict_multi(s), lambda s: os_.predict_multi(s), prompts, 8, cfg["layers"])
    assert g_tok == o_tok
    for s in range(3):
        for step, (a, b) in enumerate(zip(g_logits[s], o_logits[s])):
            assert_close(a, b, f"gpt2 seq {s} step {step}")


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_ragged_shapes_keep_input_order(built_library, tensor_cores):
    """Samples of different (variable) shapes in one predict_multi call are grouped internally and
    come back in input order."""
    cfg = dict(vocab=101, ctx=32, dim=32, layers=2, heads=4, ffn=64)
    js = mw.build_gpt2_step(**cfg)
    rng = np.random.default_rng(3)
    lens = [3, 7, 3, 1, 7, 12]
    samples = [[np.array([float(rng.integers(0, 101))], np.float32), np.array([float(n)], np.float32)] +
               [rng.normal(0, 1, (n, 32)).astype(np.float32) for _ in range(2)] for n in lens]
    check_against_oracle(js, samples, tensor_cores, "ragged gpt2 step")


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_batch_position_invariance(built_library, tensor_cores):
    """A sample's result must not depend on the batch size or its place in the batch (the sharding of
    predict_multi must not change arithmetic)."""
    m, _ = load(mw.build_resnet50(size=64, width=16, classes=10), tensor_cores)
    x = mw.inputs_resnet50(37, size=64)
    full = m.predict_batch([x])[0]
    part = m.predict_batch([x[20:29]])[0]
    np.testing.assert_array_equal(full[20:29], part)
    np.testing.assert_array_equal(full[36], m.predict([x[36]])[0])


def test_device_resident_matches_host_path(built_library):
    import torch
    m, _ = load(mw.build_small_cnn(), True)
    x = mw.inputs_small_cnn(64)
    host = m.predict_batch([x])[0]
    d_in = torch.from_numpy(x).cuda()
    d_out = torch.empty((64, 10), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    m.predict_batch_device([d_in.data_ptr()], [[32, 32, 3]], 64, [d_out.data_ptr()])
    m.sync()
    np.testing.assert_array_equal(d_out.cpu().numpy(), host)


def test_two_streams_take_turns_on_one_model(built_library):
    """Calls on one model queued on two different streams without any synchronisation in between share the device's
    intermediate buffers; the library orders them on the device, so every call must give what it gives alone."""
    import torch
    m, _ = load(mw.build_resnet50(size=64, width=16, classes=10, top="linear"), True)
    xs = [mw.inputs_resnet50(24, size=64, seed=5 + i) for i in range(4)]
    want = [m.predict_batch([x])[0] for x in xs]
    d_in = [torch.from_numpy(x).cuda() for x in xs]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    torch.cuda.synchronize()
    for rep in range(3):
        d_out = [torch.full((24, 10), float("nan"), device="cuda") for _ in xs]
        torch.cuda.synchronize()
        for i in range(len(xs)):
            m.predict_batch_device([d_in[i].data_ptr()], [[64, 64, 3]], 24, [d_out[i].data_ptr()], stream=streams[i % 2].cuda_stream)
        torch.cuda.synchronize()
        m.sync()
        for i in range(len(xs)):
            np.testing.assert_array_equal(d_out[i].cpu().numpy(), want[i], err_msg=f"round {rep}, call {i}")


def test_predict_from_several_host_threads(built_library):
    """model::predict is const and may be called from several threads on one shared model (the reference's own
    concurrency exercise is predict_multi(..., parallelly = true)): four threads, each with its own samples, must get
    what a single thread gets."""
    import threading
    m, _ = load(mw.build_small_cnn(), True)
    x = mw.inputs_small_cnn(4 * 24)
    want = m.predict_batch([x])[0]
    results, errors = {}, []

    def worker(t):
        try:
            out = []
            for rep in range(6):
                for i in range(t * 24, (t + 1) * 24, 8):
                    out.append(m.predict_batch([x[i:i + 8]])[0])
            results[t] = out
        except Exception as e:  # pragma: no cover - reported below
            errors.append(e)

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(4)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors
    for t in range(4):
        for k, got in enumerate(results[t]):
            i = t * 24 + (k % 3) * 8
            np.testing.assert_array_equal(got, want[i:i + 8])


def test_in_process_multi_device_matches_one_device(built_library):
    """predict_multi on one model loaded on several devices (contiguous blocks of ceil(n / G) samples, one host thread,
    stream and weight replica per device): bitwise what the one-device model gives, in input order, for a sample count
    that does not divide evenly and for ragged (variable-shape) samples.  Needs at least two GPUs."""
    n_dev = fdeep_b200.device_count()
    if n_dev < 2:
        pytest.skip("needs at least two CUDA devices")
    text = model_text(mw.build_resnet50(size=64, width=16, classes=10, top="linear"))
    one = fdeep_b200.read_model_from_string(text, verify=False, devices=[0])
    x = mw.inputs_resnet50(37, size=64)
    want = one.predict_batch([x])[0]
    for g in (2, 4, 8):
        if g > n_dev:
            break
        many = fdeep_b200.read_model_from_string(text, verify=False, devices=list(range(g)))
        assert many.num_devices() == g
        got = many.predict_batch([x])[0]
        np.testing.assert_array_equal(got, want, err_msg=f"{g} devices")
        separate = many.predict_multi([[np.array(x[i])] for i in range(37)])
        for i in range(37):
            np.testing.assert_array_equal(separate[i][0], want[i], err_msg=f"{g} devices, sample {i}")
    # ragged samples: shape groups are sharded one by one, results return in input order
    cfg = dict(vocab=101, ctx=32, dim=32, layers=2, heads=4, ffn=64)
    text = model_text(mw.build_gpt2_step(**cfg))
    rng = np.random.default_rng(3)
    lens = [3, 7, 3, 1, 7, 12, 3, 3, 7, 1, 3]
    samples = [[np.array([float(rng.integers(0, 101))], np.float32), np.array([float(n)], np.float32)] +
               [rng.normal(0, 1, (n, 32)).astype(np.float32) for _ in range(2)] for n in lens]
    want = fdeep_b200.read_model_from_string(text, verify=False, devices=[0]).predict_multi(samples)
    got = fdeep_b200.read_model_from_string(text, verify=False, devices=list(range(min(n_dev, 4)))).predict_multi(samples)
    for s in range(len(lens)):
        for a, b in zip(got[s], want[s]):
            np.testing.assert_array_equal(a, b, err_msg=f"ragged sample {s}")


def test_embedding_index_out_of_range_raises(built_library):
    b = mw.ModelBuilder("m")
    i = b.input([3])
    o = mw.embedding(b, i, "e", np.zeros((4, 2), np.float32))
    m, _ = load(b.to_json([o], [[3, 2]]), True)
    m.predict([np.array([0.0, 3.0, 1.0], np.float32)])
    with pytest.raises(fdeep_b200.FdeepError, match="strictly less"):
        m.predict([np.array([0.0, 4.0, 1.0], np.float32)])
    m.predict([np.array([2.0, 3.0, 1.0], np.float32)])  # the context stays usable


def test_shape_errors_at_predict(built_library):
    m, _ = load(mw.build_small_cnn(), True)
    with pytest.raises(fdeep_b200.FdeepError, match="Invalid inputs shape"):
        m.predict([np.zeros((16, 32, 3), np.float32)])
    assert m.get_input_shapes() == [[32, 32, 3]] and m.get_output_shapes() == [[10]]
    assert m.name() == "small_cnn" and len(m.hash()) == 64
    assert m.predict_multi([]) == []


@pytest.mark.parametrize("path", [pytest.param(0, id="ffma"), pytest.param(1, id="tcgen05")])
@pytest.mark.parametrize("M,N,K", [(128, 128, 32), (300, 72, 64), (1000, 200, 100), (77, 10, 36), (4096, 256, 2304), (1, 1000, 2048),
                                   (129, 65, 4), (513, 384, 1152)])
def test_gemm_kernel(built_library, path, M, N, K):
    """fdk_gemm against a float64 product.  The tcgen05 path must keep fp32-class accuracy (3xTF32)."""
    import torch
    g = torch.Generator(device="cpu").manual_seed(M * 7 + N * 3 + K)
    A = torch.randn(M, K, generator=g)
    W = torch.randn(N, K, generator=g)
    bias = torch.randn(N, generator=g)
    want = torch.relu(A.double() @ W.double().T + bias.double())
    dA, dW, dB = A.cuda(), W.cuda(), bias.cuda()
    dC = torch.full((M, N), float("nan"), device="cuda")
    torch.cuda.synchronize()
    fdeep_b200.gemm(path, dA.data_ptr(), K, dW.data_ptr(), K, dC.data_ptr(), N, M, N, K, d_bias=dB.data_ptr(), relu=True)
    torch.cuda.synchronize()
    got = dC.cpu().double()
    # error relative to the magnitude of the terms of the dot product, as for any fp32 GEMM
    denom = (A.double().abs() @ W.double().abs().T + bias.double().abs()).clamp_min(1e-30)
    err = ((got - want).abs() / denom).max().item()
    assert err < 2e-6, f"path {path} {M}x{N}x{K}: relative error {err:.3e}"


def test_tile_width_does_not_change_results(built_library):
    """The contraction kernel takes 64-column tiles when 128-column tiles would leave half of the SMs idle (few rows).
    That choice depends on the number of rows, so it must not touch a result: the first rows of a large product (wide
    tiles) equal, bit for bit, the same rows computed alone (narrow tiles), with a bias, a ReLU and a ragged last tile."""
    import torch
    from fdeep_b200 import capi
    torch.manual_seed(5)
    for N, K in ((512, 1152), (1000, 256), (200, 96)):
        big, small = 40000, 300
        A = torch.randn(big, K, device="cuda")
        W = torch.randn(N, K, device="cuda")
        b = torch.randn(N, device="cuda")
        C1 = torch.empty(big, N, device="cuda")
        C2 = torch.empty(small, N, device="cuda")
        capi.gemm(1, A.data_ptr(), K, W.data_ptr(), K, C1.data_ptr(), N, big, N, K, d_bias=b.data_ptr(), relu=True)
        capi.gemm(1, A.data_ptr(), K, W.data_ptr(), K, C2.data_ptr(), N, small, N, K, d_bias=b.data_ptr(), relu=True)
        torch.cuda.synchronize()
        assert capi.tc_status() == 0
        assert torch.equal(C1[:small], C2), f"N={N} K={K}"
        ref = torch.relu(A[:small].double() @ W.double().T + b.double())
        assert float((C2.double() - ref).abs().max()) <= 2e-6 * float((A[:small].abs().double() @ W.abs().double().T).max())


@pytest.mark.parametrize("M,N,K", [(64, 768, 768), (64, 768, 3072), (64, 3072, 768), (1, 1000, 2048), (37, 1001, 260), (64, 50257, 768),
                                   (5, 300, 64), (64, 64, 36), (3, 130, 8), (64, 2304, 768), (17, 8, 4), (64, 128, 32)])
def test_row_product_kernel(built_library, M, N, K):
    """The tcgen05 kernel for products of at most 64 rows (fdk_gemm path 3: blocks of weight rows x slices of K, one
    thread-block cluster per block, partial tiles summed through distributed shared memory) against a float64
    product: full and ragged blocks, K with a partial last k block, rows and columns that are not multiples of four,
    one slice and eight.  Twice each: the second launch finds the first one's leftovers in shared memory."""
    import torch
    g = torch.Generator(device="cpu").manual_seed(M * 7 + N * 3 + K)
    A, W, bias = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g), torch.randn(N, generator=g)
    want = torch.relu(A.double() @ W.double().T + bias.double())
    denom = (A.double().abs() @ W.double().abs().T + bias.double().abs()).clamp_min(1e-30)
    dA, dW, dB = A.cuda(), W.cuda(), bias.cuda()
    results = []
    for rep in range(2):
        dC = torch.full((M, N), float("nan"), device="cuda")
        torch.cuda.synchronize()
        fdeep_b200.gemm(3, dA.data_ptr(), K, dW.data_ptr(), K, dC.data_ptr(), N, M, N, K, d_bias=dB.data_ptr(), relu=True)
        torch.cuda.synchronize()
        got = dC.cpu().double()
        err = ((got - want).abs() / denom).max().item()
        assert err < 2e-6, f"{M}x{N}x{K}: relative error {err:.3e}"
        results.append(got)
    assert torch.equal(results[0], results[1])
    # the rows of a product do not depend on how many rows the launch has
    if M > 2:
        dC = torch.full((2, N), float("nan"), device="cuda")
        fdeep_b200.gemm(3, dA.data_ptr(), K, dW.data_ptr(), K, dC.data_ptr(), N, 2, N, K, d_bias=dB.data_ptr(), relu=True)
        torch.cuda.synchronize()
        assert torch.equal(dC.cpu().double(), results[0][:2])


@pytest.mark.parametrize("mma", ["0", "1"], ids=["ffma", "mma_3xtf32"])
def test_skinny_gemm_kernel(built_library, mma):
    """The weight-streaming kernel for at most 64 rows (fdk_gemm path 2) against a float64 product, in both of its
    forms: exact FFMA products (FDK_SKINNY_MMA=0) and three TF32 tensor-core products per fp32 product (the default; chosen when the
    library is first asked; hence a child process per form).  Single-slice and sliced shapes, ragged edges."""
    import subprocess, sys, textwrap
    code = textwrap.dedent("""
        import sys, torch
        sys.path.insert(0, %r)
        import fdeep_b200
        worst = 0.0
        for M, N, K in [(64, 768, 768), (64, 768, 3072), (64, 3072, 768), (1, 1000, 2048), (37, 1001, 260), (64, 50257, 768), (5, 300, 64), (64, 64, 36)]:
            g = torch.Generator(device="cpu").manual_seed(M * 7 + N * 3 + K)
            A, W, bias = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g), torch.randn(N, generator=g)
            want = torch.relu(A.double() @ W.double().T + bias.double())
            dA, dW, dB = A.cuda(), W.cuda(), bias.cuda()
            for rep in range(2):   # twice: the arrival counters must be back at zero
                dC = torch.full((M, N), float("nan"), device="cuda")
                torch.cuda.synchronize()
                fdeep_b200.gemm(2, dA.data_ptr(), K, dW.data_ptr(), K, dC.data_ptr(), N, M, N, K, d_bias=dB.data_ptr(), relu=True)
                torch.cuda.synchronize()
                got = dC.cpu().double()
                denom = (A.double().abs() @ W.double().abs().T + bias.double().abs()).clamp_min(1e-30)
                err = ((got - want).abs() / denom).max().item()
                assert err < 2e-6, f"{M}x{N}x{K}: relative error {err:.3e}"
                worst = max(worst, err)
        print("worst", worst)
    """ % os.path.join(os.path.dirname(HERE), "frugally-deep_b200"))
    env = dict(os.environ, FDK_SKINNY_MMA=mma)
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_decode_session_matches_host_loop(built_library, tensor_cores):
    """The device-resident decode session (key/value rows kept on the GPU, greedy choice on the GPU) against the
    same loop carried through host memory with predict_multi, and against the oracle's token choice."""
    from oracle import OracleModel
    cfg = dict(vocab=211, ctx=64, dim=64, layers=3, heads=4, ffn=128)
    first_js, step_js = mw.build_gpt2_step(first=True, **cfg), mw.build_gpt2_step(first=False, **cfg)
    prompts = mw.inputs_gpt2_prompts(3, vocab=211, prompt_len=5)
    new_tokens = 8
    mf, tf = load(first_js, tensor_cores)
    ms, ts = load(step_js, tensor_cores)
    h_logits, h_tok = greedy_decode(mf.predict_multi, ms.predict_multi, prompts, new_tokens, cfg["layers"])
    of, os_ = OracleModel(json_text=tf), OracleModel(json_text=ts)
    _, o_tok = greedy_decode(lambda s: of.predict_multi(s), lambda s: os_.predict_multi(s), prompts, new_tokens, cfg["layers"])
    total = prompts.shape[1] + new_tokens
    sess = fdeep_b200.DecodeSession(mf, ms, batch=3, max_len=total)
    s_tok = [[] for _ in range(3)]
    for pos in range(total - 1):
        feed = prompts[:, pos] if pos < prompts.shape[1] else None
        nxt, logits = sess.step(feed, want_logits=True)
        for s in range(3):
            assert_close(logits[s], h_logits[s][pos][0], f"session logits seq {s} pos {pos}", rel=1e-6)
            if pos + 1 >= prompts.shape[1]:
                s_tok[s].append(int(nxt[s]))
    assert sess.length == total - 1
    assert s_tok == h_tok == o_tok
    with pytest.raises(fdeep_b200.FdeepError, match="max_len"):
        sess.step(None)
        sess.step(None)
    # a new batch of sequences in the same session (fdk_session_reset): other prompts first, then the first ones again,
    # which must give the same logits and tokens bit for bit (buffers and the recorded position are reused)
    other = mw.inputs_gpt2_prompts(3, seed=9, vocab=211, prompt_len=5)
    runs = []
    for p in (other, prompts):
        sess.reset()
        assert sess.length == 0
        with pytest.raises(fdeep_b200.FdeepError, match="needs tokens"):
            sess.step(None)
        sess.reset()
        log = []
        for pos in range(total - 1):
            nxt, logits = sess.step(p[:, pos] if pos < p.shape[1] else None, want_logits=True)
            log.append((nxt.copy(), logits.copy()))
        runs.append(log)
    for pos in range(total - 1):
        for s in range(3):
            assert_close(runs[1][pos][1][s], h_logits[s][pos][0], f"session after reset: logits seq {s} pos {pos}", rel=1e-6)
    again = [[int(runs[1][pos][0][s]) for pos in range(prompts.shape[1] - 1, total - 1)] for s in range(3)]
    assert again == h_tok
    assert not all(np.array_equal(a[1], b[1]) for a, b in zip(runs[0], runs[1]))
    sess.close()


def test_skinny_products_flag(built_library):
    """Opt-in weight-streaming split-K kernel for products with at most 64 rows (dense heads, one decode position):
    the decode loop with it, through the session with its key/value cache, against the oracle."""
    from oracle import OracleModel
    cfg = dict(vocab=307, ctx=32, dim=256, layers=2, heads=4, ffn=1024)
    first_js, step_js = mw.build_gpt2_step(first=True, **cfg), mw.build_gpt2_step(first=False, **cfg)
    tf, ts = model_text(first_js), model_text(step_js)
    mf = fdeep_b200.read_model_from_string(tf, verify=False, skinny_products=True)
    ms = fdeep_b200.read_model_from_string(ts, verify=False, skinny_products=True)
    prompts = mw.inputs_gpt2_prompts(5, vocab=307, prompt_len=4)
    new_tokens = 6
    of, os_ = OracleModel(json_text=tf), OracleModel(json_text=ts)
    o_logits, o_tok = greedy_decode(lambda s: of.predict_multi(s), lambda s: os_.predict_multi(s), prompts, new_tokens, cfg["layers"])
    total = prompts.shape[1] + new_tokens
    sess = fdeep_b200.DecodeSession(mf, ms, batch=5, max_len=total)
    tok = [[] for _ in range(5)]
    for pos in range(total - 1):
        nxt, logits = sess.step(prompts[:, pos] if pos < prompts.shape[1] else None, want_logits=True)
        for s in range(5):
            assert_close(logits[s], o_logits[s][pos][0], f"skinny session seq {s} pos {pos}")
            if pos + 1 >= prompts.shape[1]:
                tok[s].append(int(nxt[s]))
    assert tok == o_tok
    sess.close()


@pytest.fixture(scope="module")
def gpt2_small(built_library):
    """Config 5 at its configured shape (GPT-2-small: 12 blocks, width 768, 12 heads, feed-forward 3072, vocabulary
    50257, 1024 positions), loaded exactly as the benchmark loads it (products of at most 64 rows on the
    weight-streaming kernel), next to the oracle on the same two model files.  Built once: each file is 0.87 GB."""
    from oracle import OracleModel
    cfg = dict(vocab=50257, ctx=1024, dim=768, layers=12, heads=12, ffn=3072)
    tf = model_text(mw.build_gpt2_step(first=True, **cfg))
    mf = fdeep_b200.read_model_from_string(tf, verify=False, skinny_products=True)
    of = OracleModel(json_text=tf)
    del tf
    ts = model_text(mw.build_gpt2_step(first=False, **cfg))
    ms = fdeep_b200.read_model_from_string(ts, verify=False, skinny_products=True)
    os_ = OracleModel(json_text=ts)
    del ts
    return cfg, mf, ms, of, os_


def test_gpt2_small_decode_at_configured_shape(gpt2_small, monkeypatch):
    """The benchmarked decode configuration against the oracle: 64 sequences in the session (the batch the benchmark
    runs), an 8-token prompt and 8 generated tokens; the first 4 sequences are also run through the oracle's own
    greedy loop over the two incremental graphs.  Logits within 1e-4 at every position, identical greedy ids, with the
    positions replayed from the recorded graph and launched one by one."""
    cfg, mf, ms, of, os_ = gpt2_small
    n_seq, n_check, prompt_len, new_tokens = 64, 4, 8, 8
    prompts = mw.inputs_gpt2_prompts(n_seq, vocab=cfg["vocab"], prompt_len=prompt_len)
    o_logits, o_tok = greedy_decode(lambda s: of.predict_multi(s, threads=n_check), lambda s: os_.predict_multi(s, threads=n_check),
                                    prompts[:n_check], new_tokens, cfg["layers"])
    total = prompt_len + new_tokens
    runs = {}
    for graph in ("1", "0"):
        monkeypatch.setenv("FDK_SESSION_GRAPH", graph)
        sess = fdeep_b200.DecodeSession(mf, ms, batch=n_seq, max_len=total)
        tok = [[] for _ in range(n_check)]
        log = []
        for pos in range(total - 1):
            nxt, logits = sess.step(prompts[:, pos] if pos < prompt_len else None, want_logits=True)
            log.append(logits.copy())
            for s in range(n_check):
                assert_close(logits[s], o_logits[s][pos][0], f"gpt2-small graph={graph} seq {s} pos {pos}")
                if pos + 1 >= prompt_len:
                    tok[s].append(int(nxt[s]))
        sess.close()
        assert tok == o_tok, f"greedy ids differ from the oracle's (graph={graph})"
        runs[graph] = log
    for a, b in zip(runs["1"], runs["0"]):
        assert np.array_equal(a, b), "replayed and directly launched positions differ"


@pytest.mark.parametrize("skinny", [False, True], ids=["tiles", "skinny"])
def test_decode_session_replayed_positions(built_library, skinny, monkeypatch):
    """A session keeps its length on the device and replays the launches of a position from a recorded graph.  The
    logits and tokens must not depend on that: the same decode with the length on the host (one plan per length,
    FDK_SESSION_DEVICE_LEN=0), launched directly (FDK_SESSION_GRAPH=0) and replayed, and two sessions of different
    batch sizes taking turns on the same models (the larger one makes the engine's arena grow, so the smaller one's
    recording must be renewed)."""
    cfg = dict(vocab=307, ctx=48, dim=128, layers=3, heads=4, ffn=256)
    tf, ts = model_text(mw.build_gpt2_step(first=True, **cfg)), model_text(mw.build_gpt2_step(first=False, **cfg))
    mf = fdeep_b200.read_model_from_string(tf, verify=False, skinny_products=skinny)
    ms = fdeep_b200.read_model_from_string(ts, verify=False, skinny_products=skinny)
    prompts = mw.inputs_gpt2_prompts(7, vocab=307, prompt_len=4)
    total = 20

    def decode(n_seq, interleave_with=None):
        sess = fdeep_b200.DecodeSession(mf, ms, batch=n_seq, max_len=total)
        other = fdeep_b200.DecodeSession(mf, ms, batch=interleave_with, max_len=total) if interleave_with else None
        out = []
        for pos in range(total):
            nxt, logits = sess.step(prompts[:n_seq, pos] if pos < prompts.shape[1] else None, want_logits=True)
            out.append((nxt.copy(), logits.copy()))
            if other is not None and pos >= 3:
                other.step(prompts[:interleave_with, pos - 3] if pos - 3 < prompts.shape[1] else None)
        sess.close()
        if other is not None:
            other.close()
        return out

    monkeypatch.setenv("FDK_SESSION_DEVICE_LEN", "0")
    host_len = decode(3)
    monkeypatch.delenv("FDK_SESSION_DEVICE_LEN")
    monkeypatch.setenv("FDK_SESSION_GRAPH", "0")
    direct = decode(3)
    monkeypatch.delenv("FDK_SESSION_GRAPH")
    replayed = decode(3)
    shared = decode(3, interleave_with=7)
    for pos in range(total):
        for name, run in (("direct", direct), ("replayed", replayed), ("replayed, engine shared", shared)):
            assert np.array_equal(run[pos][0], host_len[pos][0]), f"{name}: tokens differ at position {pos}"
            assert np.array_equal(run[pos][1], host_len[pos][1]), f"{name}: logits differ at position {pos}"


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_rms_unit_group_normalisation(built_library, tensor_cores):
    from test_oracle import norms_model
    js, x, wants = norms_model()
    m, got = check_against_oracle(js, [[x], [x * 3.0 + 1.0]], tensor_cores, "normalisations", rel=1e-5)
    for g, w, name in zip(got[0], wants, ("rms", "unit", "group", "group_plain")):
        assert_close(g, w.astype(np.float32), name, rel=1e-5)


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_gru_without_reset_after(built_library, tensor_cores):
    from test_oracle import gru_plain_model
    for T, Fdim, U in ((6, 4, 8), (5, 7, 5), (12, 32, 64)):
        js, x, _ = gru_plain_model(T, Fdim, U, seed=T)
        rng = np.random.default_rng(U)
        xs = [[rng.normal(size=x.shape).astype(np.float32)] for _ in range(9)]
        check_against_oracle(js, xs, tensor_cores, f"gru reset_after=False T{T} F{Fdim} U{U}")


def test_weight_text_forms_decode_alike(built_library):
    """decode_floats (import_model.hpp:136-171): the exporter's 1024-character base64 chunks (decoded on several host
    threads when the array is large), one unchunked string with padding, chunks that cut through a group of four
    characters, text with line breaks, and plain numbers must load the same weights."""
    rng = np.random.default_rng(77)
    K, N = 1031, 1100   # 1.1 M floats: the threaded path; K * N * 4 bytes is not a multiple of 3: padded text
    kernel = (rng.normal(size=(K, N)) * 0.05).astype(np.float32)
    small = (rng.normal(size=(N, 7)) * 0.05).astype(np.float32)
    bias = rng.normal(size=7).astype(np.float32)
    b = mw.ModelBuilder("m")
    i = b.input([K])
    d = mw.dense(b, mw.dense(b, i, "wide", kernel, None), "narrow", small, bias)
    js = b.to_json([d], [[7]])
    xs = [[rng.normal(size=K).astype(np.float32)] for _ in range(5)]
    base = fdeep_b200.read_model_from_string(model_text(js), verify=False).predict_multi(xs)
    want = [x[0].astype(np.float64) @ kernel.astype(np.float64) @ small.astype(np.float64) + bias for x in xs]
    for s in range(5):
        assert_close(base[s][0], want[s].astype(np.float32), "dense chain vs float64")

    def rewritten(form):
        out = json.loads(json.dumps(js))
        for layer, params in out["trainable_params"].items():
            for key, val in params.items():
                text = "".join(val)
                if form == "one string":
                    params[key] = text
                elif form == "odd chunks":
                    params[key] = [text[j:j + 1001] for j in range(0, len(text), 1001)]
                elif form == "line breaks":
                    params[key] = ["\n".join(text[j:j + 76] for j in range(0, len(text), 76))]
                elif form == "numbers" and layer == "narrow":
                    params[key] = [float(v) for v in (small.reshape(-1) if key == "weights" else bias)]
        return out

    for form in ("one string", "odd chunks", "line breaks", "numbers"):
        got = fdeep_b200.read_model_from_string(model_text(rewritten(form)), verify=False).predict_multi(xs)
        for s in range(5):
            assert np.array_equal(got[s][0], base[s][0]), f"{form}: sample {s} differs"


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_conv2d_transpose_shapes(built_library, tensor_cores):
    """Conv2DTranspose (convolution.hpp:443-469): on the tensor-core path as one stride-1 implicit GEMM per output phase
    (input channels a multiple of 4), else through the gathered patch matrix; against the oracle and torch."""
    from test_oracle import CONV2D_TRANSPOSE_CASES, conv2d_transpose_model
    rng = np.random.default_rng(31)
    for case in CONV2D_TRANSPOSE_CASES:
        js, x, want = conv2d_transpose_model(case)
        xs = [[x]] + [[rng.normal(size=x.shape).astype(np.float32)] for _ in range(4)]
        m, got = check_against_oracle(js, xs, tensor_cores, f"conv2d transpose {case}")
        assert_close(got[0][0], want.astype(np.float32), f"conv2d transpose {case} vs torch")
    # with what the plan folds into the epilogue: batch normalisation, a residual Add and a ReLU
    H, W, C, N = 9, 7, 8, 16
    b = mw.ModelBuilder("m")
    i = b.input([H, W, C])
    skip = b.input([2 * H, 2 * W, N])
    t = mw.conv2d_transpose(b, i, "up", (rng.normal(size=(4, 4, N, C)) * 0.2).astype(np.float32), rng.normal(size=N).astype(np.float32), 2, "same")
    t = mw.batch_norm(b, t, "bn", rng.normal(size=N).astype(np.float32), rng.uniform(0.5, 2.0, size=N).astype(np.float32),
                      rng.normal(size=N).astype(np.float32), rng.normal(size=N).astype(np.float32))
    t = mw.add_layers(b, [t, skip], "add")
    t = mw.relu(b, t, "relu")
    js = b.to_json([t], [[2 * H, 2 * W, N]])
    xs = [[rng.normal(size=(H, W, C)).astype(np.float32), rng.normal(size=(2 * H, 2 * W, N)).astype(np.float32)] for _ in range(70)]
    check_against_oracle(js, xs, tensor_cores, "conv2d transpose + bn + add + relu")


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_recurrent_layers_on_two_chains(built_library, tensor_cores):
    """From 256 samples on, the two halves of a batch walk their time steps on two streams (recurrent_ops.hpp:117-293 per
    sample, samples are independent): every sample must come out bit for bit as in a batch that takes one chain,
    for LSTM (sequences and states), both GRU forms, SimpleRNN and a reversed (Bidirectional) walk."""
    rng = np.random.default_rng(41)
    T, Fdim, U, n = 5, 12, 32, 300
    mk = lambda g, nb=None: (rng.normal(size=(Fdim, g * U)).astype(np.float32) * 0.4, rng.normal(size=(U, g * U)).astype(np.float32) * 0.3,
                             rng.normal(size=(nb or g) * U).astype(np.float32) * 0.1)
    b = mw.ModelBuilder("m")
    i = b.input([T, Fdim])
    outs, shapes = [], []
    seq, hs, cs = mw.lstm(b, i, "lstm", *mk(4), return_sequences=True, return_state=True)
    outs += [seq, hs, cs]; shapes += [[T, U], [U], [U]]
    outs.append(mw.gru(b, i, "gru_after", *mk(3, 6), reset_after=True)); shapes.append([U])
    outs.append(mw.gru(b, i, "gru_before", *mk(3), reset_after=False, return_sequences=True)); shapes.append([T, U])
    outs.append(mw.bidirectional(b, i, "bi", "SimpleRNN", mk(1), mk(1), "concat", return_sequences=True)); shapes.append([T, 2 * U])
    text = model_text(b.to_json(outs, shapes))
    xs = [[rng.normal(size=(T, Fdim)).astype(np.float32)] for _ in range(n)]
    m = fdeep_b200.read_model_from_string(text, verify=False, tensor_cores=tensor_cores)
    many = m.predict_multi(xs)              # two chains
    few = m.predict_multi(xs[:100]) + m.predict_multi(xs[100:200]) + m.predict_multi(xs[200:])   # one chain each
    want = oracle_outputs(text, xs[:6] + xs[-6:])
    for s_ in range(n):
        for o_ in range(len(shapes)):
            assert np.array_equal(many[s_][o_], few[s_][o_]), f"sample {s_} output {o_}: the batch it was computed in shows"
    for k, s_ in enumerate(list(range(6)) + list(range(n - 6, n))):
        for o_ in range(len(shapes)):
            assert_close(many[s_][o_], want[k][o_], f"two chains sample {s_} output {o_}")


def test_lstm_step_in_one_launch_matches_two_launches(built_library):
    """LSTM whose cell runs in the recurrent product's epilogue (recurrent_ops.hpp:164-181 in one launch per time step)
    against the same model loaded with the cell as a launch of its own: bit for bit, and both against the oracle."""
    rng = np.random.default_rng(21)
    # (timesteps, features, units, samples): one column tile whose second half lies beyond N (16 units), ragged last
    # column tile (48, 80), several row tiles with a partial last one, a contraction of several accumulator groups (256)
    for case, (T, Fdim, U, n) in enumerate(((5, 8, 16, 3), (6, 12, 48, 37), (4, 20, 80, 130), (3, 32, 256, 300), (9, 16, 128, 64))):
        W = rng.normal(size=(Fdim, 4 * U)).astype(np.float32) * 0.4
        Uw = rng.normal(size=(U, 4 * U)).astype(np.float32) * (1.5 / np.sqrt(U))
        bias = None if case == 1 else rng.normal(size=4 * U).astype(np.float32) * 0.1
        for seq, state in ((True, True), (False, False)):
            b = mw.ModelBuilder("m")
            i = b.input([T, Fdim])
            refs = mw.lstm(b, i, "l", W, Uw, bias, return_sequences=seq, return_state=state)
            refs = list(refs) if state else [refs]
            shapes = [[T, U] if seq else [U]] + ([[U], [U]] if state else [])
            text = model_text(b.to_json(refs, shapes))
            xs = [[rng.normal(size=(T, Fdim)).astype(np.float32)] for _ in range(n)]
            fused = fdeep_b200.read_model_from_string(text, verify=False, fused_cells=True).predict_multi(xs)
            apart = fdeep_b200.read_model_from_string(text, verify=False).predict_multi(xs)
            want = oracle_outputs(text, xs[:8])
            for s in range(n):
                for o in range(len(shapes)):
                    assert np.array_equal(fused[s][o], apart[s][o]), f"case {case} seq={seq} sample {s} output {o}: the two forms differ"
                    if s < 8:
                        assert_close(fused[s][o], want[s][o], f"lstm case {case} seq={seq} sample {s} output {o}")


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_bidirectional_and_stacked_cells(built_library, tensor_cores):
    from test_oracle import bidirectional_models, stacked_rnn_model
    for T, Fdim, U in ((7, 5, 8), (16, 32, 64)):
        js, x, wants = bidirectional_models(T, Fdim, U)
        rng = np.random.default_rng(T)
        xs = [[x]] + [[rng.normal(size=x.shape).astype(np.float32)] for _ in range(6)]
        m, got = check_against_oracle(js, xs, tensor_cores, f"bidirectional T{T} F{Fdim} U{U}")
        for g, w in zip(got[0], wants):
            assert_close(g, w.astype(np.float32), "bidirectional vs torch")
        for rs in (True, False):
            js, x, wants = stacked_rnn_model(T, Fdim, U, return_sequences=rs)
            xs = [[x]] + [[rng.normal(size=x.shape).astype(np.float32)] for _ in range(6)]
            check_against_oracle(js, xs, tensor_cores, f"stacked cells T{T} F{Fdim} U{U} seq={rs}")
    # the other wrapped classes, both GRU bias layouts
    rng = np.random.default_rng(3)
    T, Fdim, U = 9, 6, 12
    b = mw.ModelBuilder("m")
    i = b.input([T, Fdim])
    outs, shapes = [], []
    for k, (cls, g, nb) in enumerate((("GRU", 3, 6), ("GRU", 3, 3), ("SimpleRNN", 1, 1))):
        mk = lambda: (rng.normal(size=(Fdim, g * U)).astype(np.float32) * 0.4, rng.normal(size=(U, g * U)).astype(np.float32) * 0.4,
                      rng.normal(size=nb * U).astype(np.float32) * 0.1)
        outs.append(mw.bidirectional(b, i, f"bi{k}", cls, mk(), mk(), "sum" if k else "concat", return_sequences=True, reset_after=nb == 6))
        shapes.append([T, U if k else 2 * U])
    xs = [[rng.normal(size=(T, Fdim)).astype(np.float32)] for _ in range(5)]
    check_against_oracle(b.to_json(outs, shapes), xs, tensor_cores, "bidirectional GRU / SimpleRNN")


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_attention_variants_and_prelu(built_library, tensor_cores):
    from test_oracle import attention_zoo, gqa_model, prelu_model
    rng = np.random.default_rng(8)
    for dims in ((5, 7, 6, 4), (33, 70, 48, 20)):
        js, xs, wants = attention_zoo(*dims)
        samples = [xs] + [[rng.normal(size=a.shape).astype(np.float32) for a in xs] for _ in range(4)]
        m, got = check_against_oracle(js, samples, tensor_cores, f"attention zoo {dims}")
        for g, w in zip(got[0], wants):
            assert_close(g, w.astype(np.float32), "attention vs numpy")
    for kw in (dict(), dict(use_bias=False, use_gate=True, Hkv=1), dict(Tq=9, Tk=40, dim=64, Hq=8, Hkv=2, hd=16, out_dim=64, use_gate=True)):
        js, xs, want = gqa_model(**kw)
        samples = [xs] + [[rng.normal(size=a.shape).astype(np.float32) for a in xs] for _ in range(4)]
        m, got = check_against_oracle(js, samples, tensor_cores, f"gqa {kw}")
        assert_close(got[0][0], want.astype(np.float32), "gqa vs numpy")
    js, xs, wants = prelu_model()
    samples = [xs] + [[rng.normal(size=a.shape).astype(np.float32) for a in xs] for _ in range(4)]
    m, got = check_against_oracle(js, samples, tensor_cores, "prelu", rel=1e-6)
    for g, w in zip(got[0], wants):
        assert_close(g, w, "prelu vs numpy", rel=1e-6)


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_einsum_dense(built_library, tensor_cores):
    from test_oracle import EINSUM_CASES, einsum_model
    rng = np.random.default_rng(12)
    cases = list(EINSUM_CASES) + [("abc,cde->abde", (40, 64), (64, 8, 16), "de", "relu"), ("abcd,cde->abe", (40, 8, 16), (8, 16, 64), "e", None)]
    for case in cases:
        js, x, want = einsum_model(case)
        samples = [[x]] + [[rng.normal(size=x.shape).astype(np.float32)] for _ in range(4)]
        m, got = check_against_oracle(js, samples, tensor_cores, f"einsum {case[0]} bias {case[3]}")
        assert_close(got[0][0], want.astype(np.float32), "einsum vs numpy")


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_conv3d(built_library, tensor_cores):
    from test_oracle import CONV3D_CASES, conv3d_model
    rng = np.random.default_rng(14)
    cases = list(CONV3D_CASES) + [((8, 12, 12, 16), (3, 3, 3), 32, 1, "same", 1, False), ((4, 6, 6, 16), (2, 2, 2), 16, 2, "valid", 1, True)]
    for case in cases:
        js, x, want = conv3d_model(case)
        samples = [[x]] + [[rng.normal(size=x.shape).astype(np.float32)] for _ in range(3)]
        m, got = check_against_oracle(js, samples, tensor_cores, f"conv3d {case}")
        assert_close(got[0][0], want.astype(np.float32), "conv3d vs torch")
    # a batch that spans many tiles, and results that do not depend on the batch (sample 0 alone against sample 0 of 37)
    js, x, want = conv3d_model(((6, 18, 22, 8), (3, 3, 3), 16, (1, 2, 1), "same", 1, False))
    samples = [[x]] + [[rng.normal(size=x.shape).astype(np.float32)] for _ in range(36)]
    m, got = check_against_oracle(js, samples[:5], tensor_cores, "conv3d batch")
    many = m.predict_multi(samples)
    assert np.array_equal(many[0][0], got[0][0])
    assert_close(many[0][0], want.astype(np.float32), "conv3d batch vs torch")


def test_byte_inputs_are_scaled_on_the_device(built_library):
    """fdk_model_predict_multi_u8: bytes scaled into [low, high] on the GPU give bit for bit what the float entry
    point gives on the same values converted on the host (byte * ((high - low) / 255) + low in float), for one
    contiguous batch, for separately allocated samples (gathered through the staging buffer) and for two inputs."""
    rng = np.random.default_rng(21)
    js = mw.build_small_cnn()
    m = fdeep_b200.read_model_from_string(model_text(js))
    for low, high in ((0.0, 1.0), (-1.0, 1.0), (-123.68, 131.32)):
        img = rng.integers(0, 256, size=(37, 32, 32, 3), dtype=np.uint8)
        scale = np.float32((np.float32(high) - np.float32(low)) / np.float32(255.0))
        as_float = img.astype(np.float32) * scale + np.float32(low)
        want = m.predict_batch([as_float])[0]
        got = m.predict_batch([img], bytes_range=(low, high))[0]
        assert np.array_equal(got, want)
        separate = [[np.array(img[i])] for i in (5, 3, 30, 11)]
        got2 = m.predict_multi(separate, bytes_range=(low, high))
        for k, i in enumerate((5, 3, 30, 11)):
            assert np.array_equal(got2[k][0], want[i])
    from oracle import OracleModel
    o = OracleModel(json_text=model_text(js))
    img = rng.integers(0, 256, size=(3, 32, 32, 3), dtype=np.uint8)
    got = m.predict_batch([img], bytes_range=(0.0, 1.0))[0]
    for i in range(3):
        assert_close(got[i], o.predict([img[i].astype(np.float32) * np.float32(1.0 / 255.0)])[0], "bytes vs oracle")
    # a large block goes through in chunks: the byte staging offsets must follow
    js = mw.build_small_cnn(size=64)
    m = fdeep_b200.read_model_from_string(model_text(js))
    img = rng.integers(0, 256, size=(1024, 64, 64, 3), dtype=np.uint8)
    want = m.predict_batch([img.astype(np.float32) * np.float32(1.0 / 255.0)])[0]
    got = m.predict_batch([img], bytes_range=(0.0, 1.0))[0]
    assert np.array_equal(got, want)


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_preprocessing_and_upsampling(built_library, tensor_cores):
    from test_oracle import preprocessing_model
    rng = np.random.default_rng(30)
    for dims in ((5, 6, 3), (17, 23, 8)):
        js, xs, wants = preprocessing_model(*dims)
        samples = [xs] + [[rng.normal(size=a.shape).astype(np.float32) for a in xs] for _ in range(4)]
        m, got = check_against_oracle(js, samples, tensor_cores, f"preprocessing {dims}", rel=1e-6)
        for g, w in zip(got[0], wants):
            assert_close(g, w.astype(np.float32), "vs numpy", rel=2e-5)  # float32 positions and weights against float64


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_repeat_crop_upsample3d(built_library, tensor_cores):
    """RepeatVector, CenterCrop and UpSampling3D move values without arithmetic: bit-exact against the oracle and numpy."""
    from test_oracle import repeat_crop_upsample3d_model
    rng = np.random.default_rng(31)
    for dims in ((3, 7, 9, 4), (2, 16, 21, 8)):
        js, xs, wants = repeat_crop_upsample3d_model(*dims)
        samples = [xs] + [[rng.normal(size=a.shape).astype(np.float32) for a in xs] for _ in range(5)]
        m, got = check_against_oracle(js, samples, tensor_cores, f"repeat/crop/upsample3d {dims}", rel=0.0)
        for g, w in zip(got[0], wants):
            assert np.array_equal(g, w)
    # an input smaller than the target is resized first (centercrop_layer.hpp:36-40)
    b = mw.ModelBuilder("m")
    i = b.input([4, 4, 2])
    small = b.to_json([mw.center_crop(b, i, "crop", 6, 3)], [[6, 3, 2]])
    check_against_oracle(small, [[rng.normal(size=(4, 4, 2)).astype(np.float32)] for _ in range(3)], tensor_cores, "CenterCrop of a small input", rel=2e-5)


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_time_distributed(built_library, tensor_cores):
    """TimeDistributed(Dense) and TimeDistributed(Conv2D): the wrapped layer on every slice of the first axis."""
    from test_oracle import time_distributed_model
    rng = np.random.default_rng(32)
    for dims in ((5, 6, 4, 7, 8, 3, 5), (9, 32, 16, 12, 12, 8, 16)):
        js, xs, wants = time_distributed_model(*dims)
        samples = [xs] + [[rng.normal(size=a.shape).astype(np.float32) for a in xs] for _ in range(4)]
        m, got = check_against_oracle(js, samples, tensor_cores, f"time distributed {dims}")
        for g, w in zip(got[0], wants):
            assert_close(g, w.astype(np.float32), "time distributed vs torch")



@pytest.mark.parametrize("tensor_cores", PATHS)
def test_more_layer_classes(built_library, tensor_cores):
    """Resizing (nearest, bilinear, area, cropping), CenterCrop of a small input, Dot, adaptive pooling, the Threshold /
    HardShrink / SoftShrink / SparsePlus / Squareplus classes, augmentation names that pass through, Discretization,
    IntegerLookup and CategoryEncoding: the engine against the oracle, and against numpy / torch where a formula exists."""
    from test_oracle import more_layers_model
    rng = np.random.default_rng(43)
    for dims in ((9, 7, 3), (24, 21, 8)):
        js, xs, wants = more_layers_model(*dims)
        others = []
        for _ in range(3):
            other = [rng.normal(size=a.shape).astype(np.float32) for a in xs[:3]]
            other += [rng.integers(0, 50, size=xs[3].shape).astype(np.float32), rng.uniform(0, 7.99, size=xs[4].shape).astype(np.float32),
                      rng.integers(0, 5, size=(1,)).astype(np.float32)]
            others.append(other)
        m, got = check_against_oracle(js, [xs] + others, tensor_cores, f"more layers {dims}", rel=2e-5)
        if dims == (9, 7, 3):
            for k, (g, w) in enumerate(zip(got[0], wants)):
                if w is not None:
                    np.testing.assert_allclose(g, w, rtol=2e-5, atol=2e-6, err_msg=f"output {k}")


@pytest.mark.parametrize("tensor_cores", PATHS)
def test_conv_lstm(built_library, tensor_cores):
    """ConvLSTM1D / ConvLSTM2D (strides, dilation, both paddings, sequences and states, other activations): the engine against
    the oracle on several samples, and against the float64 loop over the time steps."""
    from test_oracle import CONV_LSTM_CASES, conv_lstm_case
    rng = np.random.default_rng(47)
    for k, case in enumerate(CONV_LSTM_CASES):
        js, x, wants = conv_lstm_case(**case)
        samples = [[x]] + [[rng.normal(size=x.shape).astype(np.float32)] for _ in range(4)]
        m, got = check_against_oracle(js, samples, tensor_cores, f"conv lstm case {k}", rel=5e-5)
        for g, w in zip(got[0], wants):
            assert g.shape == w.shape
            np.testing.assert_allclose(g, w, rtol=1e-4, atol=1e-5, err_msg=f"case {k}")


def test_category_encoding_value_outside_raises(built_library):
    b = mw.ModelBuilder("m")
    i = b.input([3])
    m, _ = load(b.to_json([mw.category_encoding(b, i, "cat", 4, "count")], [[4]]), True)
    np.testing.assert_array_equal(m.predict([np.array([0.0, 3.9, 1.0], np.float32)])[0], np.array([1, 1, 0, 1], np.float32))
    with pytest.raises(fdeep_b200.FdeepError, match="num_tokens"):
        m.predict([np.array([0.0, 4.0, 1.0], np.float32)])
    m.predict([np.array([2.0, 3.0, 1.0], np.float32)])  # the context stays usable
