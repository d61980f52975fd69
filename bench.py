#!/usr/bin/env python
"""Benchmark of the predict hot path on N B200 GPUs, one process per GPU.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # CPU arm: the oracle's predict_multi on the host cores

The printed line is the ResNet-50 workload (Keras-applications topology, 224x224x3, 1000 classes, seeded He-normal
weights): one step is one pass of predict over ONE batch of 256 synthetic images (N(0,1), seeded) split in contiguous
blocks of 256 / N over the GPUs (strong scaling; the model is replicated, samples are independent, there is no
collective on the data path).  `value` is timed on the device with inputs already resident in HBM; `e2e` goes through
the host-buffer C-ABI call (pinned host memory, H2D and D2H inside the timed region).  The second half of the headline
metric, GPT-2-small-shaped greedy decode (64 sequences split over the GPUs), is measured in the same run and attached
under the key `gpt2_decode` (--no-decode leaves it out; --workload gpt2_decode prints it as the line itself).
Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "frugally-deep_b200"))

WORKLOADS = {
    "resnet50": dict(builder="build_resnet50", inputs="inputs_resnet50", shape=[224, 224, 3], batch=256, unit="images/s",
                     metric="resnet50_224_fp32_images_per_sec"),
    "mobilenetv2": dict(builder="build_mobilenetv2", inputs="inputs_mobilenetv2", shape=[224, 224, 3], batch=512, unit="images/s",
                        metric="mobilenetv2_224_fp32_images_per_sec"),
    "small_cnn": dict(builder="build_small_cnn", inputs="inputs_small_cnn", shape=[32, 32, 3], batch=1024, unit="images/s",
                      metric="small_cnn_fp32_images_per_sec"),
    "text_lstm": dict(builder="build_text_lstm", inputs="inputs_text_lstm", shape=[200], batch=4096, unit="sequences/s",
                      metric="text_lstm_fp32_sequences_per_sec"),
}


def profile_figure(file_name: str, key: str):
    """A measured figure kept in a summary under profiles/ as `key = value` (so that it is updated together with the
    capture it comes from); None when the file or the key is missing."""
    import re
    try:
        with open(os.path.join(ROOT, "profiles", file_name)) as f:
            m = re.search(r"`" + re.escape(key) + r"\s*=\s*([0-9.eE+-]+)`", f.read())
        return float(m.group(1)) if m else None
    except OSError:
        return None


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML polled from a thread every few
    milliseconds (read-only queries); nvidia-smi in a loop if the NVML binding is missing."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, uuid: str = ""):
        self.gpu = gpu_index
        self.uuid = uuid
        self.samples = []   # (sm_mhz, max_mhz, set of reasons)
        self.proc = None
        self.thread = None
        self.stop_flag = threading.Event()
        self.nvml = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            try:
                h = pynvml.nvmlDeviceGetHandleByUUID(self.uuid if self.uuid.startswith("GPU-") else "GPU-" + self.uuid)
            except Exception:
                h = pynvml.nvmlDeviceGetHandleByIndex(self.gpu)
            self.nvml = (pynvml, h)
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read_smi, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _poll_nvml(self):
        nv, h = self.nvml
        bits = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        try:
            mx = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
        except Exception:
            mx = None
        while not self.stop_flag.is_set():
            try:
                sm = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                self.samples.append((sm, mx, {n for n, b in bits.items() if mask & b}))
            except Exception:
                pass
            time.sleep(0.005)

    def _read_smi(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.proc.stdout:
            f = [x.strip() for x in line.split(",")]
            if len(f) >= 6:
                try:
                    self.samples.append((float(f[0]), float(f[1]), {n for n, v in zip(names, f[2:6]) if v.lower().startswith("active")}))
                except ValueError:
                    continue

    def stop(self):
        self.stop_flag.set()
        if self.proc is not None:
            self.proc.terminate()  # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)
        if self.nvml is None and self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no NVML binding and no nvidia-smi"], "samples": 0}
        sm = [x[0] for x in self.samples]
        mx = [x[1] for x in self.samples if x[1] is not None]
        reasons = set()
        for x in self.samples:
            reasons |= x[2]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_workload(name: str):
    from fdeep_b200 import model_writer as mw
    w = WORKLOADS[name]
    js = getattr(mw, w["builder"])()
    return w, json.dumps(js, allow_nan=False, separators=(",", ":"))


def cpu_baseline(text: str, w: dict, inputs: np.ndarray, seconds_target: float = 15.0):
    """Times the CPU oracle (a restatement of the reference's algorithm; the reference itself needs Eigen
    and FunctionalPlus, which are not available) on a bounded sample with one worker per host core."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from oracle import OracleModel
    cores = os.cpu_count() or 1
    m = OracleModel(json_text=text)
    t0 = time.perf_counter()
    m.predict([inputs[0]])
    one = time.perf_counter() - t0
    n = int(max(cores, min(len(inputs), seconds_target / max(one, 1e-6) * cores)))
    n = max(cores, (n // cores) * cores)
    n = min(n, len(inputs))
    samples = [[inputs[i]] for i in range(n)]
    t0 = time.perf_counter()
    m.predict_multi(samples, threads=cores)
    dt = time.perf_counter() - t0
    return {"value": n / dt, "unit": w["unit"], "cores": cores, "kind": "port",
            "sample": f"{n} samples of the workload through the oracle's predict_multi with {cores} worker threads, {dt:.1f} s"}


GPT2_SMALL = dict(vocab=50257, ctx=1024, dim=768, layers=12, heads=12, ffn=3072)
GPT2_REDUCED = dict(vocab=4099, ctx=256, dim=256, layers=4, heads=4, ffn=1024)
GPT2_PROMPT, GPT2_NEW = 32, 128


def gpt2_texts(cfg):
    from fdeep_b200 import model_writer as mw
    dump = lambda js: json.dumps(js, allow_nan=False, separators=(",", ":"))
    return dump(mw.build_gpt2_step(first=True, **cfg)), dump(mw.build_gpt2_step(first=False, **cfg))


def gpt2_cpu_baseline(texts, cfg, positions: int = 16):
    """The decode loop on the host cores: the oracle's predict_multi over the two incremental graphs, the caller
    carrying the growing past tensors (what a user of the reference does), one sequence per worker thread, for the
    first `positions` positions of the workload's prompts.  Later positions attend over more rows and cost a little
    more; the weight products dominate (0.12 GMAC per token)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from oracle import OracleModel
    from fdeep_b200 import model_writer as mw
    cores = os.cpu_count() or 1
    n_seq = max(1, min(64, cores))
    first, step = OracleModel(json_text=texts[0]), OracleModel(json_text=texts[1])
    prompts = mw.inputs_gpt2_prompts(n_seq, seed=1, vocab=cfg["vocab"], prompt_len=GPT2_PROMPT)
    L = cfg["layers"]
    pasts = None
    t0 = time.perf_counter()
    for pos in range(positions):
        base = [[np.array([prompts[s, pos]], np.float32), np.array([float(pos)], np.float32)] for s in range(n_seq)]
        if pos == 0:
            outs = first.predict_multi(base, threads=n_seq)
            pasts = [[outs[s][1 + l] for l in range(L)] for s in range(n_seq)]
        else:
            outs = step.predict_multi([base[s] + pasts[s] for s in range(n_seq)], threads=n_seq)
            pasts = [[np.concatenate([pasts[s][l], outs[s][1 + l]], axis=0) for l in range(L)] for s in range(n_seq)]
    dt = time.perf_counter() - t0
    return {"value": n_seq * positions / dt, "unit": "tokens/s", "cores": n_seq, "kind": "port",
            "sample": f"{n_seq} sequences x the first {positions} positions through the oracle's predict_multi "
                      f"({n_seq} worker threads, past tensors carried by the caller), {dt:.1f} s"}


def run_reference(args):
    """CPU arm: the oracle's predict_multi on all host cores, a bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w, text = build_workload(args.workload)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from oracle import OracleModel
    from fdeep_b200 import model_writer as mw
    cores = os.cpu_count() or 1
    per_step = max(cores, min(w["batch"], 2 * cores))
    x = getattr(mw, w["inputs"])(per_step)
    samples = [[x[i]] for i in range(per_step)]
    ref_exe = os.path.join(ROOT, "oracle", "_ref", "ref_driver")
    kind, what = "port", ("CPU oracle (restatement of the reference's algorithm; the reference needs Eigen 3.4.0 and "
                          "FunctionalPlus 0.2.24, which are not available here)")
    if os.path.exists(ref_exe):
        # the reference itself, built by oracle/build_ref.py: fdeep::model::predict_multi(samples, parallelly = true)
        import tempfile
        import build_ref
        kind, what = "reference", "the reference's own predict_multi (oracle/_ref, compiled from its headers)"
        with tempfile.TemporaryDirectory() as tmp:
            mp, ip, op = os.path.join(tmp, "m.json"), os.path.join(tmp, "in.bin"), os.path.join(tmp, "out.bin")
            with open(mp, "w") as f:
                f.write(text)
            build_ref.write_samples(ip, samples)
            r = subprocess.run([ref_exe, mp, ip, op, str(max(args.steps, 2))], capture_output=True, text=True, check=True)
            dt = float(r.stdout.split("seconds_per_pass")[1].split()[0]) * args.steps
    else:
        m = OracleModel(json_text=text)
        for _ in range(min(args.warmup, 1)):
            m.predict_multi(samples, threads=cores)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            m.predict_multi(samples, threads=cores)
        dt = time.perf_counter() - t0
    value = per_step * args.steps / dt
    line = {"impl": "reference", "metric": w["metric"], "value": value, "unit": w["unit"], "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
            "scaling": "strong" if args.workload == "resnet50" else "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload} predict_multi, {per_step} samples per step on the host cores (a bounded sample of the "
                                   f"{w['batch']}-sample batch)",
                       "reference": what},
            "cpu_baseline": {"value": value, "unit": w["unit"], "cores": cores, "kind": kind,
                             "sample": f"{per_step} samples per step, {args.steps} steps, {cores} worker threads"},
            "e2e": {"value": value, "unit": w["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    if args.workload == "resnet50" and not args.no_decode:
        cfg = GPT2_REDUCED if args.small else GPT2_SMALL
        dec = gpt2_cpu_baseline(gpt2_texts(cfg), cfg)
        line["gpt2_decode"] = {"metric": "gpt2_small_decode_tokens_per_sec", "value": dec["value"], "unit": "tokens/s", "impl": "reference",
                               "cpu_baseline": dec}
    print(json.dumps(line))


def measure_gpt2_decode(args, dist=None):
    """Config 5: GPT-2-small-shaped greedy decode through the device-resident session (fdk_session_*): 64 sequences
    split in contiguous blocks over the GPUs, a 32-token prompt consumed one token per call, then 128 generated
    tokens.  One bench step = one whole decode of all sequences; the metric counts every position processed (prompt
    positions included: each is one call of the incremental graph).  Returns the JSON line as a dict on rank 0."""
    import torch
    import fdeep_b200
    from fdeep_b200 import model_writer as mw
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = GPT2_REDUCED if args.small else GPT2_SMALL
    total_seq = args.decode_batch or 64
    lo, hi = fdeep_b200.shard_block(total_seq, world, rank)
    batch = max(hi - lo, 1)   # a rank without sequences still decodes one, so that every rank runs the same code
    prompt_len, new_tokens = GPT2_PROMPT, GPT2_NEW
    positions = prompt_len + new_tokens - 1
    texts = gpt2_texts(cfg)
    t0 = time.perf_counter()
    first = fdeep_b200.read_model_from_string(texts[0], verify=False, devices=[local_rank], tensor_cores=not args.no_tensor_cores,
                                              skinny_products=True)
    step = fdeep_b200.read_model_from_string(texts[1], verify=False, devices=[local_rank], tensor_cores=not args.no_tensor_cores,
                                             skinny_products=True)
    load_s = time.perf_counter() - t0
    all_prompts = mw.inputs_gpt2_prompts(total_seq, seed=1, vocab=cfg["vocab"], prompt_len=prompt_len)
    prompts = all_prompts[lo:lo + batch] if hi > lo else all_prompts[:1]
    steps = max(1, min(args.steps, args.decode_steps))
    warmup = max(1, min(args.warmup, 3))

    # one session serves every decode: reset() starts a new batch of sequences in the same device buffers, so that the
    # timed region holds the positions and no allocation (cudaMalloc / cudaFree of the 0.75 GB of cache storage took
    # between 7 and 190 ms per decode on these boxes, from one process to the next)
    sess = fdeep_b200.DecodeSession(first, step, batch=batch, max_len=positions)

    def decode():
        sess.reset()
        out = None
        for pos in range(positions):
            out, _ = sess.step(prompts[:, pos] if pos < prompt_len else None)
        return out

    for _ in range(warmup):
        decode()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    sampler = ClockSampler(local_rank, str(torch.cuda.get_device_properties(local_rank).uuid))
    if rank == 0:
        sampler.start()
    l0 = first.launch_count() + step.launch_count()
    t0 = time.perf_counter()
    for _ in range(steps):
        decode()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    launches = first.launch_count() + step.launch_count() - l0
    clocks = sampler.stop() if rank == 0 else None
    sess.close()
    if dist is not None:
        t = torch.tensor([dt], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
        dist.barrier()
    del first, step
    if rank != 0:
        return None
    value = total_seq * positions * steps / dt
    d, L, f, V = cfg["dim"], cfg["layers"], cfg["ffn"], cfg["vocab"]
    weights = L * (4 * d * d + 2 * d * f) + d * V   # matrices every position streams once for all resident sequences
    kv_avg = 2 * L * (positions / 2.0) * d * batch   # rows read back by the attention blocks, averaged over the loop
    bytes_per_pos = 4.0 * (weights + kv_avg)         # per GPU
    peaks = read_peaks()
    ach = bytes_per_pos * positions * steps / dt / 1e9
    line = {"metric": "gpt2_small_decode_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "gpt2_decode: %d sequences in all (%d on this GPU), %d prompt + %d generated tokens, one position per call "
                                   "of the incremental graph (dim %d, %d blocks, vocabulary %d), greedy, device-resident key/value rows, "
                                   "positions after the second replayed from one recorded CUDA graph, one session reset between decodes"
                                   % (total_seq, batch, prompt_len, new_tokens, d, L, V),
                       "positions_per_step": positions, "model_load_s": load_s},
            "ms_per_position": dt / steps / positions * 1e3,
            "per_gpu": value / world,
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 4 * batch * prompt_len, "d2h_bytes_per_step": 4 * batch * positions,
                    "note": "the session is the host-facing call: tokens in from host memory, chosen tokens back, every position"},
            "gpu_launches": int(launches), "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"], "traffic": None,
                         "kernel": "whole position (%d launches): every weight matrix streamed once per position, key/value rows read back"
                                   % (launches // max(1, positions * steps)),
                         "algorithmic_bytes_per_position": bytes_per_pos, "peak_source": peaks["source"] + " copy bandwidth"},
            "cpu_baseline": None}
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = gpt2_cpu_baseline(texts, cfg)
    return line


def build_cpp_dropin(out_dir: str):
    """Compiles the end-to-end benchmark program of the C++ drop-in header (tests/cpp/bench_dropin.cpp) against the
    in-tree library; returns the executable's path or None when no host compiler is at hand."""
    import shutil
    if shutil.which("g++") is None:
        return None
    exe = os.path.join(out_dir, "bench_dropin")
    src = os.path.join(ROOT, "tests", "cpp", "bench_dropin.cpp")
    lib_dir = os.path.join(ROOT, "frugally-deep_b200")
    cmd = ["g++", "-std=c++14", "-O2", "-I", os.path.join(lib_dir, "include"), src, "-o", exe, "-L", lib_dir, "-lfdeep_b200",
           "-Wl,-rpath," + lib_dir, "-pthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    return exe if r.returncode == 0 else None


def e2e_cpp_dropin(text: str, in_shape, batch: int, steps: int, device: int):
    """The same step through the C++ drop-in API as a user of the reference writes it: fdeep::load_model, one
    separately allocated (pageable) fdeep::tensor per sample, model.predict_multi.  Returns None when it cannot run."""
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        exe = build_cpp_dropin(tmp)
        if exe is None:
            return None
        path = os.path.join(tmp, "model.json")
        with open(path, "w") as f:
            f.write(text)
        env = dict(os.environ, FDEEP_B200_DEVICES=str(device))
        r = subprocess.run([exe, path, str(batch), str(steps)] + [str(d) for d in in_shape], capture_output=True, text=True, env=env, timeout=600)
        if r.returncode != 0:
            return {"error": (r.stderr or r.stdout)[-300:]}
        try:
            return json.loads(r.stdout.strip().split("\n")[-1])
        except ValueError:
            return {"error": r.stdout[-300:]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="resnet50", choices=sorted(WORKLOADS) + ["gpt2_decode"])
    ap.add_argument("--small", action="store_true", help="decode: a reduced model (quick functional run)")
    ap.add_argument("--batch", type=int, default=0, help="samples per GPU per step (default: the workload's batch split over the GPUs)")
    ap.add_argument("--decode-batch", type=int, default=0, help="decode: sequences in all (default 64)")
    ap.add_argument("--decode-steps", type=int, default=3, help="decode: at most this many whole decodes are timed")
    ap.add_argument("--no-decode", action="store_true", help="resnet50: do not attach the decode measurement")
    ap.add_argument("--no-tensor-cores", action="store_true", help="use the exact-fp32 FFMA contraction kernels")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--fused-cells", action="store_true", help="LSTM: the cell in the recurrent product's epilogue (one launch per time step)")
    ap.add_argument("--layer-table", action="store_true",
                    help="print the device time of every operation of one step (CUDA events around each launch) on stderr")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        if args.workload == "gpt2_decode":
            if int(os.environ.get("RANK", "0")) != 0:
                return
            cfg = GPT2_REDUCED if args.small else GPT2_SMALL
            dec = gpt2_cpu_baseline(gpt2_texts(cfg), cfg)
            print(json.dumps({"impl": "reference", "metric": "gpt2_small_decode_tokens_per_sec", "value": dec["value"], "unit": "tokens/s",
                              "n_gpus": args.gpus, "steps": 1, "warmup": 0, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                              "dtype": "f32", "data": "synthetic", "config": {"workload": "gpt2_decode on the host cores: " + dec["sample"]},
                              "cpu_baseline": dec, "e2e": {"value": dec["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
            return
        run_reference(args)
        return

    import torch
    import fdeep_b200
    from fdeep_b200 import model_writer as mw

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    host_group = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        # a second group on the host side: ranks that must WAIT while rank 0 measures alone do so here, on the CPU (a NCCL
        # barrier parks a spinning kernel on the waiting ranks' GPUs, which would share them with the measurement)
        host_group = dist.new_group(backend="gloo")

    if args.workload == "gpt2_decode":
        line = measure_gpt2_decode(args, dist)
        if rank == 0:
            print(json.dumps(line))
        if dist is not None:
            dist.destroy_process_group()
        return

    w, text = build_workload(args.workload)
    # One batch of the workload's size split in contiguous blocks over the GPUs (strong scaling), as predict_multi
    # shards it; --batch gives every GPU that many samples instead (weak scaling).
    strong = args.batch == 0
    total = w["batch"]
    if strong:
        lo, hi = fdeep_b200.shard_block(total, world, rank)
        batch = max(hi - lo, 1)
    else:
        batch = args.batch
        total = batch * world
    model = fdeep_b200.read_model_from_string(text, verify=False, devices=[local_rank], tensor_cores=not args.no_tensor_cores,
                                              fused_cells=args.fused_cells)
    x_all = getattr(mw, w["inputs"])(total if strong else batch, seed=1 if strong else 1 + rank)
    x_host = np.ascontiguousarray(x_all[lo:lo + batch]) if strong else x_all
    in_shape = list(x_host.shape[1:])
    out_shape = model.infer_shapes([in_shape])[0]
    info = model.plan_info([in_shape])
    stream = torch.cuda.Stream()  # explicit stream: the kernels are queued on it and the events recorded on it

    def timed_device_pass(x_np, n):
        """n samples per step, inputs resident in HBM: (ms for args.steps steps, launches, clocks)."""
        d_in = torch.from_numpy(x_np).cuda()
        d_out = torch.empty([n] + out_shape, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()

        def step():
            model.predict_batch_device([d_in.data_ptr()], [in_shape], n, [d_out.data_ptr()], stream=stream.cuda_stream)

        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        model.sync()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(local_rank, str(torch.cuda.get_device_properties(local_rank).uuid))
        if rank == 0:
            sampler.start()
        launches0 = model.launch_count()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for _ in range(args.steps):
            step()
        ev1.record(stream)
        torch.cuda.synchronize()
        t_ms = ev0.elapsed_time(ev1)
        n_launch = model.launch_count() - launches0
        clk = sampler.stop() if rank == 0 else None
        model.sync()
        if dist is not None:
            t = torch.tensor([t_ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_ms = float(t.item())
            dist.barrier()
        return t_ms, n_launch, clk, d_in

    # ---- device-resident timing (value) ----
    ms, launches, clocks, d_in = timed_device_pass(x_host, batch)
    value = total * args.steps / (ms * 1e-3)

    # ---- the same with the workload's whole batch on every GPU (weak scaling), for comparison at N > 1 ----
    weak = None
    if strong and world > 1:
        x_weak = getattr(mw, w["inputs"])(w["batch"], seed=1 + rank)
        ms_w, _, _, d_weak = timed_device_pass(x_weak, w["batch"])
        weak = {"value": world * w["batch"] * args.steps / (ms_w * 1e-3), "unit": w["unit"], "ms_per_step": ms_w / args.steps,
                "samples_per_gpu": w["batch"], "scaling": "weak"}
        del d_weak, x_weak

    # ---- end to end through the host-buffer C-ABI call (pinned host memory, H2D + D2H timed) ----
    x_pin = torch.from_numpy(x_host).pin_memory()
    x_np = x_pin.numpy()
    model.predict_batch([x_np])  # warm-up of the staging buffers
    model.predict_batch([x_np])
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        out = model.predict_batch([x_np])[0]
    e2e_s = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = total * args.steps / e2e_s
    h2d = int(x_np.nbytes)
    d2h = int(out.nbytes)

    # ---- the same call with byte images (image workloads, rank 0): what a caller of tensor_from_bytes + predict_multi
    # gets when the conversion runs on the GPU (fdk_model_predict_multi_u8): a quarter of the host-to-device bytes ----
    e2e_bytes = None
    if rank == 0 and len(in_shape) == 3 and in_shape[2] in (1, 3, 4):
        u8_pin = torch.from_numpy(np.random.default_rng(1).integers(0, 256, size=[batch] + list(in_shape), dtype=np.uint8)).pin_memory()
        u8_np = u8_pin.numpy()
        model.predict_batch([u8_np], bytes_range=(0.0, 1.0))
        model.predict_batch([u8_np], bytes_range=(0.0, 1.0))
        t0 = time.perf_counter()
        for _ in range(args.steps):
            model.predict_batch([u8_np], bytes_range=(0.0, 1.0))
        e2e_bytes = {"value": batch * args.steps / (time.perf_counter() - t0), "unit": w["unit"] + " (this rank)",
                     "h2d_bytes_per_step": int(u8_np.nbytes), "d2h_bytes_per_step": d2h,
                     "entry": "fdk_model_predict_multi_u8: uint8 images scaled to [0, 1] on the GPU"}

    # ---- roofline of the dominant kernel, timed live with CUDA events (rank 0) ----
    roofline = None
    path = "tc"
    if rank == 0:
        peaks = read_peaks()
        recs = model.profile([d_in.data_ptr()], [in_shape], batch)
        recs = model.profile([d_in.data_ptr()], [in_shape], batch)  # second pass: warm
        gemms = [r for r in recs if r["kind"] == "gemm"]
        ops = [r for r in recs if r["kind"] == "op"]
        if args.layer_table:
            # one line per contraction launch (rows, columns, contraction length, algorithmic TFLOP/s, kernel) and per
            # operation (for memory-bound operations M holds the bytes read + written)
            for r in recs:
                if r["kind"] == "gemm":
                    print("gemm %-30s %8.3f ms  M=%-9d N=%-5d K=%-5d %7.1f TFLOP/s  %s" %
                          (r["layer"], r["ms"], r["M"], r["N"], r["K"], r["flops"] / r["ms"] / 1e9 if r["ms"] > 0 else 0.0, r["path"]),
                          file=sys.stderr)
                else:
                    gbs = r["M"] / (r["ms"] * 1e-3) / 1e9 if r["ms"] > 0 and r["M"] > 0 else 0.0
                    print("op   %-30s %8.3f ms  kind=%-3s %s" % (r["layer"], r["ms"], r["path"], ("%8.1f GB/s" % gbs) if gbs else ""),
                          file=sys.stderr)
        ops_ms = sum(r["ms"] for r in ops)
        g_ms = sum(r["ms"] for r in gemms)
        g_flops = sum(r["flops"] for r in gemms)
        path = "tc" if any(r["path"] == "tc" for r in gemms) else "ffma"
        if args.workload == "mobilenetv2":
            # Memory-bound workload: the floor is every layer output written once and read once (53.4 MB per image);
            # the depthwise launches (operation kind 2) are listed one by one against the measured copy bandwidth.
            alg_bytes = 53.4e6 * batch
            ach = alg_bytes / (ms / args.steps * 1e-3) / 1e9
            dw = [r for r in ops if r["path"] == "2"]
            dw_ms = sum(r["ms"] for r in dw)
            dw_bytes = sum(r["M"] for r in dw)
            roofline = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                        "traffic": None, "kernel": "whole step against the layer-output floor (53.4 MB per image)",
                        "algorithmic_bytes_per_step": alg_bytes, "peak_source": peaks["source"] + " copy bandwidth",
                        "depthwise": {"launches": len(dw), "ms_per_step": dw_ms, "bytes_per_step": dw_bytes,
                                      "gbs": dw_bytes / (dw_ms * 1e-3) / 1e9 if dw_ms > 0 else None,
                                      "frac": dw_bytes / (dw_ms * 1e-3) / 1e9 / peaks["hbm_gbs"] if dw_ms > 0 else None,
                                      "per_launch_gbs": [round(r["M"] / (r["ms"] * 1e-3) / 1e9, 1) for r in dw if r["ms"] > 0]},
                        "contraction_ms_per_step": g_ms, "all_ops_ms_per_step": ops_ms}
        else:
            if path == "tc":
                # FP32 semantics through 3xTF32: three tensor-core products per algorithmic product.  The TF32 peak is
                # taken as half of the measured dense bf16 peak (sustained figure: the kernel runs inside a long step).
                peak = peaks["bf16_tflops_sustained"] / 2.0
                peak_note = "half of the %s sustained dense bf16 cuBLAS peak (TF32-class pipe); 3xTF32 caps frac at 1/3" % peaks["source"]
            else:
                peak = 2 * 128 * 148 * 1.965e9 / 1e12  # FFMA: 128 lanes x 2 flop x 148 SMs x max clock
                peak_note = "nominal fp32 FFMA peak at the maximum SM clock (no measured figure)"
            achieved = g_flops / (g_ms * 1e-3) / 1e12 if g_ms > 0 else 0.0
            traffic = None
            if path == "tc" and args.workload == "resnet50" and batch == 256:
                # DRAM bytes per contraction launch (read + written, average over the step's launches) from a one-pass ncu
                # capture of this very workload, kept with its command under profiles/
                traffic = profile_figure("gemm_tc_kernel_resnet50_b256_dram.md", "dram_bytes_per_launch")
            roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak if peak else None,
                        "frac_issued": (3.0 if path == "tc" else 1.0) * achieved / peak if peak else None,
                        "traffic": traffic, "traffic_unit": "bytes per launch",
                        "kernel": "gemm_tc_kernel (tcgen05 3xTF32)" if path == "tc" else "gemm_ffma_kernel",
                        "launches_per_step": len(gemms), "kernel_ms_per_step": g_ms, "all_ops_ms_per_step": ops_ms,
                        "peak_source": peak_note, "hbm_gbs_peak": peaks["hbm_gbs"],
                        # tcgen05.mma.kind::tf32 issued back to back on all SMs with zero operands: the pipe's ceiling, for
                        # context beside `peak` (microbench/tf32_mma_peak.cu; figure kept under profiles/)
                        "tf32_pipe_tflops_measured_burst": profile_figure("microbench_tf32_mma_peak_and_design_probes.md", "tf32_pipe_tflops_burst")
                        if path == "tc" else None}
            # the slowest layers of this step, for the record (name, ms, TFLOP/s)
            slow = sorted(gemms, key=lambda r: -r["ms"])[:5]
            roofline["slowest_launches"] = [{"layer": r["layer"], "ms": round(r["ms"], 4), "M": r["M"], "N": r["N"], "K": r["K"],
                                             "tflops": round(r["flops"] / (r["ms"] * 1e-3) / 1e12, 1) if r["ms"] > 0 else None} for r in slow]

    cpu = None
    if rank == 0 and not args.no_cpu_baseline and world == 1:
        cpu = cpu_baseline(text, w, x_all)

    # ---- the drop-in C++ API end to end (rank 0, one GPU): pageable fdeep::tensor per sample, model.predict_multi ----
    e2e_cpp = None
    if rank == 0 and world == 1 and args.workload in ("resnet50", "mobilenetv2", "small_cnn"):
        e2e_cpp = e2e_cpp_dropin(text, in_shape, total, max(2, min(args.steps, 5)), local_rank)

    del d_in
    # ---- one process, all N devices, through fdk_model_predict_multi (the library's own sharding): rank 0 while the
    # other ranks wait at the barrier with their GPUs idle ----
    e2e_inprocess = None
    if dist is not None:
        torch.cuda.synchronize()
        dist.barrier(group=host_group)
    if rank == 0 and world > 1 and torch.cuda.device_count() >= world:
        try:
            multi = fdeep_b200.read_model_from_string(text, verify=False, devices=list(range(world)), tensor_cores=not args.no_tensor_cores)
            x_full = torch.from_numpy(np.ascontiguousarray(x_all[:total])).pin_memory().numpy()
            multi.predict_batch([x_full])
            multi.predict_batch([x_full])
            t0 = time.perf_counter()
            for _ in range(args.steps):
                multi.predict_batch([x_full])
            e2e_inprocess = {"value": total * args.steps / (time.perf_counter() - t0), "unit": w["unit"], "devices": world,
                             "entry": "fdk_model_predict_multi on one model loaded on all devices (one host thread, stream and weight replica per device)"}
            del multi
        except Exception as e:  # reported, not fatal: the per-process numbers stand
            e2e_inprocess = {"error": str(e)[:200]}
    if dist is not None:
        dist.barrier(group=host_group)

    decode = None
    if args.workload == "resnet50" and not args.no_decode:
        del model
        decode = measure_gpt2_decode(args, dist)

    if rank == 0:
        line = {"metric": w["metric"], "value": value, "unit": w["unit"], "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic",
                "config": {"workload": f"{args.workload}: one batch of {total} samples per step split over {world} GPU(s) "
                                       f"({batch} on this one), input {in_shape}, seeded random weights",
                           "contraction": "tcgen05 3xTF32" if path == "tc" else "FFMA fp32",
                           "l2": "inputs (%.0f MB) + intermediates (%.0f MB) per GPU and step against the 126 MB L2" %
                                 (x_host.nbytes / 1e6, info["arena_bytes_per_sample"] * batch / 1e6),
                           "flops_per_sample": info["flops_per_sample"], "arena_bytes_per_sample": info["arena_bytes_per_sample"]},
                "per_gpu": value / world, "per_gpu_weak": weak,
                "e2e": {"value": e2e_value, "unit": w["unit"], "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
                "e2e_byte_images": e2e_bytes, "e2e_cpp_dropin": e2e_cpp, "e2e_inprocess": e2e_inprocess,
                "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu}
        if decode is not None:
            line["gpt2_decode"] = decode
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
