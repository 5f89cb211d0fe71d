#!/usr/bin/env python3
"""Benchmark of the llmcp Q8_0 hot path on B200.

Workload (the whole-model configuration of the benchmark list, batch 1): a random-init
Qwen3.5-4B-architecture model packed with --quant q8_0 (seeded synthetic weights with the real
shapes and dtypes; the real checkpoint is not available offline), 1024 x token 9419 prefill, then
greedy decode.  One "step" is one decode step of the whole model: every weight byte of the arena
streams from HBM once (4.47 GB, far more than the 126 MB L2, so no cache flush is needed
between steps).

  value  decode tokens/s with token, state and logits resident in HBM (engine interface),
         timed with CUDA events on the launching stream, max over ranks.  It is measured in
         the fast arithmetic mode (config.mode); the exact mode, whose every f32 result is
         bit-identical to the reference's order of operations, is timed beside it (exact_mode);
  e2e    the same steps through the reference-facing AOT ABI entry point with host buffers:
         token, cos and sin rows go host -> device, the 248320-float logits row comes back
         and the argmax is taken on the host, as tools/llmcp-benchmark does;
  roofline  the decode GEMV (N=9216, K=2560, the gate_proj/up_proj shape) timed alone with
         CUDA events over a ring of 12 weight copies (301 MB);
  roofline_gemm  the prefill GEMM (1024 x 9216 x 2560) on the tcgen05 tensor cores, alone;
  cpu_baseline  the CPU oracle (a restatement of the reference's arithmetic; the reference's
         own AOT build needs an MLIR toolchain that is not installed) on all host cores, on
         the same 1024-token context; its greedy tokens and logits are also what the GPU arm's
         are compared with (tokens_match_oracle, max_abs_logit_diff, min_top2_margin).

N > 1 (torchrun): one sequence decoded by all N GPUs, tensor parallel inside the engine (every
projection split by output rows, heads and state by head, the vocabulary projection by rows;
exchanges are the library's own peer-store all-gather kernels, four per layer): scaling is
"strong" and value is that one sequence's tokens/s.  The replica figure (a full engine and a
sequence per GPU, no exchange on the data path, sum over ranks) is reported beside it under
"replicas"; `--parallelism replicas` makes it the headline instead.

`--impl reference` times the CPU oracle alone on the same workload and prints the same line; that
arm loads no CUDA library.

Other keys: `batch` (64 sequences decoded together, two prompt sets; `--batch 0` skips it),
`prefill_tokens_per_second`, `parity`, `whole_step_roofline`.  `--only gemv|gemm|attn` run one kernel on
a small case (what a profiler captures); `--only timeline` and `--only prefill-timeline` print the
device timeline of a decode step and the time per kernel family of a 1024-token prefill.
"""
import argparse
import ctypes as C
import json
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SEED = 20261125
TOKEN = 9419
PREFILL = 1024
M2_DECODE_TOK_S = 11.39  # published Q8_0 decode tok/s on Apple M2, 4 threads (reference README.md:140)
GEMV_N, GEMV_K, GEMV_RING = 9216, 2560, 12
GEMV_BYTES = GEMV_N * (GEMV_K // 32) * 34 + GEMV_K * 4 + GEMV_N * 4  # weights + f32 x + f32 y = 25,114,624
# dram__bytes_read.sum + dram__bytes_write.sum of one gemv_q8_cols80_kernel launch of this shape, from an ncu
# capture of `bench.py --only gemv` (not measured in this run; the 36,864-byte result stays in L2).
GEMV_DRAM_TRAFFIC = 25_097_216
GEMM_M, GEMM_N, GEMM_K = 1024, 9216, 2560  # the gate_proj/up_proj prefill GEMM
GEMM_FORM = 1  # the engine's default form of the TMA-fed tensor-core GEMM (int8 planes, packed f32x2 arithmetic)


def measured_peaks():
    """(HBM GB/s, dense bf16 TFLOP/s burst, "measured" | "fallback")."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["hbm_gbs"]), float(data["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed regions run.

    NVML is read directly (queries only) every millisecond from a thread, so that a timed region
    of a few tens of milliseconds still holds tens of samples; if the NVML binding is missing,
    `nvidia-smi -lms 20` is read instead.
    """

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device = device
        self.samples = []  # (host time, sm MHz, reasons bitmask or None, nvidia-smi text or None)
        self.windows = []  # [begin, end] host times of the timed regions
        self.proc = None
        self.nvml = None
        self.max_clock = None
        self.running = False
        self.how = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            index = self.device
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            if visible and all(v.strip().isdigit() for v in visible.split(",")):
                index = int(visible.split(",")[self.device])
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_clock = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.running = True
            self.how = "NVML queries every ms from a thread"
            threading.Thread(target=self._poll, daemon=True).start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.how = "nvidia-smi every 20 ms"
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _poll(self):
        n = self.nvml
        while self.running:
            try:
                clock = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                reasons = int(n.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                self.samples.append((time.perf_counter(), clock, reasons, None))
            except Exception:
                pass
            time.sleep(0.001)

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), None, None, line.strip()))

    def wait_first_sample(self, seconds=5.0):
        deadline = time.perf_counter() + seconds
        while (self.proc or self.running) and not self.samples and time.perf_counter() < deadline:
            time.sleep(0.01)

    def open_window(self):
        self.windows.append([time.perf_counter(), None])

    def close_window(self):
        self.windows[-1][1] = time.perf_counter()

    def stop(self):
        self.running = False
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        clocks, max_clock, reasons = [], self.max_clock, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = lambda t: any(b <= t <= (e if e is not None else t) for b, e in self.windows)
        for stamp, clock, mask, text in list(self.samples):
            if self.windows and not inside(stamp):
                continue
            if text is None:
                clocks.append(clock)
                n = self.nvml
                for name, bit in (("hw_slowdown", n.nvmlClocksEventReasonHwSlowdown),
                                  ("hw_thermal_slowdown", n.nvmlClocksEventReasonHwThermalSlowdown),
                                  ("sw_thermal_slowdown", n.nvmlClocksEventReasonSwThermalSlowdown),
                                  ("sw_power_cap", n.nvmlClocksEventReasonSwPowerCap)):
                    if mask & int(bit):
                        reasons.add(name)
                continue
            parts = [p.strip() for p in text.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                max_clock = float(parts[2])
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks),
                "sampled": f"{self.how}; samples inside the timed loops (device arm, both modes, and ABI arm)"}


CONTAINER = pathlib.Path("/dev/shm") / f"llmcp_b200_synth_{SEED}.bin"


def ensure_container(local_rank):
    """One synthetic container per node in /dev/shm, written by local rank 0 with the host-only
    packer binary (no CUDA library is involved)."""
    if local_rank == 0 and not CONTAINER.exists():
        tool = ROOT / "llmcp_b200" / "bin" / "llmcp-pack"
        if not tool.exists():
            raise SystemExit(f"{tool} is missing: run `python -m llmcp_b200.build`")
        tmp = CONTAINER.with_suffix(f".{os.getpid()}.part")
        subprocess.run([str(tool), "--synthetic", str(SEED), "--out", str(tmp)], check=True, stdout=subprocess.DEVNULL)
        os.replace(tmp, CONTAINER)
    while not CONTAINER.exists():
        time.sleep(0.2)
    return CONTAINER


def read_container(path):
    """(bytes as a numpy array over a read-only map, manifest dict) without the CUDA library:
    the header holds the arena length at byte 16, the JSON manifest follows the arena."""
    import mmap
    with open(path, "rb") as f:
        mapped = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    data = np.frombuffer(mapped, dtype=np.uint8)
    arena_bytes = int.from_bytes(data[16:24].tobytes(), "little")
    manifest = json.loads(data[arena_bytes:].tobytes().decode().rstrip("\0"))
    return data, manifest


ORACLE_DIMS = dict(full_interval=4, heads=16, kv_heads=4, head_dim=256, rotary=64, lin_k_heads=16, lin_v_heads=32,
                   lin_k_dim=128, lin_v_dim=128, conv_kernel=4)  # Qwen3.5-4B text (lib/Runtime/AotRuntime.cpp:41-43)


class OracleRun:
    """The CPU oracle on the benchmark's context: 1024 x token 9419, then greedy steps."""

    def __init__(self, data, manifest, steps, mode="fma"):
        import oracle
        self.oracle = oracle
        self.threads = oracle.set_num_threads()  # every host core, whatever OMP_NUM_THREADS was inherited
        self.model = oracle.Model(data, manifest, ORACLE_DIMS, mode=mode)
        self.state = self.model.new_state(PREFILL + steps + 2)
        begin = time.perf_counter()
        self.logits = [self.model.forward(self.state, [TOKEN] * PREFILL, 0)]
        self.prefill_s = time.perf_counter() - begin
        self.tokens = [oracle.argmax(self.logits[0])]
        self.position = PREFILL

    def decode(self, steps, keep_logits=True):
        """`steps` greedy steps; returns tokens/s of the loop (forward + host argmax, as
        tools/llmcp-benchmark times it)."""
        begin = time.perf_counter()
        for _ in range(steps):
            logits = self.model.forward(self.state, [self.tokens[-1]], self.position)
            self.position += 1
            self.tokens.append(self.oracle.argmax(logits))
            if keep_logits:
                self.logits.append(logits)
        return steps / (time.perf_counter() - begin)

    def forced(self, tokens):
        """Logits of every position when fed `tokens` (another run's greedy chain) after the prompt."""
        rows = [self.logits[0]]
        for token in tokens:
            rows.append(self.model.forward(self.state, [token], self.position))
            self.position += 1
        return rows

    def close(self):
        self.model.close()


def gemv_roofline(L, torch, device, ring=GEMV_RING, sweeps=20, flags=3):
    """Decode GEMV alone: CUDA events on the launching stream over a ring of weight copies.
    flags: 1 dependent launch, 2 L2 prefetch of later sets, 16 tree-reduced row sums (fast mode)."""
    lib = L.lib()
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device="cuda").manual_seed(SEED)
    wq = torch.randint(-127, 128, (ring, GEMV_N, GEMV_K), dtype=torch.int8, device="cuda", generator=gen)
    wd = (torch.rand((ring, GEMV_N, GEMV_K // 32), device="cuda", generator=gen) * 1e-3).to(torch.float16)
    x = torch.randn((1, GEMV_K), device="cuda", generator=gen)
    aq = torch.empty(GEMV_K, dtype=torch.int8, device="cuda")
    scales = torch.empty(GEMV_K // 32, dtype=torch.float32, device="cuda")
    y = torch.empty(GEMV_N, dtype=torch.float32, device="cuda")
    ptr = lambda t: C.c_void_p(t.data_ptr())
    assert lib.llmcp_dev_act_quant(ptr(x), 0, C.c_int64(1), C.c_int64(GEMV_K), ptr(aq), ptr(scales), C.c_void_p(stream)) == 0

    def sweep(times, stream):
        for _ in range(times):
            for r in range(ring):
                rc = lib.llmcp_dev_gemv_q8(ptr(aq), ptr(scales), C.c_int64(GEMV_K), ptr(wq[r]), ptr(wd[r]),
                                           C.c_int64(GEMV_N), ptr(y), 0, 0, 0, flags, C.c_void_p(stream))
                assert rc == 0, L.last_error()

    sweep(3, stream)
    torch.cuda.synchronize()
    # One pass over the ring is captured as a CUDA graph (as the decode step itself is), so the
    # events time the kernels and not the Python call overhead between launches.
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        sweep(1, torch.cuda.current_stream().cuda_stream)
    graph.replay()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    begin.record()
    for _ in range(sweeps):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    us = begin.elapsed_time(end) * 1e3 / (sweeps * ring)
    return GEMV_BYTES / us / 1e3, us, sweeps * ring  # GB/s, us per launch, launches


def gemm_alone(L, torch, repeats=5, form=GEMM_FORM):
    """Prefill GEMM alone (tcgen05 kernel, f16-valued operand planes) on device buffers: returns
    (us per launch, int8 TOP/s).  The planes are made once, as the engine makes the weight planes
    at load; the timed launches are the GEMM only."""
    lib = L.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    gen = torch.Generator(device="cuda").manual_seed(SEED)
    nb = GEMM_K // 32
    wq = torch.randint(-127, 128, (GEMM_N, GEMM_K), dtype=torch.int8, device="cuda", generator=gen)
    wd = (torch.rand((GEMM_N, nb), device="cuda", generator=gen) * 1e-3).to(torch.float16)
    x = torch.randn((GEMM_M, GEMM_K), device="cuda", generator=gen)
    aq = torch.empty((GEMM_M, GEMM_K), dtype=torch.int8, device="cuda")
    scales = torch.empty((GEMM_M, nb), dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = torch.empty((GEMM_M, GEMM_N), dtype=torch.float32, device="cuda")
    ptr = lambda t: C.c_void_p(t.data_ptr())
    assert lib.llmcp_dev_act_quant(ptr(x), 0, C.c_int64(GEMM_M), C.c_int64(GEMM_K), ptr(aq), ptr(scales), stream) == 0
    lib.llmcp_dev_gemm_q8_tma_scale_pitch.restype = C.c_int64
    pitch = int(lib.llmcp_dev_gemm_q8_tma_scale_pitch(C.c_int64(GEMM_M)))
    ah = torch.empty((GEMM_M, GEMM_K), dtype=torch.float16, device="cuda")
    ast = torch.zeros((nb, pitch), dtype=torch.float32, device="cuda")
    wh = torch.empty((GEMM_N, GEMM_K), dtype=torch.float16, device="cuda")
    wst = torch.empty((nb, GEMM_N), dtype=torch.float32, device="cuda")
    assert lib.llmcp_dev_q8_gemm_planes(ptr(aq), ptr(scales), 0, C.c_int64(GEMM_M), C.c_int64(GEMM_K), ptr(ah), ptr(ast), stream) == 0
    assert lib.llmcp_dev_q8_gemm_planes(ptr(wq), ptr(wd), 1, C.c_int64(GEMM_N), C.c_int64(GEMM_K), ptr(wh), ptr(wst), stream) == 0

    def launch():
        a, w = (ah, wh) if form >= 2 else (aq, wq)
        rc = lib.llmcp_dev_gemm_q8_tma(form, ptr(a), ptr(ast), C.c_int64(GEMM_M), C.c_int64(GEMM_K), ptr(w), ptr(wst),
                                       C.c_int64(GEMM_N), ptr(y), 0, 0, ptr(status), C.c_uint32(0), 0, stream)
        assert rc == 0, L.last_error()

    for _ in range(3):
        launch()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    begin.record()
    for _ in range(repeats):
        launch()
    end.record()
    torch.cuda.synchronize()
    us = begin.elapsed_time(end) * 1e3 / repeats
    assert int(status.item()) == 0, "a bounded wait inside the GEMM ran out"
    return us, 2.0 * GEMM_M * GEMM_N * GEMM_K / us / 1e6


def attention_alone(L, repeats=4, position=1030):
    """One-token attention of a full-attention layer (16 query heads, 4 KV heads, head_dim 256)
    against `position` cached keys, through the operator entry point with host buffers: the small
    case the profiler captures for the decode attention kernels.  Returns the last output row."""
    rng = np.random.default_rng(SEED)
    nh, nkv, hd, rot, cap = 16, 4, 256, 64, position + 70

    def bf16(a):
        bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
        return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)

    qg = bf16(rng.standard_normal((1, nh * 2 * hd)))
    k = bf16(rng.standard_normal((1, nkv * hd)))
    v = bf16(rng.standard_normal((1, nkv * hd)))
    norm = np.zeros(hd, dtype=np.uint16)
    cos, sin = L.make_cos_sin(position, rot, 1e7)
    cache = bf16(rng.standard_normal((2, nkv, cap, hd)))
    out = None
    for _ in range(repeats):
        out, _ = L.ops.attention(qg, k, v, norm, norm, cos[None], sin[None], cache, position, nh, nkv, hd, rot)
    return out[0]


def decode_timeline(L, torch, mode):
    """Prints the device timeline of one decode step at 1032 cached positions: per kernel family its
    launches, summed duration and the summed distance from the previous kernel's end to its own start
    (negative = it started while the previous one ran), then start -> end of every kernel of the first
    four layers and of the step's tail.  Stamps come from the PyTorch profiler (CUPTI activity
    records of a plain CUDA-graph replay: kernels overlap as they do in the bench)."""
    import collections
    import tempfile
    from torch.profiler import ProfilerActivity, profile

    torch.zeros(1, device="cuda")
    arena = L.Arena().load(ensure_container(0))
    engine = L.Engine(arena.data, L.default_dims(), capacity=PREFILL + 136, mode=mode)
    _, token = engine.forward([TOKEN] * PREFILL, 0)
    out, _ = engine.generate(token, PREFILL, 8)
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        out, ms = engine.generate(int(out[-1]), PREFILL + 8, 4)
        torch.cuda.synchronize()
    with tempfile.TemporaryDirectory() as folder:
        trace = os.path.join(folder, "trace.json")
        prof.export_chrome_trace(trace)
        events = [e for e in json.load(open(trace))["traceEvents"] if e.get("cat") == "kernel"]
    events.sort(key=lambda e: e["ts"])
    starts = [i for i, e in enumerate(events) if "embedding" in e["name"]]
    step = events[starts[1]:starts[2]]
    t0 = step[0]["ts"]

    def short(name):
        name = name.replace("(anonymous namespace)::", "").replace("<unnamed>::", "")
        return name.split("(")[0].replace("llmcp_b200::", "").replace("void ", "")

    families = collections.defaultdict(lambda: [0, 0.0, 0.0])
    previous_end = None
    for e in step:
        entry = families[short(e["name"])]
        entry[0] += 1
        entry[1] += e["dur"]
        entry[2] += 0.0 if previous_end is None else e["ts"] - previous_end
        previous_end = e["ts"] + e["dur"]
    span = step[-1]["ts"] + step[-1]["dur"] - t0
    print(f"mode {mode}: {ms / 4 * 1e3:.1f} us per token over 4 steps; this step spans {span:.1f} us in {len(step)} kernels")
    for name, (n, dur, gap) in sorted(families.items(), key=lambda kv: -kv[1][1]):
        print(f"{name[:56]:56s} n={n:4d} dur={dur:8.1f} us  start-after-previous-end={gap:8.1f} us  avg={dur / n:6.2f}")
    for e in step[:42] + step[-6:]:
        print(f"{e['ts'] - t0:8.2f} -> {e['ts'] - t0 + e['dur']:8.2f} (+{e['dur']:6.2f})  {short(e['name'])[:64]}")


def prefill_timeline(L, torch, mode):
    """Per kernel family of one 1024-token prefill: launches and summed device time (PyTorch
    profiler, CUPTI activity records of a plain run; kernels of a prefill run back to back)."""
    import collections
    import tempfile
    from torch.profiler import ProfilerActivity, profile

    torch.zeros(1, device="cuda")
    arena = L.Arena().load(ensure_container(0))
    engine = L.Engine(arena.data, L.default_dims(), capacity=PREFILL + 16, mode=mode)
    for _ in range(2):
        engine.reset()
        engine.forward([TOKEN] * PREFILL, 0, want_logits=False)
    engine.reset()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        engine.forward([TOKEN] * PREFILL, 0, want_logits=False)
        torch.cuda.synchronize()
    with tempfile.TemporaryDirectory() as folder:
        trace = os.path.join(folder, "trace.json")
        prof.export_chrome_trace(trace)
        events = [e for e in json.load(open(trace))["traceEvents"] if e.get("cat") == "kernel"]
    events.sort(key=lambda e: e["ts"])
    first = max(i for i, e in enumerate(events) if "embedding" in e["name"])
    events = events[first:]

    def short(name):
        name = name.replace("(anonymous namespace)::", "").replace("<unnamed>::", "")
        return name.split("(")[0].replace("llmcp_b200::", "").replace("void ", "")

    families = collections.defaultdict(lambda: [0, 0.0])
    for e in events:
        entry = families[short(e["name"])]
        entry[0] += 1
        entry[1] += e["dur"]
    span = events[-1]["ts"] + events[-1]["dur"] - events[0]["ts"]
    total = sum(v[1] for v in families.values())
    print(f"mode {mode}: prefill of {PREFILL} tokens spans {span / 1e3:.2f} ms in {len(events)} kernels (sum of durations {total / 1e3:.2f} ms)")
    for name, (n, dur) in sorted(families.items(), key=lambda kv: -kv[1][1]):
        print(f"{name[:64]:64s} n={n:4d} total={dur / 1e3:8.3f} ms  share={dur / total:6.1%}  avg={dur / n:8.1f} us")


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--cpu-steps", type=int, default=16, help="decode steps of the CPU baseline sample")
    parser.add_argument("--mode", default="fast", choices=["fast", "exact"], help="arithmetic mode `value` is measured in")
    parser.add_argument("--parallelism", default="tp", choices=["tp", "replicas"],
                        help="N > 1: tp = one sequence over N GPUs (strong scaling, the default), replicas = one sequence per GPU")
    parser.add_argument("--batch", type=int, default=64, help="sequences of the batched-decode measurement (0 = skip it)")
    parser.add_argument("--only", default="all", choices=["all", "gemv", "gemm", "attn", "timeline", "prefill-timeline"],
                        help="gemv / gemm / attn: run just that kernel on a small case (what the profiler captures); "
                             "timeline: kernel start / end stamps of one decode step (CUDA-graph replay) as text; "
                             "prefill-timeline: device time per kernel family of one 1024-token prefill")
    args = parser.parse_args()
    steps, warmup = max(1, args.steps), max(3, args.warmup)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    workload = ("whole model, Qwen3.5-4B architecture, Q8_0, batch 1 per GPU: greedy decode after a 1024-token "
                "prefill of token 9419")

    if args.impl == "reference":
        # The reference's own CPU implementation needs MLIR/LLVM 20 to exist at all; the CPU oracle
        # restates it.  Rank 0 alone runs, on every host core, on the same 1024-token context as the
        # GPU arm; each step is one greedy decode step of the whole model.  No CUDA library is loaded.
        if rank != 0:
            return
        data, manifest = read_container(ensure_container(0))
        ref_steps, ref_warmup = min(steps, 32), min(warmup, 3)
        run = OracleRun(data, manifest, ref_steps + ref_warmup)
        run.decode(ref_warmup, keep_logits=False)
        tok_s = run.decode(ref_steps, keep_logits=False)
        run.close()
        print(json.dumps({
            "impl": "reference", "metric": "decode_tokens_per_second", "value": tok_s, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": ref_steps, "warmup": ref_warmup, "ms_per_step": 1e3 / tok_s,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": tok_s / M2_DECODE_TOK_S,
            "dtype": "int8xint8->int32, f32 accumulate", "data": "synthetic",
            "config": {"workload": workload, "seed": SEED, "mode": "cpu oracle, fma accumulate"},
            "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": run.threads, "kind": "port",
                             "sample": f"{ref_steps} greedy decode steps after the 1024-token prefill, all host threads",
                             "prefill_tokens_per_second": PREFILL / run.prefill_s},
            "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
        return

    import llmcp_b200 as L
    import torch
    import torch.distributed as dist

    if L.device_count() < 1:
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    L.set_device(local_rank)
    if args.only == "gemv":
        gbs, us, count = gemv_roofline(L, torch, local_rank, ring=6, sweeps=2, flags=19 if args.mode == "fast" else 3)
        print(json.dumps({"only": "gemv", "shape": [1, GEMV_N, GEMV_K], "us_per_launch": us, "gbs": gbs, "launches": count}))
        return
    if args.only == "attn":
        L.set_mode(args.mode)
        row = attention_alone(L)
        print(json.dumps({"only": "attn", "shape": {"heads": 16, "kv_heads": 4, "head_dim": 256, "keys": 1031},
                          "checksum": int(row.astype(np.int64).sum())}))
        return
    if args.only == "gemm":
        us, tops = gemm_alone(L, torch)
        print(json.dumps({"only": "gemm", "shape": [GEMM_M, GEMM_N, GEMM_K], "us_per_launch": us, "int8_tops": tops}))
        return
    if args.only == "timeline":
        decode_timeline(L, torch, args.mode)
        return
    if args.only == "prefill-timeline":
        prefill_timeline(L, torch, args.mode)
        return
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(value):
        if world == 1:
            return value
        t = torch.tensor([value], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    path = ensure_container(local_rank)
    barrier()
    arena = L.Arena().load(path)
    dims = L.default_dims()
    capacity = PREFILL + 2 * (warmup + steps) + 16
    prompt = [TOKEN] * PREFILL
    sampler = ClockSampler(local_rank)
    sampler.start()
    sampler.wait_first_sample()

    # ---- device-resident arm, once per arithmetic mode ---------------------------------------
    # N > 1: one sequence decoded by all N GPUs (tensor parallel: every projection split by output
    # rows, heads split by head, exchanges by the library's peer-store all-gather kernel); the
    # replica throughput (one sequence per GPU, no exchange) is measured beside it.
    tp = None
    if world > 1 and args.parallelism == "tp":
        from llmcp_b200 import parallel
        tp = parallel.TensorParallel(dims, rank, world, local_rank, max_tokens=PREFILL)

    def device_arm(mode, group):
        engine = L.Engine(arena.data, dims, capacity=capacity, device=local_rank, mode=mode, tp=group, max_tokens=PREFILL)
        engine.forward(prompt, 0, want_logits=False)  # warm-up prefill (allocates the workspace)
        engine.reset()
        torch.cuda.synchronize()
        barrier()
        t0 = time.perf_counter()
        first_logits, first = engine.forward(prompt, 0)
        prefill_s = max_over_ranks(time.perf_counter() - t0)
        warm_tokens, _ = engine.generate(first, PREFILL, warmup)
        before = L.launch_count()
        barrier()
        sampler.open_window()
        tokens, device_ms = engine.generate(int(warm_tokens[-1]), PREFILL + warmup, steps)
        barrier()
        sampler.close_window()
        launches = L.launch_count() - before
        return {"ms": max_over_ranks(device_ms), "launches": launches, "prefill_s": prefill_s,
                "tokens": [first] + warm_tokens.tolist() + tokens.tolist(), "first_logits": first_logits, "engine": engine}

    other = "exact" if args.mode == "fast" else "fast"
    main_arm = device_arm(args.mode, tp)
    if world > 1:
        main_arm.pop("engine").close()
    side_arm = device_arm(other, tp)
    side_arm.pop("engine").close()
    device_ms, launches = main_arm["ms"], main_arm["launches"]
    sequences = 1 if tp is not None else world
    value = sequences * steps / (device_ms / 1e3)
    replicas = None
    if tp is not None:
        # One full engine per GPU, each with its own sequence: the no-exchange figure, and (exact
        # mode) the single-GPU tokens the tensor-parallel ones have to equal.
        replica_arm = device_arm(args.mode, None)
        replica_arm.pop("engine").close()
        replica_exact = replica_arm if args.mode == "exact" else device_arm("exact", None)
        if replica_exact is not replica_arm:
            replica_exact.pop("engine").close()
        tp_exact = main_arm if args.mode == "exact" else side_arm
        replicas = {"value": world * steps / (replica_arm["ms"] / 1e3), "unit": "tokens/s", "ms_per_step": replica_arm["ms"] / steps,
                    "scaling": "weak", "tp_tokens_equal_single_gpu_exact_mode": tp_exact["tokens"] == replica_exact["tokens"]}

    # ---- against the CPU oracle on the same context (rank 0 of a one-GPU run) ----------------
    # The oracle's greedy chain from the same prompt, its logits at every position of the chain and
    # its top-1/top-2 margins; the GPU engine is fed the oracle's tokens (teacher forcing), so one
    # low-margin position cannot derail the comparison of the positions behind it.
    check, cpu_baseline = None, None
    if rank == 0 and world == 1:
        run = OracleRun(arena.data, arena.manifest, args.cpu_steps)
        tok_s = run.decode(args.cpu_steps)
        margins = [run.oracle.top2_margin(row) for row in run.logits]
        engine = main_arm["engine"]
        engine.reset()
        logits, token = engine.forward(prompt, 0)
        worst = float(np.abs(logits - run.logits[0]).max())
        same = [token == run.tokens[0]]
        for i in range(args.cpu_steps):
            logits, token = engine.forward([run.tokens[i]], PREFILL + i)
            worst = max(worst, float(np.abs(logits - run.logits[i + 1]).max()))
            same.append(token == run.tokens[i + 1])
        n = args.cpu_steps + 1
        exact_tokens = side_arm["tokens"] if other == "exact" else main_arm["tokens"]
        check = {"positions": n, "tokens_match_oracle": bool(all(same)), "tokens_equal": int(sum(same)),
                 "max_abs_logit_diff": worst, "min_top2_margin": float(min(margins)),
                 "median_top2_margin": float(np.median(margins)),
                 "exact_mode_tokens_match_oracle": exact_tokens[:n] == run.tokens[:n],
                 "how": "engine fed the oracle's greedy tokens (1024-token prompt + cpu-steps positions); logits compared "
                        "position by position; exact mode: its own greedy chain against the oracle's"}
        # The same positions through the reference's other accumulate variant (multiply-then-add,
        # Q8Scalar.cpp:192-199): how far two orders of f32 rounding that the reference itself
        # ships move the logits of this random-init model.
        alt = OracleRun(arena.data, arena.manifest, args.cpu_steps, mode="muladd")
        alt_rows = alt.forced(run.tokens[:args.cpu_steps])
        check["reference_fma_vs_muladd_max_abs"] = float(max(np.abs(a - b).max() for a, b in zip(alt_rows, run.logits)))
        alt.close()
        cpu_baseline = {"value": tok_s, "unit": "tokens/s", "cores": run.threads, "kind": "port",
                        "sample": f"{args.cpu_steps} greedy decode steps after the same 1024-token prefill, CPU oracle "
                                  "(OpenMP, all host threads)",
                        "prefill_tokens_per_second": PREFILL / run.prefill_s}
        run.close()
    if "engine" in main_arm:
        main_arm.pop("engine").close()

    # ---- end-to-end arm ----------------------------------------------------------------------
    # One GPU or replicas: through the AOT ABI entry points with host buffers, as tools/llmcp-benchmark
    # calls them.  Tensor parallel: the engine's forward call on every rank (token in from the host,
    # the assembled logits row out to the host, argmax on the host): the AOT ABI has no notion of ranks.
    if tp is None:
        L.set_mode(args.mode)
        runtime = L.AotRuntime(dims)
        assert runtime.init(max_sequence=capacity)
        logits = np.zeros(dims.vocab, dtype=np.float32)  # one host row for every call, as llmcp-benchmark.cpp:84-101 keeps
        step = lambda tokens, position: runtime.forward(arena, tokens, position, position + len(tokens), logits)
    else:
        e2e_engine = L.Engine(arena.data, dims, capacity=capacity, device=local_rank, mode=args.mode, tp=tp, max_tokens=PREFILL)
        step = lambda tokens, position: e2e_engine.forward(tokens, position)[0]
    logits = step(prompt, 0)
    pos = PREFILL
    for _ in range(warmup):
        logits = step([int(np.argmax(logits))], pos)
        pos += 1
    barrier()
    sampler.open_window()
    t0 = time.perf_counter()
    e2e_tokens = []
    for _ in range(steps):
        e2e_tokens.append(int(np.argmax(logits)))
        logits = step([e2e_tokens[-1]], pos)
        pos += 1
    torch.cuda.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    sampler.close_window()
    clocks = sampler.stop()
    barrier()
    # e2e prefill: a fresh 1024-token call through the same entry point
    t0 = time.perf_counter()
    step(prompt, 0)
    e2e_prefill_s = max_over_ranks(time.perf_counter() - t0)
    if tp is not None:
        e2e_engine.close()
        tp.close()
    L.lib().llmcp_b200_release_all()
    if L.last_error():
        raise SystemExit("library error: " + L.last_error())
    same = e2e_tokens == main_arm["tokens"][warmup:warmup + steps]

    bytes_per_step = 4.61e9  # weights 4.468 GB + recurrent state 0.101 GB + KV and logits
    result = {
        "metric": "decode_tokens_per_second", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": device_ms / steps, "higher_is_better": True,
        "scaling": "strong" if tp is not None else "weak",
        "vs_baseline": value / sequences / M2_DECODE_TOK_S, "dtype": "int8xint8->int32, f32 accumulate", "data": "synthetic",
        "config": {"workload": workload if tp is None else workload.replace("batch 1 per GPU", f"batch 1 over {world} GPUs"),
                   "mode": args.mode, "seed": SEED,
                   "parallelism": f"tp{world}: rows of every projection, heads and vocabulary split over {world} GPUs; "
                                  "peer-store all-gather kernels, 4 per layer" if tp is not None
                   else f"replica x{world}" if world > 1 else "single GPU",
                   "l2": "each step streams the 4.47 GB arena, far larger than L2; no flush needed",
                   "vs_baseline_is": "per-GPU value / 11.39 tok/s published for Apple M2 (reference README.md:140)"},
        f"{other}_mode": {"value": sequences * steps / (side_arm["ms"] / 1e3), "unit": "tokens/s",
                          "ms_per_step": side_arm["ms"] / steps,
                          "prefill_tokens_per_second": PREFILL / side_arm["prefill_s"]},
        "e2e": {"value": sequences * steps / e2e_s, "unit": "tokens/s", # one packet in: position, token, cos row, sin row; logits row, token and status word back
                "h2d_bytes_per_step": (16 + 2 * dims.rotary * 4) * world,
                "d2h_bytes_per_step": (dims.vocab * 4 + 16) * world, "tokens_match_device_arm": bool(same)},
        "gpu_launches": int(launches) * world,
        "clocks": clocks,
        "prefill_tokens_per_second": {"tokens": PREFILL, "engine": PREFILL / main_arm["prefill_s"],
                                      "e2e_abi": PREFILL / e2e_prefill_s},
        "whole_step_roofline": {"bytes_per_step": bytes_per_step, "gpus_sharing_the_bytes": 1 if tp is None else world,
                                "achieved_gbs": bytes_per_step / (1 if tp is None else world) / (device_ms / steps / 1e3) / 1e9},
    }
    if replicas:
        result["replicas"] = replicas
    if check:
        result["parity"] = check
        result["tokens_match_oracle"] = check["tokens_match_oracle"]
        result["min_top2_margin"] = check["min_top2_margin"]

    if rank == 0:
        peak, tensor_peak, peak_kind = measured_peaks()
        fast = args.mode == "fast"
        gbs, us, gemv_launches = gemv_roofline(L, torch, local_rank, flags=19 if fast else 3)
        gbs_other, us_other, _ = gemv_roofline(L, torch, local_rank, flags=3 if fast else 19)
        result["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                              "traffic": GEMV_DRAM_TRAFFIC, "traffic_source": "ncu capture of `bench.py --only gemv`, not this run",
                              "kernel": "gemv_q8_cols80_kernel" + ("<fast>" if fast else ""), "shape": [1, GEMV_N, GEMV_K],
                              "us_per_launch": us, "launches_timed": gemv_launches, "peak_kind": f"of {peak_kind}",
                              "algorithmic_bytes_per_launch": GEMV_BYTES,
                              f"{other}_mode": {"achieved": gbs_other, "frac": gbs_other / peak, "us_per_launch": us_other}}
        result["whole_step_roofline"]["frac"] = result["whole_step_roofline"]["achieved_gbs"] / peak
        gemm_us, tops = gemm_alone(L, torch)
        int8_peak = 2.0 * tensor_peak  # no int8 peak is on file: twice the measured dense bf16 burst
        # The f32 accumulation per 32-block (convert, scale product, fma) runs on the CUDA cores:
        # 3 operations per (row, column, block) on 148 SMs x 128 lanes at the sampled SM clock.
        sm_mhz = clocks.get("sm_mhz") or clocks.get("sm_max_mhz") or 1965.0
        epilogue_us = GEMM_M * GEMM_N * (GEMM_K // 32) * 3 / (148 * 128 * sm_mhz)
        result["roofline_gemm"] = {"bound": "tensor", "kernel": "gemm_q8_tma_kernel", "shape": [GEMM_M, GEMM_N, GEMM_K],
                                   "us_per_launch": gemm_us, "achieved": tops, "unit": "int8 TOP/s", "peak": int8_peak,
                                   "peak_kind": f"2 x bf16 burst, of {peak_kind}", "frac": tops / int8_peak,
                                   "epilogue_bound_us": epilogue_us,
                                   "epilogue_bound_tops": 2.0 * GEMM_M * GEMM_N * GEMM_K / epilogue_us / 1e6,
                                   "frac_of_epilogue_bound": epilogue_us / gemm_us}
    if rank == 0 and world == 1 and args.batch > 1:
        # Batch of independent sequences (the batched configuration of the benchmark list): every
        # sequence prefilled with its own 1024 tokens, then all decoded together, one token each per
        # step.  Two prompt sets: all 1024 x token 9419, and ids drawn per sequence.
        batch, batch_steps = args.batch, 16
        engine = L.Engine(arena.data, dims, capacity=PREFILL + 2 * batch_steps + 8, device=local_rank, mode=args.mode, batch=batch)
        rng = np.random.default_rng(SEED + 5)
        sets = {}
        for name in ("all_9419", "per_sequence_random"):
            engine.reset()
            firsts = []
            t0 = time.perf_counter()
            for b in range(batch):
                ids = prompt if name == "all_9419" else rng.integers(0, dims.vocab, PREFILL).tolist()
                engine.select_sequence(b)
                firsts.append(engine.forward(ids, 0, want_logits=False)[1])
            batch_prefill_s = time.perf_counter() - t0
            warm, _ = engine.generate_batch(firsts, PREFILL, 4)
            tokens_b, ms_b = engine.generate_batch(warm[-1], PREFILL + 4, batch_steps)
            sets[name] = {"value": batch * batch_steps / (ms_b / 1e3), "unit": "tokens/s", "ms_per_step": ms_b / batch_steps,
                          "prefill_tokens_per_second": batch * PREFILL / batch_prefill_s,
                          "distinct_sequences": len({tuple(col) for col in tokens_b.T.tolist()})}
        engine.close()
        # per step: weights once, and per sequence the recurrent state (read and written) and the KV cache
        step_bytes = 4.47e9 + batch * (2 * 100.7e6 + 8 * 4096 * (PREFILL + 4 + batch_steps // 2))
        result["batch"] = {"sequences": batch, "steps": batch_steps, "mode": args.mode, "sets": sets,
                           "bytes_per_step": step_bytes,
                           "achieved_gbs": step_bytes / (sets["all_9419"]["ms_per_step"] / 1e3) / 1e9,
                           "parity": "each sequence against its own one-sequence oracle run: tests/test_gpu_batch.py"}
    if cpu_baseline:
        result["cpu_baseline"] = cpu_baseline
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
