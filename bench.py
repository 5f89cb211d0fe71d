#!/usr/bin/env python3
"""Benchmark of the llmcp Q8_0 hot path on B200.

Workload (BASELINE.json configs[4], batch 1): a random-init Qwen3.5-4B-architecture model
packed with --quant q8_0 (seeded synthetic weights with the real shapes and dtypes; the real
checkpoint is not available offline), 1024 x token 9419 prefill, then greedy decode.  One
"step" is one decode step of the whole model: every weight byte of the arena streams from HBM
once (4.47 GB, far more than the 126 MB L2, so no cache flush is needed between steps).

  value  decode tokens/s with token, state and logits resident in HBM (engine interface),
         timed with CUDA events on the launching stream, max over ranks;
  e2e    the same steps through the reference-facing AOT ABI entry point with host buffers:
         token, cos and sin rows go host -> device, the 248320-float logits row comes back
         and the argmax is taken on the host, as tools/llmcp-benchmark does;
  roofline  the decode GEMV (N=9216, K=2560, the gate_proj/up_proj shape; BASELINE.json
         configs[0]) timed alone with CUDA events over a ring of 12 weight copies (301 MB);
  cpu_baseline  the CPU oracle (a restatement of the reference's arithmetic; the reference's
         own AOT build needs an MLIR toolchain that is not installed) on the host cores.

N > 1 (torchrun): every rank holds a full replica and decodes its own sequence; no collective
on the data path, so scaling is "weak" and value is the sum over ranks.

`--impl reference` times the CPU oracle alone on the same workload and prints the same line.
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
# dram__bytes_read.sum + dram__bytes_write.sum of one gemv_q8_cols80_kernel launch of this shape, from the
# ncu capture summarised in profiles/gemv_q8_cols80_9216x2560.md (the 36,864-byte result stays in L2).
GEMV_DRAM_TRAFFIC = 25_097_216
GEMM_M, GEMM_N, GEMM_K = 1024, 9216, 2560  # the gate_proj/up_proj prefill GEMM (BASELINE.json configs[1] shape)


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device = device
        self.lines = []  # (host time, text)
        self.windows = []  # [begin, end] host times of the timed regions
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def wait_first_sample(self, seconds=5.0):
        deadline = time.perf_counter() + seconds
        while self.proc and not self.lines and time.perf_counter() < deadline:
            time.sleep(0.01)

    def open_window(self):
        self.windows.append([time.perf_counter(), None])

    def close_window(self):
        self.windows[-1][1] = time.perf_counter()

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = lambda t: any(b <= t <= (e if e is not None else t) for b, e in self.windows)
        for stamp, line in self.lines:
            if self.windows and not inside(stamp):
                continue
            parts = [p.strip() for p in line.split(",")]
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
                "sampled": "nvidia-smi every 20 ms, samples inside the two timed loops (device arm and ABI arm)"}


def container_path(local_rank, world):
    """One synthetic container per node in /dev/shm, written by local rank 0."""
    import llmcp_b200 as L
    path = pathlib.Path("/dev/shm") / f"llmcp_b200_synth_{SEED}.bin"
    if local_rank == 0 and not path.exists():
        data = L.synthetic_container(L.default_dims(), SEED)
        tmp = path.with_suffix(f".{os.getpid()}.tmp")
        data.tofile(tmp)
        os.replace(tmp, path)
        del data
    return path


def oracle_decode(arena, steps, warmup, prefill=8):
    """Greedy decode with the CPU oracle: returns (tokens/s, tokens, threads)."""
    import llmcp_b200 as L
    import oracle
    d = L.default_dims()
    model = oracle.Model(arena.data, arena.manifest, dict(
        full_interval=d.full_interval, heads=d.heads, kv_heads=d.kv_heads, head_dim=d.head_dim, rotary=d.rotary,
        lin_k_heads=d.lin_k_heads, lin_v_heads=d.lin_v_heads, lin_k_dim=d.lin_k_dim, lin_v_dim=d.lin_v_dim,
        conv_kernel=d.conv_kernel))
    state = model.new_state(prefill + warmup + steps + 1)
    logits = model.forward(state, [TOKEN] * prefill, 0)  # also unpacks the weights once
    pos, tokens = prefill, []
    for _ in range(warmup):
        logits = model.forward(state, [oracle.argmax(logits)], pos)
        pos += 1
    begin = time.perf_counter()
    for _ in range(steps):
        tokens.append(oracle.argmax(logits))
        logits = model.forward(state, [tokens[-1]], pos)
        pos += 1
    seconds = time.perf_counter() - begin
    model.close()
    return steps / seconds, tokens, oracle.num_threads()


def gemv_roofline(L, torch, device, ring=GEMV_RING, sweeps=20):
    """Decode GEMV alone: CUDA events on the launching stream over a ring of weight copies."""
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
                                           C.c_int64(GEMV_N), ptr(y), 0, 0, 0, 1, C.c_void_p(stream))
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


def gemm_alone(L, torch, repeats=5):
    """Prefill GEMM alone (tcgen05 kernel) on device buffers: returns (us per launch, int8 TOP/s)."""
    lib = L.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    gen = torch.Generator(device="cuda").manual_seed(SEED)
    nb = GEMM_K // 32
    wq = torch.randint(-127, 128, (GEMM_N, GEMM_K), dtype=torch.int8, device="cuda", generator=gen)
    wd = (torch.rand((GEMM_N, nb), device="cuda", generator=gen) * 1e-3).to(torch.float16)
    x = torch.randn((GEMM_M, GEMM_K), device="cuda", generator=gen)
    aq = torch.empty((GEMM_M, GEMM_K), dtype=torch.int8, device="cuda")
    scales = torch.empty((GEMM_M, nb), dtype=torch.float32, device="cuda")
    wd32 = wd.float().contiguous()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = torch.empty((GEMM_M, GEMM_N), dtype=torch.float32, device="cuda")
    ptr = lambda t: C.c_void_p(t.data_ptr())
    assert lib.llmcp_dev_act_quant(ptr(x), 0, C.c_int64(GEMM_M), C.c_int64(GEMM_K), ptr(aq), ptr(scales), stream) == 0

    def launch():
        rc = lib.llmcp_dev_gemm_q8_tc(ptr(aq), ptr(scales), C.c_int64(GEMM_M), C.c_int64(GEMM_K), ptr(wq), ptr(wd32),
                                      C.c_int64(GEMM_N), ptr(y), 0, 0, ptr(status), stream)
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


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--cpu-steps", type=int, default=8, help="decode steps of the CPU baseline sample")
    parser.add_argument("--only", default="all", choices=["all", "gemv", "gemm", "attn"],
                        help="gemv / gemm / attn: run just that kernel on a small case (what the profiler captures)")
    args = parser.parse_args()
    steps, warmup = max(1, args.steps), max(3, args.warmup)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    import llmcp_b200 as L

    if args.impl == "reference":
        # The reference's own CPU implementation needs MLIR/LLVM 20 to exist at all; the CPU
        # oracle restates it.  Rank 0 alone runs; each step is one greedy decode step of the
        # whole model (a short 8-token context keeps the run within minutes; decode cost is
        # dominated by the 4.47 GB of weights and barely depends on the context length).
        if rank != 0:
            return
        arena = L.Arena().load(container_path(0, 1))
        ref_steps = min(steps, 32)
        tok_s, tokens, threads = oracle_decode(arena, ref_steps, min(warmup, 3))
        print(json.dumps({
            "impl": "reference", "metric": "decode_tokens_per_second", "value": tok_s, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": ref_steps, "warmup": min(warmup, 3), "ms_per_step": 1e3 / tok_s,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": tok_s / M2_DECODE_TOK_S, "dtype": "int8xint8->int32, f32 accumulate",
            "data": "synthetic",
            "config": {"workload": "configs[4]: Qwen3.5-4B-architecture Q8_0 whole model, batch 1, greedy decode",
                       "context": "8-token prefill (bounded sample)", "seed": SEED},
            "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": threads, "kind": "port",
                             "sample": f"{ref_steps} greedy decode steps after an 8-token prefill, all host threads"},
            "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
        return

    import torch
    import torch.distributed as dist

    if L.device_count() < 1:
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    L.set_device(local_rank)
    if args.only == "gemv":
        gbs, us, count = gemv_roofline(L, torch, local_rank, ring=6, sweeps=2)
        print(json.dumps({"only": "gemv", "shape": [1, GEMV_N, GEMV_K], "us_per_launch": us, "gbs": gbs, "launches": count}))
        return
    if args.only == "attn":
        row = attention_alone(L)
        print(json.dumps({"only": "attn", "shape": {"heads": 16, "kv_heads": 4, "head_dim": 256, "keys": 1031},
                          "checksum": int(row.astype(np.int64).sum())}))
        return
    if args.only == "gemm":
        us, tops = gemm_alone(L, torch)
        print(json.dumps({"only": "gemm", "shape": [GEMM_M, GEMM_N, GEMM_K], "us_per_launch": us, "int8_tops": tops}))
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

    path = container_path(local_rank, world)
    barrier()
    while not path.exists():
        time.sleep(0.2)
    arena = L.Arena().load(path)
    dims = L.default_dims()
    capacity = PREFILL + 2 * (warmup + steps) + 16

    # ---- device-resident arm --------------------------------------------------------------
    engine = L.Engine(arena.data, dims, capacity=capacity, device=local_rank)
    prompt = [TOKEN] * PREFILL
    engine.forward(prompt, 0, want_logits=False)  # warm-up prefill (allocates the workspace)
    engine.reset()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    _, first = engine.forward(prompt, 0, want_logits=False)
    prefill_s = time.perf_counter() - t0
    warm_tokens, _ = engine.generate(first, PREFILL, warmup)
    sampler = ClockSampler(local_rank)
    sampler.start()
    sampler.wait_first_sample()
    launches_before = L.launch_count()
    barrier()
    sampler.open_window()
    tokens, device_ms = engine.generate(int(warm_tokens[-1]), PREFILL + warmup, steps)
    barrier()
    sampler.close_window()
    launches = L.launch_count() - launches_before
    device_ms = max_over_ranks(device_ms)
    value = world * steps / (device_ms / 1e3)
    engine.close()

    # ---- end-to-end arm through the AOT ABI ------------------------------------------------
    runtime = L.AotRuntime(dims)
    assert runtime.init(max_sequence=capacity)
    logits = np.zeros(dims.vocab, dtype=np.float32)  # one host row for every call, as llmcp-benchmark.cpp:84-101 keeps
    runtime.forward(arena, prompt, 0, PREFILL, logits)
    pos = PREFILL
    for _ in range(warmup):
        runtime.forward(arena, [int(np.argmax(logits))], pos, pos + 1, logits)
        pos += 1
    barrier()
    sampler.open_window()
    t0 = time.perf_counter()
    e2e_tokens = []
    for _ in range(steps):
        e2e_tokens.append(int(np.argmax(logits)))
        runtime.forward(arena, [e2e_tokens[-1]], pos, pos + 1, logits)
        pos += 1
    torch.cuda.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    sampler.close_window()
    clocks = sampler.stop()
    barrier()
    # e2e prefill: a fresh 1024-token call through the same entry point
    t0 = time.perf_counter()
    runtime.forward(arena, prompt, 0, PREFILL)
    e2e_prefill_s = max_over_ranks(time.perf_counter() - t0)
    L.lib().llmcp_b200_release_all()
    if L.last_error():
        raise SystemExit("library error: " + L.last_error())
    same = e2e_tokens[1:] == tokens.tolist()[:steps - 1]

    result = {
        "metric": "decode_tokens_per_second", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": device_ms / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / world / M2_DECODE_TOK_S, "dtype": "int8xint8->int32, f32 accumulate", "data": "synthetic",
        "config": {"workload": "configs[4]: Qwen3.5-4B-architecture Q8_0 whole model, batch 1 per GPU, greedy decode "
                               "after a 1024-token prefill of token 9419",
                   "seed": SEED, "parallelism": f"replica x{world}" if world > 1 else "single GPU",
                   "l2": "each step streams the 4.47 GB arena, far larger than L2; no flush needed",
                   "vs_baseline_is": "per-GPU value / 11.39 tok/s published for Apple M2 (reference README.md:140)"},
        "e2e": {"value": world * steps / e2e_s, "unit": "tokens/s", # one packet in: position, token, cos row, sin row; logits row, token and status word back
                "h2d_bytes_per_step": 16 + 2 * dims.rotary * 4,
                "d2h_bytes_per_step": dims.vocab * 4 + 16, "tokens_match_device_arm": bool(same)},
        "gpu_launches": int(launches) * world,
        "clocks": clocks,
        "prefill_tokens_per_second": {"tokens": PREFILL, "engine": PREFILL / prefill_s, "e2e_abi": PREFILL / e2e_prefill_s},
    }

    if rank == 0:
        peak, peak_kind = measured_peaks()
        gbs, us, gemv_launches = gemv_roofline(L, torch, local_rank)
        result["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                              "traffic": GEMV_DRAM_TRAFFIC, "kernel": "gemv_q8_cols80_kernel", "shape": [1, GEMV_N, GEMV_K],
                              "us_per_launch": us, "launches_timed": gemv_launches, "peak_kind": f"of {peak_kind}",
                              "algorithmic_bytes_per_launch": GEMV_BYTES,
                              "whole_model_effective_gbs": 4.61e9 / (device_ms / steps / 1e3) / 1e9}
    if rank == 0 and world == 1:
        tok_s, cpu_tokens, threads = oracle_decode(arena, args.cpu_steps, 1)
        result["cpu_baseline"] = {"value": tok_s, "unit": "tokens/s", "cores": threads, "kind": "port",
                                  "sample": f"{args.cpu_steps} greedy decode steps after an 8-token prefill of the same "
                                            "model with the CPU oracle (OpenMP, all host threads)"}
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
