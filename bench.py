#!/usr/bin/env python
"""Benchmark of the B200 PSSA inference forward path.  `python bench.py --gpus N --steps K --warmup W`

Workload `prefill_c4` (BASELINE.json configs[3]): stacked PSSA, 12 blocks, d_model 768, state 64, key 64,
512-slot full memory bank per block, vocab 16384, bf16 projections on the tensor cores, fp32 scan and retrieval;
one step = batched prefill of 32 independent sequences x 2048 tokens on each GPU (token ids uniform in [1, V),
random-init weights N(0, 0.02), decays exp(A) ~ U(0.9, 0.999); synthetic, seeded). Metric: prefill tokens per
second. `value` is timed with CUDA events on device-resident ids (pssa_b200_model_prefill_batch_dev); `e2e` goes
through the host-pointer C ABI (pssa_b200_model_prefill_batch: pinned host ids in, host logits out).

At N > 1 every rank prefills its own 32 sequences (independent lanes: no collective on the data path).

`roofline` describes the kernel with the largest share of the step, timed live by the library's per-kernel CUDA
events. `extra` (N = 1 only) adds the operator-alone workloads of BASELINE.json: the scan (configs[1]), the
retrieval operator (configs[2]) and batched decode.

`--impl reference` times the CPU restatement of the reference's token-serial prefill (oracle/, all host threads)
on a bounded sample of the same workload.
"""
import argparse
import json
import os
import pathlib
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CFG = dict(depth=12, d_vocab=16384, d_latent=768, d_state=64, d_mem_key=64, mem_capacity=512)
LANES, T = 32, 2048
WORKLOAD = ("prefill_c4: 12-block PSSA (d 768, state 64, key 64, 512 slots, vocab 16384), bf16 projections, fp32 scan "
            "and retrieval; 32 sequences x 2048 tokens per GPU")
CPU_SAMPLE_LANES, CPU_SAMPLE_T = 16, 16
# dram bytes per scan element, from the ncu capture of the scan kernel summarised under profiles/
NCU_SCAN_TRAFFIC_BYTES_PER_ELEM = 11.87
# dram bytes per token row of one ssm_fused_kernel launch, from its ncu capture summarised under profiles/
# (read 225.5 MB + write 119.9 MB over 32768 rows); traffic grows in proportion to the rows
NCU_SSM_TRAFFIC_BYTES_PER_ROW = (225.52e6 + 119.92e6) / 32768


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops_sustained"]), "measured"
    return 6650.0, 1400.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        load = [c for c, p in zip(sm, power) if p > 0.5 * max(power)] or sm  # samples taken while the GPU worked
        return {"sm_mhz": statistics.median(load), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm),
                "power_w_max": max(power)}


def synth_weights(seed: int):
    """Seeded synthetic parameters of the C4 model as {(layer, tensor id): array}, plus banks per block."""
    from pssa_b200 import model as M
    rng = np.random.default_rng(seed)
    d, s, k, cap, v = CFG["d_latent"], CFG["d_state"], CFG["d_mem_key"], CFG["mem_capacity"], CFG["d_vocab"]

    def normal(*shape):
        return rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)

    tensors = {(-1, M.EMBED): normal(v, d), (-1, M.UNEMBED): normal(v, d)}
    banks = []
    for l in range(CFG["depth"]):
        for tid, shape in ((M.W_DELTA, (d, d)), (M.W_B, (s, d)), (M.W_C, (s, d)), (M.W_QX, (k, d)), (M.W_QH, (k, d)),
                           (M.W_GATE, (d, d)), (M.W_PROJ, (d, d)), (M.MLP_W1, (2 * d, d)), (M.MLP_W2, (d, 2 * d)),
                           (M.AD_DOWN, (16, d)), (M.AD_UP, (d, 16)), (M.AD_CONS, (d, 16))):
            tensors[(l, tid)] = normal(*shape)
        u = rng.uniform(0.9, 0.999, d * s)
        tensors[(l, M.A_MAT)] = np.log(np.expm1(-np.log(u))).astype(np.float32)  # exp(-softplus(raw)) = u
        dirs = rng.standard_normal((cap, k))
        dirs /= np.linalg.norm(dirs, axis=1, keepdims=True)
        keys = (dirs * rng.uniform(0, 0.9, (cap, 1))).astype(np.float32)
        norm_sq = (keys.astype(np.float64) ** 2).sum(1).astype(np.float32)
        banks.append((keys, norm_sq, rng.standard_normal((cap, d), dtype=np.float32)))
    return tensors, banks


def oracle_model(tensors, banks):
    import oracle as O
    om = O.Model.new(CFG["depth"], CFG["d_vocab"], CFG["d_latent"], CFG["d_state"], CFG["d_mem_key"], CFG["mem_capacity"],
                     tau_mem=0.1, seed=1)
    for (layer, tid), arr in tensors.items():
        om.tensor(layer, tid)[:] = arr.ravel()
    for l, (keys, norm_sq, values) in enumerate(banks):
        om.tensor(l, O.BANK_KEYS)[:] = keys.ravel()
        om.tensor(l, O.BANK_NORM_SQ)[:] = norm_sq
        om.tensor(l, O.BANK_VALUES)[:] = values.ravel()
        om.set_bank_meta(l, CFG["mem_capacity"], 0)
    return om


def cpu_sample_ids(seed=7):
    return np.random.default_rng(seed).integers(1, CFG["d_vocab"], (CPU_SAMPLE_LANES, CPU_SAMPLE_T)).astype(np.uint64)


def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import oracle as O
    threads = max(1, O.lib().pssa_oracle_hardware_threads())
    tensors, banks = synth_weights(1234)
    om = oracle_model(tensors, banks)
    ids = cpu_sample_ids()
    times = []
    for _ in range(args.warmup + args.steps):
        sec, _ = om.prefill_lanes_timed(ids, threads)
        times.append(sec)
    times = times[args.warmup:]
    ms = 1e3 * sum(times) / len(times)
    value = ids.size / (ms / 1e3)
    sample = (f"{CPU_SAMPLE_LANES} sequences x {CPU_SAMPLE_T} tokens of the same 12-block model per step, token-serial "
              f"prefill_inference, lanes over {threads} host threads")
    print(json.dumps({
        "impl": "reference", "metric": "prefill_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def kernel_roofline(name, launches, ms, rows, peak_hbm, peak_tf, tc_distances=False):
    """Algorithmic work of one launch of `name` on `rows` token rows of the C4 block -> achieved rate."""
    d, s, k, cap = CFG["d_latent"], CFG["d_state"], CFG["d_mem_key"], CFG["mem_capacity"]
    per = ms / launches / 1e3
    if "ssm_fused" in name:
        # in: delta, x (4d each), B, C (4s each); out: y fp32 + bf16 (6d); carry in and out once per lane
        byts = rows * ((2 * d + 2 * s) * 4 + 6 * d) + LANES * 2 * d * s * 4
        exps = rows * d * s
        return {"bound": "hbm", "achieved": byts / per / 1e9, "peak": peak_hbm, "unit": "GB/s",
                "frac": byts / per / 1e9 / peak_hbm, "traffic": NCU_SSM_TRAFFIC_BYTES_PER_ROW * rows,
                "limiter": "exp (MUFU) throughput: d*s exponentials per token against 16 per SM per clock",
                "limiter_achieved_gexp_s": exps / per / 1e9, "limiter_peak_gexp_s": 148 * 16 * 1.965,
                "limiter_frac": exps / per / 1e9 / (148 * 16 * 1.965)}
    if "gemm_bf16" in name:
        # algorithmic flops of a block's dense products (the value read counts once, not its six bf16 partial products)
        flop = 2 * rows * d * ((2 * d + 2 * s + k + 16) + k + d + 2 * d + 2 * d) + 2 * rows * d * cap
        if tc_distances:  # the query-key inner products of the distance stage run there too (counted once, like the value read)
            flop += 2 * rows * cap * k
        # `ms` covers every tensor-core launch of the step: report the aggregate rate
        return {"bound": "tensor", "achieved": flop * CFG["depth"] / (ms / 1e3) / 1e12, "peak": peak_tf, "unit": "TFLOP/s",
                "frac": flop * CFG["depth"] / (ms / 1e3) / 1e12 / peak_tf}
    if "poincare_distance" in name:
        byts = rows * (k * 4 + cap * 4)
        return {"bound": "hbm", "achieved": byts / per / 1e9, "peak": peak_hbm, "unit": "GB/s", "frac": byts / per / 1e9 / peak_hbm,
                "limiter": "FP32 FMA pipe (fast mode: packed fp32 squared differences, 2 ops per key dimension)"
                if "f32" in name else "fp64 FMA + log1p/sqrt (distances are f64 like the reference)"}
    return None


def run_decode_extra(model, gpu, torch, peak_hbm):
    """Batched greedy decode of 256 concurrent streams on the same 12-block model (the decode half of BASELINE's
    long-context configuration): 16-token prompts, then timed steps of one token per stream through
    pssa_b200_model_decode_step, greedy ids back on the host every step (they are the next step's input)."""
    streams, warm, steps = 256, 4, 64
    rng = np.random.default_rng(7)
    model.reset_recurrent_state()
    _, ids = model.prefill_batch([rng.integers(1, CFG["d_vocab"], 16) for _ in range(streams)], want_logits=False,
                                 want_greedy=True)
    for _ in range(warm):
        ids = model.decode_step(ids, want_logits=False, want_greedy=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        ids = model.decode_step(ids, want_logits=False, want_greedy=True)
    torch.cuda.synchronize()
    sec = (time.perf_counter() - t0) / steps
    # the same step captured as a CUDA graph, ids fed back on the device: no host round trip per token
    ids_dev = torch.tensor(ids.astype(np.int32), device="cuda", dtype=torch.int32)
    graph = model.capture_greedy_decode_graph(ids_dev)
    for _ in range(warm):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    graph_sec = e0.elapsed_time(e1) / 1e3 / steps
    gpu.poll_status()
    d, s = CFG["d_latent"], CFG["d_state"]
    state_bytes = streams * CFG["depth"] * d * s * 4 * 2  # every carry read and written once per step
    v, k = CFG["d_vocab"], CFG["d_mem_key"]
    weight_elems = v * d + CFG["depth"] * (2 * d * d + 2 * s * d + 2 * k * d + d * d + 4 * d * d + 32 * d)  # head + blocks
    weight_bytes = weight_elems * 2
    return {"workload": "greedy decode, 256 streams x 1 token per step, 12-block model, ids to host every step",
            "ms_per_step": sec * 1e3, "tokens_per_s": streams / sec, "steps": steps,
            "cuda_graph": {"ms_per_step": graph_sec * 1e3, "tokens_per_s": streams / graph_sec,
                           "note": "one captured greedy step replayed; ids stay on the device (CUDA events)"},
            "roofline": {"bound": "hbm", "achieved": (state_bytes + weight_bytes) / sec / 1e9, "peak": peak_hbm, "unit": "GB/s",
                         "frac": (state_bytes + weight_bytes) / sec / 1e9 / peak_hbm,
                         "note": "algorithmic bytes = recurrent state in and out + bf16 weights once; the step is 136 "
                                 "launches of which 73 are M = 256 GEMM tiles bound by their own latency"}}


def run_generate_c1(gpu):
    """configs[0], the reference's own CPU case: one block, vocabulary 8192, d 192, state 64, 512 slots; batch 1,
    prefill 512 tokens then 200 greedy tokens (the reference publishes 200 tokens in 226 ms on its CPU path)."""
    import pssa_b200
    from pssa_b200 import _native as N
    from pssa_b200 import model as M
    v, d, s, k, cap = 8192, 192, 64, 64, 512
    rng = np.random.default_rng(3)
    out = {}
    for name, precision in (("fp32_exact", N.PRECISION_FP32_EXACT), ("bf16", N.PRECISION_BF16)):
        m = pssa_b200.PSSAModel(gpu, 1, v, d, s, k, cap, tau_mem=0.1, streams=1, precision=precision)
        nrm = lambda *shape: (rng.standard_normal(shape) * 0.02).astype(np.float32)  # noqa: E731
        m.set_tensor(-1, M.EMBED, nrm(v, d))
        m.set_tensor(-1, M.UNEMBED, nrm(v, d))
        for tid, shape in ((M.W_DELTA, (d, d)), (M.W_B, (s, d)), (M.W_C, (s, d)), (M.W_QX, (k, d)), (M.W_QH, (k, d)),
                           (M.W_GATE, (d, d)), (M.W_PROJ, (d, d)), (M.MLP_W1, (2 * d, d)), (M.MLP_W2, (d, 2 * d)),
                           (M.AD_DOWN, (16, d)), (M.AD_UP, (d, 16)), (M.AD_CONS, (d, 16))):
            m.set_tensor(0, tid, nrm(*shape))
        u = rng.uniform(0.9, 0.999, d * s)
        m.set_tensor(0, M.A_MAT, np.log(np.expm1(-np.log(u))).astype(np.float32))
        dirs = rng.standard_normal((cap, k))
        dirs /= np.linalg.norm(dirs, axis=1, keepdims=True)
        keys = (dirs * rng.uniform(0, 0.9, (cap, 1))).astype(np.float32)
        m.set_bank(0, keys, (keys.astype(np.float64) ** 2).sum(1).astype(np.float32), rng.standard_normal((cap, d)).astype(np.float32), cap)
        ids = np.random.default_rng(0).integers(1, v, 512)
        m.generate_greedy(ids, 8)  # warm-up
        m.reset_recurrent_state()
        t0 = time.perf_counter()
        m.prefill_batch([ids], [0], want_logits=False, want_greedy=True)
        t1 = time.perf_counter()
        m.reset_recurrent_state()
        toks = m.generate_greedy(ids, 200)
        t2 = time.perf_counter()
        out[name] = {"prefill_512_ms": (t1 - t0) * 1e3, "prefill_plus_200_tokens_ms": (t2 - t1) * 1e3,
                     "decode_ms_per_token": ((t2 - t1) - (t1 - t0)) * 1e3 / 200, "tokens": int(len(toks))}
        m.close()
    out["workload"] = "one block, vocab 8192, d 192, state 64, 512 slots; batch 1, 512-token prefill + 200 greedy tokens, host wall clock"
    return out


def run_extras(gpu, torch, peak_hbm):
    """Operator-alone workloads of BASELINE.json (N = 1 only)."""
    extra = {}
    stream = torch.cuda.current_stream()

    def timed(fn, steps, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    # configs[1]: scan operator alone, 64 x 4096 x 8192 fp32 (inputs 17 GB >> L2)
    lanes, t, stride = 64, 4096, 8192
    a = torch.empty(lanes, t, stride, device="cuda").uniform_(0.9, 0.999)
    b = torch.randn(lanes, t, stride, device="cuda")
    h = torch.empty_like(a)
    ms = timed(lambda: gpu.scan_states_dev(a, b, None, h, None, lanes, t, stride), 10)
    elems = lanes * t * stride
    gbs = elems * 12 / (ms / 1e3) / 1e9
    extra["scan_c2"] = {"workload": "associative scan alone, 64 x 4096 x 8192 fp32, all prefix states", "ms": ms,
                        "positions_per_s": lanes * t / (ms / 1e3),
                        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak_hbm, "unit": "GB/s", "frac": gbs / peak_hbm,
                                     "traffic": NCU_SCAN_TRAFFIC_BYTES_PER_ELEM * elems, "kernel": "scan_chunk_apply<4,4,false>"}}
    del a, b, h
    torch.cuda.empty_cache()
    extra["generate_c1"] = run_generate_c1(gpu)
    # configs[2]: retrieval operator, 512 slots, key/value dim 128, 64 x 4096 queries in the ball, tau 0.1
    rows, dk, dv, cap = 64 * 4096, 128, 128, 512
    g = torch.Generator(device="cuda").manual_seed(5)
    dirs = torch.randn(cap, dk, device="cuda", generator=g)
    keys = dirs / dirs.norm(dim=1, keepdim=True) * torch.rand(cap, 1, device="cuda", generator=g) * 0.9
    norm_sq = (keys.double() ** 2).sum(1).float()
    vals = torch.randn(cap, dv, device="cuda", generator=g)
    qd = torch.randn(rows, dk, device="cuda", generator=g)
    q = qd / qd.norm(dim=1, keepdim=True) * torch.rand(rows, 1, device="cuda", generator=g) * 0.9
    w = torch.zeros(rows, cap, device="cuda")
    m = torch.zeros(rows, dv, device="cuda")
    ref_sel = None
    for name, top_k, f32d, tcd in (("top8", 8, False, False), ("all_slots", 0, False, False), ("top8_f32_distance", 8, True, False),
                                   ("all_slots_f32_distance", 0, True, False), ("top8_tc_distance", 8, False, True),
                                   ("all_slots_tc_distance", 0, False, True)):
        ms = timed(lambda: gpu.memory_read_dev(q, keys, norm_sq, vals, rows, dk, dv, cap, cap, 0.1, m, top_k=top_k, weights=w,
                                               q_is_euclidean=False, f32_distance=f32d, tc_distance=tcd), 5, warm=2)
        byts = rows * (dk * 4 + dv * 4 + (64 if top_k else cap * 4))
        row = {"workload": "Poincare retrieval, 512 slots, key/value dim 128, 262144 queries, tau 0.1"
                           + (", distances from tensor-core inner products (three bf16 pieces per operand)" if tcd else
                              ", distances accumulated in fp32 (differences first)" if f32d else ", distances in f64 like the reference"),
               "ms": ms, "queries_per_s": rows / (ms / 1e3),
               "roofline": {"bound": "hbm", "achieved": byts / (ms / 1e3) / 1e9, "peak": peak_hbm, "unit": "GB/s",
                            "frac": byts / (ms / 1e3) / 1e9 / peak_hbm,
                            "limiter": "distance epilogue + softmax (the inner products run on the tensor cores)" if tcd else
                                       "FP32 FMA pipe (2 ops per key dimension per slot)" if f32d else "fp64 distance arithmetic"}}
        if top_k:
            sel = w != 0  # the selected slot sets of every query
            if not f32d and not tcd:
                ref_sel = sel.clone()
            elif ref_sel is not None:
                row["queries_with_the_f64_slot_set"] = float((sel == ref_sel).all(dim=1).float().mean().item())
        extra[f"retrieval_c3_{name}"] = row
    return extra


def run_b200(args):
    import torch
    import torch.distributed as dist

    import pssa_b200
    from pssa_b200 import _native as N

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    gpu = pssa_b200.B200Dispatch(local)
    stream = torch.cuda.current_stream()
    gpu.set_stream(stream)

    tensors, banks = synth_weights(1234)  # the same model on every rank (weights are replicated)
    model = pssa_b200.PSSAModel(gpu, tau_mem=0.1, streams=256, precision=N.PRECISION_BF16, **CFG)
    for (layer, tid), arr in tensors.items():
        model.set_tensor(layer, tid, arr)
    for l, (keys, norm_sq, values) in enumerate(banks):
        model.set_bank(l, keys, norm_sq, values, CFG["mem_capacity"])

    rng = np.random.default_rng(100 + rank)  # every rank prefills its own sequences
    ids_host = rng.integers(1, CFG["d_vocab"], (LANES, T)).astype(np.uint64)
    ids_dev = torch.from_numpy(ids_host.astype(np.int64)).to(torch.int32).cuda().contiguous()
    offsets = (np.arange(LANES) * T).astype(np.uint32)
    lengths = np.full(LANES, T, np.uint32)
    logits_dev = torch.empty(LANES, CFG["d_vocab"], device="cuda")

    def step():
        model.prefill_batch_dev(ids_dev, offsets, lengths, None, logits_dev, None)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # samples cover warm-up and the timed region
    warm = max(3, args.warmup)
    for _ in range(warm):
        step()
    barrier()
    launches0 = gpu.launch_count()
    gpu.profile_begin()
    t_begin = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_begin.record(stream)
    for _ in range(args.steps):
        step()
    t_end.record(stream)
    barrier()
    prof = gpu.profile_end()
    launches = gpu.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    tmax = torch.tensor([t_begin.elapsed_time(t_end)], device="cuda")
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    ms_per_step = float(tmax.item()) / args.steps
    value = world * LANES * T / (ms_per_step / 1e3)

    # ---- end to end: pinned host ids in, host logits out, through pssa_b200_model_prefill_batch
    import ctypes
    ids_pinned = torch.from_numpy(ids_host.view(np.int64)).pin_memory()
    logits_pinned = torch.empty(LANES, CFG["d_vocab"]).pin_memory()
    vp = ctypes.c_void_p

    def e2e_step():
        gpu._check(gpu._lib.pssa_b200_model_prefill_batch(model._h, vp(ids_pinned.data_ptr()), vp(offsets.ctypes.data),
                                                          vp(lengths.ctypes.data), None, LANES, vp(logits_pinned.data_ptr()), None))

    e2e_step()
    barrier()
    e2e_steps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    te = torch.tensor([(time.perf_counter() - t0) / e2e_steps], device="cuda")
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    finite = bool(torch.isfinite(logits_pinned).all())
    e2e = {"value": world * LANES * T / float(te.item()), "unit": "tok/s", "h2d_bytes_per_step": int(ids_host.nbytes),
           "d2h_bytes_per_step": int(logits_pinned.numel() * 4), "steps": e2e_steps,
           "note": f"pssa_b200_model_prefill_batch, host ids -> host last-token logits (finite: {finite})"}

    line = None
    if rank == 0:
        peak_hbm, peak_tf, peak_kind = measured_peaks()
        rows = LANES * T
        total_prof = sum(ms for _, ms in prof.values())
        kernels = []
        gemm_ms = sum(ms for name, (_, ms) in prof.items() if "gemm_bf16" in name)
        gemm_launches = sum(n for name, (n, _) in prof.items() if "gemm_bf16" in name)
        merged = {name: v for name, v in prof.items() if "gemm_bf16" not in name}
        merged["gemm_bf16_tcgen05_kernel (all tiles)"] = (gemm_launches, gemm_ms)
        for name, (n, ms) in sorted(merged.items(), key=lambda kv: -kv[1][1]):
            row = {"kernel": name, "launches_per_step": n / args.steps, "ms_per_step": ms / args.steps, "share": ms / total_prof}
            roof = kernel_roofline(name, n / args.steps, ms / args.steps, rows, peak_hbm, peak_tf,
                                   tc_distances=any("Poincare" in k for k in prof))
            if roof:
                row["roofline"] = roof
            if "gemm_bf16" in name:  # the tensor-core launches by epilogue family
                row["parts"] = {k[k.index("[") + 1:-1] if "[" in k else k: {"launches_per_step": v[0] / args.steps, "ms_per_step": v[1] / args.steps}
                                for k, v in prof.items() if "gemm_bf16" in k}
            kernels.append(row)
        top = kernels[0]
        roofline = dict(top.get("roofline") or {"bound": "hbm", "achieved": None, "peak": peak_hbm, "unit": "GB/s", "frac": None})
        roofline.setdefault("traffic", None)
        roofline.update({"kernel": top["kernel"], "kernel_ms_per_step": top["ms_per_step"], "share_of_step": top["share"],
                         "peak_kind": f"of {peak_kind}"})
        cpu = None
        parity = None
        if world == 1 and not args.no_cpu:
            import oracle as O
            threads = max(1, O.lib().pssa_oracle_hardware_threads())
            om = oracle_model(tensors, banks)
            sample_ids = cpu_sample_ids()
            om.prefill_lanes_timed(sample_ids[:threads, :2], threads)  # warm the clones' pages
            sec, ref_logits = om.prefill_lanes_timed(sample_ids, threads)
            cpu = {"value": sample_ids.size / sec, "unit": "tok/s", "cores": threads, "kind": "port",
                   "sample": f"{CPU_SAMPLE_LANES} sequences x {CPU_SAMPLE_T} tokens of the same model, token-serial prefill, "
                             f"{threads} host threads (C++ restatement of the reference CPU path)"}
            model.reset_recurrent_state()
            got, _ = model.prefill_batch([list(x) for x in sample_ids])
            parity = {"max_abs_logit_err_bf16_vs_cpu_fp32": float(np.max(np.abs(got - ref_logits))),
                      "logit_scale": float(np.max(np.abs(ref_logits))),
                      "greedy_agree": int(np.sum(np.argmax(got[:, 1:], 1) == np.argmax(ref_logits[:, 1:], 1))),
                      "lanes": CPU_SAMPLE_LANES}
        line = {
            "metric": "prefill_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sequences_per_gpu": LANES, "seq_len": T, "parallelism": f"dp{world} (independent lanes)",
                       "l2_policy": "each step streams 3.3 GB of activations and 0.6 GB of weights/banks through HBM, far larger "
                                    "than the 126 MB L2; no flush needed"},
            "roofline": roofline, "kernels": kernels, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches),
            "clocks": clocks, "parity": parity,
        }
    del logits_dev
    if world == 1 and rank == 0 and not args.no_extras:
        decode_extra = run_decode_extra(model, gpu, torch, measured_peaks()[0])
        model.close()
        torch.cuda.empty_cache()
        line["extra"] = run_extras(gpu, torch, measured_peaks()[0])
        line["extra"]["decode_c5"] = decode_extra
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    gpu.close()


def run_seqpar(args):
    """BASELINE's long-context configuration: 8 sequences x 65536 tokens of the same 12-block model, time-sharded over
    the N ranks (strong scaling: the job is fixed, a rank holds 8 x 65536/N token rows). One step = one sharded
    prefill from zero state, per-block all-gather of the shard maps over NCCL inside the timed region."""
    import torch
    import torch.distributed as dist

    import pssa_b200
    from pssa_b200 import _native as N
    from pssa_b200 import seqpar as SP

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus or world < 2:
        raise SystemExit("--workload seqpar_c5 needs --gpus N >= 2 under torch.distributed.run")
    lanes, t_full = 8, args.seq_len
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    gpu = pssa_b200.B200Dispatch(local)
    stream = torch.cuda.current_stream()
    gpu.set_stream(stream)
    tensors, banks = synth_weights(1234)
    model = pssa_b200.PSSAModel(gpu, tau_mem=0.1, streams=lanes, precision=N.PRECISION_BF16, **CFG)
    for (layer, tid), arr in tensors.items():
        model.set_tensor(layer, tid, arr)
    for l, (keys, norm_sq, values) in enumerate(banks):
        model.set_bank(l, keys, norm_sq, values, CFG["mem_capacity"])
    rows_rank = lanes * ((t_full + world - 1) // world)
    model.set_max_rows(rows_rank)
    sp = SP.SequenceParallelPrefill(model, max_lanes=lanes)
    prompts = np.random.default_rng(100).integers(1, CFG["d_vocab"], (lanes, t_full))  # the same job on every rank
    ids, offsets, lengths = SP.pack_shard(list(prompts), world, rank)
    ids_dev = torch.from_numpy(ids.astype(np.int64)).to(torch.int32).cuda()
    logits_dev = torch.empty(lanes, CFG["d_vocab"], device="cuda")

    def step():
        model.reset_recurrent_state()
        model.prefill_batch_dev(ids_dev, offsets, lengths, None, logits_dev, None)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    warm = max(3, args.warmup)
    for _ in range(warm):
        step()
    barrier()
    gpu.profile_begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    prof = gpu.profile_end()
    tmax = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    ms = float(tmax.item()) / args.steps
    if rank == 0:
        total = sum(v for _, v in prof.values())
        print(json.dumps({
            "metric": "prefill_tokens_per_s", "value": lanes * t_full / (ms / 1e3), "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"seqpar_c5: 12-block PSSA, {lanes} sequences x {t_full} tokens time-sharded over {world} GPUs "
                                   f"({rows_rank} token rows per GPU), per-block NCCL all-gather of the shard maps"},
            "kernels": [{"kernel": k, "ms_per_step": v / args.steps, "share": v / total}
                        for k, (_, v) in sorted(prof.items(), key=lambda kv: -kv[1][1])],
            "exchange_bytes_per_rank_per_block": lanes * (CFG["d_latent"] + CFG["d_latent"] * CFG["d_state"]) * 4,
        }))
    sp.close()
    dist.destroy_process_group()
    gpu.close()


def main():
    global LANES
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the operator-alone extras (N = 1)")
    ap.add_argument("--lanes", type=int, default=LANES,
                    help="sequences per GPU; anything but the default is a reduced case for profiler captures, not the benchmark")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline and parity sample (profiler captures)")
    ap.add_argument("--workload", default="prefill_c4", choices=["prefill_c4", "seqpar_c5"],
                    help="prefill_c4 is the benchmark; seqpar_c5 is the long-context time-sharded prefill (N >= 2)")
    ap.add_argument("--seq-len", type=int, default=65536, help="sequence length of the seqpar_c5 workload")
    args = ap.parse_args()
    if args.lanes != LANES:
        global WORKLOAD
        WORKLOAD = WORKLOAD.replace(f"{LANES} sequences", f"{args.lanes} sequences (REDUCED CASE, not the benchmark)")
        LANES = args.lanes
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "seqpar_c5":
        run_seqpar(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
