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

At N > 1 the line also carries, under `extra`, BASELINE.json's long-context configuration run on the same N GPUs after
the timed region: `seqpar_c5` (8 sequences x 65536 tokens, time-sharded over the ranks, strong scaling) and `decode_c5`
(256 concurrent streams x 256 greedy tokens, streams sharded over the ranks), each with its own device-timed
ms per step, tokens per second and a comparison with the same job on one GPU.

`--impl reference` times the CPU restatement of the reference's token-serial prefill (oracle/) on a bounded sample of
the same workload with the reference's own protocol (examples/inference_prefill_bench.rs:10,141-182): one warm-up, then
the median over the timed rounds, on all host threads (the line's value) and on one thread.

`--workload scan_c2` runs the scan operator alone (BASELINE.json configs[1]; `--lanes` scales it down for a profiler
capture); `--workload seqpar_c5` runs the time-sharded prefill alone.
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
CPU_ROUNDS = 7          # timed rounds of the CPU baseline after one warm-up round (median reported)
PARITY_T = T            # the parity leg compares logits after this many tokens: the benchmark's own sequence length
CPU_SAMPLE = (f"{CPU_SAMPLE_LANES} sequences x {CPU_SAMPLE_T} tokens of the same 12-block model per round, token-serial "
              "prefill_inference of the C++ restatement of the reference CPU path, one lane per host thread; one warm-up "
              "round, median of the timed rounds; single-thread figure: 1 sequence x 16 tokens per round")
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


def bench_config(world: int):
    """The `config` object of the JSON line; both arms print the same one."""
    return {"workload": WORKLOAD, "sequences_per_gpu": LANES, "seq_len": T, "parallelism": f"dp{world} (independent lanes)",
            "l2_policy": "each step streams 3.3 GB of activations and 0.6 GB of weights/banks through HBM, far larger "
                         "than the 126 MB L2; no flush needed",
            "cpu_sample": CPU_SAMPLE}


def cpu_rounds(om, ids, threads, rounds, warm=1):
    """The reference's CPU timing protocol (examples/inference_prefill_bench.rs:10,141-182): `warm` untimed rounds,
    then `rounds` timed ones; returns (seconds per round list, last logits)."""
    logits = None
    for _ in range(warm):
        om.prefill_lanes_timed(ids, threads)
    secs = []
    for _ in range(rounds):
        sec, logits = om.prefill_lanes_timed(ids, threads)
        secs.append(sec)
    return secs, logits


def cpu_baseline_object(om, threads, rounds):
    """All-cores and single-thread tokens per second of the CPU restatement on the bounded sample."""
    ids = cpu_sample_ids()
    secs, _ = cpu_rounds(om, ids, threads, rounds)
    all_cores = ids.size / statistics.median(secs)
    secs1, _ = cpu_rounds(om, ids[:1], 1, rounds)
    single = ids[:1].size / statistics.median(secs1)
    return {"value": all_cores, "unit": "tok/s", "cores": threads, "kind": "port", "sample": CPU_SAMPLE, "rounds": rounds,
            "ms_per_round_median": 1e3 * statistics.median(secs), "ms_per_round_min": 1e3 * min(secs),
            "single_thread": {"value": single, "unit": "tok/s", "cores": 1, "rounds": rounds,
                              "ms_per_round_median": 1e3 * statistics.median(secs1)}}, secs


def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import oracle as O
    threads = max(1, O.lib().pssa_oracle_hardware_threads())
    tensors, banks = synth_weights(1234)
    om = oracle_model(tensors, banks)
    ids = cpu_sample_ids()
    rounds = args.steps  # the reference's own protocol uses 7; the driver's --steps decides here
    secs, _ = cpu_rounds(om, ids, threads, rounds, warm=max(1, args.warmup))
    ms = 1e3 * statistics.median(secs)
    value = ids.size / (ms / 1e3)
    secs1, _ = cpu_rounds(om, ids[:1], 1, CPU_ROUNDS)
    single = ids[:1].size / statistics.median(secs1)
    print(json.dumps({
        "impl": "reference", "metric": "prefill_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": bench_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port", "sample": CPU_SAMPLE,
                         "rounds": rounds, "statistic": "median over the timed rounds (one step = one round of the sample)",
                         "ms_per_round_min": 1e3 * min(secs),
                         "single_thread": {"value": single, "unit": "tok/s", "cores": 1, "rounds": CPU_ROUNDS}},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def kernel_roofline(name, launches, ms, rows, peak_hbm, peak_tf, tc_distances=False):
    """Algorithmic work of one launch of `name` on `rows` token rows of the C4 block -> achieved rate."""
    d, s, k, cap = CFG["d_latent"], CFG["d_state"], CFG["d_mem_key"], CFG["mem_capacity"]
    per = ms / launches / 1e3
    if "ssm_fused" in name:
        # algorithmic bytes per token row: read delta, x (4d each), B, C (4s each), write y (4d) = (3d + 2s) * 4 = 9728 B at
        # d 768 / s 64, plus every lane's carry in and out once. The bf16 copy of y the kernel also writes (2d per row) is
        # a by-product for the next GEMM and is not counted.
        byts = rows * (3 * d + 2 * s) * 4 + LANES * 2 * d * s * 4
        exps = rows * d * s
        return {"bound": "hbm", "achieved": byts / per / 1e9, "peak": peak_hbm, "unit": "GB/s",
                "frac": byts / per / 1e9 / peak_hbm, "traffic": NCU_SSM_TRAFFIC_BYTES_PER_ROW * rows,
                "bytes_counted": "(3d + 2s) * 4 = 9728 B per token row + 2 * d * s * 4 B of carry per lane",
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


def decode_bytes(streams):
    """Algorithmic HBM bytes of one decode step: every stream's recurrent state in and out, bf16 weights once."""
    d, s, v, k = CFG["d_latent"], CFG["d_state"], CFG["d_vocab"], CFG["d_mem_key"]
    state_bytes = streams * CFG["depth"] * d * s * 4 * 2
    weight_elems = v * d + CFG["depth"] * (2 * d * d + 2 * s * d + 2 * k * d + d * d + 4 * d * d + 32 * d)  # head + blocks
    return state_bytes + weight_elems * 2


def run_decode_c5(model, gpu, torch, dist, world, rank, peak_hbm, streams_total=256, steps=256, check=True):
    """The decode half of BASELINE's long-context configuration: 256 concurrent streams x 256 greedy tokens on the
    12-block model, streams sharded over the ranks (stream i lives on rank i mod N, like independent lanes). 16-token
    prompts, then `steps` timed steps of one token per stream through pssa_b200_model_decode_step: ids from the host
    in, greedy ids back to the host every step (they are the next step's input), so the timed loop IS the end-to-end
    path. Timed per rank with CUDA events around the loop, max over ranks."""
    mine = np.arange(rank, streams_total, world)
    n = len(mine)
    rng = np.random.default_rng(7)
    prompts = [rng.integers(1, CFG["d_vocab"], 16) for _ in range(streams_total)]
    stream = torch.cuda.current_stream()

    def generate(which, n_steps, collective):
        slots = np.arange(len(which), dtype=np.uint32)
        for sl in slots:
            model.reset_recurrent_state(int(sl))
        _, ids = model.prefill_batch([prompts[i] for i in which], slots, want_logits=False, want_greedy=True)
        for _ in range(4):
            ids = model.decode_step(ids, slots, want_logits=False, want_greedy=True)
        if world > 1 and collective:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = gpu.launch_count()
        e0.record(stream)
        out = []
        for _ in range(n_steps):
            ids = model.decode_step(ids, slots, want_logits=False, want_greedy=True)
            out.append(ids)
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n_steps, np.stack(out), (gpu.launch_count() - launches0) / n_steps

    ms, tokens, launches = generate(mine, steps, True)
    t = torch.tensor([ms], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    out = {"workload": f"greedy decode, {streams_total} streams x {steps} tokens, 12-block model, streams sharded over {world} GPU(s) "
                       f"({n} per GPU), ids host -> device and greedy ids device -> host every step",
           "ms_per_step": ms, "tokens_per_s": streams_total / (ms / 1e3), "steps": steps, "scaling": "strong",
           "gpu_launches_per_step": launches,
           "e2e": {"value": streams_total / (ms / 1e3), "unit": "tok/s", "h2d_bytes_per_step": int(n * 8), "d2h_bytes_per_step": int(n * 8),
                   "note": "the timed loop already crosses the host every step"},
           "roofline": {"bound": "hbm", "achieved": decode_bytes(n) / (ms / 1e3) / 1e9, "peak": peak_hbm, "unit": "GB/s",
                        "frac": decode_bytes(n) / (ms / 1e3) / 1e9 / peak_hbm,
                        "note": "algorithmic bytes per GPU per step = its streams' recurrent state in and out + bf16 weights once"}}
    if world > 1 and check and rank == 0:
        # the same streams decoded alone on this GPU inside the full 256-stream batch: token sequences must be equal
        _, all_tokens, _ = generate(np.arange(streams_total), min(steps, 32), False)
        out["greedy_tokens_equal_single_gpu_batch"] = bool(np.array_equal(all_tokens[:, mine], tokens[: all_tokens.shape[0]]))
        out["compared_steps"] = int(all_tokens.shape[0])
    if world > 1:
        dist.barrier()
    if world == 1:
        # the same step captured as a CUDA graph, ids fed back on the device: no host round trip per token
        ids_dev = torch.tensor(tokens[-1].astype(np.int32), device="cuda", dtype=torch.int32)
        graph = model.capture_greedy_decode_graph(ids_dev)
        for _ in range(4):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(64):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        graph_ms = e0.elapsed_time(e1) / 64
        out["cuda_graph"] = {"ms_per_step": graph_ms, "tokens_per_s": streams_total / (graph_ms / 1e3),
                             "roofline_frac": decode_bytes(n) / (graph_ms / 1e3) / 1e9 / peak_hbm,
                             "note": "one captured greedy step replayed; ids stay on the device (CUDA events)"}
    gpu.poll_status()
    return out


def run_seqpar_c5(model, gpu, torch, dist, world, rank, steps=3, check=True):
    """The prefill half of BASELINE's long-context configuration on the N GPUs of this run: 8 sequences x 65536 tokens,
    every sequence cut into N contiguous time shards (strong scaling: the job is fixed). One step = one sharded prefill
    from zero state with the per-block all-gather of the shard maps over NCCL inside the timed region. N = 1 runs the
    same job on one GPU (time chunks inside the GPU, no exchange)."""
    from pssa_b200 import seqpar as SP
    lanes, t_full = 8, 65536
    rows_rank = lanes * ((t_full + world - 1) // world)
    model.set_max_rows(rows_rank)
    stream = torch.cuda.current_stream()
    sp = SP.SequenceParallelPrefill(model, max_lanes=lanes) if world > 1 else None
    prompts = np.random.default_rng(100).integers(1, CFG["d_vocab"], (lanes, t_full))  # the same job on every rank
    ids, offsets, lengths = SP.pack_shard(list(prompts), world, rank)
    ids_dev = torch.from_numpy(ids.astype(np.int64)).to(torch.int32).cuda()
    logits_dev = torch.zeros(lanes, CFG["d_vocab"], device="cuda")
    slots = np.arange(lanes, dtype=np.uint32)

    def step():
        for sl in range(lanes):
            model.reset_recurrent_state(sl)
        model.prefill_batch_dev(ids_dev, offsets, lengths, slots, logits_dev, None)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(2):
        step()
    barrier()
    gpu.profile_begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    barrier()
    prof = gpu.profile_end()
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / steps
    total = sum(v for _, v in prof.values()) or 1.0
    rec = (CFG["d_latent"] + CFG["d_latent"] * CFG["d_state"]) * 4
    out = {"workload": f"seqpar_c5: 12-block PSSA, {lanes} sequences x {t_full} tokens time-sharded over {world} GPU(s) "
                       f"({rows_rank} token rows per GPU)" + (", per-block NCCL all-gather of the shard maps" if world > 1 else ""),
           "ms_per_step": ms, "tokens_per_s": lanes * t_full / (ms / 1e3), "steps": steps, "scaling": "strong",
           "kernels": [{"kernel": k, "ms_per_step": v / steps, "share": v / total}
                       for k, (_, v) in sorted(prof.items(), key=lambda kv: -kv[1][1])[:6]],
           "exchange_bytes_per_record": rec}
    if world > 1:
        # every rank ends with the same final state; the logits of a lane are those of the rank that owns its last token
        gathered = torch.empty(world, lanes, CFG["d_vocab"], device="cuda")
        dist.all_gather_into_tensor(gathered, logits_dev)
        sharded = SP.select_owner_rows(gathered.cpu().numpy(), [t_full] * lanes, world)
        sp.close()
        if check:
            # parity with one GPU: rank 0 prefills the first sequence whole (time chunks inside the GPU, no exchange)
            if rank == 0:
                model.set_max_rows(t_full)
                model.reset_recurrent_state(0)
                one = torch.zeros(1, CFG["d_vocab"], device="cuda")
                ids0 = torch.from_numpy(prompts[0].astype(np.int64)).to(torch.int32).cuda()
                model.prefill_batch_dev(ids0, np.zeros(1, np.uint32), np.array([t_full], np.uint32), np.zeros(1, np.uint32), one, None)
                torch.cuda.synchronize()
                ref = one.cpu().numpy()[0]
                out["parity_vs_single_gpu"] = {"sequence": 0, "tokens": t_full,
                                               "max_abs_logit_diff": float(np.max(np.abs(sharded[0] - ref))),
                                               "logit_scale": float(np.max(np.abs(ref))),
                                               "greedy_equal": bool(np.argmax(sharded[0][1:]) == np.argmax(ref[1:]))}
            dist.barrier()
    model.set_max_rows(65536)
    gpu.poll_status()
    return out


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
    # the headline form of configs[2]: exact top-8 in ONE kernel with compact results (8 slots + 8 weights per query)
    slots8 = torch.zeros(rows, 8, dtype=torch.int32, device="cuda")
    w8 = torch.zeros(rows, 8, device="cuda")
    handed = torch.zeros(1, dtype=torch.int32, device="cuda")

    def fused_top8(values=vals):
        gpu.memory_read_topk_dev(q, keys, norm_sq, values, rows, dk, dv, cap, cap, 0.1, 8, m, slots8, w8, handed_over=handed,
                                 q_is_euclidean=False)

    for name, top_k, f32d, tcd in (("top8_separate_f64_kernels", 8, False, False), ("all_slots", 0, False, False), ("top8_f32_distance", 8, True, False),
                                   ("all_slots_f32_distance", 0, True, False), ("top8_tc_distance", 8, False, True),
                                   ("all_slots_tc_distance", 0, False, True), ("top8", 8, False, False)):
        one_kernel = name == "top8"
        if one_kernel:
            ms = timed(fused_top8, 10, warm=3)
        else:
            ms = timed(lambda: gpu.memory_read_dev(q, keys, norm_sq, vals, rows, dk, dv, cap, cap, 0.1, m, top_k=top_k, weights=w,
                                                   q_is_euclidean=False, f32_distance=f32d, tc_distance=tcd, no_fused=True), 5, warm=2)
        byts = rows * (dk * 4 + dv * 4 + (64 if top_k else cap * 4))
        row = {"workload": "Poincare retrieval, 512 slots, key/value dim 128, 262144 queries, tau 0.1"
                           + (", exact top-8 in one kernel: tensor-core pre-filter in TMEM, f64 re-scoring of the candidates, "
                              "(distance bits, slot) selection, softmax and value read; compact results" if one_kernel else
                              ", distances from tensor-core inner products (three bf16 pieces per operand)" if tcd else
                              ", distances accumulated in fp32 (differences first)" if f32d else ", distances in f64 like the reference"),
               "ms": ms, "queries_per_s": rows / (ms / 1e3),
               "roofline": {"bound": "hbm", "achieved": byts / (ms / 1e3) / 1e9, "peak": peak_hbm, "unit": "GB/s",
                            "frac": byts / (ms / 1e3) / 1e9 / peak_hbm,
                            "limiter": "tensor-core pre-filter + per-row sweeps of the accumulator + L2 reads of the candidates' keys and values" if one_kernel else
                                       "distance epilogue + softmax (the inner products run on the tensor cores)" if tcd else
                                       "FP32 FMA pipe (2 ops per key dimension per slot)" if f32d else "fp64 distance arithmetic"}}
        if one_kernel:
            sel = torch.zeros(rows, cap, dtype=torch.bool, device="cuda")
            sel.scatter_(1, slots8.long(), True)
            row["queries_with_the_f64_slot_set"] = float((sel == ref_sel).all(dim=1).float().mean().item())
            row["rows_handed_to_the_exact_stage"] = int(handed.item())
            del sel
        elif top_k:
            sel = w != 0  # the selected slot sets of every query
            if not f32d and not tcd:
                ref_sel = sel.clone()
            elif ref_sel is not None:
                row["queries_with_the_f64_slot_set"] = float((sel == ref_sel).all(dim=1).float().mean().item())
        extra[f"retrieval_c3_{name}"] = row
    # configs[2] as written: the top-8 read of all 64 x 4096 queries PLUS one gated rank-1 plastic write per sequence to
    # the winning (nearest) slot of the sequence's last query, 64 ordered writes in one launch (the gate is history
    # dependent). The rank-1 write is not a reference code path; its parity is against the restatement (tests/test_write_gpu.py).
    n_seq = 64
    last = torch.arange(n_seq, device="cuda") * (rows // n_seq) + (rows // n_seq - 1)
    vals_rw = vals.clone()
    conf = torch.ones(cap, device="cuda")
    seen = torch.zeros(cap, dtype=torch.int64, device="cuda")
    meta = torch.tensor([cap, 0], dtype=torch.int64, device="cuda")
    target = torch.randn(n_seq, dv, device="cuda", generator=g)
    surprise = torch.full((n_seq,), 50.0, device="cuda")  # damage = 0.08 * 50 * gain: a slot last seen long ago is overwritten
    steps_t = torch.arange(1, n_seq + 1, dtype=torch.int64, device="cuda") * 4096
    slots_out = torch.zeros(n_seq, dtype=torch.int64, device="cuda")
    key_rows = q[last].contiguous()

    def write_only():
        # the winning slot = the selected slot with the largest weight (the nearest) of the read just done
        win = slots8[last].gather(1, w8[last].argmax(dim=1, keepdim=True)).squeeze(1).to(torch.int32)
        gpu.bank_insert_protected_dev(keys, norm_sq, vals_rw, conf, seen, meta, cap, dk, dv, key_rows, target, surprise, steps_t,
                                      n_seq, slots_out, win, 0.1)

    def read_write():
        fused_top8(vals_rw)
        write_only()

    read_write()
    torch.cuda.synchronize()
    accepted = int((slots_out >= 0).sum().item())  # first round: every slot was last seen at step 0
    ms_rw = timed(read_write, 5, warm=2)
    ms_w = timed(write_only, 20, warm=2)
    byts = rows * (dk * 4 + dv * 4 + 64) + n_seq * (dk + dv + 3) * 4
    extra["retrieval_c3_top8_read_plus_write"] = {
        "workload": "Poincare retrieval as BASELINE configs[2] words it: exact top-8 read of 262144 queries (one kernel) plus 64 "
                    "refractory-gated rank-1 writes to the winning slots (one per sequence, ordered, one launch)",
        "ms": ms_rw, "write_only_ms": ms_w, "writes": n_seq, "writes_accepted_first_round": accepted, "queries_per_s": rows / (ms_rw / 1e3),
        "roofline": {"bound": "hbm", "achieved": byts / (ms_rw / 1e3) / 1e9, "peak": peak_hbm, "unit": "GB/s",
                     "frac": byts / (ms_rw / 1e3) / 1e9 / peak_hbm,
                     "limiter": "the read dominates; the write is one CTA walking 64 gates in order (latency bound, (k + d + 3) * 4 B each)"}}
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
            cpu, _ = cpu_baseline_object(om, threads, CPU_ROUNDS)
            # parity at the benchmark's own sequence length: the first lanes of the timed batch, all PARITY_T tokens,
            # one lane per host thread through the token-serial CPU path (about a minute)
            n_par = max(1, min(8, threads, LANES))
            par_ids = ids_host[:n_par, :PARITY_T]
            t0 = time.perf_counter()
            _, ref_logits = om.prefill_lanes_timed(par_ids, n_par)
            cpu_sec = time.perf_counter() - t0
            model.reset_recurrent_state()
            got, _ = model.prefill_batch([list(x) for x in par_ids])
            err = np.max(np.abs(got - ref_logits), axis=1)
            top2 = np.sort(ref_logits[:, 1:], axis=1)[:, -2:]
            gap = top2[:, 1] - top2[:, 0]
            agree = np.argmax(got[:, 1:], 1) == np.argmax(ref_logits[:, 1:], 1)
            decisive = gap > 2 * err
            parity = {"tokens": int(PARITY_T), "lanes": int(n_par), "blocks": CFG["depth"],
                      "max_abs_logit_err_bf16_vs_cpu_fp32": float(err.max()), "logit_scale": float(np.max(np.abs(ref_logits))),
                      "tolerance_max_abs": 2e-2, "within_tolerance": bool(err.max() <= 2e-2),
                      "greedy_agree": int(agree.sum()), "min_top2_gap": float(gap.min()),
                      "lanes_with_decisive_gap": int(decisive.sum()), "greedy_agree_where_decisive": int((agree & decisive).sum()),
                      "cpu_seconds": cpu_sec}
        line = {
            "metric": "prefill_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": bench_config(world),
            "roofline": roofline, "kernels": kernels, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches),
            "clocks": clocks, "parity": parity,
        }
    del logits_dev
    if not args.no_extras:
        # BASELINE's long-context configuration on the same GPUs (every rank takes part; rank 0 reports)
        peak_hbm = measured_peaks()[0]
        dd = dist if world > 1 else None
        decode_extra = run_decode_c5(model, gpu, torch, dd, world, rank, peak_hbm)
        seqpar_extra = run_seqpar_c5(model, gpu, torch, dd, world, rank)
        model.close()
        torch.cuda.empty_cache()
        if rank == 0:
            line["extra"] = run_extras(gpu, torch, peak_hbm) if world == 1 else {}
            line["extra"]["decode_c5"] = decode_extra
            line["extra"]["seqpar_c5"] = seqpar_extra
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


def run_scan_c2(args):
    """BASELINE configs[1] alone: all prefix states of h_t = a_t h_{t-1} + b_t over [lanes, 4096, 8192] fp32 (`--lanes`
    below 64 is a reduced case for profiler captures; 8 lanes = 3.2 GB on the device, still far above the L2)."""
    import torch

    import pssa_b200
    lanes = args.lanes if args.lanes != LANES else 64
    t, stride = 4096, 8192
    torch.cuda.set_device(0)
    gpu = pssa_b200.B200Dispatch(0)
    stream = torch.cuda.current_stream()
    gpu.set_stream(stream)
    a = torch.empty(lanes, t, stride, device="cuda").uniform_(0.9, 0.999)
    b = torch.randn(lanes, t, stride, device="cuda")
    h = torch.empty_like(a)
    for _ in range(max(3, args.warmup)):
        gpu.scan_states_dev(a, b, None, h, None, lanes, t, stride)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        gpu.scan_states_dev(a, b, None, h, None, lanes, t, stride)
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    peak_hbm, _, kind = measured_peaks()
    elems = lanes * t * stride
    gbs = elems * 12 / (ms / 1e3) / 1e9
    print(json.dumps({"metric": "scan_positions_per_s", "value": lanes * t / (ms / 1e3), "unit": "positions/s", "n_gpus": 1,
                      "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
                      "dtype": "f32", "data": "synthetic",
                      "config": {"workload": f"scan_c2: associative scan alone, {lanes} x {t} x {stride} fp32, all prefix states"
                                             + ("" if lanes == 64 else " (REDUCED CASE, not the benchmark)")},
                      "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak_hbm, "unit": "GB/s", "frac": gbs / peak_hbm,
                                   "traffic": NCU_SCAN_TRAFFIC_BYTES_PER_ELEM * elems, "peak_kind": f"of {kind}"},
                      "gpu_launches": int(gpu.launch_count())}))
    gpu.close()


def run_retrieval_c3(args):
    """BASELINE configs[2]'s read alone: the exact top-8 Poincare read of 64 x 4096 queries against one 512-slot bank in
    one kernel (the same inputs as the `retrieval_c3_top8` entry of the benchmark's extras); for profiler captures."""
    import torch

    import pssa_b200
    torch.cuda.set_device(0)
    gpu = pssa_b200.B200Dispatch(0)
    stream = torch.cuda.current_stream()
    gpu.set_stream(stream)
    rows, dk, dv, cap = 64 * 4096, 128, 128, 512
    g = torch.Generator(device="cuda").manual_seed(5)
    dirs = torch.randn(cap, dk, device="cuda", generator=g)
    keys = dirs / dirs.norm(dim=1, keepdim=True) * torch.rand(cap, 1, device="cuda", generator=g) * 0.9
    norm_sq = (keys.double() ** 2).sum(1).float()
    vals = torch.randn(cap, dv, device="cuda", generator=g)
    qd = torch.randn(rows, dk, device="cuda", generator=g)
    q = qd / qd.norm(dim=1, keepdim=True) * torch.rand(rows, 1, device="cuda", generator=g) * 0.9
    m = torch.zeros(rows, dv, device="cuda")
    slots8 = torch.zeros(rows, 8, dtype=torch.int32, device="cuda")
    w8 = torch.zeros(rows, 8, device="cuda")
    handed = torch.zeros(1, dtype=torch.int32, device="cuda")

    def read():
        gpu.memory_read_topk_dev(q, keys, norm_sq, vals, rows, dk, dv, cap, cap, 0.1, 8, m, slots8, w8, handed_over=handed,
                                 q_is_euclidean=False)

    for _ in range(max(3, args.warmup)):
        read()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        read()
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    peak_hbm, _, kind = measured_peaks()
    byts = rows * (dk * 4 + dv * 4 + 64)
    print(json.dumps({"metric": "retrieval_queries_per_s", "value": rows / (ms / 1e3), "unit": "queries/s", "n_gpus": 1,
                      "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
                      "dtype": "f64 distances of the candidates, bf16 x 3 pre-filter", "data": "synthetic",
                      "config": {"workload": "retrieval_c3: exact top-8 Poincare read, 512 slots, key/value dim 128, 262144 queries, one kernel"},
                      "roofline": {"bound": "hbm", "achieved": byts / (ms / 1e3) / 1e9, "peak": peak_hbm, "unit": "GB/s",
                                   "frac": byts / (ms / 1e3) / 1e9 / peak_hbm, "peak_kind": f"of {kind}"},
                      "rows_handed_to_the_exact_stage": int(handed.item()), "gpu_launches": int(gpu.launch_count())}))
    gpu.close()


def run_decode(args):
    """The decode half of BASELINE's long-context configuration alone on one GPU (256 streams, `--steps` greedy tokens
    each after 16-token prompts); the same leg as `extra.decode_c5` of the benchmark line, for profiler captures."""
    import torch

    import pssa_b200
    from pssa_b200 import _native as N
    torch.cuda.set_device(0)
    gpu = pssa_b200.B200Dispatch(0)
    gpu.set_stream(torch.cuda.current_stream())
    tensors, banks = synth_weights(1234)
    model = pssa_b200.PSSAModel(gpu, tau_mem=0.1, streams=256, precision=N.PRECISION_BF16, **CFG)
    for (layer, tid), arr in tensors.items():
        model.set_tensor(layer, tid, arr)
    for l, (keys, norm_sq, values) in enumerate(banks):
        model.set_bank(l, keys, norm_sq, values, CFG["mem_capacity"])
    peak_hbm, _, kind = measured_peaks()
    leg = run_decode_c5(model, gpu, torch, None, 1, 0, peak_hbm, steps=args.steps)
    print(json.dumps({"metric": "decode_tokens_per_s", "value": leg["tokens_per_s"], "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
                      "warmup": 4, "ms_per_step": leg["ms_per_step"], "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": "decode_c5: " + leg["workload"]}, "roofline": dict(leg["roofline"], peak_kind=f"of {kind}"),
                      "e2e": leg["e2e"], "cuda_graph": leg.get("cuda_graph"), "gpu_launches": int(leg["gpu_launches_per_step"] * args.steps)}))
    model.close()
    gpu.close()


def run_gemm_plain(args):
    """One plain bf16 tensor-core product alone (8192 x 8192 x 8192, fp32 out), the shape the GEMM kernel's own ceiling
    is quoted on; runs as CTA pairs. For profiler captures and for comparing against MEASURED_PEAKS.json's cuBLAS rate."""
    import torch

    import pssa_b200
    torch.cuda.set_device(0)
    gpu = pssa_b200.B200Dispatch(0)
    stream = torch.cuda.current_stream()
    gpu.set_stream(stream)
    m = n = k = 8192
    x = torch.randn(m, k, device="cuda")
    w = torch.randn(n, k, device="cuda") * 0.02
    out = torch.empty(m, n, device="cuda")
    for _ in range(max(3, args.warmup)):
        gpu.gemm_xwt_dev(x, w, m, n, k, out)
    torch.cuda.synchronize()
    gpu.profile_begin()  # the entry point also rounds both operands to bf16 (two small kernels): time the product alone
    for _ in range(args.steps):
        gpu.gemm_xwt_dev(x, w, m, n, k, out)
    torch.cuda.synchronize()
    prof = gpu.profile_end()
    launches, ms = next(v for name, v in prof.items() if name.startswith("gemm_bf16_tcgen05_kernel"))
    ms /= launches
    _, peak_tf, kind = measured_peaks()
    tf = 2.0 * m * n * k / (ms / 1e3) / 1e12
    print(json.dumps({"metric": "gemm_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
                      "ms_per_step": ms, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": "gemm_plain: 8192 x 8192 x 8192 bf16 operands, fp32 accumulate and output, clusters of two CTAs on 256 x 256 tiles"},
                      "roofline": {"bound": "tensor", "achieved": tf, "peak": peak_tf, "unit": "TFLOP/s", "frac": tf / peak_tf,
                                   "peak_kind": f"of {kind} (sustained cuBLAS bf16)"},
                      "gpu_launches": int(gpu.launch_count())}))
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
    ap.add_argument("--workload", default="prefill_c4", choices=["prefill_c4", "seqpar_c5", "scan_c2", "retrieval_c3", "decode_c5", "gemm_plain"],
                    help="prefill_c4 is the benchmark; seqpar_c5 is the long-context time-sharded prefill (N >= 2); scan_c2 is "
                         "the scan operator alone; retrieval_c3 is the one-kernel top-8 memory read alone; decode_c5 is the 256-stream greedy decode alone; gemm_plain is one 8192^3 product")
    ap.add_argument("--seq-len", type=int, default=65536, help="sequence length of the seqpar_c5 workload")
    args = ap.parse_args()
    if args.workload == "scan_c2":
        return run_scan_c2(args)
    if args.workload == "retrieval_c3":
        return run_retrieval_c3(args)
    if args.workload == "decode_c5":
        return run_decode(args)
    if args.workload == "gemm_plain":
        return run_gemm_plain(args)
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
