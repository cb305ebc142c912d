"""Benchmark of the HashAttention sparse-decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload config1|config2|config3]
    python bench.py --impl reference ...        # the CPU arm: the reference's algorithm on host cores

A step is one decode step of one attention layer over one batch: hash-encode the new query and
key (+ cache append), Hamming-score the key-hash cache, budget-select, sparse GQA attention.
Consecutive steps run on different layer instances (own K/V/hash cache, own hash weights), as
the layers of a model do, so every step's inputs come from HBM and not from L2; the instances
of one "token" are replayed as one CUDA graph, the way a serving loop launches a decode step.

Prints ONE JSON line (rank 0). `value` is algorithmic HBM bytes per second over all GPUs with
everything resident in HBM; `us_per_layer` is the same measurement as time; `e2e` is measured
through the public host-buffer call (H2D of q/k/v, step, D2H of the result, every step).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HQ, HKV, D = 32, 8, 128
WORKLOADS = {
    # name: description, batch, lengths, heavy budget, layer instances kept resident
    "config1": dict(desc="BASELINE configs[1]: B=1, S=32768, 32q/8kv heads, d=128, init 128 / recent 128 / heavy 1/32",
                    batch=1, lens=lambda: [32768], heavy=1.0 / 32, layers=16, index=1),
    "config2": dict(desc="BASELINE configs[2] decode part: B=32, S_b uniform in [16384,65536] (seeded), heavy 1/16, "
                         "shuffled 256-token pages", batch=32, lens=None, heavy=1.0 / 16, layers=2, index=2),
    "config3": dict(desc="BASELINE configs[3] on one GPU: B=4, S=131072, heavy 1/32",
                    batch=4, lens=lambda: [131072] * 4, heavy=1.0 / 32, layers=3, index=3),
}
INIT, RECENT = 128, 128
METRIC, UNIT = "sparse_decode_attn_hbm_gbs", "GB/s"

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu
# capture summarised in profiles/ (None until a capture of that workload exists)
NCU_TRAFFIC = {"config1": 17146880}  # sparse_gather_kernel, profiles/decode_kernels_config1_ncu_full.md


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def tensor_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    return 1590.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"


def workload_lens(name):
    w = WORKLOADS[name]
    if w["lens"] is not None:
        return w["lens"]()
    from hashattention_b200 import synthetic
    return synthetic.ragged_lengths(w["index"], w["batch"], 16384, 65536)


# --------------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "nvidia-smi not available"}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, sm_max, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); sm_max.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "no samples"}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(sm_max), "reasons": sorted(reasons),
                "power_w_max": max(power), "samples": len(sm)}


# --------------------------------------------------------------------------------------------
# CPU arm: the reference's algorithm (oracle port) on the host cores
# --------------------------------------------------------------------------------------------
def cpu_reference_run(workload: str, max_steps: int, warmup: int, budget_s: float):
    """Times oracle.decode_step (the restatement of the reference's forward: re-hash all keys,
    full sort, dense masked softmax) on host cores. Returns (seconds per step, steps run, threads,
    bytes per step, sample description)."""
    import torch
    import __graft_entry__ as entry
    entry.load_package()
    from hashattention_b200 import synthetic
    from oracle import hashattn_oracle as orc

    threads = len(os.sched_getaffinity(0))
    torch.set_num_threads(threads)
    w = WORKLOADS[workload]
    lens = workload_lens(workload)
    full_bytes = synthetic.algorithmic_bytes(lens, HQ, HKV, INIT, RECENT, w["heavy"])["total"]
    # a bounded sample: the first sequence of the batch, all heads; bytes scaled accordingly
    S = lens[0]
    sample_bytes = synthetic.algorithmic_bytes([S], HQ, HKV, INIT, RECENT, w["heavy"])["total"]
    usa = synthetic.make_usa(HQ, D, seed=0, bf16=True).float()
    g = torch.Generator().manual_seed(1000 + w["index"])
    q = torch.randn(1, HQ, D, generator=g).bfloat16().float()
    k = torch.randn(1, HKV, S, D, generator=g)
    k[..., list(synthetic.OUTLIER_CHANNELS)] *= synthetic.OUTLIER_SCALE
    k = k.bfloat16().float()
    v = torch.randn(1, HKV, S, D, generator=g).bfloat16().float()
    with torch.no_grad():
        t0 = time.perf_counter()
        orc.decode_step(usa, q, k, v, INIT, RECENT, w["heavy"])
        first = time.perf_counter() - t0
        n_warm = max(0, min(warmup, 3, int(budget_s * 0.2 / max(first, 1e-9))))
        for _ in range(n_warm):
            orc.decode_step(usa, q, k, v, INIT, RECENT, w["heavy"])
        n = max(1, min(max_steps, int(budget_s / max(first, 1e-9))))
        t0 = time.perf_counter()
        for _ in range(n):
            orc.decode_step(usa, q, k, v, INIT, RECENT, w["heavy"])
        per_step = (time.perf_counter() - t0) / n
    sample = (f"{n} steps of sequence 0 of {workload} (S={S}, all 32 heads, fp32 torch CPU ops in the reference's "
              f"structure: re-hash all keys, full sort, dense masked softmax)")
    # seconds per FULL step of the workload = sample time scaled by the byte ratio (sequences are independent)
    return per_step * full_bytes / sample_bytes, n, threads, full_bytes, sample


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    per_step, n, threads, nbytes, sample = cpu_reference_run(args.workload, args.steps, args.warmup, 60.0)
    value = nbytes / per_step / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "steps_run": n, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "us_per_layer": per_step * 1e6,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {WORKLOADS[args.workload]['desc']}"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    ha = entry.load_package()
    from hashattention_b200 import synthetic

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    w = WORKLOADS[args.workload]
    lens = workload_lens(args.workload)
    if args.batch:  # fewer sequences, or the workload's sequences repeated
        lens = (lens * ((args.batch + len(lens) - 1) // len(lens)))[:args.batch]
    B, L = len(lens), args.layers or w["layers"]
    budget = ha.Budget(INIT, w["heavy"], RECENT)
    nbytes = synthetic.algorithmic_bytes(lens, HQ, HKV, INIT, RECENT, w["heavy"])

    # ---- L layer instances, each with its own cache, hash weights and step inputs -----------
    # weak scaling: every rank decodes its own batch of sequences (independent (sequence,
    # kv-head) units, no collective on the path)
    ctxs, qs, kns, vns, outs = [], [], [], [], []
    gen = torch.Generator(device=dev).manual_seed(7 + rank)
    for l in range(L):
        cache = ha.PagedHashKVCache(B, HKV, max(lens), dev, shuffle_seed=100 * rank + l)
        synthetic.fill_cache_on_device(cache, lens, seed=1000 * rank + l)
        ctx = ha.SparseDecodeContext(cache, budget, synthetic.make_usa(HQ, D, seed=l, bf16=True).packed(dev))
        ctx.hash_prefill()
        ctxs.append(ctx)
        qs.append(torch.randn(B, HQ, D, generator=gen, device=dev).bfloat16())
        kns.append(torch.randn(B, HKV, D, generator=gen, device=dev).bfloat16())
        vns.append(torch.randn(B, HKV, D, generator=gen, device=dev).bfloat16())
        outs.append(torch.empty(B, HQ, D, dtype=torch.bfloat16, device=dev))
    torch.cuda.synchronize()
    for ctx in ctxs:
        ctx.check_status()
    # what was fed in, so that a result can be tied to its inputs: the seeds and a digest of layer instance 0
    # (step inputs, the first page of keys and its hash codes as the prefill kernel wrote them)
    import hashlib
    digest = hashlib.sha256()
    for t in (qs[0], kns[0], vns[0], ctxs[0].cache.k_pages[int(ctxs[0].cache.page_table[0, 0])],
              ctxs[0].cache.hash_pages[int(ctxs[0].cache.page_table[0, 0])]):
        digest.update(t.contiguous().view(torch.uint8).cpu().numpy().tobytes())
    inputs = {"seeds": {"step_inputs": 7 + rank, "cache_of_instance_l": f"{1000 * rank} + l", "page_shuffle": f"{100 * rank} + l",
                        "hash_weights_of_instance_l": "l (torch default Linear init, rounded to bf16)"},
              "sha256_instance0": digest.hexdigest()}

    def capture(fn, layers):
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for l in layers:  # warm-up launch outside capture
                fn(l)
            side.synchronize()
            with torch.cuda.graph(g, stream=side):
                for l in layers:
                    fn(l)
        torch.cuda.current_stream().wait_stream(side)
        return g

    def full(l):
        ctxs[l].decode_step(qs[l], kns[l], vns[l], out=outs[l])

    g_token = capture(full, range(L))                       # one "token": all L layer instances
    g_single = [capture(full, [l]) for l in range(L)]       # for step counts not divisible by L

    def run_steps(n):
        for _ in range(n // L):
            g_token.replay()
        for l in range(n % L):
            g_single[l].replay()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        fn(n)
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) * 1e-3  # seconds, max over ranks

    # ---- the timed region --------------------------------------------------------------------
    run_steps(max(args.warmup, 3))
    sampler = ClockSampler(local) if rank == 0 else None
    t_total = timed(run_steps, args.steps)
    # keep the same workload running a little longer so the clock samples are under load
    t_end = time.perf_counter() + 1.5
    while sampler is not None and time.perf_counter() < t_end:
        run_steps(L * 64)
        torch.cuda.synchronize()
    clocks = sampler.stop() if sampler is not None else None
    for ctx in ctxs:
        ctx.check_status()
    per_step = t_total / args.steps
    value = world * nbytes["total"] / per_step / 1e9

    # ---- per-stage device time (stage graphs over the same L instances) ----------------------
    stage_fns = {
        "hash_decode": lambda l: ctxs[l].hash_decode(qs[l], kns[l], vns[l]),
        "score_select": lambda l: ctxs[l].score_select(),
        "sparse_decode": lambda l: ctxs[l].sparse_decode(qs[l], out=outs[l]),
    }
    reps = max(4, min(200, args.steps // L))
    stage_us = {}
    for name, fn in stage_fns.items():
        g = capture(fn, range(L))
        for _ in range(3):
            g.replay()
        stage_us[name] = timed(lambda n, g=g: [g.replay() for _ in range(n)], reps) / (reps * L) * 1e6
    att_bytes = nbytes["kv"] + nbytes["qo"]
    peak, peak_src = peaks()
    att_gbs = att_bytes / (stage_us["sparse_decode"] * 1e-6) / 1e9
    # small steps run the gather as clusters that merge among themselves: 3 kernels per step, no merge kernel
    clustered = int(ctxs[0].lib.ha_decode_step_launches(ctxs[0].shape, ctxs[0].c_budget)) == 3
    roofline = {"bound": "hbm", "kernel": "sparse_gather_kernel (cluster variant, merges in the cluster)" if clustered
                else "sparse_gather_kernel + sparse_merge_kernel", "achieved": att_gbs, "peak": peak, "unit": "GB/s",
                "frac": att_gbs / peak, "traffic": NCU_TRAFFIC.get(args.workload), "peak_source": peak_src,
                "algorithmic_bytes_per_launch": att_bytes, "us_per_launch": stage_us["sparse_decode"]}
    pipeline = {"bytes_per_step": nbytes, "achieved": nbytes["total"] / per_step / 1e9, "peak": peak,
                "frac": nbytes["total"] / per_step / 1e9 / peak, "frac_of_8tbs": nbytes["total"] / per_step / 8e12,
                "stage_us": stage_us}

    # ---- prefill key-hash build (tcgen05 GEMM chain) over the same caches ------------------------
    n_pre = max(1, min(L, 8))
    for l in range(min(L, 2)):
        ctxs[l].hash_prefill()
    t_pre = timed(lambda n: [ctxs[i % L].hash_prefill() for i in range(n)], n_pre) / n_pre
    pre_flops = 2.0 * 36864 * HQ * sum(lens)  # 3 GEMMs of the 128-128-128-32 MLP per token and query head
    tpeak, tpeak_src = tensor_peak()
    prefill = {"kernel": "hash_prefill_tc_kernel", "tokens": sum(lens), "ms": t_pre * 1e3,
               "tflops_algorithmic": pre_flops / t_pre / 1e12, "peak_tflops": tpeak, "peak_source": tpeak_src,
               "frac": pre_flops / t_pre / 1e12 / tpeak,
               "note": "executed MACs are 1.56x the algorithmic ones (hi/lo bf16 split of the hidden activations)"}
    for ctx in ctxs:
        ctx.check_status()

    # ---- end to end through the host-buffer entry point --------------------------------------
    bufs = [ha.HostStepBuffers(c) for c in ctxs]
    for l in range(L):
        bufs[l].q_host.copy_(qs[l]); bufs[l].k_host.copy_(kns[l]); bufs[l].v_host.copy_(vns[l])
    n_e2e = max(1, min(args.steps, 4000))

    def e2e_steps(n):
        for i in range(n):
            ha.decode_step_host(ctxs[i % L], bufs[i % L], synchronize=True, use_graph=True)

    e2e_steps(min(n_e2e, 3 * L))
    barrier()
    t0 = time.perf_counter()
    e2e_steps(n_e2e)
    barrier()
    t_e2e = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_e2e, op=dist.ReduceOp.MAX)
    e2e_per_step = float(t_e2e.item()) / n_e2e
    assert torch.equal(bufs[0].out_host.to(dev), outs[0]), "host-buffer path disagrees with the device path"
    e2e = {"value": world * nbytes["total"] / e2e_per_step / 1e9, "unit": UNIT, "us_per_layer": e2e_per_step * 1e6,
           "steps": n_e2e, "h2d_bytes_per_step": bufs[0].h2d_bytes, "d2h_bytes_per_step": bufs[0].d2h_bytes}

    # ---- CPU baseline on rank 0 at N = 1 -------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_per_step, n_cpu, threads, _, sample = cpu_reference_run(args.workload, 50, 2, 15.0)
        cpu = {"value": nbytes["total"] / cpu_per_step / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": sample, "us_per_layer": cpu_per_step * 1e6}

    # kernels of this library launched inside the timed region (the library reports how many one step takes)
    launches_per_step = int(ctxs[0].lib.ha_decode_step_launches(ctxs[0].shape, ctxs[0].c_budget))

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": per_step * 1e3, "us_per_layer": per_step * 1e6,
            "tokens_per_s_per_layer": world * B / per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{args.workload}: {w['desc']}", "per_gpu_batch": B, "layer_instances": L,
                       "l2": f"inputs larger than L2: {L} layer instances x {nbytes['total'] / 1e6:.1f} MB touched per "
                             f"step, visited round-robin", "launch": "CUDA graph of one step per layer instance",
                       "partition": "each GPU decodes its own sequences (all 8 kv heads); no collective on the path"},
            "launches_per_step": launches_per_step, "inputs": inputs, "roofline": roofline, "pipeline": pipeline, "prefill_hash": prefill, "e2e": e2e, "cpu_baseline": cpu, "clocks": clocks,
            "gpu_launches": launches_per_step * args.steps,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100000)
    ap.add_argument("--warmup", type=int, default=1600)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="config1")
    ap.add_argument("--layers", type=int, default=0, help="layer instances kept resident (0 = workload default)")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch (profiling small cases)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
