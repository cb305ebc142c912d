"""Benchmark of the HashAttention sparse-decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload config3|config1|config2]
    python bench.py --impl reference ...        # the CPU arm: the reference's algorithm on host cores

A step is one decode step of one attention layer over one batch: hash-encode the new query and
key (+ cache append), Hamming-score the key-hash cache, budget-select, sparse GQA attention.
Consecutive steps run on different layer instances (own K/V/hash cache, own hash weights), as
the layers of a model do, so every step's inputs come from HBM and not from L2; the instances
of one "token" are replayed as one CUDA graph, the way a serving loop launches a decode step.

The default workload is BASELINE configs[3] (B=4, S=131072, heavy 1/32). On N GPUs the SAME
problem is cut by kv-head (8 / N kv-heads per GPU, their query heads, hash weights and caches):
strong scaling, no collective on the path, one all-gather of the outputs at the end (timed apart).
At N=1 the line also carries configs[1] and configs[2] as secondary blocks.

Prints ONE JSON line (rank 0). `value` is algorithmic HBM bytes per second of the whole problem
with everything resident in HBM (median of R timed regions of K steps each); `us_per_layer` is the
same measurement as time; `e2e` is measured through the host-buffer C-ABI call (q/k/v read from
pinned host memory, result and status written back, stream wait, every step).
"""
from __future__ import annotations

import argparse
import gc
import hashlib
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
    # name: description, batch, lengths, heavy budget
    "config1": dict(desc="BASELINE configs[1]: B=1, S=32768, 32q/8kv heads, d=128, init 128 / recent 128 / heavy 1/32",
                    batch=1, lens=lambda: [32768], heavy=1.0 / 32, index=1),
    "config2": dict(desc="BASELINE configs[2] decode part: B=32, S_b uniform in [16384,65536] (seeded), heavy 1/16, "
                         "shuffled 256-token pages", batch=32, lens=None, heavy=1.0 / 16, index=2),
    "config3": dict(desc="BASELINE configs[3]: B=4, S=131072, 32q/8kv heads, d=128, init 128 / recent 128 / heavy 1/32, "
                         "cut by kv-head over the GPUs",
                    batch=4, lens=lambda: [131072] * 4, heavy=1.0 / 32, index=3),
}
INIT, RECENT = 128, 128
METRIC, UNIT = "sparse_decode_attn_hbm_gbs", "GB/s"
REPEATS = 9                     # timed regions of K steps each; the median is reported
L2_BYTES = 126e6
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "ncu_traffic.json")


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


def ncu_traffic(workload: str, kernel: str):
    """dram bytes per launch of the dominant kernel from the ncu capture summarised under profiles/
    (a small JSON written next to the summary, keyed by workload; its `kernel` must be the kernel
    this build launches, else the figure is stale and None is reported)."""
    try:
        with open(TRAFFIC_FILE) as f:
            entry = json.load(f).get(workload)
    except (OSError, ValueError):
        return None, None
    if not entry or entry.get("kernel") != kernel:
        return None, entry.get("summary") if entry else None
    return entry.get("dram_bytes_per_launch"), entry.get("summary")


def config_block(name):
    """What both arms print as `config`: the workload and nothing that depends on the arm."""
    w = WORKLOADS[name]
    lens = workload_lens(name)
    return {"workload": f"{name}: {w['desc']}", "batch": len(lens), "context_min": min(lens), "context_max": max(lens),
            "init_budget": INIT, "recent_budget": RECENT, "heavy_budget": w["heavy"], "q_heads": HQ, "kv_heads": HKV,
            "head_dim": D}


def workload_lens(name):
    w = WORKLOADS[name]
    if w["lens"] is not None:
        return w["lens"]()
    from hashattention_b200 import synthetic
    return synthetic.ragged_lengths(w["index"], w["batch"], 16384, 65536)


def percentile(xs, q):
    xs = sorted(xs)
    pos = q * (len(xs) - 1)
    lo, hi = int(math.floor(pos)), int(math.ceil(pos))
    return xs[lo] + (xs[hi] - xs[lo]) * (pos - lo)


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
def cpu_reference_run(workload: str, max_steps: int, warmup: int, budget_s: float, variants=("as_is",)):
    """Times the reference's decode attention on the host cores through the oracle port, on a bounded
    sample of the workload (sequence 0, all 32 heads), in up to two variants:
      as_is         the reference as it stands: every key re-hashed with the 32 key MLPs on every step,
                    full sort, dense masked softmax (hashattention_llama.py:405-408, 430, 585-615)
      cached_signs  the reference's own cached-signature branch (:409-420): q_embedding of the query,
                    k_embedding of the new key only, stored key signs, baddbmm - like for like with a
                    key-hash cache
    with the stages (hash / sort-select / attention) timed separately. Returns a dict per variant:
    seconds per FULL step of the workload (sample time scaled by the byte ratio: sequences are
    independent), stage seconds, steps run; plus threads, bytes per step and the sample description."""
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
    S = lens[0]
    sample_bytes = synthetic.algorithmic_bytes([S], HQ, HKV, INIT, RECENT, w["heavy"])["total"]
    scale = full_bytes / sample_bytes
    usa = synthetic.make_usa(HQ, D, seed=0, bf16=True).float()
    g = torch.Generator().manual_seed(1000 + w["index"])
    q = torch.randn(1, HQ, D, generator=g).bfloat16().float()
    k = torch.randn(1, HKV, S, D, generator=g)
    k[..., list(synthetic.OUTLIER_CHANNELS)] *= synthetic.OUTLIER_SCALE
    k = k.bfloat16().float()
    v = torch.randn(1, HKV, S, D, generator=g).bfloat16().float()
    heavy = w["heavy"]

    def stages_as_is():
        t = [time.perf_counter()]
        k_rep = k.repeat_interleave(HQ // HKV, dim=1)
        k_pre = orc.mlp_preact(orc.nets_from_usa(usa, "k"), k_rep)
        q_pre = orc.mlp_preact(orc.nets_from_usa(usa, "q"), q[:, :, None, :])
        span = orc.span_scores(q_pre, k_pre)
        t.append(time.perf_counter())
        mask = orc.select_mask(span, INIT, RECENT, heavy, bit_step=2.0)
        t.append(time.perf_counter())
        orc.masked_attention(q, k, v, mask)
        t.append(time.perf_counter())
        return [t[i + 1] - t[i] for i in range(3)]

    past = {}

    def stages_cached():
        if "signs" not in past:  # the state a real run would carry from step to step (not timed)
            k_rep = k[:, :, :S - 1].repeat_interleave(HQ // HKV, dim=1)
            past["signs"] = torch.sign(orc.mlp_preact(orc.nets_from_usa(usa, "k"), k_rep))
        t = [time.perf_counter()]
        span = orc.cached_span(usa, q, k[:, :, S - 1:], past["signs"], HQ // HKV)
        t.append(time.perf_counter())
        mask = orc.select_mask(span, INIT, RECENT, heavy, bit_step=2.0)
        t.append(time.perf_counter())
        orc.masked_attention(q, k, v, mask)
        t.append(time.perf_counter())
        return [t[i + 1] - t[i] for i in range(3)]

    out = {}
    share = budget_s / len(variants)
    with torch.no_grad():
        for name in variants:
            fn = stages_as_is if name == "as_is" else stages_cached
            first = sum(fn())
            n_warm = max(0, min(warmup, 3, int(share * 0.2 / max(first, 1e-9))))
            for _ in range(n_warm):
                fn()
            n = max(1, min(max_steps, int(share / max(first, 1e-9))))
            runs = [fn() for _ in range(n)]
            per = [statistics.median(r[i] for r in runs) for i in range(3)]
            out[name] = {"s_per_step": sum(per) * scale, "steps": n,
                         "stage_s": {"hash": per[0] * scale, "sort_select": per[1] * scale, "attention": per[2] * scale}}
    sample = (f"sequence 0 of {workload} (S={S}, all 32 heads, fp32 torch CPU ops in the reference's structure), "
              f"median of the steps run, scaled by the byte ratio {scale:.3g} to the whole batch")
    return out, threads, full_bytes, sample


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    res, threads, nbytes, sample = cpu_reference_run(args.workload, max(1, args.steps), args.warmup, 60.0)
    per_step = res["as_is"]["s_per_step"]
    value = nbytes / per_step / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "steps_run": res["as_is"]["steps"], "warmup": args.warmup, "ms_per_step": per_step * 1e3,
        "us_per_layer": per_step * 1e6, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": config_block(args.workload),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample,
                         "variant": "as_is (re-hashes every key each step, full sort, dense masked softmax)",
                         "stage_us": {k: v * 1e6 for k, v in res["as_is"]["stage_s"].items()}},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
class Bench:
    """One workload on this rank's GPU: L layer instances of this rank's kv-head shard."""

    def __init__(self, ha, synthetic, name, dev, rank, world, layers=0, batch=0):
        import torch
        self.torch, self.ha, self.dev, self.rank, self.world, self.name = torch, ha, dev, rank, world, name
        w = WORKLOADS[name]
        lens = workload_lens(name)
        if batch:  # fewer sequences, or the workload's sequences repeated (profiling small cases)
            lens = (lens * ((batch + len(lens) - 1) // len(lens)))[:batch]
        self.lens, self.heavy = lens, w["heavy"]
        self.B = len(lens)
        self.j0, self.j1 = ha.partition.kv_head_range(HKV, world, rank)
        self.hkv = self.j1 - self.j0
        self.budget = ha.Budget(INIT, w["heavy"], RECENT)
        self.nbytes = synthetic.algorithmic_bytes(lens, HQ, HKV, INIT, RECENT, w["heavy"])           # whole problem
        self.nbytes_gpu = synthetic.algorithmic_bytes(lens, self.hkv * 4, self.hkv, INIT, RECENT, w["heavy"])
        # enough instances that one round over them touches well over the L2 capacity
        self.L = layers or max(3, min(16, math.ceil(3.0 * L2_BYTES / self.nbytes_gpu["total"])))
        self.ctxs, self.qs, self.kns, self.vns, self.outs = [], [], [], [], []
        for l in range(self.L):
            # the same problem on every rank count: seeds depend on (instance, global kv-head), never on the rank
            cache = ha.PagedHashKVCache(self.B, self.hkv, max(lens), dev, shuffle_seed=100 + l)
            synthetic.fill_cache_on_device(cache, lens, seed=1000 + l, kv_head0=self.j0)
            packed = synthetic.make_usa(HQ, D, seed=l, bf16=True).packed(dev)
            if world > 1:
                packed = packed.slice_heads(self.j0 * 4, self.j1 * 4)
            ctx = ha.SparseDecodeContext(cache, self.budget, packed)
            ctx.hash_prefill()
            self.ctxs.append(ctx)
            gen = torch.Generator(device=dev).manual_seed(7 + l)
            q = torch.randn(self.B, HQ, D, generator=gen, device=dev).bfloat16()
            kn = torch.randn(self.B, HKV, D, generator=gen, device=dev).bfloat16()
            vn = torch.randn(self.B, HKV, D, generator=gen, device=dev).bfloat16()
            q, kn, vn = ha.partition.shard_step_inputs(q, kn, vn, world, rank)
            self.qs.append(q); self.kns.append(kn); self.vns.append(vn)
            self.outs.append(torch.empty_like(q))
        torch.cuda.synchronize()
        self.check()
        self.launches_per_step = int(self.ctxs[0].lib.ha_decode_step_launches(self.ctxs[0].shape, self.ctxs[0].c_budget))

    def check(self):
        for ctx in self.ctxs:
            ctx.check_status()

    def inputs_digest(self):
        """Seeds and a digest of layer instance 0 (step inputs, the first page of keys and its hash codes)."""
        c = self.ctxs[0].cache
        digest = hashlib.sha256()
        page0 = int(c.page_table[0, 0])
        for t in (self.qs[0], self.kns[0], self.vns[0], c.k_pages[page0], c.hash_pages[page0]):
            digest.update(t.contiguous().view(self.torch.uint8).cpu().numpy().tobytes())
        return {"seeds": {"step_inputs_of_instance_l": "7 + l", "cache_of_instance_l_kv_head_j": "(1000 + l) * 64 + j",
                          "page_shuffle": "100 + l",
                          "hash_weights_of_instance_l": "l (torch default Linear init, rounded to bf16)"},
                "sha256_instance0_rank0": digest.hexdigest()}

    # -- graphs ------------------------------------------------------------------------------
    def capture(self, fn, layers):
        torch = self.torch
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for l in layers:  # eager launch outside capture (whatever the library sets up at first use)
                fn(l)
            side.synchronize()
            with torch.cuda.graph(g, stream=side):
                for l in layers:
                    fn(l)
        torch.cuda.current_stream().wait_stream(side)
        g.replay()  # instantiation / upload of the graph happens here, not inside a timed region
        torch.cuda.synchronize()
        return g

    def full(self, l):
        self.ctxs[l].decode_step(self.qs[l], self.kns[l], self.vns[l], out=self.outs[l])

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        self.torch.cuda.synchronize()

    def timed(self, fn, n):
        """fn(n) between two events, a barrier and a device synchronisation on both sides; seconds, max over ranks."""
        torch = self.torch
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        e0.record()
        fn(n)
        e1.record()
        self.barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=self.dev, dtype=torch.float64)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) * 1e-3

    def prepare_step_graphs(self):
        L = self.L
        self.g_token = self.capture(self.full, range(L))                  # one "token": all L layer instances
        self.g_single = [self.capture(self.full, [l]) for l in range(L)]  # for step counts not divisible by L

    def run_steps(self, n):
        for _ in range(n // self.L):
            self.g_token.replay()
        for l in range(n % self.L):
            self.g_single[l].replay()

    def measure_steps(self, steps, warmup, repeats=REPEATS):
        self.run_steps(max(warmup, 3))
        per = [self.timed(self.run_steps, steps) / steps for _ in range(repeats)]
        self.check()
        return {"median": statistics.median(per), "p10": percentile(per, 0.1), "p90": percentile(per, 0.9),
                "min": min(per), "max": max(per), "repeats": repeats}

    def measure_stages(self, steps):
        """Device time of the step's stages, each as its own graph over the same L instances: the encoder, scoring +
        plan, selection + attention (separate library calls here; inside ha_decode_step they overlap through
        programmatic launches, and small shapes run a single-pass cluster selection instead: `step_kernels`)."""
        L = self.L
        fns = {
            "hash_decode": lambda l: self.ctxs[l].hash_decode(self.qs[l], self.kns[l], self.vns[l]),
            "score_plan": lambda l: self.ctxs[l].score_plan(),
            "select_attend": lambda l: self.ctxs[l].select_attend(self.qs[l], out=self.outs[l]),
        }
        reps = max(4, min(200, steps // L))
        out = {}
        for name, fn in fns.items():
            g = self.capture(fn, range(L))
            for _ in range(3):
                g.replay()
            per = [self.timed(lambda n, g=g: [g.replay() for _ in range(n)], reps) / (reps * L) for _ in range(3)]
            out[name] = statistics.median(per) * 1e6
        return out

    def measure_prefill(self):
        L = self.L
        n_pre = max(1, min(L, 8))
        for l in range(min(L, 2)):
            self.ctxs[l].hash_prefill()
        t_pre = self.timed(lambda n: [self.ctxs[i % L].hash_prefill() for i in range(n)], n_pre) / n_pre
        flops = 2.0 * 36864 * (self.hkv * 4) * sum(self.lens)  # 3 GEMMs of the 128-128-128-32 MLP per token and query head
        self.check()
        return t_pre, flops

    def measure_e2e(self, steps):
        """ha_decode_step_host with host buffers: (a) replayed as one CUDA graph per call, (b) one C-ABI call
        per step (eager). Host wall clock, max over ranks; every step waits for its result."""
        torch, ha, L = self.torch, self.ha, self.L
        bufs = [ha.HostStepBuffers(c) for c in self.ctxs]
        for l in range(L):
            bufs[l].q_host.copy_(self.qs[l]); bufs[l].k_host.copy_(self.kns[l]); bufs[l].v_host.copy_(self.vns[l])
        n = max(1, min(steps, 4000))
        res = {}
        for mode, use_graph in (("graph", True), ("eager", False)):
            def run(k):
                for i in range(k):
                    ha.decode_step_host(self.ctxs[i % L], bufs[i % L], synchronize=True, use_graph=use_graph)
            run(min(n, 3 * L))
            per = []
            for _ in range(3):
                self.barrier()
                t0 = time.perf_counter()
                run(n)
                self.barrier()
                t = torch.tensor([time.perf_counter() - t0], device=self.dev, dtype=torch.float64)
                if self.world > 1:
                    import torch.distributed as dist
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                per.append(float(t.item()) / n)
            res[mode] = statistics.median(per)
        assert torch.equal(bufs[0].out_host.to(self.dev), self.outs[0]), "host-buffer path disagrees with the device path"
        return res, n, bufs[0].h2d_bytes, bufs[0].d2h_bytes

    def final_gather(self):
        """The one exchange of the partitioned path: all-gather of the per-rank outputs [B, Hq/N, D] along the
        head axis (NCCL). Returns (gathered output of instance 0, seconds per gather, max over ranks)."""
        full = self.ha.partition.gather_output(self.outs[0])
        if self.world == 1:
            return full, 0.0
        for _ in range(3):
            self.ha.partition.gather_output(self.outs[0])
        reps = 20
        t = self.timed(lambda n: [self.ha.partition.gather_output(self.outs[0]) for _ in range(n)], reps) / reps
        return full, t

    def free(self):
        self.ctxs = self.qs = self.kns = self.vns = self.outs = None
        self.g_token = self.g_single = None
        gc.collect()
        self.torch.cuda.empty_cache()


def pipeline_block(b: Bench, per_step, stage_us, peak):
    total = b.nbytes["total"]
    return {"bytes_per_step": b.nbytes, "achieved": total / per_step / 1e9, "peak": peak,
            "frac": total / per_step / 1e9 / peak, "frac_of_8tbs": total / per_step / 8e12, "stage_us": stage_us}


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
    if HKV % world != 0:
        raise SystemExit(f"{HKV} kv-heads cannot be cut over {world} GPUs")
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peak, peak_src = peaks()

    b = Bench(ha, synthetic, args.workload, dev, rank, world, args.layers, args.batch)
    inputs = b.inputs_digest() if rank == 0 else None
    b.prepare_step_graphs()

    # ---- the timed regions ---------------------------------------------------------------------
    sampler = ClockSampler(local) if rank == 0 and not args.steps_only else None
    t = b.measure_steps(args.steps, args.warmup, repeats=1 if args.steps_only else REPEATS)
    # keep the same workload running a little longer so the clock samples are under load
    t_end = time.perf_counter() + 1.5
    while sampler is not None and time.perf_counter() < t_end:
        b.run_steps(b.L * 16)
        torch.cuda.synchronize()
    clocks = sampler.stop() if sampler is not None else None
    per_step = t["median"]
    value = b.nbytes["total"] / per_step / 1e9
    if args.steps_only:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                              "warmup": args.warmup, "us_per_layer": per_step * 1e6, "config": config_block(args.workload),
                              "batch": b.B, "layer_instances": b.L, "step_kernels": b.ctxs[0].step_path(),
                              "note": "--steps-only: no stage, prefill, end-to-end or CPU measurements"}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    out_full, t_gather = b.final_gather()
    out_digest = hashlib.sha256(out_full.contiguous().view(torch.uint8).cpu().numpy().tobytes()).hexdigest()

    stage_us = b.measure_stages(args.steps)
    att_bytes = b.nbytes_gpu["kv"] + b.nbytes_gpu["qo"]
    att_gbs = att_bytes / (stage_us["select_attend"] * 1e-6) / 1e9
    kernel = "select_attend_kernel + select_attend_merge_kernel"
    traffic, traffic_src = ncu_traffic(args.workload if world == 1 else f"{args.workload}/gpus{world}", kernel)
    roofline = {"bound": "hbm", "kernel": kernel, "achieved": att_gbs, "peak": peak, "unit": "GB/s",
                "frac": att_gbs / peak, "frac_of_8tbs": att_gbs / 8000.0, "traffic": traffic, "traffic_source": traffic_src,
                "peak_source": peak_src, "algorithmic_bytes_per_launch": att_bytes,
                "us_per_launch": stage_us["select_attend"], "per": "GPU (this rank's kv-heads)",
                "note": "the selection + attention stage of the step timed as its own graph over the same layer instances "
                        "(ha_select_attend on the plan ha_score_plan left); bytes: the K/V rows it attends + q/out"}
    pipeline = pipeline_block(b, per_step, stage_us, peak * world)
    pipeline["peak_note"] = f"{world} x {peak} GB/s" if world > 1 else peak_src

    t_pre, pre_flops = b.measure_prefill()
    tpeak, tpeak_src = tensor_peak()
    prefill = {"kernel": "hash_prefill_tc_kernel", "tokens": sum(b.lens), "query_heads": b.hkv * 4, "ms": t_pre * 1e3,
               "tflops_algorithmic": pre_flops / t_pre / 1e12, "peak_tflops": tpeak, "peak_source": tpeak_src,
               "frac": pre_flops / t_pre / 1e12 / tpeak, "per": "GPU",
               "note": "executed MACs are 1.56x the algorithmic ones (hi/lo bf16 split of the hidden activations)"}

    e2e_s, n_e2e, h2d, d2h = b.measure_e2e(args.steps)
    e2e = {"value": b.nbytes["total"] / e2e_s["graph"] / 1e9, "unit": UNIT, "us_per_layer": e2e_s["graph"] * 1e6,
           "us_per_layer_eager_call": e2e_s["eager"] * 1e6, "steps": n_e2e,
           "how": "ha_decode_step_host per step, q/k/v in pinned host memory, result + status back, stream wait; "
                  "value: the call replayed as a CUDA graph; eager: one C-ABI call per step",
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
    L_primary, launches, step_path = b.L, b.launches_per_step, b.ctxs[0].step_path()
    per_gpu_batch, hkv_local = b.B, b.hkv
    nbytes_primary = b.nbytes
    b.free()

    # ---- secondary workloads (one GPU only): BASELINE configs[1] and configs[2] -----------------
    secondary = {}
    if world == 1 and not args.no_secondary:
        for name in ("config1", "config2"):
            if name == args.workload:
                continue
            s = Bench(ha, synthetic, name, dev, rank, world)
            s.prepare_step_graphs()
            ts = s.measure_steps(max(args.steps, 4 * s.L), args.warmup)
            st = s.measure_stages(args.steps)
            blk = pipeline_block(s, ts["median"], st, peak)
            blk.update({"workload": f"{name}: {WORKLOADS[name]['desc']}", "us_per_layer": ts["median"] * 1e6,
                        "us_per_layer_p10_p90": [ts["p10"] * 1e6, ts["p90"] * 1e6], "layer_instances": s.L,
                        "launches_per_step": s.launches_per_step, "step_kernels": s.ctxs[0].step_path()})
            secondary[name] = blk
            s.free()

    # ---- CPU baseline on rank 0 at N = 1 -------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        res, threads, _, sample = cpu_reference_run(args.workload, 20, 1, 24.0, variants=("as_is", "cached_signs"))
        a = res["as_is"]
        cpu = {"value": nbytes_primary["total"] / a["s_per_step"] / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": sample, "us_per_layer": a["s_per_step"] * 1e6,
               "variants": {k: {"us_per_layer": v["s_per_step"] * 1e6, "steps": v["steps"], "cores": threads,
                                "stage_us": {s_: x * 1e6 for s_, x in v["stage_s"].items()}} for k, v in res.items()},
               "gpu_us_per_layer": per_step * 1e6}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": per_step * 1e3, "us_per_layer": per_step * 1e6,
            "us_per_layer_p10_p90": [t["p10"] * 1e6, t["p90"] * 1e6], "repeats": t["repeats"],
            "tokens_per_s_per_layer": per_gpu_batch / per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_block(args.workload),
            "setup": {"kv_heads_per_gpu": hkv_local, "layer_instances": L_primary,
                      "l2": f"inputs larger than L2: {L_primary} layer instances x {nbytes_primary['total'] / world / 1e6:.1f} MB "
                            f"touched per step and GPU, visited round-robin",
                      "launch": "CUDA graph of one step per layer instance, replayed once untimed after capture",
                      "partition": f"kv-heads cut over {world} GPU(s): {hkv_local} per GPU; no collective on the path, "
                                   f"one all-gather of the outputs at the end (final_gather_us)"},
            "final_gather_us": t_gather * 1e6, "out_sha256_instance0": out_digest,
            "launches_per_step": launches, "step_kernels": step_path, "inputs": inputs, "roofline": roofline, "pipeline": pipeline,
            "secondary": secondary, "prefill_hash": prefill, "e2e": e2e, "cpu_baseline": cpu, "clocks": clocks,
            "gpu_launches": launches * args.steps,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------------
# BASELINE configs[4]: the whole Llama-3.1-8B-architecture model, tensor-parallel, greedy decode
# --------------------------------------------------------------------------------------------
CONFIG4_DESC = ("BASELINE configs[4]: Llama-3.1-8B architecture (32 layers, hidden 4096, 32q/8kv heads, d=128, FFN 14336, "
                "vocab 128256), random bf16 weights, HashAttention on every layer (init 128 / recent 128 / heavy 1/32), "
                "batch 8, prefill 32768 random token ids, greedy decode, tensor-parallel with an all-reduce after "
                "attention and after the MLP")


def run_config4(args):
    """`--steps` greedy decode steps of the whole model (every layer, batch 8) after a prefill of `--prefill`
    tokens; one process per GPU, q/k/v/w1/w3 column-parallel, wo/w2 row-parallel, NCCL all-reduce after
    attention and MLP. Prints decode tokens/s (whole batch, all GPUs together)."""
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    ha = entry.load_package()
    from hashattention_b200 import llama_tp

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    batch = args.batch or 8
    cfg = llama_tp.LlamaTPConfig(max_seq_len=args.prefill + args.steps + args.warmup + 8)
    if args.layers:
        cfg.n_layers = args.layers
    model = llama_tp.TPLlama(cfg, world, rank, dev, batch, seed=0)
    tokens = llama_tp.tokens_for(cfg, batch, args.prefill).to(dev)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sync()
    t0 = time.perf_counter()
    cur = model.prefill(tokens)
    sync()
    prefill_s = time.perf_counter() - t0
    model.check_status()

    nxt = torch.empty_like(cur)
    for _ in range(2):  # eager steps first (lazy initialisation of the libraries involved)
        model.decode_step(cur, nxt)
        cur.copy_(nxt)
    sync()
    launch = "CUDA graph of one decode step (all layers, both all-reduces per layer)"
    graph = None
    try:
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                model.decode_step(cur, nxt)
                cur.copy_(nxt)
        torch.cuda.current_stream().wait_stream(side)
    except Exception as e:  # a collective that cannot be captured: run the steps eagerly
        graph, launch = None, f"eager (graph capture failed: {type(e).__name__})"
        torch.cuda.synchronize()

    def step():
        if graph is not None:
            graph.replay()
        else:
            model.decode_step(cur, nxt)
            cur.copy_(nxt)

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(local) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    sync()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    seconds = float(t.item()) * 1e-3
    clocks = sampler.stop() if sampler is not None else None
    model.check_status()
    seq_len = int(model.ctxs[0].cache.seq_lens[0])
    launches = int(model.ctxs[0].lib.ha_decode_step_launches(model.ctxs[0].shape, model.ctxs[0].c_budget))
    if rank == 0:
        line = {
            "metric": "decode_tokens_per_s", "value": batch * args.steps / seconds, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds / args.steps * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"config4: {CONFIG4_DESC}", "batch": batch, "prefill_tokens": args.prefill,
                       "layers": cfg.n_layers, "parallelism": f"tp{world}"},
            "prefill_s": prefill_s, "context_at_end": seq_len, "launch": launch,
            "attention_kernels_per_layer": model.ctxs[0].step_path(), "sample_tokens": cur[:4].tolist(),
            "gpu_launches": launches * cfg.n_layers * args.steps, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    # A captured graph that holds NCCL kernels must be gone before the communicator is torn down (a teardown in
    # the other order has been seen to block); the ranks leave together, without waiting for destructors.
    graph = None
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=600)
    ap.add_argument("--warmup", type=int, default=60)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + ["config4"], default="config3")
    ap.add_argument("--prefill", type=int, default=32768, help="config4: prompt length")
    ap.add_argument("--layers", type=int, default=0, help="layer instances kept resident (0 = sized to exceed L2)")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch (profiling small cases)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip the configs[1] / configs[2] blocks")
    ap.add_argument("--steps-only", action="store_true",
                    help="warm up, time the steps, print a short line and stop (for profiler captures of small cases)")
    args = ap.parse_args()
    if args.workload == "config4":
        if args.impl == "reference":
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable": "the reference's full-model host (efficiency/model.py, "
                                  "generate.py) imports modules that are not in its repository; no CPU arm for config4"}))
            return
        if args.steps == 600 and args.warmup == 60:  # the defaults of the layer-step workloads
            args.steps, args.warmup = 256, 8
        run_config4(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
