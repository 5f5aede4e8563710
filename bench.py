"""Benchmark of the 4-bit decode hot path: Llama-3-8B-shape greedy decode, batch 1, on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--ctx C] [--small]

A step is one greedy decode token (the whole layer stack, output head and argmax) at a context of `--ctx`
tokens already in the KV cache. `value` is tokens/s with everything resident on the device (CUDA-graph
replays, device-side token feedback), timed with CUDA events on the launching stream; `e2e` is the same metric
through the per-token C-ABI call the reference's host would make (swlm_decode: token id in from pinned host
memory, token id out, one synchronisation per token). Random-init weights of the named shape, seeded.

With --impl reference the CPU oracle (a scalar restatement of the reference's arithmetic; the reference's
Metal kernels cannot run here) decodes a bounded sample of the same workload on the host cores.
"""
import argparse
import dataclasses
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from __graft_entry__ import load_package  # noqa: E402

METRIC = "4-bit decode tok/s, Llama-3-8B shape bs1"
NOMINAL_HBM_GBS = 8000.0
NCU_TRAFFIC_RATIO = 123.679 / 122.683


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def measured_tensor_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    return 1590.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs (read-only queries)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def count(self):
        return len(self.rows)

    def alive(self):
        return self.proc is not None and self.proc.poll() is None

    def wait_first(self, seconds):
        t0 = time.perf_counter()
        while self.alive() and not self.rows and time.perf_counter() - t0 < seconds:
            time.sleep(0.02)

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons), "samples": len(sm)}


def model_config(pkg, args, max_seq, world=1):
    if args.small:  # debugging aid; never the reported workload
        return pkg.ModelConfig("llama", hidden=1024, intermediate=2816, layers=4, heads=8, kv_heads=2, head_dim=128,
                               vocab=8192, max_seq=max_seq, max_batch=args.batch)
    if args.model == "lfm2":
        # hybrid conv/attention shape; output head tied to a Q4 embedding table (the MLX-bundle convention)
        # (under tensor parallelism the head is a tensor of its own: a vocabulary-sharded table cannot serve the gather)
        return pkg.lfm2_like_config(max_seq=max_seq, max_batch=args.batch, tie_embeddings=world == 1)
    return pkg.llama3_8b_config(max_seq=max_seq, max_batch=args.batch)


def shape_name(args):
    return "small-debug" if args.small else ("LFM2-1.2B-like shape (10 conv + 6 attention layers, tied Q4 head)" if args.model == "lfm2" else "Llama-3-8B shape")


def metric_name(args):
    if args.model == "llama" and args.batch == 1 and getattr(args, "kv", "bf16") == "bf16":
        return METRIC
    return f"4-bit decode tok/s, {'LFM2-1.2B-like' if args.model == 'lfm2' else 'Llama-3-8B'} shape bs{args.batch}" + (
        {"bf16": "", "q8": ", 8-bit KV"}.get(getattr(args, "kv", "bf16"), ", rotated 4-bit KV"))


def workload_name(args):
    kv = {"bf16": "", "q8": ", 8-bit group-32 KV cache", "rotor-q4": ", rotated 4-bit group-64 KV cache",
          "rotor-q4-qjl16": ", rotated 4-bit group-64 KV cache with 16 projected K residuals per row"}[getattr(args, "kv", "bf16")]
    return shape_name(args) + f", 4-bit g64 weights, batch {args.batch}, greedy decode at context {args.ctx}" + kv


def cpu_baseline(pkg, builder, weights, cfg, sample_steps, ctx):
    """Oracle decode on the host cores over a bounded sample: `sample_steps` tokens at a short context."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_binding

    so = os.path.join(ROOT, "oracle", "liboracle.so")
    if not os.path.exists(so):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle")], check=True)
    orc = oracle_binding.Oracle(so)
    # every host core, whatever OMP_NUM_THREADS says (torch.distributed.run exports OMP_NUM_THREADS=1)
    orc.set_threads(os.cpu_count() or 1)
    cores = orc.threads()
    import dataclasses
    small_cfg = dataclasses.replace(cfg, max_seq=sample_steps + 2, max_batch=1)
    om = orc.model(small_cfg.buffers_desc())
    om.load(builder, weights)
    tok = np.array([1], dtype=np.int32)
    tok = om.decode(tok)  # warm the caches / page in the weights
    t0 = time.perf_counter()
    for _ in range(sample_steps):
        tok = om.decode(tok)
    dt = time.perf_counter() - t0
    return {"value": sample_steps / dt, "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"{sample_steps} greedy decode steps of the full model at context <= {sample_steps + 1} "
                      f"(the context-{ctx} KV read is 11% of a step's bytes and is not part of the CPU sample)"}


def tp_parity_check(pkg, dist, rank, world, local_rank):
    """Correctness evidence for a tensor-parallel line: a small Llama-shape model sharded over the same ranks decodes
    24 greedy steps, and every rank compares its tokens with the CPU oracle of the unsharded model (the oracle is the
    checker here, nothing of it is timed). Returns a short description, raises on a mismatch."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_binding

    cfg = pkg.ModelConfig("llama", hidden=1024, intermediate=2048, layers=3, heads=16, kv_heads=8, head_dim=64,
                          vocab=4096, max_seq=96, max_batch=1)
    builder = pkg.DispatchPlanBuilder(cfg)
    weights = pkg.synth_model_weights(builder, seed=5)
    store = pkg.WeightStore(local_rank, tp_rank=rank, tp_size=world)
    model = pkg.load_model(store, builder, weights)
    pkg.tp.attach(model, dist)
    om = oracle_binding.Oracle(os.path.join(ROOT, "oracle", "liboracle.so")).model(cfg.buffers_desc())
    om.load(builder, weights)
    prompt = np.random.default_rng(2).integers(0, cfg.vocab, size=(1, 6), dtype=np.int32)
    g, o = model.prefill(prompt), om.prefill(prompt)
    bad, steps = 0, 24
    for _ in range(steps):
        bad += int((g != o).sum())
        g, o = model.decode(o), om.decode(o)
    status = pkg.tp.status(model)
    model.close()
    store.close()
    gathered = [None] * world
    dist.all_gather_object(gathered, (bad, status))
    if any(b > 1 or st != 0 for b, st in gathered):
        raise SystemExit(f"tensor-parallel parity check failed: (mismatches, status) per rank = {gathered}")
    return f"ok ({steps} greedy steps of a 3-layer 1024-wide model on {world} GPUs, every rank against the CPU oracle: " \
           f"{sum(b for b, _ in gathered)} token mismatches (ties), exchange status 0)"


def run_reference(args, pkg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = model_config(pkg, args, 64)
    builder = pkg.DispatchPlanBuilder(cfg)
    weights = pkg.synth_model_weights(builder, seed=3)
    steps = max(1, min(args.steps, 8))
    base = cpu_baseline(pkg, builder, weights, cfg, steps, args.ctx)
    line = {"impl": "reference", "metric": metric_name(args), "value": base["value"], "unit": "tok/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": 1, "ms_per_step": 1000.0 / base["value"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16 activations, fp32 accumulate, 4-bit weights",
            "data": "synthetic (seeded random-init weights of the named shape)",
            "config": {"workload": workload_name(args), "note": "CPU oracle on host cores; the reference's Metal kernels are unavailable on this box"},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def run_op(args, pkg):
    """Op-level lines: `--op qgemv` (one quantized GEMV/GEMM shape, rotating through enough distinct weight sets
    to exceed L2) and `--op flash` (flash-decode over a synthetic KV cache). One JSON line each."""
    import ctypes as C

    import torch

    torch.cuda.set_device(0)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    store = pkg.WeightStore(0)
    lib = store.lib
    peak, peak_src = measured_peaks()
    sptr = C.c_void_p(stream.cuda_stream)
    if args.op == "qgemv":
        n, k, m = args.n, args.k, args.m
        per_set = n * k * 0.5625
        # --min-mb 0: one weight set, i.e. L2-resident weights when they fit (shows the compute-side ceiling)
        sets = 1 if args.min_mb <= 0 else max(2, int(np.ceil(args.min_mb * 1e6 / per_set)))
        for i in range(sets):
            store.add_q4_mlx(f"w{i}", *pkg.synth_q4(n, k, seed=i))
        x = torch.randn(m, k, device="cuda").bfloat16()
        y = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)

        def one_round():
            for i in range(sets):
                lib.check(lib.swlm_op_qgemm_dev(store.handle, f"w{i}".encode(), m, x.data_ptr(), y.data_ptr(), sptr))

        for _ in range(max(3, args.warmup)):
            one_round()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            one_round()
        e1.record(stream)
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (args.steps * sets)
        bytes_per_launch = per_set + 2 * m * k + 2 * m * n
        gbs = bytes_per_launch / (us * 1e-6) / 1e9
        if m >= 64:  # tensor-core (tcgen05) prefill product: the bound is the tensor pipe, not HBM
            tfs = 2.0 * m * n * k / (us * 1e-6) / 1e12
            tpeak, tsrc = measured_tensor_peak()
            print(json.dumps({"metric": "q4 prefill GEMM TFLOP/s", "value": tfs, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
                              "config": {"workload": f"q4g64 GEMM N={n} K={k} M={m} (tcgen05), {sets} distinct weight sets in rotation"},
                              "us_per_launch": us, "flops_per_launch": 2.0 * m * n * k, "weight_stream_gbs": gbs,
                              "roofline": {"bound": "tensor", "achieved": tfs, "peak": tpeak, "unit": "TFLOP/s", "frac": tfs / tpeak,
                                           "peak_source": tsrc, "traffic": None}}))
            store.close()
            return
        print(json.dumps({"metric": "qGEMV HBM GB/s", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
                          "config": {"workload": f"q4g64 GEMV N={n} K={k} M={m}, {sets} distinct weight sets in rotation ({sets * per_set / 1e6:.0f} MB > L2)"},
                          "us_per_launch": us, "bytes_per_launch": bytes_per_launch,
                          "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                                       "peak_source": peak_src, "frac_of_nominal_8TBs": gbs / NOMINAL_HBM_GBS, "traffic": None}}))
    elif args.op == "flash":
        B, H, KV, D, ctx = args.m, 32, 8, 128, args.ctx
        q = torch.randn(B, H, D, device="cuda").bfloat16()
        kc = torch.randn(B, KV, ctx, D, device="cuda").bfloat16()
        vc = torch.randn(B, KV, ctx, D, device="cuda").bfloat16()
        out = torch.empty(B, H, D, device="cuda", dtype=torch.bfloat16)
        scratch = torch.empty(lib.swlm_op_flash_decode_scratch_bytes(B, H, KV, D, ctx), device="cuda", dtype=torch.uint8)
        flush = torch.empty(256 << 20, device="cuda", dtype=torch.uint8)
        kv_bytes = 2 * B * KV * ctx * D * 2
        small = kv_bytes < (160 << 20)

        def call():
            lib.check(lib.swlm_op_flash_decode_dev(store.handle, B, H, KV, D, ctx, ctx, 1.0 / np.sqrt(D), q.data_ptr(), kc.data_ptr(),
                                                   vc.data_ptr(), out.data_ptr(), scratch.data_ptr(), sptr))

        for _ in range(max(3, args.warmup)):
            call()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(args.steps):
            if small:
                flush.fill_(1)  # the cache fits in L2: evict it between timed calls
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            call()
            e1.record(stream)
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        us = total * 1e3 / args.steps
        gbs = kv_bytes / (us * 1e-6) / 1e9
        print(json.dumps({"metric": "flash-decode HBM GB/s", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
                          "config": {"workload": f"flash-decode GQA 32q/8kv x128, batch {B}, context {ctx}",
                                     "l2": "L2 flushed between calls" if small else "KV cache larger than L2"},
                          "us_per_call": us, "bytes_per_call": kv_bytes,
                          "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                                       "peak_source": peak_src, "frac_of_nominal_8TBs": gbs / NOMINAL_HBM_GBS, "traffic": None}}))
    store.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", choices=["qgemv", "flash"], default=None, help="op-level line instead of the decode benchmark")
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--min-mb", type=float, default=400.0, help="rotate through at least this many MB of distinct weights")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="swlm")
    ap.add_argument("--ctx", type=int, default=4096, help="tokens in the KV cache when the timed region starts")
    ap.add_argument("--prefill", choices=["real", "synthetic"], default="real",
                    help="how the KV cache gets its `ctx` tokens: by running the prompt, or random bf16 rows")
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--model", choices=["llama", "lfm2"], default="llama", help="llama: Llama-3-8B shape; lfm2: the hybrid conv/attention shape")
    ap.add_argument("--batch", type=int, default=1, help="sequences decoded together (1..64), all at the same position")
    ap.add_argument("--kv", choices=["bf16", "q8", "rotor-q4", "rotor-q4-qjl16"], default="bf16",
                    help="KV cache elements: bf16, 8-bit groups of 32 (36-byte blocks), or the rotated 4-bit groups of 64 "
                         "(the reference's default policy for plain transformer graphs), optionally with 16 projected K residuals per row")
    ap.add_argument("--cpu-sample-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    pkg = load_package()

    if args.model == "lfm2" and args.ctx == 4096:
        args.ctx = 2048   # the hybrid configuration's prompt length
    if args.batch > 1 and args.prefill == "real":
        args.prefill = "synthetic"   # chunked prompt ingestion serves one sequence; a batch gets random cache rows
    if args.impl == "reference":
        run_reference(args, pkg)
        return
    if args.op:
        run_op(args, pkg)
        return

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    tp_parity = tp_parity_check(pkg, dist, rank, world, local_rank) if world > 1 else None
    warm = max(3, args.warmup)
    max_seq = args.ctx + 2 * (warm + args.steps) + 64 + 8 * 64   # + room for the clock sampler's extra warm-up bursts
    cfg = model_config(pkg, args, max_seq, world)
    if args.kv == "q8":
        cfg = dataclasses.replace(cfg, kv_scheme=0x10)
    elif args.kv.startswith("rotor-q4"):
        cfg = dataclasses.replace(cfg, kv_scheme=0x71, kv_qjl_dim=16 if args.kv.endswith("qjl16") else 0)
        if args.prefill == "real":
            args.prefill = "synthetic"   # prompts over an 8-bit cache go token by token; the timed region is the decode
    builder = pkg.DispatchPlanBuilder(cfg)
    weights = pkg.synth_model_weights(builder, seed=3)
    store = pkg.WeightStore(local_rank, tp_rank=rank, tp_size=world)
    model = pkg.load_model(store, builder, weights)
    if world > 1:
        pkg.tp.attach(model, dist)
    # a stream of our own: torch's default stream has handle 0, which the C ABI reads as "use your own"
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    model.set_stream(stream.cuda_stream)

    # ---- context: `ctx` tokens in the KV cache ---------------------------------------------------------------
    rng = np.random.default_rng(7)
    prefill_info = None
    if args.prefill == "real":
        prompt = rng.integers(0, cfg.vocab, size=(args.batch, args.ctx), dtype=np.int32)
        torch.cuda.synchronize()
        t_pf = time.perf_counter()
        tok = model.prefill(prompt)   # host tokens in, first generated token out (synchronous)
        t_pf = time.perf_counter() - t_pf
        prefill_info = {"prompt_tokens": int(args.ctx), "seconds": t_pf, "tok_s": args.ctx / t_pf,
                        "how": "chunked prompt ingestion on 1 GPU" if world == 1 else "chunked prompt ingestion, partial rows summed across %d GPUs per chunk" % world}
    else:
        rows = pkg.f32_to_bf16(rng.normal(size=(args.ctx, cfg.head_dim)).astype(np.float32))
        kv_local = cfg.kv_heads // world
        for layer in range(cfg.kv_layer_count):
            for b in range(args.batch):
                for h in range(kv_local):
                    model.write_kv(0, layer, b, h, rows)
                    model.write_kv(1, layer, b, h, rows)
        model.set_position(args.ctx)
        tok = np.arange(1, args.batch + 1, dtype=np.int32)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput ---------------------------------------------------------------------------
    # clocks are sampled from before the warm-up until after the timed steps (nvidia-smi needs a moment to start;
    # a 128-step region alone lasts only a quarter of a second), so "under load" covers warm-up + timed region
    sampler = ClockSampler(local_rank)
    sampler.start()
    sampler.wait_first(3.0)
    model.decode_n_async(tok, warm)
    barrier()
    bursts = 0
    # same load until a few samples exist; every rank must run the same number of steps, so with several ranks
    # the count is fixed
    while (bursts < 2) if world > 1 else (sampler.count() < 4 and sampler.alive() and bursts < 8):
        model.decode_n_async(None, 64)
        barrier()
        bursts += 1
    launches0 = model.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    model.decode_n_async(None, args.steps)
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    launches = model.launches - launches0
    clocks = sampler.stop()
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    tokens = model.read_tokens(args.steps)
    if world > 1:
        # the timed computation itself: every rank must have produced the same tokens, and no exchange may have timed out
        mine = (np.asarray(tokens).reshape(-1).tolist(), pkg.tp.status(model))
        everyone = [None] * world
        dist.all_gather_object(everyone, mine)
        if any(t != everyone[0][0] or st != 0 for t, st in everyone):
            raise SystemExit("tensor-parallel ranks diverged in the timed region or an exchange timed out")
        tp_parity += "; the timed steps' tokens are identical on all ranks"

    # ---- end to end through the per-token call ----------------------------------------------------------------
    tok = tokens[-1]
    for _ in range(3):
        tok = model.decode(tok)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        tok = model.decode(tok)   # H2D token id from pinned memory, graph replay, D2H token id, synchronise
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())

    # ---- roofline of the dominant kernel: every qGEMV launch of a step, back to back ------------------------
    P = pkg.plan
    reps = 20
    wide = args.batch > 16   # one row per sequence through the tensor-core product: no per-kind timing hook there
    if wide:
        gemv_ms = attn_ms = ms / args.steps   # the whole step stands in for both
    else:
        model.profile_kind(P.STEP_QGEMV, 3)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record(stream)
        model.profile_kind(P.STEP_QGEMV, reps)
        g1.record(stream)
        barrier()
        gemv_ms = g0.elapsed_time(g1) / reps
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        model.profile_kind(P.STEP_ATTN_DECODE, 3)
        barrier()
        a0.record(stream)
        model.profile_kind(P.STEP_ATTN_DECODE, reps)
        a1.record(stream)
        barrier()
        attn_ms = a0.elapsed_time(a1) / reps

    weight_bytes = cfg.q4_weight_elems() * 0.5625 / world            # per GPU, per step
    kv_row_bytes = {"bf16": cfg.head_dim * 2, "q8": cfg.head_dim // 32 * 36}.get(args.kv, cfg.head_dim // 64 * 36)
    kv_bytes = args.batch * cfg.kv_layer_count * (cfg.kv_heads // world) * kv_row_bytes * 2 * model.position
    kv_bytes += args.batch * cfg.kv_layer_count * cfg.kv_heads * cfg.kv_qjl_dim * 2 * model.position   # projected K residuals
    n_gemv = sum(1 for l in model.describe().splitlines() if "qgemv" in l)
    kernel_name = "qgemv1_kernel" if args.batch == 1 else "qgemv_kernel"
    kernel_scope = "all %d launches of one decode step, timed back to back" % n_gemv
    if wide:
        kernel_name, kernel_scope = "qgemm_tc_kernel", "weight bytes over the WHOLE decode step; the products are not timed apart at more than 16 sequences"
    peak, peak_src = measured_peaks()
    achieved = weight_bytes / (gemv_ms * 1e-3) / 1e9
    roofline = {
        "bound": "hbm", "kernel": "%s (%s)" % (kernel_name, kernel_scope),
        "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
        "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
        "bytes_per_launch_avg": weight_bytes / n_gemv, "avg_launch_us": gemv_ms * 1e3 / n_gemv,
        # dram__bytes_read.sum + dram__bytes_write.sum over algorithmic bytes, from an ncu capture of one layer's four
        # product shapes (123.68 MB of HBM traffic for 122.68 MB of weights), applied to this run's average launch:
        # an estimate carried over from that capture, not a counter read in this run
        "traffic": weight_bytes / n_gemv * NCU_TRAFFIC_RATIO,
        "traffic_source": "estimate: ncu capture of the four product shapes of one layer, ratio %.4f to algorithmic bytes" % NCU_TRAFFIC_RATIO,
        "attention": {"kernel": "attn_split_kernel" if args.kv == "bf16" else "attn_q8_split_kernel", "bytes_per_step": kv_bytes,
                      "achieved": kv_bytes / (attn_ms * 1e-3) / 1e9, "unit": "GB/s"},
        "whole_step": {"weight_bytes": weight_bytes, "weight_GBs": weight_bytes / (ms / args.steps * 1e-3) / 1e9,
                       "weight_plus_kv_GBs": (weight_bytes + kv_bytes) / (ms / args.steps * 1e-3) / 1e9,
                       "frac_of_measured_peak_weights_only": weight_bytes / (ms / args.steps * 1e-3) / 1e9 / peak,
                       "frac_of_nominal_8TBs_weights_only": weight_bytes / (ms / args.steps * 1e-3) / 1e9 / NOMINAL_HBM_GBS},
    }

    base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        base = cpu_baseline(pkg, builder, weights, cfg, args.cpu_sample_steps, args.ctx)

    if rank == 0:
        value = args.steps * args.batch / (ms * 1e-3)
        line = {
            "metric": metric_name(args), "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 activations, fp32 accumulate, 4-bit weights",
            "data": "synthetic (seeded random-init weights of the named shape; KV context: %s)" % args.prefill,
            "config": {"workload": workload_name(args), "parallelism": "tp%d" % world if world > 1 else "single GPU",
                       "l2": "inputs larger than L2: %.2f GB of weights streamed per step" % (weight_bytes / 1e9),
                       "launches_per_step": model.launches_per_step, "context_at_end": model.position},
            "e2e": {"value": args.steps * args.batch / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 4 * args.batch, "d2h_bytes_per_step": 4 * args.batch},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": roofline,
            "cpu_baseline": base,
            "prefill": prefill_info,
        }
        if tp_parity:
            line["tp_parity"] = tp_parity
        print(json.dumps(line))
    model.close()
    store.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
