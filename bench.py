"""Benchmark of the INT8 paged decode attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (per GPU): one attention layer of Qwen2.5-7B geometry (28 q heads, 4 kv heads, head_dim 128, block 16),
128 requests x 32768 context, q_len 1, int8 K/V with static per-channel scales, pages randomly permuted;
synthetic seeded data (no dataset or checkpoint involved). A step is one pass of the decode-attention path over
the batch. The metric is the KV bytes the kernel must read (sum L * Hkv * D * 2) per second, summed over GPUs;
microseconds per call and decode tokens/s (requests per step / time) are reported beside it.
Requests are sharded over GPUs (each rank owns its requests and their pages): weak scaling, no collective in
the data path.

One JSON line is printed by rank 0. `--impl reference` times the CPU restatement of the reference's PyTorch
implementation B (oracle/) on the host cores instead, on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "int8-kvcache_b200"))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

BATCH, CTX = 128, 32768
HQ, HKV, D, BLOCK = 28, 4, 128, 16
METRIC = "int8_paged_decode_attention_kv_bandwidth_128x32k"
UNIT = "GB/s"
H100_PUBLISHED_GBS = 2439.0   # reference's own kernel, H100, 128 x 32k (docs/tables/kernels_h100.md:53)
WORKLOAD = f"decode_attention {BATCH}x{CTX} per GPU, Hq{HQ}/Hkv{HKV}/D{D}/block{BLOCK}, q_len 1, int8 KV static per-channel"


def kv_bytes(seq_lens):
    return int(sum(seq_lens)) * HKV * D * 2


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (earlier measurement on this pool)"


class ClockSampler:
    """nvidia-smi in the background during the timed region: SM clock and throttle reasons."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.file,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            pass

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        self.proc.wait()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6:
                continue
            try:
                sm.append(float(parts[0])), mx.append(float(parts[1]))
            except ValueError:
                continue
            reasons.update(n for n, v in zip(names, parts[2:]) if v == "Active")
        os.unlink(self.file.name)
        if not sm:
            return None
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's implementation B on the host cores
# --------------------------------------------------------------------------------------------------------
def cpu_sample_case(requests, seed=1002):
    """`requests` requests of the benchmark workload (same shapes and distributions), generated on the CPU."""
    from kvq_b200 import workloads

    return workloads.paged_case(seed, HQ, HKV, D, [1] * requests, [CTX] * requests, BLOCK,
                                num_blocks=requests * (CTX // BLOCK) + 1)


def cpu_run(case):
    from oracle import kvq_oracle as orc

    st = case["static"]
    args = (case["q"].float().numpy(), case["kq"].numpy(), case["vq"].numpy(), case["cu_seqlens_q"].numpy(),
            case["seq_lens"].numpy(), case["block_table"].numpy(), case["softmax_scale"], st["k_scale"].numpy(),
            st["v_scale"].numpy())
    t0 = time.perf_counter()
    orc.paged_static_attention(*args, short_q=8, p_tile=32)
    return time.perf_counter() - t0


def cpu_baseline(requests=16, repeats=3):
    case = cpu_sample_case(requests)
    cpu_run(case)                                   # warm-up (BLAS thread pool, page faults)
    t = min(cpu_run(case) for _ in range(repeats))
    return {"value": kv_bytes([CTX] * requests) / t / 1e9, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
            "sample": f"{requests} of the {BATCH} requests (x{CTX} context), numpy port of kvq/int8_ref.py "
                      f"implementation B, BLAS threads = all cores, best of {repeats}",
            "seconds_per_sample": t}


def run_reference_arm(args, rank):
    if rank != 0:
        return
    requests = 8
    case = cpu_sample_case(requests)
    for _ in range(args.warmup):
        cpu_run(case)
    times = [cpu_run(case) for _ in range(args.steps)]
    t = sum(times) / len(times)
    value = kv_bytes([CTX] * requests) / t / 1e9
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 (int32 accumulate), fp32 softmax", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sample": f"each step = {requests} of the {BATCH} requests on the host CPU"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                             "sample": f"{requests} requests x {CTX} context per step; oracle/kvq_oracle.py (numpy "
                                       "restatement of kvq/int8_ref.py implementation B; the reference is Python and "
                                       "is not present on the GPU box)"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------------
def run_ours(args, rank, world, local_rank):
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from kvq_b200 import _native
    from kvq_b200 import cuda_kernels as ck
    from kvq_b200 import workloads

    lib = ck.ext()   # raises if the native library is missing: there is no fallback path
    batch, ctx = args.batch, args.ctx
    q_len = args.q_len
    ctx_range = (args.ctx_min, ctx) if args.ctx_min else None
    case = workloads.decode_batch_on_device(batch, ctx, dev, seed=1002 + rank, q_len=q_len, ctx_range=ctx_range)
    q, kq, vq, st = case["q"], case["kq"], case["vq"], case["static"]
    cu, sl, bt = case["cu_seqlens_q"], case["seq_lens"], case["block_table"]
    scale = case["softmax_scale"]
    out = torch.empty_like(q)
    bytes_per_step = kv_bytes(case["seq_lens_list"])

    def step():
        ck.decode_attention(q, kq, vq, out, cu, sl, bt, scale, st, max_query_len=q_len)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warmup = args.warmup if args.profile else max(args.warmup, 3)
    for _ in range(warmup):
        step()
    sync_all()
    assert ck.decode_status(dev) == 0, "attention kernel reported an expired wait"

    # ---- timed region: K steps, device events; a second pair of events per step brackets the main kernel ----
    def new_event():
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    k_start = [new_event() for _ in range(args.steps)]
    k_stop = [new_event() for _ in range(args.steps)]
    t_start, t_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    t_start.record()
    for i in range(args.steps):
        lib.kvq_debug_kernel_events(k_start[i].cuda_event, k_stop[i].cuda_event)
        step()
    t_stop.record()
    sync_all()
    lib.kvq_debug_kernel_events(None, None)
    elapsed_ms = t_start.elapsed_time(t_stop)
    kernel_ms = [a.elapsed_time(b) for a, b in zip(k_start, k_stop)]
    if sampler is not None and elapsed_ms < 1500 and not args.profile:   # keep the sampler alive long enough to see loaded clocks
        t_end = time.time() + 1.5
        while time.time() < t_end:
            step()
        torch.cuda.synchronize()
    clocks = sampler.stop() if sampler is not None else None

    if args.profile:   # profiling runs (ncu): kernel timings only
        print(json.dumps({"profile_run": True, "batch": batch, "ctx": ctx, "q_len": q_len, "ctx_min": args.ctx_min, "kernel_us": [k * 1e3 for k in kernel_ms],
                          "GBps": [bytes_per_step / (k * 1e-3) / 1e9 for k in kernel_ms]}), flush=True)
        return
    # ---- end to end through the public API with host buffers ----
    hk = torch.randn(batch, HKV, D).to(torch.bfloat16).pin_memory()
    hv = torch.randn(batch, HKV, D).to(torch.bfloat16).pin_memory()
    hq = q.cpu().pin_memory()
    last = sl.cpu().long() - 1
    h_slots = (bt.cpu().long()[torch.arange(batch), last // BLOCK] * BLOCK + last % BLOCK).pin_memory()
    h_cu, h_sl, h_bt = cu.cpu().pin_memory(), sl.cpu().pin_memory(), bt.cpu().pin_memory()
    h_out = torch.empty(q.shape, dtype=q.dtype).pin_memory()
    # all host inputs of a step live in ONE pinned staging buffer, mirrored by one device buffer: one H2D copy
    host_inputs = {"q": hq, "k": hk, "v": hv, "slots": h_slots, "cu": h_cu, "sl": h_sl, "bt": h_bt}
    offsets, total = {}, 0
    for name, t in host_inputs.items():
        offsets[name] = total
        total += (t.numel() * t.element_size() + 255) // 256 * 256
    h_stage = torch.empty(total, dtype=torch.uint8).pin_memory()
    d_stage = torch.empty(total, dtype=torch.uint8, device=dev)

    def view(buf, name):
        t = host_inputs[name]
        n = t.numel() * t.element_size()
        return buf[offsets[name]:offsets[name] + n].view(t.dtype).view(t.shape)

    for name, t in host_inputs.items():
        view(h_stage, name).copy_(t)
    d_q, d_k, d_v, d_slots, d_cu, d_sl, d_bt = (view(d_stage, n) for n in ("q", "k", "v", "slots", "cu", "sl", "bt"))
    h2d = total
    d2h = h_out.numel() * h_out.element_size()

    def e2e_step():
        d_stage.copy_(h_stage, non_blocking=True)
        ck.quant_reshape_and_cache(d_k, d_v, kq, vq, d_slots, st)
        ck.paged_attention(d_q, kq, vq, out, d_cu, d_sl, d_bt, 1, scale, st)
        h_out.copy_(out, non_blocking=True)
        torch.cuda.synchronize()      # the caller needs the result on the host

    for _ in range(3):
        e2e_step()
    sync_all()
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    for _ in range(args.steps):
        e2e_step()
    e_stop.record()
    sync_all()
    e2e_ms = e_start.elapsed_time(e_stop)

    if world > 1:
        t = torch.tensor([elapsed_ms, e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms = float(t[0]), float(t[1])
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    ms_per_step = elapsed_ms / args.steps
    value = world * bytes_per_step / (ms_per_step * 1e-3) / 1e9
    peak, peak_src = peaks()
    k_ms = float(np.mean(kernel_ms))
    achieved = bytes_per_step / (k_ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / H100_PUBLISHED_GBS,
        "vs_baseline_note": "reference's own CUDA kernel on H100, 2439 GB/s (published; no B200 number exists)",
        "dtype": "int8 (int32 accumulate), fp32 softmax", "data": "synthetic",
        "config": {"workload": WORKLOAD if (batch, ctx) == (BATCH, CTX) else f"decode_attention {batch}x{ctx} per GPU (non-headline size)", "global_requests": batch * world, "sharding": f"requests over {world} GPU(s)",
                   "l2": "inputs (4.3 GB of KV per step) are larger than L2", "timed_call": "cuda_kernels.decode_attention"},
        "us_per_call": ms_per_step * 1e3, "decode_tok_per_s": batch * world / (ms_per_step * 1e-3),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": peak_src, "frac_of_nominal_8TBs": achieved / 8000.0, "kernel": "decode_kernel<128,false>",
                     "kernel_us": k_ms * 1e3, "algorithmic_bytes_per_launch": bytes_per_step,
                     "traffic": TRAFFIC_16X32K * batch // 16 if ctx == CTX else None,
                     "traffic_source": "ncu capture of 16x32768 scaled by requests (profiles/)"},
        "e2e": {"value": world * bytes_per_step / (e2e_ms / args.steps * 1e-3) / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "us_per_step": e2e_ms / args.steps * 1e3,
                "path": "pinned host staging buffer (q, new K/V, slots, metadata) -> one H2D copy -> quant_reshape_and_cache -> paged_attention -> "
                        "D2H of the output; the KV cache itself is resident state"},
        "gpu_launches": args.steps * 3,
        "clocks": clocks,
    }
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------------------------
# --suite kernels: every kernel of the path on the other benchmark configurations (one JSON line each)
# --------------------------------------------------------------------------------------------------------
def run_suite(args):
    """Steady-state device time per call of every kernel on the path. Each case builds N independent copies of
    its buffers (N x footprint >= 256 MB = 2x L2, so every call finds its data in DRAM), captures the N calls
    back to back in one CUDA graph and reports replay time / N: launch latency overlaps the previous call, as it
    does inside a model step."""
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    from kvq_b200 import cuda_kernels as ck
    from kvq_b200 import workloads

    peak, _ = peaks()

    def copies(footprint):
        return max(1, min(64, -(-(256 << 20) // footprint)))

    def timed(fns, reps=10):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for fn in fns:
                fn()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for fn in fns:
                fn()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3 / len(fns))
        return float(np.median(ts))

    def emit(kernel, workload, us, nbytes, n, **extra):
        print(json.dumps({"suite": "kernels", "kernel": kernel, "workload": workload, "us": round(us, 2),
                          "algorithmic_bytes": nbytes, "GBps": round(nbytes / us / 1e3, 1),
                          "frac_of_measured_peak": round(nbytes / us / 1e3 / peak, 3),
                          "timing": f"{n} independent copies back to back in one CUDA graph, replay time / {n}, median of 10",
                          **extra}), flush=True)

    st = None
    # fused quantize + cache write (config 1 = 8192 tokens)
    for T in (64, 256, 2048, 8192):
        nbytes = T * (HKV * D * 6 + 8)
        n = copies(nbytes)
        c = workloads.write_case(1001, T * n, HKV, D, num_blocks=max(4096, T * n // BLOCK * 2), block_size=BLOCK, smooth=False)
        st = {k: v.to(dev) for k, v in c["static"].items()}
        key, value, slots = c["key"].to(dev), c["value"].to(dev), c["slots"].to(dev)
        kc = torch.zeros(c["num_blocks"], BLOCK, HKV, D, dtype=torch.int8, device=dev)
        vc = torch.zeros_like(kc)
        fns = [(lambda i=i: ck.quant_reshape_and_cache(key[i * T:(i + 1) * T], value[i * T:(i + 1) * T], kc, vc,
                                                       slots[i * T:(i + 1) * T], st)) for i in range(n)]
        emit("quant_cache_kernel", f"{T} tokens x {HKV} x {D} K and V, random slots", timed(fns), nbytes, n)
        del key, value, kc, vc
    # page dequantization (config 1 round trip = 512 pages)
    for P in (512, 8192):
        nbytes = P * BLOCK * HKV * D * 2 * 3
        n = copies(nbytes)
        kc = torch.randint(-127, 128, (P * n, BLOCK, HKV, D), dtype=torch.int8, device=dev)
        vc = torch.randint(-127, 128, (P * n, BLOCK, HKV, D), dtype=torch.int8, device=dev)
        ko = torch.empty(n, P, BLOCK, HKV, D, dtype=torch.bfloat16, device=dev)
        vo = torch.empty_like(ko)
        ids = torch.randperm(P * n, device=dev).to(torch.int32).view(n, P)
        zero, idx = torch.zeros(P, dtype=torch.int32, device=dev), torch.arange(P, dtype=torch.int32, device=dev)
        fns = [(lambda i=i: ck.dequant_pages(kc, vc, ko[i], vo[i], ids[i:i + 1], zero, idx, st)) for i in range(n)]
        emit("dequant_pages_kernel", f"{P} pages x {BLOCK} x {HKV} x {D}, K and V", timed(fns), nbytes, n)
        del kc, vc, ko, vo
    # calibration statistics of one step's new rows (the reference's hook does eight torch reductions per step)
    from kvq_b200 import capture
    for T in (256, 8192):
        nbytes = T * HKV * D * 2 * 2
        n = copies(nbytes)
        key = torch.randn(n, T, HKV, D, device=dev).to(torch.bfloat16)
        value = torch.randn(n, T, HKV, D, device=dev).to(torch.bfloat16)
        capture.reset()
        capture.MAX_SAMPLE_TOKENS, keep = 0, capture.MAX_SAMPLE_TOKENS   # statistics only: no host-side row sampling
        fns = [(lambda i=i: capture.record("layer", key[i], value[i])) for i in range(n)]
        us = timed(fns)
        capture.MAX_SAMPLE_TOKENS = keep

        def torch_reductions(i):
            for x in (key[i], value[i]):
                xf = x.float()
                xf.abs().amax(0), xf.amax(0), xf.amin(0), xf.double().sum(0)

        emit("calib_stats_kernel", f"{T} tokens x {HKV} x {D} K and V", us, nbytes, n,
             torch_reductions_us=round(timed([(lambda i=i: torch_reductions(i)) for i in range(n)]), 2))
        del key, value
    # standalone q quantization through the C ABI (the Python wrapper would add two allocations per call)
    lib = ck.ext()
    for T in (128, 2048):
        nbytes = T * HQ * D * 3 + T * HQ * 4
        n = copies(nbytes)
        q = torch.randn(n, T, HQ, D, device=dev).to(torch.bfloat16)
        qi = torch.empty(n, T, HQ, D, dtype=torch.int8, device=dev)
        qs = torch.empty(n, T, HQ, 1, dtype=torch.float32, device=dev)
        fns = [(lambda i=i: lib.kvq_quant_q(q[i].data_ptr(), st["k_scale"].data_ptr(), qi[i].data_ptr(), qs[i].data_ptr(),
                                            T, HQ, HKV, D, 128, HQ * D, D, 1, torch.cuda.current_stream().cuda_stream))
               for i in range(n)]
        emit("quant_q_kernel<128>", f"{T} tokens x {HQ} heads", timed(fns), nbytes, n)
        del q, qi, qs

    def attention_case(name, batch, ctx, q_len=1, ctx_range=None, seed=5, **extra):
        per = batch * (ctx if ctx_range is None else (ctx_range[0] + ctx_range[1]) // 2) * HKV * D * 2
        n = copies(per)
        c = workloads.decode_batch_on_device(batch * n, ctx, dev, seed=seed, q_len=q_len, ctx_range=ctx_range)
        out = torch.empty_like(c["q"])
        cu = torch.arange(0, (batch + 1) * q_len, q_len, dtype=torch.int32, device=dev)
        rows = batch * q_len

        def call(i):
            ck.decode_attention(c["q"][i * rows:(i + 1) * rows], c["kq"], c["vq"], out[i * rows:(i + 1) * rows], cu,
                                c["seq_lens"][i * batch:(i + 1) * batch], c["block_table"][i * batch:(i + 1) * batch],
                                c["softmax_scale"], c["static"], max_query_len=q_len)

        us = timed([(lambda i=i: call(i)) for i in range(n)])
        emit("decode_attention (plan + decode + merge)", name, us, kv_bytes(c["seq_lens_list"]) // n, n, **extra)

    for batch, ctx in ((1, 32768), (8, 32768), (32, 32768), (64, 4096), (128, 4096), (256, 1024)):
        attention_case(f"{batch} x {ctx}, q_len 1", batch, ctx)
    attention_case("config 3: 256 requests, q_len 8, ctx U[1024, 8192]", 256, 0, q_len=8, ctx_range=(1024, 8192), seed=1003,
                   note="KV bytes counted once although 4 m tiles (56 rows) use them; average over the copies")


def run_prefill_suite(args):
    """Long-query attention (more than SHORT_Q query tokens per request) on the INT8 cache, both routes: the
    INT8-page tensor-core kernel (prefill_attention) and the reference's route (dequantize pages to a temporary
    bf16 cache + vLLM's paged FlashAttention, a library kernel). Tensor-bound: TFLOP/s = 4 * rows * visible keys
    * head_dim / time, against the measured dense bf16 peak. K/V (>= 130 MB per case except the smallest) are read
    through L2 many times by design, so no L2 flush applies."""
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    from kvq_b200 import cuda_kernels as ck
    from kvq_b200 import workloads

    try:
        peak_tf = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]
        peak_src = "measured"
    except Exception:  # noqa: BLE001
        peak_tf, peak_src = 1590.0, "fallback"

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return float(np.median(ts))

    for batch, q_len, ctx in ((16, 64, 4096), (32, 512, 512), (8, 4096, 4096), (4, 2048, 8192), (1, 16384, 16384)):
        c = workloads.decode_batch_on_device(batch, ctx, dev, seed=1005, q_len=q_len)
        q, cu, sl, bt, st = c["q"], c["cu_seqlens_q"], c["seq_lens"], c["block_table"], c["static"]
        out = torch.zeros_like(q)
        flops = 4.0 * batch * HQ * D * (q_len * (ctx - q_len) + q_len * (q_len + 1) / 2)
        ms = timed(lambda: ck.prefill_attention(q, c["kq"], c["vq"], out, cu, sl, bt, c["softmax_scale"], st))
        assert ck.prefill_status() == 0
        line = {"suite": "prefill", "workload": f"{batch} requests x {q_len} query tokens, context {ctx}",
                "kernel": "prefill_ws_kernel (INT8 pages, tcgen05)", "ms": round(ms, 4),
                "TFLOPs": round(flops / ms / 1e9, 1), "frac_of_bf16_peak": round(flops / ms / 1e9 / peak_tf, 3),
                "peak": f"{peak_tf} TFLOP/s dense bf16 ({peak_src})", "timing": "CUDA events, median of 10 calls after 3 warm-ups"}
        try:
            plan = ck.plan_long(cu.cpu(), sl.cpu(), BLOCK)
            out2 = torch.zeros_like(q)
            ms2 = timed(lambda: ck.long_attention(q, c["kq"], c["vq"], out2, cu, sl, bt, q_len, plan, c["softmax_scale"], st))
            line["dequant_plus_flash_attention_ms"] = round(ms2, 4)
            line["dequant_plus_flash_attention_TFLOPs"] = round(flops / ms2 / 1e9, 1)
            line["rel_l2_between_routes"] = round(float((out.float() - out2.float()).norm() / out2.float().norm()), 5)
        except Exception as e:  # noqa: BLE001  (vLLM's kernel is optional)
            line["dequant_plus_flash_attention_ms"] = None
            line["flash_attention_unavailable"] = str(e)[:120]
        print(json.dumps(line), flush=True)
        del c, q, out


# --------------------------------------------------------------------------------------------------------
# --workload model_step: full decode step of a Qwen2.5-7B-geometry decoder (a caller of the hot path)
# --------------------------------------------------------------------------------------------------------
def run_model_step(args, rank, world, local_rank):
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from kvq_b200.decode_step import DecodeStep

    total_requests, ctx = args.model_requests, args.model_ctx
    batch = total_requests // world
    model = DecodeStep(dev, batch, ctx, seed=rank).capture()

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        model.step()
    sync_all()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        model.step()
    b.record()
    sync_all()
    ms = a.elapsed_time(b)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    if rank == 0:
        tpot = ms / args.steps
        print(json.dumps({
            "workload": "model_step", "metric": "decode_tokens_per_s", "value": batch * world / (tpot * 1e-3), "unit": "tok/s",
            "tpot_ms": tpot, "n_gpus": world, "steps": args.steps, "scaling": "strong (fixed 512 requests)" if world > 1 else "n/a",
            "config": {"model": "Qwen2.5-7B geometry, random-init bf16 weights, vocab 152064", "requests": batch * world,
                       "requests_per_gpu": batch, "context": ctx, "kv_cache": "int8_static paged, block 16",
                       "parallelism": f"requests sharded over {world} GPU(s), weights replicated"},
            "kv_bytes_per_step_per_gpu": model.kv_bytes_per_step(), "weight_bytes_per_gpu": model.weight_bytes(),
            "data": "synthetic"}), flush=True)
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one decode_kernel launch, from the ncu capture summarised in
# profiles/decode_kernel_16x32k_ncu_full.md: 541,588,224 bytes for 16 requests x 32768 context. Traffic is
# proportional to the requests (every CTA streams its slice of the KV bytes once), so it is scaled to the batch.
TRAFFIC_16X32K = 537_499_392 + 4_088_832


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--batch", type=int, default=BATCH, help="requests per GPU (default: the headline 128)")
    ap.add_argument("--ctx", type=int, default=CTX, help="context length (default: the headline 32768)")
    ap.add_argument("--workload", default="attention", choices=["attention", "model_step"],
                    help="model_step: full 28-layer decode step (512 requests x 6144 context over all GPUs)")
    ap.add_argument("--model-requests", type=int, default=512)
    ap.add_argument("--model-ctx", type=int, default=6144)
    ap.add_argument("--suite", default=None, choices=["kernels", "prefill"],
                    help="extra per-kernel lines instead of the headline (prefill: long-query attention, both routes)")
    ap.add_argument("--q-len", type=int, default=1, help="query tokens per request (profile runs; headline is 1)")
    ap.add_argument("--ctx-min", type=int, default=0, help="draw contexts uniformly from [ctx-min, ctx] (profile runs)")
    ap.add_argument("--profile", action="store_true", help="kernel timings only, exact --warmup (for ncu captures)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        if args.steps == 20 and args.warmup == 5:
            args.steps, args.warmup = 5, 3
        run_reference_arm(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA GPU (there is no CPU path for the product arm)")
    if args.workload == "model_step":
        run_model_step(args, rank, world, local_rank)
        return
    if args.suite == "kernels":
        run_suite(args)
        return
    if args.suite == "prefill":
        run_prefill_suite(args)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
