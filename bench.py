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

One JSON line is printed by rank 0. Beside the headline it carries: `roofline` (the main kernel against the
measured HBM copy rate), `e2e` (the same step from pinned host buffers through the public API), `output_check` (8 of
the timed batch's requests recomputed by the CPU oracle after the timed loop), `strong` (the fixed 128 x 32k layer
sharded 128/N requests per GPU with the NCCL all-gather of the outputs inside the timed step), `model_step` (the
28-layer decode step of benchmark configuration 4 with 512/N requests per GPU) and, at N = 1, `cpu_baseline`.

`--impl reference` times the reference's own PyTorch implementation B on the host cores instead (oracle/_ref, staged
by oracle/build_ref.py; the numpy restatement in oracle/ where that is absent), each step a bounded sample of the
same workload.
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
    return 6650.0, "fallback (no MEASURED_PEAKS.json next to bench.py)"


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
CPU_SAMPLE_REQUESTS = 8     # requests of the 128 that one CPU step computes (both CPU legs use this sample)


def cpu_sample_case(requests=CPU_SAMPLE_REQUESTS, seed=1002):
    """`requests` requests of the benchmark workload (same shapes and distributions), generated on the CPU."""
    from kvq_b200 import workloads

    return workloads.paged_case(seed, HQ, HKV, D, [1] * requests, [CTX] * requests, BLOCK,
                                num_blocks=requests * (CTX // BLOCK) + 1)


def cpu_runner(case):
    """(fn, kind, description): fn() computes the sample once on the host cores and returns seconds.
    kind "reference": the reference's own PyTorch implementation B (kvq/int8_ref.py paged_static_attention with
    Cfg(p_tile=32), byte-compiled into oracle/_ref by oracle/build_ref.py), torch threads = all cores.
    kind "port": the numpy restatement in oracle/kvq_oracle.py, where oracle/_ref is absent."""
    from oracle import build_ref

    st = case["static"]
    mods = build_ref.load()
    if mods is not None:
        _, _, int8_ref = mods
        torch.set_num_threads(os.cpu_count())
        fn = int8_ref.paged_static_attention(int8_ref.Cfg(p_tile=32), st, cache_is_int8=True, short_q=8)
        args = (case["q"].float(), case["kq"], case["vq"], case["cu_seqlens_q"], case["seq_lens"], case["block_table"],
                case["softmax_scale"])

        def run():
            t0 = time.perf_counter()
            fn(*args)
            return time.perf_counter() - t0

        return run, "reference", ("the reference's PyTorch implementation B (kvq/int8_ref.py, p_tile 32) from oracle/_ref, "
                                  f"torch threads = {torch.get_num_threads()}")
    from oracle import kvq_oracle as orc

    args = (case["q"].float().numpy(), case["kq"].numpy(), case["vq"].numpy(), case["cu_seqlens_q"].numpy(),
            case["seq_lens"].numpy(), case["block_table"].numpy(), case["softmax_scale"], st["k_scale"].numpy(),
            st["v_scale"].numpy())

    def run():
        t0 = time.perf_counter()
        orc.paged_static_attention(*args, short_q=8, p_tile=32)
        return time.perf_counter() - t0

    return run, "port", "numpy restatement of kvq/int8_ref.py implementation B (oracle/kvq_oracle.py; oracle/_ref absent)"


def cpu_baseline(repeats=5):
    """The CPU leg of the GPU arm's line: same sample and same statistic (mean) as `--impl reference`."""
    case = cpu_sample_case()
    run, kind, what = cpu_runner(case)
    run()                                   # warm-up (thread pool, page faults)
    t = float(np.mean([run() for _ in range(repeats)]))
    return {"value": kv_bytes([CTX] * CPU_SAMPLE_REQUESTS) / t / 1e9, "unit": UNIT, "cores": os.cpu_count(), "kind": kind,
            "sample": f"{CPU_SAMPLE_REQUESTS} of the {BATCH} requests (x{CTX} context) per step, mean of {repeats} steps; {what}",
            "seconds_per_sample": t}


REFERENCE_ARM_BUDGET_S = 240.0   # wall-time bound of the whole CPU arm


def run_reference_arm(args, rank):
    """--steps / --warmup are honoured; only if the run would exceed REFERENCE_ARM_BUDGET_S of wall time are the
    timed steps cut short, and the line then says how many ran."""
    if rank != 0:
        return
    requests = CPU_SAMPLE_REQUESTS
    case = cpu_sample_case(requests)
    run, kind, what = cpu_runner(case)
    t_begin = time.perf_counter()
    for _ in range(args.warmup):
        run()
    times = []
    for _ in range(args.steps):
        times.append(run())
        if time.perf_counter() - t_begin > REFERENCE_ARM_BUDGET_S and len(times) >= 3:
            break
    t = sum(times) / len(times)
    value = kv_bytes([CTX] * requests) / t / 1e9
    sample = f"each step = {requests} of the {BATCH} requests (x{CTX} context) on the host CPU; {what}"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": len(times),
            "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 (int32 accumulate), fp32 softmax", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sample": sample},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": os.cpu_count(), "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    if len(times) < args.steps:
        line["steps_requested"] = args.steps
        line["steps_note"] = f"stopped after {len(times)} steps: wall-time bound of {REFERENCE_ARM_BUDGET_S:.0f} s for the CPU arm"
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------------
def output_check(case, out_ref, ck, rank, picks=8):
    """After the timed loop: `picks` requests of the timed batch (first, last and a seeded sample) are run once more
    through decode_attention as a batch of their own and recomputed by the CPU oracle from the very pages the
    kernel read (pulled from HBM through the block table). Bar: max-abs 1e-2, mean-abs 1e-3 against the fp32 oracle."""
    from oracle import kvq_oracle as orc

    n_req = len(case["q_lens"])
    rng = np.random.default_rng(1002)
    sel = sorted({0, n_req - 1, *rng.choice(n_req, size=min(picks, n_req), replace=False).tolist()})[:picks]
    q_len = case["q_lens"][0]
    cu_all = case["cu_seqlens_q"].cpu().numpy()
    seq = case["seq_lens"].cpu().numpy()
    rows = np.concatenate([np.arange(cu_all[r], cu_all[r + 1]) for r in sel])
    idx = torch.as_tensor(sel, device=case["q"].device)
    q_sel = case["q"][torch.as_tensor(rows, device=case["q"].device)].contiguous()
    out_sel = torch.zeros_like(q_sel)
    cu_sel = torch.arange(0, (len(sel) + 1) * q_len, q_len, dtype=torch.int32, device=q_sel.device)
    ck.decode_attention(q_sel, case["kq"], case["vq"], out_sel, cu_sel, case["seq_lens"][idx].contiguous(),
                        case["block_table"][idx].contiguous(), case["softmax_scale"], case["static"], max_query_len=q_len)
    torch.cuda.synchronize()
    got = out_sel.float().cpu().numpy()
    st = {k: v.cpu().numpy() for k, v in case["static"].items()}
    bs = case["kq"].shape[1]
    worst = {"max_abs": 0.0, "mean_abs": 0.0}
    for i, r in enumerate(sel):
        L = int(seq[r])
        pages = case["block_table"][r, :(L + bs - 1) // bs].long()
        k_r, v_r = case["kq"][pages].cpu().numpy(), case["vq"][pages].cpu().numpy()      # [pages, bs, H, D]
        bt_r = np.arange(k_r.shape[0], dtype=np.int32)[None]
        ref = orc.paged_static_attention(q_sel[i * q_len:(i + 1) * q_len].float().cpu().numpy(), k_r, v_r,
                                         np.array([0, q_len]), np.array([L]), bt_r, case["softmax_scale"],
                                         st["k_scale"], st["v_scale"])
        err = orc.compare(ref, got[i * q_len:(i + 1) * q_len])
        worst = {k: max(worst[k], err[k]) for k in worst}
    ok = worst["max_abs"] <= 1e-2 and worst["mean_abs"] <= 1e-3
    if not ok:
        raise SystemExit(f"bench.py: output check failed on requests {sel}: {worst}")
    return {"requests": sel, "max_abs": worst["max_abs"], "mean_abs_worst_request": worst["mean_abs"],
            "bar": "max-abs 1e-2, mean-abs 1e-3 vs the fp32 CPU oracle", "ok": True}


def run_ours(args, rank, world, local_rank):
    dev = torch.device("cuda", local_rank)
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

    # ---- strong scaling: the FIXED headline layer (128 requests in total) sharded 128 / N requests per GPU, with the
    #      NCCL all-gather of every rank's output rows inside the timed step ----
    strong, strong_error = None, None
    collective, strong_graphed = "none (one GPU)", False
    try:
        if (batch, ctx, q_len) == (BATCH, CTX, 1) and BATCH % world == 0:
            from kvq_b200 import sharding

            n = BATCH // world
            q_n, out_n, cu_n, sl_n, bt_n = q[:n], out[:n], cu[:n + 1], sl[:n], bt[:n]
            gathered = torch.empty(BATCH, HQ, D, dtype=out.dtype, device=dev) if world > 1 else None
            # the gather: this library's peer-store kernel over NVLink where symmetric memory is available, else NCCL
            peer, collective = None, "none (one GPU)"
            if world > 1:
                collective = f"NCCL all_gather of [{n}, {HQ}, {D}] bf16 output rows per rank inside the timed step"
                try:
                    if os.environ.get("KVQ_GATHER", "peer") == "peer":
                        peer = sharding.PeerGather(n, (HQ, D), out.dtype, dev)
                        collective = (f"kvq_peer_allgather: every rank stores its [{n}, {HQ}, {D}] bf16 output rows into every "
                                      "peer's buffer over NVLink and waits for the peers' flags, inside the timed step")
                except Exception as e:   # no symmetric memory on this box: the library route
                    peer = None
                    collective += f" (peer route unavailable: {type(e).__name__})"
                agreed = torch.tensor([1 if peer is not None else 0], device=dev)
                dist.all_reduce(agreed, op=dist.ReduceOp.MIN)   # every rank takes the same route
                if int(agreed.item()) == 0 and peer is not None:
                    peer = None
                    collective = (f"NCCL all_gather of [{n}, {HQ}, {D}] bf16 output rows per rank inside the timed step "
                                  "(peer route unavailable on another rank)")
            out_c = out_n.contiguous()

            def strong_step():
                ck.decode_attention(q_n, kq, vq, out_c, cu_n, sl_n, bt_n, scale, st, max_query_len=1)
                if peer is not None:
                    peer.gather(out_c)
                elif world > 1:
                    sharding.gather_outputs(out_c, [n] * world, out=gathered)

            for _ in range(3):
                strong_step()
            sync_all()
            # one step = one CUDA graph replay (attention call + gather), as a serving engine would run a decode step
            run_step, strong_graphed = strong_step, False
            if os.environ.get("KVQ_STRONG_GRAPH", "1") == "1":
                try:
                    side = torch.cuda.Stream()
                    side.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(side):
                        strong_step()
                    torch.cuda.current_stream().wait_stream(side)
                    sgraph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(sgraph):
                        strong_step()
                    run_step, strong_graphed = sgraph.replay, True
                except Exception:   # capture not possible here (e.g. the collective): eager steps
                    torch.cuda.synchronize()
            for _ in range(2):
                run_step()
            sync_all()
            s_start, s_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s_start.record()
            for _ in range(args.steps):
                run_step()
            s_stop.record()
            sync_all()
            strong = s_start.elapsed_time(s_stop)
            if peer is not None:
                peer.check()   # raises if a wait for a peer's rows ran out
    except Exception as e:   # the headline line is still printed; the record says what happened
        strong, strong_error = None, f"{type(e).__name__}: {e}"[:300]
        torch.cuda.synchronize()

    # ---- output check: a seeded subset of the timed batch recomputed by the CPU oracle ----
    check = None
    if rank == 0 and not args.no_check:
        try:
            check = output_check(case, out_ref=None, ck=ck, rank=rank)
        except Exception as e:   # the checker failing to run is reported, not fatal to the measurement
            check = {"ok": False, "error": f"{type(e).__name__}: {e}"[:300]}

    if world > 1:
        t = torch.tensor([elapsed_ms, e2e_ms, strong or 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms, strong = float(t[0]), float(t[1]), (float(t[2]) if strong is not None else None)
    if rank != 0:
        return None

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
                   "l2": "inputs (4.3 GB of KV per step) are larger than L2", "timed_call": "cuda_kernels.decode_attention",
                   "scales": "analytic 4.5 sigma_c / 127 per (kv head, channel) instead of absmax / 127 over the generated "
                             "pool (no bf16 copy of the 4.3 GB pool is ever held); same int8 value distribution"},
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
    if check is not None:
        line["output_check"] = check
    if strong_error is not None:
        line["strong"] = {"error": strong_error}
    if strong is not None:
        s_ms = strong / args.steps
        line["strong"] = {
            "workload": f"the fixed {BATCH} x {CTX} layer, {BATCH // world} requests per GPU",
            "us_per_step": s_ms * 1e3, "value": BATCH * CTX * HKV * D * 2 / (s_ms * 1e-3) / 1e9, "unit": UNIT,
            "decode_tok_per_s": BATCH / (s_ms * 1e-3),
            "collective": collective, "cuda_graph": strong_graphed,
            "speedup_vs_one_gpu_step_of_this_run": ms_per_step / s_ms,
            "note": "the weak-scaling step above runs the whole 128-request layer on every GPU, so its time is this "
                    "run's one-GPU time for the fixed layer"}
    if world == 1 and not args.no_cpu:
        try:
            line["cpu_baseline"] = cpu_baseline()
        except Exception as e:   # never lose the GPU line to the CPU leg
            line["cpu_baseline"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    return line


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
def model_step_record(args, rank, world, dev, steps):
    """Benchmark configuration 4: one decode step of a 28-layer Qwen2.5-7B-geometry decoder (random bf16 weights,
    kvq_b200/decode_step.py), `--model-requests` (512) requests x `--model-ctx` (6144) context in the int8_static
    paged cache, requests sharded over the GPUs, weights replicated, no collective inside the step. Every rank
    times `steps` graph replays; the record carries the slowest rank's time."""
    from kvq_b200.decode_step import DecodeStep

    total_requests, ctx = args.model_requests, args.model_ctx
    batch = total_requests // world
    model = DecodeStep(dev, batch, ctx, seed=rank).capture()

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(3):
        model.step()
    sync_all()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        model.step()
    b.record()
    sync_all()
    ms = a.elapsed_time(b)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    kv_b, w_b = model.kv_bytes_per_step(), model.weight_bytes()
    del model
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    tpot = ms / steps
    peak, _ = peaks()
    return {"workload": "model_step", "metric": "decode_tokens_per_s", "value": batch * world / (tpot * 1e-3), "unit": "tok/s",
            "tpot_ms": tpot, "n_gpus": world, "steps": steps, "scaling": "strong (fixed total requests)",
            "config": {"model": "Qwen2.5-7B geometry, random-init bf16 weights, vocab 152064", "requests": batch * world,
                       "requests_per_gpu": batch, "context": ctx, "kv_cache": "int8_static paged, block 16",
                       "parallelism": f"requests sharded over {world} GPU(s), weights replicated, CUDA-graphed step"},
            "kv_bytes_per_step_per_gpu": kv_b, "weight_bytes_per_gpu": w_b,
            "hbm_floor_ms": (kv_b + w_b) / (peak * 1e9) * 1e3,
            "frac_of_hbm_floor": (kv_b + w_b) / (peak * 1e9) * 1e3 / tpot, "data": "synthetic"}


# --------------------------------------------------------------------------------------------------------
# --suite ref_kernel: the reference's own CUDA kernels, built for this GPU from a checkout given at run time
# --------------------------------------------------------------------------------------------------------
def run_ref_kernel_suite(args):
    """Side-by-side device times of this library and of the reference's CUDA extension (kvq/cuda/int8_kv.cu, JIT-built
    by the reference's own kvq/cuda_kernels.py:ext() from the checkout at --ref-path; nothing of it is part of this
    repository) on the same inputs: eager calls, a 256 MB L2 flush before each, median of 10. One JSON line per case,
    with the difference between the two kernels' outputs."""
    import statistics

    if not args.ref_path or not os.path.exists(os.path.join(args.ref_path, "kvq", "cuda", "int8_kv.cu")):
        print(json.dumps({"suite": "ref_kernel", "unavailable": "--ref-path must point at a checkout of the reference "
                          "(kvq/cuda/int8_kv.cu)"}), flush=True)
        return
    sys.path.insert(0, os.path.abspath(args.ref_path))
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    from kvq import cuda_kernels as rck   # the reference's module

    from kvq_b200 import cuda_kernels as ck
    from kvq_b200 import workloads

    t0 = time.time()
    rck.ext()
    build_s = round(time.time() - t0, 1)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(reps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        return statistics.median(ts)

    common = {"suite": "ref_kernel", "timing": "eager call, 256 MB L2 flush before each, CUDA events, median of 10",
              "reference_build_s": build_s}
    cases = ((128, 32768, 1, None, "headline 128 x 32768"), (16, 32768, 1, None, "16 x 32768 (one rank of 8)"),
             (1, 32768, 1, None, "1 x 32768"), (128, 4096, 1, None, "128 x 4096"),
             (256, 0, 8, (1024, 8192), "config 3: 256 requests, q_len 8, ctx U[1024, 8192]"))
    for batch, ctx, q_len, rng, name in cases:
        c = workloads.decode_batch_on_device(batch, ctx, dev, seed=1002 if q_len == 1 else 1003, q_len=q_len, ctx_range=rng)
        st = c["static"]
        out_r, out_o = torch.zeros_like(c["q"]), torch.zeros_like(c["q"])
        T = c["q"].shape[0]
        segm = None
        if batch <= 32:   # vLLM hands split-KV scratch to small batches (16 segments)
            segm = (torch.empty(T, HQ, 16, D, device=dev), torch.empty(T, HQ, 16, device=dev), torch.empty(T, HQ, 16, device=dev))
        meta = (c["cu_seqlens_q"], c["seq_lens"], c["block_table"], c["softmax_scale"], st)
        t_ref = timed(lambda: rck.decode_attention(c["q"], c["kq"], c["vq"], out_r, *meta, segm=segm, max_query_len=q_len))
        t_our = timed(lambda: ck.decode_attention(c["q"], c["kq"], c["vq"], out_o, *meta, max_query_len=q_len))
        nbytes = kv_bytes(c["seq_lens_list"])
        d = (out_r.float() - out_o.float()).abs()
        print(json.dumps(dict(common, case=name, reference_us=round(t_ref, 1), ours_us=round(t_our, 1),
                              reference_GBps=round(nbytes / t_ref / 1e3), ours_GBps=round(nbytes / t_our / 1e3),
                              speedup=round(t_ref / t_our, 2), max_abs_diff_between_kernels=float(d.max()),
                              identical_fraction=float((d == 0).float().mean()))), flush=True)
        del c, out_r, out_o
    for T in (128, 8192):
        w = workloads.write_case(1001, T, HKV, D, num_blocks=4096, smooth=False)
        st = {k: v.to(dev) for k, v in w["static"].items()}
        key, value, slots = w["key"].to(dev), w["value"].to(dev), w["slots"].to(dev)
        kc = torch.zeros(4096, BLOCK, HKV, D, dtype=torch.int8, device=dev)
        vc, kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(kc), torch.zeros_like(kc)
        t_ref = timed(lambda: rck.quant_reshape_and_cache(key, value, kc, vc, slots, st))
        t_our = timed(lambda: ck.quant_reshape_and_cache(key, value, kc2, vc2, slots, st))
        print(json.dumps(dict(common, case=f"quantize + cache write, {T} tokens", reference_us=round(t_ref, 1),
                              ours_us=round(t_our, 1), speedup=round(t_ref / t_our, 2),
                              cache_bytes_equal=bool(torch.equal(kc, kc2) and torch.equal(vc, vc2)))), flush=True)


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
    ap.add_argument("--no-check", action="store_true", help="skip the oracle check of the timed batch's outputs")
    ap.add_argument("--no-model-step", action="store_true", help="skip the model_step sub-record (configuration 4)")
    ap.add_argument("--batch", type=int, default=BATCH, help="requests per GPU (default: the headline 128)")
    ap.add_argument("--ctx", type=int, default=CTX, help="context length (default: the headline 32768)")
    ap.add_argument("--workload", default="attention", choices=["attention", "model_step"],
                    help="model_step: only the full 28-layer decode step (512 requests x 6144 context over all GPUs)")
    ap.add_argument("--model-requests", type=int, default=512)
    ap.add_argument("--model-ctx", type=int, default=6144)
    ap.add_argument("--suite", default=None, choices=["kernels", "prefill", "ref_kernel"],
                    help="extra per-kernel lines instead of the headline (prefill: long-query attention, both routes; "
                         "ref_kernel: the reference's CUDA extension built from --ref-path, side by side)")
    ap.add_argument("--ref-path", default=None, help="checkout of the reference (for --suite ref_kernel)")
    ap.add_argument("--q-len", type=int, default=1, help="query tokens per request (profile runs; headline is 1)")
    ap.add_argument("--ctx-min", type=int, default=0, help="draw contexts uniformly from [ctx-min, ctx] (profile runs)")
    ap.add_argument("--profile", action="store_true", help="kernel timings only, exact --warmup (for ncu captures)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA GPU (there is no CPU path for the product arm)")
    if args.suite == "kernels":
        run_suite(args)
        return
    if args.suite == "prefill":
        run_prefill_suite(args)
        return
    if args.suite == "ref_kernel":
        run_ref_kernel_suite(args)
        return
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.workload == "model_step":
        line = model_step_record(args, rank, world, dev, args.steps)
    else:
        line = run_ours(args, rank, world, local_rank)
        headline = (args.batch, args.ctx, args.q_len) == (BATCH, CTX, 1) and not args.profile
        if headline and not args.no_model_step and args.model_requests % world == 0:
            torch.cuda.empty_cache()
            try:
                ms = model_step_record(args, rank, world, dev, min(args.steps, 10))
            except Exception as e:   # the headline line is still printed; the record says what happened
                ms = {"workload": "model_step", "error": f"{type(e).__name__}: {e}"[:300]}
            if line is not None:
                line["model_step"] = ms
    if rank == 0 and line is not None:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
