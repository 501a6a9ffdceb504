#!/usr/bin/env python
"""Benchmark of the decode-attention hot path (split-KV flash decoding over the fp16 KV cache).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Default workload `decode_3b_L1048576`: Qwen2.5-3B attention shape (16 query / 2 kv heads, head_dim 128,
36 layers), KV length 1,048,576, fp16 KV i.i.d. N(0,1).  One STEP is the attention of one decoded token:
36 decode-attention calls, one per layer, each over that layer's own KV buffers (1 GiB per layer, 36 GiB
in all, so every call streams from HBM, never from L2).  With N GPUs the KV rows are cut into N contiguous
slices (strong scaling); each call is local partial -> exchange of the (m, l, O) records -> merge, the exchange done
by the merge kernel itself with peer stores over NVLink (--exchange nccl: NCCL all-gather instead).

The metric is KV GB/s: algorithmic KV bytes (2 * n_kv * L * head_dim * 2 B per call) per second of step time.
Prints ONE JSON line (rank 0).
"""
import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: n_head, n_kv, head_dim, layers, L
    "decode_3b_L1048576": dict(n_head=16, n_kv=2, head_dim=128, layers=36, L=1048576),
    "decode_3b_L131072": dict(n_head=16, n_kv=2, head_dim=128, layers=36, L=131072),
    "decode_7b_L32768": dict(n_head=28, n_kv=4, head_dim=128, layers=28, L=32768),
    "decode_7b_L16384": dict(n_head=28, n_kv=4, head_dim=128, layers=28, L=16384),
    "decode_7b_L4096": dict(n_head=28, n_kv=4, head_dim=128, layers=28, L=4096),
    "decode_7b_L1024": dict(n_head=28, n_kv=4, head_dim=128, layers=28, L=1024),
}
PREFILL_WORKLOADS = {
    # Llama-3-8B attention shape: one 512-token chunk at KV offset n_past, RoPE theta 5e5 (normal pairing)
    "prefill_8b_off0": dict(n_head=32, n_kv=8, head_dim=128, batch=512, n_past=0, theta=5e5, layers=32),
    "prefill_8b_off4096": dict(n_head=32, n_kv=8, head_dim=128, batch=512, n_past=4096, theta=5e5, layers=32),
    "prefill_8b_off8192": dict(n_head=32, n_kv=8, head_dim=128, batch=512, n_past=8192, theta=5e5, layers=32),
}
NCU_READ_PER_KV_BYTE = 134.272 / 134.218     # dram__bytes_read.sum / algorithmic K+V bytes of the captured launch
NCU_WRITE_BYTES_PER_LAUNCH = 4.46e6           # dram__bytes_write.sum of the captured launch
CPU_SAMPLE_L = 131072      # rows of ONE layer call the CPU baseline / reference arm processes per step


def kv_bytes(w, L=None):
    L = w["L"] if L is None else L
    return 2 * w["n_kv"] * L * w["head_dim"] * 2


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return json.load(open(p)), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


# ---------------------------------------------------------------------------------------------------
# clocks: read-only NVML sampling during the timed region
class ClockSampler:
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = None
            try:
                import torch
                uuid = str(torch.cuda.get_device_properties(index).uuid)
                self.h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self._reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                mask = self._reasons_fn(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.005)

    def start(self):
        if self.nv:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()

    def stop(self):
        if self._t:
            self._stop.set()
            self._t.join()
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------------
# CPU side: the reference's own scalar attention (oracle/_ref) or its C restatement (oracle/)
class CpuAttentionSample:
    """Decode-attention calls of the workload's shape over the first CPU_SAMPLE_L KV rows on the host cores: the
    reference's own CPU attention when it was compiled (kind "reference"), else the C restatement (kind "port").
    The inputs are made once; run(calls) times `calls` back-to-back layer calls and returns the seconds."""

    def __init__(self, w, threads=None):
        from oracle.oracle import Oracle, RefLib
        self.L = L = min(CPU_SAMPLE_L, w["L"])
        self.n_head, self.n_kv, self.hd = n_head, n_kv, hd = w["n_head"], w["n_kv"], w["head_dim"]
        rng = np.random.default_rng(7)
        self.q = rng.standard_normal((n_head, hd), dtype=np.float32).astype(np.float16).astype(np.float32)
        self.kc = rng.standard_normal((n_kv, L, hd), dtype=np.float32).astype(np.float16).astype(np.float32)
        self.vc = rng.standard_normal((n_kv, L, hd), dtype=np.float32).astype(np.float16).astype(np.float32)
        self.scale = np.float32(1.0 / np.sqrt(hd))
        ncpu = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        self.threads = threads or min(n_head, ncpu)
        if RefLib.available():
            self.ref = RefLib()
            self.kind = "reference"
        else:
            import ctypes
            self.ref = None
            self.kind = "port"
            self.out = np.empty_like(self.q)
            self.f32p = ctypes.POINTER(ctypes.c_float)
            self.fn = Oracle().L.oracle_attend_head
            self.fn.argtypes = [self.f32p] * 4 + [ctypes.c_int] * 6 + [ctypes.c_float, self.f32p]
        self.cores = self.threads

    def _one_call(self):
        L, n_head = self.L, self.n_head
        if self.ref is not None:
            _, used = self.ref.attend_mt(self.q, self.kc, self.vc, L, self.scale, self.threads)
            self.cores = used
            return
        f32p, fn = self.f32p, self.fn

        def work(t):
            score = np.empty(L, np.float32)
            for h in range(t, n_head, self.threads):
                fn(self.q.ctypes.data_as(f32p), self.kc.ctypes.data_as(f32p), self.vc.ctypes.data_as(f32p),
                   self.out.ctypes.data_as(f32p), h, n_head, self.n_kv, self.hd, L, L, self.scale, score.ctypes.data_as(f32p))
        th = [threading.Thread(target=work, args=(t,)) for t in range(self.threads)]
        for x in th:
            x.start()
        for x in th:
            x.join()

    def run(self, calls):
        t0 = time.perf_counter()
        for _ in range(calls):
            self._one_call()
        return time.perf_counter() - t0

    def describe(self, calls):
        return ("%d layer calls of the workload shape, each over the first %d KV rows (fp32 cache, %d host threads, one per "
                "query head)" % (calls, self.L, self.cores))


REFERENCE_ARM_CALLS = 8     # layer calls per step of the reference arm (about two seconds of host work)
CPU_BASELINE_CALLS = 48     # layer calls of the cpu_baseline leg (10 to 15 seconds of host work)


def run_reference_arm(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cpu = CpuAttentionSample(w)
    times = []
    for i in range(args.warmup + args.steps):
        dt = cpu.run(REFERENCE_ARM_CALLS)
        if i >= args.warmup:
            times.append(dt)
    ms = 1e3 * float(np.mean(times))
    gbs = REFERENCE_ARM_CALLS * kv_bytes(w, cpu.L) / (ms * 1e-3) / 1e9
    sample = cpu.describe(REFERENCE_ARM_CALLS)
    line = {
        "impl": "reference", "metric": "decode_attn_kv_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "sample": sample, **{k: w[k] for k in ("n_head", "n_kv", "head_dim")}},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cpu.cores, "kind": cpu.kind, "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------
def run_b200(args, w):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d: launch with torch.distributed.run --nproc-per-node %d" % (args.gpus, world, args.gpus))
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from orin_llm_b200 import build, ops
    from orin_llm_b200.dist import PeerSplitKVDecoder, SplitKVDecoder, slice_bounds
    build.build()
    ops.init(local_rank)
    # Launch ordering of the decode kernels (oattn_set_decode_overlap).  2: the split kernel may fetch its first K/V
    # tiles while the previous call's merge drains.  Its precondition holds here as in the reference's decode graph:
    # the position word is constant during a step and every layer call has its own cache.  Measured: +13 % at 1K-4K
    # rows, +4 % at 8 GPUs (131072 rows per GPU), neutral for 1M rows on one GPU.
    if args.overlap < 0:
        args.overlap = 2
    ops.set_decode_overlap(args.overlap)

    n_head, n_kv, hd, layers, L = w["n_head"], w["n_kv"], w["head_dim"], w["layers"], w["L"]
    scale = 1.0 / float(np.sqrt(hd))
    bounds = slice_bounds(L, world)
    lo, hi = bounds[rank], bounds[rank + 1]
    n_loc = hi - lo
    gen = torch.Generator("cuda").manual_seed(1234 + rank)
    Kc = [torch.randn(n_kv, n_loc, hd, device="cuda", dtype=torch.float16, generator=gen) for _ in range(layers)]
    Vc = [torch.randn(n_kv, n_loc, hd, device="cuda", dtype=torch.float16, generator=gen) for _ in range(layers)]
    gq = torch.Generator("cuda").manual_seed(99)       # q is replicated: same seed on every rank
    q = torch.randn(layers, n_head, hd, device="cuda", generator=gq).half().float()
    out = torch.zeros(layers, n_head, hd, device="cuda")
    d_len = torch.tensor([n_loc], dtype=torch.int32, device="cuda")
    d_pos = torch.tensor([n_loc - 1], dtype=torch.int32, device="cuda")
    exchange = "none"
    dec = None
    if world > 1:
        exchange = args.exchange
        if exchange.startswith("peer"):
            try:
                dec = PeerSplitKVDecoder(n_head, n_kv, hd, fused=(exchange == "peer"))
            except Exception as e:      # no peer-mapped memory on this box: fall back to the NCCL all-gather
                if rank == 0:
                    print("peer exchange unavailable (%s); using the NCCL all-gather" % e, file=sys.stderr)
                exchange = "nccl"
        # every rank must take the same path
        flag = torch.tensor([1 if exchange.startswith("peer") else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            exchange = "nccl"
            dec = SplitKVDecoder(n_head, n_kv, hd)

    def step():
        if world == 1:
            for l in range(layers):
                ops.flash_attention_decode_ind(q[l], Kc[l], Vc[l], out[l], n_head, n_kv, hd, n_loc, d_pos, scale)
        else:
            for l in range(layers):
                dec.decode(q[l], Kc[l], Vc[l], n_loc, d_len, scale, out[l])

    def barrier():
        if world > 1:
            dist.barrier()

    def timed(fn, steps):
        barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if world > 1 and exchange != "nccl":
        # the kernel-driven exchange must give what the collective gives: check one layer call on every rank
        chk = SplitKVDecoder(n_head, n_kv, hd)
        want = torch.empty(n_head, hd, device="cuda")
        chk.decode(q[0], Kc[0], Vc[0], n_loc, d_len, scale, want)
        torch.cuda.synchronize()
        if not torch.allclose(out[0], want, rtol=1e-5, atol=1e-6):
            raise SystemExit("peer exchange result differs from the all-gather result on rank %d" % rank)

    # ---- timed region: kernel path with everything resident in HBM ----
    # The step is replayed from a CUDA graph, as the reference replays its decode step
    # (src/model_gpu.cu:295-344); --no-graph launches it eagerly instead.
    if args.no_graph:
        n_prof = min(args.steps * layers, 4096)
        ops.profile_enable(n_prof)
        run_step = step
        l0 = ops.launch_count()
    else:
        # event pairs around the split kernel of the first `n_prof_graph` layer calls, recorded as graph nodes
        # (a few, not all 36: every event node costs the graph a few microseconds)
        n_prof_graph = int(os.environ.get("OATTN_BENCH_PROFILE_CALLS", "4"))
        ops.profile_enable(n_prof_graph)
        l0 = ops.launch_count()
        cap_stream = torch.cuda.Stream()
        cap_stream.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=cap_stream, capture_error_mode="thread_local"):
            step()
        launches_per_step = ops.launch_count() - l0
        graph.replay()
        torch.cuda.synchronize()
        run_step = graph.replay
    sampler = ClockSampler(local_rank)
    sampler.start()
    total_ms = timed(run_step, args.steps)
    clocks = sampler.stop()
    launches = (ops.launch_count() - l0) if args.no_graph else launches_per_step * args.steps
    kern_ms = ops.profile_collect()
    ops.profile_enable(0)
    ms_per_step = total_ms / args.steps
    bytes_per_step = kv_bytes(w) * layers
    value = bytes_per_step / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the public API with HOST buffers ----
    # Per step: q, k_new, v_new of all layer calls come from pinned host memory in one copy, every call appends its
    # new row to the cache (fused) and attends, the results go back to host memory in one copy; one sync per step.
    # One pinned host block holds the step's inputs (q, k_new, v_new of every layer call), one holds its result.
    n_in = layers * (n_head + 2 * n_kv) * hd
    h_in = torch.randn(n_in).half().float().pin_memory()
    d_in = torch.empty(n_in, device="cuda")
    dq = d_in[: layers * n_head * hd].view(layers, n_head, hd)
    dk = d_in[layers * n_head * hd: layers * (n_head + n_kv) * hd].view(layers, n_kv, hd)
    dv = d_in[layers * (n_head + n_kv) * hd:].view(layers, n_kv, hd)
    hout = torch.empty(layers, n_head, hd).pin_memory()
    owner = rank == world - 1       # the rank whose slice holds the newest row

    def e2e_body():
        d_in.copy_(h_in, non_blocking=True)                 # host -> device: this step's inputs
        fused_peer = world > 1 and exchange == "peer"
        if world > 1 and owner and not fused_peer:
            # the rank that holds the newest row appends it for every layer first (these exchanges have no fused
            # append), so that no decode call directly follows a write to its own cache
            for l in range(layers):
                ops.kv_store_ind(Kc[l], Vc[l], dk[l], dv[l], n_kv, hd, n_loc, d_pos)
        for l in range(layers):
            if world == 1:
                ops.attn_decode(dq[l], dk[l], dv[l], Kc[l], Vc[l], out[l], n_head, n_kv, hd, n_loc, d_pos, scale,
                                ops.FUSE_KV_APPEND, None)
            elif fused_peer:
                # the owner of the newest row appends it inside its split kernel, as the single-GPU call does
                dec.decode_fused(dq[l], dk[l] if owner else None, dv[l] if owner else None, Kc[l], Vc[l], n_loc, d_len, None,
                                 scale, None, out[l], fuse=ops.FUSE_KV_APPEND if owner else ops.FUSE_NONE)
            else:
                dec.decode(dq[l], Kc[l], Vc[l], n_loc, d_len, scale, out[l])
        hout.copy_(out, non_blocking=True)                  # device -> host: the step's result

    ops.profile_enable(0)
    for _ in range(3):
        e2e_body()
        torch.cuda.current_stream().synchronize()
    if args.no_graph:
        def e2e_step():
            e2e_body()
            torch.cuda.current_stream().synchronize()
    else:
        # the host<->device copies (pinned memory) are part of the captured step; one synchronisation per step
        e2e_stream = torch.cuda.Stream()
        e2e_stream.wait_stream(torch.cuda.current_stream())
        e2e_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(e2e_graph, stream=e2e_stream, capture_error_mode="thread_local"):
            e2e_body()

        def e2e_step():
            e2e_graph.replay()
            torch.cuda.current_stream().synchronize()
        e2e_step()
    e2e_ms = timed(e2e_step, args.steps) / args.steps
    e2e_value = bytes_per_step / (e2e_ms * 1e-3) / 1e9
    h2d = layers * (n_head + 2 * n_kv) * hd * 4
    d2h = layers * n_head * hd * 4

    if exchange.startswith("peer") and dec.status() != 0:
        raise SystemExit("peer exchange: a bounded wait for the peers' records ran out (rank %d)" % rank)

    def finish():
        # Tearing the NCCL communicator / peer mappings down can block for minutes on some hosts; every rank has
        # its results by now, so leave through a barrier and a hard exit instead.
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)

    if rank != 0:
        finish()
        return

    peaks, peak_kind = measured_peaks()
    k_ms = float(np.mean(kern_ms)) if kern_ms else None
    per_launch_bytes = kv_bytes(w, n_loc)
    achieved = per_launch_bytes / (k_ms * 1e-3) / 1e9 if k_ms else None
    roofline = {
        "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
        "frac": (achieved / peaks["hbm_gbs"]) if achieved else None,
        "traffic": None, "kernel": "decode_split_kernel<128,false>", "kernel_ms": k_ms, "launches_timed": len(kern_ms),
        "algorithmic_bytes_per_launch": per_launch_bytes, "peak_source": peak_kind + " (MEASURED_PEAKS.json hbm_gbs)",
        "frac_of_nominal_8tbs": (achieved / 8000.0) if achieved else None,
    }
    # DRAM traffic of one split-kernel launch, from the ncu capture summarised in profiles/decode_split_kernel_L131072.md
    # (16/2 heads, 131072 rows: dram__bytes_read 134.272 MB for 134.218 MB of K/V, dram__bytes_write 4.2-4.7 MB).  Reads
    # grow with the rows streamed and are scaled by the bytes of this launch; the writes (split partials) do not
    # depend on the length and are added as captured.
    if per_launch_bytes:
        roofline["traffic"] = NCU_READ_PER_KV_BYTE * per_launch_bytes + NCU_WRITE_BYTES_PER_LAUNCH
        roofline["traffic_source"] = ("ncu capture at L=131072 (profiles/decode_split_kernel_L131072.md): reads scaled by "
                                      "bytes streamed, writes as captured")

    cpu = None
    if not args.no_cpu_baseline:
        smp = CpuAttentionSample(w)
        smp.run(1)
        dt = smp.run(CPU_BASELINE_CALLS)
        cpu = {"value": CPU_BASELINE_CALLS * kv_bytes(w, smp.L) / dt / 1e9, "unit": "GB/s", "cores": smp.cores,
               "kind": smp.kind, "sample": smp.describe(CPU_BASELINE_CALLS), "seconds": dt}

    # ---- comparison leg: the reference's own decode kernel (src/kernels.cu, recompiled unmodified for sm_100a) on
    # one layer call of this workload, same buffers; single GPU, device 0 only, group <= 8 (its limits)
    ref_cuda = None
    if world == 1 and local_rank == 0 and not args.no_ref_cuda and n_head // n_kv <= 8 and n_loc % 128 == 0:
        from oracle.oracle import RefCuda
        if RefCuda.available():
            rc = RefCuda()
            r_out = torch.empty(n_head, hd, device="cuda")
            rc.flash_attention_decode_ind(q[0], Kc[0], Vc[0], r_out, n_head, n_kv, hd, n_loc, d_pos, scale)
            torch.cuda.synchronize()
            reps = 3
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(reps):
                rc.flash_attention_decode_ind(q[i % layers], Kc[i % layers], Vc[i % layers], r_out, n_head, n_kv, hd, n_loc,
                                              d_pos, scale)
            e1.record()
            torch.cuda.synchronize()
            r_ms = e0.elapsed_time(e1) / reps
            rc.flash_attention_decode_ind(q[0], Kc[0], Vc[0], r_out, n_head, n_kv, hd, n_loc, d_pos, scale)
            m_out = torch.empty(n_head, hd, device="cuda")
            ops.flash_attention_decode_ind(q[0], Kc[0], Vc[0], m_out, n_head, n_kv, hd, n_loc, d_pos, scale)
            torch.cuda.synchronize()
            ref_cuda = {"value": per_launch_bytes / (r_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_call": r_ms,
                        "kernel": "flash_attention_decode_ind of the reference (src/kernels.cu:1993-2000), compiled for sm_100a",
                        "max_abs_diff_to_this_repo": float((r_out - m_out).abs().max().item())}

    line = {
        "metric": "decode_attn_kv_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": args.workload, "n_head": n_head, "n_kv": n_kv, "head_dim": hd, "layers_per_step": layers,
                   "kv_len": L, "kv_rows_per_gpu": n_loc, "parallelism": "kv-split x%d" % world,
                   "launch": "eager" if args.no_graph else "cuda graph replay of the step",
                   "launch_order": {0: "ordinary launches", 1: "programmatic dependent launches",
                                    2: "programmatic dependent launches, K/V prefetch ahead of the dependency wait"}[args.overlap],
                   "exchange": {"none": "single GPU", "peer": "merge kernel stores its record into every peer's buffer (NVLink peer stores), waits for the peers' records (generation-tagged words) and merges",
                                "peer-split": "as peer, with the wait and final merge in a launch of their own",
                                "nccl": "NCCL all-gather of the records"}[exchange],
                   "l2": "inputs larger than L2: each of the %d layer calls of a step reads its own %.0f MiB of KV" % (
                       layers, per_launch_bytes / 2**20)},
        "pct_of_8tbs": 100.0 * value / (8000.0 * world),
        "roofline": roofline, "cpu_baseline": cpu, "reference_cuda_kernel": ref_cuda,
        "e2e": {"value": e2e_value, "unit": "GB/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    print(json.dumps(line))
    finish()


def prefill_flops(w):
    """Causal algorithmic FLOPs of one chunk: 4 * head_dim * n_head * sum_t (n_past + t + 1)."""
    b, n_past = w["batch"], w["n_past"]
    return 4 * w["head_dim"] * w["n_head"] * (b * n_past + b * (b + 1) // 2)


def run_b200_prefill(args, w):
    """Secondary workloads: chunked-prefill attention, one GPU.  A step = `layers` fused prefill calls
    (RoPE q/k, KV append, causal attention), each on its own KV buffers."""
    import torch
    from orin_llm_b200 import build, ops
    if args.gpus != 1:
        raise SystemExit("prefill runs on one GPU")
    build.build()
    torch.cuda.set_device(0)
    ops.init(0)
    n_head, n_kv, hd, batch, n_past, layers = w["n_head"], w["n_kv"], w["head_dim"], w["batch"], w["n_past"], w["layers"]
    n_ctx = n_past + batch
    scale = 1.0 / float(np.sqrt(hd))
    gen = torch.Generator("cuda").manual_seed(5)
    Kc = [torch.randn(n_kv, n_ctx, hd, device="cuda", dtype=torch.float16, generator=gen) for _ in range(layers)]
    Vc = [torch.randn(n_kv, n_ctx, hd, device="cuda", dtype=torch.float16, generator=gen) for _ in range(layers)]
    q = torch.randn(layers, batch, n_head, hd, device="cuda", generator=gen)
    k = torch.randn(layers, batch, n_kv, hd, device="cuda", generator=gen)
    v = torch.randn(layers, batch, n_kv, hd, device="cuda", generator=gen)
    out = torch.empty(layers, batch, n_head, hd, device="cuda")
    rope = (ops.ROPE_NORMAL, hd, w["theta"], None)

    def step():
        for l in range(layers):
            ops.attn_prefill(q[l], k[l], v[l], Kc[l], Vc[l], out[l], n_head, n_kv, hd, n_ctx, n_past, batch, scale,
                             ops.FUSE_ALL, rope)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    l0 = ops.launch_count()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    launches = ops.launch_count() - l0
    ms = e0.elapsed_time(e1) / args.steps
    flops = prefill_flops(w) * layers
    tflops = flops / (ms * 1e-3) / 1e12
    peaks, peak_kind = measured_peaks()
    assert ops.prefill_status(n_head, n_kv, hd, batch) == 0

    # ---- comparison leg: the reference's own prefill sequence (rope q, rope k, kv_store_batch, flash_attention;
    # src/model_gpu.cu:379-384) with its kernels recompiled unmodified for sm_100a, on one layer's buffers
    ref_cuda = None
    if not args.no_ref_cuda and n_head // n_kv <= 8 and n_ctx % 128 == 0:
        from oracle.oracle import RefCuda
        if RefCuda.available():
            rc = RefCuda()
            r_out = torch.empty(batch, n_head, hd, device="cuda")
            rK, rV = Kc[0].clone(), Vc[0].clone()

            def ref_call():
                rq, rk = q[0].clone(), k[0].clone()
                rc.rope_batch(rq, ops.ROPE_NORMAL, batch * n_head, hd, hd, w["theta"], n_past, n_head)
                rc.rope_batch(rk, ops.ROPE_NORMAL, batch * n_kv, hd, hd, w["theta"], n_past, n_kv)
                rc.kv_store_batch(rK, rV, rk, v[0], n_kv, hd, n_ctx, n_past, batch)
                rc.flash_attention(rq, rK, rV, r_out, n_head, n_kv, hd, n_ctx, n_past, batch, scale)
            ref_call()
            torch.cuda.synchronize()
            reps = 5
            e0.record()
            for _ in range(reps):
                ref_call()
            e1.record()
            torch.cuda.synchronize()
            r_ms = e0.elapsed_time(e1) / reps
            ref_cuda = {"value": prefill_flops(w) / (r_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_call": r_ms,
                        "kernel": "rope_normal_batch x2 + kv_store_batch + flash_attention of the reference "
                                  "(src/kernels.cu), compiled for sm_100a; includes two small device copies of q and k",
                        "max_abs_diff_to_this_repo": float((r_out - out[0]).abs().max().item())}
    line = {
        "metric": "prefill_attn_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": args.workload, "n_head": n_head, "n_kv": n_kv, "head_dim": hd, "chunk": batch,
                   "kv_offset": n_past, "layers_per_step": layers, "rope_theta": w["theta"],
                   "l2": "K/V of one call (%.0f MiB) are re-read by the 16 query tiles of a kv head from L2 by design; "
                         "the %d layer calls of a step use distinct buffers" % (2 * n_kv * n_ctx * hd * 2 / 2**20, layers)},
        "roofline": {"bound": "tensor", "achieved": tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": tflops / peaks["bf16_tflops"], "traffic": None,
                     "peak_source": peak_kind + " (MEASURED_PEAKS.json bf16_tflops, burst)",
                     "frac_of_nominal_2250": tflops / 2250.0,
                     "note": "achieved = causal algorithmic FLOPs / step time, prologue kernel included"},
        "reference_cuda_kernel": ref_cuda,
        "gpu_launches": int(launches), "clocks": clocks,
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="decode_3b_L1048576", choices=sorted(WORKLOADS) + sorted(PREFILL_WORKLOADS))
    ap.add_argument("--layers", type=int, default=None, help="override the layer calls per step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-ref-cuda", action="store_true", help="skip the reference-CUDA-kernel comparison leg")
    ap.add_argument("--exchange", default="peer", choices=["peer", "peer-split", "nccl"], help="multi-GPU record exchange")
    ap.add_argument("--overlap", type=int, default=-1, choices=[-1, 0, 1, 2],
                    help="decode launch ordering (oattn_set_decode_overlap); -1: 2")
    ap.add_argument("--no-graph", action="store_true", help="launch the step eagerly instead of replaying a CUDA graph")
    args = ap.parse_args()
    if args.workload in PREFILL_WORKLOADS:
        w = dict(PREFILL_WORKLOADS[args.workload])
        if args.layers:
            w["layers"] = args.layers
        if args.impl == "reference":
            raise SystemExit("the reference arm is defined for the decode workloads")
        return run_b200_prefill(args, w)
    w = dict(WORKLOADS[args.workload])
    if args.layers:
        w["layers"] = args.layers
    if args.impl == "reference":
        run_reference_arm(args, w)
    else:
        run_b200(args, w)


if __name__ == "__main__":
    main()
