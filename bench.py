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
KV_SHIFT_WORKLOAD = "kv_shift_8b_ctx8192"
PREFILL_WORKLOADS = {
    # Llama-3-8B attention shape: one 512-token chunk at KV offset n_past, RoPE theta 5e5 (normal pairing)
    "prefill_8b_off0": dict(n_head=32, n_kv=8, head_dim=128, batch=512, n_past=0, theta=5e5, layers=32),
    "prefill_8b_off4096": dict(n_head=32, n_kv=8, head_dim=128, batch=512, n_past=4096, theta=5e5, layers=32),
    "prefill_8b_off8192": dict(n_head=32, n_kv=8, head_dim=128, batch=512, n_past=8192, theta=5e5, layers=32),
}
# DRAM traffic of one launch of the decode kernel, from an ncu capture (dram__bytes_read.sum, dram__bytes_write.sum) of
# a 16/2-head, 131072-row launch: reads per algorithmic K+V byte, and the writes (partials, independent of the length).
NCU_READ_PER_KV_BYTE = 134.316 / 134.218
NCU_WRITE_BYTES_PER_LAUNCH = 4.23e6
NCU_CAPTURE = "ncu capture of decode_split_kernel<128,false>, 16/2 heads, 131072 rows"
MIN_DISTINCT_KV_BYTES = 512 << 20      # a step of a secondary workload touches at least this much KV (4x L2)


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
    """Decode-attention layer calls of the workload's shape over the workload's FULL KV length on the host cores: the
    reference's own CPU attention when it was compiled (kind "reference"), else the C restatement (kind "port").
    The reference is single-threaded; here one host thread per query head runs its loop, all the threads the path can
    use.  The inputs are made once; run(calls) times `calls` back-to-back layer calls and returns the seconds."""

    def __init__(self, w, threads=None):
        from oracle.oracle import Oracle, RefLib
        self.L = L = w["L"]
        self.n_head, self.n_kv, self.hd = n_head, n_kv, hd = w["n_head"], w["n_kv"], w["head_dim"]
        self.layers = w["layers"]
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
        return ("%d layer call(s) of the workload's %d per step, each over all %d KV rows (fp32 cache, %d host threads, one "
                "per query head)" % (calls, self.layers, self.L, self.cores))


REFERENCE_ARM_CALLS = 1     # layer calls per step of the reference arm (one to two seconds of host work at 1M rows)
CPU_BASELINE_CALLS = 8      # layer calls of the cpu_baseline leg (10 to 15 seconds of host work at 1M rows)


def run_reference_arm(args, w):
    """The reference's own CPU attention on the same workload: one full-length layer call per step (a bounded sample
    of the step's layer calls; GB/s is per byte of KV attended, so the sample size does not enter the metric)."""
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
        "config": {"workload": args.workload, "kv_len": w["L"], "layers_per_step": w["layers"], "sample": sample,
                   **{k: w[k] for k in ("n_head", "n_kv", "head_dim")}},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cpu.cores, "kind": cpu.kind, "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------
LAUNCH_ORDER = {0: "ordinary launches", 1: "programmatic dependent launches",
                2: "programmatic dependent launches, K/V tiles fetched ahead of the dependency wait"}
EXCHANGE = {"none": "single GPU",
            "peer": "a launch of one CTA per head behind the decode launch stores the record into every peer's buffer (NVLink "
                    "peer stores), waits for the peers' records (generation-tagged words) and merges",
            "peer-split": "as peer, with the wait and final merge in a launch of their own",
            "nccl": "NCCL all-gather of the records"}


class Dist:
    """Process-group plumbing of one bench process."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus:
            raise SystemExit("--gpus %d but WORLD_SIZE=%d: launch with torch.distributed.run --nproc-per-node %d" % (
                args.gpus, self.world, args.gpus))
        torch.cuda.set_device(self.local_rank)
        self.host_group = None
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            # no NVLink multicast object behind the symmetric-memory buffers: the kernels use plain peer stores only,
            # and no rank should ever exit while bound to one
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            self.host_group = dist.new_group(backend="gloo")     # barriers that wait on the host, not in a GPU kernel

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()

    def host_barrier(self):
        if self.world > 1:
            self.dist.barrier(group=self.host_group)

    def max_over_ranks(self, ms):
        if self.world == 1:
            return ms
        t = self.torch.tensor([ms], device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def timed(self, fn, steps):
        """`steps` calls of fn bracketed by barrier + synchronize on both sides; device time, max over ranks."""
        torch = self.torch
        self.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        self.barrier()
        return self.max_over_ranks(e0.elapsed_time(e1))

    def finish(self):
        # Tearing the NCCL communicator / peer mappings down can block for minutes on some hosts; every rank has its
        # results by now, so leave through a host-side barrier (the GPUs stay idle meanwhile) and a hard exit.
        if self.world > 1:
            self.torch.cuda.synchronize()
            self.host_barrier()
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)


def oracle_check_multi_gpu(D, w, q0, K0, V0, out0, scale, head=5):
    """N > 1: one head of the merged output of layer 0 against the CPU oracle over ALL rows of the sequence.  The kv
    head's slices are gathered to every rank (512 MiB at 1M rows); rank 0 runs the reference's scalar attention
    (oracle/_ref, else the C restatement) while the others wait on the host."""
    torch, dist = D.torch, D.dist
    n_head, n_kv, hd = w["n_head"], w["n_kv"], w["head_dim"]
    kv = head * n_kv // n_head
    n_loc = K0.shape[1]
    sizes = torch.tensor([n_loc], device="cuda")
    all_sizes = [torch.zeros_like(sizes) for _ in range(D.world)]
    dist.all_gather(all_sizes, sizes)
    if any(int(x.item()) != n_loc for x in all_sizes):
        return {"skipped": "slices differ in length"}
    Kf = torch.empty(D.world, n_loc, hd, device="cuda", dtype=torch.float16)
    Vf = torch.empty_like(Kf)
    dist.all_gather_into_tensor(Kf, K0[kv].contiguous())
    dist.all_gather_into_tensor(Vf, V0[kv].contiguous())
    res = None
    if D.rank == 0:
        from oracle.oracle import Oracle, RefLib
        L = D.world * n_loc
        kc = Kf.view(1, L, hd).float().cpu().numpy()
        vc = Vf.view(1, L, hd).float().cpu().numpy()
        qh = q0[head:head + 1].cpu().numpy()
        if RefLib.available():
            want, _ = RefLib().attend_mt(qh, kc, vc, L, np.float32(scale), 1)
            kind = "reference"
        else:
            want = Oracle().attend(qh, kc, vc, L, np.float32(scale))
            kind = "port"
        err = np.abs(out0[head:head + 1].cpu().numpy() - want)
        res = {"head": head, "rows": L, "max_abs": float(err.max()), "mean_abs": float(err.mean()), "oracle": kind,
               "tolerance": {"max_abs": 1e-2, "mean_abs": 1e-3}}
        if not (err.max() <= 1e-2 and err.mean() <= 1e-3):
            raise SystemExit("multi-GPU result differs from the CPU oracle: %r" % (res,))
    del Kf, Vf
    D.host_barrier()
    return res


def bench_decode(D, args, w, name, steps, warmup, exchange_arg="none", with_ref_cuda=False):
    """One decode workload on this process group: the device-resident figure, the end-to-end figure through the public
    API with host buffers, the decode kernel's own duration.  Returns a dict (the same on every rank)."""
    torch, dist = D.torch, D.dist
    from orin_llm_b200 import ops
    from orin_llm_b200.dist import PeerSplitKVDecoder, SplitKVDecoder, slice_bounds
    world, rank = D.world, D.rank
    n_head, n_kv, hd, layers, L = w["n_head"], w["n_kv"], w["head_dim"], w["layers"], w["L"]
    scale = 1.0 / float(np.sqrt(hd))
    bounds = slice_bounds(L, world)
    lo, hi = bounds[rank], bounds[rank + 1]
    n_loc = hi - lo
    n_ctx = n_loc
    gen = torch.Generator("cuda").manual_seed(1234 + rank)
    Kc = [torch.randn(n_kv, n_ctx, hd, device="cuda", dtype=torch.float16, generator=gen) for _ in range(layers)]
    Vc = [torch.randn(n_kv, n_ctx, hd, device="cuda", dtype=torch.float16, generator=gen) for _ in range(layers)]
    gq = torch.Generator("cuda").manual_seed(99)       # q is replicated: same seed on every rank
    q = torch.randn(layers, n_head, hd, device="cuda", generator=gq).half().float()
    out = torch.zeros(layers, n_head, hd, device="cuda")
    d_len = torch.tensor([n_loc], dtype=torch.int32, device="cuda")
    d_pos = torch.tensor([n_loc - 1], dtype=torch.int32, device="cuda")
    d_gpos = torch.tensor([L - 1], dtype=torch.int32, device="cuda")     # position in the whole sequence (RoPE angle)
    exchange, dec = "none", None
    if world > 1:
        exchange = exchange_arg
        if exchange.startswith("peer"):
            try:
                dec = PeerSplitKVDecoder(n_head, n_kv, hd, fused=(exchange == "peer"))
            except Exception as e:      # no peer-mapped memory on this box: fall back to the NCCL all-gather
                if rank == 0:
                    print("peer exchange unavailable (%s); using the NCCL all-gather" % e, file=sys.stderr)
                exchange = "nccl"
        flag = torch.tensor([1 if exchange.startswith("peer") else 0], device="cuda")      # every rank takes the same path
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            exchange = "nccl"
            dec = SplitKVDecoder(n_head, n_kv, hd)

    def step():
        if world == 1:
            for l in range(layers):
                ops.flash_attention_decode_ind(q[l], Kc[l], Vc[l], out[l], n_head, n_kv, hd, n_ctx, d_pos, scale)
        else:
            for l in range(layers):
                dec.decode(q[l], Kc[l], Vc[l], n_loc, d_len, scale, out[l])

    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    checks = {}
    if world > 1:
        if exchange != "nccl":
            # the kernel-driven exchange must give what the collective gives: one layer call on every rank
            chk = SplitKVDecoder(n_head, n_kv, hd)
            want = torch.empty(n_head, hd, device="cuda")
            chk.decode(q[0], Kc[0], Vc[0], n_loc, d_len, scale, want)
            torch.cuda.synchronize()
            if not torch.allclose(out[0], want, rtol=1e-5, atol=1e-6):
                raise SystemExit("peer exchange result differs from the all-gather result on rank %d" % rank)
            checks["peer_vs_allgather"] = "equal (rtol 1e-5) on every rank"
        checks["oracle"] = oracle_check_multi_gpu(D, w, q[0], Kc[0], Vc[0], out[0], scale)

    # ---- timed region: kernel path with everything resident in HBM; the step is replayed from a CUDA graph, as the
    # reference replays its decode step (src/model_gpu.cu:295-344); --no-graph launches it eagerly instead
    l0 = ops.launch_count()
    if args.no_graph:
        run_step = step
    else:
        cap_stream = torch.cuda.Stream()
        cap_stream.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=cap_stream, capture_error_mode="thread_local"):
            step()
        launches_per_step = ops.launch_count() - l0
        graph.replay()
        torch.cuda.synchronize()
        run_step = graph.replay
    sampler = ClockSampler(D.local_rank)
    sampler.start()
    total_ms = D.timed(run_step, steps)
    clocks = sampler.stop()
    launches = (ops.launch_count() - l0) if args.no_graph else launches_per_step * steps
    # One launch on its own: event pairs around the decode kernel of a few layer calls (event-record nodes in a small
    # graph of their own; between such nodes consecutive launches cannot overlap), outside the timed region.
    n_iso = min(4, layers)
    ops.profile_enable(n_iso)
    iso_stream = torch.cuda.Stream()
    iso_stream.wait_stream(torch.cuda.current_stream())
    iso_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(iso_graph, stream=iso_stream, capture_error_mode="thread_local"):
        for l in range(n_iso):
            if world == 1:
                ops.flash_attention_decode_ind(q[l], Kc[l], Vc[l], out[l], n_head, n_kv, hd, n_ctx, d_pos, scale)
            else:
                dec.decode(q[l], Kc[l], Vc[l], n_loc, d_len, scale, out[l])
    D.barrier()
    for _ in range(3):
        iso_graph.replay()
    torch.cuda.synchronize()
    iso_ms = ops.profile_collect()
    ops.profile_enable(0)
    D.barrier()
    ms_per_step = total_ms / steps
    bytes_per_step = kv_bytes(w) * layers
    value = bytes_per_step / (ms_per_step * 1e-3) / 1e9


    # ---- end to end through the public API with HOST buffers ----
    # Per step: the unrotated q, k_new, v_new of all layer calls come from pinned host memory in one copy; every call
    # rotates q and k (RoPE theta 1e6, neox pairing), appends the new row to its cache and attends, all inside the
    # decode launch; the results go back to pinned host memory in one copy; one synchronisation per step.
    n_in = layers * (n_head + 2 * n_kv) * hd
    h_in = torch.randn(n_in).half().float().pin_memory()
    d_in = torch.empty(n_in, device="cuda")
    dq = d_in[: layers * n_head * hd].view(layers, n_head, hd)
    dk = d_in[layers * n_head * hd: layers * (n_head + n_kv) * hd].view(layers, n_kv, hd)
    dv = d_in[layers * (n_head + n_kv) * hd:].view(layers, n_kv, hd)
    hout = torch.empty(layers, n_head, hd).pin_memory()
    owner = rank == world - 1       # the rank whose slice holds the newest row
    rope = (ops.ROPE_NEOX, hd, 1e6, None)

    def e2e_body():
        d_in.copy_(h_in, non_blocking=True)                 # host -> device: this step's inputs
        fused_peer = world > 1 and exchange == "peer"
        if world > 1 and not fused_peer:
            # these exchanges have no fused prologue: rotate q everywhere; the rank that holds the newest row rotates and
            # appends it for every layer first, so that no decode call directly follows a write to its own cache
            for l in range(layers):
                ops.rope_neox_ind(dq[l], n_head, hd, hd, 1e6, d_gpos)
                if owner:
                    ops.rope_neox_ind(dk[l], n_kv, hd, hd, 1e6, d_gpos)
                    ops.kv_store_ind(Kc[l], Vc[l], dk[l], dv[l], n_kv, hd, n_ctx, d_pos)
        for l in range(layers):
            if world == 1:
                ops.attn_decode(dq[l], dk[l], dv[l], Kc[l], Vc[l], out[l], n_head, n_kv, hd, n_ctx, d_pos, scale,
                                ops.FUSE_ALL, rope)
            elif fused_peer:
                # every rank rotates q; the owner of the newest row also rotates and appends it inside its launch
                dec.decode_fused(dq[l], dk[l] if owner else None, dv[l] if owner else None, Kc[l], Vc[l], n_ctx, d_len, d_gpos,
                                 scale, rope, out[l], fuse=ops.FUSE_ALL if owner else ops.FUSE_ROPE_Q)
            else:
                dec.decode(dq[l], Kc[l], Vc[l], n_ctx, d_len, scale, out[l])
        hout.copy_(out, non_blocking=True)                  # device -> host: the step's result

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
    e2e_ms = D.timed(e2e_step, steps) / steps
    if exchange.startswith("peer") and dec.status() != 0:
        raise SystemExit("peer exchange: a bounded wait for the peers' records ran out (rank %d)" % rank)

    peaks, peak_kind = measured_peaks()
    # The timed region holds nothing but launches of the decode kernel, `layers` per step, so its device time divided by
    # the launches is the kernel's average launch duration there (consecutive launches overlap at their ends by
    # programmatic dependent launch; the isolated figure is given next to it).
    k_ms = ms_per_step / layers
    per_launch_bytes = kv_bytes(w, n_loc)
    achieved = per_launch_bytes / (k_ms * 1e-3) / 1e9 if k_ms else None
    G = n_head // n_kv
    roofline = {
        "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
        "frac": (achieved / peaks["hbm_gbs"]) if achieved else None,
        # reads grow with the rows streamed and are scaled by the bytes of this launch; the writes (partials) do not
        # depend on the length and are added as captured
        "traffic": NCU_READ_PER_KV_BYTE * per_launch_bytes + NCU_WRITE_BYTES_PER_LAUNCH,
        "traffic_source": NCU_CAPTURE + ": dram__bytes_read.sum scaled by the bytes streamed, dram__bytes_write.sum as captured",
        "kernel": "decode_split_kernel<%d,%s>" % (hd, "true" if G > 8 else "false"), "kernel_ms": k_ms,
        "kernel_ms_how": "CUDA events around the timed region / launches in it (only this kernel is launched there)",
        "launches_timed": layers * steps, "algorithmic_bytes_per_launch": per_launch_bytes,
        "isolated_launch_ms": float(np.mean(iso_ms)) if iso_ms else None,
        "peak_source": peak_kind + " (MEASURED_PEAKS.json hbm_gbs)",
        "frac_of_nominal_8tbs": (achieved / 8000.0) if achieved else None,
    }

    # ---- comparison leg: the reference's own decode kernel (src/kernels.cu, recompiled unmodified for sm_100a) on
    # one layer call of this workload, same buffers; single GPU, device 0 only, group <= 8 (its limits)
    ref_cuda = None
    if with_ref_cuda and world == 1 and D.local_rank == 0 and G <= 8 and n_ctx % 128 == 0:
        from oracle.oracle import RefCuda
        if RefCuda.available():
            rc = RefCuda()
            r_out = torch.empty(n_head, hd, device="cuda")
            rc.flash_attention_decode_ind(q[0], Kc[0], Vc[0], r_out, n_head, n_kv, hd, n_ctx, d_pos, scale)
            torch.cuda.synchronize()
            reps = 3
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(reps):
                rc.flash_attention_decode_ind(q[i % layers], Kc[i % layers], Vc[i % layers], r_out, n_head, n_kv, hd, n_ctx,
                                              d_pos, scale)
            e1.record()
            torch.cuda.synchronize()
            r_ms = e0.elapsed_time(e1) / reps
            rc.flash_attention_decode_ind(q[0], Kc[0], Vc[0], r_out, n_head, n_kv, hd, n_ctx, d_pos, scale)
            m_out = torch.empty(n_head, hd, device="cuda")
            ops.flash_attention_decode_ind(q[0], Kc[0], Vc[0], m_out, n_head, n_kv, hd, n_ctx, d_pos, scale)
            torch.cuda.synchronize()
            ref_cuda = {"value": per_launch_bytes / (r_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_call": r_ms,
                        "kernel": "flash_attention_decode_ind of the reference (src/kernels.cu:1993-2000), compiled for sm_100a",
                        "max_abs_diff_to_this_repo": float((r_out - m_out).abs().max().item())}

    res = {
        "value": value, "unit": "GB/s", "ms_per_step": ms_per_step, "steps": steps,
        "config": {"workload": name, "n_head": n_head, "n_kv": n_kv, "head_dim": hd, "layers_per_step": layers,
                   "kv_len": L, "kv_rows_per_gpu": n_loc, "parallelism": "kv-split x%d" % world,
                   "launch": "eager" if args.no_graph else "cuda graph replay of the step",
                   "launch_order": LAUNCH_ORDER[args.overlap], "exchange": EXCHANGE[exchange],
                   "l2": "inputs larger than L2: each of the %d layer calls of a step reads its own %.0f MiB of KV (%.0f MiB "
                         "per step)" % (layers, per_launch_bytes / 2**20, layers * per_launch_bytes / 2**20)},
        "pct_of_8tbs": 100.0 * value / (8000.0 * world),
        "roofline": roofline, "reference_cuda_kernel": ref_cuda,
        "e2e": {"value": bytes_per_step / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": layers * (n_head + 2 * n_kv) * hd * 4, "d2h_bytes_per_step": layers * n_head * hd * 4,
                "fused": "RoPE(q), RoPE(k), KV append inside the decode launch"},
        "gpu_launches": int(launches), "clocks": clocks, "checks": checks or None,
    }
    return res


def bench_kv_shift(args, reps=5):
    """Context rolling (cuda::kv_shift, src/kernels.cu:1682-1700) on the Llama-3-8B cache at n_ctx 8192 (1 GiB of K and V):
    drop the first 4096 rows of every layer and kv head, slide the rest down, clear the tail.  GB/s = bytes read + bytes
    written / time; next to it the reference's own kernel (one thread per column walking the rows serially) on the same
    cache when it was compiled."""
    import torch
    from orin_llm_b200 import ops
    n_layer, n_kv, n_ctx, hd, n_keep, shift = 32, 8, 8192, 128, 0, 4096
    cache = ops.KVCache(n_layer, n_kv, n_ctx, hd)
    cache.buf.normal_()
    moved = (n_ctx - shift - n_keep) * hd * 2 * n_kv * n_layer * 2      # bytes that change place (K and V)
    cleared = shift * hd * 2 * n_kv * n_layer * 2
    traffic = 2 * moved + cleared
    sampler = ClockSampler(0)

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps
    sampler.start()
    ms = timed(lambda: ops.kv_shift(cache.k, cache.v, n_layer, n_kv, hd, n_ctx, n_keep, shift))
    clocks = sampler.stop()
    peaks, peak_kind = measured_peaks()
    res = {"value": traffic / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms, "steps": reps,
           "config": {"cache_bytes": int(cache.buf.numel() * 2), "n_layer": n_layer, "n_kv": n_kv, "n_ctx": n_ctx, "n_keep": n_keep,
                      "shift": shift, "l2": "the cache (1 GiB) is larger than L2"},
           "roofline": {"bound": "hbm", "achieved": traffic / (ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": traffic / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "traffic": None,
                        "algorithmic_bytes_per_launch": traffic, "kernel": "kv_shift_kernel",
                        "peak_source": peak_kind + " (MEASURED_PEAKS.json hbm_gbs)"},
           "clocks": clocks, "gpu_launches": reps + 1, "reference_cuda_kernel": None}
    if not args.no_ref_cuda:
        from oracle.oracle import RefCuda
        if RefCuda.available():
            rc = RefCuda()
            r_ms = timed(lambda: rc.kv_shift(cache.k, cache.v, n_layer, n_kv, hd, n_ctx, n_keep, shift))
            res["reference_cuda_kernel"] = {"value": traffic / (r_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_call": r_ms,
                                            "kernel": "kv_shift of the reference (src/kernels.cu:1682-1700), compiled for sm_100a"}
    return res


def free_device_memory():
    import gc
    import torch
    gc.collect()
    torch.cuda.empty_cache()


def secondary_layers(w):
    """Layer calls per step of a secondary decode workload: the model's, or more where a call's KV is so small that the
    model's calls together would fit in L2."""
    return max(w["layers"], -(-MIN_DISTINCT_KV_BYTES // kv_bytes(w)))


def run_b200(args, w):
    D = Dist(args)
    from orin_llm_b200 import build, ops
    build.build()
    ops.init(D.local_rank)
    # Launch ordering of the decode kernel (oattn_set_decode_overlap).  2: a call may fetch its first K/V tiles while the
    # previous call's merge drains.  Its precondition holds here as in the reference's decode graph: the position word
    # is constant during a step and every layer call has its own cache.
    if args.overlap < 0:
        args.overlap = 2
    ops.set_decode_overlap(args.overlap)
    main = bench_decode(D, args, w, args.workload, args.steps, args.warmup, args.exchange, with_ref_cuda=not args.no_ref_cuda)
    if D.rank != 0:
        D.finish()
        return
    free_device_memory()

    secondary = None
    if D.world == 1 and not args.no_secondary:
        # the other configurations the metric is quoted on, a short pass each, same process, own clock samples
        secondary = {}
        for name in sorted(WORKLOADS):
            if name == args.workload or not name.startswith("decode_7b"):
                continue
            sw = dict(WORKLOADS[name])
            sw["layers"] = secondary_layers(sw)
            r = bench_decode(D, args, sw, name, args.secondary_steps, 3)
            free_device_memory()
            secondary[name] = {k: r[k] for k in ("value", "unit", "ms_per_step", "steps", "roofline", "e2e", "clocks", "gpu_launches")}
            secondary[name]["config"] = {k: r["config"][k] for k in ("layers_per_step", "kv_len", "l2")}
        for name in sorted(PREFILL_WORKLOADS):
            r = bench_prefill(args, dict(PREFILL_WORKLOADS[name]), name, args.secondary_steps, 3, with_ref_cuda=False)
            free_device_memory()
            secondary[name] = {k: r[k] for k in ("value", "unit", "ms_per_step", "steps", "roofline", "clocks", "gpu_launches")}
            secondary[name]["config"] = {k: r["config"][k] for k in ("chunk", "kv_offset", "layers_per_step", "l2")}

        r = bench_kv_shift(args)
        secondary["kv_shift_8b_ctx8192"] = r
        free_device_memory()

    cpu = None
    if D.world == 1 and not args.no_cpu_baseline:
        smp = CpuAttentionSample(w)
        smp.run(1)
        dt = smp.run(CPU_BASELINE_CALLS)
        cpu = {"value": CPU_BASELINE_CALLS * kv_bytes(w, smp.L) / dt / 1e9, "unit": "GB/s", "cores": smp.cores,
               "kind": smp.kind, "sample": smp.describe(CPU_BASELINE_CALLS), "seconds": dt}

    line = {
        "metric": "decode_attn_kv_gbs", "value": main["value"], "unit": "GB/s", "n_gpus": D.world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": main["config"],
        "pct_of_8tbs": main["pct_of_8tbs"], "roofline": main["roofline"], "cpu_baseline": cpu,
        "reference_cuda_kernel": main["reference_cuda_kernel"], "e2e": main["e2e"], "gpu_launches": main["gpu_launches"],
        "clocks": main["clocks"], "checks": main["checks"], "secondary": secondary,
    }
    print(json.dumps(line))
    D.finish()


def prefill_flops(w):
    """Causal algorithmic FLOPs of one chunk: 4 * head_dim * n_head * sum_t (n_past + t + 1)."""
    b, n_past = w["batch"], w["n_past"]
    return 4 * w["head_dim"] * w["n_head"] * (b * n_past + b * (b + 1) // 2)


def bench_prefill(args, w, name, steps, warmup, with_ref_cuda=True):
    """Chunked-prefill attention on one GPU.  A step = `layers` fused prefill calls (RoPE q/k, KV append, causal
    attention), each on its own KV buffers.  Returns a dict."""
    import torch
    from orin_llm_b200 import ops
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

    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    l0 = ops.launch_count()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    launches = ops.launch_count() - l0
    ms = e0.elapsed_time(e1) / steps
    flops = prefill_flops(w) * layers
    tflops = flops / (ms * 1e-3) / 1e12
    peaks, peak_kind = measured_peaks()
    assert ops.prefill_status(n_head, n_kv, hd, batch) == 0

    # ---- comparison leg: the reference's own prefill sequence (rope q, rope k, kv_store_batch, flash_attention;
    # src/model_gpu.cu:379-384) with its kernels recompiled unmodified for sm_100a, on one layer's buffers
    ref_cuda = None
    if with_ref_cuda and n_head // n_kv <= 8 and n_ctx % 128 == 0:
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
    return {
        "metric": "prefill_attn_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": 1, "steps": steps,
        "warmup": max(warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": name, "n_head": n_head, "n_kv": n_kv, "head_dim": hd, "chunk": batch,
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


def run_b200_prefill(args, w):
    import torch
    from orin_llm_b200 import build, ops
    if args.gpus != 1:
        raise SystemExit("prefill runs on one GPU")
    build.build()
    torch.cuda.set_device(0)
    ops.init(0)
    print(json.dumps(bench_prefill(args, w, args.workload, args.steps, args.warmup, with_ref_cuda=not args.no_ref_cuda)))


def run_b200_kv_shift(args):
    import torch
    from orin_llm_b200 import build, ops
    build.build()
    torch.cuda.set_device(0)
    ops.init(0)
    print(json.dumps(bench_kv_shift(args, reps=args.steps)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="decode_3b_L1048576", choices=sorted(WORKLOADS) + sorted(PREFILL_WORKLOADS) + [KV_SHIFT_WORKLOAD])
    ap.add_argument("--layers", type=int, default=None, help="override the layer calls per step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-ref-cuda", action="store_true", help="skip the reference-CUDA-kernel comparison leg")
    ap.add_argument("--exchange", default="peer", choices=["peer", "peer-split", "nccl"], help="multi-GPU record exchange")
    ap.add_argument("--overlap", type=int, default=-1, choices=[-1, 0, 1, 2],
                    help="decode launch ordering (oattn_set_decode_overlap); -1: 2")
    ap.add_argument("--no-secondary", action="store_true", help="skip the short passes over the other configurations")
    ap.add_argument("--secondary-steps", type=int, default=5)
    ap.add_argument("--no-graph", action="store_true", help="launch the step eagerly instead of replaying a CUDA graph")
    args = ap.parse_args()
    if args.workload == KV_SHIFT_WORKLOAD:
        if args.impl == "reference" or args.gpus != 1:
            raise SystemExit("context rolling is timed on one GPU, on this repository's arm")
        return run_b200_kv_shift(args)
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
