#!/usr/bin/env python
"""Benchmark of the BSI tensor-dot hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Default workload (fc1): one step = one pass of the hot path over one batch, the fixed76 chunk-scale BSI dot of
the FC1-like shape (Q=512 fp16 activations x R=8192 keys x D=2048; fc2: Q=512 x R=2048 x D=8192), keys prebuilt,
queries packed. The K-step region is timed ``--repeats`` times: ``value`` is effective TOPS = 2*Q*R*D / time of the
MEDIAN region with every operand resident in HBM; ``timing`` holds best and worst, SM cycles per step and the time
of a single launch after an L2 flush; ``sustained`` a leg of back-to-back replays lasting ``--sustained-seconds``.
``e2e`` is the same metric through the public ``bsi_ops`` entry points starting from pinned HOST activations and
ending with the float32 result back on the host. The fc1 line also carries ``fc2`` (the second dot shape, N = 1)
and ``opt_6_7b`` (tokens/s of the tensor-parallel OPT-6.7B forward on the same ranks) unless ``--extras 0``.

N > 1 (launched under torchrun, one rank per GPU): the keys are sharded along R, every rank owns an R-row shard
of the same size (weak scaling) and there is no data-path collective in the dot itself; timing is the max over
ranks. The ``opt_6_7b`` block is strong scaling: the same batch over R-sharded keys with the activation exchange.

Other workloads: ``pack`` / ``pack-lean`` / ``ewah`` time the HBM-bound kernels of the path (GB/s against the
measured copy bandwidth); ``opt-125m`` / ``opt-6.7b`` time the OPT forward with every q/k/v/out/fc1/fc2 linear as
a BSI op (tokens/s; N > 1: tensor parallel over R-sharded keys, strong scaling, see bsipytorch_b200/opt_tp.py).

``--impl reference`` times the reference's CPU path (the bsiCPP-semantics port under oracle/) on the host cores,
on a bounded sample of the same workload, and, where the reference's own kernels were compiled, those too.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    "fc1": dict(Q=512, R=8192, D=2048, name="FC1-like BSI dot Q=512 R=8192 D=2048 (fp16 acts, 1% outliers x20), dp=2, fixed76 chunkscale"),
    "fc2": dict(Q=512, R=2048, D=8192, name="FC2-like BSI dot Q=512 R=2048 D=8192 (fp16 relu acts), dp=2, fixed76 chunkscale"),
}
L2_BYTES = 126 * 1024 * 1024
# dram__bytes_read.sum + dram__bytes_write.sum of one dot launch, from the ncu capture summarised
# under profiles/ (None until a capture of that workload exists).
NCU_TRAFFIC_BYTES = {"fc1": 18061056, "fc2": 21090000, "pack": 134321152 + 85714944, "pack-lean": 134263552 + 39758592,
                     "ewah": 58746112 + 39424 + 59124992 + 8368384}


def make_inputs(wl, seed=123):
    """Seeded synthetic activations/weights with the configuration's shapes and distributions."""
    import torch
    g = torch.Generator().manual_seed(seed)
    Q, R, D = wl["Q"], wl["R"], wl["D"]
    q = torch.randn(Q, D, generator=g, dtype=torch.float32)
    if wl is WORKLOADS["fc1"]:
        mask = torch.rand(Q, D, generator=g) < 0.01
        q = torch.where(mask, q * 20.0, q)
    else:
        q = torch.relu(q)
    q = q.to(torch.float16)
    k = torch.randn(R, D, generator=g, dtype=torch.float32) * 0.02
    return q, k


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm_gbs=d.get("hbm_gbs"), bf16=d.get("bf16_tflops"), bf16_sustained=d.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


def dot_config(wl):
    """The `config` object of a dot workload; both arms print the same one."""
    set_bytes = wl["R"] * wl["D"] + wl["Q"] * wl["D"] + wl["Q"] * wl["R"] * 4
    nsets = max(2, int(-(-2 * L2_BYTES // set_bytes)))
    return {"workload": wl["name"],
            "l2": f"GPU arm: {nsets} rotating operand sets, {nsets * set_bytes / 2**20:.0f} MiB > 126 MiB L2; CPU arm: host memory"}


def int8_library_peak(dev):
    """Dense int8 throughput of the library GEMM on this GPU (torch._int_mm, 8192^3, best of 10, CUDA events):
    the second denominator beside 2 x the measured bf16 figure."""
    import torch
    n = 8192
    a = torch.randint(-64, 64, (n, n), dtype=torch.int8, device=dev)
    b = torch.randint(-64, 64, (n, n), dtype=torch.int8, device=dev).t().contiguous().t()
    for _ in range(3):
        torch._int_mm(a, b)
    torch.cuda.synchronize()
    best = 1e30
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch._int_mm(a, b)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    del a, b
    return 2.0 * n ** 3 / (best * 1e-3) / 1e12


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed regions run (read-only)."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        if self.nv is not None and self._thread is None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def host_threads():
    """Threads the CPU arm uses: every core this process may run on (a launcher such as torchrun sets
    OMP_NUM_THREADS=1 for its workers; the CPU baseline is meant to have all the host cores)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_port_rate(q, k, target_s, threads=0):
    """Times the CPU port on a bounded sample of query rows; returns (TOPS, rows, seconds, threads)."""
    from oracle import oracle as o
    keys = o.CpuKeyset(k.numpy(), 2)
    qn = q.float().numpy()
    if threads <= 0:
        threads = host_threads()
    nthreads = threads
    rows = min(2 * nthreads, qn.shape[0])
    t0 = time.perf_counter()
    keys.dot(qn[:rows], threads)
    t = time.perf_counter() - t0
    want = int(max(rows, min(qn.shape[0], rows * target_s / max(t, 1e-6))))
    want = max(nthreads, (want // nthreads) * nthreads) if want >= nthreads else want
    want = min(want, qn.shape[0])
    passes, t0 = 0, time.perf_counter()
    while True:                       # whole passes over the sample until the time budget is used
        keys.dot(qn[:want], threads)
        passes += 1
        t = time.perf_counter() - t0
        if t >= target_s or passes >= 1000:
            break
    ops = 2.0 * want * k.shape[0] * k.shape[1] * passes
    return ops / t / 1e12, f"{want} of {qn.shape[0]} query rows x all {k.shape[0]} keys, {passes} passes", t, nthreads


def run_reference(args, wl, rank, world):
    """The reference's CPU implementation of the path (port; the bsiCPP sources are not vendored)."""
    if rank != 0:
        return
    from oracle import oracle as o
    q, k = make_inputs(wl)
    keys = o.CpuKeyset(k.numpy(), 2)
    qn = q.float().numpy()
    nthreads = host_threads()
    # each step is a bounded sample of the workload's query rows, sized so that the whole run
    # (warm-up + steps) stays around two minutes whatever K is
    per_step = min(5.0, 120.0 / max(1, args.steps + args.warmup))
    rows = min(2 * nthreads, qn.shape[0])
    keys.dot(qn[:rows], nthreads)                                  # first touch (page faults, thread start-up)
    t0 = time.perf_counter()
    keys.dot(qn[:rows], nthreads)
    t = time.perf_counter() - t0
    rows = int(min(qn.shape[0], max(1, rows * per_step / max(t, 1e-6))))
    for _ in range(args.warmup):
        keys.dot(qn[:rows], nthreads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        keys.dot(qn[:rows], nthreads)
    t = time.perf_counter() - t0
    ops = 2.0 * rows * wl["R"] * wl["D"] * args.steps
    tops = ops / t / 1e12
    sample = f"{rows} of {wl['Q']} query rows x all {wl['R']} keys per step"
    line = {
        "impl": "reference", "metric": "BSI dot effective TOPS", "value": tops, "unit": "TOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int64", "data": "synthetic",
        "config": dot_config(wl),
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": nthreads, "kind": "port", "sample": sample},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    ref_gpu = time_reference_gpu_kernels(wl)
    if ref_gpu is not None:
        line["reference_gpu_kernels"] = ref_gpu
    print(json.dumps(line), flush=True)


def time_reference_gpu_kernels(wl):
    """Extra, informational: the reference's own fixed76 dot kernels (bsi_cuda_kernels.cu compiled
    unmodified for sm_100a, rsweep4 + cp.async staging) on the same workload and GPU. None when the
    compiled reference kernels or a GPU are not available."""
    try:
        import torch
        from oracle import ref_gpu
        if not ref_gpu.available():
            return None
        q, k = make_inputs(wl)
        dev = "cuda"
        qw, _, qs = ref_gpu.pack_queries_chunk(q.to(dev), 2, 7)
        kw, _, ks, _ = ref_gpu.pack_rows(k.to(dev), 2, 6)
        Bw = ref_gpu.slice_weights(6, k.shape[0], dev, ks)
        nsets = 6
        sets = [(qw.clone(), qs.clone(), kw.clone(), Bw.clone()) for _ in range(nsets)]
        for i in range(5):
            ref_gpu.dot_fixed76(*sets[i % nsets], 1e-4)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n = 60
        e0.record()
        for i in range(n):
            ref_gpu.dot_fixed76(*sets[i % nsets], 1e-4)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
        return {"kernel": "popcount_weighted_keys_literal_fused_bmma_tc_kernel_tm32_fixed76_chunkscale_rsweep4 (+ torch.zeros of the output, as the reference does)",
                "ms_per_step": ms, "value": 2.0 * wl["Q"] * wl["R"] * wl["D"] / (ms * 1e-3) / 1e12, "unit": "TOPS"}
    except Exception as e:  # informational only
        return {"unavailable": str(e)[:200]}


HBM_WORKLOADS = {
    "pack": dict(rows=4096, D=16384, lean=False,
                 name="quantise + bit-slice pack of fp16 activations [4096, 16384] (relu of N(0,1)): 7 slices + int8 image + chunk scales, dp=2"),
    "pack-lean": dict(rows=4096, D=16384, lean=True,
                      name="quantise + pack of fp16 activations [4096, 16384] (relu of N(0,1)): int8 image + chunk scales only (the fused layer path), dp=2"),
    "ewah": dict(rows=4096, D=16384, lean=False,
                 name="EWAH/verbatim encode (flags, sizes, offsets, emit) of the 28672 slices x 256 words of packed relu activations [4096, 16384], threshold 0.5"),
}


def run_hbm(args, rank, world, local_rank):
    """The HBM-bound kernels of the path, each as its own workload: GB/s of algorithmic bytes against the
    measured copy bandwidth. Inputs rotate over sets larger than L2; N > 1 runs independent replicas."""
    import ctypes as C

    import torch

    from bsipytorch_b200 import capi
    spec = HBM_WORKLOADS[args.workload]
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    rows, D = spec["rows"], spec["D"]
    W, chunks, bits = D // 64, D // 256, 7
    L = capi.lib()
    g = torch.Generator().manual_seed(5)
    nsets = 3
    xs = [torch.relu(torch.randn(rows, D, generator=g)).to(torch.float16).to(dev) for _ in range(nsets)]
    words = [torch.empty(rows, bits, W, dtype=torch.int64, device=dev) for _ in range(nsets)]
    q8 = torch.empty(rows, D, dtype=torch.int8, device=dev)
    sc = torch.empty(rows, chunks, dtype=torch.float32, device=dev)
    stream = capi.stream_ptr()

    def pack(i, lean):
        capi.check(L.bsi_b200_quantize_pack(capi.ptr(xs[i]), 1, rows, D, D, 2, bits, 1, None if lean else capi.ptr(words[i]),
                                            capi.ptr(sc), None, capi.ptr(q8), D, stream), "quantize_pack")

    if args.workload == "ewah":
        for i in range(nsets):
            pack(i, False)
        S = rows * bits
        scratch = torch.empty(max(int(L.bsi_b200_ewah_scratch_bytes(S)), 8), dtype=torch.uint8, device=dev)
        cap = S * (W + 1)
        out = torch.empty(cap, dtype=torch.int64, device=dev)
        off = torch.empty(S, dtype=torch.int64, device=dev)
        length = torch.empty(S, dtype=torch.int32, device=dev)
        flags = torch.empty(S, dtype=torch.int32, device=dev)
        total = torch.zeros(1, dtype=torch.int64, device=dev)

        def step(i):
            capi.check(L.bsi_b200_ewah_encode(capi.ptr(words[i % nsets]), S, W, C.c_double(0.5), capi.ptr(scratch), scratch.numel(),
                                              capi.ptr(out), cap, capi.ptr(off), capi.ptr(length), capi.ptr(flags),
                                              capi.ptr(total), stream), "ewah_encode")
        step(0)
        torch.cuda.synchronize()
        stream_words = int(total.item())
        # flags pass reads the words once, the size pass the compressible slices again, emit reads all and writes the stream
        bytes_step = 2 * S * W * 8 + stream_words * 8 + S * 24
        launches, kernel = 4, "ewah_flags_kernel + ewah_size_kernel + ewah_offsets_kernel + ewah_emit_kernel"
        extra = {"stream_words": stream_words, "input_words": S * W}
    else:
        lean = spec["lean"]

        def step(i):
            pack(i % nsets, lean)
        bytes_step = rows * D * 2 + rows * D + rows * chunks * 4 + (0 if lean else rows * bits * W * 8)
        launches, kernel = 1, "quantize_pack_chunk_fast_kernel<__half>"
        extra = {}
    warmup, K = max(3, args.warmup), args.steps
    for i in range(warmup):
        step(i)
    sampler = ClockSampler(local_rank)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler.start()
    e0.record()
    for i in range(K):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    sampler.stop()
    ms = e0.elapsed_time(e1)
    # end to end through the public module, from pinned host activations (pack only)
    e2e = None
    if args.workload != "ewah":
        import bsipytorch_b200
        host = xs[0].cpu().pin_memory()
        n = max(3, min(10, args.e2e_steps))
        back = torch.empty(rows, chunks, dtype=torch.float32).pin_memory()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(n):
            cap_q = bsipytorch_b200.bsi_ops.build_bsi_queries_cuda_batch_packed(host.to(dev, non_blocking=True), 2, 0.5)
            back.copy_(bsipytorch_b200.bsi_ops.debug_query_batch_tensors(cap_q)["scales"], non_blocking=True)
        t1.record()
        torch.cuda.synchronize()
        e2e_ms = t0.elapsed_time(t1) / n
        e2e = {"value": bytes_step / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": rows * D * 2,
               "d2h_bytes_per_step": rows * chunks * 4, "ms_per_step": e2e_ms, "steps": n,
               "path": "pinned host fp16 -> H2D -> build_bsi_queries_cuda_batch_packed -> D2H chunk scales"}
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    if rank == 0:
        peaks = measured_peaks()
        gbs = bytes_step * K / (ms * 1e-3) / 1e9
        line = {"metric": "BSI " + args.workload + " GB/s", "value": gbs * world, "unit": "GB/s", "n_gpus": world, "steps": K,
                "warmup": warmup, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "fp16 -> int64 fixed point -> 7-bit slices / int8" if args.workload != "ewah" else "u64",
                "data": "synthetic",
                "config": {"workload": spec["name"], "l2": f"{nsets} rotating input sets of {rows * D * 2 >> 20} MiB (> 126 MiB L2 in total)",
                           "parallelism": "independent replicas" if world > 1 else "1 GPU", **extra},
                "e2e": e2e, "gpu_launches": K * launches, "clocks": sampler.summary(),
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": gbs / peaks["hbm_gbs"], "peak_source": peaks["source"] + " copy bandwidth",
                             "traffic": NCU_TRAFFIC_BYTES.get(args.workload), "kernel": kernel,
                             "algorithmic_bytes_per_step": bytes_step}}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


OPT_WORKLOADS = {
    "opt-125m": dict(batch=8, seq=128, dtype="float16"),
    "opt-6.7b": dict(batch=16, seq=256, dtype="float16"),
}


def measure_opt(workload, steps, warmup, e2e_steps, rank, world, local_rank, opt_impl="tp", exchange="auto",
                microbatches=2, cuda_graph=1, kernel_split=False, fuse_ln=False):
    """Times the OPT forward next-token pass (every q/k/v/out/fc1/fc2 linear a BSI op) inside an initialised
    process group; returns the measurements as a dict (max over ranks, CUDA events)."""
    import torch
    import torch.distributed as dist

    import bsipytorch_b200
    from bsipytorch_b200 import opt

    spec = OPT_WORKLOADS[workload]
    dev = torch.device("cuda", local_rank)
    cfg = opt.CONFIGS[workload]
    B, T = spec["batch"], spec["seq"]
    dtype = getattr(torch, spec["dtype"])
    if opt_impl == "tp":
        # fused QKV key set, head-sharded attention, token-sharded residual stream, packed int8 exchanges
        from bsipytorch_b200.opt_tp import build_opt_tp
        model = build_opt_tp(workload, dtype=dtype, device=dev, seed=0, rank=rank, world=world,
                             exchange=exchange, microbatches=microbatches, fuse_ln=fuse_ln, check_status=False)
        graphed = bool(cuda_graph) and (world == 1 or model.exchange == "peer")
        if graphed:
            model.capture(spec["batch"], spec["seq"])
        # this library's kernels per layer: 4 fused linears + the activation packs (two of them inside the add +
        # LayerNorm + pack kernel; the fc2 one disappears when fc1 re-quantises in its epilogue) + the flag barriers
        layer0 = model.layers[0]
        launches_per_layer = 4 + (3 if layer0.fuse_requant else 4) + (getattr(model, "barriers_per_layer", 6) if (world > 1 and model.exchange == "peer") else 0)
        scheme = ("tensor parallel: R-sharded BSI linears, head-sharded attention, token-sharded residual; packed int8 "
                  "activations and linear outputs " + ("stored straight into peer buffers over NVLink by the pack / linear kernels"
                                                       if model.exchange == "peer" else "moved by NCCL all-gather / all-to-all"))
        exchange_used = model.exchange if world > 1 else "none"
    else:
        # one BSIQuantizedLinear per nn.Linear, each followed by an fp16 all-gather of its outputs
        model = opt.build_opt_bsi(workload, dtype=dtype, device=dev, seed=0, rank=rank, world=world)
        launches_per_layer = 12     # 6 x (pack + fused linear)
        graphed = False
        scheme = "R-sharded BSI linears + fp16 all-gather of every output"
        exchange_used = "nccl all-gather" if world > 1 else "none"
    ids_host = torch.randint(0, cfg.vocab_size, (B, T), generator=torch.Generator().manual_seed(0)).pin_memory()
    ids = ids_host.to(dev)
    tok_host = torch.empty(B, dtype=torch.long).pin_memory()
    warmup = max(3, warmup)
    K = steps

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.no_grad():
        for _ in range(warmup):
            tok = model.next_token(ids)
        sampler = ClockSampler(local_rank)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        sampler.start()
        ev0.record()
        for _ in range(K):
            tok = model.next_token(ids)
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)
        e2e_steps = max(3, min(K, e2e_steps))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(e2e_steps):
            x = ids_host.to(dev, non_blocking=True)
            tok_host.copy_(model.next_token(x), non_blocking=True)
        e1.record()
        barrier()
        sampler.stop()
        e2e_ms = e0.elapsed_time(e1)
    if kernel_split:
        # device time per kernel over three more steps (CUPTI records through torch.profiler; informational,
        # printed to stderr by rank 0, outside every timed region)
        import collections
        from torch.profiler import ProfilerActivity, profile
        barrier()
        with torch.no_grad(), profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(3):
                model.next_token(ids)
            torch.cuda.synchronize()
        if rank == 0:
            per = collections.defaultdict(list)
            for e in prof.events():
                if e.device_type == torch.autograd.DeviceType.CUDA:
                    per[e.name[:72]].append(e.device_time)
            print("kernel | launches/step | ms/step | median us | max us", file=sys.stderr)
            for name, v in sorted(per.items(), key=lambda kv: -sum(kv[1]))[:14]:
                v = sorted(v)
                print(f"{name} | {len(v) / 3:.0f} | {sum(v) / 3e3:.3f} | {v[len(v) // 2]:.1f} | {v[-1]:.1f}", file=sys.stderr)
    t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])
    status = bsipytorch_b200.bsi_ops.device_status()
    st = torch.tensor([status], dtype=torch.int64, device=dev)
    if world > 1:
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
    h, f, L = cfg.hidden_size, cfg.ffn_dim, cfg.num_hidden_layers
    res = dict(B=B, T=T, K=K, warmup=warmup, ms=ms, e2e_ms=e2e_ms, e2e_steps=e2e_steps, status=int(st[0]), graphed=graphed,
               scheme=scheme, exchange=exchange_used, launches=K * L * launches_per_layer, clocks=sampler.summary(),
               bsi_ops_step=L * 2.0 * B * T * (4 * h * h + 2 * h * f), tok=tok)
    del model
    torch.cuda.empty_cache()
    return res


def run_opt(args, rank, world, local_rank):
    """OPT forward next-token pass with every q/k/v/out/fc1/fc2 linear as a BSI op; tokens/s.

    N > 1: tensor parallel over R-sharded keys (strong scaling: the batch is fixed)."""
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    r = measure_opt(args.workload, args.steps, args.warmup, args.e2e_steps, rank, world, local_rank, args.opt_impl,
                    args.exchange, args.microbatches, args.cuda_graph, args.kernel_split, bool(args.fuse_ln))
    if rank == 0:
        B, T, K, ms = r["B"], r["T"], r["K"], r["ms"]
        peaks = measured_peaks()
        int8_peak = 2.0 * peaks["bf16"]
        tops = r["bsi_ops_step"] * K / (ms * 1e-3) / 1e12 / world
        line = {
            "metric": "OPT BSI tokens/s", "value": B * T * K / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": K, "warmup": r["warmup"], "ms_per_step": ms / K, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "int8 x int8 -> int32 BSI linears, fp16 elsewhere",
            "data": "synthetic",
            "config": {"workload": f"{args.workload} random init, batch {B} x seq {T} uniform random ids, all q/k/v/out/fc1/fc2 as BSI ops, dp=2, fixed76 chunkscale",
                       "parallelism": f"{r['scheme']} x{world}" if world > 1 else "1 GPU",
                       "model_impl": args.opt_impl, "launch": "CUDA graph of the decoder stack" if r["graphed"] else "eager",
                       "microbatches": args.microbatches if (world > 1 and args.opt_impl == "tp") else 1,
                       "l2": "weights and activations of one forward exceed the 126 MiB L2" if args.workload != "opt-125m" else "keys of one forward (~150 MB with slices) are about the size of L2"},
            "e2e": {"value": B * T * r["e2e_steps"] / (r["e2e_ms"] * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": B * T * 8,
                    "d2h_bytes_per_step": B * 8, "ms_per_step": r["e2e_ms"] / r["e2e_steps"], "steps": r["e2e_steps"],
                    "path": "pinned host ids -> H2D -> OPTForCausalLM.next_token (BSI linears) -> D2H argmax tokens"},
            "gpu_launches": r["launches"],
            "clocks": r["clocks"],
            "roofline": {"bound": "tensor", "achieved": tops, "peak": int8_peak, "unit": "TFLOP/s", "frac": tops / int8_peak,
                         "peak_source": f"2 x {peaks['source']} bf16 burst {peaks['bf16']}", "traffic": None,
                         "kernel": "dot_i8_tcgen05 (whole-step time: includes pack, attention, LayerNorm, exchange)",
                         "algorithmic_ops_per_step": r["bsi_ops_step"]},
            "device_status": r["status"],
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4000)
    ap.add_argument("--warmup", type=int, default=40)
    ap.add_argument("--opt-impl", default="tp", choices=["tp", "layers"],
                    help="OPT workloads: tensor-parallel decoder (default) or one BSIQuantizedLinear per nn.Linear")
    ap.add_argument("--cuda-graph", type=int, default=1, help="tensor-parallel OPT: replay the decoder stack from a CUDA graph")
    ap.add_argument("--kernel-split", action="store_true",
                    help="OPT workloads: after the timed regions, print the device time per kernel of three steps to stderr")
    ap.add_argument("--fuse-ln", type=int, default=0,
                    help="tensor-parallel OPT: residual add + LayerNorm + pack in one kernel (not bit-identical to torch's LayerNorm)")
    ap.add_argument("--microbatches", type=int, default=2, help="peer exchange: sequence groups run on streams of their own")
    ap.add_argument("--exchange", default="auto", choices=["auto", "peer", "collective"],
                    help="tensor-parallel OPT: peer-memory stores (default on GPUs) or NCCL collectives")
    ap.add_argument("--workload", default="fc1", choices=sorted(WORKLOADS) + sorted(OPT_WORKLOADS) + sorted(HBM_WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=30)
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--engine", default="tcgen05")
    ap.add_argument("--repeats", type=int, default=50, help="dot workloads: how many times the K-step region is timed")
    ap.add_argument("--sustained-seconds", type=float, default=1.5, help="dot workloads: length of the sustained leg (0 = skip)")
    ap.add_argument("--isolated", type=int, default=30, help="dot workloads: single launches timed after an L2 flush (0 = skip)")
    ap.add_argument("--extras", type=int, default=1,
                    help="fc1: also report the FC2 dot (1 GPU), OPT-6.7B tokens/s on the same ranks and the library int8 GEMM rate")
    ap.add_argument("--opt-steps", type=int, default=8, help="fc1 extras: timed OPT-6.7B forwards")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.workload in HBM_WORKLOADS:
        if args.impl == "reference":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": "the reference's CPU path builds its vectors inside bsiCPP (not vendored); the dot workloads (fc1/fc2) carry the reference arm"}))
            return
        if args.steps == 4000:
            args.steps = 2000
        run_hbm(args, rank, world, local_rank)
        return
    if args.workload in OPT_WORKLOADS:
        if args.impl == "reference":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": "the reference's CPU path has no model-level driver without the HuggingFace checkpoints; the dot workloads (fc1/fc2) carry the reference arm"}))
            return
        if args.steps == 4000:
            args.steps = 20
        run_opt(args, rank, world, local_rank)
        return
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, wl, rank, world)
        return

    import ctypes as C
    import torch
    import torch.distributed as dist

    import bsipytorch_b200
    from bsipytorch_b200 import capi

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: the BSI path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ops = bsipytorch_b200.bsi_ops
    L = capi.lib()
    Q, R, D = wl["Q"], wl["R"], wl["D"]
    chunks = D // 256
    warmup = max(3, args.warmup)

    # Every rank holds its own R-row key shard (weak scaling); shards differ by seed.
    q, k = make_inputs(wl, seed=123 + rank)
    q_dev = q.to(dev)
    keys_cap, *_ = ops.build_bsi_keys_cuda(k.to(dev), 2, 0.5)
    kt = ops.debug_keys_tensors(keys_cap)
    qcap = ops.build_bsi_queries_cuda_batch_packed(q_dev, 2, 0.5)
    qt = ops.debug_query_batch_tensors(qcap)

    # Rotating operand sets so that consecutive steps do not find their operands in L2.
    set_bytes = kt["q8"].numel() + qt["q8"].numel() + Q * R * 4
    nsets = max(2, int(-(-2 * L2_BYTES // set_bytes)))
    sets = []
    for i in range(nsets):
        sets.append(dict(a8=qt["q8"].clone(), qs=qt["scales"].clone(), k8=kt["q8"].clone(),
                         bw0=kt["scales"].clone(), out=torch.empty(Q, R, dtype=torch.float32, device=dev)))
    # every operand set stands for a key set of its own: give each the bounds its builder would have registered
    register_bounds(L, capi, sets, kt, R, qt)
    engine = {"tcgen05": capi.ENGINE_TCGEN05, "simt": capi.ENGINE_SIMT}.get(args.engine)
    if engine is None and args.engine.startswith("tcgen05:"):
        engine = 1000 + int(args.engine.split(":")[1])      # single-CTA tiles of that width
    if engine is None and args.engine.startswith("pair:"):
        engine = 3000 + int(args.engine.split(":")[1])      # paired-CTA tiles of that width
    scale_inv = C.c_float(float(1.0 / 10.0 ** 4))
    if args.engine == "bmma":      # b1 mma.sync engine: reads the slice words, not the int8 image
        for s_ in sets:
            s_["aw"], s_["kw"] = qt["words"].clone(), kt["words"].clone()
            s_["Bw"] = kt["slice_weights"].clone()
    elif engine is None:
        raise SystemExit("unknown --engine " + args.engine)

    def step(i):
        s = sets[i % nsets]
        if args.engine == "bmma":
            rc = L.bsi_b200_dot_words(capi.ptr(s["aw"]), capi.ptr(s["qs"]), chunks, 7, D // 64, capi.ptr(s["kw"]),
                                      capi.ptr(s["Bw"]), 6, R, Q, scale_inv, R, capi.ptr(s["out"]), None, capi.stream_ptr())
            if rc != 0:
                capi.check(rc, "bsi_b200_dot_words")
            return
        rc = L.bsi_b200_dot_i8(capi.ptr(s["a8"]), s["a8"].shape[1], capi.ptr(s["qs"]), chunks, capi.ptr(s["k8"]),
                               s["k8"].shape[1], capi.ptr(s["bw0"]), Q, R, chunks, scale_inv, capi.ptr(s["out"]),
                               R, None, engine, capi.stream_ptr())
        if rc != 0:
            capi.check(rc, "bsi_b200_dot_i8")

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    assert torch.equal(sets[0]["out"], sets[1 % nsets]["out"])
    want_out, *_ = ops.batch_dot_product_multiquery_cuda_batch_caps(qcap, keys_cap)
    assert torch.equal(sets[0]["out"], want_out), "bench operands give a different result than the bsi_ops path"

    # One CUDA graph of nsets steps; K steps = K // nsets replays + (K % nsets) direct launches.
    side = torch.cuda.Stream(device=dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        step(0)
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for i in range(nsets):
                step(i)
    torch.cuda.synchronize()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # The timed region is exactly K steps between two barriers; it is taken `repeats` times (default 50) so that the
    # reported value is the median region, with the best and the spread beside it.
    K = args.steps
    reps, rem = divmod(K, nsets)
    region_ms = []
    sampler.start()
    for _ in range(max(1, args.repeats)):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record()
        for _ in range(reps):
            graph.replay()
        for i in range(rem):
            step(i)
        ev1.record()
        barrier()
        region_ms.append(ev0.elapsed_time(ev1))
    sampler.stop()
    clocks = sampler.summary()
    launches = K

    # Sustained leg: back-to-back replays for at least args.sustained_seconds, its own clock record (the power cap
    # pulls the SM clock down within a second of dense tensor work).
    sustained = None
    if args.sustained_seconds > 0:
        s2 = ClockSampler(local_rank)
        n_rep = max(1, int(args.sustained_seconds / max(1e-6, (sorted(region_ms)[len(region_ms) // 2] * 1e-3) * nsets / K)) // 8)
        es0, es1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        s2.start()
        t_wall = time.perf_counter()
        es0.record()
        total_steps = 0
        while True:
            for _ in range(n_rep):
                graph.replay()
            total_steps += n_rep * nsets
            torch.cuda.synchronize()
            if time.perf_counter() - t_wall >= args.sustained_seconds:
                break
        es1.record()
        barrier()
        s2.stop()
        sustained = (es0.elapsed_time(es1), total_steps, s2.summary())

    # Isolated launches: one dot after an L2 flush (a 256 MiB fill), CUDA events around the single launch.
    isolated_us = []
    if args.isolated > 0:
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        for i in range(args.isolated):
            flush.fill_(i & 1)
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            step(i)
            a1.record()
            torch.cuda.synchronize()
            isolated_us.append(a0.elapsed_time(a1) * 1e3)
        del flush

    # End to end through the public entry points, host buffers in and out. Two streams alternate, each with its own
    # pinned output buffer, so that the 16.8 MB device-to-host read of one step overlaps the upload, pack and dot of
    # the next (the steps stay whole: every step uploads its activations and downloads its result inside the region).
    x_host = q.pin_memory()
    out_hosts = [torch.empty(Q, R, dtype=torch.float32).pin_memory() for _ in range(2)]
    lanes = [torch.cuda.Stream(device=dev) for _ in range(2)]

    def e2e_step(i):
        with torch.cuda.stream(lanes[i % 2]):
            x = x_host.to(dev, non_blocking=True)
            cap = ops.build_bsi_queries_cuda_batch_packed(x, 2, 0.5)
            out, *_ = ops.batch_dot_product_multiquery_cuda_batch_caps(cap, keys_cap)
            out_hosts[i % 2].copy_(out, non_blocking=True)
            out.record_stream(lanes[i % 2])

    cur = torch.cuda.current_stream(dev)
    for ln in lanes:
        ln.wait_stream(cur)
    for i in range(4):
        e2e_step(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for ln in lanes:
        ln.wait_stream(cur)
    e0.record()
    for ln in lanes:
        ln.wait_stream(cur)       # both lanes start after e0
    for i in range(args.e2e_steps):
        e2e_step(i)
    for ln in lanes:
        cur.wait_stream(ln)
    e1.record()
    barrier()
    out_host = out_hosts[(args.e2e_steps - 1) % 2]
    e2e_ms = e0.elapsed_time(e1)
    assert torch.equal(out_host, want_out.cpu())

    t = torch.tensor(region_ms + [e2e_ms, sustained[0] if sustained else 0.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    region_ms = sorted(float(v) for v in t[:len(region_ms)])
    e2e_ms, sus_ms = float(t[-2]), float(t[-1])
    ms = region_ms[len(region_ms) // 2]
    status = ops.device_status()

    # The second dot shape of the metric (N = 1 only): same protocol, fewer repeats.
    fc2_block = None
    if world == 1 and args.workload == "fc1" and args.extras:
        fc2_block = time_fc2(dev, ops, L, capi)
    unregister_bounds(L, capi, sets)
    for s_ in sets:
        s_.clear()
    del sets
    torch.cuda.empty_cache()

    # The other half of the metric: OPT-6.7B tokens/s on the same ranks (tensor parallel, strong scaling).
    opt_block = None
    if args.extras and args.workload == "fc1":
        try:
            r = measure_opt("opt-6.7b", args.opt_steps, 3, 3, rank, world, local_rank, "tp", args.exchange,
                            args.microbatches, args.cuda_graph)
            opt_block = {"tokens_per_s": r["B"] * r["T"] * r["K"] / (r["ms"] * 1e-3), "ms_per_step": r["ms"] / r["K"],
                         "steps": r["K"], "warmup": r["warmup"], "batch": r["B"], "seq": r["T"], "exchange": r["exchange"],
                         "status": r["status"], "scaling": "strong", "launch": "CUDA graph of the decoder stack" if r["graphed"] else "eager",
                         "e2e_tokens_per_s": r["B"] * r["T"] * r["e2e_steps"] / (r["e2e_ms"] * 1e-3), "clocks": r["clocks"],
                         "bsi_tops_per_gpu": r["bsi_ops_step"] * r["K"] / (r["ms"] * 1e-3) / 1e12 / world}
        except Exception as e:      # the headline line must not be lost to the secondary block
            opt_block = {"unavailable": str(e)[:300]}

    if rank == 0:
        ops_step = 2.0 * Q * R * D * world
        tops = ops_step * K / (ms * 1e-3) / 1e12
        best_tops = ops_step * K / (region_ms[0] * 1e-3) / 1e12
        e2e_tops = ops_step * args.e2e_steps / (e2e_ms * 1e-3) / 1e12
        peaks = measured_peaks()
        int8_peak = 2.0 * peaks["bf16"]
        per_gpu_tops = tops / world
        alg_bytes = Q * 7 * D // 8 + R * 6 * D // 8 + Q * chunks * 4 + R * 4 + Q * R * 4
        lib_peak = int8_library_peak(dev) if args.extras else None
        mhz = clocks.get("sm_mhz")
        line = {
            "metric": "BSI dot effective TOPS", "value": tops, "unit": "TOPS", "n_gpus": world, "steps": K,
            "warmup": warmup, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x int8 -> int32 (bit-exact with the sliced popcount), fp32 chunk combine",
            "data": "synthetic",
            "config": dot_config(wl),
            "run": {"engine": args.engine, "keys_per_gpu": R, "launch": f"CUDA graph of {nsets} steps replayed",
                    "timed_region": f"{K} steps between barriers, taken {len(region_ms)} times: value = median region, max over ranks per region"},
            "timing": {"regions": len(region_ms), "median_us_per_step": 1e3 * ms / K, "best_us_per_step": 1e3 * region_ms[0] / K,
                       "worst_us_per_step": 1e3 * region_ms[-1] / K, "best_tops": best_tops,
                       "sm_cycles_per_step": (1e3 * ms / K) * mhz if mhz else None,
                       "isolated_launch_us": ({"median": sorted(isolated_us)[len(isolated_us) // 2], "min": min(isolated_us), "launches": len(isolated_us),
                                               "how": "one dot after a 256 MiB L2 flush, CUDA events around the single launch (includes launch latency)"}
                                              if isolated_us else None)},
            "e2e": {"value": e2e_tops, "unit": "TOPS", "h2d_bytes_per_step": Q * D * 2,
                    "d2h_bytes_per_step": Q * R * 4, "ms_per_step": e2e_ms / args.e2e_steps, "steps": args.e2e_steps,
                    "path": "pinned host fp16 -> H2D -> build_bsi_queries_cuda_batch_packed -> batch_dot_product_multiquery_cuda_batch_caps -> D2H fp32 (two streams alternate, so one step's download overlaps the next step's upload and compute)"},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": per_gpu_tops, "peak": int8_peak, "unit": "TFLOP/s",
                         "frac": per_gpu_tops / int8_peak,
                         "peak_source": f"2 x {peaks['source']} bf16 burst {peaks['bf16']} (dense int8 = 2 x bf16 on this part)",
                         "traffic": NCU_TRAFFIC_BYTES[args.workload] if args.engine == "tcgen05" else None,
                         "kernel": {"tcgen05": "dot_i8_tcgen05_pair_kernel", "bmma": "dot_words_bmma_kernel", "simt": "dot_i8_simt_kernel"}.get(args.engine, "dot_i8_tcgen05_pair_kernel"),
                         "algorithmic_ops_per_launch": 2.0 * Q * R * D, "algorithmic_bytes_per_launch": alg_bytes,
                         "hbm_frac_of_measured": (alg_bytes / (ms / K * 1e-3) / 1e9) / peaks["hbm_gbs"],
                         "library_int8_gemm_tops": lib_peak,
                         "frac_of_library_int8_gemm": (per_gpu_tops / lib_peak) if lib_peak else None},
            "device_status": status,
        }
        if sustained is not None:
            sus_tops = ops_step * sustained[1] / (sus_ms * 1e-3) / 1e12
            sus_peak = 2.0 * peaks["bf16_sustained"] if peaks.get("bf16_sustained") else None
            line["sustained"] = {"seconds": sus_ms * 1e-3, "steps": sustained[1], "value": sus_tops, "unit": "TOPS",
                                 "peak": sus_peak, "frac": (sus_tops / world / sus_peak) if sus_peak else None,
                                 "peak_source": "2 x measured bf16 sustained", "clocks": sustained[2]}
        if fc2_block is not None:
            line["fc2"] = fc2_block
        if opt_block is not None:
            line["opt_6_7b"] = opt_block
        if world == 1:
            cpu_tops, sample, secs, cores = cpu_port_rate(q, k, args.cpu_seconds)
            line["cpu_baseline"] = {"value": cpu_tops, "unit": "TOPS", "cores": cores, "kind": "port",
                                    "sample": f"{sample}, {secs:.1f} s"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def register_bounds(L, capi, sets, key_tensors, R, query_tensors=None):
    """The bench times the C entry point on copies of one packed key set and one packed query batch. The bsi_ops
    entry points register, for the images they own, the sums that let a dot accumulate in integers where that is
    provably exact (row sums of the keys at build time, chunk sums of squares of the queries around each dot), so
    the copies get the same registration -- what a user's capsules have."""
    if "abs_sum" not in key_tensors:
        return
    for s in sets:
        capi.check(L.bsi_b200_register_key_bounds(capi.ptr(s["k8"]), capi.ptr(key_tensors["abs_sum"]), R, 64),
                   "bsi_b200_register_key_bounds")
        if query_tensors is not None and "sq_norms" in query_tensors:
            capi.check(L.bsi_b200_register_query_bounds(capi.ptr(s["a8"]), capi.ptr(query_tensors["sq_norms"]),
                                                        query_tensors["sq_norms"].shape[1]), "bsi_b200_register_query_bounds")


def unregister_bounds(L, capi, sets):
    for s in sets:
        L.bsi_b200_unregister_key_bounds(capi.ptr(s["k8"]))
        L.bsi_b200_unregister_query_bounds(capi.ptr(s["a8"]))


def time_fc2(dev, ops, L, capi):
    """FC2-like dot (Q=512, R=2048, D=8192) with the protocol of the headline: rotating operand sets, graph replays,
    median of 20 regions of 400 steps."""
    import ctypes as C

    import torch
    wl = WORKLOADS["fc2"]
    Q, R, D = wl["Q"], wl["R"], wl["D"]
    chunks = D // 256
    q, k = make_inputs(wl, seed=123)
    keys_cap, *_ = ops.build_bsi_keys_cuda(k.to(dev), 2, 0.5)
    kt = ops.debug_keys_tensors(keys_cap)
    qcap = ops.build_bsi_queries_cuda_batch_packed(q.to(dev), 2, 0.5)
    qt = ops.debug_query_batch_tensors(qcap)
    set_bytes = kt["q8"].numel() + qt["q8"].numel() + Q * R * 4
    nsets = max(2, int(-(-2 * L2_BYTES // set_bytes)))
    sets = [dict(a8=qt["q8"].clone(), qs=qt["scales"].clone(), k8=kt["q8"].clone(), bw0=kt["scales"].clone(),
                 out=torch.empty(Q, R, dtype=torch.float32, device=dev)) for _ in range(nsets)]
    scale_inv = C.c_float(float(1.0 / 10.0 ** 4))
    register_bounds(L, capi, sets, kt, R, qt)

    def step(i):
        s = sets[i % nsets]
        capi.check(L.bsi_b200_dot_i8(capi.ptr(s["a8"]), s["a8"].shape[1], capi.ptr(s["qs"]), chunks, capi.ptr(s["k8"]),
                                     s["k8"].shape[1], capi.ptr(s["bw0"]), Q, R, chunks, scale_inv, capi.ptr(s["out"]),
                                     R, None, capi.ENGINE_TCGEN05, capi.stream_ptr()), "bsi_b200_dot_i8")
    for i in range(nsets):
        step(i)
    torch.cuda.synchronize()
    want, *_ = ops.batch_dot_product_multiquery_cuda_batch_caps(qcap, keys_cap)
    assert torch.equal(sets[0]["out"], want)
    side = torch.cuda.Stream(device=dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        step(0)
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for i in range(nsets):
                step(i)
    torch.cuda.synchronize()
    graph.replay()
    K = 400
    reps = max(1, K // nsets)
    K = reps * nsets
    regions = []
    for _ in range(20):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        regions.append(e0.elapsed_time(e1))
    regions.sort()
    ms = regions[len(regions) // 2]
    tops = 2.0 * Q * R * D * K / (ms * 1e-3) / 1e12
    peaks = measured_peaks()
    unregister_bounds(L, capi, sets)
    return {"workload": wl["name"], "value": tops, "unit": "TOPS", "us_per_step": 1e3 * ms / K, "best_us_per_step": 1e3 * regions[0] / K,
            "steps": K, "regions": len(regions), "frac": tops / (2.0 * peaks["bf16"]),
            "l2": f"{nsets} rotating operand sets, {nsets * set_bytes / 2**20:.0f} MiB"}


if __name__ == "__main__":
    main()
