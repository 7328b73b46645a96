#!/usr/bin/env python3
"""Benchmark of the DIN-style CTR inference hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one batch of `--requests` requests (1 user x 1000 candidate items
each) through embedding pooling -> fused attention unit -> MLP tower.
Prints ONE JSON line: DIN predictions/s (whole job over all ranks), the
end-to-end figure with host buffers, the roofline of the dominant kernel, the
embedding-pool bandwidth on the sum-pooling configuration, the CPU baseline and
the clocks seen during the timed region.

With N > 1 the script expects to be launched by torch.distributed.run; every
rank serves its own requests on its own GPU (replicas, no data-path collective).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from __graft_entry__ import load_package  # noqa: E402


def checker_path():
    """The CPU oracle's Python bindings live with the tests; only the cpu_baseline leg and the output checks
    made outside the timed regions import them."""
    p = os.path.join(ROOT, "tests")
    if p not in sys.path:
        sys.path.insert(0, p)

ATT_FLOP_PER_PAIR = 2 * (144 * 80 + 80 * 40 + 40)      # attention MLP 144-80-40-1 per (candidate, step)
N_CAND, T_STEPS = 1000, 100


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "tf_burst": d["bf16_tflops"], "tf_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tf_burst": 1590.0, "tf_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """SM clock and throttle reasons of one GPU while the timed region runs: NVML polled every 2 ms from a
    thread (read-only queries), nvidia-smi at its fastest interval when NVML cannot be loaded."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None
        self.sm, self.mx, self.reasons, self.stop_flag, self.thread, self.nvml = [], None, set(), False, None, None

    def _handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            import torch
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode() if not uuid.startswith("GPU-") else uuid.encode())
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.index)

    def _poll(self, nv, h):
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self.stop_flag:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                mask = int(reasons_fn(h))
                for name, bit in self.BITS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        try:
            nv, h = self._handle()
            self.mx = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            self.nvml = nv
            self.thread = threading.Thread(target=self._poll, args=(nv, h), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.nvml is not None:
            self.stop_flag = True
            self.thread.join(timeout=1.0)
            return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.mx,
                    "reasons": sorted(self.reasons), "samples": len(self.sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0])); mx = float(r[1])
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvidia-smi"}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


# ---------------------------------------------------------------------------------------------
def run_ours(args):
    import numpy as np
    import torch
    load_package()
    from x_deeplearning_b200 import din, ops, workloads

    rank, local_rank, world = dist_env()
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    pk = peaks()
    R, K, W, NB = args.requests, args.steps, args.warmup, args.batches

    model = workloads.din_model(seed=0)
    net = din.DinModel(model)
    staged = [net.stage(workloads.din_requests(model, 1000 * rank + 17 + i, R, N_CAND)) for i in range(NB)]
    plans = [net.upload(staged[i], slot=i) for i in range(NB)]
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        import torch.distributed as dist
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- what is about to be timed gives the oracle's answer: one request of the first batch, outside the timed region
    if rank == 0:
        checker_path()
        import din_oracle
        req0 = workloads.din_requests(model, 1000 * rank + 17, R, N_CAND)
        one = {k: v for k, v in req0.items()}
        one.update(requests=1, user_ids=req0["user_ids"][:1], seq_len=req0["seq_len"][:1],
                   hist_item=req0["hist_item"][:int(req0["seq_len"][0])], hist_cate=req0["hist_cate"][:int(req0["seq_len"][0])],
                   cand_item=req0["cand_item"][:N_CAND], cand_cate=req0["cand_cate"][:N_CAND])
        got0 = net.forward_device(plans[0]).cpu().numpy()[:N_CAND]
        parity_err = float(np.abs(got0 - din_oracle.forward(model, one)).max())
        assert parity_err <= 2e-3, "DIN probabilities of the benchmark's first request differ from the oracle by %g" % parity_err
    else:
        parity_err = None

    # ---- device-resident throughput (inputs already in HBM) --------------------------------
    for i in range(W):
        net.forward_device(plans[i % NB])
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(K)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    e0.record()
    for i in range(K):
        net.forward_device(plans[i % NB], marks=marks[i])
    e1.record()
    barrier()
    clocks = sampler.stop()
    dev_ms = max_over_ranks(e0.elapsed_time(e1))
    assert ops.device_status() == 0, "a bounded wait ran out inside a tensor-core kernel"
    pool_ms = statistics.mean(m[0].elapsed_time(m[1]) for m in marks)
    att_ms = statistics.mean(m[2].elapsed_time(m[3]) for m in marks)
    # the same K steps with consecutive steps on two streams (every step has buffers of its own): the pooling launch of
    # one step, bound by memory latency, then shares the SMs with the attention kernel of the other, bound by the SFU
    side = [torch.cuda.Stream(), torch.cuda.Stream()]
    main = torch.cuda.current_stream()
    for st in side:
        st.wait_stream(main)
    for i in range(W):
        with torch.cuda.stream(side[i & 1]):
            net.forward_device(plans[i % NB])
    for st in side:
        main.wait_stream(st)
    barrier()
    o0, o1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    o0.record()
    for st in side:
        st.wait_stream(main)
    for i in range(K):
        with torch.cuda.stream(side[i & 1]):
            net.forward_device(plans[i % NB])
    for st in side:
        main.wait_stream(st)
    o1.record()
    barrier()
    two_stream_ms = max_over_ranks(o0.elapsed_time(o1))
    assert ops.device_status() == 0

    # ---- end to end through the reference-facing API: PredictorManager / Predictor of the C++ host
    # runtime, pinned HOST buffers fed every step, probabilities copied back to the host every step
    from x_deeplearning_b200 import blaze_api, din_netdef
    text, feed_names = din_netdef.build(model)
    mgr = blaze_api.PredictorManager()
    din_netdef.register_tables(mgr, model)
    mgr.load_model_text(text, optimize=True)
    pred = mgr.create_predictor(device_type=1, device_id=local_rank)
    host_feeds = []
    for i in range(NB):
        req = workloads.din_requests(model, 1000 * rank + 17 + i, R, N_CAND)
        host_feeds.append({n: torch.from_numpy(a).pin_memory() for n, a in din_netdef.feeds_of(model, req).items()})
    for n, t in host_feeds[0].items():
        pred.reshape(n, list(t.shape))
    out_host = torch.empty((R * N_CAND, 2), dtype=torch.float32).pin_memory()
    out_np = out_host.numpy()

    def e2e_step(i):
        for n, t in host_feeds[i % NB].items():
            pred.feed_raw(n, t.data_ptr(), t.numel() * t.element_size())      # H2D on the predictor's stream
        pred.forward()                                                        # all kernels + stream sync
        pred.output("output", into=out_np)                                    # D2H of the probabilities

    for i in range(W):
        e2e_step(i)
    e2e_launches = pred.launches()
    barrier()
    t0 = time.perf_counter()
    for i in range(K):
        e2e_step(i)
    torch.cuda.synchronize()
    sync_local_ms = (time.perf_counter() - t0) * 1e3      # every step ends with a host-visible result
    barrier()
    sync_ms = max_over_ranks(sync_local_ms)

    # The same K steps served the way Blaze is deployed: one Predictor per serving thread (each thread owns
    # a stream), all created from the one PredictorManager, so that one request's copies overlap another's
    # kernels. Every step still feeds its own host buffers and reads its own result back inside the timed region.
    import threading
    P = max(1, args.serving_threads)
    ready, go = threading.Barrier(P + 1), threading.Barrier(P + 1)
    errors = []

    def serve(t):
        try:
            torch.cuda.set_device(local_rank)
            pr = mgr.create_predictor(device_type=1, device_id=local_rank)
            for n, tt in host_feeds[0].items():
                pr.reshape(n, list(tt.shape))
            o_host = torch.empty((R * N_CAND, 2), dtype=torch.float32).pin_memory()
            o_np = o_host.numpy()
            feeds = [[(n, tt.data_ptr(), tt.numel() * tt.element_size()) for n, tt in hf.items()] for hf in host_feeds]

            def step(i):
                for n, ptr, nbytes in feeds[i % NB]:
                    pr.feed_raw(n, ptr, nbytes)
                pr.forward()
                pr.output("output", into=o_np)
            for i in range(W):
                step(i)
            ready.wait()
            go.wait()
            for i in range(t, K, P):
                step(i)
        except Exception as e:                     # surfaced by the main thread
            errors.append(e)
            try:
                ready.abort(); go.abort()
            except Exception:
                pass

    threads = [threading.Thread(target=serve, args=(t,)) for t in range(P)]
    for th in threads:
        th.start()
    ready.wait()
    barrier()
    t0 = time.perf_counter()
    go.wait()
    for th in threads:
        th.join()
    e2e_local_ms = (time.perf_counter() - t0) * 1e3
    if errors:
        raise errors[0]
    barrier()
    e2e_ms = max_over_ranks(e2e_local_ms)
    h2d_bytes = int(sum(t.numel() * t.element_size() for t in host_feeds[0].values()))

    preds = R * N_CAND * K * world
    att_flops = ATT_FLOP_PER_PAIR * N_CAND * T_STEPS * R
    achieved_tf = att_flops / (att_ms * 1e-3) / 1e12
    line = {
        "metric": "DIN predictions/sec", "value": preds / (two_stream_ms * 1e-3), "unit": "predictions/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": two_stream_ms / K, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "DIN-style model, 1 user x 1000 candidates per request, T=100, tables 5M/10k/8x100k x 18 fp16",
                   "requests_per_step": R, "parallelism": "replicas x%d (one process per GPU, no collective)" % world,
                   "streams": "consecutive steps alternate between two CUDA streams (each step has buffers of its own), as "
                              "the serving threads of the end-to-end leg do; one stream alone is under one_stream",
                   "l2": "rotating %d pre-generated batches; tables (240 MB) and per-step intermediates exceed L2" % NB},
        "e2e": {"value": preds / (e2e_ms * 1e-3), "unit": "predictions/s",
                "h2d_bytes_per_step": h2d_bytes,
                "d2h_bytes_per_step": R * N_CAND * 2 * 4, "ms_per_step": e2e_ms / K,
                "api": "blaze::PredictorManager/Predictor (C++ host runtime) fed pinned host buffers",
                "serving_threads": P, "one_thread_ms_per_step": sync_ms / K,
                "launches_per_step": e2e_launches},
        "gpu_launches": din.DinModel.LAUNCHES_PER_FORWARD * K,
        "roofline": {"kernel": "din_att_tc_kernel", "bound": "tensor", "achieved": achieved_tf,
                     "peak": pk["tf_sustained"], "unit": "TFLOP/s", "frac": achieved_tf / pk["tf_sustained"],
                     # DRAM bytes per launch: 415 KB measured by ncu on a 4-request launch (q, k and the result
                     # only), scaled by the requests of one launch
                     "traffic": 103872 * R, "traffic_source": "ncu capture of 4 requests scaled by requests per launch",
                     "peak_source": pk["source"] + " (sustained bf16)", "ms_per_launch": att_ms,
                     "pool_ms_per_step": pool_ms},
        "one_stream": {"ms_per_step": dev_ms / K, "value": preds / (dev_ms * 1e-3),
                       "how": "the same K steps on one stream; the per-kernel times of the roofline entry come from this pass"},
        "clocks": clocks,
        "parity": {"checked": "request 0 of batch 0 (1000 candidates) against the CPU oracle before timing",
                   "max_abs_err": parity_err, "tol": 2e-3},
    }
    if world > 1 and not args.no_sharded:
        # the path that has collectives: measured after the replica leg, on the same process group
        del net, plans, staged, pred, mgr
        torch.cuda.empty_cache()
        leg = ShardedLeg(rank, world, args.table_rows, args.partial_dtype, args.sharded_impl, args.capacity_factor)
        line["sharded"] = leg.run(min(K, 20), W)
    if rank == 0 and world == 1 and not args.no_cpu:
        line["embedding_pool"] = bench_pool(pk)
        line["embedding_pool"]["hbm_resident"] = bench_pool_hbm(pk)
        line["fused_gemm"] = bench_gemm(pk)
        line["dien"] = bench_dien()
        line["cpu_baseline"] = cpu_baseline_din(model, workloads, cores=1, budget_s=args.cpu_seconds)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def bench_pool(pk):
    """Sum-pooling configuration (1M x 16 fp32, 512 x 20 segments) and a 128x larger batch of it:
    achieved HBM GB/s of pool_kernel from CUDA events, algorithmic bytes per launch."""
    import numpy as np
    import torch
    from x_deeplearning_b200 import ops, workloads
    out = {}
    for label, batch, reps in (("config", 512, 200), ("scaled_batch_65536", 65536, 20)):
        cfg = workloads.embedding_config(seed=0, batch=batch)
        table = ops.Table(torch.from_numpy(cfg["table"]), torch.float32)
        y = torch.zeros((batch, 320), device="cuda")
        groups, n_ids = [], 0
        for g, grp in enumerate(cfg["groups"]):
            n_ids += len(grp["ids"])
            groups.append(ops.make_group(table, torch.from_numpy(grp["ids"]).cuda(), torch.from_numpy(grp["values"]).cuda(),
                                         torch.from_numpy(grp["offsets"]).cuda(), [dict(udf=0, out=y, col=16 * g)],
                                         torch.float32, segments_are_offsets=True))
        plan = ops.PoolPlan(groups)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        flush2 = torch.ones(64 << 20, dtype=torch.float32, device="cuda")
        for _ in range(5):
            plan.run()
        nbytes = n_ids * (8 + 4 + 64) + batch * 20 * 4 + batch * 320 * 4

        def timed(mode):
            ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
            torch.cuda.synchronize()
            for a, b in ev:
                if mode != "warm":
                    flush.zero_()                  # 256 MB write: evicts the 64 MB table from L2
                if mode == "clean":
                    flush2.sum()                   # then a 256 MB read: the dirty lines are written back before
                                                   # the timed launch, so it finds L2 cold AND clean
                a.record(); plan.run(); b.record()
            torch.cuda.synchronize()
            ms = statistics.median(a.elapsed_time(b) for a, b in ev)
            return ms, nbytes / (ms * 1e-3) / 1e9
        ms, gbs = timed("dirty" if label == "config" else "warm")
        out[label] = {"ms_per_launch": ms, "algorithmic_bytes": nbytes, "achieved_gbs": gbs,
                      "frac_of_measured_copy_peak": gbs / pk["hbm_gbs"], "frac_of_8tbs_nominal": gbs / 8000.0,
                      "l2": "flushed before each launch (256 MB written)" if label == "config" else "inputs exceed L2"}
        if label == "config":
            for mode, note in (("clean", "256 MB written then 256 MB read before each launch: cold L2 without "
                                         "write-backs of the flush buffer inside the timed launch"),
                               ("warm", "back to back, table (64 MB) L2-resident")):
                ms2, gbs2 = timed(mode)
                out[label]["l2_" + mode] = {"ms_per_launch": ms2, "achieved_gbs": gbs2,
                                            "frac_of_measured_copy_peak": gbs2 / pk["hbm_gbs"], "l2": note}
        del table, y, groups, plan
    out["peak_gbs"] = pk["hbm_gbs"]
    out["peak_source"] = pk["source"]
    return out


def bench_gemm(pk, reps=30):
    """The tcgen05 GEMM on three shapes: the parallel-GEMM configuration as written (8 branches of
    [4096, 256] x [256, 128] + bias + PReLU into [4096, 1024]), the same with M = 65536 (launch overhead below
    2 %), and the compute-bound first layer of the large-table MLP ([65536, 1280] x [1280, 1024])."""
    import torch
    from x_deeplearning_b200 import capi, ops
    out = {}
    slope = torch.full((1,), 0.25, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timed(run, flush_l2):
        for _ in range(3):
            run()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
        torch.cuda.synchronize()
        for a, b in ev:
            if flush_l2:
                flush.zero_()
            a.record(); run(); b.record()
        torch.cuda.synchronize()
        return statistics.median(a.elapsed_time(b) for a, b in ev)

    for label, M in (("parallel_gemm_config", 4096), ("parallel_gemm_m65536", 65536)):
        P, K, N = 8, 256, 128
        A = torch.randn((P, M, K), device="cuda", dtype=torch.float16)
        Wk = torch.randn((P, N, K), device="cuda", dtype=torch.float16) / 16
        bias = torch.randn((P, N), device="cuda") * 0.01
        Y = torch.empty((M, P * N), device="cuda", dtype=torch.float16)
        run = lambda: ops.gemm(A, Wk, Y=Y, bias=bias, trans_b=True, batch=P, M=M, N=N, K=K, lda=K, ldb=K, ldy=P * N,
                               strides=(M * K, N * K, N, N), bias_kind=capi.XB_BIAS_ROW, epilogue=capi.XB_EPI_PRELU,
                               ep=(slope, None, None), ep_count=1, engine=capi.XB_GEMM_TCGEN05)
        ms = timed(run, flush_l2=(M == 4096))
        nbytes = 2 * (P * M * K + P * N * K + M * P * N) + 4 * P * N
        flops = 2.0 * P * M * N * K
        out[label] = {"ms_per_launch": ms, "achieved_gbs": nbytes / (ms * 1e-3) / 1e9, "tflops": flops / (ms * 1e-3) / 1e12,
                      "frac_of_measured_copy_peak": nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], "bound": "hbm (85 flop/B)",
                      "l2": "flushed before each launch (256 MB written)" if M == 4096 else "inputs exceed L2"}
        del A, Wk, Y
    M, K, N = 65536, 1280, 1024
    A = torch.randn((M, K), device="cuda", dtype=torch.float16)
    Wk = torch.randn((N, K), device="cuda", dtype=torch.float16) / K ** 0.5
    bias = torch.randn(N, device="cuda") * 0.01
    Y = torch.empty((M, N), device="cuda", dtype=torch.float16)
    run = lambda: ops.gemm(A, Wk, Y=Y, bias=bias, trans_b=True, M=M, N=N, K=K, epilogue=capi.XB_EPI_PRELU,
                           ep=(slope, None, None), ep_count=1, engine=capi.XB_GEMM_TCGEN05)
    ms = timed(run, flush_l2=False)
    tf = 2.0 * M * N * K / (ms * 1e-3) / 1e12
    out["mlp_layer1_m65536"] = {"ms_per_launch": ms, "tflops": tf, "frac_of_measured_burst_bf16": tf / pk["tf_burst"],
                                "frac_of_measured_sustained_bf16": tf / pk["tf_sustained"], "bound": "tensor (512 flop/B)"}
    out["peaks"] = {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops_burst": pk["tf_burst"], "bf16_tflops_sustained": pk["tf_sustained"],
                    "source": pk["source"]}
    return out


def bench_pool_hbm(pk, reps=40, only=None):
    """Pooling against tables that do NOT fit L2, ids rotating over 8 pre-generated batches (only the Zipf head
    of a table can stay L2-resident):
      shard25m_dim32  one 25 M x 32 fp16 shard (1.6 GB) of the large-table configuration, 8192 samples x 40
                      feature groups, id lists of 1..30, Zipf(1.05), sum pooling into [8192, 1280] fp16;
      item5m_dim18    the DIN item table, 5 M x 18 fp16 (240 MB at its 48-byte pitch), 65536 x 4 segments,
                      id lists of 1..50, Zipf(1.1), sum pooling into [65536, 72] fp16.
    Algorithmic bytes per launch: 8 B id + one row (dim * 2 B) per id, 4 B offset + dim * 2 B output per segment."""
    import numpy as np
    import torch
    from x_deeplearning_b200 import capi, ops, workloads
    cases = {"shard25m_dim32": dict(rows=25_000_000, dim=32, batch=8192, groups=40, max_len=30, s=1.05),
             "item5m_dim18": dict(rows=5_000_000, dim=18, batch=65536, groups=4, max_len=50, s=1.1)}
    out = {}
    for label, c in cases.items():
        if only and label != only:
            continue
        rows, dim, batch, G = c["rows"], c["dim"], c["batch"], c["groups"]
        tb = ops.Table.__new__(ops.Table)
        pitch = int(capi.lib().xb_table_row_pitch(dim, capi.XB_F16))
        tb.rows, tb.dim, tb.dtype, tb.pitch = rows, dim, torch.float16, pitch
        tb.buf = torch.empty((rows, pitch // 2), dtype=torch.float16, device="cuda")
        for r0 in range(0, rows, 1 << 22):
            tb.buf[r0:r0 + (1 << 22)].normal_(0, 0.01)
        tb.desc = capi.TableDesc()
        tb.desc.weights, tb.desc.rows, tb.desc.dim, tb.desc.dtype, tb.desc.row_pitch_bytes = tb.buf.data_ptr(), rows, dim, capi.XB_F16, pitch
        tb.slot_keys = tb.slot_rows = None
        y = torch.zeros((batch, G * dim), dtype=torch.float16, device="cuda")
        NB = 8
        rng = np.random.default_rng(5)
        plans, n_ids = [], 0
        for b in range(NB):
            groups = []
            for g in range(G):
                counts = rng.integers(1, c["max_len"] + 1, batch).astype(np.int32)
                n = int(counts.sum())
                ids = workloads.zipf_ids(rng, rows, n, c["s"])
                off = np.zeros(batch + 1, np.int32)
                np.cumsum(counts, out=off[1:])
                if b == 0:
                    n_ids += n
                groups.append(ops.make_group(tb, torch.from_numpy(ids).cuda(), None, torch.from_numpy(off).cuda(),
                                             [dict(udf=0, out=y, col=dim * g)], torch.float16, segments_are_offsets=True))
            plans.append(ops.PoolPlan(groups))
        for b in range(NB):
            plans[b].run()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
        torch.cuda.synchronize()
        for i, (a, b_) in enumerate(ev):
            a.record(); plans[i % NB].run(); b_.record()
        torch.cuda.synchronize()
        ms = statistics.median(a.elapsed_time(b_) for a, b_ in ev)
        nbytes = n_ids * (8 + dim * 2) + batch * G * 4 + batch * G * dim * 2
        gbs = nbytes / (ms * 1e-3) / 1e9
        # what a bare gather of uniformly random rows of this table reaches (no pooling, no output)
        n_probe = 8_000_000
        probe_rows = torch.randint(0, rows, (n_probe,), dtype=torch.int32, device="cuda")
        sink = torch.zeros(1, device="cuda")
        probe = lambda: ops.check(capi.lib().xb_gather_probe(tb.desc, probe_rows.data_ptr(), n_probe, sink.data_ptr(), ops.stream()))
        probe()
        pa, pb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        pa.record()
        for _ in range(5):
            probe()
        pb.record()
        torch.cuda.synchronize()
        probe_ms = pa.elapsed_time(pb) / 5
        ceiling = n_probe * (dim * 2 + 4) / (probe_ms * 1e-3) / 1e9
        out[label] = {"ms_per_launch": ms, "ids_per_launch": n_ids, "algorithmic_bytes": nbytes, "achieved_gbs": gbs,
                      "frac_of_measured_copy_peak": gbs / pk["hbm_gbs"], "table_bytes": rows * pitch,
                      "random_gather_ceiling_gbs": ceiling,
                      "random_gather_ceiling_note": "xb_gather_probe: %d uniformly random rows of this table, row bytes + 4 B "
                                                    "row number each, nothing else; Zipf ids let the pooling launch exceed "
                                                    "it through L2 hits" % n_probe,
                      "frac_of_random_gather_ceiling": gbs / ceiling,
                      "l2": "table exceeds L2; ids rotate over %d batches" % NB}
        del probe_rows
        del tb, y, plans
        torch.cuda.empty_cache()
    return out


class ReferenceDin:
    """The DIN-style model on the reference's OWN CPU implementation (oracle/_ref/libblaze_cpu.so: its operators,
    Workspace, Net and qed_sparse_puller compiled unmodified, driven through the un-fused NetDef of
    din_netdef.build_unfused), one request of 1000 candidates per Net::Run. None when that library was not built."""

    def __init__(self, model, workloads):
        import tempfile
        import numpy as np
        checker_path()
        import orc
        import refnet
        from x_deeplearning_b200 import din_netdef
        self.np, self.refnet, self.din_netdef, self.workloads, self.model = np, refnet, din_netdef, workloads, model
        self.dir = tempfile.mkdtemp(prefix="xdl_ref_")
        self.qed = os.path.join(self.dir, "din.qed")
        tables = {"item": (np.arange(len(model["item"]), dtype=np.int64), model["item"]),
                  "cate": (np.arange(len(model["cate"]), dtype=np.int64), model["cate"])}
        for g, w in enumerate(model["user"]):
            tables["user%d" % g] = (np.arange(len(w), dtype=np.int64), w)
        orc.RefStore(tables, self.qed).close()              # written by the reference's own store code
        self.text, _ = din_netdef.build_unfused(model)
        self.blas = refnet.blas_name()

    @staticmethod
    def available():
        checker_path()
        import orc
        import refnet
        return refnet.lib() is not None and orc.ref_lib() is not None

    def net(self):
        return self.refnet.RefNet(self.text, self.qed)

    def feeds(self, seed, n_cand=N_CAND):
        np = self.np
        req = self.workloads.din_requests(self.model, seed, 1, n_cand)
        return {n: (a.astype(np.float32) if n.endswith(".values") else a)
                for n, a in self.din_netdef.feeds_of(self.model, req).items()}

    @staticmethod
    def run(net, feeds):
        for n, a in feeds.items():
            net.feed(n, a)
        net.run()
        return net.output("output")

    def close(self):
        import shutil
        shutil.rmtree(self.dir, ignore_errors=True)


def cpu_baseline_din(model, workloads, cores, budget_s):
    """The reference's CPU path on a bounded sample of the same workload: its own operators when
    oracle/_ref/libblaze_cpu.so exists (kind "reference"), else the CPU oracle (kind "port")."""
    if ReferenceDin.available():
        ref = ReferenceDin(model, workloads)
        net, feeds = ref.net(), ref.feeds(99)
        ReferenceDin.run(net, feeds)
        t0, n = time.time(), 0
        while time.time() - t0 < budget_s:
            ReferenceDin.run(net, feeds)
            n += 1
        dt = time.time() - t0
        net.close()
        ref.close()
        return {"value": n * N_CAND / dt, "unit": "predictions/s", "cores": cores, "kind": "reference",
                "sample": "%d requests of 1 user x %d candidates (T=100) in %.1f s; the reference's own CPU operators "
                          "(Workspace::CreateNet + Net::Run on the un-fused NetDef, qed_sparse_puller), one thread; %s"
                          % (n, N_CAND, dt, ref.blas)}
    checker_path()
    import din_oracle
    n_cand = 100                                        # 100 of the 1000 candidates of one request
    req = workloads.din_requests(model, 99, 1, n_cand)
    din_oracle.forward(model, req)
    t0, n = time.time(), 0
    while time.time() - t0 < budget_s:
        din_oracle.forward(model, req)
        n += 1
    dt = time.time() - t0
    return {"value": n * n_cand / dt, "unit": "predictions/s", "cores": cores, "kind": "port",
            "sample": "%d passes of 1 request x %d candidates (T=100) in %.1f s; plain-C fp32 restatement "
                      "(oracle/oracle.c), single thread" % (n, n_cand, dt)}


# ---------------------------------------------------------------------------------------------
_REF_MODEL = None      # set before the worker processes fork, so the tables are shared copy-on-write


def _ref_worker(a):
    seed, n_cand, reps = a
    checker_path()
    import din_oracle
    from x_deeplearning_b200 import workloads
    model = _REF_MODEL
    req = workloads.din_requests(model, seed, 1, n_cand)
    for _ in range(reps):
        din_oracle.forward(model, req)
    return n_cand * reps


def run_reference(args):
    """The reference arm: the reference's own CPU implementation of the path on all host cores, same workload
    (one request = 1 user x 1000 candidates, T = 100, the 5 M / 10 k / 8 x 100 k tables). One Net per host thread,
    every step each thread serves one request (Blaze's deployment: one predictor per serving thread). Falls
    back to the oracle port when oracle/_ref/libblaze_cpu.so was not built."""
    rank, _, world = dist_env()
    if rank != 0:
        return
    load_package()
    from x_deeplearning_b200 import workloads
    cores = os.cpu_count() or 1
    config = {"workload": "DIN-style model, 1 user x 1000 candidates per request, T=100, tables 5M/10k/8x100k x 18 fp16",
              "requests_per_step": cores, "parallelism": "%d host threads, one reference Net each" % cores}
    model = workloads.din_model(seed=0)
    if ReferenceDin.available():
        import threading
        ref = ReferenceDin(model, workloads)
        nets = [ref.net() for _ in range(cores)]
        feeds = [ref.feeds(100 + i) for i in range(cores)]

        def step():
            ths = [threading.Thread(target=ReferenceDin.run, args=(nets[i], feeds[i])) for i in range(cores)]
            for t in ths:
                t.start()
            for t in ths:
                t.join()
        for _ in range(max(1, min(args.warmup, 2))):
            step()
        t0 = time.time()
        for _ in range(args.steps):
            step()
        dt = time.time() - t0
        preds = args.steps * cores * N_CAND
        kind = "reference"
        sample = ("each step: %d threads x 1 request x %d candidates (T=100) through the reference's own CPU operators "
                  "(un-fused NetDef, Workspace::CreateNet + Net::Run, qed_sparse_puller); %s" % (cores, N_CAND, ref.blas))
        for n in nets:
            n.close()
        ref.close()
    else:
        import multiprocessing as mp
        checker_path()
        import orc
        orc.lib()
        global _REF_MODEL
        n_cand = 200
        _REF_MODEL = model
        ctx = mp.get_context("fork")
        with ctx.Pool(cores) as pool:
            jobs = lambda: [(100 + i, n_cand, 1) for i in range(cores)]
            for _ in range(max(1, min(args.warmup, 1))):
                pool.map(_ref_worker, jobs())
            t0 = time.time()
            preds = 0
            for _ in range(args.steps):
                preds += sum(pool.map(_ref_worker, jobs()))
            dt = time.time() - t0
        kind = "port"
        sample = "each step: %d processes x 1 request x %d candidates (T=100), plain-C restatement" % (cores, n_cand)
        config["parallelism"] = "%d host processes" % cores
    v = preds / dt
    print(json.dumps({
        "impl": "reference", "metric": "DIN predictions/sec", "value": v, "unit": "predictions/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "cpu_baseline": {"value": v, "unit": "predictions/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": v, "unit": "predictions/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def bench_dien(reps=20, R=74):
    """C4: the DIEN-style model (GRU over the behaviour list, attention scores, AUGRU per candidate, tower) on
    R requests x 1000 candidates, device-resident inputs, CUDA events. Parity of this path is a test
    (tests/test_gpu_dien.py); here it is timed."""
    import torch
    from x_deeplearning_b200 import dien, ops, workloads
    model = workloads.dien_model(0, item_rows=200_000, cate_rows=10_000, user_rows=10_000, emb_sigma=0.5)
    net = dien.DienModel(model)
    plans = [net.upload(net.stage(workloads.din_requests(model, 40 + i, R, N_CAND)), slot=i) for i in range(4)]
    for i in range(3):
        net.forward_dien(plans[i % 4])
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(reps):
        net.forward_dien(plans[i % 4])
    t1.record()
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    ms = t0.elapsed_time(t1) / reps
    return {"ms_per_step": ms, "requests_per_step": R, "candidates_per_request": N_CAND, "T": T_STEPS,
            "predictions_per_s": R * N_CAND / (ms * 1e-3),
            "path": "pooling, xb_gru, attention scores (sigmoid, softmax over steps), xb_augru_shared (tcgen05), "
                    "tower GEMMs with PReLU epilogues"}


def run_micro(args):
    """Small stand-alone cases of single kernels, sized for a profiler capture that ends by itself
    (a few launches, inputs larger than L2 where DRAM figures matter, well under a few GB)."""
    import numpy as np
    import torch
    load_package()
    from x_deeplearning_b200 import capi, din, ops, workloads
    torch.cuda.set_device(0)
    reps = args.steps
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.micro == "att":
        model = workloads.din_model(seed=0, item_rows=200_000, cate_rows=10_000, user_rows=10_000, emb_sigma=0.5)
        net = din.DinModel(model)
        p = net.upload(net.stage(workloads.din_requests(model, 3, args.requests, N_CAND)))
        net.forward_device(p)
        torch.cuda.synchronize()
        t0.record()
        for _ in range(reps):
            net.att(p["q"], p["k"].view(-1, 36), p["R"], N_CAND, T_STEPS, out=p["att"], engine=args.att_engine)
    elif args.micro == "tower":
        model = workloads.din_model(seed=0, item_rows=200_000, cate_rows=10_000, user_rows=10_000, emb_sigma=0.5)
        net = din.DinModel(model)
        p = net.upload(net.stage(workloads.din_requests(model, 3, args.requests, N_CAND)))
        net.forward_device(p)
        torch.cuda.synchronize()
        t0.record()
        for _ in range(reps):
            net.tower(p["user_emb"], p["q"], p["k"].view(-1, 36), p["att"], p["R"], N_CAND, T_STEPS, out=p["prob"])
    elif args.micro == "pool":
        cfg = workloads.embedding_config(seed=0, batch=65536)
        table = ops.Table(torch.from_numpy(cfg["table"]), torch.float32)
        y = torch.zeros((65536, 320), device="cuda")
        groups = [ops.make_group(table, torch.from_numpy(g["ids"]).cuda(), torch.from_numpy(g["values"]).cuda(),
                                 torch.from_numpy(g["offsets"]).cuda(), [dict(udf=0, out=y, col=16 * i)],
                                 torch.float32, segments_are_offsets=True) for i, g in enumerate(cfg["groups"])]
        plan = ops.PoolPlan(groups)
        plan.run()
        t0.record()
        for _ in range(reps):
            plan.run()
    elif args.micro == "pool_hbm":
        print(json.dumps({"micro": "pool_hbm", **bench_pool_hbm(peaks(), reps=reps, only=args.case)}))
        return
    elif args.micro == "gemm":
        P, M, K, N = 8, 65536, 256, 128            # the parallel-GEMM configuration with M scaled 16x (A = 268 MB)
        A = torch.randn((P, M, K), device="cuda", dtype=torch.float16)
        Wk = torch.randn((P, N, K), device="cuda", dtype=torch.float16) / 16
        bias = torch.randn((P, N), device="cuda") * 0.01
        slope = torch.full((1,), 0.25, device="cuda")
        Y = torch.empty((M, P * N), device="cuda", dtype=torch.float16)
        run = lambda: ops.gemm(A, Wk, Y=Y, bias=bias, trans_b=True, batch=P, M=M, N=N, K=K, lda=K, ldb=K, ldy=P * N,
                               strides=(M * K, N * K, N, N), bias_kind=capi.XB_BIAS_ROW, epilogue=capi.XB_EPI_PRELU,
                               ep=(slope, None, None), ep_count=1, engine=capi.XB_GEMM_TCGEN05)
        run()
        t0.record()
        for _ in range(reps):
            ops.gemm(A, Wk, Y=Y, bias=bias, trans_b=True, batch=P, M=M, N=N, K=K, lda=K, ldb=K, ldy=P * N,
                     strides=(M * K, N * K, N, N), bias_kind=capi.XB_BIAS_ROW, epilogue=capi.XB_EPI_PRELU,
                     ep=(slope, None, None), ep_count=1, engine=capi.XB_GEMM_TCGEN05)
    elif args.micro == "gemm_mlp":
        # first layer of the large-table configuration's MLP at 8x its per-GPU batch: compute-bound (512 flop/B)
        M, K, N = 65536, 1280, 1024
        A = torch.randn((M, K), device="cuda", dtype=torch.float16)
        Wk = torch.randn((N, K), device="cuda", dtype=torch.float16) / K ** 0.5
        bias = torch.randn(N, device="cuda") * 0.01
        slope = torch.full((1,), 0.25, device="cuda")
        Y = torch.empty((M, N), device="cuda", dtype=torch.float16)
        run = lambda: ops.gemm(A, Wk, Y=Y, bias=bias, trans_b=True, M=M, N=N, K=K, epilogue=capi.XB_EPI_PRELU,
                               ep=(slope, None, None), ep_count=1, engine=capi.XB_GEMM_TCGEN05)
        run()
        t0.record()
        for _ in range(reps):
            run()
        extra = {"tflops": 2.0 * M * N * K / 1e12}
    t1.record()
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    ms = t0.elapsed_time(t1) / reps
    line = {"micro": args.micro, "launches": reps, "status": "ok", "ms_per_launch": ms}
    if args.micro == "gemm_mlp":
        line["tflop_per_s"] = extra["tflops"] / (ms * 1e-3)
    print(json.dumps(line))


def run_batching(args):
    """Request batching through the Predictor API: `--requests` predictors of the DIN-style model, each holding one
    request (1 user x 1000 candidates) in host buffers; every round feeds all of them, runs them and reads the
    outputs back. Arm "alone": each predictor runs Forward() in turn. Arm "batched": with InitScheduler(enable_batching)
    the Forward(cb) calls are stacked by the batch thread into one run. Wall clock, host to host."""
    import threading
    import time
    import numpy as np
    load_package()
    from x_deeplearning_b200 import blaze_api as api, din_netdef, workloads
    model = workloads.din_model(seed=0, item_rows=200_000, cate_rows=10_000, user_rows=10_000, emb_sigma=0.5)
    text, _ = din_netdef.build(model)
    P = args.requests
    feeds = [din_netdef.feeds_of(model, workloads.din_requests(model, 100 + i, 1, N_CAND)) for i in range(P)]
    outs = [np.empty((N_CAND, 2), np.float32) for _ in range(P)]

    def arm(batched):
        api.init_scheduler(batched, max_batch_size=P, batch_timeout_micros=200)
        mgr = api.PredictorManager()
        din_netdef.register_tables(mgr, model)
        mgr.load_model_text(text, optimize=True)
        preds = [mgr.create_predictor() for _ in range(P)]
        done = [threading.Event() for _ in range(P)]

        phase = {"feed": 0.0, "forward": 0.0, "output": 0.0}

        def round_():
            t_a = time.perf_counter()
            for p, f in zip(preds, feeds):
                for n, a in f.items():
                    p.feed(n, a)
            t_b = time.perf_counter()
            if batched:
                for p, ev in zip(preds, done):
                    ev.clear()
                    p.forward_async(ev.set)
                for ev in done:
                    assert ev.wait(60)
            else:
                for p in preds:
                    p.forward()
            t_c = time.perf_counter()
            for p, o in zip(preds, outs):
                p.output("output", into=o)
            t_d = time.perf_counter()
            phase["feed"] += t_b - t_a
            phase["forward"] += t_c - t_b
            phase["output"] += t_d - t_c
        for _ in range(max(args.warmup, 3)):
            round_()
        phase = {k: 0.0 for k in phase}
        t = time.perf_counter()
        for _ in range(args.steps):
            round_()
        dt = (time.perf_counter() - t) / args.steps
        for p in preds:
            p.close()
        mgr.close()
        api.init_scheduler(False)
        return dt, {k: v / args.steps * 1e3 for k, v in phase.items()}, outs[0].copy()
    b0, t0 = api.batching_stats()
    dt_alone, ph_alone, first_alone = arm(False)
    dt_batched, ph_batched, first_batched = arm(True)
    b1, t1 = api.batching_stats()
    assert np.array_equal(first_alone, first_batched)
    print(json.dumps({"micro": "batching", "predictors": P, "candidates_per_request": N_CAND, "rounds": args.steps,
                      "alone": {"ms_per_round": dt_alone * 1e3, "predictions_per_s": P * N_CAND / dt_alone,
                                "phase_ms": ph_alone},
                      "batched": {"ms_per_round": dt_batched * 1e3, "predictions_per_s": P * N_CAND / dt_batched,
                                  "phase_ms": ph_batched, "requests_per_merged_run": (t1 - t0) / max(b1 - b0, 1)},
                      "note": "wall clock, host buffers in and out, one submitting thread; phase_ms.forward is "
                              "Forward() of every predictor in turn (alone) or Forward(cb) of all until the last callback (batched)"}))


def shard_table_values(table, rows, dim, xp):
    """Value of element (row, col) of sharded table `table`: a counter-based hash, so that any rank and the CPU
    checker can materialise any row of a 200 M-row table without storing it. `rows` is an int64 array (numpy or
    torch); returns [len(rows), dim] float32 in (-0.0301, 0.0301) on the same backend."""
    if xp.__name__ == "numpy":
        r = rows.astype(xp.int64)[:, None]
        c = xp.arange(dim, dtype=xp.int64)[None, :]
    else:
        r = rows.to(xp.int64)[:, None]
        c = xp.arange(dim, dtype=xp.int64, device=rows.device)[None, :]
    h = (r * 1000003 + c * 7919 + (table + 1) * 104729) & 0x7fffffff
    h = (h * 48271) % 2147483647                       # products stay below 2^62
    h = (h >> 7) % 6021
    if xp.__name__ == "numpy":
        return (h - 3010).astype(xp.float32) * xp.float32(1e-5)
    return (h - 3010).to(xp.float32) * 1e-5


class ShardedLeg:
    """Row-sharded pooling + MLP (the large-table configuration): 4 tables x `table_rows` rows x dim 32 fp16
    sharded by id % world, 65536 x 40 feature groups split by sample over the ranks, ids routed and pooled
    vectors returned with NCCL all-to-all, then the MLP 1280-1024-512-256-1 (PReLU, sigmoid) data-parallel."""
    N_TABLES, GPT, DIM, BATCH = 4, 10, 32, 65536

    def __init__(self, rank, world, table_rows, partial_dtype="f16", impl="abi", capacity_factor=0.0):
        if capacity_factor <= 0.0:
            capacity_factor = min(2.0, 1.1 + 0.08 * world)
        import numpy as np
        import torch
        from x_deeplearning_b200 import capi, ops, sharded, workloads
        self.rank, self.world, self.rows_total = rank, world, table_rows
        self.torch, self.ops, self.capi, self.sharded = torch, ops, capi, sharded
        self.comm, self.gops = sharded.DistComm(), sharded.GpuShardOps(partial_dtype=partial_dtype)
        self.partial_dtype, self.impl = partial_dtype, impl
        n_tables, gpt, dim = self.N_TABLES, self.GPT, self.DIM
        self.B = B = self.BATCH // world
        rng = np.random.default_rng(100 + rank)
        self.tables = []
        for t in range(n_tables):
            local_rows = (table_rows - rank + world - 1) // world
            tb = ops.Table.__new__(ops.Table)
            tb.rows, tb.dim, tb.dtype, tb.pitch = local_rows, dim, torch.float16, dim * 2
            tb.buf = torch.empty((local_rows, dim), dtype=torch.float16, device="cuda")
            for r0 in range(0, local_rows, 1 << 22):          # local row l of this shard is global row l*world + rank
                l = torch.arange(r0, min(r0 + (1 << 22), local_rows), dtype=torch.int64, device="cuda")
                tb.buf[r0:r0 + l.numel()] = shard_table_values(t, l * world + rank, dim, torch).to(torch.float16)
            tb.desc = capi.TableDesc()
            tb.desc.weights, tb.desc.rows, tb.desc.dim, tb.desc.dtype, tb.desc.row_pitch_bytes = \
                tb.buf.data_ptr(), local_rows, dim, capi.XB_F16, dim * 2
            tb.slot_keys = tb.slot_rows = None
            self.tables.append(tb)
        self.host_feeds, self.feeds = [], []
        for t in range(n_tables):
            counts = rng.integers(1, 31, gpt * B).astype(np.int32)
            n = int(counts.sum())
            ids = workloads.zipf_ids(rng, table_rows, n, 1.05)
            off = np.zeros(len(counts) + 1, np.int32)
            np.cumsum(counts, out=off[1:])
            self.host_feeds.append((ids, off))
            self.feeds.append((torch.from_numpy(ids).cuda(), torch.from_numpy(off).cuda(), n))
        self.ctx = None
        if impl == "abi":
            # the whole step behind the C ABI: one routing problem over all tables, NCCL called by the library
            import torch.distributed as dist
            uid = [sharded.ShardContext.unique_id() if rank == 0 else None]
            if world > 1:
                dist.broadcast_object_list(uid, src=0)
            max_ids = int(1.05 * n_tables * gpt * B * 15.5) + 4096
            self.ctx = sharded.ShardContext(rank, world, self.tables, [gpt * B] * n_tables, dim, max_ids, partial_dtype,
                                            capacity_factor=capacity_factor, unique_id=uid[0])
            self.all_ids = torch.cat([f[0] for f in self.feeds])
            base, parts = 0, []
            for f in self.feeds:
                parts.append(f[1][:-1] + base)
                base += f[2]
            parts.append(torch.full((1,), base, dtype=torch.int32, device="cuda"))
            self.all_off = torch.cat(parts)
            assert self.all_ids.numel() <= max_ids
        self.dims = dims = [n_tables * gpt * dim, 1024, 512, 256, 1]
        wrng = np.random.default_rng(7)                       # the dense weights are replicated: same seed on every rank
        self.W_host = [workloads.fp16_round(wrng.normal(0, 1.0 / dims[i] ** 0.5, (dims[i + 1], dims[i]))) for i in range(4)]
        self.b_host = [workloads.fp16_round(wrng.normal(0, 0.01, dims[i + 1])) for i in range(4)]
        self.Ws = [torch.from_numpy(w).cuda().to(torch.float16) for w in self.W_host]
        self.bs = [torch.from_numpy(b).cuda() for b in self.b_host]
        self.slope = torch.full((1,), 0.25, device="cuda")
        self.pooled = torch.empty((B, dims[0]), dtype=torch.float16, device="cuda")
        self.acts = [torch.empty((B, dims[i + 1]), dtype=torch.float16, device="cuda") for i in range(4)]
        self.phases = []

    def step(self, timed=False):
        torch, ops, capi = self.torch, self.ops, self.capi
        events = []

        def mark(name):
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            events.append((name, e))
        if timed:
            mark("start")
        # the four tables share the ownership rule: one routing pass and one pair of exchanges for all of them
        if self.ctx is not None:
            self.ctx.pool(self.all_ids, self.all_off, self.N_TABLES * self.GPT, self.pooled)
            esz = 2 if self.partial_dtype == "f16" else 4
            stats = {"routed_bytes": self.world * self.ctx.bucket_capacity * 8,
                     "returned_bytes": self.world * self.N_TABLES * self.GPT * self.B * self.DIM * esz}
            if timed:
                mark("sharded_pool")
        else:
            stats = self.sharded.sharded_pool_tables(self.comm, self.gops, self.tables, self.DIM, [f[0] for f in self.feeds],
                                                     [None] * self.N_TABLES, [f[1] for f in self.feeds],
                                                     [self.GPT] * self.N_TABLES, self.pooled, mark=mark if timed else None)
        self.mlp()
        if timed:
            mark("mlp")
            self.phases.append(events)
        return stats

    def mlp(self):
        ops, capi = self.ops, self.capi
        x = self.pooled
        for i in range(4):
            last = i == 3
            ops.gemm(x, self.Ws[i], Y=self.acts[i], bias=self.bs[i], trans_b=True, M=self.B, N=self.dims[i + 1], K=self.dims[i],
                     epilogue=capi.XB_EPI_SIGMOID if last else capi.XB_EPI_PRELU,
                     ep=(None if last else self.slope, None, None), ep_count=0 if last else 1)
            x = self.acts[i]

    def run_pipelined(self, steps):
        """Three steps in flight on three streams: xb_sharded_pool_begin of step i+2 (bucket ids, id exchange),
        xb_sharded_pool_pool of step i+1 (owner pooling, partial-sum exchange) and xb_sharded_pool_combine + MLP of step
        i. Every rank issues them in that order, so the exchanges of the one communicator run in the same order
        everywhere. Returns the CUDA events around `steps` steps on this rank's main stream."""
        torch = self.torch
        if not hasattr(self, "side"):
            self.side = (torch.cuda.Stream(), torch.cuda.Stream())
        s_begin, s_pool = self.side
        main = torch.cuda.current_stream()
        groups = self.N_TABLES * self.GPT
        s_begin.wait_stream(main)
        s_pool.wait_stream(main)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()

        def begin():
            with torch.cuda.stream(s_begin):
                self.ctx.begin(self.all_ids, self.all_off)

        def pool():
            with torch.cuda.stream(s_pool):
                self.ctx.pool_stage()
        begin()
        if steps > 1:
            begin()
        pool()
        for i in range(steps):
            if i + 2 < steps:
                begin()
            if i + 1 < steps:
                pool()
            self.ctx.combine(groups, self.pooled)
            self.mlp()
        e1.record()
        main.wait_stream(s_begin)
        main.wait_stream(s_pool)
        return e0, e1

    def check(self, n_check=48):
        """One step, then this rank's first `n_check` samples against the CPU oracle: pooled vectors (un-sharded
        QuickEmbeddingDict::Get semantics over the rows the hash generator names) and the final sigmoid."""
        import numpy as np
        checker_path()
        import orc
        torch = self.torch
        self.step()
        torch.cuda.synchronize()
        B, dim, gpt = self.B, self.DIM, self.GPT
        want = np.zeros((n_check, self.dims[0]), np.float32)
        mag = np.zeros((n_check, self.dims[0]), np.float32)
        for t, (ids, off) in enumerate(self.host_feeds):
            for g in range(gpt):
                lo, hi = int(off[g * B]), int(off[g * B + n_check])
                seg_ids = ids[lo:hi]
                counts = (off[g * B + 1:g * B + n_check + 1] - off[g * B:g * B + n_check]).astype(np.int32)
                uniq, inv = np.unique(seg_ids, return_inverse=True)
                rows = shard_table_values(t, uniq, dim, np).astype(np.float16).astype(np.float32)
                col = (t * gpt + g) * dim
                ones = np.ones(len(seg_ids), np.float32)
                orc.embedding_pool(rows, inv.astype(np.int64), ones, counts, [dict(udf=0, out=want, col=col)])
                orc.embedding_pool(np.abs(rows), inv.astype(np.int64), ones, counts, [dict(udf=0, out=mag, col=col)])
        got = self.pooled[:n_check].float().cpu().numpy()
        # fp16 partial sums and an fp16 result: a few half-precision roundings of the magnitude sum
        tol = (4.0 if self.partial_dtype == "f16" else 1.0) * 2.0 ** -11
        pooled_rel = float((np.abs(got - want) / np.maximum(mag, 1e-6)).max())
        x = got                                                # the MLP of the oracle reads what the GPU pooled
        for i in range(4):
            x = orc.gemm_op(x, self.W_host[i], self.b_host[i], transb=True)
            x = orc.sigmoid(x) if i == 3 else orc.prelu(x, np.full(1, 0.25, np.float32)).astype(np.float16).astype(np.float32)
        prob_abs = float(np.abs(self.acts[3][:n_check].float().cpu().numpy() - x).max())
        res = torch.tensor([pooled_rel / tol, prob_abs / 2e-3], dtype=torch.float64, device="cuda")
        import torch.distributed as dist
        dist.all_reduce(res, op=dist.ReduceOp.MAX)
        ok = bool(res[0].item() <= 1.0 and res[1].item() <= 1.0)
        return {"ok": ok, "samples_checked_per_rank": n_check, "pooled_max_err_over_tol": float(res[0].item()),
                "pooled_tol_rel_to_magnitude_sum": tol, "prob_max_abs_err": float(res[1].item()) * 2e-3, "prob_tol": 2e-3,
                "oracle": "orc.embedding_pool + orc.gemm_op on the rows the generator names (all ranks, max)"}

    def run(self, steps, warmup):
        import torch.distributed as dist
        torch = self.torch
        parity = self.check()
        if not parity["ok"]:
            # the verdict is the maximum over all ranks, so every rank takes this exit together; nothing is timed
            overflow = bool(self.ctx.overflow()) if self.ctx is not None else False
            return {"error": "row-sharded path differs from the CPU oracle; no timing taken", "parity": parity,
                    "bucket_overflow_on_rank0": overflow, "n_gpus": self.world}
        for _ in range(max(warmup, 3)):
            self.step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier(); torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            stats = self.step()
        e1.record()
        dist.barrier(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        pipelined = None
        if self.ctx is not None:
            serial_prob = self.acts[3].clone()
            for _ in range(2):
                self.run_pipelined(3)
            dist.barrier(); torch.cuda.synchronize()
            p0, p1 = self.run_pipelined(steps)
            dist.barrier(); torch.cuda.synchronize()
            tp = torch.tensor([p0.elapsed_time(p1)], dtype=torch.float64, device="cuda")
            dist.all_reduce(tp, op=dist.ReduceOp.MAX)
            same = torch.tensor([1.0 if torch.equal(serial_prob, self.acts[3]) else 0.0], dtype=torch.float64, device="cuda")
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            pms = float(tp.item()) / steps
            pipelined = {"ms_per_step": pms, "samples_per_s": self.BATCH / (pms * 1e-3),
                         "same_bits_as_one_step_at_a_time": bool(same.item() == 1.0),
                         "how": "three streams: xb_sharded_pool_begin of step i+2, xb_sharded_pool_pool of step i+1, "
                                "xb_sharded_pool_combine + MLP of step i; both exchanges of a step overlap kernels of its "
                                "neighbours"}
        # where a step spends its time on this rank: a few more steps with an event after every phase (outside the
        # timed region; the host gaps between phases show up here too)
        if self.ctx is not None:
            self.ctx.profile(True)
        lib_phases = {}
        for _ in range(5):
            self.step(timed=True)
            if self.ctx is not None:
                torch.cuda.synchronize()
                for k, v in self.ctx.phase_ms().items():
                    lib_phases[k] = lib_phases.get(k, 0.0) + v / 5
        if self.ctx is not None:
            self.ctx.profile(False)
        torch.cuda.synchronize()
        phase_ms = {}
        for events in self.phases:
            for (_, a), (name, b) in zip(events[:-1], events[1:]):
                phase_ms[name] = phase_ms.get(name, 0.0) + a.elapsed_time(b) / len(self.phases)
        assert self.ops.device_status() == 0
        if self.ctx is not None:
            overflowed = bool(self.ctx.overflow())          # reported, and the line then says the step dropped ids
        ms = float(t.item()) / steps
        return {"ms_per_step": ms, "samples_per_s": self.BATCH / (ms * 1e-3), "steps": steps, "n_gpus": self.world,
                "table_rows": self.rows_total, "tables": self.N_TABLES, "dim": self.DIM,
                "ids_per_rank_step": sum(f[2] for f in self.feeds),
                "routed_bytes_per_rank_step": stats["routed_bytes"], "returned_bytes_per_rank_step": stats["returned_bytes"],
                "partial_dtype": self.partial_dtype, "steps_in_flight": pipelined,
                "bucket_overflow": overflowed if self.ctx is not None else False,
                "impl": ("xb_sharded_pool: one C-ABI call per step, NCCL inside the library, fixed-capacity id buckets, "
                         "no host synchronisation" if self.ctx is not None else
                         "python orchestration over torch.distributed (bucket sizes read back every step)"),
                "phase_ms_rank0": dict({k: round(v, 4) for k, v in phase_ms.items()},
                                       **({"inside_sharded_pool": {k: round(v, 4) for k, v in lib_phases.items()}}
                                          if lib_phases else {})),
                "parity": parity, "timing": "max over ranks, CUDA events; MLP 1280-1024-512-256-1 included"}


def run_sharded(args):
    """The row-sharded leg alone. Launch under torch.distributed.run; prints one JSON line on rank 0."""
    import torch
    import torch.distributed as dist
    load_package()
    rank, local_rank, world = dist_env()
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    leg = ShardedLeg(rank, world, args.table_rows, args.partial_dtype, args.sharded_impl, args.capacity_factor)
    out = leg.run(args.steps, args.warmup)
    if rank == 0:
        print(json.dumps(dict({"micro": "sharded"}, **out)))
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--requests", type=int, default=74,
                    help="requests per step (each 1 user x 1000 candidates); 74 requests = 592 attention tiles = 4 x 148 SMs")
    ap.add_argument("--batches", type=int, default=8, help="distinct pre-generated request batches that are cycled")
    ap.add_argument("--serving-threads", type=int, default=4,
                    help="Predictors (one per host thread, each with its own stream) of the end-to-end leg")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline and pooling side measurements")
    ap.add_argument("--table-rows", type=int, default=200_000_000, help="rows per table of the row-sharded leg")
    ap.add_argument("--partial-dtype", default="f16", choices=["f16", "f32"],
                    help="dtype of the partial sums the owners return in the row-sharded leg (f32 for the 1e-5 bar)")
    ap.add_argument("--sharded-impl", default="abi", choices=["abi", "python"],
                    help="row-sharded leg: the one-call C-ABI step (NCCL inside the library) or the Python orchestration")
    ap.add_argument("--capacity-factor", type=float, default=0.0,
                    help="row-sharded leg: id bucket capacity as a multiple of the mean bucket (an overflow is reported, "
                         "never silent); 0 = 1.1 + 0.08 x ranks, which covers the Zipf(1.05) ids of the benchmark (the "
                         "hottest id alone is 8 %% of all ids and lands on one owner)")
    ap.add_argument("--no-sharded", action="store_true", help="skip the row-sharded leg of a multi-GPU run")
    ap.add_argument("--att-engine", type=int, default=0, help="--micro att: 0 library's choice, 2 per-step tcgen05, "
                    "3 paired, 4 split")
    ap.add_argument("--case", default=None, help="--micro pool_hbm: run one case only (shard25m_dim32 | item5m_dim18)")
    ap.add_argument("--micro", choices=["att", "pool", "pool_hbm", "gemm", "gemm_mlp", "tower", "sharded", "batching", "dien"], help="run --steps launches of one kernel on a small case "
                    "(for profiler captures) instead of the benchmark")
    args = ap.parse_args()
    if args.micro == "sharded":
        return run_sharded(args)
    if args.micro == "dien":
        load_package()
        import torch
        torch.cuda.set_device(0)
        print(json.dumps(dict({"micro": "dien"}, **bench_dien(reps=args.steps))))
        return
    if args.micro == "batching":
        return run_batching(args)
    if args.micro:
        return run_micro(args)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
