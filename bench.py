"""CD-k RBM training throughput on B200: `python bench.py --gpus N --steps K --warmup W`.

One "step" is one contrastive-divergence update (positive phase, k Gibbs steps,
statistics, all-reduce when N > 1, momentum update) of the configuration named in
`config.workload`; the metric is training examples per second over all N GPUs.
N > 1 is launched with torchrun (one rank per GPU); torch.distributed (gloo) only
carries the NCCL id, the barrier and the max-over-ranks of the device-timed interval -
the work itself runs in libb200mat.so.

`--impl reference` times the CPU restatement of the reference's eigenmat path (the
oracle: the reference's own C++ needs Eigen, which is not available, so it cannot be
built) on the host cores, on a bounded sample of the same workload.
Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "CD-k RBM training examples/sec"
UNIT = "examples/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=p["hbm_gbs"], tensor=p["bf16_tflops_sustained"], source="measured")
    return dict(hbm=6650.0, tensor=1400.0, source="fallback")


class ClockSampler(object):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.QUERY,
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.25)
        self.proc.terminate()
        clocks, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.samples:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz, mx = float(parts[0]), float(parts[1])
            except ValueError:
                continue
            smax = mx
            if t0 - 0.1 <= ts <= t1 + 0.3:
                clocks.append(mhz)
                for n, v in zip(names, parts[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        med = float(np.median(clocks)) if clocks else None
        return dict(sm_mhz=med, sm_max_mhz=smax, reasons=sorted(reasons), samples=len(clocks))


def make_engine(cm, cfg, world, rank):
    from deepnet_b200.fused_rbm import FusedRBM
    if len(cfg["layers"]) > 2:
        from deepnet_b200.fused_dbm import FusedDBM
        if world > 1:
            raise SystemExit("the DBM configuration is benchmarked on one GPU")
        eng = FusedDBM(cm, [l["numdims"] for l in cfg["layers"]], cfg["batchsize"], [e["weight"] for e in cfg["edges"]],
                       cfg["hyperparams"], seed=cfg["seed"])
        eng.timeline = None
        return eng
    V, H = cfg["layers"][0]["numdims"], cfg["layers"][1]["numdims"]
    return FusedRBM(cm, V, H, cfg["batchsize"], cfg["edges"][0]["weight"], cfg["hyperparams"],
                    edge_hyperparams=cfg["edges"][0].get("hyperparams"), visible=cfg["layers"][0]["activation"],
                    binary_data=cfg["binary"], seed=cfg["seed"], world_size=world, rank=rank)


def workload(config, cases):
    """Model spec and `cases` synthetic training cases (generated here, never read from disk)."""
    from deepnet_b200 import configs, synthetic
    if config == 4:
        # building 10^6 x 8192 cases is neither needed nor possible on the host: a pool of
        # minibatches from the same generator (Bernoulli(p_i), p_i ~ Beta(0.3, 2)) is cycled
        cfg = configs.build(4, cases=4)      # parameters and hyper-parameters only
        data, _ = synthetic.binary_data(8192, cases, 1004)
        cfg["data"] = data
    else:
        cfg = configs.build(config, cases=cases)
    cfg["binary"] = config in (0, 2, 3, 4)   # inputs exact in TF32 (0/1 or small integer counts)
    return cfg


def run_ours(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch N > 1 with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
    from deepnet_b200 import b200mat as cm
    from deepnet_b200 import configs
    cm.cuda_set_device(local)
    cm.cublas_init()
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        dist.init_process_group("gloo", rank=rank, world_size=world)
        ids = [cm.dp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        cm.dp_init(ids[0], world, rank)

    def barrier():
        cm.cuda_sync_threads()
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x):
        if dist is None:
            return x
        import torch
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    config = args.config
    pool = 4
    B = configs.build(config, cases=4)["batchsize"] if config != 4 else 4096
    cfg = workload(config, pool * B)
    if world > 1:
        # each rank trains on its own shard of the global minibatch: different data per rank
        from deepnet_b200 import synthetic
        if config == 4:
            cfg["data"], _ = synthetic.binary_data(8192, pool * B, 1004 + 7919 * rank)
    V, H = cfg["layers"][0]["numdims"], cfg["layers"][1]["numdims"]
    k = cfg["hyperparams"].gibbs_steps
    if config in (2, 3):
        pool = 2
        cfg["data"] = cfg["data"][:, :pool * B]
    eng = make_engine(cm, cfg, world, rank)

    # ---- device-resident inputs --------------------------------------------------------
    dev_batches = [cm.CUDAMatrix(cfg["data"][:, i * B:(i + 1) * B]) for i in range(pool)]
    for s in range(args.warmup):
        eng.TrainOneBatch(s, dev_batches[s % pool])
    eng.read_loss()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    eng.timeline = []
    barrier()
    e0, e1 = cm.Event(), cm.Event()
    t_wall0 = time.time()
    e0.record()
    launches = 0
    for s in range(args.steps):
        eng.TrainOneBatch(args.warmup + s, dev_batches[s % pool])
        launches += eng.kernel_launches
    e1.record()
    ms = e0.elapsed_ms(e1)
    barrier()
    t_wall1 = time.time()
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    timeline, eng.timeline = eng.timeline, None
    loss = eng.read_loss() / (args.steps * B)
    status = cm.read_status()
    ms = max_over_ranks(ms)
    value = args.steps * B * world / (ms * 1e-3)

    # ---- per-kernel figures from the events recorded inside the timed region -------------
    agg = {}
    for name, flops, nbytes, a, b in timeline:
        d = agg.setdefault(name, [0, 0.0, 0.0, 0.0])
        d[0] += 1
        d[1] += a.elapsed_ms(b)
        d[2] += flops
        d[3] += nbytes
    peaks = measured_peaks()
    gemm_ms = sum(v[1] for n, v in agg.items() if n.startswith("gemm"))
    gemm_flops = sum(v[2] for n, v in agg.items() if n.startswith("gemm"))
    # tensor-pipe work per algorithmic product, in half-precision terms (each the flops of the product
    # at the fp16/bf16 rate): up = hi.lo + lo.hi + hi.hi, down (0/1 samples) = two terms, statistics =
    # positive half (0/1 data) two + negative half three
    kg = float(getattr(getattr(eng, "hyp", None), "gibbs_steps", 1))
    passes = {"gemm_up": (3 * kg + 2) / (kg + 1), "gemm_down": 2, "gemm_stats": 2.5}   # the first up product reads 0/1 data
    hw_flops = sum(v[2] * passes.get(n, 1) for n, v in agg.items() if n.startswith("gemm"))
    kernels = {n: dict(launches=v[0], ms_per_launch=round(v[1] / v[0], 5),
                       tflops=round(v[2] / (v[1] * 1e-3) / 1e12, 2) if v[2] else None,
                       gbs=round(v[3] / (v[1] * 1e-3) / 1e9, 1) if v[3] else None) for n, v in agg.items()}
    # dominant kernel: the up half-step product (k_gemm_tc, sigmoid + Bernoulli epilogue),
    # the largest share of the step.  achieved = algorithmic flops of one launch (2 V H B)
    # / its mean CUDA-event duration inside the timed region.
    up = agg.get("gemm_up")
    if up is None:
        # no per-launch events for this engine: algorithmic flops of the whole update / its time
        achieved = configs.flops_per_example(config) * B / (ms / args.steps * 1e-3) / 1e12
        roofline = dict(bound="tensor", achieved=round(achieved, 3), peak=peaks["tensor"], unit="TFLOP/s",
                        frac=round(achieved / peaks["tensor"], 5), traffic=None,
                        kernel="k_gemm_tc (whole update; launch-latency-bound at this size)",
                        peak_source="%s bf16 dense sustained (MEASURED_PEAKS.json)" % peaks["source"])
    else:
      achieved = up[2] / (up[1] * 1e-3) / 1e12
      roofline = dict(bound="tensor", achieved=round(achieved, 2), peak=peaks["tensor"], unit="TFLOP/s",
                      frac=round(achieved / peaks["tensor"], 4),
                      # dram__bytes_read.sum + dram__bytes_write.sum of one such launch at this workload
                      # (ncu capture summarised in profiles/k_gemm_tc_up_c4.md); other workloads: not captured
                      traffic=1.43e9 if config == 4 else None,
                      kernel="k_gemm_tc<256, sigmoid+Bernoulli> (tcgen05 kind::f16: three fp16 terms hi.lo + lo.hi "
                             "+ hi.hi on x * 2^e = hi + lo per k-block, paired CTAs)",
                      peak_source="%s bf16 dense sustained (MEASURED_PEAKS.json); three half-precision terms "
                                  "make one fp32-grade product" % peaks["source"],
                      launches=up[0], ms_per_launch=round(up[1] / up[0], 4),
                      share_of_step=round(up[1] / ms, 4) if world == 1 else None,
                      all_gemm_algorithmic_tflops=round(gemm_flops / (gemm_ms * 1e-3) / 1e12, 2),
                      all_gemm_issued_f16_tflops=round(hw_flops / (gemm_ms * 1e-3) / 1e12, 2),
                      all_gemm_share_of_step=round(gemm_ms / ms, 4) if world == 1 else None)

    # ---- end to end: host batches in, loss out, every step --------------------------------
    host = []
    for i in range(2):
        arr, ptr = cm.host_alloc((V, B))
        arr[...] = cfg["data"][:, i * B:(i + 1) * B]
        host.append((arr, ptr))
    stage = [cm.empty((V, B)), cm.empty((V, B))]
    nbytes = V * B * 4
    e2e_steps = max(2, min(args.steps, 10))
    barrier()
    stage[0].prefetch_from_pinned(host[0][1], nbytes)
    f0, f1 = cm.Event(), cm.Event()
    f0.record()
    for s in range(e2e_steps):
        cm.prefetch_wait()                                  # this step's batch has landed
        if s + 1 < e2e_steps:                               # next batch travels during this step
            cm.prefetch_fence()
            stage[(s + 1) & 1].prefetch_from_pinned(host[(s + 1) & 1][1], nbytes)
        eng.TrainOneBatch(args.warmup + args.steps + s, stage[s & 1])
        eng.read_loss()                                     # device -> host, every step
    f1.record()
    e2e_ms = max_over_ranks(f0.elapsed_ms(f1))
    e2e_value = e2e_steps * B * world / (e2e_ms * 1e-3)
    for _, ptr in host:
        cm.host_free(ptr)

    out = None
    if rank == 0:
        out = dict(metric=METRIC, value=round(value, 1), unit=UNIT, n_gpus=world, steps=args.steps,
                   warmup=args.warmup, ms_per_step=round(ms / args.steps, 4), higher_is_better=True, scaling="weak",
                   vs_baseline=None, dtype="f32", data="synthetic",
                   config=dict(workload=cfg["name"], visible=V, hidden=H, batch_per_gpu=B, global_batch=B * world,
                               gibbs_steps=k, parallelism="dp%d" % world,
                               cache="working set (weights 268 MB x3, states) exceeds the 126 MB L2; no flush needed"
                               if config == 4 else "small working set: L2-resident, as in training"),
                   clocks=clocks, gpu_launches=launches,
                   e2e=dict(value=round(e2e_value, 1), unit=UNIT, h2d_bytes_per_step=nbytes, d2h_bytes_per_step=4,
                            steps=e2e_steps),
                   roofline=roofline, kernels=kernels, mean_sq_error_per_case=round(loss, 4), device_status=status)
    if dist is not None:
        cm.dp_destroy()
        dist.destroy_process_group()
    return out


def cpu_step_rate(config, sample_batch, steps, warmup, threads):
    """examples/s of the oracle (per-call eigenmat path) at batch `sample_batch`, full layer sizes.

    Every timed update starts from the initial parameters: once the visible probabilities of
    the sparse synthetic data underflow to denormals (from the second update on at this
    learning rate) the CPU's sgemm slows down about twentyfold, which would say more about
    denormal handling than about the path.
    """
    os.environ.setdefault("OMP_NUM_THREADS", str(threads))
    os.environ.setdefault("OPENBLAS_NUM_THREADS", str(threads))
    from oracle import eigenmat_oracle as em
    from deepnet_b200 import dbm
    cfg = workload(config, sample_batch * 2)
    m = dbm.DBM(em, cfg["layers"], cfg["edges"], cfg["hyperparams"], sample_batch, cfg["optimizer"], seed=cfg["seed"])
    data = em.CUDAMatrix(cfg["data"])
    w0 = [np.array(e.params["weight"].asarray(), copy=True) for e in m.edge]
    times = []
    for s in range(warmup + steps):
        for e, w in zip(m.edge, w0):
            e.params["weight"].overwrite(w)
            e.gradient_history.assign(0)
        for l in m.layer:
            l.params["bias"].assign(0)
            l.gradient_history.assign(0)
        m.SetBatch([data.slice((s & 1) * sample_batch, ((s & 1) + 1) * sample_batch)])
        t = time.perf_counter()
        m.TrainOneBatch(0)
        times.append(time.perf_counter() - t)
    dt = sum(times[warmup:]) / steps
    return sample_batch / dt, dt, cfg


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    cores = os.cpu_count() or 1
    sample_batch = 256 if args.config == 4 else None
    from deepnet_b200 import configs
    if sample_batch is None:
        sample_batch = configs.build(args.config, cases=4)["batchsize"]
    steps = max(1, min(args.steps, 3))
    warm = 1
    rate, dt, cfg = cpu_step_rate(args.config, sample_batch, steps, warm, cores)
    V, H = cfg["layers"][0]["numdims"], cfg["layers"][1]["numdims"]
    sample = "%d timed CD-%d updates at batch %d (full %dx%d layers) on %d host threads" % (
        steps, cfg["hyperparams"].gibbs_steps, sample_batch, V, H, cores)
    return dict(impl="reference", metric=METRIC, value=round(rate, 2), unit=UNIT, n_gpus=args.gpus, steps=steps,
                warmup=warm, ms_per_step=round(dt * 1e3, 2), higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype="f32", data="synthetic",
                config=dict(workload=cfg["name"], visible=V, hidden=H, batch_per_gpu=sample_batch,
                            gibbs_steps=cfg["hyperparams"].gibbs_steps, parallelism="cpu"),
                cpu_baseline=dict(value=round(rate, 2), unit=UNIT, cores=cores, kind="port", sample=sample),
                e2e=dict(value=round(rate, 2), unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=4, help="benchmark configuration 0..4 (default 4, the headline)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.config not in (0, 1, 2, 3, 4):
        raise SystemExit("--config must be 0..4")
    if args.impl == "reference":
        out = run_reference(args)
        if out is not None:
            print(json.dumps(out), flush=True)
        return
    args.warmup = max(args.warmup, 3)
    out = run_ours(args)
    if out is None:
        return
    if args.gpus == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        sample_batch = 256 if args.config == 4 else out["config"]["batch_per_gpu"]
        rate, dt, cfg = cpu_step_rate(args.config, sample_batch, 1, 1, cores)
        out["cpu_baseline"] = dict(value=round(rate, 2), unit=UNIT, cores=cores, kind="port",
                                   sample="1 timed CD-%d update at batch %d (full layer sizes), %.1f s" % (
                                       cfg["hyperparams"].gibbs_steps, sample_batch, dt))
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
