"""CD-k RBM training throughput on B200: `python bench.py --gpus N --steps K --warmup W`.

One "step" is one contrastive-divergence update (positive phase, k Gibbs steps,
statistics, all-reduce when N > 1, momentum update) of the configuration named in
`config.workload`; the metric is training examples per second over all N GPUs.
N > 1 is launched with one process per GPU (torchrun or any launcher that sets RANK /
LOCAL_RANK / WORLD_SIZE); the ranks find each other through a file and NCCL
(deepnet_b200/rendezvous.py) - no framework is imported, the work runs in libb200mat.so.

`value` times K plain updates; a second pass of K updates with CUDA events around every
launch gives the per-kernel table and `roofline` (so the headline carries no
instrumentation).  `e2e` feeds every update from pinned host memory and reads the loss back.

`--impl reference` times the CPU restatement of the reference's eigenmat path (the
oracle: the reference's own C++ needs Eigen, which is not available, so it cannot be
built) on the host cores, on a bounded sample of the same workload (the same batch and layer sizes, a few updates), in a child process
whose thread count is set explicitly.  Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time
import zlib

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "CD-k RBM training examples/sec"
UNIT = "examples/s"

# DRAM bytes read + written by one launch of the dominant kernel (the up half-step product of
# configuration 4) in the ncu capture of this build; other workloads were not captured.
UP_PRODUCT_DRAM_BYTES_C4 = 1.33e9
RAMP_SECONDS = 0.6     # load applied before the warm-up updates so that the GPU is at its steady clocks


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=p["hbm_gbs"], tensor=p["bf16_tflops_sustained"], tensor_burst=p.get("bf16_tflops"),
                    source="measured")
    return dict(hbm=6650.0, tensor=1400.0, tensor_burst=1590.0, source="fallback")


class ClockSampler(object):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.samples = []
        self.proc = None

    def start(self):
        if os.environ.get("B200_BENCH_SAMPLER") == "none":
            return
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


def ramp_updates(config):
    """Updates that make up about RAMP_SECONDS of load at each configuration's speed
    (B200_BENCH_RAMP overrides the count: 0 keeps a profiler capture short)."""
    if os.environ.get("B200_BENCH_RAMP"):
        return int(os.environ["B200_BENCH_RAMP"])
    return 30 if config == 4 else 1000


def make_engine(cm, cfg, world, rank, group=None):
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
                    binary_data=cfg["binary"], seed=cfg["seed"], world_size=world, rank=rank, group=group)


def workload(config, cases, data_seed=None):
    """Model spec and `cases` synthetic training cases (generated here, never read from disk)."""
    from deepnet_b200 import configs, synthetic
    if config == 4:
        # building 10^6 x 8192 cases is neither needed nor possible on the host: a pool of
        # minibatches from the same generator (Bernoulli(p_i), p_i ~ Beta(0.3, 2)) is cycled
        cfg = configs.build(4, cases=4)      # parameters and hyper-parameters only
        data, _ = synthetic.binary_data(8192, cases, 1004 if data_seed is None else data_seed)
        cfg["data"] = data
    else:
        cfg = configs.build(config, cases=cases)
    cfg["binary"] = config in (0, 2, 3, 4)   # inputs exact in TF32 (0/1 or small integer counts)
    return cfg


def time_updates(cm, eng, batches, first_step, steps, group):
    """K plain updates between two CUDA events on the library stream -> (ms, launches)."""
    group.barrier()
    e0, e1 = cm.Event(), cm.Event()
    e0.record()
    launches = 0
    for s in range(steps):
        eng.TrainOneBatch(first_step + s, batches[s % len(batches)])
        launches += eng.kernel_launches
    e1.record()
    ms = e0.elapsed_ms(e1)
    group.barrier()
    return group.max(ms), launches


def small_config_line(cm, config, steps, warmup):
    """examples/s, ms per update and algorithmic TFLOP/s of one of the small configurations (1 GPU)."""
    from deepnet_b200 import configs
    from deepnet_b200.rendezvous import Group
    B = configs.build(config, cases=4)["batchsize"]
    pool = 2 if config in (2, 3) else 4
    cfg = workload(config, pool * B)
    cm.set_rng_column_offset(0)
    eng = make_engine(cm, cfg, 1, 0)
    batches = [cm.CUDAMatrix(cfg["data"][:, i * B:(i + 1) * B]) for i in range(pool)]
    ramp = ramp_updates(config)
    for s in range(ramp + warmup):
        eng.TrainOneBatch(s, batches[s % pool])
    eng.read_loss()
    ms, launches = time_updates(cm, eng, batches, ramp + warmup, steps, Group(cm, 1, 0))
    loss = eng.read_loss() / (steps * B)
    per = ms / steps
    return dict(workload=cfg["name"], value=round(B / (per * 1e-3), 1), unit=UNIT, ms_per_step=round(per, 4),
                steps=steps, algorithmic_tflops=round(configs.flops_per_example(config) * B / (per * 1e-3) / 1e12, 3),
                gpu_launches_per_step=launches // steps, mean_sq_error_per_case=round(loss, 4))


def tf32_peak(cm, peaks):
    """TFLOP/s of this library's own one-term kind::tf32 product at the headline product's size
    (8192 x 4096 x 8192): the tensor pipe's TF32 rate as this box delivers it, next to the
    driver-measured bf16 figure (TF32 runs at half the bf16 rate by design)."""
    rng = np.random.default_rng(1)
    n = 8192
    a = cm.CUDAMatrix((rng.standard_normal((n, n)) * 0.01).astype(np.float32))
    b = cm.CUDAMatrix(rng.random((n, 4096), dtype=np.float32))
    out = cm.empty((n, 4096))
    cm.set_gemm_path(1)
    cm.set_dot_precision(1)
    try:
        for _ in range(3):
            cm.dot(a.T, b, target=out)
        e0, e1 = cm.Event(), cm.Event()
        reps = 10
        e0.record()
        for _ in range(reps):
            cm.dot(a.T, b, target=out)
        e1.record()
        ms = e0.elapsed_ms(e1) / reps
    finally:
        cm.set_dot_precision(0)
        cm.set_gemm_path(0)
    for m in (a, b, out):
        m.free_device_memory()
    return 2.0 * n * n * 4096 / (ms * 1e-3) / 1e12


def run_ours(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world and world == 1 and args.gpus > 1:
        raise SystemExit("launch N > 1 with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
    from deepnet_b200 import b200mat as cm
    from deepnet_b200 import configs
    from deepnet_b200.rendezvous import Group
    cm.cuda_set_device(local)
    cm.cublas_init()
    group = Group(cm, world, rank)

    config = args.config
    pool = 4
    B = configs.build(config, cases=4)["batchsize"] if config != 4 else 4096
    # each rank trains on its own shard of the global minibatch: different data per rank
    cfg = workload(config, pool * B, data_seed=1004 + 7919 * rank if world > 1 else None)
    V, H = cfg["layers"][0]["numdims"], cfg["layers"][1]["numdims"]
    k = cfg["hyperparams"].gibbs_steps
    if config in (2, 3):
        pool = 2
        cfg["data"] = cfg["data"][:, :pool * B]
    eng = make_engine(cm, cfg, world, rank, group)

    # ---- device-resident inputs: the headline ------------------------------------------
    dev_batches = [cm.CUDAMatrix(cfg["data"][:, i * B:(i + 1) * B]) for i in range(pool)]
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)                  # the sampler is running before the GPU is (an idle GPU has to ramp up again)
    # A GPU that comes out of idle needs about half a second of load before its clocks and power
    # management settle: the first 10-20 updates of configuration 4 run 5-7 % slower than the
    # steady state (21.0 against 19.7 ms measured with 3 and with 25 updates before the timed ones).
    # So the engine first runs about RAMP_SECONDS of updates, then the W warm-up updates, then the timed ones.
    ramp = ramp_updates(config)          # the same count on every rank (each update is a collective when N > 1)
    for r in range(ramp):
        eng.TrainOneBatch(r, dev_batches[r % pool])
        if r % 8 == 7:
            cm.cuda_sync_threads()
    for s in range(args.warmup):         # warm-up directly before the timed region
        eng.TrainOneBatch(ramp + s, dev_batches[s % pool])
    eng.read_loss()
    t_wall0 = time.time()
    ms, launches = time_updates(cm, eng, dev_batches, ramp + args.warmup, args.steps, group)
    t_wall1 = time.time()
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    loss = eng.read_loss() / (args.steps * B)
    value = args.steps * B * world / (ms * 1e-3)

    # ---- the same updates again with CUDA events around every launch: the per-kernel table -----
    eng.timeline = []
    group.barrier()
    g0, g1 = cm.Event(), cm.Event()
    g0.record()
    for s in range(args.steps):
        eng.TrainOneBatch(ramp + args.warmup + args.steps + s, dev_batches[s % pool])
    g1.record()
    inst_ms = g0.elapsed_ms(g1)
    timeline, eng.timeline = eng.timeline, None
    eng.read_loss()
    status = cm.read_status()
    agg = {}
    for name, flops, nbytes, a, b in timeline or []:
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
    kg = float(k)
    passes = {"gemm_up": (3 * kg + 2) / (kg + 1), "gemm_down": 2, "gemm_stats": 2.5}   # the first up product reads 0/1 data
    hw_flops = sum(v[2] * passes.get(n, 1) for n, v in agg.items() if n.startswith("gemm"))
    kernels = {n: dict(launches=v[0], ms_per_launch=round(v[1] / v[0], 5),
                       tflops=round(v[2] / (v[1] * 1e-3) / 1e12, 2) if v[2] else None,
                       gbs=round(v[3] / (v[1] * 1e-3) / 1e9, 1) if v[3] else None) for n, v in agg.items()}
    tf32 = None
    if rank == 0 and config == 4 and not args.no_tf32_peak:
        tf32 = tf32_peak(cm, peaks)
    # dominant kernel: the up half-step product (k_gemm_tc, sigmoid + Bernoulli epilogue),
    # the largest share of the step.  achieved = algorithmic flops of one launch (2 V H B)
    # / its mean CUDA-event duration.
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
                        traffic=UP_PRODUCT_DRAM_BYTES_C4 if config == 4 else None,
                        traffic_source="ncu dram__bytes_read.sum + dram__bytes_write.sum, one launch" if config == 4 else None,
                        kernel="k_gemm_tc<256, sigmoid+Bernoulli> (tcgen05 kind::f16: three fp16 terms hi.lo + lo.hi "
                               "+ hi.hi on x * 2^e = hi + lo per k-block, paired CTAs)",
                        peak_source="%s bf16 dense sustained (MEASURED_PEAKS.json); three half-precision terms "
                                    "make one fp32-grade product" % peaks["source"],
                        frac_of_bf16_burst=round(achieved / peaks["tensor_burst"], 4) if peaks.get("tensor_burst") else None,
                        tf32_peak_measured=round(tf32, 1) if tf32 else None,
                        tf32_peak_source="this library's one-term kind::tf32 product, 8192 x 4096 x 8192, same run" if tf32 else None,
                        frac_of_tf32_measured=round(achieved / tf32, 4) if tf32 else None,
                        launches=up[0], ms_per_launch=round(up[1] / up[0], 4),
                        share_of_step=round(up[1] / inst_ms, 4) if world == 1 else None,
                        all_gemm_algorithmic_tflops=round(gemm_flops / (gemm_ms * 1e-3) / 1e12, 2),
                        all_gemm_issued_f16_tflops=round(hw_flops / (gemm_ms * 1e-3) / 1e12, 2),
                        all_gemm_share_of_step=round(gemm_ms / inst_ms, 4) if world == 1 else None,
                        instrumented_ms_per_step=round(inst_ms / args.steps, 4))

    # ---- end to end: host batches in, loss out, every step --------------------------------
    host = []
    for i in range(2):
        arr, ptr = cm.host_alloc((V, B))
        arr[...] = cfg["data"][:, i * B:(i + 1) * B]
        host.append((arr, ptr))
    stage = [cm.empty((V, B)), cm.empty((V, B))]
    nbytes = V * B * 4
    e2e_steps = max(2, min(args.steps, 10))
    group.barrier()
    cm.cuda_sync_threads()                                  # nothing in flight: the first copy starts inside the timed region
    f0, f1 = cm.Event(), cm.Event()
    f0.record()
    stage[0].prefetch_from_pinned(host[0][1], nbytes)       # the first step waits for its own batch, the later ones overlap theirs
    for s in range(e2e_steps):
        cm.prefetch_wait()                                  # this step's batch has landed
        if s + 1 < e2e_steps:                               # next batch travels during this step
            cm.prefetch_fence()
            stage[(s + 1) & 1].prefetch_from_pinned(host[(s + 1) & 1][1], nbytes)
        eng.TrainOneBatch(ramp + args.warmup + 2 * args.steps + s, stage[s & 1])
        eng.loss_begin(s & 1)                               # device -> host, every step, behind the update
        if s > 0:
            eng.loss_end((s - 1) & 1)                       # the previous update's loss has arrived
    eng.loss_end((e2e_steps - 1) & 1)
    f1.record()
    e2e_ms = group.max(f0.elapsed_ms(f1))
    e2e_value = e2e_steps * B * world / (e2e_ms * 1e-3)
    for _, ptr in host:
        cm.host_free(ptr)

    # ---- the same loop with the host batches in the data feed's own format: 0/1 data one bit per value
    # (4 MB instead of 134 MB per update over PCIe), unpacked on the device by the feed's gather kernel,
    # which also writes the batch's 16-bit parts.  An extra figure; `e2e` above is the fp32 host path.
    e2e_packed = None
    if cfg["binary"] and config == 4 and getattr(eng, "f16", False):
        words = (V + 31) // 32
        hostp = []
        for i in range(2):
            arr, ptr = cm.host_alloc((words, B))
            bits = np.zeros((B, words * 32), np.uint8)
            bits[:, :V] = cfg["data"][:, i * B:(i + 1) * B].T
            arr[...] = np.ascontiguousarray(np.packbits(bits, axis=1, bitorder="little").view("<u4").T).view(np.float32)
            hostp.append((arr, ptr))
        stagep = [cm.empty((words, B)), cm.empty((words, B))]
        batch, batch_aux = cm.empty((V, B)), cm.empty_aux((V, B))
        pbytes = words * B * 4
        group.barrier()
        cm.cuda_sync_threads()
        p0, p1 = cm.Event(), cm.Event()
        p0.record()
        stagep[0].prefetch_from_pinned(hostp[0][1], pbytes)
        for s in range(e2e_steps):
            cm.prefetch_wait()
            if s + 1 < e2e_steps:
                cm.prefetch_fence()
                stagep[(s + 1) & 1].prefetch_from_pinned(hostp[(s + 1) & 1][1], pbytes)
            cm.feed_gather(stagep[s & 1], True, V, (0, 0), False, 0, batch, out_aux=batch_aux, aux_mode=2, aux_exp=14)
            eng.TrainOneBatch(ramp + args.warmup + 3 * args.steps + s, batch, batch_aux)
            eng.loss_begin(s & 1)
            if s > 0:
                eng.loss_end((s - 1) & 1)
        eng.loss_end((e2e_steps - 1) & 1)
        p1.record()
        pms = group.max(p0.elapsed_ms(p1))
        e2e_packed = dict(value=round(e2e_steps * B * world / (pms * 1e-3), 1), unit=UNIT, h2d_bytes_per_step=pbytes,
                          d2h_bytes_per_step=4, steps=e2e_steps,
                          note="host batches bit-packed (the data feed's storage format), unpacked by feed_gather on the device")
        for _, ptr in hostp:
            cm.host_free(ptr)

    # ---- replicas: every rank applied the same all-reduced statistics, so the parameters must
    # be the same bits everywhere (checksum of W per rank, compared on every rank)
    replicas_identical = None
    if world > 1 and hasattr(eng, "W") and not isinstance(eng.W, list):
        crc = zlib.crc32(np.ascontiguousarray(np.array(eng.W.asarray())).tobytes())
        lo, hi = group.gather(float(crc & 0xffff)), group.gather(float(crc >> 16))
        replicas_identical = len(set(zip(lo, hi))) == 1

    out = None
    if rank == 0:
        out = dict(metric=METRIC, value=round(value, 1), unit=UNIT, n_gpus=world, steps=args.steps,
                   warmup=args.warmup, ms_per_step=round(ms / args.steps, 4), higher_is_better=True, scaling="weak",
                   vs_baseline=None, dtype="f32", data="synthetic",
                   config=dict(workload=cfg["name"], visible=V, hidden=H, batch_per_gpu=B, global_batch=B * world,
                               gibbs_steps=k, parallelism="dp%d" % world, ramp_up_updates=ramp,
                               exchange=("none" if world == 1 else ("peer-memory reduce + update kernel" if getattr(eng, "dp_peer", False)
                                                                    else "NCCL all-reduce")),
                               cache="working set (weights 268 MB x3, states) exceeds the 126 MB L2; no flush needed"
                               if config == 4 else "small working set: L2-resident, as in training"),
                   clocks=clocks, gpu_launches=launches,
                   e2e=dict(value=round(e2e_value, 1), unit=UNIT, h2d_bytes_per_step=nbytes, d2h_bytes_per_step=4,
                            steps=e2e_steps),
                   roofline=roofline, kernels=kernels, mean_sq_error_per_case=round(loss, 4), device_status=status)
        if replicas_identical is not None:
            out["replicas_identical"] = replicas_identical
        if e2e_packed is not None:
            out["e2e_packed"] = e2e_packed
    if hasattr(eng, "close"):
        eng.close(group)                 # (peer-memory exchange: unmapped only when no rank can still store into a replica)
    group.barrier()
    group.close()
    if rank == 0 and world == 1 and config == 4 and not args.no_other_configs:
        # the other configurations of the benchmark set, a few updates each (1 GPU)
        del eng, dev_batches, stage
        out["other_configs"] = [small_config_line(cm, c, 50, 5) for c in (0, 1, 2, 3)]
    return out


# ---- CPU arm ------------------------------------------------------------------------------
def cpu_worker(args):
    """Runs inside a child process whose environment fixed the thread counts before numpy loaded.
    Times the oracle (per-call eigenmat path) at batch `--cpu-batch`, full layer sizes.

    Every timed update starts from the initial parameters: once the visible probabilities of
    the sparse synthetic data underflow to denormals (from the second update on at this
    learning rate) the CPU's sgemm slows down about twentyfold, which would say more about
    denormal handling than about the path.
    """
    import threadpoolctl
    from oracle import eigenmat_oracle as em
    from deepnet_b200 import dbm
    sample_batch, steps, warmup = args.cpu_batch, args.steps, args.warmup
    cfg = workload(args.config, sample_batch * 2)
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
    blas = [p["num_threads"] for p in threadpoolctl.threadpool_info() if p.get("user_api") == "blas"]
    V, H = cfg["layers"][0]["numdims"], cfg["layers"][1]["numdims"]
    print(json.dumps(dict(rate=sample_batch / dt, dt=dt, blas_threads=max(blas) if blas else None,
                          omp_threads=int(os.environ.get("OMP_NUM_THREADS", "0")), name=cfg["name"], V=V, H=H,
                          gibbs_steps=cfg["hyperparams"].gibbs_steps, batch=sample_batch)), flush=True)


def cpu_arm(config, sample_batch, steps, warmup, threads):
    """The CPU path on `threads` host threads, in a child whose thread counts are set explicitly (a
    launcher's OMP_NUM_THREADS=1 must not decide what the baseline runs on)."""
    env = dict(os.environ)
    for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        env[var] = str(threads)
    env["OMP_WAIT_POLICY"] = "passive"
    cmd = [sys.executable, os.path.abspath(__file__), "--cpu-worker", "--config", str(config), "--cpu-batch",
           str(sample_batch), "--steps", str(steps), "--warmup", str(warmup)]
    res = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, text=True, check=True)
    r = json.loads(res.stdout.strip().splitlines()[-1])
    r["threads"] = r["blas_threads"] or threads
    return r


def cpu_sample_batch(config, one_thread=False):
    """The configuration's own minibatch (4096 cases at config 4: one CD-10 update is 12.6 TFLOP, a quarter
    of a minute on 16 host threads); the single-thread figure of config 4 is taken on 256 cases."""
    from deepnet_b200 import configs
    if config == 4:
        return 256 if one_thread else 4096
    return configs.build(config, cases=4)["batchsize"]


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    cores = os.cpu_count() or 1
    threads = args.cpu_threads or cores
    sample_batch = cpu_sample_batch(args.config)
    steps = max(1, min(args.steps, 3))
    warm = 1
    r = cpu_arm(args.config, sample_batch, steps, warm, threads)
    rate, dt = r["rate"], r["dt"]
    sample = "%d timed CD-%d updates at batch %d (full %dx%d layers) on %d host threads (of %d cores)" % (
        steps, r["gibbs_steps"], sample_batch, r["V"], r["H"], r["threads"], cores)
    return dict(impl="reference", metric=METRIC, value=round(rate, 2), unit=UNIT, n_gpus=args.gpus, steps=steps,
                warmup=warm, ms_per_step=round(dt * 1e3, 2), higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype="f32", data="synthetic",
                config=dict(workload=r["name"], visible=r["V"], hidden=r["H"], batch_per_gpu=sample_batch,
                            gibbs_steps=r["gibbs_steps"], parallelism="cpu"),
                cpu_baseline=dict(value=round(rate, 2), unit=UNIT, cores=r["threads"], kind="port", sample=sample),
                e2e=dict(value=round(rate, 2), unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=4, help="benchmark configuration 0..4 (default 4, the headline)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true")
    ap.add_argument("--no-tf32-peak", action="store_true")
    ap.add_argument("--cpu-threads", type=int, default=0, help="host threads of the CPU arm (default: all cores)")
    ap.add_argument("--cpu-worker", action="store_true", help=argparse.SUPPRESS)
    ap.add_argument("--cpu-batch", type=int, default=256, help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.config not in (0, 1, 2, 3, 4):
        raise SystemExit("--config must be 0..4")
    if args.cpu_worker:
        return cpu_worker(args)
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
        sample_batch, one_batch = cpu_sample_batch(args.config), cpu_sample_batch(args.config, one_thread=True)
        warm = 0 if args.config == 4 else 1          # (one update of config 4 is already 15-35 s of CPU work)
        r = cpu_arm(args.config, sample_batch, 1, warm, cores)
        one = cpu_arm(args.config, one_batch, 1, warm, 1)
        what = "1 timed CD-%d update at batch %%d (full layer sizes)" % r["gibbs_steps"]
        out["cpu_baseline"] = dict(
            value=round(r["rate"], 2), unit=UNIT, cores=r["threads"], kind="port",
            sample="%s, %.1f s on %d threads" % (what % sample_batch, r["dt"], r["threads"]),
            # the reference's own build never enables OpenMP (eigenmat/Makefile): its path runs on one thread
            one_thread=dict(value=round(one["rate"], 2), unit=UNIT, cores=one["threads"],
                            sample="%s, %.1f s on 1 thread" % (what % one_batch, one["dt"])))
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
