"""Benchmark of the MoE block: tokens/s of one layer pass.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c3|c2|c2s|c3s|c4|c5|tiny] [--no-extra] [--no-cpu-baseline]

A step is one pass of the block (router -> top-4 -> permutation -> grouped
gate_up + SwiGLU -> grouped down -> combine + residual) over one batch of
seeded synthetic tokens.  One JSON line is printed by rank 0.

The default workload at every N is the gpt-oss-120b-shape layer ("c3": 128 experts,
T = 6144 tokens per GPU), the configuration the target of the benchmark description is
quoted on: all experts local at N = 1; at N > 1 the experts are sharded over the ranks
(expert e on rank e % N) and every rank brings its own 6144 tokens (weak scaling), rows
read from peer memory over NVLink or sent with NCCL.  The line then also carries the
strong-scaling reading (the 6144 tokens split over the ranks), the NCCL transport, and
"ep_parity": 32 tokens of every rank against the CPU code and the two transports
against each other.  At N = 1 the same line carries "layer_20b" (configuration 2: 32
experts, T = 7168) and "decode_mxfp4" (configuration 4: MXFP4 weights, T = 64 / 256 /
1024, Zipf-skewed router), each with its own roofline.

Other workloads (each prints its own line):
  c2    the 20b-shape layer as the headline workload (N > 1: not sharded, 32 experts
        split like any other count that N divides)
  c2s   a quarter-size 20b-shape layer (8 experts, T = 1792) for profiler captures
  c3s   an eighth-size 120b-shape layer (16 experts, T = 768: the same 192 rows per
        expert) for profiler captures of the GEMMs
  c3r   the 120b-shape routing problem (T = 6144, 128 experts) with narrow experts, for
        profiler captures of the router, permutation and combine kernels
  c4    the MXFP4 decode shapes as their own line
  c5    one decode step of the full 120b-architecture model (36 layers, 6144
        sequences with 512 positions of KV context), experts sharded over N >= 2 GPUs,
        with the MoE share of the step time
  tiny  a 16-token layer (smoke runs)

--impl reference times the reference's own CPU code (oracle/_ref when it was
built from the reference tree, else the C port in oracle/) on all host cores, on
a bounded sample of the same workload per step.
"""
from __future__ import annotations

import argparse
import json
import os

# The CPU legs (reference arm, CPU baseline, parity checks) use every core this process may
# run on; a launcher that pins OMP_NUM_THREADS to 1 (torch.distributed.run does) must not
# decide that, and the OpenMP runtime reads the variable when it is first loaded - which
# importing numpy or torch may already do - so it is set before any other import.
os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
import pathlib
import statistics
import sys
import threading
import time

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"


def read_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


def nvml_handle(cuda_index):
    """NVML handle of a CUDA device, found by its PCI address (NVML may list GPUs the process
    cannot see, in another order); falls back to the index.  Read-only use."""
    import pynvml

    pynvml.nvmlInit()
    try:
        import torch

        p = torch.cuda.get_device_properties(cuda_index)
        bus = "%08x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
        return pynvml, pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
    except Exception:
        return pynvml, pynvml.nvmlDeviceGetHandleByIndex(cuda_index)


def run_near_gpu(cuda_index):
    """Restrict this process to the CPUs NVML names as near the GPU, so that the pinned host
    buffers it allocates from here on sit on that socket's memory.  Returns the CPU count."""
    try:
        nv, h = nvml_handle(cuda_index)
        words = nv.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        near = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        near &= os.sched_getaffinity(0)
        if near:
            os.sched_setaffinity(0, near)
        return len(os.sched_getaffinity(0))
    except Exception:
        return None


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs
    (read-only queries)."""

    def __init__(self, index, period=0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.stop_flag = [], set(), False
        self.max_mhz = None
        try:
            self.nv, self.dev = nvml_handle(index)
            self.max_mhz = self.nv.nvmlDeviceGetMaxClockInfo(self.dev, self.nv.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if not self.nv:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksEventReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksEventReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksEventReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksEventReasonSwPowerCap: "sw_power_cap",
        }
        while not self.stop_flag:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.dev, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.dev)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def result(self):
        self.stop_flag = True
        self.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons)}


def workload_shape(name):
    from gpt_oss_b200 import synth

    return synth.SHAPES[name]


def device_weights(shape, dev, dtype_out="bf16"):
    """Seeded bf16 weights generated on the device (N(0,0.02); biases N(0,0.01))."""
    import torch

    g = torch.Generator(device=dev)
    g.manual_seed(shape.seed)
    H, IM, E = shape.hidden_dim, shape.intermediate_dim, shape.n_experts

    def normal(size, std, dtype=torch.bfloat16):
        return (torch.randn(size, generator=g, device=dev, dtype=torch.float32) * std).to(dtype)

    w = {
        "w_router": normal((E, H), 0.02),
        "b_router": normal((E,), 0.02).float(),
        "w_mlp1": torch.empty((E, 2 * IM, H), device=dev, dtype=torch.bfloat16),
        "b_mlp1": normal((E, 2 * IM), 0.01).float(),
        "w_mlp2": torch.empty((E, H, IM), device=dev, dtype=torch.bfloat16),
        "b_mlp2": normal((E, H), 0.01).float(),
    }
    for e in range(E):  # per expert, to bound the fp32 temporary
        w["w_mlp1"][e] = normal((2 * IM, H), 0.02)
        w["w_mlp2"][e] = normal((H, IM), 0.02)
    return w


def host_weights_f32(w):
    return {k: v.float().cpu().numpy() for k, v in w.items()}


def cpu_sample(shape, w_host, t_host, x_host, n_tokens, kind):
    """Times the CPU implementation on the first n_tokens of the batch."""
    oracle = entry.load_oracle()
    d = dict(w_host)
    d["t"], d["x"], d["pos"] = t_host[:n_tokens], x_host[:n_tokens], None
    t0 = time.perf_counter()
    oracle.moe_layer(d, shape, which=("ref" if kind == "reference" else "oracle"), taps=False)
    return time.perf_counter() - t0


def oracle_router_np(oracle, t, w_router, b_router, K):
    """Top-K expert ids of every row of t by the CPU oracle's router (cheap)."""
    import ctypes

    T, H = t.shape
    E = w_router.shape[0]
    lib = ctypes.CDLL(str(oracle.ORACLE_LIB))
    fp, ip = ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_int)
    lg = np.zeros((T, E), np.float32)
    ti = np.full((T, K), -1, np.int32)
    tv = np.zeros((T, K), np.float32)
    lib.oracle_router.argtypes = [fp, ip] + [ctypes.c_int] * 4 + [fp, fp, fp, ip, fp]
    t = np.ascontiguousarray(t, np.float32)
    w_router = np.ascontiguousarray(w_router, np.float32)
    b_router = np.ascontiguousarray(b_router, np.float32)
    rc = lib.oracle_router(t.ctypes.data_as(fp), None, T, H, E, K, w_router.ctypes.data_as(fp),
                           b_router.ctypes.data_as(fp), lg.ctypes.data_as(fp),
                           ti.ctypes.data_as(ip), tv.ctypes.data_as(fp))
    if rc != 0:
        raise RuntimeError("oracle_router failed")
    return ti


def run_reference_arm(args, shape):
    """The reference's CPU implementation on the host cores (rank 0 only).  The sample's
    tokens are routed first; only the experts they select get weights drawn (the CPU code
    never reads the others, which stay untouched zero pages)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    oracle = entry.load_oracle()
    if not oracle.ORACLE_LIB.exists():
        oracle.build(native=True)
    kind = "reference" if oracle.have_ref() else "port"
    cores = oracle.num_threads("ref" if kind == "reference" else "oracle")
    if cores < 2 and len(os.sched_getaffinity(0)) > 1:
        raise SystemExit("the CPU baseline would run on one thread although the box has more cores")
    g = torch.Generator().manual_seed(shape.seed)
    H, IM, E, K = shape.hidden_dim, shape.intermediate_dim, shape.n_experts, shape.experts_per_token

    def normal(size, std):
        return (torch.randn(size, generator=g) * std).bfloat16().float().numpy()

    n_sample = args.cpu_tokens
    w = {"w_router": normal((E, H), 0.02), "b_router": normal((E,), 0.02),
         "b_mlp1": normal((E, 2 * IM), 0.01), "b_mlp2": normal((E, H), 0.01)}
    t = normal((n_sample, H), 1.0)
    x = normal((n_sample, H), 1.0)
    used = np.unique(oracle_router_np(oracle, t, w["w_router"], w["b_router"], K))
    w["w_mlp1"] = np.zeros((E, 2 * IM, H), np.float32)
    w["w_mlp2"] = np.zeros((E, H, IM), np.float32)
    for e in used:
        w["w_mlp1"][e] = normal((2 * IM, H), 0.02)
        w["w_mlp2"][e] = normal((H, IM), 0.02)
    for _ in range(min(args.warmup, 1)):
        cpu_sample(shape, w, t, x, n_sample, kind)
    times = [cpu_sample(shape, w, t, x, n_sample, kind) for _ in range(args.steps)]
    total = sum(times)
    value = n_sample * args.steps / total
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": shape.name, "tokens_per_step": n_sample,
                   "note": "CPU path of the reference on a bounded sample per step"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": f"{n_sample} tokens x {shape.experts_per_token} experts per step"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def host_weights_for(w, used, shape):
    """fp32 host copies of the layer for the CPU code: router and biases whole, expert
    matrices only for the experts in `used` (the others stay untouched zero pages)."""
    H, IM, E = shape.hidden_dim, shape.intermediate_dim, shape.n_experts
    d = {k: w[k].float().cpu().numpy() for k in ("w_router", "b_router", "b_mlp1", "b_mlp2")}
    d["w_mlp1"] = np.zeros((E, 2 * IM, H), np.float32)
    d["w_mlp2"] = np.zeros((E, H, IM), np.float32)
    for e in used:
        d["w_mlp1"][e] = w["w_mlp1"][e].float().cpu().numpy()
        d["w_mlp2"][e] = w["w_mlp2"][e].float().cpu().numpy()
    return d


def cpu_baseline_for(args, shape, w, t, x0, routing_topk_i):
    """Times the CPU code on the first tokens of the batch (about 12 s of work)."""
    oracle = entry.load_oracle()
    if not oracle.ORACLE_LIB.exists():
        oracle.build(native=True)
    kind = "reference" if oracle.have_ref() else "port"
    T, K = shape.n_tokens, shape.experts_per_token

    def sample(n):
        w_host = host_weights_for(w, np.unique(routing_topk_i[:n]), shape)
        return cpu_sample(shape, w_host, t[:n].float().cpu().numpy(), x0[:n].float().cpu().numpy(),
                          n, kind)

    if args.cpu_tokens:
        n_cpu = min(T, args.cpu_tokens)
        sec = sample(n_cpu)
    else:
        n_cpu = min(T, 64)
        sec = sample(n_cpu)
        want = min(T, max(64, int(12.0 / (sec / n_cpu)) // 64 * 64))
        if want > 2 * n_cpu:
            n_cpu = want
            sec = sample(n_cpu)
    return {"value": n_cpu / sec, "unit": UNIT,
            "cores": oracle.num_threads("ref" if kind == "reference" else "oracle"), "kind": kind,
            "sample": f"first {n_cpu} tokens of the batch, {K} experts each, {sec:.1f} s"}


def timed_forward(eng, t, x, T, steps, stream, barrier, world, dev, names, warm=3, stage_events=True):
    """`steps` passes of the layer between CUDA events on the launching stream (barrier and
    synchronize on both sides, max over ranks).  With `stage_events` the library also records
    an event pair around every stage (they cost 1-3 % of the step: an event between two
    kernels undoes their programmatic dependent launch)."""
    import torch
    import torch.distributed as dist

    for _ in range(warm):
        eng.forward(0, t, x, None, T, stream)
    barrier()
    if eng.device_status() != 0:
        raise SystemExit("device status non-zero after warm-up")
    eng.set_option("time_stages", 1 if stage_events else 0)
    barrier()
    launches0 = eng.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        eng.forward(0, t, x, None, T, stream)
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    launches = eng.launch_count() - launches0
    if world > 1:
        tt = torch.tensor([ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt.item())
    stage_ms = {s: eng.stage_ms(s) for s in names} if stage_events else None
    eng.set_option("time_stages", 0)
    return {"ms": ms, "stage_ms": stage_ms, "launches": launches}


def measure_layer(args, pkg, shape, dev, rank, world, local_rank, barrier, with_e2e, with_cpu,
                  with_parity):
    """One MoE layer workload: all experts local at world 1, expert parallel (owner =
    e % world, every rank its own `shape.n_tokens` tokens: weak scaling) otherwise."""
    import torch
    import torch.distributed as dist

    T, H, IM, E, K = (shape.n_tokens, shape.hidden_dim, shape.intermediate_dim, shape.n_experts,
                      shape.experts_per_token)
    ep = world > 1
    eng = pkg.MoeEngine(H, IM, E, K, n_layers=1, max_tokens=T, swiglu_limit=shape.swiglu_limit,
                        ep_rank=rank if ep else 0, ep_size=world if ep else 1, device=local_rank)
    w = device_weights(shape, dev)  # same seed on every rank: one set of weights, sharded
    eng.load_layer_bf16(0, w["w_router"], w["b_router"], w["w_mlp1"], w["b_mlp1"], w["w_mlp2"],
                        w["b_mlp2"], on_device=True)
    if ep:
        uid = torch.zeros(128, dtype=torch.uint8, device=dev)
        if rank == 0:
            uid.copy_(torch.frombuffer(bytearray(pkg.MoeEngine.ep_unique_id()), dtype=torch.uint8))
        dist.broadcast(uid, 0)
        eng.ep_init(bytes(uid.cpu().numpy().tobytes()))
    g = torch.Generator(device=dev)
    g.manual_seed(shape.seed + 1000 + rank)
    t = torch.randn((T, H), generator=g, device=dev).bfloat16()
    x0 = torch.randn((T, H), generator=g, device=dev).bfloat16()
    x = x0.clone()
    stream = torch.cuda.current_stream().cuda_stream
    names = ["route", "permute", "gate_up", "down", "combine"] + (["dispatch", "return"] if ep else [])
    transport = eng.ep_transport if ep else -1

    # warm-up, then the timed region of the line
    for _ in range(args.warmup):
        eng.forward(0, t, x, None, T, stream)
    x.copy_(x0)
    sampler = ClockSampler(local_rank)
    sampler.start()
    # the line's value: K steps as a caller runs them; then the same K steps once more with
    # the library's event pairs around every stage, which the stage table and the rooflines
    # are taken from
    main = timed_forward(eng, t, x, T, args.steps, stream, barrier, world, dev, names, warm=0,
                         stage_events=False)
    staged = timed_forward(eng, t, x, T, args.steps, stream, barrier, world, dev, names, warm=0)
    clocks = sampler.result()
    out = {"ms_per_step": main["ms"] / args.steps, "stage_ms": staged["stage_ms"],
           "ms_per_step_with_stage_events": staged["ms"] / args.steps,
           "launches": main["launches"], "clocks": clocks, "transport": transport,
           "value": world * T * args.steps / (main["ms"] * 1e-3)}
    routing = eng.get_routing(T)

    if ep:
        side_steps = max(3, min(args.steps, 20))
        strong = timed_forward(eng, t, x, T // world, side_steps, stream, barrier, world, dev, names)
        out["strong_scaling"] = {"tokens_per_gpu": T // world,
                                 "value": world * (T // world) * side_steps / (strong["ms"] * 1e-3),
                                 "unit": UNIT, "ms_per_step": strong["ms"] / side_steps,
                                 "stage_ms": strong["stage_ms"]}
        if transport == 1:
            eng.set_option("ep_transport", 0)
            other = timed_forward(eng, t, x, T, side_steps, stream, barrier, world, dev, names)
            eng.set_option("ep_transport", 1)
            out["nccl_send_recv"] = {"value": world * T * side_steps / (other["ms"] * 1e-3),
                                     "unit": UNIT, "ms_per_step": other["ms"] / side_steps,
                                     "stage_ms": other["stage_ms"]}

    if with_parity:
        out["parity"] = parity_check(pkg, eng, shape, w, t, x0, rank, world, dev, stream, barrier,
                                     transport)

    if with_e2e:
        out["e2e"] = measure_e2e(args, eng, shape, t, x0, world, dev, barrier, ep)

    if with_cpu and rank == 0:
        out["cpu_baseline"] = cpu_baseline_for(args, shape, w, t, x0, routing["topk_i"])
    eng.close()
    del w
    torch.cuda.empty_cache()
    return out


def parity_check(pkg, eng, shape, w, t, x0, rank, world, dev, stream, barrier, transport):
    """Untimed.  One pass on this rank's tokens with a zero residual; 32 seeded tokens of it
    against the CPU code (all experts), expert ids exactly, block output within the stated
    tolerance; under expert parallelism also the two transports against each other.  The
    worst figures over the ranks are returned."""
    import torch
    import torch.distributed as dist

    T, K = shape.n_tokens, shape.experts_per_token
    oracle = entry.load_oracle()
    if not oracle.ORACLE_LIB.exists():
        oracle.build(native=True)
    kind = "ref" if oracle.have_ref() else "oracle"

    def one_pass():
        x = torch.zeros_like(x0)
        eng.forward(0, t, x, None, T, stream)
        barrier()
        if eng.device_status() != 0:
            raise SystemExit("device status non-zero in the parity pass")
        return x

    x_a = one_pass()
    routing = eng.get_routing(T)
    across = None  # largest difference between the two transports' results
    if transport == 1:
        eng.set_option("ep_transport", 0)
        x_b = one_pass()
        eng.set_option("ep_transport", 1)
        across = float((x_a.float() - x_b.float()).abs().max().item())
    rng = np.random.default_rng(shape.seed + rank)
    idx = np.sort(rng.choice(T, 32, replace=False))
    d = host_weights_for(w, np.unique(routing["topk_i"][idx]), shape)
    d["t"] = t[idx].float().cpu().numpy()
    d["x"] = np.zeros_like(d["t"])
    d["pos"] = None
    sub = type(shape)(shape.name, 32, shape.hidden_dim, shape.intermediate_dim, shape.n_experts, K,
                      shape.swiglu_limit, shape.seed)
    want = oracle.moe_layer(d, sub, which=kind)
    got = x_a[idx].float().cpu().numpy()
    err = np.abs(got - want["e_agg"])
    res = [float(err.max()), float(err.mean() / np.abs(want["e_agg"]).mean()),
           float(not np.array_equal(routing["topk_i"][idx], want["topk_i"])),
           across or 0.0]
    if world > 1:
        tt = torch.tensor(res, device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        res = [float(v) for v in tt.tolist()]
    return {"checker": "oracle/_ref (the reference's CPU code)" if kind == "ref" else "oracle port",
            "tokens_per_rank": 32, "max_abs": res[0], "mean_rel": res[1],
            "indices_exact": res[2] == 0.0,
            # the NCCL transport rounds the owner's per-row sum to bf16 once more
            "max_abs_between_transports": None if across is None else res[3],
            "within_tolerance": res[0] <= 2e-2 and res[1] <= 1e-2 and res[2] == 0.0}


def measure_e2e(args, eng, shape, t, x0, world, dev, barrier, ep):
    """The same layer through the host-buffer entry points: every step copies its inputs in
    from pinned host memory and its result back out.  The streamed pair submit / wait
    keeps three batches in flight, each in its own pinned buffers, so the copies of
    neighbouring steps overlap the kernels; with the RMSNorm of the block on the device
    only the residual stream crosses the bus."""
    import torch
    import torch.distributed as dist

    T, H = shape.n_tokens, shape.hidden_dim
    t_h = t.cpu().pin_memory()
    x_h = x0.cpu().pin_memory()
    e2e_steps = max(3, min(args.steps, 20))

    def timed_host(fn):
        fn(3)
        barrier()
        t0 = time.perf_counter()
        fn(e2e_steps)
        barrier()
        sec = time.perf_counter() - t0
        if world > 1:
            tt = torch.tensor([sec], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            sec = float(tt.item())
        return world * T * e2e_steps / sec

    def sync_steps(n):
        for _ in range(n):
            eng.forward_host(0, t_h, x_h, None, T)

    bufs = [(t_h, x_h)] + [(t_h.clone().pin_memory(), x_h.clone().pin_memory()) for _ in range(2)]

    def streamed(with_t):
        def steps(n):
            tickets = []
            for i in range(n):
                if i >= 3:
                    eng.forward_host_wait(tickets[i - 3])  # its buffers are free again
                tb, xb = bufs[i % 3]
                tickets.append(eng.forward_host_submit(0, tb if with_t else None, xb, None, T))
            for tk in tickets[-3:]:
                eng.forward_host_wait(tk)
        return steps

    one_call = timed_host(sync_steps)
    res = {"unit": UNIT, "steps": e2e_steps,
           "one_call_per_step": {"value": one_call, "h2d_bytes_per_step": 2 * T * H * 2,
                                 "d2h_bytes_per_step": T * H * 2}}
    if ep and eng.ep_transport != 1:
        # the NCCL transport synchronises with the host in every layer: no streamed variant
        res.update(value=one_call, h2d_bytes_per_step=2 * T * H * 2, d2h_bytes_per_step=T * H * 2,
                   how="gptoss_moe_forward_host: t and x in, block on the device, x out, per step")
        return res
    with_t = timed_host(streamed(True))
    eng.load_ffn_norm(0, np.ones(H, dtype=np.float32))
    value = timed_host(streamed(False))
    res.update(value=value, h2d_bytes_per_step=T * H * 2, d2h_bytes_per_step=T * H * 2,
               how="gptoss_moe_forward_host_submit / _wait, three batches in flight; x in, "
                   "RMSNorm + block on the device, x out",
               streamed_with_t_from_host={"value": with_t, "h2d_bytes_per_step": 2 * T * H * 2})
    return res


def layer_rooflines(shape, stage_ms, peaks, timed_s, rows_per_rank_scale=1.0, local_experts=None):
    """Roofline entries of the dominant kernel (gate_up GEMM) of a layer measurement:
    against the tensor peak (algorithmic flops 2*A*2IM*H) and against the HBM copy
    bandwidth (weights once, gathered rows in, activations out)."""
    T, H, IM, E, K = (shape.n_tokens, shape.hidden_dim, shape.intermediate_dim, shape.n_experts,
                      shape.experts_per_token)
    El = E if local_experts is None else local_experts
    n_assign = T * K * rows_per_rank_scale
    flops = 2.0 * n_assign * 2 * IM * H
    peak_kind = "bf16_tflops" if timed_s < 1.0 else "bf16_tflops_sustained"
    sec = stage_ms["gate_up"] * 1e-3
    tflops = flops / sec / 1e12
    alg_bytes = El * 2 * IM * H * 2 + n_assign * H * 2 + n_assign * IM * 2
    gbs = alg_bytes / sec / 1e9
    tensor = {"kernel": "grouped_gemm_pair_kernel<swiglu> (gate_up, CTA pairs)", "bound": "tensor",
              "achieved": tflops, "peak": peaks[peak_kind], "unit": "TFLOP/s",
              "frac": tflops / peaks[peak_kind], "peak_source": f"{peaks['source']} {peak_kind}",
              "algorithmic_flops_per_launch": flops, "kernel_ms": stage_ms["gate_up"]}
    hbm = {"kernel": tensor["kernel"], "bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"],
           "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
           "peak_source": f"{peaks['source']} hbm_gbs",
           "algorithmic_bytes_per_launch": alg_bytes, "kernel_ms": stage_ms["gate_up"]}
    return tensor, hbm, alg_bytes


def binding_roofline(tensor, hbm):
    """The ceiling that bounds the launch: the one whose floor (algorithmic work / peak) is the
    longer time.  Returns (binding, other)."""
    floor_t = tensor["algorithmic_flops_per_launch"] / (tensor["peak"] * 1e12)
    floor_h = hbm["algorithmic_bytes_per_launch"] / (hbm["peak"] * 1e9)
    tensor["floor_ms"], hbm["floor_ms"] = floor_t * 1e3, floor_h * 1e3
    return (hbm, tensor) if floor_h > floor_t else (tensor, hbm)


def run_ours(args, shape):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # several ranks share the host: each keeps to the CPUs (and so the memory) near its GPU
    near_cpus = run_near_gpu(local_rank) if world > 1 else None
    pkg = entry.load_package()
    T, H, IM, E, K = (shape.n_tokens, shape.hidden_dim, shape.intermediate_dim, shape.n_experts,
                      shape.experts_per_token)
    if world > 1 and E % world:
        raise SystemExit(f"{E} experts do not split over {world} GPUs")
    res = measure_layer(args, pkg, shape, dev, rank, world, local_rank, barrier, with_e2e=True,
                        with_cpu=(world == 1 and not args.no_cpu_baseline), with_parity=not args.no_extra)

    extras = {}
    if not args.no_extra and world == 1 and args.workload == "c3":
        # the 20b-shape layer (configuration 2) and the MXFP4 decode shapes (configuration 4)
        # ride in the same line
        import copy

        side = copy.copy(args)
        side.steps = max(3, min(args.steps, 30))
        side.warmup = 3
        c2 = measure_layer(side, pkg, workload_shape("c2"), dev, 0, 1, local_rank, barrier,
                           with_e2e=False, with_cpu=False, with_parity=False)
        extras["layer_20b"] = c2
        side.steps = max(3, min(args.steps, 30))
        extras["decode_mxfp4"] = measure_decode_mxfp4(side, pkg, dev)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = read_peaks()
    timed_s = res["ms_per_step"] * args.steps * 1e-3
    tensor, hbm, alg_bytes = layer_rooflines(shape, res["stage_ms"], peaks, timed_s,
                                             local_experts=E // world)
    # DRAM traffic of one gate_up launch, from the ncu capture named in profiles/: the ratio
    # of measured to algorithmic bytes of the captured small case applied to this launch
    ratio = TRAFFIC_RATIO.get(shape.name if world == 1 else None)
    tensor["traffic"] = hbm["traffic"] = ratio * alg_bytes if ratio else None
    tensor["traffic_unit"] = hbm["traffic_unit"] = "bytes/launch"
    tensor["traffic_source"] = hbm["traffic_source"] = TRAFFIC_SOURCE if ratio else None
    stage = res["stage_ms"]
    n_assign = T * K
    main_roof, other_roof = binding_roofline(tensor, hbm)
    tensor = main_roof  # the per-stage figures below ride on the binding entry
    tensor["stage_ms"] = stage
    tensor["down_tflops"] = 2.0 * n_assign * H * IM / (stage["down"] * 1e-3) / 1e12
    tensor["route_gbs"] = (T * H * 2 + E * H * 2 + T * K * 8) / (stage["route"] * 1e-3) / 1e9
    tensor["route_frac_of_hbm"] = tensor["route_gbs"] / peaks["hbm_gbs"]
    tensor["combine_gbs"] = ((n_assign * H * 2 + 2 * T * H * 2) / (stage["combine"] * 1e-3) / 1e9
                             if world == 1 else None)
    tensor["hbm_peak_gbs"] = peaks["hbm_gbs"]
    # the whole layer against both ceilings
    layer_flops = 2.0 * n_assign * 3 * IM * H
    layer_bytes = (E // world) * 3 * IM * H * 2 + T * H * 2 + 2 * n_assign * IM * 2 + 2 * T * H * 2
    tensor["layer_tflops"] = layer_flops / (res["ms_per_step"] * 1e-3) / 1e12
    tensor["layer_frac_of_tensor_peak"] = tensor["layer_tflops"] / peaks["bf16_tflops"]
    tensor["layer_frac_of_hbm_streaming"] = (layer_bytes / peaks["hbm_gbs"] / 1e9) / (res["ms_per_step"] * 1e-3)

    how = {-1: "all experts local", 0: f"expert parallel x{world} (NCCL send/recv)",
           1: f"expert parallel x{world} (rows read from peer memory over NVLink)"}[res["transport"]]
    line = {
        "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": shape.name, "tokens_per_gpu": T, "hidden": H, "intermediate": IM,
                   "experts": E, "experts_per_gpu": E // world, "top_k": K, "parallelism": how,
                   "l2": "inputs larger than L2 (expert weights %.2f GB per GPU streamed every step)"
                         % (((E // world) * 3 * IM * H * 2) / 1e9)},
        "roofline": main_roof, "roofline_" + other_roof["bound"]: other_roof,
        "cpu_baseline": res.get("cpu_baseline"),
        "e2e": res["e2e"], "gpu_launches": res["launches"], "clocks": res["clocks"],
        "stage_ms": stage, "ms_per_step_with_stage_events": res["ms_per_step_with_stage_events"],
        "host_cpus_near_gpu": near_cpus,
        "stage_timing": "the K steps run a second time with an event pair around every stage "
                        "(an event between two kernels undoes their dependent launch)",
    }
    if world > 1 and res["transport"] == 1:
        # the exchange against the link: under uniform routing (N-1)/N of the T*K rows an owner
        # multiplies are pulled from peers inside the permute stage (the stage also holds the
        # sort and the local rows, so the rate is a lower bound), and (N-1)/N of the T*K
        # expert outputs are stored into peers' memory by the down GEMM's epilogue, under its
        # tiles: the rate the link has to carry for that to stay hidden
        remote = (world - 1) / world * n_assign * H * 2
        # a token with several experts on one owner is pulled once: under uniform routing each
        # of the other ranks' tokens needs this owner with probability 1 - (1 - 1/N)^K
        pulled = (world - 1) * T * (1.0 - (1.0 - 1.0 / world) ** K) * H * 2
        line["nvlink"] = {
            "bytes_pulled_per_rank_per_step": pulled, "bytes_pushed_per_rank_per_step": remote,
            "gather_gbs_lower_bound": pulled / (stage["permute"] * 1e-3) / 1e9,
            "push_gbs_under_down_gemm": remote / (stage["down"] * 1e-3) / 1e9,
            "peak": 770.0, "unit": "GB/s per direction per GPU",
            "peak_source": "measured peer copy on this pool (900 nominal)",
            "gather_floor_ms": pulled / 770e9 * 1e3,
            "ms_outside_the_gemms": stage["route"] + stage["permute"] + stage["combine"]
                                    + stage.get("dispatch", 0.0) + stage.get("return", 0.0),
        }
    for key in ("strong_scaling", "nccl_send_recv", "parity"):
        if key in res:
            line["ep_parity" if (key == "parity" and world > 1) else key] = res[key]
    for name, ex in extras.items():
        if name == "layer_20b":
            s20 = workload_shape("c2")
            t20, h20, _ = layer_rooflines(s20, ex["stage_ms"], peaks, ex["ms_per_step"] * 30e-3)
            m20, o20 = binding_roofline(t20, h20)
            line[name] = {"workload": s20.name, "value": ex["value"], "unit": UNIT,
                          "ms_per_step": ex["ms_per_step"], "stage_ms": ex["stage_ms"],
                          "roofline": m20, "roofline_" + o20["bound"]: o20,
                          "route_gbs": (s20.n_tokens * H * 2 + s20.n_experts * H * 2 + s20.n_tokens * K * 8)
                                       / (ex["stage_ms"]["route"] * 1e-3) / 1e9}
        else:
            line[name] = ex
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ratio of measured DRAM traffic (ncu dram__bytes_read.sum + dram__bytes_write.sum) to the
# algorithmic bytes of the gate_up launch, per workload the capture covers
TRAFFIC_RATIO = {"gpt-oss-120b-moe-layer-T6144": 559.6 / 566.2,
                 "gpt-oss-120b-moe-layer-16experts-T768": 559.6 / 566.2,
                 "gpt-oss-20b-moe-layer-T7168": 401.6 / 348.0,
                 "gpt-oss-20b-moe-layer-8experts-T1792": 401.6 / 348.0}
TRAFFIC_SOURCE = ("ncu dram__bytes_read+write of the small-case capture under profiles/ scaled to "
                  "this launch by its algorithmic bytes")


def c4_tokens(T, H, g, dev):
    """Decode-batch activations of configuration 4: t with sigma 0.25 (the weights' rms is
    0.094, so pre-activations stay around the clamp), a N(0,1) residual."""
    import torch

    t = (torch.randn((T, H), generator=g, device=dev) * 0.25).bfloat16()
    x = torch.randn((T, H), generator=g, device=dev).bfloat16()
    return t, x


def c4_layer(pkg, dev, max_tokens=1024, n_experts=None):
    """Configuration 4: the 120b-shape layer with MXFP4 expert weights - e2m1 codes uniform
    over the 16 values, e8m0 scales uniform in 2^-8 .. 2^-4 - and a router whose bias
    makes expert popularity follow Zipf(1.1) over a seeded permutation of the experts.
    Returns the loaded engine and the tensors it was loaded from."""
    import torch

    shape = workload_shape("c3")
    H, IM, K = shape.hidden_dim, shape.intermediate_dim, shape.experts_per_token
    E = n_experts or shape.n_experts
    g = torch.Generator(device=dev)
    g.manual_seed(4)
    eng = pkg.MoeEngine(H, IM, E, K, max_tokens=max_tokens, weight_format=pkg.WEIGHTS_MXFP4,
                        device=dev.index or 0)

    def codes(rows, k):
        return torch.randint(0, 256, (E, rows, k // 2), generator=g, device=dev, dtype=torch.uint8)

    def scales(rows, k):
        return torch.randint(119, 124, (E, rows, k // 32), generator=g, device=dev,
                             dtype=torch.uint8)

    ranks = torch.randperm(E, generator=g, device=dev).float() + 1.0
    zipf = ranks.pow(-1.1)
    # logits = bias + noise with sigma ~1.07 (t has sigma 0.25, router weights 0.08); a
    # Gaussian of that width selects about like Gumbel noise of scale 0.83, for which
    # P(expert) is proportional to exp(bias / 0.83): bias = 0.83 * log(Zipf weight)
    w = {"b_router": ((zipf / zipf.sum()).log().float() * 0.83).contiguous(),
         "w_router": (torch.randn((E, H), generator=g, device=dev) * 0.08).bfloat16(),
         "b_mlp1": (torch.randn((E, 2 * IM), generator=g, device=dev) * 0.01).float(),
         "b_mlp2": (torch.randn((E, H), generator=g, device=dev) * 0.01).float(),
         "w1_codes": codes(2 * IM, H), "w1_scales": scales(2 * IM, H),
         "w2_codes": codes(H, IM), "w2_scales": scales(H, IM)}
    eng.load_layer_mxfp4(0, w["w_router"], w["b_router"], w["w1_codes"], w["w1_scales"], w["b_mlp1"],
                         w["w2_codes"], w["w2_scales"], w["b_mlp2"], on_device=True)
    return {"engine": eng, "weights": w, "H": H, "IM": IM, "E": E, "K": K}


def measure_decode_mxfp4(args, pkg, dev):
    """Configuration 4 at T = 64 / 256 / 1024: tokens/s, stage times and the rate at which
    the packed weights of the touched experts stream from HBM (the kernel's roofline)."""
    import torch

    case = c4_layer(pkg, dev)
    eng, H, IM, E = case["engine"], case["H"], case["IM"], case["E"]
    torch.cuda.empty_cache()
    peaks = read_peaks()
    stream = torch.cuda.current_stream().cuda_stream
    per_expert_bytes = 3 * IM * H // 2 + 3 * IM * H // 32
    g = torch.Generator(device=dev)
    g.manual_seed(44)
    results = {}
    for T in (64, 256, 1024):
        t, x = c4_tokens(T, H, g, dev)
        for _ in range(max(3, args.warmup)):
            eng.forward(0, t, x, None, T, stream)
        torch.cuda.synchronize()
        if eng.device_status() != 0:
            raise SystemExit("device status non-zero")
        # the step time without events between the stages (they keep a kernel's set-up from
        # overlapping its predecessor's tail), the stage times from a second pass with them
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(args.steps):
            eng.forward(0, t, x, None, T, stream)
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1) / args.steps
        eng.set_option("time_stages", 1)
        ev2, ev3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev2.record()
        for _ in range(args.steps):
            eng.forward(0, t, x, None, T, stream)
        ev3.record()
        torch.cuda.synchronize()
        ms_staged = ev2.elapsed_time(ev3) / args.steps
        stage_ms = {s: eng.stage_ms(s) for s in ("route", "permute", "gate_up", "down", "combine")}
        eng.set_option("time_stages", 0)
        r = eng.get_routing(T)
        counts = np.bincount(r["topk_i"].ravel(), minlength=E)
        touched = int((counts > 0).sum())
        gemm_ms = stage_ms["gate_up"] + stage_ms["down"]
        gbs = touched * per_expert_bytes / (gemm_ms * 1e-3) / 1e9
        results[str(T)] = {
            "tokens_per_s": T / (ms * 1e-3), "ms_per_step": ms,
            "ms_per_step_with_stage_events": ms_staged, "stage_ms": stage_ms,
            "experts_touched": touched, "busiest_expert_share": float(counts.max() / counts.sum()),
            "roofline": {"kernel": "grouped_gemm_pair_kernel<*, mxfp4> (gate_up + down)",
                         "bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} hbm_gbs",
                         "algorithmic_bytes_per_step": touched * per_expert_bytes},
        }
    out = {"workload": "gpt-oss-120b-moe-layer-mxfp4-decode", "weights": "MXFP4 (e2m1 + e8m0/32)",
           "routing": "Zipf(1.1)-biased router", "launches": eng.launch_count(), "decode": results}
    eng.close()
    torch.cuda.empty_cache()
    return out


def run_decode_mxfp4(args):
    """--workload c4: configuration 4 as its own line (the T = 1024 figures on top)."""
    import torch

    pkg = entry.load_package()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    sampler = ClockSampler(0)
    sampler.start()
    res = measure_decode_mxfp4(args, pkg, dev)
    clocks = sampler.result()
    top = res["decode"]["1024"]
    shape = workload_shape("c3")
    line = {
        "metric": METRIC, "value": top["tokens_per_s"], "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": top["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "gpt-oss-120b-moe-layer-mxfp4-decode-T1024", "hidden": shape.hidden_dim,
                   "intermediate": shape.intermediate_dim, "experts": shape.n_experts,
                   "top_k": shape.experts_per_token, "weights": res["weights"],
                   "routing": res["routing"], "l2": "inputs larger than L2 (1.69 GB of "
                   "packed expert weights streamed every step)"},
        "roofline": dict(top["roofline"], traffic=None), "decode": res["decode"],
        "cpu_baseline": None, "e2e": None, "gpu_launches": res["launches"], "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def run_decode_120b(args):
    """--workload c5: one decode step of a 120b-architecture model (36 layers, hidden 2880,
    64 query / 8 KV heads of 64, sinks, 128-token window on even layers, 128 experts top-4,
    vocabulary 201088), random-init weights generated on the device, 6144 sequences split
    over the GPUs, each with 512 positions of synthetic KV context; experts sharded over
    the ranks (16 per GPU at 8).  Needs at least 2 GPUs: the bf16 experts alone are 229 GB.
    GPTOSS_C5_LAYERS / GPTOSS_C5_SEQS cut the layer / sequence count for development runs
    (reported in the line)."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun")
    layers = int(os.environ.get("GPTOSS_C5_LAYERS", "36"))
    if world < 2 and layers > 24:
        raise SystemExit("workload c5 needs at least 2 GPUs (229 GB of bf16 expert weights)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pkg = entry.load_package()
    ctx, total_seqs = 512, int(os.environ.get("GPTOSS_C5_SEQS", "6144"))
    B = total_seqs // world
    steps, warmup = args.steps, args.warmup
    cfg = dict(vocab_size=201088, hidden_dim=2880, n_experts=128, experts_per_token=4,
               intermediate_dim=2880, n_layers=layers, head_dim=64, n_attn_heads=64, n_kv_heads=8,
               seq_len=ctx + warmup + steps + 8, initial_context_length=4096, rope_theta=150000.0,
               rope_scaling_factor=32.0, sliding_window=128, swiglu_limit=7.0)
    V, H, IM, E, D = cfg["vocab_size"], cfg["hidden_dim"], cfg["intermediate_dim"], cfg["n_experts"], 64
    dq, dkv = cfg["n_attn_heads"] * D, cfg["n_kv_heads"] * D
    eng = pkg.DecodeEngine(cfg, B, device=local_rank, ep_rank=rank, ep_size=world)
    moe = eng.moe(ep_rank=rank, ep_size=world, device=local_rank)

    def normal(gen, size, std, dtype=torch.bfloat16):
        return (torch.randn(size, generator=gen, device=dev, dtype=torch.float32) * std).to(dtype)

    g = torch.Generator(device=dev)
    g.manual_seed(3)  # the same weights on every rank
    for name in ("token_embedding_table", "out"):
        eng.set_tensor(name, 0, normal(g, (V, H), 0.02))
    eng.set_tensor("rms_out_w", 0, torch.ones(H, device=dev))
    layer_shape = synth_shape_120b()
    for l in range(layers):
        eng.set_tensor("w_qkv", l, normal(g, (dq + 2 * dkv, H), 0.02))
        eng.set_tensor("b_qkv", l, normal(g, (dq + 2 * dkv,), 0.01, torch.float32))
        eng.set_tensor("w_o", l, normal(g, (H, dq), 0.02))
        eng.set_tensor("b_o", l, normal(g, (H,), 0.01, torch.float32))
        eng.set_tensor("attn_sinks", l, normal(g, (cfg["n_attn_heads"],), 0.02, torch.float32))
        eng.set_tensor("rms_attn_w", l, torch.ones(H, device=dev))
        eng.set_tensor("rms_ffn_w", l, torch.ones(H, device=dev))
        layer_shape.seed = 3000 + l
        w = device_weights(layer_shape, dev)  # all 128 experts; the engine keeps this rank's
        moe.load_layer_bf16(l, w["w_router"], w["b_router"], w["w_mlp1"], w["b_mlp1"], w["w_mlp2"],
                            w["b_mlp2"], on_device=True)
        del w
    torch.cuda.empty_cache()
    if world > 1:
        uid = torch.zeros(128, dtype=torch.uint8, device=dev)
        if rank == 0:
            uid.copy_(torch.frombuffer(bytearray(pkg.MoeEngine.ep_unique_id()), dtype=torch.uint8))
        dist.broadcast(uid, 0)
        moe.ep_init(bytes(uid.cpu().numpy().tobytes()))
    # synthetic context: 512 cached positions per sequence and layer
    gk = torch.Generator(device=dev)
    gk.manual_seed(7000 + rank)
    rows = 128
    for l in range(layers):
        for r0 in range(0, B, rows):
            n = min(rows, B - r0)
            k = torch.randn((n, ctx, dkv), generator=gk, device=dev, dtype=torch.bfloat16)
            v = torch.randn((n, ctx, dkv), generator=gk, device=dev, dtype=torch.bfloat16)
            eng.set_kv(l, r0, 0, k, v)
    rng = np.random.default_rng(11 + rank)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def run(n, first_pos):
        for i in range(n):
            tokens = rng.integers(0, V, size=B, dtype=np.int32)
            eng.step(tokens, np.full(B, first_pos + i, np.int32))

    run(warmup, ctx)
    barrier()
    moe.set_option("time_stages", 1)
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    t0 = time.perf_counter()
    run(steps, ctx + warmup)
    ev1.record()
    barrier()
    wall = time.perf_counter() - t0
    clocks = sampler.result()
    ms = ev0.elapsed_time(ev1)
    if world > 1:
        tt = torch.tensor([ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt.item())
    names = ["route", "permute", "gate_up", "down", "combine"] + (["dispatch", "return"] if world > 1 else [])
    stage_ms = {s: moe.stage_ms(s) for s in names}
    moe_ms_per_step = sum(stage_ms.values()) * layers
    launches = moe.launch_count()
    transport = moe.ep_transport if world > 1 else -1
    eng.close()
    if rank == 0:
        peaks = read_peaks()
        step_ms = ms / steps
        gate_up_flops = 2.0 * B * 4 * 2 * IM * H  # this rank's share of the assignments, on average
        line = {
            "metric": "decode_tokens_per_s", "value": world * B * steps / (ms * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": step_ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": f"gpt-oss-120b-decode-step-{layers}L-B{total_seqs}-ctx{ctx}",
                       "sequences_per_gpu": B, "layers": layers, "kv_context": ctx,
                       "parallelism": f"data parallel x{world} outside the experts, expert parallel x{world} "
                                      + ("(peer memory)" if transport == 1 else "(NCCL send/recv)"),
                       "l2": "weights and KV cache far larger than L2"},
            "moe_share": moe_ms_per_step / step_ms, "moe_ms_per_step": moe_ms_per_step,
            "moe_stage_ms_per_layer": stage_ms,
            "roofline": {"kernel": "grouped_gemm_pair_kernel<swiglu, 6> (gate_up, per layer)",
                         "bound": "tensor", "achieved": gate_up_flops / (stage_ms["gate_up"] * 1e-3) / 1e12,
                         "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                         "frac": gate_up_flops / (stage_ms["gate_up"] * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"],
                         "peak_source": f"{peaks['source']} bf16_tflops_sustained", "traffic": None},
            "cpu_baseline": None,
            # every step already goes through the public call with host token / position
            # arrays in and host next-token ids out
            "e2e": {"value": world * B * steps / wall, "unit": UNIT,
                    "h2d_bytes_per_step": 8 * B, "d2h_bytes_per_step": 4 * B},
            "gpu_launches": launches, "clocks": clocks,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def synth_shape_120b():
    entry.load_package()
    from gpt_oss_b200 import synth

    return synth.MoeShape("gpt-oss-120b-layer", 0, 2880, 2880, 128, 4, 7.0, 0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3",
                    choices=["c3", "c2", "c2s", "c3s", "c3r", "c4", "c5", "tiny"])
    ap.add_argument("--cpu-tokens", type=int, default=None,
                    help="tokens in the CPU sample (default 256 for ours, 64 for reference)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the parity pass and the workloads measured beside the headline one")
    args = ap.parse_args()
    entry.load_package()
    if args.workload == "c4" and args.impl == "ours":
        args.steps = args.steps if args.steps is not None else 50
        args.warmup = max(3, args.warmup if args.warmup is not None else 5)
        run_decode_mxfp4(args)
        return
    if args.workload == "c5" and args.impl == "ours":
        args.steps = args.steps if args.steps is not None else 8
        args.warmup = max(3, args.warmup if args.warmup is not None else 3)
        run_decode_120b(args)
        return
    shape = workload_shape("c3" if args.workload in ("c4", "c5") else args.workload)
    if args.impl == "reference":
        args.steps = args.steps if args.steps is not None else 5
        args.warmup = args.warmup if args.warmup is not None else 1
        args.cpu_tokens = args.cpu_tokens or 64
        run_reference_arm(args, shape)
    else:
        args.steps = args.steps if args.steps is not None else 100
        args.warmup = max(3, args.warmup if args.warmup is not None else 10)
        if args.workload in ("c2s", "c3s", "c3r", "tiny"):
            args.no_extra = True
        run_ours(args, shape)


if __name__ == "__main__":
    main()
