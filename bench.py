"""Benchmark of the MoE block: tokens/s of one layer pass.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c2|c3|c2s|c4|c5|tiny] [--no-extra] [--no-cpu-baseline]

A step is one pass of the block (router -> top-4 -> permutation -> grouped
gate_up + SwiGLU -> grouped down -> combine + residual) over one batch of
seeded synthetic tokens.  One JSON line is printed by rank 0.

N=1 runs the gpt-oss-20b-shape layer at T=7168 ("c2"), the configuration the
single-GPU metric is quoted on.  N>1 runs one such replica per GPU (the
reference serves the 20b shape as data-parallel replicas, getp_run.cpp:1035-1060),
so per-GPU work is fixed ("weak") and no data-path collective is involved.
The same line carries "layer_120b": the 120b-shape layer (T=6144 per GPU, 128
experts) measured in the same run, with the experts sharded over the ranks when
N>1 (rows read from peer memory over NVLink, or NCCL send/recv; both timed), a
strong-scaling reading (the 6144 tokens split over the ranks) beside the weak one.

Other workloads (each prints its own line):
  c3    the 120b-shape layer as the headline workload
  c2s   a quarter-size 20b-shape layer (8 experts, T=1792) for profiler captures
  c4    the 120b-shape layer with MXFP4 expert weights at decode batch sizes
        T = 64 / 256 / 1024 under a Zipf-skewed router
  c5    one decode step of the full 120b-architecture model (36 layers, 6144
        sequences with 512 positions of KV context), experts sharded over N >= 2 GPUs,
        with the MoE share of the step time
  tiny  a 16-token layer (smoke runs)

--impl reference times the reference's own CPU code (oracle/_ref when it was
built from the reference tree, else the C port in oracle/) on the host cores, on
a bounded sample of the same workload per step.
"""
from __future__ import annotations

import argparse
import json
import os
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
# workloads whose gate_up DRAM traffic is covered by the ncu capture of the small 20b-shape case
C2S_RATIO_WORKLOADS = ("gpt-oss-20b-moe-layer-T7168", "gpt-oss-20b-moe-layer-8experts-T1792")


def read_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs
    (read-only queries)."""

    def __init__(self, index, period=0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.stop_flag = [], set(), False
        self.max_mhz = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.dev = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.dev, pynvml.NVML_CLOCK_SM)
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


def run_reference_arm(args, shape):
    """The reference's CPU implementation on the host cores (rank 0 only)."""
    import torch

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # all the host cores this process may use (torchrun pins OMP_NUM_THREADS to 1)
    os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    oracle = entry.load_oracle()
    if not oracle.ORACLE_LIB.exists():
        oracle.build(native=True)
    kind = "reference" if oracle.have_ref() else "port"
    cores = oracle.num_threads("ref" if kind == "reference" else "oracle")
    g = torch.Generator().manual_seed(shape.seed)
    # weights drawn on the CPU here (same distributions); the sample is what matters
    H, IM, E = shape.hidden_dim, shape.intermediate_dim, shape.n_experts

    def normal(size, std):
        return (torch.randn(size, generator=g) * std).bfloat16().float().numpy()

    w = {"w_router": normal((E, H), 0.02), "b_router": normal((E,), 0.02),
         "w_mlp1": normal((E, 2 * IM, H), 0.02), "b_mlp1": normal((E, 2 * IM), 0.01),
         "w_mlp2": normal((E, H, IM), 0.02), "b_mlp2": normal((E, H), 0.01)}
    n_sample = args.cpu_tokens
    t = normal((n_sample, H), 1.0)
    x = normal((n_sample, H), 1.0)
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


def measure_c3_layer(args, pkg, dev, rank, world, local_rank, barrier):
    """The 120b-shape layer (T=6144 tokens per GPU, 128 experts) beside the headline
    workload: all experts local at N=1, expert parallel (owner = e % N) at N>1.  Weak
    scaling: every rank brings its own 6144 tokens."""
    import torch
    import torch.distributed as dist

    shape = workload_shape("c3")
    T, H, IM, E, K = (shape.n_tokens, shape.hidden_dim, shape.intermediate_dim, shape.n_experts,
                      shape.experts_per_token)
    eng = pkg.MoeEngine(H, IM, E, K, n_layers=1, max_tokens=T, swiglu_limit=shape.swiglu_limit,
                        ep_rank=rank, ep_size=world, device=local_rank)
    w = device_weights(shape, dev)  # same seed on every rank: one set of weights, sharded
    eng.load_layer_bf16(0, w["w_router"], w["b_router"], w["w_mlp1"], w["b_mlp1"], w["w_mlp2"],
                        w["b_mlp2"], on_device=True)
    del w
    torch.cuda.empty_cache()
    if os.environ.get("GPTOSS_GEMM_IMPL"):
        eng.set_option("gemm_impl", int(os.environ["GPTOSS_GEMM_IMPL"]))
    if world > 1:
        uid = torch.zeros(128, dtype=torch.uint8, device=dev)
        if rank == 0:
            uid.copy_(torch.frombuffer(bytearray(pkg.MoeEngine.ep_unique_id()), dtype=torch.uint8))
        dist.broadcast(uid, 0)
        eng.ep_init(bytes(uid.cpu().numpy().tobytes()))
    g = torch.Generator(device=dev)
    g.manual_seed(shape.seed + 2000 + rank)
    t = torch.randn((T, H), generator=g, device=dev).bfloat16()
    x = torch.randn((T, H), generator=g, device=dev).bfloat16()
    stream = torch.cuda.current_stream().cuda_stream
    steps = max(3, min(args.steps, 30))
    names = ["route", "permute", "gate_up", "down", "combine"]
    if world > 1:
        names += ["dispatch", "return"]

    def timed(T=T):
        for _ in range(3):
            eng.forward(0, t, x, None, T, stream)
        barrier()
        if eng.device_status() != 0:
            raise SystemExit("device status non-zero in the 120b-shape layer")
        eng.set_option("time_stages", 1)
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(steps):
            eng.forward(0, t, x, None, T, stream)
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            tt = torch.tensor([ms], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        stage_ms = {s: eng.stage_ms(s) for s in names}
        eng.set_option("time_stages", 0)
        return {"value": world * T * steps / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms / steps,
                "steps": steps, "stage_ms": stage_ms}

    # expert parallelism: rows read from the peers' memory where the ranks could map each
    # other (the default then), and over NCCL send / recv for comparison
    transport = eng.ep_transport if world > 1 else -1
    res = timed()
    other = strong = None
    if world > 1:
        # strong-scaling reading: the same 6144 tokens split over the ranks
        strong = timed(T // world)
        strong["tokens_per_gpu"] = T // world
    overlap = None
    if transport == 1:
        eng.set_option("ep_overlap", 1)
        overlap = timed()
        eng.set_option("ep_overlap", 0)
        eng.set_option("ep_transport", 0)
        other = timed()
    eng.close()
    how = {-1: "all experts local", 0: f"expert parallel x{world} (NCCL send/recv)",
           1: f"expert parallel x{world} (rows read from peer memory over NVLink)"}[transport]
    out = {"workload": shape.name, "tokens_per_gpu": T, "experts": E, "parallelism": how}
    out.update(res)
    # rank 0's own gate_up launch; under expert parallelism its row count varies a little
    # around T*K per rank
    out["gate_up_tflops"] = 2.0 * T * K * 2 * IM * H / (res["stage_ms"]["gate_up"] * 1e-3) / 1e12
    if strong is not None:
        out["strong_scaling"] = strong
    if overlap is not None:
        out["peer_memory_with_gather_overlap"] = overlap
    if other is not None:
        out["nccl_send_recv"] = other
    return out


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
        dist.init_process_group("nccl", device_id=dev)

    pkg = entry.load_package()
    T, H, IM, E, K = (shape.n_tokens, shape.hidden_dim, shape.intermediate_dim, shape.n_experts,
                      shape.experts_per_token)
    eng = pkg.MoeEngine(H, IM, E, K, n_layers=1, max_tokens=T, swiglu_limit=shape.swiglu_limit,
                        device=local_rank)
    w = device_weights(shape, dev)
    eng.load_layer_bf16(0, w["w_router"], w["b_router"], w["w_mlp1"], w["b_mlp1"], w["w_mlp2"],
                        w["b_mlp2"], on_device=True)
    if os.environ.get("GPTOSS_GEMM_IMPL"):  # 0 = single-CTA tcgen05, 2 = CTA pairs
        eng.set_option("gemm_impl", int(os.environ["GPTOSS_GEMM_IMPL"]))
    if os.environ.get("GPTOSS_PAIR_STAGES"):  # tuning aid
        eng.set_option("pair_stages", int(os.environ["GPTOSS_PAIR_STAGES"]))
    if os.environ.get("GPTOSS_SKIP_EPILOGUE"):  # measurement aid: main loop only
        eng.set_option("skip_epilogue", int(os.environ["GPTOSS_SKIP_EPILOGUE"]))
    g = torch.Generator(device=dev)
    g.manual_seed(shape.seed + 1000 + rank)
    t = torch.randn((T, H), generator=g, device=dev).bfloat16()
    x0 = torch.randn((T, H), generator=g, device=dev).bfloat16()
    x = x0.clone()
    stream = torch.cuda.current_stream().cuda_stream

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        eng.forward(0, t, x, None, T, stream)
    barrier()
    if eng.device_status() != 0:
        raise SystemExit("device status non-zero after warm-up")
    x.copy_(x0)
    eng.set_option("time_stages", 1)
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    launches0 = eng.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        eng.forward(0, t, x, None, T, stream)
    ev1.record()
    barrier()
    clocks = sampler.result()
    elapsed_ms = ev0.elapsed_time(ev1)
    launches = eng.launch_count() - launches0
    stage_ms = {s: eng.stage_ms(s) for s in ("route", "permute", "gate_up", "down", "combine")}
    eng.set_option("time_stages", 0)
    if world > 1:
        tt = torch.tensor([elapsed_ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        elapsed_ms = float(tt.item())
    value = world * T * args.steps / (elapsed_ms * 1e-3)

    # end to end through the host-buffer entry point: pinned host inputs copied in,
    # result copied out, every step
    # (a) one call per step that copies in, computes, copies out and returns;
    # (b) the streaming pair submit / wait: three batches in flight, each in its own pinned
    #     buffers, so the copies of neighbouring steps overlap the kernels.  Every step still
    #     moves its own inputs in and its own result out.
    t_h = t.cpu().pin_memory()
    x_h = x0.cpu().pin_memory()
    e2e_steps = max(3, min(args.steps, 20))

    def timed_host(fn):
        fn(2)
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

    e2e_sync_value = timed_host(sync_steps)
    e2e_streamed_t = timed_host(streamed(True))
    # (c) as (b), but only the residual stream crosses the bus: the block's RMSNorm (scale 1
    #     here) runs on the device, as in the model, instead of the caller sending t as well
    eng.load_ffn_norm(0, np.ones(H, dtype=np.float32))
    e2e_value = timed_host(streamed(False))

    extra = None
    if not args.no_extra and args.workload == "c2":
        extra = measure_c3_layer(args, pkg, dev, rank, world, local_rank, barrier)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = read_peaks()
    n_assign = T * K
    flops_gate_up = 2.0 * n_assign * 2 * IM * H
    timed_s = elapsed_ms * 1e-3
    peak_kind = "bf16_tflops" if timed_s < 1.0 else "bf16_tflops_sustained"
    achieved = flops_gate_up / (stage_ms["gate_up"] * 1e-3) / 1e12
    # DRAM traffic of one gate_up launch: the ncu capture of the small case c2s read and wrote
    # 377.2 MB against 348.0 MB algorithmic (weights once, rows in, activations out); c2 has four
    # times the rows and four times the experts, so the same ratio is applied to its bytes.
    alg_bytes = E * 2 * IM * H * 2 + n_assign * H * 2 + n_assign * IM * 2
    gate_up_traffic = (377.2 / 348.0) * alg_bytes if shape.name in C2S_RATIO_WORKLOADS else None
    roofline = {
        "kernel": ("grouped_gemm_tc_kernel<240, swiglu> (gate_up, single CTA)"
                   if os.environ.get("GPTOSS_GEMM_IMPL") == "0"
                   else "grouped_gemm_pair_kernel<swiglu, 6> (gate_up, CTA pairs)"),
        "bound": "tensor",
        "achieved": achieved, "peak": peaks[peak_kind], "unit": "TFLOP/s",
        "frac": achieved / peaks[peak_kind], "peak_source": f"{peaks['source']} {peak_kind}",
        "traffic": gate_up_traffic, "traffic_unit": "bytes/launch",
        "traffic_source": "ncu dram__bytes_read+write of the c2s capture (377.2 MB, a quarter of the "
                          "rows and of the experts), scaled by rows x experts",
        "kernel_ms": stage_ms["gate_up"],
        "stage_ms": stage_ms,
        "down_tflops": 2.0 * n_assign * H * IM / (stage_ms["down"] * 1e-3) / 1e12,
        "route_gbs": (T * H * 2 + E * H * 2 + T * K * 8) / (stage_ms["route"] * 1e-3) / 1e9,
        "combine_gbs": (n_assign * H * 2 + 2 * T * H * 2) / (stage_ms["combine"] * 1e-3) / 1e9,
        "hbm_peak_gbs": peaks["hbm_gbs"],
    }

    cpu_baseline = None
    if not args.no_cpu_baseline and world == 1:  # the CPU figure is a 1-process measurement
        oracle = entry.load_oracle()
        if not oracle.ORACLE_LIB.exists():
            oracle.build(native=True)
        kind = "reference" if oracle.have_ref() else "port"
        w_host = host_weights_f32(w)

        def sample(n):
            return cpu_sample(shape, w_host, t[:n].float().cpu().numpy(),
                              x0[:n].float().cpu().numpy(), n, kind)

        if args.cpu_tokens:
            n_cpu = min(T, args.cpu_tokens)
            sec = sample(n_cpu)
        else:
            # size the sample for about 12 s of CPU work on this box's cores
            n_cpu = min(T, 64)
            sec = sample(n_cpu)
            want = min(T, max(64, int(12.0 / (sec / n_cpu)) // 64 * 64))
            if want > 2 * n_cpu:
                n_cpu = want
                sec = sample(n_cpu)
        cpu_baseline = {"value": n_cpu / sec, "unit": UNIT,
                        "cores": oracle.num_threads("ref" if kind == "reference" else "oracle"),
                        "kind": kind,
                        "sample": f"first {n_cpu} tokens of the batch, {K} experts each, {sec:.1f} s"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": shape.name, "tokens_per_gpu": T, "hidden": H, "intermediate": IM,
                   "experts": E, "top_k": K, "parallelism": f"replicas x{world}",
                   "l2": "inputs larger than L2 (expert weights %.2f GB streamed every step)"
                         % ((E * 3 * IM * H * 2) / 1e9)},
        "roofline": roofline, "cpu_baseline": cpu_baseline,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": T * H * 2,
                "d2h_bytes_per_step": T * H * 2, "steps": e2e_steps,
                "how": "gptoss_moe_forward_host_submit / _wait, three batches in flight; x in, "
                       "RMSNorm + block on the device, x out",
                "streamed_with_t_from_host": {"value": e2e_streamed_t,
                                              "h2d_bytes_per_step": 2 * T * H * 2},
                "one_call_per_step": {"value": e2e_sync_value,
                                      "h2d_bytes_per_step": 2 * T * H * 2}},
        "gpu_launches": launches, "clocks": clocks,
    }
    if extra is not None:
        extra["gate_up_frac_of_peak"] = extra["gate_up_tflops"] / peaks["bf16_tflops"]
        line["layer_120b"] = extra
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_decode_mxfp4(args):
    """--workload c4: the 120b-shape layer with MXFP4 expert weights at decode batch
    sizes T = 64 / 256 / 1024, router biased so that expert popularity is skewed
    (Zipf(1.1) weights over a seeded permutation of the experts).  Bound by HBM: the
    packed weights of every touched expert are streamed once per layer pass."""
    import torch

    pkg = entry.load_package()
    shape = workload_shape("c3")
    H, IM, E, K = shape.hidden_dim, shape.intermediate_dim, shape.n_experts, shape.experts_per_token
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    g = torch.Generator(device=dev)
    g.manual_seed(4)
    eng = pkg.MoeEngine(H, IM, E, K, max_tokens=1024, weight_format=pkg.WEIGHTS_MXFP4)
    if os.environ.get("GPTOSS_SKIP_EPILOGUE"):  # measurement aid
        eng.set_option("skip_epilogue", int(os.environ["GPTOSS_SKIP_EPILOGUE"]))

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
    b_router = (zipf / zipf.sum()).log().float() * 0.83
    w_router = (torch.randn((E, H), generator=g, device=dev) * 0.08).bfloat16()
    b1 = (torch.randn((E, 2 * IM), generator=g, device=dev) * 0.01).float()
    b2 = (torch.randn((E, H), generator=g, device=dev) * 0.01).float()
    eng.load_layer_mxfp4(0, w_router, b_router, codes(2 * IM, H), scales(2 * IM, H), b1,
                         codes(H, IM), scales(H, IM), b2, on_device=True)
    torch.cuda.empty_cache()
    peaks = read_peaks()
    stream = torch.cuda.current_stream().cuda_stream
    per_expert_bytes = 3 * IM * H // 2 + 3 * IM * H // 32
    results = {}
    sampler = ClockSampler(0)
    sampler.start()
    for T in (64, 256, 1024):
        t = (torch.randn((T, H), generator=g, device=dev) * 0.25).bfloat16()
        x = torch.randn((T, H), generator=g, device=dev).bfloat16()
        for _ in range(args.warmup):
            eng.forward(0, t, x, None, T, stream)
        torch.cuda.synchronize()
        if eng.device_status() != 0:
            raise SystemExit("device status non-zero")
        eng.set_option("time_stages", 1)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(args.steps):
            eng.forward(0, t, x, None, T, stream)
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1) / args.steps
        stage_ms = {s: eng.stage_ms(s) for s in ("route", "permute", "gate_up", "down", "combine")}
        eng.set_option("time_stages", 0)
        r = eng.get_routing(T)
        counts = np.bincount(r["topk_i"].ravel(), minlength=E)
        touched = int((counts > 0).sum())
        gemm_ms = stage_ms["gate_up"] + stage_ms["down"]
        results[T] = {
            "tokens_per_s": T / (ms * 1e-3), "ms_per_step": ms, "stage_ms": stage_ms,
            "experts_touched": touched, "busiest_expert_share": float(counts.max() / counts.sum()),
            "weight_gbs": touched * per_expert_bytes / (gemm_ms * 1e-3) / 1e9,
        }
    clocks = sampler.result()
    top = results[1024]
    line = {
        "metric": METRIC, "value": top["tokens_per_s"], "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": top["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "gpt-oss-120b-moe-layer-mxfp4-decode-T1024", "hidden": H,
                   "intermediate": IM, "experts": E, "top_k": K, "weights": "MXFP4 (e2m1 + e8m0/32)",
                   "routing": "Zipf(1.1)-biased router", "l2": "inputs larger than L2 (1.69 GB of "
                   "packed expert weights streamed every step)"},
        "roofline": {"kernel": "grouped_gemm_pair_kernel<*, 5, mxfp4> (gate_up + down)",
                     "bound": "hbm", "achieved": top["weight_gbs"], "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": top["weight_gbs"] / peaks["hbm_gbs"],
                     "peak_source": f"{peaks['source']} hbm_gbs", "traffic": None},
        "decode": {str(k): v for k, v in results.items()}, "cpu_baseline": None,
        "e2e": None, "gpu_launches": eng.launch_count(), "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    eng.close()


def run_decode_120b(args):
    """--workload c5: one decode step of a 120b-architecture model (36 layers, hidden 2880,
    64 query / 8 KV heads of 64, sinks, 128-token window on even layers, 128 experts top-4,
    vocabulary 201088), random-init weights generated on the device, 6144 sequences split
    over the GPUs, each with 512 positions of synthetic KV context; experts sharded over
    the ranks (16 per GPU at 8).  Needs at least 2 GPUs: the bf16 experts alone are 229 GB.
    GPTOSS_C5_LAYERS cuts the layer count for development runs (reported in the line)."""
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
    ctx, total_seqs = 512, 6144
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
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c2s", "c4", "c5", "tiny"])
    ap.add_argument("--cpu-tokens", type=int, default=None,
                    help="tokens in the CPU sample (default 256 for ours, 64 for reference)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the 120b-shape layer measured beside the headline workload")
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
        run_ours(args, shape)


if __name__ == "__main__":
    main()
