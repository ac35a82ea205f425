"""Benchmark of the MoE layer path: `python bench.py --gpus N --steps K --warmup W [--impl reference]`.

Workload (N = 1): the Flash-Next-shaped decode layer — hidden 2048, 512 routed experts, softmax top-10 renormalised,
one always-on shared expert, intermediate 512, IQ3_S expert weights quantised from N(0, 0.02), router scaled so the
top-10 mass is about 0.6, bf16 activations N(0,1), 64 decode tokens, 4 stacked layers (each layer has its own router
and experts and reads the step's activations). One step = one pass of the 64 tokens through the 4 layers, router to
combine. The expert weights of the 4 layers (2.8 GB) are far larger than L2, so every step streams them from HBM.

One JSON line on stdout (rank 0):
  value      layer-tokens per second = tokens * layers / step time, inputs resident in HBM, CUDA-event timed
  e2e        the same through host buffers: pinned-host -> device copy of the activations and device -> host copy of
             the layer outputs inside the timed region
  roofline   the dominant kernel (the grouped gate/up + SwiGLU product): GGUF block bytes of the gate and up matrices
             of the experts it touched / its CUDA-event duration, against the measured HBM copy bandwidth
  cpu_baseline  the CPU path timed on this box's host cores on a bounded sample (one layer, the same 64 tokens)

`--impl reference` times the reference's CPU implementation of the path (the reference's own sources compiled in place
under oracle/_ref when present, else the oracle restatement) on the same workload, one layer per step.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
TOKENS, LAYERS = 64, 4
SEED = 20261125


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=50)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="b200", choices=("b200", "reference"))
    p.add_argument("--workload", default="c2", choices=("c1", "c2", "c3", "c4", "c5"),
                   help="layer shape (tqllm_b200.synth.CONFIGS); c2 is the headline workload, the others are for profiling")
    p.add_argument("--tokens", type=int, default=0, help="tokens per step per GPU (default: 64; 4096 / 2048 / 8192 for c3 / c4 / c5)")
    p.add_argument("--layers", type=int, default=0, help="stacked layers per step (default: 4 for c2, else 1)")
    p.add_argument("--graph", type=int, default=1, help="1: replay the step as a CUDA graph (expert parallel: the compute phases only, the collectives between them are "
                        "issued directly); 0: launch everything directly")
    p.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    p.add_argument("--sweep", action="store_true", help="also time 1 / 4 / 16 tokens (extra keys, not the headline)")
    return p.parse_args()


def peaks(key="hbm_gbs"):
    """the roofline denominator: the pool's measured copy bandwidth (GB/s) or burst bf16 GEMM rate (TFLOP/s), else the stated fallback"""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        return float(json.load(open(path))[key]), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}[key], "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs"""
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            self.t.join(timeout=2)

    def summary(self):
        sm = sorted(int(r[1]) for r in self.rows if len(r) >= 8 and r[1].isdigit())
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 8 and r[4 + i].lower().startswith("active") for r in self.rows)]
        mx = max(int(r[2]) for r in self.rows if len(r) >= 8 and r[2].isdigit())
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": mx, "reasons": reasons, "samples": len(sm)}


FMT_NAMES = {12: "Q4_K", 20: "IQ4_NL", 21: "IQ3_S", 23: "IQ4_XS", 323: "NVFP4G"}


def workload_name(shape, tokens, layers):
    fm = "+".join(dict.fromkeys(FMT_NAMES[t] for t in shape.types))
    kind = {"c2": "c2 flash-next decode", "c1": "c1 small", "c3": "c3 flash-next prefill", "c4": "c4 minimax", "c5": "c5 prefill"}[shape.name[:2]]
    return (f"{kind}: H{shape.hidden} E{shape.experts} top{shape.topk}{'+1 shared' if shape.shared else ''} F{shape.ff} {fm}, "
            f"{tokens} tokens x {layers} stacked layers")


def defaults(args):
    if not args.tokens:
        args.tokens = {"c3": 4096, "c4": 2048, "c5": 8192}.get(args.workload, TOKENS)
    if not args.layers:
        args.layers = LAYERS if args.workload == "c2" else 1


def make_layers(synth, shape, layers, device, experts=None):
    scale = synth.solve_router_scale(shape, 0.6) if shape.name.startswith("c2") else 1.0      # c2: top-10 mass about 0.6
    return [synth.make_layer(shape, SEED + 17 * l, device, experts=experts, router_scale=scale) for l in range(layers)], scale


# ------------------------------------------------------------------------------------------------ CPU arm ----
def cpu_layer_time(kind_wanted, shape, layer, x, threads):
    """seconds for one layer forward of x on the host cores; returns (seconds, kind)"""
    import numpy as np

    import oracle
    orc = oracle.oracle()
    ref = oracle.reference() if kind_wanted == "reference" else None
    xf = x.float().cpu().numpy()
    raw = [t.cpu().numpy() for t in layer.raw]
    sh = tuple(t.cpu().numpy() for t in layer.shared_raw) if layer.shared_raw is not None else None
    rw = layer.router_w.cpu().numpy()
    E = rw.shape[0]
    t0 = time.perf_counter()
    if ref is not None:
        logits = orc.router_logits(rw, xf)          # the reference CPU path has no router GEMV of its own (moe.cu is CUDA)
        ref.moe_layer(x=xf, topk=shape.topk, ff=shape.ff, gating=shape.gating, norm=shape.norm, scale=shape.scale, types=shape.types,
                      gate=raw[0], up=raw[1], down=raw[2], experts=E, logits_in=logits, shared=sh, threads=threads)
        kind = "reference"
    else:
        orc.moe_layer(x=xf, router_w=rw, topk=shape.topk, ff=shape.ff, gating=shape.gating, norm=shape.norm, scale=shape.scale,
                      types=shape.types, gate=raw[0], up=raw[1], down=raw[2], experts=E, shared=sh, threads=threads)
        kind = "port"
    return time.perf_counter() - t0, kind


def run_reference(args):
    """the reference's CPU implementation of the path on this box's host cores; rank 0 only"""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch

    from tqllm_b200 import synth
    shape = synth.CONFIGS[args.workload]
    threads = os.cpu_count() or 1
    layers, rscale = make_layers(synth, shape, 1, "cpu")
    x = synth.make_tokens(shape, args.tokens, SEED, "cpu")
    steps = max(1, min(args.steps, 200))          # one layer pass (about 0.3 s on 16 cores) per step
    for _ in range(min(args.warmup, 3)):
        cpu_layer_time("reference", shape, layers[0], x, threads)
    times = []
    kind = "port"
    for _ in range(steps):
        dt, kind = cpu_layer_time("reference", shape, layers[0], x, threads)
        times.append(dt)
    t = sum(times) / len(times)
    v = args.tokens / t
    print(json.dumps({
        "metric": METRIC, "value": v, "unit": UNIT, "impl": "reference", "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 3),
        "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(shape, args.tokens, args.layers), "sample": "one layer per step", "router_scale": rscale},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": kind,
                         "sample": f"1 of {args.layers} layers, {args.tokens} tokens, {steps} steps"},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ------------------------------------------------------------------------------------------------ GPU arm ----
def run_b200(args):
    import torch
    import torch.distributed as dist

    from tqllm_b200 import moe, synth

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the MoE path has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    shape = synth.CONFIGS[args.workload]
    T, L = args.tokens, args.layers
    if world > 1 and args.workload != "c2":
        raise SystemExit("bench.py: the expert-parallel arm runs the c2 workload")
    router_all = None
    if world > 1:
        # expert parallel: every rank draws the same layer (same seed), keeps the banks of its own expert block only
        from tqllm_b200 import ep
        first, count = ep.expert_range(shape.experts, world, rank)
        rscale = synth.solve_router_scale(shape, 0.6)
        layers, router_all = [], []
        H, F = shape.hidden, shape.ff
        for l in range(L):
            sl = synth.make_layer(shape, SEED + 17 * l, dev, router_scale=rscale)
            cut = lambda raw, i: raw[first * synth.raw_bytes(shape.types[i], (F, F, H)[i], (H, H, F)[i]):
                                     (first + count) * synth.raw_bytes(shape.types[i], (F, F, H)[i], (H, H, F)[i])].clone()
            layers.append(moe.MoeLayer(shape, sl.router_w[first:first + count], tuple(cut(sl.raw[i], i) for i in range(3)), sl.shared_raw,
                                       experts=count, device=dev))
            router_all.append(sl.router_w.contiguous())
            del sl
            torch.cuda.empty_cache()
        synth_layers = []
    else:
        synth_layers, rscale = make_layers(synth, shape, L, dev)
        layers = [moe.MoeLayer.from_synth(sl, device=dev) for sl in synth_layers]
    host_layer0 = synth_layers[0] if rank == 0 and not args.no_cpu and world == 1 and args.workload == "c2" else None
    if host_layer0 is not None:      # keep only the first layer's raw blocks (for the CPU baseline), on the host
        host_layer0 = synth.Layer(shape, host_layer0.router_w.cpu(), None, tuple(t.cpu() for t in host_layer0.raw),
                                  tuple(t.cpu() for t in host_layer0.shared_raw))
    del synth_layers
    torch.cuda.empty_cache()
    x = synth.make_tokens(shape, T, SEED + rank, dev)
    outs = [torch.empty(T, shape.hidden, dtype=torch.bfloat16, device=dev) for _ in range(L)]
    if world == 1:
        for lay in layers:
            lay.reserve(T)

    if world > 1:
        from tqllm_b200 import ep
        comm = ep.TorchComm()
        H, F = shape.hidden, shape.ff
        eps = [ep.CudaEpLayer(lay, rw, shape.experts, world, rank) for lay, rw in zip(layers, router_all)]

        def step():
            for l, e in enumerate(eps):
                outs[l] = ep.ep_forward(e, comm, x)
        graphed = None            # built after the warm-up, on the timing stream: compute phases as CUDA graphs, collectives direct
    else:
        def step():
            for lay, o in zip(layers, outs):
                lay.forward(x, out=o)

    # pinned host buffers of the end-to-end leg
    x_host = x.cpu().pin_memory()
    out_host = torch.empty(L, T, shape.hidden, dtype=torch.bfloat16).pin_memory()

    def step_e2e():
        x.copy_(x_host, non_blocking=True)
        step()
        for l in range(L):
            out_host[l].copy_(outs[l], non_blocking=True)

    stream = torch.cuda.Stream(dev)
    graph = None
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            step()
        stream.synchronize()
        if args.graph and world == 1:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step()
        elif args.graph:                   # expert parallel: only the compute phases are captured, no collective is
            graphed = [ep.GraphedEpForward(e, comm, x) for e in eps]

            def step():
                for l, gf in enumerate(graphed):
                    outs[l] = gf()
        run = graph.replay if graph is not None else step

        def timed(fn, steps):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
            torch.cuda.synchronize()
            ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
                dist.barrier()
            return float(ms) / steps

        for _ in range(args.warmup):
            run()
        with ClockSampler(local) as clocks:
            ms_step = timed(run, args.steps)
        for _ in range(min(args.warmup, 3)):
            step_e2e()
        ms_e2e = timed(step_e2e, args.steps)

        if world == 1:
            # dominant kernel, timed alone with events on the launching stream: the grouped gate/up + SwiGLU product
            art = [lay.artefacts() for lay in layers]
            plans, ids = [], []
            ST = T if shape.shared else 0                         # rows of the always-on shared expert
            for lay in layers:
                lg = moe.router(lay.router_w, x)
                if shape.gating == 1:
                    i, w, _ = moe.topk_softmax(lg, lay.experts, shape.topk, shape.scale)
                else:
                    i, w = moe.route_sigmoid(lg, lay.experts, shape.topk, lay.sel_bias, shape.norm, shape.scale)
                plans.append(moe.dispatch(i, lay.experts, ST))
            act = torch.zeros(T * shape.topk + ST, shape.ff, dtype=torch.float32, device=dev)
            XDT = {torch.bfloat16: 2, torch.float16: 1, torch.float32: 0}[x.dtype]
            shp = lambda lay, i: C.byref(lay.sh[i].c) if shape.shared else None
            import ctypes as C
            from tqllm_b200.capi import lib, BF16

            wsb = lib.b2moe_expert_workspace_bytes(layers[0].gate.type, T, shape.hidden, XDT)
            ews = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)

            def gateup(l):
                lay = layers[l]
                return lib.b2moe_expert_gateup_swiglu(C.byref(lay.gate.c), C.byref(lay.up.c), shp(lay, 0), shp(lay, 1),
                                                      x.data_ptr(), XDT, plans[l].buf.data_ptr(), T, shape.topk, ST, act.data_ptr(),
                                                      ews.data_ptr(), ews.numel(), stream.cuda_stream)
            for l in range(L):
                assert gateup(l) == 0

            def time_stage(fn):
                """mean microseconds of fn(layer) over the layers, each launch bracketed by events on the launching stream"""
                for l in range(L):
                    assert fn(l) == 0
                evs = []
                for _ in range(max(3, min(args.steps, 20))):
                    for l in range(L):
                        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        a.record(stream); fn(l); b.record(stream)
                        evs.append((a, b))
                torch.cuda.synchronize()
                return 1e3 * sum(a.elapsed_time(b) for a, b in evs) / len(evs)

            k_ms = time_stage(gateup) * 1e-3
            # the other stages, the same way (reported as stage_us; they explain ms_per_step)
            F32 = 0
            st = stream.cuda_stream
            A = T * shape.topk
            logits = torch.zeros(T, shape.experts + 1, dtype=torch.float32, device=dev)
            idb = torch.zeros(T, shape.topk, dtype=torch.int32, device=dev)
            wts = torch.zeros(T, shape.topk, dtype=torch.float32, device=dev)
            yb = torch.zeros(A + ST, shape.hidden, dtype=torch.float32, device=dev)
            ob = torch.zeros(T, shape.hidden, dtype=torch.bfloat16, device=dev)
            dws = torch.empty(max(lib.b2moe_expert_workspace_bytes(layers[0].down.type, A + ST, shape.ff, F32), 16), dtype=torch.uint8, device=dev)
            plan2 = moe.Plan(shape.experts, T, shape.topk, ST, dev)
            dsw = torch.empty(max(lib.b2moe_dispatch_workspace_bytes(shape.experts, A), 16), dtype=torch.uint8, device=dev)
            bias = lambda l: None if layers[l].sel_bias is None else layers[l].sel_bias.data_ptr()
            stage_us = {
                "router": time_stage(lambda l: lib.b2moe_router(layers[l].router_w.data_ptr(), None, x.data_ptr(), XDT, logits.data_ptr(),
                                                                shape.experts + 1, shape.hidden, shape.experts, T, st)),
                "topk": time_stage((lambda l: lib.b2moe_topk_softmax(logits.data_ptr(), shape.experts + 1, idb.data_ptr(), wts.data_ptr(), None,
                                                                     shape.experts, shape.topk, T, shape.scale, st)) if shape.gating == 1 else
                                   (lambda l: lib.b2moe_route_sigmoid(logits.data_ptr(), shape.experts + 1, bias(l), idb.data_ptr(), wts.data_ptr(),
                                                                      shape.experts, shape.topk, int(shape.norm), shape.scale, T, st))),
                "dispatch": time_stage(lambda l: lib.b2moe_dispatch(idb.data_ptr(), T, shape.topk, shape.experts, ST, plan2.buf.data_ptr(),
                                                                    dsw.data_ptr(), dsw.numel(), st)),
                "gateup_swiglu": k_ms * 1e3,
                "down": time_stage(lambda l: lib.b2moe_expert_down(C.byref(layers[l].down.c), shp(layers[l], 2), act.data_ptr(),
                                                                   plans[l].buf.data_ptr(), T, shape.topk, ST, yb.data_ptr(), dws.data_ptr(),
                                                                   dws.numel(), st)),
                "combine": time_stage(lambda l: lib.b2moe_combine(yb.data_ptr(), None, wts.data_ptr(), None, T, shape.topk, shape.hidden, ST,
                                                                  ob.data_ptr(), BF16, st)),
            }
        else:
            torch.cuda.synchronize()
            plans, stage_us, k_ms = None, None, None
            n_active_rank = sum(int(e.buf["plan"][0]) for e in eps) / L      # this rank's active experts per layer (with the shared one)
    gu_bytes = 2 * synth.raw_bytes(shape.types[0], shape.ff, shape.hidden)
    peak, peak_kind = peaks()
    bound, roof_unit = "hbm", "GB/s"
    if world == 1:
        n_active = sum(p.n_active for p in plans) / L            # includes the shared expert
        achieved = n_active * gu_bytes / (k_ms * 1e-3) / 1e9
        weight_bytes_step = sum(p.n_active for p in plans) * shape.expert_bytes()
        roof_kernel = "grouped gate/up + SwiGLU"
        if T * shape.topk >= 128 * shape.experts:                # >= 128 tokens per expert: the tensor cores bound the product
            bound, roof_unit = "tensor", "TFLOP/s"
            achieved = 4.0 * shape.hidden * shape.ff * (T * shape.topk + (T if shape.shared else 0)) / (k_ms * 1e-3) / 1e12
            peak, peak_kind = peaks("bf16_tflops")
    else:
        # per-GPU view: the whole layer (exchanges included) against this GPU's HBM: expert bytes it streamed / step time
        n_active = n_active_rank
        weight_bytes_step = n_active_rank * L * shape.expert_bytes()
        achieved = weight_bytes_step / (ms_step * 1e-3) / 1e9
        k_ms = ms_step / L
        roof_kernel = "whole expert-parallel layer on rank 0 (dispatch + combine exchanges included)"
    value = world * T * L / (ms_step * 1e-3)
    e2e = world * T * L / (ms_e2e * 1e-3)
    # DRAM bytes per launch of the dominant kernel: one ncu capture of the c2 gate/up kernel (profiles/iq3s_grouped_decode_c2_t64.md:
    # 317.7 MB read + 1.4 MB written with 353 experts active) scaled by the experts this launch touched; traffic grows with them
    traffic, traffic_src = None, None
    if world == 1 and args.workload == "c2" and T * shape.topk < 32 * shape.experts:
        traffic = (317.7e6 + 1.4e6) / 353.0 * n_active
        traffic_src = "ncu dram__bytes_read+write of one capture, scaled by active experts (profiles/iq3s_grouped_decode_c2_t64.md)"

    sweep = None
    if args.sweep and world == 1:
        # decode batches of 1 / 4 / 16 tokens: all L layers per step, replayed as a CUDA graph like the headline step, CUDA events
        sweep = {}
        with torch.cuda.stream(stream):
            for ts in (1, 4, 16):
                xs = x[:ts].contiguous()
                os_ = [torch.empty(ts, shape.hidden, dtype=torch.bfloat16, device=dev) for _ in range(L)]

                def small_step():
                    for lay, o in zip(layers, os_):
                        lay.forward(xs, out=o)
                for _ in range(3):
                    small_step()
                stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    small_step()
                for _ in range(5):
                    g.replay()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps = 50
                stream.synchronize()
                e0.record(stream)
                for _ in range(reps):
                    g.replay()
                e1.record(stream)
                stream.synchronize()
                us_layer = e0.elapsed_time(e1) * 1e3 / (reps * L)
                act_l = sum(lay.artefacts()["n_active"] for lay in layers) / L
                sweep[str(ts)] = {"us_per_layer": us_layer, "tokens_per_s": ts / (us_layer * 1e-6), "active_experts": act_l,
                                  "expert_weight_gbs": act_l * shape.expert_bytes() / (us_layer * 1e-6) / 1e9}
                del g
            for lay in layers:
                lay.reserve(T)

    cpu = None
    if host_layer0 is not None:
        threads = os.cpu_count() or 1
        xc = x.cpu()
        dt, kind = cpu_layer_time("port", shape, host_layer0, xc, threads)          # warm-up pass, also sizes the sample
        reps = max(1, min(64, int(10.0 / max(dt, 1e-3))))                            # about 10 s of CPU work
        total = sum(cpu_layer_time("port", shape, host_layer0, xc, threads)[0] for _ in range(reps))
        cpu = {"value": T * reps / total, "unit": UNIT, "cores": threads, "kind": kind,
               "sample": f"1 of {L} layers, {T} tokens, {reps} passes ({total:.1f} s)"}

    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(shape, T, L), "tokens": T, "layers": L, "router_scale": rscale,
                       "parallelism": "single GPU" if world == 1 else f"ep{world}: {shape.experts // world} experts per GPU, {T} tokens per GPU, "
                                      "NCCL all-gather dispatch + all-to-all combine",
                       "l2": "per-step expert weights (GBs) exceed the 126 MB L2; no flush needed", "cuda_graph": (graph is not None) or ("compute phases only" if world > 1 and args.graph else False),
                       "activations": "bf16 in, bf16 out, fp32 intermediates"},
            "e2e": {"value": e2e, "unit": UNIT, "ms_per_step": ms_e2e, "h2d_bytes_per_step": x_host.numel() * 2,
                    "d2h_bytes_per_step": out_host.numel() * 2},
            "gpu_launches": args.steps * L * (6 if world == 1 else 9),   # per layer: router, route + dispatch, gate/up, fp16 rows, down, combine
                                                                      # (expert parallel: + top-k, local ids, rank-ordered reduce)
            "roofline": {"bound": bound, "kernel": roof_kernel, "achieved": achieved, "peak": peak, "unit": roof_unit,
                         "frac": achieved / peak, "peak_kind": peak_kind, "traffic": traffic, "traffic_source": traffic_src,
                         "kernel_ms": k_ms,
                         "active_experts_per_launch": n_active, "bytes_per_expert": gu_bytes},
            "expert_weight_gbs": weight_bytes_step / (ms_step * 1e-3) / 1e9,
            "expert_weight_frac_of_8tbs": weight_bytes_step / (ms_step * 1e-3) / 8e12,
            "stage_us": stage_us, "sweep": sweep, "cpu_baseline": cpu, "clocks": clocks.summary(),
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    a = parse()
    defaults(a)
    run_reference(a) if a.impl == "reference" else run_b200(a)
