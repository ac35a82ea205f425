"""Benchmark of the MoE layer path: `python bench.py --gpus N --steps K --warmup W [--impl reference]`.

Workload (N = 1): the Flash-Next-shaped decode layer — hidden 2048, 512 routed experts, softmax top-10 renormalised,
one always-on shared expert, intermediate 512, IQ3_S expert weights quantised from N(0, 0.02), router scaled so the
top-10 mass is about 0.6, bf16 activations N(0,1), 64 decode tokens, 4 stacked layers (each layer has its own router
and experts and reads the step's activations). One step = one pass of the 64 tokens through the 4 layers, router to
combine. The expert weights of the 4 layers (2.8 GB) are far larger than L2, so every step streams them from HBM.

One JSON line on stdout (rank 0):
  value      layer-tokens per second = tokens * layers / step time, inputs resident in HBM, CUDA-event timed: the K-step
             region is timed `--repeats` times and the median taken (min / max under "repeats")
  e2e        the same through host buffers: pinned-host -> device copy of the activations and device -> host copy of
             the layer outputs of every step inside the timed region; two buffer sets, the copies on their own streams
             (they overlap the neighbouring steps' layer calls); serial_ms_per_step = everything on one stream
  roofline   the dominant kernel (the grouped gate/up + SwiGLU product, timed alone): GGUF block bytes of the gate and
             up matrices of the experts it touched / its CUDA-event duration, against the measured HBM copy bandwidth
  sweep, workloads   extra records, not the headline: the decode batch sweep (1 / 4 / 16 tokens) of the same layers and
             one record per other benchmark configuration (c3 4096 tokens, c4 16 and 2048 tokens, c5 8192 tokens)
  cpu_baseline  the reference's production CPU expert pool timed on this box's host cores on a bounded sample

`--impl reference` times the reference's CPU implementation of the path on the same workload, one layer per step: its
production expert pool (CpuMissPool: int8 AVX2 gate / up dots) where the checker library holds it, with the
reference's fp32 host path (dequantize_host + moe_expert_ffn) as a second, labelled record.
"""
from __future__ import annotations

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

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
TOKENS, LAYERS = 64, 4
SEED = 20261125
# dense tensor-core peaks nobody measured on this pool: NVIDIA's per-GPU figures for B200 (labelled "nominal" wherever used)
NOMINAL_TFLOPS = {"int8": 4500.0, "fp4": 9000.0}


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
    p.add_argument("--graph", type=int, default=1, help="1: replay the step as a CUDA graph (expert parallel: the compute phases only, the "
                        "collectives between them are issued directly); 0: launch everything directly")
    p.add_argument("--repeats", type=int, default=30, help="how many times the K-step region is timed (the median is reported)")
    p.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    p.add_argument("--no-extras", action="store_true", help="skip the sweep and the records of the other configurations")
    p.add_argument("--iq3s-layout", default="codes", choices=("codes", "gguf"), help="bank layout of IQ3_S experts")
    p.add_argument("--ring", default="", help="nbuf,stages,slot_tiles: force the decode kernels' shared-memory configuration (A/B timing)")
    p.add_argument("--column-split", type=int, default=0, help="1 / 2 / 4: most warps of the decode kernels that share a row job (0: the library's default)")
    p.add_argument("--peer-exchange", type=int, default=1, help="expert parallel: 1 = the two fixed-size exchanges of a layer over peer memory "
                   "(the library's own put / wait kernels), 0 = NCCL collectives")
    p.add_argument("--overlap", type=int, default=1, help="0: plain stream order between the launches of a layer instead of programmatic dependent launch")
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


def cpu_model():
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


# ------------------------------------------------------------------------------------------------ CPU arms ----
class CpuLayer:
    """one layer of the workload on the host: raw GGUF blocks as numpy arrays + the routing inputs"""

    def __init__(self, shape, layer, x):
        self.shape = shape
        self.x = x.float().cpu().numpy()
        self.raw = [t.cpu().numpy() for t in layer.raw]
        self.sh = tuple(t.cpu().numpy() for t in layer.shared_raw) if layer.shared_raw is not None else None
        self.rw = layer.router_w.cpu().numpy()
        self.bias = None if layer.sel_bias is None else layer.sel_bias.cpu().numpy()
        self.E = self.rw.shape[0]


def pool_threads():
    """workers of the reference's pool: it pins them to CPUs 1 .. T and the calling thread to CPU 0"""
    return max(1, (os.cpu_count() or 2) - 1)


def time_pool_layer(cl: CpuLayer, pool, orc, ref):
    """seconds for one layer through the reference's production path: router logits (fp32 dots), moe_route, CpuMissPool, combine"""
    sh = cl.shape
    t0 = time.perf_counter()
    logits = orc.router_logits(cl.rw, cl.x)
    ids, w = (ref or orc).route(sh.gating, logits, sh.topk, sh.norm, sh.scale, cl.bias)
    pool.layer(x=cl.x, ids=ids, weights=w, ff=sh.ff, types=sh.types, gate=cl.raw[0], up=cl.raw[1], down=cl.raw[2], experts=cl.E, shared=cl.sh)
    return time.perf_counter() - t0


def time_fp32_layer(cl: CpuLayer, orc, ref, threads):
    """seconds for one layer through the fp32 host path (the reference's dequantize_host + moe_expert_ffn, or the oracle port)"""
    sh = cl.shape
    t0 = time.perf_counter()
    if ref is not None:
        logits = orc.router_logits(cl.rw, cl.x)          # the reference CPU path has no router GEMV of its own (moe.cu is CUDA)
        ref.moe_layer(x=cl.x, topk=sh.topk, ff=sh.ff, gating=sh.gating, norm=sh.norm, scale=sh.scale, types=sh.types, gate=cl.raw[0],
                      up=cl.raw[1], down=cl.raw[2], experts=cl.E, logits_in=logits, shared=cl.sh, sel_bias=cl.bias, threads=threads)
        return time.perf_counter() - t0, "reference"
    orc.moe_layer(x=cl.x, router_w=cl.rw, topk=sh.topk, ff=sh.ff, gating=sh.gating, norm=sh.norm, scale=sh.scale, types=sh.types,
                  gate=cl.raw[0], up=cl.raw[1], down=cl.raw[2], experts=cl.E, shared=cl.sh, sel_bias=cl.bias, threads=threads)
    return time.perf_counter() - t0, "port"


def pool_usable(shape):
    """the production pool has int8 kernels for IQ3_S gate / up rows (it dequantises any other type row by row); its job
    arrays hold up to 8 token columns, which the shim respects"""
    return shape.hidden % 256 == 0 and shape.ff % 32 == 0 and all(t in (12, 20, 21, 23) for t in shape.types)


def cpu_arm(cl: CpuLayer, budget_s: float, max_reps: int, want_fp32: bool):
    """the CPU records: production pool (when it can be had) and, if wanted, the fp32 path; each on about budget_s of work"""
    import oracle
    orc, ref = oracle.oracle(), oracle.reference()
    ncpu = os.cpu_count() or 1
    out = {}
    if want_fp32:
        dt, kind = time_fp32_layer(cl, orc, ref, ncpu)
        reps = max(1, min(max_reps, int(budget_s / max(dt, 1e-3))))
        tot = sum(time_fp32_layer(cl, orc, ref, ncpu)[0] for _ in range(reps))
        out["fp32"] = {"value": cl.x.shape[0] * reps / tot, "unit": UNIT, "cores": ncpu, "kind": kind,
                       "path": "fp32 host path: dequantize_host + moe_route + moe_expert_ffn + moe_combine, one thread per expert",
                       "sample": f"1 layer, {cl.x.shape[0]} tokens, {reps} passes ({tot:.1f} s)", "ms_per_layer": tot / reps * 1e3}
    pool = oracle.reference_pool() if pool_usable(cl.shape) else None
    if pool is not None:
        threads = pool_threads()
        pool.create(threads, cl.shape.hidden, cl.shape.ff)       # pins this thread to CPU 0 from here on
        dt = time_pool_layer(cl, pool, orc, ref)
        reps = max(1, min(max_reps, int(budget_s / max(dt, 1e-3))))
        tot = sum(time_pool_layer(cl, pool, orc, ref) for _ in range(reps))
        out["pool"] = {"value": cl.x.shape[0] * reps / tot, "unit": UNIT, "cores": threads + 1, "kind": "reference",
                       "path": "production CPU expert pool of the reference (CpuMissPool: int8 AVX2 gate / up dots, bf16 / fp16 rounding), "
                               f"{threads} pinned workers + the calling thread",
                       "sample": f"1 layer, {cl.x.shape[0]} tokens, {reps} passes ({tot:.1f} s)", "ms_per_layer": tot / reps * 1e3,
                       "nproc": ncpu, "cpu": cpu_model()}
    return out


def run_reference(args):
    """the reference's CPU implementation of the path on this box's host cores; rank 0 only"""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from tqllm_b200 import synth
    shape = synth.CONFIGS[args.workload]
    layers, rscale = make_layers(synth, shape, 1, "cpu")
    x = synth.make_tokens(shape, args.tokens, SEED, "cpu")
    cl = CpuLayer(shape, layers[0], x)
    import oracle
    orc, ref = oracle.oracle(), oracle.reference()
    ncpu = os.cpu_count() or 1
    steps, warm = max(1, min(args.steps, 200)), min(args.warmup, 3)
    fp32_dt, fp32_kind = time_fp32_layer(cl, orc, ref, ncpu)         # second record: the fp32 host path, a few passes
    fp32_reps = max(1, min(10, int(5.0 / max(fp32_dt, 1e-3))))
    fp32_t = sum(time_fp32_layer(cl, orc, ref, ncpu)[0] for _ in range(fp32_reps)) / fp32_reps
    pool = oracle.reference_pool() if pool_usable(shape) else None
    if pool is not None:
        threads = pool_threads()
        pool.create(threads, shape.hidden, shape.ff)
        fn = lambda: time_pool_layer(cl, pool, orc, ref)
        kind, cores, path = "reference-production", threads + 1, f"CpuMissPool, {threads} pinned workers + the calling thread"
    else:
        fn = lambda: time_fp32_layer(cl, orc, ref, ncpu)[0]
        kind, cores, path = fp32_kind, ncpu, "fp32 host path (no production pool for this configuration or host)"
    for _ in range(warm):
        fn()
    times = [fn() for _ in range(steps)]
    t = sum(times) / len(times)
    v = args.tokens / t
    print(json.dumps({
        "metric": METRIC, "value": v, "unit": UNIT, "impl": "reference", "n_gpus": args.gpus, "steps": steps, "warmup": warm,
        "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8+f32" if pool is not None else "f32",
        "data": "synthetic",
        "config": {"workload": workload_name(shape, args.tokens, args.layers), "sample": "one layer per step", "router_scale": rscale},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": kind, "path": path, "nproc": ncpu, "cpu": cpu_model(),
                         "sample": f"1 of {args.layers} layers, {args.tokens} tokens, {steps} steps"},
        "fp32_path": {"value": args.tokens / fp32_t, "unit": UNIT, "cores": ncpu, "kind": fp32_kind, "ms_per_layer": fp32_t * 1e3,
                      "path": "dequantize_host + moe_route + moe_expert_ffn + moe_combine, one thread per expert", "passes": fp32_reps},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ------------------------------------------------------------------------------------------------ GPU arm ----
def graph_of(torch, stream, fn):
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        fn()
    return g


def pipelined_e2e_ms(torch, stream, x_host, xs, outs_dev, outs_host, runs, n):
    """ms per step of n end-to-end steps with the copies on their own streams: step i's host -> device copy, its layer calls
    and its device -> host copy run in that order, but the copies of one step overlap the layer calls of its neighbours (two
    sets of device and host buffers, taken in turn). Every copy lies between the two events on the launching stream."""
    s_in, s_out = torch.cuda.Stream(stream.device), torch.cuda.Stream(stream.device)
    ev = lambda: [torch.cuda.Event(), torch.cuda.Event()]
    in_done, comp_done, out_done = ev(), ev(), ev()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for st in (stream, s_in, s_out):
        st.synchronize()
    e0.record(stream)
    s_in.wait_event(e0)
    for i in range(n):
        b = i & 1
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(comp_done[b])                          # step i - 2 has read this input buffer
            xs[b].copy_(x_host, non_blocking=True)
            in_done[b].record(s_in)
        stream.wait_event(in_done[b])
        if i >= 2:
            stream.wait_event(out_done[b])                             # step i - 2's outputs have left this output buffer
        with torch.cuda.stream(stream):
            runs[b]()
            comp_done[b].record(stream)
        with torch.cuda.stream(s_out):
            s_out.wait_event(comp_done[b])
            outs_host[b].copy_(outs_dev[b], non_blocking=True)
            out_done[b].record(s_out)
    for b in range(min(n, 2)):
        stream.wait_event(out_done[b])
    e1.record(stream)
    stream.synchronize()
    return e0.elapsed_time(e1) / n


def event_ms(torch, stream, fn, n):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    stream.synchronize()
    e0.record(stream)
    for _ in range(n):
        fn()
    e1.record(stream)
    stream.synchronize()
    return e0.elapsed_time(e1) / n


def expert_products(torch, moe, lib, C, lay, x, shape, stream):
    """closures that launch the two expert products of layer `lay` on tokens x, with their plan, for stage timing"""
    T = x.shape[0]
    ST = T if shape.shared else 0
    lg = moe.router(lay.router_w, x)
    if shape.gating == 1:
        ids, _, _ = moe.topk_softmax(lg, lay.experts, shape.topk, shape.scale)
    else:
        ids, _ = moe.route_sigmoid(lg, lay.experts, shape.topk, lay.sel_bias, shape.norm, shape.scale)
    plan = moe.dispatch(ids, lay.experts, ST)
    A = T * shape.topk
    XDT = {torch.bfloat16: 2, torch.float16: 1, torch.float32: 0}[x.dtype]
    act = torch.zeros(A + ST, shape.ff, dtype=torch.float32, device=x.device)
    y = torch.zeros(A + ST, shape.hidden, dtype=torch.float32, device=x.device)
    gws = torch.empty(max(lib.b2moe_expert_workspace_bytes(lay.gate.type, T, shape.hidden, XDT), 16), dtype=torch.uint8, device=x.device)
    dws = torch.empty(max(lib.b2moe_expert_workspace_bytes(lay.down.type, A + ST, shape.ff, 0), 16), dtype=torch.uint8, device=x.device)
    shp = lambda i: C.byref(lay.sh[i].c) if shape.shared else None
    st = stream.cuda_stream

    def gateup():
        rc = lib.b2moe_expert_gateup_swiglu(C.byref(lay.gate.c), C.byref(lay.up.c), shp(0), shp(1), x.data_ptr(), XDT, plan.buf.data_ptr(), T,
                                            shape.topk, ST, act.data_ptr(), gws.data_ptr(), gws.numel(), st)
        assert rc == 0, rc

    def down():
        rc = lib.b2moe_expert_down(C.byref(lay.down.c), shp(2), act.data_ptr(), plan.buf.data_ptr(), T, shape.topk, ST, y.data_ptr(),
                                   dws.data_ptr(), dws.numel(), st)
        assert rc == 0, rc
    return gateup, down, plan, (act, y, gws, dws, ids, lg)


def bank_bytes_of(lib, bank):
    return lib.b2moe_bank_bytes(bank.type, bank.rows, bank.cols)


def workload_record(torch, moe, synth, lib, C, stream, dev, cfg, tokens, layout):
    """one record of another benchmark configuration: one layer, `tokens` tokens, the layer as a CUDA-graph replay and its
    gate/up product alone, with both roofline fractions"""
    shape = synth.CONFIGS[cfg]
    sl = synth.make_layer(shape, SEED + 7, dev)
    x = synth.make_tokens(shape, tokens, SEED + 9, dev)
    bias_note = None
    if cfg == "c5":
        x, bias_note = zipf_router(torch, shape, sl.router_w, x, dev)
    lay = moe.MoeLayer.from_synth(sl, device=dev, iq3s_layout=layout)
    del sl
    torch.cuda.empty_cache()
    out = torch.empty(tokens, shape.hidden, dtype=torch.bfloat16, device=dev)
    with torch.cuda.stream(stream):
        for _ in range(2):
            lay.forward(x, out=out)
        stream.synchronize()
        g = graph_of(torch, stream, lambda: lay.forward(x, out=out))
        for _ in range(2):
            g.replay()
        layer_ms = event_ms(torch, stream, g.replay, 10)
        art = lay.artefacts()
        n_active = art["n_active"]
        counts = art["counts"].cpu().numpy()[:shape.experts]
        gateup, down, plan, keep = expert_products(torch, moe, lib, C, lay, x, shape, stream)
        gateup(); down()
        gu_ms = event_ms(torch, stream, gateup, 10)
        dn_ms = event_ms(torch, stream, down, 10)
        status = int(plan.buf[3])
    A = tokens * shape.topk + (tokens if shape.shared else 0)
    gu_bytes = n_active * 2 * synth.raw_bytes(shape.types[0], shape.ff, shape.hidden)
    flops_gu = 4.0 * shape.hidden * shape.ff * A
    hbm, _ = peaks()
    bf16, _ = peaks("bf16_tflops")
    rec = {
        "workload": workload_name(shape, tokens, 1), "tokens": tokens, "layer_us": layer_ms * 1e3, "layer_tokens_per_s": tokens / (layer_ms * 1e-3),
        "gateup_us": gu_ms * 1e3, "down_us": dn_ms * 1e3, "active_experts": n_active, "tokens_per_expert_mean": tokens * shape.topk / shape.experts,
        "tokens_per_expert_max": int(counts.max()), "status": status,
        "gateup_gbs": gu_bytes / (gu_ms * 1e-3) / 1e9, "gateup_hbm_frac": gu_bytes / (gu_ms * 1e-3) / 1e9 / hbm,
        "gateup_tflops": flops_gu / (gu_ms * 1e-3) / 1e12, "gateup_frac_of_bf16_measured": flops_gu / (gu_ms * 1e-3) / 1e12 / bf16,
        "layer_expert_weight_gbs": n_active * shape.expert_bytes() / (layer_ms * 1e-3) / 1e9,
    }
    # which roofline binds: weights streamed once per active expert against the flops at the measured bf16 rate
    t_hbm, t_tensor = gu_bytes / (hbm * 1e9), flops_gu / (bf16 * 1e12)
    rec["bound"] = "hbm" if t_hbm >= t_tensor else "tensor"
    rec["roofline_frac"] = max(t_hbm, t_tensor) / (gu_ms * 1e-3)
    if bias_note:
        rec["routing"] = bias_note
    del lay, g
    torch.cuda.empty_cache()
    return rec


def run_b200(args):
    import ctypes as C

    import torch
    import torch.distributed as dist

    from tqllm_b200 import capi, moe, synth
    lib = capi.lib
    lib.b2moe_harness_overlap(1 if args.overlap else 0)
    if args.column_split:
        lib.b2moe_harness_column_split(args.column_split)
    if args.ring:
        lib.b2moe_harness_ring(*[int(v) for v in args.ring.split(",")])

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the MoE path has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        return run_ep(args, torch, dist, capi, moe, synth, rank, world, local, dev)
    shape = synth.CONFIGS[args.workload]
    T, L = args.tokens, args.layers
    synth_layers, rscale = make_layers(synth, shape, L, dev)
    layers = [moe.MoeLayer.from_synth(sl, device=dev, iq3s_layout=args.iq3s_layout) for sl in synth_layers]
    x = synth.make_tokens(shape, T, SEED, dev)
    cpu_layer = CpuLayer(shape, synth_layers[0], x) if not args.no_cpu and args.workload == "c2" else None
    del synth_layers
    torch.cuda.empty_cache()
    out_all = torch.empty(L, T, shape.hidden, dtype=torch.bfloat16, device=dev)      # the layers' outputs side by side: one copy back
    outs = [out_all[l] for l in range(L)]
    for lay in layers:
        lay.reserve(T)

    def step():
        for lay, o in zip(layers, outs):
            lay.forward(x, out=o)

    # pinned host buffers of the end-to-end leg
    x_host = x.cpu().pin_memory()
    out_host = torch.empty(L, T, shape.hidden, dtype=torch.bfloat16).pin_memory()

    run_holder = [step]                     # the layer calls of one step: the graph replay once it is captured

    def step_e2e():
        x.copy_(x_host, non_blocking=True)
        run_holder[0]()
        out_host.copy_(out_all, non_blocking=True)

    stream = torch.cuda.Stream(dev)
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            step()
        stream.synchronize()
        n0 = lib.b2moe_harness_launches()
        step()
        launches_per_step = int(lib.b2moe_harness_launches() - n0)       # counted by the library: every kernel it launched in one step
        stream.synchronize()
        graph = graph_of(torch, stream, step) if args.graph else None
        run = graph.replay if graph is not None else step
        run_holder[0] = run
        for _ in range(args.warmup):
            run()
        R = max(1, args.repeats)
        with ClockSampler(local) as clocks:
            reg = [event_ms(torch, stream, run, args.steps) for _ in range(R)]       # ms per step of each K-step region
        for _ in range(min(args.warmup, 3)):
            step_e2e()
        reg_e2e = [event_ms(torch, stream, step_e2e, args.steps) for _ in range(max(1, min(R, 10)))]
        ms_step, ms_e2e_serial = statistics.median(reg), statistics.median(reg_e2e)
        # the same with a second set of buffers and the copies on their own streams (the figure that is reported)
        x_b, out_all_b = torch.empty_like(x), torch.empty_like(out_all)
        out_host_b = torch.empty_like(out_host).pin_memory()

        def step_b():
            for l, lay in enumerate(layers):
                lay.forward(x_b, out=out_all_b[l])

        x_b.copy_(x)
        step_b()
        stream.synchronize()
        run_b = graph_of(torch, stream, step_b).replay if args.graph else step_b
        pipe = (torch, stream, x_host, [x, x_b], [out_all, out_all_b], [out_host, out_host_b], [run, run_b])
        pipelined_e2e_ms(*pipe, max(args.steps, 4))
        reg_e2e = [pipelined_e2e_ms(*pipe, args.steps) for _ in range(max(1, min(R, 10)))]
        ms_e2e = statistics.median(reg_e2e)
        if not torch.equal(out_host, out_host_b):
            raise SystemExit("bench.py: the two buffer sets of the end-to-end leg disagree")

        # stage timings: every stage of a layer alone (CUDA events on the launching stream around graph replays), averaged over the layers
        prods = [expert_products(torch, moe, lib, C, lay, x, shape, stream) for lay in layers]

        def time_stage(fns, reps=max(3, min(args.steps, 20))):
            """mean microseconds of one call: the calls (one per layer) replayed as a CUDA graph, so that the host's launch cost
            is not on the clock"""
            for f in fns:
                f()
            stream.synchronize()
            g = graph_of(torch, stream, lambda: [f() for f in fns])
            g.replay()
            return event_ms(torch, stream, g.replay, reps) * 1e3 / len(fns)

        gu_call_us = time_stage([p[0] for p in prods])
        dn_call_us = time_stage([p[1] for p in prods])
        lib.b2moe_harness_skip_staging(1)          # the product kernels alone (their activation staging launch left out)
        try:
            gu_us = time_stage([p[0] for p in prods])
            dn_us = time_stage([p[1] for p in prods])
        finally:
            lib.b2moe_harness_skip_staging(0)
        st = stream.cuda_stream
        ST = T if shape.shared else 0
        A = T * shape.topk
        XDT = {torch.bfloat16: 2, torch.float16: 1, torch.float32: 0}[x.dtype]
        logits = torch.zeros(T, shape.experts + 1, dtype=torch.float32, device=dev)
        idb = torch.zeros(T, shape.topk, dtype=torch.int32, device=dev)
        wts = torch.zeros(T, shape.topk, dtype=torch.float32, device=dev)
        ob = torch.zeros(T, shape.hidden, dtype=torch.bfloat16, device=dev)
        plan2 = moe.Plan(shape.experts, T, shape.topk, ST, dev)
        dsw = torch.empty(max(lib.b2moe_dispatch_workspace_bytes(shape.experts, A), 16), dtype=torch.uint8, device=dev)
        bias = lambda lay: None if lay.sel_bias is None else lay.sel_bias.data_ptr()

        def ok(rc):
            assert rc == 0, rc
        stage_us = {
            "router": time_stage([(lambda lay=lay: ok(lib.b2moe_router(lay.router_w.data_ptr(), None, x.data_ptr(), XDT, logits.data_ptr(),
                                                                       shape.experts + 1, shape.hidden, shape.experts, T, st))) for lay in layers]),
            "route_dispatch": time_stage([(lambda lay=lay: ok(lib.b2moe_route_dispatch(shape.gating, logits.data_ptr(), shape.experts + 1, bias(lay),
                                                                                    idb.data_ptr(), wts.data_ptr(), None, shape.experts, shape.topk,
                                                                                    int(shape.norm), shape.scale, T, 0, ST, plan2.buf.data_ptr(),
                                                                                    dsw.data_ptr(), dsw.numel(), st))) for lay in layers]),
            "gateup_swiglu_call": gu_call_us, "gateup_swiglu_kernel": gu_us, "down_call": dn_call_us, "down_kernel": dn_us,
            "combine": time_stage([(lambda p=p: ok(lib.b2moe_combine(p[3][1].data_ptr(), None, wts.data_ptr(), None, T, shape.topk, shape.hidden,
                                                                     ST, ob.data_ptr(), capi.BF16, st))) for p in prods]),
        }
        plans = [p[2] for p in prods]
        n_active = sum(p.n_active for p in plans) / L            # includes the shared expert
        status = max(int(p.buf[3]) for p in plans)
        gu_bank = sum(bank_bytes_of(lib, lay.gate) + bank_bytes_of(lib, lay.up) for lay in layers) / L
        del prods
        torch.cuda.empty_cache()

        # decode batch sweep on the same layers: 1 / 4 / 16 tokens, the L-layer step replayed as a CUDA graph
        sweep = None
        if not args.no_extras and args.workload == "c2":
            sweep = {}
            for ts in (1, 4, 16):
                xs = x[:ts].contiguous()
                os_ = [torch.empty(ts, shape.hidden, dtype=torch.bfloat16, device=dev) for _ in range(L)]

                def small_step():
                    for lay, o in zip(layers, os_):
                        lay.forward(xs, out=o)
                for _ in range(3):
                    small_step()
                stream.synchronize()
                g = graph_of(torch, stream, small_step)
                for _ in range(5):
                    g.replay()
                us_layer = event_ms(torch, stream, g.replay, 50) * 1e3 / L
                act_l = sum(lay.artefacts()["n_active"] for lay in layers) / L
                sweep[str(ts)] = {"us_per_layer": us_layer, "tokens_per_s": ts / (us_layer * 1e-6), "active_experts": act_l,
                                  "expert_weight_gbs": act_l * shape.expert_bytes() / (us_layer * 1e-6) / 1e9}
                del g
            for lay in layers:
                lay.reserve(T)

        # the fixed-total-batch anchor of the multi-GPU runs: 512 tokens on this one GPU, the same 4 layers
        fixed = None
        if not args.no_extras and args.workload == "c2":
            xf = synth.make_tokens(shape, 512, SEED + 100, dev)
            of = [torch.empty(512, shape.hidden, dtype=torch.bfloat16, device=dev) for _ in range(L)]

            def step_fixed():
                for lay, o in zip(layers, of):
                    lay.forward(xf, out=o)
            for _ in range(3):
                step_fixed()
            stream.synchronize()
            g = graph_of(torch, stream, step_fixed)
            g.replay()
            ms_f = event_ms(torch, stream, g.replay, 20)
            fixed = {"tokens_total": 512, "tokens_per_gpu": 512, "ms_per_step": ms_f, "layer_tokens_per_s": 512 * L / (ms_f * 1e-3)}
            del g, of
            for lay in layers:
                lay.reserve(T)

    gu_bytes = 2 * synth.raw_bytes(shape.types[0], shape.ff, shape.hidden)
    peak, peak_kind = peaks()
    bound, roof_unit = "hbm", "GB/s"
    k_ms = gu_us * 1e-3
    achieved = n_active * gu_bytes / (k_ms * 1e-3) / 1e9
    weight_bytes_step = n_active * L * shape.expert_bytes()
    if T * shape.topk >= 128 * shape.experts:                # >= 128 tokens per expert: the tensor cores bound the product
        bound, roof_unit = "tensor", "TFLOP/s"
        achieved = 4.0 * shape.hidden * shape.ff * (T * shape.topk + (T if shape.shared else 0)) / (k_ms * 1e-3) / 1e12
        peak, peak_kind = peaks("bf16_tflops")
    value = T * L / (ms_step * 1e-3)
    e2e = T * L / (ms_e2e * 1e-3)
    # DRAM bytes of one launch of the dominant kernel: the bytes of the gate and up banks of the experts it touched, in the
    # layout it reads (IQ3_S as 4-bit codes: 134 bytes per 256 weights against the 110 of the GGUF block). A constant of the
    # layout, not a live counter; one ncu capture of this kernel measured 1.00x of it.
    traffic = n_active * gu_bank / max(1, layers[0].experts)
    graphed = graph is not None

    workloads = None
    if not args.no_extras and args.workload == "c2":
        del layers, graph
        torch.cuda.empty_cache()
        workloads = {}
        for key, cfg, toks in (("c4_decode_16", "c4", 16), ("c3_prefill_4096", "c3", 4096), ("c4_prefill_2048", "c4", 2048), ("c5_prefill_8192", "c5", 8192)):
            try:
                workloads[key] = workload_record(torch, moe, synth, lib, C, stream, dev, cfg, toks, args.iq3s_layout)
            except Exception as e:                                  # a record that fails must not take the headline with it
                workloads[key] = {"error": f"{type(e).__name__}: {e}"[:300]}

    cpu = None
    if cpu_layer is not None:
        arms = cpu_arm(cpu_layer, 8.0, 64, want_fp32=True)       # last: the reference's pool pins this thread to CPU 0
        cpu = arms.get("pool") or arms.get("fp32")
        if cpu is not None and "fp32" in arms and cpu is not arms["fp32"]:
            cpu = dict(cpu, fp32_path=arms["fp32"])

    print(json.dumps({
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8+f32", "data": "synthetic",
        "config": {"workload": workload_name(shape, T, L), "tokens": T, "layers": L, "router_scale": rscale, "parallelism": "single GPU",
                   "l2": "per-step expert weights (GBs) exceed the 126 MB L2; no flush needed", "cuda_graph": graphed, "e2e_leg": ("every step: pinned H2D copy of its tokens, " + ("the same graph replay" if graphed else "direct launches") + ", one D2H copy of all layer outputs; two buffer sets taken in turn, copies on their own streams so that they overlap the neighbouring steps' layer calls; e2e.serial_ms_per_step = the same on one stream"), "dependent_launch_overlap": bool(args.overlap),
                   "activations": "bf16 in, bf16 out; expert products on integer tensor-core MMA over 15-bit fixed-point activations, fp32 sums",
                   "iq3s_bank_layout": args.iq3s_layout},
        "repeats": {"n": len(reg), "ms_per_step_median": ms_step, "ms_per_step_min": min(reg), "ms_per_step_max": max(reg),
                    "e2e_n": len(reg_e2e), "e2e_min": min(reg_e2e), "e2e_max": max(reg_e2e)},
        "e2e": {"value": e2e, "unit": UNIT, "ms_per_step": ms_e2e, "serial_ms_per_step": ms_e2e_serial, "h2d_bytes_per_step": x_host.numel() * 2,
                "d2h_bytes_per_step": out_host.numel() * 2},
        "gpu_launches": args.steps * launches_per_step, "launches_per_step": launches_per_step,
        "roofline": {"bound": bound, "kernel": "grouped gate/up + SwiGLU product (its launch alone)", "achieved": achieved, "peak": peak, "unit": roof_unit,
                     "frac": achieved / peak, "peak_kind": peak_kind, "traffic": traffic,
                     "traffic_source": "bytes of the banks the launch reads in their HBM layout (a constant of the layout, not a counter)",
                     "kernel_ms": k_ms, "active_experts_per_launch": n_active, "bytes_per_expert": gu_bytes, "status": status},
        "expert_weight_gbs": weight_bytes_step / (ms_step * 1e-3) / 1e9,
        "expert_weight_frac_of_8tbs": weight_bytes_step / (ms_step * 1e-3) / 8e12,
        "stage_us": stage_us, "sweep": sweep, "fixed_total_512": fixed, "workloads": workloads,
        "nominal_peaks_not_measured": {"int8_tops_dense": NOMINAL_TFLOPS["int8"], "fp4_tflops_dense": NOMINAL_TFLOPS["fp4"],
                                       "note": "NVIDIA's per-GPU B200 figures; only the HBM copy rate and the bf16 GEMM rate were measured on this pool"},
        "cpu_baseline": cpu, "clocks": clocks.summary(),
    }))


def zipf_router(torch, shape, router_w, x, dev):
    """Zipf(s = 1.2) pressure on the routing: router rows of expert e grow along a direction every token shares, by an amount
    that falls like log(rank^-1.2), tuned so that the hottest expert holds about 10x the mean token count; returns (x, note)"""
    d = torch.zeros(shape.hidden, device=dev)
    d[::5] = 1.0
    d /= d.norm()
    x = (x.float() + 3.0 * d).to(x.dtype)
    rank = torch.arange(1, shape.experts + 1, device=dev, dtype=torch.float32)
    base = router_w.clone()
    lo, hi, ratio, w = 0.0, 4.0, 1.0, base
    for _ in range(18):
        c = 0.5 * (lo + hi)
        w = base + (c * -1.2 * torch.log(rank))[:, None] * d[None, :] / 3.0
        cnt = torch.bincount((x.float() @ w.T).topk(shape.topk, -1).indices.flatten(), minlength=shape.experts).float()
        ratio = float(cnt.max() / cnt.mean())
        lo, hi = (c, hi) if ratio < 10.0 else (lo, c)
    router_w.copy_(w)
    return x, f"Zipf(1.2) routing pressure through the router rows: hottest expert {ratio:.1f}x the mean token count"


def ep_layers(torch, moe, synth, ep, shape, L, rank, world, dev, layout, rscale=1.0, zipf_tokens=None, order_of=None):
    """every rank draws the same layers (same seed) and keeps the banks of its own expert block only; order_of(layer) may
    return a placement (b2moe_place_experts) in which the experts are stacked before the blocks are cut"""
    first, count = ep.expert_range(shape.experts, world, rank)
    H, F = shape.hidden, shape.ff
    out, note = [], None
    for l in range(L):
        sl = synth.make_layer(shape, SEED + 17 * l, dev, router_scale=rscale)
        if zipf_tokens is not None:
            _, note = zipf_router(torch, shape, sl.router_w, zipf_tokens, dev)
        if order_of is not None:
            sl = synth.permute_experts(sl, order_of(sl))
        cut = lambda raw, i: raw[first * synth.raw_bytes(shape.types[i], (F, F, H)[i], (H, H, F)[i]):
                                 (first + count) * synth.raw_bytes(shape.types[i], (F, F, H)[i], (H, H, F)[i])].clone()
        lay = moe.MoeLayer(shape, sl.router_w[first:first + count], tuple(cut(sl.raw[i], i) for i in range(3)), sl.shared_raw,
                           experts=count, device=dev, iq3s_layout=layout)
        out.append(ep.CudaEpLayer(lay, sl.router_w.contiguous(), shape.experts, world, rank,
                                  sel_bias_all=None if sl.sel_bias is None else sl.sel_bias.contiguous()))
        del sl
        torch.cuda.empty_cache()
    return out, note


def ep_record(torch, dist, moe, synth, ep, comm, stream, dev, rank, world, cfg, total_tokens, a2a, layout, reps=10):
    """one expert-parallel record of another configuration: one layer, total_tokens over all ranks, direct launches; the time is
    the maximum over the ranks. The Zipf-routed configuration (c5) is timed twice: contiguous expert blocks, and the load-aware
    placement that b2moe_place_experts derives from the routing histogram of the same tokens (b2moe_count)."""
    shape = synth.CONFIGS[cfg]
    T = max(1, total_tokens // world)
    x_all = synth.make_tokens(shape, T * world, SEED + 9, dev)                # the same tokens on every rank; a rank routes its slice
    zx = x_all if cfg == "c5" else None
    if cfg == "c5":
        d = torch.zeros(shape.hidden, device=dev)
        d[::5] = 1.0
        d /= d.norm()
        x_shift = (x_all.float() + 3.0 * d).to(x_all.dtype)
    else:
        x_shift = x_all
    x = x_shift[rank * T:(rank + 1) * T].contiguous()
    fwd = ep.ep_forward_a2a if a2a else ep.ep_forward
    loads = {}

    def histogram(sl):                      # routed-id counts of all tokens on the full expert set: the same on every rank
        logits = moe.router(sl.router_w.contiguous(), x_shift, None)
        if shape.gating == synth.SOFTMAX:
            ids, _, _ = moe.topk_softmax(logits, shape.experts, shape.topk, shape.scale)
        else:
            ids, _ = moe.route_sigmoid(logits, shape.experts, shape.topk, sl.sel_bias, shape.norm, shape.scale)
        counts = torch.zeros(shape.experts, dtype=torch.int64, device=dev)
        moe.count_ids(ids.contiguous().view(-1), counts)
        return counts

    def placed(sl):
        counts = histogram(sl)
        order, load = moe.place_experts(counts, world)
        loads["contiguous"] = [int(v) for v in counts.view(world, -1).sum(1).tolist()]
        loads["load_aware"] = [int(v) for v in load.tolist()]
        return order

    def timed(order_of):
        eps, note = ep_layers(torch, moe, synth, ep, shape, 1, rank, world, dev, layout, zipf_tokens=zx, order_of=order_of)
        with torch.cuda.stream(stream):
            dist.barrier()                                               # the ranks finish building their layers at different times
            for _ in range(2):
                fwd(eps[0], comm, x)
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                fwd(eps[0], comm, x)
            e1.record(stream)
            torch.cuda.synchronize()
            ms = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            n_active = torch.tensor([float(int(eps[0].buf["plan"][0]))], device=dev)
            status = torch.tensor([float(int(eps[0].buf["plan"][3]))], device=dev)
            dist.all_reduce(n_active, op=dist.ReduceOp.SUM)
            dist.all_reduce(status, op=dist.ReduceOp.MAX)
        del eps
        torch.cuda.empty_cache()
        return float(ms), float(n_active), int(status), note

    ms, n_active, status, note = timed(None)
    rec = {"workload": workload_name(shape, T * world, 1), "tokens_total": T * world, "tokens_per_gpu": T,
           "dispatch": "all-to-all (count exchange + variable-size records)" if a2a else "all-gather", "placement": "contiguous expert blocks",
           "layer_us": ms * 1e3, "layer_tokens_per_s": T * world / (ms * 1e-3), "active_experts_all_ranks": n_active,
           "expert_weight_gbs_all_ranks": n_active * shape.expert_bytes() / (ms * 1e-3) / 1e9, "status": status}
    if note:
        rec["routing"] = note
    if cfg == "c5":
        ms2, _, status2, _ = timed(placed)
        rec["load_aware_placement"] = {"layer_us": ms2 * 1e3, "layer_tokens_per_s": T * world / (ms2 * 1e-3), "status": status2,
                                       "assignments_per_rank_contiguous": loads.get("contiguous"),
                                       "assignments_per_rank_load_aware": loads.get("load_aware"),
                                       "how": "b2moe_count histogram of the same tokens -> b2moe_place_experts -> experts stacked in that order"}
    return rec


def run_ep(args, torch, dist, capi, moe, synth, rank, world, local, dev):
    """expert parallel over `world` GPUs of one box: every rank keeps the banks of its own expert block and routes its own tokens"""
    from tqllm_b200 import ep
    lib = capi.lib
    shape = synth.CONFIGS[args.workload]
    T, L = args.tokens, args.layers
    rscale = synth.solve_router_scale(shape, 0.6) if args.workload == "c2" else 1.0
    eps, _ = ep_layers(torch, moe, synth, ep, shape, L, rank, world, dev, args.iq3s_layout, rscale)
    layers = [e.layer for e in eps]
    x = synth.make_tokens(shape, T, SEED + rank, dev)
    comm = ep.TorchComm()                   # NCCL: the variable-size all-to-all records, and the fallback
    hc, exchange = comm, "NCCL all-gather dispatch + all-to-all combine"
    if args.peer_exchange:
        try:
            hc = ep.PeerComm()
            hc.all_gather(torch.zeros(4, 16, dtype=torch.uint8, device=dev))       # set-up and one exchange; every rank fails or none does
            torch.cuda.synchronize()
            hc.check()
            exchange = "dispatch and combine exchanges over peer memory (put + bounded wait kernels, plain NVLink stores)"
        except Exception as e:
            hc, exchange = comm, exchange + f" (peer memory unavailable: {type(e).__name__}: {e})"[:200]
    if hc is not comm:                      # the two transports must give the same bits
        for e in eps:
            want = ep.ep_forward(e, comm, x).clone()
            got = ep.ep_forward(e, hc, x)
            torch.cuda.synchronize()
            if not torch.equal(got, want):
                raise SystemExit("bench.py: the peer-memory exchange and the NCCL exchange disagree")
    outs = [None] * L

    def step_direct():
        for l, e in enumerate(eps):
            outs[l] = ep.ep_forward(e, hc, x)
    step = step_direct

    x_host = x.cpu().pin_memory()
    out_host = torch.empty(L, T, shape.hidden, dtype=torch.bfloat16).pin_memory()
    stream = torch.cuda.Stream(dev)
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            step()
        stream.synchronize()
        n0 = lib.b2moe_harness_launches()
        step()
        launches_per_step = int(lib.b2moe_harness_launches() - n0)
        stream.synchronize()
        graph_note, whole = False, None
        if args.graph and getattr(hc, "capturable", False):
            # the peer-memory exchanges are the library's own kernels (bounded waits, device-side sequence numbers): the whole
            # step, exchanges included, is one graph
            captured = 1
            try:
                whole = torch.cuda.CUDAGraph()
                with torch.cuda.graph(whole, stream=stream):
                    step_direct()
            except Exception:
                captured, whole = 0, None
            flag = torch.tensor([captured], dtype=torch.int32, device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)                 # every rank replays a graph or none does; also: nobody replays
            torch.cuda.synchronize()                                     # (and waits on a peer) while a peer is still capturing
            if int(flag):
                step = whole.replay
                graph_note = "whole step, peer-memory exchanges included"
            else:
                whole = None
        elif args.graph:                 # only the compute phases are captured, no collective is
            graphed = [ep.GraphedEpForward(e, hc, x) for e in eps]

            def step_graphed():
                for l, gf in enumerate(graphed):
                    outs[l] = gf()
            step = step_graphed
            graph_note = "compute phases only"

        def step_e2e():
            x.copy_(x_host, non_blocking=True)
            step()
            for l in range(L):
                out_host[l].copy_(outs[l], non_blocking=True)

        def timed(fn, steps):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
            torch.cuda.synchronize()
            ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            dist.barrier()
            return float(ms) / steps

        for _ in range(args.warmup):
            step()
        R = max(1, min(args.repeats, 10))
        with ClockSampler(local) as clocks:
            reg = [timed(step, args.steps) for _ in range(R)]
        for _ in range(min(args.warmup, 3)):
            step_e2e()
        reg_e2e = [timed(step_e2e, args.steps) for _ in range(max(1, min(R, 5)))]
        ms_step, ms_e2e = statistics.median(reg), statistics.median(reg_e2e)
        # where a layer's time goes on this rank: every phase bracketed by events (direct launches, not the graphed ones)
        phase_us = ep.phase_times(eps[0], hc, x, reps=20)
        torch.cuda.synchronize()
        n_active = sum(int(e.buf["plan"][0]) for e in eps) / L      # this rank's active experts per layer (with the shared one)
        # a fixed total batch beside the weak-scaling value: 512 tokens over all ranks, the same 4 layers
        fixed = None
        if not args.no_extras and args.workload == "c2" and 512 % world == 0:
            xf = synth.make_tokens(shape, 512 // world, SEED + 100 + rank, dev)
            gf = [ep.GraphedEpForward(e, hc, xf) for e in eps] if args.graph else None

            def step_fixed():
                for l, e in enumerate(eps):
                    gf[l]() if gf is not None else ep.ep_forward(e, hc, xf)
            for _ in range(3):
                step_fixed()
            ms_f = statistics.median([timed(step_fixed, args.steps) for _ in range(3)])
            fixed = {"tokens_total": 512, "tokens_per_gpu": 512 // world, "ms_per_step": ms_f, "layer_tokens_per_s": 512 * L / (ms_f * 1e-3)}
            del gf
    workloads = None
    if not args.no_extras and args.workload == "c2":
        del eps, layers
        graphed = whole = step = None
        torch.cuda.empty_cache()
        workloads = {}
        for key, cfg, toks, a2a in (("c4_decode_16", "c4", 16, False), ("c4_prefill_2048", "c4", 2048, True), ("c5_prefill_8192", "c5", 8192, True)):
            try:
                workloads[key] = ep_record(torch, dist, moe, synth, ep, comm if a2a else hc, stream, dev, rank, world, cfg, toks, a2a, args.iq3s_layout)
            except Exception as e:                                  # every rank fails or none does: the shapes are the same everywhere
                workloads[key] = {"error": f"{type(e).__name__}: {e}"[:300]}
    wait_status = 0
    if hc is not comm:                      # a wait that ran out (a peer more than its bound late) shows here; the medians survive one stall
        st = hc.status.clone()
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
        wait_status = int(st)
        if wait_status and rank == 0:
            print(f"bench.py: a peer-memory wait ran out during this run (status {wait_status})", file=sys.stderr)
    peak, peak_kind = peaks()
    weight_bytes_step = n_active * L * shape.expert_bytes()
    achieved = weight_bytes_step / (ms_step * 1e-3) / 1e9
    value = world * T * L / (ms_step * 1e-3)
    e2e = world * T * L / (ms_e2e * 1e-3)
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8+f32", "data": "synthetic",
            "config": {"workload": workload_name(shape, T, L), "tokens": T, "layers": L, "router_scale": rscale,
                       "parallelism": f"ep{world}: {shape.experts // world} experts per GPU, {T} tokens per GPU, {exchange}",
                       "l2": "per-step expert weights exceed the 126 MB L2; no flush needed",
                       "cuda_graph": graph_note, "peer_wait_status": wait_status, "iq3s_bank_layout": args.iq3s_layout},
            "repeats": {"n": len(reg), "ms_per_step_median": ms_step, "ms_per_step_min": min(reg), "ms_per_step_max": max(reg)},
            "e2e": {"value": e2e, "unit": UNIT, "ms_per_step": ms_e2e, "h2d_bytes_per_step": x_host.numel() * 2,
                    "d2h_bytes_per_step": out_host.numel() * 2},
            "gpu_launches": args.steps * launches_per_step, "launches_per_step": launches_per_step,
            "roofline": {"bound": "hbm", "kernel": "whole expert-parallel layer on rank 0 (dispatch + combine exchanges included)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind, "traffic": None,
                         "kernel_ms": ms_step / L, "active_experts_per_launch": n_active,
                         "bytes_per_expert": 2 * synth.raw_bytes(shape.types[0], shape.ff, shape.hidden)},
            "expert_weight_gbs": weight_bytes_step / (ms_step * 1e-3) / 1e9, "stage_us": phase_us,
            "fixed_total_512": fixed, "workloads": workloads,
            "cpu_baseline": None, "clocks": clocks.summary(),
        }))
    dist.destroy_process_group()


if __name__ == "__main__":
    a = parse()
    defaults(a)
    run_reference(a) if a.impl == "reference" else run_b200(a)
