"""Benchmark of the MoMoE layer hot path: forward + backward tokens/s on the headline layer
(D=2048, H=1024, N=128 experts, K=8 per token, bf16, 16384 tokens per GPU; synthetic seeded inputs).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--save-percent P] [--impl reference]

Prints ONE JSON line.  `value` is measured with inputs resident in HBM; `e2e` runs the same step through the
public `MoE` module starting from pinned host memory and reading the loss back every step.  `roofline` describes
the grouped GEMM launch that takes the largest share of the step, timed with CUDA events inside the timed
region.  `cpu_baseline` (rank 0, 1 GPU only) and `--impl reference` time the CPU restatement of the reference
layer on the host cores on a bounded sample of the same layer.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "momoe-impl_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

METRIC = "MoE layer fwd+bwd tokens/sec (D2048 H1024 N128 K8 bf16)"
CFG = dict(D=2048, H=1024, N=128, K=8, Ks=0, B=8, S=2048, w_std=0.02, zipf=False)
# Optional second workload (--workload large_ep): the large expert-parallel layer, 65536 tokens per GPU, router biased
# with a Zipf(1.1) profile so that the busiest expert receives about 8x the mean.  Not the headline metric.
LARGE_EP = dict(D=7168, H=2048, N=256, K=8, Ks=0, B=32, S=2048, w_std=0.006, zipf=True)
CPU_SAMPLE_TOKENS = 2048


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(tflops=float(p.get("bf16_tflops_sustained", p.get("bf16_tflops"))), hbm=float(p["hbm_gbs"]),
                    source="measured (MEASURED_PEAKS.json, sustained bf16)")
    return dict(tflops=1400.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs (read-only queries)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        # nvidia-smi numbers the box's GPUs; CUDA's device `index` counts inside CUDA_VISIBLE_DEVICES when that is set
        visible = [v.strip() for v in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",") if v.strip()]
        if index < len(visible):
            index = visible[index]
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [v.strip() for v in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
                power.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [s for s, p in zip(sm, power) if p > 0.5 * max(power)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power)}


def make_weights(seed, N, D, H, device, n_total, std=0.02):
    g = torch.Generator(device="cpu").manual_seed(seed)
    Wg = (torch.randn(D, n_total, generator=g) * std).bfloat16()
    # expert weights are generated on the device, a few experts at a time (the fp32 draw of a whole tensor would
    # double its footprint)
    gd = torch.Generator(device=device).manual_seed(seed + 1)
    W1 = torch.empty((N, D, 2 * H), dtype=torch.bfloat16, device=device)
    W2 = torch.empty((N, H, D), dtype=torch.bfloat16, device=device)
    for e0 in range(0, N, 16):
        e1 = min(N, e0 + 16)
        W1[e0:e1] = (torch.randn(e1 - e0, D, 2 * H, generator=gd, device=device) * std).bfloat16()
        W2[e0:e1] = (torch.randn(e1 - e0, H, D, generator=gd, device=device) * std).bfloat16()
    return Wg.to(device), W1, W2


def zipf_biases(x_MD, Wg, N, K, target=8.0, seed=7):
    """Router biases b_e = -alpha * 1.1 * ln(rank_e), rank = seeded permutation of 1..N, alpha by bisection so that
    the busiest expert gets `target` x the mean number of tokens on these inputs."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    rank_e = (torch.randperm(N, generator=g) + 1).float().to(x_MD.device)
    shape = -1.1 * torch.log(rank_e)
    p = torch.softmax((x_MD @ Wg).float(), dim=-1)
    lo, hi = 0.0, 1.0
    for _ in range(24):
        mid = 0.5 * (lo + hi)
        sel = torch.topk(p + mid * shape[None, :], K, dim=-1).indices
        counts = torch.bincount(sel.reshape(-1), minlength=N).float()
        ratio = float(counts.max() / counts.mean())
        if ratio < target:
            lo = mid
        else:
            hi = mid
    return (0.5 * (lo + hi)) * shape


def cpu_sample(steps, warmup, seed=0):
    """CPU restatement of the same layer on a bounded sample (CPU_SAMPLE_TOKENS tokens per step)."""
    from oracle import momoe_oracle as orc
    c = CFG
    torch.manual_seed(seed)
    torch.set_num_threads(os.cpu_count() or 1)
    Wg = (torch.randn(c["D"], c["N"]) * 0.02).bfloat16()
    W1 = (torch.randn(c["N"], c["D"], 2 * c["H"]) * 0.02).bfloat16()
    W2 = (torch.randn(c["N"], c["H"], c["D"]) * 0.02).bfloat16()
    state = orc.cpu_baseline_prepare(Wg, W1, W2)
    del W1, W2
    x = torch.randn(1, CPU_SAMPLE_TOKENS, c["D"])
    biases = torch.zeros(c["N"])
    for _ in range(warmup):
        orc.cpu_baseline_step(state, x, biases, c["K"], c["Ks"])
    t0 = time.perf_counter()
    for _ in range(steps):
        orc.cpu_baseline_step(state, x, biases, c["K"], c["Ks"])
    dt = (time.perf_counter() - t0) / steps
    return dict(value=CPU_SAMPLE_TOKENS / dt, unit="tokens/s", cores=torch.get_num_threads(), kind="port",
                sample="%d tokens per step of the same layer (D%d H%d N%d K%d), fp32 torch on host cores, %d steps"
                       % (CPU_SAMPLE_TOKENS, c["D"], c["H"], c["N"], c["K"], steps),
                ms_per_step=dt * 1e3)


def run_reference_arm(args, rank):
    if rank != 0:
        return
    cb = cpu_sample(args.steps, max(1, min(args.warmup, 3)))
    line = dict(metric=METRIC, value=cb["value"], unit="tokens/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=cb["ms_per_step"], higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="f32", data="synthetic", impl="reference",
                config=dict(workload="cfg2 headline layer D2048 H1024 N128 K8, bounded CPU sample",
                            tokens_per_step=CPU_SAMPLE_TOKENS, save_percent=0),
                cpu_baseline={k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
                e2e=dict(value=cb["value"], unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0)
    print(json.dumps(line), flush=True)


def run_triton_reference(args):
    """Context only (not part of the measurement contract): the UNMODIFIED reference package, installed with pip into
    baseline/_ref, on the same GPU, same layer, same timing protocol.  Its Triton kernels autotune during warm-up."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "momoe")):
        print(json.dumps({"impl": "reference-triton", "unavailable": "baseline/_ref is not installed"}))
        return
    sys.path[:] = [ref_dir] + [p for p in sys.path if os.path.join(ROOT, "momoe-impl_b200") != p]
    import momoe as ref   # the reference package
    assert os.path.dirname(ref.__file__).startswith(ref_dir)
    c = CFG
    D, H, N, K, Ks = c["D"], c["H"], c["N"], c["K"], c["Ks"]
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    Wg, W1, W2 = make_weights(1234, N, D, H, dev, N, c["w_std"])
    moe = ref.MoE(D, H, N, K, Ks, save_percent=args.save_percent, Wg_DN=Wg, Wl1_ND2H=W1, Wl2_NHD=W2)
    del W1, W2
    gen = torch.Generator(device="cpu").manual_seed(100)
    x = torch.randn(c["B"], c["S"], D, generator=gen).bfloat16().to(dev).requires_grad_(True)
    g = torch.randn(c["B"], c["S"], D, generator=gen).bfloat16().to(dev)

    def step():
        for p in moe.parameters():
            p.grad = None
        x.grad = None
        moe(x).backward(g)

    for _ in range(max(args.warmup, 12)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    M = c["B"] * c["S"]
    print(json.dumps(dict(metric=METRIC, impl="reference-triton", value=M / (ms * 1e-3), unit="tokens/s", n_gpus=1,
                          steps=args.steps, ms_per_step=ms, dtype="bf16", data="synthetic",
                          config=dict(workload="cfg2 headline layer, reference package from baseline/_ref",
                                      save_percent=args.save_percent))), flush=True)


def ep_parity_preflight(rank, world, dev):
    """Untimed correctness check of the expert-parallel path before a multi-GPU measurement: one reduced step (1024
    tokens per rank, D512 H256, 8 experts per rank, K=4, save_percent 50) through `ExpertParallelMoE` on this rank's
    token shard and expert block against the single-GPU `MoE` on all tokens and all experts, same seeded problem on
    every rank.  y must be identical bit for bit (same kernels, same per-row arithmetic, same summation order);
    gradients are compared by cosine similarity.  Every figure is the worst over the ranks."""
    import torch.distributed as dist
    import momoe
    from momoe import ep, ops
    Mr, D, H, K, Ks, sp = 1024, 512, 256, 4, 0, 50
    N = 8 * world
    Nl = N // world
    g = torch.Generator().manual_seed(4321)
    x_all = torch.randn(world, 1, Mr, D, generator=g).bfloat16()
    W1 = (torch.randn(N, D, 2 * H, generator=g) * 0.03).bfloat16()
    W2 = (torch.randn(N, H, D, generator=g) * 0.03).bfloat16()
    Wg = (torch.randn(D, N, generator=g) * 0.05).bfloat16()
    gy_all = torch.randn(world, 1, Mr, D, generator=g).bfloat16()
    biases = torch.randn(N, generator=g) * 0.05

    def cos(a, b):
        a, b = a.double().flatten(), b.double().flatten()
        return float(a @ b / (a.norm() * b.norm()).clamp_min(1e-300))

    ref = momoe.MoE(D, H, N, K, Ks, save_percent=sp, Wg_DN=Wg.to(dev), Wl1_ND2H=W1.to(dev), Wl2_NHD=W2.to(dev))
    moe = ep.ExpertParallelMoE(D, H, N, K, Ks, save_percent=sp, Wg_DN=Wg.to(dev),
                               Wl1_ND2H=W1[rank * Nl:(rank + 1) * Nl].to(dev),
                               Wl2_NHD=W2[rank * Nl:(rank + 1) * Nl].to(dev), capacity_factor=float(world))
    moe.forward_chunks = 2     # the overlapped two-half forward pass that the measured layer uses at its size
    with torch.no_grad():
        ref.biases_N.copy_(biases.to(dev))
        moe.biases_N.copy_(biases.to(dev))
    xa = x_all.reshape(1, world * Mr, D).to(dev).requires_grad_(True)
    ya = ref(xa)
    ya.backward(gy_all.reshape(1, world * Mr, D).to(dev))
    xr = x_all[rank].to(dev).requires_grad_(True)
    yr = moe(xr)
    yr.backward(gy_all[rank].to(dev))
    torch.cuda.synchronize()
    ops.check_status(dev)
    sl = slice(rank * Mr, (rank + 1) * Mr)
    gwg = moe.router.Wg_DN.grad.float().clone()
    dist.all_reduce(gwg)
    res = torch.tensor([1.0 if torch.equal(yr[0], ya[0, sl]) else 0.0,
                        cos(xr.grad[0], xa.grad[0, sl]),
                        cos(moe.Wl1_ND2H.grad, ref.momoe.Wl1_ND2H.grad[rank * Nl:(rank + 1) * Nl]),
                        cos(moe.Wl2_NHD.grad, ref.momoe.Wl2_NHD.grad[rank * Nl:(rank + 1) * Nl]),
                        cos(gwg, ref.router.Wg_DN.grad),
                        1.0 if torch.equal(moe.biases_N, ref.biases_N) else 0.0], dtype=torch.float64, device=dev)
    dist.all_reduce(res, op=dist.ReduceOp.MIN)
    r = res.tolist()
    del ref, moe, ya, yr
    torch.cuda.empty_cache()
    return dict(case="1024 tokens per rank, D512 H256, 8 experts per rank, K4, save_percent 50, peer transport, "
                     "forward pass in two overlapping halves",
                y_bit_exact=bool(r[0] == 1.0), dx_cos=round(r[1], 6), dw1_cos=round(r[2], 6), dw2_cos=round(r[3], 6),
                dwg_cos=round(r[4], 6), bias_update_equal=bool(r[5] == 1.0))


def extra_records(args, dev, moe, x_dev, g_dev, M):
    """Untimed-for-`value` records of the 1-GPU line: the same layer at save_percent 100 (nothing recomputed), and the
    unmodified reference package's own Triton kernels on this GPU (a subprocess of `--impl reference-triton`)."""
    import momoe
    out = {}
    try:
        m100 = momoe.MoE(moe.D, moe.H, moe.N, moe.K, moe.Ks, save_percent=100, Wg_DN=moe.router.Wg_DN.detach(),
                         Wl1_ND2H=moe.momoe.Wl1_ND2H.detach(), Wl2_NHD=moe.momoe.Wl2_NHD.detach())

        def step():
            for p in m100.parameters():
                p.grad = None
            x_dev.grad = None
            m100(x_dev).backward(g_dev)

        for _ in range(3):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms100 = e0.elapsed_time(e1) / args.steps
        out["save_percent_100"] = dict(ms_per_step=round(ms100, 4), tokens_per_s=round(M / (ms100 * 1e-3), 1),
                                       steps=args.steps)
        del m100
        for p in moe.parameters():
            p.grad = None
        x_dev.grad = None
        torch.cuda.empty_cache()
    except Exception as err:   # a record, not the measurement: never take the line down
        out["save_percent_100"] = {"unavailable": repr(err)[:200]}
    ref_dir = os.path.join(ROOT, "baseline", "_ref", "momoe")
    if not os.path.isdir(ref_dir):
        out["reference_triton"] = {"unavailable": "baseline/_ref is not installed"}
        return out
    try:
        res = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference-triton", "--steps",
                              str(args.steps), "--warmup", "12", "--save-percent", str(args.save_percent)],
                             capture_output=True, text=True, timeout=600, cwd=ROOT)
        lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
        d = json.loads(lines[-1]) if lines else {"unavailable": (res.stderr or "no output")[-300:]}
        if "ms_per_step" in d:
            out["reference_triton"] = dict(ms_per_step=round(d["ms_per_step"], 4), tokens_per_s=round(d["value"], 1),
                                           save_percent=args.save_percent, steps=d.get("steps"),
                                           what="unmodified reference package (baseline/_ref), its Triton kernels "
                                                "autotuned during 12 warm-up steps, same GPU, layer and protocol")
        else:
            out["reference_triton"] = {"unavailable": str(d.get("unavailable"))[:300]}
    except Exception as err:
        out["reference_triton"] = {"unavailable": repr(err)[:200]}
    return out


INFER = dict(D=2048, H=768, N=128, K=8, tokens=(1, 8, 64, 256, 1024, 4096, 16384), w_std=0.02)


def run_inference(args, dev):
    """--workload inference: forward-only latency of the 30B-A3B-class layer (D2048 H768 N128 K8) through the
    `MoMoE` module for batches of 1..16384 tokens, router logits N(0,1) + expert bias N(0,0.5).  Each batch is timed
    eagerly (host launches included) and as a replayed CUDA graph of the same calls; the HBM figure is the bytes
    every touched expert's weights occupy (3*D*H*2 per expert) plus the token rows moved, over the graph time."""
    import momoe
    from momoe import ops
    c = INFER
    D, H, N, K = c["D"], c["H"], c["N"], c["K"]
    peaks = measured_peaks()
    Wg, W1, W2 = make_weights(1234, N, D, H, dev, N, c["w_std"])
    layer = momoe.MoMoE(D, H, N, K, save_percent=0, Wl1_ND2H=W1, Wl2_NHD=W2)
    del W1, W2
    gen = torch.Generator(device=dev).manual_seed(5)
    e_bias = 0.5 * torch.randn(N, generator=gen, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # larger than L2
    points = []
    for T in ((args.infer_tokens,) if args.infer_tokens > 0 else c["tokens"]):
        x = torch.randn(1, T, D, generator=gen, device=dev).bfloat16()
        logits = (torch.randn(T, N, generator=gen, device=dev) + e_bias).bfloat16()
        zeros = torch.zeros(N, device=dev)

        def fwd(inference=True):
            with torch.no_grad():
                idx, w, _ = ops.route_topk(logits, zeros, K, 0, dense=False)
                plan = ops.RoutingPlan.from_topk(idx, w, N, D, H, 0)
                y, _, _ = ops.experts_forward(plan, x, layer.Wl1_ND2H.detach(), layer.Wl2_NHD.detach(),
                                              inference=inference)
            return y, plan.sizes

        for _ in range(3):
            y, sizes = fwd()
        torch.cuda.synchronize()
        ops.check_status()
        touched = int((sizes > 0).sum())
        l0 = ops.LAUNCHES
        fwd()
        launches = ops.LAUNCHES - l0
        if args.infer_tokens > 0:
            for _ in range(3):
                flush.zero_()
                fwd()
            torch.cuda.synchronize()
            points.append(dict(tokens=T, experts_touched=touched, launches=launches))
            continue
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fwd()

        def timed(fn):
            ts = []
            for _ in range(max(args.steps, 5)):
                flush.zero_()
                e0 = torch.cuda.Event(enable_timing=True)
                e1 = torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            return statistics.median(ts)

        t_eager = timed(fwd)
        t_graph = timed(graph.replay)
        ops.check_status()
        streaming = T * K <= ops.DECODE_MAX_AVG_ROWS * N
        t_tile = None
        if T * K <= 128 * N:
            # the same batch forced through the other kernel family, for the cross-over
            keep = ops.DECODE_MAX_AVG_ROWS
            ops.DECODE_MAX_AVG_ROWS = 0 if streaming else 128
            fwd()
            graph2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph2):
                fwd()
            t_other = timed(graph2.replay)
            del graph2
            ops.DECODE_MAX_AVG_ROWS = keep
            if not streaming:
                t_tile, t_graph_streaming = t_graph, t_other
            else:
                t_tile, t_graph_streaming = t_other, t_graph
        nbytes = touched * 3 * D * H * 2 + T * D * 2 * 2 + T * K * (2 * D + 2 * H) * 2
        flops = 6.0 * T * K * D * H
        points.append(dict(tokens=T, experts_touched=touched, launches=launches,
                           kernels="weight-streaming" if streaming else "256-row tiles",
                           ms_eager=round(t_eager, 4), ms_graph=round(t_graph, 4),
                           ms_graph_256_row_tiles=round(t_tile, 4) if t_tile is not None else None,
                           ms_graph_weight_streaming=round(t_graph_streaming, 4) if t_tile is not None else None, hbm_gbs=round(nbytes / t_graph / 1e6, 1),
                           hbm_frac=round(nbytes / t_graph / 1e6 / peaks["hbm"], 3),
                           tflops=round(flops / t_graph / 1e9, 1),
                           tokens_per_s=round(T / t_graph * 1e3, 1)))
        del graph
    print(json.dumps(dict(metric="MoE layer forward latency per token batch (D2048 H768 N128 K8 bf16)", unit="ms",
                          higher_is_better=False, n_gpus=1, dtype="bf16", data="synthetic",
                          config=dict(workload="inference forward, token batches 1..16384, L2 flushed between "
                                               "iterations; not the headline workload"),
                          peak_hbm_gbs=peaks["hbm"], peak_source=peaks["source"], points=points)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--save-percent", type=float, default=0.0)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference-triton"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-memory leg (profiling runs)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the untimed extra records of the 1-GPU line (save_percent 100, reference package)")
    ap.add_argument("--experts", type=int, default=CFG["N"], help="reduced case for profiler captures")
    ap.add_argument("--tokens", type=int, default=CFG["B"] * CFG["S"], help="reduced case for profiler captures")
    ap.add_argument("--forward-only", action="store_true",
                    help="time forward passes only (per-call breakdown of the forward transfers; not the headline metric)")
    ap.add_argument("--infer-tokens", type=int, default=0,
                    help="inference workload: one batch size only, eager calls only (profiler captures)")
    ap.add_argument("--workload", default="headline", choices=["headline", "large_ep", "inference"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.impl == "reference-triton":
        if rank == 0:
            run_triton_reference(args)
        return

    import torch.distributed as dist
    import __graft_entry__
    if rank == 0:
        __graft_entry__.build()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # the only NCCL collectives here are barriers and the reduction of a timing scalar: no in-switch reduction
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
        dist.barrier()
    import momoe
    from momoe import ops

    if args.workload == "inference":
        if rank == 0:
            run_inference(args, dev)
        return

    ep_parity = ep_parity_preflight(rank, world, dev) if world > 1 else None

    c = dict(CFG if args.workload == "headline" else LARGE_EP)
    reduced = args.workload == "headline" and (args.experts != c["N"] or args.tokens != c["B"] * c["S"])
    if reduced:
        c.update(N=args.experts, B=1, S=args.tokens)
    D, H, N, K, Ks = c["D"], c["H"], c["N"], c["K"], c["Ks"]
    M = c["B"] * c["S"]
    if world > 1:
        from momoe import ep
        Wg, W1, W2 = make_weights(1234, N // world, D, H, dev, N, c["w_std"])   # this rank's expert block
        moe = ep.ExpertParallelMoE(D, H, N, K, Ks, save_percent=args.save_percent, Wg_DN=Wg, Wl1_ND2H=W1,
                                   Wl2_NHD=W2, group=dist.group.WORLD)
        parallelism = "ep%d" % world
    else:
        Wg, W1, W2 = make_weights(1234, N, D, H, dev, N, c["w_std"])
        moe = momoe.MoE(D, H, N, K, Ks, save_percent=args.save_percent, Wg_DN=Wg, Wl1_ND2H=W1, Wl2_NHD=W2)
        parallelism = "single"
    del W1, W2
    gen = torch.Generator(device="cpu").manual_seed(100 + rank)
    x_host = torch.randn(c["B"], c["S"], D, generator=gen).bfloat16().pin_memory()
    g_dev = torch.randn(c["B"], c["S"], D, generator=gen).bfloat16().to(dev)
    x_dev = x_host.to(dev).requires_grad_(True)
    if c["zipf"]:
        b = zipf_biases(x_dev.detach().reshape(M, D), Wg, N, K)
        if world > 1:
            dist.broadcast(b, 0)      # every rank routes with rank 0's bias profile
        with torch.no_grad():
            moe.biases_N.copy_(b)

    def zero_grads():
        for p in moe.parameters():
            p.grad = None
        x_dev.grad = None

    def step_resident():
        if args.forward_only:
            with torch.no_grad():
                moe(x_dev)
            return
        zero_grads()
        y = moe(x_dev)
        y.backward(g_dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ------------------------------------------------------------------ device-resident throughput
    for _ in range(args.warmup):
        step_resident()
    barrier()
    ops.check_status(dev)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ops.KERNEL_EVENTS = []
    launches0 = ops.LAUNCHES
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step_resident()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop() if sampler else None
    launches = (ops.LAUNCHES - launches0) // args.steps
    events, ops.KERNEL_EVENTS = ops.KERNEL_EVENTS, None
    ops.check_status(dev)
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    tokens_per_step = M * world
    value = tokens_per_step / (ms * 1e-3)

    # per-kernel device time from the events recorded inside the timed region
    per = {}
    for name, a, b in events:
        per.setdefault(name, []).append(a.elapsed_time(b))
    msum = M * K
    unit_flops = float(msum) * D * H
    # algorithmic flops of one launch, in units of Msum*D*H (up/gate 4, down 2, dgrad-2 2, wgrads 2 and 4, dgrad-1 4)
    flops = {"momoe_up_swiglu": 4, "momoe_up_swiglu (recompute)": 4, "momoe_down_scale": 2,
             "momoe_dgrad2_swiglu_bwd": 2, "momoe_wgrad (W2)": 2, "momoe_wgrad (W1)": 4, "momoe_dgrad1": 4}
    # DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum, MB) from an ncu capture of the reduced case
    # (--experts 32 --tokens 4096); traffic grows in proportion to experts (weights) and tokens (activations), so it is
    # scaled to this run's experts and tokens.
    ncu_mb_small = {"momoe_up_swiglu": 474, "momoe_up_swiglu (recompute)": 535, "momoe_down_scale": 316,
                    "momoe_dgrad2_swiglu_bwd": 611, "momoe_wgrad (W2)": 319, "momoe_wgrad (W1)": 519,
                    "momoe_dgrad1": 534}
    traffic_scale = 0.5 * (N / 32.0 + M / 4096.0)
    peaks = measured_peaks()
    kernels = []
    for name, times in per.items():
        avg = sum(times) / len(times)
        k = dict(name=name, launches_per_step=len(times) // args.steps, ms=round(avg, 4))
        if name in flops:
            # a call that a step makes in several launches (the expert-parallel forward pass works in two halves)
            # is rated on the time of all of them together
            k["tflops"] = round(flops[name] * unit_flops / (avg * k["launches_per_step"] * 1e-3) / 1e12, 1)
        kernels.append(k)
    kernels.sort(key=lambda k: -k["ms"] * k["launches_per_step"])
    gemms = [k for k in kernels if "tflops" in k]
    roofline = None
    if gemms:
        top = gemms[0]
        roofline = dict(bound="tensor", kernel="grouped_gemm_kernel / " + top["name"], achieved=top["tflops"],
                        peak=peaks["tflops"], unit="TFLOP/s", frac=round(top["tflops"] / peaks["tflops"], 4),
                        traffic=(ncu_mb_small[top["name"]] * 1e6 * traffic_scale / top["launches_per_step"])
                        if args.workload == "headline" else None,
                        peak_source=peaks["source"],
                        traffic_note="dram__bytes_read+write per launch from an ncu capture of a 1/4-size case, scaled",
                        flops_per_launch=flops[top["name"]] * unit_flops / top["launches_per_step"],
                        ms_per_launch=top["ms"])
    layer_flops = (18.0 * K * D * H + 6.0 * D * N) * M   # algorithmic fwd+bwd flops per rank and step
    layer_tflops = layer_flops / (ms * 1e-3) / 1e12

    # ------------------------------------------------------------------ end to end from pinned host memory
    # Every step's input travels from pinned host memory to the device and every step's loss is read back, all inside
    # the timed region.  Both are pipelined the way a training loop with a data loader and asynchronous loss logging
    # is: inputs are copied ahead on a copy stream into a ring of DEPTH device buffers, and the host waits for the loss
    # of step i-(DEPTH-1) only after it has queued step i, so neither a slow copy nor a late host leaves the device
    # idle (with several ranks a late rank would make every other rank wait at the hand-shakes).
    DEPTH = 3
    copy_stream = torch.cuda.Stream(device=dev)
    xb = [x_dev] + [x_host.to(dev).requires_grad_(True) for _ in range(DEPTH - 1)]
    ready = [torch.cuda.Event() for _ in range(DEPTH)]
    consumed = [torch.cuda.Event() for _ in range(DEPTH)]

    def prefetch(i):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[i % DEPTH])     # the step that last used this buffer has finished
            with torch.no_grad():
                xb[i % DEPTH].copy_(x_host, non_blocking=True)
            ready[i % DEPTH].record(copy_stream)

    loss_host = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(DEPTH)]
    loss_ready = [torch.cuda.Event() for _ in range(DEPTH)]
    losses = []

    def step_e2e(i):
        cur = xb[i % DEPTH]
        torch.cuda.current_stream().wait_event(ready[i % DEPTH])
        for p in moe.parameters():
            p.grad = None
        cur.grad = None
        y = moe(cur)
        # Several ranks: the buffer of the step before this one is refilled now, for step i + DEPTH - 1, so that the
        # copy runs beside the backward pass's GEMMs; a host-to-device copy that runs beside the short, latency-bound
        # kernels and hand-shakes at the beginning of an expert-parallel forward pass made each of them take about
        # twice as long.  One GPU has no hand-shakes: its copy is queued at the end of the step (below) and runs beside
        # the router and the gather of the next one, where it costs the power-capped GEMMs nothing.
        if world > 1 and i >= 1:
            prefetch(i - 1 + DEPTH)
        # mean-square loss: one reduction over y (fp32 accumulation) forward, one elementwise pass backward
        loss = torch.linalg.vector_norm(y, dtype=torch.float32).square() / y.numel()
        loss.backward()
        consumed[i % DEPTH].record(torch.cuda.current_stream())
        loss_host[i % DEPTH].copy_(loss.detach().reshape(1), non_blocking=True)   # device -> host read of the result
        loss_ready[i % DEPTH].record(torch.cuda.current_stream())
        if world == 1:
            prefetch(i + DEPTH)

    def read_loss(i):
        loss_ready[i % DEPTH].synchronize()
        losses.append(float(loss_host[i % DEPTH][0]))

    ms_e2e = float("nan")
    if not args.no_e2e and not args.forward_only:
        n_pre = 3
        for i in range(DEPTH):
            prefetch(i)
        for i in range(n_pre):
            step_e2e(i)
            read_loss(i)
        barrier()
        e0.record()
        first, last = n_pre, n_pre + args.steps - 1
        for i in range(first, last + 1):
            step_e2e(i)
            if i - (DEPTH - 1) >= first:
                read_loss(i - (DEPTH - 1))
        for i in range(max(first, last - (DEPTH - 1) + 1), last + 1):
            read_loss(i)
        e1.record()
        barrier()
        ms_e2e = e0.elapsed_time(e1) / args.steps
        assert len(losses) == n_pre + args.steps and all(v == v for v in losses), "a step's loss was not read back"
    t = torch.tensor([ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_e2e = float(t.item())
    ops.check_status(dev)

    extras = {}
    if rank == 0 and world == 1 and args.workload == "headline" and not reduced and not args.forward_only \
            and not args.no_extras:
        extras = extra_records(args, dev, moe, x_dev, g_dev, M)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and args.workload == "headline":
        cb = cpu_sample(6, 1)
        cpu_baseline = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}

    if rank == 0 and args.forward_only:
        # diagnostic output only: forward passes, per-call device times
        print(json.dumps(dict(metric="MoE layer forward-only pass (diagnostic, not the headline metric)", unit="ms",
                              n_gpus=world, steps=args.steps, ms_per_forward=ms, higher_is_better=False,
                              config=dict(workload="forward only, %d tokens per GPU" % M, parallelism=parallelism),
                              kernels=kernels)), flush=True)
    elif rank == 0:
        line = dict(
            metric=METRIC if args.workload == "headline" else
            "MoE layer fwd+bwd tokens/sec (D%d H%d N%d K%d bf16)" % (D, H, N, K),
            value=value, unit="tokens/s", n_gpus=world, steps=args.steps, warmup=args.warmup,
            ms_per_step=ms, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
            config=dict(workload=("REDUCED profiling case N%d tokens %d (not the headline workload)" % (N, M)) if reduced
                        else ("large expert-parallel layer: D7168 H2048 N256 K8, 65536 tokens per GPU, Zipf(1.1) router "
                              "bias (busiest expert 8x mean), fwd+bwd (not the headline workload)")
                        if args.workload == "large_ep"
                        else "cfg2 headline layer: D2048 H1024 N128 K8, B8 S2048 (16384 tokens) per GPU, fwd+bwd",
                        tokens_per_gpu=M, save_percent=args.save_percent, parallelism=parallelism,
                        l2="inputs larger than L2 (weights 1.6 GB, activations > 0.5 GB per step)"),
            e2e=dict(value=tokens_per_step / (ms_e2e * 1e-3), unit="tokens/s", ms_per_step=ms_e2e,
                     h2d_bytes_per_step=x_host.numel() * 2, d2h_bytes_per_step=4),
            gpu_launches=launches, clocks=clocks, roofline=roofline, cpu_baseline=cpu_baseline,
            layer_tflops=round(layer_tflops, 1), layer_frac_of_peak=round(layer_tflops / peaks["tflops"], 4),
            kernels=kernels)
        line.update(extras)
        if ep_parity is not None:
            line["ep_parity"] = ep_parity
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
