#!/usr/bin/env python
"""Benchmark of the conv-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--repeats R] [--impl ours|reference] [--no-decode] [--no-sweep] [--no-headmix] [--no-keep-ktilde]

One "step" = conv-attention forward + backward (D prep, dQ/dTheta, dK/dV, partial reduction,
and for N > 1 the all-reduce of dTheta) on the bf16 training configuration
B=4, H=16, N=4096, d=64, theta (6,11), causal -- PER GPU (weak scaling: every rank holds its own
batch of 4; the only collective is the 4 KB dTheta all-reduce over NCCL).  `value` is the
whole-job FlashAttention-convention throughput 14*d*E / t (E = causal score elements); the
conv's own FLOPs are reported separately and never added to the numerator.

The timed loop of K steps is repeated R times (default 5); `ms_per_step` / `value` are the MEDIAN
loop, `ms_per_step_min` the fastest, and `ms_x_mhz` = ms_per_step x the median SM clock sampled
during the loops, so that runs at different power-capped clocks can be compared.

Also reported in the same JSON line: `e2e` (same step with host->device copies of Q,K,V,dO from
pinned memory and the device->host read of dTheta inside the timed region), `roofline` for the
dominant kernel with the whole step's fraction of peak beside it, `cpu_baseline` (the reference's
PyTorch path on the host cores, bounded sample), `decode` (fwd_inference over a 32768-long KV
cache, HBM GB/s), `sweep` (the d = 128 scaling configuration B=8, H=32, theta (6,11) at
N = 1024 ... 65536 as ONE fixed problem sharded by (batch, head) over the ranks with the dTheta
all-reduce: strong scaling), clocks sampled during the timed region.

`--impl reference` times the reference's CPU path (the oracle port, all host threads) on a
bounded sample of the same workload and prints the same kind of line with "impl": "reference".
"""
import argparse
import ctypes
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "flash-multi-token-attention_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

CFG = dict(B=4, H=16, N=4096, d=64, cq=6, ck=11)                 # training configuration (per GPU)
SWEEP = dict(B=8, H=32, d=128, cq=6, ck=11, Ns=(1024, 4096, 16384, 65536))      # scaling configuration (whole job)
DEC = dict(B=32, H=32, d=128, Nk=32768, q_len=6, cq=6, ck=11, k_splits=4)   # decode configuration (4 CTAs/SM x 148 SMs: 4096 CTAs = 6.9 waves)
METRIC = "conv-attn fwd+bwd TFLOP/s"


def flops_attn(B, H, N, d):
    E = B * H * N * (N + 1) / 2
    return 14.0 * d * E, E


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            j = json.load(f)
        return dict(tflops=j.get("bf16_tflops"), tflops_sustained=j.get("bf16_tflops_sustained"),
                    hbm=j.get("hbm_gbs"), source="measured")
    return dict(tflops=1590.0, tflops_sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except Exception:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return None
        return dict(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))


def _reference_module():
    """The reference's own ConvAttention class, loaded by file path from the checkout that BASELINE.json
    names -- when that checkout is present on this machine (it is not on a bare GPU box)."""
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            ref_root = json.load(f).get("reference_path")
        path = os.path.join(ref_root, "flash_multi_token_attention", "conv_attn", "conv_attention_pytorch.py")
        if not os.path.exists(path):
            return None
        import importlib.util
        spec = importlib.util.spec_from_file_location("_ref_conv_attention_pytorch", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod.ConvAttention
    except Exception:
        return None


def cpu_reference_sample(steps=1, warmup=0):
    """The reference's CPU path (dense scores, conv2d, softmax, autograd backward) on ONE (batch, head)
    slice of the training configuration, all host threads: the reference's own module when its checkout
    is on this machine (kind "reference"), else the oracle's restatement of it (kind "port")."""
    from oracle import conv_attn_oracle as orc
    N, d, cq, ck = CFG["N"], CFG["d"], CFG["cq"], CFG["ck"]
    Q, K, V, dO, th = orc.make_inputs(1, 1, N, d, cq, ck, seed=0, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    RefCls = _reference_module()
    kind = "reference" if RefCls is not None else "port"
    if RefCls is not None:
        mod = RefCls(1, cq, ck)
        with torch.no_grad():
            mod.conv_weight.copy_(th)

        def run():
            q, k, v = (t.clone().requires_grad_(True) for t in (Q, K, V))
            mod.conv_weight.grad = None
            out = mod(q, k, v, causal=True, softmax_scale=scale)
            (out[0] if isinstance(out, tuple) else out).backward(dO)
    else:
        def run():
            orc.conv_attn_bwd_autograd(Q, K, V, th, dO, scale, True)   # forward + backward
    ts = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        run()
        if i >= warmup:
            ts.append(time.perf_counter() - t0)
    t = sum(ts) / len(ts)
    fl, _ = flops_attn(1, 1, N, d)
    return dict(value=fl / t / 1e12, unit="TFLOP/s", cores=torch.get_num_threads(), kind=kind,
                sample="1 of %d (batch, head) slices of the workload, fwd+bwd, fp32, %d run(s), %.2f s each; "
                       "slices are independent so the full job is %dx this" % (CFG["B"] * CFG["H"], len(ts), t,
                                                                              CFG["B"] * CFG["H"]),
                host_cpus=os.cpu_count(), seconds_per_slice=t)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    steps = max(1, min(args.steps, 5))
    cb = cpu_reference_sample(steps=steps, warmup=1 if args.warmup > 0 else 0)
    line = dict(metric=METRIC, value=cb["value"], unit="TFLOP/s", n_gpus=args.gpus, steps=steps,
                warmup=1 if args.warmup > 0 else 0, ms_per_step=cb["seconds_per_slice"] * 1e3,
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic",
                impl="reference",
                config=dict(workload="train fwd+bwd B=4,H=16,N=4096,d=64,theta(6,11),causal; "
                                     "each step = one (b,h) slice of it on the host cores", **CFG),
                cpu_baseline=cb,
                e2e=dict(value=cb["value"], unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0)
    print(json.dumps(line), flush=True)


def run_reference_gpu(args):
    """Same-box GPU baseline: the reference's own CUDA extension, rebuilt for sm_100 by
    oracle/build_ref_cuda.py (square filters only), next to this library at the shapes of the reference's
    published benchmark (B=1, H=8, d=64, 7x7 filter, bf16, causal; N = 512 ... 4096).  Context, not the
    headline: prints one JSON line with the milliseconds of both, forward and backward."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    so = os.path.join(ROOT, "oracle", "_ref", "fmta_reference_cuda_sm100.so")
    if not os.path.exists(so) or not torch.cuda.is_available():
        print(json.dumps(dict(impl="reference-gpu", unavailable="oracle/_ref/fmta_reference_cuda_sm100.so has not been built "
                              "(python oracle/build_ref_cuda.py needs the reference checkout) or no GPU")), flush=True)
        return
    import importlib.util
    spec = importlib.util.spec_from_file_location("fmta_reference_cuda_sm100", so)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    import fmta_b200 as F
    dev = torch.device("cuda", 0)
    B, H, d, cq, ck = 1, 8, 64, 7, 7
    scale, pq, pk = 1.0 / math.sqrt(d), cq - 1, (ck - 1) // 2
    iters = max(3, min(args.steps, 20))

    def ms_of(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    def graph_ms_of(fn):
        """The same call captured once into a CUDA graph and replayed (host launch overhead removed)."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            keep = fn()   # noqa: F841  (outputs stay alive with the graph)
        return ms_of(graph.replay)

    points = []
    for N in (512, 1024, 2048, 4096):
        g = torch.Generator(device=dev).manual_seed(N)
        q, k, v, do = (torch.randn(B, H, N, d, device=dev, generator=g).to(torch.bfloat16) for _ in range(4))
        th = torch.randn(H, cq, ck, device=dev, generator=g) * 0.02
        th[:, cq - 1, ck // 2] += 1.0
        thb = th.to(torch.bfloat16)
        # reference: forward(Q,K,V,conv_kernel,scale,pad_q,pad_k,causal); backward takes D and M + log L in bf16
        O_r, M_r, L_r = ref.forward(q, k, v, thb, scale, pq, pk, True)
        torch.cuda.synchronize()
        lse_r = (M_r + torch.log(L_r)).to(torch.bfloat16)
        D_r = (do.float() * O_r).sum(-1).to(torch.bfloat16)
        O, M, L, LSE = F.forward(q, k, v, th, scale, pq, pk, True, return_lse=True)
        Dv = F.rowdot(do, O)
        pt = dict(N=N, max_abs_O_vs_reference=float((O - O_r).abs().max()),
                  ref_fwd_ms=ms_of(lambda: ref.forward(q, k, v, thb, scale, pq, pk, True)),
                  fwd_ms=ms_of(lambda: F.forward(q, k, v, th, scale, pq, pk, True)))

        def ref_bwd():
            ref.dq_backward(q, k, v, do, D_r, lse_r, thb, scale, pq, pk, True)
            ref.dkdv_backward(q, k, v, do, D_r, lse_r, thb, scale, pq, pk, True)
        pt["ref_bwd_ms"] = ms_of(ref_bwd)
        pt["bwd_ms"] = ms_of(lambda: F.backward(q, k, v, do, Dv, LSE, th, scale, pq, pk, True))
        pt["fwd_graph_ms"] = graph_ms_of(lambda: F.forward(q, k, v, th, scale, pq, pk, True))
        pt["bwd_graph_ms"] = graph_ms_of(lambda: F.backward(q, k, v, do, Dv, LSE, th, scale, pq, pk, True))
        points.append(pt)
    F.check_device_status(dev)
    print(json.dumps(dict(impl="reference-gpu", metric="ms per call, conv attention 7x7, B=1,H=8,d=64, bf16, causal",
                          build="reference conv_attn extension compiled with -gencode=arch=compute_100,code=sm_100 "
                                "(its own sources and flags otherwise)", iters=iters, points=points)), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"])
    ap.add_argument("--repeats", type=int, default=5, help="how often the timed loop of --steps steps is repeated (median reported)")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-context-parallel", action="store_true")
    ap.add_argument("--cp-shape", default=None, help="B,H,N,d of the sequence-sharded problem (default 1,4,65536,128)")
    ap.add_argument("--no-headmix", action="store_true")
    ap.add_argument("--no-keep-ktilde", action="store_true",
                    help="let forward and backward each build the stacked key operand (the reference-shaped pair of calls)")
    ap.add_argument("--headmix-shape", default=None, help="B,H,N,d: time only this dense head-mix shape (profiling captures)")
    ap.add_argument("--convmix-shape", default=None, help="B,H,N,d: time only conv (6,11) + mix in groups of 4 at this shape (profiling captures)")
    ap.add_argument("--sweep-max-n", type=int, default=65536)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--small", action="store_true", help="tiny shapes (profiling / debugging)")
    ap.add_argument("--train-shape", default=None, help="B,H,N,d of the training step (profiling captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.impl == "reference-gpu":
        return run_reference_gpu(args)
    args.warmup = max(args.warmup, 3)

    import torch.distributed as dist
    import fmta_b200 as F
    from fmta_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    cfg = dict(CFG)
    dec = dict(DEC)
    if args.small:
        cfg.update(B=1, H=4, N=2048)
        dec.update(B=4, H=32, Nk=16384)   # 0.5 GB of K/V: larger than L2, small enough to profile
    if args.train_shape:
        tb, th_, tn, td = (int(x) for x in args.train_shape.split(","))
        cfg.update(B=tb, H=th_, N=tn, d=td)
    B, H, N, d, cq, ck = (cfg[k] for k in ("B", "H", "N", "d", "cq", "ck"))
    scale = 1.0 / math.sqrt(d)
    pq, pk = cq - 1, (ck - 1) // 2

    g = torch.Generator().manual_seed(1234 + rank)
    host = [torch.randn(B, H, N, d, generator=g).to(torch.bfloat16).pin_memory() for _ in range(4)]
    th = torch.randn(H, cq, ck, generator=torch.Generator().manual_seed(7)) * 0.02
    th[:, cq - 1, ck // 2] += 1.0
    th = th.to(dev)
    q, k, v, do = (t.to(dev) for t in host)
    dth_host = torch.empty(H, cq, ck, dtype=torch.float32).pin_memory()
    stream = torch.cuda.current_stream()
    # the dominant kernel of the step is timed alone through the library's profiling hook
    # (cudaEventRecord around that one launch, on the launch stream)
    KERNELS = {1: "fwd_tc_kernel", 2: "fwd_band_kernel", 3: "bwd_dq_tc_kernel", 4: "bwd_dkdv_tc_kernel",
               5: "bwd_dq_kernel", 6: "bwd_dkdv_kernel", 8: "bwd_band_kernel", 9: "ktilde_window_kernel",
               10: "dk_post_mma_kernel"}
    DOMINANT = 4
    kern_ev = []   # (start, end) events around the dominant kernel, per step

    kt = None if args.no_keep_ktilde else F.ktilde_buffer(q, th)   # bf16 [B,H,cq,N,d], allocated once

    def step(q, k, v, do, record=False):
        if record:
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record(stream); e1.record(stream)       # creates the underlying CUDA events
            _lib.lib.fmta_profile_kernel(DOMINANT, ctypes.c_void_p(e0.cuda_event), ctypes.c_void_p(e1.cuda_event))
            kern_ev.append((e0, e1))
        # the forward leaves its stacked key operand in `kt`; the backward reads it instead of rebuilding it
        O, M, L, LSE = F.forward(q, k, v, th, scale, pq, pk, True, return_lse=True, ktilde=kt)
        D = F.rowdot(do, O)
        dQ, dK, dV, dTh = F.backward(q, k, v, do, D, LSE, th, scale, pq, pk, True, ktilde=kt)
        if record:
            _lib.lib.fmta_profile_kernel(0, None, None)
        if world > 1:
            dist.all_reduce(dTh)
        return O, dQ, dK, dV, dTh

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # ---- device-resident throughput ----
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    for _ in range(args.warmup):
        step(q, k, v, do)
    # keep the GPU under load for about 0.3 s more, so that nvidia-smi samples it before the timed
    # region; every rank must run the SAME number of steps (each holds an all-reduce), so rank 0
    # measures one step and the count is broadcast
    torch.cuda.synchronize()
    t_w = time.perf_counter()
    step(q, k, v, do)
    torch.cuda.synchronize()
    n_extra = torch.tensor([min(400, int(0.3 / max(time.perf_counter() - t_w, 1e-4)) + 1)], device=dev)
    if world > 1:
        dist.broadcast(n_extra, src=0)
    for _ in range(int(n_extra.item())):
        step(q, k, v, do)
    loops = [timed(lambda: step(q, k, v, do, record=True), args.steps) / args.steps for _ in range(max(1, args.repeats))]
    F.check_device_status(dev)             # raises if a bounded wait inside a tensor-core kernel ran out
    ms_step = statistics.median(loops)
    fl, E = flops_attn(B, H, N, d)
    value = world * fl / (ms_step * 1e-3) / 1e12

    # ---- end to end: host buffers in, dTheta out ----
    # Every step copies its four inputs from pinned host memory and reads dTheta back.  The copy of
    # step i+1 runs on a second stream into the other of two device buffer sets while step i
    # computes (the usual input prefetch); the first copy of a timed run is not overlapped.
    copy_stream = torch.cuda.Stream(device=dev)
    dev_bufs = [[torch.empty_like(t, device=dev) for t in host] for _ in range(2)]
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def prefetch(slot):
        copy_stream.wait_event(consumed[slot])          # the step that last read this buffer set is done
        with torch.cuda.stream(copy_stream):
            for dst, src in zip(dev_bufs[slot], host):
                dst.copy_(src, non_blocking=True)
            copied[slot].record(copy_stream)

    def e2e_run(steps):
        for ev in consumed:
            ev.record(stream)
        prefetch(0)
        for i in range(steps):
            slot = i & 1
            if i + 1 < steps:
                prefetch(slot ^ 1)
            stream.wait_event(copied[slot])
            out = step(*dev_bufs[slot])
            consumed[slot].record(stream)
            dth_host.copy_(out[4], non_blocking=True)

    e2e_run(2)
    e2e_loops = []
    for _ in range(max(1, args.repeats)):
        barrier()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        e2e_run(args.steps)
        e1.record(stream)
        barrier()
        t_ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([t_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_ms = float(t.item())
        e2e_loops.append(t_ms / args.steps)
    clocks = sampler.stop() if sampler else None
    ms_e2e = statistics.median(e2e_loops)
    h2d = sum(t.numel() * t.element_size() for t in host)
    e2e = dict(value=world * fl / (ms_e2e * 1e-3) / 1e12, unit="TFLOP/s", h2d_bytes_per_step=h2d,
               d2h_bytes_per_step=dth_host.numel() * 4, ms_per_step=ms_e2e, ms_per_step_min=min(e2e_loops),
               note="inputs of step i+1 are copied on a second stream while step i computes")

    # ---- roofline of the dominant kernel: bwd_dkdv_tc_kernel (dK~/dV on tcgen05) ----
    # The step's algorithmic work is 14*d*E (FlashAttention convention: forward S and PV = 4*d*E, backward
    # S, dP, dV, dK, dQ = 10*d*E).  Both backward kernels recompute S and dP, so each is credited half of
    # those two contractions: forward 4*d*E, dQ kernel 2*d*E + 2*d*E = 4*d*E, dK/dV kernel 4*d*E + 2*d*E =
    # 6*d*E -- the three shares add up to the step's 14*d*E.  The stacked filter taps make the dK/dV
    # kernel EXECUTE 2*d*(2*cq + 2) per entry, reported beside it.  `step_frac` is the whole step against
    # the same peak.
    peaks = measured_peaks()
    kms = statistics.mean(a_.elapsed_time(b_) for a_, b_ in kern_ev) if kern_ev else None
    roof = None
    if kms:
        ach = 6.0 * d * E / (kms * 1e-3) / 1e12
        exe = 2.0 * d * (2 * cq + 2) * E / (kms * 1e-3) / 1e12
        # DRAM bytes per launch from the committed ncu capture at B=2,H=16,N=4096 (152.2 MB read + 88.4 MB
        # written; summary under profiles/), scaled by the (batch, head)
        # units; only quoted for that sequence length and head dimension
        traffic = (152.20e6 + 88.37e6) * (B * H) / 32.0 if (N == 4096 and d == 64 and cq == 6) else None
        roof = dict(bound="tensor", kernel=KERNELS[DOMINANT], achieved=ach, peak=peaks["tflops_sustained"],
                    unit="TFLOP/s", frac=ach / peaks["tflops_sustained"], peak_source=peaks["source"] + " (sustained)",
                    traffic=traffic, traffic_unit="bytes per launch (ncu capture of a smaller case, scaled)",
                    ms_per_launch=kms, executed_tflops=exe,
                    executed_frac=exe / peaks["tflops_sustained"],
                    step_tflops=fl / (ms_step * 1e-3) / 1e12,
                    step_frac=fl / (ms_step * 1e-3) / 1e12 / peaks["tflops_sustained"],
                    step_executed_tflops=(2.0 * d * (cq + 1) + 2.0 * d * (2 * cq + 2) + 2.0 * d * (2 * cq + 2)) * E / (ms_step * 1e-3) / 1e12,
                    note="achieved counts the kernel's share (6*d*E) of the step's 14*d*E algorithmic FLOPs; it "
                         "executes 2*d*(2*c_q+2)*E (stacked filter taps on the tensor cores) = executed_tflops; "
                         "step_frac = 14*d*E / ms_per_step / peak (per GPU)")

    sm_mhz = clocks["sm_mhz"] if clocks else None
    line = dict(metric=METRIC, value=value, unit="TFLOP/s", n_gpus=world, steps=args.steps, warmup=args.warmup,
                repeats=len(loops), ms_per_step=ms_step, ms_per_step_min=min(loops),
                ms_x_mhz=(ms_step * sm_mhz) if sm_mhz else None, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
                data="synthetic",
                config=dict(workload="train fwd+bwd bf16 B=%d(per GPU),H=%d,N=%d,d=%d,theta(%d,%d),causal" % (B, H, N, d, cq, ck),
                            global_batch=B * world, parallelism="batch x head sharding, dTheta all-reduce" if world > 1 else "single GPU",
                            l2="inputs+outputs per step (%.0f MB) exceed the 126 MB L2" % ((4 * 2 + 4 * 4) * B * H * N * d / 1e6),
                            stacked_keys="built once per step (forward), kept for the backward" if kt is not None else "built by forward and by backward",
                            flops_attn_gflop=fl / 1e9, flops_conv_gflop=8 * cq * ck * E / 1e9),
                # kernels of this library per step: forward = stacked-key pre-pass, fwd_tc, fwd_band;
                # rowdot; backward = pre-pass (not when the forward's operand is kept), dq_tc, dkdv_tc, Toeplitz tiles + dKt adjoint, bwd_band,
                # partial reduction
                e2e=e2e, roofline=roof, clocks=clocks, gpu_launches=(11 if kt is None else 10) * args.steps * len(loops))

    # ---- decode (HBM-bound), rank-local, reported beside the headline ----
    if not args.no_decode:
        try:
            line["decode"] = bench_decode(F, dev, dec, peaks, world, timed)
        except torch.OutOfMemoryError as e:   # pragma: no cover
            line["decode"] = dict(error="out of memory: %s" % str(e)[:80])

    # ---- the d = 128 scaling configuration: one fixed problem, sharded by (batch, head) ----
    if not args.no_sweep and not args.small and not args.train_shape:
        try:
            line["sweep"] = bench_sweep(F, dev, world, rank, peaks, barrier, args.sweep_max_n)
        except torch.OutOfMemoryError as e:   # pragma: no cover
            line["sweep"] = dict(error="out of memory: %s" % str(e)[:80])
        F.check_device_status(dev)

    # ---- one long sequence with fewer (batch, head) pairs than GPUs: sharded along the sequence ----
    if not args.no_sweep and not args.no_context_parallel and not args.small and not args.train_shape:
        try:
            line["context_parallel"] = bench_context_parallel(F, dev, world, rank, peaks, timed, args.cp_shape)
        except torch.OutOfMemoryError as e:   # pragma: no cover
            line["context_parallel"] = dict(error="out of memory: %s" % str(e)[:80])
        F.check_device_status(dev)

    # ---- head mixing: the reference's head-conv operator (no conv) and the composed conv + mix configuration ----
    if not args.no_headmix and not args.small and not args.train_shape:
        try:
            line["headmix"] = bench_headmix(F, dev, timed, args.headmix_shape, args.convmix_shape)
        except torch.OutOfMemoryError as e:   # pragma: no cover
            line["headmix"] = dict(error="out of memory: %s" % str(e)[:80])

    if rank == 0 and not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu_reference_sample(steps=3, warmup=1)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def bench_sweep(F, dev, world, rank, peaks, barrier, max_n):
    """Scaling configuration: conv-attention forward + backward, bf16, d = 128, theta (6,11), causal,
    B x H = 8 x 32 = 256 (batch, head) units as ONE problem at each sequence length, divided among the
    ranks by fmta_b200.sharding (a head split here: every rank owns H/world heads of every batch entry),
    the filter gradient summed by sharding.allreduce_param_grad (NCCL).  Inputs are seeded per
    (sequence length, batch, head), so the problem is the same for any number of ranks.  A rank walks its
    slice in batch chunks small enough for about 24 GB of device memory per chunk."""
    import torch.distributed as dist
    from fmta_b200 import sharding
    B, H, d, cq, ck = (SWEEP[k] for k in ("B", "H", "d", "cq", "ck"))
    scale = 1.0 / math.sqrt(d)
    plan = sharding.shard_plan(B, H, 1, world, rank)
    assert plan["mode"] in ("head", "batch")
    Bl, Hl = plan["b_hi"] - plan["b_lo"], plan["h_hi"] - plan["h_lo"]
    th_full = torch.randn(H, cq, ck, generator=torch.Generator().manual_seed(11)) * 0.02
    th_full[:, cq - 1, ck // 2] += 1.0
    th = th_full[plan["h_lo"]:plan["h_hi"]].contiguous().to(dev)
    stream = torch.cuda.current_stream()
    points = []
    for N in SWEEP["Ns"]:
        if N > max_n:
            continue
        per_bh = N * d * 64                         # inputs, outputs and workspaces of one (batch, head) pair, bytes
        bchunk = max(1, min(Bl, int(24e9 // (per_bh * Hl))))
        data = []
        for b in range(plan["b_lo"], plan["b_hi"]):
            t4 = []
            for _ in range(4):
                t4.append(torch.empty(Hl, N, d, device=dev, dtype=torch.bfloat16))
            for hi, h in enumerate(range(plan["h_lo"], plan["h_hi"])):
                g = torch.Generator(device=dev).manual_seed(1000003 * N + 131 * b + h)
                for t in t4:
                    t[hi] = torch.randn(N, d, device=dev, generator=g).to(torch.bfloat16)
            data.append(t4)
        chunks = []
        for c0 in range(0, Bl, bchunk):
            chunks.append([torch.stack([data[b][i] for b in range(c0, min(Bl, c0 + bchunk))]) for i in range(4)])
        del data

        def step():
            dth = None
            for q, k, v, do in chunks:
                kt = F.ktilde_buffer(q, th)
                O, M, L, LSE = F.forward(q, k, v, th, scale, cq - 1, (ck - 1) // 2, True, return_lse=True, ktilde=kt)
                D = F.rowdot(do, O)
                dQ, dK, dV, dTh = F.backward(q, k, v, do, D, LSE, th, scale, cq - 1, (ck - 1) // 2, True, ktilde=kt)
                dth = dTh if dth is None else dth + dTh
            return sharding.allreduce_param_grad(dth, plan)      # [H, cq, ck] on every rank

        fl, E = flops_attn(B, H, N, d)
        est = fl / (150e12 * world)                  # seconds per step at about 150 TFLOP/s per GPU
        steps = max(1, min(10, int(2.0 / max(est, 1e-4))))
        step()                                       # warm-up
        barrier()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            out = step()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        tf = fl / (ms * 1e-3) / 1e12
        points.append(dict(N=N, ms_per_step=ms, steps=steps, value=tf, unit="TFLOP/s", per_gpu_tflops=tf / world,
                           frac_of_peak=tf / world / peaks["tflops_sustained"], flops_attn_tflop=fl / 1e12,
                           units_per_rank=Bl * Hl, batch_chunk=bchunk,
                           dtheta_checksum=float(out.double().abs().sum().item())))
        del chunks
        torch.cuda.empty_cache()
    return dict(metric="conv-attn fwd+bwd TFLOP/s, scaling configuration", scaling="strong",
                config=dict(workload="train fwd+bwd bf16 B=%d,H=%d,d=%d,theta(%d,%d),causal, one problem per N "
                                     "sharded by (batch, head)" % (B, H, d, cq, ck), shard_mode=plan["mode"],
                            collective="all-reduce of dTheta [H,%d,%d] fp32 (NCCL)" % (cq, ck) if world > 1 else "none"),
                peak=peaks["tflops_sustained"], peak_source=peaks["source"] + " (sustained)", points=points)


def bench_context_parallel(F, dev, world, rank, peaks, timed, shape=None):
    """One fixed problem with few (batch, head) pairs and a long sequence (default B=1,H=4,N=65536,d=128,
    theta (6,11), causal), sharded along the SEQUENCE: every rank holds the zigzag share of the positions and calls
    `context_parallel_conv_attention` (gathers of Q, K, V, dO, D, LSE over the process group, the rank's windows on
    its GPU, one all-reduce of dTheta).  A step is forward + backward through the autograd Function, gathers
    included; strong scaling.  TFLOP/s by the headline's convention."""
    from fmta_b200 import context_parallel as cp
    B, H, N, d = tuple(int(x) for x in shape.split(",")) if shape else (1, 4, 65536, 128)
    cq, ck = 6, 11
    scale = 1.0 / math.sqrt(d)
    layout = "zigzag" if N % (2 * world * cp.ALIGN) == 0 else "contiguous"
    wins = cp.windows_for_rank(N, world, rank, layout)
    n_loc = sum(hi - lo for lo, hi in wins)
    g = torch.Generator(device=dev).manual_seed(77)       # the same sequence at every world size
    ql, kl, vl, dol = (cp.take_local(torch.randn(B, H, N, d, device=dev, generator=g).to(torch.bfloat16), wins) for _ in range(4))
    gt = torch.Generator(device=dev).manual_seed(5)
    th = torch.randn(H, cq, ck, device=dev, generator=gt) * 0.02
    th[:, cq - 1, ck // 2] += 1.0
    dol32 = dol.float()
    out = {}

    def step():
        q, k, v = (t.detach().requires_grad_() for t in (ql, kl, vl))
        t = th.detach().requires_grad_()
        O = cp.context_parallel_conv_attention(q, k, v, t, scale, cq - 1, (ck - 1) // 2, True, None, layout)
        O.backward(dol32)
        out["dth"] = t.grad

    fl, E = flops_attn(B, H, N, d)
    step()
    steps = max(2, min(10, int(1.0 / max(fl / (150e12 * world), 1e-4))))
    ms = timed(step, steps) / steps
    tf = fl / (ms * 1e-3) / 1e12
    gathered = 4 * B * H * N * d * 2 + 2 * B * H * N * 4
    return dict(metric="conv-attn fwd+bwd TFLOP/s, one sequence sharded along its length", scaling="strong",
                config=dict(workload="train fwd+bwd bf16 B=%d,H=%d,N=%d,d=%d,theta(%d,%d),causal; %d (batch, head) pairs"
                                     % (B, H, N, d, cq, ck, B * H), layout=layout, windows_rank0=[list(w) for w in cp.windows_for_rank(N, world, 0, layout)],
                            collective=("all-gather of Q, K, V, dO (bf16), D, LSE: %.0f MB per rank and step; all-reduce of dTheta (NCCL)"
                                        % (gathered / 1e6)) if world > 1 else "none"),
                ms_per_step=ms, steps=steps, value=tf, unit="TFLOP/s", per_gpu_tflops=tf / world,
                frac_of_peak=tf / world / peaks["tflops_sustained"], flops_attn_tflop=fl / 1e12,
                dtheta_checksum=float(out["dth"].double().abs().sum().item()))


def bench_headmix(F, dev, timed, shape=None, convmix_shape=None):
    """Rank-local timings (ms, CUDA events) of the head-mixing operators, forward + dQ/dW + dK/dV, causal, bf16:
    the reference's head-conv attention (dense W over 16 and 32 heads, no conv) and, unless a shape is given, the
    head-mixing training configuration (theta (6,11) then groups of 4; B=2,H=32,N=8192,d=128).  TFLOP/s counts
    the attention products only (14*d per score entry), as the headline does."""
    pts = []
    g = torch.Generator(device=dev).manual_seed(11)
    shapes = [tuple(int(x) for x in shape.split(","))] if shape else [(2, 16, 4096, 64), (2, 32, 4096, 64), (2, 16, 4096, 128)]
    if convmix_shape and not shape:
        shapes = []
    for (B, H, N, d) in shapes:
        q, k, v, do = (torch.randn(B, H, N, d, device=dev, generator=g).to(torch.bfloat16) for _ in range(4))
        w = torch.randn(H, H, device=dev, generator=g) / math.sqrt(H)
        sc = 1.0 / math.sqrt(d)
        o, l, m = F.head_conv_attention_forward(q, k, v, w, sc, True)
        fns = (lambda: F.head_conv_attention_forward(q, k, v, w, sc, True),
               lambda: F.head_conv_attention_bwd_dq_dw(q, k, v, w, o, do, l, m, True, sc),
               lambda: F.head_conv_attention_bwd_dkdv(q, k, v, w, o, do, l, m, True, sc))
        ms = []
        for fn in fns:
            fn()
            ms.append(timed(fn, 3) / 3)
        E = B * H * N * (N + 1) / 2.0
        pts.append(dict(workload="head-conv attention (dense %d-head mix, no conv) B=%d,N=%d,d=%d" % (H, B, N, d),
                        fwd_ms=ms[0], dq_dw_ms=ms[1], dk_dv_ms=ms[2], value=14.0 * d * E / (sum(ms) * 1e-3) / 1e12, unit="TFLOP/s"))
        del q, k, v, do, o, l, m
    if not shape:
        B, H, N, d, G, cq, ck = 2, 32, 8192, 128, 4, 6, 11
        if convmix_shape:
            B, H, N, d = (int(x) for x in convmix_shape.split(","))
        q, k, v, do = (torch.randn(B, H, N, d, device=dev, generator=g).to(torch.bfloat16) for _ in range(4))
        th = torch.randn(H, cq, ck, device=dev, generator=g) * 0.02
        th[:, cq - 1, ck // 2] += 1.0
        w = (torch.eye(G, device=dev).repeat(H // G, 1, 1) + 0.02 * torch.randn(H // G, G, G, device=dev, generator=g)).contiguous()
        sc = 1.0 / math.sqrt(d)
        o, l, m, lse = F.conv_headmix_forward(q, k, v, w, th, sc, True, out_dtype=torch.float32)
        # the fused backward is what the autograd function calls (both halves get the exchange scratch)
        fns = (lambda: F.conv_headmix_forward(q, k, v, w, th, sc, True, out_dtype=torch.float32),
               lambda: F.conv_headmix_backward(q, k, v, w, o, do, l, m, th, True, sc, lse=lse))
        ms = [timed(fn, 1) for fn in fns]
        E = B * H * N * (N + 1) / 2.0
        pts.append(dict(workload="conv (6,11) then mix in groups of 4, B=%d,H=%d,N=%d,d=%d (cluster kernels)" % (B, H, N, d),
                        fwd_ms=ms[0], bwd_ms=ms[1], value=14.0 * d * E / (sum(ms) * 1e-3) / 1e12, unit="TFLOP/s"))
    return dict(metric="head-mix attention fwd+bwd TFLOP/s (per GPU)", points=pts)


def bench_decode(F, dev, dec, peaks, world, timed):
    B, H, d, Nk, ql, cq, ck, ks = (dec[k] for k in ("B", "H", "d", "Nk", "q_len", "cq", "ck", "k_splits"))
    g = torch.Generator(device=dev).manual_seed(5)
    K = torch.randn(B, H, Nk, d, device=dev, dtype=torch.bfloat16, generator=g)
    V = torch.randn(B, H, Nk, d, device=dev, dtype=torch.bfloat16, generator=g)
    Q = torch.randn(B, H, ql, d, device=dev, dtype=torch.bfloat16, generator=g)
    th = torch.randn(H, cq, ck, device=dev, generator=g) * 0.02
    th[:, cq - 1, ck // 2] += 1.0
    sc = 1.0 / math.sqrt(d)
    fn = lambda: F.forward_inference(Q, K, V, th, ks, sc, cq - 1, (ck - 1) // 2, False, 0)
    for _ in range(3):
        fn()
    steps = 10
    ms = timed(fn, steps) / steps
    by = 2 * B * H * Nk * d * 2 + B * H * ql * d * 2 + B * H * d * 4
    gbs = by / (ms * 1e-3) / 1e9
    # the same cache through the paged layout (256-key pages, shuffled block table) with the
    # training forward's causal mask: same bytes, reported beside the headline
    paged = None
    try:
        del K, V
        page = 256
        ppb = Nk // page
        Kp = torch.randn(B * ppb, H, page, d, device=dev, dtype=torch.bfloat16, generator=g)
        Vp = torch.randn(B * ppb, H, page, d, device=dev, dtype=torch.bfloat16, generator=g)
        table = torch.randperm(B * ppb, device=dev, generator=g).to(torch.int32).view(B, ppb).contiguous()
        fnp = lambda: F.forward_inference_paged(Q, Kp, Vp, table, th, ks, sc, cq - 1, (ck - 1) // 2,
                                                max_seq_len=Nk, offset_causal=True)
        for _ in range(3):
            fnp()
        msp = timed(fnp, steps) / steps
        paged = dict(value=world * by / (msp * 1e-3) / 1e9, unit="GB/s", ms_per_step=msp, page_size=page,
                     offset_causal=True)
        del Kp, Vp
    except torch.OutOfMemoryError:   # pragma: no cover
        paged = dict(error="out of memory")
    return dict(metric="decode HBM GB/s", value=world * gbs, unit="GB/s", ms_per_step=ms, paged=paged,
                config=dict(workload="fwd_inference bf16 B=%d(per GPU),H=%d,d=%d,Nk=%d,q_len=%d,theta(%d,%d),k_splits=%d"
                            % (B, H, d, Nk, ql, cq, ck, ks), l2="17 GB of K/V per step >> L2"),
                # DRAM traffic: the committed ncu capture at B=4,H=32,Nk=16384 read+wrote 1.02x its algorithmic
                # bytes (summary under profiles/); it grows with the (b,h) x key units
                roofline=dict(bound="hbm", kernel="decode_kernel", achieved=gbs, peak=peaks["hbm"], unit="GB/s",
                              frac=gbs / peaks["hbm"], peak_source=peaks["source"], traffic=1.02 * by,
                              traffic_unit="bytes per launch (ncu capture of a smaller case, scaled)"),
                gpu_launches=4 * steps)


if __name__ == "__main__":
    main()
