#!/usr/bin/env python3
"""Benchmark of the NVFP4 weight path on B200 (one JSON line on stdout, rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--quick]

Headline (N = 1): the six fused sibling gemvs that share one input (K = 4096, outputs 4096, 4096,
4096, 512, 64, 32; all NVFP4, M = 1) -- one launch of the tensor-core kernel k_gemv_umma per step.  `value` is the
achieved HBM rate in TB/s: algorithmic bytes of one step / device time of one step, inputs
resident in HBM, the step rotating over weight copies whose total exceeds L2 several times.
`e2e` is the same step through the C ABI with HOST buffers: the activation row is copied from
pinned host memory and the six outputs are copied back inside the timed region (weights are
model state and stay resident, as they do in the engine that calls this path).
`sub` carries the other single-GPU configurations (single gemv [12288x4096]; the vocabulary
projection; siblings at M = 2, 4, 8; the same matrix against 32 and 128 rows; MoE layer at 1, 4, 8
and 64 tokens with microseconds per layer; quantiser), each with its own byte count and fraction of
the measured HBM peak.
N > 1 (torchrun, one rank per GPU): the headline path does not shard, so every rank runs the
headline workload on its own GPU (value = sum over GPUs over the slowest rank's time, weak scaling);
the expert-parallel MoE layer, the one part with a real exchange, is reported as `ep_moe`.
All data is synthetic: seeded N(0, 0.02) bf16 weights quantised by this library's bit-exact
quantiser, N(0, 1) fp32 activations.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np
import torch

UMMA = os.environ.get('B200_NVFP4_UMMA') != '0'          # the library's default path; '0' times the CUDA-core kernels
if UMMA:
    DTYPE = 'nvfp4 weights (e2m1 + e4m3 block scales) x activations as eight e2m1 digit columns (14 fractional bits of the row maximum), fp32 accumulate'
    MATH = 'tcgen05.mma kind::mxf4nvf4.block_scale.block16, accumulators in TMEM'
    KERNEL = 'k_gemv_umma<0>'
else:
    DTYPE = 'nvfp4 weights (e2m1 + e4m3 scales), f16 products, f32 accumulate'
    MATH = 'fp32-mac' if os.environ.get('B200_NVFP4_MATH') == '1' else 'f16x2-chains'
    KERNEL = 'k_gemv_tma'

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as G  # noqa: E402

SIBLINGS = [4096, 4096, 4096, 512, 64, 32]
K_HID = 4096
L2_BYTES = 126e6


def profiled_traffic():
    """DRAM read + write bytes per launch of the headline kernel, from the committed ncu summary
    (profiles/k_gemv_umma_siblings_M1.md, line 'roofline.traffic bytes per launch: N'); None if absent."""
    import re
    p = os.path.join(ROOT, 'profiles', 'k_gemv_umma_siblings_M1.md')
    if not UMMA or not os.path.exists(p):
        return None
    m = re.search(r'roofline\.traffic bytes per launch:\s*(\d+)', open(p).read())
    return int(m.group(1)) if m else None


def measured_peaks():
    p = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d['hbm_gbs']), 'measured'
    return 6650.0, 'fallback'


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a timed region runs."""
    Q = 'clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,' \
        'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap'

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', '-i', str(self.index), '--query-gpu=' + self.Q,
                                          '--format=csv,noheader,nounits', '-lms', '100'],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True); self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(',')])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.t.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'), r[2:6]):
                if v.lower().startswith('active'):
                    reasons.add(name)
        if not sm:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': [], 'samples': 0}
        return {'sm_mhz': statistics.median(sm), 'sm_max_mhz': max(mx), 'reasons': sorted(reasons), 'samples': len(sm)}


def nv_bytes(N, K):
    return N * K // 2 + N * K // 16 + 4


def capture_steps(fns):
    """One CUDA graph holding the given steps back to back (kernel nodes keep the programmatic
    launch edges the library asks for, so consecutive steps overlap their ramp and tail)."""
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for fn in fns:
            fn()
    return g


LAST_TIMING = {}
LAST_TIMING_HEAD = {}


def time_steps(fns, steps, warmup, replays=50):
    """Times `steps` steps, step i being fns[i % len(fns)], captured back to back in CUDA graphs of at most
    about a hundred launches (whole rotations plus one shorter graph for the remainder).  The K-step
    region is replayed `replays` times, each replay bracketed by its own CUDA events on the launching
    stream; returns the MEDIAN ms per step and leaves min / max / replays in LAST_TIMING."""
    for fn in fns:
        fn()                                        # outside capture: one-time attribute set-up
    torch.cuda.synchronize()
    R = len(fns)
    G = R * max(1, min(128 // R, steps // R))          # steps per graph: whole rotations, about a hundred launches
    full = capture_steps([fns[i % R] for i in range(G)]) if steps >= G else None
    rem = capture_steps([fns[i % R] for i in range(steps % G)]) if steps % G else None
    for _ in range(max(1, (warmup + G - 1) // G)):
        (full or rem).replay()
    torch.cuda.synchronize()
    per = []
    replays = max(1, min(replays, int(2.0e6 / max(steps, 1)) or 1))        # keep very long regions to a few replays
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(replays)]
    for e0, e1 in evs:
        e0.record()
        for _ in range(steps // G if full is not None else 0):
            full.replay()
        if rem is not None:
            rem.replay()
        e1.record()
    torch.cuda.synchronize()
    per = sorted(e0.elapsed_time(e1) / steps for e0, e1 in evs)
    LAST_TIMING.clear()
    LAST_TIMING.update({'min_ms_per_step': per[0], 'max_ms_per_step': per[-1], 'replays': replays, 'steps_per_replay': steps})
    return per[len(per) // 2]


def make_weight(P, N, K, seed):
    gen = torch.Generator(device='cuda').manual_seed(seed)
    w = (torch.randn((N, K), generator=gen, device='cuda') * 0.02).to(torch.bfloat16)
    return P.quantize(w), w


def clone_weight(P, W):
    return P.Nvfp4Weight(W.packed.clone(), W.scale.clone(), W.gscale.clone())


# ---- workloads --------------------------------------------------------------------------------

def bench_siblings(P, M, steps, warmup, copies, sampler_index=None):
    base = [make_weight(P, n, K_HID, 1000 + i)[0] for i, n in enumerate(SIBLINGS)]
    sets = [base] + [[clone_weight(P, W) for W in base] for _ in range(copies - 1)]
    x = torch.randn((M, K_HID), device='cuda', generator=torch.Generator(device='cuda').manual_seed(2))
    ybuf = torch.empty(M * sum(SIBLINGS), device='cuda')       # the six outputs side by side: one copy brings them all back
    ys, o = [], 0
    for n in SIBLINGS:
        ys.append(ybuf[o:o + M * n].view(M, n)); o += M * n
    jobs = [P.make_jobs(ws, [x] * 6, ys) for ws in sets]
    split = P.split_workspace(M, K_HID, x.device) if M > 1 else None       # activations split once per call (the *_ws entry points)
    fns = [lambda ws=ws, j=j: P.gemv_multi(ws, x, M, ys, jobs=j, ws=split) for ws, j in zip(sets, jobs)]
    nbytes = sum(nv_bytes(n, K_HID) for n in SIBLINGS) + M * K_HID * 4 + M * sum(SIBLINGS) * 4
    if sampler_index is None:
        ms = time_steps(fns, steps, warmup)
        return ms, nbytes, None, (sets, x, ys, jobs, ybuf)
    with ClockSampler(sampler_index) as cs:
        ms = time_steps(fns, steps, warmup)
        if steps * ms < 400:                        # keep the region long enough to be sampled
            time_steps(fns, int(400 / max(ms, 1e-3)), 0)
    return ms, nbytes, cs.summary(), (sets, x, ys, jobs, ybuf)


def bench_siblings_e2e(P, state, steps, warmup):
    """Host buffers: x from pinned memory in, the six outputs (one device buffer) back to pinned memory (copy,
    product and copy replayed as one graph launch per step), a stream synchronisation per step.  The loop itself is C++ against the C ABI (tests/cpp/e2e_loop.cu), the way
    an engine like the reference's calls this path; Python only hands over the pointers."""
    import ctypes as C
    sets, x, ys, jobs, ybuf = state
    M, n = x.shape[0], len(SIBLINGS)
    path = os.path.join(ROOT, 'tests', 'cpp', 'libe2e_loop.so')
    if not os.path.exists(path):
        raise SystemExit('tests/cpp/libe2e_loop.so is missing: run __graft_entry__.build()')
    L = C.CDLL(path)
    L.e2e_gemv_multi_loop.restype = C.c_double
    xh = torch.randn((M, K_HID)).pin_memory()
    yh = torch.empty(ybuf.shape).pin_memory()
    rot = (P.GemvJob * (len(jobs) * n))()
    for c, j in enumerate(jobs):
        for i in range(n):
            rot[c * n + i] = j[i]
    rc = C.c_int(0)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()                      # a stream of its own: the loop captures its step into graphs, which the legacy default stream cannot do
    ms = L.e2e_gemv_multi_loop(rot, len(jobs), n, M, K_HID, C.c_void_p(xh.data_ptr()), C.c_void_p(x.data_ptr()), C.c_size_t(M * K_HID * 4),
                               C.c_void_p(ybuf.data_ptr()), C.c_void_p(yh.data_ptr()), C.c_size_t(ybuf.numel() * 4),
                               int(steps), int(warmup), C.c_void_p(s.cuda_stream), C.byref(rc))
    torch.cuda.synchronize()
    if rc.value:
        raise SystemExit('end-to-end loop failed: status %d' % rc.value)
    return ms, M * K_HID * 4, M * sum(SIBLINGS) * 4


def bench_gemv_single(P, steps, warmup, copies):
    N = 12288
    base, _ = make_weight(P, N, K_HID, 999)
    ws = [base] + [clone_weight(P, base) for _ in range(copies - 1)]
    x = torch.randn((1, K_HID), device='cuda')
    y = torch.empty((1, N), device='cuda')
    ms = time_steps([lambda W=W: P.gemm(W, x, y) for W in ws], steps, warmup)
    return ms, nv_bytes(N, K_HID) + K_HID * 4 + N * 4


def bench_gemm_wide(P, N, M, steps, warmup):
    """Prefill GEMM (configs[3]): NVFP4 [N x 4096] against M bf16 rows through b200_nvfp4_gemm_bf16 (per-token
    activation quantiser + tcgen05 mxf4nvf4 GEMM, W read once).  Returns ms, flops, W-read-once bytes, and
    the relative L2 distance of the result from the exact product (reported, not a pass/fail figure)."""
    base, wb = make_weight(P, N, K_HID, 998)
    copies = max(2, int(2.2 * L2_BYTES / nv_bytes(N, K_HID)) + 1)
    ws_ = [base] + [clone_weight(P, base) for _ in range(copies - 1)]
    x = torch.randn((M, K_HID), device='cuda', generator=torch.Generator(device='cuda').manual_seed(3)).to(torch.bfloat16)
    y = torch.empty((M, N), device='cuda')
    scratch = P.gemm_bf16_workspace(M, K_HID, x.device)
    ms = time_steps([lambda W=W: P.gemm_bf16(W, x, y, scratch) for W in ws_], steps, warmup)
    exact = x.float() @ P.dequantize(base).t()
    dev = ((y - exact).norm() / exact.norm()).item()
    return ms, 2.0 * M * N * K_HID, nv_bytes(N, K_HID) + M * K_HID * 2 + M * N * 4, dev


def bench_gemm_exact(P, N, M, steps, warmup):
    """The exact wide GEMM (b200_nvfp4_gemm_bf16_exact: weights dequantised to fp16 in the kernel, f16 MMA)."""
    base, _ = make_weight(P, N, K_HID, 998)
    copies = max(2, int(2.2 * L2_BYTES / nv_bytes(N, K_HID)) + 1)
    ws_ = [base] + [clone_weight(P, base) for _ in range(copies - 1)]
    x = torch.randn((M, K_HID), device='cuda', generator=torch.Generator(device='cuda').manual_seed(3)).to(torch.bfloat16)
    y = torch.empty((M, N), device='cuda')
    scratch = torch.empty(P.lib().b200_nvfp4_gemm_bf16_exact_workspace_bytes(M, K_HID), dtype=torch.uint8, device='cuda')
    ms = time_steps([lambda W=W: P.gemm_bf16_exact(W, x, y, scratch) for W in ws_], steps, warmup)
    exact = x.float() @ P.dequantize(base).t()
    return ms, 2.0 * M * N * K_HID, nv_bytes(N, K_HID) + M * K_HID * 2 + M * N * 4, ((y - exact).norm() / exact.norm()).item()


def bench_dense_mlp(P, steps, warmup):
    """The dense-layer MLP of the reference (kernels/layer.cu:235-254) at its shapes, one token: gate and up
    [12288 x 4096] as one 2-job launch, down [4096 x 12288] with the clamped SwiGLU applied as its
    activations are staged (b200_dense_mlp)."""
    H, I = K_HID, 12288
    sets = []
    for c in range(3):
        g, _ = make_weight(P, I, H, 900 + 3 * c); u, _ = make_weight(P, I, H, 901 + 3 * c); d, _ = make_weight(P, H, I, 902 + 3 * c)
        sets.append((g, u, d))
    x = torch.randn((1, H), device='cuda'); y = torch.empty((1, H), device='cuda')
    ws = P.dense_mlp_workspace(1, H, I, x.device)
    ms = time_steps([lambda t=t: P.dense_mlp(x, t[0], t[1], t[2], 10.0, y, ws) for t in sets], steps, warmup)
    return ms, 2 * nv_bytes(I, H) + nv_bytes(H, I) + 2 * H * 4


def bench_kda_groups(P, steps, warmup):
    """The fused sibling groups of the linear-attention layer with their real shapes (reference
    kernels/kda.cu:235-266, tests/gate_gemv_multi.cu:54-61)."""
    out = {}
    groups = {'kda_qkv_8192x4096_x3': ([8192, 8192, 8192], 4096, False), 'kda_lowrank_128_128_64_x4096': ([128, 128, 64], 4096, False),
              'kda_up_8192x128_x2_own_x': ([8192, 8192], 128, True)}
    for name, (Ns, K, own_x) in groups.items():
        nb = sum(nv_bytes(n, K) for n in Ns)
        copies = max(2, min(64, int(2.2 * L2_BYTES / nb) + 1))
        sets = [[make_weight(P, n, K, 800 + i)[0] for i, n in enumerate(Ns)]]
        sets += [[clone_weight(P, W) for W in sets[0]] for _ in range(copies - 1)]
        xs = [torch.randn((1, K), device='cuda') for _ in Ns] if own_x else [torch.randn((1, K), device='cuda')] * len(Ns)
        ys = [torch.empty((1, n), device='cuda') for n in Ns]
        jobs = [P.make_jobs(ws, xs, ys) for ws in sets]
        ms = time_steps([lambda ws=ws, j=j: P.gemv_multi(ws, xs, 1, ys, jobs=j) for ws, j in zip(sets, jobs)], steps, warmup)
        b = nb + (len(Ns) if own_x else 1) * K * 4 + sum(Ns) * 4
        out[name] = {'us': ms * 1e3, 'bytes': b, 'tbps': b / (ms * 1e-3) / 1e12, 'weight_copies_in_rotation': copies}
    return out


def build_moe_layers(P, n_layers, H, I, E, topk, seed, zipf=False):
    layers = []
    for l in range(n_layers):
        gen = torch.Generator(device='cuda').manual_seed(seed + l)
        ex = []
        for e in range(E + 1):
            tr = []
            for (o, i) in ((I, H), (I, H), (H, I)):
                w = (torch.randn((o, i), generator=gen, device='cuda') * 0.02).to(torch.bfloat16)
                tr.append(P.quantize(w))
            ex.append(tuple(tr))
        router = (torch.randn((E, H), generator=gen, device='cuda') * 0.02).to(torch.bfloat16)
        bias = torch.randn(E, generator=gen, device='cuda') * 0.1
        if zipf:
            bias = bias + zipf_bias(E).cuda()
        layers.append(P.MoeLayer(router, bias, ex[:E], ex[E], topk, H, I))
    return layers


def bench_moe(P, layers, M, steps, warmup, prepare=True):
    """prepare: build the layers' TMA descriptors first (b200_moe_prepare), so that the experts run on
    the tensor-core kernel; False times the CUDA-core experts."""
    for L in layers:
        if prepare: P.moe_prepare(L)
    H, I, E, topk = layers[0].hidden, layers[0].inter, layers[0].n_expert, layers[0].topk
    gen = torch.Generator(device='cuda').manual_seed(77)
    xs = [torch.randn((M, H), generator=gen, device='cuda') for _ in range(8)]
    y = torch.empty((M, H), device='cuda'); sel = torch.empty((M, topk), dtype=torch.int32, device='cuda')
    wts = torch.empty((M, topk), device='cuda')
    combos = [(layers[i % len(layers)], xs[i % len(xs)]) for i in range(max(len(layers), len(xs)))]
    fns, distinct = [], []
    for L, x in combos:
        fns.append(lambda L=L, x=x: P.moe_forward(L, x, y, sel, wts))
        fns[-1](); torch.cuda.synchronize()
        distinct.append(len(set(sel.cpu().numpy().ravel().tolist())))
    ms = time_steps(fns, steps, warmup)
    for L in layers:
        if prepare: P.moe_release(L)
    per_expert = 3 * nv_bytes(I, H)
    d = float(np.mean(distinct))
    nbytes = (d + 1) * per_expert + E * H * 2 + E * 4 + 2 * M * H * 4 + M * topk * 8
    return ms, nbytes, d


def bench_quantize(P, steps, warmup):
    N, K = 12288, K_HID
    ws = [(torch.randn((N, K), device='cuda') * 0.02).to(torch.bfloat16) for _ in range(3)]
    out = P.quantize(ws[0])
    ms = time_steps([lambda w=w: P.quantize(w, out=out) for w in ws], steps, warmup)
    # two passes over the bf16 input (tensor amax, then codes) plus the NVFP4 output
    return ms, 2 * N * K * 2 + nv_bytes(N, K)


def zipf_bias(E, s=1.1, seed=4, strength=0.08):
    """Expert popularity ~ Zipf(s) over a seeded permutation, applied as a ranking bias (the
    benchmark asks for Zipf-skewed routing; the router itself stays the model's)."""
    rng = np.random.default_rng(seed)
    p = 1.0 / np.arange(1, E + 1) ** s
    p = p[rng.permutation(E)]
    return torch.from_numpy((strength * np.log(p / p.mean())).astype(np.float32))


def bench_ep(P, a, rank, local, world, peak, T):
    """Expert-parallel MoE (configs[4]) through the library's C++/NCCL context (b200_ep_*): T tokens x hidden
    4096, 144 experts sharded over the ranks, top-8 + replicated shared expert, Zipf(1.1) routing bias, 3
    stacked layers, x <- rmsnorm(x + y) between layers.  world == 1 runs the same code without NCCL.
    Returns the result dict on rank 0 (None elsewhere); raises SystemExit on a parity failure."""
    import torch.distributed as dist
    dev = torch.device('cuda', local)
    Lyr, E, topk, H, I = 3, 144, 8, 4096, 1536
    Tl = T // world
    pb = zipf_bias(E)
    layers = [P.ep_gpu.RankLayer(50, l, E, topk, H, I, rank, world, dev, max_tokens=Tl, popularity_bias=pb) for l in range(Lyr)]
    g = torch.Generator(device=dev).manual_seed(123)
    x_all = torch.randn((T, H), generator=g, device=dev).to(torch.bfloat16).float()      # bf16-valued activations
    x0 = x_all[rank * Tl:(rank + 1) * Tl].contiguous()
    ys = [torch.empty((Tl, H), device=dev) for _ in range(Lyr)]
    sel = torch.empty((Tl, topk), dtype=torch.int32, device=dev); wts = torch.empty((Tl, topk), device=dev)
    barrier = dist.barrier if world > 1 else (lambda: None)

    def step(x):
        for L, y in zip(layers, ys):
            L.forward(x, y, sel, wts)
            x = x + y
            x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5)
        return x
    for _ in range(a.warmup):
        step(x0)
    torch.cuda.synchronize(); barrier()
    steps = max(3, min(a.steps, 50))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as cs:
        e0.record()
        for _ in range(steps):
            step(x0)
        e1.record()
        torch.cuda.synchronize()
    barrier()
    ms = e0.elapsed_time(e1) / steps
    # statistics of the last step (outside the timed region): bytes, load, phase times
    stats = [L.ctx.stats() for L in layers]
    nb = float(sum(L.step_bytes(Tl, st) for L, st in zip(layers, stats)))
    vec = torch.tensor([ms, nb, float(sum(st['recv_rows'] for st in stats)), float(sum(st['dispatch_bytes_out'] for st in stats)),
                        float(sum(st['combine_bytes_in'] for st in stats)), float(sum(st['dispatch_us'] for st in stats)),
                        float(sum(st['combine_us'] for st in stats)), float(sum(st['experts_us'] for st in stats))], device=dev, dtype=torch.float64)
    allv = [torch.zeros_like(vec) for _ in range(world)]
    if world > 1:
        dist.all_gather(allv, vec)
    else:
        allv = [vec]
    allv = torch.stack(allv).cpu().numpy()
    ms = float(allv[:, 0].max())                       # the slowest rank sets the time
    # end to end: tokens from pinned host memory in, outputs back, every step
    xh = x0.cpu().pin_memory(); yh = torch.empty_like(xh).pin_memory(); xd = torch.empty_like(x0)
    n_e2e = max(1, min(steps, 10))
    torch.cuda.synchronize(); barrier()
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        xd.copy_(xh, non_blocking=True)
        out = step(xd)
        yh.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / n_e2e
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64); dist.all_reduce(t, op=dist.ReduceOp.MAX); e2e_ms = t.item()
    # parity of the sharded layer on rank 0's tokens: against the single-GPU entry point on the full layer, and
    # against the CPU oracle on the first tokens (both with the activations quantised as the wide GEMM does)
    y_ep, sel_ep, wts_ep = layers[0].forward(x0)
    par = None
    if rank == 0:
        full = [P.ep_gpu.expert_weights(50, 0, e, H, I, dev) for e in range(E + 1)]
        ref_layer = P.MoeLayer(layers[0].router, layers[0].bias, full[:E], full[E], topk, H, I)
        P.moe_prepare(ref_layer)
        y_ref, sel_ref, _ = P.moe_forward(ref_layer, x0[:max(16, min(Tl, 64))].contiguous())
        n = y_ref.shape[0]
        par = {'rel_l2_vs_single_gpu': ((y_ep[:n] - y_ref).norm() / y_ref.norm()).item(), 'sel_equal': bool(torch.equal(sel_ep[:n], sel_ref))}
        if T == a.ep_tokens[0]:
            O = G.load_oracle()
            rows = [0, 1]
            sel_h, wts_h = sel_ep[rows].cpu().numpy(), wts_ep[rows].cpu().numpy()
            need = set(sel_h.ravel().tolist())
            host = [tuple(w.numpy() for w in full[e]) if (e in need or e == E) else None for e in range(E + 1)]
            yo = O.moe_experts_act_nvfp4(x0[rows].cpu().numpy(), sel_h, wts_h, host[:E], host[E])
            par['rel_l2_vs_oracle_first_tokens'] = O.rel_l2(y_ep[rows].cpu().numpy(), yo)
        P.moe_release(ref_layer)
        del full, ref_layer
    status = P.device_status()
    for L in layers:
        L.close()
    del layers
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    bad = par['rel_l2_vs_single_gpu'] > 1e-3 or not par['sel_equal'] or par.get('rel_l2_vs_oracle_first_tokens', 0.0) > 1e-3
    total_b = float(allv[:, 1].sum())
    rows = allv[:, 2]
    res = {
        'metric': 'nvfp4_moe_ep_tokens_per_s', 'value': T / (ms * 1e-3), 'unit': 'tokens/s', 'n_gpus': world, 'tokens': T, 'steps': steps,
        'ms_per_step': ms, 'us_per_layer': ms * 1e3 / Lyr, 'scaling': 'strong',
        'config': {'workload': 'expert-parallel MoE: %d tokens x 4096, 144 experts (%d per GPU), top-8 + shared expert, Zipf(1.1) routing bias, 3 stacked layers (configs[4])' % (T, E // world),
                   'collective': 'one ncclAllGather of counts + ONE grouped ncclSend/ncclRecv round each way per layer (bf16 rows + ids out, f32 rows back); host code in C++ inside the library' if world > 1 else 'none (one rank)',
                   'math': 'experts on the wide tensor-core GEMM (both operands NVFP4), rows grouped by local expert'},
        'hbm_bytes_per_step_all_gpus': total_b, 'hbm_tbps_all_gpus': total_b / (ms * 1e-3) / 1e12,
        'roofline': {'bound': 'hbm', 'kernel': 'k_gemm_mxf4 (local experts)', 'achieved': total_b / world / (ms * 1e-3) / 1e9, 'peak': peak,
                     'unit': 'GB/s per GPU', 'frac': total_b / world / (ms * 1e-3) / 1e9 / peak},
        'load_rows_per_gpu_max_over_mean': float(rows.max() / max(rows.mean(), 1e-9)),
        'nvlink': {'dispatch_bytes_out_per_gpu_per_layer': float(allv[:, 3].mean() / Lyr), 'combine_bytes_in_per_gpu_per_layer': float(allv[:, 4].mean() / Lyr),
                   'dispatch_us_per_layer_max': float(allv[:, 5].max() / Lyr), 'combine_us_per_layer_max': float(allv[:, 6].max() / Lyr),
                   'dispatch_gbps_per_gpu': float(allv[:, 3].mean() / max(allv[:, 5].max(), 1e-9) / 1e3),
                   'combine_gbps_per_gpu': float(allv[:, 4].mean() / max(allv[:, 6].max(), 1e-9) / 1e3), 'peak_gbps_per_direction': 900.0},
        'experts_us_per_layer_max': float(allv[:, 7].max() / Lyr),
        'e2e': {'value': T / (e2e_ms * 1e-3), 'unit': 'tokens/s', 'ms_per_step': e2e_ms, 'h2d_bytes_per_step': T * H * 4, 'd2h_bytes_per_step': T * H * 4},
        'parity': par, 'parity_ok': not bad, 'device_status': status, 'clocks': cs.summary(),
    }
    return res


def run_ep_all(P, a, rank, local, world, peak):
    """The expert-parallel layer at every requested token count; remembers the one-GPU result of this box so
    that later runs at N > 1 can state their speed-up over it."""
    out = {}
    n1_path = os.path.join('/tmp', 'b200_nvfp4_ep_n1.json')
    n1 = json.load(open(n1_path)) if world > 1 and os.path.exists(n1_path) else {}
    for T in a.ep_tokens:
        if T % world:
            continue
        r = bench_ep(P, a, rank, local, world, peak, T)
        if r is None:
            continue
        if str(T) in n1:
            r['speedup_vs_n1'] = n1[str(T)] / r['ms_per_step']
            r['efficiency_vs_n1'] = r['speedup_vs_n1'] / world
        out['T%d' % T] = r
    if rank == 0 and world == 1:
        try:
            json.dump({str(r['tokens']): r['ms_per_step'] for r in out.values()}, open(n1_path, 'w'))
        except OSError:
            pass
    return out


# ---- CPU baseline: the reference's CPU path restated (torch dequantise, then matmul) ------------

def cpu_siblings_step(host_sets, x):
    """reference ref/gen_moe.py:23-30 dequant + F.linear for the six sibling weights."""
    import torch.nn.functional as F
    KE2M1 = torch.tensor([0., .5, 1., 1.5, 2., 3., 4., 6.], dtype=torch.float32)
    outs = []
    for pk, sc, gs in host_sets:
        out_f, in_f = pk.shape[0], pk.shape[1] * 2
        flat = pk.reshape(-1)
        low, high = flat & 0x0F, (flat >> 4) & 0x0F
        comb = torch.stack((low, high), dim=1).reshape(out_f, in_f).long()
        vals = KE2M1[comb & 7] * torch.where((comb & 8).bool(), -1.0, 1.0)
        w = (vals.reshape(out_f, in_f // 16, 16) * (sc.float().reshape(out_f, in_f // 16, 1) / gs)).reshape(out_f, in_f)
        outs.append(F.linear(x, w))
    return outs


def cpu_dequant(pk, sc, gs):
    """reference ref/gen_moe.py:23-30: packed nibbles, e4m3 scales and the global scale to fp32 weights."""
    KE2M1 = torch.tensor([0., .5, 1., 1.5, 2., 3., 4., 6.], dtype=torch.float32)
    out_f, in_f = pk.shape[0], pk.shape[1] * 2
    flat = pk.reshape(-1)
    comb = torch.stack((flat & 0x0F, (flat >> 4) & 0x0F), dim=1).reshape(out_f, in_f).long()
    vals = KE2M1[comb & 7] * torch.where((comb & 8).bool(), -1.0, 1.0)
    return (vals.reshape(out_f, in_f // 16, 16) * (sc.float().reshape(out_f, in_f // 16, 1) / gs)).reshape(out_f, in_f)


def cpu_moe_step(x, router, bias, experts, shared, topk, scale=2.5, limit=10.0):
    """The MoE block as the reference's CPU path computes it (ref/gen_moe.py:62-96 restated): sigmoid
    router with bias-ranked top-k, renormalised gates, clamped SwiGLU experts dequantised on the fly,
    shared expert.  Returns y and the number of distinct routed experts."""
    import torch.nn.functional as F
    score = torch.sigmoid(F.linear(x, router))
    sel = torch.topk(score + bias, topk, dim=-1).indices
    w = score.gather(1, sel)
    w = w / (w.sum(-1, keepdim=True) + 1e-20) * scale

    def mlp(trip, rows):
        g = torch.clamp(F.linear(rows, cpu_dequant(*trip[0])), max=limit)
        u = torch.clamp(F.linear(rows, cpu_dequant(*trip[1])), -limit, limit)
        return F.linear(F.silu(g) * u, cpu_dequant(*trip[2]))
    y = mlp(shared, x)
    distinct = torch.unique(sel).tolist()
    for e in distinct:
        tok, slot = (sel == e).nonzero(as_tuple=True)
        y.index_add_(0, tok, mlp(experts[e], x[tok]) * w[tok, slot].unsqueeze(1))
    return y, len(distinct)


def cpu_baseline(P, state, max_seconds=20.0):
    sets, x = state[0], state[1]
    host = [(W.packed.cpu(), W.scale.cpu().view(torch.float8_e4m3fn), W.gscale.cpu()) for W in sets[0]]
    xh = x.cpu()
    cpu_siblings_step(host, xh)                       # warm-up
    n, t0 = 0, time.perf_counter()
    while True:
        cpu_siblings_step(host, xh); n += 1
        el = time.perf_counter() - t0
        if el > max_seconds or n >= 20:
            break
    return el / n, n


# ---- main ---------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=2000)
    ap.add_argument('--warmup', type=int, default=50)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--quick', action='store_true', help='headline only, no sub-workloads')
    ap.add_argument('--ep-tokens', default='256,2048', help='token counts of the expert-parallel workload')
    ap.add_argument('--gemm-shapes', default='12288x32,12288x128,12288x512,4096x32,4096x128,4096x512', help='NxM list of the prefill GEMM sub-workloads')
    ap.add_argument('--profile', default='', help='run ONE small workload a few times and exit (for ncu captures): siblings, gemm_NxM, quant, moe_mM, moe_prefill_mM')
    ap.add_argument('--only', default='', help='comma list of sub-workloads to run (gemv,lm_head,siblings,gemm,gemm_exact,dense_mlp,kda,moe,moe_prefill,ep,quant)')
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    a.ep_tokens = [int(t) for t in str(a.ep_tokens).split(',') if t]
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    peak, peak_kind = measured_peaks()
    P = G.load_package()

    if a.impl == 'reference':
        return reference_arm(a, P, rank, peak)

    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: there is no CPU fallback')
    torch.cuda.set_device(local)
    P.lib()                                            # fail now if the library is missing
    P.set_option(P.OPT_STABLE_WEIGHTS, 1)              # weights are loaded once, as in the engine
    if a.profile:
        return profile_mode(P, a.profile)
    if world > 1:
        # The headline path does not shard (every gemv is an independent unit: replicas only), so each
        # rank runs the headline workload on its own GPU and the line reports the sum; the one part of
        # the path with a real exchange, the expert-parallel MoE layer, is measured too and reported
        # as the sub-object "ep_moe".
        import torch.distributed as dist
        dist.init_process_group('nccl', device_id=torch.device('cuda', local))
        copies = 10
        torch.cuda.synchronize(); dist.barrier()
        ms, nbytes, clocks, state = bench_siblings(P, 1, a.steps, a.warmup, copies, sampler_index=local)
        LAST_TIMING_HEAD.update(LAST_TIMING)
        torch.cuda.synchronize(); dist.barrier()
        e2e_ms, h2d, d2h = bench_siblings_e2e(P, state, min(a.steps, 2000), a.warmup)
        t = torch.tensor([ms, e2e_ms], device='cuda', dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)                      # the slowest rank sets the time
        ms, e2e_ms = t.tolist()
        del state
        torch.cuda.empty_cache()
        dist.barrier()
        ep = run_ep_all(P, a, rank, local, world, peak)
        dist.barrier()
        if rank == 0:
            value = world * nbytes / (ms * 1e-3) / 1e12
            print(json.dumps({
                'metric': 'nvfp4_gemv_hbm_tbps', 'value': value, 'unit': 'TB/s', 'n_gpus': world, 'steps': a.steps,
                'warmup': a.warmup, 'ms_per_step': ms, 'higher_is_better': True, 'scaling': 'weak',
                'vs_baseline': None, 'dtype': DTYPE, 'data': 'synthetic',
                'config': {'workload': 'six fused sibling NVFP4 gemvs sharing one input, K=4096, N=[4096,4096,4096,512,64,32], M=1 (configs[1])',
                           'parallelism': 'replicas only: %d independent copies of the workload, one per GPU, no collective; value = sum over GPUs, time = slowest rank' % world,
                           'l2': 'inputs larger than L2: step i reads weight copy i mod %d (%.0f MB in rotation)' % (copies, copies * nbytes / 1e6),
                           'launch': 'steps captured back to back in CUDA graphs; programmatic dependent launch; weights declared stable',
                           'math': MATH},
                'roofline': {'bound': 'hbm', 'kernel': KERNEL, 'achieved': value * 1e3 / world, 'peak': peak, 'unit': 'GB/s per GPU',
                             'frac': value * 1e3 / world / peak, 'peak_kind': peak_kind, 'traffic': profiled_traffic(),
                             'algorithmic_bytes_per_launch': nbytes},
                'e2e': {'value': world * nbytes / (e2e_ms * 1e-3) / 1e12, 'unit': 'TB/s', 'ms_per_step': e2e_ms,
                        'h2d_bytes_per_step': h2d * world, 'd2h_bytes_per_step': d2h * world},
                'cpu_baseline': None, 'gpu_launches': a.steps, 'device_status': P.device_status(), 'clocks': clocks,
                'timing': dict(LAST_TIMING_HEAD),
                'ep_moe': ep,
            }))
        dist.destroy_process_group()
        if rank == 0 and any(not r['parity_ok'] for r in ep.values()):
            raise SystemExit('expert-parallel parity failed: %s' % {k: r['parity'] for k, r in ep.items()})
        return

    copies = 10                                        # 10 x 29.7 MB = 297 MB per rotation, > 2x L2
    ms, nbytes, clocks, state = bench_siblings(P, 1, a.steps, a.warmup, copies, sampler_index=local)
    LAST_TIMING_HEAD.update(LAST_TIMING)
    value = nbytes / (ms * 1e-3) / 1e12
    e2e_ms, h2d, d2h = bench_siblings_e2e(P, state, min(a.steps, 2000), a.warmup)
    sub = {}
    only = set(filter(None, a.only.split(',')))
    want = lambda k: not a.quick and (not only or k in only)
    sub_steps = min(a.steps, 1000)
    if want('gemv'):
        m, b = bench_gemv_single(P, sub_steps, a.warmup, copies)
        sub['gemv_12288x4096_M1'] = {'us': m * 1e3, 'bytes': b, 'tbps': b / (m * 1e-3) / 1e12,
                                      'frac_of_measured_hbm': b / (m * 1e-3) / 1e9 / peak}
    if want('lm_head'):
        N = 154880                                     # the vocabulary projection: 357 MB of weights, larger than L2 by itself
        W, _ = make_weight(P, N, K_HID, 997)
        xl = torch.randn((1, K_HID), device='cuda'); yl = torch.empty((1, N), device='cuda')
        m = time_steps([lambda: P.gemm(W, xl, yl)], max(50, sub_steps // 10), a.warmup)
        b = nv_bytes(N, K_HID) + K_HID * 4 + N * 4
        sub['gemv_154880x4096_M1'] = {'us': m * 1e3, 'bytes': b, 'tbps': b / (m * 1e-3) / 1e12,
                                       'frac_of_measured_hbm': b / (m * 1e-3) / 1e9 / peak}
        del W
    if want('siblings'):
        for M in (2, 4, 8):
            m, b, _, _ = bench_siblings(P, M, sub_steps, a.warmup, copies)
            sub['siblings_M%d' % M] = {'us': m * 1e3, 'bytes': b, 'tbps': b / (m * 1e-3) / 1e12,
                                       'frac_of_measured_hbm': b / (m * 1e-3) / 1e9 / peak}
    if want('gemm'):
        fp4_peak = 4 * 1652.6                        # dense FP4 tensor peak taken as 4x the measured bf16 burst (TFLOP/s)
        for N, M in [tuple(int(v) for v in sh.split('x')) for sh in a.gemm_shapes.split(',') if sh]:
            if True:
                m, fl, b, dev_exact = bench_gemm_wide(P, N, M, max(20, sub_steps // 5), a.warmup)
                sub['gemm_bf16_%dx4096_M%d' % (N, M)] = {
                    'us': m * 1e3, 'min_us': LAST_TIMING['min_ms_per_step'] * 1e3, 'tflops': fl / (m * 1e-3) / 1e12,
                    'frac_of_fp4_peak_4x_bf16': fl / (m * 1e-3) / 1e12 / fp4_peak, 'bytes_w_read_once': b,
                    'frac_of_measured_hbm': b / (m * 1e-3) / 1e9 / peak, 'rel_l2_vs_exact_product': dev_exact,
                    'launches_per_step': 2, 'kernels': 'k_quant_act + k_gemm_mxf4'}
    if want('gemm_exact'):
        for N, M in [tuple(int(v) for v in sh.split('x')) for sh in a.gemm_shapes.split(',') if sh]:
            m, fl, b, dev_exact = bench_gemm_exact(P, N, M, max(20, sub_steps // 5), a.warmup)
            sub['gemm_bf16_exact_%dx4096_M%d' % (N, M)] = {
                'us': m * 1e3, 'tflops': fl / (m * 1e-3) / 1e12, 'frac_of_measured_bf16_peak': fl / (m * 1e-3) / 1e12 / 1652.6,
                'frac_of_measured_hbm': b / (m * 1e-3) / 1e9 / peak, 'rel_l2_vs_exact_product': dev_exact,
                'launches_per_step': 2, 'kernels': 'k_act_f16 + k_gemm_f16w'}
    if want('dense_mlp'):
        m, b = bench_dense_mlp(P, max(50, sub_steps // 5), a.warmup)
        sub['dense_mlp_12288_M1'] = {'us': m * 1e3, 'bytes': b, 'tbps': b / (m * 1e-3) / 1e12, 'frac_of_measured_hbm': b / (m * 1e-3) / 1e9 / peak}
    if want('kda'):
        for k, v in bench_kda_groups(P, sub_steps, a.warmup).items():
            v['frac_of_measured_hbm'] = v['tbps'] * 1e3 / peak
            sub[k] = v
    if want('moe'):
        layers = build_moe_layers(P, 3, 4096, 1536, 144, 8, 4000)
        for M, prep in ((1, True), (4, True), (8, True), (64, True), (1, False)):
            m, b, d = bench_moe(P, layers, M, sub_steps, a.warmup, prep)
            sub['moe_layer_I1536_M%d%s' % (M, '' if prep else '_cuda_core')] = {
                'us_per_layer': m * 1e3, 'bytes': b, 'distinct_routed': d, 'tbps': b / (m * 1e-3) / 1e12,
                'frac_of_measured_hbm': b / (m * 1e-3) / 1e9 / peak,
                'experts': 'tensor-core (prepared layer)' if prep else 'CUDA-core'}
        del layers
    if want('moe_prefill'):
        # grouped-expert GEMM under Zipf(1.1) routing on one GPU (configs[3]): prefill widths on a prepared layer
        layers = build_moe_layers(P, 3, 4096, 1536, 144, 8, 4100, zipf=True)
        for M in (32, 128, 512):
            m, b, d = bench_moe(P, layers, M, max(20, sub_steps // 10), a.warmup, True)
            fl = 2.0 * M * 9 * 3 * 1536 * 4096
            sub['moe_prefill_zipf_I1536_M%d' % M] = {
                'us_per_layer': m * 1e3, 'bytes': b, 'distinct_routed': d, 'tbps': b / (m * 1e-3) / 1e12,
                'frac_of_measured_hbm': b / (m * 1e-3) / 1e9 / peak, 'tflops': fl / (m * 1e-3) / 1e12,
                'experts': 'wide tensor-core GEMM, rows grouped by expert'}
        del layers
        torch.cuda.empty_cache()
    ep = run_ep_all(P, a, rank, local, 1, peak) if want('ep') else {}
    if want('quant'):
        m, b = bench_quantize(P, min(sub_steps, 200), a.warmup)
        sub['quantize_12288x4096'] = {'us': m * 1e3, 'bytes': b, 'tbps': b / (m * 1e-3) / 1e12,
                                      'frac_of_measured_hbm': b / (m * 1e-3) / 1e9 / peak}
    cpu_s, cpu_n = cpu_baseline(P, state)
    out = {
        'metric': 'nvfp4_gemv_hbm_tbps', 'value': value, 'unit': 'TB/s', 'n_gpus': 1, 'steps': a.steps,
        'warmup': a.warmup, 'ms_per_step': ms, 'higher_is_better': True, 'scaling': 'weak',
        'vs_baseline': None, 'dtype': DTYPE,
        'data': 'synthetic',
        'config': {'workload': 'six fused sibling NVFP4 gemvs sharing one input, K=4096, N=[4096,4096,4096,512,64,32], M=1 (configs[1])',
                   'l2': 'inputs larger than L2: step i reads weight copy i mod %d (%.0f MB in rotation)' % (copies, copies * nbytes / 1e6),
                   'launch': 'steps captured back to back in CUDA graphs; programmatic dependent launch; weights declared stable',
                   'math': MATH},
        'roofline': {'bound': 'hbm', 'kernel': KERNEL, 'achieved': value * 1e3, 'peak': peak, 'unit': 'GB/s',
                     'frac': value * 1e3 / peak, 'peak_kind': peak_kind, 'traffic': profiled_traffic(),
                     'algorithmic_bytes_per_launch': nbytes},
        'e2e': {'value': nbytes / (e2e_ms * 1e-3) / 1e12, 'unit': 'TB/s', 'ms_per_step': e2e_ms,
                'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h},
        'cpu_baseline': {'value': nbytes / cpu_s / 1e12, 'unit': 'TB/s', 'cores': torch.get_num_threads(),
                         'kind': 'port', 'sample': '%d steps of the same six-sibling workload, torch dequantise + linear' % cpu_n,
                         'ms_per_step': cpu_s * 1e3},
        'gpu_launches': a.steps, 'device_status': P.device_status(), 'clocks': clocks, 'timing': dict(LAST_TIMING_HEAD),
        'sub': sub, 'ep_moe': ep,
    }
    print(json.dumps(out))
    if any(not r['parity_ok'] for r in ep.values()):
        raise SystemExit('expert-parallel parity failed: %s' % {k: r['parity'] for k, r in ep.items()})


def profile_mode(P, name):
    """One workload, a few plain launches, no timing and no graphs: the command ncu captures are taken from
    (the summaries under profiles/ name the exact command line)."""
    reps = 3
    if name == 'siblings':
        Ws = [make_weight(P, n, K_HID, 1000 + i)[0] for i, n in enumerate(SIBLINGS)]
        x = torch.randn((1, K_HID), device='cuda')
        for _ in range(reps):
            P.gemv_multi(Ws, x, 1)
    elif name.startswith('gemmx_'):                   # the exact wide GEMM (f16 MMA)
        N, M = (int(v) for v in name[6:].split('x'))
        Ws = [make_weight(P, N, K_HID, 998 + i)[0] for i in range(reps)]
        x = torch.randn((M, K_HID), device='cuda').to(torch.bfloat16)
        y = torch.empty((M, N), device='cuda')
        for W in Ws:
            P.gemm_bf16_exact(W, x, y)
    elif name.startswith('gemm_'):
        N, M = (int(v) for v in name[5:].split('x'))
        Ws = [make_weight(P, N, K_HID, 998 + i)[0] for i in range(reps)]          # a fresh weight per launch
        x = torch.randn((M, K_HID), device='cuda').to(torch.bfloat16)
        y = torch.empty((M, N), device='cuda'); ws = P.gemm_bf16_workspace(M, K_HID, x.device)
        for W in Ws:
            P.gemm_bf16(W, x, y, ws)
    elif name == 'quant':
        ws = [(torch.randn((12288, K_HID), device='cuda') * 0.02).to(torch.bfloat16) for _ in range(2)]
        out = None
        for w in ws:
            out = P.quantize(w, out=out)
    elif name.startswith('moe_'):
        prefill = name.startswith('moe_prefill_m')
        M = int(name.split('_m')[-1])
        layers = build_moe_layers(P, 2, 4096, 1536, 144, 8, 4100, zipf=prefill)
        for L in layers:
            P.moe_prepare(L)
        x = torch.randn((M, 4096), device='cuda', generator=torch.Generator(device='cuda').manual_seed(77))
        for i in range(reps):
            P.moe_forward(layers[i % 2], x)
    else:
        raise SystemExit('unknown --profile workload: ' + name)
    torch.cuda.synchronize()
    print(json.dumps({'profile': name, 'device_status': P.device_status()}))


def reference_arm(a, P, rank, peak):
    """The reference's CPU implementation of the path (its torch dequantise-then-matmul,
    restated) on the host cores, on the headline workload."""
    if rank != 0:
        return
    # torchrun sets OMP_NUM_THREADS=1 for its workers; this arm is the only work on the host and takes every core
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0)) if hasattr(os, 'sched_getaffinity') else (os.cpu_count() or 1)))
    O = G.load_oracle()
    rng = np.random.default_rng(1000)
    host = []
    for i, n in enumerate(SIBLINGS):
        bits = O.f32_to_bf16_bits(np.random.default_rng(1000 + i).normal(0, 0.02, (n, K_HID)).astype(np.float32))
        p, s, gs = O.quantize_tensor(O.bf16_bits_to_f32(bits))
        host.append((torch.from_numpy(p), torch.from_numpy(s).view(torch.float8_e4m3fn), torch.from_numpy(gs)))
    x = torch.from_numpy(rng.normal(0, 1, (1, K_HID)).astype(np.float32))
    steps, warm = min(a.steps, 20), min(a.warmup, 3)
    for _ in range(warm):
        cpu_siblings_step(host, x)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_siblings_step(host, x)
    sec = (time.perf_counter() - t0) / steps
    nbytes = sum(nv_bytes(n, K_HID) for n in SIBLINGS) + K_HID * 4 + sum(SIBLINGS) * 4
    v = nbytes / sec / 1e12
    print(json.dumps({
        'impl': 'reference', 'metric': 'nvfp4_gemv_hbm_tbps', 'value': v, 'unit': 'TB/s', 'n_gpus': a.gpus,
        'steps': steps, 'warmup': warm, 'ms_per_step': sec * 1e3, 'higher_is_better': True, 'scaling': 'weak',
        'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': 'six fused sibling NVFP4 gemvs sharing one input, K=4096, N=[4096,4096,4096,512,64,32], M=1 (configs[1])'},
        'cpu_baseline': {'value': v, 'unit': 'TB/s', 'cores': torch.get_num_threads(), 'kind': 'port',
                         'sample': '%d full steps (bounded from --steps %d)' % (steps, a.steps)},
        'e2e': {'value': v, 'unit': 'TB/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'ep_moe': reference_arm_moe(a) if a.gpus > 1 else None,
    }))


def reference_arm_moe(a):
    """N > 1: the GPU arm also reports the expert-parallel MoE layer ("ep_moe").  The reference has no
    multi-GPU form; its CPU path for the same layer is the restated block above, on all host threads,
    on a bounded sample: 8 tokens through one layer (the GPU arm: --ep-tokens tokens through 3 layers).  Weights are random
    NVFP4 bytes of the benchmark's shapes (drawing and quantising 435 real matrices on the CPU would
    take minutes and does not change the time of a step)."""
    H, I, E, topk, T = 4096, 1536, 144, 8, 8
    gen = torch.Generator().manual_seed(50)

    def trip(o, i):
        pk = torch.randint(0, 256, (o, i // 2), dtype=torch.uint8, generator=gen)
        sc = torch.randint(40, 72, (o, i // 16), dtype=torch.uint8, generator=gen).view(torch.float8_e4m3fn)   # scales around 0.1 .. 1.5
        return pk, sc, torch.tensor([64.0])
    experts = [(trip(I, H), trip(I, H), trip(H, I)) for _ in range(E)]
    shared = (trip(I, H), trip(I, H), trip(H, I))
    router = (torch.randn((E, H), generator=gen) * 0.02).to(torch.bfloat16).float()
    bias = torch.randn(E, generator=gen) * 0.1
    x = torch.randn((T, H), generator=gen)
    steps, warm = max(1, min(a.steps, 3)), 1
    cpu_moe_step(x, router, bias, experts, shared, topk)
    t0 = time.perf_counter()
    for _ in range(steps):
        _, distinct = cpu_moe_step(x, router, bias, experts, shared, topk)
    sec = (time.perf_counter() - t0) / steps
    nbytes = (distinct + 1) * 3 * nv_bytes(I, H) + E * H * 2 + E * 4 + 2 * T * H * 4
    v = nbytes / sec / 1e12
    return ({
        'impl': 'reference', 'metric': 'nvfp4_moe_ep_hbm_tbps', 'value': v, 'unit': 'TB/s', 'n_gpus': a.gpus,
        'steps': steps, 'warmup': warm, 'ms_per_step': sec * 1e3, 'higher_is_better': True, 'scaling': 'strong',
        'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': 'MoE layer on the host cores: 144 experts, top-8 + shared expert, hidden 4096, inter 1536 (configs[4] has no multi-GPU reference: its CPU path on one layer)'},
        'tokens_per_s': T / sec,
        'cpu_baseline': {'value': v, 'unit': 'TB/s', 'cores': torch.get_num_threads(), 'kind': 'port',
                         'sample': '%d tokens through one layer, %d distinct routed experts; %d steps' % (T, distinct, steps)},
        'e2e': {'value': v, 'unit': 'TB/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
    })


if __name__ == '__main__':
    main()
