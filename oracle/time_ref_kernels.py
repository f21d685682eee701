"""Times the REFERENCE's own CUDA kernels (oracle/_ref/libref_kernels.so, the reference's
kernels/gemv.cu and kernels/moe.cu recompiled for sm_100a) beside this library on identical
device buffers: "the kernel to beat" on the same GPU.  Test infrastructure, not product; run by hand:

    python oracle/time_ref_kernels.py

Workloads: [12288 x 4096] gemv, the six sibling gemvs (the reference fuses at most four jobs per
launch: two launches), the MoE layer at the reference's compiled geometry (inter 2048) for 1 and 4
tokens.  Launches are captured in CUDA graphs and rotate over weight copies larger than L2.
"""
import ctypes as C
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, 'tests'))
import __graft_entry__ as G          # noqa: E402
import bench                         # noqa: E402
from util import ref_kernels         # noqa: E402


def ptr(t):
    return C.c_void_p(t.data_ptr())


def main():
    P = G.load_package()
    R = ref_kernels()
    if R is None:
        raise SystemExit('oracle/_ref/libref_kernels.so is missing (built by `make -C oracle` where the reference checkout exists)')
    P.set_option(P.OPT_STABLE_WEIGHTS, 1)
    st = lambda: C.c_void_p(torch.cuda.current_stream().cuda_stream)
    K, copies = 4096, 10
    rows = []

    # [12288 x 4096] gemv
    base, _ = bench.make_weight(P, 12288, K, 999)
    ws = [base] + [bench.clone_weight(P, base) for _ in range(copies - 1)]
    x = torch.randn((1, K), device='cuda'); y = torch.empty((1, 12288), device='cuda')
    ours = bench.time_steps([lambda W=W: P.gemm(W, x, y) for W in ws], 500, 10)
    ref = bench.time_steps([lambda W=W: R.ref_gemm_nvfp4(ptr(y), ptr(W.packed), ptr(W.scale), ptr(W.gscale), ptr(x), 1, 12288, K, st()) for W in ws], 500, 10)
    rows.append(('gemv [12288 x 4096], M = 1', ref * 1e3, ours * 1e3))
    del ws, base

    # six siblings
    sib = bench.SIBLINGS
    base = [bench.make_weight(P, n, K, 1000 + i)[0] for i, n in enumerate(sib)]
    sets = [base] + [[bench.clone_weight(P, W) for W in base] for _ in range(copies - 1)]
    ys = [torch.empty((1, n), device='cuda') for n in sib]
    ours = bench.time_steps([lambda s=s: P.gemv_multi(s, x, 1, ys) for s in sets], 500, 10)
    vp = C.c_void_p

    def ref_group(s, lo, hi):
        n = hi - lo
        arr = lambda f: (vp * n)(*[f(i) for i in range(lo, hi)])
        R.ref_gemv_multi(arr(lambda i: ys[i].data_ptr()), arr(lambda i: s[i].packed.data_ptr()), arr(lambda i: s[i].scale.data_ptr()),
                         arr(lambda i: s[i].gscale.data_ptr()), arr(lambda i: x.data_ptr()), (C.c_int * n)(*sib[lo:hi]), n, K, st())
    ref = bench.time_steps([lambda s=s: (ref_group(s, 0, 4), ref_group(s, 4, 6)) for s in sets], 500, 10)
    rows.append(('six sibling gemvs, M = 1 (reference: two launches)', ref * 1e3, ours * 1e3))
    del sets, base

    # MoE layer at the reference's compiled geometry
    H, I, E, topk = R.ref_moe_hidden(), R.ref_moe_inter(), R.ref_moe_experts(), R.ref_moe_topk()
    layers = bench.build_moe_layers(P, 3, H, I, E, topk, 4100)
    for L in layers: P.moe_prepare(L)
    for M in (1, 4):
        xs = [torch.randn((M, H), device='cuda') for _ in range(4)]
        yo = torch.empty((M, H), device='cuda'); sel = torch.empty((M, topk), dtype=torch.int32, device='cuda'); wts = torch.empty((M, topk), device='cuda')
        wsr = torch.zeros(R.ref_moe_workspace_floats(M), dtype=torch.float32, device='cuda')
        combos = [(layers[i % 3], xs[i % 4]) for i in range(12)]
        ours = bench.time_steps([lambda L=L, x=x: P.moe_forward(L, x, yo, sel, wts) for L, x in combos], 300, 10)
        ref = bench.time_steps([lambda L=L, x=x: R.ref_moe_forward(ptr(x), ptr(L.router), ptr(L.bias), ptr(L.table), ptr(L.shared_table), E, topk,
                                                                    ptr(yo), ptr(sel), ptr(wts), ptr(wsr), M, st()) for L, x in combos], 300, 10)
        rows.append(('MoE layer, inter %d, M = %d' % (I, M), ref * 1e3, ours * 1e3))
    print('%-52s %14s %14s %8s' % ('workload', 'reference (us)', 'this lib (us)', 'ratio'))
    for name, r, o in rows:
        print('%-52s %14.1f %14.1f %8.2f' % (name, r, o, r / o))
    print('device status %x' % P.device_status())


if __name__ == '__main__':
    main()
