"""GPU parity for the MoE block through the C ABI: routing identical to the oracle as a set,
gate weights within 1e-5, layer output within rel-L2 1e-3 / max-abs 2e-2 (reference gate:
tests/gate_moe.cu:133-162 compares routing as a set and y by cosine / max_rel)."""
import ctypes as C
import numpy as np
import pytest
import torch

from util import pkg, oracle, host_triple, seeded_bf16, to_dev_bf16, ref_kernels, zipf_bias, exact_prefill, REL_TOL, ABS_TOL

pytestmark = pytest.mark.gpu


def build_layer(H, I, E, topk, seed, shared=True, on_gpu=False, router_std=0.02, bias_std=0.1, zipf=False):
    """Returns (device layer, host description for the oracle).  on_gpu: weights are drawn and
    quantised on the device (the quantiser is proven bit-exact separately) and only the experts
    a test needs are copied back."""
    P, O = pkg(), oracle()
    rng = np.random.default_rng(seed)
    rb = O.f32_to_bf16_bits(rng.normal(0, router_std, (E, H)).astype(np.float32))
    bias = rng.normal(0, bias_std, E).astype(np.float32)
    if zipf:
        bias = (bias + zipf_bias(E)).astype(np.float32)
    n = E + (1 if shared else 0)
    dev = []
    if on_gpu:
        g = torch.Generator(device='cuda').manual_seed(seed)
        for e in range(n):
            tr = []
            for (o, i) in ((I, H), (I, H), (H, I)):
                w = (torch.randn((o, i), generator=g, device='cuda') * 0.02).to(torch.bfloat16)
                tr.append(P.quantize(w))
            dev.append(tuple(tr))
        host = None
    else:
        host = [(host_triple((I, H), seed * 1000 + 3 * e), host_triple((I, H), seed * 1000 + 3 * e + 1),
                 host_triple((H, I), seed * 1000 + 3 * e + 2)) for e in range(n)]
        dev = [tuple(P.Nvfp4Weight(*w) for w in t) for t in host]
    layer = P.MoeLayer(to_dev_bf16(rb), torch.from_numpy(bias).cuda(), dev[:E], dev[E] if shared else None,
                       topk, H, I)
    return layer, dict(rb=rb, bias=bias, host=host, dev=dev, E=E, topk=topk, shared=shared)


def host_experts(d, needed):
    """Oracle-side (gate, up, down) triples; experts not in `needed` are left as None."""
    out = []
    for e in range(d['E'] + (1 if d['shared'] else 0)):
        if d['host'] is not None:
            out.append(d['host'][e])
        elif e in needed or e == d['E']:
            out.append(tuple(w.numpy() for w in d['dev'][e]))
        else:
            out.append(None)
    return out


def check_layer(layer, d, x, tol=REL_TOL):
    P, O = pkg(), oracle()
    M = x.shape[0]
    y, sel, wts = P.moe_forward(layer, torch.from_numpy(x).cuda())
    torch.cuda.synchronize()
    sel_h, wts_h = sel.cpu().numpy(), wts.cpu().numpy()
    logits = O.router_logits(x, d['rb'])
    sel_o, wts_o, gap = O.route(logits, d['bias'], d['topk'])
    assert gap.min() > 1e-6, 'seed gives a near-tie in the ranking; pick another'
    for m in range(M):
        assert set(sel_h[m].tolist()) == set(sel_o[m].tolist()), m
        ref = {int(e): float(w) for e, w in zip(sel_o[m], wts_o[m])}
        assert all(abs(ref[int(e)] - float(w)) < 1e-5 for e, w in zip(sel_h[m], wts_h[m]))
        assert list(sel_h[m]) == list(sel_o[m])        # and in the same (descending) order
    ex = host_experts(d, set(sel_o.ravel().tolist()))
    yo = O.moe_experts(x, sel_o, wts_o, ex[:d['E']], ex[d['E']] if d['shared'] else None)
    r, a = O.rel_l2(y.cpu().numpy(), yo), O.max_abs(y.cpu().numpy(), yo)
    assert r <= tol and a <= ABS_TOL, (r, a)
    return y, sel, wts


def test_moe_golden(golden):
    P, O = pkg(), oracle()
    z = golden('moe')
    E, K, H, I = int(z['E']), int(z['topk']), int(z['H']), int(z['I'])
    trip = lambda e, nm: P.Nvfp4Weight(z['e%d_%s_packed' % (e, nm)], z['e%d_%s_scale' % (e, nm)], z['e%d_%s_gs' % (e, nm)])
    ex = [(trip(e, 'gate'), trip(e, 'up'), trip(e, 'down')) for e in range(E + 1)]
    layer = P.MoeLayer(to_dev_bf16(z['router_bits']), torch.from_numpy(z['bias']).cuda(), ex[:E], ex[E], K, H, I,
                       float(z['scaling']), float(z['limit']))
    y, sel, wts = P.moe_forward(layer, torch.from_numpy(z['x']).cuda())
    for m in range(int(z['M'])):
        assert set(sel[m].tolist()) == set(z['sel'][m].tolist())
        ref = {int(e): float(w) for e, w in zip(z['sel'][m], z['wts'][m])}
        assert all(abs(ref[int(e)] - float(w)) < 1e-5 for e, w in zip(sel[m].tolist(), wts[m].tolist()))
        # row 2 saturates the SwiGLU clamps and is 40x larger: judge each row on its own norm
        assert O.rel_l2(y[m].cpu().numpy(), z['y'][m]) <= REL_TOL, m


@pytest.mark.parametrize('M', [1, 4])
@pytest.mark.parametrize('shared', [True, False])
def test_moe_mid_geometry(M, shared):
    layer, d = build_layer(1024, 512, 32, 8, seed=5, shared=shared)
    x = np.random.default_rng(M).normal(0, 1, (M, 1024)).astype(np.float32)
    check_layer(layer, d, x)


@pytest.mark.parametrize('I', [1536, 2048])
def test_moe_full_geometry(I):
    """hidden 4096, 144 experts, top-8 + shared; inter 1536 (benchmark) and 2048 (reference)."""
    layer, d = build_layer(4096, I, 144, 8, seed=40 + I, on_gpu=True)
    x = np.random.default_rng(I).normal(0, 1, (4, 4096)).astype(np.float32)
    y4, sel4, wts4 = check_layer(layer, d, x)
    P = pkg()
    # token m of a batch == that token alone, bit for bit (reference include/moe.h:38-40)
    for m in range(4):
        y1, sel1, wts1 = P.moe_forward(layer, torch.from_numpy(x[m:m + 1]).cuda())
        assert torch.equal(y1[0], y4[m]) and torch.equal(sel1[0], sel4[m]) and torch.equal(wts1[0], wts4[m])
    # expert half with the routing handed in == whole block
    y = P.moe_experts(layer, torch.from_numpy(x).cuda(), sel4, wts4)
    assert torch.equal(y, y4)
    # run-to-run
    y_again, _, _ = P.moe_forward(layer, torch.from_numpy(x).cuda())
    assert torch.equal(y_again, y4)
    if I == 2048:
        R = ref_kernels()
        if R is None:
            pytest.skip('oracle/_ref/libref_kernels.so was not prebuilt')
        assert (R.ref_moe_hidden(), R.ref_moe_inter(), R.ref_moe_experts(), R.ref_moe_topk()) == (4096, 2048, 144, 8)
        p = lambda t: C.c_void_p(t.data_ptr())
        for M in (1, 4):
            xd = torch.from_numpy(x[:M]).cuda()
            ws = torch.zeros(R.ref_moe_workspace_floats(M), dtype=torch.float32, device='cuda')
            yr = torch.zeros((M, 4096), device='cuda'); selr = torch.zeros((M, 8), dtype=torch.int32, device='cuda')
            wtsr = torch.zeros((M, 8), device='cuda')
            R.ref_moe_forward(p(xd), p(layer.router), p(layer.bias), p(layer.table), p(layer.shared_table), 144, 8,
                              p(yr), p(selr), p(wtsr), p(ws), M, None)
            torch.cuda.synchronize()
            assert torch.equal(selr, sel4[:M])
            assert (wtsr - wts4[:M]).abs().max().item() < 1e-5
            O = oracle()
            assert O.rel_l2(y4[:M].cpu().numpy(), yr.cpu().numpy()) <= REL_TOL


@pytest.mark.parametrize('H,I,E,M,shared', [(1024, 512, 32, 1, True), (1024, 512, 32, 5, False), (4096, 1536, 144, 1, True),
                                            (4096, 1536, 144, 8, True), (4096, 2048, 144, 4, True)])
def test_moe_prepared_layer_runs_tensor_core_experts(H, I, E, M, shared):
    """After b200_moe_prepare the experts of up to 8 tokens run on the tensor-core kernel: same
    routing, output within tolerance of the oracle and of the CUDA-core experts, each token equal
    to that token alone bit for bit, expert half alone equal to the whole block, run to run equal."""
    P, O = pkg(), oracle()
    layer, d = build_layer(H, I, E, 8, seed=70 + M, shared=shared, on_gpu=H > 1024)
    x = np.random.default_rng(M + I).normal(0, 1, (M, H)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    y_cc, sel_cc, _ = P.moe_forward(layer, xd)
    assert P.moe_prepare(layer)
    try:
        y, sel, wts = check_layer(layer, d, x)
        assert torch.equal(sel, sel_cc)
        assert not torch.equal(y, y_cc)              # a different kernel did run
        assert O.rel_l2(y.cpu().numpy(), y_cc.cpu().numpy()) <= REL_TOL
        for m in range(M):
            y1, sel1, wts1 = P.moe_forward(layer, xd[m:m + 1].contiguous())
            assert torch.equal(y1[0], y[m]) and torch.equal(sel1[0], sel[m]) and torch.equal(wts1[0], wts[m]), m
        assert torch.equal(P.moe_experts(layer, xd, sel, wts), y)
        assert torch.equal(P.moe_forward(layer, xd)[0], y)
        assert P.device_status() == 0
    finally:
        P.moe_release(layer)
    y_after, _, _ = P.moe_forward(layer, xd)          # released: the CUDA-core experts again
    assert torch.equal(y_after, y_cc)


@pytest.mark.parametrize('H,I,E,M,topk,shared', [(1024, 512, 32, 20, 8, True), (1024, 512, 8, 75, 1, False), (4096, 1536, 144, 33, 8, True)])
def test_moe_prepared_layer_groups_rows_by_expert_beyond_8_tokens(H, I, E, M, topk, shared):
    """More than 8 tokens on a prepared layer: pairs are sorted by expert on the device and every
    expert runs chunks of up to 8 rows.  Same bar as the small-batch path, and every token still
    equals that token alone (which takes the small-batch path) bit for bit."""
    P, O = pkg(), oracle()
    layer, d = build_layer(H, I, E, topk, seed=90 + M, shared=shared, on_gpu=H > 1024)
    x = np.random.default_rng(M + I).normal(0, 1, (M, H)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    y_cc, sel_cc, _ = P.moe_forward(layer, xd)
    assert P.moe_prepare(layer)
    P.set_option(P.OPT_PREFILL_FP4, 0)               # 16 tokens and more would otherwise take the wide GEMM
    try:
        y, sel, wts = check_layer(layer, d, x)
        assert torch.equal(sel, sel_cc)
        assert not torch.equal(y, y_cc)
        assert O.rel_l2(y.cpu().numpy(), y_cc.cpu().numpy()) <= REL_TOL
        for m in (0, M // 2, M - 1):
            y1, _, _ = P.moe_forward(layer, xd[m:m + 1].contiguous())
            assert torch.equal(y1[0], y[m]), m
        assert torch.equal(P.moe_experts(layer, xd, sel, wts), y)
        assert torch.equal(P.moe_forward(layer, xd)[0], y)
        assert P.device_status() == 0
    finally:
        P.set_option(P.OPT_PREFILL_FP4, 1)
        P.moe_release(layer)


@pytest.mark.parametrize('H,I,E,M,topk,shared,zipf', [(1024, 512, 144, 32, 8, True, True), (1024, 512, 144, 128, 8, True, True),
                                                       (1024, 512, 32, 75, 1, False, False), (1024, 512, 16, 300, 2, True, True),
                                                       (4096, 1536, 144, 40, 8, True, True)])
def test_moe_prefill_widths_run_the_grouped_wide_gemm(H, I, E, M, topk, shared, zipf):
    """16 tokens and more on a prepared layer: pairs sorted by expert on the device, every expert one job per
    chunk of rows of the wide GEMM (both operands NVFP4), under Zipf(1.1)-skewed routing.  Routing
    identical to the oracle; output within 1e-3 of the oracle that quantises the activations the same
    way, a few per cent from the exact block; a token's result independent of its batch; run to run equal."""
    P, O = pkg(), oracle()
    layer, d = build_layer(H, I, E, topk, seed=200 + M, shared=shared, on_gpu=H > 1024, zipf=zipf)
    x = np.random.default_rng(M + I).normal(0, 1, (M, H)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    assert P.moe_prepare(layer)
    try:
        y, sel, wts = P.moe_forward(layer, xd)
        sel_o, wts_o, gap = O.route(O.router_logits(x, d['rb']), d['bias'], topk)
        assert gap.min() > 1e-6
        assert np.array_equal(sel.cpu().numpy(), sel_o) and np.abs(wts.cpu().numpy() - wts_o).max() < 1e-5
        rows = list(range(M)) if H <= 1024 else [0, 1, M // 2, M - 1]         # full geometry: oracle on a few tokens' experts
        ex = host_experts(d, set(sel_o[rows].ravel().tolist()))
        sh = ex[E] if shared else None
        yo = O.moe_experts_act_nvfp4(x[rows], sel_o[rows], wts_o[rows], ex[:E], sh)
        yh = y.cpu().numpy()[rows]
        r, a = O.rel_l2(yh, yo), O.max_abs(yh, yo)
        assert r <= REL_TOL and a <= ABS_TOL, (r, a)
        exact = O.moe_experts(x[rows], sel_o[rows], wts_o[rows], ex[:E], sh)
        assert 0.02 < O.rel_l2(yh, exact) < 0.25
        with exact_prefill():
            y_exact, _, _ = P.moe_forward(layer, xd)
        assert O.rel_l2(y_exact.cpu().numpy()[rows], exact) <= REL_TOL
        assert torch.equal(P.moe_forward(layer, xd)[0], y)
        assert torch.equal(P.moe_experts(layer, xd, sel, wts), y)
        lo = M - 16
        y_sub, _, _ = P.moe_forward(layer, xd[lo:].contiguous())              # the last 16 tokens on their own
        assert O.rel_l2(y_sub.cpu().numpy(), y.cpu().numpy()[lo:]) < 1e-6
        assert P.device_status() == 0
    finally:
        P.moe_release(layer)


def test_moe_prepared_layer_under_graph_capture():
    """The prepared path only launches kernels (descriptor look-up is host-side), so a layer forward
    can be captured and replayed; small-batch and grouped paths."""
    P = pkg()
    layer, d = build_layer(1024, 512, 32, 8, seed=123)
    assert P.moe_prepare(layer)
    try:
        for M in (2, 19):
            x = torch.randn((M, 1024), device='cuda')
            want, sel_w, _ = P.moe_forward(layer, x)
            y = torch.zeros_like(want); sel = torch.zeros_like(sel_w); wts = torch.zeros((M, 8), device='cuda')
            st = torch.cuda.Stream()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(st):
                P.moe_forward(layer, x, y, sel, wts)          # warm-up on the capture stream (workspace, attributes)
                st.synchronize()
                with torch.cuda.graph(g, stream=st):
                    for _ in range(3): P.moe_forward(layer, x, y, sel, wts)
            y.zero_()
            g.replay(); g.replay()
            torch.cuda.synchronize()
            assert torch.equal(y, want) and torch.equal(sel, sel_w), M
        assert P.device_status() == 0
    finally:
        P.moe_release(layer)


def test_moe_prepare_refuses_unsuitable_geometry():
    P = pkg()
    layer, _ = build_layer(1056, 544, 8, 2, seed=3)   # not multiples of 256
    assert P.moe_prepare(layer) is False


def test_route_ties_lowest_index_wins():
    """Two experts with identical router rows and biases tie exactly; the lower index must be
    ranked first (reference kernels/moe.cu:146-152)."""
    P, O = pkg(), oracle()
    H, E, K = 256, 40, 4
    rng = np.random.default_rng(1)
    w = rng.normal(0, 0.05, (E, H)).astype(np.float32)
    w[33] = w[2]; w[17] = w[2]
    rb = O.f32_to_bf16_bits(w)
    bias = np.zeros(E, np.float32)
    x = rng.normal(0, 1, (3, H)).astype(np.float32)
    x[0] = w[2] * 40                                    # make the tied experts the top choice
    dummy = P.Nvfp4Weight(*host_triple((32, 32), 1))
    layer = P.MoeLayer(to_dev_bf16(rb), torch.from_numpy(bias).cuda(), [(dummy, dummy, dummy)] * E, None, K, H, 32)
    sel, wts, logits = P.moe_route(layer, torch.from_numpy(x).cuda())
    lo = O.router_logits(x, rb)
    assert O.rel_l2(logits.cpu().numpy(), lo) < 1e-5
    so, wo, _ = O.route(logits.cpu().numpy().astype(np.float64), bias, K)
    assert np.array_equal(sel.cpu().numpy(), so)
    assert list(sel[0, :3].tolist()) == [2, 17, 33]
    assert np.abs(wts.cpu().numpy() - wo).max() < 1e-5


def test_moe_expert_tensors_at_the_4_byte_floor():
    """The reference's checkpoint only guarantees 4-byte aligned packed tensors and scales at any address
    (kernels/moe.cu:167-174).  The CUDA-core experts must run from there and match the oracle; prepare
    (the tensor-core experts) declines such a layer instead of faulting."""
    P, O = pkg(), oracle()
    H, I, E, topk = 512, 256, 8, 2
    rng = np.random.default_rng(17)
    host = [(host_triple((I, H), 9000 + 3 * e), host_triple((I, H), 9001 + 3 * e), host_triple((H, I), 9002 + 3 * e)) for e in range(E + 1)]
    keep = []

    def shifted(t):
        p, s, gs = t
        pb = torch.zeros(p.size + 16, dtype=torch.uint8, device='cuda'); pb[4:4 + p.size] = torch.from_numpy(p).cuda().reshape(-1)
        sb = torch.zeros(s.size + 16, dtype=torch.uint8, device='cuda'); sb[1:1 + s.size] = torch.from_numpy(s).cuda().reshape(-1)
        keep.extend([pb, sb])
        return P.Nvfp4Weight(pb[4:4 + p.size].view(p.shape), sb[1:1 + s.size].view(s.shape), torch.from_numpy(gs).cuda())
    dev = [tuple(shifted(w) for w in t) for t in host]
    assert dev[0][0].packed.data_ptr() % 16 == 4 and dev[0][0].scale.data_ptr() % 2 == 1
    rb = O.f32_to_bf16_bits(rng.normal(0, 0.05, (E, H)).astype(np.float32))
    bias = rng.normal(0, 0.1, E).astype(np.float32)
    layer = P.MoeLayer(to_dev_bf16(rb), torch.from_numpy(bias).cuda(), dev[:E], dev[E], topk, H, I)
    d = dict(rb=rb, bias=bias, host=host, dev=dev, E=E, topk=topk, shared=True)
    x = rng.normal(0, 1, (3, H)).astype(np.float32)
    check_layer(layer, d, x)
    assert P.moe_prepare(layer) is False
    y, _, _ = P.moe_forward_static(layer, torch.from_numpy(x).cuda())
    assert torch.isfinite(y).all()
    assert P.device_status() == 0


def test_router_of_a_batch_equals_router_of_each_token_bitwise():
    """The one-launch router product for many tokens computes every (token, expert) logit exactly as the
    single-token call does, so a token's selection does not depend on how many tokens were routed together."""
    P = pkg()
    layer, d = build_layer(4096, 256, 144, 8, seed=77, on_gpu=True)
    x = torch.randn((45, 4096), device='cuda')
    sel, wts, logits = P.moe_route(layer, x)
    for m in (0, 7, 8, 23, 44):
        s1, w1, l1 = P.moe_route(layer, x[m:m + 1].contiguous())
        assert torch.equal(l1[0], logits[m]) and torch.equal(s1[0], sel[m]) and torch.equal(w1[0], wts[m]), m
    s8, w8, l8 = P.moe_route(layer, x[:8].contiguous())
    assert torch.equal(l8, logits[:8])


def test_byte_credit_reports_what_each_call_streams():
    """The profiler hook: host-known counts at the launch sites, device-side job counts after a flush
    (the contract of the reference's dprof_bytes / dprof_set_flush, include/dprof.h:83-103)."""
    P = pkg()
    H, I, E, topk = 1024, 512, 16, 2
    layer, d = build_layer(H, I, E, topk, seed=11)
    W = P.Nvfp4Weight(*host_triple((300, 1024), 5))
    per = I * H * 0.5625
    with P.ByteCredit() as bc:
        P.gemm(W, torch.randn(1, 1024, device='cuda'))
        assert bc.by_kind == {0: 300 * 1024 * 0.5625}
        P.gemm(W, torch.randn(20, 1024, device='cuda'))                  # three passes of up to 8 rows
        assert bc.by_kind[0] == 4 * 300 * 1024 * 0.5625
        bc.by_kind.clear()
        P.moe_forward(layer, torch.randn(3, H, device='cuda'))           # CUDA-core experts: every pair streams its expert
        assert bc.by_kind[2] == 3 * (topk + 1) * 2 * per and bc.by_kind[3] == 3 * (topk + 1) * per
        assert bc.by_kind[0] == E * H * 2.0                              # the bf16 router
        assert P.moe_prepare(layer)
        try:
            bc.by_kind.clear()
            x = torch.randn(40, H, device='cuda')
            _, sel, _ = P.moe_forward(layer, x)                          # grouped on the device: known after the flush
            assert 2 not in bc.by_kind
            bc.flush()
            distinct = len(set(sel.cpu().numpy().ravel().tolist())) + 1
            jobs = bc.by_kind[3] / per
            assert distinct <= jobs <= distinct + 40 * (topk + 1) / 32 and bc.by_kind[2] == 2 * bc.by_kind[3]
            bc.by_kind.clear()
            P.moe_forward(layer, x); bc.flush(credit=False); bc.flush()  # a discarded warm-up is not billed later
            assert bc.by_kind.get(3, 0.0) == 0.0
        finally:
            P.moe_release(layer)
