"""GPU parity: every CUDA entry point, called through the C ABI, against the CPU oracle.

Bar: codes, scales and global scales bit-exact; gemv / gemm / MoE outputs within rel-L2 1e-3 and
max-abs 2e-2 of an fp64-accumulated dequant-then-matmul; expert selection identical as a set,
gate weights within 1e-5.  Structural checks follow the reference's own gates
(tests/gate_nvfp4.cu:114-125, tests/gate_gemv_multi.cu:104-128): a gemm row equals the gemv of
that row bit for bit, a fused group equals its separate gemvs bit for bit, outputs are
poison-filled first, and an all-zero result does not count as agreement.
"""
import ctypes as C
import numpy as np
import pytest
import torch

from util import (pkg, oracle, seeded_bf16, host_triple, to_dev_bf16, ref_kernels, REL_TOL, ABS_TOL)

pytestmark = pytest.mark.gpu


def dev_weight(t):
    return pkg().Nvfp4Weight(*t)


def close(y, ref):
    O = oracle()
    r, a = O.rel_l2(y, ref), O.max_abs(y, ref)
    assert r <= REL_TOL and a <= ABS_TOL, (r, a)
    assert np.abs(np.asarray(ref)).max() > 0
    return r


# ---- quantiser ---------------------------------------------------------------------------------

def _quant_case(bits):
    P, O = pkg(), oracle()
    W = P.quantize(to_dev_bf16(bits))
    torch.cuda.synchronize()
    p, s, gs = O.quantize_tensor(O.bf16_bits_to_f32(bits))
    gp, gsc, ggs = W.numpy()
    assert ggs.view(np.uint32)[0] == gs.view(np.uint32)[0]
    assert np.array_equal(gsc, s)
    assert np.array_equal(gp, p)
    return W, (p, s, gs)


def test_quantize_golden_bit_exact(golden):
    for name, tags in (('quant_normal', ['w%d' % i for i in range(5)]), ('quant_edges', list('abcde'))):
        z = golden(name)
        for t in tags:
            W, _ = _quant_case(z[t + '_bits'])
            gp, gsc, ggs = W.numpy()
            assert np.array_equal(gp, z[t + '_packed']) and np.array_equal(gsc, z[t + '_scale']), t
            assert ggs.view(np.uint32)[0] == z[t + '_gs'].view(np.uint32)[0], t
            d = pkg().dequantize(W).cpu().numpy()
            assert np.array_equal(d.view(np.uint32), z[t + '_deq'].view(np.uint32)), t


@pytest.mark.parametrize('shape', [(1, 16), (3, 48), (257, 1536), (1024, 4096), (0, 64)])
def test_quantize_random_bit_exact(shape):
    _quant_case(seeded_bf16(shape, 11 + shape[0]))


def test_quantize_wide_range_and_unaligned():
    rng = np.random.default_rng(5)
    w = (np.exp(rng.uniform(-20, 8, (64, 512))) * rng.choice([-1.0, 1.0], (64, 512))).astype(np.float32)
    w[rng.random((64, 512)) < 0.1] = 0.0
    bits = oracle().f32_to_bf16_bits(w)
    _quant_case(bits)
    # an input that starts 2 bytes past a 16-byte boundary takes the scalar load path
    P, O = pkg(), oracle()
    buf = torch.zeros(64 * 512 + 1, dtype=torch.bfloat16, device='cuda')
    buf[1:] = to_dev_bf16(bits).reshape(-1)
    W = P.quantize(buf[1:].view(64, 512))
    p, s, gs = O.quantize_tensor(O.bf16_bits_to_f32(bits))
    gp, gsc, ggs = W.numpy()
    assert np.array_equal(gp, p) and np.array_equal(gsc, s) and ggs[0] == gs[0]


def test_quantize_with_given_scale():
    P, O = pkg(), oracle()
    bits = seeded_bf16((32, 256), 3, std=1.0)
    gs = np.array([37.5], np.float32)
    W = P.quantize(to_dev_bf16(bits), gscale_in=torch.from_numpy(gs).cuda())
    p, s = O.quantize(O.bf16_bits_to_f32(bits), gs[0])
    assert np.array_equal(W.packed.cpu().numpy(), p) and np.array_equal(W.scale.cpu().numpy(), s)


def test_quantize_full_size_properties():
    """[12288 x 4096]: compared in full with the C oracle, plus the round-trip error band the
    reference records for this format (rel 0.088-0.100)."""
    import ctypes as C
    from util import c_oracle
    P, O = pkg(), oracle()
    bits = seeded_bf16((12288, 4096), 1000)
    W = P.quantize(to_dev_bf16(bits))
    L = c_oracle()
    gs = L.oracle_global_scale(bits.ctypes.data_as(C.c_void_p), bits.size)
    p = np.zeros((12288, 2048), np.uint8); s = np.zeros((12288, 256), np.uint8)
    L.oracle_quantize(bits.ctypes.data_as(C.c_void_p), 12288, 4096, C.c_float(gs), p.ctypes.data_as(C.c_void_p),
                      s.ctypes.data_as(C.c_void_p))
    gp, gsc, ggs = W.numpy()
    assert ggs[0] == np.float32(gs) and np.array_equal(gsc, s) and np.array_equal(gp, p)
    d = P.dequantize(W)
    w = to_dev_bf16(bits).float()
    rel = ((d - w).norm() / w.norm()).item()
    assert 0.085 < rel < 0.102, rel


# ---- gemv / gemm -------------------------------------------------------------------------------

GEMV_SHAPES = [(1, 96, 512), (1, 1, 32), (1, 5, 128), (2, 33, 1536), (3, 70, 4096), (4, 130, 1024),
               (5, 64, 2048), (6, 40, 96), (7, 17, 4096), (8, 257, 1536), (1, 300, 12288), (8, 64, 12288),
               (1, 9, 16), (4, 21, 48), (8, 12, 80)]           # the last three take the generic kernel


@pytest.mark.parametrize('M,N,K', GEMV_SHAPES)
def test_gemm_vs_oracle(M, N, K):
    P, O = pkg(), oracle()
    t = host_triple((N, K), 100 + N + K)
    x = np.random.default_rng(7 + M).normal(0, 1, (M, K)).astype(np.float32)
    y = torch.full((M, N), float('nan'), device='cuda')
    P.gemm(dev_weight(t), torch.from_numpy(x).cuda(), y)
    close(y.cpu().numpy(), O.gemm(x, *t))


def test_gemv_golden(golden):
    z = golden('gemv')
    for i in range(3):
        t = (z['g%d_packed' % i], z['g%d_scale' % i], z['g%d_gs' % i])
        y = pkg().gemm(dev_weight(t), torch.from_numpy(z['g%d_x' % i]).cuda()).cpu().numpy()
        close(y, z['g%d_y' % i])


def test_gemm_large_M_chunks():
    P, O = pkg(), oracle()
    t = host_triple((48, 512), 5)
    x = np.random.default_rng(8).normal(0, 1, (19, 512)).astype(np.float32)
    W = dev_weight(t)
    y = P.gemm(W, torch.from_numpy(x).cuda())
    close(y.cpu().numpy(), O.gemm(x, *t))
    for m in (0, 7, 8, 18):
        assert torch.equal(P.gemm(W, torch.from_numpy(x[m:m + 1]).cuda())[0], y[m])


def test_gemm_rows_equal_gemv_bitwise():
    P = pkg()
    for (N, K) in [(300, 4096), (64, 1536), (33, 128)]:
        W = dev_weight(host_triple((N, K), N))
        x = torch.from_numpy(np.random.default_rng(N).normal(0, 1, (8, K)).astype(np.float32)).cuda()
        for M in (1, 2, 3, 4, 5, 8):
            y = P.gemm(W, x[:M].contiguous())
            for m in range(M):
                ym = P.gemm(W, x[m:m + 1].contiguous())
                assert torch.equal(y[m], ym[0]), (N, K, M, m)
            assert (y != 0).float().mean() > 0.5


def test_pipelined_and_general_kernels_agree_bitwise(monkeypatch):
    """The two CUDA-core kernels (the fallback path when the tensor-core kernel cannot take a
    shape): M = 1 with K % 256 == 0 runs the bulk-copy pipelined kernel, everything else the
    general kernel.  Both must give the same bits, or a gemm row would differ from its gemv."""
    P = pkg()
    monkeypatch.setenv('B200_NVFP4_UMMA', '0')
    for (N, K) in [(12288, 4096), (1000, 4096), (700, 1536), (515, 256), (4096, 2048)]:
        W = dev_weight(host_triple((min(N, 1024), K), N + K)) if N <= 1024 else P.quantize(
            (torch.randn((N, K), device='cuda') * 0.02).to(torch.bfloat16))
        x = torch.randn(1, K, device='cuda')
        monkeypatch.setenv('B200_NVFP4_GENERAL', '1')
        a = P.gemm(W, x)
        monkeypatch.setenv('B200_NVFP4_GENERAL', '0')
        b = torch.full_like(a, float('nan'))
        P.gemm(W, x, b)
        assert torch.equal(a, b), (N, K)
        assert (a != 0).float().mean() > 0.9
    assert P.device_status() == 0


# ---- tensor-core kernel (K % 256 == 0, 16-byte aligned operands) ------------------------------------

@pytest.mark.parametrize('N,K,M', [(512, 256, 1), (1000, 4096, 1), (4096, 1024, 3), (700, 1536, 8), (32, 4096, 1),
                                   (64, 2048, 5), (300, 16384, 8), (300, 12288, 1), (20000, 512, 2), (129, 7168, 4),
                                   (40000, 512, 1), (40000, 256, 3)])
def test_tensor_core_gemv_vs_oracle_and_row_invariance(N, K, M):
    """Every shape class of the tensor-core kernel: several steps per stage (K up to 16384, where
    the activation rows are taken in chunks), swizzled and plain scale slabs (K/16 a multiple of
    128 or not), row tiles of 8..128, more tiles than SMs (several tiles per CTA from twice the SM
    count on).  Each row must also equal the
    single-row call bit for bit, whatever chunking or tile height the batched call used."""
    P, O = pkg(), oracle()
    t = host_triple((N, K), N + K + M)
    W = dev_weight(t)
    x = np.random.default_rng(N + M).normal(0, 1, (M, K)).astype(np.float32)
    x[M - 1] *= 37.0
    xd = torch.from_numpy(x).cuda()
    y = torch.full((M, N), float('nan'), device='cuda')
    P.gemm(W, xd, y)
    ref = O.gemm(x, *t)
    for m in range(M):
        assert O.rel_l2(y[m].cpu().numpy(), ref[m]) <= REL_TOL, m
        y1 = torch.full((1, N), float('nan'), device='cuda')
        P.gemm(W, xd[m:m + 1].contiguous(), y1)
        assert torch.equal(y[m], y1[0]), m
    assert P.device_status() == 0


def test_many_wave_tiling_equals_single_tile_rows_bitwise():
    """A projection with more than two waves of 128-row tiles is cut into CTAs of T tiles of R rows chosen by
    estimated time; a row's result must not depend on that: rows [r0, r0 + n) of the big product equal the product
    with those rows alone (one tile per CTA, another kernel variant) bit for bit, and both match the oracle."""
    P, O = pkg(), oracle()
    N, K, r0, n = 40000, 4096, 12345 - 12345 % 8, 2048
    t = host_triple((N, K), 91)
    W = dev_weight(t)
    x = np.random.default_rng(92).normal(0, 1, (1, K)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    y = torch.full((1, N), float('nan'), device='cuda')
    P.gemm(W, xd, y)
    sub = P.Nvfp4Weight(W.packed[r0:r0 + n], W.scale[r0:r0 + n], W.gscale)
    ys = torch.full((1, n), float('nan'), device='cuda')
    P.gemm(sub, xd, ys)
    assert torch.equal(y[0, r0:r0 + n], ys[0])
    ref = O.gemm(x, t[0][r0:r0 + n], t[1][r0:r0 + n], t[2])
    close(ys.cpu().numpy(), ref)
    assert P.device_status() == 0


@pytest.mark.parametrize('N,K,M', [(1000, 4096, 2), (4096, 1024, 8), (700, 1536, 5), (300, 2048, 20), (129, 4096, 64), (300, 16384, 8), (129, 7168, 4)])
def test_presplit_workspace_calls_equal_plain_calls_bitwise(N, K, M):
    """b200_nvfp4_gemm_ws / gemv_multi_ws split the activation rows once into caller scratch; the
    result must not differ from the plain calls in a single bit, also where the scratch cannot be
    used (K = 16384: the image does not fit; K = 7168: CUDA-core path)."""
    P = pkg()
    W = dev_weight(host_triple((N, K), N + K + M))
    x = torch.randn((M, K), device='cuda')
    x[M - 1] *= 29.0
    ws = P.split_workspace(M, K, x.device)
    want = P.gemm(W, x)
    got = torch.full_like(want, float('nan'))
    P.set_option(P.OPT_PREFILL_FP4, 0)               # from 16 rows on the scratch call would otherwise take the wide GEMM
    try:
        P.gemm(W, x, got, ws=ws)
    finally:
        P.set_option(P.OPT_PREFILL_FP4, 1)
    if M >= 16 and K % 256 == 0 and K <= 16384:
        # the scratch call runs the exact wide GEMM (f32 rows rounded to fp16 once): same product, not the same bits
        assert ((got - want).norm() / want.norm()).item() <= 4e-4
    else:
        assert torch.equal(got, want)
    if M <= 8:
        W2 = dev_weight(host_triple((64, K), 7 + K))
        ys = P.gemv_multi([W, W2], x, M)
        ys_ws = [torch.full_like(y, float('nan')) for y in ys]
        P.gemv_multi([W, W2], x, M, ys_ws, ws=ws)
        for a, b in zip(ys, ys_ws): assert torch.equal(a, b)
        assert torch.equal(ys[0], want)
    assert (want != 0).float().mean() > 0.5
    assert P.device_status() == 0


@pytest.mark.parametrize('N,K,M', [(300, 16384, 8), (1000, 4096, 5), (64, 12288, 8)])
def test_cuda_core_fallback_row_invariance(monkeypatch, N, K, M):
    """With the tensor-core kernel off, the CUDA-core kernels must keep the same invariant, also where
    the staged activations of all M rows do not fit shared memory (the rows then go in chunks; the
    kernel that computes a row must never depend on M)."""
    monkeypatch.setenv('B200_NVFP4_UMMA', '0')
    P, O = pkg(), oracle()
    t_ = host_triple((N, K), N + K)
    W = dev_weight(t_)
    x = torch.randn((M, K), device='cuda')
    y = P.gemm(W, x)
    close(y.cpu().numpy(), O.gemm(x.cpu().numpy(), *t_))
    for m in (0, M - 1):
        assert torch.equal(P.gemm(W, x[m:m + 1].contiguous())[0], y[m]), m
    ws = P.split_workspace(M, K, x.device)
    assert torch.equal(P.gemm(W, x, ws=ws), y)       # the scratch variant follows the same switch


def test_tensor_core_and_cuda_core_kernels_agree_within_tolerance(monkeypatch):
    """Not bit for bit (the tensor-core kernel rounds activations to 14 fractional bits of the
    row maximum, the CUDA-core kernels to fp16): both within the tolerance of the oracle, and of
    one another."""
    P, O = pkg(), oracle()
    t = host_triple((777, 2048), 5)
    W = dev_weight(t)
    x = torch.randn(3, 2048, device='cuda')
    a = P.gemm(W, x).cpu().numpy()
    monkeypatch.setenv('B200_NVFP4_UMMA', '0')
    b = P.gemm(W, x).cpu().numpy()
    assert not np.array_equal(a, b)                  # two different kernels did run
    assert O.rel_l2(a, b) <= REL_TOL
    ref = O.gemm(x.cpu().numpy(), *t)
    assert O.rel_l2(a, ref) < O.rel_l2(b, ref)       # and the tensor-core one is the finer of the two


def test_tensor_core_kernel_in_a_cuda_graph_chain():
    """Back-to-back launches without host gaps (graph replay, programmatic dependent launch): a
    late asynchronous barrier arrival of one CTA must not land in the next CTA's shared memory."""
    P = pkg()
    Ws = [P.quantize((torch.randn((4096, 4096), device='cuda') * 0.02).to(torch.bfloat16)) for _ in range(3)]
    x = torch.randn(1, 4096, device='cuda')
    want = [P.gemm(W, x) for W in Ws]
    ys = [torch.empty_like(w) for w in want]
    P.set_option(P.OPT_STABLE_WEIGHTS, 1)
    try:
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            for _ in range(2):                       # warm-up on the capture stream
                for W, y in zip(Ws, ys): P.gemm(W, x, y)
            st.synchronize()
            with torch.cuda.graph(g, stream=st):
                for _ in range(8):
                    for W, y in zip(Ws, ys): P.gemm(W, x, y)
        for _ in range(5): g.replay()
        torch.cuda.synchronize()
    finally:
        P.set_option(P.OPT_STABLE_WEIGHTS, 0)
    assert P.device_status() == 0
    for y, w in zip(ys, want): assert torch.equal(y, w)


def test_gemv_run_to_run_identical():
    P = pkg()
    W = dev_weight(host_triple((1000, 4096), 1))
    x = torch.randn(1, 4096, device='cuda')
    a = P.gemm(W, x)
    for _ in range(3):
        assert torch.equal(P.gemm(W, x), a)


def test_gemv_extreme_activation_ranges():
    """The fp16 staging is scaled per row, so huge, tiny and zero rows must all stay exact to
    the same relative tolerance."""
    P, O = pkg(), oracle()
    t = host_triple((64, 1024), 21)
    rng = np.random.default_rng(3)
    x = rng.normal(0, 1, (4, 1024)).astype(np.float32)
    x[0] *= 1e6; x[1] *= 1e-6; x[2] = 0.0; x[3, ::2] *= 1e-4
    y = P.gemm(dev_weight(t), torch.from_numpy(x).cuda()).cpu().numpy()
    ref = O.gemm(x, *t)
    for m in (0, 1, 3):
        assert O.rel_l2(y[m], ref[m]) <= REL_TOL, m
    assert np.all(y[2] == 0)


def test_gemv_unaligned_tensors_take_generic_path():
    P, O = pkg(), oracle()
    p, s, gs = host_triple((40, 256), 2)
    x = np.random.default_rng(1).normal(0, 1, (2, 256)).astype(np.float32)
    buf = torch.zeros(p.size + 4, dtype=torch.uint8, device='cuda')
    buf[4:] = torch.from_numpy(p).cuda().reshape(-1)            # 4-byte aligned only
    sbuf = torch.zeros(s.size + 1, dtype=torch.uint8, device='cuda')
    sbuf[1:] = torch.from_numpy(s).cuda().reshape(-1)           # odd address
    W = P.Nvfp4Weight(buf[4:].view(40, 128), sbuf[1:].view(40, 16), torch.from_numpy(gs).cuda())
    y = P.gemm(W, torch.from_numpy(x).cuda()).cpu().numpy()
    close(y, O.gemm(x, p, s, gs))


def test_dense_bf16_f32_gemm():
    P, O = pkg(), oracle()
    rng = np.random.default_rng(4)
    for (M, N, K) in [(1, 144, 4096), (4, 144, 4096), (3, 10, 100), (9, 7, 64)]:
        w = rng.normal(0, 0.02, (N, K)).astype(np.float32)
        x = rng.normal(0, 1, (M, K)).astype(np.float32)
        wb = O.f32_to_bf16_bits(w)
        y = P.gemm(to_dev_bf16(wb), torch.from_numpy(x).cuda()).cpu().numpy()
        ref = x.astype(np.float64) @ O.bf16_bits_to_f32(wb).astype(np.float64).T
        assert O.rel_l2(y, ref) < 1e-5
        y = P.gemm(torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda()).cpu().numpy()
        assert O.rel_l2(y, x.astype(np.float64) @ w.astype(np.float64).T) < 1e-5


def test_converters():
    P = pkg()
    x = torch.randn(1000, device='cuda')
    b = P.f32_to_bf16(x)
    assert torch.equal(b, x.to(torch.bfloat16))
    assert torch.equal(P.bf16_to_f32(b), b.float())


# ---- fused sibling gemvs -------------------------------------------------------------------------

SIBLINGS = [4096, 4096, 4096, 512, 64, 32]


@pytest.mark.parametrize('M', [1, 2, 4, 8])
def test_gemv_multi_siblings(M):
    """Six weights sharing one input, K = 4096: one launch, bit-identical to six separate calls,
    and within tolerance of the oracle."""
    P, O = pkg(), oracle()
    K = 4096
    ts = [host_triple((n, K), 1000 + i) for i, n in enumerate(SIBLINGS)]
    Ws = [dev_weight(t) for t in ts]
    xh = np.random.default_rng(2).normal(0, 1, (M, K)).astype(np.float32)
    x = torch.from_numpy(xh).cuda()
    ys = [torch.full((M, n), float('nan'), device='cuda') for n in SIBLINGS]
    P.gemv_multi(Ws, x, M, ys)
    for W, t, y in zip(Ws, ts, ys):
        sep = torch.full_like(y, float('inf'))
        P.gemm(W, x, sep)
        assert torch.equal(sep, y)
        close(y.cpu().numpy(), O.gemm(xh, *t))


def test_gemv_multi_per_job_inputs_and_ragged():
    P, O = pkg(), oracle()
    K = 128
    shapes = [130, 7, 64]
    ts = [host_triple((n, K), 50 + i) for i, n in enumerate(shapes)]
    Ws = [dev_weight(t) for t in ts]
    xs_h = [np.random.default_rng(60 + i).normal(0, 1, (1, K)).astype(np.float32) for i in range(3)]
    xs = [torch.from_numpy(a).cuda() for a in xs_h]
    ys = P.gemv_multi(Ws, xs, 1)
    for W, t, xh, x, y in zip(Ws, ts, xs_h, xs, ys):
        assert torch.equal(P.gemm(W, x), y)
        close(y.cpu().numpy(), O.gemm(xh, *t))


def test_gemv_multi_eight_jobs():
    P = pkg()
    K = 512
    Ws = [dev_weight(host_triple((16 + 9 * i, K), 70 + i)) for i in range(8)]
    x = torch.randn(2, K, device='cuda')
    ys = P.gemv_multi(Ws, x, 2)
    for W, y in zip(Ws, ys):
        assert torch.equal(P.gemm(W, x), y)


def test_error_codes_on_device_pointers():
    P = pkg()
    W = dev_weight(host_triple((8, 32), 1))
    x = torch.randn(1, 40, device='cuda')
    y = torch.empty(1, 8, device='cuda')
    ref = W.wref()
    rc = P.lib().b200_nvfp4_gemm(C.c_void_p(y.data_ptr()), C.byref(ref), C.c_void_p(x.data_ptr()), 1, 8, 40, 1, None)
    assert rc == 2
    with pytest.raises(P.B200Error):
        P.check(rc, 'gemm')


# ---- against the reference's own kernels on the same buffers ---------------------------------------

def test_gemv_vs_reference_kernel():
    R = ref_kernels()
    if R is None:
        pytest.skip('oracle/_ref/libref_kernels.so was not prebuilt')
    P, O = pkg(), oracle()
    for (M, N, K) in [(1, 1000, 4096), (4, 333, 1536), (1, 64, 128)]:
        W = dev_weight(host_triple((N, K), N + K))
        x = torch.randn(M, K, device='cuda')
        y = P.gemm(W, x)
        yr = torch.zeros_like(y)
        R.ref_gemm_nvfp4(y_ptr(yr), y_ptr(W.packed), y_ptr(W.scale), y_ptr(W.gscale), y_ptr(x), M, N, K, None)
        torch.cuda.synchronize()
        close(y.cpu().numpy(), yr.cpu().numpy())


def y_ptr(t):
    return C.c_void_p(t.data_ptr())


# ---- dense-layer MLP and the linear-attention sibling groups at their real shapes -------------------

@pytest.mark.parametrize('M,H,I', [(1, 1024, 3072), (3, 512, 768), (1, 4096, 12288)])
def test_dense_mlp_vs_oracle(M, H, I):
    """gate/up as one fused launch, clamped SwiGLU, down (reference kernels/layer.cu:235-254)."""
    P, O = pkg(), oracle()
    big = H == 4096
    if big:
        Ws = [P.quantize(to_dev_bf16(seeded_bf16(sh, 500 + i))) for i, sh in enumerate([(I, H), (I, H), (H, I)])]
        ts = [W.numpy() for W in Ws]
    else:
        ts = [host_triple((I, H), 31), host_triple((I, H), 32), host_triple((H, I), 33)]
        Ws = [dev_weight(t) for t in ts]
    x = (np.random.default_rng(M).normal(0, 1, (M, H)) * 30).astype(np.float32)      # large enough to reach the clamps
    y = P.dense_mlp(torch.from_numpy(x).cuda(), *Ws, limit=10.0).cpu().numpy()
    ref, act = O.expert_mlp(x, *ts, limit=10.0)
    assert np.abs(act).max() > 50                     # the clamps are active
    r = O.rel_l2(y, ref)
    assert r <= REL_TOL, r
    assert P.device_status() == 0


@pytest.mark.parametrize('Ns,K,own_x', [([8192, 8192, 8192], 4096, False), ([128, 128, 64], 4096, False), ([8192, 8192], 128, True)])
def test_kda_sibling_groups_real_shapes(Ns, K, own_x):
    """The fused groups of the linear-attention layer (reference kernels/kda.cu:235-266,
    tests/gate_gemv_multi.cu:54-61): fused == separate bit for bit, and within tolerance of the oracle."""
    P, O = pkg(), oracle()
    Ws = [P.quantize(to_dev_bf16(seeded_bf16((n, K), 600 + i))) for i, n in enumerate(Ns)]
    rng = np.random.default_rng(K)
    xh = [rng.normal(0, 1, (1, K)).astype(np.float32) for _ in Ns] if own_x else [rng.normal(0, 1, (1, K)).astype(np.float32)] * len(Ns)
    xs = [torch.from_numpy(a).cuda() for a in xh]
    ys = P.gemv_multi(Ws, xs, 1)
    for W, x, xa, y in zip(Ws, xs, xh, ys):
        assert torch.equal(P.gemm(W, x), y)
        rows = slice(0, 512)                              # oracle on the first rows keeps the CPU side short
        p, s, gs = W.numpy()
        close(y.cpu().numpy()[:, rows], O.gemm(xa, p[rows], s[rows], gs))
    assert P.device_status() == 0


# ---- robustness ------------------------------------------------------------------------------------

def test_bounded_wait_runs_out_and_reports():
    """A kernel whose wait can never be satisfied gives up after its limit, the kernel returns, the status
    word names the site, and the context stays usable (no trap, no hang)."""
    P = pkg()
    P.device_status(clear=True)
    assert P.device_status() == 0
    P.check(P.lib().b200_nvfp4_selftest_bounded_wait(None), 'selftest')
    torch.cuda.synchronize()
    st = P.device_status(clear=True)
    assert st >> 16 == 15 and (st & 0xffff) == 0, hex(st)
    assert P.device_status() == 0
    W = dev_weight(host_triple((64, 256), 3))            # the context still works
    x = torch.randn(1, 256, device='cuda')
    assert torch.isfinite(P.gemm(W, x)).all()


@pytest.mark.parametrize('umma', ['1', '0'])
def test_non_finite_activations_propagate(monkeypatch, umma):
    """A NaN or an infinity in an activation row must not vanish: every output of that row is non-finite on
    the tensor-core path and on the CUDA-core path alike; other rows are untouched."""
    monkeypatch.setenv('B200_NVFP4_UMMA', umma)
    P, O = pkg(), oracle()
    t = host_triple((300, 1024), 9)
    W = dev_weight(t)
    x = np.random.default_rng(2).normal(0, 1, (3, 1024)).astype(np.float32)
    x[0, 17] = np.nan; x[1, 900] = np.inf
    y = P.gemm(W, torch.from_numpy(x).cuda()).cpu().numpy()
    assert not np.isfinite(y[0]).any() and not np.isfinite(y[1]).any()
    assert O.rel_l2(y[2], O.gemm(x[2:3], *t)[0]) <= REL_TOL
    # the wide GEMM as well
    xb = torch.from_numpy(x).cuda().to(torch.bfloat16)
    yw = P.gemm_bf16(W, xb).cpu().numpy()
    assert not np.isfinite(yw[0]).any() and not np.isfinite(yw[1]).any() and np.isfinite(yw[2]).all()
