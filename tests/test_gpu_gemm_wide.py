"""GPU parity of the wide GEMM (both operands in NVFP4, tcgen05.mma kind::mxf4nvf4), called through
the C ABI, against the CPU oracle.

Bar: the per-token activation codes, scales and global scales bit-exact with the oracle's
quantize_rows (the reference's quant_block per row); outputs within rel-L2 1e-3 and max-abs 2e-2 of
O_wa = deq(W) . deq(quant(x)), fp64-accumulated.  The distance from the exact product O_w is reported
and bounded from both sides (4-bit activations cost a few per cent; a result "too close" to O_w would
mean the wrong kernel ran)."""
import numpy as np
import pytest
import torch

from util import pkg, oracle, seeded_bf16, host_triple, to_dev_bf16, REL_TOL, ABS_TOL

pytestmark = pytest.mark.gpu


def bf16_rows(M, K, seed, spread=True):
    O = oracle()
    rng = np.random.default_rng(seed)
    x = rng.normal(0, 1, (M, K))
    if spread:
        x = x * np.exp(rng.uniform(-2, 2, (M, 1)))            # tokens of very different magnitude
    return O.f32_to_bf16_bits(x.astype(np.float32))


def close(y, ref):
    O = oracle()
    r, a = O.rel_l2(y, ref), O.max_abs(y, ref)
    assert r <= REL_TOL and a <= ABS_TOL * max(1.0, float(np.abs(ref).max())), (r, a)
    assert np.abs(np.asarray(ref)).max() > 0
    return r


@pytest.mark.parametrize('M,K,f32', [(5, 256, False), (33, 512, False), (128, 4096, False), (40, 1536, True), (7, 12288, True)])
def test_quantize_tokens_bit_exact(M, K, f32):
    P, O = pkg(), oracle()
    bits = bf16_rows(M, K, M + K)
    xf = O.bf16_bits_to_f32(bits)
    if f32:
        xf = (xf * np.float32(1.0009765625) + np.float32(1e-3)).astype(np.float32)      # not bf16-representable
        xd = torch.from_numpy(xf).cuda()
    else:
        xd = to_dev_bf16(bits)
    p, s, gs = P.quantize_tokens(xd)
    rp, rs, rgs = O.quantize_rows(xf)
    assert np.array_equal(gs.cpu().numpy().view(np.uint32), rgs.view(np.uint32))
    assert np.array_equal(s.cpu().numpy(), rs)
    assert np.array_equal(p.cpu().numpy(), rp)


def test_quantize_tokens_golden(golden):
    P = pkg()
    z = golden('gemm_act')
    for i in range(2):
        p, s, gs = P.quantize_tokens(to_dev_bf16(z['a%d_xbits' % i]))
        assert np.array_equal(p.cpu().numpy(), z['a%d_xpacked' % i]) and np.array_equal(s.cpu().numpy(), z['a%d_xscale' % i])
        assert np.array_equal(gs.cpu().numpy().view(np.uint32), z['a%d_xgs' % i].view(np.uint32))


def test_quantize_tokens_zero_and_edge_rows():
    P, O = pkg(), oracle()
    x = np.zeros((4, 256), np.float32)
    x[1, 5] = -0.0; x[2] = 3.0; x[3, ::16] = np.float32(6.0); x[3, 1::16] = np.float32(0.75)    # zero row; -0; constant; ties
    p, s, gs = P.quantize_tokens(torch.from_numpy(x).cuda())
    rp, rs, rgs = O.quantize_rows(x)
    assert np.array_equal(p.cpu().numpy(), rp) and np.array_equal(s.cpu().numpy(), rs)
    assert np.array_equal(gs.cpu().numpy().view(np.uint32), rgs.view(np.uint32))


def test_gemm_bf16_golden(golden):
    P = pkg()
    z = golden('gemm_act')
    for i in range(2):
        W = P.Nvfp4Weight(z['a%d_packed' % i], z['a%d_scale' % i], z['a%d_gs' % i])
        y = P.gemm_bf16(W, to_dev_bf16(z['a%d_xbits' % i])).cpu().numpy()
        close(y, z['a%d_y' % i])


# token tiles of 32, 64, 128 and 256 columns; several token tiles; ragged N (last weight tile partly
# out of range); K/16 a multiple of 128 (swizzled scale slabs) or not (K = 512, 1536); K up to 12288
WIDE_SHAPES = [(16, 300, 512), (1, 64, 256), (33, 1000, 1024), (100, 257, 1536), (129, 700, 4096), (300, 130, 2048),
               (512, 256, 4096), (64, 64, 12288), (257, 40, 256), (20, 20000, 512), (48, 4096, 1536), (600, 200, 1536)]


@pytest.mark.parametrize('M,N,K', WIDE_SHAPES)
def test_gemm_bf16_vs_oracle(M, N, K):
    P, O = pkg(), oracle()
    t = host_triple((N, K), 300 + N + K)
    bits = bf16_rows(M, K, 9 + M)
    y = torch.full((M, N), float('nan'), device='cuda')
    P.gemm_bf16(P.Nvfp4Weight(*t), to_dev_bf16(bits), y)
    yh = y.cpu().numpy()
    x = O.bf16_bits_to_f32(bits)
    close(yh, O.gemm_act_nvfp4(x, *t))
    dev = O.rel_l2(yh, O.gemm(x, *t))
    assert 0.02 < dev < 0.2, dev                     # 4-bit activations: a few per cent off the exact product
    assert P.device_status() == 0


def test_gemm_bf16_token_independent_of_batch():
    """A token's row must not depend on the rest of the batch (its own global scale, its own MMA column)."""
    P = pkg()
    W = P.Nvfp4Weight(*host_triple((500, 1024), 77))
    x = to_dev_bf16(bf16_rows(300, 1024, 5))
    y = P.gemm_bf16(W, x)
    for rows in ([0], [7, 8, 9], list(range(100, 140)), [299]):
        sub = P.gemm_bf16(W, x[rows].contiguous())
        assert torch.equal(sub, y[rows]), rows
    assert torch.equal(P.gemm_bf16(W, x), y)         # and run-to-run identical


def test_gemm_ws_f32_rows_dispatch_and_exact_option():
    """b200_nvfp4_gemm_ws with 16 or more rows takes the wide GEMM (f32 rows quantised per token); with
    B200_OPT_PREFILL_FP4 = 0 it keeps fp32-activation accuracy and equals the plain call bit for bit."""
    P, O = pkg(), oracle()
    t = host_triple((300, 2048), 41)
    W = P.Nvfp4Weight(*t)
    x = torch.randn((40, 2048), device='cuda')
    ws = P.split_workspace(40, 2048, x.device)
    y = P.gemm(W, x, ws=ws).cpu().numpy()
    xh = x.cpu().numpy()
    close(y, O.gemm_act_nvfp4(xh, *t))
    assert O.rel_l2(y, O.gemm(xh, *t)) > 0.02
    P.set_option(P.OPT_PREFILL_FP4, 0)               # exact products: the f16 wide GEMM (f32 rows rounded to fp16 once)
    try:
        y0 = P.gemm(W, x, ws=ws)
    finally:
        P.set_option(P.OPT_PREFILL_FP4, 1)
    r0 = O.rel_l2(y0.cpu().numpy(), O.gemm(xh, *t))
    assert r0 <= 4e-4, r0
    assert O.rel_l2(y0.cpu().numpy(), P.gemm(W, x).cpu().numpy()) <= 4e-4
    # below 16 rows the scratch call is always the exact one
    assert torch.equal(P.gemm(W, x[:15].contiguous(), ws=ws), P.gemm(W, x[:15].contiguous()))


@pytest.fixture(scope='module')
def big():
    """[12288 x 4096] and [4096 x 4096] of the benchmark, quantised on the GPU (bit-exact with the oracle's
    quantiser, tested elsewhere), with their fp64 dequantised images for the oracle products."""
    P, O = pkg(), oracle()
    out = {}
    for N in (12288, 4096):
        W = P.quantize(to_dev_bf16(seeded_bf16((N, 4096), 1000 + N)))
        p, s, gs = W.numpy()
        out[N] = (W, O.dequant(p, s, gs).astype(np.float64))
    return out


@pytest.mark.parametrize('N', [12288, 4096])
def test_gemv_full_size_tensor_core_vs_oracle(big, N):
    """The benchmark's first configuration at its stated size on the default (tensor-core) path."""
    P, O = pkg(), oracle()
    W, Wd = big[N]
    x = np.random.default_rng(1).normal(0, 1, (1, 4096)).astype(np.float32)
    y = torch.full((1, N), float('nan'), device='cuda')
    P.gemm(W, torch.from_numpy(x).cuda(), y)
    ref = x.astype(np.float64) @ Wd.T
    r, a = O.rel_l2(y.cpu().numpy(), ref), O.max_abs(y.cpu().numpy(), ref)
    assert r <= REL_TOL and a <= ABS_TOL, (r, a)
    assert P.device_status() == 0


@pytest.mark.parametrize('N', [12288, 4096])
def test_gemm_bf16_full_size_vs_oracle(big, N):
    """The prefill configuration at its stated sizes: 32, 128 and 512 tokens against both matrices."""
    P, O = pkg(), oracle()
    W, Wd = big[N]
    bits = bf16_rows(512, 4096, 4, spread=False)
    x = O.bf16_bits_to_f32(bits)
    xq = O.dequant_rows(*O.quantize_rows(x)).astype(np.float64)
    ref = xq @ Wd.T
    exact = x.astype(np.float64) @ Wd.T
    xd = to_dev_bf16(bits)
    for M in (32, 128, 512):
        y = torch.full((M, N), float('nan'), device='cuda')
        P.gemm_bf16(W, xd[:M].contiguous(), y)
        yh = y.cpu().numpy()
        close(yh, ref[:M])
        assert 0.02 < O.rel_l2(yh, exact[:M]) < 0.2
    # the exact path at the same sizes (passes of 8 rows), against the exact product
    xf = torch.from_numpy(x[:32]).cuda()
    y = P.gemm(W, xf).cpu().numpy()
    assert O.rel_l2(y, exact[:32]) <= REL_TOL
    assert P.device_status() == 0


# ---- the exact wide GEMM (weights dequantised to fp16 in the kernel, tcgen05 kind::f16) --------------

@pytest.mark.parametrize('M,N,K', [(16, 300, 512), (1, 64, 256), (33, 1000, 1024), (100, 257, 1536), (129, 700, 4096),
                                   (300, 130, 2048), (512, 256, 4096), (64, 64, 12288), (20, 20000, 512), (257, 40, 256)])
def test_gemm_bf16_exact_vs_oracle(M, N, K):
    """bf16 activations, exact products: within fp32 accumulation error of the fp64 dequant-then-matmul."""
    P, O = pkg(), oracle()
    t = host_triple((N, K), 300 + N + K)
    bits = bf16_rows(M, K, 9 + M)
    y = torch.full((M, N), float('nan'), device='cuda')
    P.gemm_bf16_exact(P.Nvfp4Weight(*t), to_dev_bf16(bits), y)
    ref = O.gemm(O.bf16_bits_to_f32(bits), *t)
    r = O.rel_l2(y.cpu().numpy(), ref)
    assert r <= 1e-5, r                               # a hundred times inside the 1e-3 bar: only the fp32 accumulation over K
    assert np.abs(ref).max() > 0
    assert P.device_status() == 0


def test_gemm_bf16_exact_rows_independent_and_repeatable():
    P = pkg()
    W = P.Nvfp4Weight(*host_triple((500, 1024), 77))
    x = to_dev_bf16(bf16_rows(200, 1024, 5))
    y = P.gemm_bf16_exact(W, x)
    assert torch.equal(P.gemm_bf16_exact(W, x), y)
    for rows in ([0], [7, 8, 9], list(range(100, 140)), [199]):
        assert torch.equal(P.gemm_bf16_exact(W, x[rows].contiguous()), y[rows]), rows
    z = x.clone(); z[3] = 0; z[4, 17] = float('inf')
    yz = P.gemm_bf16_exact(W, z)
    assert torch.all(yz[3] == 0) and not torch.isfinite(yz[4]).any() and torch.equal(yz[5], y[5])


@pytest.mark.parametrize('N', [12288, 4096])
def test_gemm_bf16_exact_full_size_vs_oracle(big, N):
    P, O = pkg(), oracle()
    W, Wd = big[N]
    bits = bf16_rows(512, 4096, 4, spread=False)
    x = O.bf16_bits_to_f32(bits)
    exact = x.astype(np.float64) @ Wd.T
    xd = to_dev_bf16(bits)
    for M in (32, 128, 512):
        y = torch.full((M, N), float('nan'), device='cuda')
        P.gemm_bf16_exact(W, xd[:M].contiguous(), y)
        assert O.rel_l2(y.cpu().numpy(), exact[:M]) <= 1e-5
    assert P.device_status() == 0
