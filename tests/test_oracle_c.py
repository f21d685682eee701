"""The C restatement of the oracle against the reference-generated vectors and the numpy oracle."""
import ctypes as C
import numpy as np
import nvfp4_oracle as O
from util import c_oracle


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _quant(L, bits):
    bits = np.ascontiguousarray(bits)
    N, K = bits.shape
    gs = L.oracle_global_scale(_p(bits), bits.size)
    p = np.zeros((N, K // 2), np.uint8); s = np.zeros((N, K // 16), np.uint8)
    L.oracle_quantize(_p(bits), N, K, C.c_float(gs), _p(p), _p(s))
    return p, s, np.array([gs], np.float32)


def test_c_quant_matches_reference(golden):
    L = c_oracle()
    for name, tags in (('quant_normal', ['w%d' % i for i in range(5)]), ('quant_edges', list('abcde'))):
        z = golden(name)
        for t in tags:
            p, s, gs = _quant(L, z[t + '_bits'])
            assert gs.view(np.uint32)[0] == z[t + '_gs'].view(np.uint32)[0], t
            assert np.array_equal(s, z[t + '_scale']) and np.array_equal(p, z[t + '_packed']), t
            d = np.zeros(z[t + '_deq'].shape, np.float32)
            L.oracle_dequant(_p(p), _p(s), C.c_float(gs[0]), d.shape[0], d.shape[1], _p(d))
            assert np.array_equal(d.view(np.uint32), z[t + '_deq'].view(np.uint32)), t


def test_c_gemm_and_route(golden):
    L = c_oracle()
    z = golden('gemv')
    for i in range(3):
        x = np.ascontiguousarray(z['g%d_x' % i]); p = np.ascontiguousarray(z['g%d_packed' % i])
        s = np.ascontiguousarray(z['g%d_scale' % i]); gs = float(z['g%d_gs' % i][0])
        M, K = x.shape; N = p.shape[0]
        y = np.zeros((M, N), np.float64)
        L.oracle_gemm(_p(x), _p(p), _p(s), C.c_float(gs), M, N, K, _p(y))
        assert O.rel_l2(y, z['g%d_y' % i]) < 2e-6
    m = golden('moe')
    E, K = int(m['E']), int(m['topk'])
    for t in range(int(m['M'])):
        lg = np.ascontiguousarray(m['logits'][t].astype(np.float64))
        sel = np.zeros(K, np.int32); wts = np.zeros(K, np.float32)
        L.oracle_route(_p(lg), _p(np.ascontiguousarray(m['bias'])), E, K, C.c_float(float(m['scaling'])), 1, _p(sel), _p(wts))
        assert set(sel.tolist()) == set(m['sel'][t].tolist())
        ref = {int(e): float(w) for e, w in zip(m['sel'][t], m['wts'][t])}
        assert all(abs(ref[int(e)] - float(w)) < 1e-5 for e, w in zip(sel, wts))


def test_c_matches_numpy_on_seeded_matrix():
    L = c_oracle()
    bits = O.f32_to_bf16_bits(np.random.default_rng(9).normal(0, 0.02, (96, 1536)).astype(np.float32))
    p, s, gs = _quant(L, bits)
    p2, s2, gs2 = O.quantize_tensor(O.bf16_bits_to_f32(bits))
    assert np.array_equal(p, p2) and np.array_equal(s, s2) and gs[0] == gs2[0]
