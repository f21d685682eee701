"""The CPU oracle against vectors produced by the reference's own Python code
(tests/golden/make_golden.py).  Codes, scales and global scales must match bit for bit."""
import numpy as np
import nvfp4_oracle as O


def test_tables(golden):
    t = golden('tables')
    assert np.array_equal(O.E2M1, t['e2m1']) and np.array_equal(O.E2M1_MID, t['e2m1_mid'])
    assert np.array_equal(O.E4M3, t['e4m3']) and np.array_equal(O.E4M3_MID, t['e4m3_mid'])
    assert np.array_equal(O.E2M1, t['ke2m1'])
    ok = ~np.isnan(t['e4m3_torch'])
    assert ok.sum() == 254
    assert np.array_equal(O.E4M3_ALL[ok], t['e4m3_torch'][ok])


def _check_quant(z, tag):
    bits = z[tag + '_bits']
    w = O.bf16_bits_to_f32(bits)
    p, s, gs = O.quantize_tensor(w)
    assert gs.view(np.uint32)[0] == z[tag + '_gs'].view(np.uint32)[0], tag
    assert np.array_equal(s, z[tag + '_scale']), tag
    assert np.array_equal(p, z[tag + '_packed']), tag
    d = O.dequant(z[tag + '_packed'], z[tag + '_scale'], z[tag + '_gs'])
    assert np.array_equal(d.view(np.uint32), z[tag + '_deq'].view(np.uint32)), tag


def test_quant_normal(golden):
    z = golden('quant_normal')
    for i in range(5):
        _check_quant(z, 'w%d' % i)


def test_quant_edges(golden):
    z = golden('quant_edges')
    for tag in 'abcde':
        _check_quant(z, tag)
    # the edge file must actually contain ties, zero groups and saturated scales
    assert (z['a_scale'] == 0).any() and (z['c_scale'] == 0).any()
    assert z['d_gs'][0] == np.float32(2688.0 / 1e-12)


def test_bf16_roundtrip():
    rng = np.random.default_rng(0)
    x = rng.normal(0, 1, 4096).astype(np.float32)
    b = O.f32_to_bf16_bits(x)
    import torch
    tb = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(b, tb)
    assert np.array_equal(O.bf16_bits_to_f32(b), torch.from_numpy(x).to(torch.bfloat16).float().numpy())


def test_gemv(golden):
    z = golden('gemv')
    for i in range(3):
        y = O.gemm(z['g%d_x' % i], z['g%d_packed' % i], z['g%d_scale' % i], z['g%d_gs' % i])
        assert O.rel_l2(y, z['g%d_y' % i]) < 2e-6


def test_moe(golden):
    z = golden('moe')
    E, K = int(z['E']), int(z['topk'])
    trip = lambda e, nm: (z['e%d_%s_packed' % (e, nm)], z['e%d_%s_scale' % (e, nm)], z['e%d_%s_gs' % (e, nm)])
    experts = [(trip(e, 'gate'), trip(e, 'up'), trip(e, 'down')) for e in range(E)]
    shared = (trip(E, 'gate'), trip(E, 'up'), trip(E, 'down'))
    y, sel, wts, logits, gap = O.moe_layer(z['x'], z['router_bits'], z['bias'], experts, shared, K,
                                           float(z['scaling']), float(z['limit']))
    assert O.rel_l2(logits, z['logits']) < 2e-6
    for m in range(int(z['M'])):
        assert set(sel[m].tolist()) == set(z['sel'][m].tolist())
        order = {int(e): float(w) for e, w in zip(z['sel'][m], z['wts'][m])}
        for e, w in zip(sel[m], wts[m]):
            assert abs(order[int(e)] - float(w)) < 1e-5
    assert gap.min() > 1e-6
    assert O.rel_l2(y, z['y']) < 5e-6
    # the clamp rows must be exercised: token 2 is scaled to push gate/up past the limit
    g = O.gemm(z['x'][2:3], *experts[int(z['sel'][2][0])][0])
    assert (np.abs(g) > float(z['limit'])).any()
    _, act = O.expert_mlp(z['x'][0:1], *experts[int(z['sel'][0][0])])
    assert O.rel_l2(act[0], z['act0'][0]) < 5e-6


def test_gemm_act_golden(golden):
    """Both operands in NVFP4: per-token activation codes bit for bit, product to fp32 rounding."""
    z = golden('gemm_act')
    for i in range(2):
        x = O.bf16_bits_to_f32(z['a%d_xbits' % i])
        p, s, gs = O.quantize_rows(x)
        assert np.array_equal(p, z['a%d_xpacked' % i]) and np.array_equal(s, z['a%d_xscale' % i])
        assert np.array_equal(gs.view(np.uint32), z['a%d_xgs' % i].view(np.uint32))
        y = O.gemm_act_nvfp4(x, z['a%d_packed' % i], z['a%d_scale' % i], z['a%d_gs' % i])
        ref = z['a%d_y' % i]
        assert np.abs(y - ref).max() <= 2e-6 * max(1.0, np.abs(ref).max())
        # the price of 4-bit activations against the exact product: a few per cent, never "close"
        exact = O.gemm(x, z['a%d_packed' % i], z['a%d_scale' % i], z['a%d_gs' % i])
        assert 0.01 < O.rel_l2(y, exact) < 0.2
