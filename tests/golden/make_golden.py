#!/usr/bin/env python3
"""Generates tests/golden/*.npz by running the REFERENCE's own Python code on seeded inputs.

Run once in a container that has the reference checkout (pass its path, or rely on the default
below); the outputs are committed and are what pins the CPU oracle.  Nothing at test time reads
the reference checkout.

    python tests/golden/make_golden.py [/path/to/reference]

What is taken from the reference, unmodified, by import:
  * tools/requant_dense_nvfp4.py : quant_block, E2M1, E4M3, E4M3_MID, bf16_to_f32, and the
    global-scale expression of its main() (:215), evaluated here on the same operands
  * ref/gen_moe.py               : dequant, KE2M1
The router / expert arithmetic of ref/gen_moe.py:62-96 sits inside a main() that needs a
checkpoint, so those ~30 lines are replayed here with the same torch calls (F.linear, sigmoid,
topk(sorted=False), clamp, F.silu) on top of the imported dequant.
"""
import importlib.util, os, sys
import numpy as np
import torch
import torch.nn.functional as F

REF = sys.argv[1] if len(sys.argv) > 1 else '/root/reference'
OUT = os.path.dirname(os.path.abspath(__file__))


def _load(name, rel):
    spec = importlib.util.spec_from_file_location(name, os.path.join(REF, rel))
    mod = importlib.util.module_from_spec(spec)
    argv = sys.argv; sys.argv = [name]
    try:
        spec.loader.exec_module(mod)
    finally:
        sys.argv = argv
    return mod


rq = _load('ref_requant', 'tools/requant_dense_nvfp4.py')
gm = _load('ref_gen_moe', 'ref/gen_moe.py')


def to_bf16_bits(x):
    return torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def ref_quant_tensor(bits):
    """bf16 bit patterns [N,K] -> reference (packed, scale, gs)."""
    w = rq.bf16_to_f32(bits.tobytes()).reshape(bits.shape)
    amax = float(np.abs(w).max())
    gs = np.float32((448.0 * 6.0) / max(amax, 1e-12))         # reference :215
    p, s = rq.quant_block(w, gs)
    return w, p, s, np.array([gs], np.float32)


def ref_dequant(p, s, gs):
    N, K2 = p.shape
    sc = torch.from_numpy(s.copy()).view(torch.float8_e4m3fn)
    return gm.dequant(torch.from_numpy(p.copy()), sc, torch.from_numpy(gs.copy()), N, K2 * 2).numpy()


def case_quant():
    """Seeded N(0,0.02) weights in the benchmark's distribution, a ragged set of shapes."""
    out = {}
    for i, (N, K) in enumerate([(64, 256), (5, 16), (33, 4096), (128, 1536), (7, 128)]):
        rng = np.random.default_rng(1000 + i)
        bits = to_bf16_bits(rng.normal(0.0, 0.02, (N, K)).astype(np.float32))
        w, p, s, gs = ref_quant_tensor(bits)
        out['w%d_bits' % i] = bits; out['w%d_packed' % i] = p; out['w%d_scale' % i] = s
        out['w%d_gs' % i] = gs; out['w%d_deq' % i] = ref_dequant(p, s, gs)
    np.savez_compressed(os.path.join(OUT, 'quant_normal.npz'), **out)


def case_edges():
    """Inputs chosen to sit on decision boundaries: exact e2m1 mid-points, exact e4m3 scale
    mid-points, all-zero groups, negative zero, one huge outlier (saturating scales elsewhere
    to subnormal codes), and a tensor whose amax is 0."""
    out = {}
    # (a) with amax = 6*2^-3 the tensor scale is 2688/0.75 = 3584 and a group whose own amax is
    #     0.75 gets scale code for 448 -> eff = 0.125, so w/eff lands exactly on the grid.
    K = 64
    grid = np.array([0, .25, .5, .75, 1, 1.25, 1.5, 1.75, 2, 2.5, 3, 3.5, 4, 5, 6, 6], np.float32) * 0.125
    rows = []
    for sgn in (1.0, -1.0):
        r = np.concatenate([grid * sgn, grid[::-1] * sgn, grid * -sgn, np.roll(grid, 3) * sgn])
        rows.append(r)
    rows.append(np.zeros(K, np.float32)); rows[-1][0:16] = grid          # three all-zero groups
    z = np.zeros(K, np.float32); z[5] = -0.0; z[16:32] = -grid; rows.append(z)
    bits = to_bf16_bits(np.stack(rows))
    w, p, s, gs = ref_quant_tensor(bits)
    out.update(a_bits=bits, a_packed=p, a_scale=s, a_gs=gs, a_deq=ref_dequant(p, s, gs))
    # (b) scale mid-points: tensor amax 6.0 -> gs = 448; group amax = 6*mid/448 puts s on a
    #     mid-point of the e4m3 table whenever that value is exact in bf16.
    mids = rq.E4M3_MID[::3]
    rows = []
    for md in mids:
        r = np.zeros(16, np.float32); r[3] = np.float32(6.0) * md / np.float32(448.0); r[7] = -r[3] / 2
        rows.append(r)
    W = np.stack(rows).reshape(-1, 32) if len(rows) % 2 == 0 else np.stack(rows[:-1]).reshape(-1, 32)
    W[0, 0] = 6.0
    bits = to_bf16_bits(W)
    w, p, s, gs = ref_quant_tensor(bits)
    out.update(b_bits=bits, b_packed=p, b_scale=s, b_gs=gs, b_deq=ref_dequant(p, s, gs))
    # (c) one outlier of 1e4 beside N(0,0.02): most groups fall to tiny / subnormal scale codes.
    rng = np.random.default_rng(77)
    W = rng.normal(0.0, 0.02, (16, 128)).astype(np.float32); W[3, 17] = 1.0e4; W[9, 0:16] = 0.0
    bits = to_bf16_bits(W)
    w, p, s, gs = ref_quant_tensor(bits)
    out.update(c_bits=bits, c_packed=p, c_scale=s, c_gs=gs, c_deq=ref_dequant(p, s, gs))
    # (d) all zeros: amax 0 -> gs = 2688e12.
    bits = to_bf16_bits(np.zeros((4, 32), np.float32))
    w, p, s, gs = ref_quant_tensor(bits)
    out.update(d_bits=bits, d_packed=p, d_scale=s, d_gs=gs, d_deq=ref_dequant(p, s, gs))
    # (e) wide dynamic range, uniform in log-magnitude, random signs.
    rng = np.random.default_rng(78)
    W = (np.exp(rng.uniform(-12, 3, (24, 256))) * rng.choice([-1.0, 1.0], (24, 256))).astype(np.float32)
    bits = to_bf16_bits(W)
    w, p, s, gs = ref_quant_tensor(bits)
    out.update(e_bits=bits, e_packed=p, e_scale=s, e_gs=gs, e_deq=ref_dequant(p, s, gs))
    np.savez_compressed(os.path.join(OUT, 'quant_edges.npz'), **out)


def case_tables():
    np.savez_compressed(os.path.join(OUT, 'tables.npz'), e2m1=rq.E2M1, e2m1_mid=rq.E2M1_MID,
                        e4m3=rq.E4M3, e4m3_mid=rq.E4M3_MID, ke2m1=gm.KE2M1.numpy(),
                        e4m3_torch=torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy())


def case_gemv():
    """dequantise-then-matvec exactly as the reference's CPU path does it (fp32 torch)."""
    out = {}
    for i, (M, N, K) in enumerate([(1, 96, 512), (4, 40, 128), (8, 17, 1024)]):
        rng = np.random.default_rng(2000 + i)
        bits = to_bf16_bits(rng.normal(0.0, 0.02, (N, K)).astype(np.float32))
        w, p, s, gs = ref_quant_tensor(bits)
        x = rng.normal(0.0, 1.0, (M, K)).astype(np.float32)
        W = torch.from_numpy(ref_dequant(p, s, gs))
        y = F.linear(torch.from_numpy(x), W).numpy()
        out.update({'g%d_packed' % i: p, 'g%d_scale' % i: s, 'g%d_gs' % i: gs, 'g%d_x' % i: x, 'g%d_y' % i: y})
    np.savez_compressed(os.path.join(OUT, 'gemv.npz'), **out)


def case_gemm_act():
    """Both operands in NVFP4: activations (bf16-valued) quantised one token at a time by the
    reference's quant_block with the token's own global scale, then dequantise-and-matmul."""
    out = {}
    for i, (M, N, K) in enumerate([(5, 24, 256), (33, 40, 512)]):
        rng = np.random.default_rng(2500 + i)
        bits = to_bf16_bits(rng.normal(0.0, 0.02, (N, K)).astype(np.float32))
        w, p, s, gs = ref_quant_tensor(bits)
        xbits = to_bf16_bits((rng.normal(0.0, 1.0, (M, K)) * np.exp(rng.uniform(-3, 3, (M, 1)))).astype(np.float32))
        xp, xs, xg, xd = [], [], [], []
        for m in range(M):
            _, pm, sm, gm_ = ref_quant_tensor(xbits[m:m + 1])
            xp.append(pm); xs.append(sm); xg.append(gm_); xd.append(ref_dequant(pm, sm, gm_))
        W = torch.from_numpy(ref_dequant(p, s, gs))
        y = F.linear(torch.from_numpy(np.concatenate(xd, 0)), W).numpy()
        out.update({'a%d_packed' % i: p, 'a%d_scale' % i: s, 'a%d_gs' % i: gs, 'a%d_xbits' % i: xbits,
                    'a%d_xpacked' % i: np.concatenate(xp, 0), 'a%d_xscale' % i: np.concatenate(xs, 0),
                    'a%d_xgs' % i: np.concatenate(xg, 0), 'a%d_y' % i: y})
    np.savez_compressed(os.path.join(OUT, 'gemm_act.npz'), **out)


def case_moe():
    """The MoE block of ref/gen_moe.py:62-96 at a small geometry, M tokens one at a time."""
    H, I, E, K, M = 256, 128, 16, 4, 3
    scale, lim = 2.5, 10.0
    rng = np.random.default_rng(3000)
    out = dict(H=H, I=I, E=E, topk=K, M=M, scaling=scale, limit=lim)
    gw_bits = to_bf16_bits(rng.normal(0.0, 0.02, (E, H)).astype(np.float32) * 4)
    bias = rng.normal(0.0, 0.1, E).astype(np.float32)
    xs = (rng.normal(0.0, 1.0, (M, H)) * np.array([1.0, 1.0, 40.0])[:, None]).astype(np.float32)   # row 2 drives the clamps
    mats = {}
    for e in range(E + 1):
        for nm, (o, i) in (('gate', (I, H)), ('up', (I, H)), ('down', (H, I))):
            bits = to_bf16_bits(rng.normal(0.0, 0.02 if e < E else 0.05, (o, i)).astype(np.float32))
            w, p, s, gs = ref_quant_tensor(bits)
            mats[(e, nm)] = (p, s, gs)
            out['e%d_%s_packed' % (e, nm)] = p; out['e%d_%s_scale' % (e, nm)] = s; out['e%d_%s_gs' % (e, nm)] = gs
    gw = torch.from_numpy(rq.bf16_to_f32(gw_bits.tobytes()).reshape(E, H).copy())
    ys, sels, wtss, lgs, acts0 = [], [], [], [], []
    for m in range(M):
        x = torch.from_numpy(xs[m])
        logits = F.linear(x.unsqueeze(0), gw)[0]
        scores = logits.sigmoid()
        choice = scores + torch.from_numpy(bias)
        idx = torch.topk(choice, k=K, dim=-1, sorted=False)[1]
        wts = scores[idx]
        wts = wts / (wts.sum() + 1e-20)
        wts = wts * scale

        def expert_mlp(e):
            dq = lambda nm: torch.from_numpy(ref_dequant(*mats[(e, nm)]))
            gp, up, dn = dq('gate'), dq('up'), dq('down')
            gt = (x @ gp.T).clamp(max=lim)
            u = (x @ up.T).clamp(-lim, lim)
            return (F.silu(gt) * u) @ dn.T, gt, u

        routed = torch.zeros(H)
        for s_ in range(K):
            y, gt, u = expert_mlp(int(idx[s_]))
            if s_ == 0:
                acts0.append((F.silu(gt) * u).numpy())
            routed += y * wts[s_]
        shared, _, _ = expert_mlp(E)
        ys.append((routed + shared).numpy()); sels.append(idx.numpy().astype(np.int32))
        wtss.append(wts.numpy()); lgs.append(logits.numpy())
    out.update(router_bits=gw_bits, bias=bias, x=xs, y=np.stack(ys), sel=np.stack(sels),
               wts=np.stack(wtss), logits=np.stack(lgs), act0=np.stack(acts0))
    np.savez_compressed(os.path.join(OUT, 'moe.npz'), **out)


def case_overlay():
    """A tiny bf16 'checkpoint' (two safetensors shards; names that hit, miss and are excluded by the family
    tables; a non-bf16 tensor; a K that is not a multiple of 16) and the overlay the reference's own tool
    writes for it: tools/requant_dense_nvfp4.py run unmodified as a program."""
    import json, shutil, struct, subprocess
    mdir, odir = os.path.join(OUT, 'overlay_model'), os.path.join(OUT, 'overlay')
    for d in (mdir, odir):
        shutil.rmtree(d, ignore_errors=True); os.makedirs(d)
    rng = np.random.default_rng(4242)

    def bf(shape, std=0.02):
        return to_bf16_bits(rng.normal(0.0, std, shape).astype(np.float32))
    shards = [
        [('model.layers.0.self_attn.q_proj.weight', 'BF16', bf((64, 256))),
         ('model.layers.0.self_attn.o_proj.weight', 'BF16', bf((32, 128))),
         ('model.layers.0.mlp.gate.weight', 'BF16', bf((8, 64))),
         ('model.visual.layers.0.self_attn.o_proj.weight', 'BF16', bf((16, 32))),
         ('model.layers.1.mlp.down_proj.weight', 'BF16', bf((48, 96), 0.05)),
         ('model.layers.1.self_attn.kv_b_proj.weight', 'BF16', bf((16, 32))),
         ('model.embed_tokens.weight', 'BF16', bf((20, 32))),
         ('model.layers.2.mlp.up_proj.weight', 'F32', rng.normal(0, 0.02, (8, 32)).astype(np.float32)),
         ('model.layers.2.self_attn.f_a_proj.weight', 'BF16', bf((16, 40)))],
        [('lm_head.weight', 'BF16', bf((100, 64))),
         ('model.layers.3.self_attn.indexer.wk.weight', 'BF16', bf((24, 32))),
         ('model.layers.3.self_attn.index_kpool_compress_gate', 'BF16', bf((4, 16), 1.0)),
         ('model.layers.3.self_attn.g_b_proj.weight', 'BF16', np.zeros((8, 16), np.uint16))],
    ]
    for i, tensors in enumerate(shards):
        meta, blob, off = {}, b'', 0
        for name, dt, arr in tensors:
            b = arr.tobytes()
            meta[name] = {'dtype': dt, 'shape': list(arr.shape), 'data_offsets': [off, off + len(b)]}
            blob += b; off += len(b)
        hdr = json.dumps(meta, separators=(',', ':')).encode()
        with open(os.path.join(mdir, 'model-%05d-of-00002.safetensors' % (i + 1)), 'wb') as f:
            f.write(struct.pack('<Q', len(hdr))); f.write(hdr); f.write(blob)
    subprocess.check_call([sys.executable, os.path.join(REF, 'tools', 'requant_dense_nvfp4.py'), '--model', mdir, '--out', odir,
                           '--rows', '16', '--shard-bytes', '12000'])


if __name__ == '__main__':
    case_overlay()
    case_tables(); case_quant(); case_edges(); case_gemv(); case_gemm_act(); case_moe()
    for f in sorted(os.listdir(OUT)):
        if f.endswith('.npz'):
            print('%-20s %8d bytes' % (f, os.path.getsize(os.path.join(OUT, f))))
