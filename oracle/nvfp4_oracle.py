"""CPU oracle for the NVFP4 weight path -- TEST INFRASTRUCTURE, not product code.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import this file;
the CUDA library never calls into it and has no CPU fallback.

It restates, in plain numpy, the arithmetic of the reference's CPU path for:

  * the bf16 -> NVFP4 quantiser      reference tools/requant_dense_nvfp4.py:28-68, 209-215
  * the NVFP4 -> fp32 dequantiser    reference ref/gen_moe.py:20-30, include/nvfp4.cuh:3-7
  * dequantise-then-matvec (gemv)    reference kernels/gemv.cu:246-322 (semantics, fp64 sums here)
  * the MoE block                    reference ref/gen_moe.py:62-96, kernels/moe.cu:126-156,
                                     253-258, 584-597, include/glm5_config.h:84-91

Parity status: PINNED.  tests/golden/*.npz were produced in a container that holds the reference
checkout, by tests/golden/make_golden.py, which imports the reference's own `quant_block` and
`dequant` and runs them on seeded inputs; tests/test_oracle_golden.py checks every function below
against those files bit for bit (codes, scales, global scale) or to 1e-6 (fp32 outputs).

Format (reference include/nvfp4.cuh:3-7):
    packed [N, K/2]  uint8, LOW nibble = even k
    scale  [N, K/16] uint8 holding an fp8-e4m3 code
    gscale [1]       fp32
    w[n,k] = E2M1[nib & 7] * (-1)^(nib >> 3) * e4m3(scale[n, k/16]) / gscale
"""
import numpy as np

GROUP = 16
E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
E2M1_MID = ((E2M1[1:] + E2M1[:-1]) / 2).astype(np.float32)

# Reference model constants (include/glm5_config.h:84-91); the MoE functions take them as
# arguments so that the 1536-wide benchmark geometry and the reference's 2048 both run.
ROUTED_SCALE = 2.5
SWIGLU_LIMIT = 10.0


def e4m3_decode_table():
    """All 256 fp8-e4m3 codes -> fp32 (0x7F / 0xFF are NaN in the format; the quantiser never
    emits them).  Same construction as reference include/nvfp4.cuh:30-35."""
    c = np.arange(256, dtype=np.int32)
    s, e, m = c >> 7, (c >> 3) & 0xF, c & 7
    sub = m.astype(np.float32) * np.float32(1.0 / 8.0) * np.float32(1.0 / 64.0)
    nrm = (np.float32(1.0) + m.astype(np.float32) / np.float32(8.0)) * np.exp2((e - 7).astype(np.float32))
    v = np.where(e == 0, sub, nrm).astype(np.float32)
    return np.where(s == 1, -v, v).astype(np.float32)


E4M3_ALL = e4m3_decode_table()
E4M3 = E4M3_ALL[:127].copy()                       # positive finite codes 0..126, increasing
E4M3_MID = ((E4M3[1:] + E4M3[:-1]) / 2).astype(np.float32)
FP8_MAX = float(E4M3[-1])                          # 448


def bf16_bits_to_f32(u16):
    """uint16 bf16 bit patterns -> fp32 (reference tools/requant_dense_nvfp4.py:48-50)."""
    return (np.asarray(u16, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x):
    """fp32 -> bf16 bit patterns, round to nearest even (what torch / __float2bfloat16 do)."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) >> 16).astype(np.uint16)


def global_scale(w_f32):
    """Per-tensor scale: fp32(2688 / max(amax, 1e-12)), the quotient taken in double
    (reference tools/requant_dense_nvfp4.py:209-215)."""
    amax = float(np.abs(w_f32).max()) if w_f32.size else 0.0
    return np.float32((448.0 * 6.0) / max(amax, 1e-12))


def quantize(w_f32, gs):
    """fp32 [N, K] (K % 16 == 0) -> (packed u8 [N, K/2], scale-code u8 [N, K/16]).

    Follows reference tools/requant_dense_nvfp4.py:53-68 step by step, every operation in fp32:
    group amax -> s = clip(amax/6*gs, 0, 448) -> code = #{mid < s} (ties to the LOWER code) ->
    eff = e4m3(code)/gs -> q = w/max(eff,1e-30) -> idx = #{mid < |q|} -> sign unless idx == 0."""
    w = np.ascontiguousarray(w_f32, dtype=np.float32)
    rows, K = w.shape
    assert K % GROUP == 0
    gs = np.float32(gs)
    g = w.reshape(rows, K // GROUP, GROUP)
    amax = np.abs(g).max(-1) if rows else np.zeros((0, K // GROUP), np.float32)
    s = np.clip(amax / np.float32(6.0) * gs, np.float32(0.0), np.float32(FP8_MAX))
    code = np.searchsorted(E4M3_MID, s).astype(np.uint8)
    eff = (E4M3[code] / gs).astype(np.float32)
    q = g / np.maximum(eff, np.float32(1e-30))[:, :, None]
    idx = np.searchsorted(E2M1_MID, np.abs(q)).astype(np.uint8)
    idx |= (np.signbit(q) & (idx != 0)).astype(np.uint8) << 3
    idx = idx.reshape(rows, K)
    packed = (idx[:, 0::2] | (idx[:, 1::2] << 4)).astype(np.uint8)
    return packed, code


def quantize_tensor(w_f32):
    """Both passes of the reference tool for one tensor: (packed, scale, gs[1])."""
    gs = global_scale(w_f32)
    p, s = quantize(w_f32, gs)
    return p, s, np.array([gs], np.float32)


def dequant(packed, scale, gs):
    """NVFP4 triple -> fp32 [N, K]; same operation order as reference ref/gen_moe.py:23-30
    (code value times (scale / gs), both fp32)."""
    packed = np.asarray(packed, np.uint8)
    N, K2 = packed.shape
    K = K2 * 2
    nib = np.empty((N, K), np.uint8)
    nib[:, 0::2] = packed & 0x0F
    nib[:, 1::2] = packed >> 4
    vals = E2M1[nib & 7] * np.where(nib & 8, np.float32(-1.0), np.float32(1.0))
    sc = E4M3_ALL[np.asarray(scale, np.uint8)] / np.float32(np.asarray(gs).reshape(-1)[0])
    return (vals.reshape(N, K // GROUP, GROUP) * sc.reshape(N, K // GROUP, 1)).reshape(N, K).astype(np.float32)


def gemm(x, packed, scale, gs):
    """y[M,N] = x[M,K] . dequant(W)[N,K]^T with fp64 accumulation, returned as fp64, so the
    oracle's own rounding stays far below the 1e-3 parity tolerance."""
    W = dequant(packed, scale, gs).astype(np.float64)
    x = np.atleast_2d(np.asarray(x, np.float32)).astype(np.float64)
    return x @ W.T


def gemv(x, packed, scale, gs):
    return gemm(x, packed, scale, gs)[0]


def quantize_rows(x_f32):
    """Per-token activation quantisation of the block-scaled tensor-core GEMM: the reference's
    quant_block rule (tools/requant_dense_nvfp4.py:53-68) applied to every row on its own, with the
    row's own global scale 2688 / max(amax(row), 1e-12) (:215 evaluated per row).
    Returns packed u8 [M, K/2], scale codes u8 [M, K/16], gs f32 [M]."""
    x = np.atleast_2d(np.asarray(x_f32, np.float32))
    M, K = x.shape
    packed = np.zeros((M, K // 2), np.uint8); scale = np.zeros((M, K // GROUP), np.uint8); gs = np.zeros(M, np.float32)
    for m in range(M):
        gs[m] = global_scale(x[m])
        packed[m:m + 1], scale[m:m + 1] = quantize(x[m:m + 1], gs[m])
    return packed, scale, gs


def dequant_rows(packed, scale, gs):
    return np.concatenate([dequant(packed[m:m + 1], scale[m:m + 1], gs[m]) for m in range(packed.shape[0])], 0)


def gemm_act_nvfp4(x, packed, scale, gs):
    """y[M,N] = deq(quant_rows(x)) . deq(W)^T with fp64 accumulation: what a GEMM with BOTH operands in
    NVFP4 computes (weights as stored, activations quantised per token).  The tensor-core prefill
    path is judged against this; its distance from gemm() is the price of 4-bit activations."""
    xq = dequant_rows(*quantize_rows(x)).astype(np.float64)
    return xq @ dequant(packed, scale, gs).astype(np.float64).T


def router_logits(x, router_w_bf16_bits):
    """x[M,H] fp32 times the bf16 router matrix [E,H] (reference kernels/moe.cu:643-647)."""
    Wr = bf16_bits_to_f32(router_w_bf16_bits).astype(np.float64)
    return np.atleast_2d(np.asarray(x, np.float32)).astype(np.float64) @ Wr.T


def route(logits, bias, topk, scaling=ROUTED_SCALE, norm_prob=True):
    """Sigmoid scores, ranking by score + bias, lowest index wins a tie, weights are the
    UNBIASED scores renormalised and scaled (reference kernels/moe.cu:126-156,
    ref/gen_moe.py:66-74).  Returns sel int32 [M,topk] in descending biased score, wts fp32,
    and the gap between the topk-th and (topk+1)-th biased score per token."""
    logits = np.atleast_2d(np.asarray(logits, np.float64))
    M, E = logits.shape
    score = (1.0 / (1.0 + np.exp(-logits))).astype(np.float32)
    choice = (score + np.asarray(bias, np.float32)[None, :]).astype(np.float32)
    sel = np.zeros((M, topk), np.int32)
    wts = np.zeros((M, topk), np.float32)
    gap = np.zeros(M, np.float64)
    for m in range(M):
        c = choice[m].copy()
        for k in range(topk):
            bi = int(np.argmax(c))                  # first maximum == lowest index on ties
            sel[m, k] = bi
            wts[m, k] = score[m, bi]
            last = c[bi]
            c[bi] = -1e30
        gap[m] = float(last) - float(c.max()) if topk < E else np.inf
        d = np.float32(1.0)
        if norm_prob:
            d = np.float32(1e-20)
            for k in range(topk):
                d = np.float32(d + wts[m, k])
        wts[m] = (wts[m] / d * np.float32(scaling)).astype(np.float32)
    return sel, wts, gap


def expert_mlp(x, gate, up, down, limit=SWIGLU_LIMIT):
    """One SwiGLU expert on x[M,H]; gate/up/down are NVFP4 triples.  gate is clamped from above
    only, up on both sides (reference ref/gen_moe.py:79-87, kernels/moe.cu:253-258)."""
    g = np.minimum(gemm(x, *gate), limit)
    u = np.clip(gemm(x, *up), -limit, limit)
    act = (g / (1.0 + np.exp(-g))) * u
    Wd = dequant(*down).astype(np.float64)
    return act @ Wd.T, act


def moe_layer(x, router_w_bf16_bits, bias, experts, shared, topk, scaling=ROUTED_SCALE,
              limit=SWIGLU_LIMIT, norm_prob=True):
    """Whole block for x[M,H]: route, topk routed experts weighted by their gates, plus the
    shared expert unweighted (reference ref/gen_moe.py:62-96).  `experts` is a list of
    (gate, up, down) triples of NVFP4 triples.  Returns y fp64 [M,H], sel, wts, logits, gap."""
    x = np.atleast_2d(np.asarray(x, np.float32))
    logits = router_logits(x, router_w_bf16_bits)
    sel, wts, gap = route(logits, bias, topk, scaling, norm_prob)
    M, H = x.shape
    y = np.zeros((M, H), np.float64)
    for m in range(M):
        for k in range(topk):
            o, _ = expert_mlp(x[m:m + 1], *experts[int(sel[m, k])], limit=limit)
            y[m] += o[0] * float(wts[m, k])
    o, _ = expert_mlp(x, *shared, limit=limit)
    y += o
    return y, sel, wts, logits, gap


def moe_experts(x, sel, wts, experts, shared, limit=SWIGLU_LIMIT):
    """The expert half of the block with the routing decision supplied by the caller."""
    x = np.atleast_2d(np.asarray(x, np.float32))
    M, H = x.shape
    y = np.zeros((M, H), np.float64)
    cache = {}
    for m in range(M):
        for k in range(sel.shape[1]):
            e = int(sel[m, k])
            o, _ = expert_mlp(x[m:m + 1], *experts[e], limit=limit)
            y[m] += o[0] * float(wts[m, k])
    if shared is not None:
        o, _ = expert_mlp(x, *shared, limit=limit)
        y += o
    return y


def moe_experts_act_nvfp4(x, sel, wts, experts, shared, limit=SWIGLU_LIMIT):
    """The expert half of the block as the wide tensor-core path computes it: the same SwiGLU experts
    (reference ref/gen_moe.py:79-96) with both operands of every product in NVFP4 -- the token row is
    quantised per token before gate/up (gemm_act_nvfp4), and the SwiGLU output (rounded to fp32) is
    quantised per row again before the down projection.  Rows are processed per distinct expert."""
    x = np.atleast_2d(np.asarray(x, np.float32))
    M, H = x.shape
    y = np.zeros((M, H), np.float64)
    xq = dequant_rows(*quantize_rows(x)).astype(np.float64)

    def mlp(rows, gate, up, down):
        g = np.minimum(rows @ dequant(*gate).astype(np.float64).T, limit)
        u = np.clip(rows @ dequant(*up).astype(np.float64).T, -limit, limit)
        act = ((g / (1.0 + np.exp(-g))) * u).astype(np.float32)
        aq = dequant_rows(*quantize_rows(act)).astype(np.float64)
        return aq @ dequant(*down).astype(np.float64).T

    sel = np.asarray(sel)
    for e in sorted(set(sel.ravel().tolist())):
        tok, slot = np.nonzero(sel == e)
        y[tok] += mlp(xq[tok], *experts[e]) * np.asarray(wts, np.float64)[tok, slot][:, None]
    if shared is not None:
        y += mlp(xq, *shared)
    return y


def rel_l2(a, b):
    a = np.asarray(a, np.float64).ravel(); b = np.asarray(b, np.float64).ravel()
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def max_abs(a, b):
    return float(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64)).max()) if np.size(a) else 0.0
