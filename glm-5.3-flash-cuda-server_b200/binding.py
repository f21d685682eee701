"""ctypes binding of libb200nvfp4.so for tests and benchmarks.

The product is the shared library and its C ABI (include/b200_nvfp4.h); this file only moves
pointers.  torch is used for device memory and streams.  There is no fallback of any kind: if
the library has not been built, or a call returns a non-zero status, an exception is raised.
"""
import ctypes as C
import os
import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get('B200_NVFP4_LIB') or os.path.join(_HERE, 'libb200nvfp4.so')
_lib = None

F32, BF16 = 0, 1
GEMV_MULTI_MAX, GEMV_M_MAX = 8, 8


class WRef(C.Structure):
    _fields_ = [('p', C.c_void_p), ('packed', C.c_void_p), ('scale', C.c_void_p), ('gscale', C.c_void_p)]


class GemvJob(C.Structure):
    _fields_ = [('y', C.c_void_p), ('W', WRef), ('x', C.c_void_p), ('N', C.c_int)]


class Nvfp4Mat(C.Structure):
    _fields_ = [('packed', C.c_void_p), ('scale', C.c_void_p), ('gscale', C.c_void_p)]


class MoeLayerC(C.Structure):
    _fields_ = [('router_w', WRef), ('router_bias', C.c_void_p), ('experts', C.c_void_p),
                ('shared', C.c_void_p), ('n_expert', C.c_int), ('topk', C.c_int), ('hidden', C.c_int),
                ('inter', C.c_int), ('routed_scale', C.c_float), ('swiglu_limit', C.c_float),
                ('norm_topk', C.c_int)]


class EpStats(C.Structure):
    _fields_ = [('tokens', C.c_int), ('recv_rows', C.c_int), ('sent_remote_rows', C.c_int), ('recv_remote_rows', C.c_int),
                ('local_experts_touched', C.c_int), ('pad', C.c_int), ('dispatch_bytes_out', C.c_ulonglong),
                ('combine_bytes_in', C.c_ulonglong), ('plan_us', C.c_float), ('dispatch_us', C.c_float),
                ('experts_us', C.c_float), ('combine_us', C.c_float), ('total_us', C.c_float), ('pad2', C.c_float)]


class OverlayEntry(C.Structure):
    _fields_ = [('packed', C.c_void_p), ('scale', C.c_void_p), ('gscale', C.c_float), ('N', C.c_int), ('K', C.c_int)]


class B200Error(RuntimeError):
    pass


def lib():
    """The loaded library; raises if it has not been built (python -c 'import __graft_entry__ as g; g.build()')."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200Error('libb200nvfp4.so is missing at %s: build it first; there is no CPU fallback' % LIB_PATH)
        L = C.CDLL(LIB_PATH)
        vp, ci, st = C.c_void_p, C.c_int, C.c_size_t
        L.b200_nvfp4_strerror.restype = C.c_char_p; L.b200_nvfp4_strerror.argtypes = [ci]
        L.b200_nvfp4_version.restype = ci
        L.b200_nvfp4_device_status.argtypes = [C.POINTER(C.c_uint), ci]
        L.b200_nvfp4_selftest_bounded_wait.argtypes = [vp]
        L.b200_nvfp4_set_byte_credit.argtypes = [vp, vp]
        L.b200_nvfp4_flush_byte_credit.argtypes = [ci]
        L.b200_nvfp4_gemm.argtypes = [vp, C.POINTER(WRef), vp, ci, ci, ci, ci, vp]
        L.b200_nvfp4_gemv_multi.argtypes = [C.POINTER(GemvJob), ci, ci, ci, ci, vp]
        L.b200_nvfp4_split_workspace_bytes.restype = st; L.b200_nvfp4_split_workspace_bytes.argtypes = [ci, ci]
        L.b200_nvfp4_gemm_ws.argtypes = [vp, C.POINTER(WRef), vp, ci, ci, ci, ci, vp, vp]
        L.b200_nvfp4_gemv_multi_ws.argtypes = [C.POINTER(GemvJob), ci, ci, ci, ci, vp, vp]
        L.b200_nvfp4_gemm_bf16_workspace_bytes.restype = st; L.b200_nvfp4_gemm_bf16_workspace_bytes.argtypes = [ci, ci]
        L.b200_nvfp4_gemm_bf16.argtypes = [vp, C.POINTER(WRef), vp, ci, ci, ci, vp, vp]
        L.b200_nvfp4_quantize_tokens.argtypes = [vp, ci, ci, ci, vp, vp, vp, vp]
        L.b200_nvfp4_gemm_bf16_exact_workspace_bytes.restype = st; L.b200_nvfp4_gemm_bf16_exact_workspace_bytes.argtypes = [ci, ci]
        L.b200_nvfp4_gemm_bf16_exact.argtypes = [vp, C.POINTER(WRef), vp, ci, ci, ci, vp, vp]
        L.b200_dense_mlp_workspace_bytes.restype = st; L.b200_dense_mlp_workspace_bytes.argtypes = [ci, ci, ci]
        L.b200_dense_mlp.argtypes = [vp, C.POINTER(WRef), C.POINTER(WRef), C.POINTER(WRef), ci, ci, C.c_float, vp, vp, ci, vp]
        L.b200_f32_to_bf16.argtypes = [vp, vp, st, vp]
        L.b200_bf16_to_f32.argtypes = [vp, vp, st, vp]
        L.b200_nvfp4_quantize.argtypes = [vp, ci, ci, vp, vp, vp, vp, vp]
        L.b200_nvfp4_dequantize.argtypes = [vp, C.POINTER(Nvfp4Mat), ci, ci, vp]
        L.b200_moe_workspace_bytes.restype = st; L.b200_moe_workspace_bytes.argtypes = [C.POINTER(MoeLayerC), ci]
        L.b200_moe_route.argtypes = [vp, C.POINTER(MoeLayerC), vp, vp, vp, ci, vp]
        L.b200_moe_forward.argtypes = [vp, C.POINTER(MoeLayerC), vp, vp, vp, vp, ci, vp]
        L.b200_moe_experts.argtypes = [vp, C.POINTER(MoeLayerC), vp, vp, vp, vp, ci, vp]
        L.b200_moe_forward_static.argtypes = [vp, C.POINTER(MoeLayerC), vp, vp, vp, ci, vp]
        L.b200_moe_static_ws_limit.restype = st
        L.b200_ep_unique_id.argtypes = [vp]
        L.b200_ep_create.argtypes = [C.POINTER(vp), vp, ci, ci, C.POINTER(MoeLayerC), C.POINTER(MoeLayerC), C.POINTER(MoeLayerC), ci]
        L.b200_ep_forward.argtypes = [vp, vp, vp, vp, vp, ci, vp]
        L.b200_ep_last_stats.argtypes = [vp, C.POINTER(EpStats)]
        L.b200_ep_destroy.argtypes = [vp]
        L.b200_overlay_writer_open.argtypes = [C.POINTER(vp), C.c_char_p, C.c_uint64]
        L.b200_overlay_writer_add.argtypes = [vp, C.c_char_p, vp, vp, C.c_float, ci, ci]
        L.b200_overlay_writer_close.argtypes = [vp]
        L.b200_overlay_family.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p]
        L.b200_overlay_open.argtypes = [C.POINTER(vp), C.c_char_p]
        L.b200_overlay_count.argtypes = [vp]
        L.b200_overlay_find.argtypes = [vp, C.c_char_p, C.POINTER(OverlayEntry)]
        L.b200_overlay_close.argtypes = [vp]
        L.b200_moe_prepare.argtypes = [C.POINTER(MoeLayerC)]
        L.b200_moe_release.argtypes = [C.POINTER(MoeLayerC)]
        _lib = L
    return _lib


ENOTIMPL = 6
EXPORTS = ['b200_nvfp4_set_byte_credit', 'b200_nvfp4_flush_byte_credit', 'b200_nvfp4_strerror', 'b200_nvfp4_version', 'b200_nvfp4_device_status', 'b200_nvfp4_selftest_bounded_wait', 'b200_nvfp4_set_option', 'b200_nvfp4_gemm', 'b200_nvfp4_gemv_multi', 'b200_nvfp4_split_workspace_bytes', 'b200_nvfp4_gemm_ws', 'b200_nvfp4_gemv_multi_ws',
           'b200_nvfp4_gemm_bf16_workspace_bytes', 'b200_nvfp4_gemm_bf16', 'b200_nvfp4_quantize_tokens', 'b200_nvfp4_gemm_bf16_exact_workspace_bytes', 'b200_nvfp4_gemm_bf16_exact', 'b200_dense_mlp_workspace_bytes', 'b200_dense_mlp', 'b200_f32_to_bf16', 'b200_bf16_to_f32', 'b200_nvfp4_quantize', 'b200_nvfp4_dequantize',
           'b200_moe_workspace_bytes', 'b200_moe_route', 'b200_moe_forward', 'b200_moe_experts',
           'b200_moe_forward_static', 'b200_moe_static_ws_limit', 'b200_moe_prepare', 'b200_moe_release',
           'b200_overlay_writer_open', 'b200_overlay_writer_add', 'b200_overlay_writer_close', 'b200_overlay_family',
           'b200_overlay_open', 'b200_overlay_count', 'b200_overlay_find', 'b200_overlay_close',
           'b200_ep_unique_id', 'b200_ep_create', 'b200_ep_forward', 'b200_ep_last_stats', 'b200_ep_destroy']


def check(rc, what):
    if rc != 0:
        raise B200Error('%s failed: %s (%d)' % (what, lib().b200_nvfp4_strerror(rc).decode(), rc))


def device_status(clear=False):
    """0 unless a bounded wait inside a kernel ever ran out (synchronises the device)."""
    v = C.c_uint(0)
    check(lib().b200_nvfp4_device_status(C.byref(v), 1 if clear else 0), 'b200_nvfp4_device_status')
    return v.value


OPT_STABLE_WEIGHTS = 1
OPT_PREFILL_FP4 = 2


def set_option(option, value):
    check(lib().b200_nvfp4_set_option(int(option), int(value)), 'b200_nvfp4_set_option')


def stream_ptr(stream=None):
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


class Nvfp4Weight:
    """An NVFP4 triple resident on the device (packed u8 [N,K/2], scale u8 [N,K/16], gscale f32 [1])."""

    def __init__(self, packed, scale, gscale, device='cuda'):
        to = lambda a, dt: (torch.from_numpy(np.ascontiguousarray(a)) if isinstance(a, np.ndarray) else a).to(device=device, dtype=dt).contiguous()
        self.packed, self.scale, self.gscale = to(packed, torch.uint8), to(scale, torch.uint8), to(gscale, torch.float32)
        self.N, self.K = self.packed.shape[0], self.packed.shape[1] * 2

    def wref(self):
        return WRef(None, self.packed.data_ptr(), self.scale.data_ptr(), self.gscale.data_ptr())

    def mat(self):
        return Nvfp4Mat(self.packed.data_ptr(), self.scale.data_ptr(), self.gscale.data_ptr())

    def numpy(self):
        return self.packed.cpu().numpy(), self.scale.cpu().numpy(), self.gscale.cpu().numpy()

    @property
    def nbytes(self):
        return self.packed.numel() + self.scale.numel() + 4


def split_workspace(M, K, device):
    """Scratch for gemm(..., ws=) / gemv_multi(..., ws=): the pre-split activation images."""
    return torch.empty(lib().b200_nvfp4_split_workspace_bytes(M, K), dtype=torch.uint8, device=device)


def gemm(W, x, y=None, dtype=BF16, stream=None, ws=None):
    """y[M,N] = x[M,K] . W^T.  W: Nvfp4Weight, or a bf16/f32 torch tensor [N,K].  ws: split_workspace(M, K)."""
    x2 = x if x.dim() == 2 else x.unsqueeze(0)
    M, K = x2.shape
    if isinstance(W, Nvfp4Weight):
        N, ref = W.N, W.wref()
        assert W.K == K
    else:
        N, ref = W.shape[0], WRef(W.data_ptr(), None, None, None)
        dtype = F32 if W.dtype == torch.float32 else BF16
    if y is None:
        y = torch.empty((M, N), dtype=torch.float32, device=x.device)
    if ws is not None:
        check(lib().b200_nvfp4_gemm_ws(_ptr(y), C.byref(ref), _ptr(x2), M, N, K, dtype, _ptr(ws), stream_ptr(stream)), 'b200_nvfp4_gemm_ws')
    else:
        check(lib().b200_nvfp4_gemm(_ptr(y), C.byref(ref), _ptr(x2), M, N, K, dtype, stream_ptr(stream)), 'b200_nvfp4_gemm')
    return y if x.dim() == 2 else y[0]


def gemm_bf16_workspace(M, K, device):
    return torch.empty(lib().b200_nvfp4_gemm_bf16_workspace_bytes(M, K), dtype=torch.uint8, device=device)


def gemm_bf16(W, x_bf16, y=None, ws=None, stream=None):
    """The wide GEMM: y[M,N] f32 = x[M,K] bf16 . W^T with the activations quantised to NVFP4 per token."""
    M, K = x_bf16.shape
    assert W.K == K and x_bf16.dtype == torch.bfloat16
    if y is None:
        y = torch.empty((M, W.N), dtype=torch.float32, device=x_bf16.device)
    if ws is None:
        ws = gemm_bf16_workspace(M, K, x_bf16.device)
    ref = W.wref()
    check(lib().b200_nvfp4_gemm_bf16(_ptr(y), C.byref(ref), _ptr(x_bf16), M, W.N, K, _ptr(ws), stream_ptr(stream)), 'b200_nvfp4_gemm_bf16')
    return y


def gemm_bf16_exact(W, x_bf16, y=None, ws=None, stream=None):
    """The exact wide GEMM: y[M,N] f32 = x[M,K] bf16 . W^T, weights dequantised to fp16 in the kernel."""
    M, K = x_bf16.shape
    assert W.K == K and x_bf16.dtype == torch.bfloat16
    if y is None:
        y = torch.empty((M, W.N), dtype=torch.float32, device=x_bf16.device)
    if ws is None:
        ws = torch.empty(lib().b200_nvfp4_gemm_bf16_exact_workspace_bytes(M, K), dtype=torch.uint8, device=x_bf16.device)
    ref = W.wref()
    check(lib().b200_nvfp4_gemm_bf16_exact(_ptr(y), C.byref(ref), _ptr(x_bf16), M, W.N, K, _ptr(ws), stream_ptr(stream)), 'b200_nvfp4_gemm_bf16_exact')
    return y


def quantize_tokens(x, stream=None):
    """Per-token NVFP4 quantisation of x [M,K] (bf16 or f32): packed [M,K/2], scale [M,K/16] (returned
    row-major; the library writes it step-major), gs [M]."""
    M, K = x.shape
    dev = x.device
    packed = torch.empty((M, K // 2), dtype=torch.uint8, device=dev)
    sfb = torch.empty((K // 256, M, 16), dtype=torch.uint8, device=dev)
    gs = torch.empty(M, dtype=torch.float32, device=dev)
    check(lib().b200_nvfp4_quantize_tokens(_ptr(x), 1 if x.dtype == torch.float32 else 0, M, K, _ptr(packed), _ptr(sfb), _ptr(gs),
                                           stream_ptr(stream)), 'b200_nvfp4_quantize_tokens')
    return packed, sfb.permute(1, 0, 2).reshape(M, K // 16).contiguous(), gs


def dense_mlp_workspace(M, hidden, inter, device):
    return torch.empty(lib().b200_dense_mlp_workspace_bytes(M, hidden, inter), dtype=torch.uint8, device=device)


def dense_mlp(x, gate, up, down, limit=10.0, y=None, ws=None, stream=None):
    """y = down . (silu(min(gate.x, limit)) * clamp(up.x, -limit, limit)); x [M, hidden] f32."""
    M, H = x.shape
    I = gate.N
    if y is None:
        y = torch.empty((M, H), dtype=torch.float32, device=x.device)
    if ws is None:
        ws = dense_mlp_workspace(M, H, I, x.device)
    g, u, d = gate.wref(), up.wref(), down.wref()
    check(lib().b200_dense_mlp(_ptr(x), C.byref(g), C.byref(u), C.byref(d), H, I, float(limit), _ptr(y), _ptr(ws), M, stream_ptr(stream)),
          'b200_dense_mlp')
    return y


def gemv(W, x, y=None, stream=None):
    return gemm(W, x, y, stream=stream)


def make_jobs(weights, xs, ys):
    arr = (GemvJob * len(weights))()
    for i, (W, x, y) in enumerate(zip(weights, xs, ys)):
        arr[i] = GemvJob(y.data_ptr(), W.wref(), x.data_ptr(), W.N)
    return arr


def gemv_multi(weights, xs, M=1, ys=None, stream=None, jobs=None, ws=None):
    """Fused group: weights share K; xs is one tensor [M,K] (shared) or a list (one per job)."""
    if not isinstance(xs, (list, tuple)):
        xs = [xs] * len(weights)
    if ys is None:
        ys = [torch.empty((M, W.N), dtype=torch.float32, device=xs[0].device) for W in weights]
    if jobs is None:
        jobs = make_jobs(weights, xs, ys)
    if ws is not None:
        check(lib().b200_nvfp4_gemv_multi_ws(jobs, len(weights), M, weights[0].K, BF16, _ptr(ws), stream_ptr(stream)), 'b200_nvfp4_gemv_multi_ws')
    else:
        check(lib().b200_nvfp4_gemv_multi(jobs, len(weights), M, weights[0].K, BF16, stream_ptr(stream)), 'b200_nvfp4_gemv_multi')
    return ys


def f32_to_bf16(src, stream=None):
    dst = torch.empty(src.shape, dtype=torch.bfloat16, device=src.device)
    check(lib().b200_f32_to_bf16(_ptr(dst), _ptr(src), src.numel(), stream_ptr(stream)), 'b200_f32_to_bf16')
    return dst


def bf16_to_f32(src, stream=None):
    dst = torch.empty(src.shape, dtype=torch.float32, device=src.device)
    check(lib().b200_bf16_to_f32(_ptr(dst), _ptr(src), src.numel(), stream_ptr(stream)), 'b200_bf16_to_f32')
    return dst


def quantize(w_bf16, gscale_in=None, out=None, stream=None):
    """bf16 [N,K] device tensor -> Nvfp4Weight, bit-exact with the reference quantiser."""
    N, K = w_bf16.shape
    dev = w_bf16.device
    if out is None:
        out = Nvfp4Weight(torch.empty((N, K // 2), dtype=torch.uint8, device=dev),
                          torch.empty((N, K // 16), dtype=torch.uint8, device=dev),
                          torch.empty(1, dtype=torch.float32, device=dev), device=dev)
    check(lib().b200_nvfp4_quantize(_ptr(w_bf16), N, K, _ptr(out.packed), _ptr(out.scale), _ptr(out.gscale),
                                    _ptr(gscale_in), stream_ptr(stream)), 'b200_nvfp4_quantize')
    return out


def dequantize(W, stream=None):
    out = torch.empty((W.N, W.K), dtype=torch.float32, device=W.packed.device)
    m = W.mat()
    check(lib().b200_nvfp4_dequantize(_ptr(out), C.byref(m), W.N, W.K, stream_ptr(stream)), 'b200_nvfp4_dequantize')
    return out


class MoeLayer:
    """Device-side description of one MoE layer: router, bias, expert pointer tables."""

    def __init__(self, router_bf16, bias, experts, shared, topk, hidden, inter, routed_scale=2.5,
                 swiglu_limit=10.0, norm_topk=True):
        """experts: list of (gate, up, down) Nvfp4Weight; shared: one such triple or None."""
        dev = router_bf16.device
        self.router, self.bias, self.experts, self.shared = router_bf16, bias, experts, shared
        flat = []
        for g, u, d in experts:
            for w in (g, u, d):
                flat += [w.packed.data_ptr(), w.scale.data_ptr(), w.gscale.data_ptr()]
        self.table = torch.tensor(flat, dtype=torch.int64).to(dev)
        self.shared_table = None
        if shared is not None:
            fl = []
            for w in shared:
                fl += [w.packed.data_ptr(), w.scale.data_ptr(), w.gscale.data_ptr()]
            self.shared_table = torch.tensor(fl, dtype=torch.int64).to(dev)
        self.c = MoeLayerC(WRef(router_bf16.data_ptr(), None, None, None), bias.data_ptr(), self.table.data_ptr(),
                           self.shared_table.data_ptr() if shared is not None else None,
                           len(experts), topk, hidden, inter, routed_scale, swiglu_limit, 1 if norm_topk else 0)
        self.topk, self.hidden, self.inter, self.n_expert = topk, hidden, inter, len(experts)
        self._ws = {}

    def workspace(self, M):
        if M not in self._ws:
            n = lib().b200_moe_workspace_bytes(C.byref(self.c), M)
            self._ws[M] = torch.empty(n, dtype=torch.uint8, device=self.router.device)
        return self._ws[M]


def moe_route(layer, x, stream=None):
    x2 = x if x.dim() == 2 else x.unsqueeze(0)
    M = x2.shape[0]
    sel = torch.empty((M, layer.topk), dtype=torch.int32, device=x.device)
    wts = torch.empty((M, layer.topk), dtype=torch.float32, device=x.device)
    logits = torch.empty((M, layer.n_expert), dtype=torch.float32, device=x.device)
    check(lib().b200_moe_route(_ptr(x2), C.byref(layer.c), _ptr(sel), _ptr(wts), _ptr(logits), M, stream_ptr(stream)), 'b200_moe_route')
    return sel, wts, logits


def moe_forward(layer, x, y=None, sel=None, wts=None, stream=None):
    x2 = x if x.dim() == 2 else x.unsqueeze(0)
    M = x2.shape[0]
    dev = x.device
    y = torch.empty((M, layer.hidden), dtype=torch.float32, device=dev) if y is None else y
    sel = torch.empty((M, layer.topk), dtype=torch.int32, device=dev) if sel is None else sel
    wts = torch.empty((M, layer.topk), dtype=torch.float32, device=dev) if wts is None else wts
    ws = layer.workspace(M)
    check(lib().b200_moe_forward(_ptr(x2), C.byref(layer.c), _ptr(y), _ptr(sel), _ptr(wts), _ptr(ws), M, stream_ptr(stream)), 'b200_moe_forward')
    return y, sel, wts


def moe_prepare(layer):
    """Build the layer's TMA descriptors so that batches of up to 8 tokens run on the tensor-core
    kernels.  Returns False when the geometry does not suit them (the layer keeps the CUDA-core path)."""
    rc = lib().b200_moe_prepare(C.byref(layer.c))
    if rc == ENOTIMPL:
        return False
    check(rc, 'b200_moe_prepare')
    return True


def moe_release(layer):
    check(lib().b200_moe_release(C.byref(layer.c)), 'b200_moe_release')


def moe_experts(layer, x, sel, wts, y=None, stream=None):
    x2 = x if x.dim() == 2 else x.unsqueeze(0)
    M = x2.shape[0]
    y = torch.empty((M, layer.hidden), dtype=torch.float32, device=x.device) if y is None else y
    ws = layer.workspace(M)
    check(lib().b200_moe_experts(_ptr(x2), C.byref(layer.c), _ptr(y), _ptr(sel), _ptr(wts), _ptr(ws), M, stream_ptr(stream)), 'b200_moe_experts')
    return y


def moe_forward_static(layer, x, y=None, sel=None, wts=None, stream=None):
    """moe_forward through the library's built-in scratch (no workspace tensor is created here)."""
    x2 = x if x.dim() == 2 else x.unsqueeze(0)
    M = x2.shape[0]
    dev = x.device
    y = torch.empty((M, layer.hidden), dtype=torch.float32, device=dev) if y is None else y
    sel = torch.empty((M, layer.topk), dtype=torch.int32, device=dev) if sel is None else sel
    wts = torch.empty((M, layer.topk), dtype=torch.float32, device=dev) if wts is None else wts
    check(lib().b200_moe_forward_static(_ptr(x2), C.byref(layer.c), _ptr(y), _ptr(sel), _ptr(wts), M, stream_ptr(stream)),
          'b200_moe_forward_static')
    return y, sel, wts


def ep_unique_id():
    """128 bytes that identify a new NCCL communicator (call on one rank, hand to all)."""
    buf = C.create_string_buffer(128)
    check(lib().b200_ep_unique_id(buf), 'b200_ep_unique_id')
    return buf.raw


class EpContext:
    """An expert-parallel layer context of the library (b200_ep_*): this object only holds the handle."""

    def __init__(self, router, local, shared, rank, world, max_tokens, unique_id=None):
        self.h = C.c_void_p(0)
        self.router, self.local, self.shared = router, local, shared      # keep the tables alive
        idbuf = C.create_string_buffer(unique_id, 128) if unique_id is not None else None
        check(lib().b200_ep_create(C.byref(self.h), idbuf, rank, world, C.byref(router.c), C.byref(local.c),
                                   C.byref(shared.c) if shared is not None else None, max_tokens), 'b200_ep_create')

    def forward(self, x, y=None, sel=None, wts=None, stream=None):
        T, dev = x.shape[0], x.device
        y = torch.empty((T, self.router.hidden), dtype=torch.float32, device=dev) if y is None else y
        sel = torch.empty((T, self.router.topk), dtype=torch.int32, device=dev) if sel is None else sel
        wts = torch.empty((T, self.router.topk), dtype=torch.float32, device=dev) if wts is None else wts
        check(lib().b200_ep_forward(self.h, _ptr(x), _ptr(y), _ptr(sel), _ptr(wts), T, stream_ptr(stream)), 'b200_ep_forward')
        return y, sel, wts

    def stats(self):
        st = EpStats()
        check(lib().b200_ep_last_stats(self.h, C.byref(st)), 'b200_ep_last_stats')
        return {k: getattr(st, k) for k, _ in EpStats._fields_ if not k.startswith('pad')}

    def close(self):
        if self.h:
            check(lib().b200_ep_destroy(self.h), 'b200_ep_destroy')
            self.h = C.c_void_p(0)


class OverlayWriter:
    """safetensors overlay of NVFP4 triples, byte-compatible with the reference's requant tool."""

    def __init__(self, directory, shard_bytes=0):
        self.h = C.c_void_p(0)
        check(lib().b200_overlay_writer_open(C.byref(self.h), directory.encode(), shard_bytes), 'b200_overlay_writer_open')

    def add(self, name, packed, scale, gscale):
        """packed u8 [N,K/2], scale u8 [N,K/16]: numpy arrays (host); gscale: float."""
        packed = np.ascontiguousarray(packed, np.uint8); scale = np.ascontiguousarray(scale, np.uint8)
        N, K = packed.shape[0], packed.shape[1] * 2
        check(lib().b200_overlay_writer_add(self.h, name.encode(), packed.ctypes.data_as(C.c_void_p), scale.ctypes.data_as(C.c_void_p),
                                            C.c_float(float(gscale)), N, K), 'b200_overlay_writer_add')

    def close(self):
        check(lib().b200_overlay_writer_close(self.h), 'b200_overlay_writer_close')
        self.h = C.c_void_p(0)


def overlay_family(arch, families, name):
    return lib().b200_overlay_family(arch.encode(), families.encode() if families else None, name.encode())


class Overlay:
    """Reader: maps an overlay directory; triple(name) -> (packed, scale, gscale) numpy copies."""

    def __init__(self, directory):
        self.h = C.c_void_p(0)
        check(lib().b200_overlay_open(C.byref(self.h), directory.encode()), 'b200_overlay_open')

    def __len__(self):
        return lib().b200_overlay_count(self.h)

    def triple(self, name):
        e = OverlayEntry()
        check(lib().b200_overlay_find(self.h, name.encode(), C.byref(e)), 'b200_overlay_find')
        p = np.ctypeslib.as_array(C.cast(e.packed, C.POINTER(C.c_uint8)), shape=(e.N, e.K // 2)).copy()
        s = np.ctypeslib.as_array(C.cast(e.scale, C.POINTER(C.c_uint8)), shape=(e.N, e.K // 16)).copy()
        return p, s, np.array([e.gscale], np.float32), (e.packed % 16 == 0 and e.scale % 16 == 0)

    def close(self):
        check(lib().b200_overlay_close(self.h), 'b200_overlay_close')
        self.h = C.c_void_p(0)


CREDIT_FN = C.CFUNCTYPE(None, C.c_int, C.c_double, C.c_void_p)


class ByteCredit:
    """Collects the weight bytes the library reports per launch site (b200_nvfp4_set_byte_credit)."""

    def __init__(self):
        self.by_kind = {}
        self._cb = CREDIT_FN(lambda kind, nbytes, user: self.by_kind.__setitem__(kind, self.by_kind.get(kind, 0.0) + nbytes))

    def __enter__(self):
        check(lib().b200_nvfp4_set_byte_credit(C.cast(self._cb, C.c_void_p), None), 'b200_nvfp4_set_byte_credit')
        return self

    def flush(self, credit=True):
        check(lib().b200_nvfp4_flush_byte_credit(1 if credit else 0), 'b200_nvfp4_flush_byte_credit')

    def __exit__(self, *a):
        check(lib().b200_nvfp4_set_byte_credit(None, None), 'b200_nvfp4_set_byte_credit')
