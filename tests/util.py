"""Helpers shared by the GPU tests: seeded weights, device upload, oracle/C-oracle loaders."""
import ctypes as C
import os
import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
import __graft_entry__ as G  # noqa: E402  (conftest puts ROOT on sys.path)

REL_TOL, ABS_TOL = 1e-3, 2e-2      # the parity bar: rel-L2 and max-abs vs fp32 dequant-then-matmul


def pkg():
    return G.load_package()


def oracle():
    return G.load_oracle()


def seeded_bf16(shape, seed, std=0.02):
    O = oracle()
    return O.f32_to_bf16_bits(np.random.default_rng(seed).normal(0.0, std, shape).astype(np.float32))


def host_triple(shape, seed, std=0.02):
    O = oracle()
    return O.quantize_tensor(O.bf16_bits_to_f32(seeded_bf16(shape, seed, std)))


def to_dev_bf16(bits):
    import torch
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda().view(torch.bfloat16)


def c_oracle():
    path = os.path.join(ROOT, 'oracle', 'libnvfp4_oracle.so')
    if not os.path.exists(path):
        import subprocess
        subprocess.check_call(['make', '-C', os.path.join(ROOT, 'oracle'), 'libnvfp4_oracle.so'])
    L = C.CDLL(path)
    L.oracle_global_scale.restype = C.c_float
    L.oracle_global_scale.argtypes = [C.c_void_p, C.c_size_t]
    L.oracle_quantize.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p]
    L.oracle_dequant.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_int, C.c_void_p]
    L.oracle_gemm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_int, C.c_int, C.c_void_p]
    L.oracle_route.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p, C.c_void_p]
    L.oracle_threads.restype = C.c_int
    return L


def ref_kernels():
    """The reference's own CUDA kernels (built by oracle/Makefile where the reference checkout
    exists); None if the prebuilt library did not travel."""
    path = os.path.join(ROOT, 'oracle', '_ref', 'libref_kernels.so')
    if not os.path.exists(path):
        return None
    L = C.CDLL(path)
    vp, ci = C.c_void_p, C.c_int
    L.ref_gemm_nvfp4.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, vp]
    L.ref_gemm_bf16.argtypes = [vp, vp, vp, ci, ci, ci, vp]
    L.ref_gemv_multi.argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, vp]
    L.ref_moe_workspace_floats.restype = C.c_size_t; L.ref_moe_workspace_floats.argtypes = [ci]
    L.ref_moe_forward.argtypes = [vp, vp, vp, vp, vp, ci, ci, vp, vp, vp, vp, ci, vp]
    for f in ('ref_moe_hidden', 'ref_moe_inter', 'ref_moe_experts', 'ref_moe_topk'):
        getattr(L, f).restype = ci
    return L


def zipf_bias(E, s=1.1, seed=4, strength=0.08):
    """Expert popularity ~ Zipf(s) over a seeded permutation, as a router ranking bias (the same
    construction as the benchmark's skewed-routing configurations)."""
    rng = np.random.default_rng(seed)
    p = 1.0 / np.arange(1, E + 1) ** s
    p = p[rng.permutation(E)]
    return (strength * np.log(p / p.mean())).astype(np.float32)


class exact_prefill:
    """Context: calls with 16 or more rows keep fp32-activation accuracy (B200_OPT_PREFILL_FP4 = 0)."""

    def __enter__(self):
        pkg().set_option(pkg().OPT_PREFILL_FP4, 0)

    def __exit__(self, *a):
        pkg().set_option(pkg().OPT_PREFILL_FP4, 1)
