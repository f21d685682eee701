"""The C-ABI library loads and exports every symbol include/b200_nvfp4.h declares (no GPU work),
and the host-side argument checks answer with the documented codes."""
import ctypes as C
import os
import re
import pytest
import __graft_entry__ as G

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for f in os.listdir(os.path.join(ROOT, 'include')):
        if f.endswith('.h'):
            src = open(os.path.join(ROOT, 'include', f)).read()
            src = re.sub(r'/\*.*?\*/', '', src, flags=re.S)
            names |= set(re.findall(r'\b(b200_[a-z0-9_]+)\s*\(', src))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    pkg = G.load_package()
    if not os.path.exists(pkg.LIB_PATH):
        G.build()
    L = pkg.lib()
    syms = declared_symbols()
    assert len(syms) >= 12
    for s in syms:
        assert hasattr(L, s), 'missing export: ' + s
    assert set(pkg.EXPORTS) <= set(syms)
    assert L.b200_nvfp4_version() >= 100
    assert L.b200_nvfp4_strerror(2).decode().startswith('unsupported shape')


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    pkg = G.load_package()
    import importlib
    b = importlib.import_module(G.PKG_NAME + '.binding')
    monkeypatch.setattr(b, '_lib', None)
    monkeypatch.setattr(b, 'LIB_PATH', str(tmp_path / 'nope.so'))
    with pytest.raises(pkg.B200Error):
        b.lib()


def test_argument_checks_without_gpu():
    pkg = G.load_package()
    L = pkg.lib()
    # every one of these is rejected on the host before any CUDA call is made
    assert L.b200_nvfp4_gemm(None, None, None, 1, 8, 32, 1, None) == 1
    j = (pkg.GemvJob * 1)()
    assert L.b200_nvfp4_gemv_multi(j, 0, 1, 32, 1, None) == 1
    assert L.b200_nvfp4_gemv_multi(j, 9, 1, 32, 1, None) == 1
    assert L.b200_nvfp4_gemv_multi(j, 1, 9, 32, 1, None) == 1
    j[0] = pkg.GemvJob(16, pkg.WRef(None, 16, 16, 16), 16, 4)
    assert L.b200_nvfp4_gemv_multi(j, 1, 1, 40, 1, None) == 2          # K % 16 != 0
    j[0] = pkg.GemvJob(16, pkg.WRef(None, 18, 16, 16), 16, 4)
    assert L.b200_nvfp4_gemv_multi(j, 1, 1, 32, 1, None) == 3          # packed not 4-byte aligned
    assert L.b200_nvfp4_quantize(16, 4, 24, 16, 16, 16, None, None) == 2
    layer = pkg.MoeLayerC()
    assert L.b200_moe_forward(16, C.byref(layer), 16, 16, 16, 16, 1, None) == 1
    layer = pkg.MoeLayerC(pkg.WRef(16, None, None, None), 16, 16, None, 600, 8, 4096, 1536, 2.5, 10.0, 1)
    assert L.b200_moe_forward(16, C.byref(layer), 16, 16, 16, 16, 1, None) == 5   # n_expert > 512
    layer = pkg.MoeLayerC(pkg.WRef(16, None, None, None), 16, 16, None, 144, 8, 4100, 1536, 2.5, 10.0, 1)
    assert L.b200_moe_forward(16, C.byref(layer), 16, 16, 16, 16, 1, None) == 2
