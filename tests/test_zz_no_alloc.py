"""The workspace-free MoE entry point, b200_moe_forward_static, against b200_moe_forward.

Some hosts of the library cannot hand it a workspace: an engine that sized its buffers at
start-up with the reference's own workspace formula and must not call cudaMalloc inside the token
loop.  For them the scratch is an array inside the library.  This file is named so that pytest
collects it last; it must pass both on its own in a fresh process (first use of the array on the
device) and after every other GPU test has run.
"""
import ctypes as C
import numpy as np
import pytest
import torch

from util import pkg, oracle, REL_TOL, ABS_TOL
from test_gpu_moe import build_layer

pytestmark = pytest.mark.gpu


def test_static_workspace_matches_caller_workspace_twice_in_a_row():
    P, O = pkg(), oracle()
    layer, d = build_layer(1024, 512, 32, 8, seed=9)
    rng = np.random.default_rng(3)
    ys = []
    for call in range(2):                           # the second call finds the first call's bytes in the array
        M = 2 if call == 0 else 3
        x = torch.from_numpy(rng.normal(0, 1, (M, 1024)).astype(np.float32)).cuda()
        y_ref, sel_ref, wts_ref = P.moe_forward(layer, x)
        y = torch.full((M, 1024), float('nan'), device='cuda')
        sel = torch.full((M, 8), -1, dtype=torch.int32, device='cuda')
        wts = torch.full((M, 8), float('nan'), device='cuda')
        P.moe_forward_static(layer, x, y, sel, wts)
        torch.cuda.synchronize()
        assert torch.equal(sel, sel_ref)
        assert (wts - wts_ref).abs().max().item() <= 1e-5
        r, a = O.rel_l2(y.cpu().numpy(), y_ref.cpu().numpy()), O.max_abs(y.cpu().numpy(), y_ref.cpu().numpy())
        assert r <= REL_TOL and a <= ABS_TOL, (call, r, a)
        assert torch.isfinite(y).all() and (y != 0).float().mean() > 0.9
        ys.append(y)
    # and against the CPU oracle, so that both entry points being wrong together would show
    xh = rng.normal(0, 1, (1, 1024)).astype(np.float32)
    y, sel, wts = P.moe_forward_static(layer, torch.from_numpy(xh).cuda())
    logits = O.router_logits(xh, d['rb'])
    sel_o, wts_o, _ = O.route(logits, d['bias'], 8)
    yo = O.moe_experts(xh, sel_o, wts_o, d['host'][:32], d['host'][32])
    assert O.rel_l2(y.cpu().numpy(), yo) <= REL_TOL
    assert P.device_status() == 0


def test_static_workspace_refuses_oversized_requests():
    P = pkg()
    layer, _ = build_layer(1024, 512, 32, 8, seed=9)
    limit = P.lib().b200_moe_static_ws_limit()
    assert limit == 1 << 20
    # this entry point's scratch: logits [M, E] + activations [M, topk + 1, inter], f32, 256-byte aligned parts
    up = lambda v: (v + 255) // 256 * 256
    need = lambda M: up(M * 32 * 4) + up(M * 9 * 512 * 4)
    M = next(m for m in range(1, 1 << 12) if need(m) > limit) + 8
    x = torch.zeros((M, 1024), device='cuda')
    with pytest.raises(P.B200Error, match='documented maximum'):
        P.moe_forward_static(layer, x)
