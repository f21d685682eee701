"""Expert-parallel layer on one GPU (world size 1 exercises plan, gather, expert call, combine)
against the single-call MoE entry point; the two-rank exchange itself is covered on CPU (gloo)."""
import numpy as np
import pytest
import torch

from util import pkg, oracle, REL_TOL

pytestmark = pytest.mark.gpu


def test_ep_world1_equals_moe_forward():
    P = pkg()
    E, topk, H, I = 16, 4, 1024, 512
    dev = torch.device('cuda', 0)
    L = P.ep_gpu.RankLayer(7, 0, E, topk, H, I, 0, 1, dev)
    x = torch.randn((6, H), device=dev)
    y, sel, wts = L.forward(x)
    full = [P.ep_gpu.expert_weights(7, 0, e, H, I, dev) for e in range(E + 1)]
    ref = P.MoeLayer(L.router, L.bias, full[:E], full[E], topk, H, I)
    assert L.tensor_core and P.moe_prepare(ref)        # both sides on the tensor-core experts
    y_ref, sel_ref, wts_ref = P.moe_forward(ref, x)
    assert torch.equal(sel, sel_ref) and torch.equal(wts, wts_ref)
    assert ((y - y_ref).norm() / y_ref.norm()).item() < 1e-5
    assert L.ep.last_stats['recv_rows'] == 6 * topk
    assert L.step_bytes(6) > 0
