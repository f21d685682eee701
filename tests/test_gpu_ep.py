"""The library's expert-parallel context on one GPU (world size 1 exercises plan, pack, local copy,
unpack, local experts, combine, shared expert on the second stream) against the single-call MoE
entry point and the oracle; the exchange between ranks is covered by the 2-GPU benchmark run (which
asserts parity) and, for the host protocol, by the two-rank gloo test on CPU."""
import numpy as np
import pytest
import torch

from util import pkg, oracle, exact_prefill, REL_TOL

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('T', [6, 40])
def test_ep_world1_equals_moe_forward(T):
    P, O = pkg(), oracle()
    E, topk, H, I = 16, 4, 1024, 512
    dev = torch.device('cuda', 0)
    L = P.ep_gpu.RankLayer(7, 0, E, topk, H, I, 0, 1, dev, max_tokens=64)
    try:
        x = torch.randn((T, H), device=dev).to(torch.bfloat16).float()        # rows travel as bf16: use bf16-valued tokens
        y, sel, wts = L.forward(x)
        full = [P.ep_gpu.expert_weights(7, 0, e, H, I, dev) for e in range(E + 1)]
        ref = P.MoeLayer(L.router, L.bias, full[:E], full[E], topk, H, I)
        assert L.tensor_core and P.moe_prepare(ref)
        y_ref, sel_ref, wts_ref = P.moe_forward(ref, x)
        assert torch.equal(sel, sel_ref) and torch.equal(wts, wts_ref)
        # same kernels per row on both sides (rows are computed on their own), summed in the same slot order
        assert ((y - y_ref).norm() / y_ref.norm()).item() < 1e-6
        st = L.ctx.stats()
        assert st['recv_rows'] == T * topk and st['sent_remote_rows'] == 0 and 1 <= st['local_experts_touched'] <= E
        assert L.step_bytes(T, st) > 0
        # against the oracle (exact experts, so that the plain oracle applies)
        with exact_prefill():
            y_ex, _, _ = L.forward(x)
        host = [tuple(w.numpy() for w in t) for t in full]
        sel_o, wts_o, gap = O.route(O.router_logits(x.cpu().numpy(), O.f32_to_bf16_bits(L.router.float().cpu().numpy())), L.bias.cpu().numpy(), topk)
        assert gap.min() > 1e-6 and np.array_equal(sel.cpu().numpy(), sel_o)
        yo = O.moe_experts(x.cpu().numpy(), sel_o, wts_o, host[:E], host[E])
        assert O.rel_l2(y_ex.cpu().numpy(), yo) <= REL_TOL
        y2, _, _ = L.forward(x)
        assert torch.equal(y2, y)                      # run to run
        assert P.device_status() == 0
        P.moe_release(ref)
    finally:
        L.close()


def test_ep_rejects_too_many_tokens_and_bad_arguments():
    P = pkg()
    dev = torch.device('cuda', 0)
    L = P.ep_gpu.RankLayer(3, 0, 8, 2, 256, 256, 0, 1, dev, max_tokens=4)
    try:
        with pytest.raises(P.B200Error):
            L.forward(torch.randn((5, 256), device=dev))
    finally:
        L.close()
