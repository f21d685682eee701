"""Host logic of the expert-parallel MoE layer on CPU: two gloo ranks, expert arithmetic supplied by
the CPU oracle, result compared with the oracle's single-process layer.  (The GPU path uses the
same ExpertParallelMoE class with library calls as its closures.)"""
import os
import socket
import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import __graft_entry__ as G


def _free_port():
    s = socket.socket(); s.bind(('127.0.0.1', 0)); p = s.getsockname()[1]; s.close(); return p


def _model(H, I, E):
    O = G.load_oracle()
    rng = np.random.default_rng(11)
    q = lambda o, i: O.quantize_tensor(O.bf16_bits_to_f32(O.f32_to_bf16_bits(rng.normal(0, 0.02, (o, i)).astype(np.float32))))
    experts = [(q(I, H), q(I, H), q(H, I)) for _ in range(E + 1)]
    rb = O.f32_to_bf16_bits(rng.normal(0, 0.05, (E, H)).astype(np.float32))
    bias = rng.normal(0, 0.1, E).astype(np.float32)
    return experts, rb, bias


def _rank(rank, world, port, T, H, I, E, topk, out):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    O = G.load_oracle()
    pkg_dir = G.PKG_DIR
    import importlib.util
    spec = importlib.util.spec_from_file_location('ep_only', os.path.join(pkg_dir, 'ep.py'))
    ep = importlib.util.module_from_spec(spec); spec.loader.exec_module(ep)
    experts, rb, bias = _model(H, I, E)
    epr = E // world
    x_all = np.random.default_rng(5).normal(0, 1, (T, H)).astype(np.float32)
    x = torch.from_numpy(x_all[rank * (T // world):(rank + 1) * (T // world)])

    def route(xt):
        sel, wts, _ = O.route(O.router_logits(xt.numpy(), rb), bias, topk)
        return torch.from_numpy(sel), torch.from_numpy(wts)

    def compute(rows, eid):
        outs = [O.expert_mlp(rows[i:i + 1].numpy(), *experts[rank * epr + int(eid[i])])[0][0] for i in range(rows.shape[0])]
        return torch.from_numpy(np.stack(outs).astype(np.float32)) if outs else rows

    def shared(xt):
        return torch.from_numpy(O.expert_mlp(xt.numpy(), *experts[E])[0].astype(np.float32))

    layer = ep.ExpertParallelMoE(E, topk, H, route, compute, shared)
    y, sel, wts = layer.forward(x)
    out[rank] = (y.numpy(), sel.numpy(), layer.last_stats)
    dist.barrier()
    dist.destroy_process_group()


def test_dispatch_plan_is_stable_and_complete():
    import importlib.util
    spec = importlib.util.spec_from_file_location('ep_only', os.path.join(G.PKG_DIR, 'ep.py'))
    ep = importlib.util.module_from_spec(spec); spec.loader.exec_module(ep)
    sel = torch.tensor([[5, 0, 7], [1, 6, 2], [7, 7, 0]], dtype=torch.int32)
    order, counts = ep.dispatch_plan(sel, 2, 4)          # experts 0-1 -> rank 0, 2-3 -> 1, 4-5 -> 2, 6-7 -> 3
    assert counts.tolist() == [3, 1, 1, 4]
    assert order.tolist() == [1, 3, 8, 5, 0, 2, 4, 6, 7]   # by rank, then by (token, slot)


def test_ep_two_ranks_matches_single_process():
    T, H, I, E, topk, world = 8, 64, 32, 8, 2, 2
    port = _free_port()
    mgr = mp.Manager(); out = mgr.dict()
    mp.spawn(_rank, args=(world, port, T, H, I, E, topk, out), nprocs=world, join=True)
    O = G.load_oracle()
    experts, rb, bias = _model(H, I, E)
    x_all = np.random.default_rng(5).normal(0, 1, (T, H)).astype(np.float32)
    y_ref, sel_ref, _, _, _ = O.moe_layer(x_all, rb, bias, experts[:E], experts[E], topk)
    y = np.concatenate([out[r][0] for r in range(world)])
    sel = np.concatenate([out[r][1] for r in range(world)])
    assert np.array_equal(sel, sel_ref)
    assert O.rel_l2(y, y_ref) < 1e-5
    assert sum(out[r][2]['recv_rows'] for r in range(world)) == T * topk
