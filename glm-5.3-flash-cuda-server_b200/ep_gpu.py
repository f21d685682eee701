"""GPU side of the expert-parallel MoE layer: this rank's expert shard as library objects, and the
three closures ExpertParallelMoE needs (route / compute / shared), all of them calls into
libb200nvfp4.so.  Weights are seeded per global expert id, so every world size sees the same
model and EP(G) can be checked against EP(1)."""
import torch
from . import binding as B
from .ep import ExpertParallelMoE


def expert_weights(seed, layer, e, H, I, device):
    """(gate, up, down) of global expert e (e == n_expert means the shared expert), quantised here."""
    g = torch.Generator(device=device).manual_seed(seed * 1000003 + layer * 1009 + e)
    tr = []
    for (o, i) in ((I, H), (I, H), (H, I)):
        w = (torch.randn((o, i), generator=g, device=device) * 0.02).to(torch.bfloat16)
        tr.append(B.quantize(w))
    return tuple(tr)


def router_weights(seed, layer, E, H, device):
    g = torch.Generator(device=device).manual_seed(seed * 7919 + layer)
    router = (torch.randn((E, H), generator=g, device=device) * 0.02).to(torch.bfloat16)
    bias = torch.randn(E, generator=g, device=device) * 0.1
    return router, bias


class RankLayer:
    """One MoE layer as rank `rank` of `world` holds it: router + bias + shared expert replicated,
    experts [rank*E/world, (rank+1)*E/world) local."""

    def __init__(self, seed, layer, E, topk, H, I, rank, world, device, group=None, popularity_bias=None):
        self.E, self.topk, self.H, self.I = E, topk, H, I
        epr = E // world
        self.router, self.bias = router_weights(seed, layer, E, H, device)
        if popularity_bias is not None:
            self.bias = self.bias + popularity_bias.to(device)
        self.local = [expert_weights(seed, layer, rank * epr + j, H, I, device) for j in range(epr)]
        self.shared_w = expert_weights(seed, layer, E, H, I, device)
        # three views of the same weights for the three library calls
        self.l_route = B.MoeLayer(self.router, self.bias, self.local, None, topk, H, I)
        self.l_route.c.n_expert = E                       # the router ranks all E experts; no expert is touched
        self.l_route.n_expert = E
        self.l_local = B.MoeLayer(self.router, self.bias, self.local, None, 1, H, I)
        self.l_shared = B.MoeLayer(self.router, self.bias, [self.shared_w], None, 1, H, I)
        # descriptors for the tensor-core experts (rows grouped by local expert); False = geometry unsuitable
        self.tensor_core = B.moe_prepare(self.l_local) and B.moe_prepare(self.l_shared)
        self.ep = ExpertParallelMoE(E, topk, H, self.route, self.compute, self.shared, group)
        self.expert_bytes = 3 * (I * H // 2 + I * H // 16 + 4)

    def route(self, x):
        sel, wts, _ = B.moe_route(self.l_route, x)
        return sel, wts

    def compute(self, rows, eid):
        R = rows.shape[0]
        ones = torch.ones((R, 1), dtype=torch.float32, device=rows.device)
        return B.moe_experts(self.l_local, rows.contiguous(), eid.view(R, 1).contiguous(), ones)

    def shared(self, x):
        T = x.shape[0]
        z = torch.zeros((T, 1), dtype=torch.int32, device=x.device)
        ones = torch.ones((T, 1), dtype=torch.float32, device=x.device)
        return B.moe_experts(self.l_shared, x, z, ones)

    def forward(self, x):
        return self.ep.forward(x)

    def step_bytes(self, T_local):
        """Algorithmic bytes of the last forward on this rank: expert weights touched once each,
        router, local tokens in and out, dispatched rows in and out."""
        s = self.ep.last_stats
        return ((s['local_experts_touched'] + 1) * self.expert_bytes + self.E * self.H * 2 + self.E * 4
                + 2 * T_local * self.H * 4 + 2 * s['recv_rows'] * self.H * 4)
