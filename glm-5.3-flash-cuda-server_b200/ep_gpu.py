"""Test and benchmark plumbing for the expert-parallel MoE layer: builds this rank's shard of a seeded
layer as library objects and opens the library's expert-parallel context (b200_ep_*, C++ + NCCL inside
libb200nvfp4.so) on it.  Nothing here computes or communicates; weights are seeded per global expert
id, so every world size sees the same model and EP(G) can be checked against EP(1)."""
import torch
from . import binding as B


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


def shared_unique_id(rank, world):
    """One NCCL unique id made on rank 0 and handed to every rank over torch.distributed."""
    if world == 1:
        return None
    import torch.distributed as dist
    box = [B.ep_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    return box[0]


class RankLayer:
    """One MoE layer as rank `rank` of `world` holds it: router + bias + shared expert replicated,
    experts [rank*E/world, (rank+1)*E/world) local; `ctx` is the library's expert-parallel context."""

    def __init__(self, seed, layer, E, topk, H, I, rank, world, device, max_tokens, popularity_bias=None):
        self.E, self.topk, self.H, self.I = E, topk, H, I
        epr = E // world
        self.router, self.bias = router_weights(seed, layer, E, H, device)
        if popularity_bias is not None:
            self.bias = self.bias + popularity_bias.to(device)
        self.local = [expert_weights(seed, layer, rank * epr + j, H, I, device) for j in range(epr)]
        self.shared_w = expert_weights(seed, layer, E, H, I, device)
        # three views of the same weights for the library: the router over all E experts (its expert table is
        # never read), the local shard as a layer with topk = 1, the shared expert as a one-expert layer
        self.l_route = B.MoeLayer(self.router, self.bias, self.local, None, topk, H, I)
        self.l_route.c.n_expert = E
        self.l_route.n_expert = E
        self.l_local = B.MoeLayer(self.router, self.bias, self.local, None, 1, H, I)
        self.l_shared = B.MoeLayer(self.router, self.bias, [self.shared_w], None, 1, H, I)
        self.tensor_core = B.moe_prepare(self.l_local) and B.moe_prepare(self.l_shared)
        self.ctx = B.EpContext(self.l_route, self.l_local, self.l_shared, rank, world, max_tokens, shared_unique_id(rank, world))
        self.expert_bytes = 3 * (I * H // 2 + I * H // 16 + 4)

    def forward(self, x, y=None, sel=None, wts=None):
        return self.ctx.forward(x, y, sel, wts)

    def step_bytes(self, T_local, stats):
        """Algorithmic bytes of a forward on this rank: local expert weights touched once each + the
        shared expert, router, local tokens in and out, dispatched rows in (bf16) and out (f32)."""
        return ((stats['local_experts_touched'] + 1) * self.expert_bytes + self.E * self.H * 2 + self.E * 4
                + 2 * T_local * self.H * 4 + stats['recv_rows'] * self.H * 6)

    def close(self):
        self.ctx.close()
        B.moe_release(self.l_local); B.moe_release(self.l_shared)
