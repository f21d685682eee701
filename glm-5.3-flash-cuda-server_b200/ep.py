"""Expert-parallel MoE layer: experts sharded over the ranks of one node, one all-to-all each way.

The reference is single-GPU (all 144 experts behind one device-side table, src/engine.cu:168-195);
this file is the multi-GPU form the benchmark's expert-parallel configuration asks for.  One
process per GPU; torch.distributed is the plumbing (NCCL on GPUs, gloo in the CPU tests); the
expert arithmetic is the library's (`compute` below), never a CPU fallback on a GPU run.

Per layer, on every rank:
  1. route the rank's own tokens (router and bias are replicated)               -> sel, wts
  2. dispatch: each (token, slot) pair goes to the rank that owns expert sel; rows are ordered
     by (destination rank, token, slot) -- a stable sort, so the plan is deterministic;
     an all-to-all of the per-rank counts, then one all-to-all of the token rows and one of
     the local expert ids
  3. the owner runs the expert MLP on every row it received (local memory only)
  4. combine: the reverse all-to-all returns one output row per pair to the token's home rank
  5. home rank: y[t] = sum over slots in slot order of wts[t,k] * out[pair(t,k)] + shared(x[t])
     (the reference's fixed-order gate sum, kernels/moe.cu:584-597; shared expert replicated)
Experts are contiguous by id: rank r owns [r*E/G, (r+1)*E/G).
"""
import torch
import torch.distributed as dist


def owner_of(sel, experts_per_rank):
    return torch.div(sel, experts_per_rank, rounding_mode='floor')


def dispatch_plan(sel, experts_per_rank, world):
    """sel int [T, topk] -> (order, send_counts): `order` lists pair indices (t*topk+k) sorted by
    destination rank, stable; send_counts[g] = pairs going to rank g."""
    dest = owner_of(sel.reshape(-1).to(torch.int64), experts_per_rank)
    order = torch.sort(dest, stable=True)[1]
    counts = torch.bincount(dest, minlength=world)
    return order, counts


class ExpertParallelMoE:
    """route(x) -> (sel int32 [T,topk], wts f32 [T,topk]);
    compute(rows f32 [R,H], local_expert int32 [R]) -> f32 [R,H]  (expert MLP of the local shard);
    shared(x) -> f32 [T,H] or None."""

    def __init__(self, n_expert, topk, hidden, route, compute, shared, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        assert n_expert % self.world == 0, 'experts must divide evenly over the ranks'
        self.epr = n_expert // self.world
        self.topk, self.hidden = topk, hidden
        self.route, self.compute, self.shared = route, compute, shared
        self.last_stats = {}

    def forward(self, x):
        T, H = x.shape
        sel, wts = self.route(x)
        order, send_counts = dispatch_plan(sel, self.epr, self.world)
        tok = torch.div(order, self.topk, rounding_mode='floor')
        send_rows = x.index_select(0, tok)
        send_eid = (sel.reshape(-1).to(torch.int64).index_select(0, order) % self.epr).to(torch.int32)
        if self.world > 1:
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts, group=self.group)
            sc, rc = send_counts.tolist(), recv_counts.tolist()          # host sync: NCCL needs the splits
            R = int(sum(rc))
            recv_rows = torch.empty((R, H), dtype=x.dtype, device=x.device)
            recv_eid = torch.empty((R,), dtype=torch.int32, device=x.device)
            dist.all_to_all_single(recv_rows, send_rows, rc, sc, group=self.group)
            dist.all_to_all_single(recv_eid, send_eid, rc, sc, group=self.group)
        else:
            sc = rc = [int(send_counts.sum())]
            recv_rows, recv_eid = send_rows, send_eid
        out_rows = self.compute(recv_rows, recv_eid) if recv_rows.shape[0] else recv_rows
        if self.world > 1:
            back = torch.empty((order.numel(), H), dtype=x.dtype, device=x.device)
            dist.all_to_all_single(back, out_rows, sc, rc, group=self.group)
        else:
            back = out_rows
        # back[i] belongs to pair order[i]; put the pairs back in (token, slot) order
        pair_out = torch.empty_like(back)
        pair_out.index_copy_(0, order, back)
        y = (pair_out.view(T, self.topk, H) * wts.view(T, self.topk, 1)).sum(1)
        sh = self.shared(x) if self.shared is not None else None
        if sh is not None:
            y = y + sh
        self.last_stats = {'sent_pairs': int(sum(sc)) - int(sc[self.rank]) if self.world > 1 else 0,
                           'recv_rows': int(recv_rows.shape[0]),
                           'local_experts_touched': int(torch.unique(recv_eid).numel())}
        return y, sel, wts
