"""Multi-GPU partitioning of the quantized-linear path: one process per GPU, torch.distributed for the plumbing.

The reference is single-GPU (no collective anywhere in it); the two partitionings here are the ones the
benchmark configs prescribe:

  * dense layers: the weight is split over N (output features) in multiples of 128 rows, activations are
    replicated, every rank computes its [M, N/g] slab and the bf16 slabs are all-gathered;
  * routed MoE: experts are split evenly, tokens start sharded by rows, routes are dispatched to the rank that
    owns their expert with an all-to-all, the expert rank runs the grouped pipeline on what it received and a
    second all-to-all returns the rows, which the source rank combines with its route weights.

Everything that decides who sends what to whom is plain torch on whatever device the tensors live on, so the
exchange logic runs unchanged over gloo on CPU (tests) and NCCL on GPUs.  Split sizes of the all-to-all are read
back to the host once per step (torch's all_to_all_single needs them there).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch
import torch.distributed as dist


# ---- dense: N column sharding -----------------------------------------------------------------------------
def shard_range(n: int, world: int, rank: int, multiple: int = 128) -> tuple[int, int]:
    """Rows [begin, end) of the weight owned by `rank`: contiguous, sizes multiples of `multiple` (scale tiles are
    128 rows), the remainder spread over the first ranks."""
    if n % multiple != 0:
        raise ValueError(f"out_features {n} must be a multiple of {multiple} to shard scale tiles")
    units = n // multiple
    base, extra = divmod(units, world)
    begin = (rank * base + min(rank, extra)) * multiple
    size = (base + (1 if rank < extra else 0)) * multiple
    return begin, begin + size


def gathered_to_row_major(gathered: torch.Tensor) -> torch.Tensor:
    """[world, M, N/g] (what all_gather_into_tensor produces from equal [M, N/g] slabs) -> [M, N]."""
    world, m, n_local = gathered.shape
    return gathered.permute(1, 0, 2).reshape(m, world * n_local)


class ColumnShardedLinear:
    """y = x . W^T with W split over output features; `local_linear(x) -> [M, N/g]` is this rank's slab.

    Two ways to assemble [M, N] on every rank:
      * NCCL: `all_gather_into_tensor` of the slabs and a re-assembly copy (the default);
      * fused (`fuse_into(plan, tokens)`): every rank's full output lives in symmetric memory, the GEMM plan gets the
        address of this rank's column block inside every rank's output and its epilogue writes each tile to all of them
        while the GEMM is still running; the ranks meet at a device-side barrier before the result is used and before
        it is overwritten again.  No collective library call and no re-assembly pass are left on the data path."""

    def __init__(self, out_features: int, local_linear: Callable[[torch.Tensor], torch.Tensor], group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.out_features = out_features
        self.begin, self.end = shard_range(out_features, self.world, self.rank)
        if out_features % (self.world * 128) != 0:
            raise ValueError("equal shards are required for all_gather_into_tensor")
        self.local_linear = local_linear
        self._gathered = None
        self._fused = None
        self.active_plan = None

    def fuse_into(self, plans, tokens: int, dtype=torch.bfloat16) -> None:
        """Switches to the fused all-gather.  `plans` is one plan or a list of plans over the same weights, each offering
        set_output_peers(pointers, ld_out); every plan gets its own symmetric output buffer and forward() rotates through
        them (`active_plan` is the one the local linear has to run).  With two or more buffers a rank is never written
        while it may still read the same buffer, and one barrier per step is enough."""
        if self.world == 1:
            return
        import torch.distributed._symmetric_memory as symm_mem
        plans = list(plans) if isinstance(plans, (list, tuple)) else [plans]
        group = self.group if self.group is not None else dist.group.WORLD
        slots = []
        for plan in plans:
            full = symm_mem.empty(tokens, self.out_features, dtype=dtype, device="cuda")
            handle = symm_mem.rendezvous(full, group)
            offset_bytes = self.begin * full.element_size()
            plan.set_output_peers([int(ptr) + offset_bytes for ptr in handle.buffer_ptrs], self.out_features)
            slots.append((plan, full, handle))
        self._fused = slots
        self._step = 0
        self.active_plan = slots[0][0]

    def forward(self, x: torch.Tensor, assemble: bool = True) -> torch.Tensor:
        if self._fused is not None:
            plan, full, handle = self._fused[self._step % len(self._fused)]
            self._step += 1
            self.active_plan = plan
            if len(self._fused) == 1:
                handle.barrier(channel=0)  # nobody still reads the previous result out of this rank's only buffer
            self.local_linear(x)           # the epilogue writes this rank's columns into every rank's buffer
            handle.barrier(channel=1)      # every rank's columns have arrived
            return full
        y_local = self.local_linear(x)
        if self.world == 1:
            return y_local
        m, n_local = y_local.shape
        if self._gathered is None or self._gathered.shape != (self.world, m, n_local) or self._gathered.dtype != y_local.dtype:
            self._gathered = torch.empty(self.world, m, n_local, dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(self._gathered.view(self.world * m, n_local), y_local.contiguous(), group=self.group)
        return gathered_to_row_major(self._gathered) if assemble else self._gathered


# ---- MoE: expert parallelism ----------------------------------------------------------------------------
@dataclass
class RoutePlan:
    """Who gets which route.  Routes are numbered token * top_k + slot on the source rank."""
    order: torch.Tensor          # [R] local route ids sorted by destination rank (stable)
    send_counts: list            # routes sent to each rank
    recv_counts: list            # routes received from each rank
    local_expert: torch.Tensor   # [R] expert id relative to the destination rank, in send order


def expert_owner(expert: torch.Tensor, experts: int, world: int) -> torch.Tensor:
    per = experts // world
    return torch.div(expert, per, rounding_mode="floor")


def plan_routes(indices: torch.Tensor, experts: int, world: int, group=None) -> RoutePlan:
    """indices: [T_local, k] expert ids (any integer dtype)."""
    if experts % world != 0:
        raise ValueError("experts must divide evenly over the ranks")
    flat = indices.reshape(-1).to(torch.int64)
    dest = expert_owner(flat, experts, world)
    order = torch.sort(dest, stable=True).indices
    send = torch.bincount(dest, minlength=world)
    recv = torch.empty_like(send)
    if world > 1:
        dist.all_to_all_single(recv, send, group=group)
    else:
        recv.copy_(send)
    local_expert = (flat - dest * (experts // world))[order]
    return RoutePlan(order, send.cpu().tolist(), recv.cpu().tolist(), local_expert)


def exchange(rows: torch.Tensor, send_counts: list, recv_counts: list, world: int, group=None) -> torch.Tensor:
    """all-to-all of row blocks: rows [sum(send), ...] ordered by destination -> [sum(recv), ...] ordered by source."""
    out = torch.empty((sum(recv_counts),) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    if world > 1:
        dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
    else:
        out.copy_(rows)
    return out


def expert_parallel_moe(x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor, experts: int,
                        expert_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
                        combine_fn: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor] | None = None,
                        group=None) -> torch.Tensor:
    """One expert-parallel MoE step.

    x [T_local, H]; indices / weights [T_local, k]; expert_fn(rows [R, H], local_expert [R]) -> [R, H_out] runs the
    experts this rank owns on the routes it received (in arrival order); the result rows travel back and
    out[t] = sum_slot w[t, slot] * y[route(t, slot)] in slot order.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    t_local, k = indices.shape
    plan = plan_routes(indices, experts, world, group)
    token_of_route = torch.div(plan.order, k, rounding_mode="floor")
    sent_rows = x.index_select(0, token_of_route)
    recv_rows = exchange(sent_rows, plan.send_counts, plan.recv_counts, world, group)
    recv_expert = exchange(plan.local_expert.to(torch.int32), plan.send_counts, plan.recv_counts, world, group)
    y_recv = expert_fn(recv_rows, recv_expert)
    y_back = exchange(y_recv, plan.recv_counts, plan.send_counts, world, group)  # rows come back in send order
    # position of route r in the returned block
    position = torch.empty_like(plan.order)
    position[plan.order] = torch.arange(plan.order.numel(), device=plan.order.device)
    if combine_fn is not None:
        return combine_fn(position, weights, y_back)
    gathered = y_back.index_select(0, position).reshape(t_local, k, -1).to(torch.float32)
    out = torch.zeros(t_local, gathered.shape[-1], dtype=torch.float32, device=x.device)
    for slot in range(k):  # slot order, like the reference's combine
        out += gathered[:, slot] * weights[:, slot:slot + 1].to(torch.float32)
    return out


class LocalExperts:
    """The experts one rank owns, run with the grouped tcgen05 pipeline on whatever routes arrive."""

    def __init__(self, w_gate_up, w_down, hidden: int, intermediate: int):
        self.w_gate_up, self.w_down = w_gate_up, w_down
        self.hidden, self.inter = hidden, intermediate
        self.experts = w_gate_up.experts
        self._cache = {}

    def __call__(self, rows: torch.Tensor, local_expert: torch.Tensor) -> torch.Tensor:
        from . import ops
        r = rows.shape[0]
        if r == 0:
            return torch.empty(0, self.hidden, dtype=torch.bfloat16, device=rows.device)
        if r not in self._cache:
            self._cache = {r: (ops.MoeSortedRoutes(r, self.experts, rows.device),
                               ops.MoeSortedNvfp4Rows(r, self.experts, self.hidden, r, rows.device),
                               ops.MoeSortedNvfp4Rows(r, self.experts, self.inter, r, rows.device),
                               ops.Fp4GroupedGemmPlan(2 * self.inter, r, self.hidden, self.experts),
                               ops.Fp4GroupedGemmPlan(self.hidden, r, self.inter, self.experts))}
        routes, gu_in, dn_in, gu_plan, dn_plan = self._cache[r]
        gu_in.scales.zero_()
        dn_in.scales.zero_()
        routes.sort(local_expert.contiguous())
        gu_in.gather_quantize(rows.contiguous(), routes, 1)   # one route per received row
        gate_up = gu_plan.run(gu_in, self.w_gate_up, routes)
        dn_in.silu_mul_halves_quantize(gate_up, routes)
        down = dn_plan.run(dn_in, self.w_down, routes)
        return down.index_select(0, routes.route_to_sorted.to(torch.int64))  # back to arrival order


def device_combine(tokens: int, top_k: int):
    """combine_fn for expert_parallel_moe that uses the library's un-permute kernel."""
    def fn(position: torch.Tensor, weights: torch.Tensor, y_back: torch.Tensor) -> torch.Tensor:
        from . import ops
        holder = ops.MoeSortedRoutes(tokens * top_k, 1, y_back.device)
        holder.route_to_sorted.copy_(position.to(torch.int32))
        return ops.moe_weighted_accumulate(holder, weights.reshape(-1).to(torch.float32).contiguous(), y_back.contiguous(),
                                           tokens, top_k)
    return fn
