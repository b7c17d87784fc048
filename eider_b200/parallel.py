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

    def fuse_into(self, plans, tokens: int, dtype=torch.bfloat16, multicast: bool = True) -> None:
        """Switches to the fused all-gather.  `plans` is one plan or a list of plans over the same weights, each offering
        set_output_peers(pointers, ld_out) (and set_output_multicast); every plan gets its own symmetric output buffer and
        forward() rotates through them (`active_plan` is the one the local linear has to run).  With two or more buffers a
        rank is never written while it may still read the same buffer, and one barrier per step is enough.  With
        `multicast` and an NVLink multicast mapping behind the buffer, the epilogue writes each tile once and the switch
        copies it to every rank; otherwise it stores to each peer in turn."""
        if self.world == 1:
            return
        import torch.distributed._symmetric_memory as symm_mem
        plans = list(plans) if isinstance(plans, (list, tuple)) else [plans]
        group = self.group if self.group is not None else dist.group.WORLD
        slots = []
        self.multicast = False
        for plan in plans:
            full = symm_mem.empty(tokens, self.out_features, dtype=dtype, device="cuda")
            handle = symm_mem.rendezvous(full, group)
            offset_bytes = self.begin * full.element_size()
            plan.set_output_peers([int(ptr) + offset_bytes for ptr in handle.buffer_ptrs], self.out_features)
            mc = int(getattr(handle, "multicast_ptr", 0) or 0)
            if multicast and mc and hasattr(plan, "set_output_multicast"):
                plan.set_output_multicast(mc + offset_bytes)
                self.multicast = True
            slots.append((plan, full, handle))
        self._fused = slots
        self._step = 0
        self.active_plan = slots[0][0]
        self._barrier = PeerBarrier(group)

    def forward(self, x: torch.Tensor, assemble: bool = True) -> torch.Tensor:
        if self._fused is not None:
            plan, full, handle = self._fused[self._step % len(self._fused)]
            self._step += 1
            self.active_plan = plan
            if len(self._fused) == 1:
                self._barrier.arrive_and_wait(0)  # nobody still reads the previous result out of this rank's only buffer
            self.local_linear(x)                  # the epilogue writes this rank's columns into every rank's buffer
            self._barrier.arrive_and_wait(1)      # every rank's columns have arrived
            return full
        y_local = self.local_linear(x)
        if self.world == 1:
            return y_local
        m, n_local = y_local.shape
        if self._gathered is None or self._gathered.shape != (self.world, m, n_local) or self._gathered.dtype != y_local.dtype:
            self._gathered = torch.empty(self.world, m, n_local, dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(self._gathered.view(self.world * m, n_local), y_local.contiguous(), group=self.group)
        return gathered_to_row_major(self._gathered) if assemble else self._gathered

    def check(self) -> None:
        """Raises if a device-side meeting of the fused path gave up waiting (a peer never arrived)."""
        if self._fused is not None:
            self._barrier.check()


class PeerBarrier:
    """Device-side barrier of the ranks of one node on a signal pad in symmetric memory, through the library's bounded
    barrier kernel: a rank whose peer never arrives gets a status word after about a second instead of a spinning kernel.
    The epochs live on the device, so a CUDA graph that contains the barrier can be replayed.  If a rank fails on the host
    before its barrier (an exception in its local linear), it simply never launches it: its peers time out, `check()`
    raises on them, and no kernel is left spinning on the shared GPU."""

    def __init__(self, group=None, timeout_cycles: int = 0):
        import ctypes as C

        import torch.distributed._symmetric_memory as symm_mem

        from . import _lib
        self._lib = _lib.load()
        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        words = self._lib.eider_b200_peer_barrier_pad_bytes() // 4
        self.pad = symm_mem.empty(words, dtype=torch.int32, device="cuda")
        self.pad.zero_()
        self.handle = symm_mem.rendezvous(self.pad, group)
        self.state = torch.zeros(self._lib.eider_b200_peer_barrier_state_bytes() // 4, dtype=torch.int32, device="cuda")
        self._pads = (C.c_void_p * self.world)(*[C.c_void_p(int(p)) for p in self.handle.buffer_ptrs])
        self.timeout_cycles = timeout_cycles
        torch.cuda.synchronize()
        dist.barrier(group)  # every pad is zero before anybody signals

    def arrive_and_wait(self, channel: int) -> None:
        from ._lib import check
        check("eider_b200_peer_barrier_on_stream",
              self._lib.eider_b200_peer_barrier_on_stream(self._pads, self.world, self.rank, channel, self.state.data_ptr(),
                                                          self.timeout_cycles, torch.cuda.current_stream().cuda_stream))

    def status(self) -> int:
        return int(self.state[-1].item()) & 0xFFFFFFFF

    def check(self) -> None:
        st = self.status()
        if st:
            raise RuntimeError(f"peer barrier gave up: channel {(st >> 8) & 0xff}, rank {st & 0xff} never arrived (status {st:#x})")


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


# ---- MoE: expert parallelism over peer memory, counts resident on the device -------------------------------------
class PeerExpertParallelMoe:
    """One rank of the expert-parallel routed-MoE layer with all routing state on the device.

    Routes are sorted by global expert on the source rank, the per-expert counts of every rank are published to every
    rank, and each source stores the NVFP4 row, its scale bytes and a return address of every route straight into the
    owner's receive buffers (expert-major order, per-expert scale tiles), so the owner can run the grouped tcgen05
    pipeline without a local permutation.  Results travel back the same way and the source combines them with its route
    weights.  Nothing is read back to the host, there is no allocation in a step, and the three meetings of the ranks are
    the library's bounded barrier, so a step can be captured in a CUDA graph.

    Construction is split in two so that tests can emulate several ranks on one GPU: `buffers` holds what peers write
    into (allocated by the caller: symmetric memory on real ranks, plain tensors when emulated) and `connect()` takes the
    pointers of every rank's buffers."""

    PEER_BUFFERS = ("counts_all", "recv_packed", "recv_scales", "recv_origin", "return_rows")

    def __init__(self, rank: int, world: int, tokens_local: int, experts: int, top_k: int, hidden: int, intermediate: int,
                 w_gate_up, w_down, capacity: int | None = None, alloc=None, device="cuda"):
        from . import _lib, ops
        if experts % world != 0:
            raise ValueError("experts must divide evenly over the ranks")
        self._lib, self._ops = _lib.load(), ops
        self.rank, self.world, self.tokens, self.experts, self.top_k = rank, world, tokens_local, experts, top_k
        self.hidden, self.inter, self.per = hidden, intermediate, experts // world
        self.routes_local = tokens_local * top_k
        self.capacity = capacity if capacity is not None else self.routes_local * world  # all routes of all ranks always fit
        self.w_gate_up, self.w_down = w_gate_up, w_down
        self.w_gate_up_interleaved = w_gate_up.interleave_gate_up()  # SiLU * up quantizer in the gate/up GEMM's epilogue
        alloc = alloc or (lambda shape, dtype: torch.zeros(shape, dtype=dtype, device=device))
        tile_h, tile_i = ops.moe_scale_tile_bytes(hidden), ops.moe_scale_tile_bytes(intermediate)
        self.tile_h, self.tile_i = tile_h, tile_i
        cap = self.capacity
        self.buffers = {
            "counts_all": alloc((world * experts,), torch.int32),
            "recv_packed": alloc((cap * (hidden // 2),), torch.uint8),
            "recv_scales": alloc((((cap + 127) // 128 + self.per) * tile_h,), torch.uint8),
            "recv_origin": alloc((cap,), torch.int32),
            "return_rows": alloc((self.routes_local * hidden,), torch.bfloat16),
        }
        z = lambda n, dt=torch.int32: torch.zeros(n, dtype=dt, device=device)
        self.routes = ops.MoeSortedRoutes(self.routes_local, experts, device)        # local sort by global expert
        self.source_packed = z(tokens_local * (hidden // 2), torch.uint8).view(tokens_local, hidden // 2)
        self.source_scales = z(ops.scale_layout_len(tokens_local, hidden), torch.uint8)
        self.expert_base, self.before_me = z(experts), z(experts)
        self.recv_offsets, self.recv_total = z(self.per + 1), z(1)
        self.recv_experts = z(cap)
        self.gate_up_out = torch.empty(cap, 2 * intermediate, dtype=torch.bfloat16, device=device)
        self.down_in_packed = z(cap * (intermediate // 2), torch.uint8).view(cap, intermediate // 2)
        self.down_in_scales = z(((cap + 127) // 128 + self.per) * tile_i, torch.uint8)
        self.down_out = torch.empty(cap, hidden, dtype=torch.bfloat16, device=device)
        self.gate_up_plan = ops.Fp4GroupedGemmPlan(2 * intermediate, cap, hidden, self.per)
        self.down_plan = ops.Fp4GroupedGemmPlan(hidden, cap, intermediate, self.per)
        self.identity = torch.arange(self.routes_local, dtype=torch.int32, device=device)
        self.indices = z(tokens_local * top_k).view(tokens_local, top_k)
        self.weights = torch.zeros(tokens_local, top_k, dtype=torch.float32, device=device)
        self.out = torch.empty(tokens_local, hidden, dtype=torch.float32, device=device)
        self._tables = None
        self.fuse_silu = True

    def connect(self, peer_pointers: dict) -> None:
        """peer_pointers[name] = list of `world` device addresses, entry q = rank q's buffer `name` as this process sees it."""
        import ctypes as C
        self._tables = {name: (C.c_void_p * self.world)(*[C.c_void_p(int(p)) for p in peer_pointers[name]])
                        for name in self.PEER_BUFFERS}

    def _call(self, name, *args):
        from ._lib import check
        check(name, getattr(self._lib, name)(*args, torch.cuda.current_stream().cuda_stream))

    # -- phase 1: route locally, publish the counts --------------------------------------------------------------
    def route_and_publish(self, x: torch.Tensor, router_logits: torch.Tensor, norm_topk_prob: bool = True) -> None:
        if router_logits.shape != (self.tokens, self.experts) or router_logits.dtype != torch.float32 or not router_logits.is_contiguous():
            raise ValueError("router_logits must be contiguous f32 [tokens_local, experts]")
        self._call("infer_moe_topk_f32_batch_on_stream", router_logits.data_ptr(), self.indices.data_ptr(), self.weights.data_ptr(),
                   self.tokens, self.experts, self.top_k, int(bool(norm_topk_prob)))
        self.routes.sort(self.indices.reshape(-1))
        self._x = x
        self._call("eider_b200_ep_publish_counts_on_stream", self.routes.expert_counts.data_ptr(), self._tables["counts_all"],
                   self.world, self.rank, self.experts)

    # -- phase 2: offsets from everybody's counts, quantize once, dispatch ---------------------------------------
    def dispatch(self) -> None:
        ops = self._ops
        self._call("eider_b200_ep_offsets_on_stream", self.buffers["counts_all"].data_ptr(), self.world, self.rank, self.experts,
                   self.expert_base.data_ptr(), self.before_me.data_ptr(), self.recv_offsets.data_ptr(), self.recv_total.data_ptr())
        q = ops.Nvfp4Matrix(self.source_packed, self.source_scales, self.tokens, self.hidden)
        ops.quantize_nvfp4(self._x, 1.0, out=q)
        r = self.routes
        self._call("eider_b200_ep_dispatch_rows_on_stream", self.source_packed.data_ptr(), self.source_scales.data_ptr(),
                   r.sorted_routes.data_ptr(), r.sorted_experts.data_ptr(), r.expert_offsets.data_ptr(), self.expert_base.data_ptr(),
                   self.before_me.data_ptr(), self._tables["recv_packed"], self._tables["recv_scales"], self._tables["recv_origin"],
                   self.routes_local, self.top_k, self.hidden, self.tile_h, self.experts, self.world, self.rank)

    # -- phase 3: the experts this rank owns, on what arrived; results go home --------------------------------------
    def run_experts_and_return(self) -> None:
        lib = self._lib
        cap = self.capacity
        self._call("eider_b200_ep_expand_experts_on_stream", self.recv_offsets.data_ptr(), self.per, self.recv_experts.data_ptr(), cap)
        if self.fuse_silu:
            wi = self.w_gate_up_interleaved
            self._call("eider_b200_nvfp4_grouped_gemm_silu_quantize_on_stream", self.gate_up_plan._plan,
                       self.buffers["recv_packed"].data_ptr(), self.buffers["recv_scales"].data_ptr(), wi.packed.data_ptr(),
                       wi.scales_tiled.data_ptr(), wi.alpha.data_ptr(), self.recv_offsets.data_ptr(), cap,
                       self.down_in_packed.data_ptr(), self.down_in_scales.data_ptr(), self.tile_i)
        else:
            self._call("eider_b200_nvfp4_grouped_gemm_on_stream", self.gate_up_plan._plan, self.buffers["recv_packed"].data_ptr(),
                       self.buffers["recv_scales"].data_ptr(), self.w_gate_up.packed.data_ptr(), self.w_gate_up.scales_tiled.data_ptr(),
                       self.gate_up_out.data_ptr(), self.w_gate_up.alpha.data_ptr(), self.recv_offsets.data_ptr(), cap)
            self._call("eider_b200_moe_silu_mul_halves_quantize_sorted_routes_nvfp4_limited_on_stream", self.gate_up_out.data_ptr(),
                       self.recv_experts.data_ptr(), self.recv_offsets.data_ptr(), self.down_in_packed.data_ptr(),
                       self.down_in_scales.data_ptr(), cap, self.inter, self.tile_i, self.recv_total.data_ptr())
        self._call("eider_b200_nvfp4_grouped_gemm_on_stream", self.down_plan._plan, self.down_in_packed.data_ptr(),
                   self.down_in_scales.data_ptr(), self.w_down.packed.data_ptr(), self.w_down.scales_tiled.data_ptr(),
                   self.down_out.data_ptr(), self.w_down.alpha.data_ptr(), self.recv_offsets.data_ptr(), cap)
        self._call("eider_b200_ep_return_rows_on_stream", self.down_out.data_ptr(), self.buffers["recv_origin"].data_ptr(),
                   self.recv_total.data_ptr(), self._tables["return_rows"], cap, self.hidden, self.world)

    # -- phase 4: weighted sum of the returned routes, slot order ----------------------------------------------------
    def combine(self) -> torch.Tensor:
        self._call("infer_moe_weighted_accumulate_sorted_bf16_batch_on_stream", self.identity.data_ptr(),
                   self.weights.reshape(-1).data_ptr(), self.buffers["return_rows"].data_ptr(), self.out.data_ptr(), self.tokens,
                   self.hidden, self.top_k)
        return self.out

    def status(self) -> int:
        st = 0
        for one in getattr(self, "twins", [self]):
            st |= one.gate_up_plan.status() | one.down_plan.status()
        return st


def peer_expert_parallel_moe(group, tokens_local, experts, top_k, hidden, intermediate, w_gate_up, w_down, capacity=None,
                             double_buffer=True):
    """The layer on real ranks: buffers in symmetric memory, the library's bounded barrier between the phases.
    Returns (layer, step) where step(x, router_logits) -> [tokens_local, hidden] f32.

    With `double_buffer` consecutive steps alternate between two sets of buffers, which makes the meeting after the combine
    unnecessary: a rank reuses a set only after it has passed the third barrier of the step in between, and every rank
    reaches that barrier only after it has finished the step before (its combine included)."""
    import torch.distributed._symmetric_memory as symm_mem
    group = group if group is not None else dist.group.WORLD
    world, rank = dist.get_world_size(group), dist.get_rank(group)

    def alloc(shape, dtype):
        t = symm_mem.empty(*shape, dtype=dtype, device="cuda")
        t.zero_()
        return t

    layers = []
    for _ in range(2 if double_buffer else 1):
        one = PeerExpertParallelMoe(rank, world, tokens_local, experts, top_k, hidden, intermediate, w_gate_up, w_down, capacity, alloc)
        handles = {name: symm_mem.rendezvous(one.buffers[name], group) for name in PeerExpertParallelMoe.PEER_BUFFERS}
        one.connect({name: list(h.buffer_ptrs) for name, h in handles.items()})
        one._handles = handles
        layers.append(one)
    layer = layers[0]
    barrier = PeerBarrier(group)
    for one in layers:
        one.barrier = barrier
    layer.twins = layers
    calls = [0]

    def step(x, router_logits, norm_topk_prob=True):
        cur = layers[calls[0] % len(layers)]
        calls[0] += 1
        cur.route_and_publish(x, router_logits, norm_topk_prob)
        barrier.arrive_and_wait(4)
        cur.dispatch()
        barrier.arrive_and_wait(5)
        cur.run_experts_and_return()
        barrier.arrive_and_wait(6)
        out = cur.combine()
        if len(layers) == 1:
            # (the next step's counts and rows land in the same buffers: a rank may start it only when every rank has combined)
            barrier.arrive_and_wait(7)
        return out

    return layer, step
