"""Sharding of the FP8 path across the GPUs of one box (one process per GPU, torch.distributed).

The reference has no multi-GPU form of this path (no NCCL, MPI or Gloo anywhere in its tree; its only transport
is a two-device layer pipeline, include/ida_native/arena.hpp:24-26), so single-GPU output is the parity target
and the partitioning below is new work:

  * dense GEMMs: weights sharded by output columns (gate/up, forward GEMMs) or by the contraction dimension
    (down projection, dgrad). A per-tensor weight scale needs the amax of the WHOLE tensor: one max-all-reduce of
    one float keeps the scale bit-identical to the single-GPU one. Row-parallel partial products are summed in
    fp32, either by an NCCL all-reduce (row_parallel_gemm_fp8) or inside the GEMM's epilogue, which adds every
    tile straight into the owning rank's slice over NVLink (RowParallelReduceScatterGemm).
  * MoE: experts are sharded (expert parallelism), tokens stay data-parallel; popular experts can be replicated so
    that a skewed load spreads evenly (ReplicaPlacement). Rows travel as E4M3 bytes (1 byte per element on the
    wire). EpMoeSwigluFp8 plans on the host and exchanges with NCCL all-to-all; EpMoeSwigluFp8Direct plans on the
    device and stores the rows straight into the serving ranks' buffers.

The planning code is pure host logic and runs on CPU tensors with the gloo backend too (tests use that).
"""
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist


def shard_range(n, world, rank, multiple=1):
    """Contiguous balanced shard [start, stop) of range(n) for `rank`; shard sizes are multiples of `multiple`
    except possibly the last one (cf_shard_range, the library's host-side sharding glue)."""
    import ctypes as C

    from . import _capi
    lo, hi = C.c_longlong(), C.c_longlong()
    _capi.check(_capi.lib().cf_shard_range(int(n), int(world), int(rank), int(multiple), C.byref(lo), C.byref(hi)))
    return int(lo.value), int(hi.value)


def allreduce_max_(t, group=None):
    """In-place max over ranks (weight amax of a sharded tensor, float32). max() is exact in any order, so every
    rank ends with the value a single GPU would have computed."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t


def allreduce_sum_(t, group=None):
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t


def all_to_all_rows(send, send_splits, recv_splits, group=None):
    """Variable-size all-to-all of the rows of a 2-D tensor. NCCL: one all_to_all_single; gloo (CPU tests) has no
    all-to-all, so the same exchange is issued as paired isend/irecv."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    recv = send.new_empty((int(sum(recv_splits)),) + tuple(send.shape[1:]))
    if dist.get_backend(group) == "nccl":
        dist.all_to_all_single(recv, send, output_split_sizes=list(recv_splits), input_split_sizes=list(send_splits),
                               group=group)
        return recv
    s_off = [0]
    for c in send_splits:
        s_off.append(s_off[-1] + int(c))
    r_off = [0]
    for c in recv_splits:
        r_off.append(r_off[-1] + int(c))
    recv[r_off[rank]:r_off[rank + 1]] = send[s_off[rank]:s_off[rank + 1]]
    reqs = []
    for peer in range(world):
        if peer == rank:
            continue
        if send_splits[peer]:
            reqs.append(dist.isend(send[s_off[peer]:s_off[peer + 1]].contiguous(), dst=peer, group=group))
        if recv_splits[peer]:
            reqs.append(dist.irecv(recv[r_off[peer]:r_off[peer + 1]], src=peer, group=group))
    for r in reqs:
        r.wait()
    return recv


@dataclass
class ReplicaPlacement:
    """Expert placement for a skewed load: the experts are laid end to end on a line, each as long as its expected share
    of the rows, and the line is cut into `world` equal pieces, one per rank. Every (expert, rank) overlap is a replica
    ("virtual expert") of that expert on that rank and receives the overlapping fraction of the expert's rows. Replica
    ids ascend along the line, so every rank owns a contiguous id range (the layout EpPlan needs), ids ascend with the
    expert id (the combine adds experts in the single-GPU order), and every rank expects the same number of rows.
    A uniform load with world | E degenerates to plain expert sharding (one replica per expert)."""
    world: int
    num_experts: int
    replica_expert: List[int]            # expert of each replica
    replica_rank: List[int]              # rank that holds it
    replica_share: List[float]           # fraction of its expert's rows it takes
    replica_start: List[int]             # [E + 1] first replica id of each expert
    replica_cum_share: List[float]       # cumulative share inside the expert (last replica of an expert: 1.0)
    rank_ranges: List[tuple]             # [world] (lo, hi) replica ids per rank

    @property
    def num_replicas(self):
        return len(self.replica_expert)

    @classmethod
    def build(cls, popularity, world, min_share=0.02, total_rows=None, tile_rows=256, rank_speed=None):
        """popularity: expected share of the rows per expert (any positive scale). Overlaps below `min_share` of a
        rank's piece are not worth a weight copy: they are merged into the expert's largest replica. The layout is
        computed by the library (cf_ep_placement_build), the same call a C++ trainer makes. With total_rows (selected
        rows of all ranks per layer) the pieces are sized for equal tile work instead of equal rows
        (cf_ep_placement_build_balanced): a rank with several small replicas pays about tile_rows / 2 padded rows each.
        rank_speed (needs total_rows): measured throughput of every rank on this work, any common unit; slower ranks
        get shorter pieces (cf_ep_placement_build_weighted)."""
        import ctypes as C

        from . import _capi
        E = len(popularity)
        pop = (C.c_double * E)(*[float(x) for x in popularity])
        pl = _capi.EpPlacementStruct()
        if total_rows and rank_speed is not None:
            assert len(rank_speed) == world
            spd = (C.c_double * world)(*[float(x) for x in rank_speed])
            _capi.check(_capi.lib().cf_ep_placement_build_weighted(pop, E, int(world), float(min_share), float(total_rows),
                                                                   int(tile_rows), spd, C.byref(pl)))
        elif total_rows:
            _capi.check(_capi.lib().cf_ep_placement_build_balanced(pop, E, int(world), float(min_share), float(total_rows),
                                                                   int(tile_rows), C.byref(pl)))
        else:
            _capi.check(_capi.lib().cf_ep_placement_build(pop, E, int(world), float(min_share), C.byref(pl)))
        V = pl.num_replicas
        return cls(world, E, list(pl.replica_expert[:V]), list(pl.replica_rank[:V]), list(pl.replica_share[:V]),
                   list(pl.replica_start[:E + 1]), list(pl.replica_cum_share[:V]),
                   [(pl.rank_lo[g], pl.rank_hi[g]) for g in range(world)])

    def local_experts(self, rank):
        lo, hi = self.rank_ranges[rank]
        return [self.replica_expert[v] for v in range(lo, hi)]


@dataclass
class EpPlan:
    """Who sends how many rows to whom for one expert-parallel MoE layer.

    Experts are sharded contiguously: rank r owns experts [e_lo(r), e_hi(r)). Every rank's compact send buffer is
    ordered by expert (so by destination rank). On the receiving side the rows arrive grouped by source rank and,
    inside each source, by local expert: each (source, local expert) run is one GEMM segment."""
    world: int
    rank: int
    num_experts: int
    counts_all: List[List[int]]          # [world][num_experts] rows each rank routes to each expert
    send_splits: List[int]               # rows this rank sends to each rank
    recv_splits: List[int]               # rows this rank receives from each rank
    seg_counts: List[int]                # per (source, local expert) segment, source-major
    seg_offsets: List[int]
    seg_weight: List[int]                # local expert index of each segment
    seg_source: List[int]                # source rank of each segment
    total_recv: int

    @staticmethod
    def expert_range(num_experts, world, rank):
        return shard_range(num_experts, world, rank)

    @classmethod
    def build(cls, counts_all, rank, ranges=None):
        """ranges: per rank the contiguous (lo, hi) expert ids it serves; default: balanced contiguous sharding."""
        world = len(counts_all)
        num_experts = len(counts_all[0])
        if ranges is None:
            ranges = [cls.expert_range(num_experts, world, r) for r in range(world)]
        send_splits = [int(sum(counts_all[rank][lo:hi])) for lo, hi in ranges]
        lo, hi = ranges[rank]
        recv_splits = [int(sum(counts_all[src][lo:hi])) for src in range(world)]
        seg_counts, seg_offsets, seg_weight, seg_source = [], [], [], []
        off = 0
        for src in range(world):
            for e in range(lo, hi):
                c = int(counts_all[src][e])
                seg_counts.append(c)
                seg_offsets.append(off)
                seg_weight.append(e - lo)
                seg_source.append(src)
                off += c
        return cls(world, rank, num_experts, [list(map(int, c)) for c in counts_all], send_splits, recv_splits,
                   seg_counts, seg_offsets, seg_weight, seg_source, off)


def gather_counts(local_counts, group=None):
    """All ranks' per-expert row counts as a host table [world][E] (one small all-gather and one device->host copy:
    the split sizes of an all-to-all have to be known on the host)."""
    world = dist.get_world_size(group)
    buf = [torch.empty_like(local_counts) for _ in range(world)]
    dist.all_gather(buf, local_counts, group=group)
    return [b.cpu().tolist() for b in buf]


class ShardedFp8Weight:
    """A logical [N_total, K] weight sharded by output columns: this rank holds rows [n_lo, n_hi). The per-tensor
    scale comes from the amax of the whole tensor (local amax, then max-all-reduce), so the E4M3 bytes of the shard
    equal the same rows of the single-GPU cache."""

    def __init__(self, cfb, w_shard, group=None):
        self.cfb = cfb
        self.w = w_shard
        self.group = group
        self.fw = cfb.Fp8Weight(w_shard, stored_out_major=True)

    def refresh(self):
        cfb = self.cfb
        cfb.fp8_amax_bf16(self.w, self.fw.amax)
        allreduce_max_(self.fw.amax, self.group)
        cfb.refresh_fp8_weight(self.fw, recompute_amax=False)
        return self.fw


def row_parallel_gemm_fp8(cfb, ctx, M, N, K_local, a8_local, a_descale, w8_local, w_descale, out_bf16, group=None,
                          a_row_descale=None, b_col_descale=None, partial=None):
    """K-sharded (row-parallel) NT GEMM: every rank multiplies its K slice — A8[:, k_lo:k_hi] against W8[:, k_lo:k_hi] —
    into an fp32 partial product, the partials are summed by an all-reduce and rounded to bf16 once. With per-tensor
    scales the result differs from the single-GPU GEMM only by the fp32 summation order."""
    if partial is None:
        partial = torch.empty((M, N), dtype=torch.float32, device=out_bf16.device)
    cfb.lt_gemm_fp8_nt(ctx, M, N, K_local, a8_local, a8_local.stride(0), False, a_descale, w8_local, w_descale, partial, N,
                       a_row_descale=a_row_descale, b_col_descale=b_col_descale)
    allreduce_sum_(partial, group)
    out_bf16.copy_(partial)
    return out_bf16


class PeerBarrier:
    """Orders the work every rank enqueues after wait() behind the work every rank enqueued before it, on the current
    stream and without a host round trip. kind "device": cf_peer_barrier (every rank stores an epoch into its word of
    every peer's flag array in symmetric memory and waits, bounded by limit_ms, for its own array to fill up: one tiny
    kernel); kind "nccl": a one-float all-reduce. Construction is collective over the group."""

    def __init__(self, cfb, ctx, group=None, device="cuda", kind="device", limit_ms=2000):
        assert kind in ("device", "nccl")
        self.cfb, self.ctx, self.group, self.limit_ms = cfb, ctx, group, int(limit_ms)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._fence = torch.zeros(1, dtype=torch.float32, device=device)
        self._flags, self._epoch, self._keep = None, 0, None
        if self.world > 1 and kind == "device":
            import torch.distributed._symmetric_memory as symm_mem
            flags = symm_mem.empty((64,), dtype=torch.int32, device=device)
            hdl = symm_mem.rendezvous(flags, group if group is not None else dist.group.WORLD)
            views = [hdl.get_buffer(r, (64,), torch.int32) for r in range(self.world)]
            flags.zero_()
            self._keep = (flags, hdl, views)
            self._flags = torch.tensor([v.data_ptr() for v in views], dtype=torch.int64, device=device)
        if self.world > 1:
            # every rank's flag words are zero before any rank may store into them
            dist.all_reduce(self._fence, group=self.group)
            torch.cuda.current_stream().synchronize()

    def wait(self):
        if self.world == 1:
            return
        if self._flags is not None:
            self._epoch += 1
            self.cfb.peer_barrier(self.ctx, self._flags, self.world, self.rank, self._epoch, self.limit_ms)
        else:
            dist.all_reduce(self._fence, group=self.group)

    @property
    def on_device(self):
        return self._flags is not None

    def share_i32(self, src, n, tables):
        """All-gather of n int32 words per rank into every rank's [world, n] table by peer stores, with the barrier in the
        same launch (device kind only). tables: int64 device tensor of the ranks' table addresses as mapped here."""
        assert self._flags is not None
        self._epoch += 1
        self.cfb.peer_share_i32(self.ctx, src, n, tables, self._flags, self.world, self.rank, self._epoch, self.limit_ms)


class RowParallelReduceScatterGemm:
    """K-sharded (row-parallel) NT GEMM whose epilogue IS the reduce-scatter: every rank adds the row slices of its fp32
    partial product straight into the owning rank's accumulation slice (bulk reduce-add copies into symmetric memory,
    over NVLink for the other ranks' slices), so the exchange overlaps the main loop tile by tile and no fp32 partial
    ever goes through a collective. Rank r ends up with rows [r * M/world, (r + 1) * M/world) of the product in bf16.
    Two accumulation slices alternate: the one used by call i is zeroed again while it is read out, and the barrier of
    call i + 1 orders that behind every rank's next use of it."""

    def __init__(self, cfb, ctx, M, N, group=None, device="cuda", barrier="device"):
        self.cfb, self.ctx, self.group, self.M, self.N = cfb, ctx, group, M, N
        self._pb = PeerBarrier(cfb, ctx, group, device, kind=barrier)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        assert M % self.world == 0 and (M // self.world) % 256 == 0, "row slices must be multiples of 256 rows"
        assert N % 32 == 0
        self.rows = M // self.world
        self._peers = []          # keeps the peer views alive
        self.acc, self.ptrs = [], []
        for _ in range(2):
            if self.world > 1:
                import torch.distributed._symmetric_memory as symm_mem
                a = symm_mem.empty((self.rows, N), dtype=torch.float32, device=device)
                hdl = symm_mem.rendezvous(a, group if group is not None else dist.group.WORLD)
                views = [hdl.get_buffer(r, (self.rows, N), torch.float32) for r in range(self.world)]
                self._peers.append((hdl, views))
                ptrs = [v.data_ptr() for v in views]
            else:
                a = torch.empty((self.rows, N), dtype=torch.float32, device=device)
                ptrs = [a.data_ptr()]
            a.zero_()
            self.acc.append(a)
            self.ptrs.append(ptrs)
        self._flip = 0
        self._barrier()           # every slice is zero before anyone adds to it

    def _barrier(self):
        self._pb.wait()

    def forward(self, a8_local, a_descale, w8_local, w_descale, out_slice_bf16, a_row_descale=None, b_col_descale=None):
        """a8_local [M, K_local] E4M3 (this rank's K slice of every row), w8_local [N, K_local]; out_slice_bf16
        [M/world, N] receives this rank's rows of the full product. a_row_descale float[M] / b_col_descale float[N]:
        per-token / per-output-channel scales shared by all ranks, applied before the partial products are summed."""
        b = self._flip
        self._flip ^= 1
        K_local = a8_local.shape[1]
        self.cfb.gemm_fp8_nt_reduce_scatter(self.ctx, self.M, self.N, K_local, a8_local, a8_local.stride(0), False, a_descale,
                                            w8_local, w_descale, self.ptrs[b], a_row_descale=a_row_descale,
                                            b_col_descale=b_col_descale)
        self._barrier()           # every rank's GEMM, and the adds it sent here, have completed
        self.cfb.f32_to_bf16_and_zero(self.acc[b], out_slice_bf16)
        return out_slice_bf16


class EpMoeSwigluFp8:
    """Expert-parallel form of ops.MoeSwigluFp8: tokens are data-parallel (this rank holds `rows` of them), experts
    are sharded over the ranks. Per layer: route locally -> counts all-gather -> E4M3 rows all-to-all -> ragged
    gate/up GEMM over (source, expert) segments with the source's activation scale -> SwiGLU + delayed-scale
    re-quantise -> ragged down GEMM -> bf16 all-to-all back -> local weighted combine."""

    def __init__(self, cfb, ctx, rows, H, F, num_experts, top_k, group=None, device="cuda", recv_capacity=None,
                 fused_return=False, fused_swiglu=False, placement=None):
        """fused_swiglu: the local gate/up weight is in the interleaved layout (fp8_interleave_gate_up) and the gate/up
        GEMM's epilogue does SwiGLU and the delayed-scale re-quantise, so the [rows, 2F] bf16 intermediate never
        exists. fused_return: the down-projection GEMM writes every segment's rows straight into the `back` buffer of the
        rank that owns the tokens (NVLink P2P stores from the GEMM epilogue into symmetric memory), which removes the
        bf16 all-to-all of the return leg; one tiny all-reduce orders the combine behind all ranks' GEMMs.
        placement: a ReplicaPlacement; the layer then dispatches over its replicas ("virtual experts") instead of the
        experts, and the local weight stacks passed to forward() hold placement.local_experts(rank) in that order."""
        self.cfb, self.ctx, self.group = cfb, ctx, group
        self.rows, self.H, self.F, self.E, self.k = rows, H, F, num_experts, top_k
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.placement = placement
        if placement is not None:
            assert placement.world == self.world and placement.num_experts == num_experts
            self.V = placement.num_replicas
            self.ranges = [tuple(r) for r in placement.rank_ranges]
            self.rep_start = torch.tensor(placement.replica_start, dtype=torch.int32, device=device)
            self.rep_cum = torch.tensor(placement.replica_cum_share, dtype=torch.float32, device=device)
            self.rwv = torch.zeros((rows, self.V), dtype=torch.float32, device=device)
        else:
            self.V = num_experts
            self.ranges = [EpPlan.expert_range(num_experts, self.world, r) for r in range(self.world)]
        self.e_lo, self.e_hi = self.ranges[self.rank]
        self.T = rows * top_k
        # worst case every token of every rank picks this rank's experts
        self.cap = recv_capacity or self.T * self.world
        dev = device
        self.counts = torch.zeros(self.V, dtype=torch.int32, device=dev)
        self.offsets = torch.zeros(self.V, dtype=torch.int32, device=dev)
        self.idx = torch.zeros((self.V, rows), dtype=torch.int32, device=dev)
        self.x8 = torch.empty((rows, H), dtype=torch.uint8, device=dev)
        self.xc = torch.empty((self.T, H), dtype=torch.uint8, device=dev)
        self.slot_x = cfb.ActSlot(ctx, cfb.E4M3_MAX)
        self.slot_h = cfb.ActSlot(ctx, cfb.E4M3_MAX)
        self.device = dev
        self.plan: Optional[EpPlan] = None
        self.fused_return = bool(fused_return) and self.world > 1
        self.fused_swiglu = bool(fused_swiglu)
        if self.fused_return:
            import torch.distributed._symmetric_memory as symm_mem
            self.back = symm_mem.empty((self.T, H), dtype=torch.bfloat16, device=dev)
            self._hdl = symm_mem.rendezvous(self.back, group if group is not None else dist.group.WORLD)
            self.peer_back = [self._hdl.get_buffer(r, (self.T, H), torch.bfloat16) for r in range(self.world)]
            for t in self.peer_back:
                assert t.data_ptr() % 16 == 0
            self._fence = torch.zeros(1, dtype=torch.float32, device=dev)

    def forward(self, x, route_weights, w_gateup8_local, w_gateup_descale, w_down8_local, w_down_descale, mixed,
                accumulate=True):
        cfb, ctx = self.cfb, self.ctx
        rows, H, F = self.rows, self.H, self.F
        cfb.moe_topk_route_f32(route_weights, rows, self.E, self.k)
        if self.placement is not None:
            # every selected (row, expert) moves to one replica of that expert; from here on "experts" are replicas
            cfb.moe_expand_route_replicas(route_weights, self.rwv, rows, self.E, self.V, self.rep_start, self.rep_cum,
                                          first_row=self.rank * rows)
            route_weights = self.rwv
        E = self.V
        cfb.moe_build_expert_row_lists(route_weights, self.counts, self.idx, rows, E)
        cfb.moe_expert_offsets_from_counts(self.counts, self.offsets, E)
        cfb.fp8_quant_act(ctx, self.slot_x, x, self.x8)
        cfb.moe_gather_all_u8(self.x8, self.xc, self.idx, self.counts, self.offsets, rows, E, H)
        # exchange: counts (host-visible), every rank's activation descale, then the rows
        plan = EpPlan.build(gather_counts(self.counts, self.group), self.rank, self.ranges)
        self.plan = plan
        dx_local = torch.empty(1, dtype=torch.float32, device=self.device)
        _copy_device_scalar(cfb, dx_local, self.slot_x.c.descale_snapshot)
        dx_all = [torch.empty(1, dtype=torch.float32, device=self.device) for _ in range(self.world)]
        dist.all_gather(dx_all, dx_local, group=self.group)
        recv8 = all_to_all_rows(self.xc, plan.send_splits, plan.recv_splits, self.group)
        R = plan.total_recv
        nseg = len(plan.seg_counts)
        dev = self.device
        seg_counts = torch.tensor(plan.seg_counts, dtype=torch.int32, device=dev)
        seg_offsets = torch.tensor(plan.seg_offsets, dtype=torch.int32, device=dev)
        seg_weight = torch.tensor(plan.seg_weight, dtype=torch.int32, device=dev)
        seg_dx = torch.cat(dx_all)[torch.tensor(plan.seg_source, device=dev)].contiguous()
        e_local = self.e_hi - self.e_lo
        yc = torch.empty((max(R, 1), H), dtype=torch.bfloat16, device=dev)
        if R > 0:
            h8 = torch.empty((R, F), dtype=torch.uint8, device=dev)
            if self.fused_swiglu:
                cfb.gemm_fp8_swiglu_quant_act(ctx, self.slot_h, nseg, e_local, seg_weight, R, F, H, seg_counts, seg_offsets,
                                              recv8, H, False, seg_dx, True, w_gateup8_local, w_gateup_descale, h8, F)
            else:
                gu = torch.empty((R, 2 * F), dtype=torch.bfloat16, device=dev)
                cfb.gemm_fp8_nt_segments(ctx, nseg, e_local, seg_weight, R, 2 * F, H, seg_counts, seg_offsets, recv8, H,
                                         False, seg_dx, True, w_gateup8_local, w_gateup_descale, gu, 2 * F)
                cfb.fp8_swiglu_quant_act(ctx, self.slot_h, gu, gu.view(-1)[F:], 2 * F, R, F, h8)
            if self.fused_return:
                # segment (src, e) returns to rank src at the row where expert e starts in src's compact order
                row0 = [int(sum(plan.counts_all[src][:self.e_lo + w])) for src, w in zip(plan.seg_source, plan.seg_weight)]
                for src, w, c, r0 in zip(plan.seg_source, plan.seg_weight, plan.seg_counts, row0):
                    assert 0 <= r0 and r0 + c <= self.T, "segment would leave the peer's buffer"
                seg_out = torch.tensor([self.peer_back[src].data_ptr() for src in plan.seg_source], dtype=torch.int64, device=dev)
                seg_row0 = torch.tensor(row0, dtype=torch.int64, device=dev)
                cfb.gemm_fp8_nt_segments_scatter(ctx, nseg, e_local, seg_weight, R, H, F, seg_counts, seg_offsets, h8, F,
                                                 False, cfb.ops._DevPtr(self.slot_h.c.descale_snapshot), False,
                                                 w_down8_local, w_down_descale, seg_out, seg_row0, H)
            else:
                cfb.gemm_fp8_nt_segments(ctx, nseg, e_local, seg_weight, R, H, F, seg_counts, seg_offsets, h8, F, False,
                                         cfb.ops._DevPtr(self.slot_h.c.descale_snapshot), False, w_down8_local,
                                         w_down_descale, yc, H)
        if self.fused_return:
            dist.all_reduce(self._fence, group=self.group)      # every rank's GEMM (and its peer stores) has completed
            back = self.back
        else:
            back = all_to_all_rows(yc[:R], plan.recv_splits, plan.send_splits, self.group)
        cfb.moe_combine_sorted_bf16(mixed, back, route_weights, self.idx, self.counts, self.offsets, rows, E, H, accumulate)


class EpMoeSwigluFp8Direct:
    """Expert-parallel SwiGLU MoE layer that never visits the host between its launches: the count table is gathered on
    the device, every rank derives the same plan from it with one small kernel (cf_moe_ep_plan), rows are permuted and
    sent in one pass straight into the serving ranks' buffers (plain stores over NVLink into symmetric memory, the
    sender's activation descale travelling with each row), each replica a rank serves is ONE ragged GEMM group whatever
    the number of sources (gate/up GEMM with the SwiGLU + re-quantise epilogue and a per-row descale, then the down
    GEMM), and the results are stored back into the owners' compact buffers the same way. Two one-float all-reduces
    order the readers behind the writers. Buffers are sized for the worst case (every token of every rank on one rank),
    so no count ever has to be known on the host.
    Weights: gate/up interleaved (fp8_interleave_gate_up), stacked in placement.local_experts(rank) order."""

    def __init__(self, cfb, ctx, rows, H, F, num_experts, top_k, placement=None, group=None, device="cuda",
                 fused_return=True, barrier="device", barrier_limit_ms=2000):
        """fused_return: the down GEMM's epilogue stores every run of result rows straight into the owner's buffer
        (cf_gemm_fp8_nt_grouped_return) instead of writing them locally and copying them out afterwards.
        barrier: "device" orders readers behind writers with cf_peer_barrier (flag words in the peers' memory, one tiny
        kernel, bounded wait of barrier_limit_ms); "nccl" uses a one-float all-reduce instead."""
        self.cfb, self.ctx, self.group = cfb, ctx, group
        self.fused_return = bool(fused_return) and H % 64 == 0
        self.rows, self.H, self.F, self.E, self.k = rows, H, F, num_experts, top_k
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if placement is None:
            placement = ReplicaPlacement.build([1.0] * num_experts, self.world)
        assert placement.world == self.world and placement.num_experts == num_experts
        assert H % 16 == 0 and F % 32 == 0
        self.placement = placement
        self.V = V = placement.num_replicas
        self.lo, self.hi = placement.rank_ranges[self.rank]
        self.n_local = self.hi - self.lo
        assert self.n_local >= 1, "a rank without replicas has nothing to serve"
        self.T = T = rows * top_k
        self.cap = cap = T * self.world
        dev = self.device = device
        i32, f32 = torch.int32, torch.float32
        self.rep_start = torch.tensor(placement.replica_start, dtype=i32, device=dev)
        self.rep_cum = torch.tensor(placement.replica_cum_share, dtype=f32, device=dev)
        self.range_lo = torch.tensor([r[0] for r in placement.rank_ranges], dtype=i32, device=dev)
        self.range_hi = torch.tensor([r[1] for r in placement.rank_ranges], dtype=i32, device=dev)
        self.rwv = torch.zeros((rows, V), dtype=f32, device=dev)
        self.front_scratch = torch.empty(max(1, cfb.moe_route_dispatch_scratch_ints(rows, V)), dtype=torch.int32, device=dev)
        self.counts = torch.zeros(V, dtype=i32, device=dev)
        self.offsets = torch.zeros(V, dtype=i32, device=dev)
        self.idx = torch.zeros((V, rows), dtype=i32, device=dev)
        self.x8 = torch.empty((rows, H), dtype=torch.uint8, device=dev)
        self.h8 = torch.empty((cap, F), dtype=torch.uint8, device=dev)
        # compact results of the down GEMM: only the copied-return form keeps them locally
        self.yc = None if self.fused_return else torch.empty((cap, H), dtype=torch.bfloat16, device=dev)
        self.send_runs = torch.zeros(V * cfb.ROW_RUN_BYTES, dtype=torch.uint8, device=dev)
        self.ret_runs = torch.zeros(self.n_local * self.world * cfb.ROW_RUN_BYTES, dtype=torch.uint8, device=dev)
        self.grp_counts = torch.zeros(self.n_local, dtype=i32, device=dev)
        self.grp_offsets = torch.zeros(self.n_local, dtype=i32, device=dev)
        self.slot_x = cfb.ActSlot(ctx, cfb.E4M3_MAX)
        self.slot_h = cfb.ActSlot(ctx, cfb.E4M3_MAX)
        self._keep = []
        self.counts_all, pcounts = self._shared((self.world, V), i32)
        self.counts_all.zero_()
        self.peer_counts_all = torch.tensor(pcounts, dtype=torch.int64, device=dev)
        self.recv8, p8 = self._shared((cap, H), torch.uint8)
        self.recv_dx, pdx = self._shared((cap,), f32)
        self.back, pback = self._shared((T, H), torch.bfloat16)
        self.recv_dx.fill_(1.0)
        self.peer_recv8 = torch.tensor(p8, dtype=torch.int64, device=dev)
        self.peer_recv_dx = torch.tensor(pdx, dtype=torch.int64, device=dev)
        self.peer_back = torch.tensor(pback, dtype=torch.int64, device=dev)
        self.back_ptrs = list(pback)
        self._pb = PeerBarrier(cfb, ctx, group, dev, kind=barrier, limit_ms=barrier_limit_ms)
        self.stage_marks = None   # set to a list to receive (stage name, CUDA event) pairs from the next forward()
        self._barrier()

    def _shared(self, shape, dtype):
        """A buffer every rank can store into: symmetric memory when there are peers, a plain tensor otherwise."""
        if self.world == 1:
            t = torch.zeros(shape, dtype=dtype, device=self.device)
            return t, [t.data_ptr()]
        import torch.distributed._symmetric_memory as symm_mem
        t = symm_mem.empty(shape, dtype=dtype, device=self.device)
        hdl = symm_mem.rendezvous(t, self.group if self.group is not None else dist.group.WORLD)
        views = [hdl.get_buffer(r, shape, dtype) for r in range(self.world)]
        self._keep.append((hdl, views))
        for v in views:
            assert v.data_ptr() % 16 == 0
        return t, [v.data_ptr() for v in views]

    def _barrier(self):
        self._pb.wait()

    def forward(self, x, route_weights, w_gateup8_local, w_gateup_descale, w_down8_local, w_down_descale, mixed,
                accumulate=True):
        cfb, ctx = self.cfb, self.ctx
        rows, H, F, V, W = self.rows, self.H, self.F, self.V, self.world
        marks = self.stage_marks          # None, or a list that receives (stage name, CUDA event) pairs of this call

        def mark(name):
            if marks is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        cfb.moe_route_dispatch_lists(route_weights, rows, self.E, self.k, self.counts, self.offsets, self.idx,
                                     self.front_scratch, replica_weights=self.rwv, num_replicas=V,
                                     replica_start=self.rep_start, replica_cum_share=self.rep_cum, first_row=self.rank * rows)
        mark("route + replica choice + dispatch lists")
        gathered = None
        if W > 1 and not self._pb.on_device:
            # the count table travels while the activation is being quantised
            gathered = dist.all_gather_into_tensor(self.counts_all, self.counts, group=self.group, async_op=True)
        elif W == 1:
            self.counts_all.copy_(self.counts.view(1, V))
        cfb.fp8_quant_act(ctx, self.slot_x, x, self.x8)
        if gathered is not None:
            gathered.wait()
        elif W > 1:
            # every rank stores its counts into every rank's table and waits for the others' (one launch)
            self._pb.share_i32(self.counts, V, self.peer_counts_all)
        mark("quantise x (count table gathered meanwhile)")
        cfb.moe_ep_plan(self.counts_all, W, self.rank, V, self.range_lo, self.range_hi, self.send_runs, self.grp_counts,
                        self.grp_offsets, self.ret_runs, recv_capacity_rows=self.cap, ctx=ctx)
        # permute + dispatch in one pass; every row carries the descale of the rank that quantised it
        cfb.moe_send_row_runs(self.x8, self.idx, rows, self.send_runs, V, rows, self.peer_recv8, H, W, self.cap,
                              tag_value=cfb.ops._DevPtr(self.slot_x.c.descale_snapshot), tag_bases=self.peer_recv_dx, ctx=ctx)
        mark("plan + permute and store rows into the serving ranks")
        self._barrier()          # every rank's rows have arrived
        mark("barrier: rows arrived")
        cfb.gemm_fp8_swiglu_quant_act(ctx, self.slot_h, self.n_local, self.n_local, None, self.cap, F, H, self.grp_counts,
                                      self.grp_offsets, self.recv8, H, False, self.recv_dx, 2, w_gateup8_local,
                                      w_gateup_descale, self.h8, F)
        mark("gate/up GEMM + SwiGLU + re-quantise")
        if self.fused_return:
            cfb.gemm_fp8_nt_grouped_return(ctx, self.n_local, self.cap, H, F, self.grp_counts, self.grp_offsets, self.h8, F,
                                           False, cfb.ops._DevPtr(self.slot_h.c.descale_snapshot), w_down8_local,
                                           w_down_descale, self.ret_runs, W, self.back_ptrs, self.T, H)
        else:
            cfb.gemm_fp8_nt_grouped(ctx, self.n_local, self.cap, H, F, self.grp_counts, self.grp_offsets, self.h8, F, False,
                                    cfb.ops._DevPtr(self.slot_h.c.descale_snapshot), False, w_down8_local, w_down_descale,
                                    self.yc, H)
            cfb.moe_send_row_runs(self.yc, None, 0, self.ret_runs, self.n_local * W, rows, self.peer_back, 2 * H, W, self.T,
                                  ctx=ctx)
        mark("down GEMM with the return leg")
        self._barrier()          # every rank's results are back
        mark("barrier: results back")
        cfb.moe_combine_sorted_bf16(mixed, self.back, self.rwv, self.idx, self.counts, self.offsets, rows, V, H, accumulate)
        mark("combine")


def _copy_device_scalar(cfb, dst_tensor, src_addr):
    """dst_tensor[0] = *(float*)src_addr, stream-ordered on the current stream (device-to-device)."""
    import ctypes as C
    rt = cfb.ops._cudart()
    rt.cudaMemcpyAsync.restype = C.c_int
    rc = rt.cudaMemcpyAsync(C.c_void_p(dst_tensor.data_ptr()), C.c_void_p(src_addr), C.c_size_t(4), C.c_int(3),
                            C.c_void_p(torch.cuda.current_stream().cuda_stream))
    if rc != 0:
        raise RuntimeError(f"cudaMemcpyAsync failed with {rc}")
