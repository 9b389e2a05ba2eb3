"""Multi-GPU parity on one box (NCCL, one process per GPU; skipped with fewer than 2 GPUs): a column-sharded weight
quantises to the same bytes as the unsharded one, and the expert-parallel MoE layer agrees with the single-GPU layer
on the concatenated tokens within the path's tolerance."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

from gpu_util import package, randn_bf16, rel_fro  # noqa: E402


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _zipf_logits(rows, E, seed, device):
    g = torch.Generator(device=device).manual_seed(seed)
    p = torch.arange(1, E + 1, device=device, dtype=torch.float32) ** -1.1
    return (torch.randn((rows, E), generator=g, device=device) + torch.log(p / p.sum())).contiguous()


def _tensorquant(cfb, x):
    am = torch.zeros(4, dtype=torch.float32, device=x.device)
    sc, de = torch.zeros_like(am), torch.zeros_like(am)
    cfb.fp8_amax_bf16(x, am)
    cfb.fp8_scale_from_amax(am, cfb.E4M3_MAX, sc, de)
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    cfb.fp8_quantize_e4m3(x, q, sc)
    return q, de


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        cfb = package()
        par = cfb.parallel
        dev = torch.device("cuda", rank)
        ctx = cfb.Fp8Ctx(act8_bytes=0)
        # ---- column-sharded weight: same E4M3 bytes and scale as the unsharded cache
        N, K = 1024, 512
        g = torch.Generator(device=dev).manual_seed(7)
        w = (torch.randn((N, K), generator=g, device=dev) * 0.02).to(torch.bfloat16)      # same on all ranks
        lo, hi = par.shard_range(N, world, rank, 128)
        sh = par.ShardedFp8Weight(cfb, w[lo:hi].contiguous())
        fw = sh.refresh()
        full = cfb.Fp8Weight(w, stored_out_major=True)
        cfb.refresh_fp8_weight(full)
        assert torch.equal(fw.fwd8, full.fwd8[lo:hi]) and fw.scale.item() == full.scale.item()
        # ---- row-parallel (K-sharded) GEMM with the fp32 all-reduce vs the unsharded GEMM
        Mr, Nr, Kr = 256, 384, 1024
        a_full = randn_bf16((Mr, Kr), seed=5, device=dev)
        w_full = randn_bf16((Nr, Kr), std=0.02, seed=6, device=dev)
        a8f, daf = _tensorquant(cfb, a_full)
        w8f, dwf = _tensorquant(cfb, w_full)
        klo, khi = par.shard_range(Kr, world, rank, 128)
        y_ref = torch.empty((Mr, Nr), dtype=torch.bfloat16, device=dev)
        cfb.lt_gemm_fp8_nt(ctx, Mr, Nr, Kr, a8f, Kr, False, daf, w8f, dwf, y_ref, Nr)
        y_rp = torch.empty_like(y_ref)
        par.row_parallel_gemm_fp8(cfb, ctx, Mr, Nr, khi - klo, a8f[:, klo:khi], daf, w8f[:, klo:khi].contiguous(), dwf, y_rp)
        assert rel_fro(y_rp.float().cpu().numpy(), y_ref.float().cpu().numpy()) < 3e-3
        # ---- the same GEMM with the reduce-scatter fused into its epilogue (bulk reduce-adds into the owners' slices
        # over NVLink): with two ranks the fp32 sum has one order, so the rows equal the all-reduce form bit for bit
        Mf, Nf, Kf = 1024, 384, 2048
        a_f = randn_bf16((Mf, Kf), seed=15, device=dev)
        w_f = randn_bf16((Nf, Kf), std=0.02, seed=16, device=dev)
        a8g, dag = _tensorquant(cfb, a_f)
        w8g, dwg = _tensorquant(cfb, w_f)
        k0, k1 = par.shard_range(Kf, world, rank, 128)
        want = torch.empty((Mf, Nf), dtype=torch.bfloat16, device=dev)
        par.row_parallel_gemm_fp8(cfb, ctx, Mf, Nf, k1 - k0, a8g[:, k0:k1], dag, w8g[:, k0:k1].contiguous(), dwg, want)
        rs = par.RowParallelReduceScatterGemm(cfb, ctx, Mf, Nf, device=dev)
        got = torch.empty((Mf // world, Nf), dtype=torch.bfloat16, device=dev)
        for _ in range(3):          # both accumulation slices, and the re-zeroing between uses
            got.zero_()
            rs.forward(a8g[:, k0:k1], dag, w8g[:, k0:k1].contiguous(), dwg, got)
            assert torch.equal(got.view(torch.int16), want[rank * (Mf // world):(rank + 1) * (Mf // world)].view(torch.int16))
        ctx.poll_status()
        # ---- expert-parallel MoE vs the single-GPU layer on all tokens
        rows, H, F, E, k = 256, 128, 256, 4, 2
        gw = torch.Generator(device=dev).manual_seed(11)
        wgu = (torch.randn((E, 2 * F, H), generator=gw, device=dev) * 0.05).to(torch.bfloat16)
        wd = (torch.randn((E, H, F), generator=gw, device=dev) * 0.05).to(torch.bfloat16)
        wgu8, dgu = _tensorquant(cfb, wgu)
        wd8, dd = _tensorquant(cfb, wd)
        xs = [randn_bf16((rows, H), seed=100 + r, device=dev) for r in range(world)]
        logits = [_zipf_logits(rows, E, 200 + r, dev) for r in range(world)]
        e_lo, e_hi = par.EpPlan.expert_range(E, world, rank)
        ep = par.EpMoeSwigluFp8(cfb, ctx, rows, H, F, E, k, device=dev)
        mixed = torch.zeros((rows, H), dtype=torch.bfloat16, device=dev)
        for step in range(2):      # second step exercises the delayed scales
            rw = logits[rank].clone()
            mixed.zero_()
            ep.forward(xs[rank], rw, wgu8[e_lo:e_hi].contiguous(), dgu, wd8[e_lo:e_hi].contiguous(), dd, mixed)
            ctx.poll_status()
        assert sum(ep.plan.send_splits) == rows * k
        # the GEMM that writes its output straight into the owners' buffers (P2P stores) gives the same bits as the
        # GEMM followed by the bf16 all-to-all
        ep2 = par.EpMoeSwigluFp8(cfb, ctx, rows, H, F, E, k, device=dev, fused_return=True)
        mixed_f = torch.zeros((rows, H), dtype=torch.bfloat16, device=dev)
        for step in range(2):
            rw2 = logits[rank].clone()
            mixed_f.zero_()
            ep2.forward(xs[rank], rw2, wgu8[e_lo:e_hi].contiguous(), dgu, wd8[e_lo:e_hi].contiguous(), dd, mixed_f)
            ctx.poll_status()
        assert torch.equal(mixed_f.view(torch.int16), mixed.view(torch.int16))
        # SwiGLU and the re-quantise done by the gate/up GEMM's epilogue: same bits again
        ep3 = par.EpMoeSwigluFp8(cfb, ctx, rows, H, F, E, k, device=dev, fused_swiglu=True)
        wgu8_il = cfb.fp8_interleave_gate_up(wgu8[e_lo:e_hi].contiguous())
        mixed_s = torch.zeros((rows, H), dtype=torch.bfloat16, device=dev)
        for step in range(2):
            rw3 = logits[rank].clone()
            mixed_s.zero_()
            ep3.forward(xs[rank], rw3, wgu8_il, dgu, wd8[e_lo:e_hi].contiguous(), dd, mixed_s)
            ctx.poll_status()
        assert torch.equal(mixed_s.view(torch.int16), mixed.view(torch.int16))
        # Host oracle on sampled tokens with the very scales the distributed layer used: this rank's activation
        # scale for x, and for every expert the SwiGLU slot scale of the rank that served it.
        import sys
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from oracle_bindings import Oracle
        orc = Oracle()

        def check_against_oracle(layer, out, weights_n, expert_of, rank_of):
            """weights_n [rows, V] sparse weights the layer combined with; column v is expert expert_of[v] served by rank_of[v]."""
            hs = layer.slot_h.scalars()
            mine = torch.tensor([hs["scale_snapshot"], hs["descale_snapshot"]], dtype=torch.float32, device=dev)
            allh = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(allh, mine)
            dxs = np.float32(layer.slot_x.scalars()["descale_snapshot"])
            x8n = layer.x8.cpu().numpy()
            sample = list(range(0, rows, 16))
            want = np.zeros((len(sample), H), dtype=np.uint16)
            for i, r in enumerate(sample):
                for v in range(weights_n.shape[1]):
                    wgt = weights_n[r, v]
                    if wgt <= 0:
                        continue
                    e = expert_of[v]
                    sh_, dh_ = (np.float32(q) for q in allh[rank_of[v]].cpu().tolist())
                    gu = orc.gemm_fp8_nt(x8n[r:r + 1], wgu8[e].cpu().numpy(), dxs, dgu[0].item())
                    h = orc.swiglu_forward(np.ascontiguousarray(gu[:, :F]), np.ascontiguousarray(gu[:, F:]))
                    ye = orc.gemm_fp8_nt(orc.quantize_bf16(h, sh_), wd8[e].cpu().numpy(), dh_, dd[0].item())
                    want[i] = orc.to_bf16(orc.bf16_to_f32(want[i:i + 1]) + wgt * orc.bf16_to_f32(ye))[0]
            err = rel_fro(out[sample].float().cpu().numpy(), orc.bf16_to_f32(want))
            assert err < 1e-2, err

        owners = [[q for q in range(world) if par.EpPlan.expert_range(E, world, q)[0] <= e < par.EpPlan.expert_range(E, world, q)[1]][0]
                  for e in range(E)]
        check_against_oracle(ep, mixed, rw.cpu().numpy(), list(range(E)), owners)
        # ---- popular experts replicated: expert 0 is expected to take most rows, so both ranks serve it; every
        # selected (row, expert) goes to exactly one replica and the rows of an expert split by the replicas' shares
        pl = par.ReplicaPlacement.build([5.0, 1.0, 1.0, 1.0], world)
        assert pl.num_replicas > E and pl.replica_expert == sorted(pl.replica_expert)
        loc = pl.local_experts(rank)
        ep4 = par.EpMoeSwigluFp8(cfb, ctx, rows, H, F, E, k, device=dev, placement=pl)
        mixed_r = torch.zeros((rows, H), dtype=torch.bfloat16, device=dev)
        for step in range(2):
            rw4 = logits[rank].clone()
            ep4.forward(xs[rank], rw4, wgu8[loc].contiguous(), dgu, wd8[loc].contiguous(), dd, mixed_r, accumulate=False)
            ctx.poll_status()
        rwv_n, rw4_n = ep4.rwv.cpu().numpy(), rw4.cpu().numpy()
        for e in range(E):
            cols = rwv_n[:, pl.replica_start[e]:pl.replica_start[e + 1]]
            assert np.array_equal(cols.sum(axis=1), rw4_n[:, e]) and ((cols > 0).sum(axis=1) <= 1).all()
        assert np.array_equal(rw4_n, rw.cpu().numpy())
        check_against_oracle(ep4, mixed_r, rwv_n, pl.replica_expert, pl.replica_rank)
        # ---- the same layer with plan, dispatch and return on the device (no host copy of the counts, rows stored
        # straight into the serving ranks' buffers, one ragged group per replica): same bits as the all-to-all form
        ep5 = par.EpMoeSwigluFp8Direct(cfb, ctx, rows, H, F, E, k, placement=pl, device=dev)
        wgu_il_loc = cfb.fp8_interleave_gate_up(wgu8[loc].contiguous())
        mixed_d = torch.zeros((rows, H), dtype=torch.bfloat16, device=dev)
        for step in range(2):
            rw5 = logits[rank].clone()
            ep5.forward(xs[rank], rw5, wgu_il_loc, dgu, wd8[loc].contiguous(), dd, mixed_d, accumulate=False)
            ctx.poll_status()
        assert torch.equal(ep5.counts, ep4.counts) and int(ep5.grp_counts.sum().item()) == ep4.plan.total_recv
        assert torch.equal(mixed_d.view(torch.int16), mixed_r.view(torch.int16))
        # ... and with the results written locally and copied out afterwards instead of leaving from the GEMM epilogue
        ep6 = par.EpMoeSwigluFp8Direct(cfb, ctx, rows, H, F, E, k, placement=pl, device=dev, fused_return=False)
        mixed_e = torch.zeros((rows, H), dtype=torch.bfloat16, device=dev)
        for step in range(2):
            rw6 = logits[rank].clone()
            ep6.forward(xs[rank], rw6, wgu_il_loc, dgu, wd8[loc].contiguous(), dd, mixed_e, accumulate=False)
            ctx.poll_status()
        assert ep5.fused_return and torch.equal(mixed_e.view(torch.int16), mixed_r.view(torch.int16))
        # ... and with a library all-reduce in place of the flag-word barrier between the ranks
        ep7 = par.EpMoeSwigluFp8Direct(cfb, ctx, rows, H, F, E, k, placement=pl, device=dev, barrier="nccl")
        mixed_n = torch.zeros((rows, H), dtype=torch.bfloat16, device=dev)
        for step in range(2):
            rw7 = logits[rank].clone()
            ep7.forward(xs[rank], rw7, wgu_il_loc, dgu, wd8[loc].contiguous(), dd, mixed_n, accumulate=False)
            ctx.poll_status()
        assert torch.equal(mixed_n.view(torch.int16), mixed_r.view(torch.int16))
        # the flag-word barrier many times in a row, every rank checking what the others wrote before the barrier
        pb = par.PeerBarrier(cfb, ctx, device=dev)
        import torch.distributed._symmetric_memory as symm_mem
        box = symm_mem.empty((world,), dtype=torch.float32, device=dev)
        hb = symm_mem.rendezvous(box, dist.group.WORLD)
        peers = [hb.get_buffer(r, (world,), torch.float32) for r in range(world)]
        box.zero_()
        dist.barrier()
        for it in range(1, 40):
            for r in range(world):
                peers[r][rank] = float(it * 10 + rank)        # a store into every rank's box (peer memory)
            pb.wait()
            got = box.clone()
            pb.wait()                                          # nobody overwrites before everybody has read
            assert got.cpu().tolist() == [float(it * 10 + r) for r in range(world)], (it, got)
        ctx.poll_status()
        # and against the single-GPU layer on all tokens: a different scale granularity (one activation scale per rank
        # instead of one over all tokens), so the two differ by FP8 quantisation noise, not by more
        single = cfb.MoeSwigluFp8(ctx, rows * world, H, F, E, k, device=dev)
        ref = torch.zeros((rows * world, H), dtype=torch.bfloat16, device=dev)
        for step in range(2):
            rw_all = torch.cat(logits).contiguous()
            ref.zero_()
            single.forward(torch.cat(xs).contiguous(), rw_all, wgu8, dgu, wd8, dd, ref)
            ctx.poll_status()
        err2 = rel_fro(mixed.float().cpu().numpy(), ref[rank * rows:(rank + 1) * rows].float().cpu().numpy())
        assert err2 < 0.12, err2
        ctx.close()
        ret[rank] = "ok"
    except Exception:  # noqa: BLE001
        import traceback
        ret[rank] = traceback.format_exc()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_sharded_weight_and_expert_parallel_moe(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mgr = mp.Manager()
    ret = mgr.dict()
    port = _free_port()
    ctxm = mp.get_context("spawn")
    procs = [ctxm.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert not p.is_alive(), "rank did not finish"
    for r in range(world):
        assert ret.get(r) == "ok", ret.get(r)
