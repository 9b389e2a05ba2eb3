"""Host-side logic of the multi-GPU path on CPU ranks (gloo, world size 2 and 3): shard ranges, the weight-amax
max-all-reduce, the expert-parallel plan and the row exchange out and back."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gpu_util import package


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, fn_name, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        globals()[fn_name](rank, world)
        ret[rank] = "ok"
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = traceback.format_exc()
    finally:
        dist.destroy_process_group()


def _run(fn_name, world):
    mgr = mp.Manager()
    ret = mgr.dict()
    port = _free_port()
    procs = [mp.get_context("spawn").Process(target=_worker, args=(r, world, port, fn_name, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert not p.is_alive(), "rank did not finish"
    for r in range(world):
        assert ret.get(r) == "ok", ret.get(r)


def test_shard_range_partitions():
    par = package().parallel
    for n, world, mult in [(28672, 8, 1), (14336, 8, 128), (4096, 3, 256), (10, 4, 1), (5, 8, 1), (0, 2, 1)]:
        cover = []
        for r in range(world):
            lo, hi = par.shard_range(n, world, r, mult)
            assert 0 <= lo <= hi <= n
            if hi < n:
                assert (hi - lo) % mult == 0
            cover += list(range(lo, hi))
        assert cover == list(range(n))
    assert par.shard_range(28672, 8, 3) == (3 * 3584, 4 * 3584)


def _amax_case(rank, world):
    par = package().parallel
    torch.manual_seed(0)
    w = torch.randn(64, 32) * 0.02                     # the whole logical weight, same on every rank
    lo, hi = par.shard_range(64, world, rank)
    local = w[lo:hi].abs().max().reshape(1).clone()
    par.allreduce_max_(local)
    assert local.item() == w.abs().max().item()        # bit-identical to the single-GPU amax
    part = torch.full((4,), float(rank + 1))
    par.allreduce_sum_(part)
    assert part[0].item() == sum(range(1, world + 1))


def test_weight_amax_allreduce_world2():
    _run("_amax_case", 2)


def _ep_case(rank, world):
    par = package().parallel
    E, rows, k, width = 6, 40, 2, 8
    g = torch.Generator().manual_seed(100 + rank)
    # each row picks k distinct experts
    picks = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(rows)])
    counts = torch.zeros(E, dtype=torch.int32)
    for e in picks.flatten().tolist():
        counts[e] += 1
    table = par.gather_counts(counts)
    assert table[rank] == counts.tolist() and len(table) == world
    plan = par.EpPlan.build(table, rank)
    assert sum(plan.send_splits) == rows * k
    # compact send buffer ordered by expert; every row tagged (source rank, expert, running index)
    send = torch.zeros((rows * k, width), dtype=torch.int32)
    pos = 0
    for e in range(E):
        for i in range(counts[e]):
            send[pos, 0], send[pos, 1], send[pos, 2] = rank, e, i
            pos += 1
    recv = par.all_to_all_rows(send, plan.send_splits, plan.recv_splits)
    assert recv.shape[0] == plan.total_recv == sum(plan.recv_splits)
    lo, hi = par.EpPlan.expert_range(E, world, rank)
    for c, off, w_idx, src in zip(plan.seg_counts, plan.seg_offsets, plan.seg_weight, plan.seg_source):
        seg = recv[off:off + c]
        assert c == table[src][lo + w_idx]
        if c:
            assert (seg[:, 0] == src).all() and (seg[:, 1] == lo + w_idx).all()
            assert seg[:, 2].tolist() == list(range(c))
    # the way back restores the sender's order exactly
    back = par.all_to_all_rows(recv * 2, plan.recv_splits, plan.send_splits)
    assert torch.equal(back, send * 2)
    # uint8 rows (what actually travels) and a rank that receives nothing
    send8 = (send[:, :4] % 251).to(torch.uint8)
    back8 = par.all_to_all_rows(par.all_to_all_rows(send8, plan.send_splits, plan.recv_splits), plan.recv_splits, plan.send_splits)
    assert torch.equal(back8, send8)


def test_expert_parallel_plan_and_exchange_world2():
    _run("_ep_case", 2)


def test_expert_parallel_plan_and_exchange_world3():
    _run("_ep_case", 3)


def test_plan_is_consistent_across_ranks():
    par = package().parallel
    rng = np.random.default_rng(0)
    table = rng.integers(0, 50, size=(4, 8)).tolist()
    plans = [par.EpPlan.build(table, r) for r in range(4)]
    for a in range(4):
        for b in range(4):
            assert plans[a].send_splits[b] == plans[b].recv_splits[a]
    assert sum(p.total_recv for p in plans) == int(np.sum(table))


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("skew", [0.0, 1.1, 2.5])
def test_replica_placement_balances_a_skewed_load(world, skew):
    """Every rank expects the same share of the rows, owns a contiguous replica range, replica ids ascend with the expert
    id, the shares of an expert's replicas sum to one, and the plan built over the replica ranges is consistent."""
    par = package().parallel
    E = 8
    pop = [(e + 1) ** -skew for e in range(E)]
    pl = par.ReplicaPlacement.build(pop, world, min_share=0.0)
    V = pl.num_replicas
    assert pl.replica_expert == sorted(pl.replica_expert) and set(pl.replica_expert) == set(range(E))
    assert pl.replica_rank == sorted(pl.replica_rank)
    assert pl.replica_start[0] == 0 and pl.replica_start[E] == V
    load = [0.0] * world
    for e in range(E):
        ids = list(range(pl.replica_start[e], pl.replica_start[e + 1]))
        assert ids and all(pl.replica_expert[v] == e for v in ids)
        assert abs(sum(pl.replica_share[v] for v in ids) - 1.0) < 1e-9 and pl.replica_cum_share[ids[-1]] == 1.0
        assert all(pl.replica_cum_share[a] < pl.replica_cum_share[b] for a, b in zip(ids, ids[1:]))
        for v in ids:
            load[pl.replica_rank[v]] += pop[e] / sum(pop) * pl.replica_share[v]
    assert max(load) - min(load) < 1e-9
    covered = []
    for g, (lo, hi) in enumerate(pl.rank_ranges):
        assert all(pl.replica_rank[v] == g for v in range(lo, hi))
        covered += list(range(lo, hi))
    assert covered == list(range(V))
    rng = np.random.default_rng(1)
    table = rng.integers(0, 50, size=(world, V)).tolist()
    plans = [par.EpPlan.build(table, r, pl.rank_ranges) for r in range(world)]
    for a in range(world):
        for b in range(world):
            assert plans[a].send_splits[b] == plans[b].recv_splits[a]
    assert sum(p.total_recv for p in plans) == int(np.sum(table))


def test_replica_placement_drops_slivers_and_degenerates_to_sharding():
    par = package().parallel
    pl = par.ReplicaPlacement.build([1.0] * 8, 4)
    assert pl.replica_expert == list(range(8)) and pl.replica_rank == [0, 0, 1, 1, 2, 2, 3, 3]
    assert pl.rank_ranges == [(0, 2), (2, 4), (4, 6), (6, 8)]
    # a 1 % overlap with the next rank's piece is not worth a copy of the weights
    pl = par.ReplicaPlacement.build([0.505, 0.495], 2, min_share=0.05)
    assert pl.replica_expert == [0, 1] and pl.replica_rank == [0, 1]


def _placement_in_python(popularity, world, min_share=0.02):
    """The placement rule written out in Python (experts on a line cut into `world` equal pieces, slivers merged into
    the expert's largest replica): the independent statement cf_ep_placement_build is checked against."""
    E = len(popularity)
    tot = float(sum(popularity))
    p = [float(x) / tot for x in popularity]
    piece = 1.0 / world
    rep_e, rep_r, rep_len = [], [], []
    pos = 0.0
    for e in range(E):
        lo, hi = pos, pos + p[e]
        pos = hi
        g0 = min(int(lo / piece + 1e-12), world - 1)
        g1 = min(int((hi - 1e-12) / piece), world - 1) if hi > lo else g0
        parts = [[g, max(min(hi, (g + 1) * piece) - max(lo, g * piece), 0.0)] for g in range(g0, max(g1, g0) + 1)]
        keep = [q for q in parts if q[1] >= min_share * piece] or [max(parts, key=lambda q: q[1])]
        lost = sum(q[1] for q in parts) - sum(q[1] for q in keep)
        keep[max(range(len(keep)), key=lambda i: keep[i][1])][1] += lost
        for g, ov in keep:
            rep_e.append(e); rep_r.append(g); rep_len.append(ov)
    start, cum, share = [0] * (E + 1), [], []
    v = 0
    for e in range(E):
        start[e] = v
        ids = [i for i in range(len(rep_e)) if rep_e[i] == e]
        tot_e = sum(rep_len[i] for i in ids) or 1.0
        run = 0.0
        for n, i in enumerate(ids):
            sh = rep_len[i] / tot_e if p[e] > 0 else 1.0 / len(ids)
            run += sh
            share.append(sh)
            cum.append(1.0 if n == len(ids) - 1 else run)
            v += 1
    start[E] = v
    ranges, prev_hi = [], 0
    for g in range(world):
        ids = [i for i in range(v) if rep_r[i] == g]
        if ids:
            ranges.append((ids[0], ids[-1] + 1))
            prev_hi = ids[-1] + 1
        else:
            ranges.append((prev_hi, prev_hi))
    return rep_e, rep_r, share, start, cum, ranges


def test_expert_placement_from_the_library_matches_the_rule_written_in_python():
    import random
    par = package().parallel
    rnd = random.Random(7)
    cases = [([(e + 1) ** -1.1 for e in range(8)], w, 0.02) for w in (1, 2, 4, 8)]
    cases += [([1.0] * 8, 4, 0.02), ([0.505, 0.495], 2, 0.05), ([5.0, 1.0, 1.0, 1.0], 2, 0.02), ([0.0, 3.0, 0.0, 1.0], 3, 0.0)]
    for _ in range(200):
        E, w = rnd.randint(1, 40), rnd.randint(1, 16)
        pop = [rnd.random() ** 3 for _ in range(E)]
        if rnd.random() < 0.3:
            pop[rnd.randrange(E)] = 0.0
        if sum(pop) == 0:
            pop[0] = 1.0
        cases.append((pop, w, rnd.choice([0.0, 0.02, 0.1])))
    for pop, w, ms in cases:
        pl = par.ReplicaPlacement.build(pop, w, min_share=ms)
        e_, r_, sh_, st_, cum_, rg_ = _placement_in_python(pop, w, ms)
        assert pl.replica_expert == e_ and pl.replica_rank == r_ and pl.replica_start == st_
        assert [tuple(x) for x in pl.rank_ranges] == rg_
        assert np.allclose(pl.replica_share, sh_, rtol=0, atol=1e-12) and np.allclose(pl.replica_cum_share, cum_, rtol=0, atol=1e-12)
        # invariants: shares of an expert sum to 1, ranks ascend, every rank's range is contiguous
        for e in range(len(pop)):
            assert abs(sum(pl.replica_share[pl.replica_start[e]:pl.replica_start[e + 1]]) - 1.0) < 1e-9
        assert pl.replica_rank == sorted(pl.replica_rank)
    # limits are refused, not overrun
    with pytest.raises(Exception):
        par.ReplicaPlacement.build([1.0] * 300, 2)
    with pytest.raises(Exception):
        par.ReplicaPlacement.build([1.0, -1.0], 2)


def test_placement_balanced_by_tile_work_is_never_worse_and_keeps_the_invariants():
    """cf_ep_placement_build_balanced sizes the ranks' pieces for equal rows + expected padding; by its own cost model
    (rows + half a tile per replica) the busiest rank is never busier than with equal rows, and at 8 ranks under a Zipf
    load it is clearly less busy."""
    import math
    import random
    par = package().parallel
    rnd = random.Random(11)
    zipf = [25089, 14832, 9032, 5887, 4045, 2940, 2079, 1632]
    cases = [(zipf, w) for w in (1, 2, 4, 8)] + [([rnd.random() ** 2 + 0.01 for _ in range(rnd.randint(2, 32))], rnd.randint(2, 16))
                                                 for _ in range(100)]

    def worst(pl, load, total, tile):
        tot = sum(load)
        out = 0.0
        for g in range(pl.world):
            lo, hi = pl.rank_ranges[g]
            c = sum(load[pl.replica_expert[v]] / tot * total * pl.replica_share[v] + tile / 2 for v in range(lo, hi))
            out = max(out, c)
        return out

    for load, w in cases:
        total, tile = 65536, 256
        a = par.ReplicaPlacement.build(load, w)
        b = par.ReplicaPlacement.build(load, w, total_rows=total, tile_rows=tile)
        assert worst(b, load, total, tile) <= worst(a, load, total, tile) + 1e-6
        for e in range(len(load)):
            assert abs(sum(b.replica_share[b.replica_start[e]:b.replica_start[e + 1]]) - 1.0) < 1e-9
        assert b.replica_rank == sorted(b.replica_rank) and b.replica_expert == sorted(b.replica_expert)
        ids = [v for g in range(w) for v in range(*b.rank_ranges[g])]
        assert ids == list(range(b.num_replicas))
    a = par.ReplicaPlacement.build(zipf, 8)
    b = par.ReplicaPlacement.build(zipf, 8, total_rows=65536, tile_rows=256)

    def tiles(pl):
        return max(sum(math.ceil(zipf[pl.replica_expert[v]] * pl.replica_share[v] / 256) * 256 for v in range(*pl.rank_ranges[g]))
                   for g in range(8))
    assert tiles(b) <= tiles(a) - 256


def test_placement_weighted_by_rank_speed_equalises_time_and_keeps_the_invariants():
    """cf_ep_placement_build_weighted: equal speeds give the balanced placement; with unequal speeds the slowest finishing
    time (tile work / speed) is never later than with the balanced placement, and clearly earlier when one rank is slow."""
    import random
    par = package().parallel
    zipf = [25089, 14832, 9032, 5887, 4045, 2940, 2079, 1632]
    total, tile = 65536, 256

    def finish(pl, load, speed):
        tot = sum(load)
        out = 0.0
        for g in range(pl.world):
            lo, hi = pl.rank_ranges[g]
            c = sum(load[pl.replica_expert[v]] / tot * total * pl.replica_share[v] + tile / 2 for v in range(lo, hi))
            out = max(out, c / speed[g])
        return out

    for w in (2, 4, 8):
        a = par.ReplicaPlacement.build(zipf, w, total_rows=total, tile_rows=tile)
        b = par.ReplicaPlacement.build(zipf, w, total_rows=total, tile_rows=tile, rank_speed=[1.0] * w)
        assert (a.replica_expert, a.replica_rank, a.rank_ranges) == (b.replica_expert, b.replica_rank, b.rank_ranges)
        assert np.allclose(a.replica_share, b.replica_share, atol=1e-12)
    rnd = random.Random(5)
    for _ in range(60):
        w = rnd.choice([2, 4, 8])
        load = zipf if rnd.random() < 0.5 else [rnd.random() ** 2 + 0.01 for _ in range(rnd.randint(w, 24))]
        speed = [1.0 + 0.12 * (rnd.random() - 0.5) for _ in range(w)]
        a = par.ReplicaPlacement.build(load, w, total_rows=total, tile_rows=tile)
        b = par.ReplicaPlacement.build(load, w, total_rows=total, tile_rows=tile, rank_speed=speed)
        mean = sum(speed) / w
        sp = [x / mean for x in speed]
        assert finish(b, load, sp) <= finish(a, load, sp) * (1 + 1e-9)
        for e in range(len(load)):
            assert abs(sum(b.replica_share[b.replica_start[e]:b.replica_start[e + 1]]) - 1.0) < 1e-9
        ids = [v for g in range(w) for v in range(*b.rank_ranges[g])]
        assert ids == list(range(b.num_replicas))
    slow = [1.0, 0.9, 1.0, 1.0]
    a = par.ReplicaPlacement.build(zipf, 4, total_rows=total, tile_rows=tile)
    b = par.ReplicaPlacement.build(zipf, 4, total_rows=total, tile_rows=tile, rank_speed=slow)
    m = sum(slow) / 4
    assert finish(b, zipf, [x / m for x in slow]) < 0.95 * finish(a, zipf, [x / m for x in slow])
    with pytest.raises(Exception):
        par.ReplicaPlacement.build(zipf, 4, total_rows=total, tile_rows=tile, rank_speed=[1.0, 0.0, 1.0, 1.0])
