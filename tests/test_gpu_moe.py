"""GPU parity of the MoE routing / permute / grouped GEMM / combine path and the elementwise neighbours."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import (bf16_to_u16, f32_scalar, package, randn_bf16, ref_gpu_or_none, rel_fro, stream_ptr,  # noqa: E402
                      u16_to_bf16)

TOL = 1e-2


@pytest.fixture(scope="module")
def cfb():
    assert torch.cuda.is_available()
    return package()


@pytest.fixture(scope="module")
def ctx(cfb):
    c = cfb.Fp8Ctx(act8_bytes=16 << 20)
    yield c
    c.close()


@pytest.fixture(scope="module")
def refgpu():
    return ref_gpu_or_none()


def _quant(cfb, x, e5m2=False):
    am, sc, de = f32_scalar(), f32_scalar(), f32_scalar()
    cfb.fp8_amax_bf16(x, am)
    cfb.fp8_scale_from_amax(am, cfb.E5M2_MAX if e5m2 else cfb.E4M3_MAX, sc, de)
    q = torch.empty(x.shape, dtype=torch.uint8, device="cuda")
    (cfb.fp8_quantize_e5m2 if e5m2 else cfb.fp8_quantize_e4m3)(x, q, sc)
    return q, de


def _zipf_logits(rows, E, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    p = torch.arange(1, E + 1, device="cuda", dtype=torch.float32) ** -1.1
    return torch.randn((rows, E), generator=g, device="cuda") + torch.log(p / p.sum())


def _route(cfb, rows, E, k, seed):
    rw = _zipf_logits(rows, E, seed).contiguous()
    cfb.moe_topk_route_f32(rw, rows, E, k)
    counts = torch.zeros(E, dtype=torch.int32, device="cuda")
    idx = torch.full((E, rows), -1, dtype=torch.int32, device="cuda")
    cfb.moe_build_expert_row_lists(rw, counts, idx, rows, E)
    offs = torch.empty(E, dtype=torch.int32, device="cuda")
    cfb.moe_expert_offsets_from_counts(counts, offs, E)
    return rw, counts, idx, offs


def test_elementwise(cfb, oracle, refgpu):
    for n in [1, 9, 4096, 100003]:
        g, u = randn_bf16((n,), std=3.0, seed=n), randn_bf16((n,), seed=n + 1)
        out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        cfb.swiglu_forward(g, u, out)
        want = oracle.bf16_to_f32(oracle.swiglu_forward(bf16_to_u16(g), bf16_to_u16(u)))
        # expf / erff differ by an ulp between libm and the device: one bf16 ulp of the result, plus an
        # absolute floor where 1 + erf(v) cancels (large negative v)
        got = out.float().cpu().numpy()
        assert np.all(np.abs(got - want) <= 2.0 ** -7 * np.abs(want) + 1e-6)
        cfb.gelu_forward(g, out)
        want = oracle.bf16_to_f32(oracle.gelu_forward(bf16_to_u16(g)))
        got = out.float().cpu().numpy()
        assert np.all(np.abs(got - want) <= 2.0 ** -7 * np.abs(want) + 1e-6)
        if refgpu is not None:       # same device maths as the reference kernels: bit for bit
            r = torch.empty(n, dtype=torch.bfloat16, device="cuda")
            refgpu.call("ref_swiglu_forward", g, u, r, n, stream_ptr())
            torch.cuda.synchronize()
            cfb.swiglu_forward(g, u, out)
            assert torch.equal(r.view(torch.int16), out.view(torch.int16))
            refgpu.call("ref_gelu_forward", g, r, C.c_size_t(n), stream_ptr())
            torch.cuda.synchronize()
            cfb.gelu_forward(g, out)
            assert torch.equal(r.view(torch.int16), out.view(torch.int16))
    # strided bias
    rows, H = 37, 48
    x = randn_bf16((rows, 3 * H), seed=3)
    b = randn_bf16((H,), std=0.1, seed=4)
    xs = bf16_to_u16(x).copy()
    cfb.bias_add_strided_bf16(x, b, rows, H, 3 * H, H)
    oracle.bias_add_strided_bf16(xs, bf16_to_u16(b), rows, H, 3 * H, H)
    assert np.array_equal(bf16_to_u16(x), xs)
    # shapes the 16-byte path cannot take: odd width, odd slice base, odd row pitch
    for (r2, c2, stride, base) in [(19, 45, 3 * 48, 48), (19, 48, 3 * 48, 3), (19, 48, 147, 48)]:
        x2 = randn_bf16((r2, stride), seed=5)
        b2 = randn_bf16((c2,), std=0.1, seed=6)
        xs2 = bf16_to_u16(x2).copy()
        cfb.bias_add_strided_bf16(x2, b2, r2, c2, stride, base)
        oracle.bias_add_strided_bf16(xs2, bf16_to_u16(b2), r2, c2, stride, base)
        assert np.array_equal(bf16_to_u16(x2), xs2), (r2, c2, stride, base)


@pytest.mark.parametrize("rows,E,k", [(1, 3, 2), (257, 8, 2), (4096, 8, 2), (1000, 11, 3), (64, 4, 4)])
def test_routing_and_dispatch_lists(cfb, oracle, refgpu, rows, E, k):
    logits = _zipf_logits(rows, E, rows).contiguous()
    rw = logits.clone()
    cfb.moe_topk_route_f32(rw, rows, E, k)
    want = oracle.moe_topk_route(logits.cpu().numpy(), k)
    got = rw.cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=0, atol=3e-7)
    # selection may differ only on rows whose k-th and (k+1)-th probabilities are within rounding
    mism = np.any((got > 0) != (want > 0), axis=1)
    assert mism.mean() < 1e-3
    if refgpu is not None:
        r = logits.clone()
        refgpu.call("ref_moe_topk_route_f32", r, rows, E, k, stream_ptr())
        torch.cuda.synchronize()
        np.testing.assert_allclose(r.cpu().numpy(), got, rtol=0, atol=3e-7)
        assert np.array_equal(r.cpu().numpy() > 0, got > 0)
    counts = torch.full((E,), 123, dtype=torch.int32, device="cuda")
    idx = torch.full((E, rows), -1, dtype=torch.int32, device="cuda")
    cfb.moe_build_expert_row_lists(rw, counts, idx, rows, E)
    c_o, i_o = oracle.moe_build_expert_row_lists(got)
    assert np.array_equal(counts.cpu().numpy(), c_o) and np.array_equal(idx.cpu().numpy(), i_o)
    offs = torch.empty(E, dtype=torch.int32, device="cuda")
    cfb.moe_expert_offsets_from_counts(counts, offs, E)
    assert np.array_equal(offs.cpu().numpy(), oracle.moe_offsets(c_o))
    if refgpu is not None:      # the reference's list order is atomic-dependent: compare as sets
        rc = torch.zeros(E, dtype=torch.int32, device="cuda")
        ri = torch.full((E, rows), -1, dtype=torch.int32, device="cuda")
        refgpu.call("ref_moe_build_expert_row_lists", rw, rc, ri, rows, E, stream_ptr())
        torch.cuda.synchronize()
        assert np.array_equal(rc.cpu().numpy(), c_o)
        for e in range(E):
            assert sorted(ri[e, :c_o[e]].cpu().tolist()) == i_o[e, :c_o[e]].tolist()


def test_ties_pick_lowest_index(cfb):
    s = torch.zeros((2, 5), dtype=torch.float32, device="cuda")
    cfb.moe_topk_route_f32(s, 2, 5, 2)
    assert s.cpu().tolist() == [[0.5, 0.5, 0, 0, 0]] * 2


@pytest.mark.parametrize("width", [16, 64, 100, 4096])
def test_permute_and_combine(cfb, oracle, width):
    rows, E, k = 300, 6, 2
    rw, counts, idx, offs = _route(cfb, rows, E, k, 7)
    c_n, i_n, o_n = counts.cpu().numpy(), idx.cpu().numpy(), offs.cpu().numpy()
    total = int(c_n.sum())
    src8 = torch.randint(0, 255, (rows, width), dtype=torch.uint8, device="cuda")
    compact = torch.zeros((total, width), dtype=torch.uint8, device="cuda")
    cfb.moe_gather_all_u8(src8, compact, idx, counts, offs, rows, E, width)
    for e in range(E):
        sel = i_n[e, :c_n[e]]
        assert np.array_equal(compact[o_n[e]:o_n[e] + c_n[e]].cpu().numpy(), src8.cpu().numpy()[sel])
        one = torch.empty((max(int(c_n[e]), 1), width), dtype=torch.uint8, device="cuda")
        cfb.moe_gather_rows_u8(src8, one, idx[e], int(c_n[e]), width)
        assert np.array_equal(one[:c_n[e]].cpu().numpy(), src8.cpu().numpy()[sel])
    srcb = randn_bf16((rows, width), seed=8)
    e0 = int(np.argmax(c_n))
    gb = torch.empty((int(c_n[e0]), width), dtype=torch.bfloat16, device="cuda")
    cfb.moe_gather_rows_bf16(srcb, gb, idx[e0], int(c_n[e0]), width)
    assert torch.equal(gb, srcb[idx[e0, :c_n[e0]].long()])
    # combine: per-expert scatter calls, the all-experts form and the dense form agree bit for bit with the oracle
    y = randn_bf16((total, width), seed=9)
    mixed_a = randn_bf16((rows, width), seed=10)
    mixed_b = mixed_a.clone()
    m_o = bf16_to_u16(mixed_a).copy()
    rw_n, y_n = rw.cpu().numpy(), bf16_to_u16(y)
    for e in range(E):
        if c_n[e] == 0:
            continue
        cfb.moe_scatter_accumulate_rows_bf16(mixed_a, y[o_n[e]:o_n[e] + c_n[e]], rw, idx[e], int(c_n[e]), e, E, width)
        oracle.moe_scatter_accumulate_rows_bf16(m_o, np.ascontiguousarray(y_n[o_n[e]:o_n[e] + c_n[e]]), rw_n,
                                                i_n[e, :c_n[e]], e)
    cfb.moe_combine_all_bf16(mixed_b, y, rw, idx, counts, offs, rows, E, width)
    assert np.array_equal(bf16_to_u16(mixed_a), m_o) and torch.equal(mixed_a, mixed_b)
    # the single-pass form over the ascending lists: accumulating, and starting from zero
    mixed_s = randn_bf16((rows, width), seed=10)
    cfb.moe_combine_sorted_bf16(mixed_s, y, rw, idx, counts, offs, rows, E, width, accumulate=True)
    assert torch.equal(mixed_s.view(torch.int16), mixed_a.view(torch.int16))
    zero_then_all = torch.zeros((rows, width), dtype=torch.bfloat16, device="cuda")
    cfb.moe_combine_all_bf16(zero_then_all, y, rw, idx, counts, offs, rows, E, width)
    fresh = randn_bf16((rows, width), seed=13)          # stale contents must not leak into the result
    cfb.moe_combine_sorted_bf16(fresh, y, rw, idx, counts, offs, rows, E, width, accumulate=False)
    assert torch.equal(fresh.view(torch.int16), zero_then_all.view(torch.int16))
    term = randn_bf16((rows, width), seed=11)
    mixed_c = randn_bf16((rows, width), seed=12)
    m2 = bf16_to_u16(mixed_c).copy()
    cfb.moe_scale_accumulate_bf16(mixed_c, term, rw, rows, 1, E, width)
    oracle.moe_scale_accumulate_bf16(m2, bf16_to_u16(term), rw_n, 1)
    assert np.array_equal(bf16_to_u16(mixed_c), m2)


@pytest.mark.parametrize("rows,E,N,K", [(64, 2, 256, 128), (500, 8, 384, 256), (1000, 5, 272, 528), (2048, 8, 1024, 1024)])
def test_grouped_gemm_vs_oracle(cfb, ctx, oracle, rows, E, N, K):
    """Ragged per-expert GEMM in one launch, including empty experts and one expert holding most rows."""
    rw, counts, idx, offs = _route(cfb, rows, E, 2, rows + E)
    c_n, o_n = counts.cpu().numpy(), offs.cpu().numpy()
    total = int(c_n.sum())
    x8, dx = _quant(cfb, randn_bf16((rows, K), seed=1))
    xc = torch.zeros((total, K), dtype=torch.uint8, device="cuda")
    cfb.moe_gather_all_u8(x8, xc, idx, counts, offs, rows, E, K)
    w8, dw = _quant(cfb, randn_bf16((E, N, K), std=0.02, seed=2))
    out = torch.full((total + 3, N), 5.0, dtype=torch.bfloat16, device="cuda")
    cfb.gemm_fp8_nt_grouped(ctx, E, total, N, K, counts, offs, xc, K, False, dx, False, w8, dw, out, N)
    ctx.poll_status()
    xcn, w8n = xc.cpu().numpy(), w8.cpu().numpy()
    for e in range(E):
        if c_n[e] == 0:
            continue
        want = oracle.gemm_fp8_nt(np.ascontiguousarray(xcn[o_n[e]:o_n[e] + c_n[e]]), w8n[e], dx[0].item(), dw[0].item())
        got = bf16_to_u16(out[o_n[e]:o_n[e] + c_n[e]])
        assert rel_fro(oracle.bf16_to_f32(got), oracle.bf16_to_f32(want)) < 5e-3, e
    assert (out[total:] == 5.0).all()


def test_grouped_gemm_skewed_and_empty(cfb, ctx, oracle):
    E, N, K = 4, 256, 256
    counts = torch.tensor([0, 700, 0, 1], dtype=torch.int32, device="cuda")
    offs = torch.tensor([0, 0, 700, 700], dtype=torch.int32, device="cuda")
    total = 701
    xc = torch.randint(0, 0x70, (total, K), dtype=torch.uint8, device="cuda")
    w8 = torch.randint(0, 0x70, (E, N, K), dtype=torch.uint8, device="cuda")
    d = f32_scalar(1e-3)
    out = torch.zeros((total, N), dtype=torch.bfloat16, device="cuda")
    cfb.gemm_fp8_nt_grouped(ctx, E, total, N, K, counts, offs, xc, K, False, d, False, w8, d, out, N)
    ctx.poll_status()
    xcn, w8n = xc.cpu().numpy(), w8.cpu().numpy()
    want1 = oracle.gemm_fp8_nt(np.ascontiguousarray(xcn[:700]), w8n[1], 1e-3, 1e-3)
    want3 = oracle.gemm_fp8_nt(np.ascontiguousarray(xcn[700:]), w8n[3], 1e-3, 1e-3)
    assert rel_fro(oracle.bf16_to_f32(bf16_to_u16(out[:700])), oracle.bf16_to_f32(want1)) < 5e-3
    assert rel_fro(oracle.bf16_to_f32(bf16_to_u16(out[700:])), oracle.bf16_to_f32(want3)) < 5e-3


@pytest.mark.parametrize("rows,H,Ie,E", [(96, 64, 128, 3), (512, 256, 512, 8)])
def test_grouped_expert_forward_fp8(cfb, ctx, oracle, refgpu, rows, H, Ie, E):
    """moe_grouped_expert_forward_fp8 (kernels/moe.cu:1062-1127): GELU experts, rw-weighted accumulate."""
    rw, counts, idx, offs = _route(cfb, rows, E, 2, 77)
    total = int(counts.sum().item())
    x8, dx = _quant(cfb, randn_bf16((rows, H), seed=1))
    win8, dwin = _quant(cfb, randn_bf16((E, Ie, H), std=0.05, seed=2))
    wout8, dwout = _quant(cfb, randn_bf16((E, H, Ie), std=0.05, seed=3))
    mixed = randn_bf16((rows, H), std=0.1, seed=4)
    m_o = bf16_to_u16(mixed).copy()
    ctx.reserve_workspace(total * (3 * H + 4 * Ie) + 4096)
    cfb.moe_grouped_expert_forward_fp8(ctx, x8, dx, False, rw, counts, offs, idx, win8, dwin, wout8, dwout, mixed, rows,
                                       H, Ie, E, total)
    ctx.poll_status()
    oracle.moe_grouped_expert_forward_fp8(x8.cpu().numpy(), dx[0].item(), rw.cpu().numpy(), counts.cpu().numpy(),
                                          idx.cpu().numpy(), win8.cpu().numpy(), dwin[0].item(), wout8.cpu().numpy(),
                                          dwout[0].item(), m_o)
    err = rel_fro(oracle.bf16_to_f32(bf16_to_u16(mixed)), oracle.bf16_to_f32(m_o))
    assert err < TOL, err
    if refgpu is not None:
        m_r = randn_bf16((rows, H), std=0.1, seed=4)
        refgpu.call("ref_moe_grouped_expert_forward_fp8", x8, dx, 0, rw, counts, offs, idx, win8, dwin, wout8, dwout,
                    m_r, rows, H, Ie, E, total, stream_ptr())
        torch.cuda.synchronize()
        assert rel_fro(mixed.float().cpu().numpy(), m_r.float().cpu().numpy()) < TOL


def test_ragged_expert_sequence(cfb, ctx, oracle):
    """The selected-row FP8 branch of moe_expert_bank_forward (src/trainer.cu:6886-6934): per expert gather ->
    fc_in GEMM -> GELU -> re-quantise -> fc_out GEMM -> scatter-accumulate, here with device-side scheduling."""
    rows, H, Ie, E = 400, 128, 256, 4
    rw, counts, idx, offs = _route(cfb, rows, E, 2, 5)
    c_n, i_n, o_n = counts.cpu().numpy(), idx.cpu().numpy(), offs.cpu().numpy()
    total = int(c_n.sum())
    x8, dx = _quant(cfb, randn_bf16((rows, H), seed=1))
    win8, dwin = _quant(cfb, randn_bf16((E, Ie, H), std=0.05, seed=2))
    wout8, dwout = _quant(cfb, randn_bf16((E, H, Ie), std=0.05, seed=3))
    xc = torch.empty((total, H), dtype=torch.uint8, device="cuda")
    cfb.moe_gather_all_u8(x8, xc, idx, counts, offs, rows, E, H)
    h = torch.empty((total, Ie), dtype=torch.bfloat16, device="cuda")
    cfb.gemm_fp8_nt_grouped(ctx, E, total, Ie, H, counts, offs, xc, H, False, dx, False, win8, dwin, h, Ie)
    cfb.gelu_forward(h, h)
    # per-expert activation slots (first use = exact amax), as the reference's fcout ActSlots
    g8 = torch.empty((total, Ie), dtype=torch.uint8, device="cuda")
    dg = torch.zeros(E * 4, dtype=torch.float32, device="cuda")
    for e in range(E):
        if c_n[e] == 0:
            continue
        q, d = _quant(cfb, h[o_n[e]:o_n[e] + c_n[e]])
        g8[o_n[e]:o_n[e] + c_n[e]] = q
        dg[e] = d[0]
    y = torch.empty((total, H), dtype=torch.bfloat16, device="cuda")
    cfb.gemm_fp8_nt_grouped(ctx, E, total, H, Ie, counts, offs, g8, Ie, False, dg, True, wout8, dwout, y, H)
    mixed = torch.zeros((rows, H), dtype=torch.bfloat16, device="cuda")
    cfb.moe_combine_all_bf16(mixed, y, rw, idx, counts, offs, rows, E, H)
    ctx.poll_status()
    # oracle: same sequence on the host
    m_o = np.zeros((rows, H), dtype=np.uint16)
    x8n, rw_n = x8.cpu().numpy(), rw.cpu().numpy()
    for e in range(E):
        if c_n[e] == 0:
            continue
        sel = i_n[e, :c_n[e]]
        xe = oracle.moe_gather_rows(x8n, sel)
        he = oracle.gelu_forward(oracle.gemm_fp8_nt(xe, win8[e].cpu().numpy(), dx[0].item(), dwin[0].item()))
        s_e, d_e = oracle.scale_from_amax(oracle.amax_bf16(he), 448.0)
        ye = oracle.gemm_fp8_nt(oracle.quantize_bf16(he, s_e), wout8[e].cpu().numpy(), d_e, dwout[0].item())
        oracle.moe_scatter_accumulate_rows_bf16(m_o, ye, rw_n, sel, e)
    assert rel_fro(oracle.bf16_to_f32(bf16_to_u16(mixed)), oracle.bf16_to_f32(m_o)) < TOL


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_expert_parallel_device_plan_for_every_rank(cfb, world):
    """cf_moe_ep_plan evaluated for every rank of a world on one GPU, against a host restatement: send runs tile the
    serving ranks' buffers without gaps or overlaps, groups are the replicas in id order, return runs mirror the sends."""
    par = cfb.parallel
    E = 8
    pl = par.ReplicaPlacement.build([(e + 1) ** -1.1 for e in range(E)], world)
    V = pl.num_replicas
    rng = np.random.default_rng(world)
    table = rng.integers(0, 40, size=(world, V)).astype(np.int32)
    table[rng.random((world, V)) < 0.15] = 0
    counts_all = torch.from_numpy(table).cuda()
    lo = torch.tensor([r[0] for r in pl.rank_ranges], dtype=torch.int32, device="cuda")
    hi = torch.tensor([r[1] for r in pl.rank_ranges], dtype=torch.int32, device="cuda")
    run_dt = np.dtype([("src_row", "<i8"), ("dst_row", "<i8"), ("rows", "<i4"), ("dst", "<i4")])
    assert run_dt.itemsize == cfb.ROW_RUN_BYTES
    owner = [next(g for g, (a, b) in enumerate(pl.rank_ranges) if a <= v < b) for v in range(V)]
    tot = table.sum(axis=0)
    covered = {g: [] for g in range(world)}
    sends, rets, groups = {}, {}, {}
    for me in range(world):
        n_local = pl.rank_ranges[me][1] - pl.rank_ranges[me][0]
        send = torch.zeros(V * cfb.ROW_RUN_BYTES, dtype=torch.uint8, device="cuda")
        ret = torch.zeros(max(n_local, 1) * world * cfb.ROW_RUN_BYTES, dtype=torch.uint8, device="cuda")
        gc = torch.zeros(max(n_local, 1), dtype=torch.int32, device="cuda")
        go = torch.zeros(max(n_local, 1), dtype=torch.int32, device="cuda")
        cfb.moe_ep_plan(counts_all, world, me, V, lo, hi, send, gc, go, ret)
        sends[me] = send.cpu().numpy().view(run_dt)
        rets[me] = ret.cpu().numpy().view(run_dt)[:n_local * world]
        groups[me] = (gc.cpu().numpy()[:n_local], go.cpu().numpy()[:n_local])
    for me in range(world):
        a, b = pl.rank_ranges[me]
        gc, go = groups[me]
        assert np.array_equal(gc, tot[a:b]) and np.array_equal(go, np.concatenate([[0], np.cumsum(tot[a:b])[:-1]]) if b > a else gc)
        for v in range(V):
            s = sends[me][v]
            assert s["rows"] == table[me, v] and s["dst"] == owner[v]
            base = tot[pl.rank_ranges[owner[v]][0]:v].sum()
            assert s["dst_row"] == base + table[:me, v].sum()
            covered[owner[v]].append((int(s["dst_row"]), int(s["rows"])))
        for vl, v in enumerate(range(a, b)):
            for src in range(world):
                r = rets[me][vl * world + src]
                assert r["rows"] == table[src, v] and r["dst"] == src
                assert r["src_row"] == sends[src][v]["dst_row"]              # what a source sent is what returns to it
                assert r["dst_row"] == table[src, :v].sum()                  # the source's own compact order
    for g in range(world):                                                   # receive buffers: contiguous, no overlap
        pos = 0
        for start, n in sorted(x for x in covered[g] if x[1] > 0):
            assert start == pos
            pos += n
        a, b = pl.rank_ranges[g]
        assert pos == tot[a:b].sum()


def test_a_run_that_leaves_its_destination_is_skipped_and_reported(cfb):
    """The sender checks every planned run against the number of destination buffers and their row capacity before it
    stores anything (the destinations may be other GPUs' memory): an oversize run, a run with a negative row and a run
    that names no buffer are not stored at all, the guard region behind the buffer stays untouched, the good run
    arrives, and the context reports CF_ERR_DEVICE_RANGE once and stays usable. Nothing faults."""
    ctx = cfb.Fp8Ctx(0)
    width, cap, guard = 64, 16, 8
    run_dt = np.dtype([("src_row", "<i8"), ("dst_row", "<i8"), ("rows", "<i4"), ("dst", "<i4")])
    runs = np.zeros(4, dtype=run_dt)
    runs[0] = (0, 2, 6, 0)          # fine: rows 2..7
    runs[1] = (6, 12, 8, 0)         # 12 + 8 > 16: refused as a whole
    runs[2] = (14, -1, 2, 0)        # negative row
    runs[3] = (16, 0, 2, 3)         # no such buffer
    src = torch.arange(32 * width, dtype=torch.int32, device="cuda").to(torch.uint8).view(32, width).contiguous()
    dst = torch.full((cap + guard, width), 0xAB, dtype=torch.uint8, device="cuda")
    tags = torch.full((cap + guard,), -7.0, dtype=torch.float32, device="cuda")
    bases = torch.tensor([dst.data_ptr()], dtype=torch.int64, device="cuda")
    tbases = torch.tensor([tags.data_ptr()], dtype=torch.int64, device="cuda")
    tag = torch.tensor([0.5, 0, 0, 0], dtype=torch.float32, device="cuda")
    d_runs = torch.from_numpy(runs.view(np.uint8).copy()).cuda()
    cfb.moe_send_row_runs(src, None, 0, d_runs, 4, 8, bases, width, 1, cap, tag_value=tag, tag_bases=tbases, ctx=ctx)
    with pytest.raises(cfb.CanopyError) as ei:
        ctx.poll_status()
    assert ei.value.code == cfb._capi.CF_ERR_DEVICE_RANGE
    ctx.poll_status()                                      # the word was cleared; the context is usable
    want = torch.full_like(dst, 0xAB)
    want[2:8] = src[0:6]
    assert torch.equal(dst, want)
    want_t = torch.full_like(tags, -7.0)
    want_t[2:8] = 0.5
    assert torch.equal(tags, want_t)
    # the plan cuts a group that would run past the receive capacity and reports it
    world, V = 1, 2
    counts_all = torch.tensor([[10, 10]], dtype=torch.int32, device="cuda")
    lo = torch.tensor([0], dtype=torch.int32, device="cuda")
    hi = torch.tensor([2], dtype=torch.int32, device="cuda")
    send = torch.zeros(V * cfb.ROW_RUN_BYTES, dtype=torch.uint8, device="cuda")
    ret = torch.zeros(V * cfb.ROW_RUN_BYTES, dtype=torch.uint8, device="cuda")
    gc = torch.zeros(V, dtype=torch.int32, device="cuda")
    go = torch.zeros(V, dtype=torch.int32, device="cuda")
    cfb.moe_ep_plan(counts_all, world, 0, V, lo, hi, send, gc, go, ret, recv_capacity_rows=15, ctx=ctx)
    with pytest.raises(cfb.CanopyError) as ei:
        ctx.poll_status()
    assert ei.value.code == cfb._capi.CF_ERR_DEVICE_RANGE
    assert gc.cpu().tolist() == [10, 5] and go.cpu().tolist() == [0, 10]
    cfb.moe_ep_plan(counts_all, world, 0, V, lo, hi, send, gc, go, ret, recv_capacity_rows=20, ctx=ctx)
    ctx.poll_status()
    assert gc.cpu().tolist() == [10, 10]
    ctx.close()


def test_peer_barrier_passes_when_every_word_arrived_and_gives_up_within_its_limit(cfb):
    """cf_peer_barrier on one GPU: with the peer's word already at the epoch the kernel returns at once; with a word
    nothing ever sets the bounded wait runs out after its limit (5 ms), the kernel records a status code and returns
    normally, cf_ctx_poll_status reports CF_ERR_DEVICE_WAIT once and the context stays usable. Two kernels that wait on
    each other are never launched on one GPU: the second rank is a flag array this test writes itself."""
    ctx = cfb.Fp8Ctx(0)
    mine = torch.zeros(64, dtype=torch.int32, device="cuda")
    peer = torch.zeros(64, dtype=torch.int32, device="cuda")
    arrays = torch.tensor([mine.data_ptr(), peer.data_ptr()], dtype=torch.int64, device="cuda")
    # world of one: nothing to wait for
    one = torch.tensor([mine.data_ptr()], dtype=torch.int64, device="cuda")
    cfb.peer_barrier(ctx, one, 1, 0, 1, limit_ms=5)
    ctx.poll_status()
    assert mine[0].item() == 1
    # "rank 1" has already announced epoch 7
    mine.zero_()
    mine[1] = 7
    cfb.peer_barrier(ctx, arrays, 2, 0, 7, limit_ms=5)
    ctx.poll_status()
    assert mine[0].item() == 7 and peer[0].item() == 7          # this rank's word in both arrays
    # an older epoch in the peer's word is not enough; the wait gives up
    cfb.peer_barrier(ctx, arrays, 2, 0, 8, limit_ms=5)
    with pytest.raises(cfb.CanopyError) as ei:
        ctx.poll_status()
    assert ei.value.code == cfb._capi.CF_ERR_DEVICE_WAIT
    ctx.poll_status()
    # the small all-gather that rides on the barrier: this rank's words land in row 0 of both tables
    n = 9
    src = torch.arange(100, 100 + n, dtype=torch.int32, device="cuda")
    t_mine = torch.full((2, n), -1, dtype=torch.int32, device="cuda")
    t_peer = torch.full((2, n), -1, dtype=torch.int32, device="cuda")
    tables = torch.tensor([t_mine.data_ptr(), t_peer.data_ptr()], dtype=torch.int64, device="cuda")
    mine[1] = 9                                                      # "rank 1" is already at epoch 9
    cfb.peer_share_i32(ctx, src, n, tables, arrays, 2, 0, 9, limit_ms=5)
    ctx.poll_status()
    assert torch.equal(t_mine[0], src) and torch.equal(t_peer[0], src)
    assert (t_mine[1] == -1).all() and (t_peer[1] == -1).all()      # the other rank's rows are its own business
    cfb.peer_share_i32(ctx, src, n, tables, arrays, 2, 0, 10, limit_ms=5)   # nobody announces epoch 10
    with pytest.raises(cfb.CanopyError) as ei:
        ctx.poll_status()
    assert ei.value.code == cfb._capi.CF_ERR_DEVICE_WAIT
    # epochs compare modulo 2^32: a word that has wrapped past the epoch counts as arrived, one just behind it does not
    mine[1] = 3
    cfb.peer_barrier(ctx, arrays, 2, 0, 0xFFFFFFFE, limit_ms=5)
    ctx.poll_status()
    mine[1] = -16                                    # 0xFFFFFFF0: fourteen epochs behind 0xFFFFFFFE
    cfb.peer_barrier(ctx, arrays, 2, 0, 0xFFFFFFFE, limit_ms=5)
    with pytest.raises(cfb.CanopyError):
        ctx.poll_status()
    ctx.poll_status()
    ctx.close()


def test_route_expansion_over_replicas_keeps_weights_and_follows_the_shares(cfb):
    """Every selected (row, expert) keeps its weight on exactly one replica of that expert, unselected experts stay
    zero, and the rows of an expert split over its replicas in proportion to their shares."""
    par = cfb.parallel
    rows, E, k, world = 20000, 8, 2, 8
    pl = par.ReplicaPlacement.build([(e + 1) ** -1.1 for e in range(E)], world)
    V = pl.num_replicas
    rw = _zipf_logits(rows, E, 5)
    cfb.moe_topk_route_f32(rw, rows, E, k)
    start = torch.tensor(pl.replica_start, dtype=torch.int32, device="cuda")
    cum = torch.tensor(pl.replica_cum_share, dtype=torch.float32, device="cuda")
    rwv = torch.full((rows, V), -1.0, dtype=torch.float32, device="cuda")
    cfb.moe_expand_route_replicas(rw, rwv, rows, E, V, start, cum, first_row=12345)
    a, b = rw.cpu().numpy(), rwv.cpu().numpy()
    assert (b >= 0).all()
    for e in range(E):
        cols = b[:, pl.replica_start[e]:pl.replica_start[e + 1]]
        assert np.array_equal(cols.sum(axis=1), a[:, e])
        assert ((cols > 0).sum(axis=1) == (a[:, e] > 0)).all()
        n = (a[:, e] > 0).sum()
        if n > 500:
            frac = (cols > 0).sum(axis=0) / n
            want = np.array(pl.replica_share[pl.replica_start[e]:pl.replica_start[e + 1]])
            assert np.abs(frac - want).max() < 0.05, (e, frac, want)
    # another first_row picks other replicas for the same rows: the choice follows the global row index
    rwv2 = torch.zeros_like(rwv)
    cfb.moe_expand_route_replicas(rw, rwv2, rows, E, V, start, cum, first_row=99999)
    assert not torch.equal(rwv, rwv2)


@pytest.mark.parametrize("rows,E,k,replicas", [(1, 3, 2, False), (255, 8, 2, False), (256, 8, 2, True), (257, 8, 2, True),
                                               (4096, 8, 2, True), (32768, 8, 2, False), (1000, 11, 3, True),
                                               (5000, 64, 8, False), (700, 4, 4, False), (3000, 40, 2, True)])
def test_dispatch_front_end_equals_the_separate_kernels(cfb, rows, E, k, replicas):
    """cf_moe_route_dispatch_lists leaves the route weights, replica weights, counts, offsets and list entries of the
    four separate calls, bit for bit (lists in ascending row order); cells of the lists it does not fill stay untouched."""
    par = cfb.parallel
    logits = _zipf_logits(rows, E, rows + E).contiguous()
    logits[0] = 0.0                               # ties
    V = E
    start = cum = None
    if replicas:
        pl = par.ReplicaPlacement.build([(e + 1) ** -1.1 for e in range(E)], 8)
        V = pl.num_replicas
        start = torch.tensor(pl.replica_start, dtype=torch.int32, device="cuda")
        cum = torch.tensor(pl.replica_cum_share, dtype=torch.float32, device="cuda")
    # the separate kernels
    rw0 = logits.clone()
    cfb.moe_topk_route_f32(rw0, rows, E, k)
    lists_src = rw0
    rwv0 = None
    if replicas:
        rwv0 = torch.full((rows, V), -1.0, dtype=torch.float32, device="cuda")
        cfb.moe_expand_route_replicas(rw0, rwv0, rows, E, V, start, cum, first_row=777)
        lists_src = rwv0
    c0 = torch.full((V,), 5, dtype=torch.int32, device="cuda")
    i0 = torch.full((V, rows), -7, dtype=torch.int32, device="cuda")
    o0 = torch.full((V,), 5, dtype=torch.int32, device="cuda")
    cfb.moe_build_expert_row_lists(lists_src, c0, i0, rows, V)
    cfb.moe_expert_offsets_from_counts(c0, o0, V)
    # one call
    rw1 = logits.clone()
    rwv1 = torch.full((rows, V), -1.0, dtype=torch.float32, device="cuda") if replicas else None
    c1 = torch.full((V,), 9, dtype=torch.int32, device="cuda")
    i1 = torch.full((V, rows), -7, dtype=torch.int32, device="cuda")
    o1 = torch.full((V,), 9, dtype=torch.int32, device="cuda")
    need = cfb.moe_route_dispatch_scratch_ints(rows, V)
    scratch = torch.full((need + 3,), 0x5A5A5A5A, dtype=torch.int32, device="cuda")     # contents irrelevant
    cfb.moe_route_dispatch_lists(rw1, rows, E, k, c1, o1, i1, scratch, replica_weights=rwv1, num_replicas=V,
                                 replica_start=start, replica_cum_share=cum, first_row=777)
    assert torch.equal(rw1, rw0)
    if replicas:
        assert torch.equal(rwv1, rwv0)
    assert torch.equal(c1, c0) and torch.equal(o1, o0) and torch.equal(i1, i0)
    assert (scratch[need:] == 0x5A5A5A5A).all()
    if need > 1 and V <= 64:
        with pytest.raises(cfb.CanopyError):
            cfb.moe_route_dispatch_lists(rw1, rows, E, k, c1, o1, i1, scratch[:need - 1], replica_weights=rwv1, num_replicas=V,
                                         replica_start=start, replica_cum_share=cum, first_row=777)


def test_dispatch_front_end_with_no_rows_and_with_more_than_64_lists(cfb):
    par = cfb.parallel
    E = 8
    c = torch.full((E,), 9, dtype=torch.int32, device="cuda")
    o = torch.full((E,), 9, dtype=torch.int32, device="cuda")
    i = torch.empty((E, 1), dtype=torch.int32, device="cuda")
    s = torch.empty(1, dtype=torch.int32, device="cuda")
    cfb.moe_route_dispatch_lists(torch.empty((0, E), device="cuda"), 0, E, 2, c, o, i, s)
    assert c.cpu().tolist() == [0] * E and o.cpu().tolist() == [0] * E
    # 60 experts over 8 ranks: more than 64 replicas, served by the separate kernels behind the same call
    E, rows, k = 60, 900, 2
    pl = par.ReplicaPlacement.build([1.0 + 0.01 * e for e in range(E)], 8, min_share=0.0)
    V = pl.num_replicas
    assert V > 64
    start = torch.tensor(pl.replica_start, dtype=torch.int32, device="cuda")
    cum = torch.tensor(pl.replica_cum_share, dtype=torch.float32, device="cuda")
    logits = _zipf_logits(rows, E, 3).contiguous()
    rw0, rw1 = logits.clone(), logits.clone()
    rwv0 = torch.zeros((rows, V), device="cuda")
    rwv1 = torch.zeros((rows, V), device="cuda")
    c0 = torch.zeros(V, dtype=torch.int32, device="cuda"); c1 = torch.zeros_like(c0)
    o0 = torch.zeros_like(c0); o1 = torch.zeros_like(c0)
    i0 = torch.full((V, rows), -1, dtype=torch.int32, device="cuda"); i1 = i0.clone()
    cfb.moe_topk_route_f32(rw0, rows, E, k)
    cfb.moe_expand_route_replicas(rw0, rwv0, rows, E, V, start, cum)
    cfb.moe_build_expert_row_lists(rwv0, c0, i0, rows, V)
    cfb.moe_expert_offsets_from_counts(c0, o0, V)
    cfb.moe_route_dispatch_lists(rw1, rows, E, k, c1, o1, i1, s, replica_weights=rwv1, num_replicas=V, replica_start=start,
                                 replica_cum_share=cum)
    assert torch.equal(rwv1, rwv0) and torch.equal(c1, c0) and torch.equal(o1, o0) and torch.equal(i1, i0)


def test_grouped_gemm_random_ragged_counts(cfb, ctx, oracle):
    """Twenty seeded random ragged schedules (1 to 12 groups, counts from 0 to a few tiles, some exactly on tile
    boundaries), plain and fused-SwiGLU forms, against the oracle group by group; rows past the last group stay untouched."""
    import random
    rnd = random.Random(7)
    for case in range(20):
        E = rnd.randint(1, 12)
        counts_l = [rnd.choice([0, 1, 31, 32, 33, 127, 128, 129, 255, 256, 257, 300, 512, 700]) for _ in range(E)]
        if sum(counts_l) == 0:
            counts_l[rnd.randrange(E)] = 5
        N = rnd.choice([64, 128, 256, 320, 512])
        K = rnd.choice([64, 128, 256, 528])
        total = sum(counts_l)
        offs_l = [sum(counts_l[:e]) for e in range(E)]
        counts = torch.tensor(counts_l, dtype=torch.int32, device="cuda")
        offs = torch.tensor(offs_l, dtype=torch.int32, device="cuda")
        g = torch.Generator(device="cuda").manual_seed(900 + case)
        xc = torch.randint(0, 0x70, (total, K), generator=g, dtype=torch.uint8, device="cuda")
        xc |= (torch.randint(0, 2, (total, K), generator=g, dtype=torch.uint8, device="cuda") << 7)
        w8 = torch.randint(0, 0x70, (E, N, K), generator=g, dtype=torch.uint8, device="cuda")
        w8 |= (torch.randint(0, 2, (E, N, K), generator=g, dtype=torch.uint8, device="cuda") << 7)
        da, dw = f32_scalar(2.0 ** -6), f32_scalar(2.0 ** -7)
        out = torch.full((total + 5, N), 9.0, dtype=torch.bfloat16, device="cuda")
        cfb.gemm_fp8_nt_grouped(ctx, E, total, N, K, counts, offs, xc, K, False, da, False, w8, dw, out, N)
        ctx.poll_status()
        xcn, w8n = xc.cpu().numpy(), w8.cpu().numpy()
        for e in range(E):
            if counts_l[e] == 0:
                continue
            want = oracle.gemm_fp8_nt(np.ascontiguousarray(xcn[offs_l[e]:offs_l[e] + counts_l[e]]), w8n[e], 2.0 ** -6, 2.0 ** -7)
            got = bf16_to_u16(out[offs_l[e]:offs_l[e] + counts_l[e]])
            assert rel_fro(oracle.bf16_to_f32(got), oracle.bf16_to_f32(want)) < 5e-3, (case, e, counts_l, N, K)
        assert (out[total:] == 9.0).all(), (case, counts_l)
