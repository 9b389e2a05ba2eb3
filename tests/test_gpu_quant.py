"""GPU parity of the quantize / amax / scale / transpose kernels: bit-exact against the CPU oracle and,
where oracle/_ref/libref_gpu.so was built, against the reference's own kernels on the same GPU."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import (bf16_to_u16, f32_scalar, package, randn_bf16, ref_gpu_or_none, stream_ptr, u16_to_bf16)  # noqa: E402


@pytest.fixture(scope="module")
def cfb():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return package()


@pytest.fixture(scope="module")
def refgpu():
    return ref_gpu_or_none()


def _special_values():
    v = np.array([0.0, -0.0, 1.0, -1.0, 448.0, -448.0, 447.0, 464.0, 480.0, 1e30, -1e30, np.inf, -np.inf, np.nan,
                  2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -11, 2.0 ** -6, 57344.0, 61440.0, 65536.0, 2.0 ** -16, 2.0 ** -17],
                 dtype=np.float32)
    return v


@pytest.mark.parametrize("n", [1, 7, 15, 16, 17, 255, 256, 257, 4096, 4099, 1 << 20, (1 << 20) + 13])
@pytest.mark.parametrize("e5m2", [False, True])
def test_quantize_and_record_bit_exact(cfb, oracle, refgpu, n, e5m2):
    x = randn_bf16((n,), seed=n, outlier_frac=0.001)
    xs = bf16_to_u16(x)
    fp8_max = cfb.E5M2_MAX if e5m2 else cfb.E4M3_MAX
    amax = f32_scalar()
    cfb.fp8_amax_bf16(x, amax)
    assert amax[0].item() == oracle.amax_bf16(xs)
    scale, descale = f32_scalar(), f32_scalar()
    cfb.fp8_scale_from_amax(amax, fp8_max, scale, descale)
    s_o, d_o = oracle.scale_from_amax(oracle.amax_bf16(xs), fp8_max)
    assert scale[0].item() == s_o and descale[0].item() == d_o
    out = torch.full((n + 32,), 0xAB, dtype=torch.uint8, device="cuda")     # guard band behind the output
    (cfb.fp8_quantize_e5m2 if e5m2 else cfb.fp8_quantize_e4m3)(x, out, scale)
    want = oracle.quantize_bf16(xs, s_o, e5m2)
    got = out.cpu().numpy()
    assert np.array_equal(got[:n], want)
    assert (got[n:] == 0xAB).all()
    # record form with a stale (different) scale
    stale = f32_scalar(float(s_o) * 0.37)
    am2 = f32_scalar()
    out2 = torch.empty(n, dtype=torch.uint8, device="cuda")
    (cfb.fp8_quantize_e5m2_record if e5m2 else cfb.fp8_quantize_e4m3_record)(x, out2, stale, am2)
    w2, a2 = oracle.quantize_record_bf16(xs, stale[0].item(), 0.0, e5m2)
    assert np.array_equal(out2.cpu().numpy(), w2) and am2[0].item() == a2
    if refgpu is not None:
        r_out = torch.empty(n, dtype=torch.uint8, device="cuda")
        r_am = f32_scalar()
        refgpu.call("ref_fp8_quantize_e5m2_record" if e5m2 else "ref_fp8_quantize_e4m3_record", x, r_out, stale, r_am,
                    C.c_size_t(n), stream_ptr())
        torch.cuda.synchronize()
        assert torch.equal(r_out, out2) and r_am[0].item() == am2[0].item()


@pytest.mark.parametrize("e5m2", [False, True])
def test_special_values_and_saturation(cfb, oracle, refgpu, e5m2):
    v = _special_values()
    xs = oracle.to_bf16(v)
    x = u16_to_bf16(xs)
    for sc in [1.0, 3.0, 0.0, 4.48e14]:
        scale = f32_scalar(sc)
        out = torch.empty(len(v), dtype=torch.uint8, device="cuda")
        (cfb.fp8_quantize_e5m2 if e5m2 else cfb.fp8_quantize_e4m3)(x, out, scale)
        got = out.cpu().numpy()
        if refgpu is not None:      # the reference kernel on the same GPU is the authority for non-finite inputs
            r = torch.empty(len(v), dtype=torch.uint8, device="cuda")
            refgpu.call("ref_fp8_quantize_e5m2" if e5m2 else "ref_fp8_quantize_e4m3", x, r, scale, C.c_size_t(len(v)),
                        stream_ptr())
            torch.cuda.synchronize()
            assert np.array_equal(got, r.cpu().numpy()), (sc, got, r.cpu().numpy())
        want = oracle.quantize_bf16(xs, scale[0].item(), e5m2)
        prod = oracle.bf16_to_f32(xs) * np.float32(sc)
        finite_in = ~np.isnan(prod)
        assert np.array_equal(got[finite_in], want[finite_in])
        assert ((got[~finite_in] & 0x7f) == 0x7f).all()          # NaN code
    # amax ignores NaN, +Inf propagates
    am = f32_scalar()
    cfb.fp8_amax_bf16(x, am)
    assert am[0].item() == np.inf
    y = u16_to_bf16(oracle.to_bf16(np.array([1.0, np.nan, -7.0], dtype=np.float32)))
    cfb.fp8_amax_bf16(y, am)
    assert am[0].item() == 7.0


def test_all_zero_tensor(cfb, oracle):
    x = torch.zeros(1000, dtype=torch.bfloat16, device="cuda")
    am, sc, de = f32_scalar(), f32_scalar(), f32_scalar()
    cfb.fp8_amax_bf16(x, am)
    cfb.fp8_scale_from_amax(am, 448.0, sc, de)
    s_o, d_o = oracle.scale_from_amax(0.0, 448.0)
    assert am[0].item() == 0.0 and sc[0].item() == s_o and de[0].item() == d_o
    out = torch.full((1000,), 7, dtype=torch.uint8, device="cuda")
    cfb.fp8_quantize_e4m3(x, out, sc)
    assert int(out.max().item()) == 0


@pytest.mark.parametrize("offset", [1, 3, 8, 5])
def test_unaligned_slices(cfb, oracle, offset):
    """Slices that are only 2-byte (input) / 1-byte (output) aligned."""
    n = 5000
    base = randn_bf16((n + 64,), seed=offset)
    x = base[offset:offset + n]
    xs = bf16_to_u16(x)
    sc = f32_scalar(17.0)
    for out_off in [0, 1, 8, 13]:
        buf = torch.full((n + 64,), 0xCD, dtype=torch.uint8, device="cuda")
        out = buf[out_off:out_off + n]
        am = f32_scalar()
        cfb.fp8_quantize_e4m3_record(x, out, sc, am, n)
        w, a = oracle.quantize_record_bf16(xs, 17.0)
        got = buf.cpu().numpy()
        assert np.array_equal(got[out_off:out_off + n], w) and am[0].item() == a
        assert (got[:out_off] == 0xCD).all() and (got[out_off + n:] == 0xCD).all()


def test_delayed_scale_ring(cfb, oracle):
    am, sc, de = f32_scalar(), f32_scalar(), f32_scalar()
    hist = torch.zeros(8, dtype=torch.float32, device="cuda")
    cur = torch.zeros(1, dtype=torch.int32, device="cuda")
    cnt = torch.zeros(1, dtype=torch.int32, device="cuda")
    h_o = np.zeros(8, dtype=np.float32)
    c_o = n_o = 0
    rng = np.random.default_rng(0)
    for step in range(21):
        a = float(np.float32(abs(rng.standard_normal()) * 10 ** rng.uniform(-3, 3))) if step != 5 else 0.0
        am[0] = a
        if step == 13:
            cur[0] = 99      # corrupt cursor resets to 0
            c_o = 99
        cfb.fp8_update_delayed_scale(am, 448.0, sc, de, hist, 8, cur, cnt)
        s_o, d_o, c_o, n_o = oracle.update_delayed_scale(a, 448.0, h_o, 8, c_o, n_o)
        assert sc[0].item() == s_o and de[0].item() == d_o
        assert cur.item() == c_o and cnt.item() == n_o
        assert np.array_equal(hist.cpu().numpy(), h_o)
    # history_len <= 0: plain scale_from_amax, cursor/count untouched
    am[0] = 2.5
    cfb.fp8_update_delayed_scale(am, 57344.0, sc, de, None, 0, None, None)
    s_o, d_o = oracle.scale_from_amax(2.5, 57344.0)
    assert sc[0].item() == s_o and de[0].item() == d_o


@pytest.mark.parametrize("K,N", [(1, 1), (64, 64), (256, 64), (257, 65), (300, 200), (1024, 768), (37, 1000), (1000, 37),
                                 (512, 24), (16, 4096)])
def test_transpose_family(cfb, oracle, refgpu, K, N):
    x = randn_bf16((K, N), seed=K * 31 + N)
    xs = bf16_to_u16(x)
    s_o, _ = oracle.scale_from_amax(oracle.amax_bf16(xs), 448.0)
    sc = f32_scalar(float(s_o))
    direct = oracle.quantize_bf16(xs, s_o)
    t = torch.full((N * K + 16,), 0xEE, dtype=torch.uint8, device="cuda")
    cfb.fp8_quantize_transpose_e4m3(x, t, sc, K, N)
    got = t.cpu().numpy()
    assert np.array_equal(got[:N * K].reshape(N, K), direct.T) and (got[N * K:] == 0xEE).all()
    a8 = torch.full((K * N + 16,), 0xEE, dtype=torch.uint8, device="cuda")
    sn = torch.full((N * K + 16,), 0xEE, dtype=torch.uint8, device="cuda")
    cfb.fp8_quant_and_transpose_e4m3(x, a8, sn, sc, K, N)
    ga, gs = a8.cpu().numpy(), sn.cpu().numpy()
    assert np.array_equal(ga[:K * N].reshape(K, N), direct) and (ga[K * N:] == 0xEE).all()
    assert np.array_equal(gs[:K * N].reshape(N, K), direct.T) and (gs[K * N:] == 0xEE).all()
    # snap-only call (src/trainer.cu:8225-8228)
    sn2 = torch.empty(N * K, dtype=torch.uint8, device="cuda")
    cfb.fp8_quant_and_transpose_e4m3(x, None, sn2, sc, K, N)
    assert np.array_equal(sn2.cpu().numpy().reshape(N, K), direct.T)
    # plain byte transpose
    src = torch.from_numpy(direct).cuda()
    dst = torch.empty(N * K, dtype=torch.uint8, device="cuda")
    cfb.transpose_u8(src, dst, K, N)
    assert np.array_equal(dst.cpu().numpy().reshape(N, K), direct.T)
    if refgpu is not None:
        r = torch.empty(N * K, dtype=torch.uint8, device="cuda")
        refgpu.call("ref_fp8_quantize_transpose_e4m3", x, r, sc, K, N, stream_ptr())
        torch.cuda.synchronize()
        assert np.array_equal(r.cpu().numpy().reshape(N, K), direct.T)


def test_clip_probes(cfb, oracle):
    x = randn_bf16((100000,), seed=5, outlier_frac=0.01)
    xs = bf16_to_u16(x)
    sc = f32_scalar(200.0)
    am = f32_scalar()
    cfb.fp8_amax_bf16(x, am)
    stats = torch.zeros(3, dtype=torch.float32, device="cuda")
    so = np.zeros(3, dtype=np.float32)
    for _ in range(3):
        cfb.fp8_clip_probe(am, sc, 448.0, stats)
        oracle.clip_probe(am[0].item(), 200.0, 448.0, so)
    assert np.array_equal(stats.cpu().numpy(), so)
    out = torch.zeros(2, dtype=torch.float32, device="cuda")
    oo = np.zeros(2, dtype=np.float32)
    cfb.fp8_elem_clip_count(x, sc, 448.0, out)
    oracle.elem_clip_count(xs, 200.0, 448.0, oo)
    assert np.array_equal(out.cpu().numpy(), oo) and oo[0] > 0


def test_raw_pack_path(cfb, oracle, refgpu):
    n = 70001
    x = randn_bf16((n,), seed=9)
    xs = bf16_to_u16(x)
    out = torch.empty(n, dtype=torch.uint8, device="cuda")
    dq = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    am, sc, de = f32_scalar(), f32_scalar(), f32_scalar()
    bad = torch.zeros(1, dtype=torch.int32, device="cuda")
    cfb.fp8_pack_bf16_e4m3_raw_and_dequant(x, out, dq, am, sc, de, bad)
    w, wdq, a, s, d, bi, bp = oracle.pack_raw_e4m3(xs, want_dequant=True)
    assert np.array_equal(out.cpu().numpy(), w) and np.array_equal(bf16_to_u16(dq), wdq)
    assert (am[0].item(), sc[0].item(), de[0].item()) == (a, s, d) and bad.item() == 0
    back = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    cfb.fp8_unpack_e4m3_raw_bf16(out, de, back)
    assert np.array_equal(bf16_to_u16(back), oracle.unpack_raw_e4m3_bf16(w, d))
    # non-finite inputs: counted, encoded as sign|0x7f (include/ida_native/fp8_e4m3.hpp:34)
    y = x.clone()
    y[5] = float("inf"); y[77] = float("-inf"); y[1234] = float("nan")
    ys = bf16_to_u16(y)
    cfb.fp8_pack_bf16_e4m3_raw(y, out, am, sc, de, bad)
    w, _, a, s, d, bi, bp = oracle.pack_raw_e4m3(ys)
    g = out.cpu().numpy()
    assert am[0].item() == a and sc[0].item() == s and bad.item() > 0
    nanpos = np.array([1234])
    mask = np.ones(n, dtype=bool); mask[nanpos] = False
    assert np.array_equal(g[mask], w[mask]) and g[5] == 0x7f and g[77] == 0xff and (g[1234] & 0x7f) == 0x7f
    # slices that start off the 16-byte grid take the element-wise form: same bytes
    big = randn_bf16((n + 8,), seed=10)
    out_u = torch.zeros(n + 8, dtype=torch.uint8, device="cuda")
    dq_u = torch.zeros(n + 8, dtype=torch.bfloat16, device="cuda")
    am_u, sc_u, de_u = f32_scalar(), f32_scalar(), f32_scalar()
    bad_u = torch.zeros(1, dtype=torch.int32, device="cuda")
    for off in (1, 3):
        xo = big[off:off + 4099]
        cfb.fp8_pack_bf16_e4m3_raw_and_dequant(xo, out_u[off:off + 4099], dq_u[off:off + 4099], am_u, sc_u, de_u, bad_u)
        w2, wdq2, a2, s2, d2, _, _ = oracle.pack_raw_e4m3(bf16_to_u16(xo), want_dequant=True)
        assert np.array_equal(out_u[off:off + 4099].cpu().numpy(), w2) and np.array_equal(bf16_to_u16(dq_u[off:off + 4099]), wdq2)
        back_u = torch.zeros(n + 8, dtype=torch.bfloat16, device="cuda")
        cfb.fp8_unpack_e4m3_raw_bf16(out_u[off:off + 4099], de_u, back_u[off:off + 4099])
        assert np.array_equal(bf16_to_u16(back_u[off:off + 4099]), oracle.unpack_raw_e4m3_bf16(w2, d2))
    if refgpu is not None:
        r = torch.empty(n, dtype=torch.uint8, device="cuda")
        ram, rsc, rde = f32_scalar(), f32_scalar(), f32_scalar()
        rbad = torch.zeros(1, dtype=torch.int32, device="cuda")
        refgpu.call("ref_fp8_pack_bf16_e4m3_raw", y, r, ram, rsc, rde, rbad, C.c_size_t(n), stream_ptr())
        torch.cuda.synchronize()
        assert torch.equal(r, out) and ram[0].item() == am[0].item() and rbad.item() > 0


def test_quant_act_state_machine(cfb, oracle):
    """fp8_quant_act (src/trainer.cu:4732-4851): first use, steady state with snapshot, recompute."""
    ctx = cfb.Fp8Ctx(act8_bytes=1 << 20)
    slot = cfb.ActSlot(ctx, cfb.E4M3_MAX, calib_calls=0)
    out = torch.empty(1 << 16, dtype=torch.uint8, device="cuda")
    hist = np.zeros(8, dtype=np.float32)
    cur = cnt = 0
    scale_live = None
    for step in range(12):
        x = randn_bf16((1 << 16,), std=1.0 + step, seed=100 + step)
        xs = bf16_to_u16(x)
        cfb.fp8_quant_act(ctx, slot, x, out)
        a = oracle.amax_bf16(xs)
        if step == 0:
            used, used_d = oracle.scale_from_amax(a, 448.0)
        else:
            used, used_d = scale_live
        want = oracle.quantize_bf16(xs, used)
        assert np.array_equal(out.cpu().numpy(), want), step
        s_o, d_o, cur, cnt = oracle.update_delayed_scale(a, 448.0, hist, 8, cur, cnt)
        scale_live = (s_o, d_o)
        sc = slot.scalars()
        assert sc["scale"] == s_o and sc["descale"] == d_o and sc["amax"] == a
        assert sc["scale_snapshot"] == used and sc["descale_snapshot"] == used_d
        assert sc["cursor"] == cur and sc["count"] == cnt
        # recompute reproduces the forward bytes with the snapshot and mutates nothing
        out_r = torch.empty_like(out)
        cfb.fp8_quant_act(ctx, slot, x, out_r, is_recompute=True)
        assert torch.equal(out_r, out)
        assert slot.scalars()["scale"] == s_o
    ctx.close()


def test_quant_act_calibration_flip(cfb, oracle):
    """Calibration calls use an exact per-call amax; a spread > 4x commits the slot to E5M2 on the next call."""
    ctx = cfb.Fp8Ctx(act8_bytes=1 << 16)
    slot = cfb.ActSlot(ctx, cfb.E4M3_MAX, calib_calls=3)
    out = torch.empty(4096, dtype=torch.uint8, device="cuda")
    stds = [1.0, 10.0, 0.5]
    for i, sd in enumerate(stds):
        x = randn_bf16((4096,), std=sd, seed=i)
        cfb.fp8_quant_act(ctx, slot, x, out)
        xs = bf16_to_u16(x)
        s_o, _ = oracle.scale_from_amax(oracle.amax_bf16(xs), 448.0)
        assert np.array_equal(out.cpu().numpy(), oracle.quantize_bf16(xs, s_o))
    assert slot.c.calib_commit_pending == 1 and slot.c.fp8_max == cfb.E4M3_MAX
    x = randn_bf16((4096,), std=2.0, seed=9)
    cfb.fp8_quant_act(ctx, slot, x, out)
    assert slot.c.fp8_max == cfb.E5M2_MAX
    sc = slot.scalars()
    # after the flip the slot was reseeded from the widest calibration amax and then ran a steady-state step
    xs = bf16_to_u16(x)
    assert np.array_equal(out.cpu().numpy(), oracle.quantize_bf16(xs, sc["scale_snapshot"], True))
    ctx.close()


def test_refresh_weight(cfb, oracle):
    w = randn_bf16((384, 640), std=0.02, seed=3)          # stored [in,out]
    fw = cfb.Fp8Weight(w, stored_out_major=False)
    cfb.refresh_fp8_weight(fw, recompute_amax=True)
    ws = bf16_to_u16(w)
    s_o, d_o = oracle.scale_from_amax(oracle.amax_bf16(ws), 448.0)
    direct = oracle.quantize_bf16(ws, s_o)
    assert fw.scale.item() == s_o and fw.descale.item() == d_o
    assert np.array_equal(fw.bwd8.cpu().numpy(), direct) and np.array_equal(fw.fwd8.cpu().numpy(), direct.T)
    w2 = randn_bf16((640, 384), std=0.02, seed=4)         # stored [out,in] (lm_head)
    fw2 = cfb.Fp8Weight(w2, stored_out_major=True)
    fw2.amax[0] = 0.25                                    # optimiser-provided amax, no recompute
    cfb.refresh_fp8_weight(fw2, recompute_amax=False)
    s2, _ = oracle.scale_from_amax(0.25, 448.0)
    d2 = oracle.quantize_bf16(bf16_to_u16(w2), s2)
    assert np.array_equal(fw2.fwd8.cpu().numpy(), d2) and np.array_equal(fw2.bwd8.cpu().numpy(), d2.T)


def test_argument_errors(cfb):
    sc = f32_scalar(1.0)
    with pytest.raises(cfb.CanopyError):
        cfb.fp8_quantize_e4m3(randn_bf16((16,)), None, sc)
    with pytest.raises(cfb.CanopyError):
        cfb.swiglu_forward(randn_bf16((16,)), randn_bf16((16,)), torch.empty(16, dtype=torch.bfloat16, device="cuda"), n=-1)


@pytest.mark.parametrize("bf16_state", [False, True])
@pytest.mark.parametrize("n", [1, 5, 1024, 100003])
def test_lion_step_with_fused_weight_amax(cfb, oracle, refgpu, n, bf16_state):
    """lion_step (kernels/lion.cu): bit for bit against the reference kernel on the same GPU; against the host
    restatement up to the last bit a fused multiply-add may change; the fused amax feeds the weight refresh."""
    g = torch.Generator(device="cuda").manual_seed(n)
    w0 = torch.randn(n, generator=g, device="cuda").to(torch.bfloat16)
    grad = torch.randn(n, generator=g, device="cuda")
    m0 = torch.randn(n, generator=g, device="cuda") * 0.1
    if bf16_state:
        m0 = m0.to(torch.bfloat16)
    hp = (3e-3, 0.9, 0.99, 0.1)
    w, m = w0.clone(), m0.clone()
    am = f32_scalar()
    cfb.lion_step(w, m, grad, *hp, weight_amax=am, sr_seed=77)
    if refgpu is not None:
        wr, mr = w0.clone(), m0.clone()
        amr = f32_scalar()
        refgpu.call("ref_lion_step_bf16" if bf16_state else "ref_lion_step_f32", wr, mr, grad, C.c_size_t(n),
                    C.c_float(hp[0]), C.c_float(hp[1]), C.c_float(hp[2]), C.c_float(hp[3]), stream_ptr(), amr, C.c_uint(77))
        torch.cuda.synchronize()
        assert torch.equal(w.view(torch.int16), wr.view(torch.int16))
        assert torch.equal(m.view(torch.int16) if bf16_state else m, mr.view(torch.int16) if bf16_state else mr)
        assert am[0].item() == amr[0].item()
    wo = bf16_to_u16(w0).copy()
    mo = bf16_to_u16(m0).copy() if bf16_state else m0.cpu().numpy().copy()
    a_o = oracle.lion_step(wo, mo, grad.cpu().numpy(), *hp, amax=0.0, seed=77)
    diff = np.abs(bf16_to_u16(w).astype(np.int32) - wo.astype(np.int32))
    assert (diff > 1).sum() == 0 and (diff > 0).mean() < 0.02
    np.testing.assert_allclose(am[0].item(), a_o, rtol=1e-6)
    # without an amax pointer nothing is recorded
    cfb.lion_step(w0.clone(), m0.clone(), grad, *hp, weight_amax=None, sr_seed=77)
    # the recorded amax drives the weight refresh without another pass over the weight
    if n == 1024:
        wt = w.view(32, 32).contiguous()
        fw = cfb.Fp8Weight(wt, stored_out_major=True)
        fw.amax[0] = am[0]
        cfb.refresh_fp8_weight(fw, recompute_amax=False)
        s_o, _ = oracle.scale_from_amax(am[0].item(), 448.0)
        assert np.array_equal(fw.fwd8.cpu().numpy(), oracle.quantize_bf16(bf16_to_u16(wt), s_o))


@pytest.mark.parametrize("bf16_state", [False, True])
@pytest.mark.parametrize("rows,cols", [(256, 512), (100, 72), (4096, 1024), (33, 8), (300, 4104)])
def test_lion_step_with_fused_quantise_equals_step_plus_refresh(cfb, oracle, rows, cols, bf16_state):
    """The optimiser pass that also writes both E4M3 caches: weights, momentum and the recorded amax equal the plain step
    bit for bit, and the caches equal cf_refresh_fp8_weight(recompute_amax=0) run on the updated master with the amax the
    fused call quantised with (the one an earlier step left). Two steps in a row, alternating the two amax words."""
    n = rows * cols
    g = torch.Generator(device="cuda").manual_seed(n + int(bf16_state))
    w0 = torch.randn((rows, cols), generator=g, device="cuda").to(torch.bfloat16)
    m0 = torch.randn((rows, cols), generator=g, device="cuda") * 0.1
    if bf16_state:
        m0 = m0.to(torch.bfloat16)
    hp = (3e-3, 0.9, 0.99, 0.1)
    w_a, m_a = w0.clone(), m0.clone()          # plain step + refresh
    w_b, m_b = w0.clone(), m0.clone()          # fused
    amax = [f32_scalar(), f32_scalar()]        # two words, alternating: [quantise with, record into]
    cfb.fp8_amax_bf16(w0, amax[0])             # what "the previous step" left
    sc, de = f32_scalar(), f32_scalar()
    w8 = torch.zeros((rows, cols), dtype=torch.uint8, device="cuda")
    w8t = torch.zeros((cols, rows), dtype=torch.uint8, device="cuda")
    for step in range(2):
        grad = torch.randn((rows, cols), generator=g, device="cuda")
        q, r = amax[step & 1], amax[(step + 1) & 1]
        am_a = f32_scalar()
        cfb.lion_step(w_a.view(-1), m_a.view(-1), grad.view(-1), *hp, weight_amax=am_a, sr_seed=5 + step)
        fw = cfb.Fp8Weight(w_a, stored_out_major=True)
        fw.amax[0] = q[0]
        cfb.refresh_fp8_weight(fw, recompute_amax=False)
        r.zero_()
        cfb.lion_step_quantize(w_b, m_b, grad, *hp, r, q, sc, de, w8, w8t, sr_seed=5 + step)
        assert torch.equal(w_b.view(torch.int16), w_a.view(torch.int16))
        assert torch.equal(m_b.view(torch.int16) if bf16_state else m_b, m_a.view(torch.int16) if bf16_state else m_a)
        assert r[0].item() == am_a[0].item()
        assert torch.equal(w8, fw.fwd8) and torch.equal(w8t, fw.bwd8), step
        assert sc[0].item() == fw.scale[0].item() and de[0].item() == fw.descale[0].item()
        s_o, _ = oracle.scale_from_amax(q[0].item(), 448.0)
        assert np.array_equal(w8.cpu().numpy(), oracle.quantize_bf16(bf16_to_u16(w_b), s_o))
    # the native-layout cache alone
    w8_only = torch.zeros_like(w8)
    w_c, m_c = w_b.clone(), m_b.clone()
    cfb.lion_step_quantize(w_c, m_c, grad, *hp, f32_scalar(), amax[0], sc, de, w8_only, None, sr_seed=9)
    s_o, _ = oracle.scale_from_amax(amax[0][0].item(), 448.0)
    assert np.array_equal(w8_only.cpu().numpy(), oracle.quantize_bf16(bf16_to_u16(w_c), s_o))
    # shapes the vector path cannot take are refused, and the two amax words must differ
    with pytest.raises(cfb.CanopyError):
        cfb.lion_step_quantize(w_c[:, :3].contiguous(), m_c[:, :3].contiguous(), grad[:, :3].contiguous(), *hp, f32_scalar(),
                               amax[0], sc, de, w8_only, None)
    with pytest.raises(cfb.CanopyError):
        cfb.lion_step_quantize(w_c, m_c, grad, *hp, amax[0], amax[0], sc, de, w8_only, None)
