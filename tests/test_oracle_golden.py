"""Pins the CPU oracle against the reference's golden vectors (no GPU)."""
import json
import os

import numpy as np
import pytest


def _all_bf16():
    return (np.arange(65536, dtype=np.uint32) << 16).view(np.float32)


def test_e4m3_encoder_matches_reference_codec_on_every_bf16(oracle, golden_dir):
    g = np.load(os.path.join(golden_dir, "e4m3_codec_all_bf16.npz"))
    x = _all_bf16()
    got = oracle.quantize_f32(x, 1.0)
    # NVIDIA SATFINITE semantics (what k_quant_e4m3 executes): every input.
    assert np.array_equal(got, g["nv_e4m3"])
    # fp8_e4m3::pack agrees on every finite input ...
    fin = np.isfinite(x)
    assert np.array_equal(got[fin], g["ref_pack"][fin])
    # ... and the oracle's pack-flavoured encoder agrees on all of them.
    import ctypes as C
    fl = C.c_int()
    packed = np.array([oracle.lib.orc_e4m3_pack(float(v), C.byref(fl)) for v in x[~fin]], dtype=np.uint8)
    assert np.array_equal(packed, g["ref_pack"][~fin])


def test_e5m2_encoder_matches_nvidia_host_conversion(oracle, golden_dir):
    g = np.load(os.path.join(golden_dir, "e4m3_codec_all_bf16.npz"))
    assert np.array_equal(oracle.quantize_f32(_all_bf16(), 1.0, True), g["nv_e5m2"])


def test_e4m3_decoder_matches_reference_unpack(oracle, golden_dir):
    g = np.load(os.path.join(golden_dir, "e4m3_codec_all_bf16.npz"))
    got = oracle.decode(np.arange(256, dtype=np.uint8))
    want = g["ref_unpack_bits"].view(np.float32)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))


def test_probe_known_answers(oracle, golden_dir):
    import ctypes as C
    kat = json.load(open(os.path.join(golden_dir, "e4m3_probe_kat.json")))
    x = np.array(kat["input_f32_bits"], dtype=np.uint32).view(np.float32)
    fl = C.c_int()
    packed = [oracle.lib.orc_e4m3_pack(float(v), C.byref(fl)) for v in x]
    assert packed == kat["ref_pack"]
    for idx, code in kat["pinned"].items():
        assert packed[int(idx)] == code


def test_round_trip_and_ties(oracle):
    codes = np.array([c for c in range(256) if (c & 0x7f) != 0x7f], dtype=np.uint8)
    assert np.array_equal(oracle.quantize_f32(oracle.decode(codes), 1.0), codes)
    c5 = np.array([c for c in range(256) if (c & 0x7f) < 0x7c], dtype=np.uint8)
    assert np.array_equal(oracle.quantize_f32(oracle.decode(c5, True), 1.0, True), c5)
    # half of the smallest subnormal rounds to even (zero)
    assert oracle.lib.orc_e4m3_encode(2.0 ** -10) == 0
    assert oracle.lib.orc_e4m3_encode(np.nextafter(np.float32(2.0 ** -10), np.float32(1))) == 1
    assert oracle.lib.orc_e4m3_encode(464.0) == 0x7e and oracle.lib.orc_e4m3_encode(1e30) == 0x7e
    assert oracle.lib.orc_e5m2_encode(1e30) == 0x7b and oracle.lib.orc_e5m2_encode(float("-inf")) == 0xfb


def test_scale_and_delayed_ring(oracle):
    s, d = oracle.scale_from_amax(0.0, 448.0)
    assert s == np.float32(448.0) / np.float32(1e-12) and d == np.float32(1e-12) / np.float32(448.0)
    s, d = oracle.scale_from_amax(3.5, 448.0)
    assert s == np.float32(448.0) / np.float32(3.5) and d == np.float32(3.5) / np.float32(448.0)
    hist = np.zeros(8, dtype=np.float32)
    cur = cnt = 0
    amaxes = [1.0, 5.0, 2.0, 0.5, 0.25, 0.1, 0.2, 0.3, 0.4, 0.6, 0.7]
    for i, a in enumerate(amaxes):
        s, d, cur, cnt = oracle.update_delayed_scale(a, 448.0, hist, 8, cur, cnt)
        window = amaxes[max(0, i - 7): i + 1]
        assert s == np.float32(448.0) / np.float32(max(window))
        assert cur == (i + 1) % 8 and cnt == min(i + 1, 8)
    # corrupt cursor resets to slot 0 (kernels/fp8.cu:124-126)
    s, d, cur, cnt = oracle.update_delayed_scale(9.0, 448.0, hist, 8, 77, cnt)
    assert cur == 1 and hist[0] == 9.0
    # history_len <= 0 degenerates to scale_from_amax and leaves cursor/count alone
    s, d, cur2, cnt2 = oracle.update_delayed_scale(2.0, 57344.0, hist, 0, 3, 4)
    assert (cur2, cnt2) == (3, 4) and s == np.float32(57344.0) / np.float32(2.0)


def test_amax_semantics(oracle):
    x = oracle.to_bf16(np.array([1.0, -7.5, np.nan, 3.0], dtype=np.float32))
    assert oracle.amax_bf16(x) == 7.5
    x = oracle.to_bf16(np.array([1.0, np.inf], dtype=np.float32))
    assert oracle.amax_bf16(x) == np.inf
    q, am = oracle.quantize_record_bf16(oracle.to_bf16(np.array([1.0, -2.0], dtype=np.float32)), 2.0, amax_in=0.0)
    assert am == 2.0 and list(q) == [0x40, 0xc8]
    q, am = oracle.quantize_record_bf16(oracle.to_bf16(np.array([1.0], dtype=np.float32)), 1.0, amax_in=5.0)
    assert am == 5.0


def test_transpose_layouts(oracle):
    rng = np.random.default_rng(1)
    w = oracle.to_bf16(rng.standard_normal((37, 53)).astype(np.float32))
    s, _ = oracle.scale_from_amax(oracle.amax_bf16(w), 448.0)
    direct = oracle.quantize_bf16(w, s)
    assert np.array_equal(oracle.quantize_transpose_e4m3(w, s), direct.T)
    a, t = oracle.quant_and_transpose_e4m3(w, s)
    assert np.array_equal(a, direct) and np.array_equal(t, direct.T)
    assert np.array_equal(oracle.transpose_u8(direct), direct.T)


def test_topk_route_matches_reference_fixture(oracle, golden_dir):
    g = json.load(open(os.path.join(golden_dir, "moe_router_parity.json")))
    logits = np.array(g["logits"], dtype=np.float32)
    got = oracle.moe_topk_route(logits, g["top_k"])
    want = np.array(g["route_weights_pre_inhibition"], dtype=np.float32)
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-7)
    assert np.array_equal(got == 0, want == 0)
    # ties: lowest index wins (kernels/moe.cu:387-395)
    tie = oracle.moe_topk_route(np.zeros((1, 4), dtype=np.float32), 2)
    assert list(tie[0]) == [0.5, 0.5, 0.0, 0.0]


def test_expert_bank_mix_matches_reference_fixture(oracle, golden_dir):
    """tests/moe_router_parity_check.cu:158-178: trunk + per-expert fc_in -> GELU ->
    fc_out -> mixed += w*term, all bf16 tensors with fp32 accumulate."""
    g = json.load(open(os.path.join(golden_dir, "moe_router_parity.json")))
    H, E = g["H"], g["num_experts"]
    hg = np.array(g["hidden_gated"], dtype=np.float32).reshape(-1, H)
    rw = np.ascontiguousarray(np.array(g["route_weights"], dtype=np.float32).reshape(-1, E))
    rows = hg.shape[0]
    rw = np.repeat(rw, rows // rw.shape[0], axis=0).copy()
    x = oracle.to_bf16(hg)
    t_in = oracle.to_bf16(np.array(g["trunk_fc_in_w"], dtype=np.float32))
    t_out = oracle.to_bf16(np.array(g["trunk_fc_out_w"], dtype=np.float32))
    mixed = oracle.gemm_bf16_nt(oracle.gelu_forward(oracle.gemm_bf16_nt(x, t_in)), t_out)
    for e in range(E):
        w_in = oracle.to_bf16(np.array(g["expert_fc_in_w"][e], dtype=np.float32))
        w_out = oracle.to_bf16(np.array(g["expert_fc_out_w"][e], dtype=np.float32))
        term = oracle.gemm_bf16_nt(oracle.gelu_forward(oracle.gemm_bf16_nt(x, w_in)), w_out)
        oracle.moe_scale_accumulate_bf16(mixed, term, rw, e)
    want = np.array(g["mixed"], dtype=np.float32).reshape(-1, H)
    got = oracle.bf16_to_f32(mixed)
    # the fixture is the fp32 PyTorch side; bf16 storage of every tensor bounds the gap
    np.testing.assert_allclose(got, want, rtol=0, atol=6e-3)


def test_dispatch_lists_and_combine(oracle):
    rng = np.random.default_rng(2)
    rows, E, H = 50, 5, 16
    rw = oracle.moe_topk_route(rng.standard_normal((rows, E)).astype(np.float32), 2)
    counts, idx = oracle.moe_build_expert_row_lists(rw)
    assert counts.sum() == 2 * rows
    off = oracle.moe_offsets(counts)
    assert list(off) == list(np.concatenate([[0], np.cumsum(counts)[:-1]]))
    for e in range(E):
        assert list(idx[e, :counts[e]]) == [r for r in range(rows) if rw[r, e] > 0]
    src = oracle.to_bf16(rng.standard_normal((rows, H)).astype(np.float32))
    mixed_a = np.zeros((rows, H), dtype=np.uint16)
    mixed_b = np.zeros((rows, H), dtype=np.uint16)
    for e in range(E):
        sel = idx[e, :counts[e]]
        compact = oracle.moe_gather_rows(src, sel)
        assert np.array_equal(compact, src[sel])
        oracle.moe_scatter_accumulate_rows_bf16(mixed_a, compact, rw, sel, e)
        oracle.moe_scale_accumulate_bf16(mixed_b, src, rw, e)
    # dense combine adds w=0 terms for unselected experts: same bits
    assert np.array_equal(mixed_a, mixed_b)


def test_fp8_gemm_restatement_against_float64(oracle):
    rng = np.random.default_rng(3)
    M, N, K = 48, 40, 256
    a = oracle.to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    w = oracle.to_bf16((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    sa, da = oracle.scale_from_amax(oracle.amax_bf16(a), 448.0)
    sw, dw = oracle.scale_from_amax(oracle.amax_bf16(w), 448.0)
    a8, w8 = oracle.quantize_bf16(a, sa), oracle.quantize_bf16(w, sw)
    c = oracle.bf16_to_f32(oracle.gemm_fp8_nt(a8, w8, da, dw))
    ref = (oracle.decode(a8).astype(np.float64) @ oracle.decode(w8).astype(np.float64).T) * (float(da) * float(dw))
    assert np.linalg.norm(c - ref) / np.linalg.norm(ref) < 4e-3      # bf16 output rounding only
    f32 = oracle.gemm_fp8_nt(a8, w8, da, dw, out_kind=1)
    assert np.linalg.norm(f32 - ref) / np.linalg.norm(ref) < 1e-6
    # quantisation error itself vs the unquantised product stays inside the 1e-2 budget * few
    full = oracle.bf16_to_f32(a).astype(np.float64) @ oracle.bf16_to_f32(w).astype(np.float64).T
    assert np.linalg.norm(f32 - full) / np.linalg.norm(full) < 6e-2
    # strided A (lda > K) and beta=1 accumulate forms
    a_wide = np.zeros((M, 3 * K), dtype=np.uint8); a_wide[:, K:2 * K] = a8
    c2 = oracle.gemm_fp8_nt(np.ascontiguousarray(a_wide.reshape(-1)[K:]).reshape(-1), w8, da, dw, lda=3 * K, M=M)
    assert np.array_equal(c2[:, :N], oracle.gemm_fp8_nt(a8, w8, da, dw))
    acc = oracle.gemm_fp8_nt(a8, w8, da, dw, out_kind=2, C_init=np.ones((M, N), dtype=np.float32))
    np.testing.assert_allclose(acc, f32 + 1.0, rtol=1e-6)


def test_bias_orders(oracle):
    rng = np.random.default_rng(4)
    M, N, K = 8, 16, 64
    a8 = oracle.quantize_f32(rng.standard_normal((M, K)).astype(np.float32), 50.0)
    w8 = oracle.quantize_f32(rng.standard_normal((N, K)).astype(np.float32), 50.0)
    bias = oracle.to_bf16((rng.standard_normal(N) * 0.01).astype(np.float32))
    plain = oracle.gemm_fp8_nt(a8, w8, 0.02, 0.02)
    two_step = plain.copy()
    oracle.bias_add_strided_bf16(two_step, bias, M, N, N, 0)
    assert np.array_equal(oracle.gemm_fp8_nt(a8, w8, 0.02, 0.02, bias=bias, bias_mode=2), two_step)
    fused = oracle.bf16_to_f32(oracle.gemm_fp8_nt(a8, w8, 0.02, 0.02, bias=bias, bias_mode=1))
    assert np.abs(fused - oracle.bf16_to_f32(two_step)).max() <= 2 ** -7 * np.abs(fused).max()


def test_config1_cpu_reference_case(oracle):
    """The CPU reference case: fp32 A[256x512]~N(0,1), W[512x512]~N(0,0.02), bias~N(0,0.01), seed 0."""
    rng = np.random.default_rng(0)
    A = rng.standard_normal((256, 512)).astype(np.float32)
    W = (rng.standard_normal((512, 512)) * 0.02).astype(np.float32)
    b = (rng.standard_normal(512) * 0.01).astype(np.float32)
    out = oracle.linear_f32_e4m3(A, W, b)
    full = A.astype(np.float64) @ W.astype(np.float64).T + b
    assert np.linalg.norm(out - full) / np.linalg.norm(full) < 6e-2
    sa, da = oracle.scale_from_amax(oracle.amax_f32(A), 448.0)
    sw, dw = oracle.scale_from_amax(oracle.amax_f32(W), 448.0)
    deq = (oracle.decode(oracle.quantize_f32(A, sa)).astype(np.float64) * float(da)) @ \
          (oracle.decode(oracle.quantize_f32(W, sw)).astype(np.float64) * float(dw)).T + b
    assert np.linalg.norm(out - deq) / np.linalg.norm(deq) < 1e-5


def test_grouped_expert_forward_restatement(oracle):
    rng = np.random.default_rng(5)
    rows, H, Ie, E = 24, 32, 48, 3
    x = oracle.to_bf16(rng.standard_normal((rows, H)).astype(np.float32))
    sx, dx = oracle.scale_from_amax(oracle.amax_bf16(x), 448.0)
    x8 = oracle.quantize_bf16(x, sx)
    win = oracle.to_bf16((rng.standard_normal((E, Ie, H)) * 0.2).astype(np.float32))
    wout = oracle.to_bf16((rng.standard_normal((E, H, Ie)) * 0.2).astype(np.float32))
    si, di = oracle.scale_from_amax(oracle.amax_bf16(win), 448.0)
    so, do = oracle.scale_from_amax(oracle.amax_bf16(wout), 448.0)
    win8, wout8 = oracle.quantize_bf16(win, si), oracle.quantize_bf16(wout, so)
    rw = oracle.moe_topk_route(rng.standard_normal((rows, E)).astype(np.float32), 2)
    counts, idx = oracle.moe_build_expert_row_lists(rw)
    mixed = np.zeros((rows, H), dtype=np.uint16)
    oracle.moe_grouped_expert_forward_fp8(x8, dx, rw, counts, idx, win8, di, wout8, do, mixed)
    xf = oracle.decode(x8).astype(np.float64) * float(dx)
    want = np.zeros((rows, H))
    from math import erf
    gelu = np.vectorize(lambda v: 0.5 * v * (1 + erf(v / 2 ** 0.5)))
    for e in range(E):
        h = gelu(xf @ (oracle.decode(win8[e]).astype(np.float64) * float(di)).T)
        y = h @ (oracle.decode(wout8[e]).astype(np.float64) * float(do)).T
        want += rw[:, e:e + 1].astype(np.float64) * y
    got = oracle.bf16_to_f32(mixed)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 8e-3


def test_lion_step_restatement(oracle):
    """kernels/lion.cu: sign update, decoupled weight decay, hash-driven stochastic rounding, pre-rounding amax."""
    rng = np.random.default_rng(7)
    n = 1000
    w0 = oracle.to_bf16(rng.standard_normal(n).astype(np.float32))
    g = rng.standard_normal(n).astype(np.float32)
    m0 = (rng.standard_normal(n) * 0.1).astype(np.float32)
    w, m = w0.copy(), m0.copy()
    am = oracle.lion_step(w, m, g, 1e-2, 0.9, 0.99, 0.1, amax=0.0, seed=123)
    wf = oracle.bf16_to_f32(w0).astype(np.float64)
    blend = 0.9 * m0.astype(np.float64) + 0.1 * g
    w_new = wf - 1e-2 * (np.sign(blend) + 0.1 * wf)
    np.testing.assert_allclose(m, 0.99 * m0 + 0.01 * g, rtol=1e-6, atol=1e-7)
    # stochastic rounding moves a value to one of its two bf16 neighbours
    got = oracle.bf16_to_f32(w).astype(np.float64)
    assert np.all(np.abs(got - w_new) <= np.abs(w_new) * 2.0 ** -7 + 1e-30)
    assert abs(float(am) - np.abs(w_new).max()) <= 1e-6 * np.abs(w_new).max()
    # same seed, same result; different seed, different rounding somewhere
    w2, m2 = w0.copy(), m0.copy()
    oracle.lion_step(w2, m2, g, 1e-2, 0.9, 0.99, 0.1, seed=123)
    assert np.array_equal(w2, w)
    w3, m3 = w0.copy(), m0.copy()
    oracle.lion_step(w3, m3, g, 1e-2, 0.9, 0.99, 0.1, seed=124)
    assert not np.array_equal(w3, w)


@pytest.mark.parametrize("rows,H", [(5, 512), (3, 4096), (4, 96), (2, 1000)])
def test_rmsnorm_restatement(oracle, rows, H):
    """kernels/rmsnorm.cu:13-54: the restated summation order stays within fp32 rounding of a float64 mean square, the
    output is x / rms * scale rounded to bf16 once, and a row of constants normalises to +-scale."""
    rng = np.random.default_rng(H)
    x = oracle.to_bf16((rng.standard_normal((rows, H)) * 3).astype(np.float32))
    g = oracle.to_bf16((1 + 0.1 * rng.standard_normal(H)).astype(np.float32))
    out, rms = oracle.rmsnorm_forward(x, g, 1e-6)
    xf, gf = oracle.bf16_to_f32(x).astype(np.float64), oracle.bf16_to_f32(g).astype(np.float64)
    want_rms = np.sqrt((xf * xf).mean(axis=1) + 1e-6)
    assert np.allclose(rms, want_rms, rtol=2e-6)
    want = xf / rms.astype(np.float64)[:, None] * gf
    got = oracle.bf16_to_f32(out).astype(np.float64)
    assert np.all(np.abs(got - want) <= np.abs(want) * 2.0 ** -8 + 1e-30)         # one bf16 rounding (+ fp32 products)
    c = oracle.to_bf16(np.full((1, H), -2.5, dtype=np.float32))
    o2, r2 = oracle.rmsnorm_forward(c, g, 0.0)
    assert abs(r2[0] - 2.5) < 1e-6
    assert np.all(np.abs(oracle.bf16_to_f32(o2)[0] + oracle.bf16_to_f32(g)) <= np.abs(oracle.bf16_to_f32(g)) * 2.0 ** -7)


def test_act_row_clip_restatement(oracle):
    """src/trainer.cu:3940-3991 (fixed ceiling): rows above the ceiling come out with norm ~ ceiling, rows below are
    untouched, a non-positive ceiling disables the clip, and the restated reduction agrees with float64 to fp32 rounding."""
    rng = np.random.default_rng(3)
    x = oracle.to_bf16((rng.standard_normal((6, 1024)) * np.array([[0.5], [1], [2], [4], [8], [16]])).astype(np.float32))
    before = x.copy()
    nsq = oracle.act_row_clip(x, 70.0)
    ref = (oracle.bf16_to_f32(before).astype(np.float64) ** 2).sum(axis=1)
    assert np.allclose(nsq, ref, rtol=1e-5)
    norms = np.sqrt(ref)
    for r in range(6):
        if norms[r] <= 70.0:
            assert np.array_equal(x[r], before[r])
        else:
            after = np.sqrt((oracle.bf16_to_f32(x[r]).astype(np.float64) ** 2).sum())
            assert abs(after - 70.0) < 0.5 and not np.array_equal(x[r], before[r])
    y = before.copy()
    oracle.act_row_clip(y, 0.0)
    assert np.array_equal(y, before)
    # `if (norm <= ceiling) return;` (src/trainer.cu:3952): a NaN norm fails the test, the row is rescaled by
    # ceiling / NaN and becomes NaN everywhere; an infinite norm gives ceiling / inf = 0 (inf * 0 = NaN for the element)
    z = before.copy()
    z[0, 7] = 0x7fc0          # NaN
    z[1, 9] = 0x7f80          # +inf
    oracle.act_row_clip(z, 70.0)
    f = oracle.bf16_to_f32(z)
    assert np.isnan(f[0]).all()
    assert np.isnan(f[1, 9]) and np.all(f[1, np.arange(1024) != 9] == 0.0)
    assert np.array_equal(z[2:], x[2:])
