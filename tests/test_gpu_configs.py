"""The three larger workloads: SwiGLU MLP with per-token / per-channel scales, MoE SwiGLU experts and the large-shape sweep
(32768 x 8192 x 28672 E4M3 forward / E5M2 dgrad) as parity cases: reduced sizes against the oracle, full sizes through
sampled rows and size-independent properties."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import bf16_to_u16, f32_scalar, package, randn_bf16, rel_fro, u16_to_bf16  # noqa: E402

TOL = 1e-2


@pytest.fixture(scope="module")
def cfb():
    assert torch.cuda.is_available()
    return package()


@pytest.fixture(scope="module")
def ctx(cfb):
    c = cfb.Fp8Ctx(act8_bytes=1 << 20)
    yield c
    c.close()


def _rowquant(cfb, w):
    w8 = torch.empty(w.shape, dtype=torch.uint8, device="cuda")
    d = torch.empty(w.shape[0], dtype=torch.float32, device="cuda")
    cfb.fp8_quantize_rowwise_e4m3(w, w8, d)
    return w8, d


def _tensorquant(cfb, x, e5m2=False):
    am, sc, de = f32_scalar(), f32_scalar(), f32_scalar()
    cfb.fp8_amax_bf16(x, am)
    cfb.fp8_scale_from_amax(am, cfb.E5M2_MAX if e5m2 else cfb.E4M3_MAX, sc, de)
    q = torch.empty(x.shape, dtype=torch.uint8, device="cuda")
    (cfb.fp8_quantize_e5m2 if e5m2 else cfb.fp8_quantize_e4m3)(x, q, sc)
    return q, de


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 7), (17, 64), (64, 4096), (33, 14336), (5, 1000), (8, 16384),
                                       (9, 37), (21, 4100), (4, 16383), (300, 523)])
def test_rowwise_quantize_bit_exact(cfb, oracle, rows, cols):
    x = randn_bf16((rows, cols), seed=rows * cols, outlier_frac=0.01)
    x[0] = 0                                      # an all-zero row: amax clamps to 1e-12
    out = torch.full((rows, cols + 8), 0xAB, dtype=torch.uint8, device="cuda")
    sc = torch.empty(rows, dtype=torch.float32, device="cuda")
    de = torch.empty(rows, dtype=torch.float32, device="cuda")
    cfb.fp8_quantize_rowwise_e4m3(x, out, de, row_scale=sc, ld_out=cols + 8)
    w, s_o, d_o = oracle.quantize_rowwise_e4m3(bf16_to_u16(x))
    got = out.cpu().numpy()
    assert np.array_equal(got[:, :cols], w) and (got[:, cols:] == 0xAB).all()
    assert np.array_equal(sc.cpu().numpy(), s_o) and np.array_equal(de.cpu().numpy(), d_o)
    # a strided 2-byte-aligned view (row stride cols, first column dropped) takes the scalar path
    if cols > 1:
        xv = x.view(-1)[1:]
        out2 = torch.empty((rows - 1 if rows > 1 else 1, cols), dtype=torch.uint8, device="cuda")
        if rows > 1:
            de2 = torch.empty(rows - 1, dtype=torch.float32, device="cuda")
            cfb.fp8_quantize_rowwise_e4m3(xv, out2, de2, rows=rows - 1, cols=cols - 1, ld_x=cols, ld_out=cols)
            ref = np.ascontiguousarray(bf16_to_u16(x).reshape(-1)[1:1 + (rows - 1) * cols].reshape(rows - 1, cols)[:, :cols - 1])
            w2, _, d2 = oracle.quantize_rowwise_e4m3(ref)
            assert np.array_equal(out2.cpu().numpy()[:, :cols - 1], w2) and np.array_equal(de2.cpu().numpy(), d2)


@pytest.mark.parametrize("rows,cols,in_off,out_off", [(13, 4100, 0, 0), (13, 4100, 3, 5), (6, 45, 1, 2), (40, 1023, 7, 1),
                                                      (5, 6, 5, 3)])
def test_rowwise_quantize_of_rows_that_are_not_16_byte_multiples(cfb, oracle, rows, cols, in_off, out_off):
    """Rows of any length at any 2-byte (input) / 1-byte (output) alignment: head, whole vectors and tail of every row give
    the oracle's codes, scales and descales, and nothing outside the rows is written."""
    flat = randn_bf16((rows * cols + 16,), seed=cols + in_off, outlier_frac=0.02)
    xv = flat[in_off:in_off + rows * cols]
    out_flat = torch.full((rows * cols + 32,), 0xCD, dtype=torch.uint8, device="cuda")
    ov = out_flat[out_off:]
    sc = torch.empty(rows, dtype=torch.float32, device="cuda")
    de = torch.empty(rows, dtype=torch.float32, device="cuda")
    cfb.fp8_quantize_rowwise_e4m3(xv, ov, de, row_scale=sc, rows=rows, cols=cols, ld_x=cols, ld_out=cols)
    w, s_o, d_o = oracle.quantize_rowwise_e4m3(np.ascontiguousarray(bf16_to_u16(xv).reshape(rows, cols)))
    got = out_flat.cpu().numpy()
    assert np.array_equal(got[out_off:out_off + rows * cols].reshape(rows, cols), w)
    assert (got[:out_off] == 0xCD).all() and (got[out_off + rows * cols:] == 0xCD).all()
    assert np.array_equal(sc.cpu().numpy(), s_o) and np.array_equal(de.cpu().numpy(), d_o)


@pytest.mark.parametrize("rows,F", [(11, 37), (7, 1003)])
def test_swiglu_rowwise_quantise_of_odd_rows_matches_the_two_step_sequence(cfb, rows, F):
    g = randn_bf16((rows, F), std=2.0, seed=F)
    u = randn_bf16((rows, F), std=2.0, seed=F + 1)
    h = torch.empty((rows, F), dtype=torch.bfloat16, device="cuda")
    cfb.swiglu_forward(g, u, h)
    want8 = torch.empty((rows, F), dtype=torch.uint8, device="cuda")
    want_d = torch.empty(rows, dtype=torch.float32, device="cuda")
    cfb.fp8_quantize_rowwise_e4m3(h, want8, want_d)
    got8 = torch.empty((rows, F), dtype=torch.uint8, device="cuda")
    got_d = torch.empty(rows, dtype=torch.float32, device="cuda")
    cfb.swiglu_quantize_rowwise_e4m3(g, u, got8, got_d, rows, F, F)
    assert torch.equal(got8, want8) and torch.equal(got_d, want_d)
    # gate and up at different alignments: the one-row-per-block form
    flat = randn_bf16((2 * rows * F + 8,), std=2.0, seed=F + 2)
    g2, u2 = flat[:rows * F], flat[rows * F + 2:2 * rows * F + 2]
    cfb.swiglu_forward(g2.view(rows, F).contiguous(), u2.reshape(rows, F).contiguous(), h)
    cfb.fp8_quantize_rowwise_e4m3(h, want8, want_d)
    cfb.swiglu_quantize_rowwise_e4m3(g2, u2, got8, got_d, rows, F, F)
    assert torch.equal(got8, want8) and torch.equal(got_d, want_d)


@pytest.mark.parametrize("rows,F", [(9, 40), (64, 1024), (32, 14336)])
def test_swiglu_fusions_match_the_two_step_sequence(cfb, ctx, oracle, rows, F):
    """The fused kernels must produce the bytes of swiglu_forward followed by the quantise kernel (both verified
    against the reference's own kernels elsewhere); against the CPU oracle libm's expf allows rare one-step differences."""
    gu = randn_bf16((rows, 2 * F), std=2.0, seed=F)
    gate, up = gu.view(-1), gu.view(-1)[F:]
    # two-step sequence on the device
    g_c, u_c = gu[:, :F].contiguous(), gu[:, F:].contiguous()
    h = torch.empty((rows, F), dtype=torch.bfloat16, device="cuda")
    cfb.swiglu_forward(g_c, u_c, h)
    want8 = torch.empty((rows, F), dtype=torch.uint8, device="cuda")
    want_d = torch.empty(rows, dtype=torch.float32, device="cuda")
    cfb.fp8_quantize_rowwise_e4m3(h, want8, want_d)
    got8 = torch.empty((rows, F), dtype=torch.uint8, device="cuda")
    got_d = torch.empty(rows, dtype=torch.float32, device="cuda")
    cfb.swiglu_quantize_rowwise_e4m3(gate, up, got8, got_d, rows, F, 2 * F)
    assert torch.equal(got8, want8) and torch.equal(got_d, want_d)
    o8, _, o_d = oracle.quantize_rowwise_e4m3(bf16_to_u16(g_c), bf16_to_u16(u_c))
    assert (got8.cpu().numpy() != o8).mean() < 2e-3
    np.testing.assert_allclose(got_d.cpu().numpy(), o_d, rtol=2 ** -7)
    # per-tensor record form
    sc = f32_scalar(37.0)
    am_w, am_g = f32_scalar(), f32_scalar()
    w8 = torch.empty((rows, F), dtype=torch.uint8, device="cuda")
    g8 = torch.empty((rows, F), dtype=torch.uint8, device="cuda")
    cfb.fp8_quantize_e4m3_record(h, w8, sc, am_w)
    cfb.swiglu_quantize_e4m3_record(gate, up, g8, sc, am_g, rows, F, 2 * F)
    assert torch.equal(g8, w8) and am_g[0].item() == am_w[0].item()
    # slot form over three steps: identical bytes and slot scalars as swiglu_forward + fp8_quant_act
    s_a, s_b = cfb.ActSlot(ctx, cfb.E4M3_MAX), cfb.ActSlot(ctx, cfb.E4M3_MAX)
    for step in range(3):
        gu2 = randn_bf16((rows, 2 * F), std=1.0 + step, seed=100 + step)
        cfb.swiglu_forward(gu2[:, :F].contiguous(), gu2[:, F:].contiguous(), h)
        cfb.fp8_quant_act(ctx, s_a, h, w8)
        cfb.fp8_swiglu_quant_act(ctx, s_b, gu2, gu2.view(-1)[F:], 2 * F, rows, F, g8)
        assert torch.equal(g8, w8), step
        a, b = s_a.scalars(), s_b.scalars()
        for k in ("amax", "scale", "descale", "scale_snapshot", "descale_snapshot", "history", "cursor", "count"):
            assert a[k] == b[k], (step, k)


def _mlp_oracle(oracle, x_u16, wgu8, dgu, wd8, dd):
    x8, _, dx = oracle.quantize_rowwise_e4m3(x_u16)
    gu = oracle.gemm_fp8_nt(x8, wgu8, dx, dgu)
    F = wgu8.shape[0] // 2
    h8, _, dh = oracle.quantize_rowwise_e4m3(np.ascontiguousarray(gu[:, :F]), np.ascontiguousarray(gu[:, F:]))
    return oracle.gemm_fp8_nt(h8, wd8, dh, dd)


def test_config3_swiglu_mlp_reduced(cfb, ctx, oracle):
    M, H, F = 384, 256, 640
    x = randn_bf16((M, H), seed=1)
    wgu8, dgu = _rowquant(cfb, randn_bf16((2 * F, H), std=0.02, seed=2))
    wd8, dd = _rowquant(cfb, randn_bf16((H, F), std=0.02, seed=3))
    y = torch.empty((M, H), dtype=torch.bfloat16, device="cuda")
    cfb.swiglu_mlp_fp8_rowwise(ctx, x, wgu8, dgu, wd8, dd, y)
    ctx.poll_status()
    want = _mlp_oracle(oracle, bf16_to_u16(x), wgu8.cpu().numpy(), dgu.cpu().numpy(), wd8.cpu().numpy(), dd.cpu().numpy())
    assert rel_fro(y.float().cpu().numpy(), oracle.bf16_to_f32(want)) < TOL
    # column-sharded gate/up (N split in two, outputs concatenated) and row-sharded down (K split, partial sums
    # added in fp32) reproduce the unsharded result: what each of 2 GPUs would compute
    one = torch.ones(4, dtype=torch.float32, device="cuda")
    x8 = torch.empty((M, H), dtype=torch.uint8, device="cuda"); dx = torch.empty(M, dtype=torch.float32, device="cuda")
    cfb.fp8_quantize_rowwise_e4m3(x, x8, dx)
    gu_full = torch.empty((M, 2 * F), dtype=torch.bfloat16, device="cuda")
    cfb.lt_gemm_fp8_nt(ctx, M, 2 * F, H, x8, H, False, one, wgu8, one, gu_full, 2 * F, a_row_descale=dx, b_col_descale=dgu)
    gu_sh = torch.empty_like(gu_full)
    for r in range(2):
        # rank r owns gate rows [r*F/2, (r+1)*F/2) and the matching up rows
        for base in (0, F):
            lo = base + r * (F // 2)
            cfb.lt_gemm_fp8_nt(ctx, M, F // 2, H, x8, H, False, one, wgu8[lo:lo + F // 2], one, gu_sh.view(-1)[lo:], 2 * F,
                               a_row_descale=dx, b_col_descale=dgu[lo:lo + F // 2])
    assert torch.equal(gu_sh, gu_full)
    ctx.poll_status()


def test_config3_full_size_sampled(cfb, ctx, oracle):
    """M=16384, hidden 4096, ffn 14336 at full size; sampled token rows against the oracle."""
    M, H, F = 16384, 4096, 14336
    x = randn_bf16((M, H), seed=1)
    wgu8, dgu = _rowquant(cfb, randn_bf16((2 * F, H), std=0.02, seed=2))
    wd8, dd = _rowquant(cfb, randn_bf16((H, F), std=0.02, seed=3))
    y = torch.empty((M, H), dtype=torch.bfloat16, device="cuda")
    work = cfb.swiglu_mlp_fp8_rowwise(ctx, x, wgu8, dgu, wd8, dd, y)
    ctx.poll_status()
    rows = [0, 127, 128, 255, 256, 8191, 16383]
    want = _mlp_oracle(oracle, bf16_to_u16(x[rows]), wgu8.cpu().numpy(), dgu.cpu().numpy(), wd8.cpu().numpy(), dd.cpu().numpy())
    assert rel_fro(y[rows].float().cpu().numpy(), oracle.bf16_to_f32(want)) < TOL
    # per-token scaling makes rows independent: a slab computed alone reproduces the same rows bit for bit
    y2 = torch.empty((512, H), dtype=torch.bfloat16, device="cuda")
    cfb.swiglu_mlp_fp8_rowwise(ctx, x[4096:4608], wgu8, dgu, wd8, dd, y2)
    assert torch.equal(y2, y[4096:4608])
    del work


def _interleaved(cfb, wgu8, dgu):
    F = wgu8.shape[0] // 2
    il = cfb.fp8_interleave_gate_up(wgu8.view(1, 2 * F, -1)).view(2 * F, -1)
    return il, cfb.interleave_gate_up_vector(dgu, F)


@pytest.mark.parametrize("M,H,F", [(384, 256, 640), (1000, 512, 96), (130, 128, 2048)])
def test_fused_rowwise_mlp_equals_the_unfused_composite(cfb, ctx, oracle, M, H, F):
    """Gate/up GEMM with the SwiGLU product and its per-row amax in the epilogue, then the given-amax quantiser: h, the row
    scales, the E4M3 codes and the MLP output equal the unfused composite bit for bit, and the output meets the oracle."""
    x = randn_bf16((M, H), seed=1, outlier_frac=0.002)
    wgu8, dgu = _rowquant(cfb, randn_bf16((2 * F, H), std=0.05, seed=2))
    wd8, dd = _rowquant(cfb, randn_bf16((H, F), std=0.05, seed=3))
    y0 = torch.empty((M, H), dtype=torch.bfloat16, device="cuda")
    w0 = cfb.swiglu_mlp_fp8_rowwise(ctx, x, wgu8, dgu, wd8, dd, y0)
    il, dil = _interleaved(cfb, wgu8, dgu)
    y1 = torch.full((M, H), float("nan"), dtype=torch.bfloat16, device="cuda")
    w1 = cfb.swiglu_mlp_fp8_rowwise_fused(ctx, x, il, dil, wd8, dd, y1)
    ctx.poll_status()
    hs = torch.empty((M, F), dtype=torch.bfloat16, device="cuda")
    cfb.swiglu_forward(w0["gu"][:, :F].contiguous(), w0["gu"][:, F:].contiguous(), hs)
    assert torch.equal(w1["h"].view(torch.int16), hs.view(torch.int16))
    assert torch.equal(w1["hmax"], hs.float().abs().amax(dim=1))
    assert torch.equal(w1["dh"], w0["dh"]) and torch.equal(w1["h8"], w0["h8"])
    assert torch.equal(y1.view(torch.int16), y0.view(torch.int16))
    want = _mlp_oracle(oracle, bf16_to_u16(x), wgu8.cpu().numpy(), dgu.cpu().numpy(), wd8.cpu().numpy(), dd.cpu().numpy())
    assert rel_fro(y1.float().cpu().numpy(), oracle.bf16_to_f32(want)) < TOL


def test_fused_rowwise_mlp_sharded_as_two_ranks_would_run_it(cfb, ctx):
    """Gate/up split by output features, down split by its contraction dimension, emulated rank after rank on one GPU:
    the per-row amax is max-reduced over the feature shards before the quantiser, so every shard's codes equal the same
    columns of the unsharded h8; the fp32 partial products of the down projection (row and column scales applied in the
    epilogue) add up to the unsharded output within fp32 summation order."""
    M, H, F, W = 512, 256, 1024, 2
    x = randn_bf16((M, H), seed=5)
    wgu8, dgu = _rowquant(cfb, randn_bf16((2 * F, H), std=0.05, seed=6))
    wd8, dd = _rowquant(cfb, randn_bf16((H, F), std=0.05, seed=7))
    il, dil = _interleaved(cfb, wgu8, dgu)
    y_full = torch.empty((M, H), dtype=torch.bfloat16, device="cuda")
    full = cfb.swiglu_mlp_fp8_rowwise_fused(ctx, x, il, dil, wd8, dd, y_full)
    Fl = F // W
    x8, dx = full["x8"], full["dx"]
    hs, hmaxs = [], []
    for r in range(W):
        # rank r owns features [r*Fl, (r+1)*Fl): interleaved rows [2*r*Fl, 2*(r+1)*Fl)
        il_r, dil_r = il[2 * r * Fl:2 * (r + 1) * Fl].contiguous(), dil[2 * r * Fl:2 * (r + 1) * Fl].contiguous()
        h = torch.empty((M, Fl), dtype=torch.bfloat16, device="cuda")
        hmax = torch.zeros(M, dtype=torch.float32, device="cuda")
        cfb.gemm_fp8_swiglu_bf16_rowamax(ctx, M, Fl, H, x8, H, False, None, dx, il_r, None, dil_r, h, hmax)
        hs.append(h); hmaxs.append(hmax)
    hmax_all = torch.maximum(hmaxs[0], hmaxs[1])          # the max-all-reduce
    assert torch.equal(hmax_all, full["hmax"])
    acc = torch.zeros((M, H), dtype=torch.float32, device="cuda")
    one = torch.ones(4, dtype=torch.float32, device="cuda")
    for r in range(W):
        h8 = torch.empty((M, Fl), dtype=torch.uint8, device="cuda")
        dh = torch.empty(M, dtype=torch.float32, device="cuda")
        cfb.fp8_quantize_rowwise_given_amax_e4m3(hs[r], h8, hmax_all, dh)
        assert torch.equal(h8, full["h8"][:, r * Fl:(r + 1) * Fl]) and torch.equal(dh, full["dh"])
        part = torch.empty((M, H), dtype=torch.float32, device="cuda")
        cfb.lt_gemm_fp8_nt(ctx, M, H, Fl, h8, Fl, False, one, wd8[:, r * Fl:(r + 1) * Fl].contiguous(), one, part, H,
                           a_row_descale=dh, b_col_descale=dd)
        acc += part
    ctx.poll_status()
    assert rel_fro(acc.cpu().numpy(), y_full.float().cpu().numpy()) < 4e-3
    # the reduce-scatter GEMM with row and column scales on one rank (its own slice only) gives the same fp32 sums
    acc2 = torch.zeros((M, H), dtype=torch.float32, device="cuda")
    for r in range(W):
        h8 = torch.empty((M, Fl), dtype=torch.uint8, device="cuda")
        dh = torch.empty(M, dtype=torch.float32, device="cuda")
        cfb.fp8_quantize_rowwise_given_amax_e4m3(hs[r], h8, hmax_all, dh)
        cfb.gemm_fp8_nt_reduce_scatter(ctx, M, H, Fl, h8, Fl, False, one, wd8[:, r * Fl:(r + 1) * Fl].contiguous(), one,
                                       [acc2.data_ptr()], a_row_descale=dh, b_col_descale=dd)
    ctx.poll_status()
    assert rel_fro(acc2.cpu().numpy(), acc.cpu().numpy()) < 1e-6


def test_fused_rowwise_mlp_full_size_sampled(cfb, ctx, oracle):
    """M=16384, hidden 4096, ffn 14336: fused composite against sampled oracle rows and against the unfused one."""
    M, H, F = 16384, 4096, 14336
    x = randn_bf16((M, H), seed=1)
    wgu8, dgu = _rowquant(cfb, randn_bf16((2 * F, H), std=0.02, seed=2))
    wd8, dd = _rowquant(cfb, randn_bf16((H, F), std=0.02, seed=3))
    il, dil = _interleaved(cfb, wgu8, dgu)
    y = torch.empty((M, H), dtype=torch.bfloat16, device="cuda")
    cfb.swiglu_mlp_fp8_rowwise_fused(ctx, x, il, dil, wd8, dd, y)
    ctx.poll_status()
    rows = [0, 127, 128, 255, 256, 8191, 16383]
    want = _mlp_oracle(oracle, bf16_to_u16(x[rows]), wgu8.cpu().numpy(), dgu.cpu().numpy(), wd8.cpu().numpy(), dd.cpu().numpy())
    assert rel_fro(y[rows].float().cpu().numpy(), oracle.bf16_to_f32(want)) < TOL
    y0 = torch.empty((1024, H), dtype=torch.bfloat16, device="cuda")
    cfb.swiglu_mlp_fp8_rowwise(ctx, x[2048:3072], wgu8, dgu, wd8, dd, y0)
    assert torch.equal(y0.view(torch.int16), y[2048:3072].view(torch.int16))


@pytest.mark.parametrize("rows,cols", [(5, 100), (64, 4096), (33, 1000), (7, 16), (3, 1)])
def test_rowwise_quantise_with_a_given_amax_equals_the_two_pass_kernel(cfb, oracle, rows, cols):
    """Given each row's own amax, the one-pass quantiser writes the codes and descales of cf_fp8_quantize_rowwise_e4m3
    (vector path for 16-byte multiples, element path otherwise); a larger amax (as after a max over shards) scales down."""
    x = randn_bf16((rows, cols), seed=rows + cols, outlier_frac=0.01)
    x[0] = 0
    want8 = torch.empty((rows, cols), dtype=torch.uint8, device="cuda")
    want_d = torch.empty(rows, dtype=torch.float32, device="cuda")
    want_s = torch.empty(rows, dtype=torch.float32, device="cuda")
    cfb.fp8_quantize_rowwise_e4m3(x, want8, want_d, row_scale=want_s)
    amax = x.float().abs().amax(dim=1).contiguous()
    got8 = torch.full((rows, cols), 0xAB, dtype=torch.uint8, device="cuda")
    got_d = torch.empty(rows, dtype=torch.float32, device="cuda")
    got_s = torch.empty(rows, dtype=torch.float32, device="cuda")
    cfb.fp8_quantize_rowwise_given_amax_e4m3(x, got8, amax, got_d, row_scale=got_s)
    assert torch.equal(got8, want8) and torch.equal(got_d, want_d) and torch.equal(got_s, want_s)
    w, s_o, d_o = oracle.quantize_rowwise_e4m3(bf16_to_u16(x))
    assert np.array_equal(got8.cpu().numpy(), w) and np.array_equal(got_d.cpu().numpy(), d_o)
    big = (amax * 2 + 1).contiguous()
    cfb.fp8_quantize_rowwise_given_amax_e4m3(x, got8, big, got_d)
    ref = oracle.bf16_to_f32(bf16_to_u16(x)) * (np.float32(448.0) / big.cpu().numpy())[:, None]
    dec = oracle.decode(got8.cpu().numpy())
    assert np.all(np.abs(dec - ref) <= np.maximum(np.abs(ref) * 2.0 ** -4, 2.0 ** -9) + 1e-6)


def test_swiglu_bf16_rowamax_epilogue_with_per_tensor_scales(cfb, ctx):
    """The same epilogue under per-tensor scales (the reference's granularity): h and the row amax equal the unfused
    GEMM + swiglu_forward, ragged row counts included."""
    for M, H, F in [(300, 128, 96), (1024, 256, 512)]:
        a8, da = _tensorquant(cfb, randn_bf16((M, H), seed=M))
        w8, dw = _tensorquant(cfb, randn_bf16((2 * F, H), std=0.05, seed=F))
        gu = torch.empty((M, 2 * F), dtype=torch.bfloat16, device="cuda")
        cfb.lt_gemm_fp8_nt(ctx, M, 2 * F, H, a8, H, False, da, w8, dw, gu, 2 * F)
        want = torch.empty((M, F), dtype=torch.bfloat16, device="cuda")
        cfb.swiglu_forward(gu[:, :F].contiguous(), gu[:, F:].contiguous(), want)
        il = cfb.fp8_interleave_gate_up(w8.view(1, 2 * F, H)).view(2 * F, H)
        h = torch.full((M + 1, F), 9.0, dtype=torch.bfloat16, device="cuda")
        hmax = torch.zeros(M + 1, dtype=torch.float32, device="cuda")
        cfb.gemm_fp8_swiglu_bf16_rowamax(ctx, M, F, H, a8, H, False, da, None, il, dw, None, h, hmax)
        ctx.poll_status()
        assert torch.equal(h[:M].view(torch.int16), want.view(torch.int16)) and (h[M] == 9.0).all()
        assert torch.equal(hmax[:M], want.float().abs().amax(dim=1)) and hmax[M].item() == 0.0


def _zipf_logits(rows, E, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    p = torch.arange(1, E + 1, device="cuda", dtype=torch.float32) ** -1.1
    return (torch.randn((rows, E), generator=g, device="cuda") + torch.log(p / p.sum())).contiguous()


def _moe_oracle_rows(oracle, cfb, moe, x, rw, wgu8, dgu, wd8, dd, sample_rows):
    """Recomputes mixed[r] for a few token rows on the host from the quantised tensors and slot snapshots."""
    F, H, E = moe.F, moe.H, moe.E
    dx = np.float32(moe.slot_x.scalars()["descale_snapshot"])
    sh = np.float32(moe.slot_h.scalars()["scale_snapshot"])
    dh = np.float32(moe.slot_h.scalars()["descale_snapshot"])
    x8 = moe.x8.cpu().numpy()
    rw_n = rw.cpu().numpy()
    out = np.zeros((len(sample_rows), H), dtype=np.uint16)
    for i, r in enumerate(sample_rows):
        for e in range(E):
            w = rw_n[r, e]
            if w <= 0:
                continue
            gu = oracle.gemm_fp8_nt(x8[r:r + 1], wgu8[e].cpu().numpy(), dx, dgu[0].item())
            h = oracle.swiglu_forward(np.ascontiguousarray(gu[:, :F]), np.ascontiguousarray(gu[:, F:]))
            h8 = oracle.quantize_bf16(h, sh)
            ye = oracle.gemm_fp8_nt(h8, wd8[e].cpu().numpy(), dh, dd[0].item())
            acc = oracle.bf16_to_f32(out[i:i + 1]) + w * oracle.bf16_to_f32(ye)
            out[i] = oracle.to_bf16(acc)[0]
    return out


@pytest.mark.parametrize("rows,H,F,E,k", [(300, 128, 256, 4, 2), (1024, 256, 512, 8, 2)])
def test_config4_moe_swiglu_reduced(cfb, ctx, oracle, rows, H, F, E, k):
    x = randn_bf16((rows, H), seed=1)
    rw = _zipf_logits(rows, E, 3)
    wgu8, dgu = _tensorquant(cfb, randn_bf16((E, 2 * F, H), std=0.05, seed=4))
    wd8, dd = _tensorquant(cfb, randn_bf16((E, H, F), std=0.05, seed=5))
    moe = cfb.MoeSwigluFp8(ctx, rows, H, F, E, k)
    mixed = torch.zeros((rows, H), dtype=torch.bfloat16, device="cuda")
    moe.forward(x, rw, wgu8, dgu, wd8, dd, mixed)
    ctx.poll_status()
    assert int(moe.counts.sum().item()) == rows * k
    sample = list(range(0, rows, max(1, rows // 40)))
    want = _moe_oracle_rows(oracle, cfb, moe, x, rw, wgu8, dgu, wd8, dd, sample)
    assert rel_fro(mixed[sample].float().cpu().numpy(), oracle.bf16_to_f32(want)) < TOL
    # second step: delayed scales now come from the first step's amax; result stays within tolerance of the oracle
    x2 = randn_bf16((rows, H), std=1.5, seed=7)
    rw2 = _zipf_logits(rows, E, 9)
    mixed2 = torch.zeros((rows, H), dtype=torch.bfloat16, device="cuda")
    moe.forward(x2, rw2, wgu8, dgu, wd8, dd, mixed2)
    ctx.poll_status()
    want2 = _moe_oracle_rows(oracle, cfb, moe, x2, rw2, wgu8, dgu, wd8, dd, sample)
    assert rel_fro(mixed2[sample].float().cpu().numpy(), oracle.bf16_to_f32(want2)) < TOL


def test_config4_full_size_sampled(cfb, ctx, oracle):
    """32768 tokens, hidden 4096, 8 experts of ffn 14336, top-2, Zipf(1.1)-skewed load: sampled tokens against the
    oracle, conservation of the dispatch (every token lands in exactly two experts) and combine linearity."""
    rows, H, F, E, k = 32768, 4096, 14336, 8, 2
    x = randn_bf16((rows, H), seed=1)
    rw = _zipf_logits(rows, E, 3)
    wgu8, dgu = _tensorquant(cfb, randn_bf16((E, 2 * F, H), std=0.02, seed=4))
    wd8, dd = _tensorquant(cfb, randn_bf16((E, H, F), std=0.02, seed=5))
    moe = cfb.MoeSwigluFp8(ctx, rows, H, F, E, k)
    mixed = torch.zeros((rows, H), dtype=torch.bfloat16, device="cuda")
    moe.forward(x, rw, wgu8, dgu, wd8, dd, mixed)
    ctx.poll_status()
    counts = moe.counts.cpu().numpy()
    assert counts.sum() == rows * k and counts[0] > counts[-1]          # skewed load, nothing dropped
    flat = torch.cat([moe.idx[e, :counts[e]] for e in range(E)]).cpu().numpy()
    assert np.array_equal(np.bincount(flat, minlength=rows), np.full(rows, k))
    sample = [0, 1, 777, 16384, 32767]
    want = _moe_oracle_rows(oracle, cfb, moe, x, rw, wgu8, dgu, wd8, dd, sample)
    assert rel_fro(mixed[sample].float().cpu().numpy(), oracle.bf16_to_f32(want)) < TOL
    del moe


def test_config5_large_shape_forward_and_dgrad(cfb, ctx, oracle):
    """M=32768, K=8192, N=28672 E4M3 forward and the E5M2-gradient x E4M3-weight dgrad of matching shape
    (dX[32768x8192] = dY[32768x28672] . W^T with W cached [8192x28672]); sampled rows against the oracle."""
    M, K, N = 32768, 8192, 28672
    a8, da = _tensorquant(cfb, randn_bf16((M, K), seed=1))
    w = randn_bf16((N, K), std=0.02, seed=2)
    fw = cfb.Fp8Weight(w, stored_out_major=True)        # fwd8 = [N,K], bwd8 = [K,N]
    cfb.refresh_fp8_weight(fw)
    c = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    cfb.lt_gemm_fp8_nt(ctx, M, N, K, a8, K, False, da, fw.fwd8, fw.descale, c, N)
    ctx.poll_status()
    rows = [0, 255, 256, 20000, 32767]
    want = oracle.gemm_fp8_nt(a8[rows].cpu().numpy(), fw.fwd8.cpu().numpy(), da[0].item(), fw.descale.item())
    assert rel_fro(c[rows].float().cpu().numpy(), oracle.bf16_to_f32(want)) < 5e-3
    del c
    dy = (randn_bf16((M, N), seed=3).float() * 1e-3).to(torch.bfloat16)
    dy8, ddy = _tensorquant(cfb, dy, e5m2=True)
    del dy
    dxo = torch.empty((M, K), dtype=torch.bfloat16, device="cuda")
    cfb.lt_gemm_fp8_nt(ctx, M, K, N, dy8, N, True, ddy, fw.bwd8, fw.descale, dxo, K)
    ctx.poll_status()
    want = oracle.gemm_fp8_nt(dy8[rows].cpu().numpy(), fw.bwd8.cpu().numpy(), ddy[0].item(), fw.descale.item(), a_is_e5m2=True)
    assert rel_fro(dxo[rows].float().cpu().numpy(), oracle.bf16_to_f32(want)) < 5e-3
    # N-sharding over 8 GPUs: each shard's forward slice equals the same columns of the full product
    c_sh = torch.empty((1024, N // 8), dtype=torch.bfloat16, device="cuda")
    cfb.lt_gemm_fp8_nt(ctx, 1024, N // 8, K, a8, K, False, da, fw.fwd8[3 * (N // 8):4 * (N // 8)], fw.descale, c_sh, N // 8)
    c_full = torch.empty((1024, N), dtype=torch.bfloat16, device="cuda")
    cfb.lt_gemm_fp8_nt(ctx, 1024, N, K, a8, K, False, da, fw.fwd8, fw.descale, c_full, N)
    assert torch.equal(c_sh, c_full[:, 3 * (N // 8):4 * (N // 8)])
    ctx.poll_status()


@pytest.mark.parametrize("rows,H,F,E", [(700, 256, 512, 4), (64, 128, 96, 2)])
def test_fused_swiglu_gemm_matches_the_unfused_sequence(cfb, ctx, oracle, rows, H, F, E):
    """One launch (gate/up GEMM + SwiGLU + delayed-scale re-quantise in the epilogue, interleaved weight rows) against
    GEMM -> bf16 [T,2F] -> swiglu + quant_act: same E4M3 bytes, same slot scalars, over three steps."""
    k = 2
    wgu8, dgu = _tensorquant(cfb, randn_bf16((E, 2 * F, H), std=0.05, seed=4))
    wd8, dd = _tensorquant(cfb, randn_bf16((E, H, F), std=0.05, seed=5))
    wgu8_il = cfb.fp8_interleave_gate_up(wgu8)
    il = wgu8_il.cpu().numpy(); src = wgu8.cpu().numpy()
    for f in (0, 31, 32, F - 1):
        assert np.array_equal(il[1, (f // 32) * 64 + f % 32], src[1, f]) and np.array_equal(il[1, (f // 32) * 64 + 32 + f % 32], src[1, F + f])
    plain = cfb.MoeSwigluFp8(ctx, rows, H, F, E, k)
    fused = cfb.MoeSwigluFp8(ctx, rows, H, F, E, k, fused_swiglu=True)
    for step in range(3):
        x = randn_bf16((rows, H), std=1.0 + step, seed=10 + step)
        rw_a, rw_b = _zipf_logits(rows, E, 20 + step), _zipf_logits(rows, E, 20 + step)
        m_a = torch.zeros((rows, H), dtype=torch.bfloat16, device="cuda")
        m_b = torch.zeros((rows, H), dtype=torch.bfloat16, device="cuda")
        plain.forward(x, rw_a, wgu8, dgu, wd8, dd, m_a)
        fused.forward(x, rw_b, wgu8_il, dgu, wd8, dd, m_b)
        ctx.poll_status()
        assert torch.equal(fused.h8, plain.h8), step
        assert torch.equal(m_a.view(torch.int16), m_b.view(torch.int16)), step
        a, b = plain.slot_h.scalars(), fused.slot_h.scalars()
        for key in ("amax", "scale", "descale", "scale_snapshot", "descale_snapshot", "cursor", "count"):
            assert a[key] == b[key], (step, key)
    # dense form (one segment, no counts) against the same rows through the unfused kernels
    M = 300
    x8, dx = _tensorquant(cfb, randn_bf16((M, H), seed=31))
    slot_a, slot_b = cfb.ActSlot(ctx, cfb.E4M3_MAX), cfb.ActSlot(ctx, cfb.E4M3_MAX)
    gu = torch.empty((M, 2 * F), dtype=torch.bfloat16, device="cuda")
    h_a = torch.empty((M, F), dtype=torch.uint8, device="cuda")
    h_b = torch.empty((M, F), dtype=torch.uint8, device="cuda")
    for step in range(2):
        cfb.lt_gemm_fp8_nt(ctx, M, 2 * F, H, x8, H, False, dx, wgu8[0], dgu, gu, 2 * F)
        cfb.fp8_swiglu_quant_act(ctx, slot_a, gu, gu.view(-1)[F:], 2 * F, M, F, h_a)
        cfb.gemm_fp8_swiglu_quant_act(ctx, slot_b, 1, 1, None, M, F, H, None, None, x8, H, False, dx, False, wgu8_il[0], dgu, h_b, F)
        ctx.poll_status()
        assert torch.equal(h_a, h_b), step


@pytest.mark.parametrize("fused_return", [True, False])
@pytest.mark.parametrize("rows,H,F,E", [(700, 256, 512, 4), (1100, 128, 96, 8)])
def test_device_planned_expert_parallel_layer_on_one_rank(cfb, ctx, rows, H, F, E, fused_return):
    """The expert-parallel layer whose plan, dispatch and return run on the device, with a single rank (every destination
    is the local GPU): same bits as the single-GPU layer over three steps, including the delayed scales."""
    k = 2
    wgu8, dgu = _tensorquant(cfb, randn_bf16((E, 2 * F, H), std=0.05, seed=4))
    wd8, dd = _tensorquant(cfb, randn_bf16((E, H, F), std=0.05, seed=5))
    wgu8_il = cfb.fp8_interleave_gate_up(wgu8)
    single = cfb.MoeSwigluFp8(ctx, rows, H, F, E, k, fused_swiglu=True)
    direct = cfb.parallel.EpMoeSwigluFp8Direct(cfb, ctx, rows, H, F, E, k, fused_return=fused_return)
    assert direct.V == E and direct.n_local == E
    for step in range(3):
        x = randn_bf16((rows, H), std=1.0 + step, seed=40 + step)
        rw_a, rw_b = _zipf_logits(rows, E, 50 + step), _zipf_logits(rows, E, 50 + step)
        m_a = torch.zeros((rows, H), dtype=torch.bfloat16, device="cuda")
        m_b = randn_bf16((rows, H), seed=60 + step)          # overwritten: accumulate=False
        single.forward(x, rw_a, wgu8_il, dgu, wd8, dd, m_a)
        direct.forward(x, rw_b, wgu8_il, dgu, wd8, dd, m_b, accumulate=False)
        ctx.poll_status()
        assert torch.equal(rw_a, rw_b)
        assert torch.equal(direct.counts_all.view(-1), single.counts) and torch.equal(direct.grp_counts, single.counts)
        assert torch.equal(direct.grp_offsets, single.offsets)
        total = int(single.counts.sum().item())
        assert torch.equal(direct.recv8[:total], single.xc[:total])
        assert torch.equal(direct.h8[:total], single.h8[:total]), step
        assert torch.equal(m_a.view(torch.int16), m_b.view(torch.int16)), step


def test_dense_ffn_fused_against_reference_sequence_and_oracle(cfb, ctx, oracle):
    """The reference's dense FP8 FFN with per-tensor delayed scaling: fused three-launch form against the unfused operator
    sequence (bit-identical) and against the host oracle (<= 1e-2), over two steps, at a reduced size; then the
    configuration-3 size (16384 x 4096 x 14336) against sampled oracle rows."""
    for (M, H, F, sample_rows) in [(384, 256, 512, None), (16384, 4096, 14336, [0, 255, 256, 9000, 16383])]:
        wgu8, dgu = _tensorquant(cfb, randn_bf16((1, 2 * F, H), std=0.02, seed=2))
        wd8, dd = _tensorquant(cfb, randn_bf16((H, F), std=0.02, seed=3))
        wgu_il = cfb.fp8_interleave_gate_up(wgu8)[0]
        ffn = cfb.FfnSwigluFp8(ctx, M, H, F)
        sx, sh = cfb.ActSlot(ctx, cfb.E4M3_MAX), cfb.ActSlot(ctx, cfb.E4M3_MAX)
        y = torch.empty((M, H), dtype=torch.bfloat16, device="cuda")
        for step in range(2):
            x = randn_bf16((M, H), std=1.0 + step, seed=40 + step)
            ffn.forward(x, wgu_il, dgu, wd8, dd, y)
            ctx.poll_status()
            if sample_rows is None:
                # the unfused operator sequence the reference runs
                x8 = torch.empty((M, H), dtype=torch.uint8, device="cuda")
                cfb.fp8_quant_act(ctx, sx, x, x8)
                gu = torch.empty((M, 2 * F), dtype=torch.bfloat16, device="cuda")
                cfb.lt_gemm_fp8_nt(ctx, M, 2 * F, H, x8, H, False, cfb.ops._DevPtr(sx.c.descale_snapshot), wgu8[0], dgu, gu, 2 * F)
                hb = torch.empty((M, F), dtype=torch.bfloat16, device="cuda")
                cfb.swiglu_forward(gu[:, :F].contiguous(), gu[:, F:].contiguous(), hb)
                h8 = torch.empty((M, F), dtype=torch.uint8, device="cuda")
                cfb.fp8_quant_act(ctx, sh, hb, h8)
                y2 = torch.empty((M, H), dtype=torch.bfloat16, device="cuda")
                cfb.lt_gemm_fp8_nt(ctx, M, H, F, h8, F, False, cfb.ops._DevPtr(sh.c.descale_snapshot), wd8, dd, y2, H)
                assert torch.equal(ffn.h8, h8) and torch.equal(y.view(torch.int16), y2.view(torch.int16)), step
            rows = list(range(0, M, max(1, M // 24))) if sample_rows is None else sample_rows
            dx = np.float32(ffn.slot_x.scalars()["descale_snapshot"])
            s_h = np.float32(ffn.slot_h.scalars()["scale_snapshot"]); d_h = np.float32(ffn.slot_h.scalars()["descale_snapshot"])
            gu_o = oracle.gemm_fp8_nt(ffn.x8[rows].cpu().numpy(), wgu8[0].cpu().numpy(), dx, dgu[0].item())
            h_o = oracle.swiglu_forward(np.ascontiguousarray(gu_o[:, :F]), np.ascontiguousarray(gu_o[:, F:]))
            y_o = oracle.gemm_fp8_nt(oracle.quantize_bf16(h_o, s_h), wd8.cpu().numpy(), d_h, dd[0].item())
            assert rel_fro(y[rows].float().cpu().numpy(), oracle.bf16_to_f32(y_o)) < TOL, (M, step)
        del ffn


def test_rowwise_quantize_random_shapes_and_alignments(cfb, oracle):
    """Forty seeded random (rows, cols, input offset, output offset, row pitch) cases of the per-token quantiser, from one
    column to 16384, against the oracle: codes, scales, descales, and an untouched guard band around the output."""
    import random
    rnd = random.Random(2024)
    for case in range(40):
        cols = rnd.choice([1, 2, 7, 8, 9, 15, 16, 17, 63, 64, 65, 255, 511, 513, 1000, 4095, 4096, 4097, 8191, 16384]) \
            if case % 2 == 0 else rnd.randint(1, 3000)
        rows = rnd.randint(1, 40)
        pad_in, pad_out = rnd.choice([0, 0, 1, 3, 8]), rnd.choice([0, 0, 1, 5, 16])
        ld_in, ld_out = cols + pad_in, cols + pad_out
        in_off, out_off = rnd.randint(0, 9), rnd.randint(0, 17)
        flat = randn_bf16((in_off + rows * ld_in + 16,), seed=1000 + case, outlier_frac=0.02)
        out_flat = torch.full((out_off + rows * ld_out + 64,), 0x5C, dtype=torch.uint8, device="cuda")
        sc = torch.empty(rows, dtype=torch.float32, device="cuda")
        de = torch.empty(rows, dtype=torch.float32, device="cuda")
        cfb.fp8_quantize_rowwise_e4m3(flat[in_off:], out_flat[out_off:], de, row_scale=sc, rows=rows, cols=cols, ld_x=ld_in,
                                      ld_out=ld_out)
        src = bf16_to_u16(flat)[in_off:in_off + rows * ld_in].reshape(rows, ld_in)[:, :cols]
        w, s_o, d_o = oracle.quantize_rowwise_e4m3(np.ascontiguousarray(src))
        got = out_flat.cpu().numpy()
        body = got[out_off:out_off + rows * ld_out].reshape(rows, ld_out)
        key = (case, rows, cols, ld_in, ld_out, in_off, out_off)
        assert np.array_equal(body[:, :cols], w), key
        assert (body[:, cols:] == 0x5C).all() and (got[:out_off] == 0x5C).all() and (got[out_off + rows * ld_out:] == 0x5C).all(), key
        assert np.array_equal(sc.cpu().numpy(), s_o) and np.array_equal(de.cpu().numpy(), d_o), key
