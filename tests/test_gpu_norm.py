"""RMSNorm fused with the FP8 quantiser: bit-exact against the reference's own kernels on the same GPU (rmsnorm_forward
followed by fp8_quantize_e4m3_record) and against the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import bf16_to_u16 as u16, f32_scalar, package, randn_bf16, ref_gpu_or_none  # noqa: E402


@pytest.fixture(scope="module")
def cfb():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return package()

SHAPES = [(64, 4096), (257, 512), (33, 96), (19, 1000), (8, 16384), (40, 4104), (5, 8200), (700, 2048), (3000, 1024),
          (21, 14336), (9, 8192)]


def _inputs(rows, H, seed):
    x = randn_bf16((rows, H), seed=seed) * 3
    x.view(-1)[::97] *= 20
    g = (1 + 0.1 * torch.randn(H, device="cuda", generator=torch.Generator(device="cuda").manual_seed(seed + 1))).to(torch.bfloat16)
    return x.contiguous(), g.contiguous()


@pytest.mark.parametrize("rows,H", SHAPES)
def test_rmsnorm_forward_matches_reference_kernel_and_oracle(cfb, oracle, rows, H):
    x, g = _inputs(rows, H, 5)
    out = torch.empty_like(x)
    rms = torch.empty(rows, dtype=torch.float32, device="cuda")
    cfb.rmsnorm_forward(x, g, out, rms, rows, H, 1e-6)
    want, want_rms = oracle.rmsnorm_forward(u16(x), u16(g), 1e-6)
    assert np.array_equal(rms.cpu().numpy(), want_rms)
    assert np.array_equal(u16(out), want)
    ref = ref_gpu_or_none()
    if ref is not None:
        r_out = torch.empty_like(x)
        r_rms = torch.empty_like(rms)
        ref.call("ref_rmsnorm_forward", x, g, r_out, r_rms, rows, H, 1e-6, None)
        assert torch.equal(r_rms, rms)
        assert torch.equal(r_out.view(torch.int16), out.view(torch.int16))


@pytest.mark.parametrize("rows,H", SHAPES)
@pytest.mark.parametrize("keep_bf16", [True, False])
def test_rmsnorm_record_quantise_is_the_two_kernel_sequence(cfb, rows, H, keep_bf16):
    x, g = _inputs(rows, H, 9)
    normed = torch.empty_like(x)
    rms = torch.empty(rows, dtype=torch.float32, device="cuda")
    cfb.rmsnorm_forward(x, g, normed, rms, rows, H, 1e-6)
    scale = f32_scalar(37.5)
    want8 = torch.empty((rows, H), dtype=torch.uint8, device="cuda")
    want_amax = f32_scalar(0.0)
    cfb.fp8_quantize_e4m3_record(normed, want8, scale, want_amax)
    got8 = torch.zeros_like(want8)
    got_amax = f32_scalar(0.0)
    got_n = torch.zeros_like(x) if keep_bf16 else None
    got_rms = torch.zeros_like(rms)
    cfb.rmsnorm_quantize_e4m3_record(x, g, got_n, got_rms, got8, scale, got_amax, rows, H, 1e-6)
    assert torch.equal(got8, want8)
    assert torch.equal(got_amax, want_amax)
    assert torch.equal(got_rms, rms)
    if keep_bf16:
        assert torch.equal(got_n.view(torch.int16), normed.view(torch.int16))


@pytest.mark.parametrize("rows,H", [(64, 4096), (33, 96), (19, 1000), (5000, 512), (21, 14336)])
def test_rmsnorm_rowwise_quantise_is_the_two_kernel_sequence(cfb, rows, H):
    x, g = _inputs(rows, H, 13)
    normed = torch.empty_like(x)
    cfb.rmsnorm_forward(x, g, normed, None, rows, H, 1e-6)
    want8 = torch.empty((rows, H), dtype=torch.uint8, device="cuda")
    want_s = torch.empty(rows, dtype=torch.float32, device="cuda")
    want_d = torch.empty_like(want_s)
    cfb.fp8_quantize_rowwise_e4m3(normed, want8, want_d, row_scale=want_s)
    got8 = torch.zeros_like(want8)
    got_s, got_d = torch.zeros_like(want_s), torch.zeros_like(want_d)
    cfb.rmsnorm_quantize_rowwise_e4m3(x, g, None, None, got8, got_d, rows, H, 1e-6, row_scale=got_s)
    assert torch.equal(got8, want8) and torch.equal(got_s, want_s) and torch.equal(got_d, want_d)


@pytest.mark.parametrize("ticket", [True, False])
def test_rmsnorm_quant_act_follows_the_slot_state_machine(cfb, ticket):
    """Same slot history as rmsnorm_forward + fp8_quant_act over five calls with changing inputs."""
    rows, H = 96, 2048
    ctx = cfb.Fp8Ctx(0)
    slot_a = cfb.ActSlot(ctx, cfb.E4M3_MAX)
    slot_b = cfb.ActSlot(ctx, cfb.E4M3_MAX)
    if not ticket:                      # a caller-built slot without the ticket word: the ring update is its own launch
        slot_a.c.ticket = None
        slot_b.c.ticket = None
    for step in range(5):
        x, g = _inputs(rows, H, 20 + step)
        x = (x * (1 + step)).contiguous()
        g = (g * (0.5 + step)).contiguous()
        normed = torch.empty_like(x)
        cfb.rmsnorm_forward(x, g, normed, None, rows, H, 1e-6)
        want8 = torch.empty((rows, H), dtype=torch.uint8, device="cuda")
        cfb.fp8_quant_act(ctx, slot_a, normed, want8)
        got8 = torch.zeros_like(want8)
        cfb.fp8_rmsnorm_quant_act(ctx, slot_b, x, g, None, None, rows, H, got8)
        assert torch.equal(got8, want8), step
        sa, sb = slot_a.scalars(), slot_b.scalars()
        for k in ("scale", "descale", "scale_snapshot", "descale_snapshot", "history", "cursor", "count"):
            if k in sa:
                assert np.array_equal(np.asarray(sa[k]), np.asarray(sb[k])), (step, k)
    ctx.poll_status()


def test_rmsnorm_refuses_what_the_reference_cannot_reduce(cfb):
    x, g = _inputs(4, 4096, 1)
    out = torch.empty((4, 40), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(cfb.CanopyError):
        cfb.rmsnorm_forward(x, g, out, None, 4, 40, 1e-6)       # 40 threads: a partial warp
    with pytest.raises(cfb.CanopyError):
        cfb.rmsnorm_forward(x, g, out, None, 1, 16400, 1e-6)    # beyond the column limit


CLIP_SHAPES = [(64, 4096), (300, 512), (40, 1024), (33, 2048), (9, 8192)]


@pytest.mark.parametrize("rows,H", CLIP_SHAPES)
def test_rmsnorm_with_row_clip_matches_the_three_pass_sequence(cfb, oracle, rows, H):
    """Norm + act_row_clip + record-quantise in one pass against rmsnorm_forward, the host restatement of the clip, and the
    record-quantise kernel: bf16 rows, rms, E4M3 bytes and amax bit for bit. The ceiling sits inside the range of row
    norms, so some rows are rescaled and some are left alone; a few rows are made large on purpose."""
    x, g = _inputs(rows, H, 17)
    g = (g * 4).contiguous()
    x[::7] *= 30
    normed = torch.empty_like(x)
    rms = torch.empty(rows, dtype=torch.float32, device="cuda")
    cfb.rmsnorm_forward(x, g, normed, rms, rows, H, 1e-6)
    n_host = u16(normed).copy()
    norms = np.sqrt((oracle.bf16_to_f32(n_host).astype(np.float64) ** 2).sum(axis=1))
    ceiling = float(np.float32(np.median(norms) * 1.0005))
    oracle.act_row_clip(n_host, ceiling)
    clipped = np.any(n_host != u16(normed), axis=1)
    assert clipped.any() and not clipped.all()
    got = torch.zeros_like(x)
    got_rms = torch.zeros_like(rms)
    cfb.rmsnorm_clip_forward(x, g, got, got_rms, rows, H, ceiling)
    assert torch.equal(got_rms, rms)
    assert np.array_equal(u16(got), n_host)
    # ... followed by the quantiser
    from gpu_util import u16_to_bf16
    want_n = u16_to_bf16(n_host)
    scale = f32_scalar(11.0)
    want8 = torch.empty((rows, H), dtype=torch.uint8, device="cuda")
    want_amax = f32_scalar(0.0)
    cfb.fp8_quantize_e4m3_record(want_n, want8, scale, want_amax)
    got8 = torch.zeros_like(want8)
    got_amax = f32_scalar(0.0)
    cfb.rmsnorm_clip_quantize_e4m3_record(x, g, None, None, got8, scale, got_amax, rows, H, ceiling)
    assert torch.equal(got8, want8) and torch.equal(got_amax, want_amax)
    # a ceiling nothing reaches (the reference's default of 1000 on normalised rows) changes nothing
    same = torch.zeros_like(x)
    cfb.rmsnorm_clip_forward(x, g, same, None, rows, H, 1.0e9)
    assert torch.equal(same.view(torch.int16), normed.view(torch.int16))


def test_rmsnorm_clip_quant_act_and_the_warp_form_without_clip(cfb):
    """The slot state machine around the clipped pass equals norm -> clip -> fp8_quant_act; with a ceiling of zero the
    entry point is the plain fused pass."""
    rows, H = 96, 2048
    ctx = cfb.Fp8Ctx(0)
    slot_a, slot_b, slot_c = cfb.ActSlot(ctx, cfb.E4M3_MAX), cfb.ActSlot(ctx, cfb.E4M3_MAX), cfb.ActSlot(ctx, cfb.E4M3_MAX)
    for step in range(4):
        x, g = _inputs(rows, H, 70 + step)
        g = (g * (2 + step)).contiguous()
        ceiling = 60.0 * (2 + step)
        clipped = torch.empty_like(x)
        cfb.rmsnorm_clip_forward(x, g, clipped, None, rows, H, ceiling)
        want8 = torch.empty((rows, H), dtype=torch.uint8, device="cuda")
        cfb.fp8_quant_act(ctx, slot_a, clipped, want8)
        got8 = torch.zeros_like(want8)
        cfb.fp8_rmsnorm_clip_quant_act(ctx, slot_b, x, g, None, None, rows, H, got8, ceiling)
        assert torch.equal(got8, want8), step
        sa, sb = slot_a.scalars(), slot_b.scalars()
        for k in ("scale", "descale", "scale_snapshot", "descale_snapshot", "cursor", "count"):
            assert sa[k] == sb[k], (step, k)
        plain8 = torch.zeros_like(want8)
        cfb.fp8_rmsnorm_clip_quant_act(ctx, slot_c, x, g, None, None, rows, H, plain8, 0.0)
    ctx.poll_status()
    with pytest.raises(cfb.CanopyError):
        # a shape the one-pass kernel does not take needs the bf16 row buffer for the three-pass sequence
        cfb.rmsnorm_clip_quantize_e4m3_record(x, g, None, None, plain8, f32_scalar(1.0), f32_scalar(0.0), rows, 96, 10.0)


@pytest.mark.parametrize("rows,H", [(16, 4096), (12, 1024), (10, 768), (7, 96)])
def test_row_clip_on_rows_with_nan_and_inf_follows_the_reference_predicate(cfb, oracle, rows, H):
    """The reference leaves a row alone only when `norm <= ceiling` holds (src/trainer.cu:3952): a row whose squared norm
    is NaN fails that test and is rescaled by ceiling / NaN, i.e. becomes NaN everywhere; a row with an infinite norm is
    multiplied by ceiling / inf = 0 (inf * 0 = NaN for the infinite elements themselves). Host-made inputs, both the
    one-pass kernel (H % 512 == 0) and the three-pass form (other H) against the host restatement of the clip."""
    x, g2 = _inputs(rows, H, 23)
    ceiling = 50.0
    # the fused entry point sees x and gamma only, so the specials are planted in x: a NaN element makes rms NaN and the
    # whole normalised row NaN; an infinite element makes rms infinite, the finite elements 0 and itself inf * 0 = NaN
    x[1, 3] = float("nan")
    x[2, 5] = float("inf")
    normed = torch.empty_like(x)
    cfb.rmsnorm_forward(x, g2, normed, None, rows, H, 1e-6)
    want = u16(normed).copy()
    oracle.act_row_clip(want, ceiling)
    got = torch.zeros_like(x)
    cfb.rmsnorm_clip_forward(x, g2, got, None, rows, H, ceiling)
    assert np.array_equal(u16(got), want)
    # rows 1 and 2 are NaN after the norm (NaN and inf / inf); the clip must not have "skipped" them differently
    f = oracle.bf16_to_f32(u16(got))
    assert np.isnan(f[1]).all() and np.isnan(f[2]).any()
    # the quantiser behind it sees the same rows
    from gpu_util import u16_to_bf16
    scale = f32_scalar(3.0)
    want8 = torch.empty((rows, H), dtype=torch.uint8, device="cuda")
    want_amax = f32_scalar(0.0)
    cfb.fp8_quantize_e4m3_record(u16_to_bf16(want), want8, scale, want_amax)
    got8 = torch.zeros_like(want8)
    got_amax = f32_scalar(0.0)
    keep = torch.zeros_like(x)
    cfb.rmsnorm_clip_quantize_e4m3_record(x, g2, keep, None, got8, scale, got_amax, rows, H, ceiling)
    assert torch.equal(got8, want8) and torch.equal(got_amax, want_amax)
    assert np.array_equal(u16(keep), want)


@pytest.mark.parametrize("rows,H", [(40, 768), (9, 1000), (5, 12288), (21, 96)])
def test_row_clip_three_pass_form_for_other_shapes(cfb, oracle, rows, H):
    """Hidden sizes the one-pass kernel does not take (not a multiple of 512, or above 8192) run norm, clip and quantise
    as three launches with the reference's reductions: bit-identical to rmsnorm_forward + the host clip + the quantiser."""
    x, g = _inputs(rows, H, 29)
    g = (g * 4).contiguous()
    x[::3] *= 30
    normed = torch.empty_like(x)
    rms = torch.empty(rows, dtype=torch.float32, device="cuda")
    cfb.rmsnorm_forward(x, g, normed, rms, rows, H, 1e-6)
    n_host = u16(normed).copy()
    norms = np.sqrt((oracle.bf16_to_f32(n_host).astype(np.float64) ** 2).sum(axis=1))
    ceiling = float(np.float32(np.median(norms) * 1.0005))
    oracle.act_row_clip(n_host, ceiling)
    assert np.any(n_host != u16(normed))
    got = torch.zeros_like(x)
    got_rms = torch.zeros_like(rms)
    cfb.rmsnorm_clip_forward(x, g, got, got_rms, rows, H, ceiling)
    assert torch.equal(got_rms, rms) and np.array_equal(u16(got), n_host)
    from gpu_util import u16_to_bf16
    scale = f32_scalar(7.0)
    want8 = torch.empty((rows, H), dtype=torch.uint8, device="cuda")
    want_amax = f32_scalar(0.0)
    cfb.fp8_quantize_e4m3_record(u16_to_bf16(n_host), want8, scale, want_amax)
    got8 = torch.zeros_like(want8)
    got_amax = f32_scalar(0.0)
    keep = torch.zeros_like(x)
    cfb.rmsnorm_clip_quantize_e4m3_record(x, g, keep, None, got8, scale, got_amax, rows, H, ceiling)
    assert torch.equal(got8, want8) and torch.equal(got_amax, want_amax)
