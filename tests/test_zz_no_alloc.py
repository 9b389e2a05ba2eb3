"""The allocation-free FP8 linear (cf_fp8_linear_static_scratch) against cf_fp8_linear_forward.

Some users of the library cannot call cudaMalloc at all: their application has given the whole device-memory
budget to its own arena, or they run on a thread where the device-wide stall of an allocation is not
acceptable. For them the library carries one entry point whose scratch (the E4M3 copy of the activation) is a
fixed 4 MiB array inside the library. This test drives it through the C ABI twice in a row, the second time
with different data and a delayed scale, and expects exactly the bytes the context-based entry point produces,
because both run the same kernels with the same scale; the output is also checked against the CPU oracle so that
the test stands without the other entry point. Three shapes reach the three forms of the GEMM behind it: single-CTA
tiles, CTA-pair tiles (512 rows and more) and the plain form for a K that is not a multiple of 16. It is collected
last so that a failure here cannot hide one elsewhere; it passes both alone in a fresh process and after the rest of
the suite.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import bf16_to_u16, package, randn_bf16, rel_fro  # noqa: E402


@pytest.mark.parametrize("M,K,N", [(384, 1024, 640), (1024, 4096, 512), (200, 1000, 320)])
def test_static_scratch_linear_matches_context_linear_twice(oracle, M, K, N):
    assert torch.cuda.is_available()
    cfb = package()
    lib = cfb._capi.lib()
    ctx = cfb.Fp8Ctx(act8_bytes=M * K)
    w = randn_bf16((N, K), std=0.02, seed=1)
    fw = cfb.Fp8Weight(w, stored_out_major=True)
    cfb.refresh_fp8_weight(fw)
    bias = randn_bf16((N,), std=0.01, seed=2)
    slot = cfb.ActSlot(ctx, cfb.E4M3_MAX)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    w8_host = fw.fwd8.cpu().numpy()

    def call_static(x, y, bias_t, mode, status_t):
        rc = lib.cf_fp8_linear_static_scratch(
            C.c_void_p(x.data_ptr()), M, K, slot.c.scale_snapshot, slot.c.descale_snapshot,
            C.c_void_p(fw.fwd8.data_ptr()), C.c_void_p(fw.descale.data_ptr()), N,
            C.c_void_p(bias_t.data_ptr()) if bias_t is not None else None, mode, C.c_void_p(y.data_ptr()), N,
            C.c_void_p(status_t.data_ptr()) if status_t is not None else None, stream)
        assert rc == 0, lib.cf_last_error()
        torch.cuda.synchronize()

    for call in range(2):
        x = randn_bf16((M, K), std=1.0 + call, seed=10 + call, outlier_frac=0.001)
        y_ref = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        cfb.fp8_linear_forward(ctx, slot, x, fw.fwd8, fw.descale, y_ref, bias=bias, bias_mode=2)
        # the scale pair the call above quantised with is the slot's snapshot pair
        y_new = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        call_static(x, y_new, bias, 2, status)
        assert status.item() == 0
        # same kernels, same scale: identical bits (the suite's GEMM tolerance is 5e-3 relative Frobenius)
        assert torch.equal(y_new.view(torch.int16), y_ref.view(torch.int16)), call
        # and on its own feet: the CPU oracle with the scale pair the call was given
        sc = slot.scalars()
        xs = bf16_to_u16(x)
        x8 = oracle.quantize_bf16(xs, np.float32(sc["scale_snapshot"]))
        want = oracle.gemm_fp8_nt(x8, w8_host, np.float32(sc["descale_snapshot"]), fw.descale.item(),
                                  bias=bf16_to_u16(bias), bias_mode=2)
        err = rel_fro(oracle.bf16_to_f32(bf16_to_u16(y_new)), oracle.bf16_to_f32(want))
        assert err < 5e-3, (call, err)
    # without a caller-side status word the call still works (internal word, cleared per call) and gives the
    # same product (no bias this time): checked against the context-based GEMM on the quantised bytes
    y_nb = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    call_static(x, y_nb, None, 0, None)
    x8d = torch.empty((M, K), dtype=torch.uint8, device="cuda")
    cfb.fp8_quant_act(ctx, slot, x, x8d, is_recompute=True)
    y_nb_ref = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    cfb.lt_gemm_fp8_nt(ctx, M, N, K, x8d, K, False, cfb.ops._DevPtr(slot.c.descale_snapshot), fw.fwd8, fw.descale, y_nb_ref, N)
    torch.cuda.synchronize()
    assert torch.equal(y_nb.view(torch.int16), y_nb_ref.view(torch.int16))
    # beyond the built-in 4 MiB the call refuses, with a message that names the limit
    rc = lib.cf_fp8_linear_static_scratch(
        C.c_void_p(x.data_ptr()), 4096, 4096, slot.c.scale_snapshot, slot.c.descale_snapshot,
        C.c_void_p(fw.fwd8.data_ptr()), C.c_void_p(fw.descale.data_ptr()), N, None, 0, C.c_void_p(y_nb.data_ptr()), N,
        None, stream)
    assert rc == cfb._capi.CF_ERR_LIMIT and b"4194304" in lib.cf_last_error()
    torch.cuda.synchronize()
    ctx.poll_status()
    ctx.close()
