"""ctypes bindings for the CPU oracle (oracle/libcf_oracle.so) and, when they
were built, the reference-compiled comparators under oracle/_ref/.

Test infrastructure only: nothing in the product package imports this file.
"""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")

c_f = C.c_float
c_i = C.c_int
c_i64 = C.c_int64
c_p = C.c_void_p


def _ptr(a):
    if a is None:
        return None
    assert isinstance(a, np.ndarray) and a.flags["C_CONTIGUOUS"], "need contiguous ndarray"
    return a.ctypes.data_as(c_p)


def build_oracle():
    so = os.path.join(ORACLE_DIR, "libcf_oracle.so")
    src = os.path.join(ORACLE_DIR, "cf_oracle.cpp")
    if (not os.path.exists(so)) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", ORACLE_DIR, "libcf_oracle.so"], stdout=subprocess.DEVNULL)
    return so


class Oracle:
    """Thin numpy front-end over the extern "C" oracle entry points."""

    def __init__(self):
        self.lib = C.CDLL(build_oracle())
        L = self.lib
        L.orc_e4m3_encode.restype = C.c_uint8; L.orc_e4m3_encode.argtypes = [c_f]
        L.orc_e5m2_encode.restype = C.c_uint8; L.orc_e5m2_encode.argtypes = [c_f]
        L.orc_e4m3_pack.restype = C.c_uint8; L.orc_e4m3_pack.argtypes = [c_f, C.POINTER(c_i)]
        L.orc_e4m3_decode.restype = c_f; L.orc_e4m3_decode.argtypes = [C.c_uint8]
        L.orc_e5m2_decode.restype = c_f; L.orc_e5m2_decode.argtypes = [C.c_uint8]
        L.orc_amax_bf16.restype = c_f; L.orc_amax_bf16.argtypes = [c_p, c_i64]
        L.orc_amax_f32.restype = c_f; L.orc_amax_f32.argtypes = [c_p, c_i64]
        L.orc_hw_threads.restype = c_i

    # -- conversions ----------------------------------------------------------
    def to_bf16(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty(x.shape, dtype=np.uint16)
        self.lib.orc_f32_to_bf16_array(_ptr(x), _ptr(out), c_i64(x.size))
        return out

    @staticmethod
    def bf16_to_f32(h):
        return (h.astype(np.uint32) << 16).view(np.float32)

    def decode(self, codes, is_e5m2=False):
        codes = np.ascontiguousarray(codes, dtype=np.uint8)
        out = np.empty(codes.shape, dtype=np.float32)
        self.lib.orc_decode_fp8(_ptr(codes), _ptr(out), c_i64(codes.size), c_i(int(is_e5m2)))
        return out

    # -- scalars --------------------------------------------------------------
    def amax_bf16(self, x):
        return float(self.lib.orc_amax_bf16(_ptr(x), c_i64(x.size)))

    def amax_f32(self, x):
        return float(self.lib.orc_amax_f32(_ptr(x), c_i64(x.size)))

    def scale_from_amax(self, amax, fp8_max):
        s, d = c_f(), c_f()
        self.lib.orc_scale_from_amax(c_f(amax), c_f(fp8_max), C.byref(s), C.byref(d))
        return np.float32(s.value), np.float32(d.value)

    def update_delayed_scale(self, amax, fp8_max, history, history_len, cursor, count, scale=0.0, descale=0.0):
        s, d = c_f(scale), c_f(descale)
        cur, cnt = c_i(cursor), c_i(count)
        self.lib.orc_update_delayed_scale(c_f(amax), c_f(fp8_max), C.byref(s), C.byref(d), _ptr(history),
                                          c_i(history_len), C.byref(cur), C.byref(cnt))
        return np.float32(s.value), np.float32(d.value), cur.value, cnt.value

    def calib_minmax_update(self, amax, cmin, cmax):
        a, b = c_f(cmin), c_f(cmax)
        self.lib.orc_calib_minmax_update(c_f(amax), C.byref(a), C.byref(b))
        return np.float32(a.value), np.float32(b.value)

    def clip_probe(self, amax, scale, fp8_max, stats):
        self.lib.orc_clip_probe(c_f(amax), c_f(scale), c_f(fp8_max), _ptr(stats))

    def elem_clip_count(self, x, scale, fp8_max, out):
        self.lib.orc_elem_clip_count(_ptr(x), c_f(scale), c_f(fp8_max), c_i64(x.size), _ptr(out))

    # -- tensors --------------------------------------------------------------
    def quantize_bf16(self, x, scale, is_e5m2=False):
        out = np.empty(x.shape, dtype=np.uint8)
        self.lib.orc_quantize_bf16(_ptr(x), _ptr(out), c_f(scale), c_i64(x.size), c_i(int(is_e5m2)))
        return out

    def quantize_f32(self, x, scale, is_e5m2=False):
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty(x.shape, dtype=np.uint8)
        self.lib.orc_quantize_f32(_ptr(x), _ptr(out), c_f(scale), c_i64(x.size), c_i(int(is_e5m2)))
        return out

    def quantize_record_bf16(self, x, scale, amax_in=0.0, is_e5m2=False):
        out = np.empty(x.shape, dtype=np.uint8)
        am = c_f(amax_in)
        self.lib.orc_quantize_record_bf16(_ptr(x), _ptr(out), c_f(scale), C.byref(am), c_i64(x.size),
                                          c_i(int(is_e5m2)))
        return out, np.float32(am.value)

    def quantize_transpose_e4m3(self, w, scale):
        K, N = w.shape
        out = np.empty((N, K), dtype=np.uint8)
        self.lib.orc_quantize_transpose_e4m3(_ptr(w), _ptr(out), c_f(scale), c_i(K), c_i(N))
        return out

    def quant_and_transpose_e4m3(self, x, scale):
        K, N = x.shape
        a = np.empty((K, N), dtype=np.uint8)
        s = np.empty((N, K), dtype=np.uint8)
        self.lib.orc_quant_and_transpose_e4m3(_ptr(x), _ptr(a), _ptr(s), c_f(scale), c_i(K), c_i(N))
        return a, s

    def transpose_u8(self, x):
        r, c = x.shape
        out = np.empty((c, r), dtype=np.uint8)
        self.lib.orc_transpose_u8(_ptr(x), _ptr(out), c_i(r), c_i(c))
        return out

    def pack_raw_e4m3(self, x, want_dequant=False):
        out = np.empty(x.shape, dtype=np.uint8)
        dq = np.empty(x.shape, dtype=np.uint16) if want_dequant else None
        am, sc, de = c_f(), c_f(), c_f()
        bi, bp = c_i(), c_i()
        self.lib.orc_pack_raw_e4m3(_ptr(x), _ptr(out), _ptr(dq), C.byref(am), C.byref(sc), C.byref(de),
                                   C.byref(bi), C.byref(bp), c_i64(x.size))
        return out, dq, np.float32(am.value), np.float32(sc.value), np.float32(de.value), bi.value, bp.value

    def unpack_raw_e4m3_bf16(self, codes, descale):
        out = np.empty(codes.shape, dtype=np.uint16)
        self.lib.orc_unpack_raw_e4m3_bf16(_ptr(codes), c_f(descale), _ptr(out), c_i64(codes.size))
        return out

    def gemm_fp8_nt(self, A, B, a_descale, b_descale, *, lda=None, a_is_e5m2=False, b_is_e5m2=False,
                    out_kind=0, C_init=None, ldc=None, bias=None, bias_mode=0, M=None, threads=0):
        """A: uint8 [M, lda>=K] (only the first K columns of each row are read), B: uint8 [N,K]."""
        N, K = B.shape
        M = A.shape[0] if M is None else M
        lda = A.shape[1] if lda is None else lda
        ldc = N if ldc is None else ldc
        a_ds = np.atleast_1d(np.asarray(a_descale, dtype=np.float32))
        b_ds = np.atleast_1d(np.asarray(b_descale, dtype=np.float32))
        if C_init is not None:
            out = np.ascontiguousarray(C_init).copy()
        else:
            out = np.zeros((M, ldc), dtype=np.uint16 if out_kind in (0, 3) else np.float32)
        self.lib.orc_gemm_fp8_nt(c_i(M), c_i(N), c_i(K), _ptr(A), c_i64(lda), c_i(int(a_is_e5m2)), _ptr(a_ds),
                                 c_i(int(a_ds.size > 1)), _ptr(B), c_i(int(b_is_e5m2)), _ptr(b_ds),
                                 c_i(int(b_ds.size > 1)), _ptr(out), c_i64(ldc), c_i(out_kind), _ptr(bias),
                                 c_i(bias_mode), c_i(threads))
        return out

    def bias_add_strided_bf16(self, inout, bias, rows, cols, row_stride, base):
        self.lib.orc_bias_add_strided_bf16(_ptr(inout), _ptr(bias), c_i(rows), c_i(cols), c_i(row_stride), c_i(base))

    def rmsnorm_forward(self, x, scale, eps):
        """x uint16 [rows, H], scale uint16 [H] -> (out uint16 [rows, H], rms float32 [rows])."""
        rows, H = x.shape
        out = np.empty((rows, H), dtype=np.uint16)
        rms = np.empty(rows, dtype=np.float32)
        self.lib.orc_rmsnorm_forward(_ptr(x), _ptr(scale), _ptr(out), _ptr(rms), c_i64(rows), c_i(H), c_f(eps))
        return out, rms

    def act_row_clip(self, x, ceiling):
        """In place on x (uint16 [rows, cols]); returns the squared row norms the reference's reduction computes."""
        rows, cols = x.shape
        nsq = np.zeros(rows, dtype=np.float32)
        self.lib.orc_act_row_clip(_ptr(x), c_i64(rows), c_i(cols), c_f(ceiling), _ptr(nsq))
        return nsq

    def swiglu_forward(self, gate, up):
        out = np.empty(gate.shape, dtype=np.uint16)
        self.lib.orc_swiglu_forward(_ptr(gate), _ptr(up), _ptr(out), c_i64(gate.size))
        return out

    def lion_step(self, w, m, grad, lr, beta1, beta2, wd, amax=0.0, seed=0):
        """In place on w (uint16) and m (float32 or uint16). Returns the updated amax."""
        am = c_f(amax)
        self.lib.orc_lion_step(_ptr(w), _ptr(m), c_i(int(m.dtype == np.uint16)), _ptr(grad), c_i64(w.size), c_f(lr),
                               c_f(beta1), c_f(beta2), c_f(wd), C.byref(am), C.c_uint(seed))
        return np.float32(am.value)

    def quantize_rowwise_e4m3(self, a, b=None):
        """a (and optional b for the SwiGLU form): uint16 [rows, cols] contiguous."""
        rows, cols = a.shape
        out = np.empty((rows, cols), dtype=np.uint8)
        sc = np.empty(rows, dtype=np.float32)
        de = np.empty(rows, dtype=np.float32)
        self.lib.orc_quantize_rowwise_e4m3(_ptr(a), _ptr(b), c_i64(cols), _ptr(out), c_i64(cols), _ptr(sc), _ptr(de),
                                           c_i(rows), c_i(cols))
        return out, sc, de

    def gelu_forward(self, x):
        out = np.empty(x.shape, dtype=np.uint16)
        self.lib.orc_gelu_forward(_ptr(x), _ptr(out), c_i64(x.size))
        return out

    def moe_topk_route(self, logits, top_k, normalize=True):
        s = np.ascontiguousarray(logits, dtype=np.float32).copy()
        rows, E = s.shape
        self.lib.orc_moe_topk_route_f32(_ptr(s), c_i(rows), c_i(E), c_i(top_k), None, None, c_i(int(normalize)))
        return s

    def moe_build_expert_row_lists(self, rw):
        rows, E = rw.shape
        counts = np.zeros(E, dtype=np.int32)
        idx = np.full((E, rows), -1, dtype=np.int32)
        self.lib.orc_moe_build_expert_row_lists(_ptr(rw), _ptr(counts), _ptr(idx), c_i(rows), c_i(E))
        return counts, idx

    def moe_offsets(self, counts):
        off = np.empty_like(counts)
        self.lib.orc_moe_expert_offsets_from_counts(_ptr(counts), _ptr(off), c_i(counts.size))
        return off

    def moe_gather_rows(self, src, row_indices):
        src2 = src.reshape(src.shape[0], -1)
        wb = src2.shape[1] * src2.itemsize
        idx = np.ascontiguousarray(row_indices, dtype=np.int32)
        dst = np.empty((idx.size, src2.shape[1]), dtype=src.dtype)
        self.lib.orc_moe_gather_rows(_ptr(src2), _ptr(dst), _ptr(idx), c_i(idx.size), c_i(wb))
        return dst

    def moe_scatter_accumulate_rows_bf16(self, mixed, compact, rw, row_indices, expert):
        idx = np.ascontiguousarray(row_indices, dtype=np.int32)
        E = rw.shape[1]; H = mixed.shape[1]
        self.lib.orc_moe_scatter_accumulate_rows_bf16(_ptr(mixed), _ptr(compact), _ptr(rw), _ptr(idx),
                                                      c_i(idx.size), c_i(expert), c_i(E), c_i(H))

    def moe_scale_accumulate_bf16(self, mixed, term, rw, expert):
        rows, H = mixed.shape
        self.lib.orc_moe_scale_accumulate_bf16(_ptr(mixed), _ptr(term), _ptr(rw), c_i(rows), c_i(expert),
                                               c_i(rw.shape[1]), c_i(H))

    def gemm_bf16_nt(self, A, B):
        M, K = A.shape; N = B.shape[0]
        out = np.empty((M, N), dtype=np.uint16)
        self.lib.orc_gemm_bf16_nt(c_i(M), c_i(N), c_i(K), _ptr(A), _ptr(B), _ptr(out))
        return out

    def moe_grouped_expert_forward_fp8(self, hidden8, dx, rw, counts, row_indices, w_in, dwin, w_out, dwout,
                                       mixed, x_is_e5m2=False, threads=0):
        rows, H = hidden8.shape
        E, Ie = w_in.shape[0], w_in.shape[1]
        self.lib.orc_moe_grouped_expert_forward_fp8(_ptr(hidden8), c_f(dx), c_i(int(x_is_e5m2)), _ptr(rw),
                                                    _ptr(counts), _ptr(row_indices), _ptr(w_in), c_f(dwin),
                                                    _ptr(w_out), c_f(dwout), _ptr(mixed), c_i(rows), c_i(H),
                                                    c_i(Ie), c_i(E), c_i(threads))

    def linear_f32_e4m3(self, A, W, bias, threads=0):
        M, K = A.shape; N = W.shape[0]
        out = np.empty((M, N), dtype=np.float32)
        self.lib.orc_linear_f32_e4m3(_ptr(A), _ptr(W), _ptr(bias), _ptr(out), c_i(M), c_i(N), c_i(K), c_i(threads))
        return out


class RefHost:
    """The reference's own host E4M3 codec and NVIDIA's host fp8 conversion,
    compiled from where they lie into oracle/_ref/libref_host.so."""

    def __init__(self):
        path = os.path.join(ORACLE_DIR, "_ref", "libref_host.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = C.CDLL(path)
        self.lib.ref_e4m3_pack.restype = C.c_uint8; self.lib.ref_e4m3_pack.argtypes = [c_f, C.POINTER(c_i)]
        self.lib.ref_e4m3_unpack.restype = c_f; self.lib.ref_e4m3_unpack.argtypes = [C.c_uint8]
        self.lib.ref_nv_e4m3.restype = C.c_uint8; self.lib.ref_nv_e4m3.argtypes = [c_f]
        self.lib.ref_nv_e5m2.restype = C.c_uint8; self.lib.ref_nv_e5m2.argtypes = [c_f]

    def pack_array(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty(x.shape, dtype=np.uint8)
        self.lib.ref_e4m3_pack_array(_ptr(x), _ptr(out), c_i64(x.size))
        return out

    def nv_array(self, x, is_e5m2=False):
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty(x.shape, dtype=np.uint8)
        self.lib.ref_nv_array(_ptr(x), _ptr(out), c_i64(x.size), c_i(int(is_e5m2)))
        return out
