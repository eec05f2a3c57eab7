"""ctypes binding of include/vknn_cuda.h. Tensors are torch CUDA tensors (device memory only); every compute
call goes through the C-ABI entry point of the same name."""
from __future__ import annotations

import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(os.path.dirname(HERE), "include", "vknn_cuda.h")

F32, F16, BF16, I32 = 0, 1, 2, 3
EPI_NONE, EPI_BIAS, EPI_GELU_ERF, EPI_RESIDUAL = 0, 1, 2, 4
B_KN, B_NK = 0, 1
IMPL_AUTO, IMPL_SIMT, IMPL_TCGEN05 = 0, 1, 2

_lib = None


class VkcError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("libvknn_cuda error %d: %s" % (code, msg))
        self.code = code


def lib_path():
    return os.path.join(HERE, "libvknn_cuda.so")


def declared_symbols():
    """Names of the entry points include/vknn_cuda.h declares."""
    with open(HEADER) as f:
        return sorted(set(re.findall(r"VKC_API[^;(]*?\b(vkc_\w+)\s*\(", f.read())))


def exported_symbols():
    lib = load_library()
    return [s for s in declared_symbols() if hasattr(lib, s)]


def load_library():
    """Loads libvknn_cuda.so. There is no fallback: a missing library is an error."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise ImportError("libvknn_cuda.so is not built (%s); run `python -m vknn_b200.build`" % path)
    L = C.CDLL(path)
    vp, i64, i32, f32, sz = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_size_t
    L.vkc_device_count.argtypes = [C.POINTER(C.c_int)]
    L.vkc_ctx_create.argtypes = [i32, C.POINTER(vp)]
    L.vkc_ctx_destroy.argtypes = [vp]
    L.vkc_device_info.argtypes = [vp, C.c_char_p, sz, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    L.vkc_last_error.argtypes = [vp]
    L.vkc_last_error.restype = C.c_char_p
    L.vkc_ctx_set_impl.argtypes = [vp, i32]
    L.vkc_sync.argtypes = [vp, vp]
    L.vkc_launch_count.argtypes = [vp]
    L.vkc_launch_count.restype = i64
    L.vkc_extbuf_register.argtypes = [vp, C.c_size_t, C.POINTER(C.c_int)]
    L.vkc_extbuf_unregister.argtypes = [C.c_int]
    L.vkc_extbuf_lookup.argtypes = [C.c_int, C.POINTER(vp), C.POINTER(C.c_size_t)]
    L.vkc_alloc.argtypes = [vp, sz, C.POINTER(vp)]
    L.vkc_free.argtypes = [vp, vp]
    L.vkc_upload.argtypes = [vp, vp, i32, vp, i32, i64, vp]
    L.vkc_download.argtypes = [vp, vp, i32, vp, i32, i64, vp]
    L.vkc_convert.argtypes = [vp, vp, i32, vp, i32, i64, vp]
    L.vkc_gemm.argtypes = [vp, vp, vp, vp, vp, vp] + [i64] * 10 + [i32, i32, i32, vp]
    L.vkc_gemm_ex.argtypes = [vp, vp, vp, vp, vp, vp] + [i64] * 10 + [i32, i32, i32, i32, vp]
    L.vkc_gemm_gated.argtypes = [vp, vp, vp, vp, vp, vp] + [i64] * 10 + [i32, i32, i32, i32, C.POINTER(Gate), vp]
    L.vkc_gemm_config_count.argtypes = []
    L.vkc_attn_prefill.argtypes = [vp, vp, vp, vp, vp] + [i64] * 6 + [vp, vp, vp, vp, f32, i32, vp, vp, i32, vp]
    L.vkc_attn_prefill_fanout.argtypes = [vp, vp, vp, vp] + [i64] * 6 + [vp, vp, vp, vp, f32, i32, vp, i32, C.POINTER(Fanout), vp]
    L.vkc_peer_wait.argtypes = [vp, vp, i32, vp, vp]
    L.vkc_layernorm_fanout.argtypes = [vp, vp, vp, vp, i64, i64, f32, i32, C.POINTER(Fanout), vp]
    L.vkc_peer_export.argtypes = [vp, vp, C.c_char_p]
    L.vkc_peer_open.argtypes = [vp, C.c_char_p, C.POINTER(vp)]
    L.vkc_peer_close.argtypes = [vp, vp]
    L.vkc_attn_prefill_plan.argtypes = [i32] + [i64] * 5 + [i32, i32, C.POINTER(C.c_int32)]
    L.vkc_attn_prefill_items.argtypes = [i32] + [i64] * 5 + [i32, i32, i32, C.POINTER(C.c_int32), i32]
    L.vkc_attn_decode_workspace_bytes.argtypes = [i64] * 5
    L.vkc_attn_decode_items.argtypes = [i32] + [i64] * 5 + [C.POINTER(C.c_int32), i32, C.POINTER(C.c_int32), i32, C.POINTER(C.c_int32)]
    L.vkc_attn_decode_workspace_bytes.restype = sz
    L.vkc_attn_decode.argtypes = [vp, vp, vp, vp, vp] + [i64] * 5 + [vp, f32, vp, sz, i32, vp]
    L.vkc_attn_decode_noalloc_max_bytes.argtypes = []
    L.vkc_attn_decode_noalloc_max_bytes.restype = sz
    L.vkc_attn_decode_noalloc.argtypes = [vp, vp, vp, vp, vp] + [i64] * 5 + [vp, f32, i32, vp]
    L.vkc_layernorm.argtypes = [vp, vp, vp, vp, vp, i64, i64, f32, i32, vp]
    L.vkc_pointwise.argtypes = [vp, vp, vp, vp, i32, i32, vp, vp, i32, vp, vp, i32, vp]
    L.vkc_softmax.argtypes = [vp, vp, vp, i64, i64, i32, vp]
    L.vkc_strided_copy.argtypes = [vp, vp, vp, vp, vp, i32, i64, i32, vp]
    L.vkc_reduce_rows.argtypes = [vp, vp, vp, i64, i64, i32, i32, vp]
    L.vkc_strided_copy2.argtypes = [vp, vp, vp, vp, vp, vp, i32, i64, i32, vp]
    L.vkc_copy_rows.argtypes = [vp, vp, vp, vp, vp, i64, i64, i32, vp]
    L.vkc_gather_rows.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, vp]
    L.vkc_graph_begin.argtypes = [vp]
    L.vkc_graph_end.argtypes = [vp, C.POINTER(vp)]
    L.vkc_graph_launch.argtypes = [vp, vp]
    L.vkc_graph_destroy.argtypes = [vp, vp]
    L.vkc_raster_workspace_bytes.argtypes = [i64, i32, i32, i32]
    L.vkc_raster_workspace_bytes.restype = sz
    L.vkc_raster_gaussians.argtypes = [vp, vp, vp, vp, vp, i64, C.POINTER(C.c_double), C.POINTER(C.c_double), i32, i32, C.c_double, i32, vp, vp, vp, sz, vp]
    L.vkc_timer_start.argtypes = [vp, vp]
    L.vkc_timer_stop.argtypes = [vp, vp, C.POINTER(C.c_float)]
    _lib = L
    return L


def _dtype_code(t):
    import torch
    return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}[t.dtype]


def _np_dtype_code(a):
    import numpy as np
    if a.dtype == np.float32:
        return F32
    if a.dtype == np.float16:
        return F16
    raise TypeError("host arrays must be float32 or float16")


class Fanout(C.Structure):
    """Mirror of struct vkc_fanout (include/vknn_cuda.h)."""
    _fields_ = [("n_dest", C.c_int), ("dest", C.c_void_p * 8), ("flag", C.c_void_p * 8), ("state", C.c_void_p), ("mcast", C.c_void_p)]


class Gate(C.Structure):
    """Mirror of struct vkc_gate (include/vknn_cuda.h)."""
    _fields_ = [("flags", C.c_void_p), ("n", C.c_int), ("state", C.c_void_p)]


PEER_HANDLE_BYTES = 64


def _i64arr(vals):
    return (C.c_int64 * len(vals))(*[int(v) for v in vals])


PLAN_FIELDS = ("form", "query_tiles", "ctas", "rounds", "left", "pieces", "quota", "steps")
ITEM_FIELDS = ("b", "h", "qg", "j0", "n_t0", "n_t1", "slot", "last")


def attn_prefill_plan(sm_count, B, Hq, Sq, Skv, D, causal=False, has_kv_len=False):
    """How vkc_attn_prefill's tensor-core kernel spreads the shape over `sm_count` SMs (host arithmetic; needs no GPU)."""
    out = (C.c_int32 * 8)()
    rc = load_library().vkc_attn_prefill_plan(sm_count, B, Hq, Sq, Skv, D, int(bool(causal)), int(bool(has_kv_len)), out)
    if rc != 0:
        raise VkcError(rc, "vkc_attn_prefill_plan")
    return dict(zip(PLAN_FIELDS, out))


def attn_prefill_items(sm_count, B, Hq, Sq, Skv, D, cta, causal=False, has_kv_len=False):
    """The items CTA `cta` of that plan runs, in order, as dicts over ITEM_FIELDS."""
    lib, cap = load_library(), 64
    while True:
        buf = (C.c_int32 * (8 * cap))()
        n = lib.vkc_attn_prefill_items(sm_count, B, Hq, Sq, Skv, D, int(bool(causal)), int(bool(has_kv_len)), cta, buf, cap)
        if n < 0:
            raise VkcError(n, "vkc_attn_prefill_items")
        if n <= cap:
            return [dict(zip(ITEM_FIELDS, buf[8 * i:8 * i + 8])) for i in range(n)]
        cap = n


DECODE_ITEM_FIELDS = ("b", "hk", "start", "end", "pair", "last")


def attn_decode_items(sm_count, B, Hq, Hkv, Lmax, D, kv_len=None):
    """The items of every CTA of the decode split kernel for host lengths `kv_len` (list or None), and the plan
    {"grid", "slots", "min_tiles"}. Host arithmetic; needs no GPU. Raises VkcError for a shape the tensor-core form does not take."""
    lib = load_library()
    lens = (C.c_int32 * B)(*kv_len) if kv_len is not None else None
    plan, cap = (C.c_int32 * 3)(), 64
    per_cta, cta = [], 0
    while True:
        buf = (C.c_int32 * (6 * cap))()
        n = lib.vkc_attn_decode_items(sm_count, B, Hq, Hkv, Lmax, D, lens, cta, buf, cap, plan)
        if n < 0:
            raise VkcError(n, "vkc_attn_decode_items")
        if n > cap:
            cap = n
            continue
        per_cta.append([dict(zip(DECODE_ITEM_FIELDS, buf[6 * i:6 * i + 6])) for i in range(n)])
        cta += 1
        if cta >= plan[0]:
            return dict(grid=plan[0], slots=plan[1], min_tiles=plan[2]), per_cta


class Context:
    """One libvknn_cuda context (one device). `stream` arguments default to torch's current stream so that
    torch.cuda.Event timing and torch allocations order correctly with the kernels."""

    def __init__(self, device=0):
        self.lib = load_library()
        h = C.c_void_p()
        rc = self.lib.vkc_ctx_create(int(device), C.byref(h))
        if rc != 0:
            raise VkcError(rc, "vkc_ctx_create(%d) failed (no usable sm_100 device?)" % device)
        self.h = h
        self.device = int(device)

    def close(self):
        if getattr(self, "h", None):
            self.lib.vkc_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc):
        if rc != 0:
            raise VkcError(rc, self.lib.vkc_last_error(self.h).decode())

    def _stream(self, stream):
        if stream is not None:
            return C.c_void_p(stream)
        import torch
        h = torch.cuda.current_stream(self.device).cuda_stream
        # torch's default stream is the legacy NULL stream; NULL means "the context's own stream" in the C-ABI,
        # so name the legacy stream by its explicit handle (cudaStreamLegacy == 0x1) to keep torch ordering.
        return C.c_void_p(h if h else 1)

    def device_info(self):
        """(name, SM count, maximum SM clock in MHz) of the context's device."""
        name = C.create_string_buffer(128)
        sms, mhz = C.c_int(0), C.c_int(0)
        self._check(self.lib.vkc_device_info(self.h, name, 128, C.byref(sms), C.byref(mhz)))
        return name.value.decode(), sms.value, mhz.value

    def set_impl(self, impl):
        self._check(self.lib.vkc_ctx_set_impl(self.h, impl))

    def sync(self, stream=None):
        self._check(self.lib.vkc_sync(self.h, self._stream(stream)))

    def launch_count(self):
        return int(self.lib.vkc_launch_count(self.h))

    # ---- boundary transfers (host numpy <-> device torch) ----
    def upload(self, dst, src_host, stream=None):
        assert dst.is_contiguous() and src_host.flags["C_CONTIGUOUS"] and dst.numel() == src_host.size
        self._check(self.lib.vkc_upload(self.h, dst.data_ptr(), _dtype_code(dst), src_host.ctypes.data, _np_dtype_code(src_host), dst.numel(),
                                        self._stream(stream)))

    def upload_ptr(self, dst, host_ptr, host_dtype, stream=None):
        self._check(self.lib.vkc_upload(self.h, dst.data_ptr(), _dtype_code(dst), host_ptr, host_dtype, dst.numel(), self._stream(stream)))

    def download(self, dst_host, src, stream=None):
        assert src.is_contiguous() and dst_host.flags["C_CONTIGUOUS"] and src.numel() == dst_host.size
        self._check(self.lib.vkc_download(self.h, dst_host.ctypes.data, _np_dtype_code(dst_host), src.data_ptr(), _dtype_code(src), src.numel(),
                                          self._stream(stream)))

    def download_ptr(self, host_ptr, host_dtype, src, stream=None):
        self._check(self.lib.vkc_download(self.h, host_ptr, host_dtype, src.data_ptr(), _dtype_code(src), src.numel(), self._stream(stream)))

    def convert(self, dst, src, stream=None):
        self._check(self.lib.vkc_convert(self.h, dst.data_ptr(), _dtype_code(dst), src.data_ptr(), _dtype_code(src), src.numel(), self._stream(stream)))

    # ---- kernels ----
    def gemm(self, A, B, D, bias=None, residual=None, b_layout=B_KN, epilogue=None, stream=None, config=-1, gate=None):
        """A [batch?,M,K], B [batch?,K,N] (B_KN) or [batch?,N,K] (B_NK), D [batch?,M,N]; a 2-D operand broadcasts.
        config >= 0 forces one of the tensor-core kernel's configurations (see gemm_config_count).
        gate = (flags pointer, n, state tensor of two int32): A is produced by other GPUs; the kernel waits for their flags."""
        M, K = A.shape[-2:]
        N = D.shape[-1]
        batch = D.shape[0] if D.dim() == 3 else 1
        sa = A.stride(0) if A.dim() == 3 else 0
        sb = B.stride(0) if B.dim() == 3 else 0
        sd = D.stride(0) if D.dim() == 3 else 0
        if epilogue is None:
            epilogue = (EPI_BIAS if bias is not None else 0) | (EPI_RESIDUAL if residual is not None else 0)
        args = (self.h, A.data_ptr(), B.data_ptr(), bias.data_ptr() if bias is not None else None,
                residual.data_ptr() if residual is not None else None, D.data_ptr(), M, N, K, batch, sa, sb, sd,
                A.stride(-2), B.stride(-2), D.stride(-2), b_layout, epilogue, _dtype_code(A), int(config))
        if gate is None:
            self._check(self.lib.vkc_gemm_ex(*args, self._stream(stream)))
        else:
            g = Gate(int(gate[0]), int(gate[1]), gate[2].data_ptr())
            self._check(self.lib.vkc_gemm_gated(*args, C.byref(g), self._stream(stream)))

    def gemm_config_count(self):
        return int(self.lib.vkc_gemm_config_count())

    def attn_prefill(self, Q, K, V, O, scale, causal=False, mask=None, kv_len=None, stream=None):
        """Q/O [B,Hq,Sq,D], K/V [B,Hkv,Skv,D]; any strides with D contiguous (views of a packed qkv buffer are fine)."""
        B, Hq, Sq, D = Q.shape
        _, Hkv, Skv, _ = K.shape
        for t in (Q, K, V, O):
            assert t.stride(-1) == 1
        st = lambda t: _i64arr([t.stride(0), t.stride(1), t.stride(2)])  # noqa: E731
        self._check(self.lib.vkc_attn_prefill(self.h, Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), B, Hq, Hkv, Sq, Skv, D,
                                              st(Q), st(K), st(V), st(O), float(scale), int(bool(causal)),
                                              mask.data_ptr() if mask is not None else None, kv_len.data_ptr() if kv_len is not None else None,
                                              _dtype_code(Q), self._stream(stream)))

    def attn_prefill_fanout(self, Q, K, V, dests, flags, state, o_strides, scale, causal=False, kv_len=None, stream=None, mcast=None):
        """attn_prefill whose output rows are stored into every buffer of `dests` (raw device pointers mapped on this GPU,
        addressed with o_strides = (batch, head, row) element strides); `flags[d]` (pointer or None) receives this rank's
        completion count when the last block has stored; `state` is a zeroed 2 x int32 device tensor kept by the caller.
        mcast: the same buffer's address in an NVSwitch multicast mapping of all destinations (one store reaches them all)."""
        B, Hq, Sq, D = Q.shape
        _, Hkv, Skv, _ = K.shape
        for t in (Q, K, V):
            assert t.stride(-1) == 1
        f = self._fanout(dests, flags, state, mcast)
        st = lambda t: _i64arr([t.stride(0), t.stride(1), t.stride(2)])  # noqa: E731
        self._check(self.lib.vkc_attn_prefill_fanout(self.h, Q.data_ptr(), K.data_ptr(), V.data_ptr(), B, Hq, Hkv, Sq, Skv, D, st(Q), st(K), st(V),
                                                     _i64arr(list(o_strides)), float(scale), int(bool(causal)),
                                                     kv_len.data_ptr() if kv_len is not None else None, _dtype_code(Q), C.byref(f), self._stream(stream)))

    def _fanout(self, dests, flags, state, mcast=None):
        f = Fanout()
        f.n_dest = len(dests)
        for i, d in enumerate(dests):
            f.dest[i] = int(d)
            f.flag[i] = int(flags[i]) if flags is not None and flags[i] else None
        f.state = state.data_ptr()
        f.mcast = int(mcast) if mcast else None
        return f

    def layernorm_fanout(self, X, gamma, beta, dests, flags, state, eps, stream=None, mcast=None):
        """LayerNorm of X [rows, norm] whose output rows are stored at each pointer of `dests` (see attn_prefill_fanout)."""
        rows, norm = X.shape
        assert X.is_contiguous()
        f = self._fanout(dests, flags, state, mcast)
        self._check(self.lib.vkc_layernorm_fanout(self.h, X.data_ptr(), gamma.data_ptr(), beta.data_ptr() if beta is not None else None, rows, norm,
                                                  float(eps), _dtype_code(X), C.byref(f), self._stream(stream)))

    def peer_wait(self, flags_ptr, n, expected, stream=None):
        """Stream-ordered bounded wait until each of the n flag words at flags_ptr has reached expected[0] + 1."""
        self._check(self.lib.vkc_peer_wait(self.h, int(flags_ptr), n, expected.data_ptr(), self._stream(stream)))

    def raw_alloc(self, nbytes):
        p = C.c_void_p()
        self._check(self.lib.vkc_alloc(self.h, nbytes, C.byref(p)))
        return int(p.value)

    def raw_free(self, ptr):
        self._check(self.lib.vkc_free(self.h, int(ptr)))

    def peer_export(self, ptr):
        buf = C.create_string_buffer(PEER_HANDLE_BYTES)
        self._check(self.lib.vkc_peer_export(self.h, int(ptr), buf))
        return bytes(buf.raw)

    def peer_open(self, handle):
        p = C.c_void_p()
        self._check(self.lib.vkc_peer_open(self.h, C.c_char_p(handle), C.byref(p)))
        return int(p.value)

    def peer_close(self, ptr):
        self._check(self.lib.vkc_peer_close(self.h, int(ptr)))

    def attn_decode_workspace_bytes(self, B, Hq, Hkv, Lmax, D):
        return int(self.lib.vkc_attn_decode_workspace_bytes(B, Hq, Hkv, Lmax, D))

    def attn_decode(self, Q, Kc, Vc, O, scale, kv_len=None, workspace=None, stream=None):
        """Q/O [B,Hq,D], Kc/Vc [B,Hkv,Lmax,D] contiguous."""
        B, Hq, D = Q.shape
        _, Hkv, Lmax, _ = Kc.shape
        assert Q.is_contiguous() and Kc.is_contiguous() and Vc.is_contiguous() and O.is_contiguous()
        self._check(self.lib.vkc_attn_decode(self.h, Q.data_ptr(), Kc.data_ptr(), Vc.data_ptr(), O.data_ptr(), B, Hq, Hkv, Lmax, D,
                                             kv_len.data_ptr() if kv_len is not None else None, float(scale),
                                             workspace.data_ptr() if workspace is not None else None,
                                             workspace.numel() * workspace.element_size() if workspace is not None else 0, _dtype_code(Q),
                                             self._stream(stream)))

    def attn_decode_noalloc(self, Q, Kc, Vc, O, scale, kv_len=None, stream=None):
        """Same as attn_decode, but the per-split partials live in the library's fixed 16 MiB area and the call
        allocates nothing. Raises VkcError(-1) when the shape needs more than that."""
        B, Hq, D = Q.shape
        _, Hkv, Lmax, _ = Kc.shape
        assert Q.is_contiguous() and Kc.is_contiguous() and Vc.is_contiguous() and O.is_contiguous()
        self._check(self.lib.vkc_attn_decode_noalloc(self.h, Q.data_ptr(), Kc.data_ptr(), Vc.data_ptr(), O.data_ptr(), B, Hq, Hkv, Lmax, D,
                                                     kv_len.data_ptr() if kv_len is not None else None, float(scale), _dtype_code(Q),
                                                     self._stream(stream)))

    def layernorm(self, X, gamma, beta, Y, eps, stream=None):
        norm = gamma.numel()
        assert X.is_contiguous() and Y.is_contiguous()
        self._check(self.lib.vkc_layernorm(self.h, X.data_ptr(), gamma.data_ptr(), beta.data_ptr() if beta is not None else None, Y.data_ptr(),
                                           X.numel() // norm, norm, float(eps), _dtype_code(X), self._stream(stream)))

    def pointwise(self, X, Y, steps, params, operands=(), stream=None):
        """steps: flat ints, 4 per step (kind, code, operand index 1-based, unused); operands broadcast NumPy-style."""
        assert X.is_contiguous() and Y.is_contiguous()
        shape = list(X.shape) or [1]
        rank = len(shape)
        nsteps = len(steps) // 4
        strides = []
        for o in operands:
            assert o.is_contiguous()
            oshape = [1] * (rank - o.dim()) + list(o.shape)
            s, acc = [0] * rank, 1
            for d in range(rank - 1, -1, -1):
                s[d] = 0 if oshape[d] == 1 else acc
                acc *= oshape[d]
            strides += s
        ptrs = (C.c_void_p * max(len(operands), 1))(*[o.data_ptr() for o in operands])
        self._check(self.lib.vkc_pointwise(self.h, X.data_ptr(), Y.data_ptr(), _i64arr(shape), rank, nsteps,
                                           (C.c_int32 * max(len(steps), 1))(*[int(s) for s in steps]),
                                           (C.c_float * max(len(params), 1))(*[float(p) for p in params]), len(operands), ptrs,
                                           _i64arr(strides or [0]), _dtype_code(X), self._stream(stream)))

    def softmax(self, X, Y, stream=None):
        inner = X.shape[-1]
        assert X.is_contiguous() and Y.is_contiguous()
        self._check(self.lib.vkc_softmax(self.h, X.data_ptr(), Y.data_ptr(), X.numel() // inner, inner, _dtype_code(X), self._stream(stream)))

    def raster_gaussians(self, means, covs, colors, opacities, w2c, K, H, W, near=0.2, precise=True, stream=None):
        """3D Gaussian-splatting render of one view. means [n,3], covs [n,3,3], colors [n,3], opacities [n]: fp32 CUDA tensors;
        w2c 4x4 and K 3x3 host arrays (float64). Returns (rgb [H,W,3], alpha [H,W]) fp32 CUDA tensors."""
        import numpy as np
        import torch
        n = int(means.shape[0])
        for t in (means, covs, colors, opacities):
            assert t.dtype == torch.float32 and t.is_contiguous() and t.is_cuda
        w = np.ascontiguousarray(w2c, dtype=np.float64).reshape(16)
        k = np.ascontiguousarray(K, dtype=np.float64).reshape(9)
        rgb = torch.empty(H, W, 3, dtype=torch.float32, device=means.device)
        alpha = torch.empty(H, W, dtype=torch.float32, device=means.device)
        nbytes = int(self.lib.vkc_raster_workspace_bytes(n, int(H), int(W), int(bool(precise))))
        ws = torch.empty(nbytes + 256, dtype=torch.uint8, device=means.device)
        off = (-ws.data_ptr()) % 256
        self._check(self.lib.vkc_raster_gaussians(self.h, means.data_ptr(), covs.data_ptr(), colors.data_ptr(), opacities.data_ptr(), n,
                                                  w.ctypes.data_as(C.POINTER(C.c_double)), k.ctypes.data_as(C.POINTER(C.c_double)), int(H), int(W),
                                                  float(near), int(bool(precise)), rgb.data_ptr(), alpha.data_ptr(), ws.data_ptr() + off, nbytes,
                                                  self._stream(stream)))
        self._keepalive = ws  # the workspace must outlive the asynchronous launches
        return rgb, alpha

    def copy_rows(self, src, dst, src_off, dst_off, row_elems, stream=None):
        """dst[dst_off[r] + j] = src[src_off[r] + j] for every row r; the offset tables are int64 device tensors (None: r * row_elems)."""
        nrows = (src_off if src_off is not None else dst_off).numel() if (src_off is not None or dst_off is not None) else src.numel() // max(row_elems, 1)
        self._check(self.lib.vkc_copy_rows(self.h, src.data_ptr(), dst.data_ptr(), src_off.data_ptr() if src_off is not None else None,
                                           dst_off.data_ptr() if dst_off is not None else None, nrows, row_elems, _dtype_code(src), self._stream(stream)))

    def gather_rows(self, data, index, out, outer, axis_size, inner, stream=None):
        """out[o, k, :] = data[o, index[k], :] with a device-resident index tensor (float32 / float16 / bfloat16 / int32)."""
        import torch
        icode = I32 if index.dtype == torch.int32 else _dtype_code(index)
        self._check(self.lib.vkc_gather_rows(self.h, data.data_ptr(), index.data_ptr(), out.data_ptr(), outer, axis_size, index.numel(), inner,
                                             _dtype_code(data), icode, self._stream(stream)))

    def strided_copy(self, X, Y, shape, in_strides, in_offset=0, stream=None):
        self._check(self.lib.vkc_strided_copy(self.h, X.data_ptr(), Y.data_ptr(), _i64arr(shape), _i64arr(in_strides), len(shape), in_offset,
                                              _dtype_code(X), self._stream(stream)))
