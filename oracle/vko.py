"""TEST INFRASTRUCTURE — Python access to the checkers under oracle/.

* ctypes binding of libvknn_oracle.so (the C restatement of the reference CPU backend, vknn_oracle.h);
* `RefGraph`: writes the text graph spec that oracle/_ref/vknn_ref_driver (the UNMODIFIED reference
  engine) consumes, runs it, and returns the outputs — used to pin the restatement and to time the
  reference's own CPU path.

Only tests/, the smoke check and the bench's cpu_baseline / reference legs import this module. The
product (vknn_b200) never does.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import subprocess
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libvknn_oracle.so")
REF_DRIVER = os.path.join(HERE, "_ref", "vknn_ref_driver")
REF_DRIVER_CUDA = os.path.join(HERE, "_ref", "vknn_ref_driver_cuda")

_lib = None

_f32p = C.POINTER(C.c_float)
_i64p = C.POINTER(C.c_int64)
_i32p = C.POINTER(C.c_int32)


def reference_dir():
    """Where the reference tree lies: $VKNN_REFERENCE_DIR, else a `reference` folder beside the repository. None when
    neither holds the engine's sources (then oracle/_ref is used as prebuilt)."""
    for cand in (os.environ.get("VKNN_REFERENCE_DIR"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.exists(os.path.join(cand, "src", "core", "session.cpp")):
            return cand
    return None


def build():
    """Compile the C restatement (and, where the reference sources are present, oracle/_ref)."""
    subprocess.check_call(["make", "-s", "-C", HERE, "oracle"])
    ref = ["REF=" + reference_dir()] if reference_dir() else []
    subprocess.check_call(["make", "-s", "-C", HERE, "ref"] + ref)
    # the same driver linked with the CUDA plug-in (the GPU plug-in tests run it); needs the built kernel library
    if os.path.exists(os.path.join(HERE, "..", "vknn_b200", "libvknn_cuda.so")):
        subprocess.check_call(["make", "-s", "-C", HERE, "ref-cuda"] + ref)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            subprocess.check_call(["make", "-s", "-C", HERE, "oracle"])
        L = C.CDLL(LIB_PATH)
        L.vko_matmul.restype = C.c_int64
        L.vko_matmul.argtypes = [_f32p, _i64p, C.c_int, _f32p, _i64p, C.c_int, _f32p, _f32p, _i64p, C.POINTER(C.c_int)]
        L.vko_softmax.argtypes = [_f32p, _f32p, C.c_int64, C.c_int64]
        L.vko_layernorm.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_int64, C.c_int64, C.c_float]
        L.vko_binary.restype = C.c_int64
        L.vko_binary.argtypes = [_f32p, _i64p, C.c_int, _f32p, _i64p, C.c_int, C.c_int, _f32p, _i64p, C.POINTER(C.c_int)]
        L.vko_unary.argtypes = [_f32p, _f32p, C.c_int64, C.c_int, C.c_float, C.c_float]
        L.vko_pw_epilogue.restype = C.c_int
        L.vko_pw_epilogue.argtypes = [_f32p, _i64p, C.c_int, C.c_int, _i64p, _f32p, C.POINTER(_f32p), C.POINTER(_i64p), C.POINTER(C.c_int)]
        L.vko_transpose.argtypes = [_f32p, _i64p, C.c_int, _i64p, _f32p]
        L.vko_half_to_float.restype = C.c_float
        L.vko_half_to_float.argtypes = [C.c_uint16]
        L.vko_float_to_half.restype = C.c_uint16
        L.vko_float_to_half.argtypes = [C.c_float]
        L.vko_half_to_float_n.argtypes = [C.POINTER(C.c_uint16), _f32p, C.c_int64]
        L.vko_float_to_half_n.argtypes = [_f32p, C.POINTER(C.c_uint16), C.c_int64]
        L.vko_attention.restype = C.c_int
        L.vko_attention.argtypes = [_f32p, _f32p, _f32p, _f32p] + [C.c_int64] * 6 + [C.c_float, C.c_int, _i32p, _f32p, C.c_int64, C.c_int64, C.c_int]
        L.vko_encoder_layer.restype = C.c_int
        L.vko_encoder_layer.argtypes = [_f32p, _f32p] + [C.c_int64] * 5 + [_f32p] * 12 + [C.c_float, C.c_int]
        L.vko_set_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_f32p)


def _shape(s):
    arr = (C.c_int64 * max(len(s), 1))(*s)
    return arr


def set_threads(n):
    lib().vko_set_threads(int(n))


def matmul(a, b, bias=None):
    a, pa = _f(a)
    b, pb = _f(b)
    pbias = None
    if bias is not None:
        bias, pbias = _f(bias)
    osh = (C.c_int64 * 16)()
    orank = C.c_int(0)
    n = lib().vko_matmul(pa, _shape(a.shape), a.ndim, pb, _shape(b.shape), b.ndim, pbias, None, osh, C.byref(orank))
    if n < 0:
        raise ValueError("vko_matmul: bad shapes %s @ %s" % (a.shape, b.shape))
    y = np.empty([osh[i] for i in range(orank.value)], dtype=np.float32)
    lib().vko_matmul(pa, _shape(a.shape), a.ndim, pb, _shape(b.shape), b.ndim, pbias, y.ctypes.data_as(_f32p), osh, C.byref(orank))
    return y


def softmax(x):
    x, px = _f(x)
    y = np.empty_like(x)
    inner = x.shape[-1]
    lib().vko_softmax(px, y.ctypes.data_as(_f32p), x.size // inner, inner)
    return y


def layernorm(x, gamma, beta, eps):
    x, px = _f(x)
    gamma, pg = _f(gamma)
    pb = None
    if beta is not None:
        beta, pb = _f(beta)
    y = np.empty_like(x)
    norm = gamma.size
    lib().vko_layernorm(px, pg, pb, y.ctypes.data_as(_f32p), x.size // norm, norm, float(eps))
    return y


def binary(a, b, op):
    a, pa = _f(a)
    b, pb = _f(b)
    osh = (C.c_int64 * 16)()
    orank = C.c_int(0)
    lib().vko_binary(pa, _shape(a.shape), a.ndim, pb, _shape(b.shape), b.ndim, op, None, osh, C.byref(orank))
    y = np.empty([osh[i] for i in range(orank.value)], dtype=np.float32)
    lib().vko_binary(pa, _shape(a.shape), a.ndim, pb, _shape(b.shape), b.ndim, op, y.ctypes.data_as(_f32p), osh, C.byref(orank))
    return y


def unary(x, op, p0=0.0, p1=0.0):
    x, px = _f(x)
    y = np.empty_like(x)
    lib().vko_unary(px, y.ctypes.data_as(_f32p), x.size, op, p0, p1)
    return y


def pw_epilogue(primary, steps, params, operands):
    """operands: list of extra operand arrays; step operand index 1 refers to operands[0]."""
    y = np.array(primary, dtype=np.float32, copy=True, order="C")
    nsteps = len(steps) // 4
    st = (C.c_int64 * max(len(steps), 1))(*steps)
    pr = (C.c_float * max(len(params), 1))(*params)
    ops = [None] + [np.ascontiguousarray(o, dtype=np.float32) for o in operands]
    n = len(ops)
    optrs = (_f32p * n)()
    oshapes = (_i64p * n)()
    oranks = (C.c_int * n)()
    keep = []
    for i, o in enumerate(ops):
        if o is None:
            continue
        optrs[i] = o.ctypes.data_as(_f32p)
        s = _shape(o.shape)
        keep.append(s)
        oshapes[i] = C.cast(s, _i64p)
        oranks[i] = o.ndim
    rc = lib().vko_pw_epilogue(y.ctypes.data_as(_f32p), _shape(y.shape), y.ndim, nsteps, st, pr, optrs, oshapes, oranks)
    if rc:
        raise ValueError("vko_pw_epilogue failed")
    return y


def transpose(x, perm=None):
    x, px = _f(x)
    p = list(perm) if perm is not None else list(range(x.ndim))[::-1]
    y = np.empty([x.shape[i] for i in p], dtype=np.float32)
    lib().vko_transpose(px, _shape(x.shape), x.ndim, _shape(p), y.ctypes.data_as(_f32p))
    return y


def float_to_half(x):
    x, px = _f(x)
    y = np.empty(x.shape, dtype=np.uint16)
    lib().vko_float_to_half_n(px, y.ctypes.data_as(C.POINTER(C.c_uint16)), x.size)
    return y


def half_to_float(h):
    h = np.ascontiguousarray(h, dtype=np.uint16)
    y = np.empty(h.shape, dtype=np.float32)
    lib().vko_half_to_float_n(h.ctypes.data_as(C.POINTER(C.c_uint16)), y.ctypes.data_as(_f32p), h.size)
    return y


def attention(q, k, v, scale, causal=False, kv_len=None, mask=None, first_unit=0, num_units=-1, threads=0):
    q, pq = _f(q)
    k, pk = _f(k)
    v, pv = _f(v)
    B, Hq, Sq, D = q.shape
    _, Hkv, Skv, _ = k.shape
    o = np.zeros_like(q)
    pl = None
    if kv_len is not None:
        kv_len = np.ascontiguousarray(kv_len, dtype=np.int32)
        pl = kv_len.ctypes.data_as(_i32p)
    pm = None
    if mask is not None:
        mask, pm = _f(mask)
    rc = lib().vko_attention(pq, pk, pv, o.ctypes.data_as(_f32p), B, Hq, Hkv, Sq, Skv, D, float(scale), int(bool(causal)), pl, pm,
                             first_unit, num_units, threads)
    if rc:
        raise RuntimeError("vko_attention failed")
    return o


def encoder_layer(x, w, H, eps=1e-6, threads=0):
    """w: dict with ln1_g ln1_b wqkv bqkv wo bo ln2_g ln2_b w1 b1 w2 b2 (fp32, weights [K,N])."""
    x, px = _f(x)
    B, T, d = x.shape
    keys = ["ln1_g", "ln1_b", "wqkv", "bqkv", "wo", "bo", "ln2_g", "ln2_b", "w1", "b1", "w2", "b2"]
    arrs = [np.ascontiguousarray(w[k], dtype=np.float32) for k in keys]
    dmlp = arrs[8].shape[1]
    y = np.empty_like(x)
    rc = lib().vko_encoder_layer(px, y.ctypes.data_as(_f32p), B, T, d, H, dmlp, *[a.ctypes.data_as(_f32p) for a in arrs], float(eps), threads)
    if rc:
        raise RuntimeError("vko_encoder_layer failed")
    return y


# --------------------------------------------------------------------------------------------------
# Reference engine driver
# --------------------------------------------------------------------------------------------------
class RefGraph:
    """Builds the text spec + payload for vknn_ref_driver (format described in ref_driver.cpp)."""

    def __init__(self):
        self.lines = []
        self.payload = []
        self.outputs = []

    def _tensor(self, name, role, arr=None, shape=None, dtype="f32"):
        if arr is not None:
            if arr.dtype == np.int64:
                dtype = "i64"
            else:
                arr = np.ascontiguousarray(arr, dtype=np.float32)
            shape = arr.shape
            self.payload.append(arr.tobytes())
        self.lines.append("tensor %s %s %s %d %s" % (name, role, dtype, len(shape), " ".join(str(int(s)) for s in shape)))

    def input(self, name, arr):
        self._tensor(name, "input", arr=arr)

    def init(self, name, arr):
        self._tensor(name, "init", arr=np.asarray(arr))

    def inter(self, name):
        self._tensor(name, "inter", shape=())

    def output(self, name, shape):
        self._tensor(name, "output", shape=())
        self.outputs.append((name, tuple(shape)))

    def node(self, op, name, ins, outs, subop=0, fusedbias=None, **attrs):
        s = "node %s %s subop=%d in=%s out=%s" % (op, name, subop, ",".join(ins), ",".join(outs))
        if fusedbias:
            s += " fusedbias=%s" % fusedbias
        for k, v in attrs.items():
            if isinstance(v, str):
                s += " s:%s=%s" % (k, v.replace(" ", ""))
            elif isinstance(v, float):
                s += " f:%s=%r" % (k, v)
            elif isinstance(v, int):
                s += " i:%s=%d" % (k, v)
            elif isinstance(v, (list, tuple)) and v and isinstance(v[0], float):
                s += " floats:%s=%s" % (k, ",".join(repr(float(x)) for x in v))
            else:
                s += " ints:%s=%s" % (k, ",".join(str(int(x)) for x in v))
        self.lines.append(s)

    def run(self, backend="cpu", precision="high", iters=1, warmup=0, timeout=3600, vxm_fp16=False, device_io=False, cache_file=None, tuning=None,
            device=None, profile=False):
        exe = REF_DRIVER_CUDA if backend == "cuda" else REF_DRIVER
        if not os.path.exists(exe):
            raise FileNotFoundError(exe)
        with tempfile.TemporaryDirectory() as td:
            sp, dp, op = (os.path.join(td, n) for n in ("spec.txt", "data.bin", "out.bin"))
            with open(sp, "w") as f:
                f.write("\n".join(self.lines) + "\n")
            with open(dp, "wb") as f:
                for b in self.payload:
                    f.write(b)
            cmd = [exe, sp, dp, op, "--backend", backend, "--precision", precision, "--iters", str(iters), "--warmup", str(warmup), "--quiet"]
            if vxm_fp16:  # compile to a .vxm with fp16 weights first, then load the session from the file
                cmd += ["--vxm-fp16", os.path.join(td, "model.vxm")]
            if device_io:  # inputs/outputs in registered CUDA buffers (cuda driver only)
                cmd += ["--device-io"]
            if cache_file:  # Config::cacheFile: the CUDA backend keeps its GEMM autotune table in <cache_file>.cuda
                cmd += ["--cache-file", cache_file]
            if tuning:  # Hint::Tuning: off | fast | thorough
                cmd += ["--tuning", tuning]
            if device is not None:  # CUDA device ordinal (cuda driver only)
                cmd += ["--device", str(int(device))]
            if profile:  # Config::profile: the JSON line then carries the Session profiler's records
                cmd += ["--profile"]
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
            info = None
            for ln in r.stdout.splitlines():
                if ln.startswith("{"):
                    info = json.loads(ln)
            if r.returncode != 0 or info is None or not info.get("ok"):
                raise RuntimeError("vknn_ref_driver failed (%d): %s %s" % (r.returncode, r.stdout[-2000:], r.stderr[-2000:]))
            raw = np.fromfile(op, dtype=np.float32)
        outs, off = [], 0
        for o in info["outputs"]:
            n = int(np.prod(o["shape"])) if o["shape"] else 1
            outs.append(raw[off:off + n].reshape(o["shape"]))
            off += n
        return outs, info


def have_ref():
    return os.path.exists(REF_DRIVER)


# Graph builders shared by the golden generator, the parity tests and the bench's reference leg -----
def attention_graph(q, k, v, scale, mask=None):
    """The C1 / GQA pattern as an exporter emits it: Transpose(K) -> MatMul -> Mul(scale) [-> Add(mask)]
    -> Softmax -> MatMul. For GQA, q is [B,Hkv,G*Sq,D]-shaped by the caller (MatMul batch broadcast)."""
    g = RefGraph()
    g.input("q", q)
    g.input("k", k)
    g.input("v", v)
    g.init("scale", np.array([scale], dtype=np.float32))
    if mask is not None:
        g.init("mask", mask)
    for n in ("kt", "s", "ss", "p"):
        g.inter(n)
    if mask is not None:
        g.inter("sm")
    g.output("o", q.shape)
    perm = list(range(k.ndim))
    perm[-1], perm[-2] = perm[-2], perm[-1]
    g.node("Transpose", "kt", ["k"], ["kt"], perm=perm)
    g.node("MatMul", "qk", ["q", "kt"], ["s"])
    g.node("Binary", "scale", ["s", "scale"], ["ss"], subop=0)
    last = "ss"
    if mask is not None:
        g.node("Add", "mask", ["ss", "mask"], ["sm"])
        last = "sm"
    g.node("Softmax", "softmax", [last], ["p"], axis=-1)
    g.node("MatMul", "pv", ["p", "v"], ["o"])
    return g


def encoder_layer_graph(x, w, H, eps=1e-6):
    """A pre-LN ViT block as an exporter emits it (MatMul + Add bias, erf-GELU as Div/Erf/Add/Mul/Mul);
    the reference's passes turn the bias adds into fusedBias and fuse the Mul,Mul tail."""
    B, T, d = x.shape
    D = d // H
    g = RefGraph()
    g.input("x", x)
    for k in ("ln1_g", "ln1_b", "wqkv", "bqkv", "wo", "bo", "ln2_g", "ln2_b", "w1", "b1", "w2", "b2"):
        g.init(k, w[k])
    g.init("shape5", np.array([B, T, 3, H, D], dtype=np.int64))
    g.init("shape3", np.array([B, T, d], dtype=np.int64))
    g.init("i0", np.array([0], dtype=np.int64))
    g.init("i1", np.array([1], dtype=np.int64))
    g.init("i2", np.array([2], dtype=np.int64))
    g.init("scale", np.array([1.0 / np.sqrt(np.float32(D))], dtype=np.float32))
    g.init("sqrt2", np.array([np.float32(1.41421356237)], dtype=np.float32))
    g.init("one", np.array([1.0], dtype=np.float32))
    g.init("half", np.array([0.5], dtype=np.float32))
    for n in ("h1", "qkv0", "qkv", "qkv5", "qkvt", "q", "k", "v", "kt", "s", "ss", "p", "a", "at", "am", "pr0", "pr", "x1", "h2", "f0",
              "f1", "gd", "ge", "ga", "gm", "gh", "m0", "m1"):
        g.inter(n)
    g.output("y", x.shape)
    g.node("LayerNorm", "ln1", ["x", "ln1_g", "ln1_b"], ["h1"], axis=-1, epsilon=float(eps))
    g.node("MatMul", "qkv_mm", ["h1", "wqkv"], ["qkv0"])
    g.node("Add", "qkv_b", ["qkv0", "bqkv"], ["qkv"])
    g.node("Reshape", "qkv_r", ["qkv", "shape5"], ["qkv5"])
    g.node("Transpose", "qkv_t", ["qkv5"], ["qkvt"], perm=[2, 0, 3, 1, 4])
    g.node("Gather", "gq", ["qkvt", "i0"], ["q"], axis=0)
    g.node("Gather", "gk", ["qkvt", "i1"], ["k"], axis=0)
    g.node("Gather", "gv", ["qkvt", "i2"], ["v"], axis=0)
    g.node("Transpose", "k_t", ["k"], ["kt"], perm=[0, 1, 3, 2])
    g.node("MatMul", "qk", ["q", "kt"], ["s"])
    g.node("Binary", "sc", ["s", "scale"], ["ss"], subop=0)
    g.node("Softmax", "sm", ["ss"], ["p"], axis=-1)
    g.node("MatMul", "pv", ["p", "v"], ["a"])
    g.node("Transpose", "a_t", ["a"], ["at"], perm=[0, 2, 1, 3])
    g.node("Reshape", "a_r", ["at", "shape3"], ["am"])
    g.node("MatMul", "proj_mm", ["am", "wo"], ["pr0"])
    g.node("Add", "proj_b", ["pr0", "bo"], ["pr"])
    g.node("Add", "res1", ["x", "pr"], ["x1"])
    g.node("LayerNorm", "ln2", ["x1", "ln2_g", "ln2_b"], ["h2"], axis=-1, epsilon=float(eps))
    g.node("MatMul", "fc1_mm", ["h2", "w1"], ["f0"])
    g.node("Add", "fc1_b", ["f0", "b1"], ["f1"])
    g.node("Binary", "g_div", ["f1", "sqrt2"], ["gd"], subop=2)
    g.node("Unary", "g_erf", ["gd"], ["ge"], subop=15)
    g.node("Add", "g_add", ["ge", "one"], ["ga"])
    g.node("Binary", "g_mul", ["f1", "ga"], ["gm"], subop=0)
    g.node("Binary", "g_half", ["gm", "half"], ["gh"], subop=0)
    g.node("MatMul", "fc2_mm", ["gh", "w2"], ["m0"])
    g.node("Add", "fc2_b", ["m0", "b2"], ["m1"])
    g.node("Add", "res2", ["x1", "m1"], ["y"])
    return g


def vit_frontend_graph(img, wconv, bconv, cls, pos, cos, sin):
    """The caller's graph around the encoder blocks, as a ViT / RoPE exporter emits it: patch-embedding Conv (kernel =
    stride) -> Reshape -> Transpose -> Concat with the Expand-ed class token -> Add(pos) -> Slice (drop the class token) ->
    rotary embedding by Split / Neg / Concat / Mul / Add -> Tile. img [B,C,H,W]; wconv [O,C,p,p]; cls [1,1,O]; pos [1,N+1,O];
    cos, sin [N,O]. Outputs: the token sequence with the class token, the rotated patch tokens and a Tile of a Slice."""
    B, C, H, W = img.shape
    O, _, p, _ = wconv.shape
    hp, wp = H // p, W // p
    N = hp * wp
    g = RefGraph()
    g.input("img", img)
    g.input("cls", cls)  # a runtime input, so that Expand is not folded away at load time
    g.init("wconv", wconv)
    g.init("bconv", bconv)
    g.init("pos", pos)
    g.init("cos", cos)
    g.init("sin", sin)
    g.init("shape_bon", np.array([B, O, N], dtype=np.int64))
    g.init("shape_cls", np.array([B, 1, O], dtype=np.int64))
    g.init("starts", np.array([1], dtype=np.int64))
    g.init("ends", np.array([N + 1], dtype=np.int64))
    g.init("axes", np.array([1], dtype=np.int64))
    g.init("reps", np.array([1, 2, 3], dtype=np.int64))
    for n in ("pe", "pe3", "tok", "clsb", "seq", "patches", "x1", "x2", "nx2", "rot", "xc", "rs", "strided"):
        g.inter(n)
    g.output("seqpos", (B, N + 1, O))
    g.output("roped", (B, N, O))
    g.output("tiled", (B, 2 * ((N + 1) // 2), 3 * (O // 2)))
    g.node("Conv", "patch_embed", ["img", "wconv", "bconv"], ["pe"], strides=[p, p], pads=[0, 0, 0, 0], dilations=[1, 1], kernel_shape=[p, p], group=1)
    g.node("Reshape", "flat", ["pe", "shape_bon"], ["pe3"])
    g.node("Transpose", "tokens", ["pe3"], ["tok"], perm=[0, 2, 1])
    g.node("Expand", "cls_b", ["cls", "shape_cls"], ["clsb"])
    g.node("Concat", "with_cls", ["clsb", "tok"], ["seq"], axis=1)
    g.node("Add", "add_pos", ["seq", "pos"], ["seqpos"])
    g.node("Slice", "drop_cls", ["seqpos", "starts", "ends", "axes"], ["patches"])
    g.node("Split", "halves", ["patches"], ["x1", "x2"], axis=2)
    g.node("Unary", "neg", ["x2"], ["nx2"], subop=7)
    g.node("Concat", "rotate_half", ["nx2", "x1"], ["rot"], axis=2)
    g.node("Binary", "x_cos", ["patches", "cos"], ["xc"], subop=0)
    g.node("Binary", "rot_sin", ["rot", "sin"], ["rs"], subop=0)
    g.node("Add", "rope", ["xc", "rs"], ["roped"])
    g.node("Slice", "every_other", ["seqpos"], ["strided"], starts=[0, 0], ends=[N + 1, O // 2], axes=[1, 2], steps=[2, 1])
    g.node("Tile", "tile", ["strided", "reps"], ["tiled"])
    return g


def masked_pool_graph(x, thr):
    """Token selection and pooling as an exporter emits them: Greater / GreaterEqual / Equal -> Where -> Reduce{Sum, Mean, Max,
    Min, L2} over different axis sets, with and without keepdims. x [B,T,d]; thr [1,1,d] threshold initializer."""
    B, T, d = x.shape
    g = RefGraph()
    g.input("x", x)
    g.init("thr", thr)
    g.init("zero", np.zeros((1,), dtype=np.float32))
    g.init("axes_t", np.array([1], dtype=np.int64))
    for n in ("gt", "kept", "mx", "eq", "rowmean", "ge"):
        g.inter(n)
    g.output("pooled", (B, d))
    g.output("count", (B, 1, d))
    g.output("argmax_mask_sum", (T,))
    g.output("l2", (B, T))
    g.output("minv", (1, 1, d))
    g.output("ge_mean", (B, T, 1))
    g.node("Greater", "gt", ["x", "thr"], ["gt"])
    g.node("Where", "keep", ["gt", "x", "zero"], ["kept"])
    g.node("Reduce", "pool", ["kept", "axes_t"], ["pooled"], subop=1, keepdims=0)
    g.node("Reduce", "count", ["gt"], ["count"], subop=1, axes=[1], keepdims=1)
    g.node("Reduce", "mx", ["x"], ["mx"], subop=2, axes=[0, 2], keepdims=1)
    g.node("Equal", "eq", ["x", "mx"], ["eq"])
    g.node("Reduce", "eqsum", ["eq"], ["argmax_mask_sum"], subop=1, axes=[0, 2], keepdims=0)
    g.node("Reduce", "l2", ["x"], ["l2"], subop=5, axes=[-1], keepdims=0)
    g.node("Reduce", "minv", ["x"], ["minv"], subop=3, axes=[0, 1], keepdims=1)
    g.node("Reduce", "rowmean", ["x"], ["rowmean"], subop=0, axes=[2], keepdims=1)
    g.node("GreaterEqual", "ge", ["x", "rowmean"], ["ge"])
    g.node("Reduce", "ge_mean", ["ge"], ["ge_mean"], subop=0, axes=[2], keepdims=1)
    return g


def token_lookup_graph(x, table, pos, keep, upd, scat_idx, mask):
    """Index-driven data movement as an exported encoder uses it around its blocks: a rotary table looked up with positions
    computed at run time (Gather with a floating index tensor), a constant token selection (Gather with an int64 index list,
    one with a 2-D index shape), ScatterND writing update rows back at constant (batch, token) positions, later rows winning,
    and Where with a condition that broadcasts over the batch and feature axes.
    x [B,T,d]; table [P,d]; pos [T] (integral values); keep int64 [K]; upd [R,d]; scat_idx int64 [R,2]; mask [T,1]."""
    B, T, d = x.shape
    K, R = keep.shape[0], upd.shape[0]
    g = RefGraph()
    g.input("x", x)
    g.input("pos", pos)
    g.input("upd", upd)
    g.input("mask", mask)
    g.init("table", table)
    g.init("keep", keep.astype(np.int64))
    g.init("keep2d", np.array([[0, -1, 2], [T - 1, 1, 0]], dtype=np.int64))
    g.init("scat_idx", scat_idx.astype(np.int64))
    for n in ("rot", "xr"):
        g.inter(n)
    g.output("rotated_kept", (B, K, d))
    g.output("picked2d", (B, 2, 3, d))
    g.output("scattered", (B, T, d))
    g.output("chosen", (B, T, d))
    g.node("Gather", "lookup", ["table", "pos"], ["rot"], axis=0)
    g.node("Binary", "rotate", ["x", "rot"], ["xr"], subop=0)
    g.node("Gather", "select", ["xr", "keep"], ["rotated_kept"], axis=1)
    g.node("Gather", "select2d", ["x", "keep2d"], ["picked2d"], axis=-2)
    g.node("ScatterND", "writeback", ["xr", "scat_idx", "upd"], ["scattered"])
    g.node("Where", "choose", ["mask", "x", "xr"], ["chosen"])
    return g


def rope_table_graph(x, pos, inv_freq):
    """Rotary position embedding with its frequency table built in the graph, as the exported encoder does it (one outer
    product per table): freqs = Einsum("i,j->ij", pos, inv_freq) -> Concat(freqs, freqs) -> Cos / Sin -> x * cos +
    rotate_half(x) * sin. x [B,T,d]; pos [T] positions (a run-time input); inv_freq [d/2] constant. Outputs: the frequency
    table [T,d/2], and the rotated tokens [B,T,d]."""
    B, T, d = x.shape
    g = RefGraph()
    g.input("x", x)
    g.input("pos", pos)
    g.init("inv_freq", inv_freq)
    for n in ("emb", "cos", "sin", "x1", "x2", "nx2", "rot", "xc", "rs"):
        g.inter(n)
    g.output("freqs", (T, d // 2))
    g.output("roped", (B, T, d))
    g.node("Einsum", "freq_table", ["pos", "inv_freq"], ["freqs"], equation="i,j->ij")
    g.node("Concat", "both_halves", ["freqs", "freqs"], ["emb"], axis=1)
    g.node("Unary", "cos", ["emb"], ["cos"], subop=16)
    g.node("Unary", "sin", ["emb"], ["sin"], subop=17)
    g.node("Split", "halves", ["x"], ["x1", "x2"], axis=2)
    g.node("Unary", "neg", ["x2"], ["nx2"], subop=7)
    g.node("Concat", "rotate_half", ["nx2", "x1"], ["rot"], axis=2)
    g.node("Binary", "x_cos", ["x", "cos"], ["xc"], subop=0)
    g.node("Binary", "rot_sin", ["rot", "sin"], ["rs"], subop=0)
    g.node("Add", "rope", ["xc", "rs"], ["roped"])
    return g
