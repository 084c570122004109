"""ctypes binding of the CPU checker (oracle/libsp_moe_oracle.so) and of the reference's own
CPU expert code compiled in place (oracle/_ref/libsp_moe_cpu_ref.so).

Test infrastructure only: imported by tests/, by __graft_entry__.smoke() and by bench.py's
cpu_baseline / --impl reference legs. The product package never imports it.
"""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
_ORC_SO = os.path.join(ORACLE_DIR, "libsp_moe_oracle.so")
_REF_SO = os.path.join(ORACLE_DIR, "_ref", "libsp_moe_cpu_ref.so")

f32p = C.POINTER(C.c_float)
u8p = C.POINTER(C.c_uint8)
u16p = C.POINTER(C.c_uint16)
i8p = C.POINTER(C.c_int8)
i32p = C.POINTER(C.c_int32)
f64p = C.POINTER(C.c_double)


class OrcCfg(C.Structure):
    _fields_ = [("E", C.c_int32), ("NE", C.c_int32), ("NU", C.c_int32), ("FFE", C.c_int32),
                ("FFS", C.c_int32), ("eps", C.c_float)]


class OrcLayer(C.Structure):
    _fields_ = [("router_w", f32p), ("router_scale", f32p), ("router_bias", f32p),
                ("ffn_norm", f32p), ("post_ffw1", f32p), ("pre_ffw2", f32p), ("post_ffw2", f32p),
                ("post_ffw", f32p), ("dexps_scale", f32p),
                ("gu_codes", u8p), ("gu_bs", u16p), ("dn_codes", u8p), ("dn_bs", u16p),
                ("sg_codes", u8p), ("sg_bs", u16p), ("su_codes", u8p), ("su_bs", u16p),
                ("sd_codes", u8p), ("sd_bs", u16p)]


def build_oracle(with_ref=True):
    """Compile the checker and, where the reference tree is mounted (SP_REFERENCE_ROOT, or the Makefile's
    default), the reference's own CPU expert file and its own decode kernels; without the tree those two
    targets have no source and are skipped (the prebuilt files under oracle/_ref are then used as they are)."""
    subprocess.run(["make", "-s", "-C", ORACLE_DIR], check=True)
    if with_ref:
        for target in ("ref", "ref_gpu"):
            subprocess.run(["make", "-s", "-C", ORACLE_DIR, target], check=False, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_ORC_SO):
            build_oracle(with_ref=False)
        L = C.CDLL(_ORC_SO)
        L.orc_rmsnorm.argtypes = [f32p, f32p, C.c_int, C.c_float, f32p]
        L.orc_router_prep.argtypes = [f32p, f32p, C.c_int, C.c_float, f32p]
        L.orc_router_dot.argtypes = [f32p, f32p, C.c_int]
        L.orc_router_dot.restype = C.c_float
        L.orc_topk.argtypes = [f32p, C.c_int, C.c_int, i32p, f32p]
        L.orc_quant_act_int8.argtypes = [f32p, C.c_int, i8p, f32p]
        L.orc_gemv_q4b_a.argtypes = [u8p, u16p, C.c_int, C.c_int, i8p, f32p, f32p]
        L.orc_gemv_q4b_b.argtypes = [u8p, u16p, C.c_int, C.c_int, f32p, f32p]
        L.orc_tanhf.argtypes = [C.c_float]
        L.orc_tanhf.restype = C.c_float
        L.orc_gelu_mul.argtypes = [C.c_float, C.c_float]
        L.orc_gelu_mul.restype = C.c_float
        L.orc_half_to_float.argtypes = [C.c_uint16]
        L.orc_half_to_float.restype = C.c_float
        L.orc_float_to_half.argtypes = [C.c_float]
        L.orc_float_to_half.restype = C.c_uint16
        L.orc_layer_forward.argtypes = [C.POINTER(OrcCfg), C.POINTER(OrcLayer), C.c_int, C.c_int,
                                        f32p, f32p, i32p, f32p, f32p, f64p]
        L.orc_standalone_q4b.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, f32p, f32p,
                                         u8p, u16p, u8p, u16p, f32p, f32p, i32p]
        L.orc_q4b_quantize.argtypes = [f32p, C.c_int64, C.c_int, u8p, u16p]
        L.orc_q4b_dequantize.argtypes = [u8p, u16p, C.c_int64, C.c_int, f32p]
        L.orc_int_gemm_scaled.argtypes = [i8p, i8p, C.c_int, C.c_int, C.c_int, f32p, f32p, u16p]
        L.orc_set_threads.argtypes = [C.c_int]
        L.orc_set_backend.argtypes = [C.c_void_p, C.c_void_p]
        _lib = L
    return _lib


_ref = None


def ref_lib(nthreads=4):
    """The reference's moe_cpu_expert.c, or None when it was not built or this CPU lacks
    AVX-512 VNNI (sp_moe_cpu_init returns 0, moe_cpu_expert.c:216-223)."""
    global _ref
    if _ref is None:
        if not os.path.exists(_REF_SO):
            _ref = False
            return None
        flags = open("/proc/cpuinfo").read()
        if not all(f in flags for f in ("avx512f", "avx512bw", "avx512_vnni", "avx512vl")):
            _ref = False
            return None
        R = C.CDLL(_REF_SO)
        R.sp_moe_cpu_init.argtypes = [C.c_int]
        R.sp_moe_cpu_quant.argtypes = [f32p, C.c_int, i8p, f32p]
        R.sp_moe_cpu_gemv.argtypes = [u8p, u16p, C.c_int, C.c_int, i8p, f32p, f32p]
        R.sp_moe_cpu_expert.argtypes = [f32p, C.c_int, C.c_int, u8p, u16p, u8p, u16p, f32p]
        if R.sp_moe_cpu_init(nthreads) != 1:
            _ref = False
            return None
        _ref = R
    return _ref or None


def use_reference_gemv(threads):
    """Route the checker's decode-arithmetic quantisation and GEMVs through the reference's own
    sp_moe_cpu_quant / sp_moe_cpu_gemv (its thread pool, `threads` workers). Returns "reference",
    or "port" when oracle/_ref is unavailable and the restatement (OpenMP) runs instead."""
    R = ref_lib(threads)
    if R is None:
        lib().orc_set_backend(None, None)
        lib().orc_set_threads(threads)
        return "port"
    lib().orc_set_backend(C.cast(R.sp_moe_cpu_quant, C.c_void_p), C.cast(R.sp_moe_cpu_gemv, C.c_void_p))
    return "reference"


def use_port_gemv():
    lib().orc_set_backend(None, None)


def p(a, t):
    return a.ctypes.data_as(t)


def c32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ---------------------------------------------------------------- numpy-facing wrappers
def quant_act(x):
    x = c32(x)
    qx = np.empty(x.size, np.int8)
    sx = np.empty(x.size // 16, np.float32)
    lib().orc_quant_act_int8(p(x, f32p), x.size, p(qx, i8p), p(sx, f32p))
    return qx, sx


def gemv_a(codes, bs, rows, cols, qx, sx):
    y = np.empty(rows, np.float32)
    lib().orc_gemv_q4b_a(p(codes, u8p), p(bs, u16p), cols, rows, p(qx, i8p), p(sx, f32p), p(y, f32p))
    return y


def gemv_b(codes, bs, rows, cols, x):
    x = c32(x)
    y = np.empty(rows, np.float32)
    lib().orc_gemv_q4b_b(p(codes, u8p), p(bs, u16p), cols, rows, p(x, f32p), p(y, f32p))
    return y


def q4b_quantize(w):
    w = c32(w)
    rows, cols = w.shape
    codes = np.empty((rows, cols // 2), np.uint8)
    bs = np.empty((rows, cols // 32), np.uint16)
    lib().orc_q4b_quantize(p(w, f32p), rows, cols, p(codes, u8p), p(bs, u16p))
    return codes, bs


def int_gemm_scaled(A, B, scale_a, scale_b):
    """A [M][K], B [N][K] int8 -> C [M][N] f16 bits (uint16): f16(float(A.B^T) * sa[m] * sb[n])."""
    A = np.ascontiguousarray(A, np.int8); B = np.ascontiguousarray(B, np.int8)
    M, K = A.shape; N = B.shape[0]
    Cq = np.empty((M, N), np.uint16)
    lib().orc_int_gemm_scaled(p(A, i8p), p(B, i8p), M, N, K, p(c32(scale_a), f32p), p(c32(scale_b), f32p), p(Cq, u16p))
    return Cq


def q4b_dequantize(codes, bs):
    rows, cols = codes.shape[0], codes.shape[1] * 2
    w = np.empty((rows, cols), np.float32)
    lib().orc_q4b_dequantize(p(codes, u8p), p(bs, u16p), rows, cols, p(w, f32p))
    return w


def topk(logits, NU):
    logits = c32(logits)
    idx = np.empty(NU, np.int32)
    wt = np.empty(NU, np.float32)
    rc = lib().orc_topk(p(logits, f32p), logits.size, NU, p(idx, i32p), p(wt, f32p))
    return rc, idx, wt


class LayerWeights:
    """One layer in the reference's host layouts; keeps the numpy arrays alive."""
    FIELDS = ("router_w", "router_scale", "router_bias", "ffn_norm", "post_ffw1", "pre_ffw2",
              "post_ffw2", "post_ffw", "dexps_scale", "gu_codes", "gu_bs", "dn_codes", "dn_bs",
              "sg_codes", "sg_bs", "su_codes", "su_bs", "sd_codes", "sd_bs")

    def __init__(self, **kw):
        for f in self.FIELDS:
            v = kw.get(f)
            setattr(self, f, None if v is None else np.ascontiguousarray(v))

    def as_struct(self):
        s = OrcLayer()
        for name, typ in OrcLayer._fields_:
            a = getattr(self, name)
            setattr(s, name, C.cast(None, typ) if a is None else p(a, typ))
        return s


def layer_forward(cfg, w, x, flavour=0, want_margin=False):
    """x [M][E] -> dict(y, sel, wts, logits, margin). cfg = dict(E, NE, NU, FFE, FFS, eps)."""
    x = c32(x).reshape(-1, cfg["E"])
    M = x.shape[0]
    oc = OrcCfg(cfg["E"], cfg["NE"], cfg["NU"], cfg["FFE"], cfg["FFS"], cfg["eps"])
    y = np.empty_like(x)
    sel = np.empty((M, cfg["NU"]), np.int32)
    wts = np.empty((M, cfg["NU"]), np.float32)
    logits = np.empty((M, cfg["NE"]), np.float32)
    margin = np.empty(M, np.float64)
    st = w.as_struct()
    rc = lib().orc_layer_forward(C.byref(oc), C.byref(st), flavour, M, p(x, f32p), p(y, f32p),
                                 p(sel, i32p), p(wts, f32p), p(logits, f32p),
                                 p(margin, f64p) if want_margin else C.cast(None, f64p))
    return dict(rc=rc, y=y, sel=sel, wts=wts, logits=logits, margin=margin if want_margin else None)


def standalone_q4b(E, NE, NU, FF, eps, gate_inp, gate_inp_scale, gu_codes, gu_bs, dn_codes, dn_bs, hidden):
    out = np.empty(E, np.float32)
    sel = np.empty(NU, np.int32)
    rc = lib().orc_standalone_q4b(E, NE, NU, FF, eps, p(c32(gate_inp), f32p), p(c32(gate_inp_scale), f32p),
                                  p(gu_codes, u8p), p(gu_bs, u16p), p(dn_codes, u8p), p(dn_bs, u16p),
                                  p(c32(hidden), f32p), p(out, f32p), p(sel, i32p))
    return rc, out, sel


# ---------------------------------------------------------------- seeded synthetic layers (CPU, small)
def make_layer(cfg, seed, wstd=0.02, rand_norms=False, bias=None):
    """The benchmark's weight recipe: router N(0,0.02) f32; expert/shared weights N(0,0.02) then Q4B;
    scales and norm weights 1 (or uniform [0.5,1.5] when rand_norms)."""
    E, NE, FFE, FFS = cfg["E"], cfg["NE"], cfg["FFE"], cfg["FFS"]
    r = np.random.default_rng(seed)
    vec = (lambda n: r.uniform(0.5, 1.5, n).astype(np.float32)) if rand_norms else (lambda n: np.ones(n, np.float32))
    router_w = (r.standard_normal((NE, E)) * 0.02).astype(np.float32)
    gu_codes, gu_bs = q4b_quantize((r.standard_normal((NE * 2 * FFE, E)) * wstd).astype(np.float32))
    dn_codes, dn_bs = q4b_quantize((r.standard_normal((NE * E, FFE)) * wstd).astype(np.float32))
    sg_codes, sg_bs = q4b_quantize((r.standard_normal((FFS, E)) * wstd).astype(np.float32))
    su_codes, su_bs = q4b_quantize((r.standard_normal((FFS, E)) * wstd).astype(np.float32))
    sd_codes, sd_bs = q4b_quantize((r.standard_normal((E, FFS)) * wstd).astype(np.float32))
    return LayerWeights(router_w=router_w, router_scale=vec(E), router_bias=bias, ffn_norm=vec(E),
                        post_ffw1=vec(E), pre_ffw2=vec(E), post_ffw2=vec(E), post_ffw=vec(E),
                        dexps_scale=vec(NE), gu_codes=gu_codes, gu_bs=gu_bs, dn_codes=dn_codes,
                        dn_bs=dn_bs, sg_codes=sg_codes, sg_bs=sg_bs, su_codes=su_codes, su_bs=su_bs,
                        sd_codes=sd_codes, sd_bs=sd_bs)


TINY = dict(E=128, NE=8, NU=2, FFE=32, FFS=64, eps=1e-6)
SMALL = dict(E=256, NE=16, NU=4, FFE=64, FFS=128, eps=1e-6)
GEMMA = dict(E=2816, NE=128, NU=8, FFE=704, FFS=2112, eps=1e-6)
