"""ctypes front end of the CPU checkers.  TEST INFRASTRUCTURE ONLY: imported by
tests/, the smoke check and bench.py's CPU-baseline legs, never by the library.

Two backends with one interface:

* ``Port``  - oracle/libmoe_oracle.so, this repository's restatement.
* ``Ref``   - oracle/_ref/libuocr_cpu_ref.so, the reference's own
  ``uocr_cpu_ref_moe_router_f32`` / ``uocr_cpu_ref_moe_swiglu_f32``
  (src/backend/cpu_ref/uocr_cpu_ref.h:57-90) compiled unmodified.  It only
  understands f32 weights, so quantised layers are dequantised first.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

from . import quant

HERE = Path(__file__).resolve().parent
PORT_LIB = HERE / "libmoe_oracle.so"
REF_LIB = HERE / "_ref" / "libuocr_cpu_ref.so"

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")


def build(force: bool = False) -> None:
    """Compile the checkers (``make -C oracle``); the reference build is skipped when its tree is absent."""
    if force or not PORT_LIB.exists() or PORT_LIB.stat().st_mtime < (HERE / "moe_oracle.c").stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "libmoe_oracle.so"], check=True, capture_output=True)
    if force or not all((REF_LIB.parent / name).exists() for name in ("libuocr_cpu_ref.so", "libuocr_model_file.so", "libunlimitedocr_cuda.so")):
        subprocess.run(["make", "-C", str(HERE), "ref"], check=True, capture_output=True)


class _Matrix(C.Structure):
    _fields_ = [("qtype", C.c_int32), ("rows", C.c_uint32), ("cols", C.c_uint32), ("qweight", C.c_void_p),
                ("qscale", C.c_void_p), ("through_f16", C.c_int32)]


class _Layer(C.Structure):
    _fields_ = [("H", C.c_uint32), ("E", C.c_uint32), ("K", C.c_uint32), ("F", C.c_uint32), ("S", C.c_uint32),
                ("scaling", C.c_float), ("router_f16", C.c_void_p), ("logit_bias", C.c_void_p),
                ("expert_qtype", C.c_int32), ("expert_qweight", C.c_void_p), ("expert_qscale", C.c_void_p),
                ("shared_gate", _Matrix), ("shared_up", _Matrix), ("shared_down", _Matrix)]


def _ptr(a: np.ndarray | None) -> int | None:
    return None if a is None else a.ctypes.data


def _cmatrix(m: quant.Matrix, through_f16: bool = False) -> _Matrix:
    return _Matrix(m.qtype, m.rows, m.cols, _ptr(m.qweight), _ptr(m.qscale), int(through_f16))


class RouterOut:
    def __init__(self, rows: int, E: int, K: int):
        self.logits = np.zeros((rows, E), np.float32)
        self.probs = np.zeros((rows, E), np.float32)
        self.ids = np.full((rows, K), 0xFFFFFFFF, np.uint32)
        self.weights = np.zeros((rows, K), np.float32)


class LayerOut(RouterOut):
    def __init__(self, rows: int, H: int, E: int, K: int, F: int, S: int):
        super().__init__(rows, E, K)
        self.expert_ws = np.zeros((rows, K, F), np.float32)
        self.shared_ws = np.zeros((rows, S), np.float32)
        self.out = np.zeros((rows, H), np.float32)


class Port:
    """This repository's C restatement."""

    kind = "port"

    def __init__(self) -> None:
        build()
        lib = C.CDLL(str(PORT_LIB))
        lib.mo_f16_to_f32.restype = C.c_float
        lib.mo_f16_to_f32.argtypes = [C.c_uint16]
        lib.mo_f32_to_f16.restype = C.c_uint16
        lib.mo_f32_to_f16.argtypes = [C.c_float]
        lib.mo_f16_to_f32_array.argtypes = [_u16p, C.c_size_t, _f32p]
        lib.mo_f32_to_f16_array.argtypes = [_f32p, C.c_size_t, _u16p]
        lib.mo_router_f32.argtypes = [C.c_void_p, C.c_void_p] + [C.c_uint32] * 4 + [C.c_float] + [C.c_void_p] * 4
        lib.mo_route_from_logits_f32.argtypes = [_f32p] + [C.c_uint32] * 3 + [C.c_float, _f32p, _u32p, _f32p]
        lib.mo_dense_swiglu_f32.argtypes = [_f32p] * 4 + [C.c_uint32] * 3 + [_f32p] * 2
        lib.mo_rmsnorm_f32.argtypes = [_f32p, _f32p, C.c_uint32, C.c_uint32, C.c_float, _f32p]
        lib.mo_rmsnorm_f16.argtypes = [_u16p, _u16p, C.c_uint32, C.c_uint32, C.c_float, _u16p]
        lib.mo_layer_f32.argtypes = [C.c_void_p] * 8 + [C.c_uint32] * 6 + [C.c_float] + [C.c_void_p] * 7
        lib.mo_layer_slab.argtypes = [C.POINTER(_Layer), C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_int] + \
            [C.c_void_p] * 7
        lib.mo_dispatch_plan.argtypes = [_u32p] + [C.c_uint32] * 3 + [_u32p] * 3
        lib.mo_dequant_matrix.argtypes = [C.POINTER(_Matrix), _f32p]
        lib.mo_lm_head_argmax.argtypes = [C.POINTER(_Matrix), _u16p, C.c_uint32, _u32p, _f32p, C.c_void_p]
        self.lib = lib

    # -- conversions
    def f16_to_f32(self, bits: np.ndarray) -> np.ndarray:
        bits = np.ascontiguousarray(bits, np.uint16)
        out = np.empty(bits.shape, np.float32)
        assert self.lib.mo_f16_to_f32_array(bits.reshape(-1), bits.size, out.reshape(-1)) == 1
        return out

    def f32_to_f16(self, vals: np.ndarray) -> np.ndarray:
        vals = np.ascontiguousarray(vals, np.float32)
        out = np.empty(vals.shape, np.uint16)
        assert self.lib.mo_f32_to_f16_array(vals.reshape(-1), vals.size, out.reshape(-1)) == 1
        return out

    # -- reference-shaped calls (f32 weights); return (status, outputs)
    def router_f32(self, x, w, K: int, scaling: float = 1.0, *, raw_args=None):
        rows, H = x.shape
        E = w.shape[0]
        o = RouterOut(rows, E, K)
        st = self.lib.mo_router_f32(_ptr(x), _ptr(w), rows, H, E, K, scaling, _ptr(o.logits), _ptr(o.probs),
                                    _ptr(o.ids), _ptr(o.weights))
        return st, o

    def route_from_logits(self, logits: np.ndarray, K: int, scaling: float = 1.0):
        logits = np.ascontiguousarray(logits, np.float32)
        rows, E = logits.shape
        o = RouterOut(rows, E, K)
        o.logits = logits
        st = self.lib.mo_route_from_logits_f32(logits, rows, E, K, scaling, o.probs, o.ids, o.weights)
        return st, o

    def layer_f32(self, x, router, eg, eu, ed, sg, su, sd, K: int, scaling: float = 1.0):
        rows, H = x.shape
        E, F = eg.shape[0], eg.shape[1]
        S = sg.shape[0]
        o = LayerOut(rows, H, E, K, F, S)
        st = self.lib.mo_layer_f32(_ptr(x), _ptr(router), _ptr(eg), _ptr(eu), _ptr(ed), _ptr(sg), _ptr(su), _ptr(sd),
                                   rows, H, E, K, F, S, scaling, _ptr(o.logits), _ptr(o.probs), _ptr(o.ids),
                                   _ptr(o.weights), _ptr(o.expert_ws), _ptr(o.shared_ws), _ptr(o.out))
        return st, o

    def dense_swiglu_f32(self, x, gate, up, down):
        rows, H = x.shape
        F = gate.shape[0]
        mid = np.zeros((rows, F), np.float32)
        out = np.zeros((rows, H), np.float32)
        st = self.lib.mo_dense_swiglu_f32(x, gate, up, down, rows, H, F, mid, out)
        return st, mid, out

    def lm_head_argmax(self, m: quant.Matrix, x_bits: np.ndarray, want_logits: bool = False):
        """(ids uint32 [rows], scores f32 [rows], logits f32 [rows, vocab] or None): the LM head's argmax per token."""
        x_bits = np.ascontiguousarray(x_bits, np.uint16)
        rows = x_bits.shape[0]
        ids = np.zeros(rows, np.uint32)
        scores = np.zeros(rows, np.float32)
        logits = np.zeros((rows, m.rows), np.float32) if want_logits else None
        cm = _cmatrix(m)
        assert self.lib.mo_lm_head_argmax(C.byref(cm), x_bits, rows, ids, scores, _ptr(logits)) == 1
        return ids, scores, logits

    def rmsnorm_f32(self, x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros_like(x)
        assert self.lib.mo_rmsnorm_f32(x, np.ascontiguousarray(weight, np.float32), x.shape[0], x.shape[1], eps, out) == 1
        return out

    def rmsnorm_f16(self, x_bits: np.ndarray, weight_bits: np.ndarray, eps: float) -> np.ndarray:
        """fp16 bits in, fp16 bits out: the GPU path's form (f32 arithmetic, one rounding)."""
        x_bits = np.ascontiguousarray(x_bits, np.uint16)
        out = np.zeros_like(x_bits)
        assert self.lib.mo_rmsnorm_f16(x_bits, np.ascontiguousarray(weight_bits, np.uint16), x_bits.shape[0], x_bits.shape[1], eps, out) == 1
        return out

    # -- model-format call
    def layer(self, L: quant.LayerWeights, hidden: np.ndarray, residual: np.ndarray | None = None, *,
              injected_logits: np.ndarray | None = None, round_mid_f16: bool | int = False, weights_through_f16: bool = False,
              threads: int = 1) -> LayerOut:
        """round_mid_f16: bits selecting fp16 roundings: 1 the SwiGLU products, 2 the per-expert down products,
        4 the shared MLP's output, 8 the weighted routed sum (1|2|4: the tiled-GEMM contract, 1|4|8: the
        reference's NumPy fp16 contract); weights_through_f16 rounds every dequantised weight to fp16."""
        hidden = np.ascontiguousarray(hidden, np.uint16)
        rows = hidden.shape[0]
        o = LayerOut(rows, L.H, L.E, L.K, L.F, L.S)
        cl = _Layer(L.H, L.E, L.K, L.F, L.S, L.scaling, _ptr(L.router), _ptr(L.logit_bias), L.expert_qtype,
                    _ptr(L.expert_qweight), _ptr(L.expert_qscale), _cmatrix(L.shared_gate, weights_through_f16),
                    _cmatrix(L.shared_up, weights_through_f16), _cmatrix(L.shared_down, weights_through_f16))
        if residual is not None:
            residual = np.ascontiguousarray(residual, np.uint16)
        if injected_logits is not None:
            injected_logits = np.ascontiguousarray(injected_logits, np.float32)

        def run(lo: int, hi: int) -> int:
            return self.lib.mo_layer_slab(
                C.byref(cl), _ptr(hidden[lo:hi]), None if residual is None else _ptr(residual[lo:hi]),
                None if injected_logits is None else _ptr(injected_logits[lo:hi]), hi - lo, int(round_mid_f16),
                _ptr(o.logits[lo:hi]), _ptr(o.probs[lo:hi]), _ptr(o.ids[lo:hi]), _ptr(o.weights[lo:hi]),
                _ptr(o.expert_ws[lo:hi]), _ptr(o.shared_ws[lo:hi]), _ptr(o.out[lo:hi]))

        _run_sliced(run, rows, threads)
        return o

    def dispatch_plan(self, ids: np.ndarray, E: int):
        ids = np.ascontiguousarray(ids, np.uint32)
        rows, K = ids.shape
        offsets = np.zeros(E + 1, np.uint32)
        pair_rows = np.full(rows * K, 0xFFFFFFFF, np.uint32)
        inverse = np.zeros(rows * K, np.uint32)
        assert self.lib.mo_dispatch_plan(ids.reshape(-1), rows, K, E, offsets, pair_rows, inverse) == 1
        return offsets, pair_rows[: int(offsets[E])], inverse


def _run_sliced(run, rows: int, threads: int) -> None:
    threads = max(1, min(threads, rows))
    bounds = np.linspace(0, rows, threads + 1).astype(int)
    if threads == 1:
        assert run(0, rows) == 1, "oracle rejected its inputs"
        return
    with ThreadPoolExecutor(threads) as pool:   # ctypes releases the GIL during the call
        for st in pool.map(lambda i: run(int(bounds[i]), int(bounds[i + 1])), range(threads)):
            assert st == 1, "oracle rejected its inputs"


class Ref:
    """The reference's own CPU backend, compiled unmodified (f32 weights only)."""

    kind = "reference"

    def __init__(self) -> None:
        build()
        if not REF_LIB.exists():
            raise FileNotFoundError(f"{REF_LIB} not built (reference tree absent at build time)")
        lib = C.CDLL(str(REF_LIB))
        lib.uocr_cpu_ref_f16_bits_to_f32.restype = C.c_float
        lib.uocr_cpu_ref_f16_bits_to_f32.argtypes = [C.c_uint16]
        lib.uocr_cpu_ref_f32_to_f16_bits.restype = C.c_uint16
        lib.uocr_cpu_ref_f32_to_f16_bits.argtypes = [C.c_float]
        lib.uocr_cpu_ref_f16_to_f32_array.argtypes = [_u16p, C.c_size_t, _f32p]
        lib.uocr_cpu_ref_f32_to_f16_array.argtypes = [_f32p, C.c_size_t, _u16p]
        lib.uocr_cpu_ref_moe_router_f32.argtypes = [C.c_void_p, C.c_void_p] + [C.c_uint32] * 4 + [C.c_float] + \
            [C.c_void_p] * 4
        lib.uocr_cpu_ref_moe_swiglu_f32.argtypes = [C.c_void_p] * 8 + [C.c_uint32] * 6 + [C.c_float] + [C.c_void_p] * 7
        lib.uocr_cpu_ref_dense_swiglu_f32.argtypes = [_f32p] * 4 + [C.c_uint32] * 3 + [_f32p] * 2
        lib.uocr_cpu_ref_rmsnorm_f32.argtypes = [_f32p, _f32p, C.c_uint32, C.c_uint32, C.c_float, _f32p]
        self.lib = lib

    def f16_to_f32(self, bits):
        bits = np.ascontiguousarray(bits, np.uint16)
        out = np.empty(bits.shape, np.float32)
        assert self.lib.uocr_cpu_ref_f16_to_f32_array(bits.reshape(-1), bits.size, out.reshape(-1)) == 1
        return out

    def f32_to_f16(self, vals):
        vals = np.ascontiguousarray(vals, np.float32)
        out = np.empty(vals.shape, np.uint16)
        assert self.lib.uocr_cpu_ref_f32_to_f16_array(vals.reshape(-1), vals.size, out.reshape(-1)) == 1
        return out

    def router_f32(self, x, w, K: int, scaling: float = 1.0):
        rows, H = x.shape
        E = w.shape[0]
        o = RouterOut(rows, E, K)
        st = self.lib.uocr_cpu_ref_moe_router_f32(_ptr(x), _ptr(w), rows, H, E, K, scaling, _ptr(o.logits),
                                                  _ptr(o.probs), _ptr(o.ids), _ptr(o.weights))
        return st, o

    def route_from_logits(self, logits: np.ndarray, K: int, scaling: float = 1.0):
        """The unmodified router fed an identity weight matrix reproduces the given logits exactly."""
        logits = np.ascontiguousarray(logits, np.float32)
        E = logits.shape[1]
        return self.router_f32(logits, np.eye(E, dtype=np.float32), K, scaling)

    def layer_f32(self, x, router, eg, eu, ed, sg, su, sd, K: int, scaling: float = 1.0, threads: int = 1):
        rows, H = x.shape
        E, F = eg.shape[0], eg.shape[1]
        S = sg.shape[0]
        o = LayerOut(rows, H, E, K, F, S)

        def run(lo: int, hi: int) -> int:
            return self.lib.uocr_cpu_ref_moe_swiglu_f32(
                _ptr(x[lo:hi]), _ptr(router), _ptr(eg), _ptr(eu), _ptr(ed), _ptr(sg), _ptr(su), _ptr(sd), hi - lo, H,
                E, K, F, S, scaling, _ptr(o.logits[lo:hi]), _ptr(o.probs[lo:hi]), _ptr(o.ids[lo:hi]),
                _ptr(o.weights[lo:hi]), _ptr(o.expert_ws[lo:hi]), _ptr(o.shared_ws[lo:hi]), _ptr(o.out[lo:hi]))

        if threads == 1:
            return run(0, rows), o
        _run_sliced(run, rows, threads)
        return 1, o

    def dense_swiglu_f32(self, x, gate, up, down):
        rows, H = x.shape
        F = gate.shape[0]
        mid = np.zeros((rows, F), np.float32)
        out = np.zeros((rows, H), np.float32)
        st = self.lib.uocr_cpu_ref_dense_swiglu_f32(x, gate, up, down, rows, H, F, mid, out)
        return st, mid, out

    def rmsnorm_f32(self, x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros_like(x)
        assert self.lib.uocr_cpu_ref_rmsnorm_f32(x, np.ascontiguousarray(weight, np.float32), x.shape[0], x.shape[1], eps, out) == 1
        return out

    def layer(self, L: quant.LayerWeights, hidden: np.ndarray, residual: np.ndarray | None = None, *,
              threads: int = 1, f32_weights=None) -> LayerOut:
        """Dequantise the layer to f32 and run the reference layer function.  A logit bias cannot be
        expressed through the unmodified function, so biased layers are not accepted here."""
        assert L.logit_bias is None, "the reference layer function has no logit bias input"
        x = self.f16_to_f32(hidden)
        w = f32_weights if f32_weights is not None else layer_to_f32(L)
        st, o = self.layer_f32(x, *w, L.K, L.scaling, threads=threads)
        assert st == 1
        if residual is not None:
            o.out += self.f16_to_f32(residual)
        return o


def layer_to_f32(L: quant.LayerWeights):
    """(router, gate[E,F,H], up[E,F,H], down[E,H,F], shared gate/up/down) as f32, the reference function's inputs."""
    router = L.router.view("<f2").astype(np.float32)
    eg = np.empty((L.E, L.F, L.H), np.float32)
    eu = np.empty((L.E, L.F, L.H), np.float32)
    ed = np.empty((L.E, L.H, L.F), np.float32)
    for e in range(L.E):
        eg[e], eu[e], ed[e] = L.expert_f32(e)
    return router, eg, eu, ed, L.shared_gate.to_f32(), L.shared_up.to_f32(), L.shared_down.to_f32()


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1
