"""Weight formats of the MoE layer, restated in NumPy.  TEST INFRASTRUCTURE ONLY
(used by tests/, the smoke check and bench.py's input generator; the shipped
library never imports it).

The reference defines the bytes of a quantised tensor in its converter:

* Q8_0  (src/unlimitedocr_c/convert.py:2058-2066, 2322-2333): per row and per
  64-wide group ``scale = max|w| / 127`` in f32 (1.0 for an all-zero group),
  ``q = clip(rint(w / scale), -127, 127)`` as int8; the scale is stored as fp16
  *after* it was used, so dequantisation is ``q * float(f16(scale))``.
* Q4_0  (src/unlimitedocr_c/convert.py:2249-2276): per group take the element
  of largest magnitude with its sign, ``scale = f16(signed_max / -8)``; the
  rounded fp16 value is what divides the weights (a zero scale divides by 1),
  ``q = clip(rint(w / scale), -8, 7)``, stored as ``q + 8`` with the half-split
  packing: byte ``j`` (0..31) of a group = ``(q[j]+8) | (q[j+32]+8) << 4``.
* Expert slab (src/unlimitedocr_c/convert.py:966-996; strides as the GPU host
  code derives them, src/backend/metal/uocr_metal.m:13931-13963): all routed
  experts of a layer in one packed-weight slab ``[expert][gate, up, down]`` and
  one scale slab in the same order.

tests/test_oracle_golden.py pins these functions to bytes produced by the
reference's own quantiser (tests/golden/quant_q4_q8.npz).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

GROUP = 64
QTYPE_F16, QTYPE_Q8_0, QTYPE_Q4_0 = 1, 3, 4
QTYPE_BY_NAME = {"f16": QTYPE_F16, "q8_0": QTYPE_Q8_0, "q4_0": QTYPE_Q4_0}


def quantize_q8_0(w: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """f32 [rows, cols] -> (int8 [rows, cols], fp16 scales [rows, cols/64])."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, cols = w.shape
    assert cols % GROUP == 0
    g = w.reshape(rows, cols // GROUP, GROUP)
    peak = np.max(np.abs(g), axis=2)
    scale = (peak / np.float32(127)).astype(np.float32)
    scale = np.where(peak == 0, np.float32(1), scale).astype(np.float32)
    q = np.clip(np.rint(g / scale[:, :, None]), -127, 127).astype(np.int8)
    return q.reshape(rows, cols), scale.astype("<f2")


def quantize_q4_0(w: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """f32 [rows, cols] -> (packed u8 [rows, cols/2], fp16 scales [rows, cols/64])."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, cols = w.shape
    assert cols % GROUP == 0
    g = w.reshape(rows, cols // GROUP, GROUP)
    where = np.argmax(np.abs(g), axis=2)
    signed_peak = np.take_along_axis(g, where[:, :, None], axis=2)[:, :, 0]
    scale16 = (signed_peak / np.float32(-8)).astype("<f2")
    scale = scale16.astype(np.float32)
    divisor = np.where(scale == 0, np.float32(1), scale)
    q = np.clip(np.rint(g / divisor[:, :, None]), -8, 7).astype(np.int16)
    stored = (q + 8).astype(np.uint8)
    packed = stored[:, :, : GROUP // 2] | (stored[:, :, GROUP // 2 :] << 4)
    return packed.reshape(rows, cols // 2).astype(np.uint8), scale16


def unpack_q4_0(packed: np.ndarray) -> np.ndarray:
    """packed u8 [rows, cols/2] -> signed levels int8 [rows, cols]."""
    rows, half_cols = packed.shape
    p = packed.reshape(rows, half_cols // (GROUP // 2), GROUP // 2)
    lo = (p & 15).astype(np.int8) - 8
    hi = (p >> 4).astype(np.int8) - 8
    return np.concatenate([lo, hi], axis=2).reshape(rows, half_cols * 2)


def dequantize(qtype: int, qweight: np.ndarray, qscale: np.ndarray | None) -> np.ndarray:
    """The f32 values the format defines: level * float(fp16 scale)."""
    if qtype == QTYPE_F16:
        return qweight.view("<f2").astype(np.float32)
    levels = qweight.astype(np.float32) if qtype == QTYPE_Q8_0 else unpack_q4_0(qweight).astype(np.float32)
    rows, cols = levels.shape
    s = qscale.astype(np.float32)
    return (levels.reshape(rows, cols // GROUP, GROUP) * s[:, :, None]).reshape(rows, cols)


def quantize(qtype: int, w: np.ndarray) -> tuple[np.ndarray, np.ndarray | None]:
    if qtype == QTYPE_F16:
        return np.ascontiguousarray(w, dtype=np.float32).astype("<f2").view(np.uint16), None
    if qtype == QTYPE_Q8_0:
        return quantize_q8_0(w)
    if qtype == QTYPE_Q4_0:
        return quantize_q4_0(w)
    raise ValueError(f"unknown qtype {qtype}")


def packed_row_bytes(qtype: int, cols: int) -> int:
    return {QTYPE_F16: 2 * cols, QTYPE_Q8_0: cols, QTYPE_Q4_0: cols // 2}[qtype]


@dataclass
class Matrix:
    """One projection in model-file form."""

    qtype: int
    rows: int
    cols: int
    qweight: np.ndarray            # uint8 bytes, C-contiguous
    qscale: np.ndarray | None      # uint16 (fp16 bits) [rows, cols/64]

    def to_f32(self) -> np.ndarray:
        if self.qtype == QTYPE_F16:
            return self.qweight.view("<f2").reshape(self.rows, self.cols).astype(np.float32)
        body = self.qweight.reshape(self.rows, -1)
        if self.qtype == QTYPE_Q8_0:
            body = body.view(np.int8)
        return dequantize(self.qtype, body, self.qscale.view("<f2").reshape(self.rows, -1))


def make_matrix(qtype: int, w: np.ndarray) -> Matrix:
    qw, qs = quantize(qtype, w)
    return Matrix(qtype, w.shape[0], w.shape[1], np.ascontiguousarray(qw).view(np.uint8).reshape(-1),
                  None if qs is None else np.ascontiguousarray(qs).view(np.uint16))


@dataclass
class LayerWeights:
    """One MoE layer in the model file's layout."""

    H: int
    E: int
    K: int
    F: int
    S: int
    scaling: float
    router: np.ndarray                 # uint16 fp16 bits [E, H]
    expert_qtype: int
    expert_qweight: np.ndarray         # uint8 slab
    expert_qscale: np.ndarray | None   # uint16 slab
    shared_gate: Matrix
    shared_up: Matrix
    shared_down: Matrix
    logit_bias: np.ndarray | None = None   # f32 [E]; synthetic load skew only
    meta: dict = field(default_factory=dict)

    def expert_stride_bytes(self) -> int:
        return 3 * self.F * packed_row_bytes(self.expert_qtype, self.H)

    def expert_scale_stride(self) -> int:
        return 0 if self.expert_qtype == QTYPE_F16 else 3 * self.F * (self.H // GROUP)

    def expert_f32(self, e: int) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
        """Dequantised (gate [F,H], up [F,H], down [H,F]) of expert e."""
        H, F, qt = self.H, self.F, self.expert_qtype
        proj = F * packed_row_bytes(qt, H)
        base = e * 3 * proj
        nsc = 0 if qt == QTYPE_F16 else F * (H // GROUP)
        out = []
        for p, (r, c) in enumerate(((F, H), (F, H), (H, F))):
            qw = self.expert_qweight[base + p * proj : base + (p + 1) * proj]
            qs = None if qt == QTYPE_F16 else self.expert_qscale[e * 3 * nsc + p * nsc : e * 3 * nsc + (p + 1) * nsc]
            out.append(Matrix(qt, r, c, qw, qs).to_f32())
        return tuple(out)


def synth_layer(rng: np.random.Generator, *, H: int, E: int, K: int, F: int, S: int, expert_qtype: int,
                shared_qtype: int | None = None, std: float = 0.02, scaling: float = 1.0,
                logit_bias: np.ndarray | None = None) -> LayerWeights:
    """Seeded synthetic layer: weights N(0, std) quantised with the reference's rules."""
    shared_qtype = expert_qtype if shared_qtype is None else shared_qtype
    router = (rng.standard_normal((E, H), dtype=np.float32) * np.float32(std)).astype("<f2").view(np.uint16)
    proj = F * packed_row_bytes(expert_qtype, H)
    nsc = 0 if expert_qtype == QTYPE_F16 else F * (H // GROUP)
    slab = np.empty(E * 3 * proj, dtype=np.uint8)
    scales = None if expert_qtype == QTYPE_F16 else np.empty(E * 3 * nsc, dtype=np.uint16)

    def pack(job):
        idx, w = job
        qw, qs = quantize(expert_qtype, w)
        slab[idx * proj : (idx + 1) * proj] = np.ascontiguousarray(qw).view(np.uint8).reshape(-1)
        if scales is not None:
            scales[idx * nsc : (idx + 1) * nsc] = np.ascontiguousarray(qs).view(np.uint16).reshape(-1)

    def draws():   # random draws stay sequential (fixed order); quantisation of each matrix runs on a worker
        for e in range(E):
            for p, (r, c) in enumerate(((F, H), (F, H), (H, F))):
                yield e * 3 + p, rng.standard_normal((r, c), dtype=np.float32) * np.float32(std)

    if E * F * H >= 1 << 22:
        from concurrent.futures import ThreadPoolExecutor
        import os
        workers = min(16, len(os.sched_getaffinity(0)))
        with ThreadPoolExecutor(workers) as pool:
            pending = []
            for job in draws():
                pending.append(pool.submit(pack, job))
                if len(pending) > 2 * workers:
                    pending.pop(0).result()
            for f in pending:
                f.result()
    else:
        for job in draws():
            pack(job)
    sg = make_matrix(shared_qtype, rng.standard_normal((S, H), dtype=np.float32) * np.float32(std))
    su = make_matrix(shared_qtype, rng.standard_normal((S, H), dtype=np.float32) * np.float32(std))
    sd = make_matrix(shared_qtype, rng.standard_normal((H, S), dtype=np.float32) * np.float32(std))
    return LayerWeights(H, E, K, F, S, float(scaling), router, expert_qtype, slab, scales, sg, su, sd,
                        None if logit_bias is None else np.ascontiguousarray(logit_bias, dtype=np.float32))


def permute_experts(L: LayerWeights, order: np.ndarray) -> LayerWeights:
    """The same layer with its experts relabelled: slot s of the result holds expert order[s] of L (router row, logit
    bias, packed weights and scales move together).  Every token's output is unchanged up to the summation order of
    the softmax denominator (and exact probability ties, which go to the lower label); the reported ids are slots."""
    order = np.asarray(order, np.int64)
    assert sorted(order.tolist()) == list(range(L.E))
    proj = L.F * packed_row_bytes(L.expert_qtype, L.H)
    nsc = 0 if L.expert_qtype == QTYPE_F16 else L.F * (L.H // GROUP)
    slab = L.expert_qweight.reshape(L.E, 3 * proj)[order].reshape(-1)
    scales = None if L.expert_qscale is None else L.expert_qscale.reshape(L.E, 3 * nsc)[order].reshape(-1)
    return LayerWeights(L.H, L.E, L.K, L.F, L.S, L.scaling, np.ascontiguousarray(L.router.reshape(L.E, L.H)[order]), L.expert_qtype,
                        np.ascontiguousarray(slab), None if scales is None else np.ascontiguousarray(scales), L.shared_gate,
                        L.shared_up, L.shared_down, None if L.logit_bias is None else np.ascontiguousarray(L.logit_bias[order]),
                        dict(L.meta))


def synth_activations(rng: np.random.Generator, rows: int, H: int) -> np.ndarray:
    """fp16 N(0,1) activations as uint16 bits [rows, H]."""
    return rng.standard_normal((rows, H), dtype=np.float32).astype("<f2").view(np.uint16)


def zipf_logit_bias(rng: np.random.Generator, E: int, s: float = 1.1) -> np.ndarray:
    """log of a Zipf(s) popularity over a seeded permutation of the experts."""
    ranks = rng.permutation(E).astype(np.float64) + 1.0
    p = ranks ** (-s)
    return np.log(p / p.sum()).astype(np.float32)


def stable_dispatch_plan(ids: np.ndarray, E: int) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """NumPy statement of the stable expert-sorted permutation (see mo_dispatch_plan)."""
    flat = ids.reshape(-1).astype(np.int64)
    valid = flat < E
    counts = np.bincount(flat[valid], minlength=E)
    offsets = np.zeros(E + 1, dtype=np.uint32)
    offsets[1:] = np.cumsum(counts)
    order = np.argsort(np.where(valid, flat, E), kind="stable")
    pair_rows = order[: int(valid.sum())].astype(np.uint32)
    inverse = np.full(flat.shape[0], 0xFFFFFFFF, dtype=np.uint32)
    inverse[pair_rows] = np.arange(pair_rows.shape[0], dtype=np.uint32)
    return offsets, pair_rows, inverse
