"""Pins the CPU oracle (oracle/moe_oracle.c, oracle/quant.py) to the reference:
its committed golden vectors, its hand-computed unit-test cases, bytes from its
quantisers, and outputs of its CPU layer function.  No GPU involved."""
import json
import sys

import numpy as np
import pytest

sys.path.insert(0, str(__import__("pathlib").Path(__file__).resolve().parent / "golden"))
from oracle import quant  # noqa: E402
from oracle.oracle import layer_to_f32  # noqa: E402

import make_golden  # noqa: E402  (fixture shapes and seeds only; its main() is not run)


def f32(a):
    return np.ascontiguousarray(a, np.float32)


# ------------------------------------------------------------ half conversions

def test_f16_known_answers(port):
    # the reference's conversion KATs (tests/test_cpu_ref.c:39-71)
    to16 = lambda v: int(port.f32_to_f16(f32([v]))[0])
    to32 = lambda b: float(port.f16_to_f32(np.array([b], np.uint16))[0])
    assert to32(0x3C00) == 1.0 and to32(0xC000) == -2.0
    assert to16(0.0) == 0x0000 and to16(-0.0) == 0x8000
    assert to16(1.0) == 0x3C00 and to16(-2.0) == 0xC000 and to16(0.5) == 0x3800
    assert to16(65504.0) == 0x7BFF and to16(np.inf) == 0x7C00
    assert to16(np.nan) & 0x7C00 == 0x7C00
    assert to32(0x7BFF) == 65504.0


def test_f16_matches_numpy_everywhere(port):
    bits = np.arange(65536, dtype=np.uint16)
    mine = port.f16_to_f32(bits)
    theirs = bits.view("<f2").astype(np.float32)
    finite = np.isfinite(theirs)
    assert np.array_equal(mine[finite], theirs[finite])
    assert np.array_equal(np.isnan(mine), np.isnan(theirs))
    rng = np.random.default_rng(1)
    vals = np.concatenate([
        rng.standard_normal(200000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 200000).astype(np.float32),
        mine[finite],                                             # every half, exactly
        np.nextafter(mine[finite], np.float32(np.inf)),            # and its f32 neighbours
        f32([65519.99, 65520.0, 65535.0, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0000001, 2.0 ** -26, 1e-45, -1e-45]),
    ]).astype(np.float32)
    with np.errstate(over="ignore"):
        want = vals.astype("<f2").view(np.uint16)
    assert np.array_equal(port.f32_to_f16(vals), want)


def test_f16_matches_reference_build(port, ref):
    bits = np.arange(65536, dtype=np.uint16)
    a, b = port.f16_to_f32(bits), ref.f16_to_f32(bits)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    rng = np.random.default_rng(2)
    vals = rng.integers(0, 2 ** 32, 1 << 20, dtype=np.uint64).astype(np.uint32).view(np.float32)
    assert np.array_equal(port.f32_to_f16(vals), ref.f32_to_f16(vals))


# ------------------------------------------------------- reference golden vectors

@pytest.fixture(scope="module")
def tiny(golden_dir):
    return json.loads((golden_dir / "cpu_ref_tiny_moe.json").read_text())


def _close(a, b, tol):
    return np.max(np.abs(f32(a).reshape(-1) - f32(b).reshape(-1))) <= tol


@pytest.mark.parametrize("which", ["port", "ref"])
def test_reference_golden_moe_layer(which, tiny, request):
    impl = request.getfixturevalue(which)
    g = lambda k: tiny["UOCR_TINY_MOE_" + k]
    rows, H, E, K = g("ROWS"), g("HIDDEN"), g("EXPERTS"), g("TOPK")
    F, S = g("EXPERT_INTERMEDIATE"), g("SHARED_INTERMEDIATE")
    st, o = impl.layer_f32(f32(g("INPUT")).reshape(rows, H), f32(g("ROUTER")).reshape(E, H),
                           f32(g("EXPERT_GATE")).reshape(E, F, H), f32(g("EXPERT_UP")).reshape(E, F, H),
                           f32(g("EXPERT_DOWN")).reshape(E, H, F), f32(g("SHARED_GATE")).reshape(S, H),
                           f32(g("SHARED_UP")).reshape(S, H), f32(g("SHARED_DOWN")).reshape(H, S), K, g("SCALING"))
    assert st == 1
    # tolerances of tests/test_cpu_ref.c:590-605
    assert _close(o.logits, g("EXPECTED_LOGITS"), 2e-5)
    assert _close(o.probs, g("EXPECTED_PROBS"), 2e-5)
    assert o.ids.reshape(-1).tolist() == g("EXPECTED_TOP_IDS")       # row 0 holds an exact tie (experts 5, 6)
    assert _close(o.weights, g("EXPECTED_TOP_WEIGHTS"), 2e-5)
    assert _close(o.expert_ws, g("EXPECTED_EXPERT_WORKSPACE"), 3e-5)
    assert _close(o.shared_ws, g("EXPECTED_SHARED_WORKSPACE"), 3e-5)
    assert _close(o.out, g("EXPECTED"), 3e-5)


@pytest.mark.parametrize("which", ["port", "ref"])
def test_reference_golden_dense_swiglu(which, tiny, request):
    impl = request.getfixturevalue(which)
    g = lambda k: tiny["UOCR_TINY_SWIGLU_" + k]
    rows, H, F = g("ROWS"), g("HIDDEN"), g("INTERMEDIATE")
    st, mid, out = impl.dense_swiglu_f32(f32(g("INPUT")).reshape(rows, H), f32(g("GATE")).reshape(F, H),
                                         f32(g("UP")).reshape(F, H), f32(g("DOWN")).reshape(H, F))
    assert st == 1
    assert _close(mid, g("EXPECTED_WORKSPACE"), 2e-5) and _close(out, g("EXPECTED"), 2e-5)


@pytest.mark.parametrize("which", ["port", "ref"])
def test_hand_case_ties_and_rejections(which, request):
    """The hand-computed 2-row, 4-expert case of tests/test_cpu_ref.c:314-507."""
    impl = request.getfixturevalue(which)
    x = f32([[1, 2], [-1, 0.5]])
    router = f32([[1, 0], [0, 1], [1, 1], [-1, 0]])
    E, F, H = 4, 2, 2
    eye = np.eye(2, dtype=np.float32)
    eg = np.stack([eye] * E)
    eu = np.stack([eye * (e + 1) for e in range(E)])
    ed = np.stack([eye] * E)
    sg, su, sd = eye.copy(), f32([[2, 0], [0, 3]]), eye.copy()
    st, o = impl.layer_f32(x, router, f32(eg), f32(eu), f32(ed), sg, su, sd, 2, 1.0)
    assert st == 1
    assert np.allclose(o.logits, [[1, 2, 3, -1], [-1, 0.5, -0.5, 1]], atol=1e-6)
    assert o.ids.tolist() == [[2, 1], [3, 1]]
    silu = lambda v: v / (1 + np.exp(-v))
    for r in range(2):
        p = np.exp(o.logits[r] - o.logits[r].max())
        p /= p.sum()
        assert np.allclose(o.probs[r], p, atol=1e-6)
        assert o.weights[r].sum() < 1.0                                    # no renormalisation
        want = silu(x[r]) * np.array([2.0, 3.0]) * x[r]
        for s in range(2):
            e = o.ids[r, s]
            want = want + p[e] * silu(x[r]) * (e + 1) * x[r]
        assert np.allclose(o.out[r], want, atol=1e-5)
    # all-zero input: every expert ties, the lowest ids win in order
    st, t = impl.router_f32(f32([[0, 0]]), router, 2, 1.0)
    assert st == 1 and t.ids.tolist() == [[0, 1]] and np.allclose(t.weights, 0.25, atol=1e-6)
    # rejected arguments return 0
    assert impl.router_f32(x, router, 5, 1.0)[0] == 0            # top_k > n_experts
    assert impl.router_f32(x, router, 2, -1.0)[0] == 0           # negative scaling
    assert impl.router_f32(x, router, 2, float("nan"))[0] == 0
    assert impl.router_f32(x, router, 0, 1.0)[0] == 0


# --------------------------------------------------------------- weight formats

def test_quantisers_reproduce_reference_bytes(golden_dir):
    z = np.load(golden_dir / "quant_q4_q8.npz")
    for tag in ("a", "b"):
        vals = z[f"{tag}_values"]
        packed, scales = quant.quantize_q4_0(vals)
        assert np.array_equal(packed, z[f"{tag}_q4_packed"])
        assert np.array_equal(scales.view(np.uint16), z[f"{tag}_q4_scales"])
        assert np.array_equal(quant.dequantize(quant.QTYPE_Q4_0, packed, scales), z[f"{tag}_q4_dequant"])
        q8, s8 = quant.quantize_q8_0(vals)
        assert np.array_equal(q8, z[f"{tag}_q8_weight"])
        assert np.array_equal(s8.view(np.uint16), z[f"{tag}_q8_scales"])
    # edge cases of tests/test_convert.py:192-218
    a, deq = z["a_values"], z["a_q4_dequant"]
    assert np.all(deq[0, :64] == 0) and z["a_q4_scales"][0, 0] & 0x7FFF == 0   # 0 / -8 = -0.0
    assert abs(deq[1, 64] - np.float32(np.float16(-0.5 / -8.0)) * -8.0) < 1e-6
    lv = quant.unpack_q4_0(z["a_q4_packed"])
    assert lv.min() >= -8 and lv.max() <= 7 and lv[1, 64] == -8 and lv[2, 130] == -8
    err = np.abs(deq - a)
    assert err.max() <= np.abs(z["a_q4_scales"].view("<f2").astype(np.float32)).max() * 0.5 + 1e-6


def test_format_byte_counts():
    # src/model/uocr_format.h:53-99 and the per-expert sizes the Metal host derives
    assert quant.packed_row_bytes(quant.QTYPE_Q4_0, 1280) * 896 == 896 * 640
    rng = np.random.default_rng(0)
    L = quant.synth_layer(rng, H=128, E=3, K=2, F=64, S=64, expert_qtype=quant.QTYPE_Q4_0)
    assert L.expert_stride_bytes() == 3 * 64 * 64 and L.expert_scale_stride() == 3 * 64 * 2
    assert L.expert_qweight.size == 3 * L.expert_stride_bytes()
    full = dict(H=1280, F=896)
    for qt, want in ((quant.QTYPE_Q8_0, 3_440_640), (quant.QTYPE_Q4_0, 1_720_320), (quant.QTYPE_F16, 6_881_280)):
        assert 3 * full["F"] * quant.packed_row_bytes(qt, full["H"]) == want


def test_c_dequant_equals_numpy(port):
    import ctypes as C
    from oracle.oracle import _cmatrix
    rng = np.random.default_rng(3)
    w = rng.standard_normal((8, 256), dtype=np.float32) * np.float32(0.02)
    for qt in (quant.QTYPE_F16, quant.QTYPE_Q8_0, quant.QTYPE_Q4_0):
        m = quant.make_matrix(qt, w)
        out = np.zeros((8, 256), np.float32)
        cm = _cmatrix(m)
        assert port.lib.mo_dequant_matrix(C.byref(cm), out.reshape(-1)) == 1
        assert np.array_equal(out, m.to_f32())


# ------------------------------------------- the layer on model-format weights

@pytest.mark.parametrize("name,qname,seed", make_golden.tiny_cases())
def test_slab_layer_equals_stored_reference_outputs(port, golden_dir, name, qname, seed):
    z = np.load(golden_dir / "ref_layers.npz")
    rng = np.random.default_rng(seed)
    L = quant.synth_layer(rng, expert_qtype=quant.QTYPE_BY_NAME[qname], **make_golden.TINY)
    hidden = quant.synth_activations(rng, make_golden.TINY_ROWS, make_golden.TINY["H"])
    o = port.layer(L, hidden)
    assert np.array_equal(o.ids, z[f"{name}_ids"])
    for key in ("logits", "probs", "weights", "expert_ws", "shared_ws", "out"):
        assert np.array_equal(getattr(o, key).view(np.uint32), z[f"{name}_{key}"].view(np.uint32)), key
    # and threading over row slices changes nothing
    o4 = port.layer(L, hidden, threads=4)
    assert np.array_equal(o4.out, o.out) and np.array_equal(o4.ids, o.ids)


def test_stored_tie_cases(port, golden_dir):
    z = np.load(golden_dir / "ref_layers.npz")
    for k in (1, 2, 3, 6):
        st, o = port.route_from_logits(z["ties_logits"], k)
        assert st == 1
        assert np.array_equal(o.ids, z[f"ties_k{k}_ids"])
        assert np.array_equal(o.weights.view(np.uint32), z[f"ties_k{k}_weights"].view(np.uint32))
    assert z["ties_k3_ids"][3].tolist() == [2, 3, 4]      # four-way tie across the boundary: lowest ids


@pytest.mark.parametrize("qname", ["f16", "q8_0", "q4_0"])
def test_slab_layer_equals_reference_build_live(port, ref, qname):
    rng = np.random.default_rng(99)
    L = quant.synth_layer(rng, H=192, E=12, K=4, F=128, S=192, expert_qtype=quant.QTYPE_BY_NAME[qname], scaling=2.5)
    hidden = quant.synth_activations(rng, 9, 192)
    resid = quant.synth_activations(rng, 9, 192)
    a = port.layer(L, hidden, resid)
    b = ref.layer(L, hidden, resid)
    assert np.array_equal(a.ids, b.ids)
    for key in ("logits", "probs", "weights", "expert_ws", "shared_ws", "out"):
        assert np.array_equal(getattr(a, key).view(np.uint32), getattr(b, key).view(np.uint32)), key
    # the f32-weights entry point agrees too
    st, c = port.layer_f32(port.f16_to_f32(hidden), *layer_to_f32(L), L.K, L.scaling)
    assert st == 1 and np.array_equal(c.expert_ws, b.expert_ws)


def test_injected_logits_and_bias(port, ref):
    rng = np.random.default_rng(5)
    bias = rng.standard_normal(16).astype(np.float32)
    L = quant.synth_layer(rng, H=128, E=16, K=3, F=64, S=64, expert_qtype=quant.QTYPE_Q8_0, logit_bias=bias)
    hidden = quant.synth_activations(rng, 7, 128)
    o = port.layer(L, hidden)
    L0 = quant.synth_layer(np.random.default_rng(5), H=128, E=16, K=3, F=64, S=64, expert_qtype=quant.QTYPE_Q8_0)
    rng2 = np.random.default_rng(5); rng2.standard_normal(16)
    plain = port.layer(L, hidden, injected_logits=None)
    assert np.array_equal(plain.ids, o.ids)
    # logits carry the bias, and routing on them through the unmodified router gives the same ids/weights
    st, r = ref.route_from_logits(o.logits, L.K, L.scaling)
    assert st == 1 and np.array_equal(r.ids, o.ids)
    assert np.array_equal(r.weights.view(np.uint32), o.weights.view(np.uint32))
    # injected logits take the place of the router dot product
    inj = rng.standard_normal((7, 16)).astype(np.float32)
    L.logit_bias = None
    q = port.layer(L, hidden, injected_logits=inj)
    st, r = ref.route_from_logits(inj, L.K, L.scaling)
    assert np.array_equal(q.logits, inj) and np.array_equal(q.ids, r.ids)


def test_round_mid_f16_is_a_small_perturbation(port):
    rng = np.random.default_rng(6)
    L = quant.synth_layer(rng, H=128, E=8, K=2, F=64, S=64, expert_qtype=quant.QTYPE_Q4_0)
    hidden = quant.synth_activations(rng, 5, 128)
    a, b = port.layer(L, hidden), port.layer(L, hidden, round_mid_f16=True)
    assert np.array_equal(a.ids, b.ids)
    assert not np.array_equal(a.out, b.out) and np.max(np.abs(a.out - b.out)) < 1e-3
    assert np.array_equal(b.expert_ws, port.f16_to_f32(port.f32_to_f16(b.expert_ws)))


# ---------------------------------------------------------------- dispatch plan

def test_dispatch_plan_is_the_stable_sort(port):
    rng = np.random.default_rng(8)
    for rows, K, E in ((1, 6, 64), (16, 2, 8), (257, 6, 64), (5, 3, 3)):
        ids = np.stack([rng.permutation(E)[:K] for _ in range(rows)]).astype(np.uint32)
        if rows > 4:
            ids[3, 1] = E + 7                                  # an invalid id is dropped
        off, pr, inv = port.dispatch_plan(ids, E)
        off2, pr2, inv2 = quant.stable_dispatch_plan(ids, E)
        assert np.array_equal(off, off2) and np.array_equal(pr, pr2) and np.array_equal(inv, inv2)
        flat = ids.reshape(-1)
        for e in range(E):
            seg = pr[off[e]:off[e + 1]]
            assert np.all(flat[seg] == e) and np.all(np.diff(seg.astype(np.int64)) > 0)
        assert off[E] == np.count_nonzero(flat < E)


def test_fp16_contract_mode_matches_the_reference_numpy_layer(port, golden_dir):
    """The oracle's fp16 roundings (SwiGLU products, routed sum, shared output: round_mid_f16 = 1|4|8) against
    the reference's own NumPy fp16-contract layer (src/unlimitedocr_c/golden.py:544-562, :649-666), whose stored
    outputs tests/golden/make_golden.py produced on the same seeded full-size fp16 layer.  The two sum in different
    orders (serial f32 chains here, BLAS there), so logits-dependent values are compared at the reference's own
    router threshold and a few outputs differ by one fp16 step of an intermediate."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", golden_dir / "make_golden.py")
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    L, hidden, resid = mg.f16_contract_inputs()
    z = np.load(golden_dir / "f16_contract.npz")
    got = port.layer(L, hidden, resid, round_mid_f16=1 | 4 | 8, threads=6)
    assert np.array_equal(got.ids, z["ids"])
    assert np.max(np.abs(got.weights - z["weights"])) <= 5e-5        # src/unlimitedocr_c/parity_thresholds.py:66-70
    assert np.max(np.abs(got.probs - z["probs"])) <= 5e-5
    got_bits = port.f32_to_f16(got.out)
    want_bits = z["out_bits"]
    # a differing element comes from ONE fp16 step of the routed sum or the shared output (both below 2 in magnitude:
    # a step of at most 2^-10) carried through the final rounding of an output below 4 (half a step of 2^-8)
    assert np.max(np.abs(port.f16_to_f32(got_bits) - port.f16_to_f32(want_bits))) <= 2.0 ** -9
    assert np.max(np.abs(port.f16_to_f32(want_bits))) < 8.0
    assert np.mean(got_bits == want_bits) >= 0.97
    # and the mode matters: without the roundings the bits differ far more often
    plain = port.f32_to_f16(port.layer(L, hidden, resid, threads=6).out)
    assert np.mean(plain == want_bits) < np.mean(got_bits == want_bits)


def test_rmsnorm_restatement_equals_the_reference_build(port, ref):
    """uocr_cpu_ref_rmsnorm_f32 compiled from the reference tree against its restatement, bit for bit, and the fp16
    form (what the GPU computes) against the f32 form on the same values within one fp16 step."""
    rng = np.random.default_rng(77)
    for rows, cols, eps in ((1, 1280, 1e-6), (7, 1280, 1e-6), (5, 128, 0.0), (3, 2048, 1e-5)):
        x = rng.standard_normal((rows, cols), dtype=np.float32) * rng.uniform(0.1, 8.0)
        w = rng.uniform(0.5, 1.5, cols).astype(np.float32)
        a, b = port.rmsnorm_f32(x, w, eps), ref.rmsnorm_f32(x, w, eps)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
        xb, wb = x.astype("<f2").view(np.uint16), w.astype("<f2").view(np.uint16)
        got = port.rmsnorm_f16(xb, wb, eps).view("<f2").astype(np.float32)
        want = ref.rmsnorm_f32(xb.view("<f2").astype(np.float32), wb.view("<f2").astype(np.float32), eps)
        assert np.array_equal(got, want.astype("<f2").astype(np.float32))


@pytest.mark.parametrize("qname", ["q4_0", "q8_0", "f16"])
def test_lm_head_restatement_against_numpy(port, qname):
    """The fused LM head's contract (src/backend/metal/kernels/lm_head_q4.metal:25-100: strict '>' over ascending rows, NaN
    totals skipped) restated once more in NumPy on the dequantised matrix: logits within f32 summation noise, the same
    winner unless the two best NumPy logits are closer than that noise, ties to the lowest row, a NaN row never wins."""
    rng = np.random.default_rng(900)
    V, H, n = 700, 256, 5
    w = rng.standard_normal((V, H), dtype=np.float32) * 0.05
    w[300] = w[40]                                      # an exact twin: the lower id must win whenever it is the best
    m = quant.make_matrix(quant.QTYPE_BY_NAME[qname], w)
    x = quant.synth_activations(rng, n, H)
    ids, scores, logits = port.lm_head_argmax(m, x, want_logits=True)
    ref = x.view("<f2").astype(np.float64) @ m.to_f32().astype(np.float64).T
    assert np.max(np.abs(logits - ref)) <= 1e-4 * max(1.0, float(np.max(np.abs(ref))))
    assert np.array_equal(logits[:, 300], logits[:, 40])
    for t in range(n):
        order = np.argsort(-ref[t], kind="stable")
        if ids[t] != order[0]:
            assert abs(ref[t, order[0]] - ref[t, order[1]]) <= 1e-4 and ids[t] == order[1]
        assert ids[t] != 300 and scores[t] == logits[t, ids[t]]
        assert ids[t] == int(np.flatnonzero(logits[t] == logits[t].max())[0])         # first of the equal maxima
    if qname == "f16":                                   # a NaN weight: that row's logit is NaN and it never wins
        bits = m.qweight.view(np.uint16).reshape(V, H).copy()
        bits[int(ids[0]), 3] = 0x7E00
        m_nan = quant.Matrix(quant.QTYPE_F16, V, H, bits.view(np.uint8).reshape(-1), None)
        ids2, _, logits2 = port.lm_head_argmax(m_nan, x, want_logits=True)
        assert np.isnan(logits2[0, ids[0]]) and ids2[0] != ids[0]
        assert ids2[0] == int(np.nanargmax(logits2[0]))
