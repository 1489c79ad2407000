#!/usr/bin/env python3
"""Regenerates the fixtures in this folder from the reference tree.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/unlimitedocr.c
    (or set UOCR_REFERENCE_ROOT)

It writes four small files next to itself; the tests only read those files.

cpu_ref_tiny_moe.json
    The MoE and dense-SwiGLU golden vectors the reference's own unit test
    checks its CPU backend against (values of the UOCR_TINY_MOE_* and
    UOCR_TINY_SWIGLU_* arrays in tests/fixtures/cpu_ref_tiny_golden.h, used by
    tests/test_cpu_ref.c:509-607), read as text from that header.
quant_q4_q8.npz
    Seeded f32 matrices (including an all-zero group and a negative signed
    maximum, the edge cases of tests/test_convert.py:192-218) together with the
    bytes the reference's quantisers produce for them
    (src/unlimitedocr_c/convert.py: _quantize_q4_0_rows and _expected_q8_0_chunk).
ref_layers.npz
    Outputs of the reference CPU layer function itself (compiled unmodified into
    oracle/_ref) on seeded inputs: the tiny 16-token Q8_0 layer of the benchmark
    plan, a Q4_0 and an fp16 variant, plus the router on hand-made tie cases.
    Inputs are regenerated from the seed by oracle/quant.py; only outputs are stored.
f16_contract.npz
    Outputs of the reference's NumPy fp16-contract layer (src/unlimitedocr_c/golden.py:
    _moe_router_f16 :544-562 and _moe_layer_f16_bits_with_router :649-666, which rounds the SwiGLU
    products, the routed sum and the shared output to fp16) on a seeded full-size fp16 layer.  The
    functions read their weights by tensor name from a checkpoint folder; here the module's reader
    is replaced by one that serves the synthetic arrays under the same names, nothing else changes.
    Inputs are regenerated from the seed; only outputs are stored.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
import types
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))


def parse_header(path: Path, prefixes: tuple[str, ...]) -> dict:
    text = path.read_text()
    out: dict = {}
    for name, value in re.findall(r"#define\s+(UOCR_TINY_\w+)\s+([^\s]+)", text):
        if name.startswith(prefixes):
            v = value.rstrip("uf")
            out[name] = float(v) if ("." in v or "e" in v) else int(v)
    for ctype, name, body in re.findall(r"static const (float|uint32_t) (UOCR_TINY_\w+)\[[^\]]*\] = \{(.*?)\};", text, re.S):
        if name.startswith(prefixes):
            items = [t.strip() for t in body.replace("\n", " ").split(",") if t.strip()]
            out[name] = [float(t.rstrip("f")) if ctype == "float" else int(t.rstrip("u")) for t in items]
    return out


def tiny_cases():
    """(name, qtype name, seed) of the stored reference-layer runs; shapes of the tiny benchmark layer."""
    return [("tiny_q8", "q8_0", 0), ("tiny_q4", "q4_0", 10), ("tiny_f16", "f16", 20)]


TINY = dict(H=128, E=8, K=2, F=64, S=64)
TINY_ROWS = 16


FULL = dict(H=1280, E=64, K=6, F=896, S=1792)
F16_CONTRACT_SEED, F16_CONTRACT_ROWS, F16_CONTRACT_LAYER = 50, 6, 1


def f16_contract_inputs():
    """Seeded full-size fp16 layer, activations and residual of the fp16-contract fixture."""
    from oracle import quant
    rng = np.random.default_rng(F16_CONTRACT_SEED)
    L = quant.synth_layer(rng, expert_qtype=quant.QTYPE_F16, **FULL)
    hidden = quant.synth_activations(rng, F16_CONTRACT_ROWS, FULL["H"])
    resid = quant.synth_activations(rng, F16_CONTRACT_ROWS, FULL["H"])
    return L, hidden, resid


def f16_contract_tensor_names(L, layer: int) -> dict:
    """The layer's fp16 tensors under the checkpoint names the reference's NumPy functions ask for."""
    H, E, F, S = L.H, L.E, L.F, L.S
    prefix = f"model.layers.{layer}.mlp"
    out = {f"{prefix}.gate.weight": L.router.reshape(E, H)}
    slab = L.expert_qweight.view(np.uint16)
    proj = F * H
    for e in range(E):
        base = e * 3 * proj
        out[f"{prefix}.experts.{e}.gate_proj.weight"] = slab[base:base + proj].reshape(F, H)
        out[f"{prefix}.experts.{e}.up_proj.weight"] = slab[base + proj:base + 2 * proj].reshape(F, H)
        out[f"{prefix}.experts.{e}.down_proj.weight"] = slab[base + 2 * proj:base + 3 * proj].reshape(H, F)
    for key, m in (("gate_proj", L.shared_gate), ("up_proj", L.shared_up), ("down_proj", L.shared_down)):
        out[f"{prefix}.shared_experts.{key}.weight"] = m.qweight.view(np.uint16).reshape(m.rows, m.cols)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("UOCR_REFERENCE_ROOT"),
                    help="checkout of the reference project (or set UOCR_REFERENCE_ROOT)")
    args = ap.parse_args()
    if not args.reference:
        ap.error("give --reference or set UOCR_REFERENCE_ROOT")
    ref_root = Path(args.reference)

    # 1. the reference's golden header, as data
    hdr = parse_header(ref_root / "tests/fixtures/cpu_ref_tiny_golden.h", ("UOCR_TINY_MOE_", "UOCR_TINY_SWIGLU_"))
    assert len(hdr["UOCR_TINY_MOE_EXPECTED"]) == 6 and len(hdr["UOCR_TINY_MOE_EXPECTED_TOP_IDS"]) == 12
    (HERE / "cpu_ref_tiny_moe.json").write_text(json.dumps(hdr, indent=0, sort_keys=True) + "\n")

    # 2. quantiser bytes from the reference converter
    sys.path.insert(0, str(ref_root / "src"))
    from unlimitedocr_c import convert as ref_convert  # type: ignore

    rng = np.random.default_rng(7)
    a = rng.standard_normal((6, 256), dtype=np.float32) * np.float32(0.05)
    a[0, :64] = 0.0                # all-zero group
    a[1, 64] = -0.5                # negative signed maximum
    a[2, 130] = 0.75               # positive signed maximum (scale negative)
    a[3, :] = np.float32(0.02) * rng.standard_normal(256, dtype=np.float32)
    a[4, 192:] = np.float32(1e-7)  # scale underflows towards fp16 subnormals
    b = rng.standard_normal((32, 1280), dtype=np.float32) * np.float32(0.02)
    out = {}
    for tag, m in (("a", a), ("b", b)):
        packed, scales, deq = ref_convert._quantize_q4_0_rows(m, 64)
        q8w, q8s, *_ = ref_convert._expected_q8_0_chunk(m, types.SimpleNamespace(block_size=64))
        out[f"{tag}_values"] = m
        out[f"{tag}_q4_packed"] = packed
        out[f"{tag}_q4_scales"] = scales.view(np.uint16)
        out[f"{tag}_q4_dequant"] = deq
        out[f"{tag}_q8_weight"] = np.frombuffer(q8w, np.int8).reshape(m.shape)
        out[f"{tag}_q8_scales"] = np.frombuffer(q8s, np.uint16).reshape(m.shape[0], -1)
    np.savez_compressed(HERE / "quant_q4_q8.npz", **out)

    # 3. the reference layer function itself on seeded inputs
    from oracle import oracle as orc
    from oracle import quant

    orc.build(force=True)
    ref = orc.Ref()
    store = {}
    for name, qname, seed in tiny_cases():
        rng = np.random.default_rng(seed)
        L = quant.synth_layer(rng, expert_qtype=quant.QTYPE_BY_NAME[qname], **TINY)
        hidden = quant.synth_activations(rng, TINY_ROWS, TINY["H"])
        o = ref.layer(L, hidden)
        for key in ("logits", "probs", "ids", "weights", "expert_ws", "shared_ws", "out"):
            store[f"{name}_{key}"] = getattr(o, key)
    # routing on exact ties, through the unmodified router (identity weights reproduce the logits)
    ties = np.zeros((4, 8), np.float32)
    ties[1, [2, 5]] = 1.0                      # two-way tie for first place
    ties[2] = [0.5, 0.25, 0.5, 0.25, 0.5, 0.25, 0.5, 0.25]
    ties[3] = [-1, -1, 3, 3, 3, -1, 3, 2]      # tie spanning the k / k+1 boundary for k = 3
    for k in (1, 2, 3, 6):
        st, o = ref.route_from_logits(ties, k)
        assert st == 1
        store[f"ties_k{k}_ids"] = o.ids
        store[f"ties_k{k}_weights"] = o.weights
    store["ties_logits"] = ties
    np.savez_compressed(HERE / "ref_layers.npz", **store)

    # 4. the reference's NumPy fp16 contract on a synthetic full-size fp16 layer
    from unlimitedocr_c import golden as ref_golden  # type: ignore

    L, hidden, resid = f16_contract_inputs()
    names = f16_contract_tensor_names(L, layer=F16_CONTRACT_LAYER)

    def fake_reader(hf_dir, name, expected_shape=None):
        t = names[name]
        assert expected_shape is None or tuple(expected_shape) == t.shape, (name, expected_shape, t.shape)
        return t

    ref_golden.read_bf16_tensor_as_f16_bits = fake_reader
    probs, r_ids, r_w = ref_golden._moe_router_f16(hidden, names[f"model.layers.{F16_CONTRACT_LAYER}.mlp.gate.weight"])
    out_bits, ids, wts = ref_golden._moe_layer_f16_bits_with_router(hidden, resid, "synthetic", layer=F16_CONTRACT_LAYER)
    assert np.array_equal(ids, r_ids) and np.array_equal(wts, r_w)
    np.savez_compressed(HERE / "f16_contract.npz", probs=probs, ids=ids, weights=wts, out_bits=out_bits)
    print("wrote", [p.name for p in sorted(HERE.glob("*.json")) + sorted(HERE.glob("*.npz"))])


if __name__ == "__main__":
    main()
