#!/usr/bin/env python3
"""Regenerates the fixtures in this folder from the reference tree.

Run where the reference checkout is available:

    python tests/golden/make_golden.py [--reference /path/to/unlimitedocr.c]

It writes three small files next to itself; the tests only read those files.

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
"""
from __future__ import annotations

import argparse
import json
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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    ref_root = Path(ap.parse_args().reference)

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
    print("wrote", [p.name for p in sorted(HERE.glob("*.json")) + sorted(HERE.glob("*.npz"))])


if __name__ == "__main__":
    main()
