"""The C-ABI library loads without a GPU and exports every function include/uocr_cuda_moe.h declares."""
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def pkg():
    import __graft_entry__ as entry
    entry.build()
    return entry.load_package()


def declared_functions():
    text = "\n".join((ROOT / "include").glob("*.h").__next__().read_text().splitlines())
    names = set()
    for header in (ROOT / "include").glob("*.h"):
        names |= set(re.findall(r"UOCR_CUDA_API\s+[\w\s\*]+?\b(uocr_cuda_\w+)\s*\(", header.read_text()))
    assert text
    return names


def test_every_declared_symbol_is_exported_and_bound(pkg):
    lib = pkg.load_library()
    declared = declared_functions()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert declared == set(pkg.ffi.EXPORTS), declared ^ set(pkg.ffi.EXPORTS)


def test_library_answers_without_a_gpu(pkg):
    lib = pkg.load_library()
    assert lib.uocr_cuda_backend_name() == b"cuda"
    assert lib.uocr_cuda_moe_scratch_size(1280, 64, 6, 896, 1792, 1) > 0
    assert lib.uocr_cuda_moe_scratch_size(0, 64, 6, 896, 1792, 1) == 0
    # the reference's MoE scratch rule (src/runtime/uocr_memory.c:480-543) is a lower bound of ours
    n = 4096
    ref_rule = n * (64 * 4 + 6 * 8) + n * (6 * 896 + 1792) * 2
    assert lib.uocr_cuda_moe_scratch_size(1280, 64, 6, 896, 1792, n) >= ref_rule


def test_no_silent_fallback_without_a_device(pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(pkg.UocrCudaError):
        pkg.Context()


def test_struct_layouts_match_the_header(pkg):
    import ctypes as C
    # uocr_cuda_matrix: int32, 2 x uint32, 2 pointers -> 32 bytes; the layer descriptor packs without surprises
    assert C.sizeof(pkg.ffi.CMatrix) == 32
    assert pkg.ffi.CLayerDesc.expert_qweight.offset % 8 == 0
    assert C.sizeof(pkg.ffi.CLayerDesc) == 24 + 16 + 8 + 16 + 48 + 3 * 32


def test_profile_event_names_follow_the_reference_naming():
    """The names the backend reports phase durations under (no GPU needed): the reference's event names with the
    backend prefix swapped (src/backend/metal/uocr_metal.m:14447-14496 `metal.decode.moe_router`,
    `metal.decode.moe_shared_experts`, `metal.decode.moe_routed_experts`; :13509, :13902 `metal.prefill.moe_routed_bucketed_q8/_q4`)."""
    import __graft_entry__ as entry
    names = entry.load_package().ffi.profile_event_names()
    assert len(names) == len(set(names)) and all(n.startswith(("cuda.decode.moe_", "cuda.prefill.moe_")) for n in names)
    for wanted in ("cuda.decode.moe_router", "cuda.decode.moe_routed_experts", "cuda.prefill.moe_shared_experts",
                   "cuda.prefill.moe_routed_bucketed_q4", "cuda.prefill.moe_routed_bucketed_q8", "cuda.prefill.moe_routed_bucketed_f16"):
        assert wanted in names
