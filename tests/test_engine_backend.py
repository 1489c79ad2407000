"""The `"cuda"` backend behind the reference's own engine library and unchanged public ABI (include/unlimitedocr.h).

oracle/_ref/libunlimitedocr_cuda.so is the reference's engine (src/core, src/runtime, src/model, CPU backend) built
from its tree with oracle/engine_cuda_backend.patch applied to a temporary copy of src/core/uocr_api.c and this
repository's engine-side glue (unlimitedocr.c_b200/engine_shim).  CPU part: the library keeps the ABI (cpu-ref engines
open as before, through plain ctypes and through the reference's unmodified Python binding when its tree is present) and
answers the way `backend_supported` does when no CUDA device exists.  GPU part: uocr_engine_open({backend: "cuda"}) on a
model file maps the MoE layers, accounts them under MODEL_VIEWS / MOE_SCRATCH in the engine's memory report, serves the
ABI smoke request, and refuses a file whose expert slab is not contiguous with the reference host's text."""
import ctypes as C
import os
import sys
from pathlib import Path

import numpy as np
import pytest

from oracle import quant
from tests import uocr_file
from tests.conftest import ROOT

ENGINE_LIB = ROOT / "oracle" / "_ref" / "libunlimitedocr_cuda.so"
UOCR_OK, UOCR_ERROR_NOT_IMPLEMENTED = 0, -4                     # include/unlimitedocr.h:31-38
MEMORY_MODEL_VIEWS, MEMORY_MOE_SCRATCH, MEMORY_CATEGORY_COUNT = 0, 7, 10     # include/unlimitedocr.h:50-62


class CEngineOpts(C.Structure):
    """uocr_engine_opts (include/unlimitedocr.h:140-151)."""
    _fields_ = [("model_path", C.c_char_p), ("backend", C.c_char_p), ("resource_path", C.c_char_p), ("max_batch", C.c_uint32),
                ("max_prompt_tokens", C.c_uint32), ("max_gen_tokens", C.c_uint32), ("profile", C.c_uint32),
                ("reserved0", C.c_uint32), ("memory_budget_bytes", C.c_uint64)]


class CMemoryReport(C.Structure):
    """uocr_memory_report (include/unlimitedocr.h:76-98)."""
    _fields_ = [("category_live_bytes", C.c_uint64 * MEMORY_CATEGORY_COUNT), ("category_peak_bytes", C.c_uint64 * MEMORY_CATEGORY_COUNT),
                ("total_live_bytes", C.c_uint64), ("total_peak_bytes", C.c_uint64), ("estimates", C.c_uint64 * 17)]


class CPreparedRequest(C.Structure):
    """uocr_prepared_request (include/unlimitedocr.h:127-138)."""
    _fields_ = [("input_ids", C.POINTER(C.c_int32)), ("image_mask", C.POINTER(C.c_uint8)), ("n_tokens", C.c_uint32),
                ("views", C.c_void_p), ("n_views", C.c_uint32), ("crop_grid_w", C.c_uint32), ("crop_grid_h", C.c_uint32),
                ("max_new_tokens", C.c_uint32)]


@pytest.fixture(scope="module")
def engine_lib():
    if not ENGINE_LIB.exists():
        pytest.skip("the patched engine library is not built (oracle/_ref/libunlimitedocr_cuda.so needs the reference tree once)")
    lib = C.CDLL(str(ENGINE_LIB))
    lib.uocr_abi_version.restype = C.c_uint32
    lib.uocr_engine_open.restype = C.c_void_p
    lib.uocr_engine_open.argtypes = [C.POINTER(CEngineOpts)]
    lib.uocr_engine_close.argtypes = [C.c_void_p]
    lib.uocr_last_error.restype = C.c_char_p
    lib.uocr_last_error.argtypes = [C.c_void_p]
    lib.uocr_engine_backend.restype = C.c_char_p
    lib.uocr_engine_backend.argtypes = [C.c_void_p]
    lib.uocr_engine_memory_report.argtypes = [C.c_void_p, C.POINTER(CMemoryReport)]
    lib.uocr_generate_prepared.argtypes = [C.c_void_p, C.POINTER(CPreparedRequest), C.c_uint32, C.POINTER(C.c_void_p)]
    lib.uocr_result_count.restype = C.c_uint32
    lib.uocr_result_count.argtypes = [C.c_void_p]
    lib.uocr_result_free.argtypes = [C.c_void_p]
    return lib


def open_engine(lib, backend, model_path=None, max_prompt_tokens=0):
    opts = CEngineOpts(model_path=model_path.encode() if model_path else None, backend=backend.encode(), resource_path=None,
                       max_batch=0, max_prompt_tokens=max_prompt_tokens, max_gen_tokens=0, profile=0, reserved0=0,
                       memory_budget_bytes=0)
    return lib.uocr_engine_open(C.byref(opts))


def cuda_device_present():
    torch = pytest.importorskip("torch")
    return torch.cuda.is_available()


def test_public_abi_is_unchanged_and_cpu_ref_still_opens(engine_lib):
    assert engine_lib.uocr_abi_version() > 0                 # (major << 16) | (minor << 8) | patch, include/unlimitedocr.h:26
    eng = open_engine(engine_lib, "cpu-ref")
    assert eng, engine_lib.uocr_last_error(None)
    assert engine_lib.uocr_engine_backend(eng) == b"cpu-ref"
    rep = CMemoryReport()
    assert engine_lib.uocr_engine_memory_report(eng, C.byref(rep)) == UOCR_OK and rep.total_live_bytes == 0
    engine_lib.uocr_engine_close(eng)
    assert not open_engine(engine_lib, "vulkan")
    assert b"unsupported backend 'vulkan'" in engine_lib.uocr_last_error(None)


def test_cuda_backend_without_a_device_is_refused_like_metal_without_one(engine_lib):
    if cuda_device_present():
        pytest.skip("a CUDA device is present")
    assert not open_engine(engine_lib, "cuda")
    assert engine_lib.uocr_last_error(None) == b"CUDA backend is compiled but no CUDA device is available"


def test_the_reference_python_binding_loads_it_unmodified(engine_lib):
    ref_src = Path(os.environ.get("UOCR_REFERENCE_ROOT", str(ROOT.parent / "reference"))) / "src"
    if not (ref_src / "unlimitedocr_c" / "ffi.py").exists():
        pytest.skip("the reference tree is not present")
    sys.path.insert(0, str(ref_src))
    try:
        from unlimitedocr_c import ffi
    finally:
        sys.path.remove(str(ref_src))
    # the binding insists on its own build folder for a path argument; a library bound beforehand is used as it is
    ffi._LIB = ffi._bind_library(ENGINE_LIB)
    try:
        eng = ffi.Engine(ffi.EngineOptions(backend="cpu-ref"))
        assert eng.backend == "cpu-ref"
        eng.close()
        if cuda_device_present():
            eng = ffi.Engine(ffi.EngineOptions(backend="cuda", warmup=False))
            assert eng.backend == "cuda"
            eng.close()
        else:
            with pytest.raises(RuntimeError, match="no CUDA device is available"):
                ffi.Engine(ffi.EngineOptions(backend="cuda", warmup=False))
    finally:
        ffi._LIB = None


# ------------------------------------------------------------------------------------------------------------ GPU
FULL = dict(H=1280, E=64, K=6, F=896, S=1792)
MOE_LAYERS = range(1, 12)            # decoder layers 1 .. 11 (src/model/uocr_constants.h:22, :45)


@pytest.fixture(scope="module")
def model_files(tmp_path_factory):
    rng = np.random.default_rng(700)
    L = quant.synth_layer(rng, expert_qtype=quant.QTYPE_Q4_0, shared_qtype=quant.QTYPE_Q8_0, **FULL)
    folder = tmp_path_factory.mktemp("engine")
    good, gap = folder / "moe.uocr", folder / "gap.uocr"
    # what the file holds either side of the MoE layers: layer 0's dense MLP (intermediate 6848), a (shortened) LM head, norms
    H = FULL["H"]
    dense = tuple(quant.make_matrix(quant.QTYPE_Q8_0, rng.standard_normal(shape, dtype=np.float32) * 0.02)
                  for shape in ((6848, H), (6848, H), (H, 6848)))
    head = quant.make_matrix(quant.QTYPE_Q4_0, rng.standard_normal((4096, H), dtype=np.float32) * 0.02)
    norm = rng.uniform(0.5, 1.5, H).astype("<f2").view(np.uint16)
    info = uocr_file.write_moe_model(str(good), {l: L for l in MOE_LAYERS}, dense=dense, lm_head=head,
                                     post_attn_norms={l: norm for l in range(12)}, final_norm=norm)
    info["neighbour_bytes"] = sum(m.qweight.size + m.qscale.size * 2 for m in dense + (head,)) + 13 * H * 2
    uocr_file.write_moe_model(str(gap), {l: L for l in MOE_LAYERS}, break_slab_at=(3, 17))
    return str(good), str(gap), info, L


@pytest.mark.gpu
def test_engine_open_with_the_cuda_backend(engine_lib, model_files):
    if not cuda_device_present():
        pytest.fail("GPU tests need a CUDA device")
    good, gap, info, L = model_files
    eng = open_engine(engine_lib, "cuda", good, max_prompt_tokens=256)
    assert eng, engine_lib.uocr_last_error(None)
    try:
        assert engine_lib.uocr_engine_backend(eng) == b"cuda"
        rep = CMemoryReport()
        assert engine_lib.uocr_engine_memory_report(eng, C.byref(rep)) == UOCR_OK
        layer_bytes = L.expert_qweight.size + L.expert_qscale.size * 2
        # the engine's own view of the file's tensor data plus the device copy of every layer
        assert rep.category_live_bytes[MEMORY_MODEL_VIEWS] >= 2 * (11 * layer_bytes + info["neighbour_bytes"])
        assert rep.category_live_bytes[MEMORY_MOE_SCRATCH] > 0
        assert rep.total_live_bytes >= rep.category_live_bytes[MEMORY_MODEL_VIEWS] + rep.category_live_bytes[MEMORY_MOE_SCRATCH]
        # the ABI smoke request (no generated tokens) is served; generation is refused by the engine as for cpu-ref
        ids = (C.c_int32 * 4)(0, 5, 6, 7)
        mask = (C.c_uint8 * 4)(0, 0, 0, 0)
        req = CPreparedRequest(input_ids=ids, image_mask=mask, n_tokens=4, views=None, n_views=0, crop_grid_w=1, crop_grid_h=1,
                               max_new_tokens=0)
        result = C.c_void_p()
        assert engine_lib.uocr_generate_prepared(eng, C.byref(req), 1, C.byref(result)) == UOCR_OK, engine_lib.uocr_last_error(eng)
        assert engine_lib.uocr_result_count(result) == 1
        engine_lib.uocr_result_free(result)
        req.max_new_tokens = 1
        assert engine_lib.uocr_generate_prepared(eng, C.byref(req), 1, C.byref(result)) == UOCR_ERROR_NOT_IMPLEMENTED
    finally:
        engine_lib.uocr_engine_close(eng)
    # a second engine after the first is gone: the close released everything it held
    eng = open_engine(engine_lib, "cuda", good, max_prompt_tokens=64)
    assert eng, engine_lib.uocr_last_error(None)
    engine_lib.uocr_engine_close(eng)
    # the expert slab of layer 3 has a gap in front of expert 17: the text of src/backend/metal/uocr_metal.m:3037-3154
    assert not open_engine(engine_lib, "cuda", gap, max_prompt_tokens=64)
    err = engine_lib.uocr_last_error(None)
    assert b"failed to initialize CUDA backend" in err and b"not interleaved-contiguous" in err and b"layer 3" in err, err
