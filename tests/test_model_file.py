"""Mapping MoE layers from a `.uocr` model file (uocr_cuda_context_map_model).

CPU part: the files these tests write are accepted by the reference's OWN loader (src/model/uocr_model_file.c, built
unmodified into oracle/_ref/libuocr_model_file.so when the reference sources are at hand), and its view of the tensor
directory equals the one the tests hand to the library.  GPU part: layers mapped from a file behave bit for bit like
layers mapped from memory descriptors, the oracle agrees with them, and files the reference host would refuse are
refused with the same texts.
"""
import ctypes

import numpy as np
import pytest

from oracle import quant
from tests import uocr_file

torch = pytest.importorskip("torch")

TINY = dict(H=128, E=8, K=2, F=64, S=128)
FULL = dict(H=1280, E=64, K=6, F=896, S=1792)
PROFILES = [("q4_0", "q8_0"), ("q8_0", "q8_0"), ("f16", "f16")]
QT = quant.QTYPE_BY_NAME


class RefModelFile(ctypes.Structure):
    """uocr_model_file (src/model/uocr_model_file.h:9-28)."""
    _fields_ = [("data", ctypes.c_void_p), ("size", ctypes.c_size_t), ("owns_mapping", ctypes.c_int), ("fd", ctypes.c_int),
                ("header", ctypes.c_void_p), ("sections", ctypes.c_void_p), ("config", ctypes.c_void_p),
                ("tokenizer_metadata", ctypes.c_void_p), ("tokenizer_payload", ctypes.c_void_p),
                ("tokenizer_payload_size", ctypes.c_size_t), ("provenance", ctypes.c_void_p),
                ("provenance_json", ctypes.c_void_p), ("provenance_json_size", ctypes.c_size_t),
                ("tensor_directory", ctypes.c_void_p), ("tensors", ctypes.c_void_p), ("tensor_count", ctypes.c_uint32)]


@pytest.fixture(scope="module")
def ref_loader():
    from tests.conftest import ROOT
    path = ROOT / "oracle" / "_ref" / "libuocr_model_file.so"
    if not path.exists():
        pytest.skip("the reference's model-file loader is not built (oracle/_ref/libuocr_model_file.so)")
    lib = ctypes.CDLL(str(path))
    lib.uocr_model_file_find_tensor.restype = ctypes.c_void_p
    return lib


def tiny_layers(seed, expert, shared, layers=(1, 2)):
    rng = np.random.default_rng(seed)
    return {l: quant.synth_layer(rng, expert_qtype=QT[expert], shared_qtype=QT[shared], **TINY) for l in layers}


@pytest.mark.parametrize("expert,shared", PROFILES)
def test_reference_loader_accepts_the_files(ref_loader, tmp_path, expert, shared):
    layers = tiny_layers(5, expert, shared)
    path = tmp_path / "moe.uocr"
    info = uocr_file.write_moe_model(str(path), layers)
    mf, err = RefModelFile(), ctypes.create_string_buffer(512)
    assert ref_loader.uocr_model_file_open(str(path).encode(), ctypes.byref(mf), err, 512) == 0, err.value
    try:
        data = np.fromfile(path, dtype=np.uint8)
        first, count = uocr_file.read_directory(data)
        assert (mf.size, mf.tensor_count) == (info["file_size"], info["tensor_count"])
        assert (mf.tensors - mf.data, mf.tensor_count) == (first, count)
        # the reference's lookup finds every MoE tensor where the writer put it, with the bytes of the layer
        L = layers[2]
        pb = L.F * quant.packed_row_bytes(L.expert_qtype, L.H)
        for e, p in ((0, 0), (3, 1), (7, 2)):
            tid = uocr_file.tensor_id_expert(2, e, uocr_file.PROJ_GATE + p)
            entry = ref_loader.uocr_model_file_find_tensor(ctypes.byref(mf), tid)
            assert entry
            fields = uocr_file.TENSOR_ENTRY.unpack(ctypes.string_at(entry, uocr_file.TENSOR_ENTRY.size))
            assert fields[0] == tid and fields[6] == L.expert_qtype
            off, size = fields[17], fields[18]
            assert size == pb
            assert np.array_equal(data[off:off + size], L.expert_qweight[(3 * e + p) * pb:(3 * e + p + 1) * pb])
        assert not ref_loader.uocr_model_file_find_tensor(ctypes.byref(mf), uocr_file.tensor_id_router(3))
    finally:
        ref_loader.uocr_model_file_close(ctypes.byref(mf))


def test_a_broken_slab_is_still_a_valid_file(ref_loader, tmp_path):
    """The loader checks each tensor on its own; slab contiguity is the backend's rule, so the file with a gap
    inside the expert slab opens — which is why the backend must check."""
    path = tmp_path / "gap.uocr"
    uocr_file.write_moe_model(str(path), tiny_layers(6, "q4_0", "q8_0"), break_slab_at=(2, 5))
    mf, err = RefModelFile(), ctypes.create_string_buffer(512)
    assert ref_loader.uocr_model_file_open(str(path).encode(), ctypes.byref(mf), err, 512) == 0, err.value
    ref_loader.uocr_model_file_close(ctypes.byref(mf))


# ------------------------------------------------------------------------------------------------------------ GPU
@pytest.fixture(scope="module")
def pkg():
    import __graft_entry__ as entry
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; the library has no CPU path")
    torch.cuda.set_device(0)
    return entry.load_package()


def map_file(ctx, path, dims, first, count, **override):
    data = np.fromfile(path, dtype=np.uint8)
    entries, n_entries = uocr_file.read_directory(data)
    args = dict(routed_experts=dims["E"], top_k=dims["K"], first_moe_layer=first, moe_layer_count=count)
    args.update(override)
    return ctx.map_model(data.ctypes.data, data.size, data.ctypes.data + entries, n_entries, **args)


def run_stack(ctx, n_layers, hidden_bits, n):
    ctx.allocate_runtime_arenas(n)
    ctx.set_stream(torch.cuda.current_stream().cuda_stream)
    x = torch.from_numpy(hidden_bits).cuda().view(torch.float16)
    outs = []
    for i in range(n_layers):
        out = torch.zeros_like(x)
        ctx.layer_forward(i, x, n, out, residual=x)
        ctx.synchronize()
        outs.append(out.cpu().numpy().view(np.uint16))
        x = out
    return outs


@pytest.mark.gpu
@pytest.mark.parametrize("expert,shared", PROFILES)
@pytest.mark.parametrize("n", [1, 7, 96])
def test_layers_from_a_file_equal_layers_from_descriptors(pkg, port, tmp_path, expert, shared, n):
    layers = tiny_layers(7, expert, shared)
    path = tmp_path / "moe.uocr"
    uocr_file.write_moe_model(str(path), layers)
    hidden = quant.synth_activations(np.random.default_rng(8), n, TINY["H"])
    with pkg.Context() as from_file, pkg.Context() as from_desc:
        assert map_file(from_file, path, TINY, 1, 2) == 2
        for l in (1, 2):
            from_desc.map_layer(layers[l])
        assert from_file.model_view_bytes == from_desc.model_view_bytes
        got = run_stack(from_file, 2, hidden, n)
        want = run_stack(from_desc, 2, hidden, n)
    for a, b in zip(got, want):
        assert np.array_equal(a, b)
    ref = port.layer(layers[1], hidden, hidden)
    err = float(np.max(np.abs(got[0].view("<f2").astype(np.float32) - ref.out)))
    assert err <= 2e-2


@pytest.mark.gpu
def test_full_size_mixed_q4_layer_from_a_file(pkg, port, tmp_path):
    """One decoder layer of the model's shapes as the mixed-q4 profile stores it (Q4_0 routed experts, Q8_0 shared
    experts, 120 MB of tensor data), one token: takes the single-launch decode kernel and matches the oracle."""
    rng = np.random.default_rng(9)
    L = quant.synth_layer(rng, expert_qtype=quant.QTYPE_Q4_0, shared_qtype=quant.QTYPE_Q8_0, **FULL)
    path = tmp_path / "layer5.uocr"
    uocr_file.write_moe_model(str(path), {5: L})
    hidden = quant.synth_activations(rng, 1, FULL["H"])
    with pkg.Context() as ctx:
        assert map_file(ctx, path, FULL, 5, 1) == 1
        got = run_stack(ctx, 1, hidden, 1)[0]
    want = port.layer(L, hidden, hidden)
    out = got.view("<f2").astype(np.float32)
    err = float(np.max(np.abs(out - want.out)))
    cos = float(out.reshape(-1) @ want.out.reshape(-1) / np.sqrt((out * out).sum() * (want.out * want.out).sum()))
    assert err <= 2e-2 and cos >= 0.9995, (err, cos)


@pytest.mark.gpu
def test_files_the_reference_host_refuses_are_refused(pkg, tmp_path):
    layers = tiny_layers(10, "q4_0", "q8_0")
    good, gap = tmp_path / "good.uocr", tmp_path / "gap.uocr"
    uocr_file.write_moe_model(str(good), layers)
    uocr_file.write_moe_model(str(gap), layers, break_slab_at=(2, 5))
    with pkg.Context() as ctx:
        with pytest.raises(pkg.UocrCudaError, match="layer 2 are not interleaved-contiguous at expert 5"):
            map_file(ctx, gap, TINY, 1, 2)
        assert ctx.layer_count == 0                      # layer 1 was fine, but nothing stays mapped
        with pytest.raises(pkg.UocrCudaError, match="layer 3: MoE router is missing"):
            map_file(ctx, good, TINY, 1, 3)
        with pytest.raises(pkg.UocrCudaError, match="router has 8 rows for 16 experts"):
            map_file(ctx, good, TINY, 1, 2, routed_experts=16)
        with pytest.raises(pkg.UocrCudaError, match="invalid router configuration"):
            map_file(ctx, good, TINY, 1, 2, top_k=9)
        data = np.fromfile(good, dtype=np.uint8)
        entries, count = uocr_file.read_directory(data)
        with pytest.raises(pkg.UocrCudaError, match="tensor directory lies outside"):
            ctx.map_model(data.ctypes.data, entries + 100, data.ctypes.data + entries, count, routed_experts=8, top_k=2,
                          first_moe_layer=1, moe_layer_count=2)
        # a payload that points past the end of a truncated buffer
        with pytest.raises(pkg.UocrCudaError, match="outside the file"):
            ctx.map_model(data.ctypes.data, data.size - 8192, data.ctypes.data + entries, count, routed_experts=8, top_k=2,
                          first_moe_layer=1, moe_layer_count=2)
        assert ctx.layer_count == 0
        assert map_file(ctx, good, TINY, 1, 2) == 2
        with pytest.raises(pkg.UocrCudaError, match="already mapped"):
            map_file(ctx, good, TINY, 1, 2)
        ctx.unmap_model()
        assert map_file(ctx, good, TINY, 2, 1) == 1


# ------------------------------------------------------------------------------ the tensors either side of the layers
EPS = 1.0e-6                # UOCR_RMS_NORM_EPS (src/model/uocr_constants.h:27)


def neighbour_tensors(seed, qname="q8_0", S=256, V=512):
    rng = np.random.default_rng(seed)
    H, qt = TINY["H"], QT[qname]
    dense = tuple(quant.make_matrix(qt, rng.standard_normal(shape, dtype=np.float32) * 0.05) for shape in ((S, H), (S, H), (H, S)))
    head = quant.make_matrix(qt, rng.standard_normal((V, H), dtype=np.float32) * 0.05)
    norms = {l: rng.uniform(0.5, 1.5, H).astype("<f2").view(np.uint16) for l in (0, 1, 2)}
    final = rng.uniform(0.5, 1.5, H).astype("<f2").view(np.uint16)
    return dense, head, norms, final


def test_reference_loader_accepts_a_file_with_the_neighbouring_tensors(ref_loader, tmp_path):
    dense, head, norms, final = neighbour_tensors(20)
    path = tmp_path / "full.uocr"
    info = uocr_file.write_moe_model(str(path), tiny_layers(21, "q4_0", "q8_0"), dense=dense, lm_head=head, post_attn_norms=norms,
                                     final_norm=final)
    mf, err = RefModelFile(), ctypes.create_string_buffer(512)
    assert ref_loader.uocr_model_file_open(str(path).encode(), ctypes.byref(mf), err, 512) == 0, err.value
    try:
        assert mf.tensor_count == info["tensor_count"]
        for tid in (uocr_file.TENSOR_ID_LM_HEAD, uocr_file.TENSOR_ID_FINAL_NORM, uocr_file.tensor_id_post_attn_norm(2),
                    uocr_file.tensor_id_dense(uocr_file.PROJ_DOWN)):
            assert ref_loader.uocr_model_file_find_tensor(ctypes.byref(mf), tid)
    finally:
        ref_loader.uocr_model_file_close(ctypes.byref(mf))


@pytest.mark.gpu
@pytest.mark.parametrize("qname", ["q8_0", "q4_0", "f16"])
def test_neighbours_from_a_file_equal_the_same_tensors_from_memory(pkg, tmp_path, qname):
    """Dense MLP of layer 0, LM head, post-attention norms and final norm mapped from the file: every call through them
    gives bit for bit what the same tensors mapped from host arrays give."""
    dense, head, norms, final = neighbour_tensors(22, qname)
    layers = tiny_layers(23, "q4_0", "q8_0")
    path = tmp_path / "full.uocr"
    uocr_file.write_moe_model(str(path), layers, dense=dense, lm_head=head, post_attn_norms=norms, final_norm=final)
    H, n = TINY["H"], 5
    rng = np.random.default_rng(24)
    stream_rows = (rng.standard_normal((n, H), dtype=np.float32) * 2.0).astype("<f2").view(np.uint16)
    dev = lambda bits: torch.from_numpy(np.ascontiguousarray(bits)).cuda().view(torch.float16)
    data = np.fromfile(path, dtype=np.uint8)
    entries, n_entries = uocr_file.read_directory(data)
    with pkg.Context() as from_file, pkg.Context() as from_mem:
        assert map_file(from_file, path, TINY, 1, 2) == 2
        got = from_file.map_model_neighbours(data.ctypes.data, data.size, data.ctypes.data + entries, n_entries, token_capacity=16,
                                             first_moe_layer=1, moe_layer_count=2)
        assert got["dense_mlp"] == 0 and sorted(got["post_attn_norm"]) == [0, 1, 2] and got["final_norm"]
        with pytest.raises(pkg.UocrCudaError, match="already mapped"):
            from_file.map_model_neighbours(data.ctypes.data, data.size, data.ctypes.data + entries, n_entries, token_capacity=16,
                                           first_moe_layer=1, moe_layer_count=2)
        for l in (1, 2):
            from_mem.map_layer(layers[l])
        idx = from_mem.map_dense_mlp(*dense, token_capacity=16)
        from_mem.map_lm_head(head)
        assert from_file.model_view_bytes == from_mem.model_view_bytes + 4 * H * 2          # + three layer norms and the final norm
        outs = []
        for ctx, dense_idx, w0, w1, wf in ((from_file, got["dense_mlp"], got["post_attn_norm"][0], got["post_attn_norm"][1], got["final_norm"]),
                                           (from_mem, idx, dev(norms[0]), dev(norms[1]), dev(final))):
            ctx.allocate_runtime_arenas(n)
            ctx.set_stream(torch.cuda.current_stream().cuda_stream)
            a, b, c = (torch.zeros((n, H), dtype=torch.float16, device="cuda") for _ in range(3))
            ids = torch.zeros(4, dtype=torch.int32, device="cuda")
            ctx.dense_mlp_forward_normed(dense_idx, dev(stream_rows), w0, EPS, n, a)           # decoder layer 0
            ctx.layer_forward_normed(0, a, w1, EPS, n, b)                                     # decoder layer 1
            ctx.rmsnorm(b, wf, EPS, n, H, c)                                                  # final norm
            ctx.lm_head_argmax(c, 4, ids)
            ctx.synchronize()
            outs.append((a.cpu().numpy().view(np.uint16), b.cpu().numpy().view(np.uint16), ids.cpu().numpy()))
    for x, y in zip(*outs):
        assert np.array_equal(x, y)


@pytest.mark.gpu
def test_neighbour_tensors_that_do_not_fit_are_refused(pkg, tmp_path):
    dense, head, norms, final = neighbour_tensors(25)
    layers = tiny_layers(26, "q4_0", "q8_0")

    def try_map(path, match):
        data = np.fromfile(path, dtype=np.uint8)
        entries, n_entries = uocr_file.read_directory(data)
        with pkg.Context() as ctx:
            with pytest.raises(pkg.UocrCudaError, match="map the MoE layers first"):
                ctx.map_model_neighbours(data.ctypes.data, data.size, data.ctypes.data + entries, n_entries, token_capacity=8,
                                         first_moe_layer=1, moe_layer_count=2)
            map_file(ctx, path, TINY, 1, 2)
            if match is None:
                got = ctx.map_model_neighbours(data.ctypes.data, data.size, data.ctypes.data + entries, n_entries, token_capacity=8,
                                               first_moe_layer=1, moe_layer_count=2)
                return got
            with pytest.raises(pkg.UocrCudaError, match=match):
                ctx.map_model_neighbours(data.ctypes.data, data.size, data.ctypes.data + entries, n_entries, token_capacity=8,
                                         first_moe_layer=1, moe_layer_count=2)
            assert ctx.moe_scratch_bytes == 0 and ctx.layer_count == 2          # nothing of the neighbours stays behind

    bare = tmp_path / "bare.uocr"
    uocr_file.write_moe_model(str(bare), layers)
    assert try_map(bare, None) == {"dense_mlp": None, "post_attn_norm": {}, "final_norm": None}      # nothing there: nothing mapped
    short_norm = tmp_path / "short.uocr"
    uocr_file.write_moe_model(str(short_norm), layers, post_attn_norms={1: norms[1][:64]})
    try_map(short_norm, "layer 1: post-attention norm does not have the hidden size")
    wide = tmp_path / "wide.uocr"
    bad_head = quant.make_matrix(quant.QTYPE_Q8_0, np.random.default_rng(27).standard_normal((64, 2 * TINY["H"]), dtype=np.float32))
    uocr_file.write_moe_model(str(wide), layers, lm_head=bad_head, dense=dense)
    try_map(wide, "LM head")
