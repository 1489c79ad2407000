"""Writer and reader of `.uocr` model files that hold only decoder MoE layers (test infrastructure).

The on-disk format is the reference's (src/model/uocr_format.h:171-299): a 112-byte header, a section directory,
config / tokenizer-metadata / provenance records, a tensor directory of packed 140-byte entries sorted by tensor id,
and a page-aligned tensor-data section.  Tensor ids follow src/model/uocr_tensor_registry.h:22-124.  The data of one
layer is laid out the way the converter does it (src/unlimitedocr_c/convert.py:950-996): the routed experts of a
quantised layer form ONE group — every packed projection first, expert-major `[gate, up, down]`, then every scale
block in the same order — so that the packed weights and the scales are each one contiguous slab; every other
tensor's scales follow its own payload.  Everything is aligned to 16 bytes, the data section to 4096.

`tests/test_model_file.py` checks that the reference's own loader accepts these files (when the build of the
reference sources under `oracle/_ref` is present) and that the library maps layers from them.
"""
from __future__ import annotations

import struct

import numpy as np

from oracle import quant

MAGIC = b"UOCR"
FORMAT_VERSION = 1
ENDIAN_MARKER = 0x01020304
DATA_ALIGNMENT = 4096
PAYLOAD_ALIGNMENT = 16
QPROFILE_FP16, QPROFILE_MIXED_Q8_0, QPROFILE_MIXED_Q4 = 1, 2, 3
SECTION_CONFIG, SECTION_TENSOR_DIRECTORY, SECTION_TOKENIZER, SECTION_PROVENANCE, SECTION_TENSOR_DATA = 1, 2, 3, 4, 5
TOKENIZER_MAGIC, PROVENANCE_MAGIC, TENSOR_DIR_MAGIC = 0x4B4F5455, 0x564F5250, 0x52494454
USAGE_RUNTIME = 1
FLAG_ROW_MAJOR = 1
FAMILY_LM_HEAD, FAMILY_FINAL_NORM, FAMILY_LAYER_NORM, FAMILY_LAYER_DENSE_MLP = 2, 3, 5, 6
FAMILY_MOE_ROUTER, FAMILY_MOE_EXPERT, FAMILY_MOE_SHARED = 7, 8, 9
TENSOR_ID_LM_HEAD, TENSOR_ID_FINAL_NORM = 2, 3
PROJ_WEIGHT, PROJ_GATE, PROJ_UP, PROJ_DOWN = 1, 20, 21, 22

HEADER = struct.Struct("<4s7IQQ32s32s")                     # 112 bytes
SECTION = struct.Struct("<IIQQQ")                           # 32 bytes
CONFIG = struct.Struct("<27I")                              # 108 bytes
TOKENIZER = struct.Struct("<4I32s7IQQ")                     # 92 bytes
PROVENANCE = struct.Struct("<14I32s32s32s32sQQ")            # 200 bytes
TENSOR_DIR = struct.Struct("<4I")                           # 16 bytes
TENSOR_ENTRY = struct.Struct("<IIiiIIIII4I4IQQIIQQQQIIII")  # 140 bytes
assert (HEADER.size, SECTION.size, CONFIG.size, TOKENIZER.size, PROVENANCE.size, TENSOR_DIR.size,
        TENSOR_ENTRY.size) == (112, 32, 108, 92, 200, 16, 140)

# the one model configuration the loader accepts (src/model/uocr_constants.h:6-51, uocr_format.h:315-345)
MODEL_CONFIG = (129280, 128000, 830, 0, 1, 2, 128815,           # vocabulary and special tokens
                1280, 12, 10, 10, 128, 10000, 32768, 128,       # decoder
                1, 64, 6, 896, 2, 6848,                         # dense first layer, MoE
                2048, 1280, 16, 4, 1024, 640)                   # projector and vision
assert len(MODEL_CONFIG) == 27


def tensor_id_layer(layer: int, local: int) -> int:
    return 10000 + layer * 1000 + local


def tensor_id_post_attn_norm(layer: int) -> int:
    return tensor_id_layer(layer, 2)


def tensor_id_dense(projection: int) -> int:
    return tensor_id_layer(0, 30 + projection - PROJ_GATE)


def tensor_id_router(layer: int) -> int:
    return tensor_id_layer(layer, 40)


def tensor_id_shared(layer: int, projection: int) -> int:
    return tensor_id_layer(layer, 50 + projection - PROJ_GATE)


def tensor_id_expert(layer: int, expert: int, projection: int) -> int:
    return tensor_id_layer(layer, 100 + 3 * expert + projection - PROJ_GATE)


def align_up(v: int, a: int) -> int:
    return (v + a - 1) // a * a


class _Tensor:
    def __init__(self, tid, family, layer, expert, projection, qtype, rows, cols, payload, scales, rank=2):
        self.id, self.family, self.layer, self.expert, self.projection = tid, family, layer, expert, projection
        self.qtype, self.rows, self.cols, self.rank = qtype, rows, cols, rank
        self.payload = np.ascontiguousarray(payload).view(np.uint8).reshape(-1)
        self.scales = None if scales is None else np.ascontiguousarray(scales).view(np.uint8).reshape(-1)
        self.payload_offset = 0
        self.scale_offset = 0

    def entry(self) -> bytes:
        quantised = self.qtype != quant.QTYPE_F16
        row_size = 0 if not quantised else quant.packed_row_bytes(self.qtype, self.cols)
        return TENSOR_ENTRY.pack(self.id, self.family, self.layer, self.expert, self.projection, USAGE_RUNTIME, self.qtype,
                                 FLAG_ROW_MAJOR, self.rank, self.rows, self.cols, 0, 0, self.rows, self.cols, 0, 0,
                                 self.payload_offset, self.payload.size, quant.GROUP if quantised else 0, row_size,
                                 self.scale_offset if quantised else 0, self.scales.size if quantised else 0, 0, 0, 0, 0, 0, 0)


def _layer_tensors(layer: int, L: quant.LayerWeights) -> list[list[_Tensor]]:
    """The layer's tensors in id order, as layout groups (one group = payloads first, then scales)."""
    groups = [[_Tensor(tensor_id_router(layer), FAMILY_MOE_ROUTER, layer, -1, PROJ_WEIGHT, quant.QTYPE_F16, L.E, L.H,
                       L.router, None)]]
    for proj, m in ((PROJ_GATE, L.shared_gate), (PROJ_UP, L.shared_up), (PROJ_DOWN, L.shared_down)):
        groups.append([_Tensor(tensor_id_shared(layer, proj), FAMILY_MOE_SHARED, layer, -1, proj, m.qtype, m.rows, m.cols,
                               m.qweight, m.qscale)])
    qt = L.expert_qtype
    pb = L.F * quant.packed_row_bytes(qt, L.H)
    ns = 0 if qt == quant.QTYPE_F16 else L.F * (L.H // quant.GROUP)
    experts = []
    for e in range(L.E):
        for p, (proj, rows, cols) in enumerate(((PROJ_GATE, L.F, L.H), (PROJ_UP, L.F, L.H), (PROJ_DOWN, L.H, L.F))):
            w = L.expert_qweight[(3 * e + p) * pb:(3 * e + p + 1) * pb]
            s = None if ns == 0 else L.expert_qscale[(3 * e + p) * ns:(3 * e + p + 1) * ns]
            experts.append(_Tensor(tensor_id_expert(layer, e, proj), FAMILY_MOE_EXPERT, layer, e, proj, qt, rows, cols, w, s))
    if qt == quant.QTYPE_F16:
        groups.extend([t] for t in experts)
    else:
        groups.append(experts)
    return groups


def _vector(tid, family, layer, values) -> _Tensor:
    v = np.ascontiguousarray(values).view(np.uint16).reshape(-1)           # fp16 bits
    return _Tensor(tid, family, layer, -1, PROJ_WEIGHT, quant.QTYPE_F16, v.size, 0, v, None, rank=1)


def write_moe_model(path: str, layers: dict[int, quant.LayerWeights], *, break_slab_at: tuple[int, int] | None = None,
                    dense: tuple | None = None, lm_head=None, post_attn_norms: dict | None = None, final_norm=None) -> dict:
    """Write a model file with the MoE tensors of `layers` (decoder layer index -> weights).

    `break_slab_at=(layer, expert)` inserts 16 bytes of padding before that expert's gate projection, which leaves a
    file the loader accepts but whose expert slab is no longer contiguous (the case every backend has to refuse).
    Optional neighbours of the MoE layers: `dense` = (gate, up, down) matrices of decoder layer 0's MLP, `lm_head` a
    [vocabulary][hidden] matrix, `post_attn_norms` = {decoder layer: fp16 bits [hidden]}, `final_norm` fp16 bits [hidden].
    Returns {"file_size", "tensor_count", "qprofile"}."""
    groups: list[list[_Tensor]] = []
    for layer in sorted(layers):
        groups.extend(_layer_tensors(layer, layers[layer]))
    if lm_head is not None:
        groups.append([_Tensor(TENSOR_ID_LM_HEAD, FAMILY_LM_HEAD, -1, -1, PROJ_WEIGHT, lm_head.qtype, lm_head.rows, lm_head.cols,
                               lm_head.qweight, lm_head.qscale)])
    if final_norm is not None:
        groups.append([_vector(TENSOR_ID_FINAL_NORM, FAMILY_FINAL_NORM, -1, final_norm)])
    for layer, values in (post_attn_norms or {}).items():
        groups.append([_vector(tensor_id_post_attn_norm(layer), FAMILY_LAYER_NORM, layer, values)])
    if dense is not None:
        for proj, m in zip((PROJ_GATE, PROJ_UP, PROJ_DOWN), dense):
            groups.append([_Tensor(tensor_id_dense(proj), FAMILY_LAYER_DENSE_MLP, 0, -1, proj, m.qtype, m.rows, m.cols, m.qweight,
                                   m.qscale)])
    groups.sort(key=lambda g: g[0].id)
    tensors = [t for g in groups for t in g]
    assert [t.id for t in tensors] == sorted(t.id for t in tensors)
    qtypes = {t.qtype for t in tensors}
    qprofile = QPROFILE_MIXED_Q4 if quant.QTYPE_Q4_0 in qtypes else (
        QPROFILE_MIXED_Q8_0 if quant.QTYPE_Q8_0 in qtypes else QPROFILE_FP16)

    section_dir = HEADER.size
    config_off = align_up(section_dir + 5 * SECTION.size, 8)
    tok_off = align_up(config_off + CONFIG.size, 8)
    prov_off = align_up(tok_off + TOKENIZER.size, 8)
    dir_off = align_up(prov_off + PROVENANCE.size, 8)
    dir_size = TENSOR_DIR.size + len(tensors) * TENSOR_ENTRY.size
    data_off = align_up(dir_off + dir_size, DATA_ALIGNMENT)

    cursor = data_off
    for g in groups:
        for t in g:
            cursor = align_up(cursor, PAYLOAD_ALIGNMENT)
            if break_slab_at is not None and (t.layer, t.expert, t.projection) == (*break_slab_at, PROJ_GATE):
                cursor += PAYLOAD_ALIGNMENT
            t.payload_offset = cursor
            cursor += t.payload.size
        for t in g:
            if t.scales is not None:
                cursor = align_up(cursor, PAYLOAD_ALIGNMENT)
                t.scale_offset = cursor
                cursor += t.scales.size
    file_size = align_up(cursor, DATA_ALIGNMENT)

    marker = bytes(range(1, 33))            # any non-zero 32 bytes: the loader only checks that hashes are present
    with open(path, "wb") as f:
        f.truncate(file_size)
        f.write(HEADER.pack(MAGIC, FORMAT_VERSION, HEADER.size, ENDIAN_MARKER, DATA_ALIGNMENT, qprofile, 5, 0, file_size,
                            section_dir, marker, bytes(32)))
        f.seek(section_dir)
        for typ, off, size, al in ((SECTION_CONFIG, config_off, CONFIG.size, 8), (SECTION_TOKENIZER, tok_off, TOKENIZER.size, 8),
                                   (SECTION_PROVENANCE, prov_off, PROVENANCE.size, 8),
                                   (SECTION_TENSOR_DIRECTORY, dir_off, dir_size, 8),
                                   (SECTION_TENSOR_DATA, data_off, file_size - data_off, DATA_ALIGNMENT)):
            f.write(SECTION.pack(typ, 0, off, size, al))
        f.seek(config_off)
        f.write(CONFIG.pack(*MODEL_CONFIG))
        f.seek(tok_off)
        f.write(TOKENIZER.pack(TOKENIZER_MAGIC, FORMAT_VERSION, TOKENIZER.size, 1, marker, *MODEL_CONFIG[:7], 0, 0))
        f.seek(prov_off)
        f.write(PROVENANCE.pack(PROVENANCE_MAGIC, FORMAT_VERSION, PROVENANCE.size, 0, len(tensors), len(tensors), 0, 0, 1,
                                qprofile, 0, 0, 0, 0, marker, marker, marker, bytes(32), 0, 0))
        f.seek(dir_off)
        f.write(TENSOR_DIR.pack(TENSOR_DIR_MAGIC, FORMAT_VERSION, TENSOR_ENTRY.size, len(tensors)))
        for t in tensors:
            f.write(t.entry())
        for t in tensors:
            f.seek(t.payload_offset)
            f.write(t.payload.tobytes())
            if t.scales is not None:
                f.seek(t.scale_offset)
                f.write(t.scales.tobytes())
    return {"file_size": file_size, "tensor_count": len(tensors), "qprofile": qprofile}


def read_directory(data: np.ndarray) -> tuple[int, int]:
    """(byte offset of the first tensor entry, number of entries) of a model file held in a uint8 array — the two
    values the reference's loader keeps in `uocr_model_file.tensors` and `.tensor_count`
    (src/model/uocr_model_file.h:9-28)."""
    head = HEADER.unpack_from(data, 0)
    assert head[0] == MAGIC and head[1] == FORMAT_VERSION
    section_count, section_dir = head[6], head[9]
    for i in range(section_count):
        typ, _flags, off, _size, _al = SECTION.unpack_from(data, section_dir + i * SECTION.size)
        if typ == SECTION_TENSOR_DIRECTORY:
            magic, _ver, entry_size, count = TENSOR_DIR.unpack_from(data, off)
            assert magic == TENSOR_DIR_MAGIC and entry_size == TENSOR_ENTRY.size
            return off + TENSOR_DIR.size, count
    raise ValueError("model file has no tensor directory")
