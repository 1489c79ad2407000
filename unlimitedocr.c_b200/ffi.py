"""ctypes binding of libuocr_cuda_moe.so, in the style of the reference's own binding
(src/unlimitedocr_c/ffi.py:252-335: locate the shared library, declare every symbol's
signature once, wrap handles in small classes that turn status codes into exceptions).

The library is the product; this module only marshals arguments.  There is no fallback:
if the shared library is missing or the machine has no sm_100 GPU, construction raises.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path
from typing import Any

import numpy as np

QTYPE_F16, QTYPE_Q8_0, QTYPE_Q4_0 = 1, 3, 4
_ERR = 1024


class UocrCudaError(RuntimeError):
    pass


class CMatrix(C.Structure):
    _fields_ = [("qtype", C.c_int32), ("rows", C.c_uint32), ("cols", C.c_uint32), ("qweight", C.c_void_p),
                ("qscale", C.c_void_p)]


class CLayerDesc(C.Structure):
    _fields_ = [("hidden_size", C.c_uint32), ("n_experts", C.c_uint32), ("top_k", C.c_uint32),
                ("expert_intermediate", C.c_uint32), ("shared_intermediate", C.c_uint32),
                ("routed_scaling_factor", C.c_float), ("router_weight_f16", C.c_void_p),
                ("router_logit_bias", C.c_void_p), ("expert_qtype", C.c_int32), ("expert_qweight", C.c_void_p),
                ("expert_qscale", C.c_void_p), ("expert_stride_bytes", C.c_uint64), ("up_offset_bytes", C.c_uint64),
                ("down_offset_bytes", C.c_uint64), ("expert_scale_stride_values", C.c_uint64),
                ("up_scale_offset_values", C.c_uint64), ("down_scale_offset_values", C.c_uint64),
                ("shared_gate", CMatrix), ("shared_up", CMatrix), ("shared_down", CMatrix)]


class CModelFileView(C.Structure):
    """uocr_cuda_model_file_view: what the backend needs of an opened `.uocr` file."""
    _fields_ = [("data", C.c_void_p), ("size", C.c_uint64), ("tensors", C.c_void_p), ("tensor_count", C.c_uint32),
                ("routed_experts", C.c_uint32), ("moe_top_k", C.c_uint32), ("first_moe_layer", C.c_uint32),
                ("moe_layer_count", C.c_uint32), ("routed_scaling_factor", C.c_float)]


class CDebugOutputs(C.Structure):
    _fields_ = [("d_router_logits", C.c_void_p), ("d_router_probs", C.c_void_p), ("d_top_ids", C.c_void_p),
                ("d_top_weights", C.c_void_p)]


PROFILE_ADD_EVENT_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_char_p, C.c_double)       # uocr_profile_add_event_ms
MEMORY_ACCOUNT_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_uint64)          # uocr_memory_reserve / _release

EXPORTS = (
    "uocr_cuda_is_available", "uocr_cuda_backend_name", "uocr_cuda_device_count", "uocr_cuda_context_create",
    "uocr_cuda_context_destroy", "uocr_cuda_context_last_error", "uocr_cuda_context_set_stream",
    "uocr_cuda_context_set_profile_detail", "uocr_cuda_context_set_profile", "uocr_cuda_context_set_memory_tracker",
    "uocr_cuda_profile_event_name", "uocr_cuda_context_synchronize", "uocr_cuda_context_kernel_launches", "uocr_cuda_context_model_view_bytes",
    "uocr_cuda_context_moe_scratch_bytes", "uocr_cuda_context_map_moe_layer", "uocr_cuda_context_map_model", "uocr_cuda_context_unmap_model",
    "uocr_cuda_context_moe_layer_count", "uocr_cuda_context_map_model_neighbours", "uocr_cuda_context_file_dense_mlp_index",
    "uocr_cuda_context_post_attn_norm_weight", "uocr_cuda_context_final_norm_weight", "uocr_cuda_context_allocate_runtime_arenas",
    "uocr_cuda_context_release_runtime_arenas", "uocr_cuda_moe_scratch_size", "uocr_cuda_moe_router",
    "uocr_cuda_moe_dispatch_plan", "uocr_cuda_moe_dispatch_plan_noalloc", "uocr_cuda_moe_debug_dequantize", "uocr_cuda_moe_regime_name", "uocr_cuda_rmsnorm", "uocr_cuda_moe_layer_forward_normed", "uocr_cuda_context_map_dense_mlp",
    "uocr_cuda_dense_mlp_forward", "uocr_cuda_dense_mlp_forward_normed", "uocr_cuda_context_map_lm_head", "uocr_cuda_lm_head_argmax", "uocr_cuda_moe_layer_forward", "uocr_cuda_moe_stack_forward",
    "uocr_cuda_moe_layer_forward_host", "uocr_cuda_moe_stack_forward_host",
    "uocr_cuda_moe_ep_dispatch", "uocr_cuda_moe_ep_experts", "uocr_cuda_moe_ep_shared", "uocr_cuda_moe_ep_combine",
    "uocr_cuda_moe_ep_peer_forward", "uocr_cuda_moe_ep_peer_last_offsets", "uocr_cuda_moe_ep_peer_create", "uocr_cuda_moe_ep_peer_open", "uocr_cuda_moe_ep_peer_destroy",
    "uocr_cuda_moe_ep_peer_dispatch", "uocr_cuda_moe_ep_peer_scatter", "uocr_cuda_moe_ep_peer_experts",
    "uocr_cuda_moe_ep_peer_combine", "uocr_cuda_moe_ep_peer_scatter_dev", "uocr_cuda_moe_ep_peer_experts_dev",
)


def profile_event_names() -> list[str]:
    """Names under which the backend reports phase durations to the engine's profile store."""
    lib, out, i = load_library(), [], 0
    while (name := lib.uocr_cuda_profile_event_name(i)) is not None:
        out.append(name.decode())
        i += 1
    return out


def library_path() -> Path:
    """UOCR_CUDA_LIBRARY_PATH, else the in-tree build next to this file (the reference uses
    UOCR_LIBRARY_PATH / build/release the same way, src/unlimitedocr_c/ffi.py:283)."""
    env = os.environ.get("UOCR_CUDA_LIBRARY_PATH")
    return Path(env) if env else Path(__file__).resolve().parent / "libuocr_cuda_moe.so"


_lib = None


def load_library() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists():
        raise UocrCudaError(f"{path} not found: build it with `make -C {path.parent / 'csrc'}`; there is no CPU fallback")
    lib = C.CDLL(str(path))
    vp, u32, u64, sz, cp = C.c_void_p, C.c_uint32, C.c_uint64, C.c_size_t, C.c_char_p
    err = [cp, sz]
    sig = {
        "uocr_cuda_is_available": (C.c_int, []),
        "uocr_cuda_backend_name": (cp, []),
        "uocr_cuda_device_count": (C.c_int, []),
        "uocr_cuda_context_create": (vp, [cp] + err),
        "uocr_cuda_context_destroy": (None, [vp]),
        "uocr_cuda_context_last_error": (cp, [vp]),
        "uocr_cuda_context_set_stream": (C.c_int, [vp, vp]),
        "uocr_cuda_context_set_profile_detail": (C.c_int, [vp, vp]),
        "uocr_cuda_context_set_profile": (None, [vp, vp, PROFILE_ADD_EVENT_FN]),
        "uocr_cuda_context_set_memory_tracker": (None, [vp, vp, MEMORY_ACCOUNT_FN, MEMORY_ACCOUNT_FN]),
        "uocr_cuda_profile_event_name": (cp, [u32]),
        "uocr_cuda_context_synchronize": (C.c_int, [vp] + err),
        "uocr_cuda_context_kernel_launches": (u64, [vp]),
        "uocr_cuda_context_model_view_bytes": (u64, [vp]),
        "uocr_cuda_context_moe_scratch_bytes": (u64, [vp]),
        "uocr_cuda_context_map_moe_layer": (C.c_int, [vp, C.POINTER(CLayerDesc), C.POINTER(u32)] + err),
        "uocr_cuda_context_map_model": (C.c_int, [vp, C.POINTER(CModelFileView)] + err),
        "uocr_cuda_context_unmap_model": (None, [vp]),
        "uocr_cuda_rmsnorm": (C.c_int, [vp, vp, vp, C.c_float, u32, u32, vp] + err),
        "uocr_cuda_moe_layer_forward_normed": (C.c_int, [vp, u32, vp, vp, C.c_float, u32, vp, C.POINTER(CDebugOutputs)] + err),
        "uocr_cuda_context_map_dense_mlp": (C.c_int, [vp, C.POINTER(CMatrix), C.POINTER(CMatrix), C.POINTER(CMatrix), u32, C.POINTER(u32)] + err),
        "uocr_cuda_dense_mlp_forward": (C.c_int, [vp, u32, vp, vp, u32, vp] + err),
        "uocr_cuda_dense_mlp_forward_normed": (C.c_int, [vp, u32, vp, vp, C.c_float, u32, vp] + err),
        "uocr_cuda_context_map_lm_head": (C.c_int, [vp, C.POINTER(CMatrix)] + err),
        "uocr_cuda_lm_head_argmax": (C.c_int, [vp, vp, u32, vp, vp] + err),
        "uocr_cuda_context_moe_layer_count": (u32, [vp]),
        "uocr_cuda_context_map_model_neighbours": (C.c_int, [vp, C.POINTER(CModelFileView), u32] + err),
        "uocr_cuda_context_file_dense_mlp_index": (C.c_int, [vp]),
        "uocr_cuda_context_post_attn_norm_weight": (vp, [vp, u32]),
        "uocr_cuda_context_final_norm_weight": (vp, [vp]),
        "uocr_cuda_context_allocate_runtime_arenas": (C.c_int, [vp, u32, u32] + err),
        "uocr_cuda_context_release_runtime_arenas": (None, [vp]),
        "uocr_cuda_moe_scratch_size": (u64, [u32] * 6),
        "uocr_cuda_moe_router": (C.c_int, [vp, u32, vp, vp, u32, vp, vp, vp, vp] + err),
        "uocr_cuda_moe_dispatch_plan": (C.c_int, [vp, vp, u32, u32, u32, vp, vp, vp] + err),
        "uocr_cuda_moe_dispatch_plan_noalloc": (C.c_int, [vp, u32, u32, u32, vp, vp, vp, vp] + err),
        "uocr_cuda_moe_debug_dequantize": (C.c_int, [vp, u32, u32, u32, u32, vp] + err),
        "uocr_cuda_moe_regime_name": (cp, [vp, u32, u32]),
        "uocr_cuda_moe_layer_forward": (C.c_int, [vp, u32, vp, vp, vp, u32, vp, C.POINTER(CDebugOutputs)] + err),
        "uocr_cuda_moe_stack_forward": (C.c_int, [vp, u32, u32, vp, u32, vp] + err),
        "uocr_cuda_moe_layer_forward_host": (C.c_int, [vp, u32, vp, vp, u32, vp, vp, vp] + err),
        "uocr_cuda_moe_stack_forward_host": (C.c_int, [vp, u32, u32, vp, u32, vp] + err),
        "uocr_cuda_moe_ep_dispatch": (C.c_int, [vp, u32, vp, u32, vp, vp] + err),
        "uocr_cuda_moe_ep_experts": (C.c_int, [vp, u32, u32, u32, u32, vp, vp, vp] + err),
        "uocr_cuda_moe_ep_shared": (C.c_int, [vp, u32, vp, u32] + err),
        "uocr_cuda_moe_ep_combine": (C.c_int, [vp, u32, vp, vp, u32, vp] + err),
        "uocr_cuda_moe_ep_peer_create": (C.c_int, [vp, u32, C.c_uint64, vp] + err),
        "uocr_cuda_moe_ep_peer_open": (C.c_int, [vp, u32, u32, vp] + err),
        "uocr_cuda_moe_ep_peer_destroy": (None, [vp]),
        "uocr_cuda_moe_ep_peer_dispatch": (C.c_int, [vp, u32, vp, u32, vp] + err),
        "uocr_cuda_moe_ep_peer_scatter": (C.c_int, [vp, u32, vp, u32, vp] + err),
        "uocr_cuda_moe_ep_peer_experts": (C.c_int, [vp, u32, u32, vp] + err),
        "uocr_cuda_moe_ep_peer_combine": (C.c_int, [vp, u32, vp, u32, vp] + err),
        "uocr_cuda_moe_ep_peer_forward": (C.c_int, [vp, u32, vp, vp, u32, vp] + err),
        "uocr_cuda_moe_ep_peer_last_offsets": (C.c_int, [vp, u32, vp] + err),
        "uocr_cuda_moe_ep_peer_scatter_dev": (C.c_int, [vp, u32, vp, u32, vp] + err),
        "uocr_cuda_moe_ep_peer_experts_dev": (C.c_int, [vp, u32] + err),
    }
    assert set(sig) == set(EXPORTS)
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def _np_ptr(a: np.ndarray | None) -> int | None:
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


def _dev_ptr(t: Any) -> int | None:
    """Device pointer of a torch CUDA tensor (or an int address, or None)."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    assert t.is_cuda and t.is_contiguous()
    return t.data_ptr()


def make_layer_desc(L: Any) -> tuple[CLayerDesc, list]:
    """Descriptor over host arrays.  L exposes H, E, K, F, S, scaling, router (uint16 [E,H]),
    logit_bias (f32 [E] or None), expert_qtype, expert_qweight (uint8), expert_qscale (uint16 or None),
    shared_gate/up/down with qtype, rows, cols, qweight, qscale; L.meta["strides"] may give the six slab strides
    and offsets of a slab that is not densely packed.  Returns the struct and the arrays
    it points into (keep them alive until the map call returns)."""
    keep = [L.router, L.logit_bias, L.expert_qweight, L.expert_qscale]
    mats = []
    for m in (L.shared_gate, L.shared_up, L.shared_down):
        keep += [m.qweight, m.qscale]
        mats.append(CMatrix(m.qtype, m.rows, m.cols, _np_ptr(m.qweight), _np_ptr(m.qscale)))
    st = (getattr(L, "meta", None) or {}).get("strides", {})      # absent: densely packed (zeros)
    d = CLayerDesc(L.H, L.E, L.K, L.F, L.S, L.scaling, _np_ptr(L.router), _np_ptr(L.logit_bias), L.expert_qtype,
                   _np_ptr(L.expert_qweight), _np_ptr(L.expert_qscale), st.get("expert_stride_bytes", 0),
                   st.get("up_offset_bytes", 0), st.get("down_offset_bytes", 0), st.get("expert_scale_stride_values", 0),
                   st.get("up_scale_offset_values", 0), st.get("down_scale_offset_values", 0), *mats)
    return d, keep


def dispatch_plan_noalloc(top_ids, n_tokens: int, top_k: int, n_experts: int, expert_offsets, pair_rows, inverse,
                          cuda_stream: int | None = None) -> None:
    """Dispatch plan without a context, an arena or any device allocation (see the header for who needs this).
    Arguments are device buffers (torch CUDA tensors or addresses) on the current device."""
    lib = load_library()
    err = C.create_string_buffer(_ERR)
    if cuda_stream == 0:
        cuda_stream = 1   # cudaStreamLegacy
    ok = lib.uocr_cuda_moe_dispatch_plan_noalloc(_dev_ptr(top_ids), n_tokens, top_k, n_experts, _dev_ptr(expert_offsets),
                                                 _dev_ptr(pair_rows), _dev_ptr(inverse), cuda_stream, err, _ERR)
    if ok != 1:
        raise UocrCudaError(err.value.decode())


class Context:
    """One backend context on the current CUDA device (the reference's Engine plays this role for
    the whole model; this one holds MoE layers only)."""

    def __init__(self) -> None:
        self._lib = load_library()
        self._err = C.create_string_buffer(_ERR)
        self._h = None
        if not self._lib.uocr_cuda_is_available():
            raise UocrCudaError("no CUDA device visible; this backend has no CPU fallback")
        h = self._lib.uocr_cuda_context_create(None, self._err, _ERR)
        if not h:
            raise UocrCudaError(self._err.value.decode())
        self._h = h
        self._layer_k: dict[int, int] = {}
        self._layer_e: dict[int, int] = {}

    def close(self) -> None:
        if self._h:
            self._lib.uocr_cuda_context_destroy(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, ok: int) -> None:
        if ok != 1:
            raise UocrCudaError(self._err.value.decode() or self._lib.uocr_cuda_context_last_error(self._h).decode())

    # -- model and arenas
    def map_layer(self, L: Any) -> int:
        desc, keep = make_layer_desc(L)
        idx = self.map_layer_desc(desc)
        del keep
        return idx

    def map_layer_desc(self, desc: CLayerDesc) -> int:
        idx = C.c_uint32(0xFFFFFFFF)
        self._check(self._lib.uocr_cuda_context_map_moe_layer(self._h, C.byref(desc), C.byref(idx), self._err, _ERR))
        self._layer_k[idx.value] = desc.top_k
        self._layer_e[idx.value] = desc.n_experts
        return idx.value

    def map_model(self, data_address: int, size: int, tensors_address: int, tensor_count: int, *, routed_experts: int,
                  top_k: int, first_moe_layer: int, moe_layer_count: int, routed_scaling_factor: float = 1.0) -> int:
        """Map the MoE layers of an opened `.uocr` file (uocr_cuda_context_map_model).  `data_address` is the address
        of the file's first byte in host memory (a memory map or a buffer the caller keeps alive during the call),
        `tensors_address` the address of its tensor directory entries.  Returns the number of layers mapped."""
        view = CModelFileView(data_address, size, tensors_address, tensor_count, routed_experts, top_k, first_moe_layer,
                              moe_layer_count, routed_scaling_factor)
        self._check(self._lib.uocr_cuda_context_map_model(self._h, C.byref(view), self._err, _ERR))
        for i in range(moe_layer_count):
            self._layer_k[i] = top_k
            self._layer_e[i] = routed_experts
        return int(self._lib.uocr_cuda_context_moe_layer_count(self._h))

    def map_model_neighbours(self, data_address: int, size: int, tensors_address: int, tensor_count: int, *, token_capacity: int,
                             first_moe_layer: int, moe_layer_count: int) -> dict:
        """Map what the file holds either side of the MoE layers (uocr_cuda_context_map_model_neighbours): the dense MLP of
        decoder layer 0, the LM head, the post-attention norm weights and the final norm.  Returns
        {"dense_mlp": index or None, "lm_head": bool, "post_attn_norm": {layer: device address}, "final_norm": address or None}."""
        view = CModelFileView(data_address, size, tensors_address, tensor_count, 0, 0, first_moe_layer, moe_layer_count, 1.0)
        self._check(self._lib.uocr_cuda_context_map_model_neighbours(self._h, C.byref(view), token_capacity, self._err, _ERR))
        idx = int(self._lib.uocr_cuda_context_file_dense_mlp_index(self._h))
        norms = {}
        for layer in range(first_moe_layer + moe_layer_count):
            p = self._lib.uocr_cuda_context_post_attn_norm_weight(self._h, layer)
            if p:
                norms[layer] = int(p)
        fin = self._lib.uocr_cuda_context_final_norm_weight(self._h)
        return {"dense_mlp": None if idx < 0 else idx, "post_attn_norm": norms, "final_norm": int(fin) if fin else None}

    # -- the steps either side of the MoE layer
    def rmsnorm(self, x, weight, eps: float, n_tokens: int, hidden_size: int, out) -> None:
        self._check(self._lib.uocr_cuda_rmsnorm(self._h, _dev_ptr(x), _dev_ptr(weight), eps, n_tokens, hidden_size, _dev_ptr(out),
                                                self._err, _ERR))

    def layer_forward_normed(self, layer: int, stream_rows, norm_weight, eps: float, n_tokens: int, out) -> None:
        """out = MoE(RMSNorm(stream_rows) * norm_weight) + stream_rows (uocr_cuda_moe_layer_forward_normed)."""
        self._check(self._lib.uocr_cuda_moe_layer_forward_normed(self._h, layer, _dev_ptr(stream_rows), _dev_ptr(norm_weight), eps,
                                                                 n_tokens, _dev_ptr(out), None, self._err, _ERR))

    def map_dense_mlp(self, gate: Any, up: Any, down: Any, token_capacity: int) -> int:
        """gate / up / down: objects with qtype, rows, cols, qweight, qscale (host arrays), e.g. oracle.quant.Matrix."""
        keep, cm = [], []
        for m in (gate, up, down):
            w = np.ascontiguousarray(m.qweight)
            sc = None if m.qscale is None else np.ascontiguousarray(m.qscale)
            keep += [w, sc]
            cm.append(CMatrix(m.qtype, m.rows, m.cols, w.ctypes.data, None if sc is None else sc.ctypes.data))
        idx = C.c_uint32(0xFFFFFFFF)
        self._check(self._lib.uocr_cuda_context_map_dense_mlp(self._h, C.byref(cm[0]), C.byref(cm[1]), C.byref(cm[2]), token_capacity,
                                                              C.byref(idx), self._err, _ERR))
        del keep
        return idx.value

    def dense_mlp_forward(self, index: int, hidden, n_tokens: int, out, *, residual=None) -> None:
        self._check(self._lib.uocr_cuda_dense_mlp_forward(self._h, index, _dev_ptr(hidden), _dev_ptr(residual), n_tokens,
                                                          _dev_ptr(out), self._err, _ERR))

    def dense_mlp_forward_normed(self, index: int, stream_rows, norm_weight, eps: float, n_tokens: int, out) -> None:
        self._check(self._lib.uocr_cuda_dense_mlp_forward_normed(self._h, index, _dev_ptr(stream_rows), _dev_ptr(norm_weight), eps,
                                                                 n_tokens, _dev_ptr(out), self._err, _ERR))

    def map_lm_head(self, weight: Any) -> None:
        """weight: object with qtype, rows (vocabulary), cols (hidden), qweight, qscale (host arrays)."""
        w = np.ascontiguousarray(weight.qweight)
        sc = None if weight.qscale is None else np.ascontiguousarray(weight.qscale)
        cm = CMatrix(weight.qtype, weight.rows, weight.cols, w.ctypes.data, None if sc is None else sc.ctypes.data)
        self._check(self._lib.uocr_cuda_context_map_lm_head(self._h, C.byref(cm), self._err, _ERR))

    def lm_head_argmax(self, hidden, n_tokens: int, token_ids, scores=None) -> None:
        self._check(self._lib.uocr_cuda_lm_head_argmax(self._h, _dev_ptr(hidden), n_tokens, _dev_ptr(token_ids), _dev_ptr(scores),
                                                       self._err, _ERR))

    def release_runtime_arenas(self) -> None:
        self._lib.uocr_cuda_context_release_runtime_arenas(self._h)

    def unmap_model(self) -> None:
        self._lib.uocr_cuda_context_unmap_model(self._h)

    def allocate_runtime_arenas(self, token_capacity: int, batch_slots: int = 1) -> None:
        self._check(self._lib.uocr_cuda_context_allocate_runtime_arenas(self._h, batch_slots, token_capacity,
                                                                        self._err, _ERR))

    def set_stream(self, cuda_stream: int | None) -> None:
        """Run on the given cudaStream_t (e.g. torch.cuda.current_stream().cuda_stream); None restores the
        context's own stream.  Handle 0 names the legacy default stream and is passed as cudaStreamLegacy."""
        if cuda_stream == 0:
            cuda_stream = 1   # cudaStreamLegacy
        self._check(self._lib.uocr_cuda_context_set_stream(self._h, cuda_stream))

    def set_profile(self, add_event_ms) -> None:
        """add_event_ms(name: str, ms: float) receives the duration of every phase (see the header for the names); None
        switches it off.  Stands in for the engine's profile store."""
        if add_event_ms is None:
            self._profile_cb = None
            self._lib.uocr_cuda_context_set_profile(self._h, None, PROFILE_ADD_EVENT_FN())
            return
        self._profile_cb = PROFILE_ADD_EVENT_FN(lambda _store, name, ms: add_event_ms(name.decode(), ms))
        self._lib.uocr_cuda_context_set_profile(self._h, 1, self._profile_cb)

    def set_memory_tracker(self, reserve, release) -> None:
        """reserve(category: int, bytes: int) / release(category, bytes): stand-ins for the engine's memory tracker."""
        self._mem_cbs = (MEMORY_ACCOUNT_FN(lambda _t, cat, b: (reserve(cat, b), 1)[1]),
                         MEMORY_ACCOUNT_FN(lambda _t, cat, b: (release(cat, b), 1)[1]))
        self._lib.uocr_cuda_context_set_memory_tracker(self._h, 1, *self._mem_cbs)

    def set_profile_detail(self, trace) -> None:
        """Device buffer (128 * n_layers * 16 int64) that single-token stack calls fill with per-phase SM clocks:
        CTA c, layer l, point p at [(c * n_layers + l) * 16 + p] (see the header for the points; the two-barrier
        kernel writes CTA 0 only, 8 points per layer at stride 8)."""
        self._check(self._lib.uocr_cuda_context_set_profile_detail(self._h, _dev_ptr(trace)))

    def synchronize(self) -> None:
        self._check(self._lib.uocr_cuda_context_synchronize(self._h, self._err, _ERR))

    @property
    def layer_count(self) -> int:
        return self._lib.uocr_cuda_context_moe_layer_count(self._h)

    @property
    def kernel_launches(self) -> int:
        return self._lib.uocr_cuda_context_kernel_launches(self._h)

    @property
    def model_view_bytes(self) -> int:
        return self._lib.uocr_cuda_context_model_view_bytes(self._h)

    @property
    def moe_scratch_bytes(self) -> int:
        return self._lib.uocr_cuda_context_moe_scratch_bytes(self._h)

    # -- operators on device buffers (torch CUDA tensors or raw addresses)
    def router(self, layer: int, hidden, n_tokens: int, top_ids, top_weights, *, injected_logits=None, logits=None,
               probs=None) -> None:
        self._check(self._lib.uocr_cuda_moe_router(self._h, layer, _dev_ptr(hidden), _dev_ptr(injected_logits),
                                                   n_tokens, _dev_ptr(logits), _dev_ptr(probs), _dev_ptr(top_ids),
                                                   _dev_ptr(top_weights), self._err, _ERR))

    def dispatch_plan(self, top_ids, n_tokens: int, top_k: int, n_experts: int, expert_offsets, pair_rows,
                      inverse) -> None:
        self._check(self._lib.uocr_cuda_moe_dispatch_plan(self._h, _dev_ptr(top_ids), n_tokens, top_k, n_experts,
                                                          _dev_ptr(expert_offsets), _dev_ptr(pair_rows),
                                                          _dev_ptr(inverse), self._err, _ERR))

    def debug_dequantize(self, layer: int, matrix: int, expert: int, path: int, out) -> None:
        """Weights of one projection as the kernels see them (f32 [rows, cols] device tensor); see the header."""
        self._check(self._lib.uocr_cuda_moe_debug_dequantize(self._h, layer, matrix, expert, path, _dev_ptr(out),
                                                             self._err, _ERR))

    def regime_name(self, layer: int, n_tokens: int) -> str:
        """The kernels a layer call with n_tokens tokens would run."""
        return self._lib.uocr_cuda_moe_regime_name(self._h, layer, n_tokens).decode()

    def layer_forward(self, layer: int, hidden, n_tokens: int, out, *, residual=None, injected_logits=None,
                      logits=None, probs=None, top_ids=None, top_weights=None) -> None:
        dbg = None
        if any(x is not None for x in (logits, probs, top_ids, top_weights)):
            dbg = C.byref(CDebugOutputs(_dev_ptr(logits), _dev_ptr(probs), _dev_ptr(top_ids), _dev_ptr(top_weights)))
        self._check(self._lib.uocr_cuda_moe_layer_forward(self._h, layer, _dev_ptr(hidden), _dev_ptr(residual),
                                                          _dev_ptr(injected_logits), n_tokens, _dev_ptr(out), dbg,
                                                          self._err, _ERR))

    def stack_forward(self, first_layer: int, n_layers: int, hidden, n_tokens: int, out) -> None:
        self._check(self._lib.uocr_cuda_moe_stack_forward(self._h, first_layer, n_layers, _dev_ptr(hidden), n_tokens,
                                                          _dev_ptr(out), self._err, _ERR))

    # -- expert-parallel phases (device buffers)
    def ep_dispatch(self, layer: int, hidden, n_tokens: int, sorted_rows, expert_offsets) -> None:
        """Router, plan and gather; expert_offsets (device int32 [E+1]) gets the prefix sum of pairs per expert."""
        self._check(self._lib.uocr_cuda_moe_ep_dispatch(self._h, layer, _dev_ptr(hidden), n_tokens, _dev_ptr(sorted_rows),
                                                        _dev_ptr(expert_offsets), self._err, _ERR))

    def ep_experts(self, layer: int, first_expert: int, n_local_experts: int, segment_counts: np.ndarray, rows_in,
                   rows_out) -> None:
        """segment_counts: uint32 [n_sources, n_local_experts] rows received per (source, local expert)."""
        seg = np.ascontiguousarray(segment_counts, np.uint32).reshape(-1, n_local_experts)
        self._check(self._lib.uocr_cuda_moe_ep_experts(self._h, layer, first_expert, n_local_experts, seg.shape[0],
                                                       _np_ptr(seg), _dev_ptr(rows_in), _dev_ptr(rows_out), self._err, _ERR))

    def ep_shared(self, layer: int, hidden, n_tokens: int) -> None:
        self._check(self._lib.uocr_cuda_moe_ep_shared(self._h, layer, _dev_ptr(hidden), n_tokens, self._err, _ERR))

    def ep_combine(self, layer: int, rows_back, n_tokens: int, out, *, residual=None) -> None:
        self._check(self._lib.uocr_cuda_moe_ep_combine(self._h, layer, _dev_ptr(rows_back), _dev_ptr(residual), n_tokens,
                                                       _dev_ptr(out), self._err, _ERR))

    # -- expert-parallel phases with the exchange over peer memory
    def ep_peer_create(self, hidden_size: int, row_capacity: int) -> bytes:
        """Allocates this rank's exchange buffers; returns the 128 bytes of IPC handles to gather over the group."""
        buf = C.create_string_buffer(128)
        self._check(self._lib.uocr_cuda_moe_ep_peer_create(self._h, hidden_size, row_capacity, buf, self._err, _ERR))
        return buf.raw

    def ep_peer_open(self, world: int, rank: int, all_handles: bytes) -> None:
        if len(all_handles) != 128 * world:
            raise ValueError("all_handles must hold 128 bytes per rank")
        self._check(self._lib.uocr_cuda_moe_ep_peer_open(self._h, world, rank, C.c_char_p(all_handles), self._err, _ERR))

    def ep_peer_destroy(self) -> None:
        self._lib.uocr_cuda_moe_ep_peer_destroy(self._h)

    def ep_peer_dispatch(self, layer: int, hidden, n_tokens: int, expert_offsets) -> None:
        self._check(self._lib.uocr_cuda_moe_ep_peer_dispatch(self._h, layer, _dev_ptr(hidden), n_tokens, _dev_ptr(expert_offsets),
                                                             self._err, _ERR))

    def ep_peer_scatter(self, layer: int, hidden, n_tokens: int, dst_row0: np.ndarray) -> None:
        d = np.ascontiguousarray(dst_row0, np.uint32)
        self._check(self._lib.uocr_cuda_moe_ep_peer_scatter(self._h, layer, _dev_ptr(hidden), n_tokens, _np_ptr(d), self._err, _ERR))

    def ep_peer_experts(self, layer: int, segment_counts: np.ndarray) -> None:
        seg = np.ascontiguousarray(segment_counts, np.uint32)
        self._check(self._lib.uocr_cuda_moe_ep_peer_experts(self._h, layer, seg.shape[0], _np_ptr(seg), self._err, _ERR))

    def ep_peer_scatter_dev(self, layer: int, hidden, n_tokens: int, all_offsets) -> None:
        """all_offsets: device int32 [world, E + 1], every rank's expert offsets; row offsets are computed on the device."""
        self._check(self._lib.uocr_cuda_moe_ep_peer_scatter_dev(self._h, layer, _dev_ptr(hidden), n_tokens, _dev_ptr(all_offsets),
                                                                self._err, _ERR))

    def ep_peer_experts_dev(self, layer: int) -> None:
        self._check(self._lib.uocr_cuda_moe_ep_peer_experts_dev(self._h, layer, self._err, _ERR))

    def ep_peer_forward(self, layer: int, hidden, n_tokens: int, out, *, residual=None) -> None:
        """The whole expert-parallel layer call, the ranks synchronised on the device (uocr_cuda_moe_ep_peer_forward)."""
        self._check(self._lib.uocr_cuda_moe_ep_peer_forward(self._h, layer, _dev_ptr(hidden), _dev_ptr(residual), n_tokens,
                                                            _dev_ptr(out), self._err, _ERR))

    def ep_peer_last_offsets(self, world: int, n_experts: int) -> np.ndarray:
        """Every rank's expert offsets of the last ep_peer_forward call, uint32 [world, n_experts + 1]."""
        out = np.zeros((world, n_experts + 1), dtype=np.uint32)
        self._check(self._lib.uocr_cuda_moe_ep_peer_last_offsets(self._h, n_experts, out.ctypes.data, self._err, _ERR))
        return out

    def ep_peer_combine(self, layer: int, n_tokens: int, out, *, residual=None) -> None:
        self._check(self._lib.uocr_cuda_moe_ep_peer_combine(self._h, layer, _dev_ptr(residual), n_tokens, _dev_ptr(out),
                                                            self._err, _ERR))

    # -- operators on host buffers (numpy uint16 fp16 bits)
    def layer_forward_host(self, layer: int, hidden: np.ndarray, residual: np.ndarray | None = None, *,
                           want_routing: bool = False):
        hidden = np.ascontiguousarray(hidden, np.uint16)
        n = hidden.shape[0]
        out = np.empty_like(hidden)
        ids = wts = None
        if want_routing:
            k = self._layer_k[layer]
            ids, wts = np.empty((n, k), np.uint32), np.empty((n, k), np.float32)
        if residual is not None:
            residual = np.ascontiguousarray(residual, np.uint16)
        self._check(self._lib.uocr_cuda_moe_layer_forward_host(self._h, layer, _np_ptr(hidden), _np_ptr(residual), n,
                                                               _np_ptr(out), _np_ptr(ids), _np_ptr(wts), self._err,
                                                               _ERR))
        return (out, ids, wts) if want_routing else out

    def stack_forward_host(self, first_layer: int, n_layers: int, hidden: np.ndarray) -> np.ndarray:
        """Host buffers in and out (fp16 bits).  One token through the decode kernel issues no copies: the
        activations travel in the launch parameters and the kernel writes result and status into mapped host memory."""
        hidden = np.ascontiguousarray(hidden, np.uint16)
        out = np.empty_like(hidden)
        self._check(self._lib.uocr_cuda_moe_stack_forward_host(self._h, first_layer, n_layers, _np_ptr(hidden),
                                                               hidden.shape[0], _np_ptr(out), self._err, _ERR))
        return out
