"""ctypes view of the resident model plan (gf_model_*) and of operator-level entry points."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib
from .lib import check, load

vp, u32, u64, i32, sz, f32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int, C.c_size_t, C.c_float


class ModelConfig(C.Structure):
    _fields_ = [(n, u32) for n in ("hidden", "ffn", "heads", "kv_heads", "head_dim", "layers", "vocab",
                                   "sliding_window", "sliding_pattern")] + \
               [(n, f32) for n in ("rope_base_global", "rope_scale_global", "rope_base_local", "rope_scale_local",
                                   "rms_eps", "attn_softcap", "final_softcap")] + \
               [("uses_qk_norm", C.c_int32), ("kv_f16", C.c_int32), ("attention_scale", f32),
                ("context", u32), ("row_capacity", u32)]


class SelectionRequest(C.Structure):
    _fields_ = [("retain", u32), ("history_count", u32), ("history", u32 * 64)]


class CandidateResult(C.Structure):
    class _Pair(C.Structure):
        _fields_ = [("token", u32), ("logit", f32)]
    _fields_ = [("status", u32), ("count", u32), ("candidates", _Pair * 384)]

    def pairs(self):
        out = np.zeros(self.count, np.dtype([("token", np.uint32), ("logit", np.float32)]))
        for i in range(self.count):
            out[i] = (self.candidates[i].token, self.candidates[i].logit)
        return out


lib.register({
    "gf_embedding": (i32, [i32, vp, u32, u32, vp, u32, f32, vp, vp, vp]),
    "gf_rms_norm": (i32, [vp, vp, vp, u32, u32, f32, vp]),
    "gf_rms_norm_add": (i32, [vp, vp, vp, vp, u32, u32, f32, vp]),
    "gf_qk_norm_rope_store": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, f32, f32, f32, i32, vp]),
    "gf_rope_store_rows": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, f32, f32, f32, i32, vp]),
    "gf_attention_workspace_bytes": (sz, [u32, u32]),
    "gf_attention": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, f32, f32, i32, vp]),
    "gf_prefill_attention": (i32, [vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, f32, f32, vp]),
    "gf_gelu_tanh_multiply": (i32, [vp, vp, vp, u64, vp]),
    "gf_kv_scatter": (i32, [vp, vp, vp, vp, vp, u32, u32, u32, i32, vp]),
    "gf_selection_request_bytes": (sz, []),
    "gf_candidate_result_bytes": (sz, []),
    "gf_token_candidates_workspace_bytes": (sz, [u32, u32]),
    "gf_token_candidates": (i32, [vp, u32, u32, f32, vp, vp, vp, vp]),
    "gf_model_create": (i32, [C.POINTER(ModelConfig), C.POINTER(vp)]),
    "gf_model_destroy": (i32, [vp]),
    "gf_model_set_matrix": (i32, [vp, i32, u32, i32, vp, u64, u64]),
    "gf_model_set_matrix_requantized": (i32, [vp, i32, u32, vp, u64, u64]),
    "gf_model_set_vector": (i32, [vp, i32, u32, vp, u32]),
    "gf_model_load_gguf": (i32, [vp, C.c_char_p, vp]),
    "gf_model_set_reduce_hook": (i32, [vp, vp, vp]),
    "gf_model_set_token_table_vocab": (i32, [vp, u32]),
    "gf_model_shard_prepare": (i32, [vp, u32, u32, vp]),
    "gf_model_shard_arena": (vp, [vp]),
    "gf_model_shard_arena_bytes": (sz, [vp]),
    "gf_model_shard_connect": (i32, [vp, vp]),
    "gf_model_shard_connect_ipc": (i32, [vp, vp]),
    "gf_model_shard_set_wait_limit": (i32, [vp, u32]),
    "gf_model_shard_global_selection": (i32, [vp, i32]),
    "gf_add": (i32, [vp, vp, vp, u64, vp]),
    "gf_model_finalize": (i32, [vp]),
    "gf_model_reset": (i32, [vp]),
    "gf_model_position": (i32, [vp, C.POINTER(u32)]),
    "gf_model_forward": (i32, [vp, vp, u32, u32]),
    "gf_model_publish": (i32, [vp, u32]),
    "gf_model_prefill": (i32, [vp, vp, u32]),
    "gf_model_truncate": (i32, [vp, u32]),
    "gf_model_select": (i32, [vp, vp, u32]),
    "gf_model_read_candidates": (i32, [vp, vp, u32]),
    "gf_model_read_logits": (i32, [vp, u32, vp]),
    "gf_model_read_kv": (i32, [vp, u32, u32, u32, vp, vp]),
    "gf_model_synchronize": (i32, [vp]),
    "gf_model_status": (i32, [vp, C.POINTER(u32)]),
    "gf_model_stream": (vp, [vp]),
    "gf_model_tokens_dev": (vp, [vp]),
    "gf_model_logits_dev": (vp, [vp]),
    "gf_model_weight_bytes": (sz, [vp, i32]),
    "gf_model_kv_bytes_per_pass": (sz, [vp, u32]),
    "gf_model_kernel_launches": (u32, [vp]),
    "gf_model_use_graph": (i32, [vp, i32]),
    "gf_model_use_pass_kernel": (i32, [vp, i32]),
    "gf_model_use_tensor_prefill": (i32, [vp, i32]),
    "gf_model_prefill_logits_row": (u32, [vp]),
    "gf_model_weight_sweep": (i32, [vp, u32, C.POINTER(u32), C.POINTER(u64)]),
    "gf_streams_create": (i32, [vp, u32, C.POINTER(vp)]),
    "gf_streams_destroy": (i32, [vp]),
    "gf_streams_count": (u32, [vp]),
    "gf_streams_prefill": (i32, [vp, u32, vp, u32]),
    "gf_streams_decode": (i32, [vp, vp]),
    "gf_streams_set_mode": (i32, [vp, i32]),
    "gf_streams_select": (i32, [vp, vp]),
    "gf_streams_read_candidates": (i32, [vp, vp]),
    "gf_streams_read_logits": (i32, [vp, u32, vp]),
    "gf_streams_position": (i32, [vp, u32, C.POINTER(u32)]),
    "gf_streams_kv_bytes_per_step": (sz, [vp]),
})

MATRIX_KINDS = {"token_embd": 0, "output": 1, "attn_q": 2, "attn_k": 3, "attn_v": 4, "attn_output": 5,
                "ffn_gate": 6, "ffn_up": 7, "ffn_down": 8}
VECTOR_KINDS = {"output_norm": 0, "attn_norm": 1, "post_attention_norm": 2, "ffn_norm": 3, "post_ffw_norm": 4,
                "attn_q_norm": 5, "attn_k_norm": 6}
FORWARD_LOGITS, FORWARD_DEVICE_TOKENS = 1, 2


def make_config(config: dict, context: int, row_capacity: int = 2) -> ModelConfig:
    cfg = ModelConfig()
    for name, _ in ModelConfig._fields_:
        if name in config:
            setattr(cfg, name, config[name])
    cfg.context, cfg.row_capacity = context, row_capacity
    return cfg


def selection_request(retain: int, history=()) -> SelectionRequest:
    request = SelectionRequest()
    request.retain = retain
    request.history_count = len(history)
    for i, token in enumerate(history):
        request.history[i] = int(token)
    return request


class Model:
    """A resident Gemma plan on the current device.  `weights` is the dict produced by
    guffin_b200.synthetic.make_model_weights (GGUF tensor names), any iterable of
    (name, value) pairs such as synthetic.iter_model_weights, or the path of a GGUF file."""

    def __init__(self, config: dict, weights, context: int, row_capacity: int = 2, before_binding=None):
        self.L = load()
        self.config = dict(config)
        self.cfg = make_config(config, context, row_capacity)
        handle = vp()
        check(self.L.gf_model_create(C.byref(self.cfg), C.byref(handle)))
        self.handle = handle.value
        if before_binding is not None:          # options that must precede the weights (guffin_b200.tensor_parallel)
            before_binding(self)
        if isinstance(weights, (str, bytes)) or hasattr(weights, "__fspath__"):     # a GGUF file
            import os
            bound = u32()
            try:
                check(self.L.gf_model_load_gguf(self.handle, os.fsencode(weights), C.byref(bound)))
                check(self.L.gf_model_finalize(self.handle))
            except Exception:
                self.close()
                raise
            self.bound_tensors = bound.value
            return
        for name, value in (weights.items() if hasattr(weights, "items") else weights):
            parts = name.split(".")
            layer, short = (int(parts[1]), parts[2]) if parts[0] == "blk" else (0, parts[0])
            if isinstance(value, tuple):
                dtype, k, n, data = value[:4]
                data = np.ascontiguousarray(data).view(np.uint8)
                if len(value) > 4 and value[4] == "requantize":          # a Q6_K matrix bound as Q4_K
                    check(self.L.gf_model_set_matrix_requantized(self.handle, MATRIX_KINDS[short], layer, data.ctypes.data, k, n))
                else:
                    check(self.L.gf_model_set_matrix(self.handle, MATRIX_KINDS[short], layer, dtype, data.ctypes.data, k, n))
            else:
                data = np.ascontiguousarray(value, np.float32)
                check(self.L.gf_model_set_vector(self.handle, VECTOR_KINDS[short], layer, data.ctypes.data, data.size))
        check(self.L.gf_model_finalize(self.handle))

    @property
    def position(self) -> int:
        out = u32()
        check(self.L.gf_model_position(self.handle, C.byref(out)))
        return out.value

    def forward(self, tokens, logits: bool = True) -> None:
        tokens = np.ascontiguousarray(tokens, np.uint32)
        check(self.L.gf_model_forward(self.handle, tokens.ctypes.data, tokens.size, FORWARD_LOGITS if logits else 0))

    def forward_device_tokens(self, rows: int, logits: bool = True) -> None:
        check(self.L.gf_model_forward(self.handle, None, rows, (FORWARD_LOGITS if logits else 0) | FORWARD_DEVICE_TOKENS))

    def publish(self, rows: int) -> None:
        check(self.L.gf_model_publish(self.handle, rows))

    def prefill(self, tokens) -> None:
        tokens = np.ascontiguousarray(tokens, np.uint32)
        check(self.L.gf_model_prefill(self.handle, tokens.ctypes.data, tokens.size))

    def truncate(self, position: int) -> None:
        check(self.L.gf_model_truncate(self.handle, position))

    def reset(self) -> None:
        check(self.L.gf_model_reset(self.handle))

    def logits(self, row: int = 0) -> np.ndarray:
        out = np.empty(self.cfg.vocab, np.float32)
        check(self.L.gf_model_read_logits(self.handle, row, out.ctypes.data))
        return out

    def read_kv(self, layer: int, first: int, count: int):
        """Committed K and V rows [first, first + count) of one layer as f32 arrays [count, kv_width]."""
        width = self.cfg.kv_heads * self.cfg.head_dim
        k, v = np.empty((count, width), np.float32), np.empty((count, width), np.float32)
        check(self.L.gf_model_read_kv(self.handle, layer, first, count, k.ctypes.data, v.ctypes.data))
        return k, v

    def select(self, requests) -> list:
        rows = len(requests)
        array = (SelectionRequest * rows)(*requests)
        check(self.L.gf_model_select(self.handle, C.byref(array), rows))
        results = (CandidateResult * rows)()
        check(self.L.gf_model_read_candidates(self.handle, C.byref(results), rows))
        return list(results)

    def synchronize(self) -> None:
        check(self.L.gf_model_synchronize(self.handle))

    def status(self) -> int:
        out = u32()
        check(self.L.gf_model_status(self.handle, C.byref(out)))
        return out.value

    def weight_sweep(self, rows: int):
        launches, nbytes = u32(), u64()
        check(self.L.gf_model_weight_sweep(self.handle, rows, C.byref(launches), C.byref(nbytes)))
        return launches.value, nbytes.value

    def use_graph(self, enable: bool) -> None:
        check(self.L.gf_model_use_graph(self.handle, int(enable)))

    def use_tensor_prefill(self, enable: bool) -> None:
        """Long prompts through the 128-row bf16 tensor-core path (default) or the exact row path."""
        check(self.L.gf_model_use_tensor_prefill(self.handle, int(enable)))

    @property
    def prefill_logits_row(self) -> int:
        return self.L.gf_model_prefill_logits_row(self.handle)

    def use_pass_kernel(self, mode: int) -> None:
        """0: one kernel per operator; 1: the persistent decode pass kernel; 2: that, attention launched separately."""
        check(self.L.gf_model_use_pass_kernel(self.handle, int(mode)))

    @property
    def stream(self):
        return self.L.gf_model_stream(self.handle)

    def weight_bytes(self, native: bool = True) -> int:
        return self.L.gf_model_weight_bytes(self.handle, int(native))

    def kv_bytes_per_pass(self, rows: int) -> int:
        return self.L.gf_model_kv_bytes_per_pass(self.handle, rows)

    def kernel_launches(self) -> int:
        return self.L.gf_model_kernel_launches(self.handle)

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.L.gf_model_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Streams:
    """Independent conversation streams that share one plan's weights (gf_streams_*)."""

    def __init__(self, model: Model, count: int):
        self.L = load()
        self.model, self.count = model, count
        handle = vp()
        check(self.L.gf_streams_create(model.handle, count, C.byref(handle)))
        self.handle = handle.value

    def prefill(self, stream: int, tokens) -> None:
        tokens = np.ascontiguousarray(tokens, np.uint32)
        check(self.L.gf_streams_prefill(self.handle, stream, tokens.ctypes.data, tokens.size))

    def set_mode(self, mode: int) -> None:
        """0: exact row passes in groups; 1: one tensor-core pass over all streams (bf16 operands)."""
        check(self.L.gf_streams_set_mode(self.handle, mode))

    def decode(self, tokens) -> None:
        tokens = np.ascontiguousarray(tokens, np.uint32)
        assert tokens.size == self.count
        check(self.L.gf_streams_decode(self.handle, tokens.ctypes.data))

    def logits(self, stream: int) -> np.ndarray:
        out = np.empty(self.model.cfg.vocab, np.float32)
        check(self.L.gf_streams_read_logits(self.handle, stream, out.ctypes.data))
        return out

    def select(self, requests) -> list:
        assert len(requests) == self.count
        array = (SelectionRequest * self.count)(*requests)
        check(self.L.gf_streams_select(self.handle, C.byref(array)))
        results = (CandidateResult * self.count)()
        check(self.L.gf_streams_read_candidates(self.handle, C.byref(results)))
        return list(results)

    def greedy(self) -> np.ndarray:
        """The best token of every stream's current logits (one selection over all rows)."""
        results = self.select([selection_request(1)] * self.count)
        return np.array([r.candidates[0].token for r in results], np.uint32)

    def position(self, stream: int) -> int:
        out = u32()
        check(self.L.gf_streams_position(self.handle, stream, C.byref(out)))
        return out.value

    def kv_bytes_per_step(self) -> int:
        return self.L.gf_streams_kv_bytes_per_step(self.handle)

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.L.gf_streams_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
