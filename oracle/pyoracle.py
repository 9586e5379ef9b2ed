"""ctypes bindings for the CPU oracle.  TEST INFRASTRUCTURE ONLY.

`Oracle` loads liboracle.so (the C restatement, gf_oracle.c).  `Reference` loads
_ref/libguffin_ref.so (the reference engine's own CPU sources behind ref_shim.cpp) when it
has been built.  Only tests, the smoke check and bench.py's CPU-baseline legs may import this.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
Q8_0, Q4_K, Q6_K = 8, 12, 14
BLOCK_ELEMENTS = {Q8_0: 32, Q4_K: 256, Q6_K: 256}
BLOCK_BYTES = {Q8_0: 34, Q4_K: 144, Q6_K: 210}

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
_u64p = np.ctypeslib.ndpointer(np.uint64, flags="C_CONTIGUOUS")

TOKEN_LOGIT = np.dtype([("token", np.uint32), ("logit", np.float32)])
PROB = np.dtype([("token", np.uint32), ("pad", np.uint32), ("probability", np.float64), ("weight", np.float64)])


def reference_root() -> str:
    """Where the reference project is checked out: $GF_REFERENCE, else `reference` beside this repository."""
    return os.environ.get("GF_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(reference: bool = True) -> None:
    """Compile liboracle.so and, when the reference tree is present, _ref/libguffin_ref.so."""
    subprocess.run(["make", "-s", "-C", HERE, "oracle"], check=True)
    if reference:
        subprocess.run(["make", "-s", "-C", HERE, "ref"], check=False)


class SamplerOptions(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_uint32), ("top_p", C.c_float),
                ("min_p", C.c_float), ("repetition_penalty", C.c_float)]


class Distribution(C.Structure):
    class _Prob(C.Structure):
        _fields_ = [("token", C.c_uint32), ("probability", C.c_double), ("weight", C.c_double)]
    _fields_ = [("values", _Prob * 256), ("count", C.c_uint32), ("total_weight", C.c_double)]

    def tokens(self):
        return [self.values[i].token for i in range(self.count)]

    def weights(self):
        return [self.values[i].weight for i in range(self.count)]

    def probabilities(self):
        return [self.values[i].probability for i in range(self.count)]


class MT(C.Structure):
    _fields_ = [("mt", C.c_uint64 * 312), ("index", C.c_uint32)]


class Tensor(C.Structure):
    _fields_ = [("dtype", C.c_int), ("data", C.c_void_p), ("k", C.c_uint64), ("n", C.c_uint64)]


class Layer(C.Structure):
    _fields_ = [(name, Tensor) for name in
                ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")] + \
               [(name, C.c_void_p) for name in
                ("attn_norm", "post_attention_norm", "ffn_norm", "post_ffw_norm", "q_norm", "k_norm")]


class ModelConfig(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in
                ("hidden", "ffn", "heads", "kv_heads", "head_dim", "layers", "vocab",
                 "sliding_window", "sliding_pattern")] + \
               [(n, C.c_float) for n in
                ("rope_base_global", "rope_scale_global", "rope_base_local", "rope_scale_local",
                 "rms_eps", "attn_softcap", "final_softcap")] + \
               [("uses_qk_norm", C.c_int), ("kv_f16", C.c_int), ("attention_scale", C.c_float)]


class Oracle:
    def __init__(self, path: str | None = None):
        path = path or os.path.join(HERE, "liboracle.so")
        if not os.path.exists(path):
            build(reference=False)
        L = self.lib = C.CDLL(path)
        L.gfo_f16_to_f32.restype = C.c_float
        L.gfo_f16_to_f32.argtypes = [C.c_uint16]
        L.gfo_f32_to_f16_half_up.restype = C.c_uint16
        L.gfo_f32_to_f16_half_up.argtypes = [C.c_float]
        L.gfo_f32_to_f16_rne.restype = C.c_uint16
        L.gfo_f32_to_f16_rne.argtypes = [C.c_float]
        L.gfo_dequantize.argtypes = [C.c_int, _u8p, C.c_uint64, _f32p]
        L.gfo_matmul_quantized.argtypes = [C.c_int, _f32p, _u8p, C.c_uint32, C.c_uint64, C.c_uint64, _f32p]
        L.gfo_matmul_quantized_columns.argtypes = [C.c_int, _f32p, _u8p, C.c_uint32, C.c_uint64,
                                                   C.c_uint64, C.c_uint64, C.c_uint64, _f32p]
        L.gfo_matmul_quantized_f64.argtypes = [C.c_int, _f32p, _u8p, C.c_uint32, C.c_uint64, C.c_uint64, _f64p, _f64p]
        L.gfo_rms_norm.argtypes = [_f32p, _f32p, C.c_uint32, C.c_uint32, C.c_float, _f32p]
        L.gfo_gelu_tanh_multiply.argtypes = [_f32p, _f32p, C.c_uint64, _f32p]
        L.gfo_softcap.argtypes = [_f32p, C.c_uint64, C.c_float, _f32p]
        L.gfo_softmax.argtypes = [_f32p, C.c_uint32, C.c_uint32, _f32p]
        L.gfo_rope_neox.argtypes = [_f32p, _u32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, C.c_float, _f32p]
        L.gfo_attention_row.argtypes = [_f32p, _f32p, _f32p, C.c_uint32, C.c_uint32, C.c_uint32,
                                        C.c_uint32, C.c_float, C.c_float, _f32p]
        L.gfo_select_candidates.restype = C.c_uint32
        L.gfo_select_candidates.argtypes = [_f32p, C.c_uint32, C.c_float, C.c_uint32, _u32p, C.c_uint32, C.c_void_p]
        L.gfo_prepare_distribution.argtypes = [C.c_void_p, C.c_uint32, C.POINTER(SamplerOptions), C.c_uint32,
                                               _u32p, C.c_uint32, C.POINTER(Distribution)]
        L.gfo_prepare_speculative.argtypes = [C.c_uint32, C.c_uint64, _u64p, C.POINTER(Distribution),
                                              C.POINTER(C.c_double), C.POINTER(Distribution)]
        L.gfo_sample_speculative.argtypes = [C.c_uint32, C.c_double, C.POINTER(Distribution), C.c_double,
                                             C.c_double, C.POINTER(C.c_uint32), C.POINTER(C.c_int)]
        L.gfo_select_prepared.restype = C.c_uint32
        L.gfo_select_prepared.argtypes = [C.POINTER(Distribution), C.c_double]
        L.gfo_mt_seed.argtypes = [C.POINTER(MT), C.c_uint64]
        L.gfo_mt_next.restype = C.c_uint64
        L.gfo_mt_next.argtypes = [C.POINTER(MT)]
        L.gfo_uniform_double.restype = C.c_double
        L.gfo_uniform_double.argtypes = [C.POINTER(MT), C.c_double, C.c_double]
        L.gfo_make_proposal_rng.argtypes = [C.POINTER(MT), C.POINTER(MT)]
        L.gfo_next_proposal_word.restype = C.c_uint32
        L.gfo_next_proposal_word.argtypes = [C.POINTER(MT)]
        L.gfo_draft_law_compact.restype = C.c_uint32
        L.gfo_draft_law_compact.argtypes = [_f32p, C.c_uint32, C.c_uint32, C.c_float, C.c_float, _u32p, _u64p]
        L.gfo_quantize_f16_q8_0.argtypes = [C.c_void_p, C.c_uint64, _u8p]
        L.gfo_requantize_q6k_q4k.argtypes = [_u8p, C.c_uint64, _u8p]
        L.gfo_draft_law_full.restype = C.c_uint32
        L.gfo_draft_law_full.argtypes = [_f32p, C.c_uint32, C.c_float, C.c_uint32, C.c_float, C.c_float, _u64p]
        L.gfo_draft_process_logits.argtypes = [_f32p, C.c_uint32, C.c_float, C.c_float, _u32p, C.c_uint32, _f32p]
        L.gfo_model_create.restype = C.c_void_p
        L.gfo_model_create.argtypes = [C.POINTER(ModelConfig), C.POINTER(Tensor), C.c_void_p,
                                       C.POINTER(Tensor), C.POINTER(Layer), C.c_uint32]
        L.gfo_model_destroy.argtypes = [C.c_void_p]
        L.gfo_model_reset.argtypes = [C.c_void_p]
        L.gfo_model_truncate.argtypes = [C.c_void_p, C.c_uint32]
        L.gfo_model_set_kv.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, _f32p, _f32p]
        L.gfo_model_set_kv.restype = None
        L.gfo_model_seek.argtypes = [C.c_void_p, C.c_uint32]
        L.gfo_model_seek.restype = None
        L.gfo_model_position.restype = C.c_uint32
        L.gfo_model_position.argtypes = [C.c_void_p]
        L.gfo_model_append.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]
        L.gfo_model_key.restype = C.POINTER(C.c_float)
        L.gfo_model_key.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32]
        L.gfo_model_value.restype = C.POINTER(C.c_float)
        L.gfo_model_value.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32]
        L.gfo_set_threads.argtypes = [C.c_int]

    # ---- scalar helpers
    def f16_to_f32(self, bits):
        return self.lib.gfo_f16_to_f32(int(bits))

    def dequantize(self, dtype, blocks: np.ndarray) -> np.ndarray:
        blocks = np.ascontiguousarray(blocks, np.uint8).reshape(-1)
        count = blocks.size // BLOCK_BYTES[dtype]
        out = np.empty(count * BLOCK_ELEMENTS[dtype], np.float32)
        self.lib.gfo_dequantize(dtype, blocks, count, out)
        return out

    def matmul(self, dtype, x: np.ndarray, weight: np.ndarray, k: int, n: int) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32).reshape(-1, k)
        out = np.empty((x.shape[0], n), np.float32)
        self.lib.gfo_matmul_quantized(dtype, x, np.ascontiguousarray(weight, np.uint8).reshape(-1), x.shape[0], k, n, out)
        return out

    def matmul_columns(self, dtype, x, weight, k, n, begin, end, out):
        self.lib.gfo_matmul_quantized_columns(dtype, x, weight, x.shape[0], k, n, begin, end, out)

    def matmul_f64(self, dtype, x, weight, k, n):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, k)
        out = np.empty((x.shape[0], n), np.float64)
        abs_out = np.empty((x.shape[0], n), np.float64)
        self.lib.gfo_matmul_quantized_f64(dtype, x, np.ascontiguousarray(weight, np.uint8).reshape(-1),
                                          x.shape[0], k, n, out, abs_out)
        return out, abs_out

    def rms_norm(self, x, gamma, eps=1e-6):
        x = np.ascontiguousarray(x, np.float32)
        rows, hidden = x.reshape(-1, x.shape[-1]).shape
        out = np.empty_like(x)
        self.lib.gfo_rms_norm(x, np.ascontiguousarray(gamma, np.float32), rows, hidden, eps, out)
        return out

    def gelu_tanh_multiply(self, gate, up):
        gate = np.ascontiguousarray(gate, np.float32)
        out = np.empty_like(gate)
        self.lib.gfo_gelu_tanh_multiply(gate, np.ascontiguousarray(up, np.float32), gate.size, out)
        return out

    def softcap(self, x, cap):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty_like(x)
        self.lib.gfo_softcap(x, x.size, cap, out)
        return out

    def softmax(self, x):
        x = np.ascontiguousarray(x, np.float32)
        rows, cols = x.reshape(-1, x.shape[-1]).shape
        out = np.empty_like(x)
        self.lib.gfo_softmax(x, rows, cols, out)
        return out

    def rope_neox(self, x, positions, heads, head_dim, base, scale=1.0):
        x = np.ascontiguousarray(x, np.float32)
        positions = np.ascontiguousarray(positions, np.uint32)
        out = np.empty_like(x)
        self.lib.gfo_rope_neox(x, positions, positions.size, heads, head_dim, base, scale, out)
        return out

    def attention_row(self, q, keys, values, heads, kv_heads, head_dim, scale, softcap=0.0):
        q = np.ascontiguousarray(q, np.float32)
        keys = np.ascontiguousarray(keys, np.float32)
        values = np.ascontiguousarray(values, np.float32)
        count = keys.size // (kv_heads * head_dim)
        out = np.empty(heads * head_dim, np.float32)
        self.lib.gfo_attention_row(q, keys, values, count, heads, kv_heads, head_dim, scale, softcap, out)
        return out

    def select_candidates(self, logits, softcap, retain, history=()):
        logits = np.ascontiguousarray(logits, np.float32)
        history = np.ascontiguousarray(np.array(history, np.uint32))
        out = np.zeros(retain + history.size, TOKEN_LOGIT)
        n = self.lib.gfo_select_candidates(logits, logits.size, softcap, retain,
                                           history if history.size else np.zeros(1, np.uint32),
                                           history.size, out.ctypes.data)
        return out[:n]

    def prepare_distribution(self, candidates: np.ndarray, options: SamplerOptions, history=()):
        """`history` is the deduplicated request history (only used when the penalty is not 1)."""
        candidates = np.ascontiguousarray(candidates, TOKEN_LOGIT)
        history = np.ascontiguousarray(np.array(history, np.uint32))
        out = Distribution()
        top_k = 1 if options.temperature == 0.0 else options.top_k
        rc = self.lib.gfo_prepare_distribution(candidates.ctypes.data, candidates.size, C.byref(options), top_k,
                                               history if history.size else np.zeros(1, np.uint32),
                                               history.size, C.byref(out))
        return rc, out

    def prepare_speculative(self, proposal, proposal_mass, q_mass, target: Distribution):
        q_mass = np.ascontiguousarray(q_mass, np.uint64)
        acceptance = C.c_double()
        residual = Distribution()
        rc = self.lib.gfo_prepare_speculative(proposal, proposal_mass, q_mass, C.byref(target),
                                              C.byref(acceptance), C.byref(residual))
        return rc, acceptance.value, residual

    def sample_speculative(self, proposal, acceptance, residual, accept_draw, residual_draw):
        token, accepted = C.c_uint32(), C.c_int()
        rc = self.lib.gfo_sample_speculative(proposal, acceptance, C.byref(residual), accept_draw,
                                             residual_draw, C.byref(token), C.byref(accepted))
        return rc, token.value, bool(accepted.value)

    def rng(self, seed) -> MT:
        state = MT()
        self.lib.gfo_mt_seed(C.byref(state), seed)
        return state

    def proposal_rng(self, target: MT) -> MT:
        out = MT()
        self.lib.gfo_make_proposal_rng(C.byref(target), C.byref(out))
        return out

    def next_proposal_word(self, rng: MT) -> int:
        return self.lib.gfo_next_proposal_word(C.byref(rng))

    def uniform(self, rng: MT, a=0.0, b=1.0) -> float:
        return self.lib.gfo_uniform_double(C.byref(rng), a, b)

    def draft_process_logits(self, logits, temperature, repetition_penalty=1.0, history=()):
        logits = np.ascontiguousarray(logits, np.float32)
        history = np.ascontiguousarray(np.array(history, np.uint32))
        out = np.empty_like(logits)
        self.lib.gfo_draft_process_logits(logits, logits.size, temperature, repetition_penalty,
                                          history if history.size else np.zeros(1, np.uint32), history.size, out)
        return out

    def draft_law_compact(self, scores, top_k, top_p, min_p):
        scores = np.ascontiguousarray(scores, np.float32)
        ids = np.zeros(256, np.uint32)
        cdf = np.zeros(257, np.uint64)
        n = self.lib.gfo_draft_law_compact(scores, scores.size, top_k, top_p, min_p, ids, cdf)
        return ids[:n], cdf[:n + 1]

    def quantize_f16_q8_0(self, f16_bits):
        """Binary16 values (as uint16 bits, a multiple of 32) -> Q8_0 blocks."""
        f16_bits = np.ascontiguousarray(f16_bits, np.uint16)
        out = np.zeros(f16_bits.size // 32 * 34, np.uint8)
        rc = self.lib.gfo_quantize_f16_q8_0(f16_bits.ctypes.data, f16_bits.size // 32, out)
        return rc, out

    def requantize_q6k_q4k(self, q6k):
        """Q6_K blocks (210 B each) -> Q4_K blocks (144 B each), block for block."""
        q6k = np.ascontiguousarray(q6k, np.uint8).reshape(-1)
        out = np.zeros(q6k.size // 210 * 144, np.uint8)
        rc = self.lib.gfo_requantize_q6k_q4k(q6k, q6k.size // 210, out)
        return rc, out

    def draft_law_full(self, scores, temperature, top_k, top_p, min_p):
        """Full-vocabulary law: (status, cdf[vocab + 1])."""
        scores = np.ascontiguousarray(scores, np.float32)
        cdf = np.zeros(scores.size + 1, np.uint64)
        status = self.lib.gfo_draft_law_full(scores, scores.size, temperature, top_k, top_p, min_p, cdf)
        return status, cdf

    def set_threads(self, n):
        self.lib.gfo_set_threads(n)


class OracleModel:
    """Whole-model forward on the oracle.  `weights` is the dict produced by
    guffin_b200.synthetic.make_model_weights (name -> (dtype, k, n, bytes) or f32 vector)."""

    def __init__(self, oracle: Oracle, config: dict, weights: dict, context: int):
        self.oracle, self.config, self._keep = oracle, config, []
        cfg = ModelConfig()
        for name, _ in ModelConfig._fields_:
            setattr(cfg, name, config[name])
        self.cfg = cfg

        def tensor(name):
            dtype, k, n, data = weights[name]
            data = np.ascontiguousarray(data, np.uint8)
            self._keep.append(data)
            return Tensor(dtype, data.ctypes.data, k, n)

        def vec(name):
            if name not in weights:
                return None
            data = np.ascontiguousarray(weights[name], np.float32)
            self._keep.append(data)
            return data.ctypes.data

        layers = (Layer * config["layers"])()
        for l in range(config["layers"]):
            for name in ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down"):
                setattr(layers[l], name, tensor(f"blk.{l}.{name}.weight"))
            layers[l].attn_norm = vec(f"blk.{l}.attn_norm.weight")
            layers[l].post_attention_norm = vec(f"blk.{l}.post_attention_norm.weight")
            layers[l].ffn_norm = vec(f"blk.{l}.ffn_norm.weight")
            layers[l].post_ffw_norm = vec(f"blk.{l}.post_ffw_norm.weight")
            layers[l].q_norm = vec(f"blk.{l}.attn_q_norm.weight")
            layers[l].k_norm = vec(f"blk.{l}.attn_k_norm.weight")
        embd = tensor("token_embd.weight")
        head = tensor("output.weight") if "output.weight" in weights else None
        self.handle = oracle.lib.gfo_model_create(C.byref(cfg), C.byref(embd), vec("output_norm.weight"),
                                                  C.byref(head) if head is not None else None, layers, context)

    def append(self, token, want_logits=True):
        logits = np.empty(self.config["vocab"], np.float32) if want_logits else None
        self.oracle.lib.gfo_model_append(self.handle, int(token),
                                         logits.ctypes.data if want_logits else None, None)
        return logits

    def truncate(self, position):
        self.oracle.lib.gfo_model_truncate(self.handle, position)

    def reset(self):
        self.oracle.lib.gfo_model_reset(self.handle)

    def set_kv(self, layer, first, keys, values):
        """Overwrites cached rows [first, first + len(keys)) of one layer (f32 [rows, kv_width])."""
        keys, values = np.ascontiguousarray(keys, np.float32), np.ascontiguousarray(values, np.float32)
        self.oracle.lib.gfo_model_set_kv(self.handle, layer, first, keys.shape[0], keys, values)

    def seek(self, position):
        self.oracle.lib.gfo_model_seek(self.handle, position)

    @property
    def position(self):
        return self.oracle.lib.gfo_model_position(self.handle)

    def key(self, layer, position):
        w = self.config["kv_heads"] * self.config["head_dim"]
        return np.ctypeslib.as_array(self.oracle.lib.gfo_model_key(self.handle, layer, position), (w,)).copy()

    def value(self, layer, position):
        w = self.config["kv_heads"] * self.config["head_dim"]
        return np.ctypeslib.as_array(self.oracle.lib.gfo_model_value(self.handle, layer, position), (w,)).copy()

    def __del__(self):
        try:
            self.oracle.lib.gfo_model_destroy(self.handle)
        except Exception:
            pass


class Reference:
    """The reference engine's own CPU code (oracle/_ref).  `available()` is False until built."""

    PATH = os.path.join(HERE, "_ref", "libguffin_ref.so")

    @classmethod
    def available(cls) -> bool:
        return os.path.exists(cls.PATH)

    def __init__(self):
        L = self.lib = C.CDLL(self.PATH)
        L.ref_f16_to_f32.restype = C.c_float
        L.ref_f16_to_f32.argtypes = [C.c_uint16]
        L.ref_f32_to_f16.restype = C.c_uint16
        L.ref_f32_to_f16.argtypes = [C.c_float]
        L.ref_dequantize.argtypes = [C.c_int, _u8p, C.c_uint64, _f32p]
        L.ref_matmul_quantized.argtypes = [C.c_int, _f32p, _u8p, C.c_uint32, C.c_uint64, C.c_uint64, _f32p]
        L.ref_rms_norm.argtypes = [_f32p, _f32p, C.c_uint32, C.c_uint32, C.c_float, _f32p]
        L.ref_gelu_tanh_multiply.argtypes = [_f32p, _f32p, C.c_uint64, _f32p]
        L.ref_softcap.argtypes = [_f32p, C.c_uint64, C.c_float, _f32p]
        L.ref_softmax.argtypes = [_f32p, C.c_uint32, C.c_uint32, _f32p]
        L.ref_rope_neox.argtypes = [_f32p, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, _f32p]
        L.ref_attention_row.argtypes = [_f32p, _f32p, _f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                        C.c_float, C.c_float, _f32p]
        L.ref_prepare_distribution.argtypes = [C.c_void_p, C.c_uint32, C.c_float, C.c_uint32, C.c_float, C.c_float,
                                               C.c_float, _u32p, C.c_uint32, C.c_void_p, C.POINTER(C.c_double)]
        L.ref_proposal_words.argtypes = [C.c_uint64, C.c_uint32, _u32p]
        L.ref_uniform_draws.argtypes = [C.c_uint64, C.c_double, C.c_double, C.c_uint32, _f64p]
        L.ref_sample_speculative.argtypes = [C.c_uint64, C.c_float, C.c_uint32, C.c_float, C.c_float, C.c_float,
                                             _u32p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint64,
                                             C.c_uint64, _u64p, C.POINTER(C.c_uint32), C.POINTER(C.c_int),
                                             C.POINTER(C.c_uint64)]
        L.ref_sample.argtypes = [C.c_uint64, C.c_float, C.c_uint32, C.c_float, C.c_float, C.c_float, _u32p,
                                 C.c_uint32, C.c_void_p, C.c_uint32, C.POINTER(C.c_uint32)]
        L.ref_columns8_round_trip.argtypes = [C.c_int, _u8p, C.c_uint64, C.c_uint64]
        L.ref_quantize_f16_q8_0.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, _u8p]
        L.ref_requantize_q6k_q4k.argtypes = [_u8p, C.c_uint64, C.c_uint64, _u8p]

    def dequantize(self, dtype, blocks):
        blocks = np.ascontiguousarray(blocks, np.uint8).reshape(-1)
        count = blocks.size // BLOCK_BYTES[dtype]
        out = np.empty(count * BLOCK_ELEMENTS[dtype], np.float32)
        assert self.lib.ref_dequantize(dtype, blocks, count, out) == 0
        return out

    def matmul(self, dtype, x, weight, k, n):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, k)
        out = np.empty((x.shape[0], n), np.float32)
        assert self.lib.ref_matmul_quantized(dtype, x, np.ascontiguousarray(weight, np.uint8).reshape(-1),
                                             x.shape[0], k, n, out) == 0
        return out

    def rms_norm(self, x, gamma, eps=1e-6):
        x = np.ascontiguousarray(x, np.float32)
        rows, hidden = x.reshape(-1, x.shape[-1]).shape
        out = np.empty_like(x)
        assert self.lib.ref_rms_norm(x, np.ascontiguousarray(gamma, np.float32), rows, hidden, eps, out) == 0
        return out

    def gelu_tanh_multiply(self, gate, up):
        gate = np.ascontiguousarray(gate, np.float32)
        out = np.empty_like(gate)
        assert self.lib.ref_gelu_tanh_multiply(gate, np.ascontiguousarray(up, np.float32), gate.size, out) == 0
        return out

    def softcap(self, x, cap):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty_like(x)
        assert self.lib.ref_softcap(x, x.size, cap, out) == 0
        return out

    def softmax(self, x):
        x = np.ascontiguousarray(x, np.float32)
        rows, cols = x.reshape(-1, x.shape[-1]).shape
        out = np.empty_like(x)
        assert self.lib.ref_softmax(x, rows, cols, out) == 0
        return out

    def rope_neox(self, x, position_start, rows, heads, head_dim, base):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty_like(x)
        assert self.lib.ref_rope_neox(x, position_start, rows, heads, head_dim, base, out) == 0
        return out

    def attention_row(self, q, keys, values, heads, kv_heads, head_dim, scale, softcap):
        q = np.ascontiguousarray(q, np.float32)
        keys = np.ascontiguousarray(keys, np.float32)
        values = np.ascontiguousarray(values, np.float32)
        count = keys.size // (kv_heads * head_dim)
        out = np.empty(heads * head_dim, np.float32)
        assert self.lib.ref_attention_row(q, keys, values, count, heads, kv_heads, head_dim, scale, softcap, out) == 0
        return out

    def prepare_distribution(self, candidates, options: SamplerOptions, history=()):
        candidates = np.ascontiguousarray(candidates, TOKEN_LOGIT)
        history = np.ascontiguousarray(np.array(history, np.uint32))
        out = np.zeros(256, PROB)
        total = C.c_double()
        n = self.lib.ref_prepare_distribution(candidates.ctypes.data, candidates.size, options.temperature,
                                              options.top_k, options.top_p, options.min_p,
                                              options.repetition_penalty,
                                              history if history.size else np.zeros(1, np.uint32), history.size,
                                              out.ctypes.data, C.byref(total))
        return n, out[:max(n, 0)], total.value

    def proposal_words(self, seed, count):
        words = np.zeros(count, np.uint32)
        assert self.lib.ref_proposal_words(seed, count, words) == 0
        return words

    def uniform_draws(self, seed, a, b, count):
        out = np.zeros(count, np.float64)
        self.lib.ref_uniform_draws(seed, a, b, count, out)
        return out

    def sample_speculative(self, seed, options: SamplerOptions, history, candidates, proposal, proposal_mass,
                           cdf_begin, q_mass):
        candidates = np.ascontiguousarray(candidates, TOKEN_LOGIT)
        history = np.ascontiguousarray(np.array(history, np.uint32))
        q_mass = np.ascontiguousarray(q_mass, np.uint64)
        token, accepted, draws = C.c_uint32(), C.c_int(), C.c_uint64()
        rc = self.lib.ref_sample_speculative(seed, options.temperature, options.top_k, options.top_p, options.min_p,
                                             options.repetition_penalty,
                                             history if history.size else np.zeros(1, np.uint32), history.size,
                                             candidates.ctypes.data, candidates.size, proposal, proposal_mass,
                                             cdf_begin, q_mass, C.byref(token), C.byref(accepted), C.byref(draws))
        return rc, token.value, bool(accepted.value), draws.value

    def sample(self, seed, options: SamplerOptions, history, candidates):
        candidates = np.ascontiguousarray(candidates, TOKEN_LOGIT)
        history = np.ascontiguousarray(np.array(history, np.uint32))
        token = C.c_uint32()
        rc = self.lib.ref_sample(seed, options.temperature, options.top_k, options.top_p, options.min_p,
                                 options.repetition_penalty,
                                 history if history.size else np.zeros(1, np.uint32), history.size,
                                 candidates.ctypes.data, candidates.size, C.byref(token))
        return rc, token.value

    def quantize_f16_q8_0(self, f16_bits, k, n):
        f16_bits = np.ascontiguousarray(f16_bits, np.uint16)
        out = np.zeros(k * n // 32 * 34, np.uint8)
        rc = self.lib.ref_quantize_f16_q8_0(f16_bits.ctypes.data, k, n, out)
        return rc, out

    def requantize_q6k_q4k(self, q6k, k, n):
        q6k = np.ascontiguousarray(q6k, np.uint8).reshape(-1)
        out = np.zeros(k * n // 256 * 144, np.uint8)
        rc = self.lib.ref_requantize_q6k_q4k(q6k, k, n, out)
        return rc, out

    def columns8_round_trip(self, dtype, weight, k, n):
        return self.lib.ref_columns8_round_trip(dtype, np.ascontiguousarray(weight, np.uint8).reshape(-1), k, n)
