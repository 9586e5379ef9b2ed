"""Seeded synthetic GGUF-format weights, activations and model geometries.

Stands in for the real Gemma checkpoints (none ship with this repository): tensors take the
shapes, block formats and value distributions of the workloads the benchmarks name, all from a
numpy PCG64 seed so the CPU oracle and the CUDA path see identical bytes.

Block formats follow the reference's definitions (src/tensor/quantization.cpp:430-593):
Q8_0 = f16 d + 32 int8; Q4_K = f16 d, f16 dmin, 12 packed 6-bit scale/min bytes, 128 nibble
bytes; Q6_K = 128 low-nibble bytes, 64 high-bit bytes, 16 int8 scales, f16 d.
"""
from __future__ import annotations

import math

import numpy as np

Q8_0, Q4_K, Q6_K = 8, 12, 14
BLOCK_ELEMENTS = {Q8_0: 32, Q4_K: 256, Q6_K: 256}
BLOCK_BYTES = {Q8_0: 34, Q4_K: 144, Q6_K: 210}


def _positive_f16(rng: np.random.Generator, count: int, sigma: float) -> np.ndarray:
    values = np.abs(rng.normal(0.0, sigma, count)).astype(np.float16)
    values[values == 0] = max(np.float16(sigma), np.float16(6e-8))
    return values.view(np.uint8).reshape(count, 2)


def q4k_blocks(rng, count: int, sigma: float = 1e-3) -> np.ndarray:
    """d, dmin ~ |N(0, sigma)|; every 6-bit scale/min field uniform in [0, 63] (uniform bytes
    make all sixteen packed fields uniform); nibbles uniform in [0, 15]."""
    blocks = rng.integers(0, 256, (count, 144), dtype=np.uint8)
    blocks[:, 0:2] = _positive_f16(rng, count, sigma)
    blocks[:, 2:4] = _positive_f16(rng, count, sigma)
    return blocks


def q6k_blocks(rng, count: int, sigma: float = 1e-3) -> np.ndarray:
    """6-bit quants uniform; int8 sub-scales uniform in [-64, 63]; d ~ |N(0, sigma)|."""
    blocks = rng.integers(0, 256, (count, 210), dtype=np.uint8)
    blocks[:, 192:208] = rng.integers(-64, 64, (count, 16), dtype=np.int8).view(np.uint8)
    blocks[:, 208:210] = _positive_f16(rng, count, sigma)
    return blocks


def q80_blocks(rng, count: int, sigma: float = 1e-2) -> np.ndarray:
    """f16 scale ~ |N(0, sigma)|; int8 uniform in [-127, 127]."""
    blocks = np.empty((count, 34), np.uint8)
    blocks[:, 0:2] = _positive_f16(rng, count, sigma)
    blocks[:, 2:] = rng.integers(-127, 128, (count, 32), dtype=np.int8).view(np.uint8)
    return blocks


_MAKERS = {Q4_K: q4k_blocks, Q6_K: q6k_blocks, Q8_0: q80_blocks}


def make_weight(rng, dtype: int, k: int, n: int, sigma: float | None = None) -> np.ndarray:
    """Native GGUF payload of a [K, N] projection: column n owns K/block consecutive blocks."""
    assert k % BLOCK_ELEMENTS[dtype] == 0
    count = n * (k // BLOCK_ELEMENTS[dtype])
    blocks = _MAKERS[dtype](rng, count) if sigma is None else _MAKERS[dtype](rng, count, sigma)
    return blocks.reshape(-1)


def weight_bytes(dtype: int, k: int, n: int) -> int:
    return n * (k // BLOCK_ELEMENTS[dtype]) * BLOCK_BYTES[dtype]


# ---------------------------------------------------------------------------- geometries

def _config(hidden, ffn, heads, kv_heads, head_dim, layers, vocab, window, pattern,
            base_g, scale_g, base_l, scale_l, attn_cap, final_cap, qk_norm, kv_f16):
    return dict(hidden=hidden, ffn=ffn, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                layers=layers, vocab=vocab, sliding_window=window, sliding_pattern=pattern,
                rope_base_global=base_g, rope_scale_global=scale_g, rope_base_local=base_l,
                rope_scale_local=scale_l, rms_eps=1e-6, attn_softcap=attn_cap,
                final_softcap=final_cap, uses_qk_norm=qk_norm, kv_f16=kv_f16,
                attention_scale=1.0 / math.sqrt(head_dim))


def model_config(name: str) -> dict:
    """Geometries of the reference's three models (scripts/gemma3_target_reference.py:28-29,
    scripts/gemma3_reference_golden.py:41-42, tests/reference/gemma2_reference.cpp) and small
    same-shaped stand-ins for tests."""
    if name == "gemma3-12b":      # target: F16 KV, global RoPE 1e6 scaled by 1/8, local 1e4
        return _config(3840, 15360, 16, 8, 256, 48, 262144, 1024, 6, 1e6, 0.125, 1e4, 1.0, 0.0, 0.0, 1, 1)
    if name == "gemma3-270m":     # drafter: F32 KV, unscaled global RoPE
        return _config(640, 2048, 4, 1, 256, 18, 262144, 512, 6, 1e6, 1.0, 1e4, 1.0, 0.0, 0.0, 1, 0)
    if name == "gemma2-9b":
        return _config(3584, 14336, 16, 8, 256, 42, 256000, 4096, 2, 1e4, 1.0, 1e4, 1.0, 50.0, 30.0, 0, 1)
    if name == "tiny-target":     # 12B block shape shrunk: 7 layers cover a local and a global layer
        return _config(512, 1024, 4, 2, 256, 7, 2048, 16, 6, 1e6, 0.125, 1e4, 1.0, 0.0, 0.0, 1, 1)
    if name == "tiny-draft":
        return _config(256, 512, 4, 1, 256, 6, 2048, 8, 6, 1e6, 1.0, 1e4, 1.0, 0.0, 0.0, 1, 0)
    if name == "tiny-gemma2":
        return _config(512, 1024, 4, 2, 256, 4, 2048, 16, 2, 1e4, 1.0, 1e4, 1.0, 50.0, 30.0, 0, 1)
    raise KeyError(name)


def use_more_bits(layer: int, layers: int) -> bool:
    """Which layers a Q4_K_M file stores attn_v / ffn_down in Q6_K: the published llama.cpp
    quantiser rule (first and last eighth, and every third layer between), which yields 24 of
    48 layers for the 12B model as the reference's byte accounting reports."""
    return layer < layers // 8 or layer >= 7 * layers // 8 or (layer - layers // 8) % 3 == 2


def tensor_types(name: str, config: dict) -> dict:
    """Per-tensor GGUF dtype for each model family."""
    types = {}
    L = config["layers"]
    for l in range(L):
        for t in ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down"):
            if name.endswith("270m") or name == "tiny-draft":
                dtype = Q8_0
            elif name.startswith("gemma2") or name == "tiny-gemma2":
                dtype = Q4_K
            else:
                dtype = Q6_K if t in ("attn_v", "ffn_down") and use_more_bits(l, L) else Q4_K
            types[f"blk.{l}.{t}.weight"] = dtype
    if name.endswith("270m") or name == "tiny-draft":
        types["token_embd.weight"] = Q8_0
    elif name.startswith("gemma2") or name == "tiny-gemma2":
        types["token_embd.weight"] = Q6_K     # embedding rows
        types["output.weight"] = Q8_0         # separate Q8_0 head (gemma2_metal_plan.cpp:495-512)
    else:
        types["token_embd.weight"] = Q6_K
    return types


def matrix_shapes(config: dict) -> dict:
    H, F, hd = config["hidden"], config["ffn"], config["head_dim"]
    q, kv = config["heads"] * hd, config["kv_heads"] * hd
    return {"attn_q": (H, q), "attn_k": (H, kv), "attn_v": (H, kv), "attn_output": (q, H),
            "ffn_gate": (H, F), "ffn_up": (H, F), "ffn_down": (F, H)}


def iter_model_weights(name: str, seed: int, config: dict | None = None):
    """Yields (GGUF tensor name, value) one tensor at a time: value is (dtype, K, N, uint8 payload)
    for matrices and a float32 array for norm vectors.  Lets a loader upload a 12B model without
    holding all of it in host memory."""
    config = config or model_config(name)
    rng = np.random.default_rng(seed)
    types = tensor_types(name, config)
    shapes = matrix_shapes(config)
    H, V = config["hidden"], config["vocab"]

    def gamma(n):
        return (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)

    # Embedding / head blocks are scaled so that an embedded token has unit RMS after the
    # sqrt(hidden) factor, as trained checkpoints roughly do; otherwise a random tied model just
    # echoes its input token and every proposal is trivially accepted.
    def table_sigma(dtype):
        code_rms = {Q6_K: 685.0, Q8_0: 73.3, Q4_K: 300.0}[dtype]
        return 1.0 / (code_rms * math.sqrt(H))

    embd_type = types["token_embd.weight"]
    yield "token_embd.weight", (embd_type, H, V, make_weight(rng, embd_type, H, V, table_sigma(embd_type)))
    if "output.weight" in types:
        head_type = types["output.weight"]
        yield "output.weight", (head_type, H, V, make_weight(rng, head_type, H, V, table_sigma(head_type)))
    yield "output_norm.weight", gamma(H)
    for l in range(config["layers"]):
        for t, (k, n) in shapes.items():
            key = f"blk.{l}.{t}.weight"
            yield key, (types[key], k, n, make_weight(rng, types[key], k, n))
        for t in ("attn_norm", "post_attention_norm", "ffn_norm", "post_ffw_norm"):
            yield f"blk.{l}.{t}.weight", gamma(H)
        if config["uses_qk_norm"]:
            yield f"blk.{l}.attn_q_norm.weight", gamma(config["head_dim"])
            yield f"blk.{l}.attn_k_norm.weight", gamma(config["head_dim"])


def make_model_weights(name: str, seed: int, config: dict | None = None) -> dict:
    """All tensors of iter_model_weights in one dict."""
    return dict(iter_model_weights(name, seed, config))


def model_weight_bytes(name: str, config: dict | None = None) -> int:
    """Native GGUF bytes one decode pass streams: every matrix once, the tied head included."""
    config = config or model_config(name)
    types = tensor_types(name, config)
    shapes = matrix_shapes(config)
    total = 0
    for l in range(config["layers"]):
        for t, (k, n) in shapes.items():
            total += weight_bytes(types[f"blk.{l}.{t}.weight"], k, n)
        total += 4 * (4 * config["hidden"] + (2 * config["head_dim"] if config["uses_qk_norm"] else 0))
    head = types.get("output.weight", types["token_embd.weight"])
    total += weight_bytes(head, config["hidden"], config["vocab"]) + 4 * config["hidden"]
    return total
