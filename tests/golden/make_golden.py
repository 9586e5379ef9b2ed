#!/usr/bin/env python3
"""Generates the committed golden fixtures from the REFERENCE's own code.

Run where the reference tree is available (its location comes from the GF_REFERENCE environment
variable) and
oracle/_ref has been built (`make -C oracle ref`):

    python tests/golden/make_golden.py

Outputs (small, committed):
  ref_ops.npz      seeded inputs and the outputs of the reference's C++ CPU functions
                   (dequantised blocks, quantised matmul, RMSNorm, GeGLU, softcap, softmax,
                   NEOX RoPE, grouped attention), via oracle/_ref.
  ref_requant.npz  the reference's load-time weight transforms (F16 -> Q8_0, Q6_K -> Q4_K) on seeded blocks,
                   via oracle/_ref (`--only requant` writes just this file).
  ref_sampling.npz prepared target distributions, speculative accept/reject decisions,
                   proposal words and uniform draws from the reference's sampling.cpp.
  py_target.npz    logits / hidden / K / V of scripts/gemma3_target_reference.py::reference on a
                   synthetic tiny-geometry GGUF (its module constants re-pointed at that geometry).
  py_draft.npz     logits / K / V of scripts/gemma3_reference_golden.py::reference likewise.
The inputs are regenerated from seeds by the tests; only outputs are stored.
"""
from __future__ import annotations

import contextlib
import io
import os
import struct
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
REFERENCE = Path(os.environ.get("GF_REFERENCE") or Path(__file__).resolve().parents[3] / "reference")

from guffin_b200 import synthetic as syn  # noqa: E402
from oracle.pyoracle import Reference, SamplerOptions, TOKEN_LOGIT  # noqa: E402


# ---------------------------------------------------------------- seeded inputs shared with tests

def ops_inputs():
    rng = np.random.default_rng(20240611)
    data = {}
    for name, dtype in (("q4k", syn.Q4_K), ("q6k", syn.Q6_K), ("q80", syn.Q8_0)):
        k = 512 if dtype != syn.Q8_0 else 256
        n = 12
        data[f"{name}_w"] = syn.make_weight(rng, dtype, k, n, sigma=0.05)
        data[f"{name}_x"] = rng.standard_normal((2, k)).astype(np.float32)
    data["norm_x"] = rng.standard_normal((3, 640)).astype(np.float32) * 3.0
    data["norm_g"] = (1.0 + 0.1 * rng.standard_normal(640)).astype(np.float32)
    data["gate"] = (rng.standard_normal(2048) * 2.5).astype(np.float32)
    data["up"] = rng.standard_normal(2048).astype(np.float32)
    data["cap_x"] = (rng.standard_normal(512) * 40.0).astype(np.float32)
    data["soft_x"] = (rng.standard_normal((4, 97)) * 3.0).astype(np.float32)
    data["rope_x"] = rng.standard_normal((3, 4 * 256)).astype(np.float32)
    data["att_q"] = rng.standard_normal(4 * 256).astype(np.float32)
    data["att_k"] = rng.standard_normal((37, 2 * 256)).astype(np.float32)
    data["att_v"] = rng.standard_normal((37, 2 * 256)).astype(np.float32)
    return data


def requant_inputs():
    """Seeded sources of the load-time transforms: binary16 values over several magnitudes (with an
    all-zero and a constant block) and Q6_K blocks (with a block of zero sub-scales and one of zero d)."""
    rng = np.random.default_rng(20240712)
    k8, n8 = 256, 24
    values = (rng.standard_normal(k8 * n8) * rng.choice([1e-4, 1e-2, 1.0, 40.0], k8 * n8)).astype(np.float16)
    values[:32] = 0
    values[32:64] = np.float16(0.3337)
    k6, n6 = 1024, 24
    q6k = np.ascontiguousarray(syn.make_weight(rng, syn.Q6_K, k6, n6, sigma=0.05), np.uint8).reshape(-1, 210).copy()
    q6k[0, 192:208] = 0
    q6k[1, 208:210] = 0
    q6k[2, :192] = 0x55
    return {"f16": values.view(np.uint16).copy(), "f16_k": k8, "f16_n": n8, "q6k": q6k.reshape(-1), "q6k_k": k6, "q6k_n": n6}


def write_requant(ref):
    d = requant_inputs()
    rc8, q8 = ref.quantize_f16_q8_0(d["f16"], d["f16_k"], d["f16_n"])
    rc4, q4 = ref.requantize_q6k_q4k(d["q6k"], d["q6k_k"], d["q6k_n"])
    assert rc8 == 0 and rc4 == 0
    np.savez_compressed(HERE / "ref_requant.npz", q8=q8, q4=q4)


def sampling_cases(count=64):
    """Seeded candidate sets with a consistent draft law for each (built from proposal words)."""
    rng = np.random.default_rng(77)
    cases = []
    for index in range(count):
        n = int(rng.integers(45, 120))
        tokens = rng.choice(262144, n, replace=False).astype(np.uint32)
        logits = (rng.standard_normal(n) * (1.0 + 3.0 * rng.random())).astype(np.float32)
        if index % 7 == 0:
            logits[1] = logits[0]                         # exact tie: token order decides
        candidates = np.zeros(n, TOKEN_LOGIT)
        candidates["token"], candidates["logit"] = tokens, logits
        temperature = [0.7, 1.0, 0.3, 0.0][index % 4]
        penalty = 1.0 if index % 3 else 1.3
        history = rng.choice(tokens, 5, replace=False).astype(np.uint32) if penalty != 1.0 else np.zeros(0, np.uint32)
        cases.append(dict(seed=1000 + index, candidates=candidates, temperature=temperature,
                          top_k=40, top_p=0.95, min_p=0.05, penalty=penalty, history=history,
                          draft_seed=int(rng.integers(1 << 30))))
    return cases


def draft_law_for(case, support_tokens, word):
    """A deterministic 2^32-mass draft law over `support_tokens` plus two outside tokens, chosen
    so that the proposal word falls inside the bin of the token it selects."""
    rng = np.random.default_rng(case["draft_seed"])
    outside = np.array([262143, 262142], np.uint32)
    tokens = np.concatenate([np.array(support_tokens, np.uint32), outside])
    order = np.argsort(tokens)
    tokens = tokens[order]
    raw = rng.random(tokens.size) + 0.05
    raw[rng.random(tokens.size) < 0.2] = 0.0               # some support tokens get q = 0
    raw[-1] += 0.1
    cdf = np.floor(np.cumsum(raw) / raw.sum() * 4294967296.0).astype(np.uint64)
    cdf[-1] = 4294967296
    cdf = np.concatenate([[0], cdf]).astype(np.uint64)
    masses = np.diff(cdf).astype(np.uint64)
    bin_index = int(np.searchsorted(cdf, np.uint64(word), side="right") - 1)
    return tokens, masses, cdf, bin_index


# ---------------------------------------------------------------- minimal GGUF v3 writer

def write_gguf(path, tensors):
    """tensors: list of (name, dims innermost-first, ggml_type, bytes)."""
    def string(s):
        b = s.encode()
        return struct.pack("<Q", len(b)) + b
    header = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), 0)
    infos, offset, payload = b"", 0, []
    for name, dims, ggml_type, data in tensors:
        infos += string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", ggml_type, offset)
        data = bytes(data)
        pad = (-len(data)) % 32
        payload.append(data + b"\0" * pad)
        offset += len(data) + pad
    head = header + infos
    head += b"\0" * ((-len(head)) % 32)
    with open(path, "wb") as f:
        f.write(head)
        for chunk in payload:
            f.write(chunk)


def gguf_tensors(weights):
    out = []
    for name, value in weights.items():
        if isinstance(value, tuple):
            dtype, k, n, data = value
            out.append((name, (k, n), dtype, np.ascontiguousarray(data).tobytes()))
        else:
            out.append((name, (value.size,), 0, np.ascontiguousarray(value, np.float32).tobytes()))
    return out


def run_python_reference(module_name, model_name, seed, tokens, selected, cache_dtype):
    sys.path.insert(0, str(REFERENCE / "scripts"))
    import importlib
    module = importlib.import_module(module_name)
    import gemma3_reference_golden as golden
    config = syn.model_config(model_name)
    weights = syn.make_model_weights(model_name, seed)
    patch = dict(WIDTH=config["hidden"], FFN=config["ffn"], HEAD_DIM=config["head_dim"], HEADS=config["heads"],
                 LAYERS=config["layers"], VOCAB=config["vocab"], WINDOW=config["sliding_window"])
    for target in {module, golden}:
        for key, value in patch.items():
            if hasattr(target, key):
                setattr(target, key, value)
    if hasattr(module, "KV_HEADS"):
        module.KV_HEADS = config["kv_heads"]
    saved = {}
    with tempfile.TemporaryDirectory() as directory:
        path = Path(directory) / "synthetic.gguf"
        write_gguf(path, gguf_tensors(weights))
        from reference_gguf import GGUFFile
        import torch
        torch.set_num_threads(1)
        with GGUFFile(path) as gguf, torch.inference_mode(), contextlib.redirect_stdout(io.StringIO()):
            if module_name == "gemma3_target_reference":
                def save_layer(layer, k, v, hidden):
                    saved[f"k{layer}"] = k.float().numpy().copy()
                    saved[f"v{layer}"] = v.float().numpy().copy()
                logits, hidden = module.reference(gguf, list(tokens), list(selected), save_layer, cache_dtype=cache_dtype)
                saved["hidden"] = hidden.numpy().copy()
            else:
                def save_cache(layer, k, v):
                    saved[f"k{layer}"] = k.float().numpy().copy()
                    saved[f"v{layer}"] = v.float().numpy().copy()
                logits = module.reference(gguf, list(tokens), list(selected), save_cache, cache_dtype=cache_dtype)
    saved["logits"] = logits.numpy().copy()
    saved["tokens"] = np.array(tokens, np.uint32)
    saved["selected"] = np.array(selected, np.uint32)
    return saved


MODEL_CASES = {
    # fixture -> (python module, geometry, weight seed, token seed, length, cache dtype)
    "py_target": ("gemma3_target_reference", "tiny-target", 11, 5, 40, "f16"),
    "py_draft": ("gemma3_reference_golden", "tiny-draft", 12, 6, 24, "f32"),
}


def model_tokens(name):
    _, geometry, _, token_seed, length, _ = MODEL_CASES[name]
    vocab = syn.model_config(geometry)["vocab"]
    return np.random.default_rng(token_seed).integers(0, vocab, length).astype(np.uint32)


def main():
    ref = Reference()
    write_requant(ref)
    if sys.argv[1:] == ["--only", "requant"]:
        print("ref_requant.npz written to", HERE)
        return
    d = ops_inputs()
    out = {}
    for name, dtype in (("q4k", syn.Q4_K), ("q6k", syn.Q6_K), ("q80", syn.Q8_0)):
        k = d[f"{name}_x"].shape[1]
        out[f"{name}_deq"] = ref.dequantize(dtype, d[f"{name}_w"])
        out[f"{name}_y"] = ref.matmul(dtype, d[f"{name}_x"], d[f"{name}_w"], k, 12)
    out["norm_y"] = ref.rms_norm(d["norm_x"], d["norm_g"], 1e-6)
    out["geglu_y"] = ref.gelu_tanh_multiply(d["gate"], d["up"])
    out["cap_y"] = ref.softcap(d["cap_x"], 30.0)
    out["soft_y"] = ref.softmax(d["soft_x"])
    out["rope_y_1e4"] = ref.rope_neox(d["rope_x"], 1021, 3, 4, 256, 1e4)
    out["rope_y_1e6"] = ref.rope_neox(d["rope_x"], 7, 3, 4, 256, 1e6)
    out["att_y"] = ref.attention_row(d["att_q"], d["att_k"], d["att_v"], 4, 2, 256, 0.0625, 50.0)
    np.savez_compressed(HERE / "ref_ops.npz", **out)

    s = {}
    cases = sampling_cases()
    for i, case in enumerate(cases):
        options = SamplerOptions(case["temperature"], case["top_k"], case["top_p"], case["min_p"], case["penalty"])
        n, prepared, total = ref.prepare_distribution(case["candidates"], options, case["history"])
        assert n > 0
        s[f"prep_tokens_{i}"] = prepared["token"].copy()
        s[f"prep_weights_{i}"] = prepared["weight"].copy()
        s[f"prep_total_{i}"] = np.float64(total)
        word = int(ref.proposal_words(case["seed"], 1)[0])
        tokens, masses, cdf, bin_index = draft_law_for(case, prepared["token"], word)
        proposal = int(tokens[bin_index])
        q = np.array([masses[np.searchsorted(tokens, t)] for t in prepared["token"]], np.uint64)
        rc, token, accepted, draws = ref.sample_speculative(case["seed"], options, case["history"], case["candidates"],
                                                            proposal, int(masses[bin_index]), int(cdf[bin_index]), q)
        s[f"spec_{i}"] = np.array([rc, token, int(accepted), draws, proposal, word], np.int64)
        rc2, sampled = ref.sample(case["seed"], options, case["history"], case["candidates"])
        s[f"sample_{i}"] = np.array([rc2, sampled], np.int64)
    s["words_seed_42"] = ref.proposal_words(42, 8)
    s["uniform_seed_9"] = ref.uniform_draws(9, 0.0, 1.0, 16)
    s["uniform_seed_9_scaled"] = ref.uniform_draws(9, 0.0, 3.75, 16)
    np.savez_compressed(HERE / "ref_sampling.npz", **s)

    for fixture, (module, geometry, seed, _, length, cache) in MODEL_CASES.items():
        tokens = model_tokens(fixture)
        selected = [length // 2, length - 2, length - 1]
        saved = run_python_reference(module, geometry, seed, tokens, selected, cache)
        keep = {k: v for k, v in saved.items() if not k[0] in "kv" or k in ("k0", "v0", "k5", "v5")}
        np.savez_compressed(HERE / f"{fixture}.npz", **keep)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
