"""A plain, slow Qwen3 dense decoder in numpy float64: whole sequences, no cache, one function
for each part.  It is the oracle of the test suite and shares no code with ``gophonic_b200``
(it even reads safetensors by itself).

It rests on the formulas of GetStream/gophonic, cited per function as ``path:line`` inside that
project; the project's own Go code cannot be compiled in this environment (no Go toolchain), so
there is no run of it behind these functions.  Its float64 test oracle
(internal/qwen3lm/lmtest/lmtest.go:165-283) hard-codes eps = 1e-6 and theta = 1e6; here both come
from the configuration.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np


# ---- checkpoint reading (independent of the library's reader) ------------------------------
def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    """name -> float64 array.  File layout: internal/safetensors/safetensors.go:83-122; a BF16
    value widens exactly as bits << 16 (internal/q8gemm/packed.go:178-179)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        lo, hi = e["data_offsets"]
        raw = data[lo:hi]
        if e["dtype"] == "BF16":
            bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            vals = bits.view(np.float32).astype(np.float64)
        elif e["dtype"] == "F32":
            vals = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif e["dtype"] == "F16":
            vals = np.frombuffer(raw, dtype="<f2").astype(np.float64)
        else:
            raise ValueError(f"{name}: dtype {e['dtype']}")
        out[name] = vals.reshape(e["shape"])
    return out


def read_model(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """The tensors of a Qwen3 dense checkpoint by name (internal/qwen3lm/weights.go:325-351); the
    head only when the embeddings are not tied."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    heads, kvh = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or H // heads
    out = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,)}
    if not cfg.get("tie_word_embeddings", False):
        out["lm_head.weight"] = (V, H)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        out.update({p + "input_layernorm.weight": (H,), p + "post_attention_layernorm.weight": (H,),
                    p + "self_attn.q_proj.weight": (heads * d, H), p + "self_attn.k_proj.weight": (kvh * d, H),
                    p + "self_attn.v_proj.weight": (kvh * d, H), p + "self_attn.o_proj.weight": (H, heads * d),
                    p + "self_attn.q_norm.weight": (d,), p + "self_attn.k_norm.weight": (d,),
                    p + "mlp.gate_proj.weight": (I, H), p + "mlp.up_proj.weight": (I, H), p + "mlp.down_proj.weight": (H, I)})
    return out


def seeded_values(seed: int, name: str, n: int, std: float, mean: float, first: int = 0) -> np.ndarray:
    """The library's seeded fill, restated (elements first .. first + n - 1 of the flattened
    tensor): element i of tensor ``name`` is made of the two
    splitmix64 words 2i and 2i + 1 of the key sha256("seed:name")[:8] (little endian), word(j) =
    finaliser(key + (j + 1) * 0x9E3779B97F4A7C15); the sum of their eight 16-bit fields, less
    262140, times fp32(std / sqrt(2 (2^32 - 1) / 3)), plus the mean, each step rounded to fp32;
    then rounded to bfloat16 as a BF16 checkpoint stores it.  Returned as float32 (exact)."""
    import hashlib
    key = np.uint64(int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little"))
    c = np.float32(std / math.sqrt(2.0 * (2.0 ** 32 - 1.0) / 3.0))
    out = np.empty(n, dtype=np.float32)
    step = 1 << 21
    with np.errstate(over="ignore"):
        for lo in range(0, n, step):
            hi = min(n, lo + step)
            j = np.arange(2 * (first + lo), 2 * (first + hi), dtype=np.uint64)
            x = key + (j + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15)
            x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
            x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
            x = x ^ (x >> np.uint64(31))
            s = np.zeros(2 * (hi - lo), dtype=np.int64)
            for shift in (0, 16, 32, 48):
                s += ((x >> np.uint64(shift)) & np.uint64(0xFFFF)).astype(np.int64)
            s = s[0::2] + s[1::2] - 262140
            out[lo:hi] = (s.astype(np.float32) * c).astype(np.float32) + np.float32(mean)
    return bf16_round(out).astype(np.float32)


def random_weights(cfg: dict, seed: int, matrix: float = 0.02, embedding: float = 0.02, head: float = 0.02,
                   norm: float = 0.02, only=None) -> Dict[str, np.ndarray]:
    """The tensors the library's random-weights mode makes for (cfg, seed): norm vectors centred on 1,
    everything else on 0.  ``only``: a predicate on names, for models of which a test needs a part."""
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if only is not None and not only(name):
            continue
        if name.endswith("norm.weight"):
            std, mean = norm, 1.0
        elif name == "model.embed_tokens.weight":
            std, mean = embedding, 0.0
        elif name == "lm_head.weight":
            std, mean = head, 0.0
        else:
            std, mean = matrix, 0.0
        out[name] = seeded_values(seed, name, int(np.prod(shape)), std, mean).reshape(shape)
    return out


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round to nearest even bfloat16 (internal/qwen3lm/lmtest/lmtest.go:136-140)."""
    b = np.asarray(x, dtype=np.float32).view(np.uint32)
    b = (b + 0x7FFF + ((b >> 16) & 1)) & np.uint32(0xFFFF0000)
    return b.view(np.float32).astype(np.float64)


# ---- parts -----------------------------------------------------------------------------------
def embed(ids: Sequence[int], table: np.ndarray) -> np.ndarray:
    """h[t] = table[id_t], no scaling, no position term (internal/qwen3lm/evaluator.go:594-599;
    weights.go:614-619)."""
    return table[np.asarray(ids, dtype=np.int64)].astype(np.float64)


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """y = x / sqrt(mean(x^2) + eps) * weight, plain weight (internal/qwen3lm/ops.go:251-254;
    kernels_scalar.go:15-35; oracle lmtest.go:178-189)."""
    ms = np.mean(x * x, axis=-1, keepdims=True)
    return x / np.sqrt(ms + eps) * weight


def rope_tables(positions: np.ndarray, rotary_dim: int, theta: float):
    """inv_freq_i = theta^(-2i/rot), angle = pos * inv_freq_i (internal/qwen3lm/weights.go:681-688;
    evaluator.go:847-858)."""
    i = np.arange(rotary_dim // 2, dtype=np.float64)
    inv = 1.0 / np.power(theta, 2.0 * i / rotary_dim)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(ang), np.sin(ang)


def apply_rope(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """Rotate-half over the first 2*len(cos) elements of each head: element i pairs with
    i + rot/2 (internal/qwen3lm/kernels_scalar.go:73-80; ops.go:235-246).  x: [T, heads, d]."""
    half = cos.shape[-1]
    out = x.copy()
    x1, x2 = x[..., :half], x[..., half:2 * half]
    c, s = cos[:, None, :], sin[:, None, :]
    out[..., :half] = x1 * c - x2 * s
    out[..., half:2 * half] = x2 * c + x1 * s
    return out


def causal_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, window: int = 0) -> np.ndarray:
    """q: [T, heads, d]; k, v: [T, kv_heads, d].  Head h reads kv head h // (heads / kv_heads);
    scores (q.k) * scale over j <= i (and j > i - window when a window is set); softmax; sum of
    values (internal/qwen3lm/ops.go:259-293; weights.go:693; oracle lmtest.go:231-260)."""
    T, heads, d = q.shape
    group = heads // k.shape[1]
    out = np.zeros_like(q)
    for h in range(heads):
        g = h // group
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        i = np.arange(T)[:, None]
        j = np.arange(T)[None, :]
        mask = j <= i
        if window > 0:
            mask &= j > i - window
        s = np.where(mask, s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(axis=-1, keepdims=True)
        out[:, h, :] = p @ v[:, g, :]
    return out


def attention_block(x: np.ndarray, w: Dict[str, np.ndarray], prefix: str, cfg: dict, positions: np.ndarray,
                    window: int = 0) -> np.ndarray:
    """q/k/v projections, per-head RMSNorm of q and k with the shared [head_dim] weights and the
    model's eps, RoPE on both, attention, output projection (internal/qwen3lm/evaluator.go:648-678;
    ops.go:231-248; weights.go:335-346)."""
    heads, kvh = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // heads
    T = x.shape[0]
    q = (x @ w[prefix + "q_proj.weight"].T).reshape(T, heads, d)
    k = (x @ w[prefix + "k_proj.weight"].T).reshape(T, kvh, d)
    v = (x @ w[prefix + "v_proj.weight"].T).reshape(T, kvh, d)
    q = rms_norm(q, w[prefix + "q_norm.weight"], cfg["rms_norm_eps"])
    k = rms_norm(k, w[prefix + "k_norm.weight"], cfg["rms_norm_eps"])
    cos, sin = rope_tables(positions, d, cfg["rope_theta"])
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    ctx = causal_attention(q, k, v, 1.0 / math.sqrt(d), window)
    return ctx.reshape(T, heads * d) @ w[prefix + "o_proj.weight"].T


def silu(x: np.ndarray) -> np.ndarray:
    """x * sigmoid(x) (internal/qwen3lm/ops.go:454-461)."""
    return x / (1.0 + np.exp(-x))


def swiglu_ffn(x: np.ndarray, w: Dict[str, np.ndarray], prefix: str) -> np.ndarray:
    """down(silu(gate(x)) * up(x)) (internal/qwen3lm/evaluator.go:679-682; ops.go:442-452;
    oracle lmtest.go:265-274)."""
    g = x @ w[prefix + "gate_proj.weight"].T
    u = x @ w[prefix + "up_proj.weight"].T
    return (silu(g) * u) @ w[prefix + "down_proj.weight"].T


def decoder_layer(h: np.ndarray, w: Dict[str, np.ndarray], layer: int, cfg: dict, positions: np.ndarray) -> np.ndarray:
    """Pre-norm residual block: h += attn(norm(h)); h += mlp(norm(h))
    (internal/qwen3lm/evaluator.go:638-683)."""
    p = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    h = h + attention_block(rms_norm(h, w[p + "input_layernorm.weight"], eps), w, p + "self_attn.", cfg, positions)
    h = h + swiglu_ffn(rms_norm(h, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")
    return h


def head_weight(w: Dict[str, np.ndarray]) -> np.ndarray:
    """lm_head.weight if the checkpoint has it, else the embedding table (qwen3/chat.go:55-65)."""
    return w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]


def forward_logits(ids: Sequence[int], cfg: dict, w: Dict[str, np.ndarray]) -> np.ndarray:
    """Logits [T, vocab] at every position of one whole sequence starting at position 0
    (final norm then head: internal/qwen3lm/evaluator.go:699-702, 357-381)."""
    h = embed(ids, w["model.embed_tokens.weight"])
    positions = np.arange(len(ids))
    for layer in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, w, layer, cfg, positions)
    y = rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    return y @ head_weight(w).T


# ---- token selection ------------------------------------------------------------------------
def argmax_first(logits: np.ndarray) -> int:
    """First index of the largest value; a NaN never wins (qwen3/chat.go:905-914)."""
    best, at = -math.inf, 0
    for i, v in enumerate(logits):
        if v > best:
            best, at = v, i
    return at


def draw01(seed: int, draw: int) -> float:
    """splitmix64(seed + (draw + 1) * gamma) >> 40, times 2^-24 (internal/qwen3lm/gpu.metal:575-582)."""
    m = (1 << 64) - 1
    x = (seed + (draw + 1) * 0x9E3779B97F4A7C15) & m
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & m
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & m
    x ^= x >> 31
    return float(x >> 40) * (1.0 / 16777216.0)


def sample_token(logits: np.ndarray, temperature: float, top_k: int, top_p: float, seed: int, draw: int):
    """qwen3/chat.go:808-847: greedy when temperature <= 0; else the k likeliest (k = top_k, or
    1024 when top_k is 0 or above 1024), descending, ties to the lower index; weights
    exp((x - top) / T) in float32 summed in order; nucleus cut at the first prefix reaching
    top_p * total; r = u * sum walked down the list.  Returns (token, candidates, weights)."""
    logits = np.asarray(logits, dtype=np.float32)
    if not temperature > 0:
        return argmax_first(logits), None, None
    k = top_k
    if k <= 0 or k > 1024:
        k = 1024
    k = min(k, len(logits))
    order = sorted(range(len(logits)), key=lambda i: (-float(logits[i]), i))[:k]
    inv = np.float32(1.0) / np.float32(temperature)
    top = logits[order[0]]
    probs = [np.float32(math.exp(float((logits[i] - top) * inv))) for i in order]
    total = np.float32(0)
    for p in probs:
        total = np.float32(total + p)
    n = k
    if 0 < top_p < 1:
        acc = np.float32(0)
        for i, p in enumerate(probs):
            acc = np.float32(acc + p)
            if acc >= np.float32(top_p) * total:
                n, total = i + 1, acc
                break
    r = np.float32(np.float32(draw01(seed, draw)) * total)
    for i in range(n):
        r = np.float32(r - probs[i])
        if r <= 0:
            return order[i], order[:n], probs[:n]
    return order[n - 1], order[:n], probs[:n]


def greedy_generate(prompt: Sequence[int], n_new: int, cfg: dict, w: Dict[str, np.ndarray],
                    stop_ids: Sequence[int] = ()) -> List[int]:
    """Recompute the whole sequence for every new token (no cache); the stop token is not
    emitted (qwen3/chat.go:331-345)."""
    ids = list(prompt)
    out: List[int] = []
    for _ in range(n_new):
        t = argmax_first(forward_logits(ids, cfg, w)[-1])
        if t in stop_ids:
            break
        out.append(t)
        ids.append(t)
    return out
