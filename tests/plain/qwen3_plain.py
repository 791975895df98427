"""Plain, slow implementation of the Qwen3 dense decoder: the oracle of the test suite.

It rests on the reference's formulas only (beniaminp/jllm-serve is Java and Metal: its model
code cannot be compiled or imported where these tests run, so there is no golden output
from it). Every function cites the reference file and lines that give its formula, by
the file's path inside that project (`J/` = src/main/java/org/robomiri/jllm/).

Whole sequences, no cache, one function per part, tensors on the CPU. It shares no code
with the product: it reads config.json and model.safetensors with its own few lines.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

# --------------------------------------------------------------------------------------
# reading a model folder (its own reader: nothing of the product is imported)
# --------------------------------------------------------------------------------------

_NP_DTYPES = {"F32": np.float32, "F16": np.float16, "F64": np.float64, "I32": np.int32, "I64": np.int64}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """u64 little-endian header length, JSON header, raw data (J/safetensors/SafeTensors.java:269-362)."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    data = raw[8 + hlen:]
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        buf = data[lo:hi]
        shape = meta["shape"]
        if meta["dtype"] == "BF16":
            # bf16 -> f32 is bits << 16 (J/safetensors/SafeTensors.java:121-127)
            u16 = np.frombuffer(buf, dtype=np.uint16).astype(np.uint32) << 16
            arr = u16.view(np.float32)
        else:
            arr = np.frombuffer(buf, dtype=_NP_DTYPES[meta["dtype"]])
        out[name] = torch.from_numpy(arr.reshape(shape).copy())
    return out


class PlainConfig:
    """The config.json keys the Qwen3 parser reads, with its defaults (J/model/Families.java:166-171,711-719,735-800,913-914)."""

    def __init__(self, c: dict):
        self.dim = c["hidden_size"]
        self.layers = c["num_hidden_layers"]
        self.vocab = c["vocab_size"]
        self.heads = c["num_attention_heads"]
        self.kv_heads = c.get("num_key_value_heads", self.heads)
        self.head_dim = c.get("head_dim", self.dim // self.heads)
        self.ffn = c["intermediate_size"]
        self.eps = c.get("rms_norm_eps", 1e-6)
        self.theta = c.get("rope_theta", 10000.0)
        self.tied = c.get("tie_word_embeddings", False)
        self.bias = c.get("attention_bias", False)
        self.qk_norm = True               # qwen3: qkNorm = true (J/model/Families.java:168); a test of another family clears it
        self.partial = c.get("partial_rotary_factor", 1.0)
        self.rotary_dim = int(self.head_dim * self.partial) & ~1
        self.scaling = c.get("rope_scaling")
        self.max_positions = c.get("max_position_embeddings", 4096)
        # Qwen2's window rule: only with use_sliding_window, from layer max_window_layers on
        sw = c.get("sliding_window") or 0
        self.window = [0] * self.layers
        if sw > 0 and c.get("use_sliding_window", False):
            first = c.get("max_window_layers", self.layers)
            self.window = [sw if l >= first else 0 for l in range(self.layers)]


def load_plain(model_dir, dtype=torch.float32):
    model_dir = Path(model_dir)
    cfg = PlainConfig(json.loads((model_dir / "config.json").read_text()))
    w = {k: v.to(dtype) for k, v in read_safetensors(model_dir / "model.safetensors").items()}
    return cfg, w


# --------------------------------------------------------------------------------------
# the parts
# --------------------------------------------------------------------------------------

def embedding(table: torch.Tensor, tokens) -> torch.Tensor:
    """x[t] = E[token[t]], no scale for qwen3 (J/cpu/CpuBackend.java:947-958)."""
    return table[torch.as_tensor(tokens, dtype=torch.long)]


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """y = (x * (1 / sqrt(mean(x^2) + eps))) * w: scale first, then the gain (J/cpu/VectorKernels.java:630-634,675-685)."""
    ss = (x * x).sum(dim=-1, keepdim=True)
    s = 1.0 / torch.sqrt(ss / x.shape[-1] + eps)
    return (x * s) * gain


def linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    """out[t, r] = sum_c W[r, c] * in[t, c]; weights are [out, in] (J/cpu/CpuMatmul.java:390-396)."""
    y = x @ w.t()
    return y if b is None else y + b


def rope_inverse_frequencies(rotary_dim: int, theta: float, scaling: dict | None, max_positions: int) -> list[float]:
    """f_i = theta^(-2i/rotaryDim) (J/model/Rope.java:122-127); linear divides by the factor (:138-142);
    yarn blends plain and divided frequencies with a linear ramp (:186-208). Python floats are doubles."""
    half = rotary_dim // 2
    f = [1.0 / math.pow(theta, (2.0 * i) / rotary_dim) for i in range(half)]
    kind = "default" if scaling is None else scaling.get("rope_type", scaling.get("type", "default"))
    if kind == "default":
        return f
    factor = float(scaling.get("factor", 1.0))
    if kind == "linear":
        return [v / factor for v in f]
    if kind == "yarn":
        orig = int(scaling.get("original_max_position_embeddings", max_positions))
        beta_fast = float(scaling.get("beta_fast", 32))
        beta_slow = float(scaling.get("beta_slow", 1))
        truncate = bool(scaling.get("truncate", True))

        def correction_dim(rotations):
            return rotary_dim * math.log(orig / (rotations * 2 * math.pi)) / (2 * math.log(theta))

        low, high = correction_dim(beta_fast), correction_dim(beta_slow)
        low = max(math.floor(low) if truncate else low, 0)
        high = min(math.ceil(high) if truncate else high, rotary_dim - 1)
        if low == high:
            high += 0.001
        out = []
        for i in range(half):
            extra = 1.0 / math.pow(theta, (2.0 * i) / rotary_dim)
            inter = 1.0 / (factor * math.pow(theta, (2.0 * i) / rotary_dim))
            ramp = min(max((i - low) / (high - low), 0), 1)
            out.append(inter * ramp + extra * (1 - ramp))
        return out
    raise ValueError(f"rope scaling {kind!r} is not part of the plain implementation")


def rope_amplitude(scaling: dict | None) -> float:
    """Multiplier of cos and sin: yarn's attention_factor, else 0.1 ln(factor) + 1; 1 otherwise (J/model/Rope.java:75-85,170-172)."""
    if scaling is None or scaling.get("rope_type", scaling.get("type", "default")) != "yarn":
        return 1.0
    att = float(scaling.get("attention_factor", 0))
    if att > 0:
        return att
    factor = float(scaling.get("factor", 1.0))
    mscale, all_dim = float(scaling.get("mscale", 0)), float(scaling.get("mscale_all_dim", 0))
    both = mscale != 0 and all_dim != 0

    def get(scale, m):
        return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0

    return get(factor, mscale if both else 1) / get(factor, all_dim if both else 0)


def rope_table(positions, rotary_dim: int, theta: float, scaling=None, max_positions: int = 4096, dtype=torch.float32):
    """cos[p, i] = (float) cos(p * f_i), the angle in double (J/model/Rope.java:24-38)."""
    f = torch.tensor(rope_inverse_frequencies(rotary_dim, theta, scaling, max_positions), dtype=torch.float64)
    p = torch.as_tensor(positions, dtype=torch.float64)
    a = p[:, None] * f[None, :]
    amp = rope_amplitude(scaling)
    return (torch.cos(a) * amp).to(dtype), (torch.sin(a) * amp).to(dtype)


def apply_rope(v: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half pairing over the first rotary_dim values of each head: (a, b) = (v[i], v[i + half]) becomes
    (a cos - b sin, b cos + a sin) (J/cpu/VectorKernels.java:692-711). v is [T, heads, head_dim]."""
    half = cos.shape[-1]
    a, b = v[..., :half], v[..., half:2 * half]
    c, s = cos[:, None, :], sin[:, None, :]
    out = v.clone()
    out[..., :half] = a * c - b * s
    out[..., half:2 * half] = b * c + a * s
    return out


def causal_gqa_attention(q, k, v, scale: float, window: int = 0, positions=None) -> torch.Tensor:
    """Query head h reads kv head h // (H / Hkv) (J/cpu/KvCache.java:82,527); a row at position P sees keys
    [first, P] with first = max(0, P + 1 - window) under a window, else 0 (J/model/Attention.java:68-71);
    score = (q . k) * scale; softmax = exp(score - max) * (1 / sum) (J/cpu/KvCache.java:455-464,595-596);
    out = sum_s p_s v_s (:602-623). q is [T, H, hd]; k and v are [T, Hkv, hd]; returns [T, H * hd]."""
    T, H, hd = q.shape
    group = H // k.shape[1]
    pos = torch.arange(T) if positions is None else torch.as_tensor(positions)
    out = torch.zeros(T, H, hd, dtype=q.dtype)
    for h in range(H):
        kh, vh = k[:, h // group, :], v[:, h // group, :]
        scores = (q[:, h, :] @ kh.t()) * scale
        key_pos, row_pos = pos[None, :], pos[:, None]
        visible = key_pos <= row_pos
        if window > 0:
            visible &= key_pos >= row_pos + 1 - window
        scores = scores.masked_fill(~visible, float("-inf"))
        e = torch.exp(scores - scores.max(dim=-1, keepdim=True).values)
        p = e * (1.0 / e.sum(dim=-1, keepdim=True))
        out[:, h, :] = p @ vh
    return out.reshape(T, H * hd)


def silu(x: torch.Tensor) -> torch.Tensor:
    """x / (1 + e^-x) (J/cpu/VectorKernels.java:637-639)."""
    return x / (1.0 + torch.exp(-x))


def swiglu_feed_forward(xb, w_gate, w_up, w_down) -> torch.Tensor:
    """h = silu(Wgate x) * (Wup x); result = Wdown h (J/cpu/CpuBackend.java:661-669)."""
    return linear(silu(linear(xb, w_gate)) * linear(xb, w_up), w_down)


def attention_block(xb, w: dict, prefix: str, cfg: PlainConfig, window: int, cos, sin, k_v_from=None):
    """q/k/v projections, per-head q/k RMSNorm before RoPE (qwen3: qkNorm), RoPE, attention, o_proj
    (J/cpu/CpuBackend.java:422-458,595-615). Returns (result, (k, v)); `k_v_from` replaces this
    layer's own keys and values by another layer's (a layer that reads another layer's cache)."""
    T = xb.shape[0]
    b = (lambda n: w[prefix + n + ".bias"]) if cfg.bias else (lambda n: None)
    q = linear(xb, w[prefix + "q_proj.weight"], b("q_proj")).reshape(T, cfg.heads, cfg.head_dim)
    q = apply_rope(rmsnorm(q, w[prefix + "q_norm.weight"], cfg.eps) if cfg.qk_norm else q, cos, sin)
    if k_v_from is None:
        k = linear(xb, w[prefix + "k_proj.weight"], b("k_proj")).reshape(T, cfg.kv_heads, cfg.head_dim)
        v = linear(xb, w[prefix + "v_proj.weight"], b("v_proj")).reshape(T, cfg.kv_heads, cfg.head_dim)
        k = apply_rope(rmsnorm(k, w[prefix + "k_norm.weight"], cfg.eps) if cfg.qk_norm else k, cos, sin)
    else:
        k, v = k_v_from
    scale = 1.0 / math.sqrt(cfg.head_dim)  # J/model/Families.java:861
    att = causal_gqa_attention(q, k, v, scale, window)
    return linear(att, w[prefix + "o_proj.weight"], b("o_proj")), (k, v)


def forward(cfg: PlainConfig, w: dict, tokens, schedule=None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence: x += attn(norm(x)); x += mlp(norm(x)) per layer, final
    norm, LM head (tied: the embedding) (J/cpu/CpuBackend.java:936-989; J/model/ModelWeights.java:37).

    `schedule` is the order in which layers run: a list of (layer, cache_of) where cache_of is None
    for a layer run that has keys and values of its own, else the index of the earlier schedule
    entry whose keys and values it reads. None = every layer once, in order."""
    dtype = w["model.embed_tokens.weight"].dtype
    T = len(tokens)
    x = embedding(w["model.embed_tokens.weight"], tokens)
    cos, sin = rope_table(range(T), cfg.rotary_dim, cfg.theta, cfg.scaling, cfg.max_positions, dtype)
    if schedule is None:
        schedule = [(l, None) for l in range(cfg.layers)]
    kept = []
    for layer, cache_of in schedule:
        p = f"model.layers.{layer}."
        xb = rmsnorm(x, w[p + "input_layernorm.weight"], cfg.eps)
        y, kv = attention_block(xb, w, p + "self_attn.", cfg, cfg.window[layer], cos, sin,
                                None if cache_of is None else kept[cache_of])
        kept.append(kv)
        x = x + y
        xb = rmsnorm(x, w[p + "post_attention_layernorm.weight"], cfg.eps)
        x = x + swiglu_feed_forward(xb, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                    w[p + "mlp.down_proj.weight"])
    xb = rmsnorm(x, w["model.norm.weight"], cfg.eps)
    head = w["model.embed_tokens.weight"] if cfg.tied else w["lm_head.weight"]
    return linear(xb, head)


# --------------------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------------------

def argmax_lowest(logits) -> int:
    """The lowest index among equal maxima (J/sampling/Sampler.java:458-466)."""
    best = 0
    vals = logits.tolist()
    for i in range(1, len(vals)):
        if vals[i] > vals[best]:
            best = i
    return best


def sampling_weights(logits, temperature: float, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0):
    """The candidates and their unnormalised weights in drawing order (J/sampling/Sampler.java:352-419):
    top-k largest logits sorted descending (or, with top-p alone, the whole vocabulary sorted descending;
    with neither, the vocabulary in index order); w = exp((l - max) / T); top-p keeps the shortest sorted
    prefix whose cumulative share reaches top_p; min-p zeroes weights below min_p (the largest weight is 1).
    Ties sort by the lower index first."""
    l = torch.as_tensor(logits, dtype=torch.float32)
    V = l.shape[0]
    inv_t = 1.0 / temperature
    if (0 < top_k < V) or top_p < 1.0:
        order = sorted(range(V), key=lambda i: (-float(l[i]), i))
        if 0 < top_k < V:
            order = order[:top_k]
        idx = torch.tensor(order)
        is_sorted = True
    else:
        idx = torch.arange(V)
        is_sorted = False
    val = l[idx]
    w = torch.exp((val - val.max()) * inv_t).to(torch.float32)
    # top-p is over the whole distribution when top-k is off, over the top-k candidates otherwise
    total = float(w.double().sum())
    kept = len(idx)
    if is_sorted and top_p < 1.0:
        cum = 0.0
        for i in range(len(idx)):
            cum += float(w[i]) / total
            if cum >= top_p:
                kept = i + 1
                break
    idx, w = idx[:kept], w[:kept].clone()
    if min_p > 0:
        w[w < min_p] = 0.0
    return idx, w


def draw(idx, w, u: float) -> int:
    """r = u * total; the first candidate whose running sum exceeds r (J/sampling/Sampler.java:422-432)."""
    total = float(w.double().sum())
    r = u * total
    acc = 0.0
    for i in range(len(idx)):
        acc += float(w[i])
        if r < acc:
            return int(idx[i])
    return int(idx[int(torch.argmax(w))])


def greedy_generate(cfg, w, prompt, n_new: int, schedule=None) -> list[int]:
    """Whole-sequence recomputation for every new token: no cache anywhere."""
    toks = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward(cfg, w, toks, schedule)
        t = argmax_lowest(logits[-1])
        out.append(t)
        toks.append(t)
    return out
