"""Plain, slow implementation of the Qwen2 dense decoder for the tests.

Whole sequences, no cache, one function per part, torch on the CPU, 64-bit by default.
It is written from the reference's formulas (each function cites file:line of
BusyaPrime/from-scratch-inference-engine-) and shares no code with the package under
test: it reads config.json and the safetensors file with its own few lines.
`tests/golden/` holds logits of the reference's own CPU model, compiled from its
sources, for one tiny random model; test_plain.py compares this file with them.
The sliding window is not in the reference (its attention has no mask beyond causality,
src/model/nn.cpp:186-224); `window` below follows the published meaning of the
config keys: a query at position p sees keys p - window + 1 .. p.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


# ----------------------------------------------------------------------------- loading
def read_config(model_dir):
    return read_config_dict(json.loads((Path(model_dir) / "config.json").read_text()))


def read_config_dict(j):
    """Keys and defaults of src/model/model_config.cpp:9-33."""
    heads = j["num_attention_heads"]
    c = {
        "hidden": j["hidden_size"], "layers": j["num_hidden_layers"], "heads": heads,
        "kv_heads": j.get("num_key_value_heads", heads),
        "head_dim": j.get("head_dim") or j["hidden_size"] // heads,
        "inter": j["intermediate_size"], "vocab": j["vocab_size"],
        "theta": j.get("rope_theta", 10000.0), "eps": j.get("rms_norm_eps", 1e-6),
        "bias": True if j.get("model_type", "") == "qwen2" else j.get("attention_bias", False),
        "windows": [0] * j["num_hidden_layers"],
    }
    if j.get("use_sliding_window", False):
        first = j.get("max_window_layers", c["layers"])
        c["windows"] = [j["sliding_window"] if l >= first else 0 for l in range(c["layers"])]
    return c


def read_safetensors(path, dtype=torch.float64):
    """Container layout of src/model/safetensors.cpp:23-111; every tensor widened."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    base = 8 + n
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        chunk = raw[base + b:base + e]
        if meta["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(chunk, dtype="<f4").copy())
        elif meta["dtype"] == "BF16":
            bits = np.frombuffer(chunk, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(bits.view(np.float32).copy())
        elif meta["dtype"] == "F16":
            t = torch.from_numpy(np.frombuffer(chunk, dtype="<f2").astype(np.float32))
        else:
            raise ValueError(meta["dtype"])
        out[name] = t.reshape(meta["shape"]).to(dtype)
    return out


# ------------------------------------------------------------------------------- parts
def stored_as(dtype):
    """What a value becomes when it is stored in `dtype` between two operations and read back
    (None: nothing happens to it).  Not in the reference, which stores float32 everywhere:
    with torch.bfloat16 the formulas below model an engine that keeps the residual stream
    and all sums in high precision but writes every operation's result in bfloat16."""
    if dtype is None:
        return lambda t: t
    return lambda t: t.to(dtype).to(t.dtype)


def embedding(weight, ids):
    """Row copy, src/model/nn.cpp:90-108."""
    return weight[torch.as_tensor(ids, dtype=torch.long, device=weight.device)]


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * w, plain gain, src/model/nn.cpp:45-72."""
    scale = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / x.shape[-1] + eps)
    return (x * scale) * weight


def linear(x, weight, bias=None):
    """x W^T + b, W [out, in], src/model/nn.cpp:15-39."""
    y = x @ weight.T
    return y if bias is None else y + bias


def rope(x, n_heads, head_dim, theta, positions):
    """Half-rotation pairs (i, i + head_dim/2), inv_freq = theta^(-2i/head_dim),
    src/model/nn.cpp:110-149."""
    s = x.shape[0]
    half = head_dim // 2
    inv_freq = torch.tensor([theta ** (-2.0 * i / head_dim) for i in range(half)],
                            dtype=torch.float64)
    ang = torch.as_tensor(positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
    c = torch.cos(ang).to(dtype=x.dtype, device=x.device)[:, None, :]
    sn = torch.sin(ang).to(dtype=x.dtype, device=x.device)[:, None, :]
    xh = x.reshape(s, n_heads, head_dim)
    x1, x2 = xh[..., :half], xh[..., half:]
    return torch.cat([x1 * c - x2 * sn, x2 * c + x1 * sn], dim=-1).reshape(s, n_heads * head_dim)


def attention(q, k, v, n_heads, n_kv_heads, head_dim, query_offset=0, window=0, store=None):
    """Causal grouped-query attention, two-pass softmax, head h uses kv head h // group,
    keys 0..query_offset+i inclusive, src/model/nn.cpp:151-226.  `store` (not in the
    reference; see `stored_as`): the unnormalised weights exp(score - max) are stored in that
    type before they multiply the values, while their sum is taken from the exact ones - what
    a tensor-core kernel does whose weights are a bfloat16 operand."""
    q_len, total = q.shape[0], k.shape[0]
    group = n_heads // n_kv_heads
    scale = 1.0 / math.sqrt(head_dim)
    out = torch.zeros_like(q)
    for h in range(n_heads):
        kvh = h // group
        kh = k[:, kvh * head_dim:(kvh + 1) * head_dim]
        vh = v[:, kvh * head_dim:(kvh + 1) * head_dim]
        for i in range(q_len):
            last = query_offset + i
            first = max(0, last - window + 1) if window > 0 else 0
            qv = q[i, h * head_dim:(h + 1) * head_dim]
            scores = (kh[first:last + 1] @ qv) * scale
            p = torch.exp(scores - scores.max())
            if store is None:
                p = p / p.sum()
                out[i, h * head_dim:(h + 1) * head_dim] = p @ vh[first:last + 1]
            else:
                out[i, h * head_dim:(h + 1) * head_dim] = \
                    (stored_as(store)(p) @ vh[first:last + 1]) / p.sum()
    return out


def silu_mul(gate, up):
    """(g / (1 + exp(-g))) * u, src/model/nn.cpp:74-88."""
    return (gate / (1.0 + torch.exp(-gate))) * up


# ------------------------------------------------------------------------------- model
def decoder_layer(config, weights, l, x, positions, shared_kv=None):
    """One pre-norm layer on a whole sequence, src/model/model.cpp:107-141.  Returns the new
    residual stream and this layer's (k, v).  With `shared_kv` the layer attends over those
    keys and values instead of its own (a run order in which a layer reads another layer's
    cache; not in the reference).  config["store"] (optional, see `stored_as`) is applied to
    every operation's result except the residual sum."""
    c, w = config, weights
    st = stored_as(c.get("store"))
    p = f"model.layers.{l}."
    normed = st(rms_norm(x, w[p + "input_layernorm.weight"], c["eps"]))

    def project(name):
        bias = w[p + f"self_attn.{name}_proj.bias"] if c["bias"] else None
        return st(linear(normed, w[p + f"self_attn.{name}_proj.weight"], bias))
    q = st(rope(project("q"), c["heads"], c["head_dim"], c["theta"], positions))
    if shared_kv is None:
        k = st(rope(project("k"), c["kv_heads"], c["head_dim"], c["theta"], positions))
        v = project("v")
    else:
        k, v = shared_kv
    attn = st(attention(q, k, v, c["heads"], c["kv_heads"], c["head_dim"], 0, c["windows"][l],
                        c.get("store")))
    x = x + st(linear(attn, w[p + "self_attn.o_proj.weight"]))
    normed2 = st(rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"]))
    act = st(silu_mul(st(linear(normed2, w[p + "mlp.gate_proj.weight"])),
                      st(linear(normed2, w[p + "mlp.up_proj.weight"]))))
    return x + st(linear(act, w[p + "mlp.down_proj.weight"])), (k, v)


def forward(config, weights, ids, schedule=None):
    """Logits [len(ids), vocab] of one whole sequence, src/model/model.cpp:90-149.
    `schedule` (not in the reference) is a run order [(layer, cache entry, writes)]; the
    default runs every layer once on its own keys."""
    c, w = config, weights
    positions = list(range(len(ids)))
    x = embedding(w["model.embed_tokens.weight"], ids)
    if schedule is None:
        schedule = [(l, l, True) for l in range(c["layers"])]
    stored = {}
    for l, entry, writes in schedule:
        x, kv = decoder_layer(c, w, l, x, positions, None if writes else stored[entry])
        if writes:
            stored[entry] = kv
    normed = stored_as(c.get("store"))(rms_norm(x, w["model.norm.weight"], c["eps"]))
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return linear(normed, head)


def load(model_dir, dtype=torch.float64):
    return read_config(model_dir), read_safetensors(Path(model_dir) / "model.safetensors", dtype)


def logits_of(model_dir, ids, dtype=torch.float64, store=None):
    config, weights = load(model_dir, dtype)
    config["store"] = store
    return forward(config, weights, ids)


# ----------------------------------------------------------------------------- sampling
def sample(logits, temperature, top_k, top_p, u):
    """temperature -> top-k -> top-p -> inverse CDF with the uniform number `u`,
    src/sampler/sampler.cpp:25-88.  Ties in the sort go to the smaller index (the
    reference's std::sort leaves them unspecified)."""
    logits = [float(v) for v in logits]
    vocab = len(logits)
    if temperature <= 0.0:
        best = 0
        for i in range(1, vocab):
            if logits[i] > logits[best]:
                best = i
        return best
    order = sorted(range(vocab), key=lambda i: (-logits[i], i))
    keep = top_k if 0 < top_k < vocab else vocab
    inv_temp = 1.0 / temperature
    mx = logits[order[0]] * inv_temp
    probs = [math.exp(logits[order[i]] * inv_temp - mx) for i in range(keep)]
    total = sum(probs)
    probs = [p / total for p in probs]
    nucleus = keep
    if top_p < 1.0:
        cumulative = 0.0
        for i in range(keep):
            cumulative += probs[i]
            if cumulative >= top_p:
                nucleus = i + 1
                break
    threshold = u * sum(probs[:nucleus])
    cumulative = 0.0
    for i in range(nucleus):
        cumulative += probs[i]
        if threshold <= cumulative:
            return order[i]
    return order[nucleus - 1]


def greedy_generate(config, weights, prompt, max_tokens):
    """Repeated whole forward, first-maximum argmax (tests/cpp/test_engine.cpp:38-47)."""
    ids = list(prompt)
    out = []
    for _ in range(max_tokens):
        row = forward(config, weights, ids)[-1]
        token = sample(row, 0.0, 0, 1.0, 0.0)
        out.append(token)
        ids.append(token)
    return out
