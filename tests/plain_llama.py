"""Plain, slow Llama-3 decoder: the oracle every engine test compares against.

Whole sequences, no cache, no batching, one function per part, float64 math on
the CPU.  It shares no code with ``batchspec_b200``: it has its own safetensors
reader, its own config handling and its own formulas, each written from the
reference project's source (cited as ``path:line`` inside that project).

Differences of *form* (not of function) from the product path, on purpose:

* the product keeps the checkpoint's half-split rotary layout and rotates the
  pairs (j, j + head_dim/2); this file does what the reference does: permute the
  rows of Wq and Wk (tools/prepare_model/convert_weights.py:112-128) and rotate
  adjacent pairs (2j, 2j+1) (batchspec/models/modules/rope.py:27-31,
  ``interleave=True``).  Equal logits from both is itself a test.
* the product fuses QKV and gate/up; here they are fused the way the reference
  fuses them (attention/base.py:66-70, feedforward.py:35-38) and split again.

Parts the reference delegates to a library whose source is not in the project
(the llama3 frequency rule, softmax attention, SiLU) rest on the public formulas
named in the docstrings below.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

F64 = torch.float64


# --------------------------------------------------------------------------- files

_ST_DTYPES = {"F32": (np.float32, 4), "F16": (np.float16, 2), "BF16": (np.uint16, 2),
              "I32": (np.int32, 4), "I64": (np.int64, 8), "F64": (np.float64, 8)}


def read_safetensors(path) -> dict:
    """name -> float64/int64 torch tensor.  8-byte little-endian header length,
    JSON header {name: {dtype, shape, data_offsets}}, then raw little-endian data."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        npdt, _ = _ST_DTYPES[meta["dtype"]]
        b, e = meta["data_offsets"]
        arr = np.frombuffer(raw[base + b:base + e], dtype=npdt).copy()
        if meta["dtype"] == "BF16":
            arr = (arr.astype(np.uint32) << 16).view(np.float32)
        t = torch.from_numpy(arr.astype(np.int64 if meta["dtype"].startswith("I") else np.float64))
        out[name] = t.reshape(meta["shape"])
    return out


def read_model_folder(folder):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    return cfg, read_safetensors(folder / "model.safetensors")


# --------------------------------------------------------------------------- parts

def rms_norm(x, weight, eps):
    """normalization.py:24-26,38-39: x * rsqrt(mean(x^2) + eps), then * weight
    (eps inside the root, no bias, no +1 on the weight)."""
    x = x.to(F64)
    return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight.to(F64)


def permute_for_interleaved_rope(w, n_head, head_dim):
    """convert_weights.py:112-128: rows of each head go from the checkpoint's
    [first half; second half] order to adjacent pairs."""
    dim = w.shape[1]
    return w.view(n_head, 2, head_dim // 2, dim).transpose(1, 2).reshape(n_head * head_dim, dim)


def rope_frequencies(cfg):
    """f_j = theta^(-2j/hd), j in [0, hd/2); rope.py:27-31 passes rope_theta and
    rope_scale to the library.  With low/high frequency factors (rope.py:33-44) the
    library applies the public Llama-3.1 rule: wavelengths shorter than
    old_ctx/high keep f_j, longer than old_ctx/low use f_j/factor, between them a
    linear blend in old_ctx/wavelength.  A plain ``linear`` scaling divides every
    f_j by the factor (rope_scale alone)."""
    hd = head_dim_of(cfg)
    j = torch.arange(0, hd // 2, dtype=F64)
    f = float(cfg["rope_theta"]) ** (-2.0 * j / hd)
    rs = cfg.get("rope_scaling")
    if not rs:
        return f
    kind = rs.get("rope_type", rs.get("type"))
    factor = float(rs["factor"])
    if kind == "linear":
        return f / factor
    assert kind == "llama3", kind
    low, high = float(rs["low_freq_factor"]), float(rs["high_freq_factor"])
    old = float(rs["original_max_position_embeddings"])
    wavelen = 2.0 * math.pi / f
    smooth = (old / wavelen - low) / (high - low)
    blended = (1.0 - smooth) * f / factor + smooth * f
    out = torch.where(wavelen > old / low, f / factor, blended)
    return torch.where(wavelen < old / high, f, out)


def rope_interleaved(x, positions, freqs):
    """x [T, H, hd] with rotary pairs adjacent: (x[2j], x[2j+1]) turns by the
    angle positions[t] * freqs[j]  (rope.py:27, interleave=True)."""
    ang = positions.to(F64)[:, None] * freqs[None, :]            # [T, hd/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = a * c - b * s
    out[..., 1::2] = a * s + b * c
    return out


def causal_attention(q, k, v, window=None, scale=None):
    """q [T,Hq,hd], k/v [T,Hkv,hd] of ONE sequence from position 0.  Query t sees
    keys 0..t (standard_engine.py:142 causal=True), scores scaled by 1/sqrt(hd)
    (the library default when sm_scale is not given, standard_engine.py:132-143),
    query head h reads kv head h // (Hq/Hkv) (attention/base.py:32-35).
    ``window`` (not a Llama option; for parts tests) keeps keys t-window+1..t."""
    T, Hq, hd = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    out = torch.empty_like(q)
    idx = torch.arange(T)
    mask = idx[None, :] > idx[:, None]
    if window is not None:
        mask = mask | (idx[None, :] < idx[:, None] - window + 1)
    for h in range(Hq):
        s = (q[:, h, :] @ k[:, h // g, :].T) * scale
        s = s.masked_fill(mask, float("-inf"))
        out[:, h, :] = torch.softmax(s, dim=-1) @ v[:, h // g, :]
    return out


def swiglu(x, w13, w2):
    """feedforward.py:25-27,62: u = x W13^T, gate = first half, up = second half,
    (gate * sigmoid(gate)) * up, then W2."""
    u = x @ w13.T
    inter = w13.shape[0] // 2
    gate, up = u[:, :inter], u[:, inter:]
    return (gate * torch.sigmoid(gate) * up) @ w2.T


# --------------------------------------------------------------------------- model

def head_dim_of(cfg):
    return int(cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"])


def attention_layer(x, positions, cfg, w, i, freqs):
    """attention/standard.py:51-73: fused QKV, split, rotate q and k, attend, Wo."""
    Hq = cfg["num_attention_heads"]
    Hkv = cfg.get("num_key_value_heads") or Hq
    hd = head_dim_of(cfg)
    p = f"model.layers.{i}.self_attn."
    wq = permute_for_interleaved_rope(w[p + "q_proj.weight"], Hq, hd)
    wk = permute_for_interleaved_rope(w[p + "k_proj.weight"], Hkv, hd)
    wqkv = torch.cat([wq, wk, w[p + "v_proj.weight"]])            # attention/base.py:66-70
    qkv = x @ wqkv.T
    q, k, v = qkv.split([Hq * hd, Hkv * hd, Hkv * hd], dim=-1)    # attention/base.py:92-93
    T = x.shape[0]
    q = rope_interleaved(q.reshape(T, Hq, hd), positions, freqs)
    k = rope_interleaved(k.reshape(T, Hkv, hd), positions, freqs)
    y = causal_attention(q, k, v.reshape(T, Hkv, hd))
    return y.reshape(T, Hq * hd) @ w[p + "o_proj.weight"].T


def forward(cfg, w, tokens):
    """Logits [T, vocab] (float64) for one whole sequence of token ids.
    base_model.py:53-56 (pre-norm residual block), standard_model.py:90-102."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.shape[0]
    positions = torch.arange(T)
    freqs = rope_frequencies(cfg)
    eps = cfg["rms_norm_eps"]
    x = w["model.embed_tokens.weight"][tokens].to(F64)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = x + attention_layer(rms_norm(x, w[p + "input_layernorm.weight"], eps),
                                positions, cfg, w, i, freqs)
        w13 = torch.cat([w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"]])
        x = h + swiglu(rms_norm(h, w[p + "post_attention_layernorm.weight"], eps),
                       w13, w[p + "mlp.down_proj.weight"])
    x = rms_norm(x, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return x @ head.T


def greedy_generate(cfg, w, prompt, n_new):
    """sampling.py:89-90: temperature 0 is argmax.  Recomputes the whole sequence
    for every token."""
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(torch.argmax(forward(cfg, w, seq)[-1])))
    return seq[len(prompt):]


def softmax_temperature(logits, temperature):
    """sampling.py:94-112: probabilities are softmax(logits / T)."""
    return torch.softmax(logits.to(F64) / temperature, dim=-1)


def top_k_top_p_filter(probs, top_k, top_p):
    """Joint filter of sampling.py:94-99 (top_k_top_p_sampling_from_logits): keep the
    top_k most probable tokens, then of those the smallest set whose mass reaches
    top_p, renormalised.  top_k <= 0 or top_p <= 0 switches that filter off."""
    p = probs.clone()
    if top_k and top_k > 0 and top_k < p.numel():
        kth = torch.sort(p, descending=True).values[top_k - 1]
        p = torch.where(p >= kth, p, torch.zeros_like(p))
        p = p / p.sum()
    if top_p and 0 < top_p < 1:
        sp, si = torch.sort(p, descending=True)
        cum = torch.cumsum(sp, 0)
        keep = (cum - sp) < top_p
        q = torch.zeros_like(p)
        q[si[keep]] = sp[keep]
        p = q / q.sum()
    return p
