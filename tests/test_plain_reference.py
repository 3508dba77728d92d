"""The plain implementation against (1) numbers that the reference project's own
modules produced on the CPU (tests/golden/reference_parts.json, made by
tests/golden/make_reference_parts.py) and (2) its own internal consistency:
causality, the equivalence of the two rotary pairings, the llama3 frequency rule."""
import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers as H
import plain_llama as P

GOLDEN = json.loads((Path(__file__).parent / "golden" / "reference_parts.json").read_text())


@pytest.fixture(scope="module")
def model_a():
    """Tiny configuration A with the weights the golden file was made with: numpy's frozen ``RandomState`` stream,
    the same values on every torch build."""
    import sys
    sys.path.insert(0, str(Path(__file__).parent / "golden"))
    import make_reference_gpu as G
    return dict(H.TINY_A), {k: v.double() for k, v in G.anchor_weights(H.TINY_A, seed=0).items()}


def close(a, b, tol=2e-6):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    assert a.shape == b.shape
    assert np.abs(a - b).max() <= tol * max(1.0, np.abs(b).max()), np.abs(a - b).max()


def test_parts_match_the_reference_modules(model_a):
    cfg, w = model_a
    tokens = torch.tensor(GOLDEN["tokens"])
    Hq, Hkv, hd, inter = 4, 2, 16, 176
    x = w["model.embed_tokens.weight"][tokens]
    close(x, GOLDEN["embed"])
    a = P.rms_norm(x, w["model.layers.0.input_layernorm.weight"], cfg["rms_norm_eps"])
    close(a, GOLDEN["attention_norm"])
    p = "model.layers.0.self_attn."
    wq = P.permute_for_interleaved_rope(w[p + "q_proj.weight"], Hq, hd)
    wk = P.permute_for_interleaved_rope(w[p + "k_proj.weight"], Hkv, hd)
    close(a @ wq.T, GOLDEN["q"])
    close(a @ wk.T, GOLDEN["k"])
    close(a @ w[p + "v_proj.weight"].T, GOLDEN["v"])
    f = P.rms_norm(x, w["model.layers.0.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    w13 = torch.cat([w["model.layers.0.mlp.gate_proj.weight"], w["model.layers.0.mlp.up_proj.weight"]])
    u = f @ w13.T
    close(u, GOLDEN["w13_out"])
    close(u[:, :inter] @ w["model.layers.0.mlp.down_proj.weight"].T, GOLDEN["w2_of_gate_half"])
    z = P.rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    close(z, GOLDEN["final_norm"])
    logits = z @ w["lm_head.weight"].T
    close(logits[:2], GOLDEN["logits_first_rows"])
    assert torch.argmax(logits, dim=-1).tolist() == GOLDEN["greedy"]


def test_names_shapes_and_defaults_of_the_reference():
    s = GOLDEN["state_dict_shapes"]
    assert s["layers.0.attention.wqkv.weight"] == [(4 + 2 * 2) * 16, 64]          # rows [Wq; Wk; Wv]
    assert s["layers.0.feed_forward.w13.weight"] == [2 * 176, 64] and s["output.weight"] == [512, 64]
    d = GOLDEN["modelargs_defaults"]
    assert d == dict(intermediate_size=256, head_dim=32, n_local_heads=3, norm_eps=1e-5, rope_base=10000.0)
    from batchspec_b200.config import get_config
    ours, ref = get_config("llama-3.1-8b"), GOLDEN["registry_llama31_8b"]
    assert (ours.num_hidden_layers, ours.hidden_size, ours.num_attention_heads, ours.num_key_value_heads,
            ours.intermediate_size, ours.vocab_size) == (ref["n_layer"], ref["dim"], ref["n_head"],
                                                         ref["n_local_heads"], ref["intermediate_size"], ref["vocab_size"])
    assert ours.rope_theta == ref["rope_base"] and ours.rms_norm_eps == ref["norm_eps"]
    rs = ours.rope_scaling
    assert (rs.factor, rs.low_freq_factor, rs.high_freq_factor, rs.original_max_position_embeddings) == \
        (ref["scaling_factor"], ref["low_freq_factor"], ref["high_freq_factor"], ref["original_max_position_embeddings"])


def test_interleaved_rotation_of_permuted_rows_equals_half_split_rotation():
    torch.manual_seed(0)
    Hn, hd, d, T = 3, 32, 24, 6
    w = torch.randn(Hn * hd, d, dtype=torch.float64)
    x = torch.randn(T, d, dtype=torch.float64)
    pos = torch.tensor([0, 1, 2, 7, 100, 4000])
    freqs = P.rope_frequencies(dict(H.TINY_B))
    q_perm = P.rope_interleaved((x @ P.permute_for_interleaved_rope(w, Hn, hd).T).reshape(T, Hn, hd), pos, freqs)
    q = (x @ w.T).reshape(T, Hn, hd)
    ang = pos.to(torch.float64)[:, None] * freqs[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    lo, hi = q[..., :hd // 2], q[..., hd // 2:]
    half = torch.cat([lo * c - hi * s, lo * s + hi * c], dim=-1)
    # same numbers, in permuted order: entry 2j of the interleaved head is entry j of the half-split head
    assert torch.allclose(q_perm[..., 0::2], half[..., :hd // 2], atol=1e-12)
    assert torch.allclose(q_perm[..., 1::2], half[..., hd // 2:], atol=1e-12)


def test_llama3_frequency_rule():
    cfg = dict(H.TINY_B)
    f = P.rope_frequencies(cfg)
    base = 500000.0 ** (-2.0 * torch.arange(16, dtype=torch.float64) / 32)
    wavelen = 2 * math.pi / base
    assert torch.equal(f[wavelen < 64 / 4], base[wavelen < 64 / 4])              # short waves untouched
    assert torch.allclose(f[wavelen > 64 / 1], base[wavelen > 64 / 1] / 8)       # long waves divided by the factor
    mid = (wavelen >= 16) & (wavelen <= 64)
    assert mid.any() and bool(((f[mid] <= base[mid]) & (f[mid] >= base[mid] / 8)).all())
    assert torch.equal(P.rope_frequencies({**cfg, "rope_scaling": None}), base)
    assert torch.allclose(P.rope_frequencies({**cfg, "rope_scaling": dict(rope_type="linear", factor=4.0)}), base / 4)


def test_forward_is_causal_and_prefix_stable(model_a):
    cfg, w = model_a
    toks = H.random_tokens(20, cfg["vocab_size"], 4)
    full = P.forward(cfg, w, toks)
    part = P.forward(cfg, w, toks[:11])
    assert torch.allclose(full[:11], part, atol=1e-12)
    other = P.forward(cfg, w, toks[:10] + [(toks[10] + 1) % 512] + toks[11:])
    assert torch.allclose(full[:10], other[:10], atol=1e-12) and not torch.allclose(full[10:], other[10:], atol=1e-6)


def test_attention_window_and_groups():
    torch.manual_seed(1)
    T, Hq, Hkv, hd = 9, 4, 2, 8
    q, k, v = (torch.randn(T, h, hd, dtype=torch.float64) for h in (Hq, Hkv, Hkv))
    out = P.causal_attention(q, k, v)
    s = (q[5, 3] @ k[:6, 1].T) / math.sqrt(hd)
    assert torch.allclose(out[5, 3], torch.softmax(s, 0) @ v[:6, 1], atol=1e-12)          # head 3 reads kv head 1
    win = P.causal_attention(q, k, v, window=3)
    s = (q[7, 0] @ k[5:8, 0].T) / math.sqrt(hd)
    assert torch.allclose(win[7, 0], torch.softmax(s, 0) @ v[5:8, 0], atol=1e-12)


def test_sampling_filters():
    p = torch.tensor([0.4, 0.3, 0.15, 0.1, 0.05], dtype=torch.float64)
    assert torch.allclose(P.top_k_top_p_filter(p, 2, 0.0), torch.tensor([4 / 7, 3 / 7, 0, 0, 0], dtype=torch.float64))
    assert torch.allclose(P.top_k_top_p_filter(p, 0, 0.75), torch.tensor([0.4, 0.3, 0.15, 0, 0], dtype=torch.float64) / 0.85)
    both = P.top_k_top_p_filter(p, 3, 0.5)
    assert torch.allclose(both, torch.tensor([4 / 7, 3 / 7, 0, 0, 0], dtype=torch.float64))
    assert torch.allclose(P.softmax_temperature(torch.log(p), 1.0), p)
