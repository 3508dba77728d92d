"""Makes ``reference_parts.json``: outputs of the reference project's OWN modules
on the CPU, for the parts of it that run without a GPU, on tiny configuration A
with weights from numpy's frozen ``RandomState`` stream (``make_reference_gpu.anchor_weights``:
the same values on every torch build).  ``tests/test_plain_reference.py``
checks the plain implementation against these numbers.

Run once, from the repository root, with the reference on the path:

    PYTHONPATH=<reference checkout> python tests/golden/make_reference_parts.py

What runs on the CPU there: ``RMSNorm`` (models/modules/normalization.py), the
``nn.Linear`` projections and the embedding, the load hooks that fuse wq/wk/wv and
w1/w3 (modules/attention/base.py:63-77, modules/feedforward.py:33-38),
``_split_qkv`` (attention/base.py:83-94), ``ModelArgs`` defaults
(configs/model_config.py:39-55), ``get_config`` (configs/registry.py:144-179) and
greedy ``sample`` (backends/utils/sampling.py:89-90).  Rotary encoding, SiLU-mul,
attention and the cache writes call a GPU-only library there and cannot run here;
for those the plain implementation rests on the formulas cited in its docstrings.
"""
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

sys.path.insert(0, str(ROOT / "tests" / "golden"))

import helpers as H                     # noqa: E402
import make_reference_gpu as G          # noqa: E402
import plain_llama as P                 # noqa: E402
from batchspec.backends.utils.sampling import sample                      # noqa: E402  (the reference)
from batchspec.models.configs.model_config import ModelArgs               # noqa: E402
from batchspec.models.configs.registry import get_config                  # noqa: E402
from batchspec.models.standard_model import StandardTransformer           # noqa: E402


def main():
    cfgj = H.TINY_A
    w = {k: v.double() for k, v in G.anchor_weights(cfgj, seed=0).items()}
    args = ModelArgs(block_size=cfgj["max_position_embeddings"], vocab_size=cfgj["vocab_size"],
                     n_layer=cfgj["num_hidden_layers"], n_head=cfgj["num_attention_heads"], dim=cfgj["hidden_size"],
                     intermediate_size=cfgj["intermediate_size"], n_local_heads=cfgj["num_key_value_heads"],
                     head_dim=cfgj["head_dim"], rope_base=cfgj["rope_theta"], norm_eps=cfgj["rms_norm_eps"])
    model = StandardTransformer(args)
    Hq, Hkv, hd = args.n_head, args.n_local_heads, args.head_dim
    sd = {"tok_embeddings.weight": w["model.embed_tokens.weight"], "norm.weight": w["model.norm.weight"],
          "output.weight": w["lm_head.weight"]}
    for i in range(args.n_layer):
        p, q = f"model.layers.{i}.", f"layers.{i}."
        # un-fused names: the reference's load hooks fuse them
        sd[q + "attention.wq.weight"] = P.permute_for_interleaved_rope(w[p + "self_attn.q_proj.weight"], Hq, hd)
        sd[q + "attention.wk.weight"] = P.permute_for_interleaved_rope(w[p + "self_attn.k_proj.weight"], Hkv, hd)
        sd[q + "attention.wv.weight"] = w[p + "self_attn.v_proj.weight"]
        sd[q + "attention.wo.weight"] = w[p + "self_attn.o_proj.weight"]
        sd[q + "feed_forward.w1.weight"] = w[p + "mlp.gate_proj.weight"]
        sd[q + "feed_forward.w3.weight"] = w[p + "mlp.up_proj.weight"]
        sd[q + "feed_forward.w2.weight"] = w[p + "mlp.down_proj.weight"]
        sd[q + "attention_norm.weight"] = w[p + "input_layernorm.weight"]
        sd[q + "ffn_norm.weight"] = w[p + "post_attention_layernorm.weight"]
    model.load_state_dict({k: v.float() for k, v in sd.items()}, strict=True)
    model.eval()
    tokens = torch.tensor([5, 17, 400])
    out = {"tokens": tokens.tolist()}
    with torch.no_grad():
        x = model.tok_embeddings(tokens)
        layer = model.layers[0]
        a = layer.attention_norm(x)
        q, k, v = layer.attention._split_qkv(layer.attention.wqkv(a))
        f = layer.ffn_norm(x)
        u = layer.feed_forward.w13(f)
        d = layer.feed_forward.w2(u[:, :args.intermediate_size])
        z = model.norm(x)
        logits = model.output(z)
        out.update(embed=x.tolist(), attention_norm=a.tolist(), q=q.tolist(), k=k.tolist(), v=v.tolist(),
                   w13_out=u.tolist(), w2_of_gate_half=d.tolist(), final_norm=z.tolist(),
                   logits_first_rows=logits[:2].tolist(), greedy=sample(logits, 0.0, -1, 0.0).reshape(-1).tolist())
    out["state_dict_shapes"] = {k: list(t.shape) for k, t in model.state_dict().items() if k.startswith(("layers.0", "tok", "norm", "output"))}
    derived = ModelArgs(dim=96, n_head=3)
    out["modelargs_defaults"] = dict(intermediate_size=derived.intermediate_size, head_dim=derived.head_dim,
                                     n_local_heads=derived.n_local_heads, norm_eps=derived.norm_eps,
                                     rope_base=derived.rope_base)
    c = get_config("meta-llama/Llama-3.1-8B")
    out["registry_llama31_8b"] = dict(n_layer=c.n_layer, dim=c.dim, n_head=c.n_head, n_local_heads=c.n_local_heads,
                                      intermediate_size=c.intermediate_size, vocab_size=c.vocab_size,
                                      rope_base=c.rope_base, scaling_factor=c.scaling_factor,
                                      low_freq_factor=c.low_freq_factor, high_freq_factor=c.high_freq_factor,
                                      original_max_position_embeddings=c.original_max_position_embeddings,
                                      norm_eps=c.norm_eps)
    path = Path(__file__).with_name("reference_parts.json")
    path.write_text(json.dumps(out) + "\n")
    print(f"wrote {path} ({path.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
