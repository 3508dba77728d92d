"""Makes ``reference_gpu.npz``: outputs of the reference project's OWN code on a GPU, for the parts of it that
cannot run on a CPU because they call its attention library: rotary encoding (plain and llama3,
models/modules/rope.py:27-62), the SwiGLU feed-forward (models/modules/feedforward.py:62), and whole-model
logits of ``StandardEngine.generate`` (backends/standard_engine.py:109-172) for prompts and for decoded tokens,
which pass through its cache writes (modules/kv_cache.py:64-83), causal grouped-query attention
(attention/standard.py:51-73) and the tied / untied head.

``tests/test_reference_anchor.py`` checks the plain implementation against these numbers on the CPU, and, on a
GPU box that has the reference's library built, runs this file's ``run`` again and compares live.

Run once on a B200, from the repository root:

    python tests/golden/make_reference_gpu.py

The unmodified reference tree is used through ``baseline/reference_arm.py``.  Weights come from numpy's frozen
``RandomState`` streams, rounded to bfloat16, so that every torch build sees the same values.
"""
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

# Two configurations that differ in every size and option, with head sizes the reference's library takes.
ANCHOR = {
    "scaled": dict(
        architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", vocab_size=320, hidden_size=192,
        num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2, head_dim=64, intermediate_size=320,
        rms_norm_eps=1e-5, rope_theta=500000.0,
        rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                          original_max_position_embeddings=64),
        max_position_embeddings=4096, tie_word_embeddings=False),
    "plain": dict(
        architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", vocab_size=250, hidden_size=128,
        num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=1, head_dim=128, intermediate_size=208,
        rms_norm_eps=1e-6, rope_theta=10000.0, rope_scaling=None, max_position_embeddings=2048,
        tie_word_embeddings=True),
}
PROMPT_LENS = (70, 45)
N_NEW = 6
ROPE_OFFSETS = (0, 60, 8188, 32764, 131068)
ROPE_RUN = 8


def anchor_weights(cfg: dict, seed: int) -> dict:
    """checkpoint name -> float32 tensor holding bfloat16-representable values."""
    rs = np.random.RandomState(seed)
    d, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    Hq, Hkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

    def mat(*shape):
        return torch.from_numpy(rs.standard_normal(shape) * 0.08).to(torch.bfloat16).float()

    def vec(n):
        return torch.from_numpy(1.0 + rs.standard_normal((n,)) * 0.1).to(torch.bfloat16).float()

    w = {"model.embed_tokens.weight": mat(V, d)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = vec(d)
        w[p + "self_attn.q_proj.weight"] = mat(Hq * hd, d)
        w[p + "self_attn.k_proj.weight"] = mat(Hkv * hd, d)
        w[p + "self_attn.v_proj.weight"] = mat(Hkv * hd, d)
        w[p + "self_attn.o_proj.weight"] = mat(d, Hq * hd)
        w[p + "post_attention_layernorm.weight"] = vec(d)
        w[p + "mlp.gate_proj.weight"] = mat(I, d)
        w[p + "mlp.up_proj.weight"] = mat(I, d)
        w[p + "mlp.down_proj.weight"] = mat(d, I)
    w["model.norm.weight"] = vec(d)
    if not cfg["tie_word_embeddings"]:
        w["lm_head.weight"] = mat(V, d)
    return w


def anchor_prompts(cfg: dict, seed: int):
    rs = np.random.RandomState(1000 + seed)
    return [rs.randint(0, cfg["vocab_size"], size=n).tolist() for n in PROMPT_LENS]


def rope_inputs(cfg: dict):
    """q/k whose every rotary pair is (1, 0) or (0.5, -0.25): the output shows the angle of each pair directly."""
    n = len(ROPE_OFFSETS) * ROPE_RUN
    hd = cfg["head_dim"]
    q = torch.zeros((n, 2, hd))
    q[:, 0, 0::2] = 1.0
    q[:, 1, 0::2], q[:, 1, 1::2] = 0.5, -0.25
    return q, q[:, :1].clone()


def run(names=("scaled", "plain")) -> dict:
    """Runs the reference on the current CUDA device; returns the arrays of the golden file."""
    from baseline import reference_arm as RA
    RA.import_reference()
    from batchspec.models.configs.model_config import ModelArgs
    from batchspec.models.modules.feedforward import FeedForward
    from batchspec.models.modules.rope import RoPEMixin
    out = {}
    for seed, name in enumerate(names):
        cfg = ANCHOR[name]
        w = anchor_weights(cfg, seed)
        args = ModelArgs.from_dict(RA.reference_config_dict(cfg))

        # --- rotary encoding alone, at small and at very large positions
        class Holder(RoPEMixin):
            config = args
        rope = Holder()._setup_rope_kernels()
        q, k = rope_inputs(cfg)
        indptr = torch.arange(0, (len(ROPE_OFFSETS) + 1) * ROPE_RUN, ROPE_RUN, dtype=torch.int32, device="cuda")
        offsets = torch.tensor(ROPE_OFFSETS, dtype=torch.int32, device="cuda")
        for dt_name, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
            try:
                rq, rk = rope(q.to("cuda", dt), k.to("cuda", dt), indptr, offsets)
                out[f"{name}.rope_q.{dt_name}"] = rq.float().cpu().numpy()
                out[f"{name}.rope_k.{dt_name}"] = rk.float().cpu().numpy()
            except Exception as exc:                       # the library may not take this dtype
                print(f"rope in {dt_name}: {type(exc).__name__}: {exc}")

        # --- the feed-forward module alone
        with torch.device("cuda"):
            ff = FeedForward(args).to(torch.bfloat16)
        p = "model.layers.0.mlp."
        ff.load_state_dict({"w1.weight": w[p + "gate_proj.weight"], "w3.weight": w[p + "up_proj.weight"],
                            "w2.weight": w[p + "down_proj.weight"]})
        x = torch.from_numpy(np.random.RandomState(77 + seed).standard_normal((9, cfg["hidden_size"]))).to(torch.bfloat16)
        out[f"{name}.ffn_x"] = x.float().numpy()
        with torch.inference_mode():
            out[f"{name}.ffn_y"] = ff.to("cuda")(x.cuda()).float().cpu().numpy()

        # --- the whole model through StandardEngine.generate
        prompts = anchor_prompts(cfg, seed)
        with tempfile.TemporaryDirectory() as tmp:
            ckpt = Path(tmp) / "model.pth"
            sd = RA.to_reference_state_dict(cfg, w)
            torch.save({k_: v.to(torch.bfloat16).contiguous() for k_, v in sd.items()}, str(ckpt))
            eng = RA.make_engine(cfg, f"bspec-anchor-{name}", ckpt, batch=len(prompts),
                                 max_seq_len=max(PROMPT_LENS) + N_NEW, chunk=128)
        probe = RA.StepProbe(eng.model, keep_logits=True)
        seqs = RA.make_sequences(prompts, [len(pr) + N_NEW for pr in prompts])      # each ends after N_NEW tokens
        done = RA.generate_quietly(eng, seqs)
        probe.close()
        done = sorted(done, key=lambda s: s.seq_id)
        assert [n for n, _, _ in probe.steps] == [sum(PROMPT_LENS)] + [len(prompts)] * (N_NEW - 1), probe.steps
        for i, s in enumerate(done):
            out[f"{name}.tokens.{i}"] = s.content[:len(prompts[i]) + N_NEW].cpu().numpy().astype(np.int32)
        out[f"{name}.prompt_logits"] = probe.logits[0].numpy()                      # [70 + 45, vocab], slot order
        out[f"{name}.decode_logits"] = torch.stack(probe.logits[1:]).numpy()        # [N_NEW - 1, 2, vocab]
        del eng
        torch.cuda.empty_cache()
    return out


if __name__ == "__main__":
    arrays = run()
    path = Path(__file__).parent / "reference_gpu.npz"
    np.savez_compressed(path, **{k: (v.astype(np.float16) if v.dtype == np.float32 and "logits" in k else v)
                                 for k, v in arrays.items()})
    print("wrote", path, {k: v.shape for k, v in arrays.items()})
