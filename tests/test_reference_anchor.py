"""The plain implementation against what the reference project's OWN code computed on a GPU
(tests/golden/reference_gpu.npz, made by tests/golden/make_reference_gpu.py on a B200 with the unmodified
reference tree): its rotary encoding with adjacent pairs, plain and with the llama3 frequency rule, up to position
131,075; its SwiGLU feed-forward; and whole-model logits of ``StandardEngine.generate`` for two prompts and five
decoded tokens each, on two configurations that differ in every size and option.  This pins the formulas that
the reference hands to its attention library (rotation and pairing, the llama3 rule, SiLU-times-up, causal mask,
1/sqrt(head_dim) scale, grouped-query head mapping, cache order) on something other than a reading of them.

The reference ran in bfloat16 (its library takes no float32 queries): tolerances are bfloat16's.

The ``gpu`` test runs the reference again, live, where its attention library is built for this GPU
(``python -m baseline.reference_arm --prebuild`` made ``baseline/_ref_ws``), and compares the same way."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers as H
import plain_llama as P

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "tests" / "golden"))
import make_reference_gpu as G                  # noqa: E402  (configurations, weights and prompts of the golden file)

GOLDEN_FILE = ROOT / "tests" / "golden" / "reference_gpu.npz"
BF16_EPS = 2.0 ** -8


def check_against_plain(data, names=("scaled", "plain")):
    for seed, name in enumerate(names):
        cfg = G.ANCHOR[name]
        w = {k: v.double() for k, v in G.anchor_weights(cfg, seed).items()}
        freqs = P.rope_frequencies(cfg)

        # rotary encoding: every pair of the input is a known vector, so each output pair shows its angle
        q, k = G.rope_inputs(cfg)
        positions = torch.cat([torch.arange(o, o + G.ROPE_RUN) for o in G.ROPE_OFFSETS])
        for x, key in ((q, "rope_q"), (k, "rope_k")):
            got = data[f"{name}.{key}.bf16"].astype(np.float64)
            ref = P.rope_interleaved(x.double(), positions, freqs).numpy()
            # bfloat16 output, and an angle the library forms in float32 (error grows with the position)
            tol = BF16_EPS + (positions.double().numpy() * 2.0 ** -22)[:, None, None]
            assert (np.abs(got - ref) <= tol).all(), (name, key, np.abs(got - ref).max())

        # feed-forward alone: bfloat16 products with float32 accumulation, bfloat16 between the stages
        p = "model.layers.0.mlp."
        x = torch.from_numpy(data[f"{name}.ffn_x"]).double()
        ref = P.swiglu(x, torch.cat([w[p + "gate_proj.weight"], w[p + "up_proj.weight"]]), w[p + "down_proj.weight"]).numpy()
        err = np.abs(data[f"{name}.ffn_y"] - ref).max() / np.abs(ref).max()
        assert err <= 2e-2, (name, "ffn", err)

        # whole model: all prompt rows, then five decoded tokens per request (the reference's own choices)
        seqs = [data[f"{name}.tokens.{i}"].tolist() for i in range(len(G.PROMPT_LENS))]
        assert [s[:n] for s, n in zip(seqs, G.PROMPT_LENS)] == G.anchor_prompts(cfg, seed)
        refs = [P.forward(cfg, w, s).numpy() for s in seqs]
        row = 0
        for i, n in enumerate(G.PROMPT_LENS):
            got = data[f"{name}.prompt_logits"][row:row + n].astype(np.float64)
            err = np.abs(got - refs[i][:n]).max() / np.abs(refs[i]).max()
            assert err <= H.TOL["bfloat16"], (name, "prompt", i, err)
            row += n
        dec = data[f"{name}.decode_logits"].astype(np.float64)                     # [steps, request, vocab]
        for t in range(dec.shape[0]):
            for i, n in enumerate(G.PROMPT_LENS):
                err = np.abs(dec[t, i] - refs[i][n + t]).max() / np.abs(refs[i]).max()
                assert err <= H.TOL["bfloat16"], (name, "decode", t, i, err)
        # the reference's greedy choice is the plain implementation's wherever the latter's margin is clear
        for i, n in enumerate(G.PROMPT_LENS):
            for t in range(G.N_NEW):
                r = refs[i][n - 1 + t]
                top2 = np.sort(r)[-2:]
                if top2[1] - top2[0] > 2 * H.TOL["bfloat16"] * np.abs(refs[i]).max():
                    assert int(np.argmax(r)) == seqs[i][n + t], (name, "greedy", i, t)


def test_plain_implementation_matches_the_reference_run_on_a_gpu():
    check_against_plain(np.load(GOLDEN_FILE))


def test_the_anchor_would_catch_a_wrong_formula(monkeypatch):
    """The comparison is sharp enough: the other rotary pairing, a missing llama3 rule, a wrong head mapping or
    gate/up swapped each fail it."""
    data = np.load(GOLDEN_FILE)
    real_freqs, real_swiglu, real_attn = P.rope_frequencies, P.swiglu, P.causal_attention

    def no_rule(cfg):
        return real_freqs(dict(cfg, rope_scaling=None))

    def swapped(x, w13, w2):
        half = w13.shape[0] // 2
        return real_swiglu(x, torch.cat([w13[half:], w13[:half]]), w2)

    def wrong_heads(q, k, v, **kw):
        return real_attn(q, k.flip(1), v.flip(1), **kw)

    def half_split(x, positions, freqs):
        ang = positions.double()[:, None] * freqs[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        h = x.shape[-1] // 2
        a, b = x[..., :h], x[..., h:]
        return torch.cat([a * c - b * s, a * s + b * c], dim=-1)

    for attr, wrong, names in (("rope_frequencies", no_rule, ("scaled",)), ("swiglu", swapped, ("scaled", "plain")),
                               ("causal_attention", wrong_heads, ("scaled",)),
                               ("rope_interleaved", half_split, ("scaled", "plain"))):
        with monkeypatch.context() as m:
            m.setattr(P, attr, wrong)
            with pytest.raises(AssertionError):
                check_against_plain(data, names)


@pytest.mark.gpu
def test_reference_live_on_this_gpu():
    from baseline import reference_arm as RA
    if not RA.SHIPPED_WS.is_dir():
        pytest.skip("the reference's attention library is not built for this GPU (python -m baseline.reference_arm --prebuild)")
    try:
        RA.import_reference()
    except Exception as exc:                                     # noqa: BLE001
        pytest.skip(f"the reference cannot be imported here: {type(exc).__name__}: {exc}")
    check_against_plain(G.run())
