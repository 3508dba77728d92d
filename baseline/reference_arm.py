"""The reference arm: the unmodified siihwanpark/BatchSpec tree, driven through its own public path
``StandardEngine.load_model -> setup_caches -> setup_sampling_params -> setup_special_tokens ->
generate`` (batchspec/backends/standard_engine.py:23-100,145-172).  Nothing of ``batchspec_b200``
(models, kernels, engine) is on that path; this file only prepares what the reference asks for
and measures around it.

The reference ships neither ``setup.py`` nor ``pyproject.toml``, so "installing" it is putting a
copy of its tree under ``baseline/_ref`` and that folder on ``sys.path``.  Its attention, rotary
and activation kernels come from the FlashInfer library, which compiles them on first use; they
can be compiled ahead of time without a GPU (``python -m baseline.reference_arm --prebuild``)
into ``baseline/_ref_ws``, which is then copied to a fixed place in the temporary folder at run
time (the library's build files hold absolute paths).

What the reference needs and the repository has no file for:
* a checkpoint ``model.pth`` in its tensor names, with Wq/Wk rows permuted per head and q/k/v
  fused (tools/prepare_model/convert_weights.py:112-128,141-171): ``to_reference_state_dict``;
* a registry entry for sizes its table does not hold (``register_config``,
  batchspec/models/configs/registry.py);
* a tokenizer object with ``pad_token_id`` / ``eos_token_id`` / ``encode``
  (backends/base/engine.py:116-135): ``StubTokenizer``, whose end-of-sequence id no token equals,
  so that random weights never end a request early.
"""
from __future__ import annotations

import contextlib
import io
import os
import shutil
import sys
import tempfile
import time
from pathlib import Path
from typing import Dict, List, Optional

ROOT = Path(__file__).resolve().parent.parent
TREE = ROOT / "baseline" / "_ref"
SHIPPED_WS = ROOT / "baseline" / "_ref_ws"
RUN_WS = Path(tempfile.gettempdir()) / "bspec_reference_ws"


class ReferenceUnavailable(RuntimeError):
    pass


def ensure_tree() -> Path:
    """The reference's tree under ``baseline/_ref`` (copied there from ``$BSPEC_REFERENCE_SRC`` or from a
    folder ``reference`` beside the repository if it is not there yet)."""
    if (TREE / "batchspec" / "__init__.py").is_file() or (TREE / "batchspec" / "backends").is_dir():
        return TREE
    for cand in (os.environ.get("BSPEC_REFERENCE_SRC"), str(ROOT.parent / "reference")):
        if cand and (Path(cand) / "batchspec").is_dir():
            TREE.parent.mkdir(parents=True, exist_ok=True)
            shutil.copytree(cand, TREE)
            return TREE
    raise ReferenceUnavailable("no copy of siihwanpark/BatchSpec under baseline/_ref and none to copy from")


def use_workspace() -> None:
    """Point the attention library's build cache at a fixed place in the temporary folder, seeded with the
    ahead-of-time builds that travel with the repository (if any)."""
    if not RUN_WS.exists() and SHIPPED_WS.is_dir():
        tmp = RUN_WS.with_name(RUN_WS.name + f".{os.getpid()}")
        shutil.copytree(SHIPPED_WS, tmp)            # copy2: keeps the time stamps the build tool compares
        try:
            tmp.rename(RUN_WS)
        except OSError:
            shutil.rmtree(tmp, ignore_errors=True)
    os.environ["FLASHINFER_WORKSPACE_BASE"] = str(RUN_WS)
    os.environ.setdefault("FLASHINFER_CUDA_ARCH_LIST", "10.0a")


def import_reference():
    ensure_tree()
    use_workspace()
    if str(TREE) not in sys.path:
        sys.path.insert(0, str(TREE))
    import batchspec.backends.standard_engine as se       # noqa: F401  (the reference's module)
    return se


def prebuild(head_dims=(64, 128)) -> None:
    """Compile, without a GPU, the library modules the reference's bfloat16 standard path loads: rotary,
    silu-and-mul, page append and the paged prefill attention for the given head sizes; then keep them under
    ``baseline/_ref_ws``."""
    use_workspace()
    import torch
    import flashinfer
    import flashinfer.activation
    import flashinfer.page
    import flashinfer.prefill
    import flashinfer.rope
    t0 = time.time()
    flashinfer.rope.get_rope_module()
    print(f"rope {time.time() - t0:.0f}s", flush=True)
    flashinfer.activation.get_act_and_mul_module("silu")
    print(f"silu_and_mul {time.time() - t0:.0f}s", flush=True)
    flashinfer.page.get_page_module()
    print(f"page {time.time() - t0:.0f}s", flush=True)
    bf = torch.bfloat16
    for hd in head_dims:
        flashinfer.prefill.get_batch_prefill_module("fa2", bf, bf, bf, torch.int32, hd, hd, 0, False, False, False)
        print(f"batch prefill hd={hd} {time.time() - t0:.0f}s", flush=True)
    if SHIPPED_WS.exists():
        shutil.rmtree(SHIPPED_WS)
    shutil.copytree(RUN_WS, SHIPPED_WS)


class StubTokenizer:
    """What ``BaseEngine.setup_special_tokens`` reads of a tokenizer."""
    pad_token_id = 0
    eos_token_id = -1

    def encode(self, text, add_special_tokens=False):
        return [0]


def reference_config_dict(cfg: dict) -> dict:
    """config.json keys -> the reference's ``ModelArgs`` fields (models/configs/model_config.py:14-37; the
    correspondence is the one its registry entries show, registry.py:24-51)."""
    hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    out = dict(block_size=cfg.get("max_position_embeddings", 2048), vocab_size=cfg["vocab_size"],
               n_layer=cfg["num_hidden_layers"], n_head=cfg["num_attention_heads"],
               n_local_heads=cfg.get("num_key_value_heads") or cfg["num_attention_heads"], dim=cfg["hidden_size"],
               head_dim=hd, intermediate_size=cfg["intermediate_size"], rope_base=float(cfg.get("rope_theta", 10000.0)),
               norm_eps=float(cfg.get("rms_norm_eps", 1e-5)))
    rs = cfg.get("rope_scaling")
    if rs:
        kind = rs.get("rope_type", rs.get("type"))
        out["scaling_factor"] = float(rs["factor"])
        if kind == "llama3":
            out.update(low_freq_factor=rs["low_freq_factor"], high_freq_factor=rs["high_freq_factor"],
                       original_max_position_embeddings=rs["original_max_position_embeddings"])
        elif kind != "linear":
            raise ValueError(f"rope scaling {kind!r} has no counterpart in the reference")
    return out


def to_reference_state_dict(cfg: dict, hf: Dict[str, "torch.Tensor"]) -> Dict[str, "torch.Tensor"]:
    """Checkpoint-format tensors -> the reference's ``model.pth`` names and layouts
    (tools/prepare_model/convert_weights.py:29-43 names; :112-128 the per-head row permutation of Wq and Wk;
    :168-171 the fusion [q; k; v]).  w1/w3 stay separate: the reference fuses them at load
    (models/modules/feedforward.py:35-38).  A tied head becomes an explicit ``output.weight``: the reference
    never ties (models/base_model.py:126-127)."""
    import torch
    Hq = cfg["num_attention_heads"]
    Hkv = cfg.get("num_key_value_heads") or Hq
    hd = cfg.get("head_dim") or cfg["hidden_size"] // Hq

    def permute(w, n_head):
        return w.view(n_head, 2, hd // 2, w.shape[1]).transpose(1, 2).reshape(n_head * hd, w.shape[1])

    out = {"tok_embeddings.weight": hf["model.embed_tokens.weight"], "norm.weight": hf["model.norm.weight"],
           "output.weight": hf["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else hf["lm_head.weight"]}
    for i in range(cfg["num_hidden_layers"]):
        p, r = f"model.layers.{i}.", f"layers.{i}."
        out[r + "attention.wqkv.weight"] = torch.cat([permute(hf[p + "self_attn.q_proj.weight"], Hq),
                                                      permute(hf[p + "self_attn.k_proj.weight"], Hkv),
                                                      hf[p + "self_attn.v_proj.weight"]])
        out[r + "attention.wo.weight"] = hf[p + "self_attn.o_proj.weight"]
        out[r + "feed_forward.w1.weight"] = hf[p + "mlp.gate_proj.weight"]
        out[r + "feed_forward.w3.weight"] = hf[p + "mlp.up_proj.weight"]
        out[r + "feed_forward.w2.weight"] = hf[p + "mlp.down_proj.weight"]
        out[r + "attention_norm.weight"] = hf[p + "input_layernorm.weight"]
        out[r + "ffn_norm.weight"] = hf[p + "post_attention_layernorm.weight"]
    return out


def random_reference_checkpoint(cfg: dict, path: Path, seed: int = 0, device="cuda:0") -> None:
    """A ``model.pth`` of the reference's shapes with N(0, 0.02) matrices and 1 + N(0, 0.01) norms, drawn on the
    device (the benchmark's weights; values differ from this repository's random model of the same seed, the
    distributions are the same)."""
    import torch
    a = reference_config_dict(cfg)
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    bf = torch.bfloat16

    def mat(*shape):
        return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * 0.02).to(bf).cpu()

    def vec(n):
        return (1.0 + torch.randn((n,), generator=g, device=device, dtype=torch.float32) * 0.01).to(bf).cpu()

    d, I, V = a["dim"], a["intermediate_size"], a["vocab_size"]
    qkv = (a["n_head"] + 2 * a["n_local_heads"]) * a["head_dim"]
    sd = {"tok_embeddings.weight": mat(V, d), "norm.weight": vec(d), "output.weight": mat(V, d)}
    for i in range(a["n_layer"]):
        r = f"layers.{i}."
        sd[r + "attention.wqkv.weight"] = mat(qkv, d)
        sd[r + "attention.wo.weight"] = mat(d, a["n_head"] * a["head_dim"])
        sd[r + "feed_forward.w1.weight"] = mat(I, d)
        sd[r + "feed_forward.w3.weight"] = mat(I, d)
        sd[r + "feed_forward.w2.weight"] = mat(d, I)
        sd[r + "attention_norm.weight"] = vec(d)
        sd[r + "ffn_norm.weight"] = vec(d)
    torch.save(sd, str(path))


def make_engine(cfg: dict, name: str, checkpoint: Path, batch: int, max_seq_len: int, chunk: int,
                dtype="bfloat16", device="cuda:0"):
    """The reference's engine, set up the way its runner does (runner/runner.py:49-87)."""
    import torch
    se = import_reference()
    from batchspec.models.configs.registry import register_config
    register_config(name, reference_config_dict(cfg))
    eng = se.StandardEngine(StubTokenizer(), dtype=getattr(torch, dtype), device=device)
    eng.load_model(name, Path(checkpoint))
    eng.setup_caches(max_batch_size=batch, max_seq_length=max_seq_len, page_size=16, prefill_chunk_size=chunk)
    eng.setup_sampling_params(temperature=0.0, top_k=0, top_p=0.0)
    eng.setup_special_tokens()
    return eng


def make_sequences(prompts: List[List[int]], max_seq_len):
    """The reference's ``Sequence`` objects (backends/continuous/sequence.py); ``max_seq_len`` one number or one
    per prompt: a request ends when its prompt plus generated tokens reach it (continuous/scheduler.py:273-274)."""
    import torch
    import_reference()
    from batchspec.backends.continuous import Sequence
    lens = max_seq_len if isinstance(max_seq_len, (list, tuple)) else [max_seq_len] * len(prompts)
    return [Sequence(seq_id=i, max_seq_len=int(m), prompt_ids=torch.tensor(p, dtype=torch.int32, device="cuda"),
                     prompt_len=len(p)) for i, (p, m) in enumerate(zip(prompts, lens))]


class StepProbe:
    """Forward hooks on the reference's model (``torch.nn.Module`` hooks, no edit of its code): per step the number
    of tokens, a CUDA event and the host clock before the model runs, and optionally the logits it returns."""

    def __init__(self, model, keep_logits: bool = False):
        import torch
        self.torch = torch
        self.steps = []
        self.logits = []
        self.keep_logits = keep_logits
        self.h1 = model.register_forward_pre_hook(self._pre, with_kwargs=True)
        self.h2 = model.register_forward_hook(self._post)

    def _pre(self, module, args, kwargs):
        ids = kwargs.get("input_ids", args[0] if args else None)
        ev = self.torch.cuda.Event(enable_timing=True)
        ev.record()
        self.steps.append((int(ids.numel()), ev, time.perf_counter()))

    def _post(self, module, args, output):
        if self.keep_logits:
            self.logits.append(output.float().cpu())

    def close(self):
        self.h1.remove()
        self.h2.remove()


def generate_quietly(engine, sequences):
    """``generate`` with the per-step table its tracer prints (backends/continuous/tracer.py) sent nowhere."""
    with contextlib.redirect_stdout(io.StringIO()):
        return engine.generate(sequences)


def bench(cfg: dict, batch: int, prompt_len: int, steps: int, warmup: int, seed: int = 1) -> dict:
    """Decode speed of the reference at this batch: every request a ``prompt_len``-token prompt, prefilled in the
    chunks its runner picks for the batch size (runner/runner.py:69-72), then ``warmup + steps + 1`` greedy tokens
    (at least 32 untimed decode steps, until the SM clock has recovered from the prompt phase).
    Device time: CUDA events recorded before each model call, from the first timed decode step to the end of the
    last.  End to end: the host clock over the same steps (``generate`` keeps token ids on the device and reads
    one flag per request and step to test for the end of a sequence)."""
    import random
    import torch
    warmup = max(warmup, 32)             # the same count of untimed decode steps as the other arm's end-to-end run
    chunk = {2: 128, 4: 128, 8: 128, 16: 128, 32: 128, 64: 64, 128: 16, 256: 8}.get(batch, 128)
    n_new = warmup + steps + 1
    max_len = prompt_len + n_new
    tmp = Path(tempfile.mkdtemp(prefix="bspec_ref_ckpt_"))
    try:
        ckpt = tmp / "model.pth"
        random_reference_checkpoint(cfg, ckpt)
        eng = make_engine(cfg, "bspec-bench-model", ckpt, batch, max_len, chunk)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    rng = random.Random(seed)
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(prompt_len)] for _ in range(batch)]
    # a short run first: compiles and loads the library's kernels
    generate_quietly(eng, make_sequences(prompts, prompt_len + 4))
    eng.setup_caches(max_batch_size=batch, max_seq_length=max_len, page_size=16, prefill_chunk_size=chunk)
    probe = StepProbe(eng.model)
    torch.cuda.synchronize()
    done = generate_quietly(eng, make_sequences(prompts, max_len))
    end_ev = torch.cuda.Event(enable_timing=True)
    end_ev.record()
    torch.cuda.synchronize()
    t_end = time.perf_counter()
    probe.close()
    decode = [i for i, (n, _, _) in enumerate(probe.steps) if n == batch]
    # the pure decode steps are the last ones; skip ``warmup`` of them
    decode = [i for i in decode if i > max(j for j, (n, _, _) in enumerate(probe.steps) if n != batch)]
    timed = decode[warmup:]
    if len(timed) < steps:
        raise ReferenceUnavailable(f"the reference ran {len(decode)} decode steps, {warmup + steps} were asked for")
    timed = timed[:steps]
    first = probe.steps[timed[0]]
    after = probe.steps[timed[-1] + 1] if timed[-1] + 1 < len(probe.steps) else (0, end_ev, t_end)
    dev_ms = first[1].elapsed_time(after[1]) / steps
    wall_ms = (after[2] - first[2]) * 1e3 / steps
    return dict(ms_per_step=dev_ms, wall_ms_per_step=wall_ms, steps=steps, batch=batch, chunk=chunk, warmup_steps=warmup,
                generated=sum(int(s.num_generated_tokens) for s in done), model_calls=len(probe.steps))


if __name__ == "__main__":
    if "--prebuild" in sys.argv:
        prebuild()
    else:
        print(__doc__)
