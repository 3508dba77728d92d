"""What a model description may say beyond the Llama layer, shown with toy parts that are defined here and
registered without a change to the framework's files (none of them is anyone's model):

* block kinds with other slots than norm / mixer / norm / feed-forward: one with four norms, one with a single
  norm shared by two parallel branches;
* a part that runs once after the embedding (a learned absolute position table) and one on the head's output
  (a tanh soft cap);
* a mixer whose cache entry is ONE tensor per token, in pages of its own size (block tables of different
  lengths for the same request beside the attention's);
* a recurrent mixer with per-request state that is safe to capture in a CUDA graph: decode steps padded to a
  larger captured batch must not touch any live request's state.
"""
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import helpers as H
import plain_llama as P

pytestmark = pytest.mark.gpu

W, HD, RANK, CAP, MAXPOS, VOCAB = 40, 16, 12, 3.0, 96, 67
LATENT_PAGE = 3


def _register_shapes_lm():
    from batchspec_b200.config import register_config_class
    from batchspec_b200.models import LayerSpec, ModelSpec, RunEntry, register_model
    from batchspec_b200.parts import (BLOCKS, FEED_FORWARDS, INPUT_PARTS, LOGITS_PARTS, MIXERS, NORMS, Block, CacheSpec,
                                      InputPart, LogitsPart, Mixer, ParamSpec, PartSpec, register_part)

    @register_part(BLOCKS, "toy_sandwich")
    class Sandwich(Block):
        """x + post1(mixer(pre1(x))), then h + post2(ffn(pre2(h))): four norms."""
        SLOTS = {"pre1": NORMS, "mixer": MIXERS, "post1": NORMS, "pre2": NORMS, "ffn": FEED_FORWARDS, "post2": NORMS}

        def forward(self, resid, pending, ctx, cache):
            a = self.pre1.forward(resid, pending)
            y = self.post1.forward(self.mixer.forward(a, ctx, cache).float(), None)
            f = self.pre2.forward(resid, y)
            return resid, self.post2.forward(self.ffn.forward(f, ctx).float(), None)

    @register_part(BLOCKS, "toy_parallel")
    class Parallel(Block):
        """x + mixer(n(x)) + ffn(n(x)): one norm for both branches."""
        SLOTS = {"norm": NORMS, "mixer": MIXERS, "ffn": FEED_FORWARDS}

        def forward(self, resid, pending, ctx, cache):
            a = self.norm.forward(resid, pending)
            return resid, (self.mixer.forward(a, ctx, cache).float() + self.ffn.forward(a, ctx).float()).to(a.dtype)

    @register_part(MIXERS, "toy_latent")
    class Latent(Mixer):
        """Stores ONE tensor per token (c_t = x_t Wc^T, RANK numbers); a query attends causally over the cached
        latents and the mix of latents is projected back.  Reads the step's host fields: not graph-safe."""

        def __init__(self, runtime, dim, rank, page_size):
            self.runtime, self.dim, self.rank, self.page = runtime, dim, rank, page_size

        def param_specs(self):
            return {"c": ParamSpec((self.rank, self.dim)), "q": ParamSpec((self.rank, self.dim)),
                    "o": ParamSpec((self.dim, self.rank))}

        def bind(self, params):
            self.wc, self.wq, self.wo = (params[k].float() for k in "cqo")

        def cache_spec(self):
            return CacheSpec("full", (self.rank,), tensors=1, page_size=self.page)

        def forward(self, x, ctx, cache):
            t = ctx.tables[cache.group]
            assert t.page_size == self.page and cache.kv.shape[1] == 1
            pages = cache.kv.view(cache.kv.shape[0], self.page, self.rank)
            c, q = x.float() @ self.wc.T, x.float() @ self.wq.T
            out = torch.empty_like(x)
            for e in range(ctx.n_entries):
                b, en = int(ctx.h_qo_indptr[e]), int(ctx.h_qo_indptr[e + 1])
                table = torch.as_tensor(t.h_kv_indices[t.h_kv_indptr[e]:t.h_kv_indptr[e + 1]], device=x.device).long()
                pos = ctx.positions[b:en].long()
                pages[table[pos // self.page], pos % self.page] = c[b:en].to(pages.dtype)
                n_keys = int(ctx.h_kv_len[e])
                keys = pages[table].reshape(-1, self.rank)[:n_keys].float()
                s = (q[b:en] @ keys.T) / self.rank ** 0.5
                s = s.masked_fill(torch.arange(n_keys, device=x.device)[None, :] > pos[:, None], float("-inf"))
                out[b:en] = ((torch.softmax(s, -1) @ keys) @ self.wo.T).to(x.dtype)
            return out

    @register_part(INPUT_PARTS, "toy_abs_pos")
    class AbsPos(InputPart):
        def __init__(self, runtime, dim, max_pos):
            self.runtime, self.dim, self.max_pos = runtime, dim, max_pos

        def param_specs(self):
            return {"table": ParamSpec((self.max_pos, self.dim))}

        def bind(self, params):
            self.table = params["table"].float()

        def forward(self, resid, ctx):
            resid.add_(self.table[ctx.positions.long()])

    @register_part(LOGITS_PARTS, "toy_softcap")
    class SoftCap(LogitsPart):
        def __init__(self, runtime, cap):
            self.runtime, self.cap = runtime, cap

        def forward(self, logits, ctx):
            logits.copy_(self.cap * torch.tanh(logits / self.cap))

    @dataclass(frozen=True)
    class ShapesConfig:
        architecture: str
        vocab_size: int
        eps: float

        @classmethod
        def from_json_dict(cls, d):
            return cls(d["architectures"][0], d["vocab_size"], d["eps"])

        def to_json_dict(self):
            return dict(architectures=[self.architecture], vocab_size=self.vocab_size, eps=self.eps)

    def build(cfg):
        norm = PartSpec("rmsnorm", dict(dim=W, eps=cfg.eps))
        att = PartSpec("attention", dict(dim=W, n_heads=2, n_kv_heads=1, head_dim=HD, position=PartSpec("none", {})))
        latent = PartSpec("toy_latent", dict(dim=W, rank=RANK, page_size=LATENT_PAGE))
        ffn = PartSpec("swiglu", dict(dim=W, intermediate=56))
        names0 = {f"{s}.weight": f"a.{s}" for s in ("pre1", "post1", "pre2", "post2")}
        names0.update({"mixer." + k: "a." + k for k in "qkvo"})
        names0.update({"ffn.gate": "a.gate", "ffn.up": "a.up", "ffn.down": "a.down"})
        names1 = {"norm.weight": "b.n", "mixer.c": "b.c", "mixer.q": "b.q", "mixer.o": "b.o",
                  "ffn.gate": "b.gate", "ffn.up": "b.up", "ffn.down": "b.down"}
        layers = [LayerSpec(dict(pre1=norm, mixer=att, post1=norm, pre2=norm, ffn=ffn, post2=norm), names0, "toy_sandwich"),
                  LayerSpec(dict(norm=norm, mixer=latent, ffn=ffn), names1, "toy_parallel")]
        return ModelSpec(cfg.vocab_size, W, layers, [RunEntry(0), RunEntry(1)], norm, "emb", {"weight": "final"}, None,
                         input_part=PartSpec("toy_abs_pos", dict(dim=W, max_pos=MAXPOS)), input_names={"table": "pos"},
                         logits_part=PartSpec("toy_softcap", dict(cap=CAP)))

    register_config_class("ToyShapesLM", ShapesConfig)
    register_model("ToyShapesLM", build)


def _shapes_oracle(w, eps):
    def ffn(x, l):
        return P.swiglu(x, torch.cat([w[f"{l}.gate"], w[f"{l}.up"]]), w[f"{l}.down"])

    def oracle(tokens):
        T = len(tokens)
        x = w["emb"][torch.tensor(tokens)] + w["pos"][:T]
        a = P.rms_norm(x, w["a.pre1"], eps)
        q, k, v = ((a @ w[f"a.{n}"].T).reshape(T, h, HD) for n, h in (("q", 2), ("k", 1), ("v", 1)))
        y = P.causal_attention(q, k, v).reshape(T, 2 * HD) @ w["a.o"].T
        h = x + P.rms_norm(y, w["a.post1"], eps)
        x = h + P.rms_norm(ffn(P.rms_norm(h, w["a.pre2"], eps), "a"), w["a.post2"], eps)
        n = P.rms_norm(x, w["b.n"], eps)
        c, ql = n @ w["b.c"].T, n @ w["b.q"].T
        s = (ql @ c.T) / RANK ** 0.5
        s = s.masked_fill(torch.arange(T)[None, :] > torch.arange(T)[:, None], float("-inf"))
        x = x + (torch.softmax(s, -1) @ c) @ w["b.o"].T + ffn(n, "b")
        z = P.rms_norm(x, w["final"], eps) @ w["emb"].T
        return (CAP * torch.tanh(z / CAP)).numpy()
    return oracle


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_blocks_input_and_logits_parts_and_a_single_tensor_cache(tmp_path, dtype):
    from batchspec_b200.config import config_from_json_dict
    from batchspec_b200.engine import Engine, Sequence, StepEntry
    from batchspec_b200.weights import write_random_model
    _register_shapes_lm()
    cfg = config_from_json_dict(dict(architectures=["ToyShapesLM"], vocab_size=VOCAB, eps=1e-5))
    folder = write_random_model(cfg, tmp_path, seed=11, dtype=torch.float32 if dtype == "float32" else torch.bfloat16,
                                std=0.1, norm_std=0.1)
    _, w = P.read_model_folder(folder)
    oracle = _shapes_oracle(w, cfg.eps)
    eng = Engine(dtype=dtype, device="cuda:0")
    eng.load_model(model_dir=folder)
    assert set(eng.model.param_specs()) == set(w), "every slot's tensors are asked for under the names given"
    eng.setup_caches(max_batch_size=3, max_seq_length=48, page_size=4, num_pages=[20, 26])
    g_att, g_lat = eng.cache.groups
    assert (g_att.page_size, g_att.spec.tensors, g_lat.page_size, g_lat.spec.tensors) == (4, 2, LATENT_PAGE, 1)
    assert g_lat.pages.shape[2:] == (1, LATENT_PAGE * RANK) and g_att.pages.shape[2:] == (2, 4 * HD)
    assert eng.decode_graph(2) is None
    reqs = {f"s{i}": H.random_tokens(n, VOCAB, 90 + i) for i, n in enumerate((17, 29, 6, 23))}
    tol = H.TOL[dtype]
    for rid, toks in reqs.items():
        ref = oracle(toks)
        for sched in (H.whole(rid, toks), H.tail_decoded(rid, toks, tail=5), H.portions(rid, toks, [4, 2, 7, 3])):
            got = H.run_steps_in_process(eng, sched)
            assert set(got) == {(rid, p_) for p_ in range(len(toks))}
            for p_ in range(len(toks)):
                assert H.rel_err(got[(rid, p_)], ref[p_]) <= tol, (rid, p_, dtype)
    # tables of the two groups have different lengths for the same request
    eng.admit("t")
    eng.step([StepEntry("t", reqs["s1"][:10], ())])
    assert [len(t) for t in eng.cache.requests["t"].tables] == [3, 4]
    eng.release("t")
    got = H.run_steps_in_process(eng, H.mixed(reqs, seed=5, max_live=3))
    for rid, toks in reqs.items():
        ref = oracle(toks)
        for p_ in range(len(toks)):
            assert H.rel_err(got[(rid, p_)], ref[p_]) <= tol, (rid, p_, dtype)
    assert g_att.pool.high_water > 0 and g_lat.pool.high_water > g_att.pool.high_water
    eng.cache.check_invariants()
    if dtype == "float32":
        # through the scheduler, with pools so small that requests wait for pages of either group
        eng.setup_caches(max_batch_size=3, max_seq_length=40, page_size=4, num_pages=[14, 17], prefill_chunk_size=5,
                         max_tokens_per_step=9)
        eng.setup_sampling_params(temperature=0.0)
        seqs = [Sequence(rid, toks[:12], max_new_tokens=6) for rid, toks in reqs.items()]
        done = {s.seq_id: s for s in eng.generate(seqs)}
        for rid, toks in reqs.items():
            prompt = list(toks[:12])
            seq = list(prompt)
            for _ in range(6):
                seq.append(int(np.argmax(oracle(seq)[-1])))
            assert done[rid].output_ids == seq[len(prompt):], rid
        eng.cache.check_invariants()


def test_a_graph_safe_mixer_with_state_under_padded_captured_steps(tmp_path):
    """Three requests decode through a graph captured for four rows: the padding row reads and writes the reserved
    state slot, never a live request's.  Tokens equal those of the same engine without graphs."""
    from batchspec_b200.config import config_from_json_dict, register_config_class
    from batchspec_b200.engine import Engine, Sequence
    from batchspec_b200.models import ModelSpec, RunEntry, prenorm_layer, register_model
    from batchspec_b200.parts import MIXERS, Mixer, ParamSpec, PartSpec, StateSpec, register_part
    from batchspec_b200.weights import write_random_model
    DECAY = 0.7

    @register_part(MIXERS, "toy_decay_device")
    class DecayOnDevice(Mixer):
        """s_t = DECAY * s_{t-1} + x_t per request, output s_t W^T; device work only, sizes from the counts of
        tokens and entries alone."""
        graph_safe = True

        def __init__(self, runtime, dim):
            self.runtime, self.dim = runtime, dim

        def param_specs(self):
            return {"w": ParamSpec((self.dim, self.dim))}

        def bind(self, params):
            self.w = params["w"].float()

        def state_spec(self):
            return StateSpec((self.dim,), torch.float32)

        def forward(self, x, ctx, cache):
            pos, ent = ctx.positions.float(), ctx.tok_entry.long()
            same = ent[:, None] == ent[None, :]
            lag = pos[:, None] - pos[None, :]
            mix = torch.where(same & (lag >= 0), DECAY ** lag.clamp(min=0), torch.zeros_like(lag))
            slots = ctx.state_slots.long()
            first = ctx.positions[ctx.qo_indptr[:-1].long()].float()
            carried = DECAY ** (pos - first[ent] + 1)
            s = mix @ x.float() + carried[:, None] * cache.state[slots[ent]]
            cache.state[slots] = s[(ctx.qo_indptr[1:] - 1).long()]
            return (s @ self.w.T).to(x.dtype)

    @dataclass(frozen=True)
    class Cfg:
        architecture: str
        vocab_size: int

        @classmethod
        def from_json_dict(cls, d):
            return cls(d["architectures"][0], d["vocab_size"])

        def to_json_dict(self):
            return dict(architectures=[self.architecture], vocab_size=self.vocab_size)

    def build(cfg):
        norm = PartSpec("rmsnorm", dict(dim=32, eps=1e-5))
        ffn = PartSpec("swiglu", dict(dim=32, intermediate=48))
        toy = PartSpec("toy_decay_device", dict(dim=32))
        att = PartSpec("attention", dict(dim=32, n_heads=2, n_kv_heads=1, head_dim=16,
                                         position=PartSpec("rope", dict(head_dim=16, theta=100.0))))
        layers = []
        for i, mixer in enumerate((toy, att, toy)):
            names = {"norm1.weight": f"l{i}.n1", "norm2.weight": f"l{i}.n2", "ffn.gate": f"l{i}.gate",
                     "ffn.up": f"l{i}.up", "ffn.down": f"l{i}.down"}
            names.update({"mixer.w": f"l{i}.w"} if mixer is toy else {"mixer." + k: f"l{i}.{k}" for k in "qkvo"})
            layers.append(prenorm_layer(norm, mixer, norm, ffn, names))
        return ModelSpec(cfg.vocab_size, 32, layers, [RunEntry(i) for i in range(3)], norm, "emb", {"weight": "final"}, None)

    register_config_class("ToyGraphStateLM", Cfg)
    register_model("ToyGraphStateLM", build)
    cfg = config_from_json_dict(dict(architectures=["ToyGraphStateLM"], vocab_size=59))
    folder = write_random_model(cfg, tmp_path, seed=3, dtype=torch.float32, std=0.2, norm_std=0.1)
    prompts = [H.random_tokens(n, 59, 20 + i) for i, n in enumerate((7, 12, 4))]
    outs = {}
    for graphs in (False, True):
        eng = Engine(dtype="float32", device="cuda:0")
        eng.load_model(model_dir=folder)
        eng.use_cuda_graphs = graphs
        eng.setup_caches(max_batch_size=4, max_seq_length=48, page_size=4)
        eng.setup_sampling_params(temperature=0.0)
        assert eng.cache.state_tensors[0].shape[0] == 5, "four request slots and one that no request holds"
        done = eng.generate([Sequence(i, p, max_new_tokens=14) for i, p in enumerate(prompts)])
        outs[graphs] = {s.seq_id: s.output_ids for s in done}
        if graphs:
            assert eng.model.graph_safe and 4 in eng._graphs and eng._graphs[4].uses >= 10, "decode ran through a padded graph"
    assert outs[True] == outs[False]


# --------------------------------------------------------- a window at the head size of the fast bfloat16 kernels

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_layer_at_head_size_128_with_released_pages(tmp_path, dtype):
    """A two-layer description made here: layer 0 sees all keys, layer 1 a window of 40, heads of 128 numbers and
    pages of 16 tokens, i.e. the sizes at which bfloat16 steps go to the TMA decode kernels and the tensor-core prompt
    kernel.  Requests of 150 to 230 tokens are decoded far past the window, so block-table entries of pages that
    the window has passed (-1) and pages taken over by other requests reach those kernels in every way of cutting:
    whole, the tail decoded, in portions, and mixed in a pool so small that the window's pages are used again.  A
    key from outside the window that was still read (a released page, or another request's tokens in it) would
    change the average over 40 keys by far more than the tolerance."""
    from batchspec_b200.config import config_from_json_dict, register_config_class
    from batchspec_b200.engine import Engine
    from batchspec_b200.models import ModelSpec, RunEntry, prenorm_layer, register_model
    from batchspec_b200.parts import PartSpec
    from batchspec_b200.weights import write_random_model

    DIM, HQ, HKV, HEAD, WINDOW, INNER, VOC, THETA = 96, 4, 2, 128, 40, 80, 211, 10000.0

    @dataclass(frozen=True)
    class WinConfig:
        architecture: str
        vocab_size: int
        eps: float

        @classmethod
        def from_json_dict(cls, d):
            return cls(d["architectures"][0], d["vocab_size"], d["eps"])

        def to_json_dict(self):
            return dict(architectures=[self.architecture], vocab_size=self.vocab_size, eps=self.eps)

    def build(cfg):
        norm = PartSpec("rmsnorm", dict(dim=DIM, eps=cfg.eps))
        pos = PartSpec("rope", dict(head_dim=HEAD, theta=THETA))
        layers = []
        for i, window in enumerate((None, WINDOW)):
            att = PartSpec("attention", dict(dim=DIM, n_heads=HQ, n_kv_heads=HKV, head_dim=HEAD, position=pos,
                                             **({"window": window} if window else {})))
            ffn = PartSpec("swiglu", dict(dim=DIM, intermediate=INNER))
            names = {"norm1.weight": f"l{i}.n1", "norm2.weight": f"l{i}.n2", "ffn.gate": f"l{i}.gate",
                     "ffn.up": f"l{i}.up", "ffn.down": f"l{i}.down"}
            names.update({"mixer." + k: f"l{i}." + k for k in "qkvo"})
            layers.append(prenorm_layer(norm, att, norm, ffn, names))
        return ModelSpec(cfg.vocab_size, DIM, layers, [RunEntry(0), RunEntry(1)], norm, "emb", {"weight": "final"}, "head")

    register_config_class("ToyWindow128LM", WinConfig)
    register_model("ToyWindow128LM", build)
    cfg = config_from_json_dict(dict(architectures=["ToyWindow128LM"], vocab_size=VOC, eps=1e-5))
    folder = write_random_model(cfg, tmp_path, seed=31, dtype=torch.float32 if dtype == "float32" else torch.bfloat16,
                                std=0.08, norm_std=0.1)
    _, w = P.read_model_folder(folder)

    def rope(t, T):
        f = THETA ** (-2.0 * torch.arange(HEAD // 2, dtype=torch.float64) / HEAD)
        ang = torch.arange(T, dtype=torch.float64)[:, None] * f[None]
        c, sn = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        h = HEAD // 2
        return torch.cat([t[..., :h] * c - t[..., h:] * sn, t[..., :h] * sn + t[..., h:] * c], -1)

    def oracle(tokens):
        T = len(tokens)
        x = w["emb"][torch.tensor(tokens)]
        for i, window in enumerate((None, WINDOW)):
            a = P.rms_norm(x, w[f"l{i}.n1"], cfg.eps)
            q = rope((a @ w[f"l{i}.q"].T).reshape(T, HQ, HEAD), T)
            k = rope((a @ w[f"l{i}.k"].T).reshape(T, HKV, HEAD), T)
            v = (a @ w[f"l{i}.v"].T).reshape(T, HKV, HEAD)
            h = x + P.causal_attention(q, k, v, window=window).reshape(T, HQ * HEAD) @ w[f"l{i}.o"].T
            x = h + P.swiglu(P.rms_norm(h, w[f"l{i}.n2"], cfg.eps), torch.cat([w[f"l{i}.gate"], w[f"l{i}.up"]]),
                             w[f"l{i}.down"])
        return (P.rms_norm(x, w["final"], cfg.eps) @ w["head"].T).numpy()

    reqs = {f"w{i}": H.random_tokens(n, VOC, 50 + i) for i, n in enumerate((230, 150, 190, 170))}
    refs = {rid: oracle(toks) for rid, toks in reqs.items()}
    tol = H.TOL[dtype]

    def check(got, rids):
        assert set(got) == {(rid, p) for rid in rids for p in range(len(reqs[rid]))}
        for rid in rids:
            for p in range(len(reqs[rid])):
                assert H.rel_err(got[(rid, p)], refs[rid][p]) <= tol, (rid, p, dtype)

    eng = Engine(dtype=dtype, device="cuda:0")
    eng.load_model(model_dir=folder)
    eng.setup_caches(max_batch_size=4, max_seq_length=256, page_size=16, num_pages=[64, 24])
    assert [g.spec.policy for g in eng.cache.groups] == ["full", "window"]
    for rid, toks in reqs.items():
        for sched in (H.whole(rid, toks), H.tail_decoded(rid, toks, tail=64),
                      H.portions(rid, toks, [70, 2, 33, 16, 5, 48, 3])):
            check(H.run_steps_in_process(eng, sched), [rid])
    # all four live at once, decoded tokens of some beside portions of others, in a window pool that could not hold
    # one request whole (230 tokens are 15 pages; four requests share 22): the window's pages go round
    steps = H.mixed(reqs, seed=6, max_live=4, sizes=(60, 1, 1, 17, 1, 2, 33, 1, 1, 9, 1, 1))
    eng.setup_caches(max_batch_size=4, max_seq_length=256, page_size=16, num_pages=[H.max_live_tokens(steps, 16) // 16, 22])
    check(H.run_steps_in_process(eng, steps), list(reqs))
    window_pool = eng.cache.groups[1].pool
    assert window_pool.high_water <= 22 and window_pool.num_held == 0
    assert sum(-(-len(t) // 16) for t in reqs.values()) > 2 * 22, "the pool is far smaller than the requests"
