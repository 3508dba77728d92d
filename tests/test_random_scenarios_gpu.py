"""Randomised scenarios (fixed seeds): the scheduler, the cache, captured decode steps and steps launched ahead
against a roomy eager engine (float32, exact tokens), and the step function under random cuts against the plain
implementation (both dtypes).  Each scenario draws its configuration, lengths, limits, budgets, pool size and
options from its seed; a failure names the seed and what it drew."""
import random

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("random_scenarios")
    out = {}
    for name in "ABC":
        for dt, tdt in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
            out[(name, dt)] = H.make_folder(root / (name + dt), H.TINY[name][0], H.TINY[name][1], dtype=tdt)
    return out


def _engine(folder, dtype, page, max_batch, **kw):
    from batchspec_b200.engine import Engine
    eng = Engine(dtype=dtype, device="cuda:0")
    eng.load_model(model_dir=folder)
    eng.setup_caches(max_batch_size=max_batch, page_size=page, **kw)
    return eng


def _generation_scenario(seed, folders):
    from batchspec_b200.engine import Sequence
    rng = random.Random(seed)
    name = rng.choice("ABC")
    cfgj, _, page0 = H.TINY[name]
    page = rng.choice([page0, 16] if page0 < 16 else [page0])
    max_seq = min(cfgj["max_position_embeddings"], rng.choice([64, 128, 200]))
    prompts, limits = [], []
    for i in range(rng.randint(1, 16)):
        n = rng.randint(1, 20) if rng.random() < 0.5 else rng.randint(1, max_seq - 8)
        prompts.append(H.random_tokens(n, cfgj["vocab_size"], seed * 100 + i))
        limits.append(rng.randint(1, max(1, min(50, max_seq - n))))
    max_batch = rng.randint(1, 6)
    chunk = rng.choice([2, 5, 8, 16, 24, 64])
    budget = max(chunk, max_batch, rng.choice([chunk, 2 * chunk, chunk * max_batch, 48]))
    sampled = rng.random() < 0.6
    top_k, top_p = rng.choice([-1, 5, 40]), rng.choice([1.0, 0.9, 0.5])
    tight = -(-max(len(p) + m for p, m in zip(prompts, limits)) // page) + rng.randint(1, 12)
    graphs, ahead = rng.random() < 0.8, rng.random() < 0.7
    with_eos = rng.random() < 0.5
    drew = dict(seed=seed, cfg=name, page=page, max_seq=max_seq, max_batch=max_batch, chunk=chunk, budget=budget,
                sampled=sampled, top_k=top_k, top_p=top_p, pages=tight, graphs=graphs, ahead=ahead,
                lens=[len(p) for p in prompts], limits=limits)

    def run(num_pages, graphs, ahead, eos):
        eng = _engine(folders[(name, "float32")], "float32", page, max_batch, max_seq_length=max_seq,
                      prefill_chunk_size=chunk, max_tokens_per_step=budget, num_pages=num_pages)
        eng.use_cuda_graphs, eng.decode_lookahead = graphs, ahead
        if sampled:
            eng.setup_sampling_params(temperature=0.9, top_k=top_k, top_p=top_p, seed=seed)
        else:
            eng.setup_sampling_params(temperature=0.0)
        eng.setup_special_tokens(eos_token_ids=eos)
        done = eng.generate([Sequence(i, p, max_new_tokens=m) for i, (p, m) in enumerate(zip(prompts, limits))])
        eng.cache.check_invariants()
        assert all(g.pool.num_held == 0 for g in eng.cache.groups), drew
        return {s.seq_id: list(s.output_ids) for s in done}, {s.seq_id: s.finish_reason for s in done}

    roomy = sum(-(-(len(p) + m) // page) for p, m in zip(prompts, limits)) + 8
    want = run(roomy, False, False, [])
    if with_eos:
        eos = sorted({want[0][i][len(want[0][i]) // 2] for i in range(0, len(prompts), 3) if len(want[0][i]) > 3})
        if eos:
            want = run(roomy, False, False, eos)
    else:
        eos = []
    got = run(tight, graphs, ahead, eos)
    for i in want[0]:
        assert got[0][i] == want[0][i], (drew, i)
    assert got[1] == want[1], drew


@pytest.mark.parametrize("first_seed", [0, 150, 1000])
def test_generation_under_random_pressure(folders, first_seed):
    for seed in range(first_seed, first_seed + 25):
        _generation_scenario(seed, folders)


def _schedule(requests, rng, max_live, sizes, p_take, p_want):
    waiting, live, steps = list(requests.items()), {}, []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0]
        entries, ended = [], []
        for rid in [r for r in live if rng.random() < p_take] or [rng.choice(list(live))]:
            toks, pos = live[rid]
            n = min(rng.choice(sizes), len(toks) - pos)
            entries.append(dict(id=rid, tokens=list(toks[pos:pos + n]),
                                want=[i for i in range(n) if rng.random() < p_want]))
            live[rid][1] = pos + n
            if pos + n == len(toks):
                ended.append(rid)
        rng.shuffle(entries)
        for rid in ended:
            del live[rid]
        steps.append(dict(step=len(steps), entries=entries, end=ended))
    return steps


def _replay_scenario(seed, folders, oracle):
    rng = random.Random(seed)
    name, dtype = rng.choice("ABC"), rng.choice(["float32", "bfloat16"])
    cfgj, _, page0 = H.TINY[name]
    page = rng.choice([page0, 16, 64 if name == "C" else 32])
    max_pos = cfgj["max_position_embeddings"]
    top = min(max_pos, rng.choice([20, 80, 300]))
    requests = {f"r{i}": H.random_tokens(rng.randint(1, top), cfgj["vocab_size"], seed * 50 + i)
                for i in range(rng.randint(1, 7))}
    sizes = rng.choice([(1,), (2, 1), (5, 2, 9, 1, 3, 16, 1, 1, 7, 2), (64, 1, 1), (33, 17, 1), (128, 3), (300,)])
    steps = _schedule(requests, rng, rng.randint(1, 4), sizes, rng.choice([1.0, 0.75, 0.4]),
                      rng.choice([1.0, 0.5, 0.1]))
    folder = folders[(name, dtype)]
    eng = _engine(folder, dtype, page, 4, num_pages=max(1, -(-H.max_live_tokens(steps, 64) // page)))
    got = H.run_steps_in_process(eng, steps)
    drew = dict(seed=seed, cfg=name, dtype=dtype, page=page, sizes=sizes, lens={k: len(v) for k, v in requests.items()})
    for rid, toks in requests.items():
        key = (name, dtype, tuple(toks))
        if key not in oracle:
            oracle[key] = H.oracle_logits(folder, toks)
        ref = oracle[key]
        scale = np.abs(ref).max()
        for p in range(len(toks)):
            if (rid, p) in got:
                err = float(np.abs(got[(rid, p)].astype(np.float64) - ref[p]).max() / scale)
                assert err <= H.TOL[dtype], (drew, rid, p, err)


def test_step_function_under_random_cuts(folders):
    oracle = {}
    for seed in range(120):
        _replay_scenario(seed, folders, oracle)


def test_generation_with_a_windows_group_under_random_pressure(tmp_path):
    """An architecture registered here from the framework's own parts: one layer that keeps every key and two
    that read a window, so that the cache has two groups with pools of their own and the window's pool is far
    smaller than a request.  Generation through tight pools, captured steps and steps launched ahead gives the
    tokens of a roomy eager engine."""
    from dataclasses import dataclass
    from batchspec_b200.config import config_from_json_dict, register_config_class
    from batchspec_b200.engine import Sequence
    from batchspec_b200.models import ModelSpec, prenorm_layer, RunEntry, register_model
    from batchspec_b200.parts import PartSpec
    from batchspec_b200.weights import write_random_model
    W, HD, HQ, HKV, VOC = 32, 16, 2, 1, 97

    @dataclass(frozen=True)
    class WinConfig:
        architecture: str
        vocab_size: int
        eps: float
        window: int

        @classmethod
        def from_json_dict(cls, d):
            return cls(d["architectures"][0], d["vocab_size"], d["eps"], d["window"])

        def to_json_dict(self):
            return dict(architectures=[self.architecture], vocab_size=self.vocab_size, eps=self.eps,
                        window=self.window)

    def build(cfg):
        norm = PartSpec("rmsnorm", dict(dim=W, eps=cfg.eps))
        pos = PartSpec("rope", dict(head_dim=HD, theta=100.0))
        full = PartSpec("attention", dict(dim=W, n_heads=HQ, n_kv_heads=HKV, head_dim=HD, position=pos))
        near = PartSpec("attention", dict(dim=W, n_heads=HQ, n_kv_heads=HKV, head_dim=HD, window=cfg.window,
                                          position=pos))
        ffn = PartSpec("swiglu", dict(dim=W, intermediate=40))

        def names(p):
            n = {"norm1.weight": p + ".n1", "norm2.weight": p + ".n2", "ffn.gate": p + ".gate", "ffn.up": p + ".up",
                 "ffn.down": p + ".down"}
            n.update({"mixer." + k: p + "." + k for k in "qkvo"})
            return n
        layers = [prenorm_layer(norm, full, norm, ffn, names("a")), prenorm_layer(norm, near, norm, ffn, names("b")),
                  prenorm_layer(norm, near, norm, ffn, names("c"))]
        return ModelSpec(cfg.vocab_size, W, layers, [RunEntry(0), RunEntry(1), RunEntry(2)], norm, "emb",
                         {"weight": "final"}, None)

    register_config_class("ToyWindowLM", WinConfig)
    register_model("ToyWindowLM", build)
    folders = {}
    for window in (5, 17, 40):
        cfg = config_from_json_dict(dict(architectures=["ToyWindowLM"], vocab_size=VOC, eps=1e-5, window=window))
        folders[window] = write_random_model(cfg, tmp_path / f"w{window}", seed=window, dtype=torch.float32, std=0.08,
                                             norm_std=0.1)
    preempted = 0
    for seed in range(40):
        rng = random.Random(seed)
        window, page, max_seq = rng.choice(list(folders)), rng.choice([4, 8, 16]), rng.choice([64, 128, 200])
        prompts, limits = [], []
        for i in range(rng.randint(1, 12)):
            n = rng.randint(1, 20) if rng.random() < 0.5 else rng.randint(1, max_seq - 8)
            prompts.append(H.random_tokens(n, VOC, seed * 100 + i))
            limits.append(rng.randint(1, max(1, min(60, max_seq - n))))
        max_batch, chunk = rng.randint(1, 5), rng.choice([2, 5, 8, 16, 24, 64])
        budget = max(chunk, max_batch, rng.choice([chunk, 2 * chunk, 48]))
        sampled = rng.random() < 0.5
        tight = [-(-max(len(p) + m for p, m in zip(prompts, limits)) // page) + rng.randint(1, 10),
                 max((window + page - 1) // page + 1, -(-min(chunk, budget) // page)) + rng.randint(0, 4)]
        graphs, ahead = rng.random() < 0.8, rng.random() < 0.7
        drew = dict(seed=seed, window=window, page=page, max_seq=max_seq, max_batch=max_batch, chunk=chunk,
                    budget=budget, sampled=sampled, pages=tight, graphs=graphs, ahead=ahead,
                    lens=[len(p) for p in prompts], limits=limits)

        def run(num_pages, graphs, ahead):
            eng = _engine(folders[window], "float32", page, max_batch, max_seq_length=max_seq,
                          prefill_chunk_size=chunk, max_tokens_per_step=budget, num_pages=num_pages)
            eng.use_cuda_graphs, eng.decode_lookahead = graphs, ahead
            eng.setup_sampling_params(temperature=0.9 if sampled else 0.0, top_k=20, top_p=0.9, seed=seed)
            done = eng.generate([Sequence(i, p, max_new_tokens=m) for i, (p, m) in enumerate(zip(prompts, limits))])
            eng.cache.check_invariants()
            assert all(g.pool.num_held == 0 for g in eng.cache.groups), drew
            assert [g.spec.policy for g in eng.cache.groups] == ["full", "window"]
            return ({s.seq_id: list(s.output_ids) for s in done}, {s.seq_id: s.finish_reason for s in done},
                    eng.last_stats["preemptions"])
        roomy = sum(-(-(len(p) + m) // page) for p, m in zip(prompts, limits)) + 8
        want = run([roomy, roomy], False, False)
        got = run(tight, graphs, ahead)
        assert got[0] == want[0] and got[1] == want[1], drew
        assert set(want[1].values()) == {"length"}, drew
        preempted += got[2]
    assert preempted > 20


def test_random_configurations_of_the_architecture(tmp_path):
    """Every size the configuration allows, drawn at random: head sizes in steps of 16 up to 256, any number of
    heads and groups, widths, inner sizes and vocabularies that are odd or no power of two, tied or separate
    output weights, every kind of position scaling, every page size; both dtypes; mixed replay with reused pages
    against the plain implementation."""
    from batchspec_b200.engine import Engine
    for seed in range(80):
        rng = random.Random(seed)
        hd = 16 * rng.randint(1, 16) if rng.random() < 0.6 else rng.choice([64, 128, 256])
        hkv, group = rng.randint(1, 4), rng.choice([1, 2, 3, 4, 5, 8])
        hidden = rng.choice([rng.randint(4, 80) * 8, rng.randint(20, 300) * 2, rng.randint(33, 301), 256, 512])
        inter = rng.choice([rng.randint(4, 100) * 8, rng.randint(33, 400), 128 * rng.randint(1, 6)])
        vocab = rng.choice([rng.randint(50, 3000), 1024, 128 * rng.randint(1, 20)])
        scaling = rng.choice([None, dict(rope_type="linear", factor=2.0),
                              dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                   original_max_position_embeddings=64)])
        cfgj = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", vocab_size=vocab,
                    hidden_size=hidden, num_hidden_layers=rng.randint(1, 2), num_attention_heads=hkv * group,
                    num_key_value_heads=hkv, head_dim=hd, intermediate_size=inter,
                    rms_norm_eps=rng.choice([1e-5, 1e-6, 3e-4]), rope_theta=rng.choice([10000.0, 500000.0]),
                    rope_scaling=scaling, max_position_embeddings=512, tie_word_embeddings=rng.random() < 0.5)
        dtype, page = rng.choice(["float32", "bfloat16"]), rng.choice([4, 8, 16, 32, 64])
        folder = H.make_folder(tmp_path / f"s{seed}", cfgj, seed, std=min(0.08, 1.2 / hidden ** 0.5),
                               dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
        requests = {f"r{i}": H.random_tokens(rng.randint(1, rng.choice([10, 70, 300])), vocab, seed * 10 + i)
                    for i in range(rng.randint(1, 4))}
        sizes = rng.choice([(1,), (2, 1), (5, 2, 9, 1, 3, 16, 1, 1, 7, 2), (64, 1, 1), (33, 17, 1), (300,),
                            (130, 1, 1, 1)])
        steps = H.mixed(requests, seed, max_live=rng.randint(1, 4), sizes=sizes)
        eng = Engine(dtype=dtype, device="cuda:0")
        eng.load_model(model_dir=folder)
        eng.setup_caches(max_batch_size=4, page_size=page,
                         num_pages=max(1, -(-H.max_live_tokens(steps, 64) // page)))
        got = H.run_steps_in_process(eng, steps)
        drew = {k: cfgj[k] for k in ("head_dim", "num_attention_heads", "num_key_value_heads", "hidden_size",
                                      "intermediate_size", "vocab_size")}
        for rid, toks in requests.items():
            ref = H.oracle_logits(folder, toks)
            scale = np.abs(ref).max()
            for p in range(len(toks)):
                err = float(np.abs(got[(rid, p)].astype(np.float64) - ref[p]).max() / scale)
                assert err <= H.TOL[dtype], (seed, dtype, page, drew, rid, p, err)
