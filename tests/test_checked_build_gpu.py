"""The checked build of the kernels (``BSPEC_BOUNDS=1``): indices that come from data are compared with their
ranges; one found outside is recorded and its access skipped.  The checks run in a child process, which builds the
checked library into a folder of its own on first use.  Every index that is "outside" here points into memory the
test owns (the declared extents are smaller than the buffers), so a check that failed to skip would show as a
changed canary, not as a fault."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

CHILD = r'''
import sys, tempfile
from pathlib import Path
import numpy as np
import torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
from batchspec_b200.kernels import ops
import helpers as H
import plain_llama as P
assert ops.bounds_build(), "BSPEC_BOUNDS=1 must select the checked library"
dev = torch.device("cuda:0")
i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)

# 1. a whole tiny model through the engine: nothing is reported and the tokens are the plain implementation's
from batchspec_b200.engine import Engine, Sequence
with tempfile.TemporaryDirectory() as tmp:
    cfg_json, seed, page = H.TINY["A"]
    folder = H.make_folder(Path(tmp), cfg_json, seed, dtype=torch.float32)
    cfg, w = P.read_model_folder(folder)
    prompt = H.random_tokens(23, cfg_json["vocab_size"], 5)
    want = P.greedy_generate(cfg, w, prompt, 6)
    for dtype in ("float32", "bfloat16"):
        eng = Engine(dtype=dtype, device="cuda:0")
        eng.load_model(model_dir=folder)
        eng.setup_caches(max_batch_size=2, max_seq_length=64, page_size=page)
        eng.setup_sampling_params(temperature=0.0)
        got = eng.generate([Sequence(0, prompt, max_new_tokens=6)])[0].output_ids
        ops.check_status()
        assert ops.bounds_reports() == []
        if dtype == "float32":
            assert list(got) == list(want), (got, want)
print("engine ok")

# 2. rotary encoding + cache append with a page id beyond the declared pages (the buffer has ten, six are declared)
Hq, Hkv, hd, ps = 4, 2, 32, 4
for dtype in (torch.float32, torch.bfloat16):
    for n in (3, 70):                                    # the per-head kernel and the 16-byte bfloat16 kernel
        backing = torch.full((10, 2, Hkv, ps, hd), 7.0, device=dev, dtype=dtype)
        cache = backing[:6]
        qkv = torch.randn(n, (Hq + 2 * Hkv) * hd, device=dev).to(dtype)
        table = ops.rope_frequency_table(10000.0 ** (-torch.arange(hd // 2, dtype=torch.float64) * 2 / hd), dev)
        pos = torch.arange(n, device=dev, dtype=torch.int32) % ps
        ent = torch.arange(n, device=dev, dtype=torch.int32)
        pages = [(i % 6) for i in range(n)]
        pages[1] = 8                                      # outside the six declared pages, inside the buffer
        ops.rope_kv_append(qkv, Hq, Hkv, hd, table, hd, False, pos, ent, i32(list(range(n + 1))), i32(pages), cache, ps)
        torch.cuda.synchronize()
        rep = ops.bounds_reports()
        assert len(rep) == 1 and rep[0][0] == "elementwise" and rep[0][1].startswith("page id") and rep[0][2:4] == (8, 6), rep
        assert bool((backing[6:] == 7.0).all()), "the write to the page outside the range was skipped"
        assert ops.bounds_reports() == [], "a report is read once"
        # a position beyond the request's block table (one slot): reported as a slot, nothing written
        backing.fill_(7.0)
        ops.rope_kv_append(qkv[:1], Hq, Hkv, hd, table, hd, False, i32([ps * 3]), i32([0]), i32([0, 1]), i32([2]), cache, ps)
        torch.cuda.synchronize()
        rep = ops.bounds_reports()
        assert len(rep) == 1 and rep[0][1].startswith("block-table slot") and rep[0][2:4] == (3, 1), rep
        assert bool((backing == 7.0).all())
print("append ok")

# 3. the q/k/v product's epilogue (head size 128) with the same faults
Hq, Hkv, hd, ps, K, M = 4, 2, 128, 16, 256, 3
w = (torch.randn((Hq + 2 * Hkv) * hd, K, device=dev) * 0.05).bfloat16()
x = torch.randn(M, K, device=dev).bfloat16()
table = ops.rope_frequency_table(10000.0 ** (-torch.arange(hd // 2, dtype=torch.float64) * 2 / hd), dev)
backing = torch.full((10, 2, Hkv, ps, hd), 7.0, device=dev, dtype=torch.bfloat16)
got = ops.linear_qkv_rope(x, w, Hq, Hkv, hd, table, hd, False, i32([0, 1, 2]), i32([0, 1, 2]), i32([0, 1, 2, 3]),
                          i32([1, 9, 3]), backing[:6], ps)
assert got is not None
torch.cuda.synchronize()
rep = ops.bounds_reports()
assert len(rep) == 1 and rep[0][0] == "gemm_tcgen05" and rep[0][2:4] == (9, 6), rep
assert bool((backing[6:] == 7.0).all()) and bool((backing[1, :, :, 0] != 7.0).all())
print("epilogue ok")

# 4. gather of a row beyond the source, an embedding id beyond the vocabulary
resid = torch.randn(6, 48, device=dev)
out = torch.full((2, 48), 7.0, device=dev)
ops.gather_rows_add(resid[:4], None, i32([1, 5]), out)
torch.cuda.synchronize()
rep = ops.bounds_reports()
assert len(rep) == 1 and rep[0][1].startswith("row") and rep[0][2:4] == (5, 4), rep
assert torch.equal(out[0], resid[1]) and bool((out[1] == 7.0).all())
emb = torch.randn(9, 16, device=dev)
res = torch.empty(2, 16, device=dev)
ops.embed(i32([3, 7]), emb[:5], res)
torch.cuda.synchronize()
rep = ops.bounds_reports()
assert len(rep) == 1 and rep[0][1].startswith("token id") and rep[0][2:4] == (7, 5), rep
assert torch.equal(res[0], emb[3]) and bool((res[1] == 0).all())
print("gather embed ok")

# 5. attention over plain loads (float32) with a page id beyond the declared pages: that key is left out, and reported
Hq, Hkv, hd, ps = 2, 1, 16, 4
backing = torch.randn(8, 2, Hkv, ps, hd, device=dev)
qkv = torch.randn(1, (Hq + 2 * Hkv) * hd, device=dev)
out = torch.empty(1, Hq * hd, device=dev)
from types import SimpleNamespace
ctx = SimpleNamespace(qo_indptr=i32([0, 1]), positions=i32([7]), tok_entry=i32([0]), n_entries=1, n_tokens=1,
                      max_q_len=1, max_kv_len=8, extras={})
tables = SimpleNamespace(kv_indptr=i32([0, 2]), kv_indices=i32([1, 6]), page_size=ps)
ops.paged_attention(qkv, out, backing[:5], ctx, tables, Hq, Hkv, hd, hd ** -0.5, 0)
torch.cuda.synchronize()
rep = ops.bounds_reports()
assert len(rep) == 1 and rep[0][0] == "attention_generic" and rep[0][2:4] == (6, 5), rep
q = qkv[0, :Hq * hd].view(Hq, hd)
k, v = backing[1, 0, 0], backing[1, 1, 0]                 # the four keys of the page inside the range
want = torch.softmax(q @ k.T * hd ** -0.5, -1) @ v
torch.testing.assert_close(out.view(Hq, hd), want, rtol=1e-4, atol=1e-5)
# the same through the bfloat16 kernel over plain asynchronous copies (a page size that TMA does not take)
Hq, Hkv, hd, ps = 2, 1, 64, 4
backing = (torch.randn(8, 2, Hkv, ps, hd, device=dev) * 0.5).bfloat16()
qkv = torch.randn(1, (Hq + 2 * Hkv) * hd, device=dev).bfloat16()
out16 = torch.empty(1, Hq * hd, device=dev, dtype=torch.bfloat16)
ops.paged_attention(qkv, out16, backing[:5], ctx, tables, Hq, Hkv, hd, hd ** -0.5, 0)
torch.cuda.synchronize()
rep = ops.bounds_reports()
assert len(rep) == 1 and rep[0][0] == "attention_bf16" and rep[0][2:4] == (6, 5), rep
# (the skipped keys are read as zeros here, not left out: a wrong result, reported, and no access outside)
assert bool(torch.isfinite(out16.float()).all())
print("bf16 attention ok")
try:
    ops.gather_rows_add(resid[:4], None, i32([1, 5]), out.new_empty(2, 48))
    ops.check_status()
    raise SystemExit("check_status did not raise")
except ops.KernelError as e:
    assert "row" in str(e)
print("all ok")
'''


def test_checked_build_reports_and_skips(tmp_path):
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    env = dict(os.environ, BSPEC_BOUNDS="1")
    out = subprocess.run([sys.executable, str(script), str(ROOT)], capture_output=True, text=True, env=env, timeout=900)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "all ok" in out.stdout


@pytest.mark.skipif(os.environ.get("BSPEC_BOUNDS", "0") == "1", reason="the suite itself runs on the checked build")
def test_ordinary_build_carries_no_checks():
    from batchspec_b200.kernels import ops
    assert not ops.bounds_build() and ops.bounds_reports() == []
