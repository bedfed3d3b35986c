"""The Rugesun decoder on the GPU against the plain implementation
(``plain_rugesun``): each mechanism alone; whole prompts, token-by-token
decoding, portions down to two tokens, mixed batches with pages and slots
used again, long decoding past every window; keys at window and page edges and
far away, made to stand out; sizes that are 1 or equal; a layer without a
feed-forward; greedy generation through the engine."""
import math
import os

import numpy as np
import pytest
import torch

import plain_rugesun as pr
from helpers import (TOL, compare_trace, peak_tokens, random_tokens, run_trace_inprocess,
                     run_trace_subprocess, trace_mixed, trace_portions, trace_tail, trace_whole)
from rugesun_cases import CASES, PAGE_SIZES, make_folder

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = ["float32", "bfloat16"]
LENGTHS = {"A": [31, 45, 1, 2, 90, 17], "B": [23, 60, 3, 1, 41, 8], "C": [130, 75, 2, 200, 33, 64]}
NAMES = ["A", "B", "C", "Asharp", "Csharp"]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CASES.items()):
        folder = make_folder(str(tmp_path_factory.mktemp(f"rug{name}")), cfg, seed=11 + i)
        out[name] = (folder, pr.Plain(folder))
        if name in ("A", "C"):
            sharp = make_folder(str(tmp_path_factory.mktemp(f"rugsharp{name}")), cfg, seed=31 + i, sharpen=8.0)
            out[name + "sharp"] = (sharp, pr.Plain(sharp))
    return out


def sequences(name):
    key = name.replace("sharp", "")
    return {f"r{i}": random_tokens(n, CASES[key]["vocab"], 100 * i + n) for i, n in enumerate(LENGTHS[key])}


def replay(models, name, dtype, steps, tmp_path, max_tokens=None):
    folder, plain = models[name]
    out = run_trace_inprocess(folder, dtype, steps, str(tmp_path / "out"), max_tokens or peak_tokens(steps),
                              PAGE_SIZES[name.replace("sharp", "")])
    return out, plain


# In bfloat16 a router logit carries the rounding of everything before it, and where the last
# chosen expert lies within that of the first one left out, the engine may choose otherwise
# than the 64-bit plain implementation: a different, equally valid, result at that position.
# Such positions (by the plain implementation's own margin) are not compared in bfloat16, and
# the bfloat16 runs use the models whose attention is not peaked, so that what one position
# hands to later ones stays far below the tolerance.  The 32-bit runs compare everything.
ROUTING_MARGIN = 0.06
# Largest difference of a position's logits from the plain ones, relative to the largest logit.
# bfloat16: every layer norms its sum again, which passes a sub-layer's rounding on undamped
# (with a residual scale near 1 more than with 2); four such layers stay below this.
TOL16 = 5e-2


def compare(steps, out, seqs, plain, dtype, sharp=False):
    if dtype == "float32":
        # (where attention is peaked the 32-bit rounding of a score is multiplied on its way to the logits)
        return compare_trace(steps, out, seqs, plain, TOL[dtype] * (3 if sharp else 1))
    fed = {rid: 0 for rid in seqs}
    compared = skipped = 0
    for s in steps:
        row = 0
        for e in s["entries"]:
            rid, n = e["id"], len(e["tokens"])
            ref_all, margins = plain.logits(seqs[rid]), plain.margins(seqs[rid])
            for w in e.get("want", []):
                pos = fed[rid] + w
                got, ref = out[s["step"]][row], ref_all[pos].numpy()
                row += 1
                assert np.isfinite(got).all()
                if float(margins[pos]) < ROUTING_MARGIN:
                    skipped += 1
                    continue
                compared += 1
                err = float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-6))
                assert err <= TOL16, (f"step {s['step']} request {rid} position {pos} (place {w} of a portion "
                                           f"of {n} starting at {fed[rid]}): relative error {err:.3e}, "
                                           f"routing margin {float(margins[pos]):.4f}")
            fed[rid] += n
        for rid in s.get("end", []):
            fed[rid] = 0
    assert compared > 2 * skipped
    return compared


def names_for(dtype):
    return NAMES if dtype == "float32" else ["A", "B", "C"]


def runtime(dtype, **options):
    from infernum_b200.ops import core
    from infernum_b200.parts.base import Runtime
    return Runtime(DEV, dtype, err=core.new_error_word(DEV), options=options)


def rel_err(got, ref):
    ref = ref.double().cpu()
    return float((got.double().cpu() - ref).abs().max() / max(ref.abs().max().item(), 1e-9))


PART_TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2}


# ---- whole models through the trace runner -------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(models, name, dtype, tmp_path):
    if name not in names_for(dtype):
        pytest.skip("peaked attention is compared in 32-bit")
    seqs = sequences(name)
    steps = []
    for rid, seq in seqs.items():
        steps += trace_whole(rid, seq, step0=len(steps))
    out, plain = replay(models, name, dtype, steps, tmp_path)
    compare(steps, out, seqs, plain, dtype, "sharp" in name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_most_in_one_step_then_token_by_token_past_the_windows(models, name, dtype, tmp_path):
    if name not in names_for(dtype):
        pytest.skip("peaked attention is compared in 32-bit")
    seqs = {k: v for k, v in sequences(name).items() if len(v) > 3}
    steps = []
    for rid, seq in seqs.items():
        steps += trace_tail(rid, seq, 80, step0=len(steps))  # longer than every window of the cases
    out, plain = replay(models, name, dtype, steps, tmp_path)
    compare(steps, out, seqs, plain, dtype, "sharp" in name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_changing_size(models, name, dtype, tmp_path):
    if name not in names_for(dtype):
        pytest.skip("peaked attention is compared in 32-bit")
    seqs = {k: v for k, v in sequences(name).items() if len(v) > 3}
    steps = []
    for i, (rid, seq) in enumerate(seqs.items()):
        sizes = [[7, 2, 5, 3, 11, 2], [2, 2, 13, 4, 2, 9], [5, 17, 2, 3, 40], [2]][i % 4]
        steps += trace_portions(rid, seq, sizes, step0=len(steps))
    out, plain = replay(models, name, dtype, steps, tmp_path)
    compare(steps, out, seqs, plain, dtype, "sharp" in name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_batches_with_pages_and_slots_used_again(models, name, dtype, tmp_path):
    if name not in names_for(dtype):
        pytest.skip("peaked attention is compared in 32-bit")
    seqs = sequences(name)
    steps = trace_mixed(seqs, max_live=4, seed=5)
    assert max(len(s["entries"]) for s in steps) >= 3
    peak = peak_tokens(steps)
    assert peak < sum((len(v) + 63) // 64 * 64 for v in seqs.values())
    out, plain = replay(models, name, dtype, steps, tmp_path, max_tokens=peak)
    compare(steps, out, seqs, plain, dtype, "sharp" in name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "Csharp"])
def test_long_decoding(models, name, dtype, tmp_path):
    if dtype == "bfloat16":
        name = name.replace("sharp", "")
    key = name.replace("sharp", "")
    seqs = {"long": random_tokens(230, CASES[key]["vocab"], 3)}
    steps = trace_tail("long", seqs["long"], tail=226)
    out, plain = replay(models, name, dtype, steps, tmp_path)
    compare(steps, out, seqs, plain, dtype, "sharp" in name)


@pytest.mark.parametrize("dtype", DTYPES)
def test_cutting_and_batching_change_logits_by_rounding_only(models, dtype, tmp_path):
    folder, _ = models["C"]
    seqs = sequences("C")
    seq = seqs["r0"]
    runs = []
    mixed = trace_mixed(seqs, max_live=4, seed=9)
    for i, steps in enumerate([trace_whole("r0", seq), trace_portions("r0", seq, [7, 2, 5, 3, 11, 2]),
                               trace_tail("r0", seq, 50), mixed]):
        out = run_trace_inprocess(folder, dtype, steps, str(tmp_path / f"o{i}"), peak_tokens(steps) + 64, 16)
        rows, pos = {}, 0
        for s in steps:
            r = 0
            for e in s["entries"]:
                for w in e["want"]:
                    if e["id"] == "r0":
                        rows[pos + w] = out[s["step"]][r]
                    r += 1
                if e["id"] == "r0":
                    pos += len(e["tokens"])
        runs.append(rows)
    scale = max(np.abs(v).max() for v in runs[0].values())
    tol = 2e-5 if dtype == "float32" else 2e-2
    margins = models["C"][1].margins(seq)
    for other in runs[1:]:
        assert other
        for pos, row in other.items():
            if dtype == "bfloat16" and float(margins[pos]) < ROUTING_MARGIN:
                continue
            assert np.abs(row - runs[0][pos]).max() / scale <= tol, f"position {pos}"


def test_the_stream_after_every_layer(models):
    """In 32-bit the residual stream after each layer equals the plain one closely."""
    from infernum_b200.cache import CacheManager
    from infernum_b200.engine.step import ModelRunner, StepEntry
    from infernum_b200.loading import load_model
    for name in ("A", "B", "C"):
        folder, plain = models[name]
        model = load_model(folder, dtype="float32")
        cache = CacheManager(model.cache_needs(), page_size=4, num_pages=64, max_requests=2,
                             dtype=model.rt.dtype, device=model.rt.device)
        runner = ModelRunner(model, cache, max_rows=256, max_entries=2)
        seen = []
        for blk in model.layers:
            def hooked(stream, ctx, c, orig=blk.forward):
                orig(stream, ctx, c)
                seen.append(stream.residual.clone())
            blk.forward = hooked
        seq = random_tokens(50, CASES[name]["vocab"], 77)
        want = []
        pr.forward(plain.cfg, plain.weights, seq, want)
        runner.step([StepEntry(cache.admit("x"), seq, [])])
        runner.check_errors()
        for i, (got, ref) in enumerate(zip(seen, want)):
            assert rel_err(got, ref) < 2e-5, f"case {name} layer {i}"


def test_a_layer_without_feed_forward_with_and_without_its_second_norm(tmp_path):
    cfg = CASES["A"]
    seq = random_tokens(40, cfg["vocab"], 1)
    for drop in (None, ["l2.norm2", "l2.norm2.b"]):
        folder = make_folder(str(tmp_path / ("full" if drop is None else "bare")), cfg, seed=5, drop=drop)
        plain = pr.Plain(folder)
        assert ("l2.norm2" in plain.weights) == (drop is None)
        steps = trace_whole("r", seq)
        out = run_trace_inprocess(folder, "float32", steps, str(tmp_path / f"o{drop is None}"), 64, 4)
        compare_trace(steps, out, {"r": seq}, plain, TOL["float32"])


def test_the_program_itself_in_a_subprocess(models, tmp_path):
    folder, plain = models["A"]
    seqs = {k: v for k, v in sequences("A").items() if len(v) > 3}
    steps = trace_mixed(seqs, max_live=3, seed=3)
    for dtype in DTYPES:
        out = run_trace_subprocess(folder, dtype, steps, str(tmp_path / dtype), peak_tokens(steps))
        compare(steps, out, seqs, plain, dtype)


# ---- generation through the engine -----------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["Asharp", "Csharp"])
def test_greedy_generation_through_the_engine(models, name, dtype):
    import infernum_b200 as ib
    folder, plain = models[name]
    key = name.replace("sharp", "")
    model = ib.load_model(folder, dtype=dtype)
    engine = ib.Engine(model, ib.BatchConfig(max_batch_size=4, max_prefill_tokens=9, block_size=PAGE_SIZES[key],
                                             num_blocks=96, max_tokens_per_step=24))
    prompts = [random_tokens(n, CASES[key]["vocab"], 3 * n + 1) for n in (1, 6, 19, 44, 12)]
    n_new = 60  # past the windows of the cases
    opts = ib.GenerateOptions(max_new_tokens=n_new)
    got_batch = engine.generate_batch(prompts, opts)
    tie = {"float32": 1e-4, "bfloat16": 5e-2}[dtype]
    for p, got in zip(prompts, got_batch):
        assert len(got) == n_new
        seq = list(p)
        for i, tok in enumerate(got):
            logits = plain.logits(seq)[-1]
            best = int(torch.argmax(logits))
            if tok != best:
                gap = float((logits[best] - logits[tok]) / logits.abs().max())
                routed_close = dtype == "bfloat16" and float(plain.margins(seq)[-80:].min()) < ROUTING_MARGIN
                assert gap < tie or routed_close, f"token {i}: {tok} against {best}, no near-tie ({gap:.4f})"
                break  # beyond a near-tie the two runs are different sequences
            seq.append(tok)
        assert engine.generate(p, opts) == got or dtype == "bfloat16"
    if engine.decoder is not None:
        assert engine.decoder.counts["replayed"] > 0  # the recorded steps were used


def test_command_line_generate(models, tmp_path):
    """``bin/generate`` picks the architecture by config.json: from a model folder, and from
    a bare configuration with random weights."""
    import json
    import subprocess
    import sys

    from helpers import ROOT
    folder, plain = models["Asharp"]
    prompt = [5, 6, 7, 8, 9, 10]
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate"), "-m", folder,
                          ",".join(map(str, prompt)), "-n", "12", "--greedy", "--dtype", "float32", "--block-size", "4"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-3000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("5,6,7,8,9,10")][0]
    got = [int(t) for t in line.split()[1:]]
    seq = list(prompt)
    for tok in got:
        assert tok == int(torch.argmax(plain.logits(seq)[-1]))
        seq.append(tok)
    assert len(got) == 12
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(CASES["B"]))
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate"), "--config", str(cfg_path),
                          "--random-weights", "--weights-seed", "3", "1,2,3", "-n", "4", "--greedy",
                          "--block-size", "8"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-3000:]
    assert "Generated 4 tokens" in out.stdout


# ---- mechanisms alone -------------------------------------------------------------------
def step_context(cache, requests, tokens=None):
    from types import SimpleNamespace

    from infernum_b200.engine.step import ModelRunner, StepEntry
    fake = SimpleNamespace(rt=runtime(torch.float32), spec=SimpleNamespace(vocab_size=1 << 30))
    runner = ModelRunner(fake, cache)
    entries = [StepEntry(rc, tokens[i] if tokens else [0] * n, []) for i, (rc, n) in enumerate(requests)]
    runner.reserve(entries)
    return runner._build(entries)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_hashed_bigram_embedding_carries_the_previous_token_between_steps(dtype):
    from infernum_b200.cache import CacheManager
    from infernum_b200.models.model import CacheNeed
    from infernum_b200.parts import EMBEDDINGS
    from infernum_b200.weights.random_init import random_tensors
    rt = runtime(dtype)
    emb = EMBEDDINGS.get("hashed_bigram_embedding")({
        "vocab_size": 50, "hidden_size": 24, "weight": "embed", "bigram_weight": "bigram", "buckets": 7,
        "mul_prev": 5, "mul_cur": 3}, rt)
    w = random_tensors(emb.weight_specs(), 3, DEV, dtype)
    emb.bind(w)
    cache = CacheManager([CacheNeed(0, None, emb.state_spec(), None)], page_size=4, num_pages=8, max_requests=3,
                         dtype=dtype, device=DEV)
    cfg = {"embedding": {"bigram": {"buckets": 7, "mul_prev": 5, "mul_cur": 3}}}
    plain_w = {k: v.double().cpu() for k, v in w.items()}
    seqs = {"a": random_tokens(23, 50, 1), "b": random_tokens(9, 50, 2)}
    ref = {k: pr.embed(plain_w, cfg, v) for k, v in seqs.items()}
    rcs = {k: cache.admit(k) for k in seqs}
    fed = {"a": 0, "b": 0}
    # portions of unequal size side by side, single tokens among them, a request that sits out
    for plan in ([("a", 5), ("b", 1)], [("b", 2)], [("a", 1), ("b", 1)], [("a", 2), ("b", 5)], [("a", 15)]):
        toks = [seqs[k][fed[k]: fed[k] + n] for k, n in plan]
        ctx = step_context(cache, [(rcs[k], n) for k, n in plan], toks)
        stream = emb.forward_step(ctx, cache.layer_caches[0])
        row = 0
        for (k, n), t in zip(plan, toks):
            assert rel_err(stream.residual[row: row + n], ref[k][fed[k]: fed[k] + n]) < 1e-6
            assert rel_err(stream.act[row: row + n], ref[k][fed[k]: fed[k] + n]) < PART_TOL[dtype]
            row += n
            fed[k] += n
            cache.commit(rcs[k], n)
    # a slot that is used again starts a sequence anew
    cache.release(rcs["b"])
    rc = cache.admit("c")
    ctx = step_context(cache, [(rc, 4)], [seqs["a"][:4]])
    assert rel_err(emb.forward_step(ctx, cache.layer_caches[0]).residual, ref["a"][:4]) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_norm_of_a_scaled_sum(dtype):
    from infernum_b200.parts import NORMS, ResidualStream
    from infernum_b200.weights.random_init import random_tensors
    rt = runtime(dtype)
    for H in (72, 130, 1024):
        norm = NORMS.get("layernorm")({"hidden_size": H, "eps": 3e-6, "weight": "w", "bias": "w.b"}, rt)
        w = random_tensors(norm.weight_specs(), 1, DEV, dtype)
        norm.bind(w)
        x = torch.randn(6, H, device=DEV) * 3 + 1.5
        d = torch.randn(6, H, device=DEV).to(dtype)
        stream = ResidualStream(x.clone())
        stream.push(d)
        norm.renorm(stream, 1.7)
        ref = pr.layer_norm(1.7 * x.double().cpu() + d.double().cpu(), w["w"].double().cpu(), w["w.b"].double().cpu(), 3e-6)
        assert stream.pending is None
        assert rel_err(stream.residual, ref) < 1e-5
        assert rel_err(stream.act, ref) < PART_TOL[dtype]
        rows = torch.tensor([4, 0, 4], dtype=torch.int32, device=DEV)
        before = stream.residual.clone()
        out = norm.forward(stream, row_idx=rows)
        ref2 = pr.layer_norm(before.double().cpu()[[4, 0, 4]], w["w"].double().cpu(), w["w.b"].double().cpu(), 3e-6)
        assert rel_err(out, ref2) < PART_TOL[dtype]
        assert torch.equal(before, stream.residual)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("ff", [40, 192])
def test_gated_gelu_feed_forward(dtype, ff):
    from infernum_b200.parts import FEED_FORWARDS
    from infernum_b200.weights.random_init import random_tensors
    rt = runtime(dtype)
    part = FEED_FORWARDS.get("swiglu")({"hidden_size": 64, "intermediate_size": ff, "prefix": "m.",
                                        "names": {"gate": "gate", "up": "up", "down": "down"},
                                        "activation": "gelu_tanh"}, rt)
    w = {k: (v.float() * 8).to(dtype) for k, v in random_tensors(part.weight_specs(), 2, DEV, dtype).items()}
    part.bind(w)
    for n in (1, 7, 70, 256):
        x = (torch.randn(n, 64, device=DEV) * 2).to(dtype)
        ref = pr.dense_ff({k: v.double().cpu() for k, v in w.items()}, "m.", x.double().cpu())
        assert rel_err(part.forward(x), ref) < PART_TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,ff", [(6, 2, 24), (3, 1, 12), (2, 2, 20), (16, 5, 64)])
def test_mixture_of_experts(dtype, experts, top, ff):
    from infernum_b200.parts import FEED_FORWARDS
    from infernum_b200.weights.random_init import random_tensors
    rt = runtime(dtype)
    part = FEED_FORWARDS.get("moe")({"hidden_size": 48, "expert_size": ff, "experts": experts, "top": top,
                                     "prefix": "m."}, rt)
    w = {k: (v.float() * (8 if ".e" in k else 1)).to(dtype)
         for k, v in random_tensors(part.weight_specs(), 4, DEV, dtype).items()}
    part.bind(w)
    pw = {k: v.double().cpu() for k, v in w.items()}
    x = (torch.randn(37, 48, device=DEV) * 2).to(dtype)
    ids, wts, gate = part.route(x)
    ref_ids, ref_w = pr.route(pw, "m.", x.double().cpu(), top)
    assert torch.equal(ids.cpu().long(), ref_ids)
    assert rel_err(wts, ref_w) < 1e-5
    dense = torch.zeros(37, experts, dtype=torch.float64)
    dense.scatter_(1, ref_ids, ref_w)
    assert rel_err(gate, dense) < 1e-5
    assert rel_err(part.forward(x), pr.moe_ff(pw, "m.", x.double().cpu(), experts, top)) < PART_TOL[dtype]


def test_router_takes_the_lower_index_among_equal_logits():
    from infernum_b200.ops import core
    logits = torch.tensor([[1.0, 3.0, 3.0, 0.5, 3.0], [2.0, 2.0, 2.0, 2.0, 2.0]], device=DEV)
    ids = torch.empty((2, 2), dtype=torch.int32, device=DEV)
    wts = torch.empty((2, 2), dtype=torch.float32, device=DEV)
    core.moe_route(logits, None, 2, ids, wts)
    assert ids.cpu().tolist() == [[1, 2], [0, 1]]
    assert torch.allclose(wts.cpu(), torch.full((2, 2), 0.5))


def test_soft_capped_head():
    from infernum_b200.parts import HEADS
    rt = runtime(torch.float32)
    head = HEADS.get("linear_head")({"vocab_size": 33, "hidden_size": 16, "weight": "head", "softcap": 2.5}, rt)
    w = torch.randn(33, 16, device=DEV)
    head.bind({"head": w})
    x = torch.randn(5, 16, device=DEV) * 3
    ref = pr.softcap(x.double().cpu() @ w.double().cpu().T, 2.5)
    assert rel_err(head.forward(x), ref) < 1e-5


# ---- the attention kernels over a latent cache, with keys made to stand out ---------------
def latent_case(dtype, heads, kv_rank, rot_dim, page_size, lengths, new_rows, window, needles, seed=0,
                options=None):
    """Entries with ``lengths[e]`` cached-or-new tokens, the last ``new_rows[e]`` of
    them queries of this step.  ``needles``: (entry, query position, key position)
    triples: that key is made to dominate that query's scores in every head."""
    from infernum_b200.engine.step import StepContext
    from infernum_b200.ops import attention as attn_ops
    g = torch.Generator().manual_seed(seed)
    W = kv_rank + rot_dim
    E = len(lengths)
    pages_each = [-(-n // page_size) for n in lengths]
    num_pages = sum(pages_each) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    MB = max(pages_each)
    tables = torch.full((E, MB), -1, dtype=torch.int32)
    latents = [torch.randn(n, W, generator=g, dtype=torch.float64) * 0.5 for n in lengths]
    rows_e, rows_p = [], []
    for e, n in enumerate(lengths):
        for p in range(n - new_rows[e], n):
            rows_e.append(e)
            rows_p.append(p)
    N = len(rows_e)
    q = torch.randn(N, heads, W, generator=g, dtype=torch.float64) * 0.5
    for (e, qp, kp) in needles:
        r = next(i for i in range(N) if rows_e[i] == e and rows_p[i] == qp)
        direction = torch.randn(W, generator=g, dtype=torch.float64)
        direction /= direction.norm()
        latents[e][kp] = direction * 6.0
        q[r] = direction[None, :] * 10.0 + q[r] * 0.1
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    pool = torch.zeros(num_pages, 1, page_size, W, dtype=tdt)
    pool[:] = float("nan") if dtype == "float32" else 0  # pages nobody owns must not be read
    at = 0
    for e, n in enumerate(lengths):
        for b in range(pages_each[e]):
            page = perm[at]
            at += 1
            tables[e, b] = page
            chunk = latents[e][b * page_size: (b + 1) * page_size]
            pool[page, 0, : chunk.shape[0]] = chunk.to(tdt)
            pool[page, 0, chunk.shape[0]:] = 0
    # what the kernels see, rounded as they see it
    lat_r = [pool[tables[e, : pages_each[e]].long(), 0].reshape(-1, W)[:n].double() for e, n in enumerate(lengths)]
    q_r = q.to(tdt)
    scale = 0.37
    ref = torch.zeros(N, heads, kv_rank, dtype=torch.float64)
    for i in range(N):
        e, p = rows_e[i], rows_p[i]
        lo = max(0, p - window + 1) if window else 0
        keys = lat_r[e][lo: p + 1]
        for h in range(heads):
            s = (keys @ q_r[i, h].double()) * scale
            ref[i, h] = torch.softmax(s, 0) @ keys[:, :kv_rank]
    cu = [0]
    for e in range(E):
        cu.append(cu[-1] + new_rows[e])
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
    ctx = StepContext(n_rows=N, n_entries=E, token_ids=i32([0] * N), positions=i32(rows_p), row_entry=i32(rows_e),
                      cu_rows=i32(cu), q_start=i32([lengths[e] - new_rows[e] for e in range(E)]),
                      kv_len=i32(lengths), slot_ids=i32(list(range(E))), logit_rows=None,
                      block_tables=[tables.to(DEV)], host_cu_rows=cu, host_kv_len=list(lengths),
                      max_rows_per_entry=max(new_rows), max_kv_len=max(lengths), all_decode=(N == E))
    rt = runtime(tdt, **(options or {}))
    out = torch.full((N, heads, kv_rank), float("nan"), dtype=tdt, device=DEV)
    attn_ops.latent_attention(q_r.to(DEV), pool.to(DEV), out, kv_rank, ctx, ctx.block_tables[0], scale, window, rt)
    torch.cuda.synchronize()
    assert int(rt.err.item()) == 0
    return out, ref, rows_e, rows_p


# the plain kernel in both dtypes; the tensor-core kernel as its plan comes out, and with the
# plans forced that the small cases would not choose: one, two or four row tiles per CTA, keys of a
# row tile shared out over 3 or 7 CTAs
KERNELS = [("float32", None), ("bfloat16", {"attention": "plain"}), ("bfloat16", None),
           ("bfloat16", {"latent_plan": (1, 3)}), ("bfloat16", {"latent_plan": (2, 7)}),
           ("bfloat16", {"latent_plan": (2, 1)}), ("bfloat16", {"latent_plan": (4, 1)}),
           ("bfloat16", {"latent_plan": (4, 2)})]


@pytest.mark.parametrize("dtype,options", KERNELS)
@pytest.mark.parametrize("heads,kv_rank,rot_dim,page", [(3, 40, 8, 4), (8, 64, 16, 16), (1, 20, 4, 8),
                                                         (16, 128, 64, 16), (5, 96, 32, 32), (2, 32, 16, 8),
                                                         (4, 64, 48, 16)])
def test_keys_just_inside_and_outside_the_window_in_prompts_and_decoding(dtype, options, heads, kv_rank,
                                                                         rot_dim, page):
    window = 37
    tol = 1e-5 if dtype == "float32" else 2e-2
    # decoding: one query per entry; its needle sits on the window's first key, or one before it
    lengths = [200, 93, 37, 38, 5, 1]
    for shift, visible in ((window - 1, True), (window, False)):
        needles = [(e, n - 1, n - 1 - shift) for e, n in enumerate(lengths) if n - 1 - shift >= 0]
        out, ref, rows_e, rows_p = latent_case(dtype, heads, kv_rank, rot_dim, page, lengths, [1] * len(lengths),
                                               window, needles, seed=shift, options=options)
        assert rel_err(out, ref) < tol
        for (e, qp, kp) in needles:
            i = next(k for k in range(len(rows_e)) if rows_e[k] == e)
            # the needle's latent has norm 6: seen, the output is close to it; unseen, far from it
            assert (ref[i].norm(dim=-1) > 3.0).all() == visible or kv_rank < 24
    # prompts: portions behind a cached prefix; needles at the edge for queries early and late in the portion
    lengths, new = [150, 64, 90], [70, 64, 3]
    needles = [(0, 149, 149 - 36), (0, 100, 100 - 37), (0, 81, 81 - 36), (1, 63, 27), (1, 40, 3), (2, 88, 52)]
    out, ref, _, _ = latent_case(dtype, heads, kv_rank, rot_dim, page, lengths, new, window, needles, seed=5,
                                 options=options)
    assert rel_err(out, ref) < tol


@pytest.mark.parametrize("dtype,options", KERNELS)
@pytest.mark.parametrize("page", [4, 16])
def test_keys_far_away_at_page_borders_and_the_first_tokens(dtype, options, page):
    tol = 1e-5 if dtype == "float32" else 2e-2
    heads, kv_rank, rot_dim = 4, 48, 16
    # no window: a key hundreds of tokens back, the very first keys, keys on both sides of page borders
    lengths, new = [700, 333, 64, 2], [1, 40, 64, 2]
    needles = [(0, 699, 3), (1, 332, 0), (1, 300, page - 1), (1, 310, page), (1, 320, 20 * page - 1),
               (1, 325, 20 * page), (2, 63, 1), (2, 17, 16), (2, 16, 15), (3, 1, 0)]
    out, ref, _, _ = latent_case(dtype, heads, kv_rank, rot_dim, page, lengths, new, 0, needles, options=options)
    assert rel_err(out, ref) < tol
    # a wide window whose edge lies hundreds of tokens back
    out, ref, _, _ = latent_case(dtype, heads, kv_rank, rot_dim, page, [900, 600], [1, 30], 512,
                                 [(0, 899, 899 - 511), (1, 599, 599 - 512), (1, 580, 580 - 511)], options=options)
    assert rel_err(out, ref) < tol
