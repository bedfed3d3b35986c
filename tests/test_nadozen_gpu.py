"""The Nadozen decoder on the GPU against the plain implementation
(``plain_nadozen``): each mechanism alone; whole prompts, token-by-token decoding,
portions down to two tokens, mixed batches with pages and state slots used again,
long decoding past every window; keys at window and page edges and far away, made
to stand out, with a sink in the denominator; sizes that are 1 or equal; layers
that run with another layer's tensors; greedy generation through the engine."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_nadozen as pn
from helpers import (ROOT, TOL, compare_trace, peak_tokens, random_tokens, run_trace_inprocess,
                     run_trace_subprocess, trace_mixed, trace_portions, trace_tail, trace_whole)
from nadozen_cases import CASES, PAGE_SIZES, make_folder

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = ["float32", "bfloat16"]
LENGTHS = {"A": [31, 45, 1, 2, 90, 17], "B": [23, 60, 3, 1, 41, 8], "C": [130, 75, 2, 200, 33, 64],
           "D": [50, 3, 27, 1, 12]}
NAMES = ["A", "B", "C", "D", "Asharp", "Csharp"]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CASES.items()):
        folder = make_folder(str(tmp_path_factory.mktemp(f"ndz{name}")), cfg, seed=17 + i)
        out[name] = (folder, pn.Plain(folder))
        if name in ("A", "C"):
            sharp = make_folder(str(tmp_path_factory.mktemp(f"ndzsharp{name}")), cfg, seed=41 + i, sharpen=5.0)
            out[name + "sharp"] = (sharp, pn.Plain(sharp))
    return out


def sequences(name):
    key = name.replace("sharp", "")
    return {f"r{i}": random_tokens(n, CASES[key]["vocab"], 100 * i + n) for i, n in enumerate(LENGTHS[key])}


def replay(models, name, dtype, steps, tmp_path, max_tokens=None):
    folder, plain = models[name]
    out = run_trace_inprocess(folder, dtype, steps, str(tmp_path / "out"), max_tokens or peak_tokens(steps),
                              PAGE_SIZES[name.replace("sharp", "")])
    return out, plain


def names_for(dtype):
    # (where attention is peaked, bfloat16 rounding of a score is multiplied on its way to the logits)
    return NAMES if dtype == "float32" else ["A", "B", "C", "D"]


def tolerance(dtype, name):
    return TOL[dtype] * (3 if "sharp" in name else 1)


def compare(steps, out, seqs, plain, dtype, name, slack=1):
    """float32: every position within the tolerance.  bfloat16: a unit norm of a nearly
    cancelling sum (a wkv head's output at a sequence's first token is its value vector times
    the sign of one scalar; a softmax over one key and a sink) multiplies the rounding of what
    it norms, so single positions may lie far off while the run is right: at most one position
    in ten beyond the tolerance, the median at most half of it, every value finite."""
    if dtype == "float32":
        return compare_trace(steps, out, seqs, plain, tolerance(dtype, name) * slack)
    fed = {rid: 0 for rid in seqs}
    errs = []
    for s in steps:
        row = 0
        for e in s["entries"]:
            rid, n = e["id"], len(e["tokens"])
            ref_all = plain.logits(seqs[rid])
            for w in e.get("want", []):
                got, ref = out[s["step"]][row], ref_all[fed[rid] + w].numpy()
                row += 1
                assert np.isfinite(got).all()
                errs.append(float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-6)))
            fed[rid] += n
        for rid in s.get("end", []):
            fed[rid] = 0
    errs = np.sort(np.array(errs))
    tol = TOL[dtype] * slack
    over = int((errs > tol).sum())
    summary = f"{len(errs)} positions, median {np.median(errs):.3e}, worst {errs[-1]:.3e}, {over} beyond {tol:.1e}"
    assert over <= max(1, len(errs) // 10), summary
    assert np.median(errs) <= tol / 2, summary
    return summary


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
    compare(steps, out, seqs, plain, dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_most_in_one_step_then_token_by_token_past_the_windows(models, name, dtype, tmp_path):
    if name not in names_for(dtype):
        pytest.skip("peaked attention is compared in 32-bit")
    seqs = {k: v for k, v in sequences(name).items() if len(v) > 3}
    steps = []
    for rid, seq in seqs.items():
        steps += trace_tail(rid, seq, 80, step0=len(steps))  # longer than every window of the cases but one
    out, plain = replay(models, name, dtype, steps, tmp_path)
    compare(steps, out, seqs, plain, dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_changing_size(models, name, dtype, tmp_path):
    if name not in names_for(dtype):
        pytest.skip("peaked attention is compared in 32-bit")
    seqs = {k: v for k, v in sequences(name).items() if len(v) > 3}
    steps = []
    for i, (rid, seq) in enumerate(seqs.items()):
        sizes = [[2, 3, 7, 2, 16, 5], [13, 2, 2, 1, 30], [1, 2, 4, 8, 16, 32]][i % 3]
        steps += trace_portions(rid, seq, sizes, step0=len(steps))
    out, plain = replay(models, name, dtype, steps, tmp_path)
    compare(steps, out, seqs, plain, dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_batches_with_pages_and_slots_used_again(models, name, dtype, tmp_path):
    if name not in names_for(dtype):
        pytest.skip("peaked attention is compared in 32-bit")
    seqs = sequences(name)
    seqs.update({k + "again": v[::-1] for k, v in list(seqs.items())[:3]})  # more requests than slots
    steps = trace_mixed(seqs, max_live=4, seed=len(name) + 3)
    out, plain = replay(models, name, dtype, steps, tmp_path)
    compare(steps, out, seqs, plain, dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding(models, name, dtype, tmp_path):
    seq = random_tokens(260, CASES[name]["vocab"], 9)
    steps = trace_tail("long", seq, 250)
    out, plain = replay(models, name, dtype, steps, tmp_path)
    compare(steps, out, {"long": seq}, plain, dtype, name, slack=2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_cutting_and_batching_change_logits_by_rounding_only(models, dtype, tmp_path):
    """The same positions whole, cut in portions, and inside a mixed batch."""
    folder, _ = models["C"]
    seqs = {k: v for k, v in sequences("C").items() if len(v) > 40}
    runs = {}
    for label, steps in (("whole", sum((trace_whole(r, s) for r, s in seqs.items()), [])),
                         ("cut", sum((trace_portions(r, s, [3, 2, 29, 1, 17]) for r, s in seqs.items()), [])),
                         ("mixed", trace_mixed(seqs, 4, 5, decode_tail=20))):
        for i, s in enumerate(steps):
            s["step"] = i
            for e in s["entries"]:
                e["want"] = list(range(len(e["tokens"])))
        out = run_trace_inprocess(folder, dtype, steps, str(tmp_path / label), peak_tokens(steps), 16)
        rows = {r: [] for r in seqs}
        for s in steps:
            at = 0
            for e in s["entries"]:
                rows[e["id"]].append(out[s["step"]][at: at + len(e["tokens"])])
                at += len(e["tokens"])
        runs[label] = {r: np.concatenate(v) for r, v in rows.items()}
    tol = 2e-5 if dtype == "float32" else 4e-2
    for r in seqs:
        scale = np.abs(runs["whole"][r]).max()
        for label in ("cut", "mixed"):
            assert runs[label][r].shape == runs["whole"][r].shape
            assert np.abs(runs[label][r] - runs["whole"][r]).max() / scale < tol, (r, label)


def test_the_streams_after_every_layer(models):
    """The sum of the streams after every layer run, layers that share tensors included."""
    import infernum_b200 as ib
    from infernum_b200.cache import CacheManager
    from infernum_b200.engine.step import ModelRunner, StepEntry
    from infernum_b200.ops import core
    folder, plain = models["A"]
    seq = random_tokens(37, CASES["A"]["vocab"], 3)
    ref = []
    pn.forward(plain.cfg, plain.weights, seq, streams_out=ref)
    model = ib.load_model(folder, dtype="float32")
    cache = CacheManager(model.cache_needs(), page_size=4, num_pages=16, max_requests=2, dtype=model.rt.dtype,
                         device=DEV)
    runner = ModelRunner(model, cache)
    rc = cache.admit("x")
    runner.reserve([StepEntry(rc, seq, [])])
    ctx = runner._build([StepEntry(rc, seq, [])])
    with core.step_stream(DEV):
        stream = model.embedding.forward_step(ctx, None)
        for k, (item, lc) in enumerate(zip(model.schedule, cache.layer_caches)):
            model.layers[item.layer].forward(stream, ctx, lc)
            stream.flush()
            got = stream.residual.sum(dim=1)
            assert rel_err(got, ref[k]) < 1e-5, f"after layer run {k}"


def test_the_program_itself_in_a_subprocess(models, tmp_path):
    folder, plain = models["D"]
    seqs = sequences("D")
    steps = trace_mixed(seqs, max_live=4, seed=2)
    out = run_trace_subprocess(folder, "float32", steps, str(tmp_path / "o"), peak_tokens(steps))
    compare_trace(steps, out, seqs, plain, TOL["float32"])


# ---- generation through the engine -------------------------------------------------
def check_greedy(plain, prompt, got, dtype):
    """Every generated token is the plain implementation's best, or within rounding of it;
    after a near-tie the two may part, so the comparison follows what was generated."""
    seq = list(prompt)
    for i, tok in enumerate(got):
        logits = plain.logits(seq)[-1]
        best = pn.argmax(logits)
        if tok != best:
            gap = float((logits[best] - logits[tok]) / logits.abs().max())
            assert gap < (1e-4 if dtype == "float32" else 5e-2), f"token {i}: {tok} against {best}, gap {gap:.4f}"
        seq.append(tok)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_greedy_generation_through_the_engine(models, name, dtype):
    import infernum_b200 as ib
    folder, plain = models[name]
    model = ib.load_model(folder, dtype=dtype)
    page = PAGE_SIZES[name]
    engine = ib.Engine(model, ib.BatchConfig(max_batch_size=3, block_size=page, num_blocks=400 // page,
                                             max_prefill_tokens=24))
    vocab = CASES[name]["vocab"]
    prompts = [random_tokens(n, vocab, 7 * n) for n in (5, 41, 18, 2, 30)]
    outs = engine.generate_batch(prompts, ib.GenerateOptions(max_new_tokens=24))
    for prompt, got in zip(prompts, outs):
        assert len(got) == 24
        check_greedy(plain, prompt, got, dtype)
    # recurring steps ran from recordings: the mixers take entries, slots and positions from the device
    assert model.replayable
    # once more on the same engine: slots and pages that were used before
    again = engine.generate_batch(prompts[:2], ib.GenerateOptions(max_new_tokens=8))
    for prompt, got in zip(prompts[:2], again):
        check_greedy(plain, prompt, got, dtype)


def test_generation_with_too_few_pages_preempts_and_recomputes(models):
    import infernum_b200 as ib
    folder, plain = models["A"]
    model = ib.load_model(folder, dtype="float32")
    engine = ib.Engine(model, ib.BatchConfig(max_batch_size=4, block_size=4, num_blocks=30, max_prefill_tokens=16))
    prompts = [random_tokens(n, CASES["A"]["vocab"], 11 * n) for n in (20, 33, 25, 14)]
    outs = engine.generate_batch(prompts, ib.GenerateOptions(max_new_tokens=30))
    for prompt, got in zip(prompts, outs):
        check_greedy(plain, prompt, got, "float32")


def test_command_line_generate(models, tmp_path):
    """``bin/generate`` picks the architecture by config.json: from a model folder, and from
    a bare configuration with random weights."""
    import json
    folder, plain = models["D"]
    prompt = random_tokens(9, CASES["D"]["vocab"], 1)
    text = ",".join(map(str, prompt))
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate"), "-m", folder, text, "-n", "6",
                           "--greedy", "--dtype", "float32", "--block-size", "4"],
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    line = [l for l in proc.stdout.splitlines() if l.startswith(text)][0]
    got = [int(t) for t in line.split()[1:]]
    assert len(got) == 6
    check_greedy(plain, prompt, got, "float32")
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(CASES["B"]))
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate"), "--config", str(cfg_path),
                           "--random-weights", "--weights-seed", "3", "1,2,3", "-n", "4", "--greedy",
                           "--block-size", "8"], capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert "Generated 4 tokens" in proc.stdout


# ---- mechanisms alone ------------------------------------------------------------------
class Step:
    """The device tensors of a step that the recurrent kernels read."""

    def __init__(self, rows_per_entry, slots):
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
        cu = [0]
        for n in rows_per_entry:
            cu.append(cu[-1] + n)
        self.n_entries = len(rows_per_entry)
        self.n_rows = cu[-1]
        self.cu_rows = i32(cu)
        self.slot_ids = i32(slots)
        self.row_entry = i32([e for e, n in enumerate(rows_per_entry) for _ in range(n)])


def cuts_of(T, sizes):
    out, at, i = [], 0, 0
    while at < T:
        n = min(sizes[i % len(sizes)], T - at)
        out.append((at, n))
        at += n
        i += 1
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S,H", [(4, 96), (1, 40), (3, 1000), (8, 64), (2, 90), (5, 7)])
def test_streams_write_read_and_norm_in_one_pass(dtype, S, H):
    from infernum_b200.ops import core
    g = torch.Generator().manual_seed(S * H)
    N = 19
    x = torch.randn(N, S, H, generator=g, dtype=torch.float64)
    y = torch.randn(N, H, generator=g, dtype=torch.float64).to(dtype)
    mix = torch.randn(S, S, generator=g, dtype=torch.float64).float()
    oc = torch.randn(S, generator=g, dtype=torch.float64).float()
    rd = torch.randn(S, generator=g, dtype=torch.float64).float()
    w = (1 + 0.1 * torch.randn(H, generator=g, dtype=torch.float64)).to(dtype)
    b = (0.1 * torch.randn(H, generator=g, dtype=torch.float64)).to(dtype)
    xs = [x[:, s].float().double() for s in range(S)]
    new = pn.hyper_write(xs, mix.double(), oc.double(), y.double())
    ref = pn.layer_norm(pn.hyper_read(new, rd.double()), w.double(), b.double(), 1e-5)
    xd = x.float().to(DEV)
    out = torch.empty(N, H, dtype=dtype, device=DEV)
    core.hc_norm(xd, y.to(DEV), mix.to(DEV).view(-1), oc.to(DEV), rd.to(DEV), w.to(DEV), b.to(DEV), 1e-5, out)
    assert rel_err(out, ref) < PART_TOL[dtype]
    assert rel_err(xd, torch.stack(new, dim=1)) < 1e-6
    # a row gather reads the sum of the streams after the pending write and writes nothing back
    rows = torch.tensor([3, 18, 0], dtype=torch.int32, device=DEV)
    xd2 = x.float().to(DEV)
    out2 = torch.empty(3, H, dtype=dtype, device=DEV)
    core.hc_norm(xd2, y.to(DEV), mix.to(DEV).view(-1), oc.to(DEV), None, w.to(DEV), b.to(DEV), 1e-5, out2, row_idx=rows)
    ref2 = pn.layer_norm(sum(new), w.double(), b.double(), 1e-5)[rows.cpu().long()]
    assert rel_err(out2, ref2) < PART_TOL[dtype]
    assert torch.equal(xd2.cpu(), x.float())


@pytest.mark.parametrize("D", [64, 90, 7])
def test_sinusoidal_embedding_at_small_and_large_positions(D):
    from infernum_b200.parts import EMBEDDINGS
    rt = runtime(torch.float32)
    part = EMBEDDINGS.get("sinusoidal_embedding")({"vocab_size": 11, "hidden_size": D, "weight": "e", "streams": 2}, rt)
    table = torch.randn(11, D, generator=torch.Generator().manual_seed(D)).to(DEV)
    part.bind({"e": table})
    positions = [0, 1, 2, 63, 64, 1000, 4097]
    ids = [3, 0, 10, 5, 5, 1, 7]

    class Ctx:
        token_ids = torch.tensor(ids, dtype=torch.int32, device=DEV)
    Ctx.positions = torch.tensor(positions, dtype=torch.int32, device=DEV)
    stream = part.forward_step(Ctx, None)
    assert stream.residual.shape == (7, 2, D)
    for i, (p, t) in enumerate(zip(positions, ids)):
        ref = table[t].double().cpu() + pn.position_vectors(1, D, start=p)[0]
        # (the angle is a 32-bit product: its rounding grows with the position)
        assert (stream.residual[i, 0].double().cpu() - ref).abs().max() < 2e-6 + 1.5e-7 * p
        assert torch.equal(stream.residual[i, 0], stream.residual[i, 1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_shift_carries_the_last_row_between_steps(dtype):
    from infernum_b200.ops import core
    g = torch.Generator().manual_seed(1)
    D, M, T = 40, 5, 23
    h = {r: torch.randn(T, D, generator=g, dtype=torch.float64).to(dtype) for r in ("a", "b")}
    mu = torch.rand(M, D, generator=g, dtype=torch.float64).float()
    state = torch.full((3, 7 + D), 5.0, dtype=torch.float32, device=DEV)
    state[:2, 7:] = 0  # slots as admission leaves them; slot 2 and the first 7 floats belong to others
    got = {r: [] for r in h}
    plan = {"a": cuts_of(T, [1, 2, 7, 1, 1, 30]), "b": cuts_of(T, [5, 1, 1, 16, 2])}
    while any(plan.values()):
        live = [r for r in h if plan[r]]
        cuts = [plan[r].pop(0) for r in live]
        x = torch.cat([h[r][at: at + n] for r, (at, n) in zip(live, cuts)]).to(DEV)
        step = Step([n for _, n in cuts], [0 if r == "a" else 1 for r in live])
        out = torch.empty(M, x.shape[0], D, dtype=dtype, device=DEV)
        core.token_shift(x, mu.to(DEV), state, 7, step, out)
        at = 0
        for r, (_, n) in zip(live, cuts):
            got[r].append(out[:, at: at + n].cpu())
            at += n
    for r in h:
        ref = torch.stack([pn.token_shift(h[r].double(), mu[m].double()) for m in range(M)])
        assert rel_err(torch.cat(got[r], dim=1), ref) < PART_TOL[dtype]
    assert (state[2] == 5).all() and (state[:, :7] == 5).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,K", [(2, 16), (1, 28), (3, 64), (2, 10), (1, 128)])
def test_wkv_scan_in_portions_and_batches_against_the_recurrence(dtype, heads, K):
    from infernum_b200.ops import scan
    g = torch.Generator().manual_seed(heads * K)
    T = {"a": 41, "b": 18}
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)  # noqa: E731
    data = {r: {"r": rnd(n, heads * K).to(dtype), "k": (rnd(n, heads * K) * 0.5).to(dtype),
                "v": rnd(n, heads * K).to(dtype), "z": (rnd(n, heads * K) - 1.0).float()} for r, n in T.items()}
    w0 = (rnd(heads * K) * 0.5).float()
    u = rnd(heads * K).float()
    ref = {}
    for r, d in data.items():
        outs = []
        for a in range(heads):
            sl = slice(a * K, (a + 1) * K)
            decay = torch.exp(-torch.exp(d["z"][:, sl].double() + w0[sl].double()))
            o, _ = pn.wkv_recurrence(d["r"][:, sl].double(), d["k"][:, sl].double(), d["v"][:, sl].double(), decay,
                                     u[sl].double())
            outs.append(o)
        ref[r] = torch.cat(outs, dim=-1)
    rt = runtime(dtype)
    state = torch.zeros(3, 5 + heads * K * K + 9, dtype=torch.float32, device=DEV)
    plan = {"a": cuts_of(T["a"], [1, 2, 17, 1, 3, 40]), "b": cuts_of(T["b"], [4, 1, 1, 20])}
    got = {r: [] for r in T}
    while any(plan.values()):
        live = [r for r in T if plan[r]]
        cuts = [plan[r].pop(0) for r in live]
        cat = lambda key: torch.cat([data[r][key][at: at + n] for r, (at, n) in zip(live, cuts)]).to(DEV)  # noqa: E731
        step = Step([n for _, n in cuts], [2 if r == "a" else 0 for r in live])
        out = torch.empty(step.n_rows, heads * K, dtype=torch.float32, device=DEV)
        scan.wkv_scan(cat("r"), cat("k"), cat("v"), cat("z"), w0.to(DEV), u.to(DEV), state, 5, step, out, heads, rt)
        at = 0
        for r, (_, n) in zip(live, cuts):
            got[r].append(out[at: at + n].cpu())
            at += n
    for r in T:
        assert rel_err(torch.cat(got[r]), ref[r]) < 2e-5
    assert (state[1] == 0).all() and (state[:, :5] == 0).all() and (state[:, 5 + heads * K * K:] == 0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,groups,N,P,taps", [(4, 2, 20, 12, 0), (1, 1, 10, 20, 1), (3, 3, 14, 6, 2),
                                                    (2, 1, 128, 24, 4), (8, 2, 64, 32, 0), (2, 2, 16, 8, 7)])
def test_ssd_scan_in_portions_and_batches_against_the_recurrence(dtype, heads, groups, N, P, taps):
    """``taps`` > 0: x, B and C first pass the causal convolution and SiLU, whose last inputs are
    carried in the state across portions shorter than the convolution."""
    from infernum_b200.ops import scan
    g = torch.Generator().manual_seed(heads * N + P)
    T = {"a": 37, "b": 21}
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)  # noqa: E731
    inner = heads * P
    data = {r: {"xbc": rnd(n, inner + 2 * groups * N).to(dtype), "dt": rnd(n, heads + 3).to(dtype)}
            for r, n in T.items()}
    dt_bias, a_log, d_skip = rnd(heads).float(), (rnd(heads) * 0.5).float(), rnd(heads).float()
    channels = inner + 2 * groups * N
    conv_w, conv_b = (rnd(channels, taps) * 0.5).float(), rnd(channels).float()
    ref = {}
    for r, d in data.items():
        xbc = d["xbc"].double()
        if taps:
            xbc = pn.silu(pn.causal_conv(xbc, conv_w.double(), conv_b.double()))
        x = xbc[:, :inner].view(-1, heads, P)
        B = xbc[:, inner: inner + groups * N].view(-1, groups, N)
        C = xbc[:, inner + groups * N:].view(-1, groups, N)
        dt = pn.softplus(d["dt"][:, 1: 1 + heads].double() + dt_bias.double())
        outs = []
        for a in range(heads):
            gi = a // (heads // groups)
            y, _ = pn.ssd_recurrence(x[:, a], B[:, gi], C[:, gi], dt[:, a], a_log[a].double(), d_skip[a].double())
            outs.append(y)
        ref[r] = torch.cat(outs, dim=-1)
    rt = runtime(dtype)
    off_conv = heads * N * P + 4
    state = torch.zeros(3, off_conv + max(taps - 1, 0) * channels + 3, dtype=torch.float32, device=DEV)
    conv = (conv_w.to(DEV), conv_b.to(DEV), off_conv) if taps else None
    plan = {"a": cuts_of(T["a"], [2, 1, 16, 1, 3, 40]), "b": cuts_of(T["b"], [1, 1, 7, 20])}
    got = {r: [] for r in T}
    while any(plan.values()):
        live = [r for r in T if plan[r]]
        cuts = [plan[r].pop(0) for r in live]
        cat = lambda key: torch.cat([data[r][key][at: at + n] for r, (at, n) in zip(live, cuts)]).to(DEV)  # noqa: E731
        step = Step([n for _, n in cuts], [1 if r == "a" else 2 for r in live])
        out = torch.empty(step.n_rows, inner, dtype=torch.float32, device=DEV)
        scan.ssd_scan(cat("xbc"), cat("dt")[:, 1: 1 + heads], dt_bias.to(DEV), a_log.to(DEV), d_skip.to(DEV), state, 0,
                      step, out, heads, groups, N, P, rt, conv=conv)
        at = 0
        for r, (_, n) in zip(live, cuts):
            got[r].append(out[at: at + n].cpu())
            at += n
    for r in T:
        assert rel_err(torch.cat(got[r]), ref[r]) < 2e-5
    # the slot nobody had, the floats between the matrices and the convolution's inputs, and those behind them
    assert (state[0] == 0).all() and (state[:, heads * N * P: off_conv] == 0).all() and (state[:, -3:] == 0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norms_behind_the_scans(dtype):
    from infernum_b200.ops import core
    g = torch.Generator().manual_seed(4)
    N, heads, K = 9, 3, 20
    o = torch.randn(N, heads * K, generator=g)
    gate = torch.randn(N, heads * K + 5, generator=g).to(dtype)
    w = torch.randn(heads * K, generator=g)
    out = torch.empty(N, heads * K, dtype=dtype, device=DEV)
    core.head_norm_gate(o.to(DEV), gate.to(DEV)[:, 2: 2 + heads * K], w.to(DEV), heads, 1e-5, out)
    ref = pn.unit_rms(o.double().view(N, heads, K), 1e-5).reshape(N, -1) * w.double() * \
        pn.silu(gate[:, 2: 2 + heads * K].double())
    assert rel_err(out, ref) < PART_TOL[dtype]
    for parts in (1, 3, 4):
        inner = 60
        y = torch.randn(N, inner, generator=g)
        z = torch.randn(N, inner + 4, generator=g).to(dtype)
        wn = torch.randn(inner, generator=g)
        out = torch.empty(N, inner, dtype=dtype, device=DEV)
        core.gated_group_norm(y.to(DEV), z.to(DEV)[:, 4:], wn.to(DEV), parts, 1e-5, out)
        v = y.double() * pn.silu(z[:, 4:].double())
        ref = pn.unit_rms(v.view(N, parts, inner // parts), 1e-5).reshape(N, inner) * wn.double()
        assert rel_err(out, ref) < PART_TOL[dtype]


# ---- attention with normed keys, values that are the keys, a window and a sink ---------------
def attention_case(dtype, heads, kv_heads, hd, page_size, lengths, new_rows, window, needles, sinks, seed=0,
                   options=None):
    """Entries with ``lengths[e]`` cached-or-new tokens, the last ``new_rows[e]`` of them
    queries of this step.  ``needles``: (entry, query position, key position): that key
    is made to dominate that query's scores in every head."""
    from infernum_b200.engine.step import StepContext
    from infernum_b200.ops import attention as attn_ops
    g = torch.Generator().manual_seed(seed)
    E = len(lengths)
    pages_each = [-(-n // page_size) for n in lengths]
    num_pages = sum(pages_each) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    MB = max(pages_each)
    tables = torch.full((E, MB), -1, dtype=torch.int32)
    keys = [torch.randn(n, kv_heads, hd, generator=g, dtype=torch.float64) * 0.4 for n in lengths]
    vals = [torch.randn(n, kv_heads, hd, generator=g, dtype=torch.float64) for n in lengths]
    rows_e, rows_p = [], []
    for e, n in enumerate(lengths):
        for p in range(n - new_rows[e], n):
            rows_e.append(e)
            rows_p.append(p)
    N = len(rows_e)
    q = torch.randn(N, heads, hd, generator=g, dtype=torch.float64) * 0.4
    for (e, qp, kp) in needles:
        r = next(i for i in range(N) if rows_e[i] == e and rows_p[i] == qp)
        direction = torch.randn(hd, generator=g, dtype=torch.float64)
        direction /= direction.norm()
        keys[e][kp] = direction[None, :] * 6.0
        vals[e][kp] = vals[e][kp] + 20.0  # a seen needle lifts the output by about 20
        q[r] = direction[None, :] * 10.0 + q[r] * 0.1
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    k_pool = torch.zeros(num_pages, kv_heads, page_size, hd, dtype=tdt)
    v_pool = torch.zeros(num_pages, kv_heads, page_size, hd, dtype=tdt)
    at = 0
    for e, n in enumerate(lengths):
        for b in range(pages_each[e]):
            page = perm[at]
            at += 1
            tables[e, b] = page
            kc = keys[e][b * page_size: (b + 1) * page_size]
            k_pool[page, :, : kc.shape[0]] = kc.transpose(0, 1).to(tdt)
            v_pool[page, :, : kc.shape[0]] = vals[e][b * page_size: (b + 1) * page_size].transpose(0, 1).to(tdt)
    q_r = q.to(tdt)
    scale = 0.31
    G = heads // kv_heads
    ref = torch.zeros(N, heads, hd, dtype=torch.float64)
    for i in range(N):
        e, p = rows_e[i], rows_p[i]
        lo = max(0, p - window + 1) if window else 0
        for h in range(heads):
            kk = keys[e][lo: p + 1, h // G].to(tdt).double()
            vv = vals[e][lo: p + 1, h // G].to(tdt).double()
            s = (kk @ q_r[i, h].double()) * scale
            top = max(float(s.max()), float(sinks[h]))
            ex = torch.exp(s - top)
            ref[i, h] = (ex / (ex.sum() + np.exp(float(sinks[h]) - top))) @ vv
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
    out = torch.full((N, heads * hd), float("nan"), dtype=tdt, device=DEV)
    attn_ops.paged_attention(q_r.reshape(N, heads * hd).to(DEV), k_pool.to(DEV), v_pool.to(DEV), out, ctx,
                             ctx.block_tables[0], heads, scale, window, rt,
                             sink=torch.tensor(sinks, dtype=torch.float32, device=DEV))
    torch.cuda.synchronize()
    assert int(rt.err.item()) == 0
    return out.view(N, heads, hd), ref, rows_e, rows_p


KERNELS = [("float32", None), ("bfloat16", {"attention": "plain"}), ("bfloat16", None)]
SHAPES = [(6, 2, 16, 4), (2, 2, 12, 8), (8, 2, 32, 16), (4, 4, 64, 16), (16, 2, 64, 32), (1, 1, 20, 4)]


@pytest.mark.parametrize("dtype,options", KERNELS)
@pytest.mark.parametrize("heads,kv_heads,hd,page", SHAPES)
def test_keys_just_inside_and_outside_the_window_with_a_sink(dtype, options, heads, kv_heads, hd, page):
    window = 37
    tol = 1e-5 if dtype == "float32" else 2e-2
    sinks = [0.5 * ((h % 5) - 2) for h in range(heads)]
    lengths = [200, 93, 37, 38, 5, 1]
    for shift, visible in ((window - 1, True), (window, False)):
        needles = [(e, n - 1, n - 1 - shift) for e, n in enumerate(lengths) if n - 1 - shift >= 0]
        out, ref, rows_e, _ = attention_case(dtype, heads, kv_heads, hd, page, lengths, [1] * len(lengths), window,
                                             needles, sinks, seed=shift, options=options)
        assert rel_err(out, ref) < tol
        for (e, qp, kp) in needles:
            i = next(k for k in range(len(rows_e)) if rows_e[k] == e)
            assert bool((ref[i].mean(dim=-1) > 10.0).all()) == visible
    lengths, new = [150, 64, 90], [70, 64, 3]
    needles = [(0, 149, 149 - 36), (0, 100, 100 - 37), (0, 81, 81 - 36), (1, 63, 27), (1, 40, 3), (2, 88, 52)]
    out, ref, _, _ = attention_case(dtype, heads, kv_heads, hd, page, lengths, new, window, needles, sinks, seed=5,
                                    options=options)
    assert rel_err(out, ref) < tol


@pytest.mark.parametrize("dtype,options", KERNELS)
@pytest.mark.parametrize("page", [4, 16])
def test_keys_far_away_at_page_borders_and_the_first_tokens_with_a_sink(dtype, options, page):
    tol = 1e-5 if dtype == "float32" else 2e-2
    heads, kv_heads, hd = 4, 2, 32
    sinks = [-1.0, 0.0, 2.0, 0.7]
    lengths, new = [700, 333, 64, 2], [1, 40, 64, 2]
    needles = [(0, 699, 3), (1, 332, 0), (1, 300, page - 1), (1, 310, page), (1, 320, 20 * page - 1),
               (1, 325, 20 * page), (2, 63, 1), (2, 17, 16), (2, 16, 15), (3, 1, 0)]
    out, ref, _, _ = attention_case(dtype, heads, kv_heads, hd, page, lengths, new, 0, needles, sinks, options=options)
    assert rel_err(out, ref) < tol
    out, ref, _, _ = attention_case(dtype, heads, kv_heads, hd, page, [900, 600], [1, 30], 512,
                                    [(0, 899, 899 - 511), (1, 599, 599 - 512), (1, 580, 580 - 511)], sinks,
                                    options=options)
    assert rel_err(out, ref) < tol


@pytest.mark.parametrize("dtype,options", KERNELS)
@pytest.mark.parametrize("kv_heads,hd,window", [(2, 32, 0), (2, 128, 0), (8, 64, 0), (2, 64, 4000), (4, 128, 1500)])
def test_a_sink_that_dominates_takes_the_weight_away_and_counts_once(dtype, options, kv_heads, hd, window):
    """Also head sizes and windows with which prompts go to the tcgen05 kernel (no window, or one
    that no request of the step is longer than)."""
    tol = 1e-5 if dtype == "float32" else 2e-2
    heads = 8
    # head 0: a sink far above every score (the output vanishes); head 1: far below (as without one);
    # many keys, so that a sink counted once per key tile or once per slice would show
    sinks = [30.0, -30.0, 3.0, 1.0, 0.0, -2.0, 5.0, 2.5]
    out, ref, _, _ = attention_case(dtype, heads, kv_heads, hd, 16, [1500, 300, 70], [1, 100, 70], window, [], sinks,
                                    options=options)
    assert rel_err(out, ref) < tol
    assert float(out[:, 0].abs().max()) < 1e-3
    # a long portion behind a long prefix (the prompt kernel cuts its keys over a cluster) beside decoded tokens
    out, ref, _, _ = attention_case(dtype, heads, kv_heads, hd, 16, [1400, 9, 800], [256, 1, 1], window,
                                    [(0, 1399, 2), (0, 1200, 1199)], sinks, seed=3, options=options)
    # (a score near 19 beside sinks of its size: the 32-bit rounding of the score, some 1e-6 of it,
    # is the relative error of its weight, which the sinks keep from saturating)
    assert rel_err(out, ref) < (5e-5 if dtype == "float32" else tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_query_and_key_norm_and_the_write_of_keys_as_values(dtype):
    from infernum_b200.ops import core
    g = torch.Generator().manual_seed(8)
    N, nh, nkv, hd, page = 11, 4, 2, 20, 4
    x = torch.randn(N, (nh + nkv) * hd + 8, generator=g, dtype=torch.float64).to(dtype)
    qw, kw = torch.rand(hd, generator=g) + 0.5, torch.rand(hd, generator=g) + 0.5
    positions = [7, 8, 9, 10, 11, 0, 1, 2, 3, 4, 5]
    row_entry = [0] * 5 + [1] * 6
    tables = torch.tensor([[5, 2, 0], [3, 1, -1]], dtype=torch.int32)
    kp = torch.zeros(7, nkv, page, hd, dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    xd = x.to(DEV)
    rt = runtime(dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
    core.qk_norm_append(xd, qw.to(DEV), kw.to(DEV), 1e-5, nh, nkv, hd, -1, i32(positions), i32(row_entry),
                        tables.to(DEV), kp, vp, rt.err)
    assert int(rt.err.item()) == 0
    q = x[:, : nh * hd].double().view(N, nh, hd)
    k = x[:, nh * hd: (nh + nkv) * hd].double().view(N, nkv, hd)
    assert rel_err(xd[:, : nh * hd].view(N, nh, hd), pn.unit_rms(q, 1e-5) * qw.double()) < PART_TOL[dtype]
    assert torch.equal(xd[:, nh * hd:].cpu(), x[:, nh * hd:])  # keys and what lies behind them stay as projected
    kn = pn.unit_rms(k, 1e-5) * kw.double()
    for i, (p, e) in enumerate(zip(positions, row_entry)):
        pg = int(tables[e, p // page])
        assert rel_err(kp[pg, :, p % page], kn[i]) < PART_TOL[dtype]
        assert torch.equal(vp[pg, :, p % page].cpu(), x[i, nh * hd: (nh + nkv) * hd].view(nkv, hd))
