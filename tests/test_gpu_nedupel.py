"""The Nedupel design in the engine against the plain implementation (tests/plain/nedupel.py).

The tests make their own small configurations and their own weights (tests/nedupel_models.py): each mechanism alone,
whole prompts against token-by-token decoding, pieces down to two tokens, unequal batches against each request alone,
slots and pages used again, every position across page borders with sharpened attention (one far key among hundreds,
with a control that losing it would show), the first tokens, long decoding (the retention state carried for hundreds of
steps), sizes that are no multiple of 8, constants of 1, one head, one expert, cache rows of the tensor-core sizes, and
greedy generation through the package's entry point.

Tolerances. 32-bit: ||ref - got|| / ||ref|| of every row of logits within 1e-4 (the recurrent layers carry rounding
along a sequence). bfloat16: a row's ||ref - got|| is set against the request's typical row norm (the root mean square
of ||ref|| over its rows); the mean over a request's rows within 5e-2 and every row within 2e-1, and what the schedule
changes is held separately against the engine's own whole run: mean within 2e-2, every row within 1e-1. A lost state,
a wrong edge or a stale page moves rows by their whole size, and the 32-bit runs of the same tests hold every row to 1e-4.
"""
import json
import os

import numpy as np
import pytest

import nedupel_models as nm
from helpers import assert_close, rel_err
from plain import nedupel as plain

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4
BF16_MEAN_TOL, BF16_ROW_TOL, BF16_SCHEDULE_MEAN_TOL, BF16_SCHEDULE_ROW_TOL = 5e-2, 2e-1, 2e-2, 1e-1
DTYPES = ["float32", "bfloat16"]


def close(ref, got, dtype, what, whole=None):
    """`got` against the plain implementation's `ref`; in bfloat16 also against the engine's own whole run."""
    if dtype == "float32":
        return assert_close(ref, got, FP32_TOL, what)
    ref, got = np.asarray(ref, dtype=np.float64), np.asarray(got, dtype=np.float64)
    assert ref.shape == got.shape and np.all(np.isfinite(got)), what
    scale = max(float(np.sqrt((np.linalg.norm(ref, axis=-1) ** 2).mean())), 1e-30)
    rows = np.linalg.norm(ref - got, axis=-1) / scale
    assert rows.mean() <= BF16_MEAN_TOL, f"{what}: mean rel error {rows.mean():.3e}"
    assert rows.max() <= BF16_ROW_TOL, f"{what}: row {int(rows.argmax())} has rel error {rows.max():.3e}"
    if whole is not None:
        rows = np.linalg.norm(np.asarray(whole, dtype=np.float64) - got, axis=-1) / scale
        assert rows.mean() <= BF16_SCHEDULE_MEAN_TOL, f"{what}: mean rel error {rows.mean():.3e} against the whole run"
        assert rows.max() <= BF16_SCHEDULE_ROW_TOL, f"{what}: row {int(rows.argmax())} is {rows.max():.3e} off the whole run"


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return nm.write_models(tmp_path_factory.mktemp("nedupel"))


_ENGINES = {}


def engine(models, name, dtype, max_tokens=2048, **kw):
    from mynah_slm_b200.engine.engine import Engine
    key = (name, dtype, max_tokens, tuple(sorted(kw.items())))
    if key not in _ENGINES:
        _ENGINES[key] = Engine.from_folder(models[name][0], dtype=dtype, max_tokens=max_tokens, **kw)
    return _ENGINES[key]


def entry(slot, tokens, want):
    from mynah_slm_b200.engine.engine import StepEntry
    return StepEntry(slot, list(tokens), tuple(want))


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()


def run_pieces(eng, toks, cuts):
    """One sequence alone, cut at `cuts`; logits of every position."""
    slot = eng.open_sequence()
    rows, lo = [], 0
    for hi in list(cuts) + [len(toks)]:
        if hi > lo:
            rows.append(eng.step([entry(slot, toks[lo:hi], range(hi - lo))]).cpu().numpy())
            lo = hi
    eng.check_status()
    eng.close_sequence(slot)
    return np.concatenate(rows, 0)


# ------------------------------------------------------------------ each mechanism alone, whole prompts
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["latent", "retention", "moe", "dense", "hybrid", "odd", "ragged"])
def test_whole_prompts(models, name, dtype):
    _, cfg, W = models[name]
    eng = engine(models, name, dtype)
    for n in (1, 2, 3, 7, 64, 65, 150):
        toks = tokens_for(cfg, n, n)
        close(plain.forward(cfg, W, toks), run_pieces(eng, toks, []), dtype, f"{name} {dtype} whole {n}")


def test_layers_one_by_one(models):
    """The residual stream behind every layer, 32-bit, against the plain implementation's."""
    _, cfg, W = models["hybrid"]
    eng = engine(models, "hybrid", "float32")
    toks = tokens_for(cfg, 90, 5)
    ref = []
    plain.forward(cfg, W, toks, layers_out=ref)
    slot = eng.open_sequence()
    taps = {}
    eng.step([entry(slot, toks, (0,))], taps=taps)
    eng.close_sequence(slot)
    for i, r in enumerate(ref):
        assert_close(r, taps[f"layer{i}"].cpu().numpy(), FP32_TOL, f"layer {i}")


# ------------------------------------------------------------------ prefill against decoding, pieces
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["hybrid", "odd", "ragged"])
def test_token_by_token(models, name, dtype):
    _, cfg, W = models[name]
    eng = engine(models, name, dtype)
    toks = tokens_for(cfg, 75, 11)
    close(plain.forward(cfg, W, toks), run_pieces(eng, toks, range(1, 75)), dtype, f"{name} {dtype} one by one",
          whole=run_pieces(eng, toks, []))


@pytest.mark.parametrize("dtype", DTYPES)
def test_pieces_of_several_sizes(models, dtype):
    _, cfg, W = models["hybrid"]
    eng = engine(models, "hybrid", dtype)
    toks = tokens_for(cfg, 200, 12)
    ref = plain.forward(cfg, W, toks)
    whole = run_pieces(eng, toks, [])
    for cuts in ([2, 4, 6, 8, 10], [1, 3, 4, 64, 66, 128, 129, 131], [31, 32, 33, 96, 100, 140], [63, 64, 65, 70, 192]):
        close(ref, run_pieces(eng, toks, cuts), dtype, f"{dtype} cuts {cuts}", whole=whole)
    if dtype == "float32":      # pieces and the whole agree far more closely than either with float64
        assert_close(whole, run_pieces(eng, toks, [2, 4, 5, 64, 100, 101, 103]), 2e-5, "whole against pieces")


# ------------------------------------------------------------------ batches
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["hybrid", "odd"])
def test_unequal_batch_then_decode_together(models, name, dtype):
    _, cfg, W = models[name]
    eng = engine(models, name, dtype)
    lens, extra = [5, 130, 1, 66, 31], [20, 3, 12, 20, 7]
    seqs = [tokens_for(cfg, n + e, 40 + i) for i, (n, e) in enumerate(zip(lens, extra))]
    refs = [plain.forward(cfg, W, s) for s in seqs]
    wholes = [run_pieces(eng, s, []) for s in seqs]
    slots = [eng.open_sequence() for _ in seqs]
    got = [[] for _ in seqs]
    out = eng.step([entry(s, t[:n], range(n)) for s, t, n in zip(slots, seqs, lens)]).cpu().numpy()
    at = 0
    for i, n in enumerate(lens):
        got[i].append(out[at:at + n])
        at += n
    live = list(range(len(seqs)))
    step = 0
    while live:
        out = eng.step([entry(slots[i], [seqs[i][lens[i] + step]], (0,)) for i in live]).cpu().numpy()
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1])
        step += 1
        for i in [i for i in live if step >= extra[i]]:       # shorter requests end earlier
            eng.close_sequence(slots[i])
            live.remove(i)
    eng.check_status()
    for i, ref in enumerate(refs):
        close(ref, np.concatenate(got[i], 0), dtype, f"{name} {dtype} request {i}", whole=wholes[i])


def test_batch_equals_alone_in_32_bit(models):
    _, cfg, _ = models["hybrid"]
    eng = engine(models, "hybrid", "float32")
    seqs = [tokens_for(cfg, n, 60 + n) for n in (3, 77, 140)]
    alone = [run_pieces(eng, s, []) for s in seqs]
    slots = [eng.open_sequence() for _ in seqs]
    out = eng.step([entry(s, t, range(len(t))) for s, t in zip(slots, seqs)]).cpu().numpy()
    for s in slots:
        eng.close_sequence(s)
    at = 0
    for a in alone:
        assert_close(a, out[at:at + len(a)], 2e-5, "batched against alone")
        at += len(a)


# ------------------------------------------------------------------ slots and pages used again
@pytest.mark.parametrize("dtype", DTYPES)
def test_slots_and_pages_used_again(models, dtype):
    _, cfg, W = models["hybrid"]
    eng = engine(models, "hybrid", dtype, max_tokens=256, max_seqs=2)      # 4 pages, 2 slots
    seen = set()
    for round_ in range(4):
        toks_a, toks_b = tokens_for(cfg, 100 + round_, 70 + round_), tokens_for(cfg, 30 + round_, 80 + round_)
        sa, sb = eng.open_sequence(), eng.open_sequence()
        seen.update((sa, sb))
        out = eng.step([entry(sa, toks_a[:90], range(90)), entry(sb, toks_b[:20], range(20))]).cpu().numpy()
        rows_a, rows_b = [out[:90]], [out[90:]]
        for t in range(10):
            out = eng.step([entry(sa, [toks_a[90 + t]], (0,)), entry(sb, [toks_b[20 + t]], (0,))]).cpu().numpy()
            rows_a.append(out[:1])
            rows_b.append(out[1:])
        eng.check_status()
        eng.close_sequence(sa)
        eng.close_sequence(sb)
        close(plain.forward(cfg, W, toks_a[:100]), np.concatenate(rows_a, 0), dtype, f"round {round_} a")
        close(plain.forward(cfg, W, toks_b[:30]), np.concatenate(rows_b, 0), dtype, f"round {round_} b")
    assert len(seen) <= 2


# ------------------------------------------------------------------ far keys and page borders
def test_every_position_with_sharp_attention(models):
    """Sharp attention, 32-bit: every position of a prompt that spans several pages, run whole, in pieces around the
    page borders, and with its last 150 tokens decoded one by one. The control shows that another key at ONE far place
    (the first position) would be seen at this tolerance."""
    _, cfg, W = models["sharp"]
    eng = engine(models, "sharp", "float32")
    toks = tokens_for(cfg, 420, 21)
    ref = plain.forward(cfg, W, toks)
    assert_close(ref, run_pieces(eng, toks, []), FP32_TOL, "sharp whole")
    assert_close(ref, run_pieces(eng, toks, range(270, 420)), FP32_TOL, "sharp decoded")
    assert_close(ref, run_pieces(eng, toks, [63, 64, 65, 127, 128, 129, 191, 192, 256, 257, 320]), FP32_TOL, "sharp pieces")
    other = [(toks[0] + 1) % cfg["vocab"]] + toks[1:]
    assert rel_err(ref[300:], plain.forward(cfg, W, other)[300:]) > 100 * FP32_TOL, "control: the first position's key goes unseen"


def test_one_far_key_stands_out(models):
    """The same token far back and at the end, between hundreds of others, with weights under which a token's query
    finds its own latent: the attention's weight sits on ONE key hundreds of positions away. Whole and decoded."""
    import torch
    from mynah_slm_b200.engine.engine import Engine
    from mynah_slm_b200.weights.safetensors_io import write_safetensors
    folder, cfg, _ = models["latent"]
    m = cfg["layers"][0]["mixer"]
    Wt = nm.make_weights(cfg, 99)
    H, dim, rd, r = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
    # queries ignore positions (no weight on the rotated part) and equal, through W_uk, a multiple of the token's own latent
    dkv = Wt["l0.mix.dkv"].to(torch.float64)
    uk = torch.zeros((H, dim, r), dtype=torch.float64)
    q = torch.zeros((H, dim + rd, cfg["width"]), dtype=torch.float64)
    for h in range(H):
        uk[h, :, h * dim:(h + 1) * dim] = torch.eye(dim)[:, :min(dim, r - h * dim)] if h * dim < r else 0
        if h * dim < r:
            q[h, :min(dim, r - h * dim)] = 4.0 * dkv[h * dim:h * dim + min(dim, r - h * dim)]
    Wt["l0.mix.uk"] = uk.reshape(H * dim, r).to(torch.bfloat16)
    Wt["l0.mix.q"] = q.reshape(H * (dim + rd), -1).to(torch.bfloat16)
    sharp = os.path.join(os.path.dirname(folder), "latent_far")
    os.makedirs(sharp, exist_ok=True)
    with open(os.path.join(sharp, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(sharp, "model.safetensors"), Wt)
    W = {n: (t.to(torch.float64) if t.dtype.is_floating_point else t.to(torch.int64)).numpy() for n, t in Wt.items()}
    rng = np.random.default_rng(8)
    toks = rng.integers(1, cfg["vocab"], size=700).tolist()
    toks[5] = toks[-1] = 0                                 # token 0 at position 5 and at the end, nowhere between
    toks = [t if t != 0 or i in (5, 699) else 1 for i, t in enumerate(toks)]
    ref = plain.forward(cfg, W, toks)
    moved = list(toks)
    moved[5] = 1
    assert rel_err(ref[-1:], plain.forward(cfg, W, moved)[-1:]) > 1e-2, "control: the far key does not stand out"
    eng = Engine.from_folder(sharp, dtype="float32", max_tokens=1024)
    assert_close(ref, run_pieces(eng, toks, []), FP32_TOL, "far key, whole")
    assert_close(ref, run_pieces(eng, toks, range(660, 700)), FP32_TOL, "far key, decoded")
    eng16 = Engine.from_folder(sharp, dtype="bfloat16", max_tokens=1024)
    close(ref[-40:], run_pieces(eng16, toks, range(660, 700))[-40:], "bfloat16", "far key, decoded in bfloat16")


def test_tensor_core_attention_sizes(models):
    """bfloat16 with cache rows of 64 and 128 values: the tensor-core attention kernels against the plain
    implementation, and against the general kernels on the same cache, whole, in pieces and decoded."""
    from mynah_slm_b200.ops import attention_dispatch
    _, cfg, W = models["wide"]
    toks = tokens_for(cfg, 520, 41)
    ref = plain.forward(cfg, W, toks)
    eng = engine(models, "wide", "bfloat16")
    runs = {}
    for use_tc in (True, False):
        attention_dispatch.USE_TC_MASKED = use_tc
        try:
            eng_k = eng if use_tc else engine(models, "wide", "bfloat16", use_graphs=False)
            runs[use_tc] = [run_pieces(eng_k, toks, cuts) for cuts in ([], [99, 100, 101, 128, 150, 200, 201, 300, 399, 400],
                                                                       range(380, 520))]
        finally:
            attention_dispatch.USE_TC_MASKED = True
    for got_tc, got_general in zip(runs[True], runs[False]):
        close(ref, got_tc, "bfloat16", "tensor-core attention", whole=got_general)
        close(ref, got_general, "bfloat16", "general attention")
    close(ref, run_pieces(engine(models, "wide", "float32"), toks, [150, 151, 400]), "float32", "wide in 32-bit")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(models, dtype):
    _, cfg, W = models["hybrid"]
    eng = engine(models, "hybrid", dtype)
    toks = tokens_for(cfg, 330, 31)
    close(plain.forward(cfg, W, toks), run_pieces(eng, toks, range(10, 330)), dtype, f"{dtype} long decoding",
          whole=run_pieces(eng, toks, []))


def test_first_tokens(models):
    """Positions 0..5 of several sequences, as prompts of one to six tokens and decoded from the first token on."""
    _, cfg, W = models["hybrid"]
    eng = engine(models, "hybrid", "float32")
    for n in range(1, 7):
        toks = tokens_for(cfg, n, 90 + n)
        ref = plain.forward(cfg, W, toks)
        assert_close(ref, run_pieces(eng, toks, []), FP32_TOL, f"prompt of {n}")
        assert_close(ref, run_pieces(eng, toks, range(1, n)), FP32_TOL, f"decoded from the first of {n}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_large_sizes(models, dtype):
    _, cfg, W = models["large"]
    eng = engine(models, "large", dtype, max_tokens=1024)
    toks = tokens_for(cfg, 200, 61)
    ref = plain.forward(cfg, W, toks)
    whole = run_pieces(eng, toks, [])
    close(ref, whole, dtype, f"large {dtype} whole")
    close(ref, run_pieces(eng, toks, [3, 5, 64, 89, 90, 91, 150] + list(range(180, 200))), dtype, f"large {dtype} pieces",
          whole=whole)


def test_without_graphs_equals_with(models):
    _, cfg, _ = models["hybrid"]
    toks = tokens_for(cfg, 120, 33)
    a = run_pieces(engine(models, "hybrid", "float32"), toks, range(100, 120))
    b = run_pieces(engine(models, "hybrid", "float32", use_graphs=False), toks, range(100, 120))
    assert_close(a, b, 1e-6, "captured steps against launched ones")


def test_retention_chunk_by_chunk_equals_token_by_token(models):
    """Prompts through the chunked form of the retention recurrence against the same prompts token by token inside the
    kernel, alone and in an unequal batch, and the token after (the state the prompts left)."""
    from mynah_slm_b200.ops import kernels
    _, cfg, W = models["wide"]
    seqs = [tokens_for(cfg, n, 500 + n) for n in (300, 129, 5, 191)]
    runs = []
    for chunk_min in (16, 0):
        before = kernels.retention_chunk_min(chunk_min)
        try:
            eng = engine(models, "wide", "float32", use_graphs=False)
            slots = [eng.open_sequence() for _ in seqs]
            out = eng.step([entry(sl, s, range(len(s))) for sl, s in zip(slots, seqs)]).cpu().numpy()
            nxt = eng.step([entry(sl, [7], (0,)) for sl in slots]).cpu().numpy()
            for sl in slots:
                eng.close_sequence(sl)
            runs.append((out, nxt))
        finally:
            kernels.retention_chunk_min(before)
    assert_close(runs[1][0], runs[0][0], 2e-5, "chunk by chunk against token by token")
    assert_close(runs[1][1], runs[0][1], 2e-5, "the token after")
    at = 0
    for i, s in enumerate(seqs):
        ref = plain.forward(cfg, W, s + [7])
        close(ref[:-1], runs[0][0][at:at + len(s)], "float32", f"batched prompt of {len(s)}")
        close(ref[-1:], runs[0][1][i:i + 1], "float32", f"the token after the prompt of {len(s)}")
        at += len(s)


def test_random_weights_on_the_device_equal_a_written_folder(tmp_path):
    """`Engine.random` (weights and expert tables made in place) against the folder `write_random_model` writes."""
    import torch
    from mynah_slm_b200.engine.engine import Engine
    from mynah_slm_b200.registry import parse_config
    from mynah_slm_b200.weights.random_init import write_random_model
    cfg = nm.HYBRID
    folder = write_random_model(str(tmp_path / "m"), parse_config(cfg), 3, torch.bfloat16)
    a = Engine.from_folder(folder, dtype="float32", max_tokens=256)
    b = Engine.random(cfg, seed=3, dtype="float32", stored_dtype="bfloat16", max_tokens=256)
    toks = tokens_for(cfg, 50, 1)
    assert np.array_equal(run_pieces(a, toks, [20]), run_pieces(b, toks, [20]))


# ------------------------------------------------------------------ generation through the entry point
@pytest.mark.parametrize("name", ["hybrid", "odd"])
def test_greedy_generation(models, name):
    from mynah_slm_b200 import LLM
    folder, cfg, W = models[name]
    llm = LLM(folder, dtype="float32", max_tokens=1024)
    prompts = [tokens_for(cfg, n, 200 + n) for n in (4, 70, 1, 33, 129)]
    n_new = 24
    results = llm.generate(prompts, max_new=n_new, temp=0.0, ignore_eos=True, max_batch=3)
    for p, r in zip(prompts, results):
        seq = list(p)
        for t in range(n_new):
            logits = plain.forward(cfg, W, seq)[-1]
            top2 = np.sort(logits)[-2:]
            if top2[1] - top2[0] < 1e-3 * max(1.0, abs(top2[1])):
                break                                   # a near tie: either choice is right, stop comparing
            assert r.tokens[t] == int(np.argmax(logits)), f"{name}: token {t} of the prompt of {len(p)}"
            seq.append(r.tokens[t])


def test_command_line(models, tmp_path):
    """`mynah-slm run` on a folder (greedy tokens against the plain implementation, the prompts' logits written beside),
    sampling with a temperature, and `mynah-slm random` + `run --random` making the same model twice."""
    import subprocess
    import sys
    folder, cfg, W = models["hybrid"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cli = [sys.executable, os.path.join(root, "bin", "mynah-slm")]
    a, b = tokens_for(cfg, 40, 401), tokens_for(cfg, 3, 402)
    ids = lambda t: ",".join(str(x) for x in t)
    npy = tmp_path / "logits.npy"
    p = subprocess.run(cli + ["run", "-m", folder, "--tokens", ids(a), "--tokens", ids(b), "-n", "5", "--temp", "0", "--dtype", "float32",
                              "--ignore-eos", "--quiet", "--logits-out", str(npy)], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [[int(x) for x in l.split()] for l in p.stdout.strip().splitlines()]
    assert len(lines) == 2 and all(len(l) == 5 for l in lines)
    ra, rb = plain.forward(cfg, W, a), plain.forward(cfg, W, b)
    assert_close(np.concatenate([ra, rb]), np.load(npy), FP32_TOL, "--logits-out")
    for prompt, got in ((a, lines[0]), (b, lines[1])):
        seq = list(prompt)
        for t in range(5):
            logits = plain.forward(cfg, W, seq)[-1]
            top2 = np.sort(logits)[-2:]
            if top2[1] - top2[0] < 1e-3 * max(1.0, abs(top2[1])):
                break
            assert got[t] == int(np.argmax(logits))
            seq.append(got[t])
    s = subprocess.run(cli + ["run", "-m", folder, "--tokens", ids(a), "-n", "12", "--temp", "0.8", "--top-k", "20", "--seed", "3",
                              "--ignore-eos", "--quiet"], capture_output=True, text=True, timeout=600)
    assert s.returncode == 0 and len(s.stdout.split()) == 12 and all(0 <= int(x) < cfg["vocab"] for x in s.stdout.split())
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(cfg))
    w = subprocess.run(cli + ["random", "-o", str(tmp_path / "made"), "--config", str(cfg_path), "--seed", "4", "--dtype", "bfloat16"],
                       capture_output=True, text=True, timeout=600)
    assert w.returncode == 0, w.stderr[-2000:]
    runs = [subprocess.run(cli + src + ["--tokens", ids(b), "-n", "6", "--temp", "0", "--ignore-eos", "--quiet"],
                           capture_output=True, text=True, timeout=600)
            for src in (["run", "-m", str(tmp_path / "made")], ["run", "--random", str(cfg_path), "--weights-seed", "4"])]
    assert all(r.returncode == 0 for r in runs), runs[0].stderr[-1000:] + runs[1].stderr[-1000:]
    assert runs[0].stdout.split() == runs[1].stdout.split() and len(runs[0].stdout.split()) == 6


def test_trace_runner_process(models, tmp_path):
    """bin/trace_run as a process: a batch of two prompts, decoding together, one ends early."""
    import subprocess
    import sys
    folder, cfg, W = models["hybrid"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    a, b = tokens_for(cfg, 70, 301), tokens_for(cfg, 9, 302)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[66:67], "want": [0]}, {"id": "b", "tokens": b[7:8], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[67:68], "want": [0]}, {"id": "b", "tokens": b[8:9], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[68:69], "want": [0]}], "end": ["a"]}]
    out = str(tmp_path / "out")
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", out, "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps),
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    ra, rb = plain.forward(cfg, W, a), plain.forward(cfg, W, b)
    read = lambda i: np.fromfile(os.path.join(out, f"{i}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])
    assert_close(np.stack([ra[0], ra[65], rb[6]]), read(0), FP32_TOL, "step 0")
    assert_close(ra[66:67], read(1), FP32_TOL, "step 1")
    assert_close(np.stack([ra[67], rb[8]]), read(2), FP32_TOL, "step 2")
    assert_close(ra[68:69], read(3), FP32_TOL, "step 3")
