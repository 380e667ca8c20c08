"""The Supisun design in the engine against the plain implementation (tests/plain/supisun.py).

The tests make their own small configurations and their own weights (numpy generator, values that bfloat16 holds
exactly, written with the package's safetensors writer): each mechanism alone, whole prompts against token-by-token
decoding, pieces down to two tokens, unequal batches against each request alone, slots and pages used again, every
position across page borders and chunk edges in prompts and in decoding (with sharpened attention, and a control
that a chunk one token off would show), long decoding, sizes that are no multiple of 8, and greedy generation
through the package's entry point.

Tolerances. 32-bit: ||ref - got|| / ||ref|| of every row of logits within 1e-4 (the recurrent layers carry rounding
along a sequence). bfloat16: a row's ||ref - got|| is set against the request's typical row norm (the root mean square
of ||ref|| over its rows) rather than against its own, since a row of small logits says nothing about the size of
rounding errors; the mean over a request's rows within 5e-2 and every row within 2e-1: at these small widths single
rows scatter (measured on the hybrid configuration with several seeds: mean 0.013 to 0.036, largest row 0.06 to 0.10,
and 0.26 against its own norm, the same to three digits whether the prompt ran whole or token by token), so a tight
bound on every row would not hold; what the schedule changes is held separately against the engine's own whole run:
mean within 2e-2, every row within 1e-1 (prompt and decode steps use different product kernels, which round apart;
the largest row seen was 0.055). A lost state, a wrong edge or a stale page moves rows by their whole size, and the
32-bit runs of the same tests hold every row to 1e-4.
"""
import json
import os

import numpy as np
import pytest
import torch

from helpers import assert_close
from plain import supisun as plain

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4
BF16_MEAN_TOL, BF16_ROW_TOL, BF16_SCHEDULE_MEAN_TOL, BF16_SCHEDULE_ROW_TOL = 5e-2, 2e-1, 2e-2, 1e-1


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
        whole = np.asarray(whole, dtype=np.float64)
        rows = np.linalg.norm(whole - got, axis=-1) / scale
        assert rows.mean() <= BF16_SCHEDULE_MEAN_TOL, f"{what}: mean rel error {rows.mean():.3e} against the whole run"
        assert rows.max() <= BF16_SCHEDULE_ROW_TOL, f"{what}: row {int(rows.argmax())} is {rows.max():.3e} off the whole run"


def attn(heads, kv_heads, dim, vdim, scale, rot=None, mask=None, v_mix=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if mask is not None:
        m["mask"] = {"size": mask}
    if v_mix is not None:
        m["v_mix"] = v_mix
    return {"type": "attention", "mixer": m}


def mamba(inner, state, dt_rank, conv):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}


def delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def with_mlp(layer, ff):
    return dict(layer, mlp={"kind": "dense", "ff": ff} if ff else None)


def config(width, vocab, layers, taps=3, eps=1e-5, max_positions=512):
    return {"architecture": "Supisun", "vocab": vocab, "width": width, "max_positions": max_positions,
            "norm": {"eps": eps}, "canon": {"taps": taps}, "layers": layers}


# a hybrid: two mixing attention layers around a non-mixing one, partial and full rotation, chunks that are no
# multiple of a page, both recurrent mixers, one layer without feed-forward
HYBRID = config(64, 300, [
    with_mlp(attn(4, 2, 16, 24, 0.31, rot=(8, 10000.0), mask=48, v_mix=True), 96),
    with_mlp(delta(4, 2, 16, 8, 3), 80),
    with_mlp(mamba(96, 8, 4, 2), None),
    with_mlp(attn(2, 1, 32, 16, 0.2, mask=100), 72),
    with_mlp(attn(6, 2, 8, 24, 0.4, rot=(8, 500.0), mask=70, v_mix=True), 96),
    with_mlp(mamba(72, 16, 6, 4), 64),
], taps=4, max_positions=400)
# sizes that are no multiple of 8, one tap everywhere (no history), kv heads equal to heads, a chunk of one
# position, no rotation, no mask, a state of five values
ODD = config(40, 131, [
    with_mlp(mamba(44, 5, 3, 1), 52),
    with_mlp(attn(3, 3, 20, 12, 0.5, rot=(6, 77.0), mask=1), None),
    with_mlp(delta(3, 3, 12, 20, 1), 36),
    with_mlp(attn(2, 2, 12, 20, 0.25), 60),
    with_mlp(delta(4, 1, 40, 4, 2), None),
], taps=1, eps=1e-3, max_positions=256)
ONLY_ATTENTION = config(48, 200, [with_mlp(attn(4, 2, 16, 8, 0.25, rot=(16, 300.0), mask=40), None)], taps=2)
ONLY_MAMBA = config(48, 200, [with_mlp(mamba(64, 12, 5, 3), None)], taps=2)
ONLY_DELTA = config(48, 200, [with_mlp(delta(4, 2, 24, 16, 4), None)], taps=2)
ONLY_MLP = config(48, 200, [with_mlp(mamba(16, 2, 1, 2), 128)], taps=5)
# attention whose softmax is sharp (large gains): one key stands out among hundreds, so a wrong edge shows
SHARP = config(64, 150, [
    with_mlp(attn(4, 1, 16, 16, 1.0, rot=(16, 1000.0), mask=80, v_mix=True), 64),
    with_mlp(attn(2, 1, 32, 16, 0.8, rot=(8, 50.0), mask=130, v_mix=True), None),
], taps=2, max_positions=600)

# heads of 64 and 128 with keys and values alike: the sizes the tensor-core attention kernels take in bfloat16;
# chunks that are no multiple of a page or of a tile, a large state and wide keys in the recurrent layers
WIDE = config(128, 200, [
    with_mlp(attn(4, 2, 64, 64, 0.125, rot=(64, 10000.0), mask=100, v_mix=True), 128),
    with_mlp(attn(2, 1, 128, 128, 0.09, rot=(32, 500.0), mask=150), None),
    with_mlp(mamba(160, 40, 8, 4), None),
    with_mlp(delta(2, 1, 136, 24, 2), None),
    with_mlp(attn(4, 2, 64, 64, 0.2, mask=200, v_mix=True), 96),
], taps=2, max_positions=700)

# the large ends: a state of 128 and of 256 values a channel, keys of 256 in the delta rule and in attention (values
# of 8), six taps in front of the mixers and five inside them, many kv heads
LARGE = config(96, 180, [
    with_mlp(mamba(48, 128, 5, 5), None),
    with_mlp(delta(4, 2, 256, 40, 5), 64),
    with_mlp(attn(8, 8, 256, 8, 0.06, rot=(128, 10000.0), mask=90), None),
    with_mlp(mamba(40, 256, 3, 2), None),
], taps=6, max_positions=320)

CONFIGS = {"wide": WIDE, "large": LARGE, "hybrid": HYBRID, "odd": ODD, "attention": ONLY_ATTENTION, "mamba": ONLY_MAMBA, "delta": ONLY_DELTA,
           "mlp": ONLY_MLP, "sharp": SHARP}


def tensor_shapes(cfg):
    D, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, D), "pos": (cfg["max_positions"], D), "final.norm": (D,), "final.norm.b": (D,), "head": (V, D)}
    mixing = [i for i, L in enumerate(cfg["layers"]) if L["type"] == "attention" and L["mixer"].get("v_mix")]
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        s[p + "canon1"] = (D, cfg["canon"]["taps"])
        s[p + "norm1"] = s[p + "norm1.b"] = (D,)
        if L.get("mlp"):
            s[p + "norm2"] = s[p + "norm2.b"] = (D,)
            s[p + "mlp.up"], s[p + "mlp.down"] = (L["mlp"]["ff"], D), (D, L["mlp"]["ff"])
        p += "mix."
        if L["type"] == "attention":
            H, G, dim, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            s.update({p + "q": (H * dim, D), p + "k": (G * dim, D), p + "v": (G * vd, D), p + "o": (D, H * vd),
                      p + "q.norm": (H * dim,), p + "k.norm": (G * dim,)})
            if m.get("v_mix"):
                s[p + "vmix"] = ()
        elif L["type"] == "mamba1":
            I, N, R, t = m["inner"], m["state"], m["dt_rank"], m["conv"]
            s.update({p + "in": (2 * I, D), p + "conv": (I, t), p + "conv.b": (I,), p + "x": (R + 2 * N, I),
                      p + "dt": (I, R), p + "dt.b": (I,), p + "A_log": (I, N), p + "D": (I,), p + "o": (D, I)})
        else:
            H, G, dim, vd, t = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            s.update({p + "q": (G * dim, D), p + "q.conv": (G * dim, t), p + "k": (G * dim, D), p + "k.conv": (G * dim, t),
                      p + "v": (H * vd, D), p + "v.conv": (H * vd, t), p + "b": (H, D), p + "a": (H, D),
                      p + "A_log": (H,), p + "dt_bias": (H,), p + "g": (H * vd, D), p + "norm": (vd,), p + "o": (D, H * vd)})
    return s


def make_weights(cfg, seed, sharp=False):
    rng = np.random.default_rng(seed)
    W = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if name in ("embed",):
            w = rng.normal(0, 1.0, shape)
        elif name == "pos":
            w = rng.normal(0, 0.5, shape)
        elif last == "vmix":
            w = np.asarray(rng.uniform(0.2, 0.8))
        elif last == "norm" and ("q.norm" in name or "k.norm" in name):
            w = (3.0 if sharp else 1.0) * (1.0 + 0.1 * rng.normal(size=shape))
        elif last in ("norm", "norm1", "norm2", "D"):
            w = 1.0 + 0.1 * rng.normal(size=shape)
        elif last in ("b",) and len(shape) == 1:
            w = 0.1 * rng.normal(size=shape)
        elif last in ("conv", "canon1"):
            w = rng.normal(0, 0.4, shape)
        elif last in ("A_log", "dt_bias"):
            w = rng.normal(0, 0.5, shape)
        elif len(shape) == 2:
            w = rng.normal(0, 1.0 / np.sqrt(shape[1]), shape)
        else:
            w = 0.1 * rng.normal(size=shape)
        W[name] = torch.tensor(np.asarray(w), dtype=torch.float32).to(torch.bfloat16)
    return W


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (folder, config, weights as float64 numpy)."""
    from mynah_slm_b200.weights.safetensors_io import write_safetensors
    root = tmp_path_factory.mktemp("supisun")
    out = {}
    import zlib
    for name, cfg in CONFIGS.items():
        folder = os.path.join(str(root), name)
        os.makedirs(folder)
        W = make_weights(cfg, zlib.crc32(name.encode()) % 1000, sharp=name == "sharp")       # a seed that stays with the name
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(cfg, f)
        write_safetensors(os.path.join(folder, "model.safetensors"), W)
        out[name] = (folder, cfg, {n: t.to(torch.float64).numpy() for n, t in W.items()})
    return out


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


DTYPES = ["float32", "bfloat16"]


# ------------------------------------------------------------------ configuration and weights
def test_tensor_names_and_shapes(models):
    from mynah_slm_b200.engine.model import Model
    from mynah_slm_b200.registry import parse_config
    for name, (_, cfg, _) in models.items():
        specs = {ts.name: tuple(ts.shape) for _, ts in Model(parse_config(cfg).model_spec()).tensor_specs()}
        assert specs == tensor_shapes(cfg), name


# ------------------------------------------------------------------ each mechanism alone, whole prompts
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["attention", "mamba", "delta", "mlp", "hybrid", "odd"])
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
@pytest.mark.parametrize("name", ["hybrid", "odd"])
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
    for cuts in ([2, 4, 6, 8, 10], [1, 3, 4, 64, 66, 128, 129, 131], [47, 48, 49, 96, 100, 140], [63, 64, 65, 70, 192]):
        close(ref, run_pieces(eng, toks, cuts), dtype, f"{dtype} cuts {cuts}", whole=whole)
    if dtype == "float32":      # pieces and the whole agree far more closely than either with float64
        a, b = run_pieces(eng, toks, []), run_pieces(eng, toks, [2, 4, 5, 64, 100, 101, 103])
        assert_close(a, b, 2e-5, "whole against pieces")


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


# ------------------------------------------------------------------ far keys, page borders, chunk edges
def test_every_position_across_edges_sharp(models):
    """Sharp attention, 32-bit: every position of a prompt that spans several chunks and pages, run whole and with
    its last 150 tokens decoded one by one. The control shows that a chunk one token longer or shorter would be
    seen at this tolerance."""
    _, cfg, W = models["sharp"]
    eng = engine(models, "sharp", "float32")
    toks = tokens_for(cfg, 420, 21)
    ref = plain.forward(cfg, W, toks)
    assert_close(ref, run_pieces(eng, toks, []), FP32_TOL, "sharp whole")
    assert_close(ref, run_pieces(eng, toks, range(270, 420)), FP32_TOL, "sharp decoded")
    assert_close(ref, run_pieces(eng, toks, [79, 80, 81, 129, 130, 131, 160, 161, 260, 261]), FP32_TOL, "sharp pieces")
    from helpers import rel_err
    sizes = sorted({L["mixer"]["mask"]["size"] for L in cfg["layers"]})
    for size in sizes:
        for off in (-1, 1):
            other = json.loads(json.dumps(cfg))
            for L in other["layers"]:
                if L["mixer"]["mask"]["size"] == size:
                    L["mixer"]["mask"]["size"] = size + off
            assert rel_err(ref, plain.forward(other, W, toks)) > 100 * FP32_TOL, f"control: chunk {size}{off:+d} goes unseen"


def test_tensor_core_attention_under_chunks(models):
    """bfloat16 with heads of 64 and 128: the tensor-core kernels with chunk mask and given scale against the plain
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
    close(ref, run_pieces(engine(models, "wide", "float32"), toks, []), "float32", "wide in 32-bit, whole")


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


def test_long_prompts_in_pieces_side_by_side(models):
    """Prompts long enough for the scan's two-pass form (pieces that run side by side), alone and in an unequal
    batch, against the plain implementation and against the one-pass form."""
    from mynah_slm_b200.ops import kernels
    _, cfg, W = models["hybrid"]
    eng = engine(models, "hybrid", "float32")
    seqs = [tokens_for(cfg, n, 500 + n) for n in (300, 129, 5, 191)]
    refs = [plain.forward(cfg, W, s) for s in seqs]
    for s, ref in zip(seqs, refs):
        close(ref, run_pieces(eng, s, []), "float32", f"whole prompt of {len(s)}")
        close(ref, run_pieces(eng, s, [len(s) - 140]), "float32", f"prompt of {len(s)} in two pieces")
    slots = [eng.open_sequence() for _ in seqs]
    out = eng.step([entry(sl, s, range(len(s))) for sl, s in zip(slots, seqs)]).cpu().numpy()
    nxt = eng.step([entry(sl, [7], (0,)) for sl in slots]).cpu().numpy()        # the state the prompts left
    for sl in slots:
        eng.close_sequence(sl)
    at = 0
    for i, (s, ref) in enumerate(zip(seqs, refs)):
        close(ref, out[at:at + len(s)], "float32", f"batched prompt of {len(s)}")
        close(plain.forward(cfg, W, s + [7])[-1:], nxt[i:i + 1], "float32", f"the token after the prompt of {len(s)}")
        at += len(s)
    before = kernels.SCAN_PIECE_ROWS
    kernels.SCAN_PIECE_ROWS = 0
    try:
        one_pass = run_pieces(engine(models, "hybrid", "float32", use_graphs=False), seqs[0], [])
    finally:
        kernels.SCAN_PIECE_ROWS = before
    assert_close(one_pass, run_pieces(eng, seqs[0], []), 2e-5, "two passes against one")


def test_without_graphs_equals_with(models):
    _, cfg, _ = models["hybrid"]
    toks = tokens_for(cfg, 120, 33)
    a = run_pieces(engine(models, "hybrid", "float32"), toks, range(100, 120))
    b = run_pieces(engine(models, "hybrid", "float32", use_graphs=False), toks, range(100, 120))
    assert_close(a, b, 1e-6, "captured steps against launched ones")


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
