"""The kernels behind the Nedupel parts, each alone, against the plain functions of tests/plain/nedupel.py (float64):
rotation tables from frequency lists, the latent preparation with its cache write, the per-head products, the retention
preparation and recurrence (whole, in pieces, one row a step, two sequences, padding rows, state from another slot),
the table-routed experts, and the scaled embedding, residual add, norm and logits."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from plain import nedupel as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def i32(v):
    return torch.tensor(np.asarray(v), dtype=torch.int32, device=DEV)


def t32(a):
    return torch.tensor(np.asarray(a), dtype=torch.float32, device=DEV)


def rel(ref, got):
    ref, got = np.asarray(ref, dtype=np.float64), np.asarray(got, dtype=np.float64)
    return float(np.abs(ref - got).max() / max(np.abs(ref).max(), 1e-30))


def ctx_for(q_lens, slots, starts=None, pad_rows=0, tokens=None):
    """The fields of a step's context that the kernels read: rows packed sequence by sequence, then padding rows."""
    starts = starts or [0] * len(q_lens)
    tok_seq, tok_pos, cu = [], [], [0]
    for b, (n, s) in enumerate(zip(q_lens, starts)):
        tok_seq += [b] * n
        tok_pos += list(range(s, s + n))
        cu.append(cu[-1] + n)
    tok_seq += [-1] * pad_rows
    tok_pos += [0] * pad_rows
    T = len(tok_seq)
    return SimpleNamespace(tok_seq=i32(tok_seq), tok_pos=i32(tok_pos), cu_q=i32(cu), slots=i32(slots), B=len(q_lens), T=T,
                           tokens=i32(tokens if tokens is not None else [0] * T),
                           status=torch.zeros((1,), dtype=torch.int32, device=DEV), is_decode=all(n == 1 for n in q_lens),
                           max_q_len=max(q_lens))


@pytest.mark.parametrize("rot", [{"dims": 16, "base": 5000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}},
                                 {"dims": 6, "base": 20.0}])
def test_rotation_tables(rot):
    from mynah_slm_b200.ops import kernels
    from mynah_slm_b200.parts.position import rotary_frequencies
    f, mult = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    cos, sin = kernels.rope_table_freqs(3000, f, mult, DEV)
    a, m = plain.rotary_angles(np.arange(3000), rot)
    assert np.abs(cos.cpu().numpy() - np.cos(a) * m).max() < 1e-7 and np.abs(sin.cpu().numpy() - np.sin(a) * m).max() < 1e-7


@pytest.mark.parametrize("H,dim,rd,r,interleaved", [(4, 16, 8, 40, True), (1, 6, 10, 13, True), (3, 8, 16, 24, False), (2, 12, 0, 20, True)])
def test_latent_prep_and_cache_rows(H, dim, rd, r, interleaved):
    from mynah_slm_b200.ops import kernels
    from mynah_slm_b200.parts.position import rotary_frequencies
    rng = np.random.default_rng(H * 100 + r)
    HDp = (r + rd + 7) // 8 * 8
    T, start = 70, 60                                            # positions 60..129: two pages, both partly written
    q = rng.normal(size=(T, H * (dim + rd)))
    d = rng.normal(size=(T, r + rd))
    w = 1.0 + 0.1 * rng.normal(size=(r,))
    rot = {"dims": rd, "base": 300.0} if rd else None
    cos = sin = None
    if rd:
        f, mult = rotary_frequencies(rd, 300.0, None)
        cos, sin = kernels.rope_table_freqs(256, f, mult, DEV)
    p = torch.cat([t32(q), t32(d)], 1).contiguous()
    ctx = ctx_for([T], [0], starts=[start], pad_rows=2)
    p = torch.cat([p, torch.zeros((2, p.shape[1]), device=DEV)], 0).contiguous()
    pages = kernels.PageTableView(i32([0, 3]), i32([5, 2, 7]), i32([0]), 8)        # logical pages 0, 1, 2 -> 5, 2, 7
    k_cache = torch.full((8, 1, 64, HDp), 9.0, dtype=torch.float32, device=DEV)
    q_out = torch.full((T + 2, H * HDp), 9.0, dtype=torch.float32, device=DEV)
    kernels.latent_prep(p, 0, p, H * (dim + rd), q_out, H, dim, rd, r, HDp, t32(w), 1e-5, cos, sin, rd, interleaved, ctx, pages, k_cache)
    assert int(ctx.status.item()) == 0
    pos = np.arange(start, start + T)
    pairing = "interleaved" if interleaved else "half"
    c = plain.rms_unit(d[:, :r], 1e-5) * w
    kr = plain.rotate(d[:, None, r:], pos, rot, pairing)[:, 0] if rd else d[:, r:]
    rows = np.concatenate([c, kr, np.zeros((T, HDp - r - rd))], 1)
    got = torch.stack([k_cache[[5, 2, 7][ps // 64], 0, ps % 64] for ps in pos]).cpu().numpy()
    assert rel(rows, got) < 1e-5
    # nothing else was written: the rows before position 60 of the first page, those after 129 of the last, other pages
    assert float(k_cache[5, 0, :60].min()) == 9.0 and float(k_cache[7, 0, 2:].min()) == 9.0 and float(k_cache[0].min()) == 9.0
    qr = plain.rotate(q.reshape(T, H, dim + rd)[..., dim:], pos, rot, pairing) if rd else np.zeros((T, H, 0))
    qo = q_out[:T].view(T, H, HDp).cpu().numpy()
    assert rel(qr, qo[..., r:r + rd]) < 1e-5 if rd else True
    assert np.all(qo[..., r + rd:] == 0) and np.all(qo[..., :r] == 9.0) and np.all(q_out[T:].cpu().numpy() == 9.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,n_in,n_out,aligned", [(70, 3, 16, 40, True), (1, 1, 6, 13, False), (130, 5, 100, 70, False),
                                                    (9, 2, 64, 150, True), (200, 3, 96, 96, True)])
def test_head_linear(dtype, T, H, n_in, n_out, aligned):
    from mynah_slm_b200.ops import kernels
    rng = np.random.default_rng(T + n_in)
    # aligned: heads start at multiples of 8 values (what the tensor-core form needs in bfloat16); else anywhere
    head_in, in_off, head_out, out_off = (n_in + 8, 8, n_out + 9, 2) if aligned else (n_in + 5, 3, n_out + 9, 2)
    x = torch.tensor(rng.normal(size=(T, H * head_in)), dtype=dtype, device=DEV)
    W = torch.tensor(rng.normal(size=(H, n_out, n_in)), dtype=dtype, device=DEV)
    out = torch.full((T, H * head_out), 7.0, dtype=dtype, device=DEV)
    kernels.head_linear(x, head_in, in_off, W, out, head_out, out_off)
    xs = x.double().cpu().numpy().reshape(T, H, head_in)[..., in_off:in_off + n_in]
    ref = np.einsum("thi,hji->thj", xs, W.double().cpu().numpy())
    got = out.double().cpu().numpy().reshape(T, H, head_out)
    assert rel(ref, got[..., out_off:out_off + n_out]) < (1e-5 if dtype == torch.float32 else 1e-2)
    assert np.all(got[..., :out_off] == 7.0) and np.all(got[..., out_off + n_out:] == 7.0)
    if dtype == torch.bfloat16 and aligned:
        before = kernels.head_linear_plain(True)
        try:
            out2 = torch.full((T, H * head_out), 7.0, dtype=dtype, device=DEV)
            kernels.head_linear(x, head_in, in_off, W, out2, head_out, out_off)
        finally:
            kernels.head_linear_plain(before)
        assert rel(out2.double().cpu().numpy(), out.double().cpu().numpy()) < 1e-2
        # a row's bits in a small step (16-row tiles) and in a large one (64-row tiles)
        few = torch.full((3, H * head_out), 7.0, dtype=dtype, device=DEV)
        kernels.head_linear(x[:3].contiguous(), head_in, in_off, W, few, head_out, out_off)
        assert torch.equal(few, out[:3])


def plain_retention_core(q, k, v, decay, S0=None):
    T, H, dim = q.shape
    vd = v.shape[-1]
    o = np.zeros((T, H, vd))
    S = np.zeros((H, dim, vd)) if S0 is None else S0.copy()
    for t in range(T):
        for h in range(H):
            S[h] = decay[h] * S[h] + np.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    return o, S


@pytest.mark.parametrize("H,dim,vd,rot", [(3, 16, 24, 16), (1, 33, 5, 6), (2, 128, 64, 0), (2, 300, 12, 64), (2, 256, 40, 64),
                                          (4, 32, 70, 32), (2, 64, 32, 64), (1, 96, 24, 32), (2, 160, 16, 0), (1, 192, 8, 64)])
def test_retention_prep_and_scan(H, dim, vd, rot):
    from mynah_slm_b200.ops import kernels
    from mynah_slm_b200.parts.position import rotary_frequencies
    rng = np.random.default_rng(dim + vd)
    decay = rng.uniform(0.8, 1.0, size=H)
    na, nb = 71, 9
    cos = sin = None
    rotd = {"dims": rot, "base": 50.0} if rot else None
    if rot:
        f, mult = rotary_frequencies(rot, 50.0, None)
        cos, sin = kernels.rope_table_freqs(128, f, mult, DEV)
    raw = {s: (rng.normal(size=(n, H, dim)), rng.normal(size=(n, H, dim)), rng.normal(size=(n, H, vd))) for s, n in (("a", na), ("b", nb))}
    ref = {}
    for s, (q, k, v) in raw.items():
        pos = np.arange(len(q))
        ref[s] = plain_retention_core(plain.rotate(q, pos, rotd, "half"), plain.rotate(k, pos, rotd, "half") * dim ** -0.5, v, decay)
    state = torch.zeros((5, H, dim, vd), dtype=torch.float32, device=DEV)
    state[2] = 5.0                                              # another sequence's slot: must stay as it is
    got = {"a": [], "b": []}
    at = {"a": 0, "b": 0}
    # a in slot 3, b in slot 1: a prompt step of both with padding rows, pieces, then single rows
    for (n_a, n_b), pad in [((40, 5), 2), ((2, 1), 0), ((27, 1), 3), ((1, 1), 0), ((1, 1), 1)]:
        parts = []
        for s, n in (("a", n_a), ("b", n_b)):
            q, k, v = (x[at[s]:at[s] + n].reshape(n, -1) for x in raw[s])
            parts.append(np.concatenate([q, k, v], 1))
        p = t32(np.concatenate(parts + [np.zeros((pad, parts[0].shape[1]))], 0))
        ctx = ctx_for([n_a, n_b], [3, 1], starts=[at["a"], at["b"]], pad_rows=pad)
        qn, kn = kernels.retention_prep(p, 0, H * dim, H, dim, cos, sin, rot, False, dim ** -0.5, ctx)
        o = kernels.retention_scan(qn, kn, p, 2 * H * dim, t32(decay), state, ctx, H, dim, vd).cpu().numpy()
        got["a"].append(o[:n_a])
        got["b"].append(o[n_a:n_a + n_b])
        at["a"] += n_a
        at["b"] += n_b
        assert int(ctx.status.item()) == 0
    assert (at["a"], at["b"]) == (na, nb)
    for s, slot in (("a", 3), ("b", 1)):
        assert rel(ref[s][0].reshape(len(raw[s][0]), -1), np.concatenate(got[s])) < 2e-5
        assert rel(ref[s][1], state[slot].cpu().numpy()) < 2e-5
    assert float(state[2].min()) == 5.0 and float(state[2].max()) == 5.0 and float(state[0].abs().max()) == 0.0
    # the two forms of the recurrence (chunk by chunk, token by token) on one long piece from a non-zero state
    q, k, v = raw["a"]
    p = t32(np.concatenate([x.reshape(na, -1) for x in (q, k, v)], 1))
    ctx = ctx_for([na], [3])
    qn, kn = kernels.retention_prep(p, 0, H * dim, H, dim, cos, sin, rot, False, dim ** -0.5, ctx)
    outs = []
    for chunk_min in (16, 0):
        before = kernels.retention_chunk_min(chunk_min)
        try:
            st = state.clone()
            outs.append((kernels.retention_scan(qn, kn, p, 2 * H * dim, t32(decay), st, ctx, H, dim, vd).cpu().numpy(), st[3].cpu().numpy()))
        finally:
            kernels.retention_chunk_min(before)
    assert rel(outs[1][0], outs[0][0]) < 2e-5 and rel(outs[1][1], outs[0][1]) < 2e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,D,F,E,top", [(150, 48, 56, 9, 2), (5, 40, 12, 1, 1), (3, 64, 20, 7, 7), (400, 96, 200, 70, 4),
                                        (700, 128, 320, 5, 2)])
def test_table_routed_experts(dtype, T, D, F, E, top):
    from mynah_slm_b200.ops import kernels
    rng = np.random.default_rng(T + E)
    V, limit = 50, 1.3
    table = np.stack([rng.permutation(E)[:top] for _ in range(V)])
    toks = rng.integers(0, V, size=T)
    rnd = lambda *s: torch.tensor(rng.normal(size=s), dtype=dtype)
    h = rnd(T, D)
    W = {"table": table}
    for e in range(E):
        W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"] = rnd(F, D) / D ** 0.5 * 2, rnd(F, D) / D ** 0.5 * 2, rnd(D, F) / F ** 0.5
    mlp = {"router": {"top": top, "experts": E}, "expert": {"limit": limit, "ff": F}}
    ref = plain.routed_mlp(h.double().numpy(), toks, {k: (v.double().numpy() if torch.is_tensor(v) else v) for k, v in W.items()}, "", mlp)
    w_gu = torch.stack([torch.stack([W[f"e{e}.gate"], W[f"e{e}.up"]]) for e in range(E)]).to(DEV).contiguous()
    w_down = torch.stack([W[f"e{e}.down"] for e in range(E)]).to(DEV).contiguous()
    pad = 3
    ctx = ctx_for([T], [0], pad_rows=pad, tokens=list(toks) + [V + 5] * pad)        # padding rows may hold anything
    hp = torch.cat([h, torch.ones((pad, D), dtype=dtype)], 0).to(DEV).contiguous()
    out = kernels.moe_table_ffn(hp, i32(table), w_gu, w_down, ctx, top, limit, 1.702).float().cpu().numpy()
    assert int(ctx.status.item()) == 0
    assert rel(ref, out[:T]) < (2e-5 if dtype == torch.float32 else 3e-2) and np.all(out[T:] == 0)
    if dtype == torch.bfloat16:
        # three routes to one result: grouped tcgen05 products (large steps), mma.sync tile by tile, plain tiles
        before = kernels.moe_grouped_min(0)
        try:
            tiled = kernels.moe_table_ffn(hp, i32(table), w_gu, w_down, ctx, top, limit, 1.702).float().cpu().numpy()
            few = ctx_for([2], [0], tokens=list(toks[:2]))
            small = kernels.moe_table_ffn(hp[:2].contiguous(), i32(table), w_gu, w_down, few, top, limit, 1.702).float().cpu().numpy()
        finally:
            kernels.moe_grouped_min(before)
        assert rel(tiled[:T], out[:T]) < 2e-2 and np.all(tiled[T:] == 0)
        assert np.array_equal(small, tiled[:2])            # a row's bits in a 16-row tile and in a 64-row tile
        before = kernels.moe_plain(True)
        try:
            plain_out = kernels.moe_table_ffn(hp, i32(table), w_gu, w_down, ctx, top, limit, 1.702).float().cpu().numpy()
        finally:
            kernels.moe_plain(before)
        assert rel(plain_out[:T], tiled[:T]) < 2e-2
    # an expert id outside the table's range is reported and skipped
    bad = table.copy()
    bad[toks[0], 0] = E
    kernels.moe_table_ffn(hp, i32(bad), w_gu, w_down, ctx, top, limit, 1.702)
    assert int(ctx.status.item()) & 4


def test_scaled_embedding_residual_norm_and_logits():
    from mynah_slm_b200.ops import kernels
    rng = np.random.default_rng(0)
    for D in (40, 256, 1000):
        table, toks = rng.normal(size=(30, D)), rng.integers(0, 30, size=9)
        x = kernels.embed_gather(t32(table), i32(toks), scale=3.5).cpu().numpy()
        assert rel(table[toks] * 3.5, x) < 1e-6
        xs, delta, w = rng.normal(size=(9, D)), rng.normal(size=(9, D)), 0.1 * rng.normal(size=(D,))
        xt = t32(xs)
        h = kernels.rmsnorm(xt, t32(1.0 + w), 1e-5, torch.float32, delta=t32(delta), delta_scale=0.7).cpu().numpy()
        assert rel(xs + 0.7 * delta, xt.cpu().numpy()) < 1e-6 and rel(plain.offset_norm(xs + 0.7 * delta, w, 1e-5), h) < 1e-5
        rows = i32([8, 0, 0])
        xt = t32(xs)
        h = kernels.rmsnorm(xt, t32(1.0 + w), 1e-5, torch.float32, delta=t32(delta), rows=rows, delta_scale=0.7).cpu().numpy()
        assert rel(plain.offset_norm((xs + 0.7 * delta)[[8, 0, 0]], w, 1e-5), h) < 1e-5 and np.array_equal(xt.cpu().numpy(), xs.astype(np.float32))
        xt = t32(xs)
        kernels.residual_add(xt, t32(delta), 0.25)
        assert rel(xs + 0.25 * delta, xt.cpu().numpy()) < 1e-6
        z = t32(xs)
        assert rel(np.maximum(xs, 0) ** 2, kernels.activation(z, "relu2").cpu().numpy()) < 1e-6
        assert rel(xs * 0.3, kernels.scale_(t32(xs), 0.3).cpu().numpy()) < 1e-6
