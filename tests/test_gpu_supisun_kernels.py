"""The kernels behind the Supisun parts, each alone, against the plain functions of tests/plain/supisun.py (float64):
the causal convolution with its tail state (whole, in pieces, one row a step, two sequences, padding rows), the two
layer norms, the activations, the selective scan in one pass and in two, the delta rule, the gated norm. Sizes that
take the vector forms and sizes that do not."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from plain import supisun as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ctx_for(q_lens, slots, pad_rows=0, decode=False):
    """The fields of a step's context that the kernels read: rows packed sequence by sequence, then padding rows."""
    tok_seq, cu = [], [0]
    for b, n in enumerate(q_lens):
        tok_seq += [b] * n
        cu.append(cu[-1] + n)
    tok_seq += [-1] * pad_rows
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return SimpleNamespace(tok_seq=i32(tok_seq), cu_q=i32(cu), slots=i32(slots), B=len(q_lens), T=len(tok_seq),
                           is_decode=decode, max_q_len=max(q_lens))


def t32(a):
    return torch.tensor(np.asarray(a), dtype=torch.float32, device=DEV)


def rel(ref, got):
    ref, got = np.asarray(ref, dtype=np.float64), np.asarray(got, dtype=np.float64)
    return float(np.abs(ref - got).max() / max(np.abs(ref).max(), 1e-30))


@pytest.mark.parametrize("C,taps", [(64, 4), (40, 3), (36, 6), (24, 1), (16, 2)])
def test_causal_conv_pieces_and_state(C, taps):
    from mynah_slm_b200.ops import kernels
    rng = np.random.default_rng(C + taps)
    xa, xb = rng.normal(size=(71, C)), rng.normal(size=(9, C))
    w, bias = rng.normal(size=(C, taps)), rng.normal(size=(C,))
    silu = lambda v: v / (1 + np.exp(-v))
    ref_a, ref_b = silu(plain.causal_conv(xa, w, bias)), silu(plain.causal_conv(xb, w, bias))
    state = torch.zeros((5, max(taps - 1, 0), C), dtype=torch.float32, device=DEV) if taps > 1 else None
    got_a, got_b = [], []
    # sequence a in slot 3, b in slot 1: a prompt step of both (with padding rows), pieces, then single rows
    plan = [((40, 5), 2, False), ((2, 1), 0, False), ((27, 1), 3, False)] + [((1, 1), 0, True)] * 2
    at_a = at_b = 0
    for (na, nb), pad, dec in plan:
        x = np.concatenate([xa[at_a:at_a + na], xb[at_b:at_b + nb], np.zeros((pad, C))], 0)
        ctx = ctx_for([na, nb], [3, 1], pad, dec)
        out = kernels.causal_conv(t32(x), t32(w), t32(bias), state, ctx, torch.float32, act="silu").cpu().numpy()
        got_a.append(out[:na])
        got_b.append(out[na:na + nb])
        assert np.all(out[na + nb:] == 0)
        at_a, at_b = at_a + na, at_b + nb
    assert (at_a, at_b) == (71, 9)
    assert rel(ref_a, np.concatenate(got_a)) < 1e-5 and rel(ref_b, np.concatenate(got_b)) < 1e-5
    # x + conv(x) without bias or activation, bfloat16 out
    ctx = ctx_for([71], [0])
    if state is not None:
        state.zero_()
    out = kernels.causal_conv(t32(xa), t32(w), None, state, ctx, torch.bfloat16, add_input=True).float().cpu().numpy()
    assert rel(xa + plain.causal_conv(xa, w), out) < 1e-2


@pytest.mark.parametrize("D", [256, 100, 8200])
def test_layer_norms(D):
    from mynah_slm_b200.ops import kernels
    rng = np.random.default_rng(D)
    x, y = rng.normal(size=(7, D)), 3.0 + 2.0 * rng.normal(size=(7, D))
    w, b = rng.normal(size=(D,)), rng.normal(size=(D,))
    rows = torch.tensor([6, 0, 0, 3], dtype=torch.int32, device=DEV)
    got = kernels.layernorm_rows(t32(x), t32(w), t32(b), 1e-5, torch.float32, rows=rows).cpu().numpy()
    assert rel(plain.layer_norm(x[[6, 0, 0, 3]], w, b, 1e-5), got) < 1e-5
    xs = t32(x)
    copy = kernels.layernorm_add(xs, t32(y), t32(w), t32(b), 1e-5, copy=True)
    ref = x + plain.layer_norm(y, w, b, 1e-5)
    assert rel(ref, xs.cpu().numpy()) < 1e-5 and rel(ref, copy.cpu().numpy()) < 1e-5
    # a constant row: zero variance
    xs = torch.zeros((1, D), dtype=torch.float32, device=DEV)
    kernels.layernorm_add(xs, torch.full((1, D), 2.5, dtype=torch.float32, device=DEV), t32(w), t32(b), 1e-5)
    assert rel(b[None, :], xs.cpu().numpy()) < 1e-5


def test_activations():
    from mynah_slm_b200.ops import kernels
    z = np.linspace(-6, 6, 1003)
    tanh_form = 0.5 * z * (1 + np.tanh(np.sqrt(2 / np.pi) * (z + 0.044715 * z ** 3)))
    for name, ref in (("gelu_erf", plain.gelu_erf(z)), ("gelu_tanh", tanh_form), ("silu", plain.silu(z)), ("relu", np.maximum(z, 0))):
        assert rel(ref, kernels.activation(t32(z), name).cpu().numpy()) < 1e-6, name
    z8 = z[:1000].reshape(10, 100)
    assert rel(plain.gelu_erf(z8), kernels.activation(t32(z8), "gelu_erf").cpu().numpy()) < 1e-6
    assert np.abs(plain.gelu_erf(z) - tanh_form).max() > 1e-4          # the two forms are told apart at this tolerance


@pytest.mark.parametrize("inner,N,piece", [(64, 16, 0), (64, 16, 32), (40, 5, 16), (24, 130, 0)])
def test_selective_scan(inner, N, piece):
    from mynah_slm_b200.ops import kernels
    rng = np.random.default_rng(inner + N)
    lens = [150, 37]
    T = sum(lens)
    x, z, dt = rng.normal(size=(T, inner)), rng.normal(size=(T, inner)), rng.normal(size=(T, inner))
    bc = rng.normal(size=(T, 2 * N))
    A_log, D, bias = rng.normal(0, 0.5, (inner, N)), rng.normal(size=inner), rng.normal(size=inner)
    state = torch.zeros((4, inner, N), dtype=torch.float32, device=DEV)
    ctx = ctx_for(lens, [2, 0])
    before = kernels.SCAN_PIECE_ROWS
    kernels.SCAN_PIECE_ROWS = piece
    try:
        bct = t32(bc)
        y = kernels.selective_scan(t32(x), t32(z), t32(dt), bct[:, :N], bct[:, N:], t32(bias), t32(A_log), t32(D), state, ctx)
    finally:
        kernels.SCAN_PIECE_ROWS = before
    A = -np.exp(A_log)
    at = 0
    for n, slot in zip(lens, (2, 0)):
        S = np.zeros((inner, N))
        ref = np.zeros((n, inner))
        for t in range(at, at + n):
            d = plain.softplus(dt[t] + bias)
            S = np.exp(d[:, None] * A) * S + (d * x[t])[:, None] * bc[t, :N][None, :]
            ref[t - at] = (S @ bc[t, N:] + D * x[t]) * plain.silu(z[t])
        assert rel(ref, y[at:at + n].cpu().numpy()) < 2e-5
        assert rel(S, state[slot].cpu().numpy()) < 2e-5
        at += n
    assert float(state[1].abs().max()) == 0 and float(state[3].abs().max()) == 0


@pytest.mark.parametrize("H,G,dim,vd", [(4, 2, 64, 32), (3, 3, 12, 20), (2, 1, 136, 8), (2, 2, 30, 7)])
def test_delta_rule_and_gated_norm(H, G, dim, vd):
    from mynah_slm_b200.ops import kernels
    rng = np.random.default_rng(dim)
    lens = [45, 3, 33]
    T = sum(lens)
    unit = lambda a: a / np.sqrt((a * a).sum(-1, keepdims=True) + 1e-6)
    qn = unit(rng.normal(size=(T, G, dim))) * dim ** -0.5
    kn = unit(rng.normal(size=(T, G, dim)))
    v = rng.normal(size=(T, H, vd))
    g, beta = rng.uniform(0.5, 1.0, (T, H)), rng.uniform(0.1, 0.9, (T, H))
    state = t32(0.3 * rng.normal(size=(5, H, dim, vd)))          # the sequences go on from states that are not zero; the last row is no slot's
    state0 = state.cpu().numpy().copy()
    slots = [1, 0, 3][:len(lens)]
    ctx = ctx_for(lens, slots)
    o = kernels.delta_rule(t32(qn.reshape(T, -1)), t32(kn.reshape(T, -1)), t32(v.reshape(T, -1)), t32(g), t32(beta), state,
                           ctx, H, G, dim, vd).cpu().numpy().reshape(T, H, vd)
    at = 0
    for n, slot in zip(lens, slots):
        for h in range(H):
            S = state0[slot, h].astype(np.float64)
            for t in range(at, at + n):
                kk, qq = kn[t, h // (H // G)], qn[t, h // (H // G)]
                S = g[t, h] * S
                S = S + np.outer(kk, beta[t, h] * (v[t, h] - S.T @ kk))
                assert rel(S.T @ qq, o[t, h]) < 2e-5
            assert rel(S, state[slot, h].cpu().numpy()) < 2e-5
        at += n
    gate, w = rng.normal(size=(T, H * vd)), rng.normal(size=vd)
    got = kernels.gated_rmsnorm(t32(o.reshape(T, -1)), t32(gate), t32(w), H, vd, 1e-5).cpu().numpy()
    ref = plain.rms_unit(o, 1e-5) * w * plain.silu(gate).reshape(T, H, vd)
    assert rel(ref.reshape(T, -1), got) < 1e-5
