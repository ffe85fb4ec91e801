"""The Gulipel decoder on the GPU against the plain implementation (plain_gulipel.py): every mechanism alone
through its kernel, then whole models through the step function, the replay program and the generation entry
point - whole prompts, token-by-token decoding, portions down to two tokens, unequal batches, pages and state
slots that are used again, far memories, the first tokens of a sequence, the steps of the query temperature."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import plain_gulipel as plain
from gulipel_models import TINY_G, make_folder, prompts
from helpers import build_all_modes, replay_in_process, run_trace

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F64 = torch.float64


def _k():
    from xinfer_b200 import kernels
    return kernels


def _err():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def _rand(*shape, seed=0, scale=1.0):
    return torch.randn(tuple(shape), generator=torch.Generator().manual_seed(seed), dtype=F64) * scale


def _close(got, want, tol):
    got, want = got.double().cpu(), want.double()
    assert got.shape == want.shape
    assert (got - want).abs().max() <= tol * (1 + want.abs().max()), float((got - want).abs().max())


def _steps_of(cuts):
    """cuts[r] = the portion sizes of request r -> a list of steps, each a list of (request, start, count): the
    requests advance side by side, one portion each per step, in changing order."""
    at = [0] * len(cuts)
    idx = [0] * len(cuts)
    steps = []
    while any(i < len(c) for i, c in zip(idx, cuts)):
        step = []
        order = list(range(len(cuts)))
        if len(steps) % 2:
            order.reverse()
        for r in order:
            if idx[r] < len(cuts[r]):
                n = cuts[r][idx[r]]
                step.append((r, at[r], n))
                at[r] += n
                idx[r] += 1
        steps.append(step)
    return steps


def _meta(step, slots):
    counts = [n for _, _, n in step]
    q_start = np.concatenate([[0], np.cumsum(counts)])
    req = np.concatenate([np.full(n, b) for b, n in enumerate(counts)])
    pos = np.concatenate([np.arange(s, s + n) for _, s, n in step])
    return _i32(q_start), _i32(req), _i32(pos), _i32([slots[r] for r, _, _ in step])


# ---------------------------------------------------------------------------------------------
# the RMS norm and the residual arithmetic it takes in
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("branch_dtype,out_dtype", [(None, torch.bfloat16), (torch.float32, torch.float32),
                                                    (torch.bfloat16, torch.bfloat16), (torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("branch_norm,gain", [(False, False), (True, False), (True, True)])
@pytest.mark.parametrize("rows,dim", [(37, 48), (5, 1030), (130, 52)])
def test_norm_chain_with_normed_and_scaled_branch(branch_dtype, out_dtype, branch_norm, gain, rows, dim):
    if branch_dtype is None and (branch_norm or gain):
        pytest.skip("no branch")
    k = _k()
    eps, beps = 3e-6, 2e-5
    x = _rand(rows, dim, seed=1, scale=2.0).float()
    br = _rand(rows, dim, seed=2, scale=3.0).to(branch_dtype) if branch_dtype is not None else None
    w, bw, g = _rand(dim, seed=3).float(), _rand(dim, seed=4).float(), _rand(dim, seed=5).float()
    s = x.double()
    if br is not None:
        v = br.double()
        if branch_norm:
            v = plain.rms_norm(v, bw.double(), beps)
        if gain:
            v = v * g.double()
        s = s + v
    want = plain.rms_norm(s, w.double(), eps)
    out = torch.full((rows, dim), float("nan"), dtype=out_dtype, device=DEV)
    xd, err = x.to(DEV), _err()
    k.rms_chain(out, xd, w.to(DEV), eps, err, branch=br.to(DEV) if br is not None else None,
                branch_weight=bw.to(DEV) if branch_norm else None, branch_eps=beps, gain=g.to(DEV) if gain else None,
                sum_out=xd if br is not None else None)
    assert int(err.item()) == 0
    _close(out, want, 2e-5 if out_dtype == torch.float32 else 1e-2)
    _close(xd, s, 1e-6)                                  # the stream itself stays float32
    only = x.to(DEV)
    if br is not None:                                   # no norm behind the sum: the sum alone
        k.rms_chain(None, only, None, eps, err, branch=br.to(DEV), branch_weight=bw.to(DEV) if branch_norm else None,
                    branch_eps=beps, gain=g.to(DEV) if gain else None, sum_out=only)
        _close(only, s, 1e-6)


def test_norm_chain_gathers_rows():
    k = _k()
    x, w = _rand(9, 40, seed=1).float(), _rand(40, seed=2).float()
    out, err = torch.zeros(3, 40, device=DEV), _err()
    k.rms_chain(out, x.to(DEV), w.to(DEV), 1e-5, err, rows=_i32([7, 0, 4]))
    assert int(err.item()) == 0
    _close(out, plain.rms_norm(x.double()[[7, 0, 4]], w.double(), 1e-5), 1e-5)
    k.rms_chain(out, x.to(DEV), w.to(DEV), 1e-5, err, rows=_i32([7, 9, 4]))
    assert int(err.item()) != 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,dim", [(3, 48), (70, 1000), (33, 52)])
def test_two_normed_sides_are_averaged(dtype, T, dim):
    k = _k()
    a, b = _rand(T, dim, seed=1, scale=4.0).to(dtype), _rand(T, dim, seed=2, scale=0.1).to(dtype)
    wa, wb = _rand(dim, seed=3).float(), _rand(dim, seed=4).float()
    out = torch.empty(T, dim, dtype=dtype, device=DEV)
    k.dual_rms_sum(out, a.to(DEV), b.to(DEV), wa.to(DEV), wb.to(DEV), 1e-5, 0.5, 0.25)
    want = 0.5 * plain.rms_norm(a.double(), wa.double(), 1e-5) + 0.25 * plain.rms_norm(b.double(), wb.double(), 1e-5)
    _close(out, want, 1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,inter", [(3, 40), (70, 136), (300, 50)])
def test_gated_feed_forward_activation_with_biases(dtype, T, inter):
    k = _k()
    gu, b = _rand(T, 2 * inter, seed=T, scale=2.0).to(dtype), _rand(2 * inter, seed=7).float()
    out = torch.empty(T, inter, dtype=dtype, device=DEV)
    k.swiglu_bias(out, gu.to(DEV), b.to(DEV))
    z = gu.double() + b.double()
    _close(out, plain.silu(z[:, :inter]) * z[:, inter:], 1e-5 if dtype == torch.float32 else 1e-2)
    x = _rand(T, inter, seed=3).to(dtype).to(DEV)
    want = x.double().cpu() + b.double()[:inter]
    k.add_bias(x, b[:inter].contiguous().to(DEV))
    _close(x, want, 1e-6 if dtype == torch.float32 else 1e-2)


# ---------------------------------------------------------------------------------------------
# the embedding's three terms; the token before is part of a request's state
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rule", [(53, 31, 7), (1, 5, 9), (7, 0, 1), (101, 3, 1000003)])
def test_embedding_sum_carries_the_token_before_across_steps(dtype, rule):
    """Three requests in portions (one of them a single token long, one decoded one by one); the row of the pair
    table is the last one at position 0 only, and the token before a step's first one comes from the slot's state."""
    k = _k()
    V, H = 97, 40
    buckets, mp, mc = rule
    emb = dict(scale=3.0, bigram=dict(buckets=buckets, mul_prev=mp, mul_cur=mc))
    table, pair, pos = (_rand(V, H, seed=1).to(dtype), _rand(buckets + 1, H, seed=2).to(dtype),
                        _rand(64, H, seed=3).to(dtype))
    w = {"embed": table.double(), "bigram": pair.double(), "pos": pos.double()}
    toks = [torch.randint(0, V, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (23, 1, 9)]
    toks[0][5] = toks[0][4]                              # a pair of equal tokens
    want = [plain.embed(dict(embedding=emb), w, t) for t in toks]
    slots = [2, 0, 3]
    prev = torch.full((4,), -7, dtype=torch.int32, device=DEV)    # what an earlier request left in the slots
    got = [torch.zeros(len(t), H, dtype=F64) for t in toks]
    err = _err()
    for step in _steps_of([[5, 2, 1, 1, 14], [1], [1] * 9]):
        q_start, req, positions, sl = _meta(step, slots)
        ids = _i32(sum((toks[r][s:s + n] for r, s, n in step), []))
        out = torch.full((ids.numel(), H), float("nan"), device=DEV)
        k.embed_sum(out, table.to(DEV), ids, err, scale=emb["scale"], pair=pair.to(DEV), pair_rule=rule, pos_table=pos.to(DEV),
                    positions=positions, req_of_token=req, q_start=q_start, slots=sl, prev_state=prev)
        k.prev_store(prev, ids, None, q_start, sl, len(step))
        at = 0
        for r, s, n in step:
            got[r][s:s + n] = out[at:at + n].double().cpu()
            at += n
    assert int(err.item()) == 0
    for g, wnt in zip(got, want):
        _close(g, wnt, 1e-6)
    assert prev.cpu().tolist() == [toks[1][-1], -7, toks[0][-1], toks[2][-1]]


def test_embedding_sum_flags_bad_ids_and_positions():
    k = _k()
    table, pos = _rand(10, 8, seed=1).float().to(DEV), _rand(4, 8, seed=2).float().to(DEV)
    out = torch.zeros(2, 8, device=DEV)
    for ids, positions in (([3, 10], [0, 1]), ([3, 4], [3, 4])):
        err = _err()
        k.embed_sum(out, table, _i32(ids), err, pos_table=pos, positions=_i32(positions), req_of_token=_i32([0, 0]),
                    q_start=_i32([0, 2]), slots=_i32([0]))
        assert int(err.item()) != 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_gate_reads_the_layers_own_columns(dtype):
    k = _k()
    T, V, dim, cols, col0 = 50, 31, 6, 20, 12
    u, table = _rand(T, dim, seed=1, scale=2.0).to(dtype), _rand(V, cols, seed=2).to(dtype)
    ids = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(3))
    out, err = torch.empty(T, dim, dtype=dtype, device=DEV), _err()
    k.token_gate(out, u.to(DEV), table.to(DEV), col0, _i32(ids.tolist()), None, _i32([0] * T), err)
    assert int(err.item()) == 0
    _close(out, plain.gelu_tanh(u.double()) * table.double()[ids, col0:col0 + dim], 1e-5 if dtype == torch.float32 else 1e-2)


# ---------------------------------------------------------------------------------------------
# short convolutions whose last inputs are carried per request
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("K,bias", [(1, False), (2, True), (3, False), (4, True), (5, True), (9, False)])
def test_short_convolution_over_portions_and_batches(K, bias):
    """Portions shorter than the taps (one and two tokens), first tokens (nothing but zeros behind them), requests side
    by side, slots that held another request's inputs."""
    k = _k()
    C, off, width = 45, 7, 60
    lens = [31, 2, 12]
    taps, b = _rand(C, K, seed=1).float(), _rand(C, seed=2).float() if bias else None
    us = [_rand(n, width, seed=10 + n).float() for n in lens]
    want = [plain.silu(plain.causal_conv(u.double()[:, off:off + C], taps.double(), b.double() if bias else None)) for u in us]
    slots = [1, 3, 0]
    state = torch.full((4, max(K - 1, 1), C), float("nan"), device=DEV) if K > 1 else None
    if K > 1:
        state[slots] = 0.0                                # a request's row is cleared when it opens
    got = [torch.zeros(n, C, dtype=F64) for n in lens]
    for step in _steps_of([[1, 1, 2, 9, 1, 17], [2], [5, 7]]):
        q_start, req, _, sl = _meta(step, slots)
        u = torch.cat([us[r][s:s + n] for r, s, n in step]).to(DEV)
        y = torch.full((u.shape[0], C), float("nan"), device=DEV)
        k.conv_silu(y, u, off, taps.to(DEV), b.to(DEV) if bias else None, state, req, q_start, sl, len(step))
        at = 0
        for r, s, n in step:
            got[r][s:s + n] = y[at:at + n].double().cpu()
            at += n
    for g, wnt in zip(got, want):
        _close(g, wnt, 1e-5)
    if K > 1:                                             # the state holds the last K-1 inputs, oldest first
        for r, sl in enumerate(slots):
            tail = torch.cat([torch.zeros(K - 1, C), us[r][:, off:off + C]])[-(K - 1):]
            _close(state[sl], tail, 1e-6)
        assert torch.isnan(state[2]).all()                # a slot of no request is not touched


@pytest.mark.parametrize("C,off,width", [(48, 8, 64), (45, 7, 60), (130, 0, 130)])
@pytest.mark.parametrize("K", [2, 4, 8])
def test_short_convolution_over_long_runs_of_tokens(K, C, off, width):
    """Thousands of tokens in a step, so that a thread walks a run of tokens with the inputs before it in registers:
    runs that start in the middle of a request, runs that cross from one request into the next one's first tokens,
    a portion that ends inside a run, channels in fours and one by one; the same numbers as a step of few tokens."""
    k = _k()
    lens = [3011, 1702, 95]
    taps, b = _rand(C, K, seed=3).float(), _rand(C, seed=4).float()
    us = [_rand(n, width, seed=20 + n).float() for n in lens]
    want = [plain.silu(plain.causal_conv(u.double()[:, off:off + C], taps.double(), b.double())) for u in us]
    slots = [2, 0, 1]
    state = torch.zeros((3, K - 1, C), device=DEV)
    got = [torch.zeros(n, C, dtype=F64) for n in lens]
    for step in _steps_of([[2990, 21], [1702], [3, 92]]):
        q_start, req, _, sl = _meta(step, slots)
        u = torch.cat([us[r][s:s + n] for r, s, n in step]).to(DEV)
        y = torch.full((u.shape[0], C), float("nan"), device=DEV)
        k.conv_silu(y, u, off, taps.to(DEV), b.to(DEV), state, req, q_start, sl, len(step))
        at = 0
        for r, s, n in step:
            got[r][s:s + n] = y[at:at + n].double().cpu()
            at += n
    for g, wnt in zip(got, want):
        _close(g, wnt, 1e-5)
    # a short step of the same tokens gives the same bits: the taps are added in one order
    q_start, req, _, sl = _meta([(2, 0, 40)], slots)
    y_short = torch.empty(40, C, device=DEV)
    k.conv_silu(y_short, us[2][:40].to(DEV), off, taps.to(DEV), b.to(DEV), torch.zeros_like(state), req, q_start, sl, 1)
    assert torch.equal(y_short.double().cpu(), got[2][:40])


# ---------------------------------------------------------------------------------------------
# the state-space scan
# ---------------------------------------------------------------------------------------------
def _scan_inputs(lens, H, P, N, G, seed):
    out = []
    for i, n in enumerate(lens):
        out.append(dict(x=_rand(n, H, P, seed=seed + i), B=_rand(n, G, N, seed=seed + 50 + i), C=_rand(n, G, N, seed=seed + 90 + i),
                        dt=_rand(n, H, seed=seed + 130 + i, scale=2.0)))
    return out


def _run_scan(ins, cuts, slots, H, P, N, G, dt_bias, a_log, d_skip, state):
    k = _k()
    inner, gn = H * P, G * N
    got = [torch.zeros(i["x"].shape[0], inner, dtype=F64) for i in ins]
    for step in _steps_of(cuts):
        q_start, _, _, sl = _meta(step, slots)
        xbc = torch.cat([torch.cat([ins[r]["x"][s:s + n].reshape(n, inner), ins[r]["B"][s:s + n].reshape(n, gn),
                                    ins[r]["C"][s:s + n].reshape(n, gn)], dim=1) for r, s, n in step]).float().to(DEV)
        # the step sizes sit behind other columns of a wider row
        proj = torch.cat([torch.cat([torch.full((n, 3), float("nan"), dtype=F64), ins[r]["dt"][s:s + n]], dim=1)
                          for r, s, n in step]).float().to(DEV)
        y = torch.full((xbc.shape[0], inner), float("nan"), device=DEV)
        k.selective_scan(y, xbc, proj, 3, dt_bias.float().to(DEV), a_log.float().to(DEV), d_skip.float().to(DEV), state, q_start, sl,
                         len(step), H, P, N, G)
        at = 0
        for r, s, n in step:
            got[r][s:s + n] = y[at:at + n].double().cpu()
            at += n
    return got


@pytest.mark.parametrize("H,P,N,G", [(3, 8, 5, 1), (4, 12, 24, 2), (6, 16, 16, 3), (2, 33, 40, 2), (8, 8, 8, 8), (2, 64, 128, 1),
                                     (5, 7, 9, 5), (1, 100, 3, 1), (2, 4, 130, 1)])
def test_state_space_scan_equals_plain_however_it_is_cut(H, P, N, G):
    lens = [40, 3, 17]
    ins = _scan_inputs(lens, H, P, N, G, seed=H * P)
    dt_bias, a_log, d_skip = _rand(H, seed=1), _rand(H, seed=2, scale=1.5), _rand(H, seed=3)
    want = []
    for i in ins:
        f = lambda t: t.float().double()                 # the kernel reads float32 inputs
        dt = F.softplus(f(i["dt"]) + f(dt_bias))
        want.append(plain.selective_scan(f(i["x"]), f(i["B"]).repeat_interleave(H // G, dim=1),
                                         f(i["C"]).repeat_interleave(H // G, dim=1), dt, torch.exp(f(a_log)), f(d_skip))
                    .reshape(-1, H * P))
    slots = [3, 1, 0]
    whole = _run_scan(ins, [[n] for n in lens], slots, H, P, N, G, dt_bias, a_log, d_skip, torch.zeros(4, H, N, P, device=DEV))
    state = torch.zeros(4, H, N, P, device=DEV)
    state[2] = float("nan")
    cut = _run_scan(ins, [[7, 1, 1, 2, 29], [1, 2], [1] * 17], slots, H, P, N, G, dt_bias, a_log, d_skip, state)
    for a, b, wnt in zip(whole, cut, want):
        _close(a, wnt, 2e-5)
        _close(b, wnt, 2e-5)
    assert torch.isnan(state[2]).all() and torch.isfinite(state[[0, 1, 3]]).all()


def test_state_space_scan_remembers_one_token_for_hundreds():
    """One head forgets nothing (a tiny decay rate) and another everything: a value written at token 3 under a key
    that no other token uses is read back 600 tokens later by the first head only - in one portion, and decoded
    token by token across many steps."""
    H, P, N, G, n = 2, 8, 16, 1, 620
    x, B, C = _rand(n, H, P, seed=1, scale=0.1), torch.zeros(n, G, N, dtype=F64), torch.zeros(n, G, N, dtype=F64)
    B[:, 0, 1:] = _rand(n, N - 1, seed=2)
    C[:, 0, 1:] = _rand(n, N - 1, seed=3, scale=0.01)
    B[3, 0, 0], x[3] = 1.0, 5.0                          # channel 0 of the state is written once
    C[610, 0] = 0.0
    C[610, 0, 0] = 1.0                                   # and read once, alone
    dt = torch.full((n, H), 0.5413, dtype=F64)           # softplus -> 1.0
    a_log = torch.tensor([-12.0, 3.0], dtype=F64)        # decays exp(-6e-6) and exp(-20) per token
    ins = [dict(x=x, B=B, C=C, dt=dt)]
    zero = torch.zeros(H, dtype=F64)
    f = lambda t: t.float().double()
    want = plain.selective_scan(f(x), f(B).repeat_interleave(H, dim=1), f(C).repeat_interleave(H, dim=1), F.softplus(f(dt)),
                                torch.exp(f(a_log)), zero)
    for cuts in ([[n]], [[590] + [1] * 30], [[2, 300, 5, 303, 10]]):
        got = _run_scan(ins, cuts, [0], H, P, N, G, zero, a_log, zero, torch.zeros(1, H, N, P, device=DEV))[0].view(n, H, P)
        _close(got, want, 2e-5)
        assert (got[610, 0] - 5.0).abs().max() < 0.05 and got[610, 1].abs().max() < 1e-6


# ---------------------------------------------------------------------------------------------
# the gated delta rule
# ---------------------------------------------------------------------------------------------
def _delta_inputs(lens, H, G, d, dv, seed):
    out = []
    for i, n in enumerate(lens):
        out.append(dict(q=_rand(n, G, d, seed=seed + i), k=_rand(n, G, d, seed=seed + 40 + i), v=_rand(n, H, dv, seed=seed + 80 + i),
                        b=_rand(n, H, seed=seed + 120 + i, scale=2.0), a=_rand(n, H, d, seed=seed + 160 + i, scale=2.0)))
    return out


def _delta_plain(i, H, G, d, dv, dt_bias, a_log, unit_eps=1e-6):
    f = lambda t: t.float().double()
    q, k = f(i["q"]), f(i["k"])
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + unit_eps) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)
    q, k = q.repeat_interleave(H // G, dim=1), k.repeat_interleave(H // G, dim=1)
    decay = torch.exp(-torch.exp(f(a_log))[None, :, None] * F.softplus(f(i["a"]) + f(dt_bias).view(1, H, d)))
    return plain.delta_rule(q, k, f(i["v"]), torch.sigmoid(f(i["b"])), decay).reshape(-1, H * dv)


def _run_delta(ins, cuts, slots, H, G, d, dv, dt_bias, a_log, state, unit_eps=1e-6):
    k = _k()
    got = [torch.zeros(i["q"].shape[0], H * dv, dtype=F64) for i in ins]
    for step in _steps_of(cuts):
        q_start, _, _, sl = _meta(step, slots)
        qkv = torch.cat([torch.cat([ins[r]["q"][s:s + n].reshape(n, G * d), ins[r]["k"][s:s + n].reshape(n, G * d),
                                    ins[r]["v"][s:s + n].reshape(n, H * dv)], dim=1) for r, s, n in step]).float().to(DEV)
        proj = torch.cat([torch.cat([torch.full((n, 5), float("nan"), dtype=F64), ins[r]["b"][s:s + n]], dim=1)
                          for r, s, n in step]).float().to(DEV)
        # the decay's pre-activations at the front of rows that hold something else behind them
        ag = torch.cat([torch.cat([ins[r]["a"][s:s + n].reshape(n, H * d), torch.full((n, 4), float("nan"), dtype=F64)], dim=1)
                        for r, s, n in step]).float().to(DEV)
        o = torch.full((qkv.shape[0], H * dv), float("nan"), device=DEV)
        k.delta_rule(o, qkv, proj, 5, ag, dt_bias.reshape(-1).float().to(DEV), a_log.float().to(DEV), state, q_start, sl, len(step),
                     H, G, d, dv, unit_eps)
        at = 0
        for r, s, n in step:
            got[r][s:s + n] = o[at:at + n].double().cpu()
            at += n
    return got


@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 16, 8), (6, 6, 24, 16), (2, 1, 40, 20), (1, 1, 64, 48), (8, 2, 8, 8), (2, 2, 128, 64),
                                      (3, 1, 5, 7), (2, 1, 130, 3), (1, 1, 3, 100)])
def test_delta_rule_equals_plain_however_it_is_cut(H, G, d, dv):
    lens = [40, 3, 17]
    ins = _delta_inputs(lens, H, G, d, dv, seed=H * d)
    dt_bias, a_log = _rand(H, d, seed=1), _rand(H, seed=2, scale=1.5)
    want = [_delta_plain(i, H, G, d, dv, dt_bias, a_log) for i in ins]
    slots = [3, 1, 0]
    whole = _run_delta(ins, [[n] for n in lens], slots, H, G, d, dv, dt_bias, a_log, torch.zeros(4, H, d, dv, device=DEV))
    state = torch.zeros(4, H, d, dv, device=DEV)
    state[2] = float("nan")
    cut = _run_delta(ins, [[7, 1, 1, 2, 29], [1, 2], [1] * 17], slots, H, G, d, dv, dt_bias, a_log, state)
    for a, b, wnt in zip(whole, cut, want):
        _close(a, wnt, 2e-5)
        _close(b, wnt, 2e-5)
    assert torch.isnan(state[2]).all() and torch.isfinite(state[[0, 1, 3]]).all()


def test_delta_rule_reads_its_own_write_and_keeps_it_for_hundreds_of_tokens():
    """With beta = 1 and an empty state the token's own value comes straight back (the read-out follows the write).
    A key channel that does not decay keeps what it holds while the others forget; a second write under the same
    key replaces the first value instead of adding to it."""
    H, G, d, dv, n = 1, 1, 8, 4, 500
    q, k = torch.zeros(n, G, d, dtype=F64), torch.zeros(n, G, d, dtype=F64)
    v = _rand(n, H, dv, seed=1)
    k[:, 0, 1], q[:, 0, 2] = 1.0, 1.0                     # everybody writes under channel 1 and reads channel 2
    k[3, 0] = 0.0
    k[3, 0, 0] = 1.0                                      # token 3 writes under channel 0
    k[250, 0] = k[3, 0]                                   # token 250 writes there again
    q[3, 0] = q[249, 0] = q[499, 0] = k[3, 0]             # and these read it
    b = torch.full((n, H), 30.0, dtype=F64)               # beta = 1
    a = torch.full((n, H, d), 2.0, dtype=F64)             # every channel forgets ...
    a[:, :, 0] = -40.0                                    # ... but channel 0
    ins = [dict(q=q, k=k, v=v, b=b, a=a)]
    zero, a_log = torch.zeros(H, d, dtype=F64), torch.zeros(H, dtype=F64)
    want = _delta_plain(ins[0], H, G, d, dv, zero, a_log)
    for cuts in ([[n]], [[470] + [1] * 30], [[2, 247, 3, 248]]):
        got = _run_delta(ins, cuts, [0], H, G, d, dv, zero, a_log, torch.zeros(1, H, d, dv, device=DEV))[0]
        _close(got, want, 2e-5)
        for t, src in ((3, 3), (249, 3), (499, 250)):
            assert (got[t] * d ** 0.5 - v[src, 0]).abs().max() < 1e-3, (t, src)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,groups,part,w_len", [(5, 3, 8, 8), (40, 2, 96, 192), (7, 1, 1500, 1500), (9, 6, 20, 20), (3, 4, 7, 28),
                                                 (11, 5, 50, 50), (6, 3, 200, 600), (4, 2, 512, 512), (3, 2, 516, 516),
                                                 (700, 9, 128, 128)])
def test_gate_and_norm_over_groups_of_channels(out_dtype, T, groups, part, w_len):
    k = _k()
    W = groups * part
    y, gate, w = _rand(T, W, seed=1, scale=3.0).float(), _rand(T, W + 9, seed=2, scale=2.0).float(), _rand(w_len, seed=3).float()
    g = gate.double()[:, 4:4 + W]
    wide = w.double().repeat(W // w_len)
    tol = 2e-5 if out_dtype == torch.float32 else 1e-2
    out = torch.empty(T, W, dtype=out_dtype, device=DEV)
    k.gated_head_norm(out, y.to(DEV), gate.to(DEV), 4, w.to(DEV), part, 1e-5, gate_after=False)
    v = y.double() * plain.silu(g)
    _close(out, plain.unit_rms(v.view(T, groups, part), 1e-5).reshape(T, W) * wide, tol)
    k.gated_head_norm(out, y.to(DEV), gate.to(DEV), 4, w.to(DEV), part, 1e-5, gate_after=True)
    _close(out, plain.unit_rms(y.double().view(T, groups, part), 1e-5).reshape(T, W) * wide * torch.sigmoid(g), tol)


# ---------------------------------------------------------------------------------------------
# attention: biases, weighted norms per head, the query temperature, a gate on the heads
# ---------------------------------------------------------------------------------------------
def _paged(n_tokens_per_req, page):
    per = max((n + page - 1) // page for n in n_tokens_per_req)
    pages = per * len(n_tokens_per_req)
    table = torch.randperm(pages, generator=torch.Generator().manual_seed(5)).to(torch.int32).view(len(n_tokens_per_req), per)
    return table.contiguous(), per, pages


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,dv,q_temp", [(4, 2, 16, 24, (0.4, 7)), (2, 1, 16, 40, (1.5, 1)), (8, 8, 8, 8, None),
                                                (1, 1, 64, 16, (0.1, 16)), (6, 2, 32, 32, (0.25, 50))])
def test_attention_pieces_with_a_planted_far_key(dtype, nh, nkv, d, dv, q_temp):
    """The rows' preparation (bias, norm with a weight, temperature), the attention that takes any sizes and the
    gate, over a prompt and single tokens behind it.  Key 5 and the last query have one channel only, the same one
    (after their biases), which no other key has: the last token's heads return value 5, far back and many pages
    away."""
    k = _k()
    page, scale, eps = 8, 0.6, 1e-5
    lens = [300, 21]
    nqk, nqkv = (nh + nkv) * d, (nh + nkv) * d + nkv * dv
    bias = _rand(nqkv, seed=1, scale=0.5).float()
    wq, wk = (_rand(d, seed=2).abs() * 0.3 + 0.8).float(), (_rand(d, seed=3).abs() * 0.3 + 0.8).float()
    wq[0] = wk[0] = 3.0
    rows = [_rand(n, nqkv + nh * dv, seed=10 + n).to(dtype) for n in lens]
    r0, b64 = rows[0].double(), bias.double()
    for g in range(nkv):                                 # no key of this request has anything in channel 0 ...
        r0[:, nh * d + g * d] = -b64[nh * d + g * d]
        r0[5, nh * d + g * d:nh * d + (g + 1) * d] = -b64[nh * d + g * d:nh * d + (g + 1) * d]
        r0[5, nh * d + g * d] += 5.0                     # ... but key 5, which has nothing else
    for h in range(nh):                                  # and the last query looks at channel 0 alone
        r0[299, h * d:(h + 1) * d] = -b64[h * d:(h + 1) * d]
        r0[299, h * d] += 5.0
    rows[0] = r0.to(dtype)
    want = []
    for r in rows:
        n = r.shape[0]
        z = r.double()[:, :nqkv] + bias.double()
        q = plain.rms_norm(z[:, :nh * d].view(n, nh, d), wq.double(), eps)
        q = q * plain.query_temperature(n, dict(coef=q_temp[0], every=q_temp[1]) if q_temp else None, F64)[:, None, None]
        kk = plain.rms_norm(z[:, nh * d:nqk].view(n, nkv, d), wk.double(), eps)
        o = plain.causal_attention(q, kk, z[:, nqk:].view(n, nkv, dv), scale).reshape(n, nh * dv)
        want.append(o * torch.sigmoid(r.double()[:, nqkv:]))
    table, per, pages = _paged(lens, page)
    kc = torch.full((pages, nkv, page, d), float("nan"), dtype=dtype, device=DEV)
    vc = torch.full((pages, nkv, page, dv), float("nan"), dtype=dtype, device=DEV)
    got = [torch.zeros(n, nh * dv, dtype=F64) for n in lens]
    err = _err()
    for step in _steps_of([[2, 280, 7] + [1] * 11, [1, 20]]):
        _, req, positions, _ = _meta(step, [0, 1])
        tab = table[[r for r, _, _ in step]].contiguous().to(DEV)
        x = torch.cat([rows[r][s:s + n] for r, s, n in step]).to(DEV)
        T = x.shape[0]
        q = torch.empty(T, nh, d, dtype=dtype, device=DEV)
        k.qkv_prepare(q, kc, vc, x, wq.to(DEV), wk.to(DEV), None, positions, req, tab, per, nh, nkv, d, dv, 0, False, 1, eps, True,
                      err, bias=bias.to(DEV), q_temp=q_temp, row_len=x.shape[1])
        out = torch.empty(T, nh, dv, dtype=dtype, device=DEV)
        k.attention_plain(out, q, kc, vc, positions, req, tab, per, None, scale, err)
        gated = torch.empty(T, nh * dv, dtype=dtype, device=DEV)
        k.gate_sigmoid(gated, out.transpose(0, 1), x[:, nqkv:])
        at = 0
        for r, s, n in step:
            got[r][s:s + n] = gated[at:at + n].double().cpu()
            at += n
    assert int(err.item()) == 0
    for g, wnt in zip(got, want):
        _close(g, wnt, 3e-5 if dtype == torch.float32 else 3e-2)
    v5 = (rows[0].double()[5, nqk:nqkv] + bias.double()[nqk:]).view(nkv, dv).repeat_interleave(nh // nkv, dim=0).reshape(-1)
    last = got[0][299] / torch.sigmoid(rows[0].double()[299, nqkv:])
    assert (last - v5).abs().max() < 0.05 * (1 + v5.abs().max())


def test_query_temperature_steps_where_a_period_completes():
    """floor((p + 1) / every) changes between p = every - 2 and every - 1, and again one period on."""
    k = _k()
    nh, nkv, d, dv, every, coef = 2, 1, 8, 8, 12, 0.7
    n = 40
    rows = torch.ones(n, (nh + nkv) * d + nkv * dv)
    table, per, pages = _paged([n], 8)
    kc, vc = torch.zeros(pages, nkv, 8, d, device=DEV), torch.zeros(pages, nkv, 8, dv, device=DEV)
    q, err = torch.empty(n, nh, d, device=DEV), _err()
    k.qkv_prepare(q, kc, vc, rows.to(DEV), None, None, None, _i32(list(range(n))), _i32([0] * n), table.to(DEV), per, nh, nkv, d, dv,
                  0, False, 0, 1e-6, True, err, q_temp=(coef, every))
    got = q[:, 0, 0].double().cpu()
    want = torch.tensor([1.0 + coef * math.log((p + 1) // every + 1) for p in range(n)], dtype=F64)
    assert (got - want).abs().max() < 1e-5
    assert got[every - 2] == 1.0 and got[every - 1] > 1.4 and got[2 * every - 2] == got[every - 1] and got[2 * every - 1] > got[every - 1]


# ---------------------------------------------------------------------------------------------
# whole models: every way of cutting, pages and slots used again, layer by layer, generation
# ---------------------------------------------------------------------------------------------
LENGTHS = {"G1": [70, 45, 130, 33], "G2": [97, 41, 260, 150], "G3": [170, 1, 75, 58], "G4": [90, 2, 51, 140]}


def _row_error(got, want):
    """Root mean square over the vocabulary of the difference, its mean taken off."""
    d = got.astype(np.float64) - want
    d = d - d.mean()
    return float(np.sqrt((d * d).mean()))


def _tolerance(dtype, ref, cfg=None, w=None, p=None):
    """float32: a small share of the logits' spread (the engine's float32 against float64).  bfloat16: three
    times what rounding alone causes - the largest row error of the plain run that rounds activations to
    bfloat16 where an engine stores them."""
    spread = max(float(np.std(ref)), 1e-3)
    if dtype == "float32":
        return 3e-5 * spread
    rounded = plain.forward(cfg, w, p, round_to=torch.bfloat16).numpy()
    return max(3.0 * max(_row_error(rounded[i], ref[i]) for i in range(len(p))), 1e-3 * spread)


def _store(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY_G))
def test_every_way_of_cutting_gives_the_plain_logits(name, dtype, tmp_path):
    folder = make_folder(str(tmp_path / "model"), name, _store(dtype))
    ps = prompts(name, LENGTHS[name])
    tb = build_all_modes(ps, seed=len(name))
    out = run_trace(folder, dtype, tb.steps, str(tmp_path / "out"), max_tokens=tb.peak, page_size=TINY_G[name][2],
                    max_num_seqs=4)
    cfg, w = plain.load_folder(folder)
    ref = [plain.forward(cfg, w, p).numpy() for p in ps]
    tol = [_tolerance(dtype, r, cfg, w, p) for r, p in zip(ref, ps)]
    seen, worst = {}, {}
    for step, rows in tb.rows.items():
        got = out[step]
        assert got.shape[0] == len(rows)
        for r, ((mode, i), pos) in enumerate(rows):
            e = _row_error(got[r], ref[i][pos])
            worst[mode] = max(worst.get(mode, 0.0), e / tol[i])
            assert e <= tol[i], (f"{name} {dtype} {mode}: request {i} position {pos} (step {step}) differs by {e:.3g} "
                                 f"> {tol[i]:.3g}: the first wrong token of this mode")
            seen.setdefault((mode, i), set()).add(pos)
    for mode in ("whole", "tail", "portions", "mixed"):
        for i, p in enumerate(ps):
            assert sorted(seen[(mode, i)]) == list(range(len(p))), (mode, i)
    print(name, dtype, "worst error / tolerance per mode:", {k: f"{v:.3g}" for k, v in worst.items()})


@pytest.mark.parametrize("name,dtype", [("G1", "float32"), ("G2", "bfloat16"), ("G3", "bfloat16"), ("G4", "float32")])
def test_freed_pages_and_slots_are_used_again_and_nothing_stale_is_read(name, dtype, tmp_path):
    """Pages that go back to the pool are filled with NaN before the next step, and so is every state table's row of
    a request that ends (the token before it: an id out of range).  Eight requests pass through four slots and a
    pool of the live requests' size: the logits stay the plain ones and stay finite."""
    from xinfer_b200.engine.runner import ModelRunner
    folder = make_folder(str(tmp_path / "model"), name, _store(dtype))
    ps = prompts(name, LENGTHS[name])
    tb = build_all_modes(ps, seed=3)
    page = TINY_G[name][2]
    runner = ModelRunner(folder, dtype, block_size=page, num_blocks=(tb.peak + page - 1) // page, max_num_seqs=4,
                         poison_freed_pages=True)
    assert runner.has_state
    close, spoiled = runner.close_request, []

    def close_and_spoil(slot):
        close(slot)
        for t in runner.state.tables.values():
            t[slot].fill_(float("nan") if t.is_floating_point() else 2 ** 30)
        spoiled.append(slot)

    runner.close_request = close_and_spoil
    for t in runner.state.tables.values():               # and what the slots hold before their first request
        t.fill_(float("nan") if t.is_floating_point() else 2 ** 30)
    out = replay_in_process(runner, tb.steps)
    assert len(spoiled) > 4 * 3 and set(spoiled) == {0, 1, 2, 3}
    if any(layer["type"] == "parallel" for layer in TINY_G[name][0]["layers"]):
        assert runner.pages_poisoned > runner.num_blocks
    cfg, w = plain.load_folder(folder)
    ref = [plain.forward(cfg, w, p).numpy() for p in ps]
    tol = [_tolerance(dtype, r, cfg, w, p) for r, p in zip(ref, ps)]
    for step, rows in tb.rows.items():
        assert np.isfinite(out[step]).all(), f"step {step} read a stale page or slot"
        for r, ((mode, i), pos) in enumerate(rows):
            assert _row_error(out[step][r], ref[i][pos]) <= tol[i], (mode, i, pos)


@pytest.mark.parametrize("name", ["G1", "G3"])
def test_layers_one_by_one_in_float32(name, tmp_path):
    """The residual stream after every layer against the plain one, a prompt in two portions."""
    from xinfer_b200.engine.runner import ModelRunner, StepInput
    from xinfer_b200.parts.block import Block
    folder = make_folder(str(tmp_path / "model"), name, torch.float32)
    cfg, w = plain.load_folder(folder)
    p = prompts(name, [29])[0]
    want = []
    plain.forward(cfg, w, p, layers_out=want)
    rec, orig = [], Block.forward

    def spy(self, stream, ctx, cache, state, writes_cache):
        out = orig(self, stream, ctx, cache, state, writes_cache)
        out.settle(ctx)
        rec.append(out.x.double().cpu())
        return out

    Block.forward = spy
    try:
        runner = ModelRunner(folder, "float32", block_size=8, num_blocks=16, max_num_seqs=2)
        slot = runner.open_request()
        runner.step([StepInput(slot, p[:11], [])])
        first = list(rec)
        rec.clear()
        runner.step([StepInput(slot, p[11:], [])])
        runner.check_errors()
    finally:
        Block.forward = orig
    assert len(rec) == len(first) == len(cfg["layers"])
    for i, (a, b, ref) in enumerate(zip(first, rec, want)):
        got = torch.cat([a, b])
        assert got.dtype == F64 and (got - ref).abs().max() <= 2e-5 * (1 + ref.abs().max()), f"layer {i}"


def test_the_residual_stream_is_float32_in_the_bfloat16_engine(tmp_path):
    from xinfer_b200.engine.runner import ModelRunner
    folder = make_folder(str(tmp_path / "model"), "G1", torch.bfloat16)
    runner = ModelRunner(folder, "bfloat16", block_size=8, num_blocks=16, max_num_seqs=2)
    assert runner.model.stream_dtype == torch.float32 and runner.model.dtype == torch.bfloat16
    for t in runner.state.tables.values():
        assert t.dtype in (torch.float32, torch.int32)


def test_a_step_launches_one_norm_kernel_per_sublayer(tmp_path):
    """The norm of a sublayer's output, its learned scale, the addition and the next sublayer's norm are one kernel."""
    from xinfer_b200 import kernels
    from xinfer_b200.engine.runner import ModelRunner, StepInput
    folder = make_folder(str(tmp_path / "model"), "G1", torch.bfloat16)
    runner = ModelRunner(folder, "bfloat16", block_size=8, num_blocks=16, max_num_seqs=2)
    slot = runner.open_request()
    before = dict(kernels.launch_counts())
    runner.step([StepInput(slot, [1, 2, 3, 4, 5], [4])])
    runner.check_errors()
    after = kernels.launch_counts()
    norms = sum(after.get(n, 0) - before.get(n, 0) for n in ("rms_chain", "rmsnorm_f32"))
    adds = sum(after.get(n, 0) - before.get(n, 0) for n in ("add", "add_f32"))
    layers = TINY_G["G1"][0]["layers"]
    sublayers = sum(2 + (layer["mlp"] is not None) for layer in layers)      # mixer, feed-forward, token input
    assert norms == sublayers + 1 and adds == 0, (norms, adds, sublayers)


def _engine(folder, dtype, page, **kw):
    import json
    import os
    from xinfer_b200 import Engine, EngineConfig
    with open(os.path.join(folder, "config.json")) as f:
        limit = min(1024, json.load(f).get("max_positions", 1024))
    opts = dict(weight_path=folder, block_size=page, num_blocks=96, max_num_seqs=4, max_num_batched_tokens=64,
                prefill_chunk_size=16, disable_cuda_graph=True, max_model_len=limit)
    opts.update(kw)
    return Engine(EngineConfig(**opts), dtype)


@pytest.mark.parametrize("name", ["G1", "G4"])
def test_greedy_generation_in_float32_equals_plain(name, tmp_path):
    from xinfer_b200 import SamplingParams
    folder = make_folder(str(tmp_path / "model"), name, torch.float32)
    cfg, w = plain.load_folder(folder)
    ps = prompts(name, [1, 5, 23, 40, 9, 17])       # six requests over four slots, prompts in portions of 16
    eng = _engine(folder, "f32", TINY_G[name][2])
    outs = eng.generate_sync(SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True), ps)
    for p, o in zip(ps, outs):
        assert o.decode_output == plain.generate(cfg, w, p, 12)


@pytest.mark.parametrize("graphs", [False, True], ids=["launched", "cuda_graph"])
@pytest.mark.parametrize("name", ["G2", "G3"])
def test_long_greedy_decoding_in_bfloat16_follows_the_plain_logits(name, graphs, tmp_path):
    """Each generated token is checked against the plain logits of the sequence the engine produced (bfloat16
    may flip a near-tie): it must be the best token up to the drift.  Long enough for many pages per request and
    for the query temperature to step several times."""
    from xinfer_b200 import SamplingParams
    folder = make_folder(str(tmp_path / "model"), name, torch.bfloat16)
    cfg, w = plain.load_folder(folder)
    ps = prompts(name, [3, 30, 61])
    eng = _engine(folder, "bf16", TINY_G[name][2], disable_cuda_graph=not graphs)
    outs = eng.generate_sync(SamplingParams(max_tokens=200, ignore_eos=True), ps)
    assert eng.runner.last_used_graph == graphs
    for p, o in zip(ps, outs):
        assert o.decoded_length == 200
        seq = p + o.decode_output
        ref = plain.forward(cfg, w, seq)
        slack = 2 * 3.0 * float((plain.forward(cfg, w, seq, round_to=torch.bfloat16) - ref).abs().max())
        for i, tok in enumerate(o.decode_output):
            row = ref[len(p) + i - 1]
            assert row[tok] >= row.max() - slack, (i, tok)


def test_a_prompt_longer_than_the_position_table_is_refused(tmp_path):
    from xinfer_b200.engine.runner import ModelRunner, StepInput
    folder = make_folder(str(tmp_path / "model"), "G4", torch.float32)
    runner = ModelRunner(folder, "float32", block_size=16, num_blocks=64, max_num_seqs=2)
    assert runner.max_model_len <= TINY_G["G4"][0]["max_positions"]
    slot = runner.open_request()
    with pytest.raises(Exception):
        runner.step([StepInput(slot, [1] * (TINY_G["G4"][0]["max_positions"] + 1), [0])])
        runner.check_errors()


def test_command_line_writes_a_random_folder_and_generates_from_it(tmp_path, capsys):
    """The command line end to end: a folder from a configuration and a seed, then generation from given ids (equal
    to the plain continuation in float32) and from a seeded prompt of a given length."""
    import json
    from xinfer_b200.cli import main
    config = tmp_path / "config.json"
    config.write_text(json.dumps(TINY_G["G1"][0]))
    folder = str(tmp_path / "model")
    assert main(["--random", str(config), "--seed", "4", "--m", folder, "--store-dtype", "f32"]) == 0
    cfg, w = plain.load_folder(folder)
    capsys.readouterr()
    assert main(["--m", folder, "--dtype", "f32", "--prompts", "5,6,7|9,10", "--max-tokens", "4", "--ignore-eos",
                 "--disable-cuda-graph", "--num-blocks", "16"]) == 0
    out = capsys.readouterr().out
    assert ",".join(str(t) for t in plain.generate(cfg, w, [5, 6, 7], 4)) in out and "Decoded tokens: 8" in out
    assert main(["--m", folder, "--prompt-len", "21", "--batch", "3", "--max-tokens", "5", "--ignore-eos", "--num-blocks", "16",
                 "--seed", "1"]) == 0
    assert "Decoded tokens: 15" in capsys.readouterr().out
