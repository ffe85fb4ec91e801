"""The Mikutar decoder on the GPU against the plain implementation (plain_mikutar.py): every mechanism alone
through its kernel, then whole models through the step function, the replay program and the generation entry
point - whole prompts, token-by-token decoding, portions down to two tokens, unequal batches, pages and slots that
are used again, keys far back and at the edges of windows, chunks and pages, the first tokens of a sequence."""
import math

import numpy as np
import pytest
import torch

import plain_mikutar as plain
from mikutar_models import TINY_M, make_folder, prompts
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


def _tol(dtype):
    return 2e-5 if dtype == torch.float32 else 3e-2


# ---------------------------------------------------------------------------------------------
# the gates of the feed-forwards
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,inter", [(1, 24), (5, 40), (300, 64), (3000, 136)])
def test_relu_and_clamped_swish_gates(dtype, T, inter):
    gu = (_rand(T, 2 * inter, seed=T, scale=2.5)).to(dtype)
    g, u = gu.double()[:, :inter], gu.double()[:, inter:]
    for act, params, want in [
        ("relu", (), torch.relu(g) * u),
        ("swish_clamp", (1.5, 1.702), g.clamp(max=1.5) * torch.sigmoid(1.702 * g.clamp(max=1.5)) * (u.clamp(-1.5, 1.5) + 1)),
        ("swish_clamp", (0.5, 1.0), g.clamp(max=0.5) * torch.sigmoid(g.clamp(max=0.5)) * (u.clamp(-0.5, 0.5) + 1)),
    ]:
        out = torch.full((T, inter), float("nan"), dtype=dtype, device=DEV)
        _k().swiglu(out, gu.to(DEV), act, params)
        assert (out.double().cpu() - want).abs().max() <= (1e-5 if dtype == torch.float32 else 2e-2) * (1 + want.abs().max())
    with pytest.raises(Exception):
        _k().swiglu(out, gu.to(DEV), "swish_clamp", ())


# ---------------------------------------------------------------------------------------------
# the router
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,top,groups,keep", [(6, 2, 3, 2), (9, 3, 9, 4), (4, 1, 2, 2), (5, 2, 1, 1), (12, 5, 4, 2),
                                                (64, 6, 8, 3), (7, 7, 1, 1)])
def test_router_chooses_as_plain(dtype, E, top, groups, keep):
    T, K = 37, 52
    h = _rand(T, K, seed=E).to(dtype)
    w = _rand(E, K, seed=E + 1, scale=0.4).float()
    corr = _rand(E, seed=E + 2, scale=0.6).float()
    choice = torch.full((T, top), -7, dtype=torch.int32, device=DEV)
    weight = torch.full((T, top), float("nan"), dtype=torch.float32, device=DEV)
    req = torch.zeros(T, dtype=torch.int32)
    req[5] = -1                                                      # a padding token takes part in nothing
    _k().expert_router(choice, weight, h.to(DEV), w.to(DEV), corr.to(DEV), req.to(DEV), top, groups, keep, 2)
    idx, wt = plain.route(h.double(), w.double(), corr.double(), top, groups, keep)
    got_i, got_w = choice.cpu(), weight.double().cpu()
    for t in range(T):
        if t == 5:
            assert got_w[t].abs().max() == 0
            continue
        assert got_i[t].tolist() == idx[t].tolist(), t                 # in the order of falling choice score
        assert (got_w[t] - wt[t]).abs().max() < 1e-5
    # without a correction the choice follows the scores; with renormalized weights they sum to one
    _k().expert_router(choice, weight, h.to(DEV), w.to(DEV), None, req.to(DEV), top, 1, 1, 2, renormalize=True)
    idx0, wt0 = plain.route(h.double(), w.double(), torch.zeros(E, dtype=F64), top, 1, 1)
    assert choice.cpu()[0].tolist() == idx0[0].tolist()
    assert abs(float(weight[0].sum()) - 1.0) < 1e-5 and (weight.double().cpu()[0] - wt0[0] / wt0[0].sum()).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [3, 70])
def test_routed_experts_part_equals_plain(dtype, T):
    """The part alone, few tokens (one dense product over all experts in bfloat16) and many (grouped products),
    with a padding token, against the plain mixture."""
    from xinfer_b200.config.plan import FeedForwardSpec, RoutedExpertsSpec
    from xinfer_b200.parts import Workspace, build_part
    from xinfer_b200.parts.base import StepContext
    H, Fi, E = 48, 24, 6
    mlp = dict(kind="moe", expert=dict(ff=Fi, limit=1.5), router=dict(experts=E, top=2, groups=dict(count=3, keep=2)),
               shared=dict(ff=16, limit=0.8))
    names = [f"m.e{e}.{n}" for e in range(E) for n in ("gate", "up", "down")] + ["m.shared.gate", "m.shared.up", "m.shared.down"]
    w = {}
    for i, n in enumerate(names):
        ff = 16 if "shared" in n else Fi
        w[n] = (_rand(*((H, ff) if n.endswith("down") else (ff, H)), seed=100 + i, scale=0.2)).to(dtype).double()
    w["m.router"] = _rand(E, H, seed=7, scale=0.5).to(dtype).double()
    w["m.correction"] = _rand(E, seed=8, scale=0.5).to(dtype).double()

    class Store:
        def get(self, name, device, dt, operand=False, columns=None):
            return w[name].to(dt).to(device)

    shared = FeedForwardSpec(kind="swiglu", hidden=H, intermediate=16, activation="swish_clamp", names=("gate", "up", "down"),
                             act_params=(0.8, 1.702))
    spec = RoutedExpertsSpec(kind="routed_experts", hidden=H, intermediate=Fi, experts=E, top=2, groups=3, keep=2,
                             activation="swish_clamp", act_params=(1.5, 1.702), shared=shared)
    part = build_part("feed_forward", spec, "m.", dtype, DEV)
    part.load(Store())
    x = _rand(T, H, seed=T).to(dtype)
    req = torch.zeros(T, dtype=torch.int32)
    req[1] = -1
    ctx = StepContext(dtype=dtype, device=torch.device(DEV), num_tokens=T, num_entries=1, token_ids=_i32([0] * T),
                      positions=_i32(list(range(T))), req_of_token=req.to(DEV), q_start=_i32([0, T]), start_pos=_i32([0]),
                      slots=_i32([0]), logit_rows=_i32([0]), num_logit_rows=0, tables=[], strides=[], err=_err(),
                      workspace=Workspace(DEV), branch_dtype=torch.float32)
    out = part.forward(x.to(DEV), ctx).double().cpu()
    assert int(ctx.err.item()) == 0
    want = plain.routed_experts(x.double(), w, "m.", mlp)
    keep = [t for t in range(T) if t != 1]
    assert (out[keep] - want[keep]).abs().max() <= (2e-5 if dtype == torch.float32 else 4e-2) * (1 + want.abs().max())
    if dtype == torch.bfloat16 and T > 32:
        # the form of large prompt steps: every expert's rows through the library's product
        from xinfer_b200 import kernels
        from xinfer_b200.parts import routed_experts as form
        before, floor = kernels.launch_counts().get("expert_gather", 0), form.LIBRARY_FROM_FLOP_PER_CALL
        form.LIBRARY_FROM_FLOP_PER_CALL = 0.0
        try:
            again = part.forward(x.to(DEV), ctx).double().cpu()
        finally:
            form.LIBRARY_FROM_FLOP_PER_CALL = floor
        assert kernels.launch_counts().get("expert_gather", 0) == before + 1
        assert (again[keep] - want[keep]).abs().max() <= 4e-2 * (1 + want.abs().max())


# ---------------------------------------------------------------------------------------------
# q/k preparation: one norm over the whole projection, rotation of neighbours, keys that double as values
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,rot", [(4, 2, 12, 8), (3, 3, 16, 16), (8, 1, 32, 0), (5, 5, 6, 2)])
def test_prepare_norms_the_whole_projection_and_keeps_raw_keys_as_values(dtype, nh, nkv, d, rot):
    T, ps, eps = 21, 8, 1e-5
    gw = 4 if nh == 3 else 3                                     # columns behind q and k (a gate's), which stay
    row = _rand(T, (nh + nkv) * d + gw, seed=nh).to(dtype)
    bias = _rand((nh + nkv) * d, seed=1, scale=0.3).float()
    qw, kw = (1 + _rand(nh * d, seed=2, scale=0.3)).float(), (1 + _rand(nkv * d, seed=3, scale=0.3)).float()
    base = 300.0
    inv_freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32) if rot else None
    pos = [3 + i for i in range(T)]
    pages = (max(pos) + ps) // ps
    table = torch.randperm(pages + 2, generator=torch.Generator().manual_seed(5))[:pages].to(torch.int32)
    kc = torch.full((pages + 2, nkv, ps, d), float("nan"), dtype=dtype, device=DEV)
    vc = torch.full_like(kc, float("nan"))
    q_out = torch.full((T, nh, d), float("nan"), dtype=dtype, device=DEV)
    err = _err()
    _k().qkv_prepare(q_out, kc, vc, row.to(DEV), qw.to(DEV), kw.to(DEV), inv_freq.to(DEV) if rot else None, _i32(pos),
                     _i32([0] * T), table.to(DEV).view(1, -1), pages, nh, nkv, d, d, rot, True, 3, eps, True, err,
                     bias=bias.to(DEV), row_len=row.shape[1], value_offset=nh * d)
    assert int(err.item()) == 0
    x = row.double()[:, : (nh + nkv) * d] + bias.double()
    qp, kp = x[:, : nh * d], x[:, nh * d:]
    positions = torch.tensor(pos)
    q_ref = plain.rotate_neighbours(plain.rms_norm(qp, qw.double(), eps).view(T, nh, d), positions, rot, base)
    k_ref = plain.rotate_neighbours(plain.rms_norm(kp, kw.double(), eps).view(T, nkv, d), positions, rot, base)
    assert (q_out.double().cpu() - q_ref).abs().max() <= _tol(dtype) * (1 + q_ref.abs().max())
    for i, p in enumerate(pos):
        page, slot = int(table[p // ps]), p % ps
        assert (kc[page, :, slot].double().cpu() - k_ref[i]).abs().max() <= _tol(dtype) * (1 + k_ref.abs().max())
        assert (vc[page, :, slot].double().cpu() - kp[i].view(nkv, d)).abs().max() <= _tol(dtype) * (1 + kp.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gate_of_one_number_per_head(dtype):
    T, H, dv = 9, 5, 12
    o = _rand(T, H * dv, seed=1).to(dtype)
    g = _rand(T, H + 2, seed=2, scale=2.0).to(dtype)
    out = o.to(DEV).clone()
    _k().gate_sigmoid(out, out.view(T, H, dv).transpose(0, 1), g.to(DEV)[:, 2:])
    want = o.double().view(T, H, dv) * torch.sigmoid(g.double()[:, 2:])[:, :, None]
    assert (out.double().cpu().view(T, H, dv) - want).abs().max() <= _tol(dtype) * (1 + want.abs().max())


# ---------------------------------------------------------------------------------------------
# the attention itself: windows, chunks, capped scores, the distance bias
# ---------------------------------------------------------------------------------------------
class _Ctx:
    """The fields of a step context that the attention backend reads, for requests whose keys and values already
    lie in pages (in a scrambled order) and whose last ``len - start`` tokens are this step's queries."""

    def __init__(self, seqs, starts, ps, dtype, seed, fixed=False):
        from xinfer_b200.parts import LayerCache, Workspace
        lens = [k.shape[0] for _, k, _ in seqs]
        need = [(n + ps - 1) // ps for n in lens]
        total = sum(need) + 3
        order = torch.randperm(total, generator=torch.Generator().manual_seed(seed)).tolist()
        G, d = seqs[0][1].shape[1:]
        dv = seqs[0][2].shape[2]
        kp = torch.full((total, G, ps, d), float("nan"), dtype=dtype)
        vp = torch.full((total, G, ps, dv), float("nan"), dtype=dtype)
        self.stride = max(need) + 2
        table = torch.full((len(seqs), self.stride), -1, dtype=torch.int32)
        at = 0
        for b, (_, k, v) in enumerate(seqs):
            for p in range(need[b]):
                page = order[at]
                at += 1
                table[b, p] = page
                n = min(ps, lens[b] - p * ps)
                kp[page, :, :n] = k[p * ps:p * ps + n].transpose(0, 1).to(dtype)
                vp[page, :, :n] = v[p * ps:p * ps + n].transpose(0, 1).to(dtype)
        counts = [n - s for n, s in zip(lens, starts)]
        self.cache = LayerCache.of_keys_and_values(kp.to(DEV), vp.to(DEV), 0, ps)
        self.table = table.to(DEV)
        self.q = torch.cat([q[s:] for (q, _, _), s in zip(seqs, starts)]).to(dtype).to(DEV).contiguous()
        self.bounds = np.concatenate([[0], np.cumsum(counts)]).tolist()
        self.h_q_start = np.asarray(self.bounds, dtype=np.int32)
        self.h_start_pos = np.asarray(starts, dtype=np.int32)
        self.q_start, self.start_pos = _i32(self.bounds), _i32(starts)
        self.num_entries = self.real_entries = len(seqs)
        self.num_tokens = self.real_tokens = int(self.bounds[-1])
        self.positions = _i32([s + i for s, c in zip(starts, counts) for i in range(c)])
        self.req_of_token = _i32([b for b, c in enumerate(counts) for _ in range(c)])
        self.all_single = all(c == 1 for c in counts)
        self.fixed_shapes = fixed
        self.max_context = max(lens)
        self.workspace = Workspace(DEV)
        self.scratch = {}
        self.err = _err()
        self.strides = [self.stride]
        self.tables = [self.table]


def _attend(seqs, starts, scale, ps, dtype, window=None, chunk=None, softcap=None, slope=None, seed=0, tiled=True):
    """seqs: [(q [n, H, d], k [n, G, d], v [n, G, dv])]; runs the engine's attention for the tokens from starts[b] on."""
    from xinfer_b200.parts import attention_backend as ab
    ctx = _Ctx(seqs, starts, ps, dtype, seed)
    T, H, d = ctx.q.shape
    G, dv = seqs[0][1].shape[1], seqs[0][2].shape[2]
    out = torch.full((T, H, dv), float("nan"), dtype=dtype, device=DEV)
    ab.set_tiled(tiled)
    try:
        if dtype == torch.bfloat16 and tiled and d == dv:
            ab.prepare_step(ctx, dtype, H, G, d, ps, _k().mask_code(window, chunk), ctx.stride)
        if d == dv:
            ab.attend(out, ctx.q, ctx.cache, ctx, ctx.table, ctx.stride, window, scale, softcap=softcap, slope_exponent=slope,
                      chunk=chunk)
        else:
            _k().attention_plain(out, ctx.q, ctx.cache["k"], ctx.cache["v"], ctx.positions, ctx.req_of_token, ctx.table,
                                 ctx.stride, window, scale, ctx.err, softcap=softcap, slope_exponent=slope, chunk=chunk)
    finally:
        ab.set_tiled(True)
    torch.cuda.synchronize()
    assert int(ctx.err.item()) == 0
    res = out.double().cpu()
    return [res[a:b] for a, b in zip(ctx.bounds[:-1], ctx.bounds[1:])]


def _oracle(q, k, v, scale, window=None, chunk=None, softcap=None, slope=None):
    n, H = q.shape[0], q.shape[1]
    mask = plain.chunk_mask(n, chunk) if chunk else plain.window_mask(n, window if window else n)
    return plain.softmax_attention(q, k, v, mask, scale, softcap, plain.head_slopes(H) if slope else None)


def _qkv(n, H, G, d, dv, seed, dtype, sharp=1.0):
    q = (_rand(n, H, d, seed=seed) * sharp).to(dtype).double()
    k = _rand(n, G, d, seed=seed + 1).to(dtype).double()
    v = _rand(n, G, dv, seed=seed + 2).to(dtype).double()
    return q, k, v


# (dtype, tiled): float32 on the plain kernel, bfloat16 on the tensor-core kernels and on the plain one
FORMS = [(torch.float32, False), (torch.bfloat16, True), (torch.bfloat16, False)]


@pytest.mark.parametrize("dtype,tiled", FORMS)
@pytest.mark.parametrize("H,G,d,dv,ps", [(4, 2, 16, 16, 8), (8, 2, 32, 32, 16), (3, 1, 48, 48, 32), (6, 3, 10, 14, 8),
                                          (2, 2, 64, 64, 16)])
@pytest.mark.parametrize("mask", [dict(chunk=37, softcap=8.0, slope=8.0), dict(chunk=64, softcap=None, slope=8.0),
                                  dict(window=50), dict(chunk=7, softcap=45.0, slope=None)])
def test_attention_of_unequal_entries_equals_plain(dtype, tiled, H, G, d, dv, ps, mask):
    """Prompt portions of several lengths, one that continues a cached prefix, single tokens, all in one batch."""
    if mask.get("window") and d != dv:
        pytest.skip("a window with key and value sizes that differ is another part's case")
    lens, starts = [150, 61, 200, 97, 1], [0, 40, 199, 96, 0]
    seqs = [_qkv(n, H, G, d, dv, 10 * b, dtype, 2.0) for b, n in enumerate(lens)]
    got = _attend(seqs, starts, 0.4, ps, dtype, seed=3, tiled=tiled, **mask)
    for (q, k, v), s, o in zip(seqs, starts, got):
        ref = _oracle(q, k, v, 0.4, **mask)[s:]
        assert (o - ref).abs().max() <= _tol(dtype) * (1 + ref.abs().max())


@pytest.mark.parametrize("dtype,tiled", FORMS)
@pytest.mark.parametrize("decode", [False, True], ids=["prompt", "decoded"])
@pytest.mark.parametrize("chunk", [48, 64, 1, 120, 33])
def test_chunk_edges(dtype, tiled, decode, chunk):
    """One key is made to stand out for the last query.  The chunk's first key decides the output, the key before
    it - the last of the chunk before - must not be seen, whatever the pages' and tiles' borders are."""
    H, G, d, ps, n = 4, 2, 32, 8, 331
    first = (n - 1) // chunk * chunk
    for j, inside in [(first, True), (first - 1, False), (n - 1, True), (0, first == 0)]:
        if j < 0:
            continue
        q, k, v = _qkv(n, H, G, d, d, 5, dtype)
        for h in range(H):
            q[-1, h] = k[j, h // (H // G)] * 1.5
        q = q.to(dtype).double()
        start = n - 1 if decode else n - 9
        got = _attend([(q, k, v)], [start], 1.0, ps, dtype, chunk=chunk, tiled=tiled)[0]
        ref = _oracle(q, k, v, 1.0, chunk=chunk)[start:]
        assert (got - ref).abs().max() <= _tol(dtype) * (1 + ref.abs().max())
        for h in range(H):
            carried = (got[-1, h] - v[j, h // (H // G)]).abs().max() < 8e-2 * (1 + v.abs().max())
            assert bool(carried) == inside, (j, inside, h)


@pytest.mark.parametrize("dtype,tiled", FORMS)
@pytest.mark.parametrize("decode", [False, True], ids=["prompt", "decoded"])
@pytest.mark.parametrize("window", [48, 64, 1, 200, 11])
def test_window_edges(dtype, tiled, decode, window):
    H, G, d, ps, n = 4, 1, 16, 16, 260
    for j, inside in [(n - window, True), (n - window - 1, False), (n - 1, True)]:
        if j < 0:
            continue
        q, k, v = _qkv(n, H, G, d, d, 6, dtype)
        for h in range(H):
            q[-1, h] = k[j, 0] * 2.0
        q = q.to(dtype).double()
        start = n - 1 if decode else n - 9
        got = _attend([(q, k, v)], [start], 1.0, ps, dtype, window=window, tiled=tiled)[0]
        ref = _oracle(q, k, v, 1.0, window=window)[start:]
        assert (got - ref).abs().max() <= _tol(dtype) * (1 + ref.abs().max())
        carried = (got[-1, 0] - v[j, 0]).abs().max() < 8e-2 * (1 + v.abs().max())
        assert bool(carried) == inside, (j, inside)


@pytest.mark.parametrize("dtype,tiled", FORMS)
@pytest.mark.parametrize("decode", [False, True], ids=["prompt", "decoded"])
@pytest.mark.parametrize("where", ["first", "second", "page_end", "page_start", "tile_end", "tile_start", "far", "previous"])
def test_one_planted_key_far_back_decides_the_output(dtype, tiled, where, decode):
    """Among hundreds of keys of one long chunk one stands out for the last query - at the first tokens, at page
    and tile borders, far back; the cap must not flatten it away and the distance bias must be the small one of
    the last head's slope."""
    H, G, d, ps, n = 8, 2, 32, 16, 600
    j = {"first": 0, "second": 1, "page_end": 31, "page_start": 32, "tile_end": 63, "tile_start": 64, "far": n - 517,
         "previous": n - 2}[where]
    q, k, v = _qkv(n, H, G, d, d, 99, dtype)
    for h in range(H):
        q[-1, h] = k[j, h // (H // G)] * 1.5
    q = q.to(dtype).double()
    start = n - 1 if decode else n - 37
    got = _attend([(q, k, v)], [start], 1.0, ps, dtype, chunk=1000, softcap=60.0, slope=8.0, tiled=tiled)[0]
    ref = _oracle(q, k, v, 1.0, chunk=1000, softcap=60.0, slope=8.0)[start:]
    assert (got - ref).abs().max() <= _tol(dtype) * (1 + ref.abs().max())
    # head H-1 has the smallest slope (2^-8): a key 500 positions back loses 2 units of some 45; head 0 (slope 1/2)
    # forgets everything but its neighbours
    assert (got[-1, H - 1] - v[j, G - 1]).abs().max() < 8e-2 * (1 + v.abs().max()), "the planted key must carry the output"
    if n - 1 - j > 200:
        assert (got[-1, 0] - v[j, 0]).abs().max() > 0.5


@pytest.mark.parametrize("dtype,tiled", FORMS)
def test_the_cap_bounds_a_score_and_the_slope_orders_equal_keys(dtype, tiled):
    """All keys equal: without the bias every weight is the same; with it the weights fall by the head's slope per
    position, whatever the cap did to the (equal) scores."""
    H, G, d, n = 2, 1, 16, 40
    k = torch.ones(n, G, d, dtype=F64) * 3.0
    q = torch.ones(n, H, d, dtype=F64) * 3.0                      # raw score 144: the cap of 5 leaves 5 for every key
    v = torch.zeros(n, G, d, dtype=F64)
    v[:, 0, 0] = torch.arange(n, dtype=F64)                       # the value tells the position
    got = _attend([(q, k, v)], [0], 1.0, 8, dtype, chunk=64, softcap=5.0, slope=8.0, tiled=tiled)[0]
    for h in range(H):
        s = float(plain.head_slopes(H)[h])
        wts = torch.tensor([math.exp(-s * (n - 1 - j)) for j in range(n)], dtype=F64)
        want = float((wts * torch.arange(n, dtype=F64)).sum() / wts.sum())
        assert abs(float(got[-1, h, 0]) - want) < (1e-3 if dtype == torch.float32 else 0.2)


# ---------------------------------------------------------------------------------------------
# whole models: every way of cutting, pages and slots used again, layer by layer, generation
# ---------------------------------------------------------------------------------------------
LENGTHS = {"M1": [70, 45, 130, 33], "M2": [97, 41, 260, 150], "M3": [170, 1, 75, 58], "M4": [90, 2, 51, 140]}


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


@pytest.mark.parametrize("name", sorted(TINY_M))
def test_every_way_of_cutting_gives_the_plain_logits_in_float32_through_the_replay_program(name, tmp_path):
    dtype = "float32"
    folder = make_folder(str(tmp_path / "model"), name, _store(dtype))
    ps = prompts(name, LENGTHS[name])
    tb = build_all_modes(ps, seed=len(name))
    out = run_trace(folder, dtype, tb.steps, str(tmp_path / "out"), max_tokens=tb.peak, page_size=TINY_M[name][2],
                    max_num_seqs=4)
    cfg, w = plain.load_folder(folder)
    ref = [plain.forward(cfg, w, p).numpy() for p in ps]
    tol = [_tolerance(dtype, r, cfg, w, p) for r, p in zip(ref, ps)]
    seen = {}
    for step, rows in tb.rows.items():
        got = out[step]
        assert got.shape[0] == len(rows)
        for r, ((mode, i), pos) in enumerate(rows):
            e = _row_error(got[r], ref[i][pos])
            assert e <= tol[i], (f"{name} {mode}: request {i} position {pos} (step {step}) differs by {e:.3g} "
                                 f"> {tol[i]:.3g}: the first wrong token of this mode")
            seen.setdefault((mode, i), set()).add(pos)
    for mode in ("whole", "tail", "portions", "mixed"):
        for i, p in enumerate(ps):
            assert sorted(seen[(mode, i)]) == list(range(len(p))), (mode, i)


def _replay_with_routes(runner, steps, moe_runs):
    """``replay_in_process`` with every router call's choices kept: returns the logits per step and, per request id
    and layer run, the experts chosen at every position of the request."""
    from xinfer_b200 import kernels
    from xinfer_b200.engine.runner import StepInput
    calls, orig = [], kernels.expert_router

    def spy(choice, weight, *a, **kw):
        orig(choice, weight, *a, **kw)
        calls.append(choice.clone())

    slots, at, routes, out = {}, {}, {}, {}
    kernels.expert_router = spy
    try:
        for s in steps:
            calls.clear()
            entries = []
            for e in s["entries"]:
                if e["id"] not in slots:
                    slots[e["id"]] = runner.open_request()
                    at[e["id"]] = 0
                entries.append(StepInput(slots[e["id"]], e["tokens"], e.get("want", [])))
            logits = runner.step(entries)
            runner.check_errors()
            if logits.shape[0]:
                out[s["step"]] = logits.float().cpu().numpy().copy()
            assert len(calls) == len(moe_runs)
            chosen = [c.cpu() for c in calls]
            row = 0
            for e in s["entries"]:          # the step's rows are its entries' tokens in order
                n = len(e["tokens"])
                for run, c in zip(moe_runs, chosen):
                    routes.setdefault(e["id"], {}).setdefault(run, []).append(c[row:row + n])
                row += n
            for rid in s.get("end", []):
                runner.close_request(slots.pop(rid))
    finally:
        kernels.expert_router = orig
    assert not slots
    return out, {rid: {run: torch.cat(parts) for run, parts in per.items()} for rid, per in routes.items()}


def _check_trace(name, dtype, runner, tb, ps, cfg, w):
    """Replays the trace and compares every wanted row with the plain run of its request.  An engine that rounds
    activations may decide a router's close call the other way, after which the request is another computation:
    the engine's choices are recorded, checked to differ from the plain ones by close calls only, and followed by
    the plain run (in float32 nothing is close: the slack is a rounding error's)."""
    order = plain.layer_order(cfg)
    moe_runs = [run for run, (i, _) in enumerate(order) if (cfg["layers"][i].get("mlp") or {}).get("kind") == "moe"]
    out, routes = _replay_with_routes(runner, tb.steps, moe_runs)
    slack = 1e-5 if dtype == "float32" else 0.05
    ref, tol = {}, {}         # per request id of the trace: the plain logits along the engine's routes

    def plain_of(rid, i):
        if rid not in ref:
            given = [routes[rid].get(run) for run in range(len(order))]
            ref[rid] = plain.forward(cfg, w, ps[i], routes=given, slack=slack).numpy()
            tol[rid] = _tolerance(dtype, ref[rid], cfg, w, ps[i])
        return ref[rid], tol[rid]

    seen, worst = {}, {}
    for step, rows in tb.rows.items():
        got = out[step]
        assert got.shape[0] == len(rows)
        assert np.isfinite(got).all(), f"step {step} read a stale page"
        rid_of_row = [e["id"] for e in tb.steps[step]["entries"] for _ in e["want"]]
        for r, ((mode, i), pos) in enumerate(rows):
            want, t = plain_of(rid_of_row[r], i)
            e = _row_error(got[r], want[pos])
            worst[mode] = max(worst.get(mode, 0.0), e / t)
            assert e <= t, (f"{name} {dtype} {mode}: request {i} position {pos} (step {step}) differs by {e:.3g} "
                            f"> {t:.3g}: the first wrong token of this mode")
            seen.setdefault((mode, i), set()).add(pos)
    for mode in ("whole", "tail", "portions", "mixed"):
        for i, p in enumerate(ps):
            assert sorted(seen[(mode, i)]) == list(range(len(p))), (mode, i)
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY_M))
def test_every_way_of_cutting_gives_the_plain_logits(name, dtype, tmp_path):
    """Every request whole, with its tail token by token, in portions, and four at a time over a pool of the live
    requests' size, against the plain run."""
    from xinfer_b200.engine.runner import ModelRunner
    folder = make_folder(str(tmp_path / "model"), name, _store(dtype))
    ps = prompts(name, LENGTHS[name])
    tb = build_all_modes(ps, seed=len(name))
    page = TINY_M[name][2]
    runner = ModelRunner(folder, dtype, block_size=page, num_blocks=(tb.peak + page - 1) // page, max_num_seqs=4)
    cfg, w = plain.load_folder(folder)
    worst = _check_trace(name, dtype, runner, tb, ps, cfg, w)
    print(name, dtype, "worst error / tolerance per mode:", {k: f"{v:.3g}" for k, v in worst.items()})


@pytest.mark.parametrize("name,dtype", [("M1", "float32"), ("M2", "bfloat16"), ("M3", "bfloat16"), ("M4", "float32")])
def test_freed_pages_are_used_again_and_nothing_stale_is_read(name, dtype, tmp_path):
    """Pages that go back to the pool are filled with NaN before the next step (also the pages that windows give
    back while a request runs).  Eight requests pass through four slots and a pool of the live requests' size:
    the logits stay the plain ones and stay finite."""
    from xinfer_b200.engine.runner import ModelRunner
    folder = make_folder(str(tmp_path / "model"), name, _store(dtype))
    ps = prompts(name, LENGTHS[name])
    tb = build_all_modes(ps, seed=3)
    page = TINY_M[name][2]
    runner = ModelRunner(folder, dtype, block_size=page, num_blocks=(tb.peak + page - 1) // page, max_num_seqs=4,
                         poison_freed_pages=True)
    cfg, w = plain.load_folder(folder)
    _check_trace(name, dtype, runner, tb, ps, cfg, w)
    assert runner.pages_poisoned > runner.num_blocks


@pytest.mark.parametrize("name", ["M1", "M2", "M4"])
def test_layer_runs_one_by_one_in_float32(name, tmp_path):
    """The residual stream after every layer run (a layer that runs three times counts three times) against the
    plain one, a prompt in two portions; every pass of a repeated layer keeps a cache of its own."""
    from xinfer_b200.engine.runner import ModelRunner, StepInput
    from xinfer_b200.parts.block import Block
    folder = make_folder(str(tmp_path / "model"), name, torch.float32)
    cfg, w = plain.load_folder(folder)
    p = prompts(name, [29])[0]
    want = []
    plain.forward(cfg, w, p, streams=want)
    rec, orig = [], Block.forward

    def spy(self, stream, ctx, cache, state, writes_cache):
        out = orig(self, stream, ctx, cache, state, writes_cache)
        out.settle(ctx)
        rec.append(out.x.double().cpu())
        return out

    Block.forward = spy
    try:
        runner = ModelRunner(folder, "float32", block_size=8, num_blocks=64, max_num_seqs=2)
        slot = runner.open_request()
        runner.step([StepInput(slot, p[:11], [])])
        first = list(rec)
        rec.clear()
        runner.step([StepInput(slot, p[11:], [])])
        runner.check_errors()
    finally:
        Block.forward = orig
    assert len(rec) == len(first) == len(plain.layer_order(cfg)) == len(want)
    assert len({c["k"].data_ptr() for c in runner.layer_caches}) == len(want)
    for i, (a, b, ref) in enumerate(zip(first, rec, want)):
        got = torch.cat([a[:11], b[: len(p) - 11]])
        assert got.dtype == F64 and (got - ref).abs().max() <= 2e-5 * (1 + ref.abs().max()), f"layer run {i}"


def test_the_residual_stream_is_float32_and_the_fast_kernels_are_chosen_in_bfloat16(tmp_path):
    from xinfer_b200 import kernels
    from xinfer_b200.engine.runner import ModelRunner, StepInput
    folder = make_folder(str(tmp_path / "model"), "M2", torch.bfloat16)
    runner = ModelRunner(folder, "bfloat16", block_size=16, num_blocks=32, max_num_seqs=2)
    assert runner.model.stream_dtype == torch.float32 and runner.model.dtype == torch.bfloat16
    assert runner.model.graph_safe()
    assert all(b.mixer._plain_softmax() for b in runner.model.blocks)      # head sizes in steps of 16: tensor-core kernels
    slot = runner.open_request()
    before = dict(kernels.launch_counts())
    runner.step([StepInput(slot, list(range(40)), [39])])
    runner.step([StepInput(slot, [5], [0])])
    runner.check_errors()
    after = kernels.launch_counts()
    used = {k for k in after if after[k] > before.get(k, 0)}
    assert "attn_prefill_tc" in used and "attn_decode_tc" in used and "attention_plain" not in used, sorted(used)
    assert "expert_router" in used and "expert_gemm_mma" in used and "expert_select_gate" in used, sorted(used)


def _engine(folder, dtype, page, **kw):
    from xinfer_b200 import Engine, EngineConfig
    opts = dict(weight_path=folder, block_size=page, num_blocks=96, max_num_seqs=4, max_num_batched_tokens=64,
                prefill_chunk_size=16, disable_cuda_graph=True, max_model_len=1024)
    opts.update(kw)
    return Engine(EngineConfig(**opts), dtype)


@pytest.mark.parametrize("name", ["M1", "M3"])
def test_greedy_generation_in_float32_equals_plain(name, tmp_path):
    from xinfer_b200 import SamplingParams
    folder = make_folder(str(tmp_path / "model"), name, torch.float32)
    cfg, w = plain.load_folder(folder)
    ps = prompts(name, [1, 5, 23, 40, 9, 17])       # six requests over four slots, prompts in portions of 16
    eng = _engine(folder, "f32", TINY_M[name][2])
    outs = eng.generate_sync(SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True), ps)
    for p, o in zip(ps, outs):
        assert o.decode_output == plain.greedy(cfg, w, p, 12)


@pytest.mark.parametrize("graphs", [False, True], ids=["launched", "cuda_graph"])
@pytest.mark.parametrize("name", ["M2", "M4"])
def test_long_greedy_decoding_in_bfloat16_follows_the_plain_logits(name, graphs, tmp_path):
    """Each generated token is checked against the plain logits of the sequence the engine produced (bfloat16
    may flip a near-tie): it must be the best token up to the drift.  Long enough for many pages per request, for
    windows to pass over decoded tokens and for several chunks to begin."""
    from xinfer_b200 import SamplingParams
    folder = make_folder(str(tmp_path / "model"), name, torch.bfloat16)
    cfg, w = plain.load_folder(folder)
    ps = prompts(name, [3, 30, 61])
    eng = _engine(folder, "bf16", TINY_M[name][2], disable_cuda_graph=not graphs)
    outs = eng.generate_sync(SamplingParams(max_tokens=150, ignore_eos=True), ps)
    assert eng.runner.last_used_graph == graphs
    for p, o in zip(ps, outs):
        assert o.decoded_length == 150
        seq = p + o.decode_output
        ref = plain.forward(cfg, w, seq)
        slack = 2 * 3.0 * float((plain.forward(cfg, w, seq, round_to=torch.bfloat16) - ref).abs().max())
        for i, tok in enumerate(o.decode_output):
            row = ref[len(p) + i - 1]
            assert row[tok] >= row.max() - slack, (i, tok)


def test_command_line_writes_a_random_folder_and_generates_from_it(tmp_path, capsys):
    """The command line end to end: a folder from a configuration and a seed, then generation from given ids (equal
    to the plain continuation in float32) and from a seeded prompt of a given length."""
    import json
    from xinfer_b200.cli import main
    config = tmp_path / "config.json"
    config.write_text(json.dumps(TINY_M["M1"][0]))
    folder = str(tmp_path / "model")
    assert main(["--random", str(config), "--seed", "4", "--m", folder, "--store-dtype", "f32"]) == 0
    cfg, w = plain.load_folder(folder)
    capsys.readouterr()
    assert main(["--m", folder, "--dtype", "f32", "--prompts", "5,6,7|9,10", "--max-tokens", "4", "--ignore-eos",
                 "--disable-cuda-graph", "--num-blocks", "32"]) == 0
    out = capsys.readouterr().out
    assert ",".join(str(t) for t in plain.greedy(cfg, w, [5, 6, 7], 4)) in out and "Decoded tokens: 8" in out
    assert main(["--m", folder, "--prompt-len", "21", "--batch", "3", "--max-tokens", "5", "--ignore-eos", "--num-blocks", "32",
                 "--seed", "1"]) == 0
    assert "Decoded tokens: 15" in capsys.readouterr().out
