"""Lunelorn on the GPU: each new kernel alone against its plain statement (tests/kernel_refs.py, float64), and the
engine against the plain implementation (tests/plain_lunelorn.py) in every way of cutting the work, in float32 and in
bfloat16, through the step function, the trace program and greedy generation."""
import pytest
import torch

import plain_lunelorn as P
import tiny
import tiny_lunelorn as TL
from kernel_refs import ReferenceKernels

pytestmark = pytest.mark.gpu

REF = ReferenceKernels(torch.float64)
F32_TOL = 1e-4       # times the largest logit: float32 arithmetic against float64 through layers that run up to three times
BF16_TOL = 4e-2      # times the largest logit: activations between kernels carry 8 bits, and the tiny models' attention is peaked
BF16_SHARE = 0.7     # of the positions: a bfloat16 rounding can turn an expert choice, which the plain implementation does not follow


def float32_noise(cfg, w, toks):
    """Per position, how far the plain implementation itself moves when it is computed in float32: where a position is
    ill-conditioned (a sublayer's result near zero before its unit norm, say) no float32 engine can be closer."""
    P.F = torch.float32
    try:
        low = P.forward(cfg, w, toks).double()
    finally:
        P.F = torch.float64
    return (low - P.forward(cfg, w, toks)).abs().max(dim=-1).values


def rows_match(out, want, dtype, what="", noise=None, share=None):
    """float32: every position within F32_TOL of the largest logit (or, with ``noise``, within three times the plain
    implementation's own float32 movement there, if that is more).  bfloat16: BF16_SHARE of the positions within BF16_TOL of
    it, and the median within three quarters of it (the float32 runs are the sharp test of every mechanism; these show
    that the bfloat16 path computes the same model)."""
    top = max(1.0, float(want.abs().max()))
    err = (out.double() - want.double()).abs().max(dim=-1).values
    if dtype in ("float32", torch.float32):
        tol = torch.full_like(err, F32_TOL * top) if noise is None else torch.maximum(torch.full_like(err, F32_TOL * top), 3 * noise)
        bad = err > tol
        assert not bool(bad.any()), f"{what}: position {int(bad.nonzero()[0])}: {float(err[bad][0])} > {float(tol[bad][0])}"
    else:
        good = float((err <= BF16_TOL * top).double().mean())
        assert good >= (share or BF16_SHARE) and float(err.median()) <= (0.75 if share is None else 1.0) * BF16_TOL * top, \
            f"{what}: {good:.2f} of the positions within {BF16_TOL * top}, median {float(err.median())}; first look at {int(err.argmax())}"
    return float(err.max())


@pytest.fixture(scope="module")
def K():
    from infurnace_b200.kernels import load_cuda_kernels
    return load_cuda_kernels()


def gen(seed):
    return torch.Generator().manual_seed(seed)


def close(got, want, tol, what=""):
    err = float((got.double().cpu() - want.double().cpu()).abs().max())
    assert err <= tol, f"{what}: {err} > {tol}"


def requests(lens_new, lens_old=None, pad=0):
    """cu_q, seq_lens, state_slots (int32) for requests that bring lens_new tokens on top of lens_old; ``pad`` more
    requests of length 0 with one row each (the padding of a recorded decode step)."""
    lens_old = lens_old or [0] * len(lens_new)
    cu = [0]
    for n in lens_new:
        cu.append(cu[-1] + n)
    seq = [a + b for a, b in zip(lens_new, lens_old)]
    for _ in range(pad):
        cu.append(cu[-1] + 1)
        seq.append(0)
    slots = [2 * i + 1 for i in range(len(lens_new))] + [0] * pad       # distinct, out of order with the rows, never slot 0
    return (torch.tensor(cu, dtype=torch.int32), torch.tensor(seq, dtype=torch.int32), torch.tensor(slots, dtype=torch.int32))


# ------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("rows,width", [(1, 33), (7, 336), (70, 2048), (3, 2052), (2, 5000)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_stream_update_with_both_norms(K, rows, width, out_dtype):
    g = gen(rows * width)
    x, y = torch.randn(rows, width, generator=g), 5 * torch.randn(rows, width, generator=g)
    post, nxt = 1 + 0.3 * torch.randn(width, generator=g), 1 + 0.3 * torch.randn(width, generator=g)
    for wdt in (torch.float32, torch.bfloat16):
        for mode in ("none", "copy", "norm"):
            want, wout = x.clone().double(), torch.zeros(rows, width, dtype=torch.float64)
            REF.residual_norm_update(want, y, post.to(wdt), 1e-5, out=None if mode == "none" else wout,
                                     next_weight=nxt.to(wdt) if mode == "norm" else None)
            xd = x.cuda()
            out = None if mode == "none" else torch.zeros(rows, width, device="cuda", dtype=out_dtype)
            K.residual_norm_update(xd, y.cuda(), post.to(wdt).cuda(), 1e-5, out=out,
                                   next_weight=nxt.to(wdt).cuda() if mode == "norm" else None)
            close(xd, want, 4e-6, f"update {mode}")
            if out is not None:
                close(out, wout, 4e-6 if out_dtype == torch.float32 else 0.03, f"next input {mode}")


def test_small_stream_kernels(K):
    g = gen(3)
    x, rows, vec = torch.randn(9, 70, generator=g), torch.randn(9, 70, generator=g), torch.randn(70, generator=g)
    for acc in (True, False):
        for r_, v_ in ((rows, vec), (None, vec.bfloat16()), (rows, None)):
            want = x.clone().double()
            REF.add_rows(want, r_, v_, accumulate=acc)
            xd = x.cuda()
            K.add_rows(xd, None if r_ is None else r_.cuda(), None if v_ is None else v_.cuda(), accumulate=acc)
            close(xd, want, 1e-6, "add_rows")
        want, xd = x.clone().double(), x.cuda()
        REF.scaled_sum(want, rows, 1.3, accumulate=acc)
        K.scaled_sum(xd, rows.cuda(), 1.3, accumulate=acc)
        close(xd, want, 1e-6, "scaled_sum")
    table = torch.randn(40, 30, generator=g)
    ids = torch.randint(0, 40, (9,), generator=g, dtype=torch.int32)
    z = 2 * torch.randn(9, 6, generator=g)
    for dt in (torch.float32, torch.bfloat16):
        want, got = torch.zeros(9, 6, dtype=torch.float64), torch.zeros(9, 6, device="cuda", dtype=dt)
        REF.token_side_gate(z, table.to(dt), ids, 12, "gelu_tanh", want)
        K.token_side_gate(z.cuda(), table.to(dt).cuda(), ids.cuda(), 12, "gelu_tanh", got)
        close(got, want, 2e-6 if dt == torch.float32 else 0.03, "token side gate")
    logits = 40 * torch.randn(5, 77, generator=g)
    want, got = logits.clone().double(), logits.cuda()
    REF.softcap(want, 12.0)
    K.softcap(got, 12.0)
    close(got, want, 5e-6, "softcap")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_shift_over_steps_and_slots(K, dtype):
    """Two steps: what the second step's first rows blend with is the first step's last rows, per slot; a padding
    request leaves slot 0 alone."""
    g = gen(5)
    W, S = 72, 5
    mu = torch.rand(S, W, generator=g)
    last = torch.randn(6, W, generator=g)
    want_last, got_last = last.clone(), last.cuda()
    for lens in ([3, 1, 20], [1, 1, 2]):
        cu, seq, slots = requests(lens, [5, 5, 5], pad=1)
        n = int(cu[-1])
        h = torch.randn(n, W, generator=g).to(dtype)
        want = torch.zeros(S, n, W, dtype=torch.float64)
        REF.token_shift_mix(h, want_last, slots, cu, seq, mu, want)
        got = torch.zeros(S, n, W, device="cuda", dtype=dtype)
        K.token_shift_mix(h.cuda(), got_last, slots.cuda(), cu.cuda(), seq.cuda(), mu.cuda(), got)
        live = n - 1
        close(got[:, :live], want[:, :live], 1e-6 if dtype == torch.float32 else 0.02, "blends")
        close(got_last, want_last, 0.0, "saved rows")


SCAN_SHAPES = [(2, 8, 12), (3, 16, 8), (1, 24, 40), (3, 48, 48), (2, 64, 64), (2, 128, 300), (1, 130, 20), (2, 33, 600)]


@pytest.mark.parametrize("heads,dim,vdim", SCAN_SHAPES)
@pytest.mark.parametrize("form", ["constant", "data"])
def test_matrix_state_recurrence(K, heads, dim, vdim, form):
    """Retention's form (a constant decay per head, scaled keys, gate) and time mixing's (decay from a raw row, bonus,
    output before the update, norm weight), prompts + portions + single tokens, one launch and in blocks."""
    g = gen(heads * dim + vdim)
    hd, hv = heads * dim, heads * vdim
    decay = torch.rand(heads, generator=g) * 0.5 + 0.5 if form == "constant" else None
    w_bias = None if form == "constant" else -1.5 + torch.randn(hd, generator=g)
    bonus = None if form == "constant" else 0.5 * torch.randn(hd, generator=g)
    norm_w = None if form == "constant" else 1 + 0.2 * torch.randn(hv, generator=g)
    state_ref = torch.zeros(7, heads, dim, vdim, dtype=torch.float64)
    state = torch.zeros(7, heads, dim, vdim, device="cuda")
    old = [0, 0, 0]
    for lens in ([130, 2, 70], [1, 1, 1], [3, 200, 1]):
        cu, seq, slots = requests(lens, old, pad=1)
        n = int(cu[-1])
        wide = torch.randn(n, 3 * hd + 2 * hv + 3, generator=g)       # the operands are column slices of one product
        q, k, w = wide[:, :hd], wide[:, hd:2 * hd], wide[:, 2 * hd:3 * hd]
        v, gate = wide[:, 3 * hd:3 * hd + hv], wide[:, 3 * hd + hv:3 * hd + 2 * hv]
        want = torch.zeros(n, hv, dtype=torch.float64)
        kw = dict(decay=decay, w_bias=w_bias, key_scale=dim ** -0.5 if form == "constant" else 1.0, bonus=bonus,
                  norm_weight=norm_w, gate=gate if form == "constant" else None)
        REF.linear_scan(q, k, v, None if form == "constant" else w, heads, dim, vdim, state_ref, slots, cu, seq, want, 1e-5, **kw)
        wd = wide.cuda()
        dq, dk, dw = wd[:, :hd], wd[:, hd:2 * hd], wd[:, 2 * hd:3 * hd]
        dv, dg = wd[:, 3 * hd:3 * hd + hv], wd[:, 3 * hd + hv:3 * hd + 2 * hv]
        dkw = {a: (b.cuda() if torch.is_tensor(b) else b) for a, b in kw.items()}
        dkw["gate"] = dg if form == "constant" else None
        got = torch.zeros(n, hv, device="cuda")
        K.linear_scan(dq, dk, dv, None if form == "constant" else dw, heads, dim, vdim, state, slots.cuda(), cu.cuda(), seq.cuda(),
                      got, 1e-5, max_q_len=max(lens), **dkw)
        live = n - 1
        close(got[:live], want[:live], 2e-4, f"outputs of step {lens}")
        close(state, state_ref, 2e-4 * max(1.0, float(state_ref.abs().max())), "state")
        old = [a + b for a, b in zip(old, lens)]
    assert float(state[0].abs().max()) == 0.0          # the padding request's slot


@pytest.mark.parametrize("width", [7, 200, 1000])
def test_gated_unit_kernel(K, width):
    g = gen(width)
    zb, xb = torch.randn(width, generator=g), torch.randn(width, generator=g)
    state_ref, state = torch.zeros(6, width, dtype=torch.float64), torch.zeros(6, width, device="cuda")
    for lens in ([19, 1, 70], [1, 1, 1], [300, 2, 129], [1, 100, 1]):        # the last two: in chunks that run side by side
        cu, seq, slots = requests(lens, [4, 4, 4], pad=1)
        n = int(cu[-1])
        proj = 2 * torch.randn(n, 3 * width, generator=g)
        want, got = torch.zeros(n, width, dtype=torch.float64), torch.zeros(n, width, device="cuda")
        REF.gated_unit_scan(proj, zb, xb, state_ref, slots, cu, seq, want)
        K.gated_unit_scan(proj.cuda(), zb.cuda(), xb.cuda(), state, slots.cuda(), cu.cuda(), seq.cuda(), got, max_q_len=max(lens))
        close(got[:n - 1], want[:n - 1], 2e-5, "gated unit")
        close(state, state_ref, 1e-5, "gated unit state")


def _attention_case(K, H, G, d, dv, rot, inter, ps, dtype, lens_new, lens_old, window=0, plant=None, seed=0):
    """Stores ``lens_old`` tokens, then this step's, through rotary_store, and compares the attention of this step."""
    g = gen(seed + H * d + dv)
    base = 10000.0
    pages_n = 64
    kp_ref, vp_ref = torch.zeros(pages_n, G, ps, d, dtype=dtype), torch.zeros(pages_n, G, ps, dv, dtype=dtype)
    both = torch.zeros(pages_n, 2, G, ps, d, device="cuda", dtype=dtype) if d == dv else None      # one tensor with a stream axis
    kp = both[:, 0] if both is not None else torch.zeros(pages_n, G, ps, d, device="cuda", dtype=dtype)
    vp = both[:, 1] if both is not None else torch.zeros(pages_n, G, ps, dv, device="cuda", dtype=dtype)
    R = len(lens_new)
    order = torch.randperm(pages_n, generator=g).tolist()
    tables = torch.full((R, 24), -1, dtype=torch.int32)
    for r in range(R):
        need = -(-(lens_old[r] + lens_new[r]) // ps)
        tables[r, :need] = torch.tensor([order.pop() for _ in range(need)], dtype=torch.int32)

    def table_of(positions, dims):
        inv = base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
        ang = positions.double()[:, None] * inv[None, :]
        return torch.stack((ang.cos(), ang.sin()), dim=-1).flatten(-2).float()

    out_pair = None
    for phase, lens, olds in (("old", lens_old, [0] * R), ("new", lens_new, lens_old)):
        pos = torch.cat([torch.arange(o, o + n) for o, n in zip(olds, lens)]) if sum(lens) else torch.zeros(0, dtype=torch.long)
        n = pos.numel()
        if n == 0:
            continue
        slots = torch.cat([tables[r].long()[torch.arange(o, o + m) // ps] * ps + torch.arange(o, o + m) % ps
                           for r, (o, m) in enumerate(zip(olds, lens))]).int()
        qkv = torch.randn(n, H * d + G * (d + dv), generator=g)
        if plant is not None and phase == "new":
            qkv[:, :H * d] *= 0.05
        if plant is not None:                 # one key far back that every later query of request 0 looks for
            r0, where = plant
            row = (where - olds[r0]) + sum(lens[:r0])
            if olds[r0] <= where < olds[r0] + lens[r0]:
                qkv[row, H * d:(H + G) * d] = 0.0
                qkv[row, H * d + rot:H * d + rot + 1] = 30.0          # an entry that no rotation touches
                qkv[row, (H + G) * d:] = 5.0
            if phase == "new":
                qkv[:, rot] = 10.0
        qt, vt = (table_of(pos, rot) if rot else None), table_of(pos, dv)
        q_ref, q_got = torch.zeros(n, H * d, dtype=dtype), torch.zeros(n, H * d, device="cuda", dtype=dtype)
        REF.rotary_store(qkv, H, G, d, dv, qt, rot, inter, 1e-5, vt, inter, q_ref, kp_ref, vp_ref, slots)
        K.rotary_store(qkv.cuda(), H, G, d, dv, None if qt is None else qt.cuda(), rot, inter, 1e-5, vt.cuda(), inter, q_got, kp, vp,
                       slots.cuda())
        tol = 2e-6 if dtype == torch.float32 else 0.04
        close(q_got, q_ref, tol * 4, "rotated q")
        close(kp, kp_ref, tol * 4, "key pages")
        close(vp, vp_ref, tol * 2, "value pages")
        if phase == "new":
            cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
            seq = torch.tensor([a + b for a, b in zip(lens_old, lens_new)], dtype=torch.int32)
            want = torch.zeros(n, H * dv, dtype=torch.float64)
            REF.paged_attention_streams(q_ref, H, G, d, dv, kp_ref, vp_ref, tables, cu, seq, want, 0.3, window, vt, inter)
            got = torch.zeros(n, H * dv, device="cuda", dtype=dtype)
            K.paged_attention_streams(q_got, H, G, d, dv, kp, vp, tables.cuda(), cu.cuda(), seq.cuda(), got, 0.3, window, vt.cuda(),
                                      inter, max_q_len=max(lens), max_seq_len=int(seq.max()))
            close(got, want, 1e-5 if dtype == torch.float32 else 0.05, "attention")
            if both is not None and dtype == torch.bfloat16 and d % 16 == 0 and H // G <= 16:
                # the route of bfloat16 steps with keys and values of one width: the framework's tensor-core attention on the
                # entry's one tensor, the queries in a buffer of their own, then the turn back
                got2 = torch.zeros(n, H * dv, device="cuda", dtype=dtype)
                K.paged_attention(q_got, H, G, d, both, tables.cuda(), cu.cuda(), seq.cuda(), got2, 0.3, window, max(lens),
                                  int(seq.max()), min_q_len=min(lens))
                K.rotate_rows(got2, vt.cuda(), H, dv, dv, inter, back=True)
                close(got2, want, 0.05, "attention on tensor cores")
            out_pair = (got, want)
    return out_pair


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,rot,inter,ps", [(4, 2, 16, 8, 8, False, 16), (6, 6, 8, 16, 8, False, 8), (8, 2, 128, 128, 64, False, 16),
                                                    (3, 1, 24, 40, 12, True, 4), (2, 2, 64, 64, 0, False, 32), (5, 5, 256, 2, 256, False, 16),
                                                    (6, 2, 32, 32, 2, False, 16), (2, 2, 48, 48, 48, False, 16), (4, 4, 16, 16, 8, True, 16),
                                                    (4, 2, 80, 80, 40, False, 16), (2, 1, 96, 96, 96, False, 8), (2, 2, 256, 256, 64, False, 16),
                                                    (32, 1, 64, 64, 32, False, 16)])
def test_rotated_values_attention_kernels(K, H, G, d, dv, rot, inter, ps, dtype):
    _attention_case(K, H, G, d, dv, rot, inter, ps, dtype, [33, 1, 2, 1], [0, 70, 15, 16])
    _attention_case(K, H, G, d, dv, rot, inter, ps, dtype, [5, 1], [40, 40], window=7, seed=1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_far_key_holds_the_weight(K, dtype):
    """One key 300 positions back, at a page's last place, gets nearly all the softmax weight of every later query:
    the outputs are its value turned by the distance, which a lost or misplaced key, or a rotation by the wrong
    position, would change entirely."""
    for where in (15, 16, 31):
        got, want = _attention_case(K, 4, 2, 32, 16, 16, False, 16, dtype, [20, 1], [320, 333], plant=(0, where), seed=where)
        assert float(want[:20].abs().max()) > 0.5


def _moe_case(K, n, E, top, k, o, dtype, seed):
    g = gen(seed)
    logits = 3 * torch.randn(n, E, generator=g)
    ids_ref, gates_ref = torch.zeros(n, top, dtype=torch.int32), torch.zeros(n, top, dtype=torch.float64)
    REF.moe_route(logits, top, ids_ref, gates_ref)
    ids, gates = torch.zeros(n, top, device="cuda", dtype=torch.int32), torch.zeros(n, top, device="cuda")
    K.moe_route(logits.cuda(), top, ids, gates)
    assert torch.equal(ids.cpu(), ids_ref)
    close(gates, gates_ref, 2e-6, "gates")
    P_ = n * top
    off_ref, perm_ref, pos_ref = (torch.zeros(E + 1, dtype=torch.int32), torch.zeros(P_, dtype=torch.int32), torch.zeros(P_, dtype=torch.int32))
    REF.moe_plan(ids_ref, E, off_ref, perm_ref, pos_ref)
    off, perm, pos = (torch.zeros(E + 1, device="cuda", dtype=torch.int32), torch.zeros(P_, device="cuda", dtype=torch.int32),
                      torch.zeros(P_, device="cuda", dtype=torch.int32))
    K.moe_plan(ids, E, off, perm, pos)
    assert torch.equal(off.cpu(), off_ref) and torch.equal(perm.cpu(), perm_ref) and torch.equal(pos.cpu(), pos_ref)
    ids_b, gates_b = torch.zeros_like(ids), torch.zeros_like(gates)          # router and list in one call (one launch for few pairs)
    off_b, perm_b, pos_b = torch.zeros_like(off), torch.zeros_like(perm), torch.zeros_like(pos)
    K.moe_route_plan(logits.cuda(), top, ids_b, gates_b, off_b, perm_b, pos_b)
    assert torch.equal(ids_b, ids) and torch.equal(gates_b, gates) and torch.equal(off_b, off) and torch.equal(perm_b, perm) \
        and torch.equal(pos_b, pos)
    x = torch.randn(n, k, generator=g).to(dtype)
    w1 = (torch.randn(E, 2 * o, k, generator=g) / k ** 0.5).to(dtype)
    w2 = (torch.randn(E, k, o, generator=g) / o ** 0.5).to(dtype)
    act_ref, act = torch.zeros(P_, o, dtype=dtype), torch.zeros(P_, o, device="cuda", dtype=dtype)
    REF.moe_linear(x, w1, off_ref, perm_ref, top, act_ref, epilogue="silu_gate")
    K.moe_linear(x.cuda(), w1.cuda(), off, perm, top, act, epilogue="silu_gate")
    tol = 2e-5 if dtype == torch.float32 else 0.03
    close(act, act_ref, tol, "gate | up")
    y_ref, y = torch.zeros(P_, k, dtype=torch.float64), torch.zeros(P_, k, device="cuda")
    REF.moe_linear(act_ref, w2, off_ref, None, 1, y_ref)
    K.moe_linear(act.cuda(), w2.cuda(), off, None, 1, y)
    close(y, y_ref, tol * 2, "down")
    out_ref, out = torch.zeros(n, k, dtype=torch.float64), torch.zeros(n, k, device="cuda")
    REF.moe_combine(y_ref.float(), pos_ref, gates_ref.float(), out_ref)
    K.moe_combine(y, pos, gates, out)
    close(out, out_ref, tol * 2, "sum")
    if dtype == torch.bfloat16 and k % 8 == 0 and o % 8 == 0:
        # the padded list and the tcgen05 grouped products (the route of prompts), forced here whatever the number of pairs
        places = K.moe_padded_rows(P_, E)
        perm2, pos2 = torch.full((places,), -7, device="cuda", dtype=torch.int32), torch.zeros(P_, device="cuda", dtype=torch.int32)
        tiles = torch.full((places // K.MOE_TILE,), -7, device="cuda", dtype=torch.int32)
        K.moe_plan_padded(ids, E, off, perm2, pos2, tiles)
        starts, t_host = off.cpu().tolist(), tiles.cpu().tolist()
        counts = torch.bincount(ids_ref.reshape(-1).long(), minlength=E).tolist()
        assert all(a % K.MOE_TILE == 0 for a in starts) and starts[-1] == sum(-(-c // K.MOE_TILE) * K.MOE_TILE for c in counts)
        assert t_host == [e for e in range(E) for _ in range(-(-counts[e] // K.MOE_TILE))] + [-1] * (len(t_host) - starts[-1] // K.MOE_TILE)
        assert sorted(pos2.cpu().tolist()) == sorted(i for e in range(E) for i in range(starts[e], starts[e] + counts[e]))
        xs = torch.full((places, k), float("nan"), device="cuda", dtype=dtype)
        K.moe_gather(x.cuda(), perm2, top, tiles, xs)
        act2 = torch.full((places, o), float("nan"), device="cuda", dtype=dtype)
        K.moe_linear_grouped(xs, w1.cuda(), tiles, act2, epilogue="silu_gate")
        y2 = torch.full((places, k), float("nan"), device="cuda")
        K.moe_linear_grouped(act2, w2.cuda(), tiles, y2)
        out2 = torch.zeros(n, k, device="cuda")
        K.moe_combine(y2, pos2, gates, out2)
        K.check_device_errors()
        close(out2, out_ref, tol * 2, "sum through the padded list")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,E,top,k,o", [(1, 5, 2, 48, 24), (70, 10, 3, 160, 88), (9, 3, 3, 64, 40), (300, 40, 1, 72, 130), (33, 4, 2, 256, 128)])
def test_routed_experts_kernels(K, n, E, top, k, o, dtype):
    _moe_case(K, n, E, top, k, o, dtype, n + E)


def test_an_expert_that_nobody_chose_and_equal_logits(K):
    logits = torch.tensor([[1.0, 1.0, 1.0, 0.0], [0.0, 2.0, 2.0, -1.0]])
    ids, gates = torch.zeros(2, 2, device="cuda", dtype=torch.int32), torch.zeros(2, 2, device="cuda")
    K.moe_route(logits.cuda(), 2, ids, gates)
    assert ids.cpu().tolist() == [[0, 1], [1, 2]] and torch.allclose(gates.cpu(), torch.full((2, 2), 0.5))
    off, perm, pos = (torch.zeros(5, device="cuda", dtype=torch.int32), torch.zeros(4, device="cuda", dtype=torch.int32),
                      torch.zeros(4, device="cuda", dtype=torch.int32))
    K.moe_plan(ids, 4, off, perm, pos)
    assert off.cpu().tolist() == [0, 1, 3, 4, 4] and perm.cpu().tolist() == [0, 1, 2, 3]


def test_products_with_the_tanh_epilogue(K):
    g = gen(9)
    for n in (3, 70):
        for dtype in (torch.float32, torch.bfloat16):
            x, w = torch.randn(n, 64, generator=g).to(dtype), (torch.randn(16, 64, generator=g) / 4).to(dtype)
            want, got = torch.zeros(n, 16, dtype=torch.float64), torch.zeros(n, 16, device="cuda", dtype=dtype)
            REF.linear(x, w, want, epilogue="tanh")
            K.linear(x.cuda(), w.cuda(), got, epilogue="tanh")
            close(got, want, 2e-6 if dtype == torch.float32 else 0.01, "tanh")
    K.check_device_errors()


# ------------------------------------------------------------------------------ the engine
LENS = [37, 100, 64, 19, 130, 50, 1, 2, 3, 200]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("lunelorn"))
    out = {}
    for name in ("L1", "L2", "L3"):
        d = TL.make_model_dir(name, root)
        cfg, w = TL.load_model_dir(d)
        reqs = {f"r{i}": tiny.random_tokens(cfg["vocab"], n, 100 + i) for i, n in enumerate(LENS)}
        out[name] = (d, cfg, w, reqs, {r: P.forward(cfg, w, t).float() for r, t in reqs.items()})
    return out


def _runner(model_dir, name, dtype, pool):
    from infurnace_b200.engine.loading import EngineOptions, build_runner
    ps = TL.TINY[name]["page_size"]
    return build_runner(model_dir, EngineOptions(dtype=dtype, device="cuda", page_size=ps, num_pages=pool // ps, max_num_seqs=4,
                                                 max_num_batched_tokens=pool, max_model_len=pool))[2]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "bulk_tail", "portions", "mixed"])
@pytest.mark.parametrize("name", ["L1", "L2", "L3"])
def test_cutting_modes(models, name, mode, dtype):
    d, cfg, w, reqs, ref = models[name]
    steps = {"whole": tiny.schedule_whole, "bulk_tail": lambda r: tiny.schedule_bulk_tail(r, tail=40),
             "portions": lambda r: tiny.schedule_portions(r, seed=1),
             "mixed": lambda r: tiny.schedule_mixed(r, max_live=4, max_tokens=512, seed=2)}[mode](reqs)
    runner = _runner(d, name, dtype, 512)
    out = tiny.collect(steps, tiny.run_inprocess(runner, steps), cfg["vocab"])
    assert runner.cache.num_free_slots == 4
    assert runner.cache.free_pages() == [g.pool.num_pages for g in runner.cache.kv_groups]
    runner.rt.kernels.check_device_errors()
    if dtype == "float32":
        worst = max(rows_match(out[rid], ref[rid], dtype, f"{name} {mode} {dtype} request {rid}") for rid in reqs)
    else:         # the share of positions is taken over all requests (three of them have one to three tokens)
        worst = rows_match(torch.cat([out[rid] for rid in reqs]), torch.cat([ref[rid] for rid in reqs]), dtype, f"{name} {mode} {dtype}")
    print(f"{name} {mode} {dtype}: worst {worst:.3g} (largest logit {max(float(r.abs().max()) for r in ref.values()):.3g})")


OTHER_SIZES = {
    # width and feed-forward no multiple of 8 (the plain products), heads of 24 (no tensor-core attention), one expert, a loop
    # over the middle layer only, no side input
    "odd": TL._config(53, 100, 1e-5, [TL._ret(3, 12, 20, [0.3, 0.8, 0.99], TL._moe(1, 1, 36)),
                                      TL._par(6, 2, 24, 24, 6, 777.0, 0.2, 33, 0.7, 1.4, TL._moe(5, 5, 20)),
                                      TL._wkv(5, 20, 7, None)], loop=(1, 2, 2), cap=8.0),
    # heads of 48 and of 32 with keys and values of one width (the tensor-core attention at those sizes), as many key heads
    # as query heads and one for all, retention heads of 48 x 96, a loop over everything, side input of one column
    "tc": TL._config(211, 96, 1e-6, [TL._par(2, 2, 48, 48, 48, 5000.0, 0.15, 8, 1.0, 0.5, TL._moe(6, 2, 24)),
                                     TL._ret(2, 48, 96, [0.9, 0.999], None),
                                     TL._par(6, 1, 32, 32, 2, 20.0, 0.25, 96, 0.5, 1.0, TL._moe(3, 1, 40)),
                                     TL._wkv(3, 32, 16, TL._moe(2, 2, 8))], loop=(0, 4, 2), side=1),
    # a single layer; a time-mixing layer alone with one head
    "one": TL._config(40, 32, 1e-5, [TL._wkv(1, 32, 2, TL._moe(4, 3, 16))], side=5, cap=20.0),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(OTHER_SIZES))
def test_other_sizes_and_orders(tmp_path, name, dtype):
    """Models of other sizes, head counts, orders of layers and loops, in a mixed schedule over a small pool."""
    from infurnace_b200.engine.loading import EngineOptions, build_runner
    conf = OTHER_SIZES[name]
    d = TL.make_model_dir("_" + name, str(tmp_path), config=conf, seed=31, store="bfloat16")
    cfg, w = TL.load_model_dir(d)
    reqs = {f"r{i}": tiny.random_tokens(cfg["vocab"], n, 7 + i) for i, n in enumerate([45, 130, 3, 70, 1, 99, 20])}
    ref = {r: P.forward(cfg, w, t).float() for r, t in reqs.items()}
    steps = tiny.schedule_mixed(reqs, max_live=4, max_tokens=384, seed=3)
    runner = build_runner(d, EngineOptions(dtype=dtype, device="cuda", page_size=16, num_pages=24, max_num_seqs=4,
                                           max_num_batched_tokens=384, max_model_len=384))[2]
    out = tiny.collect(steps, tiny.run_inprocess(runner, steps), cfg["vocab"])
    runner.rt.kernels.check_device_errors()
    assert runner.cache.num_free_slots == 4 and runner.cache.free_pages() == [g.pool.num_pages for g in runner.cache.kv_groups]
    if dtype == "float32":
        for rid in reqs:
            rows_match(out[rid], ref[rid], dtype, f"{name} request {rid}", noise=float32_noise(cfg, w, reqs[rid]))
    else:
        # these models are worse conditioned than the three above (see float32_noise); the kernels' own tests are the sharp ones
        rows_match(torch.cat([out[r] for r in reqs]), torch.cat([ref[r] for r in reqs]), dtype, name, share=0.5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(models, dtype):
    """Every token alone from the first on, 300 of them."""
    d, cfg, w, _, _ = models["L3"]
    toks = tiny.random_tokens(cfg["vocab"], 300, 77)
    want = P.forward(cfg, w, toks).float()
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
    out = tiny.collect(steps, tiny.run_inprocess(_runner(d, "L3", dtype, 384), steps), cfg["vocab"])["x"]
    rows_match(out, want, dtype, "token by token")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_in_portions_then_decoding(models, dtype):
    """900 tokens: portions of 500, 133, 2 and 200 (the recurrences in blocks), then 65 tokens one by one, beside a
    second request that comes and goes."""
    d, cfg, w, _, _ = models["L3"]
    toks = tiny.random_tokens(cfg["vocab"], 900, 91)
    other = tiny.random_tokens(cfg["vocab"], 90, 92)
    want, want_other = P.forward(cfg, w, toks).float(), P.forward(cfg, w, other).float()
    steps, at = [], 0
    for i, n in enumerate([500, 133, 2, 200] + [1] * 65):
        entries = [{"id": "x", "tokens": toks[at:at + n], "want": list(range(n))}]
        if i == 1:
            entries.append({"id": "y", "tokens": other[:60], "want": list(range(60))})
        if 2 <= i < 32:
            entries.append({"id": "y", "tokens": [other[58 + i]], "want": [0]})
        steps.append({"step": i, "entries": entries, "end": ["y"] if i == 31 else []})
        at += n
    assert at == 900
    out = tiny.collect(steps, tiny.run_inprocess(_runner(d, "L3", dtype, 1088), steps), cfg["vocab"])
    rows_match(out["x"], want, dtype, "the long request")
    rows_match(out["y"], want_other, dtype, "the request beside it")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(models, tmp_path, dtype):
    d, cfg, w, reqs, ref = models["L2"]
    steps = tiny.schedule_mixed(reqs, max_live=4, max_tokens=512, seed=5)
    outputs = tiny.run_trace_run(d, dtype, steps, str(tmp_path / "out"), 512, TL.TINY["L2"]["page_size"])
    out = tiny.collect(steps, outputs, cfg["vocab"])
    rows_match(torch.cat([out[rid] for rid in reqs]), torch.cat([ref[rid] for rid in reqs]), dtype, "all requests")


def test_greedy_generation_through_the_engine_and_its_graphs(models):
    """The engine's own entry point: scheduler, portions beside decoded tokens, six requests over four slots, decode
    steps replayed from CUDA graphs.  In float32 the tokens are the plain implementation's."""
    from infurnace_b200.engine import Engine, EngineOptions, SamplingParams
    d, cfg, w, _, _ = models["L1"]
    ps = TL.TINY["L1"]["page_size"]
    prompts = [tiny.random_tokens(cfg["vocab"], n, 40 + n) for n in (1, 9, 33, 70, 5, 18)]
    want = [P.greedy(cfg, w, p, 16) for p in prompts]
    for graphs in (True, False):
        eng = Engine.from_model_dir(d, EngineOptions(dtype="float32", device="cuda", page_size=ps, num_pages=40, max_num_seqs=4,
                                                     max_num_batched_tokens=32))
        eng.runner.use_graphs = eng.runner.use_graphs and graphs
        assert eng.generate(prompts, SamplingParams(max_tokens=16)) == want
        assert (eng.runner.graph_replays > 0) == graphs
        eng.runner.cache.check()
        assert eng.runner.cache.num_free_slots == 4


def test_command_line(models, tmp_path):
    import json
    import os
    import subprocess
    import sys
    d, cfg, w, _, _ = models["L1"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bin", "infurnace-b200"), "--model", d, "--prompt-ids", "5,6,7,8",
                          "--max-tokens", "6", "--json", "--dtype", "float32", "--page-size", "16", "--max-context", "64"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    report = json.loads(out.stdout)
    assert report["generated_token_ids"] == P.greedy(cfg, w, [5, 6, 7, 8], 6) and report["model"]["architecture"] == "Lunelorn"
