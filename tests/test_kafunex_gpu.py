"""Kafunex on the GPU: each new kernel alone against its plain statement (tests/kernel_refs.py, float64), and the
engine against the plain implementation (tests/plain_kafunex.py) in every way of cutting the work, in float32 and in
bfloat16, through the step function, the trace program and greedy generation."""
import copy
import math

import pytest
import torch

import plain_kafunex as P
import tiny
import tiny_kafunex as TK
from kernel_refs import ReferenceKernels

pytestmark = pytest.mark.gpu

REF = ReferenceKernels(torch.float64)
F32_TOL = 2e-5
BF16_TOL = 4e-2      # times the largest logit: activations between kernels carry 8 bits, and the tiny models' attention is peaked


def bf16_tol(ref):
    return BF16_TOL * max(1.0, max(float(r.abs().max()) for r in ref))


@pytest.fixture(scope="module")
def K():
    from infurnace_b200.kernels import load_cuda_kernels
    return load_cuda_kernels()


def gen(seed):
    return torch.Generator().manual_seed(seed)


def close(got, want, tol, what=""):
    err = float((got.double().cpu() - want.double().cpu()).abs().max())
    assert err <= tol, f"{what}: {err} > {tol}"


# ------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("width,table_dtype", [(33, torch.float32), (336, torch.bfloat16), (64, torch.float32)])
def test_embedding_with_position_vector(K, width, table_dtype):
    g = gen(width)
    table = torch.randn(50, width, generator=g).to(table_dtype)
    ids = torch.randint(0, 50, (9,), generator=g, dtype=torch.int32)
    pos = torch.tensor([0, 1, 2, 63, 64, 1000, 12345, 400000, 1048575], dtype=torch.int32)
    inv = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange((width + 1) // 2, dtype=torch.float64) / width)
    want = torch.zeros(9, width)
    REF.embed_sinusoid(table, ids, pos, inv, want)
    got, half = torch.zeros(9, width, device="cuda"), torch.zeros(9, width, device="cuda", dtype=torch.bfloat16)
    K.embed_sinusoid(table.cuda(), ids.cuda(), pos.cuda(), inv.cuda(), got, half)
    close(got, want, 2e-6, "embedding")
    assert torch.equal(half.cpu(), got.cpu().to(torch.bfloat16))


@pytest.mark.parametrize("rows,width", [(1, 33), (7, 336), (70, 2048), (3, 2052), (2, 5000)])
def test_residual_update_with_norm_and_layer_scale(K, rows, width):
    g = gen(rows * width)
    x, y = torch.randn(rows, width, generator=g), 5 * torch.randn(rows, width, generator=g)
    gw, ls = torch.tensor(1.3), 1 + 0.3 * torch.randn(width, generator=g)
    want = x.clone().double()
    REF.residual_postnorm(want, y, gw, ls, 1e-5)
    xd, half = x.cuda(), torch.zeros(rows, width, device="cuda", dtype=torch.bfloat16)
    K.residual_postnorm(xd, y.cuda(), gw.cuda(), ls.cuda(), 1e-5, half)
    close(xd, want, 3e-6, "residual update")
    assert torch.equal(half.cpu(), xd.cpu().to(torch.bfloat16))
    xb = x.cuda()
    K.residual_postnorm(xb, y.cuda(), gw.cuda().bfloat16(), ls.cuda().bfloat16(), 1e-5)       # weights as a bfloat16 folder stores them
    want = x.clone().double()
    REF.residual_postnorm(want, y, gw.bfloat16(), ls.bfloat16(), 1e-5)
    close(xb, want, 3e-6, "residual update, bfloat16 weights")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,d,ps,own_v", [(4, 2, 16, 16, False), (3, 1, 24, 8, True), (6, 6, 8, 4, False)])
def test_whole_projection_norm_and_store(K, heads, kv, d, ps, own_v, dtype):
    g = gen(heads * d)
    n, qw, kw = 11, heads * d, kv * d
    ld = qw + kw + (kw if own_v else 0) + 5
    proj = torch.randn(n, ld, generator=g) * 3
    wq, wk = 1 + 0.2 * torch.randn(qw, generator=g), 1 + 0.2 * torch.randn(kw, generator=g)
    slots = torch.tensor([17, 3, -1, 40, 41, 42, 0, 9, 63, 25, 31], dtype=torch.int32)
    v_col = qw + kw if own_v else -1
    pages = torch.full((64 // ps, 2, kv, ps, d), 7.0)
    want_q, want_p = torch.zeros(n, qw, dtype=torch.float64), pages.clone().double()
    REF.wide_norm_store(proj, qw, kw, v_col, d, wq, wk, 1e-5, want_q, slots, want_p)
    got_q = torch.zeros(n, qw, device="cuda", dtype=dtype)
    got_p = pages.to(dtype).cuda()
    K.wide_norm_store(proj.cuda(), qw, kw, v_col, d, wq.cuda(), wk.cuda(), 1e-5, got_q, slots.cuda(), got_p)
    tol = 1e-5 if dtype == torch.float32 else 0.05
    close(got_q, want_q, tol, "q"), close(got_p, want_p, tol, "pages")
    got_q2 = torch.zeros_like(got_q)
    K.wide_norm_store(proj.cuda(), qw, kw, v_col, d, None, None, 1e-5, got_q2, None, None)      # no norm, nothing stored
    close(got_q2, proj[:, :qw], tol, "q without norm")


def _scan_inputs(heads, dim, vdim, n, seed):
    g = gen(seed)
    hd, hv = heads * dim, heads * vdim
    proj = torch.randn(n, 2 * hd + hv + 3, generator=g)
    proj[:, hd:2 * hd] *= 3
    return proj, torch.randn(hd, generator=g), 0.05 + 0.9 * torch.rand(hd, generator=g), 1 + 0.2 * torch.randn(vdim, generator=g)


@pytest.mark.parametrize("heads,dim,vdim", [(2, 8, 12), (1, 24, 40), (2, 40, 33), (3, 100, 64), (2, 32, 600), (1, 64, 300),
                                            (2, 160, 48)])
def test_gated_recurrence_kernel(K, heads, dim, vdim):
    """Unequal requests in one call (one of them padding), states that are not zero, and the same tokens cut into
    a prompt, a portion and single tokens: the state carries everything."""
    lens = [37, 1, 5, 0, 18, 200]                              # the fourth is padding: one row, length 0
    cu = [0, 37, 38, 43, 44, 62, 262]
    n, hd, hv = cu[-1], heads * dim, heads * vdim
    proj, bias, lower, nw = _scan_inputs(heads, dim, vdim, n, heads + dim + vdim)
    slots = torch.tensor([2, 0, 5, 0, 3, 6], dtype=torch.int32)
    state0 = torch.randn(7, heads, dim, vdim, generator=gen(1))
    want_state, want = state0.clone().double(), torch.zeros(n, hv, dtype=torch.float64)
    seq = torch.tensor([100, 1, 9, 0, 18, 333], dtype=torch.int32)
    REF.gated_scan(proj, 0, hd, 2 * hd, bias, lower, nw, 1e-5, want_state, slots, torch.tensor(cu, dtype=torch.int32), seq, want,
                   heads, dim, vdim)
    raw = torch.zeros(n, hv, device="cuda") if K.gated_scan_slabs(dim, vdim) > 1 else None
    assert (raw is not None) == (vdim > 256 and dim <= 128)
    state = state0.cuda()
    got = torch.zeros(n, hv, device="cuda")
    K.gated_scan(proj.cuda(), 0, hd, 2 * hd, bias.cuda(), lower.cuda(), nw.cuda(), 1e-5, state, slots.cuda(),
                 torch.tensor(cu, dtype=torch.int32).cuda(), seq.cuda(), got, heads, dim, vdim, raw=raw)
    rows = [i for i in range(n) if i != 43]
    close(got[rows], want[rows], 2e-5, "outputs"), close(state, want_state, 2e-5, "states")
    assert torch.equal(state[1].cpu(), state0[1]) and torch.equal(state[4].cpu(), state0[4])      # slots of nobody
    # request 0 again, cut 20 + 2 + 15 single tokens, from the same start: same outputs, same final state
    state2 = state0.cuda()
    got2 = torch.zeros(37, hv, device="cuda")
    start = 0
    for count in [20, 2] + [1] * 15:
        c = torch.tensor([0, count], dtype=torch.int32).cuda()
        K.gated_scan(proj[start:start + count].contiguous().cuda(), 0, hd, 2 * hd, bias.cuda(), lower.cuda(), nw.cuda(), 1e-5,
                     state2, slots[:1].cuda(), c, seq[:1].cuda(), got2[start:start + count], heads, dim, vdim,
                     raw=raw[:count] if raw is not None else None)
        start += count
    close(got2, want[:37], 2e-5, "outputs of the cut request"), close(state2[2], want_state[2], 2e-5, "its state")
    # the same step with the requests cut into blocks that run side by side
    state3, got3, before = state0.cuda(), torch.zeros(n, hv, device="cuda"), K.scan_blocked_calls
    K.gated_scan(proj.cuda(), 0, hd, 2 * hd, bias.cuda(), lower.cuda(), nw.cuda(), 1e-5, state3, slots.cuda(),
                 torch.tensor(cu, dtype=torch.int32).cuda(), seq.cuda(), got3, heads, dim, vdim, raw=raw, max_q_len=1000)
    assert K.scan_blocked_calls == before + 1           # (heads of more than 128 rows run their one kernel all the same)
    close(got3[rows], want[rows], 2e-5, "outputs in blocks"), close(state3, want_state, 2e-5, "states in blocks")
    out_bf = torch.zeros(n, hv, device="cuda", dtype=torch.bfloat16)
    K.gated_scan(proj.cuda(), 0, hd, 2 * hd, bias.cuda(), lower.cuda(), nw.cuda(), 1e-5, state0.cuda(), slots.cuda(),
                 torch.tensor(cu, dtype=torch.int32).cuda(), seq.cuda(), out_bf, heads, dim, vdim, raw=raw)
    close(out_bf[rows], want[rows], 0.05, "bfloat16 outputs")


def _attention_case(K, H, G, d, ps, chunk, dtype, lens_and_new, seed, talk=True, gate=True, slope=8.0, plant=None):
    """Requests of (length after the step, new tokens) over a shuffled page pool; compares kernel and statement."""
    g = gen(seed)
    R = len(lens_and_new)
    max_pages = max(-(-L // ps) for L, _ in lens_and_new)
    n_pages = sum(-(-L // ps) for L, _ in lens_and_new) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    bt = torch.full((R, max_pages), -1, dtype=torch.int32)
    for r, (L, _) in enumerate(lens_and_new):
        for i in range(-(-L // ps)):
            bt[r, i] = order.pop()
    pages = torch.randn(n_pages, 2, G, ps, d, generator=g)
    cu = [0]
    for _, new in lens_and_new:
        cu.append(cu[-1] + new)
    n = cu[-1]
    q = torch.randn(n, H * d, generator=g) * 1.5
    if plant is not None:                 # make one key's score stand out for the last query of request 0
        key_pos, size = plant
        L, new = lens_and_new[0]
        page, off = int(bt[0, key_pos // ps]), key_pos % ps
        for h in range(H):
            pages[page, 0, h // (H // G), off] = q[new - 1, h * d:(h + 1) * d] * size / d
        pages[page, 1, :, off] = 9.0
    tk = (torch.eye(H) + 0.5 * torch.randn(H, H, generator=g)) if talk else None
    gt = torch.randn(n, H * d + 7, generator=g) if gate else None
    seq = torch.tensor([L for L, _ in lens_and_new], dtype=torch.int32)
    cu_t = torch.tensor(cu, dtype=torch.int32)
    # entries of the block tables below a query's chunk are never read: poison them for the kernel
    bt_dev = bt.clone()
    if chunk:
        for r, (L, new) in enumerate(lens_and_new):
            first_needed = ((L - new) // chunk) * chunk // ps
            bt_dev[r, :first_needed] = -1
    pq, pp = q.to(dtype), pages.to(dtype)
    want = torch.zeros(n, H * d, dtype=torch.float64)
    REF.attention_talk(pq, H, G, d, pp, bt, cu_t, seq, want, 0.3, chunk, slope, tk, gt, 7 if gate else 0)
    got = torch.zeros(n, H * d, device="cuda", dtype=dtype)
    K.attention_talk(pq.cuda(), H, G, d, pp.cuda(), bt_dev.cuda(), cu_t.cuda(), seq.cuda(), got, 0.3, chunk=chunk,
                     slope_exponent=slope, talk=tk.cuda() if talk else None, gate=gt.cuda() if gate else None,
                     gate_col=7 if gate else 0, max_q_len=max(new for _, new in lens_and_new),
                     max_seq_len=max(L for L, _ in lens_and_new))
    return got, want


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,ps,chunk", [(4, 2, 16, 16, 24), (6, 6, 8, 8, 0), (3, 1, 24, 8, 32), (8, 2, 64, 16, 100),
                                            (5, 5, 40, 4, 9), (2, 1, 128, 32, 300), (16, 4, 32, 16, 64),
                                            (32, 8, 64, 16, 128), (24, 6, 32, 8, 50), (40, 8, 16, 16, 0)])
def test_talking_attention_kernel(K, H, G, d, ps, chunk, dtype):
    """Whole prompts, portions that begin and end inside a chunk and inside a page, single tokens just before, on
    and after a chunk's edge, and a padding row."""
    c = chunk or 50
    cases = [(70, 70), (c + 1, 1), (c, 1), (2 * c - 1, 1), (2 * c + 5, c + 3), (1, 1), (3 * c + 2, 2), (0, 1), (210, 1)]
    before = K.talk_mma_calls
    got, want = _attention_case(K, H, G, d, ps, chunk, dtype, cases, seed=H * d + chunk)
    close(got, want, 5e-5 if dtype == torch.float32 else 0.06, "attention")      # outputs of size 3; 32 heads mixed in float32
    assert (K.talk_mma_calls > before) == (dtype == torch.bfloat16 and d in (16, 32, 64, 128))      # which kernel ran


@pytest.mark.parametrize("chunk", [512, 0, 300])
def test_talking_attention_with_the_keys_split_over_ctas(K, chunk):
    """Decoded tokens over long contexts: the keys of a query are shared out to several CTAs and merged; a request
    shorter than one share, one at a chunk's first position and a padding row are among them."""
    cases = [(700, 1), (33, 1), (1500, 1), (0, 1), (512, 1), (513, 1), (1, 1), (1024, 2)]
    for H, G, d in ((8, 2, 64), (32, 4, 32)):               # one group of heads; two groups (a cluster) per tile
        before = K.talk_split_calls
        got, want = _attention_case(K, H, G, d, 16, chunk, torch.bfloat16, cases, seed=chunk + H)
        assert K.talk_split_calls == before + 1
        close(got, want, 0.06, f"split keys, {H} heads")


def test_talking_attention_variants(K):
    for kw in (dict(talk=False), dict(gate=False), dict(slope=0.0), dict(talk=False, gate=False, slope=0.0)):
        got, want = _attention_case(K, 4, 2, 16, 8, 20, torch.float32, [(45, 45), (33, 1), (7, 3)], seed=3, **kw)
        close(got, want, 2e-5, str(kw))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_far_key_and_the_keys_at_a_chunks_edge(K, dtype):
    """One key among hundreds holds nearly all the weight of the last query: inside the chunk it must be found (its
    value is 9 everywhere), one position before the chunk's first it must not be seen; as a decoded token and as the
    last token of a portion that straddles the chunk's edge."""
    for key_pos, seen in ((400, True), (399, False), (1099, True)):
        for new in (1, 23, 395):
            L = 1100 if key_pos > 1000 else 790
            got, want = _attention_case(K, 4, 4, 16, 16, 400, dtype, [(L, new)], seed=11, talk=False, gate=False, slope=0.0,
                                        plant=(key_pos, 400.0))
            close(got, want, 1e-4 if dtype == torch.float32 else 0.08, f"planted key at {key_pos}, portion of {new}")      # values of size 9
            assert (float(got[-1].float().abs().min()) > 8.9) == seen, (key_pos, new)


@pytest.mark.parametrize("epilogue", ["relu2", "silu", "sigmoid", "gelu_tanh"])
def test_products_with_a_unary_epilogue(K, epilogue):
    """On each product kernel: plain float32, few rows, tensor cores one tile per CTA, shared k range, many rows."""
    g = gen(7)
    for n, o, k, dtype in [(5, 70, 33, torch.float32), (3, 96, 64, torch.bfloat16), (40, 200, 128, torch.bfloat16),
                           (100, 416, 288, torch.bfloat16), (48, 128, 2048, torch.bfloat16), (700, 512, 256, torch.bfloat16)]:
        x, w = torch.randn(n, k, generator=g).to(dtype), (torch.randn(o, k, generator=g) / k ** 0.5).to(dtype)
        for out_dtype in (torch.float32, dtype):
            want = torch.zeros(n, o, dtype=torch.float64)
            REF.linear(x, w, want, epilogue=epilogue)
            got = torch.zeros(n, o, device="cuda", dtype=out_dtype)
            K.linear(x.cuda(), w.cuda(), got, epilogue=epilogue)
            tol = 1e-5 if dtype == torch.float32 else (2e-5 if out_dtype == torch.float32 else 0.01)
            rel = (got.double().cpu() - want).abs() / (1.0 + want.abs())          # relu(y)^2 reaches 20: rounding is relative
            assert float(rel.max()) <= tol, f"{epilogue} {n}x{o}x{k} {dtype} -> {out_dtype}: {float(rel.max())}"
    K.check_device_errors()


# ------------------------------------------------------------------------------ the engine
LENS = [37, 100, 64, 19, 130, 50, 1, 2, 3, 200]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("kafunex"))
    out = {}
    for name in ("K1", "K2", "K3"):
        d = TK.make_model_dir(name, root)
        cfg, w = P.read_model(d)
        reqs = {f"r{i}": tiny.random_tokens(cfg["vocab"], n, 100 + i) for i, n in enumerate(LENS)}
        out[name] = (d, cfg, w, reqs, {r: P.forward(cfg, w, t).float() for r, t in reqs.items()})
    return out


def _runner(model_dir, name, dtype, pool):
    from infurnace_b200.engine.loading import EngineOptions, build_runner
    ps = TK.TINY[name]["page_size"]
    return build_runner(model_dir, EngineOptions(dtype=dtype, device="cuda", page_size=ps, num_pages=pool // ps, max_num_seqs=4,
                                                 max_num_batched_tokens=pool, max_model_len=pool))[2]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "bulk_tail", "portions", "mixed"])
@pytest.mark.parametrize("name", ["K1", "K2", "K3"])
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
    tol = F32_TOL if dtype == "float32" else bf16_tol(ref.values())
    worst = ("", 0, 0.0)
    for rid in reqs:
        err = (out[rid] - ref[rid]).abs().max(dim=-1).values
        if float(err.max()) > worst[2]:
            worst = (rid, int(err.argmax()), float(err.max()))
    print(f"{name} {mode} {dtype}: worst {worst[2]:.3g} (largest logit {max(float(r.abs().max()) for r in ref.values()):.3g})")
    assert worst[2] <= tol, f"{name} {mode} {dtype}: first look at request {worst[0]} position {worst[1]}: {worst[2]}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(models, dtype):
    """Every token alone from the first on, 330 of them: over three edges of the chunk of 100 and six of the chunk of 48."""
    d, cfg, w, _, _ = models["K3"]
    toks = tiny.random_tokens(cfg["vocab"], 330, 77)
    want = P.forward(cfg, w, toks).float()
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
    out = tiny.collect(steps, tiny.run_inprocess(_runner(d, "K3", dtype, 384), steps), cfg["vocab"])["x"]
    err = (out - want).abs().max(dim=-1).values
    assert float(err.max()) <= (F32_TOL if dtype == "float32" else bf16_tol([want])), f"position {int(err.argmax())}: {float(err.max())}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_in_portions_then_decoding(models, dtype):
    """1,500 tokens: portions of 700, 333, 2 and 400 (the recurrence in blocks, attention tiles with shared-out keys,
    many chunk edges inside portions), then 65 tokens one by one, beside a second request that comes and goes."""
    d, cfg, w, _, _ = models["K3"]
    toks = tiny.random_tokens(cfg["vocab"], 1500, 91)
    other = tiny.random_tokens(cfg["vocab"], 90, 92)
    want, want_other = P.forward(cfg, w, toks).float(), P.forward(cfg, w, other).float()
    steps, at = [], 0
    for i, n in enumerate([700, 333, 2, 400] + [1] * 65):
        entries = [{"id": "x", "tokens": toks[at:at + n], "want": list(range(n))}]
        if i == 1:
            entries.append({"id": "y", "tokens": other[:60], "want": list(range(60))})
        if 2 <= i < 32:
            entries.append({"id": "y", "tokens": [other[58 + i]], "want": [0]})
        steps.append({"step": i, "entries": entries, "end": ["y"] if i == 31 else []})
        at += n
    assert at == 1500
    out = tiny.collect(steps, tiny.run_inprocess(_runner(d, "K3", dtype, 1664), steps), cfg["vocab"])
    tol = F32_TOL * 2 if dtype == "float32" else bf16_tol([want])
    err = (out["x"] - want).abs().max(dim=-1).values
    assert float(err.max()) <= tol, f"position {int(err.argmax())}: {float(err.max())}"
    assert float((out["y"] - want_other).abs().max()) <= tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(models, tmp_path, dtype):
    d, cfg, w, reqs, ref = models["K2"]
    steps = tiny.schedule_mixed(reqs, max_live=4, max_tokens=512, seed=5)
    outputs = tiny.run_trace_run(d, dtype, steps, str(tmp_path / "out"), 512, TK.TINY["K2"]["page_size"])
    out = tiny.collect(steps, outputs, cfg["vocab"])
    for rid in reqs:
        assert float((out[rid] - ref[rid]).abs().max()) <= (F32_TOL if dtype == "float32" else bf16_tol(ref.values()))


def test_greedy_generation_through_the_engine_and_its_graphs(models):
    """The engine's own entry point: scheduler, portions beside decoded tokens, six requests over four slots, decode
    steps replayed from CUDA graphs.  In float32 the tokens are the plain implementation's."""
    from infurnace_b200.engine import Engine, EngineOptions, SamplingParams
    d, cfg, w, _, _ = models["K1"]
    ps = TK.TINY["K1"]["page_size"]
    prompts = [tiny.random_tokens(cfg["vocab"], n, 40 + n) for n in (1, 9, 33, 70, 5, 18)]
    want = [P.greedy(cfg, w, p, 24) for p in prompts]
    for graphs in (True, False):
        eng = Engine.from_model_dir(d, EngineOptions(dtype="float32", device="cuda", page_size=ps, num_pages=40, max_num_seqs=4,
                                                     max_num_batched_tokens=32))
        eng.runner.use_graphs = eng.runner.use_graphs and graphs
        assert eng.generate(prompts, SamplingParams(max_tokens=24)) == want
        assert (eng.runner.graph_replays > 0) == graphs
        eng.runner.cache.check()
        assert eng.runner.cache.num_free_slots == 4


def test_command_line_and_random_weights(models, tmp_path):
    """The command line on a model folder of this design (greedy: the plain implementation's tokens), and random weights
    drawn from a configuration file that names its architecture with the single key."""
    import json
    import os
    import subprocess
    import sys
    d, cfg, w, _, _ = models["K1"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bin", "infurnace-b200"), "--model", d, "--prompt-ids", "5,6,7,8",
                          "--max-tokens", "6", "--json", "--dtype", "float32", "--page-size", "16", "--max-context", "64"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    report = json.loads(out.stdout)
    assert report["generated_token_ids"] == P.greedy(cfg, w, [5, 6, 7, 8], 6) and report["model"]["architecture"] == "Kafunex"
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(TK.TINY["K2"]["config"]))
    out = subprocess.run([sys.executable, "-m", "infurnace_b200", "--random-weights", "3", "--config", str(cfg_path),
                          "--prompt", "hello", "--char-tokenizer", "--max-tokens", "5", "--page-size", "8", "--max-context", "64",
                          "--json"], capture_output=True, text=True, timeout=600, cwd=root)
    assert out.returncode == 0, out.stderr
    assert len(json.loads(out.stdout)["generated_token_ids"]) == 5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_new_parts_in_another_arrangement(dtype):
    """A plain embedding (the block makes the stream's bfloat16 copy itself), attention with values of its own and none of
    the options, a gelu feed-forward: on the GPU kernels, a prompt portion and then single tokens."""
    from infurnace_b200.cache import CacheManager
    from infurnace_b200.engine.runner import ModelRunner, StepEntry
    from infurnace_b200.kernels import load_cuda_kernels
    from infurnace_b200.parts import DecoderModel, Runtime
    plan, w, toks, want = TK.another_arrangement()
    dev = torch.device("cuda")
    rt = Runtime(device=dev, act_dtype=dtype, kernels=load_cuda_kernels())
    cache = CacheManager(plan, page_size=4, num_pages=16, max_requests=2, dtype=dtype, device=dev)
    runner = ModelRunner(DecoderModel(plan, {k: v.to(dev, dtype) for k, v in w.items()}, rt), cache, rt, 64, 64)
    cache.add_request("a")
    got = [runner.step([StepEntry("a", toks[:13], list(range(13)))]).float().cpu().clone()]
    got += [runner.step([StepEntry("a", [t], [0])]).float().cpu().clone() for t in toks[13:]]
    err = float((torch.cat(got).double() - want).abs().max())
    assert err <= (F32_TOL if dtype == torch.float32 else bf16_tol([want])), err
