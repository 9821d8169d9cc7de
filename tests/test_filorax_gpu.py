"""Filorax on the GPU: each new kernel alone against its plain statement (tests/kernel_refs.py, float64), and the engine
against the plain implementation (tests/plain_filorax.py) in every way of cutting the work, in float32 and in bfloat16,
through the step function, the trace program and greedy generation."""
import pytest
import torch

import plain_filorax as P
import tiny
import tiny_filorax as TF
from kernel_refs import ReferenceKernels

pytestmark = pytest.mark.gpu

REF = ReferenceKernels(torch.float64)
F32_TOL = 5e-5       # times the largest logit: float32 arithmetic against float64
BF16_TOL = 4e-2      # times the largest logit: activations between kernels carry 8 bits, and the tiny models' attention is peaked
BF16_SHARE = 0.7     # of the positions: a bfloat16 rounding can turn an expert choice, which the plain implementation does not follow


def rows_match(out, want, dtype, what="", share=None):
    """float32: every position within F32_TOL of the largest logit.  bfloat16: BF16_SHARE of the positions within BF16_TOL
    of it and the median within three quarters of that (the float32 runs are the sharp test of every mechanism; these show
    that the bfloat16 path computes the same model)."""
    top = max(1.0, float(want.abs().max()))
    err = (out.double() - want.double()).abs().max(dim=-1).values
    if dtype in ("float32", torch.float32):
        bad = err > F32_TOL * top
        assert not bool(bad.any()), f"{what}: position {int(bad.nonzero()[0])}: {float(err[bad][0])} > {F32_TOL * top}"
    else:
        good = float((err <= BF16_TOL * top).double().mean())
        assert good >= (share or BF16_SHARE) and float(err.median()) <= 0.75 * BF16_TOL * top, \
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
    """cu_q, seq_lens, state_slots, req_index (int32) for requests that bring lens_new tokens on top of lens_old; ``pad``
    more requests of length 0 with one row each (the padding of a recorded decode step)."""
    lens_old = lens_old or [0] * len(lens_new)
    cu, req = [0], []
    for r, n in enumerate(lens_new):
        cu.append(cu[-1] + n)
        req += [r] * n
    seq = [a + b for a, b in zip(lens_new, lens_old)]
    for i in range(pad):
        cu.append(cu[-1] + 1)
        seq.append(0)
        req.append(len(lens_new) + i)
    slots = [2 * i + 1 for i in range(len(lens_new))] + [0] * pad       # distinct, out of order with the rows, never slot 0
    return tuple(torch.tensor(v, dtype=torch.int32) for v in (cu, seq, slots, req))


# ------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("rows,width,groups", [(1, 33, 1), (7, 336, 2), (70, 2048, 8), (3, 2052, 3), (2, 5000, 5), (5, 48, 48)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_norm_in_groups(K, rows, width, groups, out_dtype):
    g = gen(rows + width)
    x, delta = torch.randn(rows, width, generator=g) * 3, torch.randn(rows, width, generator=g)
    x[:, : width // groups] *= 20.0                      # the groups' statistics differ by far
    w = (1 + 0.3 * torch.randn(width, generator=g)).to(torch.bfloat16)
    tol = 3e-6 * 60 if out_dtype == torch.float32 else 0.3
    for mult, with_delta, with_keep in ((1.0, False, False), (0.3, True, True), (1.7, True, False)):
        xr, xg = x.clone(), x.cuda()
        want, got = torch.zeros(rows, width, dtype=torch.float64), torch.zeros(rows, width, device="cuda", dtype=out_dtype)
        hist_r, hist_g = torch.zeros(rows, 3, width), torch.zeros(rows, 3, width, device="cuda")
        REF.group_rmsnorm(xr, w, groups, 1e-5, want, delta=delta if with_delta else None, mult=mult, keep=hist_r[:, 1] if with_keep else None)
        K.group_rmsnorm(xg, w.cuda(), groups, 1e-5, got, delta=delta.cuda() if with_delta else None, mult=mult,
                        keep=hist_g[:, 1] if with_keep else None)
        close(got, want, tol, "norm")
        close(xg, xr, 6e-5, "stream")
        close(hist_g, hist_r, 6e-5, "kept rows")
    pick = torch.tensor([rows - 1, 0], dtype=torch.int32)
    want, got = torch.zeros(2, width, dtype=torch.float64), torch.zeros(2, width, device="cuda", dtype=out_dtype)
    xr, xg = x.clone(), x.cuda()
    REF.group_rmsnorm(xr, w, groups, 1e-5, want, delta=delta, mult=0.5, rows=pick)
    K.group_rmsnorm(xg, w.cuda(), groups, 1e-5, got, delta=delta.cuda(), mult=0.5, rows=pick.cuda())
    close(got, want, tol, "picked rows")
    close(xg, x, 0.0, "a stream that stays as it was")


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_average_over_depth(K, out_dtype):
    g = gen(5)
    n, width, slots = 9, 200, 5
    coeffs = [torch.randn(d + 1, generator=g).to(torch.bfloat16) for d in range(slots)]
    hist_r = torch.zeros(n, slots, width)
    hist_g = hist_r.cuda()
    x = torch.randn(n, width, generator=g)
    hist_r[:, 0], hist_g[:, 0] = x, x.cuda()
    xr, xg = x.clone(), x.cuda()
    w = (1 + 0.3 * torch.randn(width, generator=g)).to(torch.bfloat16)
    for depth in range(1, slots):
        delta = torch.randn(n, width, generator=g)
        ahead = depth % 2 == 1
        want = torch.zeros(n, width, dtype=torch.float64) if ahead else None
        got = torch.zeros(n, width, device="cuda", dtype=out_dtype) if ahead else None
        REF.depth_average(xr, delta, 0.4, hist_r, depth, coeffs[depth], out=want, next_weight=w if ahead else None, groups=4, eps=1e-6)
        K.depth_average(xg, delta.cuda(), 0.4, hist_g, depth, coeffs[depth].cuda(), out=got, next_weight=w.cuda() if ahead else None,
                        groups=4, eps=1e-6)
        close(xg, xr, 2e-5, f"stream at depth {depth}")
        close(hist_g, hist_r, 2e-5, "history")
        if ahead:
            close(got, want, 2e-4 if out_dtype == torch.float32 else 0.1, "the next norm")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,width", [(4, 320), (1, 40), (2, 33), (3, 1000), (6, 64), (16, 8), (5, 2048), (40, 264), (8, 512), (2, 256), (7, 4096)])
def test_input_convolution_over_steps_and_slots(K, dtype, taps, width):
    """Requests advance by portions of every length around the convolution's reach; what a token sees never depends on the
    cutting: every step's outputs equal the convolution over the whole sequences."""
    g = gen(taps * width)
    w = (0.5 * torch.randn(width, taps, generator=g)).to(torch.bfloat16)
    state_r = torch.zeros(9, max(taps - 1, 1), width)
    state_g = state_r.cuda()
    whole = [torch.randn(0, width).to(dtype) for _ in range(4)]
    outs = [[] for _ in range(4)]
    old = [0, 0, 0, 0]
    for lens in ([1, taps + 3, 2, 40], [1, 1, 1, taps], [2, 1, taps - 1 or 1, 1], [taps, 2, 1, 70], [300, 701, 1, 200], [1, 1, 2, 1]):
        cu, seq, slots, req = requests(lens, old, pad=2)
        n = int(cu[-1])
        h = torch.randn(n, width, generator=g).to(dtype)
        want, got = torch.zeros(n, width, dtype=torch.float64), torch.zeros(n, width, device="cuda", dtype=dtype)
        REF.causal_conv(h, w, state_r, slots, cu, seq, req, want)
        K.causal_conv(h.cuda(), w.cuda(), state_g, slots.cuda(), cu.cuda(), seq.cuda(), req.cuda(), got)
        close(got, want, 1e-5 if dtype == torch.float32 else 0.06, f"portions {lens}")
        close(state_g, state_r, 1e-6, "state")
        for r in range(4):
            whole[r] = torch.cat((whole[r], h[int(cu[r]):int(cu[r + 1])]))
            outs[r].append(want[int(cu[r]):int(cu[r + 1])])
        old = [a + b for a, b in zip(old, lens)]
    for r in range(4):                       # against the sum written out over the whole sequence
        seq_in = torch.cat((torch.zeros(taps - 1, width, dtype=torch.float64), whole[r].double()))
        direct = whole[r].double() + sum(w[:, j].double() * seq_in[j:j + whole[r].shape[0]] for j in range(taps))
        close(torch.cat(outs[r]), direct, 1e-9, "the stand-in itself")


def _latent_case(K, H, D, V, R, rot, dims, ps, dtype, lens_new, lens_old, window=0, sink=True, plant=None, seed=0, scale=0.3):
    """Stores ``lens_old`` tokens and then this step's through latent_prepare, and compares the attention of this step.
    ``plant`` = (request, position): that token's latent gets one large entry and every query of the last step looks for
    it, so that it holds nearly all the weight where it is visible."""
    g = gen(seed + H * R + rot)
    pages_n = 96
    lat_r, lat_g = torch.zeros(pages_n, 1, ps, R, dtype=dtype), torch.zeros(pages_n, 1, ps, R, device="cuda", dtype=dtype)
    rk_r = torch.zeros(pages_n, 1, ps, rot, dtype=dtype) if rot else None
    rk_g = rk_r.cuda() if rot else None
    nreq = len(lens_new)
    order = torch.randperm(pages_n, generator=g).tolist()
    tables = torch.full((nreq, 40), -1, dtype=torch.int32)
    for r in range(nreq):
        need = -(-(lens_old[r] + lens_new[r]) // ps)
        tables[r, :need] = torch.tensor([order.pop() for _ in range(need)], dtype=torch.int32)
    down_col = H * (D + rot) + 3                                   # the latent need not follow the queries directly
    stride = down_col + R + rot + H * V
    norm_w = (1 + 0.2 * torch.randn(R, generator=g)).to(torch.bfloat16 if dtype == torch.bfloat16 else torch.float32)
    sinks = (0.5 + torch.randn(H, generator=g)).to(norm_w.dtype) if sink else None
    w_abs = torch.randn(H, R, D, generator=g).to(dtype) / D ** 0.5
    base = 50.0
    result = None
    for phase, lens, olds in (("old", lens_old, [0] * nreq), ("new", lens_new, lens_old)):
        if not sum(lens):
            continue
        pos = torch.cat([torch.arange(o, o + n) for o, n in zip(olds, lens)])
        n = pos.numel()
        slots = torch.cat([tables[r].long()[torch.arange(o, o + m) // ps] * ps + torch.arange(o, o + m) % ps
                           for r, (o, m) in enumerate(zip(olds, lens))]).int()
        proj = torch.randn(n, stride, generator=g)
        if plant is not None:
            r0, where = plant
            if olds[r0] <= where < olds[r0] + lens[r0]:
                row = (where - olds[r0]) + sum(lens[:r0])
                proj[row, down_col:down_col + R] = 0.01
                proj[row, down_col + 1] = 100.0                    # after the norm: one entry of about sqrt(R), the rest none
        table = None
        if rot:
            inv = base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
            ang = pos.double()[:, None] * inv[None, :]
            table = torch.stack((ang.cos(), ang.sin()), dim=-1).flatten(-2).float()
        seg = n + 5
        qp_r, qp_g = torch.zeros(H, seg, D, dtype=dtype), torch.zeros(H, seg, D, device="cuda", dtype=dtype)
        qr_r = torch.zeros(n, H, rot) if rot else None
        qr_g = qr_r.cuda() if rot else None
        off_r, off_g = torch.zeros(H + 1, dtype=torch.int32), torch.zeros(H + 1, dtype=torch.int32, device="cuda")
        REF.latent_prepare(proj, H, D, rot, R, down_col, norm_w, 1e-5, table, dims, qp_r, qr_r, lat_r, rk_r, slots, off_r)
        K.latent_prepare(proj.cuda(), H, D, rot, R, down_col, norm_w.cuda(), 1e-5, None if table is None else table.cuda(), dims, qp_g,
                         qr_g, lat_g, rk_g, slots.cuda(), off_g)
        tol = 3e-6 if dtype == torch.float32 else 0.02
        close(qp_g, qp_r, tol * 5, "unrotated queries")
        close(lat_g, lat_r, tol * 12, "latent pages")
        assert off_g.tolist() == off_r.tolist() == [h * seg for h in range(H + 1)]
        if rot:
            close(qr_g, qr_r, 2e-5, "rotated queries")
            close(rk_g, rk_r, tol * 5, "rotated key pages")
        if phase != "new":
            continue
        q_lat = torch.einsum("hsd,hrd->hsr", qp_r.double(), w_abs.double()).float()
        if plant is not None:
            q_lat *= 0.05
            q_lat[:, :, 1] = 40.0 / scale / R ** 0.5               # a score of about 40 at the planted key
        cu, seq, _, req = requests(lens_new, lens_old)
        want = torch.zeros(H, seg, R, dtype=torch.float64)
        got = torch.zeros(H, seg, R, device="cuda", dtype=dtype)
        REF.latent_attention(q_lat, qr_r, lat_r, rk_r, tables, cu, seq, req, sinks, want, scale, window, n)
        K.latent_attention(q_lat.cuda(), qr_g, lat_g, rk_g, tables.cuda(), cu.cuda(), seq.cuda(), req.cuda(),
                           None if sinks is None else sinks.cuda(), got, scale, window, n)
        close(got[:, :n], want[:, :n], 2e-5 if dtype == torch.float32 else 0.05, "attention over latents")
        if dtype == torch.bfloat16:
            # with the step's extents: the tensor-core kernel where the sizes allow it, alone and with the context divided
            for min_keys in (256, 64):
                before, K.split_min_keys, keep = K.latent_mma_calls, min_keys, K.split_min_keys
                got = torch.full((H, seg, R), float("nan"), device="cuda", dtype=dtype)
                K.latent_attention(q_lat.cuda(), qr_g, lat_g, rk_g, tables.cuda(), cu.cuda(), seq.cuda(), req.cuda(),
                                   None if sinks is None else sinks.cuda(), got, scale, window, n, max_q_len=max(lens_new),
                                   max_seq_len=int(seq.max()))
                K.split_min_keys = keep
                assert (K.latent_mma_calls > before) == (R % 8 == 0 and R <= 256 and rot % 8 == 0)
                close(got[:, :n], want[:, :n], 0.05 if plant is None else 0.12, "attention over latents on tensor cores")
        w_val = torch.randn(H, V, R, generator=g)
        y = torch.einsum("hsr,hvr->hsv", want.float(), w_val)
        gate = proj[:, down_col + R + rot:]
        for gt in (gate, None):
            o_r, o_g = torch.zeros(n, H * V, dtype=torch.float64), torch.zeros(n, H * V, device="cuda", dtype=dtype)
            REF.gate_heads(y, gt, o_r, n)
            K.gate_heads(y.cuda(), None if gt is None else proj.cuda()[:, down_col + R + rot:], o_g, n)
            close(o_g, o_r, 1e-5 * float(y.abs().max()) if dtype == torch.float32 else 0.02 * float(y.abs().max()), "gated heads")
        result = (got[:, :n].float().cpu(), want[:, :n], lat_r)
    return result


SHAPES = [(8, 64, 80, 128, 16, 16, 16), (6, 32, 48, 128, 0, 0, 16), (3, 8, 10, 12, 6, 6, 8), (2, 12, 8, 16, 0, 0, 4),
          (16, 128, 128, 256, 64, 32, 16), (5, 24, 40, 72, 8, 8, 16), (1, 16, 16, 520, 2, 2, 32), (32, 16, 16, 64, 32, 32, 16)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,V,R,rot,dims,ps", SHAPES)
def test_latent_attention_kernels(K, H, D, V, R, rot, dims, ps, dtype):
    _latent_case(K, H, D, V, R, rot, dims, ps, dtype, [33, 1, 2, 1], [0, 70, 15, 16])
    _latent_case(K, H, D, V, R, rot, dims, ps, dtype, [5, 1, 70], [40, 40, 0], window=7, seed=1)
    _latent_case(K, H, D, V, R, rot, dims, ps, dtype, [1, 1, 1, 1, 1], [0, 1, 129, 63, 64], window=64, sink=False, seed=2)
    _latent_case(K, H, D, V, R, rot, dims, ps, dtype, [130, 17], [0, 100], window=0, sink=False, seed=3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sink", [True, False])
def test_a_far_key_and_the_windows_edges(K, dtype, sink):
    """A planted latent holds nearly all the weight of every query that sees it.  Far back without a window, at a page's
    first and last place; and with a window of w, planted w - 1 positions before the last query (just inside: the
    output is that latent) and w positions before it (just outside: it is not), in a portion and for single tokens."""
    H, R = 4, 32
    for where in (15, 16, 31):
        got, want, lat = _latent_case(K, H, 16, 16, R, 8, 8, 16, dtype, [20, 1], [320, 333], sink=sink, plant=(0, where), seed=where)
        assert float(want[:, :20, 1].min()) > 0.9 * R ** 0.5 * 0.8
    for w in (40, 33, 16, 1):
        for new, old in (([6], [70]), ([1], [75])):
            last = old[0] + new[0] - 1
            got, want, _ = _latent_case(K, H, 16, 16, R, 0, 0, 16, dtype, new, old, window=w, sink=sink, plant=(0, last - w + 1), seed=w)
            assert float(want[:, -1, 1].min()) > 0.9 * R ** 0.5 * 0.8, (w, "inside")
            if w >= new[0] > 1:
                assert float(want[:, 0, 1].min()) > 0.9 * R ** 0.5 * 0.8      # the portion's first query sees it too
            got, want, _ = _latent_case(K, H, 16, 16, R, 0, 0, 16, dtype, new, old, window=w, sink=sink, plant=(0, last - w), seed=w)
            assert float(want[:, -1, 1].abs().max()) < 0.5 * R ** 0.5, (w, "outside")
            if w >= new[0] > 1:
                assert float(want[:, 0, 1].min()) > 0.9 * R ** 0.5 * 0.8      # the portion's first query still sees it


@pytest.mark.parametrize("E,top,count,keep,extra", [(8, 3, 2, 1, 1), (6, 3, 3, 2, 0), (4, 4, 1, 1, 1), (64, 6, 8, 3, 0), (40, 1, 40, 1, 2),
                                                   (12, 4, 4, 4, 0), (256, 8, 8, 4, 0)])
def test_router_over_all_experts_in_groups(K, E, top, count, keep, extra):
    """Scores are the softmax over all experts; only the best groups' experts are chosen; weights are scores times a scale.
    The logits' rows may carry more columns than experts (the shared expert's gate rides along)."""
    g = gen(E + top)
    for n in (1, 7, 300):
        logits = torch.randn(n, E + extra, generator=g) * 2
        if n > 4:
            logits[3, :E] = 0.0                                      # all equal: the lower index wins
            logits[4, :E] = logits[4, :E].round()                    # many ties
        ids_r, gates_r = torch.zeros(n, top, dtype=torch.int32), torch.zeros(n, top, dtype=torch.float64)
        REF.moe_route(logits, top, ids_r, gates_r, experts=E, scoring="all", groups=(count, keep), weight_scale=2.5)
        ids_g, gates_g = torch.zeros(n, top, dtype=torch.int32, device="cuda"), torch.zeros(n, top, device="cuda")
        K.moe_route(logits.cuda(), top, ids_g, gates_g, experts=E, scoring="all", groups=(count, keep), weight_scale=2.5)
        assert ids_g.cpu().tolist() == ids_r.tolist()
        close(gates_g, gates_r, 1e-6, "weights")
        per = E // count
        allowed = ids_r.long() // per
        assert all(len(set(row.tolist())) <= keep for row in allowed)
        if n * top <= 4096 and E <= 256:
            off, perm, pos = (torch.zeros(E + 1, dtype=torch.int32, device="cuda"), torch.zeros(n * top, dtype=torch.int32, device="cuda"),
                              torch.zeros(n * top, dtype=torch.int32, device="cuda"))
            ids2, gates2 = torch.zeros_like(ids_g), torch.zeros_like(gates_g)
            K.moe_route_plan(logits.cuda(), top, ids2, gates2, off, perm, pos, experts=E, scoring="all", groups=(count, keep), weight_scale=2.5)
            assert ids2.cpu().tolist() == ids_r.tolist()
            close(gates2, gates_r, 1e-6, "weights of the one-launch form")
            off_r, perm_r, pos_r = torch.zeros(E + 1, dtype=torch.int32), torch.zeros(n * top, dtype=torch.int32), torch.zeros(n * top, dtype=torch.int32)
            REF.moe_plan(ids_r, E, off_r, perm_r, pos_r)
            assert off.cpu().tolist() == off_r.tolist() and perm.cpu().tolist() == perm_r.tolist() and pos.cpu().tolist() == pos_r.tolist()


def test_weighted_sum_with_a_shared_expert(K):
    g = gen(3)
    n, top, width = 11, 3, 130
    y, shared = torch.randn(n * top, width, generator=g), torch.randn(n, width, generator=g)
    pos = torch.randperm(n * top, generator=g).int()
    gates = torch.rand(n, top, generator=g)
    logits = torch.randn(n, 9, generator=g) * 3
    for sh, lg in ((None, None), (shared, None), (shared, logits[:, 8])):
        want, got = torch.zeros(n, width, dtype=torch.float64), torch.zeros(n, width, device="cuda")
        REF.moe_combine(y, pos, gates, want, sh, lg)
        K.moe_combine(y.cuda(), pos.cuda(), gates.cuda(), got, None if sh is None else sh.cuda(), None if lg is None else logits.cuda()[:, 8])
        close(got, want, 1e-5, "weighted sum")


# ------------------------------------------------------------------------------ the engine
LENS = [37, 100, 64, 19, 85, 50, 1, 2, 3, 150]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("filorax"))
    out = {}
    for name in ("F1", "F2", "F3"):
        d = TF.make_model_dir(name, root)
        cfg, w = TF.load_model_dir(d)
        reqs = {f"r{i}": tiny.random_tokens(cfg["vocab"], n, 100 + i) for i, n in enumerate(LENS)}
        out[name] = (d, cfg, w, reqs, {r: P.forward(cfg, w, t).float() for r, t in reqs.items()})
    return out


def _runner(model_dir, name, dtype, pool):
    from infurnace_b200.engine.loading import EngineOptions, build_runner
    ps = TF.TINY[name]["page_size"]
    return build_runner(model_dir, EngineOptions(dtype=dtype, device="cuda", page_size=ps, num_pages=pool // ps, max_num_seqs=4,
                                                 max_num_batched_tokens=pool, max_model_len=pool))[2]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "bulk_tail", "portions", "mixed"])
@pytest.mark.parametrize("name", ["F1", "F2", "F3"])
def test_cutting_modes(models, name, mode, dtype):
    d, cfg, w, reqs, ref = models[name]
    steps = {"whole": tiny.schedule_whole, "bulk_tail": lambda r: tiny.schedule_bulk_tail(r, tail=60),
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
    # widths that are no multiple of 8 (the plain products), heads of 24 + 10, a rank of 40, one expert, five norm groups, two taps
    "odd": TF._config(53, 100, 1e-5, 5, 0.8, 2, [
        TF._rot(3, 24, 10, 20, 40, 0.2, 777.0, TF._moe(1, 1, 36)),
        TF._win(6, 12, 6, 20, 0.3, 33, TF._moe(5, 5, 20, shared=12)),
        TF._win(5, 20, 7, 28, 0.25, 3, None, plain=True)]),
    # sizes the tensor-core routes take throughout: ranks of 64, 128 and 256, rotated parts of 16 and 64, many heads, windows of
    # 64 (a page's multiple) and 17, groups of which most are dropped, and a rotated width that is rotated only in part
    "tc": {**TF._config(211, 128, 1e-6, 1, 0.3, 4, [
        TF._rot(16, 32, 16, 32, 64, 0.15, 5000.0, TF._moe(16, 4, 64, groups=(8, 2), scale=2.0, shared=64)),
        TF._win(8, 64, 64, 128, 0.1, 64, TF._moe(8, 2, 32, groups=(4, 1), scale=1.5)),
        TF._rot(4, 64, 64, 64, 256, 0.1, 20.0, None),
        TF._win(2, 128, 128, 64, 0.08, 17, TF._moe(4, 1, 128, shared=128), plain=True)])},
    # a latent and a rotated key part of one width (their page streams have the same shape), with one head and with several
    "equal": TF._config(61, 64, 1e-5, 2, 0.5, 3, [
        TF._rot(3, 16, 32, 16, 32, 0.2, 100.0, TF._moe(4, 2, 32, groups=(2, 1), shared=16)),
        TF._win(2, 16, 16, 32, 0.25, 21, None),
        TF._rot(1, 8, 16, 24, 16, 0.3, 10000.0, TF._moe(2, 1, 16))]),
    # a single layer: the average over depth of the embedding's output and one result
    "one": TF._config(40, 32, 1e-5, 2, 1.0, 3, [TF._win(1, 32, 16, 16, 0.2, 10, TF._moe(4, 2, 16, groups=(2, 1)))]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(OTHER_SIZES))
def test_other_sizes_and_orders(tmp_path, name, dtype):
    """Models of other sizes, head counts and orders of layers, in a mixed schedule over a small pool."""
    from infurnace_b200.engine.loading import EngineOptions, build_runner
    conf = OTHER_SIZES[name]
    d = TF.make_model_dir("_" + name, str(tmp_path), config=conf, seed=31, store="bfloat16")
    cfg, w = TF.load_model_dir(d)
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
            rows_match(out[rid], ref[rid], dtype, f"{name} request {rid}")
    else:
        rows_match(torch.cat([out[r] for r in reqs]), torch.cat([ref[r] for r in reqs]), dtype, name, share=0.6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(models, dtype):
    """Every token alone from the first on, 300 of them: windows of 33 and 50 pass over decoded tokens many times, pages of
    the windowed layers go back and come again."""
    d, cfg, w, _, _ = models["F3"]
    toks = tiny.random_tokens(cfg["vocab"], 300, 77)
    want = P.forward(cfg, w, toks).float()
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
    out = tiny.collect(steps, tiny.run_inprocess(_runner(d, "F3", dtype, 384), steps), cfg["vocab"])["x"]
    rows_match(out, want, dtype, "token by token")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_in_portions_then_decoding(models, dtype):
    """900 tokens: portions of 500, 133, 2 and 200, then 65 tokens one by one, beside a second request that comes and goes."""
    d, cfg, w, _, _ = models["F3"]
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
    out = tiny.collect(steps, tiny.run_inprocess(_runner(d, "F3", dtype, 1088), steps), cfg["vocab"])
    rows_match(out["x"], want, dtype, "the long request")
    rows_match(out["y"], want_other, dtype, "the request beside it")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(models, tmp_path, dtype):
    d, cfg, w, reqs, ref = models["F2"]
    steps = tiny.schedule_mixed(reqs, max_live=4, max_tokens=512, seed=5)
    outputs = tiny.run_trace_run(d, dtype, steps, str(tmp_path / "out"), 512, TF.TINY["F2"]["page_size"])
    out = tiny.collect(steps, outputs, cfg["vocab"])
    rows_match(torch.cat([out[rid] for rid in reqs]), torch.cat([ref[rid] for rid in reqs]), dtype, "all requests")


def test_greedy_generation_through_the_engine_and_its_graphs(models):
    """The engine's own entry point: scheduler, portions beside decoded tokens, six requests over four slots, decode
    steps replayed from CUDA graphs.  In float32 the tokens are the plain implementation's."""
    from infurnace_b200.engine import Engine, EngineOptions, SamplingParams
    d, cfg, w, _, _ = models["F1"]
    ps = TF.TINY["F1"]["page_size"]
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
    d, cfg, w, _, _ = models["F1"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bin", "infurnace-b200"), "--model", d, "--prompt-ids", "5,6,7,8",
                          "--max-tokens", "6", "--json", "--dtype", "float32", "--page-size", "16", "--max-context", "64"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    report = json.loads(out.stdout)
    assert report["generated_token_ids"] == P.greedy(cfg, w, [5, 6, 7, 8], 6) and report["model"]["architecture"] == "Filorax"
