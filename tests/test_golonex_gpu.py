"""Golonex on the GPU: each new or extended kernel alone against its plain statement (tests/kernel_refs.py, float64), and
the engine against the plain implementation (tests/plain_golonex.py) in every way of cutting the work, in float32 and in
bfloat16, through the step function, the trace program and greedy generation."""
import pytest
import torch

import plain_golonex as P
import tiny
import tiny_golonex as TG
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


def cuda(*ts):
    return tuple(t.cuda() if t is not None else None for t in ts)


# ------------------------------------------------------------------------------ the recurrent unit's kernels alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,width,blocks", [(4, 320, 4), (1, 40, 1), (2, 33, 3), (3, 1000, 10), (7, 64, 64), (5, 2048, 16)])
def test_convolution_over_steps_and_slots(K, dtype, taps, width, blocks):
    """Several steps over the same slots: portions longer and shorter than the taps' reach, single tokens, a padding row."""
    g = gen(taps * 1000 + width)
    Kp = max(taps - 1, 1)
    xb, cw, cb = torch.randn(width, generator=g), torch.randn(width, taps, generator=g), torch.randn(width, generator=g)
    st_r = torch.zeros(8, Kp, width)
    st_g = st_r.cuda()
    old = [0, 0, 0]
    for step, lens in enumerate(([9, 1, 2], [1, 1, 1], [2, taps, 30], [1, 3, 1], [taps + 1, 1, 2])):
        cu, seq, slots, req = requests(lens, old, pad=1 if step == 1 else 0)
        n = int(cu[-1])
        seg = n + (step % 2) * 5
        proj = torch.randn(n, 2 * width + 3, generator=g)
        u_r, ub_r = torch.zeros(n, width, dtype=torch.float64), torch.zeros(blocks, seg, width // blocks, dtype=torch.float64)
        u_g, ub_g = torch.zeros(n, width, device="cuda"), torch.zeros(blocks, seg, width // blocks, device="cuda", dtype=dtype)
        off_r, off_g = torch.zeros(blocks + 1, dtype=torch.int32), torch.zeros(blocks + 1, dtype=torch.int32, device="cuda")
        REF.rglru_conv(proj, width + 3, xb, cw, cb, st_r, slots, cu, seq, req, u_r, ub_r, off_r)
        K.rglru_conv(proj.cuda(), width + 3, xb.cuda(), cw.cuda(), cb.cuda(), st_g, *cuda(slots, cu, seq, req), u_g, ub_g, off_g)
        close(u_g, u_r, 2e-5, f"step {step}")
        close(ub_g[:, :n], ub_r[:, :n], 2e-5 if dtype == torch.float32 else 0.08, f"step {step}, block-major")
        close(st_g, st_r, 1e-6, f"step {step}, the inputs kept")
        assert off_g.tolist() == [b * seg for b in range(blocks + 1)]
        old = [a + b for a, b in zip(old, lens)]


@pytest.mark.parametrize("width,blocks", [(320, 4), (33, 3)])
def test_convolution_hands_the_gates_two_terms(K, width, blocks):
    """A block's row twice as long: the bfloat16 roundings, then what each rounding left out; together 16 bits of every number."""
    g = gen(width)
    taps, n, bs = 3, 21, width // blocks
    cu, seq, slots, req = requests([15, 6])
    proj = torch.randn(n, 2 * width, generator=g) * 3
    xb, cw, cb = torch.randn(width, generator=g), torch.randn(width, taps, generator=g), torch.randn(width, generator=g)
    st = torch.zeros(8, taps - 1, width, device="cuda")
    u = torch.zeros(n, width, device="cuda")
    ub = torch.full((blocks, n + 4, 2 * bs), 9.0, device="cuda", dtype=torch.bfloat16)
    off = torch.zeros(blocks + 1, dtype=torch.int32, device="cuda")
    K.rglru_conv(proj.cuda(), width, xb.cuda(), cw.cuda(), cb.cuda(), st, *cuda(slots, cu, seq, req), u, ub, off)
    want = u.view(n, blocks, bs).transpose(0, 1).double().cpu()
    first, rest = ub[:, :n, :bs].double().cpu(), ub[:, :n, bs:].double().cpu()
    assert torch.equal(first, want.to(torch.bfloat16).double())
    assert float(((first + rest) - want).abs().max()) <= 2.0 ** -16 * float(want.abs().max())
    assert float((first - want).abs().max()) > 2.0 ** -11 * float(want.abs().max())          # one term alone is far coarser
    assert float(ub[:, n:].float().min()) == 9.0 and off.tolist() == [b * (n + 4) for b in range(blocks + 1)]


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,blocks", [(96, 3), (33, 1), (1000, 8), (260, 260)])
def test_recurrence_in_one_launch_and_in_chunks(K, out_dtype, width, blocks):
    """A prompt, a portion on top of it and single tokens, with decays from almost 1 to almost 0, states that are not zero,
    slots out of order and a padding row; the chunked form (long portions) against the same statement."""
    g = gen(width)
    bs = width // blocks
    ab, ib, yb = (0.5 * torch.randn(width, generator=g) for _ in range(3))
    lam = torch.linspace(-9.0, 4.0, width)
    st_r = torch.randn(8, width, generator=g)
    st_g = st_r.cuda()
    old = [0, 0, 0]
    tol = 3e-5 if out_dtype == torch.float32 else 0.05
    for step, lens in enumerate(([200, 3, 70], [1, 1, 1], [130, 2, 65], [1, 1, 1])):
        cu, seq, slots, req = requests(lens, old, pad=1 if step in (1, 3) else 0)
        n = int(cu[-1])
        seg = n + 3
        gates = torch.randn(blocks, seg, 2 * bs, generator=g) * 2
        u, proj = torch.randn(n, width, generator=g), torch.randn(n, width + 5, generator=g)
        out_r, out_g = torch.zeros(n, width, dtype=torch.float64), torch.zeros(n, width, device="cuda", dtype=out_dtype)
        REF.rglru_scan(gates, ab, ib, lam, 8.0, u, proj, 5, yb, st_r, slots, cu, seq, out_r)
        before = K.rglru_chunked_calls
        K.rglru_scan(*cuda(gates, ab, ib, lam), 8.0, u.cuda(), proj.cuda(), 5, yb.cuda(), st_g, *cuda(slots, cu, seq), out_g,
                     max_q_len=max(lens))
        assert (K.rglru_chunked_calls > before) == (max(lens) >= K.scan_block_min)
        close(out_g, out_r, tol * max(1.0, float(out_r.abs().max())), f"step {step}")
        close(st_g, st_r, 3e-5 * max(1.0, float(st_r.abs().max())), f"step {step}, state")
        old = [a + b for a, b in zip(old, lens)]


def test_stretched_rotation_table_and_values_that_are_keys(K):
    g = gen(3)
    n, H, G, d, dims, ps = 11, 4, 2, 12, 8, 4
    pos = torch.randint(0, 5000, (n,), generator=g, dtype=torch.int32)
    freq = torch.rand(dims // 2, generator=g)
    tab_r, tab_g = torch.zeros(n, dims), torch.zeros(n, dims, device="cuda")
    REF.rope_table(pos, freq, tab_r, gain=1.0693)
    K.rope_table(pos.cuda(), freq.cuda(), tab_g, gain=1.0693)
    close(tab_g, tab_r, 2e-3, "table")                 # float32 angles of some thousands
    for dtype in (torch.float32, torch.bfloat16):
        qk = torch.randn(n, (H + G) * d, generator=g)
        slots = torch.randperm(5 * ps, generator=g)[:n].to(torch.int32)
        slots[2] = -1
        q_r, q_g = torch.zeros(n, H * d, dtype=torch.float64), torch.zeros(n, H * d, device="cuda", dtype=dtype)
        pages_r = torch.zeros(5, 2, G, ps, d, dtype=torch.float64)
        pages_g = torch.zeros(5, 2, G, ps, d, device="cuda", dtype=dtype)
        REF.rotary_store(qk, H, G, d, d, tab_r, dims, True, None, None, False, q_r, pages_r[:, 0], pages_r[:, 1], slots, values_are_keys=True)
        K.rotary_store(qk.cuda(), H, G, d, d, tab_r.cuda(), dims, True, None, None, False, q_g, pages_g[:, 0], pages_g[:, 1], slots.cuda(),
                       values_are_keys=True)
        tol = 1e-5 if dtype == torch.float32 else 0.05
        close(q_g, q_r, tol, "q")
        close(pages_g, pages_r, tol, "pages")
        live = [i for i in range(n) if int(slots[i]) >= 0]
        s0 = int(slots[live[0]])
        want_v = qk[live[0], H * d:H * d + d].double()           # the value is the key before its rotation
        close(pages_g[s0 // ps, 1, 0, s0 % ps], want_v, tol, "a value")
        assert float((pages_r[s0 // ps, 0, 0, s0 % ps] - want_v).abs().max()) > 0.1


def _attention_case(g, H, G, d, ps, lens_new, lens_old, dtype, window, plant):
    """Pages of rotated keys and raw values for requests with shuffled block tables; ``plant`` = (request, distance): the key
    that far behind the request's last query is scaled so that its score stands out for that query."""
    r = len(lens_new)
    total = [a + b for a, b in zip(lens_new, lens_old)]
    pages_per = [-(-t // ps) for t in total]
    n_pages = sum(pages_per) + 2
    order = torch.randperm(n_pages, generator=g).tolist()
    bt = torch.full((r, max(pages_per)), -1, dtype=torch.int32)
    pages = torch.zeros(n_pages, 2, G, ps, d)
    at = 0
    keys = []
    for i in range(r):
        k = torch.randn(total[i], G, d, generator=g)
        keys.append(k)
        for j in range(pages_per[i]):
            bt[i, j] = order[at]
            span = k[j * ps:(j + 1) * ps]
            pages[order[at], 0, :, :span.shape[0]] = span.transpose(0, 1)
            pages[order[at], 1, :, :span.shape[0]] = (span * 0.5 + 1.0).transpose(0, 1)
            at += 1
    n = sum(lens_new)
    q = torch.randn(n, H * d, generator=g)
    if plant is not None:
        req, dist = plant
        last_row = sum(lens_new[:req + 1]) - 1
        pos = total[req] - 1 - dist
        kp = keys[req][pos]                                      # [G, d]
        q[last_row] = (kp / kp.norm(dim=-1, keepdim=True) * 6.0).repeat_interleave(H // G, dim=0).reshape(-1)
        page, off = int(bt[req, pos // ps]), pos % ps
        pages[page, 0, :, off] *= 4.0
    cu, seq, _, _ = requests(lens_new, lens_old)
    return q.to(dtype), pages.to(dtype), bt, cu, seq


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,dist", [(40, 39), (40, 40), (33, 32), (33, 33), (16, 15), (16, 16), (1, 0), (0, 303), (0, 304)])
def test_a_far_key_and_the_windows_edges(K, dtype, window, dist):
    """A planted key that holds all the weight w - 1 positions behind the last query (just inside the window) and w behind
    (just outside), far back at a page's first and last place without a window; as the last token of a portion and as a
    single decoded token beside another request."""
    H, G, d, ps = 4, 2, 32, 16
    for lens_new, lens_old in (([50, 20], [270, 3]), ([1, 1], [319, 22])):
        g = gen(window * 7 + dist)
        q, pages, bt, cu, seq = _attention_case(g, H, G, d, ps, lens_new, lens_old, dtype, window, (0, dist))
        n = q.shape[0]
        want, got = torch.zeros(n, H * d, dtype=torch.float64), torch.zeros(n, H * d, device="cuda", dtype=dtype)
        REF.paged_attention(q.double(), H, G, d, pages.double(), bt, cu, seq, want, 0.5, window, max(lens_new), max(seq.tolist()))
        K.paged_attention(q.cuda(), H, G, d, pages.cuda(), bt.cuda(), cu.cuda(), seq.cuda(), got, 0.5, window, max(lens_new),
                          max(seq.tolist()), min_q_len=min(lens_new))
        tol = 2e-5 if dtype == torch.float32 else 0.06
        close(got, want, tol * max(1.0, float(want.abs().max())), f"window {window}, distance {dist}, {lens_new}")
        row = lens_new[0] - 1
        pos = lens_new[0] + lens_old[0] - 1 - dist
        planted_v = pages[int(bt[0, pos // ps]), 1, :, pos % ps].double().repeat_interleave(H // G, dim=0).reshape(-1)
        inside = window == 0 or dist < window
        assert (float((want[row] - planted_v).abs().max()) < 0.05) == inside         # the case shows what it is meant to show


def test_softmax_weights_in_two_terms(K):
    """Every query sees three keys, one with the largest score and two whose weight relative to it, 0.33295, lies just below
    the middle of two bfloat16 numbers and is rounded down by 0.28 %.  With one term every output carries a bias of a tenth
    of a percent; with two terms (the rounding and what it left out) only the output's own rounding remains, which has no
    sign."""
    g = gen(17)
    n, ps = 400, 16
    scale = 1.09976                                   # exp(-scale) = 0.33295
    cu, seq, _, req = requests([n])
    bt = torch.randperm(n // ps, generator=g).to(torch.int32).view(1, -1)
    low = (torch.arange(n) % 3 != 0).float().view(n // ps, ps)                       # the keys that score lower, by position
    low = low[torch.argsort(bt[0].long())]                                          # ... laid out by page
    # attention over keys and values
    H, G, d = 4, 2, 64
    pages = torch.zeros(n // ps, 2, G, ps, d)
    pages[:, 0, :, :, 0] = -low[:, None, :]
    pages[:, 1] = 1.0 + torch.rand(n // ps, G, ps, d, generator=g)                  # values in (1, 2): sums keep their sign
    pages = pages.to(torch.bfloat16)
    q = torch.zeros(n, H, d)
    q[:, :, 0] = 1.0
    q = q.view(n, H * d).to(torch.bfloat16)
    want = torch.zeros(n, H * d, dtype=torch.float64)
    REF.paged_attention(q.double(), H, G, d, pages.double(), bt, cu, seq, want, scale, 3, n, n)
    bias = {}
    for terms in (1, 2):
        got = torch.zeros(n, H * d, device="cuda", dtype=torch.bfloat16)
        K.paged_attention(q.cuda(), H, G, d, pages.cuda(), bt.cuda(), cu.cuda(), seq.cuda(), got, scale, 3, n, n, min_q_len=n,
                          weight_terms=terms)
        bias[terms] = float((got.double().cpu()[2:] / want[2:] - 1.0).mean())
    assert -1.6e-3 < bias[1] < -0.7e-3 and abs(bias[2]) < 2e-4, bias
    # attention over latents: entry 0 of a latent is what the query reads, the others are compared
    heads, rank = 3, 64
    lat = 1.0 + torch.rand(n // ps, 1, ps, rank, generator=g)
    lat[:, 0, :, 0] = -low
    lat = lat.to(torch.bfloat16)
    q_lat = torch.zeros(heads, n, rank)
    q_lat[:, :, 0] = 1.0
    want = torch.zeros(heads, n, rank, dtype=torch.float64)
    REF.latent_attention(q_lat, None, lat.double(), None, bt, cu, seq, req, None, want, scale, 3, n)
    for terms in (1, 2):
        got = torch.zeros(heads, n, rank, device="cuda", dtype=torch.bfloat16)
        K.latent_attention(q_lat.cuda(), None, lat.cuda(), None, bt.cuda(), cu.cuda(), seq.cuda(), req.cuda(), None, got, scale, 3, n,
                           max_q_len=n, max_seq_len=n, weight_terms=terms)
        bias[terms] = float((got.double().cpu()[:, 2:, 1:] / want[:, 2:, 1:] - 1.0).mean())
    assert -1.6e-3 < bias[1] < -0.7e-3 and abs(bias[2]) < 2e-4, bias


def test_queries_from_a_product_of_their_own_and_the_gate_per_head(K):
    g = gen(9)
    n, H, D, rot, dims, R, ps = 7, 3, 8, 6, 4, 16, 4
    for dtype in (torch.float32, torch.bfloat16):
        proj = torch.randn(n, R + rot + H, generator=g)
        q = torch.randn(n, H * (D + rot), generator=g)
        table = torch.randn(n, dims, generator=g)
        norm_w = (1 + 0.2 * torch.randn(R, generator=g)).to(dtype)
        slots = torch.randperm(3 * ps, generator=g)[:n].to(torch.int32)
        seg = n + 2

        def run(kern, dev, cd):
            qp = torch.zeros(H, seg, D, dtype=cd, device=dev)
            qr = torch.zeros(n, H, rot, dtype=torch.float64 if cd == torch.float64 else torch.float32, device=dev)
            lat = torch.zeros(3, 1, ps, R, dtype=cd, device=dev)
            rp = torch.zeros(3, 1, ps, rot, dtype=cd, device=dev)
            off = torch.zeros(H + 1, dtype=torch.int32, device=dev)
            kern.latent_prepare(proj.to(dev), H, D, rot, R, 0, norm_w.to(dev), 1e-5, table.to(dev), dims, qp, qr, lat, rp,
                                slots.to(dev), off, q=q.to(dev), interleaved=True)
            return qp, qr, lat, rp
        want = run(REF, "cpu", torch.float64)
        got = run(K, "cuda", dtype)
        tol = 2e-5 if dtype == torch.float32 else 0.05
        for a, b, what in zip(got, want, ("plain parts", "rotated parts", "latents", "rotated keys")):
            close(a[:, :n] if what == "plain parts" else a, b[:, :n] if what == "plain parts" else b, tol, what)
        # the rotation pairs neighbours: entry 0 of a rotated part mixes with entry 1, entry 5 (beyond dims) passes
        c, s = table[0, 0].double(), table[0, 1].double()
        a0, a1 = q[0, D].double(), q[0, D + 1].double()
        assert abs(float(want[1][0, 0, 0]) - float(a0 * c - a1 * s)) < 1e-9 and float(want[1][0, 0, 5]) == float(q[0, D + 5].double())
        y = torch.randn(H, seg, 10, generator=g)
        gate = proj[:, R + rot:]
        o_r, o_g = torch.zeros(n, H * 10, dtype=torch.float64), torch.zeros(n, H * 10, device="cuda", dtype=dtype)
        REF.gate_heads(y, gate, o_r, n, per_head=True)
        K.gate_heads(y.cuda(), proj.cuda()[:, R + rot:], o_g, n, per_head=True)
        close(o_g, o_r, tol, "heads times one gate each")


@pytest.mark.parametrize("E,top,extra", [(8, 1, 1), (5, 2, 0), (4, 4, 1), (64, 6, 0), (3, 3, 2)])
def test_sigmoid_router_and_experts_that_read_weighted_rows(K, E, top, extra):
    g = gen(E * 10 + top)
    n, width = 37, 24
    logits = torch.randn(n, E + extra, generator=g) * 3
    logits[3] = 0.25                                     # all equal: the lowest indices
    logits[5, : E // 2 + 1] = 2.0                        # ties at the top
    ids_r, gates_r = torch.zeros(n, top, dtype=torch.int32), torch.zeros(n, top, dtype=torch.float64)
    ids_g, gates_g = torch.zeros(n, top, dtype=torch.int32, device="cuda"), torch.zeros(n, top, device="cuda")
    REF.moe_route(logits, top, ids_r, gates_r, experts=E, scoring="sigmoid")
    K.moe_route(logits.cuda(), top, ids_g, gates_g, experts=E, scoring="sigmoid")
    assert torch.equal(ids_g.cpu(), ids_r)
    close(gates_g, gates_r, 1e-6, "weights")
    assert ids_r[3].tolist() == list(range(top)) and float(gates_r.max()) <= 1.0
    # the one-launch form of small steps
    offs, perm, pos = (torch.zeros(k, dtype=torch.int32, device="cuda") for k in (E + 1, n * top, n * top))
    ids2, gates2 = torch.zeros_like(ids_g), torch.zeros_like(gates_g)
    K.moe_route_plan(logits.cuda(), top, ids2, gates2, offs, perm, pos, experts=E, scoring="sigmoid")
    assert torch.equal(ids2, ids_g) and torch.equal(gates2, gates_g)
    offs_r, perm_r, pos_r = (torch.zeros(k, dtype=torch.int32) for k in (E + 1, n * top, n * top))
    REF.moe_plan(ids_r, E, offs_r, perm_r, pos_r)
    assert torch.equal(perm.cpu(), perm_r) and torch.equal(offs.cpu(), offs_r)
    for dtype in (torch.float32, torch.bfloat16):
        for w in (width, 33):
            x = torch.randn(n, w, generator=g).to(dtype)
            padded = torch.cat((perm_r, torch.full((3,), -1, dtype=torch.int32)))
            xs_r, xs_g = torch.zeros(n * top + 3, w, dtype=torch.float64), torch.full((n * top + 3, w), 7.0, device="cuda", dtype=dtype)
            REF.moe_gather_scaled(x, padded, top, gates_r, xs_r)
            K.moe_gather_scaled(x.cuda(), padded.cuda(), top, gates_g, xs_g)
            close(xs_g, xs_r, 1e-6 if dtype == torch.float32 else 0.03, "weighted rows")
    y = torch.randn(n * top, width, generator=g)
    shared, sl = torch.randn(n, width, generator=g), torch.randn(n, E + extra, generator=g)
    o_r, o_g = torch.zeros(n, width, dtype=torch.float64), torch.zeros(n, width, device="cuda")
    REF.moe_combine(y, pos_r, None, o_r, shared, sl[:, E - 1])
    K.moe_combine(y.cuda(), pos, None, o_g, shared.cuda(), sl.cuda()[:, E - 1])
    close(o_g, o_r, 2e-5, "the sum without weights")
    x = torch.randn(n, width, generator=g)
    d = torch.randn(n, width, generator=g)
    xg = x.cuda()
    copy = torch.zeros(n, width, device="cuda", dtype=torch.bfloat16)
    K.scaled_sum(xg, d.cuda(), 1.0, copy=copy)
    close(xg, x + d, 1e-6, "stream")
    assert torch.equal(copy, xg.to(torch.bfloat16))


# ------------------------------------------------------------------------------ the engine
LENS = [37, 100, 64, 19, 85, 50, 1, 2, 3, 160]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("golonex"))
    out = {}
    for name in ("G1", "G2", "G3"):
        d = TG.make_model_dir(name, root)
        cfg, w = TG.load_model_dir(d)
        reqs = {f"r{i}": tiny.random_tokens(cfg["vocab"], n, 100 + i) for i, n in enumerate(LENS)}
        out[name] = (d, cfg, w, reqs, {r: P.forward(cfg, w, t).float() for r, t in reqs.items()})
    return out


def _runner(model_dir, name, dtype, pool):
    from infurnace_b200.engine.loading import EngineOptions, build_runner
    ps = TG.TINY[name]["page_size"]
    return build_runner(model_dir, EngineOptions(dtype=dtype, device="cuda", page_size=ps, num_pages=pool // ps, max_num_seqs=4,
                                                 max_num_batched_tokens=pool, max_model_len=pool))[2]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "bulk_tail", "portions", "mixed"])
@pytest.mark.parametrize("name", ["G1", "G2", "G3"])
def test_cutting_modes(models, name, mode, dtype):
    d, cfg, w, reqs, ref = models[name]
    steps = {"whole": tiny.schedule_whole, "bulk_tail": lambda r: tiny.schedule_bulk_tail(r, tail=60),
             "portions": lambda r: tiny.schedule_portions(r, seed=1),
             "mixed": lambda r: tiny.schedule_mixed(r, max_live=4, max_tokens=640, seed=2)}[mode](reqs)
    runner = _runner(d, name, dtype, 640)
    out = tiny.collect(steps, tiny.run_inprocess(runner, steps), cfg["vocab"])
    assert runner.cache.num_free_slots == 4
    assert runner.cache.free_pages() == [g.pool.num_pages for g in runner.cache.kv_groups]
    runner.rt.kernels.check_device_errors()
    if dtype == "float32":
        worst = max(rows_match(out[rid], ref[rid], dtype, f"{name} {mode} {dtype} request {rid}") for rid in reqs)
    else:         # the share of positions is taken over all requests (three of them have one to three tokens)
        worst = rows_match(torch.cat([out[rid] for rid in reqs]), torch.cat([ref[rid] for rid in reqs]), dtype, f"{name} {mode} {dtype}")
    print(f"{name} {mode} {dtype}: worst {worst:.3g} (largest logit {max(float(r.abs().max()) for r in ref.values()):.3g})")


def test_the_fast_routes_ran(models):
    """The wider model's bfloat16 steps take the tensor-core attention kernels, the chunked recurrence and the grouped
    products; its layers would otherwise pass on the plain kernels alone."""
    d, cfg, w, reqs, ref = models["G3"]
    runner = _runner(d, "G3", "bfloat16", 640)
    k = runner.rt.kernels
    before = (k.latent_mma_calls, k.rglru_chunked_calls, k.moe_tcgen05_calls, k.stream_attention_calls)
    steps = tiny.schedule_whole({"a": reqs["r9"]})
    tiny.run_inprocess(runner, steps)
    assert k.latent_mma_calls > before[0] and k.rglru_chunked_calls > before[1] and k.moe_tcgen05_calls > before[2]
    assert k.stream_attention_calls == before[3]                   # keys and values of one width: the tensor-core attention


OTHER_SIZES = {
    # widths that are no multiple of 8 (the plain products), heads of 24 + 10, ranks of 40 and 9, one expert, seven taps
    "odd": TG._config(53, 100, 1e-5, [
        TG._lat(3, 24, 10, 20, 40, 9, 0.2, 33, 777.0, TG._moe(1, 1, 36)),
        TG._rec(75, 5, 7, TG._moe(5, 5, 20, shared=12)),
        TG._att(6, 2, 20, 0.25, 3, 40.0, 6, None, scaling=(3.0, 40, 6.0, 2.0))], cap=9.0, side=7),
    # sizes the tensor-core routes take throughout: heads of 128 and 16, ranks of 128 and 256, a window that is a page's
    # multiple, blocks of 64 channels
    "tc": TG._config(211, 128, 1e-6, [
        TG._att(8, 1, 128, 0.09, 64, 5000.0, 64, TG._moe(16, 4, 64, shared=64), scaling=(2.0, 128, 32.0, 1.0)),
        TG._lat(16, 32, 16, 32, 128, 64, 0.15, 64, 5000.0, TG._moe(8, 2, 32)),
        TG._rec(256, 4, 4, None),
        TG._lat(4, 64, 64, 64, 256, 128, 0.1, 17, 20.0, None),
        TG._att(16, 16, 16, 0.25, 100, 20.0, 16, TG._moe(4, 1, 128, shared=128))], side=8),
    # a single recurrent layer, and a single attention layer with one head
    "one": TG._config(40, 32, 1e-5, [TG._rec(48, 2, 2, TG._moe(4, 2, 16))], cap=4.0),
    "head": TG._config(40, 32, 1e-5, [TG._att(1, 1, 32, 0.2, 10, 100.0, 32, None)], side=1),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(OTHER_SIZES))
def test_other_sizes_and_orders(tmp_path, name, dtype):
    """Models of other sizes, head counts and orders of layers, in a mixed schedule over a small pool."""
    from infurnace_b200.engine.loading import EngineOptions, build_runner
    conf = OTHER_SIZES[name]
    d = TG.make_model_dir("_" + name, str(tmp_path), config=conf, seed=31, store="bfloat16", sharpen=2.0)
    cfg, w = TG.load_model_dir(d)
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
    """Every token alone from the first on, 300 of them: windows of 33, 50 and 120 pass over decoded tokens, pages of the
    windowed layers go back and come again, the recurrence runs 300 steps from its slot."""
    d, cfg, w, _, _ = models["G3"]
    toks = tiny.random_tokens(cfg["vocab"], 300, 77)
    want = P.forward(cfg, w, toks).float()
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
    out = tiny.collect(steps, tiny.run_inprocess(_runner(d, "G3", dtype, 384), steps), cfg["vocab"])["x"]
    rows_match(out, want, dtype, "token by token")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_in_portions_then_decoding(models, dtype):
    """900 tokens: portions of 500, 133, 2 and 200, then 65 tokens one by one, beside a second request that comes and goes."""
    d, cfg, w, _, _ = models["G3"]
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
    out = tiny.collect(steps, tiny.run_inprocess(_runner(d, "G3", dtype, 1088), steps), cfg["vocab"])
    rows_match(out["x"], want, dtype, "the long request")
    rows_match(out["y"], want_other, dtype, "the request beside it")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(models, tmp_path, dtype):
    d, cfg, w, reqs, ref = models["G2"]
    steps = tiny.schedule_mixed(reqs, max_live=4, max_tokens=640, seed=5)
    outputs = tiny.run_trace_run(d, dtype, steps, str(tmp_path / "out"), 640, TG.TINY["G2"]["page_size"])
    out = tiny.collect(steps, outputs, cfg["vocab"])
    rows_match(torch.cat([out[rid] for rid in reqs]), torch.cat([ref[rid] for rid in reqs]), dtype, "all requests")


def test_greedy_generation_through_the_engine_and_its_graphs(models):
    """The engine's own entry point: scheduler, portions beside decoded tokens, six requests over four slots, decode
    steps replayed from CUDA graphs.  In float32 the tokens are the plain implementation's."""
    from infurnace_b200.engine import Engine, EngineOptions, SamplingParams
    d, cfg, w, _, _ = models["G1"]
    ps = TG.TINY["G1"]["page_size"]
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
    d, cfg, w, _, _ = models["G1"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bin", "infurnace-b200"), "--model", d, "--prompt-ids", "5,6,7,8",
                          "--max-tokens", "6", "--json", "--dtype", "float32", "--page-size", "16", "--max-context", "64"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    report = json.loads(out.stdout)
    assert report["generated_token_ids"] == P.greedy(cfg, w, [5, 6, 7, 8], 6) and report["model"]["architecture"] == "Golonex"
