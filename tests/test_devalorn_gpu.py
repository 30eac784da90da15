"""Devalorn in the engine against the plain implementation (``plain_devalorn``): every mechanism
alone at the kernels' interface, then whole models of several shapes under every way of
cutting and batching the work, in 32-bit and in bfloat16, and greedy generation through the
package's entry point."""
import math
import random

import pytest
import torch

import plain_devalorn as P
from helpers import Replayer, random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------ mechanisms, one by one
def test_softmax_router_kernel():
    """Shares of the softmax over ALL experts for one, some and all chosen experts, times a
    constant, renormalised or not; expert counts that are no powers of two."""
    from pretrained_rstr_b200.csrc import ops
    g = torch.Generator().manual_seed(3)
    for t, n_e in ((9, 6), (4, 1), (33, 17)):
        logits = torch.randn(t, n_e + 5, generator=g) * 2
        z = logits[:, 3:3 + n_e]
        s = torch.softmax(z.double(), dim=-1)
        for top in sorted({1, min(2, n_e), n_e}):
            weights = torch.empty(t, n_e, device=DEV)
            chosen = torch.empty(t, top, dtype=torch.int32, device=DEV)
            chosen_w = torch.empty(t, top, device=DEV)
            val, idx = torch.topk(s, top, dim=-1)
            for factor, renorm in ((1.0, False), (2.5, False), (0.5, True)):
                ops.route_scores(weights, chosen, chosen_w, logits.to(DEV)[:, 3:3 + n_e], None, top,
                                 score="softmax", renormalize=renorm, factor=factor)
                want = (val / val.sum(-1, keepdim=True) if renorm else val) * factor
                assert torch.equal(chosen.cpu().long(), idx)
                assert torch.allclose(chosen_w.cpu().double(), want, atol=1e-6)
                assert torch.allclose(weights.cpu().double(),
                                      torch.zeros(t, n_e, dtype=torch.float64).scatter(1, idx, want), atol=1e-6)
    # large logits: the softmax stays finite and the order of the logits decides
    big = torch.tensor([[400.0, 450.0, 300.0, -3.0, 449.0, 200.0]], device=DEV)
    w1, c1, cw1 = torch.empty(1, 6, device=DEV), torch.empty(1, 2, dtype=torch.int32, device=DEV), torch.empty(1, 2, device=DEV)
    ops.route_scores(w1, c1, cw1, big, None, 2, score="softmax")
    assert c1.cpu().tolist() == [[1, 4]]
    assert torch.allclose(cw1.cpu(), torch.tensor([[1 / (1 + math.exp(-1)), 1 / (1 + math.exp(1))]]), atol=1e-6)


class TimeMixCase:
    """Hand-made r, k, v, gate and decay inputs behind a stand-in for the projections' buffer."""

    def __init__(self, heads, dim, vdim, rank, seed=0, width=24):
        self.heads, self.dim, self.vdim, self.rank, self.width = heads, dim, vdim, rank, width
        self.g = torch.Generator().manual_seed(seed)
        rn = lambda *s: torch.randn(*s, generator=self.g)
        self.w2 = rn(heads * dim, rank) * 0.7
        self.w0 = rn(heads * dim) - 1.0
        self.u = rn(heads, dim) * 0.5
        self.norm_w = 1.0 + 0.1 * rn(heads * vdim)
        self.state = torch.full((3, heads, vdim, dim), 9.0, device=DEV)     # what earlier users left
        self.prev = torch.full((3, width), 5.0, device=DEV)

    def rows(self, n):
        r = lambda w: torch.randn(n, self.heads, w, generator=self.g)
        return (r(self.dim), r(self.dim), r(self.vdim), r(self.vdim),
                torch.randn(n, self.rank, generator=self.g), torch.randn(n, self.width, generator=self.g))

    def plain(self, r, k, v, gate, lr, eps, scale=1.0):
        n = r.shape[0]
        z = torch.tanh(lr.double()) @ self.w2.double().T + self.w0.double()
        w = torch.exp(-torch.exp(z)).reshape(n, self.heads, self.dim)
        o, _ = P.decayed_outer_states(r.double(), k.double(), v.double(), w, self.u.double())
        gd = gate.double()
        return P.unit_rms(o, eps) * self.norm_w.double().reshape(self.heads, self.vdim) * gd * torch.sigmoid(gd) * scale

    def run(self, parts, eps, scale=1.0, out_dtype=torch.float32, mode="scan"):
        """parts: (slot, first position, r, k, v, gate, lr, h) per request of one step.  ``mode``:
        "scan" (a CTA per (head, request, columns) and the finish after it), "step" (the finish
        inside the scan) or "segments" (portions cut into segments that run side by side)."""
        from pretrained_rstr_b200.csrc import ops
        hd, d, vd, rk = self.heads, self.dim, self.vdim, self.rank
        proj, pos, seq, qs, slots, hs = [], [], [], [0], [], []
        for b, (slot, p0, r, k, v, gate, lr, h) in enumerate(parts):
            n = r.shape[0]
            pad = torch.zeros(n, 4)
            proj.append(torch.cat([pad, r.reshape(n, -1), k.reshape(n, -1), pad, v.reshape(n, -1),
                                   gate.reshape(n, -1), pad, lr], dim=1))
            hs.append(h)
            pos += list(range(p0, p0 + n))
            seq += [b] * n
            qs.append(qs[-1] + n)
            slots.append(slot)
        proj = torch.cat(proj).to(DEV).contiguous()
        h_all = torch.cat(hs).to(DEV).contiguous()
        t = proj.shape[0]
        r_col, k_col = 4, 4 + hd * d
        v_col = 8 + 2 * hd * d
        g_col = v_col + hd * vd
        lr_col = g_col + hd * vd + 4
        raw = torch.empty(t, hd * vd, device=DEV)
        status = torch.zeros(4, dtype=torch.int32, device=DEV)
        out = torch.zeros(t, hd * vd + 8, dtype=out_dtype, device=DEV)
        if out_dtype != torch.float32:
            h_all, self.prev = h_all.to(out_dtype), self.prev.to(out_dtype)
        extra = {}
        if mode == "segments":
            n = ops.tmix_max_segments(t, len(parts) + 1) + 2
            extra = {"segments": (torch.full((n, hd, vd, d), 3.0, device=DEV),
                                  torch.full((n, hd, vd, d), 3.0, device=DEV),
                                  torch.full((n, hd, d), 3.0, device=DEV)),
                     "decays": torch.full((t + 2, hd * d + 8), 77.0, device=DEV)[:t]}
        elif mode == "step":
            extra = {"finish": (out, g_col, self.norm_w.to(DEV), eps, scale)}
        ops.tmix_scan(raw, proj, r_col, k_col, v_col, lr_col, self.w2.to(DEV), self.w0.to(DEV),
                      self.u.to(DEV).contiguous(), self.state, h_all, self.prev, _i32(qs + [qs[-1]]),
                      _i32(slots + [0]), _i32(pos), len(parts) + 1, hd, d, vd, status, **extra)
        assert int(status[0]) == 0, status.tolist()
        if mode != "step":
            ops.tmix_finish(out, raw, proj, g_col, self.norm_w.to(DEV), _i32(seq), hd, vd, eps, scale)
        self.prev = self.prev.float()
        for (slot, *_rest, h), end in zip(parts, qs[1:]):
            assert torch.equal(self.prev[slot].cpu(), h[-1].to(out_dtype).float())   # the row the next shift reads
        return out.cpu().double()[:, :hd * vd].reshape(t, hd, vd)


@pytest.mark.parametrize("mode", ["scan", "step", "segments"])
@pytest.mark.parametrize("heads,dim,vdim,rank", [(3, 16, 16, 5), (2, 80, 80, 16), (1, 8, 136, 3),
                                                 (2, 64, 64, 32), (1, 160, 16, 8), (4, 40, 24, 1),
                                                 (1, 264, 40, 2), (2, 3, 5, 4)])
def test_time_mix_kernels(heads, dim, vdim, rank, mode):
    """A whole sequence at once, in portions down to one token and longer than a segment, beside
    another request; a slot's earlier state is not read at position 0 and is carried from then
    on.  Each way the scan runs: a CTA per request's portion with the finish after it or inside,
    and in segments side by side."""
    from pretrained_rstr_b200.csrc import ops
    if mode == "step" and not ops.tmix_step_supports(dim, vdim):
        pytest.skip("a head's columns do not fit one CTA")
    case = TimeMixCase(heads, dim, vdim, rank, seed=heads + dim)
    run = lambda parts, *a, **kw: TimeMixCase.run(case, parts, *a, mode=mode, **kw)
    case.run = run
    n = 290
    a = case.rows(n)
    b = case.rows(37)
    want, want2 = case.plain(*a[:5], 1e-5, 0.9), case.plain(*b[:5], 1e-5, 0.9)
    got = case.run([(1, 0, *a)], 1e-5, 0.9)
    assert torch.allclose(got, want, atol=3e-5, rtol=3e-5)
    at, outs = 0, []
    cut = lambda rows, lo, hi: tuple(x[lo:hi] for x in rows)
    for size in (1, 2, 17, 1, 33, 16, 20, 64, 71, 65):
        part = (1, at, *cut(a, at, at + size))
        m = 1 + at % 7
        other = (2, 0, *cut(b, 0, m))
        parts = [other, part] if at % 2 else [part, other]
        got = case.run(parts, 1e-5, 0.9)
        r0 = m if at % 2 else 0
        outs.append(got[r0:r0 + size])
        other_rows = got[:m] if at % 2 else got[size:]
        assert torch.allclose(other_rows, want2[:m], atol=3e-5, rtol=3e-5)
        at += size
    assert at == n
    assert torch.allclose(torch.cat(outs), want, atol=3e-5, rtol=3e-5)
    out16 = case.run([(0, 0, *b)], 1e-5, 0.9, out_dtype=torch.bfloat16)
    assert torch.allclose(out16, want2, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("mode", ["scan", "step", "segments"])
def test_time_mix_far_token_stands_out(mode):
    """One key far back, made large, among hundreds: where the decay is slow it still carries
    the result, through a portion's start and through single tokens, and where it is fast it is
    gone; a lost state, a decay applied before the read, or a bonus that outlives its token
    would show."""
    case = TimeMixCase(2, 16, 16, 4, seed=9)
    run = lambda parts, *a, **kw: TimeMixCase.run(case, parts, *a, mode=mode, **kw)
    case.run = run
    case.w2.zero_()
    case.w0[:16] = -7.0                  # head 0: w = exp(-exp(-7)) ~ 0.9991
    case.w0[16:] = 0.0                   # head 1: w = exp(-1) ~ 0.37
    n, far = 400, 3
    rows = case.rows(n)
    r, k, v = rows[0], rows[1], rows[2]
    r[-1] = k[far]                       # the last token asks for the far one
    k[far] *= 30.0
    v[far] *= 5.0
    want = case.plain(*rows[:5], 1e-6)
    outs, at = [], 0
    for size in [130, 64, 2, 190] + [1] * 14:
        outs.append(case.run([(0, at, *(x[at:at + size] for x in rows))], 1e-6))
        at += size
    got = torch.cat(outs)
    assert at == n and torch.allclose(got, want, atol=1e-4, rtol=1e-4)
    k[far] /= 30.0
    v[far] /= 5.0
    plain_far = case.plain(*rows[:5], 1e-6)
    assert float((want[-1, 0] - plain_far[-1, 0]).abs().max()) > 0.1      # slow decay: it counts
    assert float((want[-1, 1] - plain_far[-1, 1]).abs().max()) < 1e-6     # fast decay: long gone
    # the bonus acts on the current token only: with u large, token t's own key dominates o_t
    # and is back to its plain weight in o_(t+1)
    case.u[:] = 50.0
    big = case.plain(*rows[:5], 1e-6)
    got = case.run([(1, 0, *rows)], 1e-6)
    assert torch.allclose(got, big, atol=1e-4, rtol=1e-4)


def test_time_mix_shift_kernel():
    """Blends with the previous token's row: zeros at position 0, the slot's saved row at a
    portion's start, the row before inside a portion; several requests in a step."""
    from pretrained_rstr_b200.csrc import ops
    g = torch.Generator().manual_seed(2)
    width, n_mix = 40, 5
    mu = torch.rand(n_mix, width, generator=g)
    h = torch.randn(12, width, generator=g)
    prev = torch.randn(4, width, generator=g)
    # request 0: positions 0..4 in slot 2; request 1: positions 7..9 in slot 0; request 2: one
    # token at position 3 in slot 3; request 3's first two tokens in slot 1; a padding row
    seq = [0] * 5 + [1] * 3 + [2] + [3] * 2 + [-1]
    pos = [0, 1, 2, 3, 4, 7, 8, 9, 3, 0, 1, 0]
    slots = [2, 0, 3, 1]
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 2e-2)):
        out = torch.full((12, n_mix * width + 8), 7.0, dtype=dtype, device=DEV)
        status = torch.zeros(4, dtype=torch.int32, device=DEV)
        ops.tmix_shift(out, h.to(dtype).to(DEV), prev.to(dtype).to(DEV), mu.to(DEV), _i32(seq), _i32(pos),
                       _i32([0, 5, 8, 9, 11]), _i32(slots), status)
        assert int(status[0]) == 0
        hh, pp = h.to(dtype).double(), prev.to(dtype).double()
        for s in range(n_mix):
            for (lo, hi), first in (((0, 5), None), ((5, 8), pp[0]), ((8, 9), pp[3]), ((9, 11), None)):
                want = P.shifted_blend(hh[lo:hi], mu[s].double(), first)
                assert torch.allclose(out[lo:hi, s * width:(s + 1) * width].cpu().double(), want, atol=tol, rtol=tol)
        assert float(out[11, :n_mix * width].float().abs().max()) == 0.0
        assert float((out[:, n_mix * width:].float() - 7.0).abs().max()) == 0.0
        # without blend weights: the row beside its difference from the row before; a blend's
        # projection is that pair's, M b_s = [M | M diag(mu_s)] [h | h' - h]
        pair = torch.full((12, 2 * width + 8), 7.0, dtype=dtype, device=DEV)
        ops.tmix_shift(pair, h.to(dtype).to(DEV), prev.to(dtype).to(DEV), None, _i32(seq), _i32(pos),
                       _i32([0, 5, 8, 9, 11]), _i32(slots), status)
        assert int(status[0]) == 0
        got = pair.cpu().double()
        M = torch.randn(6, width, generator=g).double()
        for (lo, hi), first in (((0, 5), None), ((5, 8), pp[0]), ((8, 9), pp[3]), ((9, 11), None)):
            before = torch.cat([(torch.zeros(width).double() if first is None else first)[None], hh[lo:hi - 1]])
            assert torch.equal(got[lo:hi, :width], hh[lo:hi])
            assert torch.allclose(got[lo:hi, width:2 * width], before - hh[lo:hi], atol=tol, rtol=tol)
            for s in range(n_mix):
                folded = torch.cat([M, M * mu[s].double()[None]], dim=1)
                want = P.shifted_blend(hh[lo:hi], mu[s].double(), first) @ M.T
                assert torch.allclose(got[lo:hi, :2 * width] @ folded.T, want, atol=20 * tol, rtol=20 * tol)
        assert float(got[11, :2 * width].abs().max()) == 0.0
        assert float((got[:, 2 * width:] - 7.0).abs().max()) == 0.0


class WindowCase:
    """A paged cache of rows [k | v] filled by hand: requests' rows lie in pages taken in a
    shuffled order from a pool whose other pages hold large numbers."""

    def __init__(self, lengths, kv_heads, dim, vdim, dtype, page=64, seed=0, fill=40.0):
        g = torch.Generator().manual_seed(seed)
        self.kv_heads, self.dim, self.vdim, self.page, self.dtype = kv_heads, dim, vdim, page, dtype
        need = sum(-(-n // page) for n in lengths)
        pages = list(range(need + 3))
        random.Random(seed).shuffle(pages)
        self.rows = [(torch.randn(n, kv_heads, dim + vdim, generator=g) * 0.5).to(dtype).float()
                     for n in lengths]
        self.max_pages = max(-(-n // page) for n in lengths) + 1
        cache = torch.full((need + 3, kv_heads, page, dim + vdim), fill)
        table = torch.full((len(lengths), self.max_pages), -1, dtype=torch.int32)
        for b, n in enumerate(lengths):
            for li in range(-(-n // page)):
                pg = pages.pop()
                table[b, li] = pg
                m = min(page, n - li * page)
                cache[pg, :, :m] = self.rows[b][li * page:li * page + m].transpose(0, 1)
        self.cache, self.table = cache.to(dtype).to(DEV), table.to(DEV)

    def put(self, b, p, row):
        """Replaces request b's row at position p (all key/value heads) after the fact."""
        self.rows[b][p] = row.to(self.dtype).float()
        pg = int(self.table[b, p // self.page])
        self.cache[pg, :, p % self.page] = row.to(self.dtype).to(DEV)

    def run(self, queries, heads, window, keep_first, scale, gate=None, slopes=None, out_scale=1.0,
            tile_rows=0):
        """queries: (request, position, q [heads, dim]); returns kernel and plain results
        [n, heads, vdim].  ``tile_rows`` 0: a CTA per (token, head); -1: the single-token
        kernel; else the tiled kernel."""
        from pretrained_rstr_b200.csrc import ops
        n = len(queries)
        q = torch.stack([x for _, _, x in queries]).reshape(n, -1).to(DEV).contiguous()
        out = torch.full((n, heads * self.vdim + 8), float("nan"), dtype=self.dtype, device=DEV)
        status = torch.zeros(4, dtype=torch.int32, device=DEV)
        gate_dev = None
        if gate is not None:                         # a column slice of a wider buffer
            wide = torch.full((n, heads + 3), 50.0)
            wide[:, 3:] = gate
            gate_dev = wide.to(DEV)[:, 3:]
        ops.wattn(out, q, self.cache, self.table, _i32([b for b, _, _ in queries]),
                  _i32([p for _, p, _ in queries]), heads, self.dim, self.vdim, window, keep_first,
                  scale, gate=gate_dev, slopes=None if slopes is None else slopes.float().to(DEV),
                  out_scale=out_scale, status=status, tile_rows=max(tile_rows, 0),
                  single=tile_rows < 0)
        assert int(status[0]) == 0, status.tolist()
        want = []
        for i, (b, p, x) in enumerate(queries):
            rows = self.rows[b][:p + 1].double()
            mask = P.window_mask(torch.tensor([p]), p + 1, window or None, keep_first)
            o = P.masked_softmax_attention(x.double()[None], rows[:, :, :self.dim], rows[:, :, self.dim:],
                                           mask, scale, positions=torch.tensor([p]),
                                           slopes=None if slopes is None else slopes.double())[0]
            if gate is not None:
                o = o * torch.sigmoid(gate[i].double())[:, None]
            want.append(o * out_scale)
        got = out.cpu().double()[:, :heads * self.vdim].reshape(n, heads, self.vdim)
        return got, torch.stack(want)


def _tile_choices(heads, kv_heads, dim, vdim):
    from pretrained_rstr_b200.csrc import ops
    most = ops.wattn_tile_rows(heads, kv_heads, dim, vdim)      # 0: the tiled kernel does not take them
    single = [-1] if ops.wattn_single_supports(heads, kv_heads, dim, vdim) else []
    return [0] + single + (sorted({1, min(5, most), most}) if most else [])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,keep_first", [(0, 0), (20, 0), (20, 7), (64, 64), (96, 3), (300, 70),
                                               (1, 0), (1, 2), (33, 100)])
def test_window_attention_kernels(dtype, window, keep_first):
    """Random rows; queries at the first tokens, at page borders, at the window's first full
    position and around the end of the kept tokens; windows shorter and longer than a page and
    than the kernels' key blocks, kept tokens beyond the window's length; with and without the
    bias and the gate; a CTA per (token, head) and tiles of rows that hold runs of consecutive
    positions, single tokens and several requests."""
    heads, kv_heads, dim, vdim = 6, 2, 24, 40
    lengths = [1, 65, 200, 700]
    case = WindowCase(lengths, kv_heads, dim, vdim, dtype, seed=4)
    g = torch.Generator().manual_seed(8)
    places = {0, 1, 2, 31, 32, 63, 64, 65, 127, 128, 199, 255, 256, 257, 511, 512, 513, 699}
    for edge in (window, keep_first, window + keep_first):
        places |= {edge + o for o in (-2, -1, 0, 1) if edge + o >= 0}
    places |= set(range(300, 312))                              # a run of consecutive rows
    queries = [(b, p, torch.randn(heads, dim, generator=g))
               for b, n in enumerate(lengths) for p in sorted(places) if p < n]
    slopes = P.distance_slopes(heads, torch.float64)
    gate = torch.randn(len(queries), heads, generator=g) * 2
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for tile_rows in _tile_choices(heads, kv_heads, dim, vdim):
        for opts in ({}, {"slopes": slopes}, {"gate": gate, "out_scale": 0.7},
                     {"slopes": slopes * 40, "gate": gate}):
            got, want = case.run(queries, heads, window, keep_first, 0.3, tile_rows=tile_rows, **opts)
            assert torch.allclose(got, want, atol=tol, rtol=tol), (tile_rows, sorted(opts))


@pytest.mark.parametrize("window,keep_first", [(0, 0), (600, 40), (100, 300)])
@pytest.mark.parametrize("n_queries", [1, 3, 9, 30])
def test_window_attention_few_single_tokens(window, keep_first, n_queries):
    """Steps of so few single tokens that the single-token kernel splits a token's keys over
    several CTAs: every number of CTAs a token, some of them without a key block of their own."""
    heads, kv_heads, dim, vdim = 6, 2, 32, 64
    lengths = [900, 40, 300]
    case = WindowCase(lengths, kv_heads, dim, vdim, torch.bfloat16, seed=11)
    g = torch.Generator().manual_seed(3)
    places = [(0, 899), (1, 39), (2, 299), (0, 0), (0, 31), (0, 32), (0, 255), (0, 256), (0, 600)]
    places = (places * 4)[:n_queries]
    queries = [(b, p, torch.randn(heads, dim, generator=g)) for b, p in places]
    slopes = P.distance_slopes(heads, torch.float64)
    gate = torch.randn(len(queries), heads, generator=g)
    got, want = case.run(queries, heads, window, keep_first, 0.2, slopes=slopes, gate=gate, tile_rows=-1)
    assert torch.allclose(got, want, atol=2e-2, rtol=2e-2)
    case32 = WindowCase(lengths, kv_heads, dim, vdim, torch.float32, seed=11)
    got, want = case32.run(queries, heads, window, keep_first, 0.2, slopes=slopes, gate=gate, tile_rows=-1)
    assert torch.allclose(got, want, atol=2e-5, rtol=2e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(1, 1, 8, 136), (8, 1, 16, 8), (3, 3, 80, 24),
                                                     (4, 2, 64, 64), (5, 5, 128, 128), (2, 1, 40, 320),
                                                     (4, 2, 6, 10), (2, 1, 5, 7), (3, 1, 12, 33)])
def test_window_attention_head_sizes(heads, kv_heads, dim, vdim, dtype):
    """One to eight query heads a key/value head; key and value sizes that differ, that are no
    multiples of 32, of 8, of 4 or of 2 (rows the kernels cannot fetch in 16-byte pieces), and
    that only the kernel of a CTA per (token, head) takes."""
    case = WindowCase([150, 70], kv_heads, dim, vdim, dtype, seed=heads + dim)
    g = torch.Generator().manual_seed(1)
    queries = [(b, p, torch.randn(heads, dim, generator=g))
               for b, n in ((0, 150), (1, 70)) for p in (0, 1, 40, 41, 63, 64, 69, 100, 149) if p < n]
    slopes = P.distance_slopes(heads, torch.float64)
    for tile_rows in _tile_choices(heads, kv_heads, dim, vdim):
        got, want = case.run(queries, heads, 41, 3, 0.2, slopes=slopes, tile_rows=tile_rows)
        tol = 3e-5 if dtype == torch.float32 else 2e-2
        assert torch.allclose(got, want, atol=tol, rtol=tol), tile_rows


@pytest.mark.parametrize("window,keep_first", [(50, 0), (50, 4), (300, 0), (64, 9), (0, 0)])
def test_window_attention_edges_stand_out(window, keep_first):
    """Keys made to dominate: the oldest key inside the window, the newest one outside, the last
    kept first token and the first one that is not kept.  A query sees exactly the marked keys
    its mask allows, in prompts' runs and alone, and far keys among hundreds count when no
    window hides them."""
    heads, kv_heads, dim, vdim = 2, 1, 16, 8
    n = 650
    case = WindowCase([n], kv_heads, dim, vdim, torch.float32, seed=6)
    g = torch.Generator().manual_seed(2)
    direction = torch.randn(dim, generator=g)
    direction /= direction.norm()
    at = 600                                                   # the query whose edges are marked
    marks = {}                                                 # position -> value it carries
    if window:
        marks[at - window + 1] = 3.0                           # just inside
        marks[at - window] = -5.0                              # just outside
    else:
        marks[3] = 3.0                                         # far back, nothing hides it
    if keep_first:
        marks[keep_first - 1] = 7.0                            # the last kept token
        marks[keep_first] = -11.0                              # the first that is not
    for p, mark in marks.items():
        row = torch.randn(kv_heads, dim + vdim, generator=g) * 0.1
        row[:, :dim] = direction * 6.0
        row[:, dim:] = mark
        case.put(0, p, row)
    queries = []
    for p in sorted({at - 1, at, at + 1, n - 1} | {keep_first + 1, 30}):
        x = torch.randn(heads, dim, generator=g) * 0.1
        x += direction * 6.0
        queries.append((0, p, x))
    for tile_rows in _tile_choices(heads, kv_heads, dim, vdim):
        got, want = case.run(queries, heads, window, keep_first, 1.0, tile_rows=tile_rows)
        assert torch.allclose(got, want, atol=2e-5, rtol=2e-5), tile_rows
    i = [p for _, p, _ in queries].index(at)
    seen = [3.0] + ([7.0] if keep_first else [])
    mean = float(want[i].mean())
    assert abs(mean - sum(seen) / len(seen)) < 0.2, mean       # the marked, visible keys carry it
    after = float(want[i + 1].mean())                          # one later: the inside key has left
    assert (abs(after - (7.0 if keep_first else 0.0)) < 0.6) if window else abs(after - 3.0) < 0.2


def test_window_attention_distance_bias_is_relative():
    """The bias is slope * (i - j): with a large slope a query all but sees itself only, at
    whichever position it stands (a bias that grew with the key's position alone would differ
    once the window moves)."""
    heads, kv_heads, dim, vdim = 2, 1, 16, 8
    case = WindowCase([400], kv_heads, dim, vdim, torch.float32, seed=3)
    g = torch.Generator().manual_seed(4)
    queries = [(0, p, torch.randn(heads, dim, generator=g) * 0.05) for p in (5, 64, 250, 399)]
    slopes = torch.tensor([30.0, 0.001], dtype=torch.float64)
    for tile_rows in _tile_choices(heads, kv_heads, dim, vdim):
        got, want = case.run(queries, heads, 100, 0, 1.0, slopes=slopes, tile_rows=tile_rows)
        assert torch.allclose(got, want, atol=2e-5, rtol=2e-5)
        for i, (_, p, _) in enumerate(queries):
            own = case.rows[0][p, 0, dim:].double()
            assert torch.allclose(got[i, 0], own, atol=1e-4)           # the steep head: itself
            assert float((got[i, 1] - own).abs().max()) > 0.05         # the flat head: an average


def test_prepare_norms_scales_rotates_and_caches():
    """The norm over the whole projection, the query's temperature by position, the rotation of
    a head's first coordinates, the cache row's layout; rows of other tokens untouched, nothing
    written for a slot of -1 or for a layer that reads another layer's cache."""
    from pretrained_rstr_b200.csrc import ops
    from pretrained_rstr_b200.parts.positions_rotary import rotary_frequencies
    heads, kv_heads, dim, vdim, page = 3, 1, 16, 24, 8
    g = torch.Generator().manual_seed(5)
    t = 6
    proj = torch.randn(t, 8 + heads * dim + kv_heads * dim + kv_heads * vdim, generator=g)
    qc, kc = 8, 8 + heads * dim
    vc = kc + kv_heads * dim
    pos = [0, 7, 8, 100, 3, 14]
    slots = [3, 2 * page + 1, -1, page, 0, 5]
    p = torch.tensor(pos)
    qw, kw = torch.rand(heads * dim, generator=g) + 0.5, torch.rand(kv_heads * dim, generator=g) + 0.5
    eps = 1e-3
    for rot, normed, coef, every in ((12, False, 0.0, 0), (0, True, 0.6, 5), (16, True, 0.25, 1)):
        cache = torch.full((3, kv_heads, page, dim + vdim), 5.0, device=DEV)
        q_out = torch.empty(t, heads * dim, device=DEV)
        ops.wattn_prepare(q_out, cache, proj.to(DEV), qc, kc, vc, qw.to(DEV) if normed else None,
                          kw.to(DEV) if normed else None, _i32(slots), _i32(pos),
                          rotary_frequencies(900.0, rot, DEV), heads, kv_heads, dim, vdim, rot, eps,
                          coef, every)
        q, k = proj[:, qc:kc].double(), proj[:, kc:vc].double()
        if normed:
            q, k = P.weighted_norm(q, qw.double(), eps), P.weighted_norm(k, kw.double(), eps)
        if every:
            q = q * P.query_temperature(p, coef, every, torch.float64)[:, None]
        want_q = P.rotate_half(q.reshape(t, heads, dim), p, 900.0, rot)
        want_k = P.rotate_half(k.reshape(t, kv_heads, dim), p, 900.0, rot)
        assert torch.allclose(q_out.cpu().double().reshape(t, heads, dim), want_q, atol=1e-5)
        flat = cache.cpu().double()
        touched = set()
        for i, s in enumerate(slots):
            if s < 0:
                continue
            row = flat[s // page, 0, s % page]
            touched.add((s // page, s % page))
            assert torch.allclose(row[:dim], want_k[i, 0], atol=1e-5)
            assert torch.allclose(row[dim:], proj[i, vc:].double(), atol=1e-6)
        for pg in range(3):
            for off in range(page):
                if (pg, off) not in touched:
                    assert float((flat[pg, 0, off] - 5.0).abs().max()) == 0.0
        # a layer that reads another layer's cache: queries only
        cache2 = torch.full_like(cache, 5.0)
        q2 = torch.empty_like(q_out)
        ops.wattn_prepare(q2, cache2, proj.to(DEV), qc, 0, 0, qw.to(DEV) if normed else None, None,
                          None, _i32(pos), rotary_frequencies(900.0, rot, DEV), heads, kv_heads, dim,
                          vdim, rot, eps, coef, every)
        assert torch.equal(q2, q_out) and float((cache2 - 5.0).abs().max()) == 0.0


# --------------------------------------------------------------------------- configurations
def _left(heads, kv_heads, dim, vdim, window, keep_first, rot_dims=None, base=10000.0, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "scale": scale if scale is not None else 1.0 / math.sqrt(dim),
            "mask": {"size": window, "keep_first": keep_first},
            "rot": {"base": base, "dims": dim if rot_dims is None else rot_dims}}


def _par(left, right_heads, right_dim, mlp, left_scale=0.7, right_scale=1.1):
    return {"type": "parallel",
            "mixer": {"left": left, "right": {"heads": right_heads, "dim": right_dim},
                      "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def _att(heads, kv_heads, dim, vdim, window, mlp, coef=0.4, every=32, kv_from=None, scale=None):
    mx = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
          "scale": scale if scale is not None else 1.0 / math.sqrt(dim), "mask": {"size": window},
          "q_temp": {"coef": coef, "every": every}}
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "attention", "mixer": mx, "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, scale=1.5):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale},
            "expert": {"ff": ff}}


def _model(vocab, width, layers, eps=1e-6):
    return {"architecture": "Devalorn", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": layers}


# Every size differs from every other one.  A: the two kinds of layer alternate, a layer that
# reads another's cache comes last and has no feed-forward, rotations that cover a part and all
# of a head, a parallel layer with routed experts, windows shorter than a page, one window with
# no kept tokens.  B: an attention layer first, windows longer than a page and than the
# kernels' key blocks, more kept tokens than a page holds, kept tokens beyond the window's
# length, as many key/value heads as heads, all experts chosen, no rotation at all, a layer
# that shares a cache two layers back with another window and other heads' slopes, a
# temperature that steps at every token.  C: parallel layers only (the time mixing's state and
# one attention cache a layer), a single head, a window of one token that sees itself and the
# kept ones, a window no prompt of the tests fills.
SHAPE_A = _model(310, 64, [
    _par(_left(4, 2, 16, 24, 24, 5, rot_dims=8), 2, 16, _dense(96)),
    _att(2, 1, 24, 16, 40, _moe(5, 2, 24), coef=0.3, every=8),
    _par(_left(2, 2, 24, 8, 12, 0, base=300.0, scale=0.3), 4, 8, _moe(3, 1, 40, scale=0.8),
         left_scale=1.2, right_scale=0.6),
    _att(2, 1, 24, 16, 18, None, coef=0.6, every=5, kv_from=1)])
SHAPE_B = _model(515, 128, [
    _att(3, 3, 40, 56, 150, _moe(4, 4, 24, scale=1.0), coef=1.0, every=1),
    _par(_left(6, 2, 8, 136, 70, 80, rot_dims=0), 3, 40, None, left_scale=0.5, right_scale=1.5),
    _att(6, 3, 40, 56, 300, _dense(72), coef=0.2, every=100, kv_from=0, scale=0.1),
    _par(_left(3, 1, 80, 40, 200, 70, rot_dims=32, base=77.0), 1, 80, _dense(200))], eps=1e-5)
SHAPE_C = _model(200, 48, [
    _par(_left(1, 1, 16, 16, 1, 3), 3, 16, _moe(4, 2, 8)),
    _par(_left(3, 1, 32, 48, 1000, 0, rot_dims=16), 1, 48, _dense(56), left_scale=1.0, right_scale=1.0)])
SHAPES = {"A": (SHAPE_A, 31), "B": (SHAPE_B, 32), "C": (SHAPE_C, 33)}
CASES = [(name, dtype) for name in SHAPES for dtype in ("float32", "bfloat16")]
TOL = {"float32": 2e-4, "bfloat16": 4e-2}
# A router's choice between two experts whose logits lie this close may fall either way once
# the stream is rounded to bfloat16 (float32: to its last bits); such a token's row, a
# legitimate other model's, is not compared, and a row after it in its request (which sees it
# through the state or the cache) that misses the tolerance is excused; both kinds together
# stay a small share of all rows, and a row with no close call before it is never excused.
CLOSE = {"float32": 1e-3, "bfloat16": 0.25}
# The same for a time-mixing head whose result is what large terms leave of one another (at a
# sequence's first token it is r . (u k) times v, and the unit norm keeps the sign alone): below
# this share of the terms' absolute sum, the inputs' rounding decides the direction.
CANCELLED = {"float32": 1e-5, "bfloat16": 0.01}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from pretrained_rstr_b200.config.registry import lookup
    from pretrained_rstr_b200.weights import make_random_model
    from pretrained_rstr_b200.weights.safetensors_io import save_file
    out = {}
    for name, (raw, seed) in SHAPES.items():
        cfg = lookup(raw).config_class.from_dict(raw)
        for dtype in ("float32", "bfloat16"):
            path = str(tmp_path_factory.mktemp(f"devalorn{name}_{dtype}"))
            make_random_model(path, cfg, seed, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
            # decisive routers: fewer tokens whose choice hangs on the last bits
            _, tensors = P.read_folder(path)
            for key in tensors:
                if key.endswith(".router"):
                    tensors[key] = tensors[key] * 3.0
            save_file(tensors, path + "/model.safetensors")
            out[(name, dtype)] = path
    return out


class Oracle(dict):
    pass


def _oracle(folder, prompts, dtype="float32"):
    cfg, tensors = P.read_folder(folder)
    out = Oracle()
    out.close = {}
    for rid, ids in prompts.items():
        gaps, kept = [], []
        out[rid] = P.forward(list(ids), tensors, cfg, margins=gaps, cancelled=kept).to(torch.float32)
        close = torch.zeros(len(ids), dtype=torch.bool)
        if gaps:
            close |= torch.stack(gaps).min(0).values < CLOSE[dtype]
        if kept:
            close |= torch.stack(kept).min(0).values < CANCELLED[dtype]
        out.close[rid] = close
    return out


def row_error(row, ref) -> float:
    """Root mean square of the difference (its mean taken off) over that of the reference row."""
    d = row.double() - ref.double()
    d = d - d.mean()
    r = ref.double() - ref.double().mean()
    return float(d.pow(2).mean().sqrt() / r.pow(2).mean().sqrt())


def compare(rows, oracle, tol):
    assert rows
    worst, skipped = 0.0, 0
    for (rid, pos), row in sorted(rows.items()):
        err = row_error(row, oracle[rid][pos])
        assert err == err, f"NaN at request {rid} position {pos}"
        close = oracle.close[rid]
        if bool(close[pos]):
            skipped += 1
            continue
        if err > tol and bool(close[:pos].any()):
            skipped += 1
            continue
        assert err <= tol, (f"request {rid} position {pos} (page offset {pos % 64}): relative "
                            f"difference {err:.3e} > {tol:.1e}")
        worst = max(worst, err)
    assert skipped <= 0.3 * len(rows), "too many close router calls for the test to mean much"
    return worst


def _prompts(name, lengths, salt=0):
    raw, seed = SHAPES[name]
    return {f"r{i}": random_tokens(n, raw["vocab"], 1000 * seed + salt + i) for i, n in enumerate(lengths)}


# ------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompts_decode_and_portions(folders, name, dtype):
    """Whole prompts in one step; the last tokens one by one (across windows' and kept tokens'
    edges); portions of several sizes, down to two tokens, cut inside pages and windows."""
    folder = folders[(name, dtype)]
    prompts = _prompts(name, [1, 2, 23, 64, 65, 150, 330])
    oracle = _oracle(folder, prompts, dtype)
    rp = Replayer(folder, dtype, max_tokens=512)
    for rid, ids in prompts.items():
        rp.step([(rid, ids, list(range(len(ids))))], end=[rid])
    compare(rp.rows, oracle, TOL[dtype])
    rp.rows.clear()
    for rid, ids in prompts.items():
        head = max(1, len(ids) - 40)
        rp.step([(rid, ids[:head], [head - 1])], end=[rid] if head == len(ids) else [])
        for i in range(head, len(ids)):
            rp.step([(rid, ids[i:i + 1], [0])], end=[rid] if i == len(ids) - 1 else [])
    compare(rp.rows, oracle, TOL[dtype])
    rp.rows.clear()
    sizes = [3, 2, 19, 2, 2, 40, 5, 64, 2, 66, 2, 130]
    for r, (rid, ids) in enumerate(prompts.items()):
        at, k = 0, r
        while at < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - at)
            k += 1
            rp.step([(rid, ids[at:at + n], list(range(n)))], end=[rid] if at + n >= len(ids) else [])
            at += n
    compare(rp.rows, oracle, TOL[dtype])


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16"), ("B", "float32"), ("C", "float32")])
def test_long_decode(folders, name, dtype):
    """Two tokens of prompt and some 340 decoded one by one: every window, the kept tokens' end
    and several pages' borders are passed by single tokens, the state is carried all the way."""
    folder = folders[(name, dtype)]
    prompts = _prompts(name, [342], salt=50)
    oracle = _oracle(folder, prompts, dtype)
    rp = Replayer(folder, dtype, max_tokens=384)
    ids = prompts["r0"]
    rp.step([("r0", ids[:2], [0, 1])])
    for i in range(2, len(ids)):
        rp.step([("r0", ids[i:i + 1], [0])])
    compare(rp.rows, oracle, TOL[dtype])


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_batches_with_reuse(folders, name, dtype):
    """Up to four live requests of unequal lengths, portions of some beside single tokens of
    others, some left out of a step, in a pool so small that pages and state slots of finished
    requests are used again: every row as if its request ran alone."""
    folder = folders[(name, dtype)]
    lengths = [130, 64, 250, 9, 33, 200, 1, 120, 2, 77]
    prompts = _prompts(name, lengths, salt=90)
    oracle = _oracle(folder, prompts, dtype)
    biggest = sorted((-(-n // 64) * 64 for n in lengths), reverse=True)
    rp = Replayer(folder, dtype, max_tokens=sum(biggest[:4]))
    rng = random.Random(5)
    waiting, live, slots_seen = list(prompts), {}, []
    while waiting or live:
        while waiting and len(live) < 4:
            live[waiting.pop(0)] = 0
        entries, end = [], []
        for rid in list(live):
            ids, at = prompts[rid], live[rid]
            left = len(ids) - at
            if rng.random() < 0.25 and len(live) > 1:
                continue                                   # left out of this step
            if left > 20 and at < len(ids) - 12:
                n = min(left - 12, rng.choice([2, 3, 8, 21, 64, 70]))
            else:
                n = 1
            entries.append((rid, ids[at:at + n], list(range(n))))
            live[rid] = at + n
            if live[rid] == len(ids):
                end.append(rid)
                del live[rid]
        if entries:
            rp.step(entries, end=end)
            slots_seen += [rp.lm.cache.slot(r) for r in live if r in rp.pos]
    cache = rp.lm.cache
    assert cache.stats["allocated"] > cache.allocators[0].num_pages
    assert cache.free_pages(0) == cache.allocators[0].num_pages
    assert len(prompts) > 4 >= len(set(slots_seen))          # state slots were used again
    compare(rp.rows, oracle, TOL[dtype])


def test_marked_token_at_every_edge(folders, tmp_path):
    """A model whose keys are made to matter: one token id whose table row is large makes its
    key and value stand out wherever it sits.  It is put just inside and just outside each
    window and the kept first tokens, in a prompt and while decoding; a window one token off, a
    kept token dropped or a lost state moves the logits far beyond the tolerance."""
    from pretrained_rstr_b200.weights.safetensors_io import save_file
    folder = folders[("A", "float32")]
    cfg, tensors = P.read_folder(folder)
    tensors = {k: v.clone() for k, v in tensors.items()}
    marked = 7
    tensors["embed"][marked] *= 6.0
    path = str(tmp_path / "marked")
    import os
    import shutil
    os.makedirs(path)
    shutil.copy(folder + "/config.json", path + "/config.json")
    save_file(tensors, path + "/model.safetensors")
    n = 120
    windows = [24, 40, 12, 18]
    rp = Replayer(path, "float32", max_tokens=4 * 128)
    prompts = {}
    for w in windows:
        for delta in (0, 1):                                     # just inside, just outside
            ids = [t if t != marked else marked + 1 for t in random_tokens(n, cfg["vocab"], 400 + w)]
            ids[n - w + (1 - delta) - 1] = marked                 # distance w - 1 + delta from the end
            prompts[f"w{w}_{delta}"] = ids
    ids = [t if t != marked else marked + 1 for t in random_tokens(n, cfg["vocab"], 500)]
    for spot in (4, 5):                                          # the last kept token and the next
        prompts[f"k{spot}"] = ids[:spot] + [marked] + ids[spot + 1:]
    oracle = _oracle(path, prompts)
    # rows differ between "inside" and "outside": the marked token matters to the last row
    for w in windows[:1]:
        a, b = oracle[f"w{w}_0"][n - 1], oracle[f"w{w}_1"][n - 1]
        assert row_error(a, b) > 20 * TOL["float32"]
    for rid, ids in prompts.items():                             # in a prompt
        rp.step([(rid, ids, [n - 2, n - 1])], end=[rid])
    compare(rp.rows, oracle, TOL["float32"])
    rp.rows.clear()
    for rid, ids in prompts.items():                             # decoding over the edge
        rp.step([(rid, ids[:n - 45], [])])
        for i in range(n - 45, n):
            rp.step([(rid, ids[i:i + 1], [0])], end=[rid] if i == n - 1 else [])
    compare(rp.rows, oracle, TOL["float32"])


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A", "bfloat16"), ("C", "float32")])
def test_greedy_generation_entry_point(folders, name, dtype):
    """``load_lm`` / ``generate_ids`` / ``generate_batch``: the scheduler's portions, batches
    and the steps launched ahead of their token ids choose the plain implementation's tokens."""
    from pretrained_rstr_b200 import generate_batch, generate_ids, load_lm
    folder = folders[(name, dtype)]
    cfg, tensors = P.read_folder(folder)
    m = load_lm(folder, gpu=True, dtype=dtype, max_lanes=3, max_batched_tokens=128,
                prefill_chunk=32, maxpos=256)
    prompts = list(_prompts(name, [1, 9, 33, 70, 130], salt=200).values())
    n_new = 10

    def agree(prompt, got):
        want = P.greedy(prompt, n_new, tensors, cfg)
        for i, (a, b) in enumerate(zip(got, want)):
            if a != b:
                row = P.forward(list(prompt) + want[:i], tensors, cfg)[-1]
                gap = abs(float(row[a] - row[b]))
                assert dtype == "bfloat16" and gap < 0.1, \
                    f"token {i} is {a}, plain says {b} (logit gap {gap:.3g})"
                return
        assert len(got) == len(want)

    agree(prompts[1], generate_ids(m, prompts[1], n_new))
    for p, got in zip(prompts, generate_batch(m, prompts, n_new)):
        agree(p, got)
    cache = m.engine.lm.cache
    assert not cache.requests
    cache.check()


def test_replay_and_generate_as_programs(folders, tmp_path):
    """``bin/trace_run`` and ``python -m pretrained_rstr_b200 generate`` on a Devalorn folder:
    the model class comes from config.json; logits of a replayed trace match the plain ones."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder = folders[("A", "float32")]
    cfg, tensors = P.read_folder(folder)
    ids = random_tokens(40, cfg["vocab"], 77)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ids[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": ids[30:32], "want": []},
                                     {"id": "b", "tokens": ids[:3], "want": [2]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": ids[32:], "want": [7]}], "end": ["a"]}]
    out = tmp_path / "out"
    proc = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype",
                           "float32", "--out", str(out), "--max-tokens", "128"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", text=True,
                          capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    want = P.forward(ids, tensors, cfg).to(torch.float32)
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1).copy())
    got1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1).copy())
    got2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(1, -1).copy())
    assert not (out / "3.f32").exists()
    for row, ref in ((got0[0], want[0]), (got0[1], want[29]), (got1[0], want[2]), (got2[0], want[39])):
        assert row_error(row, ref) < TOL["float32"]
    gen = subprocess.run([sys.executable, "-m", "pretrained_rstr_b200", "generate", "--model", folder,
                          "--dtype", "float32", "--ids", ",".join(map(str, ids[:12])), "--n", "6",
                          "--maxpos", "64"], cwd=root, capture_output=True, text=True, timeout=600)
    assert gen.returncode == 0, gen.stderr[-2000:]
    rec = json.loads(gen.stdout.strip().splitlines()[-1])
    assert rec["generated"] == P.greedy(ids[:12], 6, tensors, cfg)
