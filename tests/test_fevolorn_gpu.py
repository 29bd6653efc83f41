"""Fevolorn on the GPU against the plain implementation (tests/plain_fevolorn.py): every mechanism's
kernels alone, then whole models through trace replay in every way of cutting, and greedy generation
through the entry point."""
import math

import numpy as np
import pytest
import torch

import plain_fevolorn as pv
import replay_util as ru
from fevolorn_util import FV_A, FV_B, FV_C, sharpen, write_model

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-5, "bfloat16": 5e-2}
F64 = torch.float64


def rel(got, want):
    return float((got.double().cpu() - want).abs().max() / want.abs().max())


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device="cuda")


def err_word():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


# ---------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("S", [1, 3, 8])
def test_streams_are_read_written_and_summed(dtype, S):
    """The read, the write-back of all streams from the old ones (mix indexed [from, to]) with the next
    read and its norm in the same kernel, and the sum of the streams at chosen rows."""
    from rllm_b200.kernels import ops
    g = torch.Generator().manual_seed(S)
    T, H = 19, 52
    xs = torch.randn(S, T, H, generator=g)
    a, b, a2 = torch.randn(S, generator=g), torch.randn(S, generator=g), torch.randn(S, generator=g)
    M = torch.randn(S, S, generator=g)
    y = torch.randn(T, H, generator=g).to(DT[dtype])
    ls = torch.randn(H, generator=g).to(DT[dtype])
    alpha, w, c = torch.tensor([0.37]), torch.randn(H, generator=g).to(DT[dtype]), torch.randn(H, generator=g).to(DT[dtype])
    norm = (alpha.cuda(), w.cuda(), c.cuda())
    xd = xs.cuda()
    got = ops.streams_read(xd, a.cuda(), norm, DT[dtype])
    u = torch.einsum("s,sth->th", a.double(), xs.double())
    want = torch.tanh(0.37 * u) * w.double() + c.double()
    assert rel(got, want) <= (1e-6 if dtype == "float32" else 1e-2)
    assert rel(ops.streams_read(xd, a.cuda(), None, DT[dtype]), u) <= 1e-6
    sums = torch.empty(T, H, device="cuda")
    nxt = ops.streams_write(xd, y.cuda(), ls.cuda(), M.cuda(), b.cuda(), next_read=a2.cuda(), norm=norm, sum_out=sums)
    new = torch.einsum("st,sxh->txh", M.double(), xs.double()) + b.double()[:, None, None] * (y.double() * ls.double())[None]
    assert rel(xd, new) <= 1e-6
    u2 = torch.einsum("s,sth->th", a2.double(), new)
    assert rel(nxt, torch.tanh(0.37 * u2) * w.double() + c.double()) <= (1e-6 if dtype == "float32" else 1e-2)
    assert rel(sums, new.sum(0)) <= 1e-6
    rows = [4, 0, 18, 4]
    got = ops.streams_read(xd, None, norm, DT[dtype], rows=i32(rows))
    want = torch.tanh(0.37 * new.sum(0)[rows]) * w.double() + c.double()
    assert rel(got, want) <= (1e-6 if dtype == "float32" else 1e-2)
    # without a scale and without a reader behind it
    before = xd.double().cpu()
    assert ops.streams_write(xd, y.cuda(), None, M.cuda(), b.cuda()) is None
    assert rel(xd, torch.einsum("st,sxh->txh", M.double(), before) + b.double()[:, None, None] * y.double()[None]) <= 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_tanh_norm_alone_with_an_add_and_chosen_rows(dtype):
    from rllm_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    x, d = torch.randn(9, 40, generator=g) * 3, torch.randn(9, 40, generator=g).to(DT[dtype])
    w, c, alpha = torch.randn(40, generator=g), torch.randn(40, generator=g), torch.tensor([1.3])
    xd, out = x.cuda(), torch.empty(9, 40, dtype=DT[dtype], device="cuda")
    ops.dyt(xd, alpha.cuda(), w.cuda(), c.cuda(), out, delta=d.cuda(), writeback=True)
    s = x.double() + d.double()
    assert rel(out, torch.tanh(1.3 * s) * w.double() + c.double()) <= (1e-6 if dtype == "float32" else 1e-2)
    assert rel(xd, s) <= 1e-7
    out = torch.empty(2, 40, dtype=DT[dtype], device="cuda")
    ops.dyt(xd, alpha.cuda(), w.cuda(), c.cuda(), out, rows=i32([7, 2]))
    assert rel(out, torch.tanh(1.3 * s[[7, 2]]) * w.double() + c.double()) <= (1e-6 if dtype == "float32" else 1e-2)


def _lightning_plain(q, k, v, decay, state, lens, slots, round_act=False):
    """state [slots, heads, d, dv] (updated), returns o [T, heads * dv]; float64.  ``round_act``: the
    activated q, k and v are rounded to bfloat16 (what the tensor-core form of the chunk passes does)."""
    heads, d, dv = state.shape[1:]
    T = q.shape[0]
    out = torch.zeros(T, heads, dv, dtype=F64)
    off = 0
    for n, sl in zip(lens, slots):
        for h in range(heads):
            S = state[sl, h].clone()
            for t in range(off, off + n):
                kk, vv, qq = (pv.silu(x[t].double().view(heads, -1)[h]) for x in (k, v, q))
                if round_act:
                    kk, vv, qq = (x.float().bfloat16().double() for x in (kk, vv, qq))
                S = decay[h] * S + torch.outer(kk, vv)
                out[t, h] = S.t() @ qq
            state[sl, h] = S
        off += n
    return out.reshape(T, heads * dv)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,d,dv,lens", [(3, 20, 24, [1, 2, 37]), (1, 64, 128, [5, 1, 1]), (5, 8, 70, [140, 3, 129]),
                                             (2, 100, 16, [300, 1, 64]), (1, 200, 40, [70, 2, 1])])
def test_lightning_scan_carries_its_state_across_cuts_and_slots(dtype, heads, d, dv, lens):
    """Sequences of unequal length in one launch (the long ones go through the chunked form), one of them
    continuing from a state that an earlier call left; slots in another order than the sequences; a decay
    of one (nothing is forgotten) and a fast one."""
    from rllm_b200.kernels import ops
    g = torch.Generator().manual_seed(d)
    T, slots = sum(lens), [4, 0, 2]
    a = torch.randn(T, 2 * heads * d + heads * dv + 7, generator=g).to(DT[dtype])
    qk = heads * d
    q, k, v = a[:, :qk], a[:, qk:2 * qk], a[:, 2 * qk:2 * qk + heads * dv]
    decay = torch.tensor(([1.0, 0.4, 0.97, 0.999, 0.8] * 2)[:heads], dtype=torch.float32)
    state = torch.zeros(6, heads, d, dv)
    state[0] = torch.randn(heads, d, dv, generator=g)
    want_state = state.double().clone()
    want = _lightning_plain(q, k, v, decay.double(), want_state, lens, slots)
    ad, st = a.cuda(), state.cuda()
    err = err_word()
    starts = [0] + list(np.cumsum(lens))
    got = ops.lightning_scan(ad[:, :qk], ad[:, qk:2 * qk], ad[:, 2 * qk:2 * qk + heads * dv], decay.cuda(), st,
                             i32(starts), i32(slots), 3, err, max_q_len=max(lens))
    assert int(err.item()) == 0
    assert rel(got, want) <= 2e-6
    assert rel(st, want_state) <= 2e-6
    assert torch.equal(st[[1, 3, 5]].cpu(), state[[1, 3, 5]])


@pytest.mark.parametrize("heads,d,dv,lens,decay", [(2, 32, 64, [200, 3, 129], [1.0, 0.6]), (1, 128, 128, [150, 64, 1], [0.97]),
                                                   (3, 64, 64, [130, 1, 70], [0.999, 0.05, 0.0]), (2, 128, 64, [65, 257, 2], [0.9, 0.5]),
                                                   (1, 64, 128, [129, 16, 17], [0.8]), (2, 32, 128, [300, 5, 63], [0.99, 0.7])])
def test_lightning_chunk_passes_on_the_tensor_cores(heads, d, dv, lens, decay):
    """Long portions of bfloat16 activations at the head sizes the tensor-core form is built for: chunks of
    64 with a ragged last one, sequences shorter than a chunk beside them, a state left by an earlier call,
    decays of one, nearly zero and zero; against the token-by-token recurrence in float64 on the same
    bfloat16-rounded activations.  Weights, start states and weighted keys pass as value + remainder, so the
    result keeps float32's digits (nearly: 16 bits of mantissa a factor)."""
    from rllm_b200.kernels import ops
    g = torch.Generator().manual_seed(d + dv)
    T, slots, qk = sum(lens), [4, 0, 2], heads * d
    a = torch.randn(T, 2 * qk + heads * dv + 6, generator=g).bfloat16()
    lam = torch.tensor(decay, dtype=torch.float32)
    state = torch.zeros(6, heads, d, dv)
    state[0] = torch.randn(heads, d, dv, generator=g)
    want_state = state.double().clone()
    want = _lightning_plain(a[:, :qk], a[:, qk:2 * qk], a[:, 2 * qk:2 * qk + heads * dv], lam.double(), want_state, lens,
                            slots, round_act=True)
    ad, st, err = a.cuda(), state.cuda(), err_word()
    got = ops.lightning_scan(ad[:, :qk], ad[:, qk:2 * qk], ad[:, 2 * qk:2 * qk + heads * dv], lam.cuda(), st,
                             i32([0] + list(np.cumsum(lens))), i32(slots), 3, err, max_q_len=max(lens))
    assert int(err.item()) == 0
    assert rel(got, want) <= 3e-5
    assert rel(st, want_state) <= 3e-5
    assert torch.equal(st[[1, 3, 5]].cpu(), state[[1, 3, 5]])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps", [1, 2, 4, 7, 9])
def test_the_convolution_reads_its_tail_and_moves_it_on(dtype, taps):
    """A sequence fed as 1 + 2 + 1 + 9 + 1 tokens beside others, against the convolution of the whole
    sequence: the last taps - 1 inputs travel in the state, also when a step brings fewer than that."""
    from rllm_b200.kernels import ops
    g = torch.Generator().manual_seed(taps)
    E, cuts = 37, [1, 2, 1, 9, 1]
    x = torch.randn(sum(cuts), 2 * E, generator=g).to(DT[dtype])
    other = torch.randn(40, 2 * E, generator=g).to(DT[dtype])
    w, b = torch.randn(E, taps, generator=g), torch.randn(E, generator=g)
    xx = x[:, :E].double()
    padded = torch.cat([torch.zeros(taps - 1, E, dtype=F64), xx])
    want = pv.silu(sum(padded[j:j + len(xx)] * w.double()[:, j] for j in range(taps)) + b.double())
    tail = torch.zeros(5, max(taps - 1, 0), E, device="cuda")
    tail[1] = 7.0                                # another request's tail stays as it is
    got, at, o_at = [], 0, 0
    for n in cuts:
        m = 3 if o_at + 3 <= 40 else 0           # another sequence rides along, first or second in the batch
        rows = torch.cat([other[o_at:o_at + m], x[at:at + n]]) if n == 1 else torch.cat([x[at:at + n], other[o_at:o_at + m]])
        lens = [m, n] if n == 1 else [n, m]
        slots = [3, 2] if n == 1 else [2, 3]
        rd = rows.cuda()
        tseq = [0] * lens[0] + [1] * lens[1]
        out = ops.causal_conv(rd[:, :E], w.cuda(), b.cuda(), tail, i32([0, lens[0], lens[0] + lens[1]]), i32(tseq),
                              i32(slots), 2, True, err_word())
        got.append(out[m:m + n] if n == 1 else out[:n])
        at, o_at = at + n, o_at + m
    assert rel(torch.cat(got), want) <= (2e-6 if dtype == "float32" else 1e-2)
    assert torch.all(tail[1] == 7.0)
    if taps > 1:
        assert rel(tail[2], xx[-(taps - 1):]) <= 1e-7


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,N,lens", [(37, 10, [1, 2, 37]), (130, 16, [200, 1, 129]), (20, 40, [3, 70, 1])])
def test_selective_scan_carries_its_state_across_cuts_and_slots(dtype, E, N, lens):
    from rllm_b200.kernels import ops
    g = torch.Generator().manual_seed(E)
    T, slots, R = sum(lens), [4, 0, 2], 3
    xc = torch.randn(T, E, generator=g).to(DT[dtype])
    z = torch.randn(T, 2 * E, generator=g).to(DT[dtype])
    proj = torch.randn(T, R + 2 * N, generator=g).to(DT[dtype])
    dt_raw = torch.randn(T, E, generator=g)
    dt_b, a_log, D = torch.randn(E, generator=g), torch.randn(E, N, generator=g) - 1.0, torch.randn(E, generator=g)
    state = torch.zeros(6, N, E)
    state[0] = torch.randn(N, E, generator=g)
    ws = state.double().clone()
    want = torch.zeros(T, E, dtype=F64)
    A, off = -torch.exp(a_log.double()), 0
    for n, sl in zip(lens, slots):
        S = ws[sl].t().clone()                                   # [E, N]
        for t in range(off, off + n):
            dt = pv.softplus(dt_raw[t].double() + dt_b.double())
            x = xc[t].double()
            S = torch.exp(dt[:, None] * A) * S + (dt * x)[:, None] * proj[t, R:R + N].double()[None]
            want[t] = (S @ proj[t, R + N:].double() + D.double() * x) * pv.silu(z[t, E:].double())
        ws[sl] = S.t()
        off += n
    st, zd = state.cuda(), z.cuda()
    err = err_word()
    got = ops.selective_scan(xc.cuda(), dt_raw.cuda(), dt_b.cuda(), proj.cuda(), R, R + N, a_log.cuda(), D.cuda(),
                             zd[:, E:], st, i32([0] + list(np.cumsum(lens))), i32(slots), 3, err, max_q_len=max(lens))
    assert int(err.item()) == 0
    assert rel(got, want) <= (3e-6 if dtype == "float32" else 1e-2)
    assert rel(st, ws) <= 3e-6
    assert torch.equal(st[[1, 3, 5]].cpu(), state[[1, 3, 5]])


def _paged_attention_case(dtype, nq, nkv, dk, dv, page, window, lens, news, scale, boost=None, seed=0):
    """Sequences whose keys lie on shuffled pages; the last ``news[s]`` tokens of sequence s are this
    step's: their queries and keys are normalised per head and their keys and values written by the
    kernel, the earlier keys (already normalised) and values are in the pages.  Returns (got, want)
    [T, nq, dv] over this step's tokens."""
    from rllm_b200.kernels import ops
    g = torch.Generator().manual_seed(seed)
    eps, S = 1e-5, len(lens)
    wq, wk = torch.rand(dk, generator=g) + 0.5, torch.rand(dk, generator=g) + 0.5
    per = [-(-n // page) for n in lens]
    perm = torch.randperm(sum(per) + 3, generator=g)
    table = torch.full((S, max(per)), -1, dtype=torch.int32)
    kc = torch.zeros(sum(per) + 3, nkv, page, dk, dtype=DT[dtype])
    vc = torch.zeros(sum(per) + 3, nkv, page, dv, dtype=DT[dtype])
    rows, positions, tseq, want = [], [], [], []
    at = 0
    for s, (n, new) in enumerate(zip(lens, news)):
        table[s, :per[s]] = perm[at:at + per[s]].to(torch.int32)
        at += per[s]
        q = torch.randn(n, nq, dk, generator=g)
        k = torch.randn(n, nkv, dk, generator=g)
        v = torch.randn(n, nkv, dv, generator=g).to(DT[dtype])
        if boost is not None:
            boost(s, q, k)
        q, k = q.to(DT[dtype]), k.to(DT[dtype])
        qn = pv.unit_rms(q.double(), wq.double(), eps)
        kn = pv.unit_rms(k.double(), wk.double(), eps)
        if dtype == "bfloat16":                          # the kernel hands both on as bfloat16
            qn, kn = qn.bfloat16().double(), kn.bfloat16().double()
        for j in range(n - new):
            kc[table[s, j // page], :, j % page] = kn[j].to(DT[dtype])
            vc[table[s, j // page], :, j % page] = v[j]
        for j in range(n - new, n):
            rows.append(torch.cat([q[j].reshape(-1), k[j].reshape(-1), v[j].reshape(-1)]))
            positions.append(j)
            tseq.append(s)
            o = torch.zeros(nq, dv, dtype=F64)
            lo = max(0, j - window + 1) if window else 0
            for h in range(nq):
                kv = h // (nq // nkv)
                p = torch.softmax(kn[lo:j + 1, kv] @ qn[j, h] * scale, dim=0)
                o[h] = p @ v[lo:j + 1, kv].double()
            want.append(o)
    qkv = torch.stack(rows).cuda()
    kcd, vcd, err = kc.cuda(), vc.cuda(), err_word()
    ops.head_norm_kv_write(qkv, i32(positions), i32(tseq), wq.cuda(), wk.cuda(), eps, table.cuda(), kcd, vcd, nq, nkv,
                           dk, dv, err)
    out = torch.empty(len(rows), nq * dv, dtype=DT[dtype], device="cuda")
    ops.attention_simt_kv(qkv, qkv.shape[1], out, kcd, vcd, table.cuda(), i32(positions), i32(tseq), nq, nkv, window,
                          scale, err)
    assert int(err.item()) == 0
    return out.view(len(rows), nq, dv), torch.stack(want)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,dk,dv,page,window", [(6, 2, 24, 40, 16, 11), (4, 4, 16, 16, 4, 37), (2, 1, 64, 128, 16, 0),
                                                      (3, 3, 10, 6, 8, 1), (8, 2, 72, 200, 16, 100)])
def test_attention_with_head_norms_and_values_of_their_own_size(dtype, nq, nkv, dk, dv, page, window):
    """A prompt portion behind a cached prefix, a single decoded token and a whole short prompt in one
    launch; keys on shuffled pages; against the formula in float64."""
    got, want = _paged_attention_case(dtype, nq, nkv, dk, dv, page, window, [83, 141, 19], [50, 1, 19], dk ** -0.5 * 3)
    assert rel(got, want) <= (3e-6 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("window,page", [(5, 16), (16, 16), (17, 4), (96, 16)])
@pytest.mark.parametrize("new", [1, 30])
def test_a_key_just_inside_and_just_outside_the_window(window, page, new):
    """One key among hundreds gets a score far above the rest (queries and that key point along one axis,
    all other keys have nothing there), so whoever sees it returns its value: the query that has it as the
    oldest key of its window must, the next query must not; as a decoded token and inside a prompt
    portion, with the window's edge on and off a page border, far behind the step's first token."""
    n = 3 * window + 40
    last = n - 1

    def run(key_pos):
        def boost(s, q, k):
            q.mul_(0.05)
            q[:, :, 0] = 6.0
            k[:, :, 0] = 0.0
            k[key_pos].mul_(0.05)
            k[key_pos, :, 0] = 6.0
        return _paged_attention_case("float32", 2, 1, 8, 8, page, window, [n], [new], 4.0, boost=boost, seed=window)

    g1, w1 = run(last - window + 1)                # the oldest key the last query still sees
    g0, w0 = run(last - window)                    # one further back: hidden from the last query
    assert rel(g1, w1) <= 3e-6 and rel(g0, w0) <= 3e-6
    # seen or not seen differs at the last query by far more than rounding
    assert float((w1[-1] - w0[-1]).abs().max()) > 0.2
    assert float((g1[-1].double().cpu() - w0[-1]).abs().max()) > 0.2


@pytest.mark.parametrize("T,E,top", [(1, 5, 2), (7, 3, 3), (50, 12, 3), (300, 40, 1)])
def test_the_sigmoid_router_chooses_by_corrected_scores_and_weighs_by_the_scores(T, E, top):
    from rllm_b200.kernels import ops
    g = torch.Generator().manual_seed(T)
    z = torch.randn(T, E, generator=g) * 2
    z[0, :] = 0.3                                      # all equal: the lowest indices win
    corr = torch.randn(E, generator=g)
    ids, wts = ops.moe_choose_sigmoid(z.cuda(), top, corr.cuda(), 2.5)
    s = torch.sigmoid(z.double())
    want_ids = torch.sort(s.float() + corr, dim=-1, descending=True, stable=True).indices[:, :top]
    assert torch.equal(ids.cpu().long(), want_ids)
    assert rel(wts, torch.gather(s, 1, want_ids) * 2.5) <= 1e-6
    # the correction moves the choice and leaves the weights alone
    big = torch.zeros(E)
    big[E - 1] = 10.0
    ids2, wts2 = ops.moe_choose_sigmoid(z.cuda(), top, big.cuda(), 1.0)
    assert torch.all(ids2[:, 0] == E - 1)
    assert rel(wts2[:, 0], s[:, E - 1]) <= 1e-6
    ids3, _ = ops.moe_choose_sigmoid(z.cuda(), top, None, 1.0)
    assert torch.equal(ids3.cpu().long(), torch.sort(s.float(), dim=-1, descending=True, stable=True).indices[:, :top])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_small_steps_around_mixers_and_feed_forwards(dtype):
    """The tanh-gelu gate, the mean of two unit-rms branches, the gated unit-rms norm, the experts' sum with a
    gated shared row, and experts with the plain SiLU gate."""
    from rllm_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    tol = 2e-6 if dtype == "float32" else 1e-2
    T, I, H = 11, 36, 52
    gu = (torch.randn(T, 2 * I, generator=g) * 2).to(DT[dtype])
    out = torch.empty(T, I, dtype=DT[dtype], device="cuda")
    ops.act_mul(gu.cuda(), out, "gelu_tanh")
    assert rel(out, pv.gelu_tanh(gu[:, :I].double()) * gu[:, I:].double()) <= tol
    ops.act_mul(gu.cuda(), out, "silu")
    assert rel(out, pv.silu(gu[:, :I].double()) * gu[:, I:].double()) <= tol
    a, b = torch.randn(T, H, generator=g).to(DT[dtype]), (torch.randn(T, H, generator=g) * 5).to(DT[dtype])
    wa, wb = torch.randn(H, generator=g), torch.randn(H, generator=g)
    got = ops.rms_mean2(a.cuda(), b.cuda(), wa.cuda(), wb.cuda(), 1e-3)
    assert rel(got, 0.5 * (pv.unit_rms(a.double(), wa.double(), 1e-3) + pv.unit_rms(b.double(), wb.double(), 1e-3))) <= tol
    x, gate = torch.randn(T, H, generator=g) * 4, torch.randn(T, H + 9, generator=g).to(DT[dtype])
    got = ops.gated_rmsnorm(x.cuda(), gate.cuda()[:, 9:], wa.cuda(), 1e-3, DT[dtype])
    assert rel(got, pv.unit_rms(x.double(), wa.double(), 1e-3) * torch.sigmoid(gate[:, 9:].double())) <= tol
    K = 3
    y, cf = torch.randn(T * K, H, generator=g).to(DT[dtype]), torch.rand(T, K, generator=g)
    sh, sg = torch.randn(T, H, generator=g).to(DT[dtype]), torch.randn(T, generator=g)
    out = torch.empty(T, H, dtype=DT[dtype], device="cuda")
    ops.weighted_slot_sum(y.cuda(), cf.cuda(), out, extra=sh.cuda(), extra_gate=sg.cuda())
    want = torch.einsum("tk,tkh->th", cf.double(), y.double().view(T, K, H)) + torch.sigmoid(sg.double())[:, None] * sh.double()
    assert rel(out, want) <= tol
    E, F = 4, 24
    h = torch.randn(T, H, generator=g).to(DT[dtype])
    wgu, wd = (torch.randn(E, 2 * F, H, generator=g) * 0.2).to(DT[dtype]), (torch.randn(E, H, F, generator=g) * 0.2).to(DT[dtype])
    ids = torch.randint(0, E, (T, 2), generator=g).to(torch.int32)
    got = ops.moe_experts(h.cuda(), ids.cuda(), wgu.cuda(), wd.cuda(), float("inf"), 1.0, 0.0).view(T, 2, H)
    for t in range(T):
        for j in range(2):
            e = int(ids[t, j])
            gg, uu = wgu[e, :F].double() @ h[t].double(), wgu[e, F:].double() @ h[t].double()
            assert rel(got[t, j], wd[e].double() @ (pv.silu(gg) * uu)) <= (1e-5 if dtype == "float32" else 3e-2)


# ---------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------
@pytest.fixture(scope="module")
def fv_dirs(tmp_path_factory):
    return {"A": write_model(str(tmp_path_factory.mktemp("fv_a")), FV_A, 21, sharpen),
            "B": write_model(str(tmp_path_factory.mktemp("fv_b")), FV_B, 22, sharpen),
            "C": write_model(str(tmp_path_factory.mktemp("fv_c")), FV_C, 23, sharpen)}


CFG = {"A": FV_A, "B": FV_B, "C": FV_C}


def plain_rows(folder, dtype, reqs):
    cfg, w = pv.read_model_dir(folder, round_to=torch.bfloat16 if dtype == "bfloat16" else None)
    return {r: pv.logits(cfg, w, toks).numpy() for r, toks in reqs.items()}


def compare(got, want, reqs, dtype, what):
    """float32: every position within the tolerance.  bfloat16: rounding can turn a router's close call
    the other way, which moves that token's logits (and, through the recurrent states, later ones) by
    more than rounding; up to 5 % of the positions may do so, the rest stays within the tolerance."""
    over = total = 0
    for r, toks in reqs.items():
        have = np.stack([got[(r, p)] for p in range(len(toks))])
        err = np.abs(have - want[r]).max(axis=1) / np.abs(want[r]).max()
        assert np.isfinite(have).all()
        if dtype == "float32":
            assert err.max() <= TOL[dtype], (what, r, int(err.argmax()), float(err.max()))
        over += int((err > TOL[dtype]).sum())
        total += len(toks)
    assert over <= 0.05 * total, (what, over, total)


def make_requests(vocab, lengths, seed):
    rng = np.random.default_rng(seed)
    return {f"r{i}": [int(t) for t in rng.integers(0, vocab, size=n)] for i, n in enumerate(lengths)}


def test_layers_match_the_plain_residual_after_every_run(fv_dirs):
    """The sum of the streams after every layer run (a repeated layer counts each time) in float32."""
    from rllm_b200.engine.loading import load_model
    from rllm_b200.engine.replay import TraceSession
    cfg, w = pv.read_model_dir(fv_dirs["A"])
    toks = make_requests(FV_A["vocab"], [45], seed=2)["r0"]
    want = []
    pv.forward(cfg, w, toks, want)
    _, model = load_model(fv_dirs["A"], dtype="float32")
    sess = TraceSession(model, 64, 16, 2)
    trace, orig = [], sess.runner.build_context

    def with_trace(entries):
        ctx, a, b = orig(entries)
        ctx.extras["residual_trace"] = trace
        return ctx, a, b

    sess.runner.build_context = with_trace
    sess.step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": []}], "end": ["a"]})
    assert len(trace) == len(want) == 8
    for i, (g, x) in enumerate(zip(trace, want)):
        assert rel(g, x) <= 1e-5, i


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page", [("A", 16), ("A", 4), ("B", 8), ("C", 16)])
def test_every_way_of_cutting_gives_the_plain_logits(fv_dirs, name, page, dtype):
    """Whole prompts, token by token from the first token on, portions down to two tokens, and mixed
    batches of up to four live requests whose pages and slots are given back and used again (the pool
    holds exactly the peak); every position's logits are compared."""
    V = CFG[name]["vocab"]
    reqs = make_requests(V, [61, 1, 2, 17, 150, 33, 5], seed=7)
    want = plain_rows(fv_dirs[name], dtype, reqs)
    for what, tb in (("whole", ru.trace_whole(reqs)), ("one by one", ru.trace_tail_decode(reqs, tail=1000)),
                     ("tail decoded", ru.trace_tail_decode(reqs, tail=45)),
                     ("portions", ru.trace_portions(reqs, seed=1)), ("portions b", ru.trace_portions(reqs, seed=4)),
                     ("mixed", ru.trace_mixed(reqs, seed=2, live=4, tail=6)),
                     ("mixed b", ru.trace_mixed(reqs, seed=3, live=3, tail=30))):
        got = ru.run_trace(fv_dirs[name], dtype, tb, V, page_size=page, max_live=4)
        compare(got, want, reqs, dtype, f"{name}/{dtype}/page {page}/{what}")


def test_long_decoding_past_every_window_and_many_pages(fv_dirs):
    """A prompt of 3 tokens, then 200 tokens one by one (windows of 11 and 37; pages of 8: the windowed
    groups give pages back on the way), beside a second request that starts later."""
    V = FV_A["vocab"]
    reqs = make_requests(V, [203, 120], seed=9)
    want = plain_rows(fv_dirs["A"], "float32", reqs)
    tb = ru.TraceBuilder()
    a, b = reqs["r0"], reqs["r1"]
    tb.step([("r0", a[:3])])
    for i in range(3, 203):
        entries = [("r0", a[i:i + 1])]
        j = i - 60
        if j == 0:
            entries.append(("r1", b[:25]))
        elif 0 < j < 96:
            entries.append(("r1", b[24 + j:25 + j]))
        tb.step(entries, end=(["r0"] if i == 202 else []) + (["r1"] if j == 95 else []))
    got = ru.run_trace(fv_dirs["A"], "float32", tb, V, page_size=8)
    compare(got, want, reqs, "float32", "long decoding")


def test_a_long_prompt_goes_through_the_chunked_scans(fv_dirs):
    """Prompts long enough for the recurrences' chunked forms (side by side with a short one), whole and
    cut in the middle of a chunk, against the token-by-token plain model."""
    V = FV_A["vocab"]
    reqs = make_requests(V, [333, 9], seed=31)
    want = plain_rows(fv_dirs["A"], "float32", reqs)
    tb = ru.TraceBuilder()
    a, b = reqs["r0"], reqs["r1"]
    tb.step([("r0", a[:200]), ("r1", b)], end=["r1"])
    tb.step([("r0", a[200:])], end=["r0"])
    got = ru.run_trace(fv_dirs["A"], "float32", tb, V, page_size=16)
    compare(got, want, reqs, "float32", "chunked scans")


def test_the_runner_as_a_program_and_pools_no_larger_than_asked(fv_dirs):
    """bin/trace_run as a child process with a pool of exactly the peak of live tokens and its four slots."""
    V = FV_B["vocab"]
    reqs = make_requests(V, [40, 70, 9, 64, 3, 20], seed=13)
    want = plain_rows(fv_dirs["B"], "float32", reqs)
    tb = ru.trace_mixed(reqs, seed=5, live=4, tail=4)
    got = ru.run_trace(fv_dirs["B"], "float32", tb, V, page_size=16, subprocess_mode=True, max_live=None)
    compare(got, want, reqs, "float32", "child process")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(fv_dirs, dtype):
    """Nine requests through LLM.generate with the scheduler cutting prompts into portions of at most 16
    tokens beside decoding requests, CUDA graphs for the decode steps, more requests than sequences at a
    time.  float32: the plain implementation's tokens.  bfloat16: its choice at (nearly) all places where
    that is clear."""
    from rllm_b200 import LLM, SamplingParams
    V = FV_A["vocab"]
    rng = np.random.default_rng(17)
    prompts = [[int(t) for t in rng.integers(0, V, size=int(n))] for n in (5, 41, 1, 23, 60, 2, 9, 30, 14)]
    n_new = 12
    llm = LLM(fv_dirs["A"], dtype="fp32" if dtype == "float32" else "bf16", block_size=8, num_gpu_blocks=96,
              max_num_seqs=4, max_num_batched_tokens=24, long_prefill_token_threshold=16, enable_prefix_caching=False)
    assert llm.engine.runner.capture_graphs
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
    cfg, w = pv.read_model_dir(fv_dirs["A"], round_to=torch.bfloat16 if dtype == "bfloat16" else None)
    clear = wrong = 0
    for p, o in zip(prompts, outs):
        got = o.outputs[0].token_ids
        assert len(got) == n_new
        if dtype == "float32":
            assert got == pv.greedy(cfg, w, p, n_new)
            continue
        seq = list(p)
        for t in got:
            row = pv.logits(cfg, w, seq)[-1]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) > 6e-2 * float(row.abs().max()):
                clear += 1
                wrong += t != int(torch.argmax(row))
            seq.append(t)
    assert dtype == "float32" or (clear >= 20 and wrong <= 0.05 * clear), (clear, wrong)
    assert any(g.graph is not None for g in llm.engine.runner.graphs.values())
    llm.engine.cache.check()
    assert llm.engine.cache.usage()["num_requests"] == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_forked_request_copies_its_pages_and_every_state(fv_dirs, dtype):
    """A request is forked in the middle of a page; parent and child go on with different tokens and each
    matches the plain model on its own sequence: the partly filled page, the scan's state, the
    convolution's tail and the lightning states were copied."""
    V = FV_A["vocab"]
    base = make_requests(V, [43], seed=41)["r0"]
    ta, tb_ = make_requests(V, [20, 20], seed=42).values()
    reqs = {"a": base + ta, "b": base + tb_}
    want = plain_rows(fv_dirs["A"], dtype, reqs)
    tb = ru.TraceBuilder()
    tb.step([("a", base[:30])])
    tb.step([("a", base[30:])])
    tb.step([("a", ta[:5]), ("b", tb_[:1])], fork=[("a", "b")])
    tb.step([("a", ta[5:6]), ("b", tb_[1:9])])
    tb.step([("a", ta[6:]), ("b", tb_[9:])], end=["a", "b"])
    got = ru.run_trace(fv_dirs["A"], dtype, tb, V, page_size=16, max_tokens=256)
    for p in range(len(base)):
        got[("b", p)] = got[("a", p)]                # computed once, before the fork
    compare(got, want, reqs, dtype, "fork")
