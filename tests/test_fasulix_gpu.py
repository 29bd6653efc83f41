"""Fasulix on the GPU against the plain implementation (tests/plain_fasulix.py): every mechanism's
kernels alone, then whole models through trace replay in every way of cutting, and greedy generation
through the entry point."""
import math

import numpy as np
import pytest
import torch

import plain_fasulix as pf
import replay_util as ru
from fasulix_util import FX_A, FX_B, FX_C, FX_D, sharpen, write_model

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 4e-2}


def dev(t, dtype):
    return t.to(DT[dtype]).cuda().contiguous()


def rel(got, want):
    return float((got.double().cpu() - want).abs().max() / want.abs().max())


# ---------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mingru_scan_carries_its_state_across_cuts_and_slots(dtype):
    """Three sequences (1, 2 and 37 tokens this step), one of them continuing from a state that an earlier
    call left; slots in another order than the sequences."""
    from rllm_b200.kernels import ops
    torch.manual_seed(1)
    W, lens, slots = 50, [1, 2, 37], [4, 0, 2]
    T = sum(lens)
    a = (torch.randn(T, 3 * W) * 2).to(DT[dtype])
    bz, bx = torch.randn(W).to(DT[dtype]), torch.randn(W).to(DT[dtype])
    state = torch.zeros(6, W)
    state[0] = torch.rand(W)
    want_state = state.double().clone()
    want = torch.zeros(T, W, dtype=torch.float64)
    ad, off = a.double(), 0
    for n, sl in zip(lens, slots):
        s = want_state[sl].clone()
        for t in range(off, off + n):
            z = torch.sigmoid(ad[t, :W] + bz.double())
            u = ad[t, W:2 * W] + bx.double()
            s = (1 - z) * s + z * torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
            g = ad[t, 2 * W:]
            want[t] = s * g * torch.sigmoid(g)
        want_state[sl] = s
        off += n
    out = torch.empty(T, W, dtype=DT[dtype], device="cuda")
    st = state.cuda()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    q_start = torch.tensor([0, 1, 3, T], dtype=torch.int32, device="cuda")
    ops.mingru_scan(a.cuda(), bz.cuda(), bx.cuda(), st, q_start, torch.tensor(slots, dtype=torch.int32, device="cuda"),
                    3, out, err)
    assert int(err.item()) == 0
    assert rel(out, want) <= (1e-6 if dtype == "float32" else 1e-2)
    assert rel(st, want_state) <= 1e-6                # the state is float32 in both modes
    assert torch.equal(st[[1, 3, 5]].cpu(), state[[1, 3, 5]])


def _latent_case(dtype, T, heads, dk, dv, page, window, sink, seed=0, boost=None):
    """One sequence of T tokens whose rows lie on shuffled pages; queries at every position."""
    from rllm_b200.kernels import ops
    g = torch.Generator().manual_seed(seed)
    rows = torch.randn(T, dk, generator=g).to(DT[dtype])
    q = torch.randn(T, heads, dk, generator=g).to(DT[dtype])
    if boost is not None:
        boost(q, rows)
    n_pages = -(-T // page)
    perm = torch.randperm(n_pages + 3, generator=g)[:n_pages]
    cache = torch.zeros(n_pages + 3, 1, page, dk, dtype=DT[dtype])
    for j in range(T):
        cache[perm[j // page], 0, j % page] = rows[j]
    sk = torch.randn(heads, generator=g) + 1.0 if sink else None
    scale = dk ** -0.5
    out = torch.empty(T, heads * dv, dtype=DT[dtype], device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.latent_attention_simt(q.reshape(T, heads * dk).cuda(), out, cache.cuda(), perm.to(torch.int32).view(1, -1).cuda(),
                              torch.arange(T, dtype=torch.int32, device="cuda"),
                              torch.zeros(T, dtype=torch.int32, device="cuda"), heads, dk, dv, window, scale,
                              sk.cuda() if sink else None, err)
    assert int(err.item()) == 0
    want = torch.zeros(T, heads, dv, dtype=torch.float64)
    rd, qd = rows.double(), q.double()
    for t in range(T):
        lo = max(0, t - window + 1) if window else 0
        for h in range(heads):
            s = rd[lo:t + 1] @ qd[t, h] * scale
            top = max(float(s.max()), float(sk[h])) if sink else float(s.max())
            e = torch.exp(s - top)
            den = e.sum() + (math.exp(float(sk[h]) - top) if sink else 0.0)
            want[t, h] = (e / den) @ rd[lo:t + 1, :dv]
    return out.view(T, heads, dv), want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,sink,dk,dv,page", [(0, True, 56, 48, 16), (7, False, 24, 8, 4), (33, False, 144, 128, 8),
                                                     (1, False, 40, 40, 16), (0, False, 300, 260, 16)])
def test_latent_attention_over_paged_rows(dtype, window, sink, dk, dv, page):
    got, want = _latent_case(dtype, 75, 3, dk, dv, page, window, sink)
    assert rel(got, want) <= (3e-6 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("window,sink,dk,dv,page,heads", [(0, True, 56, 48, 16, 3), (7, False, 24, 8, 4, 5), (33, False, 144, 128, 8, 6),
                                                           (1, False, 40, 40, 16, 1), (0, False, 304, 260, 16, 2),
                                                           (40, True, 576, 512, 16, 16), (0, False, 96, 64, 32, 20)])
def test_latent_attention_on_the_tensor_cores(window, sink, dk, dv, page, heads):
    """Three sequences in one launch: a prompt portion that continues a cached prefix, a single decoded
    token, and a whole short prompt; rows on shuffled pages; against the formula in float64."""
    from rllm_b200.kernels import ops
    g = torch.Generator().manual_seed(dk + window)
    lens, news = [83, 41, 19], [50, 1, 19]
    T = sum(news)
    n_pages = sum(-(-n // page) for n in lens)
    perm = torch.randperm(n_pages + 2, generator=g)
    cache = torch.zeros(n_pages + 2, 1, page, dk, dtype=torch.bfloat16)
    width = max(-(-n // page) for n in lens)
    table = torch.full((3, width), -1, dtype=torch.int32)
    rows, used = [], 0
    for s, n in enumerate(lens):
        r = torch.randn(n, dk, generator=g).to(torch.bfloat16)
        rows.append(r)
        for j in range(n):
            if j % page == 0:
                table[s, j // page] = perm[used]
                used += 1
            cache[table[s, j // page], 0, j % page] = r[j]
    q = torch.randn(T, heads, dk, generator=g).to(torch.bfloat16)
    sk = (torch.randn(heads, generator=g) + 1.0) if sink else None
    scale = dk ** -0.5
    out = torch.empty(T, heads * dv, dtype=torch.bfloat16, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    q_start = torch.tensor([0, 50, 51, 70], dtype=torch.int32, device="cuda")
    ops.latent_attention_mma(q.reshape(T, heads * dk).cuda(), out, cache.cuda(), table.cuda(), q_start,
                             torch.tensor(lens, dtype=torch.int32, device="cuda"), 3, max(news), heads, dk, dv, window,
                             scale, sk.cuda() if sink else None, err)
    assert int(err.item()) == 0
    want = torch.zeros(T, heads, dv, dtype=torch.float64)
    off = 0
    for s, (n, m) in enumerate(zip(lens, news)):
        rd = rows[s].double()
        for i in range(m):
            p = n - m + i
            lo = max(0, p - window + 1) if window else 0
            for h in range(heads):
                sc = rd[lo:p + 1] @ q[off + i, h].double() * scale
                top = max(float(sc.max()), float(sk[h])) if sink else float(sc.max())
                e = torch.exp(sc - top)
                den = e.sum() + (math.exp(float(sk[h]) - top) if sink else 0.0)
                want[off + i, h] = (e / den) @ rd[lo:p + 1, :dv]
        off += m
    assert rel(out.view(T, heads, dv), want) <= 2e-2


@pytest.mark.parametrize("window", [5, 16, 17])
def test_a_key_just_inside_and_just_outside_the_window_and_a_far_key(window):
    """Row 3 and the query of the last token are scaled so that row 3's score stands far out.  A query sees
    it exactly while its distance is below the window; the last query, far away, must not (window) or must
    (no window) be taken over by it."""
    T = 70

    def boost(q, rows):
        rows[3] = 0.0
        rows[3, 0] = 60.0
        q[:, :, 0] = 4.0

    got, want = _latent_case("float32", T, 2, 32, 32, 16, window, False, seed=3, boost=boost)
    assert rel(got, want) <= 3e-6
    inside, outside = got[3 + window - 1, 0, 0].item(), got[3 + window, 0, 0].item()
    assert inside > 59.0 and abs(outside) < 10.0
    far, _ = _latent_case("float32", T, 2, 32, 32, 16, 0, False, seed=3, boost=boost)
    assert far[T - 1, 1, 0].item() > 59.0


def test_the_sink_takes_its_share_of_the_softmax():
    """With one visible key the attention weight is exp(s) / (exp(s) + exp(sink)), not 1."""
    got, want = _latent_case("float32", 1, 4, 16, 16, 16, 0, True, seed=5)
    assert rel(got, want) <= 3e-6
    plain, _ = _latent_case("float32", 1, 4, 16, 16, 16, 0, False, seed=5)
    assert float((got.cpu() - plain.cpu()).abs().max()) > 0.05


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latent_rows_are_normalised_rotated_in_pairs_and_written_to_their_pages(dtype):
    from rllm_b200.kernels import ops
    torch.manual_seed(2)
    T, q_rank, kv_rank, rot, rot_dims, page = 9, 24, 40, 12, 8, 4
    a = torch.randn(T, q_rank + kv_rank + rot).to(DT[dtype])
    wq, wkv = (1 + 0.1 * torch.randn(q_rank)).to(DT[dtype]), (1 + 0.1 * torch.randn(kv_rank)).to(DT[dtype])
    pos = torch.tensor([100, 101, 102, 0, 1, 2, 3, 4, 5], dtype=torch.int32)
    seq = torch.tensor([0, 0, 0, 1, 1, 1, 1, 1, 1], dtype=torch.int32)
    table = torch.full((2, 32), -1, dtype=torch.int32)
    table[0, 25] = 3
    table[1, 0], table[1, 1] = 1, 0
    base = 777.0
    inv = torch.tensor([base ** (-2.0 * i / rot_dims) for i in range(rot_dims // 2)], dtype=torch.float64)
    cache = torch.zeros(5, 1, page, kv_rank + rot, dtype=DT[dtype], device="cuda")
    cq = torch.empty(T, q_rank, dtype=DT[dtype], device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.latent_prep(a.cuda(), q_rank, kv_rank, rot, rot_dims, wq.cuda(), wkv.cuda(), 1e-5, cq, cache, table.cuda(),
                    pos.cuda(), seq.cuda(), inv.cuda(), err)
    assert int(err.item()) == 0
    ad = a.double()
    tol = 2e-6 if dtype == "float32" else 1e-2
    assert rel(cq, pf.unit_rms(ad[:, :q_rank], wq.double(), 1e-5)) <= tol
    c = pf.unit_rms(ad[:, q_rank:q_rank + kv_rank], wkv.double(), 1e-5)
    shared = pf.rotate_pairs(ad[:, q_rank + kv_rank:], pos, base, rot_dims)
    assert torch.equal(shared[:, rot_dims:], ad[:, q_rank + kv_rank + rot_dims:])       # beyond rot.dims: unchanged
    for t in range(T):
        pg = int(table[seq[t], pos[t] // page])
        row = cache[pg, 0, int(pos[t]) % page].double().cpu()
        assert float((row - torch.cat([c[t], shared[t]])).abs().max()) <= tol * 4, t


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M", [1, 5, 70])
def test_products_per_head_over_slices(dtype, M):
    from rllm_b200.kernels import ops
    torch.manual_seed(3)
    heads, K, N, extra = 3, 20, 37, 6
    a = torch.randn(M, heads, K + extra).to(DT[dtype]).cuda()
    b_kn = torch.randn(heads, K, N).to(DT[dtype]).cuda()
    c = torch.zeros(M, heads, N + 5, dtype=DT[dtype], device="cuda")
    ops.head_gemm(a[:, :, :K], b_kn, c[:, :, :N], b_kn=True)
    want = torch.einsum("mhk,hkn->mhn", a[:, :, :K].double().cpu(), b_kn.double().cpu())
    assert rel(c[:, :, :N], want) <= (2e-6 if dtype == "float32" else 1e-2)
    assert float(c[:, :, N:].abs().max()) == 0.0
    b_nk = b_kn.transpose(1, 2).contiguous()
    c2 = torch.empty(M, heads, N, dtype=DT[dtype], device="cuda")
    ops.head_gemm(a[:, :, :K], b_nk, c2, b_kn=False)
    assert rel(c2, want) <= (2e-6 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,E,top", [(1, 5, 2), (7, 3, 1), (50, 4, 4), (300, 9, 3)])
def test_routed_experts_choose_weigh_and_compute(dtype, T, E, top):
    from rllm_b200.kernels import ops
    torch.manual_seed(4)
    H, F, limit = 44, 28, 1.25
    x = torch.randn(T, H).to(DT[dtype])
    wr = torch.randn(E, H).to(DT[dtype])
    wgu = (torch.randn(E, 2 * F, H) * 0.3).to(DT[dtype])
    wd = (torch.randn(E, H, F) * 0.3).to(DT[dtype])
    ids, scores = ops.moe_route(x.cuda(), wr.cuda(), top)
    s = torch.softmax(x.double() @ wr.double().t(), dim=-1)
    val, idx = torch.topk(s, top, dim=-1)
    if dtype == "float32":
        assert torch.equal(ids.cpu().long(), idx)
    assert float((scores.double().cpu() - torch.gather(s, 1, ids.cpu().long())).abs().max()) <= 1e-5
    y = ops.moe_experts(x.cuda(), ids, wgu.cuda(), wd.cuda(), limit, 1.702)
    want = torch.zeros(T * top, H, dtype=torch.float64)
    for t in range(T):
        for k in range(top):
            e = int(ids[t, k])
            g = torch.clamp(wgu[e, :F].double() @ x[t].double(), max=limit)
            u = torch.clamp(wgu[e, F:].double() @ x[t].double(), -limit, limit)
            want[t * top + k] = wd[e].double() @ (g * torch.sigmoid(1.702 * g) * (u + 1))
    assert rel(y, want) <= (3e-6 if dtype == "float32" else 2e-2)
    out = torch.empty(T, H, dtype=DT[dtype], device="cuda")
    ops.weighted_slot_sum(y, scores, out)
    comb = (want.view(T, top, H) * scores.double().cpu()[:, :, None]).sum(1)
    assert rel(out, comb) <= (3e-6 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gate_norm_add_and_the_depth_weighted_stream(dtype):
    from rllm_b200.kernels import ops
    torch.manual_seed(5)
    T, H, K, L = 6, 52, 3, 4
    x = torch.randn(T, H)
    y = torch.randn(T * K, H).to(DT[dtype])
    sw = torch.rand(T, K)
    gate = torch.randn(T, H + 8).to(DT[dtype])
    gb, nw, nxt = (torch.randn(H).to(DT[dtype]) for _ in range(3))
    xo = torch.empty(T, H, device="cuda")
    normed = ops.gated_postnorm_add(x.cuda(), xo, y.cuda(), gate.cuda()[:, :H], gb.cuda(), nw.cuda(), 1e-5,
                                    slot_weights=sw.cuda(), next_weight=nxt.cuda(), next_eps=1e-3)
    v = (y.double().view(T, K, H) * sw.double()[:, :, None]).sum(1) * torch.sigmoid(gate.double()[:, :H] + gb.double())
    want = x.double() + pf.unit_rms(v, nw.double(), 1e-5)
    assert rel(xo, want) <= 2e-6
    assert rel(normed, pf.unit_rms(want, nxt.double(), 1e-3)) <= (2e-6 if dtype == "float32" else 1e-2)
    hist = torch.randn(L + 1, T, H).cuda()
    coeff = torch.randn(L).to(DT[dtype])
    stream = torch.empty(T, H, device="cuda")
    n2 = ops.depth_average(hist, L, coeff.cuda(), stream, nw.cuda(), 1e-5, DT[dtype])
    ws = (hist[:L].double().cpu() * coeff.double()[:, None, None]).sum(0)
    assert rel(stream, ws) <= 2e-6
    assert rel(n2, pf.unit_rms(ws, nw.double(), 1e-5)) <= (2e-6 if dtype == "float32" else 1e-2)
    rows = torch.tensor([4, 1], dtype=torch.int32, device="cuda")
    n3 = ops.depth_average(hist, L, coeff.cuda(), None, nw.cuda(), 1e-5, DT[dtype], rows=rows)
    assert torch.equal(n3, n2[[4, 1]])
    # both in one kernel: the layer's result goes to the history's last level, the stream is the weighted sum
    hist2 = hist.clone()
    stream2 = torch.empty(T, H, device="cuda")
    n4 = ops.gated_postnorm_add(x.cuda(), hist2[L - 1], y.cuda(), gate.cuda()[:, :H], gb.cuda(), nw.cuda(), 1e-5,
                                slot_weights=sw.cuda(), next_weight=nxt.cuda(), next_eps=1e-3,
                                depth=(hist2, L, coeff.cuda(), stream2))
    assert rel(hist2[L - 1], want) <= 2e-6
    ws2 = (hist[:L - 1].double().cpu() * coeff.double()[:L - 1, None, None]).sum(0) + coeff.double()[L - 1] * want
    assert rel(stream2, ws2) <= 2e-6
    assert rel(n4, pf.unit_rms(ws2, nxt.double(), 1e-3)) <= (2e-6 if dtype == "float32" else 1e-2)


# ---------------------------------------------------------------------------
# whole models through trace replay
# ---------------------------------------------------------------------------
@pytest.fixture(scope="module")
def fx_dirs(tmp_path_factory):
    return {"A": write_model(str(tmp_path_factory.mktemp("fx_a")), FX_A, 11, sharpen),
            "B": write_model(str(tmp_path_factory.mktemp("fx_b")), FX_B, 12, sharpen),
            "C": write_model(str(tmp_path_factory.mktemp("fx_c")), FX_C, 13, sharpen),
            "D": write_model(str(tmp_path_factory.mktemp("fx_d")), FX_D, 14, sharpen)}


def plain_rows(folder, dtype, reqs):
    cfg, w = pf.read_model_dir(folder, round_to=torch.bfloat16 if dtype == "bfloat16" else None)
    return {r: pf.logits(cfg, w, toks).numpy() for r, toks in reqs.items()}


def compare(got, want, reqs, dtype, what):
    """float32: every position within the tolerance.  bfloat16: rounding can turn a router's close call
    (two experts with nearly equal scores) the other way, which moves that token's logits by more than
    rounding; up to 3 % of the positions may do so, the rest stays within the tolerance."""
    over = total = 0
    for r, toks in reqs.items():
        have = np.stack([got[(r, p)] for p in range(len(toks))])
        err = np.abs(have - want[r]).max(axis=1) / np.abs(want[r]).max()
        assert np.isfinite(have).all()
        if dtype == "float32":
            assert err.max() <= TOL[dtype], (what, r, int(err.argmax()), float(err.max()))
        over += int((err > TOL[dtype]).sum())
        total += len(toks)
    assert over <= 0.03 * total, (what, over, total)


def make_requests(vocab, lengths, seed):
    rng = np.random.default_rng(seed)
    return {f"r{i}": [int(t) for t in rng.integers(0, vocab, size=n)] for i, n in enumerate(lengths)}


def test_the_cuda_core_forms_of_the_bfloat16_kernels_still_serve(fx_dirs, monkeypatch):
    """RLLM_LATENT_ATTENTION=simt and RLLM_TILE_GEMM=simt (read once per process by the library, so set before its
    first call in a child process) keep attention and the tile products off the tensor cores."""
    V = FX_B["vocab"]
    reqs = make_requests(V, [40, 9], seed=21)
    want = plain_rows(fx_dirs["B"], "bfloat16", reqs)
    monkeypatch.setenv("RLLM_LATENT_ATTENTION", "simt")
    monkeypatch.setenv("RLLM_TILE_GEMM", "simt")
    got = ru.run_trace(fx_dirs["B"], "bfloat16", ru.trace_portions(reqs, seed=2), V, page_size=16, subprocess_mode=True)
    compare(got, want, reqs, "bfloat16", "cuda-core forms")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page", [("A", 16), ("A", 4), ("B", 8), ("C", 16), ("D", 16)])
def test_every_way_of_cutting_gives_the_plain_logits(fx_dirs, name, page, dtype):
    """Whole prompts, token by token from the first token on, portions down to two tokens, and mixed
    batches of up to four live requests whose pages and slots are given back and used again (the pool
    holds exactly the peak); every position's logits are compared."""
    cfg = {"A": FX_A, "B": FX_B, "C": FX_C, "D": FX_D}[name]
    V = cfg["vocab"]
    reqs = make_requests(V, [61, 1, 2, 17, 90, 33, 5] + ([150] if name in "CD" else []), seed=7)
    want = plain_rows(fx_dirs[name], dtype, reqs)
    for what, tb in (("whole", ru.trace_whole(reqs)), ("one by one", ru.trace_tail_decode(reqs, tail=1000)),
                     ("tail decoded", ru.trace_tail_decode(reqs, tail=45)),
                     ("portions", ru.trace_portions(reqs, seed=1)), ("portions b", ru.trace_portions(reqs, seed=4)),
                     ("mixed", ru.trace_mixed(reqs, seed=2, live=4, tail=6)),
                     ("mixed b", ru.trace_mixed(reqs, seed=3, live=3, tail=30))):
        got = ru.run_trace(fx_dirs[name], dtype, tb, V, page_size=page)
        compare(got, want, reqs, dtype, f"{name}/{dtype}/page {page}/{what}")


def test_long_decoding_past_every_window_and_many_pages(fx_dirs):
    """A prompt of 3 tokens, then 200 tokens one by one (windows of 9, 20 and 37; pages of 8: the windowed
    groups give pages back on the way), beside a second request that starts later."""
    V = FX_A["vocab"]
    reqs = make_requests(V, [203, 120], seed=9)
    want = plain_rows(fx_dirs["A"], "float32", reqs)
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
    got = ru.run_trace(fx_dirs["A"], "float32", tb, V, page_size=8)
    compare(got, want, reqs, "float32", "long decoding")


def test_the_runner_as_a_program_and_pools_no_larger_than_asked(fx_dirs):
    """bin/trace_run as a child process with a pool of exactly the peak of live tokens."""
    V = FX_B["vocab"]
    reqs = make_requests(V, [40, 70, 9, 64, 3], seed=13)
    want = plain_rows(fx_dirs["B"], "float32", reqs)
    tb = ru.trace_mixed(reqs, seed=5, live=2, tail=4)
    got = ru.run_trace(fx_dirs["B"], "float32", tb, V, page_size=16, subprocess_mode=True)
    compare(got, want, reqs, "float32", "child process")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(fx_dirs, dtype):
    """Nine requests through LLM.generate with the scheduler cutting prompts into portions of at most 16
    tokens beside decoding requests, CUDA graphs for the decode steps, more requests than sequences at a
    time.  float32: the plain implementation's tokens.  bfloat16: its choice at (nearly) all places where that is clear."""
    from rllm_b200 import LLM, SamplingParams
    V = FX_A["vocab"]
    rng = np.random.default_rng(17)
    prompts = [[int(t) for t in rng.integers(0, V, size=int(n))] for n in (5, 41, 1, 23, 60, 2, 9, 30, 14)]
    n_new = 12
    llm = LLM(fx_dirs["A"], dtype="fp32" if dtype == "float32" else "bf16", block_size=8, num_gpu_blocks=96,
              max_num_seqs=4, max_num_batched_tokens=24, long_prefill_token_threshold=16, enable_prefix_caching=False)
    assert llm.engine.runner.capture_graphs
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
    cfg, w = pf.read_model_dir(fx_dirs["A"], round_to=torch.bfloat16 if dtype == "bfloat16" else None)
    clear = wrong = 0
    for p, o in zip(prompts, outs):
        got = o.outputs[0].token_ids
        assert len(got) == n_new
        if dtype == "float32":
            assert got == pf.greedy(cfg, w, p, n_new)
            continue
        seq = list(p)
        for t in got:
            row = pf.logits(cfg, w, seq)[-1]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) > 6e-2 * float(row.abs().max()):
                clear += 1
                wrong += t != int(torch.argmax(row))
            seq.append(t)
    # (a router's close call turned by rounding may move a token's logits by more than rounding)
    assert dtype == "float32" or (clear >= 20 and wrong <= 0.04 * clear), (clear, wrong)
    assert any(g.graph is not None for g in llm.engine.runner.graphs.values())
    llm.engine.cache.check()
    assert llm.engine.cache.usage()["num_requests"] == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions_scan_in_chunks_and_match_the_token_by_token_state(dtype):
    """Two sequences of 300 and 131 tokens (chunks of 64 with ragged ends) beside one of 2 tokens, from a
    non-zero state: outputs and final states against the recurrence written out."""
    from rllm_b200.kernels import ops
    torch.manual_seed(8)
    W, lens, slots = 40, [300, 2, 131], [1, 2, 0]
    T = sum(lens)
    a = (torch.randn(T, 3 * W) * 2).to(DT[dtype])
    bz, bx = torch.randn(W).to(DT[dtype]), torch.randn(W).to(DT[dtype])
    state = torch.rand(4, W)
    want_state = state.double().clone()
    want = torch.zeros(T, W, dtype=torch.float64)
    ad, off = a.double(), 0
    for n, sl in zip(lens, slots):
        s = want_state[sl].clone()
        for t in range(off, off + n):
            z = torch.sigmoid(ad[t, :W] + bz.double())
            u = ad[t, W:2 * W] + bx.double()
            s = (1 - z) * s + z * torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
            g = ad[t, 2 * W:]
            want[t] = s * g * torch.sigmoid(g)
        want_state[sl] = s
        off += n
    out = torch.empty(T, W, dtype=DT[dtype], device="cuda")
    st = state.cuda()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    q_start = torch.tensor([0, 300, 302, T], dtype=torch.int32, device="cuda")
    ops.mingru_scan(a.cuda(), bz.cuda(), bx.cuda(), st, q_start, torch.tensor(slots, dtype=torch.int32, device="cuda"),
                    3, out, err, max_q_len=300)
    assert int(err.item()) == 0
    assert rel(out, want) <= (2e-6 if dtype == "float32" else 1e-2)
    assert rel(st, want_state) <= 2e-6
    assert torch.equal(st[3].cpu(), state[3])


@pytest.mark.parametrize("window,sink,heads,dk,dv", [(0, True, 2, 144, 128), (300, False, 6, 56, 48), (0, False, 16, 576, 512)])
def test_decoding_over_long_rows_cuts_the_keys_into_splits(window, sink, heads, dk, dv):
    """Two sequences of 1500 and 700 cached rows, one new token each: few rows, many keys, so the keys are cut
    into splits of 256 whose partial sums a second kernel adds (with the sink)."""
    from rllm_b200.kernels import ops
    g = torch.Generator().manual_seed(dk)
    page, lens = 16, [1500, 700]
    n_pages = sum(-(-n // page) for n in lens)
    cache = torch.zeros(n_pages + 1, 1, page, dk, dtype=torch.bfloat16)
    table = torch.full((2, -(-max(lens) // page)), -1, dtype=torch.int32)
    perm = torch.randperm(n_pages + 1, generator=g)
    rows, used = [], 0
    for s, n in enumerate(lens):
        r = torch.randn(n, dk, generator=g).to(torch.bfloat16)
        rows.append(r)
        for b in range(-(-n // page)):
            table[s, b] = perm[used]
            cache[perm[used], 0, : min(page, n - b * page)] = r[b * page:(b + 1) * page]
            used += 1
    q = torch.randn(2, heads, dk, generator=g).to(torch.bfloat16)
    sk = (torch.randn(heads, generator=g) + 1.0) if sink else None
    scale = dk ** -0.5
    out = torch.empty(2, heads * dv, dtype=torch.bfloat16, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.latent_attention_mma(q.reshape(2, heads * dk).cuda(), out, cache.cuda(), table.cuda(),
                             torch.tensor([0, 1, 2], dtype=torch.int32, device="cuda"),
                             torch.tensor(lens, dtype=torch.int32, device="cuda"), 2, 1, heads, dk, dv, window, scale,
                             sk.cuda() if sink else None, err, max_seq_len=1504)
    assert int(err.item()) == 0
    want = torch.zeros(2, heads, dv, dtype=torch.float64)
    for s, n in enumerate(lens):
        rd = rows[s].double()
        lo = max(0, n - window) if window else 0
        for h in range(heads):
            sc = rd[lo:n] @ q[s, h].double() * scale
            top = max(float(sc.max()), float(sk[h])) if sink else float(sc.max())
            e = torch.exp(sc - top)
            den = e.sum() + (math.exp(float(sk[h]) - top) if sink else 0.0)
            want[s, h] = (e / den) @ rd[lo:n, :dv]
    assert rel(out.view(2, heads, dv), want) <= 2e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_forked_request_shares_full_pages_and_copies_the_last_page_and_the_state(fx_dirs, dtype):
    """A parent feeds 21 tokens (pages of 8: two full pages and a partly filled one in every paged group, a
    state slot per recurrence), a child is forked from it and both go on with different tokens, in portions and
    token by token: the child's one-row pages and state slot start as copies, and neither disturbs the other."""
    V = FX_A["vocab"]
    rng = np.random.default_rng(31)
    common, tail_p, tail_c = ([int(t) for t in rng.integers(0, V, size=n)] for n in (21, 30, 30))
    tb = ru.TraceBuilder()
    tb.step([("p", common)])
    tb.step([("p", tail_p[:1]), ("c", tail_c[:7])], fork=[("p", "c")])
    for i in range(1, 20):
        tb.step([("p", tail_p[i:i + 1]), ("c", tail_c[6 + i:7 + i])])
    tb.step([("p", tail_p[20:]), ("c", tail_c[26:])], end=["p", "c"])
    got = ru.run_trace(fx_dirs["A"], dtype, tb, V, page_size=8)
    reqs = {"p": common + tail_p, "c": common + tail_c}
    want = plain_rows(fx_dirs["A"], dtype, reqs)
    assert max(pos for r, pos in got if r == "c") == len(reqs["c"]) - 1
    over = 0
    for (r, pos), row in got.items():
        err = np.abs(row - want[r][pos]).max() / np.abs(want[r]).max()
        assert dtype == "bfloat16" or err <= TOL[dtype], (r, pos, float(err))
        over += err > TOL[dtype]
    assert over <= 0.03 * len(got)
