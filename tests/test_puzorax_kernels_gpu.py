"""Every kernel that the Puzorax decoder added, alone, against the plain implementation's function of the same
mechanism (float64), at sizes of the tests' own: the delta rule with a decay per key channel (token by token and
in long steps, any cut, batches, slots used again, shared q/k heads, wide keys), attention over the compressed
cache (any cut, pages in no order, windows, sinks, a partly rotated part; a loud key far away, just inside and just
outside a window, in prompts and in decoding), the softmax router with its correction, factor and identity
experts, the bigram embedding with its kept token, the layer norm's bias and the restart of the stream."""
import pytest
import torch

import plain_puzorax as P

pytestmark = pytest.mark.gpu
F64 = torch.float64
DEV = "cuda:0"


def K():
    from mivi_v4_b200.ops import kernels
    return kernels


def dev(x, dtype=torch.float32):
    return x.to(dtype).to(DEV).contiguous()


def i32(xs):
    return torch.tensor(xs, dtype=torch.int32, device=DEV)


def close(got, want, tol=2e-5, what=""):
    got, want = got.detach().double().cpu(), want.double()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert torch.isfinite(got).all(), what
    err = (got - want).abs().max().item() / max(want.abs().max().item(), 1e-30)
    assert err <= tol, f"{what}: off by {err:.3g} of the largest value (limit {tol})"


def cuts_of(T):
    return [[T], [1] * T, [2] * (T // 2) + ([T % 2] if T % 2 else []), [5, 1, T - 6], [T - 1, 1], [9, 17, T - 26]]


class _Ws:
    """A workspace for the kernels that want scratch: buffers by name."""
    def __init__(self):
        self.bufs = {}

    def get(self, name, shape, dtype):
        key = (name, tuple(shape), dtype)
        if key not in self.bufs:
            self.bufs[key] = torch.empty(shape, dtype=dtype, device=DEV)
        return self.bufs[key]


# ------------------------------------------------------------------------------------------ delta rule
def _delta_case(T, H, KV, dk, dv, seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g, dtype=F64)   # noqa: E731
    q, k, v = r(T, KV * dk), r(T, KV * dk), r(T, H * dv)
    beta, a = r(T, H), r(T, H * dk)
    dt_bias, a_log = -1.0 + r(H * dk), torch.log(0.02 + 0.98 * torch.rand(H, generator=g, dtype=F64))
    qn = q.view(T, KV, dk) / torch.sqrt((q.view(T, KV, dk) ** 2).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    kn = k.view(T, KV, dk) / torch.sqrt((k.view(T, KV, dk) ** 2).sum(-1, keepdim=True) + 1e-6)
    rep = H // KV
    dec = torch.exp(-torch.exp(a_log)[None, :, None] * torch.nn.functional.softplus(a + dt_bias).view(T, H, dk))
    want = P.delta_rule(qn.repeat_interleave(rep, 1), kn.repeat_interleave(rep, 1), v.view(T, H, dv), torch.sigmoid(beta), dec)
    return (q, k, v, beta, a, dt_bias, a_log), want.reshape(T, H * dv)


def _run_delta(k, case, cuts, H, KV, dk, dv, state, slot, ws):
    q, kk, v, beta, a, dt_bias, a_log = [dev(x) for x in case]
    outs, at = [], 0
    for n in cuts:
        rows = slice(at, at + n)
        o = torch.full((n, H * dv), float("nan"), device=DEV)
        k.delta_scan(q[rows], kk[rows], v[rows], beta[rows], a[rows], dt_bias, a_log, state, i32([slot]), i32([0, n]), o,
                     1, H, KV, dk, dv, q_scale=dk ** -0.5, max_len=n, ws=ws)
        outs.append(o)
        at += n
    return torch.cat(outs)


@pytest.mark.parametrize("H,KV,dk,dv", [(4, 2, 16, 8), (1, 1, 20, 12), (2, 1, 72, 40), (1, 1, 136, 17), (3, 3, 5, 33),
                                        (2, 1, 64, 32), (2, 2, 128, 18), (1, 1, 256, 16), (2, 1, 48, 16)])
def test_delta_rule_under_every_cut_token_by_token_and_in_long_steps(H, KV, dk, dv):
    k, T = K(), 61
    case, want = _delta_case(T, H, KV, dk, dv, seed=dk)
    for ws in (None, _Ws()):                              # without scratch every step runs the token-by-token kernel
        for cuts in cuts_of(T):
            state = torch.zeros(3, H, dv, dk, device=DEV)
            got = _run_delta(k, case, cuts, H, KV, dk, dv, state, 1, ws)
            close(got, want, 3e-5, f"cuts {cuts[:4]} scratch {ws is not None}")
            assert state[0].abs().max() == 0 and state[2].abs().max() == 0          # the other slots are untouched


def test_delta_rule_batches_and_slots_used_again():
    k = K()
    H, KV, dk, dv = 4, 2, 24, 16
    lens = [37, 1, 18, 9]
    cases = [_delta_case(n, H, KV, dk, dv, seed=100 + n) for n in lens]
    state = torch.full((6, H, dv, dk), 7.0, device=DEV)            # what an earlier sequence left behind
    slots = [4, 0, 5, 2]
    state[slots] = 0.0                                            # the cache zeroes a slot when it assigns it
    packed = [dev(torch.cat([c[0][i] for c in cases])) for i in range(5)]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    for ws in (None, _Ws()):
        st = state.clone()
        o = torch.full((sum(lens), H * dv), float("nan"), device=DEV)
        k.delta_scan(*packed, dev(cases[0][0][5]), dev(cases[0][0][6]), st, i32(slots), i32(cu), o, len(lens), H, KV, dk, dv,
                     q_scale=dk ** -0.5, max_len=max(lens), ws=ws)
        for i, (c, want) in enumerate(cases):
            # every request with the first one's dt_bias and A_log: the wanted rows are made again with them
            case_i = c[:5] + cases[0][0][5:]
            qn = case_i[0].view(-1, KV, dk) / torch.sqrt((case_i[0].view(-1, KV, dk) ** 2).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
            kn = case_i[1].view(-1, KV, dk) / torch.sqrt((case_i[1].view(-1, KV, dk) ** 2).sum(-1, keepdim=True) + 1e-6)
            dec = torch.exp(-torch.exp(case_i[6])[None, :, None]
                            * torch.nn.functional.softplus(case_i[4] + case_i[5]).view(-1, H, dk))
            want = P.delta_rule(qn.repeat_interleave(H // KV, 1), kn.repeat_interleave(H // KV, 1), case_i[2].view(-1, H, dv),
                                torch.sigmoid(case_i[3]), dec).reshape(-1, H * dv)
            close(o[cu[i]:cu[i + 1]], want, 3e-5, f"request {i} scratch {ws is not None}")
        assert (st[[1, 3]] == 7.0).all()


# ------------------------------------------------------------------------------------------ latent attention
def _latent_case(T, H, dim, rd, vd, rank, window, rot_dims, base, scale, seed, loud=None):
    """A latent attention layer whose input is its own projections (W_q, W_dkv and W_g pick columns of the input)
    and whose W_o is the identity: the wanted rows are the gated heads."""
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g, dtype=F64)   # noqa: E731
    nq, nc, ng = H * (dim + rd), rank + rd, H * vd
    W = nq + nc + ng
    h = r(T, W)
    if loud is not None and rd >= 4:
        qi, kj = loud
        half = rot_dims // 2
        vec = torch.full((rd,), 2.0, dtype=F64)
        vec[0] = vec[half] = 0.0                           # the fastest pair turns too quickly to point anywhere
        h[kj, nq + rank:nq + nc] = vec
        for a in range(H):
            h[qi, a * (dim + rd) + dim:(a + 1) * (dim + rd)] = vec
    eye = torch.eye(W, dtype=F64)
    p = {"q": eye[:nq], "dkv": eye[nq:nq + nc], "g": eye[nq + nc:], "dkv.norm": 1.0 + 0.2 * r(rank), "uk": r(H * dim, rank) / rank ** 0.5,
         "uv": r(H * vd, rank) / rank ** 0.5, "sink": r(H), "o": torch.eye(ng, dtype=F64)}
    m = {"heads": H, "dim": dim, "rot_dim": rd, "vdim": vd, "kv_rank": rank, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if rd:
        m["rot"] = {"dims": rot_dims, "base": base}
    return h, p, m, P.latent_attention(h, p, m, 1e-5)


def _run_latent(k, dtype, h, p, m, cuts, page_size, sink=True, splits=1):
    from mivi_v4_b200.parts.position import Rope
    T = h.shape[0]
    H, dim, rd, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    window, rot = (m.get("mask") or {}).get("size", 0), m.get("rot") or {"dims": 0}
    n_pages = -(-T // page_size)
    perm = torch.randperm(n_pages + 3, generator=torch.Generator().manual_seed(3))[:n_pages].tolist()     # pages in no order
    pool = torch.zeros(n_pages + 3, page_size * (rank + rd), dtype=dtype, device=DEV)
    table = i32([perm + [0] * 2])
    inv = Rope(rot["dims"], rot["base"], "half_split").rotary(DEV)[0] if rot["dims"] else None
    proj = dev(h)
    c0, g0 = H * (dim + rd), H * (dim + rd) + rank + rd
    outs, at = [], 0
    for n in cuts:
        rows = slice(at, at + n)
        pos, seq_of = i32(list(range(at, at + n))), i32([0] * n)
        qa = torch.full((n, H, rank + rd), float("nan"), device=DEV)
        k.latent_prepare(proj[rows], 0, c0, dev(p["dkv.norm"]), 1e-5, inv, pos, seq_of, table, pool, page_size, qa, H, dim, rd,
                         rank, rot["dims"])
        k.head_product(proj[rows][:, :c0].unflatten(1, (H, dim + rd)), dev(p["uk"], dtype), qa, H, dim, rank, transposed=True)
        o_lat = torch.full((n, H, rank), float("nan"), device=DEV)
        part = (torch.full((n, H, splits, rank), float("nan"), device=DEV), torch.full((n, H, splits, 2), float("nan"), device=DEV))
        k.latent_attention(qa, pool, page_size, table, pos, seq_of, o_lat, H, rank, rd, m["scale"], window=window,
                           sinks=dev(p["sink"]) if sink else None, splits=splits, part=part if splits > 1 else None)
        y = torch.full((n, H * vd), float("nan"), dtype=dtype, device=DEV)
        k.head_product(o_lat, dev(p["uv"], dtype), y.view(n, H, vd), H, rank, vd, gate=proj[rows][:, g0:g0 + H * vd])
        outs.append(y)
        at += n
    return torch.cat(outs)


LATENT_SIZES = [(10, 8, 12, 6, 24, 10, 8, 100.0, 8), (1, 20, 0, 20, 36, 0, 0, 1.0, 16), (3, 4, 6, 10, 40, 70, 6, 1e4, 8),
                (4, 32, 16, 40, 72, 64, 16, 500.0, 64), (2, 64, 32, 32, 64, 150, 32, 5e4, 16), (9, 16, 8, 16, 130, 33, 4, 50.0, 32)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dim,rd,vd,rank,window,rot_dims,base,page", LATENT_SIZES)
def test_latent_attention_under_every_cut(dtype, H, dim, rd, vd, rank, window, rot_dims, base, page):
    k, T = K(), 170
    h, p, m, want = _latent_case(T, H, dim, rd, vd, rank, window, rot_dims, base, 0.3, seed=rank)
    tol = 3e-5 if dtype == torch.float32 else 2e-2
    for cuts in ([T], [1] * T, [100] + [1] * 70, [7] * 24 + [2], [63, 65, 42]):
        close(_run_latent(k, dtype, h, p, m, cuts, page), want, tol, f"cuts {cuts[:3]}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_loud_key_far_away_and_just_inside_and_just_outside_a_window(dtype):
    """Query 139 and a key made to stand out (through the rotated part, which no norm levels): with a window of 40
    key 100 is the last one seen and key 99 the first one not; without a window the far key 0 is seen."""
    k = K()
    H, dim, rd, vd, rank, T = 2, 8, 16, 8, 16, 140
    tol = 3e-5 if dtype == torch.float32 else 2e-2
    for window, key, seen in ((40, 100, True), (40, 99, False), (40, 0, False), (0, 0, True), (140, 0, True), (139, 0, False),
                              (64, 76, True), (64, 75, False), (1, 139, True), (1, 138, False)):
        h, p, m, want = _latent_case(T, H, dim, rd, vd, rank, window, 16, 1e6, 0.5, seed=key + window, loud=(139, key))
        for cuts in ([T], [120] + [1] * 20, [139, 1]):
            close(_run_latent(k, dtype, h, p, m, cuts, 16), want, tol, f"window {window} loud key {key} cuts {cuts[:2]}")
        # the loud key decides the row where it is seen: the test would notice a mask that is one off
        c = P.rms_norm(h[key:key + 1, H * (dim + rd):H * (dim + rd) + rank], p["dkv.norm"], 1e-5)
        v_key = (c @ p["uv"].T)[0] * torch.sigmoid(h[139, H * (dim + rd) + rank + rd:])
        near = (want[139] - v_key).abs().max() < 0.05 * v_key.abs().max()
        assert bool(near) == seen, (window, key)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("splits", [2, 3, 7])
def test_keys_in_shares_give_the_same_attention(dtype, splits):
    """Shares that end inside a window, shares with no key at all (more shares than blocks of keys) and the sink
    counted once."""
    k = K()
    tol = 3e-5 if dtype == torch.float32 else 2e-2
    for T, window in ((170, 0), (170, 70), (40, 0), (3, 0)):
        h, p, m, want = _latent_case(T, 3, 8, 8, 8, 24, window, 8, 1e4, 0.4, seed=T + window)
        for cuts in ([T], [T - 2, 1, 1]):
            close(_run_latent(k, dtype, h, p, m, cuts, 16, splits=splits), want, tol, f"{splits} shares, window {window}")
        close(_run_latent(k, dtype, h, p, dict(m), [T], 16, sink=False, splits=splits),
              P.latent_attention(h, dict(p, sink=torch.full((3,), -800.0, dtype=F64)), m, 1e-5), tol, "no sink")


def test_number_of_shares_follows_the_work():
    k = K()
    assert k.latent_splits(2048, 32, 4096, 148) == 1                 # many tokens fill the device by themselves
    assert k.latent_splits(8, 32, 100, 148) == 1                     # nothing to cut
    assert 2 <= k.latent_splits(8, 32, 4096, 148) <= k.LATENT_MAX_SPLITS
    assert k.latent_splits(1, 8, 1 << 20, 148) == k.LATENT_MAX_SPLITS


def _run_latent_long(k, h_seqs, p, m, steps, page_size):
    """The tensor-core path for steps of many tokens, bfloat16.  ``h_seqs``: one [T_b, W] input per sequence;
    ``steps``: lists of how many tokens each sequence brings in that step."""
    from mivi_v4_b200.parts.position import Rope
    bf = torch.bfloat16
    B = len(h_seqs)
    H, dim, rd, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    window, rot = (m.get("mask") or {}).get("size", 0), m.get("rot") or {"dims": 0}
    per = [-(-x.shape[0] // page_size) for x in h_seqs]
    n_pages = sum(per)
    perm = torch.randperm(n_pages + 3, generator=torch.Generator().manual_seed(5))[:n_pages].tolist()
    pool = torch.zeros(n_pages + 3, page_size * (rank + rd), dtype=bf, device=DEV)
    rows_t, at = [], 0
    for n in per:
        rows_t.append(perm[at:at + n] + [0] * (max(per) - n))
        at += n
    table = i32(rows_t)
    inv = Rope(rot["dims"], rot["base"], "half_split").rotary(DEV)[0] if rot["dims"] else None
    c0, g0 = H * (dim + rd), H * (dim + rd) + rank + rd
    w_kv = torch.cat([dev(p["uk"], bf), dev(p["uv"], bf)])
    done = [0] * B
    outs = [[] for _ in range(B)]
    for lens in steps:
        N = sum(lens)
        proj = torch.cat([dev(h_seqs[b][done[b]:done[b] + lens[b]]) for b in range(B)])
        pos = i32([done[b] + i for b in range(B) for i in range(lens[b])])
        seq_of = i32([b for b in range(B) for _ in range(lens[b])])
        cu = i32([sum(lens[:b]) for b in range(B + 1)])
        starts = i32(done)
        k.latent_prepare(proj, 0, c0, dev(p["dkv.norm"]), 1e-5, inv, pos, seq_of, table, pool, page_size, None, H, dim, rd,
                         rank, rot["dims"])
        q = torch.full((N, H, dim + rd), float("nan"), dtype=bf, device=DEV)
        k.latent_query(proj, 0, inv, pos, q, H, dim, rd, rot["dims"])
        rows = sum(done[b] + lens[b] - (max(0, done[b] - window + 1) if window else 0) for b in range(B))
        c = torch.full((rows, rank), float("nan"), dtype=bf, device=DEV)
        r = torch.full((rows, rd), float("nan"), dtype=bf, device=DEV)
        k.latent_gather(pool, page_size, table, cu, starts, B, window, c, r)
        kx = (c.float() @ w_kv.float().T).to(bf)
        y = torch.full((N, H * vd), float("nan"), dtype=bf, device=DEV)
        k.latent_attention_prefill(q, kx, H * dim, r, cu, starts, B, y, H, dim, rd, vd, m["scale"], window=window,
                                   sinks=dev(p["sink"]), gate=proj[:, g0:g0 + H * vd])
        at = 0
        for b in range(B):
            outs[b].append(y[at:at + lens[b]])
            at += lens[b]
            done[b] += lens[b]
    return [torch.cat(o) for o in outs]


LONG_SIZES = [(4, 32, 16, 48, 72, 64, 16, 500.0, 64), (2, 64, 32, 32, 64, 150, 32, 5e4, 16), (3, 8, 8, 16, 24, 33, 4, 50.0, 32),
              (1, 128, 64, 128, 40, 0, 64, 1e6, 16), (5, 16, 0, 64, 16, 0, 0, 1.0, 8), (2, 24, 8, 80, 8, 1, 8, 10.0, 16)]


@pytest.mark.parametrize("H,dim,rd,vd,rank,window,rot_dims,base,page", LONG_SIZES)
def test_long_steps_on_the_tensor_cores_under_every_cut(H, dim, rd, vd, rank, window, rot_dims, base, page):
    k, T = K(), 200
    h, p, m, want = _latent_case(T, H, dim, rd, vd, rank, window, rot_dims, base, 0.3, seed=rank + H)
    for cuts in ([T], [64, 64, 72], [100, 1, 99], [63, 65, 2, 70], [129, 71]):
        got = _run_latent_long(k, [h], p, m, [[n] for n in cuts], page)[0]
        close(got, want, 2e-2, f"cuts {cuts}")


def test_long_steps_of_unequal_sequences_and_a_loud_key_at_the_window_edge():
    """Three sequences of different lengths in the same steps, each against itself alone; then the loud key just
    inside and just outside the window of the last query, in a whole prompt and in a prompt's second portion."""
    k = K()
    H, dim, rd, vd, rank = 2, 16, 16, 16, 16
    cases = [_latent_case(T, H, dim, rd, vd, rank, 50, 16, 1e6, 0.4, seed=11) for T in (150, 31, 97)]
    p, m = cases[0][1], cases[0][2]
    got = _run_latent_long(k, [c[0] for c in cases], p, m, [[70, 31, 20], [80, 0, 77]], 16)
    for b, c in enumerate(cases):                     # every case drew weights of its own: the first one's serve all
        close(got[b], P.latent_attention(c[0], p, m, 1e-5), 2e-2, f"sequence {b} of three")
    T = 140
    for window, key, seen in ((40, 100, True), (40, 99, False), (0, 0, True), (140, 0, True), (139, 0, False), (64, 76, True),
                              (64, 75, False)):
        h, p, m, want = _latent_case(T, H, dim, rd, vd, rank, window, 16, 1e6, 0.5, seed=key + window, loud=(139, key))
        for cuts in ([T], [90, 50], [120, 20]):
            got = _run_latent_long(k, [h], p, m, [[n] for n in cuts], 16)[0]
            close(got, want, 2e-2, f"window {window} loud key {key} cuts {cuts}")
        c = P.rms_norm(h[key:key + 1, H * (dim + rd):H * (dim + rd) + rank], p["dkv.norm"], 1e-5)
        v_key = (c @ p["uv"].T)[0] * torch.sigmoid(h[139, H * (dim + rd) + rank + rd:])
        assert bool((want[139] - v_key).abs().max() < 0.05 * v_key.abs().max()) == seen, (window, key)


def test_a_sink_takes_its_share_and_no_sink_is_plain_softmax():
    k = K()
    h, p, m, want = _latent_case(50, 3, 8, 4, 8, 24, 0, 4, 100.0, 0.4, seed=9)
    close(_run_latent(k, torch.float32, h, p, m, [50], 16), want, 3e-5, "with sinks")
    p0 = dict(p, sink=torch.full((3,), -800.0, dtype=F64))
    want0 = P.latent_attention(h, p0, m, 1e-5)
    assert (want0 - want).abs().max() > 1e-2 * want.abs().max()
    close(_run_latent(k, torch.float32, h, p, m, [20, 30], 16, sink=False), want0, 3e-5, "without sinks")


# ------------------------------------------------------------------------------------------ router and experts
@pytest.mark.parametrize("E,I,top,scale", [(6, 1, 2, 1.5), (5, 3, 3, 0.7), (5, 0, 1, 1.0), (3, 1, 4, 1.0), (40, 2, 6, 2.5)])
def test_softmax_router_correction_factor_and_identity_experts(E, I, top, scale):
    k = K()
    N, R, H = 57, E + I, 24
    g = torch.Generator().manual_seed(E * 10 + I)
    z = 2.0 * torch.randn(N, R, generator=g, dtype=F64).float().double()
    corr = 0.3 * torch.randn(R, generator=g, dtype=F64).float().double()
    want = P.route(z, corr, top, scale)
    dense = torch.full((N, R), float("nan"), device=DEV)
    pick = torch.zeros(N, top, dtype=torch.int32, device=DEV)
    pick_w = torch.zeros(N, top, device=DEV)
    k.route(dev(z), dense, pick, pick_w, R, 1, 1, top, False, mode=k.ROUTE_SOFTMAX, correction=dev(corr), out_scale=scale,
            n_identity=I)
    close(dense, want, 1e-5, "dense weights")
    rows = torch.arange(N)[:, None].expand(N, top)
    close(pick_w, want[rows, pick.cpu().long()], 1e-5, "picked weights")
    assert (torch.sort(pick.cpu().long(), -1).values == torch.sort(torch.topk(torch.softmax(z, -1) + corr, top, -1).indices, -1).values).all()
    if I:
        x = torch.randn(N, H, generator=g, dtype=F64)
        resid = torch.randn(N, H, generator=g, dtype=F64)
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
            out = dev(resid)
            k.identity_experts(dev(x, dtype), dense, E, I, out)
            close(out, resid + want[:, E:].sum(-1, keepdim=True) * x.to(dtype).double(), tol, "identity experts")


# ------------------------------------------------------------------------------------------ small kernels
def test_bigram_embedding_keeps_the_previous_token_between_steps():
    k = K()
    V, H, buckets, mp, mc = 50, 24, 13, 5, 3
    g = torch.Generator().manual_seed(2)
    table, bigram = torch.randn(V, H, generator=g, dtype=F64), torch.randn(buckets + 1, H, generator=g, dtype=F64)
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in (9, 1, 14)]
    cfg = {"embedding": {"bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}}
    want = [P.embedding(s, table, bigram, cfg) for s in seqs]
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
        prev = torch.full((5,), 49, dtype=torch.int32, device=DEV)               # an earlier sequence's last token
        slots = [3, 0, 4]
        got = [[] for _ in seqs]
        # three steps: the first tokens of all, then one token each, then the rest of those that have one
        for lo, hi in ((0, 4), (4, 5), (5, 99)):
            part = [(i, s[lo:hi], lo) for i, s in enumerate(seqs) if s[lo:hi]]
            toks = [t for _, ts, _ in part for t in ts]
            pos = [lo + j for _, ts, _ in part for j in range(len(ts))]
            seq_of = [b for b, (_, ts, _) in enumerate(part) for _ in ts]
            cu = [0]
            for _, ts, _ in part:
                cu.append(cu[-1] + len(ts))
            out = torch.full((len(toks), H), float("nan"), device=DEV)
            kept = torch.full((len(toks), H), float("nan"), device=DEV)
            k.embed_bigram(dev(table, dtype), dev(bigram, dtype), i32(toks), i32(pos), i32(seq_of), i32(cu),
                           i32([slots[i] for i, _, _ in part]), prev, out, kept, mp, mc)
            assert torch.equal(out, kept)
            for b, (i, ts, _) in enumerate(part):
                got[i].append(out[cu[b]:cu[b + 1]])
        for i, s in enumerate(seqs):
            ref = want[i] if dtype == torch.float32 else \
                P.embedding(s, table.to(dtype).double(), bigram.to(dtype).double(), cfg)
            close(torch.cat(got[i]), ref, tol, f"sequence {i} {dtype}")
        assert prev.tolist() == [seqs[1][-1], 49, 49, seqs[0][-1], seqs[2][-1]]


def test_layer_norm_with_bias_and_the_restart_of_the_stream():
    k = K()
    g = torch.Generator().manual_seed(4)
    x, w, b = 3.0 * torch.randn(11, 40, generator=g, dtype=F64) + 1.0, torch.randn(40, generator=g, dtype=F64), torch.randn(40, generator=g, dtype=F64)
    out = torch.empty(11, 40, device=DEV)
    k.layernorm(dev(x), dev(w), 1e-3, out, bias=dev(b))
    close(out, P.layer_norm(x, w, b, 1e-3), 1e-5, "layer norm with bias")
    rows = i32([7, 0, 3])
    out = torch.empty(3, 40, device=DEV)
    k.layernorm(dev(x), dev(w), 1e-3, out, rows, bias=dev(b))
    close(out, P.layer_norm(x[[7, 0, 3]], w, b, 1e-3), 1e-5, "chosen rows")
    y = dev(x)
    k.add_rows_vector(y, dev(2 * x), dev(b))
    close(y, 3 * x + b, 1e-6, "rows and vector")
    y = dev(x)
    k.add_rows_vector(y, None, dev(b))
    close(y, x + b, 1e-6, "vector alone")
