"""Every kernel that the Ropelix decoder added or widened, alone, against the plain implementation's function of
the same mechanism (float64), at sizes of the tests' own: softmax weights mixed between the heads (token by token
and on the tensor cores; a loud key far away, just inside and just outside a window, in prompts and in decoding;
pages in no order), attention whose values are its keys with a distance bias, a sink of score 0 and a gate per
element, the causal convolution without an activation, the gates and the walk of the gated linear recurrence (any
cut, batches, slots used again, long steps in pieces), the delta rule with one decay a head, the joining kernel
of the scaled pre-norm block, and the norm whose weight is stored around zero."""
import math

import pytest
import torch

import plain_ropelix as P

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


def tol_of(dtype):
    return 2e-5 if dtype == torch.float32 else 1.2e-2


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


def _r(seed):
    g = torch.Generator().manual_seed(seed)
    return lambda *s: torch.randn(*s, generator=g, dtype=F64)


# ------------------------------------------------------------------------------------------ the cache of a test
def _fill_cache(k, v, page_size, dtype, pages_order, n_pages):
    """Keys [T, nkv, dk] and values [T, nkv, dv] (None: the values are the keys, a page holds key rows only) of one
    sequence into a flat pool, its pages in the given order."""
    T, nkv, dk = k.shape
    dv = 0 if v is None else v.shape[-1]
    n_blocks = -(-T // page_size)
    pool = torch.zeros((n_pages, nkv * page_size * (dk + dv)), dtype=dtype, device=DEV)
    for blk in range(n_blocks):
        lo, hi = blk * page_size, min(T, (blk + 1) * page_size)
        kp = torch.zeros(nkv, page_size, dk, dtype=dtype, device=DEV)
        kp[:, :hi - lo] = k[lo:hi].permute(1, 0, 2).to(dtype)
        parts = [kp.reshape(-1)]
        if v is not None:
            vp = torch.zeros(nkv, page_size, dv, dtype=dtype, device=DEV)
            vp[:, :hi - lo] = v[lo:hi].permute(1, 0, 2).to(dtype)
            parts.append(vp.reshape(-1))
        pool[pages_order[blk]] = torch.cat(parts)
    return pool, pages_order[:n_blocks]


def _loud_keys(q, k, positions, window, every=1):
    """For every ``every``-th query one key is made to stand out for one of its heads: in turn the key just inside the
    window's far edge, the one just outside it, and one far back (or, without a window, far back and the first)."""
    nh = q.shape[1]
    G = k.shape[1]
    for n in range(0, len(positions), every):
        pos, h = positions[n], n % nh
        choices = [pos - window + 1, pos - window, pos - 3 * window - 5] if window else [pos // 3, 0, pos - 1]
        j = choices[(n // every) % 3]
        if 0 <= j <= pos:
            k[j, h // (nh // G)] = k[j, h // (nh // G)] * 0.2 + 3.0 * q[n, h] / q[n, h].norm()


# ------------------------------------------------------------------------------------------ mixed heads
MIXED = [(4, 2, 16, 8, 9, 20.0), (3, 1, 20, 20, 0, 0.0), (2, 2, 40, 72, 64, 5.0), (6, 3, 8, 136, 130, 0.0), (1, 1, 24, 12, 70, 0.0),
         (8, 8, 16, 16, 1, 3.0)]


def _mixed_want(q, k, v, talk, scale, positions, window, cap, dtype):
    qq, kq, vq = q.to(dtype).double(), k.to(dtype).double(), v.to(dtype).double()
    w = P.mix_heads(P.attention_weights(qq, kq, scale, positions, window=window, cap=cap), talk)
    return P.apply_weights(w, vq)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,dk,dv,window,cap", MIXED)
def test_mixed_heads_token_by_token_window_edges_and_far_keys(nh, nkv, dk, dv, window, cap, dtype):
    k_ = K()
    r = _r(nh * dk + dv)
    T, ps = 300, 64
    k, v = r(T, nkv, dk), r(T, nkv, dv)
    positions = [0, 1, 2, window, window + 1, 63, 64, 65, 128, 129, 200, 250, T - 2, T - 1]
    q = r(len(positions), nh, dk)
    _loud_keys(q, k, positions, window)
    talk = torch.eye(nh, dtype=F64) + 0.5 * r(nh, nh)
    scale = 1.3 / math.sqrt(dk)
    want = _mixed_want(q, k, v, talk, scale, positions, window, cap, dtype)
    pool, pages = _fill_cache(k, v, ps, dtype, [4, 0, 3, 1, 2], 6)
    N = len(positions)
    o_all = torch.full((N, nh, nkv, dv), float("nan"), device=DEV)
    out = torch.full((N, nh * dv), float("nan"), dtype=dtype, device=DEV)
    for tile in (0, 1, 2, 4):
        o_all.fill_(float("nan"))
        k_.attention_sink(dev(q.reshape(N, -1), dtype), pool, ps, i32([pages]), i32(positions), i32([0] * N), out, nh, nkv, dk, dv,
                          scale, softcap=cap, window=window, out_all=o_all, head_tile=tile)
        k_.mix_heads(o_all, dev(talk), out, nh, nkv, dv)
        close(out, want, tol_of(dtype), f"head tile {tile}")
    # the identity leaves plain grouped attention
    k_.mix_heads(o_all, dev(torch.eye(nh, dtype=F64)), out, nh, nkv, dv)
    plain = torch.full_like(out, float("nan"))
    k_.attention_sink(dev(q.reshape(N, -1), dtype), pool, ps, i32([pages]), i32(positions), i32([0] * N), plain, nh, nkv, dk, dv,
                      scale, softcap=cap, window=window)
    close(out, plain.double().cpu(), 1e-2 if dtype == torch.bfloat16 else 1e-6, "identity")


def _two_sequences(nh, nkv, dk, dv, window, seed, values_are_keys=False):
    """Two sequences for one step, the second one a later portion of its prompt (its first keys already cached), with
    loud keys at the windows' edges of some queries; pages in no order in one pool."""
    r = _r(seed)
    T1, T2, start2 = 150, 333, 120
    seqs = []
    for T, start in ((T1, 0), (T2, start2)):
        k, q = r(T, nkv, dk), r(T - start, nh, dk)
        v = None if values_are_keys else r(T, nkv, dv)
        _loud_keys(q, k, list(range(start, T)), window, every=7)
        seqs.append((q, k, v, list(range(start, T))))
    return seqs, (T1, T2, start2)


def _pool_of(seqs, ps, dtype):
    orders = ([7, 1, 4], [0, 2, 8, 3, 6, 5])
    pool = None
    for (q, k, v, _), order in zip(seqs, orders):
        part, _ = _fill_cache(k, v, ps, dtype, order, 9)
        pool = part if pool is None else pool
        for p in order:
            pool[p] = part[p]
    table = torch.zeros((2, 6), dtype=torch.int32, device=DEV)
    table[0, :3] = torch.tensor(orders[0], dtype=torch.int32)
    table[1] = torch.tensor(orders[1], dtype=torch.int32)
    return pool, table


@pytest.mark.parametrize("nh,nkv,dk,dv,window,cap", [(4, 2, 16, 32, 9, 20.0), (3, 1, 96, 32, 0, 0.0), (2, 2, 48, 80, 64, 5.0),
                                                     (2, 1, 128, 128, 130, 0.0), (8, 4, 64, 64, 70, 30.0)])
def test_mixed_heads_on_the_tensor_cores(nh, nkv, dk, dv, window, cap):
    k_ = K()
    dtype, ps = torch.bfloat16, 64
    seqs, (T1, T2, start2) = _two_sequences(nh, nkv, dk, dv, window, dk + dv)
    r = _r(5)
    talk = torch.eye(nh, dtype=F64) + 0.5 * r(nh, nh)
    scale = 1.1 / math.sqrt(dk)
    want = torch.cat([_mixed_want(q, k, v, talk, scale, pos, window, cap, dtype) for q, k, v, pos in seqs])
    pool, table = _pool_of(seqs, ps, dtype)
    N = T1 + T2 - start2
    q_all = dev(torch.cat([s[0].reshape(len(s[3]), -1) for s in seqs]), dtype)
    out = torch.full((N, nh * dv), float("nan"), dtype=dtype, device=DEV)
    for split in (True, False):
        o_all = torch.full((N, nh, nkv, dv), float("nan"), device=DEV)
        k_.attention_sink_prefill(q_all, pool, ps, table, i32([0, T1, N]), i32([0, start2]), out, 2, nh, nkv, dk, dv, scale,
                                  softcap=cap, window=window, out_all=o_all, split_weights=split)
        k_.mix_heads(o_all, dev(talk), out, nh, nkv, dv)
        close(out, want, 1.2e-2, f"tensor cores, split weights {split}")
    # and the kernel of single query tokens gives the same, token by token
    positions = i32(seqs[0][3] + seqs[1][3])
    seq_of = i32([0] * T1 + [1] * (T2 - start2))
    o_all.fill_(float("nan"))
    k_.attention_sink(q_all, pool, ps, table, positions, seq_of, out, nh, nkv, dk, dv, scale, softcap=cap, window=window,
                      out_all=o_all)
    k_.mix_heads(o_all, dev(talk), out, nh, nkv, dv)
    close(out, want, 1.2e-2, "token by token")


def test_split_weights_carry_more_of_a_weight_into_the_value_product():
    """With values that are large and nearly cancel, the rounding of the softmax weights to bfloat16 shows; the two-number
    form brings the error down by an order of magnitude."""
    k_ = K()
    nh, nkv, dk, dv, ps, T = 2, 1, 32, 32, 64, 256
    r = _r(77)
    q, k = 0.3 * r(T, nh, dk), 0.3 * r(T, nkv, dk)
    v = (100.0 + r(T, nkv, dv)).to(torch.bfloat16).double()          # exact in bfloat16: only the weights' rounding is left
    w = P.attention_weights(q.to(torch.bfloat16).double(), k.to(torch.bfloat16).double(), 0.2)
    want = P.apply_weights(w, v)
    pool, pages = _fill_cache(k, v, ps, torch.bfloat16, [0, 1, 2, 3], 4)
    errs = {}
    for split in (False, True):
        out = torch.empty((T, nh * dv), dtype=torch.float32, device=DEV)
        o_all = torch.empty((T, nh, nkv, dv), device=DEV)
        k_.attention_sink_prefill(dev(q.reshape(T, -1), torch.bfloat16), pool, ps, i32([pages]), i32([0, T]), i32([0]),
                                  torch.empty((T, nh * dv), dtype=torch.bfloat16, device=DEV), 1, nh, nkv, dk, dv, 0.2,
                                  out_all=o_all, split_weights=split)
        errs[split] = (o_all.reshape(T, -1).double().cpu() - want).abs().max().item()
    assert errs[True] < 0.02 and errs[True] * 8 < errs[False], errs


# ------------------------------------------------------------------------------------------ values that are keys
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,dk,dv,window", [(4, 1, 48, 48, 40), (3, 3, 12, 12, 7), (2, 1, 20, 20, 0), (4, 2, 32, 32, 150),
                                                 (2, 2, 64, 24, 64)])
def test_distance_bias_sink_wide_gate_and_values_that_are_keys_token_by_token(nh, nkv, dk, dv, window, dtype):
    k_ = K()
    r = _r(nh + dk)
    T, ps = 300, 64
    k = r(T, nkv, dk)
    positions = [0, 1, 2, window, window + 1, 63, 64, 65, 128, 129, 200, 250, T - 2, T - 1]
    N = len(positions)
    q = r(N, nh, dk)
    _loud_keys(q, k, positions, window)
    r1, r2 = 0.3 + r(nh).abs(), 0.1 + r(nh).abs()
    gate = r(N, nh * dv)
    scale = 1.3 / math.sqrt(dk)
    qq, kq = q.to(dtype).double(), k.to(dtype).double()
    w = P.attention_weights(qq, kq, scale, positions, window=window, bias=(r1, r2), sink=True)
    want = P.apply_weights(w, kq[..., :dv]) * torch.sigmoid(gate)
    pool, pages = _fill_cache(k, None, ps, dtype, [4, 0, 3, 1, 2], 6)
    out = torch.full((N, nh * dv), float("nan"), dtype=dtype, device=DEV)
    wide = torch.randn(N, nh * dv + 7, device=DEV)
    wide[:, 3:3 + nh * dv] = dev(gate)
    k_.attention_sink(dev(q.reshape(N, -1), dtype), pool, ps, i32([pages]), i32(positions), i32([0] * N), out, nh, nkv, dk, dv,
                      scale, window=window, sinks=torch.zeros(nh, device=DEV), gate=wide[:, 3:3 + nh * dv], gate_wide=True,
                      distance_bias=(dev(r1), dev(r2)), values_in_keys=True)
    close(out, want, tol_of(dtype), "sink, bias, gate")
    # without the sink the weights sum to one; without the bias far keys weigh more
    k_.attention_sink(dev(q.reshape(N, -1), dtype), pool, ps, i32([pages]), i32(positions), i32([0] * N), out, nh, nkv, dk, dv,
                      scale, window=window, distance_bias=(dev(r1), dev(r2)), values_in_keys=True)
    close(out, P.apply_weights(P.attention_weights(qq, kq, scale, positions, window=window, bias=(r1, r2)), kq[..., :dv]),
          tol_of(dtype), "no sink")
    k_.attention_sink(dev(q.reshape(N, -1), dtype), pool, ps, i32([pages]), i32(positions), i32([0] * N), out, nh, nkv, dk, dv,
                      scale, window=window, sinks=torch.zeros(nh, device=DEV), values_in_keys=True)
    close(out, P.apply_weights(P.attention_weights(qq, kq, scale, positions, window=window, sink=True), kq[..., :dv]),
          tol_of(dtype), "no bias")


@pytest.mark.parametrize("nh,nkv,dk,dv,window", [(4, 1, 48, 48, 40), (2, 2, 16, 16, 9), (3, 1, 96, 96, 0), (2, 1, 128, 128, 130),
                                                 (4, 2, 64, 32, 64)])
def test_distance_bias_and_values_that_are_keys_on_the_tensor_cores(nh, nkv, dk, dv, window):
    k_ = K()
    dtype, ps = torch.bfloat16, 64
    seqs, (T1, T2, start2) = _two_sequences(nh, nkv, dk, dv, window, dk + 3, values_are_keys=True)
    r = _r(9)
    r1, r2 = 0.3 + r(nh).abs(), 0.1 + r(nh).abs()
    N = T1 + T2 - start2
    gate = r(N, nh * dv)
    scale = 1.1 / math.sqrt(dk)
    wants = []
    for q, k, _, pos in seqs:
        kq = k.to(dtype).double()
        w = P.attention_weights(q.to(dtype).double(), kq, scale, pos, window=window, bias=(r1, r2), sink=True)
        wants.append(P.apply_weights(w, kq[..., :dv]))
    want = torch.cat(wants) * torch.sigmoid(gate)
    pool, table = _pool_of(seqs, ps, dtype)
    q_all = dev(torch.cat([s[0].reshape(len(s[3]), -1) for s in seqs]), dtype)
    for split in (True, False):
        out = torch.full((N, nh * dv), float("nan"), dtype=dtype, device=DEV)
        k_.attention_sink_prefill(q_all, pool, ps, table, i32([0, T1, N]), i32([0, start2]), out, 2, nh, nkv, dk, dv, scale,
                                  window=window, sinks=torch.zeros(nh, device=DEV), gate=dev(gate), gate_wide=True,
                                  distance_bias=(dev(r1), dev(r2)), values_in_keys=True, split_weights=split)
        close(out, want, 1.2e-2, f"tensor cores, split weights {split}")


# ------------------------------------------------------------------------------------------ convolution
@pytest.mark.parametrize("C,taps,bias,act", [(48, 4, True, False), (30, 1, True, False), (96, 3, False, False), (7, 2, True, True),
                                             (160, 4, False, False)])
def test_causal_convolution_without_activation_under_every_cut(C, taps, bias, act):
    k_ = K()
    r = _r(C + taps)
    T = 70
    x, w = r(T, C + 5), r(C, taps)
    b = r(C) if bias else None
    want = P.causal_conv(x[:, 2:2 + C], w, b)
    if act:
        want = P.silu(want)
    xs = dev(x)
    for cuts in cuts_of(T):
        state = torch.full((3, max(taps - 1, 1), C), 5.0, device=DEV)
        state[1] = 0.0
        outs, at = [], 0
        for n in cuts:
            o = torch.full((n, C), float("nan"), device=DEV)
            k_.causal_conv(xs[at:at + n, 2:2 + C], dev(w), None if b is None else dev(b), state if taps > 1 else None, i32([0] * n),
                           i32([0, n]), i32([1]), o, 1, act=act)
            outs.append(o)
            at += n
        close(torch.cat(outs), want, 2e-6, f"cuts {cuts[:4]}")
        assert (state[[0, 2]] == 5.0).all()


@pytest.mark.parametrize("C,taps,act", [(48, 4, False), (30, 1, False), (7, 3, True), (300, 2, False)])
def test_causal_convolution_of_a_decode_batch_in_one_kernel(C, taps, act):
    """Three sequences, a token each a step (row b is sequence b's), their slots in no order, after a prompt of their own."""
    k_ = K()
    r = _r(C * taps)
    lens, w, b = [9, 1, 14], r(C, taps), r(C)
    xs = [r(n + 6, C) for n in lens]
    wants = [P.silu(P.causal_conv(x, w, b)) if act else P.causal_conv(x, w, b) for x in xs]
    state = torch.full((5, max(taps - 1, 1), C), 5.0, device=DEV)
    slots = [3, 0, 4]
    state[slots] = 0.0
    st = state if taps > 1 else None
    cu = [0, lens[0], lens[0] + lens[1], sum(lens)]
    seq_of = [i for i, n in enumerate(lens) for _ in range(n)]
    o = torch.full((sum(lens), C), float("nan"), device=DEV)
    k_.causal_conv(dev(torch.cat([x[:n] for x, n in zip(xs, lens)])), dev(w), dev(b), st, i32(seq_of), i32(cu), i32(slots), o, 3, act=act)
    for i, n in enumerate(lens):
        close(o[cu[i]:cu[i + 1]], wants[i][:n], 2e-6, f"prompt {i}")
    for t in range(6):
        o = torch.full((3, C), float("nan"), device=DEV)
        k_.causal_conv(dev(torch.stack([x[n + t] for x, n in zip(xs, lens)])), dev(w), dev(b), st, i32([0, 1, 2]), i32([0, 1, 2, 3]),
                       i32(slots), o, 3, act=act, one_each=True)
        close(o, torch.stack([wt[n + t] for wt, n in zip(wants, lens)]), 2e-6, f"token {t}")
    assert (state[[1, 2]] == 5.0).all()


# ------------------------------------------------------------------------------------------ gated linear recurrence
def _recurrence_case(T, C, nb, seed):
    r = _r(seed)
    bs = C // nb
    u, y = r(T, C), r(T, C + 3)
    wa, wi, ba, bi = r(nb, bs, bs) / math.sqrt(bs), r(nb, bs, bs) / math.sqrt(bs), r(nb, bs), r(nb, bs)
    lam = -6.0 + 4.5 * torch.rand(C, generator=torch.Generator().manual_seed(seed), dtype=F64)
    gates = (torch.sigmoid(P.block_gates(u, wa, ba)), torch.sigmoid(P.block_gates(u, wi, bi)))
    want = P.gated_recurrence(u, gates[0], gates[1], lam) * P.gelu_tanh(y[:, 1:1 + C])
    return (u, y, wa, wi, ba, bi, lam), want


def _run_recurrence(k_, case, cuts, C, state, slot, out_dtype=torch.float32):
    u, y, wa, wi, ba, bi, lam = case
    args = [dev(wa.transpose(1, 2)), dev(wi.transpose(1, 2)), dev(ba.reshape(-1)), dev(bi.reshape(-1)), dev(lam)]
    us, ys = dev(u), dev(y)
    outs, at = [], 0
    for n in cuts:
        a = torch.full((n, C), float("nan"), device=DEV)
        x = torch.full((n, C), float("nan"), device=DEV)
        k_.block_gates(us[at:at + n].contiguous(), *args, 8.0, a, x)
        o = torch.full((n, C), float("nan"), dtype=out_dtype, device=DEV)
        k_.gated_recurrence(a, x, ys[at:at + n, 1:1 + C], state, i32([slot]), i32([0, n]), o, 1, max_len=n)
        outs.append(o)
        at += n
    return torch.cat(outs)


@pytest.mark.parametrize("C,nb", [(48, 2), (30, 1), (40, 5), (64, 64), (160, 2), (258, 1), (96, 3)])
def test_gated_recurrence_under_every_cut(C, nb):
    k_, T = K(), 61
    case, want = _recurrence_case(T, C, nb, seed=C + nb)
    for cuts in cuts_of(T):
        state = torch.zeros(3, C, device=DEV)
        close(_run_recurrence(k_, case, cuts, C, state, 1), want, 2e-5, f"cuts {cuts[:4]}")
        assert state[0].abs().max() == 0 and state[2].abs().max() == 0          # the other slots are untouched
    state = torch.zeros(3, C, device=DEV)
    close(_run_recurrence(k_, case, [T], C, state, 2, torch.bfloat16), want, 6e-3, "bfloat16 out")


def test_gated_recurrence_long_steps_in_pieces_and_a_memory_that_lasts():
    """Hundreds of tokens a step (the walk in pieces), whole and cut where the pieces do not end; a channel that
    forgets nothing to speak of carries its first input to the end."""
    k_, C, nb = K(), 70, 2
    for T in (64, 257, 1000):
        case, want = _recurrence_case(T, C, nb, seed=T)
        lam = case[6]
        lam[:4] = -12.0                                      # a = exp(-8 r softplus(-12)): all but 1
        case = case[:6] + (lam,)
        u, y, wa, wi, ba, bi, _ = case
        want = P.gated_recurrence(u, torch.sigmoid(P.block_gates(u, wa, ba)), torch.sigmoid(P.block_gates(u, wi, bi)), lam) \
            * P.gelu_tanh(y[:, 1:1 + C])
        for cuts in ([T], [T - 40, 40], [3, T - 3], [T // 2, T - T // 2]):
            state = torch.zeros(2, C, device=DEV)
            close(_run_recurrence(k_, case, cuts, C, state, 0), want, 3e-5, f"{T} tokens, cuts {cuts}")


def test_gated_recurrence_batches_and_slots_used_again():
    k_, C, nb = K(), 48, 3
    lens = [37, 1, 180, 9]
    cases = [_recurrence_case(n, C, nb, seed=200 + n) for n in lens]
    shared = cases[0][0][2:]                                 # every request with the first one's weights
    wants = []
    for (u, y, *_), _ in cases:
        wa, wi, ba, bi, lam = shared
        wants.append(P.gated_recurrence(u, torch.sigmoid(P.block_gates(u, wa, ba)), torch.sigmoid(P.block_gates(u, wi, bi)), lam)
                     * P.gelu_tanh(y[:, 1:1 + C]))
    state = torch.full((6, C), 7.0, device=DEV)              # what an earlier sequence left behind
    slots = [4, 0, 5, 2]
    state[slots] = 0.0                                       # the cache zeroes a slot when it assigns it
    us, ys = dev(torch.cat([c[0][0] for c in cases])), dev(torch.cat([c[0][1] for c in cases]))
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    wa, wi, ba, bi, lam = shared
    N = sum(lens)
    a, x = torch.empty((N, C), device=DEV), torch.empty((N, C), device=DEV)
    k_.block_gates(us, dev(wa.transpose(1, 2)), dev(wi.transpose(1, 2)), dev(ba.reshape(-1)), dev(bi.reshape(-1)), dev(lam), 8.0, a, x)
    for max_len in (max(lens), 1):                           # in pieces, and every sequence in one go
        st = state.clone()
        o = torch.full((N, C), float("nan"), device=DEV)
        k_.gated_recurrence(a, x, ys[:, 1:1 + C], st, i32(slots), i32(cu), o, len(lens), max_len=max_len)
        for i, want in enumerate(wants):
            close(o[cu[i]:cu[i + 1]], want, 3e-5, f"request {i}")
        assert (st[[1, 3]] == 7.0).all()


# ------------------------------------------------------------------------------------------ delta rule, a decay a head
def _delta_case(T, H, KV, dk, dv, seed):
    r = _r(seed)
    q, k, v = r(T, KV * dk), r(T, KV * dk), r(T, H * dv)
    beta, a = r(T, H), r(T, H)
    dt_bias = -1.0 + r(H)
    a_log = torch.log(0.02 + 0.98 * torch.rand(H, generator=torch.Generator().manual_seed(seed), dtype=F64))
    rep = H // KV
    qn = (P.unit(q.view(T, KV, dk)) * dk ** -0.5).repeat_interleave(rep, 1)
    kn = P.unit(k.view(T, KV, dk)).repeat_interleave(rep, 1)
    want = P.delta_rule(qn, kn, v.view(T, H, dv), torch.sigmoid(beta), P.head_decay(a, dt_bias, a_log))
    return (q, k, v, beta, a, dt_bias, a_log), want.reshape(T, H * dv)


@pytest.mark.parametrize("H,KV,dk,dv", [(6, 3, 32, 64), (4, 2, 16, 8), (1, 1, 20, 12), (2, 1, 72, 40), (1, 1, 136, 17), (3, 3, 5, 33),
                                        (2, 1, 64, 32), (2, 2, 128, 18)])
def test_delta_rule_with_a_decay_a_head_under_every_cut(H, KV, dk, dv):
    k_, T = K(), 61
    case, want = _delta_case(T, H, KV, dk, dv, seed=dk + H)
    q, kk, v, beta, a, dt_bias, a_log = [dev(x) for x in case]
    wide = torch.randn(T, 2 * H + 3, device=DEV)              # beta and the decay's logits as columns of a wider matrix
    wide[:, 1:1 + H], wide[:, 1 + H:1 + 2 * H] = beta, a
    for ws in (None, _Ws()):                              # without scratch every step runs the token-by-token kernel
        for cuts in cuts_of(T):
            state = torch.zeros(3, H, dv, dk, device=DEV)
            outs, at = [], 0
            for n in cuts:
                rows = slice(at, at + n)
                o = torch.full((n, H * dv), float("nan"), device=DEV)
                k_.delta_scan(q[rows], kk[rows], v[rows], wide[rows, 1:1 + H], wide[rows, 1 + H:1 + 2 * H], dt_bias, a_log, state,
                              i32([1]), i32([0, n]), o, 1, H, KV, dk, dv, q_scale=dk ** -0.5, max_len=n, ws=ws, head_decay=True)
                outs.append(o)
                at += n
            close(torch.cat(outs), want, 3e-5, f"cuts {cuts[:4]} scratch {ws is not None}")
            assert state[0].abs().max() == 0 and state[2].abs().max() == 0


# ------------------------------------------------------------------------------------------ joining kernel and norm
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [48, 200, 1030, 2048, 4100])
def test_scaled_add_norm(H, out_dtype):
    k_ = K()
    r = _r(H)
    N = 9
    y1, y2, vec, x, w = r(N, H), r(N, H), r(H), r(N, H), r(H)
    for two in (True, False):
        total = x + vec * (0.6 * y1 + (0.5 * y2 if two else 0.0))
        resid = dev(x)
        out = torch.full((N, H), float("nan"), dtype=out_dtype, device=DEV)
        k_.scaled_add_norm(dev(y1), dev(vec), resid, s1=0.6, y2=dev(y2) if two else None, s2=0.5, w=dev(w), eps=1e-5, out=out)
        close(resid, total, 2e-6, "stream")
        close(out, P.rms_norm(total, w, 1e-5), 2e-5 if out_dtype == torch.float32 else 8e-3, "normed rows")
        resid = dev(x)
        k_.scaled_add_norm(dev(y1), dev(vec), resid, s1=0.6, y2=dev(y2) if two else None, s2=0.5)
        close(resid, total, 2e-6, "stream alone")


def test_norm_part_with_a_weight_around_zero():
    from mivi_v4_b200.parts.norm import RMSNorm
    r = _r(3)
    x, w = r(5, 72), 0.3 * r(72)
    part = RMSNorm(72, 1e-5, one_plus=True)
    part.load({"weight": dev(w)})
    out = torch.empty((5, 72), device=DEV)
    part.forward(dev(x), out)
    close(out, P.rms_norm(x, w, 1e-5, one_plus=True), 2e-6)
    part = RMSNorm(72, 1e-5)
    part.load({"weight": dev(w)})
    part.forward(dev(x), out)
    close(out, P.rms_norm(x, w, 1e-5), 2e-6)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("F", [33, 48, 320, 1028])
def test_clamped_activation_four_features_a_thread_and_one(F, out_dtype):
    k_ = K()
    r = _r(F)
    N = 7
    gu = 3.0 * r(N, 2 * F)
    eye, zero = torch.eye(F, dtype=F64), torch.zeros(F, F, dtype=F64)
    want = P.clamped_glu(gu, {"gate": torch.cat([eye, zero], 1), "up": torch.cat([zero, eye], 1), "down": eye}, {"limit": 1.25})
    out = torch.full((N, F), float("nan"), dtype=out_dtype, device=DEV)
    k_.glu_clamped(dev(gu), out, 1.25, 1.702)
    close(out, want, 2e-6 if out_dtype == torch.float32 else 5e-3)
