"""Matepel family on the GPU against the float64 oracle (oracle/matepel_oracle.py): every mechanism alone through its
operator, then whole models through the serving path (ScheduleBatch → worker → kernels, decode through the captured
CUDA graphs) under every way of cutting and batching the same tokens, then greedy generation through the semi-PD
engine."""
import math

import pytest
import torch

from oracle import matepel_oracle as M
from tests import matepel_helpers as C
from tests import rimidra_helpers as H

pytestmark = pytest.mark.gpu

DEV = "cuda"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _close(got, want, dtype, what="", tol32=2e-5, tol16=3e-2):
    tol = tol32 if dtype == torch.float32 else tol16
    err = (got.double().cpu() - want.double().cpu()).abs().max().item()
    ref = want.double().abs().max().item() + 1e-9
    assert err <= tol * ref, f"{what}: max abs err {err:.3e} vs ref max {ref:.3e}"


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def i64(x):
    return torch.tensor(x, dtype=torch.int64, device=DEV)


# =================================================================================================
# mechanisms alone
# =================================================================================================
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("streams,width", [(1, 36), (2, 64), (3, 7), (8, 300)])
def test_embedding_into_streams(dtype, streams, width):
    from semi_pd_b200 import ops
    dt = DT[dtype]
    g = torch.Generator().manual_seed(width)
    table = (torch.randn(20, width, generator=g) * 2).to(dt)
    w = (1 + 0.3 * torch.randn(width, generator=g)).to(dt)
    ids = torch.randint(0, 20, (9,), generator=g)
    got = ops.embed_norm_streams(table.to(DEV), ids.to(DEV), w.to(DEV), 1e-6, streams)
    want = M.rms_norm(table.double()[ids], w, 1e-6)
    assert got.shape == (9, streams, width)
    for s in range(streams):
        _close(got[:, s], want, torch.float32, f"stream {s}", tol32=1e-6)
    raw = ops.embed_norm_streams(table.to(DEV), ids.to(DEV), None, 1e-6, streams)
    _close(raw[:, streams - 1], table.double()[ids], torch.float32, "raw rows", tol32=1e-7)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("streams,width", [(1, 40), (2, 64), (3, 1000), (4, 256), (8, 52), (2, 10500)])
def test_stream_write_read_norm(dtype, streams, width):
    """Write of one sublayer (two branch outputs, scales, bias) + read and norm of the next in one launch; the write
    alone; the read alone, of all rows and of chosen rows.  Widths above the shared-memory stash included."""
    from semi_pd_b200 import ops
    dt = DT[dtype]
    S, T = streams, 6
    g = torch.Generator().manual_seed(S * 1000 + width)
    X = torch.randn(S, T, width, generator=g) * 3
    a, b = torch.randn(T, width, generator=g).to(dt), torch.randn(T, width, generator=g).to(dt)
    bias = torch.randn(width, generator=g)
    mix = torch.eye(S) * 0.7 + 0.3 * torch.randn(S, S, generator=g)
    w_out, w_in = 1 + 0.3 * torch.randn(S, generator=g), torch.randn(S, generator=g)
    w = (1 + 0.2 * torch.randn(width, generator=g)).to(dt)
    sa, sb, mult = 0.8, 1.3, 0.6
    Xd = X.permute(1, 0, 2).contiguous().to(DEV)  # the product keeps a token's streams together
    h = ops.streams_mix_norm(Xd, w.to(DEV), 1e-6, a=a.to(DEV), b=b.to(DEV), bias=bias.to(DEV), sa=sa, sb=sb, sbias=sa,
                             mix=mix.to(DEV), out_w=w_out.to(DEV), mult=mult, in_w=w_in.to(DEV))
    y = sa * a.double() + sb * b.double() + sa * bias.double()
    X1 = M.streams_write(X.double(), y, mix, w_out, mult)
    _close(Xd.permute(1, 0, 2), X1, torch.float32, "streams after the write", tol32=2e-6)
    _close(h, M.rms_norm(M.streams_read(X1, w_in), w, 1e-6), dt, "read + norm")
    # write alone (one branch, no bias), then the plain sum of chosen rows through the norm
    ops.streams_mix_norm(Xd, None, 1e-6, a=a.to(DEV), mix=mix.to(DEV), out_w=w_out.to(DEV), mult=mult)
    X2 = M.streams_write(X1, a.double(), mix, w_out, mult)
    _close(Xd.permute(1, 0, 2), X2, torch.float32, "write alone", tol32=2e-6)
    rows = [4, 0, 5]
    hs = ops.streams_mix_norm(Xd, w.to(DEV), 1e-6, rows=i64(rows))
    _close(hs, M.rms_norm(X2.sum(0)[rows], w, 1e-6), dt, "sum of chosen rows")
    _close(Xd.permute(1, 0, 2), X2, torch.float32, "a read leaves the streams alone", tol32=2e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_clamped_gated_activation_and_gated_norms(dtype):
    from semi_pd_b200 import ops
    dt = DT[dtype]
    g = torch.Generator().manual_seed(3)
    for inter, limit in ((20, 1.0), (64, 7.0), (37, 0.25)):
        x = (torch.randn(9, 2 * inter, generator=g) * 4).to(dt)  # well beyond every limit on both sides
        got = ops.act_and_mul(x.to(DEV), "clamped_swish", limit=limit, slope=1.702)
        gate, up = x.double()[:, :inter].clamp(max=limit), x.double()[:, inter:].clamp(-limit, limit)
        _close(got, gate * torch.sigmoid(1.702 * gate) * (up + 1), dt, f"limit {limit}")
    # one norm over all heads, and a norm per head with a weight over all heads; sigmoid gate inside a wider row
    of = torch.randn(7, 3 * 10, generator=g) * 4
    wide = torch.randn(7, 50, generator=g).to(dt)
    w = (1 + 0.3 * torch.randn(30, generator=g)).to(dt)
    gate = torch.sigmoid(wide.double()[:, 12:42])
    got = ops.headnorm_gate(of.to(DEV), wide.to(DEV)[:, 12:42], 1, 30, 1e-5, weight=w.to(DEV), gate_act="sigmoid")
    _close(got, M.rms_norm(of.double(), w, 1e-5) * gate, dt, "all heads together")
    got = ops.headnorm_gate(of.to(DEV), wide.to(DEV)[:, 12:42], 3, 10, 1e-5, weight=w.to(DEV), gate_act="sigmoid")
    want = M.unit_rms(of.double().view(7, 3, 10), 1e-5).reshape(7, 30) * w.double() * gate
    _close(got, want, dt, "per head")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(2, 16, 16), (1, 8, 40), (3, 64, 32), (1, 100, 12), (2, 160, 64)])
def test_lightning_recurrence(dtype, shape):
    """SiLU applied as the kernel reads q, k, v (slices of one wider row): portions of two unequal requests against
    the token-by-token recurrence, then decoding with a padded row; a head that never forgets keeps the first tokens."""
    from semi_pd_b200 import ops
    dt = DT[dtype]
    Hh, dk, dv = shape
    T = 70
    g = torch.Generator().manual_seed(dk * 7 + dv)
    decay = [1.0] + [0.9 ** (h + 1) for h in range(Hh - 1)]
    sizes = [Hh * dk, Hh * dk, Hh * dv]
    seqs = []
    for _ in range(2):
        row = torch.randn(T, sum(sizes) + 8, generator=g).to(dt)
        q, k, v = (M.silu(t.double()) for t in row[:, : sum(sizes)].split(sizes, -1))
        o, S = M.fixed_decay_recurrence(q.view(T, Hh, dk), k.view(T, Hh, dk), v.view(T, Hh, dv), decay,
                                        torch.zeros(Hh, dk, dv, dtype=torch.float64))
        seqs.append((row, o.reshape(T, Hh * dv), S))
    state = torch.full((6, Hh, dk, dv), 5.0, device=DEV)  # stale content that position 0 must ignore
    kw = dict(num_heads=Hh, head_dim=dk, v_dim=dv, decay=torch.tensor(decay, device=DEV), cos_sin=None, rot_dims=0,
              k_scale=1.0, in_act="silu")

    def split(rows):
        return rows[:, : sum(sizes)].split(sizes, -1)

    at = [0, 0]
    for n0, n1 in ((1, 2), (17, 2), (2, 33), (16, 1)):
        rows = torch.cat([seqs[0][0][at[0]:at[0] + n0], seqs[1][0][at[1]:at[1] + n1]]).to(DEV)
        o = ops.retention(*split(rows), state, i64([3, 1]), prefix_lens=i32(at), extend_lens=i32([n0, n1]),
                          extend_start_loc=i32([0, n0]), **kw)
        _close(o, torch.cat([seqs[0][1][at[0]:at[0] + n0], seqs[1][1][at[1]:at[1] + n1]]), dt, f"portions {(n0, n1)}",
               tol32=5e-5)
        at = [at[0] + n0, at[1] + n1]
    before = state[4].clone()
    while max(at) < T:
        rows = torch.cat([seqs[0][0][at[0]:at[0] + 1], seqs[1][0][at[1]:at[1] + 1], seqs[0][0][:1]]).to(DEV)
        o = ops.retention(*split(rows), state, i64([3, 1, 4]), seq_lens=i64([at[0] + 1, at[1] + 1, 1]),
                          out_cache_loc=i64([7, 9, 0]), **kw)
        _close(o[:2], torch.cat([seqs[0][1][at[0]:at[0] + 1], seqs[1][1][at[1]:at[1] + 1]]), dt, f"decode {at}", tol32=5e-5)
        at = [at[0] + 1, at[1] + 1]
    assert torch.equal(state[4], before)
    _close(state[1], seqs[1][2], dt, "final state", tol32=5e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape,cap", [((2, 16, 16), 12.0), ((1, 8, 40), 2.0), ((3, 32, 64), 20.0), ((1, 100, 12), 0.0),
                                       ((2, 160, 64), 6.0), ((3, 64, 96), 10.0)])
def test_matrix_memory(dtype, shape, cap):
    """Gates computed in the kernel from raw projections (slices of one wider row) and biases: portions of two
    unequal requests against the token-by-token recurrence, then decoding with a padded row, then a slot used again.
    One request's input gate runs high (the running maximum climbs, the normaliser rules the denominator), the other's
    stays low (the maximum stays at its start and exp(-m) rules)."""
    from semi_pd_b200 import ops
    dt = DT[dtype]
    Hh, dk, dv = shape
    T = 70
    g = torch.Generator().manual_seed(dk * 11 + dv)
    sizes = [Hh * dk, Hh * dk, Hh * dv, Hh, Hh]
    i_bias, f_bias = torch.randn(Hh, generator=g), 2.0 + torch.randn(Hh, generator=g)
    q_scale = dk ** -0.5
    seqs = []
    for r in range(2):
        row = torch.randn(T, sum(sizes) + 8, generator=g)
        row[:, -8 - 2 * Hh: -8 - Hh] = row[:, -8 - 2 * Hh: -8 - Hh] * 3 + (4.0 if r == 0 else -14.0)  # input gate
        row = row.to(dt)
        q, k, v, zi, zf = (t.double() for t in row[:, : sum(sizes)].split(sizes, -1))
        capf = (lambda z: M.soft_cap(z, cap)) if cap > 0 else (lambda z: z)
        il, fl = capf(zi + i_bias.double()), M.log_sigmoid(capf(zf + f_bias.double()))
        o, S, n, m = M.matrix_memory_recurrence(q.view(T, Hh, dk) * q_scale, k.view(T, Hh, dk), v.view(T, Hh, dv), il, fl,
                                                torch.zeros(Hh, dk, dv, dtype=torch.float64),
                                                torch.zeros(Hh, dk, dtype=torch.float64), torch.zeros(Hh, dtype=torch.float64))
        seqs.append((row, o.reshape(T, Hh * dv), S, n, m))
    if cap >= 10:
        assert seqs[0][4].min() > 2 and seqs[1][4].max() < 0, "the test's gates do not reach both regimes"
    vdim = ops.matrix_memory_vector_dim(Hh, dk, dv)
    state = torch.full((6, Hh, dk, dv), 5.0, device=DEV)  # stale content that position 0 must ignore
    vec = torch.full((6, vdim), -3.0, device=DEV)
    kw = dict(num_heads=Hh, head_dim=dk, v_dim=dv, i_bias=i_bias.to(DEV), f_bias=f_bias.to(DEV), cap=cap, q_scale=q_scale)

    def split(rows):
        return rows[:, : sum(sizes)].split(sizes, -1)

    def run_portions(slots, plan):
        at = [0, 0]
        for n0, n1 in plan:
            rows = torch.cat([seqs[0][0][at[0]:at[0] + n0], seqs[1][0][at[1]:at[1] + n1]]).to(DEV)
            o = ops.matrix_memory(*split(rows), state, vec, i64(slots), prefix_lens=i32(at), extend_lens=i32([n0, n1]),
                                  extend_start_loc=i32([0, n0]), **kw)
            _close(o, torch.cat([seqs[0][1][at[0]:at[0] + n0], seqs[1][1][at[1]:at[1] + n1]]), dt,
                   f"portions {(n0, n1)} at {at}", tol32=1e-4)
            at = [at[0] + n0, at[1] + n1]
        return at

    at = run_portions([3, 1], ((1, 2), (17, 2), (2, 33), (16, 1)))
    before, before_v = state[4].clone(), vec[4].clone()
    while max(at) < T:
        rows = torch.cat([seqs[0][0][at[0]:at[0] + 1], seqs[1][0][at[1]:at[1] + 1], seqs[0][0][:1]]).to(DEV)
        o = ops.matrix_memory(*split(rows), state, vec, i64([3, 1, 4]), seq_lens=i64([at[0] + 1, at[1] + 1, 1]),
                              out_cache_loc=i64([7, 9, 0]), **kw)
        _close(o[:2], torch.cat([seqs[0][1][at[0]:at[0] + 1], seqs[1][1][at[1]:at[1] + 1]]), dt, f"decode {at}", tol32=1e-4)
        at = [at[0] + 1, at[1] + 1]
    assert torch.equal(state[4], before) and torch.equal(vec[4], before_v), "a padded row wrote its slot"
    _close(state[1], seqs[1][2], dt, "final matrix state", tol32=1e-4)
    blocks = -(-dv // 32)
    per = vec[1].view(Hh, blocks, dk + 1).double().cpu()
    for z in range(blocks):  # every column block keeps the same normaliser and running maximum
        _close(per[:, z, :dk], seqs[1][3], dt, "normaliser", tol32=1e-4)
        assert (per[:, z, dk] - seqs[1][4]).abs().max().item() < 1e-4
    # the slots of finished requests, taken by the same two sequences in swapped order
    seqs.reverse()
    run_portions([1, 3], ((33, 16), (2, 2), (35, 52)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", [dict(Hq=4, Hk=2, dk=16, rot=8, base=1e4, scaling=(4.0, 64, 8.0, 1.0)),
                                  dict(Hq=6, Hk=2, dk=64, rot=32, base=5e5, scaling=(6.0, 1024, 24.0, 1.0)),
                                  dict(Hq=1, Hk=1, dk=12, rot=12, base=100.0, scaling=None),
                                  dict(Hq=2, Hk=2, dk=10, rot=0, base=1e4, scaling=None),
                                  dict(Hq=3, Hk=3, dk=32, rot=32, base=5e5, scaling=(16.0, 512, 2.0, 0.5))])
def test_rotary_bias_store(dtype, case):
    """Bias, partial rotation with rescaled frequencies at small and large positions, and the fused cache write: rotated
    keys into the key pool, the biased keys BEFORE rotation into the value pool; other pool rows stay untouched."""
    from semi_pd_b200 import ops
    from semi_pd_b200.matepel import scaled_rotary_table
    dt = DT[dtype]
    Hq, Hk, dk, rot = case["Hq"], case["Hk"], case["dk"], case["rot"]
    scaling = dict(zip(("factor", "original", "fast", "slow"), case["scaling"])) if case["scaling"] else None
    g = torch.Generator().manual_seed(Hq * 100 + dk)
    pos = [0, 1, 2, 63, 64, 1000, 4097, 20000]
    T = len(pos)
    wide = torch.randn(T, Hq * dk + Hk * dk + 8, generator=g).to(dt)
    qb, kb = torch.randn(Hq * dk, generator=g), torch.randn(Hk * dk, generator=g)
    table = scaled_rotary_table(rot, case["base"], scaling, 20001, DEV)
    k_pool = torch.zeros(40, Hk, dk, dtype=dt, device=DEV)
    v_pool = torch.zeros(40, Hk, dk, dtype=dt, device=DEV)
    loc = [5, 39, 1, 17, 18, 2, 30, 9]
    wd = wide.to(DEV)
    q_out = ops.rotary_bias_store(wd[:, : Hq * dk], wd[:, Hq * dk: (Hq + Hk) * dk], None, qb.to(DEV), kb.to(DEV), k_pool,
                                  v_pool, i64(loc), i64(pos), table, rot, Hq, Hk, dk, dk)
    q = (wide.double()[:, : Hq * dk] + qb.double()).view(T, Hq, dk)
    k = (wide.double()[:, Hq * dk: (Hq + Hk) * dk] + kb.double()).view(T, Hk, dk)
    if rot:
        f, mag = M.scaled_rotary_frequencies(rot, case["base"], scaling)
        qr, kr = (M.rotate_half_partial(t, torch.tensor(pos), rot, f, mag) for t in (q, k))
    else:
        qr, kr = q, k
    _close(q_out, qr.reshape(T, -1), dt, "rotated queries", tol32=3e-6)
    _close(k_pool[loc], kr, dt, "rotated keys in the pool", tol32=3e-6)
    _close(v_pool[loc], k, dt, "unrotated keys as values", tol32=1e-6)
    rest = [i for i in range(40) if i not in loc]
    assert k_pool[rest].abs().max().item() == 0 and v_pool[rest].abs().max().item() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim", [(12, 2, 64), (4, 2, 16), (1, 1, 10), (8, 2, 128), (3, 3, 80)])
def test_softmax_with_one_more_unit(dtype, heads, kv_heads, dim):
    """Attention whose denominator is 1 + Σ exp(s): requests of unequal length whose slots are interleaved in the pool,
    decoded in one launch and extended in portions.  The one-token request has a score near 0 (the extra unit takes half
    of the weight: leaving it out would double the output) and in the long request one far key is made to win a head."""
    from semi_pd_b200 import ops
    dt = DT[dtype]
    g = torch.Generator().manual_seed(heads * 100 + dim)
    lens = [700, 129, 1, 64, 257]
    scale = dim ** -0.5
    total = sum(lens)
    perm = (torch.randperm(total, generator=g) + 1).tolist()
    k_pool = torch.zeros(total + 1, kv_heads, dim, dtype=dt)
    v_pool = torch.zeros(total + 1, kv_heads, dim, dtype=dt)
    r2t = torch.zeros(len(lens) + 1, max(lens) + 8, dtype=torch.int32)
    ks, vs, qs, at = [], [], [], 0
    for i, L in enumerate(lens):
        k = torch.randn(L, kv_heads, dim, generator=g).to(dt)
        v = torch.randn(L, kv_heads, dim, generator=g).to(dt)
        q = torch.randn(L, heads, dim, generator=g).to(dt)
        if L == 1:  # a score near 0: exp(s) is about 1, as large as the unit in the denominator
            q = (q.float() * 0.01).to(dt)
        if L > 600:  # the last head of the last queries looks at key 5, far back
            k[5, kv_heads - 1] = (6.0 * k[5, kv_heads - 1].float() / k[5, kv_heads - 1].float().norm()).to(dt)
            q[-40:, heads - 1] = (8.0 * k[5, kv_heads - 1].float()).to(dt)
        slots = perm[at:at + L]
        at += L
        k_pool[slots], v_pool[slots] = k, v
        r2t[i, :L] = torch.tensor(slots, dtype=torch.int32)
        ks.append(k), vs.append(v), qs.append(q)

    def want(i, lo, hi):
        return M.plus_one_softmax_attention(qs[i].double()[lo:hi], ks[i].double()[:hi], vs[i].double()[:hi], scale
                                            ).reshape(hi - lo, heads * dim)

    kd, vd, r2d = k_pool.to(DEV), v_pool.to(DEV), r2t.to(DEV)
    sinks = torch.zeros(heads, device=DEV)
    kw = dict(num_q_heads=heads, num_kv_heads=kv_heads, head_dim=dim, v_dim=dim, sm_scale=scale, sinks=sinks)
    rpi = i64(list(range(len(lens))))
    q = torch.stack([qs[i][-1].reshape(-1) for i in range(len(lens))]).to(DEV)
    got = ops.attn_general(q, kd, vd, r2d, rpi, seq_lens=i64(lens), **kw)
    _close(got, torch.cat([want(i, L - 1, L) for i, L in enumerate(lens)]), dt, "decode")
    ns = [40, 2, 1, 17, 33]
    q = torch.cat([qs[i][L - n:].reshape(n, -1) for i, (L, n) in enumerate(zip(lens, ns))]).to(DEV)
    starts = [sum(ns[:i]) for i in range(len(ns))]
    got = ops.attn_general(q, kd, vd, r2d, rpi, prefix_lens=i32([L - n for L, n in zip(lens, ns)]),
                           extend_lens=i32(ns), extend_start_loc=i32(starts), max_extend_len=max(ns), **kw)
    ref = torch.cat([want(i, L - n, L) for i, (L, n) in enumerate(zip(lens, ns))])
    _close(got, ref, dt, "extend")
    # what the test's inputs are made to show
    far = want(0, lens[0] - 1, lens[0])[0, (heads - 1) * dim:]
    assert (far - vs[0][5, kv_heads - 1].double()).abs().max() < 0.05 * vs[0].double().abs().max(), "the far key does not win"
    plain = vs[2].double()[0, 0]  # what a softmax without the unit gives a single key
    assert plain.abs().max() > 1.5 * want(2, 0, 1)[0, :dim].abs().max(), "the extra unit does not show"


# =================================================================================================
# whole models through the serving path
# =================================================================================================
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, make in C.CONFIGS.items():
        cfg = make()
        weights = M.make_weights(cfg, seed=C.SEEDS[name], gain=2.0 if name == "far" else 1.0)
        folder = H.write_model(tmp_path_factory.mktemp(name), cfg, weights)
        out[name] = (cfg, weights, folder)
    return out


_oracle_cache = {}


def _oracle(models, name, tokens):
    key = (name, tuple(tokens))
    if key not in _oracle_cache:
        cfg, weights, _ = models[name]
        _oracle_cache[key] = M.forward(cfg, weights, list(tokens))
    return _oracle_cache[key]


def _check(got, want, dtype, what):
    err = H.rel_err(got, want)
    tol = H.TOL[dtype]
    if dtype == "float32":
        assert err.max().item() < tol, f"{what}: worst relative error {err.max().item():.3e} at row {int(err.argmax())}"
    else:  # 16-bit: a sharp softmax between two close keys amplifies the rounding of a few rows
        assert err.median().item() < tol / 4, f"{what}: median {err.median().item():.3e}"
        assert err.max().item() < 3 * tol and (err > tol).float().mean().item() <= 0.02, \
            f"{what}: worst {err.max().item():.3e}, {(err > tol).sum()} rows off"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "ones"])
def test_residual_after_every_layer(models, name, dtype):
    """The sum of the streams after every layer of a short prompt."""
    cfg, weights, folder = models[name]
    s = H.open_session(folder, dtype, max_tokens=256, max_requests=2, cuda_graph=False)
    model = s.worker.model_runner.model
    got = {}
    model._layer_hook = lambda i, x: got.__setitem__(i, x.double().cpu())
    toks = H.prompt(19, cfg["vocab"], 19)
    s.step([{"id": "a", "tokens": toks, "want": []}])
    model._layer_hook = None
    want = []
    M.forward(cfg, weights, toks, want)
    assert len(got) == len(want)
    for r, ref in enumerate(want):
        rel = ((got[r] - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt()).item()
        assert rel < (1e-5 if dtype == "float32" else 2e-2), f"layer {r}: relative RMS error {rel:.3e}"


LENGTHS = (1, 2, 13, 150)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(C.CONFIGS))
def test_model_every_schedule(models, name, dtype):
    """Whole prompts, prompt + token-by-token decoding, portions of changing size down to two tokens, and mixed
    batches of unequal requests — each position against the whole-sequence oracle; all of it in one small pool,
    so request slots, state slots and cache runs are reused throughout."""
    cfg, _, folder = models[name]
    s = H.open_session(folder, dtype, max_tokens=640, max_requests=4)
    V = cfg["vocab"]
    prompts = {n: H.prompt(n, V, seed=n) for n in LENGTHS}
    full = lambda n: list(range(n))
    for n, toks in prompts.items():
        got = s.step([{"id": f"w{n}", "tokens": toks, "want": full(n)}])
        s.end([f"w{n}"])
        _check(got, _oracle(models, name, toks), dtype, f"{name} whole {n}")
    for n in (13, 150):
        toks, want = prompts[n], _oracle(models, name, prompts[n])
        cut = n - 9
        rows = [s.step([{"id": "d", "tokens": toks[:cut], "want": full(cut)}])]
        for p in range(cut, n):
            rows.append(s.step([{"id": "d", "tokens": [toks[p]], "want": [0]}]))
        s.end(["d"])
        _check(torch.cat(rows), want, dtype, f"{name} decode {n}")
    toks, want = prompts[150], _oracle(models, name, prompts[150])
    rows, at = [], 0
    for size in (2, 3, 64, 2, 5, 1, 1, 40, 2, 30):
        rows.append(s.step([{"id": "c", "tokens": toks[at:at + size], "want": full(size)}]))
        at += size
    assert at == 150
    s.end(["c"])
    _check(torch.cat(rows), want, dtype, f"{name} portions")
    plan = {"a": prompts[150], "b": prompts[13], "c": prompts[2], "d": H.prompt(70, V, 70), "e": H.prompt(31, V, 31)}
    cuts = {"a": [64, 2, 1, 1, 50, 1, 31], "b": [1, 1, 1, 5, 5], "c": [2], "d": [3, 60, 1, 1, 1, 1, 1, 1, 1],
            "e": [30, 1]}
    order = [["a", "b", "c", "d"], ["a", "b", "d"], ["a", "b", "d", "e"], ["a", "b", "d", "e"], ["a", "b", "d"],
             ["a", "d"], ["a", "d"], ["d"], ["d"]]
    at = {k: 0 for k in plan}
    idx = {k: 0 for k in plan}
    got = {k: [] for k in plan}
    for live in order:
        entries, ends = [], []
        for r in live:
            n = cuts[r][idx[r]]
            entries.append({"id": r, "tokens": plan[r][at[r]:at[r] + n], "want": full(n)})
            at[r] += n
            idx[r] += 1
            if at[r] == len(plan[r]):
                ends.append(r)
        out = s.step(entries)
        o = 0
        for e in entries:
            got[e["id"]].append(out[o:o + len(e["tokens"])])
            o += len(e["tokens"])
        s.end(ends)
    for r, toks in plan.items():
        assert at[r] == len(toks)
        _check(torch.cat(got[r]), _oracle(models, name, toks), dtype, f"{name} mixed {r}")


def test_long_decoding_and_far_tokens(models):
    """330 tokens, 320 of them decoded one by one, with sharp attention and memories that hardly forget; and a change
    of the FIRST token still moves the last logits by what the oracle says."""
    cfg, _, folder = models["far"]
    s = H.open_session(folder, "float32", max_tokens=768, max_requests=2)
    V = cfg["vocab"]
    toks = H.prompt(330, V, 9)
    other = [(toks[0] + 1) % V] + toks[1:]
    last = {}
    for rid, seq in (("x", toks), ("y", other)):
        s.step([{"id": rid, "tokens": seq[:10], "want": []}])
        for p in range(10, 329):
            s.step([{"id": rid, "tokens": [seq[p]], "want": []}])
        last[rid] = s.step([{"id": rid, "tokens": [seq[329]], "want": [0]}])[0].cpu().double()
        s.end([rid])
    wx, wy = _oracle(models, "far", toks)[329], _oracle(models, "far", other)[329]
    assert H.rel_err(last["x"][None], wx[None]).item() < 2 * H.TOL["float32"]
    assert H.rel_err(last["y"][None], wy[None]).item() < 2 * H.TOL["float32"]
    moved, want_moved = last["x"] - last["y"], wx - wy
    assert want_moved.abs().max() > 1e-3, "the test's weights do not carry the first token this far"
    assert (moved - want_moved).abs().max() < 0.05 * want_moved.abs().max() + 2e-5


def test_sharp_attention_sees_every_key(models):
    """With the sharp scale a query's output is mostly one key's value, wherever it is: every row of a 300-token prompt
    must match, as a whole and when the tail is fed in portions and single tokens across the run border of the pool."""
    cfg, _, folder = models["far"]
    s = H.open_session(folder, "float32", max_tokens=512, max_requests=2)
    toks = H.prompt(300, cfg["vocab"], 3)
    want = _oracle(models, "far", toks)
    got = s.step([{"id": "w", "tokens": toks, "want": list(range(300))}])
    s.end(["w"])
    _check(got, want, "float32", "sharp whole")
    rows, at = [], 0
    for size in [120, 7, 1, 1, 2, 125] + [1] * 10 + [34]:
        rows.append(s.step([{"id": "p", "tokens": toks[at:at + size], "want": list(range(size))}]))
        at += size
    assert at == 300
    _check(torch.cat(rows), want, "float32", "sharp portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_engine_greedy_generation(models, dtype):
    from semi_pd_b200.configs import ServerArgs
    from semi_pd_b200.semi_pd_scheduler import SemiPDEngine
    cfg, weights, folder = models["mixed"]
    V, n_new = cfg["vocab"], 24
    sa = ServerArgs(model_path=folder, dtype=dtype, load_format="auto", max_total_tokens=4096,
                    max_running_requests=8, context_length=512, enable_semi_pd=True, cuda_graph_bs=[1, 2, 4, 8],
                    chunked_prefill_size=48, max_prefill_tokens=256)
    eng = SemiPDEngine(sa, gpu_id=0, prefill_sm_percent=50, decode_sm_percent=50)
    try:
        prompts = [H.prompt(n, V, seed=100 + n) for n in (5, 33, 120, 61, 2, 77)]
        rids = [eng.submit(p, n_new) for p in prompts]
        done = {r.rid: r for r in eng.wait(len(rids), timeout=120)}
    finally:
        eng.shutdown()
    margin_floor = 1e-3 if dtype == "float32" else 0.3
    for rid, p in zip(rids, prompts):
        out = done[rid].output_ids
        assert len(out) == n_new
        stepper = M.Stepper(cfg, weights)
        logits = stepper.feed(list(p))[-1]
        for t, tok in enumerate(out):
            top2 = logits.topk(2).values
            if float(top2[0] - top2[1]) < margin_floor:
                break  # a near tie: either token is a correct greedy choice; stop comparing this request
            assert tok == int(logits.argmax()), f"{rid}: token {t} differs from the oracle's greedy choice"
            logits = stepper.feed([tok])[-1]
