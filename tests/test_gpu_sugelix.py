"""Sugelix family on the GPU against the float64 oracle (oracle/sugelix_oracle.py): every mechanism alone through its
operator, then whole models through the serving path (ScheduleBatch → worker → kernels, decode through the captured
CUDA graphs) under every way of cutting and batching the same tokens, then greedy generation through the semi-PD
engine."""
import math

import pytest
import torch

from oracle import sugelix_oracle as S
from tests import rimidra_helpers as H
from tests import sugelix_helpers as C

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
@pytest.mark.parametrize("width,buckets,mp,mc", [(36, 13, 7, 11), (256, 251, 1, 1), (7, 1, 3, 5)])
def test_pair_embedding_keeps_the_previous_token(dtype, width, buckets, mp, mc):
    """Two requests fed in portions (one of a single token) and then decoded beside a padded row: the pair row of a
    portion's first token comes from the request's slot, a request that starts again in a used slot ignores it."""
    from semi_pd_b200 import ops
    dt = DT[dtype]
    V = 40
    g = torch.Generator().manual_seed(width)
    table, pair = torch.randn(V, width, generator=g).to(dt), torch.randn(buckets + 1, width, generator=g).to(dt)
    cfg = {"embedding": {"scale": 3.0, "bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}}
    W = {"embed": table, "bigram": pair}
    seqs = [torch.randint(0, V, (12,), generator=g).tolist(), torch.randint(0, V, (9,), generator=g).tolist()]
    want = [S.embed(cfg, W, s) for s in seqs]
    state = torch.full((6,), 17, dtype=torch.int32, device=DEV)  # stale tokens that position 0 must ignore
    slots = i64([4, 2])
    kw = dict(pair=pair.to(DEV), buckets=buckets, mul_prev=mp, mul_cur=mc, prev_state=state, req_pool_indices=slots)
    at = [0, 0]
    for n0, n1 in ((3, 1), (1, 2), (5, 4)):
        ids = seqs[0][at[0]:at[0] + n0] + seqs[1][at[1]:at[1] + n1]
        x = ops.embed_pair(table.to(DEV), i64(ids), 3.0, prefix_lens=i32(at), extend_lens=i32([n0, n1]),
                           extend_start_loc=i32([0, n0]), **kw)
        _close(x, torch.cat([want[0][at[0]:at[0] + n0], want[1][at[1]:at[1] + n1]]), torch.float32, f"portion {at}",
               tol32=1e-6)
        at = [at[0] + n0, at[1] + n1]
    assert state[4].item() == seqs[0][8] and state[2].item() == seqs[1][6]
    # decode: the two requests and a padded row (cache slot 0, length 1) that points at request 0's slot
    for step in range(2):
        ids = [seqs[0][at[0]], seqs[1][at[1]], 5]
        x = ops.embed_pair(table.to(DEV), i64(ids), 3.0, pair=pair.to(DEV), buckets=buckets, mul_prev=mp, mul_cur=mc,
                           prev_state=state, req_pool_indices=i64([4, 2, 4]), seq_lens=i64([at[0] + 1, at[1] + 1, 1]),
                           out_cache_loc=i64([9, 3, 0]))
        _close(x[:2], torch.stack([want[0][at[0]], want[1][at[1]]]), torch.float32, f"decode {step}", tol32=1e-6)
        _close(x[2], S.embed(cfg, W, [5])[0], torch.float32, "padded row", tol32=1e-6)
        at = [at[0] + 1, at[1] + 1]
    assert state[4].item() == seqs[0][at[0] - 1], "a padded row must not write the state"
    # slot 4 is used again by a new request
    x = ops.embed_pair(table.to(DEV), i64(seqs[1][:3]), 3.0, pair=pair.to(DEV), buckets=buckets, mul_prev=mp, mul_cur=mc,
                       prev_state=state, req_pool_indices=i64([4]), prefix_lens=i32([0]), extend_lens=i32([3]),
                       extend_start_loc=i32([0]))
    _close(x, want[1][:3], torch.float32, "slot used again", tol32=1e-6)
    plain = ops.embed_pair(table.to(DEV), i64(seqs[0]), 0.5)
    _close(plain, table.double()[seqs[0]] * 0.5, torch.float32, "no pair table", tol32=1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [36, 256, 1000])
def test_residual_update_and_tanh_norm(dtype, width):
    from semi_pd_b200 import ops
    dt = DT[dtype]
    g = torch.Generator().manual_seed(width)
    T = 7
    x, x0 = torch.randn(T, width, generator=g) * 3, torch.randn(T, width, generator=g) * 3
    vec = torch.randn(width, generator=g)
    a = torch.randn(T, width, generator=g).to(dt)
    w, b = (1 + 0.2 * torch.randn(width, generator=g)).to(dt), (0.3 * torch.randn(width, generator=g)).to(dt)
    xd = x.to(DEV)
    h = ops.residual_tanh_norm(xd, w.to(DEV), b.to(DEV), 0.37, a=a.to(DEV), x0=x0.to(DEV), vec=vec.to(DEV))
    x1 = x.double() + a.double() + x0.double() + vec.double()
    _close(xd, x1, torch.float32, "update", tol32=1e-6)
    _close(h, S.tanh_norm(x1, 0.37, w, b), dt, "norm after the update", tol32=2e-6, tol16=1e-2)
    h = ops.residual_tanh_norm(xd, w.to(DEV), b.to(DEV), 1.9)
    _close(h, S.tanh_norm(x1, 1.9, w, b), dt, "norm alone", tol32=2e-6, tol16=1e-2)
    ops.residual_tanh_norm(xd, None, None, 1.0, a=a.to(DEV))
    x2 = x1 + a.double()
    _close(xd, x2, torch.float32, "update alone", tol32=1e-6)
    rows = [5, 0, 6]
    h = ops.residual_tanh_norm(xd, w.to(DEV), b.to(DEV), 0.8, rows=i64(rows))
    _close(h, S.tanh_norm(x2[rows], 0.8, w, b), dt, "chosen rows", tol32=2e-6, tol16=1e-2)
    _close(xd, x2, torch.float32, "a read leaves the stream alone", tol32=1e-7)


def _table(rot, base, factor, n=600):
    f = S.rotary_frequencies({"dims": rot, "base": base, **({"scaling": {"factor": factor}} if factor else {})})
    ang = torch.arange(n, dtype=torch.float64)[:, None] * f[None]
    return torch.cat([ang.cos(), ang.sin()], -1).float().to(DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("paired", [True, False])
@pytest.mark.parametrize("heads,kvh,dk,dv,rot", [(4, 2, 16, 24, 8), (1, 1, 10, 6, 10), (8, 4, 64, 40, 64), (2, 1, 6, 4, 0),
                                                 (4, 2, 32, 16, 16), (2, 2, 128, 128, 128)])
def test_rotary_segments_bias_rotation_cache_write(dtype, paired, heads, kvh, dk, dv, rot):
    """q, k, v as slices of one wider row: biases, rotation of the first `rot` channels in either layout at positions
    far from 0, k and v scattered into cache pools, q into a dense buffer.  Sizes in whole 16-byte vectors take the
    vector kernel, the others the element kernel."""
    from semi_pd_b200 import ops
    dt = DT[dtype]
    T = 5
    g = torch.Generator().manual_seed(dk * 31 + dv + heads)
    sizes = [heads * dk, kvh * dk, kvh * dv]
    row = torch.randn(T, sum(sizes) + (8 if dk % 8 == 0 else 3), generator=g).to(dt)
    qb, kb, vb = (torch.randn(n, generator=g) for n in sizes)
    pos, loc = [0, 1, 77, 300, 599], [9, 2, 5, 11, 3]
    rd = row.to(DEV)
    q, k, v = rd[:, : sum(sizes)].split(sizes, -1)
    k_pool, v_pool = torch.zeros(12, kvh * dk, device=DEV, dtype=dt), torch.zeros(12, kvh * dv, device=DEV, dtype=dt)
    q_out = torch.empty(T, heads * dk, device=DEV, dtype=dt)
    table = _table(rot, 300.0, 2.0) if rot else None
    ops.rotary_segments([
        ops.rotary_segment(q, q_out, heads, dk, rot, bias=qb.to(DEV)),
        ops.rotary_segment(k, k_pool, kvh, dk, rot, bias=kb.to(DEV), to_pool=True),
        ops.rotary_segment(v, v_pool, kvh, dv, 0, bias=vb.to(DEV), to_pool=True),
    ], i64(pos), table, dt, loc=i64(loc), paired=paired)
    spec = {"dims": rot, "base": 300.0, "scaling": {"factor": 2.0}}
    layout = "pairs" if paired else "halves"
    rq, rk, rv = (t.double() for t in row[:, : sum(sizes)].split(sizes, -1))
    _close(q_out, S.rotate((rq + qb.double()).view(T, heads, dk), pos, spec, layout).reshape(T, -1), dt, "q", tol16=1e-2)
    _close(k_pool[loc], S.rotate((rk + kb.double()).view(T, kvh, dk), pos, spec, layout).reshape(T, -1), dt, "k", tol16=1e-2)
    _close(v_pool[loc], rv + vb.double(), dt, "v", tol16=1e-2)
    assert float(k_pool[0].abs().max()) == 0 and float(v_pool[1].abs().max()) == 0, "other slots stay untouched"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rotary_segments_strided_heads(dtype):
    """The rotated slice of a latent attention: every head's last channels, moved into a row of another head size, and
    one shared key slice written behind the latent columns of a cache row."""
    from semi_pd_b200 import ops
    dt = DT[dtype]
    T, Hh, dim, dr, rank = 4, 3, 6, 4, 10
    g = torch.Generator().manual_seed(1)
    q = torch.randn(T, Hh * (dim + dr), generator=g).to(dt)
    ckv = torch.randn(T, rank + dr, generator=g).to(dt)
    pos, loc = [3, 0, 41, 500], [2, 7, 1, 4]
    qd, cd = q.to(DEV), ckv.to(DEV)
    q_lat = torch.zeros(T, Hh * (rank + dr), device=DEV, dtype=dt)
    pool = torch.zeros(8, rank + dr, device=DEV, dtype=dt)
    ops.rotary_segments([
        ops.rotary_segment(qd[:, dim:], q_lat[:, rank:], Hh, dr, dr, src_head=dim + dr, dst_head=rank + dr),
        ops.rotary_segment(cd[:, rank:], pool[:, rank:], 1, dr, dr, to_pool=True),
    ], i64(pos), _table(dr, 100.0, None), dt, loc=i64(loc), paired=False)
    spec = {"dims": dr, "base": 100.0}
    want_q = S.rotate(q.double().view(T, Hh, dim + dr)[..., dim:], pos, spec, "halves")
    _close(q_lat.view(T, Hh, rank + dr)[..., rank:], want_q, dt, "query slices", tol16=1e-2)
    assert float(q_lat.view(T, Hh, rank + dr)[..., :rank].abs().max()) == 0
    _close(pool[loc][:, rank:], S.rotate(ckv.double()[:, None, rank:], pos, spec, "halves")[:, 0], dt, "key slice", tol16=1e-2)
    assert float(pool[:, :rank].abs().max()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,vdim", [(4, 24), (1, 6), (2, 96), (3, 130)])
def test_gate_and_difference_of_maps(dtype, heads, vdim):
    from semi_pd_b200 import ops
    dt = DT[dtype]
    T, n = 6, heads * vdim
    g = torch.Generator().manual_seed(n)
    att = (torch.randn(T, 2 * n, generator=g) * 2).to(dt)
    wide = torch.randn(T, n + 11, generator=g).to(dt)
    gate = torch.sigmoid(wide.double()[:, 5:5 + n])
    ad, gd = att.to(DEV), wide.to(DEV)[:, 5:5 + n]
    _close(ops.heads_gate(ad[:, :n], gd, heads, vdim), att.double()[:, :n] * gate, dt, "plain gate", tol16=1e-2)
    lam, eps, post = 0.63, 1e-5, 0.7
    d = (att.double()[:, :n] - lam * att.double()[:, n:]).view(T, heads, vdim)
    want = (S.unit_rms(d, eps) * post).reshape(T, n) * gate
    got = ops.heads_gate(ad[:, :n], gd, heads, vdim, a2=ad[:, n:], lam=lam, eps=eps, post=post)
    _close(got, want, dt, "difference at unit RMS", tol16=1e-2)


def test_routing_weights_are_a_softmax_over_the_chosen():
    from semi_pd_b200 import ops
    g = torch.Generator().manual_seed(0)
    for E, top in ((8, 2), (5, 3), (2, 1), (3, 3)):
        z = torch.randn(33, E, generator=g) * 4
        ids, w = ops.moe_route_scores(z.to(DEV), E, top, score_func="softmax", renormalize=True)
        idx, want = S.route(z.double(), top)
        order = ids.long().cpu().argsort(-1)
        assert torch.equal(ids.long().cpu().gather(-1, order), idx.sort(-1).values)
        _close(w.cpu().gather(-1, order), want.gather(-1, idx.argsort(-1)), torch.float32, f"{E} experts, top {top}", tol32=1e-5)


class _Paged:
    """Requests whose cache slots are scattered over a pool, for the attention operator alone."""

    def __init__(self, lens, slots=700, seed=0):
        g = torch.Generator().manual_seed(seed)
        perm = (torch.randperm(slots, generator=g) + 1).tolist()
        self.lens, self.rows, at = lens, [], 0
        self.r2t = torch.zeros(len(lens) + 2, max(lens) + 4, dtype=torch.int32)
        self.req = list(range(1, len(lens) + 1))  # request slots 1.. (0 stays unused)
        for r, n in zip(self.req, lens):
            self.rows.append(perm[at:at + n])
            self.r2t[r, :n] = torch.tensor(perm[at:at + n], dtype=torch.int32)
            at += n
        self.slots = slots + 1

    def pool(self, per_request, dt):
        """per_request: [n_r, row] tensors → a pool [slots, row] holding them at the requests' slots."""
        pool = torch.zeros(self.slots, per_request[0].shape[1], dtype=dt)
        for rows, t in zip(self.rows, per_request):
            pool[torch.tensor(rows)] = t.to(dt)
        return pool.to(DEV)


def _standout(q, k, i, j_in, j_out, h, g, gain=6.0):
    """Make query (i, head h) look at key j_in, and look even harder at j_out should it (wrongly) be visible."""
    d = q[i, h] / q[i, h].norm()
    q[i, h] = d * gain
    k[j_in, g] = d * gain
    if j_out >= 0:
        k[j_out, g] = d * gain * 2


ATTN_CASES = [
    # name, H, G, Gv, dk, dv, window, cap, sink, latent
    ("capped", 4, 2, 2, 16, 24, None, 3.0, False, False),
    ("capped-tiles", 8, 2, 2, 64, 64, None, 20.0, False, False),
    ("two-maps", 4, 2, 1, 16, 32, 9, None, False, False),
    ("two-maps-tiles", 8, 4, 2, 64, 128, 100, None, False, False),
    ("latent", 3, 1, 1, 14, 10, 12, None, True, True),
    ("latent-tiles", 4, 1, 1, 128, 64, 40, None, True, True),
    ("latent-wide-row", 4, 1, 1, 192, 128, 150, None, True, True),
    ("latent-long-row", 2, 1, 1, 640, 512, 20, None, True, True),
    ("one", 1, 1, 1, 6, 4, 1, None, True, False),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ATTN_CASES, ids=[c[0] for c in ATTN_CASES])
def test_attention_options(dtype, case):
    """Score cap, key heads that share value heads, values inside the key rows, window and sink: ragged portions and
    decoding over scattered slots.  Chosen queries look sharply at the key just inside their window (a key far back
    without one) while the key just outside is made to attract them twice as much."""
    from semi_pd_b200 import ops
    _, Hh, G, Gv, dk, dv, window, cap, sink, latent = case
    dt = DT[dtype]
    lens, pre = [260, 41, 1], [200, 0, 0]
    g = torch.Generator().manual_seed(dk + dv)
    pg = _Paged(lens, seed=dk)
    sinks = torch.randn(Hh, generator=g) * 2 + 2 if sink else None
    qs, ks, vs, wants = [], [], [], []
    for n, p0 in zip(lens, pre):
        q, k = torch.randn(n, Hh, dk, generator=g), torch.randn(n, G, dk, generator=g)
        v = k[..., :dv].clone() if latent else torch.randn(n, Gv, dv, generator=g)
        for i in (n - 1, p0 + (n - p0) // 2, p0):  # the decoded row, one inside the portion, the portion's first
            far = 0 if window is None else i - window + 1
            if far >= 0 and i > 0:
                _standout(q, k, i, far, far - 1 if window is not None else -1, Hh - 1, (Hh - 1) // (Hh // G))
        if latent:
            v = k[..., :dv].clone()
        q, k, v = q.to(dt), k.to(dt), v.to(dt)
        v_heads = v.double()[:, [gg % Gv for gg in range(G)]]
        wants.append(S.softmax_attention(q.double(), k.double(), v_heads, 0.4, window=window, cap=cap, sinks=sinks))
        qs.append(q), ks.append(k), vs.append(v)
    k_pool = pg.pool([k.reshape(k.shape[0], -1) for k in ks], dt)
    v_pool = k_pool if latent else pg.pool([v.reshape(v.shape[0], -1) for v in vs], dt)
    kw = dict(num_q_heads=Hh, num_kv_heads=G, head_dim=dk, v_dim=dv, sm_scale=0.4, window=window or -1,
              sinks=sinks.to(DEV) if sink else None, softcap=cap or 0.0, num_v_heads=Gv,
              v_slot_stride=dk if latent else 0)
    r2t, req = pg.r2t.to(DEV), i64(pg.req)
    ext = [n - p for n, p in zip(lens, pre)]
    q_ext = torch.cat([q[p:].reshape(n - p, -1) for q, n, p in zip(qs, lens, pre)]).to(DEV)
    want_ext = torch.cat([w[p:].reshape(n - p, -1) for w, n, p in zip(wants, lens, pre)])
    starts = [0, ext[0], ext[0] + ext[1]]
    for bound in (max(ext), 0):  # the tensor-core prefill kernel where it applies, and the CUDA-core one
        got = ops.attn_general(q_ext, k_pool, v_pool, r2t, req, prefix_lens=i32(pre), extend_lens=i32(ext),
                               extend_start_loc=i32(starts), max_extend_len=bound, **kw)
        _close(got, want_ext, dt, f"portions (bound {bound})", tol16=2e-2)
    q_dec = torch.stack([q[-1].reshape(-1) for q in qs]).to(DEV)
    got = ops.attn_general(q_dec, k_pool, v_pool, r2t, req, seq_lens=i64(lens), **kw)
    _close(got, torch.stack([w[-1].reshape(-1) for w in wants]), dt, "decoding", tol16=2e-2)


# =================================================================================================
# whole models through the serving path
# =================================================================================================
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, make in C.CONFIGS.items():
        cfg = make()
        weights = S.make_weights(cfg, seed=C.SEEDS[name], gain=2.0 if name == "far" else 1.0)
        folder = H.write_model(tmp_path_factory.mktemp(name), cfg, weights)
        out[name] = (cfg, weights, folder)
    return out


_oracle_cache = {}
CLOSE_CALL = 0.02  # 16-bit runs: a routing choice this close (relative to the largest logit) may go either way


def _oracle_full(models, name, tokens):
    key = (name, tuple(tokens))
    if key not in _oracle_cache:
        cfg, weights, _ = models[name]
        margins = []
        logits = S.forward(cfg, weights, list(tokens), margins=margins)
        least = torch.stack(margins).min(0).values if margins else torch.full((len(tokens),), float("inf"))
        _oracle_cache[key] = (logits, least)
    return _oracle_cache[key]


def _oracle(models, name, tokens):
    return _oracle_full(models, name, tokens)[0]


def _check(got, want, dtype, what, margin=None):
    """margin: per row the least routing margin of the oracle; in 16 bits rows with a close call are left out (no
    test rests on one), and there must be few of them."""
    err = H.rel_err(got, want)
    tol = H.TOL[dtype]
    if dtype == "float32":
        assert err.max().item() < tol, f"{what}: worst relative error {err.max().item():.3e} at row {int(err.argmax())}"
        return
    if margin is not None:
        sure = margin >= CLOSE_CALL
        if len(sure) >= 20:
            assert sure.float().mean().item() >= 0.5, f"{what}: the test's weights make too many close routing calls"
        err = err[sure]
        if err.numel() == 0:
            return
    # 16-bit: a sharp softmax between two close keys amplifies the rounding of a few rows
    assert err.median().item() < tol / 4, f"{what}: median {err.median().item():.3e}"
    assert err.max().item() < 3 * tol and (err > tol).float().mean().item() <= 0.02, \
        f"{what}: worst {err.max().item():.3e}, {(err > tol).sum()} rows off"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "ones", "wide"])
def test_residual_after_every_layer_run(models, name, dtype):
    cfg, weights, folder = models[name]
    s = H.open_session(folder, dtype, max_tokens=256, max_requests=2, cuda_graph=False)
    model = s.worker.model_runner.model
    got = {}
    model._layer_hook = lambda i, x: got.__setitem__(i, x.double().cpu())
    toks = H.prompt(19, cfg["vocab"], 19)
    s.step([{"id": "a", "tokens": toks, "want": []}])
    model._layer_hook = None
    _, want = S.forward(cfg, weights, toks, want_layers=True)
    assert len(got) == len(want) == len(S.layer_runs(cfg))
    for r, ref in enumerate(want):
        rel = ((got[r] - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt()).item()
        assert rel < (1e-5 if dtype == "float32" else 2e-2), f"layer run {r}: relative RMS error {rel:.3e}"


LENGTHS = (1, 2, 13, 150)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(C.CONFIGS))
def test_model_every_schedule(models, name, dtype):
    """Whole prompts, prompt + token-by-token decoding, portions of changing size down to two tokens, and mixed
    batches of unequal requests — each position against the whole-sequence oracle; all of it in one small pool,
    so request slots (with their previous tokens) and cache runs are reused throughout."""
    if name == "far" and dtype == "bfloat16":
        pytest.skip("the sharp configuration is a 32-bit test: 16-bit rounding flips its near-ties")
    cfg, _, folder = models[name]
    s = H.open_session(folder, dtype, max_tokens=640, max_requests=4)
    V = cfg["vocab"]
    prompts = {n: H.prompt(n, V, seed=n) for n in LENGTHS}
    full = lambda n: list(range(n))
    for n, toks in prompts.items():
        got = s.step([{"id": f"w{n}", "tokens": toks, "want": full(n)}])
        s.end([f"w{n}"])
        want, margin = _oracle_full(models, name, toks)
        _check(got, want, dtype, f"{name} whole {n}", margin)
    for n in (13, 150):
        toks, (want, margin) = prompts[n], _oracle_full(models, name, prompts[n])
        cut = n - 9
        rows = [s.step([{"id": "d", "tokens": toks[:cut], "want": full(cut)}])]
        for p in range(cut, n):
            rows.append(s.step([{"id": "d", "tokens": [toks[p]], "want": [0]}]))
        s.end(["d"])
        _check(torch.cat(rows), want, dtype, f"{name} decode {n}", margin)
    toks, (want, margin) = prompts[150], _oracle_full(models, name, prompts[150])
    rows, at = [], 0
    for size in (2, 3, 64, 2, 5, 1, 1, 40, 2, 30):
        rows.append(s.step([{"id": "c", "tokens": toks[at:at + size], "want": full(size)}]))
        at += size
    assert at == 150
    s.end(["c"])
    _check(torch.cat(rows), want, dtype, f"{name} portions", margin)
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
        want, margin = _oracle_full(models, name, toks)
        _check(torch.cat(got[r]), want, dtype, f"{name} mixed {r}", margin)


def test_long_decoding_and_far_tokens(models):
    """330 tokens, 320 of them decoded one by one across the cache's run borders, with sharp attention; and a change of
    the FIRST token (which only the windowless attention still sees) moves the last logits by what the oracle says."""
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
    """With the sharp weights a query's output is mostly one key's value, wherever it is inside its window: every row of
    a 300-token prompt must match, as a whole and when the tail is fed in portions and single tokens across the run
    border of the pool."""
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
        stepper = S.Stepper(cfg, weights)
        logits = stepper.feed(list(p))[-1]
        for t, tok in enumerate(out):
            top2 = logits.topk(2).values
            if float(top2[0] - top2[1]) < margin_floor:
                break  # a near tie: either token is a correct greedy choice; stop comparing this request
            assert tok == int(logits.argmax()), f"{rid}: token {t} differs from the oracle's greedy choice"
            logits = stepper.feed([tok])[-1]
