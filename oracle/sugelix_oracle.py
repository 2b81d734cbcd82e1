"""Plain float64 statement of the Sugelix design, one function per mechanism, over a whole sequence at once (no cache:
every query looks its keys up in the full list).  Slow on purpose; shares no code with the package.  Weights are a
dict by checkpoint name (any float dtype, read as float64), `cfg` is the parsed config.json.

Notation: u is a sublayer's (normed) input [T, width]; H query heads, G key/value heads, dk key size, dv value size
per head; p is a token's position in its sequence, counted from 0.
"""
import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64
SWISH_SLOPE = 1.702  # the expert's sigmoid slope: fixed by the design


def f64(t):
    return torch.as_tensor(t).to(F64)


# ---- small pieces --------------------------------------------------------------------------------
def unit_rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * f64(w)


def tanh_norm(x, alpha, w, b):
    """The layer norm of this design: no statistics, tanh(alpha x) w + b with a scalar alpha."""
    return torch.tanh(float(alpha) * x) * f64(w) + f64(b)


def soft_cap(z, cap):
    return cap * torch.tanh(z / cap)


def linear(x, w, b=None):
    y = x @ f64(w).T
    return y if b is None else y + f64(b)


# ---- embedding -------------------------------------------------------------------------------------
def bigram_rows(tokens: List[int], buckets: int, mul_prev: int, mul_cur: int) -> List[int]:
    """Row of the pair table for every token: (previous · mul_prev + current · mul_cur) mod buckets, and the row
    after the last bucket for a sequence's first token."""
    return [buckets if i == 0 else (tokens[i - 1] * mul_prev + t * mul_cur) % buckets for i, t in enumerate(tokens)]


def embed(cfg, W, tokens):
    e = cfg["embedding"]
    x = f64(W["embed"])[torch.tensor(tokens)] * float(e["scale"])
    bg = e.get("bigram")
    if bg:
        rows = bigram_rows(tokens, int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"]))
        x = x + f64(W["bigram"])[torch.tensor(rows)]
    return x


# ---- rotary positions ------------------------------------------------------------------------------------
def rotary_frequencies(rot):
    dims = int(rot["dims"])
    i = torch.arange(dims // 2, dtype=F64)
    f = torch.pow(torch.tensor(float(rot["base"]), dtype=F64), -2.0 * i / dims)
    scaling = rot.get("scaling")
    return f / float(scaling["factor"]) if scaling else f


def rotate(x, positions, rot, layout):
    """x [T, heads, d]; the first rot.dims channels of every head turn by p · f_i, the rest pass.  layout "pairs":
    channel 2 i with 2 i + 1; layout "halves": channel i with i + dims / 2."""
    dims = int(rot["dims"])
    if dims == 0:
        return x
    ang = f64(positions)[:, None] * rotary_frequencies(rot)[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    if layout == "pairs":
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        turned = torch.stack([a * c - b * s, b * c + a * s], dim=-1).flatten(-2)
    else:
        a, b = x[..., : dims // 2], x[..., dims // 2: dims]
        turned = torch.cat([a * c - b * s, b * c + a * s], dim=-1)
    return torch.cat([turned, x[..., dims:]], dim=-1)


# ---- softmax attention -----------------------------------------------------------------------------------
def softmax_attention(q, k, v, scale, window=None, cap=None, sinks=None):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] of one whole sequence.  Query t sees keys j <= t, with a window only
    those with t - j < window.  Scores (q · k) scale, optionally capped by cap · tanh(· / cap).  sinks [H]: one more
    term exp(sink_h) in the denominator that carries no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    kh, vh = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)  # head h reads group h // (H / G)
    s = torch.einsum("thd,jhd->htj", q, kh) * scale
    if cap:
        s = soft_cap(s, cap)
    t, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (j <= t) if window is None else ((j <= t) & (t - j < window))
    s = s.masked_fill(~seen[None], float("-inf"))
    m = s.max(dim=-1, keepdim=True).values
    if sinks is not None:
        m = torch.maximum(m, f64(sinks)[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sinks is not None:
        den = den + torch.exp(f64(sinks)[:, None, None] - m)
    return torch.einsum("htj,jhv->thv", e / den, vh)


# ---- the three mixers ------------------------------------------------------------------------------------
def capped_attention_mixer(u, W, p, m, positions):
    """Grouped-query attention with biased projections, rotation in pairs, capped scores, no window, and a sigmoid
    gate on the concatenated heads."""
    T = u.shape[0]
    H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = linear(u, W[p + "q"], W[p + "q.b"]).view(T, H, dk)
    k = linear(u, W[p + "k"], W[p + "k.b"]).view(T, G, dk)
    v = linear(u, W[p + "v"], W[p + "v.b"]).view(T, G, dv)
    q, k = rotate(q, positions, m["rot"], "pairs"), rotate(k, positions, m["rot"], "pairs")
    window = (m.get("mask") or {}).get("size")
    o = softmax_attention(q, k, v, float(m["scale"]), window=window, cap=m.get("softcap"))
    o = o.reshape(T, H * dv) * torch.sigmoid(linear(u, W[p + "g"]))
    return linear(o, W[p + "o"])


def difference_weight(W, p, diff):
    return (math.exp(float((f64(W[p + "lq1"]) * f64(W[p + "lk1"])).sum()))
            - math.exp(float((f64(W[p + "lq2"]) * f64(W[p + "lk2"])).sum())) + diff)


def difference_attention_mixer(u, W, p, m, positions, eps):
    """Two softmax maps per head over the same values; the second is subtracted with one learned weight for the
    layer, the difference is brought to unit RMS per head and scaled by (1 - diff)."""
    T = u.shape[0]
    H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    diff = float(m["diff"])
    q = linear(u, W[p + "q"], W[p + "q.b"]).view(T, H, 2, dk)
    k = linear(u, W[p + "k"], W[p + "k.b"]).view(T, G, 2, dk)
    v = linear(u, W[p + "v"], W[p + "v.b"]).view(T, G, dv)
    window = (m.get("mask") or {}).get("size")
    maps = []
    for j in range(2):
        qj = rotate(q[:, :, j], positions, m["rot"], "halves")
        kj = rotate(k[:, :, j], positions, m["rot"], "halves")
        maps.append(softmax_attention(qj, kj, v, float(m["scale"]), window=window, cap=m.get("softcap")))
    o = maps[0] - difference_weight(W, p, diff) * maps[1]
    o = unit_rms(o, eps) * (1.0 - diff)
    o = o.reshape(T, H * dv) * torch.sigmoid(linear(u, W[p + "g"]))
    return linear(o, W[p + "o"])


def latent_attention_mixer(u, W, p, m, positions, eps):
    """Queries and keys/values through low-rank latents; every head's key is an unrotated part lifted from the latent
    plus one rotated part that all heads share; a window and a sink."""
    T = u.shape[0]
    H, dk, dr, dv, rank = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    cq = rms_norm(linear(u, W[p + "dq"]), W[p + "dq.norm"], eps)
    q = linear(cq, W[p + "uq"]).view(T, H, dk + dr)
    down = linear(u, W[p + "dkv"])
    c = rms_norm(down[:, :rank], W[p + "dkv.norm"], eps)
    rot = dict(m["rot"], dims=dr)
    k_rot = rotate(down[:, rank:].view(T, 1, dr), positions, rot, "halves")
    q_rot = rotate(q[..., dk:], positions, rot, "halves")
    k = torch.cat([linear(c, W[p + "uk"]).view(T, H, dk), k_rot.expand(T, H, dr)], dim=-1)
    v = linear(c, W[p + "uv"]).view(T, H, dv)
    qq = torch.cat([q[..., :dk], q_rot], dim=-1)
    window = (m.get("mask") or {}).get("size")
    o = softmax_attention(qq, k, v, float(m["scale"]), window=window, sinks=f64(W[p + "sink"]) if p + "sink" in W else None)
    o = o.reshape(T, H * dv) * torch.sigmoid(linear(u, W[p + "g"]))
    return linear(o, W[p + "o"])


# ---- feed-forward ------------------------------------------------------------------------------------------
def clamped_expert(h, W, p, limit):
    g = torch.clamp(linear(h, W[p + "gate"]), max=limit)
    u = torch.clamp(linear(h, W[p + "up"]), min=-limit, max=limit)
    return linear(g * torch.sigmoid(SWISH_SLOPE * g) * (u + 1.0), W[p + "down"])


def route(z, top):
    """Router logits [T, E] → (chosen experts [T, top], weights = softmax over the chosen logits)."""
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def routing_margin(z, top):
    """Per token: how far the last chosen logit is above the first one left out, relative to the largest logit
    (inf when every expert is chosen) — small values mark choices that rounding may turn."""
    if top >= z.shape[-1]:
        return torch.full(z.shape[:-1], float("inf"), dtype=F64)
    val = torch.topk(z, top + 1, dim=-1).values
    return (val[..., top - 1] - val[..., top]) / z.abs().max(-1).values.clamp_min(1e-30)


def mixture(h, W, p, mlp, margins: Optional[list] = None):
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    z = linear(h, W[p + "router"])
    idx, w = route(z, top)
    if margins is not None:
        margins.append(routing_margin(z, top))
    y = torch.zeros(h.shape[0], f64(W[p + "e0.down"]).shape[0], dtype=F64)
    for e in range(E):
        share = (w * (idx == e)).sum(-1)  # the expert's weight per token, 0 where it was not chosen
        rows = share.nonzero().flatten()
        if len(rows):
            y[rows] += share[rows, None] * clamped_expert(h[rows], W, f"{p}e{e}.", float(mlp["expert"]["limit"]))
    if mlp.get("shared"):
        y = y + clamped_expert(h, W, p + "shared.", float(mlp["shared"]["limit"]))
    return y


# ---- the model -------------------------------------------------------------------------------------------
def layer_runs(cfg):
    """(layer index, pass number or None) in execution order: layers [start, stop) run `times` times in a row."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, None) for i in range(a)]
    for t in range(times):
        runs += [(i, t if i == a else None) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n)]


def forward(cfg, W, tokens, want_layers=False, margins: Optional[list] = None):
    """tokens of ONE sequence from position 0 → logits [T, vocab] (and the residual after every layer run).  margins:
    a list that receives routing_margin [T] of every feed-forward that runs."""
    eps = float(cfg["norm"]["eps"])
    positions = list(range(len(tokens)))
    x0 = embed(cfg, W, tokens)
    x = x0.clone()
    layers = []
    for i, opens in layer_runs(cfg):
        if opens is not None:
            if opens > 0:
                x = x + x0
            x = x + f64(W["loop.step"])[opens]
        spec, p = cfg["layers"][i], f"l{i}."
        u = tanh_norm(x, W[p + "norm1.alpha"], W[p + "norm1"], W[p + "norm1.b"])
        if spec["type"] == "attention":
            x = x + capped_attention_mixer(u, W, p + "mix.", spec["mixer"], positions)
        elif spec["type"] == "attention_2":
            x = x + difference_attention_mixer(u, W, p + "mix.", spec["mixer"], positions, eps)
        else:
            x = x + latent_attention_mixer(u, W, p + "mix.", spec["mixer"], positions, eps)
        if spec.get("mlp") is not None:
            u = tanh_norm(x, W[p + "norm2.alpha"], W[p + "norm2"], W[p + "norm2.b"])
            x = x + mixture(u, W, p + "mlp.", spec["mlp"], margins)
        layers.append(x.clone())
    h = tanh_norm(x, W["final.norm.alpha"], W["final.norm"], W["final.norm.b"])
    logits = linear(h, W["head"])
    return (logits, torch.stack(layers)) if want_layers else logits


class Stepper:
    """Token-by-token use of the whole-sequence statement: keeps the tokens fed so far and recomputes."""

    def __init__(self, cfg, W):
        self.cfg, self.W, self.tokens = cfg, W, []

    def feed(self, tokens):
        """→ logits of the tokens just fed [len(tokens), vocab]."""
        self.tokens += list(tokens)
        return forward(self.cfg, self.W, self.tokens)[-len(tokens):]


# ---- configurations and random checkpoints for the tests ----------------------------------------------------
def moe_mlp(experts, top, ff, limit=2.0, shared_ff=0, shared_limit=1.0):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared_ff:
        m["shared"] = {"ff": shared_ff, "limit": shared_limit}
    return m


def attention_spec(heads, kv_heads, dim, vdim, scale, rot_dims, base=10000.0, softcap=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
         "rot": {"dims": rot_dims, "base": base}}
    if softcap:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m, "mlp": mlp}


def difference_spec(heads, kv_heads, dim, vdim, scale, rot_dims, window, diff, base=10000.0, factor=None, mlp=None):
    rot = {"dims": rot_dims, "base": base}
    if factor:
        rot["scaling"] = {"factor": factor}
    return {"type": "attention_2", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff,
                      "mask": {"size": window}, "rot": rot}}


def latent_spec(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window, base=10000.0, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                      "scale": scale, "mask": {"size": window}, "rot": {"dims": rot_dim, "base": base}}}


def make_config(layers: List[dict], width, vocab, embed_scale=1.0, bigram=None, loop=None, eps=1e-6):
    """bigram: (buckets, mul_prev, mul_cur) or None; loop: (start, stop, times) or None."""
    cfg = {"architecture": "Sugelix", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "embedding": {"scale": embed_scale}, "layers": layers}
    if bigram:
        cfg["embedding"]["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def tensor_shapes(cfg) -> Dict[str, tuple]:
    H = cfg["width"]
    shapes = {"embed": (cfg["vocab"], H)}
    bg = cfg["embedding"].get("bigram")
    if bg:
        shapes["bigram"] = (bg["buckets"] + 1, H)
    if cfg.get("loop"):
        shapes["loop.step"] = (cfg["loop"]["times"], H)

    def norm(name):
        shapes.update({name: (H,), name + ".b": (H,), name + ".alpha": ()})

    for i, spec in enumerate(cfg["layers"]):
        p, m = f"l{i}.", spec["mixer"]
        norm(p + "norm1")
        nh, dk, dv = m["heads"], m["dim"], m["vdim"]
        if spec["type"] == "latent_attention":
            dr, rq, rk = m["rot_dim"], m["q_rank"], m["kv_rank"]
            shapes.update({p + "mix.dq": (rq, H), p + "mix.dq.norm": (rq,), p + "mix.uq": (nh * (dk + dr), rq),
                           p + "mix.dkv": (rk + dr, H), p + "mix.dkv.norm": (rk,), p + "mix.uk": (nh * dk, rk),
                           p + "mix.uv": (nh * dv, rk), p + "mix.sink": (nh,), p + "mix.g": (nh * dv, H),
                           p + "mix.o": (H, nh * dv)})
        else:
            g, n = m["kv_heads"], 2 if spec["type"] == "attention_2" else 1
            shapes.update({p + "mix.q": (n * nh * dk, H), p + "mix.q.b": (n * nh * dk,), p + "mix.k": (n * g * dk, H),
                           p + "mix.k.b": (n * g * dk,), p + "mix.v": (g * dv, H), p + "mix.v.b": (g * dv,),
                           p + "mix.g": (nh * dv, H), p + "mix.o": (H, nh * dv)})
            if n == 2:
                shapes.update({p + "mix." + s: (dk,) for s in ("lq1", "lk1", "lq2", "lk2")})
        mlp = spec.get("mlp")
        if mlp is None:
            continue
        norm(p + "norm2")
        for e in range(mlp["router"]["experts"]):
            ff = mlp["expert"]["ff"]
            shapes.update({f"{p}mlp.e{e}.gate": (ff, H), f"{p}mlp.e{e}.up": (ff, H), f"{p}mlp.e{e}.down": (H, ff)})
        shapes[p + "mlp.router"] = (mlp["router"]["experts"], H)
        if mlp.get("shared"):
            sf = mlp["shared"]["ff"]
            shapes.update({p + "mlp.shared.gate": (sf, H), p + "mlp.shared.up": (sf, H), p + "mlp.shared.down": (H, sf)})
    norm("final.norm")
    shapes["head"] = (cfg["vocab"], H)
    return shapes


def make_weights(cfg, seed=0, gain=1.0) -> Dict[str, torch.Tensor]:
    """Random checkpoint, rounded to bfloat16 like a stored one: projections N(0, gain² / fan_in) (routers three times
    that, so that choices are rarely close), embedding rows of unit scale after the multiplier, norm weights around
    1 with alpha around 0.6, biases, sinks and the difference vectors N(0, 0.3²)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if last == "alpha":
            t = 0.5 + 0.2 * torch.rand(shape, generator=g)
        elif len(shape) == 1 and last in ("norm", "norm1", "norm2"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif len(shape) == 1:
            t = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g) / float(cfg["embedding"]["scale"])
        elif name in ("bigram", "loop.step"):
            t = 0.5 * torch.randn(shape, generator=g)
        elif last == "router":
            t = 3.0 * torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        else:
            t = gain * torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16)
    return out
