"""Plain float64 statement of the Matepel design, one function per mechanism, token by token where the
design is recurrent.  Slow on purpose; shares no code with the package.  Weights are a dict by checkpoint
name (any float dtype, read as float64), `cfg` is the parsed config.json.

Notation: u is a sublayer's (normed) input [T, width]; H heads; dk key size, dv value size per head; the
residual is a set of `streams` copies X [streams, T, width] that every sublayer reads through a weighted
sum and writes back through a mixing matrix.
"""
import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def f64(t):
    return torch.as_tensor(t).to(F64)


# ---- small pieces --------------------------------------------------------------------------------
def unit_rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * f64(w)


def silu(z):
    return z * torch.sigmoid(z)


def log_sigmoid(z):
    return -torch.nn.functional.softplus(-z)


def soft_cap(z, cap):
    return cap * torch.tanh(z / cap)


# ---- the streams -----------------------------------------------------------------------------------
def streams_read(X, w_in):
    """X [S, T, width], w_in [S] → Σ_s w_in[s] X_s."""
    return torch.einsum("s,stc->tc", f64(w_in), X)


def streams_write(X, y, w_mix, w_out, mult):
    """new X_t = Σ_s w_mix[s, t] X_s + mult · w_out[t] · y, every new stream from the old ones."""
    return torch.einsum("sr,stc->rtc", f64(w_mix), X) + mult * f64(w_out)[:, None, None] * y[None]


# ---- rotary positions with a two-regime frequency scaling --------------------------------------------
def scaled_rotary_frequencies(dims, base, scaling):
    """f_i = base^(-2 i / dims); with scaling {factor, original, fast, slow}: channels that turn more than
    `fast` times within `original` positions keep f_i, channels that turn fewer than `slow` times get
    f_i / factor, a linear ramp (in channel index) in between.  → (frequencies [dims / 2], magnitude)."""
    i = torch.arange(dims // 2, dtype=F64)
    f = torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def channel_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(channel_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(channel_of(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half_partial(x, positions, dims, freqs, magnitude):
    """x [T, H, d]: channel i < dims / 2 is paired with channel i + dims / 2; channels >= dims pass."""
    ang = f64(positions)[:, None] * freqs[None, :]
    c, s = (ang.cos() * magnitude)[:, None, :], (ang.sin() * magnitude)[:, None, :]
    half = dims // 2
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


# ---- softmax attention whose denominator holds one more unit -------------------------------------------
def plus_one_softmax_attention(q, k, v, scale, first_position=0):
    """q [T, H, dk]; k [P + T, G, dk], v [P + T, G, dv] hold every position of the sequence; query t stands at
    position P + t and sees positions <= its own.  p_j = exp(s_j) / (1 + Σ exp(s_j))."""
    T, H, _ = q.shape
    G = k.shape[1]
    P = k.shape[0] - T
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for t in range(T):
        n = P + t + 1
        for h in range(H):
            g = h // (H // G)
            s = (k[:n, g] @ q[t, h]) * scale
            m = max(float(s.max()), 0.0)
            e = torch.exp(s - m)
            out[t, h] = (e[:, None] * v[:n, g]).sum(0) / (math.exp(-m) + e.sum())
    return out


# ---- recurrences -----------------------------------------------------------------------------------
def fixed_decay_recurrence(q, k, v, decay, S):
    """q, k [T, H, dk], v [T, H, dv], decay [H], S [H, dk, dv]: S <- decay_h S + k_t v_tᵀ, o_t = Sᵀ q_t (new S)."""
    o = torch.zeros(q.shape[0], q.shape[1], v.shape[2], dtype=F64)
    d = f64(decay)[:, None, None]
    for t in range(q.shape[0]):
        S = d * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


def matrix_memory_recurrence(q, k, v, i_log, f_log, S, n, m):
    """Exponentially gated matrix memory with a running maximum of the log gates.  q, k [T, H, dk], v [T, H, dv],
    i_log, f_log [T, H]; S [H, dk, dv], n [H, dk], m [H].
        m' = max(f + m, i);  S' = e^(f + m − m') S + e^(i − m') k vᵀ;  n' = e^(f + m − m') n + e^(i − m') k;
        o = S'ᵀ q / (max(|n' · q|, e^(−m')) + 1e-6)."""
    o = torch.zeros(q.shape[0], q.shape[1], v.shape[2], dtype=F64)
    for t in range(q.shape[0]):
        m_new = torch.maximum(f_log[t] + m, i_log[t])
        a, b = torch.exp(f_log[t] + m - m_new), torch.exp(i_log[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        m = m_new
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        o[t] = torch.einsum("hkv,hk->hv", S, q[t]) / den[:, None]
    return o, S, n, m


# ---- mixers ----------------------------------------------------------------------------------------
def lightning_mixer(u, W, p, mx, eps, state=None):
    """→ (output [T, width], state).  state: S [H, dk, dv] or None (a sequence's start)."""
    H, dk, dv = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
    T = u.shape[0]
    q = silu(u @ f64(W[p + "q"]).T).view(T, H, dk)
    k = silu(u @ f64(W[p + "k"]).T).view(T, H, dk)
    v = silu(u @ f64(W[p + "v"]).T).view(T, H, dv)
    S = torch.zeros(H, dk, dv, dtype=F64) if state is None else state
    o, S = fixed_decay_recurrence(q, k, v, mx["decay"], S)
    y = rms_norm(o.reshape(T, H * dv), W[p + "norm"], eps) * torch.sigmoid(u @ f64(W[p + "g"]).T)
    return y @ f64(W[p + "o"]).T, S


def rotary_attention_branch(u, W, p, mx, first_position=0, cache=None):
    """The softmax branch: biased q / k projections, values = the keys before rotation.  cache: (rotated keys,
    values) of the earlier positions or None."""
    H, G, dk = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"])
    T = u.shape[0]
    q = (u @ f64(W[p + "q"]).T + f64(W[p + "q.b"])).view(T, H, dk)
    k = (u @ f64(W[p + "k"]).T + f64(W[p + "k.b"])).view(T, G, dk)
    v = k
    rot = mx.get("rot")
    if rot:
        freqs, mag = scaled_rotary_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
        pos = torch.arange(first_position, first_position + T)
        q = rotate_half_partial(q, pos, int(rot["dims"]), freqs, mag)
        k = rotate_half_partial(k, pos, int(rot["dims"]), freqs, mag)
    if cache is not None:
        k, v = torch.cat([cache[0], k], 0), torch.cat([cache[1], v], 0)
    o = plus_one_softmax_attention(q, k, v, float(mx["scale"]))
    return o.reshape(T, -1) @ f64(W[p + "o"]).T + f64(W[p + "o.b"]), (k, v)


def matrix_memory_branch(u, W, p, mx, eps, state=None):
    H, dk, dv, cap = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"]), float(mx["gate_cap"])
    T = u.shape[0]
    q = (u @ f64(W[p + "q"]).T).view(T, H, dk) * dk ** -0.5
    k = (u @ f64(W[p + "k"]).T).view(T, H, dk)
    v = (u @ f64(W[p + "v"]).T).view(T, H, dv)
    i_log = soft_cap(u @ f64(W[p + "i"]).T + f64(W[p + "i.b"]), cap)
    f_log = log_sigmoid(soft_cap(u @ f64(W[p + "f"]).T + f64(W[p + "f.b"]), cap))
    if state is None:
        state = (torch.zeros(H, dk, dv, dtype=F64), torch.zeros(H, dk, dtype=F64), torch.zeros(H, dtype=F64))
    o, S, n, m = matrix_memory_recurrence(q, k, v, i_log, f_log, *state)
    y = unit_rms(o, eps).reshape(T, H * dv) * f64(W[p + "norm"]) * torch.sigmoid(u @ f64(W[p + "g"]).T)
    return y @ f64(W[p + "o"]).T, (S, n, m)


def parallel_mixer(u, W, p, mx, eps, first_position=0, state=None):
    cache, mem = state if state is not None else (None, None)
    left, cache = rotary_attention_branch(u, W, p + "left.", mx["left"], first_position, cache)
    right, mem = matrix_memory_branch(u, W, p + "right.", mx["right"], eps, mem)
    return float(mx["left_scale"]) * left + float(mx["right_scale"]) * right, (cache, mem)


# ---- feed-forward ------------------------------------------------------------------------------------
def clamped_gated_ff(u, W, p, mlp):
    limit = float(mlp["limit"])
    g = torch.clamp(u @ f64(W[p + "gate"]).T, max=limit)
    up = torch.clamp(u @ f64(W[p + "up"]).T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (up + 1.0)) @ f64(W[p + "down"]).T


# ---- the model -----------------------------------------------------------------------------------------
def new_state(cfg):
    return {"pos": 0, "layers": [None] * len(cfg["layers"])}


def forward(cfg, W, tokens, residuals: Optional[list] = None, state: Optional[dict] = None):
    """Logits [T, vocab] of `tokens` continuing `state` (None: a new sequence; updated in place).  `residuals`
    collects the residual (the sum of the streams) after every layer."""
    eps, mult = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    S = cfg.get("streams")
    if state is None:
        state = new_state(cfg)
    p0 = state["pos"]
    tok = torch.as_tensor(tokens, dtype=torch.long)
    x = rms_norm(f64(W["embed"])[tok], W["embed.norm"], eps)
    X = torch.stack([x] * (int(S) if S else 1), 0)
    for l, spec in enumerate(cfg["layers"]):
        p = f"l{l}."
        for q in (1, 2):
            if q == 2 and spec.get("mlp") is None:
                continue
            if S:
                w_in, w_mix, w_out = W[f"{p}hc{q}.in"], W[f"{p}hc{q}.mix"], W[f"{p}hc{q}.out"]
            else:
                w_in, w_mix, w_out = torch.ones(1), torch.ones(1, 1), torch.ones(1)
            u = rms_norm(streams_read(X, w_in), W[f"{p}norm{q}"], eps)
            if q == 2:
                y = clamped_gated_ff(u, W, p + "mlp.", spec["mlp"])
            elif spec["type"] == "lightning":
                y, state["layers"][l] = lightning_mixer(u, W, p + "mix.", spec["mixer"], eps, state["layers"][l])
            elif spec["type"] == "parallel":
                y, state["layers"][l] = parallel_mixer(u, W, p + "mix.", spec["mixer"], eps, p0, state["layers"][l])
            else:
                raise ValueError(spec["type"])
            X = streams_write(X, y, w_mix, w_out, mult)
        if residuals is not None:
            residuals.append(X.sum(0))
    state["pos"] = p0 + len(tok)
    return rms_norm(X.sum(0), W["final.norm"], eps) @ f64(W["head"]).T


class Stepper:
    """A sequence fed in portions: keeps the cache / state of every layer."""

    def __init__(self, cfg, W):
        self.cfg, self.W, self.state = cfg, W, new_state(cfg)

    def feed(self, tokens, residuals=None):
        return forward(self.cfg, self.W, tokens, residuals, self.state)


# ---- configurations and random checkpoints for the tests ----------------------------------------------------
def dense_mlp(ff, limit=1.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def lightning_spec(heads, dim, vdim, decay=None, mlp=None):
    decay = decay if decay is not None else [math.exp(-2.0 ** (-h)) for h in range(heads)]
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def parallel_spec(heads, kv_heads, dim, scale, rot_dims, r_heads, r_dim, r_vdim, base=10000.0, scaling=None,
                  gate_cap=10.0, left_scale=1.0, right_scale=1.0, mlp=None):
    rot = None
    if rot_dims:
        rot = {"dims": rot_dims, "base": base}
        if scaling is not None:
            rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "rot": rot}
    right = {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "gate_cap": gate_cap}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale,
                                          "right_scale": right_scale}, "mlp": mlp}


def make_config(layers: List[dict], width, vocab, streams=2, residual_mult=1.0, eps=1e-6):
    cfg = {"architecture": "Matepel", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "residual_mult": residual_mult, "layers": layers}
    if streams:
        cfg["streams"] = streams
    return cfg


def tensor_shapes(cfg) -> Dict[str, tuple]:
    Wd, S = int(cfg["width"]), cfg.get("streams")
    out = {"embed": (int(cfg["vocab"]), Wd), "embed.norm": (Wd,)}
    for l, spec in enumerate(cfg["layers"]):
        p, mx = f"l{l}.", spec["mixer"]
        out[p + "norm1"] = (Wd,)
        if spec["type"] == "lightning":
            H, dk, dv = mx["heads"], mx["dim"], mx["vdim"]
            out.update({p + "mix.q": (H * dk, Wd), p + "mix.k": (H * dk, Wd), p + "mix.v": (H * dv, Wd),
                        p + "mix.g": (H * dv, Wd), p + "mix.o": (Wd, H * dv), p + "mix.norm": (H * dv,)})
        else:
            a, b = mx["left"], mx["right"]
            H, G, dk = a["heads"], a["kv_heads"], a["dim"]
            out.update({p + "mix.left.q": (H * dk, Wd), p + "mix.left.q.b": (H * dk,), p + "mix.left.k": (G * dk, Wd),
                        p + "mix.left.k.b": (G * dk,), p + "mix.left.o": (Wd, H * dk), p + "mix.left.o.b": (Wd,)})
            H, dk, dv = b["heads"], b["dim"], b["vdim"]
            out.update({p + "mix.right.q": (H * dk, Wd), p + "mix.right.k": (H * dk, Wd), p + "mix.right.v": (H * dv, Wd),
                        p + "mix.right.g": (H * dv, Wd), p + "mix.right.o": (Wd, H * dv), p + "mix.right.norm": (H * dv,),
                        p + "mix.right.i": (H, Wd), p + "mix.right.i.b": (H,), p + "mix.right.f": (H, Wd),
                        p + "mix.right.f.b": (H,)})
        subs = [1]
        if spec.get("mlp") is not None:
            ff = spec["mlp"]["ff"]
            out.update({p + "norm2": (Wd,), p + "mlp.gate": (ff, Wd), p + "mlp.up": (ff, Wd), p + "mlp.down": (Wd, ff)})
            subs.append(2)
        if S:
            for q in subs:
                out.update({f"{p}hc{q}.in": (S,), f"{p}hc{q}.out": (S,), f"{p}hc{q}.mix": (S, S)})
    out.update({"final.norm": (Wd,), "head": (int(cfg["vocab"]), Wd)})
    return out


def make_weights(cfg, seed=0, gain=1.0) -> Dict[str, torch.Tensor]:
    """Random bfloat16 checkpoint: projections N(0, gain² / fan_in), norm weights around 1, biases N(0, 0.3²),
    forget-gate bias shifted up (a memory that lasts), stream coefficients around an identity-like mixing."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith(".mix") and ".hc" in name:
            t = torch.eye(shape[0]) * 0.8 + 0.2 / shape[0] + 0.1 * torch.randn(shape, generator=g)
        elif ".hc" in name:
            t = (1.0 / shape[0] if name.endswith(".in") else 1.0) + 0.2 * torch.randn(shape, generator=g)
        elif name.endswith("norm") or name.endswith("norm1") or name.endswith("norm2"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name.endswith(".f.b"):
            t = 2.0 + torch.randn(shape, generator=g)
        elif name.endswith(".b"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * gain / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16)
    return out
