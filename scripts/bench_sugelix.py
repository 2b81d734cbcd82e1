"""Sugelix beside Llama and Rimidra with experts (the closest family: general softmax attention over an fp32 stream,
routed experts with a shared one) at equal size: whole-model prefill / decode throughput through the worker
(ScheduleBatch → TpModelWorker, decode through the captured CUDA graphs) and the per-kernel times of the mechanisms the
family adds, each beside the like kernel of the existing paths, with the fraction of the measured roofline.  Random
weights, synthetic tokens.  `bench.py --family sugelix` runs this; stand-alone:
python scripts/bench_sugelix.py [--sizes s,m] [--out FILE]."""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import bench_rimidra as BR  # noqa: E402  (sizes, timing helpers, the two models set beside this one)

SIZES = {
    # the Rimidra / Llama shape of the same name, plus this family's own sizes: the latents and the rotated slice
    name: dict(z, kv_rank=128, rot_dim=64, q_rank=z["width"] // 2) for name, z in BR.SIZES.items()
}
VOCAB = BR.VOCAB


def sugelix_config(z):
    """Eight layer runs: capped attention, two passes over (latent attention, two-map attention, capped attention),
    then latent attention; every layer with routed experts and a shared one."""
    from semi_pd_b200.configs import _sugelix_config
    H, G, D = z["heads"], z["kv_heads"], z["dim"]
    mlp = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}, "expert": {"ff": z["eff"], "limit": 7.0},
           "shared": {"ff": z["eff"], "limit": 7.0}}
    capped = {"type": "attention", "mlp": mlp,
              "mixer": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "softcap": 30.0,
                        "rot": {"dims": D, "base": 1e6}}}
    two = {"type": "attention_2", "mlp": mlp,
           "mixer": {"heads": H // 2, "kv_heads": max(G // 2, 1), "dim": D // 2, "vdim": D, "scale": (D // 2) ** -0.5,
                     "diff": 0.4, "mask": {"size": z["window"]},
                     "rot": {"dims": D // 2, "base": 1e5, "scaling": {"factor": 8.0}}}}
    latent = {"type": "latent_attention", "mlp": mlp,
              "mixer": {"heads": H, "dim": D, "rot_dim": z["rot_dim"], "vdim": D, "q_rank": z["q_rank"],
                        "kv_rank": z["kv_rank"], "scale": (D + z["rot_dim"]) ** -0.5, "mask": {"size": z["window"]},
                        "rot": {"dims": z["rot_dim"], "base": 1e4}}}
    cfg = {"architecture": "Sugelix", "vocab": VOCAB, "width": z["width"], "norm": {"eps": 1e-6},
           "embedding": {"scale": 12.0, "bigram": {"buckets": 8191, "mul_prev": 31, "mul_cur": 17}},
           "layers": [capped, latent, two, capped, latent], "loop": {"start": 1, "stop": 4, "times": 2}, "context": 8192}
    return _sugelix_config("sugelix-bench", cfg)


def kernel_table(z, flush):
    """Per-kernel time of this family's mechanisms and of the like kernels of the existing paths."""
    from semi_pd_b200 import ops
    from semi_pd_b200.rimidra import _rotary_table
    hbm, tf, _ = BR.peaks()
    dev, bf = "cuda", torch.bfloat16
    H, G, D, Wd = z["heads"], z["kv_heads"], z["dim"], z["width"]
    R, Dr, Wn = z["kv_rank"], z["rot_dim"], z["window"]
    n_req, L, B = 4, 2048, 64
    T = n_req * L
    rows = []

    def add(name, like, ms, flops=None, bytes_=None):
        r = {"kernel": name, "like": like, "ms": ms}
        if flops is not None:
            r["tflops"] = flops / ms / 1e9
            r["frac_of_peak"] = r["tflops"] / tf
            r["peak"] = "bf16 tensor (measured)"
        if bytes_ is not None:
            r["gbs"] = bytes_ / ms / 1e6
            r["frac_of_peak"] = r["gbs"] / hbm
            r["peak"] = "hbm (measured)"
        rows.append(r)

    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    rpi = torch.arange(n_req, device=dev, dtype=torch.int64)
    pre, ext, start = i32([0] * n_req), i32([L] * n_req), i32([r * L for r in range(n_req)])
    rpd = torch.arange(B, device=dev, dtype=torch.int64)
    sl = torch.full((B,), L, dtype=torch.int64, device=dev)
    ev = lambda fn: BR.event_ms(fn, flush=flush)
    slots = T + 256
    r2t = torch.zeros(n_req + 64, L + 64, dtype=torch.int32, device=dev)
    for r in range(n_req):
        r2t[r, :L] = torch.arange(1 + r * L, 1 + (r + 1) * L, device=dev, dtype=torch.int32)
    r2d = torch.randint(1, slots, (B + 1, L + 64), device=dev, dtype=torch.int32)
    causal = sum(i + 1 for i in range(L)) * n_req
    windowed = sum(min(i + 1, Wn) for i in range(L)) * n_req

    def attention(tag, like, Hq, Gk, Gv, dk, dv, window, pairs, latent=False, **kw):
        """prefill (FLOPs of the visible pairs) and decode (bytes of the visible keys and values, once per group)."""
        kp = torch.randn(slots, Gk, dk, device=dev, dtype=bf)
        vp = kp if latent else torch.randn(slots, Gv, dv, device=dev, dtype=bf)
        q = torch.randn(T, Hq * dk, device=dev, dtype=bf)
        qd = torch.randn(B, Hq * dk, device=dev, dtype=bf)
        args = dict(num_q_heads=Hq, num_kv_heads=Gk, head_dim=dk, v_dim=dv, sm_scale=dk ** -0.5, window=window,
                    num_v_heads=Gv, v_slot_stride=dk if latent else 0, **kw)
        ms = ev(lambda: ops.attn_general(q, kp, vp, r2t, rpi, prefix_lens=pre, extend_lens=ext, extend_start_loc=start,
                                         max_extend_len=L, **args))
        add(f"{tag}, prefill {n_req}x{L} ({Hq}/{Gk}x{dk}/{dv})", like + (" prefill" if like else ""), ms,
            flops=2.0 * Hq * (dk + dv) * pairs)
        seen = L if window <= 0 else min(L, window)
        ms = ev(lambda: ops.attn_general(qd, kp, vp, r2d, rpd, seq_lens=sl, **args))
        add(f"{tag}, decode B={B} ctx {L}", like + (" decode" if like else ""), ms,
            bytes_=B * seen * (Gk * dk + (0 if latent else Gv * dv)) * 2)

    # ---- the three attentions, each beside the general attention of the like shape without the new option ----------------
    attention("attn_general capped", "", H, G, G, D, D, -1, causal, softcap=30.0)
    attention("attn_general", "like: capped attention", H, G, G, D, D, -1, causal)
    attention("attn_general two maps over shared values", "", H, G, max(G // 2, 1), D // 2, D, Wn, windowed)
    attention("attn_general one map, own values", "like: two maps", H, G, G, D // 2, D, Wn, windowed)
    sink = torch.zeros(H, device=dev)
    attention("attn_general latent row (keys = row, values = its latent columns)", "", H, 1, 1, R + Dr, R, Wn, windowed,
              latent=True, sinks=sink)
    attention("attn_general one shared key/value head", "like: latent row", H, 1, 1, R, R, Wn, windowed, sinks=sink)
    # ---- bias + rotation + cache write over segments, beside the fixed-layout kernel ------------------------------------
    sizes = [H * D, G * D, G * D]
    wide = torch.randn(T, sum(sizes) + H * D, device=dev, dtype=bf)
    q, k, v = wide[:, : sum(sizes)].split(sizes, -1)
    qb, kb, vb = (torch.randn(n, device=dev) for n in sizes)
    kp, vp = torch.zeros(slots, G * D, device=dev, dtype=bf), torch.zeros(slots, G * D, device=dev, dtype=bf)
    q_out = torch.empty(T, H * D, device=dev, dtype=bf)
    table = _rotary_table(D, 1e6, L + 64, dev)
    locs = torch.arange(1, T + 1, device=dev)
    pos = torch.arange(T, device=dev) % L
    moved = T * (H * D * 2 + G * D * 2 + G * D * 2) * 2
    for paired in (True, False):
        segs = [ops.rotary_segment(q, q_out, H, D, D, bias=qb), ops.rotary_segment(k, kp, G, D, D, bias=kb, to_pool=True),
                ops.rotary_segment(v, vp, G, D, 0, bias=vb, to_pool=True)]
        ms = ev(lambda: ops.rotary_segments(segs, pos, table, bf, loc=locs, paired=paired))
        add(f"rotary_segments q/k/v {'pairs' if paired else 'halves'} {T}x({H}+{G}+{G})x{D}", "", ms, bytes_=moved)
    ms = ev(lambda: ops.rotary_bias_store(q, k, v, qb, kb, kp.view(slots, G, D), vp.view(slots, G, D), locs, pos, table, D,
                                          H, G, D, D))
    add(f"rotary_bias_store {T}x({H}+{G}+{G})x{D}", "like: rotation + cache write", ms, bytes_=moved)
    # ---- row kernels -----------------------------------------------------------------------------------------------------
    x32, x0 = torch.randn(T, Wd, device=dev), torch.randn(T, Wd, device=dev)
    a = torch.randn(T, Wd, device=dev, dtype=bf)
    w1, b1 = torch.ones(Wd, device=dev, dtype=bf), torch.zeros(Wd, device=dev, dtype=bf)
    ms = ev(lambda: ops.residual_tanh_norm(x32, w1, b1, 0.5, a=a))
    add(f"residual_tanh_norm {T}x{Wd}", "", ms, bytes_=T * Wd * (4 + 4 + 2 + 2))
    vec = torch.zeros(Wd, device=dev)
    ms = ev(lambda: ops.residual_tanh_norm(x32, w1, b1, 0.5, a=a, x0=x0, vec=vec))
    add(f"residual_tanh_norm opening a pass {T}x{Wd}", "", ms, bytes_=T * Wd * (4 + 4 + 4 + 2 + 2))
    ms = ev(lambda: ops.residual_rmsnorm(x32, w1, 1e-6, a=a))
    add(f"residual_rmsnorm {T}x{Wd}", "like: norm", ms, bytes_=T * Wd * (4 + 4 + 2 + 2))
    ids = torch.randint(0, VOCAB, (T,), device=dev)
    emb, pair = torch.randn(VOCAB, Wd, device=dev, dtype=bf), torch.randn(8192, Wd, device=dev, dtype=bf)
    prev = torch.zeros(n_req + 1, dtype=torch.int32, device=dev)
    ms = ev(lambda: ops.embed_pair(emb, ids, 12.0, pair=pair, buckets=8191, mul_prev=31, mul_cur=17, prev_state=prev,
                                   req_pool_indices=rpi, prefix_lens=pre, extend_lens=ext, extend_start_loc=start))
    add(f"embed_pair {T}x{Wd}", "", ms, bytes_=T * Wd * (2 + 2 + 4))
    ms = ev(lambda: ops.embed_f32(emb, ids))
    add(f"embed_f32 {T}x{Wd}", "like: embedding", ms, bytes_=T * Wd * 6)
    att = torch.randn(T, 2 * H * D, device=dev, dtype=bf)
    gate = wide[:, sum(sizes):]
    ms = ev(lambda: ops.heads_gate(att[:, : H * D], gate, H, D))
    add(f"heads_gate {T}x{H * D}", "", ms, bytes_=T * H * D * 2 * 3)
    ms = ev(lambda: ops.heads_gate(att[:, : H * D], gate, H, D, a2=att[:, H * D:], lam=0.6, eps=1e-6, post=0.6))
    add(f"heads_gate difference of maps {T}x{H * D}", "", ms, bytes_=T * H * D * 2 * 4)
    o32 = torch.randn(T, H * D, device=dev)
    ms = ev(lambda: ops.headnorm_gate(o32, gate, H, D, 1e-6, gate_act="sigmoid"))
    add(f"headnorm_gate {T}x{H * D}", "like: head norm + gate", ms, bytes_=T * H * D * (4 + 2 + 2))
    return rows


def run(sizes=("s", "m"), out=None, kernels=True):
    torch.cuda.set_device(0)
    flush = torch.zeros(160 << 20, dtype=torch.uint8, device="cuda")  # > L2, written between timed launches
    hbm, tf, src = BR.peaks()
    res = {"peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src},
           "timing": "CUDA events, 3 warm-up launches, 160 MB written between timed launches", "sizes": {}}
    for name in sizes:
        z = SIZES[name]
        entry = {"shape": z, "models": {}}
        for label, cfg in (("llama", BR.llama_config(z)), ("rimidra-moe", BR.rimidra_config(z, True)),
                           ("sugelix", sugelix_config(z))):
            entry["models"][label] = BR.model_throughput(cfg, n_prompts=4, prompt_len=2048, decode_bs=64, flush=flush)
            print(name, label, json.dumps(entry["models"][label]), file=sys.stderr, flush=True)
        if kernels:
            entry["kernels"] = kernel_table(z, flush)
            for r in entry["kernels"]:
                print(name, json.dumps(r), file=sys.stderr, flush=True)
        res["sizes"][name] = entry
    if out:
        with open(out, "w") as f:
            json.dump(res, f, indent=1)
    return res


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="s,m")
    ap.add_argument("--out", default="")
    ap.add_argument("--no-kernels", action="store_true")
    a = ap.parse_args()
    run(tuple(a.sizes.split(",")), a.out or None, not a.no_kernels)
