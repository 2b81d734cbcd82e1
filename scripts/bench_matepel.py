"""Matepel beside Llama and Rimidra (the closest family: a fixed-decay recurrence and a general softmax attention over an
fp32 stream) at equal size: whole-model prefill / decode throughput through the worker (ScheduleBatch → TpModelWorker,
decode through the captured CUDA graphs) and the per-kernel times of the mechanisms the family adds, each beside the like
kernel of the existing paths, with the fraction of the measured roofline.  Random weights, synthetic tokens.
`bench.py --family matepel` runs this; stand-alone: python scripts/bench_matepel.py [--sizes s,m] [--out FILE]."""
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
    # the Rimidra / Llama shape of the same name, plus this family's own sizes: streams, memory-branch heads
    name: dict(z, streams=2, mem_heads=z["heads"], mem_dim=64, mem_vdim=128, rot=64) for name, z in BR.SIZES.items()
}
VOCAB = BR.VOCAB


def matepel_config(z):
    """Lightning and parallel layers alternating, every layer with its feed-forward, two streams."""
    from semi_pd_b200.configs import _matepel_config
    H, G, D = z["heads"], z["kv_heads"], z["dim"]
    mlp = {"kind": "dense", "ff": z["ff"], "limit": 7.0}
    lightning = {"type": "lightning", "mlp": mlp,
                 "mixer": {"heads": H, "dim": D, "vdim": D, "decay": [1.0 - 2.0 ** (-5 - 3 * h / H) for h in range(H)]}}
    parallel = {"type": "parallel", "mlp": mlp, "mixer": {
        "left": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5,
                 "rot": {"dims": z["rot"], "base": 5e5, "scaling": {"factor": 4.0, "original": 4096, "fast": 16.0, "slow": 2.0}}},
        "right": {"heads": z["mem_heads"], "dim": z["mem_dim"], "vdim": z["mem_vdim"], "gate_cap": 12.0},
        "left_scale": 0.75, "right_scale": 1.25}}
    cfg = {"architecture": "Matepel", "vocab": VOCAB, "width": z["width"], "norm": {"eps": 1e-6}, "residual_mult": 0.5,
           "streams": z["streams"], "layers": [lightning, parallel] * (z["layers"] // 2), "context": 8192}
    return _matepel_config("matepel-bench", cfg)


def kernel_table(z, flush):
    """Per-kernel time of this family's mechanisms and of the like kernels of the existing paths."""
    from semi_pd_b200 import ops
    from semi_pd_b200.matepel import scaled_rotary_table
    hbm, tf, _ = BR.peaks()
    dev, bf = "cuda", torch.bfloat16
    H, G, D, Wd, S = z["heads"], z["kv_heads"], z["dim"], z["width"], z["streams"]
    Hm, Dm, Vm = z["mem_heads"], z["mem_dim"], z["mem_vdim"]
    n_req, L, B = 4, 2048, 64
    T = n_req * L
    rows = []

    def add(name, like, ms, flops=None, bytes_=None, peak_tf=None):
        r = {"kernel": name, "like": like, "ms": ms}
        if flops is not None:
            r["tflops"] = flops / ms / 1e9
            r["frac_of_peak"] = r["tflops"] / (peak_tf or tf)
            r["peak"] = "cuda-core fp32" if peak_tf else "bf16 tensor (measured)"
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
    loc = torch.ones(B, dtype=torch.int64, device=dev)
    ev = lambda fn: BR.event_ms(fn, flush=flush)
    # ---- the gated matrix memory and the lightning recurrence, beside plain retention ---------------------------------
    state = torch.zeros(B + 1, Hm, Dm, Vm, device=dev)
    vec = torch.zeros(B + 1, ops.matrix_memory_vector_dim(Hm, Dm, Vm), device=dev)
    sizes = [Hm * Dm, Hm * Dm, Hm * Vm, Hm, Hm]
    x = torch.randn(T, sum(sizes) + 8 - 2 * Hm % 8, device=dev, dtype=bf)
    ib, fb = torch.zeros(Hm, device=dev), torch.full((Hm,), 3.0, device=dev)
    kw = dict(num_heads=Hm, head_dim=Dm, v_dim=Vm, i_bias=ib, f_bias=fb, cap=12.0, q_scale=Dm ** -0.5)
    parts = x[:, : sum(sizes)].split(sizes, -1)
    ms = ev(lambda: ops.matrix_memory(*parts, state, vec, rpi, prefix_lens=pre, extend_lens=ext, extend_start_loc=start, **kw))
    add(f"matrix_memory prefill {n_req}x{L} ({Hm}x{Dm}x{Vm})", "", ms, flops=4.0 * Hm * Dm * Vm * T, peak_tf=BR.FP32_CORE_TFLOPS)
    xd = torch.randn(B, x.shape[1], device=dev, dtype=bf)
    pd = xd[:, : sum(sizes)].split(sizes, -1)
    ms = ev(lambda: ops.matrix_memory(*pd, state, vec, rpd, seq_lens=sl, out_cache_loc=loc, **kw))
    add(f"matrix_memory decode B={B} ({Hm}x{Dm}x{Vm})", "", ms, bytes_=B * Hm * Dm * Vm * 4 * 2)
    # plain retention at the memory's own shape: the like kernel at equal size
    dec_m = torch.full((Hm,), 0.97, device=dev)
    ms = ev(lambda: ops.retention(parts[0], parts[1], parts[2], state, rpi, Hm, Dm, Vm, dec_m, None, 0, 1.0, prefix_lens=pre,
                                  extend_lens=ext, extend_start_loc=start))
    add(f"retention prefill {n_req}x{L} ({Hm}x{Dm}x{Vm})", "like: matrix_memory prefill", ms, flops=4.0 * Hm * Dm * Vm * T,
        peak_tf=BR.FP32_CORE_TFLOPS)
    ms = ev(lambda: ops.retention(pd[0], pd[1], pd[2], state, rpd, Hm, Dm, Vm, dec_m, None, 0, 1.0, seq_lens=sl,
                                  out_cache_loc=loc))
    add(f"retention decode B={B} ({Hm}x{Dm}x{Vm})", "like: matrix_memory decode", ms, bytes_=B * Hm * Dm * Vm * 4 * 2)
    state = torch.zeros(B + 1, H, D, D, device=dev)
    qkv = torch.randn(T, 3 * H * D, device=dev, dtype=bf)
    dec = torch.full((H,), 0.97, device=dev)
    rq, rk, rv = qkv.split(H * D, dim=-1)
    qkvd = torch.randn(B, 3 * H * D, device=dev, dtype=bf)
    for act, like in (("silu", ""), (None, "like: recurrence")):
        tag = "retention with SiLU at read" if act else "retention"
        ms = ev(lambda: ops.retention(rq, rk, rv, state, rpi, H, D, D, dec, None, 0, 1.0, prefix_lens=pre, extend_lens=ext,
                                      extend_start_loc=start, in_act=act))
        add(f"{tag} prefill {n_req}x{L} ({H}x{D})", like + (" prefill" if like else ""), ms, flops=4.0 * H * D * D * T,
            peak_tf=BR.FP32_CORE_TFLOPS)
        ms = ev(lambda: ops.retention(*qkvd.split(H * D, dim=-1), state, rpd, H, D, D, dec, None, 0, 1.0, seq_lens=sl,
                                      out_cache_loc=loc, in_act=act))
        add(f"{tag} decode B={B} ({H}x{D})", like + (" decode" if like else ""), ms, bytes_=B * H * D * D * 4 * 2)
    # ---- attention with one more unit in the denominator, beside the same attention without -----------------------------
    slots = T + 256
    r2t = torch.zeros(n_req + 64, L + 64, dtype=torch.int32, device=dev)
    for r in range(n_req):
        r2t[r, :L] = torch.arange(1 + r * L, 1 + (r + 1) * L, device=dev, dtype=torch.int32)
    kp, vp = torch.randn(slots, G, D, device=dev, dtype=bf), torch.randn(slots, G, D, device=dev, dtype=bf)
    qa = torch.randn(T, H * D, device=dev, dtype=bf)
    full = sum(i + 1 for i in range(L)) * n_req
    r2d = torch.randint(1, slots, (B + 1, L + 64), device=dev, dtype=torch.int32)
    qd2 = torch.randn(B, H * D, device=dev, dtype=bf)
    for sinks, tag, like in ((torch.zeros(H, device=dev), "attn_general with a unit sink", ""),
                             (None, "attn_general", "like: attention")):
        ms = ev(lambda: ops.attn_general(qa, kp, vp, r2t, rpi, H, G, D, D, D ** -0.5, sinks=sinks, prefix_lens=pre,
                                         extend_lens=ext, extend_start_loc=start, max_extend_len=L))
        add(f"{tag}, prefill {n_req}x{L} ({H}/{G}x{D})", like + (" prefill" if like else ""), ms, flops=4.0 * H * D * full)
        ms = ev(lambda: ops.attn_general(qd2, kp, vp, r2d, rpd, H, G, D, D, D ** -0.5, sinks=sinks, seq_lens=sl))
        add(f"{tag}, decode B={B} ctx {L}", like + (" decode" if like else ""), ms, bytes_=B * L * G * D * 2 * 2)
    # ---- bias + rotation + cache write, beside the plain cache write ---------------------------------------------------
    wide = torch.randn(T, H * D + G * D, device=dev, dtype=bf)
    qb, kb = torch.randn(H * D, device=dev), torch.randn(G * D, device=dev)
    table = scaled_rotary_table(z["rot"], 5e5, {"factor": 4.0, "original": 4096, "fast": 16.0, "slow": 2.0}, L + 64, dev)
    locs = torch.arange(1, T + 1, device=dev)
    pos = torch.arange(T, device=dev) % L
    ms = ev(lambda: ops.rotary_bias_store(wide[:, : H * D], wide[:, H * D:], None, qb, kb, kp, vp, locs, pos, table, z["rot"],
                                          H, G, D, D))
    add(f"rotary_bias_store {T}x({H}+{G})x{D}", "", ms, bytes_=T * (H * D * 2 + G * D) * 2 + T * G * D * 2 * 2)
    kk, vv = wide[:, H * D:].view(T, G, D), torch.randn(T, G, D, device=dev, dtype=bf)
    ms = ev(lambda: ops.kv_store(kk, vv, kp, vp, locs))
    add(f"kv_store {T}x{G}x{D}", "like: cache write", ms, bytes_=T * G * D * 2 * 4)
    # ---- row kernels -----------------------------------------------------------------------------------------------------
    X = torch.randn(T, S, Wd, device=dev)
    a, b2 = torch.randn(T, Wd, device=dev, dtype=bf), torch.randn(T, Wd, device=dev, dtype=bf)
    w1 = torch.ones(Wd, device=dev, dtype=bf)
    mix, ow, iw = torch.eye(S, device=dev), torch.ones(S, device=dev), torch.full((S,), 1.0 / S, device=dev)
    bias = torch.zeros(Wd, device=dev)
    ms = ev(lambda: ops.streams_mix_norm(X, w1, 1e-6, a=a, b=b2, bias=bias, sa=0.75, sb=1.25, sbias=0.75, mix=mix, out_w=ow,
                                         mult=0.5, in_w=iw))
    add(f"streams_mix_norm ({S} streams, two branches) {T}x{Wd}", "", ms, bytes_=T * Wd * (8 * S + 2 + 2 + 2))
    x32 = torch.randn(T, Wd, device=dev)
    ms = ev(lambda: ops.residual_rmsnorm(x32, w1, 1e-6, a=a, b=b2))
    add(f"residual_rmsnorm {T}x{Wd}", "like: norm", ms, bytes_=T * Wd * (4 + 4 + 2 + 2 + 2))
    ids = torch.randint(0, VOCAB, (T,), device=dev)
    emb = torch.randn(VOCAB, Wd, device=dev, dtype=bf)
    ms = ev(lambda: ops.embed_norm_streams(emb, ids, w1, 1e-6, S))
    add(f"embed_norm_streams {T}x{S}x{Wd}", "", ms, bytes_=T * Wd * (2 + 4 * S))
    ms = ev(lambda: ops.embed_f32(emb, ids))
    add(f"embed_f32 {T}x{Wd}", "like: embedding", ms, bytes_=T * Wd * 6)
    gu = torch.randn(T, 2 * z["ff"], device=dev, dtype=bf)
    ms = ev(lambda: ops.act_and_mul(gu, "clamped_swish", limit=7.0, slope=1.702))
    add(f"act_and_mul clamped {T}x{z['ff']}", "", ms, bytes_=T * z["ff"] * 2 * 3)
    ms = ev(lambda: ops.act_and_mul(gu, "gelu_tanh"))
    add(f"act_and_mul gelu {T}x{z['ff']}", "like: activation", ms, bytes_=T * z["ff"] * 2 * 3)
    o32 = torch.randn(T, H * D, device=dev)
    wn = torch.ones(H * D, device=dev, dtype=bf)
    ms = ev(lambda: ops.headnorm_gate(o32, qa, 1, H * D, 1e-6, weight=wn, gate_act="sigmoid"))
    add(f"headnorm_gate all heads together, sigmoid {T}x{H * D}", "", ms, bytes_=T * H * D * (4 + 2 + 2))
    ms = ev(lambda: ops.headnorm_gate(o32, qa, H, D, 1e-6, weight=wn, gate_act="sigmoid"))
    add(f"headnorm_gate per head, sigmoid {T}x{H * D}", "", ms, bytes_=T * H * D * (4 + 2 + 2))
    ms = ev(lambda: ops.headnorm_gate(o32, qa, H, D, 1e-6))
    add(f"headnorm_gate {T}x{H * D}", "like: head norm", ms, bytes_=T * H * D * (4 + 2 + 2))
    return rows


def run(sizes=("s", "m"), out=None, kernels=True):
    torch.cuda.set_device(0)
    flush = torch.zeros(160 << 20, dtype=torch.uint8, device="cuda")  # > L2, written between timed launches
    hbm, tf, src = BR.peaks()
    res = {"peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src, "fp32_core_tflops": BR.FP32_CORE_TFLOPS},
           "timing": "CUDA events, 3 warm-up launches, 160 MB written between timed launches", "sizes": {}}
    for name in sizes:
        z = SIZES[name]
        entry = {"shape": z, "models": {}}
        for label, cfg in (("llama", BR.llama_config(z)), ("rimidra-dense", BR.rimidra_config(z, False)),
                           ("matepel", matepel_config(z))):
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
