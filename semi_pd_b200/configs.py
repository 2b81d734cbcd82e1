"""Model / server configuration for the semi-PD forward path.

`ModelConfig` carries the HF-config attributes the reference's models/llama.py reads;
`ServerArgs` keeps the reference's flag names (python/sglang/srt/server_args.py:146,185-331,
870-875) for the knobs that exist on this path; `InstanceRole` and the two SM-percentile
environment variables are python/sglang/semi_pd/utils.py:10-11,25-28.
"""
from __future__ import annotations

import dataclasses
import json
import os
from enum import Enum
from typing import List, Optional

import torch

PREFILL_ENGINE_SM_PERCENTILE = int(os.getenv("SEMI_PD_PREFILL_SM_PERCENTILE", 80))
DECODE_ENGINE_SM_PERCENTILE = int(os.getenv("SEMI_PD_DECODE_SM_PERCENTILE", 100))


class InstanceRole(Enum):
    PREFILL = 0
    DECODE = 1
    OTHER = 2


@dataclasses.dataclass
class ModelConfig:
    name: str = "llama-3-8b"
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    vocab_size: int = 128256
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    rope_scaling: Optional[dict] = None
    max_position_embeddings: int = 8192
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    is_encoder_decoder: bool = False
    # "llama" (models/llama.py) or "opt" (BASELINE configs[0]: pre-LN, learned positions, ReLU, biases)
    model_type: str = "llama"
    layer_norm_eps: float = 1e-5
    # hf_eos_token_id of the reference's ModelConfig (honoured when a request sets ignore_eos=False)
    eos_token_ids: Optional[List[int]] = None
    # DeepSeek-V2 (model_type "deepseek_v2"): MLA + MoE (models/deepseek_v2.py)
    q_lora_rank: Optional[int] = None
    kv_lora_rank: int = 512
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    n_routed_experts: Optional[int] = None
    num_experts_per_tok: int = 6
    n_shared_experts: int = 2
    moe_intermediate_size: int = 1408
    first_k_dense_replace: int = 1
    moe_layer_freq: int = 1
    routed_scaling_factor: float = 1.0
    norm_topk_prob: bool = False
    # hybrid family (model_type "rimidra"): one entry per layer — {"type": "attention" | "retention",
    # "mixer": {...sizes and constants...}, "mlp": {...} | None, "weights_of": j (optional)}
    layer_specs: Optional[List[dict]] = None
    # model_type "nupovik": layer_specs has one entry per layer RUN (a looped block repeats its layers, each
    # run with a cache / state of its own); logits are multiplied by logit_scale
    logit_scale: float = 1.0
    # model_type "matepel": the residual is kept as `num_streams` parallel copies that every sublayer reads through
    # a weighted sum and writes back through a mixing matrix (None: one plain residual); a sublayer's output is
    # multiplied by residual_mult before it is added
    num_streams: Optional[int] = None
    residual_mult: float = 1.0
    # model_type "sugelix": the embedding row is multiplied by embedding_scale; pair_embedding {"buckets", "mul_prev",
    # "mul_cur"} adds a row of a hashed (previous token, token) table (None: no such table); loop_times is how often
    # the looped block runs (1: no loop) — each pass adds its row of a [loop_times, width] step table
    embedding_scale: float = 1.0
    pair_embedding: Optional[dict] = None
    loop_times: int = 1

    @property
    def context_len(self) -> int:
        return self.max_position_embeddings

    def get_num_kv_heads(self, tp_size: int) -> int:
        # models/llama.py:119-127: replicate KV heads when tp > n_kv
        return max(1, self.num_key_value_heads // tp_size)


_PRESETS = {
    "llama-3-8b": dict(eos_token_ids=[128001, 128009]),
    "llama-3.1-8b": dict(
        rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                          original_max_position_embeddings=8192),
        max_position_embeddings=131072),
    "llama-3-70b": dict(hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                        num_attention_heads=64, num_key_value_heads=8),
    "tiny-llama-test": dict(hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                            vocab_size=1024, max_position_embeddings=2048),
    # BASELINE configs[0]: facebook/opt-125m (hand-written config, no weights offline)
    "opt-125m": dict(model_type="opt", hidden_size=768, intermediate_size=3072, num_hidden_layers=12,
                     num_attention_heads=12, num_key_value_heads=12, head_dim=64, vocab_size=50272,
                     max_position_embeddings=2048, hidden_act="relu", tie_word_embeddings=True),
    # BASELINE configs[3]: deepseek-ai/DeepSeek-V2-Lite (15.7 B parameters, 2.4 B active)
    "deepseek-v2-lite": dict(model_type="deepseek_v2", hidden_size=2048, intermediate_size=10944,
                             num_hidden_layers=27, num_attention_heads=16, num_key_value_heads=16,
                             head_dim=192, vocab_size=102400, rms_norm_eps=1e-6, rope_theta=10000.0,
                             max_position_embeddings=163840, n_routed_experts=64, num_experts_per_tok=6,
                             n_shared_experts=2, moe_intermediate_size=1408, first_k_dense_replace=1,
                             kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                             routed_scaling_factor=1.0, norm_topk_prob=False, eos_token_ids=[100001],
                             rope_scaling=dict(type="yarn", factor=40.0, beta_fast=32, beta_slow=1, mscale=0.707,
                                               mscale_all_dim=0.707, original_max_position_embeddings=4096)),
    # one 8B-shaped layer pair: exhaustive parity at real head/FFN shapes
    "llama-3-8b-2layer": dict(num_hidden_layers=2, vocab_size=4096),
}


def _rimidra_config(path: str, cfg: dict, **overrides) -> ModelConfig:
    """config.json of the Rimidra family: {"architecture", "vocab", "width", "norm": {"eps"},
    "layers": [{"type", "mixer", "mlp", "weights_of"?}, ...]} — every size and constant of a layer is
    carried per layer in `layer_specs`; nothing is assumed equal across layers."""
    layers = [dict(spec) for spec in cfg["layers"]]
    for i, spec in enumerate(layers):
        if spec["type"] not in ("attention", "retention"):
            raise ValueError(f"layer {i}: unknown mixer type {spec['type']!r}")
        j, seen = spec.get("weights_of"), {i}
        while j is not None:  # a borrowed layer may itself borrow: follow to the layer that owns tensors
            if not 0 <= j < len(layers) or j in seen:
                raise ValueError(f"layer {i}: weights_of {spec.get('weights_of')} does not lead to a layer with tensors")
            seen.add(j)
            if layers[j].get("weights_of") is None:
                break
            j = layers[j]["weights_of"]
        if j is not None:
            if layers[j]["type"] != spec["type"]:
                raise ValueError(f"layer {i}: weights_of {j} names a layer of another mixer type")
            spec["weights_of"] = int(j)
    attn = [s["mixer"] for s in layers if s["type"] == "attention"]
    kw = dict(model_type="rimidra", hidden_size=int(cfg["width"]), vocab_size=int(cfg["vocab"]),
              num_hidden_layers=len(layers), rms_norm_eps=float(cfg["norm"]["eps"]), layer_specs=layers,
              # summary fields other components print or size by; the per-layer values rule
              num_attention_heads=max([m["heads"] for m in attn] or [1]),
              num_key_value_heads=max([m.get("kv_heads", m["heads"]) for m in attn] or [1]),
              head_dim=max([m["dim"] for m in attn] or [1]), intermediate_size=0,
              max_position_embeddings=int(cfg.get("context", 8192)))
    kw.update(overrides)
    return ModelConfig(name=os.path.basename(os.path.normpath(path)) or "rimidra", **kw)


def expand_loop(layers: List[dict], loop: Optional[dict]) -> List[dict]:
    """Layer RUNS in execution order for a config whose block of layers [start, stop) is executed `times` times back
    to back with the same tensors.  Every run is a copy of its layer's spec plus "layer" (the index in the
    checkpoint's names), "weights_of" (the first run of the same layer; None for that run itself), "opens_pass"
    (the first layer of every pass of the loop) and "pass_index" (the number of that pass, None elsewhere)."""
    order = [(i, None) for i in range(len(layers))]
    if loop is not None:
        a, b, n = int(loop["start"]), int(loop["stop"]), int(loop["times"])
        if not (0 <= a < b <= len(layers)) or n < 1:
            raise ValueError(f"loop {loop} does not fit {len(layers)} layers")
        order = order[:a] + [(i, t if i == a else None) for t in range(n) for i in range(a, b)] + order[b:]
    runs, first = [], {}
    for i, t in order:
        spec = dict(layers[i])
        spec.update(layer=i, opens_pass=t is not None, pass_index=t, weights_of=first.get(i))
        first.setdefault(i, len(runs))
        runs.append(spec)
    return runs


_NUPOVIK_MIXERS = ("gla", "latent_attention", "wkv")


def _nupovik_config(path: str, cfg: dict, **overrides) -> ModelConfig:
    """config.json of the Nupovik family: {"architecture", "vocab", "width", "norm": {"eps"}, "logit_scale",
    "layers": [{"type": "gla" | "latent_attention" | "wkv", "mixer": {...}, "mlp": {...} | null}, ...],
    "loop": {"start", "stop", "times"}}.  The block of layers [start, stop) is executed `times` times back to back, re-using its
    tensors; `layer_specs` lists the layer RUNS in execution order: "layer" is the index in the checkpoint's
    names, "weights_of" the first run of the same layer (None for that run itself), "opens_pass" marks the
    first layer of every pass of the loop (the stream is re-projected together with the embedding there)."""
    layers = cfg["layers"]
    for i, spec in enumerate(layers):
        if spec["type"] not in _NUPOVIK_MIXERS:
            raise ValueError(f"layer {i}: unknown mixer type {spec['type']!r}")
        if spec.get("mlp") is not None and spec["mlp"].get("kind") not in ("dense", "moe"):
            raise ValueError(f"layer {i}: unknown feed-forward kind {spec['mlp'].get('kind')!r}")
    runs = expand_loop(layers, cfg.get("loop") or None)
    heads = [int(s["mixer"]["heads"]) for s in runs]
    kw = dict(model_type="nupovik", hidden_size=int(cfg["width"]), vocab_size=int(cfg["vocab"]),
              num_hidden_layers=len(runs), rms_norm_eps=float(cfg["norm"]["eps"]), layer_specs=runs,
              logit_scale=float(cfg.get("logit_scale", 1.0)),
              # summary fields other components print or size by; the per-layer values rule
              num_attention_heads=max(heads), num_key_value_heads=1,
              head_dim=max(int(s["mixer"]["dim"]) for s in runs), intermediate_size=0,
              max_position_embeddings=int(cfg.get("context", 8192)))
    kw.update(overrides)
    return ModelConfig(name=os.path.basename(os.path.normpath(path)) or "nupovik", **kw)


def _matepel_config(path: str, cfg: dict, **overrides) -> ModelConfig:
    """config.json of the Matepel family: {"architecture", "vocab", "width", "norm": {"eps"}, "residual_mult",
    "streams", "layers": [{"type": "lightning" | "parallel", "mixer": {...}, "mlp": {"kind": "dense", "ff",
    "limit"} | null}, ...]}.  A "lightning" mixer is {heads, dim, vdim, decay: [heads]}; a "parallel" mixer is
    {"left": {heads, kv_heads, dim, vdim, scale, rot: {dims, base, scaling: {factor, original, fast, slow}}},
    "right": {heads, dim, vdim, gate_cap}, "left_scale", "right_scale"}.  Every size and constant is carried per
    layer in `layer_specs`."""
    layers = [dict(spec) for spec in cfg["layers"]]
    for i, spec in enumerate(layers):
        if spec["type"] not in ("lightning", "parallel"):
            raise ValueError(f"layer {i}: unknown mixer type {spec['type']!r}")
        if spec.get("mlp") is not None and spec["mlp"].get("kind") != "dense":
            raise ValueError(f"layer {i}: unknown feed-forward kind {spec['mlp'].get('kind')!r}")
        m = spec["mixer"]
        if spec["type"] == "lightning":
            if len(m["decay"]) != int(m["heads"]):
                raise ValueError(f"layer {i}: {len(m['decay'])} decays for {m['heads']} heads")
        else:
            left = m["left"]
            if int(left["heads"]) % int(left.get("kv_heads", left["heads"])):
                raise ValueError(f"layer {i}: {left['heads']} heads are not a multiple of {left['kv_heads']} kv heads")
            if int(left.get("vdim", left["dim"])) != int(left["dim"]):
                raise ValueError(f"layer {i}: the values are the keys, so vdim {left['vdim']} must equal dim {left['dim']}")
            rot = left.get("rot") or {}
            if int(rot.get("dims") or 0) % 2 or int(rot.get("dims") or 0) > int(left["dim"]):
                raise ValueError(f"layer {i}: rot.dims {rot.get('dims')} must be even and at most dim {left['dim']}")
    streams = cfg.get("streams")
    if streams is not None and not 1 <= int(streams) <= 8:
        raise ValueError(f"streams {streams}: 1 to 8 are supported")
    lefts = [s["mixer"]["left"] for s in layers if s["type"] == "parallel"]
    kw = dict(model_type="matepel", hidden_size=int(cfg["width"]), vocab_size=int(cfg["vocab"]),
              num_hidden_layers=len(layers), rms_norm_eps=float(cfg["norm"]["eps"]), layer_specs=layers,
              num_streams=int(streams) if streams is not None else None,
              residual_mult=float(cfg.get("residual_mult", 1.0)),
              # summary fields other components print or size by; the per-layer values rule
              num_attention_heads=max([int(m["heads"]) for m in lefts] or [1]),
              num_key_value_heads=max([int(m.get("kv_heads", m["heads"])) for m in lefts] or [1]),
              head_dim=max([int(m["dim"]) for m in lefts] or [1]), intermediate_size=0,
              max_position_embeddings=int(cfg.get("context", 8192)))
    kw.update(overrides)
    return ModelConfig(name=os.path.basename(os.path.normpath(path)) or "matepel", **kw)


_SUGELIX_MIXERS = ("attention", "attention_2", "latent_attention")


def _sugelix_config(path: str, cfg: dict, **overrides) -> ModelConfig:
    """config.json of the Sugelix family: {"architecture", "vocab", "width", "norm": {"eps"}, "embedding": {"scale",
    "bigram": {"buckets", "mul_prev", "mul_cur"}}, "layers": [{"type", "mixer", "mlp"}, ...], "loop": {"start", "stop",
    "times"}}.  Mixers: "attention" {heads, kv_heads, dim, vdim, scale, softcap, rot: {dims, base}} (rotation in
    pairs), "attention_2" {heads, kv_heads, dim, vdim, scale, diff, mask: {size}, rot: {dims, base, scaling:
    {factor}}} (two maps per head), "latent_attention" {heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, mask:
    {size}, rot: {base}}.  Feed-forward: {"kind": "moe", "router": {experts, top}, "expert": {ff, limit}, "shared":
    {ff, limit} | null} or null.  `layer_specs` lists the layer RUNS (see expand_loop); every size and constant is
    carried per layer."""
    layers = cfg["layers"]
    for i, spec in enumerate(layers):
        if spec["type"] not in _SUGELIX_MIXERS:
            raise ValueError(f"layer {i}: unknown mixer type {spec['type']!r}")
        if spec.get("mlp") is not None and spec["mlp"].get("kind") != "moe":
            raise ValueError(f"layer {i}: unknown feed-forward kind {spec['mlp'].get('kind')!r}")
        m = spec["mixer"]
        if spec["type"] != "latent_attention":
            if int(m["heads"]) % int(m.get("kv_heads", m["heads"])):
                raise ValueError(f"layer {i}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv heads")
            rot = int((m.get("rot") or {}).get("dims") or 0)
            if rot % 2 or rot > int(m["dim"]):
                raise ValueError(f"layer {i}: rot.dims {rot} must be even and at most dim {m['dim']}")
        elif int(m["rot_dim"]) % 2:
            raise ValueError(f"layer {i}: rot_dim {m['rot_dim']} must be even")
    loop = cfg.get("loop") or None
    runs = expand_loop(layers, loop)
    emb = cfg.get("embedding") or {}
    pair = emb.get("bigram") or None
    kw = dict(model_type="sugelix", hidden_size=int(cfg["width"]), vocab_size=int(cfg["vocab"]),
              num_hidden_layers=len(runs), rms_norm_eps=float(cfg["norm"]["eps"]), layer_specs=runs,
              embedding_scale=float(emb.get("scale", 1.0)),
              pair_embedding={k: int(pair[k]) for k in ("buckets", "mul_prev", "mul_cur")} if pair else None,
              loop_times=int(loop["times"]) if loop else 1,
              # summary fields other components print or size by; the per-layer values rule
              num_attention_heads=max(int(s["mixer"]["heads"]) for s in runs),
              num_key_value_heads=max(int(s["mixer"].get("kv_heads", 1)) for s in runs),
              head_dim=max(int(s["mixer"]["dim"]) for s in runs), intermediate_size=0,
              max_position_embeddings=int(cfg.get("context", 8192)))
    kw.update(overrides)
    return ModelConfig(name=os.path.basename(os.path.normpath(path)) or "sugelix", **kw)


# config.json "architecture" -> reader
_ARCHITECTURE_READERS = {"Rimidra": _rimidra_config, "Nupovik": _nupovik_config, "Matepel": _matepel_config,
                         "Sugelix": _sugelix_config}


def load_model_config(path: str, **overrides) -> ModelConfig:
    """ModelConfig of a model folder (config.json [+ model.safetensors]); the architecture named
    there selects the reader, as the `architectures` list of an HF config selects the model class
    in the reference (python/sglang/srt/model_loader/utils.py)."""
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    arch = cfg.get("architecture") or (cfg.get("architectures") or [None])[0]
    if arch not in _ARCHITECTURE_READERS:
        raise ValueError(f"{path}: architecture {arch!r} is not supported; known: {sorted(_ARCHITECTURE_READERS)}")
    return _ARCHITECTURE_READERS[arch](path, cfg, **overrides)


def get_model_config(name: str, **overrides) -> ModelConfig:
    if os.path.isdir(name) and os.path.exists(os.path.join(name, "config.json")):
        return load_model_config(name, **overrides)
    key = name.lower().split("/")[-1]
    for cand in (key, key.replace("meta-", ""), key.replace("-instruct", "")):
        if cand in _PRESETS:
            kw = dict(_PRESETS[cand])
            kw.update(overrides)
            return ModelConfig(name=cand, **kw)
    raise ValueError(f"unknown model '{name}'; known: {sorted(_PRESETS)}")


def default_cuda_graph_bs(max_bs: int = 160) -> List[int]:
    # model_executor/cuda_graph_runner.py:116-118
    return [b for b in [1, 2, 4] + [i * 8 for i in range(1, 21)] if b <= max_bs]


@dataclasses.dataclass
class ServerArgs:
    model_path: str = "llama-3-8b"
    dtype: str = "bfloat16"
    # "dummy": synthetic weights; "safetensors": <model_path>/model.safetensors; "auto": the file
    # when model_path is a folder that has one, else dummy; "external": load_weights() by the caller
    load_format: str = "dummy"
    tp_size: int = 1
    mem_fraction_static: Optional[float] = None
    max_total_tokens: Optional[int] = None
    max_running_requests: Optional[int] = None
    chunked_prefill_size: int = 8192
    max_prefill_tokens: int = 16384
    context_length: Optional[int] = None
    enable_semi_pd: bool = False
    disable_radix_cache: bool = True     # semi-PD forces it off (server_args.py:325-331)
    disable_cuda_graph: bool = False
    cuda_graph_max_bs: int = 160
    cuda_graph_bs: Optional[List[int]] = None
    attention_backend: str = "spd"
    random_seed: int = 1234
    schedule_conservativeness: float = 1.0
    allow_auto_truncate: bool = False
    host: str = "127.0.0.1"
    port: int = 30000
    device: str = "cuda"

    def torch_dtype(self) -> torch.dtype:
        # float32: the hybrid family only (its operators exist in true 32-bit)
        return {"bfloat16": torch.bfloat16, "float16": torch.float16, "half": torch.float16,
                "auto": torch.bfloat16, "float32": torch.float32}[self.dtype]

    @staticmethod
    def add_cli_args(parser):
        parser.add_argument("--model-path", type=str, default=ServerArgs.model_path)
        parser.add_argument("--dtype", type=str, default=ServerArgs.dtype)
        parser.add_argument("--load-format", type=str, default=ServerArgs.load_format)
        parser.add_argument("--tp", "--tensor-parallel-size", dest="tp_size", type=int, default=1)
        parser.add_argument("--mem-fraction-static", type=float, default=None)
        parser.add_argument("--max-total-tokens", type=int, default=None)
        parser.add_argument("--max-running-requests", type=int, default=None)
        parser.add_argument("--chunked-prefill-size", type=int, default=ServerArgs.chunked_prefill_size)
        parser.add_argument("--max-prefill-tokens", type=int, default=ServerArgs.max_prefill_tokens)
        parser.add_argument("--context-length", type=int, default=None)
        parser.add_argument("--enable-semi-pd", action="store_true", help="Enable SemiPD.")
        parser.add_argument("--disable-radix-cache", action="store_true")
        parser.add_argument("--disable-cuda-graph", action="store_true")
        parser.add_argument("--cuda-graph-max-bs", type=int, default=ServerArgs.cuda_graph_max_bs)
        parser.add_argument("--random-seed", type=int, default=ServerArgs.random_seed)
        parser.add_argument("--allow-auto-truncate", action="store_true")
        parser.add_argument("--host", type=str, default=ServerArgs.host)
        parser.add_argument("--port", type=int, default=ServerArgs.port)

    @classmethod
    def from_cli_args(cls, ns):
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in vars(ns).items() if k in names})
