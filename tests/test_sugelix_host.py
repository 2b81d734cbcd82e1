"""Host side of the Sugelix family, no GPU: the config reader with its loop expansion and refusals, the checkpoint checks
of load_weights (map-major rows of the two-map attention, the transposed key lift of the latent attention, constants of
looped runs), the pools the model asks for (value heads fewer than key heads, a latent row, the previous-token state),
and the oracle's own consistency (the absorbed latent form, the pair rows, a sequence fed token by token)."""
import json

import pytest
import torch

from oracle import sugelix_oracle as S
from tests import rimidra_helpers as H
from tests import sugelix_helpers as C


def _folder(tmp_path, cfg, weights=None):
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    if weights is not None:
        H.write_safetensors(str(tmp_path / "model.safetensors"), weights)
    return str(tmp_path)


@pytest.mark.parametrize("name", list(C.CONFIGS))
def test_config_reader_lists_the_layer_runs(tmp_path, name):
    from semi_pd_b200.configs import get_model_config
    cfg = C.CONFIGS[name]()
    mc = get_model_config(_folder(tmp_path, cfg))
    runs = S.layer_runs(cfg)
    assert mc.model_type == "sugelix" and mc.num_hidden_layers == len(runs)
    assert mc.hidden_size == cfg["width"] and mc.vocab_size == cfg["vocab"] and mc.rms_norm_eps == cfg["norm"]["eps"]
    assert mc.embedding_scale == cfg["embedding"]["scale"] and mc.pair_embedding == cfg["embedding"].get("bigram")
    assert mc.loop_times == (cfg["loop"]["times"] if cfg.get("loop") else 1)
    assert [(s["layer"], s["pass_index"]) for s in mc.layer_specs] == runs
    first = {}
    for r, s in enumerate(mc.layer_specs):
        assert s["weights_of"] == first.get(s["layer"]) and s["type"] == cfg["layers"][s["layer"]]["type"]
        first.setdefault(s["layer"], r)


def test_loop_expansion_is_shared_with_the_other_looped_family():
    from semi_pd_b200.configs import expand_loop
    layers = [{"type": t} for t in "abcd"]
    runs = expand_loop(layers, {"start": 1, "stop": 3, "times": 3})
    assert [r["type"] for r in runs] == list("abcbcbcd")
    assert [r["opens_pass"] for r in runs] == [False, True, False, True, False, True, False, False]
    assert [r["pass_index"] for r in runs] == [None, 0, None, 1, None, 2, None, None]
    assert [r["weights_of"] for r in runs] == [None, None, None, 1, 2, 1, 2, None]
    assert [r["type"] for r in expand_loop(layers, None)] == list("abcd")
    with pytest.raises(ValueError):
        expand_loop(layers, {"start": 2, "stop": 5, "times": 2})


def test_reader_refuses_what_it_does_not_know(tmp_path):
    from semi_pd_b200.configs import get_model_config
    good = C.config_mixed()
    for change in (lambda c: c["layers"][0].update(type="retention"),
                   lambda c: c["layers"][0]["mlp"].update(kind="dense"),
                   lambda c: c["layers"][0]["mixer"].update(kv_heads=3),
                   lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7),
                   lambda c: c["layers"][0]["mixer"]["rot"].update(dims=32),
                   lambda c: c["layers"][1]["mixer"].update(rot_dim=5),
                   lambda c: c["loop"].update(stop=9),
                   lambda c: c["loop"].update(times=0),
                   lambda c: c.update(architecture="Other")):
        cfg = json.loads(json.dumps(good))
        change(cfg)
        with pytest.raises(ValueError):
            get_model_config(_folder(tmp_path, cfg))


@pytest.mark.parametrize("name", ["mixed", "ones"])
def test_checkpoint_is_checked_and_laid_out(tmp_path, name):
    from semi_pd_b200.configs import get_model_config
    from semi_pd_b200.sugelix import SugelixForCausalLM
    cfg = C.CONFIGS[name]()
    w = S.make_weights(cfg, seed=1)
    model = SugelixForCausalLM(get_model_config(_folder(tmp_path, cfg)), dtype=torch.float32, device="cpu")
    assert set(model.full_shapes()) == set(S.tensor_shapes(cfg))
    model.load_weights(w.items())
    kv, st, vec, extras = model.cache_shapes()
    assert extras == {"token_state": cfg["embedding"].get("bigram") is not None}
    assert all(s is None for s in st) and all(s is None for s in vec)
    for layer, shape in zip(model.layers, kv):
        m, mx = cfg["layers"][layer.name_index]["mixer"], layer.mixer
        p = f"l{layer.name_index}.mix."
        if layer.kind == "latent_attention":
            assert shape == (1, m["kv_rank"] + m["rot_dim"], 0)
            uk = w[p + "uk"].float().view(m["heads"], m["dim"], m["kv_rank"])
            assert torch.equal(mx.uk_t.weight.view(m["heads"], m["kv_rank"], m["dim"]), uk.transpose(1, 2))
        else:
            n = 2 if layer.kind == "attention_2" else 1
            assert shape == (n * m["kv_heads"], m["dim"], m["vdim"], m["kv_heads"])
            q_rows = mx.in_proj.weight[: n * m["heads"] * m["dim"]].view(n, m["heads"], m["dim"], -1)
            stored = w[p + "q"].float().view(m["heads"], n, m["dim"], -1)
            assert torch.equal(q_rows, stored.transpose(0, 1)), "q rows are map-major"
            assert torch.equal(mx.k_bias.view(n, m["kv_heads"], m["dim"]),
                               w[p + "k.b"].float().view(m["kv_heads"], n, m["dim"]).transpose(0, 1))
            if n == 2:
                assert mx.lam == pytest.approx(S.difference_weight(w, p, m["diff"]), rel=1e-12)
        if layer.weights_of is not None:  # a later run of a looped layer reads the first run's tensors and constants
            src = model.layers[layer.weights_of]
            assert layer.norm1 is src.norm1 and layer.mlp is src.mlp and mx.o_proj is src.mixer.o_proj
            assert getattr(mx, "lam", None) == getattr(src.mixer, "lam", None)
            assert getattr(mx, "q_bias", None) is getattr(src.mixer, "q_bias", None)
    some = next(iter(k for k in w if k.endswith("mix.o")))
    bad = dict(w)
    del bad[some]
    with pytest.raises(KeyError):
        model.load_weights(bad.items())
    bad = dict(w)
    bad[some] = bad[some][:, :-1]
    with pytest.raises(ValueError):
        model.load_weights(bad.items())


def test_pools_for_shared_value_heads_latent_rows_and_previous_tokens():
    from semi_pd_b200.memory_pool import HybridTokenToKVPool, RecurrentStatePool
    shapes = [(4, 16, 24, 2), (1, 40, 0), None, (2, 8, 8)]
    state = RecurrentStatePool(5, [None] * 4, "cpu", token_state=True)
    pool = HybridTokenToKVPool(32, 1, torch.bfloat16, shapes, "cpu", state_pool=state)
    assert pool.get_key_buffer(0).shape == (33, 4, 16) and pool.get_value_buffer(0).shape == (33, 2, 24)
    assert pool.get_value_buffer(1) is pool.get_key_buffer(1) and pool.get_key_buffer(1).shape == (33, 1, 40)
    assert pool.get_key_buffer(2) is None and pool.get_value_buffer(3).shape == (33, 2, 8)
    assert HybridTokenToKVPool.bytes_per_token(shapes, torch.bfloat16) == 2 * (4 * 16 + 2 * 24 + 40 + 2 * 16)
    assert state.prev_token.shape == (5,) and state.prev_token.dtype == torch.int32
    assert RecurrentStatePool(5, [None], "cpu").prev_token is None


def test_oracle_absorbed_latent_form_and_pair_rows():
    """What the product computes for the latent attention (queries carried into the latent space, values read from the
    latent and lifted afterwards) is the same function as the oracle's per-head keys and values."""
    cfg = C.config_mixed()
    W = S.make_weights(cfg, seed=3)
    m, p, eps = cfg["layers"][1]["mixer"], "l1.mix.", cfg["norm"]["eps"]
    T, Hh, dk, dr, dv, rank = 23, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    u = torch.randn(T, cfg["width"], dtype=torch.float64)
    pos = list(range(T))
    want = S.latent_attention_mixer(u, W, p, m, pos, eps)
    cq = S.rms_norm(S.linear(u, W[p + "dq"]), W[p + "dq.norm"], eps)
    q = S.linear(cq, W[p + "uq"]).view(T, Hh, dk + dr)
    down = S.linear(u, W[p + "dkv"])
    c = S.rms_norm(down[:, :rank], W[p + "dkv.norm"], eps)
    rot = dict(m["rot"], dims=dr)
    row = torch.cat([c, S.rotate(down[:, None, rank:], pos, rot, "halves")[:, 0]], -1)[:, None]       # the cache row
    uk, uv = S.f64(W[p + "uk"]).view(Hh, dk, rank), S.f64(W[p + "uv"]).view(Hh, dv, rank)
    q_lat = torch.cat([torch.einsum("thd,hdr->thr", q[..., :dk], uk), S.rotate(q[..., dk:], pos, rot, "halves")], -1)
    o_lat = S.softmax_attention(q_lat, row, row[..., :rank], m["scale"], window=m["mask"]["size"], sinks=S.f64(W[p + "sink"]))
    o = torch.einsum("thr,hvr->thv", o_lat, uv).reshape(T, Hh * dv) * torch.sigmoid(S.linear(u, W[p + "g"]))
    assert torch.allclose(S.linear(o, W[p + "o"]), want, rtol=1e-9, atol=1e-11)
    assert S.bigram_rows([3, 5, 5], 7, 2, 3) == [7, (3 * 2 + 5 * 3) % 7, (5 * 2 + 5 * 3) % 7]
    assert S.layer_runs(cfg) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]


def test_oracle_token_by_token_equals_whole():
    cfg = C.config_ones()
    W = S.make_weights(cfg, seed=2)
    toks = H.prompt(17, cfg["vocab"], 1)
    whole = S.forward(cfg, W, toks)
    st = S.Stepper(cfg, W)
    rows = [st.feed(toks[:5])] + [st.feed([t]) for t in toks[5:]]
    assert torch.allclose(torch.cat(rows), whole, rtol=1e-9, atol=1e-11)
