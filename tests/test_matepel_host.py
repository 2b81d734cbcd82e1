"""Host side of the Matepel family, no GPU: the config reader and its refusals, the checkpoint checks of load_weights,
the pool shapes the model asks for (a layer that owns keys / values AND a recurrent state), the position table against
the oracle's frequencies, and the oracle's own consistency (a sequence fed in portions equals the sequence fed at once)."""
import json

import pytest
import torch

from oracle import matepel_oracle as M
from tests import matepel_helpers as C
from tests import rimidra_helpers as H


def _folder(tmp_path, cfg, weights=None):
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    if weights is not None:
        H.write_safetensors(str(tmp_path / "model.safetensors"), weights)
    return str(tmp_path)


@pytest.mark.parametrize("name", list(C.CONFIGS))
def test_config_reader(tmp_path, name):
    from semi_pd_b200.configs import get_model_config
    cfg = C.CONFIGS[name]()
    mc = get_model_config(_folder(tmp_path, cfg))
    assert mc.model_type == "matepel" and mc.num_hidden_layers == len(cfg["layers"])
    assert mc.hidden_size == cfg["width"] and mc.vocab_size == cfg["vocab"] and mc.rms_norm_eps == cfg["norm"]["eps"]
    assert mc.num_streams == cfg.get("streams") and mc.residual_mult == cfg["residual_mult"]
    assert [s["type"] for s in mc.layer_specs] == [s["type"] for s in cfg["layers"]]


def test_reader_refuses_what_it_does_not_know(tmp_path):
    from semi_pd_b200.configs import get_model_config
    good = C.config_mixed()
    for change in (lambda c: c["layers"][0].update(type="conv"),
                   lambda c: c["layers"][0]["mlp"].update(kind="moe"),
                   lambda c: c["layers"][0]["mixer"].update(decay=[0.5]),
                   lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3),
                   lambda c: c["layers"][1]["mixer"]["left"].update(vdim=8),
                   lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=7),
                   lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=32),
                   lambda c: c.update(streams=9),
                   lambda c: c.update(architecture="Other")):
        cfg = json.loads(json.dumps(good))
        change(cfg)
        with pytest.raises(ValueError):
            get_model_config(_folder(tmp_path, cfg))


@pytest.mark.parametrize("name", ["mixed", "far"])
def test_checkpoint_is_checked_against_the_config(tmp_path, name):
    from semi_pd_b200 import ops
    from semi_pd_b200.configs import get_model_config
    from semi_pd_b200.matepel import MatepelForCausalLM
    cfg = C.CONFIGS[name]()
    w = M.make_weights(cfg, seed=1)
    model = MatepelForCausalLM(get_model_config(_folder(tmp_path, cfg)), dtype=torch.float32, device="cpu")
    model.load_weights(w.items())
    kv, st, vec = model.cache_shapes()
    for i, spec in enumerate(cfg["layers"]):
        m = spec["mixer"]
        if spec["type"] == "lightning":
            assert kv[i] is None and vec[i] is None and st[i] == (m["heads"], m["dim"], m["vdim"])
        else:
            a, b = m["left"], m["right"]
            assert kv[i] == (a["kv_heads"], a["dim"], a["dim"]) and st[i] == (b["heads"], b["dim"], b["vdim"])
            assert vec[i] == ops.matrix_memory_vector_dim(b["heads"], b["dim"], b["vdim"])
            assert vec[i] == b["heads"] * -(-b["vdim"] // 32) * (b["dim"] + 1)
    if cfg.get("streams") is None:  # one plain residual: unit coefficients, nothing read from the checkpoint
        assert model.num_streams == 1 and float(model.layers[0].hc1.mix) == 1.0
        assert not any(".hc" in k for k in model.full_shapes())
    missing = dict(w)
    del missing["l0.norm1"]
    with pytest.raises(KeyError):
        model.load_weights(missing.items())
    wrong = dict(w)
    wrong["final.norm"] = torch.zeros(7)
    with pytest.raises(ValueError):
        model.load_weights(wrong.items())


def test_pool_of_a_layer_with_cache_and_state():
    from semi_pd_b200.memory_pool import HybridTokenToKVPool, RecurrentStatePool
    states = RecurrentStatePool(3, [(2, 4, 6), (1, 8, 40)], device="cpu", shift_dims=[None, 18])
    pool = HybridTokenToKVPool(16, 1, torch.float32, [None, (2, 12, 12)], device="cpu", state_pool=states)
    assert pool.get_key_buffer(0) is None and pool.get_key_buffer(1).shape == (17, 2, 12)
    assert pool.get_value_buffer(1) is not pool.get_key_buffer(1)  # rotated keys and unrotated values are two buffers
    assert states.get_state(1).shape == (3, 1, 8, 40) and states.get_shift(1).shape == (3, 18)
    assert states.get_shift(0) is None


@pytest.mark.parametrize("dims,base,scaling", [(8, 1e4, (4.0, 64, 8.0, 1.0)), (16, 2e5, (6.0, 1024, 24.0, 1.0)),
                                               (12, 100.0, None), (32, 5e5, (16.0, 512, 2.0, 0.5))])
def test_position_table_follows_the_scaled_frequencies(dims, base, scaling):
    from semi_pd_b200.matepel import scaled_rotary_table
    sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
    table = scaled_rotary_table(dims, base, sc, 3000, "cpu")
    f, mag = M.scaled_rotary_frequencies(dims, base, sc)
    pos = torch.tensor([0, 1, 17, 2999], dtype=torch.float64)
    ang = pos[:, None] * f[None, :]
    want = torch.cat([ang.cos(), ang.sin()], -1) * mag
    assert (table[[0, 1, 17, 2999]].double() - want).abs().max().item() < 2e-7
    if sc is not None:  # the slowest channel is divided by the factor, the fastest is kept (when the ramp has room)
        plain = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
        assert abs(float(f[-1] / plain[-1]) - 1.0 / sc["factor"]) < 1e-12 or float(f[-1] / plain[-1]) > 1.0 / sc["factor"]
        assert float(f[0]) == float(plain[0])


@pytest.mark.parametrize("name", list(C.CONFIGS))
def test_oracle_in_portions_equals_oracle_at_once(name):
    cfg = C.CONFIGS[name]()
    w = M.make_weights(cfg, seed=C.SEEDS[name])
    toks = H.prompt(23, cfg["vocab"], 5)
    whole = M.forward(cfg, w, toks)
    st = M.Stepper(cfg, w)
    parts = torch.cat([st.feed(toks[a:b]) for a, b in ((0, 1), (1, 3), (3, 14), (14, 15), (15, 23))])
    assert (parts - whole).abs().max().item() < 1e-9
