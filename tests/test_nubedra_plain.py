"""The Nubedra design without a GPU: configuration reading and refusals, tensor names, the cache's layout for it, the
package's CPU model against the plain implementation, and the plain implementation's own sensitivity (a window off by
one key, another layer's cache, a sink left out, a decay root, the rotation's rescaling: each moves the logits by far
more than any tolerance, and leaves the positions it should not touch as they were)."""
import copy

import numpy as np
import pytest
import torch

import nubedra_helpers as nh
import plain_nubedra as plain


def test_configuration_reading_and_refusals():
    from llaisys_b200.config import ConfigError, config_from_dict
    cfg = config_from_dict(nh.CONFIGS["P"])
    spec = cfg.to_spec()
    assert spec.architecture == "Nubedra" and spec.vocab_size == 211 and spec.hidden_size == 64
    assert [c.cache_of for c in spec.order] == [None, None, 1, None]
    assert [l.block for l in spec.layers] == ["sandwich_residual"] * 4 and spec.layers[0].params["mult"] == 0.6
    assert [len(l.sublayers) for l in spec.layers] == [1, 2, 2, 2]
    mixers = [l.sublayers[0].part for l in spec.layers]
    assert [m.kind for m in mixers] == ["gated_linear_attention", "latent_attention", "latent_attention", "gated_linear_attention"]
    # a cache that another layer reads keeps every row; the reader's window is its own
    assert mixers[1].params["cache_window"] is None and mixers[1].params["window"] == 70 and mixers[2].params["window"] == 33
    assert mixers[2].params["own_kv"] is False and mixers[1].params["position"].params["yarn"]["factor"] == 4.0
    assert spec.head.params["tied_to"] == "embed" and spec.layers[0].sublayers[0].post_norm.params["offset"] == 1.0
    q = config_from_dict(nh.CONFIGS["Q"]).to_spec()
    assert q.layers[0].sublayers[0].part.params["cache_window"] == 20 and q.layers[0].sublayers[0].part.params["position"].params["yarn"] is None
    assert cfg.to_dict() == nh.CONFIGS["P"]

    def bad(edit, match):
        with pytest.raises(ConfigError, match=match):
            config_from_dict(nh.variant(nh.CONFIGS["P"], edit))

    bad(lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 0), "kv_from")            # a recurrent layer keeps no rows
    bad(lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 2), "kv_from")            # not an earlier layer
    bad(lambda c: c["layers"][2]["mixer"].__setitem__("kv_rank", 24), "differs")
    bad(lambda c: c["layers"][2]["mixer"]["rot"].__setitem__("base", 7.0), "differs")
    bad(lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 7), "even")
    bad(lambda c: c["layers"][0].__setitem__("type", "attention"), "mixers of this architecture")
    bad(lambda c: c["layers"][1]["mlp"].__setitem__("kind", "moe"), "feed-forward")
    bad(lambda c: c["layers"][0]["mixer"].__setitem__("tau", 0), "positive")
    bad(lambda c: c.__setitem__("layers", []), "non-empty")


def test_tensor_names_and_the_size_no_key_gives(tmp_path):
    from llaisys_b200.config import load_config
    from llaisys_b200.engine.model import DecoderModel
    from llaisys_b200.parts import BuildEnv
    from llaisys_b200.weights import FolderSource, SafetensorsFile, write_safetensors
    from llaisys_b200.weights.loader import WeightsError, check_tensors
    folder = nh.make_folder(tmp_path, nh.CONFIGS["P"], seed=1, gain=1.0)
    model = DecoderModel(load_config(folder).to_spec(), BuildEnv(torch.float32, torch.device("cpu")))
    names = set(model.expected_tensors())
    assert {"embed", "final.norm", "l0.norm1", "l0.norm1b", "l0.mix.a1", "l0.mix.a2", "l0.mix.a2.b", "l0.mix.norm", "l1.mix.dkv",
            "l1.mix.dkv.norm", "l1.mix.dq.norm", "l1.mix.sink", "l1.mix.g", "l1.mlp.gate", "l1.norm2b", "l3.mlp.down"} <= names
    assert "l2.mix.dkv" not in names and "l0.norm2" not in names and "head" not in names
    check_tensors(model, FolderSource(folder))
    # the decay's bottleneck has whatever size the file gives it, as long as its two matrices fit
    f = SafetensorsFile(folder / "model.safetensors")
    t = {n: f.get(n).clone() for n in f.entries}
    t["l0.mix.a1"], t["l0.mix.a2"] = t["l0.mix.a1"][:5].clone(), t["l0.mix.a2"][:, :5].clone()
    write_safetensors(folder / "model.safetensors", t)
    check_tensors(model, FolderSource(folder))
    t["l0.mix.k"] = t["l0.mix.k"][:-1].clone()
    write_safetensors(folder / "model.safetensors", t)
    with pytest.raises(WeightsError, match="l0.mix.k"):
        check_tensors(model, FolderSource(folder))


def test_what_the_cache_keeps_for_this_design():
    from llaisys_b200.cache import CacheConfig
    from llaisys_b200.cache.kv import PagedCache
    from llaisys_b200.config import config_from_dict
    from llaisys_b200.engine.model import DecoderModel
    from llaisys_b200.parts import BuildEnv
    for name, rings in (("P", [None]), ("Q", [2, 17]), ("R", [None])):
        model = DecoderModel(config_from_dict(nh.CONFIGS[name]).to_spec(), BuildEnv(torch.float32, torch.device("cpu")))
        cache = PagedCache(model.kv_needs(), model.cache_of(), model.state_sizes(), CacheConfig(max_tokens=2048, max_seqs=4),
                           torch.float32, "cpu", allocate=False)
        assert cache.rings == rings
        assert all(k[0] == 1 and k[2] == 0 for k in cache.group_keys)          # one row per token, no value pool
    assert model.state_sizes() == [0, 130 * 4, 0] and model.cache_of() == [None, None, 0]


@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_cpu_model_against_the_plain_implementation(tmp_path, name):
    from llaisys_b200.models.cpu_model import CpuModel
    folder = nh.make_folder(tmp_path, nh.CONFIGS[name], seed=3, gain=9.0)
    oracle = nh.Oracle(folder)
    toks = nh.random_requests(nh.CONFIGS[name], [90], seed=1)[0]
    m = CpuModel.from_folder(folder)
    got = np.concatenate([m.step(toks[:50])] + [m.step([t]) for t in toks[50:60]] + [m.step(toks[60:])])
    assert np.abs(got - oracle.logits(toks)).max() < 5e-5
    new = m.generate(toks[:7], 5)
    seq = list(toks[:7])
    for _ in range(5):
        seq.append(int(np.argmax(oracle.logits(seq)[-1])))
    assert new == seq[7:]


def test_rescaled_frequencies_of_the_package_against_the_plain_ones():
    from llaisys_b200.parts.rope import yarn_frequencies
    for dims, base, yarn in ((8, 5000.0, nh.YARN_A), (2, 300.0, nh.YARN_B), (32, 1e6, (8.0, 4096, 32.0, 1.0)), (6, 10000.0, None)):
        y = dict(zip(("factor", "original", "fast", "slow"), yarn)) if yarn else None
        f, mag = yarn_frequencies(dims, base, y)
        pf, pmag = plain.yarn_frequencies(dims, base, y)
        assert np.allclose(f.numpy(), pf, rtol=1e-13) and abs(mag - pmag) < 1e-15
    f, mag = plain.yarn_frequencies(8, 5000.0, dict(zip(("factor", "original", "fast", "slow"), nh.YARN_A)))
    plain_f = 5000.0 ** (-2.0 * np.arange(4) / 8)
    assert f[0] == plain_f[0] and np.isclose(f[-1], plain_f[-1] / 4.0) and mag > 1.0        # fast kept, slow stretched


def test_the_plain_implementations_own_sensitivity(tmp_path):
    cfg = nh.CONFIGS["P"]
    folder = nh.make_folder(tmp_path, cfg, seed=5, gain=9.0)
    oracle = nh.Oracle(folder)
    toks = nh.random_requests(cfg, [120], seed=2)[0]
    base = oracle.logits(toks)
    tol = 1e-4

    def moved(edit_cfg=None, edit_w=None):
        c = nh.variant(oracle.config, edit_cfg) if edit_cfg else oracle.config
        w = dict(oracle.weights)
        if edit_w:
            edit_w(w)
        return np.abs(plain.forward(c, w, toks) - base).max(axis=1)

    # the reader's window is 33: one key more changes nothing before position 33 and a lot after it
    d = moved(lambda c: c["layers"][2]["mixer"]["mask"].__setitem__("size", 34))
    assert d[:33].max() == 0 and d[33:].max() > 100 * tol
    d = moved(lambda c: c["layers"][1]["mixer"]["mask"].__setitem__("size", 69))
    assert d[:69].max() == 0 and d[69:].max() > 100 * tol
    # the reader reads layer 1's rows with its own up projections: its own down projection (there is none) is not used
    assert moved(edit_w=lambda w: w.__setitem__("l1.mix.sink", w["l1.mix.sink"] * 0)).max() > 100 * tol
    assert moved(edit_w=lambda w: w.__setitem__("l2.mix.sink", w["l2.mix.sink"] + 1.0)).max() > 100 * tol
    assert moved(lambda c: c["layers"][0]["mixer"].__setitem__("tau", 4.4)).max() > 100 * tol
    assert moved(lambda c: c["layers"][1]["mixer"]["rot"].pop("scaling")).max() > 100 * tol
    assert moved(lambda c: c.__setitem__("residual_mult", 0.9)).max() > 100 * tol
    assert moved(edit_w=lambda w: w.__setitem__("l3.norm2b", w["l3.norm2b"] - 1.0)).max() > 100 * tol      # the offset of one
    # the recurrence carries the first token to the last one
    other = [(toks[0] + 1) % cfg["vocab"]] + toks[1:]
    only_gla = nh.variant(oracle.config, lambda c: c.__setitem__("layers", [c["layers"][0]]))
    a, b = plain.forward(only_gla, oracle.weights, toks), plain.forward(only_gla, oracle.weights, other)
    assert np.abs(a[-1] - b[-1]).max() > 1e-6


def test_state_of_the_plain_recurrence_can_be_carried():
    rng = np.random.default_rng(0)
    H, dk, dv, D = 2, 5, 3, 12
    w = {"p.q": rng.normal(size=(H * dk, D)), "p.k": rng.normal(size=(H * dk, D)), "p.v": rng.normal(size=(H * dv, D)),
         "p.g": rng.normal(size=(H * dv, D)), "p.o": rng.normal(size=(D, H * dv)), "p.norm": rng.normal(size=dv),
         "p.a1": rng.normal(size=(4, D)), "p.a2": rng.normal(size=(H * dk, 4)), "p.a2.b": rng.normal(size=H * dk)}
    mix = {"heads": H, "dim": dk, "vdim": dv, "tau": 3.0}
    h = rng.normal(size=(20, D))
    whole, S = plain.gla_mixer(h, w, "p", mix, 1e-5)
    a, Sa = plain.gla_mixer(h[:7], w, "p", mix, 1e-5)
    b, Sb = plain.gla_mixer(h[7:], w, "p", mix, 1e-5, state=Sa)
    assert np.abs(np.concatenate([a, b]) - whole).max() < 1e-12 and np.abs(Sb - S).max() < 1e-12
