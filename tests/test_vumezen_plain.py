"""CPU tests of the Vumezen side: the configuration reader, the cache's pinned pages, and the plain oracle's own
sensitivity (a fault of one key, of the sink or of the pair table must move its logits by far more than the
tolerances the engine is held to, or the engine tests would prove nothing)."""
import copy
import json

import numpy as np
import pytest
import torch

import plain_vumezen as plain
import vumezen_helpers as vh
from llaisys_b200.cache.slots import SlotBook
from llaisys_b200.config import ConfigError, config_from_dict


def test_configuration_to_spec():
    cfg = config_from_dict(vh.CONFIGS["P"])
    spec = cfg.to_spec()
    assert spec.architecture == "Vumezen" and spec.vocab_size == 211 and len(spec.layers) == 3
    assert [c.cache_of for c in spec.order] == [None, 0, None]
    m0, m1, m2 = (l.sublayers[0].part.params for l in spec.layers)
    # a cache that another layer reads keeps every key; a layer of its own keeps its window (and the first keys)
    assert m0["cache_window"] is None and m1["cache_window"] is None and m2["cache_window"] == 70
    assert m1["own_kv"] is False and m0["own_kv"] and m1["window"] == 33 and m1["keep_first"] == 5
    assert m0["key_dim"] == 16 and m0["value_dim"] == 24 and m0["position"].params["dims"] == 8
    assert all(l.block == "parallel_residual" for l in spec.layers)
    r = config_from_dict(vh.CONFIGS["R"]).to_spec()
    assert len(r.layers[1].sublayers) == 1                     # a layer without a feed-forward
    assert r.layers[0].sublayers[1].part.params["shared_ff"] == 16 and r.layers[2].sublayers[1].part.params["shared_ff"] is None
    assert config_from_dict(vh.CONFIGS["Q"]).to_spec().embedding.params["pair"] is None
    assert cfg.to_dict() == vh.CONFIGS["P"]


@pytest.mark.parametrize("edit, word", [
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_from", 1), "earlier"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 4), "differ"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("heads", 3), "share"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "even"),
    (lambda c: c["layers"][0].__setitem__("type", "recurrent"), "attention"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "exceeds"),
    (lambda c: c.pop("width"), "width"),
])
def test_configuration_refusals(edit, word):
    with pytest.raises(ConfigError, match=word):
        config_from_dict(vh.variant(vh.CONFIGS["P"], edit))


def test_tensor_names_of_the_model():
    from llaisys_b200.engine.model import DecoderModel
    from llaisys_b200.parts import BuildEnv
    model = DecoderModel(config_from_dict(vh.CONFIGS["P"]).to_spec(), BuildEnv(torch.float32, torch.device("cpu")))
    names = model.expected_tensors()
    assert {"embed", "bigram", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.k", "l0.mix.v", "l0.mix.o",
            "l1.mix.q", "l1.mix.o", "l0.mlp.router", "l0.mlp.correction", "l0.mlp.e5.up", "l0.mlp.e0.down",
            "l0.mlp.shared.up", "l2.mlp.e4.down"} <= set(names)
    assert "l1.mix.k" not in names and "l1.mix.v" not in names and "l0.mlp.e6.up" not in names
    assert tuple(names["bigram"].shape) == (98, 64) and tuple(names["l0.mix.v"].shape) == (48, 64)
    assert tuple(names["l0.mix.o"].shape) == (64, 96)
    assert model.token_state_ints() == 2


def test_pinned_pages_ahead_of_a_ring():
    book = SlotBook(2, [12], [3], 64, pinned=[2])
    s = book.acquire()
    book.reserve(s, 64 * 9 + 1)
    book.commit(s, 64 * 9 + 1)
    assert len(book.pages(s, 0)) == 5 and book.pages_needed(0, 10_000) == 5 and book.pages_needed(0, 65) == 2
    assert not book.audit()
    t = book.acquire()
    book.reserve(t, 130)
    book.commit(t, 130)
    assert len(book.pages(t, 0)) == 3 and not set(book.pages(t, 0)) & set(book.pages(s, 0))
    book.release(s)
    book.release(t)
    assert book.pools[0].available == 12


def _logits(cfg, weights, tokens):
    return plain.forward(tokens, cfg, weights)


@pytest.fixture(scope="module")
def model_p(tmp_path_factory):
    folder = vh.make_folder(tmp_path_factory.mktemp("plainP"), vh.CONFIGS["P"], seed=11, attn_gain=12.0)
    o = vh.Oracle(folder)
    return o.config, o.weights


def test_the_oracle_shows_one_key_the_sink_and_the_pair_table(model_p):
    cfg, w = model_p
    tokens = vh.random_requests(cfg, [160], seed=1)[0]
    ref = _logits(cfg, w, tokens)
    scale = np.sqrt((ref ** 2).mean())

    def moved(edit, rows):
        other = _logits(vh.variant(cfg, edit), w, tokens)
        return np.abs(other - ref)[rows].max() / scale

    def unmoved(edit, rows):
        other = _logits(vh.variant(cfg, edit), w, tokens)
        return np.abs(other - ref)[rows].max() == 0.0

    first_full = 70                                        # the first query whose window no longer reaches key 0
    win = lambda d: (lambda c: c["layers"][2]["mixer"]["mask"].__setitem__("size", 70 + d))
    assert moved(win(1), slice(first_full + 3, None)) > 0.01 and moved(win(-1), slice(first_full, None)) > 0.01
    assert unmoved(win(1), slice(0, 70))                    # before the window is full its size does not matter
    keep = lambda d: (lambda c: c["layers"][2]["mixer"]["mask"].__setitem__("keep_first", 3 + d))
    assert moved(keep(1), slice(80, None)) > 0.01 and moved(keep(-1), slice(80, None)) > 0.01
    assert unmoved(keep(1), slice(0, 70))
    rd = lambda c: c["layers"][1]["mixer"]["mask"].__setitem__("size", 34)
    assert moved(rd, slice(40, None)) > 0.01                # the reading layer's own window
    assert moved(lambda c: c["embedding"]["bigram"].__setitem__("mul_prev", 8), slice(1, None)) > 0.01
    assert unmoved(lambda c: c["embedding"]["bigram"].__setitem__("mul_prev", 8), slice(0, 1))
    assert moved(lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 3), slice(0, None)) > 0.01
    # the sink: without it the weights sum to one
    s = np.array([[0.3, -1.0, 2.0]])
    p = plain.sink_softmax(s, np.ones_like(s, dtype=bool))
    e = np.exp(s)
    assert np.allclose(p, e / (1 + e.sum())) and p.sum() < 1
    # a lone very negative score: the sink takes nearly everything
    assert plain.sink_softmax(np.array([[-30.0]]), np.ones((1, 1), dtype=bool))[0, 0] < 1e-12


def test_the_oracle_one_function_at_a_time():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(5, 2, 8))
    pos = np.array([0, 1, 2, 7, 100])
    y = plain.rotate_leading(x, pos, 4, 10000.0)
    assert np.array_equal(y[..., 4:], x[..., 4:]) and np.array_equal(y[0], x[0])
    # pairs (0, 2) and (1, 3); lengths of pairs are kept; angle of pair 0 at position p is p
    assert np.allclose(y[..., 0] ** 2 + y[..., 2] ** 2, x[..., 0] ** 2 + x[..., 2] ** 2)
    assert np.allclose(y[1, 0, 0], x[1, 0, 0] * np.cos(1.0) - x[1, 0, 2] * np.sin(1.0))
    assert np.allclose(y[3, 1, 3], x[3, 1, 3] * np.cos(7 * 0.01) + x[3, 1, 1] * np.sin(7 * 0.01))
    m = plain.visible(8, 3, 2)
    assert m[7].tolist() == [True, True, False, False, False, True, True, True] and m[2].tolist() == [True] * 3 + [False] * 5
    assert plain.hashed_pair_rows([5, 7, 7], 3, 10, 11).tolist() == [11, (5 * 3 + 70) % 11, (21 + 70) % 11]
    h = rng.normal(size=(1, 6))
    w = {"router": rng.normal(size=(3, 6)), "correction": np.array([0.0, 5.0, 0.0]),
         **{f"e{e}.{n}": rng.normal(size=s) for e in range(3) for n, s in (("up", (4, 6)), ("down", (6, 4)))}}
    out = plain.routed_experts(h, w, {"router": {"experts": 3, "top": 1, "scale": 2.0}})
    gate = 1 / (1 + np.exp(-(h @ w["router"].T)))[0]
    # the correction decides the choice (expert 1), the weight is the plain gate times the scale
    assert np.allclose(out[0], 2.0 * gate[1] * (np.maximum(h @ w["e1.up"].T, 0) ** 2 @ w["e1.down"].T)[0])


def test_the_cpu_model_serves_the_design(tmp_path):
    """The package's own CPU model (float32 numpy operators; what `--device cpu` and `--test` of the command line run)
    against the plain oracle, prompt in one step and then token by token."""
    from llaisys_b200.models.cpu_model import CpuModel
    for name in ("P", "R"):
        cfg = vh.CONFIGS[name]
        folder = vh.make_folder(tmp_path / name, cfg, seed=3, attn_gain=8.0)
        oracle = vh.Oracle(folder)
        tokens = vh.random_requests(cfg, [90], seed=2)[0]
        model = CpuModel.from_folder(folder)
        got = np.concatenate([model.step(tokens[:70])] + [model.step([t]) for t in tokens[70:]])
        assert np.abs(got - oracle.logits(tokens)).max() < 2e-4
        new = model.generate(tokens[:5], 4)
        assert len(new) == 4 and new[0] == int(np.argmax(oracle.logits(tokens[:5])[-1]))
