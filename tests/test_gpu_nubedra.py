"""The Nubedra design on the GPU against its plain implementation: every mechanism alone, then whole models under every
way of cutting requests into steps, then generation and replay through the entry points."""
import json
import subprocess
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import nubedra_helpers as nh
import plain_nubedra as plain
from helpers import build_engine, compare, run_batches, run_chunked, run_mixed, run_tail_by_one, run_whole, tolerance
from nubedra_helpers import compare as compare_nb

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
DTYPES = [torch.float32, torch.bfloat16]
DEV = "cuda:0"


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def _bf16_exact(a):
    """float64 array rounded to values bfloat16 holds exactly, so both sides start from the same numbers."""
    return torch.from_numpy(np.asarray(a)).to(torch.bfloat16).to(torch.float64).numpy()


def _dev(a, dtype):
    return torch.from_numpy(np.asarray(a)).to(dtype).to(DEV)


def _env(dtype):
    from llaisys_b200.parts import BuildEnv
    return BuildEnv(dtype, torch.device(DEV))


# ----------------------------------------------------------------------------- each mechanism alone
@pytest.mark.parametrize("H", [44, 300, 2048])
@pytest.mark.parametrize("dtype", DTYPES)
def test_normed_output_into_the_stream_and_the_next_norm(dtype, H):
    from llaisys_b200.config import PartSpec
    from llaisys_b200.parts import build_part
    rng = np.random.default_rng(2)
    x, d = rng.normal(size=(9, H)) * 3, _bf16_exact(rng.normal(size=(9, H)) * 0.01)
    w_post, w_next = _bf16_exact(rng.uniform(-0.5, 0.5, size=H)), _bf16_exact(rng.uniform(-0.5, 0.5, size=H))
    spec = {"size": H, "eps": 1e-5, "tensor": "", "offset": 1.0}
    post, nxt = build_part("norm", PartSpec("rms_norm", spec), _env(dtype)), build_part("norm", PartSpec("rms_norm", spec), _env(dtype))
    post.load({"": _dev(w_post, dtype)})
    nxt.load({"": _dev(w_next, dtype)})
    xf = x.astype(np.float32).astype(np.float64)
    want_x = xf + 0.7 * plain.norm_offset(d, w_post, 1e-5)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for then in (None, nxt):
        stream = torch.from_numpy(x).float().to(DEV)
        out = post.forward_scaled_add(stream, _dev(d, torch.float32), 0.7, then=then)
        assert np.abs(stream.cpu().numpy() - want_x).max() < 2e-5          # the stream is float32 in both precisions
        if then is not None:
            assert np.abs(out.float().cpu().numpy() - plain.norm_offset(want_x, w_next, 1e-5)).max() < tol
    # the plain norm of the stream through the same weights
    got = nxt.forward(torch.from_numpy(x).float().to(DEV))
    assert np.abs(got.float().cpu().numpy() - plain.norm_offset(xf, w_next, 1e-5)).max() < tol


@pytest.mark.parametrize("act", ["relu", "silu", "gelu_tanh"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_feed_forward_with_a_chosen_activation(dtype, act):
    from llaisys_b200.config import PartSpec
    from llaisys_b200.parts import build_part
    rng = np.random.default_rng(4)
    T, H, I = 37, 40, 52
    w = {"gate": _bf16_exact(rng.normal(size=(I, H)) * 0.3), "up": _bf16_exact(rng.normal(size=(I, H)) * 0.3),
         "down": _bf16_exact(rng.normal(size=(H, I)) * 0.3)}
    h = _bf16_exact(rng.normal(size=(T, H)))
    g, u = h @ w["gate"].T, h @ w["up"].T
    a = {"relu": np.maximum(g, 0), "silu": plain.silu(g),
         "gelu_tanh": 0.5 * g * (1 + np.tanh(np.sqrt(2 / np.pi) * (g + 0.044715 * g ** 3)))}[act]
    want = (a * u) @ w["down"].T
    if act == "relu":
        assert np.abs(want - plain.dense_ff(h, {"p." + k: v for k, v in w.items()}, "p")).max() < 1e-12
    part = build_part("ffn", PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I, "act": act,
                                                    "names": {"gate": "gate", "up": "up", "down": "down"}}), _env(dtype))
    part.load({n: _dev(v, dtype) for n, v in w.items()})
    got = part.forward(_dev(h, dtype), None)
    assert got.dtype == torch.float32
    assert np.abs(got.cpu().numpy() - want).max() < (2e-5 if dtype == torch.float32 else 3e-2) * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("yarn", [None, dict(zip(("factor", "original", "fast", "slow"), nh.YARN_A)),
                                  dict(zip(("factor", "original", "fast", "slow"), nh.YARN_B))])
@pytest.mark.parametrize("dims", [0, 6, 10])
def test_rotation_of_neighbouring_pairs_in_the_per_head_product(dims, yarn):
    """The tables of the position part, applied by the kernel that also carries the queries into the latent space."""
    from llaisys_b200 import kernels
    from llaisys_b200.config import PartSpec
    from llaisys_b200.parts import build_part
    rng = np.random.default_rng(3)
    H, n_in, n_out, tail, T = 3, 7, 150, 10, 21
    x = rng.normal(size=(T, H, n_in + tail))
    m = rng.normal(size=(H, n_in, n_out))
    pos = rng.integers(0, 700, size=T)
    part = build_part("position", PartSpec("rope_interleaved", {"width": tail, "dims": dims, "base": 777.0, "yarn": yarn}), _env(torch.float32))
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    y = kernels.head_matmul(_dev(x.reshape(T, -1), torch.float32), _dev(m, torch.float32), tail=tail, tables=part.pair_tables(700),
                            tok_pos=_i32(pos), err=err).cpu().numpy().reshape(T, H, n_out + tail)
    xf = x.astype(np.float32).astype(np.float64)
    mf = m.astype(np.float32).astype(np.float64)
    assert np.abs(y[:, :, :n_out] - np.einsum("thi,hio->tho", xf[:, :, :n_in], mf)).max() < 1e-4
    assert np.abs(y[:, :, n_out:] - plain.rotate_interleaved(xf[:, :, n_in:], pos, dims, 777.0, yarn)).max() < 3e-5
    assert np.array_equal(y[:, :, n_out + dims:], x.astype(np.float32)[:, :, n_in + dims:]) and int(err.item()) == 0
    # with a gate: every head's outputs times the logistic function of its gate
    gate = rng.normal(size=(T, H + 2)) * 3
    y = kernels.head_matmul(_dev(x[:, :, :n_in].reshape(T, -1), torch.float32), _dev(m, torch.float32),
                            gate=_dev(gate, torch.float32)[:, 1:]).cpu().numpy().reshape(T, H, n_out)
    gf = gate.astype(np.float32).astype(np.float64)
    assert np.abs(y - np.einsum("thi,hio->tho", xf[:, :, :n_in], mf) * plain.sigmoid(gf[:, 1:H + 1])[:, :, None]).max() < 1e-4


def _gla_part(dtype, H, dk, dv, tau, D, rank, rng):
    from llaisys_b200.config import PartSpec
    from llaisys_b200.parts import build_part
    w = {"q": rng.normal(size=(H * dk, D)) * 0.4, "k": rng.normal(size=(H * dk, D)) * 0.4, "v": rng.normal(size=(H * dv, D)) * 0.4,
         "g": rng.normal(size=(H * dv, D)) * 0.4, "o": rng.normal(size=(D, H * dv)) * 0.2, "norm": 1 + 0.3 * rng.normal(size=dv),
         "a1": rng.normal(size=(rank, D)) * 0.4, "a2": rng.normal(size=(H * dk, rank)) * 0.6, "a2.b": rng.uniform(-1, 5, size=H * dk)}
    w = {n: _bf16_exact(v) for n, v in w.items()}
    part = build_part("mixer", PartSpec("gated_linear_attention", {"hidden_size": D, "num_heads": H, "key_dim": dk, "value_dim": dv,
                                                                  "decay_root": tau, "query_scale": dk ** -0.5, "eps": 1e-5}), _env(dtype))
    part.load({n: _dev(v, dtype) for n, v in w.items()})
    return part, {"p." + n: v for n, v in w.items()}


@pytest.mark.parametrize("shape", [(2, 12, 40, 9.0, 24, 5), (1, 130, 4, 30.0, 40, 16), (3, 33, 33, 1.0, 20, 3), (4, 64, 64, 16.0, 64, 8)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_linear_attention_alone_with_state_carried_in_slots(dtype, shape):
    """Whole sequences, then the same sequences in portions (down to single tokens) interleaved in one batch, each
    carrying its state in a slot of its own; a slot that is used again starts from zero."""
    H, dk, dv, tau, D, rank = shape
    rng = np.random.default_rng(7)
    part, w = _gla_part(dtype, H, dk, dv, tau, D, rank, rng)
    assert part.rank == rank and part.state_size() == H * dk * dv
    seqs = [_bf16_exact(rng.normal(size=(n, D))) for n in (70, 1, 23)]
    mix = {"heads": H, "dim": dk, "vdim": dv, "tau": tau}
    want = [plain.gla_mixer(s, w, "p", mix, 1e-5) for s in seqs]
    state = torch.full((6, part.state_size()), 7.0, dtype=torch.float32, device=DEV)      # stale contents of earlier users
    slots = [4, 0, 2]
    tol = 2e-4 if dtype == torch.float32 else 6e-2

    def step(who, parts_):
        x = np.concatenate(parts_)
        starts = np.concatenate([[0], np.cumsum([len(p) for p in parts_])])
        ctx = SimpleNamespace(state=lambda call: state, seq_start=_i32(starts), seq_slot=_i32([slots[i] for i in who]), n_seqs=len(who))
        out = part.forward(_dev(x, dtype), ctx, 0).cpu().numpy()
        return [out[starts[j]:starts[j + 1]] for j in range(len(who))]

    for plans in ([[70], [1], [23]], [[3, 1, 1, 60, 5], [0, 1], [1, 2, 17, 1, 2]]):
        for s in slots:
            state[s].zero_()                                                      # what the cache does when a slot is acquired
        got = [[] for _ in seqs]
        fed = [0] * len(seqs)
        for k in range(max(len(p) for p in plans)):
            who = [i for i, p in enumerate(plans) if k < len(p) and p[k] > 0]
            outs = step(who, [seqs[i][fed[i]:fed[i] + plans[i][k]] for i in who])
            for i, o in zip(who, outs):
                got[i].append(o)
                fed[i] += plans[i][k]
        for i, (g, (y, S)) in enumerate(zip(got, want)):
            scale = max(1.0, np.abs(y).max())
            assert np.abs(np.concatenate(g) - y).max() < tol * scale, (plans, i)
            assert np.abs(state[slots[i]].cpu().numpy().reshape(S.shape) - S).max() < tol * max(1.0, np.abs(S).max()), (plans, i)
    assert float(state[1].min()) == 7.0 and float(state[5].max()) == 7.0          # other sequences' rows are untouched


def test_decay_of_the_recurrence_is_formed_in_float32():
    """Decay logits of large size in both directions: a = sigmoid(z)^(1/tau) must neither overflow nor lose the small
    difference from one that a long memory lives on."""
    from llaisys_b200 import kernels
    H, dk, dv, T = 1, 8, 4, 400
    rng = np.random.default_rng(5)
    z = np.array([-60.0, -8.0, -1.0, 0.0, 3.0, 9.0, 14.0, 40.0])[None, :].repeat(T, 0)
    q, k, v = rng.normal(size=(T, dk)), rng.normal(size=(T, dk)), rng.normal(size=(T, dv))
    proj = np.concatenate([q, k, v], axis=1)
    state = torch.zeros((1, dk * dv), dtype=torch.float32, device=DEV)
    o = kernels.gla_scan(_dev(proj, torch.float32), H, dk, dv, _dev(z, torch.float32), state, _i32([0, T]), _i32([0]), 1, 1.0, 16.0)
    a = plain.sigmoid(z.astype(np.float32).astype(np.float64)) ** (1 / 16.0)
    S, want = np.zeros((dk, dv)), np.zeros((T, dv))
    pf = proj.astype(np.float32).astype(np.float64)
    for t in range(T):
        S = a[t][:, None] * S + pf[t, dk:2 * dk][:, None] * pf[t, 2 * dk:][None, :]
        want[t] = S.T @ pf[t, :dk]
    assert np.isfinite(o.cpu().numpy()).all() and np.abs(o.cpu().numpy() - want).max() < 2e-3 * np.abs(want).max()


# ----------------------------------------------------------------------------- latent attention alone, on hand-made pages
def _paged(rows_by_seq, width, dtype, ring=None, n_pages=40, seed=0):
    """A pool with the sequences' rows at scattered physical pages; returns (pool, page table, modulus)."""
    rng = np.random.default_rng(seed)
    pool = torch.full((n_pages, 1, 64, width), 99.0, dtype=dtype, device=DEV)       # stale rows that must never be seen
    free = rng.permutation(n_pages).tolist()
    tables = []
    for rows in rows_by_seq:
        n_log = -(-len(rows) // 64)
        held = [free.pop() for _ in range(n_log if ring is None else min(n_log, ring))]
        for p in range(len(rows)):
            lp = p // 64
            if ring is None or lp + ring > (len(rows) - 1) // 64:
                pool[held[lp if ring is None else lp % ring], 0, p % 64] = torch.from_numpy(rows[p]).to(dtype).to(DEV)
        tables.append(held)
    width_t = max(len(t) for t in tables)
    table = np.zeros((len(tables), width_t), dtype=np.int32)
    for i, t in enumerate(tables):
        table[i, :len(t)] = t
    return pool, _i32(table), (ring if ring is not None else width_t)


def _plain_latent_rows(q, rows, value_width, window, scale, sink, first_pos):
    """q [n, H, width] at positions first_pos.., rows [L, width] at positions 0..: float64 softmax with a sink."""
    n, H, _ = q.shape
    out = np.zeros((n, H, value_width))
    for i in range(n):
        pos = first_pos + i
        lo = max(0, pos - window + 1) if window else 0
        s = np.einsum("hw,jw->hj", q[i], rows[lo:pos + 1]) * scale
        m = np.maximum(s.max(axis=1), sink)
        e = np.exp(s - m[:, None])
        out[i] = (e / (e.sum(axis=1) + np.exp(sink - m))[:, None]) @ rows[lo:pos + 1, :value_width]
    return out


@pytest.mark.parametrize("window", [None, 1, 63, 64, 65, 130])
@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_attention_alone_keys_at_the_windows_edge(dtype, window):
    """Rows are small except two that every query scores very high: one just inside the window of the last query and one
    just outside it (without a window: the sequence's very first row).  Prompts over cached history, single tokens with
    the key range cut into slices, and a ring that has wrapped."""
    from llaisys_b200 import kernels
    rng = np.random.default_rng(11)
    H, width, vw = 5, 40, 24
    L, n_new = 300, 70                                   # 230 cached rows, 70 new ones
    rows = _bf16_exact(rng.normal(size=(L, width)) * 0.3)
    qdir = rng.normal(size=width)
    qdir /= np.linalg.norm(qdir)
    last = L - 1
    inside = last - window + 1 if window else 0
    rows[inside] = _bf16_exact(rows[inside] + 4.0 * qdir)
    if window and inside >= 1:
        rows[inside - 1] = _bf16_exact(rows[inside - 1] + 6.0 * qdir)      # must not be seen by the last query
    q = _bf16_exact(rng.normal(size=(n_new, H, width)) * 0.5 + 3.0 * qdir)
    sink = rng.uniform(-2, 2, size=H).astype(np.float32)
    want = _plain_latent_rows(q, rows, vw, window, 0.8, sink.astype(np.float64), L - n_new)
    tol = 1e-4 if dtype == torch.float32 else 4e-2
    sinks = torch.from_numpy(sink).to(DEV)
    for ring in (None, (-(-(window - 1) // 64) + 1) if window else None):
        # prompt: history from the pool, the step's rows from the dense buffer
        pool, table, mod = _paged([rows[:L - n_new]], width, dtype, ring=ring, seed=window or 0)
        got = kernels.latent_attention(False, _dev(q.reshape(n_new, -1), dtype), H, width, vw, _dev(rows[L - n_new:], dtype), pool, table,
                                       mod, 0, _i32([0, n_new]), _i32([L - n_new]), 1, n_new, window, 0.8, sinks)
        assert np.abs(got.float().cpu().numpy().reshape(n_new, H, vw) - want).max() < tol, ("prompt", ring)
        # the same with every row in the pool already (what a layer sees that reads another layer's cache)
        if ring is None:
            pool, table, mod = _paged([rows], width, dtype, seed=1)
            got = kernels.latent_attention(False, _dev(q.reshape(n_new, -1), dtype), H, width, vw, None, pool, table, mod, 0,
                                           _i32([0, n_new]), _i32([L - n_new]), 1, n_new, window, 0.8, sinks)
            assert np.abs(got.float().cpu().numpy().reshape(n_new, H, vw) - want).max() < tol, "prompt from the cache"
        # single token: the last position, all rows in the pool, in a batch with a short second sequence
        other = _bf16_exact(rng.normal(size=(3, width)))
        pool, table, mod = _paged([rows, other], width, dtype, ring=ring, seed=2)
        q2 = np.concatenate([q[-1:], q[:1]])
        want2 = _plain_latent_rows(q[:1], other, vw, window, 0.8, sink.astype(np.float64), 2)
        for splits in (1, 2, 5):
            got = kernels.latent_attention(True, _dev(q2.reshape(2, -1), dtype), H, width, vw, None, pool, table, mod, 0,
                                           _i32([0, 1, 2]), _i32([L - 1, 2]), 2, 1, window, 0.8, sinks, n_splits=splits)
            got = got.float().cpu().numpy().reshape(2, H, vw)
            assert np.abs(got[0] - want[-1]).max() < tol and np.abs(got[1] - want2[0]).max() < tol, ("token", ring, splits)


@pytest.mark.parametrize("sizes", [(272, 264), (600, 560)])
def test_latent_attention_rows_wider_than_a_block_of_queries_allows(sizes):
    """Cache rows of more than 256 elements; the widest run with fewer query rows a block."""
    from llaisys_b200 import kernels
    rng = np.random.default_rng(12)
    (width, vw), H, L = sizes, 3, 150
    rows = _bf16_exact(rng.normal(size=(L, width)) * 0.3)
    q = _bf16_exact(rng.normal(size=(L, H, width)) * 0.4)
    sink = np.zeros(H)
    want = _plain_latent_rows(q, rows, vw, 100, 0.5, sink, 0)
    pool, table, mod = _paged([rows[:0]], width, torch.float32)
    got = kernels.latent_attention(False, _dev(q.reshape(L, -1), torch.float32), H, width, vw, _dev(rows, torch.float32), pool, table, mod, 0,
                                   _i32([0, L]), _i32([0]), 1, L, 100, 0.5, torch.zeros(H, device=DEV))
    assert np.abs(got.cpu().numpy().reshape(L, H, vw) - want).max() < 1e-4


# ----------------------------------------------------------------------------- single layers at window and page edges
WINDOWS = [64, 65, 63, 1, 500, 70, 128]


@pytest.mark.parametrize("shared", [False, True])
@pytest.mark.parametrize("window", WINDOWS)
def test_latent_layers_at_window_and_page_edges(tmp_path, window, shared):
    """float32, sharp scores: one key too many or too few moves the logits far beyond the tolerance.  shared: a second
    layer reads the first one's cache through a window one key narrower (the cache then keeps every row and the window is
    a mask; else the layer's cache is a ring of pages)."""
    layers = [nh.latent(3, 8, 8, 12, 24, 20, window, scaling=nh.YARN_A)]
    if shared:
        layers.append(nh.latent(2, 4, 8, 6, 16, 20, max(1, window - 1), kv_from=0, scaling=nh.YARN_A, ff=40))
    cfg = nh.config(101, 32, layers, embed_scale=2.0, mult=0.8)
    folder = nh.make_folder(tmp_path, cfg, seed=window * 7, gain=9.0)
    oracle = nh.Oracle(folder)
    requests = nh.random_requests(cfg, [1, 200, 66, 131], seed=5)
    engine = build_engine(folder, torch.float32, max_tokens=64 * 4 + 64, max_seqs=2)
    assert (engine.cache.rings[0] is None) == shared
    like = nh.like_config(cfg)
    compare(run_whole(engine, requests), oracle, requests, torch.float32, like, f"window {window} whole")
    compare(run_tail_by_one(engine, requests, tail=140), oracle, requests, torch.float32, like, f"window {window} decoded")
    compare(run_chunked(engine, requests, [63, 2, 65, 1, 64]), oracle, requests, torch.float32, like, f"window {window} portions")
    assert not engine.cache.live_slots


@pytest.mark.parametrize("window", [1, 33, 64, 65, 500])
def test_whole_prompts_on_the_tensor_cores_against_the_path_over_the_cache(tmp_path, window, monkeypatch):
    """bfloat16, heads whose query/key and value sizes are equal: whole prompts make the heads' keys and values from the
    step's rows and run on the tensor cores; with that path switched off the same prompts run over the latent rows.
    Both get the same weights; with sharp scores (a lost key would show) they may differ only by rounding, and both agree
    with the plain implementation.  Prompts of a batch are unequal; decoding afterwards reads what the prompts cached."""
    from llaisys_b200.kernels import ops
    cfg = nh.config(101, 32, [
        nh.latent(3, 8, 8, 16, 24, 24, window, scaling=nh.YARN_A),                               # a ring of its own
        nh.latent(2, 16, 16, 32, 16, 40, max(1, window - 1), ff=40, scaling=nh.YARN_B),          # read by the next layer
        nh.latent(2, 48, 16, 64, 24, 40, window, kv_from=1, scaling=nh.YARN_B),
    ], embed_scale=2.0, mult=0.8)
    folder = nh.make_folder(tmp_path, cfg, seed=window, gain=nh.GAIN[torch.bfloat16])
    oracle = nh.Oracle(folder)
    requests = nh.random_requests(cfg, [1, 200, 66, 131], seed=5)
    got = {}
    for mma in (True, False):
        monkeypatch.setattr(ops, "MMA_ATTENTION", mma)
        engine = build_engine(folder, torch.bfloat16, max_tokens=64 * 7, max_seqs=2)
        used = [p for b in engine.model.blocks for sub in b.sublayers for p in [sub.part] if getattr(p, "w_kv_heads", None) is not None]
        assert len(used) == 3
        n0 = ops.launch_count()
        got[mma] = [run_whole(engine, requests), run_batches(engine, requests, [[1, 3], [0, 2]], [1, 150, 30, 70])]
        got[mma].append(ops.launch_count() - n0)
        for g in got[mma][:2]:
            compare_nb(g, oracle, requests, torch.bfloat16, cfg, f"tensor cores {mma}, window {window}")
        assert not engine.cache.live_slots
    assert got[True][2] != got[False][2]                                   # the two paths are not the same launches
    for a, b in zip(got[True][:2], got[False][:2]):
        for key in b:
            ref = b[key].astype(np.float64)
            rms = np.sqrt((ref ** 2).mean())
            d = a[key] - ref
            # (a window of one key leaves a weight e^s / (e^s + e^sink) per head, which follows the score's rounding directly)
            assert np.sqrt((d ** 2).mean()) <= (0.03 if window > 1 else 0.08) * rms + 2e-4, (window, key)


def test_latent_layers_without_a_window_and_without_rotation(tmp_path):
    """No mask in the configuration: every earlier key is seen (own cache, and a reader of it); no rotated dimensions."""
    cfg = nh.config(77, 40, [nh.latent(2, 8, 4, 6, 12, 10, 5, rot_dims=0), nh.latent(3, 4, 4, 8, 8, 10, 5, kv_from=0, rot_dims=0, ff=24),
                             nh.latent(2, 6, 2, 4, 8, 6, 5, ff=16)], embed_scale=1.5, mult=0.9)
    for layer in cfg["layers"]:
        del layer["mixer"]["mask"]
    folder = nh.make_folder(tmp_path, cfg, seed=8, gain=9.0)
    oracle, requests = nh.Oracle(folder), nh.random_requests(cfg, [150, 3, 70], seed=4)
    engine = build_engine(folder, torch.float32, max_tokens=64 * 6)
    assert engine.cache.rings == [None, None] or engine.cache.rings == [None]
    like = nh.like_config(cfg)
    compare(run_whole(engine, requests), oracle, requests, torch.float32, like, "no window whole")
    compare(run_tail_by_one(engine, requests, tail=80), oracle, requests, torch.float32, like, "no window decoded")
    compare(run_batches(engine, requests, [[0, 1, 2]], [100, 1, 64]), oracle, requests, torch.float32, like, "no window together")


def test_a_model_of_recurrent_layers_only(tmp_path):
    """No layer keeps keys: the cache has no page groups at all, only state rows."""
    cfg = nh.config(61, 24, [nh.gla(2, 8, 12, 3.0, ff=32), nh.gla(3, 4, 8, 20.0)], embed_scale=1.2, mult=0.75)
    for dtype in DTYPES:
        folder = nh.make_folder(tmp_path / str(dtype), cfg, seed=6, gain=nh.GAIN[dtype])
        oracle, requests = nh.Oracle(folder), nh.random_requests(cfg, [90, 2, 40], seed=3)
        engine = build_engine(folder, dtype, max_tokens=64 * 4)
        assert engine.cache.group_keys == []
        compare_nb(run_whole(engine, requests), oracle, requests, dtype, cfg, "recurrent only whole")
        compare_nb(run_batches(engine, requests, [[0, 1, 2]], [30, 1, 40]), oracle, requests, dtype, cfg, "recurrent only together")
        assert not engine.cache.live_slots


def test_the_sequences_first_tokens(tmp_path):
    """One, two and three tokens: empty history, a state that starts at zero, a softmax over one key and the sink."""
    cfg = nh.CONFIGS["P"]
    for dtype in DTYPES:
        folder = nh.make_folder(tmp_path / str(dtype), cfg, seed=2, gain=nh.GAIN[dtype])
        oracle, requests = nh.Oracle(folder), nh.random_requests(cfg, [1, 2, 3, 1], seed=9)
        engine = build_engine(folder, dtype, max_tokens=64 * 4)
        compare_nb(run_whole(engine, requests), oracle, requests, dtype, cfg, "first tokens whole")
        compare_nb(run_tail_by_one(engine, requests, tail=10), oracle, requests, dtype, cfg, "first tokens one by one")
        compare_nb(run_batches(engine, requests, [[0, 1, 2, 3]], [1, 1, 2, 1]), oracle, requests, dtype, cfg, "first tokens together")


# ----------------------------------------------------------------------------- whole models under every schedule
LENGTHS = {"P": [1, 2, 64, 71, 150, 300], "Q": [3, 65, 129, 40], "R": [1, 66, 67, 200, 131]}


class Model:
    def __init__(self, name, tmp):
        self.name, self._tmp, self._made = name, tmp, {}

    def at(self, dtype):
        if dtype not in self._made:
            cfg = nh.CONFIGS[self.name]
            folder = nh.make_folder(self._tmp / str(dtype), cfg, seed=ord(self.name), gain=nh.GAIN[dtype])
            self._made[dtype] = (cfg, folder, nh.Oracle(folder), nh.random_requests(cfg, LENGTHS[self.name], seed=ord(self.name)))
        return self._made[dtype]


@pytest.fixture(scope="module", params=["P", "Q", "R"])
def model(request, tmp_path_factory):
    return Model(request.param, tmp_path_factory.mktemp(f"nb{request.param}"))


def _rooms(requests):
    return sum(-(-len(r) // 64) * 64 for r in requests)


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_prompts_and_token_by_token(model, dtype):
    cfg, folder, oracle, requests = model.at(dtype)
    engine = build_engine(folder, dtype, max_tokens=max(_rooms([r]) for r in requests))
    compare_nb(run_whole(engine, requests), oracle, requests, dtype, cfg, f"{model.name} whole")
    compare_nb(run_tail_by_one(engine, requests, tail=10_000), oracle, requests, dtype, cfg, f"{model.name} token by token")
    compare_nb(run_tail_by_one(engine, requests, tail=32), oracle, requests, dtype, cfg, f"{model.name} tail")
    assert not engine.cache.live_slots


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batches_with_pages_and_slots_used_again(model, dtype):
    cfg, folder, oracle, requests = model.at(dtype)
    n = len(requests)
    batches = [list(range(0, n, 2)), list(range(1, n, 2))]
    prompt_lens = [max(1, len(r) - (3 + 5 * i)) for i, r in enumerate(requests)]
    room = max(_rooms([requests[r] for r in b]) for b in batches)
    engine = build_engine(folder, dtype, max_tokens=room, max_seqs=len(batches[0]))
    compare_nb(run_batches(engine, requests, batches, prompt_lens), oracle, requests, dtype, cfg, f"{model.name} batches")
    assert not engine.cache.live_slots
    assert [p.available for p in engine.cache.book.pools] == engine.cache.group_pages
    compare_nb(run_batches(engine, requests, batches[::-1], prompt_lens), oracle, requests, dtype, cfg, f"{model.name} batches again")


@pytest.mark.parametrize("dtype", DTYPES)
def test_portions_and_mixed_steps(model, dtype):
    cfg, folder, oracle, _ = model.at(dtype)
    requests = nh.random_requests(cfg, [200, 300, 129, 9], seed=41)
    engine = build_engine(folder, dtype, max_tokens=320)
    for cuts in ([70, 60, 1000], [63, 1, 64, 65, 2, 1000], [2, 200, 1000], [64], [2]):
        reqs = requests if cuts != [2] else requests[2:]
        compare_nb(run_chunked(engine, reqs, cuts), oracle, reqs, dtype, cfg, f"{model.name} portions {cuts}")
    requests = nh.random_requests(cfg, [120, 100, 210, 33], seed=43)
    plans = [[50, 1, 1, 1, 40, 1, 0, 1], [0, 0, 90], [70, 60, 0, 40, 1, 1, 30], [1, 1, 1]]
    engine = build_engine(folder, dtype, max_tokens=_rooms(requests), max_seqs=4)
    for turn in range(2):
        compare_nb(run_mixed(engine, requests, plans), oracle, requests, dtype, cfg, f"{model.name} mixed steps, turn {turn}")
        assert not engine.cache.live_slots
        requests, plans = requests[::-1], plans[::-1]


def test_long_decoding_through_captured_steps(tmp_path):
    """Hundreds of single-token steps from a short prompt: the rings wrap several times, the recurrent state is carried
    through every step, and the steps are replayed from a captured graph."""
    for dtype in DTYPES:
        cfg = nh.CONFIGS["Q"]
        folder = nh.make_folder(tmp_path / str(dtype), cfg, seed=21, gain=nh.GAIN[dtype])
        oracle = nh.Oracle(folder)
        requests = nh.random_requests(cfg, [330, 290], seed=6)
        engine = build_engine(folder, dtype, max_tokens=_rooms(requests), max_seqs=2)
        assert engine.use_graphs
        compare_nb(run_batches(engine, requests, [[0, 1]], [4, 1]), oracle, requests, dtype, cfg, "long decoding")
        assert engine.graph_replays > 250


# ----------------------------------------------------------------------------- entry points
def _greedy(oracle, prompt, n):
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(np.argmax(oracle.logits(seq)[-1])))
    return seq[len(prompt):]


def test_greedy_generation_through_the_entry_point_and_scheduler(tmp_path):
    from llaisys_b200.models import CausalLM, DeviceType
    cfg = nh.CONFIGS["P"]
    folder = nh.make_folder(tmp_path, cfg, seed=31, gain=8.0)
    oracle = nh.Oracle(folder)
    model = CausalLM(folder, DeviceType.NVIDIA, dtype="float32", max_tokens=64 * 4)
    prompts = nh.random_requests(cfg, [5, 9, 2, 70, 1, 17], seed=3)
    # four rooms of 64 tokens for six requests: two batches at least, slots, pages and state rows are used again
    outs = model.generate_batch(prompts, max_new_tokens=12, top_k=1, stop_ids=[])
    for p, new in zip(prompts, outs):
        assert new == _greedy(oracle, p, 12)
    assert model.generate(prompts[0], max_new_tokens=12) == prompts[0] + outs[0]
    assert not model.engine.cache.live_slots


def test_command_line(tmp_path):
    """python -m llaisys_b200.cli on a model folder of this design: --test compares the engine's tokens with those of
    the package's CPU model; --random-weights writes a folder from a configuration first."""
    import os
    import sys
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    folder = nh.make_folder(tmp_path / "m", nh.CONFIGS["P"], seed=17, gain=8.0)
    (tmp_path / "batch.txt").write_text("5,17,3,200,7,7,7,7,7\n[9, 8]\n1\n")
    out = subprocess.run([sys.executable, "-m", "llaisys_b200.cli", "--model", str(folder), "--batch-file", str(tmp_path / "batch.txt"),
                          "--max_steps", "6", "--test", "--dtype", "float32"], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.count("Tokens:") == 3 and "Test passed" in out.stdout
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(nh.CONFIGS["Q"]))
    out = subprocess.run([sys.executable, "-m", "llaisys_b200.cli", "--random-weights", str(cfg), "--seed", "3", "--tokens", "1,2,3",
                          "--max_steps", "4", "--test", "--dtype", "bfloat16"], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "Test passed" in out.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_of_a_trace(tmp_path, dtype):
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    cfg = nh.CONFIGS["P"]
    folder = nh.make_folder(tmp_path / "m", cfg, seed=13, gain=nh.GAIN[td])
    requests = nh.random_requests(cfg, [1, 7, 90, 20], seed=8)
    lines, rows = [], []
    # requests 0, 2 together, then decoded together; then 1 and 3 whole
    lines.append({"step": 0, "entries": [{"id": "a", "tokens": requests[0], "want": [0]},
                                         {"id": "c", "tokens": requests[2][:60], "want": list(range(60))}], "end": ["a"]})
    rows.append((0, [(0, 0)] + [(2, p) for p in range(60)]))
    for p in range(60, 90):
        lines.append({"step": p, "entries": [{"id": "c", "tokens": [requests[2][p]], "want": [0]}], "end": ["c"] if p == 89 else []})
        rows.append((p, [(2, p)]))
    lines.append({"step": 500, "entries": [], "end": []})
    lines.append({"step": 501, "entries": [{"id": "b", "tokens": requests[1], "want": list(range(7))},
                                           {"id": "d", "tokens": requests[3], "want": [19]}], "end": ["b", "d"]})
    rows.append((501, [(1, p) for p in range(7)] + [(3, 19)]))
    out_dir = tmp_path / "out"
    proc = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out_dir),
                           "--max-tokens", "128"], input="\n".join(json.dumps(l) for l in lines) + "\n", capture_output=True,
                          text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [int(l.split()[1]) for l in proc.stdout.splitlines() if l.startswith("done ")] == [l["step"] for l in lines]
    oracle = nh.Oracle(folder)
    for step, keys in rows:
        data = np.frombuffer((out_dir / f"{step}.f32").read_bytes(), dtype="<f4").reshape(len(keys), cfg["vocab"])
        for i, (r, p) in enumerate(keys):
            ref = oracle.logits(requests[r])
            # (bfloat16: single rows may lie in the heavy tail that nubedra_helpers.compare describes)
            assert np.abs(data[i] - ref[p]).max() <= tolerance(td, nh.like_config(cfg), ref) * (1 if dtype == "float32" else 8), (step, r, p)
