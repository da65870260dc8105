"""The Vumezen design on the GPU against its plain implementation: every mechanism alone, then whole models under every
way of cutting requests into steps, then generation and replay through the entry points."""
import json
import subprocess
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_vumezen as plain
import vumezen_helpers as vh
from helpers import build_engine, compare, run_batches, run_chunked, run_mixed, run_tail_by_one, run_whole, tolerance

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
DTYPES = [torch.float32, torch.bfloat16]
DEV = "cuda:0"


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def _bf16_exact(a):
    """float64 array rounded to values bfloat16 holds exactly, so both sides start from the same numbers."""
    return torch.from_numpy(np.asarray(a)).to(torch.bfloat16).to(torch.float64).numpy()


# ----------------------------------------------------------------------------- each mechanism alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_scaled_embedding_with_pair_rows_across_steps(dtype):
    from llaisys_b200 import kernels
    rng = np.random.default_rng(1)
    V, H, buckets, a, b = 50, 24, 13, 1000003, 77
    table, pair = _bf16_exact(rng.normal(size=(V, H))), _bf16_exact(rng.normal(size=(buckets + 1, H)))
    seqs = [rng.integers(0, V, size=n).tolist() for n in (7, 1, 12)]
    want = [plain.embed(s, table, 2.5, pair, {"buckets": buckets, "mul_prev": a, "mul_cur": b}) for s in seqs]
    last = torch.full((8, 2), -1, dtype=torch.int32, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    tt, tp = torch.from_numpy(table).to(dtype).to(DEV), torch.from_numpy(pair).to(dtype).to(DEV)
    slots = [5, 0, 3]
    got = [[] for _ in seqs]
    # step 1: the first 3, 1, 2 tokens; step 2: sequences 0 and 2 bring one token each; step 3: the rest of both
    plans = [[3, 1, 2], [1, 0, 1], [3, 0, 9]]
    fed = [0, 0, 0]
    for plan in plans:
        who = [i for i, n in enumerate(plan) if n]
        toks, pos, seq, start = [], [], [], [0]
        for j, i in enumerate(who):
            toks += seqs[i][fed[i]:fed[i] + plan[i]]
            pos += list(range(fed[i], fed[i] + plan[i]))
            seq += [j] * plan[i]
            start.append(len(toks))
        ctx = SimpleNamespace(tokens=_i32(toks), tok_pos=_i32(pos), tok_seq=_i32(seq), seq_start=_i32(start),
                              seq_slot=_i32([slots[i] for i in who]), err=err)
        out = kernels.embedding_pair(ctx, tt, 2.5, tp, buckets, a, b, last).cpu().numpy()
        for j, i in enumerate(who):
            got[i].append(out[start[j]:start[j + 1]])
            fed[i] += plan[i]
    assert int(err.item()) == 0
    for g, w in zip(got, want):
        assert np.abs(np.concatenate(g) - w).max() < 1e-5
    # a step that does not follow the one before it is reported, not computed silently
    ctx = SimpleNamespace(tokens=_i32([1]), tok_pos=_i32([3]), tok_seq=_i32([0]), seq_start=_i32([0, 1]), seq_slot=_i32([5]), err=err)
    kernels.embedding_pair(ctx, tt, 2.5, tp, buckets, a, b, last)
    assert int(err.item()) == 3


@pytest.mark.parametrize("H", [44, 2048])
@pytest.mark.parametrize("dtype", DTYPES)
def test_one_root_mean_square_two_weights(dtype, H):
    from llaisys_b200 import kernels
    rng = np.random.default_rng(2)
    x = rng.normal(size=(9, H)) * 3
    w = [_bf16_exact(1 + 0.1 * rng.normal(size=H)) for _ in range(2)]
    outs = kernels.rmsnorm_multi(torch.from_numpy(x).float().to(DEV), [torch.from_numpy(v).to(dtype).to(DEV) for v in w], 1e-5, dtype)
    one = kernels.rmsnorm_multi(torch.from_numpy(x).float().to(DEV), [torch.from_numpy(w[1]).to(dtype).to(DEV)], 1e-5, dtype)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    xf = x.astype(np.float32).astype(np.float64)
    for o, v in zip(outs + one, w + [w[1]]):
        assert np.abs(o.float().cpu().numpy() - plain.rms_norm(xf, v, 1e-5)).max() < tol


@pytest.mark.parametrize("dims", [0, 4, 10, 16])
def test_rotation_of_leading_dimensions(dims):
    from llaisys_b200 import kernels
    from llaisys_b200.config import PartSpec
    from llaisys_b200.parts import BuildEnv, build_part
    rng = np.random.default_rng(3)
    nh, nkv, dk, dv, T = 3, 2, 16, 6, 11
    x = rng.normal(size=(T, nh * dk + nkv * dk + nkv * dv))
    pos = rng.integers(0, 500, size=T)
    part = build_part("position", PartSpec("rope_leading", {"head_dim": dk, "dims": dims, "base": 777.0}),
                      BuildEnv(torch.float32, torch.device(DEV)))
    t = part.leading_tables(500)
    proj = torch.from_numpy(x).float().to(DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.rope_lead_append(proj, nh, nkv, dk, dv, dims, cos=t[0] if t else None, sin=t[1] if t else None, tok_pos=_i32(pos), err=err)
    xf = x.astype(np.float32).astype(np.float64)
    want = xf.copy()
    want[:, :(nh + nkv) * dk] = plain.rotate_leading(xf[:, :(nh + nkv) * dk].reshape(T, nh + nkv, dk), pos, dims, 777.0).reshape(T, -1)
    assert np.abs(proj.cpu().numpy() - want).max() < 2e-5 and int(err.item()) == 0
    assert np.array_equal(proj.cpu().numpy()[:, (nh + nkv) * dk:], x.astype(np.float32)[:, (nh + nkv) * dk:])     # values pass


@pytest.mark.parametrize("shape", [(150, 40, 7, 3, 24), (5, 64, 4, 1, 32), (33, 48, 3, 3, 16), (300, 128, 16, 2, 64)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_routed_experts_alone(dtype, shape):
    from llaisys_b200.config import PartSpec
    from llaisys_b200.parts import BuildEnv, build_part
    T, H, E, top, ff = shape
    rng = np.random.default_rng(4)
    w = {"router": _bf16_exact(rng.normal(size=(E, H)) * 0.5), "correction": _bf16_exact(rng.uniform(-0.4, 0.4, size=E))}
    for e in range(E):
        w[f"e{e}.up"], w[f"e{e}.down"] = _bf16_exact(rng.normal(size=(ff, H)) * 0.3), _bf16_exact(rng.normal(size=(H, ff)) * 0.3)
    w["shared.up"], w["shared.down"] = _bf16_exact(rng.normal(size=(24, H)) * 0.3), _bf16_exact(rng.normal(size=(H, 24)) * 0.3)
    h = _bf16_exact(rng.normal(size=(T, H)))
    p = {"router": {"experts": E, "top": top, "scale": 1.7}, "shared": {"ff": 24}}
    want = plain.routed_experts(h, w, p)
    part = build_part("ffn", PartSpec("routed_experts", {"hidden_size": H, "experts": E, "top": top, "expert_ff": ff, "route_scale": 1.7,
                                                         "shared_ff": 24}), BuildEnv(dtype, torch.device(DEV)))
    part.load({n: torch.from_numpy(v).to(torch.float32 if n == "correction" else dtype).to(DEV) for n, v in w.items()})
    from llaisys_b200 import kernels
    assert kernels.moe_tc_ok(torch.empty(1, H, dtype=dtype, device=DEV), part.up, part.down) == (dtype == torch.bfloat16)
    stream = torch.from_numpy(rng.normal(size=(T, H))).float().to(DEV)
    before = stream.clone()
    assert part.forward_into(torch.from_numpy(h).to(dtype).to(DEV), None, stream)
    got = (stream - before).cpu().numpy()
    scale = np.sqrt((want ** 2).mean())
    assert np.abs(got - want).max() < (2e-5 if dtype == torch.float32 else 3e-2) * max(scale, 1.0) * 4


# ----------------------------------------------------------------------------- attention alone: one layer, no feed-forward
# (window, kept first keys): page borders (64), one over, one under, a window of one key, a window nothing fills,
# kept keys that fill more than a page
MASKS = [(64, 0), (65, 64), (63, 65), (1, 1), (500, 3), (70, 3), (128, 129)]


@pytest.mark.parametrize("shared", [False, True])
@pytest.mark.parametrize("mask", MASKS)
def test_attention_alone_at_window_and_page_edges(tmp_path, mask, shared):
    """float32, scores spread over about +-10: one key too many or too few moves the logits by orders of magnitude
    more than the tolerance.  shared: a second layer reads the first one's cache through the same window (the cache
    then keeps every key and the window is a mask; else it is a ring behind pinned pages)."""
    window, keep = mask
    layers = [vh.layer(4, 2, 16, 24, 8, window, keep)]
    if shared:
        layers.append(vh.layer(4, 2, 16, 24, 8, window, keep, kv_from=0))
    cfg = vh.config(101, 32, layers, scale=2.0, bigram=(17, 3, 5))
    folder = vh.make_folder(tmp_path, cfg, seed=window * 7 + keep, attn_gain=12.0)
    oracle = vh.Oracle(folder)
    requests = vh.random_requests(cfg, [1, 200, 66, 131], seed=5)
    engine = build_engine(folder, torch.float32, max_tokens=64 * 4 + 64, max_seqs=2)
    like = vh.like_config(cfg)
    compare(run_whole(engine, requests), oracle, requests, torch.float32, like, f"attention {mask} whole")
    compare(run_tail_by_one(engine, requests, tail=140), oracle, requests, torch.float32, like, f"attention {mask} decoded")
    compare(run_chunked(engine, requests, [63, 2, 65, 1, 64]), oracle, requests, torch.float32, like, f"attention {mask} portions")
    assert not engine.cache.live_slots


@pytest.mark.parametrize("dim", [32, 64, 128])
@pytest.mark.parametrize("mask", MASKS)
def test_tensor_core_attention_against_the_cuda_core_one(tmp_path, mask, dim, monkeypatch):
    """bfloat16, keys and values of one width: the tensor-core kernels serve the windowed sink attention (head size 64
    over a cache that keeps every key: the tcgen05 kernel in prompts; else the mma.sync kernels).  They get the same
    bfloat16 queries, keys and values as the CUDA-core kernel, so with sharp scores (a lost key would show) the two
    may differ only by the rounding of the probabilities."""
    from llaisys_b200.kernels import ops
    window, keep = mask
    cfg = vh.config(101, 32, [vh.layer(4, 2, dim, dim, 16, window, keep), vh.layer(4, 2, dim, dim, 16, max(1, window - 1), keep + 1, kv_from=0),
                              vh.layer(3, 1, 16, 16, 16, window, keep)], scale=2.0, bigram=(17, 3, 5))
    folder = vh.make_folder(tmp_path, cfg, seed=window * 7 + keep, attn_gain=12.0)
    requests = vh.random_requests(cfg, [1, 200, 66, 131], seed=5)
    got = {}
    for mma in (True, False):
        monkeypatch.setattr(ops, "MMA_ATTENTION", mma)
        monkeypatch.setattr(ops, "TC_ATTENTION", mma)
        engine = build_engine(folder, torch.bfloat16, max_tokens=64 * 7, max_seqs=2)
        got[mma] = [run_whole(engine, requests), run_tail_by_one(engine, requests, tail=140), run_chunked(engine, requests, [63, 2, 65, 1, 64]),
                    run_batches(engine, requests, [[1, 3], [0, 2]], [1, 100, 30, 70])]
        assert not engine.cache.live_slots
    for a, b in zip(got[True], got[False]):
        for key in b:
            ref = b[key].astype(np.float64)
            rms = np.sqrt((ref ** 2).mean())
            d = a[key] - ref
            assert np.sqrt((d ** 2).mean()) <= 0.015 * rms + 2e-4 and np.abs(d).max() <= 0.1 * rms + 1e-3, (mask, key)


def test_odd_head_sizes(tmp_path):
    """Heads of 7 with 4 rotated dimensions, values of 5: nothing in the design asks for even or aligned sizes."""
    cfg = vh.config(53, 20, [vh.layer(3, 1, 7, 5, 4, 20, 2, moe=vh.moe(3, 2, 9, 7)), vh.layer(3, 1, 7, 5, 4, 11, 0, kv_from=0)],
                    scale=1.3, bigram=(11, 3, 5))
    for dtype in DTYPES:
        c = cfg if dtype == torch.float32 else vh.variant(cfg, lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 3))
        folder = vh.make_folder(tmp_path / str(dtype), c, seed=4, attn_gain=vh.GAIN[dtype])
        oracle, requests = vh.Oracle(folder), vh.random_requests(c, [1, 70, 33], seed=2)
        engine = build_engine(folder, dtype, max_tokens=64 * 3)
        compare(run_whole(engine, requests), oracle, requests, dtype, vh.like_config(c), "odd sizes whole")
        compare(run_tail_by_one(engine, requests, tail=40), oracle, requests, dtype, vh.like_config(c), "odd sizes decoded")


def test_one_far_key_that_decides(tmp_path):
    """A key hundreds of positions back that is made to dominate the softmax of every later query: it must be seen
    exactly while the mask shows it (inside the window, or among the kept first keys) in prompts and in decoding."""
    from llaisys_b200.weights import SafetensorsFile, write_safetensors
    for window, keep, special in ((1000, 0, 37), (40, 6, 5), (40, 6, 6)):
        cfg = vh.config(64, 32, [vh.layer(2, 1, 16, 16, 0, window, keep)], scale=1.0)
        folder = vh.make_folder(tmp_path / f"{window}_{special}", cfg, seed=9, attn_gain=1.0)
        f = SafetensorsFile(folder / "model.safetensors")
        t = {n: f.get(n).clone() for n in f.entries}
        # token 63 appears once, at position `special`; its embedding is large, so its key is, and every query scores it high
        t["embed"][63] = t["embed"][:63].float().mean(0).to(t["embed"].dtype) + 0.5
        t["l0.mix.k"] = t["l0.mix.q"].view(2, 16, 32)[0].clone()               # keys aligned with the queries of head 0
        write_safetensors(folder / "model.safetensors", t)
        oracle = vh.Oracle(folder)
        rng = np.random.default_rng(1)
        toks = rng.integers(0, 63, size=400).tolist()
        toks[special] = 63
        engine = build_engine(folder, torch.float32, max_tokens=512)
        like = vh.like_config(cfg)
        compare(run_whole(engine, [toks]), oracle, [toks], torch.float32, like, f"far key {special} whole")
        compare(run_tail_by_one(engine, [toks], tail=300), oracle, [toks], torch.float32, like, f"far key {special} decoded")


# ----------------------------------------------------------------------------- whole models under every schedule
LENGTHS = {"P": [1, 2, 64, 71, 150, 300], "Q": [3, 65, 129, 40], "R": [1, 66, 67, 200, 131]}


def _for_dtype(name, dtype):
    """Under bfloat16 every expert is chosen: which experts a token uses must not hang on 16-bit rounding of the
    stream (sparse routing in 16 bits is covered by test_routed_experts_alone, where both sides get the same input)."""
    cfg = vh.CONFIGS[name]
    if dtype == torch.bfloat16 and name not in vh.DENSE_ROUTING:
        def all_experts(c):
            for l in c["layers"]:
                if l["mlp"]:
                    l["mlp"]["router"]["top"] = l["mlp"]["router"]["experts"]
        cfg = vh.variant(cfg, all_experts)
    return cfg


class Model:
    def __init__(self, name, tmp):
        self.name, self._tmp, self._made = name, tmp, {}

    def at(self, dtype):
        if dtype not in self._made:
            cfg = _for_dtype(self.name, dtype)
            folder = vh.make_folder(self._tmp / str(dtype), cfg, seed=ord(self.name), attn_gain=vh.GAIN[dtype])
            self._made[dtype] = (cfg, folder, vh.Oracle(folder), vh.random_requests(cfg, LENGTHS[self.name], seed=ord(self.name)))
        return self._made[dtype]


@pytest.fixture(scope="module", params=["P", "Q", "R"])
def model(request, tmp_path_factory):
    return Model(request.param, tmp_path_factory.mktemp(f"vz{request.param}"))


def _rooms(requests):
    return sum(-(-len(r) // 64) * 64 for r in requests)


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_prompts_and_token_by_token(model, dtype):
    cfg, folder, oracle, requests = model.at(dtype)
    engine = build_engine(folder, dtype, max_tokens=max(_rooms([r]) for r in requests))
    like = vh.like_config(cfg)
    compare(run_whole(engine, requests), oracle, requests, dtype, like, f"{model.name} whole")
    compare(run_tail_by_one(engine, requests, tail=10_000), oracle, requests, dtype, like, f"{model.name} token by token")
    compare(run_tail_by_one(engine, requests, tail=32), oracle, requests, dtype, like, f"{model.name} tail")
    assert not engine.cache.live_slots


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batches_with_pages_and_slots_used_again(model, dtype):
    cfg, folder, oracle, requests = model.at(dtype)
    n = len(requests)
    batches = [list(range(0, n, 2)), list(range(1, n, 2))]
    prompt_lens = [max(1, len(r) - (3 + 5 * i)) for i, r in enumerate(requests)]
    room = max(_rooms([requests[r] for r in b]) for b in batches)
    engine = build_engine(folder, dtype, max_tokens=room, max_seqs=len(batches[0]))
    like = vh.like_config(cfg)
    compare(run_batches(engine, requests, batches, prompt_lens), oracle, requests, dtype, like, f"{model.name} batches")
    assert not engine.cache.live_slots
    assert [p.available for p in engine.cache.book.pools] == engine.cache.group_pages
    compare(run_batches(engine, requests, batches[::-1], prompt_lens), oracle, requests, dtype, like, f"{model.name} batches again")


@pytest.mark.parametrize("dtype", DTYPES)
def test_portions_and_mixed_steps(model, dtype):
    cfg, folder, oracle, _ = model.at(dtype)
    like = vh.like_config(cfg)
    requests = vh.random_requests(cfg, [200, 300, 129, 9], seed=41)
    engine = build_engine(folder, dtype, max_tokens=320)
    for cuts in ([70, 60, 1000], [63, 1, 64, 65, 2, 1000], [2, 200, 1000], [64], [2]):
        reqs = requests if cuts != [2] else requests[2:]
        compare(run_chunked(engine, reqs, cuts), oracle, reqs, dtype, like, f"{model.name} portions {cuts}")
    requests = vh.random_requests(cfg, [120, 100, 210, 33], seed=43)
    plans = [[50, 1, 1, 1, 40, 1, 0, 1], [0, 0, 90], [70, 60, 0, 40, 1, 1, 30], [1, 1, 1]]
    engine = build_engine(folder, dtype, max_tokens=_rooms(requests), max_seqs=4)
    for turn in range(2):
        compare(run_mixed(engine, requests, plans), oracle, requests, dtype, like, f"{model.name} mixed steps, turn {turn}")
        assert not engine.cache.live_slots
        requests, plans = requests[::-1], plans[::-1]


def test_long_decoding_through_captured_steps(tmp_path):
    """Hundreds of single-token steps from a short prompt: the ring wraps several times, the pair table's state moves
    with every step, and the steps are replayed from a captured graph."""
    for dtype in DTYPES:
        cfg = _for_dtype("P", dtype)
        folder = vh.make_folder(tmp_path / str(dtype), cfg, seed=21, attn_gain=vh.GAIN[dtype])
        oracle = vh.Oracle(folder)
        requests = vh.random_requests(cfg, [330, 290], seed=6)
        engine = build_engine(folder, dtype, max_tokens=_rooms(requests), max_seqs=2)
        assert engine.use_graphs
        compare(run_batches(engine, requests, [[0, 1]], [4, 1]), oracle, requests, dtype, vh.like_config(cfg), "long decoding")
        assert engine.graph_replays > 250


# ----------------------------------------------------------------------------- entry points
def _greedy(oracle, prompt, n):
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(np.argmax(oracle.logits(seq)[-1])))
    return seq[len(prompt):]


def test_greedy_generation_through_the_entry_point_and_scheduler(tmp_path):
    from llaisys_b200.models import CausalLM, DeviceType
    cfg = vh.CONFIGS["P"]
    folder = vh.make_folder(tmp_path, cfg, seed=31, attn_gain=8.0)
    oracle = vh.Oracle(folder)
    model = CausalLM(folder, DeviceType.NVIDIA, dtype="float32", max_tokens=64 * 4)
    prompts = vh.random_requests(cfg, [5, 9, 2, 70, 1, 17], seed=3)
    # four rooms of 64 tokens for six requests: two batches at least, slots and pages are used again
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
    folder = vh.make_folder(tmp_path / "m", vh.CONFIGS["P"], seed=17, attn_gain=8.0)
    (tmp_path / "batch.txt").write_text("5,17,3,200,7,7,7,7,7\n[9, 8]\n1\n")
    out = subprocess.run([sys.executable, "-m", "llaisys_b200.cli", "--model", str(folder), "--batch-file", str(tmp_path / "batch.txt"),
                          "--max_steps", "6", "--test", "--dtype", "float32"], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.count("Tokens:") == 3 and "Test passed" in out.stdout
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(vh.CONFIGS["R"]))
    out = subprocess.run([sys.executable, "-m", "llaisys_b200.cli", "--random-weights", str(cfg), "--seed", "3", "--tokens", "1,2,3",
                          "--max_steps", "4", "--test", "--dtype", "bfloat16"], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "Test passed" in out.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_of_a_trace(tmp_path, dtype):
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    cfg = _for_dtype("P", td)
    folder = vh.make_folder(tmp_path / "m", cfg, seed=13, attn_gain=vh.GAIN[td])
    requests = vh.random_requests(cfg, [1, 7, 90, 20], seed=8)
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
    oracle = vh.Oracle(folder)
    for step, keys in rows:
        data = np.frombuffer((out_dir / f"{step}.f32").read_bytes(), dtype="<f4").reshape(len(keys), cfg["vocab"])
        for i, (r, p) in enumerate(keys):
            ref = oracle.logits(requests[r])
            assert np.abs(data[i] - ref[p]).max() <= tolerance(td, vh.like_config(cfg), ref), (step, r, p)
