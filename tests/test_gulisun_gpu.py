"""The Gulisun design in the engine against its plain statement (tests/plain_gulisun.py): each mechanism alone,
then whole models in every way of cutting the work (whole prompts, a decoded tail, portions down to two tokens,
mixed batches with pages and state slots used again), keys far back that carry the score, long decoding through
captured graphs, and greedy generation through the entry point and its scheduler. Cache pages are poisoned with
NaN so that a read outside a request's own rows shows."""
import numpy as np
import pytest
import torch

import gulisun_helpers as gh
import helpers
import plain_gulisun as plain

pytestmark = pytest.mark.gpu

TOL = {"float32": 5e-5, "bfloat16": 4e-2}     # relative to the largest |logit| of the plain statement
LENGTHS = [1, 7, 33, 90, 61, 47, 2, 70, 18, 120, 64, 65, 3]


def row_errors(got, want):
    scale = max(float(np.abs(w).max()) for w in want.values())
    return np.array([float(np.abs(got[r][p].astype(np.float64) - want[r][p]).max()) / scale
                     for r in sorted(got) for p in sorted(got[r])])


def agrees(got, want, dtype):
    """float32: every row within the tolerance. bfloat16: a router's choice between two experts of nearly equal
    score may fall the other way once activations are rounded to 8 bits, which moves that token's logits (and, a
    little, those behind it) by more than rounding: with four routed layers and a single expert a token in some, a
    token in twenty meets such a choice. So most rows must be within the tolerance, the typical row well within
    it, and every row finite; what the cache and the batching do is judged in float32, where every row counts."""
    err = row_errors(got, want)
    assert np.isfinite(err).all()
    if dtype == "float32":
        return helpers.first_bad(got, want, TOL[dtype]) is None
    return (err > TOL[dtype]).mean() <= 0.15 and np.median(err) <= TOL[dtype] / 3


def session_for(folder, dtype, steps, page, **kw):
    from tinyinfer_b200.engine.replay import TraceSession
    return TraceSession(folder, dtype, helpers.peak_tokens(steps, max(64, page)), page_size=page, poison_cache=True, **kw)


def run(folder, dtype, steps, page, **kw):
    session = session_for(folder, dtype, steps, page, **kw)
    got = helpers.collect(session, steps)
    session.runner.check_status()
    session.runner.manager.check_consistency()
    return got, session


# ------------------------------------------------------------------ each mechanism alone
@pytest.mark.parametrize("kind,mlp", [("sink", None), ("plain", None), ("reader", None), ("recurrent", None),
                                      ("sink", gh.MOE_A), ("recurrent", gh.MOE_B)])
def test_one_mechanism_alone(tmp_path, kind, mlp):
    cfg = gh.single(kind, mlp)
    folder = gh.write_folder(tmp_path / "m", cfg, seed=11)
    requests = gh.random_requests(cfg, [75, 1, 2, 19], seed=4)
    want = gh.plain_logits(folder, requests)
    got, _ = run(folder, "float32", helpers.trace_whole(requests), page=8)
    assert helpers.first_bad(got, want, TOL["float32"]) is None
    got, _ = run(folder, "float32", helpers.trace_chunked(requests, seed=3), page=8)
    assert helpers.first_bad(got, want, TOL["float32"]) is None


def test_the_sink_and_the_shared_rows_carry_weight(tmp_path):
    """What the tests above can see: without the sink term, or with a reader's own rows in place of the rows of
    the layer it names, the plain logits move by far more than the tolerance."""
    cfg = gh.single("reader")
    folder = gh.write_folder(tmp_path / "m", cfg, seed=11)
    requests = gh.random_requests(cfg, [60], seed=4)
    want = gh.plain_logits(folder, requests)["r0"]

    def no_sink(c, w):
        for k in w:
            if k.endswith("mix.sink"):
                w[k] = torch.full_like(w[k], -1e30)
    assert np.abs(gh.plain_logits(folder, requests, no_sink)["r0"] - want).max() > 100 * TOL["float32"] * np.abs(want).max()


@pytest.mark.parametrize("experts,top,shared", [(5, 1, None), (6, 3, 40), (33, 4, 8), (4, 4, None)])
def test_router_against_plain(experts, top, shared):
    from tinyinfer_b200 import ops
    gen = torch.Generator().manual_seed(experts * 10 + top)
    x = torch.randn(37, 72, generator=gen)
    w = torch.randn(experts, 72, generator=gen) * 0.3
    routing = ops.route_experts(x.cuda(), w.cuda(), top, 1e-20)
    scores = torch.softmax(x.double() @ w.double().T, dim=-1)
    best, chosen = torch.topk(scores, top, dim=-1)
    assert torch.equal(routing.chosen.cpu().long(), chosen)
    assert torch.allclose(routing.weight.cpu().double(), best / (best.sum(-1, keepdim=True) + 1e-20), atol=1e-6)
    # every (token, choice) has a row of its own among its expert's rows
    slots = routing.slot_of.cpu().view(-1)
    assert sorted(slots.tolist()) == list(range(37 * top))
    assert torch.equal(routing.token_of.cpu()[slots.long()], torch.arange(37).repeat_interleave(top).int())


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1.5e-2)])
@pytest.mark.parametrize("m,batch,n,k,gap", [(1, 3, 40, 24, 8), (70, 4, 136, 64, 0), (33, 2, 8, 200, 16), (300, 5, 130, 72, 8)])
def test_batched_product_against_torch(m, batch, n, k, gap, dtype, tol):
    """Pieces side by side in the rows of x and of out, with and without the tensor-core form's alignment."""
    from tinyinfer_b200 import ops
    gen = torch.Generator().manual_seed(m + n)
    x = torch.randn(m, 5 + batch * (k + gap), generator=gen).to(dtype)
    w = (torch.randn(batch, n, k, generator=gen) / k ** 0.5).to(dtype)
    bias = torch.randn(batch, n, generator=gen)
    for offset in (0, 5 if gap != 8 else 8):
        out = torch.full((m, 3 + batch * (n + 2)), 7.0)
        got = ops.batched_linear(x.cuda(), w.cuda(), x_offset=offset, x_batch_stride=k + gap, k=k, out=out.cuda(),
                                 out_offset=3, out_batch_stride=n + 2, bias=bias.cuda(), sigmoid=True).cpu()
        for b in range(batch):
            piece = x[:, offset + b * (k + gap):offset + b * (k + gap) + k].double()
            want = torch.sigmoid(piece @ w[b].double().T + bias[b].double())
            assert (got[:, 3 + b * (n + 2):3 + b * (n + 2) + n].double() - want).abs().max() <= tol
        assert (got[:, :3] == 7.0).all() and (got[:, 3 + n:3 + n + 2] == 7.0).all()      # nothing written between the pieces


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("tokens,experts,top,ff,width", [(1, 4, 2, 24, 40), (150, 6, 3, 136, 64), (77, 9, 1, 40, 72),
                                                         (700, 5, 2, 192, 128), (333, 3, 3, 320, 64)])
def test_grouped_expert_products_against_torch(tokens, experts, top, ff, width, dtype, tol):
    """The last two shapes bring an expert enough rows for the tcgen05 form (bfloat16) and row tiles of 128."""
    from tinyinfer_b200 import ops
    gen = torch.Generator().manual_seed(tokens)
    x = torch.randn(tokens, width, generator=gen)
    router = torch.randn(experts, width, generator=gen)
    up = (torch.randn(experts, ff, width, generator=gen) / width ** 0.5).to(dtype)
    down = (torch.randn(experts, width, ff, generator=gen) / ff ** 0.5).to(dtype)
    xc = x.to(dtype)
    routing = ops.route_experts(x.cuda(), router.cuda(), top, 1e-20,
                                tile_rows=ops.expert_tile_rows(xc.cuda(), experts, top, ff))
    if tokens * top >= 96 * experts:
        assert routing.tile_rows == (128 if dtype == torch.bfloat16 else 32)
    hidden = ops.expert_linear(xc.cuda(), up.cuda(), routing, up=True)
    out = ops.expert_linear(hidden, down.cuda(), routing, up=False).cpu()
    chosen, slot_of = routing.chosen.cpu().long(), routing.slot_of.cpu().long()
    for t in range(tokens):
        for c in range(top):
            e = int(chosen[t, c])
            h = torch.relu(xc[t].double() @ up[e].double().T) ** 2
            if dtype == torch.bfloat16:
                h = h.to(dtype).double()
            want = h @ down[e].double().T
            assert (out[slot_of[t, c]].double() - want).abs().max() <= tol * max(1.0, float(want.abs().max())), (t, c)


# ------------------------------------------------------------------ whole models, every cut
def traces_for(requests, max_live=4):
    return {"whole": helpers.trace_whole(requests), "tail": helpers.trace_decode_tail(requests, tail=32),
            "chunked": helpers.trace_chunked(requests, seed=1), "mixed": helpers.trace_mixed(requests, seed=2, max_live=max_live)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page", [("MIX", 8), ("WIDE", 16)])
def test_every_cut_matches_plain(tmp_path, name, page, dtype):
    cfg = getattr(gh, name)
    folder = gh.write_folder(tmp_path / name, cfg, seed=3, dtype=dtype)
    requests = gh.random_requests(cfg, LENGTHS, seed=5)
    want = gh.plain_logits(folder, requests)
    results = {}
    for tag, steps in traces_for(requests).items():
        got, session = run(folder, dtype, steps, page, max_live=4)
        assert {r: len(v) for r, v in got.items()} == {r: len(t) for r, t in requests.items()}, tag
        assert agrees(got, want, dtype), (tag, helpers.first_bad(got, want, TOL[dtype]), np.sort(row_errors(got, want))[-8:])
        if tag == "mixed":
            stats = session.runner.manager.stats()
            assert all(g["pages_taken"] > g["pages"] for g in stats["groups"]), "pages were not used again"
        results[tag] = got
    scale = max(float(np.abs(w).max()) for w in want.values())
    for tag in ("tail", "chunked", "mixed"):        # the cuts against each other: rounding only
        assert agrees(results[tag], {r: np.stack([results["whole"][r][p] for p in range(len(t))]) for r, t in requests.items()},
                      dtype), tag


def test_two_state_slots_serve_many_requests(tmp_path):
    """Slots (recurrent state) and pages are handed from finished requests to new ones, two live at a time."""
    cfg = gh.MIX
    folder = gh.write_folder(tmp_path / "m", cfg, seed=8)
    requests = gh.random_requests(cfg, [30, 9, 41, 2, 17, 55, 5, 26], seed=9)
    want = gh.plain_logits(folder, requests)
    steps = helpers.trace_mixed(requests, seed=4, max_live=2, decode_tail=6)
    got, session = run(folder, "float32", steps, page=4, max_live=2)
    assert helpers.first_bad(got, want, TOL["float32"]) is None
    assert session.runner.manager.stats()["free_state_slots"] == 2


def test_batch_of_unequal_requests_equals_each_alone(tmp_path):
    cfg = gh.WIDE
    folder = gh.write_folder(tmp_path / "m", cfg, seed=5)
    requests = gh.random_requests(cfg, [50, 3, 128, 17], seed=2)
    together = [{"step": 0, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in requests.items()],
                 "end": list(requests)}]
    got, _ = run(folder, "float32", together, page=16)
    alone, _ = run(folder, "float32", helpers.trace_whole(requests), page=16)
    want = gh.plain_logits(folder, requests)
    assert helpers.first_bad(got, want, TOL["float32"]) is None
    scale = max(float(np.abs(w).max()) for w in want.values())
    assert max(float(np.abs(got[r][p] - alone[r][p]).max()) for r in requests for p in got[r]) / scale <= 1e-5


# ------------------------------------------------------------------ keys far back, page borders
def test_far_keys_carry_the_score(tmp_path):
    """A large score scale makes every softmax nearly one-hot on a key that lies anywhere in the context, so a
    row that is missing, misplaced or read from the wrong page changes the logits. Positions around the borders
    of pages (16) and of the attention kernel's key tiles (32) and splits are decoded one by one."""
    sharp = gh.latent(3, 16, 8, 16, 24, 40, scale=1.5)
    cfg = gh.config([dict(type="latent_attention", mixer=sharp, mlp=None),
                     dict(type="latent_attention", mixer=dict(sharp, kv_from=0), mlp=None),
                     dict(type="latent_attention_2", mixer=gh.latent(2, 16, 8, 16, 24, 40, scale=1.5), mlp=None)], width=64)
    folder = gh.write_folder(tmp_path / "m", cfg, seed=21)
    requests = gh.random_requests(cfg, [700], seed=13)
    tokens = requests["r0"]
    want = gh.plain_logits(folder, requests)
    # the premise: cutting the first 64 tokens off moves the logits of the last tokens by far more than the tolerance
    c, w = gh.read_folder(folder)
    cut = plain.forward(c, w, tokens[64:]).numpy()
    assert np.abs(cut[-40:] - want["r0"][-40:]).max() > 100 * TOL["float32"] * np.abs(want["r0"]).max()
    for steps in (helpers.trace_whole(requests), helpers.trace_decode_tail(requests, tail=140),
                  helpers.trace_chunked(requests, seed=7)):
        got, _ = run(folder, "float32", steps, page=16)
        assert helpers.first_bad(got, want, TOL["float32"]) is None
    # the same through the bfloat16 kernels (rows of 48 features: the tensor-core forms for portions and for decoding)
    folder16 = gh.write_folder(tmp_path / "m16", cfg, seed=21, dtype="bfloat16")
    want16 = gh.plain_logits(folder16, requests)
    for steps in (helpers.trace_whole(requests), helpers.trace_decode_tail(requests, tail=140),
                  helpers.trace_chunked(requests, seed=7)):
        got, _ = run(folder16, "bfloat16", steps, page=16)
        err = row_errors(got, want16)
        assert np.isfinite(err).all() and np.median(err) <= 2e-2 and (err > 0.15).mean() <= 0.02, np.sort(err)[-5:]


# ------------------------------------------------------------------ long decoding through graphs
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_replays_graphs(tmp_path, dtype):
    cfg = gh.MIX
    folder = gh.write_folder(tmp_path / "m", cfg, seed=6, dtype=dtype)
    requests = gh.random_requests(cfg, [160, 150], seed=1)
    want = gh.plain_logits(folder, requests)
    steps = [{"step": 0, "entries": [{"id": r, "tokens": t[:4], "want": [0, 1, 2, 3]} for r, t in requests.items()], "end": []}]
    for p in range(4, 150):
        steps.append({"step": p, "entries": [{"id": r, "tokens": [t[p]], "want": [0]} for r, t in requests.items()],
                      "end": list(requests) if p == 149 else []})
    got, session = run(folder, dtype, steps, page=8)
    assert session.runner.graph_replays > 100
    assert agrees(got, {r: w[:150] for r, w in want.items()}, dtype)


# ------------------------------------------------------------------ generation through the entry point
@pytest.mark.parametrize("dtype,tol", [("float32", 1e-4), ("bfloat16", 6e-2)])
def test_greedy_generation_through_the_scheduler(tmp_path, dtype, tol):
    from tinyinfer_b200 import LLM
    from tinyinfer_b200.sampling import SamplingParams
    cfg = gh.MIX
    folder = gh.write_folder(tmp_path / "m", cfg, seed=3, dtype=dtype)
    llm = LLM(folder, dtype=dtype, max_num_batched_tokens=24, max_num_seqs=3, kvcache_block_size=8,
              num_kvcache_blocks=40, prefill_chunk=9, max_model_len=128)
    assert llm.config.enable_prefix_caching is False          # a state cannot be rebuilt from pages
    prompts = list(gh.random_requests(cfg, [1, 7, 16, 33, 50], seed=6).values())
    outs = llm.generate(prompts, SamplingParams(greedy=True, max_tokens=10))
    c, w = gh.read_folder(folder)
    off = 0
    for p, o in zip(prompts, outs):
        assert o["all_token_ids"] == p + o["token_ids"] and len(o["token_ids"]) == 10
        logits = plain.forward(c, w, p + o["token_ids"]).numpy()
        for i, tok in enumerate(o["token_ids"]):          # teacher forcing: the token has (nearly) the largest plain logit
            row = logits[len(p) - 1 + i]
            off += not row.max() - row[tok] <= tol * np.abs(logits).max()
    assert off <= (0 if dtype == "float32" else 2), off    # bfloat16: see agrees()
    assert not llm.runner.manager.live_requests
    llm.runner.manager.check_consistency()
    llm.close()


def test_command_line_generates_with_a_folder_and_with_a_preset(tmp_path):
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    folder = gh.write_folder(tmp_path / "m", gh.MIX, seed=3)
    common = ["--dtype", "fp32", "--prompt-ids", "5,17,3,200", "--prompt-len", "9", "--greedy", "--max-tokens", "6",
              "--max-num-seqs", "2", "--max-num-batched-tokens", "16", "--block-size", "4", "--num-kvcache-blocks", "32",
              "--max-model-len", "64"]
    res = subprocess.run([sys.executable, str(root / "examples" / "generate.py"), "--model", str(folder)] + common,
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    rows = [json.loads(l) for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(rows) == 2 and all(len(r["token_ids"]) == 6 for r in rows)
    c, w = gh.read_folder(folder)
    logits = plain.forward(c, w, [5, 17, 3, 200] + rows[0]["token_ids"]).numpy()
    for i, tok in enumerate(rows[0]["token_ids"]):
        assert logits[3 + i].max() - logits[3 + i][tok] <= 1e-4 * np.abs(logits).max()
    res = subprocess.run([sys.executable, str(root / "examples" / "generate.py"), "--random-config", "gulisun-tiny"] + common,
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]


def random_config(seed):
    """A model of random sizes and layer order: odd head counts, ranks that are no multiple of 8 or 32, one to four
    experts a token, convolutions of two to six taps, a width that the tensor-core products refuse now and then."""
    import random
    rng = random.Random(seed)
    width = rng.choice([40, 72, 100, 136])
    layers, writers = [], []
    for i in range(rng.randint(3, 6)):
        kind = rng.choice(["latent_attention", "latent_attention_2", "rglru", "reader"])
        if kind == "reader" and not writers:
            kind = "latent_attention"
        if kind == "rglru":
            blocks = rng.choice([1, 2, 3, 4])
            mixer = dict(width=blocks * rng.choice([8, 12, 20, 32]), blocks=blocks, conv=rng.randint(2, 6))
            kind_name = "rglru"
        elif kind == "reader":
            j = rng.choice(writers)
            src = layers[j]["mixer"]
            mixer = gh.latent(rng.randint(1, 9), rng.choice([8, 12, 24]), src["rot_dim"], rng.choice([8, 20, 32]),
                              rng.choice([16, 28, 40]), src["kv_rank"], scale=rng.uniform(0.1, 0.4), base=src["rot"]["base"], kv_from=j)
            kind_name = "latent_attention"
        else:
            mixer = gh.latent(rng.randint(1, 9), rng.choice([8, 12, 24, 40]), rng.choice([4, 8, 16, 24]), rng.choice([8, 20, 32, 48]),
                              rng.choice([16, 28, 40, 64]), rng.choice([24, 40, 56, 100, 136]), scale=rng.uniform(0.1, 0.4),
                              base=rng.choice([100.0, 10000.0, 1e6]))
            kind_name = kind
            writers.append(i)
        experts = rng.randint(2, 20)
        mlp = None if rng.random() < 0.2 else gh.moe(experts, rng.randint(1, min(4, experts)), rng.choice([8, 24, 40]),
                                                     shared=rng.choice([None, 16, 56]))
        layers.append(dict(type=kind_name, mixer=mixer, mlp=mlp))
    return gh.config(layers, vocab=rng.choice([97, 256, 300]), width=width, scale=rng.choice([1.0, 4.0, 11.0]),
                     eps=rng.choice([1e-5, 1e-6]))


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_models_of_random_sizes_and_orders(tmp_path, seed):
    cfg = random_config(seed)
    page = [4, 8, 16, 32, 64, 16][seed - 1]
    requests = gh.random_requests(cfg, [70, 1, 37, 150, 2, 64], seed=seed)
    folder = gh.write_folder(tmp_path / "m", cfg, seed=seed)
    want = gh.plain_logits(folder, requests)
    for steps in (helpers.trace_whole(requests), helpers.trace_mixed(requests, seed=seed, max_live=3, decode_tail=20)):
        got, _ = run(folder, "float32", steps, page, max_live=3)
        assert helpers.first_bad(got, want, TOL["float32"]) is None, cfg
    folder16 = gh.write_folder(tmp_path / "m16", cfg, seed=seed, dtype="bfloat16")
    got, _ = run(folder16, "bfloat16", helpers.trace_mixed(requests, seed=seed, max_live=3, decode_tail=20), page, max_live=3)
    err = row_errors(got, gh.plain_logits(folder16, requests))
    assert np.isfinite(err).all() and np.median(err) <= TOL["bfloat16"] / 2, (np.median(err), cfg)
