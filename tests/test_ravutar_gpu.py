"""The Ravutar design in the engine against its plain statement (tests/plain_ravutar.py): the new kernels alone,
each mechanism alone in a model, then whole models in every way of cutting the work (whole prompts, a decoded
tail, portions down to two tokens, mixed batches with pages and state slots used again), tokens far back that
carry the result, long decoding through captured graphs, and greedy generation through the entry point and its
scheduler. Cache pages are poisoned with NaN so that a read outside a request's own rows shows."""
import copy

import numpy as np
import pytest
import torch

import helpers
import plain_ravutar as plain
import ravutar_helpers as rh

pytestmark = pytest.mark.gpu

TOL = {"float32": 5e-5, "bfloat16": 4e-2}     # relative to the largest |logit| of the plain statement
LENGTHS = [1, 7, 33, 90, 61, 47, 2, 70, 18, 120, 64, 65, 3]


def row_errors(got, want):
    scale = max(float(np.abs(w).max()) for w in want.values())
    return np.array([float(np.abs(got[r][p].astype(np.float64) - want[r][p]).max()) / scale
                     for r in sorted(got) for p in sorted(got[r])])


def agrees(got, want, dtype):
    """float32: every row within the tolerance; this is what judges the cache, the state and the batching.
    bfloat16: activations rounded to 8 bits through six or more layer runs leave a row in fifty a few times
    further off than the typical row, so nearly all rows must be within the tolerance, the typical row well within
    it, and none far outside."""
    err = row_errors(got, want)
    if not np.isfinite(err).all():
        return False
    if dtype == "float32":
        return bool(err.max() <= TOL[dtype])
    return bool((err > TOL[dtype]).mean() <= 0.03 and np.median(err) <= TOL[dtype] / 3 and err.max() <= 3 * TOL[dtype])


def run(folder, dtype, steps, page, **kw):
    from tinyinfer_b200.engine.replay import TraceSession
    session = TraceSession(folder, dtype, helpers.peak_tokens(steps, max(64, page)), page_size=page, poison_cache=True, **kw)
    got = helpers.collect(session, steps)
    session.runner.check_status()
    session.runner.manager.check_consistency()
    return got, session


# ------------------------------------------------------------------ the kernels alone
@pytest.mark.parametrize("streams,width,dtype", [(1, 40, torch.float32), (3, 72, torch.bfloat16), (8, 130, torch.float32)])
def test_streams_step_against_plain(streams, width, dtype):
    from tinyinfer_b200 import ops
    gen = torch.Generator().manual_seed(streams)
    T = 9
    x = torch.randn(streams, T, width, generator=gen)
    y = torch.randn(T, width, generator=gen).to(dtype)
    mix, out, c_in = torch.randn(streams, streams, generator=gen), torch.randn(streams, generator=gen), torch.randn(streams, generator=gen)
    w = 1 + 0.2 * torch.randn(width, generator=gen)
    xd = x.cuda()
    h = ops.streams_step(xd, ops.StreamUpdate(y.cuda(), mix.cuda(), out.cuda()), c_in.cuda(), w.cuda(), 1e-5, dtype)
    fresh = torch.einsum("st,snw->tnw", mix.double(), x.double()) + out.double()[:, None, None] * y.double()[None]
    assert (xd.cpu().double() - fresh).abs().max() < 1e-5
    u = torch.einsum("s,snw->nw", c_in.double(), fresh)
    want = plain.rms_norm(u, w.double(), 1e-5)
    assert (h.cpu().double() - want).abs().max() <= (1e-5 if dtype == torch.float32 else 3e-2) * want.abs().max()
    # only the wanted rows; nothing pending
    rows = torch.tensor([7, 2], dtype=torch.int32)
    before = xd.clone()
    h = ops.streams_step(xd, None, c_in.cuda(), w.cuda(), 1e-5, torch.float32, rows=rows.cuda())
    assert torch.equal(before, xd) and (h.cpu().double() - want[rows.long()]).abs().max() <= 1e-5 * want.abs().max()


def scan_plain(q, k, v, a, kscale, skip, S):
    """S [H, dk, dv]; q, k, a [T, H, dk]; v [T, H, dv]; returns o [T, H, dv] and the last S."""
    out = []
    for t in range(q.shape[0]):
        S = a[t][:, :, None] * S + (k[t] * kscale[t][:, None])[:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S, q[t]) + skip[:, None] * v[t])
    return torch.stack(out), S


@pytest.mark.parametrize("heads,groups,dk,dv,gate", [(3, 3, 24, 20, "sigmoid_power"), (6, 2, 20, 12, "step_size"),
                                                     (2, 1, 130, 9, "raw"), (1, 1, 8, 70, "sigmoid_power"),
                                                     (4, 4, 64, 64, "step_size"), (2, 2, 300, 5, "raw")])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_linear_scan_against_plain(heads, groups, dk, dv, gate, dtype):
    """Two requests of unequal length in two calls: the state goes through slots that lie inside a larger state.
    The first call is long enough to be cut into stretches that run side by side (the short request's are partly empty)."""
    from tinyinfer_b200 import ops
    gen = torch.Generator().manual_seed(heads * dk + dv)
    lens1, lens2 = [137, 5], [1, 22]
    per_channel = gate != "step_size"
    pad = 7                                              # other columns in front of q, k, v in their rows
    a_log, dt_bias, skip = torch.randn(heads, generator=gen) - 1, torch.randn(heads, generator=gen), torch.randn(heads, generator=gen)
    state = torch.zeros(3, 11 + heads * dk * dv)         # slots 2 and 0 are used; 11 floats of someone else's in front
    state_d = state.cuda()
    view = state_d[:, 11:].unflatten(1, (heads, dv, dk))
    S = [torch.zeros(heads, dk, dv, dtype=torch.float64) for _ in range(2)]
    for lens in (lens1, lens2):
        T = sum(lens)
        row = torch.randn(T, pad + 2 * groups * dk + heads * dv, generator=gen).to(dtype)
        g = torch.randn(T, 3 + heads * (dk if per_channel else 1), generator=gen)
        if gate == "raw":
            g = torch.sigmoid(g + 2)
        cu = torch.tensor([0, lens[0], T], dtype=torch.int32)
        slots = torch.tensor([2, 0], dtype=torch.int32)
        sg = ops.ScanGate(gate, g.cuda(), per_channel=per_channel, offset=3, tau=5.0, a_log=a_log.cuda(), dt_bias=dt_bias.cuda())
        got = ops.linear_scan(row.cuda(), row.cuda(), row.cuda(), sg, state=view, heads=heads, groups=groups, key_dim=dk,
                              value_dim=dv, q_offset=pad, k_offset=pad + groups * dk, v_offset=pad + 2 * groups * dk,
                              q_scale=0.5, skip=skip.cuda(), cu_seqlens=cu.cuda(), state_slots=slots.cuda(), num_seqs=2,
                              max_q_len=max(lens)).cpu()
        assert (ops.scan_stretches(max(lens), 2, heads, dk, dv) > 1) == (max(lens) > 100)
        r = row.double()
        per = heads // groups
        q = r[:, pad:pad + groups * dk].reshape(T, groups, dk).repeat_interleave(per, dim=1) * 0.5
        k = r[:, pad + groups * dk:pad + 2 * groups * dk].reshape(T, groups, dk).repeat_interleave(per, dim=1)
        v = r[:, pad + 2 * groups * dk:].reshape(T, heads, dv)
        gv = g[:, 3:].double()
        kscale = torch.ones(T, heads, dtype=torch.float64)
        if gate == "raw":
            a = gv.reshape(T, heads, dk)
        elif gate == "sigmoid_power":
            a = torch.exp(torch.nn.functional.logsigmoid(gv) / 5.0).reshape(T, heads, dk)
        else:
            kscale = torch.nn.functional.softplus(gv + dt_bias.double(), threshold=1e9)
            a = torch.exp(-torch.exp(a_log.double()) * kscale)[:, :, None].expand(T, heads, dk)
        at = 0
        for i, n in enumerate(lens):
            want, S[i] = scan_plain(q[at:at + n], k[at:at + n], v[at:at + n], a[at:at + n], kscale[at:at + n], skip.double(), S[i])
            assert (got[at:at + n].double().reshape(n, heads, dv) - want).abs().max() <= 2e-5 * max(1.0, want.abs().max()), (i, lens)
            at += n
    kept = state_d.cpu()
    assert (kept[:, :11] == 0).all() and (kept[1] == 0).all()
    for i, slot in enumerate((2, 0)):
        assert (kept[slot, 11:].reshape(heads, dv, dk).transpose(1, 2).double() - S[i]).abs().max() <= 2e-5 * max(1.0, S[i].abs().max())


@pytest.mark.parametrize("width,group,w_len,first", [(60, 20, 20, False), (72, 24, 72, True), (600, 600, 600, True), (64, 8, 8, False)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_group_norm_against_plain(width, group, w_len, first, dtype):
    from tinyinfer_b200 import ops
    gen = torch.Generator().manual_seed(width)
    y = torch.randn(5, width, generator=gen)
    gate = torch.randn(5, 9 + width, generator=gen).to(dtype)
    w = 1 + 0.3 * torch.randn(w_len, generator=gen)
    got = ops.gated_group_norm(y.cuda(), gate.cuda(), w.cuda(), group=group, eps=1e-5, gate_first=first, out_dtype=dtype,
                               gate_offset=9, out_scale=0.8).cpu().double()
    gz = plain.silu(gate[:, 9:].double())
    v = y.double() * gz if first else y.double()
    v = plain.unit_rms(v.reshape(5, width // group, group), 1e-5).reshape(5, width) * w.double().repeat(width // w_len)
    want = 0.8 * (v if first else v * gz)
    assert (got - want).abs().max() <= (1e-5 if dtype == torch.float32 else 2e-2) * max(1.0, want.abs().max())


def test_gelu_and_scale():
    from tinyinfer_b200 import ops
    x = torch.linspace(-6, 6, 1001)
    assert (ops.gelu(x.cuda()).cpu().double() - plain.gelu_erf(x.double())).abs().max() < 1e-6
    tanh_form = 0.5 * x.double() * (1 + torch.tanh(0.7978845608028654 * (x.double() + 0.044715 * x.double() ** 3)))
    assert (ops.gelu(x.cuda(), tanh=True).cpu().double() - tanh_form).abs().max() < 1e-6
    assert torch.equal(ops.scale_(x.clone().cuda(), 0.25).cpu(), x * 0.25)


SINK_SHAPES = [
    # hq, hkv, d, page, window, [(context, q_len)], two query tiles a CTA?
    (3, 3, 48, 5, None, [(17, 17), (31, 1)], False),                                    # the float32-arithmetic kernel
    (8, 2, 64, 16, None, [(130, 130), (129, 1), (200, 2)], False),                      # one query tile a CTA; decoding
    (8, 8, 128, 16, None, [(1500, 1), (1, 1), (256, 1), (257, 1), (1024, 1)], False),   # decoding, merged and not
    (12, 3, 128, 64, None, [(450, 61), (63, 63), (2, 2), (1100, 17)], False),
    (8, 2, 128, 64, None, [(1300, 897), (700, 513), (640, 384), (1, 1)], True),         # two query tiles a CTA
    (4, 2, 64, 32, 200, [(1500, 1000), (420, 385)], True),
    (2, 1, 128, 64, None, [(4000, 120)], False),                                        # the keys shared out over CTAs
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sink", [0.0, 2.5, -30.0])
@pytest.mark.parametrize("hq,hkv,d,page,window,work,pairs", SINK_SHAPES)
def test_paged_attention_with_a_sink(monkeypatch, dtype, sink, hq, hkv, d, page, window, work, pairs):
    """The softmax denominator's extra term and the output factor in every attention kernel of the plain decoder."""
    import test_kernels_gpu as tk
    import torch_ops as ref
    from tinyinfer_b200 import ops
    if dtype == torch.float32 and sink != 0.0:
        pytest.skip("one sink in float32")
    monkeypatch.setattr(ops, "PAIR_MIN_CTAS", 0 if pairs else 1 << 30)
    lens = [c for c, _ in work]
    bt, kv = tk.paged_setup(dtype, lens, hq, hkv, d, page, seed=1)
    tk.fill_cache(kv, bt, lens, hkv, d, page, dtype)
    pos = torch.tensor([p for c, n in work for p in range(c - n, c)], dtype=torch.int32, device="cuda")
    seq = torch.tensor([i for i, (c, n) in enumerate(work) for _ in range(n)], dtype=torch.int32, device="cuda")
    q = tk.rnd(pos.shape[0], hq, d, dtype=dtype, seed=7, std=2.0)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    args = dict(positions=pos, token_seq=seq, block_table=bt, scale=d ** -0.5, window=window, sink=sink, out_scale=0.7)
    out = ops.paged_attention(q, kv, status=status, **args)
    assert int(status.item()) == 0 and torch.isfinite(out.float()).all()
    want = ref.paged_attention(q, kv, **args)
    tk.close(out, want, dtype)
    if sink > -10 and max(lens) <= 1500 and window is None:          # few enough keys that the term carries weight
        without = ref.paged_attention(q, kv, **dict(args, sink=None))
        assert (without.float() - want.float()).abs().max() > 0.05


# ------------------------------------------------------------------ each mechanism alone
def single(kind, mlp=None, **kw):
    a, b = rh.left(4, 2, 12, 20, scale=0.35, conv=3, q_temp=(0.4, 8)), rh.right(3, 20, 12, tau=7.0)
    if kind == "attention":          # the linear branch runs beside it with weight zero
        return rh.config([rh.parallel(a, b, left_scale=1.1, right_scale=0.0, mlp=mlp)], **kw)
    if kind == "linear":
        return rh.config([rh.parallel(a, b, left_scale=0.0, right_scale=1.1, mlp=mlp)], **kw)
    if kind == "both":
        return rh.config([rh.parallel(a, b, mlp=mlp)], **kw)
    if kind == "state_space":
        return rh.config([rh.mamba(6, 12, 20, 3, conv=4, norm_groups=2, mlp=mlp)], **kw)
    raise ValueError(kind)


@pytest.mark.parametrize("kind,mlp,streams", [("attention", None, 2), ("linear", None, 2), ("both", None, None),
                                              ("state_space", None, 1), ("both", rh.dense(56), 4),
                                              ("state_space", rh.dense(24), None)])
def test_one_mechanism_alone(tmp_path, kind, mlp, streams):
    cfg = single(kind, mlp, streams=streams)
    folder = rh.write_folder(tmp_path / "m", cfg, seed=11)
    requests = rh.random_requests(cfg, [75, 1, 2, 19], seed=4)
    want = rh.plain_logits(folder, requests)
    got, _ = run(folder, "float32", helpers.trace_whole(requests), page=8)
    assert helpers.first_bad(got, want, TOL["float32"]) is None
    got, _ = run(folder, "float32", helpers.trace_chunked(requests, seed=3), page=8)
    assert helpers.first_bad(got, want, TOL["float32"]) is None


def test_what_the_tests_can_see(tmp_path):
    """The premises: without the sink's term in the denominator, with the query temperature one token late, with a
    convolution that forgets what lay before a portion, or with a state that starts a portion from zero, the plain
    logits move by far more than the tolerance."""
    cfg = single("both")
    folder = rh.write_folder(tmp_path / "m", cfg, seed=11)
    requests = rh.random_requests(cfg, [60], seed=4)
    want = rh.plain_logits(folder, requests)["r0"]
    margin = 100 * TOL["float32"] * np.abs(want).max()

    def no_sink(c, w):
        c["layers"][0]["mixer"]["test_without_sink"] = True
    assert np.abs(rh.plain_logits(folder, requests, no_sink)["r0"] - want).max() > margin

    exact = plain.query_temperature          # floor(p / every) instead of floor((p + 1) / every): differs at p = 7, 15, ...
    plain.query_temperature = lambda pos, coef, every, dtype: exact(pos - 1, coef, every, dtype)
    try:
        late = rh.plain_logits(folder, requests)["r0"]
    finally:
        plain.query_temperature = exact
    assert np.abs(late[7] - want[7]).max() > margin and np.abs(late[6] - want[6]).max() < 1e-9
    c, w = rh.read_folder(folder)
    tail = plain.forward(c, w, requests["r0"][30:]).numpy()          # history and state lost at token 30
    assert np.abs(tail[0] - want[30]).max() > margin and np.abs(tail[-1] - want[-1]).max() > margin


# ------------------------------------------------------------------ whole models, every cut
def traces_for(requests, max_live=4):
    return {"whole": helpers.trace_whole(requests), "tail": helpers.trace_decode_tail(requests, tail=32),
            "chunked": helpers.trace_chunked(requests, seed=1), "mixed": helpers.trace_mixed(requests, seed=2, max_live=max_live)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page", [("MIX", 8), ("WIDE", 16), ("ONE", 4), ("SAME", 16)])
def test_every_cut_matches_plain(tmp_path, name, page, dtype):
    cfg = getattr(rh, name)
    folder = rh.write_folder(tmp_path / name, cfg, seed=3, dtype=dtype)
    requests = rh.random_requests(cfg, LENGTHS, seed=5)
    want = rh.plain_logits(folder, requests)
    results = {}
    for tag, steps in traces_for(requests).items():
        got, session = run(folder, dtype, steps, page, max_live=4)
        assert {r: len(v) for r, v in got.items()} == {r: len(t) for r, t in requests.items()}, tag
        assert agrees(got, want, dtype), (tag, helpers.first_bad(got, want, TOL[dtype]), np.sort(row_errors(got, want))[-8:])
        if tag == "mixed":
            stats = session.runner.manager.stats()
            assert all(g["pages_taken"] > g["pages"] for g in stats["groups"]), "pages were not used again"
        results[tag] = got
    for tag in ("tail", "chunked", "mixed"):        # the cuts against each other: rounding only
        assert agrees(results[tag], {r: np.stack([results["whole"][r][p] for p in range(len(t))]) for r, t in requests.items()},
                      dtype), tag


def test_two_state_slots_serve_many_requests(tmp_path):
    """Slots (convolution histories and matrix states) and pages are handed from finished requests to new ones."""
    cfg = rh.MIX
    folder = rh.write_folder(tmp_path / "m", cfg, seed=8)
    requests = rh.random_requests(cfg, [30, 9, 41, 2, 17, 55, 5, 26], seed=9)
    want = rh.plain_logits(folder, requests)
    steps = helpers.trace_mixed(requests, seed=4, max_live=2, decode_tail=6)
    got, session = run(folder, "float32", steps, page=4, max_live=2)
    assert helpers.first_bad(got, want, TOL["float32"]) is None
    assert session.runner.manager.stats()["free_state_slots"] == 2


def test_batch_of_unequal_requests_equals_each_alone(tmp_path):
    cfg = rh.WIDE
    folder = rh.write_folder(tmp_path / "m", cfg, seed=5)
    requests = rh.random_requests(cfg, [50, 3, 128, 17], seed=2)
    together = [{"step": 0, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in requests.items()],
                 "end": list(requests)}]
    got, _ = run(folder, "float32", together, page=16)
    alone, _ = run(folder, "float32", helpers.trace_whole(requests), page=16)
    want = rh.plain_logits(folder, requests)
    assert helpers.first_bad(got, want, TOL["float32"]) is None
    scale = max(float(np.abs(w).max()) for w in want.values())
    assert max(float(np.abs(got[r][p] - alone[r][p]).max()) for r in requests for p in got[r]) / scale <= 1e-5


# ------------------------------------------------------------------ tokens far back, page borders
def test_far_tokens_carry_the_result(tmp_path):
    """A large score scale makes every softmax nearly one-hot on a key that lies anywhere in the context (or on the
    sink), and decays near one keep the first tokens in the matrix states, so a row that is missing, misplaced or
    read from the wrong page, or a state that was lost on the way, changes the logits. Positions around the borders
    of pages and of the kernels' key tiles are decoded one by one."""
    sharp = rh.left(3, 1, 16, 24, scale=1.5, conv=2, q_temp=(0.3, 64))
    cfg = rh.config([rh.parallel(sharp, rh.right(2, 16, 16, tau=40.0), left_scale=1.0, right_scale=0.5),
                     rh.parallel(sharp, rh.right(2, 16, 16, tau=40.0), left_scale=1.0, right_scale=0.5),
                     rh.mamba(4, 16, 16, 2, conv=2, norm_groups=1)], width=64, streams=2)

    def slow(t):
        t["l2.mix.A_log"] = torch.full_like(t["l2.mix.A_log"], -6.0)
    folder = rh.write_folder(tmp_path / "m", cfg, seed=21, edit=slow)
    requests = rh.random_requests(cfg, [700], seed=13)
    tokens = requests["r0"]
    want = rh.plain_logits(folder, requests)
    c, w = rh.read_folder(folder)
    cut = plain.forward(c, w, tokens[64:]).numpy()
    assert np.abs(cut[-40:] - want["r0"][-40:]).max() > 100 * TOL["float32"] * np.abs(want["r0"]).max()
    for steps in (helpers.trace_whole(requests), helpers.trace_decode_tail(requests, tail=140),
                  helpers.trace_chunked(requests, seed=7)):
        got, _ = run(folder, "float32", steps, page=16)
        assert helpers.first_bad(got, want, TOL["float32"]) is None
    folder16 = rh.write_folder(tmp_path / "m16", cfg, seed=21, dtype="bfloat16", edit=slow)
    want16 = rh.plain_logits(folder16, requests)
    for steps in (helpers.trace_whole(requests), helpers.trace_decode_tail(requests, tail=140),
                  helpers.trace_chunked(requests, seed=7)):
        got, _ = run(folder16, "bfloat16", steps, page=16)
        err = row_errors(got, want16)
        assert np.isfinite(err).all() and np.median(err) <= 2e-2 and (err > 0.15).mean() <= 0.02, np.sort(err)[-5:]


# ------------------------------------------------------------------ long decoding through graphs
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_replays_graphs(tmp_path, dtype):
    cfg = rh.MIX
    folder = rh.write_folder(tmp_path / "m", cfg, seed=6, dtype=dtype)
    requests = rh.random_requests(cfg, [160, 150], seed=1)
    want = rh.plain_logits(folder, requests)
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
    cfg = rh.MIX
    folder = rh.write_folder(tmp_path / "m", cfg, seed=3, dtype=dtype)
    llm = LLM(folder, dtype=dtype, max_num_batched_tokens=24, max_num_seqs=3, kvcache_block_size=8,
              num_kvcache_blocks=40, prefill_chunk=9, max_model_len=128)
    assert llm.config.enable_prefix_caching is False          # a state cannot be rebuilt from pages
    prompts = list(rh.random_requests(cfg, [1, 7, 16, 33, 50], seed=6).values())
    outs = llm.generate(prompts, SamplingParams(greedy=True, max_tokens=10))
    c, w = rh.read_folder(folder)
    for p, o in zip(prompts, outs):
        assert o["all_token_ids"] == p + o["token_ids"] and len(o["token_ids"]) == 10
        logits = plain.forward(c, w, p + o["token_ids"]).numpy()
        for i, tok in enumerate(o["token_ids"]):          # teacher forcing: the token has (nearly) the largest plain logit
            row = logits[len(p) - 1 + i]
            assert row.max() - row[tok] <= tol * np.abs(logits).max()
    assert not llm.runner.manager.live_requests
    llm.runner.manager.check_consistency()
    llm.close()


def test_command_line_generates_with_a_folder_and_with_a_preset(tmp_path):
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    folder = rh.write_folder(tmp_path / "m", rh.ONE, seed=3)
    common = ["--dtype", "fp32", "--prompt-ids", "5,17,3,200", "--prompt-len", "9", "--greedy", "--max-tokens", "6",
              "--max-num-seqs", "2", "--max-num-batched-tokens", "16", "--block-size", "4", "--num-kvcache-blocks", "32",
              "--max-model-len", "64"]
    res = subprocess.run([sys.executable, str(root / "examples" / "generate.py"), "--model", str(folder)] + common,
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    rows = [json.loads(l) for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(rows) == 2 and all(len(r["token_ids"]) == 6 for r in rows)
    c, w = rh.read_folder(folder)
    logits = plain.forward(c, w, [5, 17, 3, 200] + rows[0]["token_ids"]).numpy()
    for i, tok in enumerate(rows[0]["token_ids"]):
        assert logits[3 + i].max() - logits[3 + i][tok] <= 1e-4 * np.abs(logits).max()
    res = subprocess.run([sys.executable, str(root / "examples" / "generate.py"), "--random-config", "ravutar-tiny"] + common,
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]


def random_config(seed):
    """A model of random sizes and layer order: odd head counts and sizes, one to five taps, with and without
    streams, loops, query temperature and feed-forward."""
    import random
    rng = random.Random(seed)
    width = rng.choice([40, 72, 100, 136])
    layers = []
    for _ in range(rng.randint(2, 5)):
        mlp = None if rng.random() < 0.25 else rh.dense(rng.choice([24, 56, 136]))
        if rng.random() < 0.6:
            kv = rng.randint(1, 3)
            a = rh.left(kv * rng.randint(1, 3), kv, rng.choice([8, 12, 20, 40]), rng.choice([4, 8, 24, 36]),
                        scale=rng.uniform(0.1, 0.5), conv=rng.choice([None, 1, 2, 3, 5]),
                        q_temp=None if rng.random() < 0.3 else (rng.uniform(0.1, 0.6), rng.choice([1, 3, 16, 50])))
            b = rh.right(rng.randint(1, 5), rng.choice([8, 12, 36, 72]), rng.choice([4, 12, 20, 40]), tau=rng.uniform(2, 30),
                         gate_rank=rng.choice([3, 8, 16]))
            layers.append(rh.parallel(a, b, left_scale=rng.uniform(0.3, 1.5), right_scale=rng.uniform(0.3, 1.5), mlp=mlp))
        else:
            groups = rng.randint(1, 3)
            heads = groups * rng.randint(1, 3)
            vdim = rng.choice([4, 12, 20, 32])
            norm_groups = rng.choice([g for g in (1, 2, 3, 4, heads) if (heads * vdim) % g == 0])
            layers.append(rh.mamba(heads, vdim, rng.choice([8, 20, 48]), groups, conv=rng.randint(1, 5), norm_groups=norm_groups, mlp=mlp))
    loop = None
    if rng.random() < 0.6:
        start = rng.randrange(len(layers))
        loop = (start, rng.randint(start + 1, len(layers)), rng.randint(1, 3))
    return rh.config(layers, vocab=rng.choice([97, 256, 300]), width=width, eps=rng.choice([1e-5, 1e-6]),
                     logit_scale=rng.choice([0.3, 1.0, 2.0]), streams=rng.choice([None, 1, 2, 4]), loop=loop)


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_models_of_random_sizes_and_orders(tmp_path, seed):
    cfg = random_config(seed)
    page = [4, 8, 16, 32, 64, 16][seed - 1]
    requests = rh.random_requests(cfg, [70, 1, 37, 150, 2, 64], seed=seed)
    folder = rh.write_folder(tmp_path / "m", cfg, seed=seed)
    want = rh.plain_logits(folder, requests)
    for steps in (helpers.trace_whole(requests), helpers.trace_mixed(requests, seed=seed, max_live=3, decode_tail=20)):
        got, _ = run(folder, "float32", steps, page, max_live=3)
        assert helpers.first_bad(got, want, TOL["float32"]) is None, cfg
    folder16 = rh.write_folder(tmp_path / "m16", cfg, seed=seed, dtype="bfloat16")
    got, _ = run(folder16, "bfloat16", helpers.trace_mixed(requests, seed=seed, max_live=3, decode_tail=20), page, max_live=3)
    err = row_errors(got, rh.plain_logits(folder16, requests))
    assert np.isfinite(err).all() and np.median(err) <= TOL["bfloat16"] / 2, (np.median(err), cfg)
