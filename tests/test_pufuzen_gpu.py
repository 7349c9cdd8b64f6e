"""The Pufuzen decoder on the GPU against the plain restatement: each mechanism's kernels alone,
then whole models (three tiny configurations of unlike sizes) whole, token by token, in portions,
in mixed batches on few pages and slots, and through the generation entry point."""
import math

import numpy as np
import pytest
import torch

import plain_pufuzen as plain
import replay_util as ru
from tiny import random_ids
from tiny_pufuzen import TINY, make_folder, reference_logits

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from tokenizer_b200.kernels import ops as o
    return o


def rnd(*shape, seed=0, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def close(got, want, dtype, what=""):
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    bound = tol * max(1.0, float(want.abs().max()))
    err = float((got - want).abs().max())
    assert torch.isfinite(got).all() and err <= bound, f"{what}: max |diff| {err:.3e} > {bound:.3e}"


# ---- the recurrence --------------------------------------------------------------------------
def recurrence_reference(zp, u, g, state):
    """Token by token in float64: returns the outputs and the state after the last token."""
    z = 1.0 / (1.0 + torch.exp(-zp))
    cand = torch.where(u >= 0, u + 0.5, 1.0 / (1.0 + torch.exp(-u)))
    s, rows = state.clone(), []
    for t in range(zp.shape[0]):
        s = (1.0 - z[t]) * s + z[t] * cand[t]
        rows.append(s * g[t] / (1.0 + torch.exp(-g[t])))
    return torch.stack(rows), s


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,lengths", [(40, [1, 1, 1]), (72, [5, 130, 1, 17]), (320, [300]), (33, [2, 129])])
def test_min_gru_scan_carries_each_request_its_own_state(width, lengths, out_dtype):
    total, extra = sum(lengths), 11                       # the three ranges lie inside a wider product
    proj = rnd(total, 3 * width + extra, seed=1, scale=2.0)
    bias = rnd(3 * width + extra, seed=12)                # the product's bias is added by the kernel
    slots = [3, 0, 5, 1][:len(lengths)]
    state = rnd(6, width, seed=2)
    before = state.clone()
    starts = np.concatenate(([0], np.cumsum(lengths))).astype(np.int32)
    q_start = torch.tensor(starts, device=DEV)
    slot_t = torch.tensor(slots, dtype=torch.int32, device=DEV)
    out = torch.empty(total, width, dtype=out_dtype, device=DEV)
    # in two calls: every request's first half, then the rest, with the state carried between
    for part in (0, 1):
        rows, spans = [], [0]
        for r, n in enumerate(lengths):
            cut = n // 2
            lo, hi = (starts[r], starts[r] + cut) if part == 0 else (starts[r] + cut, starts[r + 1])
            rows += list(range(lo, hi))
            spans.append(len(rows))
        if not rows:
            continue
        sub = proj[torch.tensor(rows, device=DEV)].contiguous()
        sub_out = torch.empty(len(rows), width, dtype=out_dtype, device=DEV)
        longest = max(b - a for a, b in zip(spans, spans[1:]))
        ops().min_gru_scan(sub, extra, extra + width, extra + 2 * width, width, state,
                           torch.tensor(spans, dtype=torch.int32, device=DEV), slot_t, longest, sub_out, bias=bias)
        out[torch.tensor(rows, device=DEV)] = sub_out
    p = proj.double().cpu() + bias.double().cpu()
    for r, n in enumerate(lengths):
        rows = slice(starts[r], starts[r + 1])
        want, end = recurrence_reference(p[rows, extra:extra + width], p[rows, extra + width:extra + 2 * width],
                                         p[rows, extra + 2 * width:extra + 3 * width], before[slots[r]].double().cpu())
        close(out[rows], want, out_dtype, f"request {r}")
        close(state[slots[r]], end, torch.float32, f"state of request {r}")
    untouched = [s for s in range(6) if s not in slots]
    assert torch.equal(state[untouched], before[untouched])
    # the same in one call
    state2, out2 = before.clone(), torch.empty_like(out)
    ops().min_gru_scan(proj, extra, extra + width, extra + 2 * width, width, state2, q_start, slot_t, max(lengths), out2,
                       bias=bias)
    close(out2, out, out_dtype, "one call against two")
    close(state2, state, torch.float32)


# ---- activation and gate ------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [7, 136, 1500])
def test_poly_norm(dtype, n):
    wide = rnd(9, n + 40, seed=3, scale=1.5)
    coeff = torch.tensor([0.7, -0.3, 0.2, 0.05], device=DEV)
    out = torch.empty(9, n, dtype=dtype, device=DEV)
    bias = rnd(n + 40, seed=13)
    ops().poly_norm(wide[:, :n], coeff, 1e-5, out, bias=bias[:n])
    z = wide[:, :n].double().cpu() + bias[:n].double().cpu()
    norm = lambda v: v / torch.sqrt((v * v).mean(-1, keepdim=True) + 1e-5)
    close(out, 0.7 * norm(z) - 0.3 * norm(z * z) + 0.2 * norm(z ** 3) + 0.05, dtype)


def test_gated_delta_takes_a_product_whole_or_in_partial_sums():
    rows, hidden = 13, 50
    pre_wide = rnd(rows, 30 + hidden, seed=4, scale=2.0)
    pre = pre_wide[:, 30:]
    gate = torch.sigmoid(pre.double().cpu())
    y = rnd(rows, hidden, seed=5, dtype=torch.bfloat16)
    out = torch.empty(rows, hidden, device=DEV)
    ops().gated_delta(y, None, pre, out)
    close(out, y.double().cpu() * gate, torch.float32)
    parts, bias = rnd(3, rows, hidden, seed=6), rnd(hidden, seed=7)
    ops().gated_delta(parts, bias, pre, out)
    close(out, (parts.double().cpu().sum(0) + bias.double().cpu()) * gate, torch.float32)
    # the gate's own bias; lanes that 16-byte loads do not fit (a width of 50, a slice that starts at lane 30)
    pre_bias = rnd(hidden + 1, seed=14)[1:]
    ops().gated_delta(parts, bias, pre, out, pre_bias=pre_bias)
    gate = torch.sigmoid(pre.double().cpu() + pre_bias.double().cpu())
    close(out, (parts.double().cpu().sum(0) + bias.double().cpu()) * gate, torch.float32)
    wide_pre, wide_bias = rnd(rows, 64 + 32, seed=15), rnd(64, seed=16)
    y64, out64 = rnd(rows, 64, seed=17, dtype=torch.bfloat16), torch.empty(rows, 64, device=DEV)
    ops().gated_delta(y64, None, wide_pre[:, 32:], out64, pre_bias=wide_bias)
    close(out64, y64.double().cpu() * torch.sigmoid(wide_pre[:, 32:].double().cpu() + wide_bias.double().cpu()),
          torch.float32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,partials", [(50, 0), (1030, 3), (4500, 2), (256, 0)])
def test_gate_residual_add_and_norm_in_one_kernel(dtype, hidden, partials):
    rows = 7
    x = rnd(rows, hidden, seed=30)
    before = x.clone()
    wide = rnd(rows, 12 + hidden, seed=31, scale=2.0)
    pre, pre_bias, gain = wide[:, 12:], rnd(hidden, seed=32), rnd(hidden, seed=33) + 1.0
    if partials:
        y, bias = rnd(partials, rows, hidden, seed=34), rnd(hidden, seed=35)
        total = y.double().cpu().sum(0) + bias.double().cpu()
    else:
        y, bias = rnd(rows, hidden, seed=34, dtype=torch.bfloat16), None
        total = y.double().cpu()
    out = torch.empty(rows, hidden, dtype=dtype, device=DEV)
    ops().gated_add_rms_norm(x, y, bias, pre, pre_bias, gain, 1e-5, out)
    want_x = before.double().cpu() + total * torch.sigmoid(pre.double().cpu() + pre_bias.double().cpu())
    close(x, want_x, torch.float32, "the stream after the add")
    close(out, plain.rms_norm(want_x, gain.double().cpu(), 1e-5), dtype, "the normed rows")


# ---- the kernels around the cached latent -------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("q_rank,kv_rank,rot_dim,rot_dims", [(40, 48, 0, 0), (56, 24, 8, 8), (20, 130, 10, 6)])
def test_latent_rows_are_normed_rotated_and_written_to_their_slots(dtype, q_rank, kv_rank, rot_dim, rot_dims):
    rows, side = 9, 17
    row = -(-(kv_rank + rot_dim) // 16) * 16
    proj = rnd(rows, q_rank + kv_rank + rot_dim + side, seed=8, scale=3.0)
    q_gain, c_gain = rnd(q_rank, seed=9) + 1.0, rnd(kv_rank, seed=10) + 1.0
    pos = torch.tensor([0, 1, 2, 700, 5, 6, 7, 31, 1000], dtype=torch.int32, device=DEV)
    req = torch.tensor([0, 0, 0, 1, 2, 2, -1, 3, 3], dtype=torch.int32, device=DEV)      # one idle row
    slot = torch.tensor([5, 3, 20, 7, 0, 11, -1, 2, 9], dtype=torch.int32, device=DEV)
    freq = torch.tensor([77.0 ** (-2.0 * i / rot_dims) for i in range(rot_dims // 2)] or [1.0],
                        dtype=torch.float64).float().to(DEV)
    pool = torch.zeros(24, 1, row, dtype=dtype, device=DEV)
    cq = torch.zeros(rows, q_rank, dtype=dtype, device=DEV)
    ops().latent_prepare(proj, 0, q_rank, q_rank, kv_rank, rot_dim, rot_dims, q_gain, c_gain, 1e-5,
                         freq if rot_dims else None, pos, req, slot, cq, pool)
    p = proj.double().cpu()
    want_q = plain.rms_norm(p[:, :q_rank], q_gain.double().cpu(), 1e-5)
    want_c = plain.rms_norm(p[:, q_rank:q_rank + kv_rank], c_gain.double().cpu(), 1e-5)
    shared = p[:, q_rank + kv_rank:q_rank + kv_rank + rot_dim]
    if rot_dims:
        shared = plain.rotate_interleaved(shared, pos.cpu(), 77.0, rot_dims)
    live = [t for t in range(rows) if int(req[t]) >= 0]
    close(cq[live], want_q[live], dtype, "query latent")
    written = pool[slot[live].long(), 0]
    close(written[:, :kv_rank], want_c[live], dtype, "cached latent")
    if rot_dim:
        close(written[:, kv_rank:kv_rank + rot_dim], shared[live], dtype, "positional key part")
    assert float(written[:, kv_rank + rot_dim:].abs().max() if row > kv_rank + rot_dim else 0.0) == 0.0
    free = [s for s in range(24) if s not in slot[live].tolist()]
    assert float(pool[free].abs().max()) == 0.0 and float(cq[6].abs().max()) == 0.0
    # the queries' positional lanes, in place, head by head
    if rot_dims:
        heads = 3
        x = rnd(rows, heads * row, seed=11, dtype=dtype)
        kept = x.clone()
        ops().rotate_interleaved(x, heads, kv_rank, rot_dims, freq, pos, req)
        want = kept.double().cpu().view(rows, heads, row)
        want[..., kv_rank:kv_rank + rot_dims] = plain.rotate_interleaved(
            want[..., kv_rank:kv_rank + rot_dims], pos.cpu(), 77.0, rot_dims)
        close(x[live], want.view(rows, -1)[live], dtype, "rotated query lanes")
        assert torch.equal(x[6], kept[6])


def latent_cache(lengths, row, page, dtype, seed):
    """One row a token, scattered over shuffled pages: pool, tables and the dense rows."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-n // page) for n in lengths) + 2
    order = torch.randperm(n_pages, generator=g).tolist()
    pool = torch.full((n_pages * page, 1, row), float("nan"), dtype=dtype)
    tables = torch.full((len(lengths), max(-(-n // page) for n in lengths) + 1), -1, dtype=torch.int32)
    dense = []
    for r, n in enumerate(lengths):
        c = torch.randn(n, row, generator=g).to(dtype)
        for b in range(-(-n // page)):
            pg = order.pop()
            tables[r, b] = pg
            rows = slice(b * page, min(n, (b + 1) * page))
            pool[pg * page:pg * page + rows.stop - rows.start, 0] = c[rows]
        dense.append(c.float())
    return pool.to(DEV), tables.to(DEV), dense


def sink_reference(q, dense, row_req, pos, heads, window, scale, sink):
    """Every head attends over the request's rows; the values are the rows themselves; the sink
    counts once in the denominator."""
    out = torch.zeros_like(q)
    for t in range(q.shape[0]):
        c = dense[row_req[t]].double()
        lo = 0 if window is None else max(0, pos[t] - window)
        for h in range(heads):
            s = (c[lo:pos[t] + 1] @ q[t, h].double()) * scale
            top = max(float(s.max()), float(sink[h])) if sink is not None else float(s.max())
            e = torch.exp(s - top)
            total = e.sum() + (math.exp(float(sink[h]) - top) if sink is not None else 0.0)
            out[t, h] = ((e / total) @ c[lo:pos[t] + 1]).float()
    return out


@pytest.mark.parametrize("kernel,dtype,heads,row,window", [
    ("generic", torch.float32, 3, 48, None), ("generic", torch.bfloat16, 17, 144, 20), ("generic", torch.float32, 5, 32, 6),
    ("generic", torch.bfloat16, 2, 640, None),
    ("decode", torch.bfloat16, 5, 32, None), ("decode", torch.bfloat16, 16, 64, 32), ("decode", torch.bfloat16, 2, 128, None),
    ("tiles", torch.bfloat16, 3, 48, 6), ("tiles", torch.bfloat16, 4, 80, None),
    ("wide", torch.bfloat16, 2, 128, None), ("wide", torch.bfloat16, 6, 128, 95), ("wide", torch.bfloat16, 3, 64, None)])
def test_a_sink_and_values_that_are_the_key_rows_in_every_attention_kernel(kernel, dtype, heads, row, window):
    from tokenizer_b200.parts.attention import RowTiles
    o = ops()
    page = 16
    lengths = [700, 130, 1, 260]
    pool, tables, dense = latent_cache(lengths, row, page, dtype, seed=20)
    sink = torch.tensor([2.0, -1.0, 0.5, 4.0, 0.0, -3.0, 1.0, 2.5, 0.1, 0.2, 0.3, 0.4, 3.0, 1.5, -0.5, 0.7, 6.0][:heads],
                        device=DEV)
    scale = 1.0 / math.sqrt(row)
    if kernel == "decode":
        row_req, pos, spans = [0, 1, 2, 3], [n - 1 for n in lengths], None
    else:
        # a portion at the end of every request: (request, first position, rows)
        spans = [(0, 700 - 130, 130), (1, 0, 130), (2, 0, 1), (3, 260 - 97, 97)]
        row_req = [r for r, _, n in spans for _ in range(n)]
        pos = [first + i for _, first, n in spans for i in range(n)]
    q = rnd(len(pos), heads, row, seed=21, dtype=dtype, scale=2.0)
    out = torch.full((len(pos), heads * row), float("nan"), dtype=dtype, device=DEV)
    req_t, pos_t = torch.tensor(row_req, dtype=torch.int32, device=DEV), torch.tensor(pos, dtype=torch.int32, device=DEV)
    args = (q.view(len(pos), -1), pool, pool, out, tables, req_t, pos_t)
    if kernel == "generic":
        o.paged_attention_generic(*args, heads, 1, row, page, window, scale, sink=sink)
    elif kernel == "decode":
        o.decode_attention(*args, heads, 1, row, page, window, scale, sink=sink)
    else:
        note = RowTiles(o.WIDE_TILE_ROWS if kernel == "wide" else o.PREFILL_TILE_ROWS)
        words = np.zeros(note.capacity(len(pos), len(spans)), dtype=np.int32)
        counts = np.array([n for _, _, n in spans], dtype=np.int32)
        firsts = np.concatenate(([0], np.cumsum(counts)[:-1])).astype(np.int32)
        n_tiles = note.fill(words, firsts, counts, np.array([f for _, f, _ in spans], dtype=np.int32), False)
        tiles = torch.tensor(words, device=DEV).view(-1, 2)
        run = o.attention_tcgen05 if kernel == "wide" else o.prefill_attention
        run(*args, tiles, n_tiles, heads, 1, row, page, window, scale, sink=sink)
    want = sink_reference(q.float().cpu(), dense, row_req, pos, heads, window, scale, sink.cpu())
    got = out.view(len(pos), heads, row).float().cpu()
    assert torch.isfinite(got).all()
    bound = 2e-5 if dtype == torch.float32 else 3e-2
    assert float((got - want).abs().max()) <= bound * max(1.0, float(want.abs().max()))
    # the sink matters: without it the rows with a large sink come out elsewhere
    plain_softmax = sink_reference(q.float().cpu(), dense, row_req, pos, heads, window, scale, None)
    assert float((plain_softmax - want).abs().max()) > 0.1


# ---- whole models -----------------------------------------------------------------------------------
LENGTHS = {"p": [1, 2, 23, 100, 131, 64], "q": [5, 19, 97, 140, 260, 33], "r": [3, 40, 130, 64, 17, 90],
           "s": [1, 9, 70, 129, 30, 2], "t": [2, 50, 140, 7, 33]}


@pytest.fixture(scope="module", params=sorted(TINY))
def model(request, tmp_path_factory):
    folder, cfg, page = make_folder(tmp_path_factory, request.param)
    requests = {f"r{i}": random_ids(n, cfg.vocab, 300 + i) for i, n in enumerate(LENGTHS[request.param])}
    return folder, cfg, page, requests, reference_logits(folder, requests)


def replay(folder, dtype, steps, max_tokens, page, max_requests=4, use_graphs=True):
    """What the replay program does, inside this process: every step through `Engine.step` on a
    pool of `max_tokens` tokens and `max_requests` slots; returns {step: logits}."""
    from tokenizer_b200.engine import Engine, StepEntry
    engine = Engine.from_folder(folder, dtype=dtype, num_pages=-(-max_tokens // page), page_size=page,
                                max_requests=max_requests, use_graphs=use_graphs)
    live, out = {}, {}
    for record in steps:
        entries = []
        for item in record["entries"]:
            if item["id"] not in live:
                live[item["id"]] = engine.cache.open(item["id"])
            engine.cache.reserve(live[item["id"]], len(item["tokens"]))
            entries.append(StepEntry(live[item["id"]], item["tokens"], item.get("want", [])))
        logits = engine.step(entries)
        if logits.shape[0]:
            out[record["step"]] = logits.cpu().numpy()
        for name in record.get("end", []):
            engine.cache.close(live.pop(name))
        engine.cache.check()
    engine.check()
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts(model, dtype):
    folder, cfg, page, requests, want = model
    steps = ru.steps_whole(requests)
    budget = max(ru.rounded64(len(v)) for v in requests.values())
    got = ru.collect(steps, replay(folder, dtype, steps, budget, page))
    assert {k: len(v) for k, v in got.items()} == {k: len(v) for k, v in requests.items()}
    ru.compare(got, want, dtype, "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_then_token_by_token(model, dtype):
    """The last 40 tokens one by one: more than the windows of 1, 7 and 33 keys, so that a window
    passes over decoded tokens, and the recurrent state is carried through every step."""
    folder, cfg, page, requests, want = model
    steps = ru.steps_decode_tail(requests, 40)
    budget = max(ru.rounded64(len(v)) for v in requests.values())
    got = ru.collect(steps, replay(folder, dtype, steps, budget, page))
    ru.compare(got, want, dtype, "decode tail")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(2, 7, 3, 16, 2, 33, 5, 2, 64, 9), (2,), (31, 1, 1, 96)])
def test_portions(model, dtype, sizes):
    folder, cfg, page, requests, want = model
    if sizes == (2,):
        requests = {k: v for k, v in requests.items() if len(v) <= 100}
    steps = ru.steps_portions(requests, sizes)
    budget = max(ru.rounded64(len(v)) for v in requests.values())
    got = ru.collect(steps, replay(folder, dtype, steps, budget, page))
    assert {k: len(v) for k, v in got.items()} == {k: len(v) for k, v in requests.items()}
    ru.compare(got, want, dtype, f"portions {sizes}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("live", [4, 2])
def test_mixed_batches_on_pages_and_slots_that_are_used_again(model, dtype, live):
    folder, cfg, page, requests, want = model
    steps, peak = ru.steps_mixed(requests, max_live=live, seed=live)
    assert peak < sum(ru.rounded64(len(v)) for v in requests.values()) and len(requests) > live
    got = ru.collect(steps, replay(folder, dtype, steps, peak, page, max_requests=live))
    assert {k: len(v) for k, v in got.items()} == {k: len(v) for k, v in requests.items()}
    ru.compare(got, want, dtype, "mixed")


def test_replay_program_drives_the_same_engine(model, tmp_path):
    folder, cfg, page, requests, want = model
    steps, peak = ru.steps_mixed(requests, max_live=3, seed=9)
    out = ru.run_trace(folder, "float32", steps, str(tmp_path), peak, page)
    ru.compare(ru.collect(steps, out), want, "float32", "the replay program")


# ---- generation ---------------------------------------------------------------------------------------
def near_best(cfg, w, prompt, tokens, dtype):
    logits = plain.forward(cfg, w, list(prompt) + list(tokens)).float()
    lead = logits[len(prompt) - 1:-1]
    chosen = lead.gather(1, torch.tensor(tokens)[:, None])[:, 0]
    slack = 1e-4 if dtype == "float32" else 0.04 * float(logits.abs().max())
    gap = lead.max(dim=1).values - chosen
    assert float(gap.max()) <= slack, f"token {int(gap.argmax())} lies {float(gap.max())} below the best logit"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(model, dtype):
    import tokenizer_b200 as tb
    folder, cfg, page, requests, _ = model
    raw, w = plain.load_folder(folder)
    engine_model = tb.load_model(folder, dtype=dtype)
    for n in (1, 9, 70):
        prompt = random_ids(n, cfg.vocab, 500 + n)
        out = tb.generate(engine_model, prompt, tb.GenerateParams.greedy(24))
        assert out.reason == tb.StopReason.MAX_TOKENS and len(out.tokens) == 24
        if dtype == "float32":
            assert out.tokens == plain.greedy_generate(raw, w, prompt, 24)
        near_best(raw, w, prompt, out.tokens, dtype)


def test_a_batch_through_the_scheduler_with_preemption_gives_each_request_its_own_ids(model):
    """Five prompts on a pool that cannot hold them all: requests are preempted and computed
    again, which for a recurrence means a state that starts from zero again."""
    import tokenizer_b200 as tb
    folder, cfg, page, requests, _ = model
    raw, w = plain.load_folder(folder)
    engine_model = tb.load_model(folder, dtype="float32")
    prompts = [random_ids(n, cfg.vocab, 600 + n) for n in (30, 7, 55, 18, 41)]
    engine = tb.engine_for(engine_model, 192, page_size=page, max_requests=3, share_prefixes=False)
    results = tb.generate_batch(engine, prompts, tb.GenerateParams.greedy(20), max_batch_size=3, token_budget=48,
                                page_size=page)
    for prompt, result in zip(prompts, results):
        assert result.tokens == plain.greedy_generate(raw, w, prompt, 20)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_on_the_device(model, dtype):
    """300 greedy steps without a visit to the host between them (captured and replayed): windows
    slide over decoded tokens, pages behind them are given back, the states move on."""
    from tokenizer_b200.engine import Engine, StepEntry
    folder, cfg, page, requests, _ = model
    raw, w = plain.load_folder(folder)
    engine = Engine.from_folder(folder, dtype=dtype, num_pages=-(-2 * 384 // page), page_size=page, max_requests=2)
    prompts = [random_ids(5, cfg.vocab, 700), random_ids(41, cfg.vocab, 701)]
    caches, first = [], []
    for i, prompt in enumerate(prompts):
        c = engine.cache.open(i)
        engine.cache.reserve(c, len(prompt))
        first.append(int(engine.step([StepEntry(c, prompt, [len(prompt) - 1])]).argmax()))
        caches.append(c)
    history = engine.decode_steps([StepEntry(c, [t], [0]) for c, t in zip(caches, first)], 300)
    for i, prompt in enumerate(prompts):
        tokens = [first[i]] + [step[i] for step in history]
        if dtype == "float32":
            assert tokens == plain.greedy_generate(raw, w, prompt, 301)
        else:
            near_best(raw, w, prompt, tokens, dtype)


def test_the_command_line_generates_from_a_configuration_of_this_design(tmp_path):
    """`--random-weights config.json` draws the weights the configuration declares; two prompts go
    through the scheduler and print the ids each gets from the plain implementation."""
    import json
    import os
    import subprocess
    import sys
    import tokenizer_b200 as tb
    cfg, seed, page = TINY["p"]()
    path = str(tmp_path / "config.json")
    with open(path, "w") as fh:
        json.dump(cfg.to_dict(), fh)
    folder = tb.write_random_model(str(tmp_path / "same"), cfg, 0)        # the command line's default seed
    raw, w = plain.load_folder(folder)
    prompts = [random_ids(11, cfg.vocab, 801), random_ids(40, cfg.vocab, 802)]
    cli = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "qwen-infer")
    args = [sys.executable, cli, "--random-weights", path, "--weights-seed", "0", "--dtype", "float32",
            "--max-tokens", "10", "--page-size", str(page)]
    for prompt in prompts:
        args += ["--ids", ",".join(str(t) for t in prompt)]
    proc = subprocess.run(args, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    want = [" ".join(str(t) for t in plain.greedy_generate(raw, w, prompt, 10)) for prompt in prompts]
    assert proc.stdout.strip().splitlines() == want
