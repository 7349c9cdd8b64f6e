"""The Katopel decoder on the GPU against the plain restatement: each mechanism's kernels alone,
then whole models (four tiny configurations of unlike sizes) whole, token by token, in portions,
in mixed batches on few pages and slots, and through the generation entry point."""
import math

import numpy as np
import pytest
import torch

import plain_katopel as plain
import replay_util as ru
from tiny import random_ids
from tiny_katopel import SHARPEN, TINY, make_folder, reference_logits

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


def ints(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


# ---- layer norm, and the norm on a sublayer's output with the add and the next norm ----------------
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [50, 96, 2048, 9001])
def test_layer_norm_with_bias_and_a_row_gather(width, out_dtype):
    x = rnd(7, width, seed=1, scale=3.0) + 2.0
    gain, bias = rnd(width, seed=2) + 1.0, rnd(width, seed=3)
    out = torch.empty(7, width, dtype=out_dtype, device=DEV)
    ops().layer_norm(x, gain, bias, 1e-5, out)
    want = plain.layer_norm(x.double().cpu(), gain.double().cpu(), bias.double().cpu(), 1e-5)
    close(out, want, out_dtype, "layer norm")
    rows = ints([5, 0, 5])
    some = torch.empty(3, width, dtype=out_dtype, device=DEV)
    ops().layer_norm(x, gain, bias, 1e-5, some, rows=rows)
    close(some, want[[5, 0, 5]], out_dtype, "gathered rows")


@pytest.mark.parametrize("width", [50, 192, 9001])
@pytest.mark.parametrize("form", ["bf16", "f32", "partials", "two terms"])
@pytest.mark.parametrize("chained", [False, True])
def test_the_norm_behind_a_sublayer_adds_and_norms_again(width, form, chained):
    o = ops()
    x = rnd(5, width, seed=4, scale=2.0)
    g1, b1, g2, b2 = rnd(width, seed=5) + 1.0, rnd(width, seed=6), rnd(width, seed=7) + 1.0, rnd(width, seed=8)
    if form == "bf16":
        terms = [(rnd(5, width, seed=9, dtype=torch.bfloat16), 1.0)]
    elif form == "f32":
        terms = [(rnd(5, width, seed=9), 1.0)]
    elif form == "partials":
        terms = [(rnd(3, 5, width, seed=9), 1.0)]
    else:
        terms = [(rnd(2, 5, width, seed=9), 0.7), (rnd(5, width, seed=10, dtype=torch.bfloat16), 1.7)]
    y = sum((t.double().cpu() if t.dim() == 2 else t.double().cpu().sum(0)) * s for t, s in terms)
    want_x = x.double().cpu() + plain.layer_norm(y, g1.double().cpu(), b1.double().cpu(), 1e-6)
    out = torch.empty(5, width, dtype=torch.bfloat16, device=DEV) if chained else None
    got_x = x.clone()
    o.post_norm_add(got_x, terms, g1, b1, 1e-6, g2 if chained else None, b2 if chained else None, 3e-6, out)
    close(got_x, want_x, torch.float32, "the stream after the add")
    if chained:
        close(out, plain.layer_norm(want_x, g2.double().cpu(), b2.double().cpu(), 3e-6), torch.bfloat16, "the next norm")
    summed = torch.empty(5, width, dtype=torch.float32, device=DEV)
    o.scaled_sum(terms, summed)
    close(summed, y, torch.float32, "the scaled sum")


def test_what_a_pass_adds_to_the_stream():
    x, other, vector = rnd(6, 50, seed=1), rnd(6, 50, seed=2), rnd(50, seed=3)
    for a, b in ((other, vector), (None, vector), (other, None)):
        got = x.clone()
        ops().stream_inject(got, a, b)
        want = x + (a if a is not None else 0) + (b if b is not None else 0)
        assert torch.allclose(got, want, atol=1e-6)


# ---- the gated delta rule ----------------------------------------------------------------------------
def delta_inputs(groups, heads, dim, vdim, taps, total, seed, extra=5):
    """A stacked product with this mixer's columns behind `extra` foreign ones, and its small tensors."""
    channels = 2 * groups * dim + heads * vdim
    proj = rnd(total, extra + channels + 2 * heads + 3, seed=seed, scale=1.5)
    conv = rnd(channels, taps, seed=seed + 1, scale=0.7)
    a_log, dt_bias = rnd(heads, seed=seed + 2, scale=0.5), rnd(heads, seed=seed + 3, scale=0.5) - 2.0
    return proj, conv, a_log, dt_bias, channels


def plain_prepared(proj, conv, a_log, dt_bias, groups, heads, dim, vdim, extra=5):
    """q, k (unit vectors), v, beta and the decay of one request's rows from its start, in float64."""
    p = proj.double().cpu()
    channels = 2 * groups * dim + heads * vdim
    c, _ = plain.short_convolution(p[:, extra:extra + channels], conv.double().cpu())
    c = plain.silu(c)
    n = p.shape[0]
    q = plain.unit_vectors(c[:, :groups * dim].view(n, groups, dim)) * dim ** -0.5
    k = plain.unit_vectors(c[:, groups * dim:2 * groups * dim].view(n, groups, dim))
    v = c[:, 2 * groups * dim:].view(n, heads, vdim)
    beta = plain.sigmoid(p[:, extra + channels:extra + channels + heads])
    a = p[:, extra + channels + heads:extra + channels + 2 * heads] + dt_bias.double().cpu()
    decay = torch.exp(-torch.exp(a_log.double().cpu()) * plain.softplus(a))
    return q, k, v, beta, decay


def run_in_portions(lengths, cuts, slots, fn):
    """Call fn(rows of the step, spans [R + 1], slots) once per portion index: request r brings
    rows cuts[r][i] .. cuts[r][i + 1] of its own to step i (nothing when it has no such portion)."""
    starts = np.concatenate(([0], np.cumsum(lengths)))
    for i in range(max(len(c) for c in cuts) - 1):
        rows, spans, who = [], [0], []
        for r in range(len(lengths)):
            if i + 1 < len(cuts[r]):
                rows += list(range(starts[r] + cuts[r][i], starts[r] + cuts[r][i + 1]))
                spans.append(len(rows))
                who.append(slots[r])
        if rows:
            fn(rows, spans, who)


@pytest.mark.parametrize("groups,heads,dim,vdim,taps", [(2, 4, 16, 24, 4), (1, 1, 10, 6, 5), (3, 3, 64, 128, 2),
                                                         (1, 2, 260, 8, 3), (2, 2, 8, 8, 1), (2, 4, 128, 64, 4),
                                                         (1, 2, 96, 20, 3)])
@pytest.mark.parametrize("chunks", [False, True])
def test_the_delta_rule_in_portions_carries_matrices_and_kept_inputs(groups, heads, dim, vdim, taps, chunks):
    """Three requests in slots that are not their indices, cut into portions of 1, 2 and many rows (shorter
    than the convolution too), against the recurrence token by token from each request's start."""
    o = ops()
    lengths = [37, 1, 150]
    cuts = [[0, 1, 3, 4, 20, 37], [0, 1], [0, 130, 132, 133, 150]]
    slots = [2, 0, 3]
    total, extra = sum(lengths), 5
    proj, conv, a_log, dt_bias, channels = delta_inputs(groups, heads, dim, vdim, taps, total, seed=30)
    padded = o.gdn_padded_dim(dim)
    conv_off = heads * vdim * padded
    floats = -(-(conv_off + (taps - 1) * channels) // 4) * 4
    state = torch.zeros(5, floats, device=DEV)
    state[1] = 7.0                                        # a slot nobody holds must stay as it is
    out = torch.full((total, heads * vdim), float("nan"), device=DEV)

    def step(rows, spans, who):
        idx = torch.tensor(rows, device=DEV)
        sub = proj[idx].contiguous()
        row_req = ints(r for r in range(len(who)) for _ in range(spans[r + 1] - spans[r]))
        qkv = torch.empty(len(rows), channels, device=DEV)
        bg = torch.empty(len(rows), 2 * heads + groups, device=DEV)
        o.gdn_prepare(sub, extra, extra + channels, extra + channels + heads, groups, heads, dim, vdim, taps, conv,
                      a_log, dt_bias, state, conv_off, row_req, ints(spans), ints(who), qkv, bg)
        got = torch.empty(len(rows), heads * vdim, device=DEV)
        # asked to, heads of 65 to 128 lanes take the chunk form of the rule where a request brings 32 rows and more
        o.gdn_scan(qkv, bg, groups, heads, dim, vdim, state, ints(spans), ints(who), got,
                   longest=max(b - a for a, b in zip(spans, spans[1:])), chunks=chunks)
        out[idx] = got

    run_in_portions(lengths, cuts, slots, step)
    starts = np.concatenate(([0], np.cumsum(lengths)))
    for r, n in enumerate(lengths):
        rows = slice(starts[r], starts[r + 1])
        q, k, v, beta, decay = plain_prepared(proj[rows], conv, a_log, dt_bias, groups, heads, dim, vdim)
        for h in range(heads):
            g = h // (heads // groups)
            want, last = plain.gated_delta_rule(q[:, g], k[:, g], v[:, h], beta[:, h], decay[:, h])
            close(out[rows, h * vdim:(h + 1) * vdim], want, torch.float32, f"request {r} head {h}")
            kept = state[slots[r], :conv_off].view(heads, vdim, padded)[h, :, :dim].t()
            close(kept, last, torch.float32, f"the matrix of request {r} head {h}")
            assert float(state[slots[r], :conv_off].view(heads, vdim, padded)[h, :, dim:].abs().max() if padded > dim else 0) == 0
    assert torch.all(state[1] == 7.0) and torch.all(state[4] == 0.0)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("groups,heads,dim,vdim,taps", [(2, 4, 16, 64, 4), (1, 2, 128, 128, 4), (3, 3, 64, 32, 2),
                                                         (1, 1, 40, 96, 1), (2, 2, 260, 8, 3)])
def test_a_step_of_single_tokens_in_one_kernel(groups, heads, dim, vdim, taps, out_dtype):
    """Token by token through `gdn_step` (three requests, one of them absent from some steps, an idle row of a
    padded step) against the kernels for portions fed the same rows: outputs, matrices and kept inputs."""
    o = ops()
    assert o.gdn_step_supported(dim, vdim)
    steps, extra = 7, 5
    channels = 2 * groups * dim + heads * vdim
    padded = o.gdn_padded_dim(dim)
    conv_off = heads * vdim * padded
    floats = -(-(conv_off + (taps - 1) * channels) // 4) * 4
    conv = rnd(channels, taps, seed=71, scale=0.7)
    a_log, dt_bias, gain = rnd(heads, seed=72, scale=0.5), rnd(heads, seed=73, scale=0.5) - 1.0, rnd(vdim, seed=74) + 1.0
    one, many = torch.zeros(4, floats, device=DEV), torch.zeros(4, floats, device=DEV)
    width = extra + channels + 2 * heads + heads * vdim
    for step in range(steps):
        present = [0, 1, 2] if step % 3 else [0, 2]
        slots = [3, 0, 1]
        n = len(present) + 1                                                    # the last row is idle
        proj = rnd(n, width, seed=80 + step, scale=1.5)
        row_req, spans = ints(list(range(len(present))) + [-1]), ints(list(range(len(present) + 1)) + [len(present)])
        who = ints([slots[r] for r in present] + [0])
        got = torch.full((n, heads * vdim), float("nan"), dtype=out_dtype, device=DEV)
        o.gdn_step(proj, extra, extra + channels, extra + channels + heads, extra + channels + 2 * heads, groups, heads,
                   dim, vdim, taps, conv, a_log, dt_bias, gain, 1.3, 1e-5, one, conv_off, row_req, spans, who, got)
        qkv, bg = torch.empty(n, channels, device=DEV), torch.empty(n, 2 * heads + groups, device=DEV)
        o.gdn_prepare(proj, extra, extra + channels, extra + channels + heads, groups, heads, dim, vdim, taps, conv, a_log,
                      dt_bias, many, conv_off, row_req, spans, who, qkv, bg)
        raw = torch.zeros(n, heads * vdim, device=DEV)
        o.gdn_scan(qkv, bg, groups, heads, dim, vdim, many, spans, who, raw)
        want = torch.empty(n, heads * vdim, dtype=out_dtype, device=DEV)
        o.gdn_out_norm(raw, proj, extra + channels + 2 * heads, gain, 1.3, 1e-5, want, heads, vdim, row_req)
        close(got[:-1], want[:-1], out_dtype, f"step {step}")
        assert torch.isnan(got[-1].float()).all()
    close(one, many, torch.float32, "matrices and kept inputs")
    assert float(one[3].abs().max()) > 0 and float(one[2].abs().max()) == 0


@pytest.mark.parametrize("dim,chunks", [(32, False), (128, False), (128, True)])
def test_a_token_written_far_back_is_read_from_the_matrix(dim, chunks):
    """Without decay and with keys at right angles, what token 3 wrote along its key comes back whole when
    token 900 asks along the same key; a matrix that lost it on the way (a portion's edge) gives zeros."""
    o = ops()
    vdim, total = 16, 901
    qkv = torch.zeros(total, 2 * dim + vdim, device=DEV)
    bg = torch.ones(total, 3, device=DEV)                  # beta 1, decay 1, and q . k (set below)
    for t in range(total):
        qkv[t, dim + 1 + t % (dim - 1)] = 1.0              # keys e1 .. e31 in turn
        qkv[t, t % dim] = 1.0
    marker = torch.arange(1, vdim + 1, device=DEV).float()
    qkv[3, dim:2 * dim] = 0.0
    qkv[3, dim] = 1.0                                      # token 3 alone writes along e0
    qkv[3, 2 * dim:] = marker
    qkv[900, :dim] = 0.0
    qkv[900, 0] = 1.0                                      # token 900 reads along e0
    bg[:, 2] = (qkv[:, :dim] * qkv[:, dim:2 * dim]).sum(dim=1)
    state = torch.zeros(2, vdim * o.gdn_padded_dim(dim), device=DEV)
    out = torch.empty(total, vdim, device=DEV)
    at = 0
    for n in (2, 2, 500, 1, 396):                           # the write and the read lie in different steps
        o.gdn_scan(qkv[at:at + n].contiguous(), bg[at:at + n].contiguous(), 1, 1, dim, vdim, state,
                   ints([0, n]), ints([1]), out[at:at + n], longest=n, chunks=chunks)
        at += n
    assert torch.allclose(out[900], marker, atol=1e-5)


# ---- queries, keys and values of unlike head sizes ---------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim,rot", [(6, 2, 64, 128, 16), (3, 3, 10, 20, 0), (4, 1, 32, 16, 32), (2, 2, 24, 24, 6)])
def test_bias_rotation_and_the_cache_write_with_padded_rows(heads, kv, dim, vdim, rot, dtype):
    o = ops()
    n, extra, row = 9, 8, -(-max(dim, vdim) // 16) * 16
    width = heads * dim + kv * (dim + vdim)
    proj = rnd(n, extra + width + 3, seed=40)
    bias = rnd(width, seed=41)
    pos = [0, 1, 5, 1116, 70000, 3, 2, 1, 0]
    freq = torch.tensor([777.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64).float().to(DEV) if rot else None
    slots = [4, 9, 2, 7, 0, 11, 3, 8, 1]
    q = torch.full((n, heads * row), float("nan"), dtype=dtype, device=DEV)
    k_pool = torch.full((12, kv, row), float("nan"), dtype=dtype, device=DEV)
    v_pool = torch.full((12, kv, row), float("nan"), dtype=dtype, device=DEV)
    req = [0, 0, 0, 1, 2, -1, 3, 3, 3]                      # row 5 is an idle row of a padded step
    o.qkv_rotate_store(proj, extra, bias, freq, rot, ints(pos), ints(slots), ints(req), q, k_pool, v_pool, heads, kv,
                       dim, vdim, row)
    p = proj.double().cpu()[:, extra:extra + width] + bias.double().cpu()
    positions = torch.tensor(pos)
    want_q, want_k = p[:, :heads * dim].view(n, heads, dim), p[:, heads * dim:(heads + kv) * dim].view(n, kv, dim)
    if rot:
        want_q = plain.rotate_interleaved(want_q, positions, 777.0, rot)
        want_k = plain.rotate_interleaved(want_k, positions, 777.0, rot)
    want_v = p[:, (heads + kv) * dim:].view(n, kv, vdim)
    live = [t for t in range(n) if req[t] >= 0]
    tol = torch.float32 if dtype == torch.float32 else torch.bfloat16
    # float32 sines of angles up to 70,000 radians differ from float64 ones by the angle's own rounding
    loose = 1e-2 if rot else 0.0
    got_q = q.view(n, heads, row).float().cpu()
    assert float((got_q[live][:, :, :dim] - want_q[live].float()).abs().max()) <= (3e-2 if dtype == torch.bfloat16 else 1e-5 + loose)
    assert float(got_q[live][:, :, dim:].abs().max() if row > dim else 0) == 0
    for t in live:
        got_k, got_v = k_pool[slots[t]].float().cpu(), v_pool[slots[t]].float().cpu()
        assert float((got_k[:, :dim] - want_k[t].float()).abs().max()) <= (3e-2 if dtype == torch.bfloat16 else 1e-5 + loose)
        close(got_v[:, :vdim], want_v[t], tol, "values")
        assert float(got_k[:, dim:].abs().max() if row > dim else 0) == 0 and float(got_v[:, vdim:].abs().max() if row > vdim else 0) == 0
    assert torch.isnan(k_pool[slots[5]].float()).all() and torch.isnan(q[5].float()).all()


def paged(lengths, kv, row, page, dtype, seed):
    """Keys and values scattered over shuffled pages: pools, tables and the dense rows."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-n // page) for n in lengths) + 2
    order = torch.randperm(n_pages, generator=g).tolist()
    k_pool = torch.full((n_pages * page, kv, row), float("nan"), dtype=dtype)
    v_pool = torch.full((n_pages * page, kv, row), float("nan"), dtype=dtype)
    tables = torch.full((len(lengths), max(-(-n // page) for n in lengths) + 1), -1, dtype=torch.int32)
    dense = []
    for r, n in enumerate(lengths):
        k, v = torch.randn(n, kv, row, generator=g).to(dtype), torch.randn(n, kv, row, generator=g).to(dtype)
        dense.append([k, v])
    return k_pool, v_pool, tables, dense, order


def scatter(k_pool, v_pool, tables, dense, order, page):
    for r, (k, v) in enumerate(dense):
        n = k.shape[0]
        for b in range(-(-n // page)):
            pg = order.pop()
            tables[r, b] = pg
            rows = slice(b * page, min(n, (b + 1) * page))
            k_pool[pg * page:pg * page + rows.stop - rows.start] = k[rows]
            v_pool[pg * page:pg * page + rows.stop - rows.start] = v[rows]


def chunked_reference(q, dense, row_req, pos, heads, kv, chunk, scale):
    out = torch.zeros_like(q)
    for t in range(q.shape[0]):
        k, v = dense[row_req[t]]
        lo = pos[t] - pos[t] % chunk if chunk else 0
        for h in range(heads):
            g = h // (heads // kv)
            s = (k[lo:pos[t] + 1, g].double() @ q[t, h].double()) * scale
            out[t, h] = (torch.softmax(s, dim=0) @ v[lo:pos[t] + 1, g].double()).float()
    return out


@pytest.mark.parametrize("kernel,dtype,heads,kv,row,chunk", [
    ("generic", torch.float32, 3, 3, 48, 160), ("generic", torch.bfloat16, 4, 2, 144, 37), ("generic", torch.float32, 2, 1, 32, 1),
    ("decode", torch.bfloat16, 4, 2, 32, 160), ("decode", torch.bfloat16, 16, 1, 64, 37), ("decode", torch.bfloat16, 2, 2, 128, 256),
    ("tiles", torch.bfloat16, 3, 3, 48, 37), ("tiles", torch.bfloat16, 4, 2, 80, 160), ("tiles", torch.bfloat16, 2, 2, 16, 1),
    ("wide", torch.bfloat16, 4, 2, 128, 160), ("wide", torch.bfloat16, 6, 3, 128, 37), ("wide", torch.bfloat16, 2, 1, 64, 128)])
def test_keys_are_seen_inside_the_querys_own_chunk_in_every_attention_kernel(kernel, dtype, heads, kv, row, chunk):
    """The last key before every query's chunk and the first key inside it get a score that stands out
    (the query itself, scaled) and values of their own: one must be missing from the output, the other
    must dominate it.  Requests end right behind, on and before a chunk's edge."""
    from tokenizer_b200.parts.attention import RowTiles
    o = ops()
    page = 16
    lengths = [3 * chunk + 2, 2 * chunk + 1, 1, 4 * chunk] if chunk > 1 else [70, 33, 1, 16]
    k_pool, v_pool, tables, dense, order = paged(lengths, kv, row, page, dtype, seed=50)
    scale = 1.0 / math.sqrt(row)
    if kernel == "decode":
        row_req, pos, spans = [0, 1, 2, 3], [n - 1 for n in lengths], None
    else:
        take = [min(n, 130) for n in lengths]
        spans = [(r, n - m, m) for r, (n, m) in enumerate(zip(lengths, take))]
        row_req = [r for r, _, m in spans for _ in range(m)]
        pos = [first + i for _, first, m in spans for i in range(m)]
    q = rnd(len(pos), heads, row, seed=51, dtype=dtype, scale=1.0).cpu()
    # for the last row of every request: its own query direction planted, large, in the key just
    # outside its chunk and, half as large, in the first key inside
    for t in range(len(pos)):
        if t + 1 < len(pos) and row_req[t + 1] == row_req[t]:
            continue
        start = pos[t] - pos[t] % chunk
        k, v = dense[row_req[t]]
        g = 0
        direction = q[t, 0].float() / q[t, 0].float().norm()
        if start > 0:
            k[start - 1, g] = (direction * 40.0).to(dtype)
            v[start - 1, g] = 50.0
        if start < pos[t]:
            k[start, g] = (direction * 20.0).to(dtype)
            v[start, g] = -9.0
    scatter(k_pool, v_pool, tables, dense, order, page)
    k_pool, v_pool, tables = k_pool.to(DEV), v_pool.to(DEV), tables.to(DEV)
    qd = q.to(DEV)
    out = torch.full((len(pos), heads * row), float("nan"), dtype=dtype, device=DEV)
    args = (qd.view(len(pos), -1), k_pool, v_pool, out, tables, ints(row_req), ints(pos))
    if kernel == "generic":
        o.paged_attention_generic(*args, heads, kv, row, page, None, scale, chunk=chunk)
    elif kernel == "decode":
        o.decode_attention(*args, heads, kv, row, page, None, scale, chunk=chunk)
    else:
        note = RowTiles(o.WIDE_TILE_ROWS if kernel == "wide" else o.PREFILL_TILE_ROWS)
        words = np.zeros(note.capacity(len(pos), len(spans)), dtype=np.int32)
        counts = np.array([m for _, _, m in spans], dtype=np.int32)
        firsts = np.concatenate(([0], np.cumsum(counts)[:-1])).astype(np.int32)
        n_tiles = note.fill(words, firsts, counts, np.array([f for _, f, _ in spans], dtype=np.int32), False)
        tiles = torch.tensor(words, device=DEV).view(-1, 2)
        run = o.attention_tcgen05 if kernel == "wide" else o.prefill_attention
        run(*args, tiles, n_tiles, heads, kv, row, page, None, scale, chunk=chunk)
    want = chunked_reference(q.float(), dense, row_req, pos, heads, kv, chunk, scale)
    got = out.view(len(pos), heads, row).float().cpu()
    assert torch.isfinite(got).all()
    bound = 2e-5 if dtype == torch.float32 else 3e-2
    assert float((got - want).abs().max()) <= bound * max(1.0, float(want.abs().max()))
    # the edge matters: seeing the key just outside would pull head 0 of those rows to its value
    unchunked = chunked_reference(q.float(), dense, row_req, pos, heads, kv, 0, scale)
    assert chunk == 1 or float((unchunked - want).abs().max()) > 5.0


# ---- routed experts ------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,shared", [(8, 3, True), (3, 3, True), (6, 1, False), (70, 5, True)])
def test_routing_shares_and_the_gate_of_all_experts_lanes(experts, top, shared, dtype):
    o = ops()
    n, hidden, ff, sff = 37, 50, 6, 10
    h = rnd(n, hidden, seed=60, dtype=dtype)
    w = rnd(experts + int(shared), hidden, seed=61, scale=0.7)
    share = torch.full((n, experts + int(shared)), float("nan"), device=DEV)
    o.moe_route(h, w, experts, top, shared, share)
    z = h.double().cpu() @ w.double().cpu().t()
    want = torch.zeros(n, experts + int(shared), dtype=torch.float64)
    for t in range(n):
        chosen = torch.topk(z[t, :experts], top).indices
        want[t, chosen] = torch.softmax(z[t, chosen], dim=0)
        if shared:
            want[t, experts] = plain.sigmoid(z[t, experts])
    close(share, want, torch.float32, "shares")
    assert int((share[:, :experts] > 0).sum()) == n * top
    inner = experts * ff + (sff if shared else 0)
    gu = rnd(n, 2 * inner, seed=62, dtype=dtype)
    act = torch.empty(n, inner, dtype=dtype, device=DEV)
    o.moe_gate(gu, share, act, experts, ff, shared)
    lane_expert = torch.tensor([c // ff if c < experts * ff else experts for c in range(inner)])
    g = gu.double().cpu()
    close(act, plain.silu(g[:, :inner]) * g[:, inner:] * want[:, lane_expert], dtype, "gated lanes")


# ---- whole models -----------------------------------------------------------------------------------
LENGTHS = {"a": [1, 2, 23, 100, 131, 49], "b": [5, 19, 97, 201, 260, 100], "c": [3, 40, 130, 64, 1, 90],
           "d": [4, 31, 77, 150, 9, 60]}


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


def compare(got, want, dtype, what):
    """float32: every logit within 1e-4.  bfloat16: per position, the root mean square of the difference
    (its mean over the vocabulary taken off) against that of the logits themselves.  These tiny models
    norm the output of every sublayer, some of them of a handful of lanes, which carries the operands'
    rounding (2^-9 each) to the logits at about one part in a hundred and in a few positions several
    times that; a key, a state or an expert that is wrong moves a position's logits by their own size."""
    if dtype == "float32":
        return ru.compare(got, want, dtype, what)
    rel, where = [], []
    for name in sorted(got):
        for position in sorted(got[name]):
            row, ref = got[name][position], want[name][position]
            assert np.isfinite(row).all(), f"{what}: {name}[{position}] not finite"
            d, c = row - ref, ref - ref.mean()
            rel.append(float(np.sqrt(((d - d.mean()) ** 2).mean()) / np.sqrt((c ** 2).mean())))
            where.append((name, position))
    rel = np.array(rel)
    worst = int(rel.argmax())
    assert rel[worst] <= 0.25, f"{what} (bfloat16): request {where[worst][0]!r} position {where[worst][1]}: {rel[worst]:.3f}"
    assert np.percentile(rel, 90) <= 0.06, f"{what} (bfloat16): a tenth of the positions is off by {np.percentile(rel, 90):.3f} and more"


def test_every_layer_leaves_the_stream_the_plain_layers_leave(model):
    """The residual stream after every call of the order (a looped layer counts each time), float32."""
    from tokenizer_b200.engine import Engine, StepEntry
    folder, cfg, page, requests, _ = model
    ids = max(requests.values(), key=len)
    raw, w = plain.load_folder(folder)
    want = []
    plain.forward(raw, w, ids, keep=want)
    engine = Engine.from_folder(folder, dtype="float32", num_pages=-(-len(ids) // page) + 1, page_size=page,
                                max_requests=1, use_graphs=False)
    got = []
    for block in set(engine.model.blocks):
        def run(stream, ctx, cache, inner=block.forward):
            inner(stream, ctx, cache)
            got.append(stream.flush().clone())
        block.forward = run
    cache = engine.cache.open("r")
    engine.cache.reserve(cache, len(ids))
    engine.step([StepEntry(cache, ids, [0])])
    assert len(got) == len(want) == len(engine.model.order)
    for at, (a, b) in enumerate(zip(got, want)):
        # scores of the sharpened attention reach a few dozen, where float32 resolves 1e-5 of a softmax weight
        err, size = float((a.cpu() - b.float()).abs().max()), float(b.abs().max())
        assert err <= 1e-4 * max(1.0, size), f"the stream after call {at} (layer {engine.model.order[at].layer}): {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts(model, dtype):
    folder, cfg, page, requests, want = model
    steps = ru.steps_whole(requests)
    budget = max(ru.rounded64(len(v)) for v in requests.values())
    got = ru.collect(steps, replay(folder, dtype, steps, budget, page))
    assert {k: len(v) for k, v in got.items()} == {k: len(v) for k, v in requests.items()}
    compare(got, want, dtype, "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_then_token_by_token(model, dtype):
    """The last 40 tokens one by one: more than the chunks of 1 and 24 positions, so that a chunk's edge
    passes under decoded tokens, and matrices and kept inputs are carried through every step."""
    folder, cfg, page, requests, want = model
    steps = ru.steps_decode_tail(requests, 40)
    budget = max(ru.rounded64(len(v)) for v in requests.values())
    got = ru.collect(steps, replay(folder, dtype, steps, budget, page))
    compare(got, want, dtype, "decode tail")


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
    compare(got, want, dtype, f"portions {sizes}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("live", [4, 2])
def test_mixed_batches_on_pages_and_slots_that_are_used_again(model, dtype, live):
    folder, cfg, page, requests, want = model
    steps, peak = ru.steps_mixed(requests, max_live=live, seed=live)
    assert peak < sum(ru.rounded64(len(v)) for v in requests.values()) and len(requests) > live
    got = ru.collect(steps, replay(folder, dtype, steps, peak, page, max_requests=live))
    assert {k: len(v) for k, v in got.items()} == {k: len(v) for k, v in requests.items()}
    compare(got, want, dtype, "mixed")


def test_experts_chosen_token_by_token(tmp_path_factory):
    """With the router left as drawn, which experts a token uses changes from token to token (the other
    whole-model runs pin the choice, see `settle_routing`); in float32 a near tie is out of reach of rounding."""
    for name in ("a", "b"):
        folder, cfg, page = make_folder(tmp_path_factory, name, scale=dict(SHARPEN, **{r"\.router$": 20.0}), settled=False)
        requests = {f"r{i}": random_ids(n, cfg.vocab, 900 + i) for i, n in enumerate([70, 9, 131, 30, 2])}
        want = reference_logits(folder, requests)
        steps, peak = ru.steps_mixed(requests, max_live=3, seed=2)
        got = ru.collect(steps, replay(folder, "float32", steps, peak, page, max_requests=3))
        ru.compare(got, want, "float32", "experts chosen by the token")


def test_steps_launched_anew_agree_with_replayed_ones(model):
    folder, cfg, page, requests, want = model
    steps, peak = ru.steps_mixed(requests, max_live=3, seed=5)
    got = ru.collect(steps, replay(folder, "float32", steps, peak, page, max_requests=3, use_graphs=False))
    ru.compare(got, want, "float32", "without graphs")


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
    slack = 1e-4 if dtype == "float32" else 0.1 * float(logits.abs().max())
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
        near_best(raw, w, prompt, out.tokens, dtype)


def test_a_batch_through_the_scheduler_with_preemption_gives_each_request_its_own_ids(model):
    """Five prompts on a pool that cannot hold them all: requests are preempted and computed again,
    which for a recurrence means matrices and kept inputs that start from zero again."""
    import tokenizer_b200 as tb
    folder, cfg, page, requests, _ = model
    raw, w = plain.load_folder(folder)
    engine_model = tb.load_model(folder, dtype="float32")
    prompts = [random_ids(n, cfg.vocab, 600 + n) for n in (30, 7, 55, 18, 41)]
    engine = tb.engine_for(engine_model, 192, page_size=page, max_requests=3, share_prefixes=False)
    results = tb.generate_batch(engine, prompts, tb.GenerateParams.greedy(20), max_batch_size=3, token_budget=48,
                                page_size=page)
    for prompt, result in zip(prompts, results):
        near_best(raw, w, prompt, result.tokens, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_on_the_device(model, dtype):
    """300 greedy steps without a visit to the host between them (captured and replayed): chunk edges
    pass under decoded tokens, pages behind them are given back, the states move on."""
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
        near_best(raw, w, prompt, [first[i]] + [step[i] for step in history], dtype)


def test_the_command_line_generates_from_a_configuration_of_this_design(tmp_path):
    """`--random-weights config.json` draws the weights the configuration declares; two prompts go
    through the scheduler and print ids that the plain implementation ranks best."""
    import json
    import os
    import subprocess
    import sys
    import tokenizer_b200 as tb
    cfg, seed, page = TINY["a"]()
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
    lines = proc.stdout.strip().splitlines()
    assert len(lines) == 2
    for prompt, line in zip(prompts, lines):
        near_best(raw, w, prompt, [int(t) for t in line.split()], "float32")
