"""The Lizizen design in the engine against the plain implementation in ``plain_lizizen``.

First each mechanism's kernels alone (the two norms with the token shift and its state row, the
clamped gated activation, the changed scores of the attention kernels in every kernel family:
distance bias, a factor per query position, a term of score 0 in the denominator, capped
scores, a chunked mask; the two ends of differential attention), then whole models through trace
replay: whole prompts, the last tokens decoded one by one, portions down to two tokens, mixed
batches in a pool so small that pages and slots are used again, long decoding, the first tokens,
keys far away, at page borders and just inside and just outside a chunk, a sink that matters,
and greedy generation through the engine's entry point and scheduler.
"""
import math

import numpy as np
import pytest
import torch

import lizizen_configs as lc
import plain_lizizen as plain
from helpers import check_logits as _check_logits, random_prompts

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def check_logits(got, want, dtype, what):
    _check_logits(got, torch.from_numpy(np.asarray(want)), dtype, what, bf16_tolerance=6e-2, bf16_min_cosine=0.997)


def close(got, want, dtype, what, scale=None):
    got = got.double().cpu()
    want = torch.as_tensor(np.asarray(want)).double()
    scale = float(want.abs().max()) if scale is None else scale
    tol = (4e-6 if dtype == "float32" else 1.2e-2) * max(scale, 1e-6)
    err = float((got - want).abs().max())
    assert err <= tol, f"{what} ({dtype}): max error {err:.3e}, allowed {tol:.3e}"


def step_arrays(lengths, slots):
    starts = np.concatenate([[0], np.cumsum(lengths)[:-1]]).astype(np.int32)
    as_dev = lambda a: torch.tensor(np.asarray(a, dtype=np.int32)).cuda()
    return as_dev(starts), as_dev(lengths), as_dev(slots)


# ------------------------------------------------------------------------------------ kernels
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("width,two", [(64, True), (100, True), (250, False), (1536, True)])
def test_norms_and_token_shift_in_portions(dtype, width, two):
    """Two sequences cut into portions (single tokens among them) beside each other: the first
    output is the shifted norm of the whole sequences, the second the other norm of the same
    rows, and a slot's state row is the last normed row."""
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(width)
    eps = 1e-5
    seqs = [3.0 * torch.randn(23, width, generator=gen), torch.randn(9, width, generator=gen)]
    w1, w2 = 1 + 0.3 * torch.randn(width, generator=gen), 1 + 0.3 * torch.randn(width, generator=gen)
    shift = torch.rand(width, generator=gen)
    normed = [plain.rms_unit(s.double().numpy(), eps) * w1.double().numpy() for s in seqs]
    want1 = [plain.token_shift(h, shift.double().numpy()) for h in normed]
    want2 = [plain.rms_unit(s.double().numpy(), eps) * w2.double().numpy() for s in seqs]
    state = torch.zeros(4, width + 3).cuda()
    state[0].fill_(7.0)
    state[3].fill_(-7.0)
    done = [0, 0]
    got1 = [np.zeros((23, width)), np.zeros((9, width))]
    got2 = [np.zeros((23, width)), np.zeros((9, width))]
    for cuts in ([5, 3], [1, 1], [2, 2], [15, 3]):
        T = sum(cuts)
        x = torch.cat([seqs[s][done[s] : done[s] + n] for s, n in enumerate(cuts)]).cuda()
        out1 = torch.zeros(T, width, dtype=dt).cuda()
        out2 = torch.zeros(T, width, dtype=dt).cuda()
        q_start, q_len, slots = step_arrays(cuts, [2, 1])
        kernels.norm_shift(x, w1.cuda(), eps, out1, T, q_start, q_len, slots, 2, weight2=w2.cuda() if two else None,
                           out2=out2 if two else None, shift=shift.cuda(), state=state[:, :width])
        row = 0
        for s, n in enumerate(cuts):
            got1[s][done[s] : done[s] + n] = out1[row : row + n].float().cpu().numpy()
            got2[s][done[s] : done[s] + n] = out2[row : row + n].float().cpu().numpy()
            done[s] += n
            row += n
    for s in range(2):
        close(torch.from_numpy(got1[s]), want1[s], dtype, f"shifted norm of sequence {s}")
        if two:
            close(torch.from_numpy(got2[s]), want2[s], dtype, f"second norm of sequence {s}")
    close(state[2, :width], normed[0][-1], "float32", "state of slot 2", scale=float(np.abs(normed[0]).max()))
    close(state[1, :width], normed[1][-1], "float32", "state of slot 1", scale=float(np.abs(normed[1]).max()))
    assert torch.all(state[0] == 7.0) and torch.all(state[3] == -7.0) and torch.all(state[1:3, width:] == 0)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("T,F,limit", [(1, 128, 1.5), (17, 40, 0.7), (5, 8, 0.0), (300, 1000, 2.0)])
def test_clamped_gated_activation(dtype, T, F, limit):
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(F)
    gate_up = (2.0 * torch.randn(T, 2 * F, generator=gen)).to(dt)
    g, u = gate_up[:, :F].double().numpy(), gate_up[:, F:].double().numpy()
    if limit:
        g, u = np.minimum(g, limit), np.clip(u, -limit, limit)
    want = g * plain.sigmoid(1.702 * g) * (u + 1.0)
    out = torch.zeros(T, F, dtype=dt).cuda()
    kernels.clamped_glu(gate_up.cuda(), out, T, F, limit, 1.702, 1.0)
    close(out, want, dtype, "activation")


@pytest.mark.parametrize("T,F,K,limit,biased", [(1, 128, 64, 1.5, True), (17, 40, 104, 0.7, True), (8, 8960, 1536, 7.0, True),
                                                (200, 1000, 256, 0.0, False), (64, 72, 896, 2.0, False)])
def test_gated_activation_in_the_projection(T, F, K, limit, biased):
    """The same activation in the epilogue of the tensor-core projection of small steps: gate and
    up rows of one matrix, their biases, clamps, the slope of the sigmoid and the shift of up."""
    from velox_b200.ops import kernels

    gen = torch.Generator().manual_seed(F + K)
    x = torch.randn(T + 2, K, generator=gen).to(torch.bfloat16)
    w = (1.5 * torch.randn(2 * F, K, generator=gen) / math.sqrt(K)).to(torch.bfloat16)
    b = torch.randn(2 * F, generator=gen) if biased else None
    y = x[:T].double() @ w.double().T + (b.double() if biased else 0.0)
    g, u = y[:, :F].numpy(), y[:, F:].numpy()
    if limit:
        g, u = np.minimum(g, limit), np.clip(u, -limit, limit)
    want = g * plain.sigmoid(1.702 * g) * (u + 1.0)
    out = torch.full((T + 2, F), 9.0, dtype=torch.bfloat16).cuda()
    status = torch.zeros(1, dtype=torch.int32).cuda()
    kernels.gemm_bf16_glu(x.cuda(), w.cuda(), b.cuda() if biased else None, out, T, limit, 1.702, 1.0, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    close(out[:T], want, "bfloat16", "activation in the projection")
    assert torch.all(out[T:] == 9.0)


def plain_changed_attention(q, k_all, v_all, ctx, scale, temp=None, bias=None, sink=False, cap=None, chunk=None):
    """q [n, H, D] at positions ctx .. ctx + n - 1 over keys/values [ctx + n, G, D] (float64 numpy)."""
    n, H, _ = q.shape
    total, G = k_all.shape[0], k_all.shape[1]
    visible = plain.causal(total)[ctx:]
    if chunk:
        visible = visible & plain.same_chunk(total, chunk)[ctx:]
    out = np.zeros((n, H, v_all.shape[2]))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k_all[:, g].T) * scale
        if temp is not None:
            s = s * plain.query_temperature(np.arange(ctx, total, dtype=np.float64), *temp)[:, None]
        if cap:
            s = plain.softcap(s, cap)
        if bias is not None:
            s = s - plain.distance_bias(bias[0][head], bias[1][head], total)[ctx:]
        p = plain.softmax_with_zero_sink(s, visible) if sink else plain.softmax(s, visible)
        out[:, head] = p @ v_all[:, g]
    return out


def run_changed_attention(dtype, H, G, D, P, seqs, seed, temp=None, bias=False, sink=False, cap=None, chunk=None,
                          min_split_keys=256, max_cluster=1, target_ctas=296, tensor_memory=False, fixed_splits=None):
    from velox_b200.ops import attention_plan as ap
    from velox_b200.ops import kernels as k

    gen = torch.Generator().manual_seed(seed)
    total_pages = sum(-(-(q + c) // P) for q, c in seqs) + 3
    order = (torch.randperm(total_pages - 1, generator=gen) + 1).tolist()
    k_cache = torch.randn(total_pages, P, G, D, generator=gen).to(dtype)
    v_cache = torch.randn(total_pages, P, G, D, generator=gen).to(dtype)
    T = sum(q for q, _ in seqs)
    scale = 1.3 / math.sqrt(D)
    qbuf = torch.randn(T, H * D, generator=gen).to(dtype)
    longest = max(q + c for q, c in seqs)
    width = max(-(-(q + c) // P) for q, c in seqs)
    tables = torch.zeros(len(seqs), width, dtype=torch.int32)
    r1 = 2.0 * torch.rand(H, generator=gen)
    r2 = 0.05 + 0.45 * torch.rand(H, generator=gen)
    pair = (r1.double().numpy(), r2.double().numpy()) if bias else None
    table = None
    if temp is not None:
        table = torch.from_numpy(plain.query_temperature(np.arange(longest, dtype=np.float64), *temp)).float().cuda()
    q_start, q_lens, kv_lens = [], [], []
    want = np.zeros((T, H, D))
    row = 0
    for s, (q_len, ctx) in enumerate(seqs):
        kv_len = q_len + ctx
        pages = [order.pop() for _ in range(-(-kv_len // P))]
        tables[s, : len(pages)] = torch.tensor(pages, dtype=torch.int32)
        slots = [pages[i // P] * P + i % P for i in range(kv_len)]
        k_all = k_cache.view(-1, G, D)[slots].double().numpy()
        v_all = v_cache.view(-1, G, D)[slots].double().numpy()
        q = qbuf[row : row + q_len].view(q_len, H, D).double().numpy()
        want[row : row + q_len] = plain_changed_attention(q, k_all, v_all, ctx, scale, temp, pair, sink, cap, chunk)
        q_start.append(row)
        q_lens.append(q_len)
        kv_lens.append(kv_len)
        row += q_len
    plan = ap.plan_attention(
        q_lens, kv_lens,
        ap.PlanOptions(num_kv_heads=G, group=H // G, window=None, use_f32=dtype == torch.float32,
                       min_split_keys=min_split_keys, target_ctas=target_ctas, narrow_max_cluster=max_cluster,
                       narrow_global_split_keys=min_split_keys, wide_on_tensor_memory=tensor_memory, chunk=chunk or 0),
        fixed_splits=fixed_splits)
    dev = lambda x: torch.as_tensor(x, dtype=torch.int32).cuda()
    out = torch.zeros(T, H * D, dtype=dtype, device="cuda")
    partial_o = torch.zeros(max(plan.partial_rows, 1) * D, device="cuda")
    partial_lse = torch.zeros(max(plan.partial_rows, 1), device="cuda")
    for kind, items in plan.items.items():
        k.attention(kind, qbuf.cuda(), out, k_cache.cuda(), v_cache.cuda(), tables.cuda(), dev(q_start), dev(q_lens),
                    dev(kv_lens), dev(items), len(items), partial_o, partial_lse, H, G, D, None, scale,
                    cluster=plan.cluster if kind == ap.KIND_BF16_NARROW else 1, softcap=cap or 0.0,
                    distance_bias=(r1.cuda(), r2.cuda()) if bias else None, chunk=chunk or 0, sink_zero=sink,
                    row_scale=table)
    if len(plan.merge_items):
        k.attention_merge(out, dev(q_start), dev(plan.merge_items), len(plan.merge_items), partial_o, partial_lse,
                          H, G, D, max_rows=max(ap.TILE_ROWS[kind] for kind in plan.items))
    torch.cuda.synchronize()
    return out.view(T, H, D).double().cpu().numpy(), want, plan


MIXED = [(70, 0), (1, 0), (1, 130), (2, 61), (33, 100), (1, 63), (1, 64), (17, 15)]


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("H,G,D,P", [(4, 2, 16, 4), (5, 5, 48, 16), (6, 2, 80, 16), (12, 2, 128, 16), (32, 1, 64, 16),
                                     (3, 1, 112, 16), (2, 2, 192, 8)])
def test_attention_with_bias_temperature_and_zero_sink(dtype, H, G, D, P):
    """Whole prompts, portions with context, single decoded tokens, a first token and a portion
    of two tokens: distance bias, a factor per query position and the term of score 0."""
    got, want, _ = run_changed_attention(DTYPES[dtype], H, G, D, P, MIXED, seed=H + D, temp=(0.5, 7), bias=True,
                                         sink=True)
    # the first token of a sequence gives half its weight to the sink
    tol = 2e-5 if dtype == "float32" else 2.5e-2
    assert np.abs(got - want).max() <= tol * np.abs(want).max()
    without, _, _ = run_changed_attention(DTYPES[dtype], H, G, D, P, MIXED, seed=H + D, temp=(0.5, 7), bias=True)
    assert np.abs(without - want).max() > 0.1 * np.abs(want).max(), "the sink does not matter enough for this test"


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("H,G,D,P", [(4, 2, 16, 4), (6, 3, 32, 8), (8, 2, 96, 16), (4, 1, 256, 32)])
@pytest.mark.parametrize("chunk,cap", [(1, None), (7, 2.0), (64, None), (150, 5.0), (None, 1.0)])
def test_attention_with_chunks_and_capped_scores(dtype, H, G, D, P, chunk, cap):
    got, want, _ = run_changed_attention(DTYPES[dtype], H, G, D, P, MIXED + [(40, 140), (1, 149), (1, 150), (3, 299)],
                                         seed=D + (chunk or 0), cap=cap, chunk=chunk)
    tol = 2e-5 if dtype == "float32" else 2.5e-2
    assert np.abs(got - want).max() <= tol * np.abs(want).max()


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("max_cluster", [1, 4])
def test_changed_scores_with_split_key_ranges(dtype, max_cluster):
    """Long contexts whose keys are dealt out to several work items (and to the CTAs of a
    cluster): the term of score 0 enters every row once, biases use absolute positions."""
    seqs = [(1, 1999), (1, 700), (5, 1200), (130, 900)]
    got, want, plan = run_changed_attention(DTYPES[dtype], 8, 2, 64, 16, seqs, seed=3, temp=(0.3, 100), bias=True,
                                            sink=True, min_split_keys=128, max_cluster=max_cluster, target_ctas=592)
    assert len(plan.merge_items) > 0 or plan.cluster > 1
    tol = 2e-5 if dtype == "float32" else 2.5e-2
    assert np.abs(got - want).max() <= tol * np.abs(want).max()
    got, want, _ = run_changed_attention(DTYPES[dtype], 8, 2, 64, 16, seqs, seed=4, cap=3.0, chunk=500,
                                         min_split_keys=128, max_cluster=max_cluster, target_ctas=592)
    assert np.abs(got - want).max() <= tol * np.abs(want).max()


CHANGES = [dict(temp=(0.5, 7), bias=True, sink=True), dict(cap=2.0, chunk=150), dict(chunk=64), dict(cap=5.0),
           dict(bias=True), dict(sink=True, temp=(0.3, 100)), dict(chunk=1), dict(chunk=1000, cap=30.0)]


@pytest.mark.parametrize("change", range(len(CHANGES)))
@pytest.mark.parametrize("H,G,D,P", [(8, 2, 64, 16), (12, 2, 128, 16), (4, 4, 128, 64), (6, 1, 64, 8)])
def test_changed_scores_on_the_tensor_memory_family(H, G, D, P, change):
    """The same changes where long portions run on tcgen05 tiles of 128 rows x 64 keys: rows of
    one tile in different chunks, tiles wholly before a row's chunk, the term of score 0 as the
    start of a row's running sum, key ranges cut into several items."""
    from velox_b200.ops import attention_plan as ap
    from velox_b200.ops import kernels

    if not kernels.attention_has_tc(D):
        pytest.skip("no tensor-memory family for this head size")
    seqs = MIXED + [(300, 0), (200, 500), (40, 140), (129, 1), (64, 64)]
    got, want, plan = run_changed_attention(torch.bfloat16, H, G, D, P, seqs, seed=H + D + change, tensor_memory=True,
                                            **CHANGES[change])
    assert len(plan.items.get(ap.KIND_BF16_TC, ())) > 0
    assert np.abs(got - want).max() <= 2.5e-2 * np.abs(want).max()
    if change < 2:
        got, want, plan = run_changed_attention(torch.bfloat16, H, G, D, P, [(130, 900), (256, 1100), (1, 700)], seed=change,
                                                tensor_memory=True, fixed_splits=3, **CHANGES[change])
        assert len(plan.items.get(ap.KIND_BF16_TC, ())) > 0 and len(plan.merge_items) > 0
        assert np.abs(got - want).max() <= 2.5e-2 * np.abs(want).max()


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("H,G,dim,vdim,D,rot", [(4, 2, 16, 24, 32, 8), (3, 3, 12, 20, 32, 12), (1, 1, 20, 12, 48, 0),
                                                (4, 1, 128, 96, 256, 64), (6, 2, 10, 6, 32, 4), (6, 2, 64, 128, 128, 32),
                                                (2, 1, 32, 64, 64, 0), (5, 1, 16, 8, 32, 16)])
@pytest.mark.parametrize("pad", [5, 0])
def test_differential_attention_ends(dtype, H, G, dim, vdim, D, rot, pad):
    """Before the attention kernels: norm and rotation per head and map, the maps' places in a
    query row and in a cached key row, values in their pages.  After them: a1 - lambda a2, unit
    RMS, the factor and the gate."""
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(dim + vdim)
    T, P, pages, eps = 11, 4, 9, 1e-5
    qw, kw, vw = 2 * H * dim, 2 * G * dim, G * vdim
    # with pad 0 the rows are 16-byte multiples where the sizes allow it (the kernels' wide accesses)
    proj = torch.randn(T, qw + kw + vw + H * vdim + pad, generator=gen).to(dt)
    positions = torch.tensor([0, 1, 2, 3, 40, 41, 7, 99, 5, 6, 63], dtype=torch.int32)
    slots = torch.tensor([4, 5, 6, 7, 20, 21, 9, -1, 30, 31, 35], dtype=torch.int32)
    q_norm, k_norm = 1 + 0.3 * torch.randn(dim, generator=gen), 1 + 0.3 * torch.randn(dim, generator=gen)
    cos = sin = None
    if rot:
        angles = torch.arange(100, dtype=torch.float64)[:, None] * (50.0 ** (-2.0 * torch.arange(rot // 2) / rot))[None, :]
        cos, sin = angles.cos().float().cuda(), angles.sin().float().cuda()
    k_cache = torch.zeros(pages, P, G, D, dtype=dt).cuda()
    v_cache = torch.zeros(pages, P, G, D, dtype=dt).cuda()
    qbuf = torch.zeros(T, 2 * H * D, dtype=dt).cuda()
    status = torch.zeros(1, dtype=torch.int32).cuda()
    kernels.diff_prepare(proj.cuda(), qbuf, positions.cuda(), cos, sin, q_norm.cuda(), k_norm.cuda(), eps, slots.cuda(),
                         k_cache, v_cache, T, H, G, dim, vdim, D, rot, status)
    assert int(status.item()) == 0
    pos = positions.double().numpy()
    q = plain.rms_unit(proj[:, :qw].double().numpy().reshape(T, H, 2, dim), eps) * q_norm.double().numpy()
    k = plain.rms_unit(proj[:, qw : qw + kw].double().numpy().reshape(T, G, 2, dim), eps) * k_norm.double().numpy()
    if rot:
        q, k = plain.rotate_half(q, pos, 50.0, rot), plain.rotate_half(k, pos, 50.0, rot)
    v = proj[:, qw + kw : qw + kw + vw].double().numpy().reshape(T, G, vdim)
    got_q = qbuf.view(T, H, 2, D).double().cpu().numpy()
    scale = float(np.abs(q).max())
    for which in range(2):
        close(torch.from_numpy(got_q[:, :, which, which * dim : (which + 1) * dim]), q[:, :, which], dtype, f"q map {which}",
              scale=scale)
    assert np.all(got_q[:, :, 0, dim:] == 0) and np.all(got_q[:, :, 1, :dim] == 0) and np.all(got_q[:, :, 1, 2 * dim :] == 0)
    rows_k = k_cache.view(-1, G, D).double().cpu().numpy()
    rows_v = v_cache.view(-1, G, D).double().cpu().numpy()
    written = np.zeros(pages * P, bool)
    for t, slot in enumerate(slots.tolist()):
        if slot < 0:
            continue
        written[slot] = True
        close(torch.from_numpy(rows_k[slot, :, : 2 * dim]), k[t].reshape(G, 2 * dim), dtype, f"keys of token {t}", scale=scale)
        close(torch.from_numpy(rows_v[slot, :, :vdim]), v[t], dtype, f"values of token {t}")
        assert np.all(rows_k[slot, :, 2 * dim :] == 0) and np.all(rows_v[slot, :, vdim:] == 0)
    assert np.all(rows_k[~written] == 0) and np.all(rows_v[~written] == 0)

    attn = torch.randn(T, 2 * H * D, generator=gen).to(dt)
    gate = proj[:, qw + kw + vw : qw + kw + vw + H * vdim]
    lam, factor = 0.73, 0.55
    a = attn.double().numpy().reshape(T, H, 2, D)[..., :vdim]
    want = plain.rms_unit(a[:, :, 0] - lam * a[:, :, 1], eps) * factor * plain.sigmoid(gate.double().numpy().reshape(T, H, vdim))
    out = torch.zeros(T, H * vdim, dtype=dt).cuda()
    kernels.diff_combine(attn.cuda(), proj.cuda()[:, qw + kw + vw : qw + kw + vw + H * vdim], out, T, H, vdim, D, lam,
                         factor, eps)
    close(out, want.reshape(T, H * vdim), dtype, "combined maps")


# ------------------------------------------------------------------------------ whole models
CASES = {
    "small": (lc.SMALL, 4, (5, 11, 17, 60, 100), 2.0),
    "odd": (lc.ODD, 16, (1, 9, 33, 70, 150), 1.5),
    "wide": (lc.WIDE, 64, (130, 3, 65, 300, 64), 2.5),
    "mid": (lc.MID, 16, (40, 2, 101, 230, 91), 2.0),
}


def reference(cfg, tensors, tokens, collect=None):
    return plain.forward(cfg, lc.as_numpy(tensors), tokens, collect)


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, page, lengths, sharp) in CASES.items():
        folder = str(tmp_path_factory.mktemp("lizizen_" + name))
        tensors = lc.make_weights(cfg, seed=5 + len(name), sharp=sharp)
        lc.write_folder(folder, cfg, tensors)
        prompts = random_prompts(cfg["vocab"], lengths, seed=31)
        want = [reference(cfg, tensors, p) for p in prompts]
        out[name] = (folder, cfg, page, prompts, want, tensors)
    return out


def make_replayer(folder, dtype, max_tokens, page, **kw):
    from velox_b200.engine.replay import TraceReplayer

    return TraceReplayer(folder, dtype, max_tokens, block_size=page, **kw)


def replay_one(replayer, name, tokens, cuts):
    rows, start = [], 0
    for step, n in enumerate(cuts):
        rec = {"step": step, "entries": [{"id": name, "tokens": tokens[start : start + n], "want": list(range(n))}],
               "end": [name] if start + n == len(tokens) else []}
        rows.append(replayer.run_step(rec))
        start += n
    assert start == len(tokens)
    return np.concatenate(rows, axis=0)


def changing_cuts(total):
    sizes = [7, 2, 16, 3, 2, 5, 33, 2, 9, 64, 4, 2, 21]
    cuts, left, i = [], total, 0
    while left > 0:
        n = min(sizes[i % len(sizes)], left)
        if left - n == 1:
            n = left
        cuts.append(n)
        left -= n
        i += 1
    return cuts


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("case", list(CASES))
def test_whole_then_decode_then_portions(models, case, dtype):
    folder, cfg, page, prompts, want, _ = models[case]
    longest = max(len(p) for p in prompts)
    replayer = make_replayer(folder, dtype, max_tokens=max(256, -(-longest // 64) * 64), page=page)
    for index, (tokens, ref) in enumerate(zip(prompts, want)):
        L = len(tokens)
        whole = replay_one(replayer, f"w{index}", tokens, [L])
        check_logits(whole, ref, dtype, f"{case} request {index} whole")
        tail = min(32, L - 1)
        if tail > 0:
            decoded = replay_one(replayer, f"d{index}", tokens, [L - tail] + [1] * tail)
            check_logits(decoded, ref, dtype, f"{case} request {index} last {tail} one by one")
        if L > 2:
            portions = replay_one(replayer, f"p{index}", tokens, changing_cuts(L))
            check_logits(portions, ref, dtype, f"{case} request {index} in portions")
    replayer.cache.assert_consistent()
    assert replayer.cache.num_free_pages() == replayer.cache.num_total_pages
    assert replayer.cache.num_free_slots == replayer.max_live


@pytest.mark.parametrize("case", ["small", "odd"])
def test_layer_streams(models, case):
    """The stream after every layer run of the float32 path against the plain implementation's."""
    folder, cfg, page, prompts, _, tensors = models[case]
    tokens = prompts[3]
    streams = []
    reference(cfg, tensors, tokens, streams)
    replayer = make_replayer(folder, "float32", max_tokens=128, page=page, enable_graphs=False)
    seen = []
    wrapped_blocks = set()
    for block in replayer.model.blocks:
        if id(block) in wrapped_blocks:
            continue
        wrapped_blocks.add(id(block))
        def wrapped(hidden, ctx, cache, inner=block.forward):
            inner(hidden, ctx, cache)
            x = hidden.resid[: ctx.num_tokens].clone()
            if hidden.delta is not None:
                x += hidden.delta[: ctx.num_tokens].float()
            seen.append(x.double().cpu())
        block.forward = wrapped
    replay_one(replayer, "s", tokens, [len(tokens)])
    assert len(seen) == len(streams) == len(plain.run_order(cfg))
    for index, (got, want) in enumerate(zip(seen, streams)):
        close(got, want, "float32", f"stream after layer run {index}", scale=8 * float(np.abs(want).max()))


def mixed_trace(prompts, rng, max_live=4):
    progress = [0] * len(prompts)
    waiting = list(range(len(prompts)))
    live, steps = [], []
    step = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            live.append(waiting.pop(0))
        entries, ends = [], []
        for r in list(live):
            left = len(prompts[r]) - progress[r]
            if rng.random() < 0.2 and len(live) > 1:
                continue
            decoding = left <= 12 or rng.random() < 0.3
            n = 1 if decoding else min(left, int(rng.choice([2, 3, 5, 8, 13, 30])))
            if left - n == 0:
                ends.append(r)
            entries.append((r, progress[r], n))
            progress[r] += n
        if not entries:
            continue
        steps.append((step, entries, ends))
        for r in ends:
            live.remove(r)
        step += 1
    return steps


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("case", list(CASES))
def test_mixed_batches_with_pages_and_slots_used_again(models, case, dtype):
    """Every request twice, up to four live at a time in a pool that holds no more: a request's
    logits equal those of the request alone whatever shares its steps, and a slot's shift row and
    a page's keys of an earlier request do not leak into a later one."""
    folder, cfg, page, prompts, want, _ = models[case]
    order = list(range(len(prompts))) * 2
    seqs = [prompts[i] for i in order]
    steps = mixed_trace(seqs, np.random.default_rng(9))
    need = sum(sorted((-(-len(p) // 64) * 64 for p in prompts), reverse=True)[:4])
    replayer = make_replayer(folder, dtype, max_tokens=need, page=page, max_live=4)
    got = [np.zeros((len(p), cfg["vocab"]), np.float32) for p in seqs]
    slots_used = []
    for step, entries, ends in steps:
        rec = {"step": step, "end": [f"r{r}" for r in ends],
               "entries": [{"id": f"r{r}", "tokens": seqs[r][s : s + n], "want": list(range(n))} for r, s, n in entries]}
        out = replayer.run_step(rec)
        row = 0
        for r, s, n in entries:
            got[r][s : s + n] = out[row : row + n]
            row += n
        slots_used.extend(seq.slot for seq in replayer.live.values())
        replayer.cache.assert_consistent()
    for r, ref_index in enumerate(order):
        check_logits(got[r], want[ref_index], dtype, f"{case} mixed request {r}")
    assert replayer.cache.num_free_pages() == replayer.cache.num_total_pages
    assert set(slots_used) <= set(range(4))


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("case,page", [("small", 4), ("wide", 16)])
def test_long_decode(models, case, page, dtype):
    """390 tokens one by one: chunks of 10, 64 and 150 keys end and begin among them, the
    temperature changes, and the keys of all 420 positions stay for the layers without chunks."""
    folder, cfg, _, _, _, tensors = models[case]
    tokens = random_prompts(cfg["vocab"], [420], seed=4)[0]
    ref = reference(cfg, tensors, tokens)
    replayer = make_replayer(folder, dtype, max_tokens=448, page=page)
    rows = replay_one(replayer, "long", tokens, [30] + [1] * 390)
    check_logits(rows, ref, dtype, "long decode")
    replayer.cache.assert_consistent()


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_long_prompt_whole_and_in_large_portions(models, dtype):
    folder, cfg, page, _, _, tensors = models["wide"]
    tokens = random_prompts(cfg["vocab"], [600], seed=14)[0]
    ref = reference(cfg, tensors, tokens)
    replayer = make_replayer(folder, dtype, max_tokens=640, page=page)
    check_logits(replay_one(replayer, "whole", tokens, [600]), ref, dtype, "600 tokens whole")
    check_logits(replay_one(replayer, "parts", tokens, [300, 299, 1]), ref, dtype, "600 tokens as 300 + 299 + 1")


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("case", ["small", "odd"])
def test_first_tokens(models, case, dtype):
    """The first token has no previous row to shift from, sees one key and (in the scored
    attention) shares its weight with the term of score 0."""
    folder, cfg, page, prompts, want, _ = models[case]
    replayer = make_replayer(folder, dtype, max_tokens=64, page=page)
    rows = replay_one(replayer, "f", prompts[3][:6], [1, 1, 2, 2])
    check_logits(rows, want[3][:6], dtype, "first tokens one by one")
    rows = replay_one(replayer, "g", prompts[3][:6], [2, 4])
    check_logits(rows, want[3][:6], dtype, "first tokens in portions")


def needle_model(tmp_path, kind):
    """A model of one layer whose first head puts nearly all weight of an ``asker`` token's query
    on a ``marker`` token's key, wherever that key is: one row of that head's q and k lines up
    with the two tokens' normed embeddings (no shift, so that h is the normed embedding).
    ``scored``: the attention over all keys with its distance bias, temperature and sink.
    ``chunked``: differential attention with a chunk of 40 keys, the needle in the first map in a
    dimension that is not rotated; the second map and the other heads stay random."""
    width, vocab = 64, 90
    if kind == "scored":
        layer = lc.layer("attention", lc.scored(2, 1, 16, 16, 0.05, q_temp=(0.2, 30)), None)
        coef = 0.35
    else:
        layer = lc.layer("attention_2", lc.differential(2, 1, 16, 16, 1.5, 0.3, chunk=40, rot=(100.0, 4), softcap=40.0), None)
        coef = 0.1
    cfg = lc.config(width, vocab, [layer])
    tensors = {k: v.float() for k, v in lc.make_weights(cfg, seed=2).items()}
    marker, asker = 7, 11
    tensors["l0.norm1"] = torch.zeros(width)
    tensors["l0.shift"] = torch.zeros(width)
    unit = lambda v: v / (v.pow(2).mean().sqrt())  # what the RMS norm makes of an embedding row
    rows = tensors["l0.mix.q"].shape[0] // 2
    q = tensors["l0.mix.q"].view(2, rows, width)
    k = tensors["l0.mix.k"].view(1, rows, width)
    q[0, 8] = coef * unit(tensors["embed"][asker])
    k[0, 8] = coef * unit(tensors["embed"][marker])
    if kind == "scored":
        tensors["l0.mix.r1"] = torch.tensor([0.5, 1.5])
        tensors["l0.mix.r2"] = torch.tensor([0.25, 0.1])
    else:
        tensors["l0.mix.q.norm"] = torch.ones(16)
        tensors["l0.mix.k.norm"] = torch.ones(16)
    tensors = {k_: v.to(torch.bfloat16) for k_, v in tensors.items()}
    folder = str(tmp_path / f"needle_{kind}")
    lc.write_folder(folder, cfg, tensors)
    return folder, cfg, tensors, marker, asker


NEEDLES = [
    # the attention over all keys: the first key, keys at page borders, hundreds of keys back
    ("scored", 319, 0, True), ("scored", 319, 63, True), ("scored", 319, 64, True), ("scored", 319, 200, True),
    ("scored", 319, 318, True),
    # chunks of 40: the asker at the end of a chunk, in its middle, at its first position
    ("chunked", 319, 280, True), ("chunked", 319, 279, False), ("chunked", 319, 0, False), ("chunked", 319, 318, True),
    ("chunked", 300, 280, True), ("chunked", 300, 279, False), ("chunked", 300, 256, False),
    ("chunked", 320, 319, False), ("chunked", 320, 280, False), ("chunked", 321, 320, True),
]


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("kind,ask_at,needle_at,seen", NEEDLES)
def test_keys_far_away_and_at_the_edges_of_a_chunk(tmp_path, dtype, kind, ask_at, needle_at, seen):
    """A key that takes nearly all softmax weight of one query when it is seen: far back and at
    page borders for the attention over all keys; just inside and just outside the query's chunk
    for the chunked mask; the query decoded alone, inside a portion, and in a whole prompt."""
    folder, cfg, tensors, marker, asker = needle_model(tmp_path, kind)
    length = 330
    tokens = [t if t not in (marker, asker) else 20 for t in random_prompts(90, [length], seed=needle_at)[0]]
    tokens[needle_at] = marker
    tokens[ask_at] = asker
    ref = reference(cfg, tensors, tokens)
    without = list(tokens)
    without[needle_at] = 21
    other = reference(cfg, tensors, without)
    moved = float(np.abs(other[ask_at] - ref[ask_at]).max())
    if seen:
        assert moved > 0.3, f"the needle does not matter enough for this test ({moved:.3f})"
    else:
        assert moved == 0.0, f"a key outside the chunk matters ({moved:.3f})"
    lo, hi = ask_at - 3, ask_at + 4
    replayer = make_replayer(folder, dtype, max_tokens=384, page=64)
    rows = replay_one(replayer, "n", tokens, [ask_at, 1, length - ask_at - 1])
    check_logits(rows[lo:hi], ref[lo:hi], dtype, f"{kind} needle at {needle_at}, decoded")
    rows = replay_one(replayer, "m", tokens, [100, 2, ask_at - 110, 12, length - ask_at - 4])
    check_logits(rows[lo:hi], ref[lo:hi], dtype, f"{kind} needle at {needle_at}, in portions")
    rows = replay_one(replayer, "w", tokens, [length])
    check_logits(rows[lo:hi], ref[lo:hi], dtype, f"{kind} needle at {needle_at}, whole")
    replayer = make_replayer(folder, dtype, max_tokens=384, page=16)
    rows = replay_one(replayer, "s", tokens, [ask_at - 1, 2, length - ask_at - 1])
    check_logits(rows[lo:hi], ref[lo:hi], dtype, f"{kind} needle at {needle_at}, pages of 16, a portion of two")


def test_the_term_of_score_zero_matters(tmp_path, monkeypatch):
    """With small scores the term of score 0 takes a good share of every row's weight (half of
    the first token's): the engine follows the plain model with it, and the plain model without
    it gives other logits."""
    cfg = lc.config(64, 80, [lc.layer("attention", lc.scored(4, 2, 16, 16, 0.1, q_temp=(0.3, 5)), lc.dense(32, 1.0)),
                             lc.layer("attention", lc.scored(2, 2, 8, 24, 0.1), None)])
    tensors = lc.make_weights(cfg, seed=3)
    tokens = random_prompts(80, [70], seed=6)[0]
    folder = str(tmp_path / "sink")
    lc.write_folder(folder, cfg, tensors)
    ref = reference(cfg, tensors, tokens)
    for dtype in DTYPES:
        replayer = make_replayer(folder, dtype, max_tokens=128, page=16)
        check_logits(replay_one(replayer, "a", tokens, [40, 1, 1, 28]), ref, dtype, "with the term of score 0")
        check_logits(replay_one(replayer, "b", tokens, [1] * 8 + [62]), ref, dtype, "with the term of score 0, from the start")
    monkeypatch.setattr(plain, "softmax_with_zero_sink", plain.softmax)
    without = reference(cfg, tensors, tokens)
    assert np.abs(without - ref).max() > 0.2, "the term of score 0 does not matter enough for this test"


def test_command_lines_take_the_design(tmp_path, capsys):
    import json

    from velox_b200.cli import benchmark, roofline

    common = ["--model-size", "tiny-l", "--num-requests", "5", "--max-tokens", "10", "--max-model-len", "128",
              "--max-num-seqs", "4", "--max-num-batched-tokens", "64", "--max-prefill-chunk-size", "16",
              "--block-size", "8", "--workload", "short", "--seed", "3"]
    assert benchmark.main(common + ["--temperature", "0"]) == 0
    assert "decode throughput" in capsys.readouterr().out
    assert benchmark.main(common + ["--temperature", "0.7", "--top-k", "10", "--no-pipeline"]) == 0
    capsys.readouterr()
    table = tmp_path / "roofline.json"
    assert roofline.main(["--model-size", "tiny-l", "--batch", "2", "--context", "40", "--layers", "3,6", "--steps", "4",
                          "--warmup", "1", "--block-size", "8", "--output-json", str(table)]) == 0
    rows = json.loads(table.read_text())
    assert rows[0]["us_per_layer"] > 0 and rows[0]["size"] == "tiny-l"


@pytest.mark.parametrize("case", ["small", "odd"])
def test_greedy_generation_through_the_engine(models, case):
    """The engine's own entry point: its scheduler cuts prompts into portions of 8 beside decoding
    requests, two requests at a time, greedy sampling."""
    from velox_b200.engine.engine import LLM
    from velox_b200.sampling.params import SamplingParams

    folder, cfg, page, prompts, _, tensors = models[case]
    asks = [prompts[1], prompts[2], prompts[0], prompts[3]]
    for dtype in ("float32", "bfloat16"):
        llm = LLM(folder, dtype=dtype, max_model_len=96, max_num_seqs=2, max_num_batched_tokens=24,
                  max_prefill_chunk_size=8, block_size=page, num_gpu_blocks=max(8, 320 // page))
        outputs = llm.generate(asks, SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True))
        for prompt, output in zip(asks, outputs):
            assert len(output) == 9
            rows = reference(cfg, tensors, prompt + output[:-1])[len(prompt) - 1 :]
            if dtype == "float32":
                assert output == rows.argmax(-1).tolist()
            else:
                for row, token in zip(rows, output):
                    assert row[token] >= row.max() - 3e-2 * np.abs(row).max()
