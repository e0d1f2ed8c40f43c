"""The Mamivik design in the engine against the plain implementation in ``plain_mamivik``.

First each mechanism's kernels alone (the norm with the input convolution and its state rows in
portions, the delta rule's scan in portions beside other sequences and in chunks, its normed and gated output,
the norm of a column range, the latent layer's rotation in halves and its gate per output, the
scaled sum of two mixers, the tanh GELU as a gated activation, stretched rotation tables), then
whole models through trace replay: whole prompts, the last tokens decoded one by one, portions
down to two tokens, mixed batches in a pool so small that pages and slots are used again, long
decoding, the first tokens, keys far away, at page borders and just inside and just outside each
window, sinks that matter, and greedy generation through the engine's entry point and scheduler.
"""
import math

import numpy as np
import pytest
import torch

import mamivik_configs as mc
import plain_mamivik as plain
from helpers import check_logits as _check_logits, random_prompts

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def check_logits(got, want, dtype, what):
    """float32 is the sharp test, row by row.  In bfloat16 a row may be ill-conditioned: where a
    head's sum over the recurrent state nearly cancels, the division by its root mean square
    multiplies the rounding of r, k and v.  So a row in fifty (one at least) may miss the
    tolerance, by no more than a factor of four; all others are held to it."""
    want = torch.from_numpy(np.asarray(want))
    if dtype == "float32":
        _check_logits(got, want, dtype, what)
        return
    got_t = torch.from_numpy(np.ascontiguousarray(np.asarray(got))).double()
    ratio = (got_t - want.double()).abs().amax(-1) / want.double().abs().amax(-1).clamp_min(1e-3)
    loose = ratio > 6e-2
    assert int(loose.sum()) <= max(1, len(ratio) // 50), f"{what}: {int(loose.sum())} of {len(ratio)} rows miss the tolerance"
    assert float(ratio.max()) <= 0.24, f"{what}: row {int(ratio.argmax())} is off by {float(ratio.max()):.3f} of its largest logit"
    keep = ~loose
    if int(keep.sum()):
        _check_logits(np.asarray(got)[keep.numpy()], want[keep], dtype, what, bf16_tolerance=6e-2, bf16_min_cosine=0.997)


def close(got, want, dtype, what, scale=None, f32=4e-6, bf16=1.2e-2):
    got = got.double().cpu()
    want = torch.as_tensor(np.asarray(want)).double()
    scale = float(want.abs().max()) if scale is None else scale
    tol = (f32 if dtype == "float32" else bf16) * max(scale, 1e-6)
    err = float((got - want).abs().max())
    assert err <= tol, f"{what} ({dtype}): max error {err:.3e}, allowed {tol:.3e}"


def step_arrays(lengths, slots):
    starts = np.concatenate([[0], np.cumsum(lengths)[:-1]]).astype(np.int32)
    as_dev = lambda a: torch.tensor(np.asarray(a, dtype=np.int32)).cuda()
    return as_dev(starts), as_dev(lengths), as_dev(slots)


# ------------------------------------------------------------------------------------ kernels
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("width,taps", [(64, 3), (100, 2), (250, 5), (1536, 4), (48, 1), (72, 8)])
def test_norm_and_input_convolution_in_portions(dtype, width, taps):
    """Three sequences side by side, cut into portions of changing size (down to one token, and
    shorter than the taps), each with its own state row; a fourth row of the state stays as it was."""
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(width + taps)
    lengths = [37, 9, 21]
    x = [torch.randn(n, width, generator=gen) * 3.0 for n in lengths]
    w = 1.0 + 0.3 * torch.randn(1, generator=gen).expand(width).contiguous()
    cw = 0.5 * torch.randn(width, taps, generator=gen)
    eps = 1e-5
    want = []
    for rows in x:
        h = plain.rms_unit(rows.double().numpy(), eps) * w.double().numpy()
        want.append(h + plain.causal_conv(h, cw.double().numpy()))
    state = torch.zeros(5, max(taps - 1, 1) * width).cuda()
    state[3] = 7.0
    slots = [2, 0, 4]
    got = [np.zeros((n, width)) for n in lengths]
    done = [0, 0, 0]
    cuts = [[1, 1, 2, 5, 1, 3, 24], [2, 1, 6], [21]]
    for step in range(max(len(c) for c in cuts)):
        live = [s for s in range(3) if step < len(cuts[s])]
        sizes = [cuts[s][step] for s in live]
        rows = torch.cat([x[s][done[s] : done[s] + n] for s, n in zip(live, sizes)]).cuda()
        out = torch.zeros(rows.shape[0], width, dtype=dt).cuda()
        q_start, q_len, seq_slots = step_arrays(sizes, [slots[s] for s in live])
        kernels.norm_conv(rows, w.cuda(), eps, cw.t().contiguous().cuda(), state if taps > 1 else None, out, rows.shape[0], q_start,
                          q_len, seq_slots, len(live))
        at = 0
        for s, n in zip(live, sizes):
            got[s][done[s] : done[s] + n] = out[at : at + n].double().cpu().numpy()
            done[s] += n
            at += n
    for s in range(3):
        close(torch.from_numpy(got[s]), want[s], dtype, f"sequence {s}")
    assert bool((state[3] == 7.0).all())
    if taps > 1:
        last = plain.rms_unit(x[0].double().numpy(), eps)[-(taps - 1):] * w.double().numpy()
        close(state[2].view(taps - 1, width), last, "float32", "the state after the last portion")


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("heads,dim", [(2, 16), (3, 8), (1, 24), (4, 32), (2, 64), (1, 128), (2, 48), (1, 200)])
def test_delta_rule_scan_in_portions(dtype, heads, dim):
    """Two sequences in portions beside each other (one decoded token by token at the end), each
    with its own state row; the state after the last portion is the plain recurrence's."""
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(heads * 100 + dim)
    inner = heads * dim
    lengths = [45, 20]
    cuts = [[17, 1, 1, 20, 2, 1, 1, 1, 1], [3, 16, 1]]
    decay, key_eps = math.exp(-0.5), 1e-6
    w0 = (1.5 * torch.randn(inner, generator=gen)).float()
    ab = (1.5 * torch.randn(inner, generator=gen)).float()
    proj = [torch.randn(n, 4 * inner + 3, generator=gen).to(dt) for n in lengths]   # r | k | v | a and more
    logit = [(2.0 * torch.randn(n, inner, generator=gen)).to(dt) for n in lengths]
    want, want_state = [], []
    for p, l in zip(proj, logit):
        pd, ld = p.double().numpy(), l.double().numpy()
        r, k, v, a = (pd[:, i * inner : (i + 1) * inner].reshape(-1, heads, dim) for i in range(4))
        w = np.exp(-decay * plain.sigmoid(ld + w0.double().numpy())).reshape(-1, heads, dim)
        a = plain.sigmoid(a.reshape(-1, inner) + ab.double().numpy()).reshape(-1, heads, dim)
        outs, states = zip(*(plain.delta_rule_states(r[:, h], k[:, h], v[:, h], w[:, h], a[:, h]) for h in range(heads)))
        want.append(np.stack(outs, axis=1).reshape(-1, inner))
        want_state.append(np.stack(states))
    state = torch.zeros(4, inner * dim).cuda()
    state[1] = 3.0
    slots = [3, 0]
    got = [np.zeros((n, inner)) for n in lengths]
    done = [0, 0]
    for step in range(max(len(c) for c in cuts)):
        live = [s for s in range(2) if step < len(cuts[s])]
        sizes = [cuts[s][step] for s in live]
        rows = torch.cat([proj[s][done[s] : done[s] + n] for s, n in zip(live, sizes)]).cuda()
        lg = torch.cat([logit[s][done[s] : done[s] + n] for s, n in zip(live, sizes)]).cuda()
        out = torch.zeros(rows.shape[0], inner).cuda()
        q_start, q_len, seq_slots = step_arrays(sizes, [slots[s] for s in live])
        packed = torch.zeros(rows.shape[0], kernels.delta_rule_packed_width(heads, dim, dim)).cuda()
        status = torch.zeros(4, dtype=torch.int32).cuda()
        kernels.delta_rule_scan(rows[:, :inner], rows[:, inner : 2 * inner], rows[:, 2 * inner : 3 * inner],
                                rows[:, 3 * inner : 4 * inner], lg, w0.cuda(), ab.cuda(), decay, key_eps, state, out,
                                heads, dim, dim, q_start, q_len, seq_slots, len(live), rows.shape[0], packed, status)
        assert int(status[0]) == 0
        at = 0
        for s, n in zip(live, sizes):
            got[s][done[s] : done[s] + n] = out[at : at + n].double().cpu().numpy()
            done[s] += n
            at += n
    for s in range(2):
        scale = float(np.abs(want[s]).max())
        close(torch.from_numpy(got[s]), want[s], "float32", f"sequence {s}", scale=scale, f32=2e-5)
        kept = state[slots[s]].view(heads, dim, dim).transpose(1, 2)       # stored [head][column][row]
        close(kept, want_state[s], "float32", f"state of sequence {s}", f32=2e-5)
    assert bool((state[1] == 3.0).all())


@pytest.mark.parametrize("heads,dim", [(2, 16), (1, 64), (3, 24), (1, 136), (2, 10)])
def test_delta_rule_scan_in_chunks(heads, dim):
    """Steps of 512 tokens and more run in chunks of 256 tokens side by side: a portion of three
    chunks and a bit, one of exactly two, a short one and a single token in one step, from states
    that are not zero; then each sequence goes on, so that the kept states are used."""
    from velox_b200.ops import kernels

    gen = torch.Generator().manual_seed(heads + dim)
    inner = heads * dim
    first, second = [800, 512, 37, 1], [3, 600, 1, 20]
    decay, key_eps = math.exp(-0.5), 1e-6
    w0 = (1.5 * torch.randn(inner, generator=gen)).float()
    ab = (1.5 * torch.randn(inner, generator=gen)).float()
    seqs = len(first)
    proj = [torch.randn(a + b, 4 * inner, generator=gen) for a, b in zip(first, second)]
    logit = [2.0 * torch.randn(a + b, inner, generator=gen) for a, b in zip(first, second)]
    start = [0.3 * torch.randn(heads, dim, dim, generator=gen) for _ in range(seqs)]      # [head][row][column]
    want = []
    for p, l, s0 in zip(proj, logit, start):
        pd, ld = p.double().numpy(), l.double().numpy()
        r, k, v, a = (pd[:, i * inner : (i + 1) * inner].reshape(-1, heads, dim) for i in range(4))
        w = np.exp(-decay * plain.sigmoid(ld + w0.double().numpy())).reshape(-1, heads, dim)
        a = plain.sigmoid(a.reshape(-1, inner) + ab.double().numpy()).reshape(-1, heads, dim)
        outs = [plain.delta_rule_states(r[:, h], k[:, h], v[:, h], w[:, h], a[:, h], S=s0[h].double().numpy())[0]
                for h in range(heads)]
        want.append(np.stack(outs, axis=1).reshape(-1, inner))
    state = torch.zeros(seqs + 1, inner * dim).cuda()
    for s in range(seqs):
        state[s] = start[s].transpose(1, 2).reshape(-1).cuda()                             # stored [head][column][row]
    got = [np.zeros((a + b, inner)) for a, b in zip(first, second)]
    done = [0] * seqs
    for sizes in (first, second):
        total = sum(sizes)
        rows = torch.cat([proj[s][done[s] : done[s] + n] for s, n in enumerate(sizes)]).cuda()
        lg = torch.cat([logit[s][done[s] : done[s] + n] for s, n in enumerate(sizes)]).cuda()
        out = torch.zeros(total, inner).cuda()
        q_start, q_len, seq_slots = step_arrays(sizes, list(range(seqs)))
        packed = torch.zeros(total, kernels.delta_rule_packed_width(heads, dim, dim)).cuda()
        scratch = torch.zeros(kernels.delta_rule_chunk_scratch(total, seqs, heads, dim, dim)).cuda()
        status = torch.zeros(4, dtype=torch.int32).cuda()
        kernels.delta_rule_scan(rows[:, :inner], rows[:, inner : 2 * inner], rows[:, 2 * inner : 3 * inner],
                                rows[:, 3 * inner : 4 * inner], lg, w0.cuda(), ab.cuda(), decay, key_eps, state, out,
                                heads, dim, dim, q_start, q_len, seq_slots, seqs, total, packed, status,
                                chunk_scratch=scratch)
        assert int(status[0]) == 0
        at = 0
        for s, n in enumerate(sizes):
            got[s][done[s] : done[s] + n] = out[at : at + n].double().cpu().numpy()
            done[s] += n
            at += n
    for s in range(seqs):
        close(torch.from_numpy(got[s]), want[s], "float32", f"sequence {s}", scale=float(np.abs(want[s]).max()), f32=5e-5)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("T,heads,dim", [(1, 2, 16), (19, 3, 24), (300, 4, 64)])
def test_delta_rule_output_norm_and_gate(dtype, T, heads, dim):
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(T)
    inner = heads * dim
    y = (4.0 * torch.randn(T, inner, generator=gen)).float()
    z = torch.randn(T, inner + 5, generator=gen).to(dt)
    w = 1.0 + 0.3 * torch.randn(inner, generator=gen)
    eps = 1e-5
    want = (plain.rms_unit(y.double().numpy().reshape(T, heads, dim), eps).reshape(T, inner) * w.double().numpy()
            * plain.sigmoid(z.double().numpy()[:, 2 : 2 + inner]))
    out = torch.zeros(T, inner, dtype=dt).cuda()
    kernels.gated_group_norm(y.cuda(), z.cuda()[:, 2 : 2 + inner], w.cuda(), eps, heads, out, T, gate_after=True)
    close(out, want, dtype, "normed and gated heads")


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("T,n,pad", [(1, 10, 6), (33, 80, 0), (7, 36, 4)])
def test_norm_of_a_column_range(dtype, T, n, pad):
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(n)
    x = (3.0 * torch.randn(T, n + 11, generator=gen)).to(dt)
    w = 1.0 + 0.3 * torch.randn(n, generator=gen)
    want = plain.rms_unit(x.double().numpy()[:, 3 : 3 + n], 1e-5) * w.double().numpy()
    out = torch.full((T, n + pad), 9.0, dtype=dt).cuda()
    kernels.rms_rows(x.cuda()[:, 3 : 3 + n], w.cuda(), 1e-5, out, T)
    close(out[:, :n], want, dtype, "normed columns")
    assert bool((out[:, n:] == 0).all())


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("H,dim,R,rank,scaling", [(3, 16, 8, 32, (4.0, 16, 8.0, 1.0)), (1, 20, 4, 28, None),
                                                  (6, 64, 32, 128, (2.0, 64, 16.0, 2.0)), (5, 12, 12, 20, None)])
def test_latent_rows_and_queries_rotated_in_halves(dtype, H, dim, R, rank, scaling):
    """The latent layer's way into the attention kernels with the queries in a buffer of their own
    and pairs (i, i + R / 2): cached rows and query rows against the plain rotation."""
    from velox_b200.ops import kernels
    from velox_b200.parts.rope import RotaryHalf

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(H + R)
    T, P, pages = 9, 4, 6
    Dp = -(-(rank + R) // 16) * 16
    rot = mc.rot(1000.0, R, scaling)
    part = RotaryHalf({"head_dim": R, "rotary_dim": R, "theta": 1000.0, "scaling": rot.get("scaling"),
                       "max_position": 64, "angles": "float64"}, {}, dt, torch.device("cuda"))
    positions = torch.tensor([0, 1, 2, 40, 41, 5, 63, 7, 8], dtype=torch.int32)
    slots = torch.tensor([4, 5, 6, 20, 21, -1, 9, 10, 11], dtype=torch.int32)
    proj = torch.randn(T, 5 + rank + R + 3, generator=gen).to(dt)
    qsrc = torch.randn(T, H * (dim + R), generator=gen).to(dt)
    lw = 1.0 + 0.3 * torch.randn(rank, generator=gen)
    cache = torch.zeros(pages, P, 1, Dp, dtype=dt).cuda()
    queries = torch.full((T, H, Dp), 5.0, dtype=dt).cuda()
    status = torch.zeros(4, dtype=torch.int32).cuda()
    kernels.latent_prepare(proj.cuda(), 0, 5, positions.cuda(), part.cos, part.sin, lw.cuda(), 1e-5, slots.cuda(), cache,
                           queries, T, H, dim, R, rank, status, half_layout=True, q_source=qsrc.cuda())
    assert int(status[0]) == 0
    pd = proj.double().numpy()
    c = plain.rms_unit(pd[:, 5 : 5 + rank], 1e-5) * lw.double().numpy()
    k_rot = plain.rotate_halves(pd[:, 5 + rank : 5 + rank + R].reshape(T, 1, R), rot, positions.numpy())[:, 0]
    q_rot = plain.rotate_halves(qsrc.double().numpy().reshape(T, H, dim + R)[..., dim:], rot, positions.numpy())
    rows = cache.view(-1, Dp).double().cpu().numpy()
    for t, slot in enumerate(slots.tolist()):
        if slot < 0:
            continue
        close(torch.from_numpy(rows[slot, :rank]), c[t], dtype, f"latent of token {t}")
        close(torch.from_numpy(rows[slot, rank : rank + R]), k_rot[t], dtype, f"rotated key part of token {t}")
        assert np.all(rows[slot, rank + R :] == 0)
    got_q = queries.double().cpu().numpy()
    close(torch.from_numpy(got_q[:, :, rank : rank + R]), q_rot, dtype, "rotated query parts")
    assert np.all(got_q[:, :, rank + R :] == 0)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("H,G,D,rot", [(4, 2, 32, 16), (3, 3, 16, 16), (6, 2, 48, 4), (2, 1, 64, 64), (5, 1, 16, 0)])
def test_values_written_from_the_unrotated_key_columns(dtype, H, G, D, rot):
    """Rows of q | k only: q turns in place, k turns on its way into its page, and the value page gets
    the row's k as it stands (all three forms of the kernel: scalar, 16 bytes at a time, pairs)."""
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(H * D + rot)
    T, P, pages = 6, 4, 5
    spec = {"base": 100.0, "dims": rot}
    positions = torch.tensor([0, 1, 9, 30, 31, 5], dtype=torch.int32)
    slots = torch.tensor([4, 5, 6, -1, 17, 8], dtype=torch.int32)
    rows = torch.randn(T, (H + G) * D, generator=gen).to(dt)
    cos = sin = None
    if rot:
        f, _ = plain.frequencies(spec)
        angle = np.arange(40)[:, None] * f[None, :]
        cos = torch.tensor(np.cos(angle), dtype=torch.float32).cuda()
        sin = torch.tensor(np.sin(angle), dtype=torch.float32).cuda()
    k_cache = torch.zeros(pages, P, G, D, dtype=dt).cuda()
    v_cache = torch.zeros(pages, P, G, D, dtype=dt).cuda()
    status = torch.zeros(4, dtype=torch.int32).cuda()
    on_device = rows.clone().cuda()
    kernels.rope_cache_write(on_device, positions.cuda(), cos, sin, slots.cuda(), k_cache, v_cache, T, H, G, D, rot,
                             status, values_from_keys=True)
    assert int(status[0]) == 0
    rd = rows.double().numpy()
    q, k = rd[:, : H * D].reshape(T, H, D), rd[:, H * D :].reshape(T, G, D)
    q_want = plain.rotate_halves(q, spec, positions.numpy()) if rot else q
    k_want = plain.rotate_halves(k, spec, positions.numpy()) if rot else k
    close(on_device[:, : H * D].view(T, H, D), q_want, dtype, "q in place")
    assert torch.equal(on_device[:, H * D :].cpu(), rows[:, H * D :]), "the key columns of the row must stay as projected"
    kc, vc = k_cache.view(-1, G, D).double().cpu().numpy(), v_cache.view(-1, G, D).double().cpu().numpy()
    written = np.zeros(pages * P, bool)
    for t, slot in enumerate(slots.tolist()):
        if slot < 0:
            continue
        written[slot] = True
        close(torch.from_numpy(kc[slot]), k_want[t], dtype, f"rotated keys of token {t}")
        assert np.array_equal(vc[slot], k[t]), f"values of token {t} are not its unrotated keys"
    assert np.all(kc[~written] == 0) and np.all(vc[~written] == 0)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("T,H,N,K", [(1, 3, 24, 32), (40, 5, 20, 20), (9, 2, 80, 128), (70, 4, 48, 192)])
def test_per_head_product_with_a_gate_per_output(dtype, T, H, N, K):
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(T + N)
    Kp = -(-K // 16) * 16
    x = torch.randn(T, H * Kp, generator=gen).to(dt)
    w = (torch.randn(H, N, K, generator=gen) / K ** 0.5).to(dt)
    gate = torch.randn(T, 7 + H * N, generator=gen).to(dt)
    xd = x.double().numpy().reshape(T, H, Kp)[..., :K]
    want = np.einsum("thk,hnk->thn", xd, w.double().numpy()) * plain.sigmoid(gate.double().numpy()[:, 7:].reshape(T, H, N))
    out = torch.zeros(T, H * N, dtype=dt).cuda()
    kernels.headwise_linear(x.cuda(), 0, Kp, w.cuda(), out, 0, N, T, gate=gate.cuda(), gate_offset=7, gate_each=True)
    close(out, want.reshape(T, H * N), dtype, "gated per-head product")


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("T,width", [(1, 64), (13, 100), (300, 1536)])
def test_scaled_sum_of_two_mixers(dtype, T, width):
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(T)
    x = torch.randn(T, width, generator=gen)
    a, b = torch.randn(T, width, generator=gen).to(dt), torch.randn(T, width, generator=gen).to(dt)
    want = x.double() + 1.3 * a.double() + 0.7 * b.double()
    resid = x.clone().cuda()
    kernels.add_rows(resid, a.cuda(), b.cuda(), T, 1.3, 0.7)
    close(resid, want, "float32", "scaled sum", f32=1e-6)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("T,F", [(1, 128), (17, 40), (300, 1000)])
def test_tanh_gelu_as_a_gated_activation(dtype, T, F):
    from velox_b200.models.mamivik import GELU_ALPHA, GELU_CUBIC
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(F)
    gate_up = (2.5 * torch.randn(T, 2 * F, generator=gen)).to(dt)
    gd = gate_up.double().numpy()
    want = plain.gelu_tanh(gd[:, :F]) * gd[:, F:]
    out = torch.zeros(T, F, dtype=dt).cuda()
    kernels.clamped_glu(gate_up.cuda(), out, T, F, 0.0, GELU_ALPHA, 0.0, cubic=GELU_CUBIC)
    close(out, want, dtype, "gelu(gate) * up", f32=2e-6)


@pytest.mark.parametrize("T,F,K", [(1, 128, 64), (17, 40, 104), (64, 1024, 256)])
def test_tanh_gelu_in_the_projection(T, F, K):
    from velox_b200.models.mamivik import GELU_ALPHA, GELU_CUBIC
    from velox_b200.ops import kernels

    gen = torch.Generator().manual_seed(F + K)
    x = torch.randn(T, K, generator=gen).to(torch.bfloat16)
    w = (1.5 * torch.randn(2 * F, K, generator=gen) / K ** 0.5).to(torch.bfloat16)
    pre = x.double().numpy() @ w.double().numpy().T
    want = plain.gelu_tanh(pre[:, :F]) * pre[:, F:]
    out = torch.zeros(T, F, dtype=torch.bfloat16).cuda()
    status = torch.zeros(4, dtype=torch.int32).cuda()
    kernels.gemm_bf16_glu(x.cuda(), w.cuda(), None, out, T, 0.0, GELU_ALPHA, 0.0, status, cubic=GELU_CUBIC)
    assert int(status[0]) == 0
    close(out, want, "bfloat16", "gelu(gate) * up in the epilogue")


def test_stretched_rotation_tables():
    from velox_b200.parts.rope import RotaryHalf

    for base, dims, scaling in [(10000.0, 32, (2.0, 2048, 32.0, 1.0)), (50.0, 12, (8.0, 32, 4.0, 0.5)), (100.0, 8, None)]:
        rot = mc.rot(base, dims, scaling)
        part = RotaryHalf({"head_dim": dims, "rotary_dim": dims, "theta": base, "scaling": rot.get("scaling"),
                           "max_position": 300, "angles": "float64"}, {}, torch.float32, torch.device("cuda"))
        f, magnitude = plain.frequencies(rot)
        angle = np.arange(300)[:, None] * f[None, :]
        close(part.cos, np.cos(angle) * magnitude, "float32", "cos", f32=1e-6)
        close(part.sin, np.sin(angle) * magnitude, "float32", "sin", f32=1e-6)


# ------------------------------------------------------------------------------ whole models
CASES = {
    "small": (mc.SMALL, 4, (5, 11, 17, 60, 100), 2.0),
    "odd": (mc.ODD, 16, (1, 9, 33, 70, 150), 1.5),
    "wide": (mc.WIDE, 64, (130, 3, 65, 300, 64), 2.5),
    "mid": (mc.MID, 16, (40, 2, 101, 230, 91), 2.0),
    "taps": (mc.TAPS, 8, (2, 3, 1, 50, 24), 2.0),
    "broad": (mc.BROAD, 16, (7, 1, 40, 90, 18), 2.0),
    "many": (mc.MANY, 16, (12, 1, 70, 33, 5), 2.0),
}


def reference(cfg, tensors, tokens, collect=None):
    return plain.forward(cfg, mc.as_numpy(tensors), tokens, collect)


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, page, lengths, sharp) in CASES.items():
        folder = str(tmp_path_factory.mktemp("mamivik_" + name))
        tensors = mc.make_weights(cfg, seed=5 + len(name), sharp=sharp, decay_rank=mc.DECAY_RANKS[name])
        mc.write_folder(folder, cfg, tensors)
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
            if dtype == "float32":
                # the float32 path: a row's logits do not depend on how the prompt was cut
                assert np.array_equal(decoded, whole), f"{case} request {index}: decoded rows differ from the whole prompt's"
        if L > 2:
            portions = replay_one(replayer, f"p{index}", tokens, changing_cuts(L))
            check_logits(portions, ref, dtype, f"{case} request {index} in portions")
        if L > 1:
            each = replay_one(replayer, f"e{index}", tokens[: min(L, 24)], [1] * min(L, 24))
            check_logits(each, ref[: min(L, 24)], dtype, f"{case} request {index} token by token from the start")
    replayer.cache.assert_consistent()
    assert replayer.cache.num_free_pages() == replayer.cache.num_total_pages
    assert replayer.cache.num_free_slots == replayer.max_live


@pytest.mark.parametrize("case", ["small", "odd", "taps"])
def test_layer_streams(models, case):
    """The stream after every layer of the float32 path against the plain implementation's."""
    folder, cfg, page, prompts, _, tensors = models[case]
    tokens = prompts[3]
    streams = []
    reference(cfg, tensors, tokens, streams)
    replayer = make_replayer(folder, "float32", max_tokens=128, page=page, enable_graphs=False)
    seen = []
    for block in replayer.model.blocks:
        def wrapped(hidden, ctx, cache, inner=block.forward):
            inner(hidden, ctx, cache)
            x = hidden.resid[: ctx.num_tokens].clone()
            if hidden.delta is not None:
                x += hidden.delta[: ctx.num_tokens].float()
            seen.append(x.double().cpu())
        block.forward = wrapped
    replay_one(replayer, "s", tokens, [len(tokens)])
    assert len(seen) == len(streams) == len(cfg["layers"])
    for index, (got, want) in enumerate(zip(seen, streams)):
        close(got, want, "float32", f"stream after layer {index}", scale=8 * float(np.abs(want).max()))


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
    logits equal those of the request alone whatever shares its steps, and a slot's convolution
    rows and recurrent state and a page's keys of an earlier request do not leak into a later one."""
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
    if dtype == "float32":
        for r in range(len(prompts)):
            assert np.array_equal(got[r], got[r + len(prompts)]), f"{case}: request {r} differs between its two runs"
    assert replayer.cache.num_free_pages() == replayer.cache.num_total_pages
    assert set(slots_used) <= set(range(4))


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("case,page", [("small", 4), ("wide", 16)])
def test_long_decode(models, case, page, dtype):
    """390 tokens one by one: every window passes over decoded tokens, pages behind the windows go
    back to the pool, and the recurrent state runs through 420 updates."""
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
@pytest.mark.parametrize("case", ["small", "odd", "taps"])
def test_first_tokens(models, case, dtype):
    """The first tokens have fewer inputs than the convolution has taps, see fewer keys than the
    window holds, share their weight with the sink, and start the state from zero."""
    folder, cfg, page, prompts, want, _ = models[case]
    replayer = make_replayer(folder, dtype, max_tokens=64, page=page)
    rows = replay_one(replayer, "f", prompts[3][:7], [1, 1, 2, 2, 1])
    check_logits(rows, want[3][:7], dtype, "first tokens one by one")
    rows = replay_one(replayer, "g", prompts[3][:7], [2, 5])
    check_logits(rows, want[3][:7], dtype, "first tokens in portions")
    rows = replay_one(replayer, "h", prompts[3][:7], [3, 1, 3])
    check_logits(rows, want[3][:7], dtype, "first tokens, a portion as long as the taps")


def needle_model(tmp_path, kind, window):
    """A model of one layer whose first head puts nearly all weight of an ``asker`` token's query
    on a ``marker`` token's key, when that key is inside the window: one row of that head's query
    and key projections lines up with the two tokens' normed embeddings (no convolution, norm
    weight 1, so that h is the normed embedding), in a dimension that is not rotated.
    ``latent``: the needle goes through both latents (the query's and the keys') and the sink is
    far below the needle's score.  ``left``: the values are the keys, so the marker's key is also
    what the asker reads."""
    width, vocab = 64, 90
    if kind == "latent":
        layer = mc.layer("latent_attention", mc.latent(2, 16, 8, 16, width, width, 0.05, window, 100.0), None)
    else:
        layer = mc.layer("parallel", mc.parallel(mc.left(2, 1, 16, 0.05, window, 100.0, 4), 1, 8, 1.0, 0.05), None)
    cfg = mc.config(width, vocab, 2, [layer])
    tensors = {k: v.float() for k, v in mc.make_weights(cfg, seed=2, decay_rank=8).items()}
    marker, asker = 7, 11
    tensors["l0.norm1"] = torch.ones(())
    tensors["l0.canon1"] = torch.zeros(width, 2)
    unit = lambda v: v / (v.pow(2).mean().sqrt())  # what the RMS norm makes of an embedding row
    ea, em = unit(tensors["embed"][asker]), unit(tensors["embed"][marker])
    coef = 0.35
    if kind == "latent":
        # Both latents pass h through (identity down projections, norm weights 1): c = cq = h again
        # after their norms, since h has unit RMS already.
        tensors["l0.mix.dq"] = torch.eye(width)
        tensors["l0.mix.dq.norm"] = torch.ones(width)
        dkv = 0.1 * torch.randn(width + 8, width, generator=torch.Generator().manual_seed(1)) / width ** 0.5
        dkv[:width] = torch.eye(width)
        tensors["l0.mix.dkv"] = dkv
        tensors["l0.mix.dkv.norm"] = torch.ones(width)
        uq = tensors["l0.mix.uq"].view(2, 24, width)
        uk = tensors["l0.mix.uk"].view(2, 16, width)
        uq[0, 5] = coef * ea
        uk[0, 5] = coef * em
        tensors["l0.mix.sink"] = torch.tensor([0.5, -1.0])
    else:
        q = tensors["l0.mix.left.q"].view(2, 16, width)
        k = tensors["l0.mix.left.k"].view(1, 16, width)
        q[0, 9] = coef * ea
        k[0, 9] = coef * em
    tensors = {k_: v.to(torch.bfloat16) for k_, v in tensors.items()}
    folder = str(tmp_path / f"needle_{kind}_{window}")
    mc.write_folder(folder, cfg, tensors)
    return folder, cfg, tensors, marker, asker


NEEDLES = [
    # a window of 40 keys: the asker sees positions ask - 39 .. ask
    ("latent", 40, 319, 280, True), ("latent", 40, 319, 279, False), ("latent", 40, 319, 318, True),
    ("latent", 40, 300, 261, True), ("latent", 40, 300, 260, False), ("latent", 40, 300, 0, False),
    ("left", 40, 319, 280, True), ("left", 40, 319, 279, False), ("left", 40, 319, 318, True),
    ("left", 40, 300, 261, True), ("left", 40, 300, 260, False), ("left", 40, 300, 0, False),
    # a window longer than the prompt: the first key, keys at page borders, hundreds of keys back
    ("latent", 1000, 319, 0, True), ("latent", 1000, 319, 63, True), ("latent", 1000, 319, 64, True),
    ("left", 1000, 319, 0, True), ("left", 1000, 319, 64, True), ("left", 1000, 319, 200, True),
    # a window of a page and a half
    ("latent", 96, 320, 225, True), ("latent", 96, 320, 224, False), ("left", 96, 320, 225, True),
    ("left", 96, 320, 224, False),
]


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("kind,window,ask_at,needle_at,seen", NEEDLES)
def test_keys_far_away_and_at_the_edges_of_a_window(tmp_path, dtype, kind, window, ask_at, needle_at, seen):
    """A key that takes nearly all softmax weight of one query when it is seen: just inside and
    just outside the window, far back and at page borders; the query decoded alone, inside a
    portion, and in a whole prompt."""
    folder, cfg, tensors, marker, asker = needle_model(tmp_path, kind, window)
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
    elif kind == "latent":
        assert moved == 0.0, f"a key outside the window matters ({moved:.3f})"
    else:
        # the recurrent state beside the attention remembers every token, with a small weight
        assert moved < 0.1, f"a key outside the window matters ({moved:.3f})"
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


def test_the_sink_matters(tmp_path, monkeypatch):
    """With small scores the sink takes a good share of every row's weight: the engine follows the
    plain model with it, and the plain model without it gives other logits."""
    cfg = mc.config(64, 80, 3, [mc.layer("latent_attention", mc.latent(4, 16, 8, 16, 40, 24, 0.1, 30, 100.0), mc.dense(32)),
                                mc.layer("latent_attention", mc.latent(2, 8, 4, 24, 24, 16, 0.1, 9, 100.0), None)])
    tensors = mc.make_weights(cfg, seed=3)
    for index in (0, 1):
        tensors[f"l{index}.mix.sink"] = torch.tensor([3.0, 1.0, -30.0, 6.0][: cfg["layers"][index]["mixer"]["heads"]]
                                                     ).to(torch.bfloat16)
    tokens = random_prompts(80, [70], seed=6)[0]
    folder = str(tmp_path / "sink")
    mc.write_folder(folder, cfg, tensors)
    ref = reference(cfg, tensors, tokens)
    for dtype in DTYPES:
        replayer = make_replayer(folder, dtype, max_tokens=128, page=16)
        check_logits(replay_one(replayer, "a", tokens, [40, 1, 1, 28]), ref, dtype, "with the sink")
        check_logits(replay_one(replayer, "b", tokens, [1] * 8 + [62]), ref, dtype, "with the sink, from the start")
    inner = plain.attend
    monkeypatch.setattr(plain, "attend", lambda scores, mask, values, sink=None: inner(scores, mask, values))
    without = reference(cfg, tensors, tokens)
    assert np.abs(without - ref).max() > 0.2, "the sink does not matter enough for this test"


def test_values_are_the_unrotated_keys(tmp_path, monkeypatch):
    """The plain model with rotated keys as values gives other logits: the test sees the difference."""
    cfg = mc.config(64, 80, 1, [mc.layer("parallel", mc.parallel(mc.left(4, 2, 16, 0.3, 20, 10.0, 16), 1, 8, 1.5, 0.2),
                                         None)])
    tensors = mc.make_weights(cfg, seed=8, decay_rank=8)
    tokens = random_prompts(80, [50], seed=2)[0]
    folder = str(tmp_path / "values")
    mc.write_folder(folder, cfg, tensors)
    ref = reference(cfg, tensors, tokens)
    for dtype in DTYPES:
        replayer = make_replayer(folder, dtype, max_tokens=64, page=16)
        check_logits(replay_one(replayer, "a", tokens, [30, 1, 1, 18]), ref, dtype, "values from keys")
    W = mc.as_numpy(tensors)
    h = plain.mixer_input(W["embed"][np.asarray(tokens)], W, "l0.", cfg["norm"]["eps"])
    m = cfg["layers"][0]["mixer"]["left"]
    right = plain.key_value_attention(h, W, "l0.mix.left.", m)
    # the same with the rotated keys as values
    T, H, G, D = len(tokens), m["heads"], m["kv_heads"], m["dim"]
    q = plain.rotate_halves((h @ W["l0.mix.left.q"].T + W["l0.mix.left.q.b"]).reshape(T, H, D), m["rot"], np.arange(T))
    k = plain.rotate_halves((h @ W["l0.mix.left.k"].T + W["l0.mix.left.k.b"]).reshape(T, G, D), m["rot"], np.arange(T))
    k = np.repeat(k, H // G, axis=1)
    scores = np.einsum("thd,shd->hts", q, k) * m["scale"]
    wrong = plain.attend(scores, plain.window_mask(T, m["mask"]["size"]), k.transpose(1, 0, 2))
    wrong = wrong.transpose(1, 0, 2).reshape(T, H * D) @ W["l0.mix.left.o"].T
    assert np.abs(right - wrong).max() > 0.05, "rotated or unrotated values make no difference in this test"


def test_command_lines_take_the_design(tmp_path, capsys):
    import json

    from velox_b200.cli import benchmark, roofline

    common = ["--model-size", "tiny-m", "--num-requests", "5", "--max-tokens", "10", "--max-model-len", "128",
              "--max-num-seqs", "4", "--max-num-batched-tokens", "64", "--max-prefill-chunk-size", "16",
              "--block-size", "8", "--workload", "short", "--seed", "3"]
    assert benchmark.main(common + ["--temperature", "0"]) == 0
    assert "decode throughput" in capsys.readouterr().out
    assert benchmark.main(common + ["--temperature", "0.7", "--top-k", "10", "--no-pipeline"]) == 0
    capsys.readouterr()
    table = tmp_path / "roofline.json"
    assert roofline.main(["--model-size", "tiny-m", "--batch", "2", "--context", "40", "--layers", "3,6", "--steps", "4",
                          "--warmup", "1", "--block-size", "8", "--output-json", str(table)]) == 0
    rows = json.loads(table.read_text())
    assert rows[0]["us_per_layer"] > 0 and rows[0]["size"] == "tiny-m"


@pytest.mark.parametrize("case", ["small", "odd", "taps"])
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
