"""Each new kernel by itself against the plain functions of tests/plain/sarulix_plain.py (float64 on the CPU)."""
import math

import pytest
import torch

from tests.plain import sarulix_plain as plain

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DEV = "cuda:0"


def rnd(shape, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def close(got, want, tol):
    err = float((got.double().cpu() - want.double()).abs().max() / want.double().abs().max())
    assert err < tol, err


def two_steps(lens_first, lens_second):
    """Three sequences in slots 2, 0, 3 and, in the middle of the list, one without tokens and without a slot."""
    for step, lens in enumerate((lens_first, lens_second)):
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        cu = cu[:2] + cu[1:2] + cu[2:]
        yield step, lens, torch.tensor(cu, dtype=torch.int32, device=DEV), torch.tensor([2, -1, 0, 3], dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("lens_first,lens_second", [([5, 1, 9], [1, 2, 30]), ([70, 2, 1], [3, 90, 1])])
@pytest.mark.parametrize("taps,act", [(4, "none"), (2, "silu"), (1, "none"), (7, "silu")])
def test_short_conv_reads_the_last_inputs_of_the_step_before(taps, act, dtype, lens_first, lens_second):
    """Portions shorter and longer than the taps, a second step after the first, slots nobody owns left alone, rows
    beyond the sequences untouched; steps of a few tokens (one launch) and of more (the state brought up to date by a
    launch of its own)."""
    from llmgen_b200.kernels import ops
    C = 40
    w, cb, ib = rnd((C, taps), 1, 0.5), rnd((C,), 2, 0.3), rnd((C,), 3, 0.3)
    seqs = [rnd((a + b, C + 3), 10 + i, 1.0, DT[dtype]) for i, (a, b) in enumerate(zip(lens_first, lens_second))]
    state = torch.zeros(4, 11 + (taps - 1) * C, device=DEV)
    state[1] = 7.0
    outs = [[], [], []]
    for step, lens, cu, sl in two_steps(lens_first, lens_second):
        rows = torch.cat([s[:n] if step == 0 else s[lens_first[i]:] for i, (s, n) in enumerate(zip(seqs, lens))] + [seqs[0][:2]]).to(DEV)
        out = torch.full((rows.shape[0], C), float("nan"), device=DEV)
        ops.short_conv(out, rows[:, 3:], w.to(DEV), state[:, 11:], cu, sl, 4, in_bias=ib.to(DEV), conv_bias=cb.to(DEV), activation=act)
        assert bool(out[-2:].isnan().all())                       # rows that belong to no sequence
        at = 0
        for i, n in enumerate(lens):
            outs[i].append(out[at:at + n].cpu())
            at += n
    for i, s in enumerate(seqs):
        x = s.double()[:, 3:] + ib.double()
        want = plain.causal_conv(x, w.double(), cb.double())
        if act == "silu":
            want = plain.silu(want)
        close(torch.cat(outs[i]), want, 1e-5)
        if taps > 1:
            history = torch.cat([torch.zeros(taps - 1, C, dtype=torch.float64), x])[-(taps - 1):]      # zeros before the start
            close(state[[2, 0, 3][i], 11:].view(taps - 1, C), history, 1e-6)
    assert bool((state[1] == 7.0).all()) and bool((state[:, :11][[0, 2, 3]] == 0).all())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("lens_first,lens_second", [([37, 1, 64], [1, 30, 3]), ([300, 1, 530], [257, 3, 350])])
@pytest.mark.parametrize("C,blocks", [(48, 3), (36, 1), (160, 2), (20, 4)])
def test_rglru_kernels_carry_their_state_between_calls(C, blocks, dtype, lens_first, lens_second):
    """Three sequences, two steps each; the long steps of the bfloat16 engine scan in segments that run side by side."""
    from llmgen_b200.kernels import ops
    n = C // blocks
    wa, wi = rnd((blocks, n, n), 1, 0.3, DT[dtype]), rnd((blocks, n, n), 2, 0.3, DT[dtype])
    ba, bi, lam, yb = rnd((C,), 3, 0.5), rnd((C,), 4, 0.5), rnd((C,), 5, 2.0) - 3.0, rnd((C,), 6, 0.3)
    us = [rnd((a + b, C), 10 + i) for i, (a, b) in enumerate(zip(lens_first, lens_second))]
    ys = [rnd((a + b, C + 8), 20 + i, 1.0, DT[dtype]) for i, (a, b) in enumerate(zip(lens_first, lens_second))]
    state = torch.zeros(4, C + 5, device=DEV)
    state[1] = 7.0
    outs = [[], [], []]
    for step, lens, cu, sl in two_steps(lens_first, lens_second):
        cut = [(0, m) if step == 0 else (lens_first[i], lens_first[i] + m) for i, m in enumerate(lens)]
        u = torch.cat([x[a:b] for x, (a, b) in zip(us, cut)]).to(DEV).contiguous()
        y = torch.cat([x[a:b] for x, (a, b) in zip(ys, cut)]).to(DEV)
        T = u.shape[0]
        out = torch.full((T, C), float("nan"), device=DEV, dtype=DT[dtype])
        rows = ops.rglru_scratch_rows(T, 4, DT[dtype])
        assert (rows > 2 * T) == (dtype == "bfloat16" and T >= 512)
        ops.rglru(out, torch.full((rows, C), float("nan"), device=DEV), u, wa.to(DEV), wi.to(DEV), ba.to(DEV), bi.to(DEV), lam.to(DEV),
                  y[:, :C], yb.to(DEV), state, cu, sl, 4, blocks, 8.0)
        at = 0
        for i, m in enumerate(lens):
            outs[i].append(out[at:at + m].float().cpu())
            at += m
    for i, (u, y) in enumerate(zip(us, ys)):
        T = u.shape[0]
        ub = u.double().view(T, blocks, n)
        r = plain.sigmoid(torch.einsum("tbi,boi->tbo", ub, wa.double()) + ba.double().view(blocks, n)).reshape(T, C)
        ig = plain.sigmoid(torch.einsum("tbi,boi->tbo", ub, wi.double()) + bi.double().view(blocks, n)).reshape(T, C)
        S = plain.rglru_scan(u.double(), r, ig, lam.double())
        want = S * plain.gelu_tanh(y.double()[:, :C] + yb.double())
        close(torch.cat(outs[i]), want, 2e-5 if dtype == "float32" else 1e-2)
        close(state[[2, 0, 3][i], :C], S[-1], 2e-5)
    assert bool((state[1] == 7.0).all())


def test_rglru_keeps_a_decay_just_below_one_over_thousands_of_tokens():
    """lam far below zero: a = 1 - 1e-4 or so.  Held as a float, a itself would be a few parts in 1e4 off in what
    matters, 1 - a; the state after 3,000 tokens shows it."""
    from llmgen_b200.kernels import ops
    C, T = 16, 3000
    wa, wi = torch.zeros(1, C, C), torch.zeros(1, C, C)
    lam = torch.full((C,), -9.0) + rnd((C,), 1, 0.5)
    u, y = rnd((T, C), 2) + 1.0, torch.ones(T, C) * 3.0
    state = torch.zeros(1, C, device=DEV)
    cu, sl = torch.tensor([0, T], dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV)
    half = torch.full((T, C), 0.5, dtype=torch.float64)
    S = plain.rglru_scan(u.double(), half, half, lam.double())
    for dt in (torch.float32, torch.bfloat16):                 # a thread per channel; segments side by side
        state.zero_()
        out = torch.empty(T, C, device=DEV, dtype=dt)
        ops.rglru(out, torch.empty(ops.rglru_scratch_rows(T, 1, dt), C, device=DEV), u.to(DEV), wa.to(DEV, dt), wi.to(DEV, dt), None, None,
                  lam.to(DEV), y.to(DEV, dt), None, state, cu, sl, 1, 1, 8.0)
        close(state[0], S[-1], 3e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,E", [(4, 2, 16, 24), (1, 1, 10, 6), (6, 2, 40, 72), (2, 2, 128, 64), (3, 1, 136, 8)])
def test_delta_scan_carries_its_state_between_calls(H, G, D, E, dtype):
    from llmgen_b200.kernels import ops
    lens_first, lens_second = [37, 1, 20], [1, 18, 3]
    width = 2 * G * D + H * E
    qkvs = [rnd((a + b, width + 4), 10 + i, 0.8) for i, (a, b) in enumerate(zip(lens_first, lens_second))]
    betas = [rnd((a + b, H + 2), 20 + i, 1.0, DT[dtype]) for i, (a, b) in enumerate(zip(lens_first, lens_second))]
    decays = [rnd((a + b, H * D), 30 + i, 1.0) for i, (a, b) in enumerate(zip(lens_first, lens_second))]
    dt_bias, a_log = rnd((H * D,), 40, 1.0) - 2.0, rnd((H,), 41, 0.5)
    state = torch.zeros(4, H * D * E + 7, device=DEV)
    state[1] = 7.0
    outs = [[], [], []]
    for step, lens, cu, sl in two_steps(lens_first, lens_second):
        cut = [(0, m) if step == 0 else (lens_first[i], lens_first[i] + m) for i, m in enumerate(lens)]
        cat = lambda xs: torch.cat([x[a:b] for x, (a, b) in zip(xs, cut)]).to(DEV)
        qkv, beta, decay = cat(qkvs), cat(betas), cat(decays).contiguous()
        out = torch.full((qkv.shape[0], H * E), float("nan"), device=DEV)
        ops.delta_scan(out, qkv[:, 4:], beta[:, 1:1 + H], decay, dt_bias.to(DEV), a_log.to(DEV), state, cu, sl, 4, H, G, D, E, 1e-6, D ** -0.5,
                       beta_buf=torch.empty(qkv.shape[0], H + G, device=DEV))
        at = 0
        for i, m in enumerate(lens):
            outs[i].append(out[at:at + m].cpu())
            at += m
    for i in range(3):
        x = qkvs[i].double()[:, 4:]
        T = x.shape[0]
        q, k, v = x[:, :G * D].view(T, G, D), x[:, G * D:2 * G * D].view(T, G, D), x[:, 2 * G * D:].view(T, H, E)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        beta = plain.sigmoid(betas[i].double()[:, 1:1 + H])
        g = torch.exp(-torch.exp(a_log.double())[None, :, None] * plain.softplus(decays[i].double() + dt_bias.double()).view(T, H, D))
        want = plain.gated_delta_scan(q, k, v, beta, g)
        close(torch.cat(outs[i]), want.reshape(T, H * E), 2e-5)
    assert bool((state[1] == 7.0).all())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,E,softcap,gate", [(4, 2, 16, 24, 15.0, True), (3, 3, 8, 8, 0.0, False), (8, 1, 32, 16, 5.0, True),
                                                  (2, 1, 64, 128, 0.0, True), (4, 2, 128, 128, 20.0, True), (2, 2, 64, 64, 6.0, False),
                                                  (3, 1, 128, 64, 0.0, True)])
def test_attention_with_a_sink_a_bound_a_gate_and_values_of_their_own_width(H, G, D, E, softcap, gate, dtype):
    """Two sequences, the second with keys of an earlier step in shuffled pages; biases added by the preparation kernel;
    the same rows through one launch, through key parts that are merged afterwards and, in bfloat16 at the widths it
    takes, through the tensor-core kernel with float32 weights."""
    from llmgen_b200.kernels import ops
    page, scale = 16, 0.3
    lens, starts = [21, 9], [0, 40]
    dt = DT[dtype]
    tol = 2e-5 if dtype == "float32" else 3e-2
    n_pages = 12
    kc = torch.zeros(n_pages, G, page, D, device=DEV, dtype=dt)
    vc = torch.zeros(n_pages, G, page, E, device=DEV, dtype=dt)
    tables = torch.tensor([[3, 7, 0, 0], [5, 1, 9, 2]], dtype=torch.int32, device=DEV)
    width = H * D + G * D + G * E
    bias = rnd((width,), 3, 0.2)
    gq, gk = 1.0 + rnd((D,), 4, 0.1), 1.0 + rnd((D,), 5, 0.1)
    seqs = [rnd((starts[i] + lens[i], width), 10 + i, 1.0, dt) for i in range(2)]
    gates = [rnd((starts[i] + lens[i], H * E), 20 + i, 1.0, dt) for i in range(2)]

    def prep(rows, positions, slots):
        q = torch.empty(rows.shape[0], H * D, device=DEV, dtype=dt)
        ops.attn_prep(rows.to(DEV), kc, vc, torch.tensor(positions, dtype=torch.int32, device=DEV),
                      torch.tensor(slots, dtype=torch.int32, device=DEV), None, None, gq.to(DEV), gk.to(DEV), H, G, D, 0, page, 1e-5,
                      q_out=q, bias=bias.to(DEV), vd=E)
        return q

    slot_of = lambda s, p: int(tables[s, p // page]) * page + p % page
    prep(seqs[1][:40], list(range(40)), [slot_of(1, p) for p in range(40)])          # the earlier step of the second sequence
    rows = torch.cat([seqs[0], seqs[1][40:]])
    positions = list(range(21)) + list(range(40, 49))
    q = prep(rows, positions, [slot_of(0, p) for p in range(21)] + [slot_of(1, p) for p in range(40, 49)])
    g = torch.cat([gates[0], gates[1][40:]]).to(DEV) if gate else None
    bq = ops.attention_tile_queries(H, G)
    tiles = [(s, q0) for s in range(2) for q0 in range(0, lens[s], bq)]
    tile_seq = torch.tensor([t[0] for t in tiles], dtype=torch.int32, device=DEV)
    tile_q0 = torch.tensor([t[1] for t in tiles], dtype=torch.int32, device=DEV)
    ctx = torch.tensor([21, 49], dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, 21, 30], dtype=torch.int32, device=DEV)
    results = []
    for parts in (1, 3):
        out = torch.full((30, H * E), float("nan"), device=DEV, dtype=dt)
        scratch = torch.empty(ops.attention_scratch_floats(30, H, E, parts), device=DEV) if parts > 1 else None
        ops.paged_attention(out, q, q.stride(0), kc, vc, tables.view(-1), 4, ctx, cu, tile_seq, tile_q0, len(tiles), 30, H, G, D, page, 0,
                            scale, parts, 0, scratch, vd=E, softcap=softcap, sink=True, gate=g)
        results.append(out.float().cpu())
    mma_bq = ops.attention_mma_tile_queries(H, G, D, E) if dtype == "bfloat16" else 0
    assert (mma_bq > 0) == (dtype == "bfloat16" and D in (64, 128) and E in (64, 128))
    if mma_bq:
        mt = [(s, q0) for s in range(2) for q0 in range(0, lens[s], mma_bq)] + [(-1, 0)]
        out = torch.full((30, H * E), float("nan"), device=DEV, dtype=dt)
        ops.attention_mma(out, q, kc, vc, tables.view(-1), 4, ctx, cu, torch.tensor([t[0] for t in mt], dtype=torch.int32, device=DEV),
                          torch.tensor([t[1] for t in mt], dtype=torch.int32, device=DEV), len(mt), H, G, D, E, page, 0, scale,
                          softcap=softcap, sink=True, gate=g)
        results.append(out.float().cpu())
    at = 0
    for s in range(2):
        x = seqs[s].double() + bias.double()
        T = x.shape[0]
        qq = plain.rms_norm(x[:, :H * D].view(T, H, D), gq.double(), 1e-5)
        kk = plain.rms_norm(x[:, H * D:H * D + G * D].view(T, G, D), gk.double(), 1e-5)
        vv = x[:, H * D + G * D:].view(T, G, E)
        if dtype == "bfloat16":        # what the cache holds
            qq, kk, vv = (t.to(torch.bfloat16).double() for t in (qq, kk, vv))
        want = plain.sink_softmax_attention(qq, kk, vv, scale, softcap).reshape(T, H * E)
        if gate:
            want = want * plain.sigmoid(gates[s].double())
        want = want[starts[s]:]
        for got in results:
            close(got[at:at + lens[s]], want, tol)
        at += lens[s]
    # the sink is there: the first token's weights do not sum to one
    x0 = seqs[0].double()[:1] + bias.double()
    v0 = x0[:, H * D + G * D:].view(1, G, E)
    first = results[0][0].double().view(H, E) / (plain.sigmoid(gates[0].double()[0]).view(H, E) if gate else 1.0)
    ratio = first[0] / v0[0, 0]
    assert float(ratio.mean()) < 0.999


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_small_row_kernels(dtype):
    """gelu(gate) * up from an array and from slices, a bias on an array and on slices, the operand of the stream's
    re-entry, the factor on the logits."""
    from llmgen_b200.kernels import ops
    dt = DT[dtype]
    n, F = 7, 40
    x = rnd((n, 2 * F), 1, 2.0, dt)
    want = plain.gelu_tanh(x.double()[:, :F]) * x.double()[:, F:]
    out = torch.empty(n, F, device=DEV, dtype=dt)
    ops.act_rows(out, x.to(DEV), "gelu_tanh_glu")
    close(out.float(), want, 1e-5 if dtype == "float32" else 1e-2)
    parts = rnd((3, n, 2 * F), 2, 1.0)
    ops.act_rows(out, ops.Partials(parts.to(DEV).contiguous()), "gelu_tanh_glu")
    s = parts.double().sum(0)
    close(out.float(), plain.gelu_tanh(s[:, :F]) * s[:, F:], 1e-5 if dtype == "float32" else 1e-2)
    b = rnd((F,), 3)
    y = rnd((n, F), 4, 1.0, dt).to(DEV)
    want = y.double().cpu() + b.double()
    ops.add_bias(y, b.to(DEV))
    close(y.float(), want, 1e-6 if dtype == "float32" else 1e-2)
    p = ops.Partials(rnd((2, n, F), 5).to(DEV).contiguous())
    want = p.sum().double().cpu() + b.double()
    ops.add_bias(p, b.to(DEV))
    close(p.sum(), want, 1e-6)
    resid, delta, x0 = rnd((n, F), 6).to(DEV), rnd((n, F), 7, 1.0, dt).to(DEV), rnd((n, F), 8).to(DEV)
    both = torch.empty(n, 2 * F, device=DEV, dtype=dt)
    ops.concat_stream(both, resid, delta, x0)
    close(both.float(), torch.cat([resid.double().cpu() + delta.double().cpu(), x0.double().cpu()], dim=1), 1e-6 if dtype == "float32" else 1e-2)
    ops.concat_stream(both, resid, None, x0)
    close(both.float()[:, :F], resid.double().cpu(), 1e-6 if dtype == "float32" else 1e-2)
    logits = rnd((3, 11), 9, 5.0).to(DEV)
    want = 0.7 * logits.double().cpu()
    ops.logit_cap(logits, 0.0, 0.7)
    close(logits, want, 1e-6)
    ops.logit_cap(logits, 2.0, 1.0)
    close(logits, 2.0 * torch.tanh(want / 2.0), 1e-6)


def test_gelu_in_the_tiled_product_s_gated_epilogue_and_over_grouped_columns():
    """gate and up rows interleaved in groups of 16: the tensor-core product with gelu_tanh(gate) * up in its epilogue,
    and the pass over the packed product that few rows take, against the plain function."""
    from llmgen_b200.kernels import ops
    from llmgen_b200.parts.mlp import interleave_gate_up
    M, K, F = 200, 64, 96
    x = rnd((M, K), 1, 1.0, torch.bfloat16)
    wg, wu = rnd((F, K), 2, 0.3, torch.bfloat16), rnd((F, K), 3, 0.3, torch.bfloat16)
    want = plain.gelu_tanh(x.double() @ wg.double().t()) * (x.double() @ wu.double().t())
    w = interleave_gate_up(wg, wu).contiguous().to(DEV)
    out = torch.empty(M, F, device=DEV, dtype=torch.bfloat16)
    ops.gemm_tc(out, x.to(DEV), w, gated=True, activation="gelu_tanh")
    close(out.float(), want, 1e-2)
    silu = torch.empty(M, F, device=DEV, dtype=torch.bfloat16)
    ops.gemm_tc(silu, x.to(DEV), w, gated=True)                 # the default stays silu
    g = x.double() @ wg.double().t()
    close(silu.float(), g / (1 + torch.exp(-g)) * (x.double() @ wu.double().t()), 1e-2)
    packed = torch.empty(M, 2 * F, device=DEV, dtype=torch.bfloat16)
    ops.gemm_tc(packed, x.to(DEV), w)
    ops.act_rows(out, packed, "gelu_tanh_glu", group=16)
    close(out.float(), want, 1e-2)
