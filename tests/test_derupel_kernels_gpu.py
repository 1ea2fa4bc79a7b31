"""Each new kernel by itself against the plain functions of tests/plain/derupel_plain.py (float64 on the CPU)."""
import pytest
import torch

from tests.plain import derupel_plain as plain

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def rnd(shape, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def close(got, want, tol):
    err = float((got.double().cpu() - want.double()).abs().max() / want.double().abs().max())
    assert err < tol, err


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("lens_first,lens_second", [([37, 1, 64], [1, 30, 3]), ([300, 1, 530], [257, 3, 1])])
@pytest.mark.parametrize("heads,dim,vdim", [(2, 16, 24), (3, 72, 80), (1, 128, 32)])
def test_linear_attention_kernel_carries_its_state_between_calls(heads, dim, vdim, dtype, lens_first, lens_second):
    """Three sequences, two steps each, in slots 2, 0, 3; the longer steps are cut into segments that run side by side."""
    from llmgen_b200.kernels import ops
    dev = "cuda:0"
    slots = [2, 0, 3]
    decay = [1.0, 0.9, 0.5][:heads]
    width = heads * (2 * dim + vdim) + 8                        # some columns the kernel must skip
    state = torch.zeros(4, heads, dim, vdim, device=dev)
    state[1] = 7.0                                              # a slot nobody owns stays as it is
    seqs = [rnd((a + b, width), 10 + i, 0.7, DT[dtype]) for i, (a, b) in enumerate(zip(lens_first, lens_second))]
    outs = [[], [], []]
    for step, lens in enumerate((lens_first, lens_second)):
        rows = torch.cat([s[:n] if step == 0 else s[lens_first[i]:] for i, (s, n) in enumerate(zip(seqs, lens))]).to(dev)
        cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
        # a sequence without tokens and without a slot in the middle of the list is skipped
        cu = torch.cat([cu[:2], cu[1:2], cu[2:]])
        sl = torch.tensor([slots[0], -1, slots[1], slots[2]], dtype=torch.int32, device=dev)
        out = torch.full((rows.shape[0], heads * vdim), float("nan"), device=dev)
        need = ops.linear_attention_scratch_floats(rows.shape[0], 4, heads, dim, vdim)
        assert (need > 0) == (rows.shape[0] > 256)
        scratch = torch.full((need,), float("nan"), device=dev) if need else None
        ops.linear_attention(out, rows, 0, heads * dim, 2 * heads * dim, state, torch.tensor(decay, device=dev), cu, sl, 4,
                             heads, dim, vdim, silu=True, scratch=scratch)
        at = 0
        for i, n in enumerate(lens):
            outs[i].append(out[at:at + n].cpu())
            at += n
    for i, s in enumerate(seqs):
        x = s.double()
        T = x.shape[0]
        q = plain.silu(x[:, :heads * dim]).view(T, heads, dim)
        k = plain.silu(x[:, heads * dim:2 * heads * dim]).view(T, heads, dim)
        v = plain.silu(x[:, 2 * heads * dim:2 * heads * dim + heads * vdim]).view(T, heads, vdim)
        want, final = plain.decayed_outer_product_scan(q, k, v, decay)
        close(torch.cat(outs[i]), want.reshape(T, -1), 2e-5)
        close(state[slots[i]], final, 2e-5)
    assert bool((state[1] == 7.0).all())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rowwise_kernels(dtype):
    from llmgen_b200.kernels import ops
    dev, dt = "cuda:0", DT[dtype]
    n, H, F = 9, 72, 40
    tol = 1e-5 if dtype == "float32" else 1e-2
    resid, y, w = rnd((n, H), 1, 3.0), rnd((n, H), 2, 0.5, dt), 1 + rnd((H,), 3, 0.2)
    r, copy = resid.to(dev), torch.empty(n, H, dtype=dt, device=dev)
    ops.norm_add(r, y.to(dev), w.to(dev), 1e-5, copy, dt)
    want = resid.double() + plain.rms_norm(y.double(), w.double(), 1e-5)
    close(r, want, 1e-5)
    close(copy, want, tol)
    # the same from three float32 slices
    parts = rnd((3, n, H), 4, 0.5)
    r = resid.to(dev)
    ops.norm_add(r, ops.Partials(parts.to(dev)), w.to(dev), 1e-5, None, dt)
    close(r, resid.double() + plain.rms_norm(parts.double().sum(0), w.double(), 1e-5), 1e-5)
    x = rnd((n, F), 5, 1.0, dt)
    out = torch.empty(n, F, dtype=dt, device=dev)
    ops.act_rows(out, x.to(dev), "relu2")
    close(out, torch.relu(x.double()) ** 2, tol)
    gu = rnd((n, 2 * F), 6, 1.5, dt)
    ops.act_rows(out, gu.to(dev), "clamped_glu", alpha=1.702, limit=0.9)
    g = torch.clamp(gu[:, :F].double(), max=0.9)
    u = torch.clamp(gu[:, F:].double(), min=-0.9, max=0.9)
    close(out, g * plain.sigmoid(1.702 * g) * (u + 1), tol)
    o, gate = rnd((n, H), 7, 2.0), rnd((n, H + 16), 8, 1.0, dt)
    out = torch.empty(n, H, dtype=dt, device=dev)
    ops.gated_rmsnorm(out, o.to(dev), gate.to(dev)[:, 16:], w.to(dev), 1e-5)
    close(out, plain.rms_norm(o.double(), w.double(), 1e-5) * plain.sigmoid(gate[:, 16:].double()), tol)


@pytest.mark.parametrize("top,shared", [(1, False), (2, True), (3, False)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_feed_forward_matches_the_plain_one(dtype, top, shared):
    """The part itself on rows of its own: routing, grouping into tiles (some experts get no row, one gets more than a
    tile), both products, the shared expert, the sum."""
    from llmgen_b200.engine.context import Workspace
    from llmgen_b200.parts.moe import RoutedMLP
    from llmgen_b200.parts.registry import model_weight_decls  # noqa: F401  (registers the parts)
    from llmgen_b200.parts.spec import ClampedExpertSpec, RoutedMLPSpec
    from llmgen_b200.weights import random_tensors, weights_from_dict
    dev, dt = torch.device("cuda:0"), DT[dtype]
    H, E, F, T = 40, 7, 24, 90
    ex = lambda p, ff, lim: ClampedExpertSpec(ff, lim, p + "gate", p + "up", p + "down")
    spec = RoutedMLPSpec(H, "mlp.router", tuple(ex(f"mlp.e{j}.", F, 0.7) for j in range(E)), top,
                         shared=ex("mlp.shared.", 32, 1.1) if shared else None)
    decls = RoutedMLP.weight_decls(spec)
    tensors = random_tensors(decls, 5, 0.2, 0.1, torch.bfloat16)
    tensors["mlp.router"][2] = 0                # expert 2 scores 1/2 everywhere
    tensors["mlp.router"][5] *= 6               # expert 5 is chosen by about half of the rows: more than one tile
    part = RoutedMLP(spec, weights_from_dict(tensors, decls), dt, dev)

    class Ctx:
        workspace = Workspace(dev, 128)
    x = rnd((T, H), 9, 1.0, dt)
    got = part.forward(Ctx, x.to(dev)).sum()
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": F, "limit": 0.7}}
    if shared:
        mlp["shared"] = {"ff": 32, "limit": 1.1}
    want = plain.routed_ff(x.double(), {k: v.double() for k, v in tensors.items()}, "mlp.", mlp)
    close(got, want, 2e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,rot,vdim,rank", [(3, 16, 8, 24, 32), (17, 8, 4, 8, 16), (2, 24, 0, 16, 40),
                                                     (3, 16, 16, 24, 64), (17, 8, 32, 8, 128), (6, 8, 64, 16, 512),
                                                     (40, 8, 4, 8, 16), (34, 8, 16, 8, 64),      # more heads than a block has rows
                                                     (2, 8, 16, 8, 192), (2, 8, 0, 8, 256), (1, 16, 32, 8, 320)])
def test_latent_attention_kernels_match_the_plain_mixer(heads, dim, rot, vdim, rank, dtype):
    """prep, absorb, attention (whole, and a step of single tokens cut into key parts) and expand, on one sequence whose
    pages lie in shuffled order, against keys and values expanded per head."""
    from llmgen_b200.kernels import ops
    dev, dt = "cuda:0", DT[dtype]
    T, page, q_rank, eps, base = 77, 16, 24, 1e-5, 200.0
    scale = 0.4 / (rank / 32) ** 0.5          # scores of a few units whatever the latent's width
    za = rank + rot
    w = {"dq": rnd((q_rank, 32), 1, 0.3, dt), "dq.norm": 1 + rnd((q_rank,), 2, 0.2), "uq": rnd((heads * (dim + rot), q_rank), 3, 0.3, dt),
         "dkv": rnd((za, 32), 4, 0.3, dt), "dkv.norm": 1 + rnd((rank,), 5, 0.2), "uk": rnd((heads * dim, rank), 6, 0.3, dt),
         "uv": rnd((heads * vdim, rank), 7, 0.3, dt), "g": rnd((heads * vdim, 32), 8, 0.3, dt), "o": torch.eye(heads * vdim)}
    h = rnd((T, 32), 9, 1.0, dt)
    m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": {"base": base, "dims": rot}}
    want = plain.latent_attention_mixer(h.double(), {"m." + k: v.double() for k, v in w.items()}, "m.", m, eps, range(T))
    # the engine's side: the three input products by torch in float32, the rest by the kernels
    hd = h.float()
    packed = torch.cat([hd @ w["dq"].float().t(), hd @ w["dkv"].float().t(), hd @ w["g"].float().t()], dim=1).to(dt).to(dev)
    table = [4, 0, 3, 1, 2]
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    slots = torch.tensor([table[p // page] * page + p % page for p in range(T)], dtype=torch.int32, device=dev)
    inv = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)] or [0.0], dtype=torch.float64)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * inv[None, :]
    cos, sin = ang.cos().float().to(dev).contiguous(), ang.sin().float().to(dev).contiguous()
    cache = torch.zeros(5, 1, page, za, dtype=dt, device=dev)
    cq = torch.empty(T, q_rank, dtype=dt, device=dev)
    ops.latent_prep(packed, 0, q_rank, q_rank, rank, rot, w["dq.norm"].to(dev), w["dkv.norm"].to(dev), eps, cq, cache, pos, slots,
                    cos, sin, "interleaved")
    q = (cq.float() @ w["uq"].float().to(dev).t()).to(dt)
    qa = torch.empty(T, heads * za, device=dev)
    ops.latent_absorb(qa, q, w["uk"].to(dev), pos, cos, sin, heads, dim, rot, rank, "interleaved")
    bq = ops.latent_attention_tile_queries(heads)
    tiles = list(range(0, T, bq))
    dev_i = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    oa = torch.empty(T, heads * rank, device=dev)
    ops.latent_attention(oa, qa, cache, dev_i(table), 5, dev_i([T]), dev_i([0, T]), dev_i([0] * len(tiles)), dev_i(tiles), T, heads,
                         rank, rot, page, scale)
    y = torch.empty(T, heads * vdim, dtype=dt, device=dev)
    ops.latent_expand(y, oa, w["uv"].to(dev), packed[:, q_rank + za:], heads, rank, vdim)
    tol = 3e-5 if dtype == "float32" else 3e-2
    close(y, want, tol)
    # the last token alone, as a step of single tokens, its keys cut into 3 parts
    parts = 3
    scratch = torch.empty(ops.latent_attention_scratch_floats(1, heads, rank, parts), device=dev)
    o1 = torch.empty(1, heads * rank, device=dev)
    ops.latent_attention(o1, qa[T - 1:], cache, dev_i(table), 5, dev_i([T]), dev_i([0, 1]), dev_i([0]), dev_i([0]), 1, heads, rank, rot,
                         page, scale, parts, scratch)
    close(o1, oa[T - 1:].cpu(), 1e-5)
    if dtype == "bfloat16" and (rank + rot) % 16 == 0 and rank % 64 == 0:
        # these sizes went through the tensor cores: the float32 kernel on the same cache and queries differs only by
        # the rounding of the queries to bfloat16 (the weights enter the second product as three exact terms)
        ops.latent_attention_set_mma(False)
        try:
            ref = torch.empty_like(oa)
            ops.latent_attention(ref, qa, cache, dev_i(table), 5, dev_i([T]), dev_i([0, T]), dev_i([0] * len(tiles)), dev_i(tiles), T,
                                 heads, rank, rot, page, scale)
        finally:
            ops.latent_attention_set_mma(True)
        # the same result head-major in bfloat16 (what the grouped product over the heads reads), whole and from key parts
        t_pad = 128
        hm = torch.zeros(heads, t_pad, rank, dtype=torch.bfloat16, device=dev)
        ops.latent_attention(None, qa, cache, dev_i(table), 5, dev_i([T]), dev_i([0, T]), dev_i([0] * len(tiles)), dev_i(tiles), T, heads,
                             rank, rot, page, scale, out_head_major=hm)
        close(hm[:, :T].permute(1, 0, 2).reshape(T, heads * rank).float(), oa.cpu(), 1e-2)
        hm1 = torch.zeros(heads, t_pad, rank, dtype=torch.bfloat16, device=dev)
        ops.latent_attention(None, qa[T - 1:], cache, dev_i(table), 5, dev_i([T]), dev_i([0, 1]), dev_i([0]), dev_i([0]), 1, heads, rank, rot,
                             page, scale, parts, scratch, out_head_major=hm1)
        close(hm1[:, 0].reshape(1, heads * rank).float(), oa[T - 1:].cpu(), 1e-2)
        close(oa, ref.cpu(), 5e-2)             # scores of some tens here: a bfloat16 rounding of q moves a weight by a few per cent
        assert float((oa - ref).abs().max()) > 0
