"""The Lulisun decoder in the engine against the plain restatement (`plain_lulisun`): each
mechanism's kernel alone, then whole models: prompts whole, token by token, in portions down to two
tokens, unequal batches, slots and pages used again, keys at the edges of chunks and pages, long
decoding, and greedy generation through `Model.generate`."""
import math

import pytest
import torch

import lulisun_models
import plain_lulisun
from conftest import random_tokens, rel_err

# Worst row's max |a - b| / max |b| against the plain model in float64.  float32 runs: a kernel fault shows
# far above 1e-4.  bfloat16 runs keep bfloat16 activations between kernels through four layer runs of two
# mixers and up to four expert products each, on weights drawn hot (unit-variance streams): rounding
# alone reaches 5e-2 on single rows; a key too many, a lost state or a wrong expert costs 0.3 and more.
TOL = {"float32": 1e-4, "bfloat16": 8e-2}

pytestmark = pytest.mark.gpu

DEV = "cuda"


def d(t, dtype=None):
    return t.to(device=DEV, dtype=dtype or t.dtype).contiguous()


# ---------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("experts,top,groups,keep", [(12, 3, 3, 2), (16, 3, 4, 2), (6, 2, 6, 3), (5, 1, 1, 1), (64, 6, 8, 3)])
@pytest.mark.parametrize("negative", [False, True])
def test_router_choice_and_weights(experts, top, groups, keep, negative):
    """ids and weights of the route kernel equal the plain router's; with `negative` all choice scores lie
    below zero, where a removed group whose scores were merely zeroed would win."""
    from rust_inference_b200.kernels import ops
    g = torch.Generator().manual_seed(experts * 7 + top)
    n, width = 37, 48
    x = torch.randn(n, width, generator=g)
    w = {"r.router": torch.randn(experts, width, generator=g) * 0.6,
         "r.correction": torch.randn(experts, generator=g) * 0.4 - (3.0 if negative else 0.0)}
    sg = torch.randn(width, generator=g) * 0.3
    ids_p, wts_p, _ = plain_lulisun.route(x.double(), {k: v.double() for k, v in w.items()}, "r.", experts=experts,
                                          top=top, groups=groups, keep=keep)
    ids = torch.zeros(n, top, dtype=torch.int32, device=DEV)
    wts = torch.zeros(n, top, dtype=torch.float32, device=DEV)
    gate = torch.zeros(n, dtype=torch.float32, device=DEV)
    ops.moe_route(d(x), d(w["r.router"]), d(w["r.correction"]), ids, wts, top=top, groups=groups, keep=keep,
                  gate_weight=d(sg), gate_out=gate)
    order = ids.cpu().long().sort(dim=1)
    order_p = ids_p.sort(dim=1)
    assert torch.equal(order.values, order_p.values)
    got = torch.gather(wts.cpu(), 1, order.indices)
    want = torch.gather(wts_p, 1, order_p.indices).float()
    assert float((got - want).abs().max()) < 1e-5
    assert float((gate.cpu() - torch.sigmoid(x.double() @ sg.double()).float()).abs().max()) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,ff,width,n", [(6, 2, 20, 72, 50), (5, 1, 24, 128, 3), (12, 3, 48, 128, 131)])
def test_grouped_expert_products(dtype, experts, top, ff, width, n):
    """arrange + the two grouped products + the weighted sum against a loop over tokens and choices."""
    from rust_inference_b200.kernels import ops
    g = torch.Generator().manual_seed(n)
    x = (torch.randn(n, width, generator=g)).to(dtype)
    wg, wu = (torch.randn(experts, ff, width, generator=g) / math.sqrt(width)).to(dtype), \
        (torch.randn(experts, ff, width, generator=g) / math.sqrt(width)).to(dtype)
    wd = (torch.randn(experts, width, ff, generator=g) / math.sqrt(ff)).to(dtype)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(n)]).int()
    if n > 100:
        ids[:90] = ids[0]                 # one expert with more pairs than a tile holds
    wts = torch.rand(n, top, generator=g)
    pairs = n * top
    rows = ops.moe_tile_rows()
    i32 = lambda k: torch.zeros(k, dtype=torch.int32, device=DEV)
    offsets, order, tiles, n_tiles = i32(experts + 1), i32(pairs), i32(2 * (-(-pairs // rows) + experts)), i32(1)
    ids_d = d(ids)
    ops.moe_arrange(ids_d, pairs, experts, rows, offsets, order, tiles, n_tiles)
    assert sorted(order.cpu().tolist()) == list(range(pairs))
    off = offsets.cpu().tolist()
    for e in range(experts):
        assert all(int(ids.reshape(-1)[p]) == e for p in order.cpu().tolist()[off[e]:off[e + 1]])
    act = torch.empty(pairs, ff, dtype=dtype, device=DEV)
    ops.moe_grouped_simt(d(x), d(wg), d(wu), act, offsets, order, tiles, n_tiles, n_pairs=pairs, top=top)
    y = torch.empty(pairs, width, dtype=torch.float32, device=DEV)
    ops.moe_grouped_simt(act, d(wd), None, y, offsets, order, tiles, n_tiles, n_pairs=pairs, top=top)
    residual = torch.ones(n, width, dtype=torch.float32, device=DEV)
    ops.moe_combine(residual, y, d(wts), top=top)
    want = torch.ones(n, width, dtype=torch.float64)
    for t in range(n):
        for c in range(top):
            e = int(ids[t, c])
            h = x[t].double()
            a = torch.nn.functional.silu(wg[e].double() @ h) * (wu[e].double() @ h)
            if dtype == torch.bfloat16:
                a = a.to(torch.bfloat16).double()
            want[t] += wts[t, c].double() * (wd[e].double() @ a)
    assert rel_err(residual, want) < (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("experts,top,ff,width,n", [(6, 2, 24, 72, 50), (5, 1, 200, 128, 3), (12, 3, 136, 320, 700), (4, 4, 264, 64, 300)])
def test_grouped_expert_products_on_tensor_cores(experts, top, ff, width, n):
    """The tcgen05 form: activations gathered into the experts' order, tiles of 128 rows of one expert (an
    expert with several tiles, experts with none, features that are not a multiple of the tile), results
    found again through `place`."""
    from rust_inference_b200.kernels import ops, tcgen05
    g = torch.Generator().manual_seed(n + ff)
    bf = torch.bfloat16
    x = torch.randn(n, width, generator=g).to(bf)
    wg = (torch.randn(experts, ff, width, generator=g) / math.sqrt(width)).to(bf)
    wu = (torch.randn(experts, ff, width, generator=g) / math.sqrt(width)).to(bf)
    wd = (torch.randn(experts, width, ff, generator=g) / math.sqrt(ff)).to(bf)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(n)]).int()
    if n > 100 and top < experts:
        ids[: n // 2] = ids[0]               # a few experts with many rows, the others with few or none
    wts = torch.rand(n, top, generator=g)
    pairs, rows = n * top, tcgen05.GROUPED_TILE_ROWS
    i32 = lambda k: torch.zeros(k, dtype=torch.int32, device=DEV)
    offsets, order, tiles, n_tiles, place = i32(experts + 1), i32(pairs), i32(2 * (-(-pairs // rows) + experts)), i32(1), i32(pairs)
    ops.moe_arrange(d(ids), pairs, experts, rows, offsets, order, tiles, n_tiles, place)
    assert torch.equal(order[place.long()].cpu(), torch.arange(pairs, dtype=torch.int32))
    wg_d, wu_d, wd_d = d(wg), d(wu), d(wd)
    xs = torch.empty(pairs, width, dtype=bf, device=DEV)
    ops.moe_gather(d(x), xs, order, n_pairs=pairs, top=top)
    assert torch.equal(xs.cpu(), x[(order.cpu().long() // top)])
    if pairs <= 256:                                  # few pairs: the arranging kernel gathers the rows itself
        xs2 = torch.empty_like(xs)
        ops.moe_arrange(d(ids), pairs, experts, rows, offsets, order, tiles, n_tiles, place, gather=(d(x), xs2, top))
        assert torch.equal(xs2.cpu(), x[(order.cpu().long() // top)])
        xs = xs2
    act = torch.full((pairs, ff), float("nan"), dtype=bf, device=DEV)
    tcgen05.grouped_gemm(xs, wg_d, wu_d, act, offsets, tiles, n_tiles, n_pairs=pairs)
    y = torch.full((pairs, width), float("nan"), dtype=torch.float32, device=DEV)
    tcgen05.grouped_gemm(act, wd_d, None, y, offsets, tiles, n_tiles, n_pairs=pairs)
    residual = torch.ones(n, width, dtype=torch.float32, device=DEV)
    ops.moe_combine(residual, y, d(wts), top=top, place=place)
    torch.cuda.synchronize()
    tcgen05.check_status()
    want = torch.ones(n, width, dtype=torch.float64)
    xd = x.double()
    for e in range(experts):
        a = (torch.nn.functional.silu(xd @ wg[e].double().T) * (xd @ wu[e].double().T)).to(bf).double() @ wd[e].double().T
        for c in range(top):
            hit = ids[:, c] == e
            want[hit] += wts[hit, c].double()[:, None] * a[hit]
    assert rel_err(residual, want) < 2e-2


@pytest.mark.parametrize("lens,cuts", [([23, 9], (100, 5, 2, 1, 100)), ([333, 150], (1000, 140, 64, 1000))])
@pytest.mark.parametrize("heads,dim,vdim", [(2, 40, 24), (1, 72, 33), (3, 24, 40), (2, 8, 16), (1, 130, 70), (1, 300, 8)])
def test_recurrence_in_portions_and_slots(heads, dim, vdim, lens, cuts):
    """The recurrence kernel over a whole sequence, and cut into portions of 1, 2 and 5 tokens with the
    state carried in the slot, for two sequences of unequal length in one call; then the slots are used
    again from a zero state.  Runs of more than 128 new tokens are cut into pieces that are scanned side by
    side (the second set of lengths: whole, 140 + rest, 64 at a time)."""
    from rust_inference_b200.kernels import ops
    g = torch.Generator().manual_seed(dim)
    width, eps, scale = 64, 1e-5, 0.6
    w = {"q": torch.randn(heads * dim, width, generator=g) / 8, "f": torch.randn(heads * dim, width, generator=g) / 4,
         "f.b": torch.randn(heads * dim, generator=g), "lower": torch.rand(heads * dim, generator=g) * 0.95,
         "v": torch.randn(heads * vdim, width, generator=g) / 8, "norm": 1 + torch.randn(vdim, generator=g) * 0.2,
         "o": torch.eye(heads * vdim)}
    xs = [torch.randn(n, width, generator=g) for n in lens]
    wd = {k: v.double() for k, v in w.items()}
    want = [plain_lulisun.gated_recurrence(x.double(), wd, "", heads=heads, dim=dim, vdim=vdim, eps=eps)[0] * scale for x in xs]
    wz = torch.cat([w["q"], w["f"], w["v"]]).double()
    state = torch.zeros(4, heads, dim, vdim, dtype=torch.float32, device=DEV)
    slots = torch.tensor([2, 0], dtype=torch.int32, device=DEV)

    def run(portions):
        state[2].zero_()
        state[0].zero_()
        outs = [[], []]
        at = [0, 0]
        while any(a < n for a, n in zip(at, lens)):
            take = [min(portions, n - a) for a, n in zip(at, lens)]
            live = [b for b in range(2) if take[b] > 0]
            z = torch.cat([xs[b][at[b]:at[b] + take[b]].double() @ wz.T for b in live]).float()
            ends = [sum(take[b] for b in live[:i + 1]) for i in range(len(live))]
            cu = torch.tensor([0] + ends, dtype=torch.int32, device=DEV)
            out = torch.empty(z.shape[0], heads * vdim, dtype=torch.float32, device=DEV)
            piece, most = ops.recurrence_pieces(max(take), len(live), heads, dim, vdim)
            assert (piece > 0) == (max(take) > 128)
            ops.gated_recurrence(d(z), d(w["f.b"]), d(w["lower"]), d(w["norm"]), state, cu, slots[live].contiguous(), out,
                                 n_seqs=len(live), heads=heads, dim=dim, vdim=vdim, eps=eps, out_scale=scale,
                                 piece=piece, max_pieces=most, longest_run=max(take))
            o = 0
            for b in live:
                outs[b].append(out[o:o + take[b]].cpu())
                o += take[b]
                at[b] += take[b]
        return [torch.cat(o) for o in outs]

    for portions in cuts:                           # the last run uses the slots again
        got = run(portions)
        for b in range(2):
            assert rel_err(got[b], want[b]) < 2e-5, (portions, b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_chunk_edges_with_one_key_that_stands_out(dtype):
    """Attention over a paged cache whose pages are out of order: every key is small but one, whose
    score dwarfs the rest for any query.  A query in the marked key's chunk (at or after it) returns
    that key's value, a query in the next chunk (one position past the edge) does not see it, and
    the chunk's first position sees only itself.  Chunks of 24 (edges inside pages), 64 (edges on page
    borders) and 100."""
    from rust_inference_b200.kernels import ops
    hd, vhd, heads, kvh, page, n_pages, slots_pages = 16, 24, 4, 2, 64, 8, 6
    g = torch.Generator().manual_seed(3)
    n = 300
    for chunk in (24, 64, 100):
        for marked in (0, chunk - 1, chunk, 2 * chunk + 3, n - 1):
            k = torch.randn(n, kvh, hd, generator=g) * 0.01
            v = torch.randn(n, kvh, vhd, generator=g)
            k[marked] = 4.0
            q = torch.full((n, heads, hd), 1.0)
            table = torch.tensor([[5, 2, 7, 0, 3, 1]], dtype=torch.int32)
            kc = torch.zeros(n_pages, kvh, page, hd)
            vc = torch.zeros(n_pages, kvh, page, vhd)
            for p in range(n):
                kc[table[0, p // page], :, p % page] = k[p]
                vc[table[0, p // page], :, p % page] = v[p]
            pos = torch.arange(n, dtype=torch.int32)
            out = torch.empty(n, heads * vhd, dtype=dtype, device=DEV)
            ops.attention_generic(d(q.reshape(n, -1), dtype), heads * hd, d(kc, dtype), d(vc, dtype), d(table), d(pos),
                                  d(torch.zeros(n, dtype=torch.int32)), d(torch.zeros(1, dtype=torch.int32)), out,
                                  n_tokens=n, n_heads=heads, n_kv_heads=kvh, head_dim=hd, page_size=page, scale=1.0,
                                  chunk=chunk, v_head_dim=vhd, out_scale=0.5)
            out = out.float().cpu().view(n, heads, vhd)
            want = torch.zeros(n, heads, vhd, dtype=torch.float64)
            vis = plain_lulisun.chunk_visible(n, chunk)
            kk = k.to(dtype).double() if dtype == torch.bfloat16 else k.double()
            vv = v.to(dtype).double() if dtype == torch.bfloat16 else v.double()
            for h in range(heads):
                s = (q[:, h].double() @ kk[:, h // 2].T).masked_fill(~vis, float("-inf"))
                want[:, h] = 0.5 * torch.softmax(s, dim=-1) @ vv[:, h // 2]
            assert rel_err(out.reshape(n, -1), want.reshape(n, -1)) < (1e-5 if dtype == torch.float32 else 1e-2)
            last = min(n, (marked // chunk + 1) * chunk) - 1          # the last query that sees the marked key
            assert torch.allclose(out[last, 0], 0.5 * vv[marked, 0].float(), atol=2e-2)
            if last + 1 < n:
                assert not torch.allclose(out[last + 1, 0], 0.5 * vv[marked, 0].float(), atol=2e-2)
                assert torch.allclose(out[last + 1, 0], 0.5 * vv[last + 1, 0].float(), atol=1e-2)   # alone in its chunk


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("chunk", [7, 64, 100, 160])
def test_chunked_attention_on_tensor_cores(hd, chunk):
    """The tensor-core kernels (tcgen05 prefill, split decode) with a chunk mask and an output factor against
    the generic kernel on the same cache: continuations that start inside a chunk, query tiles that span
    several chunks, decode steps just before, at and just after a chunk's first position."""
    from types import SimpleNamespace
    from rust_inference_b200.kernels import attention as attn_kernels, ops
    heads, kvh, page = 4, 2, 64
    g = torch.Generator().manual_seed(chunk + hd)
    bf = torch.bfloat16
    n_pages, max_pages = 24, 8                           # 512 positions per sequence
    kc = d(torch.randn(n_pages, kvh, page, hd, generator=g).to(bf))
    vc = d(torch.randn(n_pages, kvh, page, hd, generator=g).to(bf))
    table = torch.stack([torch.randperm(n_pages, generator=g)[:max_pages] for _ in range(3)]).int()

    def run(starts, news):
        n = sum(news)
        assert all(s + k <= max_pages * page for s, k in zip(starts, news))
        pos = torch.cat([torch.arange(s, s + k) for s, k in zip(starts, news)]).int()
        seq = torch.cat([torch.full((k,), b) for b, k in enumerate(news)]).int()
        cu = torch.tensor([0] + [sum(news[:i + 1]) for i in range(len(news))], dtype=torch.int32)
        ws = {}
        ctx = SimpleNamespace(all_single=all(k == 1 for k in news), page_size=page, n_seqs=len(news), page_table=d(table),
                              seq_slot=d(torch.arange(len(news), dtype=torch.int32)), seq_start=d(torch.tensor(starts, dtype=torch.int32)),
                              seq_len=d(torch.tensor([s + k for s, k in zip(starts, news)], dtype=torch.int32)),
                              cu_seqlens=d(cu), token_pos=d(pos), token_seq=d(seq), max_new=max(news), n_tokens=n,
                              buffer=lambda name, shape, dtype: ws.setdefault((name, tuple(shape)), torch.empty(shape, dtype=dtype, device=DEV)))
        qkv = d((torch.randn(n, (heads + 2 * kvh) * hd, generator=g) * 0.5).to(bf))
        fast = torch.empty(n, heads * hd, dtype=bf, device=DEV)
        attn_kernels.attention(qkv, SimpleNamespace(k=kc, v=vc), fast, ctx, n_heads=heads, n_kv_heads=kvh, head_dim=hd,
                               scale=0.11, chunk=chunk, out_scale=0.7)
        plain = torch.empty(n, heads * hd, dtype=bf, device=DEV)
        ops.attention_generic(qkv, qkv.shape[1], kc, vc, ctx.page_table, ctx.token_pos, ctx.token_seq, ctx.seq_slot, plain,
                              n_tokens=n, n_heads=heads, n_kv_heads=kvh, head_dim=hd, page_size=page, scale=0.11, chunk=chunk,
                              out_scale=0.7)
        if not ctx.all_single:
            # the mma.sync prefill kernel (what runs where the tcgen05 one does not take the row strides)
            other = torch.empty(n, heads * hd, dtype=bf, device=DEV)
            ops.attention_prefill(qkv, qkv.shape[1], kc, vc, ctx.page_table, ctx.seq_slot, ctx.seq_start, ctx.cu_seqlens, other,
                                  n_seqs=ctx.n_seqs, max_new=ctx.max_new, n_heads=heads, n_kv_heads=kvh, head_dim=hd,
                                  page_size=page, scale=0.11, window=-chunk)
            ops.scale_(other, 0.7)
            assert rel_err(other, plain) < 2e-2, (starts, news, "mma")
        torch.cuda.synchronize()
        from rust_inference_b200.kernels import tcgen05
        tcgen05.check_status()
        assert rel_err(fast, plain) < 2e-2, (starts, news)

    run([0, 70, 5], [300, 150, 1])                       # prompts and continuations, a single token among them
    run([chunk - 1, chunk, min(3 * chunk - 1, 440)], [130, 2, 64])        # every sequence stays within its 8 pages
    for base in (chunk - 1, chunk, chunk + 1, 2 * chunk, 200, 449):
        run([base, base + 1, max(0, base - 1)], [1, 1, 1])     # decode steps around a chunk's first position


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,n", [(1, 72), (8, 2048), (37, 100), (128, 4096)])
def test_two_norms_in_one_kernel(dtype, rows, n):
    from rust_inference_b200.kernels import ops
    g = torch.Generator().manual_seed(n)
    x = torch.randn(rows, n, generator=g) * 3
    wa, wb = 1 + torch.randn(n, generator=g) * 0.2, 1 + torch.randn(n, generator=g) * 0.2
    a, b = torch.empty(rows, n, dtype=dtype, device=DEV), torch.empty(rows, n, dtype=dtype, device=DEV)
    ops.rmsnorm_pair(d(x), d(wa), d(wb), 1e-5, a, b)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert rel_err(a, plain_lulisun.plain_rmsnorm(x.double(), wa.double(), 1e-5)) < tol
    assert rel_err(b, plain_lulisun.plain_rmsnorm(x.double(), wb.double(), 1e-5)) < tol


def test_partial_rotation_and_value_cache():
    """The rotary kernel with fewer rotated channels than a head has and values of another head size."""
    from rust_inference_b200.kernels import ops
    from rust_inference_b200.parts.rope import rope_tables
    heads, kvh, hd, vhd, rot, page = 3, 1, 12, 20, 8, 64
    n = 70
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(n, (heads + kvh) * hd + kvh * vhd, generator=g)
    cos, sin = rope_tables(rot, 321.0, 256, exact_angles=True)
    pos = torch.arange(100, 100 + n, dtype=torch.int32)
    table = torch.tensor([[9, 1, 4, 2]], dtype=torch.int32)
    kc = torch.zeros(10, kvh, page, hd, device=DEV)
    vc = torch.zeros(10, kvh, page, vhd, device=DEV)
    q_dev = d(qkv)
    ops.rope_cache_write(q_dev, d(torch.from_numpy(cos)), d(torch.from_numpy(sin)), d(pos), d(torch.zeros(n, dtype=torch.int32)),
                         d(torch.zeros(1, dtype=torch.int32)), d(table), kc, vc, n_heads=heads, n_kv_heads=kvh, head_dim=hd,
                         page_size=page, style=0, write_kv=True, rot_dims=rot, v_head_dim=vhd)
    q_want = plain_lulisun.rotate_partial(qkv[:, :heads * hd].double().view(n, heads, hd), pos, 321.0, rot)
    k_want = plain_lulisun.rotate_partial(qkv[:, heads * hd:(heads + kvh) * hd].double().view(n, kvh, hd), pos, 321.0, rot)
    assert rel_err(q_dev[:, :heads * hd], q_want.reshape(n, -1)) < 1e-5
    for t in range(n):
        p = int(pos[t])
        assert rel_err(kc[table[0, p // page], :, p % page].reshape(1, -1), k_want[t].reshape(1, -1)) < 1e-5
        assert torch.equal(vc[table[0, p // page], :, p % page].cpu().reshape(-1), qkv[t, (heads + kvh) * hd:])


# ---------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    made = {}

    def get(name, pinned=False, seed=0):
        key = (name, pinned, seed)
        if key not in made:
            made[key] = lulisun_models.make(tmp_path_factory.mktemp("lulisun"), name, seed=seed, pinned=pinned)
        return made[key]
    return get


def _engine(model, dtype, **kw):
    from rust_inference_b200.engine.engine import Engine
    return Engine.from_pretrained(model.folder, dtype=dtype, max_tokens=kw.pop("max_tokens", 2048), n_slots=kw.pop("n_slots", 6), **kw)


def _run(eng, slot, tokens, portions):
    """Feed `tokens` to `slot` cut as `portions` says (a list of sizes, the last repeated); logits of every token."""
    rows, at, i = [], 0, 0
    while at < len(tokens):
        k = portions[min(i, len(portions) - 1)]
        rows.append(eng.step([slot], [tokens[at:at + k]], "all").cpu())
        at += k
        i += 1
    return torch.cat(rows)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompt_layers_and_decoding(dtype, name, models):
    """A whole prompt (the stream after every layer too), the same with its last 40 tokens one by one
    (across chunk edges and a page border), and a slot used again."""
    from rust_inference_b200.cache.sequence_cache import KVRequest, StateRequest
    model = models(name, pinned=dtype == "bfloat16")
    eng = _engine(model, dtype)
    reqs = eng.model.cache_requests()
    assert len(reqs) == len(model.cfg["layers"]) and all(isinstance(r, tuple) and isinstance(r[0], KVRequest)
                                                         and isinstance(r[1], StateRequest) for r in reqs)
    tokens = random_tokens(150, model.cfg["vocab"], 1)
    streams = []
    want = model.plain_logits(tokens, streams=streams)
    tol = TOL[dtype]

    class Streams:
        rows = []

        def __init__(self):
            self.seen = []

        def record(self, label, hidden, picked=False):
            if not picked:
                self.seen.append(hidden.float().cpu().clone())

    probe = Streams()
    s = eng.alloc_slot()
    got = eng.step([s], [tokens], "all", probe=probe)
    assert rel_err(got, want) < tol
    assert len(probe.seen) == len(streams)
    for a, b in zip(probe.seen, streams):
        assert rel_err(a, b) < tol
    eng.free_slot(s)
    s2 = eng.alloc_slot()
    assert s2 == s                                     # the slot and its pages again, stale state in them
    got = _run(eng, s2, tokens, [110, 1])
    assert rel_err(got, want) < tol
    eng.check_device_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_several_sizes(dtype, models):
    model = models("A", pinned=dtype == "bfloat16")
    eng = _engine(model, dtype)
    tokens = random_tokens(131, model.cfg["vocab"], 2)
    want = model.plain_logits(tokens)
    for portions in ([2], [1, 2, 3, 5, 7, 24, 23, 64, 2], [63, 1, 1, 66], [64, 64, 3]):
        s = eng.alloc_slot()
        assert rel_err(_run(eng, s, tokens, portions), want) < TOL[dtype], portions
        eng.free_slot(s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_batch_against_each_alone(dtype, name, models):
    """Prompts of 1, 2, 70 and 129 tokens as one batch, then decoded together while the short ones leave;
    then a second batch in the freed slots while the first still decodes."""
    model = models(name, pinned=dtype == "bfloat16")
    eng = _engine(model, dtype)
    vocab = model.cfg["vocab"]
    lens, extra = [1, 2, 70, 129], [3, 9, 30, 12]
    seqs = [random_tokens(n + e, vocab, 10 + i) for i, (n, e) in enumerate(zip(lens, extra))]
    want = [model.plain_logits(t) for t in seqs]
    slots = [eng.alloc_slot() for _ in seqs]
    got = [[] for _ in seqs]
    out = eng.step(slots, [t[:n] for t, n in zip(seqs, lens)], "all").cpu()
    o = 0
    for b, n in enumerate(lens):
        got[b].append(out[o:o + n])
        o += n
    at = list(lens)
    second = None
    while any(a < len(t) for a, t in zip(at, seqs)):
        live = [b for b in range(len(seqs)) if at[b] < len(seqs[b])]
        out = eng.step([slots[b] for b in live], [[seqs[b][at[b]]] for b in live], "last").cpu()
        for i, b in enumerate(live):
            got[b].append(out[i:i + 1])
            at[b] += 1
            if at[b] == len(seqs[b]):
                eng.free_slot(slots[b])
        if second is None and len(live) < len(seqs):
            # a new request in a slot that was just freed, alone, while the others wait
            t2 = random_tokens(77, vocab, 99)
            s = eng.alloc_slot()
            second = (rel_err(eng.step([s], [t2], "all"), model.plain_logits(t2)), s)
            eng.free_slot(s)
    for b in range(len(seqs)):
        assert rel_err(torch.cat(got[b]), want[b]) < TOL[dtype], b
    assert second is not None and second[0] < TOL[dtype]
    eng.check_device_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_captured_steps(dtype, models):
    """Three tokens of prompt, then 260 decode steps of a batch of two (captured steps from the fourth
    on), across four pages and many chunks: logits of every step against the plain model."""
    model = models("B", pinned=dtype == "bfloat16")
    eng = _engine(model, dtype)
    vocab = model.cfg["vocab"]
    seqs = [random_tokens(263, vocab, 21), random_tokens(263, vocab, 22)]
    want = [model.plain_logits(t) for t in seqs]
    slots = [eng.alloc_slot(), eng.alloc_slot()]
    eng.step(slots, [t[:3] for t in seqs], "none")
    rows = [[], []]
    for p in range(3, 263):
        out = eng.step(slots, [[t[p]] for t in seqs], "last").cpu()
        rows[0].append(out[0:1])
        rows[1].append(out[1:2])
    assert eng.decode_graph(2) is not None and eng.decode_graph(2).graph is not None
    for b in range(2):
        assert rel_err(torch.cat(rows[b]), want[b][3:]) < TOL[dtype]
    eng.check_device_status()


def test_a_far_token_reaches_through_the_state_only(models, tmp_path):
    """What a token far back contributes can only arrive through the recurrent state once its chunk has
    passed: with the recurrence's share set to zero the logits of a late position do not depend on
    the first token; with it they do, and the engine agrees with the plain model in both cases."""
    base = lulisun_models.CONFIGS["B"]
    for right_scale in (0.0, 0.6):
        cfg = {**base, "layers": [{**L, "mixer": {**L["mixer"], "right_scale": right_scale}} for L in base["layers"]]}
        def slow_decay(w):          # what the state holds of the first token is still there 230 tokens on
            w["l1.mix.right.lower"] = torch.full_like(w["l1.mix.right.lower"], 0.996)
        model = lulisun_models.make(tmp_path, f"far{int(right_scale * 10)}", cfg=cfg, edit=slow_decay)
        eng = _engine(model, "float32")
        a = random_tokens(230, cfg["vocab"], 5)
        b = [(a[0] + 1) % cfg["vocab"]] + a[1:]
        out = []
        for t in (a, b):
            s = eng.alloc_slot()
            got = _run(eng, s, t, [228, 1])
            eng.free_slot(s)
            assert rel_err(got, model.plain_logits(t)) < TOL["float32"]
            out.append(got[-1])
        differs = float((out[0] - out[1]).abs().max()) > 1e-4
        assert differs == (right_scale != 0.0)


def test_greedy_generation_through_the_api(models):
    """`Model.generate` (admission, prefill, captured decode steps, sampling on the device) against the plain
    model's greedy continuation, for prompts of unequal length."""
    from rust_inference_b200 import Model, SamplerConfig
    model = models("A")
    prompts = [random_tokens(5, model.cfg["vocab"], 31), random_tokens(40, model.cfg["vocab"], 32), [7]]
    n_new = 12
    m = Model.load(model.folder, dtype="float32", max_tokens_in_cache=1024)
    got = m.generate(prompts, n_new, SamplerConfig.plain(temperature=0.0), stop_ids=())
    for p, g in zip(prompts, got):
        assert list(g.tokens) == plain_lulisun.greedy(model.cfg, model.weights, p, n_new)


def test_trace_replay_picks_the_model_by_its_config(models, tmp_path):
    """`bin/trace_run` on a Lulisun folder: the runner builds the model its config.json names."""
    import json
    import os
    import subprocess
    import sys
    import numpy as np
    model = models("B")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    tokens = random_tokens(70, model.cfg["vocab"], 41)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": tokens[:66], "want": [0, 65]}], "end": []}]
    steps += [{"step": i + 1, "entries": [{"id": "x", "tokens": [tokens[66 + i]], "want": [0]}], "end": ["x"] if i == 3 else []}
              for i in range(4)]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model.folder, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(5)]
    want = model.plain_logits(tokens)
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1))
    assert rel_err(got0, want[[0, 65]]) < TOL["float32"]
    for i in range(4):
        got = torch.from_numpy(np.fromfile(out / f"{i + 1}.f32", dtype="<f4").reshape(1, -1))
        assert rel_err(got, want[66 + i:67 + i]) < TOL["float32"]


def test_checked_build_stays_silent_and_skips_a_bad_slot(tmp_path):
    """The checked build (indices that reach memory through a table are compared with their limits) runs a
    Lulisun model in both precisions without a record; the recurrence kernel handed a slot beyond the
    cache's slots records it and leaves state and output alone.  In a process of its own: the build is
    chosen when the package is imported."""
    import os
    import subprocess
    import sys
    import textwrap
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = textwrap.dedent("""
        import sys, pathlib, tempfile, torch
        sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r})
        import lulisun_models
        from conftest import random_tokens, rel_err
        from rust_inference_b200.engine.engine import Engine
        from rust_inference_b200.kernels import build, ops
        assert build.CHECKED and build.library_path("recurrent").endswith("checked/libri_recurrent.so")
        model = lulisun_models.make(pathlib.Path(tempfile.mkdtemp()), "B", pinned=True)
        toks = random_tokens(150, model.cfg["vocab"], 3)
        want = model.plain_logits(toks)
        for dtype in ("float32", "bfloat16"):
            eng = Engine.from_pretrained(model.folder, dtype=dtype, max_tokens=512, n_slots=3)
            s = eng.alloc_slot()
            head = eng.step([s], [toks[:140]], "all").cpu()
            tail = torch.cat([eng.step([s], [[t]], "last").cpu() for t in toks[140:]])
            assert rel_err(torch.cat([head, tail]), want) <= (1e-4 if dtype == "float32" else 8e-2)
            eng.check_device_status()
        assert ops.bounds_report() == []
        heads, dim, vdim = 2, 8, 16
        z = torch.randn(1, 2 * heads * dim + heads * vdim, device="cuda")
        state = torch.full((3, heads, dim, vdim), 5.0, device="cuda")
        out = torch.full((1, heads * vdim), 7.0, device="cuda")
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
        ops.gated_recurrence(z, torch.zeros(heads * dim, device="cuda"), torch.zeros(heads * dim, device="cuda"),
                             torch.ones(vdim, device="cuda"), state, i32([0, 1]), i32([9]), out, n_seqs=1, heads=heads,
                             dim=dim, vdim=vdim, eps=1e-5, longest_run=1)
        torch.cuda.synchronize()
        assert float((state - 5.0).abs().max()) == 0.0
        rep = ops.bounds_report()
        assert rep and rep[0][0] == "recurrent" and rep[0][1] == "a cache slot that does not exist" and rep[0][2] == 9, rep
        print("checked ok")
    """).format(root=root, tests=os.path.join(root, "tests"))
    env = dict(os.environ, RI_B200_CHECK_BOUNDS="1")
    p = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=900)
    assert p.returncode == 0 and "checked ok" in p.stdout, p.stderr[-3000:]


def test_the_command_line_on_a_lulisun_folder(models, tmp_path):
    """`bin/gguf-infer` as a process: greedy ids from a model folder (the model comes from config.json's name) equal
    the plain model's, and the random-weights mode runs from a config.json alone, with the layers' statistics."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cli = os.path.join(root, "bin", "gguf-infer")
    model = models("B")
    prompts = [random_tokens(n, model.cfg["vocab"], 70 + n) for n in (9, 1)]
    args = [sys.executable, cli, "--model", model.folder, "--temperature", "0", "--repetition-penalty", "1", "--max-tokens", "6",
            "--dtype", "float32", "--max-seq-len", "256", "--stop-ids", ""]
    for p in prompts:
        args += ["--prompt", ",".join(str(t) for t in p)]
    p = subprocess.run(args, capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert [[int(t) for t in l.split()] for l in lines] == [plain_lulisun.greedy(model.cfg, model.weights, q, 6) for q in prompts]
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(lulisun_models.CONFIGS["A"]))
    p = subprocess.run([sys.executable, cli, "--random-config", str(cfg_file), "--weights-seed", "3", "--random-prompts", "2:4:20",
                        "-n", "5", "--max-seq-len", "128", "--dump-layer-stats"], capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert len([l for l in p.stdout.splitlines() if l.strip()]) == 2 and "[L3]" in p.stderr + p.stdout
