"""The Vadodra decoder in the engine against the plain restatement (`plain_vadodra`): each mechanism's kernel
alone, then whole models: prompts whole, token by token, in portions down to two tokens, unequal batches, slots
and pages used again, keys at the edges of windows and pages, far keys, long decoding, and greedy generation
through `Model.generate`."""
import math

import pytest
import torch

import plain_vadodra
import vadodra_models
from conftest import random_tokens, rel_err

# Worst row's max |a - b| / max |b| against the plain model in float64.  float32 runs: a kernel fault shows far
# above 1e-4.  bfloat16 runs keep bfloat16 activations between kernels through four or five layers on weights
# drawn hot (unit-variance streams): rounding alone reaches a few 1e-2 on single rows; a key too many or too
# few, a lost gate or a wrong pairing costs 0.2 and more.
TOL = {"float32": 1e-4, "bfloat16": 6e-2}

pytestmark = pytest.mark.gpu

DEV = "cuda"


def d(t, dtype=None):
    return t.to(device=DEV, dtype=dtype or t.dtype).contiguous()


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


# ---------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width", [(3, 72), (5, 130), (300, 256), (7, 4100), (260, 1000), (2, 20000)])
def test_layer_norm_kernel(dtype, rows, width):
    """Few and many rows, widths that take the vector, warp and plain forms; a large common offset, where
    mean(x^2) - mean^2 would lose the variance; picked rows."""
    from rust_inference_b200.kernels import ops
    g = torch.Generator().manual_seed(rows + width)
    x = torch.randn(rows, width, generator=g) * 0.5 + 300.0
    w = 1.0 + 0.3 * torch.randn(width, generator=g)
    out = torch.empty(rows, width, dtype=dtype, device=DEV)
    ops.layernorm(d(x), d(w), 1e-5, out)
    want = plain_vadodra.centred_norm(x.double(), w.double(), 1e-5)
    assert rel_err(out, want) < (2e-4 if dtype == torch.float32 else 1e-2)
    pick = [rows - 1, 0]
    out2 = torch.empty(2, width, dtype=dtype, device=DEV)
    ops.layernorm(d(x), d(w), 1e-5, out2, i32(pick))
    assert rel_err(out2, want[pick]) < (2e-4 if dtype == torch.float32 else 1e-2)     # few rows take another form of the kernel


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("style", [0, 1])
@pytest.mark.parametrize("heads,kvh,hd,rot,own_values", [(4, 2, 32, 8, False), (3, 3, 24, 24, False), (1, 1, 80, 2, False),
                                                         (8, 1, 128, 64, False), (2, 2, 256, 256, False), (4, 1, 64, 16, False),
                                                         (5, 5, 40, 24, False), (3, 1, 64, 32, True), (2, 2, 20, 10, True)])
def test_normed_rotation_and_cache_write(dtype, style, heads, kvh, hd, rot, own_values):
    """RMS norm of every q and k head, rotation of the first channels in either pairing, the keys into the
    paged cache and the keys as projected into the value cache (or, with own_values, value columns of their own,
    copied), at positions on both sides of a page border with pages out of order.  bfloat16 heads whose sizes allow
    take the form of the kernel that moves 16 bytes per lane; the others, and float32, the plain one."""
    from rust_inference_b200.kernels import ops
    from rust_inference_b200.parts.rope import rope_tables
    g = torch.Generator().manual_seed(hd + rot + style)
    page, pos = 64, torch.tensor([62, 63, 64, 65, 130, 0])
    n = pos.numel()
    cols = (heads + kvh) * hd + (kvh * hd if own_values else 0)
    qk = (torch.randn(n, cols, generator=g) * 1.7).to(dtype)
    qw, kw = 1 + 0.3 * torch.randn(hd, generator=g), 1 + 0.3 * torch.randn(hd, generator=g)
    cos, sin = rope_tables(rot, 321.0, 200, exact_angles=True, scaling_factor=2.5)
    table = torch.tensor([[5, 2, 7, 1]], dtype=torch.int32)
    kc = torch.zeros(8, kvh, page, hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    dev = d(qk)
    ops.rope_normed_cache_write(dev, d(torch.from_numpy(cos)), d(torch.from_numpy(sin)), d(qw), d(kw), 1e-5, d(pos.int()),
                                d(torch.zeros(n, dtype=torch.int32)), i32([0]), d(table), kc, vc, n_heads=heads,
                                n_kv_heads=kvh, head_dim=hd, page_size=page, style=style, write_kv=True, rot_dims=rot,
                                values_from_keys=not own_values)
    turn = plain_vadodra.rotate_halves if style == 0 else plain_vadodra.rotate_adjacent
    q0 = qk[:, :heads * hd].double().view(n, heads, hd)
    k0 = qk[:, heads * hd:(heads + kvh) * hd].double().view(n, kvh, hd)
    values = qk[:, (heads + kvh) * hd:] if own_values else qk[:, heads * hd:]
    q_want = turn(plain_vadodra.rms_norm(q0, qw.double(), 1e-5), pos, 321.0, rot, 2.5)
    k_want = turn(plain_vadodra.rms_norm(k0, kw.double(), 1e-5), pos, 321.0, rot, 2.5)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert rel_err(dev[:, :heads * hd], q_want.reshape(n, -1)) < tol
    assert torch.equal(dev[:, heads * hd:].cpu(), qk[:, heads * hd:])          # k (and v) columns are left as they came
    for t in range(n):
        p = int(pos[t])
        assert rel_err(kc[table[0, p // page], :, p % page].reshape(1, -1), k_want[t].reshape(1, -1)) < tol
        assert torch.equal(vc[table[0, p // page], :, p % page].cpu().reshape(-1), values[t])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,width,ff", [(5, 72, 40), (130, 128, 200), (600, 256, 520)])
@pytest.mark.parametrize("limit", [0.4, 2.0])
def test_bounded_gate_epilogue(dtype, n, width, ff, limit):
    """The gate / up contraction with the bounded gate as its epilogue, in every form of the kernel (steps of few
    tokens, of more than 128, and of 512 and more), with pre-activations on both sides of the bounds; and the
    plain SiLU gate still comes out when no form is given."""
    from rust_inference_b200.kernels import linear
    g = torch.Generator().manual_seed(n + ff)
    x = torch.randn(n, width, generator=g).to(dtype)
    wg = (torch.randn(ff, width, generator=g) * (2.0 / math.sqrt(width))).to(dtype)
    wu = (torch.randn(ff, width, generator=g) * (2.0 / math.sqrt(width))).to(dtype)
    form = torch.tensor([1.702, limit, 1.0], device=DEV)
    out = torch.empty(n, ff, dtype=dtype, device=DEV)
    linear.gated(d(x), linear.Weight(d(wg)), linear.Weight(d(wu)), out, None, form=form)
    gg, uu = x.double() @ wg.double().T, x.double() @ wu.double().T
    assert float((gg > limit).double().mean()) > 0.02 and float((uu < -limit).double().mean()) > 0.02
    gc, uc = gg.clamp(max=limit), uu.clamp(-limit, limit)
    want = gc * torch.sigmoid(1.702 * gc) * (uc + 1.0)
    tol = 1e-5 if dtype == torch.float32 else 1.5e-2
    assert rel_err(out, want) < tol
    linear.gated(d(x), linear.Weight(d(wg)), linear.Weight(d(wu)), out, None)
    assert rel_err(out, torch.nn.functional.silu(gg) * uu) < tol


def test_embedding_scale():
    from rust_inference_b200.kernels import ops
    table = torch.randn(50, 72).to(torch.bfloat16)
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32)
    out = torch.empty(4, 72, device=DEV)
    ops.embed_gather(d(table), d(ids), out, 13.25)
    assert torch.equal(out.cpu(), table.float()[ids.long()] * 13.25)


def make_ctx(cache, slots, starts, counts, dtype, ws):
    """A step context for a part tested outside an engine: sequences in the given slots, continued from `starts`
    by `counts` tokens each."""
    from rust_inference_b200.engine.context import StepContext, pack_step
    tokens = [[0] * c for c in counts]
    meta, layout, sc = pack_step(starts, tokens, [[] for _ in tokens])
    o, c = layout["seq_slot"]
    meta[o:o + c] = slots
    cache.reserve([(s, st + n) for s, st, n in zip(slots, starts, counts)])
    dev = torch.from_numpy(meta).to(DEV)
    v = lambda name: dev[layout[name][0]:layout[name][0] + layout[name][1]]
    return StepContext(
        n_tokens=sc["n_tokens"], n_seqs=sc["n_seqs"], token_ids=v("token_ids"), token_pos=v("token_pos"),
        token_seq=v("token_seq"), seq_slot=v("seq_slot"), seq_start=v("seq_start"), seq_len=v("seq_len"),
        cu_seqlens=v("cu_seqlens"), logit_rows=v("logit_rows"), n_logit_rows=sc["n_logit_rows"],
        max_new=sc["max_new"], max_len=sc["max_len"], all_single=sc["all_single"], page_table=cache.page_table,
        page_size=cache.page_size, dtype=dtype, device=torch.device(DEV), workspace=ws)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dh,rd,vd,rank", [(4, 16, 8, 24, 40), (1, 40, 2, 72, 96), (8, 64, 32, 64, 64), (3, 8, 16, 8, 16)])
def test_latent_attention_part_alone(dtype, H, dh, rd, vd, rank):
    """The latent-attention mixer as a part (projection, norm and rotation into the one cached row, queries into the
    latent space, attention over the shared rows, up-map, gate, output projection) against the plain mixer, for two
    sequences of unequal length in one step, then continued by a portion and by single tokens; and a second part
    that reads the first one's rows."""
    from rust_inference_b200.cache.sequence_cache import SequenceCache
    from rust_inference_b200.engine.context import Workspace
    from rust_inference_b200.engine.engine import Engine  # noqa: F401  (loads the host runtime)
    from rust_inference_b200.parts.latent_attention import LatentAttention
    from rust_inference_b200.parts.spec import PartSpec
    width, eps = 72, 1e-5
    m = {"heads": H, "dim": dh, "rot_dim": rd, "vdim": vd, "kv_rank": rank, "scale": 0.5 / math.sqrt(dh + rd),
         "rot": {"base": 900.0, "dims": rd}}
    cfg = {"width": width, "vocab": 10, "layers": [{"type": "latent_attention", "mixer": m, "mlp": None},
                                                  {"type": "latent_attention", "mixer": {**m, "kv_from": 0}, "mlp": None}]}
    W = {k: v.float() for k, v in plain_vadodra.random_weights({**cfg, "embedding": {"scale": 1.0}}, H + rank, hot=1.5).items()}
    rope = PartSpec("rope", {"head_dim": rd, "base": 900.0, "style": "half", "rot_dims": rd, "exact_angles": True})
    names = {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "gate": "g", "o": "o"}
    run = torch.float32 if dtype == torch.float32 else torch.bfloat16
    parts = []
    for i, own in enumerate((True, False)):
        part = LatentAttention(n_heads=H, head_dim=dh, rot_dim=rd, v_head_dim=vd, kv_rank=rank, eps=eps, position=rope,
                               scale=m["scale"], own_latent=own, names=names, hidden_size=width, dtype=run, device=DEV)
        tensors = {}
        for local, ts in part.tensor_specs().items():
            t = W[f"l{i}.mix.{local}"]
            tensors[local] = d(t, torch.float32 if ts.role == "vector" else run)
        part.set_tensors(tensors)
        part.prepare(512)
        back = part.get_tensors()
        assert all(torch.equal(back[k].float().cpu(), tensors[k].float().cpu()) for k in tensors)
        parts.append(part)
    cache = SequenceCache([parts[0].cache_request()], max_tokens=1024, max_seq_len=512, dtype=run, device=DEV, n_slots=4)
    assert len(cache.groups) == 1 and cache.layer(0).v.data_ptr() == cache.layer(0).k.data_ptr()     # one row per position, no values beside it
    lens = [150, 37]
    g = torch.Generator().manual_seed(1)
    xs = [torch.randn(n, width, generator=g).to(run) for n in lens]
    want = [[plain_vadodra.latent_attention(x.double(), {k: v.double() for k, v in W.items()}, f"l{i}.mix.", cfg["layers"][i]["mixer"], eps,
                                            plain_vadodra.latent_rows(x.double(), {k: v.double() for k, v in W.items()}, "l0.mix.", m, eps))
             for x in xs] for i in range(2)]
    slots = [cache.alloc_slot(), cache.alloc_slot()]
    ws = Workspace(DEV)
    cuts = [(0, [100, 20]), (1, [30, 17]), (2, [1, 0]), (3, [1, 0]), (4, [18, 0])]
    starts = [0, 0]
    got = [[[], []], [[], []]]
    for _, take in cuts:
        live = [b for b in range(2) if take[b]]
        ctx = make_ctx(cache, [slots[b] for b in live], [starts[b] for b in live], [take[b] for b in live], run, ws)
        x = torch.cat([xs[b][starts[b]:starts[b] + take[b]] for b in live])
        for i, part in enumerate(parts):
            res = torch.zeros(x.shape[0], width, dtype=torch.float32, device=DEV)
            part.forward(d(x), res, ctx, cache.layer(0), i == 0)
            o = 0
            for b in live:
                got[i][b].append(res[o:o + take[b]].cpu())
                o += take[b]
        for b in live:
            starts[b] += take[b]
            cache.commit(slots[b], starts[b])
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for i in range(2):
        for b in range(2):
            assert rel_err(torch.cat(got[i][b]), want[i][b]) < tol, (i, b)


def _attention_part(dtype, *, heads, kvh, hd, window, rot, width, seed):
    from rust_inference_b200.parts.registry import lookup
    from rust_inference_b200.parts.spec import PartSpec
    part = lookup("mixer", "gqa_attention")(
        n_heads=heads, n_kv_heads=kvh, head_dim=hd, qkv_bias=False, window=window, scale=0.7 / math.sqrt(hd),
        position=PartSpec("rope", {"head_dim": hd, "base": 5000.0, "style": "interleaved", "rot_dims": rot,
                                   "exact_angles": True, "scaling_factor": 3.0}),
        qk_norm_eps=1e-6, values_from_keys=True, names={"q": "q", "k": "k", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"},
        hidden_size=width, dtype=dtype, device=DEV)
    assert "v_proj.weight" not in part.tensor_specs() and "v" not in part.tensor_specs()
    m = {"heads": heads, "kv_heads": kvh, "dim": hd, "vdim": hd, "scale": 0.7 / math.sqrt(hd),
         "rot": {"base": 5000.0, "dims": rot, "scaling": {"factor": 3.0}}}
    if window is not None:
        m["mask"] = {"size": window}
    cfg = {"width": width, "vocab": 10, "embedding": {"scale": 1.0}, "layers": [{"type": "attention", "mixer": m, "mlp": None}]}
    W = {k: v.float() for k, v in plain_vadodra.random_weights(cfg, seed, hot=1.5).items()}
    tensors = {local: d(W["l0.mix." + local], torch.float32 if ts.role == "vector" else dtype)
               for local, ts in part.tensor_specs().items()}
    part.set_tensors(tensors)
    part.prepare(1024)
    return part, m, W


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kvh,hd,window,rot", [(4, 2, 32, 20, 8), (2, 1, 64, 70, 32), (4, 4, 128, 129, 128), (3, 1, 24, 1, 2),
                                                     (2, 2, 64, None, 64)])
def test_window_edges_with_a_key_that_dwarfs_the_rest(dtype, heads, kvh, hd, window, rot):
    """One input row far larger than the others becomes a value that dominates whatever sees it (the values are the
    keys as projected, so the row's size reaches the output; the normalised keys do not grow with it): the outputs
    differ by orders of magnitude between the last query that still sees it and the first one that no longer does.
    In a prompt (the tensor-core prefill kernel where the sizes allow) and decoding one token at a time, with the
    large row on both sides of a page border."""
    from rust_inference_b200.cache.sequence_cache import SequenceCache
    from rust_inference_b200.engine.context import Workspace
    from rust_inference_b200.engine.engine import Engine  # noqa: F401
    width = 128
    part, m, W = _attention_part(dtype, heads=heads, kvh=kvh, hd=hd, window=window, rot=rot, width=width, seed=hd + rot)
    Wd = {k: v.double() for k, v in W.items()}
    n = 330
    ws = Workspace(DEV)
    for big in (63, 64, 130):
        g = torch.Generator().manual_seed(big)
        x = (torch.randn(n, width, generator=g) * 0.3).to(dtype)
        x[big] = x[big] * 1000.0
        want = plain_vadodra.window_attention(x.double(), Wd, "l0.mix.", m, 1e-6)
        if window is not None and big + window < n:
            inside, outside = want[big + window - 1].abs().max(), want[big + window].abs().max()
            assert float(inside) > 20 * float(outside)             # the edge is visible in the plain result
        cache = SequenceCache([part.cache_request()], max_tokens=1024, max_seq_len=512, dtype=dtype, device=DEV, n_slots=2)
        slot = cache.alloc_slot()
        got = torch.zeros(n, width, device=DEV)
        cut = 150
        at = 0
        for take in [cut] + [1] * (n - cut):
            ctx = make_ctx(cache, [slot], [at], [take], dtype, ws)
            part.forward(d(x[at:at + take]), got[at:at + take], ctx, cache.layer(0), True)
            at += take
            cache.commit(slot, at)
        # per row: the rows behind the edge are small, and must be small here too
        tol = 2e-5 if dtype == torch.float32 else 3e-2
        assert rel_err(got, want) < tol, big
        # the same prompt whole: every edge inside one step
        slot2 = cache.alloc_slot()
        got2 = torch.zeros(n, width, device=DEV)
        part.forward(d(x), got2, make_ctx(cache, [slot2], [0], [n], dtype, ws), cache.layer(0), True)
        assert rel_err(got2, want) < tol, big


# ---------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    made = {}

    def get(name, seed=0):
        if (name, seed) not in made:
            made[(name, seed)] = vadodra_models.make(tmp_path_factory.mktemp("vadodra"), name, seed=seed)
        return made[(name, seed)]
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


class Streams:
    rows = []

    def __init__(self):
        self.seen = []

    def record(self, label, hidden, picked=False):
        if not picked:
            self.seen.append(hidden.float().cpu().clone())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompt_layers_and_decoding(dtype, name, models):
    """A whole prompt (the stream after every layer too), the same with its last tokens one by one (across window
    edges and page borders), and a slot used again."""
    from rust_inference_b200.cache.sequence_cache import KVRequest
    model = models(name)
    eng = _engine(model, dtype)
    reqs = eng.model.cache_requests()
    kinds = [L["type"] for L in model.cfg["layers"]]
    for i, L in enumerate(model.cfg["layers"]):
        if L["type"] == "latent_attention" and L["mixer"].get("kv_from") is not None:
            assert i >= len(reqs) or reqs[i] is None                   # a reader keeps nothing of its own
        else:
            assert isinstance(reqs[i], KVRequest) and reqs[i].values_in_keys == (kinds[i] == "latent_attention")
    tokens = random_tokens(230, model.cfg["vocab"], 1)
    streams = []
    want = model.plain_logits(tokens, streams=streams)
    tol = TOL[dtype]
    probe = Streams()
    s = eng.alloc_slot()
    got = eng.step([s], [tokens], "all", probe=probe)
    assert rel_err(got, want) < tol
    assert len(probe.seen) == len(streams)
    for a, b in zip(probe.seen, streams):
        assert rel_err(a, b) < tol
    eng.free_slot(s)
    s2 = eng.alloc_slot()
    assert s2 == s                                     # the slot and its pages again, the old rows still in them
    got = _run(eng, s2, tokens, [60, 1])
    assert rel_err(got, want) < tol
    eng.check_device_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_portions_of_several_sizes(dtype, name, models):
    model = models(name)
    eng = _engine(model, dtype)
    tokens = random_tokens(197, model.cfg["vocab"], 2)
    want = model.plain_logits(tokens)
    for portions in ([2], [1, 2, 3, 5, 7, 20, 19, 64, 2], [63, 1, 1, 66, 66], [64, 64, 69], [150, 47]):
        s = eng.alloc_slot()
        assert rel_err(_run(eng, s, tokens, portions), want) < TOL[dtype], portions
        eng.free_slot(s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_batch_against_each_alone(dtype, name, models):
    """Prompts of 1, 2, 70 and 160 tokens as one batch, then decoded together while the short ones leave;
    then a request in a freed slot while the others still decode."""
    model = models(name)
    eng = _engine(model, dtype)
    vocab = model.cfg["vocab"]
    lens, extra = [1, 2, 70, 160], [3, 9, 30, 12]
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
            t2 = random_tokens(77, vocab, 99)
            s = eng.alloc_slot()
            second = (rel_err(eng.step([s], [t2], "all"), model.plain_logits(t2)), s)
            eng.free_slot(s)
    for b in range(len(seqs)):
        assert rel_err(torch.cat(got[b]), want[b]) < TOL[dtype], b
    assert second is not None and second[0] < TOL[dtype]
    eng.check_device_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding_through_captured_steps(dtype, name, models):
    """Three tokens of prompt, then 260 decode steps of a batch of two (captured steps from the fourth on), across
    four pages and past every window: logits of every step against the plain model."""
    model = models(name)
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


def test_a_far_token_reaches_through_the_latent_layers_only(tmp_path):
    """The first token lies outside every window of a late position, so it can reach that position's logits only
    through the causal latent attention: with a latent layer they depend on it, in a model of windowed layers
    alone they do not; the engine agrees with the plain model in both cases."""
    A = vadodra_models
    win = A.layer("attention", A.attn(heads=2, kv=1, dim=16, scale=0.25, window=9, base=1000.0, rot=8), 40, 2.0)
    lat = A.layer("latent_attention", A.latent(heads=2, dim=16, rot_dim=8, vdim=16, rank=24, scale=0.2, base=1000.0), 40, 2.0)
    base = {"architecture": "Vadodra", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 4.0}}
    for name, layers in (("windows", [win, win, win]), ("mixed", [win, lat, win])):
        model = A.make(tmp_path, name, cfg={**base, "layers": layers})
        eng = _engine(model, "float32")
        a = random_tokens(230, 97, 5)
        b = [(a[0] + 1) % 97] + a[1:]
        out = []
        for t in (a, b):
            s = eng.alloc_slot()
            got = _run(eng, s, t, [228, 1])
            eng.free_slot(s)
            assert rel_err(got, model.plain_logits(t)) < TOL["float32"]
            out.append(got[-1])
        differs = float((out[0] - out[1]).abs().max()) > 1e-4
        assert differs == (name == "mixed")


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
        assert list(g.tokens) == plain_vadodra.greedy(model.cfg, model.weights, p, n_new)
    mem = m.memory()
    per_position = 0
    for L in model.cfg["layers"]:
        mx = L["mixer"]
        if L["type"] == "attention":
            per_position += 2 * mx["kv_heads"] * mx["dim"] * 4
        elif mx.get("kv_from") is None:
            per_position += (mx["kv_rank"] + mx["rot_dim"]) * 4
    assert mem["cache_bytes_per_position"] == per_position


def test_state_dict_and_saved_folder_round_trip(models, tmp_path):
    """The tensors come back apart under the file's names, and a folder written from them loads to the same logits."""
    from rust_inference_b200 import Model
    model = models("B")
    m = Model.load(model.folder, dtype="float32", max_tokens_in_cache=512)
    sd = m.state_dict()
    assert set(sd) == set(model.weights)
    for k, v in model.weights.items():
        assert torch.equal(sd[k].float().cpu().reshape(v.shape), v), k


def test_trace_replay_picks_the_model_by_its_config(models, tmp_path):
    """`bin/trace_run` on a Vadodra folder: the runner builds the model its config.json names."""
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


def test_the_command_line_on_a_vadodra_folder(models, tmp_path):
    """`bin/gguf-infer` as a process: greedy ids from a model folder equal the plain model's, and the random-weights
    mode runs from a config.json alone, with the layers' statistics."""
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
    assert [[int(t) for t in l.split()] for l in lines] == [plain_vadodra.greedy(model.cfg, model.weights, q, 6) for q in prompts]
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(vadodra_models.CONFIGS["A"]))
    p = subprocess.run([sys.executable, cli, "--random-config", str(cfg_file), "--weights-seed", "3", "--random-prompts", "2:4:20",
                        "-n", "5", "--max-seq-len", "128", "--dump-layer-stats"], capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert len([l for l in p.stdout.splitlines() if l.strip()]) == 2 and "[L4]" in p.stderr + p.stdout


@pytest.mark.parametrize("rank,rd,heads", [(64, 32, 8), (128, 64, 3), (256, 32, 5), (512, 64, 16), (512, 32, 1), (64, 64, 128),
                                             (512, 64, 32), (256, 64, 24), (128, 32, 40)])
def test_latent_attention_on_tensor_cores(rank, rd, heads):
    """The tensor-core kernel of attention over one cached row per position against plain softmax attention over the
    same rows: prompts of unequal length in one step (row tiles that end inside a token's heads), a continuation by a
    portion, decoding with the keys cut into runs that are merged, pages out of order; one cached row made so that
    its score dwarfs the others for one head, at the first position, at a page border, and just behind the
    last query that may see it."""
    from rust_inference_b200.kernels import attention as attn_kernels, ops
    assert ops.latent_attention_mma_supports(rank, rd, 64)
    g = torch.Generator().manual_seed(rank + rd + heads)
    page, wide = 64, rank + rd
    lens = [200, 70, 33]
    n_pages = 12
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(4, 5, dtype=torch.int32)
    rows, at = [], 0
    for b, n in enumerate(lens):
        for k in range(-(-n // page)):
            table[b + 1, k] = perm[at]                                   # slots 1..3
            at += 1
        rows.append((torch.randn(n, wide, generator=g) * 0.5).to(torch.bfloat16))
    scale = 0.5 / math.sqrt(wide)
    cache = torch.zeros(n_pages, 1, page, wide, dtype=torch.bfloat16)
    for b, n in enumerate(lens):
        for p in range(n):
            cache[table[b + 1, p // page], 0, p % page] = rows[b][p]
    qs = [(torch.randn(n, heads, wide, generator=g) * 0.5).to(torch.bfloat16) for n in lens]
    # a key that one head's queries love: the query points along it
    for b, special in ((0, 0), (0, 64), (1, 63), (2, 20)):
        rows_b = rows[b]
        h = special % heads
        qs[b][:, h] = (rows_b[special].float() * (30.0 / (scale * float(rows_b[special].float().pow(2).sum())))).to(torch.bfloat16)
    dcache = d(cache)

    def plain(b, lo, hi):
        k = rows[b].double()
        s = torch.einsum("ihd,jd->hij", qs[b][lo:hi].double(), k) * scale
        pos = torch.arange(lo, hi)
        s = s.masked_fill((pos[:, None] < torch.arange(lens[b])[None, :])[None], float("-inf"))
        return torch.einsum("hij,jr->hir", torch.softmax(s, -1), k[:, :rank])        # [heads, tokens, rank]

    class Ctx:
        pass

    def run(seqs, starts, counts):
        ctx = Ctx()
        ctx.n_seqs, ctx.max_new, ctx.page_size = len(seqs), max(counts), page
        ctx.all_single = all(c == 1 for c in counts)
        ctx.max_len = max(s + c for s, c in zip(starts, counts))
        ctx.page_table = d(table)
        ctx.seq_slot, ctx.seq_start = i32([b + 1 for b in seqs]), i32(starts)
        ctx.cu_seqlens = i32([0] + torch.tensor(counts).cumsum(0).tolist())
        ctx.token_pos = i32([s + i for s, c in zip(starts, counts) for i in range(c)])
        ctx.token_seq = i32([k for k, c in enumerate(counts) for _ in range(c)])
        bufs = {}
        ctx.buffer = lambda name, shape, dtype: bufs.setdefault((name, shape), torch.empty(shape, dtype=dtype, device=DEV))
        q = torch.cat([qs[b][s:s + c] for b, s, c in zip(seqs, starts, counts)]).reshape(-1, heads * wide)
        n = q.shape[0]
        out = torch.empty(heads, n, rank, dtype=torch.bfloat16, device=DEV)
        attn_kernels.latent_attention(d(q), type("L", (), {"k": dcache}), out, ctx, n_heads=heads, key_dim=wide, rank=rank,
                                      scale=scale)
        ref = torch.empty_like(out)
        ops.attention_generic(d(q), heads * wide, dcache, dcache, ctx.page_table, ctx.token_pos, ctx.token_seq, ctx.seq_slot, ref,
                              n_tokens=n, n_heads=heads, n_kv_heads=1, head_dim=wide, page_size=page, scale=scale,
                              v_head_dim=rank, values_in_keys=True, head_major=True)
        want = torch.cat([plain(b, s, s + c) for b, s, c in zip(seqs, starts, counts)], dim=1)
        assert rel_err(out.reshape(-1, rank), want.reshape(-1, rank)) < 2e-2, (seqs, starts, counts)
        assert rel_err(out.reshape(-1, rank), ref.float().reshape(-1, rank)) < 2e-2

    run([0, 1, 2], [0, 0, 0], lens)                       # whole prompts
    run([0, 1], [150, 64], [50, 6])                       # continuations by portions
    run([1, 0, 2], [69, 199, 32], [1, 1, 1])              # decoding, the keys in runs
    run([2], [0], [1])                                    # the first token of a sequence alone


def test_checked_build_stays_silent_and_skips_a_bad_slot(tmp_path):
    """The checked build (indices that reach memory through a table are compared with their limits) runs a Vadodra
    model in both precisions without a record; the heads' norm + rotation + cache-write kernel handed a slot beyond the
    cache's slots records it and writes nothing.  In a process of its own: the build is chosen when the package is
    imported."""
    import os
    import subprocess
    import sys
    import textwrap
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = textwrap.dedent("""
        import sys, pathlib, tempfile, torch
        sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r})
        import vadodra_models
        from conftest import random_tokens, rel_err
        from rust_inference_b200.engine.engine import Engine
        from rust_inference_b200.kernels import build, ops
        from rust_inference_b200.parts.rope import rope_tables
        assert build.CHECKED and build.library_path("latent").endswith("checked/libri_latent.so")
        model = vadodra_models.make(pathlib.Path(tempfile.mkdtemp()), "C")
        toks = random_tokens(150, model.cfg["vocab"], 3)
        want = model.plain_logits(toks)
        for dtype in ("float32", "bfloat16"):
            eng = Engine.from_pretrained(model.folder, dtype=dtype, max_tokens=512, n_slots=3)
            s = eng.alloc_slot()
            head = eng.step([s], [toks[:140]], "all").cpu()
            tail = torch.cat([eng.step([s], [[t]], "last").cpu() for t in toks[140:]])
            assert rel_err(torch.cat([head, tail]), want) <= (1e-4 if dtype == "float32" else 6e-2)
            eng.check_device_status()
        assert ops.bounds_report() == []
        ops.bounds_set_limits(0, 3, 8)
        heads, kvh, hd = 2, 1, 16
        qk = torch.randn(1, (heads + kvh) * hd, device="cuda")
        cos, sin = rope_tables(hd, 100.0, 8)
        kc = torch.full((8, kvh, 64, hd), 5.0, device="cuda")
        vc = torch.full((8, kvh, 64, hd), 5.0, device="cuda")
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
        ops.rope_normed_cache_write(qk, torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda(), None, None, 1e-6, i32([0]),
                                    i32([0]), i32([9]), torch.zeros(3, 2, dtype=torch.int32, device="cuda"), kc, vc, n_heads=heads,
                                    n_kv_heads=kvh, head_dim=hd, page_size=64, style=1, write_kv=True, values_from_keys=True)
        torch.cuda.synchronize()
        assert float((kc - 5.0).abs().max()) == 0.0 and float((vc - 5.0).abs().max()) == 0.0
        rep = ops.bounds_report()
        assert rep and rep[0][0] == "elementwise" and rep[0][1] == "a cache slot that does not exist" and rep[0][2] == 9, rep
        print("checked ok")
    """).format(root=root, tests=os.path.join(root, "tests"))
    env = dict(os.environ, RI_B200_CHECK_BOUNDS="1")
    p = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=900)
    assert p.returncode == 0 and "checked ok" in p.stdout, p.stderr[-3000:]
