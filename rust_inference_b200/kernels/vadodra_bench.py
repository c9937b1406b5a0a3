"""Prefill and decode throughput of a Vadodra-style model beside a dense decoder of equal size, and the time of
each of their kernels against its roofline (`python bench.py --arch vadodra`).

Both models get random bf16 weights and the same width, depth, heads, head size and feed-forward width.  The
Vadodra model alternates its two mixers: sliding-window attention whose values are the unrotated keys, and
attention over a shared latent (the last layer reads the latent the second one cached).  A kernel's roofline time
is the slower of its multiply-adds at the measured bf16 throughput and its bytes at the measured copy bandwidth;
`x_roofline` is measured time over that.  Timed with CUDA events after warm-up, a 256 MiB write between iterations
(flushes L2).
"""
from __future__ import annotations

import json
import math
import sys
import time

import torch

from .arch_bench import Timer, _roofline_ms, _step_context, ffma_peak_tflops, throughput, time_parts as dense_parts

SIZES = {
    # width, attention heads / kv heads / head size, window, rotated channels; latent heads / unrotated and rotated
    # query channels / value channels / latent channels; feed-forward width, vocabulary
    "1k": dict(width=1024, heads=8, kv=2, hd=128, window=512, rot=64, lheads=8, ldim=128, lrot=64, lvdim=128, rank=256,
               ff=4096, vocab=32000),
    "2k": dict(width=2048, heads=16, kv=4, hd=128, window=1024, rot=64, lheads=16, ldim=128, lrot=64, lvdim=128, rank=512,
               ff=8192, vocab=32000),
    "4k": dict(width=4096, heads=32, kv=8, hd=128, window=1024, rot=128, lheads=32, ldim=128, lrot=64, lvdim=128, rank=512,
               ff=14336, vocab=32000),
}
LAYERS = 4


def vadodra_config(s: dict) -> dict:
    window = {"type": "attention", "mixer": {
        "heads": s["heads"], "kv_heads": s["kv"], "dim": s["hd"], "vdim": s["hd"], "scale": 1.0 / math.sqrt(s["hd"]),
        "mask": {"size": s["window"]}, "rot": {"base": 500000.0, "dims": s["rot"], "scaling": {"factor": 4.0}}},
        "mlp": {"kind": "dense", "ff": s["ff"], "limit": 7.0}}
    lat = {"heads": s["lheads"], "dim": s["ldim"], "rot_dim": s["lrot"], "vdim": s["lvdim"], "kv_rank": s["rank"],
           "scale": 1.0 / math.sqrt(s["ldim"] + s["lrot"]), "rot": {"base": 10000.0, "dims": s["lrot"]}}
    own = {"type": "latent_attention", "mixer": lat, "mlp": {"kind": "dense", "ff": s["ff"], "limit": 7.0}}
    reader = {"type": "latent_attention", "mixer": {**lat, "kv_from": 1}, "mlp": {"kind": "dense", "ff": s["ff"], "limit": 7.0}}
    return {"architecture": "Vadodra", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5},
            "embedding": {"scale": math.sqrt(s["width"])}, "layers": [window, own, window, reader]}


def dense_config(s: dict, max_positions: int) -> dict:
    return {"architectures": ["LlamaForCausalLM"], "hidden_size": s["width"], "num_hidden_layers": LAYERS,
            "num_attention_heads": s["heads"], "num_key_value_heads": s["kv"], "head_dim": s["hd"],
            "intermediate_size": s["ff"], "vocab_size": s["vocab"], "rope_theta": 10000.0,
            "rms_norm_eps": 1e-5, "attention_bias": False, "tie_word_embeddings": False,
            "max_position_embeddings": max_positions}


def time_parts(engine, s: dict, lens_before: list, new_tokens: int, peaks: dict, timer: Timer) -> dict:
    """Milliseconds of the two mixers and the feed-forward of a Vadodra model and of their kernels alone, for a step of
    `new_tokens` tokens per sequence on top of `lens_before` cached positions, with each kernel's roofline."""
    from . import attention as attn_kernels, linear, ops
    slots, ctx = _step_context(engine, lens_before, new_tokens, s["vocab"], 5)
    dev = engine.device
    n, width = ctx.n_tokens, s["width"]
    residual = torch.zeros(n, width, dtype=torch.float32, device=dev)
    x = (torch.randn(n, width, device=dev) * 0.5).to(torch.bfloat16)
    bf = torch.bfloat16
    out = {}

    def row(name, ms, flops, bytes_):
        ideal = _roofline_ms(flops, bytes_, peaks)
        out[name] = {"ms": round(ms, 4), "roofline_ms": round(ideal, 6), "x_roofline": round(ms / ideal, 2),
                     "bound": "tensor" if flops / (peaks["bf16_tflops"] * 1e12) > bytes_ / (peaks["hbm_gbs"] * 1e9) else "hbm"}

    # ---- norm -----------------------------------------------------------------------------------------
    block0 = engine.model.layers[0].block
    normed = torch.empty(n, width, dtype=bf, device=dev)
    stream = torch.randn(n, width, device=dev)
    row("layer_norm", timer(lambda: block0.norm.forward(stream, normed)), 0.0, n * width * 6 + width * 4)

    # ---- sliding-window attention (layer 0) --------------------------------------------------------------
    win, cache0 = block0.mixer, engine.cache.layer(0)
    hd, heads, kv, window = s["hd"], s["heads"], s["kv"], s["window"]
    out["window_mixer_ms"] = round(timer(lambda: win.forward(x, residual, ctx, cache0, True)), 4)
    vis, kv_bytes = 0, 0
    for before in lens_before:
        for p in range(before, before + new_tokens):
            vis += min(p + 1, window)
        first = max(0, before - window + 1)
        kv_bytes += (before + new_tokens - first) * kv * 2 * hd * 2
    qk = torch.randn(n, win.q_dim + win.kv_dim, device=dev).to(bf)
    mixed = torch.empty(n, win.o_dim, dtype=bf, device=dev)
    ms = timer(lambda: attn_kernels.attention(qk, cache0, mixed, ctx, n_heads=heads, n_kv_heads=kv, head_dim=hd, scale=win.scale,
                                              window=window))
    row("window_attention", ms, 4.0 * hd * vis * heads, kv_bytes + n * heads * hd * 2 * 2)
    ms = timer(lambda: win.position.apply_normed_and_store(qk, ctx, cache0, n_heads=heads, n_kv_heads=kv, head_dim=hd, write_kv=True,
                                                           q_weight=win.q_norm, k_weight=win.k_norm, eps=1e-5, values_from_keys=True))
    # q read and written, k read, k and v written
    row("norm_rotate_store", ms, 0.0, n * (2 * heads + 3 * kv) * hd * 2)

    # ---- attention over the shared latent (layer 1) ----------------------------------------------------------
    lat, cache1 = engine.model.layers[1].block.mixer, engine.cache.layer(1)
    H, d, rd, vd, rank = s["lheads"], s["ldim"], s["lrot"], s["lvdim"], s["rank"]
    wide = rank + rd
    out["latent_mixer_ms"] = round(timer(lambda: lat.forward(x, residual, ctx, cache1, True)), 4)
    causal = sum(p + 1 for before in lens_before for p in range(before, before + new_tokens))
    q_wide = (torch.randn(n, H * wide, device=dev) * 0.3).to(bf)
    o_lat = torch.empty(H * n, rank, dtype=bf, device=dev)
    ms = timer(lambda: attn_kernels.latent_attention(q_wide, cache1, o_lat, ctx, n_heads=H, key_dim=wide, rank=rank, scale=lat.scale))
    cache_bytes = sum(before + new_tokens for before in lens_before) * wide * 2
    row("latent_attention", ms, 2.0 * (wide + rank) * causal * H, cache_bytes + n * H * (wide + rank) * 2)
    # the per-head products (queries into the latent space, latents up to values) with their lists
    from . import tcgen05
    fast = tcgen05.grouped_supports(bf, lat.w_uk_t) and tcgen05.grouped_supports(bf, lat.w_uv)
    tile_rows = tcgen05.GROUPED_TILE_ROWS if fast else ops.moe_tile_rows()
    i32 = lambda k: torch.zeros(k, dtype=torch.int32, device=dev)
    offsets, order, tiles, n_tiles = i32(H + 1), i32(H * n), i32(2 * H * (-(-n // tile_rows))), i32(1)
    proj = (torch.randn(n, lat.w_in.n, device=dev) * 0.3).to(bf)
    q_nope = torch.empty(H * n, d, dtype=bf, device=dev)
    pos = lat.position

    def prepare():
        ops.latent_prepare(proj, pos.cos, pos.sin, lat.latent_norm, lat.eps, ctx.token_pos, ctx.token_seq, ctx.seq_slot,
                           ctx.page_table, cache1.k, q_nope, q_wide, offsets, order, tiles, n_tiles, n_heads=H, head_dim=d,
                           rot_dim=rd, rank=rank, rot_dims=pos.rot_dims, style=pos.style, page_size=ctx.page_size,
                           write_kv=True, tile_rows=tile_rows)
    row("latent_prepare", timer(prepare), 0.0, n * (H * (d + rd) * 2 + wide * 2) * 2)
    lists = (offsets, order, tiles, n_tiles, fast)
    q_lat = torch.empty(H * n, rank, dtype=torch.float32, device=dev)
    v = torch.empty(H * n, vd, dtype=torch.float32, device=dev)
    if fast:        # the product's epilogue rounds its result into the wide query rows itself
        row("queries_into_latent", timer(lambda: tcgen05.grouped_gemm_spread(q_nope, lat.w_uk_t, q_wide, wide, offsets, tiles, n_tiles,
                                                                             n_pairs=H * n)),
            2.0 * n * H * d * rank, H * d * rank * 2 + n * H * (d * 2 + rank * 2))
    else:
        row("queries_into_latent", timer(lambda: lat._grouped(q_nope, lat.w_uk_t, q_lat, lists, H * n)),
            2.0 * n * H * d * rank, H * d * rank * 2 + n * H * (d * 2 + rank * 4))
        row("latent_widen", timer(lambda: ops.latent_widen(q_lat, q_wide, n_tokens=n, n_heads=H, rank=rank, rot_dim=rd)), 0.0,
            n * H * rank * 6)
    row("latents_to_values", timer(lambda: lat._grouped(o_lat, lat.w_uv, v, lists, H * n)),
        2.0 * n * H * vd * rank, H * vd * rank * 2 + n * H * (rank * 2 + vd * 4))
    gated = torch.empty(n, H * vd, dtype=bf, device=dev)
    row("latent_gate", timer(lambda: ops.latent_gate(v, proj[:, lat.w_in.n - H:], gated, n_tokens=n, n_heads=H, v_head_dim=vd)),
        0.0, n * H * vd * 6)
    out["latent_products_kernel"] = "tcgen05" if fast else "ffma"

    # ---- feed-forward ------------------------------------------------------------------------------------------
    ff = block0.feed_forward
    out["feed_forward_ms"] = round(timer(lambda: ff.forward(x, residual, ctx)), 4)
    inter = ff.intermediate_size
    act = torch.empty(n, inter, dtype=bf, device=dev)
    row("gate_up", timer(lambda: linear.gated(x, ff.w_gate, ff.w_up, act, ctx, form=ff.form)), 2.0 * n * 2 * inter * width,
        2 * inter * width * 2 + n * (width + inter) * 2)
    row("down", timer(lambda: linear.into_residual(act, ff.w_down, residual, ctx)), 2.0 * n * inter * width,
        inter * width * 2 + n * (inter * 2 + width * 8))
    engine.workspace.rezero()
    for slot in slots:
        engine.free_slot(slot)
    return out


def dense_norm_and_rope(engine, s: dict, lens_before: list, new_tokens: int, peaks: dict, timer: Timer) -> dict:
    """The dense decoder's RMS norm and rotary cache-write kernels alone (the like kernels of the layer norm and of
    the norm-rotate-store kernel)."""
    slots, ctx = _step_context(engine, lens_before, new_tokens, s["vocab"], 5)
    dev, n, width = engine.device, ctx.n_tokens, s["width"]
    block, cache0 = engine.model.layers[0].block, engine.cache.layer(0)
    out = {}

    def row(name, ms, bytes_):
        ideal = _roofline_ms(0.0, bytes_, peaks)
        out[name] = {"ms": round(ms, 4), "roofline_ms": round(ideal, 6), "x_roofline": round(ms / ideal, 2), "bound": "hbm"}
    normed = torch.empty(n, width, dtype=torch.bfloat16, device=dev)
    stream = torch.randn(n, width, device=dev)
    row("rms_norm", timer(lambda: block.mixer_norm.forward(stream, normed)), n * width * 6 + width * 4)
    m = block.mixer
    qkv = torch.randn(n, m.q_dim + 2 * m.kv_dim, device=dev).to(torch.bfloat16)
    ms = timer(lambda: m.position.apply_and_store(qkv, ctx, cache0, n_heads=m.n_heads, n_kv_heads=m.n_kv_heads, head_dim=m.head_dim,
                                                  write_kv=True))
    row("rotate_store", ms, n * (2 * m.n_heads + 4 * m.n_kv_heads) * m.head_dim * 2)
    for slot in slots:
        engine.free_slot(slot)
    return out


def main(sizes: str, peaks: dict, peak_source: str, *, prefill_tokens: int = 2048, batch: int = 8, context: int | None = None,
         steps: int = 64) -> int:
    from ..config.registry import config_from_dict
    from ..engine.engine import Engine
    s = SIZES[sizes]
    if context is None:
        context = s["window"] + s["window"] // 4        # the windowed layers see a full window, the latent ones all of it
    torch.cuda.set_device(0)
    timer = Timer("cuda:0")
    peaks = dict(peaks, fp32_ffma_tflops_nominal=round(ffma_peak_tflops(), 1))
    cache_tokens = batch * (context + steps + 128) + prefill_tokens + 4096
    result = {"arch": "vadodra", "sizes": sizes, "config": s, "layers": LAYERS, "dtype": "bf16",
              "data": "synthetic (random weights, random token ids)", "peaks": dict(peaks, source=peak_source),
              "l2": "256 MiB written between timed iterations"}
    for kind, cfg in (("vadodra", vadodra_config(s)), ("dense", dense_config(s, cache_tokens))):
        t0 = time.time()
        engine = Engine.from_random(config_from_dict(cfg), seed=0, std=0.02, dtype="bfloat16", device="cuda:0",
                                    max_tokens=cache_tokens, n_slots=batch + 2)
        print(f"[bench] {kind} ready in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
        r = throughput(engine, s, prefill_tokens=prefill_tokens, batch=batch, context=context, steps=steps, timer=timer)
        if kind == "vadodra":
            r["prefill_parts"] = time_parts(engine, s, [0], prefill_tokens, peaks, timer)
            r["decode_parts"] = time_parts(engine, s, [context] * batch, 1, peaks, timer)
        else:
            r["prefill_parts"] = dense_parts(engine, "dense", s, [0], prefill_tokens, peaks, timer)
            r["prefill_parts"].update(dense_norm_and_rope(engine, s, [0], prefill_tokens, peaks, timer))
            r["decode_parts"] = dense_parts(engine, "dense", s, [context] * batch, 1, peaks, timer)
            r["decode_parts"].update(dense_norm_and_rope(engine, s, [context] * batch, 1, peaks, timer))
        engine.check_device_status()
        result[kind] = r
        del engine
        torch.cuda.empty_cache()
    # how far each kernel of the new design is from its roofline, over the like kernel of the dense decoder
    like = {"window_attention": "attention", "latent_attention": "attention", "queries_into_latent": "gate_up",
            "latents_to_values": "down", "gate_up": "gate_up", "down": "down", "layer_norm": "rms_norm",
            "norm_rotate_store": "rotate_store", "latent_prepare": "rotate_store", "latent_widen": "rotate_store",
            "latent_gate": "rotate_store"}
    ratios = {}
    for phase in ("prefill_parts", "decode_parts"):
        for name, other in like.items():
            if name in result["vadodra"][phase]:
                ratios[f"{phase[:-6]}.{name}"] = round(result["vadodra"][phase][name]["x_roofline"]
                                                       / result["dense"][phase][other]["x_roofline"], 2)
    result["x_roofline_over_dense"] = ratios
    print(json.dumps(result))
    return 0
