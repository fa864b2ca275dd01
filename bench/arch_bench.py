"""Hybrid designs beside the framework's closest existing model.  ``--arch gokapel``: Gokapel beside Gusolorn (the other stack of recurrent
layers, attention over paged rows, dense and routed feed-forwards on an fp32 residual) at equal width, depth, heads and experts, and each of
its kernels beside the like kernel (gated delta rule / mLSTM scan, block-local attention with a sink / windowed latent attention and
differential attention, stream step with dynamic tanh / scaled residual add + norm, query/key norm + rotation + append / latent prologue,
squared-ReLU experts / clamped-GLU experts, group-limited softmax / sigmoid top-k router; minGRU against the copy roofline alone).
``--arch gifetar``: Gifetar beside Gusolorn (the other stack with an fp32
residual stream, multi-head attention over paged rows and routed experts) at equal width, depth, heads and experts, and each of its
kernels beside the like kernel (differential attention / latent attention, layer-norm residual step / scaled residual add + norm,
SiLU-GLU experts / clamped-GLU experts, softmax / sigmoid top-k router).  ``--arch gusolorn``: Gusolorn beside Perelorn (the other hybrid stack:
latent attention + recurrent layers) at equal width and depth, and each of its kernels beside the like kernel (mLSTM scan / decayed
linear-attention scan, windowed sink-free latent attention / latent attention with a sink, scaled residual add + norm / output-side norm +
add, clamped-GLU experts / the SwiGLU expert path).  ``--arch perelorn``: Perelorn beside the framework's closest existing model (DeepSeek-V2 with dense feed-forwards: latent attention, same width and
about the same weight bytes), random weights, bf16, one GPU: prefill and decode throughput of the whole stack, and the time of each
new kernel against the HBM roofline (``MEASURED_PEAKS.json``), with the like kernel of the closest model where there is one.

    python bench.py --arch perelorn|gusolorn|gifetar|gokapel [--arch-sizes 1024,2048]        (prints one JSON line per measurement)

Timing: CUDA events on the launching stream, 3 warm-up runs, an L2 flush (256 MiB write) before every timed run, median of 7.
"""
from __future__ import annotations

import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mlx_sharding_b200.config import deepseek_v2_lite_config, gifetar_config, gokapel_config, gusolorn_config, perelorn_config  # noqa: E402
from mlx_sharding_b200.ops.meta import BatchMeta  # noqa: E402
from mlx_sharding_b200.parallel.pipeline import StageExecutor  # noqa: E402
from mlx_sharding_b200.utils.loader import random_model  # noqa: E402
from mlx_sharding_b200.utils.timing import flush_l2  # noqa: E402

PS = 64


def peaks():
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "of measured"
    except Exception:
        return 6650.0, "of fallback"


def timed(fn, warm=3, reps=7):
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(reps):
        flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts)


def step_meta(B, q, ctx0, dev, slots=True):
    pages_per = (ctx0 + q + PS - 1) // PS
    bts = [list(range(1 + b * pages_per, 1 + (b + 1) * pages_per)) for b in range(B)]
    return BatchMeta.build([q] * B, [ctx0] * B, bts, PS, device=dev, state_slots=list(range(1, B + 1)) if slots else None), 1 + B * pages_per


def dense_deepseek(width, layers, vocab):
    return deepseek_v2_lite_config(hidden_size=width, num_hidden_layers=layers, n_routed_experts=None, n_shared_experts=None,
                                   intermediate_size=4 * width, vocab_size=vocab, first_k_dense_replace=layers, rope_scaling=None)


def model_runs(name, model, B_dec, ctx_dec, S_pre, dev, hybrid):
    out = {}
    meta_p, pages_p = step_meta(1, S_pre, 0, dev, hybrid)
    meta_d, pages_d = step_meta(B_dec, 1, ctx_dec - 1, dev, hybrid)
    stage = StageExecutor(model, max(pages_p, pages_d) + 1, PS, num_state_slots=B_dec + 1)
    tok_p = torch.randint(0, model.cfg.vocab_size, (S_pre,), device=dev)
    tok_d = torch.randint(0, model.cfg.vocab_size, (B_dec,), device=dev)
    ms = timed(lambda: stage.forward(tok_p, meta_p))
    out["prefill_tok_s"] = S_pre / ms * 1e3
    out["prefill_ms"] = ms
    fwd = lambda: stage.forward(tok_d, meta_d)
    ms_eager = timed(fwd)
    graph = None
    try:
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for _ in range(2):
                fwd()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fwd()
        ms = timed(graph.replay)
        out["decode_mode"] = "cuda graph"
    except Exception as e:  # noqa: BLE001
        ms, out["decode_mode"] = ms_eager, f"eager (capture failed: {type(e).__name__})"
    out["decode_tok_s"] = B_dec / ms * 1e3
    out["decode_ms"] = ms
    out["decode_eager_ms"] = ms_eager
    out["weights_gb"] = model.weight_bytes() / 1e9
    del graph
    return out


def kernel_table(width, dev, hbm):
    """Each new kernel alone at one layer's shapes: decode (B=64 sequences, context 2048) is bound by the state / pool bytes it must
    move; prefill (one 2048-token prompt) is reported as time and tokens/s."""
    from mlx_sharding_b200.ops import b200 as O

    rows = []
    H, P, N, Hl, D, Lr, R = 2 * width // 64, 64, 128, 16, 128, 512, 64
    bf = torch.bfloat16

    def add(name, ms, nbytes, like=None):
        r = dict(kernel=name, ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1), frac_hbm=round(nbytes / ms / 1e6 / hbm, 3))
        if like:
            r["like_kernel"] = like
        rows.append(r)

    for phase, B, q, ctx0 in (("decode", 64, 1, 2047), ("prefill", 1, 2048, 0)):
        meta, _ = step_meta(B, q, ctx0, dev)
        T = B * q
        # selective scan
        xbc = torch.randn(T, H * P + 2 * N, device=dev).to(bf)
        dt = torch.randn(T, H, device=dev).to(bf)
        st = torch.zeros(B + 1, H, N, P, device=dev)
        v = [torch.randn(H, device=dev) for _ in range(3)]
        ms = timed(lambda: O.ssm_scan(xbc, dt, v[0], v[1], v[2], st, meta, H, P, N, 1))
        add(f"ssm_scan {phase}", ms, 2 * B * H * N * P * 4 + T * (H * P * 6 + 2 * N * 2))
        cw, cb = torch.randn(xbc.shape[1], 4, device=dev), torch.randn(xbc.shape[1], device=dev)
        cs = torch.zeros(B + 1, 3, xbc.shape[1], device=dev, dtype=bf)
        ms = timed(lambda: O.causal_conv_silu(xbc, cw, cb, cs, meta))
        add(f"causal_conv_silu {phase}", ms, T * xbc.shape[1] * 4 + 2 * B * 3 * xbc.shape[1] * 2)
        # decayed linear attention
        qkv = torch.randn(T, Hl * (3 * D + D), device=dev).to(bf)
        st2 = torch.zeros(B + 1, Hl, D, D, device=dev)
        dec = torch.full((Hl,), 0.97, device=dev)
        ms = timed(lambda: O.decay_scan(qkv, dec, st2, meta, Hl, D, D))
        add(f"decay_scan {phase}", ms, 2 * B * Hl * D * D * 4 + T * Hl * D * (3 * 2 + 4))
        # latent attention with sink vs. the framework's absorbed-latent MLA decode kernel (same shapes: 16 heads, 512 + 64)
        pool = torch.randn(1 + B * ((ctx0 + q + PS - 1) // PS), 1, PS, Lr + R, device=dev).to(bf)
        qq = torch.randn(T, Hl, Lr + R, device=dev).to(bf)
        sink = torch.zeros(Hl, device=dev)
        inv = torch.rand(R // 2, device=dev)
        nbytes = B * (ctx0 + q) * (Lr + R) * 2 + T * Hl * (2 * Lr + R) * 2
        ms = timed(lambda: O.latent_attention(qq, pool, sink, meta, 0.07, Lr, inv))
        add(f"latent_attention(sink) {phase}", ms, nbytes)
        if phase == "decode":
            ms = timed(lambda: O.mla_decode(qq, pool, meta, 0.07))
            add("mla_decode (DeepSeek-V2 absorbed, tcgen05) decode", ms, nbytes, like="latent_attention(sink) decode")
    return rows


def gusolorn_kernel_table(width, dev, hbm):
    """Gusolorn's kernels alone at one layer's shapes beside the like kernel of Perelorn / DeepSeek-V2; bytes = what the kernel must move."""
    from mlx_sharding_b200.ops import b200 as O
    from mlx_sharding_b200.ops.weights import LinearWeight

    rows = []
    H, D, Lr, R, W = 16, 128, 512, 64, width
    bf = torch.bfloat16

    def add(name, ms, nbytes, like=None):
        r = dict(kernel=name, ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1), frac_hbm=round(nbytes / ms / 1e6 / hbm, 3))
        if like:
            r["like_kernel"] = like
        rows.append(r)

    for phase, B, q, ctx0 in (("decode", 64, 1, 2047), ("prefill", 1, 2048, 0)):
        meta, _ = step_meta(B, q, ctx0, dev)
        T = B * q
        qkv = torch.randn(T, H * 4 * D, device=dev).to(bf)
        nb = D // O.mlstm_col_block(D)
        st = dict(S=torch.zeros(B + 1, H, D, D, device=dev), n=torch.zeros(B + 1, H, nb, D, device=dev), m=torch.zeros(B + 1, H, nb, device=dev))
        gates, gb = torch.randn(T, 2 * H, device=dev), torch.randn(2 * H, device=dev)
        nbytes = 2 * B * H * D * D * 4 + T * H * D * (3 * 2 + 4)
        ms = timed(lambda: O.mlstm_scan(qkv, gates, gb, st, meta, H, D, D, 15.0, D ** -0.5))
        add(f"mlstm_scan {phase}", ms, nbytes)
        st2, dec = torch.zeros(B + 1, H, D, D, device=dev), torch.full((H,), 0.97, device=dev)
        ms = timed(lambda: O.decay_scan(qkv, dec, st2, meta, H, D, D))
        add(f"decay_scan (Perelorn) {phase}", ms, nbytes, like=f"mlstm_scan {phase}")
        pool = torch.randn(1 + B * ((ctx0 + q + PS - 1) // PS), 1, PS, Lr + R, device=dev).to(bf)
        qq = torch.randn(T, H, Lr + R, device=dev).to(bf)
        sink, inv = torch.zeros(H, device=dev), torch.rand(R // 2, device=dev)
        for win in (0, 1024):
            seen = min(ctx0 + q, win) if win else ctx0 + q
            nbytes = (B * seen if q == 1 else min(ctx0 + q, seen + q)) * (Lr + R) * 2 + T * H * (2 * Lr + R) * 2
            ms = timed(lambda: O.latent_attention(qq, pool, None, meta, 0.07, Lr, inv, window=win, interleaved=True))
            add(f"latent_attention(no sink, window {win}) {phase}", ms, nbytes)
        ms = timed(lambda: O.latent_attention(qq, pool, sink, meta, 0.07, Lr, inv))
        add(f"latent_attention(sink) (Perelorn) {phase}", ms, B * (ctx0 + q) * (Lr + R) * 2 + T * H * (2 * Lr + R) * 2, like=f"latent_attention(no sink, window 0) {phase}")
        if phase == "prefill":
            ms = timed(lambda: O.latent_attention_prefill(qq.clone(), pool, None, meta, 0.07, Lr, inv, window=1024, interleaved=True))
            add("latent_attention_prefill(GEMM form, window 1024) prefill", ms, (ctx0 + q) * (Lr + R) * 2 + T * H * (2 * Lr + R) * 2)
            ms = timed(lambda: O.latent_attention_prefill(qq.clone(), pool, sink, meta, 0.07, Lr, inv))
            add("latent_attention_prefill(GEMM form, sink) (Perelorn) prefill", ms, (ctx0 + q) * (Lr + R) * 2 + T * H * (2 * Lr + R) * 2,
                like="latent_attention_prefill(GEMM form, window 1024) prefill")
        x, y = torch.randn(T, W, device=dev), torch.randn(T, W, device=dev)
        ls, w = torch.randn(W, device=dev), torch.randn(W, device=dev)
        ms = timed(lambda: O.scaled_add_norm_(x, y, ls, w, 1e-5, bf))
        add(f"scaled_add_norm {phase}", ms, T * W * (4 + 4 + 4 + 2))
        ms = timed(lambda: O.post_norm_add_(x, y, w, 1e-5, bf))
        add(f"post_norm_add (Perelorn) {phase}", ms, T * W * (4 + 4 + 4 + 2), like=f"scaled_add_norm {phase}")
        # routed experts: 16 experts, top 2, expert width 1024
        E, F, k = 16, 1024, 2
        xa = torch.randn(T, W, device=dev).to(bf)
        wg, wu = (LinearWeight(weight=(torch.randn(E, F, W, device=dev) * W ** -0.5).to(bf)) for _ in range(2))
        wd = LinearWeight(weight=(torch.randn(E, W, F, device=dev) * F ** -0.5).to(bf))
        z = torch.randn(T, E, device=dev)
        idx, wts = O.sigmoid_topk(z, E, k)
        touched = min(E, T * k)
        nbytes = touched * 3 * F * W * 2 + T * W * (2 + 4) + T * k * (2 * W * 2 + 2 * F * 2 + 2 * W * 4)
        ms = timed(lambda: O.moe_clamped_experts(xa, idx, wts, wg, wu, wd, 7.0))
        add(f"moe_clamped_experts {phase}", ms, nbytes)
        ms = timed(lambda: O.moe_experts(xa, idx, wts, wg, wu, wd, "silu"))
        add(f"moe_experts (DeepSeek-V2, SwiGLU) {phase}", ms, nbytes, like=f"moe_clamped_experts {phase}")
        ms = timed(lambda: O.sigmoid_topk(z, E, k))
        add(f"sigmoid_topk {phase}", ms, T * E * 4 + T * k * 8)
    return rows


def gusolorn_main(sizes=(1024, 2048)):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    hbm, tag = peaks()
    for width in sizes:
        for name, cfg in (("gusolorn", gusolorn_config(width=width, vocab=32000, blocks=2, heads=16, ff=4 * width, experts=16, top=2, expert_ff=width // 2)),
                          ("perelorn", perelorn_config(width=width, vocab=32000, blocks=2, heads=16, ff=4 * width, side_dim=64))):
            m = random_model(cfg, dtype=torch.bfloat16, device=dev, seed=1)
            r = model_runs(name, m, 32, 1024, 2048, dev, True)
            print(json.dumps(dict(bench="arch", model=name, width=width, layers=len(cfg["layers"]), **{k: (round(v, 3) if isinstance(v, float) else v) for k, v in r.items()})), flush=True)
            del m
            torch.cuda.empty_cache()
    for row in gusolorn_kernel_table(sizes[-1], dev, hbm):
        print(json.dumps(dict(bench="arch-kernel", roofline=f"{hbm} GB/s {tag}", **row)), flush=True)


def gifetar_kernel_table(width, dev, hbm):
    """Gifetar's kernels alone at one layer's shapes beside the like kernel of Gusolorn; bytes = what the kernel must move.  The prefill
    attention is bound by arithmetic, so it also reports TFLOP/s (both maps: 2 * heads * (dim + vdim) multiply-adds per visible key)."""
    from mlx_sharding_b200.ops import b200 as O
    from mlx_sharding_b200.ops.weights import LinearWeight

    rows = []
    H, G, D, V, W = 16, 4, 64, 128, width
    Hl, Lr, R = 16, 512, 64
    bf = torch.bfloat16

    def add(name, ms, nbytes, like=None, flops=None):
        r = dict(kernel=name, ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1), frac_hbm=round(nbytes / ms / 1e6 / hbm, 3))
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1)
        if like:
            r["like_kernel"] = like
        rows.append(r)

    for phase, B, q, ctx0 in (("decode", 64, 1, 2047), ("prefill", 1, 2048, 0)):
        meta, _ = step_meta(B, q, ctx0, dev, False)
        T, npg = B * q, 1 + B * ((ctx0 + q + PS - 1) // PS)
        kp, vp = torch.randn(npg, G, PS, 2 * D, device=dev).to(bf), torch.randn(npg, G, PS, V, device=dev).to(bf)
        u = torch.randn(T, (H + G) * 2 * D + G * V, device=dev).to(bf)
        nbytes = B * (ctx0 + q) * G * (2 * D + V) * 2 + T * H * (2 * D + V) * 2
        pairs = B * (ctx0 + q) if q == 1 else (ctx0 + q) * (ctx0 + q + 1) // 2
        flops = 2 * 2 * H * (D + V) * pairs
        args = (H, D ** -0.5, 30.0, 0.1, 1024.0, 0.7, 1e-5, 0.2, bf)
        ms = timed(lambda: O.diff_attention(u, kp, vp, meta, *args))
        add(f"diff_attention {phase}", ms, nbytes, flops=flops)
        ms = timed(lambda: O.paged_kv_append(u, H * 2 * D, (H + G) * 2 * D, kp, vp, meta))
        add(f"paged_kv_append {phase}", ms, 2 * T * G * (2 * D + V) * 2)
        pool = torch.randn(npg, 1, PS, Lr + R, device=dev).to(bf)
        qq = torch.randn(T, Hl, Lr + R, device=dev).to(bf)
        inv = torch.rand(R // 2, device=dev)
        lbytes = B * (ctx0 + q) * (Lr + R) * 2 + T * Hl * (2 * Lr + R) * 2
        lflops = 2 * Hl * (2 * Lr + R) * pairs
        ms = timed(lambda: O.latent_attention(qq, pool, None, meta, 0.07, Lr, inv, window=0, interleaved=True))
        add(f"latent_attention(no sink, no window) (Gusolorn) {phase}", ms, lbytes, like=f"diff_attention {phase}", flops=lflops)
        if phase == "prefill":
            ms = timed(lambda: O.diff_attention_prefill(u, kp, vp, meta, *args))
            add("diff_attention_prefill(GEMM form) prefill", ms, nbytes, flops=flops)
            ms = timed(lambda: O.latent_attention_prefill(qq.clone(), pool, None, meta, 0.07, Lr, inv, window=0, interleaved=True))
            add("latent_attention_prefill(GEMM form) (Gusolorn) prefill", ms, lbytes, like="diff_attention_prefill(GEMM form) prefill", flops=lflops)
        x, y = torch.randn(T, W, device=dev), torch.randn(T, W, device=dev)
        v4 = [torch.randn(W, device=dev) for _ in range(4)]
        ms = timed(lambda: O.post_layernorm_add_norm_(x, y, v4[0], v4[1], 0.5, v4[2], v4[3], 1e-5, bf))
        add(f"post_layernorm_add_norm {phase}", ms, T * W * (4 + 4 + 4 + 2))
        ms = timed(lambda: O.scaled_add_norm_(x, y, v4[0], v4[1], 1e-5, bf))
        add(f"scaled_add_norm (Gusolorn) {phase}", ms, T * W * (4 + 4 + 4 + 2), like=f"post_layernorm_add_norm {phase}")
        ms = timed(lambda: O.layernorm_cast(x, v4[0], v4[1], 1e-5, bf))
        add(f"layernorm_cast {phase}", ms, T * W * (4 + 2))
        ms = timed(lambda: O.rmsnorm_cast(x, v4[0], 1e-5, bf))
        add(f"rmsnorm_cast (Gusolorn) {phase}", ms, T * W * (4 + 2), like=f"layernorm_cast {phase}")
        # routed experts: 16 experts, top 2, expert width 1024
        E, F, k = 16, 1024, 2
        xa = torch.randn(T, W, device=dev).to(bf)
        wg, wu = (LinearWeight(weight=(torch.randn(E, F, W, device=dev) * W ** -0.5).to(bf)) for _ in range(2))
        wd = LinearWeight(weight=(torch.randn(E, W, F, device=dev) * F ** -0.5).to(bf))
        z, zb = torch.randn(T, E, device=dev), torch.randn(E, device=dev)
        idx, wts = O.softmax_topk(z, zb, E, k)
        touched = min(E, T * k)
        nbytes = touched * 3 * F * W * 2 + T * W * (2 + 4) + T * k * (2 * W * 2 + 2 * F * 2 + 2 * W * 4)
        ms = timed(lambda: O.moe_glu_experts(xa, idx, wts, wg, wu, wd))
        add(f"moe_glu_experts {phase}", ms, nbytes)
        ms = timed(lambda: O.moe_clamped_experts(xa, idx, wts, wg, wu, wd, 7.0))
        add(f"moe_clamped_experts (Gusolorn) {phase}", ms, nbytes, like=f"moe_glu_experts {phase}")
        ms = timed(lambda: O.softmax_topk(z, zb, E, k))
        add(f"softmax_topk {phase}", ms, T * E * 4 + T * k * 8)
        ms = timed(lambda: O.sigmoid_topk(z, E, k))
        add(f"sigmoid_topk (Gusolorn) {phase}", ms, T * E * 4 + T * k * 8, like=f"softmax_topk {phase}")
    return rows


def gifetar_main(sizes=(1024, 2048)):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    hbm, tag = peaks()
    for width in sizes:
        for name, cfg in (("gifetar", gifetar_config(width=width, vocab=32000, layers=8, heads=16, kv_heads=4, dim=64, vdim=128, experts=16, top=2, expert_ff=width // 2)),
                          ("gusolorn", gusolorn_config(width=width, vocab=32000, blocks=2, heads=16, ff=4 * width, experts=16, top=2, expert_ff=width // 2))):
            m = random_model(cfg, dtype=torch.bfloat16, device=dev, seed=1)
            r = model_runs(name, m, 32, 1024, 2048, dev, name != "gifetar")
            print(json.dumps(dict(bench="arch", model=name, width=width, layers=len(cfg["layers"]), **{k: (round(v, 3) if isinstance(v, float) else v) for k, v in r.items()})), flush=True)
            del m
            torch.cuda.empty_cache()
    for row in gifetar_kernel_table(sizes[-1], dev, hbm):
        print(json.dumps(dict(bench="arch-kernel", roofline=f"{hbm} GB/s {tag}", **row)), flush=True)


def gokapel_kernel_table(width, dev, hbm):
    """Gokapel's kernels alone at one layer's shapes beside the like kernel of Gusolorn (and of Gifetar for the attention); bytes = what the
    kernel must move.  Decode = 64 sequences at context 2048, prefill = one 2048-token prompt; attention blocks of 1024 positions."""
    from mlx_sharding_b200.ops import b200 as O
    from mlx_sharding_b200.ops.weights import LinearWeight

    rows = []
    H, G, D, V, W, S, BLK = 16, 4, 128, 128, width, 2, 1024
    Hl, Lr, R = 16, 512, 64
    bf = torch.bfloat16

    def add(name, ms, nbytes, like=None, flops=None):
        r = dict(kernel=name, ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1), frac_hbm=round(nbytes / ms / 1e6 / hbm, 3))
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1)
        if like:
            r["like_kernel"] = like
        rows.append(r)

    for phase, B, q, ctx0 in (("decode", 64, 1, 2047), ("prefill", 1, 2048, 0)):
        meta, _ = step_meta(B, q, ctx0, dev, True)
        T, npg = B * q, 1 + B * ((ctx0 + q + PS - 1) // PS)
        # ---- recurrences: state [slots, H, D, V] fp32 read and written once per step
        st = torch.zeros(B + 1, H, D, V, device=dev)
        qkv = torch.randn(T, 2 * H * D + H * V, device=dev).to(bf)
        beta, dt = torch.randn(T, H, device=dev).to(bf), torch.randn(T, H * D, device=dev)
        dtb, alog = torch.randn(H * D, device=dev) - 1.0, torch.log(torch.rand(H, device=dev) + 0.1)
        sbytes = (2 * B * H * D * V * 4 if q == 1 else 0) + T * (2 * H * D + H * V) * 2 + T * H * D * 4 + T * H * V * 4
        ms = timed(lambda: O.delta_scan(qkv, beta, dt, dtb, alog, st, meta, H, H, D, V, D ** -0.5))
        add(f"delta_scan {phase}", ms, sbytes)
        nb = V // O.mlstm_col_block(V)
        mst = dict(S=torch.zeros(B + 1, H, D, V, device=dev), n=torch.zeros(B + 1, H, nb, D, device=dev), m=torch.zeros(B + 1, H, nb, device=dev))
        gates, gb = torch.randn(T, 2 * H, device=dev), torch.randn(2 * H, device=dev)
        ms = timed(lambda: O.mlstm_scan(qkv, gates, gb, mst, meta, H, D, V, 15.0, D ** -0.5))
        add(f"mlstm_scan (Gusolorn) {phase}", ms, sbytes - T * H * D * 4, like=f"delta_scan {phase}")
        Rw = W
        zxg, gst = torch.randn(T, 3 * Rw, device=dev).to(bf), torch.zeros(B + 1, Rw, device=dev)
        ms = timed(lambda: O.mingru_scan(zxg, 0, Rw, 2 * Rw, Rw, gst, meta, 0.5, bf))
        add(f"mingru_scan {phase}", ms, T * Rw * (3 * 2 + 2) + (2 * B * Rw * 4 if q == 1 else 0))
        C = 2 * H * D + H * V
        cw, cb, cst = torch.randn(C, 4, device=dev), torch.zeros(C, device=dev), torch.zeros(B + 1, 3, C, device=dev).to(bf)
        ms = timed(lambda: O.causal_conv_silu(qkv, cw, cb, cst, meta))
        add(f"causal_conv_silu (shared with Perelorn) {phase}", ms, T * C * 4 + (2 * B * 3 * C * 2 if q == 1 else 0))
        # ---- attention: keys visible inside the query's block of BLK positions
        kp, vp = torch.randn(npg, G, PS, D, device=dev).to(bf), torch.randn(npg, G, PS, V, device=dev).to(bf)
        u = torch.randn(T, H * D + G * D + G * V, device=dev).to(bf)
        qn, sink = 1 + 0.1 * torch.randn(D, device=dev), torch.randn(H, device=dev)
        inv = (10000.0 ** (-2.0 * torch.arange(D // 4, dtype=torch.float64) / (D // 2))).float().to(dev)
        qf = O.qk_norm_rope_append(u, 0, H * D, H * D + G * D, H, D, qn, qn, 1e-6, inv, kp, vp, meta)
        seen = min(BLK, ctx0 + q)
        pairs = B * (((ctx0 + q - 1) % BLK) + 1) if q == 1 else sum(((p % BLK) + 1) for p in range(ctx0 + q))
        abytes = (B * seen * G * (D + V) * 2 if q == 1 else (ctx0 + q) * G * (D + V) * 2) + T * H * (D * 4 + V * 2)
        aflops = 2 * H * (D + V) * pairs
        ms = timed(lambda: O.sink_attention(qf, kp, vp, sink, meta, D ** -0.5, BLK, 0, 0.6, bf))
        add(f"sink_attention(block {BLK}) {phase}", ms, abytes, flops=aflops)
        if phase == "prefill":
            ms = timed(lambda: O.sink_attention_prefill(qf, kp, vp, sink, meta, D ** -0.5, BLK, 0, 0.6, bf))
            add(f"sink_attention_prefill(GEMM form, block {BLK}) prefill", ms, abytes, flops=aflops)
        ms = timed(lambda: O.qk_norm_rope_append(u, 0, H * D, H * D + G * D, H, D, qn, qn, 1e-6, inv, kp, vp, meta))
        add(f"qk_norm_rope_append {phase}", ms, T * (H * D + G * D + G * V) * 2 + T * H * D * 4 + T * G * (D + V) * 2)
        pool = torch.randn(npg, 1, PS, Lr + R, device=dev).to(bf)
        qq = torch.randn(T, Hl, Lr + R, device=dev).to(bf)
        linv = torch.rand(R // 2, device=dev)
        lpairs = B * min(BLK, ctx0 + q) if q == 1 else sum(min(BLK, p + 1) for p in range(ctx0 + q))
        lbytes = (B * seen * (Lr + R) * 2 if q == 1 else (ctx0 + q) * (Lr + R) * 2) + T * Hl * (2 * Lr + R) * 2
        ms = timed(lambda: O.latent_attention(qq, pool, None, meta, 0.07, Lr, linv, window=BLK, interleaved=True))
        add(f"latent_attention(window {BLK}) (Gusolorn) {phase}", ms, lbytes, like=f"sink_attention(block {BLK}) {phase}", flops=2 * Hl * (2 * Lr + R) * lpairs)
        if phase == "prefill":
            ms = timed(lambda: O.latent_attention_prefill(qq.clone(), pool, None, meta, 0.07, Lr, linv, window=BLK, interleaved=True))
            add(f"latent_attention_prefill(GEMM form, window {BLK}) (Gusolorn) prefill", ms, lbytes, like=f"sink_attention_prefill(GEMM form, block {BLK}) prefill",
                flops=2 * Hl * (2 * Lr + R) * lpairs)
        dq = torch.randn(T, Lr + R, device=dev).to(bf)
        ms = timed(lambda: O.latent_kv_prologue(dq, 0, Lr, None, torch.ones(Lr, device=dev), 1e-6, pool, meta, linv, interleaved=True))
        add(f"latent_kv_prologue (Gusolorn) {phase}", ms, 2 * T * (Lr + R) * 2, like=f"qk_norm_rope_append {phase}")
        kp2 = torch.randn(npg, G, PS, D, device=dev).to(bf)            # differential attention: two maps of 64 = the same key bytes
        u2 = torch.randn(T, (H + G) * D + G * V, device=dev).to(bf)
        dpairs = B * (ctx0 + q) if q == 1 else (ctx0 + q) * (ctx0 + q + 1) // 2
        dbytes = B * (ctx0 + q) * G * (D + V) * 2 + T * H * (D + V) * 2
        ms = timed(lambda: O.diff_attention(u2, kp2, vp, meta, H, 0.125, 30.0, 0.1, 1024.0, 0.7, 1e-5, 0.2, bf))
        add(f"diff_attention(no block limit) (Gifetar) {phase}", ms, dbytes, like=f"sink_attention(block {BLK}) {phase}", flops=2 * 2 * H * (D // 2 + V) * dpairs)
        # ---- sublayer boundary
        xs, y, gate = torch.randn(T, S, W, device=dev), torch.randn(T, W, device=dev), torch.randn(T, W, device=dev).to(bf)
        v4 = [torch.randn(W, device=dev) for _ in range(3)]
        mix, ow, iw = torch.eye(S, device=dev), torch.ones(S, device=dev), torch.ones(S, device=dev) / S
        ms = timed(lambda: O.hyper_step_(xs, y, None, gate, v4[0], mix, ow, 0.5, iw, 0.7, v4[1], v4[2], bf))
        add(f"hyper_step({S} streams, gate) {phase}", ms, T * W * (2 * S * 4 + 4 + 2 + 2))
        x1 = torch.randn(T, W, device=dev)
        ms = timed(lambda: O.scaled_add_norm_(x1, y, v4[0], v4[1], 1e-5, bf))
        add(f"scaled_add_norm (Gusolorn) {phase}", ms, T * W * (4 + 4 + 4 + 2), like=f"hyper_step({S} streams, gate) {phase}")
        # ---- routed experts: 16 experts, top 2, expert width 1024
        E, F, k = 16, 1024, 2
        xa = torch.randn(T, W, device=dev).to(bf)
        wg, wu = (LinearWeight(weight=(torch.randn(E, F, W, device=dev) * W ** -0.5).to(bf)) for _ in range(2))
        wd = LinearWeight(weight=(torch.randn(E, W, F, device=dev) * F ** -0.5).to(bf))
        z, corr = torch.randn(T, E, device=dev), 0.05 * torch.randn(E, device=dev)
        idx, wts = O.group_softmax_topk(z, corr, E, k, 4, 2)
        touched = min(E, T * k)
        ms = timed(lambda: O.moe_relu2_experts(xa, idx, wts, wu, wd))
        add(f"moe_relu2_experts {phase}", ms, touched * 2 * F * W * 2 + T * W * (2 + 4) + T * k * (2 * W * 2 + 2 * F * 2 + 2 * W * 4))
        ms = timed(lambda: O.moe_clamped_experts(xa, idx, wts, wg, wu, wd, 7.0))
        add(f"moe_clamped_experts (Gusolorn) {phase}", ms, touched * 3 * F * W * 2 + T * W * (2 + 4) + T * k * (2 * W * 2 + 2 * F * 2 + 2 * W * 4),
            like=f"moe_relu2_experts {phase}")
        ms = timed(lambda: O.group_softmax_topk(z, corr, E, k, 4, 2))
        add(f"group_softmax_topk {phase}", ms, T * E * 4 + T * k * 8)
        ms = timed(lambda: O.sigmoid_topk(z, E, k))
        add(f"sigmoid_topk (Gusolorn) {phase}", ms, T * E * 4 + T * k * 8, like=f"group_softmax_topk {phase}")
        wup = LinearWeight(weight=(torch.randn(4 * W, W, device=dev) * W ** -0.5).to(bf))
        ms = timed(lambda: O.linear_any(xa, wup, bf, "relu2"))
        add(f"up projection + squared ReLU (GEMM epilogue) {phase}", ms, 4 * W * W * 2 + T * W * 2 + T * 4 * W * 2, flops=2 * T * 4 * W * W)
        ms = timed(lambda: O.linear_any(xa, wup, bf, "gelu_erf"))
        add(f"up projection + exact gelu (GEMM, then kernel) (Gusolorn) {phase}", ms, 4 * W * W * 2 + T * W * 2 + T * 4 * W * 2, flops=2 * T * 4 * W * W,
            like=f"up projection + squared ReLU (GEMM epilogue) {phase}")
    return rows


def gokapel_main(sizes=(1024, 2048)):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    hbm, tag = peaks()
    for width in sizes:
        for name, cfg in (("gokapel", gokapel_config(width=width, vocab=32000, blocks=2, heads=16, kv_heads=4, dim=128, vdim=128, ff=4 * width, experts=16, top=2,
                                                     expert_ff=width // 2, block_size=1024, gru_width=width)),
                          ("gusolorn", gusolorn_config(width=width, vocab=32000, blocks=2, heads=16, ff=4 * width, experts=16, top=2, expert_ff=width // 2))):
            m = random_model(cfg, dtype=torch.bfloat16, device=dev, seed=1)
            r = model_runs(name, m, 32, 1024, 2048, dev, True)
            print(json.dumps(dict(bench="arch", model=name, width=width, layers=len(cfg["layers"]), **{k: (round(v, 3) if isinstance(v, float) else v) for k, v in r.items()})), flush=True)
            del m
            torch.cuda.empty_cache()
    for row in gokapel_kernel_table(sizes[-1], dev, hbm):
        print(json.dumps(dict(bench="arch-kernel", roofline=f"{hbm} GB/s {tag}", **row)), flush=True)


def main(sizes=(1024, 2048), arch="perelorn"):
    if arch == "gokapel":
        return gokapel_main(sizes)
    if arch == "gusolorn":
        return gusolorn_main(sizes)
    if arch == "gifetar":
        return gifetar_main(sizes)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    hbm, tag = peaks()
    for width in sizes:
        pc = perelorn_config(width=width, vocab=32000, blocks=2, heads=16, ff=4 * width, side_dim=64)
        pm = random_model(pc, dtype=torch.bfloat16, device=dev, seed=1)
        pbytes = pm.weight_bytes()
        r = model_runs("perelorn", pm, 32, 1024, 2048, dev, True)
        print(json.dumps(dict(bench="arch", model="perelorn", width=width, layers=len(pc["layers"]), **{k: (round(v, 3) if isinstance(v, float) else v) for k, v in r.items()})), flush=True)
        del pm
        torch.cuda.empty_cache()
        # closest existing model at about equal weight bytes: pick its depth from the bytes of a 1- and a 2-layer build
        b1 = random_model(dense_deepseek(width, 1, 32000), dtype=torch.bfloat16, device=dev, seed=1).weight_bytes()
        b2 = random_model(dense_deepseek(width, 2, 32000), dtype=torch.bfloat16, device=dev, seed=1).weight_bytes()
        layers = max(1, round((pbytes - (2 * b1 - b2)) / (b2 - b1)))
        dm = random_model(dense_deepseek(width, layers, 32000), dtype=torch.bfloat16, device=dev, seed=1)
        r = model_runs("deepseek_v2-dense", dm, 32, 1024, 2048, dev, False)
        print(json.dumps(dict(bench="arch", model="deepseek_v2 (dense ff)", width=width, layers=layers, **{k: (round(v, 3) if isinstance(v, float) else v) for k, v in r.items()})), flush=True)
        del dm
        torch.cuda.empty_cache()
    for row in kernel_table(sizes[-1], dev, hbm):
        print(json.dumps(dict(bench="arch-kernel", roofline=f"{hbm} GB/s {tag}", **row)), flush=True)


if __name__ == "__main__":
    main(tuple(int(x) for x in sys.argv[1].split(",")) if len(sys.argv) > 1 else (1024, 2048), sys.argv[2] if len(sys.argv) > 2 else "perelorn")
