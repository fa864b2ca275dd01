"""``b200`` op backend: the hand-written sm_100a kernels behind the same API as ``ops.reference``.

Loading is strict: if the extension is missing (or is not loadable) on a box with a GPU this raises —
there is no silent PyTorch fallback on the hot path.  The only non-kernel code here is argument
plumbing (views, dtype checks) and the token->sequence map derived from the step metadata.
"""
from __future__ import annotations

import importlib.util
import os
from typing import Optional, Tuple

import torch

from .meta import BatchMeta
from .weights import LinearWeight, RopeSpec

NAME = "b200"
_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_b200_C.so")
_C = None

ACT_IDS = {"none": 0, "silu": 1, "gelu_tanh": 2, "gelu_pytorch_tanh": 2, "gelu_approx": 2}


def load_extension(build_if_missing: bool = False):
    """Import the in-tree ``_b200_C.so`` (optionally building it first with ``ops/build.py``)."""
    global _C
    if _C is not None:
        return _C
    if not os.path.exists(_SO):
        if build_if_missing:
            from .build import build

            build()
        else:
            raise ImportError(
                f"{_SO} not found: build the sm_100a extension with `python -m mlx_sharding_b200.ops.build` "
                "(or __graft_entry__.build())")
    spec = importlib.util.spec_from_file_location("_b200_C", _SO)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    _C = mod
    if torch.cuda.is_available():
        # persistent scratch (split-K / attention-split workspace, tile tickets) must exist before any
        # CUDA-graph capture
        mod.init_scratch(torch.cuda.current_device(), 32 << 20)
    return _C


def C():
    return load_extension()


def is_available() -> bool:
    return os.path.exists(_SO) and torch.cuda.is_available()


def _bf16(t: torch.Tensor) -> torch.Tensor:
    if t.dtype != torch.bfloat16:
        raise TypeError(f"b200 backend runs bf16 activations/weights, got {t.dtype}")
    return t


def _dense(W: LinearWeight) -> torch.Tensor:
    """bf16 ``[.., N, K]`` view of a weight.  Only used for bf16 checkpoints and for quantised layouts the in-kernel
    dequant GEMM does not cover (2-bit, odd group sizes; expert-parallel banks): those are expanded once at
    first use.  int4 / int8 group-64/128 weights take :func:`_qpack` and stay packed in HBM."""
    if W.is_quantized:
        if W.weight is None:
            W.weight = W.dense(torch.bfloat16).contiguous()
        return W.weight
    return _bf16(W.weight)


_qpack_warned = []


def _qpack(W: LinearWeight):
    """(packed int32 codes [rows, words], scales_t, biases_t [K/g, rows]) for the in-kernel dequant GEMM, or None
    when the layout is not supported by the kernel (then the weight is expanded to bf16 once)."""
    if not W.is_quantized:
        return None
    qt = getattr(W, "_qt", None)
    if qt is None:
        K = W.in_features
        if not C().gemm_q_supported(W.bits, W.group_size, K) or W.scales.dtype != torch.bfloat16:
            if W.scales.dtype != torch.bfloat16 and not _qpack_warned:
                import logging

                logging.getLogger(__name__).warning(
                    "quantised weights with %s scale tables: the in-kernel dequant GEMM takes bf16 tables, so these weights are "
                    "dequantised exactly (stored-precision scales) to bf16 once at first use instead", W.scales.dtype)
                _qpack_warned.append(True)
            W._qt = False
            return None
        rows = W.wq.numel() // W.wq.shape[-1]
        ng = K // W.group_size
        wq = W.wq.reshape(rows, W.wq.shape[-1]).contiguous()
        if W.bits == 4:
            # load-time re-pack (same bits, kernel-friendly order): nibble j <- code 2j, nibble 4+j <- code 2j+1, so the
            # kernel's (w >> 4i) & 0x000F000F yields the adjacent pair (v_2i, v_2i+1) directly
            from ..utils import quant as _q

            wq = _q.repack_int4_pairs(wq).contiguous()
        st = W.scales.reshape(rows, ng).t().contiguous()
        bt = W.biases.reshape(rows, ng).t().contiguous()
        qt = (wq, st, bt)
        W._qt = qt
    return qt or None


# ------------------------------------------------------------------------------------------------ ops
def embed(ids: torch.Tensor, emb: LinearWeight, scale: float = 1.0, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    ids = ids.to(torch.int64).contiguous()
    if emb.is_quantized:
        return C().embed(ids, emb.wq, emb.scales, emb.biases, emb.bits, emb.group_size, float(scale))
    return C().embed(ids, _bf16(emb.weight), None, None, 0, 64, float(scale))


def rmsnorm(x, w, eps: float, gemma: bool = False, residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
            signal: Optional[Tuple[int, int]] = None):
    """``out`` / ``signal``: fused stage boundary — the norm stores straight into the next stage's inbox (peer memory) and the
    last CTA raises its flag (Gemma-2 stages end in a norm, not in a GEMM)."""
    flag, val = signal if signal is not None else (0, 0)
    return C().rmsnorm(x, w, float(eps), bool(gemma), residual, out, int(flag), int(val))


def add_rmsnorm(x, residual, w, eps, gemma=False):
    h = x + residual
    return rmsnorm(h, w, eps, gemma), h


def linear(x: torch.Tensor, W: LinearWeight, residual: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None,
           signal: Optional[Tuple[int, int]] = None, softcap: float = 0.0) -> torch.Tensor:
    fp32 = out_dtype == torch.float32
    flag, val = signal if signal is not None else (0, 0)
    q = _qpack(W)
    if q is not None:
        return C().linear_q(x, q[0], q[1], q[2], None, None, None, W.bits, W.group_size, W.out_features, residual, W.bias, 0,
                            float(softcap), fp32, out, 0, int(flag), int(val))
    return C().linear(x, _dense(W), None, residual, W.bias, 0, float(softcap), fp32, out, 0, int(flag), int(val))


def gated_up(x: torch.Tensor, Wg: LinearWeight, Wu: LinearWeight, act: str = "silu") -> torch.Tensor:
    if Wg.bias is not None or Wu.bias is not None:
        raise NotImplementedError("gated MLP with bias")
    qg, qu = _qpack(Wg), _qpack(Wu)
    if qg is not None and qu is not None:
        return C().linear_q(x, qg[0], qg[1], qg[2], qu[0], qu[1], qu[2], Wg.bits, Wg.group_size, Wg.out_features, None, None,
                            ACT_IDS[act], 0.0, False, None, 0, 0, 0)
    return C().linear(x, _dense(Wg), _dense(Wu), None, None, ACT_IDS[act], 0.0, False, None, 0, 0, 0)


def rope_(x: torch.Tensor, positions: torch.Tensor, spec: RopeSpec, rot_offset: int = 0) -> torch.Tensor:
    C().rope_(x, positions, spec.inv_freq, int(rot_offset), int(spec.rot_dim), bool(spec.interleaved), float(spec.mscale))
    return x


def kv_write(k, v, kpool, vpool, slot_mapping):
    C().kv_write(k, v, kpool, vpool, slot_mapping)


def kv_write_mla(kv, k_pe, kpool, vpool, slot_mapping, nope: int, vdim: int):
    C().kv_write_mla(kv, k_pe, kpool, vpool, slot_mapping, int(nope), int(vdim))


def _token_seq(meta: BatchMeta) -> torch.Tensor:
    ts = getattr(meta, "_token_seq", None)
    if ts is None:
        if meta.num_tokens == meta.num_seqs:
            ts = torch.arange(meta.num_seqs, dtype=torch.int32, device=meta.positions.device)
        else:
            lens = (meta.cu_seqlens[1:] - meta.cu_seqlens[:-1]).long()
            ts = torch.repeat_interleave(torch.arange(meta.num_seqs, device=lens.device), lens).to(torch.int32)
        meta._token_seq = ts
    return ts


def paged_attention(q, kpool, vpool, meta: BatchMeta, scale: float, softcap: float = 0.0):
    c = C()
    if meta.max_q_len > 1 and not softcap and c.flash_prefill_supported(kpool.shape[3], vpool.shape[3]):
        # prefill chunk / mixed batch: tensor-core causal flash attention over the paged cache
        return c.flash_prefill(q, kpool, vpool, meta.block_tables, meta.cu_seqlens, meta.context_lens, float(scale),
                               int(meta.num_tokens))
    return C().paged_attention(q, kpool, vpool, meta.block_tables, meta.positions, _token_seq(meta), float(scale),
                               float(softcap or 0.0), int(meta.max_ctx_len))


def moe_route(x, gate_w, top_k: int, method: str = "greedy", n_group: int = 1, topk_group: int = 1,
              scaling: float = 1.0, norm_topk: bool = False, extra: int = 0):
    """``extra``: always-on experts appended to the routed bank (ids E .. E+extra-1, weight 1.0) — see ``fuse_shared_experts``."""
    if method != "group_limited_greedy":
        n_group, topk_group = 1, 1
    idx, w = C().moe_route(x, _bf16(gate_w), int(top_k), int(n_group), int(topk_group), float(scaling), bool(norm_topk), int(extra))
    return idx, w


class _Join:
    """Handle of work forked onto the side stream by :func:`run_aside`; ``wait()`` joins it into the current stream."""

    def __init__(self, event):
        self.event = event

    def wait(self):
        torch.cuda.current_stream().wait_event(self.event)
        C().pdl_skip_next()  # the joining kernel depends on two streams: plain dependencies, no programmatic edge


_side_streams = {}


def run_aside(fn) -> _Join:
    """Run ``fn()`` on this device's side stream, forked from the current stream (event record / wait, so it is also legal
    inside CUDA-graph capture and becomes a parallel branch of the graph).  Used to run the shared-expert GEMMs of a
    DeepSeek MoE block concurrently with the router / permutation / expert all-to-all, which do not depend on them.
    ``fn`` must write its result into a tensor allocated *before* the fork."""
    cur = torch.cuda.current_stream()
    side = _side_streams.get(cur.device.index)
    if side is None:
        side = _side_streams[cur.device.index] = torch.cuda.Stream(device=cur.device)
    fork = torch.cuda.Event()
    fork.record(cur)
    side.wait_event(fork)
    with torch.cuda.stream(side):
        C().pdl_skip_next()  # first side kernel depends on the other stream
        fn()
        done = torch.cuda.Event()
        done.record(side)
    return _Join(done)


_aside_last = {}


def prefetch_aside(tensors, nbytes_each: int):
    """Start pulling the first ``nbytes_each`` bytes of every tensor into L2 on the side stream (forked from the current stream at
    this point, NOT joined here: nothing depends on a prefetch — :func:`join_aside` ties the side stream back once per forward so
    a graph capture ends with all its branches joined).  The main stream's kernel chain keeps its programmatic (PDL) edges."""
    cur = torch.cuda.current_stream()
    dev = cur.device.index
    side = _side_streams.get(dev)
    if side is None:
        side = _side_streams[dev] = torch.cuda.Stream(device=cur.device)
    fork = torch.cuda.Event()
    fork.record(cur)
    side.wait_event(fork)
    with torch.cuda.stream(side):
        for t in tensors:
            C().l2_prefetch(t, 0, min(int(nbytes_each), t.numel() * t.element_size()) // 16 * 16)
        done = torch.cuda.Event()
        done.record(side)
    _aside_last[dev] = done


def join_aside():
    """Join the side stream's outstanding prefetches into the current stream (end of a forward pass)."""
    cur = torch.cuda.current_stream()
    ev = _aside_last.pop(cur.device.index, None)
    if ev is not None:
        cur.wait_event(ev)
        C().pdl_skip_next()


def l2_prefetch_bytes() -> int:
    """Bytes of the next MoE block's gate / up banks (each) to prefetch into L2 during a decode layer's attention chain
    (``MLXB200_L2_PREFETCH_MB``, total across both banks; 0 = off)."""
    try:
        return int(float(os.environ.get("MLXB200_L2_PREFETCH_MB", "0")) * (1 << 20)) // 2
    except ValueError:
        return 0


def moe_experts(x, idx, w, Wg: LinearWeight, Wu: LinearWeight, Wd: LinearWeight, act: str = "silu",
                extra: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, signal: Optional[Tuple[int, int]] = None, join: Optional[_Join] = None):
    """router output -> permute -> grouped dual GEMM (act(gate)*up) -> grouped down GEMM (fp32) ->
    weighted combine (+ residual [+ P2P store & flag])."""
    c = C()
    T, k = idx.shape
    if fp8_experts_enabled(Wg) and x.shape[1] % 128 == 0:
        (gq, gs), (uq, us), (dq, ds) = _fp8pack(Wg), _fp8pack(Wu), _fp8pack(Wd)
        E = gq.shape[0]
        offs, pair_row, xp = c.moe_permute(idx, x, E)
        xq, xsf = c.quant_mxfp8(xp)
        h = c.linear_fp8(xq, xsf, gq, gs, uq, us, offs, T, None, ACT_IDS[act], False, 0, 0)
        hq, hsf = c.quant_mxfp8(h)
        y = c.linear_fp8(hq, hsf, dq, ds, None, None, offs, T, None, 0, True, 0, 0)
        if extra is not None:
            residual = extra if residual is None else residual + extra
        flag, val = signal if signal is not None else (0, 0)
        if join is not None:
            join.wait()
        return c.moe_combine(y, pair_row, w, residual, out, int(k), int(flag), int(val))
    qg, qu, qd = _qpack(Wg), _qpack(Wu), _qpack(Wd)
    if qg is not None and qu is not None and qd is not None:
        E = Wg.wq.shape[0]
        offs, pair_row, xp = c.moe_permute(idx, x, E)
        h = c.grouped_linear_q(xp, qg[0], qg[1], qg[2], qu[0], qu[1], qu[2], Wg.bits, Wg.group_size, E, Wg.out_features,
                               offs, T, ACT_IDS[act], False)
        y = c.grouped_linear_q(h, qd[0], qd[1], qd[2], None, None, None, Wd.bits, Wd.group_size, E, Wd.out_features, offs, T,
                               0, True)
    else:
        wg, wu, wd = _dense(Wg), _dense(Wu), _dense(Wd)
        E = wg.shape[0]
        offs, pair_row, xp = c.moe_permute(idx, x, E)
        h = c.grouped_linear(xp, wg, wu, offs, T, ACT_IDS[act], False)
        y = c.grouped_linear(h, wd, None, offs, T, 0, True)
    if extra is not None:
        residual = extra if residual is None else residual + extra
    flag, val = signal if signal is not None else (0, 0)
    if join is not None:
        join.wait()  # ``residual`` is produced on the side stream (shared experts)
    return c.moe_combine(y, pair_row, w, residual, out, int(k), int(flag), int(val))


def quant_mxfp8(x: torch.Tensor):
    """bf16 activations ``[R, K]`` -> (e4m3 bytes, ue8m0 scales per 32 K-values): the B operand of the block-scaled FP8 GEMMs."""
    return C().quant_mxfp8(x)


def _fp8pack(W: LinearWeight):
    """MXFP8 form of a weight (``utils/quant.py::to_mxfp8``), built once on first use from the dense / dequantised values; the
    source tensors (bf16 bank or packed MLX codes) are released — afterwards the weight lives in HBM as 1.03 bytes per parameter."""
    f = getattr(W, "_fp8", None)
    if f is None:
        from ..utils.quant import to_mxfp8

        src = W.dense(torch.bfloat16) if W.is_quantized else W.weight
        qs, sfs = [], []
        for chunk in (src.split(8) if src.dim() == 3 else [src]):     # bound the fp32 temporaries of the conversion
            q, sf = to_mxfp8(chunk)
            qs.append(q); sfs.append(sf)
        f = W._fp8 = (torch.cat(qs).contiguous(), torch.cat(sfs).contiguous())
        W.fp8_shape = tuple(src.shape)
        W.weight = W.wq = W.scales = W.biases = None
    return f


def fp8_experts_enabled(W: LinearWeight) -> bool:
    """Block-scaled FP8 expert banks.  The stage model converts at load (MLX 4/8-bit checkpoints by default, bf16 checkpoints with
    MLXB200_FP8_EXPERTS=1; ``models/deepseek_v2.py::_convert_quantized_for_b200``); packed MLX weights handed to the ops directly
    always take the exact in-kernel dequant GEMMs."""
    if getattr(W, "_fp8", None) is not None:
        return True                      # converted at load (models/deepseek_v2.py::_convert_quantized_for_b200)
    return os.environ.get("MLXB200_FP8_EXPERTS", "") == "1" and not W.is_quantized   # explicit opt-in for bf16 banks used directly


_scatter_bufs = {}
SCATTER_MAX_TOKENS = 128


def moe_block(x, gate_w, route_kw: dict, Wg: LinearWeight, Wu: LinearWeight, Wd: LinearWeight, act: str = "silu",
              residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, signal: Optional[Tuple[int, int]] = None,
              extra: int = 0, pre_norm: Optional[Tuple[torch.Tensor, float]] = None,
              next_norm: Optional[Tuple[torch.Tensor, float]] = None):
    """Router + routed (and appended shared) experts of one MoE block.

    ``pre_norm = (weight, eps)``: ``x`` is the un-normalised residual stream and the block starts with ``rmsnorm(x) * weight`` — on
    the scatter path the router kernel normalises the row in shared memory (no norm kernel).  ``next_norm = (weight, eps)``: the
    block also returns ``rmsnorm(result) * weight`` (the next layer's input norm), fused into the combine kernel on the scatter
    path; the return value is then ``(result, normed)``.
  Decode-sized batches with bf16 banks take the *scatter*
    path: the router kernel claims a slot per (token, expert) pair in the expert's fixed-stride segment and copies the token row
    there itself, the grouped GEMMs read per-expert row counts — route / counting sort / gather are ONE launch, the block is
    router -> grouped gate-up -> grouped down -> combine.  Larger batches (prefill) keep the compact counting-sort permutation."""
    c = C()
    T = x.shape[0]
    fp8 = fp8_experts_enabled(Wg) and x.shape[1] % 128 == 0
    quant = (Wg.is_quantized or Wu.is_quantized or Wd.is_quantized) and not fp8
    if quant or T > SCATTER_MAX_TOKENS or os.environ.get("MLXB200_MOE_SCATTER", "1") == "0":
        if pre_norm is not None:
            x = rmsnorm(x, pre_norm[0], pre_norm[1])
        idx, wts = moe_route(x, gate_w, extra=extra, **route_kw)
        res = moe_experts(x, idx, wts, Wg, Wu, Wd, act, residual=residual, out=out, signal=signal)
        return res if next_norm is None else (res, rmsnorm(res, next_norm[0], next_norm[1]))
    fuse_norms = os.environ.get("MLXB200_FUSE_NORMS", "1") != "0"
    if pre_norm is not None and not fuse_norms:
        x, pre_norm = rmsnorm(x, pre_norm[0], pre_norm[1]), None
    if fp8:
        (gq, gs), (uq, us), (dq, ds) = _fp8pack(Wg), _fp8pack(Wu), _fp8pack(Wd)
        E, H = gq.shape[0], x.shape[1]
    else:
        wg, wu, wd = _dense(Wg), _dense(Wu), _dense(Wd)
        E, H = wg.shape[0], x.shape[1]
    stride = 64 if T <= 64 else SCATTER_MAX_TOKENS
    key = (x.device.index, E, H, stride)
    bufs = _scatter_bufs.get(key)
    if bufs is None:
        # persistent (graph-safe) per-device buffers: row counters (zero between blocks: the combine resets them) + scattered rows
        bufs = _scatter_bufs[key] = (torch.zeros(E, dtype=torch.int32, device=x.device),
                                     torch.empty(E * stride, H, dtype=torch.bfloat16, device=x.device))
    counts, xs = bufs
    rk = dict(route_kw)
    method = rk.pop("method", "greedy")
    if method != "group_limited_greedy":
        rk["n_group"], rk["topk_group"] = 1, 1
    nw, ne = (_bf16(pre_norm[0]), float(pre_norm[1])) if pre_norm is not None else (None, 1e-6)
    idx, wts, pair_row = c.moe_route(x, _bf16(gate_w), int(rk["top_k"]), int(rk["n_group"]), int(rk["topk_group"]), float(rk["scaling"]),
                                     bool(rk["norm_topk"]), int(extra), counts, stride, xs, nw, ne)
    k = idx.shape[1]
    if fp8:
        # block-scaled FP8 experts: activations are quantised per 32-wide K block right before each GEMM (garbage rows beyond an
        # expert's count are quantised too and never read); tcgen05 kind::mxf8f6f4.block_scale applies both operands' scales
        xq, xsf = c.quant_mxfp8(xs)
        h = c.linear_fp8(xq, xsf, gq, gs, uq, us, counts, stride, None, ACT_IDS[act], False, T * k, stride)
        hq, hsf = c.quant_mxfp8(h)
        y = c.linear_fp8(hq, hsf, dq, ds, None, None, counts, stride, None, 0, True, T * k, stride)
    else:
        h = c.grouped_linear(xs, wg, wu, counts, stride, ACT_IDS[act], False, None, None, None, T * k, stride)
        y = c.grouped_linear(h, wd, None, counts, stride, 0, True, None, None, None, T * k, stride)
    flag, val = signal if signal is not None else (0, 0)
    if next_norm is not None and signal is None and fuse_norms and H <= 8192:
        normed = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
        res = c.moe_combine(y, pair_row, wts, residual, out, int(k), 0, 0, counts, _bf16(next_norm[0]), float(next_norm[1]), normed)
        return res, normed
    res = c.moe_combine(y, pair_row, wts, residual, out, int(k), int(flag), int(val), counts)
    return res if next_norm is None else (res, rmsnorm(res, next_norm[0], next_norm[1]))


def softcap_(logits, cap: float):
    return torch.tanh(logits / cap) * cap


def apply_penalties_(logits, rep_ctx, penalty, bias_idx, bias_val):
    C().apply_penalties_(logits, rep_ctx.contiguous(), penalty, bias_idx.contiguous(), bias_val.contiguous())
    return logits


_step = [0]


def sample(logits, temperature, top_p, generator: Optional[torch.Generator] = None, top_logprobs: int = 0):
    seed = generator.initial_seed() if generator is not None else 0
    _step[0] += 1
    toks, lp, ti, tl = C().sample(logits.contiguous(), temperature, top_p, int(seed) & 0x7FFFFFFFFFFFFFFF, _step[0],
                                  int(top_logprobs))
    if top_logprobs > 0:
        return toks, lp, ti, tl
    return toks, lp, None, None


def mla_absorbed_supported(num_heads: int, kv_lora_rank: int, rope_dim: int, page_size: int = 64) -> bool:
    """Shapes the tcgen05 absorbed-latent MLA decode kernel is built for (DeepSeek-V2 / V2-Lite / Coder-V2-Lite)."""
    return num_heads == 16 and kv_lora_rank == 512 and rope_dim == 64 and page_size == 64


def mla_absorbed_prologue(q, ckv, k_pe, norm_w, eps: float, pool, meta: BatchMeta, spec: RopeSpec):
    """latent = RMSNorm(c_kv) -> pool[slot][:512], rope(k_pe) -> pool[slot][512:], rope(q_pe) in place: one launch."""
    C().mla_absorbed_prologue(q, ckv, k_pe, norm_w, float(eps), pool, meta.slot_mapping, meta.positions, spec.inv_freq, float(spec.mscale))


def mla_decode(q, pool, meta: BatchMeta, scale: float, nsplit: int = 0):
    """Multi-query attention over the cached latent (d_qk 576 / d_v 512) on tcgen05: ``[B, 16, 576] -> [B, 16, 512]``."""
    return C().mla_decode(q, pool, meta.block_tables, meta.context_lens, float(scale), int(meta.max_ctx_len), int(nsplit))


def sample_block(logits, sv, tag_out, toks_out, lp_out, top_ids_out, top_lp_out):
    """Sampling driven by a step block in device memory (``parallel/graph_decode.py``): every per-step input — temperatures,
    nucleus thresholds, per-request (seed, step) RNG state, penalty contexts, bias tables, the step tag — is read by the kernels
    from the block, so the same captured CUDA graph serves greedy and sampled requests."""
    logits = logits.contiguous()
    if sv.has_pen:
        C().apply_penalties_(logits, sv.rep, sv.penalty, sv.bidx, sv.bval)
    k = 0 if top_ids_out is None else int(top_ids_out.shape[1])
    C().sample_into(logits, sv.temps, sv.top_p, sv.rng, k, toks_out, lp_out, top_ids_out, top_lp_out, sv.tag, tag_out)


def mla_rope_kv_write(q, k_pe, kv, kpool, vpool, meta: BatchMeta, spec: RopeSpec, nope: int, vdim: int):
    if not spec.interleaved:
        raise NotImplementedError("fused MLA prologue expects interleaved (traditional) rope pairs")
    C().mla_rope_kv_write(q, k_pe, kv, kpool, vpool, meta.slot_mapping, meta.positions, spec.inv_freq, float(spec.mscale),
                          int(nope), int(vdim))


# ------------------------------------------------------------------------------------------------ hybrid stacks (csrc/hybrid.cu)
# Same functions as the unfused forms in ``ops/reference.py``.  Activations are bf16 (serving) or fp32 (exact mode: the kernels are
# templated on the activation type; matrix products then go to cuBLAS in true fp32).
def _is32(dt) -> bool:
    if dt == torch.float32:
        return True
    if dt == torch.bfloat16:
        return False
    raise TypeError(f"b200 hybrid kernels take float32 / bfloat16 activations, got {dt}")


def _slots(meta: BatchMeta) -> torch.Tensor:
    if meta.state_slots is None:
        raise ValueError("this step's metadata carries no state slots")
    return meta.state_slots


def linear_any(x: torch.Tensor, W: LinearWeight, out_dtype: torch.dtype, act: str = "none") -> torch.Tensor:
    """``act(x @ W^T + W.bias)``.  bf16 operands whose shapes fit the TMA rules (K and N multiples of 8, 16-byte aligned rows) take the
    tcgen05 GEMM (bias in its epilogue); fp32 operands (exact mode) and odd shapes go to cuBLAS."""
    w = W.weight
    if (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and w.shape[0] % 8 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and x.shape[0] > 0):
        fused = act == "relu2"                      # the squared ReLU runs in the product's epilogue
        y = C().linear(x, w, None, None, W.bias, ACT_RELU2 if fused else 0, 0.0, out_dtype == torch.float32, None, 0, 0, 0)
        if fused:
            return y
    elif out_dtype == torch.float32 and x.dtype != torch.float32:
        # odd shapes with an fp32 result (scores, residual-stream inputs): the library product of the widened operands, so that the
        # result is not rounded to bf16 on its way out
        y = torch.nn.functional.linear(x.float(), w.float(), None if W.bias is None else W.bias.float())
    else:
        y = torch.nn.functional.linear(x, w, W.bias)
        y = y if y.dtype == out_dtype else y.to(out_dtype)
    if act == "gelu_erf":
        return gelu_erf_(y)
    if act == "relu2":
        return relu2_(y)
    if act != "none":
        raise NotImplementedError(act)
    return y


def gather_rows(table, ids, col0: int, ncols: int, out_dtype):
    return C().hy_gather_rows(table, ids, int(col0), int(ncols), _is32(out_dtype))


def side_gate(gx, table, ids, col0: int):
    return C().hy_side_gate(gx, table, ids, int(col0))


def gelu_erf_(x):
    return C().hy_gelu_erf_(x)


def post_norm_add_(x, y, w, eps: float, act_dtype):
    return C().hy_post_norm_add_(x, y, w, float(eps), _is32(act_dtype))


def rmsnorm_cast(x, w, eps: float, out_dtype):
    return C().hy_rmsnorm_cast(x, w, float(eps), _is32(out_dtype))


def gated_rmsnorm(y, gate, w, eps: float, groups: int, mode: str, out_dtype):
    return C().hy_gated_rmsnorm(y, gate, w, float(eps), int(groups), {"silu_pre": 0, "sigmoid_post": 1}[mode], _is32(out_dtype))


def causal_conv_silu(u, w, b, conv_state, meta: BatchMeta):
    return C().hy_causal_conv_silu(u, w, b, conv_state, meta.cu_seqlens, meta.context_lens, _slots(meta))


def ssm_scan(xbc, dt_raw, dt_bias, A_log, D, state, meta: BatchMeta, heads: int, vdim: int, nstate: int, groups: int):
    return C().hy_ssm_scan(xbc, dt_raw, dt_bias, A_log, D, state, meta.cu_seqlens, meta.context_lens, _slots(meta), int(heads), int(vdim),
                           int(nstate), int(groups), int(meta.max_q_len))


def decay_scan(qkv, decay, state, meta: BatchMeta, heads: int, dim: int, vdim: int):
    return C().hy_decay_scan(qkv, decay, state, meta.cu_seqlens, meta.context_lens, _slots(meta), int(heads), int(dim), int(vdim), int(meta.max_q_len))


def latent_kv_prologue(dqkv, q_rank: int, kv_rank: int, qn_w, kvn_w, eps: float, pool, meta: BatchMeta, inv_freq, interleaved: bool = False):
    cq = C().hy_latent_prologue(dqkv, int(q_rank), int(kv_rank), qn_w, kvn_w, float(eps), pool, meta.slot_mapping, meta.positions, inv_freq,
                                bool(interleaved))
    return cq if q_rank else None


def latent_attention(q, pool, sink, meta: BatchMeta, scale: float, kv_rank: int, inv_freq, out_dtype=None, window: int = 0,
                     interleaved: bool = False):
    return C().hy_latent_attention(q, pool, sink, meta.block_tables, meta.positions, meta.cu_seqlens, float(scale), int(kv_rank), inv_freq,
                                   int(meta.max_ctx_len), int(window), bool(interleaved))


def latent_attention_prefill(q, pool, sink, meta: BatchMeta, scale: float, kv_rank: int, inv_freq, out_dtype=None, window: int = 0,
                             interleaved: bool = False):
    """:func:`latent_attention` for a step that holds ONE sequence with many query rows (a prompt or a portion of one), as matrix
    products: gather the sequence's cached rows ``K`` ``[ctx, kv_rank + rot]`` from its pages, ``S = Q K^T`` (fp32 out), the
    masked softmax with the sink (``hy_sink_softmax``), ``out = P K[:, :kv_rank]``.  The two products run on the tensor cores
    (tcgen05 GEMM; cuBLAS fp32 in exact mode); query rows are processed in blocks so the score matrix stays below 256 MB."""
    T, H, Dq = q.shape
    ctx, page = int(meta.max_ctx_len), pool.shape[2]
    ctx0 = ctx - T
    # with a sliding window only keys from position ``lo`` on are ever seen by this step's queries; row i of K is position lo + i
    lo = max(0, ctx0 - window + 1) // 8 * 8 if window > 0 else 0
    nk, npad = ctx - lo, (ctx - lo + 7) // 8 * 8
    pages = meta.block_tables[0, :(ctx + page - 1) // page].long()
    ids = (pages[:, None] * page + torch.arange(page, device=q.device)).reshape(-1)[lo:ctx]
    if npad > nk:
        ids = torch.cat([ids, ids[:1].expand(npad - nk)])            # padding columns: any finite row (their probability is 0)
    K = gather_rows(pool.view(-1, Dq), ids.contiguous(), 0, Dq, q.dtype)
    C().hy_rotate_half_(q, meta.positions, inv_freq, int(kv_rank), bool(interleaved))
    is32 = _is32(q.dtype)
    block = max(1, (1 << 26) // (npad * H))
    if window > 0:
        block = min(block, max(64, (window + 63) // 64 * 64))         # a block of queries sees at most block + window - 1 keys
    outs = []
    for t0 in range(0, T, block):
        n = min(T, t0 + block) - t0
        # keys this block can see: positions [ka, kb) relative to ``lo``, both multiples of 8 (16-byte aligned rows and columns)
        ka = max(0, ctx0 + t0 - window + 1 - lo) // 8 * 8 if window > 0 else 0
        kb = min(npad, (ctx0 + t0 + n - lo + 7) // 8 * 8)
        Kb = K[ka:kb]
        Wk, Wc = LinearWeight(weight=Kb), LinearWeight(weight=Kb[:, :kv_rank].t().contiguous())
        s = linear_any(q[t0:t0 + n].reshape(n * H, Dq), Wk, torch.float32)
        p = C().hy_sink_softmax(s, sink, int(H), int(ctx0 + t0), float(scale), is32, int(window), int(lo + ka))
        outs.append(linear_any(p, Wc, q.dtype).view(n, H, kv_rank))
    return outs[0] if len(outs) == 1 else torch.cat(outs)


# ---- pre-norm residual step, mLSTM, sigmoid router and clamped-GLU experts (same functions as in ``ops/reference.py``)
from .reference import mlstm_col_block  # noqa: E402,F401  (a pure function of the value width: shared by both backends and the cache layout)


def scaled_add_norm_(x, y, ls, w, eps: float, act_dtype, extra=None, extra_gate=None):
    return C().hy_scaled_add_norm_(x, y, ls, w, float(eps), _is32(act_dtype), extra, extra_gate)


def mlstm_scan(qkv, gates, gate_bias, state: dict, meta: BatchMeta, heads: int, dim: int, vdim: int, cap: float, q_scale: float):
    return C().hy_mlstm_scan(qkv, gates, gate_bias, state["S"], state["n"], state["m"], meta.cu_seqlens, meta.context_lens, _slots(meta), int(heads),
                             int(dim), int(vdim), int(mlstm_col_block(vdim)), float(cap), float(q_scale), int(meta.max_q_len))


def router_logits(x, w):
    """fp32 router product (cuBLAS, TF32 off): the activations are widened, the fp32 weight is used as it is."""
    return torch.nn.functional.linear(x.float(), w)


def sigmoid_topk(z, num_experts: int, top: int):
    idx, w = C().hy_sigmoid_topk(z, int(num_experts), int(top))
    return idx, w


def softmax_topk(z, bias, num_experts: int, top: int):
    idx, w = C().hy_sigmoid_topk(z, int(num_experts), int(top), 1, bias)
    return idx, w


ACT_CLAMPED_GLU = 3      # two-weight GEMM epilogue: min(g, limit) sigmoid(1.702 .) (clamp(u, +-limit) + 1)


def clamped_glu(g, u, limit: float, out_dtype=None, row_scale=None):
    return C().hy_clamped_glu(g, u, float(limit), None, row_scale)


def _tc_ok(x, *ws) -> bool:
    """bf16 operands that satisfy the tensor-core GEMM's TMA rules (inner size and output rows multiples of 8, 16-byte aligned rows)."""
    return (x.dtype == torch.bfloat16 and x.shape[0] > 0 and x.shape[1] % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and all(w.dtype == torch.bfloat16 and w.shape[-2] % 8 == 0 for w in ws))


def clamped_gated_up(x, Wg: LinearWeight, Wu: LinearWeight, limit: float):
    """Both projections and the clamped GLU in ONE tcgen05 GEMM (two accumulators in TMEM, activation in the epilogue); exact mode and
    odd sizes: two cuBLAS products and the elementwise kernel."""
    if _tc_ok(x, Wg.weight, Wu.weight):
        return C().linear(x, Wg.weight, Wu.weight, None, None, ACT_CLAMPED_GLU, 0.0, False, None, 0, 0, 0, float(limit))
    lin = torch.nn.functional.linear
    return C().hy_clamped_glu(lin(x, Wg.weight), lin(x, Wu.weight), float(limit), None, None)


def moe_clamped_experts(x, idx, w, Wg: LinearWeight, Wu: LinearWeight, Wd: LinearWeight, limit: float):
    return _moe_experts(x, idx, w, Wg, Wu, Wd, float(limit), 0)


def moe_glu_experts(x, idx, w, Wg: LinearWeight, Wu: LinearWeight, Wd: LinearWeight):
    """Routed SiLU-GLU experts with the router weight on the expert's OUTPUT (applied in fp32 where the pairs are summed per token); same
    three paths as :func:`moe_clamped_experts`."""
    return _moe_experts(x, idx, w, Wg, Wu, Wd, 0.0, 1)


def silu_glu(g, u, out_dtype=None, row_scale=None):
    return C().hy_clamped_glu(g, u, 0.0, None, row_scale, 1)


def _moe_experts(x, idx, w, Wg: LinearWeight, Wu: LinearWeight, Wd: LinearWeight, limit: float, kind: int):
    """``kind`` 0: routed clamped-GLU experts with the router weight on the expert's input.  ``kind`` 1: SiLU-GLU experts, weight on the output.  bf16 banks whose sizes fit the grouped tcgen05 GEMM
    (expert rows multiples of 128, inner sizes multiples of 8): counting-sort permutation that scales each gathered row by its pair's
    weight -> grouped two-weight GEMM with the clamped GLU in its epilogue -> grouped down GEMM (fp32) -> sum per token.  Exact mode
    (fp32) and other sizes apply the weight to the gate / up products (linear in the input) and run either one weight-row read per
    (token, choice) pair (few rows; anything inside a graph capture) or one cuBLAS product per expert on the sorted rows."""
    c = C()
    T, k = idx.shape
    wg, wu, wd = Wg.weight, Wu.weight, Wd.weight
    E, F, K = wg.shape
    wflat = w.reshape(-1).contiguous()
    in_scale, out_wts = (wflat, None) if kind == 0 else (None, wflat)
    if _tc_ok(x) and wg.dtype == torch.bfloat16 and F % 128 == 0 and K % 128 == 0:
        offs, pair_row, xp = c.moe_permute(idx, x, E, in_scale)
        if kind == 0:
            h = c.grouped_linear(xp, wg, wu, offs, T, ACT_CLAMPED_GLU, False, act_limit=float(limit))
        else:
            h = c.grouped_linear(xp, wg, wu, offs, T, ACT_IDS["silu"], False)
        y = c.grouped_linear(h, wd, None, offs, T, 0, True)
        return c.hy_gather_sum(y, pair_row, int(k), out_wts)
    R = T * k
    if R <= PAIR_KERNEL_MAX_ROWS or torch.cuda.is_current_stream_capturing():
        ids = idx.reshape(-1).contiguous()
        h = c.hy_clamped_glu(c.hy_expert_rows_linear(x, int(k), wg, ids, False), c.hy_expert_rows_linear(x, int(k), wu, ids, False),
                             float(limit), None, in_scale, kind)
        y = c.hy_expert_rows_linear(h, 1, wd, ids, True)
        return c.hy_gather_sum(y, None, int(k), out_wts)
    flat = idx.reshape(-1).long()
    order = torch.sort(flat, stable=True).indices
    pair_row = torch.empty_like(order, dtype=torch.int32)
    pair_row[order] = torch.arange(order.numel(), device=x.device, dtype=torch.int32)
    xp = gather_rows(x, (order // k).contiguous(), 0, K, x.dtype)
    counts = torch.bincount(flat, minlength=E).tolist()
    g, u = torch.empty(R, F, dtype=x.dtype, device=x.device), torch.empty(R, F, dtype=x.dtype, device=x.device)
    r0 = 0
    for e, n in enumerate(counts):
        if n:
            torch.matmul(xp[r0:r0 + n], wg[e].t(), out=g[r0:r0 + n])
            torch.matmul(xp[r0:r0 + n], wu[e].t(), out=u[r0:r0 + n])
        r0 += n
    h = c.hy_clamped_glu(g, u, float(limit), pair_row, in_scale, kind)
    y = torch.empty(R, K, dtype=torch.float32, device=x.device)
    r0 = 0
    for e, n in enumerate(counts):
        if n:
            y[r0:r0 + n] = torch.matmul(h[r0:r0 + n], wd[e].t()).float()
        r0 += n
    return c.hy_gather_sum(y, pair_row, int(k), out_wts)


PAIR_KERNEL_MAX_ROWS = 64


# ---- sandwich layer norms, separate key / value pools, differential attention (``ops/csrc/diffattn.cu``; same functions as in ``ops/reference.py``)
def layernorm_cast(x, w, b, eps: float, out_dtype):
    return C().hy_layernorm_cast(x, w, b, float(eps), _is32(out_dtype))


def post_layernorm_add_norm_(x, y, post_w, post_b, mult: float, next_w, next_b, eps: float, act_dtype):
    return C().hy_post_layernorm_add_norm_(x, y, post_w, post_b, float(mult), next_w, next_b, float(eps), _is32(act_dtype))


def paged_kv_append(rows, k_col0: int, v_col0: int, kpool, vpool, meta: BatchMeta):
    C().hy_paged_kv_append(rows, int(k_col0), int(v_col0), kpool, vpool, meta.slot_mapping)


def diff_attention(q, kpool, vpool, meta: BatchMeta, heads: int, scale: float, softcap: float, temp_coef: float, temp_every: float, lam: float,
                   eps: float, out_mult: float, out_dtype=None):
    return C().hy_diff_attention(q, kpool, vpool, meta.block_tables, meta.positions, meta.cu_seqlens, int(heads), float(scale), float(softcap),
                                 float(temp_coef), float(temp_every), float(lam), float(eps), float(out_mult), int(meta.max_ctx_len))


def diff_attention_prefill(q, kpool, vpool, meta: BatchMeta, heads: int, scale: float, softcap: float, temp_coef: float, temp_every: float,
                           lam: float, eps: float, out_mult: float, out_dtype=None):
    """:func:`diff_attention` for a step that holds ONE sequence with many query rows (a prompt or a portion of one), as matrix products
    per key / value head ``g`` and map ``c``: gather the sequence's cached keys ``K_gc`` ``[ctx, d]`` and values ``V_g`` from its pages,
    ``S = Q_gc K_gc^T`` (fp32 out) for the ``heads / G`` query heads of the group at once, the capped, temperature-scaled causal softmax
    (``hy_sink_softmax``), ``A_gc = P V_g`` (fp32 out); one last kernel takes the difference of the two maps and its per-head norm.  The
    products run on the tensor cores (tcgen05 GEMM; cuBLAS fp32 in exact mode); query rows go in blocks so that a score matrix stays
    below 256 MB."""
    T = q.shape[0]
    P, G, page, D2 = kpool.shape
    D, V, Rg = D2 // 2, vpool.shape[3], heads // G
    ctx = int(meta.max_ctx_len)
    ctx0, npad = ctx - T, (ctx + 7) // 8 * 8
    pages = meta.block_tables[0, :(ctx + page - 1) // page].long()
    is32 = _is32(q.dtype)
    # [G, ctx (padded with any finite rows: their probability is 0), .] copies of this sequence's keys and values
    Kc = kpool[pages].permute(1, 0, 2, 3).reshape(G, -1, D2)
    Vc = vpool[pages].permute(1, 0, 2, 3).reshape(G, -1, V)
    if Kc.shape[1] < npad:
        Kc, Vc = torch.nn.functional.pad(Kc, (0, 0, 0, npad - Kc.shape[1])), torch.nn.functional.pad(Vc, (0, 0, 0, npad - Vc.shape[1]))
    Kc = Kc[:, :npad].reshape(G, npad, 2, D).permute(0, 2, 1, 3).contiguous()             # [G, 2, npad, D]
    Vt = Vc[:, :npad].transpose(1, 2).contiguous()                                         # [G, V, npad]
    Q = q[:, :heads * D2].reshape(T, G, Rg, 2, D).permute(1, 3, 0, 2, 4).contiguous()      # [G, 2, T, Rg, D]
    A = torch.empty(G, 2, T * Rg, V, dtype=torch.float32, device=q.device)
    block = max(1, (1 << 26) // (npad * Rg))
    for g in range(G):
        Wv = LinearWeight(weight=Vt[g])
        for c in range(2):
            Wk = LinearWeight(weight=Kc[g, c])
            for t0 in range(0, T, block):
                n = min(T, t0 + block) - t0
                kb = min(npad, (ctx0 + t0 + n + 7) // 8 * 8)          # keys this block of queries can see
                if kb < npad:
                    Wk_b, Wv_b = LinearWeight(weight=Kc[g, c, :kb]), LinearWeight(weight=Vt[g, :, :kb].contiguous())
                else:
                    Wk_b, Wv_b = Wk, Wv
                s = linear_any(Q[g, c, t0:t0 + n].reshape(n * Rg, D), Wk_b, torch.float32)
                p = C().hy_sink_softmax(s, None, int(Rg), int(ctx0 + t0), float(scale), is32, 0, 0, float(softcap), float(temp_coef), float(temp_every))
                A[g, c, t0 * Rg:(t0 + n) * Rg] = linear_any(p, Wv_b, torch.float32)
    return C().hy_diff_head_norm(A, int(T), int(heads), float(lam), float(eps), float(out_mult), is32)


# ---- several residual streams with dynamic-tanh norms, gated delta rule, attention with a sink inside blocks of positions, minGRU,
# ---- group-limited softmax router, squared-ReLU experts (``ops/csrc/streams.cu``; same functions as in ``ops/reference.py``)
ACT_RELU2 = 4            # single-weight GEMM epilogue: max(y, 0)^2


def relu2_(x):
    return C().hy_relu2_(x)


def stream_embed(table, ids, scale: float, streams: int):
    return C().hy_stream_embed(table, ids, float(scale), int(streams))


def dyt_cast(x, alpha: float, w, b, out_dtype):
    one = torch.ones(1, dtype=torch.float32, device=x.device)
    return C().hy_hyper_step_(x.view(x.shape[0], 1, x.shape[1]), None, None, None, None, None, None, 0.0, one, float(alpha), w, b, _is32(out_dtype))


def hyper_step_(xs, y, y2, gate, ls, mix, out_w, mult: float, in_w, alpha: float, w, b, act_dtype):
    return C().hy_hyper_step_(xs, y, y2, gate, ls, mix, out_w, float(mult), in_w, float(alpha), w, b, _is32(act_dtype))


def delta_scan(qkv, beta, dt, dt_bias, A_log, state, meta: BatchMeta, heads: int, kv_heads: int, dim: int, vdim: int, q_scale: float,
               unit_eps: float = 1e-6):
    return C().hy_delta_scan(qkv, beta, dt, dt_bias, A_log, state, meta.cu_seqlens, meta.context_lens, _slots(meta), int(heads), int(kv_heads), int(dim),
                             int(vdim), float(q_scale), float(unit_eps), int(meta.max_q_len))


def qk_norm_rope_append(rows, q_col0: int, k_col0: int, v_col0: int, heads: int, dim: int, qn_w, kn_w, eps: float, inv_freq, kpool, vpool, meta: BatchMeta):
    return C().hy_qk_norm_rope_append(rows, int(q_col0), int(k_col0), int(v_col0), int(heads), int(dim), qn_w, kn_w, float(eps), inv_freq, kpool, vpool,
                                      meta.slot_mapping, meta.positions)


def sink_attention(q, kpool, vpool, sink, meta: BatchMeta, scale: float, block: int = 0, window: int = 0, out_mult: float = 1.0, out_dtype=None,
                   out=None, out_col0: int = 0):
    return C().hy_sink_attention(q, kpool, vpool, sink, meta.block_tables, meta.positions, meta.cu_seqlens, float(scale), int(block), int(window),
                                 float(out_mult), int(meta.max_ctx_len), out, int(out_col0))


SINK_PREFILL_MIN_BLOCK = 256     # blocks of fewer positions: the products are too small to pay for their launches; the ragged kernel runs


def sink_attention_prefill(q, kpool, vpool, sink, meta: BatchMeta, scale: float, block: int = 0, window: int = 0, out_mult: float = 1.0, out_dtype=None,
                           out=None, out_col0: int = 0):
    """:func:`sink_attention` for a step that holds ONE sequence with many query rows (a prompt or a portion of one), as matrix products per
    block of positions and key / value head ``g``: gather the sequence's cached keys ``K_g`` and values ``V_g`` from the first visible
    position on, then for every block that holds queries of this step ``S = Q K_g[block]^T`` (fp32 out) for the ``H / G`` query heads of the
    group at once, the causal softmax with the sink (``hy_sink_softmax``; all keys of the slice lie in the queries' own block, so no lower
    limit is needed), ``O = P V_g[block]``.  The products run on the tensor cores (tcgen05 GEMM; cuBLAS fp32 in exact mode); query rows go in
    pieces so that a score matrix stays below 256 MB.  Sliding windows, blocks that are small or not a multiple of 8 positions: the kernel."""
    T, H, D = q.shape
    P, G, page, _ = kpool.shape
    V, Rg, adt = vpool.shape[3], H // G, kpool.dtype
    if window > 0 or meta.num_seqs != 1 or (block > 0 and (block % 8 != 0 or block < SINK_PREFILL_MIN_BLOCK)):
        return sink_attention(q, kpool, vpool, sink, meta, scale, block, window, out_mult, out_dtype, out, out_col0)
    ctx = int(meta.max_ctx_len)
    ctx0 = ctx - T
    first = ctx0 // block * block if block > 0 else 0                # first position any query of this step sees
    nk = ctx - first
    npad = (nk + 7) // 8 * 8
    pages = meta.block_tables[0, first // page:(ctx + page - 1) // page].long()
    skip = first - first // page * page
    # [G, keys from `first` on (padded with any finite rows: they lie behind every query), .] copies of this sequence's keys and values
    Kc = kpool[pages].permute(1, 0, 2, 3).reshape(G, -1, D)[:, skip:]
    Vc = vpool[pages].permute(1, 0, 2, 3).reshape(G, -1, V)[:, skip:]
    if Kc.shape[1] < npad:
        Kc, Vc = torch.nn.functional.pad(Kc, (0, 0, 0, npad - Kc.shape[1])), torch.nn.functional.pad(Vc, (0, 0, 0, npad - Vc.shape[1]))
    Kc, Vc = Kc[:, :npad].contiguous(), Vc[:, :npad]                                               # [G, npad, D], [G, npad, V]
    if out is None:
        out, out_col0 = torch.empty(T, H * V, dtype=adt, device=q.device), 0
    qa = q.to(adt).view(T, G, Rg, D).transpose(0, 1).contiguous()                                  # [G, T, Rg, D]: a head group's rows are a view
    is32 = _is32(adt)
    span = block if block > 0 else ctx
    # (the host issues every launch of this path one by one: few, large products beat many small ones, so a block's queries go in one
    # piece unless their score matrix would pass 256 MB)
    piece = max(1, (1 << 26) // (min(npad, span + 8) * Rg))
    for bs in range(first, ctx, span):
        be = min(bs + span, ctx)
        t_lo, t_hi = max(bs, ctx0) - ctx0, be - ctx0
        for t0 in range(t_lo, t_hi, piece):
            n = min(t_hi, t0 + piece) - t0
            ka, kb = bs - first, min(npad, (ctx0 + t0 + n - first + 7) // 8 * 8)            # keys this piece can see, as rows of Kc
            Vt = Vc[:, ka:kb].transpose(1, 2).contiguous()                                    # [G, V, keys] for all head groups at once
            for g in range(G):
                sg = None if sink is None else sink[g * Rg:(g + 1) * Rg]
                sc = linear_any(qa[g, t0:t0 + n].view(n * Rg, D), LinearWeight(weight=Kc[g, ka:kb]), torch.float32)
                pr = C().hy_sink_softmax(sc, sg, int(Rg), int(ctx0 + t0), float(scale), is32, 0, int(bs), 0.0, 0.0, 1.0)
                o = linear_any(pr, LinearWeight(weight=Vt[g]), torch.float32)
                c0 = out_col0 + g * Rg * V
                torch.mul(o.view(n, Rg * V), out_mult, out=out[t0:t0 + n, c0:c0 + Rg * V])  # scaled and rounded to the activation type in one pass
    return out


def mingru_scan(rows, z_col0: int, x_col0: int, g_col0: int, width: int, state, meta: BatchMeta, out_mult: float = 1.0, out_dtype=None, out=None,
                out_col0: int = 0):
    return C().hy_mingru_scan(rows, int(z_col0), int(x_col0), int(g_col0), int(width), state, meta.cu_seqlens, meta.context_lens, _slots(meta),
                              float(out_mult), int(meta.max_q_len), out, int(out_col0))


def group_softmax_topk(z, correction, num_experts: int, top: int, n_groups: int = 1, keep_groups: int = 1):
    idx, w = C().hy_group_softmax_topk(z, correction, int(num_experts), int(top), int(n_groups), int(keep_groups))
    return idx, w


def moe_relu2_experts(x, idx, w, Wu: LinearWeight, Wd: LinearWeight):
    """Routed squared-ReLU experts with the router weight on the expert's OUTPUT (applied in fp32 where the pairs are summed per token).
    bf16 banks whose sizes fit the grouped tcgen05 GEMM: counting-sort permutation -> grouped up GEMM with the squared ReLU in its
    epilogue -> grouped down GEMM (fp32) -> weighted sum per token.  Exact mode (fp32) and other sizes: one weight-row read per (token,
    choice) pair (few rows; anything inside a graph capture) or one cuBLAS product per expert on the sorted rows."""
    c = C()
    T, k = idx.shape
    wu, wd = Wu.weight, Wd.weight
    E, F, K = wu.shape
    wts = w.reshape(-1).contiguous()
    if _tc_ok(x) and wu.dtype == torch.bfloat16 and F % 128 == 0 and K % 128 == 0:
        offs, pair_row, xp = c.moe_permute(idx, x, E, None)
        h = c.grouped_linear(xp, wu, None, offs, T, ACT_RELU2, False)
        y = c.grouped_linear(h, wd, None, offs, T, 0, True)
        return c.hy_gather_sum(y, pair_row, int(k), wts)
    R = T * k
    if R <= PAIR_KERNEL_MAX_ROWS or torch.cuda.is_current_stream_capturing():
        ids = idx.reshape(-1).contiguous()
        h = c.hy_relu2_(c.hy_expert_rows_linear(x, int(k), wu, ids, False))
        y = c.hy_expert_rows_linear(h, 1, wd, ids, True)
        return c.hy_gather_sum(y, None, int(k), wts)
    flat = idx.reshape(-1).long()
    order = torch.sort(flat, stable=True).indices
    pair_row = torch.empty_like(order, dtype=torch.int32)
    pair_row[order] = torch.arange(order.numel(), device=x.device, dtype=torch.int32)
    xp = gather_rows(x, (order // k).contiguous(), 0, K, x.dtype)
    counts = torch.bincount(flat, minlength=E).tolist()
    h = torch.empty(R, F, dtype=x.dtype, device=x.device)
    r0 = 0
    for e, n in enumerate(counts):
        if n:
            torch.matmul(xp[r0:r0 + n], wu[e].t(), out=h[r0:r0 + n])
        r0 += n
    c.hy_relu2_(h)
    y = torch.empty(R, K, dtype=torch.float32, device=x.device)
    r0 = 0
    for e, n in enumerate(counts):
        if n:
            y[r0:r0 + n] = torch.matmul(h[r0:r0 + n], wd[e].t()).float()
        r0 += n
    return c.hy_gather_sum(y, pair_row, int(k), wts)
