"""Pure-PyTorch implementation of the op API (device-agnostic, fp32 internal math).

Three roles:
  1. the CPU execution path (tests, gloo plumbing config, machines without a GPU);
  2. the numerical oracle every sm_100a kernel in ``ops/csrc`` is tested against;
  3. on CUDA tensors it *is* the "straight PyTorch + cuBLAS" same-box baseline (``baseline/``).

Each function documents which upstream behaviour (SURVEY §2.2 U1–U12, §2.6 K1–K17) it reproduces.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from .meta import BatchMeta
from .weights import LinearWeight, RopeSpec

NAME = "reference"

# Oracle mode (default): every matmul accumulates and returns true fp32.  ``FAST_BASELINE = True`` turns
# this module into the "straight PyTorch + cuBLAS" baseline: bf16 tensor-core GEMMs via F.linear with bf16
# outputs, the way a plain PyTorch re-implementation of the reference pipeline would run on a B200.
FAST_BASELINE = False


# ------------------------------------------------------------------------------------------ K1
def embed(ids: torch.Tensor, emb: LinearWeight, scale: float = 1.0,
          dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Embedding gather with optional in-line affine dequant and Gemma ``sqrt(H)`` scale."""
    ids = ids.long()
    if emb.is_quantized:
        rows = LinearWeight(wq=emb.wq[ids], scales=emb.scales[ids], biases=emb.biases[ids],
                            group_size=emb.group_size, bits=emb.bits).dense(torch.float32)
    else:
        rows = emb.weight[ids].float()
    if scale != 1.0:
        # Gemma multiplies in the model dtype (reference gemma2.py:42-43)
        rows = rows.to(dtype).float() * torch.tensor(scale, dtype=dtype).float()
    return rows.to(dtype)


# ------------------------------------------------------------------------------------------ K2
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, gemma: bool = False,
            residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x * rsqrt(mean(x^2)+eps) * g`` (Gemma: ``g = 1 + w``); optional post-norm residual add
    ``residual + norm(x)`` (Gemma-2's post-attention / post-FFN norms)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    g = (1.0 + w.float()) if gemma else w.float()
    y = (y * g).to(x.dtype)
    if residual is not None:
        y = (y.float() + residual.float()).to(x.dtype)
    return y


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float,
                gemma: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """``h = x + residual`` (rounded to the activation dtype, like the unfused graph) then norm(h)."""
    h = (x.float() + residual.float()).to(x.dtype)
    return rmsnorm(h, w, eps, gemma), h


# ------------------------------------------------------------------------------------------ K3-K5, K8, K9, K12
def linear(x: torch.Tensor, W: LinearWeight, residual: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``y = x @ W^T (+ bias) (+ residual)``; fp32 accumulate, single rounding at the end."""
    if FAST_BASELINE and x.is_cuda and x.dtype != torch.float32:
        y = F.linear(x, W.dense_cached(x.dtype)).float()  # cuBLAS bf16 path (baseline role)
    else:
        y = x.float() @ W.dense(torch.float32).t()
    if W.bias is not None:
        y = y + W.bias.float()
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype or x.dtype)


def act_fn(name: str, x: torch.Tensor) -> torch.Tensor:
    if name == "silu":
        return F.silu(x)
    if name in ("gelu_tanh", "gelu_pytorch_tanh", "gelu_approx"):
        return F.gelu(x, approximate="tanh")
    raise ValueError(f"unknown activation {name}")


def gated_up(x: torch.Tensor, Wg: LinearWeight, Wu: LinearWeight, act: str = "silu") -> torch.Tensor:
    """``act(x Wg^T) * (x Wu^T)`` — SwiGLU / GeGLU first half, one rounding (K9)."""
    g = linear(x, Wg, out_dtype=torch.float32)
    u = linear(x, Wu, out_dtype=torch.float32)
    return (act_fn(act, g) * u).to(x.dtype)


# ------------------------------------------------------------------------------------------ K6
def rope_(x: torch.Tensor, positions: torch.Tensor, spec: RopeSpec, rot_offset: int = 0) -> torch.Tensor:
    """In-place rotary embedding on ``x[T, heads, D][..., rot_offset : rot_offset + rot_dim]``.

    ``interleaved=False``: half-split pairs ``(i, i + rot/2)`` (Llama / Gemma, MLX ``traditional=False``).
    ``interleaved=True`` : adjacent pairs ``(2i, 2i+1)`` (DeepSeek-V2, MLX ``traditional=True``)."""
    rd = spec.rot_dim
    ang = positions.float()[:, None] * spec.inv_freq.float().to(x.device)[None, :]  # [T, rd/2]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xs = x[..., rot_offset:rot_offset + rd].float() * spec.mscale
    if spec.interleaved:
        x1, x2 = xs[..., 0::2], xs[..., 1::2]
        o = torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1).flatten(-2)
    else:
        x1, x2 = xs[..., : rd // 2], xs[..., rd // 2:]
        o = torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)
    x[..., rot_offset:rot_offset + rd] = o.to(x.dtype)
    return x


# ------------------------------------------------------------------------------------------ K7
def kv_write(k: torch.Tensor, v: torch.Tensor, kpool: torch.Tensor, vpool: torch.Tensor,
             slot_mapping: torch.Tensor):
    """Append ``k[T,Hk,Dk]`` / ``v[T,Hk,Dv]`` into the paged pools ``[P, Hk, page, D]``."""
    page = kpool.shape[2]
    slots = slot_mapping.long()
    p, o = slots // page, slots % page
    kpool[p, :, o, :] = k.to(kpool.dtype)
    vpool[p, :, o, :] = v.to(vpool.dtype)


def kv_write_mla(kv: torch.Tensor, k_pe: torch.Tensor, kpool: torch.Tensor, vpool: torch.Tensor,
                 slot_mapping: torch.Tensor, nope: int, vdim: int):
    """MLA cache append in the reference's decompressed layout (deepseek_v2.py:120-125):
    ``K = [k_nope | k_pe broadcast over heads]`` (192), ``V`` (128); ``kv[T, heads, nope + vdim]``."""
    T, nh, _ = kv.shape
    k = torch.cat((kv[..., :nope], k_pe[:, None, :].expand(T, nh, k_pe.shape[-1])), dim=-1)
    kv_write(k, kv[..., nope:nope + vdim], kpool, vpool, slot_mapping)


def paged_attention(q: torch.Tensor, kpool: torch.Tensor, vpool: torch.Tensor, meta: BatchMeta,
                    scale: float, softcap: float = 0.0) -> torch.Tensor:
    """Causal attention of ``q[T,Hq,Dk]`` against the paged cache (which already contains this
    step's keys).  Token at absolute position ``p`` sees cache positions ``0..p``.  GQA by head
    grouping; ``softcap>0`` applies Gemma-2's ``tanh(s/cap)*cap`` to the scaled scores."""
    T, Hq, Dk = q.shape
    Hk, page, Dv = kpool.shape[1], kpool.shape[2], vpool.shape[3]
    G = Hq // Hk
    out = torch.empty(T, Hq, Dv, dtype=q.dtype, device=q.device)
    cu = meta.cu_seqlens.tolist()
    ctx = meta.context_lens.tolist()
    for b in range(meta.num_seqs):
        s, e, L = cu[b], cu[b + 1], ctx[b]
        if e == s:
            continue
        nblk = (L + page - 1) // page
        pages = meta.block_tables[b, :nblk].long()
        K = kpool[pages].permute(1, 0, 2, 3).reshape(Hk, nblk * page, Dk)[:, :L].float()
        V = vpool[pages].permute(1, 0, 2, 3).reshape(Hk, nblk * page, Dv)[:, :L].float()
        qb = q[s:e].float().permute(1, 0, 2).reshape(Hk, G, e - s, Dk)
        sc = torch.einsum("hgqd,hkd->hgqk", qb, K) * scale
        if softcap and softcap > 0:
            sc = torch.tanh(sc / softcap) * softcap
        qpos = meta.positions[s:e].long()
        kpos = torch.arange(L, device=q.device)
        mask = kpos[None, :] > qpos[:, None]
        sc = sc.masked_fill(mask[None, None], float("-inf"))
        p = torch.softmax(sc, dim=-1)
        o = torch.einsum("hgqk,hkd->hgqd", p, V).reshape(Hq, e - s, Dv).permute(1, 0, 2)
        out[s:e] = o.to(q.dtype)
    return out


# ------------------------------------------------------------------------------------------ K10
def moe_route(x: torch.Tensor, gate_w: torch.Tensor, top_k: int, method: str = "greedy",
              n_group: int = 1, topk_group: int = 1, scaling: float = 1.0,
              norm_topk: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 softmax router + top-k (greedy / group_limited_greedy) -> ``(idx int32 [T,k], w fp32 [T,k])``.
    Ties resolve to the lowest expert id; indices are returned in descending-score order."""
    scores = torch.softmax(x.float() @ gate_w.float().t(), dim=-1)
    T, E = scores.shape
    sel = scores
    if method == "group_limited_greedy" and n_group > 1:
        gs = scores.view(T, n_group, E // n_group).amax(-1)
        gidx = torch.topk(gs, topk_group, dim=-1).indices
        gmask = torch.zeros_like(gs).scatter_(1, gidx, 1.0)
        smask = gmask[:, :, None].expand(T, n_group, E // n_group).reshape(T, E)
        sel = scores.masked_fill(smask == 0, 0.0)
    # stable descending sort => deterministic tie-break on the lowest index
    order = torch.sort(sel, dim=-1, descending=True, stable=True).indices[:, :top_k]
    w = torch.gather(scores, 1, order)
    if norm_topk and top_k > 1:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    else:
        w = w * scaling
    return order.to(torch.int32), w


# ------------------------------------------------------------------------------------------ K11
def run_aside(fn):
    """Backend hook: independent work that the CUDA backend forks onto a side stream runs inline here."""
    fn()
    return None


def moe_experts(x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, Wg: LinearWeight, Wu: LinearWeight,
                Wd: LinearWeight, act: str = "silu", extra: Optional[torch.Tensor] = None,
                residual: Optional[torch.Tensor] = None, join=None) -> torch.Tensor:
    """``y[t] = sum_k w[t,k] * down_e(act(gate_e x) * up_e x) (+ extra[t]) (+ residual[t])``.
    Intermediate activations are rounded to the activation dtype exactly where the kernels round."""
    T, H = x.shape
    E = (Wg.wq if Wg.is_quantized else Wg.weight).shape[0]
    y = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    idx_l = idx.long()
    for e in range(E):
        tok, slot = torch.where(idx_l == e)
        if tok.numel() == 0:
            continue
        xe = x[tok]
        h = gated_up(xe, Wg.select_expert(e), Wu.select_expert(e), act)
        o = linear(h, Wd.select_expert(e), out_dtype=torch.float32)
        y.index_add_(0, tok, o * w[tok, slot].float()[:, None])
    if extra is not None:
        y = y + extra.float()
    if residual is not None:
        y = y + residual.float()
    return y.to(x.dtype)


# ------------------------------------------------------------------------------------------ K12 epilogue
def softcap_(logits: torch.Tensor, cap: float) -> torch.Tensor:
    return torch.tanh(logits / cap) * cap


# ------------------------------------------------------------------------------------------ K13
def apply_repetition_penalty_(logits: torch.Tensor, ctx_tokens: torch.Tensor, penalty: float) -> torch.Tensor:
    """U7: for ids in ctx: ``l<0 ? l*p : l/p`` (in place, 1-D logits)."""
    if ctx_tokens.numel() == 0 or penalty == 1.0:
        return logits
    ids = ctx_tokens.long().unique()
    sel = logits[ids]
    logits[ids] = torch.where(sel < 0, sel * penalty, sel / penalty)
    return logits


def apply_penalties_(logits: torch.Tensor, rep_ctx: torch.Tensor, penalty: torch.Tensor,
                     bias_idx: torch.Tensor, bias_val: torch.Tensor) -> torch.Tensor:
    """Batched in-place repetition penalty (reference utils.py:167-170) then logit_bias add
    (utils.py:127-130, inside ``sample``).  ``rep_ctx int32 [B, C]`` / ``bias_idx int32 [B, Nb]`` are
    padded with ``-1``."""
    B = logits.shape[0]
    for b in range(B):
        c = rep_ctx[b]
        c = c[c >= 0]
        apply_repetition_penalty_(logits[b], c, float(penalty[b]))
        bi = bias_idx[b]
        m = bi >= 0
        if m.any():
            logits[b].index_add_(0, bi[m].long(), bias_val[b][m].to(logits.dtype))
    return logits


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor,
           generator: Optional[torch.Generator] = None, top_logprobs: int = 0):
    """Batched sampler (reference shard/utils.py:126-139 + mlx_lm ``top_p_sampling``).

    ``logits`` fp32 ``[B, V]`` *after* bias / repetition penalty.  Per row: ``temp == 0`` -> argmax;
    ``0 < top_p < 1`` -> nucleus; else categorical(softmax(logits / temp)).
    Returns ``(tokens int64 [B], token_logprob fp32 [B], topk_ids, topk_logprobs)`` where logprobs are
    ``logits - logsumexp(logits)`` (temperature **not** applied — reference utils.py:131)."""
    B, V = logits.shape
    lf = logits.float()
    logprobs = lf - torch.logsumexp(lf, dim=-1, keepdim=True)
    tokens = torch.empty(B, dtype=torch.int64, device=logits.device)
    t_cpu, p_cpu = temperature.tolist(), top_p.tolist()
    for b in range(B):
        t, p = t_cpu[b], p_cpu[b]
        if t == 0:
            tokens[b] = torch.argmax(lf[b])
            continue
        probs = torch.softmax(lf[b] / t, dim=-1)
        if 0 < p < 1.0:
            sp, si = torch.sort(probs, descending=False, stable=True)
            cum = torch.cumsum(sp, dim=0)
            keep = cum > (1 - p)
            sp = torch.where(keep, sp, torch.zeros_like(sp))
            j = torch.multinomial(sp / sp.sum(), 1, generator=generator)
            tokens[b] = si[j].squeeze()
        else:
            tokens[b] = torch.multinomial(probs, 1, generator=generator).squeeze()
    tok_lp = logprobs.gather(1, tokens[:, None]).squeeze(1)
    if top_logprobs > 0:
        tk = torch.topk(logprobs, top_logprobs, dim=-1)
        return tokens, tok_lp, tk.indices, tk.values
    return tokens, tok_lp, None, None


def sample_block(logits: torch.Tensor, sv, tag_out, toks_out, lp_out, top_ids_out, top_lp_out):
    """Sampling driven by a step block (``parallel/graph_decode.py``): penalties, then per-sequence temperature / top-p with a
    per-request random stream — row ``b`` draws from a generator seeded with its ``(seed, tokens sampled so far)`` pair, so a
    request's tokens do not depend on which batch it decodes in.  Results go into the result-message views."""
    lf = logits.float().clone()
    if sv.has_pen:
        apply_penalties_(lf, sv.rep, sv.penalty, sv.bidx, sv.bval)
    B = lf.shape[0]
    rng = sv.rng.view(B, 2).tolist()
    k = 0 if top_ids_out is None else top_ids_out.shape[1]
    for b in range(B):
        g = torch.Generator(device=lf.device)
        g.manual_seed((rng[b][0] * 1000003 + rng[b][1] * 7919 + 12345) & 0x7FFFFFFFFFFFFFFF)
        t, lp, ti, tl = sample(lf[b:b + 1], sv.temps[b:b + 1], sv.top_p[b:b + 1], generator=g, top_logprobs=k)
        toks_out[b], lp_out[b] = t[0], lp[0]
        if k:
            top_ids_out[b], top_lp_out[b] = ti[0], tl[0]
    tag_out.copy_(sv.tag)


def mla_rope_kv_write(q: torch.Tensor, k_pe: torch.Tensor, kv: torch.Tensor, kpool: torch.Tensor, vpool: torch.Tensor,
                      meta: BatchMeta, spec: RopeSpec, nope: int, vdim: int):
    """DeepSeek-V2 attention prologue: rope the ``*_pe`` slices (q in place) and append
    ``K = [k_nope | rope(k_pe)]``, ``V`` to the paged cache (one fused kernel on the b200 backend)."""
    rope_(q, meta.positions, spec, nope)
    kp = k_pe.clone().unsqueeze(1)
    rope_(kp, meta.positions, spec, 0)
    kv_write_mla(kv, kp.squeeze(1), kpool, vpool, meta.slot_mapping, nope, vdim)


# ------------------------------------------------------------------------------------------ hybrid-stack mechanisms
# Unfused PyTorch forms of the ops behind recurrent / latent-attention layers (``ops/csrc/hybrid.cu`` on the CUDA backend).  All
# take the ragged step metadata: rows ``cu_seqlens[b] .. cu_seqlens[b+1]`` belong to sequence ``b``, whose recurrent state lives in
# slot ``meta.state_slots[b]``; a sequence whose step starts at position 0 starts from a zero state, whatever the slot holds.
def _seq_ranges(meta: BatchMeta):
    cu, ctx = meta.cu_seqlens.tolist(), meta.context_lens.tolist()
    slots = meta.state_slots.tolist() if meta.state_slots is not None else [0] * meta.num_seqs
    for b in range(meta.num_seqs):
        yield cu[b], cu[b + 1], ctx[b] - (cu[b + 1] - cu[b]), slots[b]


def gather_rows(table: torch.Tensor, ids: torch.Tensor, col0: int, ncols: int, out_dtype: torch.dtype) -> torch.Tensor:
    """``out[t] = table[ids[t], col0:col0+ncols]`` (embedding lookup, optionally of a column block)."""
    return table[ids.long(), col0:col0 + ncols].to(out_dtype)


def post_norm_add_(x: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float, act_dtype: torch.dtype) -> torch.Tensor:
    """Norm on the sublayer's OUTPUT: ``x += y / sqrt(mean(y^2) + eps) * w`` on the fp32 residual ``x`` (in place); returns ``x`` in
    the activation dtype (``x`` itself when that is fp32) for the next projection."""
    yf = y.float()
    x += yf * torch.rsqrt(yf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return x if act_dtype == torch.float32 else x.to(act_dtype)


def rmsnorm_cast(x: torch.Tensor, w: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(out_dtype)


def gelu_erf_(x: torch.Tensor) -> torch.Tensor:
    return x.copy_(F.gelu(x.float()).to(x.dtype))


def side_gate(gx: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, col0: int) -> torch.Tensor:
    """``gelu_tanh(gx) * table[ids, col0:col0+dim]`` (the gate of a per-layer token input)."""
    e = table[ids.long(), col0:col0 + gx.shape[1]].float()
    return (F.gelu(gx.float(), approximate="tanh") * e).to(gx.dtype)


def causal_conv_silu(u: torch.Tensor, w: torch.Tensor, b: torch.Tensor, conv_state: torch.Tensor, meta: BatchMeta) -> torch.Tensor:
    """Per-channel causal convolution + SiLU over a ragged batch.  ``u`` ``[T, C]`` (may be a column view), ``w`` ``[C, K]`` (last
    column = current token), ``conv_state`` ``[slots, K-1, C]`` = the last ``K-1`` inputs of each sequence (updated here)."""
    K = w.shape[1]
    out = torch.empty(u.shape, dtype=u.dtype, device=u.device)
    for s, e, c0, slot in _seq_ranges(meta):
        hist = conv_state[slot].to(u.dtype) if c0 > 0 else torch.zeros(K - 1, u.shape[1], dtype=u.dtype, device=u.device)
        full = torch.cat([hist, u[s:e]])
        acc = b.float().expand(e - s, -1).clone()
        for k in range(K):
            acc += full[k:k + e - s].float() * w[:, k].float()
        out[s:e] = F.silu(acc).to(u.dtype)
        if K > 1:
            conv_state[slot] = full[-(K - 1):].to(conv_state.dtype)
    return out


def ssm_scan(xbc: torch.Tensor, dt_raw: torch.Tensor, dt_bias: torch.Tensor, A_log: torch.Tensor, D: torch.Tensor,
             state: torch.Tensor, meta: BatchMeta, heads: int, vdim: int, nstate: int, groups: int) -> torch.Tensor:
    """Selective state-space recurrence per head (fp32): ``S <- exp(-exp(A_log) dt) S + dt B x^T``, ``y = S^T C + D x`` with
    ``dt = softplus(dt_raw + dt_bias)``.  ``xbc`` = ``[x: heads*vdim | B: groups*nstate | C: groups*nstate]`` after the convolution;
    ``state`` ``[slots, heads, nstate, vdim]`` fp32.  Returns fp32 ``[T, heads*vdim]``."""
    T, inner = xbc.shape[0], heads * vdim
    y = torch.empty(T, heads, vdim, dtype=torch.float32, device=xbc.device)
    x = xbc[:, :inner].float().view(T, heads, vdim)
    rep = heads // groups
    Bm = xbc[:, inner:inner + groups * nstate].float().view(T, groups, nstate).repeat_interleave(rep, 1)
    Cm = xbc[:, inner + groups * nstate:].float().view(T, groups, nstate).repeat_interleave(rep, 1)
    dt = F.softplus(dt_raw.float() + dt_bias.float(), threshold=80.0)
    a = torch.exp(-torch.exp(A_log.float()) * dt)
    for s, e, c0, slot in _seq_ranges(meta):
        S = state[slot].clone() if c0 > 0 else torch.zeros_like(state[slot])
        for t in range(s, e):
            S = a[t, :, None, None] * S + (dt[t, :, None] * Bm[t])[:, :, None] * x[t][:, None, :]
            y[t] = torch.einsum("hnp,hn->hp", S, Cm[t]) + D.float()[:, None] * x[t]
        state[slot] = S
    return y.view(T, inner)


def decay_scan(qkv: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, meta: BatchMeta, heads: int, dim: int, vdim: int) -> torch.Tensor:
    """Linear attention with a constant per-head decay (fp32 state): ``S <- decay S + k v^T``, ``o = S^T q`` on
    ``q, k, v = silu(.)`` of the columns ``[q: heads*dim | k: heads*dim | v: heads*vdim]``.  ``state`` ``[slots, heads, dim, vdim]``."""
    T = qkv.shape[0]
    act = F.silu(qkv[:, :2 * heads * dim + heads * vdim].float())
    q, k = act[:, :heads * dim].view(T, heads, dim), act[:, heads * dim:2 * heads * dim].view(T, heads, dim)
    v = act[:, 2 * heads * dim:].view(T, heads, vdim)
    o = torch.empty(T, heads, vdim, dtype=torch.float32, device=qkv.device)
    d = decay.float()[:, None, None]
    for s, e, c0, slot in _seq_ranges(meta):
        S = state[slot].clone() if c0 > 0 else torch.zeros_like(state[slot])
        for t in range(s, e):
            S = d * S + k[t][:, :, None] * v[t][:, None, :]
            o[t] = torch.einsum("hdv,hd->hv", S, q[t])
        state[slot] = S
    return o.view(T, heads * vdim)


def gated_rmsnorm(y: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, eps: float, groups: int, mode: str,
                  out_dtype: torch.dtype) -> torch.Tensor:
    """``mode='silu_pre'``: RMS norm in ``groups`` equal parts of ``y * silu(gate)``; ``mode='sigmoid_post'``: ``norm(y) * sigmoid(gate)``.
    Both times ``w``; fp32 arithmetic."""
    yf, g = y.float(), gate.float()
    if mode == "silu_pre":
        yf = yf * F.silu(g)
    T, C = yf.shape
    v = yf.view(T, groups, C // groups)
    v = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).view(T, C) * w.float()
    if mode == "sigmoid_post":
        v = v * torch.sigmoid(g)
    return v.to(out_dtype)


def _rot_half(v: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    half = inv_freq.numel()
    a = pos.float()[:, None] * inv_freq.float()
    c, s = torch.cos(a), torch.sin(a)
    while c.dim() < v.dim():
        c, s = c.unsqueeze(1), s.unsqueeze(1)
    u1, u2 = v[..., :half], v[..., half:2 * half]
    return torch.cat([u1 * c - u2 * s, u2 * c + u1 * s, v[..., 2 * half:]], -1)


def _rot_pairs(v: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """Adjacent pairs ``(2i, 2i+1)`` of the first ``2 * len(inv_freq)`` entries turn by ``pos * inv_freq[i]``."""
    half = inv_freq.numel()
    a = pos.float()[:, None] * inv_freq.float()
    c, s = torch.cos(a), torch.sin(a)
    while c.dim() < v.dim():
        c, s = c.unsqueeze(1), s.unsqueeze(1)
    u1, u2 = v[..., 0:2 * half:2], v[..., 1:2 * half:2]
    rot = torch.stack([u1 * c - u2 * s, u2 * c + u1 * s], -1).flatten(-2)
    return torch.cat([rot, v[..., 2 * half:]], -1)


def latent_kv_prologue(dqkv: torch.Tensor, q_rank: int, kv_rank: int, qn_w: Optional[torch.Tensor], kvn_w: torch.Tensor, eps: float,
                       pool: torch.Tensor, meta: BatchMeta, inv_freq: torch.Tensor, interleaved: bool = False) -> Optional[torch.Tensor]:
    """Rows ``[c_q raw: q_rank | c raw: kv_rank | k_rot raw]`` -> returns ``RMSnorm(c_q) * qn_w`` (``None`` when ``q_rank`` is 0: the
    design has no query latent); appends ``[RMSnorm(c) * kvn_w | rotate(k_rot)]`` to the paged latent pool ``[pages, 1, page, kv_rank +
    rot]`` at ``meta.slot_mapping``.  ``interleaved``: rotary pairs are ``(2i, 2i+1)`` instead of ``(i, i + rot/2)``."""
    cq = rmsnorm_cast(dqkv[:, :q_rank], qn_w, eps, dqkv.dtype) if q_rank else None
    c = rmsnorm_cast(dqkv[:, q_rank:q_rank + kv_rank], kvn_w, eps, torch.float32)
    kr = (_rot_pairs if interleaved else _rot_half)(dqkv[:, q_rank + kv_rank:].float(), meta.positions, inv_freq)
    flat = pool.view(-1, pool.shape[-1])
    flat[meta.slot_mapping.long()] = torch.cat([c, kr], -1).to(pool.dtype)
    return cq


def latent_attention(q: torch.Tensor, pool: torch.Tensor, sink: Optional[torch.Tensor], meta: BatchMeta, scale: float, kv_rank: int,
                     inv_freq: torch.Tensor, out_dtype: torch.dtype = torch.float32, window: int = 0, interleaved: bool = False) -> torch.Tensor:
    """Causal multi-query attention over the cached latent rows with a *sink* in the softmax.  ``q`` ``[T, H, kv_rank + rot]`` (latent
    part already multiplied by the key up-projection; the rot part is rotated here), keys = pool rows, values = their first
    ``kv_rank`` entries; ``p_j = exp(s_j) / (exp(sink_h) + sum_i exp(s_i))`` (``sink=None``: the ordinary softmax).  ``window > 0``: the
    query at position ``i`` sees keys ``j`` with ``0 <= i - j < window``.  Returns fp32 ``[T, H, kv_rank]``."""
    T, H, Dq = q.shape
    page = pool.shape[2]
    qf = q.float()
    qf = torch.cat([qf[..., :kv_rank], (_rot_pairs if interleaved else _rot_half)(qf[..., kv_rank:], meta.positions, inv_freq)], -1)
    out = torch.empty(T, H, kv_rank, dtype=torch.float32, device=q.device)
    bt = meta.block_tables.long()
    for b, (s, e, c0, _) in enumerate(_seq_ranges(meta)):
        n = c0 + (e - s)
        idx = torch.arange(n, device=q.device)
        rows = pool.view(-1, Dq)[bt[b, idx // page] * page + idx % page].float()               # [n, Dq]
        sc = torch.einsum("thd,nd->thn", qf[s:e], rows) * scale
        qpos = (c0 + torch.arange(e - s, device=q.device))[:, None]
        mask = idx[None, :] > qpos
        if window > 0:
            mask = mask | (idx[None, :] <= qpos - window)
        sc = sc.masked_fill(mask[:, None, :], float("-inf"))
        if sink is None:
            p = torch.softmax(sc, -1)
        else:
            sk = sink.float().view(1, H, 1).expand(e - s, H, 1)
            p = torch.softmax(torch.cat([sc, sk], -1), -1)[..., :n]
        out[s:e] = torch.einsum("thn,nd->thd", p, rows[:, :kv_rank])
    return out.to(out_dtype)


def linear_any(x: torch.Tensor, W: LinearWeight, out_dtype: torch.dtype, act: str = "none") -> torch.Tensor:
    """``act(x @ W^T + W.bias)`` for any shape / float dtype (fp32 accumulate; ``act``: none | gelu_erf | relu2 = ``max(., 0)^2``)."""
    y = linear(x, W, out_dtype=torch.float32)
    if act == "gelu_erf":
        y = F.gelu(y)
    elif act == "relu2":
        y = torch.relu(y) ** 2
    elif act != "none":
        raise NotImplementedError(act)
    return y.to(out_dtype)


def latent_attention_prefill(q, pool, sink, meta: BatchMeta, scale: float, kv_rank: int, inv_freq, out_dtype=torch.float32, window: int = 0,
                             interleaved: bool = False):
    """Single-sequence prefill form of :func:`latent_attention` (the CUDA backend runs it as two GEMMs); same math here."""
    return latent_attention(q, pool, sink, meta, scale, kv_rank, inv_freq, out_dtype, window, interleaved)


def scaled_add_norm_(x: torch.Tensor, y: torch.Tensor, ls: Optional[torch.Tensor], w: torch.Tensor, eps: float, act_dtype: torch.dtype,
                     extra: Optional[torch.Tensor] = None, extra_gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Pre-norm residual step on the fp32 stream ``x`` (in place): ``x += (y + extra * sigmoid(extra_gate)) * ls`` (``ls``: per-channel
    layer scale or ``None``; ``extra`` / ``extra_gate``: an always-on branch with one gate logit per row), then returns
    ``x / sqrt(mean(x^2) + eps) * w`` in the activation dtype: the input of the sublayer that follows."""
    yf = y.float()
    if extra is not None:
        yf = yf + extra.float() * torch.sigmoid(extra_gate.float()).reshape(-1, 1)
    x += yf * ls.float() if ls is not None else yf
    return rmsnorm_cast(x, w, eps, act_dtype)


def mlstm_col_block(vdim: int) -> int:
    """Value columns of a head that one CTA of the mLSTM scan owns (fixed per size, so the per-block copies of the normaliser state
    keep their meaning from step to step)."""
    pb = int(vdim)
    while pb > 32 and pb % 2 == 0:
        pb //= 2
    return pb


def mlstm_scan(qkv: torch.Tensor, gates: torch.Tensor, gate_bias: torch.Tensor, state: dict, meta: BatchMeta, heads: int, dim: int,
               vdim: int, cap: float, q_scale: float) -> torch.Tensor:
    """Matrix-memory recurrence with exponential gating and a running maximum (fp32), per head:
    ``i = cap tanh((gi + bi) / cap)``, ``f = logsigmoid(cap tanh((gf + bf) / cap))``, ``m' = max(f + m, i)``,
    ``S <- e^(f + m - m') S + e^(i - m') k v^T``, ``n`` likewise with ``k``, ``o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)``; ``m, S, n``
    start at zero.  ``qkv`` columns ``[q: heads*dim | k: heads*dim | v: heads*vdim | ...]`` (``q`` is multiplied by ``q_scale``),
    ``gates`` fp32 ``[T, >= 2*heads]`` = raw ``[gi | gf]``, ``gate_bias`` fp32 ``[2*heads]``.  ``state``: ``S`` ``[slots, heads, dim,
    vdim]``, ``n`` ``[slots, heads, vdim / col_block, dim]``, ``m`` ``[slots, heads, vdim / col_block]`` (one copy of ``n, m`` per
    column block).  Returns fp32 ``[T, heads*vdim]``."""
    T, H = qkv.shape[0], heads
    q = qkv[:, :H * dim].float().view(T, H, dim) * q_scale
    k = qkv[:, H * dim:2 * H * dim].float().view(T, H, dim)
    v = qkv[:, 2 * H * dim:2 * H * dim + H * vdim].float().view(T, H, vdim)
    g = gates[:, :2 * H].float() + gate_bias.float()
    ig = cap * torch.tanh(g[:, :H] / cap)
    fg = F.logsigmoid(cap * torch.tanh(g[:, H:] / cap))
    o = torch.empty(T, H, vdim, dtype=torch.float32, device=qkv.device)
    for s, e, c0, slot in _seq_ranges(meta):
        if e == s:
            continue
        if c0 > 0:
            S, n, m = state["S"][slot].clone(), state["n"][slot][:, 0].clone(), state["m"][slot][:, 0].clone()
        else:
            S, n, m = torch.zeros_like(state["S"][slot]), torch.zeros_like(state["n"][slot][:, 0]), torch.zeros_like(state["m"][slot][:, 0])
        for t in range(s, e):
            mn = torch.maximum(fg[t] + m, ig[t])
            a, b = torch.exp(fg[t] + m - mn), torch.exp(ig[t] - mn)
            S = a[:, None, None] * S + (b[:, None] * k[t])[:, :, None] * v[t][:, None, :]
            n = a[:, None] * n + b[:, None] * k[t]
            m = mn
            den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
            o[t] = torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
        state["S"][slot] = S
        state["n"][slot] = n[:, None, :].expand_as(state["n"][slot])
        state["m"][slot] = m[:, None].expand_as(state["m"][slot])
    return o.view(T, H * vdim)


def sigmoid_topk(z: torch.Tensor, num_experts: int, top: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Router on fp32 logits ``z[:, :num_experts]``: scores ``sigmoid(z)``, the ``top`` largest (ties: lowest id), weights = the chosen
    scores as they are.  Returns ``(idx int32 [T, top], w fp32 [T, top])``."""
    sc = torch.sigmoid(z[:, :num_experts].float())
    order = torch.sort(sc, dim=-1, descending=True, stable=True).indices[:, :top]
    return order.to(torch.int32), torch.gather(sc, 1, order)


def clamped_glu(g: torch.Tensor, u: torch.Tensor, limit: float, out_dtype: torch.dtype, row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gate rows ``g`` and up rows ``u`` ``[R, F]`` -> ``g' sigmoid(1.702 g') (u' + 1)`` with ``g' = min(s g, limit)``, ``u' = clamp(s u,
    +-limit)``; ``s`` = ``row_scale`` (per row, default 1): scaling a linear projection's output equals scaling its input."""
    g, u = g.float(), u.float()
    if row_scale is not None:
        g, u = g * row_scale.float()[:, None], u * row_scale.float()[:, None]
    g, u = g.clamp(max=limit), u.clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)).to(out_dtype)


def clamped_gated_up(x: torch.Tensor, Wg: LinearWeight, Wu: LinearWeight, limit: float) -> torch.Tensor:
    """First half of a clamped-GLU feed-forward: :func:`clamped_glu` of ``x Wg^T`` and ``x Wu^T`` (one fused GEMM on the b200 backend)."""
    return clamped_glu(linear(x, Wg, out_dtype=torch.float32), linear(x, Wu, out_dtype=torch.float32), limit, x.dtype)


def moe_clamped_experts(x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, Wg: LinearWeight, Wu: LinearWeight, Wd: LinearWeight,
                        limit: float) -> torch.Tensor:
    """``y[t] = sum_j expert_{idx[t,j]}(w[t,j] x[t])`` with clamped-GLU experts (:func:`clamped_glu`): the router weight scales the
    expert's INPUT.  Banks ``Wg``, ``Wu`` ``[E, F, K]``, ``Wd`` ``[E, K, F]``.  Returns fp32 ``[T, K]``."""
    T, k = idx.shape
    y = torch.zeros(T, Wd.weight.shape[1], dtype=torch.float32, device=x.device)
    il = idx.long()
    for e in range(Wg.weight.shape[0]):
        tok, slot = torch.where(il == e)
        if tok.numel() == 0:
            continue
        xe = (x[tok].float() * w[tok, slot].float()[:, None]).to(x.dtype)
        h = clamped_glu(xe.float() @ Wg.weight[e].float().t(), xe.float() @ Wu.weight[e].float().t(), limit, x.dtype)
        y.index_add_(0, tok, h.float() @ Wd.weight[e].float().t())
    return y


def router_logits(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """fp32 router product ``x W^T`` (``w`` fp32 ``[rows, K]``; ``x`` in the activation dtype is widened, never the weight narrowed)."""
    return x.float() @ w.float().t()


# ---- layer norms around every sublayer, differential attention over separate key / value pools, top-k softmax router, SiLU-GLU experts
def layernorm_cast(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """``(x - mean) / sqrt(var + eps) * w + b`` (biased variance; fp32 arithmetic) in ``out_dtype``."""
    xf = x.float()
    d = xf - xf.mean(-1, keepdim=True)
    return (d * torch.rsqrt(d.pow(2).mean(-1, keepdim=True) + eps) * w.float() + b.float()).to(out_dtype)


def post_layernorm_add_norm_(x: torch.Tensor, y: torch.Tensor, post_w: torch.Tensor, post_b: torch.Tensor, mult: float, next_w: torch.Tensor,
                             next_b: torch.Tensor, eps: float, act_dtype: torch.dtype) -> torch.Tensor:
    """Sandwich-norm residual step on the fp32 stream ``x`` (in place): ``x += mult * LN(y; post_w, post_b)``, then returns
    ``LN(x; next_w, next_b)`` in the activation dtype: the input of the sublayer that follows."""
    x += mult * layernorm_cast(y, post_w, post_b, eps, torch.float32)
    return layernorm_cast(x, next_w, next_b, eps, act_dtype)


def paged_kv_append(rows: torch.Tensor, k_col0: int, v_col0: int, kpool: torch.Tensor, vpool: torch.Tensor, meta: BatchMeta):
    """Append this step's keys and values to the pools ``[pages, kv_heads, page, d]``: row ``t`` of ``rows`` holds the keys of all heads
    from column ``k_col0`` on (``kv_heads * d_k`` wide) and the values from ``v_col0`` on; token ``t`` goes to ``meta.slot_mapping[t]``."""
    P, G, page, dk = kpool.shape
    dv = vpool.shape[3]
    slot = meta.slot_mapping.long()
    pg, off = slot // page, slot % page
    T = rows.shape[0]
    kpool[pg, :, off] = rows[:, k_col0:k_col0 + G * dk].reshape(T, G, dk).to(kpool.dtype)
    vpool[pg, :, off] = rows[:, v_col0:v_col0 + G * dv].reshape(T, G, dv).to(vpool.dtype)


def position_temperature(positions: torch.Tensor, coef: float, every: float) -> torch.Tensor:
    """``1 + coef ln(floor((p + 1) / every) + 1)`` (fp32)."""
    return 1.0 + coef * torch.log(torch.floor((positions.float() + 1.0) / every) + 1.0)


def diff_attention(q: torch.Tensor, kpool: torch.Tensor, vpool: torch.Tensor, meta: BatchMeta, heads: int, scale: float, softcap: float,
                   temp_coef: float, temp_every: float, lam: float, eps: float, out_mult: float, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Causal differential attention over paged keys / values.  ``q`` ``[T, >= heads * 2 * d]`` (head by head ``[map 1 | map 2]``), keys
    ``kpool`` ``[pages, G, page, 2 d]`` laid out the same way, values ``vpool`` ``[pages, G, page, dv]`` shared by both maps; query head ``h``
    reads key / value head ``h // (heads / G)``.  Per map: ``s = cap tanh(q . k * scale * temp(p) / cap)`` (``softcap == 0``: no cap;
    ``temp`` = :func:`position_temperature` of the query's position, 1 when ``temp_coef == 0``), softmax over the keys ``j <= p``,
    ``a = P V``.  Then ``o = a1 - lam * a2``, ``o / sqrt(mean(o^2) + eps) * out_mult`` per head.  Returns ``[T, heads * dv]``."""
    T = q.shape[0]
    P, G, page, dk2 = kpool.shape
    d, dv, rep = dk2 // 2, vpool.shape[3], heads // G
    qf = q[:, :heads * dk2].float().view(T, heads, 2, d)
    temp = position_temperature(meta.positions, temp_coef, temp_every) if temp_coef != 0.0 else torch.ones(T, device=q.device)
    out = torch.empty(T, heads, dv, dtype=torch.float32, device=q.device)
    bt = meta.block_tables.long()
    for b, (s, e, c0, _) in enumerate(_seq_ranges(meta)):
        n = c0 + (e - s)
        idx = torch.arange(n, device=q.device)
        pg, off = bt[b, idx // page], idx % page
        K = kpool[pg, :, off].float().view(n, G, 2, d).repeat_interleave(rep, 1)          # [n, H, 2, d]
        V = vpool[pg, :, off].float().repeat_interleave(rep, 1)                           # [n, H, dv]
        sc = torch.einsum("thcd,nhcd->thcn", qf[s:e], K) * (scale * temp[s:e]).view(-1, 1, 1, 1)
        if softcap:
            sc = softcap * torch.tanh(sc / softcap)
        qpos = (c0 + torch.arange(e - s, device=q.device))[:, None]
        sc = sc.masked_fill((idx[None, :] > qpos)[:, None, None, :], float("-inf"))
        a = torch.einsum("thcn,nhv->thcv", torch.softmax(sc, -1), V)
        o = a[:, :, 0] - lam * a[:, :, 1]
        out[s:e] = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * out_mult
    return out.view(T, heads * dv).to(out_dtype)


def diff_attention_prefill(q, kpool, vpool, meta: BatchMeta, heads: int, scale: float, softcap: float, temp_coef: float, temp_every: float,
                           lam: float, eps: float, out_mult: float, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Single-sequence prefill form of :func:`diff_attention` (the CUDA backend runs it as matrix products); same math here."""
    return diff_attention(q, kpool, vpool, meta, heads, scale, softcap, temp_coef, temp_every, lam, eps, out_mult, out_dtype)


def softmax_topk(z: torch.Tensor, bias: Optional[torch.Tensor], num_experts: int, top: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Router on fp32 logits ``z[:, :num_experts] + bias``: the ``top`` largest logits (ties: lowest id), weights = softmax over the chosen
    logits alone.  Returns ``(idx int32 [T, top], w fp32 [T, top])``."""
    zz = z[:, :num_experts].float()
    if bias is not None:
        zz = zz + bias.float()
    order = torch.sort(zz, dim=-1, descending=True, stable=True).indices[:, :top]
    return order.to(torch.int32), torch.softmax(torch.gather(zz, 1, order), -1)


def silu_glu(g: torch.Tensor, u: torch.Tensor, out_dtype: torch.dtype, row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(g) * u * s`` with ``s`` = ``row_scale`` (per row, default 1): scaling the input of the down projection equals scaling its
    output."""
    h = F.silu(g.float()) * u.float()
    if row_scale is not None:
        h = h * row_scale.float()[:, None]
    return h.to(out_dtype)


def moe_glu_experts(x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, Wg: LinearWeight, Wu: LinearWeight, Wd: LinearWeight) -> torch.Tensor:
    """``y[t] = sum_j w[t,j] expert_{idx[t,j]}(x[t])`` with experts ``W_down (silu(W_gate x) * (W_up x))``: the router weight scales the
    expert's OUTPUT.  Banks ``Wg``, ``Wu`` ``[E, F, K]``, ``Wd`` ``[E, K, F]``.  Returns fp32 ``[T, K]``."""
    T, k = idx.shape
    y = torch.zeros(T, Wd.weight.shape[1], dtype=torch.float32, device=x.device)
    il = idx.long()
    for e in range(Wg.weight.shape[0]):
        tok, slot = torch.where(il == e)
        if tok.numel() == 0:
            continue
        xe = x[tok].float()
        h = silu_glu(xe @ Wg.weight[e].float().t(), xe @ Wu.weight[e].float().t(), x.dtype)
        y.index_add_(0, tok, (h.float() @ Wd.weight[e].float().t()) * w[tok, slot].float()[:, None])
    return y


# ---- several residual streams mixed per sublayer with dynamic-tanh norms, gated delta rule with per-channel decays, grouped-query
# ---- attention inside fixed blocks of positions with a sink, minGRU, group-limited softmax router, squared-ReLU experts
def relu2_(x: torch.Tensor) -> torch.Tensor:
    """``max(x, 0)^2`` in place."""
    return x.copy_((torch.relu(x.float()) ** 2).to(x.dtype))


def stream_embed(table: torch.Tensor, ids: torch.Tensor, scale: float, streams: int) -> torch.Tensor:
    """``streams`` equal copies of ``table[ids] * scale``: the fp32 residual streams ``[T, streams, width]`` at the start of a stack."""
    x = table[ids.long()].float() * float(scale)
    return x[:, None, :].repeat(1, int(streams), 1).contiguous()


def dyt_cast(x: torch.Tensor, alpha: float, w: torch.Tensor, b: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """Dynamic tanh in the place of a norm: ``tanh(alpha x) * w + b`` (no row statistics; fp32 arithmetic)."""
    return (torch.tanh(float(alpha) * x.float()) * w.float() + b.float()).to(out_dtype)


def hyper_step_(xs: torch.Tensor, y: Optional[torch.Tensor], y2: Optional[torch.Tensor], gate: Optional[torch.Tensor], ls: Optional[torch.Tensor],
                mix: Optional[torch.Tensor], out_w: Optional[torch.Tensor], mult: float, in_w: torch.Tensor, alpha: float, w: torch.Tensor,
                b: torch.Tensor, act_dtype: torch.dtype) -> torch.Tensor:
    """Residual step over several streams ``xs`` fp32 ``[T, S, width]`` (in place) and the read for the sublayer that follows.
    With ``r = (y + y2) * ls * sigmoid(gate)`` (``y2``, ``ls``, ``gate`` optional: a second branch, a per-channel layer scale, gate
    logits per element): ``xs[:, t] <- sum_s mix[s, t] xs[:, s] + mult * out_w[t] * r`` for all ``t`` at once; then returns
    ``dyt(sum_s in_w[s] xs[:, s])`` in the activation dtype.  ``y is None``: only the read (the first sublayer of a stack)."""
    if y is not None:
        r = y.float()
        if y2 is not None:
            r = r + y2.float()
        if ls is not None:
            r = r * ls.float()
        if gate is not None:
            r = r * torch.sigmoid(gate.float())
        new = torch.einsum("st,nsw->ntw", mix.float(), xs) + float(mult) * out_w.float()[None, :, None] * r[:, None, :]
        xs.copy_(new)
    return dyt_cast(torch.einsum("s,nsw->nw", in_w.float(), xs), alpha, w, b, act_dtype)


def delta_scan(qkv: torch.Tensor, beta: torch.Tensor, dt: torch.Tensor, dt_bias: torch.Tensor, A_log: torch.Tensor, state: torch.Tensor,
               meta: BatchMeta, heads: int, kv_heads: int, dim: int, vdim: int, q_scale: float, unit_eps: float = 1e-6) -> torch.Tensor:
    """Gated delta rule with one decay per head and key channel (fp32), per head ``h`` with query / key head ``h // (heads / kv_heads)``:
    ``q, k`` made unit vectors (``x / sqrt(sum x^2 + unit_eps)``; ``q`` times ``q_scale``), ``b = sigmoid(beta_h)``,
    ``g = exp(-exp(A_log_h) softplus(dt + dt_bias))`` (``[dim]``), then ``S <- g[:, None] S``, ``u = b (v - S^T k)``, ``S <- S + k u^T``,
    ``o = S^T q``.  ``qkv`` columns ``[q: kv_heads*dim | k: kv_heads*dim | v: heads*vdim]`` (after the short convolution), ``beta``
    ``[T, heads]`` raw, ``dt`` ``[T, heads*dim]`` raw; ``state`` ``[slots, heads, dim, vdim]`` fp32.  Returns fp32 ``[T, heads*vdim]``."""
    T, H, G, D, V = qkv.shape[0], heads, kv_heads, dim, vdim
    q = qkv[:, :G * D].float().view(T, G, D)
    k = qkv[:, G * D:2 * G * D].float().view(T, G, D)
    v = qkv[:, 2 * G * D:2 * G * D + H * V].float().view(T, H, V)
    q = (q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + unit_eps) * q_scale).repeat_interleave(H // G, 1)
    k = (k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + unit_eps)).repeat_interleave(H // G, 1)
    bt = torch.sigmoid(beta[:, :H].float())
    g = torch.exp(-torch.exp(A_log.float()).view(1, H, 1) * F.softplus(dt[:, :H * D].float() + dt_bias.float(), threshold=30.0).view(T, H, D))
    o = torch.empty(T, H, V, dtype=torch.float32, device=qkv.device)
    for s, e, c0, slot in _seq_ranges(meta):
        if e == s:
            continue
        S = state[slot].clone() if c0 > 0 else torch.zeros_like(state[slot])
        for t in range(s, e):
            S = g[t][:, :, None] * S
            u = bt[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
            S = S + k[t][:, :, None] * u[:, None, :]
            o[t] = torch.einsum("hdv,hd->hv", S, q[t])
        state[slot] = S
    return o.view(T, H * V)


def qk_norm_rope_append(rows: torch.Tensor, q_col0: int, k_col0: int, v_col0: int, heads: int, dim: int, qn_w: torch.Tensor, kn_w: torch.Tensor,
                        eps: float, inv_freq: torch.Tensor, kpool: torch.Tensor, vpool: torch.Tensor, meta: BatchMeta) -> torch.Tensor:
    """Attention prologue on a fused projection's rows ``[.. q: heads*dim .. k: G*dim .. v: G*dv ..]``: per head ``x / sqrt(mean(x^2) + eps)
    * w`` on queries and keys (weights ``[dim]`` shared by the heads), then adjacent pairs ``(2i, 2i+1)`` of the first ``2 len(inv_freq)``
    entries turn by ``position * inv_freq[i]``; keys and (untouched) values go to the pools ``[pages, G, page, d]`` at
    ``meta.slot_mapping``.  Returns the queries fp32 ``[T, heads, dim]``."""
    P, G, page, dk = kpool.shape
    dv = vpool.shape[3]
    T = rows.shape[0]
    nrm = lambda x, w: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    q = nrm(rows[:, q_col0:q_col0 + heads * dim].float().view(T, heads, dim), qn_w)
    k = nrm(rows[:, k_col0:k_col0 + G * dk].float().view(T, G, dk), kn_w)
    if inv_freq is not None and inv_freq.numel():
        q, k = _rot_pairs(q, meta.positions, inv_freq), _rot_pairs(k, meta.positions, inv_freq)
    slot = meta.slot_mapping.long()
    pg, off = slot // page, slot % page
    kpool[pg, :, off] = k.to(kpool.dtype)
    vpool[pg, :, off] = rows[:, v_col0:v_col0 + G * dv].reshape(T, G, dv).to(vpool.dtype)
    return q.contiguous()


def sink_attention(q: torch.Tensor, kpool: torch.Tensor, vpool: torch.Tensor, sink: Optional[torch.Tensor], meta: BatchMeta, scale: float,
                   block: int = 0, window: int = 0, out_mult: float = 1.0, out_dtype: torch.dtype = torch.float32,
                   out: Optional[torch.Tensor] = None, out_col0: int = 0) -> torch.Tensor:
    """Causal grouped-query attention over paged keys / values.  ``q`` ``[T, H, d]`` (normed and rotated), pools ``[pages, G, page, d]`` /
    ``[pages, G, page, dv]``; head ``h`` reads key / value head ``h // (H / G)``.  The query at position ``i`` sees keys ``j <= i`` with
    ``floor(j / block) == floor(i / block)`` (``block > 0``: blocks counted from position 0 of the sequence) and ``i - j < window``
    (``window > 0``).  ``p_j = exp(s_j) / (exp(sink_h) + sum exp(s))`` (``sink=None``: the ordinary softmax).  The result times
    ``out_mult`` goes to ``out[:, out_col0 : out_col0 + H * dv]`` (a fresh ``[T, H * dv]`` tensor by default), which is returned."""
    T, H, D = q.shape
    P, G, page, _ = kpool.shape
    dv, rep = vpool.shape[3], H // G
    res = torch.empty(T, H, dv, dtype=torch.float32, device=q.device)
    bt = meta.block_tables.long()
    qf = q.float()
    for b, (s, e, c0, _) in enumerate(_seq_ranges(meta)):
        n = c0 + (e - s)
        idx = torch.arange(n, device=q.device)
        pg, off = bt[b, idx // page], idx % page
        K = kpool[pg, :, off].float().repeat_interleave(rep, 1)                           # [n, H, d]
        V = vpool[pg, :, off].float().repeat_interleave(rep, 1)                           # [n, H, dv]
        sc = torch.einsum("thd,nhd->thn", qf[s:e], K) * scale
        qpos = (c0 + torch.arange(e - s, device=q.device))[:, None]
        mask = idx[None, :] > qpos
        if block > 0:
            mask = mask | ((idx[None, :] // block) != (qpos // block))
        if window > 0:
            mask = mask | (idx[None, :] <= qpos - window)
        sc = sc.masked_fill(mask[:, None, :], float("-inf"))
        if sink is None:
            p = torch.softmax(sc, -1)
        else:
            sk = sink.float().view(1, H, 1).expand(e - s, H, 1)
            p = torch.softmax(torch.cat([sc, sk], -1), -1)[..., :n]
        res[s:e] = torch.einsum("thn,nhv->thv", p, V)
    res = res.view(T, H * dv) * out_mult
    if out is None:
        return res.to(out_dtype)
    out[:, out_col0:out_col0 + H * dv] = res.to(out.dtype)
    return out


def sink_attention_prefill(q, kpool, vpool, sink, meta: BatchMeta, scale: float, block: int = 0, window: int = 0, out_mult: float = 1.0,
                           out_dtype: torch.dtype = torch.float32, out: Optional[torch.Tensor] = None, out_col0: int = 0) -> torch.Tensor:
    """Single-sequence prefill form of :func:`sink_attention` (the CUDA backend runs it as matrix products); same math here."""
    return sink_attention(q, kpool, vpool, sink, meta, scale, block, window, out_mult, out_dtype, out, out_col0)


def mingru_scan(rows: torch.Tensor, z_col0: int, x_col0: int, g_col0: int, width: int, state: torch.Tensor, meta: BatchMeta,
                out_mult: float = 1.0, out_dtype: torch.dtype = torch.float32, out: Optional[torch.Tensor] = None, out_col0: int = 0) -> torch.Tensor:
    """Element-wise gated recurrence whose gates read the current token only (fp32): ``z = sigmoid(rows[z])``, candidate ``c = u + 1/2``
    where ``u = rows[x] >= 0`` and ``sigmoid(u)`` below, ``S <- (1 - z) S + z c``; the result ``S * silu(rows[g]) * out_mult`` goes to
    ``out[:, out_col0 : out_col0 + width]`` (a fresh tensor by default).  ``rows``: a fused projection's output (biases added);
    ``state`` ``[slots, width]`` fp32."""
    T = rows.shape[0]
    z = torch.sigmoid(rows[:, z_col0:z_col0 + width].float())
    u = rows[:, x_col0:x_col0 + width].float()
    c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    gt = F.silu(rows[:, g_col0:g_col0 + width].float())
    res = torch.empty(T, width, dtype=torch.float32, device=rows.device)
    for s, e, c0, slot in _seq_ranges(meta):
        if e == s:
            continue
        S = state[slot].clone() if c0 > 0 else torch.zeros_like(state[slot])
        for t in range(s, e):
            S = (1.0 - z[t]) * S + z[t] * c[t]
            res[t] = S * gt[t]
        state[slot] = S
    res = res * out_mult
    if out is None:
        return res.to(out_dtype)
    out[:, out_col0:out_col0 + width] = res.to(out.dtype)
    return out


def group_softmax_topk(z: torch.Tensor, correction: Optional[torch.Tensor], num_experts: int, top: int, n_groups: int = 1,
                       keep_groups: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    """Router on fp32 logits ``z[:, :num_experts]``: scores ``s = softmax(z)`` over all experts; the choice is made on ``s + correction``:
    with ``n_groups > 1`` the experts form equal runs of neighbours, a group's value is its largest choice score, and only experts of the
    ``keep_groups`` best groups can be chosen (the others count as minus infinity); the ``top`` largest win (ties: lowest id).  Weights =
    the chosen experts' plain ``s``.  Returns ``(idx int32 [T, top], w fp32 [T, top])``."""
    s = torch.softmax(z[:, :num_experts].float(), -1)
    c = s + correction.float() if correction is not None else s.clone()
    if n_groups > 1 and keep_groups < n_groups:
        gs = c.view(-1, n_groups, num_experts // n_groups).max(-1).values
        best = torch.sort(gs, dim=-1, descending=True, stable=True).indices[:, :keep_groups]
        ok = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, best, True)
        c = c.masked_fill(~ok.repeat_interleave(num_experts // n_groups, 1), float("-inf"))
    order = torch.sort(c, dim=-1, descending=True, stable=True).indices[:, :top]
    return order.to(torch.int32), torch.gather(s, 1, order)


def moe_relu2_experts(x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, Wu: LinearWeight, Wd: LinearWeight) -> torch.Tensor:
    """``y[t] = sum_j w[t,j] expert_{idx[t,j]}(x[t])`` with experts ``W_down relu(W_up x)^2``: the router weight scales the expert's
    OUTPUT.  Banks ``Wu`` ``[E, F, K]``, ``Wd`` ``[E, K, F]``.  Returns fp32 ``[T, K]``."""
    T, k = idx.shape
    y = torch.zeros(T, Wd.weight.shape[1], dtype=torch.float32, device=x.device)
    il = idx.long()
    for e in range(Wu.weight.shape[0]):
        tok, slot = torch.where(il == e)
        if tok.numel() == 0:
            continue
        h = (torch.relu(x[tok].float() @ Wu.weight[e].float().t()) ** 2).to(x.dtype)
        y.index_add_(0, tok, (h.float() @ Wd.weight[e].float().t()) * w[tok, slot].float()[:, None])
    return y
