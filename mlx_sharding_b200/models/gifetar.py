"""Gifetar: a sandwich-norm decoder stack.  Every layer has a *differential attention* mixer — two softmax maps per head over the same
values, subtracted with a learned weight, then a per-head unit-RMS norm — and an optional mixture-of-experts feed-forward with a
top-k softmax router and SiLU-GLU experts.  No reference counterpart (the reference serves Llama / Gemma-2 / DeepSeek-V2 only).

Block structure (``LN`` = layer norm with weight and bias; ``m`` = ``residual_mult``):

    x <- x + m * LN1b(mixer(LN1(x)))          x <- x + m * LN2b(ff(LN2(x)))   (only if the layer has a feed-forward)

Mixer, per query head ``h`` (key / value head ``g = h // (heads / kv_heads)``), maps ``c = 1, 2``:

    s_c[i, j] = cap * tanh(temp(i) * scale * q_c[i] . k_c[j] / cap),   temp(i) = 1 + coef * ln(floor((i + 1) / every) + 1),   j <= i
    a_c = softmax(s_c) V_g,   o = a_1 - lambda * a_2,   o <- o / sqrt(mean(o^2) + eps) * (1 - diff)
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff                    (one number per layer, taken at load)

No rotation: positions enter through the causal mask and the query temperature only.  The LM head is the embedding table.

Precision: the residual stream, every norm, scores / softmax / the map difference and its norm, and the router are fp32 in both dtypes;
projections and expert activations run in the model dtype (bf16 on the serving path) with fp32 accumulation.

Framework integration: layer order and every size come from ``ModelConfig.layer_specs``; each layer keeps keys ``[map 1 | map 2]`` and
values in its own pair of paged pools (``("paged_kv", kv_heads, 2 * dim, vdim, dtype)`` in the cache layout of
``engine/kv_cache.py::HybridCache``); there is no recurrent state, so sequences hold pages only.  The ops are ``ops/reference.py`` (unfused
PyTorch) / ``ops/b200.py`` (``ops/csrc/diffattn.cu``, ``ops/csrc/hybrid.cu``); each residual add is fused with the output-side norm before
it and the input-side norm after it.
"""
from __future__ import annotations

import math

import torch

from ..ops import BatchMeta, LinearWeight, RopeSpec
from .base import StageModel
from .perelorn import _pad_rows


class GifetarStage(StageModel):
    arch = "gifetar"
    PREFILL_GEMM_MIN_ROWS = 32

    def __init__(self, cfg, spec=None, dtype=torch.bfloat16, device="cpu", backend=None):
        super().__init__(cfg, spec, dtype, device, backend)
        if not (self.spec.is_first and self.spec.is_last):
            raise NotImplementedError("Gifetar runs as a single stage (the residual stream is fp32: the pipeline hand-off does not carry it)")
        self.specs = cfg.layer_specs

    # ---- cache geometry ---------------------------------------------------------------------------------------------
    def cache_layout(self):
        return [("paged_kv", int(L["mixer"]["kv_heads"]), 2 * int(L["mixer"]["dim"]), int(L["mixer"]["vdim"]), self.dtype) for L in self.specs]

    def kv_geometry(self):
        raise NotImplementedError("per-layer pools: see cache_layout()")

    # ---- weights ----------------------------------------------------------------------------------------------------
    def _lw(self, w: torch.Tensor, bias: torch.Tensor = None) -> LinearWeight:
        """Linear weight ``[out, in]`` in the model dtype; output rows zero-padded to a multiple of 8 (GEMM tile rule), the real row
        count kept in ``n_real``."""
        lw = LinearWeight(weight=_pad_rows(w.to(device=self.device, dtype=self.dtype)))
        if bias is not None:
            lw.bias = _pad_rows(bias.to(device=self.device, dtype=self.dtype)[:, None])[:, 0].contiguous()
        lw.n_real = w.shape[0]
        return lw

    def _f32(self, sd, key) -> torch.Tensor:
        return sd.pop(key).to(device=self.device, dtype=torch.float32).contiguous()

    def _ln(self, sd, key):
        return self._f32(sd, key), self._f32(sd, key + ".b")

    def sanitize(self, sd):
        return dict(sd)

    def load_state(self, sd, strict: bool = True):
        sd = dict(sd)
        dev = self.device
        emb = sd.pop("embed")
        self.embed_tokens = LinearWeight(weight=emb.to(device=dev, dtype=self.dtype).contiguous())
        self.lm_head = self._lw(emb) if emb.shape[0] % 8 else self.embed_tokens
        self.lm_head.n_real = emb.shape[0]
        for i, L in enumerate(self.specs):
            p, m, w = f"l{i}.", L["mixer"], {}
            w["norm1"], w["norm1b"] = self._ln(sd, p + "norm1"), self._ln(sd, p + "norm1b")
            D = int(m["dim"])
            names = ("q", "k", "v")
            w["qkv"] = self._lw(torch.cat([sd.pop(p + f"mix.{n}") for n in names]), torch.cat([sd.pop(p + f"mix.{n}.b") for n in names]))
            lv = {n: sd.pop(p + "mix." + n).double().cpu() for n in ("lq1", "lk1", "lq2", "lk2")}
            assert all(v.numel() == D for v in lv.values())
            w["lam"] = math.exp(float((lv["lq1"] * lv["lk1"]).sum())) - math.exp(float((lv["lq2"] * lv["lk2"]).sum())) + float(m["diff"])
            w["o"] = self._lw(sd.pop(p + "mix.o"))
            mlp = L["mlp"]
            if mlp:
                w["norm2"], w["norm2b"] = self._ln(sd, p + "norm2"), self._ln(sd, p + "norm2b")
                E = int(mlp["router"]["experts"])
                bank = lambda n: LinearWeight(weight=torch.stack([sd.pop(p + f"mlp.e{e}.{n}") for e in range(E)]).to(device=dev, dtype=self.dtype).contiguous())
                w.update(e_gate=bank("gate"), e_up=bank("up"), e_down=bank("down"))
                w["router"], w["router_b"] = self._f32(sd, p + "mlp.router"), self._f32(sd, p + "mlp.router.b")
            self.layer_weights[i] = w
        self.final_norm = self._ln(sd, "final.norm")
        self.norm_w = self.final_norm[0]
        if strict and sd:
            raise ValueError(f"unexpected checkpoint tensors: {sorted(sd)[:8]} ...")
        self.rope = RopeSpec(inv_freq=torch.zeros(1), rot_dim=0, interleaved=False)
        return self

    # ---- forward ----------------------------------------------------------------------------------------------------
    def _mm(self, x, W: LinearWeight, f32: bool = False):
        y = self.ops.linear_any(x, W, torch.float32 if f32 else self.dtype)
        return y if y.shape[1] == W.n_real else y[:, :W.n_real]

    def _attention(self, w, m, ha, meta, kpool, vpool):
        O, eps = self.ops, self.cfg.rms_norm_eps
        H, G, D, V = (int(m[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
        T = ha.shape[0]
        u = self._mm(ha, w["qkv"])                                                   # [q: H*2D | k: G*2D | v: G*V], biases added
        O.paged_kv_append(u, H * 2 * D, (H + G) * 2 * D, kpool, vpool, meta)
        qt = m.get("q_temp") or {}
        attend = O.diff_attention_prefill if (meta.num_seqs == 1 and T >= self.PREFILL_GEMM_MIN_ROWS) else O.diff_attention
        o = attend(u, kpool, vpool, meta, H, float(m["scale"]), float(m.get("softcap") or 0.0), float(qt.get("coef", 0.0)),
                   float(qt.get("every", 1.0)), w["lam"], eps, 1.0 - float(m["diff"]), self.dtype)
        return self._mm(o, w["o"], True)

    def _moe(self, w, mlp, ha):
        O = self.ops
        E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
        idx, wts = O.softmax_topk(O.router_logits(ha, w["router"]), w["router_b"], E, top)
        return O.moe_glu_experts(ha, idx, wts, w["e_gate"], w["e_up"], w["e_down"])

    def layer_forward(self, i, h, ha, meta, kv, next_norm):
        """``h``: fp32 residual stream (updated in place); ``ha``: ``LN1(h)`` in the activation dtype.  Returns the next sublayer's normed
        input (``next_norm``: weight and bias of the norm that follows this layer)."""
        O, L, w = self.ops, self.specs[i], self.layer_weights[i]
        eps, mult = self.cfg.rms_norm_eps, float(self.cfg.residual_mult)
        y = self._attention(w, L["mixer"], ha, meta, kv.k[i], kv.v[i])
        if not L["mlp"]:
            return O.post_layernorm_add_norm_(h, y, *w["norm1b"], mult, *next_norm, eps, self.dtype)
        ha = O.post_layernorm_add_norm_(h, y, *w["norm1b"], mult, *w["norm2"], eps, self.dtype)
        y = self._moe(w, L["mlp"], ha)
        return O.post_layernorm_add_norm_(h, y, *w["norm2b"], mult, *next_norm, eps, self.dtype)

    @torch.inference_mode()
    def forward(self, x, meta: BatchMeta, kv, all_logits: bool = False, layer_out=None):
        """``x``: token ids ``[T]``.  Returns fp32 logits ``[B, V]`` (``[T, V]`` with ``all_logits``).  ``layer_out``: optional list that
        receives a copy of the residual stream after every layer."""
        O, c = self.ops, self.cfg
        tokens = x.to(torch.int64).contiguous()
        n = len(self.specs)
        h = O.gather_rows(self.embed_tokens.weight, tokens, 0, c.hidden_size, torch.float32)          # fp32 residual stream
        ha = O.layernorm_cast(h, *(self.layer_weights[0]["norm1"] if n else self.final_norm), c.rms_norm_eps, self.dtype)
        for i in range(n):
            ha = self.layer_forward(i, h, ha, meta, kv, self.layer_weights[i + 1]["norm1"] if i + 1 < n else self.final_norm)
            if layer_out is not None:
                layer_out.append(h.clone())
        if not all_logits and meta.num_tokens != meta.num_seqs:
            ha = ha.index_select(0, meta.last_idx.long())
        return self._mm(ha, self.lm_head, True).contiguous()

    __call__ = forward


Model = GifetarStage
