"""Perelorn: a hybrid decoder stack — every layer has one *mixer* (Mamba-2 state-space, latent attention with a softmax sink, or
lightning attention with a constant decay), an optional dense feed-forward, and a per-layer token input.  No reference counterpart
(the reference serves Llama / Gemma-2 / DeepSeek-V2 only).

Block structure (``rms(y) = y / sqrt(mean(y^2) + eps)``; the norm sits on the sublayer's OUTPUT and the sublayer reads ``x`` itself):

    x <- x + rms(mixer(x)) * norm1          x <- x + rms(W_down gelu(W_up x)) * norm2   (only if the layer has a feed-forward)
    x <- x + rms(W_proj (gelu_tanh(W_gate x) * side_embed[token, layer block])) * side_norm

Precision: the residual stream, every norm, the softmax and everything inside a recurrence are fp32 in both dtypes; projections,
the short convolution and their activations run in the model dtype (bf16 on the serving path) with fp32 accumulation.

Framework integration: layer order and every size come from ``ModelConfig.layer_specs``; attention layers keep ``[latent | rotated
key]`` rows in a paged pool, recurrent layers keep fp32 state (+ the convolution's last inputs) in per-sequence state slots
(``engine/kv_cache.py::HybridCache``); the ops are ``ops/reference.py`` (unfused PyTorch) / ``ops/b200.py`` (``ops/csrc/hybrid.cu``).

Latent attention runs in the weight-absorbed form, like DeepSeek-V2's decode path (``models/deepseek_v2.py::_post_load``): with
``k_h = W_uk[h] c`` and ``v_h = W_uv[h] c``,  ``q_h . k_h = (W_uk[h]^T q_h) . c``  and  ``W_o sum_j p_j v_hj = (W_o[:, h] W_uv[h]) sum_j p_j c_j``,
so ``W_uk`` is folded into the query up-projection and ``W_uv`` into the output projection once at load, and attention is
multi-query over the cached latent for prefill and decode alike.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import BatchMeta, LinearWeight, RopeSpec
from .base import StageModel


def _pad_rows(w: torch.Tensor, mult: int = 8) -> torch.Tensor:
    n = w.shape[0]
    if n % mult == 0:
        return w.contiguous()
    return torch.cat([w, w.new_zeros((mult - n % mult, w.shape[1]))]).contiguous()


class PerelornStage(StageModel):
    arch = "perelorn"
    PREFILL_GEMM_MIN_ROWS = 32

    def __init__(self, cfg, spec=None, dtype=torch.bfloat16, device="cpu", backend=None):
        super().__init__(cfg, spec, dtype, device, backend)
        if not (self.spec.is_first and self.spec.is_last):
            # every layer reads the step's token ids (per-layer token input) and the residual stream is fp32: the stage hand-off of
            # the pipeline runtimes carries neither
            raise NotImplementedError("Perelorn runs as a single stage (all layers in one process)")
        self.specs = cfg.layer_specs
        self.side_table = None
        self.rope_freqs: Dict[int, torch.Tensor] = {}

    # ---- cache geometry ---------------------------------------------------------------------------------------------
    def cache_layout(self):
        out = []
        for L in self.specs:
            m = L["mixer"]
            if L["type"] == "latent_attention":
                out.append(("paged", int(m["kv_rank"]) + int(m["rot_dim"]), self.dtype))
            elif L["type"] == "mamba2":
                ch = m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"]
                out.append(("state", {"ssm": ((m["heads"], m["state"], m["vdim"]), torch.float32),
                                      "conv": ((max(m["conv"] - 1, 0), ch), self.dtype)}))
            else:
                out.append(("state", {"kv": ((m["heads"], m["dim"], m["vdim"]), torch.float32)}))
        return out

    def kv_geometry(self):
        raise NotImplementedError("hybrid stack: see cache_layout()")

    # ---- weights ----------------------------------------------------------------------------------------------------
    def _w(self, sd, key) -> LinearWeight:
        """Linear weight ``[out, in]`` in the model dtype; output rows zero-padded to a multiple of 8 (GEMM tile rule), the real row
        count kept in ``n_real``."""
        w = sd.pop(key)
        lw = LinearWeight(weight=_pad_rows(w.to(device=self.device, dtype=self.dtype)))
        lw.n_real = w.shape[0]
        return lw

    def _lw(self, w: torch.Tensor) -> LinearWeight:
        lw = LinearWeight(weight=_pad_rows(w.to(device=self.device, dtype=self.dtype)))
        lw.n_real = w.shape[0]
        return lw

    def _f32(self, sd, key) -> torch.Tensor:
        return sd.pop(key).to(device=self.device, dtype=torch.float32).contiguous()

    def sanitize(self, sd):
        return dict(sd)

    def load_state(self, sd, strict: bool = True):
        sd = dict(sd)
        c = self.cfg
        self.embed_tokens = LinearWeight(weight=sd.pop("embed").to(device=self.device, dtype=self.dtype).contiguous())
        if c.token_side_dim:
            self.side_table = sd.pop("side.embed").to(device=self.device, dtype=self.dtype).contiguous()
        for i, L in enumerate(self.specs):
            p, m, w = f"l{i}.", L["mixer"], {}
            w["norm1"] = self._f32(sd, p + "norm1")
            if L["type"] == "mamba2":
                w.update(inp=self._w(sd, p + "mix.in"), conv_w=self._f32(sd, p + "mix.conv"), conv_b=self._f32(sd, p + "mix.conv.b"),
                         dt_bias=self._f32(sd, p + "mix.dt_bias"), A_log=self._f32(sd, p + "mix.A_log"), D=self._f32(sd, p + "mix.D"),
                         gnorm=self._f32(sd, p + "mix.norm"), o=self._w(sd, p + "mix.o"))
            elif L["type"] == "lightning":
                qkvg = torch.cat([sd.pop(p + f"mix.{n}") for n in ("q", "k", "v", "g")])
                w.update(qkvg=self._lw(qkvg), gnorm=self._f32(sd, p + "mix.norm"), o=self._w(sd, p + "mix.o"),
                         decay=torch.tensor([float(d) for d in m["decay"]], dtype=torch.float32, device=self.device))
            else:
                H, D, R, V, Lr, Qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
                if int(m["rot"]["dims"]) != R:
                    raise ValueError("latent attention: rot.dims must equal rot_dim")
                dev = self.device
                uq = sd.pop(p + "mix.uq").to(dev, torch.float32).view(H, D + R, Qr)
                uk = sd.pop(p + "mix.uk").to(dev, torch.float32).view(H, D, Lr)
                uv = sd.pop(p + "mix.uv").to(dev, torch.float32).view(H, V, Lr)
                wo = sd.pop(p + "mix.o").to(dev, torch.float32)
                q_abs = torch.cat([torch.einsum("hdl,hdq->hlq", uk, uq[:, :D]), uq[:, D:]], 1).reshape(H * (Lr + R), Qr)
                o_abs = torch.einsum("whv,hvl->whl", wo.view(wo.shape[0], H, V), uv).reshape(wo.shape[0], H * Lr)
                w.update(dqkv=self._lw(torch.cat([sd.pop(p + "mix.dq"), sd.pop(p + "mix.dkv")])), qn=self._f32(sd, p + "mix.dq.norm"),
                         kvn=self._f32(sd, p + "mix.dkv.norm"), q_abs=self._lw(q_abs), o=self._lw(o_abs), sink=self._f32(sd, p + "mix.sink"))
                half = R // 2
                self.rope_freqs[i] = (float(m["rot"]["base"]) ** (-2.0 * torch.arange(half, dtype=torch.float64) / R)).float().to(dev)
            if L["mlp"]:
                w.update(norm2=self._f32(sd, p + "norm2"), up=self._w(sd, p + "mlp.up"), down=self._w(sd, p + "mlp.down"))
            if c.token_side_dim:
                w.update(side_gate=self._w(sd, p + "side.gate"), side_proj=self._w(sd, p + "side.proj"),
                         side_norm=self._f32(sd, p + "side.norm"))
            self.layer_weights[i] = w
        self.norm_w = self._f32(sd, "final.norm")
        self.lm_head = self._w(sd, "head")
        if strict and sd:
            raise ValueError(f"unexpected checkpoint tensors: {sorted(sd)[:8]} ...")
        self.rope = RopeSpec(inv_freq=torch.zeros(1), rot_dim=0, interleaved=False)
        return self

    # ---- forward ----------------------------------------------------------------------------------------------------
    def _mm(self, x, W: LinearWeight, f32: bool = False, act: str = "none"):
        y = self.ops.linear_any(x, W, torch.float32 if f32 else self.dtype, act)
        return y if y.shape[1] == W.n_real else y[:, :W.n_real]

    def _mamba2(self, w, m, ha, meta, st):
        O, eps = self.ops, self.cfg.rms_norm_eps
        H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
        inner, ch = H * P, H * P + 2 * G * N
        u = self._mm(ha, w["inp"])                                                   # [z | x B C | dt]
        xbc = O.causal_conv_silu(u[:, inner:inner + ch], w["conv_w"], w["conv_b"], st["conv"], meta)
        y = O.ssm_scan(xbc, u[:, inner + ch:inner + ch + H], w["dt_bias"], w["A_log"], w["D"], st["ssm"], meta, H, P, N, G)
        yn = O.gated_rmsnorm(y, u[:, :inner], w["gnorm"], eps, int(m["norm_groups"]), "silu_pre", self.dtype)
        return self._mm(yn, w["o"], True)

    def _lightning(self, w, m, ha, meta, st):
        O, eps = self.ops, self.cfg.rms_norm_eps
        H, D, V = m["heads"], m["dim"], m["vdim"]
        u = self._mm(ha, w["qkvg"])
        o = O.decay_scan(u, w["decay"], st["kv"], meta, H, D, V)
        on = O.gated_rmsnorm(o, u[:, 2 * H * D + H * V:], w["gnorm"], eps, 1, "sigmoid_post", self.dtype)
        return self._mm(on, w["o"], True)

    def _latent(self, i, w, m, ha, meta, pool):
        O, eps = self.ops, self.cfg.rms_norm_eps
        H, R, Lr, Qr = m["heads"], m["rot_dim"], m["kv_rank"], m["q_rank"]
        T = ha.shape[0]
        dqkv = self._mm(ha, w["dqkv"])
        cq = O.latent_kv_prologue(dqkv, Qr, Lr, w["qn"], w["kvn"], eps, pool, meta, self.rope_freqs[i])
        q = self._mm(cq, w["q_abs"])
        if not q.is_contiguous():
            q = q.contiguous()
        # one sequence with a long portion (prompt prefill): two tensor-core GEMMs around a masked softmax; ragged / decode steps: the
        # paged multi-query kernel
        attend = O.latent_attention_prefill if (meta.num_seqs == 1 and T >= self.PREFILL_GEMM_MIN_ROWS) else O.latent_attention
        o = attend(q.view(T, H, Lr + R), pool, w["sink"], meta, float(m["scale"]), Lr, self.rope_freqs[i],
                               self.dtype)
        return self._mm(o.view(T, H * Lr), w["o"], True)

    def layer_forward(self, i, h, ha, tokens, meta, kv):
        O, c, L, w = self.ops, self.cfg, self.specs[i], self.layer_weights[i]
        m, eps = L["mixer"], c.rms_norm_eps
        if L["type"] == "mamba2":
            y = self._mamba2(w, m, ha, meta, kv.state[i])
        elif L["type"] == "lightning":
            y = self._lightning(w, m, ha, meta, kv.state[i])
        else:
            y = self._latent(i, w, m, ha, meta, kv.k[i])
        ha = O.post_norm_add_(h, y, w["norm1"], eps, self.dtype)
        if L["mlp"]:
            y = self._mm(self._mm(ha, w["up"], act="gelu_erf"), w["down"], True)      # exact gelu in the up-projection's epilogue
            ha = O.post_norm_add_(h, y, w["norm2"], eps, self.dtype)
        if c.token_side_dim:
            g = O.side_gate(self._mm(ha, w["side_gate"]), self.side_table, tokens, i * c.token_side_dim)
            ha = O.post_norm_add_(h, self._mm(g, w["side_proj"], True), w["side_norm"], eps, self.dtype)
        return ha

    @torch.inference_mode()
    def forward(self, x, meta: BatchMeta, kv, all_logits: bool = False, layer_out=None):
        """``x``: token ids ``[T]``.  Returns fp32 logits ``[B, V]`` (``[T, V]`` with ``all_logits``).  ``layer_out``: optional list that
        receives a copy of the residual stream after every layer."""
        O, c = self.ops, self.cfg
        if meta.state_slots is None and any(L["type"] in ("mamba2", "lightning") for L in self.specs):      # a stack of attention layers alone holds pages only
            raise ValueError("Perelorn needs state slots in the step metadata (BatchMeta.build(..., state_slots=...))")
        tokens = x.to(torch.int64).contiguous()
        W = c.hidden_size
        h = O.gather_rows(self.embed_tokens.weight, tokens, 0, W, torch.float32)          # fp32 residual stream
        ha = h if self.dtype == torch.float32 else O.gather_rows(self.embed_tokens.weight, tokens, 0, W, self.dtype)
        for i in range(len(self.specs)):
            ha = self.layer_forward(i, h, ha, tokens, meta, kv)
            if layer_out is not None:
                layer_out.append(h.clone())
        if not all_logits and meta.num_tokens != meta.num_seqs:
            h = h.index_select(0, meta.last_idx.long())
        hn = O.rmsnorm_cast(h, self.norm_w, c.rms_norm_eps, self.dtype)
        logits = self._mm(hn, self.lm_head, True)
        if c.logit_scale != 1.0:
            logits = logits * c.logit_scale
        return logits.contiguous()

    __call__ = forward


Model = PerelornStage
