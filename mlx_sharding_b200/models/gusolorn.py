"""Gusolorn: a pre-norm hybrid decoder stack.  Every layer has one *mixer* — an mLSTM (matrix memory with exponential gating and a
running maximum) or latent attention (multi-query over a cached low-rank latent plus one shared rotated key, sliding window, optionally
reading ANOTHER layer's cached rows) — and an optional feed-forward — dense (exact gelu) or a mixture of clamped-GLU experts with a
sigmoid router and a gated always-on expert.  No reference counterpart (the reference serves Llama / Gemma-2 / DeepSeek-V2 only).

Block structure (``norm(x) = x / sqrt(mean(x^2) + eps) * (1 + w)``, weights stored around zero; ``ls*`` per-channel layer scales):

    x <- x + ls1 * mixer(norm1(x))          x <- x + ls2 * ff(norm2(x))   (only if the layer has a feed-forward)

Precision: the residual stream, every norm, the softmax, router logits and everything inside the recurrence (gates, their caps,
log-sigmoid, exponentials, the running maximum, the state and its normaliser) are fp32 in both dtypes; projections and their
activations run in the model dtype (bf16 on the serving path) with fp32 accumulation.

Framework integration: layer order and every size come from ``ModelConfig.layer_specs``; attention layers keep ``[latent | rotated
key]`` rows in a paged pool — a layer with ``kv_from`` owns no pool and aliases the named layer's (``("alias", j)`` in the cache
layout) — and mLSTM layers keep fp32 state in per-sequence state slots (``engine/kv_cache.py::HybridCache``).  The ops are
``ops/reference.py`` (unfused PyTorch) / ``ops/b200.py`` (``ops/csrc/hybrid.cu``); each residual add is fused with the norm that follows.

Latent attention runs in the weight-absorbed form (like ``models/perelorn.py`` and DeepSeek-V2's decode path): with ``k_h = W_uk[h] c``
and ``v_h = W_uv[h] c``,  ``q_h . k_h = (W_uk[h]^T q_h) . c``  and  ``W_o sum_j p_j v_hj = (W_o[:, h] W_uv[h]) sum_j p_j c_j``, so
``W_uk`` is folded into the query projection and ``W_uv`` into the output projection once at load, and attention is multi-query over
the cached rows for prefill and decode alike; a layer that reads another layer's rows only differs in these folded weights.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import BatchMeta, LinearWeight, RopeSpec
from .base import StageModel
from .perelorn import _pad_rows


class GusolornStage(StageModel):
    arch = "gusolorn"
    PREFILL_GEMM_MIN_ROWS = 32

    def __init__(self, cfg, spec=None, dtype=torch.bfloat16, device="cpu", backend=None):
        super().__init__(cfg, spec, dtype, device, backend)
        if not (self.spec.is_first and self.spec.is_last):
            # the residual stream is fp32 and layers may read an earlier layer's cache: the pipeline hand-off carries neither
            raise NotImplementedError("Gusolorn runs as a single stage (all layers in one process)")
        self.specs = cfg.layer_specs
        self.rope_freqs: Dict[int, torch.Tensor] = {}

    # ---- cache geometry ---------------------------------------------------------------------------------------------
    def cache_layout(self):
        out = []
        for L in self.specs:
            m = L["mixer"]
            if L["type"] == "latent_attention":
                if m.get("kv_from") is not None:
                    out.append(("alias", int(m["kv_from"])))
                else:
                    out.append(("paged", int(m["kv_rank"]) + int(m["rot_dim"]), self.dtype))
            else:
                H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
                nb = V // self.ops.mlstm_col_block(V)
                out.append(("state", {"S": ((H, D, V), torch.float32), "n": ((H, nb, D), torch.float32), "m": ((H, nb), torch.float32)}))
        return out

    def kv_geometry(self):
        raise NotImplementedError("hybrid stack: see cache_layout()")

    # ---- weights ----------------------------------------------------------------------------------------------------
    def _lw(self, w: torch.Tensor) -> LinearWeight:
        """Linear weight ``[out, in]`` in the model dtype; output rows zero-padded to a multiple of 8 (GEMM tile rule), the real row
        count kept in ``n_real``."""
        lw = LinearWeight(weight=_pad_rows(w.to(device=self.device, dtype=self.dtype)))
        lw.n_real = w.shape[0]
        return lw

    def _f32(self, sd, key) -> torch.Tensor:
        return sd.pop(key).to(device=self.device, dtype=torch.float32).contiguous()

    def _norm_w(self, sd, key) -> torch.Tensor:
        return (1.0 + self._f32(sd, key)).contiguous()         # stored around zero

    def sanitize(self, sd):
        return dict(sd)

    def load_state(self, sd, strict: bool = True):
        sd = dict(sd)
        dev = self.device
        self.embed_tokens = LinearWeight(weight=sd.pop("embed").to(device=dev, dtype=self.dtype).contiguous())
        for i, L in enumerate(self.specs):
            p, m, w = f"l{i}.", L["mixer"], {}
            w["norm1"], w["ls1"] = self._norm_w(sd, p + "norm1"), self._f32(sd, p + "ls1")
            if L["type"] == "mlstm":
                H = int(m["heads"])
                w.update(qkvg=self._lw(torch.cat([sd.pop(p + f"mix.{n}") for n in ("q", "k", "v", "g")])),
                         gates=self._lw(torch.cat([sd.pop(p + "mix.i"), sd.pop(p + "mix.f")])),
                         gate_bias=torch.cat([self._f32(sd, p + "mix.i.b"), self._f32(sd, p + "mix.f.b")]).contiguous(),
                         gnorm=self._f32(sd, p + "mix.norm"), o=self._lw(sd.pop(p + "mix.o")))
                assert w["gate_bias"].numel() == 2 * H
            else:
                H, D, R, V, Lr = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
                wq = sd.pop(p + "mix.q").to(dev, torch.float32).view(H, D + R, -1)
                uk = sd.pop(p + "mix.uk").to(dev, torch.float32).view(H, D, Lr)
                uv = sd.pop(p + "mix.uv").to(dev, torch.float32).view(H, V, Lr)
                wo = sd.pop(p + "mix.o").to(dev, torch.float32)
                # absorbed forms, products taken in fp32 (no TF32) and rounded once to the model dtype
                q_abs = torch.cat([torch.einsum("hdl,hdw->hlw", uk, wq[:, :D]), wq[:, D:]], 1).reshape(H * (Lr + R), -1)
                o_abs = torch.einsum("whv,hvl->whl", wo.view(wo.shape[0], H, V), uv).reshape(wo.shape[0], H * Lr)
                w.update(q_abs=self._lw(q_abs), o=self._lw(o_abs))
                if m.get("kv_from") is None:
                    w.update(dkv=self._lw(sd.pop(p + "mix.dkv")), kvn=self._f32(sd, p + "mix.dkv.norm"))
                self.rope_freqs[i] = (float(m["rot"]["base"]) ** (-2.0 * torch.arange(R // 2, dtype=torch.float64) / R)).float().to(dev)
            mlp = L["mlp"]
            if mlp:
                w["norm2"], w["ls2"] = self._norm_w(sd, p + "norm2"), self._f32(sd, p + "ls2")
                if mlp.get("kind", "dense") == "dense":
                    w.update(up=self._lw(sd.pop(p + "mlp.up")), down=self._lw(sd.pop(p + "mlp.down")))
                else:
                    E = int(mlp["router"]["experts"])
                    bank = lambda n: LinearWeight(weight=torch.stack([sd.pop(p + f"mlp.e{e}.{n}") for e in range(E)]).to(device=dev, dtype=self.dtype).contiguous())
                    w.update(e_gate=bank("gate"), e_up=bank("up"), e_down=bank("down"))
                    rows = [sd.pop(p + "mlp.router")]
                    if mlp.get("shared"):
                        # the always-on expert's gate logit rides along with the router logits: one fp32 product [experts + 1, width]
                        rows.append(sd.pop(p + "mlp.shared.sg"))
                        raw = lambda n: LinearWeight(weight=sd.pop(p + "mlp.shared." + n).to(device=dev, dtype=self.dtype).contiguous())
                        w.update(s_gate=raw("gate"), s_up=raw("up"), s_down=self._lw(sd.pop(p + "mlp.shared.down")))
                    w["router"] = torch.cat(rows).to(device=dev, dtype=torch.float32).contiguous()
            self.layer_weights[i] = w
        self.norm_w = self._norm_w(sd, "final.norm")
        self.lm_head = self._lw(sd.pop("head"))
        if strict and sd:
            raise ValueError(f"unexpected checkpoint tensors: {sorted(sd)[:8]} ...")
        self.rope = RopeSpec(inv_freq=torch.zeros(1), rot_dim=0, interleaved=True)
        return self

    # ---- forward ----------------------------------------------------------------------------------------------------
    def _mm(self, x, W: LinearWeight, f32: bool = False, act: str = "none"):
        y = self.ops.linear_any(x, W, torch.float32 if f32 else self.dtype, act)
        return y if y.shape[1] == W.n_real else y[:, :W.n_real]

    def _mlstm(self, w, m, ha, meta, st):
        O, eps = self.ops, self.cfg.rms_norm_eps
        H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        u = self._mm(ha, w["qkvg"])                                                  # [q | k | v | g]
        gates = self._mm(ha, w["gates"], True)                                       # fp32 raw [i | f]
        o = O.mlstm_scan(u, gates, w["gate_bias"], st, meta, H, D, V, float(m["gate_cap"]), float(D) ** -0.5)
        on = O.gated_rmsnorm(o, u[:, 2 * H * D + H * V:], w["gnorm"], eps, H, "sigmoid_post", self.dtype)   # per-head norm, then the gate
        return self._mm(on, w["o"], True)

    def _latent(self, i, w, m, ha, meta, pool):
        O, eps = self.ops, self.cfg.rms_norm_eps
        H, R, Lr = int(m["heads"]), int(m["rot_dim"]), int(m["kv_rank"])
        T = ha.shape[0]
        fr = self.rope_freqs[i]
        if "dkv" in w:      # own down-projection: append this step's rows; a layer with kv_from reads what the named layer appended
            O.latent_kv_prologue(self._mm(ha, w["dkv"]), 0, Lr, None, w["kvn"], eps, pool, meta, fr, interleaved=True)
        q = self._mm(ha, w["q_abs"])
        if not q.is_contiguous():
            q = q.contiguous()
        window = int((m.get("mask") or {}).get("size", 0) or 0)
        attend = O.latent_attention_prefill if (meta.num_seqs == 1 and T >= self.PREFILL_GEMM_MIN_ROWS) else O.latent_attention
        o = attend(q.view(T, H, Lr + R), pool, None, meta, float(m["scale"]), Lr, fr, self.dtype, window=window, interleaved=True)
        return self._mm(o.view(T, H * Lr), w["o"], True)

    def _moe(self, w, mlp, ha):
        """Returns ``(routed sum fp32, shared expert's output fp32 or None, its gate logits or None)``."""
        O = self.ops
        E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
        z = O.router_logits(ha, w["router"])                                          # fp32 [T, E (+1)]
        idx, wts = O.sigmoid_topk(z, E, top)
        y = O.moe_clamped_experts(ha, idx, wts, w["e_gate"], w["e_up"], w["e_down"], float(mlp["expert"]["limit"]))
        if "s_gate" not in w:
            return y, None, None
        hs = O.clamped_gated_up(ha, w["s_gate"], w["s_up"], float(mlp["shared"]["limit"]))
        return y, self._mm(hs, w["s_down"], True), z[:, E]

    def layer_forward(self, i, h, ha, meta, kv, next_norm):
        """``h``: fp32 residual stream (updated in place); ``ha``: ``norm1(h)`` in the activation dtype.  Returns the next sublayer's
        normed input (``next_norm``: the weight of the norm that follows this layer)."""
        O, L, w = self.ops, self.specs[i], self.layer_weights[i]
        m, eps = L["mixer"], self.cfg.rms_norm_eps
        y = self._mlstm(w, m, ha, meta, kv.state[i]) if L["type"] == "mlstm" else self._latent(i, w, m, ha, meta, kv.k[i])
        mlp = L["mlp"]
        if not mlp:
            return O.scaled_add_norm_(h, y, w["ls1"], next_norm, eps, self.dtype)
        ha = O.scaled_add_norm_(h, y, w["ls1"], w["norm2"], eps, self.dtype)
        if mlp.get("kind", "dense") == "dense":
            y = self._mm(self._mm(ha, w["up"], act="gelu_erf"), w["down"], True)
            return O.scaled_add_norm_(h, y, w["ls2"], next_norm, eps, self.dtype)
        y, ys, zg = self._moe(w, mlp, ha)
        return O.scaled_add_norm_(h, y, w["ls2"], next_norm, eps, self.dtype, extra=ys, extra_gate=zg)

    @torch.inference_mode()
    def forward(self, x, meta: BatchMeta, kv, all_logits: bool = False, layer_out=None):
        """``x``: token ids ``[T]``.  Returns fp32 logits ``[B, V]`` (``[T, V]`` with ``all_logits``).  ``layer_out``: optional list that
        receives a copy of the residual stream after every layer."""
        O, c = self.ops, self.cfg
        if meta.state_slots is None and any(L["type"] in ("mlstm",) for L in self.specs):      # a stack of attention layers alone holds pages only
            raise ValueError("Gusolorn needs state slots in the step metadata (BatchMeta.build(..., state_slots=...))")
        tokens = x.to(torch.int64).contiguous()
        n = len(self.specs)
        h = O.gather_rows(self.embed_tokens.weight, tokens, 0, c.hidden_size, torch.float32)          # fp32 residual stream
        ha = O.rmsnorm_cast(h, self.layer_weights[0]["norm1"] if n else self.norm_w, c.rms_norm_eps, self.dtype)
        for i in range(n):
            ha = self.layer_forward(i, h, ha, meta, kv, self.layer_weights[i + 1]["norm1"] if i + 1 < n else self.norm_w)
            if layer_out is not None:
                layer_out.append(h.clone())
        if not all_logits and meta.num_tokens != meta.num_seqs:
            ha = ha.index_select(0, meta.last_idx.long())
        return self._mm(ha, self.lm_head, True).contiguous()

    __call__ = forward


Model = GusolornStage
