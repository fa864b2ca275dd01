"""Gokapel: a decoder stack on several residual streams.  Every layer has one *mixer* — a gated delta rule with one decay per head and
key channel, or grouped-query attention inside fixed blocks of positions (with a sink) running BESIDE a minGRU — and an optional
feed-forward — dense or a mixture of experts with a group-limited softmax router and an always-on expert, all with squared-ReLU units.
No reference counterpart (the reference serves Llama / Gemma-2 / DeepSeek-V2 only).

Residual structure (``S`` streams ``x_1 .. x_S``, all equal to ``embed[token] * embedding_scale`` at the start; ``m = residual_mult``;
``dyt(u) = tanh(alpha u) * w + b`` takes the place of a norm), for sublayer ``q`` (1: mixer, 2: feed-forward):

    h = dyt_q(sum_s in_q[s] x_s)        r = sublayer(h) * ls_q * sigmoid(W_rg,q h + b_rg,q)        x_t <- sum_s mix_q[s, t] x_s + m * out_q[t] * r

and the LM head (the embedding table itself) reads ``dyt_final(sum_s x_s)``.  Layer scale ``ls``, the gated residual and the stream
weights are used where the checkpoint has their tensors; without them the step is the plain pre-norm residual sum.

Mixers (``h``: the sublayer's input):

* ``channel_delta``: ``q, k`` (``kv_heads x dim``) and ``v`` (``heads x vdim``) pass a short causal convolution and SiLU; ``q, k`` become unit
  vectors per head (``q`` times ``dim^-1/2``); ``b = sigmoid(W_b h)``; ``g = exp(-exp(A_log_h) softplus(W_a2 W_a1 h + dt_bias))`` per head and
  key channel; per head ``S <- g S``, ``u = b (v - S^T k)``, ``S <- S + k u^T``, ``o = S^T q``; ``o`` per head divided by its root mean
  square, times a weight shared by the heads, times ``sigmoid(W_g2 W_g1 h)``; output projection.
* ``parallel``: ``left_scale * attention(h) + right_scale * mingru(h)``.  Attention: per-head RMS norm of queries and keys (weights shared by
  the heads), rotation of adjacent pairs of the first ``rot.dims`` entries, scores times ``scale``, keys visible only inside the query's
  own block of ``mask.size`` positions (blocks counted from position 0), ``exp(sink_h)`` added to the softmax denominator.  minGRU:
  ``z = sigmoid(W_z h + b_z)``, ``u = W_x h + b_x``, candidate ``u + 1/2`` (``u >= 0``) or ``sigmoid(u)``, ``S <- (1 - z) S + z c``,
  output ``W_o (S * silu(W_g h))``.

Precision: the streams, every ``dyt``, positions and angles, scores / softmax, the router, and everything inside the recurrences (unit
norms, decays, step sizes, gates, states) are fp32 in both dtypes; projections, short convolutions and expert activations run in the
model dtype (bf16 on the serving path) with fp32 accumulation.

Framework integration: layer order and every size come from ``ModelConfig.layer_specs``; a ``channel_delta`` layer keeps its matrix state
and the convolution's last inputs in per-sequence state slots, a ``parallel`` layer keeps keys / values in its own pair of paged pools AND
the minGRU state in a slot (``("paged_kv", ..., {state})`` in the cache layout of ``engine/kv_cache.py::HybridCache``); a layer with
``weights_of`` shares the weight dict of the named layer and owns its cache entry.  The ops are ``ops/reference.py`` (unfused PyTorch) /
``ops/b200.py`` (``ops/csrc/streams.cu``); every sublayer boundary — stream update, read for the next sublayer, ``dyt`` — is one fused op.
"""
from __future__ import annotations

import torch

from ..ops import BatchMeta, LinearWeight, RopeSpec
from .base import StageModel
from .perelorn import _pad_rows


class GokapelStage(StageModel):
    arch = "gokapel"
    PREFILL_GEMM_MIN_ROWS = 32
    UNIT_EPS = 1e-6            # inside the root of the unit vectors of the delta rule (fixed by the design)

    def __init__(self, cfg, spec=None, dtype=torch.bfloat16, device="cpu", backend=None):
        super().__init__(cfg, spec, dtype, device, backend)
        if not (self.spec.is_first and self.spec.is_last):
            raise NotImplementedError("Gokapel runs as a single stage (fp32 residual streams: the pipeline hand-off does not carry them)")
        self.specs = cfg.layer_specs
        self.seg = {}              # layer -> {segment name: (first column, width)} of its fused input projection

    # ---- cache geometry ---------------------------------------------------------------------------------------------
    def cache_layout(self):
        out = []
        for L in self.specs:
            m = L["mixer"]
            if L["type"] == "channel_delta":
                H, G, D, V, K = (int(m[k]) for k in ("heads", "kv_heads", "dim", "vdim", "conv"))
                out.append(("state", {"S": ((H, D, V), torch.float32), "conv": ((K - 1, 2 * G * D + H * V), self.dtype)}))
            else:
                a = m["left"]
                out.append(("paged_kv", int(a["kv_heads"]), int(a["dim"]), int(a["vdim"]), self.dtype,
                            {"S": ((int(m["right"]["width"]),), torch.float32)}))
        return out

    def kv_geometry(self):
        raise NotImplementedError("hybrid stack: see cache_layout()")

    # ---- weights ----------------------------------------------------------------------------------------------------
    def _lw(self, w: torch.Tensor, bias: torch.Tensor = None) -> LinearWeight:
        """Linear weight ``[out, in]`` in the model dtype; output rows zero-padded to a multiple of 8 (GEMM tile rule), the real row
        count kept in ``n_real``."""
        lw = LinearWeight(weight=_pad_rows(w.to(device=self.device, dtype=self.dtype)))
        if bias is not None:
            lw.bias = _pad_rows(bias.to(device=self.device, dtype=self.dtype)[:, None])[:, 0].contiguous()
        lw.n_real = w.shape[0]
        return lw

    def _fused(self, parts):
        """One projection for several matrices that read the same input: ``parts`` = ``[(name, weight [rows, in], bias or None)]``.  Every
        segment starts at a multiple of 8 columns (a later product may read it in place).  Returns ``(LinearWeight, {name: (col0, rows)})``."""
        ws, bs, seg, col = [], [], {}, 0
        any_bias = any(b is not None for _, _, b in parts)
        for name, w, b in parts:
            n = w.shape[0]
            pad = (-n) % 8
            seg[name] = (col, n)
            ws.append(torch.cat([w, w.new_zeros(pad, w.shape[1])]) if pad else w)
            if any_bias:
                bb = b if b is not None else w.new_zeros(n)
                bs.append(torch.cat([bb, bb.new_zeros(pad)]) if pad else bb)
            col += n + pad
        return self._lw(torch.cat(ws), torch.cat(bs) if any_bias else None), seg

    def _f32(self, sd, key) -> torch.Tensor:
        return sd.pop(key).to(device=self.device, dtype=torch.float32).contiguous()

    def _dyt(self, sd, key):
        """``(alpha, weight, bias)`` of a dynamic-tanh norm; the scalar is taken to the host once, at load."""
        return float(sd.pop(key + ".alpha").float()), self._f32(sd, key), self._f32(sd, key + ".b")

    def sanitize(self, sd):
        return dict(sd)

    def _sublayer_weights(self, sd, p, q, w):
        S, dev = int(self.cfg.streams), self.device
        w[f"norm{q}"] = self._dyt(sd, f"{p}norm{q}")
        w[f"ls{q}"] = self._f32(sd, f"{p}ls{q}") if f"{p}ls{q}" in sd else None
        if f"{p}hc{q}.in" in sd:
            w[f"in{q}"], w[f"out{q}"], w[f"mix{q}"] = self._f32(sd, f"{p}hc{q}.in"), self._f32(sd, f"{p}hc{q}.out"), self._f32(sd, f"{p}hc{q}.mix")
        else:          # no stream weights: the plain residual sum on every stream
            w[f"in{q}"] = torch.full((S,), 1.0 / S, device=dev)
            w[f"out{q}"], w[f"mix{q}"] = torch.ones(S, device=dev), torch.eye(S, device=dev)
        if w[f"in{q}"].numel() != S or tuple(w[f"mix{q}"].shape) != (S, S):
            raise ValueError(f"{p}hc{q}: stream weights do not fit streams = {S}")
        return (sd.pop(f"{p}rg{q}"), sd.pop(f"{p}rg{q}.b")) if f"{p}rg{q}" in sd else None

    def load_state(self, sd, strict: bool = True):
        sd = dict(sd)
        dev = self.device
        emb = sd.pop("embed")
        self.embed_tokens = LinearWeight(weight=emb.to(device=dev, dtype=self.dtype).contiguous())
        self.lm_head = self._lw(emb) if emb.shape[0] % 8 else self.embed_tokens
        self.lm_head.n_real = emb.shape[0]
        for i, L in enumerate(self.specs):
            if L.get("weights_of") is not None:
                continue
            p, m, w = f"l{i}.", L["mixer"], {}
            rg = self._sublayer_weights(sd, p, 1, w)
            gate_part = [("rg", rg[0], rg[1])] if rg else []
            if L["type"] == "channel_delta":
                H, G, D, V = (int(m[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
                names = ("q", "k", "v")
                qkv = [sd.pop(p + "mix." + n) for n in names]
                if [t.shape[0] for t in qkv] != [G * D, G * D, H * V] or sd[p + "mix.b"].shape[0] != H:
                    raise ValueError(f"{p}mix: projection shapes do not fit heads / kv_heads / dim / vdim")
                # q, k, v stay adjacent (one segment): the short convolution and the scan read them as one block of columns
                parts = [("qkv", torch.cat(qkv), None)] + [(n, sd.pop(p + "mix." + n), None) for n in ("b", "a1", "g1")]
                w["proj"], w["seg"] = self._fused(parts + gate_part)
                w["conv"] = torch.cat([self._f32(sd, p + f"mix.{n}.conv") for n in names]).contiguous()
                w["conv_b"] = torch.zeros(w["conv"].shape[0], device=dev)
                if w["conv"].shape[1] != int(m["conv"]):
                    raise ValueError(f"{p}mix: convolution taps do not fit the configuration")
                w["a2"], w["g2"] = self._lw(sd.pop(p + "mix.a2")), self._lw(sd.pop(p + "mix.g2"))
                w["dt_bias"], w["A_log"] = self._f32(sd, p + "mix.dt_bias"), self._f32(sd, p + "mix.A_log")
                w["gnorm"] = self._f32(sd, p + "mix.norm").repeat(H).contiguous()            # one weight vector for all heads
                w["o"] = self._lw(sd.pop(p + "mix.o"))
            else:
                a, r = m["left"], m["right"]
                H, G, D, V, R = int(a["heads"]), int(a["kv_heads"]), int(a["dim"]), int(a["vdim"]), int(r["width"])
                parts = [(n, sd.pop(p + "mix.left." + n), None) for n in ("q", "k", "v")]
                parts += [("z", sd.pop(p + "mix.right.z"), sd.pop(p + "mix.right.z.b")), ("x", sd.pop(p + "mix.right.x"), sd.pop(p + "mix.right.x.b")),
                          ("g", sd.pop(p + "mix.right.g"), None)]
                w["proj"], w["seg"] = self._fused(parts + gate_part)
                w["qn"], w["kn"] = self._f32(sd, p + "mix.left.q.norm"), self._f32(sd, p + "mix.left.k.norm")
                w["sink"] = self._f32(sd, p + "mix.left.sink") if p + "mix.left.sink" in sd else None
                rd = int((a.get("rot") or {}).get("dims", 0) or 0)
                base = float((a.get("rot") or {}).get("base", 10000.0))
                w["inv_freq"] = (base ** (-2.0 * torch.arange(rd // 2, dtype=torch.float64) / max(rd, 1))).float().to(dev)
                # both output projections as ONE product over [attention output | minGRU output] (each scaled by its branch factor where
                # it is written); the attention part is padded to a multiple of 8 columns
                wl, wr = sd.pop(p + "mix.left.o"), sd.pop(p + "mix.right.o")
                pad = (-wl.shape[1]) % 8
                w["o_split"] = wl.shape[1] + pad
                w["o"] = self._lw(torch.cat([wl, wl.new_zeros(wl.shape[0], pad), wr], 1))
            mlp = L["mlp"]
            if mlp:
                rg2 = self._sublayer_weights(sd, p, 2, w)
                w["rg2"] = self._lw(rg2[0], rg2[1]) if rg2 else None
                if mlp.get("kind", "dense") == "dense":
                    w.update(up=self._lw(sd.pop(p + "mlp.up")), down=self._lw(sd.pop(p + "mlp.down")))
                else:
                    E = int(mlp["router"]["experts"])
                    bank = lambda n: LinearWeight(weight=torch.stack([sd.pop(p + f"mlp.e{e}.{n}") for e in range(E)]).to(device=dev, dtype=self.dtype).contiguous())
                    w.update(e_up=bank("up"), e_down=bank("down"), router=self._f32(sd, p + "mlp.router"))
                    w["correction"] = self._f32(sd, p + "mlp.correction") if p + "mlp.correction" in sd else None
                    if mlp.get("shared"):
                        w.update(s_up=self._lw(sd.pop(p + "mlp.shared.up")), s_down=self._lw(sd.pop(p + "mlp.shared.down")))
            self.layer_weights[i] = w
        for i, L in enumerate(self.specs):
            if L.get("weights_of") is not None:
                self.layer_weights[i] = self.layer_weights[int(L["weights_of"])]
        self.final_norm = self._dyt(sd, "final.norm")
        self.norm_w = self.final_norm[1]
        self.sum_in = torch.ones(int(self.cfg.streams), device=dev)
        if strict and sd:
            raise ValueError(f"unexpected checkpoint tensors: {sorted(sd)[:8]} ...")
        self.rope = RopeSpec(inv_freq=torch.zeros(1), rot_dim=0, interleaved=True)
        return self

    # ---- forward ----------------------------------------------------------------------------------------------------
    def _mm(self, x, W: LinearWeight, f32: bool = False, act: str = "none"):
        y = self.ops.linear_any(x, W, torch.float32 if f32 else self.dtype, act)
        return y if y.shape[1] == W.n_real else y[:, :W.n_real]

    @staticmethod
    def _cols(u, seg, name):
        c0, n = seg[name]
        return u[:, c0:c0 + n]

    def _channel_delta(self, w, m, ha, meta, st):
        """Returns ``(mixer output fp32 [T, width], gate logits of the gated residual or None)``."""
        O, eps, seg = self.ops, self.cfg.rms_norm_eps, w["seg"]
        H, G, D, V = (int(m[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
        u = self.ops.linear_any(ha, w["proj"], self.dtype)                            # [q k v | b | a1 | g1 | rg]
        C = 2 * G * D + H * V                                                        # q, k, v are adjacent: one convolution over all
        qkv = O.causal_conv_silu(u[:, :C], w["conv"], w["conv_b"], st["conv"], meta)
        dt = self._mm(self._cols(u, seg, "a1"), w["a2"], True)                        # fp32 raw step sizes [T, H * D]
        gate = self._mm(self._cols(u, seg, "g1"), w["g2"])
        o = O.delta_scan(qkv, self._cols(u, seg, "b"), dt, w["dt_bias"], w["A_log"], st["S"], meta, H, G, D, V, float(D) ** -0.5, self.UNIT_EPS)
        on = O.gated_rmsnorm(o, gate, w["gnorm"], eps, H, "sigmoid_post", self.dtype)
        return self._mm(on, w["o"], True), (self._cols(u, seg, "rg") if "rg" in seg else None)

    def _parallel(self, w, m, ha, meta, kpool, vpool, st):
        O, eps, seg = self.ops, self.cfg.rms_norm_eps, w["seg"]
        a = m["left"]
        H, D, V, R = int(a["heads"]), int(a["dim"]), int(a["vdim"]), int(m["right"]["width"])
        T = ha.shape[0]
        u = self.ops.linear_any(ha, w["proj"], self.dtype)                            # [q | k | v | z | x | g | rg], biases added
        q = O.qk_norm_rope_append(u, seg["q"][0], seg["k"][0], seg["v"][0], H, D, w["qn"], w["kn"], eps, w["inv_freq"], kpool, vpool, meta)
        both = torch.zeros(T, w["o_split"] + R, dtype=self.dtype, device=u.device) if w["o_split"] != H * V else \
            torch.empty(T, H * V + R, dtype=self.dtype, device=u.device)
        attend = O.sink_attention_prefill if (meta.num_seqs == 1 and T >= self.PREFILL_GEMM_MIN_ROWS) else O.sink_attention
        attend(q, kpool, vpool, w["sink"], meta, float(a["scale"]), int((a.get("mask") or {}).get("size", 0) or 0), 0,
                         float(m.get("left_scale", 1.0)), self.dtype, both, 0)
        O.mingru_scan(u, seg["z"][0], seg["x"][0], seg["g"][0], R, st["S"], meta, float(m.get("right_scale", 1.0)), self.dtype, both, w["o_split"])
        return self._mm(both, w["o"], True), (self._cols(u, seg, "rg") if "rg" in seg else None)

    def _ff(self, w, mlp, ha):
        """Returns ``(output fp32, second branch fp32 or None, gate logits or None)``."""
        O = self.ops
        gate = self._mm(ha, w["rg2"]) if w.get("rg2") is not None else None
        if mlp.get("kind", "dense") == "dense":
            return self._mm(self._mm(ha, w["up"], act="relu2"), w["down"], True), None, gate
        r = mlp["router"]
        gr = r.get("groups") or {}
        ng = int(gr.get("count", 1))
        idx, wts = O.group_softmax_topk(O.router_logits(ha, w["router"]), w["correction"], int(r["experts"]), int(r["top"]), ng, int(gr.get("keep", ng)))
        y = O.moe_relu2_experts(ha, idx, wts, w["e_up"], w["e_down"])
        ys = self._mm(self._mm(ha, w["s_up"], act="relu2"), w["s_down"], True) if "s_up" in w else None
        return y, ys, gate

    def layer_forward(self, i, xs, ha, meta, kv, nxt):
        """``xs``: fp32 residual streams ``[T, S, width]`` (updated in place); ``ha``: this layer's mixer input in the activation dtype.
        Returns the next sublayer's input (``nxt`` = ``(in weights, alpha, w, b)`` of the read that follows this layer)."""
        O, L, w = self.ops, self.specs[i], self.layer_weights[i]
        mult = float(self.cfg.residual_mult)
        if L["type"] == "channel_delta":
            y, gate = self._channel_delta(w, L["mixer"], ha, meta, kv.state[i])
        else:
            y, gate = self._parallel(w, L["mixer"], ha, meta, kv.k[i], kv.v[i], kv.state[i])
        mlp = L["mlp"]
        if not mlp:
            return O.hyper_step_(xs, y, None, gate, w["ls1"], w["mix1"], w["out1"], mult, *nxt, self.dtype)
        ha = O.hyper_step_(xs, y, None, gate, w["ls1"], w["mix1"], w["out1"], mult, w["in2"], *w["norm2"], self.dtype)
        y, y2, gate = self._ff(w, mlp, ha)
        return O.hyper_step_(xs, y, y2, gate, w["ls2"], w["mix2"], w["out2"], mult, *nxt, self.dtype)

    @torch.inference_mode()
    def forward(self, x, meta: BatchMeta, kv, all_logits: bool = False, layer_out=None):
        """``x``: token ids ``[T]``.  Returns fp32 logits ``[B, V]`` (``[T, V]`` with ``all_logits``).  ``layer_out``: optional list that
        receives the sum of the residual streams after every layer."""
        O, c = self.ops, self.cfg
        if meta.state_slots is None:
            raise ValueError("Gokapel needs state slots in the step metadata (BatchMeta.build(..., state_slots=...))")
        tokens = x.to(torch.int64).contiguous()
        n = len(self.specs)
        xs = O.stream_embed(self.embed_tokens.weight, tokens, float(c.embedding_scale), int(c.streams))     # fp32 [T, S, width]
        read = lambda j: (self.layer_weights[j]["in1"], *self.layer_weights[j]["norm1"]) if j < n else (self.sum_in, *self.final_norm)
        ha = O.hyper_step_(xs, None, None, None, None, None, None, 0.0, *read(0), self.dtype)
        for i in range(n):
            ha = self.layer_forward(i, xs, ha, meta, kv, read(i + 1))
            if layer_out is not None:
                layer_out.append(xs.sum(1))
        if not all_logits and meta.num_tokens != meta.num_seqs:
            ha = ha.index_select(0, meta.last_idx.long())
        return self._mm(ha, self.lm_head, True).contiguous()

    __call__ = forward


Model = GokapelStage
