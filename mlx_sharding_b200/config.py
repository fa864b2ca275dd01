"""Model configuration + layer-range shard specification.

Parity notes (reference = /root/reference/shard):

* The reference extends each upstream ``ModelArgs`` with ``start_layer`` / ``end_layer`` fields
  (server/model/llama.py:11-14, gemma2.py:9-12, deepseek_v2.py:11-14) whose *defaults are hard-wired*
  to 32 / 46 / 27.  We default ``end_layer`` to ``num_hidden_layers`` and accept either
  bound on its own (the reference only injects them when both are given, utils.py:37-39).
* ``model_type`` remapping ``mistral -> llama`` follows utils.py:14-17.  ``phi-msft -> phixtral`` in the
  reference points at a module that does not exist; we raise a clear error instead.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, Dict, Optional

MODEL_REMAPPING = {
    "mistral": "llama",  # reference utils.py:15
}

SUPPORTED_ARCHS = ("llama", "gemma2", "deepseek_v2", "perelorn", "gusolorn", "gifetar", "gokapel")


@dataclass(frozen=True)
class ShardSpec:
    """A pipeline stage = the contiguous layer range ``start_layer <= i < end_layer``.

    Placement rules (reference llama.py:26-36,74-77; gemma2.py:23-24; deepseek_v2.py:23-35):
    embedding on the first stage, final norm + LM head on the last stage; when the head is tied to the
    embedding the last stage also holds ``embed_tokens`` (the reference does this only for Gemma-2 and
    would crash for tied Llama — fixed here).
    """

    start_layer: int
    end_layer: int
    num_layers: int
    # Half-layer boundaries (no reference counterpart; used by ``parallel.partition.balanced_split(half_layers=True)``).
    # A decoder layer is two residual blocks (attention, MLP) that only exchange the residual stream ``h``, so a
    # stage boundary may also fall *between* them: ``skip_first_attn`` = the attention block of ``start_layer`` ran
    # on the previous stage; ``defer_last_mlp`` = the MLP block of ``end_layer - 1`` runs on the next stage.
    skip_first_attn: bool = False
    defer_last_mlp: bool = False

    def __post_init__(self):
        if not (0 <= self.start_layer < self.end_layer <= self.num_layers):
            raise ValueError(
                f"invalid layer range [{self.start_layer}, {self.end_layer}) for {self.num_layers} layers"
            )
        if self.skip_first_attn and self.defer_last_mlp and self.num_local_layers == 1:
            raise ValueError("empty stage: both blocks of its only layer live elsewhere")

    @property
    def is_first(self) -> bool:
        return self.start_layer == 0 and not self.skip_first_attn

    @property
    def is_last(self) -> bool:
        return self.end_layer == self.num_layers and not self.defer_last_mlp

    @property
    def num_local_layers(self) -> int:
        return self.end_layer - self.start_layer

    def owns_layer(self, i: int) -> bool:
        return self.start_layer <= i < self.end_layer

    def layers(self):
        return range(self.start_layer, self.end_layer)

    def runs_attn(self, i: int) -> bool:
        return self.owns_layer(i) and not (self.skip_first_attn and i == self.start_layer)

    def runs_mlp(self, i: int) -> bool:
        return self.owns_layer(i) and not (self.defer_last_mlp and i == self.end_layer - 1)

    def attn_layers(self):
        """Layers whose attention block (and therefore KV cache) lives on this stage."""
        return [i for i in self.layers() if self.runs_attn(i)]

    @property
    def num_kv_layers(self) -> int:
        return len(self.attn_layers())

    def describe(self) -> str:
        a = f"{self.start_layer}{'.5' if self.skip_first_attn else ''}"
        b = f"{self.end_layer - 1}.5" if self.defer_last_mlp else f"{self.end_layer}"
        return f"[{a}, {b})"

    @staticmethod
    def even_split(num_layers: int, num_stages: int):
        """Balanced contiguous split, e.g. 27 layers / 2 stages -> [0,14), [14,27)."""
        base, rem = divmod(num_layers, num_stages)
        out, s = [], 0
        for r in range(num_stages):
            n = base + (1 if r < rem else 0)
            out.append(ShardSpec(s, s + n, num_layers))
            s += n
        return out


@dataclass
class ModelConfig:
    """Architecture hyper-parameters parsed from an mlx-community / HF ``config.json``.

    Unknown keys are kept in ``extra`` (the upstream ``ModelArgs.from_dict`` silently drops them).
    """

    model_type: str = "llama"
    hidden_size: int = 4096
    num_hidden_layers: int = 32
    intermediate_size: int = 14336
    num_attention_heads: int = 32
    num_key_value_heads: Optional[int] = None
    head_dim: Optional[int] = None
    rms_norm_eps: float = 1e-5
    vocab_size: int = 32000
    rope_theta: float = 10000.0
    rope_traditional: bool = False
    rope_scaling: Optional[Dict[str, Any]] = None
    max_position_embeddings: int = 8192
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    mlp_bias: bool = False
    # gemma2
    query_pre_attn_scalar: Optional[float] = None
    attn_logit_softcapping: Optional[float] = None
    final_logit_softcapping: Optional[float] = None
    # deepseek_v2
    moe_intermediate_size: Optional[int] = None
    n_shared_experts: Optional[int] = None
    n_routed_experts: Optional[int] = None
    routed_scaling_factor: float = 1.0
    kv_lora_rank: Optional[int] = None
    q_lora_rank: Optional[int] = None
    qk_rope_head_dim: Optional[int] = None
    v_head_dim: Optional[int] = None
    qk_nope_head_dim: Optional[int] = None
    topk_method: str = "greedy"
    n_group: Optional[int] = None
    topk_group: Optional[int] = None
    num_experts_per_tok: Optional[int] = None
    moe_layer_freq: int = 1
    first_k_dense_replace: int = 0
    norm_topk_prob: bool = False
    # perelorn (hybrid stack: per-layer mixer / feed-forward specs, per-layer token input, logit scale)
    layer_specs: Optional[list] = None
    token_side_dim: int = 0
    logit_scale: float = 1.0
    # gifetar: every sublayer's (normed) output enters the residual stream times this factor
    residual_mult: float = 1.0
    # gokapel: number of residual streams (hyper-connections) and the factor on the embedding rows
    streams: int = 1
    embedding_scale: float = 1.0
    # quantisation (mlx affine) + sharding
    quantization: Optional[Dict[str, int]] = None
    start_layer: Optional[int] = None
    end_layer: Optional[int] = None
    extra: Dict[str, Any] = field(default_factory=dict)

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
        d = dict(d)
        if "model_type" not in d and str(d.get("architecture", "")).lower() == "perelorn":
            d = _perelorn_flat(d)
        elif "model_type" not in d and str(d.get("architecture", "")).lower() == "gusolorn":
            d = _gusolorn_flat(d)
        elif "model_type" not in d and str(d.get("architecture", "")).lower() == "gifetar":
            d = _gifetar_flat(d)
        elif "model_type" not in d and str(d.get("architecture", "")).lower() == "gokapel":
            d = _gokapel_flat(d)
        mt = d.get("model_type", "llama")
        if mt == "phi-msft":
            raise ValueError(
                "model_type 'phi-msft' is remapped to a non-existent 'phixtral' module by the reference "
                "(shard/utils.py:16); it is not supported"
            )
        d["model_type"] = MODEL_REMAPPING.get(mt, mt)
        if d["model_type"] not in SUPPORTED_ARCHS:
            raise ValueError(f"Model type {mt} not supported (supported: {SUPPORTED_ARCHS})")
        known = {f for f in cls.__dataclass_fields__ if f != "extra"}
        kw = {k: v for k, v in d.items() if k in known}
        extra = {k: v for k, v in d.items() if k not in known}
        # HF >=4.45 nests rope params
        rp = extra.get("rope_parameters")
        if isinstance(rp, dict):
            kw.setdefault("rope_theta", rp.get("rope_theta", 10000.0))
            if rp.get("rope_type", "default") != "default" and "rope_scaling" not in kw:
                kw["rope_scaling"] = rp
        cfg = cls(**kw, extra=extra)
        cfg._finalize()
        return cfg

    @classmethod
    def from_path(cls, path: str) -> "ModelConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def _finalize(self):
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        if self.model_type == "gemma2":
            if self.head_dim is None:
                self.head_dim = 256
            if self.query_pre_attn_scalar is None:
                self.query_pre_attn_scalar = float(self.head_dim)
            if self.attn_logit_softcapping is None:
                self.attn_logit_softcapping = 50.0
            if self.final_logit_softcapping is None:
                self.final_logit_softcapping = 30.0
            # Gemma-2 always ties the LM head to the embedding (reference gemma2.py:80-81)
            self.tie_word_embeddings = True
        elif self.model_type == "deepseek_v2":
            self.rope_traditional = True  # interleaved pairs
        if self.head_dim is None and self.model_type != "deepseek_v2":
            self.head_dim = self.hidden_size // self.num_attention_heads

    def to_dict(self) -> Dict[str, Any]:
        d = {k: getattr(self, k) for k in self.__dataclass_fields__ if k != "extra"}
        d = {k: v for k, v in d.items() if v is not None}
        d.update(self.extra)
        return d

    # ------------------------------------------------------------------ derived
    def shard(self, start_layer: Optional[int] = None, end_layer: Optional[int] = None) -> ShardSpec:
        s = start_layer if start_layer is not None else (self.start_layer if self.start_layer is not None else 0)
        e = end_layer if end_layer is not None else (
            self.end_layer if self.end_layer is not None else self.num_hidden_layers
        )
        return ShardSpec(int(s), int(e), self.num_hidden_layers)

    @property
    def qk_head_dim(self) -> int:
        if self.model_type == "deepseek_v2":
            return self.qk_nope_head_dim + self.qk_rope_head_dim
        return self.head_dim

    @property
    def v_dim(self) -> int:
        if self.model_type == "deepseek_v2":
            return self.v_head_dim
        return self.head_dim

    @property
    def kv_heads(self) -> int:
        # the reference caches *decompressed* per-head K/V for MLA (deepseek_v2.py:120-129)
        if self.model_type == "deepseek_v2":
            return self.num_attention_heads
        return self.num_key_value_heads

    @property
    def attn_scale(self) -> float:
        if self.model_type == "gemma2":
            return float(self.query_pre_attn_scalar) ** -0.5
        if self.model_type == "deepseek_v2":
            scale = self.qk_head_dim ** -0.5
            rs = self.rope_scaling
            if rs is not None:
                mad = rs.get("mscale_all_dim", 0)
                if mad:
                    m = yarn_get_mscale(rs["factor"], mad)
                    scale = scale * m * m
            return scale
        return self.head_dim ** -0.5

    def is_moe_layer(self, i: int) -> bool:
        return (
            self.model_type == "deepseek_v2"
            and self.n_routed_experts is not None
            and i >= self.first_k_dense_replace
            and i % self.moe_layer_freq == 0
        )


def _perelorn_flat(d: Dict[str, Any]) -> Dict[str, Any]:
    """Perelorn's nested config.json (``layers`` = list of {type, mixer, mlp}; ``norm.eps``; ``token_side.dim``; ``vocab``;
    ``width``; ``logit_scale``) -> the flat fields of :class:`ModelConfig`.  Every size is read from the file."""
    layers = [dict(type=str(L["type"]), mixer=dict(L["mixer"]), mlp=(dict(L["mlp"]) if L.get("mlp") else None)) for L in d["layers"]]
    for L in layers:
        if L["type"] not in ("mamba2", "latent_attention", "lightning"):
            raise ValueError(f"Perelorn: unknown mixer type '{L['type']}'")
        if L["mlp"] is not None and L["mlp"].get("kind", "dense") != "dense":
            raise ValueError(f"Perelorn: unknown feed-forward kind '{L['mlp'].get('kind')}'")
    side = d.get("token_side") or {}
    out = {k: v for k, v in d.items() if k not in ("architecture", "layers", "norm", "token_side", "vocab", "width", "logit_scale")}
    ff = [L["mlp"]["ff"] for L in layers if L["mlp"]]
    out.update(model_type="perelorn", hidden_size=int(d["width"]), vocab_size=int(d["vocab"]), num_hidden_layers=len(layers),
               rms_norm_eps=float(d["norm"]["eps"]), layer_specs=layers, token_side_dim=int(side.get("dim", 0)),
               logit_scale=float(d.get("logit_scale", 1.0)), intermediate_size=int(max(ff)) if ff else 0,
               num_attention_heads=int(max(L["mixer"]["heads"] for L in layers)))
    return out


def perelorn_config(width=2048, vocab=32000, blocks=4, heads=16, ff=8192, side_dim=64, **overrides) -> Dict[str, Any]:
    """A Perelorn config.json with layer sizes that resemble a real model: ``blocks`` x (mamba2, latent attention + feed-forward,
    mamba2, lightning)."""
    mamba = dict(type="mamba2", mixer=dict(conv=4, groups=1, heads=2 * width // 64, norm_groups=1, state=128, vdim=64), mlp=None)
    attn = dict(type="latent_attention", mixer=dict(dim=128, heads=heads, kv_rank=512, q_rank=1536, rot=dict(base=10000.0, dims=64),
                                                    rot_dim=64, scale=192 ** -0.5, vdim=128), mlp=dict(ff=ff, kind="dense"))
    light = dict(type="lightning", mixer=dict(decay=[1.0 - 2.0 ** -(3 + 5 * h / max(1, heads - 1)) for h in range(heads)], dim=128,
                                              heads=heads, vdim=128), mlp=None)
    d = dict(architecture="Perelorn", layers=[mamba, attn, mamba, light] * blocks, logit_scale=1.0, norm=dict(eps=1e-5),
             token_side=dict(dim=side_dim), vocab=vocab, width=width)
    d.update(overrides)
    return d


def _gusolorn_flat(d: Dict[str, Any]) -> Dict[str, Any]:
    """Gusolorn's nested config.json (``layers`` = list of {type, mixer, mlp}; ``norm.eps``; ``vocab``; ``width``) -> the flat fields of
    :class:`ModelConfig`.  Mixers: ``mlstm`` (heads, dim, vdim, gate_cap) and ``latent_attention`` (heads, dim, rot_dim, vdim, kv_rank,
    scale, rot.{base,dims}, optional mask.size = sliding window, optional kv_from = layer whose cached rows it reads).  Feed-forwards:
    ``dense`` (ff) or ``moe`` (router.{experts,top}, expert.{ff,limit}, optional shared.{ff,limit}).  Every size is read from the file."""
    layers = [dict(type=str(L["type"]), mixer=dict(L["mixer"]), mlp=(dict(L["mlp"]) if L.get("mlp") else None)) for L in d["layers"]]
    for i, L in enumerate(layers):
        m = L["mixer"]
        if L["type"] not in ("mlstm", "latent_attention"):
            raise ValueError(f"Gusolorn: unknown mixer type '{L['type']}'")
        if L["mlp"] is not None and L["mlp"].get("kind", "dense") not in ("dense", "moe"):
            raise ValueError(f"Gusolorn: unknown feed-forward kind '{L['mlp'].get('kind')}'")
        if L["type"] == "latent_attention":
            if int(m["rot"]["dims"]) != int(m["rot_dim"]):
                raise ValueError("Gusolorn latent attention: rot.dims must equal rot_dim")
            src = m.get("kv_from")
            if src is not None:
                s = layers[int(src)] if 0 <= int(src) < i else None
                if s is None or s["type"] != "latent_attention" or s["mixer"].get("kv_from") is not None:
                    raise ValueError(f"Gusolorn layer {i}: kv_from must name an earlier latent-attention layer with its own down-projection")
                sm = s["mixer"]
                if (int(sm["kv_rank"]), int(sm["rot_dim"]), float(sm["rot"]["base"])) != (int(m["kv_rank"]), int(m["rot_dim"]), float(m["rot"]["base"])):
                    raise ValueError(f"Gusolorn layer {i}: kv_from layer has another latent width or rotation")
    out = {k: v for k, v in d.items() if k not in ("architecture", "layers", "norm", "vocab", "width")}
    ff = [L["mlp"]["ff"] if L["mlp"].get("kind", "dense") == "dense" else L["mlp"]["expert"]["ff"] for L in layers if L["mlp"]]
    out.update(model_type="gusolorn", hidden_size=int(d["width"]), vocab_size=int(d["vocab"]), num_hidden_layers=len(layers),
               rms_norm_eps=float(d["norm"]["eps"]), layer_specs=layers, intermediate_size=int(max(ff)) if ff else 0,
               num_attention_heads=int(max(L["mixer"]["heads"] for L in layers)))
    return out


def gusolorn_config(width=2048, vocab=32000, blocks=2, heads=16, ff=8192, experts=16, top=2, expert_ff=1024, window=1024, **overrides) -> Dict[str, Any]:
    """A Gusolorn config.json with layer sizes that resemble a real model: ``blocks`` x (latent attention + dense feed-forward, mLSTM
    + mixture of experts, mLSTM + mixture of experts, latent attention reading the first layer's rows + mixture of experts)."""
    att = dict(dim=128, heads=heads, kv_rank=512, rot=dict(base=10000.0, dims=64), rot_dim=64, scale=192 ** -0.5, vdim=128, mask=dict(size=window))
    moe = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=expert_ff, limit=7.0), shared=dict(ff=expert_ff, limit=7.0))
    ml = dict(type="mlstm", mixer=dict(dim=128, heads=heads, vdim=128, gate_cap=15.0), mlp=moe)
    layers = []
    for b in range(blocks):
        layers += [dict(type="latent_attention", mixer=dict(att), mlp=dict(ff=ff, kind="dense")), ml, ml,
                   dict(type="latent_attention", mixer=dict(att, kv_from=4 * b), mlp=moe)]
    d = dict(architecture="Gusolorn", layers=layers, norm=dict(eps=1e-5), vocab=vocab, width=width)
    d.update(overrides)
    return d


def _gifetar_flat(d: Dict[str, Any]) -> Dict[str, Any]:
    """Gifetar's nested config.json (``layers`` = list of {type, mixer, mlp}; ``norm.eps``; ``residual_mult``; ``vocab``; ``width``) -> the
    flat fields of :class:`ModelConfig`.  Mixer ``attention``: differential attention (heads, kv_heads, dim, vdim, scale, softcap, diff,
    q_temp.{coef, every}).  Feed-forward: ``moe`` (router.{experts, top}, expert.ff) or none.  Every size is read from the file."""
    layers = [dict(type=str(L["type"]), mixer=dict(L["mixer"]), mlp=(dict(L["mlp"]) if L.get("mlp") else None)) for L in d["layers"]]
    for i, L in enumerate(layers):
        m = L["mixer"]
        if L["type"] != "attention":
            raise ValueError(f"Gifetar: unknown mixer type '{L['type']}'")
        if L["mlp"] is not None and L["mlp"].get("kind") != "moe":
            raise ValueError(f"Gifetar: unknown feed-forward kind '{L['mlp'].get('kind')}'")
        if int(m["heads"]) % int(m["kv_heads"]) != 0:
            raise ValueError(f"Gifetar layer {i}: heads must be a multiple of kv_heads")
        if L["mlp"] is not None and not (1 <= int(L["mlp"]["router"]["top"]) <= int(L["mlp"]["router"]["experts"])):
            raise ValueError(f"Gifetar layer {i}: router.top must lie in 1 .. router.experts")
    out = {k: v for k, v in d.items() if k not in ("architecture", "layers", "norm", "vocab", "width", "residual_mult")}
    ff = [L["mlp"]["expert"]["ff"] for L in layers if L["mlp"]]
    out.update(model_type="gifetar", hidden_size=int(d["width"]), vocab_size=int(d["vocab"]), num_hidden_layers=len(layers),
               rms_norm_eps=float(d["norm"]["eps"]), layer_specs=layers, intermediate_size=int(max(ff)) if ff else 0,
               residual_mult=float(d.get("residual_mult", 1.0)), tie_word_embeddings=True,
               num_attention_heads=int(max(L["mixer"]["heads"] for L in layers)))
    return out


def gifetar_config(width=2048, vocab=32000, layers=8, heads=16, kv_heads=4, dim=64, vdim=128, experts=16, top=2, expert_ff=1024,
                   **overrides) -> Dict[str, Any]:
    """A Gifetar config.json with layer sizes that resemble a real model: ``layers`` x (differential attention + mixture of experts)."""
    att = dict(diff=0.8, dim=dim, heads=heads, kv_heads=kv_heads, q_temp=dict(coef=0.1, every=1024), scale=dim ** -0.5, softcap=30.0, vdim=vdim)
    moe = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=expert_ff))
    d = dict(architecture="Gifetar", layers=[dict(type="attention", mixer=dict(att), mlp=dict(moe)) for _ in range(layers)],
             norm=dict(eps=1e-5), residual_mult=0.7, vocab=vocab, width=width)
    d.update(overrides)
    return d


def _gokapel_flat(d: Dict[str, Any]) -> Dict[str, Any]:
    """Gokapel's nested config.json (``layers`` = list of {type, mixer, mlp[, weights_of]}; ``norm.eps``; ``residual_mult``; ``streams``;
    ``embedding.scale``; ``vocab``; ``width``) -> the flat fields of :class:`ModelConfig`.  Mixers: ``channel_delta`` (heads, kv_heads, dim,
    vdim, conv) and ``parallel`` (left = attention: heads, kv_heads, dim, vdim, scale, optional rot.{base, dims}, optional mask.size;
    right = minGRU: width; left_scale, right_scale).  Feed-forwards: ``dense`` (ff), ``moe`` (router.{experts, top, groups.{count, keep}},
    expert.ff, optional shared.ff) or none.  ``weights_of: j`` = the layer runs with layer ``j``'s tensors and a cache of its own.  Every
    size is read from the file."""
    layers = []
    for L in d["layers"]:
        ent = dict(type=str(L["type"]), mixer=dict(L["mixer"]), mlp=(dict(L["mlp"]) if L.get("mlp") else None))
        if L.get("weights_of") is not None:
            ent["weights_of"] = int(L["weights_of"])
        layers.append(ent)
    for i, L in enumerate(layers):
        m = L["mixer"]
        if L["type"] not in ("channel_delta", "parallel"):
            raise ValueError(f"Gokapel: unknown mixer type '{L['type']}'")
        if L["mlp"] is not None and L["mlp"].get("kind", "dense") not in ("dense", "moe"):
            raise ValueError(f"Gokapel: unknown feed-forward kind '{L['mlp'].get('kind')}'")
        att = m if L["type"] == "channel_delta" else m["left"]
        if int(att["heads"]) % int(att["kv_heads"]) != 0:
            raise ValueError(f"Gokapel layer {i}: heads must be a multiple of kv_heads")
        if L["type"] == "parallel" and int((att.get("rot") or {}).get("dims", 0)) % 2 != 0 or \
                L["type"] == "parallel" and int((att.get("rot") or {}).get("dims", 0)) > int(att["dim"]):
            raise ValueError(f"Gokapel layer {i}: rot.dims must be even and at most dim")
        if L["mlp"] is not None and L["mlp"].get("kind", "dense") == "moe":
            r = L["mlp"]["router"]
            ng = int((r.get("groups") or {}).get("count", 1))
            keep = int((r.get("groups") or {}).get("keep", ng))
            if int(r["experts"]) % ng != 0 or not (1 <= keep <= ng):
                raise ValueError(f"Gokapel layer {i}: router.groups must split the experts evenly, 1 <= keep <= count")
            if not (1 <= int(r["top"]) <= keep * (int(r["experts"]) // ng)):
                raise ValueError(f"Gokapel layer {i}: router.top must lie in 1 .. experts of the kept groups")
        j = L.get("weights_of")
        if j is not None:
            src = layers[j] if 0 <= j < len(layers) and j != i else None
            if src is None or "weights_of" in src or (src["type"], src["mixer"], src["mlp"]) != (L["type"], L["mixer"], L["mlp"]):
                raise ValueError(f"Gokapel layer {i}: weights_of must name another layer of the same shape that owns its tensors")
    out = {k: v for k, v in d.items() if k not in ("architecture", "layers", "norm", "vocab", "width", "residual_mult", "streams", "embedding")}
    ff = [L["mlp"]["ff"] if L["mlp"].get("kind", "dense") == "dense" else L["mlp"]["expert"]["ff"] for L in layers if L["mlp"]]
    heads = [int((L["mixer"] if L["type"] == "channel_delta" else L["mixer"]["left"])["heads"]) for L in layers]
    out.update(model_type="gokapel", hidden_size=int(d["width"]), vocab_size=int(d["vocab"]), num_hidden_layers=len(layers),
               rms_norm_eps=float(d["norm"]["eps"]), layer_specs=layers, intermediate_size=int(max(ff)) if ff else 0,
               residual_mult=float(d.get("residual_mult", 1.0)), streams=int(d.get("streams", 1)),
               embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)), tie_word_embeddings=True,
               num_attention_heads=max(heads) if heads else 1)
    if out["streams"] < 1 or out["streams"] > 8:
        raise ValueError("Gokapel: streams must lie in 1 .. 8")
    return out


def gokapel_config(width=2048, vocab=32000, blocks=2, heads=16, kv_heads=4, dim=128, vdim=128, ff=8192, experts=16, top=2, expert_ff=1024,
                   block_size=1024, gru_width=None, streams=2, **overrides) -> Dict[str, Any]:
    """A Gokapel config.json with layer sizes that resemble a real model: ``blocks`` x (gated delta rule + dense feed-forward, gated delta
    rule + mixture of experts, attention beside minGRU + dense feed-forward, attention beside minGRU + mixture of experts)."""
    delta = dict(conv=4, dim=dim, heads=heads, kv_heads=heads, vdim=vdim)
    par = dict(left=dict(dim=dim, heads=heads, kv_heads=kv_heads, mask=dict(size=block_size), rot=dict(base=10000.0, dims=dim // 2),
                         scale=dim ** -0.5, vdim=vdim), left_scale=0.6, right=dict(width=gru_width or width), right_scale=0.5)
    moe = dict(kind="moe", router=dict(experts=experts, top=top, groups=dict(count=4, keep=2)), expert=dict(ff=expert_ff), shared=dict(ff=expert_ff))
    dense = dict(kind="dense", ff=ff)
    layers = []
    for _ in range(blocks):
        layers += [dict(type="channel_delta", mixer=dict(delta), mlp=dict(dense)), dict(type="channel_delta", mixer=dict(delta), mlp=dict(moe)),
                   dict(type="parallel", mixer=dict(par), mlp=dict(dense)), dict(type="parallel", mixer=dict(par), mlp=dict(moe))]
    d = dict(architecture="Gokapel", embedding=dict(scale=1.0), layers=layers, norm=dict(eps=1e-6), residual_mult=0.5, streams=streams,
             vocab=vocab, width=width)
    d.update(overrides)
    return d


def yarn_get_mscale(scale: float = 1.0, mscale: float = 1.0) -> float:
    if scale <= 1:
        return 1.0
    return 0.1 * mscale * math.log(scale) + 1.0


# ---------------------------------------------------------------------- canned configs (offline box)
def deepseek_v2_lite_config(**overrides) -> Dict[str, Any]:
    """config.json of DeepSeek-Coder-V2-Lite-Instruct (the reference's demo model, README.md:26)."""
    d = dict(
        model_type="deepseek_v2", architectures=["DeepseekV2ForCausalLM"], vocab_size=102400,
        hidden_size=2048, intermediate_size=10944, moe_intermediate_size=1408, num_hidden_layers=27,
        num_attention_heads=16, num_key_value_heads=16, n_shared_experts=2, n_routed_experts=64,
        routed_scaling_factor=1.0, kv_lora_rank=512, q_lora_rank=None, qk_rope_head_dim=64,
        v_head_dim=128, qk_nope_head_dim=128, topk_method="greedy", n_group=1, topk_group=1,
        num_experts_per_tok=6, moe_layer_freq=1, first_k_dense_replace=1, norm_topk_prob=False,
        hidden_act="silu", max_position_embeddings=163840, rms_norm_eps=1e-6, rope_theta=10000.0,
        rope_scaling=dict(beta_fast=32, beta_slow=1, factor=40, mscale=0.707, mscale_all_dim=0.707,
                          original_max_position_embeddings=4096, type="yarn"),
        attention_bias=False, tie_word_embeddings=False, bos_token_id=100000, eos_token_id=100001,
    )
    d.update(overrides)
    return d


def llama3_8b_config(**overrides) -> Dict[str, Any]:
    d = dict(
        model_type="llama", architectures=["LlamaForCausalLM"], vocab_size=128256, hidden_size=4096,
        intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
        rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=8192, tie_word_embeddings=False,
        attention_bias=False, bos_token_id=128000, eos_token_id=128009,
    )
    d.update(overrides)
    return d


def gemma2_9b_config(**overrides) -> Dict[str, Any]:
    d = dict(
        model_type="gemma2", architectures=["Gemma2ForCausalLM"], vocab_size=256000, hidden_size=3584,
        intermediate_size=14336, num_hidden_layers=42, num_attention_heads=16, num_key_value_heads=8,
        head_dim=256, rms_norm_eps=1e-6, rope_theta=10000.0, query_pre_attn_scalar=256,
        attn_logit_softcapping=50.0, final_logit_softcapping=30.0, max_position_embeddings=8192,
    )
    d.update(overrides)
    return d
