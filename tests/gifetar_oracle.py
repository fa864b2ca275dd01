"""Plain, slow restatement of the Gifetar design, one function per mechanism, straight from its equations.  It shares no code with the
package: dense tensors, whole sequences from their first token, Python loops over heads; ``float64`` by default so that it can serve as
ground truth.

A model is ``(cfg, sd)``: ``cfg`` the parsed ``config.json`` (keys ``layers``, ``norm.eps``, ``residual_mult``, ``vocab``, ``width``),
``sd`` a dict name -> tensor.  ``random_model(cfg, seed)`` draws weights for any configuration."""
import math

import torch


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def query_temperature(pos, coef, every):
    """``1 + coef ln(floor((p + 1) / every) + 1)`` per position."""
    return 1.0 + coef * torch.log(torch.floor((pos + 1) / every) + 1.0)


def capped(s, cap):
    return cap * torch.tanh(s / cap)


def diff_lambda(p, diff):
    return math.exp(float((p["lq1"] * p["lk1"]).sum())) - math.exp(float((p["lq2"] * p["lk2"]).sum())) + diff


def diff_attention_mixer(h, p, m, eps):
    """``h`` [T, width] of one sequence from its start.  ``p``: tensors of the mixer (q q.b k k.b v v.b lq1 lk1 lq2 lk2 o)."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    diff = float(m["diff"])
    q = (h @ p["q"].T + p["q.b"]).view(T, H, 2, D)
    k = (h @ p["k"].T + p["k.b"]).view(T, G, 2, D)
    v = (h @ p["v"].T + p["v.b"]).view(T, G, V)
    pos = torch.arange(T, dtype=h.dtype)
    q = q * query_temperature(pos, float(m["q_temp"]["coef"]), float(m["q_temp"]["every"])).view(T, 1, 1, 1)
    lam = diff_lambda(p, diff)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        maps = []
        for c in range(2):
            s = capped((q[:, hd, c] @ k[:, g, c].T) * float(m["scale"]), float(m["softcap"]))
            s = s.masked_fill(~causal, float("-inf"))
            maps.append(torch.softmax(s, -1) @ v[:, g])
        out[:, hd] = unit_rms(maps[0] - lam * maps[1], eps) * (1.0 - diff)
    return out.reshape(T, H * V) @ p["o"].T


def moe_ff(h, p, mlp, gaps=None):
    """``p``: ``router``, ``router.b``, ``e<i>.gate|up|down``.  The ``top`` largest logits choose the experts, a softmax over those logits
    alone weighs their outputs.  ``gaps``: list that receives the distance between the last chosen and the first rejected logit."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ p["router"].T + p["router.b"]
    if gaps is not None and top < E:
        srt = torch.sort(z, -1, descending=True).values
        gaps.append(float((srt[:, top - 1] - srt[:, top]).min()))
    val, idx = torch.topk(z, top, dim=-1)
    wt = torch.softmax(val, -1)
    out = torch.zeros(h.shape[0], p["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            a = h[t] @ p[f"e{e}.gate"].T
            u = h[t] @ p[f"e{e}.up"].T
            out[t] += wt[t, j] * ((a * torch.sigmoid(a) * u) @ p[f"e{e}.down"].T)
    return out


def sub(sd, prefix):
    return {k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)}


def forward(cfg, sd, tokens, dtype=torch.float64, layers_out=None, gaps=None):
    """Logits ``[T, vocab]`` of one sequence; ``layers_out``: list that receives the residual stream after every layer."""
    sd = {k: v.to(dtype) for k, v in sd.items()}
    eps, mult = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    x = sd["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        assert L["type"] == "attention"
        y = diff_attention_mixer(layer_norm(x, sd[p + "norm1"], sd[p + "norm1.b"], eps), sub(sd, p + "mix."), L["mixer"], eps)
        x = x + mult * layer_norm(y, sd[p + "norm1b"], sd[p + "norm1b.b"], eps)
        if L.get("mlp"):
            assert L["mlp"]["kind"] == "moe"
            y = moe_ff(layer_norm(x, sd[p + "norm2"], sd[p + "norm2.b"], eps), sub(sd, p + "mlp."), L["mlp"], gaps)
            x = x + mult * layer_norm(y, sd[p + "norm2b"], sd[p + "norm2b.b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return layer_norm(x, sd["final.norm"], sd["final.norm.b"], eps) @ sd["embed"].T


def min_router_gap(cfg, sd, tokens):
    """Smallest distance between a chosen and a rejected router logit over all tokens and layers (inf without such a choice)."""
    gaps = []
    forward(cfg, sd, tokens, gaps=gaps)
    return min(gaps) if gaps else float("inf")


def tensor_shapes(cfg):
    W, out = int(cfg["width"]), {"embed": (int(cfg["vocab"]), int(cfg["width"]))}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        names = ["norm1", "norm1b"] + (["norm2", "norm2b"] if L.get("mlp") else [])
        for n in names:
            out[p + n] = out[p + n + ".b"] = (W,)
        H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        for n, rows in (("q", H * 2 * D), ("k", G * 2 * D), ("v", G * V)):
            out[p + "mix." + n], out[p + "mix." + n + ".b"] = (rows, W), (rows,)
        for n in ("lq1", "lk1", "lq2", "lk2"):
            out[p + "mix." + n] = (D,)
        out[p + "mix.o"] = (W, H * V)
        if L.get("mlp"):
            E, F = L["mlp"]["router"]["experts"], L["mlp"]["expert"]["ff"]
            for e in range(E):
                out[p + f"mlp.e{e}.gate"] = out[p + f"mlp.e{e}.up"] = (F, W)
                out[p + f"mlp.e{e}.down"] = (W, F)
            out[p + "mlp.router"], out[p + "mlp.router.b"] = (E, W), (E,)
    out["final.norm"] = out["final.norm.b"] = (W,)
    return out


def random_model(cfg, seed=0, dtype=torch.bfloat16):
    """Weights with unit-ish activations everywhere: matrices ~ N(0, 1/in), norm weights around 1, biases and router biases small
    but not zero, the lambda vectors small."""
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".", 1)[-1] if name.startswith("l") else name
        if len(shape) == 2:
            std = 1.0 if name == "embed" else shape[1] ** -0.5
            if leaf == "mlp.router":
                std *= 3.0                       # spread the logits: fewer near-ties between experts
            t = torch.randn(shape, generator=g) * std
        elif leaf.endswith(".b"):
            t = torch.randn(shape, generator=g) * 0.2
        elif leaf.startswith("mix.l"):
            t = torch.randn(shape, generator=g) * 0.3
        else:
            t = 1.0 + torch.randn(shape, generator=g) * 0.1
        sd[name] = t.to(dtype)
    return sd
