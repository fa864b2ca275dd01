"""Plain, slow restatement of the Gokapel design, one function per mechanism, straight from its equations.  It shares no code with the
package: dense tensors, whole sequences from their first token, Python loops over tokens and heads; ``float64`` by default so that it
can serve as ground truth.

A model is ``(cfg, sd)``: ``cfg`` the parsed ``config.json`` (keys ``layers``, ``norm.eps``, ``residual_mult``, ``streams``,
``embedding.scale``, ``vocab``, ``width``), ``sd`` a dict name -> tensor.  ``random_model(cfg, seed)`` draws weights for any
configuration."""
import math

import torch


# ---------------------------------------------------------------------------------------------------------------- small pieces
def dyt(x, p, name):
    """Dynamic tanh in place of a norm: ``tanh(alpha x) * w + b``."""
    return torch.tanh(p[name + ".alpha"] * x) * p[name] + p[name + ".b"]


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def relu2(x):
    return torch.relu(x) ** 2


def sub(sd, prefix):
    return {k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)}


def short_conv_silu(u, w):
    """``u`` [T, C], ``w`` [C, taps] (last column = the current token); zeros before the start."""
    T, C = u.shape
    K = w.shape[1]
    pad = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u])
    acc = torch.zeros(T, C, dtype=u.dtype)
    for j in range(K):
        acc += pad[j:j + T] * w[:, j]
    return acc * torch.sigmoid(acc)


# ---------------------------------------------------------------------------------------------------------------- mixers
def channel_delta_mixer(h, p, m, eps):
    """Gated delta rule with one decay per head and key channel.  ``h`` [T, width] of one sequence from its start."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(h @ p["q"].T, p["q.conv"]).view(T, G, D)
    k = short_conv_silu(h @ p["k"].T, p["k.conv"]).view(T, G, D)
    v = short_conv_silu(h @ p["v"].T, p["v.conv"]).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ p["b"].T)                                                        # [T, H]
    step = torch.nn.functional.softplus((h @ p["a1"].T) @ p["a2"].T + p["dt_bias"]).view(T, H, D)
    decay = torch.exp(-torch.exp(p["A_log"]).view(1, H, 1) * step)                             # [T, H, D]
    gate = torch.sigmoid((h @ p["g1"].T) @ p["g2"].T).view(T, H, V)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(D, V, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hd] = S.T @ q[t, g]
    out = unit_rms(out, eps) * p["norm"] * gate
    return out.reshape(T, H * V) @ p["o"].T


def rotate_pairs(x, pos, dims, base):
    """Adjacent pairs ``(2i, 2i+1)`` of the first ``dims`` entries turn by ``pos * base^(-2i/dims)``.  ``x`` [T, heads, d]."""
    if not dims:
        return x
    f = base ** (-2.0 * torch.arange(dims // 2, dtype=x.dtype) / dims)
    a = pos.to(x.dtype)[:, None] * f
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    rot = torch.stack([u * c - v * s, v * c + u * s], -1).flatten(-2)
    return torch.cat([rot, x[..., dims:]], -1)


def chunked_sink_attention(h, p, m, eps):
    """Grouped-query attention whose queries see the keys of their own block of ``mask.size`` positions only, with one extra
    keyless term ``exp(sink_h)`` in the softmax denominator."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T).view(T, H, D)
    k = (h @ p["k"].T).view(T, G, D)
    v = (h @ p["v"].T).view(T, G, V)
    q, k = unit_rms(q, eps) * p["q.norm"], unit_rms(k, eps) * p["k.norm"]
    pos = torch.arange(T)
    rot = m.get("rot") or {}
    q = rotate_pairs(q, pos, int(rot.get("dims", 0)), float(rot.get("base", 10000.0)))
    k = rotate_pairs(k, pos, int(rot.get("dims", 0)), float(rot.get("base", 10000.0)))
    size = int((m.get("mask") or {}).get("size", 0) or 0)
    seen = pos[None, :] <= pos[:, None]
    if size:
        seen = seen & ((pos[None, :] // size) == (pos[:, None] // size))
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(m["scale"])
        s = s.masked_fill(~seen, float("-inf"))
        if "sink" in p:
            full = torch.cat([s, p["sink"][hd].expand(T, 1)], -1)
            w = torch.softmax(full, -1)[:, :T]
        else:
            w = torch.softmax(s, -1)
        out[:, hd] = w @ v[:, g]
    return out.reshape(T, H * V) @ p["o"].T


def min_gru(h, p):
    """Gates that read the current token only: ``S_t = (1 - z_t) S_(t-1) + z_t c_t``; read-out gated by ``silu``."""
    T = h.shape[0]
    z = torch.sigmoid(h @ p["z"].T + p["z.b"])
    u = h @ p["x"].T + p["x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    gate = h @ p["g"].T
    gate = gate * torch.sigmoid(gate)
    S = torch.zeros(z.shape[1], dtype=h.dtype)
    rows = []
    for t in range(T):
        S = (1 - z[t]) * S + z[t] * cand[t]
        rows.append(S * gate[t])
    return torch.stack(rows) @ p["o"].T


def parallel_mixer(h, p, m, eps):
    left = chunked_sink_attention(h, sub(p, "left."), m["left"], eps)
    right = min_gru(h, sub(p, "right."))
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


# ---------------------------------------------------------------------------------------------------------------- feed-forwards
def dense_ff(h, p):
    return relu2(h @ p["up"].T) @ p["down"].T


def route(h, p, r, gaps=None):
    """Scores = softmax over all experts; the choice adds ``correction`` and is limited to the ``groups.keep`` groups (of ``groups.count``
    runs of neighbours) with the largest member; weights = the chosen experts' plain scores.  Returns ``(idx, w)`` lists per token."""
    E, top = int(r["experts"]), int(r["top"])
    gr = r.get("groups") or {}
    ng, keep = int(gr.get("count", 1)), int(gr.get("keep", gr.get("count", 1)))
    s = torch.softmax(h @ p["router"].T, -1)
    c = s + p["correction"] if "correction" in p else s.clone()
    if ng > 1 and keep < ng:
        gs = c.view(-1, ng, E // ng).max(-1).values
        if gaps is not None:
            srt = torch.sort(gs, -1, descending=True).values
            gaps.append(float((srt[:, keep - 1] - srt[:, keep]).min()))
        best = torch.topk(gs, keep, dim=-1).indices
        ok = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, best, True)
        c = c.masked_fill(~ok.repeat_interleave(E // ng, 1), float("-inf"))
    if gaps is not None and top < E:
        srt = torch.sort(c, -1, descending=True).values
        d = srt[:, top - 1] - srt[:, top]
        gaps.append(float(d[torch.isfinite(d)].min()) if torch.isfinite(d).any() else float("inf"))
    idx = torch.topk(c, top, dim=-1).indices
    return idx, torch.gather(s, 1, idx)


def moe_ff(h, p, mlp, gaps=None):
    idx, w = route(h, p, mlp["router"], gaps)
    out = torch.zeros(h.shape[0], p["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += w[t, j] * (relu2(h[t] @ p[f"e{e}.up"].T) @ p[f"e{e}.down"].T)
    if mlp.get("shared"):
        out = out + dense_ff(h, sub(p, "shared."))
    return out


# ---------------------------------------------------------------------------------------------------------------- the stack
def sublayer_step(xs, sd, p, q, fn, mult):
    """Hyper-connected residual step ``q`` (1: mixer, 2: feed-forward) on the streams ``xs`` [S, T, width]."""
    hc = f"{p}hc{q}."
    u = torch.einsum("s,stw->tw", sd[hc + "in"], xs)
    h = dyt(u, sd, f"{p}norm{q}")
    y = fn(h)
    if f"{p}ls{q}" in sd:
        y = y * sd[f"{p}ls{q}"]
    if f"{p}rg{q}" in sd:
        y = y * torch.sigmoid(h @ sd[f"{p}rg{q}"].T + sd[f"{p}rg{q}.b"])
    return torch.einsum("st,sjw->tjw", sd[hc + "mix"], xs) + mult * sd[hc + "out"][:, None, None] * y[None]


def forward(cfg, sd, tokens, dtype=torch.float64, layers_out=None, gaps=None):
    """Logits ``[T, vocab]`` of one sequence; ``layers_out``: list that receives the sum of the streams after every layer."""
    sd = {k: v.to(dtype) for k, v in sd.items()}
    eps, mult, S = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0)), int(cfg.get("streams", 1))
    x = sd["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    xs = x[None].repeat(S, 1, 1)
    for i, L in enumerate(cfg["layers"]):
        p = f"l{L.get('weights_of', i)}."
        m = L["mixer"]
        if L["type"] == "channel_delta":
            mixer = lambda h: channel_delta_mixer(h, sub(sd, p + "mix."), m, eps)
        elif L["type"] == "parallel":
            mixer = lambda h: parallel_mixer(h, sub(sd, p + "mix."), m, eps)
        else:
            raise ValueError(L["type"])
        xs = sublayer_step(xs, sd, p, 1, mixer, mult)
        mlp = L.get("mlp")
        if mlp:
            ff = (lambda h: dense_ff(h, sub(sd, p + "mlp."))) if mlp.get("kind", "dense") == "dense" else (lambda h: moe_ff(h, sub(sd, p + "mlp."), mlp, gaps))
            xs = sublayer_step(xs, sd, p, 2, ff, mult)
        if layers_out is not None:
            layers_out.append(xs.sum(0))
    return dyt(xs.sum(0), sd, "final.norm") @ sd["embed"].T


def min_router_gap(cfg, sd, tokens):
    """Smallest distance between a chosen and a rejected choice score (experts and groups) over all tokens and layers."""
    gaps = []
    forward(cfg, sd, tokens, gaps=gaps)
    return min(gaps) if gaps else float("inf")


# ---------------------------------------------------------------------------------------------------------------- random models
def tensor_shapes(cfg, ranks=(8, 8)):
    W, S = int(cfg["width"]), int(cfg.get("streams", 1))
    out = {"embed": (int(cfg["vocab"]), W)}

    def norm(name):
        out[name], out[name + ".b"], out[name + ".alpha"] = (W,), (W,), ()

    for i, L in enumerate(cfg["layers"]):
        if "weights_of" in L:
            continue
        p, m = f"l{i}.", L["mixer"]
        for q in (1, 2) if L.get("mlp") else (1,):
            norm(f"{p}norm{q}")
            out[f"{p}ls{q}"] = (W,)
            out[f"{p}hc{q}.in"], out[f"{p}hc{q}.out"], out[f"{p}hc{q}.mix"] = (S,), (S,), (S, S)
            out[f"{p}rg{q}"], out[f"{p}rg{q}.b"] = (W, W), (W,)
        if L["type"] == "channel_delta":
            H, G, D, V, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            ra, rg = ranks                       # inner sizes of the two low-rank maps (decay, output gate): tensor shapes, not config
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * V)):
                out[p + "mix." + n], out[p + "mix." + n + ".conv"] = (rows, W), (rows, K)
            out[p + "mix.b"], out[p + "mix.A_log"], out[p + "mix.norm"] = (H, W), (H,), (V,)
            out[p + "mix.a1"], out[p + "mix.a2"], out[p + "mix.dt_bias"] = (ra, W), (H * D, ra), (H * D,)
            out[p + "mix.g1"], out[p + "mix.g2"] = (rg, W), (H * V, rg)
            out[p + "mix.o"] = (W, H * V)
        else:
            a, r = m["left"], m["right"]
            H, G, D, V, R = a["heads"], a["kv_heads"], a["dim"], a["vdim"], r["width"]
            out[p + "mix.left.q"], out[p + "mix.left.k"], out[p + "mix.left.v"] = (H * D, W), (G * D, W), (G * V, W)
            out[p + "mix.left.q.norm"] = out[p + "mix.left.k.norm"] = (D,)
            out[p + "mix.left.sink"], out[p + "mix.left.o"] = (H,), (W, H * V)
            for n in ("z", "x", "g"):
                out[p + "mix.right." + n] = (R, W)
            out[p + "mix.right.z.b"] = out[p + "mix.right.x.b"] = (R,)
            out[p + "mix.right.o"] = (W, R)
        mlp = L.get("mlp")
        if mlp and mlp.get("kind", "dense") == "dense":
            out[p + "mlp.up"], out[p + "mlp.down"] = (mlp["ff"], W), (W, mlp["ff"])
        elif mlp:
            E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
            for e in range(E):
                out[p + f"mlp.e{e}.up"], out[p + f"mlp.e{e}.down"] = (F, W), (W, F)
            out[p + "mlp.router"], out[p + "mlp.correction"] = (E, W), (E,)
            if mlp.get("shared"):
                out[p + "mlp.shared.up"], out[p + "mlp.shared.down"] = (mlp["shared"]["ff"], W), (W, mlp["shared"]["ff"])
    norm("final.norm")
    return out


def random_model(cfg, seed=0, dtype=torch.bfloat16, ranks=(8, 8)):
    """Weights that keep every mechanism alive: matrices ~ N(0, 1/in), norm weights around 1, stream mixes near the identity, decays
    spread between fast and slow, sinks and corrections of the size of the scores they compete with."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda shape, std=1.0: torch.randn(shape, generator=g) * std
    S = int(cfg.get("streams", 1))
    sd = {}
    for name, shape in tensor_shapes(cfg, ranks).items():
        leaf = name.split(".", 1)[-1] if name.startswith("l") else name
        if leaf.endswith(".alpha"):
            t = torch.tensor(0.6) + rn((), 0.1)
        elif leaf.endswith(".conv"):
            t = rn(shape, 0.5)
        elif leaf.endswith("hc1.mix") or leaf.endswith("hc2.mix"):
            t = torch.eye(S) * 0.9 + rn(shape, 0.1)
        elif ".hc" in "." + leaf:
            t = (1.0 / S if leaf.endswith(".in") else 1.0) + rn(shape, 0.1)
        elif leaf == "mix.A_log":
            t = torch.log(torch.rand(shape, generator=g) * 1.5 + 0.05)
        elif leaf == "mix.dt_bias":
            t = rn(shape, 1.0) - 1.0
        elif leaf == "mix.left.sink":
            t = rn(shape, 1.0)
        elif leaf == "mlp.correction":
            t = rn(shape, 0.05)
        elif leaf == "mlp.router":
            t = rn(shape, 3.0 * shape[1] ** -0.5)
        elif leaf.startswith("rg") and len(shape) == 2:
            t = rn(shape, shape[1] ** -0.5)
        elif len(shape) == 2:
            t = rn(shape, 0.5 if name == "embed" else shape[1] ** -0.5)
        elif leaf.endswith(".b"):
            t = rn(shape, 0.2)
        else:
            t = 1.0 + rn(shape, 0.1)
        sd[name] = t.to(dtype)
    return sd
