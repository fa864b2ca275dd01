"""Gokapel (several residual streams with dynamic-tanh norms; gated delta rule with per-channel decays; attention inside blocks of
positions with a sink beside a minGRU; dense and mixture-of-experts feed-forwards with a group-limited softmax router) against the plain
oracle in ``gokapel_oracle.py``: every mechanism alone, prefill against token-by-token decoding, prompt portions down to two tokens,
ragged batches against each request alone, pages and state slots that are freed and used again, keys just inside and just outside a
block, far tokens held only by a recurrent state, the sink, other sizes (one stream and three, one key/value head and as many as query
heads, two-tap and one-tap convolutions, rotation of all / some / no entries, no block limit, top-1 and all-experts routers with and
without groups, a layer without feed-forward, a layer that runs on another layer's weights), long decoding, and greedy generation through
the engine.

Runs on the CPU with the unfused ops; the ``gpu`` variants run the same cases on the sm_100a kernels in fp32 and bf16.
"""
import copy
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import gokapel_oracle as oracle  # noqa: E402

from mlx_sharding_b200.config import ModelConfig  # noqa: E402
from mlx_sharding_b200.engine.core import LLMEngine  # noqa: E402
from mlx_sharding_b200.engine.sampler import SamplingParams  # noqa: E402
from mlx_sharding_b200.engine.trace import TraceSession  # noqa: E402
from mlx_sharding_b200.models import build_stage  # noqa: E402
from mlx_sharding_b200.ops import BatchMeta, LinearWeight, get_backend  # noqa: E402
from mlx_sharding_b200.parallel.pipeline import LocalPipeline, StageExecutor  # noqa: E402
from mlx_sharding_b200.utils.checkpoint import random_state_dict  # noqa: E402

DENSE = dict(kind="dense", ff=40)
MOE = dict(kind="moe", router=dict(experts=6, top=2, groups=dict(count=3, keep=2)), expert=dict(ff=24), shared=dict(ff=16))
MOE_TOP1 = dict(kind="moe", router=dict(experts=4, top=1, groups=dict(count=1, keep=1)), expert=dict(ff=16))     # no groups, no always-on expert
MOE_ALL = dict(kind="moe", router=dict(experts=4, top=4, groups=dict(count=2, keep=2)), expert=dict(ff=8), shared=dict(ff=8))   # every expert chosen


def delta(heads, kv_heads, dim, vdim, conv, mlp):
    return dict(type="channel_delta", mixer=dict(conv=conv, dim=dim, heads=heads, kv_heads=kv_heads, vdim=vdim), mlp=copy.deepcopy(mlp))


def par(heads, kv_heads, dim, vdim, block, rot, scale, gru, mlp, ls=0.6, rs=0.5, base=100.0):
    left = dict(dim=dim, heads=heads, kv_heads=kv_heads, scale=scale, vdim=vdim)
    if block:
        left["mask"] = dict(size=block)
    if rot:
        left["rot"] = dict(base=base, dims=rot)
    return dict(type="parallel", mixer=dict(left=left, left_scale=ls, right=dict(width=gru), right_scale=rs), mlp=copy.deepcopy(mlp))


D_GQ = delta(4, 2, 8, 12, 4, DENSE)                      # two heads per query / key head
D_MH = delta(3, 3, 6, 10, 2, MOE)                        # as many; two taps; odd sizes
D_ONE = delta(2, 1, 16, 40, 1, None)                     # one tap (no history), wide values, no feed-forward
P_GQ = par(6, 2, 8, 12, 7, 4, 0.4, 20, MOE)              # three query heads per key/value head; blocks of 7; half the entries turn
P_MQ = par(3, 1, 16, 40, 16, 16, 0.2, 33, DENSE)         # one key/value head; block = page; all entries turn
P_MH = par(3, 3, 6, 10, 0, 0, 0.5, 9, MOE_TOP1)          # no block limit, no rotation
STACK = [D_GQ, P_GQ, D_MH, P_MQ, dict(D_GQ, weights_of=0), dict(P_GQ, weights_of=1)]
CASES = {"delta_gq": [D_GQ], "delta_mh_moe": [D_MH], "delta_one_tap": [D_ONE], "par_gq_moe": [P_GQ], "par_mq": [P_MQ], "par_mh_free": [P_MH],
         "stack": STACK}
DEVICES = [pytest.param("cpu", torch.float32, 2e-4, id="cpu"),
           pytest.param("cuda", torch.float32, 2e-4, id="b200-f32", marks=pytest.mark.gpu),
           pytest.param("cuda", torch.bfloat16, 6e-2, id="b200-bf16", marks=pytest.mark.gpu)]


def make_cfg(layers, width=48, vocab=96, eps=1e-3, mult=0.5, streams=2, scale=3.0, dtype=None):
    """``dtype=bfloat16``: every router takes all experts of all groups.  Under bf16 activations a score moves by a few thousandths, and over
    hundreds of routing decisions of a stack some choice is always closer than that, so a comparison with exact arithmetic cannot rest on
    them; the choice itself is compared in exact mode (same kernels, ``float`` instantiation) and, in bf16, on exact inputs (the op tests)."""
    layers = copy.deepcopy(layers)
    if dtype == torch.bfloat16:
        for L in layers:
            r = (L.get("mlp") or {}).get("router")
            if r:
                r["top"], r["groups"]["keep"] = r["experts"], r["groups"]["count"]
    return dict(architecture="Gokapel", embedding=dict(scale=scale), layers=layers, norm=dict(eps=eps), residual_mult=mult,
                streams=streams, vocab=vocab, width=width)


def make_model(cfgd, device="cpu", dtype=torch.float32, seed=3, edit=None):
    cfg = ModelConfig.from_dict(cfgd)
    sd = dict(random_state_dict(cfg, dtype=torch.bfloat16, seed=seed))
    if edit:
        edit(sd)
    model = build_stage(cfg, None, dtype, device).load_state({k: v.clone() for k, v in sd.items()})
    return model, sd


def session(model, pages=12, page_size=16, live=4):
    return TraceSession(StageExecutor(model, pages, page_size, num_state_slots=live + 1), (pages - 1) * page_size, live)


def run_whole(model, tokens, **kw):
    return session(model, **kw).step([dict(id="a", tokens=tokens, want=list(range(len(tokens))))])


def toks(n, vocab=96, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


SHOWS = 1e-2      # a fault must move the logits by this share of their largest: 50 times the exact-mode tolerance


def close(a, b, tol):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs().max().item() / max(1.0, b.abs().max().item())
    assert err < tol, f"relative error {err:.3e} >= {tol}"


def decode_after(model, t, n_prompt, **kw):
    s = session(model, **kw)
    got = [s.step([dict(id="r", tokens=t[:n_prompt], want=list(range(n_prompt)))])]
    got += [s.step([dict(id="r", tokens=[x], want=[0])]) for x in t[n_prompt:]]
    return torch.cat(got)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
@pytest.mark.parametrize("case", list(CASES))
def test_mechanism_against_oracle(case, device, dtype, tol):
    """Each layer shape alone (and the mixed stack with two layers that run on another layer's weights): whole prompt, every position;
    45 tokens span three 16-token pages and several blocks."""
    cfgd = make_cfg(CASES[case], streams=3 if case == "par_mq" else 2, dtype=dtype)
    model, sd = make_model(cfgd, device, dtype)
    t = toks(45, seed=0)
    lo = []
    want = oracle.forward(cfgd, sd, t, layers_out=lo)
    got_layers = []
    s = session(model)
    tb = s.table
    tb.add(0), tb.reserve(0, len(t))
    meta = BatchMeta.build([len(t)], [0], [tb.pages[0]], 16, device=device, state_slots=tb.state_slots([0]))
    got = model(torch.tensor(t, device=device), meta, s.stage.kv, all_logits=True, layer_out=got_layers)
    close(got, want, tol)
    for a, b in zip(got_layers, lo):                    # the sum of the streams after every layer
        close(a, b, tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES[:2])
@pytest.mark.parametrize("streams", [1, 2, 3])
def test_stream_step_alone(streams, device, dtype, tol):
    """The fused sublayer boundary against its equations: update of all streams at once from the old ones (a mix matrix far from the
    identity, indexed [from, to]), second branch, layer scale, gate, then the read and the dynamic tanh.  One stream: the plain sum."""
    O = get_backend("b200" if device == "cuda" else "reference")
    g = torch.Generator().manual_seed(streams)
    rn = lambda *s: torch.randn(*s, generator=g)
    T, W, S = 5, 40, streams
    xs, y, y2, gate, ls, mix, ow, iw, w, b = rn(T, S, W), rn(T, W), rn(T, W), rn(T, W) * 2, 1 + 0.3 * rn(W), rn(S, S), rn(S), rn(S), 1 + 0.2 * rn(W), rn(W)
    dev = lambda t: t.to(device)
    x2 = dev(xs.clone())
    ha = O.hyper_step_(x2, dev(y), dev(y2), dev(gate).to(dtype), dev(ls), dev(mix), dev(ow), 0.7, dev(iw), 0.8, dev(w), dev(b), dtype)
    r = (y + y2).double() * ls.double() * torch.sigmoid(gate.double())
    want = torch.stack([sum(mix[s, j].double() * xs[:, s].double() for s in range(S)) + 0.7 * ow[j].double() * r for j in range(S)], 1)
    close(x2, want, 1e-5)
    u = sum(iw[j].double() * want[:, j] for j in range(S))
    close(ha, torch.tanh(0.8 * u) * w.double() + b.double(), 1e-5)
    ha0 = O.hyper_step_(x2, None, None, None, None, None, None, 0.0, dev(iw), 0.8, dev(w), dev(b), dtype)        # only the read
    close(ha0, ha, 1e-6)
    close(x2, want, 1e-5)
    e = O.stream_embed(dev(rn(9, W)).to(dtype), dev(torch.tensor([3, 0, 8])), 2.5, S)
    assert e.shape == (3, S, W) and e.dtype == torch.float32 and torch.equal(e[:, 0], e[:, S - 1])


@pytest.mark.parametrize("device,dtype,tol", DEVICES[:2])
def test_router_alone(device, dtype, tol):
    """Group-limited choice with corrections: a negative choice score inside a kept group must beat every expert of a dropped group
    (dropped = minus infinity, not zero); weights are the plain scores, not renormalised, without the correction."""
    O = get_backend("b200" if device == "cuda" else "reference")
    z = torch.tensor([[4.0, 0.0, -9.0, -9.0, 3.0, 2.9], [0.0, 0.1, 0.2, 0.3, 0.4, 0.5], [1.0, 1.0, 1.0, 1.0, 1.0, 1.0]])
    corr = torch.tensor([0.0, -0.5, -0.5, -0.5, 0.0, 0.0])
    idx, w = O.group_softmax_topk(z.to(device), corr.to(device), 6, 2, 3, 1)
    s = torch.softmax(z, -1)
    # row 0: group 0 wins through expert 0; its second member has choice score s - 0.5 < 0 and is still chosen.  Row 2: the first and the
    # last group tie, the lower id is kept
    assert idx[0].tolist() == [0, 1] and idx[1].tolist() == [5, 4] and idx[2].tolist() == [0, 1]
    close(w, torch.gather(s, 1, idx.cpu().long()), 1e-6)
    p = {"router": torch.eye(6, dtype=torch.float64), "correction": corr.double()}
    oi, ow = oracle.route(z.double(), p, dict(experts=6, top=2, groups=dict(count=3, keep=1)))
    assert oi[:2].tolist() == idx[:2].tolist()
    idx, w = O.group_softmax_topk(z.to(device), None, 6, 3, 1, 1)                                     # no groups, no correction
    assert idx[0].tolist() == [0, 4, 5] and idx[2].tolist() == [0, 1, 2]                              # ties go to the lowest id
    idx, _ = O.group_softmax_topk(z.to(device), corr.to(device), 6, 4, 3, 2)
    assert sorted(idx[0].tolist()) == [0, 1, 4, 5]


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
@pytest.mark.parametrize("experts,top,groups,keep,ff,rows", [(6, 2, 3, 2, 24, 7), (4, 1, 1, 1, 16, 3), (4, 4, 2, 2, 8, 70), (8, 2, 4, 2, 128, 150)])
def test_experts_alone(experts, top, groups, keep, ff, rows, device, dtype, tol):
    """Router and routed experts as ops against the oracle's feed-forward: few rows (one weight-row read per pair), many rows (sorted
    rows, one product per expert; expert rows of 128 take the grouped tensor-core GEMM in bf16), top-1, all experts."""
    O = get_backend("b200" if device == "cuda" else "reference")
    K = 128
    g = torch.Generator().manual_seed(experts * 100 + rows)
    rn = lambda *s: torch.randn(*s, generator=g)
    bank = lambda o, i: (rn(experts, o, i) * i ** -0.5).bfloat16()
    wu, wd, wr, cr = bank(ff, K), bank(K, ff), (rn(experts, K) * 3 * K ** -0.5).bfloat16(), (0.05 * rn(experts)).bfloat16()
    p = {"router": wr.double(), "correction": cr.double()}
    for e in range(experts):
        p.update({f"e{e}.up": wu[e].double(), f"e{e}.down": wd[e].double()})
    mlp = dict(router=dict(experts=experts, top=top, groups=dict(count=groups, keep=keep)))
    for seed in range(300):                  # the router sees the same bf16-exact inputs as the oracle: only a near-tie could flip a choice
        x = torch.randn(rows, K, generator=torch.Generator().manual_seed(seed)).bfloat16()
        gaps = []
        want = oracle.moe_ff(x.double(), p, mlp, gaps)
        if not gaps or min(gaps) > 1e-4:
            break
    else:
        raise AssertionError("no input without a close routing call found")
    dev = lambda t: t.to(device=device, dtype=dtype)
    lw = lambda t: LinearWeight(weight=dev(t).contiguous())
    xa = dev(x)
    idx, wt = O.group_softmax_topk(O.router_logits(xa, wr.float().to(device)), cr.float().to(device), experts, top, groups, keep)
    close(O.moe_relu2_experts(xa, idx, wt, lw(wu), lw(wd)), want, tol if dtype == torch.bfloat16 else 1e-5)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_attention_alone(device, dtype, tol):
    """Prologue and attention as ops: 2 key/value heads, 4 query heads, 27 tokens written as 13 + 14 into 8-token pages in scrambled
    order; blocks of 10 positions; rotation of 4 of 8 entries; a sink per head; output written into columns of a wider buffer."""
    O = get_backend("b200" if device == "cuda" else "reference")
    g = torch.Generator().manual_seed(5)
    rn = lambda *s: torch.randn(*s, generator=g)
    H, G, D, V, n, pad = 4, 2, 8, 12, 27, 8
    rows = rn(n, pad + H * D + G * D + G * V).to(dtype)
    qn, kn, sink = 1 + 0.2 * rn(D), 1 + 0.2 * rn(D), rn(H)
    inv = (50.0 ** (-2.0 * torch.arange(2, dtype=torch.float64) / 4)).float()
    dev = lambda t: t.to(device)
    kp, vp = torch.zeros(6, G, 8, D, dtype=dtype, device=device), torch.zeros(6, G, 8, V, dtype=dtype, device=device)
    pages, outs = [4, 1, 5, 2], []
    for lo, hi in ((0, 13), (13, 27)):
        meta = BatchMeta.build([hi - lo], [lo], [pages], 8, device=device)
        q = O.qk_norm_rope_append(dev(rows[lo:hi]), pad, pad + H * D, pad + H * D + G * D, H, D, dev(qn), dev(kn), 1e-3, dev(inv), kp, vp, meta)
        buf = torch.zeros(hi - lo, 8 + H * V, dtype=dtype, device=device)
        O.sink_attention(q, kp, vp, dev(sink), meta, 0.35, 10, 0, 0.7, dtype, buf, 8)
        assert float(buf[:, :8].abs().max()) == 0.0
        outs.append(buf[:, 8:])
    rd = rows.double()
    pos = torch.arange(n)
    q = oracle.rotate_pairs(oracle.unit_rms(rd[:, pad:pad + H * D].view(n, H, D), 1e-3) * qn.double(), pos, 4, 50.0)
    k = oracle.rotate_pairs(oracle.unit_rms(rd[:, pad + H * D:pad + (H + G) * D].view(n, G, D), 1e-3) * kn.double(), pos, 4, 50.0)
    v = rd[:, pad + (H + G) * D:].view(n, G, V)
    seen = (pos[None, :] <= pos[:, None]) & ((pos[None, :] // 10) == (pos[:, None] // 10))
    want = torch.zeros(n, H, V, dtype=torch.float64)
    for h in range(H):
        s = (q[:, h] @ k[:, h // 2].T * 0.35).masked_fill(~seen, float("-inf"))
        e = torch.exp(s - s.max(-1, keepdim=True).values)
        want[:, h] = (e / (e.sum(-1, keepdim=True) + torch.exp(sink[h].double() - s.max(-1, keepdim=True).values))) @ v[:, h // 2] * 0.7
    close(torch.cat(outs), want.view(n, H * V), tol if dtype == torch.bfloat16 else 1e-5)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_first_tokens_and_single_token(device, dtype, tol):
    cfgd = make_cfg(STACK, dtype=dtype)
    model, sd = make_model(cfgd, device, dtype)
    for t in ([5], toks(2, seed=4), toks(3, seed=5)):
        close(run_whole(model, t), oracle.forward(cfgd, sd, t), tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
@pytest.mark.parametrize("portions", [[1] * 23, [2, 2, 2, 17], [16, 7], [15, 1, 1, 6], [3, 13, 7], [22, 1], [8, 9, 6]])
def test_portions_equal_whole(portions, device, dtype, tol):
    """Prefill against token-by-token decoding and prompts cut anywhere (page edge at 16, block edges at 7, 14, 16, 21, convolution
    histories of 1 and 3 inputs that start inside the previous portion, 2-token portions)."""
    cfgd = make_cfg(STACK, dtype=dtype)
    model, sd = make_model(cfgd, device, dtype)
    t = toks(sum(portions), seed=1)
    want = oracle.forward(cfgd, sd, t)
    s, at, got = session(model), 0, []
    for n in portions:
        got.append(s.step([dict(id="r", tokens=t[at:at + n], want=list(range(n)))]))
        at += n
    close(torch.cat(got), want, tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_ragged_batch_and_reuse_of_pages_and_slots(device, dtype, tol):
    """Unequal requests in one batch (portions beside single tokens) equal each alone; a pool of 5 pages and 2 state slots serves 4
    requests one pair after another, so every page and slot is used again — by a request that must not see what the last one left."""
    cfgd = make_cfg(STACK, dtype=dtype)
    model, sd = make_model(cfgd, device, dtype)
    reqs = {n: toks(L, seed=10 + i) for i, (n, L) in enumerate([("a", 30), ("b", 9), ("c", 17), ("d", 33)])}
    want = {n: oracle.forward(cfgd, sd, t) for n, t in reqs.items()}
    s = session(model, pages=6, page_size=16, live=2)
    assert s.table.slots is not None and s.table.slots.num_free == 2
    got = {n: [] for n in reqs}

    def step(parts, end=()):
        entries = [dict(id=n, tokens=reqs[n][lo:hi], want=list(range(hi - lo))) for n, lo, hi in parts]
        out = s.step(entries)
        at = 0
        for n, lo, hi in parts:
            got[n].append(out[at:at + hi - lo])
            at += hi - lo
        s.end(end)

    step([("a", 0, 13), ("b", 0, 1)])
    step([("a", 13, 14), ("b", 1, 8)])
    step([("b", 8, 9), ("a", 14, 29)], end=["b"])
    step([("a", 29, 30)], end=["a"])
    assert s.table.alloc.num_free == 5 and s.table.slots.num_free == 2
    step([("d", 0, 2), ("c", 0, 16)])
    step([("c", 16, 17), ("d", 2, 33)], end=["c", "d"])
    for n in reqs:
        close(torch.cat(got[n]), want[n], tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_block_edges_show(device, dtype, tol):
    """Blocks of 9 positions counted from position 0, not from where a portion starts.  Sharp queries (the query weights are scaled)
    make single keys count; the oracle with blocks of 8 or 10 gives other logits at positions around the edges, so a limit that is one
    off would show.  In a prompt, in portions that start inside a block, and decoded one by one across edges and a page border."""
    layer = par(4, 2, 8, 12, 9, 4, 0.6, 10, None, ls=1.0, rs=0.1)
    cfgd = make_cfg([layer], dtype=dtype)
    model, sd = make_model(cfgd, device, dtype, edit=lambda sd: sd["l0.mix.left.q"].mul_(4.0))
    t = toks(40, seed=7)
    want = oracle.forward(cfgd, sd, t)
    for size, ps in ((8, (8, 17, 26)), (10, (9, 18, 27))):          # first position of a block that the other size still joins to the last
        other = copy.deepcopy(cfgd)
        other["layers"][0]["mixer"]["left"]["mask"]["size"] = size
        wrong = oracle.forward(other, sd, t)
        for p in ps:
            assert (wrong[p] - want[p]).abs().max() > SHOWS * want.abs().max()
    close(run_whole(model, t), want, tol)
    close(decode_after(model, t, 4), want, tol)
    s, at, got = session(model), 0, []
    for n in (5, 6, 2, 14, 13):                                     # portions that start at positions 5, 11, 13, 27: inside blocks
        got.append(s.step([dict(id="r", tokens=t[at:at + n], want=list(range(n)))]))
        at += n
    close(torch.cat(got), want, tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_sink_shows(device, dtype, tol):
    """Large sinks take most of the softmax mass at short contexts: leaving them out, or scaling them like a score, moves the logits."""
    layer = par(4, 2, 8, 12, 12, 8, 0.3, 10, None, ls=1.0, rs=0.1)
    cfgd = make_cfg([layer], mult=1.0, dtype=dtype)
    model, sd = make_model(cfgd, device, dtype, edit=lambda sd: sd["l0.mix.left.sink"].copy_(torch.tensor([3.0, 1.0, 2.0, 4.0])))
    t = toks(30, seed=8)
    want = oracle.forward(cfgd, sd, t)
    for alt in ({k: v for k, v in sd.items() if not k.endswith("sink")}, {k: (v * 0.3 if k.endswith("sink") else v) for k, v in sd.items()}):
        assert (oracle.forward(cfgd, alt, t) - want).abs().max() > 3 * SHOWS * want.abs().max()
    close(run_whole(model, t), want, tol)
    close(decode_after(model, t, 11), want, tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
@pytest.mark.parametrize("kind", ["delta", "gru"])
def test_far_token_lives_in_the_state(kind, device, dtype, tol):
    """With slow decays (delta rule) / rarely open gates (minGRU) and attention limited to blocks of 8, only the recurrent state carries
    the first eight tokens to position 60 and beyond, four pages on: other tokens there move the late logits; a state that was lost or
    not carried across steps would show.  In a prompt, in decoding, and in portions."""
    if kind == "delta":
        cfgd = make_cfg([delta(2, 1, 8, 12, 2, None)], mult=1.0, dtype=dtype)
        edit = lambda sd: (sd["l0.mix.A_log"].fill_(-6.0), sd["l0.mix.dt_bias"].fill_(-3.0), sd["l0.mix.o"].mul_(3.0))
    else:
        cfgd = make_cfg([par(2, 1, 8, 12, 8, 4, 0.3, 24, None, ls=0.2, rs=1.5)], mult=1.0, dtype=dtype)
        edit = lambda sd: (sd["l0.mix.right.z.b"].fill_(-4.5), sd["l0.mix.right.z"].mul_(0.3), sd["l0.mix.right.o"].mul_(6.0))
    model, sd = make_model(cfgd, device, dtype, edit=edit)
    for seed in range(40):
        t = toks(70, seed=200 + seed)
        want = oracle.forward(cfgd, sd, t)
        lost = [(x + 1 + i) % 96 if i < 8 else x for i, x in enumerate(t)]
        if (oracle.forward(cfgd, sd, lost)[60:] - want[60:]).abs().max() > SHOWS * want.abs().max():
            break
    else:
        raise AssertionError("no sequence found in which the far tokens show")
    close(run_whole(model, t, pages=8), want, tol)
    close(decode_after(model, t, 55, pages=8), want, tol)
    s, at, got = session(model, pages=8), 0, []
    for n in (2, 31, 2, 30, 5):
        got.append(s.step([dict(id="r", tokens=t[at:at + n], want=list(range(n)))]))
        at += n
    close(torch.cat(got), want, tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_long_prompt_then_decode(device, dtype, tol):
    """A 290-token prompt over blocks of 300 positions (one block) and without a block limit, then single tokens whose keys are split
    over CTAs and merged (with the sink in the merge) on the GPU."""
    cfgd = make_cfg([par(4, 2, 8, 12, 300, 8, 0.3, 16, MOE_ALL), par(2, 1, 16, 40, 0, 4, 0.2, 8, None), delta(2, 2, 8, 8, 3, None)], dtype=dtype)
    model, sd = make_model(cfgd, device, dtype)
    t = toks(296, seed=9)
    want = oracle.forward(cfgd, sd, t)
    s = session(model, pages=21)
    rows = [0, 5, 6, 7, 31, 32, 100, 127, 128, 289]
    got = [s.step([dict(id="r", tokens=t[:290], want=rows)])] + [s.step([dict(id="r", tokens=[x], want=[0])]) for x in t[290:]]
    close(torch.cat(got), torch.cat([want[rows], want[290:]]), tol * (3 if dtype == torch.bfloat16 else 1))


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_long_portions_across_blocks(device, dtype, tol):
    """Portions of 40, 250 and 44 tokens over blocks of 256 positions and without a block limit: the second portion starts inside the first
    block and ends in the second (on the GPU long portions of one sequence take the matrix-product form of the attention, block by block,
    and the minGRU runs its slices of the portion side by side)."""
    cfgd = make_cfg([par(4, 2, 8, 12, 256, 8, 0.3, 40, None), par(2, 1, 16, 40, 0, 4, 0.2, 8, DENSE)], dtype=dtype)
    model, sd = make_model(cfgd, device, dtype)
    t = toks(334, seed=19)
    want = oracle.forward(cfgd, sd, t)
    s, at, got, rows = session(model, pages=23), 0, [], []
    for n in (40, 250, 44):
        want_rows = sorted({0, 1, n // 2, n - 2, n - 1} | {r - at for r in (255, 256, 257) if at <= r < at + n})
        got.append(s.step([dict(id="r", tokens=t[at:at + n], want=want_rows)]))
        rows += [at + r for r in want_rows]
        at += n
    close(torch.cat(got), want[rows], tol * (3 if dtype == torch.bfloat16 else 1))


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_long_decode(device, dtype, tol):
    """150 single-token steps after a 3-token prompt: states are read and written every step, blocks and pages come and go."""
    cfgd = make_cfg([D_GQ, P_GQ, D_ONE], dtype=dtype)
    model, sd = make_model(cfgd, device, dtype)
    t = toks(153 if dtype != torch.bfloat16 else 60, seed=5)
    close(decode_after(model, t, 3), oracle.forward(cfgd, sd, t), tol * (3 if dtype == torch.bfloat16 else 1))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 6e-2)])
def test_tensor_core_sizes(dtype, tol):
    """Width, feed-forward and expert rows that are multiples of 128, head sizes that are multiples of 8: bf16 takes the tensor-core GEMMs
    (squared ReLU in the epilogue of the dense and the grouped product); value widths of 128 use several registers per lane."""
    moe = dict(kind="moe", router=dict(experts=8, top=2, groups=dict(count=4, keep=2)), expert=dict(ff=128), shared=dict(ff=128))
    cfgd = make_cfg([delta(4, 2, 16, 32, 4, moe), par(4, 2, 16, 128, 24, 8, 0.25, 64, dict(kind="dense", ff=256)), delta(2, 2, 64, 64, 4, None)], width=128, dtype=dtype)
    model, sd = make_model(cfgd, "cuda", dtype)
    t = toks(44, seed=2)
    close(decode_after(model, t, 40), oracle.forward(cfgd, sd, t), tol)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 6e-2)])
def test_wide_values_long_context(dtype, tol):
    """Value widths of 128 and 256 (the attention kernel's 16-byte path, one and two register groups per lane) over spans long enough
    that the keys of a decoded token are split over CTAs and merged with the sink; portions of 2 to 31 tokens run the same kernel on
    many rows; a page of 16 (a tile of 32 keys spans two pages) and of 64."""
    cfgd = make_cfg([par(4, 2, 16, 128, 0, 8, 0.25, 24, None), par(2, 1, 8, 256, 288, 4, 0.35, 8, None), delta(2, 1, 32, 128, 4, None)], width=64, dtype=dtype)
    model, sd = make_model(cfgd, "cuda", dtype)
    t = toks(300, seed=13)
    want = oracle.forward(cfgd, sd, t)
    for pages, page_size in ((21, 16), (7, 64)):
        s, at, got = session(model, pages=pages, page_size=page_size), 0, []
        for n in [256, 2, 31, 5] + [1] * 6:
            got.append(s.step([dict(id="r", tokens=t[at:at + n], want=list(range(n)))]))
            at += n
        close(torch.cat(got), want, tol * (3 if dtype == torch.bfloat16 else 1))


def random_cfg(rng):
    """A configuration drawn at random: 2 to 4 owning layers of either mixer in any order plus layers that run on their weights, every
    size, constant and feed-forward kind drawn anew."""
    def moe():
        ng, keep = rng.choice([(1, 1), (2, 1), (4, 2), (3, 2), (4, 3)])
        per = rng.choice([2, 3, 4])
        d = dict(kind="moe", router=dict(experts=ng * per, top=rng.randint(1, min(4, keep * per)), groups=dict(count=ng, keep=keep)),
                 expert=dict(ff=rng.choice([24, 32, 40])))
        if rng.random() < 0.7:
            d["shared"] = dict(ff=rng.choice([16, 24]))
        return d

    def mlp():
        r = rng.random()
        return None if r < 0.15 else (dict(kind="dense", ff=rng.choice([40, 72])) if r < 0.55 else moe())

    def layer():
        kv, rep = rng.choice([1, 2, 3]), rng.choice([1, 2])
        if rng.random() < 0.5:
            return delta(kv * rep, kv, rng.choice([8, 12, 32]), rng.choice([8, 20, 32]), rng.choice([1, 2, 3, 4]), mlp())
        dim = rng.choice([8, 16, 32])
        return par(kv * rep, kv, dim, rng.choice([8, 24, 128]), rng.choice([0, 5, 16, 24, 33]), rng.choice([0, dim, dim // 2, 4]), rng.choice([0.125, 0.3]),
                   rng.choice([12, 40]), mlp(), ls=rng.choice([0.6, 1.0]), rs=rng.choice([0.5, 1.0]), base=rng.choice([10000.0, 50.0]))

    base = [layer() for _ in range(rng.randint(2, 4))]
    layers = [(j, L) for j, L in enumerate(base)] + [(j, dict(copy.deepcopy(L), weights_of=j)) for j, L in enumerate(base) if rng.random() < 0.4]
    rng.shuffle(layers)
    owner_at = {j: i for i, (j, L) in enumerate(layers) if "weights_of" not in L}
    for j, L in layers:
        if "weights_of" in L:
            L["weights_of"] = owner_at[j]
    return make_cfg([L for _, L in layers], width=rng.choice([40, 64, 72]), vocab=rng.choice([50, 77]), eps=rng.choice([1e-6, 1e-3]),
                    mult=rng.choice([0.3, 0.5, 1.0]), streams=rng.choice([1, 2, 3, 4]), scale=rng.choice([1.0, 4.0]))


@pytest.mark.parametrize("device,dtype,tol", DEVICES[:2])
def test_checkpoint_without_optional_tensors(device, dtype, tol):
    """A checkpoint without layer scales, gated-residual matrices and sinks: the loader takes what is there (plain stream update, ordinary
    softmax) and the fused projections have no gate segment."""
    cfgd = make_cfg([D_GQ, P_GQ, D_ONE], dtype=dtype)
    cfg = ModelConfig.from_dict(cfgd)
    sd = {k: v for k, v in random_state_dict(cfg, dtype=torch.bfloat16, seed=5) if not any(x in k for x in (".ls", ".rg", ".sink"))}
    model = build_stage(cfg, None, dtype, device).load_state({k: v.clone() for k, v in sd.items()})
    assert "rg" not in model.layer_weights[0]["seg"] and model.layer_weights[1]["sink"] is None and model.layer_weights[0]["ls1"] is None
    t = toks(40, seed=3)
    want = oracle.forward(cfgd, sd, t)
    close(run_whole(model, t), want, tol)
    close(decode_after(model, t, 21), want, tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES[:2])
@pytest.mark.parametrize("seed", [1, 2, 3, 4])
def test_random_configurations(seed, device, dtype, tol):
    """Configurations drawn at random (layer order, sizes, constants, shared weights), two requests stepped in portions of random sizes
    side by side, every position against the oracle.  Exact mode only: with this many routing decisions bf16 cannot be compared."""
    import random

    rng = random.Random(seed)
    cfgd = random_cfg(rng)
    model, sd = make_model(cfgd, device, dtype, seed=seed)
    reqs = {"a": toks(rng.randint(50, 80), vocab=cfgd["vocab"], seed=seed), "b": toks(rng.randint(10, 40), vocab=cfgd["vocab"], seed=seed + 1)}
    want = {n: oracle.forward(cfgd, sd, t) for n, t in reqs.items()}
    s = session(model, pages=10)
    got, at = {"a": [], "b": []}, {"a": 0, "b": 0}
    while any(at[n] < len(reqs[n]) for n in reqs):
        entries = []
        for n, sizes in (("a", [1, 2, 5, 17, 33]), ("b", [1, 1, 2, 9])):
            if at[n] < len(reqs[n]) and (n == "a" or rng.random() < 0.7):
                k = min(len(reqs[n]) - at[n], rng.choice(sizes))
                entries.append(dict(id=n, tokens=reqs[n][at[n]:at[n] + k], want=list(range(k))))
        if not entries:
            continue
        out = s.step(entries)
        o = 0
        for e in entries:
            k = len(e["tokens"])
            got[e["id"]].append(out[o:o + k])
            o, at[e["id"]] = o + k, at[e["id"]] + k
    for n in reqs:
        close(torch.cat(got[n]), want[n], tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES[:2])
def test_greedy_generation_through_engine(device, dtype, tol):
    """The engine's scheduler, sampler and (on the GPU) captured decode graphs: two requests of unequal length, greedy tokens equal
    the oracle's argmax continuation; pages and slots come back."""
    cfgd = make_cfg(STACK, dtype=dtype)
    model, sd = make_model(cfgd, device, dtype)
    eng = LLMEngine(LocalPipeline([StageExecutor(model, 16, 16, num_state_slots=4)]), 16, 16, num_groups=1, max_prefill_tokens=11)
    assert eng.table.slots is not None
    free0 = eng.table.slots.num_free
    prompts = [toks(19, seed=21), toks(4, seed=22)]
    rs = [eng.submit(p, SamplingParams(temperature=0.0), max_tokens=6) for p in prompts]
    eng.drain()
    for p, r in zip(prompts, rs):
        assert r.error is None
        seq = list(p)
        for _ in range(6):
            seq.append(int(oracle.forward(cfgd, sd, seq)[-1].argmax()))
        assert r.output == seq[len(p):]
    assert eng.table.alloc.num_free == 15 and eng.table.slots.num_free == free0


def test_config_reader_takes_every_size_from_the_file():
    cfg = ModelConfig.from_dict(make_cfg([D_MH, P_GQ, dict(D_MH, weights_of=0)], width=40, vocab=50, eps=3e-3, mult=0.25, streams=3, scale=7.0))
    assert (cfg.model_type, cfg.hidden_size, cfg.vocab_size, cfg.num_hidden_layers) == ("gokapel", 40, 50, 3)
    assert cfg.rms_norm_eps == 3e-3 and cfg.residual_mult == 0.25 and cfg.streams == 3 and cfg.embedding_scale == 7.0
    assert cfg.layer_specs[2]["weights_of"] == 0 and cfg.layer_specs[1]["mixer"]["left"]["mask"] == dict(size=7)
    assert cfg.layer_specs[0]["mlp"]["router"] == dict(experts=6, top=2, groups=dict(count=3, keep=2))
    with pytest.raises(ValueError):
        ModelConfig.from_dict(make_cfg([dict(type="unknown", mixer=dict(heads=1), mlp=None)]))
    with pytest.raises(ValueError):      # query heads must share key/value heads evenly
        ModelConfig.from_dict(make_cfg([delta(5, 2, 8, 8, 2, None)]))
    with pytest.raises(ValueError):      # the layer whose weights are used must have the same shape
        ModelConfig.from_dict(make_cfg([D_GQ, dict(D_MH, weights_of=0)]))
    with pytest.raises(ValueError):      # more experts wanted than the kept groups hold
        ModelConfig.from_dict(make_cfg([delta(2, 2, 8, 8, 2, dict(kind="moe", router=dict(experts=6, top=3, groups=dict(count=3, keep=1)), expert=dict(ff=8)))]))


def test_cache_layout_and_shared_weights():
    model, sd = make_model(make_cfg(STACK))
    lay = model.cache_layout()
    assert lay[0][0] == "state" and lay[0][1]["S"][0] == (4, 8, 12) and lay[0][1]["conv"][0] == (3, 2 * 2 * 8 + 4 * 12)
    assert lay[1][:4] == ("paged_kv", 2, 8, 12) and lay[1][5]["S"][0] == (20,)
    kv = StageExecutor(model, 4, 16, num_state_slots=3).kv
    assert kv.num_slots == 3 and kv.k[1].shape == (4, 2, 16, 8) and kv.v[3].shape == (4, 1, 16, 40) and kv.state[1]["S"].shape == (3, 20)
    assert kv.k[0] is None and kv.state[4]["S"].data_ptr() != kv.state[0]["S"].data_ptr() and kv.k[5].data_ptr() != kv.k[1].data_ptr()
    assert model.layer_weights[4] is model.layer_weights[0] and model.layer_weights[5] is model.layer_weights[1]
    assert not any(k.startswith("l4.") or k.startswith("l5.") for k in sd)


@pytest.mark.timeout(300)
def test_command_line_generation(tmp_path):
    """``generate.py`` on a synthetic model of the design: tokenizer, engine, sampler and the printed statistics."""
    import subprocess

    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(repo, "generate.py"), "--model", "synthetic:tiny-gokapel", "--prompt", "hello", "--max_tokens", "8",
                        "--device", "cpu", "--no_chat_template"], capture_output=True, text=True, timeout=240,
                       env=dict(os.environ, PYTHONPATH=repo, OMP_NUM_THREADS="1"))
    assert r.returncode == 0, r.stdout + r.stderr
    assert "Generation:" in r.stdout and "tokens-per-sec" in r.stdout
