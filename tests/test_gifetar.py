"""Gifetar (sandwich-norm stack: differential attention with a query temperature and capped scores, mixture-of-experts feed-forwards with
a top-k softmax router) against the plain oracle in ``gifetar_oracle.py``: every mechanism alone, prefill against token-by-token
decoding, prompt portions down to two tokens, ragged batches against each request alone, pages that are freed and used again, far
keys and the steps of the query temperature made visible by scaled weights, other sizes (one key/value head, as many as query heads,
value widths beyond one register set, head sizes off the 16-byte path, top-1 and all-experts routers, a layer without feed-forward),
long decoding over split keys, and greedy generation through the engine.

Runs on the CPU with the unfused ops; the ``gpu`` variants run the same cases on the sm_100a kernels in fp32 and bf16.
"""
import copy
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import gifetar_oracle as oracle  # noqa: E402

from mlx_sharding_b200.config import ModelConfig  # noqa: E402
from mlx_sharding_b200.engine.core import LLMEngine  # noqa: E402
from mlx_sharding_b200.engine.sampler import SamplingParams  # noqa: E402
from mlx_sharding_b200.engine.trace import TraceSession  # noqa: E402
from mlx_sharding_b200.models import build_stage  # noqa: E402
from mlx_sharding_b200.ops import BatchMeta, get_backend  # noqa: E402
from mlx_sharding_b200.parallel.pipeline import LocalPipeline, StageExecutor  # noqa: E402
from mlx_sharding_b200.utils.checkpoint import random_state_dict  # noqa: E402

MOE = dict(kind="moe", router=dict(experts=5, top=2), expert=dict(ff=24))
MOE_TOP1 = dict(kind="moe", router=dict(experts=4, top=1), expert=dict(ff=16))          # one expert, weight exactly 1
MOE_ALL = dict(kind="moe", router=dict(experts=3, top=3), expert=dict(ff=8))            # every expert chosen: a plain softmax gate


def attn(heads, kv_heads, dim, vdim, scale, softcap, diff, coef, every, mlp=MOE):
    return dict(type="attention", mixer=dict(diff=diff, dim=dim, heads=heads, kv_heads=kv_heads, q_temp=dict(coef=coef, every=every),
                                             scale=scale, softcap=softcap, vdim=vdim), mlp=copy.deepcopy(mlp))


GQA = attn(6, 2, 8, 12, 0.4, 4.0, 0.3, 0.7, 7)                      # three query heads per key/value head; temperature steps every 7
MQA = attn(3, 1, 16, 40, 0.2, 30.0, 0.6, 0.25, 16, MOE_TOP1)        # one key/value head
MHA = attn(3, 3, 6, 10, 0.5, 2.0, 0.45, 1.5, 5, MOE_ALL)            # as many key/value heads as query heads; head sizes off the 16-byte path
WIDE = attn(10, 1, 8, 160, 0.3, 8.0, 0.2, 0.4, 32, None)            # ten heads on one key/value head (two CTAs), wide values, no feed-forward
STACK = [GQA, MQA, MHA, WIDE]
CASES = {"gqa_moe": [GQA], "mqa_top1": [MQA], "mha_all_experts": [MHA], "wide_no_ff": [WIDE], "stack": STACK}
DEVICES = [pytest.param("cpu", torch.float32, 2e-4, id="cpu"),
           pytest.param("cuda", torch.float32, 2e-4, id="b200-f32", marks=pytest.mark.gpu),
           pytest.param("cuda", torch.bfloat16, 6e-2, id="b200-bf16", marks=pytest.mark.gpu)]


def make_cfg(layers, width=48, vocab=96, eps=1e-3, mult=0.7):
    return dict(architecture="Gifetar", layers=copy.deepcopy(layers), norm=dict(eps=eps), residual_mult=mult, vocab=vocab, width=width)


def make_model(cfgd, device="cpu", dtype=torch.float32, seed=3, edit=None):
    cfg = ModelConfig.from_dict(cfgd)
    sd = dict(random_state_dict(cfg, dtype=torch.bfloat16, seed=seed))
    if edit:
        edit(sd)
    model = build_stage(cfg, None, dtype, device).load_state({k: v.clone() for k, v in sd.items()})
    return model, sd


def session(model, pages=12, page_size=16, live=4):
    return TraceSession(StageExecutor(model, pages, page_size), (pages - 1) * page_size, live)


def run_whole(model, tokens, **kw):
    return session(model, **kw).step([dict(id="a", tokens=tokens, want=list(range(len(tokens))))])


def toks(n, vocab=96, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def pick(cfgd, sd, dtype, make, seed, gap=0.08, tries=200):
    """Tokens ``make(seed)``.  In bf16 a router logit moves by about a hundredth, so a test that compares with exact arithmetic must
    not rest on a routing decision closer than that: other seeds are tried until the oracle's routing has no close call."""
    if dtype != torch.bfloat16:
        return make(seed)
    for i in range(tries):
        t = make(seed + 1000 * i)
        if oracle.min_router_gap(cfgd, sd, t) > gap:
            return t
    raise AssertionError("no sequence without a close routing call found")


SHOWS = 1e-2      # a fault must move the logits by this share of their largest: 50 times the exact-mode tolerance (bf16 runs are less sharp)


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
    """Each layer shape alone (and the mixed stack): whole prompt, every position; 45 tokens span three 16-token pages and several
    steps of every query temperature."""
    cfgd = make_cfg(CASES[case])
    model, sd = make_model(cfgd, device, dtype)
    t = pick(cfgd, sd, dtype, lambda s: toks(45, seed=s), 0)
    close(run_whole(model, t), oracle.forward(cfgd, sd, t), tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_ops_alone(device, dtype, tol):
    """The new ops one by one against the oracle's functions, on inputs of their own: layer norm with bias, the fused residual step, the
    router, the differential attention over pools that were filled in two steps."""
    O = get_backend("b200" if device == "cuda" else "reference")
    g = torch.Generator().manual_seed(5)
    rn = lambda *s: torch.randn(*s, generator=g)
    x, y, w, b, w2, b2 = rn(7, 40) * 3 + 1, rn(7, 40), 1 + 0.2 * rn(40), rn(40), 1 + 0.2 * rn(40), rn(40)
    dev = lambda t: t.to(device)
    close(O.layernorm_cast(dev(x), dev(w), dev(b), 1e-3, dtype), oracle.layer_norm(x.double(), w.double(), b.double(), 1e-3), tol)
    xs = dev(x.clone())
    xa = O.post_layernorm_add_norm_(xs, dev(y), dev(w), dev(b), 0.3, dev(w2), dev(b2), 1e-3, dtype)
    want = x.double() + 0.3 * oracle.layer_norm(y.double(), w.double(), b.double(), 1e-3)
    close(xs, want, 1e-5)                                                              # the residual stream itself stays fp32
    close(xa, oracle.layer_norm(want, w2.double(), b2.double(), 1e-3), tol)
    z, zb = rn(9, 6), rn(6)
    idx, wt = O.softmax_topk(dev(z), dev(zb), 6, 3)
    val, ref = torch.topk(z + zb, 3, -1)
    assert torch.equal(idx.cpu().long(), ref)
    close(wt, torch.softmax(val, -1), 1e-5)
    assert torch.allclose(wt.sum(-1).cpu(), torch.ones(9), atol=1e-5)
    # attention: 2 key/value heads, 4 query heads, 21 tokens written as 13 + 8 into 8-token pages in scrambled order
    H, G, D, V, n = 4, 2, 8, 12, 21
    rows = (rn(n, (H + G) * 2 * D + G * V)).to(dtype)
    kp, vp = torch.zeros(6, G, 8, 2 * D, dtype=dtype, device=device), torch.zeros(6, G, 8, V, dtype=dtype, device=device)
    pages, outs = [4, 1, 5], []
    for lo, hi in ((0, 13), (13, 21)):
        meta = BatchMeta.build([hi - lo], [lo], [pages], 8, device=device)
        r = dev(rows[lo:hi])
        O.paged_kv_append(r, H * 2 * D, (H + G) * 2 * D, kp, vp, meta)
        outs.append(O.diff_attention(r, kp, vp, meta, H, 0.35, 3.0, 0.5, 4.0, 0.6, 1e-3, 0.8, dtype))
    rd = rows.double()
    q = rd[:, :H * 2 * D].view(n, H, 2, D) * oracle.query_temperature(torch.arange(n, dtype=torch.float64), 0.5, 4.0).view(n, 1, 1, 1)
    k, v = rd[:, H * 2 * D:(H + G) * 2 * D].view(n, G, 2, D), rd[:, (H + G) * 2 * D:].view(n, G, V)
    want = torch.zeros(n, H, V, dtype=torch.float64)
    mask = torch.tril(torch.ones(n, n, dtype=torch.bool))
    for h in range(H):
        a = [torch.softmax(oracle.capped(q[:, h, c] @ k[:, h // 2, c].T * 0.35, 3.0).masked_fill(~mask, float("-inf")), -1) @ v[:, h // 2] for c in range(2)]
        want[:, h] = oracle.unit_rms(a[0] - 0.6 * a[1], 1e-3) * 0.8
    close(torch.cat(outs), want.view(n, H * V), tol if dtype == torch.bfloat16 else 1e-5)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
@pytest.mark.parametrize("experts,top,ff,rows", [(5, 2, 24, 7), (4, 1, 16, 3), (3, 3, 8, 70), (6, 2, 128, 150)])
def test_experts_alone(experts, top, ff, rows, device, dtype, tol):
    """Router and routed experts as ops against the oracle's feed-forward: few rows (one weight-row read per pair), many rows (sorted
    rows, one product per expert; expert rows of 128 take the grouped tensor-core GEMM in bf16), top-1 (weight exactly 1), all experts."""
    from mlx_sharding_b200.ops import LinearWeight

    O = get_backend("b200" if device == "cuda" else "reference")
    K = 128
    g = torch.Generator().manual_seed(experts * 100 + rows)
    rn = lambda *s: torch.randn(*s, generator=g)
    bank = lambda o, i: (rn(experts, o, i) * i ** -0.5).bfloat16()
    wg, wu, wd, wr, br = bank(ff, K), bank(ff, K), bank(K, ff), (rn(experts, K) * 3 * K ** -0.5).bfloat16(), (0.2 * rn(experts)).bfloat16()
    p = {"router": wr.double(), "router.b": br.double()}
    for e in range(experts):
        p.update({f"e{e}.gate": wg[e].double(), f"e{e}.up": wu[e].double(), f"e{e}.down": wd[e].double()})
    mlp = dict(router=dict(experts=experts, top=top))
    for seed in range(200):                  # the router sees the same bf16-exact inputs as the oracle: only a near-tie could flip a choice
        x = torch.randn(rows, K, generator=torch.Generator().manual_seed(seed)).bfloat16()
        gaps = []
        want = oracle.moe_ff(x.double(), p, mlp, gaps)
        if not gaps or gaps[0] > 1e-3:
            break
    else:
        raise AssertionError("no input without a close routing call found")
    dev = lambda t: t.to(device=device, dtype=dtype)
    lw = lambda t: LinearWeight(weight=dev(t).contiguous())
    xa = dev(x)
    idx, wt = O.softmax_topk(O.router_logits(xa, wr.float().to(device)), br.float().to(device), experts, top)
    assert torch.allclose(wt.sum(-1).cpu(), torch.ones(rows), atol=1e-5)
    close(O.moe_glu_experts(xa, idx, wt, lw(wg), lw(wu), lw(wd)), want, tol if dtype == torch.bfloat16 else 1e-5)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_first_tokens_and_single_token(device, dtype, tol):
    cfgd = make_cfg(STACK)
    model, sd = make_model(cfgd, device, dtype)
    for t in ([5], pick(cfgd, sd, dtype, lambda s: toks(2, seed=s), 4), pick(cfgd, sd, dtype, lambda s: toks(3, seed=s), 5)):
        close(run_whole(model, t), oracle.forward(cfgd, sd, t), tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
@pytest.mark.parametrize("portions", [[1] * 23, [2, 2, 2, 17], [16, 7], [15, 1, 1, 6], [3, 13, 7], [22, 1], [8, 9, 6]])
def test_portions_equal_whole(portions, device, dtype, tol):
    """Prefill against token-by-token decoding and prompts cut anywhere (page edge at 16, temperature steps at 4, 6, 13, 15, ...,
    2-token portions)."""
    cfgd = make_cfg(STACK)
    model, sd = make_model(cfgd, device, dtype)
    t = pick(cfgd, sd, dtype, lambda s: toks(sum(portions), seed=s), 1)
    want = oracle.forward(cfgd, sd, t)
    s, at, got = session(model), 0, []
    for n in portions:
        got.append(s.step([dict(id="r", tokens=t[at:at + n], want=list(range(n)))]))
        at += n
    close(torch.cat(got), want, tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_ragged_batch_and_reuse_of_pages(device, dtype, tol):
    """Unequal requests in one batch (portions beside single tokens) equal each alone; a pool of 5 pages serves 4 requests one pair
    after another, so every page is used again — by a request that must not see what the last one left."""
    cfgd = make_cfg(STACK)
    model, sd = make_model(cfgd, device, dtype)
    reqs = {n: pick(cfgd, sd, dtype, lambda s, L=L: toks(L, seed=s), 10 + i) for i, (n, L) in enumerate([("a", 30), ("b", 9), ("c", 17), ("d", 33)])}
    want = {n: oracle.forward(cfgd, sd, t) for n, t in reqs.items()}
    s = session(model, pages=6, page_size=16, live=2)
    assert s.table.slots is None                       # no recurrent layer: sequences hold pages only
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
    assert s.table.alloc.num_free == 5
    step([("d", 0, 2), ("c", 0, 16)])
    step([("c", 16, 17), ("d", 2, 33)], end=["c", "d"])
    for n in reqs:
        close(torch.cat(got[n]), want[n], tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_temperature_steps_show(device, dtype, tol):
    """The query temperature jumps where floor((p + 1) / every) does: with every = 7 at positions 6, 13, 20, ...  Sharp queries make
    the jump visible: a temperature that stepped one position early or late would move the logits there far beyond the tolerance.  In a
    prompt and decoded one by one, across a page edge."""
    layer = attn(2, 1, 8, 12, 0.5, 25.0, 0.3, 2.0, 7, None)
    cfgd = make_cfg([layer])
    model, sd = make_model(cfgd, device, dtype, edit=lambda sd: sd["l0.mix.q"].mul_(3.0))
    t = toks(30, seed=7)
    want = oracle.forward(cfgd, sd, t)
    for every, p in ((6, 5), (8, 6)):                 # one earlier: position 5 already stepped; one later: position 6 not yet
        other = copy.deepcopy(cfgd)
        other["layers"][0]["mixer"]["q_temp"]["every"] = every
        assert (oracle.forward(other, sd, t)[p] - want[p]).abs().max() > SHOWS * want.abs().max()
    close(run_whole(model, t), want, tol)
    close(decode_after(model, t, 4), want, tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_far_key_and_capped_scores(device, dtype, tol):
    """Sharp queries (the query weights are scaled) make single keys stand out: a sequence is sought in which a query beyond position 50
    rests on the key at position 1, four pages back — changing that one token moves the late logits far beyond the tolerance — and in
    which the scores run into the cap.  In a prompt and in decoding."""
    cfgd = make_cfg([attn(4, 2, 8, 12, 0.5, 6.0, 0.3, 0.3, 16, None)])
    model, sd = make_model(cfgd, device, dtype, edit=lambda sd: sd["l0.mix.q"].mul_(4.0))
    nocap = copy.deepcopy(cfgd)
    nocap["layers"][0]["mixer"]["softcap"] = 60.0
    for seed in range(40):
        t = toks(64, seed=100 + seed)
        want = oracle.forward(cfgd, sd, t)
        lost = list(t)
        lost[1] = (t[1] + 1) % 96                     # another token far back: the logits where it is sought move
        need = 5 * SHOWS * want.abs().max()
        if (oracle.forward(cfgd, sd, lost)[50:] - want[50:]).abs().max() > need and (oracle.forward(nocap, sd, t)[50:] - want[50:]).abs().max() > need:
            break
    else:
        raise AssertionError("no sequence found in which a far key and the cap show")
    close(run_whole(model, t, pages=8), want, tol)
    close(decode_after(model, t, 50, pages=8), want, tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_lambda_and_head_norm_show(device, dtype, tol):
    """Large lambda vectors: the second map's weight differs much from ``diff`` alone, and the per-head norm sees a difference of
    nearly equal maps (small values over eps)."""
    def edit(sd):
        sd["l0.mix.lq1"].fill_(0.5); sd["l0.mix.lk1"].fill_(0.5)          # exp(8 * 0.25) = e^2
        sd["l0.mix.lq2"].fill_(-0.25); sd["l0.mix.lk2"].fill_(0.5)        # exp(-1)

    cfgd = make_cfg([attn(4, 2, 8, 12, 0.3, 20.0, 0.1, 0.0, 1, MOE)], eps=1e-2)
    model, sd = make_model(cfgd, device, dtype, edit=edit)
    t = pick(cfgd, sd, dtype, lambda s: toks(20, seed=s), 3)
    want = oracle.forward(cfgd, sd, t)
    plain = {k: (torch.zeros_like(v) if ".mix.l" in k else v) for k, v in sd.items()}
    assert (oracle.forward(cfgd, plain, t) - want).abs().max() > 5 * SHOWS * want.abs().max()
    close(run_whole(model, t), want, tol)
    close(decode_after(model, t, 9), want, tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_long_prompt_then_decode(device, dtype, tol):
    """A 290-token prompt (on the GPU a single long portion takes the matrix-product form of the attention), then single tokens whose
    keys are split over CTAs and merged."""
    cfgd = make_cfg([dict(GQA, mlp=MOE_ALL), WIDE, dict(MQA, mlp=None)])     # every expert chosen: no routing call that bf16 could flip
    model, sd = make_model(cfgd, device, dtype)
    t = toks(296, seed=9)
    want = oracle.forward(cfgd, sd, t)
    s = session(model, pages=21)
    rows = [0, 5, 6, 7, 31, 32, 100, 127, 128, 289]
    got = [s.step([dict(id="r", tokens=t[:290], want=rows)])] + [s.step([dict(id="r", tokens=[x], want=[0])]) for x in t[290:]]
    close(torch.cat(got), torch.cat([want[rows], want[290:]]), tol * (3 if dtype == torch.bfloat16 else 1))


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_long_decode(device, dtype, tol):
    """150 single-token steps after a 3-token prompt: the pools grow page by page while the temperature steps on."""
    cfgd = make_cfg([GQA, MHA])
    model, sd = make_model(cfgd, device, dtype)
    t = pick(cfgd, sd, dtype, lambda s: toks(153 if dtype != torch.bfloat16 else 60, seed=s), 5, gap=0.05, tries=400)
    close(decode_after(model, t, 3), oracle.forward(cfgd, sd, t), tol * (3 if dtype == torch.bfloat16 else 1))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 6e-2)])
def test_tensor_core_sizes(dtype, tol):
    """Width and expert rows that are multiples of 128, head sizes that are multiples of 8: bf16 takes the tensor-core GEMMs for the
    projections, the prefill attention and the grouped experts (a 40-token prompt: sorted rows; single tokens: one weight-row read per
    pair in exact mode)."""
    moe = dict(kind="moe", router=dict(experts=6, top=2), expert=dict(ff=128))
    cfgd = make_cfg([attn(4, 2, 16, 32, 0.25, 10.0, 0.3, 0.5, 8, moe), attn(4, 4, 8, 24, 0.35, 10.0, 0.2, 0.5, 8, moe)], width=128)
    model, sd = make_model(cfgd, "cuda", dtype)
    t = pick(cfgd, sd, dtype, lambda s: toks(44, seed=s), 2, gap=0.05, tries=400)
    close(decode_after(model, t, 40), oracle.forward(cfgd, sd, t), tol)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 6e-2)])
def test_wide_values_long_context(dtype, tol):
    """Value widths of 128 and 256 (the attention kernel's 16-byte shared-memory path, one and two register groups per lane) over a
    context long enough that the keys of a decoded token are split over CTAs; prompt portions of 2 to 31 tokens run the same kernel on
    many rows."""
    cfgd = make_cfg([attn(4, 2, 16, 128, 0.25, 10.0, 0.3, 0.5, 64, None), attn(2, 1, 8, 256, 0.35, 10.0, 0.2, 0.5, 100, MOE_ALL)], width=64)
    model, sd = make_model(cfgd, "cuda", dtype)
    t = toks(300, seed=13)
    want = oracle.forward(cfgd, sd, t)
    for pages, page_size in ((21, 16), (7, 64)):           # a tile of 32 keys spans two pages / lies within one
        s, at, got = session(model, pages=pages, page_size=page_size), 0, []
        for n in [256, 2, 31, 5] + [1] * 6:
            got.append(s.step([dict(id="r", tokens=t[at:at + n], want=list(range(n)))]))
            at += n
        close(torch.cat(got), want, tol * (3 if dtype == torch.bfloat16 else 1))


@pytest.mark.parametrize("device,dtype,tol", DEVICES[:2])
def test_greedy_generation_through_engine(device, dtype, tol):
    """The engine's scheduler, sampler and (on the GPU) captured decode graphs: two requests of unequal length, greedy tokens equal
    the oracle's argmax continuation."""
    cfgd = make_cfg(STACK)
    model, sd = make_model(cfgd, device, dtype)
    eng = LLMEngine(LocalPipeline([StageExecutor(model, 16, 16)]), 16, 16, num_groups=1, max_prefill_tokens=11)
    assert eng.table.slots is None
    prompts = [toks(19, seed=21), toks(4, seed=22)]
    rs = [eng.submit(p, SamplingParams(temperature=0.0), max_tokens=6) for p in prompts]
    eng.drain()
    for p, r in zip(prompts, rs):
        assert r.error is None
        seq = list(p)
        for _ in range(6):
            seq.append(int(oracle.forward(cfgd, sd, seq)[-1].argmax()))
        assert r.output == seq[len(p):]
    assert eng.table.alloc.num_free == 15


def test_config_reader_takes_every_size_from_the_file():
    cfg = ModelConfig.from_dict(make_cfg([GQA, WIDE, MHA], width=40, vocab=50, eps=3e-3, mult=0.25))
    assert (cfg.model_type, cfg.hidden_size, cfg.vocab_size, cfg.num_hidden_layers) == ("gifetar", 40, 50, 3)
    assert cfg.rms_norm_eps == 3e-3 and cfg.residual_mult == 0.25 and cfg.layer_specs[1]["mlp"] is None
    assert cfg.layer_specs[0]["mixer"]["q_temp"] == dict(coef=0.7, every=7) and cfg.layer_specs[2]["mlp"]["router"] == dict(experts=3, top=3)
    with pytest.raises(ValueError):
        ModelConfig.from_dict(make_cfg([dict(type="unknown", mixer=dict(heads=1), mlp=None)]))
    with pytest.raises(ValueError):      # query heads must share key/value heads evenly
        ModelConfig.from_dict(make_cfg([attn(5, 2, 8, 8, 0.3, 0.0, 0.1, 0.0, 1, None)]))
    with pytest.raises(ValueError):
        ModelConfig.from_dict(make_cfg([attn(2, 1, 8, 8, 0.3, 0.0, 0.1, 0.0, 1, dict(kind="dense", ff=8))]))


def test_cache_layout_has_pools_of_each_layers_own_sizes():
    model, _ = make_model(make_cfg(STACK))
    assert [e[:4] for e in model.cache_layout()] == [("paged_kv", 2, 16, 12), ("paged_kv", 1, 32, 40), ("paged_kv", 3, 12, 10), ("paged_kv", 1, 16, 160)]
    kv = StageExecutor(model, 4, 16).kv
    assert kv.num_slots == 0 and kv.k[1].shape == (4, 1, 16, 32) and kv.v[3].shape == (4, 1, 16, 160)


@pytest.mark.timeout(300)
def test_command_line_generation(tmp_path):
    """``generate.py`` on a synthetic model of the design: tokenizer, engine, sampler and the printed statistics."""
    import subprocess

    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(repo, "generate.py"), "--model", "synthetic:tiny-gifetar", "--prompt", "hello", "--max_tokens", "8",
                        "--device", "cpu", "--no_chat_template"], capture_output=True, text=True, timeout=240,
                       env=dict(os.environ, PYTHONPATH=repo, OMP_NUM_THREADS="1"))
    assert r.returncode == 0, r.stdout + r.stderr
    assert "Generation:" in r.stdout and "tokens-per-sec" in r.stdout
