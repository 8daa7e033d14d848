"""Porovik on the GPU: every mechanism's kernels against the plain implementation's function for it, then
whole models through the engine's step function, cache and state slots, scheduler and entry point."""
import math

import numpy as np
import pytest
import torch

import plain_porovik as P
import replay_util as R
from tiny_porovik import TINY, load_folder, write_tiny

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def K():
    from rosellm_b200.ops import kernels

    return kernels


def rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double().cpu() - b.double().cpu()).abs().max() / (b.double().abs().max() + 1e-30))


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


# ---- mechanisms alone ------------------------------------------------------------------------------

def test_pair_embedding_over_portions_and_reused_slots():
    """The previous token of a portion's first token comes from the slot's state; a sequence's first
    token takes row ``buckets``; a slot that is taken again starts anew when its state was zeroed."""
    from rosellm_b200.engine.context import build_host_batch

    g = torch.Generator().manual_seed(1)
    vocab, hidden, buckets, mp, mc = 50, 24, 37, 11, 3
    table, pair, pos = (torch.randn(n, hidden, generator=g) for n in (vocab, buckets + 1, 64))
    state = torch.full((4, 1), 7, dtype=torch.int32, device=DEV)  # stale tokens of earlier owners
    seqs = {1: torch.randint(0, vocab, (23,), generator=g).tolist(), 3: torch.randint(0, vocab, (9,), generator=g).tolist(),
            0: [5]}
    done = {s: 0 for s in seqs}
    got = {s: [] for s in seqs}
    for cut in ([(1, 7), (3, 1), (0, 1)], [(3, 2), (1, 1)], [(1, 15), (3, 6)]):
        hb = build_host_batch([(s, done[s], seqs[s][done[s]:done[s] + n], []) for s, n in cut])
        out = torch.empty(len(hb.token_ids), hidden, device=DEV)
        K().embed_pair(dev(hb.token_ids), dev(hb.positions), dev(hb.req_of_token), dev(hb.q_start), dev(hb.slots),
                       table.to(DEV), pos.to(DEV), pair.to(DEV), out, state, buckets=buckets, mul_prev=mp, mul_cur=mc)
        at = 0
        for s, n in cut:
            got[s].append(out[at:at + n].cpu())
            at += n
            done[s] += n
    K().check_status(torch.device(DEV))
    for s, toks in seqs.items():
        want = P.embed(toks, table.double(), pair.double(), pos.double(), buckets, mp, mc)
        assert rel(torch.cat(got[s]), want) < 1e-6
        assert int(state[s, 0]) == toks[-1]


@pytest.mark.parametrize("width", [8, 100, 1000])
def test_norm_with_scales_around_zero_and_the_fused_pair(width):
    from rosellm_b200.parts.standard import RMSNorm

    g = torch.Generator().manual_seed(width)
    y, x = torch.randn(5, width, generator=g) * 3, torch.randn(5, width, generator=g)
    w1, w2 = torch.randn(width, generator=g) * 0.2, torch.randn(width, generator=g) * 0.2
    a, b = RMSNorm(width, 1e-5, weight_offset=1.0), RMSNorm(width, 1e-3, weight_offset=1.0)
    a.bind({"weight": w1.to(DEV)})
    b.bind({"weight": w2.to(DEV)})
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 6e-3)):
        xs, nxt = x.to(DEV).clone(), torch.empty(5, width, dtype=dtype, device=DEV)
        K().rmsnorm_add_norm(y.to(DEV), a.weight, a.eps, xs, b.weight, b.eps, nxt)
        want_x = x.double() + P.norm(y.double(), w1.double(), 1e-5)
        assert rel(xs, want_x) < 1e-6
        assert rel(nxt.float(), P.norm(want_x, w2.double(), 1e-3)) < tol


def _attention_case(dtype, H, G, dk, dv, lens_new, lens_old, page, scale, temp, seed, stand_out=None, gate=True, splits=1,
                    mma=False):
    """Requests with ``lens_old`` cached tokens bring ``lens_new`` more.  The cache rows of all tokens are
    written by the store kernel (old tokens in a step of their own); returns the kernel's output
    [tokens, H, dv] and the plain result from the same (rounded) keys and values."""
    from rosellm_b200.engine.context import build_host_batch
    from rosellm_b200.parts.biased import distance_slopes

    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(seed)
    v_at = -(-dk // 8) * 8
    row = -(-(v_at + dv) // 8) * 8
    n_req = len(lens_new)
    totals = [a + b for a, b in zip(lens_new, lens_old)]
    pages_per = [-(-t // page) for t in totals]
    n_pages = sum(pages_per) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((n_req + 1, max(pages_per)), -1, dtype=torch.int32)
    at = 0
    for r in range(n_req):
        for lp in range(pages_per[r]):
            table[r + 1, lp] = order[at]
            at += 1
    table = table.to(DEV)
    pool = torch.full((n_pages, 1, G, page, row), 9.0, dtype=dt, device=DEV)
    ks = [torch.randn(t, G, dk, generator=g) * 0.7 for t in totals]
    vs = [torch.randn(t, G, dv, generator=g) for t in totals]
    n_tok = sum(lens_new)
    q = torch.randn(n_tok, H, dk, generator=g) * 0.8
    if stand_out is not None:  # request 0's last query points at one far key, hard enough to beat its distance
        key, head = stand_out
        ks[0][key, head // (H // G)] = q[lens_new[0] - 1, head] * 40.0
    # cached tokens first, then the step's own
    for new, old in ((lens_old, [0] * n_req), (lens_new, lens_old)):
        ents = [(r + 1, old[r], [0] * new[r], []) for r in range(n_req) if new[r] > 0]
        if not ents:
            continue
        hb = build_host_batch(ents)
        kk = torch.cat([ks[r][old[r]:old[r] + new[r]] for r in range(n_req) if new[r] > 0]).reshape(-1, G * dk)
        vv = torch.cat([vs[r][old[r]:old[r] + new[r]] for r in range(n_req) if new[r] > 0]).reshape(-1, G * dv)
        K().bias_kv_store(kk.to(DEV), vv.to(DEV), pool, table, dev(hb.positions), dev(hb.req_of_token), dev(hb.slots),
                          v_at=v_at, max_pos=max(totals))
    slopes = distance_slopes(H, 8.0)
    gate_t = torch.randn(n_tok, H * dv, generator=g) if gate else None
    mma = mma and K().bias_attention_tensor_cores(dt, dk, dv)
    wide = K().bias_attention_shape(H // G, mma)[1] > 16
    tiles, n_tiles = (hb.tiles_wide, len(hb.tiles_wide)) if wide else (hb.tiles, len(hb.tiles))
    out = torch.full((n_tok, H * dv), 5.0, dtype=dt, device=DEV)
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.full((len(hb.decode_reqs) * H * splits, dv), float("nan"), device=DEV)
        part_ml = torch.full((len(hb.decode_reqs) * H * splits, 2), float("nan"), device=DEV)
    K().bias_attention(q.reshape(n_tok, H * dk).to(DEV), None if gate_t is None else gate_t.to(DEV), pool, table,
                       dev(hb.q_start), dev(hb.kv_len), dev(hb.slots), out, n_heads=H, dk=dk, dv=dv, v_at=v_at, scale=scale,
                       slopes=slopes.to(DEV), temp_coef=temp[0], temp_every=temp[1], tiles=dev(tiles.reshape(-1)),
                       n_tiles=n_tiles, tile_tokens=64 if wide else 16, decode_reqs=dev(hb.decode_reqs),
                       n_decode=len(hb.decode_reqs), max_pos=max(totals), n_splits=splits, part_o=part_o, part_ml=part_ml,
                       tensor_cores=mma)
    K().check_status(torch.device(DEV))
    want = torch.empty(n_tok, H, dv, dtype=torch.float64)
    t0 = 0
    for r in range(n_req):
        kc, vc = ks[r].to(dt).double(), vs[r].to(dt).double()  # what the cache holds
        qq = torch.zeros(totals[r], H, dk, dtype=torch.float64)
        qq[lens_old[r]:] = q[t0:t0 + lens_new[r]].double()
        o = P.attention(qq, kc, vc, scale, slopes.double(), P.query_temperature(totals[r], *temp))[lens_old[r]:]
        if gate_t is not None:
            o = o * torch.sigmoid(gate_t[t0:t0 + lens_new[r]].double()).view(-1, H, dv)
        want[t0:t0 + lens_new[r]] = o
        t0 += lens_new[r]
    assert torch.all(pool[..., v_at + dv:] == 9.0) and torch.all(pool[..., dk:v_at] == 9.0)  # the fill is not written
    return out.float().cpu().view(n_tok, H, dv), want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_biased_attention_prompt_portions_and_single_tokens(dtype):
    """Portions that start inside a page and end on a page's border, of one to 40 tokens, beside single
    tokens; groups of three and of forty heads a key/value head, as many key/value heads as heads; a
    query temperature that steps inside the portions."""
    for mma in ((False,) if dtype == "float32" else (False, True)):
        # with bfloat16 operands on the tensor cores the queries and the probabilities are rounded too
        tol = 2e-5 if dtype == "float32" else (2.5e-2 if mma else 1e-2)
        for H, G, dk, dv, page, temp in ((6, 2, 20, 10, 16, (0.7, 16)), (4, 4, 64, 32, 8, (0.0, 0)), (40, 1, 8, 8, 32, (0.1, 1)),
                                         (5, 1, 16, 72, 8, (1.5, 33)), (2, 1, 130, 136, 16, (0.3, 7)), (16, 4, 128, 128, 16, (0.5, 50)),
                                         (80, 1, 24, 40, 16, (0.2, 9))):
            got, want = _attention_case(dtype, H, G, dk, dv, [40, 1, 2, 17, 1, 16], [5, 130, 0, 15, 0, 16], page, 0.3, temp, seed=H,
                                        mma=mma)
            assert rel(got, want) < tol, (H, G, dk, dv, mma)
            got, want = _attention_case(dtype, H, G, dk, dv, [33, 16, 2, 70], [0, 31, 70, 63], page, 0.2, temp, seed=H + 9, gate=False,
                                        mma=mma)
            assert rel(got, want) < tol, (H, G, dk, dv, mma, "portions only")
            got, want = _attention_case(dtype, H, G, dk, dv, [1, 1, 1], [0, 31, 32], page, 0.2, temp, seed=H + 50, mma=mma)
            assert rel(got, want) < tol, (H, G, dk, dv, mma, "single tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("splits", [2, 3, 8, 32])
def test_decoded_tokens_with_keys_cut_into_parts(dtype, splits):
    """More parts than a short request has tiles of keys (empty parts), parts that end inside a tile, beside a
    prompt portion that is not cut."""
    tol = 2e-5 if dtype == "float32" else 1e-2
    got, want = _attention_case(dtype, 6, 2, 20, 10, [1, 1, 5, 1, 1], [700, 0, 40, 63, 64], 16, 0.25, (0.7, 16), seed=splits,
                                splits=splits)
    assert rel(got, want) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", [0, 15, 16, 17, 511, 512, 897])
def test_a_far_key_that_stands_out_is_found(dtype, key):
    """Among 900 cached keys one is scored far above the rest for the head with the smallest slope: the
    output must be (nearly) that key's value, whether it is the first, sits at a page's border or far
    back; from a prompt portion's query and from a decoded token's."""
    for new, old, splits, mma in (([4], [896], 1, False), ([4], [896], 1, True), ([1], [899], 1, False), ([1], [899], 5, False)):
        got, want = _attention_case(dtype, 4, 2, 24, 12, new, old, 16, 0.5, (0.0, 0), seed=key, stand_out=(key, 3), gate=False,
                                    splits=splits, mma=mma)
        assert rel(got, want) < (2e-5 if dtype == "float32" else 2.5e-2)


def test_distance_bias_and_temperature_enter_the_scores():
    """One key at every distance with equal q.k: the weights fall off as exp(-slope * distance), and the
    temperature multiplies q.k only from the position where floor((p + 1) / every) changes."""
    slopes = P.distance_slopes(4)
    assert torch.allclose(slopes, torch.tensor([0.25, 0.0625, 0.015625, 0.00390625], dtype=torch.float64))
    t = P.query_temperature(10, 0.5, 4)
    assert torch.allclose(t[:3], torch.ones(3, dtype=torch.float64)) and abs(float(t[3]) - (1 + 0.5 * math.log(2))) < 1e-12
    assert abs(float(t[7]) - (1 + 0.5 * math.log(3))) < 1e-12
    got, want = _attention_case("float32", 4, 1, 8, 8, [9], [0], 4, 0.7, (0.5, 4), seed=3)
    assert rel(got, want) < 2e-5


def _recurrence_case(mode, dtype, H, dk, dv, lens, cuts, seed, rank=4):
    """Requests of ``lens`` tokens run through the kernel in steps of ``cuts`` tokens each (the state carried
    in slots, which start with another owner's leftovers zeroed); compares with the plain recurrence."""
    from rosellm_b200.engine.context import build_host_batch

    g = torch.Generator().manual_seed(seed)
    dt = DTYPES[dtype]
    n_req = len(lens)
    wk, wv = H * dk, H * dv
    if mode == "delta":
        names, widths = ("r", "k", "v", "a", "g", "w"), (wk, wk, wv, wk, wv, rank)
    else:
        names, widths = ("r", "a", "v"), (wk, wk, wv)
    offs, at = {}, 0
    for nme, w in zip(names, widths):
        offs[nme] = at
        at += -(-w // 8) * 8
    total_w = at
    proj = [torch.randn(n, total_w, generator=g) for n in lens]
    a_bias, w0 = torch.randn(wk, generator=g), torch.randn(wk, generator=g)
    if mode == "gated":
        w0 = torch.rand(wk, generator=g) * 0.9
    w2 = torch.randn(wk, rank, generator=g)
    out_w = 1 + 0.3 * torch.randn(wv if mode == "delta" else dv, generator=g)
    state = torch.zeros(n_req + 1, H, dk, dv, device=DEV)
    got = [[] for _ in lens]
    done = [0] * n_req
    k = 0
    while any(d < n for d, n in zip(done, lens)):
        ents, take = [], []
        for r in range(n_req):
            if done[r] < lens[r]:
                n = min(cuts[k % len(cuts)], lens[r] - done[r])
                k += 1
                ents.append((r + 1, done[r], [0] * n, []))
                take.append((r, n))
        hb = build_host_batch(ents)
        pj = torch.cat([proj[r][done[r]:done[r] + n] for r, n in take]).to(DEV)
        out = torch.full((pj.shape[0], wv), 3.0, dtype=dt, device=DEV)
        kw = dict(n_reqs=len(ents), n_heads=H, dk=dk, dv=dv, eps=1e-5, a_bias=a_bias.to(DEV), w0=w0.to(DEV),
                  out_weight=out_w.to(DEV))
        if mode == "delta":
            kw.update(w2t=w2.t().contiguous().to(DEV), rank=rank, decay_scale=math.exp(-0.5), unit_eps=1e-6)
        m = K().RECURRENCES[mode]
        prep = torch.full((H * pj.shape[0] * K().recurrence_record(m, dk, dv),), float("nan"), device=DEV)
        oraw = torch.full((pj.shape[0], wv), float("nan"), device=DEV)
        K().recurrence(m, pj, offs, state, out, dev(hb.q_start), dev(hb.slots), prep, oraw, **kw)
        at = 0
        for r, n in take:
            got[r].append(out[at:at + n].float().cpu())
            at += n
            done[r] += n
    worst = 0.0
    for r, n in enumerate(lens):
        pr = proj[r].double()
        col = lambda nme, w: pr[:, offs[nme]:offs[nme] + w]
        want = torch.empty(n, H, dv, dtype=torch.float64)
        for h in range(H):
            ks, vs_ = slice(h * dk, (h + 1) * dk), slice(h * dv, (h + 1) * dv)
            if mode == "delta":
                w = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(col("w", rank)) @ w2.double().T + w0.double()))[:, ks]
                a = torch.sigmoid(col("a", wk) + a_bias.double())[:, ks]
                o = P.delta_rule(col("r", wk)[:, ks], col("k", wk)[:, ks], col("v", wv)[:, vs_], w, a)
                o = P.rms(o, 1e-5) * out_w.double()[vs_] * torch.sigmoid(col("g", wv)[:, vs_])
            else:
                low = w0.double()[ks]
                f = low + (1 - low) * torch.sigmoid(col("a", wk)[:, ks] + a_bias.double()[ks])
                o = P.rms(P.gated_recurrence(P.silu(col("r", wk)[:, ks]), f, col("v", wv)[:, vs_]), 1e-5) * out_w.double()
            want[:, h] = o
        worst = max(worst, rel(torch.cat(got[r]).view(n, H, dv), want))
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["delta", "gated"])
def test_recurrences_whole_in_portions_and_token_by_token(mode, dtype):
    """Square and oblong states, sizes on both sides of the kernel's register tiers, portions that end on and
    inside the kernel's chunks of 16 tokens, single tokens."""
    tol = 3e-5 if dtype == "float32" else 6e-3
    for H, dk, dv in ((3, 24, 24), (2, 8, 8), (1, 64, 64), (2, 40, 24), (3, 128, 16), (2, 12, 136), (1, 130, 130)):
        if mode == "delta" and dk != dv:
            continue
        for cuts in ((1000,), (16, 1, 15, 17, 2, 33), (1,)):
            lens = [70, 1, 33] if cuts != (1,) else [20, 3]
            assert _recurrence_case(mode, dtype, H, dk, dv, lens, cuts, seed=dk + len(cuts)) < tol, (H, dk, dv, cuts)


def test_routing_by_sigmoid_scores_and_weights_on_the_experts_inputs():
    """The choice (largest scores, ties to the lower index), the weights (the scores themselves, not
    renormalised) and expert(w * h) against the plain functions, in 32 bits, for one to three choices."""
    from rosellm_b200.engine.context import Workspace
    from rosellm_b200.parts.gated import MixtureOfExperts

    class Ctx:
        pass

    for E, top, hid, ff, n in ((5, 2, 64, 12, 37), (4, 1, 96, 40, 200), (8, 3, 48, 16, 3), (16, 4, 64, 24, 70)):
        g = torch.Generator().manual_seed(E)
        W = {"router": torch.randn(E, hid, generator=g) * 0.4}
        for e in range(E):
            W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"] = (torch.randn(ff, hid, generator=g) * 0.2, torch.randn(ff, hid, generator=g) * 0.2,
                                                             torch.randn(hid, ff, generator=g) * 0.2)
        h = torch.randn(n, hid, generator=g)
        part = MixtureOfExperts(hid, ff, E, top, gate="silu", score="sigmoid", weight_input=True)
        part.bind({"router_weight": W["router"].to(DEV),
                   "gate_up_weight": torch.cat([W[f"e{e}.{w}"] for e in range(E) for w in ("gate", "up")]).to(DEV),
                   "down_weight": torch.cat([W[f"e{e}.down"] for e in range(E)]).to(DEV)})
        ctx = Ctx()
        ctx.n_tokens, ctx.workspace, ctx.act_dtype = n, Workspace(torch.device(DEV)), torch.float32
        y = torch.full((n, hid), 2.0, device=DEV)
        part.forward(ctx, h.to(DEV), y, add=False)
        want = P.moe_ff(h.double(), {k: v.double() for k, v in W.items()}, "", {"router": {"top": top}})
        assert rel(y, want) < 2e-5, (E, top)
        idx, val = P.route(h.double(), W["router"].double(), top)
        ids = ctx.workspace.get("moe_ids", (n * top,), torch.int32).view(n, top).cpu()
        wts = ctx.workspace.get("moe_weights", (n * top,), torch.float32).view(n, top).cpu()
        assert torch.equal(ids.long(), idx) and rel(wts, val) < 1e-6


# ---- whole models through the step function ------------------------------------------------------------

@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("porovik"))
    return {(name, dtype): write_tiny(name, root, decisive=dtype == "bfloat16") for name in TINY for dtype in DTYPES}


_plain: dict = {}


def plain_logits(folder, toks):
    key = (folder, tuple(toks))
    if key not in _plain:
        cfg, w = load_folder(folder)
        _plain[key] = P.forward(cfg, w, toks)
    return _plain[key]


def check(folder, reqs, trace, got, dtype):
    """float32: every wanted row within 3e-4 of the plain logits.  bfloat16 (on the folders whose routing is
    decisive): the row's error (mean taken off, root mean square over the vocabulary, over that of the
    plain row) below 0.12 for all but 3 % of the rows."""
    over, total, errs = 0, 0, []
    for s, want in zip(trace.steps, trace.wanted):
        if not want:
            continue
        arr = torch.from_numpy(got[s["step"]].astype(np.float64)).view(len(want), -1)
        for row, (rid, pos) in enumerate(want):
            ref = plain_logits(folder, reqs[rid])[pos]
            assert torch.isfinite(arr[row]).all()
            total += 1
            if dtype == "float32":
                diff = float((arr[row] - ref).abs().max())
                assert diff <= 3e-4, (f"step {s['step']}: request {rid} position {pos}: |logits - plain| = {diff:.3e}; "
                                      f"entries {[(e['id'], len(e['tokens'])) for e in s['entries']]}")
            else:
                d = arr[row] - ref
                d = d - d.mean()
                errs.append(float(d.pow(2).mean().sqrt() / (ref - ref.mean()).pow(2).mean().sqrt()))
                over += errs[-1] > 0.12
    assert over <= 0.03 * total + 1, (f"{over} of {total} rows differ from the plain logits beyond bfloat16 rounding; "
                                      f"quantiles 50/90/99 %: {np.quantile(errs, [0.5, 0.9, 0.99])}")


def requests_for(name, lens, seed):
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, TINY[name]["raw"]["vocab"], size=n).tolist() for i, n in enumerate(lens)}


def replay(folder, name, dtype, trace, out, **kw):
    return R.replay(folder, dtype, trace, str(out), page_size=TINY[name]["page_size"], **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_whole_prompts(folders, tmp_path, name, dtype):
    reqs = requests_for(name, [1, 2, 5, 16, 17, 33, 150, 300], 1)
    tr = R.whole(reqs)
    check(folders[name, dtype], reqs, tr, replay(folders[name, dtype], name, dtype, tr, tmp_path), dtype)


@pytest.mark.parametrize("graphs", [False, True], ids=["walked", "graphs"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_prefill_against_token_by_token_decoding(folders, tmp_path, name, dtype, graphs):
    """The last 40 tokens one by one (with ``graphs``: as CUDA-graph replays, the way generation runs them),
    over page borders and over the positions where the query temperature steps."""
    reqs = requests_for(name, [41, 72, 104, 3], 2)
    tr = R.tail_decoded(reqs, tail=40)
    stats = {}
    got = replay(folders[name, dtype], name, dtype, tr, tmp_path, cuda_graphs=graphs, stats=stats)
    check(folders[name, dtype], reqs, tr, got, dtype)
    assert (stats["graph_replays"] > 0) == graphs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_portions_down_to_two_tokens(folders, tmp_path, name, dtype):
    reqs = requests_for(name, [100, 37, 64, 129], 3)
    for sizes in ((7, 2, 16, 3, 2, 5, 33, 2, 1, 17), (2,), (15, 1, 16, 17)):
        tr = R.portions(reqs, sizes=sizes)
        got = replay(folders[name, dtype], name, dtype, tr, tmp_path / f"s{len(sizes)}{sizes[0]}")
        check(folders[name, dtype], reqs, tr, got, dtype)


@pytest.mark.parametrize("graphs", [False, True], ids=["walked", "graphs"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_mixed_batches_with_pages_and_slots_used_again(folders, tmp_path, name, dtype, graphs):
    """Up to four live requests, portions beside single tokens, in a pool so small that pages and state
    slots come round again; every row is compared with the request run alone (the plain implementation
    knows no batch): a state or a last token left over by a slot's earlier owner would show."""
    lens = [120, 9, 200, 33, 70, 2, 193, 64, 20, 101]
    reqs = requests_for(name, lens, 4)
    prompt_lens = {rid: max(1, len(t) - (8 if i % 2 else 40)) for i, (rid, t) in enumerate(reqs.items())}
    tr = R.mixed(reqs, prompt_lens, max_live=4, seed=5)
    peak = R.peak_tokens(tr)
    assert sum(-(-len(t) // 64) * 64 for t in reqs.values()) > 1.5 * peak
    got = replay(folders[name, dtype], name, dtype, tr, tmp_path, max_tokens=peak, cuda_graphs=graphs)
    check(folders[name, dtype], reqs, tr, got, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(folders, tmp_path, dtype):
    reqs = requests_for("A", [1, 2, 3, 4], 9)
    for i, tr in enumerate((R.whole(reqs), R.tail_decoded(reqs, tail=10), R.portions(reqs, sizes=(2, 1)))):
        check(folders["A", dtype], reqs, tr, replay(folders["A", dtype], "A", dtype, tr, tmp_path / f"f{i}"), dtype)
    reqs = requests_for("B", [420], 10)
    tr = R.tail_decoded(reqs, tail=417)
    check(folders["B", dtype], reqs, tr, replay(folders["B", dtype], "B", dtype, tr, tmp_path / "long", cuda_graphs=True), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_wide_model_with_long_contexts(tmp_path, dtype):
    """Width 1024: the products' tensor-core paths with float32 outputs, prompts of 600 and 350 tokens whole
    and in portions of up to 256, the last tokens one by one over contexts whose keys are cut into parts,
    states of 64 and 128 columns spread over several blocks."""
    from tiny_porovik import WIDE

    folder = write_tiny("WIDE", str(tmp_path), decisive=dtype == "bfloat16")
    rng = np.random.default_rng(3)
    reqs = {f"r{i}": rng.integers(0, WIDE["raw"]["vocab"], size=n).tolist() for i, n in enumerate([600, 350])}
    for i, tr in enumerate((R.whole(reqs), R.tail_decoded(reqs, tail=6), R.portions(reqs, sizes=(256, 3, 130, 64, 200)))):
        wanted = {rid: {len(t) - 1, len(t) - 2, len(t) // 2, 0, 1} for rid, t in reqs.items()}
        for s_, w_ in zip(tr.steps, tr.wanted):  # keep a few rows a request: the logits of 950 rows are not needed
            keep = [k for k, (rid, pos) in enumerate(w_) if pos in wanted[rid] or len(s_["entries"][0]["tokens"]) == 1]
            at = 0
            for e in s_["entries"]:
                n = len(e["want"])
                e["want"] = [e["want"][k - at] for k in keep if at <= k < at + n]
                at += n
            w_[:] = [w_[k] for k in keep]
        got = R.replay(folder, dtype, tr, str(tmp_path / f"w{i}"), page_size=16)
        check(folder, reqs, tr, got, dtype)


def test_trace_program_as_a_child_process(folders, tmp_path):
    reqs = requests_for("A", [40, 90, 3], 6)
    tr = R.mixed(reqs, {rid: len(t) - 5 for rid, t in reqs.items()}, max_live=2, seed=1)
    got = R.replay(folders["A", "float32"], "float32", tr, str(tmp_path), subprocess_mode=True, page_size=16)
    check(folders["A", "float32"], reqs, tr, got, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    """Prompts of unequal length through ``InferenceEngine.generate_batch`` (scheduler, portions of 16
    tokens, decode graphs, tokens chosen on the device and fed back without the host reading them): every
    generated token is the plain arg-max given the tokens before it, or within the precision's reach."""
    from rosellm_b200.engine.llm import InferenceEngine

    rng = np.random.default_rng(7)
    vocab = TINY[name]["raw"]["vocab"]
    prompts = [rng.integers(0, vocab, n).tolist() for n in (5, 37, 1, 64)]
    eng = InferenceEngine(folders[name, dtype], dtype=dtype, page_size=TINY[name]["page_size"], max_batch_size=4,
                          kv_cache_max_tokens=512, prefill_chunk_size=16, max_position_embeddings=256)
    outs = eng.generate_batch(prompts, max_new_tokens=12, stop_on_eos=False)
    assert [len(o) for o in outs] == [12] * 4
    for prompt, out in zip(prompts, outs):
        ids = list(prompt)
        for tok in out:
            ref = plain_logits(folders[name, dtype], ids)[-1]
            gap = float(ref.max() - ref[tok])
            spread = float((ref - ref.mean()).pow(2).mean().sqrt())
            assert gap <= (3e-4 if dtype == "float32" else 0.16 * spread), (gap, spread)
            ids.append(tok)
