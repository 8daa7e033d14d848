"""Lebedra on the GPU: every mechanism's kernels against the plain implementation's function
for it, then whole models through the engine's step function, cache, scheduler and entry point."""
import math
import os

import numpy as np
import pytest
import torch

import plain_lebedra as P
import replay_util as R
from tiny_lebedra import TINY, load_folder, write_tiny

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def K():
    from rosellm_b200.ops import kernels

    return kernels


def rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double().cpu() - b.double().cpu()).abs().max() / (b.double().abs().max() + 1e-30))


# ---- mechanisms alone ------------------------------------------------------------------------------

@pytest.mark.parametrize("width", [8, 100, 1000])
def test_rms_norm_store_and_add(width):
    g = torch.Generator().manual_seed(width)
    x = torch.randn(7, width, generator=g) * 3
    w = 1 + 0.3 * torch.randn(width, generator=g)
    rows = torch.tensor([5, 0, 6], dtype=torch.int32)
    ref = P.rms_norm(x.double(), w.double(), 1e-3)
    for dt, tol in ((torch.float32, 2e-6), (torch.bfloat16, 5e-3)):
        out = torch.empty(3, width, dtype=dt, device=DEV)
        K().rmsnorm(x.to(DEV), w.to(DEV), 1e-3, out, rows.to(DEV))
        assert rel(out.float(), ref[rows.long()]) < tol
    stream = torch.randn(7, width, generator=g)
    got, copy = stream.to(DEV), torch.empty(7, width, dtype=torch.bfloat16, device=DEV)
    K().rmsnorm_add(x.to(DEV), w.to(DEV), 1e-3, got, 0.35, copy)
    want = stream.double() + 0.35 * ref
    assert rel(got, want) < 2e-6
    assert torch.equal(copy, got.to(torch.bfloat16))


def _pool(n_pages, page, width, dtype):
    return torch.zeros(n_pages, 1, 1, page, width, dtype=dtype, device=DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rank, rot_dim, dims", [(40, 8, 8), (20, 16, 16), (56, 4, 2), (16, 0, 0)])
def test_latent_cache_rows_and_query_rotation(dtype, rank, rot_dim, dims):
    """The cached row is [rms_norm(c), rotated key part, zeros]; the queries' rotated parts land
    behind the latent part of their rows.  Positions reach into the thousands."""
    from rosellm_b200.parts.standard import rotary_frequencies

    dt, page, base = DTYPES[dtype], 8, 300.0
    g = torch.Generator().manual_seed(rank)
    width = -(-(rank + rot_dim) // 8) * 8
    positions = torch.tensor([0, 1, 7, 8, 9, 1234, 4095], dtype=torch.int32)
    n = len(positions)
    dkv = torch.randn(n, rank + rot_dim, generator=g)
    gamma = 1 + 0.2 * torch.randn(rank, generator=g)
    freq = rotary_frequencies(max(dims, 2), base).to(DEV)
    pool = _pool(600, page, width, dt)
    pool.fill_(7.0)  # so that the zeros beyond the row's entries are seen to be written
    table = torch.full((2, 520), -1, dtype=torch.int32)
    perm = torch.randperm(600, generator=g)[:520].to(torch.int32)
    table[1] = perm
    dev = lambda t: t.to(DEV)
    K().latent_kv_write(dev(dkv), dev(gamma), 1e-5, freq, dims, pool, dev(table), dev(positions),
                        dev(torch.zeros(n, dtype=torch.int32)), dev(torch.tensor([1], dtype=torch.int32)),
                        rank=rank, rot_dim=rot_dim, max_pos=520 * page)
    c = P.rms_norm(dkv[:, :rank].double(), gamma.double(), 1e-5)
    kr = P.rotate_pairs(dkv[:, rank:].double(), positions, dims, base) if rot_dim else dkv[:, rank:].double()
    tol = 3e-6 if dtype == "float32" else 5e-3
    # the angle position * frequency is formed in float32: at position p it is off by up to
    # p * 2^-24, and so is the turned vector, relative to its length
    angle_tol = lambda p: 4 * tol + 5.0 * p * 2.0 ** -24
    for i, p in enumerate(positions.tolist()):
        row = pool[int(table[1, p // page]), 0, 0, p % page].float().cpu()
        assert rel(row[:rank], c[i]) < tol
        if rot_dim:
            assert (row[rank:rank + rot_dim].double() - kr[i]).abs().max() < angle_tol(p)
        assert torch.all(row[rank + rot_dim:] == 0)
    if rot_dim:
        H, plain = 3, 5
        q = torch.randn(n, H * (plain + rot_dim), generator=g).to(dt)
        rows = torch.full((n, H * width), 9.0, dtype=dt, device=DEV)
        K().latent_q_rope(dev(q), rows, freq, dev(positions), n_heads=H, head_in=plain + rot_dim, plain=plain,
                          rank=rank, rot_dim=rot_dim, rot_dims=dims, row_width=width)
        qr = P.rotate_pairs(q.double().view(n, H, plain + rot_dim)[..., plain:], positions, dims, base)
        got = rows.float().cpu().view(n, H, width)
        for i, p in enumerate(positions.tolist()):
            assert (got[i, :, rank:rank + rot_dim].double() - qr[i]).abs().max() < angle_tol(p)
        assert torch.all(got[..., rank + rot_dim:] == 0) and torch.all(got[..., :rank] == 9.0)


def _attention_case(dtype, H, rank, tail, lens_new, lens_old, page, sink, scale, by_request, splits, seed,
                    stand_out=None):
    """Requests with ``lens_old`` cached rows bring ``lens_new`` query tokens.  Returns the
    kernel's output and the plain result computed from the same (rounded) inputs."""
    from rosellm_b200.engine.context import build_host_batch

    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(seed)
    W = -(-(rank + tail) // 8) * 8
    n_req = len(lens_new)
    totals = [a + b for a, b in zip(lens_new, lens_old)]
    pages_per = [-(-t // page) for t in totals]
    n_pages = sum(pages_per) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((n_req + 1, max(pages_per)), -1, dtype=torch.int32)
    pool = _pool(n_pages, page, W, dt)
    caches, at = [], 0
    for r in range(n_req):
        rows = torch.randn(totals[r], W, generator=g) * 0.7
        rows[:, rank + tail:] = 0
        caches.append(rows.to(dt))
        for lp in range(pages_per[r]):
            pg = order[at]; at += 1
            table[r + 1, lp] = pg
            chunk = caches[r][lp * page:(lp + 1) * page]
            pool[pg, 0, 0, :chunk.shape[0]] = chunk.to(DEV)
    n_tok = sum(lens_new)
    q = (torch.randn(n_tok, H, W, generator=g) * 0.8)
    q[..., rank + tail:] = 0
    if stand_out is not None:  # one query of request 0 points at one far key, ten times as hard
        qi, key = stand_out
        q[qi] = caches[0][key].float()[None, :] * 10.0
    q = q.to(dt)
    hb = build_host_batch([(r + 1, lens_old[r], [0] * lens_new[r], []) for r in range(n_req)])
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    out = torch.full((n_tok, H * rank), 5.0, dtype=dt, device=DEV)
    sink_t = None if sink is None else torch.tensor(sink, dtype=torch.float32, device=DEV)
    n_dec = len(hb.decode_reqs)
    part_o = part_ml = None
    if by_request and splits > 1:
        part_o = torch.empty(n_dec * H * splits, rank, device=DEV)
        part_ml = torch.empty(n_dec * H * splits, 2, device=DEV)
    K().latent_attention(q.view(n_tok, H * W).to(DEV), pool, table.to(DEV), dev(hb.q_start), dev(hb.kv_len),
                         dev(hb.slots), out, sink=sink_t, n_heads=H, rank=rank, scale=scale,
                         tiles=dev(hb.tiles.reshape(-1)), n_tiles=len(hb.tiles), decode_reqs=dev(hb.decode_reqs),
                         n_decode=n_dec, decode_by_request=by_request, n_splits=splits, part_o=part_o, part_ml=part_ml)
    K().check_status(torch.device(DEV))
    want = torch.empty(n_tok, H, rank, dtype=torch.float64)
    t0 = 0
    for r in range(n_req):
        kv = caches[r].double()
        for i in range(lens_new[r]):
            pos = lens_old[r] + i
            s = torch.einsum("hw,kw->hk", q[t0 + i].double(), kv[:pos + 1]) * scale
            sk = torch.tensor(sink if sink is not None else [-1e300] * H, dtype=torch.float64)
            p = P.softmax_with_sink(s[:, None, :], sk)[:, 0]
            want[t0 + i] = p @ kv[:pos + 1, :rank]
        t0 += lens_new[r]
    return out.float().cpu().view(n_tok, H, rank), want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latent_attention_prompt_portions_and_single_tokens(dtype):
    """Portions that start inside a page, end on a page's border, of one to 40 tokens, beside
    single tokens, with sinks of every size; the value is the row's first `rank` entries only."""
    tol = 2e-5 if dtype == "float32" else 2e-2
    for H, rank, tail, page in ((3, 40, 8, 16), (5, 20, 16, 8), (1, 24, 32, 8), (7, 16, 2, 4), (33, 8, 0, 8)):
        sink = [float(v) for v in torch.linspace(-3, 4, H)]
        for by_request in (False, True):  # decoded tokens as tiles of one query, or all heads in one block
            got, want = _attention_case(dtype, H, rank, tail, [40, 1, 2, 17, 1, 16], [5, 130, 0, 15, 0, 16], page, sink,
                                        0.3, by_request, 1, seed=H)
            assert rel(got, want) < tol, (H, rank, tail, by_request)
        got, want = _attention_case(dtype, H, rank, tail, [33, 16, 2], [0, 31, 70], page, sink, 0.3, False, 1, seed=H + 9)
        assert rel(got, want) < tol, (H, rank, tail, "portions only")
        got, want = _attention_case(dtype, H, rank, tail, [3, 1, 1], [0, 31, 32], page, None, 0.2, True, 1, seed=H + 50)
        assert rel(got, want) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("splits", [1, 3, 8])
def test_latent_attention_decoded_tokens_with_keys_cut_into_parts(dtype, splits):
    tol = 2e-5 if dtype == "float32" else 2e-2
    got, want = _attention_case(dtype, 6, 40, 8, [1, 1, 1, 1], [700, 0, 63, 64], 16, [0.5, -2, 3, 0, 1, 9], 0.25, True,
                                splits, seed=splits)
    assert rel(got, want) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", [0, 15, 16, 17, 511, 512, 897])
def test_a_far_key_that_stands_out_is_found(dtype, key):
    """Among 900 cached rows one is scored far above the rest: the output must be (nearly) that
    row's latent, whether the key is the first, sits at a page's border or far back; from a
    prompt portion's query and from a decoded token's."""
    for new, old, by_request, splits in (([4], [896], False, 1), ([1], [899], True, 4)):
        got, want = _attention_case(dtype, 2, 24, 8, new, old, 16, [0.0, 0.0], 1.0, by_request, splits, seed=key,
                                    stand_out=(new[0] - 1, key))
        assert rel(got, want) < (2e-5 if dtype == "float32" else 2e-2)
        assert (want[-1, 0].abs() > 0.05).any()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_head_linear_both_weight_orders(dtype):
    dt, tol = DTYPES[dtype], (2e-6 if dtype == "float32" else 8e-3)
    g = torch.Generator().manual_seed(3)
    n, H, k, m = 70, 5, 24, 40
    x = torch.randn(n, H, k + 3, generator=g).to(dt)         # heads 3 entries apart from one another
    w_kn = torch.randn(H, k, m, generator=g).to(dt)           # [head][inner][out]
    out = torch.zeros(n, H, m + 8, dtype=dt, device=DEV)
    K().head_linear(x.to(DEV), w_kn.to(DEV), out, n_tokens=n, n_heads=H, k=k, n=m, in_strides=(H * (k + 3), k + 3),
                    w_strides=(k * m, m, 1), out_strides=(H * (m + 8), m + 8))
    want = torch.einsum("thk,hkm->thm", x[..., :k].double(), w_kn.double())
    assert rel(out[..., :m].float(), want) < tol and torch.all(out[..., m:] == 0)
    w_nk = w_kn.transpose(1, 2).contiguous()                  # [head][out][inner]
    out2 = torch.zeros(n, H, m, dtype=dt, device=DEV)
    K().head_linear(x.to(DEV), w_nk.to(DEV), out2, n_tokens=n, n_heads=H, k=k, n=m, in_strides=(H * (k + 3), k + 3),
                    w_strides=(k * m, 1, k), out_strides=(H * m, m))
    assert rel(out2.float(), want) < tol


def test_gate_functions_and_token_gate():
    g = torch.Generator().manual_seed(5)
    gu = torch.randn(9, 2 * 13 + 3, generator=g) * 3
    gate, up = gu[:, :13].double(), gu[:, 16:29].double()
    want = {
        "relu": torch.relu(gate) * up,
        "silu": gate * torch.sigmoid(gate) * up,
        "gelu_tanh": P.gelu_tanh(gate) * up,
        "clamped_swish": (lambda a, b: a * torch.sigmoid(1.702 * a) * (b + 1))(gate.clamp(max=1.1), up.clamp(-1.1, 1.1)),
    }
    for name, ref in want.items():
        out = torch.zeros(9, 13, device=DEV)
        K().gated_act(gu.to(DEV), out, width=13, up_at=16, gate=K().GATES[name], alpha=1.702, limit=1.1)
        assert rel(out, ref) < 3e-6, name
    table = torch.randn(50, 36, generator=g)
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32)
    s = torch.randn(4, 16, generator=g)
    out = torch.full((4, 16), 3.0, device=DEV)
    K().token_gate(s.to(DEV), ids.to(DEV), table.to(DEV), 24, 12, out)
    assert rel(out[:, :12], P.gelu_tanh(s[:, :12].double()) * table[ids.long(), 24:36].double()) < 3e-6
    assert torch.all(out[:, 12:] == 0)


@pytest.mark.parametrize("experts, top, count, keep", [(12, 3, 4, 2), (16, 2, 2, 1), (6, 2, 1, 1), (4, 1, 1, 1),
                                                        (64, 6, 8, 3)])
def test_routing_against_plain(experts, top, count, keep):
    """Scores, group choice (with choice scores that are negative) and the chosen experts'
    weights; the layout that follows gives every pair one place among its expert's."""
    g = torch.Generator().manual_seed(experts)
    n = 150
    z = torch.randn(n, experts, generator=g) * 2
    corr = torch.randn(experts, generator=g) * 0.5 - 0.4
    router = {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}
    w = {"r.router": torch.eye(experts, dtype=torch.float64), "r.correction": corr.double()}
    idx, weight = P.route(z.double(), w, "r.", router)
    ids = torch.empty(n * top, dtype=torch.int32, device=DEV)
    wts = torch.empty(n * top, device=DEV)
    counts = torch.zeros(experts, dtype=torch.int32, device=DEV)
    K().moe_select(z.to(DEV), corr.to(DEV), top=top, group_count=count, group_keep=keep, ids=ids, weights=wts,
                   counts=counts)
    got = ids.cpu().view(n, top).long()
    assert torch.equal(got.sort(dim=1).values, idx.sort(dim=1).values)
    s = torch.softmax(z.double(), dim=-1)
    assert rel(wts.cpu().view(n, top), s.gather(1, got)) < 1e-5
    assert torch.equal(counts.cpu().long(), torch.bincount(got.flatten(), minlength=experts))
    i32 = dict(dtype=torch.int32, device=DEV)
    fill, offsets = torch.zeros(experts, **i32), torch.empty(experts + 1, **i32)
    tiles, meta = torch.empty(K().moe_max_tiles(n * top, experts) * 3, **i32), torch.empty(4, **i32)
    row_token, place_of = torch.empty(n * top, **i32), torch.empty(n * top, **i32)
    K().moe_plan(ids, counts, fill, offsets, tiles, meta, row_token, place_of, n_tokens=n, n_experts=experts, top=top)
    assert not counts.any() and torch.equal(fill.cpu().long(), torch.bincount(got.flatten(), minlength=experts))
    assert sorted(place_of.cpu().tolist()) == list(range(n * top))
    off = offsets.cpu().tolist()
    for i, place in enumerate(place_of.cpu().tolist()):
        e = int(got.flatten()[i])
        assert off[e] <= place < off[e + 1] and int(row_token[place]) == i // top
    covered = []
    for t in tiles.cpu().view(-1, 3)[:int(meta[0])].tolist():
        assert off[t[0]] <= t[1] and t[1] + t[2] <= off[t[0] + 1] and 0 < t[2] <= 64
        covered.extend(range(t[1], t[1] + t[2]))
    assert sorted(covered) == list(range(n * top))


# ---- whole models through the step function ------------------------------------------------------------

@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("lebedra"))
    return {(name, dtype): write_tiny(name, root, decisive=dtype == "bfloat16") for name in TINY for dtype in DTYPES}


_plain: dict = {}


def plain_logits(folder, toks):
    key = (folder, tuple(toks))
    if key not in _plain:
        cfg, w = load_folder(folder)
        _plain[key] = P.forward(cfg, w, toks)
    return _plain[key]


def check(folder, reqs, trace, got, dtype):
    """float32: every wanted row within 2e-4 of the plain logits.  bfloat16 (on the folders whose
    routing is decisive): the row's error (mean taken off, root mean square over the vocabulary,
    over that of the plain row) below 0.15 for all but 3 % of the rows (the sharp weights of these
    folders put the median near 0.03)."""
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
                assert diff <= 2e-4, (f"step {s['step']}: request {rid} position {pos}: |logits - plain| = {diff:.3e}; "
                                      f"entries {[(e['id'], len(e['tokens'])) for e in s['entries']]}")
            else:
                d = arr[row] - ref
                d = d - d.mean()
                errs.append(float(d.pow(2).mean().sqrt() / (ref - ref.mean()).pow(2).mean().sqrt()))
                over += errs[-1] > 0.15
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
    """The last 40 tokens one by one (with ``graphs``: as CUDA-graph replays, the way generation
    runs them), over page borders, after prompts that end inside and at the end of a page."""
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
    """Up to four live requests, portions beside single tokens, in a pool so small that pages
    and slots come round again; every row is compared with the request run alone (the plain
    implementation knows no batch)."""
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
    reqs = requests_for("X", [1, 2, 3, 4], 9)
    for i, tr in enumerate((R.whole(reqs), R.tail_decoded(reqs, tail=10), R.portions(reqs, sizes=(2, 1)))):
        check(folders["X", dtype], reqs, tr, replay(folders["X", dtype], "X", dtype, tr, tmp_path / f"f{i}"), dtype)
    reqs = requests_for("Y", [420], 10)
    tr = R.tail_decoded(reqs, tail=417)
    check(folders["Y", dtype], reqs, tr, replay(folders["Y", dtype], "Y", dtype, tr, tmp_path / "long", cuda_graphs=True), dtype)


def test_trace_program_as_a_child_process(folders, tmp_path):
    reqs = requests_for("X", [40, 90, 3], 6)
    tr = R.mixed(reqs, {rid: len(t) - 5 for rid, t in reqs.items()}, max_live=2, seed=1)
    got = R.replay(folders["X", "float32"], "float32", tr, str(tmp_path), subprocess_mode=True, page_size=16)
    check(folders["X", "float32"], reqs, tr, got, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    """Prompts of unequal length through ``InferenceEngine.generate_batch`` (scheduler, portions
    of 16 tokens, decode graphs, tokens chosen on the device): every generated token is the
    plain arg-max given the tokens before it, or within the precision's reach of it."""
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
            assert gap <= (2e-4 if dtype == "float32" else 0.16 * spread), (gap, spread)
            ids.append(tok)
