"""Vodelix on the GPU: replay through bin/trace_run against the plain implementation (whole
prompts, tails decoded token by token, portions down to two tokens, mixed batches in a pool so
small that pages and slots are used again), every new kernel alone against NumPy, keys planted far
away and at page borders with a sink that must not be left out, the recurrent state across steps
and slots used again, and greedy generation through the Python entry point and the scheduler."""
import math

import numpy as np
import pytest
import torch

import plain_vodelix as pv
import tiny_vodelix as tv
import trace_tools as tt

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

LENGTHS = {"VA": [1, 2, 19, 100, 65, 48, 33], "VB": [5, 41, 97, 230, 129, 64], "VC": [3, 70, 130, 17],
           "VL": [7, 150, 300, 64]}


@pytest.fixture(scope="module")
def cases(model_folders):
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            folder = model_folders(name, dtype)
            rng = np.random.default_rng(700 + ord(name[1]))
            reqs = tt.make_requests(rng, tv.TINY[name]["config"]["vocab"], LENGTHS[name])
            cfg, w = pv.load_folder(folder)
            made[(name, dtype)] = (folder, reqs, {r: pv.logits_all(cfg, w, t) for r, t in reqs.items()})
        return made[(name, dtype)]
    return get


# In bfloat16 a router's choice between two experts whose logits differ by less than the rounding of
# its input is a toss-up, the other expert's output is another output, and the recurrent state and the
# keys carry the difference on to the positions behind it.  (Layers that norm what they add also turn
# a sublayer's relative rounding error into an absolute one of the stream.)  So in bfloat16 whole-model
# logits are compared in the bulk: the median error and the share of positions within the bound.  The
# sharp checks of cache, state and batching are the 32-bit runs, which take the same way through the
# host's code, and the kernels' own tests, which run both types.
def _compare(got, tb, plain, dtype, label, tol_rms=3e-5):
    """(32-bit: every row's root-mean-square error relative to the row's own.  Layers that norm what
    they add carry a stream of 30 to 80 in size, whose roundings the final norm scales with it: the
    engine's 32-bit logits sit 2e-6 to 1.5e-5 from the 64-bit ones, where a wrong key or a lost state
    shows as 1e-2 and more.)"""
    errs = []
    for sid in sorted(tb.rows):
        want = tt.expected_rows(tb.rows[sid], plain)
        have = got[sid]
        assert have.shape == want.shape and np.isfinite(have).all(), (label, sid)
        errs.extend(np.sqrt(((have - want) ** 2).mean(axis=1)) / np.sqrt((want ** 2).mean(axis=1)))
    errs = np.sort(np.asarray(errs))
    print(f"{label} {dtype}: {len(errs)} rows, relative rms error median {np.median(errs):.2e}, "
          f"90 % {errs[int(0.9 * (len(errs) - 1))]:.2e}, worst {errs[-1]:.2e}")
    if dtype == "float32":
        assert errs[-1] <= tol_rms, (label, errs[-1])
    else:
        assert np.median(errs) <= 1.2e-2 and errs[int(0.9 * (len(errs) - 1))] <= 4e-2, label


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["VA", "VB", "VC"])
def test_alone_whole_tail_portions(name, dtype, cases, tmp_path):
    folder, reqs, plain = cases(name, dtype)
    ps = tv.TINY[name]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_whole(tb, reqs)
    tt.trace_tail_decode(tb, reqs)
    tt.trace_portions(tb, reqs, np.random.default_rng(7))
    got = tt.run_trace(folder, dtype, tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"))
    _compare(got, tb, plain, dtype, f"config {name}")
    if dtype == "float32":
        # (the norm kernels for few and for many rows add in different orders: cuttings agree to
        # rounding, not to the bit, and the stream's size scales that as it scales the error above)
        tt.compare_cuts([(got, tb)], dtype, f"config {name}", tol=3e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["VA", "VB", "VC"])
def test_mixed_with_page_and_slot_reuse(name, dtype, cases, tmp_path):
    folder, reqs, plain = cases(name, dtype)
    ps = tv.TINY[name]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_mixed(tb, reqs, np.random.default_rng(11), max_live=3)
    assert tb.pages_taken > tb.peak_tokens // ps, "the trace must make the pool hand pages out again"
    assert max(len(s["entries"]) for s in tb.steps) >= 3
    got = tt.run_trace(folder, dtype, tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"),
                       extra_args=["--max-live", "3"])          # three slots for all requests
    _compare(got, tb, plain, dtype, f"config {name} mixed")


def test_long_decoding(cases, tmp_path):
    folder, reqs, plain = cases("VB", "float32")
    ps = tv.TINY["VB"]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_tail_decode(tb, {"r3": reqs["r3"]}, tail=200)
    got = tt.run_trace(folder, "float32", tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"))
    tt.compare(got, tb, plain, "float32", "long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_sizes_of_the_tensor_core_kernels(dtype, cases, tmp_path):
    folder, reqs, plain = cases("VL", dtype)
    ps = tv.TINY["VL"]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_whole(tb, reqs)
    tt.trace_tail_decode(tb, reqs, tail=40)
    tt.trace_portions(tb, reqs, np.random.default_rng(3))
    tt.trace_mixed(tb, reqs, np.random.default_rng(5))
    got = tt.run_trace(folder, dtype, tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"))
    # (sums over 512 and 1,024 terms: the 32-bit bound is that much wider than at the tiny sizes)
    _compare(got, tb, plain, dtype, "config VL", tol_rms=6e-5)
    if dtype == "float32":
        tt.compare_cuts([(got, tb)], dtype, "config VL", tol=6e-5)


# ------------------------------------------------------------------ kernels
@pytest.fixture(scope="module")
def K():
    from crane_b200.kernels import get_kernels
    return get_kernels()


def _dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=dtype).to(DEV)


def _err():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("hidden", [6, 7, 96])
def test_embed_sinusoid(K, hidden):
    rng = np.random.default_rng(hidden)
    vocab = 50
    table = rng.standard_normal((vocab, hidden)).astype(np.float32)
    toks = rng.integers(0, vocab, 9)
    pos = np.array([0, 1, 2, 63, 64, 1000, 4097, 100000, 131071])
    freq = torch.tensor([10000.0 ** (-2.0 * i / hidden) for i in range((hidden + 1) // 2)], dtype=torch.float64, device=DEV)
    x = torch.full((9, hidden), 7.0, device=DEV)
    keep = torch.zeros_like(x)
    err = _err()
    K.embed_sinusoid(_dev(toks, torch.int32), _dev(pos, torch.int32), _dev(table), freq, x, keep, err)
    want = pv.embedding({"embed": table.astype(np.float64)}, toks, pos, hidden)
    assert np.abs(x.cpu().numpy() - want).max() < 1e-6 * max(1.0, np.abs(want).max())
    assert torch.equal(x, keep) and int(err.item()) == 0
    # a token that an earlier launch sampled is read from the device
    deferred = _dev([4, 9], torch.int32)
    K.embed_sinusoid(_dev([-3], torch.int32), _dev([5], torch.int32), _dev(table), freq, x[:1], None, err, deferred)
    assert np.abs(x[0].cpu().numpy() - pv.embedding({"embed": table.astype(np.float64)}, [9], [5], hidden)[0]).max() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [68, 96, 1000])
def test_add_normed_norm(K, dtype, hidden):
    from crane_b200.kernels import Partials
    rng = np.random.default_rng(hidden)
    n = 5
    x = rng.standard_normal((n, hidden)).astype(np.float32) * 3
    wd, wo = (1 + 0.3 * rng.standard_normal(hidden).astype(np.float32) for _ in range(2))
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for form in ("whole", "parts"):
        if form == "whole":
            delta = _dev(rng.standard_normal((n, hidden)) * 0.01, dtype)     # small: the norm must scale it up
            dn = delta.double().cpu().numpy()
        else:
            parts = _dev(rng.standard_normal((3, n, hidden)))
            delta = Partials(parts)
            dn = parts.sum(0).to(dtype).double().cpu().numpy()               # partial sums are rounded once
        new = x + pv.rms_norm(dn, wd, 1e-6)
        xd = _dev(x)
        out = torch.empty(n, hidden, dtype=dtype, device=DEV)
        raw = torch.empty_like(out)
        K.add_normed_norm(xd, delta, _dev(wd), 1e-6, _dev(wo), 1e-5, out, raw)
        assert np.abs(xd.cpu().numpy() - new).max() < 1e-5 * np.abs(new).max()
        assert np.abs(out.double().cpu().numpy() - pv.rms_norm(new, wo, 1e-5)).max() < tol * 4
        assert np.abs(raw.double().cpu().numpy() - new).max() < tol * np.abs(new).max()
        xd = _dev(x)                                                         # the addition alone
        K.add_normed_norm(xd, delta, _dev(wd), 1e-6, raw=raw)
        assert np.abs(xd.cpu().numpy() - new).max() < 1e-5 * np.abs(new).max()


@pytest.mark.parametrize("experts, top", [(3, 3), (5, 2), (12, 1), (40, 4), (70, 9)])
def test_route_topk(K, experts, top):
    rng = np.random.default_rng(experts)
    n = 33
    z = rng.standard_normal((n, experts)).astype(np.float32) * 3
    z[0, :] = 1.5                                   # all equal: the lowest indices win
    z[1, -1] = z[1, 0] = 9.0                        # a tie at the top
    route = torch.full((n, experts), 5.0, device=DEV)
    idx = torch.zeros((n, top), dtype=torch.int32, device=DEV)
    wt = torch.zeros((n, top), device=DEV)
    K.route_topk(_dev(z), route, idx, wt)
    want_idx, want_w = pv.route(z.astype(np.float64), {"router": np.eye(experts)}, "", top)
    assert np.array_equal(idx.cpu().numpy(), want_idx)
    assert np.abs(wt.cpu().numpy() - want_w).max() < 1e-6
    dense = np.zeros((n, experts))
    np.put_along_axis(dense, want_idx, want_w, -1)
    assert np.abs(route.cpu().numpy() - dense).max() < 1e-6
    assert idx[0].tolist() == list(range(top))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ffn_activation_and_token_gate(K, dtype):
    rng = np.random.default_rng(5)
    n, E, F, Fs = 6, 3, 5, 4
    up = _dev(rng.standard_normal((n, E * F + Fs)) * 2, dtype)
    upn = up.double().cpu().numpy()
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    out = torch.empty_like(up)
    for kind, fn in (("relu2", pv.relu_squared), ("gelu", pv.gelu_erf), ("gelu_tanh", pv.gelu_tanh)):
        K.ffn_activation(up, out, kind)
        assert np.abs(out.double().cpu().numpy() - fn(upn)).max() < tol * 4, kind
    route = rng.random((n, E)).astype(np.float32)
    route[:, 1] = 0.0
    K.ffn_activation(up, out, "gelu", _dev(route), F, E * F)
    want = pv.gelu_erf(upn)
    want[:, :E * F] *= np.repeat(route, F, axis=1)
    assert np.abs(out.double().cpu().numpy() - want).max() < tol * 4
    assert (out[:, F:2 * F] == 0).all()
    # the gate of the token input
    vocab, cols, dim, off = 11, 12, 4, 8
    side = _dev(rng.standard_normal((vocab, cols)), dtype)
    z = _dev(rng.standard_normal((n, dim)), dtype)
    toks = rng.integers(0, vocab, n)
    g = torch.empty(n, dim, dtype=dtype, device=DEV)
    K.token_gate(z, _dev(toks, torch.int32), side, off, g, _err())
    want = pv.gelu_tanh(z.double().cpu().numpy()) * side.double().cpu().numpy()[toks][:, off:off + dim]
    assert np.abs(g.double().cpu().numpy() - want).max() < tol * 4


def _step_meta(q_lens, before, page_size, rng, extra_pages=2):
    """Metadata of one step for requests that hold ``before`` tokens and bring ``q_lens`` more:
    pages in random order."""
    total = [b + q for b, q in zip(before, q_lens)]
    blocks = [(t + page_size - 1) // page_size for t in total]
    order = rng.permutation(sum(blocks) + extra_pages)
    table = -np.ones((len(total), max(blocks)), dtype=np.int32)
    nxt = 0
    for e, b in enumerate(blocks):
        table[e, :b] = order[nxt:nxt + b]
        nxt += b
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    pos = np.concatenate([np.arange(b, b + q) for b, q in zip(before, q_lens)]).astype(np.int32)
    ent = np.concatenate([np.full(q, e) for e, q in enumerate(q_lens)]).astype(np.int32)
    return table, cu, pos, ent, np.asarray(total, dtype=np.int32), len(order)


def _plain_sink_attention(q, k, v, scale, sink):
    """q [H, d] over k [T, G, d], v [T, G, m] in float64."""
    H, G = q.shape[0], k.shape[1]
    out = np.zeros((H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        e = np.exp(k[:, g] @ q[h] * scale)
        out[h] = (e / ((1.0 if sink else 0.0) + e.sum())) @ v[:, g]
    return out


@pytest.mark.parametrize("dtype, splits", [(torch.float32, 0), (torch.bfloat16, 0), (torch.bfloat16, 1), (torch.bfloat16, 4),
                                           (torch.bfloat16, 16)])
@pytest.mark.parametrize("H, G, d, m, ps", [(4, 1, 64, 80, 64), (6, 2, 16, 24, 16), (3, 3, 24, 8, 8), (8, 2, 128, 128, 32),
                                            (4, 2, 100, 128, 16)])
def test_sink_attention_with_planted_keys(K, dtype, splits, H, G, d, m, ps):
    """The projection norm, the cache write and the attention over prompts and decoded tokens.  One
    key per request is made to stand out for one query (far back, at a page's last and first
    place, the newest); other queries score so low that the sink takes nearly everything.
    ``splits`` 0: the FP32-core kernel on rows as wide as they are; else the warp-level kernels on
    rows stored at a common head size, decoded tokens with their keys in that many slices."""
    from crane_b200.parts.attention import SinkAttention
    from crane_b200.csrc.build import ATTENTION_HEAD_SIZES
    D = Dv = 0
    if splits:
        D = Dv = SinkAttention.common_head_size(d, m, ATTENTION_HEAD_SIZES)
        assert D and K.prefill_attention_supports(D, H, G) and K.decode_attention_supports(D, H, G)
    D, Dv = D or d, Dv or m
    rng = np.random.default_rng(H * 100 + d)
    lens = [700, 2 * ps + 1, 1, 37]
    scale, eps = 0.4, 1e-5
    planted = {0: 3, 1: ps - 1, 3: 36}                       # request -> position of its key
    cols = H * d + G * d + G * m
    qkv = [rng.standard_normal((n, cols)) for n in lens]
    for e, key in planted.items():
        qkv[e][key, H * d:H * d + d] *= 6.0                   # kv head 0's key
        qkv[e][-1, :d] = qkv[e][key, H * d:H * d + d] * 2     # head 0 of the last token asks for it
    qkv[1][ps, H * d:H * d + d] = -qkv[1][ps - 1, H * d:H * d + d]      # the next page's first key: the opposite
    qw, kw = 1 + 0.2 * rng.standard_normal(H * d), 1 + 0.2 * rng.standard_normal(G * d)
    store = torch.float32 if dtype == torch.float32 else torch.bfloat16
    qkv_dev = [_dev(a, store) for a in qkv]
    qkv_r = [a.double().cpu().numpy() for a in qkv_dev]
    stored = lambda a: torch.as_tensor(a).to(store).double().numpy()      # queries and cached keys are kept in the model type
    qn = [stored(pv.rms_norm(a[:, :H * d], qw, eps)).reshape(-1, H, d) for a in qkv_r]
    kn = [stored(pv.rms_norm(a[:, H * d:H * d + G * d], kw, eps)).reshape(-1, G, d) for a in qkv_r]
    vn = [a[:, H * d + G * d:].reshape(-1, G, m) for a in qkv_r]
    err = _err()
    pools = None
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    # a step of whole prompts but the last token of each longer request, then a step that decodes those
    for stage in (0, 1):
        if stage == 0:
            q_lens, before = [max(1, n - 1) for n in lens], [0] * len(lens)
        else:
            keep = [e for e, n in enumerate(lens) if n > 1]
            q_lens, before = [1] * len(keep), [lens[e] - 1 for e in keep]
        ents = list(range(len(lens))) if stage == 0 else keep
        if stage == 0:
            table, cu, pos, ent, total, n_pages = _step_meta(lens, [0] * len(lens), ps, rng)
            full_table = table
            k_pool = torch.randn(n_pages, G, ps, D, device=DEV).mul_(30).to(store)
            v_pool = torch.randn(n_pages, G, ps, Dv, device=DEV).mul_(30).to(store)
            cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
            pos = np.concatenate([np.arange(q) for q in q_lens]).astype(np.int32)
            ent = np.concatenate([np.full(q, e) for e, q in enumerate(q_lens)]).astype(np.int32)
        else:
            table = full_table[keep]
            cu = np.arange(len(keep) + 1, dtype=np.int32)
            pos = np.asarray(before, dtype=np.int32)
            ent = np.arange(len(keep), dtype=np.int32)
        rows = torch.cat([qkv_dev[e][b:b + q] for e, b, q in zip(ents, before, q_lens)])
        n = rows.shape[0]
        q_out = torch.empty(n, H * D, dtype=store, device=DEV)
        K.projection_norm_cache(rows, cols, _dev(pos, torch.int32), _dev(ent, torch.int32), _dev(table, torch.int32),
                                ps, _dev(qw), _dev(kw), eps, q_out, k_pool, v_pool, H, G, d, m, err)
        o = torch.empty(n, H * Dv, dtype=store, device=DEV)
        if not splits:
            K.paged_attention_simt(q_out, o, k_pool, v_pool, _dev(pos, torch.int32), _dev(ent, torch.int32),
                                   _dev(table, torch.int32), ps, H, G, d, 0, scale, err, dv=m, v_stride=m, sink=True)
        else:
            kv = _dev([b + q for b, q in zip(before, q_lens)], torch.int32)
            if stage == 0:
                tiles = sum((q + 63) // 64 for q in q_lens)
                K.paged_prefill_attention(q_out, o, k_pool, v_pool, _dev(cu, torch.int32), kv, _dev(table, torch.int32),
                                          ps, tiles, H, G, D, 0, scale, err, sink=True)
            else:
                part_o = torch.empty(n * H * splits, D, device=DEV)
                part_ml = torch.empty(n * H * splits, 2, device=DEV)
                K.paged_decode_attention(q_out, o, k_pool, v_pool, _dev(cu, torch.int32), kv, _dev(table, torch.int32),
                                         ps, H, G, D, 0, scale, splits, part_o, part_ml, err, sink=True)
        got = o.double().cpu().numpy().reshape(n, H, Dv)[:, :, :m]
        for i in range(n):
            e, p = ents[ent[i]], pos[i]
            want = _plain_sink_attention(qn[e][p], kn[e][:p + 1], vn[e][:p + 1], scale, True)
            assert np.abs(got[i] - want).max() < tol * max(1.0, np.abs(want).max()), (stage, e, p)
        if stage == 1:
            for j, e in enumerate(keep):
                if e in planted:                       # the planted key is (nearly) all that head 0 gets
                    assert np.abs(got[j, 0] - vn[e][planted[e], 0]).max() < 0.05 * np.abs(vn[e][planted[e], 0]).max() + 0.05
    # without the sink the single first token would return its own value whole; with it, less
    first = _plain_sink_attention(qn[2][0], kn[2][:1], vn[2][:1], scale, True)
    assert np.abs(first).max() < np.abs(vn[2][0]).max()
    assert int(err.item()) == 0


def _plain_delta(proj, H, d, R, w2, w0, ab, norm_w, eps, state):
    """The recurrence of one request from rows [r | k | v | g | a | low] in float64."""
    n, hd = proj.shape[0], H * d
    r, k, v, g, a = (proj[:, i * hd:(i + 1) * hd].reshape(n, H, d) for i in range(5))
    low = np.tanh(proj[:, 5 * hd:]) @ w2.T + w0
    decay = np.exp(-math.exp(-0.5) * pv.sigmoid(low)).reshape(n, H, d)
    rate = pv.sigmoid(a.reshape(n, hd) + ab).reshape(n, H, d)
    unit = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    S = state.copy()
    o = np.zeros((n, H, d))
    for t in range(n):
        for h in range(H):
            S[h], o[t, h] = pv.delta_rule_step(S[h], r[t, h], k[t, h], v[t, h], decay[t, h], rate[t, h], unit[t, h])
    return pv.unit_rms(o, eps).reshape(n, hd) * norm_w * pv.sigmoid(g.reshape(n, hd)), S


@pytest.mark.parametrize("dtype, blocks", [(torch.float32, 1), (torch.bfloat16, 1), (torch.float32, 4), (torch.bfloat16, 2)])
@pytest.mark.parametrize("H, d, R", [(3, 16, 4), (2, 32, 8), (1, 64, 16), (2, 128, 8), (3, 24, 5), (2, 48, 12), (1, 136, 3),
                                     (5, 18, 7), (2, 100, 9), (1, 8, 2), (9, 64, 64)])
def test_delta_rule_kernels(K, dtype, blocks, H, d, R):
    """Three steps over four slots: prompts of unequal length, their continuation (one of them a
    single token) beside a new request in a slot that was used before, with rows and entries
    that pad the step.  ``blocks`` > 1: a head's columns over that many CTAs and the norm in a
    second kernel (where the head size allows it; else the kernel takes one CTA a head by itself)."""
    rng = np.random.default_rng(H * 1000 + d)
    hd, cols = H * d, 5 * H * d + R
    w2, w0, ab = rng.standard_normal((hd, R)) * 0.5, rng.standard_normal(hd), rng.standard_normal(hd)
    norm_w = 1 + 0.2 * rng.standard_normal(hd)
    store = dtype
    w2_d = _dev(w2.T.copy(), store)                                # the kernel takes it turned over: [rank, heads d]
    w2r = w2_d.double().cpu().numpy().T
    state = torch.full((4, H, d, d), 9.0, device=DEV)              # what an earlier request left behind
    err = _err()
    tol = 5e-5 if dtype == torch.float32 else 3e-2
    plain_state = {}
    lengths = {}
    steps = [[("a", 2, 37), ("b", 0, 1), ("c", 3, 70)],            # (request, slot, tokens)
             [("a", 2, 1), ("c", 3, 19), ("d", 0, 5)],             # d takes b's slot
             [("d", 0, 2), ("a", 2, 33)]]
    for entries in steps:
        q_lens = [n for _, _, n in entries]
        n_rows = sum(q_lens) + 3                                    # three rows of no entry behind the real ones
        proj = rng.standard_normal((n_rows, cols)) * 1.5
        proj_d = _dev(proj, store)
        projr = proj_d.double().cpu().numpy()
        cu = np.concatenate([[0], np.cumsum(q_lens), [sum(q_lens)]]).astype(np.int32)      # and one entry without rows
        kv = [lengths.get(r, 0) + n for r, _, n in entries] + [0]
        slots = [s for _, s, _ in entries] + [1]                   # the padding entry names slot 1: it must stay as it is
        ent = np.concatenate([np.full(n, e) for e, n in enumerate(q_lens)] + [np.full(3, -1)]).astype(np.int32)
        aux = torch.zeros(n_rows, 3 * hd, device=DEV)
        out = torch.zeros(n_rows, hd, dtype=store, device=DEV)
        K.delta_rule_prep(proj_d, cols, _dev(ent, torch.int32), w2_d, _dev(w0), _dev(ab), aux, H, d, math.exp(-0.5),
                          1e-6, store)
        K.delta_rule_scan(proj_d, cols, aux, _dev(cu, torch.int32), _dev(kv, torch.int32), _dev(slots, torch.int32),
                          state, _dev(norm_w), 1e-5, out, H, d, err, col_blocks=blocks,
                          o_raw=torch.zeros(n_rows, hd, device=DEV) if blocks > 1 else None,
                          tok_entry=_dev(ent, torch.int32))
        got = out.double().cpu().numpy()
        for e, (r, s, n) in enumerate(entries):
            before = plain_state.get(r, np.zeros((H, d, d)))
            want, plain_state[r] = _plain_delta(projr[cu[e]:cu[e + 1]], H, d, R, w2r, w0, ab, norm_w, 1e-5, before)
            lengths[r] = lengths.get(r, 0) + n
            assert np.abs(got[cu[e]:cu[e + 1]] - want).max() < tol * max(1.0, np.abs(want).max()), (r, n)
            st = state[s].double().cpu().numpy()
            assert np.abs(st - plain_state[r]).max() < 1e-4 * max(1.0, np.abs(plain_state[r]).max()), (r, "state")
        assert (out[sum(q_lens):] == 0).all()                      # rows of no entry are left alone
        assert (state[1] == 9.0).all()                             # and so is the slot of the entry without rows
    assert int(err.item()) == 0


# ---------------------------------------------------------------- generation
def _load(folder, dtype, **opts):
    from crane_b200.generation import ModelForCausalLM
    return ModelForCausalLM.from_pretrained(folder, dtype, **opts)


def _greedy(n):
    from crane_b200.generation import GenerationConfig
    return GenerationConfig(max_new_tokens=n, temperature=None, eos_token_id=-1)


@pytest.mark.parametrize("name", ["VA", "VB", "VC"])
def test_greedy_generation_float32_equals_plain(name, model_folders):
    folder = model_folders(name, "float32")
    cfg, w = pv.load_folder(folder)
    m = _load(folder, "fp32", page_size=tv.TINY[name]["page_size"], num_pages=24, max_concurrent=3,
              max_batched_tokens=64, max_seq_len=256)
    rng = np.random.default_rng(3)
    for n in (1, 5, 17):
        prompt = rng.integers(0, cfg["vocab"], n).tolist()
        assert m.generate(prompt, _greedy(8)) == pv.greedy_generate(cfg, w, prompt, 8)
    m.runner.table.check()
    assert m.runner.table.live() == 0


@pytest.mark.parametrize("name", ["VA", "VL"])
def test_greedy_batch_bfloat16_through_the_scheduler(name, model_folders):
    """Six prompts, three slots, portions of at most 16 tokens: requests wait, slots and pages are
    used again, and decode steps replay graphs with the recurrent state in them."""
    folder = model_folders(name, "bfloat16")
    cfg, w = pv.load_folder(folder)
    m = _load(folder, "bf16", page_size=16, num_pages=40, max_concurrent=3, max_batched_tokens=48, chunk_size=16,
              max_seq_len=256)
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (12, 3, 40, 1, 25, 7)]
    outs = m.generate_batch(prompts, _greedy(20))
    ok = 0
    for prompt, toks in zip(prompts, outs):
        assert len(toks) == len(prompt) + 20 and toks[:len(prompt)] == prompt
        logits = pv.logits_all(cfg, w, toks[:-1])
        for i in range(len(prompt), len(toks)):
            row = logits[i - 1]
            # (a token that another rounding would not have chosen does not end the comparison: every later
            # one is checked against the plain logits of the sequence as it was generated)
            ok += bool(row[toks[i]] >= row.max() - 3e-2 * np.abs(row).max())
    assert ok >= 0.95 * 20 * len(prompts), ok
    m.runner.table.check()
    assert m.runner.table.live() == 0
    assert m.runner.graph_replays > 0


def test_command_line(model_folders):
    """bin/crane picks the model class from config.json."""
    import os
    import subprocess
    import sys
    folder = model_folders("VC", "float32")
    cfg, w = pv.load_folder(folder)
    crane = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "crane")
    cmd = [sys.executable, crane, "-m", folder, "--dtype", "fp32", "--prompt-ids", "5,6,7", "--max-new-tokens", "6",
           "--eos-token-id", "-1", "--page-size", "16", "--num-pages", "8", "-c", "2", "--max-batched-tokens", "32",
           "--max-seq-len", "64"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-3000:]
    assert p.stdout.strip().splitlines()[-1] == ",".join(map(str, pv.greedy_generate(cfg, w, [5, 6, 7], 6)[3:]))
