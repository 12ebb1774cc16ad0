"""Radorax on the GPU: replay through bin/trace_run against the plain implementation (whole
prompts, tails decoded token by token, portions down to two tokens, mixed batches in a pool so
small that pages and slots are used again), every new kernel alone against NumPy, keys planted
far away and at page borders, the bigram state across steps and slot reuse, and greedy generation
through the Python entry point and the scheduler."""
import numpy as np
import pytest
import torch

import plain_radorax as pr
import tiny_radorax as tr
import trace_tools as tt

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

LENGTHS = {"RA": [1, 2, 19, 100, 65, 48, 33], "RB": [5, 41, 97, 230, 129, 64], "RC": [3, 70, 130],
           "RL": [7, 150, 300, 64], "RH": [2, 90, 200, 33]}


@pytest.fixture(scope="module")
def cases(model_folders):
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            folder = model_folders(name, dtype)
            rng = np.random.default_rng(500 + len(name) + ord(name[1]))
            reqs = tt.make_requests(rng, tr.TINY[name]["config"]["vocab"], LENGTHS[name])
            cfg, w = pr.load_folder(folder)
            made[(name, dtype)] = (folder, reqs, {r: pr.logits_all(cfg, w, t) for r, t in reqs.items()})
        return made[(name, dtype)]
    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["RA", "RB", "RC", "RH"])
def test_alone_whole_tail_portions(name, dtype, cases, tmp_path):
    folder, reqs, plain = cases(name, dtype)
    ps = tr.TINY[name]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_whole(tb, reqs)
    tt.trace_tail_decode(tb, reqs)
    tt.trace_portions(tb, reqs, np.random.default_rng(7))
    got = tt.run_trace(folder, dtype, tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"))
    tt.compare(got, tb, plain, dtype, f"config {name}")
    tt.compare_cuts([(got, tb)], dtype, f"config {name}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["RA", "RB", "RH"])
def test_mixed_with_page_and_slot_reuse(name, dtype, cases, tmp_path):
    folder, reqs, plain = cases(name, dtype)
    ps = tr.TINY[name]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_mixed(tb, reqs, np.random.default_rng(11), max_live=3)
    assert tb.pages_taken > tb.peak_tokens // ps, "the trace must make the pool hand pages out again"
    assert max(len(s["entries"]) for s in tb.steps) >= 3
    got = tt.run_trace(folder, dtype, tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"),
                       extra_args=["--max-live", "3"])          # three slots for six requests
    tt.compare(got, tb, plain, dtype, f"config {name} mixed")


def test_long_decoding(cases, tmp_path):
    folder, reqs, plain = cases("RB", "float32")
    ps = tr.TINY["RB"]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_tail_decode(tb, {"r3": reqs["r3"]}, tail=200)
    got = tt.run_trace(folder, "float32", tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"))
    tt.compare(got, tb, plain, "float32", "long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_sizes_of_the_tensor_core_kernels(dtype, cases, tmp_path):
    folder, reqs, plain = cases("RL", dtype)
    ps = tr.TINY["RL"]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_whole(tb, reqs)
    tt.trace_tail_decode(tb, reqs, tail=40)
    tt.trace_portions(tb, reqs, np.random.default_rng(3))
    tt.trace_mixed(tb, reqs, np.random.default_rng(5))
    got = tt.run_trace(folder, dtype, tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"))
    tt.compare(got, tb, plain, dtype, "config RL")
    tt.compare_cuts([(got, tb)], dtype, "config RL")


# ------------------------------------------------------------------ kernels
@pytest.fixture(scope="module")
def K():
    from crane_b200.kernels import get_kernels
    return get_kernels()


def _dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=dtype).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [48, 160, 1000])
def test_combine_layernorm(K, dtype, hidden):
    from crane_b200.kernels import Partials
    rng = np.random.default_rng(hidden)
    n, slots, used = 7, 5, 4                       # the new result is history entry 3
    x = rng.standard_normal((n, hidden)).astype(np.float32)
    hist = rng.standard_normal((slots, n, hidden)).astype(np.float32)
    a = _dev(rng.standard_normal((n, hidden)), dtype)
    f_parts = _dev(rng.standard_normal((3, n, hidden)))
    dwa = rng.standard_normal(used).astype(np.float32)
    w1, b1, w2, b2 = (rng.standard_normal(hidden).astype(np.float32) for _ in range(4))
    f_sum = f_parts.sum(0).to(dtype).double().cpu().numpy()          # partial sums are rounded once
    new = x.astype(np.float64) + (a.double().cpu().numpy() + f_sum)
    mixed = sum(dwa[j] * hist[j].astype(np.float64) for j in range(used - 1)) + dwa[used - 1] * new
    want1, want2 = pr.layer_norm(mixed, w1, b1, 1e-5), pr.layer_norm(mixed, w2, b2, 1e-5)
    xd, hd = _dev(x), _dev(hist)
    o1 = torch.empty(n, hidden, dtype=dtype, device=DEV)
    o2 = torch.empty_like(o1)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    # the wanted rows alone first: nothing but the outputs may change
    rows = _dev([5, 0, 5], torch.int32)
    g1 = torch.empty(3, hidden, dtype=dtype, device=DEV)
    K.combine_layernorm(xd, hd, used, a, Partials(f_parts), _dev(dwa), rows, _dev(w1), _dev(b1), g1,
                        None, None, None, 1e-5)
    assert np.array_equal(xd.cpu().numpy(), x) and np.array_equal(hd.cpu().numpy(), hist)
    assert np.abs(g1.double().cpu().numpy() - want1[[5, 0, 5]]).max() < tol * np.abs(want1).max()
    K.combine_layernorm(xd, hd, used, a, Partials(f_parts), _dev(dwa), None, _dev(w1), _dev(b1), o1,
                        _dev(w2), _dev(b2), o2, 1e-5)
    assert np.abs(xd.cpu().numpy() - mixed).max() < 1e-5 * np.abs(mixed).max()
    assert np.abs(hd[used - 1].cpu().numpy() - new).max() < 1e-5 * np.abs(new).max()
    assert np.array_equal(hd[used:].cpu().numpy(), hist[used:]) and np.array_equal(hd[:used - 1].cpu().numpy(), hist[:used - 1])
    assert np.abs(o1.double().cpu().numpy() - want1).max() < tol * np.abs(want1).max()
    assert np.abs(o2.double().cpu().numpy() - want2).max() < tol * np.abs(want2).max()
    # no average, one branch, one norm: the plain residual addition
    xd = _dev(x)
    K.combine_layernorm(xd, None, 1, None, a, None, None, _dev(w1), _dev(b1), o1, None, None, None, 1e-5)
    plain_sum = x.astype(np.float64) + a.double().cpu().numpy()
    assert np.abs(xd.cpu().numpy() - plain_sum).max() < 1e-5 * np.abs(plain_sum).max()
    assert np.abs(o1.double().cpu().numpy() - pr.layer_norm(plain_sum, w1, b1, 1e-5)).max() < tol * 4


def test_xielu(K):
    from crane_b200.kernels import Partials
    rng = np.random.default_rng(1)
    z = np.concatenate([rng.standard_normal(4000) * 3, [0.0, -1e-5, 1e-5, -30.0, 30.0]]).astype(np.float32)
    pq = np.array([0.4, -1.3], dtype=np.float32)
    out = torch.empty(len(z), dtype=torch.float32, device=DEV)
    K.xielu(_dev(z), out, _dev(pq))
    want = pr.xielu(z.astype(np.float64), 0.4, -1.3)
    assert np.abs(out.cpu().numpy() - want).max() < 1e-5 * np.abs(want).max()
    assert np.abs(out.cpu().numpy() - want)[np.abs(z) < 1].max() < 2e-6
    parts = _dev(rng.standard_normal((2, 10, 16)))
    out = torch.empty(10, 16, dtype=torch.bfloat16, device=DEV)
    K.xielu(Partials(parts), out, _dev(pq))
    want = pr.xielu(parts.sum(0).to(torch.bfloat16).double().cpu().numpy(), 0.4, -1.3)
    assert np.abs(out.double().cpu().numpy() - want).max() < 1e-2 * np.abs(want).max()


def test_embed_bigram_keeps_the_previous_token_per_slot(K):
    rng = np.random.default_rng(2)
    vocab, hidden, buckets, mp, mc = 50, 24, 13, 1000003, 7919
    table = rng.standard_normal((vocab, hidden)).astype(np.float32)
    big = rng.standard_normal((buckets + 1, hidden)).astype(np.float32)
    state = torch.full((4,), 77, dtype=torch.int32, device=DEV)        # what an earlier request left behind
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    seqs = {2: rng.integers(0, vocab, 9).tolist(), 0: rng.integers(0, vocab, 6).tolist()}     # slot -> tokens
    done = {2: 0, 0: 0}
    for cuts in ([(2, 4), (0, 1)], [(0, 3), (2, 1)], [(2, 4), (0, 2)]):
        toks, pos, ent, cu, slots, want = [], [], [], [0], [], []
        for e, (slot, n) in enumerate(cuts):
            part = seqs[slot][done[slot]:done[slot] + n]
            before = seqs[slot][done[slot] - 1] if done[slot] else None
            rows = pr.bigram_rows(part, buckets, mp, mc, before)
            want += [table[t] + big[r] for t, r in zip(part, rows)]
            toks += part
            pos += list(range(done[slot], done[slot] + n))
            ent += [e] * n
            cu.append(cu[-1] + n)
            slots.append(slot)
            done[slot] += n
        # a row of no entry and an entry without rows behind the real ones, as a padded step has them
        toks.append(3); pos.append(0); ent.append(-1); cu.append(cu[-1]); slots.append(1)
        x = torch.zeros(len(toks), hidden, device=DEV)
        K.embed_bigram(_dev(toks, torch.int32), _dev(table), _dev(big), x, buckets, mp, mc, _dev(pos, torch.int32),
                       _dev(ent, torch.int32), _dev(cu, torch.int32), _dev(slots, torch.int32), state, err)
        got = x.cpu().numpy()
        assert np.allclose(got[:-1], np.stack(want), atol=1e-6) and np.allclose(got[-1], table[3], atol=1e-6)
    assert state.tolist() == [seqs[0][5], 77, seqs[2][8], 77] and int(err.item()) == 0
    # slot 2 again, by a new request: its first token takes the table's last row whatever the slot holds
    x = torch.zeros(1, hidden, device=DEV)
    K.embed_bigram(_dev([4], torch.int32), _dev(table), _dev(big), x, buckets, mp, mc, _dev([0], torch.int32),
                   _dev([0], torch.int32), _dev([0, 1], torch.int32), _dev([2], torch.int32), state, err)
    assert np.allclose(x.cpu().numpy()[0], table[4] + big[buckets], atol=1e-6) and state.tolist()[2] == 4


# (the second and third shapes are ones that the tensor-core kernel takes in bfloat16: aligned rows,
# 16 | n_in, 8 | n_out, more than 16 tokens; the last fills its bounds)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n, H, n_in, n_out, cols, x_off, x_head, g_off",
                         [(37, 3, 20, 12, 150, 6, 25, 90), (150, 3, 32, 24, 256, 8, 40, 128),
                          (70, 2, 256, 256, 1040, 0, 264, 528)])
def test_head_linear(K, dtype, n, H, n_in, n_out, cols, x_off, x_head, g_off):
    rng = np.random.default_rng(3)
    src = _dev(rng.standard_normal((n, cols)), dtype)
    w = _dev(rng.standard_normal((H, n_in, n_out)) * 0.3, dtype)
    out = torch.zeros(n, H * n_out + 6, dtype=dtype, device=DEV)
    s64, w64 = src.double().cpu().numpy(), w.double().cpu().numpy()
    xs = np.stack([s64[:, x_off + h * x_head: x_off + h * x_head + n_in] for h in range(H)], 1)
    want = np.einsum("thi,hio->tho", xs, w64)
    K.head_linear(src, cols, x_off, x_head, w, n_in, n_out, out, H * n_out + 6, n_out, H)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    got = out.double().cpu().numpy()[:, :H * n_out].reshape(n, H, n_out)
    assert np.abs(got - want).max() < tol * np.abs(want).max()
    if cols % 8 == 0:
        # the operand left as two partial sums (a product cut along its inner dimension)
        from crane_b200.kernels import Partials
        half = _dev(rng.standard_normal((n, cols)))
        parts = torch.stack([half, src.float() - half]).contiguous()
        x2 = parts.sum(0).to(dtype).double().cpu().numpy()
        xs2 = np.stack([x2[:, x_off + h * x_head: x_off + h * x_head + n_in] for h in range(H)], 1)
        out2 = torch.zeros_like(out)
        K.head_linear(Partials(parts), cols, x_off, x_head, w, n_in, n_out, out2, H * n_out + 6, n_out, H)
        got_p = out2.double().cpu().numpy()[:, :H * n_out].reshape(n, H, n_out)
        assert np.abs(got_p - np.einsum("thi,hio->tho", xs2, w64)).max() < tol * np.abs(want).max()
    gate = s64[:, g_off:g_off + H * n_out].reshape(n, H, n_out)
    ent = np.zeros(n, dtype=np.int32)
    ent[5] = -1                                      # a row of no entry is left as it was
    K.head_linear(src, cols, x_off, x_head, w, n_in, n_out, out, H * n_out + 6, n_out, H, tok_entry=_dev(ent, torch.int32),
                  gate=src, g_cols=cols, g_off=g_off)
    got2 = out.double().cpu().numpy()[:, :H * n_out].reshape(n, H, n_out)
    want2 = want / (1 + np.exp(-gate))
    keep = ent >= 0
    assert np.abs(got2[keep] - want2[keep]).max() < 2 * tol * np.abs(want).max()
    assert np.array_equal(got2[5], got[5])
    assert float(out[:, H * n_out:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_prep(K, dtype):
    rng = np.random.default_rng(4)
    H, dim, rot, rank, dims, ps = 3, 10, 8, 24, 4, 8
    cols, dkv_off = H * (dim + rot) + 7 + rank + rot, H * (dim + rot) + 7
    n_pos = 64
    rotp = {"dims": dims, "base": 100.0, "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}}
    cos, sin = pr.yarn_tables(rotp, np.arange(n_pos))
    # two entries: positions 13..17 of one request (its pages 5, 2, 7) and position 8 of another (pages 0, 4)
    pos = [13, 14, 15, 16, 17, 8, 0]
    ent = [0, 0, 0, 0, 0, 1, -1]
    table = np.array([[5, 2, 7], [0, 4, -1]], dtype=np.int32)
    proj = _dev(rng.standard_normal((len(pos), cols)), dtype)
    nw = rng.standard_normal(rank).astype(np.float32)
    pool = torch.zeros(9, 1, ps, rank + rot, dtype=dtype, device=DEV)
    q_abs = torch.zeros(len(pos), H * (rank + rot), dtype=dtype, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.latent_prep(proj, cols, 0, dkv_off, H, dim, rot, rank, dims, _dev(cos), _dev(sin), _dev(pos, torch.int32),
                  _dev(ent, torch.int32), _dev(table, torch.int32), pool, ps, _dev(nw), 1e-5, q_abs, err)
    p64 = proj.double().cpu().numpy()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    got_pool, got_q = pool.double().cpu().numpy(), q_abs.double().cpu().numpy().reshape(len(pos), H, rank + rot)
    written = np.zeros((9, ps), bool)
    for t, (p, e) in enumerate(zip(pos, ent)):
        if e < 0:
            assert np.abs(got_q[t]).max() == 0
            continue
        c = pr.rms_norm(p64[t, dkv_off:dkv_off + rank], nw, 1e-5)
        kr = pr.rotate_pairs(p64[t:t + 1, dkv_off + rank:dkv_off + rank + rot], cos[p:p + 1], sin[p:p + 1], dims)[0]
        row = got_pool[table[e, p // ps], 0, p % ps]
        written[table[e, p // ps], p % ps] = True
        assert np.abs(row - np.concatenate([c, kr])).max() < tol * 4
        qr = p64[t, :H * (dim + rot)].reshape(H, dim + rot)[:, dim:]
        want = pr.rotate_pairs(qr[None], cos[p:p + 1], sin[p:p + 1], dims)[0]
        assert np.abs(got_q[t, :, rank:] - want).max() < tol * 4 and np.abs(got_q[t, :, :rank]).max() == 0
    assert np.abs(got_pool[:, 0][~written]).max() == 0 and int(err.item()) == 0
    # a layer that reads another's cache writes none
    pool.zero_()
    K.latent_prep(proj, cols, 0, -1, H, dim, rot, rank, dims, _dev(cos), _dev(sin), _dev(pos, torch.int32),
                  _dev(ent, torch.int32), _dev(table, torch.int32), pool, ps, None, 1e-5, q_abs, err)
    assert float(pool.abs().max()) == 0.0


def _latent_reference(q, rows, pos, rank, scale):
    """q [H, width] at position pos over cache rows [T, width]: values are the rows' leading columns."""
    s = (rows[:pos + 1] @ q.T) * scale
    p = np.exp(s - s.max(0))
    p /= p.sum(0)
    return p.T @ rows[:pos + 1, :rank]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank, rot, heads, ps", [(32, 8, 4, 16), (72, 4, 5, 8), (80, 16, 7, 32), (128, 32, 8, 64), (176, 48, 20, 16)])
def test_attention_in_the_latent_space_with_planted_keys(K, dtype, rank, rot, heads, ps):
    """A prompt portion and single tokens over long cached contexts; for some queries one key
    (far back, first of all, at a page's last and first place, the newest) is made to stand out
    so that the output is that row or visibly not."""
    from crane_b200.parts.latent_attention import latent_attention_kernel
    rng = np.random.default_rng(rank + heads)
    width, scale = rank + rot, 0.2
    lens = [700, 3 * ps + 1, 2 * ps, 45]           # cached length after the step, per entry
    q_lens = [37, 1, 1, 45]
    planted = {0: [(0, 0), (5, 2 * ps - 1), (20, 2 * ps), (36, 699)], 1: [(0, 3)], 2: [(0, ps - 1)], 3: [(44, 0), (10, 10)]}
    rows = [rng.standard_normal((n, width)) * 0.5 for n in lens]
    n_pages = sum(-(-n // ps) for n in lens) + 2
    order = rng.permutation(n_pages)
    pool = (torch.randn(n_pages, 1, ps, width, device=DEV) * 30).to(dtype)          # never to be read
    table = -np.ones((len(lens), max(-(-n // ps) for n in lens)), dtype=np.int32)
    nxt = 0
    for e, r in enumerate(rows):
        for b in range(-(-len(r) // ps)):
            table[e, b] = order[nxt]; nxt += 1
            chunk = r[b * ps:(b + 1) * ps]
            pool[int(table[e, b]), 0, :len(chunk)] = _dev(chunk, dtype)
    rows = [pool[torch.as_tensor(table[e][table[e] >= 0].astype(np.int64)).to(DEV), 0].reshape(-1, width)[:lens[e]]
            .double().cpu().numpy() for e in range(len(lens))]
    qs, pos, ent, cu = [], [], [], [0]
    for e, (n, ql) in enumerate(zip(lens, q_lens)):
        q = rng.standard_normal((ql, heads, width)) * 0.5
        for t, key in planted[e]:
            q[t, 1 % heads] = rows[e][key] * 40.0 / max(1e-6, (rows[e][key] ** 2).sum() * scale)     # score 40 there
        qs.append(q)
        pos += list(range(n - ql, n)); ent += [e] * ql; cu.append(cu[-1] + ql)
    q_all = _dev(np.concatenate(qs).reshape(-1, heads * width), dtype)
    out = torch.zeros(q_all.shape[0], heads * rank, dtype=dtype, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    latent_attention_kernel(K, q_all, out, pool, _dev(pos, torch.int32), _dev(ent, torch.int32), _dev(cu, torch.int32),
                            _dev(lens, torch.int32), np.asarray(cu), np.asarray(lens), _dev(table, torch.int32), ps,
                            heads, rank, rot, scale, err, exact=dtype == torch.float32)
    got = out.double().cpu().numpy().reshape(-1, heads, rank)
    q64 = q_all.double().cpu().numpy().reshape(-1, heads, width)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for i, (p, e) in enumerate(zip(pos, ent)):
        want = _latent_reference(q64[i], rows[e], p, rank, scale)
        assert np.abs(got[i] - want).max() < tol * max(1.0, np.abs(want).max()), (i, p, e)
    for e in planted:
        for t, key in planted[e]:
            i = cu[e] + t
            if key <= pos[i]:                       # a planted key that the query sees is (nearly) all it gets
                assert np.abs(got[i, 1 % heads] - rows[e][key, :rank]).max() < 0.05, (e, t, key)
    assert int(err.item()) == 0


# ---------------------------------------------------------------- generation
def _load(folder, dtype, **opts):
    from crane_b200.generation import ModelForCausalLM
    return ModelForCausalLM.from_pretrained(folder, dtype, **opts)


def _greedy(n):
    from crane_b200.generation import GenerationConfig
    return GenerationConfig(max_new_tokens=n, temperature=None, eos_token_id=-1)


@pytest.mark.parametrize("name", ["RA", "RB", "RC"])
def test_greedy_generation_float32_equals_plain(name, model_folders):
    folder = model_folders(name, "float32")
    cfg, w = pr.load_folder(folder)
    m = _load(folder, "fp32", page_size=tr.TINY[name]["page_size"], num_pages=24, max_concurrent=3,
              max_batched_tokens=64, max_seq_len=256)
    rng = np.random.default_rng(3)
    for n in (1, 5, 17):
        prompt = rng.integers(0, cfg["vocab"], n).tolist()
        assert m.generate(prompt, _greedy(8)) == pr.greedy_generate(cfg, w, prompt, 8)
    m.runner.table.check()
    assert m.runner.table.live() == 0


@pytest.mark.parametrize("name", ["RA", "RL"])
def test_greedy_batch_bfloat16_through_the_scheduler(name, model_folders):
    """Six prompts, three slots, portions of at most 16 tokens: requests wait, slots and pages are
    used again, and decode steps replay graphs with the bigram state in them."""
    folder = model_folders(name, "bfloat16")
    cfg, w = pr.load_folder(folder)
    m = _load(folder, "bf16", page_size=16, num_pages=40, max_concurrent=3, max_batched_tokens=48, chunk_size=16,
              max_seq_len=256)
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (12, 3, 40, 1, 25, 7)]
    outs = m.generate_batch(prompts, _greedy(20))
    for prompt, toks in zip(prompts, outs):
        assert len(toks) == len(prompt) + 20 and toks[:len(prompt)] == prompt
        logits = pr.logits_all(cfg, w, toks[:-1])
        for i in range(len(prompt), len(toks)):
            row = logits[i - 1]
            assert row[toks[i]] >= row.max() - 3e-2 * np.abs(row).max(), (i, toks[i], int(row.argmax()))
    m.runner.table.check()
    assert m.runner.table.live() == 0


def test_command_line(model_folders):
    """bin/crane picks the model class from config.json; sampling with a temperature runs too."""
    import os
    import subprocess
    import sys
    folder = model_folders("RA", "float32")
    cfg, w = pr.load_folder(folder)
    crane = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "crane")
    cmd = [sys.executable, crane, "-m", folder, "--dtype", "fp32", "--prompt-ids", "5,6,7", "--max-new-tokens", "6",
           "--eos-token-id", "-1", "--page-size", "16", "--num-pages", "8", "-c", "2", "--max-batched-tokens", "32",
           "--max-seq-len", "64"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-3000:]
    assert p.stdout.strip().splitlines()[-1] == ",".join(map(str, pr.greedy_generate(cfg, w, [5, 6, 7], 6)[3:]))
    p = subprocess.run(cmd + ["--temperature", "0.8", "--top-k", "20", "--top-p", "0.9", "--random-weights", "--seed", "3"],
                       capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-3000:]
    assert len(p.stdout.strip().splitlines()[-1].split(",")) == 6
