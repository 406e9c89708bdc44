"""The Ledudra decoder on the GPU against the plain implementation: each mechanism's kernel alone, then whole models
through the engine under every way of cutting the work into steps, portions and batches, and greedy generation through
the library's entry point.  Configurations and weights are made here (``tiny_ledudra``)."""
import math

import pytest
import torch

import plain_ledudra as PL
from helpers import assert_close
from test_gpu_vemedra import portions, step_ctx
from tiny import random_tokens
from tiny_ledudra import CONFIGS, folder, oracle, oracle_logits

pytestmark = pytest.mark.gpu

NAMES = ["LA", "LB", "LF"]
DTYPES = ["float32", "bfloat16"]
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


# ---------------------------------------------------------------------------------------------------------------
# each mechanism alone
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [40, 192, 300, 1100, 2560])
def test_branch_norm_sum_layer_norm_and_token_shift_over_portions(width, dtype):
    """h += mult * ln_b(delta + bias), y = ln(h), out = y + (y_before - y) * shift, the last y carried in each sequence's
    slot: portions of many sizes down to single tokens, unequal sequences in one step, first tokens (zeros before)."""
    from synaptix_b200 import ops
    g = torch.Generator().manual_seed(width)
    lengths, slots = [23, 41, 5], [2, 0, 3]
    h0 = [torch.randn(n, width, generator=g) * 2 + 0.5 for n in lengths]
    delta = [(torch.randn(n, width, generator=g) * 3 + 1).to(DT[dtype]) for n in lengths]
    vec = lambda s=0.3, m=0.0: (m + s * torch.randn(width, generator=g))
    w, b, pw, pb, db, shift = vec(0.3, 1), vec(), vec(0.3, 1), vec(), vec(1.0), vec(0.5, 0.5)
    mult, eps = 0.6, 1e-5
    state = torch.full((5, width), float("nan")).cuda()
    state[slots] = 0.0
    ref_h = [a.double() + mult * PL.layer_norm(d.double() + db.double(), pw.double(), pb.double(), eps) for a, d in zip(h0, delta)]
    ref = [PL.token_shift(PL.layer_norm(x, w.double(), b.double(), eps), shift.double()) for x in ref_h]
    got = [torch.zeros(n, width) for n in lengths]
    for past, new, who in portions(lengths, [3, 1, 1, 2, 7, 1, 64]):
        ctx = step_ctx(past, new, [slots[i] for i in who], dtype=DT[dtype])
        h = torch.cat([h0[i][p:p + n] for i, p, n in zip(who, past, new)]).cuda()
        d = torch.cat([delta[i][p:p + n] for i, p, n in zip(who, past, new)]).cuda()
        out, h_after = ops.add_layernorm(h, d, w.cuda(), b.cuda(), eps, DT[dtype], post=(pw.cuda(), pb.cuda()), mult=mult,
                                         delta_bias=db.cuda(), shift=shift.cuda(), state=state, ctx=ctx,
                                         in_place=ctx.all_single)
        want_h = torch.cat([ref_h[i][p:p + n] for i, p, n in zip(who, past, new)])
        assert torch.allclose(h_after.cpu().double(), want_h, atol=2e-5, rtol=1e-5)
        out = out.float().cpu()
        t = 0
        for i, p, n in zip(who, past, new):
            got[i][p:p + n] = out[t:t + n]
            t += n
    tol = dict(atol=3e-5, rtol=3e-5) if dtype == "float32" else dict(atol=3e-2, rtol=2e-2)
    for a, r in zip(got, ref):
        assert torch.allclose(a.double(), r, **tol), float((a.double() - r).abs().max())
    assert torch.isnan(state[[1, 4]]).all()                # slots of no sequence were not touched


@pytest.mark.parametrize("dtype", DTYPES)
def test_layer_norm_of_chosen_rows_and_a_plain_delta(dtype):
    from synaptix_b200 import ops
    g = torch.Generator().manual_seed(2)
    W = 72
    h = torch.randn(9, W, generator=g)
    d = torch.randn(9, W, generator=g).to(DT[dtype])
    w, b = 1 + 0.2 * torch.randn(W, generator=g), 0.3 * torch.randn(W, generator=g)
    rows = torch.tensor([7, 0, 3], dtype=torch.int32)
    hc = h.clone().cuda()
    out, _ = ops.add_layernorm(hc, d.cuda(), w.cuda(), b.cuda(), 1e-6, DT[dtype], mult=0.5, rows=rows.cuda())
    ref = PL.layer_norm(h.double() + 0.5 * d.double(), w.double(), b.double(), 1e-6)[rows.long()]
    assert torch.equal(hc.cpu(), h)                         # chosen rows: nothing is written back
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == "float32" else dict(atol=3e-2, rtol=2e-2)
    assert torch.allclose(out.float().cpu().double(), ref, **tol)
    out, h2 = ops.add_layernorm(hc, None, w.cuda(), b.cuda(), 1e-6, DT[dtype])
    assert torch.allclose(out.float().cpu().double(), PL.layer_norm(h.double(), w.double(), b.double(), 1e-6), **tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,Dv,rot,norm", [(6, 2, 16, 12, (8, 1.0e4, dict(factor=4.0, original=64, fast=16.0, slow=2.0)), False),
                                                (4, 4, 24, 40, (24, 500.0, None), True), (2, 1, 64, 64, None, True),
                                                (3, 1, 10, 7, (6, 100.0, dict(factor=2.0, original=16, fast=4.0, slow=1.0)), False)])
def test_head_preparation(H, G, D, Dv, rot, norm, dtype):
    """Bias, shared-gain RMS norm, rotation of neighbouring pairs (also with stretched frequencies and their magnitude),
    blend of the values with another layer's, cache write at page borders, head gates."""
    from synaptix_b200 import ops
    from synaptix_b200.parts import FrequencyRamp, RotaryPairs, Runtime
    g = torch.Generator().manual_seed(H * D + Dv)
    T = 140
    pos = torch.arange(T) + 50                              # crosses the borders at 64, 128 and 192
    cols = (H + G) * D + G * Dv + H
    proj = torch.randn(T, cols, generator=g)
    bias = torch.randn(cols, generator=g) * 0.5
    qn, kn = 1 + 0.3 * torch.randn(D, generator=g), 1 + 0.3 * torch.randn(D, generator=g)
    vf = torch.randn(T, G * Dv, generator=g)
    lam = torch.tensor([0.3])
    x = (proj + bias).double()
    q, k = x[:, :H * D].view(T, H, D), x[:, H * D:(H + G) * D].view(T, G, D)
    v, gate = x[:, (H + G) * D:(H + G) * D + G * Dv], torch.sigmoid(x[:, -H:])
    if norm:
        q, k = PL.rms_unit(q, 1e-5) * qn.double(), PL.rms_unit(k, 1e-5) * kn.double()
    inv_freq, mag, dims = None, 1.0, 0
    if rot:
        dims, base, sc = rot
        q, k = PL.rotate_pairs(q, pos, dims, base, sc), PL.rotate_pairs(k, pos, dims, base, sc)
        enc = RotaryPairs(D, base, rotary_dim=dims, scaling=FrequencyRamp(**sc) if sc else None)
        enc.bind({}, Runtime(torch.device("cuda:0"), DT[dtype]))
        inv_freq, mag = enc.rotation()[0], enc.magnitude
    v = PL.mix_values(v, vf.double(), 0.3)
    dt = DT[dtype]
    kp = torch.full((6, G, 64, D), float("nan"), dtype=dt).cuda()
    vp = torch.full((6, G, 64, Dv), float("nan"), dtype=dt).cuda()
    table = torch.tensor([[4, 2, 5, 1]], dtype=torch.int32).cuda()
    qo = torch.empty(T, H * D, dtype=dt).cuda()
    go = torch.empty(T, H).cuda()
    vout = torch.empty(T, G * Dv).cuda()
    ops.heads_prepare(proj.cuda(), bias.cuda(), qo, kp, vp, pos.int().cuda(), torch.zeros(T, dtype=torch.int32).cuda(), table,
                      H, G, D, Dv, q_gain=qn.cuda() if norm else None, k_gain=kn.cuda() if norm else None, eps=1e-5,
                      inv_freq=inv_freq, rot_dims=dims, magnitude=mag, v_first_in=vf.cuda(), v_first_out=vout,
                      lam=lam.cuda(), gate_out=go)
    tol = dict(atol=3e-5, rtol=3e-5) if dtype == "float32" else dict(atol=3e-2, rtol=1e-2)
    assert torch.allclose(qo.float().cpu().double().view(T, H, D), q, **tol)
    assert torch.allclose(go.cpu().double(), gate, atol=1e-6)
    assert torch.allclose(vout.cpu().double(), v, atol=1e-5)
    pages = [4, 2, 5, 1]
    kc = torch.stack([kp[pages[int(p) // 64], :, int(p) % 64] for p in pos]).float().cpu().double()
    vc = torch.stack([vp[pages[int(p) // 64], :, int(p) % 64] for p in pos]).float().cpu().double()
    assert torch.allclose(kc, k, **tol) and torch.allclose(vc.reshape(T, -1), v, **tol)
    assert torch.isnan(kp[[0, 3]].float()).all()            # pages of nobody were not written


def _spiked(T, H, G, D, window, g, extra=()):
    """Queries, keys: the keys at the window's edge of some queries, at page borders and far back are six times the
    others', and those queries point at them: a key seen one place too far, or not far enough, changes the result by
    far more than the tolerance."""
    q = torch.randn(T, H, D, generator=g) * 0.5
    k = torch.randn(T, G, D, generator=g) * 0.5
    spikes = sorted({2, 63, 64, 127, 128, 191, 192} | set(extra))
    for j in spikes:
        if j >= T:
            continue
        k[j] *= 6.0
        look = [j, j + 1] + ([j + window - 1, j + window] if window else [T - 1])     # the last query that sees it, the first that does not
        for t in look:
            if 0 <= t < T:
                q[t] = 0.4 * q[t] + k[j].repeat_interleave(H // G, dim=0) / 6.0
    return q, k


def _run_attention(q, k, v, H, G, D, Dv, scale, window, steps, dt, **kw):
    """Write keys and values of each step into pages and attend; steps are (past, new) of one sequence."""
    from synaptix_b200 import ops
    T = q.shape[0]
    kp = torch.full((7, G, 64, D), float("nan"), dtype=dt).cuda()
    vp = torch.full((7, G, 64, Dv), float("nan"), dtype=dt).cuda()
    table = torch.tensor([[4, 2, 5, 1, 6, 3]], dtype=torch.int32).cuda()
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1).float().cuda()
    got = []
    for past, new in steps:
        ctx = step_ctx([past], [new], [0], [table], dtype=dt)
        qq = torch.empty(new, H * D, dtype=dt).cuda()
        ops.heads_prepare(proj[past:past + new].contiguous(), None, qq, kp, vp, ctx.positions, ctx.seq_of_token, table, H, G, D, Dv)
        gate = kw.get("gate")
        got.append(ops.attn_scored(qq, kp, vp, ctx, table, H, G, D, Dv, scale, window,
                                   **dict(kw, gate=None if gate is None else gate[past:past + new].contiguous())).float().cpu())
    return torch.cat(got).view(T, H, Dv)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,Dv,window", [(6, 2, 16, 12, 37), (8, 4, 64, 32, 150), (2, 2, 8, 40, None), (3, 1, 24, 10, 64),
                                              (8, 1, 64, 64, 300), (1, 1, 32, 8, 1), (16, 4, 128, 64, 100), (32, 8, 64, 64, 37),
                                              (8, 8, 128, 128, None), (16, 2, 64, 128, 70), (32, 4, 128, 128, 129), (8, 2, 32, 32, 50), (16, 16, 32, 64, 65)])
def test_sigmoid_attention_with_scores_mixed_over_heads(H, G, D, Dv, window, dtype):
    """A portion, then token by token (the keys cut into parts over the grid), the whole sequence in portions of two, and
    portions whose lengths are no multiple of a block's rows.  (In bfloat16 the shapes of 8, 16 and 32 heads of size 32, 64 or
    128 run their portions on the tensor cores.)"""
    g = torch.Generator().manual_seed(H * D + Dv)
    T, cut = 330, 200
    edge = [cut - window, cut - window + 1] if window and window < cut else []
    q, k = _spiked(T, H, G, D, window, g, extra=edge)
    v = torch.randn(T, G, Dv, generator=g)
    talk = torch.eye(H) + 0.4 * torch.randn(H, H, generator=g)
    pb = torch.randn(H, generator=g) - 2.0
    gate = torch.rand(T, H, generator=g)
    dt = DT[dtype]
    q, k, v = q.to(dt), k.to(dt), v.to(dt)
    scale = 1.2 / math.sqrt(D)
    ref = PL.sigmoid_mixed_heads(q.double(), k.double(), v.double(), torch.arange(T), scale, talk.double(), pb.double(), window)
    ref = ref * gate.double()[:, :, None]
    kw = dict(talk=talk.cuda(), head_bias=pb.cuda(), gate=gate.cuda())
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == "float32" else dict(atol=6e-2, rtol=3e-2)
    for steps in ([(0, cut)] + [(p, 1) for p in range(cut, T)], [(p, 2) for p in range(0, T, 2)], [(0, 3), (3, T - 3)],
                  [(0, 13), (13, 99), (112, 9), (121, T - 121)]):
        got = _run_attention(q, k, v, H, G, D, Dv, scale, window, steps, dt, **kw)
        bad = (got.double() - ref).abs().amax(dim=(1, 2))
        assert torch.allclose(got.double(), ref, **tol), f"first wrong query {int((bad > tol['atol'] + tol['rtol'] * ref.abs().max()).nonzero()[0])}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,Dv,window,rows,far", [(4, 2, 8, 12, 70, 10, 50), (8, 4, 64, 32, 150, 16, 100), (3, 3, 16, 16, None, 2, 3),
                                                       (2, 1, 24, 20, 9, 6, 7), (4, 1, 64, 64, 130, 32, 128), (6, 2, 32, 32, None, 12, 40),
                                                       (4, 2, 128, 128, 70, 8, 200), (16, 1, 64, 64, 64, 64, 65)])
def test_softmax_attention_with_a_bias_per_distance_bucket(H, G, D, Dv, window, rows, far, dtype):
    """The table holds large numbers, one bucket after the other favoured per head, so a distance that falls into the
    wrong bucket moves the weights by far more than the tolerance; the last bucket (every far distance) among them."""
    from synaptix_b200.parts.scored import distance_columns
    g = torch.Generator().manual_seed(H * D + rows)
    T, cut = 300, 170
    q, k = _spiked(T, H, G, D, window, g)
    v = torch.randn(T, G, Dv, generator=g)
    rel = torch.randn(rows, H, generator=g)
    for h in range(H):
        rel[(h * 3 + 1) % rows, h] += 4.0
    rel[rows - 1, 0] += 3.0
    dt = DT[dtype]
    q, k, v = q.to(dt), k.to(dt), v.to(dt)
    scale = 1.0 / math.sqrt(D)
    ref = PL.biased_softmax_heads(q.double(), k.double(), v.double(), torch.arange(T), scale, rel.double(), far, window)
    cols = distance_columns(rows, far, window)
    table = rel[torch.from_numpy(cols)].t().contiguous().cuda()
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == "float32" else dict(atol=4e-2, rtol=3e-2)
    # the last schedule's portions start and end inside pages and inside the 64-row tiles of the tensor-core kernel
    for steps in ([(0, cut)] + [(p, 1) for p in range(cut, T)], [(p, 5) for p in range(0, T, 5)],
                  [(0, 100), (100, 64), (164, 17), (181, T - 181)]):
        got = _run_attention(q, k, v, H, G, D, Dv, scale, window, steps, dt, dist_bias=table, softmax=True)
        assert torch.allclose(got.double(), ref, **tol), float((got.double() - ref).abs().max())


# ---------------------------------------------------------------------------------------------------------------
# whole models through the engine
# ---------------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def engines():
    from synaptix_b200.engine import Engine
    from synaptix_b200.models import load_model
    made = {}

    def get(name, dtype, max_tokens=2048, max_seqs=None):
        key = (name, dtype, max_tokens, max_seqs)
        if key not in made:
            eng = Engine(load_model(folder(name), dtype=dtype), max_tokens=max_tokens, max_seqs=max_seqs)
            for t in eng.cache._k + eng.cache._v:          # a kernel that reads a place no step wrote shows at once
                t.fill_(float("nan"))
            made[key] = eng
        assert made[key].cache.slots.n_live == 0
        return made[key]
    return get


def vocab(name):
    return CONFIGS[name][0]["vocab"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_every_place(engines, name, dtype):
    from synaptix_b200.engine import Entry
    eng = engines(name, dtype)
    assert type(eng.model.config).__name__ == "LedudraConfig" and eng.use_graphs
    for i, n in enumerate([1, 2, 3, 17, 64, 65, 150, 301]):
        toks = random_tokens(vocab(name), n, 100 + i)
        s = eng.open()
        got = eng.step([Entry(s, toks, list(range(n)))])
        eng.close(s)
        assert_close(got, oracle_logits(name, tuple(toks)), dtype, f"{name} {dtype} whole n={n}")


@pytest.mark.parametrize("name", NAMES)
def test_the_stream_after_every_layer(engines, name):
    from synaptix_b200.engine import Entry
    eng = engines(name, "float32")
    toks = random_tokens(vocab(name), 90, 4)
    cfg, W = oracle(name)
    _, ref = PL.forward(cfg, W, toks, return_layers=True)
    seen = []
    s = eng.open()
    entries = [Entry(s, toks, [0])]
    past, new = eng._check(entries)
    ctx = eng.plan(entries, past, new)
    ctx.observe = lambda n, h, pending: seen.append((h + pending.float()).cpu() if pending is not None else h.cpu().clone())
    eng._forward(ctx)
    eng.cache.slots.advance(s, len(toks))
    eng.close(s)
    assert len(seen) == len(ref)
    for i, (a, b) in enumerate(zip(seen, ref)):
        assert torch.allclose(a.double(), b, atol=2e-4 * float(b.abs().max())), f"{name}: layer {i}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_token_by_token_from_the_first_token(engines, name, dtype):
    """Every token a step of its own (captured steps): the first tokens of a sequence, whose shift begins from zeros,
    and on across window and page borders."""
    from synaptix_b200.engine import Entry
    eng = engines(name, dtype)
    toks = random_tokens(vocab(name), 150, 8)
    ref = oracle_logits(name, tuple(toks))
    s = eng.open()
    got = torch.cat([eng.step([Entry(s, [t], [0])]) for t in toks])
    eng.close(s)
    assert_close(got, ref, dtype, f"{name} {dtype} token by token")
    assert any(c.graph is not None for c in eng._captured.values())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("size", [2, 3, 7, 64, 100])
def test_prompts_in_portions(engines, name, dtype, size):
    from synaptix_b200.engine import Entry
    eng = engines(name, dtype)
    toks = random_tokens(vocab(name), 277, 20 + size)
    ref = oracle_logits(name, tuple(toks))
    s = eng.open()
    got = [eng.step([Entry(s, toks[a:a + size], list(range(len(toks[a:a + size]))))]) for a in range(0, len(toks), size)]
    eng.close(s)
    assert_close(torch.cat(got), ref, dtype, f"{name} {dtype} portions of {size}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_in_slots_and_pages_used_again(engines, name, dtype):
    """Batches of unequal prompts decoded together, shorter requests ending earlier; the cache holds little more than one
    batch and three slots, so every batch runs in slots, states and pages that the batch before gave back."""
    from synaptix_b200.engine import Entry
    eng = engines(name, dtype, max_tokens=512, max_seqs=3)
    V = vocab(name)
    for b, (lens, decodes) in enumerate([([5, 130, 1], [3, 40, 12]), ([64, 9, 200], [10, 30, 2]), ([2, 3, 100], [25, 1, 70])]):
        seqs = [random_tokens(V, n + d, 300 + 10 * b + i) for i, (n, d) in enumerate(zip(lens, decodes))]
        refs = [oracle_logits(name, tuple(s)) for s in seqs]
        slots = [eng.open() for _ in seqs]
        got = eng.step([Entry(s, q[:n], [n - 1]) for s, q, n in zip(slots, seqs, lens)])
        assert_close(got, torch.stack([r[n - 1] for r, n in zip(refs, lens)]), dtype, f"{name} batch {b} prompts")
        live = list(range(len(seqs)))
        for j in range(max(decodes)):
            live = [i for i in live if j < decodes[i]]
            got = eng.step([Entry(slots[i], [seqs[i][lens[i] + j]], [0]) for i in live])
            assert_close(got, torch.stack([refs[i][lens[i] + j] for i in live]), dtype, f"{name} batch {b} decode {j}")
            for i in live:
                if j == decodes[i] - 1:
                    eng.close(slots[i])
    assert eng.cache.slots.n_live == 0


@pytest.mark.parametrize("name", ["LA", "LF"])
def test_long_decoding_gives_pages_behind_the_window_back(engines, name):
    """400 tokens one by one behind a prompt, in a cache of 5 pages: it only fits because pages that every layer's window
    has passed are given back (windows of 9 to 200 positions in these models)."""
    from synaptix_b200.engine import Entry
    eng = engines(name, "float32", max_tokens=320)
    toks = random_tokens(vocab(name), 90 + 400, 77)
    ref = oracle_logits(name, tuple(toks))
    s = eng.open()
    got = [eng.step([Entry(s, toks[:90], [89])])]
    for t in toks[90:]:
        got.append(eng.step([Entry(s, [t], [0])]))
    assert any(-1 in eng.cache.slots.table(s, g) for g in range(eng.cache.n_block_tables))
    eng.close(s)
    assert_close(torch.cat(got), ref[89:], "float32", f"{name} long decoding")


@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_entry_point(name):
    """``LLM.generate`` (scheduler, decode sessions, sampling on the device): greedy tokens of unequal prompts in one
    batch equal the plain implementation's, each computed alone."""
    import synaptix_b200
    llm = synaptix_b200.LLM(folder(name), compute_dtype="float32", max_tokens=1024)
    V = vocab(name)
    prompts = [random_tokens(V, n, 900 + n) for n in (3, 41, 1, 18)]
    out = llm.generate(prompts, max_new_tokens=12, temperature=0.0)
    cfg, W = oracle(name)
    for p, new in zip(prompts, out):
        seq = list(p)
        for tok in new:
            lg = PL.forward(cfg, W, seq)[-1]
            top2 = lg.topk(2).values
            if float(top2[0] - top2[1]) > 1e-3 * float(lg.abs().max()):       # a near tie may fall either way
                assert tok == int(lg.argmax()), f"{name}: token {len(seq) - len(p)} of prompt of {len(p)}"
            seq.append(tok)
        assert len(new) == 12
    out2 = llm.generate(prompts, max_new_tokens=12, temperature=0.0, prefill_batch=5)
    assert out2 == out


@pytest.mark.parametrize("dtype", DTYPES)
def test_replay_program_with_a_batch_whose_requests_end_at_different_times(tmp_path, dtype):
    from test_gpu_trace_run import Replay
    name = "LA"
    V = vocab(name)
    seqs = {f"q{i}": random_tokens(V, n, 800 + i) for i, n in enumerate([31, 75, 12, 50])}
    refs = {k: oracle_logits(name, tuple(v)) for k, v in seqs.items()}
    r = Replay(folder(name), dtype, str(tmp_path), 192)
    heads = {"q0": 20, "q1": 60, "q2": 11}
    got = r.step([{"id": k, "tokens": seqs[k][:h], "want": [0, h - 1]} for k, h in heads.items()])
    assert_close(got, torch.stack([refs[k][j] for k, h in heads.items() for j in (0, h - 1)]), dtype, "replay: prompts")
    at = dict(heads)
    while at:
        live = list(at)
        ends = [k for k in live if at[k] + 1 == len(seqs[k])]
        got = r.step([{"id": k, "tokens": [seqs[k][at[k]]], "want": [0]} for k in live], end=ends)
        assert_close(got, torch.stack([refs[k][at[k]] for k in live]), dtype, f"replay: decode {sorted(at.values())}")
        for k in live:
            at[k] += 1
            if k in ends:
                del at[k]
    got = r.step([{"id": "q3", "tokens": seqs["q3"], "want": [49]}], end=["q3"])
    assert_close(got, refs["q3"][49:50], dtype, "replay: afterwards")
    r.finish()


def test_command_line_run_and_inspect(tmp_path):
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name = "LB"
    cfg, W = oracle(name)
    prompt = random_tokens(vocab(name), 9, 1300)
    env = dict(os.environ, PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-m", "synaptix_b200", "run", folder(name), ",".join(map(str, prompt)),
                        "--max-tokens", "6", "--temperature", "0", "--compute-dtype", "f32", "--stop-ids", "", "--json"],
                       capture_output=True, text=True, env=env, cwd=str(tmp_path))
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout.strip().splitlines()[-1])
    seq = list(prompt)
    for tok in out["outputs"][0]["tokens"]:
        lg = PL.forward(cfg, W, seq)[-1]
        top2 = lg.topk(2).values
        if float(top2[0] - top2[1]) > 1e-3 * float(lg.abs().max()):
            assert tok == int(lg.argmax())
        seq.append(tok)
    r = subprocess.run([sys.executable, "-m", "synaptix_b200", "inspect", folder(name)], capture_output=True, text=True, env=env)
    assert r.returncode == 0 and "Ledudra" in r.stdout and "layer 2: attention, no feed-forward" in r.stdout
