"""The Gamilorn design on the GPU against the plain implementation of ``tests/plain_gamilorn.py``:
each new kernel alone (inputs made so that one far key, a key just inside or just outside the
window or the kept first keys, a page's border or a lost state would show), then whole models
through ``bin/trace_run`` (whole prompts, the last tokens one by one over more tokens than the
windows are long, portions down to two tokens, mixed batches in a pool so small that pages
and state slots are used again), in float32 and bfloat16, and greedy generation through
``Engine.generate``."""

import math
from types import SimpleNamespace

import pytest
import torch

from tests import gamilorn_util as gu
from tests import plain_gamilorn as pg
from tests import replay_util as ru

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    return {name: gu.write_tiny(name, tmp_path_factory.mktemp(f"gamilorn_{name}")) for name in gu.CONFIGS}


def close(got, want, dtype, what, f32=2e-5, bf16=1.2e-2):
    got, want = got.double().cpu(), want.double().cpu()
    scale = float(want.abs().max())
    err = float((got - want).abs().max())
    bound = (f32 if dtype == "float32" else bf16) * max(scale, 1e-6)
    assert err <= bound, f"{what} ({dtype}): abs diff {err:.4g} exceeds {bound:.4g} (scale {scale:.4g})"


# ---- small kernels -------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", list(DTYPES))
def test_stream_kernels_alone(dtype):
    from deterministic_inference_b200.kernels import ops
    dt, dev = DTYPES[dtype], "cuda"
    g = torch.Generator().manual_seed(1)
    rows, width = 37, 136
    ids = torch.randint(0, 50, (rows,), generator=g, dtype=torch.int32)
    pos = torch.randint(0, 70, (rows,), generator=g, dtype=torch.int32)
    table, ptable = (torch.randn(n, width, generator=g).to(dt) for n in (50, 70))
    x = ops.embedding_positions(ids.to(dev), pos.to(dev), table.to(dev), ptable.to(dev))
    assert x.dtype == torch.float32
    want = table.double()[ids.long()] + ptable.double()[pos.long()]
    close(x, want, "float32", "embedding + position")

    # the stream takes two scaled terms (a stored tensor and split partial products) in float32
    w = torch.randn(width, generator=g) * 0.1
    a = torch.randn(rows, width, generator=g).to(dt)
    parts = torch.randn(3, rows, width, generator=g)
    stream = x.clone()
    y = ops.stream_rms_norm(stream, (1.0 + w).to(dev), 3e-5, dt,
                            add=ops.WeightedSum([(1.2, a.to(dev)), (0.7, ops.SplitSum(parts.to(dev), torch.float32))]))
    total = want + 1.2 * a.double() + 0.7 * parts.double().sum(0)
    close(stream, total, "float32", "stream after the addition")
    close(y, pg.zero_centred_norm(total, w.double(), 3e-5), dtype, "norm of the stream")
    close(ops.stream_rms_norm(stream, (1.0 + w).to(dev), 3e-5, dt), pg.zero_centred_norm(total, w.double(), 3e-5),
          dtype, "norm alone")

    z = torch.randn(rows, width, generator=g) * 3
    p, q = torch.tensor(0.3), torch.tensor(-0.8)
    sp = torch.nn.functional.softplus
    got = ops.xielu(z.to(dev), float(sp(p)), float(0.5 + sp(q)), dt)
    close(got, pg.xielu(z.double(), p.double(), q.double()), dtype, "xielu")
    logits = torch.randn(5, 77, generator=g) * 20
    close(ops.softcap_(logits.clone().to(dev), 11.0), pg.softcap(logits.double(), 11.0), "float32", "soft cap")


# ---- attention without a softmax ---------------------------------------------------------------------

def paged(n_tokens_per_seq, page, generator):
    """Block tables over shuffled pages for sequences of the given lengths."""
    need = [-(-n // page) for n in n_tokens_per_seq]
    perm = (torch.randperm(sum(need), generator=generator) + 1).tolist()
    bt = torch.zeros(len(need), max(need), dtype=torch.int32)
    for b, n in enumerate(need):
        for i in range(n):
            bt[b, i] = perm.pop()
    return bt, sum(need) + 1


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, page, window, keep", [
    (6, 2, 24, 40, 16, 37, 5),      # values wider than keys, a window that ends inside a page
    (4, 4, 16, 16, 8, None, 0),     # no window, one query head per key head
    (8, 1, 32, 16, 16, 7, 19),      # more kept keys than the window is long
    (2, 1, 128, 64, 32, 64, 0),     # no kept keys, a window of two pages
    (6, 2, 32, 48, 16, 37, 70),     # three heads to a group; kept keys beyond the first key tile
    (5, 5, 64, 192, 16, 100, 3),    # wide values
])
def test_sigmoid_attention_alone(dtype, heads, kv_heads, dim, vdim, page, window, keep):
    from deterministic_inference_b200.kernels import ops
    dt, dev = DTYPES[dtype], "cuda"
    g = torch.Generator().manual_seed(heads * 100 + dim)
    n, n2 = 150, 45
    scale = 0.9 / math.sqrt(dim)
    rnd = pg.as_stored_bf16 if dtype == "bfloat16" else (lambda t: t)
    seqs = []
    for length in (n, n2):
        q = rnd(torch.randn(length, heads, dim, generator=g))
        k = rnd(torch.randn(length, kv_heads, dim, generator=g))
        v = rnd(torch.randn(length, kv_heads, vdim, generator=g))
        seqs.append([q, k, v])
    # keys whose weight is 1 against every query of the last tokens, with values that show: just
    # inside and just outside the window of the last position, the last kept key and the first
    # that is not kept, and a far key
    q, k, v = seqs[0]
    last = n - 1
    spikes = [0, n // 2]
    if window:
        spikes += [last - window + 1, last - window]
    if keep:
        spikes += [keep - 1, keep]
    q[last - 3:] = rnd(q[last - 3:] * 0.1 + 4.0 / math.sqrt(dim))
    for j in spikes:
        k[j] = rnd(torch.full_like(k[j], 3.0 / scale / math.sqrt(dim)))
        v[j] = rnd(v[j] + 50.0 * (1 + spikes.index(j)))
    bias = torch.randn(heads * dim + kv_heads * (dim + vdim), generator=g)
    head_bias = torch.randn(heads, generator=g) - 1.0
    bt, pages = paged([n, n2], page, g)
    cache = torch.zeros(pages, kv_heads * page * (dim + vdim), dtype=dt, device=dev)
    want = [pg.sigmoid_window_attention(q.double(), k.double(), v.double(), scale, head_bias.double(),
                                        window or 10 ** 9, keep) for q, k, v in seqs]

    # steps: a long portion of the first sequence alone; then portions of both; then single tokens
    steps = [[(0, 0, 90)], [(0, 90, 2), (1, 0, 31)], [(1, 31, 1), (0, 92, 13)], [(1, 32, 13), (0, 105, 41)]]
    steps += [[(0, p, 1)] for p in range(146, n)]
    got = [torch.zeros(n, heads, vdim, dtype=torch.float64), torch.zeros(n2, heads, vdim, dtype=torch.float64)]
    q_stored = torch.zeros(n, heads, dim, dtype=dt, device=dev)      # the first sequence's q as the kernel left it
    for entries in steps:
        rows, seq_of, pos_of, slots = [], [], [], []
        for b, (s, start, count) in enumerate(entries):
            qq, kk, vv = seqs[s]
            rows.append(torch.cat([qq[start:start + count].reshape(count, -1), kk[start:start + count].reshape(count, -1),
                                   vv[start:start + count].reshape(count, -1)], dim=1))
            for p in range(start, start + count):
                seq_of.append(b)
                pos_of.append(p)
                slots.append(int(bt[s, p // page]) * page + p % page)
        x = torch.cat(rows) - bias                  # the kernel adds the bias back
        meta = SimpleNamespace(block_table=bt[[s for s, _, _ in entries]].contiguous().to(dev),
                               token_seq=torch.tensor(seq_of, dtype=torch.int32, device=dev),
                               positions=torch.tensor(pos_of, dtype=torch.int32, device=dev),
                               seq_lens=torch.tensor([st + c for _, st, c in entries], dtype=torch.int32, device=dev),
                               q_lens=[c for _, _, c in entries], kv_lens=[st + c for _, st, c in entries],
                               scratch={}, num_decode=sum(1 for _, _, c in entries if c == 1))
        qd = ops.qkv_bias_cache(x.to(dev), bias.to(dev), heads, kv_heads, dim, vdim, cache,
                                torch.tensor(slots, dtype=torch.int32, device=dev), page, dt)
        out = ops.sigmoid_attention(qd, cache, meta, scale, head_bias.to(dev), vdim, page, window, keep).cpu()
        at = 0
        for s, start, count in entries:
            got[s][start:start + count] = out[at:at + count].double()
            if s == 0:
                q_stored[start:start + count] = qd[at:at + count]
            at += count
    for s in (0, 1):
        close(got[s], want[s], dtype, f"attention of sequence {s}", f32=3e-5, bf16=8e-3)
    # the same rows in one step: a row's bits do not depend on how the sequence was cut
    meta = SimpleNamespace(block_table=bt[:1].contiguous().to(dev), token_seq=torch.zeros(n, dtype=torch.int32, device=dev),
                           positions=torch.arange(n, dtype=torch.int32, device=dev),
                           seq_lens=torch.tensor([n], dtype=torch.int32, device=dev), q_lens=[n], kv_lens=[n],
                           scratch={}, num_decode=0)
    whole = ops.sigmoid_attention(q_stored, cache, meta, scale, head_bias.to(dev), vdim, page, window, keep)
    # (tokens that came alone ran on the kernel form for decoded tokens, which associates a
    # row's sum over its keys differently: a rounding apart at most)
    cut = 146 if dtype == "bfloat16" else n
    assert torch.equal(whole.cpu().double()[:cut], got[0][:cut]), "a row's bits changed with the cutting"
    if cut < n:
        close(whole[cut:], got[0][cut:], dtype, "tokens alone against the same tokens in a prompt", bf16=4e-3)
    # the spikes did show: a wrong edge would move the last row by about 50
    assert float(want[0][last].abs().max()) > 50


# ---- the delta-rule recurrence -----------------------------------------------------------------------

@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("heads, dim, rank", [(3, 16, 4), (2, 40, 8), (2, 64, 16), (1, 128, 5), (1, 200, 2)])
def test_delta_rule_alone(dtype, heads, dim, rank):
    from deterministic_inference_b200.kernels import ops
    dt, dev = DTYPES[dtype], "cuda"
    g = torch.Generator().manual_seed(heads * 1000 + dim)
    hd = heads * dim
    lens = (70, 23)
    eps, key_eps, decay_scale = 2e-5, 1e-6, math.exp(-0.5)
    w2 = pg.as_stored_bf16(torch.randn(hd, rank, generator=g))
    w0, a_bias = torch.randn(hd, generator=g) - 3.0, torch.randn(hd, generator=g)       # slow decays: w near 1
    norm_w = 1.0 + 0.1 * torch.randn(hd, generator=g)
    projs, want = [], []
    for n in lens:
        proj = torch.randn(n, 5 * hd + rank, generator=g)
        # the first key comes back as the last query: what the state kept of token 0 shows at the end
        proj[-1, :hd] = 3.0 * proj[0, hd:2 * hd]
        projs.append(proj)
        p = proj.double()
        shape = (n, heads, dim)
        r, k, v, gate = (p[:, i * hd:(i + 1) * hd] for i in range(4))
        rate = torch.sigmoid(p[:, 4 * hd:5 * hd] + a_bias.double()).view(shape)
        decay = pg.decay_of(p[:, 5 * hd:], torch.eye(rank, dtype=torch.float64), w2.double(), w0.double()).view(shape)
        o, last = pg.delta_rule(r.reshape(shape), k.reshape(shape), v.reshape(shape), decay, rate)
        want.append((pg.unit_rms(o, eps).reshape(n, hd) * norm_w.double() * torch.sigmoid(gate), last))
    state = torch.zeros(5, heads, dim, dim, dtype=torch.float32, device=dev)
    state[0] = float("nan")                          # nobody's slot: never read into a result
    slot_of = (3, 1)
    cuts = ([1, 30, 2, 1, 1, 35], [2, 1, 1, 17, 2])
    got = [torch.zeros(n, hd, dtype=torch.float64) for n in lens]
    done = [0, 0]
    for i in range(max(len(c) for c in cuts)):
        who = [s for s in (0, 1) if i < len(cuts[s])]
        counts = [cuts[s][i] for s in who]
        x = torch.cat([projs[s][done[s]:done[s] + c] for s, c in zip(who, counts)])
        cu = [0]
        for c in counts:
            cu.append(cu[-1] + c)
        lead = 0                       # the step's leading one-token sequences: the kernel form of decoded tokens
        while lead < len(counts) and counts[lead] == 1:
            lead += 1
        step = SimpleNamespace(cu_q_lens=torch.tensor(cu, dtype=torch.int32, device=dev),
                               state_slots=torch.tensor([slot_of[s] for s in who], dtype=torch.int32, device=dev),
                               num_seqs=len(who), num_decode=lead)
        y = ops.delta_rule(x.to(dev), w2.to(dt).t().contiguous().to(dev), w0.to(dev), a_bias.to(dev), norm_w.to(dev), state, step,
                           heads, dim, rank, decay_scale, key_eps, eps, dt).cpu().double()
        for j, (s, c) in enumerate(zip(who, counts)):
            got[s][done[s]:done[s] + c] = y[cu[j]:cu[j + 1]]
            done[s] += c
    for s in (0, 1):
        close(got[s], want[s][0], dtype, f"output of sequence {s}", f32=1e-4, bf16=8e-3)
        close(state[slot_of[s]], want[s][1], "float32", f"state of sequence {s}", f32=1e-4)
    assert not torch.isnan(state[1:]).any()


# ---- whole models through the trace runner -----------------------------------------------------------

CASES = {
    "g1": ([1, 2, 17, 48, 131, 260], 31),
    "g2": ([5, 33, 64, 200], 32),
    "g3": ([3, 22, 57, 130, 333], 33),
    "g4": ([1, 9, 40, 150], 34),
}


def row_error(got, want):
    d = got.double() - want.double()
    d = d - d.mean()
    return float(d.pow(2).mean().sqrt())


@pytest.fixture(scope="module")
def plain_logits(model_dirs):
    out = {}
    for name, (lens, seed) in CASES.items():
        cfg, w = pg.read_model_dir(model_dirs[name])
        reqs = gu.requests(cfg["vocab"], lens, seed)
        exact = [pg.forward(cfg, w, r) for r in reqs]
        stored = [pg.forward(cfg, w, r, store_bf16=True) for r in reqs]
        out[name] = (cfg, reqs, exact, stored)
    return out


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("name", list(CASES))
def test_replay_all_cuttings(name, dtype, model_dirs, plain_logits, tmp_path):
    cfg, reqs, exact, stored = plain_logits[name]
    trace = ru.Trace()
    ru.mixed(trace, reqs)                             # sizes the pool; four live requests at most
    ru.whole(trace, reqs)
    ru.last_one_by_one(trace, reqs, tail=150)         # decoding over more tokens than any window
    ru.portions(trace, reqs)
    out = ru.run_trace(model_dirs[name], dtype, trace, tmp_path / "out", page_size=gu.CONFIGS[name]["page_size"])
    got = ru.read_rows(out, trace, cfg["vocab"])
    for kind in "mwtp":
        for i, r in enumerate(reqs):
            assert all((f"{kind}{i}", p) in got for p in range(len(r))), (kind, i)
    worst = 0.0
    for (key, pos), row in got.items():
        i = int(key[1:])
        scale = float(exact[i].std())
        err = row_error(row, exact[i][pos])
        if dtype == "float32":
            bound = 1e-4 * scale
        else:
            # what bfloat16 storage alone does to this request's logits, three times over
            yard = max(row_error(a, b) for a, b in zip(stored[i], exact[i]))
            bound = max(3.0 * yard, 2e-2 * scale)
        assert err <= bound, f"{name}/{dtype}: request {key} position {pos}: {err:.4g} exceeds {bound:.4g}"
        worst = max(worst, err / scale)
    print(f"{name}/{dtype}: worst difference {worst:.3e} of the logits' spread")


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_greedy_generation_through_the_entry_point(dtype, model_dirs):
    from deterministic_inference_b200 import Engine, EngineConfig, SamplingParams
    d = model_dirs["g3"]
    cfg, w = pg.read_model_dir(d)
    prompts = gu.requests(cfg["vocab"], [3, 40, 9, 77, 15], 9)
    new = 40
    eng = Engine(EngineConfig(model_path=str(d), dtype=dtype, kv_pool_tokens=384, page_size=8, max_reqs=3,
                              max_seq_len=160, max_prefill_tokens=48))
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=new, ignore_eos=True))
    eng.cache.check_invariants()
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == new
        ids = list(p)
        for t in o.token_ids:
            logits = pg.forward(cfg, w, ids)[-1]
            best = int(torch.argmax(logits))
            if t != best:
                # another token only where rounding can flip the choice; from there on the
                # engine's own continuation is followed
                gap = float(logits[best] - logits[t])
                assert dtype == "bfloat16" and gap < 0.25, f"token {t} instead of {best}, logits {gap:.3g} apart"
            ids.append(t)
