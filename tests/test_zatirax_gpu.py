"""The Zatirax design on the GPU against the plain implementation of ``tests/plain_zatirax.py``:
each new kernel alone (inputs made so that one far key, a key just inside or just outside a window
or a chunk, a page's border, a sink that is left out or a wrong rotation pair would show), then whole
models through ``bin/trace_run`` (whole prompts, the last tokens one by one over more tokens than the
masks are long, portions down to two tokens, mixed batches in a pool so small that pages and slots
are used again), in float32 and bfloat16, and greedy generation through ``Engine.generate``."""

import math
from types import SimpleNamespace

import pytest
import torch

from tests import plain_zatirax as pz
from tests import replay_util as ru
from tests import zatirax_util as zu

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    return {name: zu.write_tiny(name, tmp_path_factory.mktemp(f"zatirax_{name}")) for name in zu.CONFIGS}


def close(got, want, dtype, what, f32=2e-5, bf16=1.2e-2):
    got, want = got.double().cpu(), want.double().cpu()
    scale = float(want.abs().max())
    err = float((got - want).abs().max())
    bound = (f32 if dtype == "float32" else bf16) * max(scale, 1e-6)
    assert err <= bound, f"{what} ({dtype}): abs diff {err:.4g} exceeds {bound:.4g} (scale {scale:.4g})"


def rounder(dtype):
    return pz.as_stored_bf16 if dtype == "bfloat16" else (lambda t: t)


# ---- the float32 stream's kernels -----------------------------------------------------------------

@pytest.mark.parametrize("dtype", list(DTYPES))
def test_stream_kernels_alone(dtype):
    from deterministic_inference_b200.kernels import ops
    dt, dev = DTYPES[dtype], "cuda"
    g = torch.Generator().manual_seed(1)
    rows, width = 37, 136
    ids = torch.randint(0, 50, (rows,), generator=g, dtype=torch.int32)
    table = torch.randn(50, width, generator=g).to(dt)
    x = ops.embedding_scaled(ids.to(dev), table.to(dev), 7.25)
    assert x.dtype == torch.float32
    want = table.double()[ids.long()] * 7.25
    close(x, want, "float32", "scaled embedding")

    # a part's output joins the stream under its post norm, unrounded; then the next norm
    eps = 3e-5
    w_post, w_pre = torch.rand(width, generator=g) + 0.5, torch.rand(width, generator=g) + 0.5
    bias = torch.randn(width, generator=g)
    for kind in ("tensor", "split"):
        if kind == "tensor":
            a = torch.randn(rows, width, generator=g).to(dt)
            term_in, a64 = a.to(dev), a.double()
        else:
            parts = torch.randn(3, rows, width, generator=g)
            term_in, a64 = ops.SplitSum(parts.to(dev), torch.float32), parts.double().sum(0)
        stream = x.clone()
        y = ops.stream_rms_norm(stream, w_pre.to(dev), eps, dt, add=ops.NormedTerm(term_in, w_post.to(dev), eps))
        total = want + pz.rms_norm(a64, w_post.double(), eps)
        close(stream, total, "float32", f"stream after the normed term ({kind})")
        close(y, pz.rms_norm(total, w_pre.double(), eps), dtype, "norm of the stream")
        close(ops.NormedTerm(term_in, w_post.to(dev), eps).tensor(), pz.rms_norm(a64, w_post.double(), eps), "float32",
              "the normed term as a tensor")
        # rows gathered before the norm are the rows of the normed tensor
        idx = torch.tensor([5, 0, 36], dtype=torch.int32, device=dev)
        close(ops.gather_rows(ops.NormedTerm(term_in, w_post.to(dev), eps), idx).tensor(),
              pz.rms_norm(a64, w_post.double(), eps)[[5, 0, 36]], "float32", "gathered normed rows")
    ops.stream_add_(stream, bias=bias.to(dev))
    close(stream, total + bias.double(), "float32", "stream after a pass vector")

    # the limited gate: inputs beyond the limit on both sides
    gate_up = torch.randn(rows, 2 * 72, generator=g) * 2.5
    for limit in (0.8, 7.0):
        want_y = pz.limited_gate(gate_up[:, :72].double(), gate_up[:, 72:].double(), limit)
        close(ops.limited_gate(gate_up.to(dev), limit, 1.702, dt), want_y, dtype, "limited gate")
        halves = torch.stack([gate_up * 0.25, gate_up * 0.75])
        close(ops.limited_gate(ops.SplitSum(halves.to(dev), torch.float32), limit, 1.702, dt), want_y, dtype,
              "limited gate of split sums")


# ---- norm, rotation, cache write ---------------------------------------------------------------------

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
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, rot, scaling, norm", [
    (4, 2, 24, 40, 8, (8.0, 1.0, 4.0, 64), True),
    (3, 3, 32, 32, 32, None, True),           # a full rotation
    (2, 1, 20, 12, 10, (2.0, 0.5, 2.0, 32), False),
    (2, 2, 128, 128, 64, None, True),
    (5, 1, 16, 48, 0, None, True),            # no rotation at all
])
def test_attn_prepare_alone(dtype, heads, kv_heads, dim, vdim, rot, scaling, norm):
    from deterministic_inference_b200.kernels import ops
    dt, dev = DTYPES[dtype], "cuda"
    rnd = rounder(dtype)
    g = torch.Generator().manual_seed(dim)
    t, page, eps = 29, 8, 1e-5
    extra = 11      # columns behind q, k, v that the kernel must leave alone (a gate's)
    width = heads * dim + kv_heads * (dim + vdim) + extra
    proj = torch.randn(t, width, generator=g) * 2
    positions = torch.randint(0, 3000, (t,), generator=g, dtype=torch.int32)
    positions[0], positions[1] = 0, 2999
    qw, kw = torch.rand(dim, generator=g) + 0.5, torch.rand(dim, generator=g) + 0.5
    sc = None if scaling is None else dict(zip(("factor", "low", "high", "original"), scaling))
    freq = pz.rotary_frequencies(rot, 777.0, sc) if rot else None
    bt, pages = paged([t], page, g)
    slots = torch.tensor([int(bt[0, p // page]) * page + p % page for p in range(t)], dtype=torch.int32)
    cache = torch.zeros(pages, kv_heads * page * (dim + vdim), dtype=dt, device=dev)
    q = ops.attn_prepare(proj.to(dev), heads, kv_heads, dim, vdim, qw.to(dev) if norm else None,
                         kw.to(dev) if norm else None, eps, None if freq is None else freq.float().to(dev), rot,
                         positions.to(dev), cache, slots.to(dev), page, dt)
    x = rnd(proj.double())
    nq, nk = heads * dim, kv_heads * dim
    wq = x[:, :nq].view(t, heads, dim)
    wk = x[:, nq:nq + nk].view(t, kv_heads, dim)
    wv = x[:, nq + nk:nq + nk + kv_heads * vdim].view(t, kv_heads, vdim)
    if norm:
        wq, wk = pz.rms_norm(wq, qw.double(), eps), pz.rms_norm(wk, kw.double(), eps)
    if rot:
        # the yardstick rotates by float32 angles, as the design says; a float32 angle of 3,000 is 2e-4 off
        a32 = (positions.float()[:, None] * freq.float()[None, :]).double()
        def turn(v):
            c, s = torch.cos(a32)[:, None, :], torch.sin(a32)[:, None, :]
            h = rot // 2
            return torch.cat([v[..., :h] * c - v[..., h:rot] * s, v[..., h:rot] * c + v[..., :h] * s, v[..., rot:]], -1)
        wq, wk = turn(wq), turn(wk)
    close(q, wq, dtype, "q", f32=1e-5, bf16=5e-3)
    flat = cache.cpu().view(pages, -1)
    got_k = torch.stack([flat[int(s) // page, :kv_heads * page * dim].view(kv_heads, page, dim)[:, int(s) % page]
                         for s in slots])
    got_v = torch.stack([flat[int(s) // page, kv_heads * page * dim:].view(kv_heads, page, vdim)[:, int(s) % page]
                         for s in slots])
    close(got_k, wk, dtype, "cached keys", f32=1e-5, bf16=5e-3)
    close(got_v, wv, dtype, "cached values", f32=1e-6, bf16=4e-3)
    # nothing was written to pages the sequence does not hold
    held = set(int(p) for p in bt[0])
    assert all(float(flat[p].abs().max()) == 0 for p in range(pages) if p not in held)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("heads, dim, rot, vdim, rank", [(3, 16, 8, 24, 32), (1, 32, 16, 40, 24), (5, 12, 6, 18, 21),
                                                         (4, 64, 32, 64, 128)])
def test_latent_rows_and_the_products_per_head(dtype, heads, dim, rot, vdim, rank):
    from deterministic_inference_b200.kernels import ops
    dt, dev = DTYPES[dtype], "cuda"
    rnd = rounder(dtype)
    g = torch.Generator().manual_seed(rank)
    t, page, eps = 23, 8, 1e-5
    width = heads * (dim + rot) + rank + rot
    proj = rnd(torch.randn(t, width, generator=g) * 2)
    positions = torch.randint(0, 2000, (t,), generator=g, dtype=torch.int32)
    cw = torch.rand(rank, generator=g) + 0.5
    freq = pz.rotary_frequencies(rot, 50.0)
    bt, pages = paged([t], page, g)
    slots = torch.tensor([int(bt[0, p // page]) * page + p % page for p in range(t)], dtype=torch.int32)
    cache = torch.zeros(pages, page * (rank + rot), dtype=dt, device=dev)
    pd = proj.to(dt).to(dev)
    q = ops.latent_prepare(pd, heads, dim, rot, rank, cw.to(dev), eps, freq.float().to(dev), positions.to(dev), cache,
                           slots.to(dev), page, dt)
    key_map = rnd(torch.randn(heads, dim, rank, generator=g) * 0.3)
    ops.heads_linear(pd.as_strided((t, heads, dim), (width, dim + rot, 1)), key_map.to(dt).to(dev), q[:, :, :rank])
    x = proj.double()
    a32 = (positions.float()[:, None] * freq.float()[None, :]).double()
    def turn(v):
        c, s = torch.cos(a32), torch.sin(a32)
        while c.dim() < v.dim():
            c, s = c.unsqueeze(1), s.unsqueeze(1)
        h = rot // 2
        return torch.cat([v[..., :h] * c - v[..., h:] * s, v[..., h:] * c + v[..., :h] * s], -1)
    xq = x[:, :heads * (dim + rot)].view(t, heads, dim + rot)
    want_q = torch.cat([torch.einsum("thd,hdc->thc", xq[..., :dim], key_map.double()), turn(xq[..., dim:])], -1)
    close(q, want_q, dtype, "queries in the latent's space", f32=1e-5, bf16=8e-3)
    rows = cache.cpu().view(-1, rank + rot)[slots.long()]
    want_rows = torch.cat([pz.rms_norm(x[:, -(rank + rot):-rot], cw.double(), eps), turn(x[:, -rot:])], -1)
    close(rows, want_rows, dtype, "cached latent rows", f32=1e-5, bf16=5e-3)
    # the value map, many rows (the batched library product takes bfloat16 rows above 64) and few
    value_map = rnd(torch.randn(heads, rank, vdim, generator=g) * 0.3)
    for m in (5, 150):
        lat = rnd(torch.randn(m, heads, rank, generator=g))
        out = torch.empty(m, heads, vdim, dtype=dt, device=dev)
        ops.heads_linear(lat.to(dt).to(dev), value_map.to(dt).to(dev), out)
        close(out, torch.einsum("mhc,hce->mhe", lat.double(), value_map.double()), dtype, f"value map, {m} rows",
              f32=1e-5, bf16=8e-3)


# ---- attention -------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("heads, kv_heads, dk, dv, page, mask, size, sink, gate, in_keys", [
    (6, 2, 24, 40, 16, "chunk", 37, True, True, False),     # values wider than keys, a chunk that ends inside a page
    (4, 4, 16, 16, 8, "causal", None, False, False, False),
    (8, 1, 48, 32, 16, "window", 21, False, False, True),   # one latent row as key and, in part, as value
    (2, 1, 128, 128, 32, "window", 64, True, False, False),
    (4, 2, 64, 64, 16, "chunk", 64, True, True, False),
    (16, 1, 160, 128, 16, "window", 100, False, False, True),
    (5, 5, 20, 12, 8, "chunk", 7, True, True, False),       # a chunk shorter than a page
    (4, 2, 32, 64, 16, "chunk", 50, True, True, False),     # values wider than keys on the tensor cores
    (3, 1, 64, 192, 16, "window", 70, True, False, False),  # three rows a token, wide values
    (24, 1, 96, 64, 8, "causal", None, False, False, True), # no mask: a decoded token's chunks grow with it
])
def test_masked_attention_alone(dtype, heads, kv_heads, dk, dv, page, mask, size, sink, gate, in_keys):
    from deterministic_inference_b200.kernels import ops
    dt, dev = DTYPES[dtype], "cuda"
    rnd = rounder(dtype)
    g = torch.Generator().manual_seed(heads * 100 + dk)
    n, n2 = 150, 45
    scale = 0.9 / math.sqrt(dk)
    seqs = []
    for length in (n, n2):
        q = rnd(torch.randn(length, heads, dk, generator=g))
        k = rnd(torch.randn(length, kv_heads, dk, generator=g))
        v = k[..., :dv].clone() if in_keys else rnd(torch.randn(length, kv_heads, dv, generator=g))
        seqs.append([q, k, v])
    # keys that take nearly all the weight of the last queries, with values that show: just inside and
    # just outside the mask's edge for the last position, the very first key and a far one
    q, k, v = seqs[0]
    last = n - 1
    lo = 0 if mask == "causal" else (last - size + 1 if mask == "window" else last // size * size)
    spikes = [0, n // 2, lo] + ([lo - 1] if lo > 0 else [])
    dims = slice(dv, dk) if in_keys else slice(0, dk)       # (a latent row's value part is left as drawn)
    width = dims.stop - dims.start
    q[last - 3:, :, dims] = rnd(q[last - 3:, :, dims] * 0.1 + 3.0 / math.sqrt(width))
    for j in spikes:
        k[j][:, dims] = rnd(torch.full_like(k[j][:, dims], 4.0 / scale / math.sqrt(width)))
        if in_keys:
            k[j][:, :dv] = rnd(k[j][:, :dv] * 0.05 + 50.0 * (1 + spikes.index(j)))
            v[j] = k[j][:, :dv]
        else:
            v[j] = rnd(v[j] + 50.0 * (1 + spikes.index(j)))
    sinks = torch.randn(heads, generator=g) * 2 + 1.0 if sink else None
    gates = [rnd(torch.randn(length, 7 + heads * dv, generator=g)) for length in (n, n2)] if gate else None
    bt, pages = paged([n, n2], page, g)
    dvs = 0 if in_keys else dv
    cache = torch.zeros(pages, kv_heads * page * (dk + dvs), dtype=dt, device=dev)
    want = []
    for i, (qq, kk, vv) in enumerate(seqs):
        m = len(qq)
        vis = {"causal": pz.window_mask(m, 10 ** 9), "window": pz.window_mask(m, size or 1),
               "chunk": pz.chunk_mask(m, size or 1)}[mask]
        o = pz.softmax_attention(qq.double(), kk.double(), vv.double(), scale, vis, None if sinks is None else sinks.double())
        if gate:
            o = rnd(o) * torch.sigmoid(gates[i][:, 7:].double().view(m, heads, dv))
        want.append(o)

    def write(s, start, count):
        qq, kk, vv = seqs[s]
        flat = cache.view(pages, -1)
        for p in range(start, start + count):
            pg_, off = int(bt[s, p // page]), p % page
            for h in range(kv_heads):
                a = (h * page + off) * dk
                flat[pg_, a:a + dk] = kk[p, h].to(dt).to(dev)
                if not in_keys:
                    a = kv_heads * page * dk + (h * page + off) * dv
                    flat[pg_, a:a + dv] = vv[p, h].to(dt).to(dev)

    steps = [[(0, 0, 90)], [(0, 90, 2), (1, 0, 31)], [(1, 31, 1), (0, 92, 13)], [(1, 32, 13), (0, 105, 41)]]
    steps += [[(0, p, 1)] for p in range(146, n)]
    got = [torch.zeros(n, heads, dv, dtype=torch.float64), torch.zeros(n2, heads, dv, dtype=torch.float64)]

    def run(entries):
        # one-token sequences lead the batch, as in the engine's steps
        entries = sorted(entries, key=lambda e: e[2] != 1)
        rows, grows, seq_of, pos_of = [], [], [], []
        for b, (s, start, count) in enumerate(entries):
            write(s, start, count)
            rows.append(seqs[s][0][start:start + count])
            if gate:
                grows.append(gates[s][start:start + count])
            seq_of += [b] * count
            pos_of += list(range(start, start + count))
        meta = SimpleNamespace(block_table=bt[[s for s, _, _ in entries]].contiguous().to(dev),
                               token_seq=torch.tensor(seq_of, dtype=torch.int32, device=dev),
                               positions=torch.tensor(pos_of, dtype=torch.int32, device=dev),
                               cu_q_lens=torch.tensor([0] + list(torch.tensor([c for _, _, c in entries]).cumsum(0)),
                                                      dtype=torch.int32, device=dev),
                               seq_lens=torch.tensor([st + c for _, st, c in entries], dtype=torch.int32, device=dev),
                               q_lens=[c for _, _, c in entries], kv_lens=[st + c for _, st, c in entries],
                               scratch={}, num_decode=sum(1 for _, _, c in entries if c == 1))
        out = ops.masked_attention(torch.cat(rows).to(dt).to(dev), cache, meta, scale, kv_heads, dv, page, mask, size,
                                   None if sinks is None else sinks.to(dev),
                                   gate=torch.cat(grows).to(dt).to(dev) if gate else None, gate_col=7,
                                   values_in_keys=in_keys).cpu()
        at = 0
        for s, start, count in entries:
            yield s, start, count, out[at:at + count].double()
            at += count

    for entries in steps:
        for s, start, count, rows in run(entries):
            got[s][start:start + count] = rows
    for s in (0, 1):
        close(got[s], want[s], dtype, f"attention of sequence {s}", f32=3e-5, bf16=8e-3)
    # the same rows in one step: up to rounding whatever the cutting (the same bits where one kernel
    # form took both)
    for s, start, count, rows in run([(0, 0, n)]):
        close(rows, got[0], dtype, "whole against cut", f32=1e-6, bf16=4e-3)
    # the spikes did show: a wrong edge would move the last row by about 50
    assert float(want[0][last].abs().max()) > 20


# ---- whole models ------------------------------------------------------------------------------------------

CASES = {       # configuration -> request lengths, seed
    "z1": ([1, 2, 17, 48, 131, 260], 31),
    "z2": ([5, 33, 64, 200], 32),
    "z3": ([3, 22, 57, 130, 333], 33),
    "z4": ([1, 9, 40, 150, 300], 34),
    "z5": ([2, 31, 129, 420], 35),
}


def row_error(got, want):
    d = got.double() - want.double()
    d = d - d.mean()
    return float(d.pow(2).mean().sqrt())


@pytest.fixture(scope="module")
def plain_logits(model_dirs):
    out = {}
    for name, (lens, seed) in CASES.items():
        cfg, w = pz.read_model_dir(model_dirs[name])
        reqs = zu.requests(cfg["vocab"], lens, seed)
        exact = [pz.forward(cfg, w, r) for r in reqs]
        stored = [pz.forward(cfg, w, r, bf16_storage=True) for r in reqs]
        out[name] = (cfg, reqs, exact, stored)
    return out


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("name", list(CASES))
def test_replay_all_cuttings(name, dtype, model_dirs, plain_logits, tmp_path):
    cfg, reqs, exact, stored = plain_logits[name]
    trace = ru.Trace()
    ru.mixed(trace, reqs)                             # sizes the pool; four live requests at most
    ru.whole(trace, reqs)
    ru.last_one_by_one(trace, reqs, tail=150)         # decoding over more tokens than any mask is long
    ru.portions(trace, reqs)
    out = ru.run_trace(model_dirs[name], dtype, trace, tmp_path / "out", page_size=zu.CONFIGS[name]["page_size"])
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


@pytest.mark.parametrize("name, dtype", [("z4", "bfloat16"), ("z3", "float32")])
def test_replay_with_captured_graphs(name, dtype, model_dirs, tmp_path):
    """The step function as generation runs it: pure-decode steps and steps whose shape has come twice
    before are replayed as captured CUDA graphs, whose kernels size their grids and tile lists for the
    bucket's upper bounds and read the real lengths on the device.  Four requests of one length, cut
    alike, so that every shape repeats, and the mixed cutting on top; the replayed run against a launched
    run of the same trace (equal bits: every product is kept on the kernels whose sums do not depend on
    the row count) and against the plain implementation."""
    cfg, w = pz.read_model_dir(model_dirs[name])
    same = zu.requests(cfg["vocab"], [250] * 4, 41)
    other = zu.requests(cfg["vocab"], [33, 150, 77], 42)
    reqs = same + other
    exact = [pz.forward(cfg, w, r) for r in reqs]
    stored = [pz.forward(cfg, w, r, bf16_storage=True) for r in reqs]
    trace = ru.Trace()
    passes = {"": 96, "x": 96, "y": 96, "z": 200}      # every shape of a pass comes again in the next
    for prefix, portion in passes.items():
        ru.lockstep(trace, same, portion=portion, prefix=prefix)
    ru.mixed(trace, reqs)
    outs = {}
    for graphs in (True, False):
        out = ru.run_trace(model_dirs[name], dtype, trace, tmp_path / f"out{int(graphs)}",
                           page_size=zu.CONFIGS[name]["page_size"], cuda_graphs=graphs,
                           extra_env={"DIB200_GEMM_MAX_ROWS": "1000000", "DIB200_HEADS_LINEAR_ROWS": "1000000"})
        outs[graphs] = ru.read_rows(out, trace, cfg["vocab"])
    for key_pos, row in outs[True].items():
        assert torch.equal(row, outs[False][key_pos]), key_pos
    for (key, pos), row in outs[True].items():
        i = int(key.lstrip("xyz")[1:])
        scale = float(exact[i].std())
        err = row_error(row, exact[i][pos])
        yard = max(row_error(a, b) for a, b in zip(stored[i], exact[i]))
        bound = 1e-4 * scale if dtype == "float32" else max(3.0 * yard, 2e-2 * scale)
        assert err <= bound, f"{name}/{dtype}: request {key} position {pos}: {err:.4g} exceeds {bound:.4g}"


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("name", ["z1", "z4"])
def test_greedy_generation_through_the_entry_point(name, dtype, model_dirs):
    from deterministic_inference_b200 import Engine, EngineConfig, SamplingParams
    d = model_dirs[name]
    cfg, w = pz.read_model_dir(d)
    prompts = zu.requests(cfg["vocab"], [3, 40, 9, 77, 15], 9)
    new = 40
    eng = Engine(EngineConfig(model_path=str(d), dtype=dtype, kv_pool_tokens=384, page_size=zu.CONFIGS[name]["page_size"],
                              max_reqs=3, max_seq_len=160, max_prefill_tokens=48))
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=new, ignore_eos=True))
    eng.cache.check_invariants()
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == new
        ids = list(p)
        for t in o.token_ids:
            logits = pz.forward(cfg, w, ids)[-1]
            best = int(torch.argmax(logits))
            if t != best:
                # another token only where rounding can flip the choice; from there on the
                # engine's own continuation is followed
                gap = float(logits[best] - logits[t])
                assert dtype == "bfloat16" and gap < 0.25, f"token {t} instead of {best}, logits {gap:.3g} apart"
            ids.append(t)
