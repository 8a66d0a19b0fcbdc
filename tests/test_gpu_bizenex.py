"""Bizenex on the GPU against the plain implementation (tests/plain_bizenex.py): each new
kernel alone at sizes other than any model's, with inputs made so that a lost key, a
forgotten sink or a temperature step that is one off shows; then the engine under every way
of cutting requests into steps, in float32 and bfloat16, with and without replayed launch
sequences; then greedy generation through the Python entry point and its scheduler."""
import math
import random
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import bizenex_tiny as bz
import plain_bizenex as plain
import schedules

pytestmark = pytest.mark.gpu
BOUND = {"float32": 2e-5, "bfloat16": 3e-2}


@pytest.fixture(scope="module")
def ops():
    from rvllm_b200.kernels import cuda_ops
    return cuda_ops()


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("bz"))
    return {n: bz.write(root, n) for n in bz.CONFIGS}


def dev(t, dtype=None):
    return t.to("cuda", dtype) if dtype is not None else t.to("cuda")


def close(got, want, dtype, scale=None):
    want = torch.as_tensor(np.asarray(want), dtype=torch.float64)
    got = got.detach().to("cpu", torch.float64).reshape(want.shape)
    s = float(want.abs().max()) if scale is None else scale
    err = float((got - want).abs().max()) / max(s, 1e-30)
    assert err < (1e-5 if dtype == torch.float32 else 2e-2), err


# ---- attention with a sink and a value size of its own -----------------------------------------

def plain_attend(q, k, v, scale, sinks, first):
    """q [T, H, d] at positions first.., k [S, G, d], v [S, G, dv] (float64 arrays)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for i in range(T):
        p = first + i
        for h in range(H):
            g = h // (H // G)
            s = k[:p + 1, g] @ q[i, h] * scale
            if sinks is None:
                w = np.exp(s - s.max())
                w /= w.sum()
            else:
                w = plain.softmax_with_sink(s, float(sinks[h]))
            out[i, h] = w @ v[:p + 1, g]
    return out


def _paged(k, v, page, dtype, seed, shared):
    S, G, d = k.shape
    dv = v.shape[2]
    n_pages = -(-S // page)
    order = list(range(n_pages + 3))
    random.Random(seed).shuffle(order)
    kc = torch.zeros(n_pages + 3, page, G, d, dtype=dtype)
    vc = kc if shared else torch.zeros(n_pages + 3, page, G, dv, dtype=dtype)
    for j in range(S):
        kc[order[j // page], j % page] = k[j].to(dtype)
        if not shared:
            vc[order[j // page], j % page] = v[j].to(dtype)
    return kc, vc, order[:n_pages]


def _attend(ops, q, k, v, first, page, dtype, scale, sinks, seed=0, shared=False):
    """The kernels on queries at positions first.. of one sequence whose keys lie in shuffled
    pages.  `shared`: the values are the keys (one tensor), as latent attention reads them."""
    T, H, d = q.shape
    G, dv = k.shape[1], v.shape[2]
    kc, vc, table = _paged(k, v, page, dtype, seed, shared)
    rows = q.reshape(T, H * d).to(dtype)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    if T == 1:
        rows = torch.cat([rows, torch.full_like(rows, float("nan"))])
        ctx = SimpleNamespace(q_start=i32([0, 1, 2]), ctx_lens=i32([first + 1, 0]), token_req=i32([0, 1]),
                              n_tokens=2, n_reqs=2, n_decode=2, max_q_len=1, max_ctx_len=first + 1)
        real = 0
    else:
        ctx = SimpleNamespace(q_start=i32([0, 0, T, T]), ctx_lens=i32([0, first + T, 0]),
                              token_req=i32([1] * T), n_tokens=T, n_reqs=3, n_decode=0,
                              max_q_len=T + 5, max_ctx_len=first + T)
        real = 1
    tab = torch.full((ctx.n_reqs, len(table) + 2), -1, dtype=torch.int32)
    tab[real, :len(table)] = torch.tensor(table)
    group = SimpleNamespace(block_table=dev(tab), max_blocks=tab.shape[1], page_size=page)
    out = torch.full((rows.shape[0], H * dv), float("nan"), device="cuda", dtype=dtype)
    dk = dev(kc)
    ops.paged_attention(dev(rows), H, G, d, dk, dk if shared else dev(vc), ctx, group, scale, None,
                        out, sinks=None if sinks is None else dev(sinks.float()), v_head_dim=dv)
    return out[:T].cpu().reshape(T, H, dv)


def _case(H, G, d, dv, S, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g).to(dtype).double()     # values both sides can hold
    return rnd(S, H, d), rnd(S, G, d), rnd(S, G, dv), rnd(H).float().double()


SIZES = [(6, 2, 32, 16), (4, 4, 16, 48), (3, 1, 24, 8), (8, 4, 64, 64), (16, 2, 128, 128),
         (3, 3, 10, 6), (6, 1, 80, 80), (5, 1, 40, 40), (4, 1, 160, 160), (2, 1, 320, 320)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", SIZES)
def test_attention_with_sinks_against_plain(ops, dtype, sizes):
    H, G, d, dv = sizes
    S = 300
    q, k, v, sink = _case(H, G, d, dv, S, H + d, dtype)
    zero = torch.zeros(H, dtype=torch.float64)
    for sinks, page, first in ((sink, 16, 0), (zero, 4, 0), (sink, 8, 200), (zero, 64, 299),
                               (sink, 16, 299), (sink, 16, 298), (None, 16, 100)):
        want = plain_attend(q[first:].numpy(), k.numpy(), v.numpy(), 0.2, sinks, first)
        got = _attend(ops, q[first:], k, v, first, page, dtype, 0.2, sinks)
        close(got, want, dtype)
    if d == dv and G == 1:              # the values are the keys, one tensor
        want = plain_attend(q.numpy(), k.numpy(), k.numpy(), 0.1, sink, 0)
        close(_attend(ops, q, k, k, 0, 16, dtype, 0.1, sink, shared=True), want, dtype)
        want = plain_attend(q[299:].numpy(), k.numpy(), k.numpy(), 0.1, sink, 299)
        close(_attend(ops, q[299:], k, k, 299, 16, dtype, 0.1, sink, shared=True), want, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(8, 4, 64, 64), (5, 1, 112, 112), (4, 4, 32, 32)])
def test_short_portion_after_a_long_context(ops, dtype, sizes):
    """A few tokens at the end of 1,500: the kernels that share a block's keys out over several
    blocks and merge the parts count the sink once."""
    H, G, d, dv = sizes
    S = 1500
    q, k, v, sink = _case(H, G, d, dv, S, 7, dtype)
    sink = sink + 3.0                                              # a sink that matters
    for first in (S - 64, S - 2):
        want = plain_attend(q[first:].numpy(), k.numpy(), v.numpy(), 0.15, sink, first)
        close(_attend(ops, q[first:], k, v, first, 16, dtype, 0.15, sink), want, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(4, 2, 32, 16), (8, 4, 64, 64), (6, 1, 80, 80)])
def test_attention_one_key_stands_out(ops, dtype, sizes):
    """Among 700 keys one is made to win: the first tokens, far back, on both sides of page
    and split borders, the query's own and the one before.  A kernel that loses that key is
    off by the size of a value."""
    H, G, d, dv = sizes
    S = 700
    q, k, v, sink = _case(H, G, d, dv, S, 99, dtype)
    p = S - 1
    for page in (16, 64):
        for first in (S - 1, S - 9):                               # decoding alone, a short portion
            for key in (0, 1, 3, 63, 64, 255, 256, 257, 511, 512, p - 1, p):
                k2, v2 = k.clone(), v.clone()
                k2[key] = 4.0 * q[p].reshape(G, H // G, d)[:, 0]    # aligned with a query of each group
                v2[key] = 50.0
                want = plain_attend(q[first:].numpy(), k2.numpy(), v2.numpy(), 0.5, sink, first)
                got = _attend(ops, q[first:], k2, v2, first, page, dtype, 0.5, sink, seed=key)
                close(got, want, dtype)
                assert float(np.abs(want[-1]).max()) > 20.0, key


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sink_takes_weight(ops, dtype):
    """A sink far above every score leaves almost nothing for the values; far below, it changes
    nothing; position 0, which sees only itself, shows the sink undiluted: with a sink of 0
    and a score of 0 the value comes out halved."""
    H, G, d, dv, S = 2, 1, 16, 16, 40
    q, k, v, _ = _case(H, G, d, dv, S, 5, dtype)
    for sink in (torch.tensor([30.0, -30.0], dtype=torch.float64), torch.tensor([0.0, 2.0], dtype=torch.float64)):
        want = plain_attend(q.numpy(), k.numpy(), v.numpy(), 0.25, sink, 0)
        for first in (0, S - 1):
            got = _attend(ops, q[first:], k, v, first, 4, dtype, 0.25, sink)
            close(got, want[first:], dtype, scale=float(v.abs().max()))
    sink = torch.tensor([30.0, -30.0], dtype=torch.float64)
    got = _attend(ops, q, k, v, 0, 4, dtype, 0.25, sink).double()
    assert float(got[:, 0].abs().max()) < 1e-6 * float(v.abs().max())
    q0 = torch.zeros_like(q)
    got = _attend(ops, q0, k, v, 0, 4, dtype, 0.25, torch.zeros(2, dtype=torch.float64)).double()
    close(got[0, 1], v[0, 0] / 2, dtype)
    close(got[3, 0], v[:4, 0].sum(0) / 5, dtype)                   # four keys and the sink


# ---- unit norm, query temperature, cache write ------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(5, 2, 24, 40), (3, 3, 64, 16), (4, 1, 10, 6), (2, 0, 16, 8),
                                   (6, 3, 64, 64), (3, 1, 8, 8), (5, 5, 256, 256), (7, 0, 32, 32)])
def test_qk_unit_write(ops, dtype, sizes):
    H, G, d, dv = sizes
    g = torch.Generator().manual_seed(H * 100 + d)
    extra = 5 if (H + G) % 2 else 8        # rows that 16-byte accesses do and do not divide
    every = 7
    # positions on both sides of a temperature step: p + 1 = every - 1, every, every + 1, ...
    pos = torch.tensor([0, 1, 5, 6, 7, 12, 13, 14, 700, 69999, 4], dtype=torch.int32)
    n = pos.shape[0]
    slots = torch.tensor([4, 0, -1, 9, 2, 7, 1, 3, 8, 10, 11], dtype=torch.int32)
    rows = (torch.randn(n, H * d + G * (d + dv) + extra, generator=g) * 3).to(dtype)
    for eps, temp in ((1e-3, (0.6, every)), (1e-6, None), (None, (1.5, 1)), (None, None)):
        kc = torch.zeros(12, G, d, device="cuda", dtype=dtype) if G else None
        vc = torch.zeros(12, G, dv, device="cuda", dtype=dtype) if G else None
        drows = dev(rows.clone())
        ops.qk_unit_write(drows, H, G, d, dv, eps, temp, dev(pos), dev(slots), kc, vc)
        r64 = rows.double().numpy()
        unit = (lambda x: plain.rms_unit(x, eps)) if eps is not None else (lambda x: x)
        q = unit(r64[:, :H * d].reshape(n, H, d))
        if temp is not None:
            f = np.array([plain.query_temperature(int(p), *temp) for p in pos])
            q = q * f[:, None, None]
        close(drows[:, :H * d], q.reshape(n, H * d), dtype)
        assert torch.equal(drows[:, H * d:].cpu(), rows[:, H * d:])          # nothing else is touched
        if G:
            k = unit(r64[:, H * d:(H + G) * d].reshape(n, G, d))
            v = r64[:, (H + G) * d:(H + G) * d + G * dv].reshape(n, G, dv)
            for t in range(n):
                if slots[t] >= 0:
                    close(kc[slots[t]], k[t], dtype, scale=float(np.abs(k).max()))
                    close(vc[slots[t]], v[t], dtype)
            untouched = [s for s in range(12) if s not in slots.tolist()]
            assert float(kc[untouched].abs().max()) == 0 and float(vc[untouched].abs().max()) == 0


def test_query_temperature_steps():
    assert plain.query_temperature(0, 0.5, 4) == 1.0 and plain.query_temperature(2, 0.5, 4) == 1.0
    assert plain.query_temperature(3, 0.5, 4) == 1.0 + 0.5 * math.log(2)
    assert plain.query_temperature(7, 0.5, 4) == 1.0 + 0.5 * math.log(3)


# ---- latent rows, the products per head, the gate -----------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank", [14, 32, 88, 520])
def test_latent_norm_write(ops, dtype, rank):
    g = torch.Generator().manual_seed(rank)
    n, offset = 9, 11
    rows = (torch.randn(n, offset + rank + 3, generator=g) * 2).to(dtype)
    w = 1 + 0.2 * torch.randn(rank, generator=g)
    slots = torch.tensor([4, 0, -1, 9, 2, 7, 1, 3, 8], dtype=torch.int32)
    cache = torch.zeros(3, 4, 1, rank, device="cuda", dtype=dtype)
    ops.latent_norm_write(dev(rows), offset, rank, dev(w), 1e-4, dev(slots), cache)
    want = plain.rms_unit(rows[:, offset:offset + rank].double().numpy(), 1e-4) * w.double().numpy()
    flat = cache.view(12, rank)
    for t in range(n):
        if slots[t] >= 0:
            close(flat[slots[t]], want[t], dtype, scale=float(np.abs(want).max()))
    assert float(flat[[5, 6, 10, 11]].abs().max()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_heads_product_and_gate(ops, dtype):
    """Few tokens and many, sizes that nothing divides, with the gate in the same call and as a
    kernel of its own."""
    g = torch.Generator().manual_seed(3)
    for n, H, a, b, offset in ((7, 3, 10, 6, 4), (130, 6, 32, 96, 0), (1, 8, 112, 72, 16), (64, 5, 24, 200, 8),
                               (65, 2, 128, 64, 0), (9, 4, 512, 40, 0)):
        rows = torch.randn(n, offset + H * a + 9, generator=g).to(dtype)
        w = (torch.randn(H, a, b, generator=g) * 0.3).to(dtype)
        out = ops.new_rows(n, H * b, dtype, "cuda")
        ops.heads_product(dev(rows), offset, H, a, dev(w), out)
        x = rows[:, offset:offset + H * a].double().reshape(n, H, a)
        want = torch.einsum("nha,hab->nhb", x, w.double()).reshape(n, H * b)
        close(out, want, dtype)
        gate_rows = (torch.randn(n, 5 + H * b, generator=g) * 3).to(dtype)
        gated = want * torch.sigmoid(gate_rows[:, 5:].double())
        ops.heads_product(dev(rows), offset, H, a, dev(w), out, gate_rows=dev(gate_rows), gate_off=5)
        close(out, gated, dtype)
        y = dev(want.to(dtype))
        ops.sigmoid_gate(y, dev(gate_rows), 5)
        close(y, want.to(dtype).double() * torch.sigmoid(gate_rows[:, 5:].double()), dtype)


# ---- mixture of experts ---------------------------------------------------------------------------

@pytest.mark.parametrize("shape", [(8, 3, 2, 1), (8, 2, 1, 1), (6, 2, 3, 2), (9, 3, 3, 1), (64, 6, 8, 3),
                                   (4, 1, 1, 1), (5, 5, 1, 1), (12, 3, 12, 4), (256, 8, 8, 4), (40, 33, 1, 1)])
def test_moe_select(ops, shape):
    E, top, groups, keep = shape
    g = torch.Generator().manual_seed(E * 10 + top)
    n = 97
    logits = torch.randn(n, E, generator=g) * 2
    logits[0] = 0.0                                   # all equal: the lower index first
    logits[1, : E // 2] = 40.0                        # sigmoid gives exactly 1 for several
    logits[2] = -torch.arange(E, dtype=torch.float32)
    logits[3] = torch.arange(E, dtype=torch.float32) / E
    ids = torch.empty(n, top, dtype=torch.int32, device="cuda")
    wts = torch.empty(n, top, dtype=torch.float32, device="cuda")
    ops.moe_select(dev(logits), groups, keep, 2, 1e-20, ids, wts)
    ids, wts = ids.cpu(), wts.cpu()
    for t in range(n):
        s = plain.sigmoid(logits[t].numpy().astype(np.float32)).astype(np.float32)
        chosen, weights = plain.route(s.astype(np.float64), top, groups, keep)
        assert ids[t].tolist() == chosen.tolist(), (t, ids[t].tolist(), chosen.tolist())
        assert np.allclose(wts[t].numpy(), weights, rtol=1e-5, atol=1e-7)
        assert abs(float(wts[t].sum()) - 1.0) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(50, 5, 2, 5, 3), (96, 8, 3, 2, 1), (1024, 64, 6, 8, 3), (333, 9, 3, 1, 1),
                                   (256, 128, 8, 8, 4), (4000, 16, 4, 4, 2)])
def test_moe_route(ops, dtype, shape):
    """The router's product and the choice in one kernel against the plain route on float64
    logits of the same (rounded) rows; 1, 7, 8, 9 and 100 tokens."""
    W, E, top, groups, keep = shape
    g = torch.Generator().manual_seed(W + E)
    router = torch.randn(E, W, generator=g) * W ** -0.5
    for n in (1, 7, 8, 9, 100):
        x = (torch.randn(n, W, generator=g) * 2).to(dtype)
        ids = torch.empty(n, top, dtype=torch.int32, device="cuda")
        wts = torch.empty(n, top, dtype=torch.float32, device="cuda")
        ops.moe_route(dev(x), dev(router), groups, keep, 2, 1e-20, ids, wts)
        ids, wts = ids.cpu(), wts.cpu()
        z = x.double().numpy() @ router.double().numpy().T
        for t in range(n):
            chosen, weights = plain.route(plain.sigmoid(z[t]), top, groups, keep)
            assert ids[t].tolist() == chosen.tolist(), (n, t)
            assert np.allclose(wts[t].numpy(), weights, rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(50, 34, 5, 2), (96, 64, 6, 2), (336, 104, 10, 5), (128, 256, 4, 1),
                                   (64, 48, 16, 16), (512, 264, 4, 2)])
@pytest.mark.parametrize("n", [1, 3, 37, 300, 1500])
def test_moe_experts(ops, dtype, shape, n):
    W, F, E, top = shape
    g = torch.Generator().manual_seed(W + n)
    x = torch.randn(n, W, generator=g).to(dtype)
    gate_up = (torch.randn(E, 2 * F, W, generator=g) * W ** -0.5).to(dtype)
    down = (torch.randn(E, W, F, generator=g) * F ** -0.5).to(dtype)
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(n)]).to(torch.int32)
    if n > 2:
        ids[2] = torch.arange(top)                    # and some tokens all on the same experts
        ids[1] = torch.arange(top)
    wts = torch.rand(n, top, generator=g)
    out = torch.full((n, W), float("nan"), device="cuda", dtype=dtype)
    ops.moe_experts(dev(x), dev(ids), dev(wts), dev(gate_up), dev(down), out)
    want = np.zeros((n, W))
    gu, dn, xs = gate_up.double().numpy(), down.double().numpy(), x.double().numpy()
    for t in range(n):
        for k in range(top):
            e = int(ids[t, k])
            want[t] += float(wts[t, k]) * plain.expert(xs[t], gu[e, 0::2], gu[e, 1::2], dn[e])
    close(out, want, dtype)


def test_softcap(ops):
    x = torch.randn(5, 1001) * 40
    y = dev(x.clone())
    ops.softcap(y, 12.0)
    close(y, 12.0 * torch.tanh(x.double() / 12.0), torch.float32)


# ---- the engine ---------------------------------------------------------------------------

_models = {}


def engine(folders, name, dtype):
    from rvllm_b200.engine import load_model
    if (name, dtype) not in _models:
        _models[(name, dtype)] = load_model(folders[name], dtype, "cuda")[0]
    return _models[(name, dtype)]


def run_schedule(model, steps, page, slots=4, graphs=False):
    from rvllm_b200.engine import ModelRunner, make_cache
    cache = make_cache(model, page, schedules.tokens_held(steps, 64) // page, slots)
    runner = ModelRunner(model, cache, model.ops, use_graphs=graphs)
    got = schedules.replay(runner, steps)
    model.ops.check_status()
    assert not cache.requests and all(g.pool.in_use == 0 for g in cache.groups)
    return got, runner


_plain = {}


def compare(got, folders, name, reqs, dtype):
    """float32: every position within the bound.  bfloat16: a router score that is a close call
    may fall the other way after rounding and change a token's experts, which is no fault; so a
    few positions in a hundred may lie outside the bound."""
    over, total = [], 0
    for rid, ids in reqs.items():
        key = (name, tuple(ids))
        if key not in _plain:
            _plain[key] = bz.plain_logits(folders[name], name, ids)
        ref = _plain[key]
        scale = float(ref.abs().max())
        for p in range(len(ids)):
            err = float((got[(rid, p)].double() - ref[p]).abs().max()) / scale
            total += 1
            if not err < BOUND[dtype]:
                over.append((rid, p, err))
    assert len(over) <= (0 if dtype == "float32" else 0.04 * total), (len(over), total, over[:5])


def _requests(name, lengths, seed):
    rng = random.Random(seed)
    vocab = bz.config(name)["vocab"]
    return {f"q{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_every_cut_equals_plain(folders, name, dtype):
    """Whole prompts; a prompt then its last tokens one by one (past several temperature
    steps); portions down to two tokens; mixed batches of unequal requests on four slots,
    with more requests than slots, so that pages and slots are used again."""
    model = engine(folders, name, dtype)
    reqs = _requests(name, (130, 1, 2, 67, 200, 33, 64, 65), 3)
    compare(run_schedule(model, schedules.whole(reqs), 16)[0], folders, name, reqs, dtype)
    compare(run_schedule(model, schedules.tail_decode(reqs, 90), 8)[0], folders, name, reqs, dtype)
    compare(run_schedule(model, schedules.portions(reqs), 16)[0], folders, name, reqs, dtype)
    compare(run_schedule(model, schedules.portions(reqs, (64, 2, 100, 3)), 4)[0], folders, name, reqs, dtype)
    for seed in (0, 1):
        compare(run_schedule(model, schedules.mixed(reqs, seed), 16)[0], folders, name, reqs, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D"])
def test_replayed_steps_equal_plain(folders, name, dtype):
    """The same with captured launch sequences: single-token steps and padded mixtures are
    replayed from graphs; requests come and go, so slots and pages are used again."""
    model = engine(folders, name, dtype)
    reqs = _requests(name, (90, 5, 41, 120, 33, 70, 18), 8)
    for steps, page in ((schedules.tail_decode(reqs, 40), 16), (schedules.mixed(reqs, 2), 8),
                        (schedules.mixed(reqs, 3, max_live=3, decode_tail=20), 16)):
        got, runner = run_schedule(model, steps, page, graphs=True)
        compare(got, folders, name, reqs, dtype)
        assert runner.graph_steps > 0


def test_long_decoding(folders):
    """400 tokens one by one after a short prompt, across many pages, splits and temperature
    steps."""
    model = engine(folders, "B", "float32")
    reqs = _requests("B", (420,), 6)
    got, _ = run_schedule(model, schedules.tail_decode(reqs, 400), 16, graphs=True)
    compare(got, folders, "B", reqs, "float32")


def test_a_batch_does_not_change_a_request(folders):
    """A request beside others gives the bits it gives alone, in the same cut."""
    model = engine(folders, "A", "float32")
    reqs = _requests("A", (70, 31, 5), 12)
    alone, _ = run_schedule(model, schedules.whole({"q0": reqs["q0"]}), 16)
    steps = [{"step": 0, "entries": [{"id": r, "tokens": ids, "want": list(range(len(ids)))}
                                      for r, ids in reqs.items()], "end": list(reqs)}]
    together, _ = run_schedule(model, steps, 16)
    for p in range(70):
        assert float((alone[("q0", p)] - together[("q0", p)]).abs().max()) < 1e-5


@pytest.mark.parametrize("name", ["A", "D"])
def test_greedy_generation_through_the_entry_point(folders, name):
    """Greedy tokens through `Generator` (scheduler, portions, preemption by a small pool) equal
    the plain implementation's argmax chain."""
    from rvllm_b200 import GenerateOptions, Generator
    rng = random.Random(9)
    vocab = bz.config(name)["vocab"]
    new = 24
    tensors = bz.read_tensors(folders[name])

    def plain_greedy(ids):
        """The argmax chain, or None when two logits on the way are too close to call."""
        ids = list(ids)
        for _ in range(new):
            row = bz.plain_logits(folders[name], name, ids, tensors=tensors)[-1]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) < 1e-3 * float(row.abs().max()):
                return None
            ids.append(int(row.argmax()))
        return ids[-new:]

    prompts, want = [], []
    for n in (5, 37, 70):
        for attempt in range(20):
            p = [rng.randrange(vocab) for _ in range(n)]
            w = plain_greedy(p)
            if w is not None:
                prompts.append(p)
                want.append(w)
                break
    assert len(prompts) == 3
    gen = Generator.load(folders[name], dtype="float32")
    for opts in (GenerateOptions(max_tokens=new, block_size=16, stop_tokens=[]),
                 GenerateOptions(max_tokens=new, block_size=8, stop_tokens=[], prefill_chunk=7,
                                 max_batched_tokens=12),
                 GenerateOptions(max_tokens=new, block_size=8, stop_tokens=[], num_blocks=16,
                                 prefill_chunk=20)):
        assert gen.complete_batch(prompts, opts) == want


def test_command_line_and_trace_replay(folders, tmp_path):
    """The design through the programs a user starts: `rvllm random-model` writes a folder from a
    config.json, `rvllm cli` completes prompts of token ids, `bin/trace_run` replays steps from
    standard input and writes logits that equal the plain implementation's."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(bz.config("B")))
    folder = str(tmp_path / "model")
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "rvllm"), "random-model",
                        "--config", str(cfg_path), "--seed", "5", "--out", folder],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    tensors = bz.read_tensors(folder)
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "rvllm"), "cli", "--model", folder,
                        "--dtype", "float32", "--token-ids", "--prompt", " ".join(map(str, prompt)),
                        "--max-tokens", "5", "--block-size", "8"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    got = [int(t) for t in r.stdout.strip().splitlines()[0].split()]
    ids = list(prompt)
    for tok in got:                           # each token is the plain argmax at its place
        row = bz.plain_logits(folder, "B", ids, tensors=tensors)[-1]
        assert float(row.max() - row[tok]) < 1e-3 * float(row.abs().max())
        ids.append(tok)
    assert len(got) == 5
    reqs = _requests("B", (70, 33, 90, 41, 12), 4)
    steps = schedules.mixed(reqs, seed=2)
    vocab = bz.config("B")["vocab"]
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        cmd = [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder,
               "--dtype", dtype, "--out", str(out), "--max-tokens",
               str(schedules.tokens_held(steps, 64))]
        r = subprocess.run(cmd, input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=900)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [l for l in r.stdout.split("\n") if l.startswith("done")] == \
            [f"done {s['step']}" for s in steps]
        got, pos = {}, {k: 0 for k in reqs}
        for s in steps:
            arr = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab)
            k = 0
            for e in s["entries"]:
                for w in e["want"]:
                    got[(e["id"], pos[e["id"]] + w)] = torch.from_numpy(arr[k].copy())
                    k += 1
                pos[e["id"]] += len(e["tokens"])
            assert k == arr.shape[0]
        over, total = 0, 0
        for rid, ids in reqs.items():
            ref = bz.plain_logits(folder, "B", ids, tensors=tensors)
            for p in range(len(ids)):
                err = float((got[(rid, p)].double() - ref[p]).abs().max() / ref.abs().max())
                total += 1
                over += not err < BOUND[dtype]
        assert over <= (0 if dtype == "float32" else 0.04 * total), (dtype, over, total)
