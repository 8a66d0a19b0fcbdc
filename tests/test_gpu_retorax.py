"""Retorax on the GPU against the plain implementation (tests/plain_retorax.py): each new
kernel alone at sizes other than any model's, with inputs made so that a wrong key, a chunk
edge that is one off or a forgotten sink shows; then the engine under every way of cutting
requests into steps, in float32 and bfloat16, with and without replayed launch sequences;
then greedy generation through the Python entry point and its scheduler."""
import random
from types import SimpleNamespace

import pytest
import torch

import plain_retorax as plain
import retorax_tiny as rx
import schedules

pytestmark = pytest.mark.gpu
BOUND = {"float32": 2e-5, "bfloat16": 3e-2}
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def ops():
    from rvllm_b200.kernels import cuda_ops
    return cuda_ops()


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("rx"))
    return {n: rx.write(root, n) for n in rx.CONFIGS}


def dev(t, dtype=None):
    return t.to("cuda", dtype) if dtype is not None else t.to("cuda")


def close(got, want, dtype, scale=None):
    want = want.to(torch.float64)
    got = got.detach().to("cpu", torch.float64)
    s = float(want.abs().max()) if scale is None else scale
    err = float((got - want).abs().max()) / max(s, 1e-30)
    assert err < (1e-5 if dtype == torch.float32 else 2e-2), err


# ---- layer norm ----------------------------------------------------------------------------

@pytest.mark.parametrize("width", [96, 101, 2048, 5000, 9000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layernorm_alone_and_fused(ops, width, dtype):
    g = torch.Generator().manual_seed(width)
    n = 7
    resid = torch.randn(n, width, generator=g) * 3 + 1.5        # a mean that is not zero
    delta = (torch.randn(n, width, generator=g) * 2 - 0.7).to(dtype)
    w, b = 1 + 0.1 * torch.randn(width, generator=g), 0.1 * torch.randn(width, generator=g)
    dw, db = 1 + 0.1 * torch.randn(width, generator=g), 0.1 * torch.randn(width, generator=g)
    d64 = delta.double()
    # a norm after a sub-layer, alone: float32 out
    out = torch.empty(n, width, device="cuda")
    ops.add_layernorm(None, dev(delta), dev(dw), dev(db), 1e-3, out)
    close(out, plain.layer_norm(d64, dw.double(), db.double(), 1e-3), torch.float32)
    # stream + delta, then norm; the stream is updated
    r = dev(resid.clone())
    out = torch.empty(n, width, device="cuda", dtype=dtype)
    ops.add_layernorm(r, dev(delta), dev(w), dev(b), 1e-5, out)
    x = resid.double() + d64
    close(r, x, torch.float32)
    close(out, plain.layer_norm(x, w.double(), b.double(), 1e-5), dtype)
    # stream + LN(delta), then norm: one kernel
    r = dev(resid.clone())
    ops.add_layernorm(r, dev(delta), dev(w), dev(b), 1e-5, out, None, dev(dw), dev(db), 1e-3)
    x = resid.double() + plain.layer_norm(d64, dw.double(), db.double(), 1e-3)
    close(r, x, torch.float32)
    close(out, plain.layer_norm(x, w.double(), b.double(), 1e-5), dtype)
    # selected rows: the stream stays as it is
    r = dev(resid.clone())
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device="cuda")
    out3 = torch.empty(3, width, device="cuda", dtype=dtype)
    ops.add_layernorm(r, dev(delta), dev(w), dev(b), 1e-5, out3, rows, dev(dw), dev(db), 1e-3)
    assert torch.equal(r.cpu(), resid)
    close(out3, plain.layer_norm(x[[5, 0, 5]], w.double(), b.double(), 1e-5), dtype)
    # no delta
    ops.add_layernorm(r, None, dev(w), dev(b), 1e-5, out)
    close(out, plain.layer_norm(resid.double(), w.double(), b.double(), 1e-5), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_xielu(ops, dtype):
    g = torch.Generator().manual_seed(1)
    for shape, pq in (((5, 24), (0.3, -1.2)), ((3, 1001), (-2.0, 0.8)), ((64, 4096), (1.5, 1.5))):
        z = (torch.randn(*shape, generator=g) * 3).to(dtype)
        z[0, :4] = torch.tensor([0.0, -0.0, 1e-3, -1e-3]).to(dtype)
        act = torch.tensor(pq)
        out = torch.empty(shape, device="cuda", dtype=dtype)
        ops.xielu(dev(z), dev(act), out)
        close(out, plain.xielu(z.double(), act[0].double(), act[1].double()), dtype)


# ---- minGRU --------------------------------------------------------------------------------

def _scan_ctx(lengths, slots):
    q_start = [0]
    for n in lengths:
        q_start.append(q_start[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    return SimpleNamespace(q_start=i32(q_start), state_slot=i32(slots), n_reqs=len(lengths),
                           max_q_len=max(lengths + [1]))


@pytest.mark.parametrize("width", [40, 128, 1000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mingru_scan_portions_and_states(ops, width, dtype):
    """Requests of 1, 2, 63, 64, 65 and 700 tokens in one launch, a padding request among
    them, state slots in another order; then a second launch continues from the states."""
    g = torch.Generator().manual_seed(width)
    lengths = [1, 700, 2, 63, 5, 64, 65]
    slots = [3, 0, 6, -1, 2, 5, 1]
    n = sum(lengths)
    bias = torch.randn(2 * width, generator=g) * 0.5
    state = torch.zeros(8, width)
    state[3] = torch.randn(width, generator=g)                # request 0 comes with a past
    t = {"z.b": bias[:width].double(), "x.b": bias[width:].double()}
    dstate = dev(state.clone())
    want_state = state.double().clone()
    for launch in range(2):
        proj = torch.randn(n, 3 * width, generator=g) * 2
        proj[:, :width] -= 2.0                                # small gates: the state reaches far back
        out = torch.full((n, width), float("nan"), device="cuda", dtype=dtype)
        ops.mingru_scan(dev(proj), dev(bias), dstate, _scan_ctx(lengths, slots), out)
        a = 0
        for ln, slot in zip(lengths, slots):
            rows = proj[a:a + ln].double()
            if slot >= 0:
                z = torch.sigmoid(rows[:, :width] + t["z.b"])
                c = plain.mingru_candidate(rows[:, width:2 * width] + t["x.b"])
                gate = rows[:, 2 * width:] * torch.sigmoid(rows[:, 2 * width:])
                s = want_state[slot]
                for i in range(ln):
                    s = (1 - z[i]) * s + z[i] * c[i]
                    close(out[a + i], s * gate[i], dtype, scale=max(1.0, float((s * gate[i]).abs().max())))
                want_state[slot] = s
            a += ln
        close(dstate, want_state, torch.float32)
        assert torch.equal(dstate[7].cpu(), state[7]) and torch.equal(dstate[4].cpu(), state[4])


# ---- rotation + cache write ----------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(5, 2, 24, 40, 6), (3, 3, 64, 16, 64), (4, 1, 10, 10, 0), (2, 0, 16, 8, 4)])
def test_rope_partial_write(ops, dtype, sizes):
    H, G, d, dv, dims = sizes
    g = torch.Generator().manual_seed(H * 100 + d)
    n, extra = 9, 5
    width = H * d + G * (d + dv) + extra
    rows = torch.randn(n, width, generator=g).to(dtype)
    pos = torch.tensor([0, 1, 2, 777, 4095, 5, 100000, 31, 64], dtype=torch.int32)
    slots = torch.tensor([4, 0, -1, 9, 2, 7, 1, 3, 8], dtype=torch.int32)
    base = 300.0
    freq = None
    if dims:
        inv = (base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)).float()
        freq = (dev(inv), dims)
    kc = torch.zeros(12, G, d, device="cuda", dtype=dtype) if G else None
    vc = torch.zeros(12, G, dv, device="cuda", dtype=dtype) if G else None
    drows = dev(rows.clone())
    ops.rope_partial_write(drows, H, G, d, dv, freq, dev(pos), dev(slots), kc, vc)
    r64 = rows.double()
    turn = (lambda x: plain.rotate(x, pos, dims, base)) if dims else (lambda x: x)
    q = turn(r64[:, :H * d].reshape(n, H, d))
    close(drows[:, :H * d], q.reshape(n, H * d), dtype)
    assert torch.equal(drows[:, H * d:].cpu(), rows[:, H * d:])          # nothing else is touched
    if G:
        k = turn(r64[:, H * d:(H + G) * d].reshape(n, G, d))
        v = r64[:, (H + G) * d:(H + G) * d + G * dv].reshape(n, G, dv)
        for t in range(n):
            if slots[t] >= 0:
                close(kc[slots[t]], k[t], dtype, scale=float(k.abs().max()))
                close(vc[slots[t]], v[t], dtype)
        untouched = [s for s in range(12) if s not in slots.tolist()]
        assert float(kc[untouched].abs().max()) == 0 and float(vc[untouched].abs().max()) == 0


# ---- attention with mixed heads ----------------------------------------------------------------

def _paged(k, v, page, dtype, seed):
    """Scatter keys/values of one sequence over shuffled pages; (k pages, v pages, table)."""
    S, G, d = k.shape
    dv = v.shape[2]
    n_pages = -(-S // page)
    order = list(range(n_pages + 3))
    random.Random(seed).shuffle(order)
    kc = torch.zeros(n_pages + 3, page, G, d, dtype=dtype)
    vc = torch.zeros(n_pages + 3, page, G, dv, dtype=dtype)
    for j in range(S):
        kc[order[j // page], j % page] = k[j].to(dtype)
        vc[order[j // page], j % page] = v[j].to(dtype)
    return kc, vc, order[:n_pages]


def _attend(ops, q, k, v, first, page, dtype, scale, talk, sink, chunk, window, gate=None, seed=0):
    """The kernel on queries at positions first.. of one sequence whose keys lie in pages."""
    T, H, d = q.shape
    S, G, dv = k.shape[0], k.shape[1], v.shape[2]
    kc, vc, table = _paged(k, v, page, dtype, seed)
    width = H * d + (H * dv if gate is not None else 0)
    rows = torch.zeros(T, width, dtype=dtype)
    rows[:, :H * d] = q.reshape(T, H * d).to(dtype)
    if gate is not None:
        rows[:, H * d:] = gate.to(dtype)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    if T == 1:
        # a single token, beside a padding request as replayed single-token steps have them
        rows = torch.cat([rows, torch.full_like(rows, float("nan"))])
        ctx = SimpleNamespace(q_start=i32([0, 1, 2]), ctx_lens=i32([first + 1, 0]), token_req=i32([0, 1]),
                              n_tokens=2, n_reqs=2, n_decode=2, max_q_len=1, max_ctx_len=first + 1)
        real = 0
    else:
        # a portion between two empty requests, as padded mixtures have them
        ctx = SimpleNamespace(q_start=i32([0, 0, T, T]), ctx_lens=i32([0, first + T, 0]),
                              token_req=i32([1] * T), n_tokens=T, n_reqs=3, n_decode=0,
                              max_q_len=T + 5, max_ctx_len=first + T)
        real = 1
    tab = torch.full((ctx.n_reqs, len(table) + 2), -1, dtype=torch.int32)
    tab[real, :len(table)] = torch.tensor(table)
    group = SimpleNamespace(block_table=dev(tab), max_blocks=tab.shape[1], page_size=page)
    out = torch.full((rows.shape[0], H * dv), float("nan"), device="cuda", dtype=dtype)
    f32 = lambda x: None if x is None else dev(x.float())
    ops.paged_attention_mixed(dev(rows), H * d if gate is not None else -1, H, G, d, dv, dev(kc),
                              dev(vc), ctx, group, scale, window, chunk, f32(talk), f32(sink), out)
    return out[:T].cpu().reshape(T, H, dv)


def _case(H, G, d, dv, S, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g).to(dtype).double()     # values both sides can hold
    return rnd(S, H, d), rnd(S, G, d), rnd(S, G, dv), rnd(H, H).float().double() * 0.5, rnd(H).float().double()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(6, 2, 32, 16), (4, 4, 16, 48), (3, 1, 24, 8), (8, 4, 64, 64),
                                   (16, 2, 128, 32), (24, 8, 16, 16), (32, 4, 32, 48)])
def test_attention_mixed_against_plain(ops, dtype, sizes):
    H, G, d, dv = sizes
    S = 150
    q, k, v, talk, sink = _case(H, G, d, dv, S, H + d, dtype)
    for chunk, window, page, first in ((None, None, 16, 0), (40, None, 16, 0), (7, None, 4, 0),
                                       (64, None, 8, 100), (None, 33, 16, 60), (50, 20, 32, 90)):
        want = plain.attention_core(q[first:], k, v, 0.2, talk, sink, chunk, window, first)
        got = _attend(ops, q[first:], k, v, first, page, dtype, 0.2, talk, sink, chunk, window)
        close(got, want, dtype)
    # each option off on its own
    for talk_, sink_ in ((None, sink), (talk, None), (None, None)):
        want = plain.attention_core(q, k, v, 0.3, talk_, sink_, 48, None, 0)
        close(_attend(ops, q, k, v, 0, 16, dtype, 0.3, talk_, sink_, 48, None), want, dtype)
    # the gate
    gate = torch.randn(S, H * dv, generator=torch.Generator().manual_seed(1)).to(dtype).double()
    want = plain.attention_core(q, k, v, 0.2, talk, sink, 40, None, 0) * \
        torch.sigmoid(gate).reshape(S, H, dv)
    close(_attend(ops, q, k, v, 0, 16, dtype, 0.2, talk, sink, 40, None, gate=gate), want, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_mixed_one_key_stands_out(ops, dtype):
    """Among 600 keys one is made to win: far back in the prompt, on a page border, the first
    of its chunk, the last before the chunk (which must stay unseen), and the query's own.
    A kernel that loses or wrongly sees that key is off by the size of a value."""
    _one_key_stands_out(ops, dtype, 4, 2, 32, 16)
    _one_key_stands_out(ops, dtype, 8, 2, 32, 16)          # the tensor-core kernel in bfloat16


def _one_key_stands_out(ops, dtype, H, G, d, dv):
    S = 600
    q, k, v, talk, sink = _case(H, G, d, dv, S, 99, dtype)
    talk = torch.eye(H, dtype=torch.float64) + 0.1 * talk
    scale = 0.5
    for chunk, page in ((None, 16), (256, 16), (100, 64), (37, 8)):
        for first in (S - 1, S - 9):                               # decoding alone, a short portion
            p = S - 1
            lo = 0 if chunk is None else p // chunk * chunk
            for key in {lo, lo - 1, lo + 1, p, max(lo, p - 1), 3, 16 * (lo // 16 + 1), 16 * (lo // 16 + 1) - 1}:
                if key < 0 or key > p:
                    continue
                k2, v2 = k.clone(), v.clone()
                k2[key] = 4.0 * q[p].reshape(G, H // G, d)[:, 0]    # aligned with a query of each group
                v2[key] = 50.0
                want = plain.attention_core(q[first:], k2, v2, scale, talk, sink, chunk, None, first)
                got = _attend(ops, q[first:], k2, v2, first, page, dtype, scale, talk, sink, chunk, None,
                              seed=key)
                close(got, want, dtype)
                seen = key >= lo
                assert (float(want[-1].abs().max()) > 20.0) == seen, (chunk, key)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_mixed_sink_takes_weight(ops, dtype):
    """A sink far above every score leaves almost nothing for the values; far below, it changes
    nothing; the first position of a chunk, which sees only itself, shows the sink undiluted."""
    H, G, d, dv, S = 2, 1, 16, 16, 40
    q, k, v, talk, _ = _case(H, G, d, dv, S, 5, dtype)
    for sink in (torch.tensor([30.0, -30.0], dtype=torch.float64), torch.tensor([0.0, 2.0], dtype=torch.float64)):
        want = plain.attention_core(q, k, v, 0.25, None, sink, 10, None, 0)
        got = _attend(ops, q, k, v, 0, 4, dtype, 0.25, None, sink, 10, None)
        close(got, want, dtype, scale=float(v.abs().max()))
    sink = torch.tensor([30.0, -30.0], dtype=torch.float64)
    got = _attend(ops, q, k, v, 0, 4, dtype, 0.25, None, sink, 10, None).double()
    assert float(got[:, 0].abs().max()) < 1e-6 * float(v.abs().max())
    close(got[20, 1], v[20, 0], dtype)                             # position 20 opens a chunk


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


def compare(got, folders, name, reqs, dtype):
    for rid, ids in reqs.items():
        ref = rx.plain_logits(folders[name], name, ids)
        scale = float(ref.abs().max())
        for p in range(len(ids)):
            err = float((got[(rid, p)].double() - ref[p]).abs().max()) / scale
            assert err < BOUND[dtype], (rid, p, err)


def _requests(name, lengths, seed):
    rng = random.Random(seed)
    vocab = rx.config(name)["vocab"]
    return {f"q{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_every_cut_equals_plain(folders, name, dtype):
    """Whole prompts; a prompt then its last tokens one by one (past two chunk borders);
    portions down to two tokens; mixed batches of unequal requests on four slots, with more
    requests than slots, so that pages and slots are used again."""
    model = engine(folders, name, dtype)
    reqs = _requests(name, (130, 1, 2, 67, 200, 33, 64, 65), 3)
    compare(run_schedule(model, schedules.whole(reqs), 16)[0], folders, name, reqs, dtype)
    compare(run_schedule(model, schedules.tail_decode(reqs, 90), 8)[0], folders, name, reqs, dtype)
    compare(run_schedule(model, schedules.portions(reqs), 16)[0], folders, name, reqs, dtype)
    compare(run_schedule(model, schedules.portions(reqs, (64, 2, 100, 3)), 4)[0], folders, name, reqs, dtype)
    for seed in (0, 1):
        compare(run_schedule(model, schedules.mixed(reqs, seed), 16)[0], folders, name, reqs, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replayed_steps_equal_plain(folders, dtype):
    """The same with captured launch sequences: single-token steps and padded mixtures are
    replayed from graphs; requests come and go, so slots and pages are used again."""
    model = engine(folders, "A", dtype)
    reqs = _requests("A", (90, 5, 41, 120, 33, 70, 18), 8)
    for steps, page in ((schedules.tail_decode(reqs, 40), 16), (schedules.mixed(reqs, 2), 8),
                        (schedules.mixed(reqs, 3, max_live=3, decode_tail=20), 16)):
        got, runner = run_schedule(model, steps, page, graphs=True)
        compare(got, folders, "A", reqs, dtype)
        assert runner.graph_steps > 0


def test_a_reused_slot_starts_from_zero(folders):
    """One state slot, two requests one after the other: the second sees nothing of the first."""
    model = engine(folders, "B", "float32")
    reqs = _requests("B", (50, 50), 4)
    got, _ = run_schedule(model, schedules.whole(reqs), 16, slots=1)
    compare(got, folders, "B", reqs, "float32")


def test_long_decoding(folders):
    """400 tokens one by one after a short prompt, across many chunks and pages."""
    model = engine(folders, "B", "float32")
    reqs = _requests("B", (420,), 6)
    got, _ = run_schedule(model, schedules.tail_decode(reqs, 400), 16, graphs=True)
    compare(got, folders, "B", reqs, "float32")


@pytest.mark.parametrize("name", ["A", "D"])
def test_greedy_generation_through_the_entry_point(folders, name):
    """Greedy tokens through `Generator` (scheduler, portions, preemption by a small pool) equal
    the plain implementation's argmax chain."""
    from rvllm_b200 import GenerateOptions, Generator
    rng = random.Random(9)
    vocab = rx.config(name)["vocab"]
    new = 24

    def plain_greedy(ids):
        """The argmax chain, or None when two logits on the way are too close to call."""
        ids = list(ids)
        for _ in range(new):
            row = rx.plain_logits(folders[name], name, ids)[-1]
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
    assert len({t for w in want for t in w}) > 4
    gen = Generator.load(folders[name], dtype="float32")
    for opts in (GenerateOptions(max_tokens=new, block_size=16, stop_tokens=[]),
                 GenerateOptions(max_tokens=new, block_size=8, stop_tokens=[], prefill_chunk=7,
                                 max_batched_tokens=12),
                 GenerateOptions(max_tokens=new, block_size=8, stop_tokens=[], num_blocks=16,
                                 prefill_chunk=20)):
        assert gen.complete_batch(prompts, opts) == want
