"""The Roritar design in the engine against the plain implementation (``plain_roritar``): every mechanism alone, whole
prompts against token-by-token decoding, portions down to two tokens, batches of unequal requests, slots and pages
that are used again, keys far away and at the edges of windows, blocks and pages, long decoding, sizes that are 1 or
equal, generation through the library's own loop, and trace replay (needs a B200)."""
import numpy as np
import pytest
import torch

import plain_roritar as pr
import roritar_helpers as rh
from helpers import FP32_TOL, run_trace
from questwend_b200.cache import CacheManager
from questwend_b200.engine.engine import Engine, StepEntry, build_step_context
from questwend_b200.kernels import ops
from questwend_b200.parts import PartSpec, Runtime, build_part

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]
BF16_RMS_TOL = 0.03         # bfloat16 engine against the plain implementation that rounds the products' operands and the
                            # cached keys, values and block means: root mean square of the difference over the reference's


def close(got, ref, dtype, tol=FP32_TOL):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    if dtype == torch.float32:
        return np.abs(got - ref).max() <= tol * np.abs(ref).max()
    return np.sqrt(np.mean((got - ref) ** 2)) <= BF16_RMS_TOL * np.sqrt(np.mean(ref ** 2))


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype).to(DEV)


# ----------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("D", [16, 64, 100, 1030, 2560, 4100])
@pytest.mark.parametrize("out_dtype", DTYPES)
def test_layer_norm_in_its_three_forms(D, out_dtype):
    rng = np.random.default_rng(D)
    T, eps = 7, 1e-5
    x = rng.standard_normal((T, D)) * 3 + 5.0                 # a mean far from zero: E[v^2] - E[v]^2 would lose digits
    y, w, wy = rng.standard_normal((T, D)) + 2.0, 1 + 0.3 * rng.standard_normal(D), 1 + 0.3 * rng.standard_normal(D)
    x32, y32, w32, wy32 = (np.float32(a).astype(np.float64) for a in (x, y, w, wy))
    tol = 1e-5 if out_dtype == torch.float32 else 2.0 ** -7
    plain = ops.layernorm(dev(x32), dev(w32), eps, out_dtype).double().cpu().numpy()
    assert np.abs(plain - pr.layer_norm(x32, w32, eps)).max() <= tol * 4
    summed = x32 + pr.layer_norm(y32, wy32, eps)
    h = dev(x32)
    assert ops.layernorm(h, None, eps, add=dev(y32), add_weight=dev(wy32), write_sum=True) is None
    assert np.abs(h.double().cpu().numpy() - summed).max() <= 1e-5 * np.abs(summed).max()
    h = dev(x32)
    both = ops.layernorm(h, dev(w32), eps, out_dtype, add=dev(y32), add_weight=dev(wy32), write_sum=True).double().cpu().numpy()
    assert np.abs(h.double().cpu().numpy() - summed).max() <= 1e-5 * np.abs(summed).max()
    assert np.abs(both - pr.layer_norm(summed, w32, eps)).max() <= tol * 4
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    h = dev(x32)
    some = ops.layernorm(h, dev(w32), eps, out_dtype, add=dev(y32), add_weight=dev(wy32), rows=rows).double().cpu().numpy()
    assert np.abs(some - pr.layer_norm(summed, w32, eps)[[5, 0, 5]]).max() <= tol * 4
    assert torch.equal(h, dev(x32))                           # without write_sum the stream stays as it was


def test_xielu_and_capped_logits():
    rng = np.random.default_rng(3)
    z = np.float32(rng.standard_normal((5, 37)) * 3).astype(np.float64)
    for p, q in ((0.3, -0.2), (-2.0, 1.5), (25.0, -30.0)):
        got = ops.bias_act(dev(z), None, "xielu", torch.float32, params=dev(np.array([p, q]))).double().cpu().numpy()
        assert np.abs(got - pr.xielu(z, p, q)).max() <= 1e-5 * np.abs(pr.xielu(z, p, q)).max()
    with pytest.raises(ops.KernelError):
        ops.bias_act(dev(z), None, "xielu", torch.float32)
    got = ops.scale_softcap(dev(z), 2.5, 4.0).double().cpu().numpy()
    assert np.abs(got - 4.0 * np.tanh(z * 2.5 / 4.0)).max() <= 1e-5
    assert np.abs(ops.scale_softcap(dev(z), 0.5, 0.0).double().cpu().numpy() - 0.5 * z).max() <= 1e-6


@pytest.mark.parametrize("M, N, K", [(600, 264, 2048), (512, 1024, 2048), (1000, 72, 2056), (1, 264, 2048), (8, 100, 64), (16, 384, 256)])
def test_xielu_in_the_tensor_core_products_epilogue(M, N, K):
    """bfloat16 rows: the up projection's activation runs in the epilogue of the tcgen05 product (many rows) or of the ring
    product (up to 16); the same numbers as the library product followed by the activation kernel, up to the order of the
    32-bit sums."""
    from questwend_b200.parts.linear import linear_act
    rng = np.random.default_rng(M + N)
    x = dev(rng.standard_normal((M, K)), torch.bfloat16)
    w = dev(rng.standard_normal((N, K)) / np.sqrt(K) * 2, torch.bfloat16)
    params = dev(np.array([0.4, -0.3]))
    before = ops.LAUNCHES[0]
    got = linear_act(x, w, None, "xielu", torch.bfloat16, params=params)
    assert ops.LAUNCHES[0] - before == 1                      # one kernel: the product with its epilogue
    ops.gemm_tc_check(DEV)
    ref = pr.xielu(x.double().cpu().numpy() @ w.double().cpu().numpy().T, 0.4, -0.3)
    assert np.abs(got.double().cpu().numpy() - ref).max() <= 2.0 ** -7 * np.abs(ref).max()
    two = ops.bias_act(torch.mm(x, w.t(), out_dtype=torch.float32), None, "xielu", torch.bfloat16, params=params)
    assert np.abs((got.double() - two.double()).cpu().numpy()).max() <= 2.0 ** -7 * np.abs(ref).max()


@pytest.mark.parametrize("blocks, n", [(1, 16), (3, 16), (4, 80), (2, 136), (16, 1), (5, 7), (1, 1040)])
@pytest.mark.parametrize("wdtype", DTYPES)
def test_block_gates(blocks, n, wdtype):
    rng = np.random.default_rng(blocks * 100 + n)
    for T in (1, 16, 17, 70, 130):
        u = np.float32(rng.standard_normal((T, blocks * n))).astype(np.float64)
        wa, wi = (pr.round_bf16(rng.standard_normal((blocks, n, n))) for _ in range(2))
        ba, bi = (pr.round_bf16(rng.standard_normal((blocks, n))) for _ in range(2))
        r, i = ops.block_gates(dev(u), dev(wa, wdtype), dev(ba), dev(wi, wdtype), dev(bi))
        assert np.abs(r.double().cpu().numpy() - pr.block_gate(u, wa, ba)).max() <= 2e-5
        assert np.abs(i.double().cpu().numpy() - pr.block_gate(u, wi, bi)).max() <= 2e-5


# ----------------------------------------------------------------------------- mixers alone
def make_mixer(entry, dtype, w, width, eps=1e-5):
    import questwend_b200  # noqa: F401
    from questwend_b200.config.registry import config_from_dict
    from questwend_b200.models.roritar import _mixer
    cfg = config_from_dict(rh.config([(entry, None)], width=width))
    spec, pos_specs = _mixer(entry["type"], cfg.layers[0]["mixer"], width, eps)
    rt = Runtime(DEV, dtype)
    position = None if pos_specs is None else tuple(None if p is None else build_part("position", p, rt) for p in pos_specs)
    part = build_part("mixer", PartSpec(spec.kind, spec.params, prefix="l0.mix."), rt, position=position)
    held = {}
    for t in part.tensors():
        held[t.name] = torch.from_numpy(w[t.name]).to(dtype if t.role == "matrix" else torch.float32).to(DEV)
    part.bind(held)
    return part


def plain_mixer(entry, x, w, dtype, eps=1e-5):
    r16 = dtype == torch.bfloat16
    if entry["type"] == "rglru":
        return pr.rglru_mixer(x, w, "l0.mix.", entry["mixer"], r16)
    return pr.pooled_window_attention(x, w, "l0.mix.", entry["mixer"], eps, r16, entry["mixer"]["rot"].get("layout", "halves"))


def run_mixer(part, dtype, xs, plan):
    """``plan``: a list of steps, each a list of token counts per sequence (0: the sequence sits the step out).  Returns
    each sequence's outputs in order."""
    n_tokens = sum(len(x) for x in xs)
    cache = CacheManager([(part.kv_spec(), part.state_spec(), None)], n_tokens + 64 * len(xs) + 512, 8, max(len(x) for x in xs) + 64, dtype, DEV)
    unit = cache.unit_cache(0)
    slots = cache.open(len(xs))
    at = [0] * len(xs)
    got = [[] for _ in xs]
    for counts in plan:
        who = [i for i, c in enumerate(counts) if c]
        chunks = [xs[i][at[i]:at[i] + counts[i]] for i in who]
        ctx = build_step_context(cache, [StepEntry(slots[i], [0] * counts[i], []) for i in who], 10 ** 6, DEV)[0]
        out = part.forward(dev(np.concatenate(chunks), dtype), ctx, unit).double().cpu().numpy()
        off = 0
        for i, c in zip(who, chunks):
            got[i].append(out[off:off + len(c)])
            off += len(c)
            cache.advance(slots[i], len(c))
            at[i] += len(c)
    assert all(a == len(x) for a, x in zip(at, xs))
    return [np.concatenate(g) for g in got]


def prompt_then_tokens(lens, extra):
    return [list(lens)] + [[1] * len(lens)] * extra


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("entry", [rh.rglru(), rh.rglru(width=80, blocks=1, conv=1), rh.rglru(width=272, blocks=2, conv=8),
                                   rh.rglru(width=40, blocks=40, conv=2), rh.rglru(width=35, blocks=5, conv=3),
                                   rh.rglru(width=24, blocks=2, conv=12)])
def test_rglru_alone(entry, dtype):
    """Prompts in one step (one long enough for the chunked scan, one of a single token), then tokens one by one."""
    width = 48
    w = rh.draw_weights(rh.config([(entry, None)], width=width), 1)
    rng = np.random.default_rng(2)
    lens, extra = [300, 70, 1], 6
    xs = [pr.round_bf16(rng.standard_normal((n + extra, width))) for n in lens]
    got = run_mixer(make_mixer(entry, dtype, w, width), dtype, xs, prompt_then_tokens(lens, extra))
    for g, x in zip(got, xs):
        assert close(g, plain_mixer(entry, x, w, dtype), dtype)


def test_rglru_long_memory_in_chunks_in_order_and_token_by_token():
    """Decays close to 1 (the state remembers hundreds of tokens): the chunked scan, the scan in order (portions below the
    chunked form's bound) and single tokens agree with the plain recurrence."""
    entry, width, dtype = rh.rglru(width=64, blocks=2, conv=4), 32, torch.float32
    w = rh.draw_weights(rh.config([(entry, None)], width=width), 4, slow_decay=True)
    x = pr.round_bf16(np.random.default_rng(5).standard_normal((700, width)))
    ref = plain_mixer(entry, x, w, dtype)
    part = make_mixer(entry, dtype, w, width)
    for plan in ([[700]], [[257], [255], [188]], [[100]] * 7, [[2]] * 350, [[640]] + [[1]] * 60):
        assert close(run_mixer(part, dtype, [x], plan)[0], ref, dtype), plan[0]


ATTENTIONS = [rh.attention(), rh.attention(heads=3, kv_heads=3, dim=16, vdim=40, size=70, pool=12, dims=16, base=500.0),
              rh.attention(heads=6, kv_heads=1, dim=8, vdim=8, size=7, pool=7, dims=2, scale=0.6),
              rh.attention(heads=2, kv_heads=2, dim=136, vdim=24, size=64, pool=64, dims=8),
              rh.attention(heads=2, kv_heads=1, dim=16, vdim=264 - 8, size=3, pool=1, dims=0),
              rh.attention(heads=9, kv_heads=1, dim=8, vdim=16, size=130, pool=3, dims=8, layout="interleaved"),
              rh.attention(heads=2, kv_heads=2, dim=32, vdim=32, size=0, pool=0, dims=32),
              rh.attention(heads=2, kv_heads=1, dim=16, vdim=8, size=5, pool=0, dims=4),
              rh.attention(heads=1, kv_heads=1, dim=8, vdim=8, size=1, pool=1, dims=8)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("entry", ATTENTIONS)
def test_attention_alone(entry, dtype):
    width = 48
    w = rh.draw_weights(rh.config([(entry, None)], width=width), 6, sharp=1.5)
    rng = np.random.default_rng(7)
    lens, extra = [150, 4, 1], 9
    xs = [pr.round_bf16(rng.standard_normal((n + extra, width))) for n in lens]
    got = run_mixer(make_mixer(entry, dtype, w, width), dtype, xs, prompt_then_tokens(lens, extra))
    for g, x in zip(got, xs):
        assert close(g, plain_mixer(entry, x, w, dtype), dtype)


@pytest.mark.parametrize("size, pool", [(0, 0), (1, 1), (5, 0), (63, 4), (64, 64), (65, 7), (100, 12), (200, 3)])
@pytest.mark.parametrize("sizes", [dict(heads=4, kv_heads=2, dim=32, vdim=24), dict(heads=2, kv_heads=2, dim=64, vdim=64),
                                   dict(heads=3, kv_heads=1, dim=16, vdim=136, layout="interleaved"),
                                   dict(heads=2, kv_heads=1, dim=128, vdim=8)])
def test_prompts_on_the_tensor_cores(sizes, size, pool, monkeypatch):
    """bfloat16 steps of more than one token per sequence take the tensor-core kernel: against the plain implementation
    and against the plain kernel, for windows and blocks around the key tile of 64, prompts that cross tiles, end
    inside one or are a single token, whole, and continued in portions whose tiles start inside a page."""
    entry = rh.attention(size=size, pool=pool, dims=8, **sizes)
    width, dtype = 48, torch.bfloat16
    w = rh.draw_weights(rh.config([(entry, None)], width=width), 14, sharp=1.5)
    rng = np.random.default_rng(15)
    lens = [330, 70, 1, 64]
    xs = [pr.round_bf16(rng.standard_normal((n, width))) for n in lens]
    refs = [plain_mixer(entry, x, w, dtype) for x in xs]
    part = make_mixer(entry, dtype, w, width)
    assert ops.pool_prefill_mma_fits(dtype, sizes["dim"], sizes["vdim"])
    plans = ([lens], [[100, 3, 1, 63], [230, 67, 0, 1]], [[1, 1, 1, 1], [129, 2, 0, 2], [200, 67, 0, 61]])
    fast = [run_mixer(part, dtype, xs, plan) for plan in plans]
    real = ops.pool_attention
    monkeypatch.setattr(ops, "pool_attention", lambda *a, **k: real(*a, **{**k, "impl": "plain"}))
    slow = run_mixer(part, dtype, xs, plans[0])
    for i, ref in enumerate(refs):
        for got in fast:
            assert close(got[i], ref, dtype), i
        assert np.sqrt(np.mean((fast[0][i] - slow[i]) ** 2)) <= 0.01 * np.sqrt(np.mean(ref ** 2))
    assert not ops.pool_prefill_mma_fits(torch.float32, 64, 64) and not ops.pool_prefill_mma_fits(dtype, 24, 16)


def aligned_keys(w, n):
    """The key projection and norm made equal to the first query head's: a token's key then points where its own query
    points, and the query's weight goes to its doubles (and itself), far above every other key."""
    w["l0.mix.k"], w["l0.mix.k.norm"] = w["l0.mix.q"][:n].copy(), w["l0.mix.q.norm"].copy()
    return w


def standing_out(T, width, seed, pairs):
    """Inputs in which, for each (query, keys) of ``pairs``, the keys' tokens repeat the query's token: with sharp q and k
    that query's weight goes to those keys if it sees them, and elsewhere if it does not."""
    x = np.random.default_rng(seed).standard_normal((T, width))
    for query, keys in pairs:
        for j in keys:
            x[j] = x[query]
    return pr.round_bf16(x)


@pytest.mark.parametrize("size, pool", [(20, 5), (70, 12), (64, 64), (7, 7), (3, 1), (130, 3)])
def test_keys_at_the_edges_of_window_and_blocks(size, pool):
    """A query's double sits just inside its window, just outside it, in the block that is seen last, in the block that is
    not yet seen, far back in the first block, and at a page's first and last row: in a prompt, in a prompt cut there,
    and decoded.  Sharp q and k: a key seen or missed by one position moves the output by far more than the tolerance."""
    entry = rh.attention(heads=2, kv_heads=1, dim=16, vdim=24, size=size, pool=pool, dims=0, scale=0.5)
    width, dtype = 32, torch.float32
    w = aligned_keys(rh.draw_weights(rh.config([(entry, None)], width=width), 8, sharp=2.5), 16)
    part = make_mixer(entry, dtype, w, width)
    for q in (4 * size + 3 * pool, size + 2 * pool, size + 2 * pool + 1, 129, 192):
        if q < size + pool:
            continue
        T = q + 3                                             # the sequence ends soon after the query
        seen = (q - size + 1) // pool                         # blocks 0 .. seen - 1 are seen
        cases = {"window_in": [q - size + 1], "window_out": [q - size], "first": [0],
                 "block_in": list(range((seen - 1) * pool, seen * pool)),
                 "block_out": [j for j in range(seen * pool, (seen + 1) * pool) if j <= q - size],
                 "page_first": [64 * ((q - 1) // 64)], "page_last": [64 * ((q - 1) // 64) - 1]}
        for name, keys in cases.items():
            keys = [j for j in keys if 0 <= j < q]
            if not keys:
                continue
            x = standing_out(T, width, q, [(q, keys)])
            ref = plain_mixer(entry, x, w, dtype)
            for plan in ([[T]], [[q], [3]], [[q], [1], [1], [1]], [[q - 1], [2], [2]]):
                got = run_mixer(part, dtype, [x], plan)[0]
                assert close(got, ref, dtype), (q, name, plan[0])
    # the sharpness does what the test needs: hiding one key changes the output by much more than the tolerance
    T = 2 * size + 2
    x = standing_out(T, width, 1, [(T - 1, [T - size])])
    a = plain_mixer(entry, x, w, dtype)[T - 1]
    x[T - size] = -x[T - size]
    assert np.abs(a - plain_mixer(entry, x, w, dtype)[T - 1]).max() > 100 * FP32_TOL * np.abs(a).max()


def test_a_far_key_among_hundreds():
    """700 tokens; the query's doubles fill one block of the far past: it is seen only as that block's mean."""
    entry = rh.attention(heads=2, kv_heads=2, dim=16, vdim=16, size=40, pool=8, dims=0, scale=0.5)
    width, dtype, T = 32, torch.float32, 700
    w = aligned_keys(rh.draw_weights(rh.config([(entry, None)], width=width), 9, sharp=2.5), 32)
    x = standing_out(T, width, 10, [(T - 1, range(64, 72)), (650, range(120, 128)), (300, range(0, 8))])
    ref = plain_mixer(entry, x, w, dtype)
    part = make_mixer(entry, dtype, w, width)
    for plan in ([[T]], [[640]] + [[1]] * 60, [[299], [2], [399]]):
        assert close(run_mixer(part, dtype, [x], plan)[0], ref, dtype), plan[0]


# ----------------------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, cfgd, seed in (("mixed", rh.MIXED, 11), ("ones", rh.ONES, 12)):
        w = rh.draw_weights(cfgd, seed)
        out[name] = (rh.write_folder(str(tmp_path_factory.mktemp(name)), cfgd, w), cfgd, w)
    return out


def all_rows(eng, slot, tokens):
    return eng.step([StepEntry(slot, tokens, list(range(len(tokens))))]).double().cpu().numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "ones"])
def test_whole_prompts_portions_batches_and_reuse(models, name, dtype):
    folder, cfgd, w = models[name]
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    V = cfgd["vocab"]
    rng = np.random.default_rng(13)
    seqs = [rng.integers(0, V, n).tolist() for n in (150, 1, 67, 9)]
    refs = [pr.forward(t, w, cfgd, td == torch.bfloat16) for t in seqs]
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_batch=6)
    alone = []
    for t, ref in zip(seqs, refs):                          # each alone, whole
        (s,) = eng.open_sequences(1)
        alone.append(all_rows(eng, s, t))
        eng.close_sequences([s])
        assert close(alone[-1], ref, td)
    # all in one batch of unequal lengths, in slots and pages that were used before: the same as alone
    slots = eng.open_sequences(4)
    out = eng.step([StepEntry(s, t, list(range(len(t)))) for s, t in zip(slots, seqs)]).double().cpu().numpy()
    eng.close_sequences(slots)
    off = 0
    for t, ref, one in zip(seqs, refs, alone):
        assert close(out[off:off + len(t)], ref, td)
        if td == torch.float32:
            assert np.abs(out[off:off + len(t)] - one).max() <= FP32_TOL * np.abs(ref).max()
        off += len(t)
    # portions of several sizes, down to two tokens, in slots that were used before
    (s,) = eng.open_sequences(1)
    rows, at = [], 0
    for n in (2, 3, 60, 2, 17, 64, 2):
        rows.append(all_rows(eng, s, seqs[0][at:at + n]))
        at += n
    assert at == 150 and close(np.concatenate(rows), refs[0], td)
    eng.close_sequences([s])
    # prompts cut at unequal places, then token by token together; the shorter ones end earlier and give their slots back
    cuts = [60, 1, 3, 8]
    slots = eng.open_sequences(4)
    rows = {i: [] for i in range(4)}
    first = eng.step([StepEntry(s, t[:c], list(range(c))) for s, t, c in zip(slots, seqs, cuts)]).double().cpu().numpy()
    off = 0
    for i, c in enumerate(cuts):
        rows[i] += list(first[off:off + c])
        off += c
    pos, live = list(cuts), [i for i in range(4) if cuts[i] < len(seqs[i])]
    eng.close_sequences([slots[i] for i in range(4) if i not in live])
    while live:
        out = eng.step([StepEntry(slots[i], [seqs[i][pos[i]]], [0]) for i in live]).double().cpu().numpy()
        for r, i in enumerate(live):
            rows[i].append(out[r])
            pos[i] += 1
        done = [i for i in live if pos[i] == len(seqs[i])]
        eng.close_sequences([slots[i] for i in done])
        live = [i for i in live if i not in done]
    for i, ref in enumerate(refs):
        assert close(np.stack(rows[i]), ref, td), i
    assert eng.cache.slots.n_free == eng.max_batch and eng.cache.free_pages() == [g.pool.n for g in eng.cache._groups]


def test_a_wide_model_through_the_tensor_core_paths(tmp_path):
    """Width 2,048 and a prompt of 600 tokens: the feed-forward's activation runs in the tcgen05 product's epilogue, the
    attention's prompt on the tensor cores, the recurrence in chunks; then single tokens."""
    cfgd = rh.config([(rh.rglru(width=96, blocks=3, conv=4), rh.dense(ff=264)),
                      (rh.attention(heads=4, kv_heads=2, dim=32, vdim=16, size=100, pool=9, dims=8), rh.dense(ff=72))],
                     width=2048, vocab=128)
    w = rh.draw_weights(cfgd, 41)
    folder = rh.write_folder(str(tmp_path / "m"), cfgd, w)
    tokens = np.random.default_rng(3).integers(0, 128, 606).tolist()
    ref = pr.forward(tokens, w, cfgd, round16=True)
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=2048, max_batch=2)
    (s,) = eng.open_sequences(1)
    rows = list(all_rows(eng, s, tokens[:600]))
    for t in tokens[600:]:
        rows.append(eng.step([StepEntry(s, [t], [0])]).double().cpu().numpy()[0])
    assert close(np.stack(rows), ref, torch.bfloat16)


def test_layer_by_layer(models):
    """The stream after every scheduled run (a looped layer counts each time) against the plain implementation."""
    folder, cfgd, w = models["mixed"]
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=512, max_batch=2)
    tokens = np.random.default_rng(29).integers(0, cfgd["vocab"], 90).tolist()
    want = []
    pr.forward(tokens, w, cfgd, layers_out=want)
    (s,) = eng.open_sequences(1)
    ctx, rows = eng.build_context([StepEntry(s, tokens, [0])])
    got = []
    eng.model.forward(ctx, eng.unit_caches, rows, tap=lambda i, h: got.append(h.double().cpu().numpy()))
    assert len(got) == len(want) == 11
    for g, r in zip(got, want):
        assert np.abs(g - r).max() <= FP32_TOL * np.abs(r).max()


def test_long_decoding_over_windows_blocks_and_page_borders(models):
    folder, cfgd, w = models["mixed"]
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=512, max_batch=2)
    tokens = np.random.default_rng(19).integers(0, cfgd["vocab"], 280).tolist()
    ref = pr.forward(tokens, w, cfgd)
    (s,) = eng.open_sequences(1)
    rows = list(all_rows(eng, s, tokens[:2]))
    for t in tokens[2:]:
        rows.append(eng.step([StepEntry(s, [t], [0])]).double().cpu().numpy()[0])
    assert close(np.stack(rows), ref, torch.float32)


@pytest.mark.parametrize("layers", [[(rh.rglru(width=24, blocks=2, conv=3), rh.dense(ff=24)), (rh.rglru(width=16, blocks=1, conv=2), None)],
                                    [(rh.attention(heads=2, kv_heads=2, dim=8, vdim=8, size=3, pool=2, dims=8), rh.dense(ff=8))]],
                         ids=["no_cache_rows", "no_state"])
def test_models_with_one_kind_of_mixer_only(layers, tmp_path):
    import questwend_b200 as qw
    cfgd = rh.config(layers, width=24, vocab=40)
    w = rh.draw_weights(cfgd, 31)
    folder = rh.write_folder(str(tmp_path / "m"), cfgd, w)
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=512, max_batch=3)
    tokens = np.random.default_rng(2).integers(0, 40, 70).tolist()
    ref = pr.forward(tokens, w, cfgd)
    (s,) = eng.open_sequences(1)
    rows = list(all_rows(eng, s, tokens[:66]))
    for t in tokens[66:]:
        rows.append(eng.step([StepEntry(s, [t], [0])]).double().cpu().numpy()[0])
    eng.close_sequences([s])
    assert close(np.stack(rows), ref, torch.float32)
    for use_graph in (True, False):
        out = qw.generate(eng, [tokens[:5], tokens[:1]], max_new_tokens=8, use_graph=use_graph)
        for p, r in zip([tokens[:5], tokens[:1]], out):
            full = pr.forward(p + r.tokens, w, cfgd)
            for j, tok in enumerate(r.tokens):
                row = full[len(p) - 1 + j]
                assert row.max() - row[tok] <= 2 * FP32_TOL * np.abs(full).max()


def test_generation_through_the_library_loop(models):
    """Greedy generation with the engine's own loop, scheduler, device sampler and CUDA graphs: two batches in slots that
    are used again, one request ending early, decoding across windows, blocks and a page border; every chosen token is the
    plain implementation's choice."""
    import questwend_b200 as qw
    folder, cfgd, w = models["mixed"]
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=1024, max_batch=3)
    rng = np.random.default_rng(17)
    prompts = [rng.integers(0, cfgd["vocab"], n).tolist() for n in (20, 1, 58, 5)]
    n_new = 24
    for use_graph in (True, False):
        free = qw.generate(eng, prompts, max_new_tokens=n_new, use_graph=use_graph)
        stop = free[2].tokens[6]
        stats = qw.GenerationStats()
        res = qw.generate(eng, prompts, max_new_tokens=n_new, stop_ids=[stop], use_graph=use_graph, stats=stats)
        assert stats.batches == 2 and res[2].finish_reason == "stop" and len(res[2].tokens) <= 6
        for run in (free, res):
            for p, r in zip(prompts, run):
                ref = pr.forward(p + r.tokens, w, cfgd)
                scale = np.abs(ref).max()
                for j, tok in enumerate(r.tokens):
                    row = ref[len(p) - 1 + j]
                    assert row.max() - row[tok] <= 2 * FP32_TOL * scale, (len(p), j, tok, int(row.argmax()))
    assert eng.cache.slots.n_free == eng.max_batch


def test_trace_replay_and_command_line(models, tmp_path):
    folder, cfgd, w = models["ones"]
    V = cfgd["vocab"]
    rng = np.random.default_rng(23)
    a, b = rng.integers(0, V, 9).tolist(), rng.integers(0, V, 4).tolist()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:7], "want": [0, 6]}, {"id": "b", "tokens": b[:3], "want": [2]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[7:8], "want": []}, {"id": "b", "tokens": b[3:], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[8:], "want": [0]}], "end": ["a"]}]
    out = run_trace(folder, "float32", steps, 256, str(tmp_path / "out"))
    ra, rb = pr.forward(a, w, cfgd), pr.forward(b, w, cfgd)
    assert close(out[0], np.stack([ra[0], ra[6], rb[2]]), torch.float32)
    assert close(out[1], rb[3:4], torch.float32) and close(out[2], ra[8:9], torch.float32)
    import os
    import subprocess
    import sys
    from helpers import ROOT
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qw-cli"), "-m", folder, "-p", " ".join(map(str, a)),
                           "-n", "5", "--dtype", "float32", "--n-ctx", "128"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    ids = [int(x) for x in proc.stdout.split()]
    ref = pr.forward(a + ids, w, cfgd)
    for j, tok in enumerate(ids):
        row = ref[len(a) - 1 + j]
        assert row.max() - row[tok] <= 2 * FP32_TOL * np.abs(ref).max()
