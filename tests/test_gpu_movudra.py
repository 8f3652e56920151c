"""The Movudra design in the engine against the plain implementation (``plain_movudra``): every mechanism alone, whole
prompts against token-by-token decoding, batches of unequal requests, slots and pages that are used again, windows and
page borders, long decoding, sizes that are 1 or equal, generation through the library's own loop, and trace replay
(needs a B200)."""
import numpy as np
import pytest
import torch

import movudra_helpers as mh
import plain_movudra as pmv
from helpers import FP32_TOL, run_trace
from questwend_b200.cache import CacheManager
from questwend_b200.engine.engine import Engine, StepEntry, build_step_context
from questwend_b200.parts import PartSpec, Runtime, build_part

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]
BF16_RMS_TOL = 0.03         # bfloat16 engine against the plain implementation that rounds the products' operands: the
                            # root mean square of the difference over that of the reference (the engine also rounds the
                            # cached latents and the queries' unrotated parts, which the plain one does not)


def r16(dtype):
    return None if dtype == torch.float32 else "bf16"


def close(got, ref, dtype):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    if dtype == torch.float32:
        return np.abs(got - ref).max() <= FP32_TOL * np.abs(ref).max()
    return np.sqrt(np.mean((got - ref) ** 2)) <= BF16_RMS_TOL * np.sqrt(np.mean(ref ** 2))


# ----------------------------------------------------------------------------- every mechanism alone
def mixer_alone(entry, dtype, lens, extra, seed, width=48, slow_decay=False, sink_scale=None):
    """A mixer part on random inputs: prompts of ``lens`` tokens in one step, then ``extra`` steps of one token each,
    against the plain function on the whole sequences."""
    import questwend_b200  # noqa: F401
    from questwend_b200.config.registry import config_from_dict
    from questwend_b200.models.movudra import _mixer
    cfgd = mh.config([(entry, None)], width=width)
    w = mh.draw_weights(cfgd, seed, slow_decay=slow_decay)
    if sink_scale is not None:
        for k in w:
            if k.endswith(".sink"):
                w[k] = pmv.round_bf16(sink_scale * np.ones_like(w[k]))
    cfg = config_from_dict(cfgd)
    m = cfg.layers[0]["mixer"]
    spec, pos_spec = _mixer(entry["type"], m, width, 1e-5)
    rt = Runtime(DEV, dtype)
    position = build_part("position", pos_spec, rt) if pos_spec is not None else None
    part = build_part("mixer", PartSpec(spec.kind, spec.params, prefix="l0.mix."), rt, position=position)
    held = {}
    for t in part.tensors():
        v = torch.from_numpy(w[t.name])
        held[t.name] = v.to(dtype if t.role == "matrix" else torch.float32).to(DEV)
    part.bind(held)
    cache = CacheManager([(part.kv_spec(), part.state_spec(), None)], max(2048, sum(lens) + 64 * len(lens) + 512), 8, 2048, dtype, DEV)
    unit = cache.unit_cache(0)
    rng = np.random.default_rng(seed + 1)
    xs = [pmv.round_bf16(rng.standard_normal((n + extra, width))) for n in lens]
    refs = [pmv.MIXERS[entry["type"]](x, w, "l0.mix.", entry["mixer"], 1e-5, r16(dtype)) for x in xs]
    slots = cache.open(len(lens))
    got = [[] for _ in lens]

    def step(chunks):
        ctx = build_step_context(cache, [StepEntry(s, [0] * len(c), []) for s, c in zip(slots, chunks)], 10 ** 6, DEV)[0]
        out = part.forward(torch.from_numpy(np.concatenate(chunks)).to(dtype).to(DEV), ctx, unit).double().cpu().numpy()
        off = 0
        for i, (s, c) in enumerate(zip(slots, chunks)):
            got[i].append(out[off:off + len(c)])
            off += len(c)
            cache.advance(s, len(c))

    step([x[:n] for x, n in zip(xs, lens)])
    for j in range(extra):
        step([x[n + j:n + j + 1] for x, n in zip(xs, lens)])
    return [np.concatenate(g) for g in got], refs


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("entry", [mh.mamba(), mh.mamba(heads=2, vdim=40, state=72, groups=1, norm_groups=1, conv=1),
                                   mh.mamba(heads=4, vdim=8, state=20, groups=4, norm_groups=4, conv=8),
                                   mh.mamba(heads=2, vdim=6, state=160, groups=2, norm_groups=3, conv=2),
                                   mh.mamba(heads=1, vdim=3, state=264, groups=1, norm_groups=1, conv=2)])
def test_mamba2_alone(entry, dtype):
    got, refs = mixer_alone(entry, dtype, [70, 3, 1], 6, seed=1)
    for g, r in zip(got, refs):
        assert close(g, r, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("entry", [mh.delta(), mh.delta(heads=4, kv_heads=1, dim=72, vdim=8, conv=2),
                                   mh.delta(heads=2, kv_heads=2, dim=8, vdim=40, conv=1),
                                   mh.delta(heads=2, kv_heads=1, dim=136, vdim=6, conv=3),
                                   mh.delta(heads=1, kv_heads=1, dim=260, vdim=5, conv=2)])
def test_gated_delta_rule_alone(entry, dtype):
    got, refs = mixer_alone(entry, dtype, [66, 2, 1], 6, seed=2)
    for g, r in zip(got, refs):
        assert close(g, r, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("entry", [mh.latent(), mh.latent(heads=5, dim=16, rot_dim=12, dims=8, vdim=16, kv_rank=24, window=70, scaling=False),
                                   mh.latent(heads=17, dim=8, rot_dim=4, vdim=8, kv_rank=72, q_rank=8, window=0, base=50.0)])
def test_latent_attention_alone(entry, dtype):
    got, refs = mixer_alone(entry, dtype, [130, 4, 1], 8, seed=3)
    for g, r in zip(got, refs):
        assert close(g, r, dtype)


@pytest.mark.parametrize("window", [0, 1, 2, 63, 64, 65, 100])
@pytest.mark.parametrize("sizes", [dict(heads=3, dim=24, rot_dim=8, vdim=40, kv_rank=40), dict(heads=2, dim=64, rot_dim=16, vdim=64, kv_rank=48),
                                   dict(heads=1, dim=8, rot_dim=8, vdim=8, kv_rank=8, q_rank=8),
                                   dict(heads=2, dim=24, rot_dim=8, vdim=136, kv_rank=16, q_rank=16)])
def test_whole_prompts_on_the_tensor_cores(sizes, window, monkeypatch):
    """bfloat16 prompts that start their sequences take the tensor-core kernel (keys and values per head made from the
    latents): against the plain implementation, and against the kernel that scores the latents themselves, for windows
    around the key tile of 64 and prompts that cross two tiles, end inside one, or are a single token."""
    from questwend_b200.kernels import ops
    from questwend_b200.parts import latent_attention as la
    entry = mh.latent(window=window, **sizes)
    assert ops.latent_prefill_fits(torch.bfloat16, sizes["dim"], sizes["rot_dim"], sizes["vdim"], sizes["kv_rank"])
    calls = []
    kernel = ops.latent_prefill
    monkeypatch.setattr(ops, "latent_prefill", lambda *a, **k: calls.append(1) or kernel(*a, **k))
    got, refs = mixer_alone(entry, torch.bfloat16, [150, 64, 20, 1], 3, seed=21)
    assert len(calls) == 1                                           # the prompts' step took it, the single tokens did not
    monkeypatch.setattr(la, "PROMPT_KERNEL_MIN_TOKENS", 10 ** 9)
    plain, _ = mixer_alone(entry, torch.bfloat16, [150, 64, 20, 1], 3, seed=21)
    assert len(calls) == 1
    for g, p, r in zip(got, plain, refs):
        assert close(g, r, torch.bfloat16) and close(p, r, torch.bfloat16)
        assert np.sqrt(np.mean((g - p) ** 2)) <= 0.02 * np.sqrt(np.mean(r ** 2))


def test_a_far_token_reaches_through_a_slowly_decaying_state():
    """Decays close to 1: what the first tokens wrote is still read hundreds of tokens later, in the prompt and in the
    tokens decoded after it (a state that was lost or restarted would show)."""
    for entry in (mh.mamba(), mh.delta()):
        got, refs = mixer_alone(entry, torch.float32, [300], 40, seed=4, slow_decay=True)
        assert close(got[0], refs[0], torch.float32)
        # and the far tokens do matter: the same sequence with its first 10 inputs changed differs at the end
        x = pmv.round_bf16(np.random.default_rng(5).standard_normal((340, 48)))
        w = mh.draw_weights(mh.config([(entry, None)], width=48), 4, slow_decay=True)
        a = pmv.MIXERS[entry["type"]](x, w, "l0.mix.", entry["mixer"], 1e-5)
        x2 = x.copy()
        x2[:10] = -x2[:10]
        b = pmv.MIXERS[entry["type"]](x2, w, "l0.mix.", entry["mixer"], 1e-5)
        assert np.abs(a[-1] - b[-1]).max() > 100 * FP32_TOL * np.abs(a).max()


@pytest.mark.parametrize("window", [1, 2, 63, 64, 65, 100])
def test_window_edges_show(window):
    """A large score scale makes the softmax pick almost one key, so a window that is one token off picks another one:
    windows around the page size of 64, in a prompt that crosses two page borders and in the tokens decoded after it."""
    entry = mh.latent(heads=2, dim=16, rot_dim=4, vdim=16, kv_rank=16, q_rank=16, window=window, scale=6.0)
    got, refs = mixer_alone(entry, torch.float32, [150, 62], 12, seed=6)
    for g, r in zip(got, refs):
        assert close(g, r, torch.float32)
    wrong = dict(entry, mixer={**entry["mixer"], "mask": {"size": window + 1}})
    w = mh.draw_weights(mh.config([(entry, None)], width=48), 6)
    x = pmv.round_bf16(np.random.default_rng(7).standard_normal((162, 48)))
    a = pmv.latent_attention(x, w, "l0.mix.", entry["mixer"], 1e-5)
    b = pmv.latent_attention(x, w, "l0.mix.", wrong["mixer"], 1e-5)
    assert np.abs(a - b).max() > 1000 * FP32_TOL * np.abs(a).max()      # the plain implementation does tell them apart


def test_single_tokens_of_many_long_sequences():
    """Eight sequences of about a thousand keys: enough runs of keys that a block takes 16 (token, head) rows (few
    sequences take 4), and the merge adds up 16 runs; with and without a window."""
    for window in (0, 300):
        entry = mh.latent(heads=2, dim=16, rot_dim=4, vdim=16, kv_rank=16, q_rank=16, window=window)
        got, refs = mixer_alone(entry, torch.float32, [1000, 1010, 990, 1001, 1000, 1000, 999, 1003], 2, seed=9)
        for g, r in zip(got, refs):
            assert close(g[-2:], r[-2:], torch.float32)


def test_the_sink_counts():
    """Sinks as large as the largest scores: leaving the sink out, or scaling it, would change every output."""
    entry = mh.latent(heads=3, window=9)
    got, refs = mixer_alone(entry, torch.float32, [40, 1], 5, seed=8, sink_scale=3.0)
    for g, r in zip(got, refs):
        assert close(g, r, torch.float32)
    got0, refs0 = mixer_alone(entry, torch.float32, [40, 1], 5, seed=8, sink_scale=-30.0)     # no sink to speak of
    assert close(got0[0], refs0[0], torch.float32)
    assert np.abs(refs[0] - refs0[0]).max() > 0.05 * np.abs(refs0[0]).max()


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forwards_alone(dtype):
    from questwend_b200.models.movudra import _feed_forward
    rt = Runtime(DEV, dtype)
    width = 40
    for mlp in (mh.dense(ff=56), mh.moe(ff=24, experts=7, top=3), mh.moe(ff=8, experts=2, top=2), mh.moe(ff=16, experts=5, top=1)):
        cfgd = mh.config([(mh.mamba(), mlp)], width=width)
        w = mh.draw_weights(cfgd, 9)
        spec = _feed_forward(mlp, width)
        part = build_part("feed_forward", PartSpec(spec.kind, spec.params, prefix="l0.mlp."), rt)
        part.bind({t.name: torch.from_numpy(w[t.name]).to(dtype if t.role == "matrix" else torch.float32).to(DEV)
                   for t in part.tensors()})
        for T in (1, 5, 37):
            x = pmv.round_bf16(np.random.default_rng(T).standard_normal((T, width)))
            ref = (pmv.dense_ff(x, w, "l0.mlp.", r16(dtype)) if mlp["kind"] == "dense"
                   else pmv.moe_ff(x, w, "l0.mlp.", mlp, r16(dtype)))
            got = part.forward(torch.from_numpy(x).to(dtype).to(DEV), None).double().cpu().numpy()
            assert close(got, ref, dtype), (mlp, T)


def test_router_weights_are_the_scores_themselves():
    from questwend_b200.kernels import ops
    z = torch.tensor([[2.0, 0.0, 1.0, -1.0, 1.5], [0.0, 0.0, 0.0, 0.0, 0.0]], device=DEV)
    chosen, weight = ops.moe_route(z, 2)
    s = torch.softmax(z.double(), -1).cpu().numpy()
    assert chosen.cpu().tolist() == [[0, 4], [0, 1]]                       # ties go to the lower index
    assert np.allclose(weight.cpu().numpy(), [[s[0, 0], s[0, 4]], [0.2, 0.2]], atol=1e-6)    # not renormalised
    _, renorm = ops.moe_route(z, 2, renormalize=True)
    assert np.allclose(renorm.cpu().numpy().sum(-1), 1.0, atol=1e-6)


def test_the_prompt_kernel_is_refused_where_its_tiles_do_not_fit():
    from questwend_b200.kernels import ops
    assert ops.latent_prefill_fits(torch.bfloat16, 128, 64, 128, 512)
    assert not ops.latent_prefill_fits(torch.bfloat16, 448, 64, 256, 512)        # 3 x 64 x 520 + 2 x 64 x 264 values: too much
    assert not ops.latent_prefill_fits(torch.float32, 128, 64, 128, 512)
    assert not ops.latent_prefill_fits(torch.bfloat16, 100, 28, 128, 512)        # parts in multiples of 8


def test_paired_rotation_table():
    from questwend_b200.parts.rotary import scaled_frequencies
    for dims, base, sc in ((8, 10000.0, None), (12, 500.0, {"factor": 8.0, "fast": 16.0, "original": 64, "slow": 2.0}),
                           (2, 30.0, {"factor": 3.0, "fast": 4.0, "original": 16, "slow": 1.0})):
        f, mult = scaled_frequencies(dims, base, **(sc or {}))
        f_ref, mult_ref = pmv.yarn_frequencies(dims, base, sc)
        assert np.allclose(f.numpy(), f_ref, rtol=1e-14) and abs(mult - mult_ref) < 1e-14


# ----------------------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    import copy
    for name, cfgd, seed in (("mixed", mh.MIXED, 11), ("ones", mh.ONES, 12)):
        sized = copy.deepcopy(cfgd)
        sized["layers"][0]["mixer"].update({"decay_rank": 8, "gate_rank": 24})   # low ranks that only the tensors' shapes
        w = mh.draw_weights(sized, seed)                                        # tell: the written config.json has none
        out[name] = (mh.write_folder(str(tmp_path_factory.mktemp(name)), cfgd, w), cfgd, w)
    return out


def all_rows(eng, slot, tokens):
    return eng.step([StepEntry(slot, tokens, list(range(len(tokens))))]).double().cpu().numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "ones"])
def test_whole_prompts_decoding_batches_and_reuse(models, name, dtype):
    folder, cfgd, w = models[name]
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    V = cfgd["vocab"]
    rng = np.random.default_rng(13)
    seqs = [rng.integers(0, V, n).tolist() for n in (150, 1, 67, 9)]
    refs = [pmv.forward(cfgd, w, t, r16(td)) for t in seqs]
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_batch=6)
    assert (eng.config.layers[0]["mixer"]["decay_rank"], eng.config.layers[0]["mixer"]["gate_rank"]) == (8, 24)
    # each alone, whole
    alone = []
    for t, ref in zip(seqs, refs):
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
    assert eng.cache.slots.n_free == eng.max_batch and all(f == eng.cache.n_pages for f in eng.cache.free_pages())


@pytest.mark.parametrize("layers", [[(mh.mamba(heads=2, vdim=8, state=16, groups=2, norm_groups=2), mh.dense(ff=24)), (mh.delta(heads=2, kv_heads=2, dim=8, vdim=8), None)],
                                    [(mh.latent(heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=16, q_rank=8, window=3), mh.moe(ff=8, experts=4, top=2))]],
                         ids=["no_cache_rows", "no_state"])
def test_models_with_one_kind_of_mixer_only(layers, tmp_path):
    """A model without attention has no cache pages at all, one without recurrent layers no per-slot state: the cache
    manager, the step function and generation (CUDA graphs too) take both."""
    import questwend_b200 as qw
    cfgd = mh.config(layers, width=24, vocab=40)
    w = mh.draw_weights(cfgd, 31)
    folder = mh.write_folder(str(tmp_path / "m"), cfgd, w)
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=512, max_batch=3)
    tokens = np.random.default_rng(2).integers(0, 40, 70).tolist()
    ref = pmv.forward(cfgd, w, tokens)
    (s,) = eng.open_sequences(1)
    rows = list(all_rows(eng, s, tokens[:66]))
    for t in tokens[66:]:
        rows.append(eng.step([StepEntry(s, [t], [0])]).double().cpu().numpy()[0])
    eng.close_sequences([s])
    assert close(np.stack(rows), ref, torch.float32)
    for use_graph in (True, False):
        out = qw.generate(eng, [tokens[:5], tokens[:1]], max_new_tokens=8, use_graph=use_graph)
        for p, r in zip([tokens[:5], tokens[:1]], out):
            full = pmv.forward(cfgd, w, p + r.tokens)
            for j, tok in enumerate(r.tokens):
                row = full[len(p) - 1 + j]
                assert row.max() - row[tok] <= 2 * FP32_TOL * np.abs(full).max()


def test_generation_through_the_library_loop(models):
    """Greedy generation with the engine's own loop, scheduler, device sampler and CUDA graphs: two batches in slots that
    are used again, one request ending early; every chosen token is the plain implementation's choice."""
    import questwend_b200 as qw
    folder, cfgd, w = models["mixed"]
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=1024, max_batch=3)
    rng = np.random.default_rng(17)
    prompts = [rng.integers(0, cfgd["vocab"], n).tolist() for n in (20, 1, 66, 5)]
    n_new = 12
    for use_graph in (True, False):
        free = qw.generate(eng, prompts, max_new_tokens=n_new, use_graph=use_graph)
        stop = free[2].tokens[6]
        stats = qw.GenerationStats()
        res = qw.generate(eng, prompts, max_new_tokens=n_new, stop_ids=[stop], use_graph=use_graph, stats=stats)
        assert stats.batches == 2 and res[2].finish_reason == "stop" and len(res[2].tokens) <= 6
        for run in (free, res):
            for p, r in zip(prompts, run):
                ref = pmv.forward(cfgd, w, p + r.tokens)
                scale = np.abs(ref).max()
                for j, tok in enumerate(r.tokens):
                    row = ref[len(p) - 1 + j]
                    assert row.max() - row[tok] <= 2 * FP32_TOL * scale, (len(p), j, tok, int(row.argmax()))
    assert eng.cache.slots.n_free == eng.max_batch


def test_long_decoding_over_window_and_page_borders(models):
    folder, cfgd, w = models["mixed"]
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=512, max_batch=2)
    tokens = np.random.default_rng(19).integers(0, cfgd["vocab"], 200).tolist()
    ref = pmv.forward(cfgd, w, tokens)
    (s,) = eng.open_sequences(1)
    rows = list(all_rows(eng, s, tokens[:2]))
    for t in tokens[2:]:
        rows.append(eng.step([StepEntry(s, [t], [0])]).double().cpu().numpy()[0])
    assert close(np.stack(rows), ref, torch.float32)


def test_trace_replay_and_command_line(models, tmp_path):
    folder, cfgd, w = models["ones"]
    V = cfgd["vocab"]
    rng = np.random.default_rng(23)
    a, b = rng.integers(0, V, 9).tolist(), rng.integers(0, V, 4).tolist()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:7], "want": [0, 6]}, {"id": "b", "tokens": b[:3], "want": [2]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[7:8], "want": []}, {"id": "b", "tokens": b[3:], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[8:], "want": [0]}], "end": ["a"]}]
    out = run_trace(folder, "float32", steps, 256, str(tmp_path / "out"))
    ra, rb = pmv.forward(cfgd, w, a), pmv.forward(cfgd, w, b)
    assert 1 not in out or out[1].shape[0] == 1
    assert close(out[0], np.stack([ra[0], ra[6], rb[2]]), torch.float32)
    assert close(out[1], rb[3:4], torch.float32) and close(out[2], ra[8:9], torch.float32)
    # the command line on the same folder: greedy ids are the plain implementation's
    import subprocess
    import sys
    from helpers import ROOT
    import os
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qw-cli"), "-m", folder, "-p", " ".join(map(str, a)),
                           "-n", "5", "--dtype", "float32", "--n-ctx", "128"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    ids = [int(x) for x in proc.stdout.split()]
    ref = pmv.forward(cfgd, w, a + ids)
    for j, tok in enumerate(ids):
        row = ref[len(a) - 1 + j]
        assert row.max() - row[tok] <= 2 * FP32_TOL * np.abs(ref).max()
