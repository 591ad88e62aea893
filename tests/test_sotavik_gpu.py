"""The Sotavik design in the engine against the plain statement of it (``plain_sotavik``): every
mechanism alone, then whole models through the step function in every way of cutting and
batching, and generation through the entry point."""
import math

import numpy as np
import pytest
import torch

import plain_sotavik as ps
import tiny_sotavik as ts

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def make_model(cfg, store, dtype, max_tokens=1024, **kw):
    from supersonic_b200.engine import Model
    return Model.from_config(cfg, store, dtype=dtype, device=DEV, max_tokens=max_tokens, **kw)


def run_in_portions(model, tokens, cuts):
    """Logits of every position [T, vocab] with the sequence fed in portions of the given sizes."""
    from supersonic_b200.engine import StepEntry
    slot, at, rows = model.open_sequence(), 0, []
    for n in cuts:
        rows.append(model.step([StepEntry(slot, tokens[at:at + n], list(range(n)))]).cpu())
        at += n
    assert at == len(tokens)
    model.close_sequence(slot)
    model.check_errors()
    return torch.cat(rows).double()


def close(got, ref, dtype, what=""):
    """float32: a few units of float32 rounding of the logits' size; bfloat16: the error's root mean square
    per position against the spread of that position's logits."""
    assert torch.isfinite(got).all(), what
    if dtype == torch.float32:
        assert float((got - ref).abs().max()) < 2e-4 * max(1.0, float(ref.abs().max())), what
    else:
        rel = (got - ref).pow(2).mean(-1).sqrt() / ref.std(-1).clamp_min(1e-6)
        assert float(rel.max()) < 0.08, (what, rel.max())


def tokens_of(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg.vocab, n).tolist()


# ---- the parts alone ---------------------------------------------------------------------------------
def part_context(dtype, store, max_positions=600):
    from supersonic_b200.csrc.kernel_sets import kernel_set_for
    from supersonic_b200.parts import BuildContext, WeightAccess
    return BuildContext(torch.device(DEV), dtype, kernel_set_for(dtype), WeightAccess(store, DEV), max_positions)


def step_context(build, cache, entries):
    from supersonic_b200.engine import StepContext, pack_step
    starts = [cache.length(e.slot) for e in entries]
    batch = pack_step(entries, starts, DEV)
    for e in entries:
        cache.reserve(e.slot, len(e.tokens))
    cache.sync()
    return StepContext(batch, cache, build.kernels, build.dtype)


def mixer_in_pieces(mixer, position, build, x, pieces, dtype):
    """The mixer's output for one sequence whose rows ``x`` arrive in pieces, through a cache of its own."""
    from supersonic_b200.cache import SequenceCache
    from supersonic_b200.engine import StepEntry
    cache = SequenceCache({0: mixer.cache_need()}, 1024, 1024, dtype, DEV)
    slot, at, out = cache.acquire(), 0, []
    for n in pieces:
        ctx = step_context(build, cache, [StepEntry(slot, [0] * n)])
        res = torch.zeros(n, x.shape[1], device=DEV)
        mixer.forward(ctx, x[at:at + n].to(DEV, dtype), res, 0, True, position)
        cache.advance(slot, n)
        out.append(res.cpu())
        at += n
    return torch.cat(out).double()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("P", 0), ("P", 2), ("Q", 1), ("Q", 3)])
@pytest.mark.parametrize("window", [None, 37])
def test_latent_attention_alone(dtype, name, layer, window):
    """A prompt that crosses two page borders, then portions of two and one: every position against the
    plain statement, with and without a window (keys just inside and just outside it on both paths)."""
    from supersonic_b200.parts import MIXERS, POSITION_ENCODINGS
    cfg, store, plain = ts.build(name)
    spec = cfg.build_spec().blocks[layer]
    build = part_context(dtype, store)
    params = dict(spec.mixer.params, window=window)
    mixer = MIXERS["latent_attention"](params, spec.mixer.weights, build)
    position = POSITION_ENCODINGS[spec.position.kind](spec.position.params, {}, build)
    assert position.interleaved
    T = 150
    x = torch.randn(T, cfg.width, generator=torch.Generator().manual_seed(layer)).to(dtype)
    ref = ps.latent_attention(x.double(), plain, f"l{layer}.mix", cfg.layers[layer]["mixer"], cfg.norm_eps, window=window)
    got = mixer_in_pieces(mixer, position, build, x.float(), [130, 2, 2] + [1] * 16, dtype)
    tol = 1e-4 if dtype == torch.float32 else 0.04
    assert float((got - ref).abs().max()) < tol * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("P", 1), ("Q", 0), ("Q", 2)])
def test_gated_linear_attention_alone(dtype, name, layer):
    from supersonic_b200.parts import MIXERS
    cfg, store, plain = ts.build(name)
    spec = cfg.build_spec().blocks[layer]
    build = part_context(dtype, store)
    mixer = MIXERS["gated_linear_attention"](spec.mixer.params, spec.mixer.weights, build)
    T = 90
    x = torch.randn(T, cfg.width, generator=torch.Generator().manual_seed(7 + layer)).to(dtype)
    ref, _ = ps.gated_linear_attention(x.double(), plain, f"l{layer}.mix", cfg.layers[layer]["mixer"], cfg.norm_eps)
    got = mixer_in_pieces(mixer, None, build, x.float(), [66, 2, 3] + [1] * 19, dtype)
    tol = 1e-4 if dtype == torch.float32 else 0.05
    assert float((got - ref).abs().max()) < tol * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("P", 0), ("P", 1), ("Q", 0), ("Q", 3)])
def test_experts_alone(dtype, name, layer):
    """Top 1, 2 and 3, with and without the shared expert; a step of one token and a step of many."""
    from supersonic_b200.cache import SequenceCache
    from supersonic_b200.engine import StepEntry
    from supersonic_b200.parts import FEED_FORWARDS
    cfg, store, plain = ts.build(name)
    spec = cfg.build_spec().blocks[layer]
    build = part_context(dtype, store)
    ff = FEED_FORWARDS["experts"](spec.feed_forward.params, spec.feed_forward.weights, build)
    cache = SequenceCache({}, 512, 512, dtype, DEV)
    for T in (1, 133):
        tokens = tokens_of(cfg, T, T)
        x = torch.randn(T, cfg.width, generator=torch.Generator().manual_seed(T)).to(dtype)
        ref = ps.table_experts(x.double(), tokens, plain, f"l{layer}.mlp", cfg.layers[layer]["mlp"])
        slot = cache.acquire()
        ctx = step_context(build, cache, [StepEntry(slot, tokens)])
        res = torch.zeros(T, cfg.width, device=DEV)
        ff.forward(ctx, x.to(DEV), res)
        cache.release(slot)
        tol = 1e-4 if dtype == torch.float32 else 0.04
        assert float((res.cpu().double() - ref).abs().max()) < tol * max(1.0, float(ref.abs().max()))


def test_scalar_norm_head_scale_and_depth_average_layer_by_layer():
    """float32: the stream after every layer (norm with one gain, parallel sublayers, weighted sum over
    depth), and the scaled logits, against the plain statement."""
    from supersonic_b200.engine import StepEntry
    for name in ("P", "Q"):
        cfg, store, plain = ts.build(name)
        model = make_model(cfg, store, torch.float32)
        tokens = tokens_of(cfg, 70, 3)
        ref, layers = ps.forward(cfg.to_dict(), plain, tokens, keep_layers=True)
        seen = []
        for b in model.blocks:
            def wrapped(ctx, res, c, w, f=b.forward):
                out = f(ctx, res, c, w)
                seen.append(out.cpu().double())
                return out
            b.forward = wrapped
        slot = model.open_sequence()
        got = model.step([StepEntry(slot, tokens, list(range(len(tokens))))]).cpu().double()
        for i, s in enumerate(seen):
            assert float((s - layers[i]).abs().max()) < 1e-4 * max(1.0, float(layers[i].abs().max())), (name, i)
        close(got, ref, torch.float32, name)


# ---- whole models through the step function --------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_portions_of_every_size_and_token_by_token(dtype, name):
    cfg, store, plain = ts.build(name)
    model = make_model(cfg, store, dtype)
    T = 140
    tokens = tokens_of(cfg, T, 5)
    ref = ps.forward(cfg.to_dict(), plain, tokens)
    for cuts in ([T], [64, 64, 12], [63, 2, 2, 61, 3, 7, 2], [1] * 6 + [2] * 3 + [128], [100] + [1] * 40):
        got = run_in_portions(model, tokens, cuts)
        close(got, ref, dtype, (name, cuts))
    assert model.cache.slots.n_held == 0
    model.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["R", "S"])
def test_sizes_that_no_fast_kernel_takes_and_sizes_that_all_take(dtype, name):
    """Odd widths, ranks and head sizes (every operation on its plain kernel, also in bfloat16) and round ones
    (every fast kernel, 40 heads over one cached row): a prompt in portions, then decoding, in a batch of two."""
    from supersonic_b200.engine import StepEntry
    cfg, store, plain = ts.build(name)
    model = make_model(cfg, store, dtype)
    seqs = [tokens_of(cfg, 150, 31), tokens_of(cfg, 70, 32)]
    refs = [ps.forward(cfg.to_dict(), plain, q) for q in seqs]
    slots = [model.open_sequence() for _ in seqs]
    got = [[], []]
    plan = [((0, 100), (0, 66)), ((100, 130), (66, 68))] + [((130 + i, 131 + i), (68 + i, 69 + i) if i < 2 else None) for i in range(20)]
    for step in plan:
        entries = [StepEntry(slots[i], seqs[i][lo_hi[0]:lo_hi[1]], list(range(lo_hi[1] - lo_hi[0])))
                   for i, lo_hi in enumerate(step) if lo_hi]
        rows = model.step(entries).cpu().double()
        at = 0
        for i, lo_hi in enumerate(step):
            if lo_hi:
                got[i].append(rows[at:at + lo_hi[1] - lo_hi[0]])
                at += lo_hi[1] - lo_hi[0]
    close(torch.cat(got[0]), refs[0], dtype, name)
    close(torch.cat(got[1]), refs[1], dtype, name)
    model.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batches_against_each_alone_and_reused_slots(dtype):
    """Five requests of 1 to 131 tokens start together and decode together, the short ones ending first;
    then other requests run in the slots and pages those gave back."""
    from supersonic_b200.engine import StepEntry
    cfg, store, plain = ts.build("Q")
    model = make_model(cfg, store, dtype, max_tokens=1024)
    # the third group's long prompts run their recurrences chunk-parallel beside short ones that do not fill a chunk
    for round_, lens in enumerate(([1, 5, 64, 65, 131], [131, 2, 66], [260, 3, 195, 64], [7, 129, 64, 3])):
        decode = [3, 9, 14, 6, 11][: len(lens)]
        seqs = [tokens_of(cfg, n + d, 100 * round_ + i) for i, (n, d) in enumerate(zip(lens, decode))]
        refs = [ps.forward(cfg.to_dict(), plain, s) for s in seqs]
        slots = [model.open_sequence() for _ in seqs]
        got = [[] for _ in seqs]
        rows = model.step([StepEntry(s, q[:n], list(range(n))) for s, q, n in zip(slots, seqs, lens)]).cpu().double()
        at = 0
        for i, n in enumerate(lens):
            got[i].append(rows[at:at + n])
            at += n
        for step in range(max(decode)):
            live = [i for i in range(len(seqs)) if step < decode[i]]
            rows = model.step([StepEntry(slots[i], [seqs[i][lens[i] + step]], [0]) for i in live]).cpu().double()
            for r, i in enumerate(live):
                got[i].append(rows[r:r + 1])
            for i in live:
                if step == decode[i] - 1:
                    model.close_sequence(slots[i])          # its slot and pages go back while the others go on
        for i in range(len(seqs)):
            close(torch.cat(got[i]), refs[i], dtype, (round_, i))
        model.check_errors()
        assert model.cache.slots.n_held == 0
        model.cache.check()


def sharpened(name, layer, factor):
    """The configuration's weights with one latent layer's queries scaled up, so that each query's softmax
    stands on very few keys (far ones among them) and a misplaced key, position or sink moves the logits
    by far more than any tolerance; sinks are set near the typical top score."""
    cfg, store, plain = ts.build(name)
    t = dict(plain)
    t[f"l{layer}.mix.q"] = (plain[f"l{layer}.mix.q"].float() * factor).bfloat16()
    t[f"l{layer}.mix.sink"] = torch.linspace(2.0, 9.0, plain[f"l{layer}.mix.sink"].numel()).bfloat16()
    from supersonic_b200.weights import WeightStore
    return cfg, WeightStore.from_tensors(t), t


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_keys_page_borders_first_tokens_and_sinks_show(dtype):
    cfg, store, plain = sharpened("P", 0, 6.0)
    T = 330
    tokens = tokens_of(cfg, T, 9)
    ref = ps.forward(cfg.to_dict(), plain, tokens)
    # the test is sharp: the attention of late queries stands on keys hundreds of tokens back, and the
    # sink matters (the same layer without it gives other outputs)
    x = torch.randn(T, cfg.width, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    m = cfg.layers[0]["mixer"]
    with_sink = ps.latent_attention(x, plain, "l0.mix", m, cfg.norm_eps)
    without = ps.latent_attention(x, plain, "l0.mix", m, cfg.norm_eps, use_sink=False)
    assert float((with_sink - without).abs().max()) > 0.2 * float(with_sink.abs().max())
    near_only = ps.latent_attention(x, plain, "l0.mix", m, cfg.norm_eps, window=128)
    assert float((with_sink[200:] - near_only[200:]).abs().max()) > 0.2 * float(with_sink.abs().max())
    model = make_model(cfg, store, dtype)
    for cuts in ([T], [1, 1, 1, 61, 1, 1, 62, 2, 200], [256] + [1] * 74):
        close(run_in_portions(model, tokens, cuts), ref, dtype, cuts)


def test_long_decoding_keeps_the_recurrent_state():
    """300 tokens decoded one by one after a prompt of two, in float32: the state of the gated linear
    layers is carried and decays over hundreds of steps (tau 1 and 9 in this configuration)."""
    cfg, store, plain = ts.build("Q")
    model = make_model(cfg, store, torch.float32)
    tokens = tokens_of(cfg, 302, 21)
    ref = ps.forward(cfg.to_dict(), plain, tokens)
    close(run_in_portions(model, tokens, [2] + [1] * 300), ref, torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(dtype):
    """Prompts of unequal lengths in batches of three through ``Engine.generate`` (its scheduler, cache and
    sampler): the tokens are those the plain statement picks greedily, and in bfloat16 every picked token
    is the plain statement's first or close second choice."""
    from supersonic_b200.api import Engine
    cfg, store, plain = ts.build("P")
    model = make_model(cfg, store, dtype, max_tokens=1024, max_seq_tokens=128)
    prompts = [tokens_of(cfg, n, 40 + n) for n in (1, 9, 64, 17, 70)]
    out = Engine(model).generate(prompts, max_new_tokens=10, temperature=0.0, ignore_eos=True, batch_size=3)
    assert [len(o) for o in out] == [10] * len(prompts)
    for prompt, new in zip(prompts, out):
        seq = list(prompt)
        for tok in new:
            logits = ps.forward(cfg.to_dict(), plain, seq)[-1]
            if dtype == torch.float32:
                assert tok == int(logits.argmax())
            else:
                assert float(logits.max() - logits[tok]) < 0.05 * float(logits.std())
            seq.append(tok)
    assert model.cache.slots.n_held == 0


def test_trace_replay_of_a_model_folder(tmp_path):
    """``bin/trace_run`` on a written folder (decay rank left to the tensor's shape): a prompt step, decode
    steps and a second request in the freed slot, logits against the plain statement."""
    import json, os, subprocess, sys
    from supersonic_b200.weights import write_model_folder
    cfg, _, _ = ts.build("P")
    folder = write_model_folder(cfg, 3, str(tmp_path / "m"), std=0.15)
    d = json.load(open(folder + "/config.json"))
    for layer in d["layers"]:
        layer["mixer"].pop("decay_rank", None)
    json.dump(d, open(folder + "/config.json", "w"))
    from supersonic_b200.weights import WeightStore
    st = WeightStore.from_dir(folder)
    plain = {n: st.get(n) for n in st.names()}
    a, b = tokens_of(cfg, 70, 1), tokens_of(cfg, 5, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[66:67], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[67:70], "want": [2]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b, "want": [4]}], "end": ["b"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    ra, rb = ps.forward(d | {"layers": cfg.to_dict()["layers"]}, plain, a), ps.forward(cfg.to_dict(), plain, b)
    want = {0: ra[[0, 65]], 1: ra[[66]], 2: ra[[69]], 3: rb[[4]]}
    for i, ref in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg.vocab)).double()
        close(got, ref, torch.float32, i)
