"""The Girelix decoder in the engine against the plain float64 statement of it (``plain_girelix``).

Small configurations of the tests' own, random weights shaped so that faults show (peaked attention, sinks of the
scores' size, slow decays, routers whose choice is seldom close), and every way of cutting and batching. The same
tests run on a CPU with the plain PyTorch statements of the kernels (host logic: pages, slots, state, the two caches
of one mixer) and, marked ``gpu``, with the compiled kernels in float32 and bfloat16. The kernels are also compared
one by one with their plain statements, and those with the oracle's functions.
"""

import json

import numpy as np
import pytest
import torch

import plain_girelix as plain
import traces

from tiny_girelix import (CLOSE_CALL, CONFIGS, LEFT, LEFT_FULL, LENGTHS, PAGE, RIGHT, RIGHT_SMALL, TOL,
                          layer, make_folder, model, moe, plant, prompts)


def runner_for(folder, dtype, device, page, max_tokens, ops=None, max_requests=4, context=None, **kw):
    from akas_b200.config import EngineConfig
    from akas_b200.engine.runner import ModelRunner

    cfg = EngineConfig(dtype=dtype, device=device, page_size=page, max_tokens=max_tokens, max_requests=max_requests,
                       context=context or max_tokens, cuda_graphs=False, **kw)
    return ModelRunner(folder, cfg, ops=ops)


def oracle(config, w, tokens):
    """(logits [T, vocab], held [T]): ``held`` is False where some layer's routing was a close call, which reduced
    precision may decide the other way (float32 holds every position)."""
    margins = []
    logits = plain.forward(tokens, w, config, margins=margins).numpy()
    held = np.ones(len(tokens), dtype=bool)
    for per_layer in margins:
        held &= np.asarray(per_layer) >= CLOSE_CALL
    return logits, held


def compare(got, want, dtype, what):
    for rid, (logits, held) in want.items():
        rows = np.arange(len(logits)) if dtype == "float32" else np.nonzero(held)[0]
        if dtype != "float32":
            # positions whose routing was clear are held one by one; over all positions, the typical error is held too
            # (a choice that fell the other way is rare and moves one position far: the median does not see it)
            error = np.abs(got[rid] - logits).max(axis=-1) / np.abs(logits).max()
            assert np.median(error) <= 0.5 * TOL[dtype], f"{what}: request {rid}: median error {np.median(error):.3g}"
            if len(rows) == 0:
                continue
        bad = traces.first_bad(got[rid][rows], logits[rows], TOL[dtype])
        assert bad is None, (f"{what}: request {rid} first differs at position {rows[bad]} "
                             f"{traces.worst(got[rid][rows], logits[rows])}")


def run_modes(key, dtype, device, ops, tmp_path, modes):
    config = CONFIGS[key]
    folder, w = make_folder(config, seed=31, folder=tmp_path / key)
    reqs = {f"r{i}": p for i, p in enumerate(prompts(config["vocab"], LENGTHS[key], seed=6))}
    want = {rid: oracle(config, w, toks) for rid, toks in reqs.items()}
    page = PAGE[key]
    longest = -(-max(len(t) for t in reqs.values()) // page) * page
    for mode in modes:
        if mode == "mixed":
            steps, peak = traces.mixed(reqs, {rid: max(1, len(t) - 9) for rid, t in reqs.items()}, seed=3, live=3, page=page)
            runner = runner_for(folder, dtype, device, page, peak, ops, max_requests=3, context=longest)
        else:
            steps = getattr(traces, mode)(reqs)
            runner = runner_for(folder, dtype, device, page, longest, ops, max_requests=2)
        got = traces.replay(runner, steps)
        assert not runner.cache.live() and runner.cache.min_free_pages() == runner.cache.num_pages
        compare(got, want, dtype, f"{key}/{dtype}/{mode}")


MODES = ["whole", "tail_decoded", "portions", "mixed"]


@pytest.mark.parametrize("key", list(CONFIGS))
def test_every_way_of_cutting_on_the_plain_operations(key, tmp_path):
    from akas_b200.ops import reference

    run_modes(key, "float32", "cpu", reference, tmp_path, MODES)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", list(CONFIGS))
def test_every_way_of_cutting_on_the_kernels(key, dtype, tmp_path):
    run_modes(key, dtype, "cuda:0", None, tmp_path, MODES)


def test_config_round_trip_registry_and_inventory(tmp_path):
    from akas_b200.config import ConfigError, GirelixConfig, config_from_dict, load_config
    from akas_b200.engine.runner import kernel_kinds
    from akas_b200.ops import reference
    from akas_b200.weights.loader import WeightError

    config = config_from_dict(CONFIGS["mix"])
    assert isinstance(config, GirelixConfig) and config_from_dict(config.to_dict()) == config
    assert config_from_dict(json.loads(json.dumps(config.to_dict()))) == config
    spec = config.model_spec()
    assert all(l.mixer.kind == "parallel_mixer" and l.arrangement == "parallel" for l in spec.layers)
    assert spec.layers[1].ffn is None and spec.layers[0].ffn.num_identity == 2 and spec.layers[3].ffn.keep_groups == 3
    left, right = (branch for _, branch, _ in spec.layers[1].mixer.branches)
    assert left.values_are_keys and left.sink == "learned" and left.position.rotary == 6 and left.position.interleaved
    assert right.decay == (0.97,) and spec.layers[3].mixer.branches[0][1].position is None
    assert set(kernel_kinds(spec)) == {"attention_general", "rope", "recurrent", "moe"}
    assert set(kernel_kinds(config_from_dict(CONFIGS["bare"]).model_spec())) == {"attention_general", "rope", "recurrent"}
    folder, _ = make_folder(CONFIGS["odd"], seed=1, folder=tmp_path / "m")
    assert load_config(folder) == config_from_dict(CONFIGS["odd"])
    for change, message in ((lambda c: c["layers"][0]["mixer"]["left"].update(vdim=12), "vdim"),
                            (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5]), "decay"),
                            (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
                            (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), "groups"),
                            (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=5), "rot.dims"),
                            (lambda c: c["layers"][0].update(type="serial"), "type")):
        broken = json.loads(json.dumps(CONFIGS["odd"]))
        change(broken)
        with pytest.raises(ConfigError, match=message):
            config_from_dict(broken)
    # a checkpoint without a sink tensor, or with a feed-forward scale for a layer that has no feed-forward, is refused
    from safetensors.torch import load_file, save_file

    tensors = load_file(str(folder / "model.safetensors"))
    del tensors["l0.mix.left.sink"]
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightError, match="l0.mix.left.sink"):
        runner_for(folder, "float32", "cpu", 8, 64, reference)


def one_mechanism(config, tmp_path, seed=5, length=40, **kw):
    """The engine on the plain operations against the oracle for a one-layer model that isolates a mechanism."""
    from akas_b200.ops import reference

    folder, w = make_folder(config, seed=seed, folder=tmp_path / "one", **kw)
    toks = prompts(config["vocab"], [length], seed=seed)[0]
    runner = runner_for(folder, "float32", "cpu", 8, 64, reference)
    got = traces.replay(runner, traces.portions({"a": toks}, sizes=(9, 1, 2, 17)))["a"]
    want = plain.forward(toks, w, config).numpy()
    assert traces.first_bad(got, want, TOL["float32"]) is None, traces.worst(got, want)
    return w, toks, want


def test_sink_attention_alone(tmp_path):
    """Only the left mixer (the right one's scale is 0, no feed-forward): its result must differ from the same model
    without sinks (sinks far below every score) and from one whose values pass the rotation."""
    config = model(48, 70, [layer(LEFT, RIGHT_SMALL, None, left_scale=1.0, right_scale=0.0)])
    w, toks, want = one_mechanism(config, tmp_path)
    no_sink = dict(w, **{"l0.mix.left.sink": torch.full((LEFT["heads"],), -60.0, dtype=torch.float64)})
    assert np.abs(plain.forward(toks, no_sink, config).numpy() - want).max() > 1e-2 * np.abs(want).max()
    h = torch.randn(7, 48, dtype=torch.float64)
    m = dict(LEFT, rot=dict(base=10000.0, dims=0))
    unrotated = plain.sink_attention(h, w, "l0.mix.left.", m)
    assert (unrotated - plain.sink_attention(h, w, "l0.mix.left.", LEFT)).abs().max() > 1e-3  # the rotation matters
    # row 0 sees one key: its output is that key's projection times 1 / (1 + exp(sink - score))
    q = (h[0] @ w["l0.mix.left.q"].T).reshape(LEFT["heads"], LEFT["dim"])
    k = (h[0] @ w["l0.mix.left.k"].T).reshape(LEFT["kv_heads"], LEFT["dim"])
    group = LEFT["heads"] // LEFT["kv_heads"]
    heads = []
    for a in range(LEFT["heads"]):
        score = (q[a] @ k[a // group]) * LEFT["scale"]
        heads.append(k[a // group] / (1.0 + torch.exp(w["l0.mix.left.sink"][a] - score)))
    assert torch.allclose(torch.cat(heads) @ w["l0.mix.left.o"].T, unrotated[0], atol=1e-10)


def test_decayed_linear_attention_alone(tmp_path):
    config = model(56, 70, [layer(LEFT_FULL, RIGHT, None, left_scale=0.0, right_scale=1.0)])
    w, toks, want = one_mechanism(config, tmp_path)
    # the recurrence against its closed form: o_t = sum_{s <= t} decay^(t - s) (q_t . k_s) v_s
    h = torch.randn(9, 56, dtype=torch.float64)
    p = "l0.mix.right."
    y, state = plain.decayed_linear_attention(h, w, p, RIGHT, 1e-5)
    H, D, V = RIGHT["heads"], RIGHT["dim"], RIGHT["vdim"]
    q, k, v = (plain.silu(h @ w[p + n].T).reshape(9, H, -1) for n in ("q", "k", "v"))
    o = torch.zeros(9, H, V, dtype=torch.float64)
    for t in range(9):
        for s in range(t + 1):
            for a in range(H):
                o[t, a] += RIGHT["decay"][a] ** (t - s) * (q[t, a] @ k[s, a]) * v[s, a]
    closed = plain.rms(o.reshape(9, H * V), 1e-5) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    assert torch.allclose(closed @ w[p + "o"].T, y, atol=1e-9)
    # a state carried from a first half gives the second half's results
    first, mid = plain.decayed_linear_attention(h[:4], w, p, RIGHT, 1e-5)
    second, end = plain.decayed_linear_attention(h[4:], w, p, RIGHT, 1e-5, state=mid)
    assert torch.allclose(torch.cat([first, second]), y, atol=1e-9) and torch.allclose(end, state, atol=1e-12)


def test_routed_experts_alone(tmp_path):
    config = model(40, 70, [layer(LEFT_FULL, RIGHT_SMALL, moe(9, 3, 3, 4, 2, 28), left_scale=0.0, right_scale=0.0)])
    one_mechanism(config, tmp_path)


def test_routing_follows_the_rules():
    """The plain statement of the router (what the kernels are held to) against hand-made cases."""
    from akas_b200.ops import reference

    r = dict(experts=4, identity=2, top=2, groups=dict(count=3, keep=2))
    w = {"router": None, "correction": torch.zeros(6, dtype=torch.float64)}
    h = torch.tensor([[3.0, 0.0, 0.1, 0.05, 2.5, 2.0],    # groups (0,1) (2,3) (4,5): best groups 0 and 2
                      [0.2, 0.0, 1.0, 0.9, 0.8, 0.1]], dtype=torch.float64)
    w["router"] = torch.eye(6, dtype=torch.float64)
    chosen, weights = plain.route(h, w, "", r)
    assert chosen.tolist() == [[0, 4], [2, 3]]
    s = torch.softmax(h, dim=-1)
    assert torch.allclose(weights[0], s[0, [0, 4]] / s[0, [0, 4]].sum())
    # a correction changes the choice but not the weights' source; a negative choice score still beats a dropped group
    w["correction"] = torch.tensor([-5.0, -5.2, 0.0, 0.0, -5.1, -9.0], dtype=torch.float64)
    chosen, weights = plain.route(h[:1], w, "", dict(r, groups=dict(count=3, keep=1)))
    assert chosen.tolist() == [[2, 3]]
    w["correction"] = torch.tensor([0.0, 0.0, -5.0, -5.0, -4.0, -4.5], dtype=torch.float64)
    chosen, weights = plain.route(h[1:], w, "", r)
    assert chosen.tolist() == [[0, 1]] and torch.allclose(weights[0], s[1, [0, 1]] / s[1, [0, 1]].sum())
    # the operations' statement agrees with the oracle's on random inputs of several shapes
    g = torch.Generator().manual_seed(3)
    for outputs, count, keep, top in ((12, 4, 2, 3), (9, 3, 3, 4), (8, 1, 1, 8), (10, 5, 1, 2), (7, 7, 3, 3)):
        hh = torch.randn(50, 16, generator=g, dtype=torch.float64)
        ww = {"router": torch.randn(outputs, 16, generator=g, dtype=torch.float64),
              "correction": torch.randn(outputs, generator=g, dtype=torch.float64) * 0.2}
        want_c, want_w = plain.route(hh, ww, "", dict(experts=outputs, identity=0, top=top, groups=dict(count=count, keep=keep)))
        got_c, got_w = reference.moe_route(hh.float(), ww["router"].float(), ww["correction"].float(), count, keep, top)
        assert got_c.tolist() == want_c.tolist() and torch.allclose(got_w.double(), want_w, atol=1e-5)


# --------------------------------------------------------------------------- what a position sees


def seen_case(device, dtype, ops, tmp_path, decode):
    """Only the left mixer: the logits at position i change with the token at position j iff j <= i, for keys far
    back, at page borders and next to the query, with the query in a prompt's portion or decoded alone."""
    from akas_b200.engine.batch import StepEntry

    config = model(48, 120, [layer(LEFT, RIGHT_SMALL, None, left_scale=1.0, right_scale=0.0)])
    folder, _ = make_folder(config, seed=44, folder=tmp_path / "edge", sharp=False)
    w = plant(folder, config, key_token=119, query_token=118)  # token 119 at position j is felt by token 118 at position i
    base = prompts(118, [300], seed=9)[0]
    i = 290
    base[i] = 118

    def logits_at_i(tokens):
        runner = runner_for(folder, dtype, device, 8, 320, ops)
        if decode:
            runner.step([StepEntry("a", tokens[:i], ())])
            out = runner.step([StepEntry("a", tokens[i:i + 1], (0,))])
        else:
            runner.step([StepEntry("a", tokens[:277], ())])
            out = runner.step([StepEntry("a", tokens[277:], (i - 277,))])
        return out.float().cpu().numpy()[0]

    ref = logits_at_i(base)
    for j, seen in ((0, True), (1, True), (7, True), (8, True), (63, True), (64, True), (255, True), (256, True), (i - 1, True),
                    (i, True), (i + 1, False), (299, False)):
        changed = list(base)
        changed[j] = 119 if j != i else 7
        got = logits_at_i(changed)
        diff = np.abs(got - ref).max()
        if seen:
            assert diff > 2e-2 * np.abs(ref).max(), f"position {i} does not see {j}"
        else:
            assert diff == 0.0, f"position {i} sees {j} (difference {diff})"
        if dtype == "float32" and seen:
            want = plain.forward(changed[: i + 1], w, config)[i].numpy()
            assert np.abs(got - want).max() <= TOL[dtype] * np.abs(want).max()


@pytest.mark.parametrize("decode", [False, True])
def test_what_a_position_sees_on_the_plain_operations(decode, tmp_path):
    from akas_b200.ops import reference

    seen_case("cpu", "float32", reference, tmp_path, decode)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("decode", [False, True])
def test_what_a_position_sees_on_the_kernels(decode, dtype, tmp_path):
    seen_case("cuda:0", dtype, None, tmp_path, decode)


def far_key_case(device, dtype, ops, tmp_path):
    """One key far back among hundreds is made to stand out (its key and the last token's queries are long along a
    channel that the rotation leaves alone): the last position's attention must find it through scattered pages, in
    a portion and decoded alone."""
    from akas_b200.engine.batch import StepEntry

    config = model(48, 120, [layer(LEFT, RIGHT_SMALL, None, left_scale=1.0, right_scale=0.0)])
    folder, _ = make_folder(config, seed=47, folder=tmp_path / "far", sharp=False)
    w = plant(folder, config, key_token=119, query_token=118)
    toks = prompts(118, [500], seed=2)[0]
    toks[3], toks[-1] = 119, 118  # the key appears once, far back; the query is the last token
    want = plain.forward(toks, w, config)[-1].numpy()
    without = list(toks)
    without[3] = 5
    felt = np.abs(plain.forward(without, w, config)[-1].numpy() - want).max()
    assert felt > 0.05 * np.abs(want).max(), "the far key does not stand out"
    for cuts in ([500], [499, 1], [130, 70, 2, 290, 8]):
        runner = runner_for(folder, dtype, device, 16, 576, ops, context=512)
        runner.admit("other")  # the request's pages are not the pool's first
        runner.cache.reserve("other", 40)
        at = 0
        for c in cuts:
            out = runner.step([StepEntry("a", toks[at:at + c], (c - 1,) if at + c == 500 else ())])
            at += c
        got = out.float().cpu().numpy()[0]
        assert np.abs(got - want).max() <= TOL[dtype] * np.abs(want).max(), cuts


def test_a_far_key_is_found_on_the_plain_operations(tmp_path):
    from akas_b200.ops import reference

    far_key_case("cpu", "float32", reference, tmp_path)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_is_found_on_the_kernels(dtype, tmp_path):
    far_key_case("cuda:0", dtype, None, tmp_path)


def far_state_case(device, dtype, ops, tmp_path):
    """Only the right mixer, decays close to one: changing the first token of a long prompt changes the logits
    hundreds of tokens later, in the engine as in the plain model, across portions that end inside the scan's chunks."""
    from akas_b200.engine.batch import StepEntry

    slow = dict(RIGHT, decay=[0.999, 1.0, 0.9995])
    config = model(56, 90, [layer(LEFT_FULL, slow, None, left_scale=0.0, right_scale=1.0)])
    folder, w = make_folder(config, seed=52, folder=tmp_path / "far")
    toks = prompts(config["vocab"], [300], seed=4)[0]
    other = [(toks[0] + 5) % config["vocab"]] + toks[1:]
    out = []
    for t in (toks, other):
        runner = runner_for(folder, dtype, device, 64, 320, ops)
        for a in range(0, 299, 23):
            runner.step([StepEntry("a", t[a:min(a + 23, 299)], ())])
        out.append(runner.step([StepEntry("a", t[299:], (0,))]).float().cpu().numpy()[0])
    want = [plain.forward(t, w, config)[-1].numpy() for t in (toks, other)]
    felt = np.abs(want[0] - want[1]).max()
    assert felt > 1e-3 * np.abs(want[0]).max(), "the weights hide the far token"
    for got, ref in zip(out, want):
        assert np.abs(got - ref).max() <= TOL[dtype] * np.abs(ref).max()
    if dtype == "float32":
        assert np.abs((out[0] - out[1]) - (want[0] - want[1])).max() <= 0.05 * felt


def test_a_far_token_is_felt_through_the_state_on_the_plain_operations(tmp_path):
    from akas_b200.ops import reference

    far_state_case("cpu", "float32", reference, tmp_path)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_token_is_felt_through_the_state_on_the_kernels(dtype, tmp_path):
    far_state_case("cuda:0", dtype, None, tmp_path)


def test_a_freed_slot_starts_from_zero_and_freed_pages_are_not_read(tmp_path):
    """Two requests one after the other in a pool of one slot and just enough pages: the second gets the first one's
    slot and pages and must compute as if it were alone."""
    from akas_b200.engine.batch import StepEntry
    from akas_b200.ops import reference

    config = CONFIGS["odd"]
    folder, w = make_folder(config, seed=12, folder=tmp_path / "m")
    a, b = prompts(config["vocab"], [30, 26], seed=5)
    runner = runner_for(folder, "float32", "cpu", 8, 32, reference, max_requests=1)
    runner.step([StepEntry("a", a, ())])
    runner.release("a")
    got = runner.step([StepEntry("b", b[:11], ()),])
    got = runner.step([StepEntry("b", b[11:], tuple(range(15)))]).numpy()
    want = plain.forward(b, w, config).numpy()[11:]
    assert traces.first_bad(got, want, TOL["float32"]) is None, traces.worst(got, want)


# --------------------------------------------------------------------------- generation


def _greedy(config, w, prompt, count):
    toks = list(prompt)
    for _ in range(count):
        toks.append(int(plain.forward(toks, w, config)[-1].argmax()))
    return toks[len(prompt):]


def generation_case(device, dtype, ops, tmp_path, graphs):
    from akas_b200 import Engine, EngineConfig

    config = CONFIGS["mix"]
    folder, w = make_folder(config, seed=61, folder=tmp_path / "gen")
    ps = prompts(config["vocab"], [1, 9, 40, 23, 3], seed=8)
    cfg = EngineConfig(dtype=dtype, device=device, page_size=8, max_requests=3, context=128, max_tokens=512, prefill_chunk=13,
                       prefill_requests=2, cuda_graphs=graphs)
    with Engine(str(folder), config=cfg, ops=ops) as engine:
        results = engine.generate(ps, max_tokens=10)
    for prompt, result in zip(ps, results):
        assert result["generated_tokens"] == _greedy(config, w, prompt, 10)


def test_greedy_generation_through_the_scheduler_on_the_plain_operations(tmp_path):
    from akas_b200.ops import reference

    generation_case("cpu", "float32", reference, tmp_path, False)


@pytest.mark.gpu
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_scheduler_on_the_kernels(graphs, tmp_path):
    generation_case("cuda:0", "float32", None, tmp_path, graphs)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, tmp_path):
    """200 decoded tokens for three requests of different lengths through captured graphs, against one whole pass of
    the plain model."""
    from akas_b200 import Engine, EngineConfig, StepEntry

    config = CONFIGS["odd"]
    folder, w = make_folder(config, seed=71, folder=tmp_path / "long")
    ps = prompts(config["vocab"], [5, 70, 33], seed=3)
    feed = prompts(config["vocab"], [200, 200, 200], seed=4)
    cfg = EngineConfig(dtype=dtype, device="cuda:0", page_size=8, max_requests=4, context=512, max_tokens=2048)
    with Engine(str(folder), config=cfg) as engine:
        runner = engine.runner
        runner.step([StepEntry(i, p, ()) for i, p in enumerate(ps)])
        rows = [[] for _ in ps]
        for t in range(200):
            logits = runner.step([StepEntry(i, (feed[i][t],), (0,)) for i in range(3)]).float().cpu().numpy()
            for i in range(3):
                rows[i].append(logits[i])
        assert 4 in runner._graphs
    want = {i: oracle(config, w, p + feed[i]) for i, p in enumerate(ps)}
    want = {i: (logits[len(ps[i]):], held[len(ps[i]):]) for i, (logits, held) in want.items()}
    compare({i: np.stack(r) for i, r in enumerate(rows)}, want, dtype, f"long decoding/{dtype}")


# --------------------------------------------------------------------------- the kernels one by one


def _batch(lengths, slots, device):
    cu = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32, device=device)
    seq = torch.repeat_interleave(torch.arange(len(lengths)), torch.tensor(lengths)).to(torch.int32).to(device)
    return cu, seq, torch.tensor(slots, dtype=torch.int32, device=device)


def _close(got, want, tol, what):
    got, want = got.double().cpu(), want.double().cpu()
    err = (got - want).abs().max().item() / max(want.abs().max().item(), 1e-30)
    assert err <= tol, f"{what}: {err:.3g} > {tol}"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,vdim", [(3, 20, 24), (1, 72, 40), (2, 8, 5), (2, 130, 300), (1, 260, 16), (4, 32, 64)])
def test_decay_scan_kernel(heads, dim, vdim, dtype):
    from akas_b200.ops import cuda, reference

    cuda.require(["recurrent"])
    g = torch.Generator().manual_seed(heads * 1000 + dim)
    lengths, slots = [137, 1, 0, 64, 70], [2, 0, -1, 3, 4]  # more than two chunks, one token, none, a chunk exactly, a chunk and a bit
    n = sum(lengths)
    proj = (torch.randn(n, 2 * heads * dim + heads * vdim + 3, generator=g) * 0.7).to(dtype).cuda()
    q, k, v = proj[:, : heads * dim], proj[:, heads * dim : 2 * heads * dim], proj[:, 2 * heads * dim : 2 * heads * dim + heads * vdim]
    decay = torch.rand(heads, generator=g).mul(0.3).add(0.7).cuda()
    decay[0] = 1.0
    state = (torch.randn(5, heads, vdim, dim, generator=g) * 0.3).cuda()
    cu, _, sl = _batch(lengths, slots, "cuda")
    for write, act in ((True, "silu"), (False, "silu"), (True, None)):
        s_ref, s_got = state.clone(), state.clone()
        want = reference.decay_scan(q, k, v, decay, s_ref, cu, sl, heads, dim, vdim, 0.5, activation=act, write=write)
        got = cuda.decay_scan(q, k, v, decay, s_got, cu, sl, heads, dim, vdim, 0.5, activation=act, write=write)
        live = torch.arange(0, n)
        _close(got[live], want[live], 2e-5, "scan o")
        _close(s_got, s_ref, 2e-5, "scan state")
        assert write or torch.equal(s_got, state)
        # the same in chunks (what a step with a long portion runs)
        s_chunk = state.clone()
        got = cuda.decay_scan(q, k, v, decay, s_chunk, cu, sl, heads, dim, vdim, 0.5, activation=act, write=write, longest=max(lengths))
        _close(got[live], want[live], 3e-5, "scan o, in chunks")
        _close(s_chunk, s_ref, 3e-5, "scan state, in chunks")
        assert write or torch.equal(s_chunk, state)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_norm_options_and_scaled_add_kernels(dtype):
    from akas_b200.ops import cuda, reference

    cuda.require(["recurrent", "elementwise"])
    g = torch.Generator().manual_seed(5)
    n = 19
    tol = 1e-5 if dtype == torch.float32 else 8e-3
    for heads, vdim in ((3, 24), (1, 72), (1, 10), (2, 5)):
        o = torch.randn(n, heads * vdim, generator=g).cuda()
        gate = torch.randn(n, 200, generator=g).to(dtype).cuda()[:, 8 : 8 + heads * vdim]
        wn = torch.randn(vdim, generator=g).cuda()
        for act in ("silu", "sigmoid"):
            want = reference.gated_rmsnorm(o, wn, 1e-5, gate, heads, vdim, dtype, gate_activation=act, out_scale=0.8)
            _close(cuda.gated_rmsnorm(o, wn, 1e-5, gate, heads, vdim, dtype, gate_activation=act, out_scale=0.8), want, tol, "norm")
            wide = torch.zeros(n, heads * vdim + 24, dtype=dtype, device="cuda")
            for at in (8, 3):
                view = wide[:, at : at + heads * vdim]
                assert cuda.gated_rmsnorm(o, wn, 1e-5, gate, heads, vdim, dtype, gate_activation=act, out=view, out_scale=0.8) is view
                _close(view, want, tol, "norm into a part of wider rows")
                assert float(wide[:, :at].abs().max()) == 0.0 and float(wide[:, at + heads * vdim :].abs().max()) == 0.0
                wide.zero_()
    for c in (64, 50):
        x, a, b = (torch.randn(n, c, generator=g).cuda() for _ in range(3))
        la, lb = torch.randn(c, generator=g).cuda(), torch.randn(c, generator=g).cuda()
        _close(cuda.scaled_add(x.clone(), a, la, b, lb, 0.7), reference.scaled_add(x.clone(), a, la, b, lb, 0.7), 1e-6, "scaled add")
        _close(cuda.scaled_add(x.clone(), a, la, None, None, 1.3), reference.scaled_add(x.clone(), a, la, None, None, 1.3), 1e-6, "one addend")
        _close(cuda.scaled_add(x.clone(), a, None, None, None, 1.0), x + a, 1e-6, "plain add")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("outputs,experts,count,keep,top,c,f", [(12, 10, 4, 2, 3, 80, 48), (9, 6, 3, 3, 4, 52, 20), (8, 8, 1, 1, 8, 64, 64),
                                                              (70, 64, 5, 2, 6, 1100, 24), (4, 3, 1, 1, 1, 24, 8)])
def test_routed_experts_kernels(outputs, experts, count, keep, top, c, f, dtype):
    from akas_b200.ops import cuda, reference

    cuda.require(["moe"])
    g = torch.Generator().manual_seed(outputs * 100 + c)
    n = 45
    h = torch.randn(n, c + 8, generator=g).to(dtype).cuda()[:, :c]
    w_router = (torch.randn(outputs, c, generator=g) * (3.0 / c ** 0.5)).cuda()
    correction = (torch.randn(outputs, generator=g) * 0.2).cuda()
    want_c, want_w = reference.moe_route(h, w_router, correction, count, keep, top)
    got_c, got_w = cuda.moe_route(h, w_router, correction, count, keep, top)
    # a choice may differ where two choice scores are within rounding of each other: such rows are left out
    same = (got_c == want_c).all(dim=1)
    assert same.float().mean() > 0.9
    _close(got_w[same], want_w[same], 1e-4, "weights")
    w_gate_up = (torch.randn(experts, 2 * f, c, generator=g) * c ** -0.5).to(dtype).cuda()
    w_down = (torch.randn(experts, c, f, generator=g) * f ** -0.5).to(dtype).cuda()
    want = reference.moe_experts(h, w_gate_up, w_down, want_c, want_w)
    got = cuda.moe_experts(h, w_gate_up, w_down, want_c, want_w)  # 45 tokens: the grouped product in bfloat16 where it takes the sizes
    _close(got, want, 2e-5 if dtype == torch.float32 else 1e-2, "experts")
    # the residual update by the experts' last kernel against the plain sequence
    x0, a0 = torch.randn(n, c, generator=g).cuda(), torch.randn(n, c, generator=g).cuda()
    la, lb = torch.randn(c, generator=g).cuda(), torch.randn(c, generator=g).cuda()
    for rows in (n, 5):
        upd = cuda.moe_experts(h[:rows], w_gate_up, w_down, want_c[:rows], want_w[:rows], update=(x0[:rows].clone(), a0[:rows], la, lb, 0.7))
        _close(upd, reference.scaled_add(x0[:rows].clone(), a0[:rows], la, want[:rows], lb, 0.7), 2e-5 if dtype == torch.float32 else 1e-2, "update")
    few = cuda.moe_experts(h[:5], w_gate_up, w_down, want_c[:5], want_w[:5])  # few pairs: token by token
    _close(few, want[:5], 2e-5 if dtype == torch.float32 else 1e-2, "experts, few tokens")
    if dtype == torch.bfloat16:
        assert cuda.moe_grouped_status() == 0
        # hundreds of tokens, so that experts get several tiles of rows and some get none; and the result of a token
        # must not depend on what else the step holds
        hh = torch.randn(700, c, generator=g).to(dtype).cuda()
        cc, ww = cuda.moe_route(hh, w_router, correction, count, keep, top)
        cc[:300] = cc[0]  # crowd one choice
        big = cuda.moe_experts(hh, w_gate_up, w_down, cc, ww)
        _close(big, reference.moe_experts(hh, w_gate_up, w_down, cc, ww), 1e-2, "experts, many tokens")
        part = cuda.moe_experts(hh[100:420], w_gate_up, w_down, cc[100:420], ww[100:420])
        if c % 8 == 0 and f % 8 == 0:
            assert torch.equal(part, big[100:420]), "a token's experts depend on the batch"
        assert cuda.moe_grouped_status() == 0
    # exact ties go to the lower index, and the groups' rule holds on made-up scores
    eye_h = torch.zeros(3, outputs, dtype=dtype).cuda()
    tie_c, tie_w = cuda.moe_route(eye_h, torch.eye(outputs).cuda(), torch.zeros(outputs).cuda(), count, keep, top)
    ref_c, _ = reference.moe_route(eye_h, torch.eye(outputs).cuda(), torch.zeros(outputs).cuda(), count, keep, top)
    assert tie_c.tolist() == ref_c.tolist() and tie_c[0].tolist() == list(range(top))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,rot,page", [(6, 2, 24, 16, 8), (4, 4, 16, 16, 16), (3, 1, 20, 6, 4), (36, 2, 8, 0, 64),
                                                        (6, 1, 96, 64, 64), (2, 2, 128, 128, 32)])
def test_sink_attention_kernels(heads, kv_heads, dim, rot, page, dtype):
    """Rotation of neighbouring pairs on a part of the head, values that are the unrotated keys, learned sinks of the
    scores' size, output into a part of wider rows with a scale; prompt portions beside decoded tokens over
    scattered pages."""
    from types import SimpleNamespace

    from akas_b200.ops import cuda, reference

    cuda.require(["attention_general", "rope"])
    g = torch.Generator().manual_seed(heads + dim)
    starts, lengths = [150, 0, 77, 301], [1, 45, 30, 1]
    blocks = -(-400 // page)
    table = torch.randperm(4 * blocks, generator=g).to(torch.int32).view(4, blocks).cuda()
    k_pool = torch.randn(4 * blocks, kv_heads, page, dim, generator=g).to(dtype).cuda()
    v_pool = torch.randn(4 * blocks, kv_heads, page, dim, generator=g).to(dtype).cuda()
    n = sum(lengths)
    cu, seq, _ = _batch(lengths, [0, 1, 2, 3], "cuda")
    pos = torch.cat([torch.arange(s, s + l) for s, l in zip(starts, lengths)]).to(torch.int32).cuda()
    proj = torch.randn(n, heads * dim + kv_heads * dim + 16, generator=g).to(dtype).cuda()
    proj[:, : heads * dim] *= 2.0
    q, k = proj[:, : heads * dim], proj[:, heads * dim : (heads + kv_heads) * dim]
    rotary = {}
    if rot:
        inv_freq = (torch.tensor(10000.0, dtype=torch.float64) ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).cuda()
        cos, sin = cuda.rope_tables(pos, inv_freq)
        angle = pos.double()[:, None] * inv_freq[None, :]
        _close(cos, torch.cos(angle), 1e-6, "cos")
        rotary = dict(cos=cos, sin=sin, interleaved=True)
    pools = [(k_pool.clone(), v_pool.clone()) for _ in range(2)]
    qn = [ops.qk_norm_store(q, k, k, heads, kv_heads, dim, dim, None, None, 0.0, kp, vp, table, seq, pos, page, **rotary)
          for ops, (kp, vp) in zip((reference, cuda), pools)]
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    _close(qn[1], qn[0], tol, "rotated q")
    _close(pools[1][0], pools[0][0], tol, "k pages")
    assert torch.equal(pools[1][1], pools[0][1])
    if rot:
        # the plain statement of the rotation agrees with the oracle's, and the values stayed unrotated
        want_q = plain.rotate_pairs(q[1:46].double().cpu().reshape(45, heads, dim), rot, 10000.0).reshape(45, -1)
        _close(qn[0][1:46], want_q, tol, "rotation against the oracle")
        page_of = table[1, 44 // page].item()
        assert torch.equal(pools[1][1][page_of, :, 44 % page].reshape(-1), k[45])
    sinks = (torch.randn(heads, generator=g) * 2.0).cuda()
    # (the largest context lets the decoding request at the step's front have its keys cut into parts)
    ctx = SimpleNamespace(query_lens=tuple(lengths), decode_only=False, cu_seqlens=cu, max_context=400)
    want = reference.attention_general(qn[0], *pools[0], table, seq, pos, 0.3, None, 0, 0.0, None, None, False, None, page,
                                       sinks=sinks, out_scale=1.2)
    none = reference.attention_general(qn[0], *pools[0], table, seq, pos, 0.3, None, 0, 0.0, None, None, False, None, page)
    assert (want - none * 1.2).abs().max() > 0.05, "the sinks do not matter"
    for layout in (None, ctx):
        wide = torch.zeros(n, heads * dim + 16, dtype=dtype, device="cuda")
        view = wide[:, 8 : 8 + heads * dim]
        got = cuda.attention_general(qn[0], *pools[0], table, seq, pos, 0.3, None, 0, 0.0, None, None, False, None, page, layout,
                                     sinks=sinks, out=view, out_scale=1.2)
        assert got is view and float(wide[:, :8].abs().max()) == 0.0 and float(wide[:, 8 + heads * dim :].abs().max()) == 0.0
        _close(view, want, 2e-5 if dtype == torch.float32 else 1.5e-2, f"attention with sinks {layout is None}")
    # a step of single tokens with long pasts: keys in parts, merged; against the same step without parts
    singles = [399, 130, 64, 257]
    pos1 = torch.tensor(singles, dtype=torch.int32).cuda()
    cu1, seq1, _ = _batch([1, 1, 1, 1], [0, 1, 2, 3], "cuda")
    q1 = qn[0][:4].contiguous()
    want1 = reference.attention_general(q1, *pools[0], table, seq1, pos1, 0.3, None, 0, 0.0, None, None, False, None, page, sinks=sinks)
    for most in (0, 400):
        ctx1 = SimpleNamespace(query_lens=(1, 1, 1, 1), decode_only=True, cu_seqlens=cu1, max_context=most)
        got1 = cuda.attention_general(q1, *pools[0], table, seq1, pos1, 0.3, None, 0, 0.0, None, None, False, None, page, ctx1, sinks=sinks)
        _close(got1, want1, 2e-5 if dtype == torch.float32 else 1.5e-2, f"single tokens, keys in parts: {most > 0}")
