"""The Gigusun decoder in the engine against the plain float64 statement of it (``plain_gigusun``).

Small configurations of the tests' own, random weights shaped so that faults show (peaked attention, slow decays),
and every way of cutting and batching. The same tests run on a CPU with the plain PyTorch statements of the kernels
(host logic: pages kept behind a window, slots, state) and, marked ``gpu``, with the compiled kernels in float32
and bfloat16. The kernels are also compared one by one with their plain statements.
"""

import json
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_gigusun as plain
import traces

from tiny_gigusun import ATT, ATT_KEPT, CONFIGS, DELTA, GLA, LENGTHS, PAGE, TOL, layer, make_folder, prompts


def runner_for(folder, dtype, device, page, max_tokens, ops=None, max_requests=4, context=None, **kw):
    from akas_b200.config import EngineConfig
    from akas_b200.engine.runner import ModelRunner

    cfg = EngineConfig(dtype=dtype, device=device, page_size=page, max_tokens=max_tokens, max_requests=max_requests,
                       context=context or max_tokens, cuda_graphs=False, **kw)
    return ModelRunner(folder, cfg, ops=ops)


def compare(got, want, dtype, what):
    for rid in want:
        bad = traces.first_bad(got[rid], want[rid], TOL[dtype])
        assert bad is None, f"{what}: request {rid} first differs at position {bad} {traces.worst(got[rid], want[rid])}"


def run_modes(key, dtype, device, ops, tmp_path, modes):
    config = CONFIGS[key]
    folder, w = make_folder(config, seed=31, folder=tmp_path / key)
    reqs = {f"r{i}": p for i, p in enumerate(prompts(config["vocab"], LENGTHS[key], seed=6))}
    want = {rid: plain.forward(config, w, toks).numpy() for rid, toks in reqs.items()}
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


def test_config_round_trip_and_registry(tmp_path):
    from akas_b200.config import GigusunConfig, config_from_dict, load_config

    config = config_from_dict(CONFIGS["mix"])
    assert isinstance(config, GigusunConfig) and config_from_dict(config.to_dict()) == config
    spec = config.model_spec()
    assert [l.mixer.kind for l in spec.layers] == ["gated_delta", "attention", "gated_linear_attention", "attention",
                                                  "gated_delta", "gated_linear_attention"]
    assert spec.layers[2].ffn is None and spec.layers[1].mixer.keep_first == 3 and spec.layers[3].mixer.window == 9
    folder, _ = make_folder(CONFIGS["gla"], seed=1, folder=tmp_path / "m")
    assert load_config(folder).layers[0].options.get("rank") is None  # the rank is read from the checkpoint


def _windows(config):
    return [(l["mixer"]["mask"]["size"], l["mixer"]["mask"]["keep_first"]) for l in config["layers"] if l["type"] == "attention"]


def edge_case(device, dtype, ops, tmp_path, decode):
    """One attention layer and no feed-forward: the logits at position i change with the token at position j iff
    i sees j. Checked for j just inside and just outside the window and the kept first tokens, with the query in a
    prompt's portion or decoded alone, across page borders (pages of 8, a window of 20, 3 kept tokens)."""
    from akas_b200.engine.batch import StepEntry

    config = dict(CONFIGS["attention"], layers=[layer("attention", ATT, ff=None)])
    folder, w = make_folder(config, seed=44, folder=tmp_path / "edge")
    size, keep = ATT["mask"]["size"], ATT["mask"]["keep_first"]
    base = prompts(config["vocab"], [60], seed=9)[0]
    i = 57

    def logits_at_i(tokens):
        runner = runner_for(folder, dtype, device, 8, 128, ops)
        if decode:
            runner.step([StepEntry("a", tokens[:i], ())])
            out = runner.step([StepEntry("a", tokens[i:i + 1], (0,))])
        else:
            runner.step([StepEntry("a", tokens[:31], ())])
            out = runner.step([StepEntry("a", tokens[31:], (i - 31,))])
        return out.float().cpu().numpy()[0]

    ref = logits_at_i(base)
    for j, seen in ((i - size + 1, True), (i - size, False), (keep - 1, True), (keep, False), (0, True), (i, True), (i - 1, True)):
        changed = list(base)
        changed[j] = (changed[j] + 17) % config["vocab"]
        diff = np.abs(logits_at_i(changed) - ref).max()
        want = plain.forward(config, w, changed)[i].numpy()
        if seen:
            assert diff > 1e-3, f"position {i} does not see {j}"
        else:
            assert diff == 0.0, f"position {i} sees {j} (difference {diff})"
        if dtype == "float32":
            assert np.abs(logits_at_i(changed) - want).max() <= TOL[dtype] * np.abs(want).max()


@pytest.mark.parametrize("decode", [False, True])
def test_window_and_kept_tokens_edges_on_the_plain_operations(decode, tmp_path):
    from akas_b200.ops import reference

    edge_case("cpu", "float32", reference, tmp_path, decode)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("decode", [False, True])
def test_window_and_kept_tokens_edges_on_the_kernels(decode, dtype, tmp_path):
    edge_case("cuda:0", dtype, None, tmp_path, decode)


def test_pages_behind_the_window_are_given_back_but_not_the_kept_ones(tmp_path):
    from akas_b200.engine.batch import StepEntry
    from akas_b200.ops import reference

    config = dict(CONFIGS["attention"], layers=[layer("attention", ATT_KEPT, ff=None)])  # window 9, 11 kept tokens
    folder, _ = make_folder(config, seed=2, folder=tmp_path / "m")
    runner = runner_for(folder, "float32", "cpu", 4, 64, reference)
    runner.step([StepEntry("a", prompts(config["vocab"], [40], seed=1)[0], ())])
    blocks = runner.cache.blocks("a", 0)
    assert all(b >= 0 for b in blocks[:3]) and all(b < 0 for b in blocks[3:7]) and all(b >= 0 for b in blocks[8:])
    runner.release("a")
    assert runner.cache.min_free_pages() == runner.cache.num_pages


def far_state_case(device, dtype, ops, tmp_path):
    """A token far back must still be felt through the matrix states: with decays close to one, changing the first
    token of a long prompt changes the logits hundreds of tokens later, in the engine as in the plain model."""
    from akas_b200.engine.batch import StepEntry

    config = dict(CONFIGS["gla"], layers=[layer("gla", GLA, ff=None), layer("delta", DELTA, ff=None)])
    folder, w = make_folder(config, seed=52, folder=tmp_path / "far", slow=True)
    toks = prompts(config["vocab"], [300], seed=4)[0]
    other = [(toks[0] + 5) % config["vocab"]] + toks[1:]
    out = []
    for t in (toks, other):
        runner = runner_for(folder, dtype, device, 64, 320, ops)
        for a in range(0, 299, 23):  # portions that end in the middle of the scan's chunks
            runner.step([StepEntry("a", t[a:min(a + 23, 299)], ())])
        out.append(runner.step([StepEntry("a", t[299:], (0,))]).float().cpu().numpy()[0])
    want = [plain.forward(config, w, t)[-1].numpy() for t in (toks, other)]
    felt = np.abs(want[0] - want[1]).max()
    assert felt > 1e-3 * np.abs(want[0]).max(), "the weights hide the far token"
    for got, ref in zip(out, want):
        assert np.abs(got - ref).max() <= TOL[dtype] * np.abs(ref).max()
    if dtype == "float32":
        assert np.abs((out[0] - out[1]) - (want[0] - want[1])).max() <= 0.05 * felt


def test_a_far_token_is_felt_through_the_states_on_the_plain_operations(tmp_path):
    from akas_b200.ops import reference

    far_state_case("cpu", "float32", reference, tmp_path)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_token_is_felt_through_the_states_on_the_kernels(dtype, tmp_path):
    far_state_case("cuda:0", dtype, None, tmp_path)


def _greedy(config, w, prompt, count):
    toks = list(prompt)
    for _ in range(count):
        toks.append(int(plain.forward(config, w, toks)[-1].argmax()))
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
    """260 decoded tokens for three requests of different lengths through captured graphs (the window passes over
    decoded tokens, pages behind it are given back), against one whole pass of the plain model."""
    from akas_b200 import Engine, EngineConfig, StepEntry

    config = CONFIGS["mix"]
    folder, w = make_folder(config, seed=71, folder=tmp_path / "long")
    ps = prompts(config["vocab"], [5, 70, 33], seed=3)
    feed = prompts(config["vocab"], [260, 260, 260], seed=4)
    cfg = EngineConfig(dtype=dtype, device="cuda:0", page_size=8, max_requests=4, context=512, max_tokens=2048)
    with Engine(str(folder), config=cfg) as engine:
        runner = engine.runner
        runner.step([StepEntry(i, p, ()) for i, p in enumerate(ps)])
        rows = [[] for _ in ps]
        for t in range(260):
            logits = runner.step([StepEntry(i, (feed[i][t],), (0,)) for i in range(3)]).float().cpu().numpy()
            for i in range(3):
                rows[i].append(logits[i])
        assert 4 in runner._graphs
    for i, p in enumerate(ps):
        want = plain.forward(config, w, p + feed[i]).numpy()[len(p):]
        bad = traces.first_bad(np.stack(rows[i]), want, TOL[dtype])
        assert bad is None, (i, bad, traces.worst(np.stack(rows[i]), want))


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
@pytest.mark.parametrize("heads,dim,vdim", [(3, 20, 24), (2, 72, 136), (1, 8, 5), (2, 130, 300), (1, 260, 16), (1, 520, 40)])
def test_gla_scan_kernel(heads, dim, vdim, dtype):
    from akas_b200.ops import cuda, reference

    cuda.require(["recurrent"])
    g = torch.Generator().manual_seed(heads * 1000 + dim)
    lengths, slots = [37, 1, 0, 18], [2, 0, -1, 3]
    n = sum(lengths)
    proj = (torch.randn(n, 2 * heads * dim + heads * vdim + 3, generator=g) * 0.5).to(dtype).cuda()
    q, k, v = proj[:, : heads * dim], proj[:, heads * dim : 2 * heads * dim], proj[:, 2 * heads * dim : 2 * heads * dim + heads * vdim]
    alpha = torch.rand(n, heads * dim, generator=g).mul(0.2).add(0.8).cuda()
    state = (torch.randn(5, heads, vdim, dim, generator=g) * 0.3).cuda()
    cu, _, sl = _batch(lengths, slots, "cuda")
    for write in (True, False):
        s_ref, s_got = state.clone(), state.clone()
        want = reference.gla_scan(q, k, v, alpha, s_ref, cu, sl, heads, dim, vdim, dim ** -0.5, write=write)
        got = cuda.gla_scan(q, k, v, alpha, s_got, cu, sl, heads, dim, vdim, dim ** -0.5, write=write)
        live = torch.cat([torch.arange(0, 38), torch.arange(38, 56)])
        _close(got[live], want[live], 2e-5, "gla o")
        _close(s_got, s_ref, 2e-5, "gla state")
        assert write or torch.equal(s_got, state)


@pytest.mark.gpu
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 4, 16, 12), (6, 2, 40, 20), (2, 1, 136, 72), (1, 1, 7, 3), (2, 2, 300, 33)])
def test_delta_scan_kernel(heads, kv_heads, dim, vdim):
    from akas_b200.ops import cuda, reference

    cuda.require(["recurrent"])
    g = torch.Generator().manual_seed(heads * 1000 + dim)
    lengths, slots = [29, 0, 1, 50], [1, -1, 0, 2]
    n = sum(lengths)
    y = torch.randn(n, 2 * kv_heads * dim + heads * vdim, generator=g).cuda()
    b, a = torch.randn(n, heads, generator=g).cuda(), torch.randn(n, heads, generator=g).cuda()
    a_log, dt = (torch.randn(heads, generator=g) - 2).cuda(), torch.randn(heads, generator=g).cuda()
    y_ref = y.clone()
    beta_ref, g_ref = reference.delta_prep(y_ref, kv_heads, dim, dim ** -0.5, 1e-6, b, a, a_log, dt)
    beta, gg = cuda.delta_prep(y, kv_heads, dim, dim ** -0.5, 1e-6, b, a, a_log, dt)
    _close(y, y_ref, 1e-5, "unit q, k")
    _close(beta, beta_ref, 1e-5, "beta")
    _close(gg, g_ref, 1e-5, "g")
    gd = kv_heads * dim
    row = heads * vdim * dim + 5  # a state that is part of a wider row per slot
    wide = (torch.randn(3, -(-row // 4) * 4, generator=g) * 0.3).cuda()
    for write in (True, False):
        w_ref, w_got = wide.clone(), wide.clone()
        cu, _, sl = _batch(lengths, slots, "cuda")
        view = lambda t: t[:, : heads * vdim * dim].view(3, heads, vdim, dim)
        want = reference.delta_scan(y_ref[:, :gd], y_ref[:, gd : 2 * gd], y_ref[:, 2 * gd :], beta_ref, g_ref, view(w_ref), cu, sl,
                                    heads, kv_heads, dim, vdim, write=write)
        got = cuda.delta_scan(y_ref[:, :gd], y_ref[:, gd : 2 * gd], y_ref[:, 2 * gd :], beta_ref, g_ref, view(w_got), cu, sl,
                              heads, kv_heads, dim, vdim, write=write)
        _close(got, want, 3e-5, "delta o")
        _close(w_got, w_ref, 3e-5, "delta state")
        assert write or torch.equal(w_got, wide)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps", [2, 3, 4, 7])
def test_causal_conv_silu_kernel(taps, dtype):
    from akas_b200.ops import cuda, reference

    cuda.require(["recurrent"])
    g = torch.Generator().manual_seed(taps)
    c = 37
    lengths, slots = [1, 2, 9, 0, 5], [3, 0, 1, -1, 2]  # steps shorter than the taps reach into the state
    n = sum(lengths)
    x = torch.randn(n, c + 4, generator=g).to(dtype).cuda()[:, 2 : 2 + c]
    w = torch.randn(c, taps, generator=g).cuda()
    wide = torch.randn(4, (taps - 1) * c + 3, generator=g).cuda()
    cu, seq, sl = _batch(lengths, slots, "cuda")
    for write in (True, False):
        s_ref, s_got = wide.clone(), wide.clone()
        view = lambda t: t[:, 3:].view(4, taps - 1, c)
        want = reference.causal_conv_silu(x, w, view(s_ref), cu, seq, sl, write=write)
        got = cuda.causal_conv_silu(x, w, view(s_got), cu, seq, sl, write=write)
        _close(got, want, 1e-5, "conv")
        _close(s_got, s_ref, 1e-6, "conv state")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gates_norms_and_polynorm_kernels(dtype):
    from akas_b200.ops import cuda, reference

    cuda.require(["recurrent", "elementwise"])
    g = torch.Generator().manual_seed(5)
    n = 19
    low = torch.randn(n, 40, generator=g).to(dtype).cuda()[:, 7:18]
    w_up, bias = torch.randn(11, 50, generator=g).cuda(), torch.randn(50, generator=g).cuda()
    _close(cuda.decay_gates(low, w_up, bias, 8.0), reference.decay_gates(low, w_up, bias, 8.0), 1e-5, "decay gates")
    o = torch.randn(n, 3 * 24, generator=g).cuda()
    gate = torch.randn(n, 100, generator=g).to(dtype).cuda()[:, 9:81]
    wn = torch.randn(24, generator=g).cuda()
    tol = 1e-5 if dtype == torch.float32 else 8e-3
    _close(cuda.gated_rmsnorm(o, wn, 1e-5, gate, 3, 24, dtype), reference.gated_rmsnorm(o, wn, 1e-5, gate, 3, 24, dtype), tol, "gated norm")
    z = torch.randn(n, 333, generator=g).cuda() * 3
    coeffs = torch.tensor([0.7, -0.4, 0.2, 0.05]).cuda()
    _close(cuda.polynorm(z, coeffs, 1e-6, dtype), reference.polynorm(z, coeffs, 1e-6, dtype), tol, "polynorm")
    _close(cuda.polynorm(z.to(dtype), coeffs, 1e-6, dtype), reference.polynorm(z.to(dtype), coeffs, 1e-6, dtype), tol, "polynorm")
    h = torch.randn(n, 64, generator=g).cuda()
    table = torch.randn(30, 64, generator=g).to(dtype).cuda()
    idx = torch.randint(0, 30, (n,), generator=g).to(torch.int32).cuda()
    _close(cuda.add_rows(h.clone(), table, idx), reference.add_rows(h.clone(), table, idx), 1e-6, "add rows")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,window,keep,page", [
    (6, 2, 24, 40, 20, 3, 8), (4, 4, 16, 8, 37, 0, 16), (2, 1, 40, 24, 9, 11, 4), (20, 1, 32, 160, 300, 5, 64), (3, 3, 72, 72, 0, 0, 16)])
def test_general_attention_kernels(heads, kv_heads, dim, vdim, window, keep, page, dtype):
    """Prompt portions beside decoded tokens over scattered pages; one key is made to stand out far back (inside the
    kept tokens or the window) so that a lost key shows."""
    from akas_b200.ops import cuda, reference

    cuda.require(["attention_general"])
    g = torch.Generator().manual_seed(heads + dim)
    starts, lengths = [150, 0, 77, 301], [1, 45, 30, 1]  # tokens already cached, tokens of this step
    blocks = -(-400 // page)
    order = torch.randperm(4 * blocks, generator=g).to(torch.int32)
    table = order.view(4, blocks).cuda()
    k_pool = (torch.randn(4 * blocks, kv_heads, page, dim, generator=g)).to(dtype).cuda()
    v_pool = (torch.randn(4 * blocks, kv_heads, page, vdim, generator=g)).to(dtype).cuda()
    n = sum(lengths)
    cu, seq, _ = _batch(lengths, [0, 1, 2, 3], "cuda")
    pos = torch.cat([torch.arange(s, s + l) for s, l in zip(starts, lengths)]).to(torch.int32).cuda()
    width = heads * dim + kv_heads * dim + kv_heads * vdim + heads
    proj = torch.randn(n, width + 2, generator=g).to(dtype).cuda()
    proj[:, : heads * dim] *= 3.0  # peaked scores
    a, b, c = heads * dim, heads * dim + kv_heads * dim, heads * dim + kv_heads * dim + kv_heads * vdim
    q, k, v, gate = proj[:, :a], proj[:, a:b], proj[:, b:c], proj[:, c : c + heads]
    qw, kw = (torch.rand(dim, generator=g) + 0.5).cuda(), (torch.rand(dim, generator=g) + 0.5).cuda()
    r1, r2 = (torch.rand(heads, generator=g) * 0.8).cuda(), (torch.rand(heads, generator=g) + 0.1).cuda()
    pools = [(k_pool.clone(), v_pool.clone()) for _ in range(2)]
    qn = []
    for ops, (kp, vp) in zip((reference, cuda), pools):
        qn.append(ops.qk_norm_store(q, k, v, heads, kv_heads, dim, vdim, qw, kw, 1e-5, kp, vp, table, seq, pos, page))
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    _close(qn[1], qn[0], tol, "normed q")
    _close(pools[1][0], pools[0][0], tol, "k pages")
    assert torch.equal(pools[1][1], pools[0][1])
    from types import SimpleNamespace

    # with the step's layout at hand, bfloat16 portions of sizes it takes go to the tensor-core kernel
    ctx = SimpleNamespace(query_lens=tuple(lengths), decode_only=False, cu_seqlens=cu)
    for sink, cap, bias, gated in ((True, 12.0, True, True), (False, 0.0, False, False), (True, 0.0, False, True)):
        args = (0.3, window, keep, cap, r1 if bias else None, r2 if bias else None, sink, gate if gated else None, page)
        want = reference.attention_general(qn[0], *pools[0], table, seq, pos, *args)
        for layout in (None, ctx):
            got = cuda.attention_general(qn[0], *pools[0], table, seq, pos, *args, layout)
            _close(got, want, 2e-5 if dtype == torch.float32 else 1.5e-2, f"attention sink={sink} cap={cap} bias={bias} {layout is None}")
