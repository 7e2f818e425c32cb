"""Topidra on the GPU against the plain implementation: every mechanism alone, then whole models
in every way a request can be cut, batched and decoded, in 32-bit and in bfloat16."""

import json

import numpy as np
import pytest
import torch

import layover_b200 as lb
import plain_topidra as plain
from conftest import random_prompt, tolerance
from layover_b200 import ops
from layover_b200.cache import CacheManager
from layover_b200.engine.batch import BatchBuilder, StepEntry
from layover_b200.engine.step import StepFunction
from layover_b200.models.runtime import make_runtime
from layover_b200.parts.base import PartSpec, build_part
from layover_b200.parts.norm import Deferred
from replay_helpers import max_live_tokens, mixed, portions, run_trace, tail_decoded, whole
from topidra_configs import CONFIGS, INIT, PAGES

pytestmark = pytest.mark.gpu
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F = torch.float64


def close(got: torch.Tensor, want: torch.Tensor, dtype, what=""):
    bound = tolerance(want.float(), dtype)
    worst = (got.detach().cpu().to(F) - want.to(F)).abs().max().item()
    assert worst <= bound, f"{what}: |diff| {worst:.3e} > {bound:.3e}"


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", list(DTYPES.values()))
@pytest.mark.parametrize("width", [40, 1024, 2500])
def test_residual_norm_adds_a_normed_output_and_the_embedding(dtype, width):
    gen = torch.Generator().manual_seed(width)
    x = torch.randn(9, width, generator=gen) * 3
    delta = (torch.randn(9, width, generator=gen) * 5).to(dtype)
    extra = torch.randn(9, width, generator=gen)
    wd, w = torch.randn(width, generator=gen), torch.randn(width, generator=gen)
    want_x = x.to(F) + plain.rms_norm(delta.to(F), wd.to(F), 1e-5) + extra.to(F)
    want_h = plain.rms_norm(want_x, w.to(F), 1e-6)
    xd = x.cuda()
    out = torch.empty(9, width, dtype=dtype, device="cuda")
    ops.residual_rmsnorm(xd, delta.cuda(), wd.cuda(), 1e-5, extra.cuda(), w.cuda(), 1e-6, out)
    close(xd, want_x, torch.float32, "stream")
    close(out, want_h, dtype, "normed")
    # picked rows: the stream is only read
    xd2, rows = x.cuda(), torch.tensor([7, 2, 2], dtype=torch.int32, device="cuda")
    out2 = torch.empty(3, width, dtype=dtype, device="cuda")
    ops.residual_rmsnorm(xd2, delta.cuda(), wd.cuda(), 1e-5, None, w.cuda(), 1e-6, out2, rows)
    assert torch.equal(xd2.cpu(), x)
    close(out2, plain.rms_norm((x.to(F) + plain.rms_norm(delta.to(F), wd.to(F), 1e-5))[[7, 2, 2]], w.to(F), 1e-6), dtype, "rows")
    # a plain sum without a norm, and the sum alone
    xd3 = x.cuda()
    ops.residual_rmsnorm(xd3, delta.cuda(), None, 0.0, None, None, 0.0, None)
    close(xd3, x.to(F) + delta.to(F), torch.float32, "plain sum")


@pytest.mark.parametrize("dtype", list(DTYPES.values()))
def test_relu_gated_product_and_wide_embedding(dtype):
    gen = torch.Generator().manual_seed(5)
    gu = torch.randn(7, 2 * 24, generator=gen).to(dtype)
    out = torch.empty(7, 24, dtype=dtype, device="cuda")
    ops.gated_act(gu.cuda(), out, "relu")
    close(out, torch.relu(gu[:, :24].to(F)) * gu[:, 24:].to(F), dtype)
    table = torch.randn(30, 20, generator=gen).to(dtype)
    ids = torch.tensor([3, 29, 0, 3], dtype=torch.int32)
    x = torch.empty(4, 20, dtype=torch.float32, device="cuda")
    ops.embed(ids.cuda(), table.cuda(), x)
    assert torch.equal(x.cpu(), table.float()[ids.long()])


def mixer_harness(spec: PartSpec, tensors: dict, dtype, page_tokens=4, pages=64, slots=3):
    """One mixer part alone with its own cache manager and batch builder."""
    runtime = make_runtime(dtype, "cuda")
    part = build_part("mixer", spec, "")
    from layover_b200.csrc import build
    build.ensure_built(part.kernel_libraries(dtype) + runtime.kernel_libraries)
    part.bind({k: v.to(dtype if v.dim() == 2 else torch.float32).cuda().contiguous() for k, v in tensors.items()}, runtime)
    cache = CacheManager([(0, part.cache_need(), None)], pages, page_tokens, dtype, "cuda", slots, ops.RECORD_WORDS)
    builder = BatchBuilder(cache, torch.device("cuda"), part.tile_sizes(dtype))

    def step(entries: list[tuple]):          # [(sequence, rows of h)] -> the mixer's output rows, per entry
        made = [StepEntry(seq, [0] * rows.shape[0], []) for seq, rows in entries]
        for entry in made:
            cache.grow(entry.seq, entry.seq.num_tokens + len(entry.tokens))
        batch = builder.build(made)
        out = part.forward(torch.cat([rows for _, rows in entries]).to(dtype).cuda().contiguous(), batch, cache.view(0))
        for entry in made:
            cache.commit(entry.seq, entry.seq.num_tokens + len(entry.tokens))
        return torch.split(out.float().cpu(), [rows.shape[0] for _, rows in entries])
    return part, cache, step


def run_cuts(cache, step, rows: torch.Tensor, cuts: list[int]) -> torch.Tensor:
    seq, at, out = cache.open(f"s{cache._slots.num_used}-{len(cuts)}"), 0, []
    for count in cuts:
        out.append(step([(seq, rows[at:at + count])])[0])
        at += count
    assert at == rows.shape[0]
    cache.close(seq)
    return torch.cat(out)


def identity_attention(heads, kv, d, e, window, scale):
    """A sink attention part whose projections are identities: a row of h IS [q | k | v | gate logits]."""
    sizes = [heads * d, kv * d, kv * e, heads]
    hidden = sum(sizes)
    eye = torch.eye(hidden)
    q, k, v, g = torch.split(eye, sizes)
    o = torch.zeros(hidden, heads * e)
    o[: heads * e] = torch.eye(heads * e)
    spec = PartSpec("attention", dict(hidden=hidden, q_heads=heads, kv_heads=kv, head_dim=d, v_head_dim=e, scale=scale,
                                      window=window, position=None, qk_norm_eps=None, q="q", k="k", v="v", o="o",
                                      sink="sink", gate="g"))
    return spec, {"q": q, "k": k, "v": v, "g": g, "o": o}, sizes


def plain_identity_attention(rows, sizes, heads, kv, d, e, sink, scale, window):
    q, k, v, g = torch.split(rows.to(F), sizes, dim=1)
    n = rows.shape[0]
    o = plain.sink_softmax_attention(q.view(n, heads, d), k.view(n, kv, d), v.view(n, kv, e), sink.to(F), scale, window)
    return (o * torch.sigmoid(g)[:, :, None]).reshape(n, heads * e)


@pytest.mark.parametrize("dtype", list(DTYPES.values()))
@pytest.mark.parametrize("heads,kv,d,e,window", [(4, 2, 16, 8, 12), (2, 2, 8, 20, 5), (3, 1, 12, 12, 64),
                                                 # multiples of 16: the tensor-core kernels in bfloat16
                                                 (4, 2, 32, 16, 12), (2, 1, 16, 48, 9), (8, 2, 64, 64, 30), (3, 3, 128, 128, 17),
                                                 (2, 1, 160, 256, 20), (2, 2, 144, 144, 6)])
def test_sink_attention_sees_exactly_its_window(dtype, heads, kv, d, e, window):
    """One key gets a score far above all others: the newest the window still holds, the first it
    has dropped, keys at page borders, the very first key; as a prompt and with the query decoded."""
    scale, page, n = 0.3, 4, 41
    spec, tensors, sizes = identity_attention(heads, kv, d, e, window, scale)
    gen = torch.Generator().manual_seed(heads * 100 + window)
    sink = torch.randn(heads, generator=gen)
    part, cache, step = mixer_harness(spec, {**tensors, "sink": sink}, dtype, page_tokens=page)
    query = n - 1
    targets = {query - window + 1, query - window, query - window - 1, query, 0, 1,
               (query // page) * page, (query // page) * page - 1, query - window + 2}
    for target in sorted(t for t in targets if 0 <= t <= query):
        rows = torch.randn(n, sum(sizes), generator=gen) * 0.5
        direction = torch.zeros(d)
        direction[target % d] = 6.0
        for h in range(heads):                        # every head's query points at the target's key
            rows[query, h * d:(h + 1) * d] = direction
        for g in range(kv):
            rows[target, sizes[0] + g * d: sizes[0] + (g + 1) * d] = direction
        rows = rows.to(dtype).float()
        want = plain_identity_attention(rows, sizes, heads, kv, d, e, sink, scale, window)
        for cuts in ([n], [n - 1, 1], [n - 9] + [1] * 9, [3, 2, n - 5]):
            got = run_cuts(cache, step, rows, cuts)[:, : heads * e]
            close(got, want, dtype, f"target {target}, cuts {cuts[:3]}")
    cache.check()


@pytest.mark.parametrize("dtype", list(DTYPES.values()))
def test_the_sink_only_enlarges_the_denominator(dtype):
    heads, kv, d, e, window, scale = 2, 1, 8, 8, 6, 0.4
    spec, tensors, sizes = identity_attention(heads, kv, d, e, window, scale)
    gen = torch.Generator().manual_seed(3)
    rows = (torch.randn(15, sum(sizes), generator=gen)).to(dtype).float()
    outs = {}
    for name, sink in (("huge", torch.tensor([9.0, -30.0])), ("none", torch.tensor([-30.0, -30.0]))):
        part, cache, step = mixer_harness(spec, {**tensors, "sink": sink}, dtype)
        outs[name] = run_cuts(cache, step, rows, [15])[:, : heads * e]
        close(outs[name], plain_identity_attention(rows, sizes, heads, kv, d, e, sink, scale, window), dtype, name)
    # head 0 is damped by its sink, head 1 (sink far below every score) is not touched
    assert outs["huge"][:, :e].abs().max() < 0.2 * outs["none"][:, :e].abs().max()
    close(outs["huge"][:, e:], outs["none"][:, e:].to(F), dtype)


def identity_linear(heads, d, e, decay):
    sizes = [heads * d, heads * d, heads * e, heads * e]
    hidden = sum(sizes)
    q, k, v, g = torch.split(torch.eye(hidden), sizes)
    o = torch.zeros(hidden, heads * e)
    o[: heads * e] = torch.eye(heads * e)
    spec = PartSpec("decay_linear_attention", dict(hidden=hidden, heads=heads, head_dim=d, v_head_dim=e, decay=decay,
                                                   norm_eps=1e-6, activation="silu", q="q", k="k", v="v", gate="g", o="o",
                                                   norm="norm"))
    return spec, {"q": q, "k": k, "v": v, "g": g, "o": o}, sizes


@pytest.mark.parametrize("dtype", list(DTYPES.values()))
@pytest.mark.parametrize("heads,d,e,decay", [(2, 16, 8, [0.998, 0.6]), (1, 40, 36, 0.98), (3, 4, 70, [1.0, 0.5, 0.9]),
                                             (2, 128, 64, [0.99, 0.0]), (1, 200, 40, 0.95)])
def test_decay_scan_carries_its_state_across_any_cut(dtype, heads, d, e, decay):
    """A key hundreds of tokens back still decides the output under a slow decay; the same rows as a
    prompt, in portions down to two tokens and decoded one by one, beside another request."""
    spec, tensors, sizes = identity_linear(heads, d, e, decay)
    gen = torch.Generator().manual_seed(d)
    norm = 1 + 0.3 * torch.randn(heads * e, generator=gen)
    part, cache, step = mixer_harness(spec, {**tensors, "norm": norm}, dtype)
    n = 300
    rows = torch.randn(n, sum(sizes), generator=gen)
    rows[2, heads * d: 2 * heads * d] = 8.0          # a far key ...
    rows[n - 1, : heads * d] = 8.0                   # ... that the last query asks for
    rows = rows.to(dtype).float()
    mixer = {"heads": heads, "dim": d, "vdim": e, "decay": decay}
    names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o"}
    want = plain.lightning_mixer(rows.to(F), {**{k: tensors[v].to(F) for k, v in names.items()}, "norm": norm.to(F)},
                                 mixer, 1e-6)[:, : heads * e]
    for cuts in ([n], [n - 40] + [1] * 40, [2, 7, 2, 16, 3, 64, 100, 2, 33, 71], [17, n - 17]):
        close(run_cuts(cache, step, rows, cuts)[:, : heads * e], want, dtype, f"cuts {cuts[:4]}")
    # two requests of unequal length side by side, one in portions, one decoding; slots are used again
    other = (torch.randn(23, sum(sizes), generator=gen)).to(dtype).float()
    want_other = plain.lightning_mixer(other.to(F), {**{k: tensors[v].to(F) for k, v in names.items()}, "norm": norm.to(F)},
                                       mixer, 1e-6)[:, : heads * e]
    a, b = cache.open("a"), cache.open("b")
    got_a, got_b, at = [], [], 0
    for turn in range(23):
        count = min(13, n - at)
        out = step([(a, rows[at:at + count]), (b, other[turn:turn + 1])]) if count else step([(b, other[turn:turn + 1])])
        if count:
            got_a.append(out[0])
        got_b.append(out[-1])
        at += count
    got_a.append(step([(a, rows[at:])])[0])
    close(torch.cat(got_a)[:, : heads * e], want, dtype, "beside another")
    close(torch.cat(got_b)[:, : heads * e], want_other, dtype, "the other")
    if dtype == torch.float32:
        # portions too short for the segmented form take the same steps whatever the cut: the same bits
        again = run_cuts(cache, step, rows, [100, 1, 99, 2, 98])
        assert torch.equal(torch.cat(got_a), again)
        # a whole prompt is cut into segments that run at once: the same sums in another order
        assert ops.scan_segments([n], 4)[1] > 1
        close(run_cuts(cache, step, rows, [n]), again.to(F), torch.float32, "segmented")


# ------------------------------------------------------------------ whole models
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from safetensors.torch import load_file

    out = {}
    for index, (name, raw) in enumerate(CONFIGS.items()):
        folder = tmp_path_factory.mktemp(f"topidra-{name}")
        # seeded by the name, so that a new configuration does not change the others' weights
        lb.write_model_folder(lb.TopidraConfig.from_hf_dict(raw), folder, seed=sum(map(ord, name)), **INIT)
        out[name] = (folder, json.loads((folder / "config.json").read_text()), load_file(str(folder / "model.safetensors")))
    return out


LENGTHS = [1, 9, 70, 130, 33, 300]      # the longest is long enough for the segmented scan when it comes whole
_expected = {}
_moved = {}


def requests_for(name):
    return {f"r{i}": random_prompt(CONFIGS[name]["vocab"], n, seed=7 * len(name) + i) for i, n in enumerate(LENGTHS)}


def expected(folders, name):
    if name not in _expected:
        _, raw, weights = folders[name]
        _expected[name] = {rid: plain.forward(raw, weights, tokens)[0] for rid, tokens in requests_for(name).items()}
    return _expected[name]


def moved_by_rounding(folders, name):
    """Per request: how far rounding what a bfloat16 run stores moves each row of the plain model's logits."""
    if name not in _moved:
        _, raw, weights = folders[name]
        _moved[name] = {rid: plain.forward(raw, weights, tokens, plain.through_bfloat16)[0] - expected(folders, name)[rid]
                        for rid, tokens in requests_for(name).items()}
    return _moved[name]


def compare(rows, want, dtype, moved=None):
    for rid, reference in want.items():
        assert sorted(rows[rid]) == list(range(reference.shape[0])), f"{rid}: rows missing"
        got = torch.from_numpy(np.stack([rows[rid][p] for p in range(reference.shape[0])])).to(F)
        bound = tolerance(reference.float(), dtype)
        if dtype == torch.bfloat16:
            # Norms after every sub-layer pass bfloat16's rounding on from layer run to layer run, so the bound
            # is on a row's root mean square error, 1/16 of the row's own root mean square (a lost state, a
            # window off by one or a missing sink changes a row by about its own size), and four times
            # that for the row's largest error.
            bound = reference.pow(2).mean(dim=1).sqrt() / 16
            if moved is not None:
                # ... unless the row is ill-conditioned in the plain model itself (a first token whose q . k is
                # near zero before a norm that restores the scale): then three times what one rounding of
                # the stored tensors does to the plain model's row
                bound = torch.maximum(bound, 3 * moved[rid].pow(2).mean(dim=1).sqrt())
            worst = torch.maximum((got - reference).pow(2).mean(dim=1).sqrt(), (got - reference).abs().max(dim=1).values / 4)
        else:
            worst = (got - reference).abs().max(dim=1).values
        bad = torch.nonzero(worst > bound)
        assert bad.numel() == 0, f"{rid}: first wrong position {int(bad[0])} of {reference.shape[0]}, {worst[bad[0]].item():.3e}"


CUTS = {"whole": whole, "tail": lambda r: tail_decoded(r, tail=40), "portions": portions, "mixed": mixed}


@pytest.mark.parametrize("dtype_name", list(DTYPES))
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("cut", list(CUTS))
def test_every_cut_matches_the_plain_implementation(folders, tmp_path, name, dtype_name, cut):
    folder = folders[name][0]
    steps = CUTS[cut](requests_for(name))
    if cut == "mixed":      # so few pages and slots that a request which ends hands both to the next one
        assert max_live_tokens(steps) < sum(-(-n // 64) * 64 for n in LENGTHS)
        assert max(len(s["entries"]) for s in steps) == 4
    rows = run_trace(folder, dtype_name, steps, tmp_path, block_tokens=PAGES[name], max_requests=4)
    compare(rows, expected(folders, name), DTYPES[dtype_name],
            moved_by_rounding(folders, name) if dtype_name == "bfloat16" else None)


@pytest.mark.parametrize("name", ["mid_loop", "front_loop"])
def test_the_stream_after_every_layer_run(folders, name):
    folder, raw, weights = folders[name]
    tokens = random_prompt(raw["vocab"], 19, seed=2)
    _, after = plain.forward(raw, weights, tokens)
    model = lb.load_model(folder, dtype="float32")
    cache = lb.PagedKVCache(model, 32, block_tokens=PAGES[name], max_requests=2)
    builder = BatchBuilder(cache, model.device, model.tile_sizes())
    seq = cache.open("s")
    cache.grow(seq, len(tokens))
    taps = []

    def observe(index, x, delta):
        assert isinstance(delta, Deferred) and x.dtype == torch.float32
        taps.append(x.clone().cpu().to(F) + plain.rms_norm(delta.value.cpu().to(F), delta.weight.cpu().to(F), delta.eps))

    model.forward(builder.build([StepEntry(seq, tokens, [0])]), cache, observe=observe)
    assert len(taps) == after.shape[0]
    for run, (got, want) in enumerate(zip(taps, after)):
        close(got, want, torch.float32, f"layer run {run}")


@pytest.mark.parametrize("dtype_name", list(DTYPES))
def test_long_decoding_past_every_window_on_few_pages(folders, tmp_path, dtype_name):
    """Seven tokens of prompt, then 180 decoded one by one: every window passes over decoded tokens,
    pages go back while the request lives, and the pool holds far fewer tokens than the request has."""
    folder, raw, weights = folders["mid_loop"]
    tokens = random_prompt(raw["vocab"], 187, seed=9)
    steps = tail_decoded({"long": tokens}, tail=180)
    rows = run_trace(folder, dtype_name, steps, tmp_path, max_tokens=32, block_tokens=PAGES["mid_loop"], max_requests=1)
    compare(rows, {"long": plain.forward(raw, weights, tokens)[0]}, DTYPES[dtype_name])


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name", ["mid_loop", "linear_only"])
def test_greedy_generation_through_the_engine(folders, name, graphs):
    folder, raw, weights = folders[name]
    model = lb.load_model(folder, dtype="float32")
    prompts = [random_prompt(raw["vocab"], n, seed=n) for n in (3, 21, 40, 8, 1)]
    got = lb.generate(model, prompts, max_new_tokens=12, block_tokens=PAGES[name], cuda_graphs=graphs,
                      config=lb.EngineConfig(max_batch=3, prefill_chunk=16, prefill_budget=16))
    for prompt, tokens in zip(prompts, got):
        sequence = list(prompt)
        for token in tokens:
            logits = plain.forward(raw, weights, sequence)[0][-1]
            top = torch.topk(logits, 2).values
            if top[0] - top[1] > 1e-3 * logits.abs().max():     # a near tie may fall either way
                assert token == int(logits.argmax()), f"position {len(sequence)}"
            sequence.append(token)


def test_command_line_and_the_replay_program(folders, tmp_path):
    import subprocess
    import sys

    from conftest import ROOT

    folder, raw, weights = folders["mid_loop"]
    prompts = ([5, 17, 3, 44, 2, 9, 130], [9])
    out = subprocess.run([sys.executable, "-m", "layover_b200", "--model", str(folder), "--dtype", "fp32",
                          "--prompt-ids", ",".join(map(str, prompts[0])), "--prompt-ids", "9", "--max-new-tokens", "6",
                          "--num-blocks", "32", "--block-tokens", "4", "--max-batch", "2", "--prefill-chunk", "3"],
                         capture_output=True, text=True, cwd=ROOT, check=True)
    result = json.loads(out.stdout.strip().splitlines()[-1])
    for prompt, tokens in zip(prompts, result["generated"]):
        sequence = list(prompt)
        assert len(tokens) == 6
        for token in tokens:
            logits = plain.forward(raw, weights, sequence)[0][-1]
            top = torch.topk(logits, 2).values
            if top[0] - top[1] > 1e-3 * logits.abs().max():
                assert token == int(logits.argmax())
            sequence.append(token)
    out = subprocess.run([sys.executable, "-m", "layover_b200", "--preset", "topidra-tiny", "--random-weights", "--dtype", "bf16",
                          "--prompt-lens", "9,40", "--max-new-tokens", "4", "--num-blocks", "16"],
                         capture_output=True, text=True, cwd=ROOT, check=True)
    assert [len(g) for g in json.loads(out.stdout.strip().splitlines()[-1])["generated"]] == [4, 4]
    # the replay program as a program: five requests through four state slots, one step at a time
    requests = {f"q{i}": random_prompt(raw["vocab"], n, seed=60 + i) for i, n in enumerate([12, 30, 7, 19, 25])}
    steps = mixed(requests, live_limit=4)
    lines = "".join(json.dumps(s) + "\n" for s in steps)
    run = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(tmp_path),
                          "--max-tokens", str(max_live_tokens(steps)), "--block-tokens", "4"],
                         input=lines, capture_output=True, text=True, cwd=ROOT, check=True)
    assert [l for l in run.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    from replay_helpers import collect
    compare(collect(steps, tmp_path), {rid: plain.forward(raw, weights, tokens)[0] for rid, tokens in requests.items()},
            torch.float32)
