"""Zolapel on the device against the plain implementation (``plain_zolapel``): every mechanism
alone, whole prompts against token-by-token decoding, portions down to two tokens, batches of
unequal requests, pages and slots used again, keys at the edges of windows and pages, the first
tokens, long decoding, other sizes, the trace program and greedy generation through the entry
point; then the kernels alone."""
import json
import math
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_zolapel as plain
import replay
import tiny_zolapel as tz

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
_folders: dict = {}
_expected: dict = {}


def folder(tmp_path_factory, name, cfg, dtype):
    key = (name, dtype)
    if key not in _folders:
        path = str(tmp_path_factory.mktemp(f"zolapel_{name}_{dtype}"))
        _folders[key] = tz.write_folder(path, cfg, seed=len(name), storage=DTYPES[dtype])
    return _folders[key]


def prompts(vocab, lengths, seed=0):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


def expected(model_dir, requests, dtype="float32"):
    """float32: the plain model.  bfloat16: the plain model that stores its activations rounded to
    bfloat16 where the engine does, so that what is compared is arithmetic, not the format."""
    out = {}
    stored = None
    for rid, toks in requests.items():
        key = (model_dir, tuple(toks), dtype)
        if key not in _expected:
            stored = stored or tz.read_folder(model_dir)
            rnd = plain.bf16_round if dtype == "bfloat16" else plain.ident
            _expected[key] = plain.forward(toks, stored[1], stored[0], rnd)
        out[rid] = _expected[key]
    return out


def make_runner(model_dir, dtype, max_tokens, page_size=16, eager=True, max_live=4):
    from ginfer_b200.engine.loading import load_model
    from ginfer_b200.engine.runner import ModelRunner
    model, _ = load_model(model_dir, dtype, "cuda:0")
    budget = -(-max_tokens // 64) * 64
    return ModelRunner(model, page_size=page_size, max_num_seqs=max_live, max_seq_len=budget,
                       num_pages=budget // page_size, max_num_batched_tokens=budget,
                       enforce_eager=eager)


def row_errors(rows, want):
    """Per row: rms of the difference (mean taken off) over the rms of the expected logits."""
    worst, where, errs = 0.0, None, []
    for (rid, pos), row in sorted(rows.items()):
        ref = want[rid][pos]
        d = row.astype(np.float64) - ref
        d = d - d.mean()
        e = float(np.sqrt((d * d).mean()) / np.sqrt(((ref - ref.mean()) ** 2).mean()))
        errs.append(e)
        if not e <= worst:
            worst, where = e, (rid, pos)
    return worst, where, float(np.mean(errs)), errs


# float32: differences of summation order.  bfloat16: peaked attention and clear routing amplify
# the format's rounding, and a row whose router scores or gates were close may differ more (at
# most one row in thirty may be off for that); a misplaced page, a window off by one or a lost
# pass of the loop puts most rows near one.
LIMIT = {"float32": (2e-4, 5e-5), "bfloat16": (0.2, 0.03)}
P90 = {"float32": 1e-4, "bfloat16": 0.06}      # nine rows in ten are this close


def check(rows, want, dtype, requests):
    assert len(rows) == sum(len(t) for t in requests.values()), "a logits row is missing"
    worst, where, mean, errs = row_errors(rows, want)
    if dtype == "bfloat16":
        over = sum(e > LIMIT[dtype][0] for e in errs)
        assert over <= len(errs) // 30, f"{over} of {len(errs)} rows are off; worst {where}: {worst:.3e}"
    else:
        assert worst <= LIMIT[dtype][0], f"worst row {where}: relative error {worst:.3e}"
    assert mean <= LIMIT[dtype][1], f"mean relative error {mean:.3e}"
    assert sorted(errs)[int(0.9 * (len(errs) - 1))] <= P90[dtype], "one row in ten is off"


# ----------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("name", ["ATTENTION_ONLY", "ROUTED", "SIDE", "LOOPED"])
def test_each_mechanism_alone(tmp_path_factory, name):
    cfg = getattr(tz, name)
    d = folder(tmp_path_factory, name, cfg, "float32")
    reqs = prompts(cfg["vocab"], [70, 3, 1])
    steps = replay.cut_whole(reqs)
    rows = replay.run_in_process(make_runner(d, "float32", replay.peak_tokens(steps)), steps)
    check(rows, expected(d, reqs), "float32", reqs)


def test_a_lost_mechanism_would_show(tmp_path_factory):
    """The folders' weights make every mechanism matter: the plain model without the loop's
    additions, the side input, the head gates or the experts' weights is far from the plain model
    (so a test that passes has computed them)."""
    cfg = tz.MIXED
    d = folder(tmp_path_factory, "MIXED", cfg, "float32")
    conf, W = tz.read_folder(d)
    toks = prompts(cfg["vocab"], [60], seed=9)["r0"]
    ref = plain.forward(toks, W, conf)

    def far(changed):
        got = plain.forward(toks, changed, conf)
        d_ = (got - ref) - (got - ref).mean(-1, keepdims=True)
        return float(np.sqrt((d_ ** 2).mean()) / np.sqrt(((ref - ref.mean(-1, keepdims=True)) ** 2).mean()))
    for zeroed in ("loop.step", "side.embed", "l2.mix.g", "l0.mlp.router", "l1.ls1", "l3.norm1.b",
                   "l0.mix.k.norm"):
        W2 = dict(W)
        W2[zeroed] = np.zeros_like(W[zeroed])
        assert far(W2) > 0.02, zeroed


# ----------------------------------------------------------------------------- cuts of the same work
LENGTHS = [150, 97, 41, 5, 1, 66]


def cuts(reqs):
    mixed, _ = replay.cut_mixed(reqs, seed=3, decode_tail=20)
    singles, _ = replay.cut_mixed(reqs, seed=5, decode_tail=9, singles_first=True,
                                  sizes=(2, 2, 3, 17, 40))
    return {"whole": replay.cut_whole(reqs), "decode": replay.cut_tail_decode(reqs, tail=40),
            "portions": replay.cut_portions(reqs), "mixed": mixed, "mixed_singles_first": singles}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["MIXED", "OTHER", "ODD"])
def test_cuts_agree_with_plain(tmp_path_factory, name, dtype):
    cfg = getattr(tz, name)
    d = folder(tmp_path_factory, name, cfg, dtype)
    reqs = prompts(cfg["vocab"], LENGTHS, seed=1)
    want = expected(d, reqs, dtype)
    got = {}
    for cut, steps in cuts(reqs).items():
        # the pool holds what the live requests hold and no more: pages and slots are used again
        runner = make_runner(d, dtype, replay.peak_tokens(steps), page_size=16 if name == "MIXED" else 8)
        got[cut] = replay.run_in_process(runner, steps)
        check(got[cut], want, dtype, reqs)
    # how the work was cut changes the logits by rounding only
    for cut in got:
        for key, row in got[cut].items():
            ref = got["whole"][key]
            scale = float(np.abs(ref - ref.mean()).max())
            if dtype == "float32":
                assert float(np.abs(row - ref).max()) <= 1e-3 * scale, (cut, key)


def test_first_tokens_and_short_requests(tmp_path_factory):
    cfg = tz.MIXED
    d = folder(tmp_path_factory, "MIXED", cfg, "float32")
    reqs = prompts(cfg["vocab"], [1, 2, 3, 1, 4, 2, 1], seed=8)
    want = expected(d, reqs)
    for steps in (replay.cut_whole(reqs), replay.cut_tail_decode(reqs, tail=3)):
        rows = replay.run_in_process(make_runner(d, "float32", replay.peak_tokens(steps)), steps)
        check(rows, want, "float32", reqs)


def test_long_decoding_past_windows_and_pages_through_graphs(tmp_path_factory):
    cfg = tz.MIXED
    d = folder(tmp_path_factory, "MIXED", cfg, "float32")
    reqs = prompts(cfg["vocab"], [230], seed=2)
    steps = replay.cut_tail_decode(reqs, tail=200)       # 30 in one step, then 200 single tokens
    runner = make_runner(d, "float32", replay.peak_tokens(steps), eager=False)
    check(replay.run_in_process(runner, steps), expected(d, reqs), "float32", reqs)
    assert runner.graph_launches > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_the_large_kernels(tmp_path_factory, dtype):
    """Portions of 64 query rows and more at head size 64 reach the kernels that long prompts of
    large models use; the first layer's head size takes the plain attention kernel."""
    cfg = tz.OTHER
    d = folder(tmp_path_factory, "OTHER", cfg, dtype)
    reqs = prompts(cfg["vocab"], [300, 131], seed=3)
    steps = replay.cut_portions(reqs, sizes=replay.LONG_SIZES)
    rows = replay.run_in_process(make_runner(d, dtype, replay.peak_tokens(steps)), steps)
    check(rows, expected(d, reqs, dtype), dtype, reqs)


def test_a_long_portion_takes_the_tcgen05_grouped_products(tmp_path_factory):
    """Six hundred tokens in one step are 1,200 and 1,800 (token, expert) pairs in the routed
    layers: enough for the grouped products on tcgen05, whose results follow the plain model like
    the others'."""
    from ginfer_b200.ops import moe
    cfg = tz.MIXED
    d = folder(tmp_path_factory, "MIXED", cfg, "bfloat16")
    reqs = prompts(cfg["vocab"], [600, 70], seed=12)
    assert 600 * 2 >= moe.TCGEN05_MIN_PAIRS
    steps = replay.cut_whole(reqs)
    rows = replay.run_in_process(make_runner(d, "bfloat16", replay.peak_tokens(steps)), steps)
    check(rows, expected(d, reqs, "bfloat16"), "bfloat16", reqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_repeated_portion_shapes_replay_from_graphs(tmp_path_factory, dtype):
    """Steps with a portion of 600 tokens (1,200 and 1,800 expert pairs: the tcgen05 grouped
    products in bfloat16) come three times with the same shape, on other requests: from the
    second time on such a step is captured and replayed from a CUDA graph (routing, the plan of
    the pairs and the loop's entries included), and the logits are those of the eager engine."""
    cfg = tz.MIXED
    d = folder(tmp_path_factory, "MIXED", cfg, dtype)
    reqs = prompts(cfg["vocab"], [640, 640, 640, 640], seed=14)
    steps = []
    for rid, toks in reqs.items():
        steps.append({"step": len(steps), "end": [], "entries": [
            {"id": rid, "tokens": toks[:600], "want": [0, 599]}]})
        steps.append({"step": len(steps), "end": [rid], "entries": [
            {"id": rid, "tokens": toks[600:], "want": [39]}]})
    eager = replay.run_in_process(make_runner(d, dtype, 704), steps)
    runner = make_runner(d, dtype, 704, eager=False)
    graphs = replay.run_in_process(runner, steps)
    assert any(isinstance(k[0], str) for k in runner._graphs), "no portion graph was captured"
    assert runner.graph_launches > 0
    for key, row in eager.items():
        scale = float(np.abs(row).max())
        assert float(np.abs(graphs[key] - row).max()) <= (1e-5 if dtype == "float32" else 2e-2) * scale, key
    want = expected(d, reqs, dtype)
    worst, where, _, _ = row_errors(graphs, want)
    assert worst <= LIMIT[dtype][0], (where, worst)


# ----------------------------------------------------------------------------- a key that stands out
def _needle_tokens(W, conf):
    """A (probe, needle) pair of tokens whose score towers over the probe's score with any other
    token, in the one-layer model without rotation (a score depends on the two tokens only)."""
    L = conf["layers"][0]["mixer"]
    eps = conf["norm"]["eps"]
    h = plain.layer_norm(W["embed"], W["l0.norm1"], W["l0.norm1.b"], eps)
    V, D = h.shape[0], L["dim"]
    q = plain.rms_norm((h @ W["l0.mix.q"].T).reshape(V, L["heads"], D), W["l0.mix.q.norm"], eps)
    k = plain.rms_norm((h @ W["l0.mix.k"].T).reshape(V, 1, D), W["l0.mix.k.norm"], eps)
    s = (q[:, 0] @ k[:, 0].T) * L["scale"]                # head 0: [probe, key]
    order = np.sort(s, axis=1)
    margin = order[:, -1] - order[:, -2]
    probe = int(np.argmax(margin))
    return probe, int(np.argmax(s[probe])), float(margin[probe])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_key_just_inside_and_just_outside_the_window(tmp_path_factory, dtype):
    """One token's key is made to stand out for one probing token.  The probe is put so that the
    key is the last one its window holds, then the first one it no longer holds, at distances that
    cross a page border, as a prompt's row and as a decoded token: the engine's logits follow the
    plain ones, which differ between the two places."""
    cfg = tz.NEEDLE
    window = cfg["layers"][0]["mixer"]["mask"]["size"]
    d = folder(tmp_path_factory, "NEEDLE", cfg, dtype)
    conf, W = tz.read_folder(d)
    probe, needle, margin = _needle_tokens(W, conf)
    assert margin > 3.0
    rng = random.Random(0)
    fill = [t for t in range(cfg["vocab"]) if t not in (probe, needle)]
    reqs, at = {}, {}
    for start in (0, 5, 30):                              # the needle's position
        for dist in (window - 1, window):                 # seen last / just lost
            toks = [rng.choice(fill) for _ in range(start + dist + 1)]
            toks[start], toks[start + dist] = needle, probe
            reqs[f"n{start}_{dist}"] = toks
            at[f"n{start}_{dist}"] = start + dist
    want = expected(d, reqs, dtype)
    for start in (0, 5, 30):                              # the plain model tells the two apart
        a, b = f"n{start}_{window - 1}", f"n{start}_{window}"
        ra, rb = want[a][at[a]], want[b][at[b]]
        assert np.abs(ra - rb).max() > 0.1 * np.abs(ra).max()
    for steps in (replay.cut_whole(reqs), replay.cut_tail_decode(reqs, tail=2),
                  replay.cut_portions(reqs, sizes=(5, 2, 11))):
        runner = make_runner(d, dtype, replay.peak_tokens(steps), page_size=8)
        rows = replay.run_in_process(runner, steps)
        probes = {(rid, at[rid]): rows[(rid, at[rid])] for rid in reqs}
        worst, where, _, _ = row_errors(probes, want)
        assert worst <= (2e-4 if dtype == "float32" else 0.1), (where, worst)
        check(rows, want, dtype, reqs)


# ----------------------------------------------------------------------------- trace program, generation
def run_trace(model_dir, steps, max_tokens, out_dir, vocab, dtype="float32"):
    cmd = [sys.executable, os.path.join(replay.ROOT, "bin", "trace_run"), "--model", model_dir,
           "--dtype", dtype, "--out", out_dir, "--max-tokens", str(max_tokens)]
    p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for s in steps:
            p.stdin.write(json.dumps(s) + "\n")
            p.stdin.flush()
            assert p.stdout.readline().strip() == f"done {s['step']}"
        p.stdin.close()
        assert p.wait(timeout=120) == 0
    finally:
        if p.poll() is None:
            p.kill()
    return replay.collect(steps, lambda i: np.fromfile(os.path.join(out_dir, f"{i}.f32"),
                                                       dtype="<f4").reshape(-1, vocab))


def test_trace_program(tmp_path_factory, tmp_path):
    cfg = tz.MIXED
    d = folder(tmp_path_factory, "MIXED", cfg, "float32")
    reqs = prompts(cfg["vocab"], [90, 33, 2, 47, 64], seed=4)
    steps, peak = replay.cut_mixed(reqs, seed=7)
    os.makedirs(tmp_path / "out")
    rows = run_trace(d, steps, peak, str(tmp_path / "out"), cfg["vocab"])
    check(rows, expected(d, reqs), "float32", reqs)


@pytest.mark.parametrize("pages", [None, 14])
def test_greedy_generation_through_the_entry_point(tmp_path_factory, pages):
    from ginfer_b200.engine.llm import Engine
    from ginfer_b200.sampling import SamplingParams
    cfg = tz.MIXED
    d = folder(tmp_path_factory, "MIXED", cfg, "float32")
    reqs = prompts(cfg["vocab"], [40, 9, 75, 1, 23], seed=6)
    eng = Engine(d, dtype="float32", max_num_seqs=3, max_num_batched_tokens=64, max_seq_len=128,
                 num_kvcache_blocks=pages, kvcache_block_size=8)
    outs = eng.generate(list(reqs.values()), SamplingParams(temperature=0.0, max_tokens=10,
                                                             ignore_eos=True))
    conf, W = tz.read_folder(d)
    assert any(len(set(o)) > 2 for o in outs), outs              # no echo of one token
    for toks, out in zip(reqs.values(), outs):
        assert len(out) == 10
        seq = list(toks)
        for t in out:
            logits = plain.forward(seq, W, conf)[-1]
            if int(np.argmax(logits)) != t:              # only a close call may differ
                assert float(logits.max() - logits[t]) < 1e-3 * float(np.abs(logits).max()), (seq, t)
            seq.append(t)
    if pages is not None:
        eng.runner.cache.check()


def test_command_line(tmp_path_factory, tmp_path):
    cfg = tz.OTHER
    d = folder(tmp_path_factory, "OTHER", cfg, "float32")
    reqs = prompts(cfg["vocab"], [6, 11], seed=10)
    f = tmp_path / "prompts.txt"
    f.write_text("\n".join(json.dumps(t) for t in reqs.values()) + "\n")
    r = subprocess.run([sys.executable, os.path.join(replay.ROOT, "bin", "ginfer_generate"),
                        "--model-path", d, "--dtype", "float32", "--prompt-ids", str(f),
                        "--max-tokens", "5", "--ignore-eos", "--max-num-seqs", "2",
                        "--max-seq-len", "64", "--num-kvcache-blocks", "8"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(x) for x in r.stdout.strip().splitlines()]
    conf, W = tz.read_folder(d)
    for toks, line in zip(reqs.values(), lines):
        seq = list(toks)
        assert len(line["output_ids"]) == 5
        for t in line["output_ids"]:
            logits = plain.forward(seq, W, conf)[-1]
            if int(np.argmax(logits)) != t:
                assert float(logits.max() - logits[t]) < 1e-3 * float(np.abs(logits).max())
            seq.append(t)


# ----------------------------------------------------------------------------- kernels alone
def test_stream_update_kernel():
    from ginfer_b200.ops import prenorm
    g = torch.Generator(device="cuda").manual_seed(0)
    for act in (torch.float32, torch.bfloat16):
        for H in (88, 52, 1, 513):
            R = 37
            x = torch.randn(R, H, generator=g, device="cuda") * 2 + 0.5
            y = (torch.randn(R, H, generator=g, device="cuda") * 3).to(act)
            s = torch.randn(H, generator=g, device="cuda")
            w = torch.randn(H, generator=g, device="cuda")
            b = torch.randn(H, generator=g, device="cuda")
            full = torch.randn(R, H, generator=g, device="cuda")
            row = torch.randn(H, generator=g, device="cuda")
            tol = dict(atol=2e-5, rtol=2e-5)
            # scaled output of a sublayer, then a layer norm of the new stream
            out, a, n = prenorm.stream_update(x, act, y=y, scale=s, mult=0.3, want_act=True,
                                              norm=prenorm.NORM_LAYER, norm_weight=w,
                                              norm_bias=b, norm_eps=1e-3)
            want = x.double() + 0.3 * s.double() * y.double()
            assert torch.allclose(out.double(), want, **tol)
            assert torch.equal(a, out.to(act))
            ln = torch.from_numpy(plain.layer_norm(out.double().cpu().numpy(), w.double().cpu().numpy(),
                                                   b.double().cpu().numpy(), 1e-3)).cuda()
            assert torch.allclose(n.double(), ln, atol=2e-2 if act == torch.bfloat16 else 5e-5,
                                  rtol=1e-2 if act == torch.bfloat16 else 1e-5)
            # the RMS-normed output of a sublayer, no norm behind it
            out, a, n = prenorm.stream_update(x, act, y=y, scale=s, mult=0.7, y_rms_eps=1e-2)
            want = x.double() + 0.7 * torch.from_numpy(plain.rms_norm(
                y.double().cpu().numpy(), s.double().cpu().numpy(), 1e-2)).cuda()
            assert a is None and n is None and torch.allclose(out.double(), want, **tol)
            # a second stream and a row vector; RMS norm behind
            out, _, n = prenorm.stream_update(x, act, add_full=full, add_row=row,
                                              norm=prenorm.NORM_RMS, norm_weight=w, norm_eps=1e-4)
            want = x.double() + full.double() + row.double()
            assert torch.allclose(out.double(), want, **tol)
            rn = torch.from_numpy(plain.rms_norm(out.double().cpu().numpy(),
                                                 w.double().cpu().numpy(), 1e-4)).cuda()
            assert torch.allclose(n.double(), rn, atol=2e-2 if act == torch.bfloat16 else 5e-5,
                                  rtol=1e-2 if act == torch.bfloat16 else 1e-5)
            # rows selected, the norm only
            rows = torch.tensor([5, 0, 36, 5], dtype=torch.int32, device="cuda")
            out, _, n = prenorm.stream_update(x, act, rows=rows, want_out=False,
                                              norm=prenorm.NORM_LAYER, norm_weight=w, norm_eps=1e-3)
            ln = torch.from_numpy(plain.layer_norm(x[rows.long()].double().cpu().numpy(),
                                                   w.double().cpu().numpy(), 0.0, 1e-3)).cuda()
            assert out is None and n.shape == (4, H)
            assert torch.allclose(n.double(), ln, atol=2e-2 if act == torch.bfloat16 else 5e-5,
                                  rtol=1e-2 if act == torch.bfloat16 else 1e-5)


@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
def test_qk_norm_rotation_and_cache_write_kernel(act, interleaved):
    from ginfer_b200.ops import prenorm
    g = torch.Generator().manual_seed(3)
    for nh, nkv, hd, pairs, own_v in ((4, 2, 24, 8, False), (3, 1, 7, 3, True), (2, 2, 64, 32, False),
                                      (1, 1, 40, 0, False)):
        T, page, npages = 29, 4, 12
        k_off = nh * hd
        v_off = k_off + nkv * hd if own_v else k_off
        cols = v_off + nkv * hd + 3                      # something behind, untouched
        qkv = (torch.randn(T, cols, generator=g) * 2).to(act)
        qw, kw = torch.randn(hd, generator=g) + 1, torch.randn(hd, generator=g) + 1
        freqs = torch.rand(pairs, generator=g) if pairs else None
        pos = torch.randint(0, 500, (T,), generator=g).int()
        slots = torch.randperm(npages * page, generator=g)[:T].int()
        pages = torch.zeros(2, npages, page, nkv, hd, dtype=act)
        dev = qkv.cuda()
        dpages = pages.cuda()
        prenorm.qk_norm_rope(dev, nh, nkv, hd, k_off, v_off, qw.cuda(), kw.cuda(), 1e-3,
                             None if freqs is None else freqs.cuda(), interleaved, pos.cuda(),
                             slots.cuda(), dpages)
        x = qkv.double().numpy()
        f = np.zeros(0) if freqs is None else freqs.double().numpy()

        def want(heads, off, w):
            v = plain.rms_norm(x[:, off:off + heads * hd].reshape(T, heads, hd), w.double().numpy(), 1e-3)
            if interleaved:
                return plain.rotate_pairs(v, pos.numpy(), f)
            perm = list(range(hd))                       # halves (i, i + n) as neighbours and back
            for i in range(pairs):
                perm[2 * i], perm[2 * i + 1] = i, i + pairs
            out = np.empty_like(v)
            out[..., perm] = plain.rotate_pairs(v[..., perm], pos.numpy(), f)
            return out
        tol = 3e-2 if act == torch.bfloat16 else 2e-5
        got = dev.cpu().double().numpy()
        assert np.allclose(got[:, :k_off].reshape(T, nh, hd), want(nh, 0, qw), atol=tol, rtol=tol)
        assert np.array_equal(got[:, k_off:], x[:, k_off:])             # k, v, the rest: as they were
        flat = dpages.cpu().double().numpy().reshape(2, npages * page, nkv, hd)
        assert np.allclose(flat[0][slots.long().numpy()], want(nkv, k_off, kw), atol=tol, rtol=tol)
        assert np.array_equal(flat[1][slots.long().numpy()],
                              x[:, v_off:v_off + nkv * hd].reshape(T, nkv, hd))
        untouched = np.ones(npages * page, bool)
        untouched[slots.long().numpy()] = False
        assert not flat[:, untouched].any()
        # without slots nothing is cached and q is still prepared
        dev2, p2 = qkv.cuda(), pages.cuda()
        prenorm.qk_norm_rope(dev2, nh, nkv, hd, k_off, v_off, qw.cuda(), kw.cuda(), 1e-3,
                             None if freqs is None else freqs.cuda(), interleaved, pos.cuda(), None, p2)
        assert torch.equal(dev2, dev) and not p2.any()


def test_head_gate_and_token_gate_kernels():
    from ginfer_b200.ops import prenorm
    g = torch.Generator().manual_seed(5)
    for act in (torch.float32, torch.bfloat16):
        tol = 2e-2 if act == torch.bfloat16 else 1e-6
        T, nh, hd = 23, 3, 10
        o = torch.randn(T, nh * hd, generator=g).to(act)
        wide = (torch.randn(T, nh + 5, generator=g) * 4).to(act)
        gates = wide[:, 2:2 + nh]
        got = prenorm.head_gate(o.cuda(), wide.cuda()[:, 2:2 + nh], nh, hd).cpu().double()
        want = o.double().view(T, nh, hd) * torch.sigmoid(gates.double())[:, :, None]
        assert torch.allclose(got, want.view(T, -1), atol=tol, rtol=tol)
        V, total, dim, off = 31, 17, 5, 9
        table = torch.randn(V, total, generator=g).to(act)
        ids = torch.randint(0, V, (T,), generator=g).int()
        for zt in {torch.float32, act}:
            z = (torch.randn(T, dim, generator=g) * 2).to(zt)
            got = prenorm.token_gate(z.cuda(), ids.cuda(), table.cuda(), off).cpu().double()
            want = torch.from_numpy(plain.gelu_tanh(z.double().numpy())) \
                * table.double()[ids.long(), off:off + dim]
            assert got.shape == (T, dim) and torch.allclose(got, want, atol=tol, rtol=tol)


def test_sigmoid_router_chooses_as_plain_does():
    from ginfer_b200.ops import moe
    g = torch.Generator(device="cuda").manual_seed(1)
    for E, top in ((5, 2), (12, 1), (3, 3), (70, 6)):
        z = torch.randn(41, E, generator=g, device="cuda") * 3
        z[0] = 0.5                                       # equal scores: the lowest indices win
        z[1] = -200.0                                    # scores of zero are still chosen in order
        idx, w = moe.route(z, top, False, "sigmoid")
        wi, ww = plain.router(z.double().cpu().numpy(), np.eye(E), top)
        assert np.array_equal(idx.cpu().numpy(), wi)
        assert np.allclose(w.cpu().numpy(), ww, atol=1e-6)
        assert idx[0].tolist() == list(range(top)) and idx[1].tolist() == list(range(top))
        _, wn = moe.route(z[2:], top, True, "sigmoid")
        assert torch.allclose(wn.sum(-1), torch.ones(39, device="cuda"), atol=1e-5)


@pytest.mark.parametrize("act, K, F", [(torch.float32, 40, 24), (torch.bfloat16, 48, 40),
                                       (torch.bfloat16, 52, 20), (torch.bfloat16, 256, 136)])
def test_grouped_expert_products_scale_the_input(act, K, F):
    """Every (token, expert) pair against the expert run on that token's row times its weight;
    sizes that take the tensor-core kernel and sizes that it refuses."""
    from ginfer_b200.ops import moe
    g = torch.Generator().manual_seed(7)
    T, E, top = 150, 6, 3
    x = torch.randn(T, K, generator=g).to(act)
    up = (torch.randn(E, F, K, generator=g) * 0.3).to(act)
    down = (torch.randn(E, K, F, generator=g) * 0.3).to(act)
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).int()
    idx[:40] = torch.tensor([4, 1, 0])                   # one expert with more than a tile of rows
    wgt = torch.rand(T, top, generator=g) + 0.2
    tc = moe.on_tensor_cores(act, K, F)
    assert tc == (act == torch.bfloat16 and K % 8 == 0)
    plan = moe.Plan(idx.cuda(), E, tc)
    y = moe.grouped_relu2(x.cuda(), up.cuda(), plan, wgt.cuda())
    out = moe.combine(moe.grouped_down(y, down.cuda(), plan), plan, None, T).cpu().double()
    rnd = plain.bf16_round if act == torch.bfloat16 else plain.ident
    want = np.zeros((T, K))
    for t in range(T):
        for e, w in zip(idx[t].tolist(), wgt[t].double().tolist()):
            a = np.maximum(rnd(w * (x[t].double().numpy() @ up[e].double().numpy().T)), 0.0) ** 2
            want[t] += rnd(a) @ down[e].double().numpy().T
    tol = 3e-2 if act == torch.bfloat16 else 1e-4
    assert np.allclose(out.numpy(), want, atol=tol * np.abs(want).max(), rtol=tol)
    # weights on the output instead: the plain sum of the pairs times their weights
    y1 = moe.grouped_relu2(x.cuda(), up.cuda(), plan, None)
    out1 = moe.combine(moe.grouped_down(y1, down.cuda(), plan), plan, wgt.cuda(), T).cpu().double()
    want1 = np.zeros((T, K))
    for t in range(T):
        for e, w in zip(idx[t].tolist(), wgt[t].double().tolist()):
            want1[t] += w * plain.expert(x[t:t + 1].double().numpy(), up[e].double().numpy(),
                                         down[e].double().numpy(), rnd)[0]
    assert np.allclose(out1.numpy(), want1, atol=tol * np.abs(want1).max(), rtol=tol)


@pytest.mark.parametrize("K, F, T, E, top", [(256, 136, 1500, 6, 3), (64, 264, 700, 3, 2),
                                             (2048, 512, 1024, 40, 4)])
def test_grouped_products_on_tcgen05_equal_the_mma_kernel(K, F, T, E, top):
    """Many pairs: the persistent tcgen05 kernel over rows brought into sorted order, tiles that
    reach into the next expert's rows, experts with no rows, column tiles past an expert's matrix.
    Both first products (scaled relu^2 and the clamped gated one) and the down product against the
    ``mma.sync`` kernel on the same pairs; the scaled one also against plain arithmetic."""
    from ginfer_b200.ops import gemm_bf16, moe
    g = torch.Generator().manual_seed(11)
    x = torch.randn(T, K, generator=g).bfloat16().cuda()
    up = (torch.randn(E, F, K, generator=g) * K ** -0.5).bfloat16().cuda()
    gate_up = (torch.randn(E, 2 * F, K, generator=g) * K ** -0.5).bfloat16().cuda()
    down = (torch.randn(E, K, F, generator=g) * F ** -0.5).bfloat16().cuda()
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).int()
    idx[idx == 1] = 0 if E > 3 else 2                    # an expert without rows
    idx[:, 1] = torch.where(idx[:, 1] == idx[:, 0], (idx[:, 0] + 1) % E, idx[:, 1])
    wgt = (torch.rand(T, top, generator=g) + 0.2).cuda()
    assert moe.kernel_for(x, T * top, (K, F), (F, K)) == "tcgen05"
    tc, mma = moe.Plan(idx.cuda(), E, "tcgen05"), moe.Plan(idx.cuda(), E, True)
    assert tc.tcgen05 and not mma.tcgen05

    def by_pair(rows, plan):                             # sorted rows back in pair order
        return rows[plan.pos_of_pair.long()].float()
    y_tc, y_mma = moe.grouped_relu2(x, up, tc, wgt), moe.grouped_relu2(x, up, mma, wgt)
    ref = by_pair(y_mma, mma)
    assert torch.allclose(by_pair(y_tc, tc), ref, atol=2e-2 * float(ref.abs().max()), rtol=2e-2)
    t = 7
    for k, e in enumerate(idx[t].tolist()):
        a = (x[t].double() @ up[e].double().T) * float(wgt[t, k])
        want = torch.relu(a.bfloat16().double()) ** 2
        got = y_tc[tc.pos_of_pair[t * top + k].long()].double()
        assert torch.allclose(got, want, atol=2e-2 * float(want.abs().max()), rtol=2e-2)
    z_tc = moe.grouped_glu(x, gate_up, tc, 1.25, 1.702, 1.0)
    z_mma = moe.grouped_glu(x, gate_up, mma, 1.25, 1.702, 1.0)
    ref = by_pair(z_mma, mma)
    assert torch.allclose(by_pair(z_tc, tc), ref, atol=2e-2 * float(ref.abs().max()), rtol=2e-2)
    d_tc = moe.combine(moe.grouped_down(y_tc, down, tc), tc, None, T)
    d_mma = moe.combine(moe.grouped_down(y_tc[tc.pos_of_pair.long()][mma.pair_of_pos.long()]
                                         .contiguous(), down, mma), mma, None, T)
    assert torch.allclose(d_tc, d_mma, atol=1e-2 * float(d_mma.abs().max()), rtol=1e-2)
    gemm_bf16.check_errors("cuda:0")


def test_stream_update_adds_a_token_s_pairs_up():
    from ginfer_b200.ops import prenorm
    g = torch.Generator(device="cuda").manual_seed(4)
    for H, top in ((88, 3), (50, 1), (1024, 4)):
        R = 21
        x = torch.randn(R, H, generator=g, device="cuda")
        rows = torch.randn(R * top, H, generator=g, device="cuda")
        pos = torch.randperm(R * top, generator=g, device="cuda").int()
        w = torch.rand(R, top, generator=g, device="cuda")
        s = torch.randn(H, generator=g, device="cuda")
        for weights in (None, w):
            y = rows[pos.long()].view(R, top, H).double()
            if weights is not None:
                y = y * weights.double()[:, :, None]
            want = x.double() + 0.5 * s.double() * y.sum(1)
            out, _, _ = prenorm.stream_update(x, torch.bfloat16, y=rows, scale=s, mult=0.5,
                                              pairs=(pos, weights, top))
            assert torch.allclose(out.double(), want, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("K, F, T, E, top", [(256, 136, 1, 6, 3), (64, 264, 8, 3, 2),
                                             (2048, 96, 16, 40, 4), (72, 88, 30, 5, 2)])
def test_grouped_products_of_a_handful_of_pairs(K, F, T, E, top):
    """Decode steps of few requests: the kernel that streams an expert's rows once for up to eight
    pairs, against the ``mma.sync`` kernel on the same pairs (all three products); an expert with
    more than eight pairs has several tiles."""
    from ginfer_b200.ops import moe
    g = torch.Generator().manual_seed(13)
    x = torch.randn(T, K, generator=g).bfloat16().cuda()
    up = (torch.randn(E, F, K, generator=g) * K ** -0.5).bfloat16().cuda()
    gate_up = (torch.randn(E, 2 * F, K, generator=g) * K ** -0.5).bfloat16().cuda()
    down = (torch.randn(E, K, F, generator=g) * F ** -0.5).bfloat16().cuda()
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).int()
    if T >= 16:
        idx[:12, 0] = 2                                  # twelve pairs of one expert: two tiles
        idx[:12, 1] = 0
    wgt = (torch.rand(T, top, generator=g) + 0.2).cuda()
    assert moe.kernel_for(x, T * top, (K, F), (F, K)) == ("few" if T * top <= moe.FEW_MAX_PAIRS
                                                          else True)
    few, mma = moe.Plan(idx.cuda(), E, "few"), moe.Plan(idx.cuda(), E, True)
    assert few.few and not mma.few

    def by_pair(rows, plan):
        return rows[plan.pos_of_pair.long()].float()
    for a, b in ((moe.grouped_relu2(x, up, few, wgt), moe.grouped_relu2(x, up, mma, wgt)),
                 (moe.grouped_glu(x, gate_up, few, 1.25, 1.702, 1.0),
                  moe.grouped_glu(x, gate_up, mma, 1.25, 1.702, 1.0))):
        ref = by_pair(b, mma)
        assert torch.allclose(by_pair(a, few), ref, atol=2e-2 * float(ref.abs().max()), rtol=2e-2)
    y = moe.grouped_relu2(x, up, mma, wgt)
    y_few = y[mma.pos_of_pair.long()][few.pair_of_pos.long()].contiguous()
    d_few = moe.combine(moe.grouped_down(y_few, down, few), few, None, T)
    d_mma = moe.combine(moe.grouped_down(y, down, mma), mma, None, T)
    assert torch.allclose(d_few, d_mma, atol=1e-3 * float(d_mma.abs().max()), rtol=1e-3)

