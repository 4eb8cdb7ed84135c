"""Vilepel on the device against the plain implementation (``plain_vilepel``): every mechanism
alone, whole prompts against token-by-token decoding, portions down to two tokens, batches of
unequal requests, pages and slots used again, keys at the edges of windows and pages, long
decoding, other sizes, and greedy generation through the entry point."""
import json
import os
import random

import numpy as np
import pytest
import torch

import plain_vilepel as plain
import replay
import tiny_vilepel as tv

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
_folders: dict = {}
_expected: dict = {}


def folder(tmp_path_factory, name, cfg, dtype):
    key = (name, dtype)
    if key not in _folders:
        path = str(tmp_path_factory.mktemp(f"vilepel_{name}_{dtype}"))
        _folders[key] = tv.write_folder(path, cfg, seed=len(name), storage=DTYPES[dtype])
    return _folders[key]


def stored(model_dir):
    from ginfer_b200.weights.safetensors_io import open_model_tensors
    return {n: f.get(k) for n, (f, k) in open_model_tensors(model_dir).items()}


def prompts(vocab, lengths, seed=0):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


def expected(model_dir, cfg, requests):
    out = {}
    W = None
    for rid, toks in requests.items():
        key = (model_dir, tuple(toks))
        if key not in _expected:
            W = W or stored(model_dir)
            _expected[key] = plain.forward(cfg, W, toks).numpy()
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


# float32: differences of summation order.  bfloat16: the folders' peaked attention and clear
# routing amplify the format's rounding, so single rows may be a fifth off while the mean stays
# small, and a row whose router scores were close may choose another expert (at most one row in
# thirty may be off for that); a misplaced page, a lost state or a window off by one puts most rows
# near one.
LIMIT = {"float32": (2e-4, 5e-5), "bfloat16": (0.3, 0.1)}


def check(rows, want, dtype, requests):
    assert len(rows) == sum(len(t) for t in requests.values()), "a logits row is missing"
    worst, where, mean, errs = row_errors(rows, want)
    if dtype == "bfloat16":
        over = sum(e > LIMIT[dtype][0] for e in errs)
        assert over <= len(errs) // 30, f"{over} of {len(errs)} rows are off; worst {where}: {worst:.3e}"
    else:
        assert worst <= LIMIT[dtype][0], f"worst row {where}: relative error {worst:.3e}"
    assert mean <= LIMIT[dtype][1], f"mean relative error {mean:.3e}"


# ----------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("name", ["LATENT_ONLY", "DELTA_ONLY", "DENSE_FF", "ROUTED_FF"])
def test_each_mechanism_alone(tmp_path_factory, name):
    cfg = getattr(tv, name)
    d = folder(tmp_path_factory, name, cfg, "float32")
    reqs = prompts(cfg["vocab"], [70, 3, 1])
    steps = replay.cut_whole(reqs)
    rows = replay.run_in_process(make_runner(d, "float32", replay.peak_tokens(steps)), steps)
    check(rows, expected(d, cfg, reqs), "float32", reqs)


# ----------------------------------------------------------------------------- cuts of the same work
LENGTHS = [150, 97, 41, 5, 1, 66]


def cuts(reqs):
    mixed, _ = replay.cut_mixed(reqs, seed=3, decode_tail=20)
    singles, _ = replay.cut_mixed(reqs, seed=5, decode_tail=9, singles_first=True,
                                  sizes=(2, 2, 3, 17, 40))
    return {"whole": replay.cut_whole(reqs), "decode": replay.cut_tail_decode(reqs, tail=40),
            "portions": replay.cut_portions(reqs), "mixed": mixed, "mixed_singles_first": singles}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["MIXED", "OTHER"])
def test_cuts_agree_with_plain(tmp_path_factory, name, dtype):
    cfg = getattr(tv, name)
    d = folder(tmp_path_factory, name, cfg, dtype)
    reqs = prompts(cfg["vocab"], LENGTHS, seed=1)
    want = expected(d, cfg, reqs)
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


def test_long_decoding_past_windows_and_pages_through_graphs(tmp_path_factory):
    cfg = tv.MIXED
    d = folder(tmp_path_factory, "MIXED", cfg, "float32")
    reqs = prompts(cfg["vocab"], [230], seed=2)
    steps = replay.cut_tail_decode(reqs, tail=200)       # 30 in one step, then 200 single tokens
    runner = make_runner(d, "float32", replay.peak_tokens(steps), eager=False)
    check(replay.run_in_process(runner, steps), expected(d, cfg, reqs), "float32", reqs)
    assert runner.graph_launches > 0


def test_trace_program(tmp_path_factory, tmp_path):
    cfg = tv.OTHER
    d = folder(tmp_path_factory, "OTHER", cfg, "float32")
    reqs = prompts(cfg["vocab"], [90, 33, 2, 47, 64], seed=4)
    steps, peak = replay.cut_mixed(reqs, seed=7)
    os.makedirs(tmp_path / "out")
    # the trace program reads the vocabulary size under the design's own key
    conf = json.load(open(os.path.join(d, "config.json")))
    assert "vocab_size" not in conf
    rows = run_trace(d, steps, peak, str(tmp_path / "out"), cfg["vocab"])
    check(rows, expected(d, cfg, reqs), "float32", reqs)


def run_trace(model_dir, steps, max_tokens, out_dir, vocab):
    import subprocess
    import sys
    cmd = [sys.executable, os.path.join(replay.ROOT, "bin", "trace_run"), "--model", model_dir,
           "--dtype", "float32", "--out", out_dir, "--max-tokens", str(max_tokens)]
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


# ----------------------------------------------------------------------------- generation
@pytest.mark.parametrize("pages", [None, 14])
def test_greedy_generation_through_the_entry_point(tmp_path_factory, pages):
    from ginfer_b200.engine.llm import Engine
    from ginfer_b200.sampling import SamplingParams
    cfg = tv.MIXED
    d = folder(tmp_path_factory, "MIXED", cfg, "float32")
    reqs = prompts(cfg["vocab"], [40, 9, 75, 1, 23], seed=6)
    eng = Engine(d, dtype="float32", max_num_seqs=3, max_num_batched_tokens=64, max_seq_len=128,
                 num_kvcache_blocks=pages, kvcache_block_size=8)
    outs = eng.generate(list(reqs.values()), SamplingParams(temperature=0.0, max_tokens=10,
                                                             ignore_eos=True))
    W = stored(d)
    for toks, out in zip(reqs.values(), outs):
        assert len(out) == 10
        seq = list(toks)
        for t in out:
            logits = plain.forward(cfg, W, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if int(torch.argmax(logits)) != t:           # only a close call may differ
                assert float(top2[0] - logits[t]) < 1e-3 * float(logits.abs().max()), (seq, t)
            seq.append(t)
    if pages is not None:
        eng.runner.cache.check()


# ----------------------------------------------------------------------------- kernels alone
def test_output_norm_kernel_and_activation_and_embedding():
    from ginfer_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(0)
    for act in (torch.float32, torch.bfloat16):
        x = torch.randn(37, 88, generator=g, device="cuda")
        y = (torch.randn(37, 88, generator=g, device="cuda") * 3).to(act)
        w = torch.randn(88, generator=g, device="cuda")
        out, a = ops.outnorm_add(x, y, w, 1e-3, act)
        want = x.double() + plain.unit_rms(y.double(), 1e-3) * w.double()
        assert torch.allclose(out.double(), want, atol=1e-5, rtol=1e-5)
        assert a.dtype == act and torch.equal(a, out.to(act))
        gu = (torch.randn(19, 2 * 30, generator=g, device="cuda") * 3).to(act)
        z = ops.clamped_glu(gu, 1.25, 1.702, 1.0)
        want = plain.gelu_sigmoid_glu(gu[:, 0::2].double(), gu[:, 1::2].double(), 1.25)
        assert torch.allclose(z.double(), want, atol=2e-2 if act == torch.bfloat16 else 1e-6)
        table = torch.randn(50, 24, generator=g, device="cuda").to(act)
        ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32, device="cuda")
        e, ea = ops.embedding_scaled(ids, table, 12.5, want_act=act != torch.float32)
        assert torch.equal(e, table[ids.long()].float() * 12.5)
        assert ea is None or torch.equal(ea, e.to(act))


def test_router_kernel_chooses_as_plain_does():
    from ginfer_b200.ops import moe
    g = torch.Generator(device="cuda").manual_seed(1)
    for E, top in ((5, 2), (12, 4), (3, 1), (4, 4), (70, 6)):
        z = torch.randn(41, E, generator=g, device="cuda") * 3
        z[0] = 0.0                                       # equal scores: the lowest indices win
        idx, w = moe.route(z, top, False)
        s = torch.softmax(z.double(), -1)
        ws, wi = torch.topk(s, top, dim=-1)
        assert torch.equal(idx[1:].long(), wi[1:]) and idx[0].tolist() == list(range(top))
        assert torch.allclose(w.double(), torch.gather(s, 1, idx.long()), atol=1e-6)
        _, wn = moe.route(z, top, True)
        assert torch.allclose(wn.sum(-1), torch.ones(41, device="cuda"), atol=1e-5)


class _Ctx:
    pass


def _latent_case(window, page, keys, H=2, C=40, R=8, dtype=torch.float32):
    """A cache of ``keys`` tokens of one request on shuffled pages."""
    g = torch.Generator().manual_seed(keys)
    npages = -(-keys // page)
    order = torch.randperm(npages + 3, generator=g)[:npages]
    c_pages = torch.zeros(npages + 3, page, 1, C)
    r_pages = torch.zeros(npages + 3, page, 1, R)
    c = torch.randn(keys, C, generator=g)
    r = torch.randn(keys, R, generator=g)
    for j in range(keys):
        c_pages[order[j // page], j % page, 0] = c[j]
        r_pages[order[j // page], j % page, 0] = r[j]
    return c, r, c_pages.to(dtype).cuda(), r_pages.to(dtype).cuda(), order.int().cuda()[None, :]


@pytest.mark.parametrize("window, page, keys", [(37, 16, 100), (16, 16, 64), (33, 8, 33), (5, 4, 3)])
def test_latent_attention_sees_the_window_and_nothing_else(window, page, keys):
    """One key's score is made to stand out: just inside the window it is the answer, just
    outside it must not be seen, in prompt rows and in a single decoded row alike."""
    from ginfer_b200.ops import latent
    H, C, R = 2, 40, 8
    c, r, c_pages, r_pages, table = _latent_case(window, page, keys)
    ctx = _Ctx()
    for rows in (list(range(keys)), [keys - 1]):
        T = len(rows)
        ctx.seq_of_token = torch.zeros(T, dtype=torch.int32, device="cuda")
        ctx.positions = torch.tensor(rows, dtype=torch.int32, device="cuda")
        for back in (window - 1, window, 0, 1):          # the last seen key, the first unseen one
            q_lat = torch.zeros(H, T, C)
            q_rot = torch.zeros(T, H, R)
            for i, p in enumerate(rows):
                if p - back >= 0:
                    q_lat[:, i] = 50.0 * c[p - back] / c[p - back].norm() ** 2 * 4
            out = latent.attention(q_lat.cuda(), q_rot.cuda(), c_pages, r_pages, table, ctx, window,
                                   1.0, page).cpu()
            for i, p in enumerate(rows):
                lo = max(0, p - window + 1)
                s = (c[lo:p + 1] @ q_lat[0, i]).double()
                want = torch.softmax(s, 0) @ c[lo:p + 1].double()
                assert torch.allclose(out[0, i].double(), want, atol=1e-4), (back, p)
                if p - back >= lo and p - back >= 0:
                    assert torch.allclose(out[0, i], c[p - back], atol=1e-3)


@pytest.mark.parametrize("D, Vd", [(12, 20), (10, 7), (64, 40)])
def test_delta_rule_keeps_a_far_token_and_forgets_by_its_decays(D, Vd):
    """Kernel alone: with decays of one a value written at the first token under a key that no
    later token uses is read back hundreds of tokens later, in one portion or token by token;
    with a decay below one on half of the key channels it fades by exactly that factor."""
    from ginfer_b200.ops import delta
    H, G, T = 2, 1, 300
    g0 = torch.Generator().manual_seed(0)
    k = torch.zeros(T, G, D)
    k[0, 0, 0] = 1.0
    for t in range(1, T):
        k[t, 0, 1 + t % (D - 1)] = 1.0
    q = torch.zeros(T, G, D)
    q[:, 0, 0] = 1.0
    v = torch.randn(T, H, Vd, generator=g0)
    beta = torch.ones(T, H)
    for decay in (1.0, 0.99):
        g = torch.ones(T, H, D)
        g[:, 1, :] = decay
        want = v[0].clone()
        want[1] *= decay ** (T - 1)
        for cut in ([T], [1] * T, [7, 2, 100, 1, 190]):
            state = torch.zeros(3, H * D * Vd, device="cuda")
            ctx = _Ctx()
            ctx.num_seqs = 1
            ctx.slot_ids = torch.tensor([1], dtype=torch.int32, device="cuda")
            at, last = 0, None
            for n in cut:
                ctx.cu_seqlens_q = torch.tensor([0, n], dtype=torch.int32, device="cuda")
                sl = slice(at, at + n)
                last = delta.recurrence(q[sl].cuda().contiguous(), k[sl].cuda().contiguous(),
                                        v[sl].cuda().contiguous(), g[sl].cuda().contiguous(),
                                        beta[sl].cuda().contiguous(), state, ctx)
                at += n
            assert torch.allclose(last[-1].cpu(), want, atol=1e-4), (decay, cut[:3])
            assert float(state[0].abs().max()) == 0.0 and float(state[2].abs().max()) == 0.0


@pytest.mark.parametrize("dtype, K, F, E, top, T", [
    (torch.bfloat16, 48, 40, 5, 2, 70), (torch.bfloat16, 136, 72, 9, 3, 300),
    (torch.bfloat16, 44, 20, 4, 4, 33), (torch.float32, 48, 40, 5, 2, 70),
    (torch.bfloat16, 64, 32, 6, 1, 1)])
def test_grouped_products_against_one_pair_at_a_time(dtype, K, F, E, top, T):
    """The sorted grouped products (tensor cores for bf16 sizes that 16-byte copies can fetch, the
    plain kernel otherwise) against every (token, expert) pair computed on its own."""
    from ginfer_b200.ops import moe
    g = torch.Generator(device="cuda").manual_seed(K)
    x = torch.randn(T, K, generator=g, device="cuda").to(dtype)
    w1 = (torch.randn(E, 2 * F, K, generator=g, device="cuda") * 0.3).to(dtype)
    w2 = (torch.randn(E, K, F, generator=g, device="cuda") * 0.3).to(dtype)
    idx, wgt = moe.route(torch.randn(T, E, generator=g, device="cuda"), top, False)
    plan = moe.Plan(idx, E, moe.on_tensor_cores(dtype, K, F))
    assert plan.tensor_cores == (dtype == torch.bfloat16 and K % 8 == 0 and F % 8 == 0)
    y = moe.grouped_glu(x, w1, plan, 1.25, 1.702, 1.0)
    out = moe.combine(moe.grouped_down(y, w2, plan), plan, wgt, T)
    want = torch.zeros(T, K, dtype=torch.float64, device="cuda")
    for t in range(T):
        for k in range(top):
            e = int(idx[t, k])
            gu = (x[t].double() @ w1[e].double().T).to(dtype).double()
            z = plain.gelu_sigmoid_glu(gu[0::2], gu[1::2], 1.25).to(dtype).double()
            want[t] += float(wgt[t, k]) * (z @ w2[e].double().T)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert torch.allclose(out.double(), want, atol=tol * float(want.abs().max()), rtol=tol)


@pytest.mark.parametrize("T", [1, 8, 40, 100, 800, 1100])
def test_clamped_gate_in_the_products_epilogues(T):
    """The clamped sigmoid-gated activation inside the gated products (few tokens: the split-K
    tcgen05 kernel; many: the persistent one; in between a library product and the activation
    kernel) against the formula on the bf16-rounded gate and up values."""
    from ginfer_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(T)
    K, I = 192, 328
    x = torch.randn(T, K, generator=g, device="cuda").to(torch.bfloat16)
    wg = (torch.randn(I, K, generator=g, device="cuda") * 0.2).to(torch.bfloat16)
    wu = (torch.randn(I, K, generator=g, device="cuda") * 0.2).to(torch.bfloat16)
    lin = ops.GatedLinear(wg, wu, clamped=(1.5, 1.702, 1.0))
    z = lin(x)
    gate = (x.double() @ wg.double().T).to(torch.bfloat16).double()
    up = (x.double() @ wu.double().T).to(torch.bfloat16).double()
    want = plain.gelu_sigmoid_glu(gate, up, 1.5)
    assert z.shape == (T, I) and z.dtype == torch.bfloat16
    assert (gate > 1.5).any() and (up.abs() > 1.5).any()          # the clamps are at work
    assert float((z.double() - want).abs().max()) <= 0.03 * float(want.abs().max())
    from ginfer_b200.ops import gemm_bf16
    gemm_bf16.check_errors("cuda:0")


@pytest.mark.parametrize("B, H, G, D, Vd", [(40, 8, 4, 24, 36), (3, 2, 2, 130, 9), (50, 6, 1, 64, 32)])
def test_delta_rule_batches_against_a_loop(B, H, G, D, Vd):
    """Many requests of unequal lengths in one launch (both widths of the kernel: four lanes a
    column where the batch fills the device, sixteen where it does not), states in shuffled
    slots, against the recurrence written as a loop in float64."""
    from ginfer_b200.ops import delta
    g0 = torch.Generator().manual_seed(B)
    lens = [1 + (7 * b) % 5 for b in range(B)]
    T = sum(lens)
    q = torch.randn(T, G, D, generator=g0) / D ** 0.5
    k = torch.nn.functional.normalize(torch.randn(T, G, D, generator=g0), dim=-1)
    v = torch.randn(T, H, Vd, generator=g0)
    g = torch.rand(T, H, D, generator=g0) * 0.5 + 0.5
    beta = torch.rand(T, H, generator=g0)
    slots = torch.randperm(B + 3, generator=g0)[:B]
    state0 = torch.randn(B + 3, H * D * Vd + 5, generator=g0)
    state = state0.clone().cuda()
    ctx = _Ctx()
    ctx.num_seqs = B
    ctx.slot_ids = slots.int().cuda()
    cu = torch.tensor([0] + lens).cumsum(0)
    ctx.cu_seqlens_q = cu.int().cuda()
    o = delta.recurrence(q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda(), state, ctx).cpu()
    per = H // G
    for b in range(B):
        S = state0[slots[b], :H * D * Vd].double().reshape(H, D, Vd).clone()
        for t in range(int(cu[b]), int(cu[b + 1])):
            for n in range(H):
                S[n] = g[t, n].double()[:, None] * S[n]
                u = beta[t, n].double() * (v[t, n].double() - S[n].T @ k[t, n // per].double())
                S[n] = S[n] + torch.outer(k[t, n // per].double(), u)
                assert torch.allclose(o[t, n].double(), S[n].T @ q[t, n // per].double(), atol=1e-4)
        got = state[slots[b]].cpu()
        assert torch.allclose(got[:H * D * Vd].double(), S.reshape(-1), atol=1e-4)
        assert torch.equal(got[H * D * Vd:], state0[slots[b], H * D * Vd:])
    untouched = [s for s in range(B + 3) if s not in set(slots.tolist())]
    assert torch.equal(state[untouched].cpu(), state0[untouched])


@pytest.mark.parametrize("H, C, R, keys, window, page", [
    (16, 512, 64, 300, 150, 16), (20, 256, 32, 130, 0, 8), (5, 64, 16, 70, 33, 16),
    (3, 48, 16, 64, 64, 16)])
def test_latent_attention_on_tensor_cores_agrees_with_plain_arithmetic(H, C, R, keys, window, page):
    """The tensor-core kernel (bf16 cache) against the plain fp32 one on the same values, at the
    sizes of large layers, with more heads than a row tile and with channel counts that leave
    warps idle; every row of a prompt, so that tiles end at every place."""
    from ginfer_b200.ops import latent
    g0 = torch.Generator().manual_seed(C + keys)
    npages = -(-keys // page)
    order = torch.randperm(npages + 2, generator=g0)[:npages]
    c = (torch.randn(keys, C, generator=g0)).to(torch.bfloat16)
    r = (torch.randn(keys, R, generator=g0)).to(torch.bfloat16)
    c_pages = torch.zeros(npages + 2, page, 1, C, dtype=torch.bfloat16)
    r_pages = torch.zeros(npages + 2, page, 1, R, dtype=torch.bfloat16)
    for j in range(keys):
        c_pages[order[j // page], j % page, 0] = c[j]
        r_pages[order[j // page], j % page, 0] = r[j]
    table = order.int().cuda()[None, :]
    ctx = _Ctx()
    ctx.seq_of_token = torch.zeros(keys, dtype=torch.int32, device="cuda")
    ctx.positions = torch.arange(keys, dtype=torch.int32, device="cuda")
    q_lat = (torch.randn(H, keys, C, generator=g0) * 0.3).to(torch.bfloat16).float().cuda()
    q_rot = (torch.randn(keys, H, R, generator=g0) * 0.3).to(torch.bfloat16).float().cuda()
    scale = (C + R) ** -0.5 * 3.0
    fast = latent.attention(q_lat, q_rot, c_pages.cuda(), r_pages.cuda(), table, ctx, window, scale,
                            page)
    slow = latent.attention(q_lat, q_rot, c_pages.float().cuda(), r_pages.float().cuda(), table,
                            ctx, window, scale, page)
    assert fast.dtype == torch.bfloat16 and slow.dtype == torch.float32
    err = (fast.float() - slow).abs().max()
    assert float(err) <= 0.02 * float(slow.abs().max()), float(err)


@pytest.mark.parametrize("window", [0, 700, 520])
def test_latent_attention_shares_a_tokens_keys_among_blocks_in_small_steps(window):
    """A step of three single tokens at 798-800 keys: several blocks take a share of each token's
    key tiles and a second kernel merges them; against the plain kernel."""
    from ginfer_b200.ops import latent
    H, C, R, keys, page = 16, 256, 32, 800, 16
    g0 = torch.Generator().manual_seed(window)
    c_pages = torch.randn(keys // page + 1, page, 1, C, generator=g0).to(torch.bfloat16).cuda()
    r_pages = torch.randn(keys // page + 1, page, 1, R, generator=g0).to(torch.bfloat16).cuda()
    table = torch.arange(keys // page + 1, dtype=torch.int32, device="cuda").repeat(3, 1)
    ctx = _Ctx()
    ctx.seq_of_token = torch.arange(3, dtype=torch.int32, device="cuda")
    ctx.positions = torch.tensor([797, 798, 799], dtype=torch.int32, device="cuda")
    ctx.max_kv_len = keys
    assert latent.key_splits(3, H, min(keys, window) if window else keys) > 1
    q_lat = (torch.randn(H, 3, C, generator=g0) * 0.3).cuda()
    q_rot = (torch.randn(3, H, R, generator=g0) * 0.3).cuda()
    fast = latent.attention(q_lat, q_rot, c_pages, r_pages, table, ctx, window, 0.2, page)
    slow = latent.attention(q_lat, q_rot, c_pages.float(), r_pages.float(), table, ctx, window,
                            0.2, page)
    assert float((fast.float() - slow).abs().max()) <= 0.02 * float(slow.abs().max())
