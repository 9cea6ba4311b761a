"""Vagonex on the GPU against the plain oracle (tests/plain/vagonex_plain.py): every mechanism alone, whole prompts,
decoding through the cache and the recurrent state, prompts in pieces, batches against each request alone, reuse of
slots and pages, the edges of chunks and pages, the first tokens, far keys and the sink, long decoding, other sizes,
and generation through the engine, the replay program and the command line."""
import copy
import json
import os
import subprocess

import numpy as np
import pytest
import torch

from vagonex_cases import (CASES, assert_rows, attention, delta, lightning, make_folder, model, oracle_view, row_errors,
                           tokens)

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("vagonex")
    return {k: make_folder(base, raw, seed, k) for k, (raw, seed) in CASES.items()}


def _runner(folder, dtype, **kw):
    from hos_b200.engine import Runner
    kw.setdefault("max_tokens", 4096)
    kw.setdefault("max_seq_len", 1024)
    return Runner.from_folder(folder, dtype=dtype, **kw)


def _oracle(folder, seqs):
    from plain import vagonex_plain as P
    cfg, w = oracle_view(folder)
    return [P.forward_logits(cfg, w, s) for s in seqs]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "B", "C", "D"])
def test_whole_prompts_of_unequal_lengths(folders, case, dtype):
    vocab = CASES[case][0]["vocab"]
    seqs = [tokens(i, n, vocab) for i, n in enumerate((1, 2, 37, 150))]      # 150: beyond two pages and every chunk
    want = _oracle(folders[case], seqs)
    r = _runner(folders[case], dtype)
    slots = r.admit(len(seqs))
    got = r.step(slots, seqs, [list(range(len(s))) for s in seqs]).cpu()
    assert_rows(got, torch.cat(want), dtype, f"case {case}")
    for s in slots:
        r.release(s)
    r.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "B", "C", "D"])
def test_a_prompt_then_token_by_token(folders, case, dtype):
    """Two requests decoded side by side through the replayed single-token step, across page borders (64, 128) and
    every chunk's edge; the shorter one leaves first.  The longer one is decoded for 141 steps."""
    vocab = CASES[case][0]["vocab"]
    seqs = [tokens(20, 150, vocab), tokens(21, 90, vocab)]
    plens = [9, 61]
    want = _oracle(folders[case], seqs)
    r = _runner(folders[case], dtype)
    slots = r.admit(2)
    first = r.step(slots, [s[:n] for s, n in zip(seqs, plens)]).cpu()
    got = [[first[0:1]], [first[1:2]]]
    pos, live = list(plens), [0, 1]
    while live:
        out = r.step([slots[i] for i in live], [[seqs[i][pos[i]]] for i in live]).cpu()
        for j, i in enumerate(live):
            got[i].append(out[j:j + 1])
            pos[i] += 1
        for i in [i for i in live if pos[i] == len(seqs[i])]:
            r.release(slots[i])
        live = [i for i in live if pos[i] < len(seqs[i])]
    for i in range(2):
        assert_rows(torch.cat(got[i]), want[i][plens[i] - 1:], dtype, f"case {case} request {i}")
    r.cache.check()


@pytest.mark.parametrize("case, dtype", [("A", "float32"), ("A", "bfloat16"), ("B", "float32"), ("C", "float32"), ("D", "bfloat16")])
def test_a_prompt_in_pieces_of_many_sizes(folders, case, dtype):
    """Pieces down to two tokens and one: fewer tokens than the convolution has taps, pieces that end on a page's
    border and one past it."""
    vocab = CASES[case][0]["vocab"]
    seq = tokens(30, 230, vocab)
    want = _oracle(folders[case], [seq])[0]
    r = _runner(folders[case], dtype)
    (slot,) = r.admit(1)
    at, got = 0, []
    for k in [2, 3, 59, 1, 65, 7, 2, 40, 1, 1, 30, 19]:
        piece = seq[at:at + k]
        got.append(r.step([slot], [piece], [list(range(len(piece)))]).cpu())
        at += len(piece)
    assert at == len(seq)
    assert_rows(torch.cat(got), want, dtype, f"case {case}")
    r.release(slot)
    r.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "C"])
def test_a_batch_gives_what_each_request_gives_alone(folders, case, dtype):
    """Also a step in which one request starts while others go on by one token and by several."""
    vocab = CASES[case][0]["vocab"]
    seqs = [tokens(40 + i, n, vocab) for i, n in enumerate((75, 3, 130))]
    r = _runner(folders[case], dtype)
    alone = []
    for s in seqs:
        (slot,) = r.admit(1)
        alone.append(r.step([slot], [s], [list(range(len(s)))]).cpu())
        r.release(slot)
    slots = r.admit(3)
    both = r.step(slots, seqs, [list(range(len(s))) for s in seqs]).cpu()
    for s in slots:
        r.release(s)
    tol = 2e-5 if dtype == "float32" else 4e-2      # no row shares a sum with another: in practice they are equal
    assert float(row_errors(both, torch.cat(alone)).max()) <= tol
    slots = r.admit(2)
    r.step(slots, [seqs[0][:74], seqs[2][:100]])
    (late,) = r.admit(1)
    mixed = r.step([late, slots[1], slots[0]], [seqs[1], seqs[2][100:109], seqs[0][74:75]],
                   [[0, 1, 2], list(range(9)), [0]]).cpu()
    ref = torch.cat([alone[1], alone[2][100:109], alone[0][74:75]])
    assert float(row_errors(mixed, ref).max()) <= tol
    r.cache.check()


def test_slots_pages_and_state_that_are_freed_are_used_again(folders):
    """What a freed slot's pages and state rows still hold must never be read: they are filled with large numbers
    before the slot is taken again."""
    vocab = CASES["A"][0]["vocab"]
    first, second = tokens(50, 140, vocab), tokens(51, 100, vocab)
    want = _oracle(folders["A"], [second])[0]
    r = _runner(folders["A"], "float32", max_tokens=256)       # four pages: the second request must reuse them
    (slot,) = r.admit(1)
    r.step([slot], [first[:130]])
    for t in first[130:]:
        r.step([slot], [[t]])
    r.release(slot)
    for g in r.cache.groups:
        for t in g.k + g.v:
            t.fill_(1e4)
    for t in r.cache.state_tensors():
        t.fill_(1e4)
    (again,) = r.admit(1)
    assert again == slot
    got = [r.step([again], [second[:70]], [list(range(70))]).cpu()]
    for t in second[70:]:
        got.append(r.step([again], [[t]]).cpu())
    assert_rows(torch.cat(got), want, "float32", "second request in a used slot")
    r.release(again)
    # a request that starts with single tokens in a used slot: its state comes from the admission, not from a prompt
    for t in r.cache.state_tensors():
        t.fill_(1e4)
    (again,) = r.admit(1)
    got = [r.step([again], [[t]]).cpu() for t in second[:12]]
    assert_rows(torch.cat(got), want[:12], "float32", "token by token from the first in a used slot")
    r.release(again)
    r.cache.check()


@pytest.mark.parametrize("case", ["A", "B", "C", "D"])
def test_the_edge_of_every_chunk_in_prompts_and_in_decoding(folders, case):
    """The oracle with every chunk one key longer, or one shorter, is far from the oracle itself (so a chunk that is
    off by one cannot pass), and the library agrees with the oracle at every position, whether the token comes in a
    prompt or alone."""
    from plain import vagonex_plain as P
    raw = CASES[case][0]
    cfg, w = oracle_view(folders[case])
    seq = tokens(60, 160, raw["vocab"])
    want = P.forward_logits(cfg, w, seq)
    for d in (1, -1):
        other = copy.deepcopy(cfg)
        for layer in other["layers"]:
            if layer["mixer"].get("mask") and layer["mixer"]["mask"]["size"] + d > 0:
                layer["mixer"]["mask"]["size"] += d
        assert float(row_errors(P.forward_logits(other, w, seq), want).median()) > 2e-3, \
            "the test would not see a chunk that is off by one"
    r = _runner(folders[case], "float32")
    (slot,) = r.admit(1)
    assert_rows(r.step([slot], [seq], [list(range(len(seq)))]).cpu(), want, "float32", "in a prompt")
    r.release(slot)
    (slot,) = r.admit(1)
    r.step([slot], [seq[:5]])
    got = [r.step([slot], [[t]]).cpu() for t in seq[5:]]
    assert_rows(torch.cat(got), want[5:], "float32", "decoded alone")
    r.release(slot)


def test_a_far_key_and_the_sink_show_in_the_logits(tmp_path):
    """One layer that sees all keys, with soft scores and large sinks: without the keys that lie more than 600 tokens
    back, or without the sink in the denominator, the oracle's logits move by far more than the tolerance.  In
    decoding a row's keys are cut into shares that are merged (more than 256 keys)."""
    from plain import vagonex_plain as P
    raw = model(48, 60, [attention(2, 1, 8, 12, 0.15, rot_dims=4, mlp=None)], alpha=0.5)

    def edit(t):
        t["l0.mix.sink"] = torch.tensor([4.0, 1.0])
    folder = make_folder(tmp_path, raw, 5, "far", edit)
    cfg, w = oracle_view(folder)
    seq = tokens(70, 640, 60)
    want = P.forward_logits(cfg, w, seq)
    assert float(row_errors(P.forward_logits(cfg, w, seq, use_sink=False), want).median()) > 2e-3
    short = P.forward_logits(cfg, w, seq, drop_far=600)
    assert float(row_errors(short[610:], want[610:]).median()) > 1e-4
    for dtype in ("float32", "bfloat16"):
        r = _runner(folder, dtype)
        (slot,) = r.admit(1)
        got = [r.step([slot], [seq[:600]], [list(range(600))]).cpu()] + [r.step([slot], [[t]]).cpu() for t in seq[600:]]
        assert_rows(torch.cat(got), want, dtype, "a layer that sees all keys")
        r.release(slot)


def test_every_layer_alone(folders):
    """The residual stream after the embedding and after every layer, in 32-bit, for a prompt; then the same for the
    prompt's second half fed after its first (every mixer resumes from its cache or state)."""
    from plain import vagonex_plain as P
    for case in ("A", "B", "C", "D"):
        cfg, w = oracle_view(folders[case])
        seq = tokens(80, 90, cfg["vocab"])
        want = []
        P.forward_hidden(cfg, w, seq, taps=want)
        r = _runner(folders[case], "float32")
        (slot,) = r.admit(1)
        taps = r.hidden_states([slot], [seq])
        emb = w["embed"][seq] * cfg["embedding"]["scale"]
        assert float((taps[0].cpu().double() - emb).abs().max()) <= 1e-6 * float(emb.abs().max())
        for i, (g, x) in enumerate(zip(taps[1:], want)):
            assert float(row_errors(g.cpu(), x).max()) < 1e-5, f"case {case}: after layer {i}"
        r.release(slot)
        (slot,) = r.admit(1)
        r.step([slot], [seq[:47]])
        taps = r.hidden_states([slot], [seq[47:]])
        for i, (g, x) in enumerate(zip(taps[1:], want)):
            assert float(row_errors(g.cpu(), x[47:]).max()) < 1e-5, f"case {case}: after layer {i}, second half"
        r.release(slot)


SINGLE = {
    "attention, keys wider than values, no rotation, no chunks": attention(3, 3, 40, 8, 0.3, mlp=None),
    "attention, heads of 200 and 264 numbers": attention(2, 1, 200, 264, 0.1, chunk=50, rot_dims=200, mlp=None),
    "attention, all of a head rotated with a ramp cut at neither end": attention(
        4, 2, 16, 16, 0.5, chunk=100, rot_dims=16, base=100.0, scaling=(16.0, 32, 3.0, 1.5), mlp=None),
    "decay rule, state rows over 32 threads of 32 numbers": lightning(1, 520, 8, (0.9,), mlp=None),
    "decay rule, one key number": lightning(2, 1, 40, (0.5, 0.8), mlp=None),
    "decay rule, 272 value columns": lightning(2, 24, 272, (0.95, 0.3), mlp=None),
    "delta rule, six value heads to a key head": delta(6, 1, 20, 36, 5, mlp=None),
    "delta rule, sixteen taps, heads of 130 numbers": delta(2, 2, 130, 130, 16, mlp=None),
    "delta rule with a feed-forward": delta(2, 1, 8, 8, 2),
}


@pytest.mark.parametrize("name", list(SINGLE))
def test_one_layer_models_of_other_sizes(tmp_path, name):
    """Sizes that the kernels' shapes switch on, each as a model of one layer: a prompt, then pieces of one to five
    tokens (fewer than the taps), in 32-bit."""
    raw = model(40, 50, [SINGLE[name]], ff=16, alpha=1.3, emb_scale=2.0)
    folder = make_folder(tmp_path, raw, 31, "one")
    seq = tokens(33, 150, 50)
    want = _oracle(folder, [seq])[0]
    r = _runner(folder, "float32")
    (slot,) = r.admit(1)
    got, at = [r.step([slot], [seq[:101]], [list(range(101))]).cpu()], 101
    for k in [1, 1, 2, 5, 1, 3, 1, 1, 4, 30]:
        got.append(r.step([slot], [seq[at:at + k]], [list(range(k))]).cpu())
        at += k
    assert at == len(seq)
    assert_rows(torch.cat(got), want, "float32", name)
    r.release(slot)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wider_layers_and_a_longer_prompt(folders, dtype):
    """A prompt of 700 tokens (chunks of 300: decoding rows see more than 256 keys and are cut into shares), a piece
    of 90, then single tokens beside a second request that starts later.  At these widths and lengths the 32-bit
    rounding noise is larger: every row within 1e-4 of the logits' size and the median within 2e-5."""
    vocab = CASES["E"][0]["vocab"]
    seqs = [tokens(140, 820, vocab), tokens(141, 75, vocab)]
    want = _oracle(folders["E"], seqs)
    r = _runner(folders["E"], dtype, max_seq_len=2048)
    a, b = r.admit(2)
    probe = list(range(0, 700, 7))
    got = [r.step([a], [seqs[0][:700]], [probe]).cpu(), r.step([a], [seqs[0][700:790]], [list(range(90))]).cpu()]
    out = r.step([b, a], [seqs[1][:60], seqs[0][790:791]], [[59], [0]]).cpu()
    got.append(out[1:2])
    got_b = [out[0:1]]
    for k in range(15):
        out = r.step([a, b], [[seqs[0][791 + k]], [seqs[1][60 + k]]]).cpu()
        got.append(out[0:1])
        got_b.append(out[1:2])
    for k in range(15, 29):
        got.append(r.step([a], [[seqs[0][791 + k]]]).cpu())
    pairs = ((torch.cat(got), torch.cat([want[0][probe], want[0][700:820]])), (torch.cat(got_b), want[1][59:75]))
    for g, x in pairs:
        e = row_errors(g, x)
        if dtype == "float32":
            assert float(e.median()) <= 2e-5 and float(e.max()) <= 1e-4, f"median {float(e.median()):.2e}, worst {float(e.max()):.2e}"
        else:
            assert_rows(g, x, dtype, "wider layers")
    r.release(a)
    r.release(b)
    r.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_tokens_at_the_tensor_core_kernels_sizes(folders, dtype):
    """Requests of one and two tokens at head sizes that the tensor-core kernels take: a single token at position 0
    (the single-token kernel), two short prompts side by side (the FMA kernel), then both decoded, then a prompt of
    nine tokens beside them."""
    vocab = CASES["E"][0]["vocab"]
    seqs = [tokens(150, 12, vocab), tokens(151, 14, vocab), tokens(152, 9, vocab)]
    want = _oracle(folders["E"], seqs)
    r = _runner(folders["E"], dtype)
    (a,) = r.admit(1)
    got_a = [r.step([a], [seqs[0][:1]]).cpu()]
    (b,) = r.admit(1)
    out = r.step([b, a], [seqs[1][:2], seqs[0][1:3]], [[0, 1], [0, 1]]).cpu()
    got_b, got_a = [out[:2]], got_a + [out[2:]]
    for k in range(9):
        out = r.step([a, b], [[seqs[0][3 + k]], [seqs[1][2 + k]]]).cpu()
        got_a.append(out[0:1])
        got_b.append(out[1:2])
    (c,) = r.admit(1)
    out = r.step([c, b], [seqs[2], seqs[1][11:14]], [list(range(9)), [0, 1, 2]]).cpu()
    got_b.append(out[9:])
    for g, x in ((torch.cat(got_a), want[0]), (torch.cat(got_b), want[1]), (out[:9], want[2])):
        if dtype == "float32":
            e = row_errors(g, x)
            assert float(e.max()) <= 1e-4, f"worst {float(e.max()):.2e}"
        else:
            assert_rows(g, x, dtype, "first tokens")
    for s_ in (a, b, c):
        r.release(s_)
    r.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(folders, dtype):
    """The public entry point and its scheduler: more prompts than run side by side, unequal lengths."""
    from plain import vagonex_plain as P
    from hos_b200 import Engine
    cfg, w = oracle_view(folders["A"])
    prompts = [tokens(100 + i, n, cfg["vocab"]) for i, n in enumerate((5, 70, 1))]
    eng = Engine(folders["A"], dtype=dtype, max_batch=2, max_seq_len=256)
    got = eng.generate_ids(prompts, 10, stop_ids=[])
    for p, g in zip(prompts, got):
        assert len(g) == 10
        seq = list(p)
        for t in g if dtype == "float32" else g[:4]:
            l = P.forward_logits(cfg, w, seq)[-1]
            if dtype == "float32":
                assert float(l.max() - l[t]) < 1e-3, "the chosen token is not the oracle's best"
            else:
                assert float(l.max() - l[t]) < 0.25, "bfloat16 chose a token far from the best"
            seq.append(t)
    eng.runner.cache.check()


def test_the_replay_program_on_a_model_folder(folders, tmp_path):
    vocab = CASES["B"][0]["vocab"]
    seqs = {"x": tokens(110, 80, vocab), "y": tokens(111, 30, vocab), "z": tokens(112, 1, vocab)}
    want = dict(zip(seqs, _oracle(folders["B"], list(seqs.values()))))
    steps, rows = [], {}
    steps.append({"step": 0, "entries": [{"id": "z", "tokens": seqs["z"], "want": [0]}], "end": ["z"]})
    rows[0] = [("z", 0)]
    steps.append({"step": 1, "entries": [{"id": "x", "tokens": seqs["x"][:70], "want": [0, 69]},
                                         {"id": "y", "tokens": seqs["y"][:25], "want": []}], "end": []})
    rows[1] = [("x", 0), ("x", 69)]
    for k in range(10):
        ents = [{"id": "x", "tokens": [seqs["x"][70 + k]], "want": [0]}]
        rws = [("x", 70 + k)]
        if k < 5:
            ents.append({"id": "y", "tokens": [seqs["y"][25 + k]], "want": [0] if k % 2 else []})
            if k % 2:
                rws.append(("y", 25 + k))
        steps.append({"step": 2 + k, "entries": ents, "end": (["y"] if k == 4 else []) + (["x"] if k == 9 else [])})
        rows[2 + k] = rws
    for dtype in ("float32", "bfloat16"):
        out = str(tmp_path / ("out_" + dtype))
        p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folders["B"], "--dtype", dtype, "--out", out,
                            "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps).encode(),
                           stdout=subprocess.PIPE, stderr=subprocess.PIPE, timeout=900)
        assert p.returncode == 0, p.stderr.decode()[-2000:]
        assert [l for l in p.stdout.decode().splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
        got, ref = [], []
        for n, rws in rows.items():
            got.append(torch.from_numpy(np.fromfile(os.path.join(out, f"{n}.f32"), dtype="<f4").reshape(len(rws), vocab).copy()))
            ref.append(torch.stack([want[i][pos] for i, pos in rws]))
        assert_rows(torch.cat(got), torch.cat(ref), dtype, "replayed steps")


def test_generation_through_the_command_line(folders):
    from plain import vagonex_plain as P
    cfg, w = oracle_view(folders["C"])
    prompt = tokens(120, 6, cfg["vocab"])
    p = subprocess.run([os.path.join(ROOT, "bin", "hos"), "-m", folders["C"], "--fp32", "--repeat-penalty", "1.0", "-n", "5",
                        "-p", ",".join(map(str, prompt))], stdout=subprocess.PIPE, stderr=subprocess.PIPE, timeout=900)
    assert p.returncode == 0, p.stderr.decode()[-2000:]
    ids = [int(t) for t in p.stdout.decode().strip().split(",")]
    assert ids[:len(prompt)] == prompt and len(ids) == len(prompt) + 5
    seq = list(prompt)
    for t in ids[len(prompt):]:
        l = P.forward_logits(cfg, w, seq)[-1]
        assert float(l.max() - l[t]) < 1e-3
        seq.append(t)


def test_the_two_attention_kernels_agree_in_bfloat16(folders):
    """The tensor-core kernel against the FMA kernel on the same bfloat16 model: a prompt, a piece, single tokens."""
    from hos_b200.parts.gated_attention import GatedSoftmaxAttention
    vocab = CASES["E"][0]["vocab"]
    seq = tokens(130, 400, vocab)
    outs = []
    for use in (True, False):
        GatedSoftmaxAttention.use_tensor_cores = use
        try:
            r = _runner(folders["E"], "bfloat16")
            (slot,) = r.admit(1)
            got = [r.step([slot], [seq[:310]], [list(range(0, 310, 3))]), r.step([slot], [seq[310:380]], [list(range(70))])]
            got += [r.step([slot], [[t]]) for t in seq[380:]]
            outs.append(torch.cat(got).cpu())
            r.release(slot)
        finally:
            GatedSoftmaxAttention.use_tensor_cores = True
    assert_rows(outs[0], outs[1], "bfloat16", "the two kernels")       # one more rounding (the queries), as far apart as
                                                                       # either is from the oracle at most


def test_the_kernels_alone_against_float64():
    """The attention kernel (one share and several) and the state scan (both rules) on random rows, without a model
    around them: keys and values of unequal sizes in a paged cache whose pages lie in no order."""
    from hos_b200 import ops
    from hos_b200.parts.base import StepInfo
    dev = "cuda"
    torch.manual_seed(3)
    n, H, G, kd, vd, scale, chunk = 333, 6, 2, 24, 40, 0.2, 150
    q = torch.randn(n, H, kd, device=dev)
    k, v = torch.randn(n, G, kd, device=dev), torch.randn(n, G, vd, device=dev)
    sink, gate = torch.randn(H, device=dev), torch.randn(n, H + 3, device=dev)
    pages = (n + 63) // 64
    order = torch.randperm(pages + 2)[:pages].to(torch.int32)
    kp, vp = torch.zeros(pages + 2, G, 64, kd, device=dev), torch.zeros(pages + 2, G, 64, vd, device=dev)
    for t in range(n):
        kp[order[t // 64], :, t % 64], vp[order[t // 64], :, t % 64] = k[t], v[t]
    cache = ops.PagedKVArgs(kp, vp, order.view(1, -1).to(dev).contiguous(), 0, G, kd, vd)
    pos = torch.arange(n, dtype=torch.int32, device=dev)
    zeros = torch.zeros(n, dtype=torch.int32, device=dev)
    step = StepInfo(n, 1, None, pos, zeros, torch.tensor([0, n], dtype=torch.int32, device=dev), zeros[:1], None, True, False, n, n)
    s = torch.einsum("ihd,jhd->hij", q.double().cpu(), k.double().cpu().repeat_interleave(H // G, 1)) * scale
    i, j = torch.arange(n)[:, None], torch.arange(n)[None]
    s = s.masked_fill(~((i >= j) & (i // chunk == j // chunk)), float("-inf"))
    p = torch.softmax(torch.cat([s, sink.double().cpu().view(H, 1, 1).expand(H, n, 1)], -1), -1)[..., :n]
    want = torch.einsum("hij,jhr->ihr", p, v.double().cpu().repeat_interleave(H // G, 1))
    want = want * torch.sigmoid(gate[:, 3:].double().cpu())[..., None]
    for splits in (1, 3, 7):
        out = torch.empty(n, H * vd, device=dev)
        ops.gated_attn(q, cache, sink, gate, 3, step, out, scale, chunk, 0, splits)
        assert float((out.cpu().double().view(n, H, vd) - want).abs().max()) < 2e-5, f"{splits} shares"
    # the tensor-core kernel: bfloat16 cache and output, three sequences of which one goes on from position 100, head
    # sizes 64/128 both ways round; its error is the rounding of q, k, v and of the output to bfloat16
    for kd2, vd2 in ((64, 128), (128, 64), (128, 128), (64, 64)):
        lens, starts = (150, 70, 3), (0, 100, 0)
        tot = [a + b for a, b in zip(lens, starts)]
        n2 = sum(lens)
        q2 = torch.randn(n2, H, kd2, device=dev)
        table, nxt = torch.zeros(3, 4, dtype=torch.int32), 1
        for sq, t in enumerate(tot):
            for e in range((t + 63) // 64):
                table[sq, e] = nxt
                nxt += 2                                   # pages lie apart
        kp2 = torch.zeros(nxt + 1, G, 64, kd2, device=dev, dtype=torch.bfloat16)
        vp2 = torch.zeros(nxt + 1, G, 64, vd2, device=dev, dtype=torch.bfloat16)
        ks = [torch.randn(t, G, kd2).to(torch.bfloat16) for t in tot]
        vs = [torch.randn(t, G, vd2).to(torch.bfloat16) for t in tot]
        def place(pages, rows, hd):
            for sq, r in enumerate(rows):
                for t in range(r.shape[0]):
                    for d0 in range(0, hd, 8):             # the cache's permutation of 16-byte groups
                        c = (d0 // 8) ^ (t % 64 % 8)
                        pages[table[sq, t // 64], :, t % 64, c * 8:c * 8 + 8] = r[t, :, d0:d0 + 8].to(dev)
        place(kp2, ks, kd2)
        place(vp2, vs, vd2)
        cache2 = ops.PagedKVArgs(kp2, vp2, table.to(dev), 0, G, kd2, vd2)
        pos2 = torch.cat([s0 + torch.arange(ln) for s0, ln in zip(starts, lens)]).to(torch.int32).to(dev)
        seq2 = torch.cat([torch.full((ln,), i) for i, ln in enumerate(lens)]).to(torch.int32).to(dev)
        cu2 = torch.tensor([0, 150, 220, 223], dtype=torch.int32, device=dev)
        gate2 = torch.randn(n2, H, device=dev)
        step2 = StepInfo(n2, 3, None, pos2, seq2, cu2, torch.arange(3, dtype=torch.int32, device=dev), None, False, False, 150, 170)
        want2, at = [], 0
        qb = q2.to(torch.bfloat16).double().cpu()
        for sq, (ln, s0) in enumerate(zip(lens, starts)):
            kk, vv = ks[sq].double().repeat_interleave(H // G, 1), vs[sq].double().repeat_interleave(H // G, 1)
            sc = torch.einsum("ihd,jhd->hij", qb[at:at + ln], kk) * scale
            ii, jj = (s0 + torch.arange(ln))[:, None], torch.arange(tot[sq])[None]
            sc = sc.masked_fill(~((ii >= jj) & (ii // chunk == jj // chunk)), float("-inf"))
            pr = torch.softmax(torch.cat([sc, sink.double().cpu().view(H, 1, 1).expand(H, ln, 1)], -1), -1)[..., :tot[sq]]
            want2.append(torch.einsum("hij,jhr->ihr", pr, vv) * torch.sigmoid(gate2[at:at + ln].double().cpu())[..., None])
            at += ln
        want2 = torch.cat(want2)
        out2 = torch.empty(n2, H * vd2, device=dev, dtype=torch.bfloat16)
        assert ops.gated_attn_mma(q2, cache2, sink, gate2, 0, step2, out2, scale, chunk, 0, 3 + 2 + 1)
        err = (out2.double().cpu().view(n2, H, vd2) - want2).abs().max()
        assert float(err) < 1e-2, f"tensor-core kernel, heads of {kd2}/{vd2}: {float(err):.2e}"
        ref = torch.empty(n2, H * vd2, device=dev, dtype=torch.bfloat16)
        ops.gated_attn(q2.to(torch.bfloat16).float(), cache2, sink, gate2, 0, step2, ref, scale, chunk, 0, 1)
        assert float((out2.float() - ref.float()).abs().max()) < 1e-2
        # single tokens on the tensor cores: the last token of each of the three sequences, one share and several
        last = [149, 219, 222]
        q1, g1 = q2[last].contiguous(), gate2[last].contiguous()
        step1 = StepInfo(3, 3, None, pos2[last].contiguous(), torch.arange(3, dtype=torch.int32, device=dev),
                         torch.arange(4, dtype=torch.int32, device=dev), torch.arange(3, dtype=torch.int32, device=dev), None,
                         False, True, 1, 170)
        for shares in (1, 2, 5):
            out1 = torch.empty(3, H * vd2, device=dev, dtype=torch.bfloat16)
            assert ops.gated_attn_mma_decode(q1, cache2, sink, g1, 0, step1, out1, scale, chunk, 0, shares)
            err = (out1.double().cpu().view(3, H, vd2) - want2[last]).abs().max()
            assert float(err) < 1e-2, f"single tokens, heads of {kd2}/{vd2}, {shares} shares: {float(err):.2e}"
    # the scans: two sequences in one step, the second resuming from a state
    for rule in ("decay", "delta"):
        Hh, Gk, d, vdim = 4, 2 if rule == "delta" else 4, 20, 12
        lens, cols = (37, 21), 2 * Gk * d + Hh * vdim
        rows = torch.randn(sum(lens), cols + 5, device=dev) * 0.5
        g = torch.rand(sum(lens), Hh, device=dev) if rule == "delta" else torch.rand(Hh, device=dev)
        beta = torch.rand(sum(lens), Hh, device=dev) if rule == "delta" else None
        state = torch.randn(3, Hh, vdim, d, device=dev)
        st0 = state.clone()
        pos = torch.cat([torch.arange(37), 9 + torch.arange(21)]).to(torch.int32).to(dev)
        seqid = torch.cat([torch.zeros(37), torch.ones(21)]).to(torch.int32).to(dev)
        step = StepInfo(58, 2, None, pos, seqid, torch.tensor([0, 37, 58], dtype=torch.int32, device=dev),
                        torch.tensor([2, 0], dtype=torch.int32, device=dev), None, False, False, 37, 37)
        out = torch.empty(58, Hh * vdim, device=dev)
        ops.state_scan(rows, 5, 5 + Gk * d, 5 + 2 * Gk * d, False, g, rule == "delta", beta, state, step, out, Hh, Gk, d, vdim)
        R = rows.double().cpu()
        at = 0
        for sq, (ln, slot, fresh) in enumerate(zip(lens, (2, 0), (True, False))):
            for h in range(Hh):
                S = torch.zeros(d, vdim, dtype=torch.float64) if fresh else st0[slot, h].double().cpu().T.clone()
                kh = h // (Hh // Gk)
                for t in range(at, at + ln):
                    qq, kk = R[t, 5 + kh * d:5 + (kh + 1) * d], R[t, 5 + (Gk + kh) * d:5 + (Gk + kh + 1) * d]
                    vv = R[t, 5 + 2 * Gk * d + h * vdim:5 + 2 * Gk * d + (h + 1) * vdim]
                    gt = float(g[t, h]) if rule == "delta" else float(g[h])
                    S = gt * S
                    u = float(beta[t, h]) * (vv - S.T @ kk) if rule == "delta" else vv
                    S = S + torch.outer(kk, u)
                    assert float((out[t, h * vdim:(h + 1) * vdim].cpu().double() - S.T @ qq).abs().max()) < 1e-4, rule
                assert float((state[slot, h].cpu().double().T - S).abs().max()) < 1e-4, rule
            at += ln
        assert torch.equal(state[1], st0[1]), "a slot that took no part was written"
