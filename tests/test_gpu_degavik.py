"""GPU tests of the Degavik family: the CUDA engine (through runtime.Model, i.e. the C ABI's infer / state / sampling entry
points and its own step packing) against the plain NumPy restatement in oracle/degavik_numpy.py, on small random models made
here.  precision 1 (every product in f32) is held to a tight bound, precision 0 (bf16 tensor-core products for multi-token
steps) to the restatement's own bf16 operand-rounding error.
"""
import json

import numpy as np
import pytest

from ai00_server_b200 import capi, runtime, synth
from oracle import degavik_numpy as D

pytestmark = pytest.mark.gpu

TIGHT = 2e-4        # f32 engine vs float64 oracle, relative to the logits' spread
L = synth.degavik_layer


def row_errs(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.sqrt(((want - want.mean(-1, keepdims=True)) ** 2).mean())


def err(got, want):
    return float(row_errs(got, want).max())


class Bundle:
    def __init__(self, layers, precision=1, slots=3, kv_tokens=2048, kv_page=16, seed=0, chunk=128, tweak=None, **kw):
        self.cfg_bytes, self.st, self.w = synth.make_degavik(layers, seed=seed, **kw)
        if tweak:                                   # planted weights: edit the rounded arrays, write them again
            tweak(self.w)
            self.st = synth.pack_st_bf16({k: np.asarray(v, np.float32) for k, v in self.w.items()})
            self.w = {k: v.astype(np.float64) for k, v in D.read_safetensors(bytes(self.st)).items()}
        self.cfg = json.loads(self.cfg_bytes)
        self.m = runtime.Model(self.st, max_batch=slots, token_chunk_size=chunk, precision=precision, config=self.cfg_bytes,
                               kv_tokens=kv_tokens, kv_page=kv_page)
        self.vocab = self.cfg["vocab"]

    def tokens(self, n, seed=0):
        return [int(t) for t in np.random.default_rng(seed).integers(0, self.vocab, n)]

    def oracle(self, toks, layers=False):
        return D.run(self.cfg, self.w, toks, layers=layers)

    def feed(self, slot, toks, opt=capi.OPTION_FULL):
        return self.m.infer_raw([slot], [len(toks)], list(toks), [opt])[0].copy()

    def close(self):
        self.m.close()


def bf16_floor(b, toks, want):
    """How far the restatement itself moves when every projection's activation operand is rounded to bfloat16: the yardstick
    for precision 0, whose multi-token steps round exactly those operands."""
    D.ROUND_OPERANDS = True
    try:
        return row_errs(b.oracle(toks), want)
    finally:
        D.ROUND_OPERANDS = False


def assert_serving(got, want, floor):
    """Typical rows sit at the rounding floor; a rare row may sit far above it where operand rounding flips a close router
    decision (the restatement's own rounded run has such rows too), so rows are counted, not maximised."""
    e = row_errs(got, want)
    assert np.median(e) <= 2.0 * np.median(floor)
    assert (e > 3.0 * floor.max()).sum() <= max(1, 0.02 * len(e))


STACK = [L("retention", mlp="dense"), L("channel_delta", kv_heads=2, mlp="moe"), L("attention", kv_heads=2, window=12, keep_first=3, mlp="moe"),
         L("channel_delta", kv_heads=2, mlp="moe", weights_of=1), L("attention", heads=2, kv_heads=1, window=5, keep_first=0, rot_dims=8, mlp=None)]


@pytest.fixture(scope="module")
def stack():
    b = Bundle(STACK)
    yield b
    b.close()


@pytest.fixture(scope="module")
def stack_ref(stack):
    toks = stack.tokens(150, 5)
    return toks, stack.oracle(toks)


# ---- each mechanism alone: one- or two-layer models, residual stream after every layer and logits ----
@pytest.mark.parametrize("layers", [
    [L("retention", mlp=None)],
    [L("retention", rot_dims=6, base=50.0, mlp=None)],
    [L("channel_delta", mlp=None)],
    [L("channel_delta", kv_heads=2, conv=4, mlp=None)],
    [L("attention", mlp=None)],
    [L("attention", kv_heads=1, rot_dims=4, softcap=2.0, window=3, keep_first=4, mlp=None)],
    [L("retention", mlp="dense")],
    [L("retention", mlp="moe", experts=6, top=3)],
    [L("retention", mlp="moe", shared_ff=0)],
    [L("attention", kv_heads=2, mlp="dense"), L("retention", mlp=None), L("attention", kv_heads=2, mlp="dense", weights_of=0)],
], ids=["retention", "retention-partial-rotation", "delta", "delta-shared-keys-4-taps", "attention", "attention-sharp-mask", "dense",
        "experts", "experts-no-shared", "shared-tensors-own-cache"])
def test_single_mechanisms(layers):
    b = Bundle(layers, seed=3)
    try:
        toks = b.tokens(37, 1)
        b.m.debug_read("layers_on", 1)
        got = b.feed(0, toks)
        want, lay = b.oracle(toks, layers=True)
        buf = np.empty(len(layers) * 128 * b.cfg["width"], np.float32)
        capi.check(capi.lib().b200rwkv_debug_read(b.m._h, b"layers", capi.ptr(buf), buf.size), b.m._h)
        buf = buf.reshape(len(layers), 128, -1)[:, :len(toks)]
        for i in range(len(layers)):
            assert np.abs(buf[i] - lay[i]).max() <= 1e-4 * max(1.0, np.abs(lay[i]).max()), i
        assert err(got, want) <= TIGHT
    finally:
        b.close()


def test_whole_prompt_and_first_tokens(stack, stack_ref):
    toks, want = stack_ref
    stack.m.state.reset(0)
    assert err(stack.feed(0, toks), want) <= TIGHT
    for n in (1, 2, 3):                                        # sequences of one to three tokens: empty tails, empty states
        stack.m.state.reset(1)
        assert err(stack.feed(1, toks[:n]), want[:n]) <= TIGHT


def test_prefill_against_token_by_token(stack, stack_ref):
    toks, want = stack_ref
    stack.m.state.reset(0)
    rows = np.concatenate([stack.feed(0, [t], capi.OPTION_LAST) for t in toks])
    assert err(rows, want) <= TIGHT


@pytest.mark.parametrize("cuts", [[2, 2, 3, 64, 5, 2, 31, 17, 16, 8], [15, 1, 1, 16, 17, 2, 98], [128, 22], [7] * 21 + [3], [1, 2] * 50])
def test_portions(stack, stack_ref, cuts):
    toks, want = stack_ref
    assert sum(cuts) == len(toks)
    stack.m.state.reset(0)
    out, at = [], 0
    for c in cuts:
        out.append(stack.feed(0, toks[at:at + c]))
        at += c
    assert err(np.concatenate(out), want) <= TIGHT


def test_unequal_batch_against_each_alone(stack):
    reqs = [stack.tokens(n, 10 + n) for n in (41, 1, 19)]
    want = [stack.oracle(r) for r in reqs]
    for s in range(3):
        stack.m.state.reset(s)
    rows = stack.m.infer_raw([0, 1, 2], [len(r) for r in reqs], [t for r in reqs for t in r], [capi.OPTION_FULL] * 3)
    for r, w in zip(rows, want):
        assert err(r, w) <= TIGHT
    nxt = [3, 4, 5]                                            # decode all three together: the rows do not depend on the company
    together = stack.m.infer_raw([0, 1, 2], [1, 1, 1], nxt, [capi.OPTION_LAST] * 3)
    for s in range(3):
        assert err(together[s], stack.oracle(reqs[s] + [nxt[s]])[-1:]) <= TIGHT
    # a prompt portion of one sequence beside single tokens of two others
    more = [stack.tokens(9, 77), [6], [7]]
    mixed = stack.m.infer_raw([1, 0, 2], [9, 1, 1], more[0] + more[1] + more[2], [capi.OPTION_FULL, capi.OPTION_LAST, capi.OPTION_LAST])
    assert err(mixed[0], stack.oracle(reqs[1] + [nxt[1]] + more[0])[-9:]) <= TIGHT
    assert err(mixed[1], stack.oracle(reqs[0] + [nxt[0]] + more[1])[-1:]) <= TIGHT
    assert err(mixed[2], stack.oracle(reqs[2] + [nxt[2]] + more[2])[-1:]) <= TIGHT


def test_pages_and_slots_reused():
    b = Bundle(STACK[:3], slots=2, kv_tokens=64, kv_page=8, seed=4)
    try:
        a, c = b.tokens(60, 1), b.tokens(50, 2)
        wa, wc = b.oracle(a), b.oracle(c)
        assert err(b.feed(0, a), wa) <= TIGHT
        with pytest.raises(capi.B200Error):                    # the pool is for 64 tokens (+ one partly filled page per slot)
            b.feed(1, c)
        b.m.state.reset(1)
        b.m.state.reset(0)                                     # pages go back, states and tails are cleared ...
        assert err(b.feed(1, c), wc) <= TIGHT                  # ... and are used again by another slot, in another order
        b.m.state.reset(1)
        assert err(b.feed(0, c[:9]), wc[:9]) <= TIGHT
        assert err(b.feed(1, a[:33]), wa[:33]) <= TIGHT        # two live sequences share the pool
        assert err(b.feed(0, c[9:40]), wc[9:40]) <= TIGHT
    finally:
        b.close()


def sharpen(w):
    """Peaked softmaxes: nearly all of a row's weight sits on one visible key, so a key lost or gained at an edge of the mask
    or a page changes the row completely."""
    for k in w:
        if k.endswith("mix.temp"):
            w[k] = np.full_like(w[k], 7.0)


@pytest.mark.parametrize("window,keep", [(16, 0), (16, 5), (17, 16), (33, 2), (1, 1), (7, 40)])
def test_window_edges_kept_tokens_and_page_borders(window, keep):
    layers = [L("attention", heads=2, kv_heads=1, window=window, keep_first=keep, softcap=40.0, mlp=None),
              L("attention", heads=4, kv_heads=4, window=window, keep_first=keep, softcap=0.0, mlp="dense")]
    b = Bundle(layers, kv_page=16, seed=6, tweak=sharpen)
    try:
        toks = b.tokens(120, 3)
        want = b.oracle(toks)
        b.m.state.reset(0)
        assert err(b.feed(0, toks), want) <= TIGHT             # in a prompt
        b.m.state.reset(1)
        out = [b.feed(1, toks[:13])]
        for i in range(13, 70):                                # decoded alone across the window's first slide, the kept tokens' end
            out.append(b.feed(1, [toks[i]], capi.OPTION_LAST))  # and the page borders at 16, 32, 48, 64
        out.append(b.feed(1, toks[70:73]))
        out.append(b.feed(1, toks[73:]))                       # portions that start and end inside pages and windows
        assert err(np.concatenate(out), want) <= TIGHT
    finally:
        b.close()


def test_a_kept_first_token_carries_the_row():
    # one head, queries and keys made so that key 1 (a kept token) outscores every key of the window by a wide margin at every
    # later position: leaving the kept tokens out, or moving them, changes every row
    def plant(w):
        sharpen(w)
        w["l0.mix.talk"] = np.ones((1, 1))
    b = Bundle([L("attention", heads=1, kv_heads=1, dim=16, rot_dims=0, window=6, keep_first=2, softcap=0.0, scale=1.0, mlp=None)], seed=11,
               vocab=8, tweak=plant)
    try:
        toks = [0, 1] + [int(t) for t in np.random.default_rng(1).integers(2, 8, 300)]
        c, p = b.cfg["layers"][0]["mixer"], "l0.mix."
        mem = {}
        for t, tok in enumerate(toks):
            D.attention(b.w, p, c, 1e-5, b.w["embed"][tok], mem, t)
        K = np.stack([k[0] for k in mem["k"]])
        wins = 0
        for t in range(10, 302):
            q = D.rms((b.w[p + "q"] @ b.w["embed"][toks[t]])[None], 1e-5)[0] * b.w[p + "q.norm"]
            s = K[: t + 1] @ q
            wins += int(np.argmax(np.where([D.visible(t, j, 6, 2) for j in range(t + 1)], s, -np.inf)) < 2)
        assert wins > 40                                       # the inputs do what the test needs: many rows hang on a kept key
        want = b.oracle(toks)
        b.m.state.reset(0)
        assert err(b.feed(0, toks), want) <= TIGHT
        b.m.state.reset(1)
        b.feed(1, toks[:250], capi.OPTION_NONE)
        rows = np.concatenate([b.feed(1, [t], capi.OPTION_LAST) for t in toks[250:]])
        assert err(rows, want[250:]) <= TIGHT
    finally:
        b.close()


def test_far_tokens_through_slow_decays():
    # retention heads that forget nothing for hundreds of tokens and delta-rule channels with decays next to one: the last rows
    # depend on the first tokens through the recurrent states only
    def slow(w):
        for k in w:
            if k.endswith("mix.dt_bias"):
                w[k] = np.full_like(w[k], -9.0)
    layers = [L("retention", heads=2, decay=[1.0, 0.9995], mlp=None), L("channel_delta", heads=2, mlp=None)]
    b = Bundle(layers, seed=12, tweak=slow)
    try:
        toks = b.tokens(420, 2)
        want = b.oracle(toks)
        other = b.oracle([toks[0] ^ 1] + toks[1:])
        assert err(other[-5:], want[-5:]) > 50 * TIGHT         # the first token still shows at the end
        b.m.state.reset(0)
        assert err(b.feed(0, toks), want) <= TIGHT
        b.m.state.reset(1)
        b.feed(1, toks[:300], capi.OPTION_NONE)
        rows = np.concatenate([b.feed(1, [t], capi.OPTION_LAST) for t in toks[300:]])
        assert err(rows, want[300:]) <= TIGHT
    finally:
        b.close()


def test_long_decoding(stack):
    toks = stack.tokens(200, 9)
    want = stack.oracle(toks)
    stack.m.state.reset(0)
    out = [stack.feed(0, toks[:60])] + [stack.feed(0, [t], capi.OPTION_LAST) for t in toks[60:]]
    assert err(np.concatenate(out), want) <= TIGHT


ODD = [L("retention", heads=3, dim=10, vdim=20, rot_dims=6, mlp="moe", experts=3, top=3, ff=10, shared_ff=14),
       L("channel_delta", heads=6, kv_heads=2, dim=6, vdim=12, conv=1, mlp="moe", experts=1, top=1, ff=7, shared_ff=0),
       L("attention", heads=1, kv_heads=1, dim=8, vdim=5, rot_dims=2, window=1, keep_first=1, mlp=None),
       L("channel_delta", heads=1, kv_heads=1, dim=40, vdim=33, conv=5, mlp="dense", ff=9),
       L("attention", heads=6, kv_heads=3, dim=6, vdim=10, rot_dims=6, window=200, keep_first=0, softcap=0.0, mlp="moe", experts=9, top=4, ff=5,
         shared_ff=3),
       L("retention", heads=1, dim=34, vdim=66, rot_dims=0, decay=[0.5], mlp="dense", ff=3)]


@pytest.mark.parametrize("precision", [1, 0])
def test_other_sizes(precision):
    b = Bundle(ODD, precision=precision, width=50, vocab=61, seed=7, low_rank=3)
    try:
        toks = b.tokens(90, 4)
        want = b.oracle(toks)
        got = np.concatenate([b.feed(0, toks[:70]), b.feed(0, toks[70:72])] + [b.feed(0, [t], capi.OPTION_LAST) for t in toks[72:]])
        if precision == 1:
            assert err(got, want) <= TIGHT
        else:
            assert_serving(got, want, bf16_floor(b, toks, want))
    finally:
        b.close()


WIDE = [L("attention", heads=8, kv_heads=2, dim=64, vdim=64, rot_dims=32, window=48, keep_first=4, mlp="moe", experts=8, top=2, ff=64, shared_ff=96),
        L("channel_delta", heads=4, kv_heads=2, dim=64, vdim=128, conv=4, mlp="dense", ff=320),
        L("retention", heads=4, dim=64, vdim=64, mlp="dense", ff=320)]


@pytest.mark.parametrize("precision", [1, 0])
def test_wider_layers(precision):
    b = Bundle(WIDE, precision=precision, width=256, vocab=300, seed=5, low_rank=16)
    try:
        toks = b.tokens(140, 6)
        want = b.oracle(toks)
        got = np.concatenate([b.feed(0, toks[:100])] + [b.feed(0, [t], capi.OPTION_LAST) for t in toks[100:120]] + [b.feed(0, toks[120:])])
        if precision == 1:
            assert err(got, want) <= TIGHT
        else:
            assert_serving(got, want, bf16_floor(b, toks, want))
    finally:
        b.close()


def test_serving_precision(stack_ref):
    toks, want = stack_ref
    b = Bundle(STACK, precision=0)
    try:
        floor = bf16_floor(b, toks, want)
        assert_serving(b.feed(0, toks), want, floor)
        b.m.state.reset(0)
        out = [b.feed(0, toks[:50])] + [b.feed(0, [t], capi.OPTION_LAST) for t in toks[50:90]] + [b.feed(0, toks[90:])]
        assert_serving(np.concatenate(out), want, floor)
    finally:
        b.close()


def test_steps_of_up_to_512_tokens(stack_ref):
    toks, want = stack_ref
    b = Bundle(STACK, chunk=512)
    try:
        long = toks + b.tokens(350, 8)
        assert err(b.feed(0, long), b.oracle(long)) <= TIGHT
    finally:
        b.close()


def test_greedy_generation_through_the_runtime(stack):
    # the framework's own entry point: Runtime.infer (its token budget and slot batching) + the GPU sampling front half
    prompt = stack.tokens(21, 12)
    mem = D.new_memory(stack.cfg)
    row = D.run(stack.cfg, stack.w, prompt, mem=mem)[-1]
    want = []
    for _ in range(12):
        want.append(int(row.argmax()))
        row = D.run(stack.cfg, stack.w, [want[-1]], mem=mem)[-1]
    stack.m.state.reset(0)
    inp = runtime.RnnInput([runtime.RnnInputBatch(list(prompt), runtime.RnnOption.Last)], token_chunk_size=8)
    got = []
    while len(got) < 12:
        inp, out = stack.m.runtime.infer(inp)
        if out[0].is_empty():
            continue
        ids, probs = stack.m.sample_topk([0], top_k=4)
        assert int(ids[0, 0]) == int(out[0].data[0].argmax())
        got.append(int(ids[0, 0]))
        inp = runtime.RnnInput([runtime.RnnInputBatch([got[-1]], runtime.RnnOption.Last)], token_chunk_size=8)
    assert got == want


def test_state_snapshots_and_host_round_trip(stack, stack_ref):
    toks, want = stack_ref
    m = stack.m
    m.state.reset(0)
    stack.feed(0, toks[:50], capi.OPTION_LAST)
    snap = m.state.read(0)
    host = m.state.back(0)
    assert int(host.reshape(-1)[0]) == 50
    a = stack.feed(0, toks[50:90])
    m.state.write(snap, 1)                                     # device snapshot into another slot
    b_ = stack.feed(1, toks[50:90])
    m.state.load(host, 2)                                      # host tensor into a third
    c = stack.feed(2, toks[50:90])
    assert err(a, want[50:90]) <= TIGHT
    assert np.array_equal(a, b_) and np.array_equal(a, c)
    snap.free()
