"""GPU tests of the Kemirax family: the CUDA engine (through runtime.Model, i.e. the C ABI's infer / state / sampling entry
points and its own step packing) against the plain NumPy restatement in oracle/kemirax_numpy.py, on small random models
made here.  precision 1 (every product in f32) is held to a tight bound, precision 0 (bf16 tensor-core products for
multi-token steps) to three times the restatement's own bf16 operand-rounding error.
"""
import json

import numpy as np
import pytest

from ai00_server_b200 import capi, runtime, synth
from oracle import kemirax_numpy as K

pytestmark = pytest.mark.gpu

TIGHT = 2e-4        # f32 engine vs float64 oracle, relative to the logits' spread

YARN = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}
LA = synth.kemirax_layer


def row_errs(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.sqrt(((want - want.mean(-1, keepdims=True)) ** 2).mean())


def err(got, want):
    return float(row_errs(got, want).max())


def bf16_floor(b, toks, want):
    """Per row, how far the restatement itself moves when every projection's activation operand is rounded to bfloat16: the
    yardstick for precision 0, whose multi-token steps round exactly those operands (its one-token steps round nothing)."""
    K.ROUND_OPERANDS = True
    try:
        return row_errs(b.oracle(toks), want)
    finally:
        K.ROUND_OPERANDS = False


def assert_serving(got, want, floor):
    """Typical rows sit at the rounding floor; a rare row may sit far above it, where operand rounding flips a close router
    decision (the restatement's own rounded run has such rows too, at other places), so rows are counted, not maximised."""
    e = row_errs(got, want)
    assert np.median(e) <= 2.0 * np.median(floor)
    assert (e > 3.0 * floor.max()).sum() <= max(1, 0.02 * len(e))


class Bundle:
    def __init__(self, layers, precision=1, slots=3, kv_tokens=2048, kv_page=16, seed=0, chunk=128, **kw):
        self.cfg_bytes, self.st, self.w = synth.make_kemirax(layers, seed=seed, **kw)
        self.cfg = json.loads(self.cfg_bytes)
        self.m = runtime.Model(self.st, max_batch=slots, token_chunk_size=chunk, precision=precision, config=self.cfg_bytes,
                               kv_tokens=kv_tokens, kv_page=kv_page)
        self.vocab = self.cfg["vocab"]

    def tokens(self, n, seed=0):
        return [int(t) for t in np.random.default_rng(seed).integers(0, self.vocab, n)]

    def oracle(self, toks, layers=False):
        return K.run(self.cfg, self.w, toks, layers=layers)

    def feed(self, slot, toks, opt=capi.OPTION_FULL):
        return self.m.infer_raw([slot], [len(toks)], list(toks), [opt])[0].copy()

    def close(self):
        self.m.close()


STACK = [LA("latent_attention", scaling=YARN), LA("latent_attention", kv_from=0, scaling=YARN), LA("gla"),
         LA("latent_attention", heads=2, kv_rank=16, rot_dim=4, q_rank=12)]


@pytest.fixture(scope="module")
def stack():
    b = Bundle(STACK)
    yield b
    b.close()


@pytest.fixture(scope="module")
def stack_ref(stack):
    toks = stack.tokens(150, 5)
    return toks, stack.oracle(toks)


# ---- each mechanism alone: one-layer models, residual stream after the layer and logits ----
@pytest.mark.parametrize("layers", [
    [LA("latent_attention", mlp=False)],
    [LA("latent_attention", mlp=False, scaling=YARN, base=500.0)],
    [LA("gla", mlp=False)],
    [LA("gla", mlp=True, shared_ff=0, identity=0)],
    [LA("latent_attention", mlp=True, identity=2, top=3, experts=5)],
    [LA("latent_attention", mlp=False), LA("latent_attention", mlp=False, kv_from=0)],
], ids=["latent", "latent-yarn", "gla", "gla+experts", "latent+experts+identity", "borrowed-cache"])
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
    for n in (1, 2, 3):                       # the first tokens of a sequence: zero shift row, one-key softmax
        stack.m.state.reset(1)
        assert err(stack.feed(1, toks[:n]), want[:n]) <= TIGHT


def test_prefill_against_token_by_token(stack, stack_ref):
    toks, want = stack_ref
    stack.m.state.reset(0)
    rows = [stack.feed(0, [t], capi.OPTION_LAST) for t in toks[:70]]
    assert err(np.concatenate(rows), want[:70]) <= TIGHT


@pytest.mark.parametrize("cuts", [[2, 2, 3, 64, 5, 2, 31, 17, 16, 8], [15, 1, 1, 16, 17, 2, 98], [128, 22], [7] * 21 + [3]])
def test_portions(stack, stack_ref, cuts):
    toks, want = stack_ref
    assert sum(cuts) == len(toks)
    stack.m.state.reset(2)
    out, at = [], 0
    for c in cuts:
        out.append(stack.feed(2, toks[at:at + c]))
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
    # decode all three together, then one alone: the rows do not depend on the company
    nxt = [3, 4, 5]
    together = stack.m.infer_raw([0, 1, 2], [1, 1, 1], nxt, [capi.OPTION_LAST] * 3)
    for s in range(3):
        w = stack.oracle(reqs[s] + [nxt[s]])[-1:]
        assert err(together[s], w) <= TIGHT


def test_pages_and_slots_reused():
    b = Bundle(STACK[:3], slots=2, kv_tokens=64, kv_page=8, seed=4)
    try:
        a, c = b.tokens(60, 1), b.tokens(50, 2)
        wa, wc = b.oracle(a), b.oracle(c)
        assert err(b.feed(0, a), wa) <= TIGHT
        with pytest.raises(capi.B200Error):                    # the pool is for 64 tokens (+ one partly filled page per slot)
            b.feed(1, c)
        b.m.state.reset(1)
        b.m.state.reset(0)                                     # pages go back ...
        assert err(b.feed(1, c), wc) <= TIGHT                  # ... and are used again by another slot, in another order
        b.m.state.reset(1)
        assert err(b.feed(0, c[:9]), wc[:9]) <= TIGHT
        assert err(b.feed(1, a[:33]), wa[:33]) <= TIGHT        # two live sequences share the pool
        assert err(b.feed(0, c[9:40]), wc[9:40]) <= TIGHT
    finally:
        b.close()


def test_page_borders_and_far_keys():
    # sharp attention (large score scale): a few keys carry each softmax, so a key dropped at a page border or far back shows
    layers = [LA("latent_attention", scale=1.5, mlp=False), LA("latent_attention", scale=1.5, kv_from=0)]
    b = Bundle(layers, kv_page=16, seed=6)
    try:
        toks = b.tokens(330, 3)
        want = b.oracle(toks)
        b.m.state.reset(0)
        out = [b.feed(0, toks[:15])]
        for i in range(15, 50):                                # decode across the borders at 16, 32, 48
            out.append(b.feed(0, [toks[i]], capi.OPTION_LAST))
        out.append(b.feed(0, toks[50:]))                       # portions that start and end inside pages
        assert err(np.concatenate(out), want) <= TIGHT
        b.m.state.reset(1)
        assert err(b.feed(1, toks), want) <= TIGHT
    finally:
        b.close()


def last_row_attention(cfg, w, toks):
    """Softmax weights of the last token's only head over all keys, for a model whose FIRST layer is latent attention with
    one head (its query depends on the last two embeddings only)."""
    seq = K.Sequence(cfg)
    K.run(cfg, w, toks, seq)
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]

    def normed(t):
        return K.rms_unit(w["embed"][t], eps) * float(w["l0.norm1"])
    h, hp = normed(toks[-1]), normed(toks[-2])
    hs = h + (hp - h) * w["l0.shift"]
    q = w["l0.mix.uq"] @ (K.rms_unit(w["l0.mix.dq"] @ hs, eps) * w["l0.mix.dq.norm"])
    dn = m["dim"]
    C = np.stack([e[0] for e in seq.cache[0]])
    KR = np.stack([e[1] for e in seq.cache[0]])
    s = ((C @ w["l0.mix.uk"].T) @ q[:dn] + KR @ K.rotate(q[dn:], len(toks) - 1, m["rot"])) * m["scale"]
    return K.softmax(s)


def test_far_key_stands_out():
    # a sharp one-head attention whose last row puts nearly all its weight on ONE key hundreds of tokens back: losing that
    # key (a wrong page, a wrong split of the context) changes the row completely
    b = Bundle([LA("latent_attention", heads=1, mlp=False, scale=1.0)], seed=8)
    try:
        toks = b.tokens(400, 4)
        p = last_row_attention(b.cfg, b.w, toks)
        far = int(np.argmax(p))
        assert far < 150 and p[far] > 0.9                      # the inputs do what the test needs
        want = b.oracle(toks)
        b.m.state.reset(0)
        assert err(b.feed(0, toks), want) <= TIGHT
        b.m.state.reset(1)                                     # the same row decoded alone after a chunked prompt
        b.feed(1, toks[:200], capi.OPTION_NONE)
        b.feed(1, toks[200:399], capi.OPTION_NONE)
        assert err(b.feed(1, toks[399:], capi.OPTION_LAST), want[399:]) <= TIGHT
    finally:
        b.close()


def test_long_decoding(stack):
    toks = stack.tokens(200, 9)
    want = stack.oracle(toks)
    stack.m.state.reset(0)
    out = [stack.feed(0, toks[:60])] + [stack.feed(0, [t], capi.OPTION_LAST) for t in toks[60:]]
    assert err(np.concatenate(out), want) <= TIGHT


ODD = [LA("latent_attention", heads=3, dim=12, vdim=20, rot_dim=6, kv_rank=20, q_rank=12, experts=3, identity=2, top=3, ff=10, shared_ff=14),
       LA("gla", heads=5, dim=6, vdim=12, experts=1, identity=0, top=1, ff=7, shared_ff=0),
       LA("latent_attention", heads=1, dim=8, vdim=8, rot_dim=2, kv_rank=33, q_rank=9, mlp=False),
       LA("gla", heads=1, dim=40, vdim=33, tau=1.0, experts=9, identity=1, top=4, ff=5, shared_ff=3)]


LARGE = [LA("latent_attention", heads=20, dim=16, vdim=16, rot_dim=8, kv_rank=512, q_rank=64, experts=6, identity=2, top=4, ff=40, shared_ff=72),
         LA("gla", heads=2, dim=64, vdim=128, mlp=False),
         LA("latent_attention", heads=20, dim=16, vdim=16, rot_dim=8, kv_rank=512, q_rank=64, kv_from=0, mlp=False)]


@pytest.mark.parametrize("precision", [1, 0])
def test_largest_latent_and_many_heads(precision):
    # the largest latent the attention kernels take (16 channel chunks per lane / 16 output tiles per warp), a head count that
    # fills one head group and part of a second, a recurrent state of 32 KB per head
    b = Bundle(LARGE, precision=precision, width=128, vocab=64, seed=19, gain=0.6)
    try:
        toks = b.tokens(44, 9)
        want = b.oracle(toks)
        got = np.concatenate([b.feed(0, toks[:35])] + [b.feed(0, [t], capi.OPTION_LAST) for t in toks[35:]])
        if precision:
            assert err(got, want) <= TIGHT
        else:
            assert_serving(got, want, bf16_floor(b, toks, want))
    finally:
        b.close()


UNALIGNED = [LA("latent_attention", heads=2, dim=5, vdim=3, rot_dim=2, kv_rank=10, q_rank=7, experts=2, identity=1, top=2, ff=3, shared_ff=5),
             LA("gla", heads=3, dim=5, vdim=3, experts=3, identity=0, top=1, ff=9, shared_ff=0),
             LA("latent_attention", heads=2, dim=5, vdim=3, rot_dim=2, kv_rank=10, q_rank=7, kv_from=0, mlp=False)]


@pytest.mark.parametrize("precision", [1, 0])
def test_sizes_that_align_with_nothing(precision):
    # width, ranks and vocabulary that are no multiple of 4 or 8: every vector path has to fall back to its scalar form
    b = Bundle(UNALIGNED, precision=precision, width=50, vocab=37, seed=17, a_rank=3)
    try:
        toks = b.tokens(41, 8)
        want = b.oracle(toks)
        got = np.concatenate([b.feed(0, toks[:18])] + [b.feed(0, [t], capi.OPTION_LAST) for t in toks[18:24]] + [b.feed(0, toks[24:])])
        if precision:
            assert err(got, want) <= TIGHT
        else:
            assert_serving(got, want, bf16_floor(b, toks, want))
    finally:
        b.close()


@pytest.mark.parametrize("precision", [1, 0])
def test_other_sizes(precision):
    b = Bundle(ODD, precision=precision, width=72, vocab=101, seed=11, a_rank=5, eps=1e-3)
    try:
        toks = b.tokens(45, 2)
        want = b.oracle(toks)
        whole = b.feed(0, toks)
        cut = np.concatenate([b.feed(1, toks[:9])] + [b.feed(1, [t], capi.OPTION_LAST) for t in toks[9:20]] + [b.feed(1, toks[20:])])
        if precision:
            assert err(whole, want) <= TIGHT and err(cut, want) <= TIGHT
        else:
            floor = bf16_floor(b, toks, want)
            assert_serving(whole, want, floor)
            assert_serving(cut, want, floor)
    finally:
        b.close()


WIDE = [LA("latent_attention", heads=4, dim=32, rot_dim=16, vdim=32, kv_rank=64, q_rank=96, experts=4, top=2, ff=48, shared_ff=64),
        LA("gla", heads=4, dim=32, vdim=32, experts=4, top=2, ff=48, shared_ff=64)]


@pytest.mark.parametrize("precision", [1, 0])
def test_wide_rows_split_the_reduction(precision):
    # a width at which multi-token projections split their k range over several CTAs and add the parts in a second launch
    b = Bundle(WIDE, precision=precision, width=640, vocab=128, seed=13, gain=0.7)
    try:
        toks = b.tokens(40, 6)
        want = b.oracle(toks)
        got = np.concatenate([b.feed(0, toks[:33]), b.feed(0, toks[33:35]), b.feed(0, toks[35:])])
        if precision:
            assert err(got, want) <= TIGHT
        else:
            assert_serving(got, want, bf16_floor(b, toks, want))
    finally:
        b.close()


@pytest.mark.parametrize("precision", [1, 0])
def test_steps_of_up_to_512_tokens(precision, stack_ref):
    # token_chunk_size 512: a 150-token prompt is one step, a 330-token prompt one step of the largest bucket
    b = Bundle(STACK, precision=precision, chunk=512)
    try:
        toks, want = stack_ref
        long = b.tokens(330, 21)
        want_long = b.oracle(long)
        got = b.feed(0, toks)
        got_long = np.concatenate([b.feed(1, long[:300]), b.feed(1, long[300:])])
        rows = b.m.infer_raw([0, 2], [1, 140], [5] + long[:140], [capi.OPTION_LAST, capi.OPTION_FULL])       # a mixed step
        if precision:
            assert err(got, want) <= TIGHT and err(got_long, want_long) <= TIGHT
            assert err(rows[1], want_long[:140]) <= TIGHT
            assert err(rows[0], b.oracle(toks + [5])[-1:]) <= TIGHT
        else:
            assert_serving(got, want, bf16_floor(b, toks, want))
            assert_serving(got_long, want_long, bf16_floor(b, long, want_long))
    finally:
        b.close()


def test_serving_precision(stack_ref):
    b = Bundle(STACK, precision=0)
    try:
        toks, want = stack_ref
        floor = bf16_floor(b, toks, want)
        assert 1e-4 < np.median(floor) < 0.1
        assert_serving(b.feed(0, toks), want, floor)
        out = [b.feed(1, toks[:37])] + [b.feed(1, [t], capi.OPTION_LAST) for t in toks[37:60]] + [b.feed(1, toks[60:])]
        assert_serving(np.concatenate(out), want, floor)
    finally:
        b.close()


def test_greedy_generation_through_the_runtime(stack):
    # the framework's own entry point: Runtime.infer (its token budget and slot batching) + the GPU sampling front half
    prompt = stack.tokens(21, 12)
    seq = K.Sequence(stack.cfg)
    row = K.run(stack.cfg, stack.w, prompt, seq)[-1]
    want = []
    for _ in range(12):
        want.append(int(row.argmax()))
        row = K.run(stack.cfg, stack.w, [want[-1]], seq)[-1]
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
    back, _ = m.state.snapshot_back(snap, with_logits=True)
    assert np.array_equal(back, host)
    snap2 = m.state.snapshot_load(host)
    m.state.write(snap2, 1)
    assert np.array_equal(stack.feed(1, toks[50:90]), a)
    snap.free()
    snap2.free()
