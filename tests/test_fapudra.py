"""Fapudra on the device against the plain implementation (tests/plain_fapudra.py): each mechanism
alone (with weights and inputs made so that a lost key, a window or a kept token that is one off, a
wrong distance bucket or a lost state shows), then whole models replayed through bin/trace_run (whole
prompts, the last tokens one by one, portions down to two tokens, mixed batches on a pool so small
that pages and slots are used again), then greedy generation through the engine's entry point and
scheduler."""
import math
import os

import numpy as np
import pytest
import torch

import fapudra_tools as ft
import plain_fapudra as P
import trace_tools as tt
from mixer_tools import MixerRun, bf, close, ctx_for, cuts_of, make_kit

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def kit(cuda_device):
    return make_kit()


def npw(w, prefix="p."):
    """Torch weights -> the plain implementation's float64 arrays under a prefix."""
    return {prefix + k: v.double().numpy() for k, v in w.items()}


def plain(f, x, *args):
    return torch.from_numpy(f(x.double().numpy(), *args))


def taps_of(g, channels, taps):
    t = torch.randn(channels, taps, generator=g) / taps
    t[:, -1] += 1.0
    return t


# ------------------------------------------------------------------ small kernels
@pytest.mark.parametrize("dtype", DTYPES)
def test_scalar_norm_positions_and_capped_logits(kit, dtype):
    """An RMS norm whose weight is one number; embedded rows times a constant plus a row of the position
    table; logits capped by a tanh."""
    torch.manual_seed(0)
    T, W, eps = 13, 100, 3e-6
    x = torch.randn(T, W) * 3
    norm = kit.parts.build_norm(kit.parts.PartSpec("rmsnorm", {"size": W, "eps": eps, "scalar": True}), ctx_for(kit, dtype))
    assert {k: tuple(s.shape) for k, s in norm.weights().items()} == {"": ()}
    norm.load(lambda n: torch.tensor(1.375).cuda().to(dtype))
    resid = x.clone().cuda()
    out = torch.empty(T, W, device="cuda", dtype=dtype)
    norm.add_norm(resid, None, out)
    close(out, P.unit_rms(x.double().numpy(), eps) * 1.375, dtype, bf16=5e-3)
    table = bf(torch.randn(50, W)).float()
    pos = torch.randint(0, 50, (T,), dtype=torch.int32)
    resid = x.clone().cuda()
    kit.ops.scale_add_rows(resid, 3.5, table.cuda().to(dtype), pos.cuda())
    close(resid, x.double() * 3.5 + table.double()[pos.long()], torch.float32, f32=1e-6)
    z = (torch.randn(T, W) * 20).cuda()
    want = 12.0 * torch.tanh(z.double().cpu() / 12.0)
    kit.ops.softcap(z, 12.0)
    close(z, want, torch.float32, f32=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_sigmoid_gate(kit, dtype):
    torch.manual_seed(1)
    T, W = 9, 72
    a, wide = torch.randn(T, W), bf(torch.randn(T, W + 24) * 3)
    out = torch.empty(T, W, device="cuda", dtype=dtype)
    kit.ops.sigmoid_gate(a.cuda(), wide.cuda().to(dtype)[:, 16:16 + W], out)
    close(out, a.double() * torch.sigmoid(wide[:, 16:16 + W]), dtype, bf16=5e-3)


# ------------------------------------------------------------------ the state-space mixer
def ssm_weights(D, m, seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    H, Pv, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner, ch = H * Pv, H * Pv + 2 * G * N
    w = {"in": r(2 * inner + 2 * G * N + H, D) * 1.5 / D ** 0.5, "conv": taps_of(g, ch, taps), "conv.b": 0.2 * r(ch),
         "dt_bias": 0.5 * r(H), "A_log": r(H) - 1.0, "D": 1 + 0.2 * r(H), "norm": 1 + 0.2 * r(inner),
         "o": r(D, inner) / inner ** 0.5}
    return {k: bf(v) for k, v in w.items()}


def ssm_mixer(kit, dtype, D, m, eps, page=16, shift=False):
    inner = kit.parts.PartSpec("mamba2", {"hidden_size": D, "num_heads": m["heads"], "v_head_dim": m["vdim"],
                                          "state": m["state"], "groups": m["groups"], "conv": m["conv"],
                                          "norm_groups": m["norm_groups"], "eps": eps})
    if shift:
        inner = kit.parts.PartSpec("token_shift", {"hidden_size": D, "inner": inner, "inner_prefix": "mix.", "name": "shift"})
    return kit.parts.build_mixer(inner, ctx_for(kit, dtype, page))


TWO = [{"a": (0, 9), "b": (0, 2)}, {"a": (9, 10)}, {"b": (2, 19), "a": (10, 11)}, {"a": (11, 12), "b": (19, 20)},
       {"a": (12, 60), "b": (20, 41)}, {"a": (60, 75)}]

# width, heads, values, state, groups, taps, norm parts
SSM_SHAPES = [(64, 4, 16, 24, 2, 4, 2), (96, 8, 16, 32, 4, 3, 4), (100, 5, 12, 20, 5, 5, 1), (72, 3, 20, 8, 1, 1, 3),
              (128, 2, 64, 128, 1, 4, 1), (80, 2, 24, 200, 2, 2, 2),
              # values in multiples of 32 a head (a thread of the recurrence then holds two columns) with small and odd states
              (64, 3, 32, 16, 1, 3, 1), (96, 2, 96, 48, 2, 4, 2)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", SSM_SHAPES)
def test_state_space_mixer_in_portions_and_token_by_token(kit, dtype, shape):
    """The whole sequence in one step, in portions down to two tokens (shorter than the convolution's
    window), token by token, and two sequences beside each other: the state matrices and the
    convolution's last inputs carry over in the request's slot.  Groups of heads share B and C; the
    gated output is normed in parts."""
    D, H, Pv, N, G, taps, parts = shape
    eps = 1e-5
    m = {"heads": H, "vdim": Pv, "state": N, "groups": G, "conv": taps, "norm_groups": parts}
    mixer = ssm_mixer(kit, dtype, D, m, eps)
    w = ssm_weights(D, m, seed=41)
    assert set(mixer.weights()) == set(w)
    mixer.load(lambda n: w[n].cuda().to(dtype))
    g = torch.Generator().manual_seed(42)
    xa, xb = bf(torch.randn(75, D, generator=g)), bf(torch.randn(41, D, generator=g))
    wa, wb = plain(P.mamba2, xa, npw(w), "p.", m, eps), plain(P.mamba2, xb, npw(w), "p.", m, eps)
    tol = dict(f32=1e-4, bf16=3e-2)
    run = MixerRun(kit, mixer, dtype, 16)
    close(run.feed(xa, [75], "whole"), wa, dtype, **tol)
    close(run.feed(xa, cuts_of(75, [2, 3, 2, 17, 5, 2, 30]), "cut"), wa, dtype, **tol)
    close(run.feed(xa, [1] * 75, "single"), wa, dtype, **tol)
    got = MixerRun(kit, mixer, dtype, 16).plan({"a": xa, "b": xb}, TWO)
    close(got["a"], wa, dtype, **tol)
    close(got["b"], wb, dtype, **tol)


@pytest.mark.parametrize("dtype", DTYPES)
def test_state_space_mixer_remembers_far_back_and_slots_start_clean(kit, dtype):
    """A head that barely decays keeps what a loud token wrote hundreds of tokens ago.  Then the
    slot is given back and used by another request, which must see none of it, also when its first
    portion is a single token."""
    D, eps = 64, 1e-5
    m = {"heads": 2, "vdim": 16, "state": 16, "groups": 1, "conv": 3, "norm_groups": 1}
    mixer = ssm_mixer(kit, dtype, D, m, eps)
    w = ssm_weights(D, m, seed=43)
    w["A_log"] = bf(torch.tensor([-9.0, 0.5]))                 # head 0 all but never forgets, head 1 forgets fast
    mixer.load(lambda n: w[n].cuda().to(dtype))
    g = torch.Generator().manual_seed(44)
    x = bf(torch.randn(400, D, generator=g) * 0.3)
    x[3] = bf(torch.randn(D, generator=g) * 4)
    x2 = x.clone()
    x2[3] = bf(torch.randn(D, generator=g) * 4)
    want, want2 = plain(P.mamba2, x, npw(w), "p.", m, eps), plain(P.mamba2, x2, npw(w), "p.", m, eps)
    assert float((want[399] - want2[399]).abs().max()) > 0.02 * float(want[399].abs().max())     # token 3 still matters at 399
    run = MixerRun(kit, mixer, dtype, 16, slots=1)
    close(run.feed(x, cuts_of(380, [64, 2, 100, 7]) + [1] * 20, "first"), want, dtype, f32=1e-4, bf16=3e-2)
    y = bf(torch.randn(30, D, generator=g))
    close(run.feed(y, [1, 2, 27], "second", keep=True), plain(P.mamba2, y, npw(w), "p.", m, eps), dtype, f32=1e-4, bf16=3e-2)
    assert run.cm.state_slot("second") == 0


# ------------------------------------------------------------------ token shift
@pytest.mark.parametrize("dtype", DTYPES)
def test_token_shift_carries_the_previous_row(kit, dtype):
    """The wrapped mixer reads a blend of each row with the one before it; the row before a portion's
    first comes from the request's slot, zeros at the start of a sequence.  Channels with a factor of 1
    read the previous token alone, so a lost or stale row changes them wholesale."""
    D, eps = 72, 1e-5
    m = {"heads": 3, "vdim": 20, "state": 8, "groups": 1, "conv": 2, "norm_groups": 1}
    mixer = ssm_mixer(kit, dtype, D, m, eps, shift=True)
    w = {"mix." + k: v for k, v in ssm_weights(D, m, seed=45).items()}
    g = torch.Generator().manual_seed(46)
    mu = torch.rand(D, generator=g)
    mu[::3], mu[1::9] = 1.0, 0.0
    w["shift"] = bf(mu)
    assert set(mixer.weights()) == set(w)
    mixer.load(lambda n: w[n].cuda().to(dtype))
    xa, xb = bf(torch.randn(75, D, generator=g)), bf(torch.randn(41, D, generator=g))
    inner = {k[len("mix."):]: v for k, v in w.items() if k.startswith("mix.")}

    def ref(x):
        return plain(lambda h: P.mamba2(P.token_shift(h, w["shift"].numpy()), npw(inner), "p.", m, eps), x)
    wa, wb = ref(xa), ref(xb)
    unshifted = plain(P.mamba2, xa, npw(inner), "p.", m, eps)
    assert float((wa - unshifted).abs().max()) > 0.2 * float(wa.abs().max())
    tol = dict(f32=1e-4, bf16=3e-2)
    run = MixerRun(kit, mixer, dtype, 16, slots=2)
    close(run.feed(xa, [75], "whole"), wa, dtype, **tol)
    close(run.feed(xa, cuts_of(75, [2, 3, 2, 17, 5, 2, 30]), "cut"), wa, dtype, **tol)
    close(run.feed(xb, [1] * 41, "single"), wb, dtype, **tol)              # a slot used before: its first token sees zeros
    got = MixerRun(kit, mixer, dtype, 16).plan({"a": xa, "b": xb}, TWO)
    close(got["a"], wa, dtype, **tol)
    close(got["b"], wb, dtype, **tol)


# ------------------------------------------------------------------ sigmoid attention
TAGS = 8


def tagged(D, heads, d, scale, seed, boost):
    """Query and key weights [heads * d, D] under which one score can be made to stand out: the last
    2 * TAGS input channels are tags.  Key tag t lands on dimension t of every key head, query tag t on
    the same dimension of every query head with a large weight: a token with query tag t set gives the
    token with key tag t set a weight near 1, and every other key one near sigmoid(head bias)."""
    g = torch.Generator().manual_seed(seed)
    C = D - 2 * TAGS
    q, k = torch.zeros(heads, d, D), torch.zeros(heads, d, D)
    q[:, TAGS:, :C] = torch.randn(heads, d - TAGS, C, generator=g) / C ** 0.5
    k[:, TAGS:, :C] = torch.randn(heads, d - TAGS, C, generator=g) / C ** 0.5
    for t in range(TAGS):
        q[:, t, C + TAGS + t] = boost / scale
        k[:, t, C + t] = 1.0
    return q.reshape(heads * d, D), k.reshape(heads * d, D)


def sigmoid_case(shape, n=420):
    """Weights, inputs and what the plain implementation makes of them, plus the rows at which a window
    or a count of kept tokens that is one off, or a lost far key, must show."""
    D, H, G, d, window, first, rows, far, page = shape
    scale = 1.1 / math.sqrt(d)
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": scale, "bias_max": far}
    if window:
        m["mask"] = {"size": window, "keep_first": first}
    g = torch.Generator().manual_seed(11)
    wq, _ = tagged(D, H, d, scale, 12, boost=2.5)
    _, wk = tagged(D, G, d, scale, 13, boost=2.5)
    w = {"q": wq, "k": wk, "q.b": 0.1 * torch.randn(H * d, generator=g), "k.b": 0.1 * torch.randn(G * d, generator=g),
         "g": torch.randn(H * d, D, generator=g) / D ** 0.5, "o": torch.randn(D, H * d, generator=g) / (H * d) ** 0.5,
         "rel": 1.2 * torch.randn(rows, H, generator=g), "pb": -5.0 + 0.3 * torch.randn(H, generator=g)}
    w = {k: bf(v) for k, v in w.items()}
    C = D - 2 * TAGS
    x = torch.zeros(n, D)
    x[:, :C] = torch.randn(n, C, generator=g)
    W = window or 10 ** 6
    # keys: the first token; the last kept one and the one after it; keys at both sides of a page border; a key in
    # the middle of a page; a key among the tokens that are decoded one by one
    keys = [0, max(first - 1, 1), max(first, 2), 6 * page - 1, 6 * page, 150 + page // 2, 400, 3 * page]
    asks = {}                                                 # query position -> tag
    edge_in, edge_out, kept_in, kept_out, far_rows = [], [], [], [], []

    def ask(qi, t, into=None):
        if qi < n and qi > keys[t] and qi not in asks and qi not in keys:
            asks[qi] = t
            if into is not None:
                into.append(qi)
            return True
        return False
    for t in (3, 4, 5, 6, 7):                                  # just inside and just outside the window
        if window:
            ask(keys[t] + W - 1, t, edge_in)
            ask(keys[t] + W, t, edge_out)
        else:
            ask(keys[t] + 200, t, far_rows) or ask(n - 1 - t, t, far_rows)
    for qi in (260, 407, 415):                                # far beyond the window: only kept tokens are seen
        if window and first:
            ask(qi, 0, kept_in)
            ask(qi + 1, 1, kept_in if first >= 2 else kept_out)
        elif not window:
            ask(qi, 0, far_rows)
    for qi in (270, 409, 417):
        if window and qi - keys[2] >= W:
            ask(qi, 2, kept_out)
    for t, kpos in enumerate(keys):
        x[kpos, C + t] = 8.0
    for qi, t in asks.items():
        x[qi, C + TAGS + t] = 1.0
    x = bf(x)
    want = plain(P.sigmoid_attention, x, npw(w), "p.", m)

    def differs(**change):
        """Rows at which the plain result changes by more than a fifth of their size under a changed mask."""
        m2 = dict(m, mask=dict(m["mask"], **change))
        other = plain(P.sigmoid_attention, x, npw(w), "p.", m2)
        return set(torch.nonzero((other - want).abs().amax(1) > 0.2 * want.abs().amax(1)).flatten().tolist())
    if window:
        assert set(edge_out) <= differs(size=window + 1) and edge_out, "a window one too long does not show"
        assert set(edge_in) <= differs(size=window - 1) and edge_in, "a window one too short does not show"
        if first:
            gone = differs(keep_first=first - 1)
            assert [qi for qi in kept_in if asks[qi] == (1 if first >= 2 else 0)] and \
                {qi for qi in kept_in if keys[asks[qi]] == first - 1} <= gone, "a kept token too few does not show"
        assert kept_out and set(kept_out) <= differs(keep_first=first + 1 if first >= 2 or keys[2] == first else 3), \
            "a kept token too many does not show"
    else:
        assert far_rows
    return m, w, x, want, asks, keys


# width, heads, kv heads, head size, window, kept first tokens, rows of the distance table, bias_max, page
SIG_SHAPES = [(96, 4, 2, 32, 40, 3, 12, 60, 16), (128, 6, 1, 24, 24, 1, 20, 100, 8), (160, 4, 4, 128, 200, 4, 64, 300, 32),
              (104, 3, 3, 20, 5, 0, 8, 33, 8), (128, 4, 1, 64, None, 0, 40, 250, 16), (100, 6, 2, 12, 32, 11, 16, 90, 8),
              (96, 2, 2, 40, 64, 2, 9, 500, 16),
              # heads of 64 in groups of four; more kept first tokens than one tile of keys holds
              (128, 8, 2, 64, 70, 5, 16, 120, 16), (128, 4, 2, 64, 48, 70, 16, 120, 16)]


def sigmoid_mixer(kit, dtype, D, m, rows, page, max_tokens=640):
    mask = m.get("mask") or {}
    return kit.parts.build_mixer(kit.parts.PartSpec("sigmoid_attention", {
        "hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
        "window": mask.get("size"), "keep_first": mask.get("keep_first", 0), "scale": m["scale"],
        "bias_max": m["bias_max"], "bias_rows": rows}), ctx_for(kit, dtype, page, max_tokens))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", SIG_SHAPES)
def test_sigmoid_attention_at_the_edges_of_window_and_kept_tokens(kit, dtype, shape):
    """Queries whose one loud key is the oldest inside the window, the first outside it, the last kept
    first token, the first that is not kept, at a page border, or hundreds of tokens back: in one
    portion, in portions down to two tokens with the last forty tokens one by one, and in odd portions.
    The weights are not normalised, so a key that is wrongly seen or lost changes the row by its whole
    size; the distance table has fewer rows than distances, and ``bias_max`` lies inside the prompt."""
    D, H, G, d, window, first, rows, far, page = shape
    m, w, x, want, asks, keys = sigmoid_case(shape)
    n = x.shape[0]
    mixer = sigmoid_mixer(kit, dtype, D, m, rows, page)
    assert set(mixer.weights()) == set(w)
    mixer.load(lambda name: w[name].cuda().to(dtype))
    tol = dict(f32=5e-5, bf16=3e-2)
    run = MixerRun(kit, mixer, dtype, page, pages=n // page + 8)
    close(run.feed(x, [n], "whole"), want, dtype, **tol)
    cuts = cuts_of(n - 40, [page - 1, 2, 17, 3, page, 2, 50, 2 * page + 1]) + [1] * 40
    close(run.feed(x, cuts, "a", keep=True), want, dtype, **tol)
    if window:
        # the window gave pages back as it passed; the pages of the kept first tokens stay
        held = [p for p in run.cm.block_table("a", 0) if p >= 0]
        assert len(held) <= window // page + 2 + -(-first // page) < len(run.cm.block_table("a", 0))
    run.cm.free("a")
    close(run.feed(x, cuts_of(n, [2, 5, (window or 64), 3, (window or 64) + 1]), "c"), want, dtype, **tol)
    # two requests in the same steps: the second is the first one's tail, so equal tokens sit at other positions
    xb = x[150:].clone()
    wb = plain(P.sigmoid_attention, xb, npw(w), "p.", m)
    plan, a, b, i = [], 0, 0, 0
    while a < n or b < xb.shape[0]:
        step = {}
        if a < n:
            c = min([37, 1, 2, 64, 1, 9][i % 6], n - a)
            step["a"], a = (a, a + c), a + c
        if b < xb.shape[0] and i % 4 != 3:                    # sits every fourth step out
            c = min([1, 50, 3, 1, 1, 30][i % 6], xb.shape[0] - b)
            step["b"], b = (b, b + c), b + c
        i += 1
        if step:
            plan.append(step)
    got = MixerRun(kit, mixer, dtype, page, pages=2 * (n // page + 8)).plan({"a": x, "b": xb}, plan)
    close(got["a"], want, dtype, **tol)
    close(got["b"], wb, dtype, **tol)


@pytest.mark.parametrize("dtype", DTYPES)
def test_sigmoid_attention_distance_rows(kit, dtype):
    """With queries and keys silenced the weight of a key is sigmoid(table[bucket(i - j), head] + head
    bias) alone: the output is a sum of keys weighted by the table, and a bucket that is one off shows.
    The table's rows are few, so the logarithmic part and the last row are both in use."""
    D, H, G, d, rows, far, page = 64, 2, 1, 16, 10, 47, 8
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": 0.5, "bias_max": far}
    g = torch.Generator().manual_seed(17)
    w = {"q": torch.zeros(H * d, D), "k": torch.randn(G * d, D, generator=g) / D ** 0.5, "q.b": torch.zeros(H * d),
         "k.b": 0.1 * torch.randn(G * d, generator=g), "g": torch.zeros(H * d, D), "o": torch.randn(D, H * d, generator=g) / 6,
         "rel": torch.linspace(-4, 4, rows * H).reshape(H, rows).T.contiguous(), "pb": torch.tensor([0.5, -0.5])}
    w = {k: bf(v) for k, v in w.items()}
    x = bf(torch.randn(90, D, generator=g))
    mixer = sigmoid_mixer(kit, dtype, D, m, rows, page)
    mixer.load(lambda name: w[name].cuda().to(dtype))
    want = plain(P.sigmoid_attention, x, npw(w), "p.", m)
    shifted = dict(npw(w))
    shifted["p.rel"] = np.roll(shifted["p.rel"], 1, axis=0)
    assert float((plain(P.sigmoid_attention, x, shifted, "p.", m) - want).abs().max()) > 0.1 * float(want.abs().max())
    run = MixerRun(kit, mixer, dtype, page)
    close(run.feed(x, [90], "a"), want, dtype, f32=5e-5, bf16=3e-2)
    close(run.feed(x, cuts_of(60, [7, 2, 30]) + [1] * 30, "b"), want, dtype, f32=5e-5, bf16=3e-2)


# ------------------------------------------------------------------ delta rule with a decay per key channel
def channel_delta_weights(D, m, ra, rg, seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
    w = {"q": r(G * d, D) / D ** 0.5, "k": r(G * d, D) / D ** 0.5, "v": r(H * dv, D) / D ** 0.5, "b": r(H, D) / D ** 0.5,
         "a1": r(ra, D) / D ** 0.5, "a2": 2 * r(H * d, ra) / ra ** 0.5, "dt_bias": r(H * d), "A_log": r(H) - 1.0,
         "g1": r(rg, D) / D ** 0.5, "g2": 2 * r(H * dv, rg) / rg ** 0.5, "norm": 1 + 0.2 * r(dv),
         "o": r(D, H * dv) / (H * dv) ** 0.5,
         "q.conv": taps_of(g, G * d, taps), "k.conv": taps_of(g, G * d, taps), "v.conv": taps_of(g, H * dv, taps)}
    return {k: bf(v) for k, v in w.items()}


def channel_delta_mixer(kit, dtype, D, m, ra, rg, eps, page=16):
    return kit.parts.build_mixer(kit.parts.PartSpec("gated_delta", {
        "hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
        "v_head_dim": m["vdim"], "conv": m["conv"], "eps": eps, "decay": "channel", "a_rank": ra, "gate_rank": rg,
        "gate_act": "sigmoid"}), ctx_for(kit, dtype, page))


# width, heads, q/k heads, key size, value size, taps, inner width of the decay, of the gate
CHANNEL_SHAPES = [(64, 4, 2, 16, 24, 3, 10, 6), (96, 3, 3, 32, 32, 2, 16, 24), (100, 6, 2, 20, 36, 5, 12, 9),
                  (128, 2, 1, 128, 128, 4, 32, 32), (72, 2, 2, 8, 40, 1, 5, 7), (80, 1, 1, 200, 16, 4, 3, 40)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", CHANNEL_SHAPES)
def test_channel_delta_rule_in_portions_and_token_by_token(kit, dtype, shape):
    """The whole sequence in one step, in portions down to two tokens, token by token and two
    sequences beside each other.  The decays differ widely between the key channels of a head (the
    plain result with every channel given its head's mean decay is far off), so a kernel that decays
    a head as a whole shows."""
    D, H, G, d, dv, taps, ra, rg = shape
    eps = 1e-5
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "conv": taps}
    mixer = channel_delta_mixer(kit, dtype, D, m, ra, rg, eps)
    w = channel_delta_weights(D, m, ra, rg, seed=51)
    assert set(mixer.weights()) == set(w)
    mixer.load(lambda n: w[n].cuda().to(dtype))
    g = torch.Generator().manual_seed(52)
    xa, xb = bf(torch.randn(75, D, generator=g)), bf(torch.randn(41, D, generator=g))
    wa, wb = plain(P.channel_delta_rule, xa, npw(w), "p.", m, eps), plain(P.channel_delta_rule, xb, npw(w), "p.", m, eps)
    flat = dict(npw(w))
    flat["p.a2"] = np.repeat(flat["p.a2"].reshape(H, d, ra).mean(1, keepdims=True), d, axis=1).reshape(H * d, ra)
    flat["p.dt_bias"] = np.repeat(flat["p.dt_bias"].reshape(H, d).mean(1, keepdims=True), d, axis=1).reshape(H * d)
    other = plain(P.channel_delta_rule, xa, flat, "p.", m, eps)
    assert float((other - wa).abs().max()) > 0.1 * float(wa.abs().max())
    tol = dict(f32=1e-4, bf16=3e-2)
    run = MixerRun(kit, mixer, dtype, 16)
    close(run.feed(xa, [75], "whole"), wa, dtype, **tol)
    close(run.feed(xa, cuts_of(75, [2, 3, 2, 17, 5, 2, 30]), "cut"), wa, dtype, **tol)
    close(run.feed(xa, [1] * 75, "single"), wa, dtype, **tol)
    got = MixerRun(kit, mixer, dtype, 16).plan({"a": xa, "b": xb}, TWO)
    close(got["a"], wa, dtype, **tol)
    close(got["b"], wb, dtype, **tol)


@pytest.mark.parametrize("dtype", DTYPES)
def test_channel_delta_rule_remembers_far_back_and_slots_start_clean(kit, dtype):
    """Half the key channels of head 0 barely decay and keep what a loud token wrote hundreds of
    tokens ago (the tokens after it have a beta near 0, so they neither overwrite nor drown it); the
    other half and head 1 forget fast.  Then the slot is given back and used by
    another request, which must see none of it, also when its first portion is a single token."""
    D, H, G, d, dv, taps, ra, rg, eps = 64, 2, 1, 16, 16, 3, 8, 8, 1e-5
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "conv": taps}
    mixer = channel_delta_mixer(kit, dtype, D, m, ra, rg, eps)
    w = channel_delta_weights(D, m, ra, rg, seed=53)
    w["A_log"] = bf(torch.tensor([0.0, 0.5]))
    w["a2"] = bf(w["a2"] * 0.05)
    bias = torch.full((H, d), 1.0)
    bias[0, ::2] = -9.0                                        # softplus(-9) is about 1e-4: these rows of S stay
    w["dt_bias"] = bf(bias.reshape(-1))
    w["b"] = bf(w["b"] * 0.2)
    w["b"][:, 0] = 6.0                                         # input channel 0 decides beta: about 0 or about 1
    mixer.load(lambda n: w[n].cuda().to(dtype))
    g = torch.Generator().manual_seed(54)
    x = bf(torch.randn(400, D, generator=g) * 0.3)
    x[3] = bf(torch.randn(D, generator=g) * 4)
    x[:, 0], x[3, 0] = -1.0, 1.0                               # token 3 writes; the others barely write or erase
    x2 = x.clone()
    x2[3, 1:] = bf(torch.randn(D - 1, generator=g) * 4)
    want = plain(P.channel_delta_rule, x, npw(w), "p.", m, eps)
    want2 = plain(P.channel_delta_rule, x2, npw(w), "p.", m, eps)
    # token 3 decides the row at 399: without its state the row is off by its whole size, so the looser bound for
    # bfloat16 (the loud token's projections are rounded to 8 bits and read back 396 tokens later) loses nothing
    assert float((want[399] - want2[399]).abs().max()) > 0.5 * float(want[399].abs().max())
    run = MixerRun(kit, mixer, dtype, 16, slots=1)
    close(run.feed(x, cuts_of(380, [64, 2, 100, 7]) + [1] * 20, "first"), want, dtype, f32=1e-4, bf16=8e-2)
    y = bf(torch.randn(30, D, generator=g))
    close(run.feed(y, [1, 2, 27], "second", keep=True), plain(P.channel_delta_rule, y, npw(w), "p.", m, eps), dtype,
          f32=1e-4, bf16=3e-2)
    assert run.cm.state_slot("second") == 0


# ------------------------------------------------------------------ experts chosen within the best groups
def moe_part(kit, dtype, D, F, experts, top, groups, limit, max_tokens=1024):
    return kit.parts.build_feed_forward(kit.parts.PartSpec("moe", {
        "hidden_size": D, "intermediate_size": F, "experts": experts, "top": top, "router_bias": False,
        "router_weigh": "softmax_all", "groups": groups, "activation": "clamped_swish", "limit": limit}),
        ctx_for(kit, dtype, max_tokens=max_tokens))


def router_of(experts, top, groups):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return r


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,top,groups", [(8, 3, (4, 2)), (6, 2, (3, 1)), (9, 3, (3, 2)), (16, 4, (4, 2)), (12, 2, (6, 1)),
                                                (4, 1, None), (3, 3, None), (10, 5, (2, 1)), (64, 6, (8, 3))])
def test_choice_of_experts_within_the_best_groups(kit, dtype, experts, top, groups):
    """The chosen experts and their weights (scores of the softmax over all experts, divided by their
    sum).  With groups, a good share of the tokens choose otherwise than they would without."""
    D, T = 56, 300
    g = torch.Generator().manual_seed(61)
    moe = moe_part(kit, dtype, D, 8, experts, top, groups, 1.0)
    wr = bf(torch.randn(experts, D, generator=g) / 3)
    moe.w_router = wr.cuda().to(dtype)
    x = bf(torch.randn(T, D, generator=g))
    gaps = []
    want_idx, want_w = P.route(x.double().numpy(), wr.double().numpy(), router_of(experts, top, groups), gaps)
    if groups:
        free_idx, _ = P.route(x.double().numpy(), wr.double().numpy(), router_of(experts, top, None))
        changed = sum(set(a) != set(b) for a, b in zip(want_idx, free_idx))
        assert changed > T // 10, f"the groups change the choice of only {changed} tokens"
    sure = torch.from_numpy(gaps[0] > 1e-4)
    assert int(sure.sum()) > T * 0.95
    for rows in (x, x[7:8]):                                   # many rows and one row alone
        idx, wgt = moe.route(rows.cuda().to(dtype).contiguous())
        lo = 0 if rows.shape[0] == T else 7
        wi, ww = torch.from_numpy(want_idx)[lo:lo + rows.shape[0]], torch.from_numpy(want_w)[lo:lo + rows.shape[0]]
        keep = sure[lo:lo + rows.shape[0]]
        got = torch.zeros(rows.shape[0], experts).double().scatter_(1, idx.cpu().long(), wgt.cpu().double())
        want = torch.zeros(rows.shape[0], experts).double().scatter_(1, wi, ww)
        assert torch.equal((got > 0)[keep], (want > 0)[keep])
        torch.testing.assert_close(got[keep], want[keep], rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(got.sum(1), torch.ones(rows.shape[0]).double(), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,top,groups,T,D,F,limit", [(6, 2, (3, 2), 37, 40, 24, 0.7), (4, 1, None, 5, 40, 24, 1.0),
                                                            (3, 3, None, 1, 40, 24, 2.0), (12, 2, (4, 1), 150, 40, 24, 0.5),
                                                            (8, 2, (2, 1), 700, 40, 24, 1.0), (20, 3, (5, 3), 400, 40, 24, 1.5),
                                                            (6, 2, (2, 2), 9, 320, 264, 1.0), (5, 2, None, 70, 264, 328, 0.9)])
def test_mixture_with_clamped_experts(kit, dtype, experts, top, groups, T, D, F, limit):
    """An expert's gate is cut from above and its up projection from both sides, and the product is
    g sigmoid(1.702 g) (u + 1): the weights are large enough that the limits bite for many values.  Few
    rows (the kernels that stream the chosen experts' weights) and many rows (in bfloat16 the tcgen05
    product over rows gathered into whole tiles per expert)."""
    g = torch.Generator().manual_seed(62)
    r = lambda *s: torch.randn(*s, generator=g)
    moe = moe_part(kit, dtype, D, F, experts, top, groups, limit)
    p = {"router": bf(r(experts, D) / 3)}
    for e in range(experts):
        p.update({f"e{e}.gate": bf(r(F, D) * 1.2 / D ** 0.5), f"e{e}.up": bf(r(F, D) * 1.2 / D ** 0.5),
                  f"e{e}.down": bf(r(D, F) / F ** 0.5)})
    assert set(moe.weights()) == set(p)
    moe.load(lambda local: p[local].cuda().to(dtype))
    x = bf(r(T, D))
    f = {"router": router_of(experts, top, groups), "expert": {"ff": F, "limit": limit}}
    gaps = []
    want = plain(P.mixture, x, npw(p), "p.", f, gaps)
    cut = float((np.abs(x.double().numpy() @ npw(p)["p.e0.up"].T) > limit).mean())
    assert cut > 0.1, "the limit hardly ever bites"
    sure = torch.from_numpy(gaps[0] > 1e-3)
    got = moe.forward(x.cuda().to(dtype), None).clone()
    close(got[sure], want[sure], dtype)
    if T > 4:
        i = int(torch.nonzero(sure)[3])
        alone = moe.forward(x[i:i + 1].cuda().to(dtype).contiguous(), None).clone()
        close(alone, want[i:i + 1], dtype)


# ------------------------------------------------------------------ both branches side by side
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["fap_a", "fap_c"])
def test_parallel_mixer_with_token_shift(kit, dtype, name):
    """A whole mixer of a parallel layer as the model builds it: the token shift in front, the sigmoid
    attention and the delta rule reading the same shifted rows, their results summed with a factor each."""
    from gollmgo_b200.architectures.fapudra import fapudra_spec
    from gollmgo_b200.config.fapudra_config import FapudraConfig
    cfg, page = ft.get(name)
    D, eps = cfg["width"], cfg["norm"]["eps"]
    m = cfg["layers"][0]["mixer"]
    spec = fapudra_spec(FapudraConfig.from_dict(cfg)).layers[0].mixer
    mixer = kit.parts.build_mixer(spec, ctx_for(kit, dtype, page))
    w = {k[len("l0."):]: v for k, v in ft.random_weights(cfg, 71).items() if k.startswith(("l0.mix.", "l0.shift"))}
    assert set(mixer.weights()) == set(w)
    mixer.load(lambda n: w[n].cuda().to(dtype))
    x = bf(torch.randn(140, D, generator=torch.Generator().manual_seed(72)))
    want = plain(lambda h: P.parallel_mixer(P.token_shift(h, w["shift"].double().numpy()), npw(w), "p.mix.", m, eps), x)
    left_only = plain(lambda h: P.parallel_mixer(P.token_shift(h, w["shift"].double().numpy()), npw(w), "p.mix.",
                                                 dict(m, right_scale=0.0), eps), x)
    share = float((want - left_only).abs().max() / want.abs().max())
    assert 0.05 < share and float(left_only.abs().max()) > 0.05 * float(want.abs().max())      # both branches count
    run = MixerRun(kit, mixer, dtype, page)
    close(run.feed(x, [140], "a"), want, dtype, f32=1e-4, bf16=3e-2)
    close(run.feed(x, cuts_of(110, [33, 2, 9]) + [1] * 30, "b"), want, dtype, f32=1e-4, bf16=3e-2)


# ------------------------------------------------------------------ whole models through bin/trace_run
# longer than every window plus what is decoded one by one; one request of a single token and short ones
LENGTHS = {"fap_a": [1, 5, 37, 70, 130, 96], "fap_b": [2, 64, 65, 131, 90, 33], "fap_c": [3, 66, 40, 150, 97, 129],
           "fap_d": [4, 17, 290, 33, 65, 120], "fap_e": [2, 73, 160, 31, 210, 95]}
# float32: every row to a few units of rounding.  bfloat16: nine rows in ten within 4 % of the row's largest
# logit and none further off than what a lost key or state would cause (such a row is off by its whole size).
TOL = {"float32": (5e-5, 5e-5), "bfloat16": (4e-2, 0.15)}
_CASES = {}


def case(name, seed):
    """Weights, requests without close calls in the choice of experts, and the plain logits of a
    configuration; made once for both precisions."""
    if (name, seed) not in _CASES:
        cfg, page = ft.get(name)
        weights = ft.random_weights(cfg, seed=seed)
        requests = ft.steady_requests(cfg, weights, LENGTHS[name], seed=seed + 100)
        w = ft.as_numpy(weights)
        reference = {r: P.forward(cfg, w, toks) for r, toks in requests.items()}
        _CASES[(name, seed)] = (cfg, page, weights, requests, reference)
    return _CASES[(name, seed)]


def compare(trace, out_dir, reference, vocab, dtype):
    errs = []
    for step, exp in trace.expect.items():
        path = os.path.join(out_dir, f"{step}.f32")
        assert os.path.exists(path), f"step {step} wrote no file"
        got = np.fromfile(path, dtype="<f4").reshape(-1, vocab)
        assert got.shape[0] == len(exp), f"step {step}: {got.shape[0]} rows, expected {len(exp)}"
        for row, (name, pos) in zip(got, exp):
            ref = reference[name][pos]
            assert np.isfinite(row).all(), f"step {step} {name}@{pos}: non-finite logits"
            errs.append((float(np.abs(row - ref).max() / max(np.abs(ref).max(), 1e-6)), step, name, pos))
    most, worst = TOL[dtype]
    p90 = float(np.percentile([e[0] for e in errs], 90))
    top = max(errs)
    assert p90 <= most, f"90th percentile of the rows' errors is {p90:.3e}"
    assert top[0] <= worst, f"worst relative error {top[0]:.3e} at (step, request, position) {top[1:]}"
    return p90, top[0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ft.TINY))
def test_replay_matches_plain(tmp_path, cuda_device, name, dtype):
    """Whole prompts; prompts with their last 48 tokens one by one (every window passes over decoded
    tokens); portions down to two tokens; and two mixed schedules with up to four and three live
    requests on a pool of the trace's peak, where pages and slots are used again."""
    cfg, page, weights, requests, reference = case(name, 81)
    model_dir = ft.model_folder(tmp_path, name, cfg, weights)
    trace = tt.Trace()
    tt.whole(trace, requests)
    tt.tail_decode(trace, requests, tail=48)
    tt.portions(trace, requests)
    tt.mixed(trace, requests, max_live=4, seed=3)
    tt.mixed(trace, dict(reversed(list(requests.items()))), max_live=3, seed=4, tag="n")
    out = str(tmp_path / "out")
    tt.run_trace(model_dir, dtype, trace, out, block_size=page)
    p90, worst = compare(trace, out, reference, cfg["vocab"], dtype)
    pool, asked, shared = tt.pages_were_used_again(trace, out + "/pages.jsonl", page)
    print(f"{name} {dtype}: {len(trace.steps)} steps, {pool} pages for {asked} asked, {shared} held by several, "
          f"errors: 90 % within {p90:.2e}, worst {worst:.2e}")


@pytest.mark.parametrize("name,dtype", [("fap_a", "bfloat16"), ("fap_b", "float32"), ("fap_c", "bfloat16")])
def test_pages_given_back_are_never_read(tmp_path, cuda_device, name, dtype):
    """The mixed trace with every page overwritten by NaN the moment it is given back (the windowed
    layers give pages back all the time, but never those of the kept first tokens)."""
    cfg, page, weights, requests, reference = case(name, 81)
    model_dir = ft.model_folder(tmp_path, name, cfg, weights)
    trace = tt.Trace()
    tt.mixed(trace, requests, max_live=4, seed=7)
    tt.portions(trace, requests)
    out = str(tmp_path / "out")
    tt.run_trace(model_dir, dtype, trace, out, block_size=page, env=dict(os.environ, GOLLMGO_B200_POISON_FREED="1"))
    compare(trace, out, reference, cfg["vocab"], dtype)
    tt.pages_were_used_again(trace, out + "/pages.jsonl", page)


def test_a_checkpoint_in_bfloat16_loads_alike(tmp_path, cuda_device):
    """The same weights stored as bfloat16 (integer tables aside, that is how checkpoints come) and as
    float32 give the same logits: the test weights are exact in bfloat16."""
    cfg, page, weights, requests, reference = case("fap_c", 81)
    few = dict(list(requests.items())[:3])
    outs = []
    for stored in ("bfloat16", "float32"):
        d = ft.model_folder(tmp_path, "fap_c_" + stored, cfg, weights, dtype=stored)
        trace = tt.Trace()
        tt.whole(trace, few)
        out = str(tmp_path / ("out_" + stored))
        tt.run_trace(d, "float32", trace, out, block_size=page)
        compare(trace, out, reference, cfg["vocab"], "float32")
        outs.append([np.fromfile(os.path.join(out, f"{s}.f32"), dtype="<f4") for s in trace.expect])
    for a, b in zip(*outs):
        assert np.array_equal(a, b)


# ------------------------------------------------------------------ the entry point
def plain_greedy(cfg, weights, prompt, n):
    w = ft.as_numpy(weights)
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(P.forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]


def test_greedy_generation_through_the_engine(tmp_path, cuda_device):
    """Requests of unequal length through Engine.generate (scheduler, chunked prompts, captured
    decode steps, the device's arg-max): the plain implementation's tokens, alone and together."""
    from gollmgo_b200 import Engine, SamplingParams
    cfg, page = ft.get("fap_a")
    weights = ft.random_weights(cfg, seed=83)
    d = ft.model_folder(tmp_path, "fap_a", cfg, weights)
    prompts = list(tt.random_requests(cfg["vocab"], [1, 9, 40, 23], seed=8).values())
    eng = Engine(d, dtype="float32", block_size=page, num_blocks=24, max_batch_size=4, max_token_budget=32,
                 prefill_chunk_size=16)
    outs = eng.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    want = [plain_greedy(cfg, weights, pr, 12) for pr in prompts]
    assert [o.token_ids for o in outs] == want
    assert eng.generate([prompts[2]], SamplingParams(max_tokens=12, ignore_eos=True))[0].token_ids == want[2]
    eng.runner.cache.audit()
    assert eng.runner.cache.min_free_pages() == 24
    assert eng.runner.cache.slots.num_free == eng.runner.cache.slots.max_requests


def test_long_decoding_in_bfloat16_stays_near_the_plain_choice(tmp_path, cuda_device):
    """200 decoded tokens, past every window and over many pages, through captured decode steps: the
    tokens are (nearly) the plain implementation's best given the same history."""
    from gollmgo_b200 import Engine, SamplingParams
    cfg, page = ft.get("fap_b")
    weights = ft.random_weights(cfg, seed=84)
    d = ft.model_folder(tmp_path, "fap_b", cfg, weights)
    prompt = tt.random_requests(cfg["vocab"], [11], seed=9)["r0"]
    eng = Engine(d, dtype="bfloat16", block_size=page, num_blocks=40, max_batch_size=2, max_token_budget=64)
    toks = eng.generate([prompt], SamplingParams(max_tokens=200, ignore_eos=True))[0].token_ids
    assert len(toks) == 200
    logits = P.forward(cfg, ft.as_numpy(weights), prompt + toks)
    near = sum(float(row.max() - row[tok]) <= 0.06 * float(np.abs(row).max())
               for tok, row in zip(toks, logits[len(prompt) - 1:]))
    assert near >= 185, f"only {near} of 200 tokens are near the plain choice"
    assert eng.runner.cache.min_free_pages() == 40


def test_command_line_generates(tmp_path, cuda_device):
    import json
    import subprocess
    import sys
    cfg, page = ft.get("fap_c")
    weights = ft.random_weights(cfg, seed=85)
    d = ft.model_folder(tmp_path, "fap_c", cfg, weights)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, "-m", "gollmgo_b200", "generate", "--model", d, "--dtype", "float32",
                        "--block-size", str(page), "--num-blocks", "16", "--max-batch-size", "4", "--max-token-budget", "64",
                        "--log-level", "error", "--prompt-ids", "5,6,7", "--prompt-ids", "9", "--max-tokens", "5", "--ignore-eos"],
                       capture_output=True, text=True, cwd=root)
    assert p.returncode == 0, p.stderr
    lines = [json.loads(l) for l in p.stdout.strip().splitlines()]
    assert lines[0]["token_ids"] == plain_greedy(cfg, weights, [5, 6, 7], 5)
    assert lines[1]["token_ids"] == plain_greedy(cfg, weights, [9], 5)
