"""Vivazen: each mechanism against its plain statement, and the engine against the plain model.

The configurations are small and differ from each other in every size and option: grouped and ungrouped heads, values
wider and narrower than keys, filters of no, two and five taps, with and without a score cap, compressed rows that are no
multiple of anything, rotated parts of two features and of half the head, windows of one position, of no whole page and
of two whole pages, with and without frequency scaling, norms in one and several groups, stream constants of 1 and above,
layers without a feed-forward, layers that run another layer's tensors (after and before their owner), both layer
orders, and models of one mixer alone.  Weights are seeded random ones with the norm weights of queries and keys, the
query projections of the latent attention and the sinks scaled up, so that the attention weights are far from uniform,
the caps are reached and a sink that is left out changes the logits.

Engine cases run on the GPU (`-m gpu`, float32 and bfloat16) and, as a check of the host side alone, on the CPU over
the plain kernel statements (float32, shorter requests).
"""
from __future__ import annotations

import copy
import math

import pytest
import torch

from tests.conftest import random_tokens
from tests.helpers import assert_logits as _assert_exact, make_engine, run_in_pieces, run_requests

GPU = pytest.mark.gpu
CASES = [pytest.param("cuda", "float32", marks=GPU), pytest.param("cuda", "bfloat16", marks=GPU),
         pytest.param("refs", "float32")]


def assert_logits(got, want, dtype, what):
    """float32: every logit within 1e-4 of the largest one.  bfloat16: rows are judged by the root mean square of
    their difference against that of the logits: all within 5 %, half of them within 1.5 %."""
    if dtype in ("float32", torch.float32):
        return _assert_exact(got, want, dtype, what)
    got, want = got.detach().double().cpu(), want.double().cpu()
    assert got.shape == want.shape and torch.isfinite(got).all(), what
    rows = (got - want).pow(2).mean(1).sqrt() / want.pow(2).mean().sqrt()
    assert rows.max().item() <= 5e-2 and rows.median().item() < 1.5e-2, \
        f"{what}: worst row {rows.max().item():.3f} at {int(rows.argmax())}, median {rows.median().item():.4f}"


def _att(heads, kv, dim, vdim, scale, conv=0, cap=0.0):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if conv:
        m["conv"] = conv
    if cap:
        m["softcap"] = cap
    return m


def _lat(heads, dim, rot_dim, vdim, rank, scale, window=0, base=10000.0, scaling=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim}}
    if scaling:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if window:
        m["mask"] = {"size": window}
    return m


def _layer(kind, mixer, ff, weights_of=None):
    d = {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


def _model(vocab, width, groups, eps, alpha, layers):
    layers = copy.deepcopy(layers)
    for l in layers:                                  # a layer that borrows tensors is described as its owner is
        if "weights_of" in l:
            o = layers[l["weights_of"]]
            l["type"], l["mixer"], l["mlp"] = o["type"], copy.deepcopy(o["mixer"]), copy.deepcopy(o["mlp"])
    return {"architecture": "Vivazen", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups},
            "postln_alpha": alpha, "layers": layers}


BORROW = lambda j: {"type": None, "mixer": None, "mlp": None, "weights_of": j}

VIV_A = _model(200, 64, 2, 1e-6, 2.0, [
    _layer("latent_attention", _lat(4, 16, 8, 16, 24, 0.2, window=24, base=1000.0, scaling=(4.0, 64, 8.0, 1.0)), 96),
    _layer("attention", _att(4, 2, 32, 16, 0.2, conv=3, cap=10.0), 64),
    BORROW(0),
    _layer("attention", _att(2, 2, 16, 24, 0.3), None)])

# one group in the norm, a stream constant of 1, a borrowing layer before its owner, a window that is no whole page
VIV_B = _model(333, 96, 1, 1e-5, 1.0, [
    BORROW(1),
    _layer("attention", _att(6, 1, 16, 8, 0.3, conv=2, cap=5.0), 128),
    _layer("latent_attention", _lat(3, 32, 16, 40, 48, 0.15, window=70, base=500.0), None),
    _layer("latent_attention", _lat(2, 8, 24, 8, 40, 0.2, base=100.0, scaling=(8.0, 32, 4.0, 0.5)), 48)])

# sizes a tensor-core kernel takes; a window of two whole pages; as many key/value heads as query heads
VIV_C = _model(512, 128, 8, 1e-6, 3.5, [
    _layer("latent_attention", _lat(8, 32, 32, 32, 96, 0.12, window=128, base=300000.0, scaling=(2.0, 256, 16.0, 2.0)), 256),
    _layer("attention", _att(8, 2, 64, 64, 0.12, conv=4, cap=30.0), 128),
    _layer("attention", _att(16, 16, 16, 32, 0.25, conv=4), None),
    BORROW(0)])

# sizes that are multiples of little (a feed-forward width of 21); a window of five and a window of one position; a
# rotated part of two features
VIV_D = _model(301, 72, 3, 1e-4, 1.7, [
    _layer("attention", _att(5, 5, 10, 6, 0.3, conv=5, cap=3.0), 40),
    _layer("latent_attention", _lat(3, 12, 6, 14, 10, 0.3, window=5, base=100.0), 21),
    _layer("latent_attention", _lat(1, 6, 2, 6, 7, 0.4, window=1, base=100.0, scaling=(3.0, 16, 2.0, 1.0)), None),
    BORROW(0)])

# each mixer alone, without a feed-forward
VIV_E = _model(150, 48, 4, 1e-6, 1.0, [_layer("attention", _att(3, 1, 16, 16, 0.25, conv=4, cap=8.0), None)])
VIV_F = _model(150, 48, 2, 1e-6, 1.0, [_layer("latent_attention", _lat(3, 8, 8, 16, 16, 0.25, window=9, scaling=(2.0, 16, 4.0, 1.0)), None)])
# a width that is no multiple of 8
VIV_G = _model(97, 36, 9, 1e-5, 2.5, [_layer("attention", _att(2, 1, 12, 12, 0.3, conv=2), 30),
                                      _layer("latent_attention", _lat(2, 4, 4, 6, 12, 0.3, window=40), 18)])

VIV = {"A": VIV_A, "B": VIV_B, "C": VIV_C, "D": VIV_D, "E": VIV_E, "F": VIV_F, "G": VIV_G}


def write_vivazen(model_dir: str, raw: dict, seed: int, gain: float = 4.0, norm_gain: float = 2.0, q_gain: float = 8.0,
                  sink_gain: float = 3.0) -> None:
    """A folder of seeded random weights.  The norm weights of filtered queries and keys and the latent attention's
    query projection are scaled up (peaked attention weights, scores at the cap), the sinks are spread (some heads
    give most of their weight to the sink, some none), and the output side of every sublayer is scaled up so that
    the sublayers weigh against the scaled stream.  The gains suit widths of a hundred."""
    from janis_b200 import build_model
    from janis_b200.weights.loader import random_tensors, write_model_folder
    _, cfg, model = build_model(raw)
    tensors = random_tensors(model.tensor_specs(), seed, "cpu")
    latent = {f"l{i}" for i, l in enumerate(raw["layers"]) if l["type"] == "latent_attention"}
    for name, t in list(tensors.items()):
        layer = name.split(".")[0]
        if name.endswith(".q.norm") or name.endswith(".k.norm"):
            tensors[name] = (t.float() * norm_gain).to(torch.bfloat16)
        elif name.endswith(".mix.q") and layer in latent:
            tensors[name] = (t.float() * q_gain).to(torch.bfloat16)
        elif name.endswith(".sink"):
            tensors[name] = (t.float() * sink_gain).to(torch.bfloat16)
        elif any(name.endswith(x) for x in (".o", ".down", ".up", ".gate", ".mix.g", ".mix.v", ".mix.dkv")):
            tensors[name] = (t.float() * gain).to(torch.bfloat16)
    write_model_folder(model_dir, cfg.to_dict(), tensors, {"seed": str(seed)})


@pytest.fixture(scope="module")
def viv_dirs(tmp_path_factory):
    out = {}
    for i, (key, raw) in enumerate(VIV.items()):
        d = tmp_path_factory.mktemp(f"vivazen_{key}")
        write_vivazen(str(d), raw, 500 + i)
        out[key] = str(d)
    return out


@pytest.fixture(scope="module")
def plain(viv_dirs):
    from tests.plain import vivazen_plain as P
    loaded, memo = {}, {}

    def logits(key, tokens):
        if key not in loaded:
            loaded[key] = P.load_folder(viv_dirs[key])
        k = (key, tuple(tokens))
        if k not in memo:
            cfg, w = loaded[key]
            memo[k] = P.forward(cfg, w, list(tokens))
        return memo[k]

    return logits


@pytest.fixture(scope="module")
def engines(viv_dirs):
    made = {}

    def get(key, dtype, on, **kw):
        k = (key, dtype, on, tuple(sorted(kw.items())))
        if k not in made:
            made[k] = make_engine(viv_dirs[key], dtype, on, **kw)
        return made[k]

    yield get
    for e in made.values():
        e.close()


def keys_for(on):
    return ["A", "B", "C", "D", "E", "F", "G"] if on == "cuda" else ["A", "B", "D", "E", "F", "G"]


def _requests(vocab, lens, seed):
    return [random_tokens(vocab, n, seed + i) for i, n in enumerate(lens)]


# ---------------------------------------------------------------------------
# configuration and registry
# ---------------------------------------------------------------------------

def test_configuration_reads_back_and_guards():
    from janis_b200 import ConfigError, VivazenConfig, build_model, resolve
    cfg = VivazenConfig.from_dict(VIV_A)
    assert VivazenConfig.from_dict(cfg.to_dict()) == cfg
    assert resolve(VIV_A).name == "Vivazen"
    assert cfg.layers[0].mixer.window == 24 and cfg.layers[0].mixer.rot_scaling.factor == 4.0
    assert cfg.layers[3].mlp is None and cfg.layers[3].mixer.conv == 0 and cfg.layers[3].mixer.softcap == 0.0
    assert cfg.weight_layer(2) == 0 and cfg.weight_layer(1) == 1 and cfg.postln_alpha == 2.0 and cfg.norm_groups == 2
    _, _, model = build_model(VIV_A)
    specs = model.tensor_specs()
    assert not any(n.startswith("l2.") for n in specs) and "l3.norm2" not in specs and "l3.mix.q.conv" not in specs
    assert specs["l0.mix.dkv"].shape == (24 + 8, 64) and specs["l0.mix.q"].shape == (4 * 24, 64)
    assert specs["l0.mix.uk"].shape == (4 * 16, 24) and specs["l0.mix.g"].shape == (4, 64) and specs["l0.mix.sink"].shape == (4,)
    assert specs["l1.mix.q.conv"].shape == (128, 3) and specs["l1.mix.v.conv"].shape == (32, 3) and specs["l1.mix.talk"].shape == (4, 4)
    # a layer that runs another's tensors is that layer's block once more, with a cache line of its own
    assert [(c.layer, c.cache_line) for c in model.schedule] == [(0, 0), (1, 1), (0, 2), (2, 3)]
    needs = model.cache_line_needs()
    assert set(needs[0]) == {"kv"} and set(needs[1]) == {"kv", "filter"} and set(needs[3]) == {"kv"}
    assert needs[0]["kv"].n_kv_heads == 1 and needs[0]["kv"].head_dim == 24 + 8
    _, _, model_b = build_model(VIV_B)
    assert [(c.layer, c.cache_line) for c in model_b.schedule] == [(0, 0), (0, 1), (1, 2), (2, 3)]
    bad_layers = [
        [{"type": "conv", "mixer": {}, "mlp": None}],
        [_layer("attention", _att(4, 3, 32, 16, 0.2), None)],
        [_layer("latent_attention", _lat(4, 16, 7, 16, 24, 0.2), None)],
        [_layer("attention", _att(4, 2, 32, 16, 0.2), None), {**_layer("attention", _att(4, 2, 32, 8, 0.2), None), "weights_of": 0}],
        [{**_layer("attention", _att(4, 2, 32, 16, 0.2), None), "weights_of": 0}],
        [{**_layer("attention", _att(4, 2, 32, 16, 0.2), None), "mlp": {"kind": "sparse", "ff": 8}}]]
    for layers in bad_layers:
        with pytest.raises(ConfigError):
            VivazenConfig.from_dict({**VIV_A, "layers": layers})
    with pytest.raises(ConfigError):
        VivazenConfig.from_dict({**VIV_A, "norm": {"eps": 1e-6, "groups": 5}})


# ---------------------------------------------------------------------------
# the plain statements by hand
# ---------------------------------------------------------------------------

def test_plain_filter_norm_and_ramp_by_hand():
    from tests.plain import vivazen_plain as P
    u = torch.tensor([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0]], dtype=torch.float64)
    w = torch.tensor([[0.5, 2.0], [1.0, -1.0]], dtype=torch.float64)      # two taps: the older input first
    y = P.short_filter(u, w)
    assert torch.allclose(y, torch.tensor([[2.0, -10.0], [4.5, -10.0], [7.0, -10.0]], dtype=torch.float64))
    x = torch.tensor([[3.0, 4.0, 0.0, 2.0]], dtype=torch.float64)
    got = P.group_norm(x, torch.tensor([1.0, 2.0, 3.0, 4.0], dtype=torch.float64), 2, 0.0)
    r0, r1 = math.sqrt(12.5), math.sqrt(2.0)
    assert torch.allclose(got, torch.tensor([[3 / r0, 8 / r0, 0.0, 8 / r1]], dtype=torch.float64))
    # frequencies: 4 pairs of base 100 over 8 features; a pair that turns `fast` times or more over `original` positions
    # keeps its frequency, one that turns `slow` times or fewer is divided by the factor, a line between
    rot = {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "original": 64, "fast": 4.0, "slow": 1.0}}
    f, amp = P.ramped_frequencies(rot)
    plain_f = [100.0 ** (-2.0 * i / 8) for i in range(4)]
    where = lambda t: 8 * math.log(64 / (2 * math.pi * t)) / (2 * math.log(100.0))
    lo, hi = max(math.floor(where(4.0)), 0), min(math.ceil(where(1.0)), 7)
    assert (lo, hi) == (0, 3)
    for i in range(4):
        r = min(max((i - lo) / (hi - lo), 0.0), 1.0)
        assert abs(f[i] - (plain_f[i] / 4.0 * r + plain_f[i] * (1 - r))) < 1e-15
    assert f[0] == plain_f[0] and abs(f[3] - plain_f[3] / 4.0) < 1e-15 and abs(amp - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    # neighbours turn together: (1, 0) at position 1 with frequency pi/2 becomes (0, amp)
    t = P.turn_neighbours(torch.tensor([[[1.0, 0.0, 0.0, 1.0]]], dtype=torch.float64).repeat(2, 1, 1), torch.arange(2),
                          [math.pi / 2, math.pi], 2.0)
    assert torch.allclose(t[0, 0], torch.tensor([2.0, 0.0, 0.0, 2.0], dtype=torch.float64))
    assert torch.allclose(t[1, 0], torch.tensor([0.0, 2.0, 0.0, -2.0], dtype=torch.float64), atol=1e-12)


def test_plain_window_sink_gate_and_mixing_by_hand():
    from tests.plain import vivazen_plain as P
    # filtered attention's weights: two heads over one key/value head, scores 0 everywhere: uniform causal weights,
    # mixed by [[1, 1], [0, 2]]: head 0's weights sum to 2, head 1's are doubled
    T = 3
    q = torch.zeros(T, 2, 4, dtype=torch.float64)
    k = torch.zeros(T, 1, 4, dtype=torch.float64)
    v = torch.arange(T, dtype=torch.float64).view(T, 1, 1) + 1.0         # values 1, 2, 3
    o = P.mixed_softmax_attention(q, k, v, 1.0, 5.0, torch.tensor([[1.0, 1.0], [0.0, 2.0]], dtype=torch.float64))
    means = torch.tensor([1.0, 1.5, 2.0], dtype=torch.float64)
    assert torch.allclose(o[:, 0, 0], 2 * means) and torch.allclose(o[:, 1, 0], 2 * means)
    # a cap bounds one large score: with q.k = 100 and cap 2 the two keys' scores are 2 tanh(50) = 2 and 0
    q = torch.tensor([[[0.0]], [[10.0]]], dtype=torch.float64)
    k = torch.tensor([[[0.0]], [[10.0]]], dtype=torch.float64)
    v = torch.tensor([[[0.0]], [[1.0]]], dtype=torch.float64)
    o = P.mixed_softmax_attention(q, k, v, 1.0, 2.0, None)
    assert abs(o[1, 0, 0].item() - math.exp(2.0) / (math.exp(2.0) + 1.0)) < 1e-12
    # latent attention with zero projections for queries: every seen key has score 0; a window of 2; a sink of ln 2
    # puts 2 into the denominator; the gate is sigmoid(0) = 1/2
    W, R, dv = 4, 2, 2
    m = {"heads": 1, "dim": 2, "rot_dim": 2, "vdim": dv, "kv_rank": R, "scale": 1.0, "rot": {"base": 10.0, "dims": 2},
         "mask": {"size": 2}}
    w = {"q": torch.zeros(4, W), "dkv": torch.zeros(R + 2, W), "dkv.norm": torch.ones(R), "uk": torch.zeros(2, R),
         "uv": torch.eye(dv, R), "sink": torch.tensor([math.log(2.0)]), "g": torch.zeros(1, W), "o": torch.eye(W, dv)}
    w = {"m." + k_: t.double() for k_, t in w.items()}
    w["m.dkv"][0, 0] = 1.0                                                # c = (y_0, 0), normed to (+-sqrt 2, 0)
    y = torch.tensor([[1.0, 0, 0, 0], [-1.0, 0, 0, 0], [1.0, 0, 0, 0], [1.0, 0, 0, 0]], dtype=torch.float64)
    out = P.latent_attention_mixer(y, w, "m.", m, 0.0)
    s2 = math.sqrt(2.0)
    # position 0 sees itself: s2 / (1 + 2); 1 sees 0 and 1: 0; 2 sees 1 and 2 (not 0): 0; 3 sees 2 and 3: 2 s2 / 4
    want = torch.tensor([s2 / 3, 0.0, 0.0, 2 * s2 / 4], dtype=torch.float64) * 0.5
    assert torch.allclose(out[:, 0], want, atol=1e-12) and out[:, 1:].abs().max().item() == 0.0


# ---------------------------------------------------------------------------
# kernels against their statements
# ---------------------------------------------------------------------------

def _close(got, want, dtype, what, f32=2e-5, bf16=2e-2):
    tol = f32 if dtype == torch.float32 else bf16
    err = (got.cpu().double() - want.double()).abs().max().item()
    assert math.isfinite(err) and err <= tol * max(1.0, want.double().abs().max().item()), (what, err)


def _paged(lens, G, d, dv, dtype, seed, spare=3):
    from janis_b200.kernels.ops import PAGE
    g = torch.Generator().manual_seed(seed)
    per = [(n + PAGE - 1) // PAGE for n in lens]
    n_pages = sum(per) + spare
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(len(lens) + 2, max(per) + 1, dtype=torch.int32)
    slots = torch.randperm(len(lens) + 2, generator=g)[:len(lens)].to(torch.int32)
    at = 0
    for s in range(len(lens)):
        for j in range(per[s]):
            table[int(slots[s]), j] = order[at]
            at += 1
    k = torch.randn(n_pages, G, PAGE, d, generator=g).to(dtype)
    v = torch.randn(n_pages, G, PAGE, dv, generator=g).to(dtype)
    return k, v, table, slots


@GPU
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,window,cap,sinks,mix,in_keys", [
    (4, 2, 32, 16, 0, 10.0, False, True, False), (8, 2, 64, 64, 0, 30.0, False, True, False),
    (16, 16, 16, 32, 0, 0.0, False, True, False), (5, 5, 10, 6, 0, 3.0, False, True, False),
    (6, 1, 16, 8, 0, 5.0, True, True, False), (3, 1, 24, 40, 7, 2.0, True, False, False),
    (4, 1, 32, 24, 24, 0.0, True, False, True), (8, 1, 128, 96, 128, 0.0, True, False, True),
    (3, 1, 64, 48, 70, 0.0, True, False, True), (1, 1, 9, 7, 1, 0.0, True, False, True),
    (16, 1, 288, 256, 150, 0.0, True, False, True), (32, 4, 64, 64, 0, 20.0, False, True, False)])
def test_attention_kernel_options_against_their_statement(dtype, H, G, d, dv, window, cap, sinks, mix, in_keys):
    """The cap, the learnt sinks, the heads' weights mixed after the softmax and values that lie in the keys, on the
    tensor cores (rows together; a row a CTA; a row's keys over 3 and 7 CTAs) and in the plain kernel.  Queries stand
    at the window's edges, at page borders and far into sequences over scattered pages; the oldest key inside the
    window (or the sequence's first key) and the newest key outside it get a large score under head 0."""
    from janis_b200.kernels import ops
    from tests import kernel_refs as R
    lens = [1, 70, 129, 300]
    kp, vp, table, slots = _paged(lens, G, d, dv, dtype, 3)
    w = window or 10 ** 6
    pos, seq = [], []
    for s, n in enumerate(lens):
        for p in sorted({0, n - 1, n // 2, min(n - 1, 63), min(n - 1, 64), min(n - 1, w - 1), min(n - 1, w), min(n - 1, w + 1),
                         min(n - 1, 2 * w)}):
            pos.append(p)
            seq.append(s)
    T = len(pos)
    g = torch.Generator().manual_seed(9)
    q = torch.randn(T, H * d + 3, generator=g).to(dtype)
    for t in range(T):
        hot = (q[t, :d].float() * (3.0 / max(q[t, :d].float().norm().item(), 1e-3))).to(dtype)
        for j in ((pos[t] - w + 1, pos[t] - w) if window else (0,)):
            if j >= 0:
                kp[int(table[int(slots[seq[t]]), j // ops.PAGE]), 0, j % ops.PAGE] = hot
    M = (torch.eye(H) + 0.4 * torch.randn(H, H, generator=g)).float() if mix else None
    sv = (2.0 * torch.randn(H, generator=g)).float() if sinks else None
    tok_pos, tok_seq = torch.tensor(pos, dtype=torch.int32), torch.tensor(seq, dtype=torch.int32)
    want = torch.zeros(T, H * dv, dtype=dtype)
    R.talk_attention(q, tok_pos, tok_seq, slots, kp, None if in_keys else vp, table, M, None, want, H, G, d, dv, 0.4, 0, sinks,
                     window=window, cap=cap, sink_values=sv, mix_after=mix, values_in_keys=in_keys)
    dev = lambda x: x.cuda() if x is not None else None
    for which, one_row, chunks in ((1, False, 1), (1, True, 1), (1, True, 3), (1, True, 7), (0, False, 1)):
        ops.talk_attention_set_kernel(which)
        try:
            got = torch.full((T, H * dv), float("nan"), dtype=dtype, device="cuda")
            n = ops.talk_attention_scratch_floats(T, chunks, H, dv)
            scratch = torch.full((n,), float("nan"), device="cuda") if n else None
            stats = torch.full((ops.talk_attention_stats_floats(T, H),), float("nan"), device="cuda") if mix else None
            ops.talk_attention(dev(q), dev(tok_pos), dev(tok_seq), dev(slots), dev(kp), None if in_keys else dev(vp), dev(table),
                               dev(M), None, got, H, G, d, dv, 0.4, 0, sinks, one_row=one_row, max_keys=min(w, 300),
                               n_chunks=chunks, scratch=scratch, window=window, cap=cap, sink_values=dev(sv), mix_after=mix,
                               values_in_keys=in_keys, stats=stats)
        finally:
            ops.talk_attention_set_kernel(1)
        _close(got, want, dtype, (which, one_row, chunks))
    # the kernels that take single rows (decode steps), with bounds that cut a row's keys into one chunk and several
    for bound in (min(w, 300), 5000):
        n = ops.talk_attention_rows_floats(dtype, T, H, G, d, dv, bound)
        assert (n > 0) == (d % (4 if dtype == torch.float32 else 8) == 0 and dv % (4 if dtype == torch.float32 else 8) == 0)
        if n:
            got = torch.full((T, H * dv), float("nan"), dtype=dtype, device="cuda")
            ops.talk_attention_rows(dev(q), dev(tok_pos), dev(tok_seq), dev(slots), dev(kp), None if in_keys else dev(vp),
                                    dev(table), dev(M), got, H, G, d, dv, 0.4, torch.full((n,), float("nan"), device="cuda"),
                                    bound, sink=sinks, window=window, cap=cap, sink_values=dev(sv), values_in_keys=in_keys)
            _close(got, want, dtype, ("rows", bound))


def _tables(lens, starts, slots):
    tok_pos, tok_seq, first = [], [], []
    for s, (n, st) in enumerate(zip(lens, starts)):
        first.append(len(tok_pos))
        tok_pos += list(range(st, st + n))
        tok_seq += [s] * n
    i32 = lambda x: torch.tensor(x, dtype=torch.int32)
    return (i32(tok_pos), i32(tok_seq), i32(slots), i32(first), i32(starts), i32([a + b for a, b in zip(starts, lens)]))


@GPU
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,K,norm,unit", [(4, 2, 32, 16, 4, True, True), (5, 5, 10, 6, 5, True, True), (2, 2, 16, 24, 0, True, True),
                                                  (6, 1, 16, 8, 2, False, False), (8, 2, 64, 64, 1, True, False), (3, 1, 8, 8, 16, True, True),
                                                  (32, 8, 128, 128, 3, True, True)])
@pytest.mark.parametrize("pad,lens", [(4, [7, 1, 70, 3, 2]), (16, [7, 1, 70, 3, 2]), (16, [601, 1, 515, 3, 2])])
def test_filter_norm_store_kernel_against_its_statement(dtype, H, G, d, dv, K, norm, unit, pad, lens):
    """Sequences that start, that go on from inputs kept by an earlier step (across a page's border), that bring one
    token, and a padding sequence; the filter's kept inputs, the queries and both pools are compared.  (A step of
    many rows runs the kernel whose CTAs take several rows.)"""
    from janis_b200.kernels import ops
    from tests import kernel_refs as R
    g = torch.Generator().manual_seed(5)
    C = H * d + G * (d + dv)
    starts, slots = [0, 63, 60, 5, 0], [2, 0, 4, 1, -1]
    tabs = _tables(lens, starts, slots)
    T = sum(lens)
    per_seq = max(-(-(a + n) // ops.PAGE) for a, n in zip(starts, lens))
    n_pages = 5 * per_seq + 1
    table = torch.randperm(n_pages, generator=g)[:5 * per_seq].view(5, per_seq).to(torch.int32)
    rows = torch.randn(T, C + pad, generator=g).to(dtype)     # (rows of whole 16 bytes let the wide loads run)
    cw = torch.randn(C, K, generator=g).float() if K else None
    state = torch.randn(5, max(K - 1, 1), C, generator=g).float() if K > 1 else None
    wq, wk = (torch.randn(H * d, generator=g).float(), torch.randn(G * d, generator=g).float()) if norm else (None, None)
    kp, vp = torch.randn(n_pages, G, ops.PAGE, d, generator=g).to(dtype), torch.randn(n_pages, G, ops.PAGE, dv, generator=g).to(dtype)
    want = [torch.zeros(T, H * d, dtype=dtype), kp.clone(), vp.clone(), state.clone() if state is not None else None]
    R.qkv_conv_norm_store(rows, H, G, d, dv, cw, want[3], wq, wk, unit, 1e-5, *tabs, len(lens), want[0], want[1], want[2], table)
    dev = lambda x: x.cuda() if x is not None else None
    got = [torch.full((T, H * d), float("nan"), dtype=dtype, device="cuda"), dev(kp), dev(vp), dev(state)]
    ops.qkv_conv_norm_store(dev(rows), H, G, d, dv, dev(cw), got[3], dev(wq), dev(wk), unit, 1e-5, *[dev(t) for t in tabs],
                            len(lens), got[0], got[1], got[2], dev(table))
    live = torch.cat([torch.arange(a, a + n) for a, n, s in zip(tabs[3].tolist(), lens, slots) if s >= 0])
    _close(got[0][live.cuda()], want[0][live], dtype, "queries")
    _close(got[1], want[1], dtype, "keys")
    _close(got[2], want[2], dtype, "values")
    if state is not None:
        _close(got[3], want[3], torch.float32, "kept inputs")


@GPU
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d,dr,R,amp", [(4, 16, 8, 24, 1.07), (3, 32, 16, 48, 1.0), (1, 6, 2, 7, 1.2), (8, 32, 32, 96, 1.1), (2, 0, 8, 8, 1.0)])
def test_latent_rows_and_head_products_against_their_statements(dtype, H, d, dr, R, amp):
    from janis_b200.kernels import ops
    from tests import kernel_refs as R_
    g = torch.Generator().manual_seed(6)
    lens, starts, slots = [5, 1, 66, 2], [0, 64, 62, 0], [1, 3, 0, -1]
    tabs = _tables(lens, starts, slots)
    T, D = sum(lens), R + dr
    lat_off = H * (d + dr) + 3
    rows = torch.randn(T, lat_off + D + 2, generator=g).to(dtype)
    wc = torch.randn(R, generator=g).float()
    inv = torch.tensor([50.0 ** (-2.0 * i / dr) for i in range(dr // 2)], dtype=torch.float32)
    table = torch.randperm(12, generator=g)[:12].view(4, 3).to(torch.int32)
    kp = torch.randn(13, 1, ops.PAGE, D, generator=g).to(dtype)
    qfull = torch.randn(T, H * D, generator=g).to(dtype)
    want_q, want_k = qfull.clone(), kp.clone()
    R_.latent_rotate_store(rows, lat_off, H, d, dr, R, wc, 1e-5, inv, amp, tabs[0], tabs[1], tabs[2], want_q, want_k, table)
    got_q, got_k = qfull.cuda(), kp.cuda()
    ops.latent_rotate_store(rows.cuda(), lat_off, H, d, dr, R, wc.cuda(), 1e-5, inv.cuda(), amp, tabs[0].cuda(), tabs[1].cuda(),
                            tabs[2].cuda(), got_q, got_k, table.cuda())
    _close(got_q, want_q, dtype, "turned query parts")
    _close(got_k, want_k, dtype, "compressed rows")
    if d:
        w = torch.randn(H, R, d, generator=g).to(dtype)
        want_o, got_o = qfull.clone(), qfull.cuda()
        R_.head_linear(rows, d + dr, 0, w, want_o, D, 0)
        ops.head_linear(rows.cuda(), d + dr, 0, w.cuda(), got_o, D, 0)
        _close(got_o, want_o, dtype, "products per head", f32=5e-5, bf16=3e-2)
        few = ops.HEAD_LINEAR_FEW_ROWS // 8 + 1                  # few rows: the kernel of its own in every dtype
        assert T > ops.HEAD_LINEAR_FEW_ROWS >= few
        want_f, got_f = qfull[:few].clone(), qfull[:few].cuda()
        R_.head_linear(rows[:few], d + dr, 0, w, want_f, D, 0)
        ops.head_linear(rows[:few].cuda(), d + dr, 0, w.cuda(), got_f, D, 0)
        _close(got_f, want_f, dtype, "products per head, few rows", f32=5e-5, bf16=3e-2)


@GPU
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,groups", [(64, 2), (96, 1), (72, 3), (2304, 4), (50, 50), (4096, 8)])
def test_group_norm_and_gate_kernels_against_their_statements(dtype, W, groups):
    from janis_b200.kernels import ops
    from tests import kernel_refs as R
    g = torch.Generator().manual_seed(7)
    T = 9
    h, res, w = torch.randn(T, W, generator=g) * 3, torch.randn(T, W, generator=g).to(dtype), torch.randn(W, generator=g)
    want_h, want_y = h.clone(), torch.zeros(T, W, dtype=dtype)
    R.group_norm(want_h, res, 2.5, w, 1e-5, groups, want_y)
    got_h, got_y = h.cuda(), torch.full((T, W), float("nan"), dtype=dtype, device="cuda")
    ops.group_norm(got_h, res.cuda(), 2.5, w.cuda(), 1e-5, groups, got_y)
    _close(got_h, want_h, torch.float32, "stream", f32=3e-5 if dtype == torch.float32 else 2e-2)
    _close(got_y, want_y, dtype, "rounded stream")
    rows = torch.tensor([4, 0, 7], dtype=torch.int32)
    want_f, got_f = torch.zeros(3, W, dtype=dtype), torch.full((3, W), float("nan"), dtype=dtype, device="cuda")
    R.group_norm(h, None, 1.0, w, 1e-5, groups, want_f, rows)
    ops.group_norm(h.cuda(), None, 1.0, w.cuda(), 1e-5, groups, got_f, rows.cuda())
    _close(got_f, want_f, dtype, "chosen rows")
    if dtype == torch.bfloat16:
        out = torch.empty(T, W, dtype=torch.bfloat16, device="cuda")
        assert torch.equal(ops.round_rows(h.cuda(), out).cpu(), h.to(torch.bfloat16))
    per = W // groups
    x, gates = torch.randn(T, W, generator=g).to(dtype), torch.randn(T, 5 + groups, generator=g).to(dtype)
    want_x, got_x = x.clone(), x.cuda()
    R.sigmoid_gate(want_x, gates, 5, per=per)
    ops.sigmoid_gate(got_x, gates.cuda(), 5, per=per)
    _close(got_x, want_x, dtype, "a gate per head")


# ---------------------------------------------------------------------------
# the engine against the plain model
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("on,dtype", CASES)
def test_whole_prompts_and_decoding(engines, plain, on, dtype):
    """Prompts of unequal lengths in one batch (one of a single token), then decoded together token by token past
    every window; a second round of batches uses the freed slots and pages again."""
    for key in keys_for(on):
        eng = engines(key, dtype, on, max_tokens=2048)
        lens = [1, 40, 150, 9, 77] if on == "cuda" else [1, 30, 9]
        extra = 80 if on == "cuda" else 12
        reqs = _requests(VIV[key]["vocab"], [n + extra for n in lens], 40)
        got = run_requests(eng, reqs, lens, max_live=3)
        for i, r in enumerate(reqs):
            assert_logits(got[i], plain(key, r), dtype, f"{key} request {i} ({lens[i]} + {extra})")


@pytest.mark.parametrize("on,dtype", CASES)
def test_prefill_equals_token_by_token_decoding(engines, plain, on, dtype):
    """A request fed one token a step from its first token on: the filter's kept inputs start empty, the first
    positions see fewer keys than a window holds, and every logit equals the whole prompt's."""
    for key in (["A", "D"] if on == "refs" else ["A", "B", "C", "D"]):
        eng = engines(key, dtype, on, max_tokens=2048)
        reqs = _requests(VIV[key]["vocab"], [35 if on == "refs" else 150, 3], 55)
        got = run_requests(eng, reqs, [1, 1])
        for i, r in enumerate(reqs):
            assert_logits(got[i], plain(key, r), dtype, f"{key} request {i} token by token")


@pytest.mark.parametrize("on,dtype", CASES)
def test_a_request_alone_equals_the_request_in_a_batch(engines, on, dtype):
    """What else is in the step changes nothing beyond rounding: each request alone against the same in a batch."""
    for key in ("B", "C") if on == "cuda" else ("B",):
        eng = engines(key, dtype, on, max_tokens=2048)
        lens = [3, 90, 31] if on == "cuda" else [3, 20, 11]
        reqs = _requests(VIV[key]["vocab"], [n + 6 for n in lens], 70)
        together = run_requests(eng, reqs, lens)
        for i, r in enumerate(reqs):
            alone = run_requests(eng, [r], [lens[i]])[0]
            tol = 1e-5 if dtype == "float32" else 2e-2
            assert (alone - together[i]).abs().max().item() <= tol * together[i].abs().max().item(), (key, i)


@pytest.mark.parametrize("on,dtype", CASES)
@pytest.mark.parametrize("chunk", [2, 3, 16, 64, 65])
def test_prompts_in_pieces(engines, plain, on, dtype, chunk):
    """A prompt that comes in pieces (down to two tokens) onto what the pieces before left: the filter's kept inputs
    and the keys inside the window carry over, across pages' borders."""
    if on == "refs" and chunk in (16, 65):
        pytest.skip("the CPU cases run two sizes")
    for key in (["A", "D"] if on == "refs" or chunk < 16 else ["A", "B", "C", "D"]):
        eng = engines(key, dtype, on, max_tokens=2048)
        lens = [70, 5, 141] if on == "cuda" and chunk >= 16 else [23, 5, 40]
        reqs = _requests(VIV[key]["vocab"], lens, 90 + chunk)
        got = run_in_pieces(eng, reqs, chunk)
        for i, r in enumerate(reqs):
            assert_logits(got[i], plain(key, r), dtype, f"{key} request {i} in pieces of {chunk}")


@GPU
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_graphs(engines, plain, dtype):
    """Hundreds of decode steps from a short prompt: replayed graphs, growing length buckets, windows that slide off
    the prompt and over pages' borders, keys hundreds of positions back in the layers without a window."""
    for key in ("C", "B"):
        eng = engines(key, dtype, "cuda", max_tokens=2048)
        reqs = _requests(VIV[key]["vocab"], [420, 300], 7)
        got = run_requests(eng, reqs, [4, 2])
        for i, r in enumerate(reqs):
            assert_logits(got[i], plain(key, r), dtype, f"{key} long decoding {i}")


@pytest.mark.parametrize("on,dtype", [pytest.param("cuda", "float32", marks=GPU), pytest.param("refs", "float32")])
def test_a_far_token_and_a_window_edge_show_in_the_logits(engines, plain, on, dtype):
    """Two requests that differ in one token only.  Where the token lies inside the window of every windowed layer the
    last logits differ; the plain model says by how much, and the engine must agree with it for both, so a window
    that is one position off, or a far key that is dropped, shows as an error of the size of that difference."""
    key = "F"                                      # one latent layer, a window of nine positions
    eng = engines(key, dtype, on, max_tokens=1024)
    V, n = VIV[key]["vocab"], 40
    base = random_tokens(V, n, 123)
    for back in (8, 9):                            # the oldest position the last token sees, and the one before it
        other = list(base)
        other[n - 1 - back] = (other[n - 1 - back] + 1) % V
        want_a, want_b = plain(key, base)[-1], plain(key, other)[-1]
        differ = (want_a - want_b).abs().max().item()
        assert (differ > 1e-3) == (back == 8), (back, differ)
        for lens in ([n], [n - 4]):               # the last token in the prompt's step, and decoded alone
            got = run_requests(eng, [base, other], lens * 2)
            assert_logits(got[0][-1:], want_a[None], dtype, f"window edge {back} base")
            assert_logits(got[1][-1:], want_b[None], dtype, f"window edge {back} changed")
    key = "E"                                      # one attention layer without a window: the first token is seen from afar
    eng = engines(key, dtype, on, max_tokens=1024)
    V, n = VIV[key]["vocab"], 200 if on == "cuda" else 70
    base = random_tokens(V, n, 321)
    other = [(base[0] + 7) % V] + base[1:]
    want_a, want_b = plain(key, base)[-1], plain(key, other)[-1]
    assert (want_a - want_b).abs().max().item() > 1e-4
    got = run_requests(eng, [base, other], [n - 3, n - 3])
    assert_logits(got[0][-1:], want_a[None], dtype, "far token base")
    assert_logits(got[1][-1:], want_b[None], dtype, "far token changed")
    assert (got[0][-1] - got[1][-1]).abs().max().item() > 0.5 * (want_a - want_b).abs().max().item()


@pytest.mark.parametrize("on,dtype", [pytest.param("cuda", "float32", marks=GPU), pytest.param("refs", "float32")])
def test_greedy_generation_through_the_engine(engines, viv_dirs, on, dtype):
    """`generate` (scheduler, sampler, stop handling) against greedy decoding of the plain model."""
    from tests.plain import vivazen_plain as P
    key = "A"
    eng = engines(key, dtype, on, max_tokens=1024)
    cfg, w = P.load_folder(viv_dirs[key])
    prompts = _requests(VIV[key]["vocab"], [5, 17, 2], 11)
    n_new = 12 if on == "cuda" else 6
    replies = eng.generate(prompts, temp=0.0, max_tokens=n_new, stop=[])
    for p, r in zip(prompts, replies):
        seq = list(p)
        for _ in range(n_new):
            seq.append(int(P.forward(cfg, w, seq)[-1].argmax()))
        assert r == seq[len(p):], (p, r, seq[len(p):])


@GPU
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_and_command_line(viv_dirs, plain, dtype, tmp_path):
    """`bin/trace_run` as a user runs it: the model class comes from config.json; prompts in one batch, decoded
    together, a second batch on the freed slots; and `bin/janis generate` on the same folder."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    from tests.test_generation import ROOT, _trace
    key = "D"
    V = VIV[key]["vocab"]
    lens = [40, 9, 75, 1, 23, 130]
    reqs = [random_tokens(V, n, 210 + n) for n in lens]
    steps, peak = _trace(reqs, [max(1, n - 32) for n in lens], batch_of=3)
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", viv_dirs[key], "--dtype", dtype,
                        "--out", str(out), "--max-tokens", str(peak)],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert p.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    got = {f"r{i}": [] for i in range(len(reqs))}
    for s in steps:
        arr = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, V)
        o = 0
        for e in s["entries"]:
            got[e["id"]].append(torch.from_numpy(arr[o:o + len(e["want"])].copy()))
            o += len(e["want"])
        assert o == arr.shape[0]
    for i, r in enumerate(reqs):
        assert_logits(torch.cat(got[f"r{i}"]), plain(key, r), dtype, f"trace request {i}")
    if dtype == "float32":
        from tests.plain import vivazen_plain as P
        cfg, w = P.load_folder(viv_dirs[key])
        prompt = reqs[1]
        g = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "janis"), "generate", "--model", viv_dirs[key],
                            "--dtype", "float32", "--ids", ",".join(map(str, prompt)), "--max-tokens", "5", "--temp", "0", "--stop", ""],
                           capture_output=True, text=True, timeout=900)
        assert g.returncode == 0, g.stderr[-2000:]
        seq = list(prompt)
        for _ in range(5):
            seq.append(int(P.forward(cfg, w, seq)[-1].argmax()))
        assert ",".join(map(str, seq[len(prompt):])) in g.stdout.replace(" ", ""), g.stdout


@GPU
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_shapes_of_a_real_model(tmp_path, dtype):
    """Two layers at layer sizes of a model of a few billion weights (width 2048; 16 heads over 4 of 128 with a filter;
    16 latent heads of 64 + 32 over a compressed row of 256, a window of 200), vocabulary cut to 2,048: the kernels'
    launch shapes, vector loads and staged tiles at sizes the small models do not reach.  A prompt longer than the
    window, then decoded; beside it a short prompt."""
    from tests.plain import vivazen_plain as P
    raw = _model(2048, 2048, 8, 1e-6, 2.0, [
        _layer("attention", _att(16, 4, 128, 128, 128 ** -0.5, conv=4, cap=30.0), 4096),
        _layer("latent_attention", _lat(16, 64, 32, 64, 256, 96 ** -0.5, window=200, scaling=(4.0, 128, 16.0, 1.0)), 4096)])
    write_vivazen(str(tmp_path), raw, 77, gain=1.0, norm_gain=1.5, q_gain=2.0)
    cfg, w = P.load_folder(str(tmp_path))
    eng = make_engine(str(tmp_path), dtype, "cuda", max_tokens=1024)
    try:
        reqs = _requests(2048, [300 + 8, 5 + 8], 3)
        got = run_requests(eng, reqs, [300, 5])
        for i, r in enumerate(reqs):
            assert_logits(got[i], P.forward(cfg, w, r), dtype, f"real layer shapes, request {i}")
    finally:
        eng.close()
