"""Zadunex on the GPU: every mechanism's kernels alone against the plain functions of
tests/plain_zadunex.py, then the model through the engine: whole prompts, portions, single tokens,
unequal batches, reused slots, far tokens, long decoding, greedy generation and trace replay."""

import io
import json
from types import SimpleNamespace

import pytest
import torch

import plain_zadunex as plain
from zadunex_helpers import CONFIGS, assert_logits, plain_logits, prompts, write_folder

pytestmark = pytest.mark.gpu

DTYPES = (torch.float32, torch.bfloat16)
PART_TOL = {torch.float32: 3e-5, torch.bfloat16: 5e-2}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("zadunex_gpu")
    return {name: write_folder(root / name, name) for name in CONFIGS}


def runtime(dtype):
    from kernel_rush_kawk_b200.csrc import load_kernels
    from kernel_rush_kawk_b200.engine.model import Runtime

    return Runtime(torch.device("cuda:0"), dtype, load_kernels((16, 32)))


def rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g) * scale


def context(rt, slots, starts, q_lens, cache):
    from kernel_rush_kawk_b200.engine.step import BatchMeta, StepContext

    meta = BatchMeta(sum(q_lens), len(slots), 0, rt.device)
    meta.fill(slots, starts, [[0] * n for n in q_lens], [])
    return StepContext(rt.ops, meta, cache)


def close(got, ref, dtype, what):
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err = (got - ref).abs().max().item()
    tol = PART_TOL[dtype] * ref.abs().max().item()
    assert err <= tol, f"{what}: max |d| = {err:.3e} > {tol:.3e}; first bad row {int(((got - ref).abs() > tol).any(-1).nonzero()[0])}"


def run_part(part, rt, h, pieces, dtype, prior=()):
    """One sequence through a mixer part, cut into ``pieces``; ``prior``: sequences that used (and gave
    back) the slot before."""
    from kernel_rush_kawk_b200.cache import SequenceCache

    cache = SequenceCache([part.cache_need()], 2048, 1, 2048, rt.device, dtype)
    for seq, cuts in list(prior) + [(h, pieces)]:
        slot = cache.alloc()
        got, start = [], 0
        for n in cuts:
            cache.reserve(slot, start + n)
            cache.sync()
            ctx = context(rt, [slot], [start], [n], cache)
            got.append(part.forward(ctx, seq[start:start + n].to(dtype).cuda(), cache.view(0)))
            cache.advance(slot, n)
            start += n
        cache.free(slot)
    rt.ops.check()
    return torch.cat(got)


def as_path(w, dtype):
    """The tensors as the path stores them, and the same values in float64 for the plain functions."""
    stored = {k: v.to(torch.bfloat16) for k, v in w.items()}  # checkpoints hold bfloat16
    return {k: v.to(dtype).cuda() for k, v in stored.items()}, {k: v.double() for k, v in stored.items()}


# ----------------------------------------------------------------------------------------------
# each mechanism alone
# ----------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("streams, width", [(1, 72), (2, 64), (3, 50), (4, 33), (8, 16)])
def test_hyper_connection_norm_folds_reads_and_normalises(dtype, streams, width):
    """Two sublayers in a row: the first norm only reads; the second writes the first sublayer's output back
    through its M and b, reads through its own a, and leaves its own M and b on the stream."""
    from kernel_rush_kawk_b200.parts import HyperRMSNorm, Stream

    rt = runtime(dtype)
    ctx = SimpleNamespace(ops=rt.ops)
    S, C, rows = streams, width, 7
    X = rand((rows, S, C), 1, 3.0)
    norms, ws = [], []
    for q in range(2):
        w = {"weight": (1 + 0.3 * rand((C,), 10 + q)), "in": rand((S,), 20 + q), "out": rand((S,), 30 + q),
             "mix": rand((S, S), 40 + q)}
        part = HyperRMSNorm({"size": C, "eps": 1e-4, "streams": S})
        assert {k: tuple(s.shape) for k, s in part.tensor_specs().items()} == {k: tuple(v.shape) for k, v in w.items()}
        dev, ref = as_path(w, dtype)
        part.bind(dev, rt)
        norms.append(part)
        ws.append(ref)
    stream = Stream(X.reshape(rows, S * C).cuda())
    h1 = norms[0].forward(ctx, stream).tensor()
    Xd = X.double()
    close(h1, plain.rms_norm(torch.einsum("s,rsc->rc", ws[0]["in"], Xd), ws[0]["weight"], 1e-4), dtype, "first read")
    assert stream.branch is None and stream.fold is not None
    y = rand((rows, C), 5, 2.0).to(dtype)
    stream.branch = y.cuda()
    h2 = norms[1].forward(ctx, stream).tensor()
    X2 = torch.einsum("st,rsc->rtc", ws[0]["mix"], Xd) + ws[0]["out"][None, :, None] * y.double()[:, None, :]
    assert (stream.x.double().cpu().view(rows, S, C) - X2).abs().max() < 1e-4  # the streams are 32-bit whatever the path
    close(h2, plain.rms_norm(torch.einsum("s,rsc->rc", ws[1]["in"], X2), ws[1]["weight"], 1e-4), dtype, "fold and read")
    last = HyperRMSNorm({"size": C, "eps": 1e-4, "streams": S, "read": "sum"})
    last.bind({"weight": ws[0]["weight"].to(dtype).cuda()}, rt)
    stream.branch = y.cuda()
    h3 = last.forward(ctx, stream).tensor()
    X3 = torch.einsum("st,rsc->rtc", ws[1]["mix"], X2) + ws[1]["out"][None, :, None] * y.double()[:, None, :]
    close(h3, plain.rms_norm(X3.sum(dim=1), ws[0]["weight"], 1e-4), dtype, "the sum of the streams")


SSM_SHAPES = [  # hidden, heads, head_dim, state, groups, taps, norm parts
    (64, 4, 16, 24, 2, 4, 2),
    (48, 2, 32, 16, 1, 3, 1),
    (50, 3, 10, 7, 3, 4, 2),
    (32, 1, 64, 8, 1, 5, 4),
    (40, 6, 8, 40, 6, 2, 3),
    (32, 2, 12, 5, 2, 1, 1),
    (64, 2, 64, 128, 1, 4, 1),   # a head of 64 x 128: thirty-two rows of the state a lane
    (32, 2, 4, 200, 2, 4, 8),    # narrow heads and a long state: every lane of a warp on one column
]


def ssm_part(shape, dtype, rt, seed=50):
    from kernel_rush_kawk_b200.parts import Mamba2

    C, H, P, N, G, taps, parts = shape
    inner, ch = H * P, H * P + 2 * G * N
    m = {"heads": H, "vdim": P, "state": N, "groups": G, "conv": taps, "norm_groups": parts}
    part = Mamba2({"hidden": C, "heads": H, "head_dim": P, "state": N, "groups": G, "taps": taps, "norm_groups": parts,
                   "eps": 1e-5})
    w = {"in": rand((2 * inner + 2 * G * N + H, C), seed + 1, 0.25), "conv": rand((ch, taps), seed + 2, 0.4),
         "conv.b": rand((ch,), seed + 3, 0.2), "dt_bias": rand((H,), seed + 4, 1.0) - 0.5,
         "A_log": rand((H,), seed + 5, 1.0) - 2.5, "D": 1 + rand((H,), seed + 6, 0.3),
         "norm": 1 + rand((inner,), seed + 7, 0.2), "o": rand((C, inner), seed + 8, 0.2)}
    assert {k: tuple(s.shape) for k, s in part.tensor_specs().items()} == {k: tuple(v.shape) for k, v in w.items()}
    dev, ref = as_path(w, dtype)
    part.bind(dev, rt)
    return part, m, ref


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", SSM_SHAPES)
def test_state_space_mixer_alone(dtype, shape):
    """Whole (long enough for the scan in chunks), in pieces down to two tokens and fewer than the
    convolution's taps, token by token, and in a slot whose state another sequence left."""
    rt = runtime(dtype)
    part, m, ref = ssm_part(shape, dtype, rt)
    T = 300
    h = rand((T, shape[0]), 11).to(dtype)
    want = plain.mamba2(h.double(), ref, "", m, 1e-5)
    other = rand((70, shape[0]), 12).to(dtype)
    for pieces, prior in (([T], ()), ([127, 2, 1, 3, 129, 38], ()), ([270] + [1] * 30, ()), ([T], [(other, [69, 1])])):
        got = run_part(part, rt, h, pieces, dtype, prior=prior)
        close(got, want, dtype, f"state-space mixer {shape}, pieces {pieces[:4]}, prior {len(prior)}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_state_carries_one_loud_token_over_hundreds(dtype):
    """A head whose decay is almost one keeps a token that came hundreds of tokens (and several chunks and
    steps) earlier; a state that were lost or reset at a chunk's or a step's edge would show as silence."""
    rt = runtime(dtype)
    shape = (32, 2, 16, 16, 1, 4, 1)
    part, m, ref = ssm_part(shape, dtype, rt)
    for t in (part.a_log, ref["A_log"]):
        t.fill_(-9.0)  # rate exp(-9): the state loses a tenth in a thousand tokens
    T, loud = 700, 5
    h = rand((T, 32), 3, 0.05)
    h[loud] *= 400.0
    h = h.to(dtype)
    want = plain.mamba2(h.double(), ref, "", m, 1e-5)
    quiet = h.clone()
    quiet[loud] = 0
    base = plain.mamba2(quiet.double(), ref, "", m, 1e-5)
    assert (want[600:] - base[600:]).abs().max() > 0.2 * want[600:].abs().max()  # the case shows what it is meant to
    for pieces in ([T], [300, 256, 144], [640] + [1] * 60):
        close(run_part(part, rt, h, pieces, dtype), want, dtype, f"far token, pieces {pieces[:3]}")


ATTN_SHAPES = [  # hidden, heads, kv_heads, dim, vdim, rot, base
    (72, 6, 3, 16, 16, 16, 1e4),
    (64, 4, 1, 32, 64, 8, 2e4),
    (40, 2, 2, 24, 8, 24, 50.0),
    (48, 3, 1, 8, 40, 2, 10.0),
    (50, 3, 3, 6, 5, 4, 7.0),
    (64, 4, 2, 32, 32, 0, 1e4),
]


def attention_part(shape, dtype, rt, seed=0, scale=0.4):
    from kernel_rush_kawk_b200.parts import SinkWindowAttention

    C, H, G, D, Dv, rot, base = shape
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": scale, "rot": {"dims": rot, "base": base}}
    part = SinkWindowAttention({"hidden": C, "heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": scale, "window": None,
                                "rot_dims": rot, "rot_base": base, "sink": "zero", "bias": True, "qk_norm": "row", "eps": 1e-5})
    w = {"q": rand((H * D, C), seed + 1, 0.4), "k": rand((G * D, C), seed + 2, 0.4), "v": rand((G * Dv, C), seed + 3, 0.3),
         "o": rand((C, H * Dv), seed + 4, 0.2), "q.b": rand((H * D,), seed + 5, 0.5), "k.b": rand((G * D,), seed + 6, 0.5),
         "v.b": rand((G * Dv,), seed + 7, 0.5), "q.norm": 1 + rand((H * D,), seed + 8, 0.3), "k.norm": 1 + rand((G * D,), seed + 9, 0.3)}
    assert {k: tuple(s.shape) for k, s in part.tensor_specs().items()} == {k: tuple(v.shape) for k, v in w.items()}
    dev, ref = as_path(w, dtype)
    part.bind(dev, rt)
    return part, m, ref


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", ATTN_SHAPES)
def test_attention_with_biases_row_norms_and_the_zero_sink_alone(dtype, shape):
    rt = runtime(dtype)
    part, m, ref = attention_part(shape, dtype, rt)
    T = 200
    h = rand((T, shape[0]), 9).to(dtype)
    want = plain.attention(h.double(), ref, "", m, 1e-5)
    other = rand((80, shape[0]), 10).to(dtype)
    for pieces, prior in (([T], ()), ([63, 2, 64, 71], ()), ([150] + [1] * 50, ()), ([T], [(other, [80])])):
        close(run_part(part, rt, h, pieces, dtype, prior=prior), want, dtype, f"attention {shape}, pieces {pieces[:4]}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_zero_sink_takes_its_share_and_the_first_token_is_not_alone(dtype):
    """With tiny scores every weight is 1 / (keys + 1): the first token's output is half its value, not all of it."""
    rt = runtime(dtype)
    shape = (32, 2, 1, 16, 16, 4, 100.0)
    part, m, ref = attention_part(shape, dtype, rt, scale=1e-6)
    m["scale"] = 1e-6
    part._w_out = torch.eye(32, dtype=dtype, device="cuda")
    ref["o"] = torch.eye(32, dtype=torch.float64)
    h = rand((20, 32), 3).to(dtype)
    got = run_part(part, rt, h, [20], dtype)
    close(got, plain.attention(h.double(), ref, "", m, 1e-5), dtype, "uniform weights with the sink's share")
    v = (h.double() @ ref["v"].T + ref["v.b"])
    close(got[:1, :16], v[:1] / 2, dtype, "the first token")
    close(got[9:10, :16], v[:10].sum(dim=0, keepdim=True) / 11, dtype, "the tenth token")


def far_key_case(loud, T, dtype):
    """Keys are made from the first query head's weights, and the loud token's input is three times the last
    token's: its key points the way of the last query (the row norm takes the factor out) while its value is its
    own, so the last row's output leans on that one key among hundreds."""
    shape = (32, 2, 1, 32, 32, 2, 1000.0)
    w_seed = 0
    C, H, G, D, Dv, rot, base = shape
    w = {"q": rand((H * D, C), w_seed + 1, 0.4), "v": rand((G * Dv, C), w_seed + 3, 0.3), "o": rand((C, H * Dv), w_seed + 4, 0.2),
         "q.b": rand((H * D,), w_seed + 5, 0.1), "v.b": rand((G * Dv,), w_seed + 7, 0.5), "q.norm": 1 + rand((H * D,), w_seed + 8, 0.1)}
    w.update({"k": w["q"][:D].clone(), "k.b": w["q.b"][:D].clone(), "k.norm": w["q.norm"][:D].clone()})
    h = rand((T, C), 21, 0.5)
    h[loud] = 3.0 * h[T - 1]
    return shape, w, h.to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("loud, T", [(0, 70), (63, 200), (64, 200), (5, 600)])
def test_one_far_key_among_hundreds_is_found(dtype, loud, T):
    """The key of one token (the very first, at a page's edge, far back) stands out for the last query, in a
    whole prompt, decoded alone, and in pieces of two."""
    from kernel_rush_kawk_b200.parts import SinkWindowAttention

    rt = runtime(dtype)
    shape, w, h = far_key_case(loud, T, dtype)
    C, H, G, D, Dv, rot, base = shape
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": 0.7, "rot": {"dims": rot, "base": base}}
    part = SinkWindowAttention({"hidden": C, "heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": 0.7, "window": None,
                                "rot_dims": rot, "rot_base": base, "sink": "zero", "bias": True, "qk_norm": "row", "eps": 1e-5})
    dev, ref = as_path(w, dtype)
    part.bind(dev, rt)
    want = plain.attention(h.double(), ref, "", m, 1e-5)
    without = h.double().clone()
    without[loud] = rand((C,), 77, 0.5).double()
    other = plain.attention(without, ref, "", m, 1e-5)
    assert (want[-1] - other[-1]).abs().max() > 0.2 * want[-1].abs().max()  # the case shows what it is meant to
    for pieces in ([T], [T - 3, 1, 1, 1], [2] * (T // 2)):
        close(run_part(part, rt, h, pieces, dtype), want, dtype, f"loud token {loud} of {T}, pieces {pieces[:3]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows, inter, limit, C", [(5, 24, 1.0, 48), (40, 33, 0.6, 48), (3, 64, 7.0, 48),
                                                   (5, 40, 1.0, 64), (13, 96, 0.8, 128), (1, 33, 0.5, 96)])
def test_dense_feed_forward_with_clamped_inputs(dtype, rows, inter, limit, C):
    """Widths that are a multiple of 32 take, for few bfloat16 rows, the product whose epilogue clamps and
    multiplies; the others the product and the activation kernel."""
    from kernel_rush_kawk_b200.parts import GatedMLP

    rt = runtime(dtype)
    part = GatedMLP({"hidden": C, "intermediate": inter, "activation": "swish_clamped", "limit": limit, "slope": 1.702})
    w = {"gate": rand((inter, C), 1, 0.4), "up": rand((inter, C), 2, 0.4), "down": rand((C, inter), 3, 0.3)}
    dev, ref = as_path(w, dtype)
    part.bind(dev, rt)
    h = rand((rows, C), 4, 1.5).to(dtype)
    g = h.double() @ ref["gate"].T
    assert (g > limit).any() and (g < -limit).any()  # both sides of the clamps are exercised
    ctx = SimpleNamespace(ops=rt.ops)
    close(part.forward(ctx, h.cuda()), plain.dense_ff(h.double(), ref, "", {"limit": limit}), dtype, "clamped dense feed-forward")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(64, 5, 2, 40), (96, 8, 1, 48), (50, 3, 3, 11), (64, 16, 4, 32), (32, 40, 5, 16)])
@pytest.mark.parametrize("rows", [1, 5, 200])
def test_experts_weighted_by_the_softmax_over_all_of_them(dtype, shape, rows):
    from kernel_rush_kawk_b200.parts import RoutedExperts

    rt = runtime(dtype)
    C, E, top, F = shape
    part = RoutedExperts({"hidden": C, "experts": E, "top": top, "intermediate": F, "router_bias": False, "weights": "all"})
    w = {"router": rand((E, C), 1, 0.5)}
    for e in range(E):
        w.update({f"e{e}.gate": rand((F, C), 10 + 3 * e, 0.3), f"e{e}.up": rand((F, C), 11 + 3 * e, 0.3),
                  f"e{e}.down": rand((C, F), 12 + 3 * e, 0.3)})
    assert {k: tuple(s.shape) for k, s in part.tensor_specs().items()} == {k: tuple(v.shape) for k, v in w.items()}
    dev, ref = as_path(w, dtype)
    part.bind(dev, rt)
    h = rand((rows, C), 7, 1.5).to(dtype)
    want = plain.routed_ff(h.double(), ref, "", {"router": {"experts": E, "top": top}})
    for decode in (False, True):
        ctx = SimpleNamespace(ops=rt.ops, batch=SimpleNamespace(is_decode=decode))
        close(part.forward(ctx, h.cuda()), want, dtype, f"experts {shape}, {rows} rows, single-token step {decode}")


def test_routing_weights_are_shares_of_the_whole_softmax():
    rt = runtime(torch.float32)
    x = torch.eye(4, device="cuda")
    w = torch.tensor([[1.0, 2.0, 0.0, -1.0], [3.0, 2.0, 0.0, 5.0], [3.0, 0.5, 0.0, 5.0], [0.0, 2.0, 0.0, 4.0]], device="cuda").t().contiguous()
    experts, weights, _ = rt.ops.moe_route(x, w, None, 2, over_all=True)
    z = x @ w.t()
    for r in range(4):
        best = sorted(range(4), key=lambda e: (-float(z[r, e]), e))[:2]
        assert experts[r].tolist() == best
        assert torch.allclose(weights[r], torch.softmax(z[r], dim=0)[best], atol=1e-6)
        assert float(weights[r].sum()) < 1.0


# ----------------------------------------------------------------------------------------------
# the model through the engine
# ----------------------------------------------------------------------------------------------

def engine(folder, dtype, **kw):
    from kernel_rush_kawk_b200 import Engine

    args = dict(dtype=dtype, max_tokens=4096, max_slots=6, max_context=1024)
    args.update(kw)
    return Engine(folder, **args)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_portions_and_single_tokens_through_the_engine(folders, name, dtype):
    from kernel_rush_kawk_b200 import StepEntry

    eng = engine(folders[name], dtype)
    ids = prompts(name, [300])[0]
    ref = plain_logits(folders[name], ids)
    for pieces in ([300], [130, 2, 3, 64, 101], [250] + [1] * 50):
        slot = eng.cache.alloc()
        got, start = [], 0
        for n in pieces:
            got.append(eng.step([StepEntry(slot, ids[start:start + n], list(range(n)))]).clone())
            start += n
        eng.cache.free(slot)
        assert_logits(torch.cat(got), ref, dtype, f"{name} {dtype}, pieces {pieces[:4]}")
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_reused_slots_and_long_decoding(folders, dtype):
    """Five requests of unequal length start together (one long enough for the scan in chunks beside short ones)
    and are decoded together while the shorter ones end; their slots, states and pages are then used again by
    others. Every row against the sequence run alone in the plain implementation."""
    from kernel_rush_kawk_b200 import StepEntry

    name = "za"
    eng = engine(folders[name], dtype, max_slots=5)
    for round_ in range(2):
        lengths = [90, 1, 400, 37, 64] if round_ == 0 else [65, 130, 2]
        tails = [70, 0, 100, 20, 1] if round_ == 0 else [30, 60, 1]
        seqs = prompts(name, lengths, seed=5 + round_)
        slots = [eng.cache.alloc() for _ in seqs]
        heads = [len(ids) - t for ids, t in zip(seqs, tails)]
        first = eng.step([StepEntry(s, ids[:n], [n - 1]) for s, ids, n in zip(slots, seqs, heads)]).clone()
        for i, (ids, n) in enumerate(zip(seqs, heads)):
            assert_logits(first[i:i + 1], plain_logits(folders[name], ids)[n - 1:n], dtype, f"round {round_}, prompt {i}")
        got = {i: [] for i in range(len(seqs))}
        for t in range(max(tails)):
            live = [i for i in range(len(seqs)) if t < tails[i]]
            out = eng.step([StepEntry(slots[i], [seqs[i][heads[i] + t]], [0]) for i in live])
            for row, i in enumerate(live):
                got[i].append(out[row].clone())
            for i in range(len(seqs)):
                if t + 1 == tails[i]:
                    eng.cache.free(slots[i])
        for i, ids in enumerate(seqs):
            if tails[i] == 0:
                eng.cache.free(slots[i])
                continue
            assert_logits(torch.stack(got[i]), plain_logits(folders[name], ids)[heads[i]:], dtype, f"round {round_}, decoded sequence {i}")
        eng.cache.check()
        assert eng.cache.live == 0


def test_greedy_generation_through_the_engines_own_entry(folders):
    """Engine.generate (scheduler, captured single-token steps, selection kernel) against greedy decoding
    with the plain implementation; prompts of unequal length, one of a single token."""
    name = "zb"
    eng = engine(folders[name], "float32", max_tokens=None)
    seqs = prompts(name, [33, 1, 80], seed=9)
    steps = list(eng.generate(seqs, 12))
    assert len(steps) == 12
    cfg, w = plain.read_folder(folders[name], torch.float64)
    for i, ids in enumerate(seqs):
        ids = list(ids)
        for t in range(12):
            logits = plain.forward(cfg, w, ids)[-1]
            best = torch.topk(logits, 2).values
            if best[0] - best[1] < 1e-4:  # too close to call in 32-bit: stop comparing this sequence
                break
            assert steps[t][i] == int(logits.argmax()), f"sequence {i}, new token {t}"
            ids.append(steps[t][i])


def test_trace_replay_serves_the_design(folders, tmp_path):
    """bin/trace_run's program on a small schedule: a batch of prompts, single tokens, a request that ends."""
    from kernel_rush_kawk_b200 import replay

    name = "zc"
    a, b = prompts(name, [70, 9], seed=4)
    lines = [{"step": 0, "entries": [{"id": "a", "tokens": a[:60], "want": [0, 59]}, {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[60]], "want": [0]}, {"id": "b", "tokens": [b[8]], "want": []}], "end": ["b"]}]
    lines += [{"step": 2 + t, "entries": [{"id": "a", "tokens": [a[61 + t]], "want": [0]}], "end": ["a"] if t == 8 else []} for t in range(9)]
    out = io.StringIO()
    args = replay.build_parser().parse_args(["--model", str(folders[name]), "--dtype", "float32", "--out", str(tmp_path / "o"),
                                             "--max-tokens", "256"])
    assert replay.run(args, stdin=io.StringIO("\n".join(json.dumps(l) for l in lines) + "\n"), stdout=out) == 0
    assert out.getvalue().split() == [w for t in range(11) for w in ("done", str(t))]
    import numpy as np
    ref_a, ref_b = plain_logits(folders[name], a), plain_logits(folders[name], b)
    first = torch.from_numpy(np.fromfile(tmp_path / "o" / "0.f32", dtype="<f4").reshape(3, -1))
    assert_logits(first, torch.stack([ref_a[0], ref_a[59], ref_b[7]]), "float32", "replayed prompts")
    for t in range(10):
        row = torch.from_numpy(np.fromfile(tmp_path / "o" / f"{1 + t}.f32", dtype="<f4").reshape(1, -1))
        assert_logits(row, ref_a[60 + t:61 + t], "float32", f"replayed token {t}")
